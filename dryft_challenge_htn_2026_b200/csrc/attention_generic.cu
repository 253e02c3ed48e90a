// Causal grouped-query attention over the paged cache, one warp per (token, query head), all
// arithmetic in float32 on CUDA cores. It serves the 32-bit path of the model for every phase
// (whole prompts, continued chunks, single tokens); any head size that is a multiple of 2 up to
// 256, any head counts, an optional sliding window.
//
// Formula (reference: engine/engine.py:148-164, engine/fused.py:301-343): query head h reads
// kv head h / (nh / nkv); score = q.k * scale; a query at position p sees keys j <= p (and
// j > p - window when a window is set); softmax over the keys with a running maximum; o = P.V.
#include "common.cuh"

template <typename T>
__global__ void attention_generic_kernel(const T* q, T* out,
                                         const T* k_store, const T* v_store,
                                         const int* row_pos, const int* row_seq,
                                         const int* page_table, int pt_stride, int n_tok, int nh,
                                         int nkv, int hd, int window, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (long long)n_tok * nh) return;
    const int t = (int)(wid / nh), h = (int)(wid % nh);
    T* o = out + ((size_t)t * nh + h) * hd;
    const int pos = row_pos[t];
    if (pos < 0) {  // padding row
        for (int d = lane; d < hd; d += 32) o[d] = from_f<T>(0.f);
        return;
    }
    const int kvh = h / (nh / nkv);
    const int* pt = page_table + (size_t)row_seq[t] * pt_stride;
    const T* qr = q + ((size_t)t * nh + h) * hd;
    float qv[8], acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        qv[i] = d < hd ? to_f(qr[d]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j = lo; j <= pos; j++) {
        const size_t off = kv_offset(pt[j / DK_PAGE], nkv, kvh, j % DK_PAGE, hd);
        const T* kr = k_store + off;
        const T* vr = v_store + off;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < hd) dot += qv[i] * to_f(kr[d]);
        }
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);  // m = -inf on the first key: alpha = 0
        const float p = expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = lane + 32 * i;
            if (d < hd) acc[i] = acc[i] * alpha + p * to_f(vr[d]);
        }
        m = m_new;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f<T>(acc[i] * inv);
    }
}

DK_EXPORT int dk_attention_generic(int dtype, const void* q, void* out, const void* k_store, const void* v_store,
                                   const int* row_pos, const int* row_seq, const int* page_table, int pt_stride,
                                   int n_tok, int nh, int nkv, int hd, int window, float scale, cudaStream_t st) {
    if (hd > 256 || nh % nkv != 0) return (int)cudaErrorInvalidValue;
    long long warps = (long long)n_tok * nh;
    unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == 0)
        return dk_launch(attention_generic_kernel<float>, dim3(blocks), dim3(128), 0, st, (const float*)q,
                         (float*)out, (const float*)k_store, (const float*)v_store, row_pos, row_seq, page_table,
                         pt_stride, n_tok, nh, nkv, hd, window, scale);
    return dk_launch(attention_generic_kernel<bf16>, dim3(blocks), dim3(128), 0, st, (const bf16*)q, (bf16*)out,
                     (const bf16*)k_store, (const bf16*)v_store, row_pos, row_seq, page_table, pt_stride, n_tok, nh,
                     nkv, hd, window, scale);
}
