// Memory-bound row kernels: embedding gather + RMSNorm, residual add + RMSNorm, SiLU(gate)*up,
// and per-head RMSNorm + rotary position encoding + key/value cache write.
//
// The residual stream `h` is float32 for every model dtype; sums of squares, rsqrt, rotation and
// the residual add are computed in float32. T is the activation/weight dtype (float or bf16).
// Reference formulas (KrishP147/Dryft-Challenge-HTN-2026): engine/engine.py:107-115 (RMSNorm,
// rotate-half RoPE), engine/fused.py:152-172 (add+norm), :175-188 (SiLU*up), :415-475 (q/k norm,
// RoPE, cache write).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// h[row] = embed[tok[row]];  a[row] = rmsnorm(h[row]) * w
template <typename T>
__global__ void embed_rmsnorm_kernel(const int* tok, const T* __restrict__ embed,
                                     const float* __restrict__ w, float eps, int H, int V,
                                     float* h, T* a) {
    __shared__ float red[33];
    pdl_launch_dependents();   // before the wait: see pdl_launch_dependents
    pdl_wait();
    const size_t row = blockIdx.x;
    int t = tok[row];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);  // ids are validated on the host; never read out of bounds
    const T* e = embed + (size_t)t * H;
    float* hr = h + row * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_f(e[i]);
        hr[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
    if (w == nullptr) return;
    T* ar = a + row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ar[i] = from_f<T>(hr[i] * rs * w[i]);
}

// h[row] += delta[row] (if delta);  a[out_row] = rmsnorm(h[row]) * w.
// With `rows` the kernel gathers: out_row = blockIdx.x, row = rows[blockIdx.x], and h is not
// written back (used for the final norm at the positions whose logits are wanted).
// ``parts``: n_parts float32 partial sums [n_parts][rows of h][H] (the split-K output of the skinny
// product) that are added up in order and then added to h like delta.
template <typename T>
__global__ void add_rmsnorm_kernel(float* h, const T* delta, const float* parts, int n_parts, size_t part_stride,
                                   const int* rows, const float* __restrict__ w, float eps,
                                   int H, T* a) {
    __shared__ float red[33];
    extern __shared__ float vals[];  // H floats when gathering (h stays untouched)
    pdl_wait();
    pdl_launch_dependents();
    const size_t out_row = blockIdx.x;
    const size_t row = rows ? (size_t)rows[out_row] : out_row;
    float* hr = h + row * H;
    const T* dr = delta ? delta + row * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (dr) v += to_f(dr[i]);
        if (parts) {
            float d = 0.f;
            for (int k = 0; k < n_parts; k++) d += parts[(size_t)k * part_stride + row * H + i];
            v += d;
        }
        if (rows) vals[i] = v; else hr[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
    T* ar = a + out_row * H;
    const float* src = rows ? vals : hr;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ar[i] = from_f<T>(src[i] * rs * w[i]);
}

// The same for few rows (decode, and short prefill steps whose products leave partial sums), built
// for latency: one block per row, one or two groups of 4 columns a thread, values kept in registers
// between the two passes, every load of a pass requested before any is used, and what never comes
// from the kernel before this one (norm weight, row index) fetched before the wait for it.
// H % 4 == 0, H <= 8192.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = o;
}
template <typename T, int QPT>
__global__ void add_rmsnorm_quad_kernel(float* h, const T* delta, const float* parts, int n_parts, size_t part_stride,
                                        const int* rows, const float* __restrict__ w, float eps, int H, T* a) {
    __shared__ float red[33];
    // QPT groups of 4 columns a thread: group q of thread t is columns 4 * (t + q * blockDim.x) ...
    const size_t out_row = blockIdx.x;
    const size_t row = rows ? (size_t)rows[out_row] : out_row;
    float4 w4[QPT];
#pragma unroll
    for (int q = 0; q < QPT; q++) {
        const int c = (threadIdx.x + q * blockDim.x) * 4;
        w4[q] = c < H ? ld4(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_launch_dependents();   // before the wait: see pdl_launch_dependents
    pdl_wait();
    float4 v[QPT];
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < QPT; q++) {
        const int c = (threadIdx.x + q * blockDim.x) * 4;
        v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < H) {
            v[q] = ld4(h + row * H + c);
            if (delta) {
                const float4 d = ld4(delta + row * H + c);
                v[q].x += d.x, v[q].y += d.y, v[q].z += d.z, v[q].w += d.w;
            }
            if (parts) {
                float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
                for (int k = 0; k < n_parts; k++) {
                    const float4 p = ld4(parts + (size_t)k * part_stride + row * H + c);
                    d.x += p.x, d.y += p.y, d.z += p.z, d.w += p.w;
                }
                v[q].x += d.x, v[q].y += d.y, v[q].z += d.z, v[q].w += d.w;
            }
            if (!rows && (delta || parts)) st4(h + row * H + c, v[q]);
        }
        ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int q = 0; q < QPT; q++) {
        const int c = (threadIdx.x + q * blockDim.x) * 4;
        if (c < H)
            st4(a + out_row * H + c, make_float4(v[q].x * rs * w4[q].x, v[q].y * rs * w4[q].y, v[q].z * rs * w4[q].z, v[q].w * rs * w4[q].w));
    }
}

// out[r, c] = silu(gu[r, c]) * gu[r, I + c],  gu rows are [gate | up] of width 2*I
template <typename T>
__global__ void silu_mul_kernel(const T* gu, T* out, size_t n, int I) {
    pdl_wait();
    pdl_launch_dependents();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    size_t r = idx / I, c = idx % I;
    float g = to_f(gu[r * 2 * I + c]);
    float u = to_f(gu[r * 2 * I + I + c]);
    out[idx] = from_f<T>(g / (1.f + expf(-g)) * u);
}

// ---------------------------------------------------------------------------------------------
// One warp per (token, head) over nh query heads, nkv key heads and nkv value heads of a fused
// projection row qkv[t] = [q | k | v]. Query and key heads: optional RMSNorm over the head
// (weights qn / kn), optional rotate-half rotation by the angle table at the token's position.
// q goes to q_out [T, nh*hd]; k and v go to the token's place in the paged cache (unless
// write_kv == 0, for a layer that reads another layer's keys and values).
// Tokens with position < 0 are padding: nothing is written for them.
// With ``parts`` the projection row is the sum of n_parts float32 partial rows
// parts[k][t][heads*hd] (split-K output of the skinny product) instead of qkv[t].
// With ``dense_out`` every head (q, k and v) goes to its place in dense_out [T, heads*hd] instead,
// and nothing else is written: the step between a norm and a position encoding that a part
// applies itself before the cache is written.
template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* qkv, const float* parts, int n_parts, size_t part_stride, T* q_out,
                                          T* dense_out,
                                          const float* __restrict__ qn, const float* __restrict__ kn,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          const int* row_pos, const int* row_seq,
                                          const int* page_table, int pt_stride,
                                          T* k_store, T* v_store, int n_tok, int nh,
                                          int nkv, int hd, float eps, int write_kv) {
    // Positions, page ids, angles and norm weights never come from the kernel before this one (the
    // projection): they are fetched before the wait for it, and the projection row in one batch
    // after it, so that the wait is followed by one trip to memory, not five.
    const int lane = threadIdx.x & 31;
    const int heads = nh + 2 * nkv;
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const bool live = wid < (long long)n_tok * heads;
    const int t = live ? (int)(wid / heads) : 0, hidx = live ? (int)(wid % heads) : 0;
    const int pos = live ? row_pos[t] : -1;
    const int half = hd >> 1;
    const bool is_q = hidx < nh, is_v = hidx >= nh + nkv;
    const bool work = pos >= 0 && (is_q || write_kv || dense_out != nullptr);
    T* dst = nullptr;
    if (work) {
        if (dense_out != nullptr) {
            dst = dense_out + ((size_t)t * heads + hidx) * hd;
        } else if (is_q) {
            dst = q_out + ((size_t)t * nh + hidx) * hd;
        } else {
            const int kvh = (hidx - nh) % nkv;
            const int page = page_table[(size_t)row_seq[t] * pt_stride + pos / DK_PAGE];
            dst = (is_v ? v_store : k_store) + kv_offset(page, nkv, kvh, pos % DK_PAGE, hd);
        }
    }
    const float* nw = is_q ? qn : kn;
    float c[4], sn[4], w1[4], w2[4];   // pairs (d, d + half), d = lane + 32*i; hd <= 256 gives at most 4 pairs a lane
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane + 32 * i;
        const bool on = work && !is_v && d < half;
        c[i] = on && cos_t ? cos_t[(size_t)pos * half + d] : 1.f;
        sn[i] = on && cos_t ? sin_t[(size_t)pos * half + d] : 0.f;
        w1[i] = on && nw ? nw[d] : 1.f;
        w2[i] = on && nw ? nw[d + half] : 1.f;
    }
    pdl_launch_dependents();   // before the wait (see pdl_launch_dependents): what decode attention does before its own wait
    pdl_wait();                // reads positions, page ids and cache pages of older tokens, none of them written in this step
    if (!work) return;
    const size_t x_off = (size_t)t * heads * hd + (size_t)hidx * hd;
    float x1[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
    if (parts == nullptr) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = lane + 32 * i;
            if (d < half) x1[i] = to_f(qkv[x_off + d]), x2[i] = to_f(qkv[x_off + d + half]);
        }
    } else {
#pragma unroll 4
        for (int k = 0; k < n_parts; k++) {
            const float* pk = parts + (size_t)k * part_stride + x_off;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int d = lane + 32 * i;
                if (d < half) x1[i] += pk[d], x2[i] += pk[d + half];
            }
        }
    }
    if (is_v) {  // value head: plain copy
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int d = lane + 32 * i;
            if (d < half) dst[d] = from_f<T>(x1[i]), dst[d + half] = from_f<T>(x2[i]);
        }
        return;
    }
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) ss += x1[i] * x1[i] + x2[i] * x2[i];
        ss = warp_sum(ss);
        const float rs = rsqrtf(ss / (float)hd + eps);
#pragma unroll
        for (int i = 0; i < 4; i++) x1[i] = x1[i] * rs * w1[i], x2[i] = x2[i] * rs * w2[i];
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane + 32 * i;
        if (d < half) {
            float o1 = x1[i], o2 = x2[i];
            if (cos_t) {
                o1 = x1[i] * c[i] - x2[i] * sn[i];
                o2 = x2[i] * c[i] + x1[i] * sn[i];
            }
            dst[d] = from_f<T>(o1);
            dst[d + half] = from_f<T>(o2);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// out[i] = src[rows[i]] for rows of H floats (positions whose logits are wanted)
__global__ void gather_rows_f32_kernel(const float* src, const int* rows,
                                       float* out, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const float* s = src + (size_t)rows[blockIdx.x] * H;
    float* o = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = s[i];
}

// ---------------------------------------------------------------------------------------------
// Wide variants for many rows of bfloat16 (prefill): 16-byte accesses instead of 2-byte ones.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x, f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

// silu(gate) * up, 8 outputs a thread; I % 8 == 0.
__global__ void silu_mul_wide_kernel(const bf16* gu, bf16* out, size_t n8, int I8) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n8) return;
    const size_t r = idx / I8, c = idx % I8;
    const uint4* row = reinterpret_cast<const uint4*>(gu) + r * 2 * I8;
    float g[8], u[8], o[8];
    unpack8(row[c], g);
    unpack8(row[I8 + c], u);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = g[i] / (1.f + expf(-g[i])) * u[i];
    reinterpret_cast<uint4*>(out)[idx] = pack8(o);
}

// h += delta; a = rmsnorm(h) * w for bfloat16 delta / a, 8 elements a thread per pass, values kept
// in registers between the two passes. H % 8 == 0 and H <= 8 * 4 * blockDim.x.
__global__ void add_rmsnorm_wide_kernel(float* h, const bf16* delta, const float* __restrict__ w, float eps, int H, bf16* a) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row = blockIdx.x;
    float4* hr = reinterpret_cast<float4*>(h + row * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * H) : nullptr;
    const int n8 = H / 8;
    float v[4][8];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n8) {
            const float4 x0 = hr[2 * i], x1 = hr[2 * i + 1];
            v[it][0] = x0.x, v[it][1] = x0.y, v[it][2] = x0.z, v[it][3] = x0.w;
            v[it][4] = x1.x, v[it][5] = x1.y, v[it][6] = x1.z, v[it][7] = x1.w;
            if (dr) {
                float d[8];
                unpack8(dr[i], d);
#pragma unroll
                for (int k = 0; k < 8; k++) v[it][k] += d[k];
                hr[2 * i] = make_float4(v[it][0], v[it][1], v[it][2], v[it][3]);
                hr[2 * i + 1] = make_float4(v[it][4], v[it][5], v[it][6], v[it][7]);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) ss += v[it][k] * v[it][k];
        }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
    uint4* ar = reinterpret_cast<uint4*>(a + row * H);
    const float4* wr = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int i = threadIdx.x + it * blockDim.x;
        if (i < n8) {
            const float4 w0 = wr[2 * i], w1 = wr[2 * i + 1];
            float o[8] = {v[it][0] * rs * w0.x, v[it][1] * rs * w0.y, v[it][2] * rs * w0.z, v[it][3] * rs * w0.w,
                          v[it][4] * rs * w1.x, v[it][5] * rs * w1.y, v[it][6] * rs * w1.z, v[it][7] * rs * w1.w};
            ar[i] = pack8(o);
        }
    }
}

// The same with one warp per row (H % 256 == 0, H <= 4096): every load of the row is requested
// before any is used, the sum of squares needs shuffles only, and no block barrier is on the path.
template <int CH>   // CH = H / 256 chunks of 8 elements per lane
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* h, const bf16* delta, const float* __restrict__ w, float eps, int n_rows, bf16* a) {
    constexpr int H = CH * 256;
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (size_t)n_rows) return;
    float4* hr = reinterpret_cast<float4*>(h + row * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * H) : nullptr;
    float v[CH][8];
    uint4 d8[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
        const int i = c * 32 + lane;          // index of this lane's 8 elements
        const float4 x0 = hr[2 * i], x1 = hr[2 * i + 1];
        v[c][0] = x0.x, v[c][1] = x0.y, v[c][2] = x0.z, v[c][3] = x0.w;
        v[c][4] = x1.x, v[c][5] = x1.y, v[c][6] = x1.z, v[c][7] = x1.w;
        if (dr) d8[c] = dr[i];
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; c++) {
        const int i = c * 32 + lane;
        if (dr) {
            float d[8];
            unpack8(d8[c], d);
#pragma unroll
            for (int k = 0; k < 8; k++) v[c][k] += d[k];
            hr[2 * i] = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
            hr[2 * i + 1] = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) ss += v[c][k] * v[c][k];
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)H + eps);
    uint4* ar = reinterpret_cast<uint4*>(a + row * H);
    const float4* wr = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int c = 0; c < CH; c++) {
        const int i = c * 32 + lane;
        const float4 w0 = wr[2 * i], w1 = wr[2 * i + 1];
        float o[8] = {v[c][0] * rs * w0.x, v[c][1] * rs * w0.y, v[c][2] * rs * w0.z, v[c][3] * rs * w0.w,
                      v[c][4] * rs * w1.x, v[c][5] * rs * w1.y, v[c][6] * rs * w1.z, v[c][7] * rs * w1.w};
        ar[i] = pack8(o);
    }
}

// q/k norm + rotation + cache write for bfloat16 with head sizes that are multiples of 16. A group
// of GS lanes (GS = the power of two >= head_dim / 16) takes one (token, head); a warp takes 32 / GS
// of them. Lane j of a group holds elements [8j, 8j+8) of each half of the head.
template <int GS>
__global__ void qk_norm_rope_write_wide_kernel(const bf16* qkv, bf16* q_out, bf16* dense_out, const float* __restrict__ qn,
                                               const float* __restrict__ kn, const float* __restrict__ cos_t,
                                               const float* __restrict__ sin_t, const int* row_pos, const int* row_seq,
                                               const int* page_table, int pt_stride, bf16* k_store, bf16* v_store,
                                               int n_tok, int nh, int nkv, int hd, float eps, int write_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, j = lane % GS;
    const int heads = nh + 2 * nkv;
    const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (32 / GS) + lane / GS;
    const bool live = item < (long long)n_tok * heads;
    const int t = live ? (int)(item / heads) : 0, hidx = live ? (int)(item % heads) : 0;
    const int pos = live ? row_pos[t] : -1;
    const int half = hd >> 1, half8 = hd >> 4;
    const bool is_v = hidx >= nh + nkv;
    const bool work = pos >= 0 && (hidx < nh || write_kv || dense_out != nullptr);
    const bf16* x = qkv + (size_t)t * heads * hd + (size_t)hidx * hd;
    bf16* dst = nullptr;
    if (work) {
        if (dense_out != nullptr) {
            dst = dense_out + ((size_t)t * heads + hidx) * hd;
        } else if (hidx < nh) {
            dst = q_out + ((size_t)t * nh + hidx) * hd;
        } else {
            const int kvh = (hidx - nh) % nkv;
            const int page = page_table[(size_t)row_seq[t] * pt_stride + pos / DK_PAGE];
            dst = (hidx < nh + nkv ? k_store : v_store) + kv_offset(page, nkv, kvh, pos % DK_PAGE, hd);
        }
    }
    const bool on = work && j < half8;
    float x1[8], x2[8];
    float ss = 0.f;
    if (on) {
        const uint4 r1 = reinterpret_cast<const uint4*>(x)[j], r2 = reinterpret_cast<const uint4*>(x + half)[j];
        if (is_v) {  // value head: plain copy
            reinterpret_cast<uint4*>(dst)[j] = r1;
            reinterpret_cast<uint4*>(dst + half)[j] = r2;
        }
        unpack8(r1, x1);
        unpack8(r2, x2);
#pragma unroll
        for (int i = 0; i < 8; i++) ss += x1[i] * x1[i] + x2[i] * x2[i];
    }
#pragma unroll
    for (int o = GS / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // within the group of GS lanes
    if (!on || is_v) return;
    const float* nw = hidx < nh ? qn : kn;
    const float rs = nw ? rsqrtf(ss / (float)hd + eps) : 1.f;
    // weights and angles of this lane's 8 + 8 elements: 16-byte loads (hd % 16 == 0 keeps them aligned)
    float w1[8], w2[8], cs[8], sn[8];
    auto load8 = [](const float* p, float (&f)[8]) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    };
    if (nw) load8(nw + 8 * j, w1), load8(nw + half + 8 * j, w2);
    if (cos_t) load8(cos_t + (size_t)pos * half + 8 * j, cs), load8(sin_t + (size_t)pos * half + 8 * j, sn);
    float o1[8], o2[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float a1 = x1[i] * rs, a2 = x2[i] * rs;
        if (nw) a1 *= w1[i], a2 *= w2[i];
        o1[i] = a1, o2[i] = a2;
        if (cos_t) {
            o1[i] = a1 * cs[i] - a2 * sn[i];
            o2[i] = a2 * cs[i] + a1 * sn[i];
        }
    }
    reinterpret_cast<uint4*>(dst)[j] = pack8(o1);
    reinterpret_cast<uint4*>(dst + half)[j] = pack8(o2);
}

// ---------------------------------------------------------------------------------------------
#define DISPATCH_T(dtype, ...)                         \
    if ((dtype) == 0) { typedef float T; __VA_ARGS__; } \
    else { typedef bf16 T; __VA_ARGS__; }

static inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

DK_EXPORT int dk_embed_rmsnorm(int dtype, const int* tok, const void* embed, const float* w, float eps,
                               int n_tok, int H, int V, float* h, void* a, cudaStream_t st) {
    DISPATCH_T(dtype, return dk_launch(embed_rmsnorm_kernel<T>, dim3(n_tok), dim3(row_threads(H)), 0, st, tok,
                                       (const T*)embed, w, eps, H, V, h, (T*)a));
}

DK_EXPORT int dk_add_rmsnorm(int dtype, float* h, const void* delta, const float* parts, int n_parts,
                             long long part_stride, const int* rows, const float* w, float eps, int n_rows, int H,
                             void* a, cudaStream_t st) {
    if (dtype == 1 && parts == nullptr && rows == nullptr && H % 256 == 0 && H <= 4096 && n_rows > 64) {
        // warps a block: eight when the rows are many; fewer when blocks of eight would leave the SMs
        // with one or two blocks each (2,048 rows: 256 blocks on 148 SMs, a quarter of them idle half the time)
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int wpb = 8;
        while (wpb > 1 && (n_rows + wpb - 1) / wpb < 8 * sms) wpb >>= 1;
        const dim3 grid((n_rows + wpb - 1) / wpb), block(32 * wpb);
#define NORM_WARP(CH)                                                                                                   \
    if (H == CH * 256)                                                                                                  \
        return dk_launch(add_rmsnorm_warp_kernel<CH>, grid, block, 0, st, h, (const bf16*)delta, w, eps, n_rows, (bf16*)a)
        NORM_WARP(1); NORM_WARP(2); NORM_WARP(3); NORM_WARP(4); NORM_WARP(5); NORM_WARP(6); NORM_WARP(7); NORM_WARP(8);
        NORM_WARP(9); NORM_WARP(10); NORM_WARP(11); NORM_WARP(12); NORM_WARP(13); NORM_WARP(14); NORM_WARP(15); NORM_WARP(16);
#undef NORM_WARP
    }
    if (dtype == 1 && parts == nullptr && rows == nullptr && H % 8 == 0 && H <= 8 * 4 * row_threads(H) && n_rows > 64)
        return dk_launch(add_rmsnorm_wide_kernel, dim3(n_rows), dim3(row_threads(H)), 0, st, h, (const bf16*)delta, w, eps,
                         H, (bf16*)a);
    if ((n_rows <= 64 || parts != nullptr) && H % 4 == 0 && H <= 8192 && part_stride % 4 == 0) {
        if (H <= 4096) {
            DISPATCH_T(dtype, return dk_launch(add_rmsnorm_quad_kernel<T, 1>, dim3(n_rows), dim3((H / 4 + 31) / 32 * 32), 0, st, h,
                                               (const T*)delta, parts, n_parts, (size_t)part_stride, rows, w, eps, H, (T*)a));
        }
        DISPATCH_T(dtype, return dk_launch(add_rmsnorm_quad_kernel<T, 2>, dim3(n_rows), dim3((H / 8 + 31) / 32 * 32), 0, st, h,
                                           (const T*)delta, parts, n_parts, (size_t)part_stride, rows, w, eps, H, (T*)a));
    }
    size_t smem = rows ? (size_t)H * sizeof(float) : 0;
    if (smem > 48 * 1024) {
        DISPATCH_T(dtype, cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem));
    }
    DISPATCH_T(dtype, return dk_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(row_threads(H)), smem, st, h,
                                       (const T*)delta, parts, n_parts, (size_t)part_stride, rows, w, eps, H, (T*)a));
}

DK_EXPORT int dk_silu_mul(int dtype, const void* gu, void* out, long long n_rows, int I, cudaStream_t st) {
    size_t n = (size_t)n_rows * I;
    if (dtype == 1 && I % 8 == 0)
        return dk_launch(silu_mul_wide_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, st, (const bf16*)gu,
                         (bf16*)out, n / 8, I / 8);
    DISPATCH_T(dtype, return dk_launch(silu_mul_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st,
                                       (const T*)gu, (T*)out, n, I));
}

DK_EXPORT int dk_qk_norm_rope_write(int dtype, const void* qkv, const float* parts, int n_parts, long long part_stride,
                                    void* q_out, void* dense_out, const float* qn, const float* kn,
                                    const float* cos_t, const float* sin_t, const int* row_pos, const int* row_seq,
                                    const int* page_table, int pt_stride, void* k_store, void* v_store, int n_tok,
                                    int nh, int nkv, int hd, float eps, int write_kv, cudaStream_t st) {
    if (hd % 2 != 0 || hd > 256) return (int)cudaErrorInvalidValue;
    long long warps = (long long)n_tok * (nh + 2 * nkv);
    unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == 1 && parts == nullptr && hd % 16 == 0 && n_tok > 64) {
        const int half8 = hd / 16;
        const int gs = half8 <= 1 ? 1 : half8 <= 2 ? 2 : half8 <= 4 ? 4 : half8 <= 8 ? 8 : 16;
        const unsigned wblocks = (unsigned)((warps + 4LL * (32 / gs) - 1) / (4LL * (32 / gs)));
#define ROPE_WIDE(GS)                                                                                                  \
    return dk_launch(qk_norm_rope_write_wide_kernel<GS>, dim3(wblocks), dim3(128), 0, st, (const bf16*)qkv, (bf16*)q_out, \
                     (bf16*)dense_out, qn, kn, cos_t, sin_t, row_pos, row_seq, page_table, pt_stride, (bf16*)k_store, (bf16*)v_store, n_tok, \
                     nh, nkv, hd, eps, write_kv)
        if (gs == 1) ROPE_WIDE(1);
        if (gs == 2) ROPE_WIDE(2);
        if (gs == 4) ROPE_WIDE(4);
        if (gs == 8) ROPE_WIDE(8);
        ROPE_WIDE(16);
#undef ROPE_WIDE
    }
    DISPATCH_T(dtype, return dk_launch(qk_norm_rope_write_kernel<T>, dim3(blocks), dim3(128), 0, st, (const T*)qkv,
                                       parts, n_parts, (size_t)part_stride, (T*)q_out, (T*)dense_out, qn, kn, cos_t, sin_t, row_pos, row_seq, page_table, pt_stride,
                                       (T*)k_store, (T*)v_store, n_tok, nh, nkv, hd, eps, write_kv));
}

DK_EXPORT int dk_gather_rows_f32(const float* src, const int* rows, float* out, int n_rows, int H, cudaStream_t st) {
    return dk_launch(gather_rows_f32_kernel, dim3(n_rows), dim3(256), 0, st, src, rows, out, H);
}
