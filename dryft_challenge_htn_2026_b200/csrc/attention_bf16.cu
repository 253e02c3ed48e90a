// bfloat16 causal grouped-query attention over the paged cache on the tensor cores
// (mma.sync m16n8k16, float32 scores / softmax / accumulators). Built once per head size with
// -DHD=<multiple of 16, at most 256>.
//
//  * prefill: ragged batch of query chunks; a block owns 64 consecutive queries of one sequence
//    and one query head (4 warps x 16 rows) and walks the key pages up to its diagonal.
//  * decode: one query token per sequence; a block owns the (up to 16) query heads that share a
//    kv head and one split of the keys; its 4 warps take 16 keys each of every 64-key page, each
//    through a cp.async ring of its own (2 or 3 chunks deep), and each leaves a partial result of
//    its own; the combine kernel merges the 4 x splits partial results of a head.
// Prefill stages key/value pages ([64, HD] per kv head, contiguous) with cp.async, two stages deep. P is rounded to bfloat16 before P.V; row sums use the unrounded values.
// Reference formulas: engine/fused.py:301-343 (prefill), :478-565 (split decode + combine).
#include "attention_mma.cuh"

constexpr size_t SMEM_BYTES = 2 * STAGE_ELEMS * sizeof(bf16);

// All threads of the block copy one page (K and V of kv head kvh) into a stage.
__device__ __forceinline__ void stage_page(bf16* stage, const bf16* k_store, const bf16* v_store, int page, int nkv,
                                           int kvh) {
    const size_t off = kv_offset(page, nkv, kvh, 0, HD);
    constexpr int CPR = HD / 8;  // 16-byte chunks per row
    for (int c = threadIdx.x; c < DK_PAGE * CPR; c += blockDim.x) {
        const int row = c / CPR, col = (c % CPR) * 8;
        cp_async16(stage + row * KSTR + col, k_store + off + (size_t)row * HD + col);
        cp_async16(stage + TILE_ELEMS + row * KSTR + col, v_store + off + (size_t)row * HD + col);
    }
}

// ------------------------------------------------------------------------------------- prefill
// grid (nh, tiles). tiles[2i] = sequence, tiles[2i+1] = first query of the tile within the
// sequence's chunk. cu_q: first flat row of each sequence's chunk; seq_pos0: tokens already cached
// before the chunk (the chunk's own keys are in the cache when this runs).
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const bf16* q, bf16* out, const bf16* k_store, const bf16* v_store, const int* tiles,
                    const int* cu_q, const int* seq_pos0, const int* page_table, int pt_stride, int nh, int nkv,
                    int window, float sl2) {
    extern __shared__ __align__(16) bf16 smem[];
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    // heads vary fastest: blocks start in launch order, so every head's heaviest tile (the tiles
    // are sorted by the keys they see) starts before any light one, and the light ones fill the end
    const int seq = tiles[2 * blockIdx.y], q0 = tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x, kvh = h / (nh / nkv);
    const int q_len = cu_q[seq + 1] - cu_q[seq];
    const int pos0 = seq_pos0[seq];
    const int rows_here = min(64, q_len - q0);
    const int* pt = page_table + (size_t)seq * pt_stride;

    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;  // rows within the chunk
    const bool ok0 = r0 < q_len, ok1 = r1 < q_len;
    const size_t flat0 = (size_t)(cu_q[seq] + r0), flat1 = (size_t)(cu_q[seq] + r1);
    uint32_t qf[HD / 16][4];
    load_q_frags(qf, ok0 ? q + (flat0 * nh + h) * HD : nullptr, ok1 ? q + (flat1 * nh + h) * HD : nullptr);
    int lo[2], hi[2];
    hi[0] = ok0 ? pos0 + r0 : -1;
    hi[1] = ok1 ? pos0 + r1 : -1;
    lo[0] = window > 0 ? max(0, hi[0] - window + 1) : 0;
    lo[1] = window > 0 ? max(0, hi[1] - window + 1) : 0;
    // keys this warp's 16 rows can see at all
    const int w_first = pos0 + q0 + warp * 16;
    const int w_hi = min(w_first + 15, pos0 + q_len - 1);
    const int w_lo = window > 0 ? max(0, w_first - window + 1) : 0;

    const int max_pos = pos0 + q0 + rows_here - 1;
    const int min_pos = pos0 + q0;
    const int jt_hi = max_pos / DK_PAGE;
    const int jt_lo = window > 0 ? max(0, min_pos - window + 1) / DK_PAGE : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    stage_page(smem, k_store, v_store, pt[jt_lo], nkv, kvh);
    cp_async_commit();
    for (int jt = jt_lo; jt <= jt_hi; jt++) {
        const int cur = (jt - jt_lo) & 1;
        if (jt < jt_hi) stage_page(smem + (cur ^ 1) * STAGE_ELEMS, k_store, v_store, pt[jt + 1], nkv, kvh);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const int key0 = jt * DK_PAGE;
        if (key0 <= w_hi && key0 + DK_PAGE - 1 >= w_lo && warp * 16 < rows_here) {
            const bf16* Ks = smem + cur * STAGE_ELEMS;
            warp_attend<DK_PAGE>(qf, Ks, Ks + TILE_ELEMS, key0, lo, hi, sl2, m, l, acc);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const float inv0 = ok0 ? 1.f / l[0] : 0.f, inv1 = ok1 ? 1.f / l[1] : 0.f;
#pragma unroll
    for (int nt = 0; nt < HD / 8; nt++) {
        const int d = nt * 8 + 2 * t;
        if (ok0) *reinterpret_cast<uint32_t*>(out + (flat0 * nh + h) * HD + d) = pack_bf16(acc[nt][0] * inv0, acc[nt][1] * inv0);
        if (ok1) *reinterpret_cast<uint32_t*>(out + (flat1 * nh + h) * HD + d) = pack_bf16(acc[nt][2] * inv1, acc[nt][3] * inv1);
    }
}

// -------------------------------------------------------------------------------------- decode
// grid (nsplit, nkv * mtiles, sequences), mtiles = ceil(G / 16). row_pos[b] is the position of
// sequence b's one query token (its key is already cached); < 0 marks a padding row.
// nsplit == 1: writes out directly. Otherwise writes float32 partials
// ws_acc [(b*nh + head)*nsplit + split][HD] and ws_ml [...][2] = (max in log2 domain, row sum).
template <int D>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const bf16* q, float* ws_acc, float* ws_ml, const bf16* k_store, const bf16* v_store,
                   const int* row_pos, const int* page_table, int pt_stride, int nh, int nkv, int window, float sl2) {
    extern __shared__ __align__(16) bf16 smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int G = nh / nkv, mtiles = (G + 15) / 16;
    const int split = blockIdx.x, nsplit = gridDim.x;
    const int kvh = blockIdx.y / mtiles, mt = blockIdx.y % mtiles;
    const int b = blockIdx.z;
    const int head0 = kvh * G + mt * 16;
    const int heads_here = min(16, G - mt * 16);
    // Every warp streams its own 16 keys of each page (rows 16w..16w+15 of K and of V) through a
    // ring of D chunks of its own: no block barrier until the warps' results are merged.
    // Positions and page tables are not written by the kernel before this one, and of the cache
    // only the page of the newest token is (its key and value were just stored): chunks of older
    // pages are requested before the wait for that kernel.
    constexpr int CHUNK = 2 * 16 * KSTR;      // elements: 16 keys then 16 values
    constexpr int CPR = HD / 8;               // 16-byte pieces per row
    bf16* ring = smem + warp * D * CHUNK;
    const int pos = row_pos[b];
    const int* pt = page_table + (size_t)b * pt_stride;
    const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int t_lo = key_lo / DK_PAGE, t_hi = pos / DK_PAGE;
    const int per = (t_hi - t_lo + 1 + nsplit - 1) / nsplit;
    const int jt0 = t_lo + split * per, jt1 = pos >= 0 ? min(t_hi + 1, jt0 + per) : jt0;  // [jt0, jt1)
    const uint64_t stream_once = l2_evict_first();
    auto fetch = [&](int jt, int slot) {
        const size_t off = kv_offset(pt[jt], nkv, kvh, warp * 16, HD);
        bf16* dst = ring + slot * CHUNK;
        for (int c = lane; c < 16 * CPR; c += 32) {
            const int row = c / CPR, col = (c % CPR) * 8;
            cp_async16(dst + row * KSTR + col, k_store + off + (size_t)row * HD + col, stream_once);
            cp_async16(dst + 16 * KSTR + row * KSTR + col, v_store + off + (size_t)row * HD + col, stream_once);
        }
    };
    int issued = 0;                           // chunks requested so far; chunk i is commit group i
    for (; issued < D && jt0 + issued < min(jt1, t_hi); issued++) {
        fetch(jt0 + issued, issued);
        cp_async_commit();
    }
    pdl_wait();
    pdl_launch_dependents();
    for (; issued < D; issued++) {            // the rest of the ring (the newest page, or nothing)
        if (jt0 + issued < jt1) fetch(jt0 + issued, issued);
        cp_async_commit();
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float acc[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    if (jt0 < jt1) {
        uint32_t qf[HD / 16][4];
        const bf16* qb = q + ((size_t)b * nh + head0) * HD;
        load_q_frags(qf, g < heads_here ? qb + (size_t)g * HD : nullptr,
                     g + 8 < heads_here ? qb + (size_t)(g + 8) * HD : nullptr);
        const int lo[2] = {key_lo, key_lo}, hi[2] = {pos, pos};
        for (int jt = jt0; jt < jt1; jt++) {
            const int slot = (jt - jt0) % D;
            cp_async_wait<D - 1>();           // this warp's chunk jt has landed
            __syncwarp();
            const int key0 = jt * DK_PAGE + warp * 16;
            if (key0 <= pos && key0 + 15 >= key_lo) {
                const bf16* Ks = ring + slot * CHUNK;
                warp_attend<16>(qf, Ks, Ks + 16 * KSTR, key0, lo, hi, sl2, m, l, acc);
            }
            __syncwarp();                     // every lane is done reading the slot before it is refilled
            if (jt + D < jt1) fetch(jt + D, slot);
            cp_async_commit();
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    // Every warp saw different keys and stores its own partial result: part 4 * split + warp of
    // 4 * nsplit a head. (Adding the four up inside the block first, through shared memory and two
    // block barriers, cost 3.8 us of the kernel's 18.)
    const int parts = 4 * nsplit, part = 4 * split + warp;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const int row = g + 8 * r;
        if (row < heads_here) {
            const size_t at = ((size_t)b * nh + head0 + row) * parts + part;
            float* dst = ws_acc + at * HD + 2 * t;
#pragma unroll
            for (int nt = 0; nt < HD / 8; nt++) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(acc[nt][2 * r], acc[nt][2 * r + 1]);
            if (t == 0) *reinterpret_cast<float2*>(ws_ml + at * 2) = make_float2(m[r], l[r]);
        }
    }
}

// grid (sequences * nh / 4), 128 threads: a warp merges the parts of one head (at most 128). Lane s
// holds the (max, sum) of parts s, s + 32, s + 64 and s + 96; the partial outputs of the first 16
// parts are requested together with them, so up to 16 parts cost one trip to memory after the wait.
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* ws_acc, const float* ws_ml, bf16* out, int parts, int n_heads) {
    pdl_launch_dependents();   // before the wait: see pdl_launch_dependents
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t head = (size_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (head >= (size_t)n_heads) return;
    const float2* ml = reinterpret_cast<const float2*>(ws_ml) + head * parts;
    const float* wa = ws_acc + head * parts * HD;
    const float2 none = make_float2(-INFINITY, 0.f);
    float2 pm[4];
#pragma unroll
    for (int k = 0; k < 4; k++) pm[k] = lane + 32 * k < parts ? ml[lane + 32 * k] : none;
    float fw[4] = {0.f, 0.f, 0.f, 0.f}, inv = 0.f;
    for (int base = 0; base < HD; base += 128) {
        const int d0 = base + lane * 4;
        const bool ok = d0 < HD;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < parts; s0 += 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; u++)
                v[u] = ok && s0 + u < parts ? *reinterpret_cast<const float4*>(wa + (size_t)(s0 + u) * HD + d0)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            if (base == 0 && s0 == 0) {       // the weights of the parts, once
                float M = fmaxf(fmaxf(pm[0].x, pm[1].x), fmaxf(pm[2].x, pm[3].x));
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
                float L = 0.f;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    fw[k] = M == -INFINITY ? 0.f : exp2f(pm[k].x - M);
                    L += pm[k].y * fw[k];
                }
#pragma unroll
                for (int d = 16; d >= 1; d >>= 1) L += __shfl_xor_sync(0xffffffffu, L, d);
                inv = L > 0.f ? 1.f / L : 0.f;
            }
            const float fsrc = fw[s0 >> 5];         // a run of 16 parts lies in one group of 32
#pragma unroll
            for (int u = 0; u < 16; u++) {
                const float f = __shfl_sync(0xffffffffu, fsrc, (s0 + u) & 31);
                a.x += v[u].x * f, a.y += v[u].y * f, a.z += v[u].z * f, a.w += v[u].w * f;
            }
        }
        if (ok) {
            uint2 o;
            o.x = pack_bf16(a.x * inv, a.y * inv);
            o.y = pack_bf16(a.z * inv, a.w * inv);
            *reinterpret_cast<uint2*>(out + head * HD + d0) = o;
        }
    }
}

constexpr size_t decode_smem(int depth) { return (size_t)4 * depth * 2 * 16 * KSTR * sizeof(bf16); }

// ring depth: three chunks a warp while all blocks fit two to an SM, else two (three to an SM)
static int decode_ring_depth(long long blocks) {
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return blocks <= 2LL * sms && 2 * (decode_smem(3) + 1024) <= 227 * 1024 ? 3 : 2;
}

static int ensure_smem_attr() {
    static bool done = false;
    if (done) return 0;
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(attn_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(2));
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(attn_decode_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(3));
    if (e != cudaSuccess) return (int)e;
    done = true;
    return 0;
}

DK_EXPORT int dk_attn_head_dim() { return HD; }

DK_EXPORT int dk_attn_prefill_bf16(const void* q, void* out, const void* k_store, const void* v_store, const int* tiles,
                                   int n_tiles, const int* cu_q, const int* seq_pos0, const int* page_table,
                                   int pt_stride, int nh, int nkv, int window, float scale, cudaStream_t st) {
    if (nh % nkv != 0) return (int)cudaErrorInvalidValue;
    int e = ensure_smem_attr();
    if (e) return e;
    return dk_launch(attn_prefill_kernel, dim3(nh, n_tiles), dim3(128), SMEM_BYTES, st, (const bf16*)q, (bf16*)out,
                     (const bf16*)k_store, (const bf16*)v_store, tiles, cu_q, seq_pos0, page_table, pt_stride, nh, nkv,
                     window, scale * 1.4426950408889634f);
}

// ws_acc: n_seq * nh * 4 * nsplit * HD floats, ws_ml: n_seq * nh * 4 * nsplit * 2 floats: every warp of a
// block leaves a partial result of its own, the merge kernel adds up the 4 * nsplit of a head (nsplit <= 32).
DK_EXPORT int dk_attn_decode_bf16(const void* q, void* out, float* ws_acc, float* ws_ml, const void* k_store,
                                  const void* v_store, const int* row_pos, const int* page_table, int pt_stride,
                                  int n_seq, int nh, int nkv, int window, float scale, int nsplit, cudaStream_t st) {
    if (nh % nkv != 0 || nsplit < 1 || nsplit > 32 || ws_acc == nullptr || ws_ml == nullptr) return (int)cudaErrorInvalidValue;
    int e = ensure_smem_attr();
    if (e) return e;
    const int G = nh / nkv, mtiles = (G + 15) / 16;
    if (decode_ring_depth((long long)nsplit * nkv * mtiles * n_seq) == 3)
        e = dk_launch(attn_decode_kernel<3>, dim3(nsplit, nkv * mtiles, n_seq), dim3(128), decode_smem(3), st, (const bf16*)q,
                      ws_acc, ws_ml, (const bf16*)k_store, (const bf16*)v_store, row_pos, page_table, pt_stride, nh, nkv,
                      window, scale * 1.4426950408889634f);
    else
        e = dk_launch(attn_decode_kernel<2>, dim3(nsplit, nkv * mtiles, n_seq), dim3(128), decode_smem(2), st, (const bf16*)q,
                      ws_acc, ws_ml, (const bf16*)k_store, (const bf16*)v_store, row_pos, page_table, pt_stride, nh, nkv,
                      window, scale * 1.4426950408889634f);
    if (e) return e;
    return dk_launch(attn_combine_kernel, dim3((n_seq * nh + 3) / 4), dim3(128), 0, st, (const float*)ws_acc,
                     (const float*)ws_ml, (bf16*)out, 4 * nsplit, n_seq * nh);
}
