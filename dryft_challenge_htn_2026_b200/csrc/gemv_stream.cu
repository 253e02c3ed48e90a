// The decode-side weight-streaming product for up to 16 rows of x in bfloat16:
// out[M,N] = x[M,K] . W[N,K]^T, the same contract and epilogues as gemv_bf16 in gemm.cu
// (0 store bf16, 1 store float32, 2 W = [gate; up]: store silu(gate)*up; split-K partial sums).
//
// Persistent blocks of four streaming warps and an epilogue warp, two per SM. K is cut into SK slices; block b works on slice
// b % SK only, so its piece of x (at most 16 rows x 2560 elements) is copied into shared memory
// once and every weight byte that follows is the only traffic. The block walks tiles of 16 weight
// rows; a tile's slice is cut into stages of 256 elements of K, and stage number i of the block
// belongs to warp i % 4, which both fetches and multiplies it: it copies the stage's 16 weight
// rows into its own two-deep ring in shared memory with cp.async (one instruction per row: the 32
// lanes fetch 512 contiguous bytes of that row, and the next stages continue the same rows) and
// multiplies from shared memory on the tensor cores (ldmatrix + mma.sync, float32 accumulation).
// At the end of a tile the four warps leave their sums in shared memory for a fifth warp, which adds
// them up, applies the epilogue and stores, while the four go on streaming the next tile (two
// buffers, handed over with named barriers: waiting for the slowest warp at every tile cost 11 to
// 17 % of the kernel). There is no waiting on flags: the only waits are cp.async.wait_group and
// block barriers.
//
// Programmatic dependent launch: every warp issues the weight copies of its first stages before it
// waits for the previous kernel (weights never depend on it); x is fetched after the wait, one bulk
// copy a row by the TMA engine counted on an mbarrier (as 16-byte cp.async pieces, which queue behind
// the weight copies in the same load path, the rows of x cost 0.5 to 1.7 us of a product).
//
// (Measured on the way here: for the weights, bulk copies of the TMA engine at 512 bytes a request
// were bound by the engine's request rate; register streaming in the mma fragment layout, which touches 128
// bytes of 16 rows at a time, stayed near 4.9 TB/s; re-fetching x with every stage cost half as
// much SM ingress again as the weights.)
//
// Two fusions with the residual stream of a pre-norm block, so that a decode step needs no
// separate add+norm launch between its products:
//  * FUSE 2 (the producer): the product is added into the float32 residual stream h_out [M,N] in
//    place. With SK > 1 the slices of a tile meet through a counter: every block stores its
//    partial sums, the block that draws the last ticket adds the slices up in slice order (so the
//    result does not depend on which block that is) and owns the tile's piece of h_out. It also
//    stores the tile's contribution to every row's sum of squares of the new h, sq_out[tile][16].
//  * FUSE 1 (the consumer): x is not given; the block makes it from the residual stream,
//    x = h_in * rsqrt(sum(sq_in) / K + eps) * norm_w in bfloat16, while it fills shared memory.
// Requires K % 16 == 0, 16-byte aligned x and W, a slice of at most XMAX elements.
#include "common.cuh"

#ifdef DK_TRACE
__device__ unsigned long long gs_phase[4][8];
__device__ __forceinline__ void gs_note(int ph) {
    if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == 100 || blockIdx.x == 200 || blockIdx.x == 295)) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        gs_phase[blockIdx.x / 100 > 2 ? 3 : blockIdx.x / 100][ph] = t;
    }
}
DK_EXPORT int dk_gs_phases(unsigned long long* out) { cudaDeviceSynchronize(); return (int)cudaMemcpyFromSymbol(out, gs_phase, sizeof(gs_phase)); }
#define GS_NOTE(p) gs_note(p)
#else
#define GS_NOTE(p)
#endif

namespace {

constexpr int STAGE_K = 256;                  // elements of K per stage
constexpr int ROW_STRIDE = STAGE_K * 2 + 16;  // bytes between rows of a stage: 16 of padding keep ldmatrix conflict-free
#ifndef GS_DEPTH
#define GS_DEPTH 2
#endif
#ifndef GS_WARPS
#define GS_WARPS 4
#endif
constexpr int DEPTH = GS_DEPTH;               // stages a warp has in flight
constexpr int WARPS = GS_WARPS;
constexpr int WR = 16;                        // weight rows per stage
constexpr int STAGE_BYTES = WR * ROW_STRIDE;
constexpr int XMAX = 2560;                    // longest slice of K whose x rows are kept in shared memory

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16-byte asynchronous copy global -> shared, not kept in L1; `real` false writes zeros instead.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool real) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(real ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// 16-byte load that stays where it is written: the compiler keeps volatile asm in order, so a run
// of these is in flight together instead of each sinking to its use
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// Slice length for SK slices of K: a multiple of 16.
__host__ __device__ __forceinline__ int slice_len(int K, int SK) { return ((K + SK - 1) / SK + 15) / 16 * 16; }

struct Fuse {
    const float* h_in;    // FUSE 1: residual stream [M,K]
    const float* sq_in;   //         [sq_tiles][16] sums of squares of its rows, in any number of pieces
    const float* norm_w;  //         [K]
    float eps;
    int sq_tiles;
    float* h_out;         // FUSE 2: residual stream [M,N], += product
    float* sq_out;        //         [tiles][16]
    int* counters;        //         [tiles], zero before and after every launch
    const char* pf;       // a hint: [pf, pf + pf_bytes) (the next product's weights) is asked into L2
    size_t pf_bytes;
};

// MR: rows of x kept (8 or 16, M <= MR). MODE as in gemm.cu. Mode 2: a tile's rows 0-7 are the
// gate rows of 8 outputs and rows 8-15 their up rows, so a tile covers 8 outputs.
// gridDim.x is a multiple of SK: block b has slice b % SK and tiles b / SK, + gridDim.x / SK, ...
// (Dealing the rows out evenly instead, in tiles of unequal heights, was measured 15 % slower: the
// bytes a ring slot holds in flight shrink with the tile, and the kernel lives on bytes in flight.)
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// FUSE 0 and 1 run with a fifth warp for the epilogues; FUSE 2, whose epilogue meets other blocks,
// keeps the four warps doing it together.
template <int FUSE> struct Shape {
    static constexpr bool EPI = FUSE != 2;
    static constexpr int THREADS = (WARPS + (EPI ? 1 : 0)) * 32;
    static constexpr int RED_BUFS = EPI ? 2 : 1;
};

template <int MR, int MODE, int FUSE>
__global__ void __launch_bounds__(Shape<FUSE>::THREADS)
gemv_stream_kernel(const bf16* x, const bf16* __restrict__ W, void* out, float* ws, int M, int N, int K, int SK,
                   int tiles, Fuse fu) {
    __shared__ float rstd_s[16];
    __shared__ int last_flag;
    __shared__ __align__(8) uint64_t x_bar;   // counts the bytes of x's rows as they land
    constexpr bool EPI = Shape<FUSE>::EPI;
    constexpr int THREADS = Shape<FUSE>::THREADS;
    constexpr int RED = WARPS * WR * MR;      // floats of one buffer of the warps' sums
    constexpr int OUTS = MODE == 2 ? 8 : 16;  // outputs per tile
    constexpr int NT = MR / 8;                // 8-wide batch tiles
    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem + WARPS * DEPTH * STAGE_BYTES);  // [RED_BUFS][WARPS][WR][MR]
    uint8_t* xs = reinterpret_cast<uint8_t*>(red + Shape<FUSE>::RED_BUFS * RED);  // [MR][slice] rows of x
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const bool is_epi = EPI && warp == WARPS; // the epilogue warp: fetches and multiplies nothing
    const uint32_t ring = smem_u32(smem + (is_epi ? 0 : warp) * DEPTH * STAGE_BYTES);

    const int slice = blockIdx.x % SK;
    const int per = slice_len(K, SK);
    const int k_begin = min(K, slice * per), k_end = min(K, k_begin + per);
    const int klen = k_end - k_begin;
    const int x_stride = per * 2 + 16;        // bytes between x rows in shared memory
    const int n_stages = max(1, (klen + STAGE_K - 1) / STAGE_K);
    const int tile0 = blockIdx.x / SK, tile_step = gridDim.x / SK;
    const int my_tiles = tile0 < tiles ? (tiles - tile0 + tile_step - 1) / tile_step : 0;
    const int total = my_tiles * n_stages;    // stages of this block; stage i: tile i / n_stages, piece i % n_stages

    auto fetch = [&](int i, int slot) {       // weight rows of block stage i into this warp's ring slot
        const int tile = tile0 + (i / n_stages) * tile_step;
        const int kk = (i % n_stages) * STAGE_K;
        const int row_bytes = min(STAGE_K, klen - kk) * 2;
        if (lane * 16 >= row_bytes) return;
        const uint32_t stage = ring + slot * STAGE_BYTES + lane * 16;
#pragma unroll
        for (int r = 0; r < WR; r++) {
            const int n = tile * OUTS + (r % OUTS);
            const size_t row = (size_t)min(n, N - 1) + (r >= OUTS ? (size_t)N : 0);
            cp_async16(stage + r * ROW_STRIDE, W + row * K + k_begin + kk + lane * 8, n < N);
        }
    };

    // prologue: the first DEPTH stages of this warp, before the dependency wait
    int head = warp;                          // next block stage this warp fetches
    if (!is_epi)
        for (int d = 0; d < DEPTH; d++, head += WARPS) {
            if (head < total) fetch(head, d);
            cp_async_commit();
        }
    // The next product's weights: asked into L2 now, so that HBM keeps streaming through the short
    // kernels that follow and that product starts on warm lines. Pieces are dealt round-robin.
    if (fu.pf_bytes) {
        constexpr size_t PIECE = 16384;
        const size_t n = (fu.pf_bytes + PIECE - 1) / PIECE;
        for (size_t i = (size_t)tid * gridDim.x + blockIdx.x; i < n; i += (size_t)gridDim.x * THREADS) {
            const size_t off = i * PIECE;
            const unsigned sz = (unsigned)(fu.pf_bytes - off < PIECE ? (fu.pf_bytes - off) & ~(size_t)15 : PIECE);
            if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(fu.pf + off), "r"(sz) : "memory");
        }
    }
    if (FUSE != 1) {
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&x_bar)));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
    }
    GS_NOTE(0);
    pdl_wait();
    GS_NOTE(1);
    if (tid == 0) pdl_launch_dependents();
    // x rows of this block's slice, once
    if (FUSE == 1) {
        // A thread owns columns (groups of 4) tid, tid + 128, ... of the slice for all M rows: the
        // norm weight of a column is loaded once, and a batch of CG columns x (M rows + weight) is
        // requested before anything is used, so a batch costs one trip to L2, not one per load.
        constexpr int CG = MR == 8 ? 3 : 2;
        const int row_quads = klen / 4;
        float ssr[MR / WARPS];
#pragma unroll
        for (int r = 0; r < MR / WARPS; r++) {   // sums of squares: warp w has rows w, w + 4, ...
            const int j = warp + r * WARPS;
            float ss = 0.f;
            if (j < M && !is_epi)
#pragma unroll 8
                for (int i = lane; i < fu.sq_tiles; i += 32) ss += __ldcg(fu.sq_in + i * 16 + j);
            ssr[r] = ss;
        }
        float4 hv[CG][MR], wv[CG];
        auto request = [&](int q0) {
#pragma unroll
            for (int c = 0; c < CG; c++) {
                const int q = q0 + c * WARPS * 32;
                if (q < row_quads) {
                    wv[c] = ld_cg_f4(fu.norm_w + k_begin + q * 4);
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (m < M) hv[c][m] = ld_cg_f4(fu.h_in + (size_t)m * K + k_begin + q * 4);
                }
            }
        };
        if (!is_epi) request(tid);
#pragma unroll
        for (int r = 0; r < MR / WARPS; r++) {
            const float ss = warp_sum(ssr[r]);
            if (lane == 0 && !is_epi && warp + r * WARPS < M) rstd_s[warp + r * WARPS] = rsqrtf(ss / (float)K + fu.eps);
        }
        __syncthreads();
        for (int q0 = is_epi ? row_quads : tid; q0 < row_quads; q0 += CG * WARPS * 32) {
#pragma unroll
            for (int c = 0; c < CG; c++) {
                const int q = q0 + c * WARPS * 32;
                if (q < row_quads) {
#pragma unroll
                    for (int m = 0; m < MR; m++)
                        if (m < M) {
                            const float rs = rstd_s[m];
                            const float4 h4 = hv[c][m], w4 = wv[c];
                            __nv_bfloat162 lo = __floats2bfloat162_rn(h4.x * rs * w4.x, h4.y * rs * w4.y);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(h4.z * rs * w4.z, h4.w * rs * w4.w);
                            uint2 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&lo);
                            pk.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(xs + m * x_stride + q * 8) = pk;
                        }
                }
            }
            request(q0 + CG * WARPS * 32);
        }
        cp_async_wait<0>();                   // the first weight stages, fetched before the wait
        __syncthreads();
    } else {
        // One bulk copy a row (the TMA engine, which the weight copies of the rings do not queue in
        // front of), counted by an mbarrier that every thread waits on.
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)klen * 2;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&x_bar)), "r"(bytes * M) : "memory");
            for (int m = 0; m < M; m++)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(xs + m * x_stride)),
                             "l"(x + (size_t)m * K + k_begin), "r"(bytes), "r"(smem_u32(&x_bar))
                             : "memory");
        }
        cp_async_wait<0>();                   // this thread's weight stages, fetched before the wait
        const long long t0 = clock64();
        for (;;) {                            // bounded: a copy of valid rows cannot fail, but nothing here may hang
            uint32_t ok;
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
                         : "=r"(ok) : "r"(smem_u32(&x_bar)) : "memory");
            if (ok || clock64() - t0 > 2000000000LL) break;
        }
        __syncwarp();
    }

    GS_NOTE(2);
    float acc[2][NT][4];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int i = 0; i < NT; i++) acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.f;
    const uint32_t a_off = (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_STRIDE + 16 * (lane >> 4));
    const uint32_t b_base = smem_u32(xs) + (uint32_t)(((lane & 7) + (NT == 2 ? 8 * (lane >> 4) : 0)) * x_stride +
                                                      16 * ((lane >> 3) & 1));

    // The epilogue of one tile from the warps' sums in ``sums``: outputs o = first, first + step, ...
    auto finish_tile = [&](const float* sums, int tile, int first, int step) {
        for (int o = first; o < OUTS * MR; o += step) {
            const int i = o % OUTS, j = o / OUTS;
            const int n = tile * OUTS + i;
            if (n < N && j < M) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; w++) v += sums[w * (WR * MR) + i * MR + j];
                if (MODE == 2) {
                    float up = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; w++) up += sums[w * (WR * MR) + (8 + i) * MR + j];
                    v = v / (1.f + expf(-v)) * up;
                }
                if (SK > 1) ws[((size_t)slice * M + j) * N + n] = v;
                else if (MODE == 1) reinterpret_cast<float*>(out)[(size_t)j * N + n] = v;
                else reinterpret_cast<bf16*>(out)[(size_t)j * N + n] = __float2bfloat16_rn(v);
            }
        }
    };
    constexpr int FULL = 1, EMPTY = 3;        // named barriers FULL + buffer, EMPTY + buffer (0 is __syncthreads)
    if (is_epi) {
        for (int ti = 0; ti < my_tiles; ti++) {
            const int buf = ti & 1;
            bar_sync(FULL + buf, THREADS);    // the four warps have left their sums of tile ti
            finish_tile(red + buf * RED, tile0 + ti * tile_step, lane, 32);
            if (ti + 2 < my_tiles) bar_arrive(EMPTY + buf, THREADS);   // the buffer may be written again
        }
        return;
    }

    int tail = warp, slot = 0;                // next block stage this warp multiplies, and its ring slot
    for (int ti = 0; ti < my_tiles; ti++) {
        const int tile = tile0 + ti * tile_step;
        for (; tail < (ti + 1) * n_stages; tail += WARPS) {
            const int kk = (tail % n_stages) * STAGE_K;
            const int steps = min(STAGE_K, klen - kk) / 16;
            const uint32_t stage = ring + slot * STAGE_BYTES;
            const uint32_t xk = b_base + kk * 2;
#pragma unroll 4
            for (int ks = 0; ks < steps; ks++) {
                uint32_t a[4], b[NT == 2 ? 4 : 2];
                ldsm_x4(a, stage + a_off + ks * 32);
                if (NT == 2) {
                    uint32_t b4[4];
                    ldsm_x4(b4, xk + ks * 32);
                    b[0] = b4[0], b[1] = b4[1], b[2 % (NT * 2)] = b4[2], b[3 % (NT * 2)] = b4[3];
                } else {
                    uint32_t b2[2];
                    ldsm_x2(b2, xk + ks * 32);
                    b[0] = b2[0], b[1] = b2[1];
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) mma16816(acc[ks & 1][nt], a, b[2 * nt], b[2 * nt + 1]);
            }
            __syncwarp();                     // every lane is done reading the slot before it is refilled
            if (head < total) fetch(head, slot);
            head += WARPS;
            cp_async_commit();
            slot = (slot + 1) % DEPTH;
            cp_async_wait<DEPTH - 1>();       // this warp's next stage has landed
            __syncwarp();
        }
        // the four warps hold sums over different k: they go to shared memory to be added up
        float* mine = red + (EPI ? (ti & 1) * RED : 0) + warp * (WR * MR);
        if (EPI && ti >= 2) bar_sync(EMPTY + (ti & 1), THREADS);   // the epilogue warp is done with tile ti - 2
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            mine[g * MR + nt * 8 + 2 * t] = acc[0][nt][0] + acc[1][nt][0];
            mine[g * MR + nt * 8 + 2 * t + 1] = acc[0][nt][1] + acc[1][nt][1];
            mine[(g + 8) * MR + nt * 8 + 2 * t] = acc[0][nt][2] + acc[1][nt][2];
            mine[(g + 8) * MR + nt * 8 + 2 * t + 1] = acc[0][nt][3] + acc[1][nt][3];
#pragma unroll
            for (int c = 0; c < 4; c++) acc[0][nt][c] = acc[1][nt][c] = 0.f;
        }
        if (EPI) {                            // hand the sums to the epilogue warp and go on with the next tile
            __threadfence_block();
            bar_arrive(FULL + (ti & 1), THREADS);
            continue;
        }
        __syncthreads();
        if (FUSE == 2) {
            bool fix = true;
            if (SK > 1) {
                for (int o = tid; o < OUTS * MR; o += WARPS * 32) {
                    const int i = o % OUTS, j = o / OUTS;
                    const int n = tile * OUTS + i;
                    if (n < N && j < M) {
                        float v = 0.f;
#pragma unroll
                        for (int w = 0; w < WARPS; w++) v += red[w * (WR * MR) + i * MR + j];
                        ws[((size_t)slice * M + j) * N + n] = v;
                    }
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) {
                    const int ticket = atomicAdd(fu.counters + tile, 1);
                    last_flag = ticket == SK - 1;
                    if (last_flag) fu.counters[tile] = 0;   // every slice has drawn: ready for the next launch
                }
                __syncthreads();
                fix = last_flag != 0;
                if (fix) __threadfence();
            }
            if (fix) {
                for (int o = tid; o < OUTS * MR; o += WARPS * 32) {   // all threads: the shuffles below need whole warps
                    const int i = o % OUTS, j = o / OUTS;
                    const int n = tile * OUTS + i;
                    float sq = 0.f;
                    if (n < N && j < M) {
                        float v = 0.f;
                        if (SK > 1) {
#pragma unroll 8
                            for (int sl = 0; sl < SK; sl++) v += __ldcg(ws + ((size_t)sl * M + j) * N + n);
                        } else {
#pragma unroll
                            for (int w = 0; w < WARPS; w++) v += red[w * (WR * MR) + i * MR + j];
                        }
                        const float hv = fu.h_out[(size_t)j * N + n] + v;
                        fu.h_out[(size_t)j * N + n] = hv;
                        sq = hv * hv;
                    }
#pragma unroll
                    for (int d = 8; d >= 1; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);   // over the tile's 16 columns
                    if (i == 0 && j < M) fu.sq_out[(size_t)tile * 16 + j] = sq;
                }
            }
        } else {
            finish_tile(red, tile, tid, WARPS * 32);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    GS_NOTE(3);
}

template <int MR, int MODE, int FUSE>
int launch(const bf16* x, const bf16* W, void* out, float* ws, int M, int N, int K, int SK, int blocks, const Fuse& fu,
           cudaStream_t st) {
    const size_t smem = (size_t)WARPS * DEPTH * STAGE_BYTES + (size_t)Shape<FUSE>::RED_BUFS * WARPS * WR * MR * sizeof(float) +
                        (size_t)MR * (slice_len(K, SK) * 2 + 16);
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<MR, MODE, FUSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_smem = smem;
    }
    const int tiles = MODE == 2 ? (N + 7) / 8 : (N + 15) / 16;
    blocks = blocks / SK * SK;
    if (blocks > tiles * SK) blocks = tiles * SK;
    return dk_launch(gemv_stream_kernel<MR, MODE, FUSE>, dim3(blocks), dim3(Shape<FUSE>::THREADS), smem, st, x, W, out, ws, M, N, K,
                     SK, tiles, fu);
}

}  // namespace

// x [M,K] bf16 (M <= 16), W [N,K] bf16 (mode 2: [2N,K]); SK slices of K (SK > 1: float32 partial
// sums ws [SK][M][N], modes 0 and 1); `blocks` persistent blocks, at least SK, rounded down to a
// multiple of SK. A slice, ceil(K / SK) rounded up to 16, may have at most 2560 elements.
// fuse 1 (modes 0 and 2, K % 4 == 0): x == null, made from h_in [M,K] float32, the per-tile sums of
// squares sq_in [sq_tiles][16] of its rows, norm_w [K] and eps. fuse 2 (mode 0): the product is
// added into h_out [M,N] float32, sq_out [ceil(N/16)][16] gets the new rows' sums of squares per
// 16 columns; counters: ceil(N/16) ints, zero (the kernel leaves them zero); ws needed if SK > 1.
// pf, pf_bytes: memory (16-byte aligned) to ask into L2 while this product runs, or null / 0.
DK_EXPORT int dk_gemv_stream(const void* x, const void* W, void* out, float* ws, int M, int N, int K, int mode, int SK,
                             int blocks, int fuse, const float* h_in, const float* sq_in, int sq_tiles, const float* norm_w,
                             float eps, float* h_out, float* sq_out, int* counters, const void* pf, long long pf_bytes,
                             cudaStream_t st) {
    if (M < 1 || M > 16 || K % 16 != 0 || SK < 1 || blocks < SK || slice_len(K, SK) > XMAX) return (int)cudaErrorInvalidValue;
    if (SK > 1 && (mode == 2 || ws == nullptr)) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)W) % 16 != 0) return (int)cudaErrorInvalidValue;
    if (fuse == 1 && (mode == 1 || !h_in || !sq_in || !norm_w || ((uintptr_t)h_in | (uintptr_t)norm_w) % 16 != 0))
        return (int)cudaErrorInvalidValue;
    if (fuse == 2 && (mode != 0 || !h_out || !sq_out || (SK > 1 && !counters))) return (int)cudaErrorInvalidValue;
    if (fuse == 0 && !x) return (int)cudaErrorInvalidValue;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    if (pf_bytes < 0 || (pf_bytes > 0 && (pf == nullptr || (uintptr_t)pf % 16 != 0))) return (int)cudaErrorInvalidValue;
    Fuse fu{h_in, sq_in, norm_w, eps, sq_tiles, h_out, sq_out, counters, (const char*)pf, (size_t)pf_bytes};
#define GS_CASE(MR)                                                                                      \
    if (fuse == 1 && mode == 0) return launch<MR, 0, 1>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);   \
    if (fuse == 1) return launch<MR, 2, 1>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);                \
    if (fuse == 2) return launch<MR, 0, 2>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);                \
    if (mode == 0) return launch<MR, 0, 0>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);                \
    if (mode == 1) return launch<MR, 1, 0>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);                \
    return launch<MR, 2, 0>(xp, wp, out, ws, M, N, K, SK, blocks, fu, st);
    if (M <= 8) { GS_CASE(8) }
    GS_CASE(16)
#undef GS_CASE
}
