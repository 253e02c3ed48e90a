// The decode-side weight-streaming product for up to 16 rows of x in bfloat16:
// out[M,N] = x[M,K] . W[N,K]^T with the epilogues 0 store bf16, 1 store float32, 2 W = [gate; up]:
// store silu(gate)*up; or split-K float32 partial sums (reference: engine/fused.py:568-682).
//
// Persistent blocks of WARPS streaming warps and an epilogue warp. K is cut into SK slices; block b
// works on slice b % SK only, so its piece of x (at most 16 rows of the slice) is copied into shared
// memory once and every weight byte that follows is the only traffic. The block walks tiles of 16
// weight rows; a tile's slice is cut into stages of 256 elements of K, and stage number i of the
// block belongs to warp i % WARPS, which both fetches and multiplies it: it copies the stage's 16
// weight rows into its own two-deep ring in shared memory with cp.async (one instruction per row:
// the 32 lanes fetch 512 contiguous bytes of that row, and the next stages continue the same rows)
// and multiplies from shared memory on the tensor cores (ldmatrix + mma.sync, float32
// accumulation). At the end of a tile the streaming warps leave their sums in shared memory for the
// epilogue warp, which adds them up, applies the epilogue and stores, while the others go on
// streaming the next tile (two buffers, handed over with named barriers: waiting for the slowest
// warp at every tile cost 11 to 17 % of the kernel). There is no waiting on flags: the only waits
// are cp.async.wait_group, named barriers, and one bounded wait on the mbarrier of x.
//
// Two shapes, chosen by the host from the shared memory the slice of x needs: four streaming warps
// and two blocks an SM (the rings of both keep 19 MB in flight GPU-wide) while two such blocks fit,
// which holds up to 2,560 elements of K at 8 rows; else eight streaming warps and one block an SM
// (the same bytes in flight), which holds up to 5,560.
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
// Requires K % 16 == 0 and 16-byte aligned x and W.
#include "common.cuh"

namespace {

constexpr int STAGE_K = 256;                  // elements of K per stage
constexpr int ROW_STRIDE = STAGE_K * 2 + 16;  // bytes between rows of a stage: 16 of padding keep ldmatrix conflict-free
constexpr int DEPTH = 2;                      // stages a warp has in flight
constexpr int WR = 16;                        // weight rows per stage
constexpr int STAGE_BYTES = WR * ROW_STRIDE;
constexpr int SMEM_LIMIT = 227 * 1024;        // dynamic shared memory a block may ask for on sm_100

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16-byte asynchronous copy global -> shared, not kept in L1; `real` false writes zeros instead.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool real, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst), "l"(src), "r"(real ? 16 : 0), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
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
__device__ __forceinline__ void bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// Slice length for SK slices of K: a multiple of 16.
__host__ __device__ __forceinline__ int slice_len(int K, int SK) { return ((K + SK - 1) / SK + 15) / 16 * 16; }

// Dynamic shared memory of a block: the warps' rings, two buffers of their sums, the rows of x.
__host__ __device__ constexpr size_t smem_bytes(int warps, int mr, int slice) {
    return (size_t)warps * DEPTH * STAGE_BYTES + (size_t)2 * warps * WR * mr * sizeof(float) + (size_t)mr * (slice * 2 + 16);
}

// MR: rows of x kept (8 or 16, M <= MR). MODE as above. Mode 2: a tile's rows 0-7 are the gate rows
// of 8 outputs and rows 8-15 their up rows, so a tile covers 8 outputs.
// gridDim.x is a multiple of SK: block b has slice b % SK and tiles b / SK, + gridDim.x / SK, ...
// (Dealing the rows out evenly instead, in tiles of unequal heights, was measured 15 % slower: the
// bytes a ring slot holds in flight shrink with the tile, and the kernel lives on bytes in flight.)
template <int MR, int MODE, int WARPS>
__global__ void __launch_bounds__((WARPS + 1) * 32)
gemv_stream_kernel(const bf16* x, const bf16* __restrict__ W, void* out, float* ws, int M, int N, int K, int SK, int tiles) {
    __shared__ __align__(8) uint64_t x_bar;   // counts the bytes of x's rows as they land
    constexpr int THREADS = (WARPS + 1) * 32;
    constexpr int RED = WARPS * WR * MR;      // floats of one buffer of the warps' sums
    constexpr int OUTS = MODE == 2 ? 8 : 16;  // outputs per tile
    constexpr int NT = MR / 8;                // 8-wide batch tiles
    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem + WARPS * DEPTH * STAGE_BYTES);  // [2][WARPS][WR][MR]
    uint8_t* xs = reinterpret_cast<uint8_t*>(red + 2 * RED);                    // [MR][slice] rows of x
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const bool is_epi = warp == WARPS;        // the epilogue warp: fetches and multiplies nothing
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

    const uint64_t stream_once = l2_evict_first();   // a weight is read once a step
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
            cp_async16(stage + r * ROW_STRIDE, W + row * K + k_begin + kk + lane * 8, n < N, stream_once);
        }
    };

    // prologue: the first DEPTH stages of this warp, before the dependency wait
    int head = warp;                          // next block stage this warp fetches
    if (!is_epi)
        for (int d = 0; d < DEPTH; d++, head += WARPS) {
            if (head < total) fetch(head, d);
            cp_async_commit();
        }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&x_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();
    if (tid == 0) pdl_launch_dependents();
    // x rows of this block's slice, once: one bulk copy a row (the TMA engine, which the weight copies
    // of the rings do not queue in front of), counted by an mbarrier that every thread waits on.
    if (tid == 0) {
        const uint32_t bytes = (uint32_t)klen * 2;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&x_bar)), "r"(bytes * M) : "memory");
        for (int m = 0; m < M; m++)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             smem_u32(xs + m * x_stride)),
                         "l"(x + (size_t)m * K + k_begin), "r"(bytes), "r"(smem_u32(&x_bar))
                         : "memory");
    }
    cp_async_wait<0>();                       // this thread's weight stages, fetched before the wait
    const long long t0 = clock64();
    for (;;) {                                // bounded: a copy of valid rows cannot fail, but nothing here may hang
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(smem_u32(&x_bar)) : "memory");
        if (ok || clock64() - t0 > 2000000000LL) break;
    }
    __syncwarp();

    float acc[2][NT][4];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int i = 0; i < NT; i++) acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.f;
    const uint32_t a_off = (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_STRIDE + 16 * (lane >> 4));
    const uint32_t b_base = smem_u32(xs) + (uint32_t)(((lane & 7) + (NT == 2 ? 8 * (lane >> 4) : 0)) * x_stride +
                                                      16 * ((lane >> 3) & 1));

    constexpr int FULL = 1, EMPTY = 3;        // named barriers FULL + buffer, EMPTY + buffer (0 is __syncthreads)
    if (is_epi) {
        // The epilogue of tile ti from the streaming warps' sums: lane l takes outputs l, l + 32, ...
        for (int ti = 0; ti < my_tiles; ti++) {
            const int buf = ti & 1;
            const int tile = tile0 + ti * tile_step;
            const float* sums = red + buf * RED;
            bar_sync(FULL + buf, THREADS);    // the streaming warps have left their sums of tile ti
            for (int o = lane; o < OUTS * MR; o += 32) {
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
            if (ti + 2 < my_tiles) bar_arrive(EMPTY + buf, THREADS);   // the buffer may be written again
        }
        return;
    }

    int tail = warp, slot = 0;                // next block stage this warp multiplies, and its ring slot
    for (int ti = 0; ti < my_tiles; ti++) {
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
        // the streaming warps hold sums over different k: they go to shared memory to be added up
        float* mine = red + (ti & 1) * RED + warp * (WR * MR);
        if (ti >= 2) bar_sync(EMPTY + (ti & 1), THREADS);   // the epilogue warp is done with tile ti - 2
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            mine[g * MR + nt * 8 + 2 * t] = acc[0][nt][0] + acc[1][nt][0];
            mine[g * MR + nt * 8 + 2 * t + 1] = acc[0][nt][1] + acc[1][nt][1];
            mine[(g + 8) * MR + nt * 8 + 2 * t] = acc[0][nt][2] + acc[1][nt][2];
            mine[(g + 8) * MR + nt * 8 + 2 * t + 1] = acc[0][nt][3] + acc[1][nt][3];
#pragma unroll
            for (int c = 0; c < 4; c++) acc[0][nt][c] = acc[1][nt][c] = 0.f;
        }
        __threadfence_block();                // hand the sums to the epilogue warp and go on with the next tile
        bar_arrive(FULL + (ti & 1), THREADS);
    }
    cp_async_wait<0>();
}

template <int MR, int MODE, int WARPS>
int launch(const bf16* x, const bf16* W, void* out, float* ws, int M, int N, int K, int SK, int blocks, cudaStream_t st) {
    const size_t smem = smem_bytes(WARPS, MR, slice_len(K, SK));
    if (smem > SMEM_LIMIT) return (int)cudaErrorInvalidValue;
    static size_t attr_smem = 0;
    if (smem > attr_smem) {
        cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<MR, MODE, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_smem = smem;
    }
    const int tiles = MODE == 2 ? (N + 7) / 8 : (N + 15) / 16;
    blocks = blocks / SK * SK;
    if (blocks > tiles * SK) blocks = tiles * SK;
    return dk_launch(gemv_stream_kernel<MR, MODE, WARPS>, dim3(blocks), dim3((WARPS + 1) * 32), smem, st, x, W, out, ws, M, N, K,
                     SK, tiles);
}

}  // namespace

// Dynamic shared memory a block of `warps` streaming warps needs for `rows` rows of x (rounded up to
// 8 or 16) and SK slices of K: the host plans with it (a block may ask for at most 227 KB; two blocks
// share an SM when each stays under half of the SM's 228 KB less 1 KB).
DK_EXPORT long long dk_gemv_stream_smem(int rows, int K, int SK, int warps) {
    return (long long)smem_bytes(warps, rows <= 8 ? 8 : 16, slice_len(K, SK < 1 ? 1 : SK));
}

// x [M,K] bf16 (M <= 16), W [N,K] bf16 (mode 2: [2N,K]); SK slices of K (SK > 1: float32 partial
// sums ws [SK][M][N], modes 0 and 1); `blocks` persistent blocks, at least SK, rounded down to a
// multiple of SK; `warps` streaming warps a block, 4 or 8. Refused (cudaErrorInvalidValue) when the
// rows of a slice do not fit the shared memory of a block of that shape.
DK_EXPORT int dk_gemv_stream(const void* x, const void* W, void* out, float* ws, int M, int N, int K, int mode, int SK,
                             int blocks, int warps, cudaStream_t st) {
    if (M < 1 || M > 16 || K % 16 != 0 || SK < 1 || blocks < SK || (warps != 4 && warps != 8)) return (int)cudaErrorInvalidValue;
    if (mode < 0 || mode > 2 || (SK > 1 && (mode == 2 || ws == nullptr)) || !x) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)W) % 16 != 0) return (int)cudaErrorInvalidValue;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
#define GS_MODE(MR, WARPS)                                                                       \
    if (mode == 0) return launch<MR, 0, WARPS>(xp, wp, out, ws, M, N, K, SK, blocks, st);        \
    if (mode == 1) return launch<MR, 1, WARPS>(xp, wp, out, ws, M, N, K, SK, blocks, st);        \
    return launch<MR, 2, WARPS>(xp, wp, out, ws, M, N, K, SK, blocks, st);
#define GS_CASE(MR)                   \
    if (warps == 4) { GS_MODE(MR, 4) } \
    GS_MODE(MR, 8)
    if (M <= 8) { GS_CASE(8) }
    GS_CASE(16)
#undef GS_CASE
#undef GS_MODE
}
