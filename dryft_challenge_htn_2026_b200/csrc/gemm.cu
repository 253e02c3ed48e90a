// Matrix products out[M,N] = x[M,K] . W[N,K]^T (weights row-major [out, in], no bias), reference:
// engine/engine.py:131-146 (linear, gate/up + SiLU), engine/fused.py:568-682 (skinny GEMM).
//
//  * sgemm: true float32 on CUDA cores (FMA, no tensor-core mode), any M, N, K. Each output is
//    one sequential sum over K, so a row's result does not depend on the other rows of the batch.
//  * gemv_bf16: the decode-side skinny product for M <= 64 rows in bfloat16. It streams every
//    weight byte once from HBM straight into registers and multiplies on the tensor cores with
//    the weights as the 16-row operand ("swap A/B": the batch is the 8-wide side), float32
//    accumulation. Warps of a block split K between them and reduce through shared memory in a
//    fixed order. Requires K % 8 == 0 (16-byte loads).
// Epilogues: 0 store in T, 1 store float32 (logits), 2 W = [gate; up]: store silu(gate)*up in T.
#include "common.cuh"

// ------------------------------------------------------------------------------------------ sgemm
#define SG_BM 64
#define SG_BN 64
#define SG_BK 16

template <bool SILU>
__global__ void __launch_bounds__(256)
sgemm_kernel(const float* x, const float* __restrict__ W, float* out, int M, int N, int K) {
    __shared__ float xs[SG_BK][SG_BM + 4];
    __shared__ float ws[SG_BK][SG_BN + 4];
    __shared__ float us[SILU ? SG_BK : 1][SG_BN + 4];
    pdl_wait();
    pdl_launch_dependents();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
    const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;  // loader: row in tile, first k
    float acc[4][4] = {}, acu[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += SG_BK) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = k0 + lk + e;
            const int m = m0 + lr, n = n0 + lr;
            xs[lk + e][lr] = (m < M && k < K) ? x[(size_t)m * K + k] : 0.f;
            ws[lk + e][lr] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
            if (SILU) us[lk + e][lr] = (n < N && k < K) ? W[(size_t)(n + N) * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; kk++) {
            float a[4], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = ws[kk][tx * 4 + j];
            if (SILU) {
#pragma unroll
                for (int j = 0; j < 4; j++) u[j] = us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (SILU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float v = acc[i][j];
                if (SILU) v = v / (1.f + expf(-v)) * acu[i][j];
                out[(size_t)m * N + n] = v;
            }
        }
}

// mode 0/1: plain; mode 2: W has 2N rows [gate; up], out [M, N]
DK_EXPORT int dk_sgemm(const float* x, const float* W, float* out, int M, int N, int K, int mode, cudaStream_t st) {
    dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
    if (mode == 2) return dk_launch(sgemm_kernel<true>, grid, dim3(256), 0, st, x, W, out, M, N, K);
    return dk_launch(sgemm_kernel<false>, grid, dim3(256), 0, st, x, W, out, M, N, K);
}

// -------------------------------------------------------------------------------------- gemv_bf16
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Streaming weight load of NW 32-bit words (4: 16 bytes, 8: 32 bytes in one instruction), not
// kept in L1; `words` of them are inside the matrix (the rest read as zero).
template <int NW>
__device__ __forceinline__ void ld_weights(uint32_t (&r)[NW], const bf16* p, int words) {
    if (NW == 8 && words >= 8) {
        asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4 % NW]), "=r"(r[5 % NW]),
                       "=r"(r[6 % NW]), "=r"(r[7 % NW])
                     : "l"(p));
        return;
    }
#pragma unroll
    for (int i = 0; i < NW; i++) r[i] = 0u;
    if (words >= 4)
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                     : "l"(p));
}

// Activation load (plain, coherent: the previous kernel wrote it).
template <int NW>
__device__ __forceinline__ void ld_acts(uint32_t (&r)[NW], const bf16* p, int words) {
#pragma unroll
    for (int i = 0; i < NW; i += 4) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (words >= i + 4) v = *reinterpret_cast<const uint4*>(p + 2 * i);
        r[i] = v.x, r[i + 1] = v.y, r[i + 2] = v.z, r[i + 3] = v.w;
    }
}

// Every warp works alone on units (tile of 16 weight rows, slice of K); no shared memory, no
// block-wide synchronisation. With SK slices per tile the warps write float32 partial sums
// ws[slice][m][n] that the consuming kernel adds up in slice order (a fixed order: results do not
// depend on timing); with SK == 1 they write the result itself. Mode 2 (SiLU gate/up) needs
// SK == 1: a unit is the gate tile and the up tile of the same 16 outputs.
// K is walked in chunks of 8*NW elements: lane (g, t) loads the 2*NW elements
// [2*NW*t, 2*NW*(t+1)) of the chunk for rows g and g+8 (one instruction each; with NW = 8 the four
// lanes of a row cover a whole 128-byte line) and the same elements of x row nt*8+g. mma step s of
// the chunk uses words 2s and 2s+1 of every lane, which permutes K identically for both operands.
// NW = 8 needs K % 16 == 0 (32-byte aligned rows). Units are numbered slice-fastest, so the
// warps of a block stream neighbouring addresses.
template <int MT, int MODE, int NW>
__global__ void __launch_bounds__(256)
gemv_bf16_kernel(const bf16* x, const bf16* __restrict__ W, void* out, float* ws, int M, int N, int K, int SK,
                 int units) {
    constexpr int CH = 8 * NW;               // elements of K per chunk
    constexpr int EPT = 2 * NW;              // elements per lane per chunk
    constexpr int ROWS = MODE == 2 ? 4 : 2;  // weight rows a lane streams: (g, g+8) of gate [and of up]
    constexpr int U = MODE == 2 ? 1 : 2;     // chunks per batch; two batches are in flight
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wpc = blockDim.x >> 5;
    const int C = (K + CH - 1) / CH;
    const int cps = (C + SK - 1) / SK;
    bool waited = false;
    for (int u = blockIdx.x * wpc + (threadIdx.x >> 5); u < units; u += gridDim.x * wpc) {
        const int tile = u / SK, slice = u % SK;
        const int c_begin = slice * cps, c_end = min(C, c_begin + cps);
        const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
        const bool v_lo = n_lo < N, v_hi = n_hi < N;
        const bf16* wrow[ROWS];
        wrow[0] = W + (size_t)(v_lo ? n_lo : 0) * K + EPT * t;
        wrow[1] = W + (size_t)(v_hi ? n_hi : 0) * K + EPT * t;
        if (MODE == 2) {
            wrow[2 % ROWS] = wrow[0] + (size_t)N * K;
            wrow[3 % ROWS] = wrow[1] + (size_t)N * K;
        }
        float acc[MODE == 2 ? 2 : 1][MT][4];
#pragma unroll
        for (int h = 0; h < (MODE == 2 ? 2 : 1); h++)
#pragma unroll
            for (int i = 0; i < MT; i++) acc[h][i][0] = acc[h][i][1] = acc[h][i][2] = acc[h][i][3] = 0.f;

        uint32_t wr[2][U][ROWS][NW];
        auto words_at = [&](int c) {  // 32-bit words of this lane's part of chunk c that lie inside K
            if (c >= c_end) return 0;
            const int left = K - (c * CH + EPT * t);
            return left <= 0 ? 0 : (left >= EPT ? NW : left / 2);
        };
        auto load = [&](int buf, int c0) {
#pragma unroll
            for (int uu = 0; uu < U; uu++) {
                const int words = words_at(c0 + uu);
#pragma unroll
                for (int rr = 0; rr < ROWS; rr++)
                    ld_weights<NW>(wr[buf][uu][rr], wrow[rr] + (size_t)(c0 + uu) * CH, ((rr & 1) ? v_hi : v_lo) ? words : 0);
            }
        };
        auto consume = [&](int buf, int c0) {
#pragma unroll
            for (int uu = 0; uu < U; uu++) {
                const int words = words_at(c0 + uu);
#pragma unroll
                for (int nt = 0; nt < MT; nt++) {
                    const int m = nt * 8 + g;
                    uint32_t xr[NW];
                    ld_acts<NW>(xr, x + (size_t)(m < M ? m : 0) * K + (size_t)(c0 + uu) * CH + EPT * t, m < M ? words : 0);
#pragma unroll
                    for (int s = 0; s < NW / 2; s++) {
                        mma16816(acc[0][nt], wr[buf][uu][0][2 * s], wr[buf][uu][1][2 * s], wr[buf][uu][0][2 * s + 1],
                                 wr[buf][uu][1][2 * s + 1], xr[2 * s], xr[2 * s + 1]);
                        if (MODE == 2)
                            mma16816(acc[MODE == 2 ? 1 : 0][nt], wr[buf][uu][2 % ROWS][2 * s], wr[buf][uu][3 % ROWS][2 * s],
                                     wr[buf][uu][2 % ROWS][2 * s + 1], wr[buf][uu][3 % ROWS][2 * s + 1], xr[2 * s],
                                     xr[2 * s + 1]);
                    }
                }
            }
        };

        load(0, c_begin);  // weights do not depend on the previous kernel: in flight before the wait
        load(1, c_begin + U);
        if (!waited) {
            pdl_wait();
            waited = true;
        }
        for (int c0 = c_begin; c0 < c_end; c0 += 2 * U) {
            consume(0, c0);
            load(0, c0 + 2 * U);
            consume(1, c0 + U);
            load(1, c0 + 3 * U);
        }
#pragma unroll
        for (int nt = 0; nt < MT; nt++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int m = nt * 8 + 2 * t + (c & 1);
                const int n = (c & 2) ? n_hi : n_lo;
                if (m >= M || n >= N) continue;
                float v = acc[0][nt][c];
                if (MODE == 2) v = v / (1.f + expf(-v)) * acc[MODE == 2 ? 1 : 0][nt][c];
                if (SK > 1) ws[((size_t)slice * M + m) * N + n] = v;
                else if (MODE == 1) reinterpret_cast<float*>(out)[(size_t)m * N + n] = v;
                else reinterpret_cast<bf16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(v);
            }
        }
    }
    if (!waited) pdl_wait();
    pdl_launch_dependents();
}

template <int MT, int MODE, int NW>
static int launch_gemv(const bf16* x, const bf16* W, void* out, float* ws, int M, int N, int K, int SK, int warps,
                       int max_blocks, cudaStream_t st) {
    const int units = ((N + 15) / 16) * SK;
    int blocks = (units + warps - 1) / warps;
    if (blocks > max_blocks) blocks = max_blocks;
    return dk_launch(gemv_bf16_kernel<MT, MODE, NW>, dim3(blocks), dim3(32 * warps), 0, st, x, W, out, ws, M, N, K, SK,
                     units);
}

// x [M,K] bf16, W [N,K] bf16 (mode 2: [2N,K]). SK slices of K per 16-row tile; SK > 1 writes
// float32 partial sums ws [SK][M][N] instead of out (modes 0 and 1 only). warps per block <= 8;
// at most max_blocks blocks (warps loop over units beyond that).
DK_EXPORT int dk_gemv_bf16(const void* x, const void* W, void* out, float* ws, int M, int N, int K, int mode, int SK,
                           int warps, int max_blocks, cudaStream_t st) {
    if (M < 1 || M > 64 || K % 8 != 0 || SK < 1 || warps < 1 || warps > 8 || max_blocks < 1) return (int)cudaErrorInvalidValue;
    if (SK > 1 && (mode == 2 || ws == nullptr)) return (int)cudaErrorInvalidValue;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    const bool wide = K % 16 == 0 && ((uintptr_t)W % 32 == 0);
#define GV_MODE(MT, NW)                                                                                \
    if (mode == 0) return launch_gemv<MT, 0, NW>(xp, wp, out, ws, M, N, K, SK, warps, max_blocks, st); \
    if (mode == 1) return launch_gemv<MT, 1, NW>(xp, wp, out, ws, M, N, K, SK, warps, max_blocks, st); \
    return launch_gemv<MT, 2, NW>(xp, wp, out, ws, M, N, K, SK, warps, max_blocks, st);
#define GV_CASE(MT)              \
    if (wide) { GV_MODE(MT, 8) } \
    GV_MODE(MT, 4)
    if (M <= 8) { GV_CASE(1) }
    if (M <= 16) { GV_CASE(2) }
    if (M <= 32) { GV_CASE(4) }
    GV_CASE(8)
#undef GV_CASE
#undef GV_MODE
}

// out[m][n] = sum over slices of ws[slice][m][n], stored as bf16: for a consumer that cannot add
// the partial sums up itself.
__global__ void sum_partials_kernel(const float* ws, bf16* out, size_t mn, int SK) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float s = 0.f;
    for (int k = 0; k < SK; k++) s += ws[(size_t)k * mn + i];
    out[i] = __float2bfloat16_rn(s);
}

DK_EXPORT int dk_sum_partials(const float* ws, void* out, long long mn, int SK, cudaStream_t st) {
    return dk_launch(sum_partials_kernel, dim3((unsigned)((mn + 255) / 256)), dim3(256), 0, st, ws, (bf16*)out, (size_t)mn, SK);
}
