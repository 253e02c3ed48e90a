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
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#define GV_U 4  // 32-element chunks of K a thread has in flight per batch (2 x 16 B each)

// Warp (r, ks) of a block owns 16 weight rows (tile blockIdx.x*R + r; in mode 2 r selects gate or
// up) and the ks-th slice of K. Within a 32-element chunk of K, lane (g, t) loads the 8 elements
// 8t..8t+7 of rows g and g+8 (one 16-byte load each) and the same 8 elements of x row nt*8+g; the
// two mma steps of the chunk use elements {0..3} and {4..7} of each lane's 8, which permutes K
// identically for both operands.
template <int MT, int MODE>
__global__ void gemv_bf16_kernel(const bf16* x, const bf16* __restrict__ W, void* out,
                                 int M, int N, int K, int R, int KS) {
    extern __shared__ float red[];  // [warps][16][8*MT]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int r = warp / KS, ks = warp % KS;
    const int tile = MODE == 2 ? blockIdx.x : blockIdx.x * R + r;
    const int n_lo = tile * 16 + g, n_hi = n_lo + 8;
    const bool v_lo = n_lo < N, v_hi = n_hi < N;
    const size_t w_row0 = MODE == 2 ? (size_t)r * N : 0;
    const bf16* wlo = W + (w_row0 + (v_lo ? n_lo : 0)) * (size_t)K + 8 * t;
    const bf16* whi = W + (w_row0 + (v_hi ? n_hi : 0)) * (size_t)K + 8 * t;
    const int C = (K + 31) >> 5;
    const int cps = (C + KS - 1) / KS;
    const int c_begin = ks * cps, c_end = min(C, c_begin + cps);

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    uint4 wl[2][GV_U], wh[2][GV_U];
    const uint4 zero = make_uint4(0, 0, 0, 0);
    auto load = [&](int buf, int c0) {
#pragma unroll
        for (int u = 0; u < GV_U; u++) {
            const int c = c0 + u;
            const bool ok = c < c_end && (c * 32 + 8 * t) < K;
            wl[buf][u] = (ok && v_lo) ? ldg_stream(wlo + (size_t)c * 32) : zero;
            wh[buf][u] = (ok && v_hi) ? ldg_stream(whi + (size_t)c * 32) : zero;
        }
    };
    auto consume = [&](int buf, int c0) {
#pragma unroll
        for (int u = 0; u < GV_U; u++) {
            const int c = c0 + u;
            const bool ok = c < c_end && (c * 32 + 8 * t) < K;
#pragma unroll
            for (int nt = 0; nt < MT; nt++) {
                const int m = nt * 8 + g;
                uint4 xr = zero;
                if (ok && m < M) xr = *reinterpret_cast<const uint4*>(x + (size_t)m * K + c * 32 + 8 * t);
                mma16816(acc[nt], wl[buf][u].x, wh[buf][u].x, wl[buf][u].y, wh[buf][u].y, xr.x, xr.y);
                mma16816(acc[nt], wl[buf][u].z, wh[buf][u].z, wl[buf][u].w, wh[buf][u].w, xr.z, xr.w);
            }
        }
    };

    load(0, c_begin);  // weights do not depend on the previous kernel: in flight before the wait
    pdl_wait();
    for (int c0 = c_begin; c0 < c_end; c0 += 2 * GV_U) {
        load(1, c0 + GV_U);
        consume(0, c0);
        load(0, c0 + 2 * GV_U);
        consume(1, c0 + GV_U);
    }
    pdl_launch_dependents();

    const int NB = 8 * MT;
    float* mine = red + (size_t)warp * 16 * NB;
#pragma unroll
    for (int nt = 0; nt < MT; nt++) {
        mine[g * NB + nt * 8 + 2 * t] = acc[nt][0];
        mine[g * NB + nt * 8 + 2 * t + 1] = acc[nt][1];
        mine[(g + 8) * NB + nt * 8 + 2 * t] = acc[nt][2];
        mine[(g + 8) * NB + nt * 8 + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    const int tiles_here = MODE == 2 ? 1 : R;
    for (int idx = threadIdx.x; idx < tiles_here * NB * 16; idx += blockDim.x) {
        const int i = idx & 15, j = (idx >> 4) % NB, rr = idx / (16 * NB);
        const int n = (MODE == 2 ? blockIdx.x : blockIdx.x * R + rr) * 16 + i;
        if (n >= N || j >= M) continue;
        float s = 0.f;
        for (int k = 0; k < KS; k++) s += red[((size_t)(rr * KS + k) * 16 + i) * NB + j];
        if (MODE == 2) {
            float u = 0.f;
            for (int k = 0; k < KS; k++) u += red[((size_t)(KS + k) * 16 + i) * NB + j];
            s = s / (1.f + expf(-s)) * u;
        }
        if (MODE == 1) reinterpret_cast<float*>(out)[(size_t)j * N + n] = s;
        else reinterpret_cast<bf16*>(out)[(size_t)j * N + n] = __float2bfloat16_rn(s);
    }
}

template <int MT, int MODE>
static int launch_gemv(const bf16* x, const bf16* W, void* out, int M, int N, int K, int R, int KS, cudaStream_t st) {
    const int warps = (MODE == 2 ? 2 : R) * KS;
    const int tiles = (N + 15) / 16;
    const unsigned blocks = MODE == 2 ? tiles : (tiles + R - 1) / R;
    const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(gemv_bf16_kernel<MT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        attr_set = true;
    }
    return dk_launch(gemv_bf16_kernel<MT, MODE>, dim3(blocks), dim3(32 * warps), smem, st, x, W, out, M, N, K, R, KS);
}

// x [M,K] bf16, W [N,K] bf16 (mode 2: [2N,K]); R row tiles and KS K-slices per block, R*KS <= 32
// (mode 2: 2*KS <= 32).
DK_EXPORT int dk_gemv_bf16(const void* x, const void* W, void* out, int M, int N, int K, int mode, int R, int KS,
                           cudaStream_t st) {
    if (M < 1 || M > 64 || K % 8 != 0 || R < 1 || KS < 1 || (mode == 2 ? 2 : R) * KS > 32) return (int)cudaErrorInvalidValue;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
#define GV_CASE(MT)                                                                       \
    if (mode == 0) return launch_gemv<MT, 0>(xp, wp, out, M, N, K, R, KS, st);            \
    if (mode == 1) return launch_gemv<MT, 1>(xp, wp, out, M, N, K, R, KS, st);            \
    return launch_gemv<MT, 2>(xp, wp, out, M, N, K, R, KS, st);
    if (M <= 8) { GV_CASE(1) }
    if (M <= 16) { GV_CASE(2) }
    if (M <= 32) { GV_CASE(4) }
    GV_CASE(8)
#undef GV_CASE
}
