// Matrix products out[M,N] = x[M,K] . W[N,K]^T (weights row-major [out, in], no bias), reference:
// engine/engine.py:131-146 (linear, gate/up + SiLU).
//
//  * sgemm: true float32 on CUDA cores (FMA, no tensor-core mode), any M, N, K. Each output is
//    one sequential sum over K, so a row's result does not depend on the other rows of the batch.
//    Epilogues: 0/1 store, 2 W = [gate; up]: store silu(gate)*up.
//  * sum_partials: adds up the float32 partial sums of a split-K bfloat16 product for a consumer
//    that cannot do it while it reads.
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

// ----------------------------------------------------------------------------------- partial sums
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
