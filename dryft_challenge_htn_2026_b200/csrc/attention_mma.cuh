// Device helpers shared by the bfloat16 attention kernels built per head size (-DHD=...): the
// shared-memory layout of staged keys and values, the mma.sync / ldmatrix / cp.async wrappers, the
// query fragments and the online-softmax update of one warp over 16 staged keys.
#pragma once
#include "common.cuh"

#ifndef HD
#error "compile with -DHD=<head size>"
#endif
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");

constexpr int KSTR = HD + 8;                      // shared-memory row stride (elements): 16 B of padding
constexpr int TILE_ELEMS = DK_PAGE * KSTR;        // one staged K or V page
constexpr int STAGE_ELEMS = 2 * TILE_ELEMS;       // K then V

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void cp_async16(bf16* smem, const bf16* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
// the same with a cache policy (see l2_evict_first): a decode step reads a sequence's keys and values once
__device__ __forceinline__ void cp_async16(bf16* smem, const bf16* gmem, uint64_t policy) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(a), "l"(gmem), "l"(policy) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Q fragments of 16 rows; row_ptr0/1: the rows of lane group g and g+8 (nullptr: row of zeros).
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[HD / 16][4], const bf16* row0, const bf16* row1) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        const int c = ks * 16 + 2 * t;
        qf[ks][0] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c) : 0u;
        qf[ks][1] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c) : 0u;
        qf[ks][2] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c + 8) : 0u;
        qf[ks][3] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c + 8) : 0u;
    }
}

// One warp: 16 query rows against NKEYS staged keys (rows of Ks / Vs), online softmax update.
// Row r (0: lane group g, 1: g+8) may see keys with lo[r] <= absolute position <= hi[r].
// Scores are kept in the log2 domain: sl2 = scale * log2(e).
template <int NKEYS>
__device__ __forceinline__ void warp_attend(const uint32_t (&qf)[HD / 16][4], const bf16* Ks, const bf16* Vs, int key0,
                                            const int (&lo)[2], const int (&hi)[2], float sl2, float (&m)[2],
                                            float (&l)[2], float (&acc)[HD / 8][4]) {
    const int lane = threadIdx.x & 31, t = lane & 3;
    float s[NKEYS / 8][4];
#pragma unroll
    for (int i = 0; i < NKEYS / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    const int j = lane >> 3;
#pragma unroll
    for (int np = 0; np < NKEYS / 16; np++) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t b[4];
            ldsm_x4(b, Ks + (np * 16 + (lane & 7) + 8 * (j >> 1)) * KSTR + ks * 16 + 8 * (j & 1));
            mma16816(s[2 * np], qf[ks], b[0], b[1]);
            mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NKEYS / 8; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int key = key0 + nt * 8 + 2 * t + (c & 1), r = c >> 1;
            const float v = (key >= lo[r] && key <= hi[r]) ? s[nt][c] * sl2 : -INFINITY;
            s[nt][c] = v;
            mx[r] = fmaxf(mx[r], v);
        }
    }
    float ms[2], alpha[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        ms[r] = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = exp2f(m[r] - ms[r]);
        m[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NKEYS / 8; nt++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const float p = exp2f(s[nt][c] - ms[c >> 1]);
            s[nt][c] = p;
            sum[c >> 1] += p;
        }
    }
    l[0] = l[0] * alpha[0] + sum[0];
    l[1] = l[1] * alpha[1] + sum[1];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) {
        acc[i][0] *= alpha[0];
        acc[i][1] *= alpha[0];
        acc[i][2] *= alpha[1];
        acc[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < NKEYS / 16; kk++) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HD / 16; dp++) {
            uint32_t b[4];
            ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 15)) * KSTR + dp * 16 + 8 * (lane >> 4));
            mma16816(acc[2 * dp], a, b[0], b[1]);
            mma16816(acc[2 * dp + 1], a, b[2], b[3]);
        }
    }
}

