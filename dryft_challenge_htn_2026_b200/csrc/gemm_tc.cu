// The prefill matrix product on the 5th-generation tensor cores:
//   out[M,N] = x[M,K] . W[N,K]^T                         (mode 0, bfloat16 out)
//   out[M,N] = silu(x . Wgate^T) * (x . Wup^T)           (mode 2, W = [gate; up], N rows each)
//   q, K cache, V cache <- x . [Wq; Wk; Wv]^T             (modes 3, 4: per-head RMSNorm and rotation of
//                          q and k in the epilogue, q to its tensor, k and v into the paged cache)
// float32 accumulation in tensor memory. Reference: the reference engine hands these products to
// the library (engine/fused.py:993-995) and runs SiLU*up as a separate kernel (:175-188); here the
// gated product writes silu(gate)*up directly, so the [M, 2N] intermediate never exists.
//
// One persistent block per SM walks 128 x BN tiles of the output (mode 2: 128 rows x 128 outputs,
// from a gate tile and an up tile side by side in one 256-column accumulator); two accumulators
// alternate in tensor memory so the epilogue of a tile overlaps the mma of the next.
//   warp 0   producer: one thread issues TMA tile loads (cp.async.bulk.tensor.2d, 128-byte
//            swizzle) of x [128 x 64] and W [BN x 64] into a shared-memory ring of 4 stages (up
//            to 12 when few rows of x are loaded); an mbarrier per stage counts the bytes.
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma (cta_group::1, kind::f16,
//            M = 128, N = BN, K = 16, four per stage) from shared-memory matrix descriptors, and
//            tcgen05.commit hands each stage back / signals the epilogue.
//   warps 2-5 epilogue: tcgen05.ld of the accumulator (32 lanes x 32 columns a warp at a time),
//            conversion, SiLU*up in mode 2, bfloat16 stores.
// Rows of x beyond M, rows of W beyond N and columns beyond K are zero-filled by TMA; stores are
// masked. K must be a multiple of 8 (16-byte global strides). Every mbarrier wait is bounded: if
// one runs out the block stores a code in *err, still frees its tensor memory, and returns.
//
// The same kernel serves decode steps of 17 to 128 rows, where the weights are the traffic and a
// few tiles cannot fill the GPU: K is cut into SK slices, a unit of work is (tile, slice), and the
// float32 partial sums of a unit go to ws [SK][M][N] for the consumer to add up (mode 0). There
// the producer requests the weight tiles of its first stages as the very first thing a block does,
// before the tensor memory is allocated and before the wait for the previous kernel (weights never
// depend on it), and the rows of x after the wait. A block with a single unit (every decode step
// the planner sizes) takes one accumulator, and its epilogue goes through the shared memory of the
// ring, which is free by then: the warps that own the tensor-memory lanes of existing rows copy
// the raw sums there, then all four warps work out SiLU*up and store whole rows side by side. (A
// lane storing its own row from registers wrote 32 half-used sectors an instruction, and one or two
// warps did all the arithmetic: 2 us and 4 us of a 10 and 23 us product at 64 rows.)
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128, BK = 64;
constexpr int MAX_STAGES = 12;
#ifndef DK_WAIT_CYCLES
#define DK_WAIT_CYCLES 2000000000LL               // about a second: a wait this long has failed
#endif
constexpr long long WAIT_CYCLES = DK_WAIT_CYCLES;
#ifdef DK_TEST_STALL
// Test build only: with the flag set the producer requests nothing, so every wait of the other
// roles runs out (after DK_WAIT_CYCLES, which such a build makes short) and the error path runs:
// code in *err, tensor memory freed, kernel returns.
__device__ int dk_stall_flag;
DK_EXPORT int dk_test_stall(int on) { return (int)cudaMemcpyToSymbol(dk_stall_flag, &on, sizeof(int)); }
#define DK_STALLED (dk_stall_flag != 0)
#else
#define DK_STALLED false
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// the clock is read only when the first try did not get through
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (clock64() - t0 > WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst)),
                 "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// the same with a cache policy (see l2_evict_first): the weight tiles of a decode step, read once
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(
            smem_u32(dst)),
        "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart,
// groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// What the epilogue of modes 3 and 4 needs beside the product: the fused projection's columns are heads of
// hd (64 or 128) columns, nh of q, then nkv of k, then nkv of v. The float32 accumulator row of a
// token goes through the per-head RMSNorm (weights qn / kn, may be null) and the rotate-half
// rotation by the angles at its position (tables [positions][hd/2], may be null) exactly as in
// qk_norm_rope_write, without the rounding to bfloat16 in between; q goes to q_out [M, nh*hd], k
// and v to the token's place in the paged cache (not when write_kv == 0). Rows with position < 0
// are padding: nothing is stored for them.
struct QkvEpilogue {
    bf16 *q_out, *k_store, *v_store;
    const float *qn, *kn, *cos_t, *sin_t;
    const int *row_pos, *row_seq, *page_table;
    int pt_stride, nh, nkv, hd, write_kv;
    float eps;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void load16(const float* p, float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        f[i] = v.x, f[i + 1] = v.y, f[i + 2] = v.z, f[i + 3] = v.w;
    }
}
__device__ __forceinline__ void store16(bf16* p, const float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i += 8) {
        uint4 pk;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; j++) q[j] = __floats2bfloat162_rn(f[i + 2 * j], f[i + 2 * j + 1]);
        *reinterpret_cast<uint4*>(p + i) = pk;
    }
}

// The epilogue of modes 3 (hd 128) and 4 (hd 64) for one accumulator row: columns [n0, n0 + BN) of
// the projection, BN / HDT heads. Every tcgen05.ld is executed by the whole warp; only the stores
// depend on the lane's row. First the scale of every head's norm, then the head in pieces of 16
// columns and their partners half a head further: a piece's angles serve all heads of the tile, and
// those of the next piece are requested before this one is worked on (with four warps an SM nothing
// else hides the latency of a load).
template <int BN, int HDT>
__device__ __forceinline__ void qkv_epilogue_row(const QkvEpilogue& qe, uint32_t acc, int row, int M, int n0, int N) {
    constexpr int HALF = HDT / 2, HEADS = BN / HDT;
    const int pos = row < M ? qe.row_pos[row] : -1;
    const float* cos_r = qe.cos_t ? qe.cos_t + (size_t)max(pos, 0) * HALF : nullptr;
    const float* sin_r = qe.cos_t ? qe.sin_t + (size_t)max(pos, 0) * HALF : nullptr;
    float cs[2][16], sn[2][16];
    if (cos_r) load16(cos_r, cs[0]), load16(sin_r, sn[0]);
    int page = 0;
    if (pos >= 0 && qe.write_kv) page = qe.page_table[(size_t)qe.row_seq[row] * qe.pt_stride + pos / DK_PAGE];
    float rs[HEADS];
    bf16* dst[HEADS];
#pragma unroll
    for (int hi = 0; hi < HEADS; hi++) {
        const int head = (n0 + hi * HDT) / HDT;
        const bool there = n0 + hi * HDT < N, is_q = head < qe.nh, is_v = head >= qe.nh + qe.nkv;
        dst[hi] = nullptr;
        rs[hi] = 1.f;
        if (!there) continue;
        if (pos >= 0 && (is_q || qe.write_kv))
            dst[hi] = is_q ? qe.q_out + ((size_t)row * qe.nh + head) * HDT
                           : (is_v ? qe.v_store : qe.k_store) + kv_offset(page, qe.nkv, (head - qe.nh) % qe.nkv, pos % DK_PAGE, HDT);
        if (!is_v && (is_q ? qe.qn : qe.kn) != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int c = 0; c < HDT; c += 32) {
                uint32_t v[32];
                tmem_ld32(acc + hi * HDT + c, v);
#pragma unroll
                for (int i = 0; i < 32; i++) ss += __uint_as_float(v[i]) * __uint_as_float(v[i]);
            }
            rs[hi] = rsqrtf(ss / (float)HDT + qe.eps);
        }
    }
#pragma unroll
    for (int c = 0; c < HALF; c += 16) {
        const int cur = (c / 16) & 1;
        if (cos_r && c + 16 < HALF) load16(cos_r + c + 16, cs[cur ^ 1]), load16(sin_r + c + 16, sn[cur ^ 1]);
#pragma unroll
        for (int hi = 0; hi < HEADS; hi++) {
            const int head = (n0 + hi * HDT) / HDT;
            if (n0 + hi * HDT >= N) continue;
            const bool is_q = head < qe.nh, is_v = head >= qe.nh + qe.nkv;
            uint32_t a[16], b[16];
            tmem_ld16(acc + hi * HDT + c, a);
            tmem_ld16(acc + hi * HDT + HALF + c, b);
            if (dst[hi] == nullptr) continue;
            float x1[16], x2[16];
#pragma unroll
            for (int i = 0; i < 16; i++) x1[i] = __uint_as_float(a[i]), x2[i] = __uint_as_float(b[i]);
            if (!is_v) {
                const float* nw = is_q ? qe.qn : qe.kn;
                if (nw) {
                    float w[16];
                    load16(nw + c, w);
#pragma unroll
                    for (int i = 0; i < 16; i++) x1[i] = x1[i] * rs[hi] * w[i];
                    load16(nw + HALF + c, w);
#pragma unroll
                    for (int i = 0; i < 16; i++) x2[i] = x2[i] * rs[hi] * w[i];
                }
                if (cos_r) {
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float o1 = x1[i] * cs[cur][i] - x2[i] * sn[cur][i], o2 = x2[i] * cs[cur][i] + x1[i] * sn[cur][i];
                        x1[i] = o1, x2[i] = o2;
                    }
                }
            }
            store16(dst[hi] + c, x1);
            store16(dst[hi] + HALF + c, x2);
        }
    }
}

// Order of the output tiles. Row tiles run fastest, so the blocks that work at the same time share a
// few panels of W; but only within a group of group_m row tiles, whose rows of x (group_m x 128 x K)
// are sized to stay in the L2 while the group walks all panels of W. (Without groups a step of
// 32,768 rows re-read its 168 MB of x for every one of the 76 panels of the gated product: 8.9 GB
// of DRAM reads for 0.27 GB of operands.) tile -> (row tile, panel).
__device__ __forceinline__ void tile_place(int tile, int m_tiles, int n_tiles, int group_m, int& mt, int& nt) {
    const int per_group = group_m * n_tiles;
    const int g = tile / per_group, r = tile - g * per_group;
    const int gm = min(group_m, m_tiles - g * group_m);
    mt = g * group_m + r % gm;
    nt = r / gm;
}

// MODE 0: W tile rows [n0, n0+BN). MODE 2 (BN = 256): rows [n0, n0+128) of gate at accumulator
// columns 0..127 and the same rows of up (row offset N) at columns 128..255; n0 counts outputs.
// Persistent: block b computes tiles b, b + gridDim.x, ... in the order of tile_place. Two accumulators of BN columns alternate in tensor memory: the
// mma of a tile runs while the epilogue warps drain the tile before it.
template <int BN, int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, bf16* out, int M,
               int N, int K, int m_tiles, int tiles, int group_m, int* err, int SK, float* ws, int STAGES, int a_bytes,
               const __grid_constant__ QkvEpilogue qe) {
    constexpr int B_BYTES = BN * BK * 2;
    // Shared memory: STAGES tiles of x a_bytes apart, then STAGES weight tiles, then the barriers.
    // a_bytes = rows of x that are really loaded x 128 bytes. The mma always reads 128 rows (A_BYTES)
    // from a tile's start: with fewer loaded rows (a decode step) it reads on into the next tiles of
    // x or the weight tiles behind them. Those rows of the accumulator are garbage and never stored;
    // what they cost is nothing, what they save is shared memory for more weight tiles in flight.
    constexpr int TMEM_TWO = 2 * BN <= 256 ? 256 : 512;   // two accumulators; allocations are powers of two
    constexpr int TMEM_ONE = BN <= 128 ? 128 : 256;       // one, where a block has a single unit of work
    constexpr int OUT_COLS = MODE == 2 ? BN / 2 : BN;   // outputs per tile
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);   // the swizzle pattern repeats every 1024 bytes
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * a_bytes;
    const uint32_t stage_tx = (uint32_t)(B_BYTES + a_bytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_b + STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;     // [2] mma -> epilogue
    uint64_t* acc_empty = acc_full + 2;      // [2] epilogue -> mma
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + BK - 1) / BK;
    const int k_per = (k_blocks + SK - 1) / SK;   // k blocks per slice; unit u = (tile u / SK, slice u % SK)
    const int units = tiles * SK;
    const bool early_w = SK > 1 || ws != nullptr || m_tiles == 1;   // decode: weights before the wait
    const bool single = units <= (int)gridDim.x;  // a block has one unit of work
    const uint32_t tmem_cols = single ? TMEM_ONE : TMEM_TWO;
    // whether that unit's tile fits the ring's shared memory as float32 rows (see the epilogue)
    const bool staged = single && STAGES * (B_BYTES + a_bytes) >= BM * (BN + 4) * 4;
    int early = 0;                                // stages whose weight tiles thread 0 requests before the block is set up

    if (!early_w) pdl_wait();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&map_x) : "memory");
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // Decode: the weight tiles of the first unit's first stages are requested here, before the
        // tensor memory is there (its allocation waits while a block of the kernel before, still
        // running on this SM, holds its columns) and long before the rows of x may be read.
        if (early_w && !DK_STALLED) {
            const uint64_t stream_once = l2_evict_first();
            const int unit = blockIdx.x, tile = unit / SK, slice = unit % SK;
            int mt, nt;
            tile_place(tile, m_tiles, tiles / m_tiles, group_m, mt, nt);
            const int n0 = nt * OUT_COLS;
            const int kb0 = slice * k_per, kb1 = min(k_blocks, kb0 + k_per);
            for (int kb = kb0; kb < kb1 && early < STAGES; kb++, early++) {
                uint8_t* stage = smem_b + early * B_BYTES;
                mbar_expect_tx(&full[early], stage_tx);
                if (MODE == 2) {
                    tma_load_2d(stage, &map_w, kb * BK, n0, &full[early], stream_once);
                    tma_load_2d(stage + B_BYTES / 2, &map_w, kb * BK, N + n0, &full[early], stream_once);
                } else {
                    tma_load_2d(stage, &map_w, kb * BK, n0, &full[early], stream_once);
                }
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0 && !DK_STALLED) {  // ---------------------------------------------- producer
            const uint64_t stream_once = l2_evict_first();
            int it = 0;   // stages issued so far, over all units of this block
            int s = 0;    // it % STAGES, and round = (it / STAGES) & 1, kept by counting (no division on this path)
            uint32_t round = 0;
            bool waited = !early_w;
            int early_kb[MAX_STAGES], early_m0[MAX_STAGES];   // stages whose rows of x are still to be requested
            auto flush = [&](int n) {                 // the previous kernel's output may be read from here on
                pdl_wait();
                pdl_launch_dependents();
                waited = true;
                for (int j = 0; j < n; j++) tma_load_2d(smem_a + j * a_bytes, &map_x, early_kb[j] * BK, early_m0[j], &full[j]);
            };
            for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
                const int tile = unit / SK, slice = unit % SK;
                int mt, nt;
                tile_place(tile, m_tiles, tiles / m_tiles, group_m, mt, nt);
                const int m0 = mt * BM, n0 = nt * OUT_COLS;
                const int kb0 = slice * k_per, kb1 = min(k_blocks, kb0 + k_per);
                for (int kb = kb0; kb < kb1; kb++, it++, s = s + 1 == STAGES ? 0 : s + 1, round ^= (s == 0)) {
                    if (!waited && it == STAGES) flush(STAGES);   // the ring is full of weights
                    if (it >= STAGES && !mbar_wait(&empty[s], round ^ 1)) {
                        atomicExch(err, 1);
                        unit = units;
                        break;
                    }
                    uint8_t* stage = smem_b + s * B_BYTES;
                    if (it >= early) mbar_expect_tx(&full[s], stage_tx);
                    if (waited) {
                        tma_load_2d(smem_a + s * a_bytes, &map_x, kb * BK, m0, &full[s]);
                    } else {
                        early_kb[it] = kb;
                        early_m0[it] = m0;
                    }
                    if (it < early) continue;
                    if (early_w) {            // a decode step reads a weight tile once
                        if (MODE == 2) {
                            tma_load_2d(stage, &map_w, kb * BK, n0, &full[s], stream_once);
                            tma_load_2d(stage + B_BYTES / 2, &map_w, kb * BK, N + n0, &full[s], stream_once);
                        } else {
                            tma_load_2d(stage, &map_w, kb * BK, n0, &full[s], stream_once);
                        }
                    } else if (MODE == 2) {
                        tma_load_2d(stage, &map_w, kb * BK, n0, &full[s]);
                        tma_load_2d(stage + B_BYTES / 2, &map_w, kb * BK, N + n0, &full[s]);
                    } else {
                        tma_load_2d(stage, &map_w, kb * BK, n0, &full[s]);
                    }
                }
            }
            if (!waited) flush(it);
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---------------------------------------------------------- mma issuer
            int iter = 0, s = 0;
            uint32_t round = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < units && ok; unit += gridDim.x, iter++) {
                const int slice = unit % SK;
                const int kb0 = slice * k_per, kb1 = min(k_blocks, kb0 + k_per);
                const int buf = iter & 1;
                if (iter >= 2 && !mbar_wait(&acc_empty[buf], ((iter >> 1) & 1) ^ 1)) {   // the epilogue has drained it
                    atomicExch(err, 4);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem + buf * BN;
                for (int kb = kb0; kb < kb1; kb++, s = s + 1 == STAGES ? 0 : s + 1, round ^= (s == 0)) {
                    if (!mbar_wait(&full[s], round)) {
                        atomicExch(err, 2);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem_a + s * a_bytes), b_addr = smem_u32(smem_b + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++)
                        umma_f16(d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), IDESC, (kb > kb0) | (k != 0));
                    umma_commit(&empty[s]);   // the stage is free once these mma have read it
                }
                umma_commit(&acc_full[buf]);  // arrives when every mma above has finished
            }
        }
    } else {  // -------------------------------------------------------------------------- epilogue
        const int q = warp & 3;               // the quarter of the tensor-memory lanes this warp may read
        int iter = 0;
        if (early_w) pdl_wait();              // nothing is stored before the previous kernel is done
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x, iter++) {
            const int tile = unit / SK, slice = unit % SK;
            const int buf = iter & 1;
            int mt, nt;
            tile_place(tile, m_tiles, tiles / m_tiles, group_m, mt, nt);
            const int m0 = mt * BM, n0 = nt * OUT_COLS;
            const int row = m0 + q * 32 + lane;
            const bool arrived = mbar_wait(&acc_full[buf], (iter >> 1) & 1);
            if (!arrived) {
                atomicExch(err, 3);
                if (!staged) break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + buf * BN + ((uint32_t)(q * 32) << 16);
            if (MODE < 3 && staged) {
                // A decode step: the block's one tile goes through shared memory (the ring is done with: every
                // stage has been read by the mma that filled this accumulator), so that a row leaves as whole
                // 16-byte pieces side by side. Straight from the registers every lane would store to a row of
                // its own: 32 separate half-used sectors an instruction, 2 us for a tile of 64 x 128 partial sums.
                // In mode 2 the raw gate and up sums are staged side by side and SiLU * up is worked out on the way
                // out, by all four warps: the tensor-memory lanes of the rows that exist belong to one or two.
                constexpr int W = MODE == 2 ? 2 * OUT_COLS : OUT_COLS;   // staged floats a row
                constexpr int LD = W + 4;                                // LD / 4 is odd: no bank conflicts
                float* stg = reinterpret_cast<float*>(smem);
                if (arrived && q * 32 < M - m0) {
                    float* dst = stg + (q * 32 + lane) * LD;
#pragma unroll 1
                    for (int c = 0; c < W; c += 64) {
                        uint32_t v[32], u[32];
                        tmem_ld32_nowait(acc + c, v);
                        if (c + 32 < W) tmem_ld32_nowait(acc + c + 32, u);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (c + i < W) *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (c + 32 + i < W) *reinterpret_cast<uint4*>(dst + c + 32 + i) = make_uint4(u[i], u[i + 1], u[i + 2], u[i + 3]);
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
                const int rows_here = min(M - m0, BM);
                const int t = (warp - 2) * 32 + lane;
                if (arrived) {
                    for (int idx = t; idx < rows_here * (OUT_COLS / 4); idx += 128) {
                        const int r = idx / (OUT_COLS / 4), c = (idx % (OUT_COLS / 4)) * 4;
                        float4 f = *reinterpret_cast<const float4*>(stg + r * LD + c);
                        if (MODE == 2) {
                            const float4 up = *reinterpret_cast<const float4*>(stg + r * LD + OUT_COLS + c);
                            f.x = __fdividef(f.x, 1.f + __expf(-f.x)) * up.x;   // 2 ulp: far below the bf16 rounding that follows
                            f.y = __fdividef(f.y, 1.f + __expf(-f.y)) * up.y;
                            f.z = __fdividef(f.z, 1.f + __expf(-f.z)) * up.z;
                            f.w = __fdividef(f.w, 1.f + __expf(-f.w)) * up.w;
                        }
                        const int col = n0 + c;
                        if (col >= N) continue;
                        if (ws != nullptr) {
                            float* dst = ws + ((size_t)slice * M + m0 + r) * N + col;
                            if (N % 4 == 0) {
                                *reinterpret_cast<float4*>(dst) = f;
                            } else {
                                const float e[4] = {f.x, f.y, f.z, f.w};
                                for (int i = 0; i < 4 && col + i < N; i++) dst[i] = e[i];
                            }
                        } else {
                            bf16* dst = out + (size_t)(m0 + r) * N + col;
                            if (N % 4 == 0) {
                                uint2 pk;
                                *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(f.x, f.y);
                                *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(f.z, f.w);
                                *reinterpret_cast<uint2*>(dst) = pk;
                            } else {
                                const float e[4] = {f.x, f.y, f.z, f.w};
                                for (int i = 0; i < 4 && col + i < N; i++) dst[i] = __float2bfloat16_rn(e[i]);
                            }
                        }
                    }
                }
                break;                                              // the block's only unit
            }
            if (MODE == 3) qkv_epilogue_row<BN, 128>(qe, acc, row, M, n0, N);
            if (MODE == 4) qkv_epilogue_row<BN, 64>(qe, acc, row, M, n0, N);
#pragma unroll 1
            for (int c = 0; c < (MODE >= 3 ? 0 : OUT_COLS); c += 32) {
                uint32_t v[32];
                tmem_ld32(acc + c, v);
                float f[32];
#pragma unroll
                for (int i = 0; i < 32; i++) f[i] = __uint_as_float(v[i]);
                if (MODE == 2) {
                    uint32_t u[32];
                    tmem_ld32(acc + OUT_COLS + c, u);
                    // only rows that exist: the others hold zeros or whatever the mma read beyond the loaded rows,
                    // and a division by the slow path (zero, infinite or NaN operands) for 100 idle rows of a decode
                    // step made this epilogue 10 us longer
                    if (row < M) {
#pragma unroll
                        for (int i = 0; i < 32; i++) f[i] = __fdividef(f[i], 1.f + __expf(-f[i])) * __uint_as_float(u[i]);   // 2 ulp: far below the bf16 rounding that follows
                    }
                }
                if (row < M && ws != nullptr) {   // float32 partial sums of this slice
                    float* dst = ws + ((size_t)slice * M + row) * N + n0 + c;
                    if (n0 + c + 32 <= N && c + 32 <= OUT_COLS && (N % 4 == 0)) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
                    } else {
                        for (int i = 0; i < 32; i++)
                            if (n0 + c + i < N && c + i < OUT_COLS) dst[i] = f[i];
                    }
                } else if (row < M) {
                    bf16* dst = out + (size_t)row * N + n0 + c;
                    if (n0 + c + 32 <= N && c + 32 <= OUT_COLS && (N % 8 == 0)) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 pk;
                            __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int j = 0; j < 4; j++) p[j] = __floats2bfloat162_rn(f[i + 2 * j], f[i + 2 * j + 1]);
                            *reinterpret_cast<uint4*>(dst + i) = pk;
                        }
                    } else {
                        for (int i = 0; i < 32; i++)
                            if (n0 + c + i < N && c + i < OUT_COLS) dst[i] = __float2bfloat16_rn(f[i]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
            }
        }
    }
    // ---- teardown: everyone arrives, then the allocating warp frees the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (!early_w) pdl_launch_dependents();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

// Row-major bf16 matrix [rows, cols]: tiles of box_rows x 64 columns, 128-byte swizzle, zero fill.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled enc = encoder();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN, int MODE>
int launch(const bf16* x, const bf16* W, bf16* out, int M, int N, int K, int* err, int SK, float* ws, cudaStream_t st,
           const QkvEpilogue& qe = QkvEpilogue{}) {
    constexpr int OUT_COLS = MODE == 2 ? BN / 2 : BN;
    constexpr int B_BYTES = BN * BK * 2;
    // rows of x a TMA box loads: all 128 of a tile, or for a single tile of few rows (a decode step)
    // the next of 16, 32, 64 that holds them, which leaves shared memory for more weight tiles in flight
    const int a_rows = M > 64 ? 128 : M > 32 ? 64 : M > 16 ? 32 : 16;
    const int a_bytes = a_rows * BK * 2;
    const int m_tiles = (M + BM - 1) / BM, tiles = m_tiles * ((N + OUT_COLS - 1) / OUT_COLS);
    const int units = tiles * SK;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    constexpr size_t TAIL = (2 * MAX_STAGES + 4) * sizeof(uint64_t) + 16;
    const size_t budget = 200 * 1024;
    int stages = (int)(budget / (B_BYTES + a_bytes));
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const size_t smem = 1024 + (size_t)stages * (B_BYTES + a_bytes) + TAIL;
    static size_t attr = 0;
    if (smem > attr) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr = smem;
    }
    // row tiles a group: about 40 MB of x (a third of the L2), at least 8
    int group_m = (int)((40LL << 20) / ((long long)BM * K * 2));
    group_m = group_m < 8 ? 8 : group_m;
    CUtensorMap mx, mw;
    int e = make_map(&mx, x, M, K, a_rows);
    if (e) return e;
    e = make_map(&mw, W, MODE == 2 ? 2LL * N : N, K, MODE == 2 ? BN / 2 : BN);
    if (e) return e;
    return dk_launch(gemm_tc_kernel<BN, MODE>, dim3(units < sms ? units : sms), dim3(192), smem, st, mx, mw, out, M, N, K,
                     m_tiles, tiles, group_m, err, SK, ws, stages, a_bytes, qe);
}

}  // namespace

// x [M,K] bf16, W [N,K] bf16 (mode 2: [2N,K] = gate rows then up rows), out [M,N] bf16.
// err: device int, receives a code if a bounded wait ran out. K % 8 == 0; 16-byte aligned x, W.
// ws != null (mode 0): float32 results into ws [SK][M][N] instead of out, the partial sums of SK
// slices of K (every slice at least one block of 64 columns; SK = 1: the product itself in
// float32). bn: weight rows a tile, a multiple of 16 from 128 to 256 (mode 2: half of them gate
// rows, half up rows): the planner picks the height whose tiles and slices load the SMs most evenly.
DK_EXPORT int dk_gemm_tc(const void* x, const void* W, void* out, int M, int N, int K, int mode, int* err, int SK, float* ws,
                         int bn, cudaStream_t st) {
    if (M < 1 || N < 1 || K < 8 || K % 8 != 0 || err == nullptr || SK < 1) return (int)cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)W) % 16 != 0) return (int)cudaErrorInvalidValue;
    const int k_blocks = (K + 63) / 64, k_per = (k_blocks + SK - 1) / SK;
    if (SK > 1 && (mode != 0 || ws == nullptr || (SK - 1) * k_per >= k_blocks)) return (int)cudaErrorInvalidValue;
    if (ws != nullptr && mode != 0) return (int)cudaErrorInvalidValue;
#define TILE_HEIGHT(BN)                                                                                          \
    if (bn == BN && mode == 2) return launch<BN, 2>((const bf16*)x, (const bf16*)W, (bf16*)out, M, N, K, err, SK, ws, st); \
    if (bn == BN && mode == 0) return launch<BN, 0>((const bf16*)x, (const bf16*)W, (bf16*)out, M, N, K, err, SK, ws, st)
    TILE_HEIGHT(128); TILE_HEIGHT(144); TILE_HEIGHT(160); TILE_HEIGHT(176); TILE_HEIGHT(192);
    TILE_HEIGHT(208); TILE_HEIGHT(224); TILE_HEIGHT(240); TILE_HEIGHT(256);
#undef TILE_HEIGHT
    return (int)cudaErrorInvalidValue;
}

// The fused q/k/v projection of a prefill step with the work of qk_norm_rope_write in its epilogue
// (see QkvEpilogue): x [M,K] bf16, W [(nh + 2 nkv) * hd, K] bf16 = [Wq; Wk; Wv], hd 64 or 128;
// q_out [M, nh*hd] bf16; k_store, v_store [pages, nkv, 64, hd] bf16; qn, kn [hd] or null; cos_t,
// sin_t [positions, hd/2] or null; row_pos, row_seq [M]; page_table [sequences, pt_stride].
DK_EXPORT int dk_gemm_tc_qkv(const void* x, const void* W, int M, int K, int* err, void* q_out, void* k_store, void* v_store,
                             const float* qn, const float* kn, const float* cos_t, const float* sin_t, const int* row_pos,
                             const int* row_seq, const int* page_table, int pt_stride, int nh, int nkv, int hd, float eps,
                             int write_kv, cudaStream_t st) {
    if (M < 1 || K < 8 || K % 8 != 0 || err == nullptr || (hd != 64 && hd != 128) || nh < 1 || nkv < 1)
        return (int)cudaErrorInvalidValue;
    if (((uintptr_t)x | (uintptr_t)W | (uintptr_t)q_out | (uintptr_t)k_store | (uintptr_t)v_store | (uintptr_t)qn |
         (uintptr_t)kn | (uintptr_t)cos_t | (uintptr_t)sin_t) % 16 != 0)
        return (int)cudaErrorInvalidValue;
    QkvEpilogue qe{(bf16*)q_out, (bf16*)k_store, (bf16*)v_store, qn, kn, cos_t, sin_t, row_pos, row_seq, page_table,
                   pt_stride, nh, nkv, hd, write_kv, eps};
    if (hd == 128) return launch<256, 3>((const bf16*)x, (const bf16*)W, nullptr, M, (nh + 2 * nkv) * hd, K, err, 1, nullptr, st, qe);
    return launch<256, 4>((const bf16*)x, (const bf16*)W, nullptr, M, (nh + 2 * nkv) * hd, K, err, 1, nullptr, st, qe);
}
