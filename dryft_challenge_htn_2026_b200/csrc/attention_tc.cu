// Prefill attention on the 5th-generation tensor cores: ragged causal grouped-query flash
// attention over the paged cache with S = Q.K^T and O += P.V as tcgen05.mma, accumulators in
// tensor memory, tiles fed by TMA. Built per head size with -DHD=64 or -DHD=128. (Steps of two pages
// with S buffers of 128 columns, four softmax threads a row and one block an SM holding all 512
// columns of its tensor memory halve the instructions of S but leave no second block to fill the
// gaps: measured slower from 2,048 tokens on, 53 vs 50 us, 564 vs 518 us at 8,192.)
// Formulas as attention_bf16.cu (reference: engine/fused.py:301-343): scores scaled by
// scale*log2(e), running maximum and sum in float32, P rounded to bfloat16 before P.V.
//
// A block works on items: 128 consecutive queries of one sequence and one query head. It walks the
// item's keys in steps of 64 (one cache page).
//   warp 5, one thread: TMA loads (Q once an item; K and V of each step as [64 keys x 64 columns]
//       boxes, 128-byte swizzle, straight from the page the table names; two stages each), and
//       the draw of the block's next item from the counter.
//   warp 4, one thread: all tcgen05.mma:
//       S[128 x 64] = Q.K^T   (both operands from shared memory) into one of two S buffers,
//       O[128 x HD] += P.V    (P from tensor memory, V from shared memory, N-major).
//   warps 0-3: softmax, one thread per query row: it reads its row of S from tensor memory
//       (tcgen05.ld) into registers, keeps the running maximum, rescales its row of O in tensor
//       memory when the maximum moved, writes P as bfloat16 back into tensor memory over its S
//       buffer (tcgen05.st), and at the end normalises and stores its row of O. (Two threads a
//       row, which agree on the maximum through shared memory and a barrier of their two warps
//       every step, were 9 to 10 % slower: 56 vs 51 us at 2,048 tokens, 511 vs 471 us at 8,192.)
// Tensor memory: S0 | S1 | O = 64 + 64 + 128 columns. S runs two steps ahead of P.V: the mma thread
// issues S of steps 0 and 1 at once, and S of step j + 2 right behind P.V of step j, into the buffer
// whose P that product has just read (the mma of one thread execute in issue order): the softmax
// warps always find the next S waiting, and the products of a block run under its own softmax. K
// of step j + 2 is fetched as soon as S of step j has been computed, V as soon as P.V has. Two
// blocks fit on an SM (96 KB shared, 256 columns of tensor memory each).
// What a step costs (a timeline of block clocks, test build): the exponentials of the SM's two
// blocks, which fall into step with each other, take 1,070 clocks (16 a clock), their mma 1,290 as
// issued here: S = Q.K^T with 64 keys a step reads 6 KB of shared memory per 128 x 64 x 16 product,
// 48 clocks at 128 bytes a clock against 33 of arithmetic, so S is bound by shared memory (384
// clocks a step against 262 for P.V, whose A operand comes from tensor memory). A step of the two
// blocks takes about 1,480. Q in tensor memory instead (S in the TS form, shared memory for K only)
// needs 64 more columns, which leaves one S buffer for two blocks an SM: built and measured, 4-7 %
// slower on the whole prefill (every latency between softmax and mma is then in the open). Two
// query tiles a block with 128-key steps and all 512 columns of tensor memory (S_A | S_B | O_A |
// O_B, one softmax thread a row, the products of one tile issued while the other tile's softmax
// runs) was built too and gave the same results, but 529 us against 477 at 8,192 tokens (623 with
// two threads a row): the exponential unit does 16 a clock and SM (measured), 1,024 clocks for a
// tile's 128 x 128 scores, a tile's two products take 1,050, and with one S buffer a tile the
// two follow one another: 4,150 clocks for two tiles x 128 keys where the two blocks of this
// kernel need 2,960 for the same work.
// The grid is persistent: two blocks an SM, each takes the next (tile, head) from a counter in
// global memory until none is left. (With a block per tile the SMs did not take a new block while
// one of their two was still running: the light tiles started only when a whole SM had drained,
// and 40 % of the block slots stood empty. A likely cause, not verified: ten warps of 96 registers
// fit an SM twice only if the second block's warps fall on the schedulers the first left emptier.) The tiles come sorted by the keys they see, so the
// heavy ones start first and the light ones fill the end.
// Every mbarrier wait is bounded; a wait that runs out stores a code in *err, and the block still
// frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

#ifndef HD
#error "compile with -DHD=64 or -DHD=128"
#endif
static_assert(HD == 64 || HD == 128, "tensor-core prefill attention is built for head sizes 64 and 128");

namespace {

constexpr int BM = 128, BN = DK_PAGE;             // queries per block, keys per step (one cache page)
constexpr int PAGES = BN / DK_PAGE;
constexpr int CPT = BN;                           // key columns of a step a softmax thread takes: its whole row
constexpr int SOFT = 128;                         // softmax threads, one a query row; then the mma warp, then the loader warp
constexpr int THREADS = SOFT + 64;
constexpr int BLOCKS_PER_SM = BN == 64 ? 2 : 1;
constexpr int TMEM_ALLOC = 2 * BN + 128 <= 256 ? 256 : 512;   // S0 | S1 | O; allocations are powers of two
constexpr int OC = 32;                            // columns of O a thread handles at a time
constexpr int HALVES = HD / 64;                   // 64-column swizzle atoms across the head
constexpr int Q_BYTES = BM * HD * 2, KV_BYTES = BN * HD * 2;   // Q tile; one stage of K or of V
constexpr int Q_ATOM_BYTES = BM * 128;            // the 128 query rows of one 64-column atom
constexpr int KV_ATOM_BYTES = BN * 128;           // the key rows of one 64-column atom
#ifndef DK_WAIT_CYCLES
#define DK_WAIT_CYCLES 2000000000LL               // about a second: a wait this long has failed
#endif
constexpr long long WAIT_CYCLES = DK_WAIT_CYCLES;
#ifdef DK_TEST_STALL
// Test build only: with the flag set the loader thread requests nothing, so the waits of the mma
// thread and the softmax warps run out (after DK_WAIT_CYCLES, which such a build makes short) and
// the error path runs: code in *err, tensor memory freed, kernel returns.
__device__ int dk_stall_flag;
DK_EXPORT int dk_test_stall(int on) { return (int)cudaMemcpyToSymbol(dk_stall_flag, &on, sizeof(int)); }
#define DK_STALLED (dk_stall_flag != 0)
#else
#define DK_STALLED false
#endif
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// the clock is read only when the barrier is not through yet (most waits of the mma thread find it through)
// try_wait lets the hardware suspend the thread for a while instead of having it poll: a polling
// thread takes issue slots from the softmax warps of the other block on its scheduler
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (clock64() - t0 > WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// K-major operand, 128-byte swizzle: rows 128 bytes apart, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// N-major operand (V: keys are the rows in shared memory, the head columns are contiguous),
// 128-byte swizzle: the next 64 columns are KV_ATOM_BYTES away, the next 8 keys 1024 bytes.
__device__ __forceinline__ uint64_t desc_n_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(KV_ATOM_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d),
                 "l"(a), "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d),
                 "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// (no wait inside: call tmem_wait_ld() before the registers are used)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
// 2^x, one MUFU instruction (-inf gives 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// maximum of three, one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// grid min(items, 2 * SMs), 192 threads; item = tile * nh + head. tiles[2i] = sequence,
// tiles[2i+1] = first query (of 128) within the sequence's chunk. q / out [T, nh*HD]; map_q over q
// as [T, nh*HD]; map_k / map_v over one layer's K / V store as [pages * nkv * 64, HD].
// sched[0]: next item, sched[1]: blocks that are done; both zero before the launch and after it.
// Threads 0..127: softmax, thread t has query row t (warp w may read the tensor-memory lanes
// 32 w .. 32 w + 31). Warp 4, one thread: every tcgen05.mma. Warp 5, one thread: every TMA load.
// The per-step barriers (K, V, S, P, O) complete once a step and bar_q once an item: their phases
// run on over the items (step, items count what this block has done so far).
__global__ void __launch_bounds__(THREADS, BLOCKS_PER_SM)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, bf16* out, const int* tiles, int n_items, const int* cu_q,
                       const int* seq_pos0, const int* page_table, int pt_stride, int nh, int nkv, int window, float sl2,
                       int* err, int* sched) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
    const uint32_t q_s = smem_u32(smem), k_s = q_s + Q_BYTES, v_s = k_s + 2 * KV_BYTES;   // Q, K stages 0 1, V stages 0 1
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Q_BYTES + 4 * KV_BYTES);
    // one barrier per stage / buffer: step t (counted over all items of the block) uses number t & 1
    uint64_t *bar_q = bars, *bar_k = bars + 1, *bar_v = bars + 3, *bar_s = bars + 5, *bar_p = bars + 7, *bar_o = bars + 9;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    // [1] a wait ran out; [2], [3]: the block's items, the k-th in slot 2 + (k & 1), written by the loader thread
    volatile int* item_slot = reinterpret_cast<volatile int*>(bars + 12);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_wait();
    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int b = 0; b < 2; b++)
            mbar_init(bar_k + b, 1), mbar_init(bar_v + b, 1), mbar_init(bar_s + b, 1), mbar_init(bar_o + b, 1), mbar_init(bar_p + b, SOFT);
        item_slot[1] = 0;
        item_slot[2] = atomicAdd(&sched[0], 1);             // the block's first item
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    constexpr int MMA_WARP = SOFT / 32, LOAD_WARP = MMA_WARP + 1;
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_ALLOC)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t t_s = tmem, t_o = tmem + 2 * BN;        // S buffers (and P over them) of BN columns each, then O of HD columns

    // What an item (tile, head) is, as every role needs it.
    struct Item {
        int h, kvh, rows_here, flat0, min_pos, max_pos, pos0, q0, blk_lo, n_blk;
        const int* pt;
    };
    auto item_of = [&](int item) {
        Item it;
        const int seq = tiles[2 * (item / nh)];
        it.q0 = tiles[2 * (item / nh) + 1];
        it.h = item % nh, it.kvh = it.h / (nh / nkv);
        it.pos0 = seq_pos0[seq];
        it.rows_here = min(BM, cu_q[seq + 1] - cu_q[seq] - it.q0);
        it.flat0 = cu_q[seq] + it.q0;                      // first flat row of this tile
        it.pt = page_table + (size_t)seq * pt_stride;
        it.min_pos = it.pos0 + it.q0, it.max_pos = it.min_pos + it.rows_here - 1;
        it.blk_lo = window > 0 ? max(0, it.min_pos - window + 1) / BN : 0;
        it.n_blk = it.max_pos / BN - it.blk_lo + 1;
        return it;
    };
    // loader only; t0 = the item's first step
    auto load_kv = [&](const CUtensorMap* map, uint32_t stages, uint64_t* bar, const Item& it, uint32_t t0, int j) {
        const uint32_t b = (t0 + j) & 1;
        mbar_expect_tx(bar + b, KV_BYTES);
        for (int pg = 0; pg < PAGES; pg++) {
            int page = it.pt[min((it.blk_lo + j) * PAGES + pg, pt_stride - 1)];
            if (page < 0) page = 0;                         // a page the sequence does not hold (past its end, or given back by a window): any page will do, its keys are masked
            const int row = (page * nkv + it.kvh) * DK_PAGE;
            for (int hh = 0; hh < HALVES; hh++)
                tma_load_2d(stages + b * KV_BYTES + hh * KV_ATOM_BYTES + pg * (DK_PAGE * 128), map, hh * 64, row, bar + b);
        }
    };
    auto load_q = [&](const Item& it) {
        mbar_expect_tx(bar_q, Q_BYTES);
        for (int hh = 0; hh < HALVES; hh++) tma_load_2d(q_s + hh * Q_ATOM_BYTES, &map_q, it.h * HD + hh * 64, it.flat0, bar_q);
    };

    uint32_t step = 0, items = 0;                          // steps and items this block has finished
    for (;;) {
    // the item's number was left by the loader thread before the block barrier that ended the last item
    const int item = item_slot[2 + (items & 1)];
    if (item >= n_items || item_slot[1]) break;
    const Item cur = item_of(item);
    const int h = cur.h, rows_here = cur.rows_here, flat0 = cur.flat0, min_pos = cur.min_pos, pos0 = cur.pos0, q0 = cur.q0;
    const int blk_lo = cur.blk_lo, n_blk = cur.n_blk;

    // Step j of the item is step t = step + j of the block; it uses stage / buffer / barrier t & 1, whose
    // barriers are then in their phase (t >> 1) & 1.
    if (warp == LOAD_WARP) {
        if (lane == 0 && DK_STALLED) item_slot[1] = 1;      // (test build) nothing is requested: the others' waits run out
        if (lane == 0 && !DK_STALLED) {  // ------------------------------------------- loader: every TMA
            load_q(cur);
            load_kv(&map_k, k_s, bar_k, cur, step, 0);
            load_kv(&map_v, v_s, bar_v, cur, step, 0);
            if (n_blk > 1) load_kv(&map_k, k_s, bar_k, cur, step, 1), load_kv(&map_v, v_s, bar_v, cur, step, 1);
            // the block's next item, for every role to read after this item's last barrier. (Requesting that item's
            // Q and first pages here too, as this one lets go of the buffers, was measured 3 us an item slower.)
            item_slot[2 + ((items + 1) & 1)] = atomicAdd(&sched[0], 1);
            bool ok = true;
            // in the order in which the stages come free: S(j) is done with K(j), then P.V(j-1) with V(j-1)
            for (int j = 0; j + 2 < n_blk && ok; j++) {
                const uint32_t t = step + j;
                if (!mbar_wait(bar_s + (t & 1), (t >> 1) & 1)) { ok = false; break; }
                load_kv(&map_k, k_s, bar_k, cur, step, j + 2);
                if (j >= 1) {
                    if (!mbar_wait(bar_o + ((t - 1) & 1), ((t - 1) >> 1) & 1)) { ok = false; break; }
                    load_kv(&map_v, v_s, bar_v, cur, step, j + 1);
                }
            }
            if (ok && n_blk > 2) {                          // the last value page: after P.V(n - 3)
                const uint32_t t = step + n_blk - 3;
                ok = mbar_wait(bar_o + (t & 1), (t >> 1) & 1);
                if (ok) load_kv(&map_v, v_s, bar_v, cur, step, n_blk - 1);
            }
            if (!ok) atomicExch(err, 3), item_slot[1] = 1;
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {  // ------------------------------------------------------------ every tcgen05.mma
            // S(j) = Q . K(j)^T into buffer (step + j) & 1
            // descriptors: the start address sits in the low bits in units of 16 bytes, so a tile further on is an addition
            const uint64_t dq = desc_k_major(q_s), dk = desc_k_major(k_s), dv = desc_n_major(v_s);
            auto issue_s = [&](int j) {
                const uint32_t b = (step + j) & 1;
                const uint64_t dkb = dk + (uint64_t)((b * KV_BYTES) >> 4);
#pragma unroll
                for (int hh = 0; hh < HALVES; hh++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        umma_ss(t_s + b * BN, dq + (uint64_t)((hh * Q_ATOM_BYTES + k * 32) >> 4),
                                dkb + (uint64_t)((hh * KV_ATOM_BYTES + k * 32) >> 4), IDESC_S, (hh | k) != 0);
                umma_commit(bar_s + b);
            };
            // S runs two steps ahead of P.V: S(0) and S(1) at once, then S(i + 2) right behind P.V(i), whose P it
            // overwrites. The mma of one thread execute in the order of their issue, so S(i + 2) needs no wait
            // for P.V(i) to end. (With S one step ahead and that wait, a timeline of the steps showed the
            // chain P(i-1) -> P.V(i-1) -> its barrier -> S(i+1) -> softmax(i+1) at 1,500 clocks a step where
            // the exponentials of the SM's two blocks take 1,070 and their mma 1,050.)
            bool ok = mbar_wait(bar_q, items & 1) && mbar_wait(bar_k + (step & 1), (step >> 1) & 1);
            if (ok) {
                fence_after();
                issue_s(0);
            }
            if (ok && n_blk > 1) {
                ok = mbar_wait(bar_k + ((step + 1) & 1), ((step + 1) >> 1) & 1);
                if (ok) {
                    fence_after();
                    issue_s(1);
                }
            }
            for (int i = 0; i < n_blk && ok; i++) {
                const uint32_t t = step + i, b = t & 1, ph = (t >> 1) & 1;
                if (!mbar_wait(bar_p + b, ph)) { ok = false; break; }
                if (!mbar_wait(bar_v + b, ph)) { ok = false; break; }   // P is written, V is here
                fence_after();
#pragma unroll
                for (int k = 0; k < BN / 16; k++)
                    umma_ts(t_o, t_s + b * BN + k * 8, dv + (uint64_t)((b * KV_BYTES + k * 16 * 128) >> 4), IDESC_PV, (i | k) != 0);   // the item's first product overwrites O
                umma_commit(bar_o + b);
                if (i + 2 < n_blk) {                        // S of the step after next, into the buffer whose P was just used
                    const uint32_t t2 = t + 2;
                    if (!mbar_wait(bar_k + (t2 & 1), (t2 >> 1) & 1)) { ok = false; break; }
                    fence_after();
                    issue_s(i + 2);
                }
            }
            if (!ok) atomicExch(err, 1), item_slot[1] = 1;
        }
    } else {  // ------------------------------------------------------------------ softmax, a thread a row
        const int r = threadIdx.x;                           // row within the tile = tensor-memory lane
        const bool valid = r < rows_here;
        const int qpos = pos0 + q0 + r;
        const int key_lo = window > 0 ? max(0, qpos - window + 1) : 0;
        const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_blk && ok; i++) {
            const uint32_t t = step + i, b = t & 1, ph = (t >> 1) & 1;
            const int key0 = (blk_lo + i) * BN;
            if (!mbar_wait(bar_s + b, ph)) { ok = false; break; }
            fence_after();
            uint32_t v[CPT];
#pragma unroll
            for (int c = 0; c < CPT; c += 32) tmem_ld32(t_s + lane_off + b * BN + c, *reinterpret_cast<uint32_t(*)[32]>(v + c));
            tmem_wait_ld();
            // every key of the step visible to every row of the tile: no per-element test
            const bool open = window <= 0 && (blk_lo + i) * BN + BN - 1 <= min_pos;
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (open) {
#pragma unroll
                for (int j = 0; j < CPT; j += 2) mx4[(j >> 1) & 3] = max3(mx4[(j >> 1) & 3], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            } else {
#pragma unroll
                for (int j = 0; j < CPT; j++) {
                    const int key = key0 + j;
                    const float sc = (valid && key <= qpos && key >= key_lo) ? __uint_as_float(v[j]) : -INFINITY;
                    v[j] = __float_as_uint(sc);
                    mx4[j & 3] = fmaxf(mx4[j & 3], sc);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sl2;   // sl2 > 0: scaling keeps the order
            float m_new = fmaxf(m, mx);
            // a maximum that moved by less than 8 (a factor 256) keeps the old reference: P stays well inside
            // float32 / bfloat16 range, the final O / l is the same, and O need not be rescaled
            if (m != -INFINITY && m_new - m < 8.f) m_new = m;
            const float ms = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = m_new == m ? 1.f : ex2(m - ms);
            // O of the earlier steps is rescaled when the reference moved, once P.V of the last step is complete
            // (that of the steps before it then is too). Each thread of a row takes its share of the columns of O.
            if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {   // tcgen05.ld/st are warp-wide: all lanes or none
                if (!mbar_wait(bar_o + (b ^ 1), ((t - 1) >> 1) & 1)) { ok = false; break; }
                fence_after();
#pragma unroll 1
                for (int c = 0; c < HD; c += OC) {
                    uint32_t o[OC];
                    tmem_ld32(t_o + lane_off + c, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < OC; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                    tmem_st32(t_o + lane_off + c, o);
                }
            }
            // P = exp2(S * sl2 - m), its sum, and P as bfloat16 over the first columns of this S buffer
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t p[CPT / 2];
#pragma unroll
            for (int j = 0; j < CPT; j += 2) {
                const float e0 = ex2(fmaf(__uint_as_float(v[j]), sl2, -ms)), e1 = ex2(fmaf(__uint_as_float(v[j + 1]), sl2, -ms));
                sum4[(j >> 1) & 3] += e0 + e1;
                __nv_bfloat162 pk = __floats2bfloat162_rn(e0, e1);
                p[j / 2] = *reinterpret_cast<uint32_t*>(&pk);
            }
            tmem_st32(t_s + lane_off + b * BN, p);
            l = l * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            m = m_new;
            tmem_wait_st();
            fence_before();
            mbar_arrive(bar_p + b);
        }
        if (ok) ok = mbar_wait(bar_o + ((step + n_blk - 1) & 1), ((step + n_blk - 1) >> 1) & 1);
        if (ok) {
            fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(flat0 + r) * nh + h) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += OC) {
                uint32_t o[OC];
                tmem_ld32(t_o + lane_off + c, o);
                tmem_wait_ld();
                if (valid) {
#pragma unroll
                    for (int j = 0; j < OC; j += 8) {
                        uint4 pk;
                        __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            pp[u] = __floats2bfloat162_rn(__uint_as_float(o[j + 2 * u]) * inv, __uint_as_float(o[j + 2 * u + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + j) = pk;
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(err, 2), item_slot[1] = 1;
        }
    }
    // everyone is done with the item: O has been read out of tensor memory, the item slot is free
    step += n_blk, items++;
    fence_before();
    __syncthreads();
    fence_after();
    }
    pdl_launch_dependents();
    if (threadIdx.x == 0 && atomicAdd(&sched[1], 1) == (int)gridDim.x - 1) sched[0] = 0, sched[1] = 0;   // the last block leaves zeros for the next launch
    if (warp == MMA_WARP) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_ALLOC) : "memory");
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

// Row-major bf16 matrix [rows, cols]: boxes of box_rows x 64 columns, 128-byte swizzle, zero fill.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, int box_rows) {
    EncodeTiled enc = encoder();
    if (!enc) return (int)cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace

DK_EXPORT int dk_attn_tc_head_dim() { return HD; }

// q, out [n_tok, nh*HD] bf16; k_store, v_store [n_pages, nkv, 64, HD] bf16; tiles [n_tiles][2] =
// (sequence, first query of a 128-row tile within its chunk); err: device int for a wait that ran out;
// sched: two device ints, zero (the kernel leaves them zero), not shared with a launch on another stream.
DK_EXPORT int dk_attn_prefill_tc(const void* q, void* out, const void* k_store, const void* v_store, long long n_tok,
                                 long long n_pages, const int* tiles, int n_tiles, const int* cu_q, const int* seq_pos0,
                                 const int* page_table, int pt_stride, int nh, int nkv, int window, float scale, int* err,
                                 int* sched, cudaStream_t st) {
    if (nh % nkv != 0 || err == nullptr || sched == nullptr || pt_stride < 1) return (int)cudaErrorInvalidValue;
    constexpr size_t smem = 1024 + Q_BYTES + 4 * KV_BYTES + 14 * sizeof(uint64_t);
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr = true;
    }
    CUtensorMap mq, mk, mv;
    int e = make_map(&mq, q, n_tok, (long long)nh * HD, BM);
    if (!e) e = make_map(&mk, k_store, n_pages * nkv * DK_PAGE, HD, DK_PAGE);
    if (!e) e = make_map(&mv, v_store, n_pages * nkv * DK_PAGE, HD, DK_PAGE);
    if (e) return e;
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long n_items = (long long)n_tiles * nh;
    if (n_items > 0x7fffffffLL - 4 * sms) return (int)cudaErrorInvalidValue;
    const long long slots = (long long)BLOCKS_PER_SM * sms;
    const int blocks = (int)(n_items < slots ? n_items : slots);
    return dk_launch(attn_prefill_tc_kernel, dim3(blocks), dim3(THREADS), smem, st, mq, mk, mv, (bf16*)out, tiles, (int)n_items,
                     cu_q, seq_pos0, page_table, pt_stride, nh, nkv, window, scale * 1.4426950408889634f, err, sched);
}
