"""Host-side launch planning (no GPU): how products are cut into slices and tiles, how many key
splits decode attention gets. The kernels refuse plans that break these invariants; the planners
must never produce one."""
import itertools

from dryft_challenge_htn_2026_b200.csrc import api


def test_stream_plan_keeps_a_slice_of_x_in_shared_memory_and_splits_only_when_allowed():
    sms = api.sm_count()
    for M, N, K in itertools.product((1, 8, 16), (72, 2560, 6144, 151936), (304, 2560, 4096, 5120, 9728, 20000)):
        for mode, partial in ((api.MODE_STORE, False), (api.MODE_STORE, True), (api.MODE_STORE_F32, False), (api.MODE_SILU, False)):
            plan = api.stream_plan(M, N, K, mode, partial)
            if plan is None:                      # only when K needs slices that the caller or the epilogue cannot take
                assert K > 2560 and (mode == api.MODE_SILU or not partial)
                assert api._stream_smem(M, K, 1, 8) > 227 * 1024 and api._stream_smem(M, K, 1, 4) > 227 * 1024
                continue
            sk, blocks, warps = plan
            assert sk >= 1 and blocks >= sk and warps in (4, 8)
            smem = api._stream_smem(M, K, sk, warps)
            assert smem <= 227 * 1024
            assert blocks == (2 * sms if warps == 4 and 2 * (smem + 1024) <= 228 * 1024 else sms)   # two blocks an SM only where two fit
            assert sk == 1 or (partial and mode != api.MODE_SILU)
    # the hidden sizes of the three benchmark models at a batch of 8: whole rows of x in shared memory, the
    # gated product and the float32 head included (no slices, so no fall-back to another kernel)
    for K in (2560, 4096, 5120):
        for mode in (api.MODE_SILU, api.MODE_STORE_F32, api.MODE_STORE):
            sk, blocks, warps = api.stream_plan(8, 9728, K, mode)
            assert sk == 1 and (warps, blocks) == ((4, 2 * sms) if K == 2560 else (8, sms))


def test_skinny_tc_plan_gives_every_slice_work_and_no_more_units_than_sms():
    for M, N, K in itertools.product((9, 16, 64, 128), (304, 2560, 6144, 9728, 151936), (64, 520, 2560, 4096, 9728)):
        for mode, partial in ((api.MODE_STORE, True), (api.MODE_STORE, False), (api.MODE_SILU, False), (api.MODE_STORE_F32, False)):
            bn, sk = api.skinny_tc_plan(M, N, K, mode, partial)
            kb = (K + 63) // 64
            assert bn in api.TC_TILE_HEIGHTS
            assert sk >= 1 and (sk - 1) * ((kb + sk - 1) // sk) < kb          # no slice without a block of K
            assert sk == 1 or (mode == api.MODE_STORE and partial)
            if sk > 1:
                assert ((N + bn - 1) // bn) * sk <= api.sm_count()
    # the gated product of the benchmark model: the tile width that covers most SMs in one wave
    assert api.skinny_tc_plan(64, 9728, 2560, api.MODE_SILU) == (144, 1)
    if api.sm_count() == 148:
        # 12,288 outputs in tiles of 88: 140 blocks; 17,408 in tiles of 120: 146 (256-row tiles would leave 52 and 12 SMs idle)
        assert api.skinny_tc_plan(64, 12288, 4096, api.MODE_SILU) == (176, 1)
        assert api.skinny_tc_plan(64, 17408, 5120, api.MODE_SILU) == (240, 1)
        # 4,096 outputs over 4,096 columns: 29 tiles of 144 rows in 5 slices (145 blocks of 13 blocks of K) beat 32 x 4 of 16
        assert api.skinny_tc_plan(64, 4096, 4096, api.MODE_STORE, True) == (144, 5)


def test_decode_splits_depend_on_the_batch_only_and_stay_within_what_the_merge_takes():
    seen = {}
    for n_seq, nkv, group in itertools.product((1, 2, 8, 16, 32, 64, 128, 500), (1, 2, 8), (1, 4, 16, 20)):
        n = api.decode_splits(n_seq, nkv, group)
        assert 1 <= n <= 8
        for pages in (16, 64, 512, 4096):      # long page tables: more splits while the blocks still fit at once
            wide = api.decode_splits(n_seq, nkv, group, pages)
            assert n <= wide <= api.DECODE_MAX_SPLITS and (wide == n or wide * 16 <= pages)
            blocks = n_seq * nkv * ((group + 15) // 16)
            assert wide == n or blocks * wide <= 2 * api.sm_count()
        seen[(n_seq, nkv, group)] = n
    assert seen[(8, 8, 4)] == 4 and seen[(32, 8, 4)] == 1 and seen[(64, 8, 4)] == 4   # measured choices for the benchmark model
    assert seen[(1, 8, 4)] == 8
    if api.sm_count() == 148:
        assert api.decode_splits(1, 8, 4, 64) == 8 and api.decode_splits(1, 8, 4, 512) == 32 and api.decode_splits(8, 8, 4, 512) == 4


def test_gemm_tc_fills_gpu_is_about_the_last_wave():
    assert api.gemm_tc_fills_gpu(2048, 19456 // 2)            # 16 x 38 tiles: 4.1 waves
    assert not api.gemm_tc_fills_gpu(2048, 2560)              # 160 tiles on 148 SMs: a second wave of 12
    assert api.gemm_tc_fills_gpu(128 * 148, 256)


def test_the_tensor_core_product_is_picked_for_prefill_only_where_its_tiles_fill_the_gpu():
    """128 x 256 tiles, one persistent block an SM: the benchmark model's q/k/v and gated products fill
    their waves at 2,048 tokens, its o and down projections (160 tiles) and short prompts do not,
    and with a lower bar (what the tests use to force the path) everything does."""
    assert api.gemm_tc_fills_gpu(2048, 6144) and api.gemm_tc_fills_gpu(2048, 19456)
    assert not api.gemm_tc_fills_gpu(2048, 2560) and not api.gemm_tc_fills_gpu(512, 6144)
    assert api.gemm_tc_fills_gpu(130, 640, 0.0)
    for M, N in itertools.product((129, 512, 2048, 8192, 32768), (640, 2560, 6144, 19456)):
        tiles = -(-M // 128) * -(-N // 256)
        assert api.gemm_tc_fills_gpu(M, N) == (tiles / api.sm_count() / -(-tiles // api.sm_count()) >= 0.8)


def test_gated_tile_height_follows_the_waves():
    """Long prefill steps take the largest tiles; where 192-row tiles need no more waves than 256-row
    ones (512 rows of the benchmark model: 304 tiles or 408 on 148 SMs, three waves either way) they win."""
    assert api.gated_tc_plan(2048, 9728) == (256, 1) and api.gated_tc_plan(8192, 9728) == (256, 1)
    if api.sm_count() == 148:
        assert api.gated_tc_plan(512, 9728) == (192, 1) and api.gated_tc_plan(1024, 9728) == (256, 1)
        assert api.gated_tc_plan(512, 17408) == (256, 1) and api.gated_tc_plan(512, 12288) == (256, 1)
    for M, N in itertools.product((129, 300, 512, 1024, 4096), (104, 9728, 12288, 17408)):
        bn, sk = api.gated_tc_plan(M, N)
        assert bn in (192, 256) and sk == 1
