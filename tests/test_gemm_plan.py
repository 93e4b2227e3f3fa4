"""The planner of the tcgen05 matrix product (tile width and shares of k), which needs no GPU."""

from oxr_inference_b200 import ops


def test_gemm_plan_is_a_valid_launch():
    """Whatever sizes come, the plan is a width the kernel takes and a number of shares its workspace holds."""
    for m in (17, 64, 100, 128, 129, 500, 2048, 5000):
        for n, k in ((64, 64), (509, 96), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096), (5120, 25600)):
            tile_n, splits = ops._gemm_plan(m, n, k)
            assert 16 <= tile_n <= 256 and tile_n % 16 == 0
            assert 1 <= splits <= -(-k // 64)
            tiles = -(-m // 128) * -(-n // tile_n)
            assert splits == 1 or splits * tiles * 128 * tile_n * 4 <= ops.GEMM_WORKSPACE_BYTES


def test_gemm_plan_fills_the_gpu():
    """Few rows and a narrow weight: shares of k or narrow tiles give about one block per SM; many rows: wide tiles."""
    tile_n, splits = ops._gemm_plan(64, 4096, 12288)
    assert 100 <= -(-4096 // tile_n) * splits <= ops.num_sms()
    tile_n, splits = ops._gemm_plan(64, 24576, 4096)
    assert splits == 1 and 100 <= -(-24576 // tile_n) <= ops.num_sms()
    assert ops._gemm_plan(8192, 24576, 4096) == (256, 1)


def test_pair_kernel_takes_the_long_steps_only():
    assert ops._gemm_pair_plan(256, 4096, 4096) == 0
    for m in (512, 2048, 8192):
        for n, k in ((6144, 4096), (24576, 4096), (4096, 12288)):
            tile_n = ops._gemm_pair_plan(m, n, k)
            assert tile_n % 32 == 0 and 64 <= tile_n <= 256
    assert ops._gemm_pair_plan(512, 4096, 4096) == 128          # 64 tiles for 74 pairs, not 32 wide ones


def test_few_rows_form_where_w_is_narrow_and_rows_are_few(monkeypatch):
    # clusters of 1 to 8 blocks that run at a time, as a GPU of 148 SMs in 8 groups of 18 or 19 would report them
    monkeypatch.setattr(ops, "_few_rows_clusters", lambda shares: {1: 148, 2: 72, 3: 48, 4: 32, 5: 24, 6: 24, 7: 16, 8: 16}[shares])
    assert ops._gemm_few_rows_plan(64, 4096, 12288) == 4       # 32 tiles: four shares each
    assert ops._gemm_few_rows_plan(64, 6144, 4096) == 3
    assert ops._gemm_few_rows_plan(64, 24576, 4096) == 0       # 192 tiles fill the SMs as they are
    assert ops._gemm_few_rows_plan(192, 4096, 12288) == 4
    assert ops._gemm_few_rows_plan(257, 4096, 12288) == 0      # a tile is at most 256 wide
    assert ops._gemm_few_rows_plan(64, 4096, 64) == 0          # one k step cannot be shared
    assert ops._gemm_few_rows_plan(64, 5120, 8192) == 3        # 40 tiles: clusters of 3 all run at once
    monkeypatch.setattr(ops, "_few_rows_clusters", lambda shares: 30 if shares == 4 else 148 // shares)
    assert ops._gemm_few_rows_plan(64, 4096, 12288) == 3       # 32 clusters of 4 would not run at once
    monkeypatch.setattr(ops, "_few_rows_clusters", lambda shares: {1: 148, 2: 74, 3: 45, 4: 33, 5: 26, 6: 22, 7: 15, 8: 15}[shares])
    assert ops._gemm_few_rows_plan(192, 6144, 4096) == 2       # 48 tiles: 45 clusters of 3 are too few
    assert ops._gemm_few_rows_plan(200, 6144, 4096) == 0       # from 193 rows on two shares do not pay
    assert ops._gemm_few_rows_plan(256, 4096, 12288) == 4
    assert ops._gemm_few_rows_plan(64, 2560, 9728) == 4        # 20 tiles: 6 shares would run, 4 are as fast or faster
    assert ops._gemm_few_rows_plan(256, 2560, 9728) == 6       # many rows and a long k: more shares pay
    assert ops._gemm_few_rows_plan(256, 2560, 4096) == 4
