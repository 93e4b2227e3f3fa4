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


class _FakeAttnLib:
    """Stands in for the attention library's one question that the plan asks: how many pieces get a block each."""

    def __init__(self, pieces):
        self.pieces = pieces

    def oxr_attn_one_round_of_pieces(self):
        return self.pieces


def test_decode_attention_takes_projections_only_with_a_block_per_piece(monkeypatch):
    """The plan that decides whether a step of single tokens hands its raw q|k|v to the attention kernel: the sizes TMA gathers need, no
    more pieces than one round of blocks, not the even cut, and the switch."""
    import torch

    monkeypatch.setattr(ops, "FUSE_QKV", True)
    monkeypatch.setattr(ops, "DECODE_CUT", "auto")
    monkeypatch.setattr(ops, "_attn_lib", lambda d: _FakeAttnLib(296))
    maps = object()
    step = dict(num_heads=32, num_kv_heads=8, kv_len_bound=2048)
    assert ops.attention_takes_projections(128, torch.bfloat16, 16, maps)
    assert ops.attention_takes_projections(128, torch.bfloat16, 16, maps, requests=8, **step)        # 64 units x 4 pieces
    assert not ops.attention_takes_projections(128, torch.bfloat16, 16, maps, requests=64, **step)   # 512 units
    assert not ops.attention_takes_projections(128, torch.bfloat16, 16, maps, requests=8, uneven=True, **step)
    assert not ops.attention_takes_projections(128, torch.float32, 16, maps, requests=8, **step)
    assert not ops.attention_takes_projections(80, torch.bfloat16, 16, maps, requests=8, **step)
    assert not ops.attention_takes_projections(128, torch.bfloat16, 4, maps, requests=8, **step)
    assert not ops.attention_takes_projections(128, torch.bfloat16, 24, maps, requests=8, **step)     # not a power of two
    assert not ops.attention_takes_projections(128, torch.bfloat16, 16, None, requests=8, **step)
    monkeypatch.setattr(ops, "_attn_lib", lambda d: _FakeAttnLib(148))                                # one block per SM
    assert not ops.attention_takes_projections(128, torch.bfloat16, 16, maps, requests=8, **step)
    monkeypatch.setattr(ops, "FUSE_QKV", False)
    assert not ops.attention_takes_projections(128, torch.bfloat16, 16, maps)


def test_a_step_of_single_tokens_knows_itself():
    import torch

    from oxr_inference_b200.parts.base import StepContext

    z = torch.zeros(0, dtype=torch.int32)

    def ctx(q_lens):
        return StepContext(n_tokens=sum(q_lens), n_requests=len(q_lens), token_ids=z, positions=z, req_of_token=z, cu_q=z, ctx_lens=z, state_slots=z,
                           logit_rows=z, no_store_slots=z, groups=[], q_lens=q_lens)

    assert ctx([1, 1, 1]).single_tokens
    assert not ctx([1, 2, 1]).single_tokens
    assert not ctx([3]).single_tokens
    assert not ctx([2, 0]).single_tokens       # as many tokens as requests, but not one each
