"""Each CUDA kernel alone against its plain PyTorch statement (tests/plain/kernels_plain.py), at sizes other than
the engine's: odd widths, head sizes in steps of 16, group sizes that do not divide the tile, several page sizes."""

import math

import pytest
import torch

from plain import kernels_plain as KP

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from oxr_inference_b200 import ops as _ops

    torch.backends.cuda.matmul.allow_tf32 = False
    return _ops


def _tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [64, 100, 4096])
def test_embedding(ops, dtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(301, hidden, device=DEV, generator=g).to(dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    out = ops.embedding(ids, table, dtype, status)
    assert torch.equal(out, table[ids.long()])
    ops.check_status(status)
    bad = torch.tensor([3, 301], dtype=torch.int32, device=DEV)
    out = ops.embedding(bad, table, dtype, status)
    assert torch.equal(out[0], table[3]) and not out[1].any()
    with pytest.raises(ops.KernelError, match="vocabulary"):
        ops.check_status(status)


def test_embedding_widens_and_narrows(ops):
    table = torch.randn(50, 72, device=DEV)
    ids = torch.arange(50, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    assert torch.equal(ops.embedding(ids, table, torch.bfloat16, status), table.bfloat16())
    assert torch.equal(ops.embedding(ids, table.bfloat16(), torch.float32, status), table.bfloat16().float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 2560, 10300])
def test_add_rms_norm(ops, dtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(1)
    n = 37
    x = torch.randn(n, hidden, device=DEV, generator=g).to(dtype)
    res = torch.randn(n, hidden, device=DEV, generator=g) * 3
    w = 1 + 0.1 * torch.randn(hidden, device=DEV, generator=g)
    eps = 1e-5
    # first layer: no residual yet
    out, r0 = ops.add_rms_norm(x, None, w, eps)
    want, want_r = KP.add_rms_norm(x, None, w, eps)
    torch.testing.assert_close(out.float(), want, **_tol(dtype))
    assert torch.equal(r0, want_r)
    # later layers: residual updated in place
    res_in = res.clone()
    out, r1 = ops.add_rms_norm(x, res_in, w, eps)
    want, want_r = KP.add_rms_norm(x, res, w, eps)
    assert r1.data_ptr() == res_in.data_ptr()
    torch.testing.assert_close(r1, want_r, atol=0, rtol=0)
    torch.testing.assert_close(out.float(), want, **_tol(dtype))
    # chosen rows only, residual untouched
    rows = torch.tensor([36, 0, 5], dtype=torch.int32, device=DEV)
    before = res.clone()
    out, none = ops.add_rms_norm(x, res, w, eps, rows=rows)
    assert none is None and torch.equal(res, before)
    torch.testing.assert_close(out.float(), want[rows.long()], **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [160, 77, 12288])
def test_silu_mul(ops, dtype, inter):
    g = torch.Generator(device=DEV).manual_seed(2)
    gu = (torch.randn(9, 2 * inter, device=DEV, generator=g) * 3).to(dtype)
    torch.testing.assert_close(ops.silu_mul(gu).float(), KP.silu_mul(gu), **_tol(dtype))


def _interleave8(gate, up):
    """[.., I] and [.., I] -> [.., 2 I] with groups of 8 columns (or rows of a weight, given as [I, K]) alternating."""
    return torch.stack([gate.reshape(*gate.shape[:-1], -1, 8), up.reshape(*up.shape[:-1], -1, 8)], dim=-2).reshape(*gate.shape[:-1], -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [160, 24, 12288])
def test_silu_mul_on_interleaved_columns(ops, dtype, inter):
    g = torch.Generator(device=DEV).manual_seed(2)
    gu = (torch.randn(9, 2 * inter, device=DEV, generator=g) * 3).to(dtype)
    mixed = _interleave8(gu[:, :inter], gu[:, inter:]).contiguous()
    assert torch.equal(ops.silu_mul(mixed, interleave=8), ops.silu_mul(gu))
    with pytest.raises(ops.KernelError):
        ops.silu_mul(gu[:, :20].contiguous(), interleave=8)


@pytest.mark.parametrize("M", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("inter,K", [(160, 96), (24, 64), (12288, 4096), (1000, 1032)])
@pytest.mark.parametrize("stream", [True, False], ids=["stream", "skinny"])
def test_gated_decode_gemm_applies_silu_in_its_epilogue(ops, monkeypatch, stream, M, inter, K):
    """silu(x Wg^T) * (x Wu^T) from ONE kernel when the weight's gate and up rows alternate in groups of 8, against the
    plain formula, from the weight-streaming kernel and from the register-fed skinny kernel; and the same call with gate
    and up side by side, which runs product and SiLU kernel apart."""
    monkeypatch.setattr(ops, "STREAM_GEMM", stream)
    g = torch.Generator(device=DEV).manual_seed(21)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    wg = (torch.randn(inter, K, device=DEV, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(inter, K, device=DEV, generator=g) * 0.05).bfloat16()
    w = _interleave8(wg.T.contiguous(), wu.T.contiguous()).T.contiguous()     # rows alternate
    assert torch.equal(w[:8], wg[:8]) and torch.equal(w[8:16], wu[:8]) and torch.equal(w[16:24], wg[8:16])
    before = ops.launch_count
    got = ops.gated_silu_linear(x, w, interleave=8)
    assert ops.launch_count == before + 1, "one kernel"
    want = KP.silu_mul(torch.cat([x.float() @ wg.float().T, x.float() @ wu.float().T], dim=1))
    torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=2e-2)
    side_by_side = torch.cat([wg, wu]).contiguous()
    torch.testing.assert_close(ops.gated_silu_linear(x, side_by_side).float(), want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("M,pair_tile", [(40, 0), (150, 0), (300, 64), (3100, 0)])
@pytest.mark.parametrize("inter,K", [(160, 96), (24, 64), (1000, 1032), (12288, 512)])
def test_gated_tcgen05_gemm_applies_silu_in_its_epilogue(ops, monkeypatch, M, pair_tile, inter, K):
    """The same from the tcgen05 kernels (one SM per tile, and the pair kernel where it is forced or planned): tile
    widths that are odd multiples of 16, ragged edges, both against the plain formula."""
    if pair_tile:
        monkeypatch.setattr(ops, "_gemm_pair_plan", lambda m, n, k: pair_tile)
    g = torch.Generator(device=DEV).manual_seed(22)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    wg = (torch.randn(inter, K, device=DEV, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(inter, K, device=DEV, generator=g) * 0.05).bfloat16()
    w = _interleave8(wg.T.contiguous(), wu.T.contiguous()).T.contiguous()
    status = ops.new_status(DEV)
    before = ops.launch_count
    got = ops.gated_silu_linear(x, w, interleave=8)
    assert ops.launch_count == before + 1, "one kernel"
    ops.check_status(status)
    want = KP.silu_mul(torch.cat([x.float() @ wg.float().T, x.float() @ wu.float().T], dim=1))
    torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,D,n", [(4, 2, 16, 23), (6, 2, 32, 23), (5, 5, 48, 23), (32, 8, 128, 23), (3, 1, 256, 23),
                                      # many tokens: the kernel with 16-byte accesses (bf16, head sizes 64, 128, 256)
                                      (5, 3, 64, 150), (32, 8, 128, 300), (3, 1, 256, 77), (7, 1, 128, 64)])
def test_qk_norm_rope_store(ops, dtype, H, KV, D, n):
    g = torch.Generator(device=DEV).manual_seed(3)
    pages, P, maxpos, eps = 50, 8, 300, 1e-5
    qkv = torch.randn(n, (H + 2 * KV) * D, device=DEV, generator=g).to(dtype)
    qw = 1 + 0.2 * torch.randn(D, device=DEV, generator=g)
    kw = 1 + 0.2 * torch.randn(D, device=DEV, generator=g)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
    fr = torch.outer(torch.arange(maxpos, dtype=torch.float), inv)
    cos, sin = fr.cos().to(DEV), fr.sin().to(DEV)
    positions = torch.randint(0, maxpos, (n,), device=DEV, generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * P, device=DEV, generator=g)[:n].int()
    slots[4] = -1  # not stored
    k_cache = torch.full((pages, P, KV, D), 9.0, device=DEV, dtype=dtype)
    v_cache = torch.full((pages, P, KV, D), 9.0, device=DEV, dtype=dtype)
    status = ops.new_status(DEV)
    q = ops.qk_norm_rope_store(qkv, qw, kw, cos, sin, positions, slots, k_cache, v_cache, H, KV, D, eps, status)
    ops.check_status(status)
    wq, wk, wv = KP.qk_norm_rope(qkv, qw, kw, cos, sin, positions, H, KV, D, eps)
    torch.testing.assert_close(q.float(), wq, **_tol(dtype))
    kc, vc = k_cache.view(-1, KV, D).float(), v_cache.view(-1, KV, D).float()
    stored = slots >= 0
    torch.testing.assert_close(kc[slots[stored].long()], wk[stored], **_tol(dtype))
    assert torch.equal(vc[slots[stored].long()], wv[stored])
    untouched = torch.ones(pages * P, dtype=torch.bool, device=DEV)
    untouched[slots[stored].long()] = False
    assert (kc[untouched] == 9.0).all() and (vc[untouched] == 9.0).all(), "a slot outside the step's was written"
    # a slot beyond the pool is reported, not written
    slots2 = slots.clone()
    slots2[0] = pages * P
    ops.qk_norm_rope_store(qkv, qw, kw, cos, sin, positions, slots2, k_cache, v_cache, H, KV, D, eps, status)
    with pytest.raises(ops.KernelError, match="slot"):
        ops.check_status(status)


def test_qk_norm_rope_parts_can_be_switched_off(ops):
    g = torch.Generator(device=DEV).manual_seed(4)
    H, KV, D, n = 2, 1, 32, 5
    qkv = torch.randn(n, (H + 2 * KV) * D, device=DEV, generator=g)
    k_cache = torch.zeros(2, 4, KV, D, device=DEV)
    v_cache = torch.zeros(2, 4, KV, D, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    status = ops.new_status(DEV)
    q = ops.qk_norm_rope_store(qkv, None, None, None, None, pos, slots, k_cache, v_cache, H, KV, D, 1e-6, status)
    assert torch.equal(q.view(n, -1), qkv[:, :H * D])
    assert torch.equal(k_cache.view(-1, D)[:n], qkv[:, H * D:(H + KV) * D])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 509, 96), (16, 160, 96), (17, 192, 160), (150, 333, 77), (64, 4096, 1030)])
def test_gemm_f32(ops, M, N, K):
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(M, K, device=DEV, generator=g)
    w = torch.randn(N, K, device=DEV, generator=g)
    got = ops.linear(x, w)
    want = (x.double() @ w.double().T).float()
    torch.testing.assert_close(got, want, atol=1e-4 * math.sqrt(K), rtol=1e-5)
    # a row's result does not depend on how many rows there are: bit-identical alone and in the batch
    for r in (0, M - 1):
        assert torch.equal(ops.linear(x[r:r + 1].contiguous(), w)[0], got[r])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(509, 96), (192, 160), (4096, 4096), (1000, 12288), (6144, 1032), (40, 520), (151936, 256)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_stream_bf16(ops, M, N, K, out_dtype):
    """The weight-streaming kernel of decode steps: ragged N (509, 1000, 40: a last group of fewer than 16 rows), K that
    is no multiple of the 512-wide slices (96, 160, 1032, 520) or spans many (12288), more groups than blocks and fewer,
    one and two 8-row tiles of x. A row's result does not depend on the rows beside it."""
    assert ops.STREAM_GEMM and M <= ops.STREAM_MAX_ROWS
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    assert got.dtype == out_dtype
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)
    for r in (0, M - 1):
        assert torch.equal(ops.linear(x[r:r + 1].contiguous(), w, out_dtype)[0], got[r])


@pytest.mark.parametrize("M", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("N,K,N2", [(512, 96, 304), (4096, 4096, 6144), (1000, 12288, 160), (4096, 520, 24576), (136, 160, 48)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_stream_with_the_norm_folded_in(ops, M, N, K, N2, gated):
    """product + residual add + RMSNorm + next product as TWO kernels: the first adds its product into the fp32 residual
    stream and leaves residual * norm weight and the rows' sums of squares block by block, the second scales its sums. Against
    the three kernels they replace (same roundings: product to bf16, normalised rows to bf16), with a residual whose rows
    differ in size by orders of magnitude so that a wrong row's inverse norm shows."""
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    res = torch.randn(M, N, device=DEV, generator=g) * (10.0 ** torch.arange(M, device=DEV).remainder(4).float()).unsqueeze(1)
    nw = 1 + 0.3 * torch.randn(N, device=DEV, generator=g)
    w2 = (torch.randn(N2, N, device=DEV, generator=g) * 0.05).bfloat16()
    eps = 1e-5
    # the kernels they replace
    normed, res_want = ops.add_rms_norm(ops.linear(x, w), res.clone(), nw, eps)
    want = ops.gated_silu_linear(normed, w2, ops.GATE_UP_INTERLEAVE) if gated else ops.linear(normed, w2)
    status = ops.new_status(DEV)
    res_got = res.clone()
    fused = ops.linear_add(x, w, res_got, nw, eps)
    assert fused is not None
    lazy, res_out = fused
    assert res_out.data_ptr() == res_got.data_ptr()
    assert torch.equal(res_got, res_want)                      # the same bf16 product plus the same residual, exactly
    sums = lazy.sums[:lazy.blocks, :M].sum(0)
    torch.testing.assert_close(sums, res_want.square().sum(1), rtol=1e-5, atol=0)
    torch.testing.assert_close(lazy.materialize().float(), normed.float(), atol=0, rtol=2 ** -7)   # one bf16 step
    got = ops.gated_silu_linear(lazy, w2, ops.GATE_UP_INTERLEAVE) if gated else ops.linear(lazy, w2)
    ops.check_status(status)
    assert got.shape == want.shape and got.dtype == want.dtype
    scale = want.float().abs().max().item()
    assert (got.float() - want.float()).abs().max().item() <= 2e-2 * scale
    # against plain 32-bit arithmetic as well
    r32 = (x.float() @ w.float().T).bfloat16().float() + res
    n32 = (r32 * torch.rsqrt(r32.square().mean(1, keepdim=True) + eps) * nw.float()).bfloat16().float()
    p32 = n32 @ w2.float().T
    if gated:   # gate and up rows alternate in groups of 8
        p32 = p32.view(M, N2 // 16, 2, 8)
        p32 = (torch.nn.functional.silu(p32[:, :, 0]) * p32[:, :, 1]).reshape(M, N2 // 2)
    assert (got.float() - p32).abs().max().item() <= 2e-2 * p32.abs().max().item()
    # a row's result does not depend on the rows beside it
    for r in (0, M - 1):
        rr = res[r:r + 1].clone()
        lz, _ = ops.linear_add(x[r:r + 1].contiguous(), w, rr, nw, eps)
        one = ops.gated_silu_linear(lz, w2, ops.GATE_UP_INTERLEAVE) if gated else ops.linear(lz, w2)
        assert torch.equal(rr[0], res_got[r]) and torch.equal(one[0], got[r])


def test_gemm_stream_norm_folding_refuses_what_it_cannot_do(ops):
    g = torch.Generator(device=DEV).manual_seed(12)
    x = torch.randn(17, 64, device=DEV, generator=g).bfloat16()          # more rows than the fused kernels take
    w = torch.randn(128, 64, device=DEV, generator=g).bfloat16()
    nw = torch.ones(128, device=DEV)
    assert ops.linear_add(x, w, torch.zeros(17, 128, device=DEV), nw, 1e-6) is None
    assert ops.linear_add(x[:4].float(), w.float(), torch.zeros(4, 128, device=DEV), nw, 1e-6) is None   # 32-bit
    # a consumer that is not a product normalises with the norm kernel; so does a 32-bit product
    res = torch.randn(8, 128, device=DEV, generator=g)
    normed, _ = ops.add_rms_norm(ops.linear(x[:8].contiguous(), w), res.clone(), nw, 1e-6)
    lazy, _ = ops.linear_add(x[:8].contiguous(), w, res.clone(), nw, 1e-6)
    torch.testing.assert_close(lazy.materialize().float(), normed.float(), atol=0, rtol=2 ** -7)
    w32 = torch.randn(48, 128, device=DEV, generator=g)
    torch.testing.assert_close(ops.linear(lazy, w32).float(), ops.linear(normed, w32).float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(509, 96), (192, 160), (4096, 4096), (1000, 12288)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_skinny_bf16(ops, monkeypatch, M, N, K, out_dtype):
    monkeypatch.setattr(ops, "STREAM_GEMM", False)    # the register-fed kernel that the streaming kernel is compared with
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 64)   # every row count the kernel takes, also those linear() sends elsewhere
    g = torch.Generator(device=DEV).manual_seed(6)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    got = ops.linear(x, w, out_dtype)
    assert got.dtype == out_dtype
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (65, 509, 96), (200, 300, 256), (129, 128, 1000), (300, 160, 4096),
                                   (2048, 4096, 4096), (1000, 12288, 160), (77, 64, 64)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_bf16(ops, M, N, K, out_dtype):
    """The TMA + tcgen05 kernel that takes every bf16 product of more rows than the skinny kernel's: whole tiles,
    ragged edges in M, N and K, both output types, with the tile width and shares that linear() plans."""
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    assert got.dtype == out_dtype and got.shape == (M, N)
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K,tile_n,splits", [(17, 509, 4096, 128, 8), (64, 4096, 12288, 96, 3), (100, 1000, 1032, 112, 6),
                                                 (130, 136, 2048, 48, 4), (300, 1024, 8192, 256, 2), (33, 777, 520, 16, 8)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_split_k(ops, monkeypatch, M, N, K, tile_n, splits, out_dtype):
    """Few tiles and a long K: the k steps of a tile are dealt out to shares, the partial tiles meet in the workspace
    and the last unit of a tile adds them in the order of the shares. Twice in a row (the tickets are left zeroed),
    bit-identical."""
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 16)
    monkeypatch.setattr(ops, "_gemm_few_rows_plan", lambda m, n, k: 0)
    monkeypatch.setattr(ops, "_gemm_plan", lambda m, n, k: (tile_n, splits))
    g = torch.Generator(device=DEV).manual_seed(10)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    again = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    assert torch.equal(got, again)
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K,shares", [(64, 256, 64, 1), (17, 509, 96, 1), (100, 1000, 1032, 3), (256, 136, 2048, 8), (33, 4096, 4096, 4),
                                          (5, 300, 328, 2), (200, 777, 520, 1), (128, 4096, 12288, 4), (250, 900, 1100, 5), (96, 6144, 4096, 3),
                                          (1, 130, 8, 1), (77, 128, 4096, 7)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_few_rows_cluster(ops, monkeypatch, M, N, K, shares, out_dtype):
    """The few-rows kernel: it computes the transpose (W's rows on the 128-row side of the tiles, the rows of x as the
    tile's width), the shares of a tile's k steps are the blocks of a cluster and add their partial tiles through
    distributed shared memory; with one share and with several, twice in a row."""
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 0)
    monkeypatch.setattr(ops, "_gemm_few_rows_plan", lambda m, n, k: shares)
    g = torch.Generator(device=DEV).manual_seed(13)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    again = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    assert got.shape == (M, N) and torch.equal(got, again)
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("tile_n", [16, 48, 80, 144, 176, 208, 240, 256])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_every_tile_width(ops, monkeypatch, tile_n, out_dtype):
    """The tile's width is a run-time choice, any multiple of 16 up to 256: ragged edges in M, N and K at each."""
    monkeypatch.setattr(ops, "_gemm_few_rows_plan", lambda m, n, k: 0)
    monkeypatch.setattr(ops, "_gemm_plan", lambda m, n, k: (tile_n, 1))
    M, N, K = 150, 1000, 328
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("M,N,K,tile_n", [(256, 256, 64, 256), (300, 1000, 328, 192), (1000, 2664, 1032, 256), (130, 136, 2048, 64),
                                          (700, 520, 4096, 32), (3100, 1536, 512, 224)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_pair(ops, monkeypatch, M, N, K, tile_n, out_dtype):
    """The two-SM kernel (tcgen05 cta_group::2, each block of a pair stages half of W's tile): whole and ragged tiles,
    a last pair whose second block has no rows at all, every k tail, widths from 32 to 256."""
    monkeypatch.setattr(ops, "SKINNY_MAX_ROWS", 0)
    monkeypatch.setattr(ops, "_gemm_few_rows_plan", lambda m, n, k: 0)
    monkeypatch.setattr(ops, "_gemm_pair_plan", lambda m, n, k: tile_n)
    g = torch.Generator(device=DEV).manual_seed(12)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    status = ops.new_status(DEV)
    got = ops.linear(x, w, out_dtype)
    ops.check_status(status)
    assert got.dtype == out_dtype and got.shape == (M, N)
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, atol=2e-4 * math.sqrt(K) * 0.05, rtol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want, atol=1e-2, rtol=1e-2)


def test_linear_large_bf16_with_rows_that_are_not_16_byte_words_falls_to_the_library(ops):
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(200, 250, device=DEV, generator=g).bfloat16()
    w = (torch.randn(300, 250, device=DEV, generator=g) * 0.05).bfloat16()
    want = x.float() @ w.float().T
    torch.testing.assert_close(ops.linear(x, w, torch.float32), want, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(ops.linear(x, w).float(), want, atol=2e-2, rtol=2e-2)


def test_linear_keeps_a_32bit_weight_32bit(ops):
    g = torch.Generator(device=DEV).manual_seed(8)
    x = torch.randn(5, 96, device=DEV, generator=g).bfloat16()
    w = torch.randn(40, 96, device=DEV, generator=g)
    got = ops.linear(x, w)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), (x.float() @ w.T), atol=1e-1, rtol=1e-2)


# ------------------------------------------------------------------------------------------------ attention
def _paged_case(g, q_lens, ctx_lens, H, KV, D, P, dtype, extra_pages=3):
    """Random q, a cache whose pages are handed out in shuffled order, block tables, tile lists."""
    n = len(q_lens)
    need = [-(-c // P) for c in ctx_lens]
    total = sum(need) + extra_pages
    order = torch.randperm(total, generator=torch.Generator().manual_seed(11)).tolist()
    width = max(need) + 1
    table = torch.full((n, width), -7, dtype=torch.int32)  # unused entries hold rubbish on purpose
    at = 0
    for r in range(n):
        table[r, :need[r]] = torch.tensor(order[at:at + need[r]], dtype=torch.int32)
        at += need[r]
    k_cache = torch.randn(total, P, KV, D, device=DEV, generator=g).to(dtype)
    v_cache = torch.randn(total, P, KV, D, device=DEV, generator=g).to(dtype)
    T = sum(q_lens)
    q = torch.randn(T, H, D, device=DEV, generator=g).to(dtype)
    cu = [0]
    for x in q_lens:
        cu.append(cu[-1] + x)
    return q, k_cache, v_cache, table.to(DEV), cu


def _release_behind_window(table, q_lens, ctx_lens, P, window):
    """What the cache manager does as a window moves on: the block-table entries of pages that lie wholly behind the
    window of a request's first new token become -1 (the pages were given back, and may hold another request's keys)."""
    if window <= 0:
        return table
    table = table.clone()
    for r, (ql, c) in enumerate(zip(q_lens, ctx_lens)):
        table[r, :max(0, c - ql - window + 1) // P] = -1
    return table


def _tiles(ops, q_lens, H, KV, D, dtype, page_size=None):
    """The tile lists the kernels of this dtype want: each request's new tokens cut into tiles (with a page size: the
    lists for a cache whose K and V are fetched by TMA)."""
    out = {}
    for spec in ops.attention_tile_specs(H, KV, D, dtype, page_size):
        tpt, fewest, most = spec
        req, tok = [], []
        for r, ql in enumerate(q_lens):
            if fewest <= ql <= most:
                for t0 in range(0, ql, tpt):
                    req.append(r)
                    tok.append(t0)
        out[spec] = (torch.tensor(req + [0], dtype=torch.int32, device=DEV), torch.tensor(tok + [0], dtype=torch.int32, device=DEV), len(req))
    return out


def _run_attn(ops, q, k_cache, v_cache, table, cu, q_lens, ctx_lens, scale, window, generic=False):
    H, D, KV, P = q.shape[1], q.shape[2], k_cache.shape[2], k_cache.shape[1]
    tiles = _tiles(ops, q_lens, H, KV, D, torch.float32 if generic else q.dtype)
    status = ops.new_status(DEV)
    out = ops.paged_attention(q, k_cache, v_cache, tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                              ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=table,
                              page_size=P, scale=scale, window=window, kv_len_bound=max(ctx_lens), status=status, generic=generic)
    ops.check_status(status)
    return out


KINDS = [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)]
KIND_IDS = ["float32", "bfloat16-tensorcore", "bfloat16-generic"]


@pytest.mark.parametrize("dtype,generic", KINDS, ids=KIND_IDS)
@pytest.mark.parametrize("H,KV,D,P", [(4, 2, 16, 16), (6, 2, 32, 8), (8, 1, 64, 16), (5, 5, 48, 4), (20, 1, 16, 16),
                                      (32, 8, 128, 16), (2, 2, 256, 64), (3, 1, 80, 16), (80, 1, 32, 16)])
@pytest.mark.parametrize("window", [0, 13])
def test_paged_attention_mixed_batch(ops, dtype, generic, H, KV, D, P, window):
    g = torch.Generator(device=DEV).manual_seed(20 + D)
    q_lens = [1, 37, 2, 1, 70, 8, 9]      # decode tokens beside prompt portions, around the short/long boundary
    ctx_lens = [1, 37, 130, 200, 75, 8, 140]  # position 0 alone; a whole prompt; portions deep into a context
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, dtype)
    table = _release_behind_window(table, q_lens, ctx_lens, P, window)
    scale = D ** -0.5
    got = _run_attn(ops, q, k_cache, v_cache, table, cu, q_lens, ctx_lens, scale, window, generic)
    want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, scale, window)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.float(), want, **tol)


@pytest.mark.parametrize("dtype,generic", KINDS, ids=KIND_IDS)
def test_attention_finds_one_far_key_and_respects_the_window_edge(ops, dtype, generic):
    """One key among hundreds is made to match the query so strongly that it takes all the weight: if the kernel
    skipped it (a page's edge, the first or last key, the key just inside the window) the output would be far off.
    The key just outside the window is made as strong and must be ignored."""
    H, KV, D, P = 4, 2, 32, 8
    ctx = 389
    g = torch.Generator(device=DEV).manual_seed(30)
    for far in (0, 7, 8, 255, 256, 388 - 20, 388):
        for window in (0, 21):
            q, k_cache, v_cache, table, cu = _paged_case(g, [1], [ctx], H, KV, D, P, dtype)
            k_cache.mul_(0.05)
            qpos = ctx - 1
            target = far if window == 0 else max(far, qpos - window + 1)   # a key inside the window
            pages = table[0].tolist()

            def key(pos):
                return k_cache[pages[pos // P], pos % P]
            for kvh in range(KV):
                key(target)[kvh] = q[0, kvh * (H // KV)].float().mul(3.0).to(dtype)
                if window and qpos - window >= 0:
                    key(qpos - window)[kvh] = q[0, kvh * (H // KV)].float().mul(6.0).to(dtype)   # just outside
            got = _run_attn(ops, q, k_cache, v_cache, table, cu, [1], [ctx], 1.0, window, generic)
            want = KP.paged_attention(q, k_cache, v_cache, cu, [ctx], table, 1.0, window)
            tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
            torch.testing.assert_close(got.float(), want, **tol)
            # the first head of each group must have picked exactly the target's value
            v_t = v_cache[pages[target // P], target % P].float()
            for kvh in range(KV):
                torch.testing.assert_close(got[0, kvh * (H // KV)].float(), v_t[kvh], atol=5e-2, rtol=5e-2)


def test_attention_fp32_is_bit_identical_however_the_queries_are_cut(ops):
    H, KV, D, P = 6, 2, 32, 8
    g = torch.Generator(device=DEV).manual_seed(31)
    ctx = 150
    q, k_cache, v_cache, table, cu = _paged_case(g, [ctx], [ctx], H, KV, D, P, torch.float32)
    whole = _run_attn(ops, q, k_cache, v_cache, table, cu, [ctx], [ctx], D ** -0.5, 0)
    pos = 0
    for c in (7, 2, 13, 1, 50, 3, 74):
        part = _run_attn(ops, q[pos:pos + c].contiguous(), k_cache, v_cache, table, [0, c], [c], [pos + c], D ** -0.5, 0)
        assert torch.equal(part, whole[pos:pos + c]), f"portion at {pos} of {c} differs from the whole run"
        pos += c


def test_attention_reports_a_page_outside_the_pool(ops):
    H, KV, D, P = 2, 1, 16, 8
    g = torch.Generator(device=DEV).manual_seed(32)
    q, k_cache, v_cache, table, cu = _paged_case(g, [1], [20], H, KV, D, P, torch.float32)
    table[0, 1] = k_cache.shape[0] + 5
    with pytest.raises(ops.KernelError, match="page"):
        _run_attn(ops, q, k_cache, v_cache, table, cu, [1], [20], 1.0, 0)


def test_attention_refuses_a_head_size_it_cannot_do(ops):
    with pytest.raises(ValueError, match="multiples of 16"):
        ops.attention_tile_specs(4, 2, 24, torch.bfloat16)


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (6, 2, 32, 8), (16, 1, 64, 16), (2, 2, 256, 32)])
@pytest.mark.parametrize("window", [0, 300])
def test_split_kv_decode_on_long_contexts(ops, H, KV, D, P, window):
    """Few decoded tokens over long contexts: the keys of each request are cut over several blocks whose partial
    results are merged. One request has a single key (most of its pieces are empty), one a few new tokens."""
    g = torch.Generator(device=DEV).manual_seed(50 + D)
    q_lens = [1, 1, 1, 5]
    ctx_lens = [1500, 333, 1, 1029]
    assert ops.attention_splits(4 if H // KV <= 16 else 8, H, KV, max(ctx_lens)) > 1
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    table = _release_behind_window(table, q_lens, ctx_lens, P, window)
    got = _run_attn(ops, q, k_cache, v_cache, table, cu, q_lens, ctx_lens, D ** -0.5, window)
    assert ops.last_short_attention_kernel(D) == "attn_mma_decode_kernel"
    want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (6, 2, 32, 8), (3, 3, 64, 16)])
def test_prefill_kernel_on_long_portions(ops, H, KV, D, P):
    """Portions of hundreds of tokens, from position 0 and deep inside a context, several key blocks each."""
    g = torch.Generator(device=DEV).manual_seed(60 + D)
    q_lens = [300, 130, 64]
    ctx_lens = [300, 517, 1000]
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    for window in (0, 77):
        released = _release_behind_window(table, q_lens, ctx_lens, P, window)
        got = _run_attn(ops, q, k_cache, v_cache, released, cu, q_lens, ctx_lens, D ** -0.5, window)
        want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
        torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------------------------------------ sampling
def test_greedy_takes_the_first_maximum(ops):
    logits = torch.randn(6, 1000, device=DEV)
    logits[0, 500] = logits[0, 700] = 50.0
    logits[1, 999] = 60.0
    logits[2, 0] = 60.0
    logits[3] = 1.0
    got = ops.sample(logits).tolist()
    assert got[0] == 500 and got[1] == 999 and got[2] == 0 and got[3] == 0
    assert got[4:] == logits[4:].argmax(-1).tolist()


@pytest.mark.parametrize("vocab", [509, 151936])
def test_temperature_sampling_follows_the_cdf_and_its_seed(ops, vocab):
    g = torch.Generator(device=DEV).manual_seed(40)
    rows = 16
    logits = torch.randn(rows, vocab, device=DEV, generator=g) * 2
    temp = torch.full((rows,), 0.7, device=DEV)
    temp[3] = 0.0  # greedy among the sampled
    seeds = [123456789012345 + 17 * r for r in range(rows)]
    lo = torch.tensor([(s & 0xFFFFFFFF) - (1 << 32) if (s & 0xFFFFFFFF) >= (1 << 31) else (s & 0xFFFFFFFF) for s in seeds], dtype=torch.int32, device=DEV)
    hi = torch.tensor([s >> 32 for s in seeds], dtype=torch.int32, device=DEV)
    counter = torch.arange(rows, dtype=torch.int32, device=DEV)
    got = ops.sample(logits, temp, lo, hi, counter).tolist()
    assert got[3] == int(logits[3].argmax())
    for r in range(rows):
        if r == 3:
            continue
        cdf, target = KP.sample_interval(logits[r].cpu(), 0.7, seeds[r], r)
        i = got[r]
        below = float(cdf[i - 1]) if i > 0 else 0.0
        slack = 1e-5 * float(cdf[-1])
        assert below - slack <= target <= float(cdf[i]) + slack, f"row {r}: index {i} does not hold the target"
    # the same row gives the same token whatever else is in the batch and wherever it sits
    alone = ops.sample(logits[5:6].contiguous(), temp[5:6].contiguous(), lo[5:6].contiguous(), hi[5:6].contiguous(),
                       counter[5:6].contiguous()).tolist()
    assert alone == [got[5]]
    # different counters give different draws somewhere
    again = ops.sample(logits, temp, lo, hi, counter + 100).tolist()
    assert again != got


def test_repetition_penalty(ops):
    logits = torch.tensor([[2.0, -2.0, 3.0, -1.0], [2.0, -2.0, 3.0, -1.0]], device=DEV)
    seen = torch.zeros(3, 4, dtype=torch.uint8, device=DEV)
    ops.mark_seen(seen, torch.tensor([2, 2, 0], dtype=torch.int32, device=DEV), torch.tensor([0, 1, 3], dtype=torch.int32, device=DEV))
    assert seen.tolist() == [[0, 0, 0, 1], [0, 0, 0, 0], [1, 1, 0, 0]]
    ops.repetition_penalty(logits, seen, torch.tensor([2, 0], dtype=torch.int32, device=DEV), torch.tensor([2.0, 1.0], device=DEV))
    assert logits.tolist() == [[1.0, -4.0, 3.0, -1.0], [2.0, -2.0, 3.0, -1.0]]


def test_no_cpu_path(ops):
    with pytest.raises(ops.KernelError, match="CUDA device only"):
        ops.silu_mul(torch.zeros(2, 4))


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (8, 2, 64, 8), (4, 4, 128, 64), (16, 1, 64, 256), (2, 2, 256, 32)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("uneven", [False, True])
def test_split_kv_decode_with_tma_gathers(ops, H, KV, D, P, window, uneven):
    """The split-KV kernel fetching K and V by TMA from a pool of several layers (the layer is chosen by a row offset
    into the pool's tensor map): against the plain statement, and against the cp.async version of the same kernel. Every
    request cut into the same number of pieces, and (``uneven``: what the engine says of such lengths) all key blocks dealt
    out evenly to one round of blocks."""
    g = torch.Generator(device=DEV).manual_seed(70 + D)
    q_lens = [1, 1, 1, 5, 2]
    ctx_lens = [1500, 333, 1, 1029, 64]
    layers, layer = 3, 1
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    table = _release_behind_window(table, q_lens, ctx_lens, P, window)
    assert window == 0 or (table[0] == -1).sum() >= (1500 - 300) // P - 1
    k_pool = torch.randn(layers, *k_cache.shape, device=DEV, generator=g).bfloat16()
    v_pool = torch.randn(layers, *v_cache.shape, device=DEV, generator=g).bfloat16()
    k_pool[layer], v_pool[layer] = k_cache, v_cache
    maps = ops.make_kv_maps(k_pool, v_pool, P)
    assert maps is not None
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16)
    tma_tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    status = ops.new_status(DEV)
    common = dict( cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                  block_table=table, page_size=P, scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status)
    got = ops.paged_attention(q, k_pool[layer], v_pool[layer], tiles=tma_tiles, kv_maps=maps, layer_in_pool=layer, uneven=uneven, **common)
    assert ops.last_short_attention_kernel(D) == ("attn_tma_decode_walk_kernel (one round)" if uneven else "attn_tma_decode_kernel")
    plain_gather = ops.paged_attention(q, k_pool[layer], v_pool[layer], tiles=tiles, **common)
    ops.check_status(status)
    want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.float(), plain_gather.float(), atol=4e-3, rtol=4e-3)


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (6, 2, 64, 8), (3, 3, 64, 16), (4, 1, 128, 64), (40, 1, 64, 16)])
def test_prefill_kernel_with_tma_gathers_on_long_portions(ops, H, KV, D, P):
    """The tcgen05 prefill kernel (256-row tiles, K and V by TMA): portions of hundreds of tokens from position 0 and deep inside a
    context, beside short entries that go to the split-KV kernel in the same call."""
    g = torch.Generator(device=DEV).manual_seed(80 + D)
    q_lens = [300, 130, 64, 1, 9]
    ctx_lens = [300, 517, 1000, 77, 9]
    layers, layer = 2, 1
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    k_pool = torch.randn(layers, *k_cache.shape, device=DEV, generator=g).bfloat16()
    v_pool = torch.randn(layers, *v_cache.shape, device=DEV, generator=g).bfloat16()
    k_pool[layer], v_pool[layer] = k_cache, v_cache
    maps = ops.make_kv_maps(k_pool, v_pool, P)
    assert maps is not None
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    assert any(spec[0] == max(1, 256 // min(H // KV, 256)) and spec[1] > 1 for spec in tiles), "the long list is cut for 256-row tiles"
    status = ops.new_status(DEV)
    for window in (0, 77):
        released = _release_behind_window(table, q_lens, ctx_lens, P, window)
        got = ops.paged_attention(q, k_pool[layer], v_pool[layer], tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                                  ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=released, page_size=P,
                                  scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps, layer_in_pool=layer)
        ops.check_status(status)
        want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
        torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,D,P,n_req,long_ctx", [(32, 8, 128, 16, 80, 2000), (16, 4, 64, 8, 50, 6000), (16, 16, 128, 32, 30, 1300)])
@pytest.mark.parametrize("window", [0, 300])
def test_split_kv_decode_walking_over_more_pieces_than_blocks_fit(ops, H, KV, D, P, n_req, long_ctx, window):
    """More (request, KV head, split) pieces than blocks fit on the GPU at once: the launcher then starts one round of
    blocks that walk over the pieces. Ragged contexts (one key; around a key block's edge; thousands), mostly one
    decoded token each and a few short portions; a shape with one split and shapes with several; behind a window the
    block tables name released pages."""
    g = torch.Generator(device=DEV).manual_seed(90 + D + n_req)
    ctx_lens = ([1, 63, 64, 65, long_ctx, 129, 2, 700] * n_req)[:n_req]
    q_lens = [1] * n_req
    q_lens[3], q_lens[7] = 3, 8         # short portions ride in the same kernel
    ctx_lens = [max(c, ql) for c, ql in zip(ctx_lens, q_lens)]
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    released = _release_behind_window(table, q_lens, ctx_lens, P, window)
    maps = ops.make_kv_maps(k_cache[None], v_cache[None], P)
    assert maps is not None
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    short = ops.attention_tile_specs(H, KV, D, torch.bfloat16, P)[0]
    splits = ops.attention_splits(tiles[short][2], H, KV, max(ctx_lens))
    assert tiles[short][2] * KV * splits > 2 * ops.num_sms(), "the case must outgrow one round of blocks"
    assert (n_req == 30) == (splits == 1), "one shape with a single piece per request, the others with several"
    status = ops.new_status(DEV)
    got = ops.paged_attention(q, k_cache, v_cache, tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                              ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=released, page_size=P,
                              scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps, layer_in_pool=0)
    ops.check_status(status)
    assert ops.last_short_attention_kernel(D) == "attn_tma_decode_walk_kernel"
    want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
    # told that the lengths differ much (they do), the step takes the even cut instead: the same kernel, every block with the
    # same share of all keys (640 (request, KV head) units in the first shape: two units share a start in shared memory)
    again = ops.paged_attention(q, k_cache, v_cache, tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                                ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=released, page_size=P,
                                scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps, layer_in_pool=0,
                                uneven=True)
    ops.check_status(status)
    assert ops.last_short_attention_kernel(D) == "attn_tma_decode_walk_kernel (one round)"
    assert (n_req == 80) == (tiles[short][2] * KV > 512)
    torch.testing.assert_close(again.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (4, 2, 64, 8), (6, 1, 128, 128)])
@pytest.mark.parametrize("window", [0, 300])
def test_split_kv_decode_even_cut_of_very_different_lengths(ops, H, KV, D, P, window):
    """The even cut: one key beside eight thousand, a block's run ending exactly at a request's end (64, 128 keys), requests
    that get one piece and requests that get dozens, short portions among the decoded tokens; with a window the tables name
    released pages. A far key is made to stand out in the longest request so that a lost piece shows."""
    g = torch.Generator(device=DEV).manual_seed(95 + D)
    ctx_lens = [1, 5000, 64, 65, 3000, 129, 2, 700, 8000, 63, 128, 256]
    q_lens = [1, 1, 1, 3, 1, 1, 2, 8, 1, 1, 1, 1]
    q, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    if window == 0:      # request 8's key 1234 answers its query: without it the output is another
        page = int(table[8, 1234 // P])
        k_cache[page, 1234 % P] = (q[cu[8], ::H // KV] * 3).to(k_cache.dtype)
    released = _release_behind_window(table, q_lens, ctx_lens, P, window)
    maps = ops.make_kv_maps(k_cache[None], v_cache[None], P)
    assert maps is not None
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    status = ops.new_status(DEV)
    got = ops.paged_attention(q, k_cache, v_cache, tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                              ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=released, page_size=P,
                              scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps, layer_in_pool=0,
                              uneven=True)
    ops.check_status(status)
    assert ops.last_short_attention_kernel(D) == "attn_tma_decode_walk_kernel (one round)"
    want = KP.paged_attention(q, k_cache, v_cache, cu, ctx_lens, table, D ** -0.5, window)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,D,P", [(32, 8, 128, 16), (8, 2, 64, 8), (2, 2, 256, 32), (40, 1, 64, 16), (6, 3, 192, 64)])
@pytest.mark.parametrize("window", [0, 300])
@pytest.mark.parametrize("norm,rotate,store", [(True, True, True), (False, True, True), (True, False, True), (True, True, False)])
def test_decode_attention_takes_the_raw_projections(ops, monkeypatch, H, KV, D, P, window, norm, rotate, store):
    """A step of one token per request given to the split-KV kernel as raw q|k|v projections: the kernel normalises and
    rotates q and the new k itself, stores k and v, and attends. Against the stand-alone q/k norm + rotation + store kernel
    followed by the same attention kernel on a copy of the pool: the same cache afterwards (every other row untouched) and
    the same output. New tokens at a key block's first and last row, as a request's only key, behind thousands of keys;
    more q heads per KV head than a tile has rows; without norm, without rotation, and for a layer that stores nothing."""
    monkeypatch.setattr(ops, "FUSE_QKV", True)     # whatever the environment's switches say
    monkeypatch.setattr(ops, "DECODE_CUT", "auto")
    g = torch.Generator(device=DEV).manual_seed(170 + D + H)
    ctx_lens = [65, 1500, 64, 1, 333, 129, 2, 700, 1029, 63, 128, 256]
    n = len(ctx_lens)
    # as many of them as get a block for each of their pieces (at head sizes of 192 and more an SM holds one block, not two)
    while not ops.attention_takes_projections(D, torch.bfloat16, P, True, requests=n, num_heads=H, num_kv_heads=KV, kv_len_bound=max(ctx_lens[:n])):
        n -= 1
    assert n >= 6
    ctx_lens = ctx_lens[:n]
    q_lens = [1] * n
    layers, layer, eps, maxpos = 2, 1, 1e-5, max(ctx_lens) + 3
    _, k_cache, v_cache, table, cu = _paged_case(g, q_lens, ctx_lens, H, KV, D, P, torch.bfloat16)
    table = _release_behind_window(table, q_lens, ctx_lens, P, window)
    k_pool = torch.randn(layers, *k_cache.shape, device=DEV, generator=g).bfloat16()
    v_pool = torch.randn(layers, *v_cache.shape, device=DEV, generator=g).bfloat16()
    k_pool[layer], v_pool[layer] = k_cache, v_cache
    qkv = torch.randn(n, (H + 2 * KV) * D, device=DEV, generator=g).bfloat16()
    qw = 1 + 0.2 * torch.randn(D, device=DEV, generator=g) if norm else None
    kw = 1 + 0.2 * torch.randn(D, device=DEV, generator=g) if norm else None
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
    fr = torch.outer(torch.arange(maxpos, dtype=torch.float), inv)
    cos, sin = (fr.cos().to(DEV), fr.sin().to(DEV)) if rotate else (None, None)
    positions = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(table[r, (c - 1) // P]) * P + (c - 1) % P for r, c in enumerate(ctx_lens)], dtype=torch.int32, device=DEV)
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    short = ops.attention_tile_specs(H, KV, D, torch.bfloat16, P)[0]
    assert ops.attention_splits(tiles[short][2], H, KV, max(ctx_lens)) > 1, "the new token's piece is to be one of several"
    status = ops.new_status(DEV)
    common = dict(tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                  block_table=table, page_size=P, scale=D ** -0.5, window=window, kv_len_bound=max(ctx_lens), status=status, layer_in_pool=layer,
                  uneven=False)
    name = "attn_tma_decode_kernel"
    # the two kernels, on a copy of the pool
    k_two, v_two = k_pool.clone(), v_pool.clone()
    q = ops.qk_norm_rope_store(qkv, qw, kw, cos, sin, positions, slots if store else torch.full_like(slots, -1), k_two[layer], v_two[layer],
                               H, KV, D, eps, status)
    want = ops.paged_attention(q, k_two[layer], v_two[layer], kv_maps=ops.make_kv_maps(k_two, v_two, P), **common)
    assert ops.last_short_attention_kernel(D) == name
    # the one kernel
    maps = ops.make_kv_maps(k_pool, v_pool, P)
    assert ops.attention_takes_projections(D, torch.bfloat16, P, maps, requests=n, num_heads=H, num_kv_heads=KV, kv_len_bound=max(ctx_lens))
    before = (k_pool.clone(), v_pool.clone())
    got = ops.decode_attention_from_projections(qkv, qw, kw, cos, sin, k_pool[layer], v_pool[layer], store=store, num_heads=H, num_kv_heads=KV,
                                                head_dim=D, eps=eps, kv_maps=maps, **common)
    ops.check_status(status)
    assert ops.last_short_attention_kernel(D) == name
    # v is a copy; k is computed in fp32 and rounded once by both kernels, whose compiled sums may differ in the last bit of
    # fp32: at most one bf16 step apart; every row but the new tokens' stays as it was
    assert torch.equal(v_pool, v_two)
    torch.testing.assert_close(k_pool.float(), k_two.float(), rtol=2.0 ** -7, atol=1e-6)
    new_rows = torch.zeros(k_pool[layer].numel() // (KV * D), dtype=torch.bool, device=DEV)
    if store:
        new_rows[slots.long()] = True
    for now, was in ((k_pool, before[0]), (v_pool, before[1])):
        assert torch.equal(now[0], was[0]), "another layer of the pool was written"
        assert torch.equal(now[layer].view(-1, KV * D)[~new_rows], was[layer].view(-1, KV * D)[~new_rows]), "a row of another token was written"
    if store:
        assert not torch.equal(k_pool[layer].view(-1, KV * D)[new_rows], before[0][layer].view(-1, KV * D)[new_rows])
    torch.testing.assert_close(got.float(), want.float(), atol=4e-3, rtol=2.0 ** -7)   # one bf16 step where a key moved by one
    if not norm:
        return
    # and against the plain statement of both steps
    wq, wk, wv = KP.qk_norm_rope(qkv, qw, kw, cos, sin, positions, H, KV, D, eps)
    if store:
        kc, vc = before[0][layer].clone().view(-1, KV, D), before[1][layer].clone().view(-1, KV, D)
        kc[slots.long()], vc[slots.long()] = wk.bfloat16(), wv.bfloat16()
    else:
        kc, vc = before[0][layer], before[1][layer]
    plain = KP.paged_attention(wq.bfloat16(), kc.view_as(k_cache), vc.view_as(v_cache), cu, ctx_lens, table, D ** -0.5, window)
    torch.testing.assert_close(got.float(), plain, atol=2e-2, rtol=2e-2)


def test_decode_attention_from_projections_refuses_what_it_cannot_do(ops, monkeypatch):
    monkeypatch.setattr(ops, "FUSE_QKV", True)
    monkeypatch.setattr(ops, "DECODE_CUT", "auto")
    H, KV, D, P, n = 4, 2, 64, 16, 3
    k_pool = torch.zeros(1, 8, P, KV, D, device=DEV, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    maps = ops.make_kv_maps(k_pool, v_pool, P)
    assert not ops.attention_takes_projections(48, torch.bfloat16, P, maps)       # head size not a multiple of 64
    assert not ops.attention_takes_projections(D, torch.float32, P, maps)
    assert not ops.attention_takes_projections(D, torch.bfloat16, 4, maps)        # pages too small for a TMA box
    assert not ops.attention_takes_projections(D, torch.bfloat16, P, None)
    # only with a block for every piece: not when a round of blocks walks over more pieces, nor with the even cut
    assert ops.attention_takes_projections(D, torch.bfloat16, P, maps, requests=8, num_heads=H, num_kv_heads=KV, kv_len_bound=2048)
    assert not ops.attention_takes_projections(D, torch.bfloat16, P, maps, requests=400, num_heads=H, num_kv_heads=KV, kv_len_bound=2048)
    assert not ops.attention_takes_projections(D, torch.bfloat16, P, maps, requests=8, num_heads=H, num_kv_heads=KV, kv_len_bound=8192, uneven=True)
    q_lens, ctx_lens = [1, 2, 1], [5, 9, 3]       # one request brings two tokens
    tiles = _tiles(ops, q_lens, H, KV, D, torch.bfloat16, P)
    qkv = torch.zeros(sum(q_lens), (H + 2 * KV) * D, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="one token per request"):
        ops.decode_attention_from_projections(qkv, None, None, None, None, k_pool[0], v_pool[0], store=True, num_heads=H, num_kv_heads=KV,
                                              head_dim=D, eps=1e-6, tiles=tiles, cu_q=torch.tensor([0, 1, 3, 4], dtype=torch.int32, device=DEV),
                                              ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                                              block_table=torch.zeros(n, 2, dtype=torch.int32, device=DEV), page_size=P, scale=1.0, window=0,
                                              kv_len_bound=16, status=ops.new_status(DEV), kv_maps=maps)


def test_tma_gathers_are_refused_for_sizes_they_cannot_do(ops):
    pool = torch.zeros(1, 4, 4, 2, 128, device=DEV, dtype=torch.bfloat16)
    assert ops.make_kv_maps(pool, pool, 4) is None          # pages of 4 tokens
    pool = torch.zeros(1, 4, 16, 2, 48, device=DEV, dtype=torch.bfloat16)
    assert ops.make_kv_maps(pool, pool, 16) is None         # head size 48
    assert ops.make_kv_maps(pool.float(), pool.float(), 16) is None
