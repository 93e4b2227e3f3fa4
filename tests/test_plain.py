"""The plain implementation itself: against logits the reference's own model produced (tests/golden), and its
parts against textbook statements."""

from pathlib import Path

import torch
from safetensors.torch import load_file

from plain import qwen3_plain as QP

GOLDEN = Path(__file__).resolve().parent / "golden"


def _golden():
    import importlib.util

    spec = importlib.util.spec_from_file_location("make_reference_golden", GOLDEN / "make_reference_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    t = load_file(str(GOLDEN / "reference_tiny.safetensors"))
    ids = t.pop("golden.token_ids").tolist()
    want = t.pop("golden.reference_logits")
    return dict(mod.CONFIG), t, ids, want


def test_plain_matches_the_reference_models_logits():
    cfg, weights, ids, want = _golden()
    got = QP.logits(cfg, weights, ids)
    assert got.shape == want.shape == (32, 61)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
    # and in 64-bit the two agree as closely as fp32 rounding of the reference allows
    got64 = QP.logits(cfg, {k: v.double() for k, v in weights.items()}, ids)
    torch.testing.assert_close(got64.float(), want, atol=2e-5, rtol=2e-5)


def test_rms_norm_and_rotation():
    torch.manual_seed(3)
    x = torch.randn(5, 3, 8, dtype=torch.float64)
    w = torch.rand(8, dtype=torch.float64) + 0.5
    y = QP.rms_norm(x, w, 1e-6)
    ms = x.pow(2).mean(-1)
    torch.testing.assert_close((y / w).pow(2).mean(-1), ms / (ms + 1e-6), atol=1e-12, rtol=0)
    cos, sin = QP.rope_tables(8, 10000.0, 5, torch.float64)
    r = QP.rotate_half_split(x, cos, sin)
    # a rotation keeps the length of each (j, j + D/2) pair, and position 0 is the identity
    torch.testing.assert_close(r[..., :4] ** 2 + r[..., 4:] ** 2, x[..., :4] ** 2 + x[..., 4:] ** 2)
    torch.testing.assert_close(r[0], x[0])
    # the score of a rotated pair depends on the distance only
    q = torch.randn(1, 1, 8, dtype=torch.float64).expand(5, 1, 8)
    rq = QP.rotate_half_split(q, cos, sin)
    torch.testing.assert_close((rq[1] * rq[3]).sum(), (rq[2] * rq[4]).sum())


def test_attention_mask_and_window():
    torch.manual_seed(0)
    n, H, KV, D = 9, 4, 2, 8
    q, k, v = torch.randn(n, H, D), torch.randn(n, KV, D), torch.randn(n, KV, D)
    full = QP.causal_attention(q, k, v, D ** -0.5)
    # the first query sees only the first key
    torch.testing.assert_close(full[0], v[0].repeat_interleave(2, dim=0))
    # changing a later key or value never changes an earlier query's output
    k2, v2 = k.clone(), v.clone()
    k2[5:] += 1.0
    v2[5:] -= 1.0
    torch.testing.assert_close(QP.causal_attention(q, k2, v2, D ** -0.5)[:5], full[:5])
    # window 1: each query sees itself alone; a window as long as the sequence changes nothing
    torch.testing.assert_close(QP.causal_attention(q, k, v, D ** -0.5, window=1), v.repeat_interleave(2, dim=1))
    torch.testing.assert_close(QP.causal_attention(q, k, v, D ** -0.5, window=n), full)
    # window 3: keys more than 2 behind are invisible
    k3 = k.clone()
    k3[0] += 100.0
    w3 = QP.causal_attention(q, k, v, D ** -0.5, window=3)
    torch.testing.assert_close(QP.causal_attention(q, k3, v, D ** -0.5, window=3)[3:], w3[3:])


def test_greedy_is_argmax_of_recomputed_logits():
    cfg, weights, ids, _ = _golden()
    out = QP.greedy(cfg, weights, ids[:4], 3)
    seq = ids[:4]
    for t in out:
        assert t == int(QP.logits(cfg, weights, seq)[-1].argmax())
        seq = seq + [t]
