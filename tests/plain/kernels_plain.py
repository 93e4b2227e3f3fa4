"""Plain PyTorch statements of what each CUDA kernel computes, for the kernel-alone tests. fp32 (or fp64) on
whatever device the inputs are on; loops instead of cleverness. Shares no code with the engine."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def add_rms_norm(x, residual, weight, eps):
    """oxr_runtime/language.py:94-99 with the sum kept in fp32: (normed, new residual)."""
    s = x.float() if residual is None else x.float() + residual.float()
    return s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight.float(), s


def silu_mul(gate_up):
    """oxr_runtime/language.py:102-104."""
    gate, up = gate_up.float().chunk(2, dim=-1)
    return F.silu(gate) * up


def qk_norm_rope(qkv, q_weight, k_weight, cos, sin, positions, H, KV, D, eps):
    """oxr_runtime/kernels.py:133-154 without its bf16 rounding points: returns q [n,H,D], k [n,KV,D], v [n,KV,D]."""
    n = qkv.shape[0]
    q, k, v = qkv.float().view(n, H + 2 * KV, D).split((H, KV, KV), dim=1)
    half = D // 2

    def norm_rope(x, w):
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            y = y * w.float()
        if cos is None:
            return y
        c, s = cos[positions.long()].float()[:, None, :], sin[positions.long()].float()[:, None, :]
        y1, y2 = y[..., :half], y[..., half:]
        return torch.cat((y1 * c - y2 * s, y1 * s + y2 * c), dim=-1)

    return norm_rope(q, q_weight), norm_rope(k, k_weight), v


def paged_attention(q, k_cache, v_cache, cu_q, ctx_lens, block_table, scale, window=0):
    """tests/test_language_fused.py:19-57 (gather the request's pages, flatten, cut to its length, attend with the
    queries aligned to the end), one request and one head at a time. q [T,H,D]; caches [pages,P,KV,D]."""
    T, H, D = q.shape
    KV = k_cache.shape[2]
    rep = H // KV
    out = torch.zeros(T, H, D, dtype=torch.float32, device=q.device)
    for r in range(len(ctx_lens)):
        a, b = int(cu_q[r]), int(cu_q[r + 1])
        n, m = b - a, int(ctx_lens[r])
        pages = block_table[r].long().clamp(min=0)
        k = k_cache[pages].flatten(0, 1)[:m].float()
        v = v_cache[pages].flatten(0, 1)[:m].float()
        for i in range(n):
            p = m - n + i  # absolute position of this query
            lo = max(0, p - window + 1) if window > 0 else 0
            for h in range(H):
                kk, vv = k[lo:p + 1, h // rep], v[lo:p + 1, h // rep]
                s = (kk @ q[a + i, h].float()) * scale
                out[a + i, h] = s.softmax(0) @ vv
    return out


_M64 = (1 << 64) - 1


def uniform_from(seed: int, counter: int) -> float:
    """The sampler's random number: splitmix64 of seed + golden * (counter + 1), top 24 bits, in [0, 1)."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z = z ^ (z >> 31)
    return (z >> 40) / 16777216.0


def sample_interval(logits_row, temperature, seed, counter):
    """For temperature sampling by inverse CDF: (cdf in fp64, target). Index i is a right answer when
    cdf[i-1] <= target < cdf[i] up to rounding."""
    p = torch.exp((logits_row.double() - logits_row.double().max()) / temperature)
    cdf = torch.cumsum(p, 0)
    return cdf, uniform_from(seed, counter) * float(cdf[-1])
