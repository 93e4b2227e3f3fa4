"""Times one kernel of this package alone at given sizes (CUDA events around a CUDA graph of repeated calls, after
warm-up, inputs rotated so that every call reads memory that is not in L2), and prints one JSON line. Also the
command to put under ``ncu``.

    python -m oxr_inference_b200.ops.microbench gemm --m 8 --n 24576 --k 4096
    python -m oxr_inference_b200.ops.microbench attention --batch 8 --q-len 1 --context 2048
    python -m oxr_inference_b200.ops.microbench attention --batch 1 --q-len 2048 --context 2048
    python -m oxr_inference_b200.ops.microbench norm --rows 8 --hidden 4096
    python -m oxr_inference_b200.ops.microbench rope --tokens 2048
    OXR_B200_TIMELINE=1 python -m oxr_inference_b200.ops.microbench timeline --batch 8 --context 2048

``timeline`` runs decode steps of a few layers of Qwen3-8B's sizes through the engine (CUDA graphs and all) with the kernels'
timeline stamps compiled in, and prints, kernel by kernel in the order of one step, when its blocks were released, when
the first and the last of them ended, and the gap since the kernel before.
"""

from __future__ import annotations

import argparse
import json
import statistics

import torch

from oxr_inference_b200 import ops


def _time(fn, reps: int, warmup: int = 3) -> float:
    """Microseconds per call on the device: `reps` calls are captured into one CUDA graph (as a decode step's kernels
    are) and the graph's replay is timed, so host launch overhead is not part of the number."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(warmup):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            fn(i)
    times = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / reps)
    return statistics.median(times)


def gemm(args) -> dict:
    m, n, k = args.m, args.n, args.k
    copies = max(2, int(300e6 // (n * k * 2)) + 1)  # rotate over > 2 x L2 of weights
    ws = [torch.randn(n, k, device="cuda").mul_(0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(m, k, device="cuda").bfloat16()
    out_dtype = torch.float32 if args.fp32_out else torch.bfloat16
    if args.library:   # cuBLAS through torch.mm, for comparison
        us = _time(lambda i: torch.mm(x, ws[i % copies].t()), args.reps)
    elif args.gated:   # silu(gate) * up of a weight whose gate and up rows alternate in groups of 8
        us = _time(lambda i: ops.gated_silu_linear(x, ws[i % copies], ops.GATE_UP_INTERLEAVE), args.reps)
    else:
        us = _time(lambda i: ops.linear(x, ws[i % copies], out_dtype), args.reps)
    bytes_ = n * k * 2 + m * k * 2 + m * n * (4 if args.fp32_out else 2)
    return {"kernel": "torch.mm (cuBLAS)" if args.library else "gated_silu_linear" if args.gated else "linear", "m": m, "n": n, "k": k, "us": round(us, 2), "GB/s": round(bytes_ / us / 1e3, 1),
            "TFLOP/s": round(2 * m * n * k / us / 1e6, 2)}


def attention(args) -> dict:
    H, KV, D, P = args.heads, args.kv_heads, args.head_dim, args.page_size
    B, q_len, ctx = args.batch, args.q_len, args.context
    pages_per = -(-ctx // P)
    layers = max(2, int(300e6 // (B * pages_per * P * KV * D * 2 * 2)) + 1)
    n_pages = B * pages_per
    pools = [(torch.randn(n_pages, P, KV, D, device="cuda").bfloat16(), torch.randn(n_pages, P, KV, D, device="cuda").bfloat16())
             for _ in range(layers)]
    table = torch.randperm(n_pages, device="cuda").int().view(B, pages_per).contiguous()
    q = torch.randn(B * q_len, H, D, device="cuda").bfloat16()
    cu = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32, device="cuda")
    ctx_lens = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    if args.ragged:   # decoding requests of very different lengths: from q_len + 16 keys up to the given context
        gen = torch.Generator().manual_seed(1)
        ctx_lens = torch.randint(q_len + 16, ctx + 1, (B,), generator=gen).int()
        if not args.unsorted:      # the engine runs a decode step's requests longest context first
            ctx_lens = ctx_lens.sort(descending=True).values
        ctx_lens = ctx_lens.cuda()
    tiles = {}
    for spec in ops.attention_tile_specs(H, KV, D, torch.bfloat16, None if args.no_tma else P):
        tpt, lo, hi = spec
        req, tok = [], []
        if lo <= q_len <= hi:
            for r in range(B):
                for t0 in range(0, q_len, tpt):
                    req.append(r)
                    tok.append(t0)
        tiles[spec] = (torch.tensor(req + [0], dtype=torch.int32, device="cuda"), torch.tensor(tok + [0], dtype=torch.int32, device="cuda"), len(req))
    status = ops.new_status("cuda")
    k_pool = torch.stack([p[0] for p in pools])
    v_pool = torch.stack([p[1] for p in pools])
    del pools
    maps = None if args.no_tma else ops.make_kv_maps(k_pool, v_pool, P)

    from oxr_inference_b200.parts.base import uneven_lengths
    uneven = uneven_lengths(ctx_lens.tolist())     # what the engine tells the kernel about such a step

    common = dict(tiles=tiles, cu_q=cu, ctx_lens=ctx_lens, block_table=table, page_size=P, scale=D ** -0.5, window=0, kv_len_bound=ctx,
                  status=status, kv_maps=maps, uneven=uneven)
    if args.from_projections or args.with_rope_kernel:
        # a decode step's attention from the raw q|k|v projections: in one kernel, or behind the q/k norm + RoPE + store kernel
        if q_len != 1:
            raise SystemExit("--from-projections / --with-rope-kernel: a step of one token per request (--q-len 1)")
        qkv = torch.randn(B, (H + 2 * KV) * D, device="cuda").bfloat16()
        qw, kw = torch.ones(D, device="cuda"), torch.ones(D, device="cuda")
        angles = torch.outer(torch.arange(ctx + 1, dtype=torch.float), 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float) / D)))
        cos, sin = angles.cos().cuda(), angles.sin().cuda()
        positions = (ctx_lens - 1).int()
        slots = (table.gather(1, (positions // P).long()[:, None])[:, 0] * P + positions % P).int()
        if args.from_projections and not ops.attention_takes_projections(D, torch.bfloat16, P, maps, requests=B, num_heads=H, num_kv_heads=KV,
                                                                         kv_len_bound=ctx, uneven=uneven):
            raise SystemExit("the attention kernel does not take the projections itself for this step")

    def run(i):
        layer = i % layers
        if args.from_projections:
            ops.decode_attention_from_projections(qkv, qw, kw, cos, sin, k_pool[layer], v_pool[layer], store=True, num_heads=H, num_kv_heads=KV,
                                                  head_dim=D, eps=1e-6, layer_in_pool=layer, **common)
            return
        x = q
        if args.with_rope_kernel:
            x = ops.qk_norm_rope_store(qkv, qw, kw, cos, sin, positions, slots, k_pool[layer], v_pool[layer], H, KV, D, 1e-6, status)
        ops.paged_attention(x, k_pool[layer], v_pool[layer], layer_in_pool=layer, **common)
    us = _time(run, args.reps)
    ops.check_status(status)
    lens = ctx_lens.tolist()
    kv_bytes = sum(lens) * KV * D * 2 * 2
    flops = sum(4 * H * D * (c - q_len + i + 1) for c in lens for i in range(q_len))
    name = ("decode_attention_from_projections" if args.from_projections else
            "qk_norm_rope_store + paged_attention" if args.with_rope_kernel else "paged_attention")
    return {"kernel": name, "batch": B, "q_len": q_len, "context": ctx if not args.ragged else f"{min(lens)}..{max(lens)}", "heads": H, "kv_heads": KV, "head_dim": D,
            "us": round(us, 2), "KV GB/s": round(kv_bytes / us / 1e3, 1), "TFLOP/s": round(flops / us / 1e6, 2)}


def norm(args) -> dict:
    rows, hidden = args.rows, args.hidden
    copies = max(2, int(300e6 // (rows * hidden * 12)) + 1) if rows * hidden * 12 > 1e6 else 4
    xs = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(copies)]
    rs = [torch.randn(rows, hidden, device="cuda") for _ in range(copies)]
    w = torch.ones(hidden, device="cuda")
    us = _time(lambda i: ops.add_rms_norm(xs[i % copies], rs[i % copies], w, 1e-6), args.reps)
    return {"kernel": "add_rms_norm", "rows": rows, "hidden": hidden, "us": round(us, 2),
            "GB/s": round(rows * hidden * (2 + 4 + 4 + 2) / us / 1e3, 1)}


def rope(args) -> dict:
    """q/k head norm + rotation + store of K and V into a layer's pages, for ``tokens`` new tokens."""
    H, KV, D, P, T = args.heads, args.kv_heads, args.head_dim, args.page_size, args.tokens
    width = (H + 2 * KV) * D
    copies = max(2, int(300e6 // (T * width * 4)) + 1) if T * width * 4 > 1e6 else 4
    qkvs = [torch.randn(T, width, device="cuda").bfloat16() for _ in range(copies)]
    qw, kw = torch.ones(D, device="cuda"), torch.ones(D, device="cuda")
    angles = torch.outer(torch.arange(max(T, 4096), dtype=torch.float), 1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float) / D)))
    cos, sin = angles.cos().cuda(), angles.sin().cuda()
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    pages = -(-T // P)
    slots = (torch.randperm(pages, device="cuda").int().repeat_interleave(P)[:T] * P + pos % P).int()
    pools = [(torch.zeros(pages, P, KV, D, device="cuda", dtype=torch.bfloat16), torch.zeros(pages, P, KV, D, device="cuda", dtype=torch.bfloat16))
             for _ in range(copies)]
    status = ops.new_status("cuda")
    us = _time(lambda i: ops.qk_norm_rope_store(qkvs[i % copies], qw, kw, cos, sin, pos, slots, pools[i % copies][0], pools[i % copies][1],
                                                H, KV, D, 1e-6, status), args.reps)
    ops.check_status(status)
    return {"kernel": "qk_norm_rope_store", "tokens": T, "heads": H, "kv_heads": KV, "head_dim": D, "us": round(us, 2),
            "GB/s": round(T * width * 2 * 2 / us / 1e3, 1)}


def timeline(args) -> dict:
    import ctypes

    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.ops import build
    from oxr_inference_b200.sampling import SamplingParams

    if not build.TIMELINE:
        raise SystemExit("set OXR_B200_TIMELINE=1: the stamps are compiled in only then (libraries of their own, *_tl)")
    B, ctx, D = args.batch, args.context, args.head_dim
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": args.hidden, "intermediate_size": args.intermediate,
           "num_hidden_layers": args.layers, "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads, "head_dim": D,
           "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "vocab_size": args.vocab, "tie_word_embeddings": False,
           "max_position_embeddings": ctx + 512}
    engine = Engine(random_config=cfg, seed=0, settings=EngineSettings(
        dtype="bfloat16", page_size=args.page_size, num_pages=B * (ctx // args.page_size + 12) + 64, max_running=max(B, 8), cuda_graphs=True,
        max_positions=ctx + 512))
    gen = torch.Generator().manual_seed(0)
    for _ in range(B):
        engine.add_request(torch.randint(0, args.vocab, (ctx,), generator=gen).tolist(), SamplingParams(max_tokens=64, ignore_eos=True))
    while engine.scheduler.waiting or any(r.pending > 1 for r in engine.scheduler.running):
        engine.step()
    for _ in range(6):
        engine.step()          # decode steps: graphs captured, clocks up
    torch.cuda.synchronize()
    words = 1 << 15
    readers = [(ops._lib(), "oxr_tl_read_stream"), (ops._lib(), "oxr_tl_read_elem"), (ops._lib(), "oxr_tl_read_rope"),
               (ops._attn_lib(D), "oxr_tl_read_attn")]

    def read(lib, name):
        buf = (ctypes.c_ulonglong * words)()
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = [ctypes.c_void_p, ctypes.c_int], ctypes.c_int
        fn(buf, words)
        return [tuple(buf[i * 6 + j] for j in range(6)) for i in range(words // 6) if buf[i * 6]]

    for lib, name in readers:
        read(lib, name)        # clears
    torch.cuda.synchronize()
    engine.step()
    torch.cuda.synchronize()
    records = sorted((r for lib, name in readers for r in read(lib, name)), key=lambda r: r[1])
    names = {1: "stream gemm", 2: "rms norm", 3: "qk norm rope", 4: "attention", 5: "attention"}
    launches: list[dict] = []
    for r in records:      # a launch: records of one kind released within 2.5 us of each other (and, for products, of one size)
        kind = names.get(r[0], str(r[0]))
        size = (r[3], r[4]) if r[0] == 1 else None
        if launches and launches[-1]["kind"] == kind and launches[-1]["size"] == size and r[1] - launches[-1]["released"] < 2500:
            launches[-1]["records"].append(r)
        else:
            launches.append({"kind": kind, "size": size, "released": r[1], "records": [r]})
    t0, rows, before = launches[0]["released"], [], None
    for launch in launches:
        rs = launch["records"]
        released, first_end, last_end = min(r[1] for r in rs), min(r[2] for r in rs), max(r[2] for r in rs)
        row = {"kernel": launch["kind"] + (f" N={launch['size'][0]} K={launch['size'][1]}" if launch["size"] else ""), "blocks": len(rs),
               "released_us": round((released - t0) / 1e3, 2), "first_block_ends_us": round((first_end - released) / 1e3, 2),
               "last_block_ends_us": round((last_end - released) / 1e3, 2),
               "gap_since_kernel_before_us": None if before is None else round((released - before) / 1e3, 2)}
        if launch["kind"] == "stream gemm":   # how long before their release the blocks were resident: earliest and latest block
            row["resident_before_release_us"] = [round(max(r[1] - r[5] for r in rs) / 1e3, 2), round(min(r[1] - r[5] for r in rs) / 1e3, 2)]
        if launch["kind"] == "attention":
            row["first_keys_us"] = [round(min(r[3] - r[1] for r in rs if r[3]) / 1e3, 2), round(max(r[3] - r[1] for r in rs if r[3]) / 1e3, 2)]
            row["keys_streamed_us"] = [round(min(r[4] - r[1] for r in rs if r[4]) / 1e3, 2), round(max(r[4] - r[1] for r in rs if r[4]) / 1e3, 2)]
        rows.append(row)
        before = last_end
    for row in rows:
        print(json.dumps(row))
    return {"kernel": "timeline", "batch": B, "context": ctx, "layers": args.layers, "launches": len(rows),
            "step_us": round((max(r[2] for r in records) - t0) / 1e3, 1)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--fp32-out", action="store_true")
    g.add_argument("--library", action="store_true", help="time torch.mm (cuBLAS) on the same sizes instead")
    g.add_argument("--gated", action="store_true", help="the product with the SiLU epilogue (n counts gate and up rows)")
    g.set_defaults(run=gemm)
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--q-len", type=int, default=1)
    a.add_argument("--context", type=int, default=2048)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--no-tma", action="store_true", help="gather K and V with cp.async instead of TMA")
    a.add_argument("--ragged", action="store_true", help="contexts drawn between q_len + 16 and --context instead of all equal")
    a.add_argument("--unsorted", action="store_true", help="with --ragged: leave the requests in the order drawn")
    a.add_argument("--from-projections", action="store_true",
                   help="a decode step's attention from raw q|k|v projections: norm, rotation and cache store inside the attention kernel")
    a.add_argument("--with-rope-kernel", action="store_true", help="the same work as two kernels: q/k norm + RoPE + store, then attention")
    a.set_defaults(run=attention)
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=8)
    n.add_argument("--hidden", type=int, default=4096)
    n.set_defaults(run=norm)
    r = sub.add_parser("rope")
    r.add_argument("--tokens", type=int, default=2048)
    r.add_argument("--heads", type=int, default=32)
    r.add_argument("--kv-heads", type=int, default=8)
    r.add_argument("--head-dim", type=int, default=128)
    r.add_argument("--page-size", type=int, default=16)
    r.set_defaults(run=rope)
    t = sub.add_parser("timeline", help="kernel by kernel through one decode step (needs OXR_B200_TIMELINE=1)")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=2048)
    t.add_argument("--layers", type=int, default=4)
    t.add_argument("--hidden", type=int, default=4096)
    t.add_argument("--intermediate", type=int, default=12288)
    t.add_argument("--heads", type=int, default=32)
    t.add_argument("--kv-heads", type=int, default=8)
    t.add_argument("--head-dim", type=int, default=128)
    t.add_argument("--vocab", type=int, default=151936)
    t.add_argument("--page-size", type=int, default=16)
    t.set_defaults(run=timeline)
    for p in (g, a, n, r):
        p.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    torch.backends.cuda.matmul.allow_tf32 = False
    print(json.dumps(args.run(args)))


if __name__ == "__main__":
    main()
