"""Each part alone on the GPU against the plain implementation's function for it, and a toy architecture made of
the built-in parts plus a mixer with state of its own that is defined and registered here, in the test."""

import pytest
import torch

from plain import qwen3_plain as QP

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _runtime(dtype=torch.float32, max_positions=128):
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts.base import Runtime

    dev = torch.device("cuda", torch.cuda.current_device())
    return Runtime(device=dev, dtype=dtype, max_positions=max_positions, status=ops.new_status(dev), page_size=8)


def _fill(part, seed=0, scale=0.3):
    """Random tensors for every parameter of a part; returns them by local name (fp32, on the host)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, info in part.parameters().items():
        t = torch.randn(info.shape, generator=g)
        t = 1 + 0.1 * t if info.init == "around_one" else scale * t
        out[name] = t
        part.assign(name, t)
    part.finish_loading()
    return out


def test_rms_norm_part():
    from oxr_inference_b200.parts import NORMS

    rt = _runtime()
    norm = NORMS.build("rms_norm", rt, size=96, eps=1e-5)
    w = _fill(norm)["weight"].to(DEV)
    x, res = torch.randn(7, 96, device=DEV), torch.randn(7, 96, device=DEV)
    out, new_res = norm.forward(x, None)
    torch.testing.assert_close(out, QP.rms_norm(x, w, 1e-5), atol=1e-5, rtol=1e-5)
    assert torch.equal(new_res, x)
    out, new_res = norm.forward(x, res.clone())
    torch.testing.assert_close(new_res, x + res)
    torch.testing.assert_close(out, QP.rms_norm(x + res, w, 1e-5), atol=1e-5, rtol=1e-5)
    rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    torch.testing.assert_close(norm.forward_rows(x, res, rows), QP.rms_norm(x + res, w, 1e-5)[rows.long()], atol=1e-5, rtol=1e-5)


def test_rotary_table_part_is_the_reference_formula():
    from oxr_inference_b200.parts import POSITION_ENCODINGS

    rope = POSITION_ENCODINGS.build("rope_neox", _runtime(max_positions=300), dim=48, theta=1e6)
    cos, sin = rope.tables()
    want_cos, want_sin = QP.rope_tables(48, 1e6, 300, torch.float32)
    assert cos.dtype == torch.float32 and torch.equal(cos.cpu(), want_cos) and torch.equal(sin.cpu(), want_sin)


def test_swiglu_part():
    from oxr_inference_b200.parts import FEED_FORWARDS

    for dtype in (torch.float32, torch.bfloat16):
        ff = FEED_FORWARDS.build("swiglu", _runtime(dtype), hidden_size=96, intermediate_size=160)
        w = {k: v.to(DEV) for k, v in _fill(ff, scale=0.1).items()}
        if dtype == torch.bfloat16:
            w = {k: v.bfloat16().float() for k, v in w.items()}
        h = torch.randn(9, 96, device=DEV).to(dtype)
        want = QP.swiglu(h.float(), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
        tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
        torch.testing.assert_close(ff.forward(h).float(), want, **tol)


def _one_layer_context(mixer, rt, q_lens, starts, page_size=8):
    """A cache for one mixer and a step context in which request i brings q_lens[i] tokens at position starts[i]."""
    from oxr_inference_b200.cache import CacheManager, make_cache_plan
    from oxr_inference_b200.engine.batch import BatchBuilder, StepEntry

    plan = make_cache_plan([mixer.cache_need()], [None])
    manager = CacheManager(plan, page_size=page_size, num_pages=64, max_requests=4, device=rt.device, dtype=rt.dtype)
    builder = BatchBuilder(manager, mixer.tile_specs(), rt.device, rt.status)
    return manager, builder, StepEntry


@pytest.mark.parametrize("window", [0, 9])
def test_attention_part_in_portions_equals_the_plain_whole_sequence(window):
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts import MIXERS, POSITION_ENCODINGS

    rt = _runtime()
    cfg = {"num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "rms_norm_eps": 1e-5}
    rope = POSITION_ENCODINGS.build("rope_neox", rt, dim=32, theta=1e4)
    attn = MIXERS.build("gqa_attention", rt, rope, hidden_size=96, num_heads=6, num_kv_heads=2, head_dim=32, scale=32 ** -0.5,
                        qk_norm=True, eps=1e-5, window=window)
    w = {"p." + k: v.to(DEV) for k, v in _fill(attn, scale=0.15).items()}
    n = 45
    h = torch.randn(n, 96, device=DEV)
    cos, sin = QP.rope_tables(32, 1e4, n, torch.float32)
    want = QP.attention_block(h, w, "p.", cfg, cos.to(DEV), sin.to(DEV), window)
    manager, builder, StepEntry = _one_layer_context(attn, rt, None, None)
    rc = manager.open("r")
    pos, outs = 0, []
    for c in (7, 2, 20, 1, 15):
        assert manager.reserve(rc, pos + c)
        ctx = builder.build([StepEntry(rc, [0] * c, [])])
        outs.append(attn.forward(h[pos:pos + c].contiguous(), ctx, manager.layer_cache(0, ctx)))
        manager.advance(rc, pos + c)
        pos += c
    ops.check_status(rt.status)
    torch.testing.assert_close(torch.cat(outs), want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("window", [0, 9])
def test_attention_part_decodes_from_the_raw_projections_in_bfloat16(monkeypatch, window):
    """Two requests, a portion of a prompt each and then one token at a time: at a head size and page size where the
    split-KV kernel takes the raw projections itself (norm, rotation and cache store inside it), the part must take that
    path for the single-token steps and give what it gives with the stand-alone kernel before the attention, and what the
    plain implementation gives on the whole sequences."""
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts import MIXERS, POSITION_ENCODINGS

    D, H, KV, hidden = 64, 6, 2, 96
    cfg = {"num_attention_heads": H, "num_key_value_heads": KV, "head_dim": D, "rms_norm_eps": 1e-5}
    lens, first = (41, 30), (20, 11)
    hs = [torch.randn(n, hidden, device=DEV).bfloat16() for n in lens]
    taken = {"fused": 0}
    real = ops.decode_attention_from_projections

    def counting(*a, **k):
        taken["fused"] += 1
        return real(*a, **k)

    monkeypatch.setattr(ops, "decode_attention_from_projections", counting)
    monkeypatch.setattr(ops, "DECODE_CUT", "auto")
    outs = {}
    for fuse in (True, False):
        monkeypatch.setattr(ops, "FUSE_QKV", fuse)
        rt = _runtime(torch.bfloat16)
        rope = POSITION_ENCODINGS.build("rope_neox", rt, dim=D, theta=1e4)
        attn = MIXERS.build("gqa_attention", rt, rope, hidden_size=hidden, num_heads=H, num_kv_heads=KV, head_dim=D, scale=D ** -0.5,
                            qk_norm=True, eps=1e-5, window=window)
        w = {"p." + k: v.to(DEV).bfloat16().float() for k, v in _fill(attn, scale=0.15).items()}
        manager, builder, StepEntry = _one_layer_context(attn, rt, None, None)
        rcs = [manager.open("a"), manager.open("b")]
        got = [[], []]
        pos = [0, 0]

        def step(counts):
            entries = []
            for i, c in enumerate(counts):
                if c:
                    assert manager.reserve(rcs[i], pos[i] + c)
                    entries.append((i, c, StepEntry(rcs[i], [0] * c, [])))
            ctx = builder.build([e for _, _, e in entries])
            x = torch.cat([hs[i][pos[i]:pos[i] + c] for i, c, _ in entries]).contiguous()
            o = attn.forward(x, ctx, manager.layer_cache(0, ctx))
            at = 0
            for i, c, _ in entries:
                got[i].append(o[at:at + c])
                manager.advance(rcs[i], pos[i] + c)
                pos[i] += c
                at += c

        step(first)
        before = taken["fused"]
        while pos[0] < lens[0] or pos[1] < lens[1]:
            step([1 if pos[i] < lens[i] else 0 for i in range(2)])
        ops.check_status(rt.status)
        assert (taken["fused"] - before == lens[0] - first[0]) == fuse, "the single-token steps did not take the expected path"
        outs[fuse] = [torch.cat(g).float() for g in got]
        for i, n in enumerate(lens):
            cos, sin = QP.rope_tables(D, 1e4, n, torch.float32)
            want = QP.attention_block(hs[i].float(), w, "p.", cfg, cos.to(DEV), sin.to(DEV), window)
            # a sum of 384 bf16 products: its error goes with the size of its terms, not of its result: within one bf16 step of the
            # largest outputs (measured: half of that)
            torch.testing.assert_close(outs[fuse][i], want, atol=2.0 ** -7 * float(want.abs().max()), rtol=2.0 ** -6)
    for a, b in zip(outs[True], outs[False]):     # the same arithmetic up to the last bit of fp32 before a rounding to bf16
        torch.testing.assert_close(a, b, atol=4e-3, rtol=2.0 ** -6)


def test_block_part_carries_the_residual_like_the_plain_layer():
    from oxr_inference_b200.parts import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS

    rt = _runtime()
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-6, "hidden_size": 64,
           "num_hidden_layers": 1}
    rope = POSITION_ENCODINGS.build("rope_neox", rt, dim=16, theta=1e4)
    attn = MIXERS.build("gqa_attention", rt, rope, hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, scale=0.25, eps=1e-6)
    n1, n2 = NORMS.build("rms_norm", rt, size=64, eps=1e-6), NORMS.build("rms_norm", rt, size=64, eps=1e-6)
    ff = FEED_FORWARDS.build("swiglu", rt, hidden_size=64, intermediate_size=128)
    block = ARRANGEMENTS.build("pre_norm", attn, n1, ff, n2)
    w = {}
    for prefix, part, seed in (("model.layers.0.self_attn.", attn, 1), ("model.layers.0.input_layernorm.", n1, 2),
                               ("model.layers.0.mlp.", ff, 3), ("model.layers.0.post_attention_layernorm.", n2, 4)):
        w.update({prefix + k: v.to(DEV) for k, v in _fill(part, seed, 0.15).items()})
    n = 21
    x = torch.randn(n, 64, device=DEV)
    cos, sin = QP.rope_tables(16, 1e4, n, torch.float32)
    want = QP.decoder_layer(x, w, 0, cfg, cos.to(DEV), sin.to(DEV))
    manager, builder, StepEntry = _one_layer_context(attn, rt, None, None)
    rc = manager.open("r")
    assert manager.reserve(rc, n)
    ctx = builder.build([StepEntry(rc, [0] * n, [])])
    out, residual = block.forward(x, None, ctx, manager.layer_cache(0, ctx))
    torch.testing.assert_close(out + residual, want, atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("plain_norm_in_second_block", [False, True])
def test_blocks_hand_their_last_projection_to_the_next_norm_in_a_bf16_decode_step(monkeypatch, plain_norm_in_second_block):
    """Two pre-norm blocks on five rows in bfloat16: with the norms folded into the products around them (the block leaves
    its last projection to the next norm, the norm leaves the row's scale to the next product) and with every kernel on
    its own the residual stream and the output agree within bf16 rounding; and the 32-bit plain layers say the same. A norm
    that does not take part (defined here) gets whole tensors and the blocks around it still fold what they can."""
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, DeferredLinear
    from oxr_inference_b200.parts.base import Norm, ParamInfo

    if "toy_unfused_rms" not in NORMS:
        @NORMS.register("toy_unfused_rms")
        class ToyNorm(Norm):
            def __init__(self, runtime, *, size, eps):
                self.runtime, self.size, self.eps, self.weight = runtime, size, eps, None

            def parameters(self):
                return {"weight": ParamInfo((self.size,), init="around_one", role="vector")}

            def assign(self, name, tensor):
                self.weight = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()

            def forward(self, x, residual):
                assert isinstance(x, torch.Tensor)      # never a deferred projection, never asked to be lazy
                return ops.add_rms_norm(x, residual, self.weight, self.eps)

    rt = _runtime(torch.bfloat16)
    hidden, inter = 96, 208
    cfg = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 1e-5, "hidden_size": hidden,
           "num_hidden_layers": 2}
    rope = POSITION_ENCODINGS.build("rope_neox", rt, dim=32, theta=1e4)
    blocks, w = [], {}
    for layer in range(2):
        attn = MIXERS.build("gqa_attention", rt, rope, hidden_size=hidden, num_heads=3, num_kv_heads=1, head_dim=32, scale=32 ** -0.5,
                            eps=1e-5)
        kind = "toy_unfused_rms" if (plain_norm_in_second_block and layer == 1) else "rms_norm"
        n1, n2 = NORMS.build(kind, rt, size=hidden, eps=1e-5), NORMS.build("rms_norm", rt, size=hidden, eps=1e-5)
        ff = FEED_FORWARDS.build("swiglu", rt, hidden_size=hidden, intermediate_size=inter)
        blocks.append(ARRANGEMENTS.build("pre_norm", attn, n1, ff, n2))
        for prefix, part, seed in ((f"model.layers.{layer}.self_attn.", attn, 10 * layer + 1), (f"model.layers.{layer}.input_layernorm.", n1, 10 * layer + 2),
                                   (f"model.layers.{layer}.mlp.", ff, 10 * layer + 3), (f"model.layers.{layer}.post_attention_layernorm.", n2, 10 * layer + 4)):
            # projections live in bfloat16 in the parts, norm weights in 32-bit
            w.update({prefix + k: (v if "layernorm" in prefix else v.bfloat16().float()).to(DEV) for k, v in _fill(part, seed, 0.15).items()})
    assert blocks[0].supports_deferred and blocks[0].accepts_deferred_input
    assert blocks[1].accepts_deferred_input != plain_norm_in_second_block
    rows = 5
    x = torch.randn(rows, hidden, device=DEV).bfloat16()

    def run(fold: bool):
        monkeypatch.setattr(ops, "FUSE_MAX_ROWS", 16 if fold else 0)
        seen = []
        real = ops.linear_add
        monkeypatch.setattr(ops, "linear_add", lambda *a, **k: (seen.append(1), real(*a, **k))[1])
        from oxr_inference_b200.cache import CacheManager, make_cache_plan
        from oxr_inference_b200.engine.batch import BatchBuilder, StepEntry
        plan = make_cache_plan([blk.mixer.cache_need() for blk in blocks], [None, None])
        manager = CacheManager(plan, page_size=8, num_pages=64, max_requests=8, device=rt.device, dtype=rt.dtype)
        builder = BatchBuilder(manager, blocks[0].mixer.tile_specs(), rt.device, rt.status)
        reqs = [manager.open(f"r{i}") for i in range(rows)]      # five requests of one token each: a decode step
        for r in reqs:
            assert manager.reserve(r, 1)
        ctx = builder.build([StepEntry(r, [0], []) for r in reqs])
        h, residual = x, None
        defer_first = blocks[1].accepts_deferred_input
        h, residual = blocks[0].forward(h, residual, ctx, manager.layer_cache(0, ctx), defer_output=defer_first)
        assert isinstance(h, DeferredLinear) == defer_first
        h, residual = blocks[1].forward(h, residual, ctx, manager.layer_cache(1, ctx))
        ops.check_status(rt.status)
        monkeypatch.setattr(ops, "linear_add", real)
        return h.float() + residual, len(seen)

    folded, n_folded = run(True)
    apart, n_apart = run(False)
    # every norm that follows a projection folds when it takes part: two inside the blocks, one between them
    assert n_folded == (2 if plain_norm_in_second_block else 3)
    assert n_apart == n_folded      # asked every time, refused (None) when switched off
    scale = apart.abs().max().item()
    assert (folded - apart).abs().max().item() <= 2e-2 * scale
    # each request is one token at position 0: the plain layers on a one-token sequence each
    cos, sin = QP.rope_tables(32, 1e4, 1, torch.float32)
    for i in range(rows):
        want = x[i:i + 1].float()
        for layer in range(2):
            want = QP.decoder_layer(want, w, layer, cfg, cos.to(DEV), sin.to(DEV))
        assert (folded[i:i + 1] - want).abs().max().item() <= 3e-2 * want.abs().max().item()


def test_embedding_and_head_parts_tied_and_untied():
    from oxr_inference_b200.parts.decoder import OutputHead, TokenEmbedding

    rt = _runtime()
    emb = TokenEmbedding(rt, vocab_size=50, hidden_size=24)
    table = _fill(emb)["weight"].to(DEV)
    ids = torch.tensor([0, 49, 7], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids), table[ids.long()])
    h = torch.randn(3, 24, device=DEV)
    tied = OutputHead(rt, emb, vocab_size=50, hidden_size=24, tied=True)
    assert tied.parameters() == {}
    torch.testing.assert_close(tied.forward(h), h @ table.T, atol=1e-5, rtol=1e-5)
    own = OutputHead(rt, emb, vocab_size=50, hidden_size=24, tied=False)
    w = _fill(own, seed=5)["weight"].to(DEV)
    torch.testing.assert_close(own.forward(h), h @ w.T, atol=1e-5, rtol=1e-5)


# ---------------------------------------------------------------------------------------------------------------
# A toy architecture, defined here: layer 0 is the built-in attention + feed-forward; layer 1 has a mixer that keeps
# a running sum of its inputs as per-request state; the schedule runs layer 0, layer 1, and layer 0 AGAIN, the
# second run reading the keys and values the first run stored. Nothing under oxr_inference_b200/ knows about it.
# ---------------------------------------------------------------------------------------------------------------
TOY = {"architectures": ["ToyScheduleForTests"], "hidden_size": 32, "intermediate_size": 48, "vocab_size": 50, "heads": 4,
       "kv_heads": 2, "head_dim": 16, "eps": 1e-5, "theta": 1e4, "max_positions": 128}


def _register_toy():
    from oxr_inference_b200.config.registry import ARCHITECTURES, Architecture, register_architecture
    from oxr_inference_b200.parts import MIXERS, LayerSpec, Mixer, ModelSpec, ParamInfo, PartSpec, ScheduleEntry, StateNeed

    if "toy_running_mean" not in MIXERS:
        @MIXERS.register("toy_running_mean")
        class RunningMean(Mixer):
            """y[t] = gain * mean of the inputs at positions 0..t of the same request. State: the sum so far."""

            def __init__(self, runtime, position, *, hidden_size):
                self.runtime, self.hidden, self.gain = runtime, hidden_size, None

            def parameters(self):
                return {"gain": ParamInfo((self.hidden,), init="around_one", role="vector")}

            def assign(self, name, tensor):
                assert name == "gain"
                self.gain = tensor.to(self.runtime.device, torch.float32)

            def cache_need(self):
                return StateNeed((self.hidden,), torch.float32)

            def forward(self, h, ctx, cache):
                # no host round trip (the step may be captured in a CUDA graph): a running sum over the packed tokens,
                # minus what the requests before this one brought, plus the request's sum so far from its state slot
                x = h.float()
                total = torch.cumsum(x, 0)
                cu, req = ctx.cu_q.long(), ctx.req_of_token.long()
                before = (total[cu[:-1]] - x[cu[:-1]])[req]
                slots = ctx.state_slots.long()
                run = cache.state[slots][req] + total - before
                cache.state.index_copy_(0, slots, run[cu[1:] - 1])
                return (run / (ctx.positions.float() + 1)[:, None] * self.gain).to(h.dtype)

    if "ToyScheduleForTests" not in ARCHITECTURES:
        def spec(c):
            norm = lambda p: PartSpec("rms_norm", {"size": c["hidden_size"], "eps": c["eps"]}, prefix=p)  # noqa: E731
            ff = lambda p: PartSpec("swiglu", {"hidden_size": c["hidden_size"], "intermediate_size": c["intermediate_size"]}, prefix=p)  # noqa: E731
            rope = PartSpec("rope_neox", {"dim": c["head_dim"], "theta": c["theta"]})
            attn = PartSpec("gqa_attention", {"hidden_size": c["hidden_size"], "num_heads": c["heads"], "num_kv_heads": c["kv_heads"],
                                              "head_dim": c["head_dim"], "scale": c["head_dim"] ** -0.5, "eps": c["eps"]},
                            prefix="model.layers.0.self_attn.")
            toy = PartSpec("toy_running_mean", {"hidden_size": c["hidden_size"]}, prefix="model.layers.1.mixer.")
            layers = (
                LayerSpec(attn, norm("model.layers.0.input_layernorm."), ff("model.layers.0.mlp."),
                          norm("model.layers.0.post_attention_layernorm."), position=rope),
                LayerSpec(toy, norm("model.layers.1.input_layernorm."), ff("model.layers.1.mlp."),
                          norm("model.layers.1.post_attention_layernorm.")),
            )
            return ModelSpec(
                architecture="ToyScheduleForTests", hidden_size=c["hidden_size"], vocab_size=c["vocab_size"],
                embedding=PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": c["hidden_size"]}, prefix="model.embed_tokens."),
                layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)),
                final_norm=norm("model.norm."),
                head=PartSpec("linear_head", {"vocab_size": c["vocab_size"], "hidden_size": c["hidden_size"], "tied": True}, prefix="lm_head."),
                max_positions=c["max_positions"])

        register_architecture(Architecture("ToyScheduleForTests", lambda raw, gen: dict(raw), spec))


def _toy_plain(w, ids):
    """The toy model on a whole sequence, written out with the plain implementation's functions."""
    c = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5}
    n, eps = len(ids), 1e-5
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    cos, sin = QP.rope_tables(16, 1e4, n, torch.float32)
    p = "model.layers.0."

    def qkv(h):
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(n, 4, 16)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(n, 2, 16)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, 2, 16)
        q = QP.rotate_half_split(QP.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps), cos, sin)
        k = QP.rotate_half_split(QP.rms_norm(k, w[p + "self_attn.k_norm.weight"], eps), cos, sin)
        return q, k, v

    def mlp(x, q):
        h = QP.rms_norm(x, w[q + "post_attention_layernorm.weight"], eps)
        return x + QP.swiglu(h, w[q + "mlp.gate_proj.weight"], w[q + "mlp.up_proj.weight"], w[q + "mlp.down_proj.weight"])

    # run 1 of layer 0
    q, k0, v0 = qkv(QP.rms_norm(x, w[p + "input_layernorm.weight"], eps))
    x = mlp(x + QP.causal_attention(q, k0, v0, 0.25).reshape(n, 64) @ w[p + "self_attn.o_proj.weight"].T, p)
    # layer 1: running mean
    h = QP.rms_norm(x, w["model.layers.1.input_layernorm.weight"], eps)
    mean = torch.cumsum(h, 0) / torch.arange(1, n + 1)[:, None]
    x = mlp(x + mean * w["model.layers.1.mixer.gain"], "model.layers.1.")
    # run 2 of layer 0: its own queries, the keys and values of run 1
    q, _, _ = qkv(QP.rms_norm(x, w[p + "input_layernorm.weight"], eps))
    x = mlp(x + QP.causal_attention(q, k0, v0, 0.25).reshape(n, 64) @ w[p + "self_attn.o_proj.weight"].T, p)
    return QP.rms_norm(x, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T


def test_a_toy_architecture_with_a_stateful_mixer_registers_builds_and_steps(tmp_path):
    from safetensors.torch import load_file

    from oxr_inference_b200.engine.batch import StepEntry
    from oxr_inference_b200.engine.runtime import ModelRunner
    from oxr_inference_b200.weights import write_random_model

    _register_toy()
    folder = write_random_model(TOY, tmp_path / "toy", seed=3, dtype="float32", std=0.15)
    w = load_file(str(folder / "model.safetensors"))
    assert "model.layers.1.mixer.gain" in w and "model.layers.1.self_attn.q_proj.weight" not in w
    runner = ModelRunner.from_folder(folder, dtype="float32", page_size=8, num_pages=32, max_requests=3)
    plan = runner.model.cache_plan
    assert len(plan.groups) == 1 and plan.groups[0].num_layers == 1, "the second run of layer 0 has no cache of its own"
    assert len(plan.states) == 1 and plan.entries[2].store is False and plan.entries[1].state == 0

    g = torch.Generator().manual_seed(5)
    seqs = {k: torch.randint(0, 50, (n,), generator=g).tolist() for k, n in (("a", 37), ("b", 20))}
    want = {k: _toy_plain(w, v) for k, v in seqs.items()}
    # request a in portions, request b beside it: a portion, then decoded tokens
    a, b = runner.cache.open("a"), runner.cache.open("b")
    got = {"a": [], "b": []}
    plan_a, plan_b = [5, 2, 11, 1, 18], [12, 1, 1, 1, 5]
    pa = pb = 0
    for ca, cb in zip(plan_a, plan_b):
        assert runner.cache.reserve(a, pa + ca) and runner.cache.reserve(b, pb + cb)
        logits = runner.step([StepEntry(a, seqs["a"][pa:pa + ca], list(range(ca))), StepEntry(b, seqs["b"][pb:pb + cb], list(range(cb)))])
        got["a"].append(logits[:ca])
        got["b"].append(logits[ca:])
        pa, pb = pa + ca, pb + cb
    runner.check()
    for k in seqs:
        torch.testing.assert_close(torch.cat(got[k]).cpu(), want[k], atol=1e-4, rtol=1e-4)
    # a new request on a used slot starts from zeroed state
    runner.cache.close(a)
    c = runner.cache.open("c")
    assert c.state_slot == a.state_slot and runner.cache.reserve(c, 37)
    again = runner.step([StepEntry(c, seqs["a"], list(range(37)))])
    torch.testing.assert_close(again.cpu(), want["a"], atol=1e-4, rtol=1e-4)


def test_the_toy_stateful_architecture_generates_through_the_engine_with_and_without_cuda_graphs(tmp_path):
    """The same toy model through ``Engine.generate``: with CUDA graphs a step whose bucket is captured for the first
    time must still advance each request's state once, not twice; with so few pages that requests are preempted, a
    recomputed request starts from zeroed state again. Greedy tokens equal the plain statement's either way."""
    from safetensors.torch import load_file

    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams
    from oxr_inference_b200.weights import write_random_model

    _register_toy()
    folder = write_random_model(TOY, tmp_path / "toy", seed=3, dtype="float32", std=0.15)
    w = load_file(str(folder / "model.safetensors"))
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 50, (n,), generator=g).tolist() for n in (3, 17, 9, 30, 1)]
    new = 24

    def plain_greedy(ids):
        ids, out = list(ids), []
        for _ in range(new):
            out.append(int(_toy_plain(w, ids)[-1].argmax()))
            ids.append(out[-1])
        return out

    want = [plain_greedy(p) for p in prompts]
    for graphs, pages in ((True, 64), (False, 64), (True, 14)):
        engine = Engine(folder, EngineSettings(dtype="float32", page_size=8, num_pages=pages, max_running=4, cuda_graphs=graphs,
                                               max_step_tokens=64, prefill_chunk=16))
        got = engine.generate(prompts, SamplingParams(max_tokens=new, ignore_eos=True))
        assert [c.token_ids for c in got] == want, f"cuda_graphs={graphs}, {pages} pages"
        assert (engine.counters["graph_steps"] > 0) == graphs
        if pages == 14:
            assert engine.preemptions > 0, "the small pool was meant to force a preemption"
        engine.runner.cache.check()


# ---------------------------------------------------------------------------------------------------------------
# A second toy architecture, also defined here: layer 0 is the built-in attention (no q/k norm) under a position
# encoding of its own (angles that grow linearly in the pair index) with a feed-forward that ROUTES each token to two
# of four small experts; layer 1 is the built-in attention with NO position encoding and a window, with the built-in
# feed-forward; the embedding is scaled by a constant and the head, untied, adds a bias (both defined here). Parts are
# chosen layer by layer; nothing under oxr_inference_b200/ knows them.
# ---------------------------------------------------------------------------------------------------------------
TOY2 = {"architectures": ["ToyRoutedForTests"], "hidden_size": 48, "intermediate_size": 40, "vocab_size": 61, "heads": 6,
        "kv_heads": 3, "head_dim": 16, "eps": 1e-6, "experts": 4, "expert_size": 24, "window": 6, "max_positions": 96,
        "embedding_scale": 3.0}


def _register_toy2():
    from oxr_inference_b200.config.registry import ARCHITECTURES, Architecture, register_architecture
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts import (EMBEDDINGS, FEED_FORWARDS, HEADS, POSITION_ENCODINGS, Embedding, FeedForward, Head, LayerSpec,
                                          ModelSpec, ParamInfo, PartSpec, PositionEncoding, ScheduleEntry)

    if "toy_scaled_embedding" not in EMBEDDINGS:
        @EMBEDDINGS.register("toy_scaled_embedding")
        class ScaledEmbedding(Embedding):
            """x = scale * table[ids]"""

            def __init__(self, runtime, *, vocab_size, hidden_size, scale):
                self.runtime, self.shape, self.scale, self.weight = runtime, (vocab_size, hidden_size), scale, None

            def parameters(self):
                return {"weight": ParamInfo(self.shape)}

            def assign(self, name, tensor):
                self.weight = tensor.to(self.runtime.device, self.runtime.store_dtype(self.parameters()[name], tensor.dtype))

            def forward(self, ids):
                return (self.weight[ids.long()].float() * self.scale).to(self.runtime.dtype)

    if "toy_biased_head" not in HEADS:
        @HEADS.register("toy_biased_head")
        class BiasedHead(Head):
            """logits = h W^T + b, with a matrix of its own"""

            def __init__(self, runtime, embedding, *, vocab_size, hidden_size):
                self.runtime, self.v, self.h, self.w = runtime, vocab_size, hidden_size, {}

            def parameters(self):
                return {"weight": ParamInfo((self.v, self.h)), "bias": ParamInfo((self.v,), role="vector")}

            def assign(self, name, tensor):
                self.w[name] = tensor.to(self.runtime.device, self.runtime.store_dtype(self.parameters()[name], tensor.dtype)).contiguous()

            def forward(self, h):
                return ops.linear(h, self.w["weight"], torch.float32) + self.w["bias"]

    if "toy_linear_angles" not in POSITION_ENCODINGS:
        @POSITION_ENCODINGS.register("toy_linear_angles")
        class LinearAngles(PositionEncoding):
            """Pair j of a head turns by position * (j + 1) / 7 radians: the same rotation kernel, another table."""

            def __init__(self, runtime, *, dim):
                angles = torch.outer(torch.arange(runtime.max_positions, dtype=torch.float), (torch.arange(dim // 2, dtype=torch.float) + 1) / 7)
                self.cos, self.sin = angles.cos().to(runtime.device), angles.sin().to(runtime.device)

            def tables(self):
                return self.cos, self.sin

    if "toy_top2_experts" not in FEED_FORWARDS:
        @FEED_FORWARDS.register("toy_top2_experts")
        class Top2Experts(FeedForward):
            """Router logits in fp32 -> softmax -> the two largest, renormalised -> sum of p * W_out[e] relu(W_in[e] h)."""

            def __init__(self, runtime, *, hidden_size, experts, expert_size):
                self.runtime, self.h, self.e, self.i = runtime, hidden_size, experts, expert_size
                self.w = {}

            def parameters(self):
                return {"router.weight": ParamInfo((self.e, self.h), role="vector"),
                        "w_in": ParamInfo((self.e, self.i, self.h)), "w_out": ParamInfo((self.e, self.h, self.i))}

            def assign(self, name, tensor):
                info = self.parameters()[name]
                self.w[name] = tensor.to(self.runtime.device, self.runtime.store_dtype(info, tensor.dtype))

            def forward(self, h):
                p = torch.softmax(h.float() @ self.w["router.weight"].float().T, -1)
                top, idx = p.topk(2, -1)
                top = top / top.sum(-1, keepdim=True)
                out = torch.zeros_like(h, dtype=torch.float32)
                for e in range(self.e):
                    rows, slot = (idx == e).nonzero(as_tuple=True)
                    if rows.numel():
                        x = h[rows].float()
                        y = torch.relu(x @ self.w["w_in"][e].float().T) @ self.w["w_out"][e].float().T
                        out.index_add_(0, rows, y * top[rows, slot][:, None])
                return out.to(h.dtype)

    if "ToyRoutedForTests" not in ARCHITECTURES:
        def spec(c):
            H = c["hidden_size"]
            norm = lambda p: PartSpec("rms_norm", {"size": H, "eps": c["eps"]}, prefix=p)  # noqa: E731

            def attn(i, **more):
                return PartSpec("gqa_attention", {"hidden_size": H, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"], "head_dim": c["head_dim"],
                                                  "scale": c["head_dim"] ** -0.5, "eps": c["eps"], **more}, prefix=f"model.layers.{i}.self_attn.")
            layers = (
                LayerSpec(attn(0, qk_norm=False), norm("model.layers.0.input_layernorm."),
                          PartSpec("toy_top2_experts", {"hidden_size": H, "experts": c["experts"], "expert_size": c["expert_size"]}, prefix="model.layers.0.moe."),
                          norm("model.layers.0.post_attention_layernorm."), position=PartSpec("toy_linear_angles", {"dim": c["head_dim"]})),
                LayerSpec(attn(1, window=c["window"]), norm("model.layers.1.input_layernorm."),
                          PartSpec("swiglu", {"hidden_size": H, "intermediate_size": c["intermediate_size"]}, prefix="model.layers.1.mlp."),
                          norm("model.layers.1.post_attention_layernorm."), position=None),
            )
            return ModelSpec(
                architecture="ToyRoutedForTests", hidden_size=H, vocab_size=c["vocab_size"],
                embedding=PartSpec("toy_scaled_embedding", {"vocab_size": c["vocab_size"], "hidden_size": H, "scale": c["embedding_scale"]},
                                   prefix="model.embed_tokens."),
                layers=layers, schedule=(ScheduleEntry(0), ScheduleEntry(1)), final_norm=norm("model.norm."),
                head=PartSpec("toy_biased_head", {"vocab_size": c["vocab_size"], "hidden_size": H}, prefix="lm_head."),
                max_positions=c["max_positions"])

        register_architecture(Architecture("ToyRoutedForTests", lambda raw, gen: dict(raw), spec))


def _toy2_plain(w, ids):
    c, n, eps = TOY2, len(ids), TOY2["eps"]
    H, KV, D = c["heads"], c["kv_heads"], c["head_dim"]
    x = c["embedding_scale"] * w["model.embed_tokens.weight"][torch.tensor(ids)]
    angles = torch.outer(torch.arange(n, dtype=torch.float), (torch.arange(D // 2, dtype=torch.float) + 1) / 7)
    for layer in (0, 1):
        p = f"model.layers.{layer}."
        h = QP.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(n, H, D)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(n, KV, D)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, KV, D)
        if layer == 0:   # no q/k norm, linear angles
            q, k = QP.rotate_half_split(q, angles.cos(), angles.sin()), QP.rotate_half_split(k, angles.cos(), angles.sin())
            a = QP.causal_attention(q, k, v, D ** -0.5)
        else:            # q/k norm, no rotation, window
            q, k = QP.rms_norm(q, w[p + "self_attn.q_norm.weight"], eps), QP.rms_norm(k, w[p + "self_attn.k_norm.weight"], eps)
            a = QP.causal_attention(q, k, v, D ** -0.5, window=c["window"])
        x = x + a.reshape(n, H * D) @ w[p + "self_attn.o_proj.weight"].T
        h = QP.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        if layer == 0:
            prob = torch.softmax(h @ w[p + "moe.router.weight"].T, -1)
            top, idx = prob.topk(2, -1)
            top = top / top.sum(-1, keepdim=True)
            y = torch.zeros_like(h)
            for t in range(n):
                for j in range(2):
                    e = int(idx[t, j])
                    y[t] += top[t, j] * (torch.relu(h[t] @ w[p + "moe.w_in"][e].T) @ w[p + "moe.w_out"][e].T)
            x = x + y
        else:
            x = x + QP.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return QP.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T + w["lm_head.bias"]


def test_a_toy_architecture_with_routed_experts_and_its_own_position_encoding(tmp_path):
    from safetensors.torch import load_file

    from oxr_inference_b200.engine.batch import StepEntry
    from oxr_inference_b200.engine.runtime import ModelRunner
    from oxr_inference_b200.weights import write_random_model

    _register_toy2()
    folder = write_random_model(TOY2, tmp_path / "toy2", seed=4, dtype="float32", std=0.2)
    w = load_file(str(folder / "model.safetensors"))
    assert w["model.layers.0.moe.w_in"].shape == (4, 24, 48) and "model.layers.0.self_attn.q_norm.weight" not in w
    assert "model.layers.1.self_attn.q_norm.weight" in w and "lm_head.weight" in w and w["lm_head.bias"].shape == (61,)
    runner = ModelRunner.from_folder(folder, dtype="float32", page_size=8, num_pages=24, max_requests=2)
    plan = runner.model.cache_plan
    assert len(plan.groups) == 2, "a layer that keeps all keys and a layer with a window have pools of their own"

    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, TOY2["vocab_size"], (45,), generator=g).tolist()
    want = _toy2_plain(w, ids)
    # the routing must actually vary, or the test would not see a wrong expert
    x0 = TOY2["embedding_scale"] * w["model.embed_tokens.weight"][torch.tensor(ids)]
    h0 = QP.rms_norm(x0, w["model.layers.0.input_layernorm.weight"], TOY2["eps"])
    assert len({int(i) for i in (h0 @ w["model.layers.0.moe.router.weight"].T).argmax(-1)}) >= 3
    rc = runner.cache.open("r")
    got, pos = [], 0
    for c in (17, 2, 9, 1, 1, 15):
        assert runner.cache.reserve(rc, pos + c)
        got.append(runner.step([StepEntry(rc, ids[pos:pos + c], list(range(c)))]))
        pos += c
    runner.check()
    torch.testing.assert_close(torch.cat(got).cpu(), want, atol=1e-4, rtol=1e-4)
    # the window's pages were given back as it passed them
    assert sum(p == -1 for p in rc.tables[1]) >= 3 and all(p != -1 for p in rc.tables[0])
