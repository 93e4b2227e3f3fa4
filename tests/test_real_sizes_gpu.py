"""The engine at Qwen3-8B's layer sizes (hidden 4096, 32 query and 8 KV heads of 128, feed-forward 12288, vocabulary
151,936, untied head, pages of 16 tokens) against the plain implementation run in fp32 on the same device with the
same weights: in 32-bit at the full depth of 36 layers, in bfloat16 with four layers; several requests under every way
of cutting the work, with so few pages that they are used again; and generation of many requests through the entry
point with CUDA graphs. The reference checks its fused path the same way, against a plain fp32 statement of the model
(tests/test_language_fused.py:144-160, 250-278), at a tiny size only.

Weights are random (drawn on the device, bf16-rounded, the same draws for both sides); the q/k head-norm weights are
scaled up so that attention is peaked and a lost, doubled or misplaced key would show.
"""

import pytest
import torch

import util
from plain import qwen3_plain as QP

pytestmark = pytest.mark.gpu

SHARPEN = 2.0


def _config(layers):
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": layers,
            "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "vocab_size": 151936, "tie_word_embeddings": False, "max_position_embeddings": 4096}


def _plain_weights(model, seed):
    """The draws ``fill_random`` made (same seed, names, device), as fp32 tensors for the plain implementation."""
    from oxr_inference_b200.weights import random_tensor

    w = {}
    for name, (_, _, info) in model.named_parameters().items():
        t = random_tensor(name, info, seed, std=0.02, norm_std=0.1, device="cuda", dtype=torch.bfloat16).float()
        if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
            t = t * SHARPEN ** 0.5
        w[name] = t
    return w


def _sharpen(model):
    for block in model.blocks:
        block.mixer.q_norm.mul_(SHARPEN ** 0.5)
        block.mixer.k_norm.mul_(SHARPEN ** 0.5)


def _run_trace(runner, steps, seqs, want, dtype, what):
    """``steps``: lists of (request, tokens in this step, offsets inside them whose logits are compared, ends after it).
    Requests are opened at their first step; pages are reserved as ``bin/trace_run`` does."""
    from oxr_inference_b200.engine.batch import StepEntry

    live, pos = {}, {}
    for n, step in enumerate(steps):
        entries, rows, ended = [], [], []
        for key, count, wanted, end in step:
            if key not in live:
                live[key] = runner.cache.open(key)
                pos[key] = 0
                assert live[key] is not None
            rc, p = live[key], pos[key]
            assert runner.cache.reserve(rc, p + count), f"{what} step {n}: no pages left for {key}"
            entries.append(StepEntry(rc, seqs[key][p:p + count], list(wanted)))
            rows.append((key, [p + o for o in wanted]))
            pos[key] = p + count
            if end:
                ended.append(key)
        got = runner.step(entries)
        r = 0
        for key, places in rows:
            if places:
                util.compare(got[r:r + len(places)], want[key][places], dtype, f"{what} step {n}: request {key} positions {places}")
                r += len(places)
        assert r == got.shape[0]
        for key in ended:
            runner.cache.close(live.pop(key))
    runner.check()
    assert not live, f"{what}: requests left open: {sorted(live)}"
    runner.cache.check()


def _cuttings(lengths):
    """The four cuttings for requests ``r0, r1, ...`` of the given lengths."""
    keys = [f"r{i}" for i in range(len(lengths))]
    whole = [[(k, n, [0, n // 2, n - 1], True)] for k, n in zip(keys, lengths)]
    decoded = []
    for k, n in zip(keys, lengths):
        head = n - 32
        decoded.append([(k, head, [head - 1], False)])
        decoded += [[(k, 1, [0], p == n - 1)] for p in range(head, n)]
    portions = []
    sizes = [7, 2, 61, 3, 2, 31, 1, 16, 2, 129, 8, 40]
    for k, n in zip(keys, lengths):
        p, i = 0, 0
        while p < n:
            c = min(sizes[i % len(sizes)], n - p)
            portions.append([(k, c, [0, c - 1] if c > 1 else [0], p + c == n)])
            p, i = p + c, i + 1
    # mixed: every request live at once; each step gives some a portion, the others a decoded token, one sits out
    mixed, p = [], {k: 0 for k in keys}
    chunk = {k: s for k, s in zip(keys, (70, 33, 150, 9, 64))}
    n_step = 0
    while any(p[k] < n for k, n in zip(keys, lengths)):
        step = []
        for j, (k, n) in enumerate(zip(keys, lengths)):
            if p[k] >= n or (n_step + j) % 4 == 3:
                continue
            c = 1 if p[k] >= n - 24 else min(chunk[k], n - 24 - p[k])
            step.append((k, c, [c - 1], p[k] + c == n))
            p[k] += c
        if step:
            mixed.append(step)
        n_step += 1
    return {"whole": whole, "most, then 32 one by one": decoded, "portions": portions, "mixed": mixed}


@pytest.mark.parametrize("dtype,layers", [("float32", 36), ("bfloat16", 4)])
def test_every_cutting_at_qwen3_8b_sizes(dtype, layers):
    from oxr_inference_b200.engine.runtime import ModelRunner

    cfg = _config(layers)
    torch.backends.cuda.matmul.allow_tf32 = False
    lengths = [300, 77, 190]
    # 44 pages of 16 tokens: one more than the three requests need together (19 + 5 + 12, and the scratch page), so
    # that every cutting runs on pages the cutting before it gave back
    runner = ModelRunner.from_config(cfg, seed=5, dtype=dtype, page_size=16, num_pages=44, max_requests=4)
    _sharpen(runner.model)
    w = _plain_weights(runner.model, 5)
    g = torch.Generator().manual_seed(8)
    seqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    want = {k: QP.logits(cfg, w, ids).cpu() for k, ids in seqs.items()}
    del w
    torch.cuda.empty_cache()
    for what, steps in _cuttings(lengths).items():
        _run_trace(runner, steps, seqs, want, dtype, f"{dtype}, {layers} layers, {what}")
    assert runner.cache.free_pages == runner.cache.usable_pages


def test_generation_of_many_requests_at_qwen3_8b_sizes_with_cuda_graphs_is_plain_greedy():
    """Seventy requests (twelve at a time) through ``Engine.generate`` in 32-bit with four layers of Qwen3-8B's sizes: the scheduler, prompt
    portions beside decoding, CUDA graphs with padding rows at head size 128 and the 151,936-wide head inside the graph,
    pages given back and used again, a pool too small for all of them at once. Every request's tokens equal the plain
    implementation's greedy tokens."""
    import random

    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams

    cfg = _config(4)
    torch.backends.cuda.matmul.allow_tf32 = False
    engine = Engine(random_config=cfg, seed=6, settings=EngineSettings(
        dtype="float32", page_size=16, num_pages=20, max_running=12, max_step_tokens=256, prefill_chunk=96, cuda_graphs=True))
    _sharpen(engine.runner.model)
    w = _plain_weights(engine.runner.model, 6)
    rng = random.Random(3)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.choice([1, 2, 7, 16, 17, 40, 100]))] for _ in range(70)]
    steps = [rng.choice([1, 2, 5, 9, 40, 70]) for _ in prompts]   # the long ones grow by pages that may not be there
    got = engine.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True) for n in steps])
    assert engine.counters["graph_steps"] > 0 and engine.preemptions > 0

    def plain_greedy(prompt, n):   # QP.greedy with the head on the last position only
        ids, out = list(prompt), []
        for _ in range(n):
            out.append(int((QP.hidden_states(cfg, w, ids)[-1] @ w["lm_head.weight"].T).argmax()))
            ids.append(out[-1])
        return out

    for i, (p, n, c) in enumerate(zip(prompts, steps, got)):
        assert c.token_ids == plain_greedy(p, n), f"request {i} (prompt of {len(p)}, {n} new tokens)"
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages == engine.runner.cache.usable_pages
