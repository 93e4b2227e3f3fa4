"""Generation through the Python entry point on the GPU: greedy against the plain implementation, CUDA-graph
replay against eager steps, temperature sampling that does not depend on batching or preemption, repetition
penalty, and the command line."""

import json
import subprocess
import sys

import pytest
import torch

import util
from plain import qwen3_plain as QP
from util import make_folder, plain_logits, token_ids

pytestmark = pytest.mark.gpu


def _engine(folder, name, dtype, **kw):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine

    kw.setdefault("num_pages", 64)
    kw.setdefault("max_running", 4)
    return Engine(folder, EngineSettings(dtype=dtype, page_size=util.PAGE[name], **kw))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("engine")
    return {name: make_folder(tmp, name, seed=11) for name in ("A", "B")}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_float32_is_the_plain_implementations(folders, name, graphs):
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders[name]
    cfg, w = QP.read_model(folder)
    prompts = [token_ids(name, n, seed=21) for n in ((5, 17, 33) if name == "A" else (1, 12, 40, 64))]
    steps = 8 if name == "A" else 12
    want = [QP.greedy(cfg, w, p, steps) for p in prompts]
    engine = _engine(folder, name, "float32", cuda_graphs=graphs)
    got = engine.generate(prompts, SamplingParams(max_tokens=steps, ignore_eos=True))
    assert [c.token_ids for c in got] == want
    assert all(c.finish_reason == "length" and c.prompt_tokens == len(p) for c, p in zip(got, prompts))
    assert (engine.counters["graph_steps"] > 0) == graphs
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages == engine.runner.cache.usable_pages


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_picks_near_maxima_of_the_plain_logits(folders, name):
    """bfloat16 may break a near-tie the other way; every token it picks must still be within twice the largest
    bfloat16 error seen on these models (2.4e-2 of the logits' scale, on both logits of a near-tie) of the plain
    implementation's maximum, given the engine's own earlier tokens."""
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders[name]
    prompts = [token_ids(name, n, seed=22) for n in (7, 30, 61)]
    engine = _engine(folder, name, "bfloat16")
    got = engine.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    for prompt, c in zip(prompts, got):
        seq = prompt + c.token_ids
        logits = plain_logits(folder, seq[:-1])
        scale = logits.abs().max().item()
        for i, tok in enumerate(c.token_ids):
            row = logits[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - 2 * 2.5e-2 * scale, f"token {i} = {tok} is not near the plain maximum"


def test_requests_of_very_different_lengths_decode_with_the_even_cut(tmp_path, monkeypatch):
    """Head size 64 and pages of 8 tokens (TMA gathers), one layer with a window: four requests of 6 to 900 tokens decode
    together. The engine notices that their lengths differ much, keys its CUDA graph by that, and the split-KV kernel deals
    all key blocks out evenly instead of cutting every request alike; the tokens lie near the plain maxima, with graphs and
    without, and a batch of requests of one length keeps the equal pieces."""
    from oxr_inference_b200 import ops
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams

    monkeypatch.setattr(ops, "DECODE_CUT", "auto")     # the default: the engine decides (an environment variable may say otherwise)
    name = "uneven64"
    util.CONFIGS[name] = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 128, "intermediate_size": 96,
                          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "rms_norm_eps": 1e-6,
                          "rope_theta": 1e4, "vocab_size": 300, "tie_word_embeddings": False, "max_position_embeddings": 1024,
                          "eos_token_id": 299, "use_sliding_window": True, "sliding_window": 400,
                          "layer_types": ["full_attention", "sliding_attention"]}
    try:
        folder = make_folder(tmp_path, name, seed=5)
        prompts = [token_ids(name, n, seed=31) for n in (6, 900, 40, 333)]
        same = [token_ids(name, 200, seed=32 + i) for i in range(4)]
    finally:
        del util.CONFIGS[name]
    for graphs in (True, False):
        engine = Engine(folder, EngineSettings(dtype="bfloat16", page_size=8, num_pages=400, max_running=4, cuda_graphs=graphs,
                                               max_step_tokens=2048))
        got = engine.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
        assert ops.last_short_attention_kernel(64) == "attn_tma_decode_walk_kernel (one round)"
        if graphs:
            assert engine.graphs.last_key[2] is True
        for prompt, c in zip(prompts, got):
            seq = prompt + c.token_ids
            logits = plain_logits(folder, seq[:-1])
            scale = logits.abs().max().item()
            for i, tok in enumerate(c.token_ids):
                row = logits[len(prompt) - 1 + i]
                assert row[tok] >= row.max() - 2 * 2.5e-2 * scale, f"token {i} = {tok} is not near the plain maximum"
        engine.generate(same, SamplingParams(max_tokens=4, ignore_eos=True))
        assert ops.last_short_attention_kernel(64) == "attn_tma_decode_kernel"
        if graphs:
            assert engine.graphs.last_key[2] is False
        engine.runner.cache.check()


def test_cuda_graph_replay_equals_eager_steps(folders):
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders["B"]
    prompts = [token_ids("B", n, seed=23) for n in (3, 20, 50)]
    runs = []
    for graphs in (False, True):
        engine = _engine(folder, "B", "bfloat16", cuda_graphs=graphs)
        runs.append([c.token_ids for c in engine.generate(prompts, SamplingParams(max_tokens=40, ignore_eos=True))])
    assert runs[0] == runs[1]


def test_temperature_sampling_does_not_depend_on_batching_or_preemption(folders):
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders["B"]
    prompts = [token_ids("B", n, seed=24) for n in (1, 12, 40, 64)]
    params = [SamplingParams(max_tokens=12, temperature=0.7, seed=1000 + i, ignore_eos=True) for i in range(4)]
    together = _engine(folder, "B", "float32").generate(prompts, params)
    alone = [_engine(folder, "B", "float32", cuda_graphs=False).generate([p], [q])[0] for p, q in zip(prompts, params)]
    assert [c.token_ids for c in together] == [c.token_ids for c in alone]
    greedy = _engine(folder, "B", "float32").generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert [c.token_ids for c in greedy] != [c.token_ids for c in together], "temperature 0.7 should not equal greedy everywhere"
    # so few pages that requests are pushed out and recomputed: the draws must come out the same
    squeezed = _engine(folder, "B", "float32", num_pages=15, max_step_tokens=24, prefill_chunk=9)
    again = squeezed.generate(prompts, params)
    assert squeezed.preemptions > 0, "this cache is too small to run the four requests without preemption"
    assert [c.token_ids for c in again] == [c.token_ids for c in together]
    # another seed, other tokens
    other = _engine(folder, "B", "float32").generate(prompts[3:], [SamplingParams(max_tokens=12, temperature=0.7, seed=5, ignore_eos=True)])
    assert other[0].token_ids != together[3].token_ids


def test_chunked_prefill_under_a_small_token_budget_gives_the_same_tokens(folders):
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders["A"]
    cfg, w = QP.read_model(folder)
    prompts = [token_ids("A", n, seed=25) for n in (5, 17, 33, 90)]
    want = [QP.greedy(cfg, w, p, 8) for p in prompts]
    engine = _engine(folder, "A", "float32", max_step_tokens=11, prefill_chunk=7, num_pages=20)
    got = engine.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [c.token_ids for c in got] == want


def test_eos_stops_generation(folders):
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders["A"]
    cfg, w = QP.read_model(folder)
    prompt = token_ids("A", 9, seed=26)
    free_run = QP.greedy(cfg, w, prompt, 6)
    cut = max(i for i in range(6) if free_run[i] not in free_run[:i])  # the last token that is new when it appears
    engine = _engine(folder, "A", "float32")
    stopped = engine.generate([prompt], SamplingParams(max_tokens=6, stop_token_ids=(free_run[cut],)))[0]
    assert stopped.token_ids == free_run[:cut] and stopped.finish_reason == "stop"


def test_repetition_penalty_follows_the_reference_rule(folders):
    """Greedy with a penalty: recompute with the plain implementation, dividing positive and multiplying other
    logits of every token seen so far, prompt included (oxr_runtime/engine.py:632-639)."""
    from oxr_inference_b200.sampling import SamplingParams

    folder = folders["A"]
    cfg, w = QP.read_model(folder)
    prompt = token_ids("A", 12, seed=27)
    seq, want = list(prompt), []
    for _ in range(8):
        row = QP.logits(cfg, w, seq)[-1].clone()
        seen = torch.tensor(sorted(set(seq)))
        row[seen] = torch.where(row[seen] > 0, row[seen] / 1.8, row[seen] * 1.8)
        want.append(int(row.argmax()))
        seq.append(want[-1])
    engine = _engine(folder, "A", "float32")
    got = engine.generate([prompt], SamplingParams(max_tokens=8, repetition_penalty=1.8, ignore_eos=True))[0]
    assert got.token_ids == want
    assert want != QP.greedy(cfg, w, prompt, 8), "this prompt and penalty were chosen so that the penalty changes the tokens"


def test_step_failure_is_loud_and_pages_come_back(folders):
    from oxr_inference_b200.sampling import SamplingParams
    from oxr_inference_b200 import ops

    engine = _engine(folders["A"], "A", "float32", cuda_graphs=False)
    engine.add_request([5, 999999], SamplingParams(max_tokens=2))  # a token id outside the vocabulary
    with pytest.raises(ops.KernelError, match="vocabulary"):
        engine.step()
    assert not engine.has_work() and engine.runner.cache.free_pages == engine.runner.cache.usable_pages
    ok = engine.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))
    assert len(ok[0].token_ids) == 2, "the engine stays usable after a failed step"


def test_done_callback_and_cancel(folders):
    """A request's ``done`` callback gets its completion in the step in which it ends; ``cancel()`` ends a running request
    at the next step, gives its pages back and leaves the others' tokens as they would have been."""
    from oxr_inference_b200.sampling import SamplingParams

    engine = _engine(folders["A"], "A", "float32")
    alone = engine.generate([token_ids("A", 9, seed=4)], SamplingParams(max_tokens=12, ignore_eos=True))[0]
    seen = []
    keep = engine.add_request(token_ids("A", 9, seed=4), SamplingParams(max_tokens=12, ignore_eos=True), done=seen.append)
    drop = engine.add_request(token_ids("A", 30, seed=5), SamplingParams(max_tokens=50, ignore_eos=True), done=seen.append)
    for _ in range(4):
        engine.step()
    assert not seen and len(drop.output) >= 2
    drop.cancel()
    while engine.has_work():
        engine.step()
    assert [c.request_id for c in seen] == [drop.id, keep.id]
    assert seen[0].finish_reason == "cancelled" and seen[1].finish_reason == "length"
    assert seen[1].token_ids == alone.token_ids
    engine.runner.check()
    assert not engine.runner.cache.open_requests()


def test_command_line(folders, tmp_path):
    folder = folders["A"]
    cfg, w = QP.read_model(folder)
    out = tmp_path / "result.json"
    cmd = [sys.executable, "-m", "oxr_inference_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6",
           "--max-tokens", "5", "--dtype", "float32", "--num-pages", "32", "--max-running", "4", "--ignore-eos", "--out", str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(util.ROOT), timeout=600)
    assert res.returncode == 0, res.stderr
    rows = [json.loads(line) for line in res.stdout.strip().splitlines()]
    assert [r["token_ids"] for r in rows] == [QP.greedy(cfg, w, [5, 17, 3], 5), QP.greedy(cfg, w, [9, 8, 7, 6], 5)]
    assert json.loads(out.read_text())["results"][0]["finish_reason"] == "length"


def test_text_goes_in_and_out_through_the_tokenizer_of_the_model_folder(folders, tmp_path):
    """With a ``tokenizer.json`` beside the weights a prompt may be text and the completion carries text
    (oxr_runtime/prompt.py:26-38 loads the folder's tokenizer the same way); without one, text is refused."""
    import shutil

    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    from oxr_inference_b200.sampling import SamplingParams

    folder = tmp_path / "with_tokenizer"
    shutil.copytree(folders["A"], folder)
    words = ["<unk>", "the", "page", "reads", "a", "table", "of", "rows", "and", "columns", "total", "sum"]
    vocab = {word: 20 + 3 * i for i, word in enumerate(words)}       # ids inside the model's 256, not 0..n
    tok = Tokenizer(WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    cfg, w = QP.read_model(folder)
    text = "the page reads a table of rows"
    ids = [vocab[x] for x in text.split()]
    engine = _engine(folder, "A", "float32")
    assert engine.tokenizer is not None
    by_text, by_ids = engine.generate([text, ids], SamplingParams(max_tokens=6, ignore_eos=True))
    want = QP.greedy(cfg, w, ids, 6)
    assert by_text.token_ids == want and by_ids.token_ids == want and by_text.prompt_tokens == len(ids)
    known = {i: word for word, i in vocab.items()}
    assert by_text.text == " ".join(known[t] for t in want if t in known)   # ids without a word decode to nothing
    plain = _engine(folders["A"], "A", "float32")
    assert plain.tokenizer is None and plain.generate([ids], SamplingParams(max_tokens=2, ignore_eos=True))[0].text is None
    with pytest.raises(ValueError, match="tokenizer.json"):
        plain.add_request(text)


def test_per_stage_timers_and_the_step_log(folders):
    """With ``profile=True`` the engine keeps cumulative seconds and counts per stage and one record per step, as the
    reference does under OXR_PROFILE=1 (oxr_runtime/engine.py:65-104); without it nothing is recorded."""
    from oxr_inference_b200.sampling import SamplingParams

    prompts = [token_ids("A", n, seed=31) for n in (3, 40)]
    engine = _engine(folders["A"], "A", "bfloat16", profile=True)
    engine.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    summary, steps = engine.profile.summary(), engine.profile.steps
    assert {"schedule", "build", "wait", "commit", "forward", "decode_graph"} <= set(summary)
    assert len(steps) == engine.counters["steps"] and sum(st["tokens"] for st in steps) == engine.counters["step_tokens"]
    assert sum(st["graph"] for st in steps) == engine.counters["graph_steps"] > 0
    assert all(st["ms"] > 0 for st in steps) and steps[-1]["held"] > 40
    assert summary["decode_graph"]["n"] + summary["forward"]["n"] == engine.counters["step_tokens"]
    quiet = _engine(folders["A"], "A", "bfloat16")
    quiet.generate(prompts, SamplingParams(max_tokens=3, ignore_eos=True))
    assert quiet.profile.summary() == {} and quiet.profile.steps == []


def test_smoke_entry():
    import __graft_entry__

    __graft_entry__.smoke()


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "float32")])
def test_many_random_requests_under_page_pressure_equal_plain_greedy(folders, name, dtype):
    """Forty requests of random lengths through a cache that holds only a few of them at a time, with a small token
    budget: admission, portions, decoding in and out of CUDA graphs, growth, preemption and recomputation, release and
    reuse of pages and state slots all happen many times; every request must still produce exactly the plain
    implementation's greedy tokens."""
    import random

    from oxr_inference_b200.sampling import SamplingParams

    folder = folders[name]
    cfg, w = QP.read_model(folder)
    rng = random.Random(5)
    prompts = [token_ids(name, rng.choice([1, 2, 5, 9, 17, 33, 60, 90]), seed=100 + i) for i in range(40)]
    steps = [rng.choice([1, 3, 8, 20]) for _ in prompts]
    engine = _engine(folder, name, dtype, num_pages=12 if name == "A" else 22, max_running=5, max_step_tokens=40, prefill_chunk=24)
    params = [SamplingParams(max_tokens=n, ignore_eos=True) for n in steps]
    got = engine.generate(prompts, params)
    assert engine.preemptions > 0, "the cache is meant to be too small for this workload"
    assert engine.counters["graph_steps"] > 0
    cache = {}
    for p, n, c in zip(prompts, steps, got):
        key = (tuple(p), n)
        if key not in cache:
            cache[key] = QP.greedy(cfg, w, p, n)
        assert c.token_ids == cache[key] and c.finish_reason == "length"
    engine.runner.cache.check()
    assert engine.runner.cache.free_pages == engine.runner.cache.usable_pages and engine.runner.cache.free_slots == 5
