"""Trace replay on the GPU against the plain implementation: every way of cutting the same requests.

Each (configuration, dtype) pair gets one ``bin/trace_run`` process; the tests feed it steps and compare the
logits files with whole-sequence logits of ``tests/plain/qwen3_plain.py``.
"""

import pytest

import util
from util import Replay, compare, make_folder, plain_logits, token_ids

pytestmark = pytest.mark.gpu

CASES = [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")]
LENGTHS = {"A": [5, 17, 33, 100], "B": [1, 12, 40, 64, 131]}


@pytest.fixture(scope="module", params=CASES, ids=lambda c: f"{c[0]}-{c[1]}")
def replay(request, tmp_path_factory):
    name, dtype = request.param
    tmp = tmp_path_factory.mktemp(f"replay_{name}_{dtype}")
    folder = make_folder(tmp, name, seed=3)
    # 448 tokens of cache: the mixed test below cannot run without pages being handed out again
    r = Replay(folder, dtype, tmp / "out", max_tokens=448, page_size=util.PAGE[name])
    yield name, dtype, folder, r
    assert r.close() == 0


def test_each_request_alone_and_whole(replay):
    name, dtype, folder, r = replay
    for n in LENGTHS[name]:
        ids = token_ids(name, n, seed=1)
        got = r.step([{"id": f"w{n}", "tokens": ids, "want": list(range(n))}], end=[f"w{n}"])
        compare(got, plain_logits(folder, ids), dtype, f"whole request of {n}")


def test_most_in_one_step_then_32_one_by_one(replay):
    name, dtype, folder, r = replay
    for n in (40, 131):
        ids = token_ids(name, n, seed=2)
        want = plain_logits(folder, ids)
        head = n - 32
        got = r.step([{"id": "d", "tokens": ids[:head], "want": [head - 1]}])
        compare(got, want[head - 1:head], dtype, f"last row of the first {head}")
        for p in range(head, n):
            got = r.step([{"id": "d", "tokens": [ids[p]], "want": [0]}], end=["d"] if p == n - 1 else [])
            compare(got, want[p:p + 1], dtype, f"decoded position {p} of {n}")


def test_portions_of_changing_size(replay):
    name, dtype, folder, r = replay
    n = 150
    ids = token_ids(name, n, seed=3)
    want = plain_logits(folder, ids)
    cuts = [7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 8, 40, 2, 6]
    assert sum(cuts) == n
    pos = 0
    for i, c in enumerate(cuts):
        got = r.step([{"id": "p", "tokens": ids[pos:pos + c], "want": list(range(c))}], end=["p"] if i == len(cuts) - 1 else [])
        compare(got, want[pos:pos + c], dtype, f"portion {i} of {c} tokens at {pos}")
        pos += c


def test_first_tokens_of_a_sequence(replay):
    name, dtype, folder, r = replay
    ids = token_ids(name, 3, seed=4)
    want = plain_logits(folder, ids)
    got = r.step([{"id": "f", "tokens": ids[:1], "want": [0]}])
    compare(got, want[:1], dtype, "position 0 alone")
    got = r.step([{"id": "f", "tokens": ids[1:3], "want": [0, 1]}], end=["f"])
    compare(got, want[1:3], dtype, "positions 1-2")


def test_long_decoding(replay):
    name, dtype, folder, r = replay
    n = 200
    ids = token_ids(name, n, seed=5)
    want = plain_logits(folder, ids)
    got = r.step([{"id": "l", "tokens": ids[:3], "want": [2]}])
    compare(got, want[2:3], dtype, "prompt of 3")
    for p in range(3, n):
        got = r.step([{"id": "l", "tokens": [ids[p]], "want": [0]}], end=["l"] if p == n - 1 else [])
        compare(got, want[p:p + 1], dtype, f"decoded position {p}")


def test_mixed_requests_with_pages_used_again(replay):
    """Up to four live requests; portions of some beside decoded tokens of others; requests end and new ones
    start on the pages just given back (448 tokens of cache, far less than the sum of all requests)."""
    name, dtype, folder, r = replay
    lengths = [90, 61, 120, 33, 75, 110, 48, 100]
    seqs = {f"m{i}": token_ids(name, n, seed=10 + i) for i, n in enumerate(lengths)}
    want = {k: plain_logits(folder, v) for k, v in seqs.items()}
    pos = {k: 0 for k in seqs}
    waiting = list(seqs)
    live: list[str] = []
    portion = {"m0": 50, "m1": 7, "m2": 64, "m3": 2, "m4": 30, "m5": 41, "m6": 9, "m7": 16}
    step_no = 0
    while waiting or live:
        # admit while there is room for the request's whole length rounded up to 64
        def held(k):
            return -(-len(seqs[k]) // 64) * 64
        while waiting and len(live) < 4 and sum(held(k) for k in live) + held(waiting[0]) <= 448:
            live.append(waiting.pop(0))
        entries, checks, ended = [], [], []
        for j, k in enumerate(live):
            if (step_no + j) % 5 == 4:
                continue  # this request sits the step out
            left = len(seqs[k]) - pos[k]
            prompt_part = len(seqs[k]) - 32
            if pos[k] < prompt_part:
                c = min(portion[k], prompt_part - pos[k])
                wanted = [c - 1] if c > 1 else [0]
                if c > 2:
                    wanted = [0, c - 1]
            else:
                c, wanted = 1, [0]
            entries.append({"id": k, "tokens": seqs[k][pos[k]:pos[k] + c], "want": wanted})
            checks.append((k, [pos[k] + w for w in wanted]))
            pos[k] += c
            if c == left:
                ended.append(k)
        if entries:
            got = r.step(entries, end=ended)
            row = 0
            for k, places in checks:
                for p in places:
                    compare(got[row:row + 1], want[k][p:p + 1], dtype, f"step {step_no}: request {k} position {p}")
                    row += 1
            assert row == got.shape[0]
        for k in ended:
            live.remove(k)
        step_no += 1
        assert step_no < 2000


def _qwen3(h, inter, layers, heads, kv, d, vocab, eps=1e-6, theta=1e4, tie=False, window=None, types=None):
    c = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": h, "intermediate_size": inter,
         "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv, "rms_norm_eps": eps,
         "rope_theta": theta, "vocab_size": vocab, "tie_word_embeddings": tie, "max_position_embeddings": 512,
         "eos_token_id": vocab - 1}
    if d is not None:
        c["head_dim"] = d
    if window:
        c.update(use_sliding_window=True, sliding_window=window, layer_types=types)
    return c


# Sizes that the two tiny configurations do not reach: a width and an intermediate size that are no multiple of 8
# (66: not even of 4), head sizes 48, 80, 96, 112 and 256, one head, as many groups as heads, windows on some layers.
ODD_SIZES = {
    "width100": _qwen3(100, 100, 2, 7, 1, 16, 1001),
    "width66": _qwen3(66, 36, 2, 11, 11, 16, 97),
    "head48": _qwen3(80, 72, 1, 5, 5, 48, 1000),
    "head80": _qwen3(136, 200, 4, 3, 1, 80, 333, eps=1e-5, theta=5e5, tie=True),
    "head96_window": _qwen3(192, 264, 2, 2, 2, 96, 777, window=17, types=["sliding_attention", "full_attention"]),
    "head112": _qwen3(224, 96, 1, 2, 1, 112, 50, eps=1e-3),
    "one_head256": _qwen3(64, 48, 1, 1, 1, 256, 64),
    # head sizes 64 and 128 with a windowed layer and small pages: in bfloat16 these run the TMA split-KV kernel and the
    # tcgen05 prefill kernel over block tables whose front pages the window has passed and given back
    "head64_window": _qwen3(128, 96, 2, 4, 2, 64, 300, window=40, types=["sliding_attention", "full_attention"]),
    "head128_window": _qwen3(256, 128, 3, 2, 1, 128, 211, eps=1e-5, window=33,
                             types=["full_attention", "sliding_attention", "sliding_attention"]),
}
# Tokens per page of each: sizes that do not divide 64 (24, 40), that are larger than 64 (128, 256), and the small
# powers of two that TMA gathers take.
ODD_PAGES = {"width100": 24, "width66": 40, "head48": 256, "head80": 8, "head96_window": 16, "head112": 128, "one_head256": 64,
             "head64_window": 8, "head128_window": 16}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ODD_SIZES))
def test_random_trace_at_odd_sizes(name, dtype, tmp_path):
    """A seeded random trace (up to four live requests, random portions and sit-outs, random wanted places, some
    requests dropped before their end, 448 tokens of cache) on a configuration of odd sizes."""
    import random

    rng = random.Random(len(name) * 131 + len(dtype))
    util.CONFIGS[name] = ODD_SIZES[name]
    try:
        folder = make_folder(tmp_path, name, seed=7)
    finally:
        del util.CONFIGS[name]
    vocab = ODD_SIZES[name]["vocab_size"]
    page_size = ODD_PAGES[name]
    max_tokens = 448 if page_size <= 64 else 3 * page_size   # few pages either way, so that they are used again
    r = Replay(folder, dtype, tmp_path / "out", max_tokens=max_tokens, page_size=page_size)
    lengths = [rng.choice([1, 2, 3, 15, 16, 17, 33, 64, 65, 100, 129, rng.randint(1, 190)]) for _ in range(8)]
    seqs = {f"q{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}
    want = {k: plain_logits(folder, v) for k, v in seqs.items()}
    stop_at = {k: (len(v) if rng.random() < 0.8 else rng.randint(1, len(v))) for k, v in seqs.items()}
    pos = {k: 0 for k in seqs}
    waiting, live, step_no = list(seqs), [], 0

    unit = max(64, page_size)   # a request's count is rounded up to 64, or to the engine's pages if those are larger

    def held(k):
        return -(-len(seqs[k]) // unit) * unit

    while waiting or live:
        while waiting and len(live) < 4 and sum(held(k) for k in live) + held(waiting[0]) <= max_tokens:
            live.append(waiting.pop(0))
        entries, checks, ended = [], {}, []
        for k in live:
            if rng.random() < 0.2:
                continue
            left = stop_at[k] - pos[k]
            c = min(left, rng.choice([1, 1, 1, 1, 2, 2, 3, 5, 8, 15, 16, 17, 31, 33, 64]))
            wanted = sorted(rng.sample(range(c), rng.randint(0, min(c, 3))))
            entries.append({"id": k, "tokens": seqs[k][pos[k]:pos[k] + c], "want": wanted})
            checks[k] = [pos[k] + w for w in wanted]
            pos[k] += c
            if c == left:
                ended.append(k)
        if entries:
            rng.shuffle(entries)
            got = r.step(entries, end=ended)
            row = 0
            for e in entries:
                for p in checks[e["id"]]:
                    compare(got[row:row + 1], want[e["id"]][p:p + 1], dtype, f"{name} step {step_no}: request {e['id']} position {p}")
                    row += 1
        for k in ended:
            live.remove(k)
        step_no += 1
        assert step_no < 5000
    assert r.close() == 0
