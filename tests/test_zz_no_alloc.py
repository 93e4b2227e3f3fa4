"""The allocation-free sampling entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the moment they sample (all memory belongs to another
runtime's pool, or their serving loop forbids allocator calls after warm-up). For them ``oxr_sample_static`` keeps
its scratch in a static device array inside the library. This test calls it the way such a caller would, with
``ctypes`` on the built library and raw device pointers, and checks its tokens against the regular entry point
(``ops.sample``, whose scratch comes from torch's allocator): on two calls in a row, the second smaller than the
first so that words left over from the first call lie beyond what the second one writes, and once more after a
greedy-only call. A request beyond the static array's size must be refused with a message.

The file is named so that pytest collects it last.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from oxr_inference_b200.ops import build

    lib = build.core_library()
    fn = lib.oxr_sample_static
    p, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [p, p, i, i, p, p, p, p, p, ctypes.c_char_p, i]
    fn.restype = i
    return fn


def _call(fn, logits, temperature=None, lo=None, hi=None, counter=None):
    out = torch.full((logits.shape[0],), -1, dtype=torch.int32, device=logits.device)
    msg = ctypes.create_string_buffer(512)

    def ptr(t):
        return None if t is None else t.data_ptr()
    code = fn(out.data_ptr(), logits.data_ptr(), logits.shape[0], logits.shape[1], ptr(temperature), ptr(lo), ptr(hi), ptr(counter),
              torch.cuda.current_stream().cuda_stream, msg, len(msg))
    return code, msg.value.decode(), out


def test_static_scratch_sampling_matches_the_regular_entry_point_on_calls_in_a_row():
    from oxr_inference_b200 import ops

    fn = _entry()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(77)

    def case(rows, vocab):
        logits = torch.randn(rows, vocab, device=dev, generator=g) * 2
        temp = torch.full((rows,), 0.8, device=dev)
        temp[::3] = 0.0  # every third row greedy
        lo = torch.randint(-2**31, 2**31 - 1, (rows,), device=dev, generator=g, dtype=torch.int64).to(torch.int32)
        hi = torch.randint(0, 2**31 - 1, (rows,), device=dev, generator=g, dtype=torch.int64).to(torch.int32)
        counter = torch.arange(rows, dtype=torch.int32, device=dev)
        return logits, temp, lo, hi, counter

    # first call: many rows, a vocabulary that is no multiple of the chunk; second call right after it: fewer rows, fewer
    # chunks (what the first call left in the array lies beyond and between what the second writes)
    for rows, vocab in ((24, 151936), (5, 5000), (9, 151936)):
        args = case(rows, vocab)
        code, msg, got = _call(fn, *args)
        assert code == 0, msg
        want = ops.sample(*args)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"{rows} x {vocab}: static-scratch tokens differ from the regular entry point's"
    # greedy only (no temperature array at all), then sampled again
    logits = torch.randn(7, 30000, device=dev, generator=g)
    code, msg, got = _call(fn, logits)
    assert code == 0, msg
    assert torch.equal(got, ops.sample(logits)) and torch.equal(got.long(), logits.argmax(-1))
    args = case(16, 70001)
    code, msg, got = _call(fn, *args)
    assert code == 0 and torch.equal(got, ops.sample(*args))


def test_sizes_beyond_the_static_array_are_refused_with_a_message():
    fn = _entry()
    rows, vocab = 1024, 151936  # 1024 rows x 75 chunks = 76800 > 65536
    logits = torch.zeros(rows, vocab, device="cuda")
    code, msg, out = _call(fn, logits)
    assert code == 200 and "static array holds" in msg and "oxr_sample" in msg
    torch.cuda.synchronize()
    assert (out == -1).all(), "a refused call must launch nothing"
    code, msg, _ = _call(fn, logits[:0])
    assert code == 201 and "rows" in msg
    temp = torch.ones(4, device="cuda")
    code, msg, _ = _call(fn, logits[:4].contiguous(), temp)
    assert code == 201 and "seed" in msg
