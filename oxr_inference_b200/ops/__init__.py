"""Python entry points of the hand-written sm_100a kernels (``csrc/``), one function per kernel.

Every function launches on torch's current CUDA stream, takes and returns torch tensors (used as storage
only) and raises :class:`KernelError` when a launcher refuses its arguments. There is no CPU path and no
fallback: tensors that are not on a CUDA device are an error, and a missing compiler or failed build raises
``BuildError`` at the first call.

Matrix products (the reference's go to cuBLAS through ``nn.Linear``, oxr_runtime/language.py:223-244): the 32-bit
path, the decode-sized bf16 products (at most ``SKINNY_MAX_ROWS`` rows) and the larger bf16 products all run on
this package's own kernels; ``torch.mm`` is kept only for bf16 matrices whose rows TMA cannot fetch.
"""

from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

from oxr_inference_b200.ops import build
from oxr_inference_b200.ops.build import BuildError  # noqa: F401

SKINNY_MAX_ROWS = 16
STREAM_MAX_ROWS = 16
STREAM_GEMM = os.environ.get("OXR_B200_STREAM", "1") != "0"
"""Whether bf16 products of at most ``STREAM_MAX_ROWS`` rows (decode steps) run the weight-streaming kernel (a persistent
block per SM whose producer warp fills a shared-memory ring with cp.async.bulk, also while the kernel before it still
runs) instead of the register-fed skinny kernel. ``OXR_B200_STREAM=0`` switches back, for comparisons."""
STATUS_NAMES = {
    1: "token id outside the vocabulary", 2: "cache slot outside the pool", 3: "position outside the rotary table",
    4: "block table names a page outside the pool", 5: "a bounded wait inside a kernel ran out",
}
_DT = {torch.float32: 0, torch.bfloat16: 1}

CHAIN_KERNELS = os.environ.get("OXR_B200_CHAIN", "1") != "0"
"""Whether RMSNorm, q/k norm + RoPE, split-KV attention and the tcgen05 GEMMs are launched programmatically
dependent on the kernel before them: each is scheduled while its predecessor finishes, fetches what no kernel of the step
writes (weights, old keys) and waits with ``griddepcontrol.wait`` before it touches activations. ``OXR_B200_CHAIN=0``
turns it off."""

launch_count = 0
"""Kernels of this package launched so far in this process (cuBLAS calls are not counted)."""


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported; kernels take float32 and bfloat16") from None


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


def _stream() -> int:
    """Handle of the current CUDA stream. The raw getter costs a fraction of a microsecond; `torch.cuda.current_stream()`
    builds a Stream object per call (several microseconds, per kernel launch of an eager step)."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _done(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        if code >= 1000:
            raise KernelError(f"{what}: CUDA error {code - 1000} at launch")
        raise KernelError(f"{what}: launcher refused its arguments (code {code})")
    launch_count += 1


_core = None


def _lib():
    global _core
    if _core is None:
        lib = build.core_library()
        p, i, f = c_void_p, c_int, c_float
        lib.oxr_embedding.argtypes = [p, p, p, i, i, i, i, i, p, p]
        lib.oxr_add_rms_norm.argtypes = [p, p, p, p, p, p, i, i, f, i, p]
        lib.oxr_silu_mul.argtypes = [p, p, i, i, i, i, p]
        lib.oxr_cast.argtypes = [p, p, c_size_t, i, i, p]
        lib.oxr_qk_norm_rope_store.argtypes = [p, p, p, p, p, p, p, p, p, p, i, i, i, i, f, i, c_longlong, i, i, i, i, p, p]
        lib.oxr_gemm_f32_nt.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_gemm_skinny_bf16.argtypes = [p, p, p, i, i, i, i, p]
        lib.oxr_gemm_skinny_gated_bf16.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_gemm_stream_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_gemm_stream_gated_bf16.argtypes = [p, p, p, i, i, i, p, p]
        lib.oxr_gemm_stream_add_bf16.argtypes = [p, p, p, p, p, p, p, i, i, i, p, p]
        lib.oxr_gemm_stream_add_bf16.restype = c_int
        lib.oxr_gemm_stream_scaled_bf16.argtypes = [p, p, p, i, f, p, i, i, i, i, p, p]
        lib.oxr_gemm_stream_scaled_bf16.restype = c_int
        lib.oxr_gemm_stream_blocks.argtypes = [i]
        lib.oxr_gemm_stream_blocks.restype = c_int
        lib.oxr_gemm_tcgen05_bf16.argtypes = [p, p, p, i, i, i, i, i, i, p, p, p, p]
        lib.oxr_gemm_tcgen05_pair_bf16.argtypes = [p, p, p, i, i, i, i, i, p, p]
        lib.oxr_gemm_tcgen05_gated_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_gemm_few_rows_cluster_bf16.argtypes = [p, p, p, i, i, i, i, i, p, p]
        lib.oxr_gemm_few_rows_max_clusters.argtypes = [i]
        lib.oxr_gemm_tcgen05_pair_gated_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_sample.argtypes = [p, p, i, i, p, p, p, p, p, p]
        lib.oxr_sample_chunks.argtypes = [i]
        lib.oxr_sample_chunks.restype = c_int
        lib.oxr_repetition_penalty.argtypes = [p, p, p, p, i, i, p]
        lib.oxr_mark_seen.argtypes = [p, p, p, i, i, p]
        for name in ("oxr_embedding", "oxr_add_rms_norm", "oxr_silu_mul", "oxr_cast", "oxr_qk_norm_rope_store",
                     "oxr_gemm_f32_nt", "oxr_gemm_skinny_bf16", "oxr_gemm_skinny_gated_bf16", "oxr_gemm_stream_bf16", "oxr_gemm_stream_gated_bf16", "oxr_gemm_tcgen05_bf16", "oxr_gemm_tcgen05_pair_bf16", "oxr_gemm_tcgen05_gated_bf16", "oxr_gemm_few_rows_cluster_bf16", "oxr_gemm_few_rows_max_clusters",
                     "oxr_gemm_tcgen05_pair_gated_bf16", "oxr_sample", "oxr_repetition_penalty", "oxr_mark_seen"):
            getattr(lib, name).restype = c_int
        lib.oxr_set_chain.argtypes = [c_int]
        lib.oxr_set_chain.restype = None
        lib.oxr_set_chain(int(CHAIN_KERNELS))
        _core = lib
    return _core


_attn: dict[int, ctypes.CDLL] = {}


def _attn_lib(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        p, i, f = c_void_p, c_int, c_float
        lib.oxr_paged_attention.argtypes = [p, p, p, p, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p]
        lib.oxr_paged_attention.restype = c_int
        lib.oxr_paged_attention_bf16.argtypes = [p, p, p, p, p, p, i, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p, p, p, i, i, i, i, p, p]
        lib.oxr_attn_make_kv_maps.argtypes = [p, p, p, ctypes.c_ulonglong, i, i]
        lib.oxr_attn_make_kv_maps.restype = c_int
        lib.oxr_paged_attention_fused_decode_bf16.argtypes = [p, p, p, p, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p, p, p, i, i, p, p, p, p, f, i, i,
                                                              p, p]
        lib.oxr_paged_attention_fused_decode_bf16.restype = c_int
        lib.oxr_attn_one_round_of_pieces.argtypes = []
        lib.oxr_attn_one_round_of_pieces.restype = c_int
        lib.oxr_attn_even_cut_slots.argtypes = [i]
        lib.oxr_attn_even_cut_slots.restype = c_int
        lib.oxr_paged_attention_bf16.restype = c_int
        lib.oxr_attn_tile_rows.argtypes = [i]
        lib.oxr_attn_tile_rows.restype = c_int
        lib.oxr_attn_head_dim.restype = c_int
        lib.oxr_attn_last_short_kernel.restype = c_int
        if lib.oxr_attn_head_dim() != head_dim:
            raise BuildError(f"attention library for head size {head_dim} reports {lib.oxr_attn_head_dim()}")
        rows = tuple(lib.oxr_attn_tile_rows(kind) for kind in range(4))
        if rows != (GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA):
            raise BuildError(f"attention library tiles have {rows} rows; the host builds its tile lists for "
                             f"{(GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA)}")
        lib.oxr_set_chain.argtypes = [c_int]
        lib.oxr_set_chain.restype = None
        lib.oxr_set_chain(int(CHAIN_KERNELS))
        _attn[head_dim] = lib
    return lib


SHORT_KERNELS = {0: None, 1: "attn_mma_decode_kernel", 2: "attn_tma_decode_kernel", 3: "attn_tma_decode_walk_kernel",
                 4: "attn_tma_decode_walk_kernel (one round)"}


def last_short_attention_kernel(head_dim: int) -> str | None:
    """Name of the split-KV kernel that the last ``paged_attention`` call with short tiles launched for this head size."""
    return SHORT_KERNELS[_attn_lib(head_dim).oxr_attn_last_short_kernel()]


def warm_up(head_dims: tuple[int, ...] = ()) -> None:
    """Build and load what a model needs, before the first step."""
    _lib()
    for d in head_dims:
        _attn_lib(d)


_status: dict[torch.device, torch.Tensor] = {}


def new_status(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device's status word: [code, detail, 0, 0]; kernels write the first error they meet. One per device, shared
    by everything that runs there."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _status:
        _status[device] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[device]


def check_status(status: torch.Tensor) -> None:
    """Read the status word (synchronises) and raise if a kernel reported an error; clears it."""
    code, detail = status[:2].tolist()
    if code != 0:
        status.zero_()
        raise KernelError(f"a kernel reported: {STATUS_NAMES.get(code, code)} (at index {detail})")


# --------------------------------------------------------------------------------------------------- ops
def embedding(ids: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype, status: torch.Tensor) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` (oxr_runtime/decode_graph.py:75); an id outside the table sets the status word."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    n, (vocab, hidden) = ids.numel(), table.shape
    out = torch.empty((n, hidden), dtype=out_dtype, device=table.device)
    code = _lib().oxr_embedding(out.data_ptr(), table.data_ptr(), ids.data_ptr(), n, hidden, vocab, _dtype_code(table),
                                _DT[out_dtype], status.data_ptr(), _stream())
    _done(code, "embedding")
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, *,
                 rows: torch.Tensor | None = None, keep_residual: bool = True):
    """RMSNorm with the residual add fused in (oxr_runtime/language.py:69-72,94-99).

    ``sum = x + residual`` (fp32; just ``x`` when ``residual`` is None), ``out = sum * rsqrt(mean(sum^2) + eps) *
    weight`` rounded to ``x.dtype``. The fp32 residual stream is updated in place (created when None) and returned
    unless ``keep_residual`` is False. With ``rows`` (int32 indices) only those rows are normalised, output row i
    coming from input row ``rows[i]``; the residual is then left untouched.
    """
    _need(x, "x")
    _need(weight, "weight", torch.float32)
    n, hidden = x.shape
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of {hidden}")
    if residual is not None:
        _need(residual, "residual", torch.float32)
        if residual.shape != x.shape:
            raise KernelError(f"residual {tuple(residual.shape)} does not match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out, res_out = rows.numel(), None
    else:
        n_out = n
        res_out = None if not keep_residual else (residual if residual is not None else
                                                  torch.empty((n, hidden), dtype=torch.float32, device=x.device))
    out = torch.empty((n_out, hidden), dtype=x.dtype, device=x.device)
    code = _lib().oxr_add_rms_norm(out.data_ptr(), _ptr(res_out), x.data_ptr(), _ptr(residual), weight.data_ptr(),
                                   _ptr(rows), n_out, hidden, float(eps), _dtype_code(x), _stream())
    _done(code, "add_rms_norm")
    return out, res_out


def silu_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` (oxr_runtime/language.py:102-104) for ``gate_up = [gate | up]`` along the last axis, or,
    with ``interleave`` 8, for gate and up alternating in groups of 8 columns (what ``GATE_UP_INTERLEAVE`` rows of a
    stacked weight produce)."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even number of columns")
    if interleave not in (0, GATE_UP_INTERLEAVE) or (interleave and two_i % (2 * interleave)):
        raise KernelError(f"silu_mul: interleave {interleave} with {two_i} columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    code = _lib().oxr_silu_mul(out.data_ptr(), gate_up.data_ptr(), n, two_i // 2, interleave, _dtype_code(gate_up), _stream())
    _done(code, "silu_mul")
    return out


GATE_UP_INTERLEAVE = 8
"""Rows per group when a weight stacks a gate and an up projection alternately: what one block of the skinny GEMM sees
as its rows g and g + 8."""


def gated_silu_linear(x: torch.Tensor, weight: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)`` for a weight that stacks Wg and Wu: side by side (``interleave`` 0: one product,
    then the SiLU kernel) or alternating in groups of 8 rows. With alternating rows a bf16 product runs the kernel
    ``linear`` would pick for its size (skinny, one-SM or two-SM tcgen05) with an epilogue that applies SiLU to the fp32
    sums and writes the gated product alone; 32-bit runs the product and then the SiLU kernel on interleaved columns.
    ``x`` may be a :class:`NormedLazily`."""
    if isinstance(x, NormedLazily):
        out = _scaled_linear(x, weight, gated=True) if interleave == GATE_UP_INTERLEAVE else None
        if out is not None:
            return out
        x = x.materialize()
    _need(x, "x")
    _need(weight, "weight")
    m, k = x.shape
    n = weight.shape[0]
    fused = (interleave == GATE_UP_INTERLEAVE and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and n % 16 == 0
             and k % 8 == 0 and weight.shape[1] == k and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)
    if fused:
        lib = _lib()
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
        if STREAM_GEMM and m <= STREAM_MAX_ROWS:
            _done(lib.oxr_gemm_stream_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k,
                                                 new_status(x.device).data_ptr(), _stream()), "gemm_stream_gated")
        elif m <= SKINNY_MAX_ROWS:
            _done(lib.oxr_gemm_skinny_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _stream()), "gemm_skinny_gated")
        elif _gemm_pair_plan(m, n, k):
            _done(lib.oxr_gemm_tcgen05_pair_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _gemm_pair_plan(m, n, k),
                                                       new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair_gated")
        else:
            tile_n, _ = _gemm_plan(m, n, k, False)   # the gated epilogue has no shares of k
            _done(lib.oxr_gemm_tcgen05_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, tile_n,
                                                  new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_gated")
        return out
    return silu_mul(linear(x, weight), interleave)


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _need(x, "x")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    code = _lib().oxr_cast(out.data_ptr(), x.data_ptr(), x.numel(), _dtype_code(x), _DT[dtype], _stream())
    _done(code, "cast")
    return out


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                       cos: torch.Tensor | None, sin: torch.Tensor | None, positions: torch.Tensor,
                       slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int,
                       num_kv_heads: int, head_dim: int, eps: float, status: torch.Tensor) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotary encoding of both, K and V stored at ``slots`` of one layer's pool;
    returns q ``[n, H, D]`` (oxr_runtime/kernels.py:66-99). A None weight skips that norm, None tables skip the
    rotation, a negative slot skips that token's store."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    _need(slots, "slots", torch.int32)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected (H + 2 KV) * D = {width}")
    for w, nm in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, nm, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"{nm} has {w.numel()} entries for head size {head_dim}")
    rotate = cos is not None
    max_positions = 0
    if rotate:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [max_positions, head_dim / 2]")
        max_positions = cos.shape[0]
    num_slots = k_cache.numel() // (num_kv_heads * head_dim)
    q = torch.empty((n, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    code = _lib().oxr_qk_norm_rope_store(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos),
        _ptr(sin), positions.data_ptr(), slots.data_ptr(), n, num_heads, num_kv_heads, head_dim, float(eps),
        max_positions, num_slots, int(q_weight is not None), int(k_weight is not None), int(rotate), _dtype_code(qkv),
        status.data_ptr(), _stream())
    _done(code, "qk_norm_rope_store")
    return q


GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA = 16, 16, 64, 256
SHORT_MAX_TOKENS = 8
"""Requests that bring at most this many tokens go to the split-KV kernel, longer portions to the prefill kernel."""
MAX_SPLITS = 32


@functools.lru_cache(maxsize=None)
def num_sms() -> int:
    """Multiprocessors of the current device (the launchers ask the device as well); where no device is present, as
    when plans are inspected on a machine without a GPU, a B200's 148."""
    if torch.cuda.is_available():
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return 148


def _tokens_per_tile(num_heads: int, num_kv_heads: int, rows: int) -> int:
    return rows // min(num_heads // num_kv_heads, rows)


def tma_gathers_possible(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether K and V of such a cache can be fetched by TMA: bf16, head size a multiple of 64, pages of 8 * 2^k tokens."""
    return dtype == torch.bfloat16 and head_dim % 64 == 0 and page_size >= 8 and page_size & (page_size - 1) == 0


def _long_rows(head_dim: int, tma: bool) -> int:
    return PREFILL_ROWS_TMA if tma and head_dim <= 128 else PREFILL_ROWS


def attention_tile_specs(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype,
                         page_size: int | None = None) -> list[tuple[int, int, int]]:
    """The tile lists the attention kernels of this dtype read: (tokens per tile, fewest, most new tokens of the
    requests the list covers). The host cuts each request's new tokens into such tiles. With a ``page_size`` that
    allows TMA gathers the long tiles are 256 rows (the tcgen05 prefill kernel), else 64."""
    build.check_head_dim(head_dim)
    big = 1 << 30
    if dtype == torch.bfloat16:
        tma = page_size is not None and tma_gathers_possible(head_dim, page_size, dtype)
        return [(_tokens_per_tile(num_heads, num_kv_heads, DECODE_ROWS), 1, SHORT_MAX_TOKENS),
                (_tokens_per_tile(num_heads, num_kv_heads, _long_rows(head_dim, tma)), SHORT_MAX_TOKENS + 1, big)]
    return [(_tokens_per_tile(num_heads, num_kv_heads, GENERIC_ROWS), 1, big)]


DECODE_BLOCKS_PER_SM = 2
"""Blocks of the split-KV kernel that fit on one SM (its shared memory is the limit)."""


DECODE_CUT = os.environ.get("OXR_B200_DECODE_CUT", "auto")
"""How the split-KV kernel with TMA gathers cuts a step's keys: ``equal``: every request
into the same number of pieces; ``even``: ALL key blocks of the step dealt out evenly to one round of blocks, so that
requests of very different lengths still give every block the same share (a block's run may end one request and begin the
next); ``auto`` (default): the even cut for the steps whose caller says that the lengths differ much (``uneven``), equal
pieces otherwise (with lengths alike the even cut only costs: 3 us per layer at batch 8), and equal pieces also for more than
``EVEN_CUT_MAX_TILES`` requests: the engine runs a decode step's requests longest first, so that hundreds of them dealt out
piece by piece come out even by themselves (decode steps of Qwen3-4B sizes, contexts drawn up to 2,048 to 8,192 keys, eight
layers: 8 requests 0.98 against 1.05 ms, 64: 1.83 against 2.10, 128: 1.97 against 2.30, 256: 3.34 against 3.24)."""
EVEN_CUT_MAX_TILES = 192


def attention_splits(n_short_tiles: int, num_heads: int, num_kv_heads: int, kv_len_bound: int) -> int:
    """Into how many pieces the split-KV kernel cuts each request's keys. Blocks run in waves of
    ``num_sms() * DECODE_BLOCKS_PER_SM``; a block walks its piece's 64-key blocks one after the other and spends about
    as long as 4.5 of them before its first keys arrive and after its last (measured on a B200: 7 us against 1.6 us per
    block). The number of pieces with the least waves x (4.5 + blocks per piece) wins, the smaller among equals; no
    piece is shorter than 128 keys. Depends only on sizes the host knows before the step (fixed inside a CUDA
    graph)."""
    group = num_heads // num_kv_heads
    blocks = max(1, n_short_tiles * num_kv_heads * -(-group // min(group, DECODE_ROWS)))
    slots = num_sms() * DECODE_BLOCKS_PER_SM
    key_blocks = max(1, -(-kv_len_bound // 64))
    best, best_cost = 1, None
    for splits in range(1, max(1, min(MAX_SPLITS, kv_len_bound // 128)) + 1):
        cost = -(-blocks * splits // slots) * (4.5 + -(-key_blocks // splits))
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    return best


class KVMaps:
    """The two TMA tensor maps (K, V) of one cache group's pool, in 64-byte aligned host memory."""

    def __init__(self, raw: ctypes.Array, address: int, pool_ptrs: tuple[int, int], rows_per_layer: int):
        self.raw, self.address, self.pool_ptrs, self.rows_per_layer = raw, address, pool_ptrs, rows_per_layer


def make_kv_maps(k_pool: torch.Tensor, v_pool: torch.Tensor, page_size: int) -> KVMaps | None:
    """Tensor maps over a group's whole pool ``[layers, pages, page_size, KV, D]`` so that the split-KV kernel can
    fetch K and V by TMA; None when the sizes do not allow it (the kernel then gathers with cp.async)."""
    if k_pool.dtype != torch.bfloat16 or not k_pool.is_cuda:
        return None
    layers, pages, page, kv, d = k_pool.shape
    if d % 64 != 0 or page_size < 8 or page_size & (page_size - 1):
        return None
    raw = ctypes.create_string_buffer(2 * 128 + 64)
    address = (ctypes.addressof(raw) + 63) & ~63
    code = _attn_lib(d).oxr_attn_make_kv_maps(address, k_pool.data_ptr(), v_pool.data_ptr(), layers * pages * page, kv * d, page_size)
    if code != 0:
        return None
    return KVMaps(raw, address, (k_pool.data_ptr(), v_pool.data_ptr()), pages * page)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, tiles: dict, cu_q: torch.Tensor,
                    ctx_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, scale: float, window: int,
                    kv_len_bound: int, status: torch.Tensor, generic: bool = False, kv_maps: KVMaps | None = None,
                    layer_in_pool: int = 0, uneven: bool = False) -> torch.Tensor:
    """Causal grouped-query attention of the step's new tokens over the paged cache
    (oxr_runtime/attention.py:47-109). ``q`` is ``[tokens, H, D]``; ``k_cache`` / ``v_cache`` are one layer's pool
    ``[pages, page_size, KV, D]``; ``window`` > 0 limits a query to its last ``window`` keys; ``tiles`` maps each
    spec of :func:`attention_tile_specs` to ``(tile_req, tile_tok0, count)``; ``kv_len_bound`` is an upper bound of
    the context lengths. float32 runs the fp32 CUDA-core kernel, bfloat16 the tensor-core kernels (``generic``
    forces the CUDA-core kernel, which then needs the float32 tile spec). With ``kv_maps`` (of the pool that
    ``k_cache`` / ``v_cache`` are layer ``layer_in_pool`` of) the split-KV kernel fetches K and V by TMA. ``uneven``: the
    caller knows that the requests' lengths differ much (see ``DECODE_CUT``)."""
    _need(q, "q")
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    for t, nm in ((cu_q, "cu_q"), (ctx_lens, "ctx_lens"), (block_table, "block_table")):
        _need(t, nm, torch.int32)
    _, num_heads, head_dim = q.shape
    num_pages, page, num_kv_heads, d2 = k_cache.shape
    if page != page_size or d2 != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError(f"cache pool {tuple(k_cache.shape)} does not fit page size {page_size} / head size {head_dim}")
    lib = _attn_lib(head_dim)
    out = torch.empty_like(q)
    common = (cu_q.data_ptr(), ctx_lens.data_ptr(), block_table.data_ptr(), block_table.shape[-1], page_size, num_pages,
              num_heads, num_kv_heads, float(scale), int(window))
    if q.dtype == torch.float32 or generic:
        (spec,) = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.float32)
        tile_req, tile_tok0, n = tiles[spec]
        code = lib.oxr_paged_attention(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), tile_req.data_ptr(),
                                       tile_tok0.data_ptr(), n, *common, _dtype_code(q), status.data_ptr(), _stream())
        _done(code, "paged_attention")
        return out
    long_rows = _long_rows(head_dim, kv_maps is not None)
    short, long_ = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.bfloat16, page_size if kv_maps is not None else None)
    if long_ not in tiles:
        raise KernelError(f"no tile list for long tiles of {long_rows} rows: the batch was cut for {sorted(tiles)}")
    s_req, s_tok, n_short = tiles[short]
    l_req, l_tok, n_long = tiles[long_]
    splits, cut, part_o, part_ml, counters = _split_kv_plan(lib, n_short, num_heads, num_kv_heads, head_dim, kv_len_bound, kv_maps is not None,
                                                            uneven, q.device)
    code = lib.oxr_paged_attention_bf16(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), s_req.data_ptr(),
                                        s_tok.data_ptr(), n_short, l_req.data_ptr(), l_tok.data_ptr(), n_long, *common, splits,
                                        _ptr(part_o), _ptr(part_ml), _ptr(counters),
                                        kv_maps.address if kv_maps is not None else None,
                                        layer_in_pool * kv_maps.rows_per_layer if kv_maps is not None else 0, long_rows, q.shape[0], cut,
                                        status.data_ptr(), _stream())
    global launch_count
    _done(code, "paged_attention_bf16")
    launch_count += 1 if n_long and n_short else 0
    return out


def _wants_even_cut(n_short: int, tma: bool, uneven: bool) -> bool:
    return bool(n_short) and tma and (DECODE_CUT == "even" or (DECODE_CUT == "auto" and uneven and n_short <= EVEN_CUT_MAX_TILES))


def _split_kv_plan(lib, n_short: int, num_heads: int, num_kv_heads: int, head_dim: int, kv_len_bound: int, tma: bool, uneven: bool,
                   device: torch.device):
    """Pieces per request, the cut (0 equal pieces, 1 the even cut) and the scratch of the split-KV kernel for ``n_short`` tiles."""
    splits = attention_splits(n_short, num_heads, num_kv_heads, kv_len_bound) if n_short else 1
    part_o = part_ml = counters = None
    cut = 0
    group = num_heads // num_kv_heads
    units = n_short * num_kv_heads * -(-group // min(group, DECODE_ROWS))
    slots = units * splits if splits > 1 else 0
    if _wants_even_cut(n_short, tma, uneven):
        # all key blocks of the step dealt out evenly to one round of blocks (requests of any mix of lengths): the library
        # says how many partial results that can make, or 0 if it cannot do it for so many units
        even = lib.oxr_attn_even_cut_slots(units)
        if even > 0:
            cut, slots = 1, max(slots, even)
    if slots:
        part_o = torch.empty(slots * DECODE_ROWS * head_dim, dtype=torch.float32, device=device)
        part_ml = torch.empty(slots * DECODE_ROWS * 2, dtype=torch.float32, device=device)
        counters = _ticket_counters(device, units)
    return splits, cut, part_o, part_ml, counters


FUSE_QKV = os.environ.get("OXR_B200_FUSE_QKV", "1") != "0"
"""Whether a decode step's attention takes the raw q|k|v projections itself (``decode_attention_from_projections``) where it can."""


def attention_takes_projections(head_dim: int, dtype: torch.dtype, page_size: int, kv_maps: KVMaps | None, *, requests: int = 0,
                                num_heads: int = 0, num_kv_heads: int = 0, kv_len_bound: int = 0, uneven: bool = False) -> bool:
    """Whether ``decode_attention_from_projections`` can run: bfloat16, the cache group's tensor maps, a head size that is a
    multiple of 64 and pages of 8 * 2^k tokens (what the split-KV kernel with TMA gathers needs); and, when ``requests`` says
    how many single-token requests the step has, that their pieces get a block each (no more than one round of blocks, not
    the even cut): only that form of the kernel takes the projections. (A block that walks over many pieces would prepare q
    for each of them; at 64 requests of 2,048 keys that cost more than the kernel it saves.)"""
    if not (FUSE_QKV and dtype == torch.bfloat16 and kv_maps is not None and head_dim % 64 == 0 and page_size >= 8
            and page_size & (page_size - 1) == 0):
        return False
    if requests:
        if _wants_even_cut(requests, True, uneven):
            return False
        group = num_heads // num_kv_heads
        units = requests * num_kv_heads * -(-group // min(group, DECODE_ROWS))
        if units * attention_splits(requests, num_heads, num_kv_heads, kv_len_bound) > _attn_lib(head_dim).oxr_attn_one_round_of_pieces():
            return False
    return True


def decode_attention_from_projections(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                                      cos: torch.Tensor | None, sin: torch.Tensor | None, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                                      store: bool, num_heads: int, num_kv_heads: int, head_dim: int, eps: float, tiles: dict,
                                      cu_q: torch.Tensor, ctx_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, scale: float,
                                      window: int, kv_len_bound: int, status: torch.Tensor, kv_maps: KVMaps, layer_in_pool: int = 0,
                                      uneven: bool = False) -> torch.Tensor:
    """``qk_norm_rope_store`` and ``paged_attention`` of a step in which EVERY request brings one token, as one kernel: row r of
    ``qkv`` ``[n, (H + 2 KV) * D]`` is request r's token, its position is ``ctx_lens[r] - 1``, its cache row the one the block
    table names for that position. ``store=False`` writes nothing and attends to what the cache holds. Returns ``[n, H, D]``.
    Call it only where ``attention_takes_projections`` (asked with the step's requests) says yes. Measured on a B200, Qwen3-8B
    sizes, 8 requests of 2,048 keys: the decode step 3.32 against 3.42 ms."""
    _need(qkv, "qkv", torch.bfloat16)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    for t, nm in ((cu_q, "cu_q"), (ctx_lens, "ctx_lens"), (block_table, "block_table")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected (H + 2 KV) * D = {(num_heads + 2 * num_kv_heads) * head_dim}")
    num_pages, page, kvh, d2 = k_cache.shape
    if page != page_size or d2 != head_dim or kvh != num_kv_heads or v_cache.shape != k_cache.shape:
        raise KernelError(f"cache pool {tuple(k_cache.shape)} does not fit page size {page_size} / {num_kv_heads} heads of {head_dim}")
    if not attention_takes_projections(head_dim, qkv.dtype, page_size, kv_maps, requests=n, num_heads=num_heads, num_kv_heads=num_kv_heads,
                                       kv_len_bound=kv_len_bound, uneven=uneven):
        raise KernelError(f"attention cannot take the projections itself for {n} requests at head size {head_dim}, page size {page_size}")
    for w, nm in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, nm, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"{nm} has {w.numel()} entries for head size {head_dim}")
    max_positions = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [max_positions, head_dim / 2]")
        max_positions = cos.shape[0]
    lib = _attn_lib(head_dim)
    short, _ = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.bfloat16, page_size)
    s_req, s_tok, n_short = tiles[short]
    if n_short != n or cu_q.numel() < n + 1:
        raise KernelError(f"{n} rows of projections but {n_short} single-token tiles: not a step of one token per request")
    splits, cut, part_o, part_ml, counters = _split_kv_plan(lib, n_short, num_heads, num_kv_heads, head_dim, kv_len_bound, True, uneven,
                                                            qkv.device)
    out = torch.empty((n, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    code = lib.oxr_paged_attention_fused_decode_bf16(
        out.data_ptr(), qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), s_req.data_ptr(), s_tok.data_ptr(), n_short,
        cu_q.data_ptr(), ctx_lens.data_ptr(), block_table.data_ptr(), block_table.shape[-1], page_size, num_pages, num_heads, num_kv_heads,
        float(scale), int(window), splits, _ptr(part_o), _ptr(part_ml), _ptr(counters), kv_maps.address,
        layer_in_pool * kv_maps.rows_per_layer, cut, _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), float(eps), max_positions,
        int(store), status.data_ptr(), _stream())
    _done(code, "paged_attention_fused_decode_bf16")
    return out


_counters: dict[torch.device, torch.Tensor] = {}
_outgrown: list[torch.Tensor] = []


def _ticket_counters(device: torch.device, units: int) -> torch.Tensor:
    """Zeroed ticket counters of the split-KV kernel, one per (tile, KV head group). The kernel leaves them zero, so
    one array serves every launch on a stream. An array that is outgrown is kept, not freed: a captured CUDA graph
    may hold its address."""
    t = _counters.get(device)
    if t is None or t.numel() < units:
        if t is not None:
            _outgrown.append(t)
        t = torch.zeros(max(units, 1 << 16), dtype=torch.int32, device=device)
        _counters[device] = t
    return t


GEMM_SPLITS = (1, 2, 3, 4, 6, 8)
GEMM_WORKSPACE_BYTES = 64 << 20
_GEMM_RING_BYTES = 227 * 1024 - 1024 - 256    # shared memory the kernel's stage ring may fill
_split_buffers: dict = {}


def _gemm_cost(m: int, n: int, k: int, tile_n: int, splits: int) -> float:
    """Microseconds the tcgen05 product is expected to take with tiles of 128 x ``tile_n`` and ``splits`` shares per
    tile. The constants are fitted to this kernel on a B200 (Qwen3-8B's four products at 17 to 8192 rows):

    * a 64-wide k step of one block takes 0.085 + 0.00144 * tile_n microseconds (shared-memory fill from L2), and no
      less than 0.24 (the round trip of a stage through TMA and the tensor core, divided by the stages in flight);
    * a wave of blocks takes at least the time HBM needs for the parts of W it streams (5.9 TB/s), and the two
      limits overlap all but about 15 %;
    * a split unit writes its partial tile and the last unit of a tile adds them up: 6.4 microseconds plus 0.065 per
      row and 128 columns, which later waves hide only by half;
    * 2.2 microseconds before the first block computes.
    """
    rows = -(-m // 128)
    tiles, steps = rows * -(-n // tile_n), -(-k // 64)
    per = -(-steps // splits)
    step_us = max(0.24, 0.085 + 0.00144 * tile_n)
    units = tiles * splits
    w_bytes = tile_n * 128 * per / rows        # blocks of the same wave share the W tiles of their column
    t = 2.2
    full, rest = divmod(units, num_sms())
    for active, count in ((num_sms(), full), (rest, 1 if rest else 0)):
        fill, stream = per * step_us, active * w_bytes / 5.9e6
        t += count * (max(fill, stream) + 0.15 * min(fill, stream))
    if splits > 1:
        waves = -(-units // num_sms())
        t += (1 + 0.5 * (waves - 1)) * (6.4 + 0.065 * min(m, 128) * tile_n / 128)
    return t


@functools.lru_cache(maxsize=None)
def _gemm_plan(m: int, n: int, k: int, may_split: bool = True) -> tuple[int, int]:
    """(tile width, shares of k per tile) of the tcgen05 product: the cheapest by ``_gemm_cost`` among widths of 32 to
    256 columns in steps of 16 and 1 to 8 shares whose partial tiles fit the workspace; the first found among equals."""
    best, best_cost = (128, 1), None
    steps = -(-k // 64)
    for tile_n in range(256, 16, -16):
        tiles = -(-m // 128) * -(-n // tile_n)
        for splits in (GEMM_SPLITS if may_split else (1,)):
            if splits > steps or (splits > 1 and splits * tiles * 128 * tile_n * 4 > GEMM_WORKSPACE_BYTES):
                continue
            cost = _gemm_cost(m, n, k, tile_n, splits)
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = (tile_n, splits), cost
    return best


GEMM_FEW_ROWS = 256          # the widest tile of a tcgen05 product
GEMM_FEW_ROWS_ANY_SHARES = 192


@functools.lru_cache(maxsize=None)
def _few_rows_clusters(shares: int) -> int:
    """Clusters of ``shares`` blocks of the few-rows kernel that the GPU holds at a time."""
    return int(_lib().oxr_gemm_few_rows_max_clusters(shares))


def _gemm_few_rows_plan(m: int, n: int, k: int) -> int:
    """Shares of k for the few-rows kernel (W on the 128-row side of the tiles, the rows of x as the tile's width, the
    shares of a tile the blocks of one cluster), or 0 where the ordinary kernel is to run. It stages no padding rows
    and adds the shares' partial tiles through distributed shared memory, which pays when W is narrow: N / 128 tiles
    are then far fewer than SMs and k is dealt out so that about one block per SM results. The plan is the most shares
    with which the clusters of all tiles run at once, at least two and at most four (clusters of five and more were
    level or up to 1.5 us slower, except with many rows and a long k: from 193 rows and 128 k steps on at most 8, a
    portable cluster). Measured on
    a B200 with Qwen3-8B's and 32B's products: level with cuBLAS or ahead of it from 17 to 128 rows (down projection at
    64 rows: 20.0 us, cuBLAS 22.1, the ordinary kernel with shares through a workspace 23.1); from 193 rows on only
    three shares or more still beat the ordinary kernel (each block fetches all rows of x for its k steps)."""
    if m > GEMM_FEW_ROWS:
        return 0
    tiles, steps = -(-n // 128), -(-k // 64)
    most = 8 if (m > GEMM_FEW_ROWS_ANY_SHARES and steps >= 128) else 4
    for shares in range(min(most, num_sms() // tiles, steps), 1, -1):
        if tiles <= _few_rows_clusters(shares):
            return shares if (m <= GEMM_FEW_ROWS_ANY_SHARES or shares >= 3) else 0
    return 0


GEMM_PAIR_MIN_ROWS = 512
STEP_TILE_ROWS = 256
"""Rows of the widest GEMM tile (the two-SM kernel's): a step of a few tokens more than a multiple of it pays for a whole
tile row. Whoever plans steps may ask for it."""


@functools.lru_cache(maxsize=None)
def _gemm_pair_plan(m: int, n: int, k: int) -> int:
    """Tile width for the two-SM product kernel (256 x width tiles, a pair of blocks each), or 0 where the one-SM
    kernel is to run. In isolated short runs the two kernels are level below about 3,000 rows; in long runs, where
    the power cap sets the clock, the pair kernel (a third less shared-memory traffic per flop) is 5 to 8 % faster
    from 512 rows on (sum of Qwen3-8B's four products, 150 calls each: 173 against 190 us at 512 rows, 604 against
    649 us at 2,048), and a 2,048-token prefill step takes 28.1 instead of 30.5 ms. The width is the one with the
    least waves of pairs times the time of a k step at that width (0.094 + 0.00128 width microseconds)."""
    if m < GEMM_PAIR_MIN_ROWS:
        return 0
    pairs = num_sms() // 2
    best, best_cost = 0, None
    for tile_n in (256, 224, 192, 160, 128, 96, 64):
        tiles = -(-m // 256) * -(-n // tile_n)
        cost = -(-tiles // pairs) * (0.094 + 0.00128 * tile_n)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = tile_n, cost
    return best


GEMM_MAX_SPLIT_TILES = GEMM_WORKSPACE_BYTES // (2 * 128 * 16 * 4)   # the most tiles a split product can have


def _gemm_split_buffers(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Workspace of the split product (one fp32 partial tile per unit) and its zeroed tickets (one per tile), made once
    per device at their full size and never replaced: a captured CUDA graph keeps their addresses. Products on one
    stream follow one another, and the kernel leaves the tickets zeroed."""
    got = _split_buffers.get(device)
    if got is None:
        got = (torch.empty(GEMM_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device),
               torch.zeros(GEMM_MAX_SPLIT_TILES, dtype=torch.int32, device=device))
        _split_buffers[device] = got
    return got


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ weight.T`` for ``weight [out, in]``, no bias (oxr_runtime/language.py:223-231), fp32 accumulation.

    float32 x float32 runs the fp32 CUDA-core kernel (no TF32). bfloat16 x bfloat16 runs the skinny kernel up to
    ``SKINNY_MAX_ROWS`` rows and the TMA + tcgen05 kernel beyond (cuBLAS only when a row is not a whole number of
    16-byte words). A weight kept in float32 under bfloat16 activations is multiplied in fp32 and the result
    rounded once.
    """
    if isinstance(x, NormedLazily):
        out = _scaled_linear(x, weight, gated=False) if out_dtype in (None, torch.bfloat16) else None
        if out is not None:
            return out
        x = x.materialize()
    _need(x, "x")
    _need(weight, "weight")
    m, k = x.shape
    n, k2 = weight.shape
    if k != k2:
        raise KernelError(f"linear: x has {k} columns, weight has {k2}")
    out_dtype = out_dtype or x.dtype
    lib = _lib()
    if weight.dtype == torch.float32:
        x32 = cast(x, torch.float32)
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        _done(lib.oxr_gemm_f32_nt(out.data_ptr(), x32.data_ptr(), weight.data_ptr(), m, n, k, _stream()), "gemm_f32")
        return cast(out, out_dtype)
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: activations {x.dtype} with weight {weight.dtype} is not a supported pair")
    if STREAM_GEMM and m <= STREAM_MAX_ROWS and k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        _done(lib.oxr_gemm_stream_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype],
                                       new_status(x.device).data_ptr(), _stream()), "gemm_stream")
        return out
    if m <= SKINNY_MAX_ROWS and k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        _done(lib.oxr_gemm_skinny_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], _stream()),
              "gemm_skinny")
        return out
    if k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        few = _gemm_few_rows_plan(m, n, k)
        if few:
            _done(lib.oxr_gemm_few_rows_cluster_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], few,
                                                     new_status(x.device).data_ptr(), _stream()), "gemm_few_rows_cluster")
            return out
        pair_tile = _gemm_pair_plan(m, n, k)
        if pair_tile:
            _done(lib.oxr_gemm_tcgen05_pair_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], pair_tile,
                                                 new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair")
            return out
        tile_n, splits = _gemm_plan(m, n, k)
        partial = tickets = None
        if splits > 1:
            if splits * -(-m // 128) * -(-n // tile_n) * 128 * tile_n * 4 > GEMM_WORKSPACE_BYTES:
                raise KernelError(f"linear: {splits} shares of {m} x {n} in tiles of {tile_n} columns outgrow the workspace")
            partial, tickets = _gemm_split_buffers(x.device)
        code = lib.oxr_gemm_tcgen05_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], tile_n, splits,
                                         _ptr(partial), _ptr(tickets), new_status(x.device).data_ptr(), _stream())
        _done(code, "gemm_tcgen05")
        return out
    # rows that are not whole 16-byte words cannot be fetched by TMA: the library product takes them
    if out_dtype == torch.float32:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    return torch.mm(x, weight.t())


FUSE_MAX_ROWS = min(16, int(os.environ.get("OXR_B200_FUSE_ROWS", "16")))
"""Decode steps of up to this many rows fold their norms into the products around them (0: never)."""
"""Most rows for which a decode step's RMSNorms are folded into the products around them."""


class NormedLazily:
    """``RMSNorm(residual) * weight`` with the row's scale still to be applied: ``y = bf16(residual * weight)`` and, per block
    of the product that wrote it, the sums of squares of the block's columns of the residual (``ops.linear_add``).
    ``ops.linear`` and ``ops.gated_silu_linear`` take it in place of x and scale their sums by rsqrt(mean + eps) row by row;
    ``materialize()`` runs the norm kernel on the residual for anyone else."""

    def __init__(self, y: torch.Tensor, residual: torch.Tensor, sums: torch.Tensor, blocks: int, weight: torch.Tensor, eps: float):
        self.y, self.residual, self.sums, self.blocks, self.weight, self.eps = y, residual, sums, blocks, weight, float(eps)

    @property
    def shape(self) -> torch.Size:
        return self.y.shape

    def materialize(self) -> torch.Tensor:
        return add_rms_norm(torch.zeros_like(self.y), self.residual, self.weight, self.eps, keep_residual=False)[0]


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None, norm_weight: torch.Tensor, eps: float
               ) -> tuple[NormedLazily, torch.Tensor] | None:
    """``add_rms_norm(linear(x, weight), residual, norm_weight, eps)`` for a decode step without the norm kernel: ONE kernel
    multiplies, rounds the product to bf16 as ``linear`` would, adds it into the fp32 residual stream (in place when one is
    given), and leaves the new residual times the norm's weight in bf16 and the rows' sums of squares, block by block; the
    row's scale rsqrt(mean + eps) is applied by the product that takes the result (:class:`NormedLazily`) to its fp32 sums.
    None when the sizes do not allow it (more than ``FUSE_MAX_ROWS`` rows, not bf16, ...): the caller then runs the two
    kernels."""
    m, k = x.shape
    n = weight.shape[0]
    if not (STREAM_GEMM and 0 < m <= FUSE_MAX_ROWS and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and k % 8 == 0 and n % 8 == 0 and weight.shape[1] == k and x.is_contiguous() and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and norm_weight.numel() == n and norm_weight.dtype == torch.float32):
        return None
    if residual is not None:
        _need(residual, "residual", torch.float32)
        if residual.shape != (m, n):
            raise KernelError(f"residual {tuple(residual.shape)} does not match the product's {(m, n)}")
    lib = _lib()
    blocks = lib.oxr_gemm_stream_blocks(n)
    res_out = residual if residual is not None else torch.empty((m, n), dtype=torch.float32, device=x.device)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sums = torch.empty((blocks, 16), dtype=torch.float32, device=x.device)
    code = lib.oxr_gemm_stream_add_bf16(res_out.data_ptr(), _ptr(residual), y.data_ptr(), sums.data_ptr(), norm_weight.data_ptr(),
                                        x.data_ptr(), weight.data_ptr(), m, n, k, new_status(x.device).data_ptr(), _stream())
    _done(code, "gemm_stream_add")
    return NormedLazily(y, res_out, sums, blocks, norm_weight, eps), res_out


def _scaled_linear(x: NormedLazily, weight: torch.Tensor, gated: bool) -> torch.Tensor | None:
    """``linear`` (or, ``gated``, silu(gate) * up on a weight with alternating rows) of a lazily normalised x in ONE kernel
    that scales its sums row by row; None when the sizes do not allow it."""
    m, k = x.y.shape
    n = weight.shape[0]
    if not (STREAM_GEMM and m <= STREAM_MAX_ROWS and weight.dtype == torch.bfloat16 and weight.shape[1] == k and k % 8 == 0
            and weight.data_ptr() % 16 == 0 and x.blocks <= num_sms() and (not gated or n % 16 == 0)):
        return None
    out = torch.empty((m, n // 2 if gated else n), dtype=torch.bfloat16, device=weight.device)
    code = _lib().oxr_gemm_stream_scaled_bf16(out.data_ptr(), x.y.data_ptr(), x.sums.data_ptr(), x.blocks, x.eps, weight.data_ptr(), m, n, k,
                                              int(gated), new_status(weight.device).data_ptr(), _stream())
    _done(code, "gemm_stream_scaled")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seed_lo: torch.Tensor | None = None,
           seed_hi: torch.Tensor | None = None, counter: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of fp32 ``logits``: the first maximum where ``temperature`` <= 0 (or None), else a draw
    from softmax(logits / temperature) decided by (seed, counter) alone."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
        for t, nm in ((seed_lo, "seed_lo"), (seed_hi, "seed_hi"), (counter, "counter")):
            if t is None:
                raise KernelError(f"sample: {nm} is required with a temperature")
            _need(t, nm, torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = _lib()
    # per row and vocabulary chunk: maximum, its index, sum of exponentials
    scratch = torch.empty(3 * rows * lib.oxr_sample_chunks(vocab), dtype=torch.int32, device=logits.device)
    code = lib.oxr_sample(out.data_ptr(), logits.data_ptr(), rows, vocab, _ptr(temperature), _ptr(seed_lo),
                          _ptr(seed_hi), _ptr(counter), scratch.data_ptr(), _stream())
    _done(code, "sample")
    global launch_count
    launch_count += 1  # two kernels
    return out


def repetition_penalty(logits: torch.Tensor, seen: torch.Tensor, row_slot: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for tokens marked in ``seen[row_slot[r]]`` a positive logit is divided by ``penalty[r]``, any other
    multiplied (oxr_runtime/engine.py:632-639)."""
    _need(logits, "logits", torch.float32)
    _need(seen, "seen", torch.uint8)
    _need(row_slot, "row_slot", torch.int32)
    _need(penalty, "penalty", torch.float32)
    rows, vocab = logits.shape
    code = _lib().oxr_repetition_penalty(logits.data_ptr(), seen.data_ptr(), row_slot.data_ptr(), penalty.data_ptr(), rows,
                                         vocab, _stream())
    _done(code, "repetition_penalty")


def mark_seen(seen: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor) -> None:
    """``seen[slots[i], tokens[i]] = 1``."""
    _need(seen, "seen", torch.uint8)
    _need(slots, "slots", torch.int32)
    _need(tokens, "tokens", torch.int32)
    code = _lib().oxr_mark_seen(seen.data_ptr(), slots.data_ptr(), tokens.data_ptr(), tokens.numel(), seen.shape[1], _stream())
    _done(code, "mark_seen")
