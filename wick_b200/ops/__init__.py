"""The kernels, as Python functions over CUDA tensors.

Every function checks its arguments (device, dtype, shape, contiguity), passes
raw pointers and the current CUDA stream to an exported C function of one of
the libraries built from ``wick_b200/csrc``, and raises :class:`KernelError`
with the library's message if the call is refused.  There is no fallback of
any kind: without a CUDA device or without ``nvcc`` these functions raise.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from .build import BuildError, load_library

from ..layout import PAGE


class KernelError(RuntimeError):
    pass


_CT = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_int64, "f": ctypes.c_float}

# Argument kinds of an exported function: p pointer, i int32, l int64, f float; the
# last pointer is always the stream.


def _dt(t: torch.Tensor) -> str:
    if t.dtype == torch.bfloat16:
        return "bf16"
    if t.dtype == torch.float32:
        return "f32"
    raise KernelError(f"unsupported element type {t.dtype} (bfloat16 and float32 are built)")


class _Lib:
    """A loaded library with lazily configured functions."""

    def __init__(self, name, sources, defines=()):
        self._lib = load_library(name, sources, defines)
        self._fns: Dict[str, object] = {}
        self._lib.wick_page_size.restype = ctypes.c_int
        built_for = int(self._lib.wick_page_size())
        if built_for != PAGE:
            raise KernelError(f"{name} was built for cache pages of {built_for} positions, the package uses {PAGE}")

    def fn(self, name: str, sig: str):
        f = self._fns.get(name)
        if f is None:
            try:
                f = getattr(self._lib, name)
            except AttributeError:
                raise KernelError(f"{name} is not exported by {self._lib._name}") from None
            f.argtypes = [_CT[c] for c in sig]
            f.restype = ctypes.c_int
            self._fns[name] = f
        return f

    def call(self, name: str, sig: str, *args, kernels: int = 1):
        rc = self.fn(name, sig)(*args)
        if rc != 0:
            raise KernelError(self._lib.wick_last_error().decode("utf-8", "replace"))
        launches[0] += kernels


_libs: Dict[str, _Lib] = {}

# Kernels launched through this module so far (a captured step counts them once,
# at capture; the engine adds them again at every replay).
launches = [0]

# WICK_B200_PLAIN=1 (or PLAIN_KERNELS = True): every matrix product and every attention runs
# through its plain CUDA-core twin (float32 accumulation, no tensor cores, no bulk copies),
# whatever the compute dtype: the slow form that the fast kernels are held against, for
# telling a kernel's fault from a model's.
PLAIN_KERNELS = os.environ.get("WICK_B200_PLAIN", "") not in ("", "0")


def plain_kernels() -> bool:
    return PLAIN_KERNELS


CORE_SOURCES = ["core.cu", "sample.cu", "state.cu"]


def _core() -> _Lib:
    lib = _libs.get("core")
    if lib is None:
        lib = _libs["core"] = _Lib("wick_core", CORE_SOURCES)
    return lib


def _simt() -> _Lib:
    lib = _libs.get("simt")
    if lib is None:
        lib = _libs["simt"] = _Lib("wick_gemm_simt", ["gemm_simt.cu"])
    return lib


ATTN_SOURCES = ["attn.cu", "attn_decode.cu", "attn_decode_parts.cu", "attn_prompt_mma.cu", "attn_prompt_tc.cu"]


def _attn(head_dim: int) -> _Lib:
    key = f"attn{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
            raise KernelError(f"attention kernels take a head_dim that is a multiple of 16 between 16 and 256, "
                              f"not {head_dim}")
        # WICK_B200_ATTN_DEFINES: further -D definitions for experiments (e.g. "WICK_DECODE_WARPS=4,WICK_DECODE_TILES=3")
        more = [d for d in os.environ.get("WICK_B200_ATTN_DEFINES", "").split(",") if d]
        lib = _libs[key] = _Lib(f"wick_attn_hd{head_dim}", ATTN_SOURCES, [f"WICK_HD={head_dim}"] + more)
    return lib


# One device word that kernels write a code to when a bounded wait gives up or an index they
# were given lies outside its table.
_status: Optional[torch.Tensor] = None
_STATUS_TEXT = {1: "gemm_tc gave up waiting for a free shared-memory stage", 2: "gemm_tc gave up waiting for a TMA copy",
                3: "gemm_tc gave up waiting for the accumulator", 4: "attention decode gave up waiting for its bulk copies",
                5: "gemm_tc gave up waiting for a free accumulator",
                7: "attention (tcgen05) gave up waiting for a copy or an accumulator",
                8: "attention decode (tensor cores) gave up waiting for its TMA copies",
                10: "attention decode was given a length or a page outside its page table or its cache",
                99: "the test kernel gave up waiting for nothing (nobody arrives on its barrier)"}


def status_tensor(device) -> torch.Tensor:
    global _status
    if _status is None or _status.device != torch.device(device):
        _status = torch.zeros(1, dtype=torch.int32, device=device)
    return _status


def check_status() -> None:
    """Raise if a kernel gave up a bounded wait (this synchronises the device)."""
    if _status is not None:
        code = int(_status.item())
        if code != 0:
            _status.zero_()
            raise KernelError(f"a kernel reported a fault: {_STATUS_TEXT.get(code, 'code %d' % code)}; its output is invalid")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_scope_stream: List[Optional[int]] = [None]


@contextlib.contextmanager
def stream_scope():
    """Inside the scope every kernel of this module goes to the stream that is
    current at entry.  (Asked once: torch's lookup of the current stream costs as
    much host time as a launch, and a short prompt's step is bound by the host.)"""
    before = _scope_stream[0]
    _scope_stream[0] = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _scope_stream[0] = before


def _stream() -> int:
    s = _scope_stream[0]
    return torch.cuda.current_stream().cuda_stream if s is None else s


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(name: str, t: torch.Tensor, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the kernels have no CPU form)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, has {tuple(t.shape)}")


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [n, width] rows of ``table`` [vocab, width] at int32 ``tokens`` [n]."""
    _cuda("table", table)
    _cuda("tokens", tokens, torch.int32)
    n, (vocab, width) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    _cuda("out", out, torch.float32, (n, width))
    _core().call(f"wick_embed_{_dt(table)}", "pppiilp", _p(table), _p(tokens), _p(out), n, width, vocab, _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, *,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norm of float32 ``x`` [n, width] into ``out_dtype``.

    delta: float32 [splits, n, width]; added to ``x`` (in index order) before the norm,
    and, when every row is normalised, in place.  rows: int32 indices (a row may be named
    more than once); only those rows are normalised, the result has len(rows) rows, and
    ``x`` itself is left as it was."""
    _cuda("x", x, torch.float32)
    n, width = x.shape
    _cuda("weight", weight, torch.float32, (width,))
    splits = 0
    if delta is not None:
        _cuda("delta", delta, torch.float32)
        _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (n, width),
              f"delta must be [splits, {n}, {width}], is {tuple(delta.shape)}")
        splits = delta.shape[0]
    if rows is not None:
        _cuda("rows", rows, torch.int32)
    n_out = n if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    _cuda("out", out, out_dtype, (n_out, width))
    _core().call(f"wick_rmsnorm_{_dt(out)}", "ppilpfppiip", _p(x), _p(delta), splits, n, _p(weight), float(eps),
                 _p(rows), _p(out), n_out, width, _stream())
    return out


def add_delta(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta[0] + delta[1] + ... in place (float32)."""
    _cuda("x", x, torch.float32)
    _cuda("delta", delta, torch.float32)
    _need(delta.dim() == 3 and tuple(delta.shape[1:]) == tuple(x.shape), "delta must be [splits, *x.shape]")
    _core().call("wick_add_delta", "ppilp", _p(x), _p(delta), delta.shape[0], x.numel(), _stream())
    return x


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, amplitude: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of ``positions[t] * inv_freq[i]`` (float32 product), each [n, half], times ``amplitude``."""
    _cuda("positions", positions, torch.int32)
    _cuda("inv_freq", inv_freq, torch.float32)
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _core().call("wick_rope_table", "ppppiifp", _p(positions), _p(inv_freq), _p(cos), _p(sin), n, half, float(amplitude), _stream())
    return cos, sin


def qk_norm_rope_append(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, *,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv: Optional[torch.Tensor],
                        page_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor,
                        write_kv: bool = True, q_out: Optional[torch.Tensor] = None,
                        dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Per-head RMS norm of q and k (if weights are given), half-split rotation
    (if tables are given), then q -> ``q_out`` [n, n_heads, head_dim] and k, v ->
    the cache ``kv`` [pages, 2, n_kv, 64, head_dim] at each token's position.

    qkv: [n, (n_heads + 2 n_kv) head_dim] in the activation dtype, or float32
    partial sums [splits, n, ...] (then ``dtype`` names the activation dtype)."""
    _cuda("qkv", qkv)
    width = (n_heads + 2 * n_kv) * head_dim
    parts = qkv.dim() == 3
    if parts:
        _need(qkv.dtype == torch.float32 and qkv.shape[2] == width and dtype is not None,
              f"partial sums must be float32 [splits, n, {width}] and come with the activation dtype")
        n, splits, act = qkv.shape[1], qkv.shape[0], dtype
    else:
        _need(qkv.dim() == 2 and qkv.shape[1] == width, f"qkv must be [n, {width}], is {tuple(qkv.shape)}")
        n, splits, act = qkv.shape[0], 0, qkv.dtype
    for nm, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _cuda(nm, w, torch.float32, (head_dim,))
    _need((q_weight is None) == (k_weight is None), "q and k norm weights come together")
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, head_dim // 2))
        _cuda("sin", sin, torch.float32, (n, head_dim // 2))
    if write_kv:
        _cuda("kv", kv, act)
        _need(kv.dim() == 5 and tuple(kv.shape[1:]) == (2, n_kv, PAGE, head_dim),
              f"kv must be [pages, 2, {n_kv}, {PAGE}, {head_dim}], is {tuple(kv.shape)}")
    _cuda("page_table", page_table, torch.int32)
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _cuda("positions", positions, torch.int32, (n,))
    if q_out is None:
        q_out = torch.empty((n, n_heads, head_dim), dtype=act, device=qkv.device)
    _cuda("q_out", q_out, act, (n, n_heads, head_dim))
    _core().call(f"wick_qk_norm_rope_append_{_dt(q_out)}", "ppiiiiippfpppppippip",
                 None if parts else _p(qkv), _p(qkv) if parts else None, splits, n, n_heads, n_kv, head_dim,
                 _p(q_weight), _p(k_weight), float(eps), _p(cos), _p(sin), _p(q_out), _p(kv) if write_kv else None,
                 _p(page_table), page_table.shape[-1], _p(seq_of_token), _p(positions), 1 if write_kv else 0,
                 _stream())
    return q_out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    _cuda("gate", gate)
    _cuda("up", up, gate.dtype, gate.shape)
    out = torch.empty_like(gate)
    _core().call(f"wick_silu_mul_{_dt(gate)}", "ppplp", _p(gate), _p(up), _p(out), gate.numel(), _stream())
    return out


# ---------------------------------------------------------------------------
def gemm_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, *, gated: bool = False,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [m, k] times w [n, k] transposed on the CUDA cores, float32 accumulation.
    gated: w is [2n, k] (gate rows, then up rows); returns silu(x gate^T) * (x up^T)."""
    _cuda("x", x)
    _cuda("w", w, x.dtype)
    m, k = x.shape
    _need(w.dim() == 2 and w.shape[1] == k, f"w must be [n, {k}], is {tuple(w.shape)}")
    n = w.shape[0] // 2 if gated else w.shape[0]
    if gated:
        _need(w.shape[0] % 2 == 0, "gated weight needs an even number of rows")
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _cuda("out", out, out_dtype, (m, n))
    name = f"wick_gemm_simt_{_dt(x)}_{_dt(out)}" + ("_gated" if gated else "")
    if name not in ("wick_gemm_simt_bf16_bf16", "wick_gemm_simt_bf16_f32", "wick_gemm_simt_f32_f32",
                    "wick_gemm_simt_bf16_bf16_gated", "wick_gemm_simt_f32_f32_gated"):
        raise KernelError(f"no matrix product from {x.dtype} to {out_dtype}" + (" (gated)" if gated else ""))
    _simt().call(name, "pppiiip", _p(x), _p(w), _p(out), m, n, k, _stream())
    return out


# ---------------------------------------------------------------------------
Q_TILE = 64         # query rows per work item of the prompt attention kernels


def attention_tiles(batch) -> int:
    """How many work items the prompt attention kernels cut this step into: one per 64 new
    tokens of a sequence, numbered sequence by sequence (a kernel finds its item's sequence
    and first row from the step's ``cu_seqlens``)."""
    if getattr(batch, "q_tiles", None) is not None:
        return batch.q_tiles                 # (a captured step: the most there can be; a kernel skips items beyond the last)
    return sum((q + Q_TILE - 1) // Q_TILE for q in batch.q_lens)


def attention_prompt_kind(head_dim: int, dtype: torch.dtype, plain: bool = False) -> str:
    """Which prompt kernel runs: ``tc`` (tcgen05: bfloat16, head sizes 64 and 128),
    ``mma`` (mma.sync: bfloat16, other head sizes up to 128) or ``plain`` (CUDA
    cores: float32, larger heads, and the twin the others are checked against)."""
    if plain or PLAIN_KERNELS or dtype != torch.bfloat16 or head_dim > 128:
        return "plain"
    return "tc" if head_dim in (64, 128) else "mma"


def attention_prompt(q: torch.Tensor, kv: torch.Tensor, batch, scale: float,
                     out: Optional[torch.Tensor] = None, plain: bool = False, kind: Optional[str] = None) -> torch.Tensor:
    """Causal attention of the step's new tokens over the cache (which already
    holds their keys and values).  q: [n, heads, d]; kv: [pages, 2, kv_heads, 64, d].
    ``kind`` (see :func:`attention_prompt_kind`) picks a kernel by hand."""
    _cuda("q", q)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, q.dtype)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_tokens, f"q has {n} rows, the batch {batch.n_tokens} tokens")
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, q.dtype, q.shape)
    kind = kind or attention_prompt_kind(hd, q.dtype, plain)
    _need(kind == "plain" or q.dtype == torch.bfloat16, "the tensor-core attention kernels take bfloat16")
    n_tiles = attention_tiles(batch)
    if kind == "tc":
        _attn(hd).call("wick_attn_prompt_tc_bf16", "plplpipippiiifpp", _p(q), n, _p(kv), kv.shape[0], _p(out),
                       n_tiles, _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start),
                       _p(batch.page_table), batch.table_width, n_heads, n_kv, float(scale),
                       _p(status_tensor(q.device)), _stream())
        return out
    _attn(hd).call("wick_attn_prompt_mma_bf16" if kind == "mma" else f"wick_attn_prompt_{_dt(q)}", "pppipippiiifp",
                   _p(q), _p(kv), _p(out), n_tiles, _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start), _p(batch.page_table),
                   batch.table_width, n_heads, n_kv, float(scale), _stream())
    return out


_decode_split: Dict[tuple, int] = {}


def attention_decode_kind(head_dim: int, dtype: torch.dtype, plain: bool = False) -> str:
    """Which of the CUDA-core decode kernels :func:`attention_decode` runs: ``fast`` (from
    bulk-copied page tiles) or ``plain``.  (The tensor-core decode attention, bfloat16 at head
    sizes 64 and 128, is :func:`attention_decode_parts`.)"""
    return "plain" if plain or PLAIN_KERNELS else "fast"


def attention_decode_split(head_dim: int, dtype: torch.dtype, plain: bool = False) -> int:
    """Cached positions handled by one block of the decode kernel."""
    kind = attention_decode_kind(head_dim, dtype, plain)
    key = (head_dim, dtype, kind)
    v = _decode_split.get(key)
    if v is None:
        lib = _attn(head_dim)._lib
        name = {"plain": "wick_attn_decode_plain_split",
                "fast": f"wick_attn_decode_split_{'bf16' if dtype == torch.bfloat16 else 'f32'}"}[kind]
        f = getattr(lib, name)
        f.restype = ctypes.c_int
        f.argtypes = []
        v = _decode_split[key] = int(f())
    return v


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, max_kv_len: int,
                                    dtype: torch.dtype = torch.bfloat16, plain: bool = False) -> int:
    split = attention_decode_split(head_dim, dtype, plain)
    return n_seqs * n_heads * max(1, -(-max_kv_len // split)) * (head_dim + 2)


def attention_decode(q: torch.Tensor, kv: torch.Tensor, batch, scale: float, scratch: torch.Tensor,
                     out: Optional[torch.Tensor] = None, max_kv_len: Optional[int] = None,
                     plain: bool = False) -> torch.Tensor:
    """One new token per sequence, on the CUDA cores (float32, and bfloat16 at head sizes the
    tensor-core kernel does not take).  scratch: float32, at least
    :func:`attention_decode_scratch_floats` elements; it holds the per-split partial results
    between the two kernels.  plain: the form without shared-memory staging."""
    _cuda("q", q)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, q.dtype)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_seqs, f"decode attention takes one token per sequence: {n} rows, {batch.n_seqs} sequences")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, q.dtype, q.shape)
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    kind = attention_decode_kind(hd, q.dtype, plain)
    if kind == "plain":
        _attn(hd).call(f"wick_attn_decode_plain_{_dt(q)}", "pppplpiipiiifp", _p(q), _p(kv), _p(out),
                       _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table),
                       batch.table_width, n_heads, n_kv, float(scale), _stream(), kernels=2)
    else:
        _attn(hd).call(f"wick_attn_decode_{_dt(q)}", "pppplpiipiiifpp", _p(q), _p(kv), _p(out),
                       _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table),
                       batch.table_width, n_heads, n_kv, float(scale), _p(status_tensor(q.device)), _stream(),
                       kernels=2)
    return out


def attention_decode_parts_supported(n_seqs: int, n_heads: int, n_kv: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core decode attention whose work is cut by each sequence's own
    length takes this problem: bfloat16, head size 64 or 128, at most 8 query heads per kv head."""
    if dtype != torch.bfloat16 or head_dim not in (64, 128) or n_kv <= 0 or n_heads % n_kv != 0 or n_heads // n_kv > 8:
        return False
    return n_seqs <= 2048


def attention_decode_parts_scratch(n_seqs: int, n_heads: int, n_kv: int, head_dim: int, max_kv_len: int) -> int:
    """float32 words of scratch that :func:`attention_decode_parts` needs."""
    f = _attn(head_dim)._lib.wick_attn_decode_parts_scratch
    f.restype = ctypes.c_longlong
    f.argtypes = [ctypes.c_int] * 4
    return int(f(n_seqs, n_heads, n_kv, max_kv_len))


def attention_decode_parts(q: torch.Tensor, kv: torch.Tensor, batch, scale: float, scratch: torch.Tensor,
                           out: Optional[torch.Tensor] = None, max_kv_len: Optional[int] = None) -> torch.Tensor:
    """One new token per sequence over the cache (which already holds its key and value).
    q: bfloat16 [n, heads, d].  scratch: float32, at least
    :func:`attention_decode_parts_scratch` words.  How a sequence's positions are cut into
    parts, and the order in which the parts are merged, depend on its own length only."""
    _cuda("q", q, torch.bfloat16)
    n, n_heads, hd = q.shape
    _cuda("kv", kv, torch.bfloat16)
    _need(kv.dim() == 5 and kv.shape[1] == 2 and kv.shape[3] == PAGE and kv.shape[4] == hd,
          f"kv must be [pages, 2, kv_heads, {PAGE}, {hd}], is {tuple(kv.shape)}")
    n_kv = kv.shape[2]
    _need(n == batch.n_seqs, f"decode attention takes one token per sequence: {n} rows, {batch.n_seqs} sequences")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty_like(q)
    _cuda("out", out, torch.bfloat16, q.shape)
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    _attn(hd).call("wick_attn_decode_parts_bf16", "pplpplpiipiiifpp", _p(q), _p(kv), kv.shape[0], _p(out), _p(scratch),
                   scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table), batch.table_width,
                   n_heads, n_kv, float(scale), _p(status_tensor(q.device)), _stream(), kernels=2 if mk > 128 else 1)
    return out


def attention_decode_parts_fused(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, *,
                                 q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], kv: torch.Tensor, batch,
                                 scale: float, scratch: torch.Tensor, write_kv: bool = True,
                                 max_kv_len: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`attention_decode_parts` from the projection's float32 partial sums ``qkv``
    [splits, n, (n_heads + 2 n_kv) head_dim]: per-head norm of q and k, rotation, the new key
    and value into the cache (unless ``write_kv`` is False), attention, merge — two launches."""
    _cuda("qkv", qkv, torch.float32)
    width = (n_heads + 2 * n_kv) * head_dim
    n = batch.n_seqs
    _need(qkv.dim() == 3 and tuple(qkv.shape[1:]) == (n, width), f"qkv must be [splits, {n}, {width}], is {tuple(qkv.shape)}")
    for nm, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _cuda(nm, w, torch.float32, (head_dim,))
    _need((q_weight is None) == (k_weight is None), "q and k norm weights come together")
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, head_dim // 2))
        _cuda("sin", sin, torch.float32, (n, head_dim // 2))
    _cuda("kv", kv, torch.bfloat16)
    _need(kv.dim() == 5 and tuple(kv.shape[1:]) == (2, n_kv, PAGE, head_dim),
          f"kv must be [pages, 2, {n_kv}, {PAGE}, {head_dim}], is {tuple(kv.shape)}")
    _cuda("scratch", scratch, torch.float32)
    if out is None:
        out = torch.empty((n, n_heads, head_dim), dtype=torch.bfloat16, device=qkv.device)
    _cuda("out", out, torch.bfloat16, (n, n_heads, head_dim))
    mk = batch.max_kv_len if max_kv_len is None else max_kv_len
    _attn(head_dim).call("wick_attn_decode_parts_fused_bf16", "pippfppiplpplpiipiiifpp", _p(qkv), qkv.shape[0], _p(q_weight),
                         _p(k_weight), float(eps), _p(cos), _p(sin), 1 if write_kv else 0, _p(kv), kv.shape[0], _p(out),
                         _p(scratch), scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table), batch.table_width,
                         n_heads, n_kv, float(scale), _p(status_tensor(qkv.device)), _stream(), kernels=2 if mk > 128 else 1)
    return out


# ---------------------------------------------------------------------------
# Mechanisms of layers beyond the plain pre-norm decoder: the norm after the residual sum, a
# feed-forward's squared ReLU, the soft cap of logits, attention with options (csrc/attn_masked.cu)
# and experts chosen by a table (csrc/moe.cu).
LAYER_SOURCES = ["layer_ops.cu", "attn_masked.cu", "attn_multi.cu", "moe.cu", "ssm.cu", "gla.cu"]

MASKS = {"causal": 0, "block": 1, "window": 2}
PAIRINGS = {"neighbours": 0, "halves": 1}


def _layer() -> _Lib:
    lib = _libs.get("layer")
    if lib is None:
        lib = _libs["layer"] = _Lib("wick_layer", LAYER_SOURCES)
    return lib


def scaled_add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], alpha: float, weight: torch.Tensor, eps: float,
                       out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """x <- rms(alpha * x + delta[0] + delta[1] + ...) * weight, in place (float32 [n, width]).
    Returns the same rows in ``out_dtype``; for float32 that is ``x`` itself."""
    _cuda("x", x, torch.float32)
    n, width = x.shape
    _cuda("weight", weight, torch.float32, (width,))
    splits = 0
    if delta is not None:
        _cuda("delta", delta, torch.float32)
        _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (n, width),
              f"delta must be [splits, {n}, {width}], is {tuple(delta.shape)}")
        splits = delta.shape[0]
    out = None if out_dtype == torch.float32 else torch.empty((n, width), dtype=out_dtype, device=x.device)
    name = "wick_scaled_add_rmsnorm_f32" if out is None else f"wick_scaled_add_rmsnorm_{_dt(out)}"
    _layer().call(name, "ppifpfpiip", _p(x), _p(delta), splits, float(alpha), _p(weight), float(eps), _p(out), n, width,
                  _stream())
    return x if out is None else out


def relu_squared_(a: torch.Tensor) -> torch.Tensor:
    """a <- max(a, 0)^2 in place."""
    _cuda("a", a)
    _layer().call(f"wick_relu_squared_{_dt(a)}", "plp", _p(a), a.numel(), _stream())
    return a


def soft_cap_(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z <- cap * tanh(z / cap) in place (float32)."""
    _cuda("z", z, torch.float32)
    _layer().call("wick_soft_cap", "plfp", _p(z), z.numel(), float(cap), _stream())
    return z


def to_activation(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """float32 -> the activation type (float32: ``x`` itself)."""
    _cuda("x", x, torch.float32)
    if dtype == torch.float32:
        return x
    _need(dtype == torch.bfloat16, f"no conversion to {dtype}")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _layer().call("wick_to_activation_bf16", "pplp", _p(x), _p(out), x.numel(), _stream())
    return out


def _kv_pages(name: str, kv: torch.Tensor, dtype, n_kv: int, d: int, e: int) -> None:
    _cuda(name, kv, dtype)
    per_page = n_kv * PAGE * (d + e)
    _need(kv.dim() >= 2 and kv[0].numel() == per_page,
          f"{name} must hold pages of {n_kv} x {PAGE} x ({d} + {e}) elements, is {tuple(kv.shape)}")


def stream_update(x: torch.Tensor, delta: Optional[torch.Tensor], *, scale: Optional[torch.Tensor] = None,
                  rms: Optional[Tuple[torch.Tensor, float]] = None, norm: Optional[tuple] = None,
                  out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The residual stream's own kernel.  ``x`` (float32 [n, width]) <- x + f(delta[0] + delta[1] + ...), in place:
    f divides the sum by its root mean square and multiplies it by a weight (``rms`` = (weight, eps)), then
    multiplies it by ``scale`` (float32 [width]), each where given.  With ``out_dtype`` the new rows also go out in
    that type: after the norm ``("tanh", alpha, w, b)`` (tanh(alpha x) * w + b) or ``("rms", w, eps)``
    (x / sqrt(mean(x^2) + eps) * w) if ``norm`` is given, else as they are (for float32 that is ``x`` itself).  ``rows`` (int32 indices, a row may be named twice): only those rows go
    out, and ``x`` itself is left as it was."""
    _cuda("x", x, torch.float32)
    n, width = x.shape
    splits = 0
    if delta is not None:
        _cuda("delta", delta, torch.float32)
        _need(delta.dim() == 3 and tuple(delta.shape[1:]) == (n, width),
              f"delta must be [splits, {n}, {width}], is {tuple(delta.shape)}")
        splits = delta.shape[0]
    if scale is not None:
        _cuda("scale", scale, torch.float32, (width,))
    rms_w, rms_eps = (None, 0.0) if rms is None else rms
    if rms_w is not None:
        _cuda("rms weight", rms_w, torch.float32, (width,))
    alpha = w = b = None
    out_eps = 0.0
    if norm is not None:
        _need(norm[0] in ("tanh", "rms") and out_dtype is not None,
              "the stream kernel knows the tanh norm and the norm by the root mean square, and a norm has a result type")
        if norm[0] == "tanh":
            _, alpha, w, b = norm
            _cuda("alpha", alpha, torch.float32, (1,))
            _cuda("b", b, torch.float32, (width,))
        else:
            _, w, out_eps = norm
        _cuda("w", w, torch.float32, (width,))
    if rows is not None:
        _cuda("rows", rows, torch.int32)
    n_out = n if rows is None else rows.numel()
    out = None
    if out_dtype is not None and not (norm is None and rows is None and out_dtype == torch.float32):
        out = torch.empty((n_out, width), dtype=out_dtype, device=x.device)
    if delta is None and out is None:
        return x if out_dtype is not None else None
    name = f"wick_stream_update_{_dt(out)}" if out is not None else "wick_stream_update_f32"
    _layer().call(name, "ppippfpppfppiiip", _p(x), _p(delta), splits, _p(scale), _p(rms_w), float(rms_eps),
                  _p(alpha), _p(w), _p(b), float(out_eps), _p(rows), _p(out), n, n_out, width, _stream())
    if out is not None:
        return out
    return x if out_dtype is not None else None


def gelu_gate_rows(z: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, offset: int, dtype: torch.dtype) -> torch.Tensor:
    """gelu(z[t, j]) * table[tokens[t], offset + j] in ``dtype``; gelu in its tanh form, float32.  z: float32 [n, dim]."""
    _cuda("z", z, torch.float32)
    _cuda("table", table, dtype)
    _cuda("tokens", tokens, torch.int32)
    n, dim = z.shape
    _need(table.dim() == 2 and 0 <= offset and offset + dim <= table.shape[1], f"the table has no columns {offset} .. {offset + dim}")
    _need(tokens.numel() == n, f"{n} rows and {tokens.numel()} tokens")
    out = torch.empty((n, dim), dtype=dtype, device=z.device)
    _layer().call(f"wick_gelu_gate_rows_{_dt(out)}", "pppplilip", _p(z), _p(table), _p(tokens), _p(out), n, dim, table.shape[1],
                  int(offset), _stream())
    return out


ATTN_MULTI_MAX_V = 512      # the most numbers of a value row that attention_multi accumulates


def attention_multi(q: torch.Tensor, store: torch.Tensor, batch, scale: float, *, maps: int, kv_heads: int, v_dim: int,
                    window: int = 0, keep_first: int = 0, sink: Optional[torch.Tensor] = None,
                    combine: Optional[Tuple[float, float, float]] = None, rows_of: Optional[int] = None,
                    out_dtype: torch.dtype) -> torch.Tensor:
    """Attention of the step's tokens over the cache (which already holds their own rows) with ``maps`` score maps
    a head.  q: [n, H, maps * dm]; map a scores the a-th dm numbers of a key row and has a softmax of its own; all
    maps weigh the same values.  Visible to the query at position p: with ``window`` > 0 the keys j <= p with
    p - j < window or j < ``keep_first``, else every j <= p.  ``sink``: float32 [H], joins every map's denominator.

    Two layouts of ``store``: pages of keys and values ([kv_heads][64][maps * dm] keys, then [kv_heads][64][v_dim]
    values), or, with ``rows_of`` = R, pages of [64][R] rows whose first ``v_dim`` numbers are also the value
    (one key head; maps * dm = R).

    maps = 2 with ``combine`` = (lambda, eps, factor): the result is y = y_1 - lambda y_2, then
    y / sqrt(mean(y^2) + eps) * factor over a head's values; q in the activation type.  maps = 1: q is float32 and
    so is the result.  Returns [n, H, v_dim] in ``out_dtype``."""
    _cuda("q", q)
    n, H, d = q.shape
    _need(maps in (1, 2) and d % maps == 0, f"a head of {d} numbers is not {maps} maps")
    _need(n == batch.n_tokens, f"q has {n} rows, the batch {batch.n_tokens} tokens")
    dm = d // maps
    _cuda("store", store)
    T = store.dtype
    if rows_of is not None:
        _need(kv_heads == 1 and d == rows_of and v_dim <= rows_of and store[0].numel() == PAGE * rows_of,
              f"store must hold pages of {PAGE} rows of {rows_of} numbers, is {tuple(store.shape)}")
        page_elems, k_row, v_off, v_row = PAGE * rows_of, rows_of, 0, rows_of
    else:
        _kv_pages("store", store, T, kv_heads, d, v_dim)
        page_elems, k_row, v_off, v_row = kv_heads * PAGE * (d + v_dim), d, kv_heads * PAGE * d, v_dim
    _need(v_dim <= ATTN_MULTI_MAX_V, f"values of {v_dim} numbers are beyond {ATTN_MULTI_MAX_V}")
    if sink is not None:
        _cuda("sink", sink, torch.float32, (H,))
    if maps == 2:
        _need(combine is not None and q.dtype == T and out_dtype == T, "two maps are combined, in the activation type")
        name = f"wick_attn_multi2_{_dt(q)}"
        lam, eps, factor = combine
    else:
        _need(q.dtype == torch.float32 and out_dtype == torch.float32, "one map takes and gives float32")
        name = f"wick_attn_multi1_{'bf16' if T == torch.bfloat16 else 'f32'}"
        lam, eps, factor = 0.0, 0.0, 1.0
    out = torch.empty((n, H, v_dim), dtype=out_dtype, device=q.device)
    # A step of few tokens: eight warps a block, heads that read the same rows together, and the visible keys cut into
    # runs (a block each, records merged by a second kernel) until the step fills the device about twice.  How many keys
    # a token can see at most is known from the window or from the step's bound on cached positions.
    few = 1 if (batch.is_decode or n * H <= 8 * 148) else 0
    runs, partial = 1, None
    if few:
        group = 1 if maps == 2 else (4 if (H // kv_heads) % 4 == 0 else (2 if (H // kv_heads) % 2 == 0 else 1))
        bound = getattr(batch, "kv_bound", None) or batch.max_kv_len
        keys = min(bound, window + keep_first) if window > 0 else bound
        tiles = (max(1, keys) + 31) // 32
        runs = max(1, min(-(-2 * 148 // (n * (H // group))), tiles // 2, 16))        # (a run is two tiles of 32 keys at least)
        if runs > 1:
            need = n * H * maps * runs * (4 + (v_dim + 127) // 128 * 128)
            ws = getattr(batch, "workspace", None)
            partial = ws.get("attention_multi", need, torch.float32) if ws is not None else \
                torch.empty(need, dtype=torch.float32, device=q.device)
    _layer().call(name, "ppppppiiiiiililifiipfffiipp", _p(q), _p(store), _p(out), _p(batch.seq_of_token), _p(batch.positions),
                  _p(batch.page_table), batch.table_width, n, H, kv_heads, dm, v_dim, page_elems, k_row, v_off, v_row, float(scale),
                  int(window), int(keep_first), _p(sink), float(lam), float(eps), float(factor), few, runs, _p(partial), _stream(),
                  kernels=2 if partial is not None else 1)
    return out


def latent_finish(parts: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, gate_heads: int, *, dtype: torch.dtype,
                  q_weight: torch.Tensor, kv_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], pairing: str = "neighbours", rows: Optional[torch.Tensor],
                  page_table: torch.Tensor, seq_of_token: torch.Tensor, positions: torch.Tensor, flat: bool = False):
    """From the float32 partial sums ``parts`` [splits, n, q_rank + kv_rank + rot_dim + gate_heads] of a latent
    attention's down-projections: the query latent rms(.) * q_weight -> [n, q_rank] in ``dtype``; the latent
    rms(.) * kv_weight and the key part, turned by the angles of ``cos`` / ``sin`` [n, rot_dim / 2], -> the token's
    row of ``rows`` (pages of [64][kv_rank + rot_dim]; None: nothing is stored); sigmoid of the gates -> float32
    [n, gate_heads] (None if there are none).  Returns (query latent, gates); with ``flat`` (and ``rows``) also the step's
    own latents [n, kv_rank] and key parts [n, rot_dim] as arrays of their own, in ``dtype``."""
    _cuda("parts", parts, torch.float32)
    W = q_rank + kv_rank + rot_dim + gate_heads
    _need(parts.dim() == 3 and parts.shape[2] == W, f"parts must be [splits, n, {W}], is {tuple(parts.shape)}")
    n = parts.shape[1]
    _cuda("q_weight", q_weight, torch.float32, (q_rank,))
    if kv_weight is not None:
        _cuda("kv_weight", kv_weight, torch.float32, (kv_rank,))
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, rot_dim // 2) if rot_dim else None)
        _cuda("sin", sin, torch.float32, (n, rot_dim // 2) if rot_dim else None)
    if rows is not None:
        _cuda("rows", rows, dtype)
        _need(rows[0].numel() == PAGE * (kv_rank + rot_dim), f"rows must hold pages of {PAGE} x {kv_rank + rot_dim}, is {tuple(rows.shape)}")
    _cuda("page_table", page_table, torch.int32)
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _cuda("positions", positions, torch.int32, (n,))
    cq = torch.empty((n, q_rank), dtype=dtype, device=parts.device)
    gate = torch.empty((n, gate_heads), dtype=torch.float32, device=parts.device) if gate_heads else None
    use_rot = cos is not None and rot_dim > 0
    flat_c = flat_kr = None
    if flat and rows is not None:
        flat_c = torch.empty((n, kv_rank), dtype=dtype, device=parts.device)
        flat_kr = torch.empty((n, rot_dim), dtype=dtype, device=parts.device)
    _layer().call(f"wick_latent_finish_{_dt(cq)}", "piiiiiippfppippppppippp", _p(parts), parts.shape[0], n, q_rank, kv_rank, rot_dim,
                  gate_heads, _p(q_weight), _p(kv_weight), float(eps), _p(cos) if use_rot else None, _p(sin) if use_rot else None,
                  PAIRINGS[pairing], _p(cq), _p(gate), _p(rows), _p(flat_c), _p(flat_kr), _p(page_table), page_table.shape[-1],
                  _p(seq_of_token), _p(positions), _stream())
    if flat:
        return cq, gate, flat_c, flat_kr
    return cq, gate


def latent_query(q_parts: torch.Tensor, heads: int, d: int, rot_dim: int, *, cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], pairing: str = "neighbours", dtype: torch.dtype) -> torch.Tensor:
    """A latent attention's queries as they are: the float32 partial sums [splits, n, heads * (d + rot_dim)] added up, the
    last ``rot_dim`` numbers of every head turned by the angles, in ``dtype`` [n, heads, d + rot_dim]."""
    _cuda("q_parts", q_parts, torch.float32)
    W = heads * (d + rot_dim)
    _need(q_parts.dim() == 3 and q_parts.shape[2] == W, f"q_parts must be [splits, n, {W}], is {tuple(q_parts.shape)}")
    n = q_parts.shape[1]
    use_rot = cos is not None and rot_dim > 0
    if use_rot:
        _cuda("cos", cos, torch.float32, (n, rot_dim // 2))
        _cuda("sin", sin, torch.float32, (n, rot_dim // 2))
    out = torch.empty((n, heads, d + rot_dim), dtype=dtype, device=q_parts.device)
    _layer().call(f"wick_latent_query_{_dt(out)}", "piiiiippipp", _p(q_parts), q_parts.shape[0], n, heads, d, rot_dim,
                  _p(cos) if use_rot else None, _p(sin) if use_rot else None, PAIRINGS[pairing], _p(out), _stream())
    return out


# ---- prompt attention on the tensor cores with keys and values described by strides ---------------------------------
def _flex(dk: int, dv: int) -> _Lib:
    key = f"flex{dk}_{dv}"
    lib = _libs.get(key)
    if lib is None:
        lib = _libs[key] = _Lib(f"wick_attn_flex_k{dk}_v{dv}", ["attn_flex.cu"], [f"WICK_DK={dk}", f"WICK_DV={dv}"])
    return lib


def attention_flex_supported(dk: int, dv: int, dtype: torch.dtype) -> bool:
    """Whether :func:`attention_flex` takes query / key vectors of ``dk`` and values of ``dv`` numbers."""
    return (dtype == torch.bfloat16 and not PLAIN_KERNELS and dk % 16 == 0 and 16 <= dk <= 256 and dv % 16 == 0
            and 16 <= dv <= 128)


def flex_source(t: Optional[torch.Tensor] = None, *, tile_elems: int = 0, const_off: int = 0, hdiv: int = 1, hmul: int = 0,
                hmod: int = 1, hmul2: int = 0, row_stride: int = 0, length: int = 0, paged: bool = False) -> List[int]:
    """Where the rows of one source of :func:`attention_flex` lie.  A tile of 64 keys of sequence b for head h starts at
    ``page_table[b][tile] * tile_elems`` (paged) or at ``(first token of b + 64 tile) * row_stride`` (flat: one row per
    token of the step), plus ``const_off + (h // hdiv) * hmul + (h % hmod) * hmul2``; rows are ``row_stride`` apart and
    give ``length`` numbers.  All in elements of bfloat16."""
    return [0 if t is None else t.data_ptr(), tile_elems, const_off, hdiv, hmul, hmod, hmul2, row_stride, length, 1 if paged else 0]


def attention_flex(q: torch.Tensor, k0: List[int], k1: List[int], v: List[int], batch, scale: float, *, dv: int, window: int = 0,
                   keep_first: int = 0, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Attention of a prompt's tokens on the tensor cores.  q: bfloat16 [n, heads, dk]; a key row is ``k0``'s numbers
    followed by ``k1``'s (sources as :func:`flex_source` makes them; flat sources need sequences that start at position
    0), a value row ``v``'s.  Visible to the query at position p: the keys j <= p with p - j < window or j < keep_first
    (window 0: every j <= p).  ``sink`` float32 [heads]; ``gate`` float32 [n, heads], a factor of the bfloat16 result.
    Returns [n, heads, dv] in ``out_dtype`` (float32 or bfloat16)."""
    import numpy as np
    _cuda("q", q, torch.bfloat16)
    n, heads, dk = q.shape
    _need(n == batch.n_tokens, f"q has {n} rows, the batch {batch.n_tokens} tokens")
    _need(attention_flex_supported(dk, dv, q.dtype), f"no tensor-core attention for vectors of {dk} and values of {dv} numbers")
    if sink is not None:
        _cuda("sink", sink, torch.float32, (heads,))
    if gate is not None:
        _cuda("gate", gate, torch.float32, (n, heads))
        _need(out_dtype == torch.bfloat16, "the gate is a factor of the bfloat16 result")
    out = torch.empty((n, heads, dv), dtype=out_dtype, device=q.device)
    src = np.asarray(k0 + k1 + v, dtype=np.int64)
    _flex(dk, dv).call("wick_attn_flex_bf16", "pppppppippiiiiifp", _p(q), src.ctypes.data, _p(out) if out_dtype == torch.float32 else None,
                       _p(out) if out_dtype == torch.bfloat16 else None, _p(gate), _p(sink), _p(batch.cu_seqlens), batch.n_seqs,
                       _p(batch.start), _p(batch.page_table), batch.table_width, attention_tiles(batch), heads, int(window),
                       int(keep_first), float(scale), _stream())
    return out


def combine_maps(a: torch.Tensor, lam: float, eps: float, factor: float, *, lib: Tuple[int, int]) -> torch.Tensor:
    """a: float32 [n, H, 2, e], two maps' results a head.  Returns bfloat16 [n, H, e]: y = a_1 - lam a_2, then
    y / sqrt(mean(y^2) + eps) * factor over e.  ``lib``: the (dk, dv) of the attention library that made ``a``."""
    _cuda("a", a, torch.float32)
    n, H, two, e = a.shape
    _need(two == 2, "two maps a head")
    out = torch.empty((n, H, e), dtype=torch.bfloat16, device=a.device)
    _flex(*lib).call("wick_combine_maps_bf16", "pplifffp", _p(a), _p(out), n * H, e, float(lam), float(eps),
                     float(factor), _stream())
    return out


def latent_absorb(q_parts: torch.Tensor, uk: torch.Tensor, heads: int, d: int, rot_dim: int, kv_rank: int, *,
                  cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], pairing: str = "neighbours") -> torch.Tensor:
    """A latent attention's queries carried into the space of the cached rows.  ``q_parts``: float32 partial sums
    [splits, n, heads * (d + rot_dim)], a head laid out as [d | rot_dim]; ``uk``: [heads * d, kv_rank].  Returns
    float32 [n, heads, kv_rank + rot_dim]: [Wuk_h^T q_h[:d] | q_h[d:] turned by the angles]."""
    _cuda("q_parts", q_parts, torch.float32)
    W = heads * (d + rot_dim)
    _need(q_parts.dim() == 3 and q_parts.shape[2] == W, f"q_parts must be [splits, n, {W}], is {tuple(q_parts.shape)}")
    n = q_parts.shape[1]
    _cuda("uk", uk, None, (heads * d, kv_rank))
    use_rot = cos is not None and rot_dim > 0
    if use_rot:
        _cuda("cos", cos, torch.float32, (n, rot_dim // 2))
        _cuda("sin", sin, torch.float32, (n, rot_dim // 2))
    out = torch.empty((n, heads, kv_rank + rot_dim), dtype=torch.float32, device=q_parts.device)
    _layer().call(f"wick_latent_absorb_{_dt(uk)}", "pipiiiiippipp", _p(q_parts), q_parts.shape[0], _p(uk), n, heads, d, rot_dim,
                  kv_rank, _p(cos) if use_rot else None, _p(sin) if use_rot else None, PAIRINGS[pairing], _p(out), _stream())
    return out


def latent_expand(y: torch.Tensor, uv: torch.Tensor, gate: Optional[torch.Tensor], heads: int, v_dim: int, kv_rank: int, *,
                  dtype: torch.dtype) -> torch.Tensor:
    """out[t, h] = gate[t, h] * Wuv_h y[t, h].  y: float32 [n, heads, kv_rank] (a head's weighted sum of cached
    latents); ``uv``: [heads * v_dim, kv_rank] in ``dtype``; gate: float32 [n, heads] or None.  Returns [n, heads * v_dim]."""
    _cuda("y", y, torch.float32)
    n = y.shape[0]
    _need(tuple(y.shape) == (n, heads, kv_rank), f"y must be [n, {heads}, {kv_rank}], is {tuple(y.shape)}")
    _cuda("uv", uv, dtype, (heads * v_dim, kv_rank))
    if gate is not None:
        _cuda("gate", gate, torch.float32, (n, heads))
    out = torch.empty((n, heads * v_dim), dtype=dtype, device=y.device)
    _layer().call(f"wick_latent_expand_{_dt(out)}", "pppiiiipp", _p(y), _p(uv), _p(gate), n, heads, v_dim, kv_rank, _p(out), _stream())
    return out



def qkv_finish(parts: torch.Tensor, n_heads: int, n_kv: int, d: int, e: int, *, dtype: torch.dtype,
               bias: Optional[torch.Tensor] = None, q_weight: Optional[torch.Tensor] = None,
               k_weight: Optional[torch.Tensor] = None, eps: float = 0.0, cos: Optional[torch.Tensor] = None,
               sin: Optional[torch.Tensor] = None, rot_dims: int = 0, pairing: str = "neighbours", maps: int = 1,
               v_keep: Optional[torch.Tensor] = None, v_mode: int = 0,
               blend: Optional[torch.Tensor] = None, kv: Optional[torch.Tensor], page_table: torch.Tensor,
               seq_of_token: torch.Tensor, positions: torch.Tensor, write_kv: bool = True,
               q_span: Optional[int] = None, k_span: Optional[int] = None, norm_after_rotation: bool = False,
               keys_are_values: bool = False) -> torch.Tensor:
    """From the q/k/v projection's float32 partial sums ``parts`` [splits, n, H d + G d + G e (+ more)]:
    biases, RMS norms of q and k over spans the length of their weight vectors (a head, or the
    whole projection; ``q_span`` / ``k_span`` without a weight vector: the span is divided by its root
    mean square and no more), rotation of the first ``rot_dims`` elements of every q and k head by the
    angles whose ``cos`` and ``sin`` [n, rot_dims / 2] are given (``pairing``: which two elements
    turn together; ``maps``: a head is that many vectors side by side, each turned on its own;
    ``norm_after_rotation``: the norm follows the rotation), the value blend
    (``v_mode`` 1: the values are also kept in ``v_keep`` [n, G e]; 2: v <- (1 - blend) v + blend
    v_keep), then q -> the result [n, H, d] in ``dtype`` and k, v -> the token's place in ``kv``.
    ``keys_are_values``: the rows hold no values; a head's value is its key as projected, before norm
    and rotation.  Columns behind q, k and v (an output gate's) are left alone."""
    _cuda("parts", parts, torch.float32)
    W = (n_heads + n_kv) * d + (0 if keys_are_values else n_kv * e)
    _need(parts.dim() == 3 and parts.shape[2] >= W, f"parts must be [splits, n, {W} or more], is {tuple(parts.shape)}")
    n, cols = parts.shape[1], parts.shape[2]
    if bias is not None:
        _cuda("bias", bias, torch.float32, (W,))
    if q_weight is not None:
        _cuda("q_weight", q_weight, torch.float32)
        q_span = q_weight.numel()
    if k_weight is not None:
        _cuda("k_weight", k_weight, torch.float32)
        k_span = k_weight.numel()
    if cos is not None:
        _cuda("cos", cos, torch.float32, (n, rot_dims // 2))
        _cuda("sin", sin, torch.float32, (n, rot_dims // 2))
    if v_mode:
        _cuda("v_keep", v_keep, torch.float32, (n, n_kv * e))
    if v_mode == 2:
        _cuda("blend", blend, torch.float32)
        _need(blend.numel() == 1, "the blend factor is one number")
    if write_kv:
        _kv_pages("kv", kv, dtype, n_kv, d, e)
    _cuda("page_table", page_table, torch.int32)
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _cuda("positions", positions, torch.int32, (n,))
    q_out = torch.empty((n, n_heads, d), dtype=dtype, device=parts.device)
    _need(maps >= 1 and d % maps == 0, f"a head of {d} numbers is not {maps} vectors")
    flags = (1 if keys_are_values else 0) | (2 if norm_after_rotation else 0)
    _layer().call(f"wick_qkv_finish_{_dt(q_out)}", "piipiiiipipifppiiipippppippiiip", _p(parts), parts.shape[0], n, _p(bias),
                  n_heads, n_kv, d, e, _p(q_weight), int(q_span or 0), _p(k_weight), int(k_span or 0), float(eps), _p(cos), _p(sin),
                  rot_dims if cos is not None else 0, PAIRINGS[pairing], int(maps), _p(v_keep), v_mode, _p(blend), _p(q_out),
                  _p(kv) if write_kv else None, _p(page_table), page_table.shape[-1], _p(seq_of_token), _p(positions),
                  1 if write_kv else 0, int(cols), flags, _stream())
    return q_out


def gate_rows_(y: torch.Tensor, parts: torch.Tensor, first_col: int) -> torch.Tensor:
    """y[t, j] <- y[t, j] * sigmoid(g[t, j]) in place, g the sum (in index order) of the float32 partial sums
    ``parts`` [splits, n, cols] at the columns from ``first_col`` on; the sigmoid is evaluated in float32."""
    _cuda("y", y)
    _cuda("parts", parts, torch.float32)
    n, width = y.shape[0], y[0].numel()
    _need(parts.dim() == 3 and parts.shape[1] == n and first_col + width <= parts.shape[2],
          f"parts must be [splits, {n}, {first_col + width} or more], is {tuple(parts.shape)}")
    _layer().call(f"wick_gate_rows_{_dt(y)}", "ppiiiiip", _p(y), _p(parts), parts.shape[0], n, width, parts.shape[2], int(first_col),
                  _stream())
    return y


def weighted_sum(terms, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [1, n, width]: f_0 sum(a_0) + f_1 sum(a_1) + ... for ``terms`` = [(a_i float32 [splits_i, n, width], f_i)];
    every a_i's partial sums are added in index order, the terms in the order given.  At most four terms."""
    _need(1 <= len(terms) <= 4, "one to four terms")
    a0 = terms[0][0]
    _cuda("term", a0, torch.float32)
    n, width = a0.shape[1], a0.shape[2]
    ptrs, splits, factors = [], [], []
    for a, f in terms:
        _cuda("term", a, torch.float32)
        _need(a.dim() == 3 and tuple(a.shape[1:]) == (n, width), f"every term must be [splits, {n}, {width}]")
        ptrs.append(_p(a)); splits.append(a.shape[0]); factors.append(float(f))
    while len(ptrs) < 4:
        ptrs.append(None); splits.append(0); factors.append(0.0)
    if out is None:
        out = torch.empty((1, n, width), dtype=torch.float32, device=a0.device)
    _layer().call("wick_weighted_sum", "pifpifpifpifplp", ptrs[0], splits[0], factors[0], ptrs[1], splits[1], factors[1],
                  ptrs[2], splits[2], factors[2], ptrs[3], splits[3], factors[3], _p(out), n * width, _stream())
    return out


def concat_activation(a: torch.Tensor, b: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """[a | b] row by row in ``dtype``: a, b float32 [n, wa], [n, wb] -> [n, wa + wb]."""
    _cuda("a", a, torch.float32)
    _cuda("b", b, torch.float32)
    _need(a.dim() == 2 and b.dim() == 2 and a.shape[0] == b.shape[0], "two matrices of as many rows")
    n, wa, wb = a.shape[0], a.shape[1], b.shape[1]
    out = torch.empty((n, wa + wb), dtype=dtype, device=a.device)
    _layer().call(f"wick_concat_activation_{_dt(out)}", "pppiiip", _p(a), _p(b), _p(out), n, wa, wb, _stream())
    return out


def attention_masked_kind(d: int, v_dim: int, dtype: torch.dtype, is_decode: bool, plain: bool = False) -> str:
    """Which kernel :func:`attention_masked` runs.  With keys and values of one size that is a
    multiple of 16: ``bulk`` for a decode step (one token per sequence: CUDA cores from bulk-copied
    page tiles, the positions split over blocks, both dtypes); for a prompt's tokens in bfloat16
    ``tc`` (tcgen05, sizes 64 and 128) or ``mma`` (mma.sync, other sizes up to 128).  Everything else, and the twin that
    the former are checked against: ``warp`` (CUDA cores straight from the cache)."""
    if plain or PLAIN_KERNELS or d != v_dim or d % 16 != 0 or d > 256:
        return "warp"
    if is_decode:
        return "bulk"
    if dtype != torch.bfloat16 or d > 128:
        return "warp"
    return "tc" if d in (64, 128) else "mma"


def attention_masked(q: torch.Tensor, kv: torch.Tensor, batch, scale: float, *, n_kv: int, v_dim: int,
                     mask: str = "causal", mask_size: int = 0, sink: Optional[torch.Tensor] = None,
                     kind: Optional[str] = None) -> torch.Tensor:
    """Attention of the step's tokens (a prompt's or one per sequence) over the cache, which
    already holds their keys and values.  q: [n, H, d]; result [n, H, v_dim].  ``mask``:
    ``causal`` (every earlier key), ``block`` (earlier keys in the query's own block of
    ``mask_size`` positions, blocks counted from position 0) or ``window`` (the last
    ``mask_size`` positions).  ``sink``: float32 [H], a score per head that joins the
    softmax's denominator without a value.  ``kind`` picks a kernel by hand (see
    :func:`attention_masked_kind`)."""
    _cuda("q", q)
    n, n_heads, d = q.shape
    _kv_pages("kv", kv, q.dtype, n_kv, d, v_dim)
    _need(n == batch.n_tokens, f"q has {n} rows, the batch {batch.n_tokens} tokens")
    if sink is not None:
        _cuda("sink", sink, torch.float32, (n_heads,))
    out = torch.empty((n, n_heads, v_dim), dtype=q.dtype, device=q.device)
    kind = kind or attention_masked_kind(d, v_dim, q.dtype, batch.is_decode)
    if kind == "bulk":
        _need(d == v_dim and batch.is_decode, "the bulk-copy kernel takes one token per sequence and one head size")
        mk = batch.kv_bound
        need = attention_decode_scratch_floats(batch.n_seqs, n_heads, d, mk, q.dtype)
        ws = getattr(batch, "workspace", None)
        scratch = ws.get("attention_decode", need, torch.float32) if ws is not None else \
            torch.empty(need, dtype=torch.float32, device=q.device)
        _attn(d).call(f"wick_attn_decode_masked_{_dt(q)}", "pppplpiipiiifpiipp", _p(q), _p(kv), _p(out), _p(scratch),
                      scratch.numel(), _p(batch.kv_len), n, mk, _p(batch.page_table), batch.table_width, n_heads, n_kv,
                      float(scale), _p(status_tensor(q.device)), MASKS[mask], int(mask_size), _p(sink), _stream(), kernels=2)
        return out
    if kind == "tc":
        _need(q.dtype == torch.bfloat16 and d == v_dim and d in (64, 128), "the tcgen05 kernel takes bfloat16 heads of 64 or 128")
        _attn(d).call("wick_attn_prompt_tc_masked_bf16", "plplpipippiiifpiipp", _p(q), n, _p(kv), kv.shape[0], _p(out),
                      attention_tiles(batch), _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start), _p(batch.page_table),
                      batch.table_width, n_heads, n_kv, float(scale), _p(status_tensor(q.device)), MASKS[mask], int(mask_size),
                      _p(sink), _stream())
        return out
    if kind == "mma":
        _need(q.dtype == torch.bfloat16 and d == v_dim, "the tensor-core kernel takes bfloat16 and one head size")
        _attn(d).call("wick_attn_prompt_mma_masked_bf16", "pppipippiiifiipp", _p(q), _p(kv), _p(out), attention_tiles(batch),
                      _p(batch.cu_seqlens), batch.n_seqs, _p(batch.start), _p(batch.page_table), batch.table_width, n_heads,
                      n_kv, float(scale), MASKS[mask], int(mask_size), _p(sink), _stream())
        return out
    _layer().call(f"wick_attn_masked_{_dt(q)}", "ppppppiiiiiifiipp", _p(q), _p(kv), _p(out), _p(batch.seq_of_token),
                  _p(batch.positions), _p(batch.page_table), batch.table_width, n, n_heads, n_kv, d, v_dim, float(scale),
                  MASKS[mask], int(mask_size), _p(sink), _stream())
    return out


def moe_table_up(x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """hidden[t, c] = silu(gate x_t) * (up x_t) with the matrices of expert ``table[tokens[t], c]``.
    x [n, width]; table int32 [vocab, top]; gate_up [experts, 2, ff, width] -> [n, top, ff].  With ``gate_up`` of shape
    [experts, 1, ff, width] the experts have one matrix and hidden = max(up x_t, 0)^2."""
    _cuda("x", x)
    n, width = x.shape
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("table", table, torch.int32)
    _cuda("gate_up", gate_up, x.dtype)
    _need(gate_up.dim() == 4 and gate_up.shape[1] in (1, 2) and gate_up.shape[3] == width,
          "gate_up must be [experts, 2 or 1, ff, width]")
    top, ff = table.shape[1], gate_up.shape[2]
    hidden = torch.empty((n, top, ff), dtype=x.dtype, device=x.device)
    _layer().call(f"wick_moe_up_{_dt(x)}", "pppiippiiiip", _p(x), _p(tokens), _p(table), top, gate_up.shape[0], _p(gate_up),
                  _p(hidden), n, width, ff, 1 if gate_up.shape[1] == 2 else 0, _stream())
    return hidden


def moe_table_down(hidden: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, down: torch.Tensor, weight: float,
                   base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 out[t] = sum(base[:, t]) + weight * sum over c of down[table[tokens[t], c]] hidden[t, c].
    down [experts, width, ff]; base float32 [splits, n, width] or None."""
    _cuda("hidden", hidden)
    n, top, ff = hidden.shape
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("table", table, torch.int32)
    _need(table.shape[1] == top, "the table's width is the number of choices")
    _cuda("down", down, hidden.dtype)
    _need(down.dim() == 3 and down.shape[2] == ff, "down must be [experts, width, ff]")
    width = down.shape[1]
    splits = 0
    if base is not None:
        _cuda("base", base, torch.float32)
        _need(base.dim() == 3 and tuple(base.shape[1:]) == (n, width), f"base must be [splits, {n}, {width}]")
        splits = base.shape[0]
    out = torch.empty((n, width), dtype=torch.float32, device=hidden.device)
    # (few pairs: the kernel leaves every pair's product in y and sums them per token afterwards)
    y = torch.zeros((n * top, width), dtype=torch.float32, device=hidden.device) if n * top <= 12000 else None
    _layer().call(f"wick_moe_down_{_dt(hidden)}", "pppiipfpippiiip", _p(hidden), _p(tokens), _p(table), top, down.shape[0],
                  _p(down), float(weight), _p(base), splits, _p(y), _p(out), n, width, ff, _stream(), kernels=2 if y is not None else 1)
    return out


def moe_route(tokens: torch.Tensor, table: torch.Tensor, n_experts: int, pad: int = 1) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """The step's (token, choice) pairs sorted by expert: (counts int32 [experts], row_of int32
    [n, top], expert_of_tile): pair (t, c) is row ``row_of[t, c]`` of the sorted order, in which
    expert 0's pairs come first and pairs of one expert keep their order (-1: the table names no
    expert).  With ``pad`` > 1 every expert's rows start at a multiple of ``pad`` (the rows between
    belong to nobody) and ``expert_of_tile`` int32 names the expert of every ``pad`` rows."""
    n = tokens.numel()
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("table", table, torch.int32)
    top = table.shape[1]
    counts = torch.zeros(n_experts, dtype=torch.int32, device=tokens.device)
    expert_of = torch.empty((n, top), dtype=torch.int32, device=tokens.device)
    row_of = torch.empty((n, top), dtype=torch.int32, device=tokens.device)
    tiles = torch.zeros((n * top + pad - 1) // pad + n_experts, dtype=torch.int32, device=tokens.device) if pad > 1 else None
    _layer().call("wick_moe_route", "ppiipppiipp", _p(tokens), _p(table), top, n_experts, _p(expert_of), _p(counts), _p(row_of),
                  n, int(pad), _p(tiles), _stream(), kernels=2)
    return counts, row_of, tiles


def moe_gather(x: torch.Tensor, row_of: torch.Tensor, n_rows: int) -> torch.Tensor:
    """xs[row_of[t, c]] = x[t]: the rows of x in the sorted order, [n_rows, width]."""
    _cuda("x", x)
    n, width = x.shape
    _cuda("row_of", row_of, torch.int32)
    top = row_of.shape[1]
    xs = torch.zeros((n_rows, width), dtype=x.dtype, device=x.device)      # (rows between the experts' stay zero)
    _layer().call(f"wick_moe_gather_{_dt(x)}", "ppipiip", _p(x), _p(row_of), top, _p(xs), n, width, _stream())
    return xs


def moe_combine(y: torch.Tensor, row_of: torch.Tensor, weight: float, base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 out[t] = sum(base[:, t]) + weight * sum over c of y[row_of[t, c]]."""
    _cuda("y", y, torch.float32)
    _cuda("row_of", row_of, torch.int32)
    n, top = row_of.shape
    width = y.shape[1]
    splits = 0
    if base is not None:
        _cuda("base", base, torch.float32)
        _need(base.dim() == 3 and tuple(base.shape[1:]) == (n, width), f"base must be [splits, {n}, {width}]")
        splits = base.shape[0]
    out = torch.empty((n, width), dtype=torch.float32, device=y.device)
    _layer().call("wick_moe_combine", "ppifpipiip", _p(y), _p(row_of), top, float(weight), _p(base), splits, _p(out), n, width,
                  _stream())
    return out


# ---- experts chosen by a router ---------------------------------------------------------------------------------------
ROUTER_SCORES = {"softmax": 0, "sigmoid": 1}


def moe_router(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, *, renormalize: bool = False,
               scores: str = "softmax", groups: int = 0, keep: int = 0, scale: float = 1.0, norm_eps: float = 0.0,
               outputs: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """From the router's logits (float32 partial sums [splits, n, outputs]; with ``outputs`` a row's first ``outputs`` columns,
    the row holding further columns of the same product): scores = softmax over the outputs, or the
    sigmoid of each (``scores``); the ``top`` outputs with the largest score + ``correction`` (float32 [outputs] or None)
    are chosen, the lowest index among equals.  ``groups`` > 0: the outputs form that many equal groups of neighbours, a
    group's score is the sum of its two largest corrected scores, and only outputs of the ``keep`` best groups can be chosen.
    Returns (choice int32 [n, top], weight float32 [n, top]: the chosen outputs' scores, divided by (their sum +
    ``norm_eps``) if ``renormalize``, times ``scale``; ident int32 [n] = 0 .. n - 1: with it as token ids, ``choice`` is the
    table of the kernels that read experts from a table)."""
    _cuda("logits", logits, torch.float32)
    _need(logits.dim() == 3, "the router's logits come as partial sums [splits, n, outputs]")
    _need(scores in ROUTER_SCORES, f"router scores are {', '.join(ROUTER_SCORES)}, not {scores!r}")
    splits, n, ld = logits.shape
    n_out = ld if outputs is None else int(outputs)
    _need(0 < n_out <= ld, f"{n_out} outputs in rows of {ld} numbers")
    if correction is not None:
        _cuda("correction", correction, torch.float32, (n_out,))
    choice = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weight = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    ident = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _layer().call("wick_moe_router", "piiiipiipppiiiffp", _p(logits), splits, n, ld, n_out, _p(correction), int(top), 1 if renormalize else 0,
                  _p(choice), _p(weight), _p(ident), ROUTER_SCORES[scores], int(groups), int(keep), float(scale), float(norm_eps),
                  _stream())
    return choice, weight, ident


def moe_expert_down(hidden: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """float32 y [n * top, width]: y[t * top + c] = down[table[tokens[t], c]] hidden[t, c]; rows of pairs whose table entry
    names no expert are zero.  down [experts, width, ff]."""
    _cuda("hidden", hidden)
    n, top, ff = hidden.shape
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("table", table, torch.int32)
    _need(table.shape[1] == top, "the table's width is the number of choices")
    _cuda("down", down, hidden.dtype)
    _need(down.dim() == 3 and down.shape[2] == ff, "down must be [experts, width, ff]")
    width = down.shape[1]
    y = torch.zeros((n * top, width), dtype=torch.float32, device=hidden.device)
    _layer().call(f"wick_moe_expert_down_{_dt(hidden)}", "pppiippiiip", _p(hidden), _p(tokens), _p(table), top, down.shape[0], _p(down),
                  _p(y), n, width, ff, _stream())
    return y


def moe_combine_weighted(y: torch.Tensor, row_of: Optional[torch.Tensor], choice: torch.Tensor, weight: torch.Tensor,
                         x: Optional[torch.Tensor], n_experts: int, base: Optional[torch.Tensor] = None,
                         base_gate: Optional[torch.Tensor] = None, base_gate_col: int = 0) -> torch.Tensor:
    """float32 out[t] = sum over c of weight[t, c] * r(t, c): r is row ``row_of[t, c]`` of ``y`` (row t * top + c without
    ``row_of``) where ``choice[t, c]`` < ``n_experts``, and ``x[t]`` itself where it is ``n_experts`` or more (an expert
    that returns its input; nothing if ``x`` is None).  y float32 [rows, width]; x [n, width].  ``base`` (float32 partial
    sums [splits, n, width]): what every token uses, added to the sum, times sigmoid(g_t) where ``base_gate`` (float32
    partial sums [splits, n, cols]) gives a number g_t per token in its column ``base_gate_col``."""
    _cuda("y", y, torch.float32)
    _cuda("choice", choice, torch.int32)
    n, top = choice.shape
    _cuda("weight", weight, torch.float32, (n, top))
    width = y.shape[1]
    if row_of is not None:
        _cuda("row_of", row_of, torch.int32, (n, top))
    dt = "f32"
    if x is not None:
        _cuda("x", x, None, (n, width))
        dt = _dt(x)
    bs = gs = gate_ld = 0
    if base is not None:
        _cuda("base", base, torch.float32)
        _need(base.dim() == 3 and tuple(base.shape[1:]) == (n, width), f"base must be [splits, {n}, {width}]")
        bs = base.shape[0]
    if base_gate is not None:
        _cuda("base_gate", base_gate, torch.float32)
        _need(base is not None and base_gate.dim() == 3 and base_gate.shape[1] == n and 0 <= base_gate_col < base_gate.shape[2],
              f"base_gate must be [splits, {n}, cols] with column {base_gate_col} among them")
        gs, gate_ld = base_gate.shape[0], base_gate.shape[2]
    out = torch.empty((n, width), dtype=torch.float32, device=y.device)
    gate_ptr = _p(base_gate) + 4 * int(base_gate_col) if base_gate is not None else _p(base_gate)
    _layer().call(f"wick_moe_combine_weighted_{dt}", "pppppiipiipipiip", _p(y), _p(row_of), _p(choice), _p(weight), _p(x), int(n_experts),
                  top, _p(out), n, width, _p(base), bs, gate_ptr, gs, gate_ld, _stream())
    return out


# ---- gated linear attention -------------------------------------------------------------------------------------------
GLA_CHUNK = 64            # tokens of one chunk of a long prompt's scan
GLA_CHUNKED_FROM = 192    # a prompt step of this many tokens or more is scanned in chunks


def gla_mix(parts: torch.Tensor, *, heads: int, key_dim: int, v_dim: int, w2: torch.Tensor, b2: Optional[torch.Tensor], q_scale: float,
            tau: float, records: torch.Tensor, batch) -> torch.Tensor:
    """The recurrence of a step's tokens.  ``parts``: the input projection's float32 partial sums [splits, n, cols], a row
    laid out [q: H dk | k: H dk | v: H dv | g: H dv | low: r].  q <- q * ``q_scale``; the decay per key channel is
    a = sigmoid(w2 low + b2)^(1 / tau) (``w2`` float32 [H dk, r]); per head S <- diag(a) S + k v^T and o = S^T q.
    ``records``: float32 [slots, H dv dk], a sequence's state (a column of S lies together), read and brought up to date for
    the slots of ``batch``.  Returns o float32 [n, H dv]."""
    _cuda("parts", parts, torch.float32)
    _need(parts.dim() == 3, "the projection comes as partial sums [splits, n, cols]")
    splits, n, cols = parts.shape
    hk, hv = heads * key_dim, heads * v_dim
    _cuda("w2", w2, torch.float32)
    _need(w2.dim() == 2 and w2.shape[0] == hk, f"w2 must be [{hk}, rank], is {tuple(w2.shape)}")
    rank = w2.shape[1]
    if b2 is not None:
        _cuda("b2", b2, torch.float32, (hk,))
    _cuda("records", records, torch.float32)
    _need(records.dim() == 2 and records.shape[1] == hv * key_dim, f"records must be [slots, {hv * key_dim}], are {tuple(records.shape)}")
    _need(n == batch.n_tokens, f"{n} rows, the batch has {batch.n_tokens} tokens")
    qkav = torch.empty((n, 3 * hk + hv), dtype=torch.float32, device=parts.device)
    y = torch.empty((n, hv), dtype=torch.float32, device=parts.device)
    max_q = 1 if batch.is_decode else 0          # (0: unknown to the host, as in a captured prompt step)
    chunk, chunks, chunk_state, chunk_decay = GLA_CHUNK, 0, None, None
    if not batch.is_decode and n >= GLA_CHUNKED_FROM:
        chunks = n // chunk + batch.n_seqs
        chunk_state = torch.empty((chunks, hv * key_dim), dtype=torch.float32, device=parts.device)
        chunk_decay = torch.empty((chunks, hk), dtype=torch.float32, device=parts.device)
    _layer().call("wick_gla_mix", "piiiiiiippffplpipppiiippp", _p(parts), splits, n, cols, heads, key_dim, v_dim, rank, _p(w2), _p(b2),
                  float(q_scale), float(tau), _p(records), hv * key_dim, _p(batch.slots), batch.n_seqs, _p(batch.cu_seqlens),
                  _p(qkav), _p(y), max_q, chunk, chunks, _p(chunk_state), _p(chunk_decay), _stream(),
                  kernels=1 + (3 if chunks else 1))
    return y


def gla_norm_gate(y: torch.Tensor, parts: torch.Tensor, g_col: int, heads: int, v_dim: int, weight: torch.Tensor, eps: float,
                  dtype: torch.dtype) -> torch.Tensor:
    """Every head's ``v_dim`` numbers of y (float32 [n, H dv]) divided by their root mean square and multiplied by ``weight``
    (float32 [dv], shared by the heads), then by silu(g), g the columns from ``g_col`` on of the float32 partial sums
    ``parts`` [splits, n, cols]; [n, H dv] in ``dtype``."""
    _cuda("y", y, torch.float32)
    _cuda("parts", parts, torch.float32)
    n = y.shape[0]
    _need(tuple(y.shape) == (n, heads * v_dim), f"y must be [n, {heads * v_dim}]")
    _need(parts.dim() == 3 and parts.shape[1] == n and parts.shape[2] >= g_col + heads * v_dim, "parts must hold the gate's columns")
    _cuda("weight", weight, torch.float32, (v_dim,))
    out = torch.empty((n, heads * v_dim), dtype=dtype, device=y.device)
    _layer().call(f"wick_gla_norm_gate_{_dt(out)}", "ppiiiiiipfpp", _p(y), _p(parts), parts.shape[0], n, parts.shape[2], int(g_col), heads,
                  v_dim, _p(weight), float(eps), _p(out), _stream())
    return out


def embed_sinusoid(table: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, freq: Optional[torch.Tensor], scale: float
                   ) -> torch.Tensor:
    """float32 [n, width]: rows of ``table`` at ``tokens`` times ``scale`` plus, with ``freq`` (float32 [ceil(width / 2)]), the
    positions' vectors: element 2 i gets sin(p freq[i]), element 2 i + 1 the cosine, the angle a float32 product."""
    _cuda("table", table)
    n, (vocab, width) = tokens.numel(), table.shape
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("positions", positions, torch.int32, (n,))
    if freq is not None:
        _cuda("freq", freq, torch.float32, ((width + 1) // 2,))
    out = torch.empty((n, width), dtype=torch.float32, device=table.device)
    _layer().call(f"wick_embed_sinusoid_{_dt(table)}", "ppppfpiip", _p(table), _p(tokens), _p(positions), _p(freq), float(scale), _p(out),
                  n, width, _stream())
    return out


def stream_offset_(x: torch.Tensor, x0: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> torch.Tensor:
    """x <- x + x0 + vec in place (float32 [n, width]; x0 of the same shape or None; vec float32 [width] or None)."""
    _cuda("x", x, torch.float32)
    n, width = x.shape
    if x0 is not None:
        _cuda("x0", x0, torch.float32, (n, width))
    if vec is not None:
        _cuda("vec", vec, torch.float32, (width,))
    _layer().call("wick_stream_offset", "pppiip", _p(x), _p(x0), _p(vec), n, width, _stream())
    return x


# ---- a state-space recurrence with its short convolution ----------------------------------------------------------------
def ssm_record_floats(heads: int, head_dim: int, state: int, groups: int, taps: int) -> int:
    """float32 numbers of one sequence's record: the convolution's last ``taps`` - 1 inputs, then the state."""
    return (taps - 1) * (heads * head_dim + 2 * groups * state) + heads * head_dim * state


SSM_CHUNK = 64            # tokens of one chunk of a long prompt's scan
SSM_CHUNKED_FROM = 192    # a prompt step of this many tokens or more is scanned in chunks


def ssm_mix(parts: torch.Tensor, *, heads: int, head_dim: int, state: int, groups: int, taps: int, conv_w: torch.Tensor,
            conv_b: Optional[torch.Tensor], dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: Optional[torch.Tensor],
            records: torch.Tensor, batch) -> torch.Tensor:
    """The recurrence of a step's tokens.  ``parts``: the input projection's float32 partial sums [splits, n, cols], a row
    laid out [z: H P | x: H P | B: G N | C: G N | dt: H].  x, B and C pass a causal convolution per channel (``conv_w``
    [channels, taps], the last tap the token's own; zeros before position 0) and silu; dt <- softplus(dt + dt_bias);
    per head S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d_skip x.  ``records``: float32 [slots, record], a
    sequence's last inputs and state (see :func:`ssm_record_floats`), read and brought up to date for the slots of
    ``batch``.  Returns y float32 [n, H P]."""
    _cuda("parts", parts, torch.float32)
    _need(parts.dim() == 3, "the projection comes as partial sums [splits, n, cols]")
    splits, n, cols = parts.shape
    inner, channels = heads * head_dim, heads * head_dim + 2 * groups * state
    _cuda("conv_w", conv_w, torch.float32, (channels, taps))
    if conv_b is not None:
        _cuda("conv_b", conv_b, torch.float32, (channels,))
    _cuda("dt_bias", dt_bias, torch.float32, (heads,))
    _cuda("a_log", a_log, torch.float32, (heads,))
    if d_skip is not None:
        _cuda("d_skip", d_skip, torch.float32, (heads,))
    _cuda("records", records, torch.float32)
    record = ssm_record_floats(heads, head_dim, state, groups, taps)
    _need(records.dim() == 2 and records.shape[1] == record, f"records must be [slots, {record}], are {tuple(records.shape)}")
    _need(n == batch.n_tokens, f"{n} rows, the batch has {batch.n_tokens} tokens")
    xbc = torch.empty((n, channels), dtype=torch.float32, device=parts.device)
    y = torch.empty((n, inner), dtype=torch.float32, device=parts.device)
    max_q = 1 if batch.is_decode else 0          # (0: unknown to the host, as in a captured prompt step)
    # A prompt step of many tokens is scanned in chunks side by side (three kernels instead of one); what the chunks' states
    # need is scratch of this call.
    chunk, chunks, chunk_state, chunk_decay = SSM_CHUNK, 0, None, None
    if not batch.is_decode and n >= SSM_CHUNKED_FROM:
        chunks = n // chunk + batch.n_seqs
        chunk_state = torch.empty((chunks, inner * state), dtype=torch.float32, device=parts.device)
        chunk_decay = torch.empty((chunks, heads), dtype=torch.float32, device=parts.device)
    _layer().call("wick_ssm_mix", "piiiiiiiipppppplpippppppiiippp", _p(parts), splits, n, cols, heads, head_dim, state, groups, taps,
                  _p(conv_w), _p(conv_b), _p(dt_bias), _p(a_log), _p(d_skip), _p(records), record, _p(batch.slots), batch.n_seqs,
                  _p(batch.cu_seqlens), _p(batch.start), _p(batch.seq_of_token), _p(batch.positions), _p(xbc), _p(y), max_q,
                  chunk, chunks, _p(chunk_state), _p(chunk_decay), _stream(),
                  kernels=(2 if taps > 1 else 1) + (3 if chunks else 1))
    return y


def ssm_gate_norm(y: torch.Tensor, parts: torch.Tensor, weight: torch.Tensor, eps: float, runs: int, dtype: torch.dtype) -> torch.Tensor:
    """g = y * silu(z), z the first columns of the float32 partial sums ``parts`` [splits, n, cols]; each of ``runs`` equal
    parts of g is divided by its own root mean square and multiplied by ``weight``; [n, inner] in ``dtype``."""
    _cuda("y", y, torch.float32)
    _cuda("parts", parts, torch.float32)
    n, inner = y.shape
    _need(parts.dim() == 3 and parts.shape[1] == n and parts.shape[2] >= inner, "parts must be [splits, n, inner or more]")
    _cuda("weight", weight, torch.float32, (inner,))
    out = torch.empty((n, inner), dtype=dtype, device=y.device)
    _layer().call(f"wick_ssm_gate_norm_{_dt(out)}", "ppiiiiipfpp", _p(y), _p(parts), parts.shape[0], n, parts.shape[2], inner, int(runs),
                  _p(weight), float(eps), _p(out), _stream())
    return out


# ---------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum (int32 [rows])."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_argmax", "ppiip", _p(logits), _p(out), rows, vocab, _stream())
    return out


def sample_temperature(logits: torch.Tensor, temperature: float, uniforms: torch.Tensor,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature): the first index whose
    cumulative probability (in index order) reaches uniforms[row] times the total."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _cuda("uniforms", uniforms, torch.float32, (rows,))
    _need(temperature > 0, "temperature must be positive (0 means greedy: use argmax)")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_sample_temperature", "pppiifp", _p(logits), _p(uniforms), _p(out), rows, vocab,
                 float(1.0 / temperature), _stream())
    return out


def top_k(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The k largest entries of each row, sorted by value (descending), ties by
    index (ascending): (float32 [rows, k], int32 [rows, k])."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _need(1 <= k <= min(vocab, 1024), f"top_k on the device takes 1 <= k <= min(vocab, 1024), not {k}")
    vals = torch.empty((rows, k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    _core().call("wick_top_k", "pppiiip", _p(logits), _p(vals), _p(idx), rows, vocab, k, _stream())
    return vals, idx


def pick_sorted(vals: torch.Tensor, idx: torch.Tensor, uniforms: torch.Tensor, temperature: float, min_p: float,
                top_p: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row from candidates sorted by logit (descending): the
    probabilities at ``temperature``, the min-p and top-p cuts and the draw with
    the row's uniform number, as ``sampling.sampler.pick_from_sorted`` does them
    on the host (int32 [rows])."""
    _cuda("vals", vals, torch.float32)
    rows, k = vals.shape
    _cuda("idx", idx, torch.int32, (rows, k))
    _cuda("uniforms", uniforms, torch.float32, (rows,))
    _need(temperature > 0.0, "pick_sorted needs a temperature above 0")
    probs = torch.empty_like(vals)
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=vals.device)
    _cuda("out", out, torch.int32, (rows,))
    _core().call("wick_pick_sorted", "pppppiifffp", _p(vals), _p(idx), _p(uniforms), _p(probs), _p(out), rows, k,
                 float(temperature), float(min_p), float(top_p), _stream())
    return out


def repetition_penalty(logits: torch.Tensor, histories, penalty: float) -> torch.Tensor:
    """In place: every distinct token of histories[row] has its logit divided by
    ``penalty`` if positive, multiplied otherwise."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _need(len(histories) == rows, "one history per row")
    r, t = [], []
    for i, h in enumerate(histories):
        d = sorted(set(int(x) for x in h))
        r += [i] * len(d)
        t += d
    if not t:
        return logits
    dev = torch.tensor([r, t], dtype=torch.int32).to(logits.device)
    _core().call("wick_repetition_penalty", "pppiifp", _p(logits), _p(dev[0]), _p(dev[1]), len(t), vocab,
                 float(penalty), _stream())
    return logits


# ---------------------------------------------------------------------------
# The per-sequence state record on the device (csrc/state.cu) and the kernels that
# move a batch from one decode step to the next without the host.
SEQ_STATE_WORDS = 8
SEQ_LENGTH, SEQ_NEXT, SEQ_FINISHED, SEQ_GENERATED, SEQ_LIMIT, SEQ_ROW = range(6)


def seq_state_set(state: torch.Tensor, slots: torch.Tensor, values: torch.Tensor) -> None:
    """state[slots[i]] = values[i] (int32 records of SEQ_STATE_WORDS words)."""
    _cuda("state", state, torch.int32)
    n = slots.numel()
    _cuda("slots", slots, torch.int32, (n,))
    _cuda("values", values, torch.int32, (n, SEQ_STATE_WORDS))
    _need(state.dim() == 2 and state.shape[1] == SEQ_STATE_WORDS, "state must be [slots, 8]")
    _core().call("wick_seq_state_set", "pppip", _p(state), _p(slots), _p(values), n, _stream())


def step_prepare(state: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor,
                 start: torch.Tensor, kv_len: torch.Tensor) -> None:
    """The fields of a decode step from the sequences' records: the token sampled last, its
    position, and the cached length before and after the step."""
    n = slots.numel()
    _cuda("state", state, torch.int32)
    for nm, t in (("slots", slots), ("tokens", tokens), ("positions", positions), ("start", start), ("kv_len", kv_len)):
        _cuda(nm, t, torch.int32, (n,))
    _core().call("wick_step_prepare", "ppppppip", _p(state), _p(slots), _p(tokens), _p(positions), _p(start), _p(kv_len),
                 n, _stream())


def step_advance(state: torch.Tensor, slots: torch.Tensor, ids: torch.Tensor, kv_len: torch.Tensor,
                 stops: Optional[torch.Tensor], seen: Optional[torch.Tensor], vocab: int) -> None:
    """After sampling: every running sequence of the step takes its sampled token (ids[i]) as
    its next one and its new length, or is marked finished (a stop token, or its limit).
    ids has one element more than there are rows; it receives the kernels' status word."""
    n = slots.numel()
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (n,))
    _cuda("ids", ids, torch.int32, (n + 1,))
    _cuda("kv_len", kv_len, torch.int32, (n,))
    n_stops = 0
    if stops is not None and stops.numel():
        _cuda("stops", stops, torch.int32)
        n_stops = stops.numel()
    if seen is not None:
        _cuda("seen", seen, torch.uint8)
        _need(seen.dim() == 2 and seen.shape[1] == vocab, f"seen must be [rows, {vocab}]")
    _core().call("wick_step_advance", "pppppipipip", _p(state), _p(slots), _p(ids), _p(kv_len),
                 _p(stops) if n_stops else None, n_stops, _p(seen), vocab, _p(status_tensor(state.device)), n, _stream())


def rng_uniforms(rng: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One uniform number in [0, 1) per row from the generator (xoshiro256**, int64 [rows of the
    batch, 4]) of the row's sequence; the generators of running sequences move on."""
    n = slots.numel()
    _cuda("rng", rng, torch.int64)
    _need(rng.dim() == 2 and rng.shape[1] == 4, "rng must be [rows, 4]")
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (n,))
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=state.device)
    _cuda("out", out, torch.float32, (n,))
    _core().call("wick_rng_uniforms", "ppppip", _p(rng), _p(state), _p(slots), _p(out), n, _stream())
    return out


def seen_prompt(seen: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor,
                seq_of_token: torch.Tensor) -> None:
    """Mark a prompt step's tokens as seen in their sequences' rows of ``seen`` (uint8 [rows, vocab])."""
    _cuda("seen", seen, torch.uint8)
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32)
    n = tokens.numel()
    _cuda("tokens", tokens, torch.int32, (n,))
    _cuda("seq_of_token", seq_of_token, torch.int32, (n,))
    _core().call("wick_seen_prompt", "pippppip", _p(seen), seen.shape[1], _p(state), _p(slots), _p(tokens),
                 _p(seq_of_token), n, _stream())


def penalty_seen(logits: torch.Tensor, seen: torch.Tensor, state: torch.Tensor, slots: torch.Tensor, penalty: float) -> None:
    """In place: the logit of every token seen in the row's sequence is divided by ``penalty``
    if positive, multiplied otherwise."""
    _cuda("logits", logits, torch.float32)
    rows, vocab = logits.shape
    _cuda("seen", seen, torch.uint8)
    _need(seen.dim() == 2 and seen.shape[1] == vocab, f"seen must be [rows, {vocab}]")
    _cuda("state", state, torch.int32)
    _cuda("slots", slots, torch.int32, (rows,))
    _core().call("wick_penalty_seen", "ppippfip", _p(logits), _p(seen), vocab, _p(state), _p(slots), float(penalty), rows,
                 _stream())


def wait_gives_up(limit_ms: float = 1.0) -> bool:
    """Run the kernel whose wait nothing can satisfy (one block, one barrier, no copies): its
    bounded wait gives up after ``limit_ms`` and leaves code 99 in the status word, which
    :func:`check_status` then reports.  Returns whether the wait gave up."""
    st = status_tensor("cuda")
    flag = torch.zeros(1, dtype=torch.int32, device=st.device)
    _core().call("wick_wait_gives_up", "pilpp", _p(st), 99, int(limit_ms * 1e6), _p(flag), _stream())
    return bool(flag.item())
