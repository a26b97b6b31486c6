"""Typed wrappers over the kernel library: they check dtypes, layouts and devices, and pass raw
pointers with the current CUDA stream.  Every function needs CUDA tensors; none has a CPU path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError

F32, BF16 = 0, 1
_c_void_p, _c_int, _c_long, _c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} has no kernel (float32 and bfloat16 do)")


def _stream() -> ctypes.c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _check(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None, dense: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if dense and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = float(table[ids[t]]); out is float32 [tokens, hidden]."""
    _check(table, "table"); _check(ids, "ids", torch.int32); _check(out, "out", torch.float32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out.shape != (tokens, hidden):
        raise KernelError(f"embed: out is {tuple(out.shape)}, expected {(tokens, hidden)}")
    _lib.core().call("mrun_embed", _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out),
                     _c_int(tokens), _c_int(hidden), _c_int(vocab), _stream())
    return out


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid (+= delta) then out = rmsnorm(resid) * weight; with ``rows`` only those rows are
    normed and resid is left as it is."""
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32); _check(out, "out")
    hidden = resid.shape[-1]
    n_rows = resid.shape[0] if rows is None else rows.numel()
    if delta is not None:
        _check(delta, "delta", out.dtype)
        if delta.shape != resid.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs resid {tuple(resid.shape)}")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    if weight.numel() != hidden or out.shape != (n_rows, hidden):
        raise KernelError(f"add_rmsnorm: weight {tuple(weight.shape)}, out {tuple(out.shape)}, "
                          f"expected hidden {hidden}, rows {n_rows}")
    _lib.core().call("mrun_add_rmsnorm", _ptr(resid), _ptr(delta), _ptr(weight), _c_float(eps), _ptr(out),
                     dtype_code(out.dtype), _ptr(rows), _c_int(n_rows), _c_int(hidden), _stream())
    return out


def add_layernorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid (+= delta) then out = (resid - mean) * rsqrt(variance + eps) * weight, the variance the
    mean of the squared deviations; with ``rows`` only those rows are normed and resid is left as
    it is.  ``delta`` is 32-bit or of ``out``'s dtype."""
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32); _check(out, "out")
    hidden = resid.shape[-1]
    n_rows = resid.shape[0] if rows is None else rows.numel()
    if delta is not None:
        _check(delta, "delta")
        if delta.shape != resid.shape or delta.dtype not in (torch.float32, out.dtype):
            raise KernelError(f"add_layernorm: delta {tuple(delta.shape)} {delta.dtype} vs resid {tuple(resid.shape)}, "
                              f"out {out.dtype}")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    if weight.numel() != hidden or out.shape != (n_rows, hidden):
        raise KernelError(f"add_layernorm: weight {tuple(weight.shape)}, out {tuple(out.shape)}, "
                          f"expected hidden {hidden}, rows {n_rows}")
    _lib.core().call("mrun_add_layernorm", _ptr(resid), _ptr(delta), dtype_code(delta.dtype if delta is not None else out.dtype),
                     _ptr(weight), _c_float(eps), _ptr(out), dtype_code(out.dtype), _ptr(rows), _c_int(n_rows),
                     _c_int(hidden), _stream())
    return out


def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float,
                   share: float = 0.5) -> torch.Tensor:
    """float32 ``share * (rmsnorm(a) * weight_a + rmsnorm(b) * weight_b)`` row by row (eps inside the
    root); ``a`` and ``b`` are float32 [rows, hidden]."""
    for name, t in (("a", a), ("b", b), ("weight_a", weight_a), ("weight_b", weight_b)):
        _check(t, name, torch.float32)
    rows, hidden = a.shape
    if b.shape != a.shape or weight_a.numel() != hidden or weight_b.numel() != hidden:
        raise KernelError(f"pair_norm_mean: a {tuple(a.shape)}, b {tuple(b.shape)}, weights {weight_a.numel()} / {weight_b.numel()}")
    out = torch.empty_like(a)
    _lib.core().call("mrun_pair_norm_mean", _ptr(a), _ptr(b), _ptr(weight_a), _ptr(weight_b), _c_float(eps),
                     _c_float(share), _ptr(out), _c_int(rows), _c_int(hidden), _stream())
    return out


def pair_norm_add_layernorm(resid: torch.Tensor, pending, weight: torch.Tensor, eps: float, out: torch.Tensor,
                            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid += share * (rmsnorm(a) * weight_a + rmsnorm(b) * weight_b) for a :class:`PendingPairNorm`,
    then out = layer norm of resid with ``weight``; with ``rows`` only those rows are worked on and
    resid is left as it is."""
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32); _check(out, "out")
    for name, t in (("a", pending.a), ("b", pending.b), ("weight_a", pending.weight_a), ("weight_b", pending.weight_b)):
        _check(t, name, torch.float32)
    hidden = resid.shape[-1]
    n_rows = resid.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _check(rows, "rows", torch.int32)
    if pending.a.shape != resid.shape or pending.b.shape != resid.shape or weight.numel() != hidden \
            or pending.weight_a.numel() != hidden or pending.weight_b.numel() != hidden or out.shape != (n_rows, hidden):
        raise KernelError(f"pair_norm_add_layernorm: resid {tuple(resid.shape)}, a {tuple(pending.a.shape)}, "
                          f"b {tuple(pending.b.shape)}, out {tuple(out.shape)}")
    _lib.core().call("mrun_pair_norm_add_layernorm", _ptr(resid), _ptr(pending.a), _ptr(pending.b), _ptr(pending.weight_a),
                     _ptr(pending.weight_b), _c_float(pending.eps), _c_float(pending.share), _ptr(weight), _c_float(eps),
                     _ptr(out), dtype_code(out.dtype), _ptr(rows), _c_int(n_rows), _c_int(hidden), _stream())
    return out


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor,
                 magnitude: float = 1.0) -> torch.Tensor:
    """out[t, j] = magnitude * (cos, sin)(positions[t] * inv_freq[j]); inv_freq is float64."""
    _check(positions, "positions", torch.int32); _check(inv_freq, "inv_freq", torch.float64)
    _check(out, "out", torch.float32)
    tokens, half = positions.numel(), inv_freq.numel()
    if out.shape != (tokens, half, 2):
        raise KernelError(f"rotary_table: out is {tuple(out.shape)}, expected {(tokens, half, 2)}")
    _lib.core().call("mrun_rotary_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _c_int(tokens),
                     _c_int(half), ctypes.c_double(magnitude), _stream())
    return out


def qk_norm_rope_cache(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       rot: Optional[torch.Tensor], rotary_dim: int, slots: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       page_size: int) -> None:
    """In place on the q part of ``qkv``; k and v go into the pages that ``slots`` names."""
    _check(qkv, "qkv")
    tokens = qkv.shape[0]
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_cache: qkv is {tuple(qkv.shape)}, expected width "
                          f"{(heads + 2 * kv_heads) * head_dim}")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_cache: {name} has {w.numel()} elements, head_dim is {head_dim}")
    if rot is not None:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rotary_dim // 2, 2):
            raise KernelError(f"qk_norm_rope_cache: rot is {tuple(rot.shape)}, expected "
                              f"{(tokens, rotary_dim // 2, 2)}")
    if slots is not None:
        _check(slots, "slots", torch.int32)
        if slots.numel() != tokens:
            raise KernelError("qk_norm_rope_cache: one slot per token is needed")
        for name, c in (("k_cache", k_cache), ("v_cache", v_cache)):
            _check(c, name, qkv.dtype)
            if c.dim() != 4 or c.shape[1:] != (kv_heads, page_size, head_dim):
                raise KernelError(f"qk_norm_rope_cache: {name} is {tuple(c.shape)}, expected "
                                  f"[pages, {kv_heads}, {page_size}, {head_dim}]")
    _lib.core().call("mrun_qk_norm_rope_cache", _ptr(qkv), dtype_code(qkv.dtype), _ptr(q_weight),
                     _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary_dim if rot is not None else 0),
                     _ptr(slots), _ptr(k_cache), _ptr(v_cache), _c_int(tokens), _c_int(heads),
                     _c_int(kv_heads), _c_int(head_dim), _c_int(page_size), _stream())


def proj_norm_rope_cache(x: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, dim: int,
                         vdim: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                         rot: Optional[torch.Tensor], rotary_dim: int, pairing: str, slots: Optional[torch.Tensor],
                         k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_size: int) -> None:
    """RMS norm of q and of k over the whole projection (all heads of a token together, weights of
    that size), rotation of the first ``rotary_dim`` features of every head, k and v into the
    pages ``slots`` names (key pages [pages, kv_heads, page, dim], value pages [.., vdim]).  ``x``:
    rows whose q, k and v heads start at columns ``q_off``, ``k_off``, ``v_off``; q is worked on in
    place.  ``k_off`` < 0: the rows have no keys and values."""
    ld = _strided_rows(x, "x")
    tokens = x.shape[0]
    for name, w, n in (("q_weight", q_weight, heads * dim), ("k_weight", k_weight, kv_heads * dim)):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != n:
                raise KernelError(f"proj_norm_rope_cache: {name} has {w.numel()} elements, the projection has {n}")
    if rot is not None:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rotary_dim // 2, 2):
            raise KernelError(f"proj_norm_rope_cache: rot is {tuple(rot.shape)}, expected {(tokens, rotary_dim // 2, 2)}")
    if k_off >= 0 and slots is not None:
        _check(slots, "slots", torch.int32)
        for name, c, n in (("k_cache", k_cache, dim), ("v_cache", v_cache, vdim)):
            _check(c, name, x.dtype)
            if c.dim() != 4 or c.shape[1:] != (kv_heads, page_size, n):
                raise KernelError(f"proj_norm_rope_cache: {name} is {tuple(c.shape)}, expected "
                                  f"[pages, {kv_heads}, {page_size}, {n}]")
    width = x.shape[1]
    if q_off + heads * dim > width or (k_off >= 0 and (k_off + kv_heads * dim > width or v_off + kv_heads * vdim > width)):
        raise KernelError("proj_norm_rope_cache: the heads do not fit the rows")
    _lib.core().call("mrun_proj_norm_rope_cache", _ptr(x), _c_long(ld), _c_long(q_off), _c_long(k_off), _c_long(v_off),
                     dtype_code(x.dtype), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot),
                     _c_int(rotary_dim if rot is not None else 0), _c_int(PAIRINGS[pairing]),
                     _ptr(slots if k_off >= 0 else None), _ptr(k_cache), _ptr(v_cache), _c_int(tokens), _c_int(heads),
                     _c_int(kv_heads), _c_int(dim), _c_int(vdim), _c_int(page_size), _stream())


def head_norm_rope_cache(x: torch.Tensor, q_off: int, k_off: int, v_off: int, heads: int, kv_heads: int, dim: int,
                         vdim: int, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                         rot: Optional[torch.Tensor], rotary_dim: int, pairing: str, slots: Optional[torch.Tensor],
                         k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], page_size: int) -> None:
    """RMS norm of every q and k head over its own ``dim`` features (weights of ``dim`` entries that
    the heads share; None: no norm), rotation of the first ``rotary_dim`` features of every head,
    k and v into the pages ``slots`` names (key pages [pages, kv_heads, page, dim], value pages
    [.., vdim]).  ``x``: rows whose q, k and v heads start at columns ``q_off``, ``k_off``,
    ``v_off``; q is worked on in place.  ``v_off`` < 0: the values are the keys as projected,
    before norm and rotation."""
    ld = _strided_rows(x, "x")
    tokens = x.shape[0]
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != dim:
                raise KernelError(f"head_norm_rope_cache: {name} has {w.numel()} elements, a head has {dim}")
    if rot is not None:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rotary_dim // 2, 2):
            raise KernelError(f"head_norm_rope_cache: rot is {tuple(rot.shape)}, expected {(tokens, rotary_dim // 2, 2)}")
    if slots is not None:
        _check(slots, "slots", torch.int32)
        for name, c, n in (("k_cache", k_cache, dim), ("v_cache", v_cache, vdim)):
            _check(c, name, x.dtype)
            if c.dim() != 4 or c.shape[1:] != (kv_heads, page_size, n):
                raise KernelError(f"head_norm_rope_cache: {name} is {tuple(c.shape)}, expected "
                                  f"[pages, {kv_heads}, {page_size}, {n}]")
    width = x.shape[1]
    if q_off + heads * dim > width or k_off + kv_heads * dim > width or (v_off >= 0 and v_off + kv_heads * vdim > width):
        raise KernelError("head_norm_rope_cache: the heads do not fit the rows")
    _lib.core().call("mrun_head_norm_rope_cache", _ptr(x), _c_long(ld), _c_long(q_off), _c_long(k_off), _c_long(v_off),
                     dtype_code(x.dtype), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(rot),
                     _c_int(rotary_dim if rot is not None else 0), _c_int(PAIRINGS[pairing]), _ptr(slots), _ptr(k_cache),
                     _ptr(v_cache), _c_int(tokens), _c_int(heads), _c_int(kv_heads), _c_int(dim), _c_int(vdim),
                     _c_int(page_size), _stream())


def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, block_tables: torch.Tensor, token_slot: torch.Tensor,
                            positions: torch.Tensor, heads: int, scale: float, window: int = 0, sink: bool = False,
                            gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of every token over its request's pages, 32-bit arithmetic on CUDA cores.

    ``q`` may be a view into a wider buffer: row t starts ``q_stride`` elements after row t-1.
    ``block_tables`` has one row per state slot; ``token_slot[t]`` names the row of token t.
    The value pages may have another feature size than the key pages.  ``sink``: one more term of
    score 0 without a value in the softmax's denominator.  ``gate``: [tokens, heads] in q's dtype
    (rows may be strided), whose sigmoid multiplies each head's output.
    """
    _check(q, "q", dense=False); _check(out, "out", q.dtype)
    _check(k_cache, "k_cache", q.dtype); _check(v_cache, "v_cache", q.dtype)
    _check(block_tables, "block_tables", torch.int32); _check(token_slot, "token_slot", torch.int32)
    _check(positions, "positions", torch.int32)
    pages, kv_heads, page_size, head_dim = k_cache.shape
    tokens = positions.numel()
    if v_cache.dim() != 4 or v_cache.shape[:3] != k_cache.shape[:3]:
        raise KernelError("paged_attention: k and v caches differ in pages, heads or page size")
    value_dim = v_cache.shape[3]
    if out.shape != (tokens, heads * value_dim) or token_slot.numel() != tokens:
        raise KernelError(f"paged_attention: out {tuple(out.shape)} / token_slot {token_slot.numel()} "
                          f"do not match {tokens} tokens of {heads}x{value_dim}")
    if block_tables.dim() != 2:
        raise KernelError("paged_attention: block_tables must be [slots, max_blocks]")
    gate_stride = 0
    if gate is not None:
        gate_stride = _strided_rows(gate, "gate")
        if gate.shape != (tokens, heads) or gate.dtype != q.dtype:
            raise KernelError(f"paged_attention: gate is {tuple(gate.shape)} {gate.dtype}, expected {(tokens, heads)} {q.dtype}")
    _lib.core().call("mrun_paged_attention_generic", _ptr(q), _c_long(q_stride), _ptr(out), _ptr(k_cache),
                     _ptr(v_cache), dtype_code(q.dtype), _ptr(block_tables), _c_int(block_tables.shape[1]),
                     _ptr(token_slot), _ptr(positions), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                     _c_int(head_dim), _c_int(value_dim), _c_int(page_size), _c_long(pages * kv_heads * page_size),
                     _c_float(scale), _c_int(window), _c_int(1 if sink else 0), _ptr(gate), _c_long(gate_stride), _stream())
    return out


GATE_FUNCTIONS = {"silu": 1, "gelu_tanh": 2}      # codes of the C ABI (MRUN_GATE_*); 0 = no gated epilogue


def gate_code(activation: str) -> int:
    try:
        return GATE_FUNCTIONS[activation]
    except KeyError:
        raise KernelError(f"no kernel has the gate function {activation!r} "
                          f"(known: {', '.join(sorted(GATE_FUNCTIONS))})") from None


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False, activation: str = "silu") -> torch.Tensor:
    """out = act(gate) * up.  Plain layout: gate_up[:, :I] are the gates, gate_up[:, I:] the ups.
    Interleaved: runs of eight gates followed by the eight ups of the same outputs."""
    _check(gate_up, "gate_up"); _check(out, "out", gate_up.dtype)
    tokens, inter = out.shape
    if gate_up.shape != (tokens, 2 * inter):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    _lib.core().call("mrun_swiglu", _ptr(gate_up), _ptr(out), dtype_code(out.dtype), _c_int(tokens),
                     _c_int(inter), _c_int(8 if interleaved else 0), _c_int(gate_code(activation)), _stream())
    return out


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, n] += bias[n] in place; bias is float32."""
    _check(y, "y"); _check(bias, "bias", torch.float32)
    if y.dim() != 2 or bias.numel() != y.shape[1]:
        raise KernelError(f"add_bias: y {tuple(y.shape)} vs bias {tuple(bias.shape)}")
    _lib.core().call("mrun_add_bias", _ptr(y), dtype_code(y.dtype), _ptr(bias), _c_int(y.shape[0]),
                     _c_int(y.shape[1]), _stream())
    return y


SKINNY_ROWS = 16      # the decode GEMM takes up to this many rows


def skinny_ok(x, w: torch.Tensor) -> bool:
    """Whether the decode GEMM takes this product: few rows, bf16, K a multiple of 32."""
    if isinstance(x, NormedRows):
        x = x.xw
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0)


SUMS_UNIT = 2.0 ** -30        # a row's total of squares is a 64-bit integer in these units


class NormedRows:
    """The output of an RMSNorm whose row scale has not been applied yet: ``xw`` holds
    bf16(stream * norm weight) and ``sums`` (int64, a row each) each row's total of squares of the stream
    in units of 2^-30.  The decode GEMM takes it as its x and applies rsqrt(total / width + eps)
    to its own sums (so does the tcgen05 GEMM for 17 to 128 rows); :meth:`finish` makes the plain
    normed rows."""

    def __init__(self, xw: torch.Tensor, sums: torch.Tensor, eps: float):
        self.xw, self.sums, self.eps = xw, sums, float(eps)

    @property
    def shape(self):
        return self.xw.shape

    @property
    def dtype(self):
        return self.xw.dtype

    @property
    def device(self):
        return self.xw.device

    def finish(self) -> torch.Tensor:
        tokens, width = self.xw.shape
        out = torch.empty_like(self.xw)
        _lib.core().call("mrun_norm_finish", _ptr(self.xw), _ptr(self.sums), _c_float(self.eps), _ptr(out),
                         _c_int(tokens), _c_int(width), _stream())
        return out


class RowSums:
    """Zeroed per-row totals for the products of one step: one buffer per device, cleared once at
    the start of a step (:meth:`begin_step`: one memset, which a captured step replays) and handed
    out slice by slice, so that no product clears its own."""

    ROWS = 16 * 1024
    _arenas = {}

    @classmethod
    def begin_step(cls, device: torch.device) -> None:
        arena = cls._arenas.get(device)
        if arena is None:
            arena = cls._arenas[device] = [torch.zeros(cls.ROWS, dtype=torch.int64, device=device), 0]
        arena[0].zero_()                   # always: a captured step must clear what other steps left
        arena[1] = 0

    @classmethod
    def take(cls, device: torch.device, rows: int = 16) -> torch.Tensor:
        """The next ``rows`` zeroed totals of the step (a multiple of 16 is taken), or a fresh
        zeroed tensor outside a step or when the step has used all of its buffer."""
        rows = -(-rows // 16) * 16
        arena = cls._arenas.get(device)
        if arena is None or arena[1] + rows > cls.ROWS:
            return torch.zeros(rows, dtype=torch.int64, device=device)
        arena[1] += rows
        return arena[0][arena[1] - rows:arena[1]]


class PendingLinear:
    """A product ``x @ w.T`` that has not run yet: a part returns it as its output where the norm
    that follows can run it with the residual sum and the norm folded into its epilogue
    (:func:`linear_into_norm`).  :meth:`compute` runs it as an ordinary product."""

    def __init__(self, x: torch.Tensor, w: torch.Tensor):
        self.x, self.w = x, w

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    def compute(self) -> torch.Tensor:
        return linear(self.x, self.w)


class PendingPostNorm:
    """A branch output (float32 rows) that joins the stream as ``scale * rmsnorm(branch) * weight``
    and has not been added yet: the norm that follows adds it and norms the new rows in one
    kernel (:func:`post_norm_add`).  :meth:`compute` makes the addend itself."""

    def __init__(self, branch: torch.Tensor, weight: torch.Tensor, eps: float, scale: float, act: torch.dtype):
        self.branch, self.weight, self.eps, self.scale, self.act = branch, weight, float(eps), float(scale), act

    @property
    def shape(self):
        return self.branch.shape

    def compute(self) -> torch.Tensor:
        addend = torch.zeros_like(self.branch)
        post_norm_add(addend, self.branch, self.weight, self.scale, self.eps, None, 0.0, None)
        return addend.to(self.act)


class PendingPairNorm:
    """Two branch outputs (float32 rows) that join the stream as ``share * (rmsnorm(a) * weight_a +
    rmsnorm(b) * weight_b)`` and have not been combined yet: a layer norm that follows norms both,
    adds them and norms the new rows in one kernel (:func:`pair_norm_add_layernorm`).
    :meth:`compute` makes the addend itself (float32)."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float,
                 share: float):
        self.a, self.b, self.weight_a, self.weight_b = a, b, weight_a, weight_b
        self.eps, self.share = float(eps), float(share)

    @property
    def shape(self):
        return self.a.shape

    def compute(self) -> torch.Tensor:
        return pair_norm_mean(self.a, self.b, self.weight_a, self.weight_b, self.eps, self.share)


PENDING = (PendingLinear, PendingPostNorm, PendingPairNorm)      # what a block may hand to the norm after it unadded


def _normed(x):
    """(rows, totals pointer, eps) of a product's x, which may be :class:`NormedRows`."""
    if isinstance(x, NormedRows):
        return x.xw, _ptr(x.sums), _c_float(x.eps)
    return x, _ptr(None), _c_float(0.0)


def gemm_skinny(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                swiglu_rows: bool = False, activation: str = "silu", rows: int = 0) -> torch.Tensor:
    """y = x @ w.T for at most 16 rows, reading w once at HBM speed.  ``swiglu_rows``: w holds gate
    and up rows interleaved in runs of eight and y = act(gate) * up has half as many columns.
    ``x`` may be :class:`NormedRows`.  ``w`` is a weight: the kernel asks for its first rows while
    the decode GEMM launched before it may still be running, so it must not be that launch's
    output (x, the stream and every output are touched only after that kernel has finished).
    ``rows``: the rows of w a block takes (8..16; 0: the count that fills the device most evenly)."""
    x, sums, eps = _normed(x)
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    out = torch.empty((m, n // 2 if swiglu_rows else n), dtype=out_dtype, device=x.device)
    _lib.core().call("mrun_gemm_skinny", _ptr(x), _ptr(w), _ptr(out), dtype_code(out_dtype),
                     _c_int(gate_code(activation) if swiglu_rows else 0), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(out.shape[1]),
                     sums, eps, _ptr(None), _ptr(None), _ptr(None), _ptr(None), _c_int(rows), _stream())
    return out


def norm_fusable(pending, resid: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear_into_norm` takes this pending product and residual stream."""
    return (isinstance(pending, PendingLinear) and (skinny_ok(pending.x, pending.w) or tc5_ok(pending.x, pending.w))
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == pending.shape
            and resid.shape[1] % 32 == 0 and weight.numel() == resid.shape[1])


def linear_into_norm(pending: PendingLinear, resid: torch.Tensor, weight: torch.Tensor, eps: float,
                     rows: int = 0) -> NormedRows:
    """resid += pending.x @ pending.w.T (32-bit, in place) and the RMSNorm of the new rows with
    ``weight``, as :class:`NormedRows`: one kernel (the decode GEMM up to 16 rows, the tcgen05
    GEMM up to 128)."""
    skinny = skinny_ok(pending.x, pending.w)
    x, in_sums, in_eps = _normed(pending.x)
    w = pending.w
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or resid.shape != (m, n) or weight.numel() != n:
        raise KernelError(f"linear_into_norm: x {tuple(x.shape)}, w {tuple(w.shape)}, resid {tuple(resid.shape)}, "
                          f"weight {tuple(weight.shape)}")
    xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    out_sums = RowSums.take(x.device, m)
    head = (_ptr(x), _ptr(w), _ptr(None), dtype_code(torch.bfloat16), _c_int(0), _c_int(m), _c_int(n), _c_int(k),
            _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(n), in_sums, in_eps, _ptr(resid),
            _ptr(weight), _ptr(xw), _ptr(out_sums))
    if skinny:
        _lib.core().call("mrun_gemm_skinny", *head, _c_int(rows), _stream())
    else:
        _lib.core().call("mrun_gemm_tc5", *head, _c_int(0), _ptr(_tc5_status(x.device)), _stream())
    return NormedRows(xw, out_sums, eps)


def gemm_f32_nt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w.T in IEEE 32-bit with a fixed summation order.  x may have a row stride."""
    _check(x, "x", torch.float32, dense=False); _check(w, "w", torch.float32)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or x.stride(1) != 1:
        raise KernelError(f"gemm_f32_nt: x {tuple(x.shape)} (strides {x.stride()}) vs w {tuple(w.shape)}")
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _check(out, "out", torch.float32)
    if out.shape != (m, n):
        raise KernelError(f"gemm_f32_nt: out is {tuple(out.shape)}, expected {(m, n)}")
    _lib.core().call("mrun_gemm_f32_nt", _ptr(x), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else k), _c_long(n), _stream())
    return out


TC5_ROWS = 128            # the tcgen05 GEMM takes up to this many rows
# Whether products of 17 to 128 rows go to the tcgen05 GEMM.  Off: measured on B200 at the
# Qwen3-8B shapes it loses to the vendor library at 32, 64 and 128 rows (a kernel that holds tensor
# memory has its multiprocessor to itself, so nothing of its start overlaps the kernel before).
TC5_GEMM = False


def _tc5_status(device: torch.device) -> torch.Tensor:
    return status_word(device, "gemm_tc5", {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue",
                                            4: "the exchange inside a cluster"})


def tc5_ok(x, w: torch.Tensor) -> bool:
    """Whether the tcgen05 GEMM takes this product: 17..128 rows, bf16, K a multiple of 64."""
    if isinstance(x, NormedRows):
        x = x.xw
    return (TC5_GEMM and isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.dim() == 2 and SKINNY_ROWS < x.shape[0] <= TC5_ROWS
            and x.shape[1] % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


_sm_count = {}


def sm_count(device: torch.device) -> int:
    n = _sm_count.get(device)
    if n is None:
        n = _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemm_tc5(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu_rows: bool = False,
             activation: str = "silu", split: int = 0) -> torch.Tensor:
    """y = x @ w.T for 1..128 rows on the tcgen05 tensor cores (TMA-fed, accumulators in tensor
    memory, k split over thread-block clusters whose blocks exchange partial sums through
    distributed shared memory; ``split`` = 0 lets the library choose the cluster size).
    ``swiglu_rows`` as in :func:`gemm_skinny`; ``x`` may be :class:`NormedRows`; ``w`` is a weight
    (its first tiles are asked for before the kernel before has finished).  A wait inside the
    kernel that runs out sets the status word that :func:`tc5_check` reads."""
    x, sums, eps = _normed(x)
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_tc5: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    out = torch.empty((m, n // 2 if swiglu_rows else n), dtype=out_dtype, device=x.device)
    _lib.core().call("mrun_gemm_tc5", _ptr(x), _ptr(w), _ptr(out), dtype_code(out_dtype),
                     _c_int(gate_code(activation) if swiglu_rows else 0), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(out.shape[1]),
                     sums, eps, _ptr(None), _ptr(None), _ptr(None), _ptr(None), _c_int(split),
                     _ptr(_tc5_status(x.device)), _stream())
    return out


_status_words = {}       # (device, kernel name) -> (int32[1] on the device, {code: role})


def status_word(device: torch.device, kernel: str, roles: dict) -> torch.Tensor:
    """The word a kernel with bounded waits reports into (zero = fine), one per device and kernel,
    never reallocated, so that captured graphs may keep its address.  :func:`tc5_check` reads it."""
    entry = _status_words.get((device, kernel))
    if entry is None:
        entry = _status_words[(device, kernel)] = (torch.zeros(1, dtype=torch.int32, device=device), dict(roles))
    return entry[0]


def tc5_check(device: Optional[torch.device] = None) -> None:
    """Raises if a tcgen05 kernel on the device gave up on a wait (and clears its status word)."""
    for (dev, kernel), (status, roles) in list(_status_words.items()):
        if device is not None and dev != device:
            continue
        code = int(status.item())
        if code:
            status.zero_()
            raise KernelError(f"{kernel}: {roles.get(code, 'a role')} waited longer than its budget on {dev}; "
                              f"the results of that call are invalid")


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w.T (+ bias).  float32: this library's own IEEE kernel.  bfloat16 with at most 16
    rows (decode): this library's weight-streaming tensor-core kernel (``x`` may then be
    :class:`NormedRows`).  bfloat16 otherwise (prefill): the vendor GEMM library with 32-bit
    accumulation (the reference calls its array library's matmul for the same products and adds
    an optional bias after it, crates/mrun-engine/src/load.rs:294-306)."""
    if isinstance(x, NormedRows):
        if skinny_ok(x, w) or tc5_ok(x, w):
            y = (gemm_skinny if skinny_ok(x, w) else gemm_tc5)(x, w, out_dtype or torch.bfloat16)
            return y if bias is None else add_bias(y, bias)
        x = x.finish()
    if x.dtype == torch.float32:
        y = gemm_f32_nt(x, w)
    else:
        _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
        if skinny_ok(x, w):
            y = gemm_skinny(x, w, out_dtype or torch.bfloat16)
        elif tc5_ok(x, w):
            y = gemm_tc5(x, w, out_dtype or torch.bfloat16)
        elif out_dtype is None or out_dtype == torch.bfloat16:
            y = torch.mm(x, w.t())
        else:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
    return y if bias is None else add_bias(y, bias)


def linear_or_pending(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """The last product of a part whose caller accepts a :class:`PendingLinear`: left pending in
    bfloat16 without a bias (the norm after it then runs it with the residual sum folded in: in
    the decode GEMM's epilogue up to 16 rows, as the vendor GEMM's accumulate-into-C above),
    computed otherwise."""
    if bias is None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return PendingLinear(x, w)
    return linear(x, w, bias=bias)


def accumulate_ok(pending, resid: torch.Tensor) -> bool:
    """Whether :func:`linear_add_into` takes this pending product and residual stream."""
    return (isinstance(pending, PendingLinear) and isinstance(pending.x, torch.Tensor) and not tc5_ok(pending.x, pending.w)
            and not skinny_ok(pending.x, pending.w)
            and pending.x.dtype == torch.bfloat16 and pending.w.dtype == torch.bfloat16 and pending.x.dim() == 2
            and resid.dtype == torch.float32 and resid.is_contiguous() and tuple(resid.shape) == tuple(pending.shape))


def linear_add_into(resid: torch.Tensor, pending: PendingLinear) -> torch.Tensor:
    """resid += pending.x @ pending.w.T in place: the vendor GEMM with bfloat16 operands, 32-bit
    accumulation and the 32-bit stream as its C and D, so that the product is never rounded to
    bfloat16, written and read again (prompt portions and decode batches above 16 rows)."""
    return torch.addmm(resid, pending.x, pending.w.t(), out_dtype=torch.float32, out=resid)


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           min_p: Optional[torch.Tensor] = None, keys: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits; per-row parameter arrays, None = neutral."""
    _check(logits, "logits", torch.float32); _check(out, "out", torch.int32)
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("top_k", top_k, torch.int32), ("min_p", min_p, torch.float32),
                        ("keys", keys, torch.int64)):
        if t is not None:
            _check(t, name, dt)
            if t.numel() < rows:
                raise KernelError(f"sample: {name} has {t.numel()} entries for {rows} rows")
    if out.numel() < rows:
        raise KernelError(f"sample: out has {out.numel()} entries for {rows} rows")
    _lib.core().call("mrun_sample", _ptr(logits), _c_int(rows), _c_int(vocab), _ptr(temperature), _ptr(top_p),
                     _ptr(top_k), _ptr(min_p), _ptr(keys), _ptr(out), _stream())
    return out


def top_logprobs(logits: torch.Tensor, n: int):
    """(ids int32 [rows, n], log-probabilities float32 [rows, n]) of the n most likely tokens of
    each row of float32 logits, most likely first, ties by the smaller id."""
    _check(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    n = max(1, min(int(n), vocab))
    ids = torch.empty((rows, n), dtype=torch.int32, device=logits.device)
    values = torch.empty((rows, n), dtype=torch.float32, device=logits.device)
    _lib.core().call("mrun_top_logprobs", _ptr(logits), _c_int(rows), _c_int(vocab), _c_int(n), _ptr(ids),
                     _ptr(values), _stream())
    return ids, values


def apply_token_mask(logits: torch.Tensor, rows: torch.Tensor, words: torch.Tensor, mask_vocab: torch.Tensor) -> None:
    """In place: logits[rows[m], i] = -inf wherever bit i of words[m] is clear or i >= mask_vocab[m].
    ``words``: int32 [masks, words a mask] (the bits of unsigned 32-bit words), 32 tokens a word."""
    _check(logits, "logits", torch.float32); _check(rows, "rows", torch.int32)
    _check(words, "words", torch.int32); _check(mask_vocab, "mask_vocab", torch.int32)
    masks = rows.numel()
    if words.dim() != 2 or words.shape[0] != masks or mask_vocab.numel() != masks:
        raise KernelError(f"apply_token_mask: {masks} rows, words {tuple(words.shape)}, {mask_vocab.numel()} vocabularies")
    _lib.core().call("mrun_apply_token_mask", _ptr(logits), _c_int(logits.shape[1]), _ptr(rows), _ptr(words),
                     _c_int(words.shape[1]), _ptr(mask_vocab), _c_int(masks), _stream())


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: the logits of the ids in recent[row] (negative = empty) are penalised."""
    _check(logits, "logits", torch.float32); _check(recent, "recent", torch.int32)
    _check(penalty, "penalty", torch.float32)
    rows, vocab = logits.shape
    if recent.dim() != 2 or recent.shape[0] != rows or penalty.numel() < rows:
        raise KernelError(f"repetition_penalty: recent {tuple(recent.shape)}, penalty {penalty.numel()}, rows {rows}")
    _lib.core().call("mrun_repetition_penalty", _ptr(logits), _c_int(rows), _c_int(vocab), _ptr(recent),
                     _c_int(recent.shape[1]), _ptr(penalty), _stream())


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> None:
    """dst.view(-1)[index[i]] = value[i] for int32 tensors."""
    _check(dst, "dst", torch.int32); _check(index, "index", torch.int32); _check(value, "value", torch.int32)
    if index.numel() != value.numel():
        raise KernelError("scatter_i32: index and value differ in length")
    _lib.core().call("mrun_scatter_i32", _ptr(dst), _ptr(index), _ptr(value), _c_int(index.numel()),
                     _c_long(dst.numel()), _stream())


def select_tokens(ids: torch.Tensor, previous: torch.Tensor, source: torch.Tensor) -> None:
    """ids[r] = previous[source[r]] where source[r] >= 0 (int32 tensors)."""
    _check(ids, "ids", torch.int32); _check(previous, "previous", torch.int32); _check(source, "source", torch.int32)
    if source.numel() != ids.numel():
        raise KernelError("select_tokens: one source per row is needed")
    _lib.core().call("mrun_select_tokens", _ptr(ids), _ptr(previous), _ptr(source), _c_int(ids.numel()),
                     _c_int(previous.numel()), _stream())



# ------------------------------------------------------------------ latent attention, sandwich norms, routing

def gemm_f32_nt_batched(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b] = x[b] @ w[b].T in IEEE 32-bit with a fixed summation order.  ``x`` [batch, M, K] and
    ``out`` [batch, M, N] may be strided views (unit stride along the last axis: the heads of a
    row laid side by side); ``w`` is dense [batch, N, K]."""
    _check(x, "x", torch.float32, dense=False); _check(w, "w", torch.float32); _check(out, "out", torch.float32, dense=False)
    batch, m, k = x.shape
    n = w.shape[1]
    if w.shape != (batch, n, k) or out.shape != (batch, m, n) or x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError(f"gemm_f32_nt_batched: x {tuple(x.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    _lib.core().call("mrun_gemm_f32_nt_batched", _ptr(x), _ptr(w), _ptr(out), _c_int(batch), _c_int(m), _c_int(n),
                     _c_int(k), _c_long(x.stride(1) if m > 1 else max(k, x.stride(1))),
                     _c_long(out.stride(1) if m > 1 else max(n, out.stride(1))),
                     _c_long(x.stride(0)), _c_long(n * k), _c_long(out.stride(0)), _stream())
    return out


def linear_per_head(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[:, h] = x[:, h] @ w[h].T for every head h: ``x`` [tokens, heads, K] and ``out``
    [tokens, heads, N] may be views into wider rows, ``w`` is dense [heads, N, K].  float32: this
    library's IEEE kernel; bfloat16: the vendor library's batched product with 32-bit sums."""
    if x.dtype == torch.float32:
        gemm_f32_nt_batched(x.transpose(0, 1), w, out.transpose(0, 1))
    else:
        _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    return out


PAIRINGS = {"half": 0, "interleaved": 1}     # which features a rotation pairs: (i, i + n/2) or (2i, 2i + 1)


def latent_prepare(down: torch.Tensor, q_weight: Optional[torch.Tensor], kv_weight: torch.Tensor, eps: float,
                   rot: Optional[torch.Tensor], rot_dims: int, pairing: str, slots: Optional[torch.Tensor],
                   cq: Optional[torch.Tensor], cache: Optional[torch.Tensor], q_rank: int, kv_rank: int,
                   rot_dim: int) -> None:
    """Rows of ``down`` = [query latent | key/value latent | shared key part].  ``cq`` gets the
    normed query latent; the token's row of ``cache`` ([pages, 1, page_size, width], named by
    ``slots``) gets [normed key/value latent | shared key part, its first ``rot_dims`` features
    rotated | zeros]."""
    _check(down, "down", dense=False)
    tokens = down.shape[0]
    if down.dim() != 2 or down.stride(1) != 1 or down.shape[1] != q_rank + kv_rank + rot_dim:
        raise KernelError(f"latent_prepare: down is {tuple(down.shape)}, expected width {q_rank + kv_rank + rot_dim}")
    _check(kv_weight, "kv_weight", torch.float32)
    if kv_weight.numel() != kv_rank:
        raise KernelError("latent_prepare: the key/value norm weight does not have kv_rank elements")
    if q_rank:
        _check(q_weight, "q_weight", torch.float32); _check(cq, "cq", down.dtype)
        if q_weight.numel() != q_rank or cq.shape != (tokens, q_rank):
            raise KernelError("latent_prepare: the query latent's weight or output does not have q_rank columns")
    width = kv_rank + rot_dim
    if slots is not None:
        _check(slots, "slots", torch.int32); _check(cache, "cache", down.dtype)
        if slots.numel() != tokens or cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] < width:
            raise KernelError(f"latent_prepare: cache is {tuple(cache.shape)}, expected [pages, 1, page_size, >= {width}]")
        width = cache.shape[3]
    if rot_dims:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rot_dims // 2, 2):
            raise KernelError(f"latent_prepare: rot is {tuple(rot.shape)}, expected {(tokens, rot_dims // 2, 2)}")
    _lib.core().call("mrun_latent_prepare", _ptr(down), dtype_code(down.dtype), _c_long(down.stride(0)),
                     _ptr(q_weight), _ptr(kv_weight), _c_float(eps), _ptr(rot), _c_int(rot_dims),
                     _c_int(PAIRINGS[pairing]), _ptr(slots), _ptr(cq), _ptr(cache if slots is not None else None),
                     _c_int(tokens), _c_int(q_rank), _c_int(kv_rank), _c_int(rot_dim), _c_int(width), _stream())


def latent_query(q: torch.Tensor, rot: Optional[torch.Tensor], rot_dims: int, pairing: str, q_att: torch.Tensor,
                 heads: int, dim: int, rot_dim: int, kv_rank: int) -> None:
    """``q`` [tokens, heads * (dim + rot_dim)] (rows may be strided); fills ``q_att[t, h, kv_rank:]``
    with the head's rotated part and zeros ([tokens, heads, width])."""
    ldq = _strided_rows(q, "q"); _check(q_att, "q_att", q.dtype)
    tokens = q.shape[0]
    if q.shape != (tokens, heads * (dim + rot_dim)) or q_att.dim() != 3 or q_att.shape[:2] != (tokens, heads) \
            or q_att.shape[2] < kv_rank + rot_dim:
        raise KernelError(f"latent_query: q {tuple(q.shape)}, q_att {tuple(q_att.shape)}")
    if rot_dims:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rot_dims // 2, 2):
            raise KernelError(f"latent_query: rot is {tuple(rot.shape)}, expected {(tokens, rot_dims // 2, 2)}")
    _lib.core().call("mrun_latent_query", _ptr(q), _c_long(ldq), dtype_code(q.dtype), _ptr(rot), _c_int(rot_dims),
                     _c_int(PAIRINGS[pairing]), _ptr(q_att), _c_int(tokens), _c_int(heads), _c_int(dim),
                     _c_int(rot_dim), _c_int(kv_rank), _c_int(q_att.shape[2]), _stream())


def post_norm_add(stream: torch.Tensor, branch: torch.Tensor, w_post: torch.Tensor, scale: float, eps_post: float,
                  w_next: Optional[torch.Tensor], eps_next: float, out: Optional[torch.Tensor],
                  rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """stream += scale * rmsnorm(branch) * w_post (32-bit, in place), then out = rmsnorm(stream) *
    w_next (skipped when ``w_next`` is None).  With ``rows`` only those rows are computed and the
    stream is left as it is.  ``branch`` is float32."""
    _check(stream, "stream", torch.float32); _check(branch, "branch", torch.float32)
    _check(w_post, "w_post", torch.float32)
    hidden = stream.shape[1]
    n_rows = stream.shape[0] if rows is None else rows.numel()
    if branch.shape != stream.shape or w_post.numel() != hidden:
        raise KernelError(f"post_norm_add: stream {tuple(stream.shape)}, branch {tuple(branch.shape)}, weight {w_post.numel()}")
    code = F32
    if w_next is not None:
        _check(w_next, "w_next", torch.float32); _check(out, "out")
        if w_next.numel() != hidden or out.shape != (n_rows, hidden):
            raise KernelError(f"post_norm_add: out {tuple(out.shape)}, expected {(n_rows, hidden)}")
        code = dtype_code(out.dtype)
    if rows is not None:
        _check(rows, "rows", torch.int32)
    _lib.core().call("mrun_post_norm_add", _ptr(stream), _ptr(branch), _ptr(w_post), _c_float(scale),
                     _c_float(eps_post), _ptr(w_next), _c_float(eps_next), _ptr(out if w_next is not None else None),
                     _c_int(code), _ptr(rows), _c_int(n_rows), _c_int(hidden), _stream())
    return out


ROUTER_SCORES = {"softmax": 0, "sigmoid": 1, "logit": 2}


def route_top_k(logits: torch.Tensor, top: int, score: str = "softmax", renormalize: bool = False,
                chosen: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [tokens, experts]: each token's ``top`` largest scores at their experts' places
    (divided by their sum if ``renormalize``), zero elsewhere.  ``score`` = ``"logit"``: the logits
    themselves are ranked and the chosen experts weigh the softmax over the chosen logits only.
    ``bias`` (float32, one entry an expert) is added to the logits first.  ``logits`` may be the
    first columns of wider rows (a product padded to a vendor-friendly width)."""
    _check(logits, "logits", torch.float32, dense=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError(f"route_top_k: logits has strides {logits.stride()}, expected rows of unit stride")
    tokens, experts = logits.shape
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != experts:
            raise KernelError(f"route_top_k: bias has {bias.numel()} entries for {experts} experts")
    weights = torch.empty((tokens, experts), dtype=torch.float32, device=logits.device)
    if chosen is not None:
        _check(chosen, "chosen", torch.int32)
        if chosen.shape != (tokens, top):
            raise KernelError(f"route_top_k: chosen is {tuple(chosen.shape)}, expected {(tokens, top)}")
    _lib.core().call("mrun_route_top_k", _ptr(logits), _c_long(logits.stride(0)), _ptr(bias), _ptr(weights), _ptr(chosen),
                     _c_int(tokens), _c_int(experts), _c_int(top), _c_int(ROUTER_SCORES[score]),
                     _c_int(1 if renormalize else 0), _stream())
    return weights


def relu2_scaled(u: torch.Tensor, weights: Optional[torch.Tensor], experts: int, ff: int) -> torch.Tensor:
    """relu(u)^2 column by column; column c < experts * ff is also multiplied by
    ``weights[t, c // ff]`` (float32 [tokens, experts]); later columns are not."""
    _check(u, "u")
    tokens, columns = u.shape
    if weights is not None:
        _check(weights, "weights", torch.float32)
        if weights.shape != (tokens, experts):
            raise KernelError(f"relu2_scaled: weights {tuple(weights.shape)}, expected {(tokens, experts)}")
    else:
        experts, ff = 0, columns
    act = torch.empty_like(u)
    _lib.core().call("mrun_relu2_scaled", _ptr(u), _ptr(act), dtype_code(u.dtype), _ptr(weights), _c_int(tokens),
                     _c_int(columns), _c_int(experts), _c_int(max(1, ff)), _stream())
    return act


def soft_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place on float32."""
    _check(x, "x", torch.float32)
    _lib.core().call("mrun_soft_cap", _ptr(x), _c_long(x.numel()), _c_float(cap), _stream())
    return x


def scale(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place on float32."""
    _check(x, "x", torch.float32)
    _lib.core().call("mrun_scale_f32", _ptr(x), _c_long(x.numel()), _c_float(factor), _stream())
    return x


# ------------------------------------------------------------------ a routed feed-forward's rows sorted by expert

def moe_sort(chosen: torch.Tensor, weights: torch.Tensor):
    """Sorts the (token, chosen expert) pairs by expert.  ``chosen``: int32 [tokens, top];
    ``weights``: float32 [tokens, experts].  Returns ``ends`` (int32 [experts]: where each expert's
    rows end), ``source`` (int32 [pairs]: the token of every row), ``row_weight`` (float32
    [pairs]) and ``dest`` (int32 [tokens, top]: the row of every pair)."""
    _check(chosen, "chosen", torch.int32); _check(weights, "weights", torch.float32)
    tokens, top = chosen.shape
    experts = weights.shape[1]
    if weights.shape[0] != tokens:
        raise KernelError(f"moe_sort: chosen {tuple(chosen.shape)} vs weights {tuple(weights.shape)}")
    dev = chosen.device
    books = torch.zeros((3, experts), dtype=torch.int32, device=dev)          # counts, ends, cursor
    source = torch.empty(tokens * top, dtype=torch.int32, device=dev)
    row_weight = torch.empty(tokens * top, dtype=torch.float32, device=dev)
    dest = torch.empty((tokens, top), dtype=torch.int32, device=dev)
    _lib.core().call("mrun_moe_sort", _ptr(chosen), _ptr(weights), _c_int(tokens), _c_int(experts), _c_int(top),
                     _ptr(books[0]), _ptr(books[1]), _ptr(books[2]), _ptr(source), _ptr(row_weight), _ptr(dest), _stream())
    return books[1], source, row_weight, dest


def gather_rows(x: torch.Tensor, source: torch.Tensor) -> torch.Tensor:
    """out[r] = x[source[r]]."""
    _check(x, "x"); _check(source, "source", torch.int32)
    out = torch.empty((source.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _lib.core().call("mrun_gather_rows", _ptr(x), dtype_code(x.dtype), _ptr(source), _ptr(out), _c_int(source.numel()),
                     _c_int(x.shape[1]), _stream())
    return out


def relu2_rows(u: torch.Tensor, row_weight: torch.Tensor) -> torch.Tensor:
    """relu(u)^2 times the row's weight."""
    _check(u, "u"); _check(row_weight, "row_weight", torch.float32)
    if row_weight.numel() != u.shape[0]:
        raise KernelError("relu2_rows: one weight per row is needed")
    act = torch.empty_like(u)
    _lib.core().call("mrun_relu2_rows", _ptr(u), _ptr(act), dtype_code(u.dtype), _ptr(row_weight), _c_int(u.shape[0]),
                     _c_int(u.shape[1]), _stream())
    return act


def combine_rows(base: Optional[torch.Tensor], rows: torch.Tensor, dest: torch.Tensor) -> torch.Tensor:
    """float32 out[t] = base[t] + sum over k of rows[dest[t, k]], added in the order of k."""
    _check(rows, "rows", torch.bfloat16); _check(dest, "dest", torch.int32)
    tokens, top = dest.shape
    width = rows.shape[1]
    if base is not None:
        _check(base, "base")
        if base.shape != (tokens, width) or base.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError(f"combine_rows: base {tuple(base.shape)} {base.dtype}")
    out = torch.empty((tokens, width), dtype=torch.float32, device=rows.device)
    _lib.core().call("mrun_combine_rows", _ptr(base), _c_int(1 if base is not None and base.dtype == torch.float32 else 0),
                     _ptr(rows), dtype_code(rows.dtype), _ptr(dest), _ptr(out), _c_int(tokens), _c_int(top),
                     _c_int(width), _stream())
    return out


def grouped_linear(x: torch.Tensor, w: torch.Tensor, ends: torch.Tensor) -> torch.Tensor:
    """y[r] = x[r] @ w[g].T for the rows r of group g (rows ends[g-1] .. ends[g]): the vendor
    library's grouped product in bfloat16 with 32-bit sums.  ``w``: [groups, out, in], which may
    be a strided view as long as ``in`` has unit stride."""
    _check(x, "x", torch.bfloat16); _check(w, "w", torch.bfloat16, dense=False); _check(ends, "ends", torch.int32)
    return torch.nn.functional.grouped_mm(x, w.transpose(-2, -1), offs=ends)


# ------------------------------------------------------------------ several residual streams a token

def embed_streams(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, copies: int) -> torch.Tensor:
    """out[t, s] = float(table[ids[t]]) for each of the ``copies`` streams; out is float32
    [tokens, copies * hidden]."""
    _check(table, "table"); _check(ids, "ids", torch.int32); _check(out, "out", torch.float32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out.shape != (tokens, copies * hidden):
        raise KernelError(f"embed_streams: out is {tuple(out.shape)}, expected {(tokens, copies * hidden)}")
    _lib.core().call("mrun_embed_streams", _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), _c_int(tokens),
                     _c_int(hidden), _c_int(vocab), _c_int(copies), _stream())
    return out


def embed_bigram(table: torch.Tensor, pairs: Optional[torch.Tensor], ids: torch.Tensor, positions: torch.Tensor,
                 token_slot: torch.Tensor, state: Optional[torch.Tensor], out: torch.Tensor, copies: int, scale: float,
                 buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """out[t, s] = table[ids[t]] * scale + pairs[row(t)] for each of the ``copies`` streams; row(t)
    = (previous token * mul_prev + token * mul_cur) mod buckets, row ``buckets`` at position 0.
    ``state`` (int32 [slots, 1]) holds the last token every request brought and is left up to
    date.  ``pairs`` None: the scaled row alone.  Padding rows (negative position) become zero."""
    _check(table, "table"); _check(ids, "ids", torch.int32); _check(out, "out", torch.float32)
    _check(positions, "positions", torch.int32); _check(token_slot, "token_slot", torch.int32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out.shape != (tokens, copies * hidden):
        raise KernelError(f"embed_bigram: out is {tuple(out.shape)}, expected {(tokens, copies * hidden)}")
    rows = None
    if pairs is not None:
        _check(pairs, "pairs", table.dtype); _check(state, "state", torch.int32)
        if pairs.shape != (buckets + 1, hidden):
            raise KernelError(f"embed_bigram: pairs is {tuple(pairs.shape)}, expected {(buckets + 1, hidden)}")
        rows = torch.empty(tokens, dtype=torch.int32, device=ids.device)
    _lib.core().call("mrun_embed_bigram", _ptr(table), _ptr(pairs), dtype_code(table.dtype), _ptr(ids), _ptr(positions),
                     _ptr(token_slot), _ptr(state), _ptr(rows), _ptr(out), _c_int(tokens), _c_int(hidden), _c_int(vocab),
                     _c_int(copies), _c_float(scale), _c_int(buckets), _c_long(mul_prev), _c_long(mul_cur), _stream())
    return out


class PendingStreams:
    """A sublayer's output (float32 rows) that has not been written into the token's streams yet,
    with the coefficients of the write: x_t <- sum_s mix[s, t] x_s + out[t] * y (``mix`` and
    ``out`` None: the plain residual sum).  The next read of the streams applies it
    (:func:`streams_step`)."""

    def __init__(self, y: torch.Tensor, mix: Optional[torch.Tensor], out: Optional[torch.Tensor]):
        self.y, self.mix, self.out = y, mix, out


def streams_step(streams: torch.Tensor, pending: Optional[PendingStreams], in_c: Optional[torch.Tensor],
                 norm_weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype, count: int,
                 rows: Optional[torch.Tensor] = None, want_sum: bool = False):
    """Applies the pending write to the ``count`` streams of every token (float32 [tokens, count *
    width], in place), forms u = sum_s in_c[s] x_s (``in_c`` None: the plain sum) and returns its
    RMS norm times ``norm_weight`` in ``out_dtype`` (``want_sum``: the 32-bit u itself instead).
    With ``rows`` (int32) only those tokens are read and the streams stay as they are."""
    _check(streams, "streams", torch.float32)
    tokens = streams.shape[0]
    width = streams.shape[1] // count
    n_rows = tokens if rows is None else rows.numel()
    y = mix = out_c = None
    if pending is not None:
        y, mix, out_c = pending.y, pending.mix, pending.out
        _check(y, "y", torch.float32)
        if y.shape != (tokens, width):
            raise KernelError(f"streams_step: the pending output is {tuple(y.shape)}, expected {(tokens, width)}")
        for name, c, n in (("mix", mix, count * count), ("out", out_c, count)):
            if c is not None:
                _check(c, name, torch.float32)
                if c.numel() != n:
                    raise KernelError(f"streams_step: {name} has {c.numel()} entries, expected {n}")
    if in_c is not None:
        _check(in_c, "in", torch.float32)
        if in_c.numel() != count:
            raise KernelError(f"streams_step: in has {in_c.numel()} entries, expected {count}")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    h = u = None
    if want_sum:
        u = torch.empty((n_rows, width), dtype=torch.float32, device=streams.device)
    else:
        _check(norm_weight, "norm_weight", torch.float32)
        if norm_weight.numel() != width:
            raise KernelError(f"streams_step: the norm weight has {norm_weight.numel()} entries, the width is {width}")
        h = torch.empty((n_rows, width), dtype=out_dtype, device=streams.device)
    _lib.core().call("mrun_streams_step", _ptr(streams), _ptr(y), _ptr(mix), _ptr(out_c), _ptr(in_c),
                     _ptr(None if want_sum else norm_weight), _c_float(eps), _ptr(h),
                     _c_int(dtype_code(out_dtype if h is not None else torch.float32)), _ptr(u), _ptr(rows),
                     _c_int(n_rows), _c_int(count), _c_int(width), _stream())
    return u if want_sum else h


# ------------------------------------------------------------------ recurrent mixers

def causal_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, ctx, residual: bool, silu: bool) -> torch.Tensor:
    """Causal convolution per channel over each request's tokens (the last tap meets the token
    itself), added to x (``residual``) and/or passed through SiLU.  ``x``: [tokens, channels],
    rows may be strided; ``weight``: float32 [channels, taps]; ``state``: [slots, taps - 1,
    channels] in x's dtype, the request's last inputs, read and left up to date (empty with one
    tap, which sees the token itself only)."""
    _check(x, "x", dense=False); _check(weight, "weight", torch.float32); _check(state, "state", x.dtype)
    tokens, channels = x.shape
    taps = weight.shape[1]
    if x.stride(1) != 1 or weight.shape[0] != channels or state.shape[1:] != (taps - 1, channels):
        raise KernelError(f"causal_conv: x {tuple(x.shape)}, weight {tuple(weight.shape)}, state {tuple(state.shape)}")
    out = torch.empty((tokens, channels), dtype=x.dtype, device=x.device)
    _lib.core().call("mrun_causal_conv", _ptr(x), _c_long(x.stride(0)), _ptr(weight), _ptr(state), _ptr(out),
                     _c_long(channels), dtype_code(x.dtype), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot),
                     _c_int(ctx.num_segments), _c_int(ctx.max_q_len), _c_int(channels), _c_int(taps),
                     _c_int(1 if residual else 0), _c_int(1 if silu else 0), _stream())
    return out


def _strided_rows(t: torch.Tensor, name: str) -> int:
    _check(t, name, dense=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be rows of contiguous features")
    return t.stride(0)


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx,
               heads: int, dim: int, vdim: int, silu_inputs: bool) -> torch.Tensor:
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over each request's tokens, from
    and into ``state`` (float32 [slots, heads, dim, vdim]).  q, k, v: column slices of one matrix
    of rows.  Returns float32 [tokens, heads * vdim]."""
    ld = _strided_rows(q, "q")
    if _strided_rows(k, "k") != ld or _strided_rows(v, "v") != ld or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("decay_scan: q, k and v must be slices of one matrix")
    _check(decay, "decay", torch.float32); _check(state, "state", torch.float32)
    tokens = q.shape[0]
    if q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim \
            or state.shape[1:] != (heads, dim, vdim) or decay.numel() != heads:
        raise KernelError("decay_scan: sizes do not match")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    scratch = torch.empty(tokens * (2 * heads * dim + heads * vdim), dtype=torch.float32, device=q.device)
    _lib.core().call("mrun_decay_scan", _ptr(q), _ptr(k), _ptr(v), _c_long(ld), dtype_code(q.dtype), _ptr(decay),
                     _ptr(state), _ptr(out), _ptr(scratch), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot),
                     _c_int(ctx.num_segments), _c_int(tokens), _c_int(heads), _c_int(dim), _c_int(vdim),
                     _c_int(1 if silu_inputs else 0), _stream())
    return out


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, ctx, heads: int, kv_heads: int,
               dim: int, vdim: int) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over each request's tokens (see
    ``csrc/recurrent.cu``).  q, k ([tokens, kv_heads * dim]) and v ([tokens, heads * vdim]):
    column slices of one matrix; ``a``: float32 [tokens, heads * dim]; ``b``: [tokens, heads],
    rows may be strided.  Returns float32 [tokens, heads * vdim]."""
    ld = _strided_rows(q, "q")
    if _strided_rows(k, "k") != ld or _strided_rows(v, "v") != ld or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("delta_scan: q, k and v must be slices of one matrix")
    ldb = _strided_rows(b, "b")
    _check(a, "a", torch.float32); _check(a_log, "a_log", torch.float32); _check(dt_bias, "dt_bias", torch.float32)
    _check(state, "state", torch.float32)
    tokens = q.shape[0]
    if q.shape[1] != kv_heads * dim or k.shape[1] != kv_heads * dim or v.shape[1] != heads * vdim \
            or a.shape != (tokens, heads * dim) or b.shape != (tokens, heads) or b.dtype != q.dtype \
            or a_log.numel() != heads or dt_bias.numel() != heads * dim or state.shape[1:] != (heads, dim, vdim):
        raise KernelError("delta_scan: sizes do not match")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    scratch = torch.empty(tokens * (2 * kv_heads * dim + heads * (vdim + dim + 1)), dtype=torch.float32, device=q.device)
    _lib.core().call("mrun_delta_scan", _ptr(q), _ptr(k), _ptr(v), _c_long(ld), dtype_code(q.dtype),
                     _c_int(heads // kv_heads), _ptr(a), _ptr(b), _c_long(ldb), _ptr(a_log), _ptr(dt_bias), _ptr(state),
                     _ptr(out), _ptr(scratch), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot), _c_int(ctx.num_segments),
                     _c_int(tokens), _c_int(heads), _c_int(dim), _c_int(vdim), _stream())
    return out


def gated_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, bias: torch.Tensor, tau: float,
               state: torch.Tensor, ctx, heads: int, dim: int, vdim: int) -> torch.Tensor:
    """Linear attention with a decay per head and key channel over each request's tokens: g =
    sigmoid(a + bias)^(1 / tau), S <- g * S (rows) + k v^T, o = S^T (q * dim^-1/2), from and into
    ``state`` (float32 [slots, heads, dim, vdim]).  q, k ([tokens, heads * dim]) and v ([tokens,
    heads * vdim]): column slices of one matrix; ``a``: float32 [tokens, heads * dim]; ``bias``:
    float32 [heads * dim].  Returns float32 [tokens, heads * vdim]."""
    ld = _strided_rows(q, "q")
    if _strided_rows(k, "k") != ld or _strided_rows(v, "v") != ld or k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("gated_scan: q, k and v must be slices of one matrix")
    _check(a, "a", torch.float32); _check(bias, "bias", torch.float32); _check(state, "state", torch.float32)
    tokens = q.shape[0]
    if q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim \
            or a.shape != (tokens, heads * dim) or bias.numel() != heads * dim or state.shape[1:] != (heads, dim, vdim):
        raise KernelError("gated_scan: sizes do not match")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    scratch = torch.empty(tokens * heads * (3 * dim + vdim), dtype=torch.float32, device=q.device)
    _lib.core().call("mrun_gated_scan", _ptr(q), _ptr(k), _ptr(v), _c_long(ld), dtype_code(q.dtype), _ptr(a), _ptr(bias),
                     _c_float(tau), _ptr(state), _ptr(out), _ptr(scratch), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot),
                     _c_int(ctx.num_segments), _c_int(tokens), _c_int(heads), _c_int(dim), _c_int(vdim), _stream())
    return out


GATE_SHAPES = {"sigmoid": 0, "silu": 1}        # what a gated norm passes its gate through


def gated_norm(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float, groups: int,
               out_dtype: torch.dtype, gate_function: str = "sigmoid") -> torch.Tensor:
    """Per group of ``o.shape[1] // groups`` features: o / sqrt(mean(o^2) + eps) * weight *
    f(gate), f the sigmoid or SiLU (``gate_function``).  ``o``: float32 [tokens, features]; ``weight``: float32, one entry per feature
    of a row or of a group; ``gate``: [tokens, features] in ``out_dtype``, rows may be strided."""
    _check(o, "o", torch.float32); _check(weight, "weight", torch.float32)
    ldg = _strided_rows(gate, "gate")
    tokens, features = o.shape
    n = features // groups
    if gate.shape != o.shape or gate.dtype != out_dtype or weight.numel() not in (n, features) or n * groups != features:
        raise KernelError("gated_norm: sizes do not match")
    out = torch.empty((tokens, features), dtype=out_dtype, device=o.device)
    _lib.core().call("mrun_gated_norm", _ptr(o), _ptr(weight), _c_int(weight.numel()), _ptr(gate), _c_long(ldg),
                     dtype_code(out_dtype), _c_float(eps), _ptr(out), _c_int(tokens), _c_int(groups), _c_int(n),
                     _c_int(GATE_SHAPES[gate_function]), _stream())
    return out


def head_gate(y: torch.Tensor, gate: torch.Tensor, heads: int) -> torch.Tensor:
    """In place: every head of ``y`` ([tokens, heads * n]) times the 32-bit sigmoid of its entry
    of ``gate`` ([tokens, heads] in the dtype of ``y``, rows may be strided)."""
    _check(y, "y")
    ldg = _strided_rows(gate, "gate")
    tokens, features = y.shape
    if gate.shape != (tokens, heads) or gate.dtype != y.dtype or features % heads:
        raise KernelError("head_gate: sizes do not match")
    _lib.core().call("mrun_head_gate", _ptr(y), _ptr(gate), _c_long(ldg), dtype_code(y.dtype), _c_int(tokens), _c_int(heads),
                     _c_int(features // heads), _stream())
    return y


# ------------------------------------------------------------------ differential attention

def diff_rope_cache(qkv: torch.Tensor, rot: Optional[torch.Tensor], rot_dims: int, slots: Optional[torch.Tensor],
                    k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                    page_size: int) -> None:
    """Rotates the q and k vectors of ``qkv`` ([tokens, 2 heads dim | 2 kv_heads dim | kv_heads
    vdim], maps outermost) in place and stores k and v in the pages ``slots`` names (key pages
    [2, pages, kv_heads, page, dim], value pages [chunks, pages, kv_heads, page, vdim / chunks])."""
    _check(qkv, "qkv"); _check(k_cache, "k_cache", qkv.dtype); _check(v_cache, "v_cache", qkv.dtype)
    tokens = qkv.shape[0]
    chunks, pages = v_cache.shape[0], v_cache.shape[1]
    if k_cache.shape != (2, pages, kv_heads, page_size, dim) or v_cache.shape != (chunks, pages, kv_heads, page_size, vdim // chunks) \
            or qkv.shape[1] != 2 * heads * dim + 2 * kv_heads * dim + kv_heads * vdim:
        raise KernelError("diff_rope_cache: sizes do not match")
    if rot is not None:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rot_dims // 2, 2):
            raise KernelError(f"diff_rope_cache: rot is {tuple(rot.shape)}")
    if slots is not None:
        _check(slots, "slots", torch.int32)
    _lib.core().call("mrun_diff_rope_cache", _ptr(qkv), _c_long(qkv.stride(0)), dtype_code(qkv.dtype), _ptr(rot),
                     _c_int(rot_dims if rot is not None else 0), _ptr(slots), _ptr(k_cache), _ptr(v_cache), _c_long(pages),
                     _c_int(tokens), _c_int(heads), _c_int(kv_heads), _c_int(dim), _c_int(vdim), _c_int(vdim // chunks),
                     _c_int(page_size), _stream())


def diff_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                   token_slot: torch.Tensor, positions: torch.Tensor, heads: int, vdim: int, scale: float,
                   lam: float, eps: float, out_scale: float, window: int = 0) -> torch.Tensor:
    """Both maps of a differential attention, their combination a1 - lam * a2 and the head norm
    (times ``out_scale``) in one kernel on CUDA cores, 32-bit arithmetic.  ``q``: rows [2, heads,
    dim], may be a column slice of a wider matrix."""
    ld = _strided_rows(q, "q")
    _check(k_cache, "k_cache", q.dtype); _check(v_cache, "v_cache", q.dtype)
    _check(block_tables, "block_tables", torch.int32); _check(token_slot, "token_slot", torch.int32)
    _check(positions, "positions", torch.int32)
    maps, pages, kv_heads, page_size, dim = k_cache.shape
    tokens = positions.numel()
    if maps != 2 or q.shape != (tokens, 2 * heads * dim) or v_cache.shape[1:4] != (pages, kv_heads, page_size) \
            or v_cache.shape[0] * v_cache.shape[4] != vdim:
        raise KernelError("diff_attention: sizes do not match")
    out = torch.empty((tokens, heads * vdim), dtype=q.dtype, device=q.device)
    _lib.core().call("mrun_diff_attention", _ptr(q), _c_long(ld), _ptr(out), _ptr(k_cache), _ptr(v_cache),
                     dtype_code(q.dtype), _ptr(block_tables), _c_int(block_tables.shape[1]), _ptr(token_slot),
                     _ptr(positions), _c_long(pages), _c_int(tokens), _c_int(heads), _c_int(kv_heads), _c_int(dim),
                     _c_int(vdim), _c_int(v_cache.shape[4]), _c_int(page_size), _c_float(scale), _c_float(lam),
                     _c_float(eps), _c_float(out_scale), _c_int(window), _stream())
    return out


def diff_combine(maps: torch.Tensor, heads: int, vdim: int, lam: float, eps: float, out_scale: float) -> torch.Tensor:
    """``maps``: [2, chunks, tokens, heads * vdim / chunks], the maps' outputs chunk by chunk;
    returns (a1 - lam * a2) / rms over each head's ``vdim`` values * ``out_scale``."""
    _check(maps, "maps")
    two, chunks, tokens, row = maps.shape
    if two != 2 or row * chunks != heads * vdim:
        raise KernelError("diff_combine: sizes do not match")
    out = torch.empty((tokens, heads * vdim), dtype=maps.dtype, device=maps.device)
    _lib.core().call("mrun_diff_combine", _ptr(maps), _ptr(out), dtype_code(maps.dtype), _c_int(tokens), _c_int(heads),
                     _c_int(vdim), _c_int(vdim // chunks), _c_float(lam), _c_float(eps), _c_float(out_scale), _stream())
    return out


# ------------------------------------------------------------------ experts chosen by a table

def table_route(token_ids: torch.Tensor, table: torch.Tensor, experts: int, chosen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [tokens, experts]: 1 / top at the experts that row ``token id`` of ``table`` (int32
    [vocab, top]) names, zero elsewhere; ``chosen`` (int32 [tokens, top]) gets the experts."""
    _check(token_ids, "token_ids", torch.int32); _check(table, "table", torch.int32)
    tokens = token_ids.numel()
    vocab, top = table.shape
    weights = torch.empty((tokens, experts), dtype=torch.float32, device=token_ids.device)
    if chosen is not None:
        _check(chosen, "chosen", torch.int32)
        if chosen.shape != (tokens, top):
            raise KernelError(f"table_route: chosen is {tuple(chosen.shape)}, expected {(tokens, top)}")
    _lib.core().call("mrun_table_route", _ptr(token_ids), _ptr(table), _ptr(weights), _ptr(chosen), _c_int(tokens),
                     _c_int(vocab), _c_int(experts), _c_int(top), _stream())
    return weights


def clamped_glu(u: torch.Tensor, weights: Optional[torch.Tensor], blocks: int, ff: int, limit: float, alpha: float,
                up_offset: float = 1.0, out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``u``: [rows, blocks * 2 * ff], a block of [gate | up] columns per expert.  Returns [rows,
    blocks * ff]: g * sigmoid(alpha * g) * (clamp(up, +-limit) + up_offset) with g = min(gate,
    limit), times ``weights[row, block]`` (float32 [rows, blocks]) or ``weights[row]`` (float32
    [rows]).  ``limit`` infinite: no clamp (alpha = 1 and up_offset = 0: SiLU(gate) * up).  ``u``,
    ``weights`` and ``out`` may be column slices of wider matrices.  ``bias`` (float32, laid out like a
    row of ``u``) is added to gate and up before the clamp: the projections' biases, never rounded
    into ``u``."""
    ldu = _strided_rows(u, "u")
    rows = u.shape[0]
    if u.shape[1] != blocks * 2 * ff:
        raise KernelError(f"clamped_glu: u is {tuple(u.shape)}, expected width {blocks * 2 * ff}")
    per_block, ldw = 0, 0
    if weights is not None:
        _check(weights, "weights", torch.float32, dense=False)
        if weights.dim() == 2 and weights.shape == (rows, blocks) and weights.stride(1) == 1:
            per_block, ldw = 1, weights.stride(0)
        elif weights.dim() == 1 and weights.numel() == rows:
            ldw = weights.stride(0)
        elif weights.dim() == 2 and weights.shape == (rows, 1):
            ldw = weights.stride(0)
        else:
            raise KernelError(f"clamped_glu: weights {tuple(weights.shape)}")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != blocks * 2 * ff:
            raise KernelError(f"clamped_glu: bias has {bias.numel()} entries, a row has {blocks * 2 * ff}")
    if out is None:
        out = torch.empty((rows, blocks * ff), dtype=u.dtype, device=u.device)
    lda = _strided_rows(out, "out")
    if out.shape != (rows, blocks * ff) or out.dtype != u.dtype:
        raise KernelError(f"clamped_glu: out is {tuple(out.shape)} {out.dtype}")
    _lib.core().call("mrun_clamped_glu", _ptr(u), _c_long(ldu), _ptr(out), _c_long(lda), dtype_code(u.dtype), _ptr(weights),
                     _c_long(ldw), _c_int(per_block), _c_int(rows), _c_int(blocks), _c_int(ff), _c_float(limit),
                     _c_float(alpha), _c_float(up_offset), _ptr(bias), _stream())
    return out


def route_grouped(logits: torch.Tensor, experts: int, top: int, groups: int, keep: int, group_top: int, scale: float,
                  chosen: Optional[torch.Tensor] = None):
    """The choice of a router with sigmoid scores over groups of experts.  ``logits``: float32
    [tokens, experts] or [tokens, experts + 1] (the last column the gate of a shared expert).
    Returns (float32 [tokens, experts]: score / (sum of the chosen + 1e-20) * ``scale`` at the
    chosen experts, zero elsewhere; float32 [tokens]: the sigmoid of the last column, or None).
    The experts form ``groups`` equal groups of neighbours, a group's score is the sum of its
    ``group_top`` largest scores, and only experts of the ``keep`` best groups can be chosen.
    ``logits`` may be the first columns of wider rows (a product padded to a vendor-friendly
    width): its row stride is passed on."""
    _check(logits, "logits", torch.float32, dense=False)
    tokens, columns = logits.shape
    if columns not in (experts, experts + 1):
        raise KernelError(f"route_grouped: logits is {tuple(logits.shape)}, expected {experts} or {experts + 1} columns")
    if logits.stride(1) != 1 or logits.stride(0) < columns:
        raise KernelError(f"route_grouped: logits has strides {logits.stride()}, expected rows of unit stride")
    weights = torch.empty((tokens, experts), dtype=torch.float32, device=logits.device)
    shared = torch.empty(tokens, dtype=torch.float32, device=logits.device) if columns > experts else None
    if chosen is not None:
        _check(chosen, "chosen", torch.int32)
        if chosen.shape != (tokens, top):
            raise KernelError(f"route_grouped: chosen is {tuple(chosen.shape)}, expected {(tokens, top)}")
    _lib.core().call("mrun_route_grouped", _ptr(logits), _c_long(logits.stride(0)), _ptr(weights), _ptr(shared), _ptr(chosen),
                     _c_int(tokens), _c_int(experts), _c_int(top), _c_int(groups), _c_int(keep), _c_int(group_top),
                     _c_float(scale), _stream())
    return weights, shared
