"""Python face of the CUDA kernels: argument checks, then a ``ctypes`` call on the current stream.

Every function here launches hand-written kernels from this folder (matrix products
with many rows go to cuBLAS through ``torch.matmul``, as the reference's prefill does
with ``cublasGemmEx``/``cublasSgemm``, src/gpu_cuda.cu:11788-11879).  Nothing falls
back to the CPU: tensors that are not on a CUDA device are refused.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build

PAGE = 64  # tokens per cache page; must equal BN_PAGE in common.cuh

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly:
    ``torch.cuda.current_stream()`` builds a Python object per call, several microseconds of a launch)."""
    try:
        return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))
    except AttributeError:  # a torch without these entry points
        return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    # the usual case in one test (a launch asks this of ten tensors); what fails it is named below
    if (t.__class__ is torch.Tensor and t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype is dtype)
            and (dims is None or t.dim() == dims)):
        return
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got {tuple(t.shape)}")


def _check(status: int, what: str) -> None:
    if status == 0:
        return
    if status == 1:
        raise KernelError(f"{what}: sizes or pointers refused by the kernel launcher")
    raise KernelError(f"{what}: CUDA launch failed with error {status - 2}")


LAUNCHES = 0  # kernels of this library launched through this module (bench.py reads and resets it)
PROFILE = None  # a dict while kernel classes are being timed (engine/diagnostics.py): entry point -> [(event, event)]


def _timed(key: str, call):
    """Run ``call`` between two CUDA events kept under ``key`` (only while PROFILE is a dict)."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = call()
    b.record()
    PROFILE.setdefault(key, []).append((a, b))
    return out


_entry_points = {}  # (family, name) -> the library's entry point, its result type set


def _fn(family: str, name: str):
    global LAUNCHES
    LAUNCHES += 1
    f = _entry_points.get((family, name))
    if f is None:
        f = getattr(build.library(family), name)
        f.restype = c_int
        _entry_points[(family, name)] = f
    if PROFILE is not None:
        return lambda *args: _timed(f"{family}.{name}", lambda: f(*args))
    return f


# Arguments that never change, made once: building a ctypes object costs a fifth of a microsecond, and
# a launch has twenty of them.  (Python ints go to C as int without a wrapper; pointers need c_void_p,
# an int would be cut to 32 bits; floats need c_float.)
_NULL = c_void_p(None)
_F0 = c_float(0.0)


# ---- embedding ----------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, bad_token: torch.Tensor,
                 scale: float = 1.0) -> torch.Tensor:
    """out[t] = float32(table[tokens[t]]) * scale; sets bad_token[0] = 1 on an id outside the table."""
    _need(table, "table", dims=2)
    _need(tokens, "tokens", torch.int32, 1)
    _need(out, "out", torch.float32, 2)
    _need(bad_token, "bad_token", torch.int32)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width:
        raise KernelError(f"out {tuple(out.shape)} does not hold {n} rows of width {width}")
    _check(_fn("embed", "bn_embed_gather")(_ptr(table), _code(table), _ptr(tokens), _ptr(out), int(n),
                                           int(width), int(table.shape[0]), c_float(scale),
                                           _ptr(bad_token), _stream()), "embed_gather")
    return out


EMBED_NORMED_MAX_WIDTH = (200 * 1024) // 4 - 32  # rows that fit the fused kernel's shared memory


def embed_gather_normed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, bad_token: torch.Tensor, scale: float,
                        weight: torch.Tensor, eps: float, next_weight: Optional[torch.Tensor] = None, next_eps: float = 0.0,
                        next_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """out[t] = rmsnorm(float32(table[tokens[t]]) * scale) * weight: the stream starts as the normed embedding rows.
    With ``next_weight`` also returns rmsnorm(out) * next_weight in ``next_dtype``: the first reader's norm, taken in
    the same pass.  Sets bad_token[0] = 1 on an id outside the table (its rows are zeros)."""
    _need(table, "table", dims=2)
    _need(tokens, "tokens", torch.int32, 1)
    _need(out, "out", torch.float32, 2)
    _need(bad_token, "bad_token", torch.int32)
    _need(weight, "weight", dims=1)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width or weight.shape[0] != width or width > EMBED_NORMED_MAX_WIDTH:
        raise KernelError(f"embed_gather_normed: out {tuple(out.shape)} / gain {tuple(weight.shape)} do not fit {n} rows of width {width}")
    h = None
    if next_weight is not None:
        _need(next_weight, "next_weight", dims=1)
        if next_weight.shape[0] != width:
            raise KernelError("embed_gather_normed: the reader's gain does not fit")
        h = torch.empty((n, width), dtype=next_dtype or torch.float32, device=out.device)
    _check(_fn("embed", "bn_embed_gather_normed")(
        _ptr(table), _code(table), _ptr(tokens), _ptr(out), int(n), int(width), int(table.shape[0]), c_float(scale), _ptr(weight),
        int(_code(weight)), c_float(eps), _ptr(next_weight), int(_code(next_weight)) if next_weight is not None else 0,
        c_float(next_eps), _ptr(h), int(_code(h)) if h is not None else 0, _ptr(bad_token), _stream()), "embed_gather_normed")
    return h


# ---- norm ---------------------------------------------------------------------------------
def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_x: bool = True) -> torch.Tensor:
    """x += delta (if given), out = rmsnorm(x) * weight.  With ``rows`` only those rows are read
    and ``out`` holds them densely; x is then left as it is."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", dims=1)
    _need(out, "out", dims=2)
    width = x.shape[1]
    if weight.shape[0] != width or out.shape[1] != width:
        raise KernelError(f"widths differ: x {width}, weight {weight.shape[0]}, out {out.shape[1]}")
    n_parts, part_stride = 1, 0
    if delta is not None:
        _need(delta, "delta")
        if delta.dim() == 3:  # partial sums of a product that split its inner dimension
            n_parts, part_stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        if tuple(delta.shape[-2:]) != tuple(x.shape) or delta.dim() not in (2, 3):
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows, write_x = rows.shape[0], False
    else:
        n_rows = x.shape[0]
    if out.shape[0] < n_rows:
        raise KernelError(f"out has {out.shape[0]} rows, {n_rows} are written")
    _check(_fn("norm", "bn_add_rmsnorm")(_ptr(x), _ptr(delta), int(_code(delta) if delta is not None else 0),
                                         int(n_parts), ctypes.c_longlong(part_stride), _ptr(weight), int(_code(weight)), _ptr(out), int(_code(out)),
                                         _ptr(rows), int(n_rows), int(width), c_float(eps),
                                         int(1 if write_x else 0), _stream()), "add_rmsnorm")
    return out


def scaled_add_rmsnorm(x: torch.Tensor, alpha: float, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                       out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The norm after the sum: x = rmsnorm(alpha * x + delta) * weight, in place on the float32 residual;
    ``out`` (optional, any float type) receives the same rows for the products that read them next."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", dims=1)
    width = x.shape[1]
    if weight.shape[0] != width:
        raise KernelError(f"widths differ: x {width}, weight {weight.shape[0]}")
    if delta is not None:
        _need(delta, "delta", dims=2)
        if tuple(delta.shape) != tuple(x.shape):
            raise KernelError(f"delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    if out is not None:
        _need(out, "out", dims=2)
        if tuple(out.shape) != tuple(x.shape):
            raise KernelError(f"out {tuple(out.shape)} does not match x {tuple(x.shape)}")
    _check(_fn("norm", "bn_scaled_add_rmsnorm")(_ptr(x), c_float(alpha), _ptr(delta), int(_code(delta) if delta is not None else 0),
                                                _ptr(weight), int(_code(weight)), _ptr(out),
                                                int(_code(out) if out is not None else 0), int(x.shape[0]), int(width),
                                                c_float(eps), _stream()), "scaled_add_rmsnorm")
    return out


# ---- activation ---------------------------------------------------------------------------
def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate and up rows as alternating blocks of 8 rows: [g0..g7, u0..u7, g8..g15, u8..u15, ...]."""
    I, K = gate.shape
    if I % 8:
        raise KernelError(f"feed-forward width {I} must be a multiple of 8")
    return torch.stack([gate.reshape(I // 8, 8, K), up.reshape(I // 8, 8, K)], dim=1).reshape(2 * I, K).contiguous()


def silu_mul(h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_i) * up_i for rows of h that alternate 8 gate and 8 up values
    (the layout ``interleave_gate_up`` gives the product's output)."""
    _need(h, "h", dims=2)
    _need(out, "out", h.dtype, 2)
    inter = h.shape[1] // 2
    if h.shape[1] != 2 * inter or out.shape != (h.shape[0], inter):
        raise KernelError(f"silu_mul: h {tuple(h.shape)} and out {tuple(out.shape)} do not fit")
    _check(_fn("act", "bn_silu_mul")(_ptr(h), _ptr(out), int(_code(h)), int(h.shape[0]), int(inter),
                                     _stream()), "silu_mul")
    return out


def glu_mul(h: torch.Tensor, out: torch.Tensor, act: int = 0) -> torch.Tensor:
    """``silu_mul`` with the gate's activation by code (ACT_SILU, ACT_GELU_TANH)."""
    _need(h, "h", dims=2)
    _need(out, "out", h.dtype, 2)
    inter = h.shape[1] // 2
    if h.shape[1] != 2 * inter or out.shape != (h.shape[0], inter):
        raise KernelError(f"glu_mul: h {tuple(h.shape)} and out {tuple(out.shape)} do not fit")
    _check(_fn("act", "bn_glu_mul")(_ptr(h), _ptr(out), int(_code(h)), int(h.shape[0]), int(inter), int(act), _stream()),
           "glu_mul")
    return out


def gated_lookup(pre: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, dim: int, act: int = 0) -> torch.Tensor:
    """out[t, j] = act(pre[t, j]) * table[tokens[t], col0 + j] for j < dim (an id outside the table gives zeros);
    ``pre`` may be a view into wider rows; the result has ``pre``'s type."""
    if not pre.is_cuda or pre.dim() != 2 or pre.stride(1) != 1 or pre.shape[1] < dim:
        raise KernelError("gated_lookup: pre must be a CUDA matrix with unit inner stride and at least dim columns")
    _need(table, "table", dims=2)
    _need(tokens, "tokens", torch.int32, 1)
    n = tokens.shape[0]
    if pre.shape[0] < n or col0 < 0 or col0 + dim > table.shape[1]:
        raise KernelError("gated_lookup: sizes do not fit")
    out = torch.empty((n, dim), dtype=pre.dtype, device=pre.device)
    _check(_fn("act", "bn_gated_lookup")(_ptr(pre), int(pre.stride(0)), int(_code(pre)), _ptr(table), int(_code(table)),
                                         int(table.shape[1]), int(col0), int(table.shape[0]), _ptr(tokens), _ptr(out), int(n),
                                         int(dim), int(act), _stream()), "gated_lookup")
    return out


def glu_limited(h: torch.Tensor, out: torch.Tensor, limit: float, slope: float) -> torch.Tensor:
    """Rows of h hold ``inter`` gate values and then ``inter`` up values: g = min(gate, limit),
    u = clamp(up, -limit, limit), out = g * sigmoid(slope * g) * (u + 1)."""
    _need(h, "h", dims=2)
    _need(out, "out", h.dtype, 2)
    inter = h.shape[1] // 2
    if h.shape[1] != 2 * inter or tuple(out.shape) != (h.shape[0], inter):
        raise KernelError(f"glu_limited: h {tuple(h.shape)} and out {tuple(out.shape)} do not fit")
    _check(_fn("act", "bn_glu_limited")(_ptr(h), _ptr(out), int(_code(h)), int(h.shape[0]), int(inter), c_float(limit),
                                        c_float(slope), _stream()), "glu_limited")
    return out


def glu_halves(h: torch.Tensor, out: torch.Tensor, act: int = 0) -> torch.Tensor:
    """Rows of h hold ``inter`` gate values and then ``inter`` up values: out = act(gate) * up
    (ACT_SILU, ACT_GELU_TANH)."""
    _need(h, "h", dims=2)
    _need(out, "out", h.dtype, 2)
    inter = h.shape[1] // 2
    if h.shape[1] != 2 * inter or tuple(out.shape) != (h.shape[0], inter):
        raise KernelError(f"glu_halves: h {tuple(h.shape)} and out {tuple(out.shape)} do not fit")
    _check(_fn("act", "bn_glu_halves")(_ptr(h), _ptr(out), int(_code(h)), int(h.shape[0]), int(inter), int(act), _stream()),
           "glu_halves")
    return out


def scale_softcap(x: torch.Tensor, scale: float, softcap: float) -> torch.Tensor:
    """In place on float32 x: x * scale, then softcap * tanh(x / softcap) when softcap is not 0."""
    _need(x, "x", torch.float32)
    _check(_fn("act", "bn_scale_softcap")(_ptr(x), ctypes.c_longlong(x.numel()), c_float(scale), c_float(softcap),
                                          _stream()), "scale_softcap")
    return x


# ---- rotary + cache append ----------------------------------------------------------------
def rope_append(x: torch.Tensor, n_rot_heads: int, head_dim: int, rotary_dims: int, theta_scale: float,
                tok_pos: torch.Tensor, *, k_off: int = 0, v_off: int = 0, n_kv_heads: int = 0,
                tok_seq: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                page_table: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
                v_cache: Optional[torch.Tensor] = None) -> None:
    """Rotate the first ``n_rot_heads`` heads of every row of x in place; when a cache is given,
    write the key heads at ``k_off`` and the value heads at ``v_off`` of each row into it."""
    _need(x, "x", dims=2)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    n = tok_pos.shape[0]
    if x.shape[0] < n or n_rot_heads * head_dim > x.shape[1]:
        raise KernelError("rope_append: x is too small for the heads and tokens given")
    pt_stride = 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", x.dtype, 4)
        _need(v_cache, "v_cache", x.dtype, 4)
        if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError(f"rope_append: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
        if max(k_off, v_off) + n_kv_heads * head_dim > x.shape[1]:
            raise KernelError("rope_append: key/value offsets run past the row")
        pt_stride = page_table.shape[1]
    _check(_fn("rope", "bn_rope_append")(_ptr(x), int(_code(x)), int(n), int(x.shape[1]), int(n_rot_heads),
                                         int(head_dim), int(rotary_dims), c_float(theta_scale), _ptr(tok_pos),
                                         int(k_off), int(v_off), int(n_kv_heads), _ptr(tok_seq), _ptr(slots),
                                         _ptr(page_table), int(pt_stride), _ptr(k_cache), _ptr(v_cache),
                                         _stream()), "rope_append")


def unit_norm_append(x: torch.Tensor, n_q_heads: int, head_dim: int, eps: float, tok_pos: torch.Tensor, *,
                     k_off: int = 0, v_off: int = 0, n_kv_heads: int = 0, tok_seq: Optional[torch.Tensor] = None,
                     slots: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                     k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None) -> None:
    """Divide each of the first ``n_q_heads`` heads of every row of x by its root mean square, in
    place; when a cache is given, do the same to the key heads at ``k_off`` and write them, and the
    value heads at ``v_off`` as they are, into it (a value head has the width of ``v_cache``'s rows)."""
    _need(x, "x", dims=2)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    n = tok_pos.shape[0]
    if x.shape[0] < n or n_q_heads * head_dim > x.shape[1]:
        raise KernelError("unit_norm_append: x is too small for the heads and tokens given")
    pt_stride, v_dim = 0, 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", x.dtype, 4)
        _need(v_cache, "v_cache", x.dtype, 4)
        v_dim = v_cache.shape[3]
        if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or tuple(k_cache.shape[:3]) != tuple(v_cache.shape[:3]):
            raise KernelError(f"unit_norm_append: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} does not fit")
        if k_off + n_kv_heads * head_dim > x.shape[1] or v_off + n_kv_heads * v_dim > x.shape[1]:
            raise KernelError("unit_norm_append: key/value offsets run past the row")
        pt_stride = page_table.shape[1]
    _check(_fn("unit_norm", "bn_unit_norm_append")(_ptr(x), int(_code(x)), int(n), int(x.shape[1]), int(n_q_heads),
                                                   int(head_dim), c_float(eps), int(k_off), int(v_off), int(n_kv_heads),
                                                   int(v_dim), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots), _ptr(page_table),
                                                   int(pt_stride), _ptr(k_cache), _ptr(v_cache), _stream()),
           "unit_norm_append")


def slice_norm_append(x: torch.Tensor, q_len: int, wq: torch.Tensor, k_off: int, wk: torch.Tensor, v_off: int,
                      n_kv_heads: int, head_dim: int, v_dim: int, eps: float, *, v_other: Optional[torch.Tensor] = None,
                      blend: float = 0.0, tok_seq: Optional[torch.Tensor] = None, tok_pos: Optional[torch.Tensor] = None,
                      slots: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                      k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None) -> None:
    """RMS norms with gains over the first ``q_len`` numbers of every row of x (all query heads at once) and over
    the ``n_kv_heads * head_dim`` numbers at ``k_off`` (all key heads), in place; the values at ``v_off`` become
    (1 - blend) v + blend v_other when ``v_other`` (a view with unit inner stride, one row per row of x) is given;
    with a cache, the keys and values are then written into it."""
    _need(x, "x", dims=2)
    _need(wq, "wq", dims=1)
    _need(wk, "wk", wq.dtype, 1)
    k_len, v_len = n_kv_heads * head_dim, n_kv_heads * v_dim
    n = x.shape[0]
    if wq.shape[0] != q_len or wk.shape[0] != k_len or max(q_len, k_off + k_len, v_off + v_len) > x.shape[1]:
        raise KernelError("slice_norm_append: slices or gains do not fit the rows")
    other_stride = 0
    if v_other is not None:
        if (not v_other.is_cuda or v_other.dtype != x.dtype or v_other.dim() != 2 or v_other.stride(1) != 1
                or v_other.shape[0] < n or v_other.shape[1] < v_len):
            raise KernelError("slice_norm_append: v_other must be a CUDA view of x's type with unit inner stride that holds the values")
        other_stride = v_other.stride(0)
    pt_stride = 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", x.dtype, 4)
        _need(v_cache, "v_cache", x.dtype, 4)
        if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != tuple(k_cache.shape[:3]) + (v_dim,):
            raise KernelError(f"slice_norm_append: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} does not fit")
        if tok_pos.shape[0] != n:
            raise KernelError("slice_norm_append: one position per row")
        pt_stride = page_table.shape[1]
    _check(_fn("unit_norm", "bn_slice_norm_append")(
        _ptr(x), int(_code(x)), int(n), int(x.shape[1]), 0, int(q_len), _ptr(wq), int(k_off), int(k_len), _ptr(wk),
        int(_code(wq)), c_float(eps), int(v_off), c_void_p(v_other.data_ptr()) if v_other is not None else _NULL,
        int(other_stride), c_float(blend), int(n_kv_heads), int(head_dim), int(v_dim), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots),
        _ptr(page_table), int(pt_stride), _ptr(k_cache), _ptr(v_cache), _stream()), "slice_norm_append")


def qk_norm_append(src: torch.Tensor, out: torch.Tensor, tok_pos: torch.Tensor, *, q_len: int, k_off: int, k_len: int,
                   bias: Optional[torch.Tensor] = None, q_span: int = 0, wq: Optional[torch.Tensor] = None, k_span: int = 0,
                   wk: Optional[torch.Tensor] = None, eps: float = 1e-6, temp_coef: float = 0.0, temp_every: int = 0,
                   v_off: int = 0, n_kv_heads: int = 0, head_dim: int = 0, n_v_heads: int = 0, v_dim: int = 0,
                   tok_seq: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                   page_table: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
                   v_cache: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Queries, keys and values from the float32 rows ``src`` of their stacked projection into ``out`` (the same
    columns, in the compute type): ``bias`` added; RMS norms with gains over spans of ``q_span`` numbers of the
    first ``q_len`` (the queries) and of ``k_span`` numbers of the ``k_len`` at ``k_off`` (the keys) (a span of
    one head norms heads one by one with one gain for all, a span of the whole slice norms all heads at once,
    0: none); the queries times 1 + ``temp_coef`` * ln(floor((position + 1) / ``temp_every``) + 1) (0: no
    factor); with a cache the keys (``n_kv_heads`` heads of ``head_dim``) and the values at ``v_off``
    (``n_v_heads`` heads of ``v_dim``) are written into it."""
    _need(src, "src", torch.float32, 2)
    _need(out, "out", dims=2)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    n, row = tok_pos.shape[0], src.shape[1]
    if src.shape[0] < n or out.shape[0] < n or out.shape[1] != row or q_len > k_off or k_off + k_len > row:
        raise KernelError("qk_norm_append: rows or slices do not fit")
    if bias is not None:
        _need(bias, "bias", dims=1)
        if bias.shape[0] != row:
            raise KernelError("qk_norm_append: the bias does not fit the row")
    w_code = 0
    for span, w, length, nm in ((q_span, wq, q_len, "wq"), (k_span, wk, k_len, "wk")):
        if span:
            _need(w, nm, dims=1)
            if w.shape[0] != span or length % span:
                raise KernelError(f"qk_norm_append: gain {nm} of {w.shape[0]} numbers does not fit spans of {span} in {length}")
            if w_code and _code(w) != w_code:
                raise KernelError("qk_norm_append: both gains must be of one type")
            w_code = _code(w)
    pt_stride = 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", out.dtype, 4)
        _need(v_cache, "v_cache", out.dtype, 4)
        if (tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], n_v_heads, PAGE, v_dim)
                or k_len != n_kv_heads * head_dim or v_off < k_off + k_len or v_off + n_v_heads * v_dim > row):
            raise KernelError(f"qk_norm_append: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} does not fit")
        pt_stride = page_table.shape[1]
    _check(_fn("unit_norm", "bn_qk_norm_append")(
        _ptr(src), int(src.stride(0)), _ptr(bias), int(_code(bias)) if bias is not None else 0, _ptr(out), int(_code(out)),
        int(out.stride(0)), int(n), int(row), int(q_len), int(q_span), _ptr(wq) if q_span else _NULL, int(k_off), int(k_len),
        int(k_span), _ptr(wk) if k_span else _NULL, int(w_code), c_float(eps), c_float(temp_coef), int(temp_every), int(v_off),
        int(n_kv_heads), int(head_dim), int(n_v_heads), int(v_dim), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots), _ptr(page_table),
        int(pt_stride), _ptr(k_cache), _ptr(v_cache), _stream()), "qk_norm_append")
    return out


def diff_combine(maps: torch.Tensor, out: torch.Tensor, n_heads: int, per_group: int, v_dim: int, lam: float, eps: float,
                 post: float, tail: int = 0) -> torch.Tensor:
    """Two attention maps over the same values combined per token and head: o = a1 - ``lam`` a2, divided by its root
    mean square over the head's ``v_dim`` numbers (``eps`` inside the root), times ``post``.  ``maps`` is float32
    ``[n, 2 * n_heads * v_dim]`` with the maps of the ``per_group`` heads that share a key/value head laid out as
    [group][map][head in group][v_dim]; ``out`` ``[n, n_heads * v_dim + tail]`` holds the heads in their own order and
    behind them a one and ``tail`` - 1 zeros (``tail`` > 0: the product that reads the rows then adds a bias that is
    stored as a column of its matrix)."""
    _need(maps, "maps", torch.float32, 2)
    _need(out, "out", dims=2)
    if (maps.shape[1] != 2 * n_heads * v_dim or out.shape[1] != n_heads * v_dim + tail or out.shape[0] < maps.shape[0]
            or n_heads % per_group or not 0 <= tail <= 32):
        raise KernelError("diff_combine: sizes do not fit")
    _check(_fn("unit_norm", "bn_diff_combine")(_ptr(maps), int(maps.stride(0)), _ptr(out), int(_code(out)), int(out.stride(0)),
                                               int(maps.shape[0]), int(n_heads), int(per_group), int(v_dim), c_float(lam),
                                               c_float(eps), c_float(post), int(tail), _stream()), "diff_combine")
    return out


def gate_rows(x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """x <- x * sigmoid(g), number by number, in place; x and g ``[n, m]`` views of one type with unit inner stride."""
    if (not x.is_cuda or not g.is_cuda or x.dim() != 2 or g.dim() != 2 or x.dtype != g.dtype or x.stride(1) != 1
            or g.stride(1) != 1 or g.shape[0] < x.shape[0] or g.shape[1] != x.shape[1]):
        raise KernelError("gate_rows: x and g must be CUDA matrices of one type and width with unit inner stride")
    _check(_fn("act", "bn_gate_rows")(c_void_p(x.data_ptr()), int(x.stride(0)), c_void_p(g.data_ptr()), int(g.stride(0)),
                                      int(_code(x)), int(x.shape[0]), int(x.shape[1]), _stream()), "gate_rows")
    return x


# ---- attention ----------------------------------------------------------------------------
def sigmoid_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_tokens: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, window: int, tok_seq: torch.Tensor, tok_pos: torch.Tensor,
                      slots: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                      rel: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                      gate: Optional[torch.Tensor] = None, gate_stride: int = 0, gate_per_head: bool = False,
                      max_keys: int = 0) -> torch.Tensor:
    """Causal attention without a softmax of every new token over its sequence's pages: a key at distance
    n < window (window 0: every earlier key) weighs sigmoid(q . k * scale + rel[min(n, last)][head]); with ``mix``
    ``[heads, heads]`` float32 the heads' weights are mixed, weight_h <- sum_g mix[h, g] weight_g; head h sums
    the values of its own key/value head; ``gate`` (a view with unit inner stride, row stride ``gate_stride``)
    holds one number per output number (or per head) whose logistic function multiplies the result.  q may be a
    view into a wider row; a value head has the width of ``v_cache``'s rows.  ``max_keys``: a bound on the keys
    any token sees; with few tokens the keys of a token are dealt out over several blocks."""
    if not q.is_cuda or q.stride(-1) != 1:
        raise KernelError("sigmoid_attention: q must be a CUDA tensor with unit inner stride")
    _need(out, "out", q.dtype, 2)
    for t, nm in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", q.dtype, 4)
    _need(v_cache, "v_cache", q.dtype, 4)
    v_dim = v_cache.shape[3]
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or tuple(k_cache.shape[:3]) != tuple(v_cache.shape[:3]):
        raise KernelError(f"sigmoid_attention: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim} / value width]")
    if n_heads % n_kv_heads:
        raise KernelError(f"sigmoid_attention: {n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
    if out.shape[0] < n_tokens or out.shape[1] != n_heads * v_dim:
        raise KernelError("sigmoid_attention: out does not fit")
    n_rel = 0
    if rel is not None:
        _need(rel, "rel", torch.float32, 2)
        if rel.shape[1] != n_heads or rel.shape[0] < 1:
            raise KernelError(f"sigmoid_attention: bias table {tuple(rel.shape)} is not [distances, {n_heads}]")
        n_rel = rel.shape[0]
    if mix is not None:
        _need(mix, "mix", torch.float32, 2)
        if tuple(mix.shape) != (n_heads, n_heads):
            raise KernelError(f"sigmoid_attention: the mixing matrix {tuple(mix.shape)} is not [{n_heads}, {n_heads}]")
    gate_mode = 0
    if gate is not None:
        gate_mode = 1 if gate_per_head else 2
        need = n_heads if gate_per_head else n_heads * v_dim
        if not gate.is_cuda or gate.dtype != q.dtype or gate.stride(-1) != 1 or gate.shape[-1] < need or gate_stride <= 0:
            raise KernelError("sigmoid_attention: gate must be a CUDA view of q's type with unit inner stride that holds the gates")
    smem_of = getattr(build.library("sigmoid_attention"), "bn_sigmoid_attention_smem")
    smem_of.restype = c_int
    if smem_of(int(_code(q)), int(n_heads), int(n_kv_heads), int(head_dim), int(v_dim), int(mix is not None)) > 200 * 1024:
        raise KernelError(f"sigmoid_attention: {n_heads} heads of {head_dim} / {v_dim} numbers do not fit a block's shared memory")
    splits = 1
    if max_keys > DECODE_CHUNK and n_tokens < 2 * n_sms(q.device):
        splits = min((max_keys + DECODE_CHUNK - 1) // DECODE_CHUNK, max(1, 4 * n_sms(q.device) // n_tokens))
    part = None
    if splits > 1:
        part = torch.empty(n_tokens * splits * n_heads * v_dim, dtype=torch.float32, device=q.device)
        global LAUNCHES
        LAUNCHES += 1  # the kernel that adds the splits up
    _check(_fn("sigmoid_attention", "bn_sigmoid_attention")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(_code(q)), int(n_tokens), int(n_heads), int(n_kv_heads),
        int(head_dim), int(v_dim), c_float(scale), int(window), _ptr(rel), int(n_rel), _ptr(mix),
        c_void_p(gate.data_ptr()) if gate is not None else _NULL, int(gate_stride), int(gate_mode), _ptr(tok_seq), _ptr(tok_pos),
        _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(part), int(splits),
        _stream()), "sigmoid_attention")
    return out


def attention_general(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_tokens: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, scale: float, window: int, tok_seq: torch.Tensor,
                      tok_pos: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, *, keep_first: int = 0,
                      rel: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      gate_stride: int = 0, max_keys: int = 0, chunk: int = 0, v_dim: int = 0,
                      sink: Optional[torch.Tensor] = None, v_share: int = 1) -> torch.Tensor:
    """Causal attention of every new token over its sequence's pages; q may be a view into a wider row.
    ``max_keys`` (optional): a bound on the keys any of the tokens sees; with few tokens and many keys the
    keys of a token are then shared out over several blocks whose results a second kernel merges.

    A value head may have another width than a key head (the width of ``v_cache``'s rows).  With a
    window, keys at positions below ``keep_first`` stay visible.  ``rel`` ``[distances, n_heads]``
    float32 is added to the scaled scores by distance (the last row serves every longer distance).
    ``gate`` (a view with unit inner stride, row stride ``gate_stride``) holds one number per token and
    head whose logistic function multiplies the head's output.  ``chunk`` > 0 (in place of a window):
    positions are cut into chunks of so many and a token sees the earlier keys of its own chunk.
    ``v_cache`` None with ``v_dim``: the values are the first ``v_dim`` numbers of the key rows.
    ``sink`` float32 ``[n_heads]``: a score per head that stands in the softmax's denominator once, with no key
    and no value.  ``v_share`` > 1: so many consecutive key heads read one value head (``v_cache`` has
    ``n_kv_heads / v_share`` heads): several maps of scores over the same values."""
    if not q.is_cuda or q.stride(-1) != 1:
        raise KernelError("attention: q must be a CUDA tensor with unit inner stride")
    if v_share < 1 or n_kv_heads % v_share or (v_share > 1 and v_cache is None):
        raise KernelError(f"attention: {n_kv_heads} key heads cannot share values {v_share} at a time")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.shape[0] != n_heads:
            raise KernelError(f"attention: {sink.shape[0]} sink scores for {n_heads} heads")
    v_row = 0
    if v_cache is None:
        if not 0 < v_dim <= head_dim:
            raise KernelError("attention: values inside the key rows need 0 < v_dim <= head_dim")
        v_cache, v_row, inner = k_cache, head_dim, v_dim
    else:
        inner = v_cache.shape[3]
    _need(out, "out", dims=2)
    out_wide = out.dtype == torch.float32 and q.dtype != torch.float32  # the sums unrounded, whatever the compute type
    if out.dtype != q.dtype and not out_wide:
        raise KernelError(f"attention: out must be of q's type or float32, not {out.dtype}")
    for t, nm in ((tok_seq, "tok_seq"), (tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", q.dtype, 4)
    _need(v_cache, "v_cache", q.dtype, 4)
    v_dim = inner
    if (tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim)
            or tuple(v_cache.shape[:3]) != (k_cache.shape[0], n_kv_heads // v_share, PAGE)):
        raise KernelError(f"attention: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim} / value width]")
    if not 0 < head_dim <= 2048 or v_dim > 1024:
        raise KernelError(f"attention: head_dim={head_dim} (at most 2048) or the value width {v_dim} (at most 1024) is not supported")
    if chunk < 0 or (chunk > 0 and (window > 0 or keep_first > 0)):
        raise KernelError("attention: chunks take the place of a window")
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
    if out.shape[0] < n_tokens or out.shape[1] != n_heads * v_dim:
        raise KernelError("attention: out does not fit")
    n_rel = 0
    if rel is not None:
        _need(rel, "rel", torch.float32, 2)
        if rel.shape[1] != n_heads or rel.shape[0] < 1:
            raise KernelError(f"attention: bias table {tuple(rel.shape)} is not [distances, {n_heads}]")
        n_rel = rel.shape[0]
    if gate is not None:
        if not gate.is_cuda or gate.dtype != q.dtype or gate.stride(-1) != 1 or gate.shape[-1] < n_heads or gate_stride <= 0:
            raise KernelError("attention: gate must be a CUDA view of q's type with unit inner stride and one number per head")
    splits = 1
    # blocks per split: one per token and head, or per token and group of heads where the kernel takes the heads of a
    # key/value head four or two at a time (few tokens, rows of whole 16-byte pieces)
    per_block = 1
    piece = 4 if q.dtype == torch.float32 else 8
    if n_tokens <= 256 and head_dim % piece == 0 and v_dim % piece == 0 and (v_row or v_dim) % piece == 0 and v_dim // piece <= 128:
        gq = n_heads // n_kv_heads
        per_block = 4 if gq % 4 == 0 else (2 if gq % 2 == 0 else 1)
    blocks = n_tokens * n_heads // per_block
    if max_keys > 2 * DECODE_CHUNK and blocks < 2 * n_sms(q.device):
        splits = min(16, (max_keys + DECODE_CHUNK - 1) // DECODE_CHUNK, max(1, 4 * n_sms(q.device) // blocks))
    if (keep_first or rel is not None or gate is not None or v_dim != head_dim or splits > 1 or chunk or v_row
            or sink is not None or v_share > 1 or out_wide):
        part = None
        if splits > 1:
            part = torch.empty(n_tokens * n_heads * splits * (v_dim + 2), dtype=torch.float32, device=q.device)
            global LAUNCHES
            LAUNCHES += 1  # the kernel that merges the splits
        _check(_fn("attention", "bn_attention_general_ex")(
            _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(_code(q)), int(n_tokens), int(n_heads),
            int(n_kv_heads), int(head_dim), int(v_dim), c_float(scale), int(window), int(keep_first), int(chunk), int(v_row),
            _ptr(rel), int(n_rel), _ptr(gate), int(gate_stride), _ptr(tok_seq), _ptr(tok_pos), _ptr(slots), _ptr(page_table),
            int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(part), int(splits), _ptr(sink), int(v_share),
            int(out_wide), _stream()), "attention_general")
        return out
    _check(_fn("attention", "bn_attention_general")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(_code(q)), int(n_tokens), int(n_heads),
        int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tok_seq), _ptr(tok_pos),
        _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _stream()),
        "attention_general")
    return out


def attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                      seq_start: torch.Tensor, seq_pos0: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, *, keep_first: int = 0,
                      rel: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_stride: int = 0,
                      precise: bool = False, chunk: int = 0, v_dim: int = 0, sink: Optional[torch.Tensor] = None,
                      v_share: int = 1) -> torch.Tensor:
    """bfloat16 causal attention of runs of new tokens on the tensor cores; block i handles up to 64
    new tokens of sequence tile_seq[i] from its row tile_row0[i] on.  ``keep_first``, ``rel`` and ``gate`` as
    for ``attention_general``; a value head may have a width of its own (``v_cache``'s rows; with ``precise``); ``precise``: the softmax weights enter the second product with 16 bits of
    mantissa (as two bfloat16 terms) instead of 8.  ``chunk``, ``v_cache`` None with ``v_dim``, ``sink``, ``v_share``
    and a float32 ``out`` as for ``attention_general``."""
    if not q.is_cuda or q.stride(-1) != 1 or q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: q must be a bfloat16 CUDA tensor with unit inner stride")
    v_row = 0
    if v_cache is None:
        if not 0 < v_dim <= head_dim:
            raise KernelError("attention_prefill: values inside the key rows need 0 < v_dim <= head_dim")
        v_cache, v_row, inner = k_cache, head_dim, v_dim
    else:
        inner = v_cache.shape[3]
    _need(out, "out", dims=2)
    out_wide = out.dtype == torch.float32
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("attention_prefill: out must be bfloat16 or float32")
    if v_share < 1 or n_kv_heads % v_share or (v_share > 1 and v_cache is None):
        raise KernelError(f"attention_prefill: {n_kv_heads} key heads cannot share values {v_share} at a time")
    if sink is not None:
        _need(sink, "sink", torch.float32, 1)
        if sink.shape[0] != n_heads:
            raise KernelError(f"attention_prefill: {sink.shape[0]} sink scores for {n_heads} heads")
    for t, nm in ((tile_seq, "tile_seq"), (tile_row0, "tile_row0"), (seq_start, "seq_start"), (seq_pos0, "seq_pos0"),
                  (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    v_dim = inner
    if (tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim)
            or tuple(v_cache.shape[:3]) != (k_cache.shape[0], n_kv_heads // v_share, PAGE)):
        raise KernelError(f"attention_prefill: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim} / value width]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads or v_dim % 16 or v_dim > 256:
        raise KernelError(f"attention_prefill: head_dim={head_dim}, value width {v_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if v_dim != head_dim and not precise:
        raise KernelError("attention_prefill: a value width of its own is built for precise weights only")
    if out.shape[1] != n_heads * v_dim or q_stride % 8:
        raise KernelError("attention_prefill: out or q_stride does not fit")
    n_rel = 0
    if rel is not None:
        _need(rel, "rel", torch.float32, 2)
        if rel.shape[1] != n_heads or rel.shape[0] < 1:
            raise KernelError(f"attention_prefill: bias table {tuple(rel.shape)} is not [distances, {n_heads}]")
        n_rel = rel.shape[0]
    if gate is not None and (not gate.is_cuda or gate.dtype != torch.bfloat16 or gate.stride(-1) != 1
                             or gate.shape[-1] < n_heads or gate_stride <= 0):
        raise KernelError("attention_prefill: gate must be a bfloat16 CUDA view with unit inner stride and one number per head")
    if keep_first or rel is not None or gate is not None or precise or chunk or v_row or sink is not None or v_share > 1 or out_wide:
        _check(_fn("attention_prefill", "bn_attention_prefill_ex")(
            _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]), int(n_heads),
            int(n_kv_heads), int(head_dim), int(v_dim), c_float(scale), int(window), int(keep_first), int(chunk), int(v_row),
            _ptr(rel), int(n_rel), _ptr(gate),
            int(gate_stride), int(bool(precise)), _ptr(tile_seq), _ptr(tile_row0), _ptr(seq_start), _ptr(seq_pos0), _ptr(slots),
            _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(sink), int(v_share), int(out_wide),
            _stream()), "attention_prefill")
        return out
    _check(_fn("attention_prefill", "bn_attention_prefill")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]), int(n_heads),
        int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tile_seq), _ptr(tile_row0),
        _ptr(seq_start), _ptr(seq_pos0), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), _stream()), "attention_prefill")
    return out


USE_TCGEN05_ATTENTION = True  # prefill attention with head sizes up to 128 runs on tcgen05 (attention_prefill_tc.cu)


def attention_prefill_tc(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         scale: float, window: int, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                         seq_start: torch.Tensor, seq_pos0: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                         k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
    """bfloat16 causal attention of runs of new tokens on tcgen05 tensor cores with TMA-fed operands;
    block i handles up to 128 new tokens of sequence tile_seq[i] from its row tile_row0[i] on.
    Head sizes up to 128."""
    if not q.is_cuda or q.dim() != 2 or q.stride(-1) != 1 or q.stride(0) != q_stride or q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: q must be a bfloat16 CUDA matrix with unit inner stride")
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tile_seq, "tile_seq"), (tile_row0, "tile_row0"), (seq_start, "seq_start"), (seq_pos0, "seq_pos0"),
                  (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_prefill_tc: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 128 or n_heads % n_kv_heads:
        raise KernelError(f"attention_prefill_tc: head_dim={head_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if out.shape[1] != n_heads * head_dim or q_stride % 8 or n_heads * head_dim > q_stride or out.shape[0] < q.shape[0]:
        raise KernelError("attention_prefill_tc: out or q_stride does not fit")
    _check(_fn("attention_prefill_tc", "bn_attention_prefill_tc")(
        _ptr(q), int(q_stride), int(q.shape[0]), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]),
        int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), _ptr(tile_seq), _ptr(tile_row0),
        _ptr(seq_start), _ptr(seq_pos0), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(q.device)), _stream()), "attention_prefill_tc")
    return out


DECODE_CHUNK = 128  # positions per block of the decode attention; must equal DEC_CHUNK in attention_decode.cu


def attention_decode(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_seqs: int, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: int, tok_pos: torch.Tensor, slots: torch.Tensor,
                     page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, max_len: int) -> torch.Tensor:
    """bfloat16 attention of one new token per sequence (row b of q is sequence b), split over the
    keys.  ``max_len`` bounds every sequence's length after this step; it sizes the scratch."""
    if not q.is_cuda or q.stride(-1) != 1 or q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: q must be a bfloat16 CUDA tensor with unit inner stride")
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads:
        raise KernelError(f"attention_decode: head_dim={head_dim}, heads {n_heads}/{n_kv_heads} not supported")
    if out.shape[0] < n_seqs or out.shape[1] != n_heads * head_dim or tok_pos.shape[0] < n_seqs:
        raise KernelError("attention_decode: out or tok_pos does not fit")
    n_splits = max(1, (max_len + DECODE_CHUNK - 1) // DECODE_CHUNK)
    part_o = torch.empty((n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    _check(_fn("attention_decode", "bn_attention_decode")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(n_seqs), int(n_heads), int(n_kv_heads),
        int(head_dim), c_float(scale), int(window), _ptr(tok_pos), _ptr(slots), _ptr(page_table),
        int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache), _ptr(part_o), _ptr(part_ml), int(n_splits),
        _stream()), "attention_decode")
    return out


_FORCE_SPLITS = 0  # tests and experiments: a fixed number of blocks per sequence in attention_decode_fused
# (more than eight take the path that merges through global memory and a ticket)


def decode_splits(pages: int, blocks_per_split: int) -> int:
    """How many blocks share one sequence's pages in ``attention_decode_fused``.

    A block walks its pages one after another, about 0.75 us each; blocks that share a sequence
    merge their results inside a thread-block cluster, which costs about as much as five pages.
    So a split pays only when it shortens the walk by more than that: few sequences, or long
    ones.  Up to eight blocks per sequence are one cluster; more (up to 32) merge through global
    memory block by block, which costs as much as 0.7 pages more for every block and pays from
    some 16,000 positions on for one or two sequences.  No more than 256 blocks in all: clusters
    are placed within one GPC, and beyond that number a second wave of blocks starts.
    ``pages`` is the bound the step was recorded for; sequences are taken to fill three quarters
    of it, and the kernel shares a sequence's pages evenly among its blocks whatever the bound.
    Measured at 8 key/value heads of 128 (us, 520 positions, 1 against the chosen number of
    splits): 1 sequence 10.3 / 5.5, 4: 10.6 / 7.6, 8: 11.4 / 10.2, 12: 12.2 / 11.2 (three
    splits 18.6), 16: 12.6 / 12.2 (four 20.1), 24: 13.6 (two 15.7); at 2,000 positions 8
    sequences 31.7 / 15.6, 16: 34.9 / 26.0; one sequence of 64,000 positions: 8 splits 111, 32
    splits 59."""
    cap = max(1, min(pages, 256 // max(1, blocks_per_split)))
    filled = 0.75 * pages
    best, best_cost = 1, filled
    for s in (2, 3, 4, 5, 6, 7, 8, 12, 16, 24, 32):
        if s > cap:
            break
        cost = float(-(-int(filled) // s)) + (5.0 if s <= 8 else 5.0 + 0.7 * s)
        if cost < best_cost:
            best, best_cost = s, cost
    return best


DECODE_ITEM_BLOCKS = 450  # a work list may come to so many blocks (three per SM run at once)
_FORCE_ITEM_GROUP = 0  # tests: a work list in groups of this many whatever the batch


def decode_items(seq_pages, blocks_per_seq: int, group: Optional[int] = None, capacity: Optional[int] = None):
    """For a batch of unequal lengths: which block of ``attention_decode_fused`` works on what.

    ``seq_pages[b]`` is the number of cache pages sequence b's new token sees.  Returns
    ``(group, items)`` or None when the plain grid (every sequence alike) serves as well: few
    blocks (the plain grid then splits every sequence), lengths that differ little, or so many
    sequences that more blocks would only queue.  ``items`` lists, in the order in which blocks
    start, ``sequence | split << 16 | splits << 24`` or -1 (nothing); its length is a multiple of
    ``group``, and each run of ``group`` entries (one thread-block cluster) is either the
    ``group`` splits of one long sequence or sequences that are not split.  A sequence is long
    when it has more than 1/group of the longest one's pages; long sequences come first, so that
    the launch does not end on them.  ``group`` is the largest of 2, 3, 4 that keeps the blocks
    within ``DECODE_ITEM_BLOCKS``.  Measured (us per launch, plain grid against work list): 8
    sequences of 513 to 2,560 positions at 40 heads of 128: 49 / 34; 32 sequences of 129 to 2,176
    at 8 key/value heads of 128: 36 / 31; 64 such sequences at 8 heads of 64: 37 / 40 (not used).
    With ``group`` given (a recorded step keeps the shape of its grid) only the list is made,
    padded to ``capacity`` entries."""
    n = len(seq_pages)
    if n == 0 or n > 65535:
        return None
    total, longest = sum(seq_pages), max(seq_pages)

    def long_ones(s: int):
        limit = -(-longest // s)
        return [b for b in range(n) if seq_pages[b] > limit]

    def fits(s: int) -> bool:
        k = len(long_ones(s))
        return (s * k + n - k) * blocks_per_seq <= DECODE_ITEM_BLOCKS

    uneven = longest >= 12 and longest * n >= 1.5 * total
    if group is None and _FORCE_ITEM_GROUP:
        group = _FORCE_ITEM_GROUP
        chosen = long_ones(group) if group > 1 else []
    elif group is None:
        sizes = [s for s in (2, 3, 4) if fits(s)]
        if n * blocks_per_seq <= 128 or not uneven or not sizes:
            return None
        group = max(sizes)
        chosen = long_ones(group)
    else:
        # the grid's shape is given; if the batch has meanwhile become even, or splitting its long
        # sequences would now take too many blocks, nothing is split and the list only orders
        chosen = long_ones(group) if group > 1 and (_FORCE_ITEM_GROUP or (uneven and fits(group))) else []
    is_long = set(chosen)
    items = []
    for b in sorted(chosen, key=lambda b: -seq_pages[b]):
        items.extend(b | (z << 16) | (group << 24) for z in range(group))
    items.extend(b | (1 << 24) for b in sorted((b for b in range(n) if b not in is_long), key=lambda b: -seq_pages[b]))
    size = capacity if capacity is not None else -(-len(items) // group) * group
    if len(items) > size or size % group:
        raise KernelError(f"decode_items: {len(items)} entries do not fit a capacity of {size} in groups of {group}")
    items.extend([-1] * (size - len(items)))
    return group, items


def attention_decode_fused(qkv: torch.Tensor, k_off: int, v_off: int, out: torch.Tensor, n_seqs: int, n_heads: int,
                           n_kv_heads: int, head_dim: int, scale: float, window: int, rotary_dims: int,
                           theta_scale: float, tok_pos: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, max_len: int,
                           items: Optional[torch.Tensor] = None, item_group: int = 0) -> torch.Tensor:
    """The decode step's attention in one launch on tensor cores (attention_decode_tc.cu): rotary
    encoding of the raw queries and of the new key (``rotary_dims`` = 0: none), the new key and value
    written into the cache at ``tok_pos``, attention split over the keys, and the combination of
    the splits.  ``qkv`` holds one raw
    q|k|v row per sequence with the key heads at element ``k_off`` and the value heads at ``v_off``.
    ``items`` / ``item_group``: the work list of ``decode_items`` on the device, for batches of
    unequal lengths."""
    _need(qkv, "qkv", torch.bfloat16, 2)
    _need(out, "out", torch.bfloat16, 2)
    for t, nm in ((tok_pos, "tok_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", torch.bfloat16, 4)
    _need(v_cache, "v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_decode_fused: cache {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads or rotary_dims % 2 or rotary_dims > head_dim:
        raise KernelError(f"attention_decode_fused: head_dim={head_dim}, heads {n_heads}/{n_kv_heads}, "
                          f"rotary_dims={rotary_dims} not supported")
    if max(k_off, v_off) + n_kv_heads * head_dim > qkv.shape[1] or n_heads * head_dim > qkv.shape[1]:
        raise KernelError("attention_decode_fused: offsets run past the row")
    if out.shape[0] < n_seqs or out.shape[1] != n_heads * head_dim or tok_pos.shape[0] < n_seqs or qkv.shape[0] < n_seqs:
        raise KernelError("attention_decode_fused: out, qkv or tok_pos does not fit")
    if items is not None:
        _need(items, "items", torch.int32, 1)
        if not 1 <= item_group <= 8 or items.shape[0] % item_group or items.shape[0] == 0:
            raise KernelError(f"attention_decode_fused: {items.shape[0]} items in groups of {item_group}")
        part_o = torch.empty((n_seqs * n_heads * item_group * head_dim,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n_seqs * n_heads * item_group * 2,), dtype=torch.float32, device=qkv.device)
        _scr, counters = _split_scratch(qkv.device)
        _check(_fn("attention_decode_tc", "bn_attention_decode_tc_items")(
            _ptr(qkv), int(qkv.shape[1]), int(k_off), int(v_off), _ptr(out), int(out.shape[1]), int(n_seqs),
            int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), int(rotary_dims),
            c_float(theta_scale), _ptr(tok_pos), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
            _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(qkv.device)), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            int(counters.numel()), _ptr(items), int(items.shape[0]), int(item_group), _stream()), "attention_decode_fused")
        return out
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    blocks_per_split = n_seqs * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16)
    want_splits = decode_splits(pages, blocks_per_split)
    if _FORCE_SPLITS:
        want_splits = max(1, min(pages, _FORCE_SPLITS))
    pages_per_block = (pages + want_splits - 1) // want_splits
    n_splits = (pages + pages_per_block - 1) // pages_per_block
    part_o = torch.empty((n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
    part_ml = torch.empty((n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
    _scr, counters = _split_scratch(qkv.device)
    _check(_fn("attention_decode_tc", "bn_attention_decode_tc")(
        _ptr(qkv), int(qkv.shape[1]), int(k_off), int(v_off), _ptr(out), int(out.shape[1]), int(n_seqs),
        int(n_heads), int(n_kv_heads), int(head_dim), c_float(scale), int(window), int(rotary_dims),
        c_float(theta_scale), _ptr(tok_pos), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache),
        _ptr(v_cache), int(k_cache.shape[0]), _ptr(tc_status(qkv.device)), _ptr(part_o), _ptr(part_ml), int(n_splits),
        int(pages_per_block), _ptr(counters),
        int(counters.numel()), _stream()), "attention_decode_fused")
    return out


# ---- matrix products ----------------------------------------------------------------------
SKINNY_MAX_ROWS = 16  # float32: warp-per-column kernel up to this many rows
MMA_MAX_ROWS = 64  # bfloat16: the streaming kernels (linear_tc.cu, linear_mma.cu) up to this many rows; the library
# product is faster beyond (5.5 against 5.8 ms for a decode step of 96 sequences at 32 layers of width 4096)
TC_MAX_ROWS = MMA_MAX_ROWS
USE_TCGEN05 = True  # small-batch bfloat16 products run on tcgen05 (linear_tc.cu); False: mma.sync (linear_mma.cu)
_n_sms = {}


def n_sms(device) -> int:
    """Streaming multiprocessors of ``device`` (asked once)."""
    key = torch.device(device).index or 0
    if key not in _n_sms:
        _n_sms[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _n_sms[key]



_SCRATCH_FLOATS = 8 * 1024 * 1024  # 32 MB of split-K partial tiles, shared by all products of a device
_N_COUNTERS = 8192
_scratch = {}


def _split_scratch(device):
    """Scratch and ticket counters of the split-K reduction, one set per device, made on first use."""
    key = torch.device(device).index or 0
    got = _scratch.get(key)
    if got is None:
        got = _scratch[key] = (torch.empty(_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                               torch.zeros(_N_COUNTERS, dtype=torch.int32, device=device))
    return got


def _mma_splits(M: int, N: int, K: int, sms: int) -> int:
    """How many ways the inner dimension is split so that about four blocks per SM stream weights."""
    blocks = (N + 63) // 64
    want = 4 * sms
    if blocks >= want or blocks > _N_COUNTERS:
        return 1
    mp = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    fit = _SCRATCH_FLOATS // (blocks * 64 * mp)
    splits = max(1, min((want + blocks - 1) // blocks, K // 256, fit))
    chunks = (K + 127) // 128  # the kernel works in chunks of 128 along K and leaves no split empty
    per = (chunks + splits - 1) // splits
    return (chunks + per - 1) // per


_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """One int per device that a TMA-fed kernel (the tcgen05 product, the tensor-core decode
    attention) sets when a wait inside it gave up (0 = fine)."""
    key = torch.device(device).index or 0
    got = _tc_status.get(key)
    if got is None:
        got = _tc_status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return got


_tc_status_ptr = {}


def _tc_status_arg(device: torch.device) -> c_void_p:
    """The status word of ``device`` as a launch argument (made once per device)."""
    got = _tc_status_ptr.get(device.index)
    if got is None:
        got = _tc_status_ptr[device.index] = _ptr(tc_status(device))
    return got


def check_tc_status(device) -> None:
    """Raise if a TMA-fed kernel on ``device`` reported a wait that gave up (synchronises)."""
    code = int(tc_status(device).item())
    if code:
        tc_status(device).zero_()
        _split_scratch(device)[1].zero_()  # tickets of the launch that gave up may be left over
        what = {1: "linear_tc: a stage never filled (TMA load)", 2: "linear_tc: a stage was never released (MMA commit)",
                3: "linear_tc: the accumulator never completed",
                4: "attention_decode_tc: a cache page never arrived (TMA load)",
                5: "attention_prefill_tc: a wait inside the kernel gave up",
                6: "linear_tc: a slice of partial sums from another block of the cluster never arrived",
                7: "gemm_tc: a wait inside the kernel gave up"}.get(code, f"code {code}")
        raise KernelError(f"{what}; the result of that launch is not valid")


class RowScaled:
    """Rows of activations that still lack their RMS scale: the value of row m is
    ``x[m] / sqrt(sum_p ss[p, m] / width + eps)``.  A product whose epilogue added to the residual
    (``linear(..., sink=...)``) leaves the next norm's output in this form: x = residual * gain in
    bfloat16 and, per block of the product, the sum of squares of its slice of every residual row.
    The product that consumes the rows scales its result rows instead (W (s x) = s (W x))."""

    def __init__(self, x: torch.Tensor, ss: torch.Tensor, width: int, eps: float):
        self.x, self.ss, self.width, self.eps = x, ss, int(width), float(eps)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device

    def dense(self) -> torch.Tensor:
        """The rows with their scale applied (for a consumer that cannot apply it itself)."""
        scale = torch.rsqrt(self.ss.sum(0)[: self.x.shape[0]] / self.width + self.eps)
        return (self.x.float() * scale[:, None]).to(self.x.dtype)


class NormSink:
    """Where a product's result goes when the RMSNorm after it is fused into its epilogue: the
    float32 residual it is added to, and that norm's weight and eps."""

    def __init__(self, residual: torch.Tensor, weight: torch.Tensor, eps: float):
        self.residual, self.weight, self.eps = residual, weight, float(eps)


USE_FUSED_NORM = True  # products of few rows add to the residual and prepare the next norm in their epilogue
# (tests and comparisons set it to False)


ACT_SILU, ACT_GELU_TANH = 0, 1  # the gate's activation in a gated product (BN_ACT_* in common.cuh)
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}


def linear_tc(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
              cluster: int = 0, sink: Optional[NormSink] = None, _checked: bool = False, act: int = 0):
    """x[M, K] . w[N, K]^T for M <= 64 in bfloat16 on tcgen05 tensor cores with TMA-fed operands.
    ``cluster`` blocks (1 to 8) share the inner dimension of each 128-row tile of w and add their
    parts up through distributed shared memory (0: chosen from the number of tiles).  ``x`` may be
    ``RowScaled``.  With ``sink`` the product is added to ``sink.residual`` in place and the result
    is the ``RowScaled`` output of the norm that follows.  (``_checked``: ``linear`` has looked at w
    and at the sizes already.)"""
    scaled = x if isinstance(x, RowScaled) else None
    if scaled is not None:
        x = scaled.x
    _need(x, "x", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if not _checked:
        _need(w, "w", torch.bfloat16, 2)
        if w.shape[1] != K or M > TC_MAX_ROWS or K % 8 or (swiglu and N % 16) or not 0 <= cluster <= 8:
            raise KernelError(f"linear_tc: x {tuple(x.shape)}, w {tuple(w.shape)}, cluster {cluster} not supported")
    fn = _fn("linear_tc", "bn_linear_tc_ex")
    dev = x.device
    if scaled is not None:
        ss_rows = scaled.ss
        _need(ss_rows, "ss", torch.float32, 2)
        if ss_rows.shape[1] < M or scaled.width != K:
            raise KernelError(f"linear_tc: row sums {tuple(ss_rows.shape)} of width {scaled.width} do not fit x {tuple(x.shape)}")
        row = (c_void_p(ss_rows.data_ptr()), ss_rows.shape[0], ss_rows.shape[1], c_float(1.0 / scaled.width), c_float(scaled.eps))
    else:
        row = (_NULL, 0, 0, _F0, _F0)
    if sink is not None:
        res = sink.residual
        _need(res, "residual", torch.float32, 2)
        _need(sink.weight, "norm weight", dims=1)
        if swiglu or tuple(res.shape) != (M, N) or sink.weight.shape[0] != N or sink.weight.dtype not in _DT:
            raise KernelError(f"linear_tc: residual {tuple(res.shape)} / norm weight {tuple(sink.weight.shape)} do not fit "
                              f"a product [{M}, {N}]")
        if cluster == 0:
            cluster = _auto_cluster(N, K)
        tiles = (N + 127) // 128
        xg = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        ss = torch.empty((tiles * cluster, M), dtype=torch.float32, device=dev)
        _check(fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(res.data_ptr()), 0, M, N, K, N, 3,
                  cluster, *row, c_void_p(sink.weight.data_ptr()), _DT[sink.weight.dtype], c_void_p(xg.data_ptr()),
                  c_void_p(ss.data_ptr()), M, _tc_status_arg(dev), _stream()), "linear_tc")
        return RowScaled(xg, ss, N, sink.eps)
    out_dtype = out_dtype or x.dtype
    cols = N // 2 if swiglu else N
    out = torch.empty((M, cols), dtype=out_dtype, device=dev)
    _check(fn(c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), _DT[out_dtype], M, N, K, cols,
              (2 | act << 8) if swiglu else 0, cluster, *row, _NULL, 0, _NULL, _NULL, 0, _tc_status_arg(dev), _stream()), "linear_tc")
    return out


_auto_clusters = {}  # (N, K) -> how many blocks share a tile's inner dimension (a property of the sizes and the device)


def _auto_cluster(N: int, K: int) -> int:
    got = _auto_clusters.get((N, K))
    if got is None:
        f = getattr(build.library("linear_tc"), "bn_linear_tc_auto_cluster")
        f.restype = c_int
        got = _auto_clusters[(N, K)] = int(f(int(N), int(K)))
    return got


# Many-row bfloat16 products on this library's tcgen05 kernel (gemm_tc.cu) instead of the library product
# followed by separate kernels.  "fused": where the kernel's epilogue replaces a pass over the activations
# and that saves more than its main loop loses against the library's (measured on a B200 at widths 4096
# and 14336: the SwiGLU epilogue from 1,024 rows on, 0.88 to 0.98 of the library product + activation
# kernel; the residual + norm epilogue from 2,048 rows on for inner sizes up to 8192, 0.85 to 0.95 of the
# library product + norm kernel; plain products are 1.09 to 1.16 of the library's and stay there).
# True: every product that fits.  False: none.
USE_OWN_GEMM = "fused"
GEMM_MIN_ROWS = 65            # True: from so many rows on
OWN_GEMM_SWIGLU_MIN_ROWS = 1024
OWN_GEMM_SINK_MIN_ROWS = 2048
OWN_GEMM_SINK_MAX_K = 8192


def own_gemm_sink_rows(rows: int) -> bool:
    """Whether a product of so many rows may take the residual + norm epilogue of ``gemm_tc``."""
    if USE_OWN_GEMM is True:
        return rows >= GEMM_MIN_ROWS
    return USE_OWN_GEMM == "fused" and rows >= OWN_GEMM_SINK_MIN_ROWS


def gemm_tc(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
            sink: Optional[NormSink] = None, act: int = 0):
    """x[M, K] . w[N, K]^T for many rows in bfloat16 on tcgen05 tensor cores (gemm_tc.cu).  ``x`` may be
    ``RowScaled``; ``swiglu`` and ``sink`` as for ``linear`` (the activation, or the residual add with
    the next norm's gain and sums of squares, happen in the product's epilogue)."""
    scaled = x if isinstance(x, RowScaled) else None
    if scaled is not None:
        x = scaled.x
    _need(x, "x", torch.bfloat16, 2)
    _need(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or K % 8 or N % 8 or (swiglu and N % 16) or (swiglu and sink is not None):
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)} not supported")
    fn = _fn("gemm_tc", "bn_gemm_tc")
    if scaled is not None:
        _need(scaled.ss, "ss", torch.float32, 2)
        if scaled.ss.shape[1] < M or scaled.width != K:
            raise KernelError(f"gemm_tc: row sums {tuple(scaled.ss.shape)} of width {scaled.width} do not fit x {tuple(x.shape)}")
        row = (_ptr(scaled.ss), int(scaled.ss.shape[0]), int(scaled.ss.shape[1]), c_float(1.0 / scaled.width),
               c_float(scaled.eps))
    else:
        row = (c_void_p(None), int(0), int(0), c_float(0.0), c_float(0.0))
    status = _ptr(tc_status(x.device))
    if sink is not None:
        res = sink.residual
        _need(res, "residual", torch.float32, 2)
        _need(sink.weight, "norm weight", dims=1)
        if scaled is not None or tuple(res.shape) != (M, N) or sink.weight.shape[0] != N or sink.weight.dtype not in _DT:
            raise KernelError(f"gemm_tc: residual {tuple(res.shape)} / norm weight {tuple(sink.weight.shape)} do not fit "
                              f"a product [{M}, {N}]")
        xg = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        parts = getattr(build.library("gemm_tc"), "bn_gemm_tc_parts")
        parts.restype = c_int
        ss = torch.empty((parts(int(N)), M), dtype=torch.float32, device=x.device)
        _check(fn(_ptr(x), _ptr(w), int(M), int(N), int(K), c_void_p(None), int(0), int(0), int(3), *row,
                  _ptr(res), _ptr(sink.weight), int(_DT[sink.weight.dtype]), _ptr(xg), _ptr(ss), int(M), status,
                  _stream()), "gemm_tc")
        return RowScaled(xg, ss, N, sink.eps)
    out_dtype = out_dtype or x.dtype
    cols = N // 2 if swiglu else N
    out = torch.empty((M, cols), dtype=out_dtype, device=x.device)
    _check(fn(_ptr(x), _ptr(w), int(M), int(N), int(K), _ptr(out), int(_DT[out_dtype]), int(cols),
              int((2 | act << 8) if swiglu else 0), *row, c_void_p(None), c_void_p(None), int(0), c_void_p(None), c_void_p(None),
              int(0), status, _stream()), "gemm_tc")
    return out


def gemm_pairs(on: Optional[bool] = None) -> bool:
    """Whether ``gemm_tc`` runs pairs of blocks as one (tcgen05 cta_group::2, the default) or every block
    alone; with an argument, sets it.  Returns the setting before the call."""
    f = getattr(build.library("gemm_tc"), "bn_gemm_tc_pairs")
    f.restype = c_int
    return bool(f(int(-1 if on is None else int(bool(on)))))


def _own_gemm_fits(x, w: torch.Tensor, swiglu: bool, out_dtype, kind: str) -> bool:
    """``kind``: "plain", "swiglu", "sink", or "scaled" (rows that lack their scale: the library product
    would need them made dense first)."""
    M, K = x.shape
    N = w.shape[0]
    if not (USE_OWN_GEMM and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and M >= GEMM_MIN_ROWS
            and K % 8 == 0 and N % (16 if swiglu else 8) == 0 and (N // 2 if swiglu else N) % 8 == 0
            and out_dtype in (None, torch.bfloat16, torch.float32)):
        return False
    if USE_OWN_GEMM is True or kind == "scaled":
        return True
    if kind == "swiglu":
        return M >= OWN_GEMM_SWIGLU_MIN_ROWS
    if kind == "sink":
        return M >= OWN_GEMM_SINK_MIN_ROWS and K <= OWN_GEMM_SINK_MAX_K
    return False


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, swiglu: bool = False,
           partial_sums: bool = False, sink: Optional[NormSink] = None, act: int = 0):
    """x[M, K] . w[N, K]^T.  A weight kept in float32 makes the product float32 whatever x is.

    ``x`` may be ``RowScaled`` (the output of a norm that a product's epilogue prepared).  With
    ``sink`` the product is added to ``sink.residual`` and the result is the output of the norm
    that follows it: ``RowScaled`` when the product of few rows does it in its epilogue,
    else a tensor from the norm kernel.

    ``swiglu``: w holds gate and up rows in alternating blocks of 8 and the result is
    act(gate) * up, ``[M, N / 2]`` (``act``: ACT_SILU or ACT_GELU_TANH).  ``partial_sums``: return the float32 partial sums
    ``[parts, M, N]`` of a product that split its inner dimension instead of their sum
    (``add_rmsnorm`` can add them up); by default the product sums them itself.
    """
    _need(w, "w", dims=2)
    if x.shape[1] != w.shape[1] or len(x.shape) != 2:
        raise KernelError(f"linear: x {tuple(x.shape)} and w {tuple(w.shape)} do not share the inner size")
    M, K = x.shape
    N = w.shape[0]
    few = w.dtype == torch.bfloat16 and K % 8 == 0 and (not swiglu or N % 16 == 0)
    small = few and M <= MMA_MAX_ROWS
    streams = few and M <= TC_MAX_ROWS and not partial_sums and USE_TCGEN05
    fast = streams and x.dtype == torch.bfloat16
    if sink is not None:
        if fast and USE_FUSED_NORM and not swiglu and tuple(sink.residual.shape) == (M, N):
            return linear_tc(x, w, sink=sink, _checked=True)
        if (not swiglu and not isinstance(x, RowScaled) and tuple(sink.residual.shape) == (M, N)
                and _own_gemm_fits(x, w, False, None, "sink") and not partial_sums):
            return gemm_tc(x, w, sink=sink)
        delta = linear(x, w, out_dtype=out_dtype, swiglu=swiglu, act=act)
        normed = torch.empty((M, sink.residual.shape[1]), dtype=delta.dtype, device=delta.device)
        return add_rmsnorm(sink.residual, delta, sink.weight, sink.eps, normed)
    if isinstance(x, RowScaled):
        if fast:
            return linear_tc(x, w, out_dtype=out_dtype or x.dtype, swiglu=swiglu, _checked=True, act=act)
        if _own_gemm_fits(x.x, w, swiglu, out_dtype, "scaled") and not partial_sums:
            return gemm_tc(x, w, out_dtype=out_dtype or x.dtype, swiglu=swiglu, act=act)
        x = x.dense()
    _need(x, "x", dims=2)
    out_dtype = out_dtype or x.dtype
    if x.dtype != w.dtype:
        x = x.to(w.dtype)
    if streams:
        return linear_tc(x, w, out_dtype=out_dtype, swiglu=swiglu, _checked=True, act=act)
    if _own_gemm_fits(x, w, swiglu, out_dtype, "swiglu" if swiglu else "plain") and not partial_sums:
        return gemm_tc(x, w, out_dtype=out_dtype, swiglu=swiglu, act=act)
    if small:
        fn = _fn("linear_mma", "bn_linear_mma")
        splits = _mma_splits(M, N, K, n_sms(x.device))
        scratch, counters = _split_scratch(x.device)
        tail = (_ptr(scratch), ctypes.c_longlong(scratch.numel()), _ptr(counters), int(counters.numel()), _stream())
        if swiglu:
            out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
            _check(fn(_ptr(x), _ptr(w), _ptr(out), int(_DT[out_dtype]), int(M), int(N), int(K), int(N // 2),
                      int(2 | act << 8), int(splits), *tail), "linear_mma")
            return out
        if partial_sums and splits > 1:
            out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            _check(fn(_ptr(x), _ptr(w), _ptr(out), int(0), int(M), int(N), int(K), int(N), int(1),
                      int(splits), *tail), "linear_mma")
            return out
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _check(fn(_ptr(x), _ptr(w), _ptr(out), int(_DT[out_dtype]), int(M), int(N), int(K), int(N), int(0),
                  int(splits), *tail), "linear_mma")
        return out
    if M <= SKINNY_MAX_ROWS and K % 8 == 0:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        # a matrix with few rows shares its inner dimension out over several blocks (a property of the matrix alone)
        n_splits = getattr(build.library("linear"), "bn_linear_skinny_splits")
        n_splits.restype = c_int
        splits = n_splits(int(N), int(K))
        partial = torch.empty((splits, M, N), dtype=torch.float32, device=x.device) if splits > 1 else None
        _check(_fn("linear", "bn_linear_skinny")(_ptr(x), _ptr(w), int(_code(w)), _ptr(out), int(_DT[out_dtype]),
                                                 int(M), int(N), int(K), int(N),
                                                 _ptr(partial) if partial is not None else c_void_p(None), _stream()),
               "linear_skinny")
        if splits > 1:
            global LAUNCHES
            LAUNCHES += 1  # the kernel that adds the splits
    else:
        # Many rows: the library product, float32 accumulation, no reduced-precision float32 mode.
        if w.dtype == torch.float32:
            if torch.backends.cuda.matmul.allow_tf32:
                raise KernelError("float32 products need torch.backends.cuda.matmul.allow_tf32 = False")
            product = lambda: torch.matmul(x, w.t())
        elif out_dtype == torch.float32:
            product = lambda: torch.mm(x, w.t(), out_dtype=torch.float32)
        else:
            product = lambda: torch.matmul(x, w.t())
        out = product() if PROFILE is None else _timed("library.matmul", product)
        out = out if out.dtype == out_dtype else out.to(out_dtype)
    if swiglu:
        res = torch.empty((M, N // 2), dtype=out.dtype, device=x.device)
        return glu_mul(out, res, act)
    return out


# ---- mLSTM ----------------------------------------------------------------------------------
def mlstm_gates(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, n_heads: int, cap: float) -> torch.Tensor:
    """float32 ``[T, 2 * heads]``: per head the soft-capped log input gate, then the log forget gate
    (the logarithm of the logistic function of the soft-capped pre-activation).  ``w`` ``[2 * heads, width]``
    holds the input gate's rows first, ``bias`` ``[2 * heads]`` likewise."""
    _need(h, "h", dims=2)
    _need(w, "w", dims=2)
    _need(bias, "bias", w.dtype, 1)
    if w.shape != (2 * n_heads, h.shape[1]) or bias.shape[0] != 2 * n_heads:
        raise KernelError(f"mlstm_gates: w {tuple(w.shape)} / bias {tuple(bias.shape)} do not fit {n_heads} heads of width {h.shape[1]}")
    gates = torch.empty((h.shape[0], 2 * n_heads), dtype=torch.float32, device=h.device)
    _check(_fn("mlstm", "bn_mlstm_gates")(_ptr(h), int(_code(h)), int(h.shape[0]), int(h.shape[1]), _ptr(w), _ptr(bias),
                                          int(_code(w)), int(n_heads), c_float(cap), _ptr(gates), _stream()), "mlstm_gates")
    return gates


def mlstm_state_floats(dim: int, vdim: int) -> int:
    """Floats of one head's state: the matrix ``[dim, vdim]``, the normaliser ``[dim]`` and the stabiliser."""
    return dim * vdim + dim + 1


def mlstm_recurrence(qkv: torch.Tensor, k_off: int, v_off: int, gates: torch.Tensor, state: torch.Tensor,
                     seq_start: torch.Tensor, slots: torch.Tensor, n_seqs: int, n_heads: int, dim: int, vdim: int,
                     q_scale: float, chunks: bool = False) -> torch.Tensor:
    """The matrix-memory recurrence over the new tokens of every sequence, from and into ``state``
    ``[slots, heads, mlstm_state_floats]`` (float32); returns the heads' raw outputs, float32
    ``[T, heads * vdim]``.  Rows of ``qkv`` hold the query heads first, key heads at ``k_off``, value heads
    at ``v_off``.  ``chunks``: for runs of many tokens, the same sums taken 32 tokens at a time as small matrix
    products (head sizes in multiples of 4; agrees with the token-by-token form to rounding)."""
    _need(qkv, "qkv", dims=2)
    _need(gates, "gates", torch.float32, 2)
    _need(state, "state", torch.float32, 3)
    _need(seq_start, "seq_start", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    T = qkv.shape[0]
    if (state.shape[1] != n_heads or state.shape[2] != mlstm_state_floats(dim, vdim) or gates.shape != (T, 2 * n_heads)
            or max(n_heads * dim, k_off + n_heads * dim, v_off + n_heads * vdim) > qkv.shape[1]
            or seq_start.shape[0] < n_seqs + 1 or slots.shape[0] < n_seqs):
        raise KernelError("mlstm_recurrence: sizes do not fit")
    out = torch.empty((T, n_heads * vdim), dtype=torch.float32, device=qkv.device)
    entry = "bn_mlstm_chunks" if chunks and dim % 4 == 0 and (2 * 32 * (dim + 4) + 33 * dim + 2200) * 4 <= 200 * 1024 else "bn_mlstm_recurrence"
    _check(_fn("mlstm", entry)(_ptr(qkv), int(_code(qkv)), int(qkv.shape[1]), int(k_off), int(v_off),
                                               _ptr(gates), _ptr(state), _ptr(seq_start), _ptr(slots), int(n_seqs),
                                               int(n_heads), int(dim), int(vdim), c_float(q_scale), _ptr(out), _stream()),
           "mlstm_recurrence")
    return out


def mlstm_output(o: torch.Tensor, gain: torch.Tensor, g: torch.Tensor, g_stride: int, n_heads: int, vdim: int, eps: float,
                 dtype: torch.dtype) -> torch.Tensor:
    """Per head o / rms(o), times ``gain`` (over all heads), times the logistic function of ``g`` (a view
    ``[T, heads * vdim]`` with row stride ``g_stride``); result in ``dtype``."""
    _need(o, "o", torch.float32, 2)
    _need(gain, "gain", dims=1)
    if not g.is_cuda or g.dtype != dtype or g.stride(-1) != 1 or g.shape[-1] != n_heads * vdim or gain.shape[0] != n_heads * vdim:
        raise KernelError("mlstm_output: gate or gain does not fit")
    out = torch.empty((o.shape[0], n_heads * vdim), dtype=dtype, device=o.device)
    _check(_fn("mlstm", "bn_mlstm_output")(_ptr(o), _ptr(gain), int(_code(gain)), _ptr(g), int(g_stride), int(_DT[dtype]),
                                           int(o.shape[0]), int(n_heads), int(vdim), c_float(eps), _ptr(out), _stream()),
           "mlstm_output")
    return out


# ---- rotary pairs, parallel blocks, latents ------------------------------------------------------
def rotary_pairs_append(x: torch.Tensor, freqs: torch.Tensor, tok_pos: torch.Tensor, *, xq: Optional[torch.Tensor] = None,
                        q_off: int = 0, n_q_heads: int = 0,
                        q_head_stride: int = 0, q_rot_off: int = 0, k_off: int = 0, n_k_heads: int = 0, k_head_stride: int = 0,
                        k_rot_off: int = 0, k_row: int = 0, v_off: int = 0, v_head_stride: int = 0, v_row: int = 0,
                        tok_seq: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
                        page_table: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
                        v_cache: Optional[torch.Tensor] = None, norm_len: int = 0, norm_w: Optional[torch.Tensor] = None,
                        norm_eps: float = 0.0, split_halves: bool = False, magnitude: float = 1.0,
                        freqs64: Optional[torch.Tensor] = None) -> None:
    """Rotary encoding in place: in every row of x the pairs (2i, 2i + 1), i < len(freqs) (with ``split_halves``
    the pairs (i, i + len(freqs)); cos and sin both times ``magnitude``),
    of the rotated part of each query head (heads ``q_head_stride`` apart from ``q_off``, the part at ``q_rot_off``
    inside a head) and of each key head (likewise) are turned by ``tok_pos * freqs[i]``.  With a cache the first
    ``k_row`` numbers of every key head go there after rotation, and (``v_cache``) the first ``v_row`` numbers of
    the heads at ``v_off`` as they were before it, so ``v_off`` may equal ``k_off``.  ``xq``: the tensor that holds
    the query heads when it is not x (x then holds the key and value heads only).  ``norm_len`` > 0 (one key head): the
    key row's first ``norm_len`` numbers are first divided by their root mean square (``norm_eps`` inside the root) and
    multiplied by ``norm_w``, in place: a latent that is cached normed, in the same launch."""
    _need(x, "x", dims=2)
    xq = x if xq is None else xq
    _need(xq, "xq", x.dtype, 2)
    if xq.shape[0] < tok_pos.shape[0]:
        raise KernelError("rotary_pairs_append: xq has fewer rows than there are tokens")
    _need(freqs, "freqs", torch.float32, 1)
    if freqs64 is not None:  # the same table in double precision: angles are then taken in double precision too
        _need(freqs64, "freqs64", torch.float64, 1)
        if freqs64.shape[0] != freqs.shape[0]:
            raise KernelError("rotary_pairs_append: both tables hold one frequency per pair")
    _need(tok_pos, "tok_pos", torch.int32, 1)
    n = tok_pos.shape[0]
    if x.shape[0] < n:
        raise KernelError("rotary_pairs_append: x has fewer rows than there are tokens")
    pt_stride = 0
    if k_cache is not None:
        for t, nm in ((tok_seq, "tok_seq"), (slots, "slots")):
            _need(t, nm, torch.int32, 1)
        _need(page_table, "page_table", torch.int32, 2)
        _need(k_cache, "k_cache", x.dtype, 4)
        if tuple(k_cache.shape[1:]) != (n_k_heads, PAGE, k_row):
            raise KernelError(f"rotary_pairs_append: key cache {tuple(k_cache.shape)} is not [pages, {n_k_heads}, {PAGE}, {k_row}]")
        if v_cache is not None:
            _need(v_cache, "v_cache", x.dtype, 4)
            if tuple(v_cache.shape[1:]) != (n_k_heads, PAGE, v_row) or v_cache.shape[0] != k_cache.shape[0]:
                raise KernelError(f"rotary_pairs_append: value cache {tuple(v_cache.shape)} is not [pages, {n_k_heads}, {PAGE}, {v_row}]")
        pt_stride = page_table.shape[1]
    elif v_cache is not None:
        raise KernelError("rotary_pairs_append: a value cache needs a key cache")
    if norm_len:
        _need(norm_w, "norm_w", dims=1)
        if norm_w.shape[0] != norm_len or n_k_heads != 1 or norm_len > k_rot_off:
            raise KernelError("rotary_pairs_append: the normed part must be one key head's numbers in front of its rotated part")
    _check(_fn("rotary_pairs", "bn_rotary_pairs_append")(
        _ptr(xq), int(xq.shape[1]), _ptr(x), int(_code(x)), int(n), int(x.shape[1]), _ptr(freqs), int(freqs.shape[0]), _ptr(tok_pos), int(q_off),
        int(n_q_heads), int(q_head_stride), int(q_rot_off), int(k_off), int(n_k_heads), int(k_head_stride), int(k_rot_off),
        int(k_row), int(v_off), int(v_head_stride), int(v_row), _ptr(tok_seq), _ptr(slots), _ptr(page_table), int(pt_stride),
        _ptr(k_cache), _ptr(v_cache), int(norm_len), _ptr(norm_w), int(_code(norm_w)) if norm_w is not None else 0,
        c_float(norm_eps), int(bool(split_halves)), c_float(magnitude), _ptr(freqs64), _stream()), "rotary_pairs_append")


def residual_add(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor] = None,
                 cast: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += a (+ b) on the float32 residual; with ``cast`` returns the new rows in that type."""
    _need(x, "x", torch.float32, 2)
    _need(a, "a", dims=2)
    if a.shape != x.shape or (b is not None and b.shape != x.shape):
        raise KernelError("residual_add: shapes differ")
    if b is not None:
        _need(b, "b", dims=2)
    out = torch.empty(x.shape, dtype=cast, device=x.device) if cast is not None and cast != torch.float32 else None
    _check(_fn("norm", "bn_residual_add")(_ptr(x), _ptr(a), int(_code(a)), _ptr(b), int(_code(b)) if b is not None else 0,
                                          _ptr(out), int(_code(out)) if out is not None else 0,
                                          ctypes.c_longlong(x.numel()), _stream()), "residual_add")
    return x if cast == torch.float32 else out


RESIDUAL_NORMS_MAX_WIDTH = (200 * 1024) // 4 - 32  # rows that fit the fused kernel's shared memory


def residual_add_norms(x: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], w1: torch.Tensor, w2: Optional[torch.Tensor],
                       eps: float, out_dtype: torch.dtype):
    """x += a (+ b) on the float32 residual (the two deltas are added to each other first), and in the same pass
    the norms that read the new rows next: ``(x / rms(x) * w1, x / rms(x) * w2 or None)`` in ``out_dtype``."""
    _need(x, "x", torch.float32, 2)
    _need(a, "a", dims=2)
    _need(w1, "w1", dims=1)
    if a.shape != x.shape or (b is not None and (b.shape != x.shape or not b.is_cuda)) or w1.shape[0] != x.shape[1]:
        raise KernelError("residual_add_norms: sizes do not fit")
    if w2 is not None:
        _need(w2, "w2", w1.dtype, 1)
        if w2.shape[0] != x.shape[1]:
            raise KernelError("residual_add_norms: the second gain does not fit")
    out1 = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    out2 = torch.empty(x.shape, dtype=out_dtype, device=x.device) if w2 is not None else None
    _check(_fn("norm", "bn_residual_add_norms")(_ptr(x), _ptr(a), int(_code(a)), _ptr(b), int(_code(b)) if b is not None else 0,
                                                _ptr(w1), _ptr(w2), int(_code(w1)), c_float(eps), _ptr(out1), _ptr(out2),
                                                int(_code(out1)), int(x.shape[0]), int(x.shape[1]), _stream()), "residual_add_norms")
    return out1, out2


def add_normed(x: torch.Tensor, y: torch.Tensor, wy: torch.Tensor, eps_y: float, w: Optional[torch.Tensor] = None,
               eps: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x += y / sqrt(mean(y^2) + eps_y) * wy on the float32 residual; with ``w`` also returns
    x / sqrt(mean(x^2) + eps) * w of the new rows in ``out_dtype`` (the norm that reads them next)."""
    _need(x, "x", torch.float32, 2)
    _need(y, "y", dims=2)
    _need(wy, "wy", dims=1)
    if y.shape != x.shape or wy.shape[0] != x.shape[1] or (w is not None and w.shape[0] != x.shape[1]):
        raise KernelError("add_normed: sizes do not fit")
    out = None
    if w is not None:
        _need(w, "w", dims=1)
        out = torch.empty(x.shape, dtype=out_dtype or y.dtype, device=x.device)
    _check(_fn("norm", "bn_add_normed")(_ptr(x), _ptr(y), int(_code(y)), _ptr(wy), int(_code(wy)), c_float(eps_y), _ptr(w),
                                        int(_code(w)) if w is not None else 0, c_float(eps), _ptr(out),
                                        int(_code(out)) if out is not None else 0, int(x.shape[0]), int(x.shape[1]),
                                        _stream()), "add_normed")
    return out


def rmsnorm_slices(x: torch.Tensor, eps: float, off0: int, len0: int, w0: torch.Tensor, off1: int = 0, len1: int = 0,
                   w1: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS norms of one or two slices of every row of x, in place, each with a gain of its own."""
    _need(x, "x", dims=2)
    _need(w0, "w0", dims=1)
    if w1 is not None:
        _need(w1, "w1", w0.dtype, 1)
    if w0.shape[0] != len0 or (len1 > 0 and (w1 is None or w1.shape[0] != len1)):
        raise KernelError("rmsnorm_slices: a gain does not fit its slice")
    _check(_fn("norm", "bn_rmsnorm_slices")(_ptr(x), int(_code(x)), int(x.shape[1]), int(x.shape[0]), int(off0), int(len0),
                                            _ptr(w0), int(off1), int(len1), _ptr(w1), int(_code(w0)), c_float(eps),
                                            _stream()), "rmsnorm_slices")
    return x


# ---- gated delta rule ---------------------------------------------------------------------------
def delta_state_floats(heads: int, kv_heads: int, dim: int, vdim: int, taps: int) -> int:
    """Floats of one sequence's state: the heads' matrices, then the convolutions' last ``taps - 1`` inputs."""
    return heads * dim * vdim + (taps - 1) * (2 * kv_heads * dim + heads * vdim)


def delta_rule(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, conv_w: torch.Tensor, taps: int, b_off: int,
               a_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, tok_seq: torch.Tensor,
               seq_start: torch.Tensor, slots: torch.Tensor, n_seqs: int, heads: int, kv_heads: int, dim: int,
               vdim: int) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel over the new tokens of every sequence, from
    and into ``state`` ``[slots, delta_state_floats]`` (float32): short convolutions (``conv_w``: the tap tables
    of the q, k and v channels one after another, ``[channels, taps]``) and SiLU on the projections in ``proj``,
    unit q and k, beta = sigmoid of the ``heads`` numbers at ``b_off`` in ``proj``'s rows, decay = exp(-exp(``a_log``)
    softplus(``a_raw`` + ``dt_bias``)) with ``a_raw`` the first ``heads * dim`` columns of a float32 matrix,
    then S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q token by token.  Returns o, float32
    ``[T, heads * vdim]``."""
    _need(proj, "proj", dims=2)
    _need(conv_w, "conv_w", dims=2)
    _need(a_raw, "a_raw", torch.float32, 2)
    _need(dt_bias, "dt_bias", conv_w.dtype, 1)
    _need(a_log, "a_log", conv_w.dtype, 1)
    _need(state, "state", torch.float32, 2)
    for t, nm in ((tok_seq, "tok_seq"), (seq_start, "seq_start"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    T = tok_seq.shape[0]
    n_qk, n_v = kv_heads * dim, heads * vdim
    if (conv_w.shape != (2 * n_qk + n_v, taps) or b_off + heads > proj.shape[1] or a_raw.shape[0] < T or a_raw.shape[1] < heads * dim
            or dt_bias.shape[0] != heads * dim or a_log.shape[0] != heads or proj.shape[0] < T
            or state.shape[1] != delta_state_floats(heads, kv_heads, dim, vdim, taps) or seq_start.shape[0] < n_seqs + 1):
        raise KernelError("delta_rule: sizes do not fit")
    if dim > 256:
        raise KernelError(f"delta_rule: dim={dim} must be at most 256")
    dev = proj.device
    qn = torch.empty((T, n_qk), dtype=torch.float32, device=dev)
    kn = torch.empty((T, n_qk), dtype=torch.float32, device=dev)
    vc = torch.empty((T, n_v), dtype=torch.float32, device=dev)
    decay = torch.empty((T, heads * dim), dtype=torch.float32, device=dev)
    beta = torch.empty((T, heads), dtype=torch.float32, device=dev)
    out = torch.empty((T, n_v), dtype=torch.float32, device=dev)
    global LAUNCHES
    if taps > 1:
        LAUNCHES += 1  # the kernel that keeps the convolutions' last inputs
    _check(_fn("delta_rule", "bn_delta_prepare")(
        _ptr(proj), int(_code(proj)), int(T), int(proj.shape[1]), int(q_off), int(k_off), int(v_off), int(kv_heads), int(heads),
        int(dim), int(vdim), int(taps), _ptr(conv_w), int(_code(conv_w)), _ptr(state), ctypes.c_longlong(state.shape[1]),
        ctypes.c_longlong(heads * dim * vdim), _ptr(tok_seq), _ptr(seq_start), _ptr(slots), int(n_seqs), int(b_off),
        _ptr(a_raw), int(a_raw.shape[1]), _ptr(dt_bias), _ptr(a_log), c_float(dim ** -0.5), _ptr(qn), _ptr(kn), _ptr(vc), _ptr(decay), _ptr(beta),
        _stream()), "delta_prepare")
    _check(_fn("delta_rule", "bn_delta_rule")(
        _ptr(qn), _ptr(kn), _ptr(vc), _ptr(decay), _ptr(beta), _ptr(state), ctypes.c_longlong(state.shape[1]), _ptr(seq_start),
        _ptr(slots), int(n_seqs), int(heads), int(kv_heads), int(dim), int(vdim), _ptr(out), _stream()), "delta_rule")
    return out


def delta_output(o: torch.Tensor, gain: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int, eps: float,
                 dtype: torch.dtype) -> torch.Tensor:
    """Per head o / rms(o) (over ``vdim``, ``eps`` inside the root), times ``gain`` ``[vdim]`` (shared by the heads), times the
    logistic function of ``gate`` (float32, a view ``[T, heads * vdim]`` with unit inner stride); result in ``dtype``."""
    _need(o, "o", torch.float32, 2)
    _need(gain, "gain", dims=1)
    if (not gate.is_cuda or gate.dtype != torch.float32 or gate.stride(-1) != 1 or gate.shape[-1] != heads * vdim
            or gain.shape[0] != vdim or o.shape[1] != heads * vdim):
        raise KernelError("delta_output: gate or gain does not fit")
    out = torch.empty((o.shape[0], heads * vdim), dtype=dtype, device=o.device)
    _check(_fn("delta_rule", "bn_delta_output")(_ptr(o), _ptr(gain), int(_code(gain)), c_void_p(gate.data_ptr()),
                                                int(gate.stride(0)), int(_DT[dtype]), int(o.shape[0]), int(heads), int(vdim),
                                                c_float(eps), _ptr(out), _stream()), "delta_output")
    return out


# ---- mixture of experts -----------------------------------------------------------------------
def sigmoid_attention_prefill_fits(n_heads: int, n_kv_heads: int, head_dim: int, v_dim: int) -> bool:
    """Whether the tensor-core kernel for runs of new tokens takes these sizes (bfloat16 only)."""
    fn = getattr(build.library("sigmoid_attention_prefill"), "bn_sigmoid_attention_prefill_fits")
    fn.restype = c_int
    return bool(fn(int(n_heads), int(n_kv_heads), int(head_dim), int(v_dim)))


def sigmoid_attention_prefill(q: torch.Tensor, q_stride: int, out: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                              scale: float, window: int, tile_seq: torch.Tensor, tile_row0: torch.Tensor, seq_start: torch.Tensor,
                              seq_pos0: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor, k_cache: torch.Tensor,
                              v_cache: torch.Tensor, *, rel: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                              gate: Optional[torch.Tensor] = None, gate_stride: int = 0, gate_per_head: bool = False,
                              splits: int = 1) -> torch.Tensor:
    """``sigmoid_attention`` for runs of new tokens in bfloat16 on the tensor cores: block i of the step's list
    handles up to 64 new tokens of sequence tile_seq[i] from its row tile_row0[i] on, 16 at a time, each by a
    cluster of one thread block per key/value head.  The same arguments and the same result up to rounding.
    ``splits`` > 1, for steps in which no listed block holds more than 16 rows (one token per sequence: then
    ``tile_row0`` may be None): the pages a block of rows sees are dealt out over so many clusters, and a second
    kernel adds their sums up."""
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.stride(-1) != 1:
        raise KernelError("sigmoid_attention_prefill: q must be a bfloat16 CUDA tensor with unit inner stride")
    _need(out, "out", q.dtype, 2)
    for t, nm in ((tile_seq, "tile_seq"), (seq_start, "seq_start"), (seq_pos0, "seq_pos0"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    if tile_row0 is not None:
        _need(tile_row0, "tile_row0", torch.int32, 1)
    elif splits <= 1:
        raise KernelError("sigmoid_attention_prefill: only a step whose pages are dealt out may leave tile_row0 out")
    _need(page_table, "page_table", torch.int32, 2)
    _need(k_cache, "k_cache", q.dtype, 4)
    _need(v_cache, "v_cache", q.dtype, 4)
    v_dim = v_cache.shape[3]
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or tuple(k_cache.shape[:3]) != tuple(v_cache.shape[:3]):
        raise KernelError(f"sigmoid_attention_prefill: cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim} / value width]")
    if out.shape[1] != n_heads * v_dim or not sigmoid_attention_prefill_fits(n_heads, n_kv_heads, head_dim, v_dim):
        raise KernelError("sigmoid_attention_prefill: sizes do not fit this kernel")
    n_rel = 0
    if rel is not None:
        _need(rel, "rel", torch.float32, 2)
        if rel.shape[1] != n_heads or rel.shape[0] < 1:
            raise KernelError(f"sigmoid_attention_prefill: bias table {tuple(rel.shape)} is not [distances, {n_heads}]")
        n_rel = rel.shape[0]
    if mix is not None:
        _need(mix, "mix", torch.float32, 2)
        if tuple(mix.shape) != (n_heads, n_heads):
            raise KernelError(f"sigmoid_attention_prefill: the mixing matrix {tuple(mix.shape)} is not [{n_heads}, {n_heads}]")
    gate_mode = 0
    if gate is not None:
        gate_mode = 1 if gate_per_head else 2
        need = n_heads if gate_per_head else n_heads * v_dim
        if not gate.is_cuda or gate.dtype != q.dtype or gate.stride(-1) != 1 or gate.shape[-1] < need or gate_stride <= 0:
            raise KernelError("sigmoid_attention_prefill: gate must be a CUDA view of q's type with unit inner stride that holds the gates")
    part = None
    if splits > 1:
        part = torch.empty(out.shape[0] * splits * n_heads * v_dim, dtype=torch.float32, device=q.device)
        global LAUNCHES
        LAUNCHES += 1  # the kernel that adds the splits up
    _check(_fn("sigmoid_attention_prefill", "bn_sigmoid_attention_prefill")(
        _ptr(q), int(q_stride), _ptr(out), int(out.shape[1]), int(tile_seq.shape[0]), int(n_heads), int(n_kv_heads), int(head_dim),
        int(v_dim), c_float(scale), int(window), _ptr(rel), int(n_rel), _ptr(mix),
        c_void_p(gate.data_ptr()) if gate is not None else _NULL, int(gate_stride), int(gate_mode), _ptr(tile_seq), _ptr(tile_row0),
        _ptr(seq_start), _ptr(seq_pos0), _ptr(slots), _ptr(page_table), int(page_table.shape[1]), _ptr(k_cache), _ptr(v_cache),
        _ptr(part), int(max(1, splits)), int(out.shape[0]), _stream()), "sigmoid_attention_prefill")
    return out


def moe_route(h: torch.Tensor, w_router: torch.Tensor, top: int, renormalise: bool = False, softmax: bool = False,
              weight_scale: float = 1.0, sum_eps: float = 0.0):
    """Per token the ``top`` experts with the largest router logits (float32 products), and their scores as
    weights: the logistic function of each logit, or with ``softmax`` the softmax over all experts; divided by
    the chosen ones' sum (+ ``sum_eps``) with ``renormalise``, then times ``weight_scale``:
    ``(ids int32 [T, top], weights float32 [T, top])``."""
    _need(h, "h", dims=2)
    _need(w_router, "w_router", dims=2)
    if w_router.shape[1] != h.shape[1] or not 0 < top <= min(w_router.shape[0], 32) or w_router.shape[0] > 1024:
        raise KernelError(f"moe_route: router {tuple(w_router.shape)}, top {top} do not fit rows of width {h.shape[1]}")
    ids = torch.empty((h.shape[0], top), dtype=torch.int32, device=h.device)
    weights = torch.empty((h.shape[0], top), dtype=torch.float32, device=h.device)
    _check(_fn("moe", "bn_moe_route_ex")(_ptr(h), int(_code(h)), int(h.shape[0]), int(h.shape[1]), _ptr(w_router),
                                         int(_code(w_router)), int(w_router.shape[0]), int(top), int(bool(renormalise)),
                                         int(bool(softmax)), c_float(weight_scale), c_float(sum_eps), _ptr(ids), _ptr(weights),
                                         _stream()), "moe_route")
    return ids, weights


def moe_table_route(tokens: torch.Tensor, table: torch.Tensor, top: int, n_experts: int):
    """Experts by token id: ``(ids int32 [T, top], weights float32 [T, top])`` with ids = ``table[token, :top]`` and
    every weight 1 / top (an id or an entry out of range takes weight 0)."""
    _need(tokens, "tokens", torch.int32, 1)
    _need(table, "table", torch.int32, 2)
    if not 0 < top <= table.shape[1]:
        raise KernelError(f"moe_table_route: a table of {table.shape[1]} columns has no {top} experts per token")
    T = tokens.shape[0]
    ids = torch.empty((T, top), dtype=torch.int32, device=tokens.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=tokens.device)
    _check(_fn("moe", "bn_moe_table_route")(_ptr(tokens), int(T), _ptr(table), int(table.shape[0]), int(table.shape[1]), int(top),
                                            int(n_experts), c_float(1.0 / top), _ptr(ids), _ptr(weights), _stream()),
           "moe_table_route")
    return ids, weights


MOE_FEW_SMEM = 200 * 1024  # bytes of shared memory the streaming expert kernels may take (moe.cu: MOE_SMEM_MAX)


def moe_few_fits(width: int, top: int, ff: int) -> bool:
    """Whether the streaming expert kernels hold a token's input (``width`` float32) and its experts' activations
    (``top * ff`` float32) in a block's shared memory."""
    return 4 * width <= MOE_FEW_SMEM and 4 * top * ff <= MOE_FEW_SMEM


def moe_experts_few(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                    w_down: torch.Tensor, limit: float, slope: float, scale_input: bool,
                    add: Optional[torch.Tensor] = None, act: int = -1) -> torch.Tensor:
    """The chosen experts of every token, streamed once per (token, expert): float32 ``[T, width]``, the sum over
    a token's experts plus ``add``.  The weight multiplies the expert's input (``scale_input``) or its output.
    ``act`` < 0: the clamped unit with ``limit`` and ``slope``; ACT_SILU / ACT_GELU_TANH: act(gate) * up.
    ``w_gate_up`` ``[experts, 2 * ff, width]`` holds an expert's gate rows and then its up rows, ``w_down``
    ``[experts, width, ff]``; both in h's type."""
    _need(h, "h", dims=2)
    T, width = h.shape
    _need(ids, "ids", torch.int32, 2)
    _need(weights, "weights", torch.float32, 2)
    top = ids.shape[1]
    _need(w_gate_up, "w_gate_up", h.dtype, 3)
    _need(w_down, "w_down", h.dtype, 3)
    E, ff = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    if (tuple(w_gate_up.shape) != (E, 2 * ff, width) or tuple(w_down.shape) != (E, width, ff)
            or tuple(ids.shape) != (T, top) or tuple(weights.shape) != (T, top) or not moe_few_fits(width, top, ff)):
        raise KernelError("moe_experts_few: sizes do not fit")
    if add is not None:
        _need(add, "add", dims=2)
        if tuple(add.shape) != (T, width):
            raise KernelError("moe_experts_few: add does not fit")
    y = torch.empty((T * top, ff), dtype=h.dtype, device=h.device)
    w_up = w_gate_up[:, ff:]
    _check(_fn("moe", "bn_moe_gate_up_ex")(_ptr(h), int(_code(h)), int(T), int(width), _ptr(ids), _ptr(weights),
                                           int(bool(scale_input)), _ptr(w_gate_up), c_void_p(w_up.data_ptr()),
                                           ctypes.c_longlong(2 * ff * width), int(ff), int(top), c_float(limit),
                                           c_float(slope), int(act), _ptr(y), _stream()), "moe_gate_up")
    out = torch.empty((T, width), dtype=torch.float32, device=h.device)
    _check(_fn("moe", "bn_moe_down")(_ptr(y), int(_code(y)), int(T), int(ff), _ptr(ids), _ptr(weights),
                                     int(not scale_input), _ptr(w_down), int(width), int(top), _ptr(add),
                                     int(_code(add) if add is not None else 0), _ptr(out), _stream()), "moe_down")
    return out


def moe_count(ids: torch.Tensor, n_experts: int) -> torch.Tensor:
    """int32 ``[experts]``: how many (token, expert) items chose each expert."""
    _need(ids, "ids", torch.int32, 2)
    counts = torch.zeros(n_experts, dtype=torch.int32, device=ids.device)
    _check(_fn("moe", "bn_moe_count")(_ptr(ids), int(ids.numel()), _ptr(counts), _stream()), "moe_count")
    return counts


def moe_sort(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, counts: torch.Tensor, scale_input: bool,
             cap: int = 0):
    """Sort the (token, expert) items by expert: ``(x_sorted, place int32 [T * top], offsets int32 [experts + 1])``.
    Item i went to row ``place[i]`` of ``x_sorted``, which holds its token's row of h (times its weight with
    ``scale_input``).  ``cap`` = 0: the experts' rows are packed, expert e's are rows ``offsets[e] ..
    offsets[e + 1]`` of ``[T * top, width]``.  ``cap`` > 0 (at least the largest of ``counts``): expert e's rows
    begin at ``e * cap`` of ``[experts * cap, width]``; rows that no item took hold nothing."""
    _need(h, "h", dims=2)
    _need(ids, "ids", torch.int32, 2)
    _need(weights, "weights", torch.float32, 2)
    _need(counts, "counts", torch.int32, 1)
    T, width = h.shape
    top, n_experts = ids.shape[1], counts.shape[0]
    book = torch.empty(2 * n_experts + 1, dtype=torch.int32, device=h.device)
    offsets, cursor = book[:n_experts + 1], book[n_experts + 1:]
    place = torch.empty(T * top, dtype=torch.int32, device=h.device)
    rows = n_experts * cap if cap > 0 else T * top
    x_sorted = torch.empty((rows, width), dtype=h.dtype, device=h.device)
    _check(_fn("moe", "bn_moe_scatter")(_ptr(h), int(_code(h)), int(T), int(width), _ptr(ids), _ptr(weights),
                                        int(bool(scale_input)), int(top), int(n_experts), int(cap), _ptr(counts),
                                        _ptr(offsets), _ptr(cursor), _ptr(place), _ptr(x_sorted), _stream()), "moe_sort")
    global LAUNCHES
    LAUNCHES += 1
    return x_sorted, place, offsets


def moe_gather(y_sorted: torch.Tensor, place: torch.Tensor, weights: torch.Tensor, scale_output: bool,
               add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 ``[T, width]``: per token the sum of its experts' rows of ``y_sorted`` (times their weight with
    ``scale_output``), plus ``add``."""
    _need(y_sorted, "y_sorted", dims=2)
    _need(place, "place", torch.int32, 1)
    _need(weights, "weights", torch.float32, 2)
    T, top = weights.shape
    width = y_sorted.shape[1]
    if y_sorted.shape[0] < T * top or place.shape[0] != T * top:
        raise KernelError("moe_gather: sizes do not fit")
    if add is not None:
        _need(add, "add", dims=2)
        if tuple(add.shape) != (T, width):
            raise KernelError("moe_gather: add does not fit")
    out = torch.empty((T, width), dtype=torch.float32, device=y_sorted.device)
    _check(_fn("moe", "bn_moe_gather")(_ptr(y_sorted), int(_code(y_sorted)), int(T), int(width), _ptr(place), _ptr(weights),
                                       int(bool(scale_output)), int(top), _ptr(add), int(_code(add) if add is not None else 0),
                                       _ptr(out), _stream()), "moe_gather")
    return out


def batched_matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``[B, M, K] . [B, N, K]^T -> [B, M, N]`` by the library's batched product (float32 sums; float32 inputs
    in true float32): the experts of a mixture at once, each on its own block of rows."""
    _need(x, "x", dims=3)
    _need(w, "w", x.dtype, 3)
    if x.shape[0] != w.shape[0] or x.shape[2] != w.shape[2]:
        raise KernelError(f"batched_matmul: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    if w.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("float32 products need torch.backends.cuda.matmul.allow_tf32 = False")
    product = lambda: torch.bmm(x, w.transpose(1, 2))
    return product() if PROFILE is None else _timed("library.bmm", product)


def matmul_into(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = x . w^T by the library product, written into ``out`` (a slice of a larger buffer, say): for
    many products of many rows whose results lie side by side.  float32 products are true float32."""
    _need(x, "x", dims=2)
    _need(w, "w", x.dtype, 2)
    _need(out, "out", x.dtype, 2)
    if x.shape[1] != w.shape[1] or tuple(out.shape) != (x.shape[0], w.shape[0]):
        raise KernelError(f"matmul_into: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    if w.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("float32 products need torch.backends.cuda.matmul.allow_tf32 = False")
    product = lambda: torch.matmul(x, w.t(), out=out)
    return product() if PROFILE is None else _timed("library.matmul", product)


# ---- sampling -----------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "logits", torch.float32, 2)
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    n = logits.shape[0]
    _scr, counters = _split_scratch(logits.device)
    if n > counters.numel():
        raise KernelError(f"argmax: at most {counters.numel()} rows at a time")
    part_v = torch.empty(n * 64, dtype=torch.float32, device=logits.device)
    part_i = torch.empty(n * 64, dtype=torch.int32, device=logits.device)
    _check(_fn("sampling", "bn_argmax")(_ptr(logits), int(logits.shape[1]), int(n), int(logits.shape[1]),
                                        _ptr(out), _ptr(part_v), _ptr(part_i), _ptr(counters), _stream()), "argmax")
    return out


def sample_temperature(logits: torch.Tensor, temperature: float, rng_state: torch.Tensor,
                       out: Optional[torch.Tensor] = None, index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row from softmax(logits / temperature).  ``rng_state`` holds xorshift64* states
    (int64 bit patterns); row r uses and advances state ``index[r]`` (or r without an index)."""
    _need(logits, "logits", torch.float32, 2)
    _need(rng_state, "rng_state", torch.int64, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    elif rng_state.shape[0] < logits.shape[0]:
        raise KernelError("sample_temperature: one generator state per row is needed")
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    _check(_fn("sampling", "bn_sample_temperature")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                                    int(logits.shape[1]), c_float(temperature), _ptr(rng_state),
                                                    _ptr(index), _ptr(out), _stream()), "sample_temperature")
    return out


def sample_topp(logits: torch.Tensor, temperature: float, topp: float, rng_state: torch.Tensor,
                out: Optional[torch.Tensor] = None, index: Optional[torch.Tensor] = None,
                probs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Nucleus sampling: one draw per row from the smallest set of most probable tokens whose
    mass exceeds ``topp``.  ``probs`` is scratch of the shape of ``logits``."""
    _need(logits, "logits", torch.float32, 2)
    _need(rng_state, "rng_state", torch.int64, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    if probs is None:
        probs = torch.empty_like(logits)
    _need(probs, "probs", torch.float32, 2)
    if probs.shape[0] < logits.shape[0] or probs.shape[1] != logits.shape[1]:
        raise KernelError("sample_topp: probs scratch does not fit")
    out = out if out is not None else torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, 1)
    _check(_fn("sampling", "bn_sample_topp")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                             int(logits.shape[1]), c_float(temperature), c_float(topp),
                                             _ptr(rng_state), _ptr(index), _ptr(probs), _ptr(out), _stream()),
           "sample_topp")
    return out


def repeat_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_len: torch.Tensor, penalty: float,
                   index: Optional[torch.Tensor] = None) -> None:
    """In place: for each distinct id among the first recent_len[s] entries of recent[s] (s = index[r]
    or r), logit > 0 ? logit / penalty : logit * penalty."""
    _need(logits, "logits", torch.float32, 2)
    _need(recent, "recent", torch.int32, 2)
    _need(recent_len, "recent_len", torch.int32, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    _check(_fn("sampling", "bn_repeat_penalty")(_ptr(logits), int(logits.shape[1]), int(logits.shape[0]),
                                                int(logits.shape[1]), _ptr(recent), int(recent.shape[1]),
                                                _ptr(recent_len), _ptr(index), c_float(penalty), _stream()),
           "repeat_penalty")


def sampler_accept(recent: torch.Tensor, recent_len: torch.Tensor, recent_pos: torch.Tensor, tokens: torch.Tensor,
                   index: Optional[torch.Tensor] = None) -> None:
    """Push tokens[r] into the ring of recent tokens of state row index[r] (or r)."""
    _need(recent, "recent", torch.int32, 2)
    _need(recent_len, "recent_len", torch.int32, 1)
    _need(recent_pos, "recent_pos", torch.int32, 1)
    _need(tokens, "tokens", torch.int32, 1)
    if index is not None:
        _need(index, "index", torch.int32, 1)
    _check(_fn("sampling", "bn_sampler_accept")(_ptr(recent), int(recent.shape[1]), _ptr(recent_len),
                                                _ptr(recent_pos), _ptr(index), _ptr(tokens), int(tokens.shape[0]),
                                                _stream()), "sampler_accept")
