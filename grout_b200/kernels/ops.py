"""Typed, checked entry points of the CUDA kernels.

Each function takes torch CUDA tensors, checks dtype, shape and contiguity,
and launches the kernel on torch's current stream.  Nothing here computes: a
tensor that is not on the GPU, or a size a kernel does not take, raises.
"""
from __future__ import annotations

import ctypes
import functools
import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from .build import module

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_CODES = {"p": _P, "i": _I, "f": _F, "l": _L}
_FUNCS = {}


class KernelError(RuntimeError):
    pass


_OWN_ERRORS = {-1: "the kernel refused its arguments (bad size or pointer)",
               -2: "no kernel for this combination of sizes and types",
               -3: "size beyond the kernel's stated maximum"}


def _fn(mod: str, name: str, sig: str):
    key = (mod, name)
    f = _FUNCS.get(key)
    if f is None:
        f = getattr(module(mod), name)
        f.argtypes = [_CODES[c] for c in sig]
        f.restype = c_int
        _FUNCS[key] = f
    return f


_LAUNCHES = 0


def launch_count() -> int:
    """Kernel launches made through this module so far (a decode-attention call
    with more than one split counts its merge kernel too)."""
    return _LAUNCHES


class OpProfile:
    """Per-operation device times of steps that are launched one by one (not
    replayed from a graph): CUDA events around every call of this module, with
    the bytes each call has to move and the flops it has to do, so that the
    report can set every kernel against the machine's peaks.  (The reference's
    per-op totals: src/model.rs:1139-1142, 1183-1207, filled at 4370-4379.)"""

    def __init__(self, hbm_gbs: Optional[float] = None, tflops: Optional[float] = None,
                 lead_us: int = 80):
        """``lead_us``: how long the device is kept busy in front of every timed
        call (a timer kernel), so that the call and its events are queued by the
        time the device gets to them and the interval is the kernel's own; 0
        for none."""
        self.hbm_gbs, self.tflops, self.lead_us = hbm_gbs, tflops, int(lead_us)
        self.records = []          # (name, start event, end event, bytes, flops); the last two may be callables

    def add(self, name, a, b, nbytes, flops) -> None:
        self.records.append((name, a, b, nbytes, flops))

    def totals(self):
        """name -> [calls, ms, bytes, flops], after waiting for the device."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b, nbytes, flops in self.records:
            r = out.setdefault(name, [0, 0.0, 0.0, 0.0])
            r[0] += 1
            r[1] += a.elapsed_time(b)
            r[2] += float(nbytes() if callable(nbytes) else nbytes)
            r[3] += float(flops() if callable(flops) else flops)
        return out

    def report(self) -> str:
        rows = sorted(self.totals().items(), key=lambda kv: -kv[1][1])
        whole = sum(r[1] for _n, r in rows) or 1.0
        head = ("op profile (an event pair around every call, each kernel alone on the device; steps are "
                "not replayed from graphs)\n")
        head += f"  {'op':<22}{'calls':>7}{'total_ms':>10}{'avg_us':>9}{'share':>7}{'GB/s':>9}{'TFLOP/s':>9}"
        if self.hbm_gbs or self.tflops:
            head += f"{'of hbm':>8}{'of mma':>8}"
        lines = [head]
        for name, (calls, ms, nbytes, flops) in rows:
            gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            tfs = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
            line = (f"  {name:<22}{calls:>7}{ms:>10.3f}{ms / calls * 1e3:>9.2f}{ms / whole:>7.1%}"
                    f"{gbs:>9.0f}{tfs:>9.1f}")
            if self.hbm_gbs or self.tflops:
                line += f"{(gbs / self.hbm_gbs if self.hbm_gbs else 0):>8.2f}"
                line += f"{(tfs / self.tflops if self.tflops else 0):>8.2f}"
            lines.append(line)
        return "\n".join(lines)


_PROFILE: Optional[OpProfile] = None


def set_profile(profile: Optional[OpProfile]) -> None:
    """Turns the per-operation profile on (an ``OpProfile``) or off (None)."""
    global _PROFILE
    _PROFILE = profile


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


def _profiled(name: str, cost):
    """Decorator: with a profile on, brackets the call with events and notes
    ``cost(result, *args, **kw) -> (bytes, flops)``."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kw):
            prof = _PROFILE
            if prof is None:
                return fn(*args, **kw)
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            if prof.lead_us:
                _fn("elementwise", "gb_delay_ns", "lp")(prof.lead_us * 1000, _stream())
            a.record()
            out = fn(*args, **kw)
            b.record()
            nbytes, flops = cost(out, *args, **kw)
            prof.add(name, a, b, nbytes, flops)
            return out
        return wrapper
    return deco


def _cost_io(out, *args, **kw):
    """What goes in and what comes out, each once."""
    outs = out if isinstance(out, (tuple, list)) else (out,)
    return _nbytes(*args, *kw.values(), *outs), 0


def _cost_gemm(out, x, w, *args, **kw):
    M, K = x.shape
    N = w.shape[0]
    return _nbytes(x, w, out), 2.0 * M * N * K


def _cost_attention(out, q, k_pages, *args, **kw):
    """Keys and values of the live sequences once, q in, the result out; flops of
    the two products over the keys every query row sees (lengths are on the
    device: they are read when the report is made)."""
    nq, D = q.shape[1], q.shape[2]
    nkv, item = k_pages.shape[1], k_pages.element_size()
    kv_len, slots, cu_q, window = kw.get("kv_len"), kw.get("slots"), kw.get("cu_q"), kw.get("window")
    if kv_len is None:
        return _nbytes(q, out), 0
    live = (slots >= 0)
    lens = torch.where(live, kv_len, torch.zeros_like(kv_len)).double()
    if cu_q is not None:
        rows = torch.where(live, cu_q[1:] - cu_q[:-1], torch.zeros_like(kv_len)).double()
    else:
        rows = live.double()
    pairs = rows * (lens - rows) + rows * (rows + 1) / 2        # (query, visible key) pairs, causal
    if window:
        pairs = torch.minimum(pairs, rows * float(window))
        lens = torch.minimum(lens, rows + float(window))
    kv_bytes = (lens.sum() * (2 * nkv * D * item))
    pair_sum = pairs.sum()
    base = _nbytes(q, out)
    return (lambda: base + float(kv_bytes.item())), (lambda: 4.0 * nq * D * float(pair_sum.item()))


def _cost_qk_prepare(out, qkv, nq, nkv, D):
    """The projection in, q out, and k and v out (to their pages or to a tensor)."""
    q = out[0]
    kv_bytes = q.shape[0] * 2 * nkv * D * q.element_size()
    return _nbytes(qkv, q) + kv_bytes, 0


LAUNCH_LOG: Optional[list] = None     # when a list: one label per kernel launched, in order


def _check(rc: int, what: str, kernels: int = 1, detail: str = "") -> None:
    global _LAUNCHES
    if rc == 0:
        _LAUNCHES += kernels
        if LAUNCH_LOG is not None and kernels > 0:
            LAUNCH_LOG.extend([what + detail] + [what + " (second kernel)"] * (kernels - 1))
        return
    if rc in _OWN_ERRORS:
        raise KernelError(f"{what}: {_OWN_ERRORS[rc]}")
    raise KernelError(f"{what}: CUDA error {rc} at launch ({_cuda_error_name(rc)})")


def _cuda_error_name(rc: int) -> str:
    try:
        return str(torch.cuda.cudart().cudaGetErrorString(torch.cuda.cudart().cudaError(rc)))
    except Exception:
        return "cudaError_t value"


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"kernels take float32 or bfloat16 activations, not {dtype}")


def _need(t: Optional[torch.Tensor], name: str, dtype=None, ndim=None) -> None:
    if t is None:
        raise KernelError(f"{name} is missing")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, found {tuple(t.shape)}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------- embedding
@_profiled("embed", lambda out, table, ids: (_nbytes(ids, out, out), 0))
def embed(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    _need(table, "embedding table", ndim=2)
    _need(ids, "token ids", torch.int32, 1)
    V, H = table.shape
    out = torch.empty((ids.shape[0], H), dtype=table.dtype, device=table.device)
    sfx = _suffix(table.dtype)
    _check(_fn("embed", f"gb_embed_{sfx}", "pppiiip")(
        table.data_ptr(), ids.data_ptr(), out.data_ptr(), ids.shape[0], H, V, _stream()), "embed")
    return out


@_profiled("embed_scaled", lambda out, table, ids, scale, **k: (_nbytes(ids, out) + out.numel() * table.element_size(), 0))
def embed_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float,
                 into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """scale * table[ids[t]] as 32-bit rows [T, H] (the product is 32-bit whatever the table's
    type), written into ``into`` when given."""
    out = into
    _need(table, "embedding table", ndim=2)
    _need(ids, "token ids", torch.int32, 1)
    V, H = table.shape
    if out is None:
        out = torch.empty((ids.shape[0], H), dtype=torch.float32, device=table.device)
    else:
        _need(out, "embedding output", torch.float32, 2)
        if tuple(out.shape) != (ids.shape[0], H):
            raise KernelError(f"the output is {tuple(out.shape)}, expected {(ids.shape[0], H)}")
    _check(_fn("embed", f"gb_embed_scaled_{_suffix(table.dtype)}", "ppfpiiip")(
        table.data_ptr(), ids.data_ptr(), float(scale), out.data_ptr(), ids.shape[0], H, V, _stream()),
        "embed_scaled")
    return out


@_profiled("embed_pos_norm", lambda out, table, positions, ids, pos, w, eps: (_nbytes(ids, pos, out) + out.numel() * 2 * table.element_size(), 0))
def embed_pos_norm(table: torch.Tensor, positions: torch.Tensor, ids: torch.Tensor,
                   token_pos: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """rmsnorm(table[ids[t]] + positions[token_pos[t]]) * weight as 32-bit rows [T, H]: the
    sum and the norm are 32-bit whatever the tables' type."""
    _need(table, "embedding table", ndim=2)
    _need(positions, "position table", table.dtype, 2)
    _need(ids, "token ids", torch.int32, 1)
    _need(token_pos, "token positions", torch.int32, 1)
    _need(weight, "norm weight", torch.float32, 1)
    V, H = table.shape
    if positions.shape[1] != H or weight.shape[0] != H or token_pos.shape[0] != ids.shape[0]:
        raise KernelError("the tables, the norm weight and the position list do not fit together")
    out = torch.empty((ids.shape[0], H), dtype=torch.float32, device=table.device)
    _check(_fn("embed", f"gb_embed_pos_norm_{_suffix(table.dtype)}", "pppppfpiiiip")(
        table.data_ptr(), positions.data_ptr(), ids.data_ptr(), token_pos.data_ptr(),
        weight.data_ptr(), float(eps), out.data_ptr(), ids.shape[0], H, V, positions.shape[0],
        _stream()), "embed_pos_norm")
    return out


# ---------------------------------------------------------------- norm
@_profiled("add_rmsnorm", _cost_io)
def add_rmsnorm(res_in: Optional[torch.Tensor], delta: Optional[torch.Tensor],
                weight: torch.Tensor, eps: float, *, dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, write_res: bool = True
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """(res_in + delta) in 32-bit -> (residual, normed).  Without ``rows`` the
    residual is updated in place when ``res_in`` is given.  ``delta`` may also be
    a stack of 32-bit partial sums [S, T, N] (what a split-K product leaves): they
    are added in order."""
    parts = None
    if delta is not None and delta.dim() == 3:
        _need(delta, "partial sums", torch.float32, 3)
        parts, delta = delta, None
    src = res_in if res_in is not None else (delta if delta is not None else
                                             (parts[0] if parts is not None else None))
    if src is None:
        raise KernelError("add_rmsnorm needs a residual or a delta")
    if res_in is not None:
        _need(res_in, "residual", torch.float32, 2)
    if delta is not None:
        _need(delta, "delta", dtype, 2)
        if res_in is not None and delta.shape != res_in.shape:
            raise KernelError(f"residual {tuple(res_in.shape)} and delta {tuple(delta.shape)} differ")
    if parts is not None and res_in is not None and tuple(parts.shape[1:]) != tuple(res_in.shape):
        raise KernelError(f"residual {tuple(res_in.shape)} and partial sums {tuple(parts.shape)} differ")
    _need(weight, "norm weight", ndim=1)
    N = src.shape[1]
    if weight.shape[0] != N:
        raise KernelError(f"norm weight has {weight.shape[0]} elements for rows of {N}")
    w_is_f32 = weight.dtype == torch.float32
    if not w_is_f32 and weight.dtype != dtype:
        raise KernelError(f"norm weight must be float32 or {dtype}, found {weight.dtype}")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        n_rows = rows.shape[0]
    else:
        n_rows = src.shape[0]
    res_out = None
    if write_res:
        if rows is None and res_in is not None:
            res_out = res_in
        else:
            res_out = torch.empty((n_rows, N), dtype=torch.float32, device=src.device)
    y = torch.empty((n_rows, N), dtype=dtype, device=src.device)
    sfx = _suffix(dtype)
    _check(_fn("norm", f"gb_add_rmsnorm_{sfx}", "pppilppifppiip")(
        _ptr(res_in), _ptr(delta), _ptr(parts), 0 if parts is None else parts.shape[0],
        0 if parts is None else parts.stride(0), _ptr(rows), weight.data_ptr(), int(w_is_f32),
        float(eps), _ptr(res_out), y.data_ptr(), n_rows, N, _stream()), "add_rmsnorm")
    return res_out, y


class _LayerNormArgs(ctypes.Structure):
    _fields_ = [("res_in", _P), ("delta", _P), ("parts", _P), ("n_parts", _I), ("part_stride", _L),
                ("rows", _P), ("post_w", _P), ("post_b", _P), ("post_eps", _F), ("post_center", _I),
                ("mult", _F), ("offset", _P), ("w", _P), ("b", _P), ("eps", _F), ("center", _I),
                ("res_out", _P), ("y", _P), ("n_rows", _I), ("N", _I)]


@_profiled("add_layernorm", _cost_io)
def add_layernorm(res_in: Optional[torch.Tensor], delta: Optional[torch.Tensor],
                  weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float,
                  center: bool = True, *, dtype: torch.dtype,
                  rows: Optional[torch.Tensor] = None, write_res: bool = True, mult: float = 1.0,
                  offset: Optional[torch.Tensor] = None, post_weight: Optional[torch.Tensor] = None,
                  post_bias: Optional[torch.Tensor] = None, post_eps: float = 0.0,
                  post_center: bool = True) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """v = res_in + mult * post(delta) + offset in 32-bit -> (residual, norm(v)).

    ``post`` is the layer norm (post_weight, post_bias, post_eps) that ``delta``
    passes through first, the identity without ``post_weight``; ``norm`` is the
    layer norm (weight, bias, eps), and without ``weight`` only the sum is made.
    A norm that does not ``center`` leaves the mean in.  ``delta`` is [T, N] in
    ``dtype`` or a stack of 32-bit partial sums [S, T, N], added in order;
    ``offset`` is a 32-bit vector [N]; norm weights and biases are 32-bit.  Without
    ``rows`` the residual is updated in place when ``res_in`` is given."""
    parts = None
    if delta is not None and delta.dim() == 3:
        _need(delta, "partial sums", torch.float32, 3)
        parts, delta = delta, None
    src = res_in if res_in is not None else (delta if delta is not None else
                                             (parts[0] if parts is not None else None))
    if src is None:
        raise KernelError("add_layernorm needs a residual or a delta")
    if res_in is not None:
        _need(res_in, "residual", torch.float32, 2)
    if delta is not None:
        _need(delta, "delta", dtype, 2)
        if res_in is not None and delta.shape != res_in.shape:
            raise KernelError(f"residual {tuple(res_in.shape)} and delta {tuple(delta.shape)} differ")
    if parts is not None and res_in is not None and tuple(parts.shape[1:]) != tuple(res_in.shape):
        raise KernelError(f"residual {tuple(res_in.shape)} and partial sums {tuple(parts.shape)} differ")
    N = src.shape[1]
    for t, nm in ((weight, "norm weight"), (bias, "norm bias"), (post_weight, "inner norm weight"),
                  (post_bias, "inner norm bias"), (offset, "offset")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != N:
                raise KernelError(f"{nm} has {t.shape[0]} elements for rows of {N}")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        n_rows = rows.shape[0]
    else:
        n_rows = src.shape[0]
    res_out = None
    if write_res or weight is None:
        if rows is None and res_in is not None:
            res_out = res_in
        else:
            res_out = torch.empty((n_rows, N), dtype=torch.float32, device=src.device)
    y = torch.empty((n_rows, N), dtype=dtype, device=src.device) if weight is not None else None
    a = _LayerNormArgs()
    a.res_in, a.delta, a.parts = _ptr(res_in), _ptr(delta), _ptr(parts)
    a.n_parts = 0 if parts is None else parts.shape[0]
    a.part_stride = 0 if parts is None else parts.stride(0)
    a.rows, a.post_w, a.post_b = _ptr(rows), _ptr(post_weight), _ptr(post_bias)
    a.post_eps, a.post_center, a.mult, a.offset = float(post_eps), int(post_center), float(mult), _ptr(offset)
    a.w, a.b, a.eps, a.center = _ptr(weight), _ptr(bias), float(eps), int(center)
    a.res_out, a.y, a.n_rows, a.N = _ptr(res_out), _ptr(y), n_rows, N
    _check(_fn("layernorm", f"gb_add_layernorm_{_suffix(dtype)}", "pp")(
        ctypes.addressof(a), _stream()), "add_layernorm")
    return res_out, y


class _PostNormArgs(ctypes.Structure):
    _fields_ = [("res_in", _P), ("delta", _P), ("parts", _P), ("n_parts", _I), ("part_stride", _L),
                ("rows", _P), ("post_w", _P), ("post_eps", _F), ("scale", _P), ("w", _P),
                ("eps", _F), ("res_out", _P), ("y", _P), ("n_rows", _I), ("N", _I)]


@_profiled("add_postnorm", _cost_io)
def add_postnorm(res_in: Optional[torch.Tensor], delta: Optional[torch.Tensor], *,
                 dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                 post_weight: Optional[torch.Tensor] = None, post_eps: float = 0.0,
                 scale: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                 eps: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """v = res_in + scale * rmsnorm(delta; post_weight, post_eps) in 32-bit -> (v, y), where
    y = rmsnorm(v; weight, eps) or, without ``weight``, v itself, in ``dtype``.  Without
    ``post_weight`` delta is added as it is, without ``scale`` unscaled.  ``delta`` is [T, N]
    in ``dtype`` or a stack of 32-bit partial sums [S, T, N], added in order; all vectors
    are 32-bit [N].  Without ``rows`` the stream is updated in place when given."""
    parts = None
    if delta is not None and delta.dim() == 3:
        _need(delta, "partial sums", torch.float32, 3)
        parts, delta = delta, None
    src = res_in if res_in is not None else (delta if delta is not None else
                                             (parts[0] if parts is not None else None))
    if src is None:
        raise KernelError("add_postnorm needs a residual or a delta")
    if res_in is not None:
        _need(res_in, "residual", torch.float32, 2)
    if delta is not None:
        _need(delta, "delta", dtype, 2)
    for t in (delta, parts[0] if parts is not None else None):
        if t is not None and res_in is not None and tuple(t.shape) != tuple(res_in.shape):
            raise KernelError(f"residual {tuple(res_in.shape)} and delta {tuple(t.shape)} differ")
    N = src.shape[1]
    for t, nm in ((post_weight, "inner norm weight"), (scale, "scale"), (weight, "norm weight")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != N:
                raise KernelError(f"{nm} has {t.shape[0]} elements for rows of {N}")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
    n_rows = rows.shape[0] if rows is not None else src.shape[0]
    nothing_added = delta is None and parts is None
    if nothing_added and rows is None and weight is None and dtype == torch.float32:
        return res_in, res_in                       # the stream is its own 32-bit reading
    if rows is None and res_in is not None:
        res_out = None if nothing_added else res_in
    else:
        res_out = torch.empty((n_rows, N), dtype=torch.float32, device=src.device)
    y = torch.empty((n_rows, N), dtype=dtype, device=src.device)
    a = _PostNormArgs()
    a.res_in, a.delta, a.parts = _ptr(res_in), _ptr(delta), _ptr(parts)
    a.n_parts = 0 if parts is None else parts.shape[0]
    a.part_stride = 0 if parts is None else parts.stride(0)
    a.rows, a.post_w, a.post_eps, a.scale = _ptr(rows), _ptr(post_weight), float(post_eps), _ptr(scale)
    a.w, a.eps, a.res_out, a.y, a.n_rows, a.N = _ptr(weight), float(eps), _ptr(res_out), y.data_ptr(), n_rows, N
    _check(_fn("norm", f"gb_add_postnorm_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "add_postnorm")
    return (res_in if res_out is None else res_out), y


# ---------------------------------------------------------------- q/k preparation
class _QkPrepareArgs(ctypes.Structure):
    _fields_ = [("qkv", _P), ("q_w", _P), ("k_w", _P), ("inv_freq", _P), ("token_seq", _P),
                ("token_pos", _P), ("slots", _P), ("block_table", _P), ("q_out", _P),
                ("kv_out", _P), ("k_pages", _P), ("v_pages", _P), ("eps", _F),
                ("n_tokens", _I), ("nq", _I), ("nkv", _I), ("D", _I), ("rot_dim", _I),
                ("max_pages", _I), ("page", _I), ("qkv_parts", _P), ("n_parts", _I),
                ("part_stride", _L), ("v_from_k", _I), ("Dv", _I), ("Ds", _I),
                ("q_temp_coef", _F), ("q_temp_every", _I), ("interleaved", _I)]


@_profiled("qk_prepare", lambda out, qkv, nq, nkv, D, **k: _cost_qk_prepare(out, qkv, nq, nkv, D))
def qk_prepare(qkv: torch.Tensor, nq: int, nkv: int, D: int, *, q_w=None, k_w=None,
               eps: float = 0.0, inv_freq=None, rot_dim: int = 0, token_seq, token_pos, slots,
               block_table=None, k_pages=None, v_pages=None, page: int = 0,
               want_kv_out: bool = False, values_are_keys: bool = False,
               v_dim: Optional[int] = None, q_temp: Optional[Tuple[float, int]] = None,
               interleaved: bool = False):
    """Returns (q [T, nq, Ds], kv_out or None); writes k, v into the pages when given.
    ``qkv`` may be a stack of 32-bit partial sums [S, T, width] of the projection
    (bf16 engines only): they are added in order.  ``values_are_keys``: the
    projection holds q and k only, and a value is its key before the rotation.
    ``v_dim``: the size of a value head in the projection when it is not D; the
    rows that are written (q, kv_out, pages) are then Ds wide, Ds being the pages'
    row width (at least D and ``v_dim``) or, without pages, the larger of the two,
    and end in zeros.  ``q_temp`` = (coef, every): a query at position p is
    multiplied, after its norm, by 1 + coef * ln(floor((p + 1) / every) + 1).
    ``interleaved``: the rotation pairs element 2j with 2j + 1 (else j with j + rot_dim / 2)."""
    parts = None
    if qkv.dim() == 3:
        _need(qkv, "qkv partial sums", torch.float32, 3)
        if k_pages is not None and k_pages.dtype != torch.bfloat16:
            raise KernelError("partial sums of qkv are taken with a bfloat16 cache only")
        parts, dt = qkv, torch.bfloat16
    else:
        _need(qkv, "qkv", ndim=2)
        dt = qkv.dtype
    T = qkv.shape[-2]
    Dv = int(v_dim) if v_dim else D
    if Dv != D and (values_are_keys or nkv == 0):
        raise KernelError("values of another size than the keys need a v projection")
    Ds = int(k_pages.shape[-1]) if k_pages is not None else max(D, Dv)
    if Ds < max(D, Dv):
        raise KernelError(f"pages with rows of {Ds} cannot hold heads of {D} and {Dv}")
    width = (nq + nkv) * D + (0 if values_are_keys else nkv * Dv)
    if qkv.shape[-1] != width:
        raise KernelError(f"the projection has {qkv.shape[-1]} columns, expected {nq} + {nkv} heads of "
                          f"{D}" + ("" if values_are_keys else f" and {nkv} of {Dv}") + f" = {width}")
    w_is_f32 = int(dt == torch.float32)      # without norm weights: whatever the entry point takes
    for w, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if w is not None:
            _need(w, nm, ndim=1)
            if w.shape[0] != D:
                raise KernelError(f"{nm} has {w.shape[0]} elements for head_dim {D}")
            w_is_f32 = int(w.dtype == torch.float32)
    if q_w is not None and k_w is not None and q_w.dtype != k_w.dtype:
        raise KernelError("q and k norm weights must have one dtype")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] * 2 != rot_dim:
            raise KernelError("inv_freq must hold rot_dim / 2 entries")
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(token_seq, "token_seq", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    q = torch.empty((T, nq, Ds), dtype=dt, device=qkv.device)
    kv_out = torch.empty((T, 2 * nkv, Ds), dtype=dt, device=qkv.device) if want_kv_out else None
    a = _QkPrepareArgs()
    a.qkv, a.q_w, a.k_w, a.inv_freq = (None if parts is not None else qkv.data_ptr()), _ptr(q_w), \
        _ptr(k_w), _ptr(inv_freq)
    if parts is not None:
        a.qkv_parts, a.n_parts, a.part_stride = parts.data_ptr(), parts.shape[0], parts.stride(0)
    a.token_seq, a.token_pos, a.slots = token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr()
    a.q_out, a.kv_out = q.data_ptr(), _ptr(kv_out)
    a.eps, a.n_tokens, a.nq, a.nkv, a.D, a.rot_dim = float(eps), T, nq, nkv, D, int(rot_dim)
    a.v_from_k = int(values_are_keys)
    a.interleaved = int(bool(interleaved) and inv_freq is not None)
    a.Dv, a.Ds = Dv, Ds
    if q_temp:
        a.q_temp_coef, a.q_temp_every = float(q_temp[0]), int(q_temp[1])
    if k_pages is not None:
        _need(k_pages, "k pages", dt, 4)
        _need(v_pages, "v pages", dt, 4)
        _need(block_table, "block table", torch.int32, 2)
        if tuple(k_pages.shape[1:]) != (nkv, page, Ds) or v_pages.shape != k_pages.shape:
            raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, {nkv}, {page}, {Ds}]")
        a.block_table, a.k_pages, a.v_pages = block_table.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr()
        a.max_pages, a.page = block_table.shape[1], page
    sfx = _suffix(dt)
    f = _fn("qk_prepare", f"gb_qk_prepare_{sfx}", "pip")
    _check(f(ctypes.addressof(a), w_is_f32, _stream()), "qk_prepare")
    return q, kv_out


@_profiled("kv_write", lambda out, kv, *a, **k: (2 * _nbytes(kv), 0))
def kv_write(kv: torch.Tensor, nkv: int, D: int, *, token_seq, token_pos, slots, block_table,
             k_pages, v_pages, page: int) -> None:
    _need(kv, "kv rows", ndim=3)
    if tuple(kv.shape[1:]) != (2 * nkv, D):
        raise KernelError(f"kv rows are {tuple(kv.shape)}, expected [T, {2 * nkv}, {D}]")
    _need(k_pages, "k pages", kv.dtype, 4)
    _need(v_pages, "v pages", kv.dtype, 4)
    _need(block_table, "block table", torch.int32, 2)
    sfx = _suffix(kv.dtype)
    _check(_fn("qk_prepare", f"gb_kv_write_{sfx}", "pppppppiiiiip")(
        kv.data_ptr(), token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr(),
        block_table.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), kv.shape[0], nkv, D,
        block_table.shape[1], page, _stream()), "kv_write")


# ---------------------------------------------------------------- attention
def _attn_common(q, k_pages, v_pages, block_table, token_seq, token_pos, slots, page):
    _need(q, "q", ndim=3)
    T, nq, D = q.shape
    _need(k_pages, "k pages", q.dtype, 4)
    _need(v_pages, "v pages", q.dtype, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    if nq % nkv:
        raise KernelError(f"{nq} query heads cannot share {nkv} kv heads")
    _need(block_table, "block table", torch.int32, 2)
    _need(token_seq, "token_seq", torch.int32, 1)
    _need(token_pos, "token_pos", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    return T, nq, nkv, D


def _check_sinks(sinks, nq: int) -> None:
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != nq:
            raise KernelError(f"{sinks.shape[0]} sinks for {nq} query heads")


@_profiled("attn_generic", lambda out, q, *a, **k: (_nbytes(q, out), 0))
def attn_generic(q, k_pages, v_pages, block_table, *, token_seq, token_pos, slots, page: int,
                 scale: float, window: Optional[int] = None, softcap: Optional[float] = None,
                 sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    T, nq, nkv, D = _attn_common(q, k_pages, v_pages, block_table, token_seq, token_pos, slots, page)
    _check_sinks(sinks, nq)
    out = torch.empty_like(q)
    sfx = _suffix(q.dtype)
    _check(_fn("attn_generic", f"gb_attn_generic_{sfx}", "ppppippppiiiiififpip")(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr(),
        out.data_ptr(), T, nq, nkv, D, page, float(scale), int(window or 0), float(softcap or 0.0),
        _ptr(sinks), int(keep_first or 0), _stream()), "attn_generic")
    return out


# ---------------------------------------------------------------- matrix products
@_profiled("gemm_f32", _cost_gemm)
def gemm_f32(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a [M, K] . w [N, K]^T in true 32-bit on the CUDA cores."""
    _need(a, "activations", torch.float32, 2)
    _need(w, "weight", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _check(_fn("gemm_f32", "gb_gemm_nt_f32", "pppiiiiiip")(
        a.data_ptr(), w.data_ptr(), c.data_ptr(), M, N, K, K, K, N, _stream()), "gemm_f32")
    return c


# ---------------------------------------------------------------- elementwise
@_profiled("silu_mul", _cost_io)
def silu_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """silu(gate) * up.  ``interleave`` 0: gate in the first half of the columns,
    up in the second; g > 0: groups of g gate columns followed by their g up columns."""
    _need(gate_up, "gate|up", ndim=2)
    T, two_i = gate_up.shape
    if two_i % 2 or (interleave and two_i % (2 * interleave)):
        raise KernelError("gate|up must have an even number of columns (of whole groups)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    sfx = _suffix(gate_up.dtype)
    _check(_fn("elementwise", f"gb_silu_mul_{sfx}", "ppiiip")(
        gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, int(interleave), _stream()), "silu_mul")
    return out


@_profiled("gelu_tanh_mul", _cost_io)
def gelu_tanh_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """gelu_tanh(gate) * up, gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)));
    the layout of ``gate_up`` is that of ``silu_mul``."""
    _need(gate_up, "gate|up", ndim=2)
    T, two_i = gate_up.shape
    if two_i % 2 or (interleave and two_i % (2 * interleave)):
        raise KernelError("gate|up must have an even number of columns (of whole groups)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", f"gb_gelu_tanh_mul_{_suffix(gate_up.dtype)}", "ppiiip")(
        gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, int(interleave), _stream()), "gelu_tanh_mul")
    return out


GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu": 2}


@_profiled("relu_mul", _cost_io)
def relu_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """max(gate, 0) * up; the layout of ``gate_up`` is that of ``silu_mul``."""
    _need(gate_up, "gate|up", ndim=2)
    T, two_i = gate_up.shape
    if two_i % 2 or (interleave and two_i % (2 * interleave)):
        raise KernelError("gate|up must have an even number of columns (of whole groups)")
    out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", f"gb_relu_mul_{_suffix(gate_up.dtype)}", "ppiiip")(
        gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, int(interleave), _stream()), "relu_mul")
    return out


@_profiled("bias_gate_mul", _cost_io)
def bias_gate_mul(gate_up: torch.Tensor, bias: torch.Tensor, activation: str, dtype: torch.dtype,
                  interleave: int = 0) -> torch.Tensor:
    """act(gate + bias_g) * (up + bias_u) on the 32-bit sums ``gate_up`` [T, 2 I] of a fused
    gate|up product, rounded once to ``dtype``; ``bias`` [2 I] 32-bit in the layout of
    ``gate_up`` (``interleave`` as in ``silu_mul``); ``activation`` silu, gelu_tanh or relu."""
    _need(gate_up, "gate|up sums", torch.float32, 2)
    _need(bias, "gate|up bias", torch.float32, 1)
    T, two_i = gate_up.shape
    if two_i % 2 or (interleave and two_i % (2 * interleave)) or bias.shape[0] != two_i:
        raise KernelError("gate|up must have an even number of columns (of whole groups) and a bias for each")
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"activation '{activation}': one of {list(GATE_ACTIVATIONS)}")
    out = torch.empty((T, two_i // 2), dtype=dtype, device=gate_up.device)
    _check(_fn("elementwise", f"gb_bias_gate_mul_{_suffix(dtype)}", "pppiiiip")(
        gate_up.data_ptr(), bias.data_ptr(), out.data_ptr(), T, two_i // 2, int(interleave),
        GATE_ACTIVATIONS[activation], _stream()), "bias_gate_mul")
    return out


@_profiled("add_bias", lambda out, x, bias: (2 * _nbytes(x), 0))
def add_bias_(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[..., :] += bias in place on contiguous 32-bit rows."""
    _need(x, "rows", torch.float32)
    _need(bias, "bias", torch.float32, 1)
    if x.shape[-1] != bias.shape[0] or not x.is_contiguous():
        raise KernelError(f"rows of {x.shape[-1]} (contiguous) and a bias of {bias.shape[0]} do not fit")
    _check(_fn("elementwise", "gb_add_bias_f32", "pplip")(
        x.data_ptr(), bias.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], _stream()), "add_bias")
    return x


@_profiled("relu_squared", _cost_io)
def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, squared in 32-bit."""
    _need(x, "tensor")
    out = torch.empty_like(x)
    _check(_fn("elementwise", f"gb_relu_squared_{_suffix(x.dtype)}", "pplp")(
        x.data_ptr(), out.data_ptr(), x.numel(), _stream()), "relu_squared")
    return out


@_profiled("scale_softcap", lambda out, x, *a: (2 * _nbytes(x), 0))
def scale_softcap_(x: torch.Tensor, scale: float, cap: Optional[float]) -> torch.Tensor:
    """x <- cap * tanh(x * scale / cap) in place on 32-bit values (no cap: x * scale)."""
    _need(x, "tensor", torch.float32)
    _check(_fn("elementwise", "gb_scale_softcap_f32", "plffp")(
        x.data_ptr(), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_softcap")
    return x


@_profiled("cast", lambda out, x, dtype: ((0, 0) if out is x else (_nbytes(x, out), 0)))
def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need(x, "tensor")
    if x.dtype == dtype:
        return x
    pair = {(torch.float32, torch.bfloat16): "gb_cast_f32_to_bf16",
            (torch.bfloat16, torch.float32): "gb_cast_bf16_to_f32"}.get((x.dtype, dtype))
    if pair is None:
        raise KernelError(f"no conversion kernel from {x.dtype} to {dtype}")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(_fn("elementwise", pair, "pplp")(x.data_ptr(), out.data_ptr(), x.numel(), _stream()),
           "cast")
    return out


@_profiled("library_mm", _cost_gemm)
def library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """x [M, K] . w [N, K]^T by the library's matrix product (cuBLAS through
    torch.mm): the prompt products for which the reference calls a library too
    (src/cublas.rs:287-307).  It is here so that the profile sees it."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


SKINNY_MAX_ROWS = 64


class _SkinnyArgs(ctypes.Structure):
    _fields_ = [("x", _P), ("W", _P), ("y", _P), ("scratch", _P), ("counters", _P), ("M", _I),
                ("N", _I), ("K", _I)]


class _Workspace:
    """Scratch of the kernels that split a sum over blocks, one per device:
    32-bit partial tiles and arrival counters.  The counters are zero between
    launches (the kernels leave them so).  Launches that share it must be ordered
    on one stream, which every step of this library is."""

    def __init__(self):
        self.scratch = None
        self.counters = None
        self._kept = []     # outgrown buffers stay alive: captured graphs still point at them

    def get(self, device, n_floats: int, n_counters: int):
        if self.scratch is None or self.scratch.numel() < n_floats:
            self._kept.append(self.scratch)
            self.scratch = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device)
        if self.counters is None or self.counters.numel() < n_counters:
            self._kept.append(self.counters)
            self.counters = torch.zeros(max(n_counters, 1 << 16), dtype=torch.int32, device=device)
        return self.scratch, self.counters


_WORKSPACES = {}
_SKINNY_PLANS = {}


def skinny_plan(M: int, N: int, K: int, out_f32: bool, silu: bool):
    """(blocks, scratch floats, counters) of the decode product for this shape:
    as many blocks as the GPU holds at once, each streaming an equal share of the
    weights; it depends on N, K and M's bucket (<= 8, 16, 32, 64) only."""
    bucket = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    key = (bucket, N, K, bool(out_f32), bool(silu), torch.cuda.current_device())
    plan = _SKINNY_PLANS.get(key)
    if plan is None:
        out = (c_int * 3)()
        _check(_fn("gemm_skinny_bf16", "gb_gemm_skinny_plan", "iiiiip")(
            bucket, N, K, int(out_f32), int(silu), ctypes.addressof(out)), "gemm_skinny_plan", 0)
        plan = _SKINNY_PLANS[key] = (out[0], out[1], out[2])
    return plan


@_profiled("gemm_skinny_bf16", _cost_gemm)
def gemm_skinny_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                     silu_mul: bool = False) -> torch.Tensor:
    """x [M <= 64, K] . w [N, K]^T, bf16 in, 32-bit accumulate; the decode-time
    linear.  With ``silu_mul`` the rows of ``w`` are gate and up rows interleaved
    in groups of 8 and the result is silu(gate) * up, [M, N / 2]."""
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if M > SKINNY_MAX_ROWS:
        raise KernelError(f"gemm_skinny_bf16 takes at most {SKINNY_MAX_ROWS} rows, got {M}")
    if K % 8:
        raise KernelError(f"gemm_skinny_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    if silu_mul and N % 16:
        raise KernelError(f"the interleaved gate|up product needs N to be a multiple of 16, got {N}")
    y = torch.empty((M, N // 2 if silu_mul else N), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    with torch.cuda.device(x.device):
        _blocks, n_floats, n_counters = skinny_plan(M, N, K, out_dtype == torch.float32, silu_mul)
        ws = _WORKSPACES.setdefault(x.device.index or 0, _Workspace())
        scratch, counters = ws.get(x.device, n_floats, n_counters)
        a = _SkinnyArgs()
        a.x, a.W, a.y = x.data_ptr(), w.data_ptr(), y.data_ptr()
        a.scratch, a.counters = scratch.data_ptr(), counters.data_ptr()
        a.M, a.N, a.K = M, N, K
        _check(_fn("gemm_skinny_bf16", "gb_gemm_skinny_bf16", "piip")(
            ctypes.addressof(a), int(out_dtype == torch.float32), int(silu_mul), _stream()),
            "gemm_skinny_bf16")
    return y


# ---------------------------------------------------------------- tcgen05 matrix product
class _TcArgs(ctypes.Structure):
    _fields_ = [("out", _P), ("scratch", _P), ("counters", _P), ("error", _P), ("rowsA", _I),
                ("rowsB", _I), ("K", _I), ("ld", _I), ("transpose_out", _I), ("out_f32", _I),
                ("silu", _I), ("dep_b", _I), ("stamps", _P), ("split_k", _I), ("bias", _P)]


_GATE_CODES = {"silu": 1, "gelu_tanh": 3, "relu": 5}     # the products' codes of a gate|up epilogue


def _gate_code(gate_act: str, bias, silu_mul: bool, n_fused: int):
    """The epilogue's code and the bias it adds first (32-bit, one entry per fused row)."""
    if gate_act not in _GATE_CODES:
        raise KernelError(f"gate activation '{gate_act}': one of {sorted(_GATE_CODES)}")
    if bias is not None:
        if not silu_mul:
            raise KernelError("a bias goes with the gate|up epilogue")
        _need(bias, "gate|up bias", torch.float32, 1)
        if bias.shape[0] != n_fused:
            raise KernelError(f"the gate|up bias has {bias.shape[0]} entries for {n_fused} fused rows")
    return _GATE_CODES[gate_act]


_TC_PLANS = {}
_TC_ERRORS = {}
_TC_ERROR_NAMES = {111: "a role of the tcgen05 attention kernel waited 2 s on a barrier",
                   101: "the MMA warp waited 2 s for a stage that never arrived",
                   102: "the TMA producer waited 2 s for a stage that was never released",
                   103: "the epilogue waited 2 s for an accumulator that was never finished",
                   104: "the MMA warp waited 2 s for an accumulator that was never drained",
                   121: "the pair product's MMA lane waited 2 s for a stage that never arrived",
                   122: "the pair product's producer waited 2 s for a stage that was never released",
                   123: "the pair product's epilogue waited 2 s for an accumulator that was never finished",
                   124: "the pair product's MMA lane waited 2 s for an accumulator that was never drained"}


def _tc_error_flag(device) -> torch.Tensor:
    i = torch.device(device).index or 0
    if i not in _TC_ERRORS:
        _TC_ERRORS[i] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_ERRORS[i]


def check_kernel_errors() -> None:
    """Reads the flags that kernels with bounded waits set when a wait expires
    (this synchronises with the device); raises if any is set."""
    for i, flag in _TC_ERRORS.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            raise KernelError(f"tensor-memory kernel on cuda:{i}: {_TC_ERROR_NAMES.get(code, code)}")


def tc_wait_selftest(device, limit_us: int = 1000) -> int:
    """Runs the give-up path of the tensor-memory kernels by itself: one block
    whose first role waits ``limit_us`` on a barrier nobody arrives at, records its
    code in the device's error flag and raises the block's abort flag, which ends
    the second role's (long) wait.  Nothing is in flight and nothing else waits.
    Returns how many roles left (2); ``check_kernel_errors`` then raises."""
    dev = torch.device(device)
    left = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _check(_fn("gemm_tc", "gb_tc_wait_selftest", "plpp")(
            _tc_error_flag(dev).data_ptr(), int(limit_us) * 1000, left.data_ptr(), _stream()),
            "tc_wait_selftest")
    return int(left.item())


@_profiled("gemm_tc_bf16", _cost_gemm)
def gemm_tc_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                 swap: Optional[bool] = None, silu_mul: bool = False,
                 stamps: Optional[torch.Tensor] = None, split_out: bool = False,
                 relu_squared: bool = False, gate_act: str = "silu",
                 bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] . w [N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in
    tensor memory).  ``swap``: put the weight rows on the 128-row side of the MMA
    and the activation rows on the narrow side (the layout for few rows); by
    default chosen when M <= 64.  ``silu_mul`` (with swap): the rows of ``w`` are
    gate and up rows interleaved in groups of 8 and the result is
    silu(gate) * up, [M, N / 2].  ``split_out`` (with swap): when the product has
    too few tiles to fill the GPU, K is cut S ways and the S 32-bit partial
    products are returned as [S, M, N] for the consumer to add (its norm or q/k
    preparation does so in the kernel it runs anyway); otherwise the result is the
    ordinary [M, N].  ``relu_squared``: every output becomes max(y, 0)^2, squared in
    32-bit before the rounding (not with ``silu_mul`` or ``split_out``).  ``gate_act``
    (with ``silu_mul``): "silu", "gelu_tanh" or "relu", the activation the gate passes
    through; ``bias`` (with ``silu_mul``) [N] 32-bit in the order of ``w``'s rows: added to
    the 32-bit sums of gate and up before the activation."""
    gate_code = _gate_code(gate_act, bias, silu_mul, w.shape[0])
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if K % 8:
        raise KernelError(f"gemm_tc_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    swap = (M <= 64) if swap is None else bool(swap)
    if silu_mul and (not swap or N % 16):
        raise KernelError("the interleaved gate|up epilogue needs the swapped layout and N % 16 == 0")
    if relu_squared and (silu_mul or split_out):
        raise KernelError("the squared relu goes with neither the gate|up epilogue nor partial sums")
    n_out = N // 2 if silu_mul else N
    y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    A, B = (w, x) if swap else (x, w)
    with torch.cuda.device(x.device):
        key = (A.shape[0], B.shape[0], K, torch.cuda.current_device())
        plan = _TC_PLANS.get(key)
        if plan is None:
            out = (c_int * 5)()
            _check(_fn("gemm_tc", "gb_gemm_tc_plan", "iiip")(
                A.shape[0], B.shape[0], K, ctypes.addressof(out)), "gemm_tc_plan", 0)
            plan = _TC_PLANS[key] = (out[0], out[1], out[2], out[3], out[4])
        split = plan[4] if (split_out and swap and not silu_mul) else 0
        if split:
            y = torch.empty((split, M, N), dtype=torch.float32, device=x.device)
        ws = _WORKSPACES.setdefault(x.device.index or 0, _Workspace())
        scratch, counters = ws.get(x.device, plan[2], plan[3])
        a = _TcArgs()
        a.out, a.scratch, a.counters = y.data_ptr(), scratch.data_ptr(), counters.data_ptr()
        a.error = _tc_error_flag(x.device).data_ptr()
        a.rowsA, a.rowsB, a.K, a.ld = A.shape[0], B.shape[0], K, n_out
        a.transpose_out, a.out_f32 = int(swap), int(out_dtype == torch.float32 or bool(split))
        a.split_k = split
        a.silu = 2 if relu_squared else (gate_code if silu_mul else 0)
        a.bias = _ptr(bias)
        a.dep_b = int(swap)                             # the activations are another kernel's output
        a.stamps = _ptr(stamps)     # int64 [blocks, 8]: phase times of every block, for tuning
        _check(_fn("gemm_tc", "gb_gemm_tc_bf16", "pppp")(
            A.data_ptr(), B.data_ptr(), ctypes.addressof(a), _stream()), "gemm_tc_bf16",
            detail=f" {N}x{K}" + ((" " + gate_act) if silu_mul else "") + (" relu2" if relu_squared else "") +
            (f" split {split}" if split else ""))
    return y


class _Tc2Args(ctypes.Structure):
    _fields_ = [("out", _P), ("error", _P), ("M", _I), ("N", _I), ("K", _I), ("ld", _I),
                ("out_f32", _I), ("silu", _I), ("bn", _I), ("bias", _P)]


_TC_ERROR_NAMES.update({121: "the pair product's MMA lane waited 2 s for a stage that never arrived",
                        122: "the pair product's loads waited 2 s for a stage that was never released",
                        123: "the pair product's epilogue waited 2 s for an accumulator",
                        124: "the pair product's MMA lane waited 2 s for an accumulator to be drained"})


def gemm_tc2_takes(n_out: int, out_dtype) -> bool:
    """Whether the pair product can store rows of ``n_out`` columns (16 bytes at a time)."""
    return (n_out * (4 if out_dtype == torch.float32 else 2)) % 16 == 0


def gemm_tc2_pays(M: int, N: int, device, fused_silu: bool) -> bool:
    """Whether the pair product is at least as fast as the library's for this shape.
    It is for the gate|up product with its fused SiLU when the rounds of tiles it runs
    are mostly full: the useful share M N / (whole rounds x pairs x 256 x 256) is at
    least 3/4.  Measured (us, pair / library product plus SiLU kernel; N 19,456, K 2,560):
    384 rows (share 0.51) 52 / 39, 512 (0.69) 53 / 51, 768 (0.77) 68 / 69, 1,024 (0.82)
    84 / 85, 2,048 (0.91) 149 / 162; N 51,200, K 5,120: 128 rows (0.45) 109 / 106, 256
    (0.90) 115 / 133, 384 (0.68) 193 / 165, 2,048 (0.98) 722 / 821.  A product without an
    epilogue to fuse never pays: 6,144 x 2,560 at 2,048 rows 47.0 / 46.2, 10,240 x 5,120
    172.7 / 157.2, and the library is ahead at every smaller row count."""
    if not fused_silu:
        return False
    pairs = max(1, _sm_count(device) // 2)
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    whole_rounds = (tiles + pairs - 1) // pairs
    return 4 * M * N >= 3 * whole_rounds * pairs * 256 * 256


@_profiled("gemm_tc2_bf16", _cost_gemm)
def gemm_tc2_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.bfloat16,
                  silu_mul: bool = False, tile_cols: int = 0,
                  relu_squared: bool = False, gate_act: str = "silu",
                  bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] . w [N, K]^T for many rows on pairs of SMs (tcgen05.mma.cta_group::2,
    tiles of 256 rows and ``tile_cols`` columns: a multiple of 16 up to 256, by
    default chosen by the kernel's launcher for the shape).  ``silu_mul``: the rows of ``w`` are gate and up rows
    interleaved in groups of 8 and the result is silu(gate) * up, [M, N / 2].
    ``relu_squared`` (instead): every output becomes max(y, 0)^2, squared in 32-bit.
    ``gate_act`` (with ``silu_mul``): "silu", "gelu_tanh" or "relu"; ``bias`` (with
    ``silu_mul``) [N] 32-bit in the order of ``w``'s rows, added to the sums before the gate."""
    gate_code = _gate_code(gate_act, bias, silu_mul, w.shape[0])
    _need(x, "activations", torch.bfloat16, 2)
    _need(w, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)} for activations of width {K}")
    if relu_squared and silu_mul:
        raise KernelError("one epilogue at a time")
    if K % 8:
        raise KernelError(f"gemm_tc2_bf16 needs an inner size that is a multiple of 8, got {K}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"output must be bfloat16 or float32, not {out_dtype}")
    if silu_mul and (N % 16 or out_dtype != torch.bfloat16):
        raise KernelError("the interleaved gate|up epilogue needs N % 16 == 0 and a bfloat16 output")
    n_out = N // 2 if silu_mul else N
    if (n_out * (4 if out_dtype == torch.float32 else 2)) % 16:
        raise KernelError(f"gemm_tc2_bf16 stores 16 bytes at a time: {n_out} output columns do not allow it")
    y = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    if M == 0:
        return y
    a = _Tc2Args()
    a.out, a.error = y.data_ptr(), _tc_error_flag(x.device).data_ptr()
    a.M, a.N, a.K, a.ld = M, N, K, n_out
    a.out_f32, a.bn = int(out_dtype == torch.float32), int(tile_cols)
    a.silu = 2 if relu_squared else (gate_code if silu_mul else 0)
    a.bias = _ptr(bias)
    with torch.cuda.device(x.device):
        _check(_fn("gemm_tc2", "gb_gemm_tc2_bf16", "pppp")(
            x.data_ptr(), w.data_ptr(), ctypes.addressof(a), _stream()), "gemm_tc2_bf16")
    return y


# ---------------------------------------------------------------- fast bf16 attention
class _PrefillArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("k_pages", _P), ("v_pages", _P), ("block_table", _P), ("cu_q", _P),
                ("slots", _P), ("kv_len", _P), ("out", _P), ("n_seqs", _I), ("nq", _I),
                ("nkv", _I), ("max_pages", _I), ("window", _I), ("n_qblocks", _I),
                ("scale_log2", _F), ("sinks", _P), ("cap_log2", _F), ("cap_inv", _F),
                ("keep_first", _I)]


class _DecodeArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("k_pages", _P), ("v_pages", _P), ("block_table", _P), ("slots", _P),
                ("kv_len", _P), ("out", _P), ("part_o", _P), ("part_ml", _P), ("n_seqs", _I),
                ("nq", _I), ("nkv", _I), ("max_pages", _I), ("page", _I), ("window", _I),
                ("n_splits", _I), ("scale_log2", _F), ("sinks", _P), ("cap_log2", _F),
                ("cap_inv", _F), ("keep_first", _I)]


def _set_cap_and_sinks(a, scale: float, softcap: Optional[float], sinks, nq: int) -> None:
    """Fills the fields that every tensor-core attention kernel's arguments end with: the
    sinks and the score cap C as (C log2 e, scale / C), zeros for none."""
    _check_sinks(sinks, nq)
    a.sinks = _ptr(sinks)
    a.cap_log2 = float(softcap) * _LOG2E if softcap else 0.0
    a.cap_inv = float(scale) / float(softcap) if softcap else 0.0


_LOG2E = 1.4426950408889634
PREFILL_ROWS = 64          # query rows per block of the prefill kernel
PREFILL_ATTENTION = "tc"      # "tc": tcgen05 where the shape allows; "mma": the mma.sync kernel


def fast_attention_modules(D: int, nq: int, nkv: int, page: int = 64) -> Tuple[str, ...]:
    """The tensor-core attention sources that heads of this shape can reach (a model
    compiles what it needs and no more)."""
    mods: Tuple[str, ...] = ()
    if fast_attention_takes(D, nq, nkv, page):
        mods += ("attn_prefill_bf16", "attn_decode_bf16")
        if attn_prefill_tc_takes(D, nq, nkv, page):
            mods += ("attn_prefill_tc",)
        if attn_decode_tma_takes(D, nq, nkv, page):
            mods += ("attn_decode_tma",)
    return mods
_SM_COUNT = {}


def _sm_count(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SM_COUNT:
        _SM_COUNT[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SM_COUNT[i]


def fast_attention_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    """Shapes the tensor-core kernels accept; others go to the plain kernel."""
    return D % 16 == 0 and 16 <= D <= 128 and page == 64 and nq % nkv == 0 and nq // nkv <= 16


def _q_blocks(q_lens, n_qblocks, rows: int, T: int, n_seqs: int) -> int:
    """Blocks of ``rows`` query rows: counted from the host's copy of the
    sequences' row counts, or taken as given (an upper bound; the kernels find each
    block's sequence on the device and blocks beyond the real count do nothing)."""
    if q_lens:
        if sum(q_lens) != T or len(q_lens) != n_seqs:
            raise KernelError("q_lens do not describe the step's rows")
        return sum((n + rows - 1) // rows for n in q_lens)
    if n_qblocks is None:
        return T // rows + n_seqs
    return int(n_qblocks)


@_profiled("attn_prefill_bf16", _cost_attention)
def attn_prefill_bf16(q, k_pages, v_pages, block_table, *, cu_q, slots, kv_len, q_lens=(),
                      page: int, scale: float, window: Optional[int] = None,
                      n_qblocks: Optional[int] = None, softcap: Optional[float] = None,
                      sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Causal attention of whole prompts (or their continuation) on the tensor
    cores.  ``keep_first``: with a window, a sequence's first keys that stay visible behind it.  The grid is sized from ``q_lens``, the host's copy of the sequences'
    row counts, or, without them, from ``n_qblocks`` (an upper bound of the
    64-row blocks; by default the most the rows and sequences can make)."""
    T, nq, D = q.shape
    _need(q, "q", torch.bfloat16, 3)
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (cu_q, "cu_q"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    n_seqs = slots.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or kv_len.shape[0] != n_seqs:
        raise KernelError("cu_q, slots and kv_len do not describe one list of sequences")
    out = torch.empty_like(q)
    a = _PrefillArgs()
    a.q, a.k_pages, a.v_pages, a.block_table = q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr()
    a.cu_q, a.slots, a.kv_len, a.out = cu_q.data_ptr(), slots.data_ptr(), kv_len.data_ptr(), out.data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = n_seqs, nq, nkv, block_table.shape[1]
    a.window = int(window or 0)
    a.n_qblocks = _q_blocks(q_lens, n_qblocks, PREFILL_ROWS, T, n_seqs)
    a.scale_log2 = float(scale) * _LOG2E
    a.keep_first = int(keep_first or 0)
    _set_cap_and_sinks(a, scale, softcap, sinks, nq)
    _check(_fn("attn_prefill_bf16", "gb_attn_prefill_bf16", "piip")(
        ctypes.addressof(a), D, page, _stream()), "attn_prefill_bf16")
    return out


class _AttnTcArgs(ctypes.Structure):
    _fields_ = [("block_table", _P), ("cu_q", _P), ("slots", _P), ("kv_len", _P), ("out", _P),
                ("error", _P), ("n_seqs", _I), ("nq", _I), ("nkv", _I), ("max_pages", _I),
                ("window", _I), ("n_qblocks", _I), ("scale_log2", _F), ("sinks", _P),
                ("cap_log2", _F), ("cap_inv", _F), ("keep_first", _I)]


PREFILL_TC_ROWS = 0        # query rows per block of the tcgen05 prefill kernel: 128, 256 or 0 = by size


def prefill_tc_rows(blocks_of_256: int, nq: int, device) -> int:
    """256 rows a block (two query blocks that share their key tiles, one block
    an SM) unless that leaves most SMs without a block; then 128 (half-size
    blocks, two an SM).  Measured on 32 heads of 128: 512 tokens 21.8 us with 128
    rows against 25.7 us with 256; from 1,024 tokens on 256 rows are faster."""
    if PREFILL_TC_ROWS:
        return PREFILL_TC_ROWS
    return 256 if 5 * blocks_of_256 * nq >= 3 * _sm_count(device) else 128


def attn_prefill_tc_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    return D in (64, 128) and page == 64 and nq % nkv == 0


@_profiled("attn_prefill_tc", _cost_attention)
def attn_prefill_tc(q, k_pages, v_pages, block_table, *, cu_q, slots, kv_len, q_lens=(),
                    page: int, scale: float, window: Optional[int] = None,
                    rows_per_block: int = 0, n_qblocks: Optional[int] = None,
                    softcap: Optional[float] = None,
                    sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Causal attention of whole prompts (or their continuation) with both
    products on the tcgen05 tensor cores.  Pages must hold finite values in the
    rows beyond a sequence's length (the cache zero-fills its pages).  The grid is
    sized from ``q_lens`` (the host's copy of the row counts) or, without them,
    from ``n_qblocks``, an upper bound of the blocks of ``rows_per_block`` rows."""
    _need(q, "q", torch.bfloat16, 3)
    T, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (cu_q, "cu_q"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    n_seqs = slots.shape[0]
    if cu_q.shape[0] != n_seqs + 1 or kv_len.shape[0] != n_seqs:
        raise KernelError("cu_q, slots and kv_len do not describe one list of sequences")
    out = torch.empty_like(q)
    a = _AttnTcArgs()
    a.block_table, a.cu_q, a.slots, a.kv_len = (block_table.data_ptr(), cu_q.data_ptr(),
                                                slots.data_ptr(), kv_len.data_ptr())
    a.out, a.error = out.data_ptr(), _tc_error_flag(q.device).data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = n_seqs, nq, nkv, block_table.shape[1]
    a.window = int(window or 0)
    rows = int(rows_per_block) if rows_per_block else \
        prefill_tc_rows(_q_blocks(q_lens, None, 256, T, n_seqs), nq, q.device)
    a.n_qblocks = _q_blocks(q_lens, n_qblocks, rows, T, n_seqs)
    a.scale_log2 = float(scale) * _LOG2E
    a.keep_first = int(keep_first or 0)
    _set_cap_and_sinks(a, scale, softcap, sinks, nq)
    _check(_fn("attn_prefill_tc", "gb_attn_prefill_tc", "ppppiliiip")(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), ctypes.addressof(a), T,
        k_pages.shape[0], D, page, rows, _stream()), "attn_prefill_tc")
    return out


DECODE_SPLITS_OVERRIDE: Optional[int] = None      # for experiments


def decode_splits(n_seqs: int, nkv: int, max_kv_len: int, device) -> int:
    """How many ways the keys of a sequence are split.  Blocks run in waves of
    three per SM; with S splits a block streams 1/S of a sequence's 32-key tiles
    plus a fixed cost of about three tiles (query load, merge, partial store), so
    the step costs waves(S) * (tiles / S + 3).  The smallest S within 3 % of the
    cheapest is taken, with at least 256 keys a split."""
    if DECODE_SPLITS_OVERRIDE:
        return DECODE_SPLITS_OVERRIDE
    slots = 3 * _sm_count(device)
    pairs = max(1, n_seqs * nkv)
    tiles = max(1, (max_kv_len + 31) // 32)
    most = max(1, min(64, (max_kv_len + 255) // 256))
    cost = {s: ((pairs * s + slots - 1) // slots) * (tiles / s + 3.0) for s in range(1, most + 1)}
    best = min(cost.values())
    return min(s for s, c in cost.items() if c <= 1.03 * best)


def _keys_visited(max_kv_len: int, window: Optional[int], page: int, keep_first: int = 0) -> int:
    """The most keys a decode row reads: its sequence's, or with a window the
    window's and the kept first ones, rounded out to the tiles that hold them."""
    if not window:
        return max_kv_len
    kept = (int(keep_first or 0) + page - 1) // page * page
    return min(max_kv_len, window + page - 1 + kept)


@_profiled("attn_decode_bf16", _cost_attention)
def attn_decode_bf16(q, k_pages, v_pages, block_table, *, slots, kv_len, page: int, scale: float,
                     max_kv_len: int, window: Optional[int] = None,
                     n_splits: Optional[int] = None, softcap: Optional[float] = None,
                     sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys (split-K).
    ``keep_first``: with a window, a sequence's first keys that stay visible behind it."""
    _need(q, "q", torch.bfloat16, 3)
    B, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    if slots.shape[0] != B or kv_len.shape[0] != B:
        raise KernelError("one slot and one length per query row are needed")
    # (a window bounds the keys a row visits, whatever its sequence's length)
    ns = int(n_splits) if n_splits else decode_splits(
        B, nkv, _keys_visited(max_kv_len, window, page, keep_first), q.device)
    out = torch.empty_like(q)
    part_o = part_ml = None
    if ns > 1:
        # scratch of the split: 32-bit partials of every (sequence, head, split)
        ws = _WORKSPACES.setdefault(q.device.index or 0, _Workspace())
        scratch, _counters = ws.get(q.device, B * nq * ns * (D + 2), 1)
        part_o = scratch[:B * nq * ns * D]
        part_ml = scratch[B * nq * ns * D:B * nq * ns * (D + 2)]
    a = _DecodeArgs()
    a.q, a.k_pages, a.v_pages, a.block_table = q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr()
    a.slots, a.kv_len, a.out = slots.data_ptr(), kv_len.data_ptr(), out.data_ptr()
    a.part_o, a.part_ml = _ptr(part_o), _ptr(part_ml)
    a.n_seqs, a.nq, a.nkv, a.max_pages, a.page = B, nq, nkv, block_table.shape[1], page
    a.window, a.n_splits, a.scale_log2 = int(window or 0), ns, float(scale) * _LOG2E
    a.keep_first = int(keep_first or 0)
    _set_cap_and_sinks(a, scale, softcap, sinks, nq)
    _check(_fn("attn_decode_bf16", "gb_attn_decode_bf16", "pip")(
        ctypes.addressof(a), D, _stream()), "attn_decode_bf16", 2 if ns > 1 else 1)
    return out


class _DecodeTmaArgs(ctypes.Structure):
    _fields_ = [("q", _P), ("block_table", _P), ("slots", _P), ("kv_len", _P), ("out", _P),
                ("part_o", _P), ("part_ml", _P), ("counters", _P), ("error", _P), ("n_seqs", _I),
                ("nq", _I), ("nkv", _I), ("max_pages", _I), ("window", _I), ("n_splits", _I),
                ("scale_log2", _F), ("stamps", _P), ("sinks", _P), ("cap_log2", _F),
                ("cap_inv", _F), ("keep_first", _I)]


DECODE_TMA_STAMPS: Optional[torch.Tensor] = None      # int64 [blocks, 12] for tuning, or None
_TC_ERROR_NAMES[131] = "a role of the decode attention kernel waited 2 s on a barrier"
# Which decode attention runs: "auto" takes the TMA kernel where the shape allows and the
# step has at least DECODE_TMA_PAIRS (sequence, kv head) pairs, with two stages (three blocks
# an SM) below DECODE_TMA_DEEP_PAIRS pairs and three stages (two blocks an SM) from there
# on, and the cp.async kernel for fewer pairs; "tma" and "mma" force one.  Measured inside
# the decode step at 32 query and 8 kv heads of 128 with 2,100 keys a sequence (ms a step,
# cp.async / TMA with two stages / with three): 1 sequence 2.38 / 2.50 / 2.48, 4 sequences
# 2.57 / 2.57 / 2.55, 8 sequences 2.74 / 2.72 / 2.78, 16 sequences 3.19 / 3.10 / 3.18, 32
# sequences 4.35 / 4.27 / 4.04, 64 sequences 6.41 / 6.22 / 5.99.  Timed by itself, one call
# after the other, the TMA kernel is the faster or the equal at every size (16.8 against
# 17.9 us at 8 sequences, 86 against 97 at 64); inside a step of very few sequences, where
# a short kernel comes before it, its longer start (descriptor fetch, barrier set-up, the
# hand-over from the loading lane) shows.
DECODE_ATTENTION = "auto"
DECODE_TMA_PAIRS = 64
DECODE_TMA_DEEP_PAIRS = 256
DECODE_TMA_STAGES = 0         # tiles of a block in shared memory (0: by the number of pairs)
_ATTN_COUNTERS = {}


def attn_decode_tma_takes(D: int, nq: int, nkv: int, page: int) -> bool:
    return D in (64, 128) and page == 64 and nq % nkv == 0 and nq // nkv <= 16


def decode_tma_splits(n_seqs: int, nkv: int, max_kv_len: int, device, per_sm: int = 2) -> int:
    """How many ways the keys of a sequence are split for the TMA kernel: blocks
    run in waves of ``per_sm`` per SM; with S splits a block streams 1/S of a
    sequence's 64-key tiles plus a fixed cost of about six tiles (descriptor and
    block-table loads before the first copy, the partial store and the combining
    at the end), so the step costs waves(S) * (tiles / S + 6).  The smallest S
    within 3 % of the cheapest is taken, with at least 256 keys a split.
    Measured (us, 32 query and 8 kv heads of 128): 8 sequences of 2,049 keys 16.8
    with the 4 splits this picks (19.8 with 2, 21.7 with 8); 64 sequences 86.3 with
    1 (99.4 with 2); one sequence 9.1 with 8 or 9 (17.7 with 2)."""
    if DECODE_SPLITS_OVERRIDE:
        return DECODE_SPLITS_OVERRIDE
    places = per_sm * _sm_count(device)
    pairs = max(1, n_seqs * nkv)
    tiles = max(1, (max_kv_len + 63) // 64)
    most = max(1, min(64, (max_kv_len + 255) // 256))
    cost = {s: ((pairs * s + places - 1) // places) * (-(-tiles // s) + 6.0) for s in range(1, most + 1)}
    best = min(cost.values())
    return min(s for s, c in cost.items() if c <= 1.03 * best)


@_profiled("attn_decode_tma", _cost_attention)
def attn_decode_tma(q, k_pages, v_pages, block_table, *, slots, kv_len, page: int, scale: float,
                    max_kv_len: int, window: Optional[int] = None,
                    n_splits: Optional[int] = None, stages: int = 0,
                    softcap: Optional[float] = None,
                    sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys, the tiles
    brought in by TMA and the splits combined by the block that finishes last (one
    launch).  Heads of 64 or 128, pages of 64 tokens."""
    _need(q, "q", torch.bfloat16, 3)
    B, nq, D = q.shape
    _need(k_pages, "k pages", torch.bfloat16, 4)
    _need(v_pages, "v pages", torch.bfloat16, 4)
    nkv = k_pages.shape[1]
    if tuple(k_pages.shape[1:]) != (nkv, page, D) or v_pages.shape != k_pages.shape:
        raise KernelError(f"pages are {tuple(k_pages.shape)}, expected [*, nkv, {page}, {D}]")
    for t, nm in ((block_table, "block table"), (slots, "slots"), (kv_len, "kv_len")):
        _need(t, nm, torch.int32)
    if slots.shape[0] != B or kv_len.shape[0] != B:
        raise KernelError("one slot and one length per query row are needed")
    stages = int(stages or DECODE_TMA_STAGES) or (2 if B * nkv < DECODE_TMA_DEEP_PAIRS else 3)
    per_sm = {2: 3, 3: 2, 4: 1}.get(stages, 2) if D == 128 else 3
    ns = int(n_splits) if n_splits else decode_tma_splits(
        B, nkv, _keys_visited(max_kv_len, window, page, keep_first), q.device, per_sm)
    out = torch.empty_like(q)
    a = _DecodeTmaArgs()
    if ns > 1:
        ws = _WORKSPACES.setdefault(q.device.index or 0, _Workspace())
        scratch, _c = ws.get(q.device, B * nq * ns * (D + 2), 1)
        dev = q.device.index or 0
        counters = _ATTN_COUNTERS.get(dev)
        if counters is None or counters.numel() < B * nkv:
            counters = _ATTN_COUNTERS[dev] = torch.zeros(max(B * nkv, 1 << 16), dtype=torch.int32,
                                                         device=q.device)
        a.part_o, a.part_ml = scratch.data_ptr(), scratch[B * nq * ns * D:].data_ptr()
        a.counters = counters.data_ptr()
    a.q, a.block_table, a.slots = q.data_ptr(), block_table.data_ptr(), slots.data_ptr()
    a.kv_len, a.out, a.error = kv_len.data_ptr(), out.data_ptr(), _tc_error_flag(q.device).data_ptr()
    a.n_seqs, a.nq, a.nkv, a.max_pages = B, nq, nkv, block_table.shape[1]
    a.window, a.n_splits, a.scale_log2 = int(window or 0), ns, float(scale) * _LOG2E
    a.stamps = _ptr(DECODE_TMA_STAMPS)
    a.keep_first = int(keep_first or 0)
    _set_cap_and_sinks(a, scale, softcap, sinks, nq)
    with torch.cuda.device(q.device):
        _check(_fn("attn_decode_tma", "gb_attn_decode_tma", "pplpiiip")(
            k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], ctypes.addressof(a), D, page,
            stages, _stream()), "attn_decode_tma")
    return out


# ---------------------------------------------------------------- attention dispatch
def attention(q, k_pages, v_pages, block_table, *, step, page: int, scale: float,
              window: Optional[int] = None, softcap: Optional[float] = None,
              sinks: Optional[torch.Tensor] = None, keep_first: int = 0) -> torch.Tensor:
    """Attention of the step's queries over their sequences' cached keys.
    32-bit tensors take the plain 32-bit kernel; bfloat16 takes the tensor-core
    kernels where they accept the shape and the plain kernel elsewhere.
    ``softcap`` c: scores become c * tanh(score / c); ``sinks`` [nq] float32: one
    more term exp(sinks[h]) in the denominator of query head h; ``keep_first`` F: with a
    window, key j < F stays visible to every later query (at its own position)."""
    _T, nq, D = q.shape
    keep_first = int(keep_first or 0) if window else 0
    extra = dict(softcap=softcap, sinks=sinks, keep_first=keep_first)
    if q.dtype == torch.bfloat16 and fast_attention_takes(D, nq, k_pages.shape[1], page):
        nkv = k_pages.shape[1]
        if step.decode and attn_decode_tma_takes(D, nq, nkv, page) and (
                DECODE_ATTENTION == "tma" or
                (DECODE_ATTENTION == "auto" and step.n_seqs * nkv >= DECODE_TMA_PAIRS)):
            return attn_decode_tma(q, k_pages, v_pages, block_table, slots=step.slots,
                                   kv_len=step.kv_len, page=page, scale=scale,
                                   max_kv_len=step.max_kv_len, window=window, **extra)
        if step.decode:
            return attn_decode_bf16(q, k_pages, v_pages, block_table, slots=step.slots,
                                    kv_len=step.kv_len, page=page, scale=scale,
                                    max_kv_len=step.max_kv_len, window=window, **extra)
        # the grid comes from the host's copy of the lengths; a captured step has
        # none, and the kernels then take the most blocks its rows can make
        if PREFILL_ATTENTION == "tc" and attn_prefill_tc_takes(D, nq, k_pages.shape[1], page):
            return attn_prefill_tc(q, k_pages, v_pages, block_table, cu_q=step.cu_q,
                                   slots=step.slots, kv_len=step.kv_len, q_lens=step.q_lens,
                                   page=page, scale=scale, window=window, **extra)
        return attn_prefill_bf16(q, k_pages, v_pages, block_table, cu_q=step.cu_q,
                                 slots=step.slots, kv_len=step.kv_len, q_lens=step.q_lens,
                                 page=page, scale=scale, window=window, **extra)
    return attn_generic(q, k_pages, v_pages, block_table, token_seq=step.token_seq,
                        token_pos=step.token_pos, slots=step.slots, page=page, scale=scale,
                        window=window, softcap=softcap, sinks=sinks, keep_first=keep_first)


# ---------------------------------------------------------------- gated delta rule
class _DeltaArgs(ctypes.Structure):
    _fields_ = [("proj", _P), ("conv_w", _P), ("a_log", _P), ("dt_bias", _P), ("norm_w", _P),
                ("token_seq", _P), ("cu_q", _P), ("slots", _P), ("state", _P), ("state_stride", _L),
                ("prep", _P), ("o", _P), ("y", _P), ("n_tokens", _I), ("n_seqs", _I), ("H", _I),
                ("G", _I), ("dk", _I), ("dv", _I), ("taps", _I), ("unit_eps", _F), ("norm_eps", _F),
                ("prep_stride", _I), ("few_rows", _I)]


def delta_state_floats(H: int, G: int, dk: int, dv: int, taps: int) -> int:
    """Floats of one sequence's state: the convolutions' tail, then the heads' matrices."""
    return (taps - 1) * (2 * G * dk + H * dv) + H * dv * dk


def _cost_delta(out, proj, state, *a, H, G, dk, dv, taps, **k):
    T = proj.shape[0]
    n_seqs = k["slots"].shape[0]
    return (_nbytes(proj, out) + 2 * T * (2 * G * dk + 2 * H * dv + 2 * H) * 4 +
            2 * n_seqs * H * dk * dv * 4, 6.0 * T * H * dk * dv)


@_profiled("delta_forward", _cost_delta)
def delta_forward(proj: torch.Tensor, state: torch.Tensor, conv_w: torch.Tensor,
                  a_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor, *, H: int,
                  G: int, dk: int, dv: int, taps: int, unit_eps: float, norm_eps: float,
                  token_seq, cu_q, slots, dtype: torch.dtype, max_rows: Optional[int] = None) -> torch.Tensor:
    """The gated delta rule on the rows of a step.  ``proj`` [T, C] 32-bit: the columns
    q [G dk] | k [G dk] | v [H dv] | gate [H dv] | b [H] | a [H] of the mixer's one
    projection; ``state`` [slots, delta_state_floats] 32-bit, updated in place for the
    sequences whose slot is not negative; ``conv_w`` [2 G dk + H dv, taps].  Returns
    y [T, H dv] in ``dtype``: every head's read-out, normalised over dv, times ``norm_w``
    and silu(gate).  ``max_rows``: the most rows any sequence of the step brings, when the
    host knows it (a decode step: 1); steps of at most four rows a sequence take one launch less."""
    _need(proj, "projection", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    Cc = 2 * G * dk + H * dv
    T = proj.shape[0]
    if proj.shape[1] != Cc + H * dv + 2 * H:
        raise KernelError(f"the projection has {proj.shape[1]} columns, expected {Cc + H * dv + 2 * H}")
    if state.shape[1] != delta_state_floats(H, G, dk, dv, taps):
        raise KernelError(f"a sequence's state has {state.shape[1]} floats, expected "
                          f"{delta_state_floats(H, G, dk, dv, taps)}")
    for t, nm, shape in ((conv_w, "convolution weights", (Cc, taps)), (a_log, "A_log", (H,)),
                         (dt_bias, "dt_bias", (H,)), (norm_w, "norm weight", (dv,))):
        _need(t, nm, torch.float32)
        if tuple(t.shape) != shape:
            raise KernelError(f"{nm} are {tuple(t.shape)}, expected {shape}")
    for t, nm in ((token_seq, "token_seq"), (cu_q, "cu_q"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    n_seqs = slots.shape[0]
    if token_seq.shape[0] != T or cu_q.shape[0] != n_seqs + 1:
        raise KernelError("token_seq, cu_q and slots do not describe the step's rows")
    # rows that start on 16 bytes; behind a row's own values, room for the scalars of the
    # group of four rows that it opens
    prep_stride = (Cc + 2 * H + 3) // 4 * 4 + 48 * H
    prep = torch.empty((T, prep_stride), dtype=torch.float32, device=proj.device)
    o = torch.empty((T, H, dv), dtype=torch.float32, device=proj.device)
    y = torch.empty((T, H * dv), dtype=dtype, device=proj.device)
    a = _DeltaArgs()
    a.proj, a.conv_w, a.a_log, a.dt_bias, a.norm_w = (proj.data_ptr(), conv_w.data_ptr(),
                                                      a_log.data_ptr(), dt_bias.data_ptr(), norm_w.data_ptr())
    a.token_seq, a.cu_q, a.slots = token_seq.data_ptr(), cu_q.data_ptr(), slots.data_ptr()
    a.state, a.state_stride = state.data_ptr(), state.stride(0)
    a.prep, a.o, a.y = prep.data_ptr(), o.data_ptr(), y.data_ptr()
    a.n_tokens, a.n_seqs, a.H, a.G, a.dk, a.dv, a.taps = T, n_seqs, H, G, dk, dv, taps
    a.unit_eps, a.norm_eps, a.prep_stride = float(unit_eps), float(norm_eps), prep_stride
    a.few_rows = 0 if max_rows is None or not 0 < max_rows <= 4 else (2 if max_rows == 1 else 1)
    _check(_fn("delta", f"gb_delta_forward_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "delta_forward", 3 if a.few_rows else 4)
    return y


# ---------------------------------------------------------------- groups of heads
@_profiled("head_group", _cost_io)
def head_group(x: torch.Tensor, first: int, count: int) -> torch.Tensor:
    """Heads first .. first + count of x [T, H, D] as a tensor of their own (a copy by the
    library's kernel; it is here so that the profile and the launch log see it)."""
    _need(x, "rows per head", ndim=3)
    out = x[:, first:first + count].contiguous()
    _check(0, "head_group")
    return out


@_profiled("join_heads", _cost_io)
def join_heads(parts) -> torch.Tensor:
    """Tensors [T, h_i, D] side by side along the heads (the library's kernel, logged)."""
    out = torch.cat(list(parts), dim=1)
    _check(0, "join_heads")
    return out


# ---------------------------------------------------------------- retention
class _RetentionArgs(ctypes.Structure):
    _fields_ = [("proj", _P), ("decay", _P), ("inv_freq", _P), ("token_pos", _P), ("cu_q", _P),
                ("slots", _P), ("state", _P), ("state_stride", _L), ("qk", _P), ("o", _P), ("chunk_state", _P),
                ("y", _P),
                ("n_tokens", _I), ("n_seqs", _I), ("H", _I), ("dk", _I), ("dv", _I), ("rot_dim", _I),
                ("k_scale", _F), ("norm_eps", _F), ("max_rows", _I)]


RETENTION_CHUNK = 64         # rows of a chunk of the kernel's chunked form
RETENTION_CHUNK_MIN = 256    # a sequence of this many rows in a step: the step goes chunk by chunk


def _cost_retention(out, proj, state, *a, H, dk, dv, **k):
    T = proj.shape[0]
    n_seqs = k["slots"].shape[0]
    return (_nbytes(proj, out) + T * (4 * H * dk + 2 * H * dv) * 4 + 2 * n_seqs * H * dk * dv * 4,
            4.0 * T * H * dk * dv)


@_profiled("retention_forward", _cost_retention)
def retention_forward(proj: torch.Tensor, state: torch.Tensor, decay: torch.Tensor,
                      inv_freq: Optional[torch.Tensor], *, H: int, dk: int, dv: int, rot_dim: int,
                      k_scale: float, norm_eps: float, token_pos, cu_q, slots,
                      dtype: torch.dtype, max_rows: Optional[int] = None) -> torch.Tensor:
    """Retention on the rows of a step.  ``proj`` [T, 2 H dk + 2 H dv] 32-bit: the columns
    q | k | v | gate of the mixer's one projection; ``state`` [slots, H dk dv] 32-bit, updated
    in place for the sequences whose slot is not negative; ``decay`` [H] 32-bit; ``inv_freq``
    [rot_dim / 2] the rotation's frequencies (element i of a head goes with element
    i + rot_dim / 2).  Returns y [T, H dv] in ``dtype``: every head's read-out S^T q,
    divided by its root mean square over dv (``norm_eps`` under the root), times silu(gate).
    ``max_rows``: the most rows any sequence of the step brings, when the caller knows it (a
    step of one row a sequence is one kernel; a step with a sequence of many rows runs all
    chunks of 64 rows side by side and joins them through the states at their starts)."""
    _need(proj, "projection", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    _need(decay, "decay", torch.float32, 1)
    T = proj.shape[0]
    if proj.shape[1] != 2 * H * dk + 2 * H * dv:
        raise KernelError(f"the projection has {proj.shape[1]} columns, expected {2 * H * dk + 2 * H * dv}")
    if state.shape[1] != H * dk * dv or decay.shape[0] != H:
        raise KernelError(f"a sequence's state has {state.shape[1]} floats, expected {H * dk * dv}, "
                          f"and there is a decay for each of {H} heads")
    if rot_dim:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] * 2 != rot_dim or rot_dim > dk:
            raise KernelError("inv_freq must hold rot_dim / 2 entries, rot_dim at most the head's size")
    for t, nm in ((token_pos, "token_pos"), (cu_q, "cu_q"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    n_seqs = slots.shape[0]
    if token_pos.shape[0] != T or cu_q.shape[0] != n_seqs + 1:
        raise KernelError("token_pos, cu_q and slots do not describe the step's rows")
    dev = proj.device
    qk = torch.empty((T, 2, H, dk), dtype=torch.float32, device=dev)
    o = torch.empty((T, H, dv), dtype=torch.float32, device=dev)
    y = torch.empty((T, H * dv), dtype=dtype, device=dev)
    a = _RetentionArgs()
    a.proj, a.decay, a.inv_freq = proj.data_ptr(), decay.data_ptr(), _ptr(inv_freq)
    a.token_pos, a.cu_q, a.slots = token_pos.data_ptr(), cu_q.data_ptr(), slots.data_ptr()
    a.state, a.state_stride = state.data_ptr(), state.stride(0)
    a.qk, a.o, a.y = qk.data_ptr(), o.data_ptr(), y.data_ptr()
    a.n_tokens, a.n_seqs, a.H, a.dk, a.dv, a.rot_dim = T, n_seqs, H, dk, dv, int(rot_dim)
    a.k_scale, a.norm_eps = float(k_scale), float(norm_eps)
    a.max_rows = int(max_rows) if max_rows else 0
    chunked = a.max_rows >= RETENTION_CHUNK_MIN
    if chunked:   # one matrix a head for every chunk of every sequence
        chunk_state = torch.empty((T // RETENTION_CHUNK + n_seqs, H * dk * dv), dtype=torch.float32, device=dev)
        a.chunk_state = chunk_state.data_ptr()
    _check(_fn("retention", f"gb_retention_forward_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "retention_forward", 1 if a.max_rows == 1 and dv <= 256 else 5 if chunked else 3)
    return y


# ---------------------------------------------------------------- gated linear recurrence
class _RglruArgs(ctypes.Structure):
    _fields_ = [("proj", _P), ("bias", _P), ("conv_w", _P), ("conv_b", _P), ("wa_t", _P), ("ba", _P),
                ("wi_t", _P), ("bi", _P), ("lam", _P), ("token_seq", _P), ("cu_q", _P), ("slots", _P),
                ("state", _P), ("state_stride", _L), ("u", _P), ("ab", _P), ("out", _P),
                ("chunks", _P), ("start", _P),
                ("n_tokens", _I), ("n_seqs", _I), ("C", _I), ("blocks", _I), ("taps", _I),
                ("factor", _F), ("max_rows", _I)]

RGLRU_CHUNK = 64        # rows of a chunk of the recurrence's scan (RG_CHUNK of the kernel)
RGLRU_FEW_ROWS = 32     # up to this many rows the gates come from one kernel (RG_FEW of the kernel)


def _cost_rglru(out, proj, state, *a, **k):
    T, C2 = proj.shape
    C = C2 // 2
    bw = C // k["blocks"]
    return (_nbytes(proj, out) + T * C * 4 * 6, 4.0 * T * C * bw)


@_profiled("rglru_forward", _cost_rglru)
def rglru_forward(proj: torch.Tensor, state: torch.Tensor, bias: torch.Tensor, conv_w: torch.Tensor,
                  conv_b: torch.Tensor, wa_t: torch.Tensor, ba: torch.Tensor, wi_t: torch.Tensor,
                  bi: torch.Tensor, lam: torch.Tensor, *, blocks: int, taps: int, factor: float,
                  token_seq, cu_q, slots, dtype: torch.dtype, max_rows: Optional[int] = None) -> torch.Tensor:
    """The gated linear recurrence on the rows of a step.  ``proj`` [T, 2 C] 32-bit: the
    columns y | x of the mixer's projection, ``bias`` [2 C] their biases; ``conv_w`` [C, taps]
    and ``conv_b`` [C] the convolution over x; ``wa_t``, ``wi_t`` [blocks, C / blocks, C / blocks]
    the gates' matrices per part of the channels, each stored [in, out], with biases ``ba``,
    ``bi`` [C]; ``lam`` [C]; the decay is exp(-factor * r * softplus(lam)).  ``state``
    [slots, taps * C] 32-bit: the last taps - 1 inputs of the convolution, then S; updated
    in place for sequences whose slot is not negative.  ``max_rows``: the most rows any sequence
    of the step brings, when the caller knows it (sequences of more than a chunk's rows are
    scanned chunk by chunk).  Returns S * gelu_tanh(y) [T, C] in ``dtype``."""
    _need(proj, "projection", torch.float32, 2)
    _need(state, "state", torch.float32, 2)
    T, C2 = proj.shape
    C = C2 // 2
    if C2 % 2 or C % blocks:
        raise KernelError(f"{C2} columns are not two branches of {blocks} equal parts")
    bw = C // blocks
    for t, nm, shape in ((bias, "projection biases", (2 * C,)), (conv_w, "convolution weights", (C, taps)),
                         (conv_b, "convolution bias", (C,)), (wa_t, "decay gate", (blocks, bw, bw)),
                         (wi_t, "input gate", (blocks, bw, bw)), (ba, "decay gate bias", (C,)),
                         (bi, "input gate bias", (C,)), (lam, "lam", (C,))):
        _need(t, nm, torch.float32)
        if tuple(t.shape) != shape:
            raise KernelError(f"{nm} are {tuple(t.shape)}, expected {shape}")
    if state.shape[1] != taps * C:
        raise KernelError(f"a sequence's state has {state.shape[1]} floats, expected {taps * C}")
    for t, nm in ((token_seq, "token_seq"), (cu_q, "cu_q"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    n_seqs = slots.shape[0]
    if token_seq.shape[0] != T or cu_q.shape[0] != n_seqs + 1:
        raise KernelError("token_seq, cu_q and slots do not describe the step's rows")
    dev = proj.device
    u = torch.empty((T, C), dtype=torch.float32, device=dev)
    ab = torch.empty((T, 2, C), dtype=torch.float32, device=dev)
    out = torch.empty((T, C), dtype=dtype, device=dev)
    chunks = torch.empty((T // RGLRU_CHUNK + n_seqs, 2, C), dtype=torch.float32, device=dev)
    start = torch.empty((n_seqs, C), dtype=torch.float32, device=dev)
    a = _RglruArgs()
    a.proj, a.bias, a.conv_w, a.conv_b = proj.data_ptr(), bias.data_ptr(), conv_w.data_ptr(), conv_b.data_ptr()
    a.wa_t, a.ba, a.wi_t, a.bi, a.lam = wa_t.data_ptr(), ba.data_ptr(), wi_t.data_ptr(), bi.data_ptr(), lam.data_ptr()
    a.token_seq, a.cu_q, a.slots = token_seq.data_ptr(), cu_q.data_ptr(), slots.data_ptr()
    a.state, a.state_stride = state.data_ptr(), state.stride(0)
    a.u, a.ab, a.out = u.data_ptr(), ab.data_ptr(), out.data_ptr()
    a.chunks, a.start = chunks.data_ptr(), start.data_ptr()
    a.n_tokens, a.n_seqs, a.C, a.blocks, a.taps, a.factor = T, n_seqs, C, int(blocks), int(taps), float(factor)
    a.max_rows = int(max_rows) if max_rows else 0
    most = min(a.max_rows, T) if a.max_rows else T
    kernels = (1 if T <= RGLRU_FEW_ROWS else 2) + (1 if most <= RGLRU_CHUNK else 2)
    _check(_fn("rglru", f"gb_rglru_forward_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "rglru_forward", kernels)
    return out


# ---------------------------------------------------------------- latent attention
class _LatentArgs(ctypes.Structure):
    _fields_ = [("proj", _P), ("norm_w", _P), ("inv_freq", _P), ("token_seq", _P), ("token_pos", _P),
                ("slots", _P), ("block_table", _P), ("pages", _P), ("q_plain", _P), ("q_full", _P),
                ("n_tokens", _I), ("H", _I), ("dn", _I), ("dr", _I), ("R", _I), ("dv", _I), ("Ds", _I),
                ("max_pages", _I), ("page", _I), ("eps", _F)]


@_profiled("latent_prepare", lambda out, proj, *a, **k: (_nbytes(proj) + _nbytes(*out), 0))
def latent_prepare(proj: torch.Tensor, norm_w: torch.Tensor, inv_freq: Optional[torch.Tensor], *,
                   H: int, dn: int, dr: int, R: int, dv: int, eps: float, token_seq, token_pos,
                   slots, block_table, pages, page: int, dtype: torch.dtype):
    """What latent attention does between its projection and its attention.  ``proj``
    [T, H (dn + dr) + R + dr + H dv] 32-bit: queries (per head dn plain, dr rotated
    elements) | the down projection | the gate.  Stores the row [c | k_rot | zeros] of
    every token whose slot is not negative in ``pages`` [n, 1, page, Ds] (c: the first R
    numbers of the down projection, RMS-normalised times ``norm_w``; k_rot: its last dr,
    rotated: element 2i with element 2i + 1 by position * inv_freq[i]).  Returns
    (q_plain [T, H, dn], q_full [T, H, Ds]) in ``dtype``; of q_full the columns from R on
    are written (the rotated query part, then zeros), the first R are left to the caller."""
    _need(proj, "projection", torch.float32, 2)
    _need(norm_w, "latent norm weight", torch.float32, 1)
    T = proj.shape[0]
    _need(pages, "latent pages", dtype, 4)
    Ds = pages.shape[-1]
    if proj.shape[1] != H * (dn + dr) + R + dr + H * dv or norm_w.shape[0] != R:
        raise KernelError(f"the projection has {proj.shape[1]} columns, expected "
                          f"{H * (dn + dr) + R + dr + H * dv}; the norm weight {norm_w.shape[0]} for {R}")
    if tuple(pages.shape[1:]) != (1, page, Ds) or Ds < R + dr:
        raise KernelError(f"pages are {tuple(pages.shape)}, expected [*, 1, {page}, >= {R + dr}]")
    if dr:
        _need(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] * 2 != dr:
            raise KernelError("inv_freq must hold dr / 2 entries")
    for t, nm in ((token_seq, "token_seq"), (token_pos, "token_pos"), (slots, "slots")):
        _need(t, nm, torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    q_plain = torch.empty((T, H, dn), dtype=dtype, device=proj.device)
    q_full = torch.empty((T, H, Ds), dtype=dtype, device=proj.device)
    a = _LatentArgs()
    a.proj, a.norm_w, a.inv_freq = proj.data_ptr(), norm_w.data_ptr(), _ptr(inv_freq)
    a.token_seq, a.token_pos, a.slots = token_seq.data_ptr(), token_pos.data_ptr(), slots.data_ptr()
    a.block_table, a.pages = block_table.data_ptr(), pages.data_ptr()
    a.q_plain, a.q_full = q_plain.data_ptr(), q_full.data_ptr()
    a.n_tokens, a.H, a.dn, a.dr, a.R, a.dv, a.Ds = T, H, dn, dr, R, dv, Ds
    a.max_pages, a.page, a.eps = block_table.shape[1], int(page), float(eps)
    _check(_fn("latent", f"gb_latent_prepare_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "latent_prepare")
    return q_plain, q_full


class _HeadsMmArgs(ctypes.Structure):
    _fields_ = [("x", _P), ("w", _P), ("out", _P), ("g", _P), ("T", _I), ("H", _I), ("K", _I),
                ("N", _I), ("ldx", _I), ("ldo", _I), ("ldg", _I)]


@_profiled("heads_mm", lambda out, x, w, *a, **k: (_nbytes(x, w) + x.shape[0] * w.shape[0] * w.shape[1] * x.element_size(),
                                                    2.0 * x.shape[0] * w.shape[0] * w.shape[1] * w.shape[2]))
def heads_mm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *,
             gate: Optional[torch.Tensor] = None, gate_col: int = 0) -> torch.Tensor:
    """A product per head: out[t, h, :N] = w[h] x[t, h, :K] with x [T, H, ldx >= K], w [H, N, K]
    and out [T, H, ldo >= N] (made [T, H, N] when not given; columns from N on are left as
    they are).  ``gate`` [T, ld] 32-bit: the result is multiplied, on its 32-bit sums, by
    sigmoid(gate[t, gate_col + h N + n])."""
    _need(x, "rows per head", ndim=3)
    _need(w, "weights per head", x.dtype, 3)
    T, H, ldx = x.shape
    Hw, N, K = w.shape
    if Hw != H or K > ldx or not x.is_contiguous() or not w.is_contiguous():
        raise KernelError(f"rows {tuple(x.shape)} and weights {tuple(w.shape)} do not fit together")
    if out is None:
        out = torch.empty((T, H, N), dtype=x.dtype, device=x.device)
    _need(out, "result", x.dtype, 3)
    if out.shape[0] != T or out.shape[1] != H or out.shape[2] < N or not out.is_contiguous():
        raise KernelError(f"the result is {tuple(out.shape)}, expected [{T}, {H}, >= {N}]")
    a = _HeadsMmArgs()
    a.x, a.w, a.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    a.T, a.H, a.K, a.N, a.ldx, a.ldo = T, H, K, N, ldx, out.shape[2]
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        if gate.shape[0] != T or gate_col + H * N > gate.shape[1] or gate.stride(1) != 1:
            raise KernelError("the gate's rows do not hold the heads' columns")
        a.g, a.ldg = gate.data_ptr() + 4 * int(gate_col), gate.stride(0)
    _check(_fn("latent", f"gb_heads_mm_{_suffix(x.dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "heads_mm")
    return out


# ---------------------------------------------------------------- routed experts
class _MoeArgs(ctypes.Structure):
    _fields_ = [("x", _P), ("router_w", _P), ("correction", _P), ("w_gate", _P), ("w_up", _P),
                ("w_down", _P), ("ids", _P), ("wts", _P), ("rank", _P), ("counts", _P),
                ("offsets", _P), ("perm", _P), ("act", _P), ("out", _P), ("T", _I), ("W", _I),
                ("F", _I), ("E", _I), ("n_identity", _I), ("top", _I), ("n_groups", _I),
                ("keep_groups", _I), ("limit", _F), ("slope", _F), ("score_fn", _I),
                ("weigh_input", _I), ("up_offset", _F), ("router_bias", _P)]


_MOE_COUNTS = {}
MOE_SCORE_FNS = {"softmax": 0, "sigmoid": 1, "softmax_top": 2}     # the route kernel's codes


def _cost_moe(out, x, router_w, correction, w_gate, w_up, w_down, *, top, **k):
    T, W = x.shape
    E, F = w_gate.shape[0], w_gate.shape[1]
    used = min(E, T * top)
    return (_nbytes(x, out) + used * 3 * F * W * w_gate.element_size(), 6.0 * T * top * F * W)


@_profiled("moe_forward", _cost_moe)
def moe_forward(x: torch.Tensor, router_w: torch.Tensor, correction: Optional[torch.Tensor],
                w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, *, top: int,
                n_identity: int = 0, n_groups: int = 1, keep_groups: int = 1,
                limit: float = math.inf, slope: float = 1.0, score_fn: str = "softmax",
                weigh_input: bool = False, up_offset: float = 1.0, want_choice: bool = False,
                router_bias: Optional[torch.Tensor] = None):
    """A feed-forward of routed experts on rows x [T, W] -> 32-bit partial sums
    [top, T, W], choice j of every token in [j], already weighted; their sum is the
    feed-forward's output.  ``router_w`` [E + n_identity, W] and ``correction`` are
    32-bit; the experts' weights [E, F, W], [E, F, W], [E, W, F] have the type of x.
    The last ``n_identity`` router outputs stand for experts that return their input.
    ``score_fn`` "sigmoid" scores every output by itself instead of by the softmax,
    "softmax_top" lets the logits choose and weighs the chosen by the softmax over their
    logits alone; ``router_bias`` (32-bit) is added to the logits;
    ``correction`` may be None; ``weigh_input`` multiplies the expert's input, not its
    result, by the weight; an expert is Wd (g sigmoid(slope g) (u + up_offset)) with g
    and u clamped at ``limit``.
    With ``want_choice`` also returns (ids [T, top] int32, weights [T, top])."""
    _need(x, "activations", ndim=2)
    T, W = x.shape
    _need(router_w, "router weight", torch.float32, 2)
    if correction is not None:
        _need(correction, "score correction", torch.float32, 1)
    if score_fn not in MOE_SCORE_FNS:
        raise KernelError(f"score function '{score_fn}': one of {sorted(MOE_SCORE_FNS)}")
    if router_bias is not None:
        _need(router_bias, "router bias", torch.float32, 1)
        if router_bias.shape[0] != router_w.shape[0]:
            raise KernelError("the router's bias and its weight do not fit together")
    for t, nm in ((w_gate, "gate weights"), (w_up, "up weights"), (w_down, "down weights")):
        _need(t, nm, x.dtype, 3)
    E, F = w_gate.shape[0], w_gate.shape[1]
    n_all = E + n_identity
    if tuple(w_gate.shape) != (E, F, W) or tuple(w_up.shape) != (E, F, W) or \
            tuple(w_down.shape) != (E, W, F) or tuple(router_w.shape) != (n_all, W) or \
            (correction is not None and correction.shape[0] != n_all):
        raise KernelError("the experts' weights, the router and the correction do not fit together")
    dev = x.device
    ids = torch.empty((T, top), dtype=torch.int32, device=dev)
    wts = torch.empty((T, top), dtype=torch.float32, device=dev)
    rank = torch.empty((T, top), dtype=torch.int32, device=dev)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    perm = torch.empty((T * top,), dtype=torch.int32, device=dev)
    act = torch.empty((T * top, F), dtype=x.dtype, device=dev)
    out = torch.empty((top, T, W), dtype=torch.float32, device=dev)
    key = (dev.index or 0, E)
    counts = _MOE_COUNTS.get(key)      # zero between calls: the kernels leave it so
    if counts is None:
        counts = _MOE_COUNTS[key] = torch.zeros((E + 1,), dtype=torch.int32, device=dev)
    a = _MoeArgs()
    a.x, a.router_w, a.correction = x.data_ptr(), router_w.data_ptr(), _ptr(correction)
    a.w_gate, a.w_up, a.w_down = w_gate.data_ptr(), w_up.data_ptr(), w_down.data_ptr()
    a.ids, a.wts, a.rank, a.counts = ids.data_ptr(), wts.data_ptr(), rank.data_ptr(), counts.data_ptr()
    a.offsets, a.perm, a.act, a.out = offsets.data_ptr(), perm.data_ptr(), act.data_ptr(), out.data_ptr()
    a.T, a.W, a.F, a.E, a.n_identity, a.top = T, W, F, E, int(n_identity), int(top)
    a.n_groups, a.keep_groups, a.limit, a.slope = int(n_groups), int(keep_groups), float(limit), float(slope)
    a.score_fn, a.weigh_input, a.up_offset = MOE_SCORE_FNS[score_fn], int(weigh_input), float(up_offset)
    a.router_bias = _ptr(router_bias)
    _check(_fn("moe", f"gb_moe_forward_{_suffix(x.dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "moe_forward", 3)
    return (out, ids, wts) if want_choice else out


# ---------------------------------------------------------------- forget-gate linear attention
class _Hgrn2Args(ctypes.Structure):
    _fields_ = [("proj", _P), ("ld", _L), ("q_col", _I), ("f_col", _I), ("v_col", _I), ("f_bias", _P),
                ("lower", _P), ("norm_w", _P), ("cu_q", _P), ("slots", _P), ("state", _P),
                ("state_stride", _L), ("o", _P), ("y", _P), ("y_ld", _L), ("n_tokens", _I),
                ("n_seqs", _I), ("H", _I), ("dk", _I), ("dv", _I), ("norm_eps", _F), ("out_scale", _F),
                ("qb", _P), ("chunk_state", _P), ("chunk_decay", _P), ("max_rows", _I)]


HGRN2_CHUNK = 64          # rows of a chunk of the kernel's chunked form (HG_CHUNK)
HGRN2_CHUNK_MIN = 256     # a sequence of this many rows in a step: the step goes chunk by chunk


def _cost_hgrn2(out, proj, state, *a, H, dk, dv, **k):
    """The step's rows once, the states of its sequences read and written (an upper bound:
    padding sequences store nothing), and per row and head 2 dk dv multiply-adds for the
    state and as many for the read-out."""
    T = proj.shape[0]
    n_seqs = k["slots"].shape[0]
    return (T * (2 * H * dk + 2 * H * dv) * 4 + _nbytes(out) + 2 * n_seqs * H * dk * dv * 4,
            4.0 * T * H * dk * dv)


@_profiled("hgrn2_forward", _cost_hgrn2)
def hgrn2_forward(proj: torch.Tensor, state: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor,
                  norm_w: torch.Tensor, *, H: int, dk: int, dv: int, q_col: int, f_col: int,
                  v_col: int, norm_eps: float, cu_q, slots, dtype: torch.dtype,
                  out_scale: float = 1.0, into: Optional[torch.Tensor] = None,
                  max_rows: int = 0) -> torch.Tensor:
    """Linear attention whose forget gate decides what is written, on the 32-bit sums of a
    projection ``proj`` [T, ld] whose columns from ``q_col``, ``f_col`` (H dk each) and
    ``v_col`` (H dv) are this mixer's: q = silu(zq), f = lower + (1 - lower) sigmoid(zf +
    f_bias); per head S <- diag(f) S + (1 - f) v^T, o = S^T q; y = rmsnorm(o) * norm_w *
    out_scale in ``dtype``.  ``state`` [slots + 1, H dk dv] (32-bit) is read and updated for
    the sequences of ``cu_q`` whose slot is not negative.  ``into``: a 2-D view [T, H dv] of a
    wider row to write into (its row pitch is kept); else a new tensor.  ``max_rows``: the most
    rows a sequence brings (0: unknown, taken as all of them); from ``HGRN2_CHUNK_MIN`` on the step
    goes chunk by chunk (the same sums in another order)."""
    out = into
    if (proj is None or not proj.is_cuda or proj.dtype != torch.float32 or proj.dim() != 2
            or proj.stride(1) != 1):
        raise KernelError("projection sums must be a 32-bit [T, columns] CUDA view with unit stride")
    T, ld = proj.shape[0], proj.stride(0)
    for c, n in ((q_col, H * dk), (f_col, H * dk), (v_col, H * dv)):
        if c < 0 or c + n > proj.shape[1]:
            raise KernelError(f"columns {c}..{c + n} lie outside the projection's {proj.shape[1]}")
    _need(state, "state", torch.float32, 2)
    if state.shape[1] != H * dk * dv:
        raise KernelError(f"state rows hold {state.shape[1]} floats, expected {H * dk * dv}")
    for t, nm, n in ((f_bias, "forget bias", H * dk), (lower, "lower bound", H * dk), (norm_w, "norm weight", dv)):
        _need(t, nm, torch.float32, 1)
        if t.shape[0] != n:
            raise KernelError(f"{nm} has {t.shape[0]} elements, expected {n}")
    _need(cu_q, "cu_q", torch.int32, 1)
    _need(slots, "slots", torch.int32, 1)
    if out is None:
        out = torch.empty((T, H * dv), dtype=dtype, device=proj.device)
    elif (out.dim() != 2 or tuple(out.shape) != (T, H * dv) or out.dtype != dtype or out.stride(1) != 1
          or not out.is_cuda):
        raise KernelError("the output view must be [T, H dv] of the activation type with unit stride")
    o = torch.empty((T, H, dv), dtype=torch.float32, device=proj.device)
    a = _Hgrn2Args()
    a.proj, a.ld, a.q_col, a.f_col, a.v_col = proj.data_ptr(), ld, int(q_col), int(f_col), int(v_col)
    a.f_bias, a.lower, a.norm_w = f_bias.data_ptr(), lower.data_ptr(), norm_w.data_ptr()
    a.cu_q, a.slots, a.state, a.state_stride = cu_q.data_ptr(), slots.data_ptr(), state.data_ptr(), state.stride(0)
    a.o, a.y, a.y_ld = o.data_ptr(), out.data_ptr(), out.stride(0)
    a.n_tokens, a.n_seqs, a.H, a.dk, a.dv = T, slots.shape[0], int(H), int(dk), int(dv)
    a.norm_eps, a.out_scale = float(norm_eps), float(out_scale)
    a.max_rows = int(max_rows) if max_rows else T
    chunked = a.max_rows >= HGRN2_CHUNK_MIN
    if chunked:
        entries = T // HGRN2_CHUNK + slots.shape[0]
        qb = torch.empty((T, H, dk), dtype=torch.float32, device=proj.device)
        chunk_state = torch.empty((entries, H, dk, dv), dtype=torch.float32, device=proj.device)
        chunk_decay = torch.empty((entries, H, dk), dtype=torch.float32, device=proj.device)
        a.qb, a.chunk_state, a.chunk_decay = qb.data_ptr(), chunk_state.data_ptr(), chunk_decay.data_ptr()
    _check(_fn("hgrn2", f"gb_hgrn2_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "hgrn2_forward", 4 if chunked else 2)
    return out


# ---------------------------------------------------------------- gated sums, depth average, norm
class _GatedTerm(ctypes.Structure):
    _fields_ = [("delta", _P), ("parts", _P), ("n_parts", _I), ("part_stride", _L), ("gate", _P),
                ("gate_ld", _L), ("gate_bias", _P)]


class _GatedNormArgs(ctypes.Structure):
    _fields_ = [("res_in", _P), ("term", _GatedTerm * 2), ("hist", _P), ("hist_stride", _L),
                ("n_hist", _I), ("avg_w", _P), ("rows", _P), ("norm_w", _P), ("eps", _F),
                ("res_out", _P), ("y", _P), ("n_rows", _I), ("N", _I)]


@_profiled("gated_norm", lambda out, res_in, terms, **k: (
    _nbytes(res_in, *out, *[t for term in terms for t in term[:2]])
    + (k.get("n_hist") or 0) * (_nbytes(res_in) if res_in is not None else 0), 0))
def gated_norm(res_in: Optional[torch.Tensor], terms, *, dtype: torch.dtype,
               hist: Optional[torch.Tensor] = None, n_hist: int = 0,
               avg_w: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
               norm_w: Optional[torch.Tensor] = None, eps: float = 0.0):
    """X = res_in + sum over up to two ``terms`` (delta, gate logits, gate bias) of
    sigmoid(gate + bias) * delta (a term without gate is added as it is; delta is [T, N]
    in ``dtype`` or a stack of 32-bit partial sums [S, T, N]; the gate's logits are a 32-bit
    2-D view [T, N] whose row pitch is kept); then, with ``hist`` [n, T, N]: X is stored as
    entry ``n_hist`` and x' = sum_j avg_w[j] hist[j] over j <= n_hist, else x' = X; then
    y = rmsnorm(x') * norm_w (or x' itself without ``norm_w``) in ``dtype``.  Returns (x', y);
    x' replaces ``res_in`` in place unless ``rows`` picks rows (then nothing is stored in
    ``hist`` either).  All sums are 32-bit."""
    src = res_in
    a = _GatedNormArgs()
    if res_in is not None:
        _need(res_in, "residual", torch.float32, 2)
    if len(terms) > 2:
        raise KernelError("at most two gated terms")
    for i, (delta, gate, bias) in enumerate(terms):
        if delta is None:
            continue
        g = a.term[i]
        if delta.dim() == 3:
            _need(delta, "partial sums", torch.float32, 3)
            g.parts, g.n_parts, g.part_stride = delta.data_ptr(), delta.shape[0], delta.stride(0)
            shape = tuple(delta.shape[1:])
        else:
            _need(delta, "delta", dtype, 2)
            g.delta, shape = delta.data_ptr(), tuple(delta.shape)
        if src is None:
            src = delta[0] if delta.dim() == 3 else delta
        if shape != tuple(src.shape):
            raise KernelError(f"a term of {shape} for a stream of {tuple(src.shape)}")
        if gate is not None:
            if (gate.dtype != torch.float32 or gate.dim() != 2 or tuple(gate.shape) != shape
                    or gate.stride(1) != 1 or not gate.is_cuda):
                raise KernelError("gate logits must be a 32-bit [T, N] view with unit stride")
            g.gate, g.gate_ld = gate.data_ptr(), gate.stride(0)
            if bias is not None:
                _need(bias, "gate bias", torch.float32, 1)
                g.gate_bias = bias.data_ptr()
    if src is None:
        raise KernelError("gated_norm needs a residual or a term")
    T, N = src.shape
    if hist is not None:
        _need(hist, "earlier results", torch.float32, 3)
        _need(avg_w, "averaging weights", torch.float32, 1)
        if tuple(hist.shape[1:]) != (T, N) or not 0 <= n_hist < hist.shape[0] or avg_w.shape[0] != n_hist + 1:
            raise KernelError("the earlier results, their count and the weights do not fit together")
        a.hist, a.hist_stride, a.n_hist, a.avg_w = hist.data_ptr(), hist.stride(0), int(n_hist), avg_w.data_ptr()
    if norm_w is not None:
        _need(norm_w, "norm weight", torch.float32, 1)
        if norm_w.shape[0] != N:
            raise KernelError(f"norm weight has {norm_w.shape[0]} elements for rows of {N}")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
    n_rows = rows.shape[0] if rows is not None else T
    res_out = res_in if (rows is None and res_in is not None) else \
        torch.empty((n_rows, N), dtype=torch.float32, device=src.device)
    y = torch.empty((n_rows, N), dtype=dtype, device=src.device)
    a.res_in, a.rows, a.norm_w, a.eps = _ptr(res_in), _ptr(rows), _ptr(norm_w), float(eps)
    a.res_out, a.y, a.n_rows, a.N = res_out.data_ptr(), y.data_ptr(), n_rows, N
    _check(_fn("gated_norm", f"gb_gated_norm_{_suffix(dtype)}", "pp")(ctypes.addressof(a), _stream()),
           "gated_norm")
    return res_out, y


@_profiled("head_gate", lambda out, x, gate, *a, **k: (_nbytes(x) + out.numel() * out.element_size(), 0))
def head_gate(x: torch.Tensor, gate: Optional[torch.Tensor], v_dim: int, mult: float = 1.0,
              into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * v_dim + d] = x[t, h, d] * sigmoid(gate[t, h]) * mult for d < v_dim, with x
    [T, heads, Ds] (Ds >= v_dim), ``gate`` a 32-bit 2-D view [T, heads] of logits whose row
    pitch is kept (None: no gate), and ``into`` a 2-D view [T, heads * v_dim] of a wider row
    to write into, or None for a new tensor."""
    out = into
    _need(x, "heads", ndim=3)
    T, nq, Ds = x.shape
    if gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (T, nq) or gate.stride(1) != 1
                             or not gate.is_cuda):
        raise KernelError("gate logits must be a 32-bit [T, heads] view with unit stride")
    if out is None:
        out = torch.empty((T, nq * v_dim), dtype=x.dtype, device=x.device)
    elif tuple(out.shape) != (T, nq * v_dim) or out.dtype != x.dtype or out.stride(1) != 1 or not out.is_cuda:
        raise KernelError("the output view must be [T, heads * v_dim] of x's type with unit stride")
    _check(_fn("elementwise", f"gb_head_gate_{_suffix(x.dtype)}", "pplpliiiifp")(
        x.data_ptr(), _ptr(gate), 0 if gate is None else gate.stride(0), out.data_ptr(), out.stride(0),
        T, nq, Ds, int(v_dim), float(mult), _stream()), "head_gate")
    return out


# ---------------------------------------------------------------- sampling
@_profiled("argmax", lambda out, logits: (_nbytes(logits), 0))
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """First maximum of every row of 32-bit logits -> int32 [rows]."""
    _need(logits, "logits", torch.float32, 2)
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    scratch = torch.empty((logits.shape[0], 64), dtype=torch.float32, device=logits.device)
    _check(_fn("sample", "gb_argmax_f32", "piippp")(
        logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(), scratch.data_ptr(),
        _stream()), "argmax", 2)
    return out


@_profiled("sample", lambda out, logits, *a: (_nbytes(logits), 0))
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """One token per row from temperature / top-k / top-p sampling with the
    uniform draw ``u[row]``; a temperature <= 1e-5 means argmax."""
    _need(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    for t, nm, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                      (top_p, "top_p", torch.float32), (u, "u", torch.float32)):
        _need(t, nm, dt, 1)
        if t.shape[0] != n:
            raise KernelError(f"{nm} has {t.shape[0]} entries for {n} rows")
    out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _check(_fn("sample", "gb_sample_f32", "piipppppp")(
        logits.data_ptr(), n, logits.shape[1], temperature.data_ptr(), top_k.data_ptr(),
        top_p.data_ptr(), u.data_ptr(), out.data_ptr(), _stream()), "sample")
    return out
