"""Python face of the sm_100a kernels: argument checks, then the launch.

Every function takes torch tensors that live on the CUDA device, checks types,
shapes and contiguity on the host, and launches on torch's current stream, so
the launches can be captured into a CUDA graph with everything else.  There is
no CPU implementation and no library fallback behind these calls; a tensor on
another device is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from . import csrc

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    """The address for a ``c_void_p`` parameter (ctypes takes the integer as it is; None is NULL)."""
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle on the current device.  (Asked of torch's C layer directly: a
    launcher is called hundreds of times a step, and ``torch.cuda.current_stream()`` builds a
    Python object each time.)"""
    if _raw_stream is None or _raw_device is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(_raw_device())


def _need(t: torch.Tensor, what: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the CUDA device (it is on {t.device}); there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, not {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{what} must have {ndim} dimensions, not {t.dim()}")


def _rows_contiguous(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise KernelError(f"{what} must be 2-D with dense rows (shape {tuple(t.shape)}, strides {t.stride()})")
    return t.stride(0)


_prototyped = set()


class KernelTimes:
    """Device time of every launcher of this package by kernel class, for as long as the context
    lasts: a CUDA event before and one after each call (the launches then run one after the other
    as usual, but a kernel that would overlap the one ahead of it through programmatic dependent
    launch is still charged its whole length: the figures are shares, not a step's time; captured
    graphs hide their kernels, so the runner steps eagerly meanwhile).

        with ops.KernelTimes() as kt:
            runner.step(...)
        kt.totals()        # {"gemm_tcgen05": microseconds, ...}
    """

    active: Optional["KernelTimes"] = None

    def __init__(self):
        self.records = []          # (name, start event, end event)

    def __enter__(self):
        if KernelTimes.active is not None:
            raise KernelError("KernelTimes does not nest")
        KernelTimes.active = self
        return self

    def __exit__(self, *exc):
        KernelTimes.active = None
        torch.cuda.synchronize()
        return False

    def totals(self) -> dict:
        """Microseconds per launcher name, and the number of calls under "<name> calls"."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.records:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b) * 1e3
            out[name + " calls"] = out.get(name + " calls", 0) + 1
        return out


class _Timed:
    """A launcher that, while a ``KernelTimes`` is open, brackets its call with two events."""

    def __init__(self, fn, name: str):
        self.fn, self.name = fn, name

    def __call__(self, *args):
        kt = KernelTimes.active
        if kt is None:
            return self.fn(*args)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = self.fn(*args)
        b.record()
        kt.records.append((self.name, a, b))
        return rc


_wrapped = {}


def _fn(lib_name: str, fn_name: str, argtypes, label: Optional[str] = None):
    """The exported function, wrapped so that ``KernelTimes`` sees its launches under ``label`` (the function's
    name without its prefix when none is given: an entry that grew an argument keeps its kernel class)."""
    key = (lib_name, fn_name)
    got = _wrapped.get(key)
    if got is not None:
        return got
    lib = csrc.load(lib_name)
    fn = getattr(lib, fn_name)
    if key not in _prototyped:
        fn.argtypes = argtypes
        fn.restype = c_int
        err = getattr(lib, f"lgml_{lib_name}_last_error")
        err.restype = ctypes.c_char_p
        _prototyped.add(key)
        _wrapped[key] = _Timed(fn, label or (fn_name[len("lgml_"):] if fn_name.startswith("lgml_") else fn_name))
    return _wrapped[key]


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of this package have been called (a launcher starts one
    kernel; split-KV attention starts two).  Launches replayed by a CUDA graph are not
    counted here; the runner knows how many a graph holds."""
    return _launches


def _check(lib_name: str, rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        err = getattr(csrc.load(lib_name), f"lgml_{lib_name}_last_error")
        err.restype = ctypes.c_char_p
        raise KernelError(f"{what}: {err().decode('utf-8', 'replace')} (code {rc})")


# ----------------------------------------------------------------------------------------
# elementwise
# ----------------------------------------------------------------------------------------

def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]] as float32."""
    _need(table, "embedding table", ndim=2)
    _need(ids, "token ids", torch.int32, 1)
    _need(out, "embedding output", torch.float32, 2)
    if not table.is_contiguous() or not out.is_contiguous():
        raise KernelError("embedding table and output must be contiguous")
    n, width = out.shape
    if ids.numel() != n or table.shape[1] != width:
        raise KernelError(f"embed_rows: shapes disagree: table {tuple(table.shape)}, ids {tuple(ids.shape)}, out {tuple(out.shape)}")
    fn = _fn("elementwise", "lgml_embed_rows", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _check("elementwise", fn(_ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), n, width, table.shape[0], _ptr(status), _stream()), "embed_rows")
    return out


class Partials:
    """The float32 partial sums of a matrix product cut along K: ``data`` is
    [n_parts, rows, width]; the kernel that reads them adds the parts in order and then
    ``bias`` (per column) if there is one."""

    def __init__(self, data: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.data, self.bias = data, bias

    @property
    def shape(self):
        return self.data.shape[1:]

    def sum(self) -> torch.Tensor:
        """The product itself (for a part that does not read partial sums)."""
        y = self.data.sum(dim=0)
        return y if self.bias is None else y + self.bias


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta=None,
            rows: Optional[torch.Tensor] = None, delta_scale: float = 1.0) -> torch.Tensor:
    """out = rmsnorm(x [+ delta_scale * delta]) * weight.  With ``delta`` (a tensor, or ``Partials``) and
    no ``rows`` the sum is written back to x (the residual add); with ``rows`` output row r
    reads x[rows[r]]."""
    _need(x, "norm input", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(out, "norm output", ndim=2)
    width = x.shape[1]
    n_rows = out.shape[0]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != width or weight.numel() != width:
        raise KernelError(f"rmsnorm: shapes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is None and n_rows != x.shape[0]:
        raise KernelError("rmsnorm: without a row list the output has the input's rows")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        if rows.numel() != n_rows:
            raise KernelError("rmsnorm: one output row per listed row")
    ddt, n_parts, stride, dbias, dptr = F32, 1, 0, None, None
    if isinstance(delta, Partials):
        d = delta.data
        _need(d, "residual delta parts", torch.float32, 3)
        if tuple(d.shape[1:]) != tuple(x.shape) or not d.is_contiguous():
            raise KernelError("rmsnorm: delta parts must be [parts, rows, width] and contiguous")
        n_parts, stride, dbias, dptr = d.shape[0], d.shape[1] * d.shape[2], delta.bias, d
    elif delta is not None:
        _need(delta, "residual delta", ndim=2)
        if delta.shape != x.shape or not delta.is_contiguous():
            raise KernelError("rmsnorm: delta must have the input's shape and be contiguous")
        ddt, dptr = dtype_code(delta.dtype), delta
    fn = _fn("elementwise", "lgml_rmsnorm_scaled", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                    c_int, c_int, c_float, c_float, c_void_p], label="rmsnorm")
    _check("elementwise", fn(_ptr(x), _ptr(dptr), ddt, n_parts, stride, _ptr(dbias), _ptr(weight), _ptr(rows), _ptr(out),
                             dtype_code(out.dtype), n_rows, width, float(eps), float(delta_scale), _stream()), "rmsnorm")
    return out


def dyt_norm(x: torch.Tensor, weight: torch.Tensor, shift: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor, delta=None,
             rows: Optional[torch.Tensor] = None, pre_scale: float = 1.0) -> torch.Tensor:
    """out = tanh(alpha * pre_scale * (x [+ delta])) * weight + shift (a norm without mean or variance);
    ``alpha`` is one float32 on the device.  ``delta`` and ``rows`` as for ``rmsnorm``."""
    _need(x, "norm input", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(shift, "norm shift", torch.float32, 1)
    _need(alpha, "norm alpha", torch.float32)
    _need(out, "norm output", ndim=2)
    width = x.shape[1]
    n_rows = out.shape[0]
    if not x.is_contiguous() or not out.is_contiguous() or out.shape[1] != width or weight.numel() != width or shift.numel() != width or alpha.numel() != 1:
        raise KernelError(f"dyt_norm: shapes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is None and n_rows != x.shape[0]:
        raise KernelError("dyt_norm: without a row list the output has the input's rows")
    if rows is not None:
        _need(rows, "row list", torch.int32, 1)
        if rows.numel() != n_rows:
            raise KernelError("dyt_norm: one output row per listed row")
    ddt, n_parts, stride, dbias, dptr = F32, 1, 0, None, None
    if isinstance(delta, Partials):
        d = delta.data
        _need(d, "residual delta parts", torch.float32, 3)
        if tuple(d.shape[1:]) != tuple(x.shape) or not d.is_contiguous():
            raise KernelError("dyt_norm: delta parts must be [parts, rows, width] and contiguous")
        n_parts, stride, dbias, dptr = d.shape[0], d.shape[1] * d.shape[2], delta.bias, d
    elif delta is not None:
        _need(delta, "residual delta", ndim=2)
        if delta.shape != x.shape or not delta.is_contiguous():
            raise KernelError("dyt_norm: delta must have the input's shape and be contiguous")
        ddt, dptr = dtype_code(delta.dtype), delta
    fn = _fn("elementwise", "lgml_dyt_norm", [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_void_p])
    _check("elementwise", fn(_ptr(x), _ptr(dptr), ddt, n_parts, stride, _ptr(dbias), _ptr(weight), _ptr(shift), _ptr(alpha), float(pre_scale),
                             _ptr(rows), _ptr(out), dtype_code(out.dtype), n_rows, width, _stream()), "dyt_norm")
    return out


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, alpha: float, limit: float, paired: bool = False) -> torch.Tensor:
    """out[t, f] = g * sigmoid(alpha g) * (u + 1) with g = min(gate[t, f], limit), u = clamp(up[t, f], -limit, limit);
    gate|up laid out as for ``silu_mul``."""
    _need(gate_up, "gate|up", ndim=2)
    _need(out, "activation", gate_up.dtype, 2)
    n, two_f = gate_up.shape
    if two_f != 2 * out.shape[1] or out.shape[0] != n or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"glu_clamped: shapes disagree: gate|up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    fn = _fn("elementwise", "lgml_glu_clamped", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p])
    _check("elementwise", fn(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), n, out.shape[1], 1 if paired else 0, float(alpha), float(limit),
                             _stream()), "glu_clamped")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False) -> torch.Tensor:
    """out[t, f] = silu(gate[t, f]) * up[t, f]; gate|up are the two halves of a row, or, with
    ``paired``, neighbours (gate at 2f, up at 2f + 1)."""
    _need(gate_up, "gate|up", ndim=2)
    _need(out, "activation", gate_up.dtype, 2)
    n, two_f = gate_up.shape
    if two_f != 2 * out.shape[1] or out.shape[0] != n or not gate_up.is_contiguous() or not out.is_contiguous():
        raise KernelError(f"silu_mul: shapes disagree: gate|up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    fn = _fn("elementwise", "lgml_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check("elementwise", fn(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), n, out.shape[1], 1 if paired else 0, _stream()), "silu_mul")
    return out


def relu_sq(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = relu(x)^2 element by element (in place when ``out`` is None)."""
    _need(x, "activation input")
    out = x if out is None else out
    if out.shape != x.shape or out.dtype != x.dtype or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("relu_sq: input and output must be contiguous and alike")
    fn = _fn("elementwise", "lgml_relu_sq", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check("elementwise", fn(_ptr(x), _ptr(out), dtype_code(x.dtype), x.numel(), _stream()), "relu_sq")
    return out


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += delta, the sum in float32."""
    _need(x, "residual stream", torch.float32)
    _need(delta, "residual delta")
    if x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous():
        raise KernelError("residual_add: shapes disagree or not contiguous")
    fn = _fn("elementwise", "lgml_residual_add", [c_void_p, c_void_p, c_int, c_longlong, c_void_p])
    _check("elementwise", fn(_ptr(x), _ptr(delta), dtype_code(delta.dtype), x.numel(), _stream()), "residual_add")
    return x


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32: x *= scale, then x = cap * tanh(x / cap) when cap > 0."""
    _need(x, "tensor to scale", torch.float32)
    if not x.is_contiguous():
        raise KernelError("scale_cap: tensor must be contiguous")
    fn = _fn("elementwise", "lgml_scale_cap", [c_void_p, c_longlong, c_float, c_float, c_void_p])
    _check("elementwise", fn(_ptr(x), x.numel(), float(scale), float(cap or 0.0), _stream()), "scale_cap")
    return x


def l2_ahead(t: torch.Tensor, n_bytes: Optional[int] = None, keep: bool = True) -> None:
    """Ask L2 for the first ``n_bytes`` of ``t`` (all of it when None); returns at once."""
    if not t.is_contiguous():
        raise KernelError("l2_ahead: tensor must be contiguous")
    total = t.numel() * t.element_size()
    n = total if n_bytes is None else min(int(n_bytes), total)
    fn = _fn("elementwise", "lgml_l2_ahead", [c_void_p, c_longlong, c_int, c_void_p])
    _check("elementwise", fn(_ptr(t), n, 1 if keep else 0, _stream()), "l2_ahead")


def fill_normal(out: torch.Tensor, mean: float, sd: float, seed: int) -> torch.Tensor:
    """Seeded N(mean, sd^2) fill on the device."""
    _need(out, "tensor to fill")
    if not out.is_contiguous():
        raise KernelError("fill_normal: tensor must be contiguous")
    fn = _fn("elementwise", "lgml_fill_normal", [c_void_p, c_int, c_longlong, c_float, c_float, c_ulonglong, c_void_p])
    _check("elementwise", fn(_ptr(out), dtype_code(out.dtype), out.numel(), float(mean), float(sd), seed & 0xFFFFFFFFFFFFFFFF, _stream()), "fill_normal")
    return out


# ----------------------------------------------------------------------------------------
# matrix products
# ----------------------------------------------------------------------------------------

def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = a[M,K] . w[N,K]^T (+ bias), true float32 with a fixed summation order."""
    _need(a, "gemm input", torch.float32, 2)
    _need(w, "gemm weight", torch.float32, 2)
    _need(out, "gemm output", ndim=2)
    lda, ldw, ldc = _rows_contiguous(a, "gemm input"), _rows_contiguous(w, "gemm weight"), _rows_contiguous(out, "gemm output")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm_f32: bias length is not N")
    fn = _fn("gemm_f32", "lgml_gemm_f32", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check("gemm_f32", fn(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), dtype_code(out.dtype), M, N, K, lda, ldw, ldc, _stream()), "gemm_f32")
    return out


# ----------------------------------------------------------------------------------------
# position encoding + cache write, attention
# ----------------------------------------------------------------------------------------

PAIRING = {"half": 0, "adjacent": 1}


def rope_kv_write(qkv, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, n_rot: int, pairing: str, k_pages: torch.Tensor, v_pages: torch.Tensor, n_heads: int,
                  n_kv_heads: int, head_dim: int, status: torch.Tensor, write_kv: bool = True,
                  q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate the first ``n_rot`` dimensions of q and k by the positions and store k and v in
    their cells (``write_kv`` False: q only, for a layer that reads another layer's cache).
    ``qkv`` is [tokens, (H + 2 Hkv) D] in the cache's type (q is then rotated in place unless
    ``q_out`` is given), or ``Partials`` of a projection cut along K (``q_out`` is then made
    if absent).  ``inv_freq``: float32 [n_rot / 2], or [2, n_rot / 2] with the part of each
    frequency that float32 lost in the second row (angles at positions in the thousands are
    then as exact as at the first ones).  Returns the rotated q as [tokens, H D] (a view of qkv when in place)."""
    _need(k_pages, "key pages", ndim=4)
    _need(v_pages, "value pages", k_pages.dtype, 4)
    cache_dt = k_pages.dtype
    width = (n_heads + 2 * n_kv_heads) * head_dim
    bias = None
    if isinstance(qkv, Partials):
        src = qkv.data
        _need(src, "qkv parts", torch.float32, 3)
        if not src.is_contiguous() or src.shape[2] != width:
            raise KernelError("rope_kv_write: parts must be [parts, tokens, (H + 2 Hkv) D] and contiguous")
        n_parts, n, lds, stride, bias = src.shape[0], src.shape[1], width, src.shape[1] * width, qkv.bias
        if q_out is None:
            q_out = torch.empty((n, n_heads * head_dim), dtype=cache_dt, device=src.device)
    else:
        src = qkv
        _need(src, "qkv", ndim=2)
        lds = _rows_contiguous(src, "qkv")
        n_parts, n, stride = 1, src.shape[0], 0
        if src.shape[1] != width:
            raise KernelError("rope_kv_write: qkv width is not (H + 2 Hkv) D")
        if q_out is None:
            if src.dtype != cache_dt:
                raise KernelError(f"rope_kv_write: qkv is {src.dtype} but the cache is {cache_dt}; give q_out")
            q_out = src[:, : n_heads * head_dim]
    _need(q_out, "rotated q", cache_dt, 2)
    ldq = _rows_contiguous(q_out, "rotated q")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    freq_lo = None
    if inv_freq.dim() == 2:          # [2, n_rot / 2]: the frequencies, and what float32 lost of each
        if inv_freq.shape[0] != 2 or not inv_freq.is_contiguous():
            raise KernelError("rope_kv_write: frequencies with low parts are a contiguous [2, n_rot / 2]")
        inv_freq, freq_lo = inv_freq[0], inv_freq[1]
    _need(inv_freq, "rotary frequencies", torch.float32, 1)
    if positions.numel() != n or seq_of_token.numel() != n or q_out.shape != (n, n_heads * head_dim):
        raise KernelError("rope_kv_write: one position, one request index and one q row per token")
    n_pages, hkv, page, d = k_pages.shape
    if (hkv, d) != (n_kv_heads, head_dim) or v_pages.shape != k_pages.shape or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelError(f"rope_kv_write: pages {tuple(k_pages.shape)} do not fit {n_kv_heads} KV heads of {head_dim}")
    if not block_table.is_contiguous():
        raise KernelError("rope_kv_write: the block table is not contiguous")
    if n_rot % 2 or n_rot > head_dim or inv_freq.numel() < max(n_rot // 2, 1):
        raise KernelError(f"rope_kv_write: n_rot {n_rot} must be even, at most head_dim, and have n_rot / 2 frequencies")
    fn = _fn("rope_cache", "lgml_rope_kv_write", [c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_void_p, c_void_p])
    _check("rope_cache", fn(_ptr(src), dtype_code(src.dtype), lds, n_parts, stride, _ptr(bias), _ptr(q_out), dtype_code(cache_dt), ldq,
                            _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(inv_freq), _ptr(freq_lo), n_rot,
                            PAIRING[pairing], _ptr(k_pages), _ptr(v_pages), n_pages, page, n, n_heads, n_kv_heads, head_dim,
                            1 if write_kv else 0, _ptr(status), _stream()), "rope_kv_write")
    return q_out


def paged_attention_ref(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                        k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                        status: torch.Tensor, softcap: float = 0.0) -> torch.Tensor:
    """out[t, h] = attention of query (t, h) over its request's cached keys at positions
    <= its own (the last ``window`` of them if window > 0).  ``q`` may be a column slice
    of a wider buffer.  ``softcap`` > 0 caps the scaled scores: s -> softcap * tanh(s / softcap)."""
    _need(q, "queries", ndim=2)
    _need(out, "attention output", q.dtype, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    n_pages, hkv, page, d = k_pages.shape
    _need(k_pages, "key pages", q.dtype, 4)
    _need(v_pages, "value pages", q.dtype, 4)
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d):
        raise KernelError(f"paged_attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {n_heads} heads of {d}")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("paged_attention: pages and block table must be contiguous")
    fn = _fn("attention_ref", "lgml_paged_attention_ref", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                           c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p])
    _check("attention_ref", fn(_ptr(q), dtype_code(q.dtype), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1],
                               _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(out), ldo, n, n_heads, hkv, d, float(scale), int(window or 0),
                               float(softcap or 0.0), _ptr(status), _stream()), "paged_attention_ref")
    return out


def sink_qkv_store(proj: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                   k_pages: torch.Tensor, v_pages: torch.Tensor, n_heads: int, status: torch.Tensor, temp_coef: float = 0.0,
                   temp_every: int = 1, v_mode: int = 0, v_keep: Optional[torch.Tensor] = None,
                   v_lambda: Optional[torch.Tensor] = None, write_kv: bool = True) -> torch.Tensor:
    """From the fused projection's float32 output ``proj`` [tokens, q | k | v | ...]: q times its
    position's temperature 1 + coef ln(floor((p + 1) / every) + 1) into a buffer of the cache's
    type (returned, [tokens, H D]); k and v into their cells (the value pages may have fewer heads
    than the key pages: several key heads then share a value head).  ``v_mode`` 1 also keeps v in
    ``v_keep`` (float32 [tokens, Hkv Dv]); 2 stores (1 - lambda) v + lambda v_keep instead of v."""
    _need(proj, "projection output", torch.float32, 2)
    _need(k_pages, "key pages", ndim=4)
    _need(v_pages, "value pages", k_pages.dtype, 4)
    ldp = _rows_contiguous(proj, "projection output")
    n = proj.shape[0]
    n_pages, hkv, page, d = k_pages.shape
    hv, dv = v_pages.shape[1], v_pages.shape[3]
    if (v_pages.shape[0], v_pages.shape[2]) != (n_pages, page) or hkv % hv or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelError(f"sink_qkv_store: key pages {tuple(k_pages.shape)} and value pages {tuple(v_pages.shape)} do not go together")
    if proj.shape[1] < n_heads * d + (hkv * d + hv * dv if write_kv else 0):
        raise KernelError(f"sink_qkv_store: {proj.shape[1]} columns do not hold q, k and v")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if positions.numel() != n or seq_of_token.numel() != n or not block_table.is_contiguous():
        raise KernelError("sink_qkv_store: one position and one request index per token, and a contiguous block table")
    if v_mode:
        _need(v_keep, "kept values", torch.float32, 2)
        if tuple(v_keep.shape) != (n, hv * dv) or not v_keep.is_contiguous():
            raise KernelError(f"sink_qkv_store: kept values must be a contiguous [{n}, {hv * dv}]")
    if v_mode == 2:
        _need(v_lambda, "mixing weight", torch.float32)
    q_out = torch.empty((n, n_heads * d), dtype=k_pages.dtype, device=proj.device)
    fn = _fn("attention_sink", "lgml_sink_qkv_store", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
                                                       c_void_p, c_int, c_void_p, c_void_p])
    _check("attention_sink", fn(_ptr(proj), ldp, _ptr(q_out), dtype_code(k_pages.dtype), q_out.stride(0), _ptr(positions), _ptr(seq_of_token),
                                _ptr(block_table), block_table.shape[1], _ptr(k_pages), _ptr(v_pages), n_pages, page, n, n_heads, hkv, hv, d, dv,
                                float(temp_coef), int(temp_every), int(v_mode), _ptr(v_keep), _ptr(v_lambda), 1 if write_kv else 0,
                                _ptr(status), _stream()), "sink_qkv_store")
    return q_out


def _value_pages(v_pages: torch.Tensor, k_pages: torch.Tensor, who: str):
    """(value heads, value size, elements between value rows) of value pages that are their own tensor
    or a column range of wider cells (the first columns of the key cells, say)."""
    n_pages, hkv, page, _ = k_pages.shape
    hv, dv = v_pages.shape[1], v_pages.shape[3]
    ldv = v_pages.stride(2)
    if (v_pages.shape[0], v_pages.shape[2]) != (n_pages, page) or hkv % hv or v_pages.stride(3) != 1 or ldv < dv \
            or v_pages.stride(1) != page * ldv or v_pages.stride(0) != hv * page * ldv:
        raise KernelError(f"{who}: value pages {tuple(v_pages.shape)} (strides {v_pages.stride()}) do not go with key pages {tuple(k_pages.shape)}")
    return hv, dv, ldv


def sink_attention(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                   k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                   status: torch.Tensor, slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """out[t, h] = sum_j w_j v_j over the request's keys at positions j <= p with p - j < window (all j <= p
    when window is 0) or j < ``keep_first`` (the request's first tokens stay visible beyond the window),
    w_j = exp(s_j) / (exp(sink_h) + sum exp(s)), s_j = cap((q . k_j) scale) - slope_h (p - j), cap(s) = softcap tanh(s / softcap)
    (``softcap`` 0: s itself);
    then times sigmoid(gate[t, h]) element by element when ``gate`` (float32, pre-sigmoid; may be a
    column slice) is given.  Keys have head size D, values Dv.  The value pages may have fewer heads than the
    key pages (key heads g Hkv / Hv ... share value head g) and may be a column range of wider cells.
    ``out`` has the queries' type or is float32."""
    _need(q, "queries", ndim=2)
    _need(out, "attention output", ndim=2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", q.dtype, 4)
    _need(v_pages, "value pages", q.dtype, 4)
    n_pages, hkv, page, d = k_pages.shape
    hv, dv, ldv = _value_pages(v_pages, k_pages, "sink_attention")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * dv) or out.dtype not in (q.dtype, torch.float32):
        raise KernelError(f"sink_attention: q {tuple(q.shape)} / out {tuple(out.shape)} {out.dtype} do not fit {n_heads} heads of {d} and {dv}")
    if not k_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("sink_attention: pages and block table must be contiguous")
    for t, what in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None:
            _need(t, what, torch.float32, 1)
            if t.numel() != n_heads or not t.is_contiguous():
                raise KernelError(f"sink_attention: one of the {what} per head")
    ldg = 0
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        ldg = _rows_contiguous(gate, "gate")
        if tuple(gate.shape) != (n, n_heads * dv):
            raise KernelError(f"sink_attention: gate {tuple(gate.shape)} is not [{n}, {n_heads * dv}]")
    fn = _fn("attention_sink", "lgml_sink_attention", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                       c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                       c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p])
    _check("attention_sink", fn(_ptr(q), dtype_code(q.dtype), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1],
                                _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(slopes), _ptr(sinks), _ptr(gate), ldg, _ptr(out),
                                dtype_code(out.dtype), ldo, n, n_heads, hkv, hv, d, dv, ldv, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first or 0),
                                _ptr(status), _stream()), "sink_attention")
    return out


SINK_TILE_TOKENS = 64      # query tokens per tile of the tensor-core sink attention


def sink_attention_mma(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                       v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int, status: torch.Tensor,
                       slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                       gate: Optional[torch.Tensor] = None, keep_first: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """``sink_attention`` for prompts and portions on tensor cores: bfloat16, pages of 64, head sizes
    up to 128.  ``tiles`` int32 [n_tiles, 4]: (request row, first token row, tokens <= 64, 0), each
    tile within one request (``StepBatch.attention_tiles(SINK_TILE_TOKENS)``).  ``out`` bfloat16 or float32."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", ndim=2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    hv, dv, ldv = _value_pages(v_pages, k_pages, "sink_attention_mma")
    _need(positions, "positions", torch.int32, 1)
    _need(tiles, "tiles", torch.int32, 2)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * dv) or tiles.shape[1] != 4 or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"sink_attention_mma: q {tuple(q.shape)} / out {tuple(out.shape)} {out.dtype} / tiles {tuple(tiles.shape)} do not fit")
    if not k_pages.is_contiguous() or not block_table.is_contiguous() or not tiles.is_contiguous():
        raise KernelError("sink_attention_mma: pages, block table and tiles must be contiguous")
    for t, what in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None:
            _need(t, what, torch.float32, 1)
            if t.numel() != n_heads or not t.is_contiguous():
                raise KernelError(f"sink_attention_mma: one of the {what} per head")
    ldg = 0
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        ldg = _rows_contiguous(gate, "gate")
        if tuple(gate.shape) != (n, n_heads * dv):
            raise KernelError(f"sink_attention_mma: gate {tuple(gate.shape)} is not [{n}, {n_heads * dv}]")
    fn = _fn("attention_sink", "lgml_sink_attention_mma", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                                           c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                           c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p])
    _check("attention_sink", fn(_ptr(q), ldq, _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(block_table), block_table.shape[1], _ptr(k_pages),
                                _ptr(v_pages), n_pages, page, _ptr(slopes), _ptr(sinks), _ptr(gate), ldg, _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                ldo, n_heads, hkv, hv, d, dv, ldv, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first or 0), _ptr(status), _stream()),
           "sink_attention_mma")
    return out


def sink_twin_supports(q: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, gate: Optional[torch.Tensor]) -> bool:
    """Whether ``sink_attention_twin`` takes these operands: pages of 64, keys and values of one head
    size, 64 or 128, and q, out and the gate readable in 16-byte pieces."""
    return (PREFILL_ATTENTION == "tcgen05" and k_pages.shape[2] == 64 and k_pages.shape[3] in (64, 128) and v_pages.shape[3] == k_pages.shape[3]
            and prefill_tc_supports(q, out)
            and (gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.stride(0) % 4 == 0 and gate.data_ptr() % 16 == 0)))


def sink_attention_twin(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                        v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int, status: torch.Tensor,
                        slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None,
                        gate: Optional[torch.Tensor] = None, softcap: float = 0.0) -> torch.Tensor:
    """``sink_attention`` for prompts and portions on tcgen05 tensor cores: the two-tile kernel of
    ``prefill_attention_twin`` with the slopes' bias on the scores, the sink in the denominator and
    the gate on the output.  bfloat16, pages of 64, keys and values of one head size (64 or 128).
    ``tiles`` as for ``prefill_attention_twin`` (``prefill_twin_tile_tokens``)."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", torch.bfloat16, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    _need(positions, "positions", torch.int32, 1)
    _need(tiles, "tiles", torch.int32, 2)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d) or tiles.shape[1] != 4 or v_pages.shape != k_pages.shape:
        raise KernelError(f"sink_attention_twin: q {tuple(q.shape)} / out {tuple(out.shape)} / tiles {tuple(tiles.shape)} / values "
                          f"{tuple(v_pages.shape)} do not fit")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous() or not tiles.is_contiguous():
        raise KernelError("sink_attention_twin: pages, block table and tiles must be contiguous")
    for t, what in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None:
            _need(t, what, torch.float32, 1)
            if t.numel() != n_heads or not t.is_contiguous():
                raise KernelError(f"sink_attention_twin: one of the {what} per head")
    ldg = 0
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        ldg = _rows_contiguous(gate, "gate")
        if tuple(gate.shape) != (n, n_heads * d):
            raise KernelError(f"sink_attention_twin: gate {tuple(gate.shape)} is not [{n}, {n_heads * d}]")
    fn = _fn("attention_prefill_twin", "lgml_sink_attention_twin", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                                                    c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                                                    c_int, c_float, c_float, c_int, c_void_p, c_void_p])
    _check("attention_prefill_twin", fn(_ptr(q), ldq, _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(block_table), block_table.shape[1],
                                        _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(slopes), _ptr(sinks), _ptr(gate), ldg, _ptr(out), ldo,
                                        n_heads, hkv, d, float(scale), float(softcap or 0.0), int(window or 0), _ptr(status), _stream()), "sink_attention_twin")
    return out


def sink_decode_splits(n_tokens: int, n_kv_heads: int, group: int, reach: int) -> int:
    """Key ranges of the split sink attention: enough CTAs to cover the SMs twice, at least two pages
    a range, at most 64 ranges, and none of them empty.  ``reach``: the most keys a query sees."""
    ctas = max(n_tokens * n_kv_heads * -(-group // 8), 1)
    pages = max(reach, 1) // 64 + 2          # a window of w keys can touch w / 64 + 2 pages
    want = max(1, min((2 * sm_count()) // ctas, pages // 2, 64))
    per = -(-pages // want)
    return -(-pages // per)


def sink_decode(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int, status: torch.Tensor, n_splits: int,
                slopes: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                keep_first: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """``sink_attention`` for decoding and short portions (bfloat16, pages of 64): each token's keys cut into
    ``n_splits`` ranges, the query heads of a KV head scored together, the ranges merged by a second kernel.
    ``out`` bfloat16 or float32."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", ndim=2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    hv, dv, ldv = _value_pages(v_pages, k_pages, "sink_decode")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * dv) or out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"sink_decode: q {tuple(q.shape)} / out {tuple(out.shape)} {out.dtype} do not fit {n_heads} heads of {d} and {dv}")
    if not k_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("sink_decode: pages and block table must be contiguous")
    for t, what in ((slopes, "slopes"), (sinks, "sinks")):
        if t is not None:
            _need(t, what, torch.float32, 1)
            if t.numel() != n_heads or not t.is_contiguous():
                raise KernelError(f"sink_decode: one of the {what} per head")
    ldg = 0
    if gate is not None:
        _need(gate, "gate", torch.float32, 2)
        ldg = _rows_contiguous(gate, "gate")
        if tuple(gate.shape) != (n, n_heads * dv):
            raise KernelError(f"sink_decode: gate {tuple(gate.shape)} is not [{n}, {n_heads * dv}]")
    scratch = torch.empty(n * n_heads * n_splits * (dv + 2), dtype=torch.float32, device=q.device) if n_splits > 1 else None
    fn = _fn("attention_sink", "lgml_sink_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                    c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p])
    _check("attention_sink", fn(_ptr(q), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(k_pages),
                                _ptr(v_pages), n_pages, page, _ptr(slopes), _ptr(sinks), _ptr(gate), ldg, _ptr(out), 1 if out.dtype == torch.float32 else 0,
                                ldo, _ptr(scratch), int(n_splits), n, n_heads, hkv, hv, d, dv, ldv, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first or 0),
                                _ptr(status), _stream()), "sink_decode")
    return out


# ----------------------------------------------------------------------------------------
# per head, around attention: differential maps, latent keys and values
# ----------------------------------------------------------------------------------------

def diff_combine(maps: torch.Tensor, out: torch.Tensor, n_heads: int, n_key_heads: int, lam: float, eps: float, out_scale: float) -> torch.Tensor:
    """Differential attention's combination: ``maps`` [tokens, 2 H Dv] holds two attention outputs per
    head, in the order (key head g, map m, head r of the group); out[t, h] = o / sqrt(mean(o^2) + eps) *
    out_scale with o = a1 - lam a2."""
    _need(maps, "attention maps", ndim=2)
    _need(out, "combined output", ndim=2)
    ldi, ldo = _rows_contiguous(maps, "attention maps"), _rows_contiguous(out, "combined output")
    n = maps.shape[0]
    if maps.shape[1] % (2 * n_heads) or out.shape != (n, maps.shape[1] // 2) or n_heads % n_key_heads:
        raise KernelError(f"diff_combine: maps {tuple(maps.shape)} / out {tuple(out.shape)} do not fit {n_heads} heads on {n_key_heads}")
    dv = maps.shape[1] // (2 * n_heads)
    fn = _fn("attention_heads", "lgml_diff_combine", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                                      c_float, c_void_p])
    _check("attention_heads", fn(_ptr(maps), dtype_code(maps.dtype), ldi, _ptr(out), dtype_code(out.dtype), ldo, n, n_heads, n_key_heads, dv,
                                 float(lam), float(eps), float(out_scale), _stream()), "diff_combine")
    return out


def latent_prepare(q_proj: torch.Tensor, down: torch.Tensor, norm_w: torch.Tensor, eps: float, inv_freq: torch.Tensor, n_rot: int,
                   positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, cells: torch.Tensor, n_heads: int,
                   head_dim: int, rot_dim: int, rank: int, status: torch.Tensor, write_kv: bool = True, rot_mag: float = 1.0):
    """Latent attention between its projections and attention.  ``q_proj`` float32 [tokens, H (D + Dr)]
    (per head D plain, then Dr rotated entries), ``down`` float32 [tokens, R + Dr].  The first R columns
    of ``down``, over their root mean square, times ``norm_w``, are the latent c; the last Dr are a key
    part that is rotated (the first ``n_rot`` entries, pairs (2i, 2i + 1), ``inv_freq`` [2, n_rot / 2]:
    the float32 frequencies and what float32 lost of them).  [c | rotated part] goes into the token's
    cell of ``cells`` [pages, 1, page, R + Dr].  Returns (q_plain [tokens, H D], q_full [tokens,
    H (R + Dr)]) in the cells' type; of q_full only the rotated Dr entries behind each head's first R
    are written (``head_linear`` fills those).  ``rot_mag`` multiplies every cosine and sine (a frequency
    scaling that lengthens the rotated vectors)."""
    _need(q_proj, "query projection", torch.float32, 2)
    _need(down, "down projection", torch.float32, 2)
    _need(cells, "latent cells", ndim=4)
    _need(norm_w, "latent norm weight", torch.float32, 1)
    _need(inv_freq, "frequencies", torch.float32, 2)
    n = q_proj.shape[0]
    n_pages, one, page, width = cells.shape
    if one != 1 or width != rank + rot_dim or not cells.is_contiguous():
        raise KernelError(f"latent_prepare: cells {tuple(cells.shape)} are not [pages, 1, page, {rank + rot_dim}]")
    if q_proj.shape[1] != n_heads * (head_dim + rot_dim) or tuple(down.shape) != (n, rank + rot_dim) or norm_w.numel() != rank:
        raise KernelError(f"latent_prepare: q {tuple(q_proj.shape)} / down {tuple(down.shape)} do not fit {n_heads} heads of {head_dim} + {rot_dim}, rank {rank}")
    if n_rot % 2 or n_rot > rot_dim or tuple(inv_freq.shape) != (2, max(n_rot // 2, 1)) or not inv_freq.is_contiguous():
        raise KernelError(f"latent_prepare: {n_rot} rotated entries of {rot_dim}, frequencies {tuple(inv_freq.shape)}")
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if positions.numel() != n or seq_of_token.numel() != n or not block_table.is_contiguous():
        raise KernelError("latent_prepare: one position and one request index per token, and a contiguous block table")
    ldq, ldd = _rows_contiguous(q_proj, "query projection"), _rows_contiguous(down, "down projection")
    q_plain = torch.empty((n, n_heads * head_dim), dtype=cells.dtype, device=cells.device)
    q_full = torch.empty((n, n_heads * (rank + rot_dim)), dtype=cells.dtype, device=cells.device)
    fn = _fn("attention_heads", "lgml_latent_prepare", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p,
                                                        c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check("attention_heads", fn(_ptr(q_proj), ldq, _ptr(down), ldd, _ptr(norm_w), float(eps), _ptr(inv_freq[0]), _ptr(inv_freq[1]), int(n_rot),
                                 _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(cells), dtype_code(cells.dtype),
                                 n_pages, page, _ptr(q_plain), q_plain.stride(0), _ptr(q_full), q_full.stride(0), n, n_heads, head_dim, rot_dim,
                                 rank, 1 if write_kv else 0, float(rot_mag), _ptr(status), _stream()), "latent_prepare")
    return q_plain, q_full


def head_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, x_head_stride: int, out_head_stride: int,
                gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A product per head: out[t, h * out_head_stride + o] = sum_k x[t, h * x_head_stride + k] w[h, o, k];
    ``w`` [H, O, K] contiguous, x and out 2-D with dense rows, all of one type (float32 sums).  With ``gate``
    (float32, the output's columns, dense rows) the result is multiplied by sigmoid(gate)."""
    _need(x, "head_linear input", ndim=2)
    _need(w, "head_linear weights", x.dtype, 3)
    _need(out, "head_linear output", x.dtype, 2)
    ldx, ldo = _rows_contiguous(x, "head_linear input"), _rows_contiguous(out, "head_linear output")
    H, O, K = w.shape
    n = x.shape[0]
    if not w.is_contiguous() or out.shape[0] != n or (H - 1) * x_head_stride + K > x.shape[1] or (H - 1) * out_head_stride + O > out.shape[1]:
        raise KernelError(f"head_linear: x {tuple(x.shape)} / w {tuple(w.shape)} / out {tuple(out.shape)} with head strides {x_head_stride}, {out_head_stride} do not fit")
    ldg = 0
    if gate is not None:
        _need(gate, "head_linear gate", torch.float32, 2)
        ldg = _rows_contiguous(gate, "head_linear gate")
        if gate.shape[0] != n or (H - 1) * out_head_stride + O > gate.shape[1]:
            raise KernelError(f"head_linear: gate {tuple(gate.shape)} does not cover the output's columns")
    fn = _fn("attention_heads", "lgml_head_linear", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_void_p])
    _check("attention_heads", fn(_ptr(x), ldx, int(x_head_stride), _ptr(w), _ptr(out), ldo, int(out_head_stride), dtype_code(x.dtype), n, H, O, K,
                                 _ptr(gate), ldg, _stream()), "head_linear")
    return out


# ----------------------------------------------------------------------------------------
# mixture of experts
# ----------------------------------------------------------------------------------------

ROUTER_MODES = {"softmax": 0, "sigmoid": 1}


def moe_router(h: torch.Tensor, w_router: torch.Tensor, b_router: Optional[torch.Tensor], top: int, mode: str = "softmax",
               route_scale: float = 1.0, n_extra: int = 0):
    """The ``top`` experts with the largest float32 logits W_r h + b_r per token (ties: the lower index)
    and the softmax over those logits alone: (ids int32 [tokens, top], weights float32 [tokens, top]).
    ``mode`` "sigmoid": the scores are sigmoid(W_r h); the experts with the largest score + b_r are chosen, and
    the weights are the chosen scores over their sum (+ 1e-20), times ``route_scale``.  ``n_extra``: the last
    rows of ``w_router`` are no experts; the sigmoids of their logits come back as a third result
    float32 [tokens, n_extra]."""
    _need(h, "router input", ndim=2)
    _need(w_router, "router weight", torch.float32, 2)
    ldh = _rows_contiguous(h, "router input")
    n, E = h.shape
    X = w_router.shape[0] - int(n_extra)
    if mode not in ROUTER_MODES or n_extra < 0 or X <= 0:
        raise KernelError(f"moe_router: mode '{mode}' with {n_extra} extra rows of {w_router.shape[0]}")
    if w_router.shape[1] != E or not w_router.is_contiguous() or not 0 < top <= X:
        raise KernelError(f"moe_router: weight {tuple(w_router.shape)} does not fit rows of {E}, or {top} of {X} experts")
    if b_router is not None:
        _need(b_router, "router bias", torch.float32, 1)
        if b_router.numel() != X:
            raise KernelError("moe_router: one bias per expert")
    ids = torch.empty((n, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=h.device)
    extra = torch.empty((n, n_extra), dtype=torch.float32, device=h.device) if n_extra else None
    fn = _fn("moe", "lgml_moe_router_mode", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                             c_int, c_void_p, c_void_p], label="moe_router")
    _check("moe", fn(_ptr(h), dtype_code(h.dtype), ldh, _ptr(w_router), _ptr(b_router), _ptr(ids), _ptr(wts), n, E, X, int(top), ROUTER_MODES[mode],
                     float(route_scale), int(n_extra), _ptr(extra), _stream()), "moe_router")
    return (ids, wts, extra) if n_extra else (ids, wts)


def _also(also, also_w, n: int, E: int, who: str):
    """A term every token gets beside its experts' (float32 [tokens, E]) and the token's weight on it (float32 [tokens])."""
    if also is None:
        return
    _need(also, "shared term", torch.float32, 2)
    _need(also_w, "shared term's weights", torch.float32)
    if tuple(also.shape) != (n, E) or also_w.numel() != n or not also.is_contiguous() or not also_w.is_contiguous():
        raise KernelError(f"{who}: shared term {tuple(also.shape)} with weights {tuple(also_w.shape)} does not fit [{n}, {E}]")


def _moe_shapes(h, ids, wts, w_gu, w_down, who: str, gated: bool = True):
    for t, what in ((w_gu, "gate|up"), (w_down, "down")):
        _need(t, f"experts' {what} matrices", h.dtype, 3)
        if not t.is_contiguous():
            raise KernelError(f"{who}: the {what} matrices must be contiguous")
    _need(ids, "chosen experts", torch.int32, 2)
    _need(wts, "experts' weights", torch.float32, 2)
    n, E = h.shape
    X, F2, _ = w_gu.shape
    F, top = (F2 // 2 if gated else F2), ids.shape[1]
    if tuple(w_gu.shape) != (X, 2 * F if gated else F, E) or tuple(w_down.shape) != (X, E, F) or tuple(ids.shape) != (n, top) \
            or tuple(wts.shape) != (n, top) or not ids.is_contiguous() or not wts.is_contiguous():
        raise KernelError(f"{who}: shapes disagree: h {tuple(h.shape)}, gate|up {tuple(w_gu.shape)}, down {tuple(w_down.shape)}, ids {tuple(ids.shape)}")
    return n, E, F, X, top


def moe_experts_rows(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, gated: bool = True,
                     also: Optional[torch.Tensor] = None, also_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_s wts[t, s] W_down[e] (silu(W_gate[e] h_t) * (W_up[e] h_t)), e = ids[t, s]: float32
    [tokens, E].  The experts' matrices stacked: ``w_gu`` [X, 2 F, E] with the gate row of a feature followed
    by its up row, ``w_down`` [X, E, F].  A block per (token, chosen expert): the form for few tokens and for
    the 32-bit path.  ``gated`` False: experts without a gate, ``w_gu`` [X, F, E] and the activation relu squared.
    ``also`` / ``also_w``: out += also_w[t] * also[t] (a shared expert's output and the token's gate on it)."""
    _need(h, "experts' input", ndim=2)
    ldh = _rows_contiguous(h, "experts' input")
    n, E, F, X, top = _moe_shapes(h, ids, wts, w_gu, w_down, "moe_experts_rows", gated)
    _also(also, also_w, n, E, "moe_experts_rows")
    act = torch.empty((n * top, F), dtype=h.dtype, device=h.device)
    out = torch.empty((n, E), dtype=torch.float32, device=h.device)
    fn = _fn("moe", "lgml_moe_experts_rows_form", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check("moe", fn(_ptr(h), dtype_code(h.dtype), ldh, _ptr(ids), _ptr(wts), _ptr(w_gu), _ptr(w_down), _ptr(act), _ptr(out), n, E, F, X,
                     top, 0 if gated else 1, _ptr(also), _ptr(also_w), _stream()), "moe_experts_rows")
    return out


MOE_TILE_ROWS = 128


def moe_grouped_supports(h: torch.Tensor, w_gu: torch.Tensor, gated: bool = True) -> bool:
    """Whether the grouped forms take these operands: bfloat16, widths that are multiples of 8."""
    return (h.dtype == torch.bfloat16 and h.dim() == 2 and h.stride(1) == 1 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
            and w_gu.shape[1] % (16 if gated else 8) == 0 and w_gu.shape[2] % 8 == 0)


def _moe_tiles(n_rows: int, X: int) -> int:
    return -(-n_rows // MOE_TILE_ROWS) + min(X, n_rows)


def moe_experts_grouped(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """``moe_experts_rows`` for many tokens, bfloat16, on ``mma.sync``: the (token, chosen expert) rows sorted by
    expert on the device and cut into tiles of 128 rows of one expert; float32 [tokens, E].  No host value is
    read: the launches are the same whatever the router chose.  (The form ``moe_experts_tcgen05`` replaced;
    ``LGML_MOE_GROUPED=mma`` selects it.)"""
    _need(h, "experts' input", torch.bfloat16, 2)
    ldh = _rows_contiguous(h, "experts' input")
    n, E, F, X, top = _moe_shapes(h, ids, wts, w_gu, w_down, "moe_experts_grouped")
    if not moe_grouped_supports(h, w_gu):
        raise KernelError("moe_experts_grouped: widths and row strides must be multiples of 8 and the input 16-byte aligned")
    n_rows = n * top
    max_tiles = _moe_tiles(n_rows, X)
    rows = torch.empty(n_rows, dtype=torch.int32, device=h.device)
    tiles = torch.empty(3 * max_tiles + 1, dtype=torch.int32, device=h.device)
    act = torch.empty((n_rows, F), dtype=torch.bfloat16, device=h.device)
    y = torch.empty((n_rows, E), dtype=torch.float32, device=h.device)
    out = torch.empty((n, E), dtype=torch.float32, device=h.device)
    fn = _fn("moe", "lgml_moe_experts_grouped", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check("moe", fn(_ptr(h), ldh, _ptr(ids), _ptr(wts), _ptr(w_gu), _ptr(w_down), _ptr(rows), _ptr(tiles), max_tiles, _ptr(act),
                     _ptr(y), _ptr(out), n, E, F, X, top, _stream()), "moe_experts_grouped")
    return out


def moe_experts_tcgen05(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor,
                        status: torch.Tensor, gated: bool = True, also: Optional[torch.Tensor] = None,
                        also_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``moe_experts_rows`` for many tokens, bfloat16, on tcgen05: the (token, chosen expert) rows are sorted by
    expert on the device, the tokens' rows gathered into tiles of 128 rows of one expert, and the two products
    run as grouped products of the tcgen05 kernel (a tile reads the matrices of its expert; the gate|up product
    applies the SiLU gate in its epilogue); a token's rows are then added, weighted, in the order of its experts.
    float32 [tokens, E].  No host value is read.  ``gated`` False: experts without a gate (``w_gu`` [X, F, E], the
    first product's epilogue is relu squared); ``also`` / ``also_w`` as for ``moe_experts_rows``."""
    _need(h, "experts' input", torch.bfloat16, 2)
    ldh = _rows_contiguous(h, "experts' input")
    n, E, F, X, top = _moe_shapes(h, ids, wts, w_gu, w_down, "moe_experts_tcgen05", gated)
    _also(also, also_w, n, E, "moe_experts_tcgen05")
    if not moe_grouped_supports(h, w_gu, gated):
        raise KernelError("moe_experts_tcgen05: widths and row strides must be multiples of 8 and the input 16-byte aligned")
    n_rows = n * top
    max_tiles = _moe_tiles(n_rows, X)
    dev = h.device
    rows = torch.empty(n_rows, dtype=torch.int32, device=dev)
    pos = torch.empty(n_rows, dtype=torch.int32, device=dev)
    tiles = torch.empty(3 * max_tiles + 1, dtype=torch.int32, device=dev)
    a_perm = torch.empty((max_tiles * MOE_TILE_ROWS, E), dtype=torch.bfloat16, device=dev)
    act = torch.empty((max_tiles * MOE_TILE_ROWS, F), dtype=torch.bfloat16, device=dev)
    y = torch.empty((max_tiles * MOE_TILE_ROWS, E), dtype=torch.float32, device=dev)
    out = torch.empty((n, E), dtype=torch.float32, device=dev)
    stream = _stream()
    fn = _fn("moe", "lgml_moe_group_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check("moe", fn(_ptr(ids), _ptr(rows), _ptr(tiles), max_tiles, n, X, top, stream), "moe_group_rows")
    fn = _fn("moe", "lgml_moe_gather_rows", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check("moe", fn(_ptr(h), ldh, _ptr(rows), _ptr(tiles), max_tiles, _ptr(a_perm), _ptr(pos), E, top, stream), "moe_gather_rows")
    fn = _fn("gemm_tcgen05", "lgml_gemm_tcgen05_grouped", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                                           c_void_p, c_void_p])
    _check("gemm_tcgen05", fn(_ptr(a_perm), _ptr(w_gu), _ptr(act), 0, max_tiles, 2 * F if gated else F, E, X, F, _ptr(tiles), 1 if gated else 2,
                              _ptr(status), stream), "gemm_tcgen05_grouped")
    _check("gemm_tcgen05", fn(_ptr(act), _ptr(w_down), _ptr(y), 1, max_tiles, E, F, X, E, _ptr(tiles), 0, _ptr(status), stream),
           "gemm_tcgen05_grouped")
    fn = _fn("moe", "lgml_moe_weighted_sum_also", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p], label="moe_weighted_sum")
    _check("moe", fn(_ptr(y), _ptr(pos), _ptr(wts), _ptr(out), n, E, top, _ptr(also), _ptr(also_w), stream), "moe_weighted_sum")
    return out


# ----------------------------------------------------------------------------------------
# token shift, the minGRU recurrence, the per-layer token input
# ----------------------------------------------------------------------------------------

def _delta_parts(delta, x: torch.Tensor, who: str):
    """(pointer tensor, parts, stride between parts, bias) of a float32 delta or ``Partials`` for x's rows."""
    if delta is None:
        return None, 1, 0, None
    if isinstance(delta, Partials):
        d = delta.data
        _need(d, "residual delta parts", torch.float32, 3)
        if tuple(d.shape[1:]) != tuple(x.shape) or not d.is_contiguous():
            raise KernelError(f"{who}: delta parts must be [parts, rows, width] and contiguous")
        return d, d.shape[0], d.shape[1] * d.shape[2], delta.bias
    _need(delta, "residual delta", torch.float32, 2)
    if delta.shape != x.shape or not delta.is_contiguous():
        raise KernelError(f"{who}: delta must be float32 of the input's shape and contiguous")
    return delta, 1, 0, None


def _state_rows(state: torch.Tensor, width: int, who: str) -> int:
    _need(state, "state slots", torch.float32, 2)
    if state.stride(1) != 1 or state.shape[1] < width:
        raise KernelError(f"{who}: the state's rows must be dense and hold {width} floats, not {tuple(state.shape)}")
    return state.stride(0)


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, seq_of_token: torch.Tensor, seq_start: torch.Tensor,
                slots: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = h[t] + (h[t - 1] - h[t]) * mu per channel, within each request; the row before a request's first
    token of this step is ``state[slot]`` (zeros for a new request), which then takes the step's last row of h.
    h float32 [tokens, W]; ``state`` float32 [slots, >= W] (rows may be part of wider rows)."""
    _need(h, "token shift input", torch.float32, 2)
    _need(mu, "token shift weights", torch.float32, 1)
    _need(out, "token shift output", ndim=2)
    n, W = h.shape
    if not h.is_contiguous() or not out.is_contiguous() or tuple(out.shape) != (n, W) or mu.numel() != W:
        raise KernelError(f"token_shift: shapes disagree: h {tuple(h.shape)}, mu {tuple(mu.shape)}, out {tuple(out.shape)}")
    ld = _state_rows(state, W, "token_shift")
    fn = _fn("token_mix", "lgml_token_shift", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(h), _ptr(mu), _ptr(state), ld, _ptr(seq_of_token), _ptr(seq_start), _ptr(slots), _ptr(out), dtype_code(out.dtype), n, W,
                           _stream()), "token_shift")
    return out


def mingru_chunk_tokens() -> int:
    fn = getattr(csrc.load("token_mix"), "lgml_mingru_chunk_tokens")
    fn.argtypes, fn.restype = [], c_int
    return fn()


def mingru_scan(proj: torch.Tensor, state: torch.Tensor, seq_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor,
                chunks: Optional[torch.Tensor] = None, chunk_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The minGRU recurrence over every request's tokens of this step: ``proj`` float32 [tokens, 3 W] holds per token
    the gate's logits a, the candidate's input u and the output gate's input g; z = sigmoid(a), c = u + 1/2 (u >= 0) or
    sigmoid(u); S <- (1 - z) S + z c from ``state[slot]`` (which takes the last S); out[t] = S_t * silu(g_t).
    With ``chunks`` (int32 [n, 2], token rows [first, past the last) of pieces of the requests' portions, a request's
    pieces in a row) and ``chunk_start`` (int32 [requests + 1]) the pieces run side by side: their products of
    (1 - z) and scans from zero first, a chain over a request's pieces, then every piece from its true start."""
    _need(proj, "minGRU projections", torch.float32, 2)
    _need(out, "minGRU output", ndim=2)
    n = proj.shape[0]
    W = out.shape[1]
    ld = _rows_contiguous(proj, "minGRU projections")
    if proj.shape[1] != 3 * W or out.shape[0] != n or not out.is_contiguous():
        raise KernelError(f"mingru_scan: projections {tuple(proj.shape)} do not fit an output of {tuple(out.shape)}")
    sld = _state_rows(state, W, "mingru_scan")
    n_seqs = slots.numel()
    if chunks is None:
        fn = _fn("token_mix", "lgml_mingru_scan", [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check("token_mix", fn(_ptr(proj), ld, _ptr(state), sld, _ptr(seq_start), _ptr(slots), _ptr(out), dtype_code(out.dtype), n_seqs, W, _stream()),
               "mingru_scan")
        return out
    _need(chunks, "chunks", torch.int32, 2)
    _need(chunk_start, "chunk starts", torch.int32, 1)
    n_chunks = chunks.shape[0]
    if chunks.shape[1] != 2 or not chunks.is_contiguous() or chunk_start.numel() != n_seqs + 1:
        raise KernelError("mingru_scan: chunks are [n, 2] and chunk starts one more than the requests")
    ab = torch.empty((2, n_chunks, W), dtype=torch.float32, device=proj.device)
    fn = _fn("token_mix", "lgml_mingru_chunks", [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(proj), ld, _ptr(state), sld, _ptr(chunks), _ptr(chunk_start), n_chunks, _ptr(slots), _ptr(ab), _ptr(out),
                           dtype_code(out.dtype), n_seqs, W, _stream()), "mingru_chunks")
    return out


def residual_fold(x: torch.Tensor, delta, scale: float = 1.0, copy_dtype: Optional[torch.dtype] = None):
    """x += scale * delta (a float32 tensor or ``Partials``; None: nothing is added), and, with ``copy_dtype``, x in
    that type as a second result."""
    _need(x, "residual stream", torch.float32, 2)
    if not x.is_contiguous():
        raise KernelError("residual_fold: the residual stream must be contiguous")
    dptr, n_parts, stride, dbias = _delta_parts(delta, x, "residual_fold")
    xb = torch.empty(x.shape, dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
    fn = _fn("token_mix", "lgml_side_fold", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(x), _ptr(dptr), n_parts, stride, _ptr(dbias), float(scale), _ptr(xb), dtype_code(copy_dtype) if xb is not None else F32,
                           x.shape[0], x.shape[1], _stream()), "residual_fold")
    return xb


def token_side(x: torch.Tensor, delta, delta_scale: float, token_ids: torch.Tensor, table: torch.Tensor, col0: int, w_gate: torch.Tensor,
               w_proj: torch.Tensor, norm_w: torch.Tensor, eps: float, out_scale: float) -> torch.Tensor:
    """In place on the float32 residual stream, one kernel: x += delta_scale * delta; y = W_proj (gelu_tanh(W_gate x) *
    table[token, col0 : col0 + dim]); x += out_scale * y / rms(y) * norm_w."""
    _need(x, "residual stream", torch.float32, 2)
    _need(table, "token table", w_gate.dtype, 2)
    _need(w_gate, "side gate", ndim=2)
    _need(w_proj, "side projection", w_gate.dtype, 2)
    _need(norm_w, "side norm weight", torch.float32, 1)
    _need(token_ids, "token ids", torch.int32, 1)
    n, W = x.shape
    dim = w_gate.shape[0]
    if not x.is_contiguous() or tuple(w_gate.shape) != (dim, W) or tuple(w_proj.shape) != (W, dim) or norm_w.numel() != W or token_ids.numel() != n \
            or not w_gate.is_contiguous() or not w_proj.is_contiguous() or table.stride(1) != 1:
        raise KernelError(f"token_side: shapes disagree: x {tuple(x.shape)}, gate {tuple(w_gate.shape)}, proj {tuple(w_proj.shape)}")
    dptr, n_parts, stride, dbias = _delta_parts(delta, x, "token_side")
    fn = _fn("token_mix", "lgml_token_side", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                              c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(x), _ptr(dptr), n_parts, stride, _ptr(dbias), float(delta_scale), _ptr(token_ids), _ptr(table), table.stride(0), int(col0),
                           table.shape[0], _ptr(w_gate), _ptr(w_proj), _ptr(norm_w), float(eps), float(out_scale), dtype_code(w_gate.dtype), n, W, dim,
                           _stream()), "token_side")
    return x


def side_gate(gate: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, col0: int, out_dtype: torch.dtype) -> torch.Tensor:
    """g[t, j] = gelu_tanh(gate[t, j]) * table[token_t, col0 + j]; gate float32 [tokens, dim], g in the table's type."""
    _need(gate, "side gate logits", torch.float32, 2)
    _need(table, "token table", out_dtype, 2)
    n, dim = gate.shape
    if not gate.is_contiguous() or table.stride(1) != 1 or token_ids.numel() != n:
        raise KernelError("side_gate: shapes disagree")
    g = torch.empty((n, dim), dtype=out_dtype, device=gate.device)
    fn = _fn("token_mix", "lgml_side_gate", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(gate), _ptr(token_ids), _ptr(table), table.stride(0), int(col0), table.shape[0], _ptr(g), dtype_code(out_dtype), n, dim,
                           _stream()), "side_gate")
    return g


def side_add(x: torch.Tensor, y: torch.Tensor, norm_w: torch.Tensor, eps: float, out_scale: float) -> torch.Tensor:
    """x += out_scale * y / rms(y) * norm_w, row by row; both float32."""
    _need(x, "residual stream", torch.float32, 2)
    _need(y, "side output", torch.float32, 2)
    _need(norm_w, "side norm weight", torch.float32, 1)
    if x.shape != y.shape or not x.is_contiguous() or not y.is_contiguous() or norm_w.numel() != x.shape[1]:
        raise KernelError("side_add: shapes disagree")
    fn = _fn("token_mix", "lgml_side_add", [c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p])
    _check("token_mix", fn(_ptr(x), _ptr(y), _ptr(norm_w), float(eps), float(out_scale), x.shape[0], x.shape[1], _stream()), "side_add")
    return x


# ----------------------------------------------------------------------------------------
# the gated delta rule

# ----------------------------------------------------------------------------------------
# layers that norm what they read and what they add; short convolutions; state-space recurrence
# ----------------------------------------------------------------------------------------

def sandwich_norm(x: torch.Tensor, w_pre: Optional[torch.Tensor], eps: float, out: Optional[torch.Tensor], delta=None,
                  w_post: Optional[torch.Tensor] = None, units=None, row_add: Optional[torch.Tensor] = None,
                  rows: Optional[torch.Tensor] = None, conv=None) -> Optional[torch.Tensor]:
    """One kernel over the rows of the float32 residual stream x [tokens, E]:

        m   = delta                                               (a float32 tensor), or
        m   = 1/2 (a / rms(a) u_a + b / rms(b) u_b)                 (``delta`` = (a, b), ``units`` = (u_a, u_b))
        x  += LN(m) w_post (+ row_add)                            (``w_post`` None: m is added as it is)
        out = LN(x) w_pre                                         (``w_pre`` None: no output)

    with LN(v) = (v - mean) / sqrt(var + eps), var the mean of the squared deviations.  With ``rows`` (int32 on the
    device) only those rows are normed and x is not written.

    ``conv`` = (w_t float32 [taps, E], state float32 [slots, >= (taps - 1) E], slots int32 [tokens]) for a step in which
    every request brings ONE token (row r is request r's): out = h + sum_j w_t[j] h_(t - taps + 1 + j) with h = LN(x) w_pre,
    the earlier rows of h from the request's slot, which then takes this one (what ``short_conv`` with ``residual``
    computes from a float32 h, in the same order)."""
    _need(x, "residual stream", torch.float32, 2)
    n, E = x.shape
    if not x.is_contiguous():
        raise KernelError("sandwich_norm: the residual stream must be contiguous")
    d1 = d2 = u1 = u2 = None
    if isinstance(delta, (tuple, list)):
        d1, d2 = delta
        u1, u2 = units
    elif delta is not None:
        d1 = delta
    for t, what in ((d1, "delta"), (d2, "second delta")):
        if t is not None:
            _need(t, what, torch.float32, 2)
            if tuple(t.shape) != (n, E) or not t.is_contiguous():
                raise KernelError(f"sandwich_norm: the {what} must be a contiguous float32 [{n}, {E}], not {tuple(t.shape)}")
    for t, what in ((u1, "unit weight"), (u2, "second unit weight"), (w_post, "weight of the norm on the delta"), (row_add, "added row"),
                    (w_pre, "norm weight")):
        if t is not None:
            _need(t, what, torch.float32, 1)
            if t.numel() != E or not t.is_contiguous():
                raise KernelError(f"sandwich_norm: the {what} must hold {E} floats")
    n_out = n
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_out = rows.numel()
    if w_pre is not None:
        _need(out, "norm output", ndim=2)
        if tuple(out.shape) != (n_out, E) or not out.is_contiguous():
            raise KernelError(f"sandwich_norm: output {tuple(out.shape)} is not a contiguous [{n_out}, {E}]")
    if n_out == 0:
        return out if w_pre is not None else None
    conv_w = conv_state = conv_slots = None
    taps, ld_state = 0, 0
    if conv is not None:
        conv_w, conv_state, conv_slots = conv
        _need(conv_w, "convolution weights", torch.float32, 2)
        _need(conv_slots, "slots", torch.int32, 1)
        taps = conv_w.shape[0]
        if conv_w.shape[1] != E or not conv_w.is_contiguous() or conv_slots.numel() != n or rows is not None or w_pre is None:
            raise KernelError("sandwich_norm: the convolution in the same kernel takes [taps, E] weights, one slot per row, all rows and a norm")
        ld_state = _state_rows(conv_state, (taps - 1) * E, "sandwich_norm") if taps > 1 else 0
    fn = _fn("norm_conv", "lgml_sandwich_norm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p])
    _check("norm_conv", fn(_ptr(x), _ptr(d1), _ptr(d2), _ptr(u1), _ptr(u2), _ptr(w_post), _ptr(row_add), _ptr(w_pre), _ptr(rows),
                           _ptr(out if w_pre is not None else None), dtype_code(out.dtype) if w_pre is not None else F32, n_out, E, float(eps),
                           _ptr(conv_w), _ptr(conv_state if taps > 1 else None), ld_state, _ptr(conv_slots), taps, _stream()), "sandwich_norm")
    return out if w_pre is not None else None


CONV_MAX_TAPS = 8


def short_conv(u: torch.Tensor, w_t: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], seq_of_token: torch.Tensor,
               seq_start: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, act: str = "none", residual: bool = False) -> torch.Tensor:
    """A causal convolution over time on each channel, within each request:

        out[t, c] = [u[t, c] +] act(bias[c] + sum_j w_t[j, c] * u[t - taps + 1 + j, c])

    u float32 [tokens, C] (may be a column slice); ``w_t`` float32 [taps, C], its last row weighs the current token.
    Inputs before a request's first token of this step come from ``state[slot]`` (float32 [slots, >= (taps - 1) C],
    the oldest first; zeros for a new request), which then takes the request's last taps - 1 inputs.
    ``act``: "none" or "silu"; ``residual``: the input is added to the result."""
    _need(u, "convolution input", torch.float32, 2)
    _need(w_t, "convolution weights", torch.float32, 2)
    _need(out, "convolution output", ndim=2)
    n, C = u.shape
    taps = w_t.shape[0]
    ld_in, ld_out = _rows_contiguous(u, "convolution input"), _rows_contiguous(out, "convolution output")
    if w_t.shape[1] != C or not w_t.is_contiguous() or tuple(out.shape) != (n, C):
        raise KernelError(f"short_conv: shapes disagree: u {tuple(u.shape)}, weights {tuple(w_t.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "convolution bias", torch.float32, 1)
        if bias.numel() != C:
            raise KernelError("short_conv: one bias per channel")
    if act not in ("none", "silu"):
        raise KernelError(f"short_conv: unknown activation '{act}'")
    ld_state = _state_rows(state, (taps - 1) * C, "short_conv") if taps > 1 else 0
    fn = _fn("norm_conv", "lgml_short_conv", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check("norm_conv", fn(_ptr(u), ld_in, _ptr(w_t), _ptr(bias), _ptr(state if taps > 1 else None), ld_state, _ptr(seq_of_token), _ptr(seq_start),
                           _ptr(slots), _ptr(out), dtype_code(out.dtype), ld_out, n, C, taps, 1 if act == "silu" else 0, 1 if residual else 0,
                           _stream()), "short_conv")
    return out


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = a z / rms(z) + b z^2 / rms(z^2) + c z^3 / rms(z^3) + e per row, powers element by element, rms(v) =
    sqrt(mean(v^2) + eps); ``coef`` float32 [4] = (a, b, c, e); z float32 [tokens, F]."""
    _need(z, "activation input", torch.float32, 2)
    _need(coef, "activation coefficients", torch.float32, 1)
    _need(out, "activation output", ndim=2)
    if coef.numel() != 4 or tuple(out.shape) != tuple(z.shape):
        raise KernelError(f"poly_norm: four coefficients and an output of the input's shape, not {tuple(coef.shape)} and {tuple(out.shape)}")
    ldz, ldo = _rows_contiguous(z, "activation input"), _rows_contiguous(out, "activation output")
    fn = _fn("norm_conv", "lgml_poly_norm", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check("norm_conv", fn(_ptr(z), ldz, _ptr(coef), _ptr(out), dtype_code(out.dtype), ldo, z.shape[0], z.shape[1], float(eps), _stream()), "poly_norm")
    return out


def conv_rope_store(proj: torch.Tensor, w_t: torch.Tensor, state: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                    seq_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor, mag: float, n_rot: int,
                    k_pages: torch.Tensor, v_pages: torch.Tensor, n_heads: int, status: torch.Tensor, write_kv: bool = True) -> torch.Tensor:
    """From the projection's float32 output ``proj`` [tokens, q (H D) | k (G D) | ...]: q and k through a short causal
    convolution per channel (``w_t`` float32 [taps, (H + G) D], the last row weighs the current token; the last
    taps - 1 projected rows of a request wait in ``state[slot]``); the values are the convolved keys' first Dv entries,
    unrotated; q and k turn by their positions in pairs (i, i + n_rot / 2) with the frequencies ``inv_freq`` ([n_rot / 2]
    float32, or [2, n_rot / 2] with what float32 lost of each) and cos and sin times ``mag``; k and v go to their
    cells, q (returned, [tokens, H D]) to a buffer of the cache's type."""
    _need(proj, "projection output", torch.float32, 2)
    _need(w_t, "convolution weights", torch.float32, 2)
    _need(k_pages, "key pages", ndim=4)
    _need(v_pages, "value pages", k_pages.dtype, 4)
    ldp = _rows_contiguous(proj, "projection output")
    n = proj.shape[0]
    n_pages, G, page, D = k_pages.shape
    Dv = v_pages.shape[3]
    C = (n_heads + G) * D
    taps = w_t.shape[0]
    if tuple(v_pages.shape[:3]) != (n_pages, G, page) or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelError(f"conv_rope_store: key pages {tuple(k_pages.shape)} and value pages {tuple(v_pages.shape)} do not go together")
    if proj.shape[1] < C or w_t.shape[1] != C or not w_t.is_contiguous():
        raise KernelError(f"conv_rope_store: {proj.shape[1]} columns / weights {tuple(w_t.shape)} do not fit q and k of {C} channels")
    for t, what in ((positions, "positions"), (seq_of_token, "request index of tokens")):
        _need(t, what, torch.int32, 1)
        if t.numel() != n:
            raise KernelError(f"conv_rope_store: one of the {what} per token")
    _need(block_table, "block table", torch.int32, 2)
    if not block_table.is_contiguous():
        raise KernelError("conv_rope_store: the block table is not contiguous")
    freq_lo = None
    if inv_freq.dim() == 2:
        if inv_freq.shape[0] != 2 or not inv_freq.is_contiguous():
            raise KernelError("conv_rope_store: frequencies with low parts are a contiguous [2, n_rot / 2]")
        inv_freq, freq_lo = inv_freq[0], inv_freq[1]
    _need(inv_freq, "rotary frequencies", torch.float32, 1)
    if n_rot % 2 or n_rot > D or inv_freq.numel() < max(n_rot // 2, 1):
        raise KernelError(f"conv_rope_store: n_rot {n_rot} must be even, at most the head size {D}, and have n_rot / 2 frequencies")
    ld_state = _state_rows(state, (taps - 1) * C, "conv_rope_store") if taps > 1 else 0
    q_out = torch.empty((n, n_heads * D), dtype=k_pages.dtype, device=proj.device)
    fn = _fn("rope_cache", "lgml_conv_rope_store", [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                    c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int,
                                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check("rope_cache", fn(_ptr(proj), ldp, _ptr(w_t), _ptr(state if taps > 1 else None), ld_state, taps, _ptr(q_out), dtype_code(k_pages.dtype),
                            q_out.stride(0), _ptr(positions), _ptr(seq_of_token), _ptr(seq_start), _ptr(slots), _ptr(block_table), block_table.shape[1],
                            _ptr(inv_freq), _ptr(freq_lo), float(mag), int(n_rot), _ptr(k_pages), _ptr(v_pages), n_pages, page, n, n_heads, G, D, Dv,
                            1 if write_kv else 0, _ptr(status), _stream()), "conv_rope_store")
    return q_out


SSD_PIECE_TOKENS = 64      # tokens of a piece when a long portion's recurrence runs in pieces side by side


def ssd_scan(xbc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor, state: torch.Tensor,
             seq_start: torch.Tensor, slots: torch.Tensor, n_heads: int, n_groups: int, head_dim: int, n_state: int, pieces=None) -> torch.Tensor:
    """The state-space recurrence of a step's tokens, request by request (all float32):

        dt = softplus(dt_raw + dt_bias_h);  S <- exp(-exp(A_log_h) dt) S + dt B x^T;  y = S^T C + D_h x

    ``xbc`` [tokens, x (Hs P) | B (G N) | C (G N)] and ``dt_raw`` [tokens, Hs] may be column slices; head h reads group
    h // (Hs / G).  S ([N, P] per head, stored column by column) lives in ``state[slot]`` (float32 [slots, >= Hs P N]).
    Returns y float32 [tokens, Hs P].

    ``pieces`` = (int32 [n_pieces, 2] rows (first token row, the row past the last), int32 [requests + 1] the first
    piece of every request), as ``StepBatch.scan_pieces`` gives them: the pieces run side by side in three launches.
    Every piece is scanned from zero (what it leaves and the product of its decays are kept), a chain over each
    request's pieces turns that into the state every piece starts from (and the slot's new state), and every
    piece is scanned again from there, which gives y."""
    _need(xbc, "convolved x, B and C", torch.float32, 2)
    _need(dt_raw, "step sizes", torch.float32, 2)
    ldx, ldd = _rows_contiguous(xbc, "convolved x, B and C"), _rows_contiguous(dt_raw, "step sizes")
    n = xbc.shape[0]
    inner = n_heads * head_dim
    if xbc.shape[1] != inner + 2 * n_groups * n_state or tuple(dt_raw.shape) != (n, n_heads):
        raise KernelError(f"ssd_scan: xbc {tuple(xbc.shape)} / dt {tuple(dt_raw.shape)} do not fit {n_heads} heads of {head_dim}, {n_groups} groups of {n_state}")
    for t, what in ((dt_bias, "step bias"), (a_log, "decay logarithms"), (d_skip, "skip weights")):
        _need(t, what, torch.float32, 1)
        if t.numel() != n_heads or not t.is_contiguous():
            raise KernelError(f"ssd_scan: one of the {what} per head")
    ld_state = _state_rows(state, inner * n_state, "ssd_scan")
    y = torch.empty((n, inner), dtype=torch.float32, device=xbc.device)
    n_seqs = seq_start.numel() - 1
    fn = _fn("ssd", "lgml_ssd_scan", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])

    def scan(st, ld, starts, slot_ids, out, count, in_pieces, from_zero, decay):
        _check("ssd", fn(_ptr(xbc), ldx, _ptr(dt_raw), ldd, _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(st), ld, _ptr(starts), _ptr(slot_ids),
                         _ptr(out), inner, count, n_heads, n_groups, head_dim, n_state, 1 if in_pieces else 0, 1 if from_zero else 0, _ptr(decay),
                         _stream()), "ssd_scan")

    if pieces is None:
        scan(state, ld_state, seq_start, slots, y, n_seqs, False, False, None)
        return y
    rows, first = pieces
    _need(rows, "pieces", torch.int32, 2)
    _need(first, "first pieces", torch.int32, 1)
    if rows.shape[1] != 2 or not rows.is_contiguous() or first.numel() != n_seqs + 1:
        raise KernelError("ssd_scan: pieces are a contiguous [n, 2] and one first piece per request and one behind")
    n_pieces = rows.shape[0]
    scratch = torch.empty((n_pieces, inner * n_state), dtype=torch.float32, device=xbc.device)
    decay = torch.empty((n_pieces, n_heads), dtype=torch.float32, device=xbc.device)
    scan(scratch, inner * n_state, rows, None, None, n_pieces, True, True, decay)
    chain = _fn("ssd", "lgml_ssd_chain", [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check("ssd", chain(_ptr(scratch), inner * n_state, _ptr(decay), _ptr(state), ld_state, _ptr(first), _ptr(slots), n_seqs, n_heads, head_dim, n_state,
                        _stream()), "ssd_chain")
    scan(scratch, inner * n_state, rows, None, y, n_pieces, True, False, None)
    return y


def ssd_gate_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """out = (y silu(z)) over the root mean square of each of ``groups`` equal parts of a row, times ``weight``; y and z
    float32 [tokens, inner] (z may be a column slice)."""
    _need(y, "recurrence output", torch.float32, 2)
    _need(z, "gate", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    n, inner = y.shape
    ldy, ldz = _rows_contiguous(y, "recurrence output"), _rows_contiguous(z, "gate")
    if tuple(z.shape) != (n, inner) or weight.numel() != inner or inner % groups:
        raise KernelError(f"ssd_gate_norm: y {tuple(y.shape)}, z {tuple(z.shape)}, weight {tuple(weight.shape)}, {groups} parts do not fit")
    out = torch.empty((n, inner), dtype=out_dtype, device=y.device)
    fn = _fn("ssd", "lgml_ssd_gate_norm", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check("ssd", fn(_ptr(y), ldy, _ptr(z), ldz, _ptr(weight), _ptr(out), dtype_code(out_dtype), inner, n, inner, int(groups), float(eps), _stream()),
           "ssd_gate_norm")
    return out


# ----------------------------------------------------------------------------------------

def delta_prepare(proj: torch.Tensor, a_pre: torch.Tensor, conv_w: torch.Tensor, state: torch.Tensor, conv_off: int,
                  seq_of_token: torch.Tensor, seq_start: torch.Tensor, slots: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  n_heads: int, n_kv_heads: int, dim: int, vdim: int):
    """Everything of a delta-rule mixer that tokens can do side by side.  ``proj`` float32
    [tokens, q (G D) | k (G D) | v (H Dv) | beta (H) | ...]; ``a_pre`` float32 [tokens, H D];
    ``conv_w`` float32 [2 G D + H Dv, taps]; ``state`` float32 [slots, floats] whose part from
    ``conv_off`` on holds each request's last taps - 1 convolution inputs (updated here).
    Returns (q | k | v after convolution, SiLU and the norms [tokens, C]; per head the D decays, beta and
    three zeros [tokens, H, D + 4])."""
    _need(proj, "projection output", torch.float32, 2)
    _need(a_pre, "decay input", torch.float32, 2)
    _need(conv_w, "convolution weights", torch.float32, 2)
    _need(state, "state slots", torch.float32, 2)
    for t, what in ((seq_of_token, "request index of tokens"), (seq_start, "first tokens of requests"), (slots, "slots")):
        _need(t, what, torch.int32, 1)
    _need(a_log, "decay rates", torch.float32, 1)
    _need(dt_bias, "decay bias", torch.float32, 1)
    ldp, lda = _rows_contiguous(proj, "projection output"), _rows_contiguous(a_pre, "decay input")
    n, S = proj.shape[0], slots.numel()
    C = 2 * n_kv_heads * dim + n_heads * vdim
    taps = conv_w.shape[1]
    if conv_w.shape[0] != C or not conv_w.is_contiguous() or not state.is_contiguous():
        raise KernelError(f"delta_prepare: convolution weights {tuple(conv_w.shape)} do not fit {C} channels")
    if proj.shape[1] < C + n_heads or a_pre.shape != (n, n_heads * dim) or a_log.numel() != n_heads or dt_bias.numel() != n_heads * dim:
        raise KernelError("delta_prepare: shapes disagree")
    if seq_of_token.numel() != n or seq_start.numel() != S + 1 or state.shape[1] < conv_off + (taps - 1) * C:
        raise KernelError("delta_prepare: the batch's description or the state's size does not fit")
    out_c = torch.empty((n, C), dtype=torch.float32, device=proj.device)
    gb = torch.empty((n, n_heads, dim + 4), dtype=torch.float32, device=proj.device)
    fn = _fn("delta_rule", "lgml_delta_prepare", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_longlong, c_longlong, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                  c_int, c_int, c_void_p])
    _check("delta_rule", fn(_ptr(proj), ldp, _ptr(a_pre), lda, _ptr(conv_w), taps, _ptr(state), state.stride(0), int(conv_off), _ptr(seq_of_token),
                            _ptr(seq_start), _ptr(slots), _ptr(a_log), _ptr(dt_bias), _ptr(out_c), _ptr(gb), n, S, n_heads,
                            n_kv_heads, dim, vdim, _stream()), "delta_prepare")
    return out_c, gb


def delta_scan(qkv_c: torch.Tensor, gb: torch.Tensor, state: torch.Tensor, seq_start: torch.Tensor, slots: torch.Tensor,
               n_heads: int, n_kv_heads: int, dim: int, vdim: int) -> torch.Tensor:
    """The recurrence S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over each request's
    tokens in order, from and into its slot of ``state`` (S of head h at floats [h D Dv, (h + 1) D Dv)).
    ``qkv_c`` [tokens, q | k | v] and ``gb`` [tokens, H, D + 4] (per head the decays, then beta) as
    ``delta_prepare`` returns them.  Returns o float32 [tokens, H Dv]."""
    n = qkv_c.shape[0]
    _need(qkv_c, "prepared q, k, v", torch.float32, 2)
    _need(gb, "decays and beta", torch.float32, 3)
    _need(state, "state slots", torch.float32, 2)
    if qkv_c.shape[1] != 2 * n_kv_heads * dim + n_heads * vdim or tuple(gb.shape) != (n, n_heads, dim + 4) \
            or state.shape[1] < n_heads * dim * vdim or not (state.is_contiguous() and qkv_c.is_contiguous() and gb.is_contiguous()):
        raise KernelError("delta_scan: shapes disagree")
    o = torch.empty((n, n_heads * vdim), dtype=torch.float32, device=qkv_c.device)
    fn = _fn("delta_rule", "lgml_delta_scan", [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_int, c_void_p])
    _check("delta_rule", fn(_ptr(qkv_c), _ptr(gb), _ptr(state), state.stride(0), _ptr(seq_start), _ptr(slots), _ptr(o),
                            slots.numel(), n_heads, n_kv_heads, dim, vdim, _stream()), "delta_scan")
    return o


def delta_output(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float, out_dtype: torch.dtype, n_heads: int) -> torch.Tensor:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * sigmoid(gate[t, h]) per head of size Dv = len(weight)."""
    _need(o, "read-out", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(gate, "gate", torch.float32, 2)
    n, dv = o.shape[0], weight.numel()
    ldg = _rows_contiguous(gate, "gate")
    if o.shape[1] != n_heads * dv or tuple(gate.shape) != (n, n_heads * dv) or not o.is_contiguous():
        raise KernelError("delta_output: shapes disagree")
    out = torch.empty((n, n_heads * dv), dtype=out_dtype, device=o.device)
    fn = _fn("delta_rule", "lgml_delta_output", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check("delta_rule", fn(_ptr(o), _ptr(weight), _ptr(gate), ldg, _ptr(out), dtype_code(out_dtype), out.stride(0), n, n_heads, dv, float(eps),
                            _stream()), "delta_output")
    return out


# ----------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------

def argmax_rows(logits: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = index of the largest logit of row r; the lowest index wins a tie."""
    _need(logits, "logits", torch.float32, 2)
    _need(out, "token output", torch.int32, 1)
    ld = _rows_contiguous(logits, "logits")
    n = logits.shape[0]
    if out.numel() != n:
        raise KernelError("argmax_rows: one output per row")
    if scratch is None:
        scratch = torch.empty(max(64 * n, 1), dtype=torch.int32, device=logits.device)
    if scratch.numel() < 64 * n or scratch.element_size() != 4:
        raise KernelError("argmax_rows: scratch needs 64 32-bit words per row")
    fn = _fn("sampling", "lgml_argmax_rows", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, logits.shape[1], _ptr(out), _ptr(scratch), _stream()), "argmax_rows")
    return out


TOPK_MAX = 128


def topk_rows(logits: torch.Tensor, k: int, out_vals: Optional[torch.Tensor] = None, out_ids: Optional[torch.Tensor] = None):
    """The k best candidates of every row, ordered by (logit descending, id ascending), as the
    sampler's top_k leaves them: (values float32 [rows, k], ids int32 [rows, k])."""
    _need(logits, "logits", torch.float32, 2)
    ld = _rows_contiguous(logits, "logits")
    n, v = logits.shape
    if not 1 <= k <= min(v, TOPK_MAX):
        raise KernelError(f"topk_rows: k = {k} must be between 1 and min(vocabulary {v}, {TOPK_MAX})")
    if out_vals is None:
        out_vals = torch.empty((n, k), dtype=torch.float32, device=logits.device)
    if out_ids is None:
        out_ids = torch.empty((n, k), dtype=torch.int32, device=logits.device)
    _need(out_vals, "top-k values", torch.float32, 2)
    _need(out_ids, "top-k ids", torch.int32, 2)
    if tuple(out_vals.shape) != (n, k) or tuple(out_ids.shape) != (n, k) or not out_vals.is_contiguous() or not out_ids.is_contiguous():
        raise KernelError("topk_rows: outputs must be contiguous [rows, k]")
    fn = _fn("sampling", "lgml_topk_rows", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, v, int(k), _ptr(out_vals), _ptr(out_ids), _stream()), "topk_rows")
    return out_vals, out_ids


def sample_candidates(vals: torch.Tensor, ids: torch.Tensor, params: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """The chain after top_k on its candidates (``topk_rows``): top_p, min_p, temperature, draw.
    ``params`` float32 [rows, 3]: top_p, ln(min_p) or -inf, temperature > 0; ``uniform`` float64
    [rows]; ``out`` int32 [rows]."""
    _need(vals, "candidate values", torch.float32, 2)
    _need(ids, "candidate ids", torch.int32, 2)
    _need(params, "chain parameters", torch.float32, 2)
    _need(uniform, "uniform numbers", torch.float64, 1)
    _need(out, "token output", torch.int32, 1)
    n, k = vals.shape
    if tuple(ids.shape) != (n, k) or tuple(params.shape) != (n, 3) or uniform.numel() != n or out.numel() != n \
            or not (vals.is_contiguous() and ids.is_contiguous() and params.is_contiguous()):
        raise KernelError("sample_candidates: shapes disagree")
    fn = _fn("sampling", "lgml_sample_candidates", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(vals), _ptr(ids), n, k, _ptr(params), _ptr(uniform), _ptr(out), _stream()), "sample_candidates")
    return out


def sampler_edits(logits: torch.Tensor, edits: torch.Tensor, params: torch.Tensor) -> torch.Tensor:
    """In place on the rows of ``logits``: the sampler's logit bias, then its history penalties.
    ``edits`` int32 [rows, stride]: per row (n_bias, n_hist, n_bias x (id, float bits of the
    bias), n_hist x (id, count)); ``params`` float32 [rows, 3]: repeat, frequency, presence."""
    _need(logits, "logits", torch.float32, 2)
    _need(edits, "sampler edits", torch.int32, 2)
    _need(params, "penalty parameters", torch.float32, 2)
    ld = _rows_contiguous(logits, "logits")
    n, v = logits.shape
    if edits.shape[0] != n or tuple(params.shape) != (n, 3) or not edits.is_contiguous() or not params.is_contiguous():
        raise KernelError("sampler_edits: one row of edits and of parameters per row of logits")
    fn = _fn("sampling", "lgml_sampler_edits", [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, n, v, _ptr(edits), edits.shape[1], _ptr(params), _stream()), "sampler_edits")
    return logits


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Row r: argmax if temperature[r] <= 0, else the inverse-CDF draw of
    softmax(logits[r] / temperature[r]) at uniform[r]."""
    _need(logits, "logits", torch.float32, 2)
    _need(temperature, "temperatures", torch.float32, 1)
    _need(uniform, "uniform numbers", torch.float64, 1)
    _need(out, "token output", torch.int32, 1)
    ld = _rows_contiguous(logits, "logits")
    r = logits.shape[0]
    if temperature.numel() != r or uniform.numel() != r or out.numel() != r:
        raise KernelError("sample_rows: one temperature, uniform number and output per row")
    fn = _fn("sampling", "lgml_sample_rows", [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check("sampling", fn(_ptr(logits), ld, r, logits.shape[1], _ptr(temperature), _ptr(uniform), _ptr(out), _stream()), "sample_rows")
    return out


# ----------------------------------------------------------------------------------------
# bfloat16 matrix products and the fast attention paths
# ----------------------------------------------------------------------------------------

def tcgen05_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA wants 16-byte aligned operands whose row strides are multiples of 16 bytes."""
    return (x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_splits_memo = {}


def tcgen05_splits(M: int, N: int, K: int) -> int:
    """K ranges of a product (remembered per shape: a step asks for the same few shapes again and again)."""
    key = (M, N, K)
    got = _splits_memo.get(key)
    if got is None:
        got = _splits_memo[key] = _tcgen05_splits(M, N, K)
    return got


def _tcgen05_splits(M: int, N: int, K: int) -> int:
    """K ranges for a product with few tokens: enough CTAs to cover the SMs about twice (once
    from 65 tokens on: every range writes and the next kernel reads M x N float32 partial sums,
    which with many tokens is no longer small beside the weights; at 64 tokens nine ranges of
    the output projection still win 0.9 us over five and cost the norm behind them 0.6), each
    with at least four 64-wide K blocks."""
    if M > 64:
        fn = getattr(csrc.load("gemm_tcgen05"), "lgml_gemm_tcgen05_pair_ranges", None)
        if fn is not None:
            fn.argtypes, fn.restype = [c_int, c_int, c_int], c_int
            ranges = fn(M, N, K)
            if ranges:          # on pairs of CTAs: the kernel library knows how it would cut K
                return ranges
    if M > 256:
        return 1
    tiles = -(-N // 128)
    k_blocks = -(-K // 64)
    cover = (2 * sm_count()) // tiles if M <= 64 else -(-sm_count() // tiles)
    splits = max(1, min(cover, k_blocks // 4, 16))
    # no range without K blocks: 64 blocks in 9 ranges of 8 would leave the ninth empty
    return -(-k_blocks // -(-k_blocks // splits))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], bias: Optional[torch.Tensor], status: torch.Tensor,
                 n_splits: Optional[int] = None, scratch: Optional[torch.Tensor] = None, swiglu: bool = False,
                 partials_ok: bool = False, checked: bool = False, relu_sq: bool = False):
    """out[M,N] = x[M,K] . w[N,K]^T (+ bias) on tcgen05 tensor cores; bfloat16 in, float32
    accumulation, out bfloat16 or float32.  ``swiglu``: the rows of w (and bias) come in
    (gate, up) pairs and out[M, N/2] = silu(gate) * up.  ``partials_ok``: when K is cut, return
    ``Partials`` (the float32 partial sums and the bias) instead of adding them up here.
    ``checked``: the caller (``gemm_bf16``) has checked x and w and chosen ``n_splits`` by
    ``tcgen05_splits``."""
    if not checked:
        _need(x, "gemm input", torch.bfloat16, 2)
        _need(w, "gemm weight", torch.bfloat16, 2)
    ldx, ldw = _rows_contiguous(x, "gemm input"), _rows_contiguous(w, "gemm weight")
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K:
        raise KernelError(f"gemm_tcgen05: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if bias is not None:
        _need(bias, "gemm bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm_tcgen05: bias length is not N")
    if swiglu and relu_sq:
        raise KernelError("gemm_tcgen05: one activation at a time")
    if n_splits is None:
        n_splits = 1 if (swiglu or relu_sq) else tcgen05_splits(M, N, K)
    elif checked:
        pass
    elif M > 64 and n_splits > 1 and tcgen05_splits(M, N, K) and os.environ.get("LGML_GEMM_PAIR") != "0":
        # on pairs of CTAs a K range is a whole number of 128-element stages, and none may be empty
        stages = -(-K // 128)
        n_splits = -(-stages // -(-stages // min(n_splits, stages)))
    n_splits = max(1, min(n_splits, -(-K // 64)))
    if (swiglu or relu_sq) and n_splits != 1:
        raise KernelError("gemm_tcgen05: an epilogue with an activation takes no K split")
    raw = partials_ok and n_splits > 1
    if n_splits > 1:
        need = n_splits * M * N
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=x.device)
        if scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"gemm_tcgen05: scratch of {scratch.numel()} floats, {need} needed")
    ldy, y_f32 = n_out, 0
    if not raw:
        _need(out, "gemm output", ndim=2)
        ldy = _rows_contiguous(out, "gemm output")
        if out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"gemm_tcgen05: output {tuple(out.shape)} {out.dtype} does not fit [{M}, {n_out}]")
        y_f32 = 1 if out.dtype == torch.float32 else 0
    fn = _fn("gemm_tcgen05", "lgml_gemm_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _check("gemm_tcgen05", fn(_ptr(x), _ptr(w), _ptr(bias), _ptr(None if raw else out), y_f32, M, N, K, ldx, ldw, ldy,
                              n_splits, _ptr(scratch if n_splits > 1 else None), 1 if swiglu else (2 if relu_sq else 0), 0 if raw else 1, _ptr(status),
                              _stream()), "gemm_tcgen05")
    if raw:
        return Partials(scratch[: n_splits * M * N].view(n_splits, M, N), bias)
    return out


def gemm_cublas(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The library product (the reference engine's matrix products are a library's too)."""
    if bias is None and out_dtype == torch.bfloat16:
        return torch.mm(x, w.t())
    y = torch.mm(x, w.t(), out_dtype=torch.float32)
    if bias is not None:
        y += bias
    return y if out_dtype == torch.float32 else y.to(out_dtype)


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None,
              backend: str = "auto", status: Optional[torch.Tensor] = None, partials_ok: bool = False):
    """y[M,N] = x[M,K] . w[N,K]^T (+ bias) with bfloat16 operands and float32 accumulation;
    y is bfloat16 or float32.  ``backend``: "tcgen05" is the hand-written tensor-core kernel,
    "cublas" the library product; "auto" takes tcgen05 whenever its operands fit TMA's
    alignment rules.  With ``partials_ok`` the result may be ``Partials``."""
    _need(x, "gemm input", torch.bfloat16, 2)
    _need(w, "gemm weight", torch.bfloat16, 2)
    if x.shape[1] != w.shape[1]:
        raise KernelError(f"gemm_bf16: shapes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if x.shape[0] == 0:
        return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
    if backend == "cublas" or (backend == "auto" and not tcgen05_supports(x, w)):
        return gemm_cublas(x, w, out_dtype, bias)
    if backend not in ("auto", "tcgen05"):
        raise KernelError(f"unknown gemm backend '{backend}'")
    if status is None:
        raise KernelError("gemm_bf16: the tcgen05 kernel needs the status word")
    n_splits = tcgen05_splits(x.shape[0], w.shape[0], x.shape[1])
    if partials_ok and n_splits > 1:          # the partial sums are the result: no output to make
        return gemm_tcgen05(x, w, None, bias, status, n_splits=n_splits, partials_ok=True, checked=True)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    return gemm_tcgen05(x, w, out, bias, status, n_splits=n_splits, checked=True)


def gemm_bf16_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, bias_pairs: Optional[torch.Tensor], status: torch.Tensor) -> torch.Tensor:
    """act[M, F] = silu(x . gate^T) * (x . up^T) in one kernel; ``w_pairs`` [2F, K] holds the
    gate and up rows of each feature next to each other (gate first)."""
    out = torch.empty((x.shape[0], w_pairs.shape[0] // 2), dtype=torch.bfloat16, device=x.device)
    if x.shape[0] == 0:
        return out
    return gemm_tcgen05(x, w_pairs, out, bias_pairs, status, swiglu=True)


GLU_CLAMPED_FUSED = os.environ.get("LGML_GLU_FUSED") != "0"     # the clamped gated activation in the product's epilogue


def gemm_bf16_glu_clamped(x: torch.Tensor, w_pairs: torch.Tensor, alpha: float, limit: float, status: torch.Tensor) -> torch.Tensor:
    """act[M, F] = g sigmoid(alpha g) (u + 1) with g = min(x . gate^T, limit), u = clamp(x . up^T, -limit, limit), in one
    kernel; ``w_pairs`` [2F, K] holds the gate and up rows of each feature next to each other (gate first)."""
    _need(x, "gemm input", torch.bfloat16, 2)
    _need(w_pairs, "gemm weight", torch.bfloat16, 2)
    ldx, ldw = _rows_contiguous(x, "gemm input"), _rows_contiguous(w_pairs, "gemm weight")
    M, K = x.shape
    N = w_pairs.shape[0]
    if w_pairs.shape[1] != K or N % 2:
        raise KernelError(f"gemm_bf16_glu_clamped: shapes disagree: x {tuple(x.shape)}, w {tuple(w_pairs.shape)}")
    out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
    if M == 0:
        return out
    fn = _fn("gemm_tcgen05", "lgml_gemm_tcgen05_glu_clamped", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                               c_float, c_void_p, c_void_p])
    _check("gemm_tcgen05", fn(_ptr(x), _ptr(w_pairs), _ptr(out), 0, M, N, K, ldx, ldw, out.stride(0), float(alpha), float(limit), _ptr(status),
                              _stream()), "gemm_tcgen05_glu_clamped")
    return out


def gemm_bf16_relu_sq(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], status: torch.Tensor) -> torch.Tensor:
    """act[M, F] = relu(x . w^T + bias)^2 in one kernel (bfloat16 in and out)."""
    out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
    if x.shape[0] == 0:
        return out
    return gemm_tcgen05(x, w, out, bias, status, relu_sq=True)


_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count if torch.cuda.is_available() else 148
    return _sm_count


def decode_splits(n_tokens: int, n_kv_heads: int, group: int, max_kv_len: int, page: int = 64) -> int:
    """How many ranges the keys of a token are cut into.  A range costs its CTA's start and its
    share of the merge whatever its length, so: at least four pages a range; as many CTAs as fill
    the SMs twice over, or once over while there are few of them to begin with and the context is
    short (one or two requests up to 4,096 tokens: the step waits for the slowest CTA, not for
    bandwidth); and no more than 16 ranges, or a 16th of the pages where that is more (the merge
    reads every range of a head).  Measured with `kernel_bench decode_attention`, 32 heads on 8 KV
    heads of 128, merge included: one request at 2,176 tokens 10.2 us with 9 ranges, 8.6 with 16,
    9.6 with 18; at 8,192 tokens 13.8 us with 16, 15.7 with 37; at 32,768 tokens 38.3 us with 16,
    31.7 with 37; two requests at 2,176 tokens 9.7 us with 9, 11.1 with 16, at 8,192 tokens 18.6 us
    with 16, 21.1 with 9 or 18; eight requests 18.4 us
    with 4 ranges, 21.8 with 3, 23.4 with 5."""
    ctas = max(n_tokens * n_kv_heads * ((group + 7) // 8), 1)
    pages = max(1, -(-max_kv_len // page))
    per_sm = 1 if ctas <= 16 and pages <= 64 else 2
    return max(1, min(-(-pages // 4), (per_sm * sm_count()) // ctas, max(16, pages // 16), 512))


def decode_attention(q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                     k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                     status: torch.Tensor, n_splits: int, scratch: Optional[torch.Tensor] = None, max_new_tokens: int = 16) -> torch.Tensor:
    """bfloat16 split-KV attention: each token over its request's cells.  Scratch (float32,
    ``decode_attention_scratch_floats`` elements) is needed when n_splits > 1.
    ``max_new_tokens``: the most tokens one request brings in this step (the kernel starts
    fetching older pages before the kernels ahead of it have finished)."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", torch.bfloat16, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    _need(positions, "positions", torch.int32, 1)
    _need(seq_of_token, "request index of tokens", torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d):
        raise KernelError(f"decode_attention: q {tuple(q.shape)} / out {tuple(out.shape)} do not fit {n_heads} heads of {d}")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous() or v_pages.shape != k_pages.shape:
        raise KernelError("decode_attention: pages and block table must be contiguous")
    if n_splits > 1:
        need = n * n_heads * n_splits * (d + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32, 1)
        if scratch.numel() < need:
            raise KernelError(f"decode_attention: scratch of {scratch.numel()} floats, {need} needed")
    fn = _fn("attention_decode", "lgml_decode_attention", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                                           c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p])
    _check("attention_decode", fn(_ptr(q), ldq, _ptr(positions), _ptr(seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(k_pages),
                                  _ptr(v_pages), n_pages, page, _ptr(out), ldo, _ptr(scratch if n_splits > 1 else None), n_splits, n, n_heads, hkv, d,
                                  float(scale), int(window or 0), int(max_new_tokens), _ptr(status), _stream()), "decode_attention")
    return out


def prefill_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per tile of the prefill attention kernel for this grouping of heads."""
    hpc = min(n_heads // n_kv_heads, 8)
    return 16 * (8 // hpc)


def _prefill_attention_call(library: str, symbol: str, label: str, q, positions, tiles, block_table, k_pages, v_pages, out, n_heads, scale,
                            window, status) -> torch.Tensor:
    """The checks and the call that the three prefill attention kernels share (one signature)."""
    _need(q, "queries", torch.bfloat16, 2)
    _need(out, "attention output", torch.bfloat16, 2)
    ldq, ldo = _rows_contiguous(q, "queries"), _rows_contiguous(out, "attention output")
    n = q.shape[0]
    _need(k_pages, "key pages", torch.bfloat16, 4)
    _need(v_pages, "value pages", torch.bfloat16, 4)
    n_pages, hkv, page, d = k_pages.shape
    _need(positions, "positions", torch.int32, 1)
    _need(tiles, "tiles", torch.int32, 2)
    _need(block_table, "block table", torch.int32, 2)
    if q.shape[1] != n_heads * d or out.shape != (n, n_heads * d) or tiles.shape[1] != 4:
        raise KernelError(f"{label}: q {tuple(q.shape)} / out {tuple(out.shape)} / tiles {tuple(tiles.shape)} do not fit")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous() or not tiles.is_contiguous():
        raise KernelError(f"{label}: pages, block table and tiles must be contiguous")
    fn = _fn(library, symbol, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                               c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    _check(library, fn(_ptr(q), ldq, _ptr(positions), _ptr(tiles), tiles.shape[0], _ptr(block_table), block_table.shape[1],
                       _ptr(k_pages), _ptr(v_pages), n_pages, page, _ptr(out), ldo, n_heads, hkv, d, float(scale),
                       int(window or 0), _ptr(status), _stream()), label)
    return out


def prefill_attention(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                      k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                      status: torch.Tensor) -> torch.Tensor:
    """bfloat16 tensor-core attention for prompts and portions (``mma.sync``).  ``tiles`` is int32
    [n_tiles, 4]: (request row, first token row, tokens, 0), each tile within one request
    and at most ``prefill_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill", "lgml_prefill_attention", "prefill_attention", q, positions, tiles, block_table,
                                   k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_tc_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per tile of the tcgen05 prefill attention kernel: 128 rows / heads per CTA."""
    return 128 // min(n_heads // n_kv_heads, 8)


def prefill_attention_tc(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                         k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                         status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention for prompts and portions on tcgen05 tensor cores (S and the page's
    output in tensor memory), one tile of 128 rows per CTA.  ``tiles`` as for
    ``prefill_attention``, each at most ``prefill_tc_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill_tc", "lgml_prefill_attention_tc", "prefill_attention_tc", q, positions, tiles,
                                   block_table, k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_twin_tile_tokens(n_heads: int, n_kv_heads: int) -> int:
    """Tokens per CTA of the two-tile tcgen05 prefill attention kernel: 2 x (128 rows / heads per CTA)."""
    return 2 * (128 // min(n_heads // n_kv_heads, 8))


def prefill_attention_twin(q: torch.Tensor, positions: torch.Tensor, tiles: torch.Tensor, block_table: torch.Tensor,
                           k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, n_heads: int, scale: float, window: int,
                           status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention for prompts and portions on tcgen05 tensor cores, two tiles of 128
    rows per CTA (scores, P and the output in tensor memory), for head sizes 64 and 128.
    ``tiles`` as for ``prefill_attention``, each at most ``prefill_twin_tile_tokens`` long."""
    return _prefill_attention_call("attention_prefill_twin", "lgml_prefill_attention_twin", "prefill_attention_twin", q, positions, tiles,
                                   block_table, k_pages, v_pages, out, n_heads, scale, window, status)


def prefill_tc_supports(q: torch.Tensor, out: torch.Tensor) -> bool:
    """The tcgen05 kernel reads q and writes out in 16-byte pieces."""
    return q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0


# which kernel runs prompts and portions: "tcgen05" (default: two tiles per CTA for head sizes 64
# and 128, one tile otherwise), "single" (one tile per CTA for every head size) or "mma" (the
# mma.sync kernel)
PREFILL_ATTENTION = os.environ.get("LGML_PREFILL_ATTENTION", "tcgen05")

# a portion of at most this many tokens per request is run by the decode kernel
DECODE_MAX_Q = 8


def paged_attention(q, batch, cache, out, n_heads: int, scale: float, window: int, status: torch.Tensor) -> torch.Tensor:
    """bfloat16 attention over the paged cache; picks the kernel by the batch's shape: the
    split-KV kernel when every request brings a few tokens, the tensor-core kernel for
    prompts and portions (head sizes up to 128), the general kernel otherwise."""
    d = cache.k.shape[3]
    hkv = cache.k.shape[1]
    if cache.k.shape[2] == 64 and d % 16 == 0:
        if batch.max_q_len <= DECODE_MAX_Q:
            n_splits = batch.decode_splits if getattr(batch, "decode_splits", None) else decode_splits(q.shape[0], hkv, n_heads // hkv, batch.max_kv_len)
            return decode_attention(q, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, out, n_heads, scale,
                                    window, status, n_splits, max_new_tokens=batch.max_q_len)
        if d in (64, 128) and PREFILL_ATTENTION == "tcgen05" and prefill_tc_supports(q, out):
            tiles = batch.attention_tiles(prefill_twin_tile_tokens(n_heads, hkv))
            return prefill_attention_twin(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
        if d <= 128 and PREFILL_ATTENTION in ("tcgen05", "single") and prefill_tc_supports(q, out):
            tiles = batch.attention_tiles(prefill_tc_tile_tokens(n_heads, hkv))
            return prefill_attention_tc(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
        if d <= 128:
            tiles = batch.attention_tiles(prefill_tile_tokens(n_heads, hkv))
            return prefill_attention(q, batch.positions, tiles, cache.block_table, cache.k, cache.v, out, n_heads, scale, window, status)
    return paged_attention_ref(q, batch.positions, batch.seq_of_token, cache.block_table, cache.k, cache.v, out, n_heads,
                               scale, window, status)
