"""Python face of the CUDA kernels: checks on the host, then one C call.

Every function here validates what the kernel cannot (device, dtype, layout,
size limits) and raises a clear error instead of launching; the launchers
return an error code for what they refuse themselves.  There is no CPU path
and no library stand-in: a tensor that is not on a CUDA device is an error.

Matrix products are the exception the engine shares with the reference, which
also leaves them to a library (`F.linear`, python/logssms/layers/linear.py:26):
bfloat16 products go to cuBLAS through torch, float32 products to the engine's
own FFMA kernel so that no reduced-precision matrix mode can take part.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build
from .fusion import NormedRows, ResidualJoin, ScaledRows, SummedRows      # the fusion protocol (re-exported here)
from .profiler import PROFILER

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_ERRORS = {-1: "dtype is neither float32 nor bfloat16", -2: "a size the kernel does not take",
           -3: "a size beyond the kernel's limit"}
_fn_cache: dict[tuple[str, str], ctypes._CFuncPtr] = {}
launch_count = 0        # kernels of this package launched so far (a launcher adds what it launches)


class KernelError(RuntimeError):
    pass


def _fn(lib: str, name: str, argtypes):
    key = (lib, name)
    f = _fn_cache.get(key)
    if f is None:
        f = getattr(build.load(lib), name)
        f.argtypes = argtypes
        f.restype = c_int
        _fn_cache[key] = f
    if PROFILER.enabled:                  # opt-in: every launch between two events, summed per kernel class
        return lambda *args: PROFILER.timed(lib, name, lambda: f(*args))
    return f


def _check(code: int, name: str, detail: str = "", launches: int = 1) -> None:
    global launch_count
    if code == 0:
        launch_count += launches
        return
    if code < 0:
        raise KernelError(f"{name} refused the call: {_ERRORS.get(code, code)} {detail}")
    raise KernelError(f"{name}: CUDA error {code} at launch {detail}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """Raw handle of torch's current stream on the current device (the C call: the Python `Stream` object
    costs microseconds, and every launch asks)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}: the kernels take float32 and bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("logssms_b200 kernels run on CUDA tensors only; there is no CPU path")


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


# --------------------------------------------------------------------------- embedding
def embed_gather(table: torch.Tensor, ids: torch.Tensor, multiplier: float,
                 bad_ids: torch.Tensor | None = None) -> torch.Tensor:
    _cuda(table, ids)
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous [vocab, hidden] matrix")
    V, H = table.shape
    out = torch.empty((ids.numel(), H), dtype=table.dtype, device=table.device)
    f = _fn("embed", "lb_embed_gather", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                                         c_int, c_void_p])
    _check(f(_ptr(out), _ptr(table), _ptr(ids), ids.numel(), H, V, multiplier, _ptr(bad_ids), _code(table),
             _stream()), "embed_gather")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _cuda(src, rows)
    _i32(rows, "rows")
    _need(src.dim() == 2 and src.is_contiguous(), "gather_rows wants a contiguous matrix")
    out = torch.empty((rows.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
    f = _fn("embed", "lb_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(out), _ptr(src), _ptr(rows), rows.numel(), src.shape[1], _code(src), _stream()), "gather_rows")
    return out


# --------------------------------------------------------------------------- norms
def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None, *,
                other: torch.Tensor | None = None, in_scales=(1.0, 1.0), out_scales=(1.0,),
                want_residual: bool = True, residual_out: torch.Tensor | None = None, in_place: bool = True):
    """(outputs, new_residual): residual add + RMSNorm with one or two scaled outputs.
    The new residual is written in place of `residual` when one is given, unless `in_place` is off
    (then into `residual_out`, or a new tensor)."""
    _cuda(x, weight, residual, other)
    _need(x.dim() == 2 and x.is_contiguous(), "add_rmsnorm wants a contiguous [rows, width] input")
    rows, H = x.shape
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(),
          "norm weight must be a contiguous float32 vector of the row width")
    for t, name in ((residual, "residual"), (other, "other")):
        if t is not None:
            _need(t.shape == x.shape and t.dtype == x.dtype and t.is_contiguous(), f"{name} must match the input")
    _need(1 <= len(out_scales) <= 2, "one or two outputs")
    out0 = torch.empty_like(x)
    out1 = torch.empty_like(x) if len(out_scales) == 2 else None
    if in_place:
        res_out = residual if residual is not None else (torch.empty_like(x) if want_residual else None)
    else:
        res_out = (residual_out if residual_out is not None else torch.empty_like(x)) if want_residual else None
    f = _fn("norm", "lb_add_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(other), _ptr(residual), _ptr(res_out), _ptr(weight), _ptr(out0), _ptr(out1), rows, H,
             eps, in_scales[0], in_scales[1], out_scales[0], out_scales[-1], _code(x), _stream()),
           "add_rmsnorm", f"(width {H})")
    return ((out0,) if out1 is None else (out0, out1)), res_out


GATE_ONLY, NORM_BEFORE_GATE, NORM_AFTER_GATE = 0, 1, 2


def gated_rmsnorm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, eps: float, groups: int,
                  gate_scale: float, mode: int) -> torch.Tensor:
    """Grouped RMSNorm with SiLU gate (`mode` NORM_BEFORE_GATE / NORM_AFTER_GATE) or the bare
    y * silu(gate) product (`GATE_ONLY`).  `gate` may be a column view of a wider matrix."""
    _cuda(y, gate, weight)
    _need(y.dim() == 2 and y.is_contiguous(), "gated_rmsnorm wants a contiguous [rows, width] input")
    rows, width = y.shape
    _need(gate.shape == y.shape and gate.dtype == y.dtype and gate.stride(1) == 1, "gate must match y, unit column stride")
    _need(width % groups == 0, "width must be a multiple of groups")
    if mode != GATE_ONLY:
        _need(weight is not None and weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(),
              "gated norm weight must be a contiguous float32 vector of the row width")
    out = torch.empty_like(y)
    f = _fn("norm", "lb_gated_rmsnorm", [c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int,
                                         c_float, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(y), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), rows, width // groups, groups, eps,
             gate_scale, mode, _code(y), _stream()), "gated_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, act_scale: float) -> torch.Tensor:
    _cuda(gate_up)
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0,
          "swiglu wants a contiguous [rows, 2*I] matrix")
    rows, two_i = gate_up.shape
    out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    f = _fn("norm", "lb_swiglu", [c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p])
    _check(f(_ptr(gate_up), _ptr(out), rows, two_i // 2, act_scale, _code(gate_up), _stream()), "swiglu")
    return out


def scale(x: torch.Tensor, s: float, to_f32: bool = False) -> torch.Tensor:
    """round(x * s) in x's dtype, or float32(x) * s with `to_f32`."""
    _cuda(x)
    _need(x.is_contiguous(), "scale wants a contiguous tensor")
    out = torch.empty(x.shape, dtype=torch.float32 if to_f32 else x.dtype, device=x.device)
    f = _fn("norm", "lb_scale", [c_void_p, c_void_p, c_long, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(x), _ptr(out), x.numel(), s, int(to_f32), _code(x), _stream()), "scale")
    return out


# --------------------------------------------------------------------------- rotary + cache store
def rope_table(inv_freq: torch.Tensor, rows: int) -> torch.Tensor:
    """[rows, 2*half] float32: cos | sin of position * inv_freq."""
    _cuda(inv_freq)
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be contiguous float32")
    half = inv_freq.numel()
    table = torch.empty((rows, 2 * half), dtype=torch.float32, device=inv_freq.device)
    f = _fn("rope", "lb_rope_table", [c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(_ptr(table), _ptr(inv_freq), rows, half, _stream()), "rope_table")
    return table


def rope_kv_store(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                  slot_mapping: torch.Tensor, cos_sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  key_scale: float, write_kv: bool = True) -> torch.Tensor:
    """qkv: [tokens, (Hq + 2*Hkv) * head_dim], columns q | k | v (row stride free).  Returns the rotated
    queries [tokens, Hq, head_dim]; stores scaled+rotated keys and the values at `slot_mapping` (token
    index in the page pool) unless `write_kv` is off."""
    _cuda(qkv, positions, slot_mapping, cos_sin, k_cache, v_cache)
    Hq, Hkv, hd = num_heads, num_kv_heads, head_dim
    tokens = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.shape[1] == (Hq + 2 * Hkv) * hd and qkv.stride(1) == 1,
          "qkv must be [tokens, (Hq + 2*Hkv) * head_dim] with unit column stride")
    _i32(positions, "positions")
    _i32(slot_mapping, "slot_mapping")
    _need(positions.numel() == tokens and slot_mapping.numel() == tokens, "one position and one slot per token")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 2,
          "cos/sin table must be contiguous float32 [positions, rotary_dim]")
    rotary_dim = cos_sin.shape[1]
    _need(rotary_dim % 2 == 0 and rotary_dim <= hd, f"rotary_dim {rotary_dim} must be even and within head_dim {hd}")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == qkv.dtype == v_cache.dtype
          and k_cache.shape[-2:] == (Hkv, hd) and v_cache.shape == k_cache.shape,
          "k/v cache must be contiguous [..., kv_heads, head_dim] of the activation dtype")
    q_out = torch.empty((tokens, Hq, hd), dtype=qkv.dtype, device=qkv.device)
    row_stride = qkv.stride(0) if tokens > 1 else qkv.shape[1]
    base = qkv.data_ptr()
    item = qkv.element_size()
    f = _fn("rope", "lb_rope_kv_store", [c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int,
                                         c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                         c_int, c_int, c_void_p])
    _check(f(base, base + Hq * hd * item, base + (Hq + Hkv) * hd * item, row_stride, _ptr(positions),
             _ptr(slot_mapping), _ptr(cos_sin), cos_sin.shape[0], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), tokens,
             Hq, Hkv, hd, rotary_dim, key_scale, int(write_kv), _code(qkv), _stream()), "rope_kv_store")
    return q_out


# --------------------------------------------------------------------------- attention
def attention_splits(num_tokens: int, num_heads: int, num_kv_heads: int, max_context: int) -> int:
    """How many ranges each context is cut into so that the grid covers the SMs a few times over."""
    G = num_heads // num_kv_heads
    tile = 8 if G >= 8 else (4 if G > 2 else G)
    items = max(1, num_tokens * num_kv_heads * (-(-G // tile)))
    return max(1, min(_SPLIT_TARGET_CTAS // items, -(-max_context // 64), 256))


_SPLIT_TARGET_CTAS = 592        # 4 CTAs on each of the 148 SMs


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     token_req: torch.Tensor, positions: torch.Tensor, scale: float, window: int = 0, *,
                     splits: int = 1, token_list: torch.Tensor | None = None, out: torch.Tensor | None = None,
                     scratch: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """Split-KV attention, each token on its own over its request's pages.  q: [tokens, Hq, hd]; caches:
    [pages, page_size, Hkv, hd]; block_table: [requests, max_pages] int32; token_req / positions: per token its
    request row and absolute position.  Returns [tokens, Hq, hd].  `token_list` (int32) restricts the call to those tokens; the other rows of `out`
    are left as they are.  `scratch`: float32 buffers (>= tokens*Hq*splits*hd and >= tokens*Hq*splits*2
    elements) for the ranges' partial results; allocated here when missing."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, token_list)
    tokens, Hq, hd = q.shape
    _need(q.is_contiguous(), "q must be contiguous")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == q.dtype == v_cache.dtype and k_cache.shape[3] == hd,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(token_req, "token_req")
    _i32(positions, "positions")
    sel = tokens
    if token_list is not None:
        _i32(token_list, "token_list")
        sel = token_list.numel()
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    part_o = part_ml = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(sel * Hq * splits * hd, dtype=torch.float32, device=q.device),
                       torch.empty(sel * Hq * splits * 2, dtype=torch.float32, device=q.device))
        part_o, part_ml = scratch
        _need(part_o.dtype == torch.float32 == part_ml.dtype and part_o.numel() >= sel * Hq * splits * hd
              and part_ml.numel() >= sel * Hq * splits * 2, "attention scratch is too small or not float32")
    f = _fn("attention_decode", "lb_attention_decode",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(token_req), _ptr(positions), _ptr(token_list), sel, Hq, Hkv, hd, page_size, scale, int(window or 0),
             int(splits), _ptr(part_o), _ptr(part_ml), _code(q), _stream()), "attention_decode",
           launches=2 if splits > 1 else 1)
    return out


_decode_counters: dict[torch.device, torch.Tensor] = {}


def _counters_for(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed int32 counters kept per device; the fused decode kernel leaves them at zero."""
    t = _decode_counters.get(device)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
        _decode_counters[device] = t
    return t


def decode_step_splits(num_tokens: int, num_heads: int, num_kv_heads: int, max_context: int, listed: bool = False,
                       head_dim: int = 64) -> int:
    """Most key ranges per token for `attention_decode_step` (about one CTA per SM with heads of up to 64, about two
    with larger ones) or, `listed`, for `attention_decode_listed` (about two), never more ranges than 256-key pieces of
    the longest context (the kernel itself uses fewer ranges for a short context)."""
    G = num_heads // num_kv_heads
    tile = 8 if G >= 8 else (4 if G > 2 else G)
    items = max(1, num_tokens * num_kv_heads * (-(-G // tile)))
    target = _WIDE_TARGET_CTAS if (listed or head_dim > 64) else _STEP_TARGET_CTAS
    splits = max(1, min(target // items, -(-max_context // 256), 256))
    # up to 8 ranges are the CTAs of one cluster and merge through distributed shared memory (about 2 us off the
    # kernel); with a dozen (token, head) items that many ranges fill the GPU, so more would only cost that path
    return min(splits, 8) if items >= 12 else splits


# Heads of up to 64: about one CTA per SM.  Up to 9 tokens the 256-key pieces of the context set the number of ranges,
# not this; from 10 tokens on fewer, longer ranges win, the more so beside the state update that shares the SMs:
# 36-layer decode steps over 2,048-key contexts (head 64) with 296 / 160 took 1.66 / 1.62 ms at batch 16, 1.92 / 1.90 ms
# at 32, 2.56 / 2.39 ms at 64 (444: 2.68 ms).
_STEP_TARGET_CTAS = 160
# Heads of 128 (a CTA's chain per key is twice as long), and the listed rows of a step that also holds a prompt portion
# (the last link of the attention branch, with little beside them): shorter ranges win.  16 layers of 1.5B-Deep size
# (head 128) with 296 / 160: 1.38 / 1.42 ms at batch 24, 1.52 / 1.62 ms at 32; the 1.5B-Deep serving run 2,220 / 1,970
# generated tok/s; 64 tokens of 4,096 keys at 7B size (one range either way): no difference.
_WIDE_TARGET_CTAS = 296


def attention_decode_step(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                          slot_mapping: torch.Tensor, cos_sin: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, token_req: torch.Tensor, scale: float, key_scale: float,
                          window: int = 0, write_kv: bool = True, *, splits: int = 1) -> torch.Tensor:
    """The whole attention of a decode step in one launch: every row of `qkv` ([tokens, (Hq + 2 Hkv) * hd],
    columns q | k | v) is the only new token of its request.  Rotates q and the new key, stores the new
    key/value at `slot_mapping` (unless `write_kv` is off: then the position was stored by another layer
    and is read from the cache), attends over the request's pages and merges the key ranges.
    Returns [tokens, Hq, hd]."""
    _cuda(qkv, positions, slot_mapping, cos_sin, k_cache, v_cache, block_table, token_req)
    Hq, Hkv, hd = num_heads, num_kv_heads, head_dim
    tokens = qkv.shape[0]
    _need(qkv.dim() == 2 and qkv.shape[1] == (Hq + 2 * Hkv) * hd and qkv.stride(1) == 1,
          "qkv must be [tokens, (Hq + 2*Hkv) * head_dim] with unit column stride")
    for t_, n_ in ((positions, "positions"), (slot_mapping, "slot_mapping"), (token_req, "token_req")):
        _i32(t_, n_)
        _need(t_.numel() == tokens, f"one entry of {n_} per token")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.dim() == 2,
          "cos/sin table must be contiguous float32 [positions, rotary_dim]")
    rotary_dim = cos_sin.shape[1]
    _need(rotary_dim % 2 == 0 and rotary_dim <= hd, f"rotary_dim {rotary_dim} must be even and within head_dim {hd}")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == qkv.dtype == v_cache.dtype and k_cache.shape[2:] == (Hkv, hd),
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of the activation dtype")
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    page_size = k_cache.shape[1]
    out = torch.empty((tokens, Hq, hd), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = counters = None
    splits = int(splits)
    if splits > 1:
        part_o = torch.empty(tokens * Hq * splits * hd, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(tokens * Hq * splits * 2, dtype=torch.float32, device=qkv.device)
        counters = _counters_for(qkv.device, tokens * Hq)
    row_stride = qkv.stride(0) if tokens > 1 else qkv.shape[1]
    f = _fn("attention_decode_fused", "lb_attention_decode_fused",
            [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_long, c_void_p, c_int, c_void_p])
    _check(f(_ptr(qkv), row_stride, _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(token_req), _ptr(positions), _ptr(slot_mapping), _ptr(cos_sin), cos_sin.shape[0], rotary_dim, tokens,
             Hq, Hkv, hd, page_size, scale, key_scale, int(window or 0), int(write_kv), splits, _ptr(part_o),
             _ptr(part_ml), _ptr(counters), k_cache.shape[0], _ptr(error_word(qkv.device)), _code(qkv), _stream()),
           "attention_decode_step")
    return out


def attention_decode_listed_ok(q: torch.Tensor, k_cache: torch.Tensor) -> bool:
    """Does `attention_decode_listed` take these operands (bfloat16, head size up to 128, at most 16 query heads per
    key/value head)?  Else `attention_decode`."""
    return (q.dtype == torch.bfloat16 and q.dim() == 3 and k_cache.dim() == 4 and q.shape[2] <= 128 and q.shape[2] % 16 == 0
            and q.shape[1] % k_cache.shape[2] == 0 and q.shape[1] // k_cache.shape[2] <= 16 and q.is_contiguous())


def attention_decode_listed(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            token_req: torch.Tensor, positions: torch.Tensor, token_list: torch.Tensor, count: int,
                            scale: float, window: int = 0, *, splits: int = 1, out: torch.Tensor | None = None) -> torch.Tensor:
    """The decode-step attention kernel (tensor-core form: the query heads of a key/value head as one tile, key ranges
    merged through the cluster's shared memory) for `count` listed rows of a step that holds prompt portions as well.
    q [rows, Hq, hd]: rotated queries; every key and value, the rows' own included, is in the cache already.  Rows of
    `out` that are not listed are left as they are."""
    _cuda(q, k_cache, v_cache, block_table, token_req, positions, token_list, out)
    _need(attention_decode_listed_ok(q, k_cache), "attention_decode_listed takes bfloat16, head sizes up to 128, groups up to 16")
    rows, Hq, hd = q.shape
    _need(k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape and k_cache.dtype == q.dtype
          == v_cache.dtype and k_cache.shape[3] == hd, "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    for t_, n_ in ((token_req, "token_req"), (positions, "positions"), (token_list, "token_list")):
        _i32(t_, n_)
    _need(token_list.numel() >= count and token_req.numel() == rows == positions.numel(), "one entry per row; a list of `count` rows")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    part_o = part_ml = counters = None
    splits = int(splits)
    if splits > 1:
        part_o = torch.empty(count * Hq * splits * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(count * Hq * splits * 2, dtype=torch.float32, device=q.device)
        counters = _counters_for(q.device, count * Hq)
    f = _fn("attention_decode_fused", "lb_attention_decode_listed",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0), _ptr(token_req),
             _ptr(positions), _ptr(token_list), count, Hq, Hkv, hd, page_size, scale, int(window or 0), splits, _ptr(part_o),
             _ptr(part_ml), _ptr(counters), k_cache.shape[0], _ptr(error_word(q.device)), _stream()), "attention_decode_listed")
    return out


def attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, start_pos: torch.Tensor, tiles: torch.Tensor, num_tiles: int,
                      scale: float, window: int = 0, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention for prompt portions (bfloat16).  `tiles`: int32 [n, 2] = (request index,
    first token of a 64-token tile within that request's portion).  Rows of `out` that no tile covers
    are left as they are.  Other arguments as for `attention_decode`."""
    _cuda(q, k_cache, v_cache, block_table, cu_seqlens, start_pos, tiles)
    tokens, Hq, hd = q.shape
    _need(q.dtype == torch.bfloat16, "attention_prefill is the bfloat16 kernel; float32 runs the general kernel")
    _need(q.is_contiguous(), "q must be contiguous")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.shape == k_cache.shape
          and k_cache.dtype == q.dtype == v_cache.dtype and k_cache.shape[3] == hd,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    page_size, Hkv = k_cache.shape[1], k_cache.shape[2]
    _need(hd % 16 == 0 and hd <= 256, f"attention takes head sizes in steps of 16 up to 256, got {hd}")
    _need(Hq % Hkv == 0, f"query heads ({Hq}) must be a multiple of key/value heads ({Hkv})")
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(start_pos, "start_pos")
    _i32(tiles, "tiles")
    _need(tiles.numel() >= 2 * num_tiles, "tiles holds fewer pairs than num_tiles")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    f = _fn("attention_prefill", "lb_attention_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_float, c_int, c_int, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), block_table.stride(0),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(tiles), num_tiles, Hq, Hkv, hd, page_size, scale,
             int(window or 0), _code(q), _stream()), "attention_prefill")
    return out


ATTENTION_TILE = 64        # query tokens per CTA of the prefill kernel
ATTENTION_TC_TILE = 128    # and of its tcgen05 form
ATTENTION_TC = os.environ.get("LOGSSMS_B200_ATTN_TC", "1") != "0"


def attention_prefill_tc_ok(q: torch.Tensor, k_cache: torch.Tensor) -> bool:
    """Does the tcgen05 prompt-attention kernel take these operands (bfloat16, head size 64 or 128, pages of a
    multiple of 64 tokens)?  Else `attention_prefill`."""
    return (ATTENTION_TC and q.dtype == torch.bfloat16 and q.dim() == 3 and q.shape[2] in (64, 128) and k_cache.dim() == 4
            and k_cache.shape[1] % 64 == 0 and k_cache.shape[3] == q.shape[2] and q.shape[1] % k_cache.shape[2] == 0
            and q.is_contiguous() and k_cache.is_contiguous())


def prefill_splits(num_tiles: int, num_heads: int, max_context: int) -> int:
    """Key ranges per 128-query tile for `attention_prefill_tc`: a step of few tiles over a long context (a prompt
    portion far into its prompt) would leave most SMs idle with one CTA per (tile, head), so the keys are shared out
    until the grid fills the SMs, each range keeping at least 512 keys."""
    items = max(1, num_tiles * num_heads)
    return max(1, min(_SM_COUNT // items, max_context // 512, 16))


_SM_COUNT = 148


def attention_prefill_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, start_pos: torch.Tensor, tiles: torch.Tensor, num_tiles: int,
                         scale: float, window: int = 0, *, out: torch.Tensor | None = None, splits: int = 1) -> torch.Tensor:
    """`attention_prefill` on the tcgen05 tensor cores: the same arguments, but `tiles` lists 128-token tiles.
    `splits` > 1 cuts every tile's keys into that many ranges, each a CTA of its own, merged by a second kernel.
    `check_kernel_errors()` reports a kernel whose internal wait gave up."""
    _cuda(q, k_cache, v_cache, block_table, cu_seqlens, start_pos, tiles)
    _need(attention_prefill_tc_ok(q, k_cache), "attention_prefill_tc takes bfloat16, head size 64 or 128 and pages of a multiple of 64 tokens")
    tokens, Hq, hd = q.shape
    _need(v_cache.shape == k_cache.shape and v_cache.is_contiguous() and v_cache.dtype == k_cache.dtype == q.dtype,
          "caches must be contiguous [pages, page_size, kv_heads, head_dim] of q's dtype")
    pages, page_size, Hkv = k_cache.shape[0], k_cache.shape[1], k_cache.shape[2]
    _need(block_table.dim() == 2 and block_table.dtype == torch.int32 and block_table.stride(1) == 1,
          "block table must be a row-major int32 matrix")
    _i32(cu_seqlens, "cu_seqlens")
    _i32(start_pos, "start_pos")
    _i32(tiles, "tiles")
    _need(tiles.numel() >= 2 * num_tiles, "tiles holds fewer pairs than num_tiles")
    if out is None:
        out = torch.empty_like(q)
    _need(out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous(), "out must match q")
    err = error_word(q.device)
    splits = max(1, int(splits))
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty(num_tiles * Hq * splits * ATTENTION_TC_TILE * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(num_tiles * Hq * splits * ATTENTION_TC_TILE * 2, dtype=torch.float32, device=q.device)
    f = _fn("attention_prefill_tc", "lb_attention_prefill_tc",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_long, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), tokens, pages, _ptr(block_table), block_table.stride(0),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(tiles), num_tiles, Hq, Hkv, hd, page_size, scale, int(window or 0),
             _ptr(err), splits, _ptr(part_o), _ptr(part_ml), _stream()), "attention_prefill_tc", launches=2 if splits > 1 else 1)
    return out


# --------------------------------------------------------------------------- Mamba2
def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor,
                  cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor, num_requests: int,
                  max_len: int, region_ends: tuple[int, int], region_scales: tuple[float, float, float]) -> torch.Tensor:
    """x: [tokens, C] (column view allowed); weight: [C, K] float32; state: [slots, C, K-1] of x's dtype,
    read then rewritten in place.  Returns silu(conv) as a contiguous [tokens, C]."""
    _cuda(x, weight, bias, state, cu_seqlens, start_pos, slots)
    tokens, C = x.shape
    K = weight.shape[1]
    _need(x.stride(1) == 1, "conv input needs unit column stride")
    _need(weight.dtype == torch.float32 and weight.shape == (C, K) and weight.is_contiguous(), "conv weight must be float32 [C, K]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (C,) and bias.is_contiguous()), "conv bias must be float32 [C]")
    _need(2 <= K <= 8, f"conv kernel sizes 2..8 are built, got {K}")
    _need(state.dtype == x.dtype and state.is_contiguous() and state.shape[1:] == (C, K - 1),
          "conv state must be contiguous [slots, C, K-1] of the activation dtype")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, n)
    out = torch.empty((tokens, C), dtype=x.dtype, device=x.device)
    f = _fn("conv", "lb_causal_conv1d", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                         c_float, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(state), _ptr(out), _ptr(cu_seqlens),
             _ptr(start_pos), _ptr(slots), num_requests, max_len, C, K, region_ends[0], region_ends[1],
             region_scales[0], region_scales[1], region_scales[2], _code(x), _stream()), "causal_conv1d",
           launches=1 if max_len <= 8 else 2)
    return out


def _ssm_state_ok(state: torch.Tensor, act: torch.dtype) -> bool:
    return state.is_contiguous() and (state.dtype == torch.float32 or (state.dtype == torch.bfloat16 == act))


def ssm_scan(conv: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
             state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
             num_requests: int, num_heads: int, head_dim: int, state_dim: int, num_groups: int,
             dt_scale: float, gate: torch.Tensor | None = None, gate_scale: float = 1.0, *,
             request_list: torch.Tensor | None = None, num_listed: int = 0,
             out: torch.Tensor | None = None, beside: bool = False) -> torch.Tensor:
    """conv: [tokens, nh*P + 2*G*N] (x | B | C; a column view is fine); dt: [tokens, nh] view; state: float32 (or,
    with bfloat16 activations, bfloat16: rounded once per call) [slots, nh, P, N], updated in place.  Returns y [tokens, nh*P]; with `gate` ([tokens, nh*P] view)
    the result is y * silu(gate * gate_scale), the gate of a mixer that has no norm.  `request_list`
    (int32 indices into the batch, `num_listed` of them) restricts the call to those requests; the rows
    of `out` that belong to other requests are left as they are.  `beside`: other kernels of the step run at the same
    time (on another stream): the launch then takes a grid that is resident at once and walks its items, instead of one
    CTA per item that would take every SM slot before them."""
    _cuda(conv, dt, A_log, dt_bias, D, state, cu_seqlens, start_pos, slots, gate, request_list, out)
    if request_list is not None:
        _i32(request_list, "request_list")
        _need(request_list.numel() >= num_listed, "request_list is shorter than num_listed")
        num_requests = num_listed
    if gate is not None:
        _need(gate.shape == (conv.shape[0], num_heads * head_dim) and gate.stride(1) == 1 and gate.dtype == conv.dtype,
              "gate must be a [tokens, heads * head_dim] view of the activation dtype")
    tokens, C = conv.shape
    _need(conv.stride(1) == 1, "conv output needs unit column stride")
    _need(dt.shape == (tokens, num_heads) and dt.stride(1) == 1 and dt.dtype == conv.dtype, "dt must be a [tokens, heads] view")
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (D, "D")):
        _need(t.dtype == torch.float32 and t.shape == (num_heads,) and t.is_contiguous(), f"{n} must be float32 [heads]")
    _need(_ssm_state_ok(state, conv.dtype) and state.shape[1:] == (num_heads, head_dim, state_dim),
          "SSM state must be contiguous float32 (or bfloat16 beside bfloat16 activations) [slots, heads, P, N]")
    _need(state_dim % 4 == 0 and state_dim <= 256, f"state sizes in steps of 4 up to 256 are built, got {state_dim}")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots")):
        _i32(t, n)
    y = out if out is not None else torch.empty((tokens, num_heads * head_dim), dtype=conv.dtype, device=conv.device)
    _need(y.shape == (tokens, num_heads * head_dim) and y.dtype == conv.dtype and y.is_contiguous(), "out must be [tokens, heads * head_dim]")
    f = _fn("ssm", "lb_ssm_scan", [c_void_p, c_int, c_long, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                   c_long, c_float, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(_ptr(conv), C, conv.stride(0) if tokens > 1 else C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D),
             _ptr(state), _ptr(y), _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), num_requests, num_heads, head_dim,
             state_dim, num_groups, dt_scale, _ptr(gate), gate.stride(0) if gate is not None else 0, gate_scale,
             _ptr(request_list), int(bool(beside)), int(state.dtype == torch.bfloat16), _code(conv), _stream()), "ssm_scan")
    return y


SSD_TC = os.environ.get("LOGSSMS_B200_SSD_TC", "1") != "0"
SSD_TC_CHUNK = 128


def ssd_chunk_scan_tc_ok(head_dim: int, state_dim: int, chunk_len: int) -> bool:
    """Does the tcgen05 chunk-scan kernel take these sizes (head size 64 or 128: the kernels that make the chunk
    states before it take no larger heads; state size 64..256 in steps of 64, chunks of 128 tokens)?"""
    return (SSD_TC and head_dim in (64, 128) and state_dim % 64 == 0 and 64 <= state_dim <= 256
            and chunk_len == SSD_TC_CHUNK)


def ssd_chunk_len(chunk_size: int, head_dim: int, state_dim: int) -> int:
    """Chunk length the tensor-core SSD kernels will use for these sizes (at most `chunk_size`), or 0
    when they do not take them (then the token-by-token scan runs everything)."""
    if chunk_size >= SSD_TC_CHUNK and ssd_chunk_scan_tc_ok(head_dim, state_dim, SSD_TC_CHUNK):
        return SSD_TC_CHUNK                   # the tcgen05 chunk scan wants its 128 rows
    lib = build.load("ssd")
    f = lib.lb_ssd_chunk_len
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return int(f(int(chunk_size), int(head_dim), int(state_dim)))


def ssd_prefill(conv: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
                state: torch.Tensor, cu_seqlens: torch.Tensor, start_pos: torch.Tensor, slots: torch.Tensor,
                chunks: torch.Tensor, num_chunks: int, req_chunks: torch.Tensor, num_long: int, chunk_len: int,
                num_heads: int, head_dim: int, state_dim: int, num_groups: int, dt_scale: float,
                gate: torch.Tensor | None = None, gate_scale: float = 1.0, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """Chunked scan of the listed prompt portions (bfloat16, tensor cores).  `chunks`: int32 [n, 2] =
    (request index, first token of the chunk within its portion); `req_chunks`: int32 [m, 3] = (request
    index, its first chunk, its number of chunks).  Arguments otherwise as `ssm_scan`; rows of `out`
    outside the listed requests are left as they are."""
    _cuda(conv, dt, A_log, dt_bias, D, state, cu_seqlens, start_pos, slots, chunks, req_chunks, gate, out)
    tokens, C = conv.shape
    _need(conv.dtype == torch.bfloat16 and conv.is_contiguous(), "ssd_prefill takes a contiguous bfloat16 conv output")
    _need(dt.shape == (tokens, num_heads) and dt.stride(1) == 1 and dt.dtype == conv.dtype, "dt must be a [tokens, heads] view")
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (D, "D")):
        _need(t.dtype == torch.float32 and t.shape == (num_heads,) and t.is_contiguous(), f"{n} must be float32 [heads]")
    _need(_ssm_state_ok(state, conv.dtype) and state.shape[1:] == (num_heads, head_dim, state_dim),
          "SSM state must be contiguous float32 or bfloat16 [slots, heads, P, N]")
    for t, n in ((cu_seqlens, "cu_seqlens"), (start_pos, "start_pos"), (slots, "slots"), (chunks, "chunks"), (req_chunks, "req_chunks")):
        _i32(t, n)
    _need(chunks.numel() >= 2 * num_chunks and req_chunks.numel() >= 3 * num_long, "work lists are shorter than their counts")
    if gate is not None:
        _need(gate.shape == (tokens, num_heads * head_dim) and gate.stride(1) == 1 and gate.dtype == conv.dtype,
              "gate must be a [tokens, heads * head_dim] view of the activation dtype")
    y = out if out is not None else torch.empty((tokens, num_heads * head_dim), dtype=conv.dtype, device=conv.device)
    _need(y.shape == (tokens, num_heads * head_dim) and y.dtype == conv.dtype and y.is_contiguous(), "out must be [tokens, heads * head_dim]")
    scratch = torch.empty((max(num_chunks, 1), num_heads, head_dim, state_dim), dtype=torch.float32, device=conv.device)
    chunk_a = torch.empty((max(num_chunks, 1), num_heads), dtype=torch.float32, device=conv.device)
    s_in = torch.empty(scratch.shape, dtype=torch.bfloat16, device=conv.device)
    gate_stride = gate.stride(0) if gate is not None else 0
    # the chunk scan on the tcgen05 kernel where it takes the sizes
    tc = ssd_chunk_scan_tc_ok(head_dim, state_dim, chunk_len) and conv.data_ptr() % 16 == 0 and y.data_ptr() % 16 == 0
    f = _fn("ssd", "lb_ssd_prefill", [c_void_p, c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_float, c_int, c_int, c_int,
                                      c_void_p])
    _check(f(_ptr(conv), C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D), _ptr(state), _ptr(y),
             _ptr(cu_seqlens), _ptr(start_pos), _ptr(slots), _ptr(chunks), num_chunks, _ptr(req_chunks), num_long,
             _ptr(scratch), _ptr(s_in), _ptr(chunk_a), num_heads, head_dim, state_dim, num_groups, chunk_len, dt_scale,
             _ptr(gate), gate_stride, gate_scale, 0 if tc else 1, int(state.dtype == torch.bfloat16), _code(conv), _stream()),
           "ssd_prefill", f"(head_dim {head_dim}, state_dim {state_dim}, chunk {chunk_len})", launches=2 if tc else 3)
    if tc:
        err = error_word(conv.device)
        g = _fn("ssd_tc", "lb_ssd_chunk_scan_tc",
                [c_void_p, c_long, c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_long, c_float, c_void_p, c_void_p])
        _check(g(_ptr(conv), tokens, C, _ptr(dt), dt.stride(0), _ptr(A_log), _ptr(dt_bias), _ptr(D), _ptr(y),
                 _ptr(cu_seqlens), _ptr(chunks), num_chunks, _ptr(s_in), num_heads, head_dim, state_dim, num_groups,
                 chunk_len, dt_scale, _ptr(gate), gate_stride, gate_scale, _ptr(err), _stream()),
               "ssd_chunk_scan_tc", f"(head_dim {head_dim}, state_dim {state_dim}, chunk {chunk_len})")
    return y


# --------------------------------------------------------------------------- matrix products
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    _cuda(a, w, bias)
    _need(a.dtype == w.dtype == torch.float32, "gemm_f32 takes float32 operands")
    _need(a.dim() == 2 and a.stride(1) == 1 and w.dim() == 2 and w.is_contiguous() and a.shape[1] == w.shape[1],
          "gemm_f32 wants a [M, K] (row-strided) and w [N, K]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.shape == (w.shape[0],)), "bias must be float32 [N]")
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    f = _fn("gemm_f32", "lb_gemm_f32", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                                        c_float, c_void_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, K, out_scale, _stream()), "gemm_f32")
    return out


def linear_join_ok(x, w: torch.Tensor, bias, join: ResidualJoin | None) -> bool:
    """Can `linear_join` take this product?  Few bfloat16 rows (the consumers norm at most 16), whole blocks of 16
    output columns, a residual of the output's shape."""
    if join is None or isinstance(x, NormedRows) or not _skinny_ok(x, w, bias, 16) or w.shape[0] % 16:
        return False
    r = join.residual
    return r is None or (r.dtype == torch.bfloat16 and r.shape == (x.shape[0], w.shape[0]) and r.is_contiguous())


def linear_join(x: torch.Tensor, w: torch.Tensor, bias, join: ResidualJoin, *, out_scale: float = 1.0) -> SummedRows:
    """x @ w^T (+ bias, * out_scale) whose epilogue joins the residual stream: see `ResidualJoin`, `SummedRows`."""
    _need(linear_join_ok(x, w, bias, join), "linear_join takes at most 16 bfloat16 rows and N a multiple of 16")
    M, Kdim = x.shape
    N = w.shape[0]
    other = join.other_tensor()
    _need(other is None or (other.dtype == torch.bfloat16 and other.shape == (M, N) and other.is_contiguous()),
          "the other branch must be contiguous bfloat16 [M, N]")
    _cuda(x, w, bias, other, join.residual)
    vsum = torch.empty((M, N), dtype=torch.float32, device=x.device)
    partial = torch.empty((N // 16, M), dtype=torch.float32, device=x.device)
    res_out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    f = _fn("linear_skinny", "lb_linear_skinny_join",
            [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_float,
             c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), M, N, Kdim, out_scale, _ptr(other), _ptr(join.residual),
             join.in_scales[0], join.in_scales[1], _ptr(vsum), _ptr(res_out), _ptr(partial), _stream()), "linear_skinny_join")
    return SummedRows(vsum, res_out, partial)


def summed_rmsnorm(rows: SummedRows, weight: torch.Tensor, eps: float, out_scales) -> tuple:
    """The RMSNorm of summed rows as a kernel of its own: for a consumer that cannot norm them itself (the built-in
    products can), same rounding points as `add_rmsnorm`."""
    v = rows.vsum
    _cuda(v, weight)
    M, H = v.shape
    _need(v.dtype == torch.float32 and v.is_contiguous(), "summed rows are contiguous float32")
    _need(weight.dtype == torch.float32 and weight.shape == (H,) and weight.is_contiguous(),
          "norm weight must be a contiguous float32 vector of the row width")
    _need(1 <= len(out_scales) <= 2, "one or two outputs")
    act = rows.residual.dtype
    out0 = torch.empty((M, H), dtype=act, device=v.device)
    out1 = torch.empty((M, H), dtype=act, device=v.device) if len(out_scales) == 2 else None
    f = _fn("norm", "lb_summed_rmsnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float,
                                          c_int, c_void_p])
    _check(f(_ptr(v), _ptr(weight), _ptr(out0), _ptr(out1), M, H, eps, out_scales[0], out_scales[-1],
             _DTYPE_CODE[act], _stream()), "summed_rmsnorm")
    return (out0,) if out1 is None else (out0, out1)


# Rows up to which a norm rides in the products that consume it (and a product's epilogue joins the residual stream
# for it).  The kernels take 16; measured on 36-layer decode steps, 12 rows take 1.57 instead of 1.65 ms and 16 rows
# 1.78 instead of 1.96 ms with the norm as a kernel of its own: every CTA of a consumer norms all rows for itself.
DEFERRED_NORM_MAX_ROWS = 8


def deferred_norm_ok(x) -> bool:
    """Can a norm over these rows ride in the prologue of the products that consume it?"""
    if isinstance(x, SummedRows):
        return 0 < x.shape[0] <= DEFERRED_NORM_MAX_ROWS and x.shape[1] % 8 == 0
    return (x.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= DEFERRED_NORM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.shape[1] <= 2048 and x.is_contiguous())


def _skinny_normed(nr: NormedRows, w: torch.Tensor, bias, out_scale: float, out_f32: bool, swiglu_scale) -> torch.Tensor:
    M, Kdim = nr.x.shape
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=w.device)
    if nr.summed:
        _check(_summed_fn()(_ptr(nr.x.vsum), _ptr(nr.x.partial), nr.x.partial.shape[0], _ptr(nr.weight), nr.eps, nr.scale,
                            _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
                            swiglu_scale if swiglu_scale is not None else 1.0, mode,
                            None, None, None, None, None, 0, 0, 0, 0, 0, 1.0, 1.0, 1.0, _stream()), "linear_skinny_summed")
        return out
    write = nr.shared["residual_out"] is not None and not nr.shared["written"]
    f = _fn("linear_skinny", "lb_linear_skinny_normed",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_void_p, c_void_p,
             c_void_p, c_long, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(nr.x), _ptr(nr.other), _ptr(nr.residual), _ptr(nr.shared["residual_out"]) if write else None,
             _ptr(nr.weight), nr.eps, nr.in_scales[0], nr.in_scales[1], nr.scale, _ptr(w), _ptr(bias), _ptr(out), N, M, N,
             Kdim, out_scale, swiglu_scale if swiglu_scale is not None else 1.0, mode, _stream()), "linear_skinny_normed")
    if write:
        nr.shared["written"] = True
    return out


def _summed_fn():
    return _fn("linear_skinny", "lb_linear_skinny_summed",
               [c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                c_float, c_float, c_float, c_void_p])


# At or below this many rows a bfloat16 product goes to the weight-streaming kernel (which takes up to 64).  Measured
# on 36-layer decode steps: with the library above 32 rows a step of 48 rows takes 2.48 instead of 2.72 ms and one of
# 64 rows 2.77 instead of 3.07 ms; with the library above 16 rows a step of 24 rows 2.62 instead of 2.18 ms.
SKINNY_MAX_ROWS = 32


def _skinny_ok(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, max_rows: int | None = None) -> bool:
    max_rows = SKINNY_MAX_ROWS if max_rows is None else max_rows
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= max_rows
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())))


_PLAIN, _OUT_F32, _SWIGLU = 0, 1, 2


def linear_skinny(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
                  out_f32: bool = False, swiglu_scale: float | None = None) -> torch.Tensor:
    """The weight-streaming product for at most 64 bfloat16 rows: x [M, K] @ w[N, K]^T, with the bias,
    output multiplier, float32 output or SwiGLU (w = [gate rows; up rows]) done on the sums."""
    _cuda(x, w, bias)
    _need(_skinny_ok(x, w, bias, 64), "linear_skinny takes at most 64 bfloat16 rows, K a multiple of 8, 16-byte aligned operands")
    M, Kdim = x.shape
    _need(w.dim() == 2 and w.shape[1] == Kdim, "weight must be [N, K]")
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        _need(N % 2 == 0 and bias is None and not out_f32 and out_scale == 1.0, "the SwiGLU form takes [gate; up] rows and nothing else")
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    _need(bias is None or bias.shape == (N,), "bias must be [N]")
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    f = _fn("linear_skinny", "lb_linear_skinny", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int,
                                                  c_int, c_float, c_float, c_int, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
             swiglu_scale if swiglu_scale is not None else 1.0, mode, _stream()), "linear_skinny")
    return out


_gemm_error: dict[torch.device, torch.Tensor] = {}
# Which kernel takes bfloat16 products of more rows than the weight streamer.  "auto" and "library": cuBLAS through
# torch, the SwiGLU as a kernel of its own behind it.  "tcgen05": the engine's own tcgen05 kernel with its fused
# epilogues.  Measured at 2048 x 4096 x 1024 (gate|up of a 2,048-token prompt): the library product 16.3 us + SwiGLU
# kernel 7.1 us = 23.4 us against 33.4 us for the fused tcgen05 kernel, whose 128 x 128 one-CTA tiles are bound by
# L2 -> SM traffic (64 FLOP per byte; the library runs 256 x 256 two-CTA tiles); at 64 rows its 128-row tile is
# half empty.  It stays selectable and tested, and is not the default until it wins.
GEMM_MODE = os.environ.get("LOGSSMS_B200_GEMM", "auto")


def _tcgen05_ok(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] > 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.shape[1] % 8 == 0 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous())))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
                 out_f32: bool = False, swiglu_scale: float | None = None) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), with the
    bias, output multiplier, float32 output or SwiGLU (w = [gate rows; up rows]) done on the sums.
    `check_kernel_errors()` reports a kernel whose internal wait gave up."""
    _cuda(x, w, bias)
    _need(_tcgen05_ok(x, w, bias), "gemm_tcgen05 takes bfloat16 operands, K a multiple of 8, 16-byte aligned")
    M, Kdim = x.shape
    _need(w.dim() == 2 and w.shape[1] == Kdim, "weight must be [N, K]")
    N = w.shape[0]
    mode = _PLAIN
    if swiglu_scale is not None:
        _need(N % 2 == 0 and bias is None and not out_f32 and out_scale == 1.0, "the SwiGLU form takes [gate; up] rows and nothing else")
        N //= 2
        mode = _SWIGLU
    elif out_f32:
        mode = _OUT_F32
    _need(bias is None or bias.shape == (N,), "bias must be [N]")
    out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    err = error_word(x.device)
    f = _fn("gemm_tcgen05", "lb_gemm_tcgen05", [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int,
                                                c_float, c_float, c_int, c_void_p, c_void_p])
    _check(f(_ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, out_scale,
             swiglu_scale if swiglu_scale is not None else 1.0, mode, _ptr(err), _stream()), "gemm_tcgen05")
    return out


def error_word(device) -> torch.Tensor:
    """The int32 word on `device` into which a kernel whose bounded wait gave up writes where it stopped (0: none
    did).  One per device, shared by all such kernels; the scheduler reads it with every step's sampled ids, the
    trace replay after every step."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device(device.type, torch.cuda.current_device())
    err = _gemm_error.get(device)
    if err is None:
        with torch.inference_mode(False):      # an ordinary tensor, whoever asks first: the host may set and clear it anywhere
            err = _gemm_error[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return err


def raise_kernel_error(code: int, device=None) -> None:
    """Clear the error word of `device` (all devices when None) and raise what `code` says."""
    for dev, err in _gemm_error.items():
        if device is None or _same_device(dev, device):
            err.zero_()
    raise KernelError(f"a wait inside a kernel gave up, its results are not valid (role {(code >> 24) & 0x3F}, "
                      f"block {(code >> 12) & 0xFFF}, step {code & 0xFFF})")


def _same_device(a, b) -> bool:
    a, b = torch.device(a), torch.device(b)
    return a.type == b.type and (a.index is None or b.index is None or a.index == b.index)


def check_kernel_errors(device=None) -> None:
    """Raise if a kernel gave up on one of its bounded waits since the last check (synchronises)."""
    for dev, err in _gemm_error.items():
        if device is not None and not _same_device(dev, device):
            continue
        code = int(err.item())
        if code:
            raise_kernel_error(code, dev)


def linear_conv_step_ok(x, w: torch.Tensor, bias, conv_state: torch.Tensor, max_rows: int | None = None) -> bool:
    """Should `linear_conv_step` take these operands (else: `linear`, then `causal_conv1d`)?  `max_rows`: the most
    rows (default: as many as go to the weight streamer at all; the kernel itself takes 64)."""
    if conv_state.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.data_ptr() % 16:
        return False
    if bias is not None and not (bias.dtype == torch.bfloat16 and bias.is_contiguous()):
        return False
    if isinstance(x, NormedRows):
        return w.shape[1] == x.shape[1]
    return _skinny_ok(x, w, bias, max_rows)


def linear_conv_step(x, w: torch.Tensor, bias, conv_weight: torch.Tensor, conv_bias, conv_state: torch.Tensor,
                     slots: torch.Tensor, start_pos: torch.Tensor, first: int, last: int,
                     region_ends: tuple[int, int], region_scales: tuple[float, float, float]) -> torch.Tensor:
    """x @ w^T (+ bias) for a decode batch (every row the single new token of its own request), with the
    depthwise conv step done on the output columns [first, last) before they are stored: those columns come
    back as silu(conv(...)) and `conv_state` ([slots, last - first, taps - 1]) is shifted in place.  `x` may be
    `NormedRows`.  `region_ends` are column indices relative to `first`."""
    normed = isinstance(x, NormedRows)
    _need(linear_conv_step_ok(x, w, bias, conv_state, 64), "linear_conv_step takes few bfloat16 rows (see linear_skinny)")
    C = last - first
    taps = conv_weight.shape[1]
    _need(conv_weight.dtype == torch.float32 and conv_weight.shape == (C, taps) and conv_weight.is_contiguous(), "conv weight must be float32 [C, K]")
    _need(conv_bias is None or (conv_bias.dtype == torch.float32 and conv_bias.shape == (C,) and conv_bias.is_contiguous()), "conv bias must be float32 [C]")
    _need(conv_state.is_contiguous() and conv_state.shape[1:] == (C, taps - 1), "conv state must be contiguous [slots, C, K-1]")
    _i32(slots, "slots")
    _i32(start_pos, "start_pos")
    M, Kdim = x.shape
    N = w.shape[0]
    _need(slots.numel() >= M and start_pos.numel() >= M and 0 <= first <= last <= N, "one slot and start per row; columns within the output")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
    if normed and x.summed:
        _check(_summed_fn()(_ptr(x.x.vsum), _ptr(x.x.partial), x.x.partial.shape[0], _ptr(x.weight), x.eps, x.scale,
                            _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, 1.0, 1.0, _PLAIN,
                            _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state), _ptr(slots), _ptr(start_pos), first, last, taps,
                            region_ends[0], region_ends[1], region_scales[0], region_scales[1], region_scales[2], _stream()),
               "linear_conv_step")
        return out
    write = normed and x.shared["residual_out"] is not None and not x.shared["written"]
    f = _fn("linear_skinny", "lb_linear_skinny_conv",
            [c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_void_p,
             c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_float, c_float, c_float, c_void_p])
    if normed:
        head = (None, 0, _ptr(x.x), _ptr(x.other), _ptr(x.residual), _ptr(x.shared["residual_out"]) if write else None,
                _ptr(x.weight), x.eps, x.in_scales[0], x.in_scales[1], x.scale)
    else:
        _cuda(x)
        head = (_ptr(x), x.stride(0), None, None, None, None, None, 0.0, 1.0, 1.0, 1.0)
    _check(f(*head, _ptr(w), _ptr(bias), _ptr(out), N, M, N, Kdim, _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state),
             _ptr(slots), _ptr(start_pos), first, last, taps, region_ends[0], region_ends[1], region_scales[0],
             region_scales[1], region_scales[2], _stream()), "linear_conv_step")
    if write:
        x.shared["written"] = True
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, out_scale: float = 1.0,
           out_f32: bool = False, lazy_scale: bool = False):
    """round(round(x [M, K] @ w[N, K]^T + bias) * out_scale) in x's dtype, or as float32 with `out_f32`.
    With `lazy_scale` (the caller's consumer takes `ScaledRows`) a product whose kernel has no epilogue for the
    multiplier comes back as `ScaledRows` instead of going through the scale kernel.

    float32 activations: the engine's own 32-bit kernel.  bfloat16: at most 64 rows go to the
    weight-streaming kernel (a decode step is bound by reading the weights once); more rows go to
    cuBLAS through torch (32-bit accumulation).  bfloat16 activations with a weight that is stored in
    32-bit: the 32-bit kernel on widened activations, result rounded once.  `x` may be `NormedRows`."""
    if isinstance(x, NormedRows):
        if (w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == x.shape[1] and w.data_ptr() % 16 == 0
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous()))):
            return _skinny_normed(x, w, bias, out_scale, out_f32, None)
        x = x.tensor()
    _cuda(x, w, bias)
    if x.dtype == torch.float32:
        return gemm_f32(x, w.float(), None if bias is None else bias.float(), out_scale)
    if w.dtype == torch.float32:
        y = gemm_f32(x.float(), w, None if bias is None else bias.float()).to(x.dtype)
    elif _skinny_ok(x, w, bias):
        return linear_skinny(x, w, bias, out_scale=out_scale, out_f32=out_f32)
    elif GEMM_MODE == "tcgen05" and _tcgen05_ok(x, w, bias):
        return gemm_tcgen05(x, w, bias, out_scale=out_scale, out_f32=out_f32)
    else:
        # the library product, asked for as mm / addmm: the same cuBLAS call as `F.linear` makes, with 4 us less of
        # dispatch on the host per call (a prompt step of a new shape is bound by the host)
        product = (lambda: torch.mm(x, w.t())) if bias is None else (lambda: torch.addmm(bias.to(x.dtype), x, w.t()))
        y = PROFILER.timed("library", "mm", product) if PROFILER.enabled else product()
    if lazy_scale and not out_f32 and out_scale != 1.0:
        return ScaledRows(y, out_scale)
    if out_f32 or out_scale != 1.0:
        y = scale(y, out_scale, to_f32=out_f32)
    return y


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act_scale: float) -> torch.Tensor:
    """silu(round(gate * act_scale)) * up with [gate | up] = x @ w_gate_up^T (w rows: gate, then up).
    `x` may be `NormedRows`."""
    if isinstance(x, NormedRows):
        if (w_gate_up.dtype == torch.bfloat16 and w_gate_up.is_contiguous() and w_gate_up.shape[1] == x.shape[1]
                and w_gate_up.shape[0] % 2 == 0 and w_gate_up.data_ptr() % 16 == 0):
            return _skinny_normed(x, w_gate_up, None, 1.0, False, act_scale)
        x = x.tensor()
    if _skinny_ok(x, w_gate_up, None):
        return linear_skinny(x, w_gate_up, swiglu_scale=act_scale)
    if GEMM_MODE == "tcgen05" and _tcgen05_ok(x, w_gate_up, None):
        return gemm_tcgen05(x, w_gate_up, swiglu_scale=act_scale)
    return swiglu(linear(x, w_gate_up), act_scale)
