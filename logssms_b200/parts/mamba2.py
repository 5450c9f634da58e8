"""Mamba2 (SSD) mixer: in_proj -> causal conv -> selective scan -> gate / gated norm -> out_proj."""
from __future__ import annotations

import math

import torch

from ..cache import CacheNeeds, StateNeed
from ..ops import kernels as K
from ..registry import MIXERS
from .base import MATRIX, VECTOR, ParamSpec, Part, normal_init, ones_init


def _a_log_init(gen, shape):
    return torch.log(1.0 + 15.0 * torch.rand(shape, generator=gen, dtype=torch.float32))          # log U[1, 16]


def _dt_bias_init(gen, shape):
    lo, hi = math.log(1e-3), math.log(1e-1)
    dt = torch.exp(lo + (hi - lo) * torch.rand(shape, generator=gen, dtype=torch.float32))        # log-uniform step
    return dt + torch.log(-torch.expm1(-dt))                                                       # softplus^-1(dt)


@MIXERS.register("mamba2")
class Mamba2(Part):
    """Per-request state: the conv window (last K-1 scaled inputs per channel, activation dtype) and
    the SSM state [heads, P, N] in float32 (the reference keeps it in the activation dtype,
    python/logssms/cache/radix/state_pool.py:25-32).

    Flow and constants: python/logssms/layers/mamba2.py:70-149; kernels' formulas:
    python/logssms/kernel/linear_attention/packed_conv.py:96-140,
    python/logssms/kernel/linear_attention/mamba2.py:27-36 and :261-292,
    python/logssms/kernel/norm.py:55-86."""
    takes_normed_rows = True      # forward() passes its input straight into a product
    kernels = ("conv", "ssm", "ssd", "ssd_tc", "norm", "linear_skinny", "gemm_tcgen05")

    def __init__(self, spec, perturb_init: bool = False, shared: dict | None = None):
        self.spec = spec
        self._perturb = perturb_init
        self.in_w = self.in_b = self.conv_w = self.conv_b = None
        self.A_log = self.dt_bias = self.D = self.norm_w = self.out_w = self.out_b = None
        self._chunk_len = 0

    def param_specs(self):
        s = self.spec
        jitter = 0.1 if self._perturb else 0.0
        bias_init = normal_init(0.02 if self._perturb else 0.0)
        specs = {
            "in_proj.weight": ParamSpec((s.proj_size, s.hidden_size), MATRIX),
            "conv1d.weight": ParamSpec((s.conv_dim, 1, s.conv_kernel), VECTOR, normal_init(0.2)),
            "A_log": ParamSpec((s.num_heads,), VECTOR, _a_log_init, torch.float32),
            "dt_bias": ParamSpec((s.num_heads,), VECTOR, _dt_bias_init),
            "D": ParamSpec((s.num_heads,), VECTOR, ones_init(jitter)),
            "out_proj.weight": ParamSpec((s.hidden_size, s.inner_size), MATRIX),
        }
        if s.proj_bias:
            specs["in_proj.bias"] = ParamSpec((s.proj_size,), VECTOR, bias_init)
        if s.conv_bias:
            specs["conv1d.bias"] = ParamSpec((s.conv_dim,), VECTOR, bias_init)
        if s.gated_norm:
            specs["norm.weight"] = ParamSpec((s.inner_size,), VECTOR, ones_init(jitter))
        if s.out_bias:
            specs["out_proj.bias"] = ParamSpec((s.hidden_size,), VECTOR, bias_init)
        return specs

    def bind(self, t):
        s = self.spec
        self.in_w, self.out_w = t["in_proj.weight"], t["out_proj.weight"]
        act = self.in_w.dtype
        self.in_b = t.get("in_proj.bias")
        self.out_b = t.get("out_proj.bias")
        if act != torch.float32:
            self.in_b = None if self.in_b is None else self.in_b.to(act)
            self.out_b = None if self.out_b is None else self.out_b.to(act)
        self.conv_w = t["conv1d.weight"].reshape(s.conv_dim, s.conv_kernel).contiguous()
        self.conv_b = t.get("conv1d.bias")
        self.A_log, self.dt_bias, self.D = t["A_log"], t["dt_bias"], t["D"]
        self.norm_w = t.get("norm.weight")

    def setup(self, rt) -> None:
        s = self.spec
        self._chunk_len = K.ssd_chunk_len(s.chunk_size, s.head_dim, s.state_dim) if rt.dtype == torch.bfloat16 else 0
        # The recurrent state between steps: 32-bit unless the engine's user asks for the activation dtype, in which
        # the reference keeps it (python/logssms/cache/naive/manager.py:445-451): half the bytes of a decode step's
        # state update, one rounding of the state per step.
        choice = rt.options.get("ssm_state_dtype", "float32")
        if choice not in ("float32", "activation"):
            raise ValueError(f"ssm_state_dtype must be float32 or activation, got {choice!r}")
        self._state_dtype = torch.float32 if choice == "float32" else None

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(states=(
            StateNeed("conv", (s.conv_dim, s.conv_kernel - 1), None),
            StateNeed("ssm", (s.num_heads, s.head_dim, s.state_dim), getattr(self, "_state_dtype", torch.float32)),
        ))

    def forward(self, x: torch.Tensor, ctx, cache_layer: int, writes_cache: bool = True) -> torch.Tensor:
        s = self.spec
        m = s.multipliers
        inner, C = s.inner_size, s.conv_dim
        states = ctx.cache.states[cache_layer]
        regions = ((inner, inner + s.num_groups * s.state_dim), (m[1], m[2], m[3]))
        if ctx.max_len == 1 and K.linear_conv_step_ok(x, self.in_w, self.in_b, states["conv"]):
            # a decode step: the conv step rides in the projection's epilogue (its columns come back convolved)
            proj = K.linear_conv_step(x, self.in_w, self.in_b, self.conv_w, self.conv_b, states["conv"], ctx.slots,
                                      ctx.start_pos, inner, inner + C, *regions)
            z, conv, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
        else:
            proj = K.linear(x, self.in_w, self.in_b)
            z, xbc, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
            conv = K.causal_conv1d(xbc, self.conv_w, self.conv_b, states["conv"], ctx.cu_seqlens, ctx.start_pos,
                                   ctx.slots, ctx.num_requests, ctx.max_len, *regions)
        gate = None if s.gated_norm else z          # the bare gate rides in the scan's epilogue
        head = (conv, dt, self.A_log, self.dt_bias, self.D, states["ssm"], ctx.cu_seqlens, ctx.start_pos, ctx.slots)
        sizes = (s.num_heads, s.head_dim, s.state_dim, s.num_groups, m[4])
        if x.dtype == torch.bfloat16 and ctx.has_long_portions and self._chunk_len:
            # long portions in chunks on the tensor cores; decoded tokens and short portions token by token: other
            # requests, other rows of y.  In a captured step the token-by-token kernel, which is bound by the states it
            # streams, runs beside the chunked kernels, which are not, on a stream to spare.
            chunks, n_chunks, per_request, n_long = ctx.long_portion_chunks(self._chunk_len)
            _, _, short_list, n_short = ctx.requests_by_portion()
            y = torch.empty((conv.shape[0], inner), dtype=conv.dtype, device=conv.device)
            beside = ctx.fork() if n_short > 0 else None
            K.ssd_prefill(*head, chunks, n_chunks, per_request, n_long, self._chunk_len, *sizes, gate, m[0], out=y)
            if n_short > 0:
                short = lambda: K.ssm_scan(*head, ctx.num_requests, *sizes, gate, m[0], request_list=short_list,
                                           num_listed=n_short, out=y, beside=beside is not None)
                if beside is not None:
                    beside(short)()
                else:
                    short()
        else:
            y = K.ssm_scan(*head, ctx.num_requests, *sizes, gate, m[0])
        if s.gated_norm:
            mode = K.NORM_BEFORE_GATE if s.norm_before_gate else K.NORM_AFTER_GATE
            y = K.gated_rmsnorm(y, z, self.norm_w, s.norm_eps, s.num_groups, m[0], mode)
        return K.linear(y, self.out_w, self.out_b)
