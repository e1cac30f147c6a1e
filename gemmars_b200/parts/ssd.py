"""Selective state space with one decay per head (the state-space duality form): a recurrent
mixer whose state per head is a matrix S [state, vdim].

With inner = heads * vdim, N = state, G = groups, one product W_in h gives
[z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C together pass a short causal
filter over time (``conv`` taps per channel, with a bias) and SiLU.  dt <- softplus(dt + dt_bias).
Head i reads group i // (heads / groups):
  S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x.
y (heads side by side) times silu(z), then divided by its root mean square in ``norm_groups``
equal parts, times ``norm``, then W_o, added into the residual.

The product is written in float32; filter, step size, decay and state are float32 work.  Per
sequence the part keeps S and the filter's last ``conv - 1`` inputs.  Parameters: hidden_size,
heads, vdim, state, groups, norm_groups, conv, norm_eps, out_scale (default 1).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import StateNeed
from .base import Part, TensorWant, register_part
from .linear import Linear


class StateSpaceDual(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.norm_groups, self.taps = int(p["groups"]), int(p["norm_groups"]), int(p["conv"])
        self.eps = float(p["norm_eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        self.inner = self.heads * self.vdim
        if self.heads % self.groups:
            raise ValueError(f"ssd: {self.heads} heads are not a multiple of {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"ssd: {self.inner} channels cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"ssd: a filter of {self.taps} taps is not supported (1 to 8)")
        if self.n_state > 256:
            raise ValueError(f"ssd: a state of {self.n_state} is larger than the kernel takes (256)")
        self.channels = self.inner + 2 * self.groups * self.n_state     # what the filter runs over: x | B | C
        self.proj = self.o = self.filter = self.filter_bias = self.a_log = self.dt_bias = self.skip = self.norm = None

    def wants(self):
        h, c = self.hidden_size, self.channels
        return {"in": TensorWant((self.inner + c + self.heads, h)), "o": TensorWant((h, self.inner)),
                "conv": TensorWant((c, self.taps), "vector"), "conv_bias": TensorWant((c,), "vector"),
                "dt_bias": TensorWant((self.heads,), "vector"), "A_log": TensorWant((self.heads,), "vector"),
                "D": TensorWant((self.heads,), "vector"), "norm": TensorWant((self.inner,), "vector")}

    def load(self, t):
        self.proj, self.o = Linear(t["in"]), Linear(t["o"])
        self.filter, self.filter_bias = t["conv"].contiguous(), t["conv_bias"].contiguous()
        self.a_log, self.dt_bias = t["A_log"].contiguous(), t["dt_bias"].contiguous()
        self.skip, self.norm = t["D"].contiguous(), t["norm"].contiguous()

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("recurrent", ())]

    def cache_needs(self):
        return [StateNeed((self.taps - 1, self.channels)), StateNeed((self.heads, kernels.recurrent_state_floats(self.n_state, self.vdim)))]

    def weight_bytes(self):
        small = sum(4 * t.numel() for t in (self.filter, self.filter_bias, self.a_log, self.dt_bias, self.skip, self.norm)
                    if t is not None)
        return self.proj.bytes() + self.o.bytes() + small

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if not writes_cache:
            raise ValueError("ssd: a recurrent mixer cannot run on another layer's state")
        filter_state, state = caches
        inner, c, gn = self.inner, self.channels, self.groups * self.n_state
        p = self.proj(h, out_dtype=torch.float32)
        t = p.shape[0]
        f = torch.empty((t, c), dtype=torch.float32, device=p.device)
        kernels.short_filter(p[:, inner:inner + c], self.filter, self.filter_bias, filter_state, ctx.cu_seqlens, ctx.tok_seq,
                             ctx.seq_slot, f, act=True)
        y = torch.empty((t, inner), dtype=torch.float32, device=p.device)
        kernels.ssd_scan(f[:, :inner], f[:, inner:inner + gn], f[:, inner + gn:], p[:, inner + c:], self.a_log, self.dt_bias,
                         self.skip, state, ctx.cu_seqlens, ctx.seq_slot, y, self.heads, self.groups, self.n_state, self.vdim)
        out = torch.empty((t, inner), dtype=self.act_dtype, device=p.device)
        kernels.gated_group_norm(y, p[:, :inner], self.norm, out, inner // self.norm_groups, self.eps, True, self.out_scale)
        self.o.add_into(out, residual)


register_part("mixer", "ssd", StateSpaceDual)
