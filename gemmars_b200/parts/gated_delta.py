"""Gated delta rule: a recurrent mixer whose state per head is a matrix S [dim, vdim].

For one token, with h the mixer's input:
  q, k = W_q h, W_k h (kv_heads x dim), v = W_v h (heads x vdim); each passes a short causal filter
  over time (``conv`` taps per channel) and SiLU; q and k become unit vectors per head
  (x / sqrt(|x|^2 + 1e-6)), q also times dim^-1/2; head i reads q/k head i // (heads / kv_heads);
  beta = sigmoid(W_b h), g = exp(-exp(A_log) * softplus(W_a h + dt_bias)), one of each per head;
  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (the read-out sees this token's write);
  o / rms(o) * norm * silu(W_g h) per head, then W_o, added into the residual.

The six projections are one product written in float32: everything after it that enters the
recurrence (filters, unit norms, gates, decay, state) is float32 work.  Per sequence the part keeps
the state S and the filter's last ``conv - 1`` inputs.  Parameters: hidden_size, heads, kv_heads,
dim, vdim, conv, norm_eps, out_scale (a factor on the mixer's output, default 1).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import StateNeed
from .base import Part, TensorWant, register_part
from .linear import Linear

UNIT_EPS = 1e-6


class GatedDeltaRule(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.eps = float(p["norm_eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.heads} heads are not a multiple of {self.kv_heads} q/k heads")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"gated_delta: a filter of {self.taps} taps is not supported (1 to 8)")
        if self.dim > 256:
            raise ValueError(f"gated_delta: q/k heads of {self.dim} are wider than the kernel takes (256)")
        self.qk, self.hv = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk + self.hv            # what the filter runs over: q | k | v
        self.proj = self.o = self.filter = self.a_log = self.dt_bias = self.norm = None

    def wants(self):
        h, qk, hv, nh, k = self.hidden_size, self.qk, self.hv, self.heads, self.taps
        return {"q": TensorWant((qk, h)), "k": TensorWant((qk, h)), "v": TensorWant((hv, h)), "g": TensorWant((hv, h)),
                "b": TensorWant((nh, h)), "a": TensorWant((nh, h)), "o": TensorWant((h, hv)),
                "q_conv": TensorWant((qk, k), "vector"), "k_conv": TensorWant((qk, k), "vector"),
                "v_conv": TensorWant((hv, k), "vector"), "A_log": TensorWant((nh,), "vector"),
                "dt_bias": TensorWant((nh,), "vector"), "norm": TensorWant((self.vdim,), "vector")}

    def load(self, t):
        # one product: [q | k | v | g | b | a]
        self.proj = Linear(torch.cat([t[n] for n in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.o = Linear(t["o"])
        self.filter = torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = t["A_log"].contiguous(), t["dt_bias"].contiguous(), t["norm"].contiguous()

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("recurrent", ())]

    def cache_needs(self):
        return [StateNeed((self.taps - 1, self.channels)), StateNeed((self.heads, kernels.recurrent_state_floats(self.dim, self.vdim)))]

    def weight_bytes(self):
        small = sum(4 * t.numel() for t in (self.filter, self.a_log, self.dt_bias, self.norm) if t is not None)
        return self.proj.bytes() + self.o.bytes() + small

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if not writes_cache:
            raise ValueError("gated_delta: a recurrent mixer cannot run on another layer's state")
        filter_state, state = caches
        qk, hv, nh, c = self.qk, self.hv, self.heads, self.channels
        p = self.proj(h, out_dtype=torch.float32)
        t = p.shape[0]
        f = torch.empty((t, c), dtype=torch.float32, device=p.device)
        kernels.short_filter(p[:, :c], self.filter, None, filter_state, ctx.cu_seqlens, ctx.tok_seq, ctx.seq_slot, f, act=True)
        y = torch.empty((t, hv), dtype=torch.float32, device=p.device)
        kernels.delta_rule(f[:, :qk], f[:, qk:2 * qk], f[:, 2 * qk:], p[:, c + hv:c + hv + nh], p[:, c + hv + nh:],
                           self.a_log, self.dt_bias, state, ctx.cu_seqlens, ctx.seq_slot, y, nh, self.kv_heads, self.dim,
                           self.vdim, float(self.dim) ** -0.5)
        out = torch.empty((t, hv), dtype=self.act_dtype, device=p.device)
        kernels.gated_group_norm(y, p[:, c:c + hv], self.norm, out, self.vdim, self.eps, False, self.out_scale)
        self.o.add_into(out, residual)


register_part("mixer", "gated_delta", GatedDeltaRule)
