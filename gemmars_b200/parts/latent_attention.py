"""Latent attention: causal attention whose keys and values are expanded from one cached
low-rank row per position, shared by all heads, with an optional sigmoid gate per head.

For a token with input h at position p (H heads; per head ``dim`` unrotated and ``rot_dim``
rotated query/key dims, value size ``vdim``; latent size ``rank``):

    q       = Wq h                      laid out head by head as [dim | rot_dim]
    kv      = Wdkv h                    [rank | rot_dim]
    c       = rmsnorm(kv[:rank]) * w    the latent;   kr = rotate(kv[rank:], p), shared by all heads
    k[h]    = [Wuk[h] c | kr],  v[h] = Wuv[h] c
    s[h, j] = (q_nope[h] . Wuk[h] c_j + rotate(q_rot[h], p) . kr_j) * scale,  j <= p
    o[h]    = sigmoid(Wg h)[h] * sum_j softmax_j(s[h])[j] v_j[h];   residual += Wo concat(o)

Only [c | kr] is cached, one row of ``rank + rot_dim`` values per position (a ``KVNeed`` with one
kv head and no separate values).  Both expansions are moved off the keys: Wuk[h]^T is applied to
the query (q_nope[h] . Wuk[h] c = (Wuk[h]^T q_nope[h]) . c) and Wuv[h] to the attention's output
over the latents (sum_j p_j Wuv[h] c_j = Wuv[h] sum_j p_j c_j), so prompts, continued prompts and
single tokens all run one attention kernel over the cached rows, with all heads sharing them.

All sizes and constants are parameters: hidden_size, num_heads, dim, rot_dim, vdim, rank, scale,
norm_eps, gate (whether the output gate exists), window (None: all keys), position (a PartSpec of
kind ``rotary`` with the interleaved layout, or None).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import KVNeed
from .base import Part, TensorWant, build_part, register_part
from .linear import Linear
from .rotary import Rotary


class LatentAttention(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.rot_dim = int(p["rot_dim"])
        self.vdim = int(p["vdim"])
        self.rank = int(p["rank"])
        self.scale = float(p["scale"])
        self.eps = float(p.get("norm_eps", 1e-6))
        self.gated = bool(p.get("gate", True))
        self.window = p.get("window")
        pos = p.get("position")
        self.position = build_part("position", pos, compute) if pos is not None else None
        if self.position is not None:
            if not isinstance(self.position, Rotary) or self.position.layout != "interleaved":
                raise ValueError("latent_attention: the kernel that writes the cache rows rotates interleaved pairs; "
                                 "its position encoding must be a rotary part with that layout, or none")
            if self.position.rotary_dim > self.rot_dim:
                raise ValueError(f"latent_attention: cannot rotate {self.position.rotary_dim} of {self.rot_dim} dims")
        if min(self.num_heads, self.rank, self.vdim) <= 0 or self.dim < 0 or self.rot_dim < 0 or self.dim + self.rot_dim <= 0:
            raise ValueError("latent_attention: heads, rank and vdim must be positive, and a head must have query dims")
        self.proj = self.o = self.uk_t = self.uv = self.norm_w = None

    # ---- weights
    def wants(self):
        h, nh, r = self.hidden_size, self.num_heads, self.rank
        w = {"q": TensorWant((nh * (self.dim + self.rot_dim), h)), "dkv": TensorWant((r + self.rot_dim, h)),
             "dkv_norm": TensorWant((r,), "vector"), "uk": TensorWant((nh * self.dim, r)),
             "uv": TensorWant((nh * self.vdim, r)), "o": TensorWant((h, nh * self.vdim))}
        if self.gated:
            w["g"] = TensorWant((nh, h))
        return w

    def load(self, t):
        nh, r = self.num_heads, self.rank
        # one product reads the input once: queries, then the latent and the key part, then the gate logits
        self.proj = Linear(torch.cat([t["q"], t["dkv"]] + ([t["g"]] if self.gated else []), dim=0))
        self.o = Linear(t["o"])
        # [heads, rank, dim]: the matrix that carries a head's unrotated query dims into the latent space
        self.uk_t = t["uk"].view(nh, self.dim, r).transpose(1, 2).contiguous()
        self.uv = t["uv"].view(nh, self.vdim, r).contiguous()
        self.uk = t["uk"].view(nh, self.dim, r).contiguous()     # as stored: for prompts that expand the keys
        self.norm_w = t["dkv_norm"].contiguous()

    def kernel_units(self):
        units = kernels.gemm_units(self.compute) + kernels.latent_attention_units(self.compute, self.rank, self.rot_dim,
                                                                                  self.dim, self.vdim)
        return units + ([("grouped_gemm", ())] if self.compute != "float32" else [])

    def cache_needs(self):
        return [KVNeed(1, self.rank + self.rot_dim, self.window, value_dim=0)]

    def weight_bytes(self):
        per = self.uk_t.element_size()     # a decode step reads the transposed copy, not self.uk
        return self.proj.bytes() + self.o.bytes() + (self.uk_t.numel() + self.uv.numel()) * per + 4 * self.norm_w.numel()

    # ---- step
    def forward(self, ctx, h, residual, caches, writes_cache=True):
        nh, dim, rd, r, vd = self.num_heads, self.dim, self.rot_dim, self.rank, self.vdim
        group, kc, _ = caches[0]
        t = h.shape[0]
        nq = nh * (dim + rd)
        proj = self.proj(h, out_dtype=torch.float32)          # norms, angles and the gate are float32 work
        q_nope = torch.empty((t, nh * dim), dtype=self.act_dtype, device=h.device)
        qa = torch.empty((t, nh * (r + rd)), dtype=self.act_dtype, device=h.device)
        gate = torch.empty((t, nh), dtype=torch.float32, device=h.device) if self.gated else None
        rot = self.position.rotary_dim if self.position is not None else 0
        # a prompt step whose sequences all start at position 0 (no cached prefix) may expand keys and
        # values per head, which is less arithmetic than attention over the latent rows
        expand = (self.window is None and t >= kernels.LATENT_EXPAND_MIN_TOKENS and ctx.host is not None
                  and not any(ctx.host["seq_start"]) and kernels.latent_expand_usable(h.dtype, r, dim, rd, vd))
        dense = torch.empty((t, r + rd), dtype=self.act_dtype, device=h.device) if expand else None
        kernels.latent_prepare(proj[:, :nq], proj[:, nq:nq + r + rd], proj[:, nq + r + rd:] if self.gated else None,
                               self.norm_w, self.eps, self.position.inv_freq(h.device) if rot else None, rot, self.scale,
                               q_nope, qa, gate, kc.view(-1, group.page_size, r + rd) if writes_cache else None,
                               group.page_table, group.page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, nh, dim, rd, r,
                               dense=dense)
        if expand:
            return self._expanded(ctx, q_nope, qa, gate, dense, residual)
        if dim:
            kernels.heads_gemm(q_nope.view(t, nh, dim), self.uk_t, qa.view(t, nh, r + rd)[:, :, :r], nh)
        else:
            qa.view(t, nh, r + rd)[:, :, :r].zero_()
        lat = torch.empty((t, nh * r), dtype=self.act_dtype, device=h.device)
        kernels.latent_attention(ctx, qa, lat, nh, r, rd, kc.view(-1, group.page_size, r + rd), group.page_table,
                                 group.page_size, self.window)
        o = torch.empty((t, nh * vd), dtype=self.act_dtype, device=h.device)
        kernels.heads_gemm(lat.view(t, nh, r), self.uv, o.view(t, nh, vd), nh, scale=gate)
        self.o.add_into(o, residual)


    def _expanded(self, ctx, q_nope, qa, gate, dense, residual):
        """Attention of a prompt step over keys and values expanded per head.  Every head gets rows
        [v | k_nope | k_rot] of its own for the step's tokens (two grouped products from the step's
        latents, the rotated key part copied to every head) and queries [0 | q_nope | q_rot]; the
        attention kernel then runs with vdim in the latent's place, one head per grid layer, and
        multiplies the gate into its output."""
        nh, dim, rd, r, vd = self.num_heads, self.dim, self.rot_dim, self.rank, self.vdim
        t = q_nope.shape[0]
        kd = vd + dim + rd
        rows = torch.empty((nh, t + 64, kd), dtype=self.act_dtype, device=q_nope.device)
        rows[:, t:].zero_()                                   # a last tile reads past the last token
        hs = rows.stride(0)
        kernels.grouped_gemm(dense, dense.stride(0), 0, None, 1, self.uv, vd * r, rows, kd, hs, None, None, 0, 0, None, nh, t,
                             t, vd, r, what="latent_expand_v")
        kernels.grouped_gemm(dense, dense.stride(0), 0, None, 1, self.uk, dim * r, rows[:, :, vd:], kd, hs, None, None, 0, 0,
                             None, nh, t, t, dim, r, what="latent_expand_k")
        rows[:, :t, vd + dim:] = dense[:, r:]                 # copies: the shared rotated key part, to every head
        q = torch.empty((t, nh, kd), dtype=self.act_dtype, device=q_nope.device)
        q[:, :, :vd].zero_()
        q[:, :, vd:vd + dim] = q_nope.view(t, nh, dim)
        q[:, :, vd + dim:] = qa.view(t, nh, r + rd)[:, :, r:]
        o = torch.empty((t, nh * vd), dtype=self.act_dtype, device=q_nope.device)
        kernels.latent_attention_mma(q.view(t, nh * kd), o, nh, vd, dim + rd, rows, None, 64, ctx.cu_seqlens, ctx.seq_start,
                                     ctx.seq_slot, ctx.max_new, None, 1, head_stride=hs, out_scale=gate)
        self.o.add_into(o, residual)


register_part("mixer", "latent_attention", LatentAttention)
