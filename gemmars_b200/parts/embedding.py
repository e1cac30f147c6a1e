"""Token embedding and output head.

Embedding: x[t] = E[token[t]] (* scale when the plan gives one), into the float32 residual
stream (src/qwen.rs:669-672: no scale).  Head: logits = h @ W.T in float32, for the rows that
are asked for only (src/qwen.rs:632-638); its weight may be the embedding's tensor (tied,
src/qwen.rs:472-485).

``positions`` (embedding, default none): rows of a second table, a learned vector per position
that is added to the token's row unscaled, x[t] += P[position of t]; a sequence cannot grow
beyond the table.  ``logit_scale`` (head, default 1): the float32 logits are multiplied by it."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part
from .linear import Linear


class Embedding(Part):
    category = "embedding"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.scale = spec.params.get("scale") or 1.0
        self.n_positions = int(spec.params.get("positions") or 0)
        self.table = self.positions = None

    def wants(self):
        w = {"weight": TensorWant((self.vocab_size, self.hidden_size), "matrix")}
        if self.n_positions:
            w["positions"] = TensorWant((self.n_positions, self.hidden_size), "matrix")
        return w

    def load(self, tensors):
        self.table = tensors["weight"].contiguous()
        if self.n_positions:
            self.positions = tensors["positions"].contiguous()

    def kernel_units(self):
        return [("elementwise", ())] + ([("rows", ())] if self.n_positions else [])

    def forward(self, ctx, tokens, out):
        kernels.embed_gather(self.table, tokens, out, float(self.scale))
        if self.n_positions:
            if ctx.max_total > self.n_positions and ctx.pad_slot is None:
                raise ValueError(f"a sequence of {ctx.max_total} tokens is longer than the position table "
                                 f"({self.n_positions} rows)")
            kernels.gather_add(self.positions, ctx.tok_pos, out)


class LinearHead(Part):
    category = "head"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.vocab_size = int(spec.params["vocab_size"])
        self.hidden_size = int(spec.params["hidden_size"])
        self.logit_scale = float(spec.params.get("logit_scale") or 1.0)
        self.proj = None

    def wants(self):
        return {"weight": TensorWant((self.vocab_size, self.hidden_size), "matrix")}

    def load(self, tensors):
        self.proj = Linear(tensors["weight"])

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + ([("rows", ())] if self.logit_scale != 1.0 else [])

    def forward(self, ctx, h):
        with kernels.profile_category("lm_head"):
            logits = self.proj(h, out_dtype=torch.float32)
            if self.logit_scale != 1.0:
                kernels.scale_rows(logits, self.logit_scale)
            return logits

    def weight_bytes(self):
        return self.proj.bytes()


register_part("embedding", "embedding", Embedding)
register_part("head", "linear_head", LinearHead)
