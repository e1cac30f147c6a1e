"""Several mixers side by side: all read the same input, and the layer's mixer output is the
sum of theirs, each times a factor of its own.

``branches``: a list of {"name", "spec" (the branch's PartSpec), "scale"}.  Each branch adds
into the same float32 rows, in the order listed; the factor is handed to the branch as its
``out_scale`` parameter, which it applies in float32 before its output product.  Tensors, cache
needs, kernels and weight bytes are the branches' own, its tensors under ``<name>.<short name>``.
"""
from __future__ import annotations

import dataclasses

from .base import Part, build_part, register_part


class SideBySide(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.branches = []
        for br in spec.params["branches"]:
            child = br["spec"]
            scale = float(br.get("scale", 1.0)) * float(child.params.get("out_scale", 1.0))
            child = dataclasses.replace(child, params={**child.params, "out_scale": scale})
            self.branches.append((str(br["name"]), build_part("mixer", child, compute)))
        if not self.branches:
            raise ValueError("side_by_side: no branches")
        # the checkpoint names of the branches' tensors, under this part's own short names
        for name, part in self.branches:
            for short, ckpt in part.spec.tensors.items():
                spec.tensors.setdefault(f"{name}.{short}", ckpt)

    def wants(self):
        return {f"{name}.{short}": want for name, part in self.branches for short, want in part.wants().items()}

    def load(self, tensors):
        for name, part in self.branches:
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    def kernel_units(self):
        return [u for _, part in self.branches for u in part.kernel_units()]

    def cache_needs(self):
        return [n for _, part in self.branches for n in part.cache_needs()]

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.branches)

    @property
    def capture_depends_on_length(self):
        return any(part.capture_depends_on_length for _, part in self.branches)

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        at = 0
        caches = list(caches or [])
        for _, part in self.branches:
            n = len(part.cache_needs())
            part.forward(ctx, h, residual, caches[at:at + n], writes_cache)
            at += n


register_part("mixer", "side_by_side", SideBySide)
