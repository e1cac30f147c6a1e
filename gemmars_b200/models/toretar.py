"""Toretar: configuration, plan, tensor names.

A decoder whose layers are parallel blocks: one RMSNorm, and a latent attention mixer and a
routed feed-forward (with a shared expert) that both read the norm's output and both add into the
residual stream.  The configuration lists the layers one by one; every layer carries its own
mixer sizes and its own feed-forward (or none), so layers of one model may differ.

config.json::

    {"architecture": "Toretar", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                                "shared": null | {"ff", "limit"}}}, ...]}

Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}``,
``l<i>.mlp.{router,router.b,e<j>.{gate,up,down},shared.{gate,up,down,sg}}``, ``final.norm``, ``head``.

This module is all that knows the architecture: it turns the configuration into a ``ModelPlan``
of generic parts (``parallel`` block, ``latent_attention`` mixer, ``moe`` feed-forward, ``rmsnorm``,
``rotary`` with interleaved pairs).
"""
from __future__ import annotations

import dataclasses
from typing import Tuple

from ..config.base import ConfigError, ModelConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("latent_attention",)
FFN_KINDS = ("moe",)
#: constants of the experts' activation that the design fixes: y = g * sigmoid(ALPHA g) * (u + SHIFT)
ALPHA, SHIFT = 1.702, 1.0


def _num(problems, where, obj, name, kind=int, positive=True, allow_zero=False):
    v = obj.get(name) if isinstance(obj, dict) else None
    ok = isinstance(v, int) and not isinstance(v, bool) if kind is int else (
        isinstance(v, (int, float)) and not isinstance(v, bool))
    if not ok:
        problems.append(f"{where}.{name}: expected {'an integer' if kind is int else 'a number'}, got {v!r}")
        return None
    if positive and (v < 0 or (v == 0 and not allow_zero)):
        problems.append(f"{where}.{name}: must be positive, got {v!r}")
        return None
    return kind(v)


@dataclasses.dataclass(frozen=True)
class ToretarConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    #: one entry per layer, as config.json lists them (checked; plain dicts)
    layers: Tuple[dict, ...]

    @classmethod
    def from_dict(cls, raw):
        if not isinstance(raw, dict):
            raise ConfigError("config.json: the top level must be an object")
        p = []
        vocab = _num(p, "config", raw, "vocab")
        width = _num(p, "config", raw, "width")
        eps = _num(p, "norm", raw.get("norm"), "eps", float)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            p.append("layers: expected a list of at least one layer")
            layers = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]"
            if not isinstance(layer, dict):
                p.append(f"{w}: expected an object")
                continue
            if layer.get("type") not in MIXERS:
                p.append(f"{w}.type: unknown mixer {layer.get('type')!r} (known: {', '.join(MIXERS)})")
                continue
            m = layer.get("mixer")
            for name in ("heads", "vdim", "kv_rank"):
                _num(p, w + ".mixer", m, name)
            dim = _num(p, w + ".mixer", m, "dim", allow_zero=True)
            rd = _num(p, w + ".mixer", m, "rot_dim", allow_zero=True)
            _num(p, w + ".mixer", m, "scale", float)
            if dim == 0 and rd == 0:
                p.append(f"{w}.mixer: dim and rot_dim are both 0")
            if rd:
                rot = m.get("rot") if isinstance(m, dict) else None
                _num(p, w + ".mixer.rot", rot, "base", float)
                dims = _num(p, w + ".mixer.rot", rot, "dims", allow_zero=True)
                if dims is not None and (dims % 2 or dims > rd):
                    p.append(f"{w}.mixer.rot.dims: {dims} is odd or more than rot_dim ({rd})")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in FFN_KINDS:
                kind = mlp.get("kind") if isinstance(mlp, dict) else mlp
                p.append(f"{w}.mlp.kind: unknown feed-forward {kind!r} (known: {', '.join(FFN_KINDS)})")
                continue
            experts = _num(p, w + ".mlp.router", mlp.get("router"), "experts")
            top = _num(p, w + ".mlp.router", mlp.get("router"), "top")
            if experts and top and top > experts:
                p.append(f"{w}.mlp.router.top: {top} of {experts} experts")
            _num(p, w + ".mlp.expert", mlp.get("expert"), "ff")
            _num(p, w + ".mlp.expert", mlp.get("expert"), "limit", float)
            if mlp.get("shared") is not None:
                _num(p, w + ".mlp.shared", mlp.get("shared"), "ff")
                _num(p, w + ".mlp.shared", mlp.get("shared"), "limit", float)
        if p:
            raise ConfigError("config.json: " + "; ".join(p))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def to_dict(self):
        return {"architecture": "Toretar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": [dict(layer) for layer in self.layers]}


def _mixer_spec(cfg: ToretarConfig, m: dict, prefix: str) -> PartSpec:
    rd = int(m["rot_dim"])
    rot = m.get("rot") or {}
    position = None
    if rd and int(rot.get("dims", 0)):
        position = PartSpec("rotary", {"head_dim": rd, "rotary_dim": int(rot["dims"]), "theta": float(rot["base"]),
                                       "layout": "interleaved"})
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": rd,
        "vdim": int(m["vdim"]), "rank": int(m["kv_rank"]), "scale": float(m["scale"]), "norm_eps": cfg.norm_eps,
        "gate": True, "window": None, "position": position,
    }, {"q": prefix + "q", "dkv": prefix + "dkv", "dkv_norm": prefix + "dkv.norm", "uk": prefix + "uk",
        "uv": prefix + "uv", "g": prefix + "g", "o": prefix + "o"})


def _ffn_spec(cfg: ToretarConfig, mlp: dict, prefix: str) -> PartSpec:
    experts = int(mlp["router"]["experts"])
    shared = mlp.get("shared")
    names = {"router": prefix + "router", "router_bias": prefix + "router.b"}
    for e in range(experts):
        for part in ("gate", "up", "down"):
            names[f"e{e}.{part}"] = f"{prefix}e{e}.{part}"
    if shared is not None:
        for part in ("gate", "up", "down", "sg"):
            names[f"shared.{part}"] = f"{prefix}shared.{part}"
    return PartSpec("moe", {
        "hidden_size": cfg.width, "experts": experts, "top": int(mlp["router"]["top"]),
        "ff": int(mlp["expert"]["ff"]), "limit": float(mlp["expert"]["limit"]), "alpha": ALPHA, "shift": SHIFT,
        "router_bias": True,
        "shared": None if shared is None else {"ff": int(shared["ff"]), "limit": float(shared["limit"]), "gate": True},
    }, names)


def build_plan(cfg: ToretarConfig, names=None) -> ModelPlan:
    def norm(name):
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"norm": norm(f"l{i}.norm1"), "mixer": _mixer_spec(cfg, layer["mixer"], f"l{i}.mix.")}
        if layer.get("mlp") is not None:
            parts["ffn"] = _ffn_spec(cfg, layer["mlp"], f"l{i}.mlp.")
        layers.append(LayerSpec(parts, "parallel"))
    plan = ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": None},
                           {"weight": "embed"}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width}, {"weight": "head"}),
        max_positions=0, stop_ids=[])
    plan.validate()
    return plan


def checkpoint_layout(cfg: ToretarConfig) -> dict:
    """{tensor name: (shape, kind)} of a complete checkpoint (kind as weights.random_init reads it)."""
    w = cfg.width
    out = {"embed": ((cfg.vocab, w), "matrix")}
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        nh, dim, rd, vd, r = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        p = f"l{i}.mix."
        out[f"l{i}.norm1"] = ((w,), "norm")
        out[p + "q"] = ((nh * (dim + rd), w), "matrix")
        out[p + "dkv"] = ((r + rd, w), "matrix")
        out[p + "dkv.norm"] = ((r,), "norm")
        out[p + "uk"] = ((nh * dim, r), "matrix")
        out[p + "uv"] = ((nh * vd, r), "matrix")
        out[p + "g"] = ((nh, w), "matrix")
        out[p + "o"] = ((w, nh * vd), "matrix")
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        p = f"l{i}.mlp."
        ff = int(mlp["expert"]["ff"])
        for e in range(int(mlp["router"]["experts"])):
            out[f"{p}e{e}.gate"] = ((ff, w), "matrix")
            out[f"{p}e{e}.up"] = ((ff, w), "matrix")
            out[f"{p}e{e}.down"] = ((w, ff), "matrix")
        out[p + "router"] = ((int(mlp["router"]["experts"]), w), "matrix")
        out[p + "router.b"] = ((int(mlp["router"]["experts"]),), "bias")
        if mlp.get("shared") is not None:
            fs = int(mlp["shared"]["ff"])
            out[p + "shared.gate"] = ((fs, w), "matrix")
            out[p + "shared.up"] = ((fs, w), "matrix")
            out[p + "shared.down"] = ((w, fs), "matrix")
            out[p + "shared.sg"] = ((1, w), "matrix")
    out["final.norm"] = ((w,), "norm")
    out["head"] = ((cfg.vocab, w), "matrix")
    return out


register_architecture(["Toretar", "toretar"], ToretarConfig, build_plan, checkpoint_layout)
