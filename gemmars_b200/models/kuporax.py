"""Kuporax: configuration, plan, tensor names.

A decoder whose layers carry a norm on both sides of each sublayer and whose mixers are of two
kinds, listed layer by layer in the configuration: ``delta`` (a gated delta rule) and ``parallel``
(softmax attention over a sliding window with capped scores beside a state-space recurrence, both
reading the same input, their outputs added with a factor each).  A learned vector per position is
added to the token embedding; the feed-forward is gated with the tanh form of GELU; the logits are
scaled by a constant.

config.json::

    {"architecture": "Kuporax", "vocab": V, "width": W, "max_positions": P, "logit_scale": s,
     "norm": {"eps": e},
     "layers": [{"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"},
                 "mlp": null | {"kind": "dense", "ff"}},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "conv", "scale", "softcap",
                                    "mask": {"size"}, "rot": {"base", "dims"}},
                           "right": {"heads", "vdim", "state", "groups", "norm_groups", "conv"},
                           "left_scale", "right_scale"},
                 "mlp": ...}, ...]}

Tensors: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b`` (stored
around zero), ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.

This module is all that knows the architecture: it turns the configuration into a ``ModelPlan``
of generic parts (``sandwich`` block, ``gated_delta``, ``side_by_side`` of ``capped_attention`` and
``ssd``, ``gated_mlp`` with ``gelu_tanh``, ``rmsnorm`` with offset 1, ``rotary``).
"""
from __future__ import annotations

import dataclasses
from typing import Tuple

from ..config.base import ConfigError, ModelConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("delta", "parallel")
FFN_KINDS = ("dense",)


def _num(problems, where, obj, name, kind=int, allow_zero=False):
    v = obj.get(name) if isinstance(obj, dict) else None
    ok = isinstance(v, int) and not isinstance(v, bool) if kind is int else (
        isinstance(v, (int, float)) and not isinstance(v, bool))
    if not ok:
        problems.append(f"{where}.{name}: expected {'an integer' if kind is int else 'a number'}, got {v!r}")
        return None
    if v < 0 or (v == 0 and not allow_zero):
        problems.append(f"{where}.{name}: must be positive, got {v!r}")
        return None
    return kind(v)


def _check_delta(p, w, m):
    for name in ("heads", "kv_heads", "dim", "vdim", "conv"):
        _num(p, w, m, name)
    if isinstance(m, dict) and isinstance(m.get("heads"), int) and isinstance(m.get("kv_heads"), int) and m["kv_heads"] > 0 \
            and m["heads"] % m["kv_heads"]:
        p.append(f"{w}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")


def _check_left(p, w, m):
    for name in ("heads", "kv_heads", "dim", "vdim"):
        _num(p, w, m, name)
    _num(p, w, m, "conv", allow_zero=True)
    _num(p, w, m, "scale", float)
    _num(p, w, m, "softcap", float, allow_zero=True)
    _num(p, w + ".mask", m.get("mask") if isinstance(m, dict) else None, "size")
    rot = m.get("rot") if isinstance(m, dict) else None
    _num(p, w + ".rot", rot, "base", float)
    dims = _num(p, w + ".rot", rot, "dims", allow_zero=True)
    if dims is not None and isinstance(m.get("dim"), int) and (dims % 2 or dims > m["dim"]):
        p.append(f"{w}.rot.dims: {dims} is odd or more than dim ({m['dim']})")


def _check_right(p, w, m):
    for name in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
        _num(p, w, m, name)


@dataclasses.dataclass(frozen=True)
class KuporaxConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    logit_scale: float
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
        max_positions = _num(p, "config", raw, "max_positions")
        logit_scale = _num(p, "config", raw, "logit_scale", float)
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
            kind, m = layer.get("type"), layer.get("mixer")
            if kind not in MIXERS:
                p.append(f"{w}.type: unknown mixer {kind!r} (known: {', '.join(MIXERS)})")
                continue
            if not isinstance(m, dict):
                p.append(f"{w}.mixer: expected an object")
                continue
            if kind == "delta":
                _check_delta(p, w + ".mixer", m)
            else:
                _check_left(p, w + ".mixer.left", m.get("left"))
                _check_right(p, w + ".mixer.right", m.get("right"))
                _num(p, w + ".mixer", m, "left_scale", float)
                _num(p, w + ".mixer", m, "right_scale", float)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in FFN_KINDS:
                got = mlp.get("kind") if isinstance(mlp, dict) else mlp
                p.append(f"{w}.mlp.kind: unknown feed-forward {got!r} (known: {', '.join(FFN_KINDS)})")
                continue
            _num(p, w + ".mlp", mlp, "ff")
        if p:
            raise ConfigError("config.json: " + "; ".join(p))
        return cls(vocab=vocab, width=width, max_positions=max_positions, logit_scale=logit_scale, norm_eps=eps,
                   layers=tuple(layers))

    def to_dict(self):
        return {"architecture": "Kuporax", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}


def _delta_spec(cfg, m, prefix) -> PartSpec:
    names = {k: prefix + k for k in ("q", "k", "v", "g", "b", "a", "o", "A_log", "dt_bias", "norm")}
    names.update({k + "_conv": f"{prefix}{k}.conv" for k in ("q", "k", "v")})
    return PartSpec("gated_delta", {"hidden_size": cfg.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]),
                                    "dim": int(m["dim"]), "vdim": int(m["vdim"]), "conv": int(m["conv"]),
                                    "norm_eps": cfg.norm_eps}, names)


def _left_spec(cfg, m, prefix) -> PartSpec:
    dims = int(m["rot"]["dims"])
    position = None
    if dims:
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(m["rot"]["base"]),
                                       "layout": "half"})
    taps = int(m["conv"])
    names = {k: prefix + k for k in ("q", "k", "v", "g", "o")}
    names.update({k + "_bias": f"{prefix}{k}.b" for k in ("q", "k", "v")})
    if taps:
        names.update({k + "_conv": f"{prefix}{k}.conv" for k in ("q", "k", "v")})
    return PartSpec("capped_attention", {
        "hidden_size": cfg.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "bias": True, "conv": taps, "window": int(m["mask"]["size"]), "scale": float(m["scale"]),
        "softcap": float(m["softcap"]), "gate": True, "position": position}, names)


def _right_spec(cfg, m, prefix) -> PartSpec:
    names = {k: prefix + k for k in ("in", "o", "conv", "dt_bias", "A_log", "D", "norm")}
    names["conv_bias"] = prefix + "conv.b"
    return PartSpec("ssd", {"hidden_size": cfg.width, "heads": int(m["heads"]), "vdim": int(m["vdim"]),
                            "state": int(m["state"]), "groups": int(m["groups"]), "norm_groups": int(m["norm_groups"]),
                            "conv": int(m["conv"]), "norm_eps": cfg.norm_eps}, names)


def _mixer_spec(cfg, layer, prefix) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "delta":
        return _delta_spec(cfg, m, prefix)
    return PartSpec("side_by_side", {"branches": [
        {"name": "left", "spec": _left_spec(cfg, m["left"], prefix + "left."), "scale": float(m["left_scale"])},
        {"name": "right", "spec": _right_spec(cfg, m["right"], prefix + "right."), "scale": float(m["right_scale"])}]})


def build_plan(cfg: KuporaxConfig, names=None) -> ModelPlan:
    def norm(name, after=False):
        params = {"size": cfg.width, "eps": cfg.norm_eps, "offset": 1.0}
        if after:
            params["after_sublayer"] = True
        return PartSpec("rmsnorm", params, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        parts = {"mixer_norm": norm(f"l{i}.norm1"), "mixer": _mixer_spec(cfg, layer, f"l{i}.mix."),
                 "mixer_post_norm": norm(f"l{i}.norm1b", True)}
        if layer.get("mlp") is not None:
            parts["ffn_norm"] = norm(f"l{i}.norm2")
            parts["ffn"] = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": int(layer["mlp"]["ff"]),
                                                  "activation": "gelu_tanh"},
                                    {k: f"l{i}.mlp.{k}" for k in ("gate", "up", "down")})
            parts["ffn_post_norm"] = norm(f"l{i}.norm2b", True)
        layers.append(LayerSpec(parts, "sandwich"))
    plan = ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": None,
                                         "positions": cfg.max_positions}, {"weight": "embed", "positions": "pos"}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "logit_scale": cfg.logit_scale},
                      {"weight": "head"}),
        max_positions=cfg.max_positions, stop_ids=[],
        # a layer without a feed-forward may still carry the norms around one
        ignored_tensors=[f"l{i}.norm2*" for i, layer in enumerate(cfg.layers) if layer.get("mlp") is None])
    plan.validate()
    return plan


def checkpoint_layout(cfg: KuporaxConfig) -> dict:
    """{tensor name: (shape, kind)} of a complete checkpoint (kind as weights.random_init reads it)."""
    w = cfg.width
    out = {"embed": ((cfg.vocab, w), "matrix"), "pos": ((cfg.max_positions, w), "matrix")}
    for i, layer in enumerate(cfg.layers):
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") is not None else ()):
            out[f"l{i}.{n}"] = ((w,), "small")
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "delta":
            nh, g, d, vd, k = (int(m[x]) for x in ("heads", "kv_heads", "dim", "vdim", "conv"))
            for n, rows in (("q", g * d), ("k", g * d), ("v", nh * vd)):
                out[p + n] = ((rows, w), "matrix")
                out[p + n + ".conv"] = ((rows, k), "filter")
            out[p + "g"] = ((nh * vd, w), "matrix")
            out[p + "b"] = ((nh, w), "matrix")
            out[p + "a"] = ((nh, w), "matrix")
            out[p + "A_log"] = ((nh,), "log_rate")
            out[p + "dt_bias"] = ((nh,), "small")
            out[p + "norm"] = ((vd,), "norm")
            out[p + "o"] = ((w, nh * vd), "matrix")
        else:
            a, q = m["left"], p + "left."
            nh, g, d, vd, k = (int(a[x]) for x in ("heads", "kv_heads", "dim", "vdim", "conv"))
            for n, rows in (("q", nh * d), ("k", g * d), ("v", g * vd)):
                out[q + n] = ((rows, w), "matrix")
                out[q + n + ".b"] = ((rows,), "bias")
                if k:
                    out[q + n + ".conv"] = ((rows, k), "filter")
            out[q + "g"] = ((nh * vd, w), "matrix")
            out[q + "o"] = ((w, nh * vd), "matrix")
            s, q = m["right"], p + "right."
            nh, vd, n_state, g, k = (int(s[x]) for x in ("heads", "vdim", "state", "groups", "conv"))
            inner, ch = nh * vd, nh * vd + 2 * g * n_state
            out[q + "in"] = ((inner + ch + nh, w), "matrix")
            out[q + "conv"] = ((ch, k), "filter")
            out[q + "conv.b"] = ((ch,), "bias")
            out[q + "dt_bias"] = ((nh,), "small")
            out[q + "A_log"] = ((nh,), "log_rate")
            out[q + "D"] = ((nh,), "norm")
            out[q + "norm"] = ((inner,), "norm")
            out[q + "o"] = ((w, inner), "matrix")
        if layer.get("mlp") is not None:
            ff = int(layer["mlp"]["ff"])
            out[f"l{i}.mlp.gate"] = ((ff, w), "matrix")
            out[f"l{i}.mlp.up"] = ((ff, w), "matrix")
            out[f"l{i}.mlp.down"] = ((w, ff), "matrix")
    out["final.norm"] = ((w,), "small")
    out["head"] = ((cfg.vocab, w), "matrix")
    return out


register_architecture(["Kuporax", "kuporax"], KuporaxConfig, build_plan, checkpoint_layout)
