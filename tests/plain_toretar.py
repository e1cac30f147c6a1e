"""A plain, slow implementation of the Toretar design in float64 numpy, one function per
mechanism, written from the design's equations.  It shares no code with the package: it reads
the safetensors file itself and expands every head's keys and values from the latents, which the
package never does.

Notation: x [T, W] residual rows; h = norm(x); per layer  x <- x + mixer(h) + ffn(h).
"""
import json
import os
import struct

import numpy as np


def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = data[a:b]
        if info["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = arr.astype(np.float64).reshape(info["shape"])
    return out


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rotate_pairs(v, positions, dims, base):
    """v [T, ..., d]: dims 2i and 2i+1 (i < dims/2) turn by positions * base^(-2i/dims); the rest stay."""
    out = v.copy()
    for i in range(dims // 2):
        ang = np.asarray(positions, dtype=np.float64) * base ** (-2.0 * i / dims)
        c = np.cos(ang).reshape((-1,) + (1,) * (v.ndim - 2))
        s = np.sin(ang).reshape((-1,) + (1,) * (v.ndim - 2))
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def softmax(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def latent_attention(h, w, p, m, eps, positions=None):
    """The mixer on rows h [T, W] of ONE sequence from position 0 (or at ``positions``, all keys
    of which are in h)."""
    t = h.shape[0]
    positions = np.arange(t) if positions is None else positions
    nh, dim, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(t, nh, dim + rd)
    kv = h @ w[p + "dkv"].T
    c = rms_norm(kv[:, :r], w[p + "dkv.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    kr = rotate_pairs(kv[:, r:], positions, rot["dims"], rot["base"])            # [T, rd], one for all heads
    qr = rotate_pairs(q[:, :, dim:], positions, rot["dims"], rot["base"])        # [T, nh, rd]
    ku = (c @ w[p + "uk"].T).reshape(t, nh, dim)
    v = (c @ w[p + "uv"].T).reshape(t, nh, vd)
    out = np.zeros((t, nh, vd))
    for i in range(t):
        for a in range(nh):
            s = (ku[:i + 1, a] @ q[i, a, :dim] + kr[:i + 1] @ qr[i, a]) * m["scale"]
            out[i, a] = softmax(s) @ v[:i + 1, a]
    gate = sigmoid(h @ w[p + "g"].T)                                           # [T, nh]
    return (out * gate[:, :, None]).reshape(t, nh * vd) @ w[p + "o"].T


def expert(h, gate, up, down, limit, alpha=1.702, shift=1.0):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + shift)) @ down.T


def route(h, router, bias, top):
    """(indices [T, top] by falling logit, weights [T, top] = softmax over the chosen logits)."""
    z = h @ router.T + bias
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    return idx, softmax(np.take_along_axis(z, idx, -1))


def moe(h, w, p, mlp):
    idx, wt = route(h, w[p + "router"], w[p + "router.b"], mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            e = f"{p}e{idx[t, k]}."
            out[t] += wt[t, k] * expert(h[t:t + 1], w[e + "gate"], w[e + "up"], w[e + "down"], mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        s = p + "shared."
        out += sigmoid(h @ w[s + "sg"].T) * expert(h, w[s + "gate"], w[s + "up"], w[s + "down"], mlp["shared"]["limit"])
    return out


def layer(x, w, i, spec, eps):
    h = rms_norm(x, w[f"l{i}.norm1"], eps)
    y = latent_attention(h, w, f"l{i}.mix.", spec["mixer"], eps)
    if spec.get("mlp") is not None:
        y = y + moe(h, w, f"l{i}.mlp.", spec["mlp"])
    return x + y


def forward(cfg, w, tokens, residuals=None):
    """Logits [T, vocab] of one sequence; ``residuals`` (a list) receives x after every layer."""
    x = w["embed"][np.asarray(tokens)]
    eps = cfg["norm"]["eps"]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, eps)
        if residuals is not None:
            residuals.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def generate(cfg, w, prompt, max_tokens, stop=()):
    """Greedy: the first largest logit, until a stop token (kept in the output) or max_tokens."""
    toks, out = list(prompt), []
    for _ in range(max_tokens):
        nxt = int(np.argmax(forward(cfg, w, toks)[-1]))
        out.append(nxt)
        if nxt in stop:
            return out, "stop"
        toks.append(nxt)
    return out, "length"
