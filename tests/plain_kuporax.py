"""Kuporax in plain numpy float64, one function per mechanism, whole sequences only.

It shares nothing with the package: it reads a config.json object and a {tensor name: array}
dictionary and walks a sequence from its first token.  The recurrent mixers run token by token
exactly as their update rules are written; attention builds the full score matrix.

Notation: T tokens, W model width; ``h`` [T, W] is a sublayer's input; a matrix M stored
[out, in] is applied as ``h @ M.T``.
"""
import numpy as np


# ---- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_scale(x, eps):
    """x divided by sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is a deviation from one."""
    return rms_scale(x, eps) * (1.0 + w)


def short_conv(u, taps, bias=None):
    """Causal per-channel filter.  u [T, C], taps [C, K]; the last column weighs the current
    token, column K-1-d the token d steps back; nothing before the sequence's start."""
    T, C = u.shape
    K = taps.shape[1]
    y = np.zeros((T, C))
    for d in range(min(K, T)):
        y[d:] += u[:T - d] * taps[:, K - 1 - d]
    if bias is not None:
        y = y + bias
    return y


def rotate_half(x, positions, base, dims):
    """x [T, H, D]: the first ``dims`` dimensions of each head turn; dimension i pairs with
    i + dims/2 and turns by positions * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None].astype(np.float64) * freq[None, :]            # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---- recurrences and attention on prepared inputs
def delta_scan(q, k, v, beta, decay, state=None):
    """q, k [T, G, D] (unit vectors, q scaled), v [T, H, V], beta and decay [T, H].  Per head:
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q.  Returns (out [T, H, V], S [H, D, V])."""
    T, H, V = v.shape
    G, D = q.shape[1], q.shape[2]
    S = np.zeros((H, D, V)) if state is None else state.copy()
    out = np.zeros((T, H, V))
    for head in range(H):
        g = head // (H // G)
        for t in range(T):
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + np.outer(k[t, g], u)
            out[t, head] = S[head].T @ q[t, g]
    return out, S


def ssd_scan(x, B, C, dt, rate, skip, state=None):
    """x [T, H, V], B and C [T, G, N], dt [T, H] (after softplus), rate = exp(A_log) [H], skip [H].
    S <- exp(-rate dt) S + dt B x^T; y = S^T C + skip x.  Returns (y [T, H, V], S [H, N, V])."""
    T, H, V = x.shape
    G, N = B.shape[1], B.shape[2]
    S = np.zeros((H, N, V)) if state is None else state.copy()
    y = np.zeros((T, H, V))
    for head in range(H):
        g = head // (H // G)
        for t in range(T):
            S[head] = np.exp(-rate[head] * dt[t, head]) * S[head] + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S[head].T @ C[t, g] + skip[head] * x[t, head]
    return y, S


def capped_attention(q, k, v, q_pos, k_pos, scale, cap, size):
    """q [Tq, H, D] at positions q_pos, k [Tk, G, D] and v [Tk, G, V] at positions k_pos.  A query
    at i sees the keys at j with 0 <= i - j < size (all earlier ones when size is None).
    score = (q . k) scale, then cap tanh(score / cap) when cap; softmax.  Returns [Tq, H, V]."""
    H, G = q.shape[1], k.shape[1]
    dist = np.asarray(q_pos)[:, None] - np.asarray(k_pos)[None, :]
    seen = (dist >= 0) & ((dist < size) if size else True)
    out = np.zeros((q.shape[0], H, v.shape[2]))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale
        if cap:
            s = cap * np.tanh(s / cap)
        s = np.where(seen, s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        out[:, head] = (p / p.sum(-1, keepdims=True)) @ v[:, g]
    return out


# ---- mixers
def delta_mixer(h, P, m, eps):
    """Gated delta rule.  P: the mixer's tensors by short name; m: its sizes."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ P["q"].T, P["q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ P["k"].T, P["k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ P["v"].T, P["v.conv"])).reshape(T, H, V)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ P["b"].T)                                            # [T, H]
    decay = np.exp(-np.exp(P["A_log"]) * softplus(h @ P["a"].T + P["dt_bias"]))
    gate = silu(h @ P["g"].T).reshape(T, H, V)
    out, _ = delta_scan(q, k, v, beta, decay)
    out = rms_scale(out, eps) * P["norm"] * gate
    return out.reshape(T, H * V) @ P["o"].T


def window_attention(h, P, m, eps):
    """Softmax attention with biases, short filters, partial rotation, capped scores, a sliding
    window and an output gate."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q, k, v = (h @ P[n].T + P[n + ".b"] for n in "qkv")
    if m["conv"]:
        q, k, v = (short_conv(x, P[n + ".conv"]) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rotate_half(q.reshape(T, H, D), pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half(k.reshape(T, G, D), pos, m["rot"]["base"], m["rot"]["dims"])
    out = capped_attention(q, k, v.reshape(T, G, V), pos, pos, m["scale"], m["softcap"], m["mask"]["size"])
    out = out.reshape(T, H * V) * sigmoid(h @ P["g"].T)
    return out @ P["o"].T


def ssd_mixer(h, P, m, eps):
    """Selective state space with a scalar decay per head."""
    T = h.shape[0]
    H, V, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * V
    zxbcdt = h @ P["in"].T
    z = zxbcdt[:, :inner]
    xbc = silu(short_conv(zxbcdt[:, inner:2 * inner + 2 * G * N], P["conv"], P["conv.b"]))
    dt = softplus(zxbcdt[:, 2 * inner + 2 * G * N:] + P["dt_bias"])         # [T, H]
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y, _ = ssd_scan(x, B, C, dt, np.exp(P["A_log"]), P["D"])
    y = y.reshape(T, inner) * silu(z)
    y = rms_scale(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * P["norm"]
    return y @ P["o"].T


def parallel_mixer(h, P, m, eps):
    left = window_attention(h, sub(P, "left."), m["left"], eps)
    right = ssd_mixer(h, sub(P, "right."), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ffn(h, P):
    return (gelu_tanh(h @ P["gate"].T) * (h @ P["up"].T)) @ P["down"].T


MIXERS = {"delta": delta_mixer, "parallel": parallel_mixer}


# ---- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token; with ``return_layers`` also the
    residual stream after every layer, [layers, T, W]."""
    tensors = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    tokens = np.asarray(tokens)
    eps = config["norm"]["eps"]
    x = tensors["embed"][tokens] + tensors["pos"][np.arange(len(tokens))]
    layers = []
    for i, layer in enumerate(config["layers"]):
        P = sub(tensors, f"l{i}.")
        mixed = MIXERS[layer["type"]](offset_norm(x, P["norm1"], eps), sub(P, "mix."), layer["mixer"], eps)
        x = x + offset_norm(mixed, P["norm1b"], eps)
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            y = dense_ffn(offset_norm(x, P["norm2"], eps), sub(P, "mlp."))
            x = x + offset_norm(y, P["norm2b"], eps)
        layers.append(x.copy())
    logits = (offset_norm(x, tensors["final.norm"], eps) @ tensors["head"].T) * config["logit_scale"]
    return (logits, np.stack(layers)) if return_layers else logits


def load_folder(folder):
    """(config.json object, {tensor name: float64 array}) of a model folder; the safetensors file
    is read here, by hand: 8 bytes of header length, the JSON header, then the data."""
    import json
    import os
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        tensors[name] = a.astype(np.float64).reshape(info["shape"])
    return config, tensors


def generate(config, tensors, prompt, n, stop=()):
    """Greedy continuation: (tokens, reason); the first largest logit wins; a stop token ends the
    run and is the last token returned."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, tensors, toks)[-1]))
        out.append(nxt)
        if nxt in stop:
            return out, "stop"
        toks.append(nxt)
    return out, "length"
