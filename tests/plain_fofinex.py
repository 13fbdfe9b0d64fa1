"""A plain, slow Fofinex in numpy float64: one function per mechanism, written from the design's equations.

It shares no code with the library: the tests compare the library's kernels, cache and step function with it.
A model is (config dict as in config.json, {tensor name: float64 array}); `forward` runs one whole sequence
and returns the logits of every position (and, if asked, the residual stream after every layer).
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small pieces

def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, variance = mean squared deviation; no bias."""
    mu = x.mean(-1, keepdims=True)
    d = x - mu
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w may be 1)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


# ----------------------------------------------------------------------------- rotation

def yarn_frequencies(dims, base, scaling):
    """The dims/2 frequencies and the factor on cos and sin.  `scaling` None: plain rotary frequencies, factor 1."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, dims, base, scaling):
    """x [T, ..., n]: the first `dims` of the last axis rotated, element i paired with i + dims/2."""
    f, mag = yarn_frequencies(dims, base, scaling)
    half = dims // 2
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]                 # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    cos, sin = (np.cos(a) * mag).reshape(shape), (np.sin(a) * mag).reshape(shape)
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------- latent attention

def latent_kv(h, positions, m, W, p, eps):
    """What a latent-attention layer caches for its tokens: the normed latent c [T, kv_rank] and the rotated
    shared key part [T, rot_dim]."""
    r = m["kv_rank"]
    ckv = h @ W[p + "dkv"].T
    c = rms_norm(ckv[:, :r], W[p + "dkv.norm"], eps)
    rot = m["rot"]
    k_rot = rotate_half(ckv[:, r:], positions, rot["dims"], rot["base"], rot.get("scaling"))
    return c, k_rot


def latent_attention(h, positions, m, W, p, eps, shared=None):
    """h [T, width] of one sequence from its first token on.  `shared` = (c, k_rot) of another layer."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).reshape(T, H, dn + dr)
    c, k_rot = shared if shared is not None else latent_kv(h, positions, m, W, p, eps)
    rot = m["rot"]
    q_nope = q[..., :dn]
    q_rot = rotate_half(q[..., dn:], positions, rot["dims"], rot["base"], rot.get("scaling"))
    k_nope = (c @ W[p + "uk"].T).reshape(T, H, dn)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hd in range(H):
        s = (q_nope[:, hd] @ k_nope[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        w = np.exp(s - s.max(-1, keepdims=True))
        w /= w.sum(-1, keepdims=True)
        out[:, hd] = w @ v[:, hd]
    return out.reshape(T, H * dv) @ W[p + "o"].T, (c, k_rot)


# ----------------------------------------------------------------------------- mLSTM

def mlstm(h, m, W, p, eps):
    """Matrix memory with exponential gating, token by token from an empty state."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)                      # log input gate [T, H]
    gf = log_sigmoid(cap * np.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))         # log forget gate
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S, n, mx = np.zeros((dk, dv)), np.zeros(dk), 0.0
        for t in range(T):
            m_new = max(gf[t, hd] + mx, gi[t, hd])
            a, b = math.exp(gf[t, hd] + mx - m_new), math.exp(gi[t, hd] - m_new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            o = S.T @ q[t, hd] / (max(abs(n @ q[t, hd]), math.exp(-mx)) + 1e-6)
            out[t, hd] = o / math.sqrt((o * o).mean() + eps)
    y = out.reshape(T, H * dv) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward

def dense_ff(h, W, p):
    a = h @ W[p + "gate"].T + W[p + "gate.b"]
    b = h @ W[p + "up"].T + W[p + "up.b"]
    return (gelu_tanh(a) * b) @ W[p + "down"].T + W[p + "down.b"]


def expert(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def route(h, mlp, W, p):
    """For each token the chosen experts and their weights: ([T, top] indices, [T, top] weights)."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    groups, keep = r["groups"]["count"], r["groups"]["keep"]
    s = sigmoid(h @ W[p + "router"].T)                                               # [T, E]
    choice = s + W[p + "correction"]
    per = E // groups
    idx = np.zeros((h.shape[0], top), dtype=np.int64)
    wts = np.zeros((h.shape[0], top))
    for t in range(h.shape[0]):
        g = choice[t].reshape(groups, per)
        group_score = np.sort(g, axis=1)[:, ::-1][:, :2].sum(1)
        kept = np.argsort(-group_score, kind="stable")[:keep]
        masked = np.full(E, -np.inf)
        for gi in kept:
            masked[gi * per:(gi + 1) * per] = choice[t, gi * per:(gi + 1) * per]
        chosen = np.argsort(-masked, kind="stable")[:top]
        idx[t] = chosen
        wts[t] = s[t, chosen] * r["scale"]
    return idx, wts


def moe_ff(h, mlp, W, p):
    idx, wts = route(h, mlp, W, p)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wts[t]):
            out[t] += w * expert(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += expert(h, W, p + "shared.") * sigmoid(h @ W[p + "shared.sg"].T)
    return out


# ----------------------------------------------------------------------------- the model

def forward(config, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence given whole."""
    eps = float(config["norm"]["eps"])
    tokens = np.asarray(tokens)
    T = len(tokens)
    positions = np.arange(T)
    x = layer_norm(W["embed"][tokens], W["embed.norm"], eps)
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        h = layer_norm(x, W[f"l{i}.norm1"], eps)
        if layer["type"] == "latent_attention":
            y, kept[i] = latent_attention(h, positions, m, W, p, eps, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "mlstm":
            y = mlstm(h, m, W, p, eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, W[f"l{i}.norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, W[f"l{i}.norm2"], eps)
            y = dense_ff(h, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(h, mlp, W, f"l{i}.mlp.")
            x = x + layer_norm(y, W[f"l{i}.norm2b"], eps)
        after.append(x.copy())
    logits = layer_norm(x, W["final.norm"], eps) @ W["embed"].T
    return (logits, np.stack(after)) if return_layers else logits
