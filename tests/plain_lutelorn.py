"""Plain, slow Lutelorn for the tests: whole sequences, no cache, one function per mechanism.

Lutelorn is a decoder-only model whose layers are listed in its config.json; each layer has one
of three mixers (softmax attention with grouped keys, a rotation on part of each head, a tanh cap
on the scores, values blended with an earlier layer's, and an output gate; linear attention with
a fixed decay per head; RWKV-style time mixing with a data-dependent decay per channel) and
optionally a gated feed-forward.  The residual stream is scaled by a constant at every sublayer.

Everything here is float64 numpy on whole sequences, written from the equations and sharing no
code with `qstream_b200` (the safetensors reader is the one of `plain_gptj`, also test code).
Notation: T tokens, D width, H heads, G key/value heads, dk / dv per-head sizes of keys / values.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from plain_gptj import read_safetensors


def load_model(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    for f in sorted(folder.glob("*.safetensors")):
        w.update(read_safetensors(f))
    return cfg, w


# --------------------------------------------------------------------------- small functions

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, weight, eps, offset=0.0):
    """x / sqrt(mean(x^2) + eps) * (offset + weight), over the last axis."""
    r = np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return x / r * (offset + weight)


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# --------------------------------------------------------------------------- embedding

def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous, current); the first token of a
    sequence takes the row behind the buckets."""
    tokens = np.asarray(tokens, dtype=np.int64)
    rows = np.empty(len(tokens), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (tokens[:-1] * mul_prev + tokens[1:] * mul_cur) % buckets
    return rows


def embed(cfg, w, tokens):
    e = cfg["embedding"]
    x = w["embed"][np.asarray(tokens)] * e["scale"]
    bg = e.get("bigram")
    if bg:
        x = x + w["bigram"][bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


# --------------------------------------------------------------------------- rotation

def rotate_pairs(v, positions, dims, base):
    """v [T, heads, d]: dims 2i and 2i+1 (2i < dims) turn by positions * base^(-2i/dims)."""
    out = v.copy()
    if not dims:
        return out
    i = np.arange(dims // 2)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- softmax attention

def capped_attention(q, k, v, scale, softcap):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; causal, every earlier key visible."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, h] = (p / p.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out


def attention_mixer(h, w, p, m, positions, eps, shared):
    """`shared` carries the first value-mixing layer's values to the later ones."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, positions, rot["dims"], rot["base"])
        k = rotate_pairs(k, positions, rot["dims"], rot["base"])
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = float(w[p + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    o = capped_attention(q, k, v, m["scale"], m.get("softcap"))
    o = o.reshape(T, H * dv) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- linear attention with decay

def decayed_linear_attention(q, k, v, decay):
    """Per head: S_t = decay S_{t-1} + k_t v_t^T (S [dk, dv], zero at the start), o_t = S_t^T q_t."""
    T, H, dk = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv))
    for h in range(H):
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def lightning_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    o = decayed_linear_attention(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms_norm(o, w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- time mixing (wkv)

def wkv_recurrence(r, k, v, decay, bonus):
    """Per head: o_t = (S_{t-1} + diag(bonus) k_t v_t^T)^T r_t, then S_t = diag(decay_t) S_{t-1} + k_t v_t^T.
    r, k, v, decay [T, H, d]; bonus [H, d]."""
    T, H, d = r.shape
    out = np.zeros((T, H, d))
    for h in range(H):
        S = np.zeros((d, d))
        for t in range(T):
            kv = np.outer(k[t, h], v[t, h])
            out[t, h] = (S + bonus[h][:, None] * kv).T @ r[t, h]
            S = decay[t, h][:, None] * S + kv
    return out


def wkv_mixer(h, w, p, m, eps):
    T, D = h.shape
    H, d = m["heads"], m["dim"]
    before = np.vstack([np.zeros((1, D)), h[:-1]])

    def mixed(name):
        return h + (before - h) * w[p + "mu." + name]

    r = (mixed("r") @ w[p + "r"].T).reshape(T, H, d)
    k = (mixed("k") @ w[p + "k"].T).reshape(T, H, d)
    v = (mixed("v") @ w[p + "v"].T).reshape(T, H, d)
    gate = silu(mixed("g") @ w[p + "g"].T)
    decay = np.exp(-np.exp(np.tanh(mixed("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).reshape(T, H, d)
    o = wkv_recurrence(r, k, v, decay, w[p + "u"])
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forward

def gated_mlp(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# --------------------------------------------------------------------------- the model

def residual_stream(cfg, w, tokens):
    """The residual stream after the embedding's layers: a list with one [T, D] array per layer."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    positions = np.arange(len(tokens))
    x = embed(cfg, w, tokens)
    shared, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps, 1.0)
        kind = layer["type"]
        if kind == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], positions, eps, shared)
        elif kind == "lightning":
            y = lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif kind == "wkv":
            y = wkv_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer '{kind}'")
        x = x + m * y
        if layer.get("mlp"):
            x = x + m * gated_mlp(rms_norm(x, w[p + "norm2"], eps, 1.0), w, p + "mlp.")
        after.append(x)
    return after


def logits_whole(cfg, w, tokens):
    """Logits [T, vocab] at every position of one sequence."""
    x = residual_stream(cfg, w, tokens)[-1]
    return rms_norm(x, w["final.norm"], cfg["norm"]["eps"], 1.0) @ w["head"].T


def generate_greedy(cfg, w, prompt, max_new_tokens):
    tokens = list(prompt)
    for _ in range(max_new_tokens):
        tokens.append(int(np.argmax(logits_whole(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
