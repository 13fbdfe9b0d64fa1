"""Small Lutelorn models for the tests: configurations that differ in every size and option, and weights
drawn here with numpy so that every mechanism carries weight in the logits (the library's own random
weights are small and would let a wrong gate or a lost state pass)."""
from __future__ import annotations

import json

import numpy as np
import torch

from qstream_b200.weights.safetensors_io import write_safetensors


def attention_layer(heads, kv_heads, dim, vdim, rot=None, scale=None, softcap=0.0, v_mix=False, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
         "softcap": softcap, "v_mix": v_mix}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lightning_layer(dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def wkv_layer(heads, dim, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


DENSE = lambda ff: {"kind": "dense", "ff": ff}      # noqa: E731

# A: every mixer, grouped keys, a partial rotation, capped scores, values blended across three layers,
#    feed-forwards on some layers of each kind.
CONFIG_A = {
    "architecture": "Lutelorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
    "embedding": {"scale": 1.7, "bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 7}},
    "layers": [
        attention_layer(4, 2, 16, 8, rot=(8, 10000.0), softcap=5.0, v_mix=True, mlp=DENSE(96)),
        lightning_layer(16, 8, [0.5, 0.9, 0.995], mlp=None),
        wkv_layer(2, 32, mlp=DENSE(80)),
        attention_layer(4, 2, 16, 8, rot=(8, 10000.0), softcap=5.0, v_mix=True, mlp=None),
        lightning_layer(24, 40, [0.97, 0.8], mlp=DENSE(72)),
        attention_layer(2, 2, 32, 8, rot=None, softcap=0.0, v_mix=True, scale=0.3, mlp=None),
        wkv_layer(3, 16, mlp=None),
    ],
}
# B: sizes that A makes equal are different here and the other way round: one key head per query head, the whole
#    head rotated, values as wide as keys, no cap, no blending, a residual factor and an embedding scale of 1,
#    no pair table, one head, sizes that are no multiples of 8 or 16.
CONFIG_B = {
    "architecture": "Lutelorn", "vocab": 131, "width": 48, "norm": {"eps": 2e-6}, "residual_mult": 1.0,
    "embedding": {"scale": 1.0},
    "layers": [
        wkv_layer(1, 24, mlp=DENSE(50)),
        attention_layer(3, 3, 12, 12, rot=(12, 500.0), mlp=None),
        lightning_layer(20, 12, [0.93], mlp=DENSE(64)),
        attention_layer(6, 1, 10, 14, rot=(4, 2e5), softcap=12.0, mlp=DENSE(40)),
    ],
}
# C: head sizes that the bfloat16 tensor-core attention takes (multiples of 16), values narrower and wider than keys.
CONFIG_C = {
    "architecture": "Lutelorn", "vocab": 160, "width": 128, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
    "embedding": {"scale": 0.7, "bigram": {"buckets": 101, "mul_prev": 3, "mul_cur": 11}},
    "layers": [
        lightning_layer(32, 64, [0.9, 0.999], mlp=None),
        attention_layer(4, 2, 64, 32, rot=(32, 10000.0), softcap=8.0, v_mix=True, mlp=DENSE(192)),
        wkv_layer(2, 64, mlp=None),
        attention_layer(2, 2, 48, 32, rot=(16, 1e5), softcap=0.0, v_mix=True, mlp=None),
        attention_layer(2, 1, 16, 80, rot=None, softcap=20.0, scale=0.2, mlp=None),
    ],
}
# D: heads whose sizes do not add up to the width, one key head for five query heads, a value size that only the
#    generic attention kernel takes beside one that the tensor-core kernel takes, every layer with a feed-forward.
CONFIG_D = {
    "architecture": "Lutelorn", "vocab": 1000, "width": 160, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
    "embedding": {"scale": 2.0, "bigram": {"buckets": 997, "mul_prev": 1000003, "mul_cur": 999983}},
    "layers": [
        wkv_layer(5, 32, mlp=DENSE(200)),
        attention_layer(5, 1, 48, 32, rot=(24, 3e5), softcap=25.0, v_mix=True, mlp=DENSE(136)),
        lightning_layer(48, 16, [0.6, 0.99, 0.9999], mlp=DENSE(264)),
        attention_layer(5, 1, 48, 32, rot=(24, 3e5), softcap=25.0, v_mix=True, mlp=DENSE(136)),
        attention_layer(2, 2, 24, 40, rot=(8, 100.0), softcap=2.0, scale=0.5, mlp=DENSE(64)),
    ],
}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "D": CONFIG_D}


def make_weights(cfg: dict, seed: int, decay_rank: int = 5) -> dict[str, np.ndarray]:
    """float32 arrays by checkpoint name; the caller rounds them to the stored type."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n_out, n_in, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(n_in), size=(n_out, n_in))

    w = {"embed": rng.normal(0, 1.0, (V, D)), "final.norm": rng.normal(0, 0.2, D), "head": mat(V, D, 2.0)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        w["bigram"] = rng.normal(0, 1.0, (bg["buckets"] + 1, D))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = rng.normal(0, 0.2, D)
        H, d = m["heads"], m["dim"]
        if layer["type"] == "attention":
            G, dv = m["kv_heads"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(H * d, D), mat(G * d, D), mat(G * dv, D)
            w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"] = (rng.normal(0, 0.3, n) for n in (H * d, G * d, G * dv))
            w[p + "mix.g"], w[p + "mix.o"] = mat(H * dv, D), mat(D, H * dv, 1.5)
            if m.get("v_mix"):
                w[p + "mix.vmix"] = np.asarray(rng.uniform(0.25, 0.75))
        elif layer["type"] == "lightning":
            dv = m["vdim"]
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                w[p + "mix." + n] = mat(rows, D, 1.5)
            w[p + "mix.o"] = mat(D, H * dv, 1.5)
            w[p + "mix.norm"] = 1.0 + rng.normal(0, 0.2, H * dv)
        else:
            n = H * d
            for name in ("r", "k", "v", "g"):
                w[p + "mix." + name] = mat(n, D, 1.5)
                w[p + "mix.mu." + name] = rng.uniform(0, 1, D)
            w[p + "mix.mu.w"] = rng.uniform(0, 1, D)
            w[p + "mix.w1"], w[p + "mix.w2"] = mat(decay_rank, D, 2.0), mat(n, decay_rank, 2.0)
            w[p + "mix.w0"] = rng.normal(-1.0, 1.0, n)
            w[p + "mix.u"] = rng.normal(0, 0.5, (H, d))
            w[p + "mix.norm"] = 1.0 + rng.normal(0, 0.2, n)
            w[p + "mix.o"] = mat(D, n, 1.5)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            w[p + "norm2"] = rng.normal(0, 0.2, D)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, D, 1.5), mat(F, D, 1.5), mat(D, F, 1.5)
    return {k: np.asarray(v, dtype=np.float32) for k, v in w.items()}


def write_folder(folder, cfg: dict, weights: dict, dtype: str):
    """config.json + model.safetensors with the weights rounded to `dtype`."""
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    write_safetensors(folder / "model.safetensors", {k: torch.from_numpy(np.array(v, dtype=np.float32)).to(dt) for k, v in weights.items()})
    return folder


def make_folder(tmp_path, which: str, dtype: str, seed: int = 0):
    cfg = CONFIGS[which]
    return write_folder(tmp_path / f"lutelorn_{which}_{dtype}", cfg, make_weights(cfg, seed + "ABCD".index(which)), dtype), cfg


def logits_error(got, ref):
    """Per row: the root mean square of the difference (means taken off) over that of the reference."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all()
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))


# float32: rounding of 32-bit sums and of the exponentials only; fixed before the first run on a GPU.
# bfloat16: these weights are large on purpose (every branch moves the logits, so a wrong gate or a lost state
# shows), which also amplifies the rounding of activations to 8 bits of mantissa between kernels: a row may be off
# by a tenth of its spread, the rows of a request by 3 % on average.  A structural fault is off by the whole spread.
F32_LIMIT = 3e-5
BF16_ROW_LIMIT, BF16_MEAN_LIMIT = 1e-1, 3e-2


def assert_close(got, ref, dtype, what=""):
    e = logits_error(got, ref)
    limit = F32_LIMIT if dtype == "float32" else BF16_ROW_LIMIT
    assert e.max() <= limit, f"{what}: error {e.max():.3e} of the logits' spread at row {int(e.argmax())} (limit {limit})"
    if dtype == "bfloat16":
        assert e.mean() <= BF16_MEAN_LIMIT, f"{what}: mean error {e.mean():.3e} of the logits' spread"
