"""Small Fofinex models for the tests: configurations that differ in every size and option, and weights drawn here
with numpy so that every mechanism carries weight in the logits (forget gates close to one, so that the matrix
memory reaches hundreds of tokens back; sharp attention scores, so that single far keys count; router corrections
large enough to make choice scores negative)."""
from __future__ import annotations

import json

import numpy as np
import torch

from qstream_b200.weights.safetensors_io import SafetensorsFile, write_safetensors


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, scaling=None, dims=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim if dims is None else dims, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def mlstm_layer(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=(1, 1), scale=1.0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# A: both mixers, a layer that reads another's latents with other head sizes, YaRN-scaled and plain rotations,
#    experts in groups with a shared expert and without groups or shared expert, a layer without feed-forward.
CONFIG_A = {
    "architecture": "Fofinex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        latent_layer(3, 16, 8, 24, 40, 48, 0.6, scaling=(4.0, 64, 8.0, 2.0), mlp=moe(8, 2, 24, groups=(4, 2), scale=1.5, shared=40)),
        mlstm_layer(2, 16, 24, 10.0, mlp=dense(96)),
        latent_layer(2, 8, 8, 16, 24, 48, 0.9, scaling=(4.0, 64, 8.0, 2.0), kv_from=0, mlp=None),
        mlstm_layer(3, 8, 16, 6.0, mlp=moe(6, 3, 16, scale=1.0)),
        latent_layer(2, 8, 16, 8, 16, 24, 0.4, base=500.0, mlp=dense(40)),
    ],
}
# B: sizes that are no multiples of 8, one head, one expert per token, groups of one expert, all groups kept, a cap
#    so large that it never binds and one that always does, a rotation over part of the rotated dims only.
CONFIG_B = {
    "architecture": "Fofinex", "vocab": 131, "width": 50, "norm": {"eps": 2e-6},
    "layers": [
        mlstm_layer(1, 12, 20, 50.0, mlp=moe(5, 1, 14, groups=(5, 3), scale=2.5, shared=18)),
        latent_layer(1, 10, 6, 14, 12, 20, 1.2, base=200.0, scaling=(16.0, 32, 4.0, 0.5), mlp=dense(36)),
        mlstm_layer(5, 4, 6, 0.7, mlp=None),
        latent_layer(4, 6, 12, 10, 18, 14, 0.5, base=1e5, dims=8, mlp=moe(4, 4, 10, groups=(2, 2), scale=0.5)),
        latent_layer(2, 12, 12, 6, 22, 14, 0.7, base=1e5, dims=8, kv_from=3, mlp=None),
    ],
}
# C: sizes that the bfloat16 tensor-core kernels take (multiples of 16), a latent wider than any head, sixteen
#    experts in eight groups.
CONFIG_C = {
    "architecture": "Fofinex", "vocab": 160, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        mlstm_layer(2, 48, 32, 15.0, mlp=dense(192)),
        latent_layer(4, 16, 32, 32, 48, 64, 0.35, base=5e5, scaling=(8.0, 128, 16.0, 1.0), mlp=moe(16, 3, 32, groups=(8, 5), scale=1.7, shared=64)),
        latent_layer(2, 32, 32, 48, 32, 64, 0.5, base=5e5, scaling=(8.0, 128, 16.0, 1.0), kv_from=1, mlp=dense(96)),
        mlstm_layer(4, 16, 64, 8.0, mlp=moe(8, 2, 48, groups=(2, 1), scale=1.0)),
    ],
}


def without_experts(cfg: dict) -> dict:
    """The same model with a dense feed-forward in the place of every mixture: nothing in it is chosen, so the
    bfloat16 engine's rounding moves no row by more than rounding."""
    out = json.loads(json.dumps(cfg))
    for layer in out["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            layer["mlp"] = dense(2 * layer["mlp"]["expert"]["ff"])
    return out


# W: a latent wider than the tensor-core prompt kernel takes (320 with the rotated part: prompts go through the
#    generic attention kernel, single tokens through the split-KV kernel), and a sharing layer right behind its source.
CONFIG_W = {
    "architecture": "Fofinex", "vocab": 120, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        latent_layer(2, 16, 32, 16, 24, 288, 0.3, base=1e4, scaling=(2.0, 64, 8.0, 1.0), mlp=dense(64)),
        latent_layer(3, 8, 32, 24, 40, 288, 0.25, base=1e4, scaling=(2.0, 64, 8.0, 1.0), kv_from=0, mlp=None),
    ],
}
# M: matrix memories only (the cache holds no keys at all).  L: latent attention only.
CONFIG_M = {
    "architecture": "Fofinex", "vocab": 64, "width": 48, "norm": {"eps": 1e-5},
    "layers": [mlstm_layer(2, 8, 24, 9.0, mlp=None), mlstm_layer(3, 16, 8, 20.0, mlp=dense(56))],
}
CONFIG_L = {
    "architecture": "Fofinex", "vocab": 72, "width": 64, "norm": {"eps": 1e-6},
    "layers": [latent_layer(4, 8, 8, 16, 32, 24, 0.5, base=300.0, mlp=moe(4, 2, 24, groups=(2, 1), scale=1.2, shared=16)),
               latent_layer(2, 16, 16, 8, 16, 48, 0.45, base=1e6, scaling=(32.0, 16, 2.0, 1.0), mlp=None)],
}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "Bd": without_experts(CONFIG_B), "Cd": without_experts(CONFIG_C),
           "W": CONFIG_W, "M": CONFIG_M, "L": CONFIG_L}


def make_weights(cfg: dict, seed: int) -> dict[str, np.ndarray]:
    """float32 arrays by checkpoint name; the caller rounds them to the stored type."""
    rng = np.random.default_rng(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(n_out, n_in, gain=1.0):
        return rng.normal(0.0, gain / np.sqrt(n_in), size=(n_out, n_in))

    def norm(n):
        return 1.0 + rng.normal(0, 0.2, n)

    w = {"embed": rng.normal(0, 1.0, (V, D)), "embed.norm": norm(D), "final.norm": norm(D)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = norm(D), norm(D) * 0.7
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "mlstm":
            for n, rows in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                w[p + "mix." + n] = mat(rows, D, 1.5)
            w[p + "mix.o"], w[p + "mix.norm"] = mat(D, H * dv, 1.5), norm(H * dv)
            w[p + "mix.i"], w[p + "mix.f"] = mat(H, D, 1.0), mat(H, D, 1.0)
            w[p + "mix.i.b"], w[p + "mix.f.b"] = rng.normal(0, 1.0, H), rng.normal(4.0, 1.0, H)
        else:
            dr, rq, r = m["rot_dim"], m["q_rank"], m["kv_rank"]
            w[p + "mix.dq"], w[p + "mix.dq.norm"] = mat(rq, D), norm(rq)
            w[p + "mix.uq"] = mat(H * (d + dr), rq, 1.0)
            if m.get("kv_from") is None:
                w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(r + dr, D, 1.5), norm(r)
            w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * d, r, 1.0), mat(H * dv, r, 1.5)
            w[p + "mix.o"] = mat(D, H * dv, 1.5)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"], w[p + "norm2b"] = norm(D), norm(D) * 0.7
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(F, D, 1.5), mat(F, D, 1.5), mat(D, F, 1.5)
            w[p + "mlp.gate.b"], w[p + "mlp.up.b"], w[p + "mlp.down.b"] = rng.normal(0, 0.3, F), rng.normal(0, 0.3, F), rng.normal(0, 0.3, D)
        else:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                w[f"{p}mlp.e{e}.up"], w[f"{p}mlp.e{e}.down"] = mat(F, D, 1.5), mat(D, F, 2.0)
            w[p + "mlp.router"], w[p + "mlp.correction"] = mat(E, D, 1.0), rng.normal(0, 0.5, E)
            if mlp.get("shared"):
                S = mlp["shared"]["ff"]
                w[p + "mlp.shared.up"], w[p + "mlp.shared.down"], w[p + "mlp.shared.sg"] = mat(S, D, 1.5), mat(D, S, 1.5), mat(1, D, 2.0)
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
    return write_folder(tmp_path / f"fofinex_{which}_{dtype}", cfg, make_weights(cfg, seed + "ABCWML".index(which[0])), dtype), cfg


def load_plain(folder):
    """(config dict, {name: float64 array}) of a folder, as the plain model takes them: the stored values exactly."""
    cfg = json.loads((folder / "config.json").read_text())
    f = SafetensorsFile(folder / "model.safetensors")
    try:
        w = {name: f.read(name).to(torch.float64).numpy().copy() for name in f.names()}
    finally:
        f.close()
    return cfg, w


def logits_error(got, ref):
    """Per row: the root mean square of the difference (means taken off) over that of the reference."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all()
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))


def is_routed(cfg: dict) -> bool:
    return any(layer.get("mlp") and layer["mlp"]["kind"] == "moe" for layer in cfg["layers"])


# float32: rounding of 32-bit sums and of the exponentials only, amplified by these weights (gates that span several
# powers of e, a quotient whose denominator is a sum that cancels); a structural fault is off by a hundred times
# the limit at least.  bfloat16: the weights are large on purpose, which
# also amplifies the rounding of activations between kernels; and where two experts' choice scores lie closer than
# that rounding, the bfloat16 engine may choose the other one, which moves that row's logits by a whole expert's
# output (and the rows after it a little, through the memories): so a few rows may lie outside the row limit, but
# not many, and the median must hold; a model without routed experts (`routed=False`) gets no such allowance.  A
# structural fault is off by the logits' whole spread in most rows.
F32_LIMIT = 2e-4
BF16_ROW_LIMIT, BF16_MEDIAN_LIMIT, BF16_OUTLIERS, BF16_OUTLIER_LIMIT = 1e-1, 3e-2, 0.12, 1.5


def assert_close(got, ref, dtype, what="", routed=False):
    e = logits_error(got, ref)
    if dtype == "float32":
        assert e.max() <= F32_LIMIT, f"{what}: error {e.max():.3e} of the logits' spread at row {int(e.argmax())} (limit {F32_LIMIT})"
        return
    over = e > BF16_ROW_LIMIT
    # without experts: a row in twenty, where the matrix memory's denominator nearly cancels, and never far
    allowed, worst = (max(1, int(BF16_OUTLIERS * len(e))), BF16_OUTLIER_LIMIT) if routed else (max(1, len(e) // 20), 0.5)
    assert over.sum() <= allowed and e.max() <= worst, \
        f"{what}: {int(over.sum())} of {len(e)} rows beyond {BF16_ROW_LIMIT}, worst {e.max():.3e} at row {int(e.argmax())}"
    assert np.median(e) <= BF16_MEDIAN_LIMIT, f"{what}: median error {np.median(e):.3e} of the logits' spread"
