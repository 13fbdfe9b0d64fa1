"""Lutelorn's configuration, read from its own config.json keys.

A Lutelorn model lists its layers: `layers[i]` names the layer's mixer (`type`: "attention", "lightning" or
"wkv"), the mixer's sizes and constants (`mixer`), and its feed-forward (`mlp`: {"kind": "dense", "ff": n} or
null).  Around them: `vocab`, `width`, `norm.eps`, `residual_mult`, `embedding.scale` and
`embedding.bigram` (`buckets`, `mul_prev`, `mul_cur`).  Every size and constant comes from these keys; the one
size they do not give, the rank of the wkv mixer's decay bottleneck, is taken from the checkpoint's tensors
(a model made here writes it as `mixer.decay_rank`).  The model names no longest sequence; `max_positions`
(the library's own key, default 32,768) bounds the table of rotation angles and the engine's context.

Tensor names: `embed`, `bigram`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.<name>`, `l<i>.mlp.gate|up|down`,
`final.norm`, `head`; linear weights are [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional

from ..errors import QsError, QStreamError
from .specs import (AttentionSpec, BlockSpec, DecayAttentionSpec, GatedMlpSpec, HeadSpec, LayerRun, ModelSpec,
                    PairEmbeddingSpec, PositionSpec, RmsNormSpec, WkvSpec)

MIXERS = ("attention", "lightning", "wkv")
DEFAULT_MAX_POSITIONS = 32768


def _bad(detail: str, code=QsError.INVALID_MODEL):
    return QStreamError(code, "config.json: " + detail)


def _get(d, key, what, kinds, optional=False, default=None):
    if not isinstance(d, dict):
        raise _bad(f"{what} must be an object")
    v = d.get(key)
    if v is None:
        if optional:
            return default
        raise _bad(f"{what} lacks '{key}'")
    if isinstance(v, bool) and bool not in (kinds if isinstance(kinds, tuple) else (kinds,)):
        raise _bad(f"{what}.{key} must be {kinds}, got {v!r}")
    if not isinstance(v, kinds):
        raise _bad(f"{what}.{key} has the wrong type: {v!r}")
    return v


def _positive_int(d, key, what, optional=False, default=None):
    v = _get(d, key, what, int, optional, default)
    if v is not None and v < 1:
        raise _bad(f"{what}.{key}={v} must be positive")
    return v


@dataclass(frozen=True)
class LutelornConfig:
    vocab: int
    width: int
    layers: tuple                       # the config's own layer objects (dicts), checked
    eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[dict]              # {"buckets", "mul_prev", "mul_cur"} or None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Lutelorn"
    model_type = "lutelorn"

    # ----------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict) -> "LutelornConfig":
        emb = _get(d, "embedding", "config", dict, optional=True, default={})
        bigram = emb.get("bigram")
        if bigram is not None:
            bigram = {k: _get(bigram, k, "embedding.bigram", int) for k in ("buckets", "mul_prev", "mul_cur")}
            if bigram["buckets"] < 1:
                raise _bad(f"embedding.bigram.buckets={bigram['buckets']} must be positive")
        layers = _get(d, "layers", "config", list)
        if not layers:
            raise _bad("'layers' is empty")
        cfg = cls(
            vocab=_positive_int(d, "vocab", "config"),
            width=_positive_int(d, "width", "config"),
            layers=tuple(copy.deepcopy(layer) for layer in layers),
            eps=float(_get(_get(d, "norm", "config", dict), "eps", "norm", (int, float))),
            residual_mult=float(_get(d, "residual_mult", "config", (int, float), optional=True, default=1.0)),
            embedding_scale=float(_get(emb, "scale", "embedding", (int, float), optional=True, default=1.0)),
            bigram=bigram,
            max_positions=_positive_int(d, "max_positions", "config", optional=True, default=DEFAULT_MAX_POSITIONS),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise _bad(f"norm.eps={self.eps} must be positive")
        mixed_values = None
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            kind = _get(layer, "type", what, str)
            if kind not in MIXERS:
                raise _bad(f"{what}.type '{kind}' is not one of {MIXERS}", QsError.UNSUPPORTED_ARCH)
            m = _get(layer, "mixer", what, dict)
            what += ".mixer"
            heads = _positive_int(m, "heads", what)
            dim = _positive_int(m, "dim", what)
            if kind == "attention":
                kv = _positive_int(m, "kv_heads", what, optional=True, default=heads)
                vdim = _positive_int(m, "vdim", what, optional=True, default=dim)
                if heads % kv:
                    raise _bad(f"{what}: {heads} heads are no multiple of {kv} kv_heads")
                rot = m.get("rot")
                if rot is not None:
                    dims = _get(rot, "dims", what + ".rot", int)
                    base = _get(rot, "base", what + ".rot", (int, float))
                    if dims < 0 or dims % 2 or dims > dim or not base > 0:
                        raise _bad(f"{what}.rot: dims={dims} must be even and within dim={dim}, base={base} positive")
                _get(m, "scale", what, (int, float))
                cap = _get(m, "softcap", what, (int, float), optional=True, default=0)
                if cap < 0:
                    raise _bad(f"{what}.softcap={cap} must not be negative")
                if m.get("v_mix"):
                    if mixed_values is not None and mixed_values != (kv, vdim):
                        raise _bad(f"{what}: layers that mix values must agree in kv_heads and vdim")
                    mixed_values = (kv, vdim)
            elif kind == "lightning":
                _positive_int(m, "vdim", what, optional=True, default=dim)
                decay = _get(m, "decay", what, list)
                if len(decay) != heads or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise _bad(f"{what}.decay must list one number per head ({heads})")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _get(mlp, "kind", f"layers[{i}].mlp", str) != "dense":
                    raise _bad(f"layers[{i}].mlp.kind '{mlp['kind']}' is not 'dense'", QsError.UNSUPPORTED_ARCH)
                _positive_int(mlp, "ff", f"layers[{i}].mlp")

    def to_dict(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(self.bigram)
        return {"architecture": self.architecture, "model_type": self.model_type, "vocab": self.vocab,
                "width": self.width, "layers": [copy.deepcopy(layer) for layer in self.layers],
                "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "embedding": emb,
                "max_positions": self.max_positions}

    # ----------------------------------------------------------------- the model
    def _mixer_spec(self, i: int, kind: str, m: dict, first_mixing_layer: Optional[int]):
        D, p = self.width, f"l{i}.mix."
        heads, dim = m["heads"], m["dim"]
        if kind == "attention":
            names = {"q": p + "q", "k": p + "k", "v": p + "v", "q_bias": p + "q.b", "k_bias": p + "k.b",
                     "v_bias": p + "v.b", "gate": p + "g", "out": p + "o"}
            value_mix = None
            if m.get("v_mix"):
                # every layer that mixes values holds the scalar, the first does not use it
                names["value_mix"] = p + "vmix"
                value_mix = "first" if first_mixing_layer == i else "blend"
            rot = m.get("rot")
            position = None
            if rot is not None and rot["dims"] > 0:
                position = PositionSpec(rotary_dim=rot["dims"], base=float(rot["base"]), max_positions=self.max_positions)
            return AttentionSpec(width=D, n_heads=heads, n_kv_heads=m.get("kv_heads", heads), head_dim=dim,
                                 v_head_dim=m.get("vdim", dim), position=position, qkv_bias=True, gate=True,
                                 score_scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                                 value_mix=value_mix, names=names)
        if kind == "lightning":
            return DecayAttentionSpec(width=D, n_heads=heads, key_dim=dim, value_dim=m.get("vdim", dim),
                                      decay=tuple(float(x) for x in m["decay"]), eps=self.eps,
                                      names={n: p + n for n in ("q", "k", "v", "g", "o", "norm")})
        names = {n: p + n for n in ("r", "k", "v", "g", "o", "w1", "w2", "w0", "u", "norm")}
        names.update({"mu_" + n: p + "mu." + n for n in ("r", "k", "v", "g", "w")})
        return WkvSpec(width=D, n_heads=heads, head_dim=dim, eps=self.eps, decay_rank=int(m.get("decay_rank", -1)),
                       names=names)

    def model_spec(self) -> ModelSpec:
        D = self.width
        first_mixing = next((i for i, layer in enumerate(self.layers)
                             if layer["type"] == "attention" and layer["mixer"].get("v_mix")), None)
        blocks = []
        for i, layer in enumerate(self.layers):
            norms = {"input": RmsNormSpec(D, self.eps, offset=1.0, names={"weight": f"l{i}.norm1"})}
            ffn = None
            if layer.get("mlp") is not None:
                norms["post_mixer"] = RmsNormSpec(D, self.eps, offset=1.0, names={"weight": f"l{i}.norm2"})
                ffn = GatedMlpSpec(width=D, inner=layer["mlp"]["ff"], activation="silu",
                                   names={n: f"l{i}.mlp.{n}" for n in ("gate", "up", "down")})
            blocks.append(BlockSpec(arrangement="scaled_residual", residual_scale=self.residual_mult, norms=norms,
                                    mixer=self._mixer_spec(i, layer["type"], layer["mixer"], first_mixing), ffn=ffn))
        b = self.bigram or {}
        emb_names = {"weight": "embed"}
        if self.bigram is not None:
            emb_names["pair"] = "bigram"
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, width=D, max_positions=self.max_positions,
            embedding=PairEmbeddingSpec(vocab_size=self.vocab, width=D, scale=self.embedding_scale,
                                        buckets=b.get("buckets", 0), mul_prev=b.get("mul_prev", 0),
                                        mul_cur=b.get("mul_cur", 0), stream_dtype="float32", names=emb_names),
            layers=tuple(blocks),
            schedule=tuple(LayerRun(layer=i, cache=i) for i in range(len(blocks))),
            final_norm=RmsNormSpec(D, self.eps, offset=1.0, names={"weight": "final.norm"}),
            head=HeadSpec(vocab_size=self.vocab, width=D, bias=False, tied=False, names={"weight": "head"}),
        )
