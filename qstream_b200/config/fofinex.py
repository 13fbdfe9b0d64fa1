"""Fofinex's configuration, read from its own config.json keys.

A Fofinex model lists its layers: `layers[i]` names the layer's mixer (`type`: "latent_attention" or "mlstm"), the
mixer's sizes and constants (`mixer`), and its feed-forward (`mlp`: {"kind": "dense", "ff": n}, {"kind": "moe",
"expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "shared": {"ff"} or absent}, or
null).  Around them: `vocab`, `width`, `norm.eps`.  Every size and constant comes from these keys.  The embedding is
followed by a norm, every sublayer has a norm before and after it, the residual stream is 32-bit, and the head is the
embedding table.  The model names no longest sequence; `max_positions` (the library's own key, default 32,768) bounds
the engine's context only: rotation angles are computed from the position, not looked up.

Tensor names: `embed`, `embed.norm`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.<name>`, `l<i>.mlp.<name>`,
`final.norm`; linear weights are [out, in].
"""
from __future__ import annotations

import copy
from dataclasses import dataclass

from ..errors import QsError, QStreamError
from .lutelorn import _bad, _get, _positive_int
from .specs import (BlockSpec, GatedMlpSpec, HeadSpec, LatentAttentionSpec, LayerRun, MlstmSpec, ModelSpec,
                    NormedEmbeddingSpec, RotaryHalfSpec, RoutedExpertsSpec, StreamNormSpec)

MIXERS = ("latent_attention", "mlstm")
DEFAULT_MAX_POSITIONS = 32768


def _number(d, key, what, optional=False, default=None):
    v = _get(d, key, what, (int, float), optional, default)
    return None if v is None else float(v)


@dataclass(frozen=True)
class FofinexConfig:
    vocab: int
    width: int
    layers: tuple                       # the config's own layer objects (dicts), checked
    eps: float
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Fofinex"
    model_type = "fofinex"

    # ----------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict) -> "FofinexConfig":
        layers = _get(d, "layers", "config", list)
        if not layers:
            raise _bad("'layers' is empty")
        cfg = cls(vocab=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
                  layers=tuple(copy.deepcopy(layer) for layer in layers),
                  eps=_number(_get(d, "norm", "config", dict), "eps", "norm"),
                  max_positions=_positive_int(d, "max_positions", "config", optional=True, default=DEFAULT_MAX_POSITIONS))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise _bad(f"norm.eps={self.eps} must be positive")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            kind = _get(layer, "type", what, str)
            if kind not in MIXERS:
                raise _bad(f"{what}.type '{kind}' is not one of {MIXERS}", QsError.UNSUPPORTED_ARCH)
            m = _get(layer, "mixer", what, dict)
            what += ".mixer"
            for key in ("heads", "dim", "vdim"):
                _positive_int(m, key, what)
            if kind == "mlstm":
                if _number(m, "gate_cap", what) <= 0:
                    raise _bad(f"{what}.gate_cap must be positive")
            else:
                for key in ("q_rank", "kv_rank", "rot_dim"):
                    _positive_int(m, key, what)
                _number(m, "scale", what)
                rot = _get(m, "rot", what, dict)
                dims = _get(rot, "dims", what + ".rot", int)
                if dims < 0 or dims % 2 or dims > m["rot_dim"] or not _number(rot, "base", what + ".rot") > 0:
                    raise _bad(f"{what}.rot: dims={dims} must be even and within rot_dim={m['rot_dim']}, base positive")
                sc = rot.get("scaling")
                if sc is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        if not _number(sc, key, what + ".rot.scaling") > 0:
                            raise _bad(f"{what}.rot.scaling.{key} must be positive")
                src = m.get("kv_from")
                if src is not None:
                    ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
                    other = self.layers[src] if ok else None
                    if not ok or other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise _bad(f"{what}.kv_from={src!r} must name an earlier latent-attention layer with a W_dkv of its own")
                    for key in ("kv_rank", "rot_dim", "rot"):
                        if other["mixer"].get(key) != m.get(key):
                            raise _bad(f"{what}.{key} differs from that of layer {src}, whose cache it reads")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            what = f"layers[{i}].mlp"
            mk = _get(mlp, "kind", what, str)
            if mk == "dense":
                _positive_int(mlp, "ff", what)
            elif mk == "moe":
                _positive_int(_get(mlp, "expert", what, dict), "ff", what + ".expert")
                r = _get(mlp, "router", what, dict)
                E, top = _positive_int(r, "experts", what + ".router"), _positive_int(r, "top", what + ".router")
                _number(r, "scale", what + ".router", optional=True, default=1.0)
                g = r.get("groups") or {"count": 1, "keep": 1}
                count, keep = _positive_int(g, "count", what + ".router.groups"), _positive_int(g, "keep", what + ".router.groups")
                if E % count or keep > count or keep * (E // count) < top or top > E:
                    raise _bad(f"{what}.router: {E} experts, {count} groups, {keep} kept, top {top} do not fit together")
                if mlp.get("shared") is not None:
                    _positive_int(mlp["shared"], "ff", what + ".shared")
            else:
                raise _bad(f"{what}.kind '{mk}' is not 'dense' or 'moe'", QsError.UNSUPPORTED_ARCH)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "model_type": self.model_type, "vocab": self.vocab,
                "width": self.width, "layers": [copy.deepcopy(layer) for layer in self.layers],
                "norm": {"eps": self.eps}, "max_positions": self.max_positions}

    # ----------------------------------------------------------------- the model
    def _norm(self, name: str) -> StreamNormSpec:
        return StreamNormSpec(self.width, self.eps, center=True, names={"weight": name})

    def _mixer_spec(self, i: int, kind: str, m: dict):
        D, p = self.width, f"l{i}.mix."
        if kind == "mlstm":
            names = {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "i", "f")}
            names.update({"i_bias": p + "i.b", "f_bias": p + "f.b"})
            return MlstmSpec(width=D, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                             gate_cap=float(m["gate_cap"]), eps=self.eps, names=names)
        shares = m.get("kv_from") is not None
        names = {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "uk": p + "uk", "uv": p + "uv", "o": p + "o"}
        if not shares:
            names.update({"dkv": p + "dkv", "dkv_norm": p + "dkv.norm"})
        rot = m["rot"]
        scaling = rot.get("scaling")
        position = RotaryHalfSpec(rotary_dim=rot["dims"], base=float(rot["base"]),
                                  scaling={k: float(v) for k, v in scaling.items()} if scaling else None)
        return LatentAttentionSpec(width=D, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                                   v_head_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"],
                                   score_scale=float(m["scale"]), eps=self.eps, position=position, shares_cache=shares,
                                   names=names)

    def _ffn_spec(self, i: int, mlp: dict):
        D, p = self.width, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            names = {n: p + n for n in ("gate", "up", "down")}
            names.update({n + "_bias": p + n + ".b" for n in ("gate", "up", "down")})
            return GatedMlpSpec(width=D, inner=mlp["ff"], activation="gelu_new", bias=True, names=names)
        r = mlp["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        names = {"router": p + "router", "correction": p + "correction"}
        for e in range(r["experts"]):
            names[f"up{e}"], names[f"down{e}"] = f"{p}e{e}.up", f"{p}e{e}.down"
        shared = mlp.get("shared")
        if shared is not None:
            names.update({"shared_up": p + "shared.up", "shared_down": p + "shared.down", "shared_gate": p + "shared.sg"})
        return RoutedExpertsSpec(width=D, n_experts=r["experts"], inner=mlp["expert"]["ff"], top=r["top"],
                                 groups=g["count"], keep=g["keep"], route_scale=float(r.get("scale", 1.0)),
                                 activation="relu2", shared_inner=shared["ff"] if shared is not None else 0, names=names)

    def model_spec(self) -> ModelSpec:
        D = self.width
        blocks, schedule = [], []
        for i, layer in enumerate(self.layers):
            norms = {"input": self._norm(f"l{i}.norm1"), "post_input": self._norm(f"l{i}.norm1b")}
            ffn = None
            if layer.get("mlp") is not None:
                norms["post_mixer"], norms["post_ffn"] = self._norm(f"l{i}.norm2"), self._norm(f"l{i}.norm2b")
                ffn = self._ffn_spec(i, layer["mlp"])
            blocks.append(BlockSpec(arrangement="sandwich", norms=norms, ffn=ffn,
                                    mixer=self._mixer_spec(i, layer["type"], layer["mixer"])))
            src = layer["mixer"].get("kv_from")
            schedule.append(LayerRun(layer=i, cache=i if src is None else src))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, width=D, max_positions=self.max_positions,
            embedding=NormedEmbeddingSpec(vocab_size=self.vocab, width=D, eps=self.eps, center=True, stream_dtype="float32",
                                          names={"weight": "embed", "norm": "embed.norm"}),
            layers=tuple(blocks), schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=HeadSpec(vocab_size=self.vocab, width=D, bias=False, tied=True, names={}),
        )
