"""Lutelorn's configuration and what it declares, without a GPU."""
import copy

import numpy as np
import pytest
import torch

import qstream_b200 as qs
from qstream_b200.cache import SequenceCache, StateNeed, StateStore
from qstream_b200.config import LutelornConfig, config_from_dict
from qstream_b200.engine.model import declared_tensors
from lutelorn_util import CONFIGS, make_folder


def test_the_architecture_is_found_by_its_name_and_round_trips():
    cfg = config_from_dict(CONFIGS["A"])
    assert isinstance(cfg, LutelornConfig)
    again = config_from_dict(cfg.to_dict())
    assert again == cfg
    assert config_from_dict({**CONFIGS["B"], "architecture": None, "model_type": "lutelorn"}).vocab == 131


def test_every_size_comes_from_the_configuration():
    spec = config_from_dict(CONFIGS["A"]).model_spec()
    d = declared_tensors(spec)
    assert d["embed"].shape == (97, 64) and d["bigram"].shape == (54, 64) and d["head"].shape == (97, 64)
    assert d["l0.mix.q"].shape == (64, 64) and d["l0.mix.k"].shape == (32, 64) and d["l0.mix.v"].shape == (16, 64)
    assert d["l0.mix.g"].shape == (32, 64) and d["l0.mix.o"].shape == (64, 32) and d["l0.mix.vmix"].shape == ()
    assert d["l4.mix.q"].shape == (48, 64) and d["l4.mix.v"].shape == (80, 64) and d["l4.mix.norm"].shape == (80,)
    assert d["l2.mix.w1"].shape == (-1, 64) and d["l2.mix.w2"].shape == (64, -1) and d["l2.mix.u"].shape == (2, 32)
    assert "l1.norm2" not in d and d["l2.mlp.gate"].shape == (80, 64)
    mixes = [b.mixer.value_mix for b in spec.layers if b.mixer.kind == "attention"]
    assert mixes == ["first", "blend", "blend"]
    c = config_from_dict(CONFIGS["C"]).model_spec()         # a layer that does not ask for it blends nothing
    assert [b.mixer.value_mix for b in c.layers if b.mixer.kind == "attention"] == ["first", "blend", None]
    assert spec.layers[5].mixer.position is None and spec.layers[5].mixer.scale == 0.3 and spec.layers[5].mixer.softcap == 0.0
    assert [b.residual_scale for b in spec.layers] == [0.6] * 7
    b = config_from_dict(CONFIGS["B"]).model_spec()
    assert "bigram" not in declared_tensors(b) and b.embedding.buckets == 0
    assert all(layer.mixer.value_mix is None for layer in b.layers if layer.mixer.kind == "attention")


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "not one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "no multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not 'dense'"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=16), "agree"),
    (lambda c: c.pop("width"), "lacks 'width'"),
    (lambda c: c["norm"].update(eps=0), "positive"),
    (lambda c: c.update(vocab=True), "vocab"),
])
def test_a_bad_configuration_is_refused_with_a_reason(change, word):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises(qs.QStreamError, match=word):
        config_from_dict(cfg)


def test_the_checkpoint_gives_the_size_the_configuration_does_not(tmp_path):
    folder, _ = make_folder(tmp_path, "A", "float32")
    model = qs.load_model(folder, dtype="float32", device="cpu", allow_mmap=False)   # a host model must own its bytes
    assert model.blocks[2].mixer.w["w1"].shape == (5, 64)
    needs = model.state_needs()
    assert set(needs) == {1, 2, 4, 6, "embedding"} and set(needs[2]) == {"matrix", "last_input"}
    assert needs[4].shape == (2, 40, 24) and needs["embedding"].dtype == torch.int32
    kv = model.kv_needs()
    assert kv[0].head_dim == 16 and kv[0].value_dim == 8 and kv[5].head_dim == 32
    with pytest.raises(qs.QStreamError, match="only a checkpoint gives"):
        qs.write_model_folder(tmp_path / "x", config_from_dict(CONFIGS["A"]), 0)


def test_state_store_keeps_several_tensors_per_part_and_clears_a_slot():
    store = StateStore({3: StateNeed((2, 4)), "e": StateNeed((1,), torch.int32),
                        5: {"m": StateNeed((3,)), "h": StateNeed((2,), torch.bfloat16)}}, 4, "cpu")
    assert store.get(3).shape == (4, 2, 4) and store.get(5, "m").shape == (4, 3) and store.get("e").dtype == torch.int32
    store.get(3)[:] = 1.0
    store.get(5, "m")[:] = 2.0
    store.get(5, "h")[:] = 3.0
    store.get("e")[:] = 4
    store.reset(2)
    for t in (store.get(3), store.get(5, "m"), store.get(5, "h"), store.get("e")):
        assert float(t[2].abs().sum()) == 0.0 and float(t[1].abs().sum()) > 0.0
    assert store.get(9) is None


def test_cache_pages_take_the_values_head_size():
    from qstream_b200.cache import KvNeed
    cache = SequenceCache({0: KvNeed(2, 16, 0, 8), 1: KvNeed(2, 16)}, {}, 128, 2, 128, torch.float32, "cpu")
    assert cache.view(0).k.shape[-1] == 16 and cache.view(0).v.shape[-1] == 8 and cache.view(1).v.shape[-1] == 16
    assert len(cache.groups) == 2
