"""Fofinex's configuration: reading, validation, the model it describes; and the plain model's own pieces on inputs
whose results are known."""
import copy
import math

import numpy as np
import pytest

import qstream_b200 as qs
from qstream_b200.config.fofinex import FofinexConfig
from qstream_b200.engine.model import declared_tensors
from qstream_b200.errors import QStreamError
from qstream_b200.parts.rotary import scaled_frequencies

import plain_fofinex as P
from fofinex_util import CONFIGS, make_weights


@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_the_declared_tensors_are_the_checkpoint_s(which):
    cfg = qs.config_from_dict(CONFIGS[which])
    assert isinstance(cfg, FofinexConfig)
    decl = declared_tensors(cfg.model_spec())
    weights = make_weights(CONFIGS[which], 0)
    assert set(decl) == set(weights)
    for name, d in decl.items():
        assert tuple(d.shape) == weights[name].shape, name
    assert qs.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_the_schedule_points_a_sharing_layer_at_the_entry_it_reads():
    spec = qs.config_from_dict(CONFIGS["A"]).model_spec()
    assert [r.cache for r in spec.schedule] == [0, 1, 0, 3, 4]
    assert spec.layers[2].mixer.shares_cache and not spec.layers[0].mixer.shares_cache
    assert spec.layers[2].ffn is None and spec.head.tied


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=40), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "router"),
    (lambda c: c["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, needle):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises(QStreamError) as e:
        qs.config_from_dict(cfg)
    assert needle in str(e.value)


@pytest.mark.parametrize("dims,base,scaling", [(8, 1e4, None), (32, 5e5, dict(factor=8.0, original=128, fast=16.0, slow=1.0)),
                                               (6, 200.0, dict(factor=16.0, original=32, fast=4.0, slow=0.5))])
def test_the_library_s_frequencies_are_the_plain_ones(dims, base, scaling):
    f, mag = scaled_frequencies(dims, base, scaling)
    pf, pmag = P.yarn_frequencies(dims, base, scaling)
    np.testing.assert_allclose(f.numpy(), pf, rtol=1e-14)
    assert mag == pytest.approx(pmag, rel=1e-15)
    if scaling:
        assert mag == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)
        assert (pf <= np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)]) * (1 + 1e-12)).all()


def test_the_plain_router_on_a_hand_made_case():
    """Two groups of four, one kept, three chosen: the kept group's negative choice score beats every expert of the
    dropped group, and the weights are the scores without the correction."""
    z = np.array([[3.0, 2.0, -1.0, -2.0, 1.0, 1.0, 1.0, 1.0]])
    W = {"r.router": np.eye(8), "r.correction": np.array([0.0, 0.0, -0.9, -0.9, -0.2, -0.2, -0.2, -0.2])}
    mlp = {"router": {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 2, "keep": 1}}}
    idx, wts = P.route(z, mlp, W, "r.")
    assert idx.tolist() == [[0, 1, 2]]
    np.testing.assert_allclose(wts[0], 2.0 / (1.0 + np.exp(-z[0, :3])))


def test_the_plain_matrix_memory_forgets_and_normalises():
    """With a forget gate of one and equal input gates the memory is a sum: o is the q-weighted mean of the values."""
    T, dk, dv = 6, 4, 3
    rng = np.random.default_rng(0)
    h = np.eye(T, 8)
    W = {"m.q": np.zeros((dk, 8)), "m.k": np.zeros((dk, 8)), "m.v": rng.normal(size=(dv, 8)), "m.g": np.zeros((dv, 8)),
         "m.i": np.zeros((1, 8)), "m.f": np.zeros((1, 8)), "m.i.b": np.zeros(1), "m.f.b": np.array([1e4]),
         "m.norm": np.ones(dv), "m.o": np.eye(dv)}
    W["m.q"][0, :] = 2.0
    W["m.k"][0, :] = 2.0
    out = P.mlstm(h, {"heads": 1, "dim": dk, "vdim": dv, "gate_cap": 1e6}, W, "m.", 0.0)
    v = h @ W["m.v"].T
    for t in range(T):
        mean = v[:t + 1].mean(0)
        np.testing.assert_allclose(out[t], 0.5 * mean / np.sqrt((mean ** 2).mean()), rtol=1e-4)
