"""Fofinex's mechanisms one at a time, each kernel (or the few kernels of one mechanism) against the plain model's
function for it: norms around a branch, the rotate-half rotation with scaled frequencies, the latent's preparation
and cache write, the matrix memory's gates, scan and output (in order and in chunks, state carried on), the
router's choice, and the experts both ways."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_fofinex as P
from qstream_b200.config.specs import RoutedExpertsSpec
from qstream_b200.csrc import ops
from qstream_b200.parts import Runtime, part_class
from qstream_b200.parts.rotary import scaled_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV)


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("center", [True, False])
@pytest.mark.parametrize("D", [50, 320, 4096])
def test_norms_around_a_branch(center, D):
    rng = np.random.default_rng(D)
    x, y = rng.normal(1.0, 2.0, (7, D)), rng.normal(-0.5, 3.0, (7, D))
    wy, w = 1 + rng.normal(0, 0.2, D), 1 + rng.normal(0, 0.2, D)
    norm = (lambda v, ww: P.layer_norm(v, ww, 1e-5)) if center else (lambda v, ww: P.rms_norm(v, ww, 1e-5))
    x32, y32 = x.astype(np.float32).astype(np.float64), y.astype(np.float32).astype(np.float64)
    want_x = x32 + norm(y32, wy.astype(np.float32).astype(np.float64))
    want_h = norm(want_x, w.astype(np.float32).astype(np.float64))
    xd = dev(x)
    h = ops.branch_norm(xd, dev(w), 1e-5, center, branch=dev(y), branch_weight=dev(wy))
    np.testing.assert_allclose(xd.cpu().numpy(), want_x, rtol=0, atol=2e-5)
    np.testing.assert_allclose(h.cpu().numpy(), want_h, rtol=0, atol=2e-5)
    # the pieces alone: a norm in place; a branch added without a norm to follow; a bfloat16 result
    xd = dev(x)
    ops.branch_norm(xd, dev(w), 1e-5, center, in_place=True)
    np.testing.assert_allclose(xd.cpu().numpy(), norm(x32, w.astype(np.float32).astype(np.float64)), rtol=0, atol=2e-5)
    xd = dev(x)
    assert ops.branch_norm(xd, None, 1e-5, center, branch=dev(y), branch_weight=dev(wy), want_norm=False) is None
    np.testing.assert_allclose(xd.cpu().numpy(), want_x, rtol=0, atol=2e-5)
    hb = ops.branch_norm(dev(x), dev(w, torch.bfloat16), 1e-5, center, out_dtype=torch.bfloat16)
    assert hb.dtype == torch.bfloat16
    np.testing.assert_allclose(hb.float().cpu().numpy(), norm(x32, dev(w, torch.bfloat16).double().cpu().numpy()), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("scaling", [None, dict(factor=8.0, original=128, fast=16.0, slow=1.0)])
@pytest.mark.parametrize("sizes", [(3, 16, 8, 24, 20, 8), (1, 10, 6, 14, 12, 4), (4, 32, 32, 64, 48, 32)])
def test_latent_preparation_and_rotation(scaling, sizes):
    """RMS norms of both latents, the shared key part rotated and written into pages with the latent (twice: keys
    and values), every head's rotated query part; positions up to a hundred thousand."""
    H, dn, dr, r, rq, dims = sizes
    rng = np.random.default_rng(r)
    pos = np.array([0, 1, 63, 64, 65, 1000, 99999, 130])
    T = len(pos)
    d = rng.normal(0, 2.0, (T, rq + r + dr)).astype(np.float32)
    q = rng.normal(0, 1.0, (T, H * (dn + dr))).astype(np.float32)
    wq, wkv = ((1 + rng.normal(0, 0.2, n)).astype(np.float32) for n in (rq, r))
    f, mag = scaled_frequencies(dims, 1e4, scaling)
    f = f.to(DEV)
    n_pages = 99999 // 64 + 1
    table = np.full((2, n_pages), -1, dtype=np.int32)
    used = sorted({int(p) // 64 for p in pos})
    table[1, used] = np.arange(len(used))[::-1]                 # pages in another order than positions
    kc = torch.zeros((len(used), 1, 64, r + dr), device=DEV)
    vc = torch.zeros((len(used), 1, 64, r), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    slot = i32(np.full(T, 1))
    dd = dev(d)
    cq = ops.latent_prepare(dd[:, :rq], dev(wq), rq, dd[:, rq:], dev(wkv), r, dr, dims, f, mag, 1e-5, slot, i32(pos),
                            i32(table), 64, kc, vc, status)
    d64 = d.astype(np.float64)
    np.testing.assert_allclose(cq.cpu().numpy(), P.rms_norm(d64[:, :rq], wq, 1e-5), atol=3e-6, rtol=1e-5)
    c = P.rms_norm(d64[:, rq:rq + r], wkv, 1e-5)
    kr = P.rotate_half(d64[:, rq + r:], pos, dims, 1e4, scaling)
    for t, p in enumerate(pos):
        page = table[1, p // 64]
        np.testing.assert_allclose(kc[page, 0, p % 64].cpu().numpy(), np.concatenate([c[t], kr[t]]), atol=5e-6, rtol=1e-5)
        np.testing.assert_allclose(vc[page, 0, p % 64].cpu().numpy(), c[t], atol=5e-6, rtol=1e-5)
    assert int(status.item()) == 0 and float(kc.abs().sum(-1).gt(0).sum()) == T        # nothing else was written
    q_abs = torch.zeros((T, H * (r + dr)), device=DEV)
    ops.latent_q_rotate(q_abs, dev(q), H, dn, dr, r, dims, f, mag, slot, i32(pos))
    want = P.rotate_half(q.astype(np.float64).reshape(T, H, dn + dr)[..., dn:], pos, dims, 1e4, scaling)
    got = q_abs.cpu().numpy().reshape(T, H, r + dr)
    np.testing.assert_allclose(got[..., r:], want, atol=5e-6, rtol=1e-5)
    assert not got[..., :r].any()


def plain_memory(q, k, v, raw_i, raw_f, cap, dk):
    """The matrix memory from given projections, through the plain model's function: identity matrices stand for
    the projections, the gate's weight and the output projection are neutral."""
    T, H = raw_i.shape
    dv = v.shape[1] // H
    cols = np.concatenate([q, k, v, raw_i, raw_f], axis=1)
    n = cols.shape[1]
    W, at = {}, 0
    for name, width in (("q", H * dk), ("k", H * dk), ("v", H * dv), ("i", H), ("f", H)):
        W["m." + name] = np.eye(n)[at:at + width]
        at += width
    W.update({"m.i.b": np.zeros(H), "m.f.b": np.zeros(H), "m.g": np.zeros((H * dv, n)), "m.norm": np.full(H * dv, 2.0), "m.o": np.eye(H * dv)})
    return P.mlstm(cols, {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}, W, "m.", 1e-6)


@pytest.mark.parametrize("H,dk,dv,cap", [(2, 16, 24, 10.0), (1, 12, 20, 50.0), (5, 4, 6, 0.7), (3, 48, 32, 15.0), (2, 256, 8, 8.0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_matrix_memory_in_order_in_chunks_and_carried_on(H, dk, dv, cap, dtype):
    rng = np.random.default_rng(H * dk)
    lens = [300, 1, 70]                                         # the first is long enough to be cut into chunks
    slots = [4, 0, 2]
    state = torch.zeros((6, H * (dv + 1) * dk + H), device=DEV)
    matrix, maximum = state[:, :H * (dv + 1) * dk].view(6, H, dv + 1, dk), state[:, H * (dv + 1) * dk:]
    data, refs = [], []
    for n in lens:
        q, k, v = (dev(rng.normal(0, 1.0, (n, H * w)), dtype).float().cpu().numpy().astype(np.float64) for w in (dk, dk, dv))
        raw = rng.normal(0, 3.0, (n, 2 * H))
        raw[:, H:] += 4.0
        raw = raw.astype(np.float32).astype(np.float64)
        data.append((q, k, v, raw))
        refs.append(plain_memory(q, k, v, raw[:, :H], raw[:, H:], cap, dk))

    def run(pieces, chunked):
        """pieces: per sequence (first, last) rows of its data in this step."""
        rows = [np.concatenate([d[j][a:b] for d, (a, b) in zip(data, pieces)]) for j in range(4)]
        starts = np.concatenate([[0], np.cumsum([b - a for a, b in pieces])])
        T = int(starts[-1])
        q, k, v = (dev(rows[j], dtype) for j in range(3))
        a, w, m = ops.mlstm_gates(dev(rows[3]), cap, maximum, i32(starts), i32(slots), len(slots), H)
        chunks = None
        if chunked:
            cs, owners = [0], [0]
            for (lo, hi), s0 in zip(pieces, starts):
                cs += [int(s0) + min(hi - lo, c + 64) for c in range(0, hi - lo, 64)]
                owners.append(len(cs) - 1)
            chunks = (i32(cs), i32(np.arange(len(cs) - 1)), i32(owners), len(cs) - 1)
        o = ops.state_scan("gated", q, k, v, matrix, i32(starts), i32(slots), len(slots), H, dk, dv + 1, token_decay=a,
                           token_weight=w, q_scale=dk ** -0.5, chunks=chunks)
        gate = torch.zeros((T, H * dv), device=DEV, dtype=dtype)
        y = ops.mlstm_output(o, m, torch.full((H * dv,), 2.0, device=DEV), gate, H, dv, 1e-6, torch.float32)
        return [y[starts[i]:starts[i + 1]].cpu().numpy() for i in range(len(pieces))]

    tol = dict(atol=2e-4, rtol=2e-4)
    for chunked in (False, True):
        state.zero_()
        got = run([(0, n) for n in lens], chunked)
        for g, r in zip(got, refs):
            np.testing.assert_allclose(g, r, **tol)              # both sides: weight 2, gate sigmoid(0)
    # carried on: a first step of (200, 0, 69) tokens, then the rest, the long one in chunks
    state.zero_()
    first = run([(0, 200), (0, 0), (0, 69)], True)
    state_before = state.clone()
    second = run([(200, 300), (0, 1), (69, 70)], False)
    for g1, g2, r in zip(first, second, refs):
        np.testing.assert_allclose(np.concatenate([g1, g2]), r, **tol)
    assert not torch.equal(state_before[4], state[4]) and torch.equal(state_before[1], state[1])     # only the step's slots change


@pytest.mark.parametrize("E,top,groups,keep", [(8, 2, 4, 2), (6, 3, 1, 1), (5, 1, 5, 3), (16, 3, 8, 5), (8, 3, 2, 1), (64, 6, 8, 4)])
def test_router_choice(E, top, groups, keep):
    rng = np.random.default_rng(E + top)
    T = 257
    z = rng.normal(0, 2.0, (T, E + 1)).astype(np.float32)
    corr = rng.normal(0, 1.0, E).astype(np.float32)
    idx, wts, gate = ops.moe_route(dev(z), dev(corr), E, top, groups, keep, 1.7, gate_col=E)
    mlp = {"router": {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}}
    W = {"r.router": np.eye(E), "r.correction": corr.astype(np.float64)}
    pidx, pwts = P.route(z[:, :E].astype(np.float64), mlp, W, "r.")
    assert (idx.cpu().numpy() == pidx).all()
    np.testing.assert_allclose(wts.cpu().numpy(), pwts, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(gate.cpu().numpy(), P.sigmoid(z[:, E].astype(np.float64)), rtol=1e-5, atol=1e-6)


def test_router_prefers_a_negative_score_of_a_kept_group():
    """The case that tells minus infinity from zero: the kept group's third expert has a negative choice score while
    every expert of the dropped group has a positive one; and the weights leave the correction out."""
    z = np.random.default_rng(0).normal(0, 1.0, (64, 8)).astype(np.float32)
    corr = np.array([1.0, 1.0, -2.0, -2.5, 0.0, 0.0, 0.0, 0.0], dtype=np.float32)
    idx, wts, _ = ops.moe_route(dev(z), dev(corr), 8, 3, 2, 1, 2.0)
    idx, wts = idx.cpu().numpy(), wts.cpu().numpy()
    assert (idx[:, :2].min(1) == 0).all() and (idx[:, :2].max(1) == 1).all()
    third = np.where(z[:, 2] + 0.0 > z[:, 3] - 0.0, 2, 3)          # sigmoid is monotone; the corrections differ by 0.5
    s = P.sigmoid(z.astype(np.float64))
    want_third = np.where(s[:, 2] - 2.0 >= s[:, 3] - 2.5, 2, 3)
    assert (idx[:, 2] == want_third).all() and third.shape == want_third.shape
    np.testing.assert_allclose(wts, 2.0 * np.take_along_axis(s, idx.astype(np.int64), 1), rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 9, 200])
def test_experts_both_ways(dtype, T):
    """Few tokens: every pair finds its expert's matrices on the device.  Many: pairs ordered by expert, a product per
    expert (some experts get no token at all).  With and without the shared expert."""
    D, F, E, top = 48, 24, 12, 3
    rng = np.random.default_rng(T)
    for shared in (40, 0):
        spec = RoutedExpertsSpec(width=D, n_experts=E, inner=F, top=top, groups=4, keep=2, route_scale=1.5, shared_inner=shared)
        names = {"router": (E, D, 3.0), "correction": (E,), **{f"up{e}": (F, D, 1.5) for e in range(E)}, **{f"down{e}": (D, F, 1.5) for e in range(E)}}
        if shared:
            names.update({"shared_up": (shared, D, 1.5), "shared_down": (D, shared, 1.5), "shared_gate": (1, D, 2.0)})
        tensors = {}
        for name, shape in names.items():
            a = rng.normal(0, 0.5, shape) if len(shape) == 1 else rng.normal(0, shape[2] / np.sqrt(shape[1]), shape[:2])
            tensors[name] = dev(a, dtype)
        part = part_class("feed_forward", "routed_experts")(spec, tensors, Runtime(dtype=dtype, device=torch.device(DEV)))
        h = dev(rng.normal(0, 1.0, (T, D)), dtype)
        step = SimpleNamespace(batch=SimpleNamespace(tok_slot=i32(np.zeros(T)), decode=False))
        got = part.forward(h, step).cpu().numpy()
        W = {"x." + ("router" if n == "router" else "correction" if n == "correction" else
                     n.replace("shared_gate", "shared.sg").replace("shared_", "shared.") if n.startswith("shared") else
                     f"e{n[2:]}.up" if n.startswith("up") else f"e{n[4:]}.down"): t.double().cpu().numpy() for n, t in tensors.items()}
        mlp = {"router": {"experts": E, "top": top, "scale": 1.5, "groups": {"count": 4, "keep": 2}}, "shared": {"ff": shared} if shared else None}
        want = P.moe_ff(h.double().cpu().numpy(), mlp, W, "x.")
        if dtype == torch.float32:
            np.testing.assert_allclose(got, want, atol=2e-4, rtol=2e-4)
        else:       # hidden activations are rounded to bfloat16 between the two products
            assert np.abs(got - want).max() <= 0.03 * np.abs(want).max()


@pytest.mark.parametrize("H,cap", [(1, 50.0), (5, 0.7), (16, 12.0)])
def test_gates_as_a_scan_equal_the_walk_in_order(H, cap):
    """A long sequence takes its chain of maxima as a scan over runs of tokens; pieces of a hundred tokens walk it in
    order, carrying the maximum in the slot.  Both against the recurrence written out."""
    rng = np.random.default_rng(H)
    n = 1000
    raw = rng.normal(0, 4.0, (n, 2 * H)).astype(np.float32)
    raw[:, H:] += 3.0
    state = torch.zeros((3, H), device=DEV)
    whole = ops.mlstm_gates(dev(raw), cap, state, i32([0, n]), i32([1]), 1, H)
    state2 = torch.zeros((3, H), device=DEV)
    pieces = [ops.mlstm_gates(dev(raw[a:a + 100]), cap, state2, i32([0, 100]), i32([2]), 1, H) for a in range(0, n, 100)]
    i = cap * np.tanh(raw[:, :H].astype(np.float64) / cap)
    f = P.log_sigmoid(cap * np.tanh(raw[:, H:].astype(np.float64) / cap))
    m, want = np.zeros(H), []
    for t in range(n):
        m_new = np.maximum(f[t] + m, i[t])
        want.append((np.exp(f[t] + m - m_new), np.exp(i[t] - m_new), m_new))
        m = m_new
    for j in range(3):
        ref = np.stack([w[j] for w in want])
        np.testing.assert_allclose(whole[j].cpu().numpy(), ref, rtol=2e-5, atol=1e-6)
        np.testing.assert_allclose(torch.cat([p[j] for p in pieces]).cpu().numpy(), ref, rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(state[1].cpu().numpy(), m, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(state2[2].cpu().numpy(), m, rtol=1e-6, atol=1e-6)
    assert not state[0].any() and not state[2].any()
