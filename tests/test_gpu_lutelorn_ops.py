"""Each mechanism of the Lutelorn parts alone: the library's kernel against the plain function of
`plain_lutelorn`, on inputs made so that a fault shows (a far key that must win, a state that must
survive steps, windows of values just inside and outside what a step brings)."""
import numpy as np
import pytest
import torch

import plain_lutelorn as P
from qstream_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def close(got, ref, tol, what=""):
    got = got.float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    scale = np.abs(ref).max() + 1e-30
    assert np.abs(got - ref).max() <= tol * scale, f"{what}: {np.abs(got - ref).max() / scale:.3e} of the largest value"


# --------------------------------------------------------------------------- norms and small kernels

@pytest.mark.parametrize("D", [48, 192, 1000])
@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_rms_norm_and_update(D, offset):
    rng = np.random.default_rng(D)
    x, y, w = rng.normal(0, 3, (7, D)), rng.normal(0, 1, (7, D)), rng.normal(0, 0.3, D)
    h = ops.rmsnorm(dev(x), dev(w), 1e-5, offset)
    close(h, P.rms_norm(x, w, 1e-5, offset), 2e-6, "norm")
    xd = dev(x)
    h = ops.rmsnorm(xd, dev(w), 1e-5, offset, out_dtype=torch.bfloat16, update=dev(y), mult=0.6)
    close(xd, x + 0.6 * y, 1e-6, "update in place")
    close(h, P.rms_norm(x + 0.6 * y, w, 1e-5, offset), 6e-3, "norm after the update, bfloat16")
    xd = dev(x)
    assert ops.rmsnorm(xd, None, 0.0, update=dev(y, torch.bfloat16), mult=-2.0, want_norm=False) is None
    close(xd, x - 2.0 * dev(y, torch.bfloat16).float().cpu().numpy(), 1e-6, "update alone, bfloat16 branch")


@pytest.mark.parametrize("n,group", [(96, 96), (96, 24), (60, 12), (128, 0), (2048, 2048), (4096, 128)])
def test_gated_group_norm(n, group):
    rng = np.random.default_rng(n + group)
    o, w, g = rng.normal(0, 2, (5, n)), rng.normal(1, 0.2, n), rng.normal(0, 2, (5, n))
    ref = o.copy()
    if group:
        ref = P.unit_rms(o.reshape(5, n // group, group), 1e-5).reshape(5, n)
    for act, f in (("sigmoid", P.sigmoid), ("silu", P.silu)):
        got = ops.gated_group_norm(dev(o), group, dev(w), dev(g), act, 1e-5, torch.float32)
        close(got, ref * w * f(g), 3e-6, f"group {group} {act}")
    got = ops.gated_group_norm(dev(o), group, None, None, None, 1e-5, torch.float32)
    close(got, ref, 3e-6, "no weight, no gate")


@pytest.mark.parametrize("F", [50, 64, 2056])
def test_gated_activation(F):
    rng = np.random.default_rng(F)
    ab = rng.normal(0, 2, (9, 2 * F))
    close(ops.gated_act(dev(ab), "silu"), P.silu(ab[:, :F]) * ab[:, F:], 2e-6)
    abb = dev(ab, torch.bfloat16)
    ref = abb.float().cpu().numpy().astype(np.float64)
    close(ops.gated_act(abb, "silu"), P.silu(ref[:, :F]) * ref[:, F:], 5e-3, "bfloat16")


def test_pair_embedding_across_steps():
    """Two sequences in one packed batch, then one more token each: the pair row of a step's first token comes
    from the token that the step before ended with; a sequence's first token takes the table's last row."""
    rng = np.random.default_rng(1)
    V, D, B = 40, 24, 11
    table, pair = rng.normal(0, 1, (V, D)), rng.normal(0, 1, (B + 1, D))
    cfg = {"embedding": {"scale": 0.3, "bigram": {"buckets": B, "mul_prev": 13, "mul_cur": 5}}}
    w = {"embed": table, "bigram": pair}
    a, b = [3, 39, 7, 7, 20], [11, 0, 38]
    last = torch.full((4, 1), -7, dtype=torch.int32, device=DEV)           # slots 2 and 0; stale values must not be read
    toks = i32(a[:4] + b[:2])
    x = ops.embedding_hashed(dev(table), dev(pair), 0.3, B, 13, 5, toks, i32([2] * 4 + [0] * 2), i32([0, 1, 2, 3, 0, 1]),
                             last, torch.float32)
    ops.keep_last_rows(last, toks.view(-1, 1), i32([0, 4, 6]), i32([2, 0]), 2)
    close(x[:4], P.embed(cfg, w, a)[:4], 1e-6, "first step, sequence a")
    close(x[4:], P.embed(cfg, w, b)[:2], 1e-6, "first step, sequence b")
    assert last.view(-1).tolist() == [0, -7, 7, -7]
    x = ops.embedding_hashed(dev(table), dev(pair), 0.3, B, 13, 5, i32([b[2], a[4], 0]), i32([0, 2, -1]), i32([2, 4, 0]),
                             last, torch.float32)
    close(x[0], P.embed(cfg, w, b)[2], 1e-6, "second step, sequence b")
    close(x[1], P.embed(cfg, w, a)[4], 1e-6, "second step, sequence a")
    assert float(x[2].abs().max()) == 0.0


def test_token_shift_across_steps():
    rng = np.random.default_rng(2)
    D = 40
    h = rng.normal(0, 1, (9, D))
    mu = rng.uniform(0, 1, (5, D))
    before = np.vstack([np.zeros((1, D)), h[:-1]])
    ref = np.stack([h + (before - h) * m for m in mu])
    last = torch.full((3, D), 9.0, device=DEV)
    got = []
    for a, b in ((0, 4), (4, 5), (5, 9)):                                  # 4 tokens, 1 token, 4 tokens, all in slot 1
        n = b - a
        hd = dev(h[a:b])
        got.append(ops.token_shift(hd, dev(mu), last, i32([1] * n), i32(range(a, b))).cpu().numpy())
        ops.keep_last_rows(last, hd, i32([0, n]), i32([1]), 1)
    close(np.concatenate(got, axis=1), ref, 1e-6)
    assert float(last[0].min()) == 9.0 and float(last[2].min()) == 9.0


# --------------------------------------------------------------------------- matrix states

def scan_in_steps(mode, q, k, v, cuts, H, dk, dv, dtype=torch.float32, **kw):
    """One sequence in slot 1 of three, cut into steps at `cuts`; slots 0 and 2 must stay untouched."""
    state = torch.zeros((3, H, dv, dk), device=DEV)
    state[0] = 5.0
    state[2] = -3.0
    out = []
    for a, b in zip([0] + cuts, cuts + [q.shape[0]]):
        extra = {key: (val[a:b].contiguous() if key == "decay_logits" else val) for key, val in kw.items()}
        o = ops.state_scan(mode, dev(q[a:b], dtype), dev(k[a:b], dtype), dev(v[a:b], dtype), state, i32([0, b - a]), i32([1]), 1,
                           H, dk, dv, **extra)
        out.append(o.cpu().numpy())
    assert float(state[0].min()) == 5.0 and float(state[2].max()) == -3.0
    return np.concatenate(out)


@pytest.mark.parametrize("H,dk,dv", [(4, 32, 16), (3, 24, 40), (2, 64, 16), (1, 96, 128), (2, 128, 128), (1, 200, 8)])
def test_decay_attention_state(H, dk, dv):
    rng = np.random.default_rng(dk + dv)
    T = 150
    q, k, v = (rng.normal(0, 1, (T, H * d)) for d in (dk, dk, dv))
    decay = np.array([0.5, 0.9, 0.999, 1.0][:H])
    # the first token is loud: with a decay near one it must still be heard at the end, through every cut
    k[0] *= 20.0
    ref = P.decayed_linear_attention(P.silu(q).reshape(T, H, dk), P.silu(k).reshape(T, H, dk), P.silu(v).reshape(T, H, dv), decay)
    ref = ref.reshape(T, H * dv)
    hd = dev(decay)
    for cuts in ([], [1, 2, 3], [8, 9, 17, 64, 65], list(range(1, T))):
        got = scan_in_steps("decay", q, k, v, cuts, H, dk, dv, head_decay=hd, in_activation="silu")
        close(got, ref, 2e-5, f"cuts {cuts[:4]}")


@pytest.mark.parametrize("H,d", [(5, 64), (1, 24), (3, 16), (2, 128), (1, 256)])
def test_wkv_state(H, d):
    rng = np.random.default_rng(d)
    T = 100
    r, k, v = (rng.normal(0, 1, (T, H * d)) for _ in range(3))
    dlog = rng.normal(-1.5, 1.5, (T, H * d))
    u = rng.normal(0, 0.5, (H, d))
    ref = P.wkv_recurrence(r.reshape(T, H, d), k.reshape(T, H, d), v.reshape(T, H, d), np.exp(-np.exp(dlog)).reshape(T, H, d), u)
    ref = ref.reshape(T, H * d)
    for cuts in ([], [1, 2], [7, 8, 9, 50], list(range(1, T))):
        got = scan_in_steps("wkv", r, k, v, cuts, H, d, d, decay_logits=dev(dlog), bonus=dev(u))
        close(got, ref, 2e-5, f"cuts {cuts[:4]}")


@pytest.mark.parametrize("mode,H,dk,dv", [("decay", 3, 32, 48), ("decay", 2, 128, 64), ("wkv", 4, 64, 64), ("wkv", 1, 24, 24)])
def test_chunks_side_by_side_equal_the_walk_in_order(mode, H, dk, dv):
    """Three sequences of 300, 1 and 131 tokens cut into chunks of 64 (the last ones ragged), from states that
    earlier steps left: outputs and final states equal those of the plain recurrence."""
    rng = np.random.default_rng(dk)
    lens = [300, 1, 131]
    slots = [2, 0, 3]
    T = sum(lens)
    q, k, v = (rng.normal(0, 1, (T, H * d)) for d in (dk, dk, dv))
    dlog, u, decay = rng.normal(-2.5, 1.0, (T, H * dk)), rng.normal(0, 0.5, (H, dk)), np.array([0.999, 0.9, 0.97, 0.5][:H])
    kw = dict(head_decay=dev(decay)) if mode == "decay" else dict(decay_logits=dev(dlog), bonus=dev(u))
    # a first step of 5 tokens per sequence leaves a state; the plain model sees both steps as one sequence
    pre = [rng.normal(0, 1, (5, 3, H * max(dk, dv))) for _ in lens]
    state = torch.zeros((4, H, dv, dk), device=DEV)
    starts, chunk_starts, owners, row = [0], [0], [0], 0
    for n in lens:
        chunk_starts += [row + min(n, a + 64) for a in range(0, n, 64)]
        row += n
        starts.append(row)
        owners.append(len(chunk_starts) - 1)
    n_chunks = len(chunk_starts) - 1
    for j, p in enumerate(pre):
        kw0 = dict(kw)
        if mode == "wkv":
            kw0["decay_logits"] = dev(np.full((5, H * dk), -2.0))
        ops.state_scan(mode, dev(p[:, 0, :H * dk]), dev(p[:, 1, :H * dk]), dev(p[:, 2, :H * dv]), state, i32([0, 5]), i32([slots[j]]), 1,
                       H, dk, dv, **kw0)
    got = ops.state_scan(mode, dev(q), dev(k), dev(v), state, i32(starts), i32(slots), 3, H, dk, dv,
                         chunks=(i32(chunk_starts), i32(range(n_chunks)), i32(owners), n_chunks), **kw).cpu().numpy()
    for j, (a, b) in enumerate(zip(starts, starts[1:])):
        p = pre[j]
        qq = np.concatenate([p[:, 0, :H * dk], q[a:b]]).reshape(-1, H, dk)
        kk = np.concatenate([p[:, 1, :H * dk], k[a:b]]).reshape(-1, H, dk)
        vv = np.concatenate([p[:, 2, :H * dv], v[a:b]]).reshape(-1, H, dv)
        if mode == "decay":
            ref = P.decayed_linear_attention(qq, kk, vv, decay)
        else:
            w = np.exp(-np.exp(np.concatenate([np.full((5, H * dk), -2.0), dlog[a:b]]))).reshape(-1, H, dk)
            ref = P.wkv_recurrence(qq, kk, vv, w, u)
        close(got[a:b], ref[5:].reshape(b - a, -1), 3e-5, f"sequence {j}")
    # the states left behind: one more token per sequence must continue them
    one = ops.state_scan(mode, dev(q[:3]), dev(k[:3]), dev(v[:3]), state, i32([0, 1, 2, 3]), i32(slots), 3, H, dk, dv,
                         **(dict(kw, decay_logits=dev(dlog[:3])) if mode == "wkv" else kw)).cpu().numpy()
    for j, (a, b) in enumerate(zip(starts, starts[1:])):
        p = pre[j]
        qq = np.concatenate([p[:, 0, :H * dk], q[a:b], q[j:j + 1]]).reshape(-1, H, dk)
        kk = np.concatenate([p[:, 1, :H * dk], k[a:b], k[j:j + 1]]).reshape(-1, H, dk)
        vv = np.concatenate([p[:, 2, :H * dv], v[a:b], v[j:j + 1]]).reshape(-1, H, dv)
        if mode == "decay":
            ref = P.decayed_linear_attention(qq, kk, vv, decay)
        else:
            w = np.exp(-np.exp(np.concatenate([np.full((5, H * dk), -2.0), dlog[a:b], dlog[j:j + 1]]))).reshape(-1, H, dk)
            ref = P.wkv_recurrence(qq, kk, vv, w, u)
        close(one[j], ref[-1].reshape(-1), 3e-5, f"the token after sequence {j}")


def test_states_of_a_batch_with_idle_and_padding_sequences():
    """Three sequences of unequal lengths in one step, a sequence entry without a slot between them and rows that
    belong to nobody at the end: each sequence equals itself alone, the rest is zero."""
    rng = np.random.default_rng(3)
    H, dk, dv = 2, 32, 24
    lens = [5, 1, 17]
    T = sum(lens) + 4 + 3
    q, k, v = (rng.normal(0, 1, (T, H * d)) for d in (dk, dk, dv))
    state = torch.zeros((5, H, dv, dk), device=DEV)
    starts = [0, 5, 9, 10, 27]                                             # the second entry (4 rows) has no slot
    o = ops.state_scan("decay", dev(q), dev(k), dev(v), state, i32(starts), i32([4, -1, 0, 2]), 4, H, dk, dv,
                       head_decay=dev(np.array([0.9, 0.7]))).cpu().numpy()
    for a, b in ((0, 5), (9, 10), (10, 27)):
        ref = P.decayed_linear_attention(q[a:b].reshape(-1, H, dk), k[a:b].reshape(-1, H, dk), v[a:b].reshape(-1, H, dv), [0.9, 0.7])
        close(o[a:b], ref.reshape(b - a, -1), 2e-5)
    assert np.abs(o[5:9]).max() == 0.0 and np.abs(o[27:]).max() == 0.0
    assert float(state[1].abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0


# --------------------------------------------------------------------------- attention

def paged_attention(q, k, v, H, G, dk, dv, scale, softcap, dtype, page_order, rot=None, blend=None, fast=False, gate=None):
    """One sequence through rope_store and the attention kernel, its pages in `page_order`."""
    T = q.shape[0]
    n_pages = len(page_order)
    kc = torch.zeros((n_pages + 1, G, 64, dk), dtype=dtype, device=DEV)
    vc = torch.full((n_pages + 1, G, 64, dv), 7.0, dtype=dtype, device=DEV)   # stale values in every page
    table = torch.full((2, n_pages), -1, dtype=torch.int32, device=DEV)
    table[1, :n_pages] = i32(page_order)
    slot, pos = i32([1] * T), i32(range(T))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    qd, kd, vd = dev(q, dtype), dev(k, dtype), dev(v, dtype)
    cs, R = None, 0
    if rot:
        R, base = rot
        ang = np.arange(T)[:, None] * base ** (-np.arange(0, R, 2) / R)
        cs = dev(np.stack([np.cos(ang), np.sin(ang)], -1))
    ops.rope_store(qd, kd, vd, H, G, dk, R, cs, slot, pos, table, 64, kc, vc, status, v_head_dim=dv,
                   v_first=dev(blend[0], dtype) if blend else None, v_mix=blend[1] if blend else 0.0)
    out = ops.attention(qd, H, G, dk, scale, 0, slot, pos, table, 64, kc, vc, status, v_head_dim=dv, softcap=softcap)
    assert int(status.item()) == 0
    if fast:
        # the bfloat16 kernels of prompts (tensor cores, pieces of 128 and fewer rows) and of single tokens (keys
        # split over CTAs), with a gate on the way out; they must agree with the generic kernel and the gate
        from qstream_b200.csrc import attention_bf16
        g = dev(gate, dtype)
        pieces = [(a, min(128, T - a), a, 1) for a in range(0, T, 128)][::-1]
        tiles = torch.tensor(pieces, dtype=torch.int32, device=DEV)
        pre = attention_bf16.prefill(qd, H, G, dk, scale, 0, tiles, table, 64, kc, vc, status, v_head_dim=dv,
                                     softcap=softcap, gate=g)
        rows = [T - 1, 3, 64, 200]
        dec = attention_bf16.decode(qd[rows].contiguous(), H, G, dk, scale, 0, i32([1] * 4), i32(rows), table, 64, kc, vc,
                                    512, status, v_head_dim=dv, softcap=softcap, gate=g[rows].contiguous())
        assert int(status.item()) == 0
        return out, pre, dec, rows
    return out


@pytest.mark.parametrize("H,G,dk,dv,softcap,rot", [(4, 2, 80, 48, 25.0, (40, 3e5)), (3, 3, 12, 12, 0.0, (12, 500.0)),
                                                     (6, 1, 10, 14, 4.0, None), (2, 2, 64, 64, 0.0, (16, 1e4)),
                                                     (8, 4, 32, 128, 8.0, (32, 1e4))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_a_far_key_that_wins(H, G, dk, dv, softcap, rot, dtype):
    """Key 3 of 330 is made to win at every late query (q and that key scaled up): the output there must be that
    key's value, through pages out of order; queries before it must not see it."""
    rng = np.random.default_rng(dk * dv)
    T = 330
    q, k, v = (rng.normal(0, 1, (T, n)) for n in (H * dk, G * dk, G * dv))
    if not rot:                     # without a rotation the far key can be aligned with every query
        k[3] = np.tile(q[200:, :dk].mean(0), G) * 3.0
    lam = 0.35
    v_first = rng.normal(0, 1, (T, G * dv))
    if dtype == torch.bfloat16:
        q, k, v, v_first = (dev(a, dtype).float().cpu().numpy().astype(np.float64) for a in (q, k, v, v_first))
    scale = 0.11
    qr, kr = q.reshape(T, H, dk), k.reshape(T, G, dk)
    if rot:
        qr, kr = P.rotate_pairs(qr, np.arange(T), *rot), P.rotate_pairs(kr, np.arange(T), *rot)
    vv = (1 - lam) * v + lam * v_first
    ref = P.capped_attention(qr, kr, vv.reshape(T, G, dv), scale, softcap).reshape(T, H * dv)
    got = paged_attention(q, k, v, H, G, dk, dv, scale, softcap, dtype, [4, 0, 5, 2, 1, 3], rot, (v_first, lam))
    close(got, ref, 2e-5 if dtype == torch.float32 else 2e-2, "blended values, pages out of order")
    # a model stores what the kernel stored: the plain reference on unrounded values is the bound above


@pytest.mark.parametrize("H,G,dk,dv,softcap,rot", [(4, 2, 64, 32, 8.0, (32, 1e4)), (2, 1, 32, 64, 0.0, (16, 1e5)),
                                                     (2, 2, 80, 80, 20.0, None), (3, 1, 128, 16, 5.0, (64, 2e6)),
                                                     (2, 2, 16, 256, 0.0, None), (1, 1, 256, 48, 50.0, (256, 1e4)),
                                                     (8, 2, 128, 128, 20.0, (64, 5e5)), (8, 1, 64, 32, 0.0, (64, 1e4)),
                                                     (12, 2, 32, 48, 6.0, None), (4, 1, 192, 64, 0.0, None)])
def test_tensor_core_and_split_attention_kernels(H, G, dk, dv, softcap, rot):
    rng = np.random.default_rng(dk + 7 * dv)
    T = 330
    q, k, v, gate = (rng.normal(0, 1, (T, n)) for n in (H * dk, G * dk, G * dv, H * dv))
    if not rot:
        k[3] = np.tile(q[200:, :dk].mean(0), G) * 3.0
    q, k, v, gate = (dev(a, torch.bfloat16).float().cpu().numpy().astype(np.float64) for a in (q, k, v, gate))
    scale = 1.3 * dk ** -0.5
    qr, kr = q.reshape(T, H, dk), k.reshape(T, G, dk)
    if rot:
        qr, kr = P.rotate_pairs(qr, np.arange(T), *rot), P.rotate_pairs(kr, np.arange(T), *rot)
    ref = P.capped_attention(qr, kr, v.reshape(T, G, dv), scale, softcap).reshape(T, H * dv)
    out, pre, dec, rows = paged_attention(q, k, v, H, G, dk, dv, scale, softcap, torch.bfloat16, [2, 5, 0, 1, 4, 3], rot,
                                          fast=True, gate=gate)
    close(out, ref, 2e-2, "generic")
    close(pre, ref * P.sigmoid(gate), 2e-2, "prompt kernel")
    close(dec, (ref * P.sigmoid(gate))[rows], 2e-2, "single-token kernel")


def test_softcap_limits_a_huge_score():
    """One key with a score of 300: capped at 5 it keeps a weight that the others can rival; uncapped it takes all."""
    rng = np.random.default_rng(9)
    T, H, dk, dv = 70, 1, 16, 8
    q, k, v = rng.normal(0, 1, (T, dk)), rng.normal(0, 1, (T, dk)), rng.normal(0, 1, (T, dv))
    k[10] = q[-1] * 300.0 / (q[-1] @ q[-1])
    for cap in (5.0, 0.0):
        ref = P.capped_attention(q.reshape(T, 1, dk), k.reshape(T, 1, dk), v.reshape(T, 1, dv), 1.0, cap).reshape(T, dv)
        got = paged_attention(q, k, v, H, 1, dk, dv, 1.0, cap, torch.float32, [1, 0])
        close(got, ref, 2e-5, f"cap {cap}")
    assert np.abs(ref[-1] - v[10]).max() < 1e-6          # uncapped: the last query returns exactly that value
