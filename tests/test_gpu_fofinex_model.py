"""Fofinex through the engine, against the plain float64 model: whole prompts, token-by-token decoding, prompts cut
into portions, batches of unequal requests, slots and pages used again, long decoding across page and graph borders,
single far keys, greedy generation through the library's entry point."""
import copy

import numpy as np
import pytest

import qstream_b200 as qs
import plain_fofinex as P
import fofinex_util
from fofinex_util import CONFIGS, is_routed, latent_layer, load_plain, logits_error, make_folder, make_weights, mlstm_layer, write_folder
from util import random_tokens

pytestmark = pytest.mark.gpu

CASES = [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "bfloat16"),
         ("Bd", "bfloat16"), ("Cd", "bfloat16")]
_REFS = {}


def reference(key, pcfg, w, toks):
    """The plain model's logits of a sequence, computed once per (model, sequence)."""
    k = (key, tuple(toks))
    if k not in _REFS:
        _REFS[k] = P.forward(pcfg, w, toks)
    return _REFS[k]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(key, plain config, plain weights, library model) per configuration and type, made once."""
    made = {}

    def get(which, dtype):
        if (which, dtype) not in made:
            folder, _ = make_folder(tmp_path_factory.mktemp("fofinex"), which, dtype)
            pcfg, w = load_plain(folder)
            made[which, dtype] = ((which, dtype), pcfg, w, qs.load_model(folder, dtype=dtype, device="cuda"))
        return made[which, dtype]
    return get


def assert_close(got, ref, dtype, what="", cfg=None):
    fofinex_util.assert_close(got, ref, dtype, what, routed=cfg is None or is_routed(cfg))


# other makes of model: whole prompts and single tokens only
OTHER_CASES = [(which, dtype) for which in ("W", "M", "L") for dtype in ("float32", "bfloat16")]


def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("which,dtype", CASES + OTHER_CASES)
def test_whole_prompts(models, which, dtype):
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=512, max_batch=2)
    # An empty memory's first output is v times the sign of k.q (the quotient's denominator is |n.q| = b |k.q|): a token
    # whose k.q lies within bfloat16's rounding of zero tests no kernel, and the memories-only model met one.
    rng = np.random.default_rng(21 if which == "M" else 1)
    for n in (1, 2, 33, 64, 65, 389):       # from 256 tokens on the matrix memory cuts the prompt into chunks
        toks = random_tokens(rng, n, pcfg["vocab"])
        slot = engine.acquire()
        got = engine.step([slot], [toks], [all_places(n)]).cpu().numpy()
        engine.release(slot)
        assert_close(got, reference(key, pcfg, w, toks), dtype, f"{n} tokens", pcfg)
    engine.check_status()
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", CASES + OTHER_CASES)
@pytest.mark.parametrize("graphs", [True, False])
def test_token_by_token_equals_the_prompt(models, which, dtype, graphs):
    """The first tokens of a sequence one by one from an empty state, then on across a page border."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2, use_graphs=graphs)
    toks = random_tokens(np.random.default_rng(2), 70, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([slot], [[t]], [[0]]).cpu().numpy()[0] for t in toks]
    engine.release(slot)
    assert_close(np.stack(got), ref, dtype, "one by one", pcfg)
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 65])
def test_portions(models, which, dtype, portion):
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2)
    toks = random_tokens(np.random.default_rng(3), 150, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = []
    for a in range(0, len(toks), portion):
        piece = toks[a:a + portion]
        got.append(engine.step([slot], [piece], [all_places(len(piece))]).cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, f"portions of {portion}", pcfg)
    engine.check_status()


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_a_long_prompt_in_long_portions(models, which, dtype):
    """Portions beyond 256 tokens run the matrix memory's chunks from a state that earlier portions left."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=1024, max_batch=1)
    toks = random_tokens(np.random.default_rng(9), 700, pcfg["vocab"])
    ref = reference(key, pcfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([slot], [toks[a:b]], [all_places(b - a)]).cpu().numpy() for a, b in ((0, 300), (300, 301), (301, 700))]
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, "portions of 300, 1 and 399", pcfg)
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
def test_batches_of_unequal_requests_and_reused_slots(models, which, dtype):
    """Prompts of unequal lengths in one step, then one token each until the shorter ones end; a second batch
    takes the slots and pages the first gave back (fewer pages than the two batches need together)."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=3)
    rng = np.random.default_rng(4)
    for lens, prompt in (((130, 1, 67), (100, 1, 40)), ((64, 129, 3), (33, 128, 2)), ((300, 20, 5), (290, 3, 1))):
        reqs = [random_tokens(rng, n, pcfg["vocab"]) for n in lens]
        refs = [reference(key, pcfg, w, t) for t in reqs]
        slots = [engine.acquire() for _ in reqs]
        got = [[] for _ in reqs]
        first = engine.step(slots, [t[:p] for t, p in zip(reqs, prompt)], [all_places(p) for p in prompt]).cpu().numpy()
        at = 0
        for i, p in enumerate(prompt):
            got[i].append(first[at:at + p])
            at += p
        pos = list(prompt)
        live = list(range(len(reqs)))
        for i in [i for i in live if pos[i] == len(reqs[i])]:       # a request that was all prompt
            engine.release(slots[i])
            live.remove(i)
        while live:
            out = engine.step([slots[i] for i in live], [[reqs[i][pos[i]]] for i in live], [[0]] * len(live)).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
            for i in [i for i in live if pos[i] == len(reqs[i])]:
                engine.release(slots[i])
                live.remove(i)
        for i, ref in enumerate(refs):
            assert_close(np.concatenate(got[i]), ref, dtype, f"request {i} of lengths {lens}", pcfg)
        engine.cache.check()
    engine.check_status()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "bfloat16"), ("Cd", "bfloat16")])
def test_long_decoding(models, which, dtype):
    """300 tokens one by one after a short prompt: across four page borders and the 256-token border at which
    the engine changes to another captured step; a second sequence runs along and ends early."""
    key, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=2)
    rng = np.random.default_rng(5)
    a, b = random_tokens(rng, 330, pcfg["vocab"]), random_tokens(rng, 90, pcfg["vocab"])
    ra, rb = reference(key, pcfg, w, a), reference(key, pcfg, w, b)
    sa, sb = engine.acquire(), engine.acquire()
    first = engine.step([sa, sb], [a[:30], b[:5]], [[29], [4]]).cpu().numpy()
    ga, gb = [first[0]], [first[1]]
    for i in range(300):
        both = 5 + i < len(b)
        out = engine.step([sa, sb] if both else [sa], [[a[30 + i]], [b[5 + i]]] if both else [[a[30 + i]]]).cpu().numpy()
        ga.append(out[0])
        if both:
            gb.append(out[1])
        elif sb is not None:
            engine.release(sb)
            sb = None
    engine.release(sa)
    assert_close(np.stack(ga), ra[29:], dtype, "long sequence", pcfg)
    assert_close(np.stack(gb), rb[4:], dtype, "short sequence", pcfg)
    engine.check_status()


# Sharp scores: with a factor of 6 on q.k a query's softmax rests on one or two keys, anywhere among the hundreds
# before it, so a key that is lost, one place off or read from the wrong page moves the row's logits by their whole
# spread; and a forget gate close to one lets the first tokens of a sequence weigh on the last.
def sharp(factor):
    return {"architecture": "Fofinex", "vocab": 80, "width": 96, "norm": {"eps": 1e-5},
            "layers": [latent_layer(2, 16, 16, 32, 24, 32, factor, base=1e4, scaling=(2.0, 256, 32.0, 1.0), mlp=None),
                       mlstm_layer(2, 16, 16, 30.0, mlp=None),
                       latent_layer(3, 16, 16, 16, 24, 32, factor, base=1e4, scaling=(2.0, 256, 32.0, 1.0), kv_from=0, mlp=None)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_far_keys_in_prompts_and_in_decoding(tmp_path, dtype):
    # bfloat16 rounds a score of 30 by a tenth, which is a tenth of the key's weight: less sharp there
    cfg = sharp(12.0 if dtype == "float32" else 5.0)
    weights = make_weights(cfg, 11)
    weights["l1.mix.f.b"] = np.full_like(weights["l1.mix.f.b"], 9.0)        # forgets a ten-thousandth per token
    folder = write_folder(tmp_path / "sharp", cfg, weights, dtype)
    pcfg, w = load_plain(folder)
    toks = random_tokens(np.random.default_rng(12), 600, cfg["vocab"])
    ref = P.forward(pcfg, w, toks)
    # the sharpness is there: the last rows lose much of their logits when the first 64 keys are cut off
    cut = P.forward(pcfg, w, toks[64:])
    assert np.median(logits_error(cut[-100:], ref[-100:])) > (0.2 if dtype == "float32" else 0.1)
    model = qs.load_model(folder, dtype=dtype, device="cuda")
    engine = qs.Engine(model, max_tokens=1024, max_batch=2)
    slot = engine.acquire()
    got = [engine.step([slot], [toks[:520]], [all_places(520)]).cpu().numpy()]
    got += [engine.step([slot], [[t]], [[0]]).cpu().numpy() for t in toks[520:]]
    engine.release(slot)
    e = logits_error(np.concatenate(got), ref)
    if dtype == "float32":
        assert e.max() <= 3e-4, (e.max(), int(e.argmax()))
    else:                                               # sharp scores amplify the rounding of q and k as well
        assert np.median(e) <= 0.03 and np.quantile(e, 0.95) <= 0.1 and e.max() <= 0.5, (np.median(e), e.max(), int(e.argmax()))
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
def test_greedy_generation_through_the_entry_point(models, which, dtype):
    """More requests than slots, so batches follow one another through the generation loop and the scheduler
    hands slots on.  Every token must be the plain model's choice given the tokens before it."""
    key, pcfg, w, model = models(which, dtype)
    rng = np.random.default_rng(6)
    prompts = [random_tokens(rng, n, pcfg["vocab"]) for n in (5, 1, 40, 2, 66)]
    engine = qs.Engine(model, max_tokens=64 * 6, max_batch=2)
    res = qs.generate(engine, prompts, max_new_tokens=8, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert len(res.batches) >= 3 and all(len(t) == 8 for t in res.tokens)
    for prompt, got in zip(prompts, res.tokens):
        toks = list(prompt)
        for g in got:
            logits = P.forward(pcfg, w, toks)[-1]
            best = int(np.argmax(logits))
            if g != best:
                assert dtype == "bfloat16" and logits[best] - logits[g] < 0.1 * (logits.max() - logits.min()), (toks, g, best)
            toks.append(g)
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


def test_a_model_made_from_a_seed_runs_and_saves(tmp_path):
    """`CausalLM.random` and the folder that `write_model_folder` writes hold the same model."""
    config = qs.config_from_dict(copy.deepcopy(CONFIGS["A"]))
    scales = qs.InitScales(0.2, 0.1, 0.1)
    folder = qs.write_model_folder(tmp_path / "made", config, seed=3, dtype="float32", scales=scales)
    pcfg, w = load_plain(folder)
    toks = random_tokens(np.random.default_rng(7), 50, pcfg["vocab"])
    ref = P.forward(pcfg, w, toks)
    for model in (qs.load_model(folder, dtype="float32"), qs.CausalLM.random(config, 3, "float32", "cuda", scales)):
        engine = qs.Engine(model, max_tokens=128, max_batch=1)
        slot = engine.acquire()
        assert_close(engine.step([slot], [toks], [all_places(50)]).cpu().numpy(), ref, "float32", "seeded model")
