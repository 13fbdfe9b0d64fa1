"""Lutelorn through the engine, against the plain float64 model: whole prompts, token-by-token decoding,
prompts cut into portions, batches of unequal requests, slots and pages used again, long decoding across
page and graph borders, greedy generation through the library's entry point."""
import numpy as np
import pytest

import qstream_b200 as qs
import plain_lutelorn as P
from lutelorn_util import CONFIGS, assert_close, make_folder
from util import random_tokens

pytestmark = pytest.mark.gpu

CASES = [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("C", "float32"), ("C", "bfloat16"),
         ("D", "float32"), ("D", "bfloat16")]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(folder, plain config, plain weights, library model) per configuration and type, made once."""
    made = {}

    def get(which, dtype):
        if (which, dtype) not in made:
            folder, _ = make_folder(tmp_path_factory.mktemp("lutelorn"), which, dtype)
            pcfg, w = P.load_model(folder)
            made[which, dtype] = (folder, pcfg, w, qs.load_model(folder, dtype=dtype, device="cuda"))
        return made[which, dtype]
    return get


def all_places(n):
    return list(range(n))


@pytest.mark.parametrize("which,dtype", CASES)
def test_whole_prompts(models, which, dtype):
    _, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=512, max_batch=2)
    rng = np.random.default_rng(1)
    for n in (1, 2, 63, 64, 65, 200, 389):       # from 256 tokens on the state mixers cut the prompt into chunks
        toks = random_tokens(rng, n, pcfg["vocab"])
        slot = engine.acquire()
        got = engine.step([slot], [toks], [all_places(n)]).cpu().numpy()
        engine.release(slot)
        assert_close(got, P.logits_whole(pcfg, w, toks), dtype, f"{n} tokens")
    engine.check_status()
    engine.cache.check()


@pytest.mark.parametrize("which,dtype", CASES)
@pytest.mark.parametrize("graphs", [True, False])
def test_token_by_token_equals_the_prompt(models, which, dtype, graphs):
    """The first tokens of a sequence one by one from an empty state, then on across a page border."""
    _, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2, use_graphs=graphs)
    toks = random_tokens(np.random.default_rng(2), 70, pcfg["vocab"])
    ref = P.logits_whole(pcfg, w, toks)
    slot = engine.acquire()
    got = [engine.step([slot], [[t]], [[0]]).cpu().numpy()[0] for t in toks]
    engine.release(slot)
    assert_close(np.stack(got), ref, dtype, "one by one")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 65])
def test_portions(models, which, dtype, portion):
    _, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=256, max_batch=2)
    toks = random_tokens(np.random.default_rng(3), 150, pcfg["vocab"])
    ref = P.logits_whole(pcfg, w, toks)
    slot = engine.acquire()
    got = []
    for a in range(0, len(toks), portion):
        piece = toks[a:a + portion]
        got.append(engine.step([slot], [piece], [all_places(len(piece))]).cpu().numpy())
    engine.release(slot)
    assert_close(np.concatenate(got), ref, dtype, f"portions of {portion}")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
def test_batches_of_unequal_requests_and_reused_slots(models, which, dtype):
    """Prompts of unequal lengths in one step, then one token each until the shorter ones end; a second batch
    takes the slots and pages the first gave back (fewer pages than the two batches need together)."""
    _, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=3)
    rng = np.random.default_rng(4)
    for lens, prompt in (((130, 1, 67), (100, 1, 40)), ((64, 129, 3), (33, 128, 2)), ((90, 70, 110), (89, 1, 64)),
                         ((300, 20, 5), (290, 3, 1))):
        reqs = [random_tokens(rng, n, pcfg["vocab"]) for n in lens]
        refs = [P.logits_whole(pcfg, w, t) for t in reqs]
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
            assert_close(np.concatenate(got[i]), ref, dtype, f"request {i} of lengths {lens}")
        engine.cache.check()
    engine.check_status()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_long_decoding(models, which, dtype):
    """300 tokens one by one after a short prompt: across four page borders and the 256-token border at which
    the engine changes to another captured step; a second sequence runs along and ends early."""
    _, pcfg, w, model = models(which, dtype)
    engine = qs.Engine(model, max_tokens=64 * 8, max_batch=2)
    rng = np.random.default_rng(5)
    a, b = random_tokens(rng, 330, pcfg["vocab"]), random_tokens(rng, 90, pcfg["vocab"])
    ra, rb = P.logits_whole(pcfg, w, a), P.logits_whole(pcfg, w, b)
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
    assert_close(np.stack(ga), ra[29:], dtype, "long sequence")
    assert_close(np.stack(gb), rb[4:], dtype, "short sequence")
    engine.check_status()


@pytest.mark.parametrize("which,dtype", CASES)
def test_greedy_generation_through_the_entry_point(models, which, dtype):
    """More requests than slots, so batches follow one another through the generation loop and the scheduler
    hands slots on.  Every token must be the plain model's choice given the tokens before it."""
    _, pcfg, w, model = models(which, dtype)
    rng = np.random.default_rng(6)
    prompts = [random_tokens(rng, n, pcfg["vocab"]) for n in (5, 1, 40, 2, 66)]
    engine = qs.Engine(model, max_tokens=64 * 6, max_batch=2)
    res = qs.generate(engine, prompts, max_new_tokens=10, sampling=qs.SamplingConfig.greedy(), stop_tokens=())
    assert len(res.batches) >= 3 and all(len(t) == 10 for t in res.tokens)
    for prompt, got in zip(prompts, res.tokens):
        toks = list(prompt)
        for g in got:
            logits = P.logits_whole(pcfg, w, toks)[-1]
            best = int(np.argmax(logits))
            if g != best:
                assert dtype == "bfloat16" and logits[best] - logits[g] < 0.05 * (logits.max() - logits.min()), (toks, g, best)
            toks.append(g)
    engine.cache.check()
    assert engine.cache.slots.n_free == engine.cache.slots.n_slots


def test_a_model_made_from_a_seed_runs_and_saves(tmp_path):
    """`CausalLM.random` and the folder that `write_model_folder` writes hold the same model."""
    cfg = dict(CONFIGS["A"])
    cfg["layers"] = [dict(layer, mixer=dict(layer["mixer"], **({"decay_rank": 6} if layer["type"] == "wkv" else {})))
                     for layer in cfg["layers"]]
    config = qs.config_from_dict(cfg)
    folder = qs.write_model_folder(tmp_path / "made", config, seed=3, dtype="float32", scales=qs.InitScales(0.2, 0.1, 0.1))
    pcfg, w = P.load_model(folder)
    toks = random_tokens(np.random.default_rng(7), 50, pcfg["vocab"])
    ref = P.logits_whole(pcfg, w, toks)
    for model in (qs.load_model(folder, dtype="float32"), qs.CausalLM.random(config, 3, "float32", "cuda", qs.InitScales(0.2, 0.1, 0.1))):
        engine = qs.Engine(model, max_tokens=128, max_batch=1)
        slot = engine.acquire()
        assert_close(engine.step([slot], [toks], [all_places(50)]).cpu().numpy(), ref, "float32", "seeded model")
