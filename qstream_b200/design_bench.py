"""Prefill and decode throughput of a Lutelorn model beside a GPT-J model of equal size, and the kernels that
Lutelorn adds, each against its roofline (`bench.py --design lutelorn`).

Sizes resemble a real model's layers: a width, heads of 128 (attention: a quarter as many key heads), a gated
feed-forward of 8/3 width on every layer, the mixers in the order lightning, attention, lightning, wkv; the
GPT-J model beside it has the same width, number of layers and heads and a feed-forward of 4 width, which gives
nearly the same number of weights per layer.  Weights are random, tokens uniform.

Timing: CUDA events on the launching stream, three warm-up runs, a buffer larger than L2 written between timed
kernels (per-kernel table) or steps that read more than L2 holds (models).
"""
from __future__ import annotations

import json

SIZES = {"w2048": dict(width=2048, layers=8), "w4096": dict(width=4096, layers=4)}
VOCAB = 32000
FP32_LANES_PER_SM, SMS = 128, 148


def lutelorn_config(width: int, layers: int) -> dict:
    heads = width // 128
    ff = (width * 8 // 3 + 255) // 256 * 256
    mlp = {"kind": "dense", "ff": ff}
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * i / max(heads - 1, 1)) for i in range(heads)]
    kinds = {
        "lightning": {"type": "lightning", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "decay": decay}, "mlp": mlp},
        "attention": {"type": "attention", "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128,
                                                     "rot": {"dims": 64, "base": 10000.0}, "scale": 128 ** -0.5, "softcap": 50.0,
                                                     "v_mix": True}, "mlp": mlp},
        "wkv": {"type": "wkv", "mixer": {"heads": width // 64, "dim": 64, "decay_rank": 64}, "mlp": mlp},
    }
    order = ["lightning", "attention", "lightning", "wkv"]
    return {"architecture": "Lutelorn", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
            "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31337, "mul_cur": 7919}},
            "layers": [kinds[order[i % 4]] for i in range(layers)], "max_positions": 8192}


def gptj_config(width: int, layers: int) -> dict:
    return dict(n_layer=layers, n_embd=width, n_head=width // 128, n_positions=8192, vocab_size=VOCAB, rotary_dim=64,
                n_inner=4 * width, activation_function="gelu_new", layer_norm_epsilon=1e-5, architectures=["GPTJForCausalLM"])


class Timer:
    def __init__(self, torch):
        self.torch = torch
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def kernel(self, fn, repeats=10, warmup=3) -> float:
        """Milliseconds of one call, L2 flushed before each timed call."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        total = 0.0
        for _ in range(repeats):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / repeats


def model_throughput(qs, torch, np, model, vocab, prompt_len, batch, ctx, steps, warmup):
    """Tokens per second of one prompt of `prompt_len` tokens, and of decode steps of `batch` sequences that end at
    a context of `ctx`."""
    from .csrc import ops
    from .engine import TokenFeed
    rng = np.random.default_rng(0)
    engine = qs.Engine(model, max_tokens=max(batch * ctx, prompt_len) + 64, max_batch=batch, max_context=max(ctx, prompt_len))
    times = []
    for _ in range(3 + 3):
        slot = engine.acquire()
        toks = [int(t) for t in rng.integers(0, vocab, prompt_len)]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([slot], [toks])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.release(slot)
    prefill_ms = sum(times[3:]) / 3
    slots = [engine.acquire() for _ in range(batch)]
    start = ctx - steps - warmup
    logits = None
    per = max(1, 4096 // start)
    outs = []
    for i in range(0, batch, per):
        outs.append(engine.step(slots[i:i + per], [[int(t) for t in rng.integers(0, vocab, start)] for _ in slots[i:i + per]]).clone())
    tokens = ops.argmax(torch.cat(outs))
    rows = list(range(batch))

    def one():
        nonlocal tokens
        tokens = ops.argmax(engine.step(slots, TokenFeed(tokens, rows)))
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    engine.check_status()
    ms = a.elapsed_time(b) / steps
    launches = ops.launch_count() - n0
    del engine
    torch.cuda.empty_cache()
    return {"prefill_tokens": prompt_len, "prefill_ms": round(prefill_ms, 3), "prefill_tok_s": round(prompt_len * 1e3 / prefill_ms, 1),
            "decode_batch": batch, "decode_context": ctx, "decode_ms": round(ms, 4), "decode_tok_s": round(batch * 1e3 / ms, 1),
            "launches": launches}


def kernel_table(torch, np, pk, width=2048, T=4096, batch=32, ctx=2048):
    """Each kernel of the new parts and the like kernel of the GPT-J parts by itself: milliseconds and the fraction
    of its roofline (copy bandwidth, bfloat16 tensor peak, or 32-bit multiply-add peak of the CUDA cores)."""
    from .csrc import attention_bf16, ops
    t = Timer(torch)
    bf, f32 = torch.bfloat16, torch.float32
    dev = "cuda"
    H, d = width // 128, 128
    G = max(1, H // 4)
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32 = 2.0 * FP32_LANES_PER_SM * SMS * pk.get("sm_max_mhz", 1965.0) * 1e6
    rows = []

    def add(name, like, ms, nbytes=0, flops=0, bound="hbm"):
        peak = {"hbm": hbm, "tensor": tens, "fp32": fp32}[bound]
        done = (nbytes if bound == "hbm" else flops) / (ms * 1e-3)
        rows.append({"kernel": name, "like": like, "ms": round(ms, 4), "bound": bound, "frac": round(done / peak, 4)})

    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)          # noqa: E731
    for n_rows, tag in ((T, "prompt"), (batch, "decode")):
        x = torch.randn(n_rows, width, device=dev)
        y = torch.randn(n_rows, width, device=dev)
        w = torch.randn(width, device=dev, dtype=bf)
        xb = x.to(bf)
        add(f"rmsnorm {tag}", "layernorm", t.kernel(lambda: ops.rmsnorm(x, w, 1e-6, 1.0, out_dtype=bf)), n_rows * width * 6)
        add(f"rmsnorm + update {tag}", "layernorm", t.kernel(lambda: ops.rmsnorm(x, w, 1e-6, 1.0, out_dtype=bf, update=y, mult=0.0)),
            n_rows * width * 14)
        add(f"layernorm {tag} (GPT-J)", "", t.kernel(lambda: ops.layernorm(xb, w, w, 1e-5, settled=True)), n_rows * width * 4)
        o = torch.randn(n_rows, width, device=dev)
        g = torch.randn(n_rows, width, device=dev, dtype=bf)
        add(f"gated group norm {tag}", "layernorm", t.kernel(lambda: ops.gated_group_norm(o, width, w, g, "sigmoid", 1e-6, bf)),
            n_rows * width * 8)
        mu = torch.rand(5, width, device=dev)
        last = torch.zeros(batch, width, device=dev, dtype=bf)
        slot = i32([0] * n_rows) if tag == "prompt" else i32(list(range(batch)))
        pos = i32(list(range(n_rows))) if tag == "prompt" else i32([ctx - 1] * batch)
        add(f"token shift {tag}", "layernorm", t.kernel(lambda: ops.token_shift(xb, mu, last, slot, pos)), n_rows * width * 12)
        ab = torch.randn(n_rows, 2 * ((width * 8 // 3 + 255) // 256 * 256), device=dev, dtype=bf)     # the models' feed-forward width
        add(f"gated activation {tag}", "(in GPT-J's product)", t.kernel(lambda: ops.gated_act(ab, "silu")), ab.numel() * 3)

    # matrix states: one prompt of T tokens (cut into chunks, as the mixers do from 256 tokens on), and `batch` single tokens
    from .parts.recurrent import CHUNK_TOKENS
    n_chunks = T // CHUNK_TOKENS
    chunks = (i32(list(range(0, T + 1, CHUNK_TOKENS))), i32(list(range(n_chunks))), i32([0, n_chunks]), n_chunks)
    one_start, one_slot = i32([0, T]), i32([0])
    dec_start, dec_slot = i32(list(range(batch + 1))), i32(list(range(batch)))
    for mode, heads, dk in (("decay", H, d), ("wkv", width // 64, 64)):
        n = heads * dk
        q, k, v = (torch.randn(T, n, device=dev, dtype=bf) for _ in range(3))
        state = torch.zeros(batch, heads, dk, dk, device=dev)
        extra = dict(head_decay=torch.full((heads,), 0.99, device=dev)) if mode == "decay" else \
            dict(decay_logits=torch.randn(T, n, device=dev), bonus=torch.randn(heads, dk, device=dev, dtype=bf))
        ms = t.kernel(lambda: ops.state_scan(mode, q, k, v, state, one_start, one_slot, 1, heads, dk, dk, chunks=chunks, **extra))
        # the chunks' own part and the part of the state they start from: 2 + 1 multiply-adds per state element and token
        add(f"state scan {mode} prompt {T} (4 kernels)", "attention prompt", ms, flops=6.0 * T * heads * dk * dk, bound="fp32")
        qd, kd, vd = q[:batch], k[:batch], v[:batch]
        if mode == "wkv":
            extra["decay_logits"] = extra["decay_logits"][:batch]
        ms = t.kernel(lambda: ops.state_scan(mode, qd, kd, vd, state, dec_start, dec_slot, batch, heads, dk, dk, **extra))
        add(f"state scan {mode} decode {batch}", "attention decode", ms, 2 * state.numel() * 4)

    # attention: prompt of T tokens, decode of `batch` tokens at context ctx; GPT-J's form (values as wide as keys, no
    # cap, no gate, a key head per query head) and Lutelorn's (grouped keys, capped scores, gate)
    dslot, dpos = i32(list(range(batch))), i32([ctx - 1] * batch)
    for name, g_heads, cap, gated in (("(GPT-J)", H, 0.0, False), ("capped, gated, grouped", G, 50.0, True)):
        n_pages = batch * ctx // 64
        kc = torch.randn(n_pages, g_heads, 64, d, device=dev, dtype=bf)
        vc = torch.randn(n_pages, g_heads, 64, d, device=dev, dtype=bf)
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, ctx // 64)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        q = torch.randn(T, H * d, device=dev, dtype=bf)
        gate = torch.randn(T, H * d, device=dev, dtype=bf) if gated else None
        tl = min(T, ctx)
        tiles = torch.tensor([(a, min(128, tl - a), a, 0) for a in range(0, tl, 128)][::-1], dtype=torch.int32, device=dev)
        qp, gp = q[:tl], (gate[:tl] if gated else None)
        ms = t.kernel(lambda: attention_bf16.prefill(qp, H, g_heads, d, d ** -0.5, 0, tiles, table, 64, kc, vc, status,
                                                     softcap=cap, gate=gp))
        add(f"attention prompt {tl} {name}", "" if not gated else "attention prompt (GPT-J)", ms, flops=4.0 * H * d * tl * tl / 2, bound="tensor")
        qd = q[:batch].contiguous()
        gd = gate[:batch].contiguous() if gated else None
        ms = t.kernel(lambda: attention_bf16.decode(qd, H, g_heads, d, d ** -0.5, 0, dslot, dpos, table, 64, kc, vc, ctx, status,
                                                    softcap=cap, gate=gd))
        add(f"attention decode {batch} x {ctx} {name}", "" if not gated else "attention decode (GPT-J)", ms, batch * ctx * g_heads * d * 4)
    return rows


def run(args, pk) -> int:
    import numpy as np
    import torch
    import qstream_b200 as qs
    out = {"impl": "ours", "design": "lutelorn", "beside": "gptj", "dtype": "bf16", "data": "synthetic token ids, random weights",
           "peaks": {k: pk[k] for k in ("hbm_gbs", "bf16_tflops", "source")}, "sizes": {}}
    for name, size in SIZES.items():
        entry = {}
        for which, cfg in (("lutelorn", lutelorn_config(**size)), ("gptj", gptj_config(**size))):
            model = qs.CausalLM.random(qs.config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
            r = model_throughput(qs, torch, np, model, VOCAB, 2048, 8, 1024, min(args.steps, 32), max(3, min(args.warmup, 4)))
            r["weights_mb"] = round(model.weight_bytes / 2**20, 1)
            entry[which] = r
            del model
            torch.cuda.empty_cache()
        out["sizes"][name] = entry
    out["kernels"] = kernel_table(torch, np, pk)
    print(json.dumps(out))
    return 0
