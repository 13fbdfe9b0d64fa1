"""Mixers that carry a matrix of state per head from token to token instead of keys and values.

`DecayAttention` ("lightning"): linear attention with a fixed decay per head,
    S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t,
q, k, v = act(W h); the concatenated heads get one RMS norm, a sigmoid gate from h, and W_o.

`Wkv` ("wkv"): RWKV-style time mixing.  Five mixes of h with the previous token's h feed r, k, v, the gate and a
two-matrix bottleneck whose output d gives the decay w = exp(-exp(d + w0)) per token and key channel;
    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t,  S_t = diag(w_t) S_{t-1} + k_t v_t^T;
each head's o is divided by its root mean square, then weight, silu gate, W_o.

Both keep S in 32-bit per sequence (`StateNeed`), zero when a slot is taken, read at the start of a step and
written at its end by one kernel that walks a sequence's tokens in order (csrc/recurrent.cu); single tokens and
short prompts take that path, a long prompt is cut into chunks that run side by side and are joined by a prefix
over the chunks' states.  The projections are matrix products in the engine's type; decays, the recurrence,
its output and the norms are 32-bit.
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..csrc import ops
from ..errors import QsError, QStreamError
from ..weights.loader import TensorDecl
from .base import Mixer, register
from .linear import linear


CHUNK_TOKENS = 64            # a long prompt is cut into chunks of this many tokens that run side by side
CHUNKED_FROM = 256           # the longest sequence of a step from which that pays


def scan_chunks(batch, device):
    """The step's sequences cut into chunks for `ops.state_scan`, or None where the walk in order serves: single
    tokens, short prompts, and captured steps (whose host lists are not the step's)."""
    cached = getattr(batch, "_scan_chunks", False)
    if cached is not False:
        return cached
    out = None
    n_new = batch.new_tokens
    if n_new and len(n_new) == batch.n_seq and sum(n_new) == batch.n_tokens and max(n_new) >= CHUNKED_FROM:
        import numpy as np
        starts, owners, row = [0], [0], 0
        for n in n_new:
            starts += [row + min(n, a + CHUNK_TOKENS) for a in range(0, n, CHUNK_TOKENS)]
            row += n
            owners.append(len(starts) - 1)
        n_chunks = len(starts) - 1
        host = torch.from_numpy(np.concatenate([starts, np.arange(n_chunks), owners]).astype(np.int32))
        dev = host.pin_memory().to(device, non_blocking=True) if device.type == "cuda" else host
        out = (dev[:n_chunks + 1], dev[n_chunks + 1:2 * n_chunks + 1], dev[2 * n_chunks + 1:], n_chunks)
    batch._scan_chunks = out
    return out


class DecayAttention(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hk, hv = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim
        return {"q": TensorDecl((hk, spec.width)), "k": TensorDecl((hk, spec.width)), "v": TensorDecl((hv, spec.width)),
                "g": TensorDecl((hv, spec.width)), "o": TensorDecl((spec.width, hv)), "norm": TensorDecl((hv,), "norm_weight")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if len(spec.decay) != spec.n_heads:
            raise QStreamError(QsError.INVALID_MODEL, f"{len(spec.decay)} decays for {spec.n_heads} heads")
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()    # one product for all four
        self.w_out, self.norm = tensors["o"], tensors["norm"]
        self.decay = torch.tensor(spec.decay, dtype=torch.float32).to(runtime.device)

    def state_need(self):
        s = self.spec
        return StateNeed((s.n_heads, s.value_dim, s.key_dim), torch.float32)

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        hk, hv = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        p = linear(h, self.w_in)
        o = ops.state_scan("decay", p[:, :hk], p[:, hk:2 * hk], p[:, 2 * hk:2 * hk + hv], step.state(cache_id),
                           b.seq_start, b.seq_slot, b.n_seq, s.n_heads, s.key_dim, s.value_dim,
                           head_decay=self.decay, in_activation=s.activation, chunks=scan_chunks(b, h.device))
        y = ops.gated_group_norm(o, hv, self.norm, p[:, 2 * hk + hv:], "sigmoid", s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


MIXES = ("r", "k", "v", "g", "w")


class Wkv(Mixer):
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        n, D, R = spec.n_heads * spec.head_dim, spec.width, spec.decay_rank
        d = {name: TensorDecl((n, D)) for name in ("r", "k", "v", "g")}
        d.update({"o": TensorDecl((D, n)), "w1": TensorDecl((R, D)), "w2": TensorDecl((n, R)),
                  "w0": TensorDecl((n,), "bias"), "u": TensorDecl((spec.n_heads, spec.head_dim), "bias"),
                  "norm": TensorDecl((n,), "norm_weight")})
        d.update({"mu_" + m: TensorDecl((D,), "fraction") for m in MIXES})
        return d

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.w = {name: tensors[name] for name in ("r", "k", "v", "g", "o", "w1", "w2")}
        self.w0 = tensors["w0"].float().contiguous()
        self.u, self.norm = tensors["u"].contiguous(), tensors["norm"]
        self.mu = torch.stack([tensors["mu_" + m].float() for m in MIXES]).contiguous()        # [5, D] float32

    def state_need(self):
        s = self.spec
        return {"matrix": StateNeed((s.n_heads, s.head_dim, s.head_dim), torch.float32),
                "last_input": StateNeed((s.width,), self.runtime.dtype)}

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        n = s.n_heads * s.head_dim
        last = step.state(cache_id, "last_input")
        mixed = ops.token_shift(h, self.mu, last, b.tok_slot, b.tok_pos)
        ops.keep_last_rows(last, h, b.seq_start, b.seq_slot, b.n_seq)      # after the shift has read it
        r, k, v = (linear(mixed[i], self.w[name]) for i, name in enumerate(("r", "k", "v")))
        gate = linear(mixed[3], self.w["g"])
        d = linear(linear(mixed[4], self.w["w1"], activation="tanh"), self.w["w2"], self.w0, out_dtype=torch.float32)
        o = ops.state_scan("wkv", r, k, v, step.state(cache_id, "matrix"), b.seq_start, b.seq_slot, b.n_seq,
                           s.n_heads, s.head_dim, s.head_dim, decay_logits=d, bonus=self.u, chunks=scan_chunks(b, h.device))
        y = ops.gated_group_norm(o, s.head_dim, self.norm, gate, "silu", s.eps, h.dtype)
        return linear(y, self.w["o"], None, residuals=residuals, out_dtype=out_dtype)


class Mlstm(Mixer):
    """Matrix memory with exponential gates.  q, k, v and the output gate are one product in the engine's type; the
    two gate projections are a product of their own with a 32-bit result.  `ops.mlstm_gates` turns the log gates into
    the recurrence's factors a_t, b_t with the running maximum m per sequence and head; the scan (the kernel of the
    other matrix-state mixers, in its "gated" form) carries S and, as one more column, the normaliser n; the last
    kernel divides, takes each head's unit RMS, the weight and the sigmoid gate."""
    captures_any_step = True

    @classmethod
    def declare(cls, spec):
        hk, hv, H = spec.n_heads * spec.key_dim, spec.n_heads * spec.value_dim, spec.n_heads
        return {"q": TensorDecl((hk, spec.width)), "k": TensorDecl((hk, spec.width)), "v": TensorDecl((hv, spec.width)),
                "g": TensorDecl((hv, spec.width)), "o": TensorDecl((spec.width, hv)), "norm": TensorDecl((hv,), "norm_weight"),
                "i": TensorDecl((H, spec.width)), "f": TensorDecl((H, spec.width)),
                "i_bias": TensorDecl((H,), "bias"), "f_bias": TensorDecl((H,), "bias")}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).contiguous()
        self.b_gates = torch.cat([tensors["i_bias"].float(), tensors["f_bias"].float()]).contiguous()
        self.w_out, self.norm = tensors["o"], tensors["norm"]

    def state_need(self):
        s = self.spec
        return {"matrix": StateNeed((s.n_heads, s.value_dim + 1, s.key_dim), torch.float32),
                "maximum": StateNeed((s.n_heads,), torch.float32)}

    def forward(self, h, step, cache_id, residuals=(), out_dtype=None):
        s, b = self.spec, step.batch
        hk, hv = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        p = linear(h, self.w_in)
        raw = linear(h, self.w_gates, self.b_gates, out_dtype=torch.float32)
        a, w, m = ops.mlstm_gates(raw, s.gate_cap, step.state(cache_id, "maximum"), b.seq_start, b.seq_slot, b.n_seq, s.n_heads)
        o = ops.state_scan("gated", p[:, :hk], p[:, hk:2 * hk], p[:, 2 * hk:2 * hk + hv], step.state(cache_id, "matrix"),
                           b.seq_start, b.seq_slot, b.n_seq, s.n_heads, s.key_dim, s.value_dim + 1, token_decay=a,
                           token_weight=w, q_scale=s.key_dim ** -0.5, chunks=scan_chunks(b, h.device))
        y = ops.mlstm_output(o, m, self.norm, p[:, 2 * hk + hv:], s.n_heads, s.value_dim, s.eps, h.dtype)
        return linear(y, self.w_out, None, residuals=residuals, out_dtype=out_dtype)


register("mixer", "lightning", DecayAttention)
register("mixer", "mlstm", Mlstm)
register("mixer", "wkv", Wkv)
