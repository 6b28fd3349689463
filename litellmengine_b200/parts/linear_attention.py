"""Gated linear attention: a mixer whose memory is a fixed-size state per request, not pages."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from ..cache import StateNeed
from ..config.specs import MixerSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .attention import BranchMixer
from .context import StageContext, StepPrelude
from .registry import register_mixer


class ScanWork(StepPrelude):
    """How the recurrence kernels cut a step.  An entry of fewer than `CHUNKED_FROM` tokens (a single
    decoded token, a short portion) is one work item that runs in one pass from the request's state to
    the request's state.  A longer portion is cut into chunks of `CHUNK` tokens that run side by side:
    every chunk first computes its own contribution from a zero state, a chain kernel then walks each
    entry's chunks in order to find the state that enters each, and a second pass over the chunks
    produces the outputs.  Items are int32 (entry, first row, tokens, scratch index); chains (entry,
    first scratch index, chunks)."""
    name = "scan_work"
    CHUNK = 64
    CHUNKED_FROM = 256

    @dataclass
    class Views:
        short: torch.Tensor          # int32 [num_short, 4]
        chunks: torch.Tensor         # int32 [num_chunks, 4]
        chains: torch.Tensor         # int32 [num_chains, 3]
        num_short: int
        num_chunks: int
        num_chains: int

    def sections(self, max_tokens: int, max_entries: int):
        return {"short": 4 * max_entries, "chunks": 4 * (max_tokens // self.CHUNK + max_entries),
                "chains": 3 * max_entries}

    def fill(self, facts, out):
        short, chunks, chains = [], [], []
        for i, (q0, n) in enumerate(zip(facts.q_start.tolist(), facts.q_len.tolist())):
            if n < self.CHUNKED_FROM:
                short.append((i, q0, n, 0))
                continue
            first = len(chunks)
            for at in range(0, n, self.CHUNK):
                chunks.append((i, q0 + at, min(self.CHUNK, n - at), len(chunks)))
            chains.append((i, first, len(chunks) - first))
        for key, rows in (("short", short), ("chunks", chunks), ("chains", chains)):
            if rows:
                flat = np.asarray(rows, dtype=np.int64).reshape(-1)
                out[key][:len(flat)] = flat
        return len(short), len(chunks), len(chains)

    def views(self, dev, filled):
        ns, nc, nh = filled
        return ScanWork.Views(dev["short"][:4 * ns].view(ns, 4), dev["chunks"][:4 * nc].view(nc, 4),
                              dev["chains"][:3 * nh].view(nh, 3), ns, nc, nh)


@register_mixer("gla")
class GatedLinearAttention(BranchMixer):
    """Per head a state S [D, V] (32-bit, one per request and stage, zero at admission):

        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t

    with q = W_q x / sqrt(D), k = W_k x, v = W_v x and a decay per key channel alpha = sigmoid(z)^(1/tau),
    z = W_a2 (W_a1 x) + b (a low-rank projection; its second half runs in 32-bit inside the decay kernel).
    Each head's o is RMS-normed over V with one weight [V] shared by the heads, multiplied by silu(W_g x),
    and the concatenated heads go through W_o.  One product yields [q | k | v | g | a1] per token in
    float32; the recurrence, the norm and the gate are one kernel."""

    graph_safe = True           # kernels on the current stream only; their grids follow the step's entries,
    any_division_safe = False   # so a captured graph serves steps with the same work lists (see graph_variant)

    _DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight", "norm": "o_norm.weight", "a1": "a_proj.0.weight", "a2": "a_proj.1.weight",
                      "a2_bias": "a_proj.1.bias"}

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        params = dict(spec.params)
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        if self.H <= 0 or self.D <= 0 or self.V <= 0:
            raise ValueError("gated linear attention needs positive heads, key width and value width")
        self.tau = float(params.get("tau", 1.0))
        if not self.tau > 0:
            raise ValueError("tau must be positive")
        self.rank = params.get("rank")                  # None: read from the stored tensors
        self.eps = float(params.get("eps", 1e-6))          # of the per-head output norm
        self.spec, self.hidden, self.dtype, self.device = spec, hidden_size, compute_dtype, torch.device(device)
        self.names = dict(self._DEFAULT_NAMES, **dict(spec.tensor_names))
        self.q_off, self.k_off = 0, self.H * self.D
        self.v_off = 2 * self.H * self.D
        self.g_off = self.v_off + self.H * self.V
        self.a_off = self.g_off + self.H * self.V
        self.in_width = self.a_off + (self.rank or 0)
        self.out_width = self.H * self.V
        self.w2 = self.b2 = self.norm_w = None
        if self.device.type == "cuda" and not ops.gla_supported(self.D, self.V):
            raise ValueError(f"gated linear attention: a state of {self.D} x {self.V} per head is more than "
                             "the recurrence kernel keeps in one block's registers")

    def parameters(self) -> Dict[str, ParamSpec]:
        n, r = self.names, self.rank if self.rank is not None else -1
        hd, hv = self.H * self.D, self.H * self.V
        return {n["q"]: ParamSpec((hd, self.hidden)), n["k"]: ParamSpec((hd, self.hidden)),
                n["v"]: ParamSpec((hv, self.hidden)), n["g"]: ParamSpec((hv, self.hidden)),
                n["o"]: ParamSpec((self.hidden, hv)),
                n["norm"]: ParamSpec((self.V,), role="scale", init=("one_plus_normal", 0.01)),
                n["a1"]: ParamSpec((r, self.hidden)),
                n["a2"]: ParamSpec((hd, r), role="scale", init=("normal", 0.02)),
                n["a2_bias"]: ParamSpec((hd,), role="scale", init=("normal", 0.02))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        n = self.names
        rows = [t[n[k]] for k in ("q", "k", "v", "g", "a1")]
        self.rank = rows[-1].shape[0]
        if t[n["a2"]].shape[1] != self.rank:
            raise ValueError("the two halves of the decay projection disagree on their rank")
        self.in_width = self.a_off + self.rank
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows) else rows[0].dtype
        self.w_in = torch.cat([x.to(dt) for x in rows], dim=0).contiguous()
        self.w_o = t[n["o"]].contiguous()
        # the decay kernel reads the second half transposed, [rank, channels]
        self.w2, self.b2 = t[n["a2"]].float().t().contiguous(), t[n["a2_bias"]].float().contiguous()
        self.norm_w = t[n["norm"]].float().contiguous()
        ops.prepare_streaming(self.w_in)
        ops.prepare_streaming(self.w_o)

    def cache_need(self):
        return StateNeed((self.H, self.D, self.V), "float32")

    def step_prelude(self):
        return ScanWork()

    graph_variant_group = ("scan_work",)

    def graph_variant(self, batch, padded: bool):
        work = batch.preludes.get(ScanWork.name)
        return (work.num_short, work.num_chunks, work.num_chains) if work is not None else 0

    def mix(self, proj, col0, ctx: StageContext, out, out_col0, out_scale):
        b, (H, D, V) = ctx.batch, (self.H, self.D, self.V)
        if ctx.state is None:
            raise RuntimeError("gated linear attention was given no state")
        offs = (col0 + self.q_off, col0 + self.k_off, col0 + self.v_off, col0 + self.g_off)
        if b.max_q_len == 1:
            # a decode step: the states stream through once, and the kernel makes the decays itself
            ops.gla_step(proj, offs, None, self.norm_w, self.eps, D ** -0.5, out_scale, out, out_col0, ctx.state,
                         b.entry_slot, b.entry_q_start, b.num_entries, H, D, V,
                         decay=(col0 + self.a_off, self.rank, self.w2, self.b2, self.tau))
            return
        alpha = ops.gla_decay(proj, col0 + self.a_off, self.rank, self.w2, self.b2, self.tau)
        common = (proj, offs, alpha, self.norm_w, self.eps, D ** -0.5, out_scale, out, out_col0, ctx.state, b.entry_slot,
                  b.entry_q_start, b.entry_q_len)
        work = b.preludes.get(ScanWork.name)
        if work is None:                                     # no work lists: every entry in one pass
            ops.gla_scan(*common, None, b.num_entries, ops.GLA_FULL, None, None, H, D, V)
            return
        if work.num_short:
            ops.gla_scan(*common, work.short, work.num_short, ops.GLA_FULL, None, None, H, D, V)
        if work.num_chunks:
            scratch_s = torch.empty((work.num_chunks, H, D, V), dtype=torch.float32, device=proj.device)
            scratch_a = torch.empty((work.num_chunks, H, D), dtype=torch.float32, device=proj.device)
            ops.gla_scan(*common, work.chunks, work.num_chunks, ops.GLA_LOCAL, scratch_s, scratch_a, H, D, V)
            ops.gla_chain(ctx.state, scratch_s, scratch_a, work.chains, work.num_chains, b.entry_slot, H, D, V)
            ops.gla_scan(*common, work.chunks, work.num_chunks, ops.GLA_OUT, scratch_s, scratch_a, H, D, V)


class _HeadDecayRecurrence(BranchMixer):
    """What the recurrences with ONE decay number per (token, head) share: a state per head that the
    recurrence kernels of gated linear attention walk (S [D, V], optionally a normaliser n [D] beside it),
    the step's `ScanWork` (short entries in one pass, long portions as chunks that run side by side and a
    chain over them), a kernel of their own for decode steps.  A subclass says what its projection holds
    (`_pieces`), what the scan reads (`_scan_inputs`) and how a decode step is launched (`_step`)."""

    graph_safe = True
    any_division_safe = False
    graph_variant_group = ("scan_work",)
    normaliser = False
    gate = "silu"

    def _setup(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device, names, extra_state: int):
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        if self.H <= 0 or self.D <= 0 or self.V <= 0:
            raise ValueError("a recurrent mixer needs positive heads, key width and value width")
        self.spec, self.hidden, self.dtype, self.device = spec, hidden_size, compute_dtype, torch.device(device)
        self.eps = float(dict(spec.params).get("eps", 1e-6))          # of the per-head output norm
        self.names = dict(names, **dict(spec.tensor_names))
        hd, hv = self.H * self.D, self.H * self.V
        self.q_off, self.k_off, self.v_off, self.g_off = 0, hd, 2 * hd, 2 * hd + hv
        self.in_width = 2 * hd + 2 * hv
        self.out_width = hv
        self.columns = self.V + (1 if self.normaliser else 0)          # of a head's state that the kernels walk
        self.head_floats = self.D * self.columns + extra_state
        if self.device.type == "cuda" and not ops.gla_supported(self.D, self.columns):
            raise ValueError(f"a state of {self.D} x {self.columns} per head is more than the recurrence kernel keeps "
                             "in one block's registers")

    def cache_need(self):
        return StateNeed((self.H, self.head_floats), "float32")

    def step_prelude(self):
        return ScanWork()

    def graph_variant(self, batch, padded: bool):
        work = batch.preludes.get(ScanWork.name)
        return (work.num_short, work.num_chunks, work.num_chains) if work is not None else 0

    def _load_in_out(self, t, keys) -> None:
        n = self.names
        rows = [t[n[k]] for k in keys]
        dt = torch.float32 if any(x.dtype == torch.float32 for x in rows) else rows[0].dtype
        self.w_in = torch.cat([x.to(dt) for x in rows], dim=0).contiguous()
        self.w_o = t[n["o"]].contiguous()
        ops.prepare_streaming(self.w_in)
        ops.prepare_streaming(self.w_o)

    def mix(self, proj, col0, ctx: StageContext, out, out_col0, out_scale):
        b, (H, D, V) = ctx.batch, (self.H, self.D, self.V)
        if ctx.state is None:
            raise RuntimeError("a recurrent mixer was given no state")
        offs = (col0 + self.q_off, col0 + self.k_off, col0 + self.v_off, col0 + self.g_off)
        if b.max_q_len == 1:                    # a decode step: the states stream through once
            self._step(proj, col0, offs, ctx, out, out_col0, out_scale)
            return
        alpha, a_tok, a_head, kscale, nfloor = self._scan_inputs(proj, col0, offs, ctx)
        norm_w, norm_stride = self._norm()
        scan = lambda items, n, mode, ss, sa: ops.recur_scan(
            proj, offs, alpha, a_tok, a_head, kscale, nfloor, norm_w, norm_stride, self.gate, self.eps, self.q_scale,
            out_scale, out, out_col0, ctx.state, self.head_floats, b.entry_slot, b.entry_q_start, b.entry_q_len, items, n,
            mode, ss, sa, H, D, V)
        work = b.preludes.get(ScanWork.name)
        if work is None:                        # no work lists: every entry in one pass
            scan(None, b.num_entries, ops.GLA_FULL, None, None)
            return
        if work.num_short:
            scan(work.short, work.num_short, ops.GLA_FULL, None, None)
        if work.num_chunks:
            scratch_s = torch.empty((work.num_chunks, H, D * self.columns), dtype=torch.float32, device=proj.device)
            scratch_a = torch.empty((work.num_chunks, H, D), dtype=torch.float32, device=proj.device)
            scan(work.chunks, work.num_chunks, ops.GLA_LOCAL, scratch_s, scratch_a)
            ops.recur_chain(ctx.state, self.head_floats, scratch_s, scratch_a, work.chains, work.num_chains, b.entry_slot,
                            H, D, V, self.normaliser)
            scan(work.chunks, work.num_chunks, ops.GLA_OUT, scratch_s, scratch_a)


@register_mixer("retention")
class RetentionMixer(_HeadDecayRecurrence):
    """Linear attention with one FIXED decay per head and no denominator.  Per head a state S [D, V] (32-bit, one
    per request and stage, zero at admission):

        S_t = decay_h S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t

    with q = W_q x and k = W_k x rotated by the mixer's position part (a half-split rotation of the first
    rotary_dim entries of each head), k times D^-1/2 (applied to the finished sums o, which are linear in k),
    v = W_v x.  Each head's o is divided by its root mean square (no weight), multiplied by silu(W_g x), and the
    concatenated heads go through W_o.  One product yields [q | k | v | g] per token in float32.  Prompt
    portions: a rotation kernel, then the recurrence kernels; decode steps: one kernel that rotates too."""

    _DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight"}

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        self._setup(spec, hidden_size, compute_dtype, device, self._DEFAULT_NAMES, 0)
        decay = dict(spec.params).get("decay")
        if decay is None or len(decay) != self.H or any(not 0.0 <= float(x) <= 1.0 for x in decay):
            raise ValueError("retention needs one decay in [0, 1] per head")
        self.decay = torch.tensor([float(x) for x in decay], dtype=torch.float32, device=self.device)
        self.q_scale = self.D ** -0.5
        self.rot = None
        if spec.position.kind != "none":
            from .registry import lookup
            part = lookup("position", spec.position.kind)(spec.position, self.D, device)
            if not hasattr(part, "inv_freq") or not hasattr(part, "rotary_dim"):
                raise ValueError("retention rotates q and k: its position part must be a rotation")
            self.rot = (part.inv_freq, part.rotary_dim)

    def parameters(self) -> Dict[str, ParamSpec]:
        n, hd, hv = self.names, self.H * self.D, self.H * self.V
        return {n["q"]: ParamSpec((hd, self.hidden)), n["k"]: ParamSpec((hd, self.hidden)),
                n["v"]: ParamSpec((hv, self.hidden)), n["g"]: ParamSpec((hv, self.hidden)),
                n["o"]: ParamSpec((self.hidden, hv))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self._load_in_out(t, ("q", "k", "v", "g"))

    def _norm(self):
        return None, 0

    def _scan_inputs(self, proj, col0, offs, ctx):
        if self.rot is not None:
            ops.rotate_qk(proj, offs[0], offs[1], self.H, self.H, self.D, self.rot[1], self.rot[0], ctx.batch.positions)
        return self.decay, 0, 1, None, None

    def _step(self, proj, col0, offs, ctx, out, out_col0, out_scale):
        b = ctx.batch
        rotation = (self.rot[0], self.rot[1], b.positions) if self.rot is not None else None
        ops.recur_step(proj, offs, self.decay, (0, 1, 0), None, 0, self.gate, self.eps, self.q_scale, out_scale, out,
                       out_col0, ctx.state, self.head_floats, b.entry_slot, b.entry_q_start, b.num_entries, self.H,
                       self.D, self.V, rotation=rotation)


@register_mixer("mlstm")
class MatrixMemoryMixer(_HeadDecayRecurrence):
    """A matrix memory with exponential gating (mLSTM).  Per head S [D, V], a normaliser n [D] and a running
    maximum m (all 32-bit, zero at admission; m starts at 0):

        i = cap tanh((W_i x + b_i) / cap),  f = logsigmoid(cap tanh((W_f x + b_f) / cap))     (log gates, per head)
        m' = max(f + m, i),  S' = exp(f + m - m') S + exp(i - m') k v^T,  n' likewise with k alone
        o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

    with q = W_q x D^-1/2 (applied to the finished sums), k = W_k x, v = W_v x.  Each head's o is divided by its
    root mean square, the concatenated heads are multiplied by a weight over all heads and by sigmoid(W_g x), then
    W_o.  One product yields [q | k | v | g | i | f] per token in float32.  Prompt portions: a kernel walks each
    entry's gates in order (the maxima are a scalar chain) and leaves exp(f + m - m'), exp(i - m'), exp(-m') per
    (token, head); with those the recurrence is linear and runs in the kernels of gated linear attention, the
    normaliser as one more column of the state.  Decode steps: one kernel that makes the gates itself."""

    normaliser = True
    gate = "sigmoid"

    _DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight", "norm": "o_norm.weight", "i": "i_proj.weight", "i_bias": "i_proj.bias",
                      "f": "f_proj.weight", "f_bias": "f_proj.bias"}

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        self._setup(spec, hidden_size, compute_dtype, device, self._DEFAULT_NAMES, 1)     # + the running maximum
        self.cap = float(dict(spec.params).get("gate_cap", 15.0))
        if not self.cap > 0:
            raise ValueError("gate_cap must be positive")
        self.q_scale = self.D ** -0.5
        self.i_off = self.in_width
        self.f_off = self.in_width + self.H
        self.in_width += 2 * self.H
        self.m_off = self.D * self.columns
        self.i_bias = self.f_bias = self.norm_w = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, hd, hv = self.names, self.H * self.D, self.H * self.V
        return {n["q"]: ParamSpec((hd, self.hidden)), n["k"]: ParamSpec((hd, self.hidden)),
                n["v"]: ParamSpec((hv, self.hidden)), n["g"]: ParamSpec((hv, self.hidden)),
                n["o"]: ParamSpec((self.hidden, hv)),
                n["norm"]: ParamSpec((hv,), role="scale", init=("one_plus_normal", 0.01)),
                n["i"]: ParamSpec((self.H, self.hidden)), n["f"]: ParamSpec((self.H, self.hidden)),
                n["i_bias"]: ParamSpec((self.H,), role="scale", init=("normal", 0.5)),
                n["f_bias"]: ParamSpec((self.H,), role="scale", init=("one_plus_normal", 0.5))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self._load_in_out(t, ("q", "k", "v", "g", "i", "f"))
        self.i_bias, self.f_bias = t[n["i_bias"]].float().contiguous(), t[n["f_bias"]].float().contiguous()
        self.norm_w = t[n["norm"]].float().contiguous()

    def _norm(self):
        return self.norm_w, self.V

    def _scan_inputs(self, proj, col0, offs, ctx):
        b = ctx.batch
        gates = ops.recur_gates(proj, col0 + self.i_off, col0 + self.f_off, self.i_bias, self.f_bias, self.cap, ctx.state,
                                self.m_off, self.head_floats, b.entry_slot, b.entry_q_start, b.entry_q_len,
                                b.num_entries, self.H)
        return gates[0], self.H, 1, gates[1], gates[2]

    def _step(self, proj, col0, offs, ctx, out, out_col0, out_scale):
        b = ctx.batch
        ops.recur_step(proj, offs, None, None, self.norm_w, self.V, self.gate, self.eps, self.q_scale, out_scale, out,
                       out_col0, ctx.state, self.head_floats, b.entry_slot, b.entry_q_start, b.num_entries, self.H,
                       self.D, self.V, gates=(col0 + self.i_off, col0 + self.f_off, self.i_bias, self.f_bias, self.cap))
