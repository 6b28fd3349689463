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
