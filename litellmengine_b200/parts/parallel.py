"""A mixer made of mixers: several branches read the same input side by side and their results are
added with fixed weights."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.specs import MixerSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .context import StageContext
from .registry import lookup, register_mixer


@register_mixer("parallel")
class ParallelMixer:
    """result = sum_i scale_i * branch_i(x) for the branches of `spec.branches` (any registered mixers that
    are `BranchMixer`s), whose tensors live under the mixer's prefix plus each branch's own.

    Every branch ends in an output projection, so the weighted sum is ONE product: the branches write
    their pre-projection activations, each already times its scale (in 32-bit, before the rounding to the
    compute dtype), into column ranges of one buffer, and the output matrices stand side by side along
    the input axis.  Likewise every branch begins with projections of the same x: their matrices are
    stacked into one and each branch reads its columns of the one float32 result.  A stage that runs
    this mixer keeps whatever its branches keep: pages for one, a state for another."""

    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        if len(spec.branches) < 2 or len(spec.branch_scales) != len(spec.branches):
            raise ValueError("a parallel mixer needs at least two branches and one scale for each")
        self.spec, self.hidden, self.dtype = spec, hidden_size, compute_dtype
        self.branches = [lookup("mixer", b.kind)(b, hidden_size, compute_dtype, device) for b in spec.branches]
        for b in self.branches:
            if not hasattr(b, "mix"):
                raise ValueError(f"a {type(b).__name__} cannot stand beside other mixers (it offers no `mix`)")
        self.scales = [float(x) for x in spec.branch_scales]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        self.any_division_safe = all(getattr(b, "any_division_safe", False) for b in self.branches)
        self.w_in = self.w_o = None
        self.in_cols: List[int] = []
        self.out_cols: List[int] = []

    def _prefixed(self):
        return [(b_spec.weight_prefix, b) for b_spec, b in zip(self.spec.branches, self.branches)]

    def parameters(self) -> Dict[str, ParamSpec]:
        return {f"{prefix}.{name}": p for prefix, b in self._prefixed() for name, p in b.parameters().items()}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        for prefix, b in self._prefixed():
            b.load({n[len(prefix) + 1:]: x for n, x in t.items() if n.startswith(prefix + ".")})
        ins, outs = [b.w_in for b in self.branches], [b.w_o for b in self.branches]
        dt = torch.float32 if any(x.dtype == torch.float32 for x in ins + outs) else ins[0].dtype
        self.w_in = torch.cat([x.to(dt) for x in ins], dim=0).contiguous()
        self.w_o = torch.cat([x.to(dt) for x in outs], dim=1).contiguous()
        self.in_cols = [sum(b.in_width for b in self.branches[:i]) for i in range(len(self.branches))]
        self.out_cols = [sum(b.out_width for b in self.branches[:i]) for i in range(len(self.branches))]
        for b in self.branches:
            b.fused_by_parent()
        ops.prepare_streaming(self.w_in)
        ops.prepare_streaming(self.w_o)

    def cache_need(self):
        needs = [b.cache_need() for b in self.branches]
        return [n for n in needs if n is not None]

    def step_prelude(self):
        made = []
        for b in self.branches:
            make = getattr(b, "step_prelude", None)
            one = make() if make is not None else None
            if one is not None:
                made += list(one) if isinstance(one, (list, tuple)) else [one]
        return made

    def graph_variant(self, batch, padded: bool):
        return tuple(b.graph_variant(batch, padded) for b in self.branches if hasattr(b, "graph_variant"))

    def forward(self, x: torch.Tensor, ctx: StageContext):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        out = torch.empty((x.shape[0], self.w_o.shape[1]), dtype=self.dtype, device=x.device)
        for b, scale, c_in, c_out in zip(self.branches, self.scales, self.in_cols, self.out_cols):
            b.mix(proj, c_in, ctx, out, c_out, scale)
        return ops.linear(out, self.w_o, out_dtype=torch.float32, partials_ok=getattr(ctx, "partials_ok", False))
