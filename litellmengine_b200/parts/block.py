"""A layer put together from its parts, and the arrangements that wire them."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..config.specs import BlockSpec
from ..weights.loader import ParamSpec
from .context import StageContext
from .registry import lookup, register_arrangement


class Block:
    """Holds one layer's mixer, feed-forward and norms, each chosen by the layer's spec."""

    def __init__(self, spec: BlockSpec, hidden_size: int, compute_dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = compute_dtype
        self.mixer_norm = lookup("norm", spec.mixer_norm.kind)(spec.mixer_norm, hidden_size)
        self.feed_forward_norm = lookup("norm", spec.feed_forward_norm.kind)(spec.feed_forward_norm, hidden_size)
        self.mixer = lookup("mixer", spec.mixer.kind)(spec.mixer, hidden_size, compute_dtype, device)
        # a layer may be its mixer only: then it has no feed-forward and no norm for one
        self.feed_forward = None
        if spec.feed_forward is not None:
            self.feed_forward = lookup("feed_forward", spec.feed_forward.kind)(
                spec.feed_forward, hidden_size, compute_dtype, device)
        else:
            self.feed_forward_norm = None
        self.arrangement = lookup("arrangement", spec.arrangement)

    def _children(self):
        s = self.spec
        out = [(s.mixer_norm_name, self.mixer_norm), (s.mixer.weight_prefix, self.mixer)]
        if self.feed_forward is not None:
            out += [(s.feed_forward_norm_name, self.feed_forward_norm), (s.feed_forward.weight_prefix, self.feed_forward)]
        return out

    def parts(self):
        """The parts that may offer a prelude, a graph variant or weights to count."""
        return [p for p in (self.mixer, self.feed_forward) if p is not None]

    def parameters(self) -> Dict[str, ParamSpec]:
        out = {}
        for prefix, part in self._children():
            for name, p in part.parameters().items():
                out[f"{prefix}.{name}" if name else prefix] = p      # '' : the tensor is named like the part
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            mine = {n[len(prefix) + 1:]: t for n, t in tensors.items() if n.startswith(prefix + ".")}
            if prefix in tensors and "" in part.parameters():
                mine[""] = tensors[prefix]
            part.load({n: t for n, t in mine.items() if n in part.parameters()})

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        return self.arrangement(self, h, delta, ctx)


@register_arrangement("pre_norm")
def pre_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (src/model/qwen3.cpp:948-968).

    `h` is the float32 residual stream; `delta` is the previous layer's feed-forward output
    that has not been added yet (None if nothing is pending).  Each add is fused into the norm
    that follows it, so the layer returns its own feed-forward output as the next pending delta,
    unless the part added it to `h` itself (in the epilogue of its last product).
    """
    from ..csrc import ops
    if not getattr(block.mixer_norm, "accepts_partials", False):
        delta = ops.as_tensor(delta)
    x = block.mixer_norm.forward(h, block.dtype, delta=delta, write_sum=delta is not None)
    ctx.partials_ok = getattr(block.feed_forward_norm, "accepts_partials", False)
    ctx.residual = h                                            # a part may add its result here itself and return None
    a = block.mixer.forward(x, ctx)
    y = block.feed_forward_norm.forward(h, block.dtype, delta=a, write_sum=a is not None)
    extra = {}
    if getattr(block.feed_forward, "supports_partials", False):
        extra["partials_ok"] = True                             # the next norm (or `pre_norm` above) adds the splits
    if getattr(block.feed_forward, "supports_residual", False):
        extra["residual"] = h
    f = block.feed_forward.forward(y, **extra)
    return h, f


@register_arrangement("branch_norm")
def branch_norm(block: Block, h: torch.Tensor, delta: Optional[torch.Tensor], ctx: StageContext):
    """h += norm1(mixer(h)); h += norm2(ffn(h)): the norms sit on the sublayers' outputs and the
    sublayers read the stream itself.

    `h` is the float32 residual stream and is complete on entry and on return (nothing is pending, so
    `delta` passes through as None).  A sublayer's products want their input in the compute dtype: the
    kernel that adds a normed output to the stream also writes the new stream in that dtype, and hands
    it to the next sublayer, across layers too, through `batch.tables["stream_copy"]` (a pair of the
    stream it is a copy of and the copy); the first layer of a model finds there what the embedding
    kernel wrote.  In the float32 mode the stream is its own copy.
    """
    from ..csrc import ops
    if delta is not None:
        ops.residual_add(h, ops.as_tensor(delta))
    tables = ctx.batch.tables
    narrow = None if block.dtype == torch.float32 else block.dtype
    held = tables.pop("stream_copy", None)
    if narrow is None:
        x = h
    elif held is not None and held[0] is h:
        x = held[1]
    else:
        x = h.to(narrow)
    ctx.partials_ok = True                                      # the norm kernel adds a product's k-splits as it reads
    ctx.residual = None                                         # the norm stands between the product and the stream
    a = block.mixer.forward(x, ctx)
    x = block.mixer_norm.add_normed(h, a, narrow)
    if block.feed_forward is not None:
        extra = {"partials_ok": True} if getattr(block.feed_forward, "supports_partials", False) else {}
        f = block.feed_forward.forward(x if narrow is not None else h, **extra)
        x = block.feed_forward_norm.add_normed(h, f, narrow)
    if narrow is not None:
        tables["stream_copy"] = (h, x)
    return h, None
