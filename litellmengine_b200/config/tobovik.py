"""Typed configuration of the Tobovik design, read from its config.json.

The file names the design with `"architecture": "Tobovik"` and gives `vocab`, `width`, `norm.eps` and a
list `layers`.  A layer entry has `type` ('parallel' or 'gla'), the sizes of its mixer under `mixer`, its
feed-forward under `mlp` ({"kind": "dense", "ff": n}, or null for a layer without one), and optionally
`weights_of: j`: the layer then has no tensors of its own and runs layer j's, with a cache and a
recurrent state of its own.  Tensors of layer i start with `l<i>.`; linear weights are [out, in].

What the design fixes, and therefore lives here and in the parts rather than in the file:
  * a sinusoidal position vector (base 10000, sine at even entries, cosine at odd ones) is added to the
    token embedding; mixers use no rotation;
  * norms are RMS norms without a one-plus weight, placed on each sublayer's OUTPUT
    (x += norm1(mixer(x)); x += norm2(ff(x))); a final norm precedes the output head, which is a tensor of
    its own;
  * 'parallel' = a softmax attention ('left': grouped query heads, biased q/k/v, RMS norm over the whole
    q and k projections, a logarithmic query temperature, a sigmoid output gate) beside a gated linear
    attention ('right'), summed with the weights `left_scale` and `right_scale`;
  * 'gla' = the gated linear attention alone: a decay per key channel alpha = sigmoid(z)^(1/tau) from a
    low-rank projection whose rank is the stored tensors' inner size, a per-head RMS norm of the output
    with one weight shared by the heads, a silu output gate;
  * the dense feed-forward is down(silu(gate x) * (up x)).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import ConfigError, register_architecture
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec, StageSpec)

SINUSOID_BASE = 10000.0
MAX_POSITION = 1 << 20        # the design has no learned or tabulated positions, so nothing caps a sequence


def _need(d: Dict[str, Any], key: str, kind, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"Missing required config field: {where}{key}")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError(f"config field {where}{key} must be a positive integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config field {where}{key} must be a number, got {v!r}")
        return float(v)
    if kind is str:
        if not isinstance(v, str):
            raise ConfigError(f"config field {where}{key} must be a string, got {v!r}")
        return v
    raise TypeError(kind)


_GLA_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("a1", "a1"), ("a2", "a2"),
              ("a2_bias", "a2.b"))
_ATTN_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
               ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))


def _gla_spec(m: Dict[str, Any], where: str, prefix: str, eps: float) -> MixerSpec:
    tau = _need(m, "tau", float, where)
    if not tau > 0:
        raise ConfigError(f"config field {where}tau must be positive")
    rank = m.get("rank")
    if rank is not None and (isinstance(rank, bool) or not isinstance(rank, int) or rank <= 0):
        raise ConfigError(f"config field {where}rank must be a positive integer when given")
    return MixerSpec(kind="gla", num_heads=_need(m, "heads", int, where), head_dim=_need(m, "dim", int, where),
                     value_dim=_need(m, "vdim", int, where), weight_prefix=prefix,
                     params=(("tau", tau), ("rank", rank), ("eps", eps)), tensor_names=_GLA_NAMES)


def _softmax_spec(m: Dict[str, Any], where: str, prefix: str, eps: float) -> MixerSpec:
    heads, kv = _need(m, "heads", int, where), _need(m, "kv_heads", int, where)
    if heads % kv:
        raise ConfigError(f"config field {where}heads must be a multiple of {where}kv_heads")
    temp = None
    if m.get("q_temp") is not None:
        t = m["q_temp"]
        temp = (_need(t, "coef", float, where + "q_temp."), _need(t, "every", int, where + "q_temp."))
    return MixerSpec(kind="gated_attention", num_heads=heads, num_kv_heads=kv, head_dim=_need(m, "dim", int, where),
                     value_dim=_need(m, "vdim", int, where), qk_norm=NormSpec("rmsnorm", eps),
                     qk_norm_scope="projection", position=PositionSpec(kind="none"),
                     scale=_need(m, "scale", float, where), bias=True, query_temperature=temp,
                     output_gate="sigmoid", weight_prefix=prefix, tensor_names=_ATTN_NAMES)


@register_architecture("Tobovik")
@dataclass(frozen=True)
class TobovikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Any, ...]           # the file's layer entries, kept as read (nested tuples of pairs)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TobovikConfig":
        vocab, width = _need(d, "vocab", int, ""), _need(d, "width", int, "")
        eps = _need(d.get("norm"), "eps", float, "norm.")
        if not eps > 0:
            raise ConfigError("config field norm.eps must be positive")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Missing required config field: layers")
        cfg = cls(vocab=vocab, width=width, eps=eps, layers=tuple(_freeze(x) for x in layers))
        cfg.plan()                    # every other check is the plan's
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": [_thaw(x) for x in self.layers]}

    # what the engine's entry points ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def torch_dtype(self) -> str:
        return "bfloat16"

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i runs (itself, unless it says `weights_of`)."""
        layers = [_thaw(x) for x in self.layers]
        seen = set()
        while layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"layers[{i}].weights_of runs in a circle")
            seen.add(i)
            j = layers[i]["weights_of"]
            if isinstance(j, bool) or not isinstance(j, int) or not 0 <= j < len(layers):
                raise ConfigError(f"layers[{i}].weights_of must name a layer, got {j!r}")
            i = j
        return i

    def plan(self) -> ModelPlan:
        norm = NormSpec(kind="rmsnorm", eps=self.eps, weight_name="")
        layers = [_thaw(x) for x in self.layers]
        owners = [self.owner_of(i) for i in range(len(layers))]
        block_of, blocks = {}, []
        for i in sorted(set(owners)):
            e, where = layers[i], f"layers[{i}]."
            kind, m = _need(e, "type", str, where), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Missing required config field: {where}mixer")
            if kind == "parallel":
                left = _softmax_spec(m.get("left"), where + "mixer.left.", "left", self.eps)
                right = _gla_spec(m.get("right"), where + "mixer.right.", "right", self.eps)
                mixer = MixerSpec(kind="parallel", branches=(left, right), weight_prefix="mix",
                                  branch_scales=(_need(m, "left_scale", float, where + "mixer."),
                                                 _need(m, "right_scale", float, where + "mixer.")))
            elif kind == "gla":
                mixer = _gla_spec(m, where + "mixer.", "mix", self.eps)
            else:
                raise ConfigError(f"{where}type={kind!r} is not a mixer of this design ('parallel', 'gla')")
            ffn = None
            if e.get("mlp") is not None:
                ff_kind = _need(e["mlp"], "kind", str, where + "mlp.")
                if ff_kind != "dense":
                    raise ConfigError(f"{where}mlp.kind={ff_kind!r} is not built (only 'dense')")
                ffn = FeedForwardSpec(kind="swiglu", intermediate_size=_need(e["mlp"], "ff", int, where + "mlp."),
                                      weight_prefix="mlp", tensor_names=_FF_NAMES)
            block_of[i] = len(blocks)
            blocks.append(BlockSpec(arrangement="branch_norm", mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm, weight_prefix=f"l{i}", mixer_norm_name="norm1",
                                    feed_forward_norm_name="norm2"))
        # a layer that says `weights_of` runs its owner's mixer, feed-forward and norms: the owner's entry counts
        plan = ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            order=tuple(StageSpec(block=block_of[j]) for j in owners), final_norm=norm,
            tie_word_embeddings=False, max_position=MAX_POSITION, embedding_name="embed",
            final_norm_name="final.norm", output_name="head",
            embedding_position=PositionSpec(kind="sinusoid_added", theta=SINUSOID_BASE))
        plan.validate()
        return plan


def _freeze(x):
    if isinstance(x, dict):
        return ("__dict__",) + tuple((k, _freeze(v)) for k, v in x.items())
    if isinstance(x, list):
        return ("__list__",) + tuple(_freeze(v) for v in x)
    return x


def _thaw(x):
    if isinstance(x, tuple) and x and x[0] == "__dict__":
        return {k: _thaw(v) for k, v in x[1:]}
    if isinstance(x, tuple) and x and x[0] == "__list__":
        return [_thaw(v) for v in x[1:]]
    return x
