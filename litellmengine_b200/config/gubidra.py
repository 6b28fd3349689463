"""Typed configuration of the Gubidra design, read from its config.json.

The file names the design with `"architecture": "Gubidra"` and gives `vocab`, `width`, `norm.eps`,
`embedding.scale`, optionally `streams` (copies of the residual stream joined by learned connections),
optionally `loop` ({"start", "stop", "times"}: layers start .. stop-1 run `times` times in a row with the
same tensors, each pass with a cache and state of its own), and a list `layers`.  A layer entry has `type`
('attention', 'mlstm' or 'retention'), the sizes and constants of its mixer under `mixer`, and its
feed-forward under `mlp` ({"kind": "moe", "expert": {...}, "router": {...}}, or null for a layer without
one).  Tensors of layer i start with `l<i>.`; linear weights are [out, in].

What the design fixes, and therefore lives here and in the parts rather than in the file:
  * the token's embedding row is multiplied by `embedding.scale`; there is no position vector;
  * norms are layer norms with a weight and no bias, in front of each sublayer; a final norm precedes the
    output head, which is a tensor of its own;
  * 'attention' = grouped-query softmax attention without rotation: scores times `scale` plus a learned
    bias by distance (a table `rel` [rows, heads]; distances below rows/2 have a row each, larger ones
    share rows in logarithmic steps up to `bias_max`), a sliding window of `mask.size` keys, one sigmoid
    output gate per head;
  * 'mlstm' = a matrix memory per head with exponential gating: log gates capped by `gate_cap`, a running
    maximum that starts at 0, a normaliser with the floor exp(-maximum), then a per-head RMS norm, a weight
    over all heads, a sigmoid gate;
  * 'retention' = linear attention with the fixed per-head decays of `decay`, a half-split rotation
    (`rot.base`, `rot.dims`) on q and k, keys times dim^-1/2, a weightless per-head RMS norm, a silu gate;
  * the feed-forward is a mixture of experts: sigmoid scores, experts in `groups.count` groups of
    neighbours of which the best `groups.keep` (by the sum of their two largest scores) may be chosen
    from, the `top` largest scores normalised to sum one and multiplied by `router.scale`; an expert is
    down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate x, limit), u = clamp(up x, -limit, limit).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .registry import ConfigError, register_architecture
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec, PositionSpec, StageSpec
from .tobovik import _freeze, _need, _thaw

MAX_POSITION = 1 << 20        # nothing of the design is tabulated by absolute position

_ATTN_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("rel", "rel"))
_RET_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"))
_MLSTM_NAMES = _RET_NAMES + (("norm", "norm"), ("i", "i"), ("i_bias", "i.b"), ("f", "f"), ("f_bias", "f.b"))


def _attention_spec(m: Dict[str, Any], where: str) -> MixerSpec:
    heads, kv = _need(m, "heads", int, where), _need(m, "kv_heads", int, where)
    if heads % kv:
        raise ConfigError(f"config field {where}heads must be a multiple of {where}kv_heads")
    window = None
    if m.get("mask") is not None:
        window = _need(m["mask"], "size", int, where + "mask.")
    far = _need(m, "bias_max", float, where)
    rows = m.get("bias_rows")                     # optional: only the stored table knows it otherwise
    if rows is not None and (isinstance(rows, bool) or not isinstance(rows, int) or rows < 2):
        raise ConfigError(f"config field {where}bias_rows must be an integer of at least 2 when given")
    return MixerSpec(kind="gated_attention", num_heads=heads, num_kv_heads=kv, head_dim=_need(m, "dim", int, where),
                     value_dim=_need(m, "vdim", int, where), position=PositionSpec(kind="none"), window=window,
                     scale=_need(m, "scale", float, where), output_gate="sigmoid", output_gate_scope="head",
                     distance_bias=(rows if rows is not None else -1, far), weight_prefix="mix", tensor_names=_ATTN_NAMES)


def _retention_spec(m: Dict[str, Any], where: str, eps: float) -> MixerSpec:
    heads, dim = _need(m, "heads", int, where), _need(m, "dim", int, where)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or any(
            isinstance(x, bool) or not isinstance(x, (int, float)) or not 0.0 <= x <= 1.0 for x in decay):
        raise ConfigError(f"config field {where}decay must list one number in [0, 1] per head")
    position = PositionSpec(kind="none")
    if m.get("rot") is not None:
        dims = _need(m["rot"], "dims", int, where + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config field {where}rot.dims must be even and at most {where}dim")
        position = PositionSpec(kind="rope", theta=_need(m["rot"], "base", float, where + "rot."), rotary_dim=dims)
    return MixerSpec(kind="retention", num_heads=heads, head_dim=dim, value_dim=_need(m, "vdim", int, where),
                     position=position, weight_prefix="mix", tensor_names=_RET_NAMES,
                     params=(("decay", tuple(float(x) for x in decay)), ("eps", eps)))


def _mlstm_spec(m: Dict[str, Any], where: str, eps: float) -> MixerSpec:
    cap = _need(m, "gate_cap", float, where)
    if not cap > 0:
        raise ConfigError(f"config field {where}gate_cap must be positive")
    return MixerSpec(kind="mlstm", num_heads=_need(m, "heads", int, where), head_dim=_need(m, "dim", int, where),
                     value_dim=_need(m, "vdim", int, where), weight_prefix="mix", tensor_names=_MLSTM_NAMES,
                     params=(("gate_cap", cap), ("eps", eps)))


def _moe_spec(mlp: Dict[str, Any], where: str) -> FeedForwardSpec:
    kind = _need(mlp, "kind", str, where)
    if kind != "moe":
        raise ConfigError(f"{where}kind={kind!r} is not built (only 'moe')")
    ex, ro = mlp.get("expert"), mlp.get("router")
    experts, top = _need(ro, "experts", int, where + "router."), _need(ro, "top", int, where + "router.")
    if top > experts:
        raise ConfigError(f"config field {where}router.top exceeds {where}router.experts")
    groups = None
    if ro.get("groups") is not None:
        count = _need(ro["groups"], "count", int, where + "router.groups.")
        keep = _need(ro["groups"], "keep", int, where + "router.groups.")
        if experts % count or keep > count or keep * (experts // count) < top:
            raise ConfigError(f"{where}router.groups: {count} groups of which {keep} are kept do not fit {experts} "
                              f"experts of which {top} are chosen")
        groups = (count, keep)
    limit = _need(ex, "limit", float, where + "expert.")
    if not limit > 0:
        raise ConfigError(f"config field {where}expert.limit must be positive")
    return FeedForwardSpec(kind="moe", intermediate_size=_need(ex, "ff", int, where + "expert."), weight_prefix="mlp",
                           params=(("experts", experts), ("top", top), ("groups", groups),
                                   ("route_scale", _need(ro, "scale", float, where + "router.")), ("limit", limit),
                                   ("expert_prefix", "e")))


@register_architecture("Gubidra")
@dataclass(frozen=True)
class GubidraConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    streams: int                      # 0: one residual stream, plainly added to
    loop: Tuple[int, int, int]        # (start, stop, times); (0, 0, 1) when the file has none
    layers: Tuple[Any, ...]           # the file's layer entries, kept as read (nested tuples of pairs)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GubidraConfig":
        vocab, width = _need(d, "vocab", int, ""), _need(d, "width", int, "")
        eps = _need(d.get("norm"), "eps", float, "norm.")
        if not eps > 0:
            raise ConfigError("config field norm.eps must be positive")
        scale = 1.0 if d.get("embedding") is None else _need(d["embedding"], "scale", float, "embedding.")
        streams = 0 if d.get("streams") is None else _need(d, "streams", int, "")
        if streams > 8:
            raise ConfigError("config field streams: at most 8 streams are built")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Missing required config field: layers")
        loop = (0, 0, 1)
        if d.get("loop") is not None:
            lp = d["loop"]
            for key in ("start", "stop"):
                if isinstance(lp.get(key), bool) or not isinstance(lp.get(key), int) or lp[key] < 0:
                    raise ConfigError(f"config field loop.{key} must be a non-negative integer")
            loop = (lp["start"], lp["stop"], _need(lp, "times", int, "loop."))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError("config field loop: start <= stop <= number of layers does not hold")
        cfg = cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, streams=streams, loop=loop,
                  layers=tuple(_freeze(x) for x in layers))
        cfg.plan()                    # every other check is the plan's
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embedding_scale}, "layers": [_thaw(x) for x in self.layers]}
        if self.streams:
            d["streams"] = self.streams
        if self.loop != (0, 0, 1):
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    # what the engine's entry points ask of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def torch_dtype(self) -> str:
        return "bfloat16"

    def run_order(self) -> List[int]:
        """The layers' indices in the order they run."""
        a, b, times = self.loop
        n = len(self.layers)
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def plan(self) -> ModelPlan:
        norm = NormSpec(kind="layernorm", eps=self.eps, weight_name="")
        blocks = []
        for i, frozen in enumerate(self.layers):
            e, where = _thaw(frozen), f"layers[{i}]."
            kind, m = _need(e, "type", str, where), e.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Missing required config field: {where}mixer")
            if kind == "attention":
                mixer = _attention_spec(m, where + "mixer.")
            elif kind == "retention":
                mixer = _retention_spec(m, where + "mixer.", self.eps)
            elif kind == "mlstm":
                mixer = _mlstm_spec(m, where + "mixer.", self.eps)
            else:
                raise ConfigError(f"{where}type={kind!r} is not a mixer of this design ('attention', 'mlstm', 'retention')")
            ffn = _moe_spec(e["mlp"], where + "mlp.") if e.get("mlp") is not None else None
            blocks.append(BlockSpec(arrangement="hyper_pre_norm" if self.streams else "pre_norm", mixer=mixer,
                                    feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm, weight_prefix=f"l{i}",
                                    mixer_norm_name="norm1", feed_forward_norm_name="norm2",
                                    connections=(self.streams, "hc1", "hc2") if self.streams else None))
        plan = ModelPlan(
            hidden_size=self.width, vocab_size=self.vocab, blocks=tuple(blocks),
            order=tuple(StageSpec(block=j) for j in self.run_order()), final_norm=norm,
            tie_word_embeddings=False, max_position=MAX_POSITION, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", embedding_scale=self.embedding_scale,
            streams=self.streams)
        plan.validate()
        return plan
