"""Small Gubidra configurations for the tests, and random weights for them.

The configurations differ from one another in every size and option: widths that are no powers of two,
one, two and four residual streams and none at all, a looped span of layers and none, grouped and
ungrouped query heads, key and value widths that differ, windows of a few keys (shorter than a page, and
longer than several), an attention layer without a window, rotations over a part of a head and over all
of it and none, decays of 1 (never forgets) and 0 (forgets at once), expert groups of one expert, of
several, and none, a layer without a feed-forward.  Weights are drawn so that activations are of order one
and a lost key, a lost state or a wrong constant moves the logits by far more than rounding.  This file
does not import the engine.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch


def _attn(heads, kv, dim, vdim, window, scale, far, rows):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far, "bias_rows": rows}
    if window:
        m["mask"] = {"size": window}
    return m


def _ret(heads, dim, vdim, decay, rot_dims=0, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return m


def _mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _moe(experts, top, ff, limit, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _config(vocab, width, eps, scale, layers, streams=None, loop=None):
    d = {"architecture": "Gubidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if streams is not None:
        d["streams"] = streams
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# A: two streams, layers 1..2 run twice, a window shorter than a page, partial rotation, a layer without feed-forward
GUBI_A = _config(101, 40, 1e-5, 3.5, [
    _layer("attention", _attn(4, 2, 16, 24, 9, 0.3, 40, 8), _moe(6, 2, 20, 1.2, 2.0, (3, 2))),
    _layer("retention", _ret(3, 8, 16, (0.9, 0.97, 1.0), rot_dims=4, base=500.0), _moe(4, 1, 24, 0.8, 1.0)),
    _layer("mlstm", _mlstm(2, 16, 8, 6.0), None),
    _layer("retention", _ret(2, 16, 8, (0.0, 0.8)), _moe(6, 3, 12, 2.0, 0.7, (6, 4))),
], streams=2, loop=(1, 3, 2))
GUBI_A_PAGE = 16

# B: one plain residual stream, no loop, ungrouped heads, an attention layer without a window, key width == value width
GUBI_B = _config(131, 48, 3e-6, 1.0, [
    _layer("mlstm", _mlstm(3, 8, 24, 15.0), _moe(5, 2, 16, 1.5, 1.5)),
    _layer("attention", _attn(3, 3, 32, 32, 0, 0.2, 100, 12), _moe(8, 2, 16, 1.0, 2.5, (2, 1))),
    _layer("attention", _attn(2, 1, 8, 16, 21, 0.5, 16, 6), None),
    _layer("retention", _ret(2, 24, 40, (0.95, 0.99), rot_dims=24, base=1.0e6), _moe(5, 5, 8, 3.0, 1.0)),
])
GUBI_B_PAGE = 4

# C: four streams, the whole model looped, head size 64, a window over several pages, longer sequences
GUBI_C = _config(211, 64, 1e-5, 8.0, [
    _layer("retention", _ret(2, 32, 64, (0.984, 0.9995), rot_dims=32, base=10000.0), _moe(8, 2, 32, 1.5, 1.5, (4, 2))),
    _layer("attention", _attn(4, 2, 64, 64, 130, 0.125, 200, 16), _moe(8, 2, 32, 1.5, 1.5, (4, 2))),
    _layer("mlstm", _mlstm(2, 32, 64, 10.0), _moe(4, 2, 48, 1.0, 1.0)),
], streams=4, loop=(0, 3, 2))
GUBI_C_PAGE = 16

# D: one stream WITH connections (streams = 1), a loop of one layer three times, odd sizes throughout
GUBI_D = _config(89, 36, 1e-6, 0.5, [
    _layer("mlstm", _mlstm(1, 12, 20, 3.0), _moe(3, 1, 10, 1.0, 1.0, (3, 1))),
    _layer("attention", _attn(6, 3, 4, 12, 5, 1.0, 9, 4), _moe(4, 2, 6, 0.5, 3.0)),
], streams=1, loop=(0, 1, 3))
GUBI_D_PAGE = 8


def run_order(cfg) -> list:
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, written out from the design's naming rules."""
    W, S = cfg["width"], cfg.get("streams")
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, e in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", e["mixer"]
        out[f"l{i}.norm1"] = (W,)
        if e["type"] == "attention":
            out.update({f"{p}.q": (m["heads"] * m["dim"], W), f"{p}.k": (m["kv_heads"] * m["dim"], W),
                        f"{p}.v": (m["kv_heads"] * m["vdim"], W), f"{p}.g": (m["heads"], W),
                        f"{p}.o": (W, m["heads"] * m["vdim"]), f"{p}.rel": (m["bias_rows"], m["heads"])})
        else:
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({f"{p}.q": (hd, W), f"{p}.k": (hd, W), f"{p}.v": (hv, W), f"{p}.g": (hv, W), f"{p}.o": (W, hv)})
            if e["type"] == "mlstm":
                out.update({f"{p}.norm": (hv,), f"{p}.i": (m["heads"], W), f"{p}.i.b": (m["heads"],),
                            f"{p}.f": (m["heads"], W), f"{p}.f.b": (m["heads"],)})
        if S:
            out.update({f"l{i}.hc1.in": (S,), f"l{i}.hc1.out": (S,), f"l{i}.hc1.mix": (S, S)})
        if e.get("mlp"):
            ff, E = e["mlp"]["expert"]["ff"], e["mlp"]["router"]["experts"]
            out[f"l{i}.norm2"] = (W,)
            out[f"l{i}.mlp.router"] = (E, W)
            for x in range(E):
                out.update({f"l{i}.mlp.e{x}.gate": (ff, W), f"l{i}.mlp.e{x}.up": (ff, W), f"l{i}.mlp.e{x}.down": (W, ff)})
            if S:
                out.update({f"l{i}.hc2.in": (S,), f"l{i}.hc2.out": (S,), f"l{i}.hc2.mix": (S, S)})
    return out


def random_weights(cfg: dict, seed: int, sharp: float = 2.5) -> Dict[str, torch.Tensor]:
    """float32 tensors whose values are exactly representable in bfloat16 (so a bfloat16 run and a float32
    run hold the same model).  Matrices N(0, 1/fan_in), the query matrices of attention times `sharp` so
    that softmax is peaked and single keys matter; the distance table N(0, 1); gate biases N(0, 1) (the
    forget gate's + 2); norm weights 1 + N(0, 0.1); the streams' mixing matrices near a rotation of the
    identity, their input and output weights around 1 / streams and 1; router rows N(0, 4 / fan_in) so
    that scores spread between 0 and 1; the experts' down matrices a quarter of that, so that a 16-bit run's
    other choice on a close call between two experts stays a small step."""
    rng = np.random.RandomState(seed)
    S = cfg.get("streams") or 1
    kinds = {i: e["type"] for i, e in enumerate(cfg["layers"])}
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        layer = int(name[1:name.index(".")]) if name[0] == "l" and name[1].isdigit() else -1
        if name.endswith(".rel"):
            t = rng.normal(0.0, 1.0, shape)
        elif name.endswith(".f.b"):
            t = rng.normal(2.0, 1.0, shape)
        elif name.endswith(".i.b"):
            t = rng.normal(0.0, 1.0, shape)
        elif ".hc" in name and name.endswith(".mix"):
            t = np.eye(S) * 0.8 + rng.normal(0.0, 0.25, shape)
        elif ".hc" in name and name.endswith(".in"):
            t = 1.0 / S + rng.normal(0.0, 0.2, shape)
        elif ".hc" in name and name.endswith(".out"):
            t = 1.0 + rng.normal(0.0, 0.3, shape)
        elif name.endswith(".router"):
            t = rng.normal(0.0, 2.0 * shape[1] ** -0.5, shape)
        elif len(shape) == 1:
            t = 1.0 + rng.normal(0.0, 0.1, shape)
        elif name == "embed":
            t = rng.normal(0.0, 1.0, shape)
        else:
            t = rng.normal(0.0, shape[1] ** -0.5, shape)
            if name.endswith(".mix.q") and kinds.get(layer) == "attention":
                t = t * sharp
            if name.endswith(".down"):            # a close call between two experts then moves the stream by little
                t = t * 0.25
        w[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16).to(torch.float32)
    return w


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()
