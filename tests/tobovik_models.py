"""Small Tobovik configurations for the tests, and random weights for them.

The configurations differ from one another in every size and option: widths that are no powers of
two, key and value widths that differ (and one where they are equal), grouped and ungrouped query
heads, a query temperature whose step is a few tokens (so that it changes inside short prompts), decay
exponents tau of 1 and more, branch scales other than 1, a layer without a feed-forward, layers that run
another layer's tensors (an earlier one and a later one), ranks of the decay projection.
Weights are drawn so that activations are of order one and a lost key, a lost state or a wrong
constant moves the logits by far more than rounding.  This file does not import the engine.
"""
from __future__ import annotations

import copy
from typing import Dict

import numpy as np
import torch


def _left(heads, kv, dim, vdim, coef=0.4, every=4, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if every:
        m["q_temp"] = {"coef": coef, "every": every}
    return m


def _right(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _parallel(left, right, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _gla(heads, dim, vdim, tau, ff):
    return {"type": "gla", "mixer": _right(heads, dim, vdim, tau), "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _shared(layer, j):
    out = copy.deepcopy(layer)
    out["weights_of"] = j
    return out


def _config(vocab, width, eps, layers):
    return {"architecture": "Tobovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A: a gla layer first, a layer without feed-forward, a layer that runs a LATER layer's tensors
_A_PAR = _parallel(_left(4, 2, 16, 32), _right(1, 8, 16, 1.0), 1.25, 0.5, 72)
_A_GLA = _gla(3, 16, 8, 4.0, 0)
TOBO_A = _config(97, 40, 1e-5, [_A_GLA, _shared(_A_PAR, 2), _A_PAR, _shared(_A_GLA, 0)])
TOBO_A_PAGE, TOBO_A_RANK = 4, 6

# B: ungrouped heads, key width == value width, no query temperature, two different parallel layers
_B_PAR0 = _parallel(_left(3, 3, 32, 32, every=0, scale=0.3), _right(2, 24, 40, 2.0), 0.7, 1.1, 56)
_B_PAR1 = _parallel(_left(2, 1, 8, 24, coef=0.9, every=7), _right(2, 16, 16, 12.0), 1.0, 1.0, 88)
TOBO_B = _config(131, 48, 3e-6, [_B_PAR0, _B_PAR1, _gla(2, 32, 48, 8.0, 64), _shared(_B_PAR0, 0), _shared(_B_PAR1, 1)])
TOBO_B_PAGE, TOBO_B_RANK = 16, 3

# C: head size 64 with keys and values alike (a bfloat16 run takes the tuned attention kernels), longer sequences
_C_PAR = _parallel(_left(4, 2, 64, 64, coef=0.2, every=32, scale=0.09), _right(2, 32, 64, 24.0), 0.75, 0.6, 96)
TOBO_C = _config(211, 64, 1e-5, [_C_PAR, _gla(2, 16, 32, 6.0, 96), _shared(_C_PAR, 0)])
TOBO_C_PAGE, TOBO_C_RANK = 16, 8


# D: head size 128 with keys and values alike: a bfloat16 run takes the tcgen05 prompt kernel and the TMA decode kernel
_D_PAR = _parallel(_left(4, 2, 128, 128, coef=0.5, every=16, scale=0.11), _right(1, 64, 128, 4.0), 1.0, 0.6, 80)
TOBO_D = _config(157, 96, 1e-5, [_D_PAR, _shared(_D_PAR, 0)])
TOBO_D_PAGE, TOBO_D_RANK = 16, 4

# E: linear attention only: a model without pages
TOBO_E = _config(89, 32, 1e-6, [_gla(2, 16, 16, 2.0, 48), _gla(1, 32, 8, 32.0, 0), _shared(_gla(2, 16, 16, 2.0, 48), 0)])
TOBO_E_PAGE, TOBO_E_RANK = 8, 5


def num_owner_layers(cfg) -> list:
    return [i for i, e in enumerate(cfg["layers"]) if e.get("weights_of") is None]


def tensor_shapes(cfg: dict, rank: int) -> Dict[str, tuple]:
    """Names and shapes of a model's tensors, written out from the design's naming rules."""
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],),
                            "head": (cfg["vocab"], cfg["width"])}

    def gla(p, m):
        hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
        out.update({f"{p}.q": (hd, W), f"{p}.k": (hd, W), f"{p}.v": (hv, W), f"{p}.g": (hv, W), f"{p}.o": (W, hv),
                    f"{p}.norm": (m["vdim"],), f"{p}.a1": (rank, W), f"{p}.a2": (hd, rank), f"{p}.a2.b": (hd,)})

    def soft(p, m):
        hq, hk, hv, ho = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
        out.update({f"{p}.q": (hq, W), f"{p}.q.b": (hq,), f"{p}.k": (hk, W), f"{p}.k.b": (hk,), f"{p}.v": (hv, W),
                    f"{p}.v.b": (hv,), f"{p}.q.norm": (hq,), f"{p}.k.norm": (hk,), f"{p}.g": (ho, W), f"{p}.o": (W, ho)})

    for i in num_owner_layers(cfg):
        e = cfg["layers"][i]
        out[f"l{i}.norm1"] = (W,)
        if e["type"] == "parallel":
            soft(f"l{i}.mix.left", e["mixer"]["left"])
            gla(f"l{i}.mix.right", e["mixer"]["right"])
        else:
            gla(f"l{i}.mix", e["mixer"])
        if e.get("mlp"):
            ff = e["mlp"]["ff"]
            out[f"l{i}.norm2"] = (W,)
            out.update({f"l{i}.mlp.gate": (ff, W), f"l{i}.mlp.up": (ff, W), f"l{i}.mlp.down": (W, ff)})
    return out


def random_weights(cfg: dict, rank: int, seed: int, sharp: float = 3.0, decay_bias: float = 2.0) -> Dict[str, torch.Tensor]:
    """float32 tensors whose values are exactly representable in bfloat16 (so a bfloat16 run and a float32
    run hold the same model).  Matrices N(0, 1/fan_in); biases N(0, 0.3); norm weights 1 + N(0, 0.1), the
    query norm's times `sharp` so that softmax is peaked and single keys matter; the decay's bias N(0, 1)
    + `decay_bias` so that the decays spread between fast and slow."""
    rng = np.random.RandomState(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        if name.endswith(".a2.b"):
            t = rng.normal(decay_bias, 1.0, shape)
        elif name.endswith(".b"):
            t = rng.normal(0.0, 0.3, shape)
        elif name.endswith("q.norm"):
            t = sharp * (1.0 + rng.normal(0.0, 0.1, shape))
        elif len(shape) == 1:
            t = 1.0 + rng.normal(0.0, 0.1, shape)
        elif name == "embed":
            t = rng.normal(0.0, 1.0, shape)
        else:
            t = rng.normal(0.0, shape[1] ** -0.5, shape)
        w[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16).to(torch.float32)
    return w


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    return np.random.RandomState(seed).randint(0, cfg["vocab"], size=n).tolist()
