"""A plain, slow restatement of the Tobovik design: whole sequences, no cache, no state carried
between calls, one function per mechanism.  It shares no code with the engine; the tests compare
the engine with it.

Notation.  h [T, W] is a sublayer's input (the residual stream itself: this design puts its norms
on the sublayers' OUTPUTS), p the position of a token in its sequence (from 0), `w` a dict of
tensors by name, `pre` a name prefix.  `act` rounds activations the way a run mode would (identity
for the 32-bit mode); everything the design keeps in 32-bit stays unrounded.
"""
import math

import torch


def identity(x):
    return x


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def sinusoid(positions, width, dtype=torch.float64):
    """[T, width]: entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos of the same angle."""
    p = positions.to(torch.float64)[:, None]
    i = torch.arange((width + 1) // 2, dtype=torch.float64)[None, :]
    ang = p * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width)
    out = torch.zeros((positions.numel(), 2 * ((width + 1) // 2)), dtype=torch.float64)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)
    return out[:, :width].to(dtype)


def embed(ids, w, width):
    ids = torch.as_tensor(ids, dtype=torch.long)
    x = w["embed"][ids].to(torch.float64)
    return x + sinusoid(torch.arange(ids.numel()), width)


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    p = positions.to(torch.int64)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(torch.float64))


def softmax_side(h, w, pre, m, eps, act=identity):
    """Grouped-query causal softmax attention with biased projections, a norm over the WHOLE q (and
    k) projection, a query temperature, no rotation, and a sigmoid output gate."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    x = act(h)
    q = x @ w[f"{pre}.q"].T + w[f"{pre}.q.b"]
    k = x @ w[f"{pre}.k"].T + w[f"{pre}.k.b"]
    v = act(x @ w[f"{pre}.v"].T + w[f"{pre}.v.b"])
    q = rms_norm(q, w[f"{pre}.q.norm"], eps)
    k = act(rms_norm(k, w[f"{pre}.k.norm"], eps))
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(torch.arange(T), qt["coef"], qt["every"])[:, None]
    q = act(q).view(T, H, D)
    k = k.view(T, G, D)
    v = v.view(T, G, V)
    out = torch.zeros((T, H, V), dtype=h.dtype)
    visible = torch.tril(torch.ones((T, T), dtype=torch.bool))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(x @ w[f"{pre}.g"].T)
    return act(act(out.reshape(T, H * V)) * gate) @ w[f"{pre}.o"].T


def gla_decay_log(x, w, pre, tau):
    """ln(alpha) = ln(sigmoid(z)) / tau with z = W_a2 (W_a1 x) + b, per key channel."""
    z = (x @ w[f"{pre}.a1"].T) @ w[f"{pre}.a2"].T + w[f"{pre}.a2.b"]
    return torch.nn.functional.logsigmoid(z) / tau


def gla_recurrence(q, k, v, log_alpha, state=None):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token.
    q, k, log_alpha [T, H, D]; v [T, H, V]; state [H, D, V] or None (zeros).  Returns (o, state)."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros((H, D, V), dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros((T, H, V), dtype=q.dtype)
    for t in range(T):
        S = torch.exp(log_alpha[t])[:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gla_side(h, w, pre, m, eps, act=identity):
    """Gated linear attention with a per-key-channel decay, a per-head output norm with one weight
    shared by the heads, and a silu gate."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    x = act(h)
    q = (x @ w[f"{pre}.q"].T) * D ** -0.5
    k = x @ w[f"{pre}.k"].T
    v = x @ w[f"{pre}.v"].T
    la = gla_decay_log(x, w, pre, m["tau"])
    o, _ = gla_recurrence(q.view(T, H, D), k.view(T, H, D), v.view(T, H, V), la.view(T, H, D))
    o = rms_norm(o, w[f"{pre}.norm"], eps).reshape(T, H * V)
    g = x @ w[f"{pre}.g"].T
    return act(o * (g * torch.sigmoid(g))) @ w[f"{pre}.o"].T


def mixer(h, w, layer, pre, eps, act=identity):
    m = layer["mixer"]
    if layer["type"] == "parallel":
        left = softmax_side(h, w, f"{pre}.mix.left", m["left"], eps, act)
        right = gla_side(h, w, f"{pre}.mix.right", m["right"], eps, act)
        return m["left_scale"] * left + m["right_scale"] * right
    if layer["type"] == "gla":
        return gla_side(h, w, f"{pre}.mix", m, eps, act)
    raise ValueError(layer["type"])


def dense_ff(h, w, pre, act=identity):
    x = act(h)
    g = x @ w[f"{pre}.gate"].T
    return act(act(g * torch.sigmoid(g)) * act(x @ w[f"{pre}.up"].T)) @ w[f"{pre}.down"].T


def forward(ids, w, cfg, act=identity, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of a whole sequence; with `return_layers` also the residual stream after
    every layer run."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = embed(ids, w, cfg["width"]).to(dtype)
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        j = i
        while cfg["layers"][j].get("weights_of") is not None:
            j = cfg["layers"][j]["weights_of"]
        pre = f"l{j}"
        x = x + rms_norm(mixer(x, w, layer, pre, eps, act), w[f"{pre}.norm1"], eps)
        if layer.get("mlp"):
            x = x + rms_norm(dense_ff(x, w, f"{pre}.mlp", act), w[f"{pre}.norm2"], eps)
        seen.append(x.clone())
    logits = act(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits


def bf16_round(x):
    return x.to(torch.bfloat16).to(x.dtype)


def bf16_round_jittered(seed):
    """Rounds to bfloat16 after a relative jitter of one bfloat16 rounding step: another computation of
    the same values in bfloat16 (another summation order, another place of rounding) differs by as much.
    Positions whose logits move a lot under it are ill conditioned in bfloat16, whoever computes them."""
    g = torch.Generator().manual_seed(seed)

    def act(x):
        u = torch.rand(x.shape, generator=g, dtype=torch.float64) * 2.0 - 1.0
        return (x * (1.0 + u * 2.0 ** -8)).to(torch.bfloat16).to(x.dtype)
    return act
