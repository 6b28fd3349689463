"""A plain, slow restatement of the Gubidra design: whole sequences, no cache, no state carried
between calls, one function per mechanism.  It shares no code with the engine; the tests compare
the engine with it.

Notation.  x [T, W] is a sublayer's (normed) input, p the position of a token in its sequence (from
0), `w` a dict of tensors by name, `pre` a name prefix, `m` a mixer's entry of the configuration.
`act` rounds activations the way a run mode would (identity for the 32-bit mode); what the design
keeps in 32-bit stays unrounded.  Everything runs in float64 unless `act` rounds it.
"""
import math

import torch

F64 = torch.float64


def identity(x):
    return x


def bf16_round(x):
    """What a 16-bit run mode does to an activation between two kernels."""
    return x.to(torch.bfloat16).to(x.dtype)


def bf16_round_jittered(seed):
    """The same rounding after a relative nudge of up to half a unit in the last place: another
    implementation's rounding of the same exact value."""
    g = torch.Generator().manual_seed(seed)

    def act(x):
        nudge = (torch.rand(x.shape, generator=g, dtype=torch.float64) - 0.5) * 2.0 ** -8
        return (x * (1.0 + nudge.to(x.dtype))).to(torch.bfloat16).to(x.dtype)
    return act


def hyper_step(xs, y, inp, out, mix):
    """One sublayer's update of the streams xs (a list of [T, W]): x_t <- sum_s mix[s, t] x_s + out[t] y."""
    S = len(xs)
    return [sum(mix[s, t] * xs[s] for s in range(S)) + out[t] * y for t in range(S)]


def hyper_input(xs, inp):
    return sum(inp[s] * xs[s] for s in range(len(xs)))


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight, var = mean of squared deviations, no bias."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d * torch.rsqrt(d.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def rms_unit(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def embed(ids, w, scale):
    return w["embed"][torch.as_tensor(ids, dtype=torch.long)].to(F64) * scale


# ---- the distance bias of the attention mixer ---------------------------------------------------
def distance_bucket(n, rows, far):
    """Row of the bias table for a distance n >= 0: exact for n < rows/2, logarithmic steps up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def attention_core(q, k, v, rel, scale, far, window, first_position=0):
    """q [T, H, D] against keys k [N, G, D] and values v [N, G, V] whose last T belong to the queries (the
    first query sits at `first_position` = N - T): scores * scale + rel[bucket(i - j), h], keys j with
    0 <= i - j < window, softmax.  Returns [T, H, V]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rows = rel.shape[0]
    row_of = [distance_bucket(n, rows, far) for n in range(first_position + T)]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        i = first_position + t
        lo = 0 if window is None else max(0, i - window + 1)
        js = list(range(lo, i + 1))
        bias = rel[[row_of[i - j] for j in js]]                     # [n, H]
        for h in range(H):
            g = h // (H // G)
            p = torch.softmax((k[js, g] @ q[t, h]) * scale + bias[:, h], dim=0)
            out[t, h] = p @ v[js, g]
    return out


def attention(x, w, pre, m, act=identity):
    """Grouped-query softmax attention: no rotation, a learned bias by distance, a window of the last
    `mask.size` keys, one sigmoid output gate per head."""
    T = x.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    xa = act(x)
    q = act(xa @ w[f"{pre}.q"].T).view(T, H, D)
    k = act(xa @ w[f"{pre}.k"].T).view(T, G, D)
    v = act(xa @ w[f"{pre}.v"].T).view(T, G, V)
    gate = torch.sigmoid(xa @ w[f"{pre}.g"].T)                    # [T, H]
    window = m["mask"]["size"] if m.get("mask") else None
    out = attention_core(q, k, v, w[f"{pre}.rel"].to(F64), m["scale"], m["bias_max"], window) * gate[:, :, None]
    return act(out.reshape(T, H * V)) @ w[f"{pre}.o"].T


# ---- mLSTM ----------------------------------------------------------------------------------------
def mlstm_core(q, k, v, ig, fg, state=None):
    """q, k [T, H, D] (q already scaled), v [T, H, V], log gates ig, fg [T, H].  Returns o [T, H, V] (divided by
    its normaliser, not yet normed) and the state (S, n, mx)."""
    T, H, D = q.shape
    V = v.shape[2]
    if state is None:
        state = (torch.zeros(H, D, V, dtype=F64), torch.zeros(H, D, dtype=F64), torch.zeros(H, dtype=F64))
    S, n, mx = (t.clone() for t in state)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        new = torch.maximum(fg[t] + mx, ig[t])
        keep, put = torch.exp(fg[t] + mx - new), torch.exp(ig[t] - new)
        S = keep[:, None, None] * S + put[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + put[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    return o, (S, n, mx)


def log_gates(zi, zf, cap):
    """The capped log input gate and log forget gate from their pre-activations."""
    return cap * torch.tanh(zi / cap), torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))


def mlstm(x, w, pre, m, eps, act=identity, state=None):
    """Matrix memory with exponential gating and a running maximum that starts at 0.  `state` (S, n, mx)
    per head continues a sequence; the new state is returned beside the output."""
    T = x.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    xa = act(x)
    q = (xa @ w[f"{pre}.q"].T).view(T, H, D) * D ** -0.5
    k = (xa @ w[f"{pre}.k"].T).view(T, H, D)
    v = (xa @ w[f"{pre}.v"].T).view(T, H, V)
    ig, fg = log_gates(xa @ w[f"{pre}.i"].T + w[f"{pre}.i.b"], xa @ w[f"{pre}.f"].T + w[f"{pre}.f.b"], cap)
    o, state = mlstm_core(q, k, v, ig, fg, state)
    o = rms_unit(o, eps).reshape(T, H * V) * w[f"{pre}.norm"] * torch.sigmoid(xa @ w[f"{pre}.g"].T)
    return act(o) @ w[f"{pre}.o"].T, state


# ---- retention ------------------------------------------------------------------------------------
def rotate_half(t, positions, dims, base):
    """Rotate the first `dims` entries of every head: entry i pairs with entry i + dims/2."""
    half = dims // 2
    f = torch.pow(torch.tensor(base, dtype=F64), -2.0 * torch.arange(half, dtype=F64) / dims)
    a = positions.to(F64)[:, None] * f[None, :]                 # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v2 = t[..., :half], t[..., half:dims]
    return torch.cat([u * c - v2 * s, v2 * c + u * s, t[..., dims:]], dim=-1)


def retention_core(q, k, v, decay, state=None):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for q, k [T, H, D], v [T, H, V], decay [H]."""
    T, H, D = q.shape
    V = v.shape[2]
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def retention(x, w, pre, m, eps, act=identity, state=None, first_position=0):
    """Linear attention with one fixed decay per head, rotary positions on q and k, no denominator."""
    T = x.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    xa = act(x)
    pos = torch.arange(first_position, first_position + T)
    q = (xa @ w[f"{pre}.q"].T).view(T, H, D)
    k = (xa @ w[f"{pre}.k"].T).view(T, H, D)
    v = (xa @ w[f"{pre}.v"].T).view(T, H, V)
    if m.get("rot"):
        q = rotate_half(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_half(k, pos, m["rot"]["dims"], m["rot"]["base"])
    k = k * D ** -0.5
    o, S = retention_core(q, k, v, torch.tensor(m["decay"], dtype=F64), state)
    g = xa @ w[f"{pre}.g"].T
    o = rms_unit(o, eps).reshape(T, H * V) * (g * torch.sigmoid(g))
    return act(o) @ w[f"{pre}.o"].T, S


# ---- routed feed-forward ----------------------------------------------------------------------------
def route(x, w_router, r):
    """(chosen experts [T, top], their weights [T, top]) from sigmoid scores, experts limited to the best
    groups (a group's score: the sum of its two largest scores)."""
    s = torch.sigmoid(x @ w_router.T)                             # [T, E]
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    if r.get("groups"):
        count, keep = r["groups"]["count"], r["groups"]["keep"]
        per = E // count
        gs = s.view(T, count, per).topk(min(2, per), dim=-1).values.sum(-1)      # [T, count]
        best = gs.topk(keep, dim=-1).indices
        ok = torch.zeros(T, count, dtype=torch.bool)
        ok.scatter_(1, best, True)
        allowed = ok[:, :, None].expand(T, count, per).reshape(T, E)
    pick = s.masked_fill(~allowed, -1.0).topk(r["top"], dim=-1).indices
    chosen = s.gather(1, pick)
    return pick, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def expert(x, w, pre, limit, act=identity):
    g = torch.clamp(x @ w[f"{pre}.gate"].T, max=limit)
    u = torch.clamp(x @ w[f"{pre}.up"].T, min=-limit, max=limit)
    return act(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"{pre}.down"].T


def moe(x, w, pre, mlp, act=identity):
    xa = act(x)
    pick, weight = route(xa, w[f"{pre}.router"].to(F64), mlp["router"])
    out = torch.zeros(x.shape[0], w[f"{pre}.e0.down"].shape[0], dtype=F64)
    for e in range(mlp["router"]["experts"]):
        rows, slots = (pick == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += weight[rows, slots][:, None] * expert(xa[rows], w, f"{pre}.e{e}", mlp["expert"]["limit"], act)
    return out


# ---- the whole model --------------------------------------------------------------------------------
def run_order(cfg):
    """Indices of the layers in the order they run (a looped span repeats with the same tensors)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def mixer(kind, x, w, pre, m, eps, act):
    if kind == "attention":
        return attention(x, w, pre, m, act)
    if kind == "mlstm":
        return mlstm(x, w, pre, m, eps, act)[0]
    if kind == "retention":
        return retention(x, w, pre, m, eps, act)[0]
    raise ValueError(kind)


def forward(cfg, w, ids, act=identity, layers_out=None):
    """Logits [T, vocab] of one sequence from its first token.  `layers_out`: a list that receives the
    residual stream (the sum of the streams) after every layer run."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = embed(ids, w, cfg["embedding"]["scale"])
    streams = cfg.get("streams")
    xs = [x0.clone() for _ in range(streams)] if streams else None
    x = x0
    for i in run_order(cfg):
        e, L = cfg["layers"][i], f"l{i}"
        subs = [(1, lambda u: mixer(e["type"], u, w, f"{L}.mix", e["mixer"], eps, act))]
        if e.get("mlp"):
            subs.append((2, lambda u: moe(u, w, f"{L}.mlp", e["mlp"], act)))
        for q, fn in subs:
            if xs is None:
                x = x + fn(layer_norm(x, w[f"{L}.norm{q}"], eps))
                continue
            a, b, mix = w[f"{L}.hc{q}.in"], w[f"{L}.hc{q}.out"], w[f"{L}.hc{q}.mix"]
            y = fn(layer_norm(hyper_input(xs, a), w[f"{L}.norm{q}"], eps))
            xs = hyper_step(xs, y, a, b, mix)
        if layers_out is not None:
            layers_out.append(x.clone() if xs is None else sum(xs))
    if xs is not None:
        x = sum(xs)
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
