"""The Tobovik design in the engine against the plain implementation of `plain_tobovik.py`: every
mechanism's kernel alone, then whole models in every way of cutting a request into steps, mixed
batches with pages and state slots used again, long decoding under CUDA graphs, and greedy generation
through the engine's own entry point and scheduler."""
import math

import numpy as np
import pytest
import torch

import plain_tobovik as pt
import replay_helpers as rh
import tobovik_models as tm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CASES = {"A": (tm.TOBO_A, tm.TOBO_A_PAGE, tm.TOBO_A_RANK, 3), "B": (tm.TOBO_B, tm.TOBO_B_PAGE, tm.TOBO_B_RANK, 5),
         "C": (tm.TOBO_C, tm.TOBO_C_PAGE, tm.TOBO_C_RANK, 9), "D": (tm.TOBO_D, tm.TOBO_D_PAGE, tm.TOBO_D_RANK, 11),
         "E": (tm.TOBO_E, tm.TOBO_E_PAGE, tm.TOBO_E_RANK, 13)}
# root mean square over the vocabulary of (difference minus its mean), as a fraction of the reference
# logits' spread; the float32 run is measured against the plain code in double precision
LIMIT = {"float32": 1e-4, "bfloat16": 0.12}


def model_of(case):
    cfg, page, rank, seed = CASES[case]
    return cfg, page, tm.random_weights(cfg, rank, seed)


def _spread_error(row, ref_row, spread):
    d = np.asarray(row, dtype=np.float64) - ref_row
    return float(np.sqrt(np.mean((d - d.mean()) ** 2))) / spread


class Reference:
    """Whole-sequence logits of the plain code in double precision, and for each position the error that
    rounding activations to bfloat16 alone causes there (the plain code run again with that rounding, and
    with the rounding jittered by one step): where a sublayer's output is nearly zero (a linear-attention
    head whose q . k cancels at a sequence's first tokens), the norm on it blows the rounding up, even
    flips its sign, and no implementation in bfloat16 can be held to more than a few times that."""

    def __init__(self, cfg, w, reqs, dtype):
        self.rows = {r: pt.forward(t, w, cfg).numpy() for r, t in reqs.items()}
        self.spread = float(np.sqrt(np.mean([np.var(v) for v in self.rows.values()])))
        self.dtype = dtype
        self.own = {}
        if dtype == "bfloat16":
            for r, t in reqs.items():
                runs = [pt.forward(t, w, cfg, act=pt.bf16_round).numpy()]
                runs += [pt.forward(t, w, cfg, act=pt.bf16_round_jittered(seed)).numpy() for seed in (1, 2, 3)]
                self.own[r] = [max(_spread_error(x[p], self.rows[r][p], self.spread) for x in runs) for p in range(len(t))]

    def limit(self, r, pos):
        return max(LIMIT[self.dtype], 3.0 * self.own[r][pos]) if self.own else LIMIT[self.dtype]


def plain_rows(cfg, w, reqs, dtype="float32"):
    return Reference(cfg, w, reqs, dtype)


def assert_close(got, ref, dtype, what):
    assert got, "nothing was compared"
    held = 0
    for (r, pos) in sorted(got):
        err, limit = _spread_error(got[(r, pos)], ref.rows[r][pos], ref.spread), ref.limit(r, pos)
        assert err <= limit, f"{what}: request {r} position {pos}: {err:.3e} > {limit:.1e}"
        held += limit <= 2 * LIMIT[dtype]
    assert held >= 0.8 * len(got), "too few positions are well conditioned for this to be a test"


def requests(cfg, lengths, seed):
    return {f"r{i}": tm.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lengths)}


# ---- whole models, every cutting ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D", "E"])
def test_every_cutting_matches_plain(case, dtype):
    cfg, page, w = model_of(case)
    reqs = requests(cfg, [1, 2, 3, 37, 90, 150], seed=1)
    ref = plain_rows(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=33)),
                        ("portions", rh.trace_portions(reqs, seed=2)),
                        ("mixed", rh.trace_mixed(reqs, seed=3, max_live=3))):
        # a pool just large enough, and three slots for six requests: pages and slots are used again
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=3)
        assert_close(rh.run_trace(runner, steps), ref, dtype, f"{case} {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_takes_the_chunked_scan_and_agrees(dtype):
    """700 tokens in one step run the recurrence chunk by chunk (three kernels); in portions, and decoded
    token by token at the end, the single-pass kernel: all agree with the plain code."""
    cfg, page, w = model_of("C")
    reqs = requests(cfg, [700, 300], seed=4)
    ref = plain_rows(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=40)),
                        ("portions", rh.trace_portions(reqs, seed=5, sizes=(2, 61, 64, 65, 128, 257, 300)))):
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_graphs(dtype):
    """Two prompt tokens, then 200 single-token steps of two requests side by side: steps of one shape are
    replayed as a captured graph, the state moves on once per replay."""
    cfg, page, w = model_of("A")
    reqs = requests(cfg, [202, 180], seed=6)
    ref = plain_rows(cfg, w, reqs, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:2], "want": [0, 1]} for r, t in reqs.items()], "end": []}]
    for k in range(2, 202):
        live = [(r, t) for r, t in reqs.items() if k < len(t)]
        steps.append({"step": len(steps), "entries": [{"id": r, "tokens": [t[k]], "want": [0]} for r, t in live],
                      "end": [r for r, t in live if k == len(t) - 1]})
    runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
    assert_close(rh.run_trace(runner, steps), ref, dtype, "long decoding")
    assert runner.graph_replays > 100


def test_batch_does_not_change_a_request():
    """The same request alone and beside others of other lengths: float32 logits agree to rounding."""
    cfg, page, w = model_of("B")
    reqs = requests(cfg, [64, 5, 33], seed=7)
    alone = {}
    for r, t in reqs.items():
        runner = rh.make_runner(cfg, w, "float32", page, 256, max_requests=3)
        alone.update(rh.run_trace(runner, rh.trace_whole({r: t})))
    runner = rh.make_runner(cfg, w, "float32", page, 256, max_requests=3)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
              "end": list(reqs)}]
    together = rh.run_trace(runner, steps)
    for key, row in alone.items():
        assert np.abs(row - together[key]).max() <= 2e-5 * max(1.0, np.abs(row).max()), key


def test_greedy_generation_through_the_engine_and_scheduler():
    """`PagedGenerateEngine.generate`: chunked prompts, decode batches, more requests than slots, a pool
    that forces preemption; the tokens are the plain code's greedy tokens."""
    from litellmengine_b200.engine import PagedGenerateEngine
    cfg, page, w = model_of("A")
    prompts = [tm.random_tokens(cfg, n, 50 + i) for i, n in enumerate([9, 30, 3, 17, 22])]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(pt.forward(ids, w, cfg)[-1].argmax()))
        want.append(ids[len(p):])
    runner = rh.make_runner(cfg, w, "float32", page, 64, max_requests=3, max_tokens_per_step=32)
    engine = PagedGenerateEngine(runner, chunk=8)
    got = engine.generate(prompts, new)
    assert got == want
    assert engine.scheduler.num_preemptions > 0
    runner.cache.check_invariants()


# ---- mechanisms alone -------------------------------------------------------------------------------
def _ops():
    from litellmengine_b200.csrc import ops
    return ops


def _i32(x):
    return torch.as_tensor(x, dtype=torch.int32, device=DEV)


def test_sinusoid_is_added_to_the_embedding():
    ops = _ops()
    width, vocab = 50, 31
    table = torch.randn(vocab, width)
    ids = [3, 30, 0, 7, 7]
    positions = [0, 1, 977, 4096, 100000]
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(25, dtype=torch.float64) / width)
    for dt in (torch.float32, torch.bfloat16):
        tab = table.to(dt)
        h, copy = ops.embedding_sinusoid(_i32(ids), tab.to(DEV), _i32(positions), inv.to(DEV), status,
                                         copy_dtype=None if dt == torch.float32 else dt)
        ref = tab[ids].double() + pt.sinusoid(torch.tensor(positions), width)
        assert (h.double().cpu() - ref).abs().max() < 3e-7 * 4
        if copy is not None:
            assert torch.equal(copy.cpu(), h.cpu().to(dt))
    assert status.tolist() == [0, 0]


def test_norm_of_a_branch_output_joins_the_stream():
    ops = _ops()
    T, H, eps = 7, 72, 1e-5
    h, y, w = torch.randn(T, H), torch.randn(T, H) * 3, 1 + 0.1 * torch.randn(H)
    ref = h.double() + pt.rms_norm(y.double(), w.double(), eps)
    hd = h.to(DEV)
    copy = ops.rmsnorm_add(hd, y.to(DEV), w.to(DEV), eps, torch.bfloat16)
    assert (hd.double().cpu() - ref).abs().max() < 1e-5
    assert torch.equal(copy.cpu(), hd.cpu().to(torch.bfloat16))


def _paged(T, page, nkv, dk, dv, dtype, shuffle_seed=0):
    """One request of T tokens in slot 1 of 3, its pages scattered over a pool."""
    n = -(-T // page)
    order = np.random.RandomState(shuffle_seed).permutation(n + 5)[:n]
    table = torch.full((3, n + 2), -1, dtype=torch.int32)
    table[1, :n] = torch.from_numpy(order.astype(np.int32))
    keys = torch.zeros((n + 5, nkv, page, dk), dtype=dtype, device=DEV)
    values = torch.zeros((n + 5, nkv, page, dv), dtype=dtype, device=DEV)
    return keys, values, table.to(DEV)


@pytest.mark.parametrize("scope", ["projection", "head", None])
def test_prepare_bias_norm_temperature_and_page_write(scope):
    ops = _ops()
    T, nq, nkv, dk, dv, page, eps, coef, every = 19, 4, 2, 24, 40, 4, 1e-5, 0.7, 5
    g = torch.Generator().manual_seed(1)
    proj = torch.randn(T, 7 + nq * dk + nkv * dk + nkv * dv, generator=g)
    bq, bk, bv = (torch.randn(n, generator=g) for n in (nq * dk, nkv * dk, nkv * dv))
    whole = scope == "projection"
    qw = 1 + 0.2 * torch.randn(nq * dk if whole else dk, generator=g)
    kw = 1 + 0.2 * torch.randn(nkv * dk if whole else dk, generator=g)
    keys, values, table = _paged(T, page, nkv, dk, dv, torch.float32)
    pos = torch.arange(T)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    q = ops.attention_prepare(proj.to(DEV), 7, 7 + nq * dk, 7 + (nq + nkv) * dk, (bq.to(DEV), bk.to(DEV), bv.to(DEV)),
                              qw.to(DEV) if scope else None, kw.to(DEV) if scope else None, scope, eps, (coef, every),
                              keys, values, _i32(pos), _i32([0] * T), _i32([1]), table, nq, nkv, dk, dv, page, status,
                              torch.float32)
    p64 = proj.double()
    q_ref = p64[:, 7:7 + nq * dk] + bq.double()
    k_ref = p64[:, 7 + nq * dk:7 + (nq + nkv) * dk] + bk.double()
    v_ref = p64[:, 7 + (nq + nkv) * dk:] + bv.double()
    if whole:
        q_ref, k_ref = pt.rms_norm(q_ref, qw.double(), eps), pt.rms_norm(k_ref, kw.double(), eps)
    elif scope == "head":
        q_ref = pt.rms_norm(q_ref.view(T, nq, dk), qw.double(), eps).reshape(T, -1)
        k_ref = pt.rms_norm(k_ref.view(T, nkv, dk), kw.double(), eps).reshape(T, -1)
    q_ref = q_ref * pt.query_temperature(pos, coef, every)[:, None]
    assert (q.double().cpu() - q_ref).abs().max() < 2e-5
    tab = table[1].cpu()
    for t in range(T):
        kp = keys[tab[t // page], :, t % page].reshape(-1).double().cpu()
        vp = values[tab[t // page], :, t % page].reshape(-1).double().cpu()
        assert (kp - k_ref[t]).abs().max() < 2e-5 and (vp - v_ref[t]).abs().max() < 2e-5
    assert status.tolist() == [0, 0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 15, 16, 17, 300, 511, 512, 600])
def test_attention_finds_one_far_key(far, dtype):
    """641 keys of which ONE (at a page's first or last place, at the sequence's first place, hundreds of
    tokens back) matches the last query: softmax puts nearly all weight on it, so losing it, or taking its
    neighbour for it, changes the output completely.  Keys and values differ in width; the output is
    gated and scaled and lands in a column range of a wider buffer."""
    ops = _ops()
    T, nq, nkv, dk, dv, page, scale, out_scale = 641, 4, 2, 24, 40, 16, 0.5, 0.75
    g = torch.Generator().manual_seed(far)
    k = torch.randn(T, nkv, dk, generator=g) * 0.3
    v = torch.randn(T, nkv, dv, generator=g)
    q = torch.randn(T, nq, dk, generator=g) * 0.3
    for h in range(nq):
        q[-1, h] = 6.0 * k[far, h // (nq // nkv)] / k[far, h // (nq // nkv)].norm() * (1 + 0.1 * h)
        k[far, h // (nq // nkv)] *= 4.0
    gate = torch.randn(T, 5 + nq * dv, generator=g)
    q, k, v = (x.to(dtype).to(torch.float32) for x in (q, k, v))
    keys, values, table = _paged(T, page, nkv, dk, dv, dtype, shuffle_seed=far)
    tab = table[1].cpu()
    for t in range(T):
        keys[tab[t // page], :, t % page] = k[t].to(dtype).to(DEV)
        values[tab[t // page], :, t % page] = v[t].to(dtype).to(DEV)
    out = torch.zeros((T, 3 + nq * dv + 2), dtype=dtype, device=DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    ops.paged_attention_generic_kv(q.reshape(T, -1).to(dtype).to(DEV), keys, values, _i32(torch.arange(T)), _i32([0] * T),
                                   _i32([1]), table, nq, nkv, dk, dv, page, None, scale, status, out, 3,
                                   gate=gate.to(DEV), gate_off=5, out_scale=out_scale)
    ref = torch.zeros(T, nq, dv, dtype=torch.float64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(nq):
        s = (q[:, h].double() @ k[:, h // 2].double().T) * scale
        p = torch.softmax(s.masked_fill(~causal, float("-inf")), dim=-1)
        ref[:, h] = p @ v[:, h // 2].double()
        assert p[-1, far] > 0.9
    ref = ref.reshape(T, -1) * torch.sigmoid(gate[:, 5:].double()) * out_scale
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    got = out[:, 3:3 + nq * dv].double().cpu()
    assert (got - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
    assert float(out[:, :3].abs().max()) == 0 and float(out[:, 3 + nq * dv:].abs().max()) == 0
    assert status.tolist() == [0, 0]


def test_decay_is_sigmoid_to_the_power_one_over_tau():
    ops = _ops()
    T, rank, C, tau = 71, 5, 300, 3.0
    proj = torch.randn(T, 11 + rank) * 4
    w2, b2 = torch.randn(C, rank) * 3, torch.randn(C) * 10          # z far out on both sides
    la = ops.gla_decay(proj.to(DEV), 11, rank, w2.t().contiguous().to(DEV), b2.to(DEV), tau)
    z = proj[:, 11:].double() @ w2.double().T + b2.double()
    ref = torch.sigmoid(z) ** (1.0 / tau)
    assert torch.isfinite(la).all() and float(la.min()) >= 0.0 and float(la.max()) <= 1.0
    # the decode kernel makes the same decays itself: with k = 0 and a state of ones, S' = alpha
    H, D, V = 3, C // 3, 8
    wide = torch.zeros(T, 11 + rank + 2 * H * D + 2 * H * V)
    wide[:, :11 + rank] = proj
    state = torch.ones((T, H, D, V), dtype=torch.float32, device=DEV)
    o0 = 11 + rank
    ops.gla_step(wide.to(DEV), (o0, o0 + H * D, o0 + 2 * H * D, o0 + 2 * H * D + H * V), None, torch.ones(V, device=DEV),
                 1e-5, 1.0, 1.0, torch.empty((T, H * V), device=DEV), 0, state, _i32(list(range(T))), _i32(list(range(T))),
                 T, H, D, V, decay=(11, rank, w2.t().contiguous().to(DEV), b2.to(DEV), tau))
    assert (state[:, :, :, 0].reshape(T, C).double().cpu() - ref).abs().max() < 1e-6
    assert (la.double().cpu() - ref).abs().max() < 1e-6
    # far out on the negative side the decay is tiny but its logarithm is still right
    small = ref > 1e-30
    assert ((torch.log(la.double().cpu()[small]) - torch.log(ref[small])).abs() / (1 + torch.log(ref[small]).abs())).max() < 1e-5


@pytest.mark.parametrize("H,D,V", [(2, 8, 16), (3, 16, 8), (2, 24, 40), (1, 64, 64), (2, 128, 128), (1, 48, 100),
                                   (1, 128, 256)])
def test_recurrence_in_one_pass_in_portions_and_in_chunks(H, D, V):
    """The recurrence kernel against the token-by-token recurrence in double precision: an entry in one
    pass; the same tokens in portions that carry the state in the request's slot (down to one token); cut
    into chunks that run side by side (local pass, chain, output pass); token by token through the kernel
    of decode steps.  A channel that never decays
    carries an impulse from the first token to the last; a channel that decays at once forgets it."""
    ops = _ops()
    T, eps, out_scale = 333, 1e-5, 0.9
    g = torch.Generator().manual_seed(H * 1000 + D)
    W = 2 * H * D + 2 * H * V
    proj = torch.randn(T, 3 + W, generator=g)
    la = -torch.rand(T, H * D, generator=g) * 0.3
    la[:, 0] = 0.0                    # never decays
    la[:, 1] = -40.0                  # forgets at once
    proj[0, 3 + H * D:3 + H * D + 2] = 25.0      # an impulse in k of those two channels at the first token
    norm_w = 1 + 0.1 * torch.randn(V, generator=g)
    offs = (3, 3 + H * D, 3 + 2 * H * D, 3 + 2 * H * D + H * V)
    q, k = (proj[:, o:o + H * D].double().view(T, H, D) for o in offs[:2])
    v, gt = (proj[:, o:o + H * V].double().view(T, H, V) for o in offs[2:])
    o_ref, s_ref = pt.gla_recurrence(q * D ** -0.5, k, v, la.double().view(T, H, D))
    ref = (pt.rms_norm(o_ref, norm_w.double(), eps) * (gt * torch.sigmoid(gt)) * out_scale).reshape(T, -1)
    slots = _i32([2])

    def run(cuts, chunk=None, step=False):
        state = torch.zeros((4, H, D, V), dtype=torch.float32, device=DEV)
        state[1] = 7.0                                                    # another request's state stays untouched
        out = torch.zeros((T, H * V + 4), dtype=torch.float32, device=DEV)
        pd, lad, nw = proj.to(DEV), torch.exp(la).to(DEV), norm_w.to(DEV)         # the kernels take the decays themselves
        at = 0
        for n in cuts:
            args = (pd[at:at + n], offs, lad[at:at + n], nw, eps, D ** -0.5, out_scale, out[at:at + n], 2, state, slots,
                    _i32([0]), _i32([n]))
            if step and n == 1:
                ops.gla_step(*args[:-1], 1, H, D, V)
            elif chunk is None:
                ops.gla_scan(*args, None, 1, ops.GLA_FULL, None, None, H, D, V)
            else:
                items = [(0, c, min(chunk, n - c), i) for i, c in enumerate(range(0, n, chunk))]
                ss = torch.empty((len(items), H, D, V), dtype=torch.float32, device=DEV)
                sa = torch.empty((len(items), H, D), dtype=torch.float32, device=DEV)
                it = _i32(items)
                ops.gla_scan(*args, it, len(items), ops.GLA_LOCAL, ss, sa, H, D, V)
                ops.gla_chain(state, ss, sa, _i32([(0, 0, len(items))]), 1, slots, H, D, V)
                ops.gla_scan(*args, it, len(items), ops.GLA_OUT, ss, sa, H, D, V)
            at += n
        assert at == T
        assert float((state[1] - 7.0).abs().max()) == 0 and float(state[0].abs().max()) == 0
        return out.double().cpu(), state[2].double().cpu()

    scale = max(1.0, float(ref.abs().max()))
    for what, (got, s) in (("one pass", run([T])), ("portions", run([1, 2, 16, 17, 1, 64, 100, 31, 101])),
                           ("chunks", run([T], chunk=64)), ("chunks after a portion", run([70, T - 70], chunk=32)),
                           ("a portion, then the decode kernel token by token", run([33] + [1] * (T - 33), step=True))):
        assert (got[:, 2:2 + H * V] - ref).abs().max() < 2e-5 * scale, what
        assert float(got[:, :2].abs().max()) == 0, what
        assert (s - s_ref).abs().max() < 2e-5 * max(1.0, float(s_ref.abs().max())), what
    assert s_ref[:, 0].abs().max() > 10 and s_ref[:, 1].abs().max() < 10        # the impulse is there, and is forgotten


# ---- as a user runs it --------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_replays_a_model_folder(tmp_path, dtype):
    """bin/trace_run on a folder with config.json and model.safetensors (bfloat16 tensors, the decay
    projection's rank known from the tensors alone): a mixed trace with four live requests."""
    import json
    import os
    import subprocess
    from litellmengine_b200.weights import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, page, w = model_of("B")
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(model_dir / "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in w.items()})
    reqs = requests(cfg, [70, 33, 129, 1, 200], seed=8)
    steps = rh.trace_mixed(reqs, seed=2, max_live=4)
    out_dir = str(tmp_path / "out")
    proc = subprocess.run(
        [os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", out_dir,
         "--max-tokens", str(rh.peak_tokens(steps, 64)), "--max-requests", "4"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    got = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            got[s["step"]] = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(wanted, cfg["vocab"])
    rows = rh.collect(steps, got)
    assert len(rows) == sum(len(t) for t in reqs.values())
    assert_close(rows, plain_rows(cfg, w, reqs, dtype), dtype, f"trace_run {dtype}")


def test_command_line_generates_from_a_model_folder(tmp_path):
    """The engine's command line picks the model class by config.json and generates greedily."""
    import json
    import os
    import subprocess
    import sys
    from litellmengine_b200.weights import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, page, w = model_of("A")
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(model_dir / "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in w.items()})
    prompt = tm.random_tokens(cfg, 11, 77)
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(pt.forward(ids, w, cfg)[-1].argmax()))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(model_dir), "--input-ids",
                           ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert proc.stdout.strip().split("\n")[-1] == ",".join(map(str, ids[len(prompt):]))
