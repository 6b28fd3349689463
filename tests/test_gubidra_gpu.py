"""The Gubidra design in the engine against the plain implementation of `plain_gubidra.py`: every
mechanism's kernel alone (with inputs made so that a lost key, a wrong edge or a lost state shows), then
whole models in every way of cutting a request into steps, mixed batches with pages and state slots used
again, long decoding under CUDA graphs, and greedy generation through the engine's own entry point and
scheduler."""
import math

import numpy as np
import pytest
import torch

import gubidra_models as gm
import plain_gubidra as pg
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

CASES = {"A": (gm.GUBI_A, gm.GUBI_A_PAGE, 3), "B": (gm.GUBI_B, gm.GUBI_B_PAGE, 5), "C": (gm.GUBI_C, gm.GUBI_C_PAGE, 9),
         "D": (gm.GUBI_D, gm.GUBI_D_PAGE, 11)}
# root mean square over the vocabulary of (difference minus its mean), as a fraction of the reference
# logits' spread; the float32 run is measured against the plain code in double precision
LIMIT = {"float32": 1e-4, "bfloat16": 0.12}


def model_of(case):
    cfg, page, seed = CASES[case]
    return cfg, page, gm.random_weights(cfg, seed)


def _spread_error(row, ref_row, spread):
    d = np.asarray(row, dtype=np.float64) - ref_row
    return float(np.sqrt(np.mean((d - d.mean()) ** 2))) / spread


class Reference:
    """Whole-sequence logits of the plain code in double precision, and for each position the error that
    rounding activations to bfloat16 alone causes there (the plain code run again with that rounding, and
    with the rounding jittered): a recurrent head's output at a sequence's first tokens is (q . k) v through
    a norm, so where q . k nearly cancels rounding decides its sign, and a routed feed-forward may choose
    another expert on a close call; no implementation in bfloat16 can be held to more than a few times that."""

    def __init__(self, cfg, w, reqs, dtype):
        self.rows = {r: pg.forward(cfg, w, t).numpy() for r, t in reqs.items()}
        self.spread = float(np.sqrt(np.mean([np.var(v) for v in self.rows.values()])))
        self.dtype = dtype
        self.own, self.rounded = {}, {}
        if dtype == "bfloat16":
            for r, t in reqs.items():
                runs = [pg.forward(cfg, w, t, act=pg.bf16_round).numpy()]
                runs += [pg.forward(cfg, w, t, act=pg.bf16_round_jittered(seed)).numpy() for seed in (1, 2)]
                self.rounded[r] = runs
                self.own[r] = [max(_spread_error(x[p], self.rows[r][p], self.spread) for x in runs) for p in range(len(t))]

    def limit(self, r, pos):
        return max(LIMIT[self.dtype], 3.0 * self.own[r][pos]) if self.own else LIMIT[self.dtype]

    def error(self, row, r, pos):
        """Against the plain code in double precision; a bfloat16 run also against the plain code's own rounded
        runs (a close call that one of them decided the same way), whichever is nearest."""
        errs = [_spread_error(row, self.rows[r][pos], self.spread)]
        errs += [_spread_error(row, x[pos], self.spread) for x in self.rounded.get(r, [])]
        return min(errs)


def assert_close(got, ref, dtype, what):
    """float32: every position within the limit.  bfloat16: a routed feed-forward turns a close call between two
    experts into a jump that the plain code's own roundings need not hit at the same token, so a few positions
    (5 in 100) may exceed their limit; the sharp test of every edge is the float32 one."""
    assert got, "nothing was compared"
    held, over = 0, []
    for (r, pos) in sorted(got):
        err, limit = ref.error(got[(r, pos)], r, pos), ref.limit(r, pos)
        if err > limit:
            over.append(f"{what}: request {r} position {pos}: {err:.3e} > {limit:.1e}")
        held += limit <= 2 * LIMIT[dtype]
    allowed = 0 if dtype == "float32" else max(2, int(0.05 * len(got)))
    assert len(over) <= allowed, "; ".join(over[:5])
    assert held >= 0.7 * len(got), "too few positions are well conditioned for this to be a test"


def requests(cfg, lengths, seed):
    return {f"r{i}": gm.random_tokens(cfg, n, seed * 100 + i) for i, n in enumerate(lengths)}


# ---- whole models, every cutting ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_every_cutting_matches_plain(case, dtype):
    cfg, page, w = model_of(case)
    reqs = requests(cfg, [1, 2, 3, 37, 90, 150], seed=1)
    ref = Reference(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=33)),
                        ("portions", rh.trace_portions(reqs, seed=2)),
                        ("mixed", rh.trace_mixed(reqs, seed=3, max_live=3))):
        # a pool just large enough, and three slots for six requests: pages and slots are used again
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=3)
        assert_close(rh.run_trace(runner, steps), ref, dtype, f"{case} {name}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_takes_the_chunked_scan_and_agrees(dtype):
    """600 tokens in one step run the recurrences chunk by chunk (local pass, chain, output pass; the
    gates of the matrix memory walk the whole portion first); in portions, and decoded token by token
    at the end, the single-pass kernels: all agree with the plain code.  The window of 130 keys passes
    over page borders in prompts and in decoding."""
    cfg, page, w = model_of("C")
    reqs = requests(cfg, [600, 300], seed=4)
    ref = Reference(cfg, w, reqs, dtype)
    for name, steps in (("whole", rh.trace_whole(reqs)), ("decode", rh.trace_tail_decode(reqs, tail=140)),
                        ("portions", rh.trace_portions(reqs, seed=5, sizes=(2, 61, 64, 65, 128, 257, 300)))):
        runner = rh.make_runner(cfg, w, dtype, page, rh.peak_tokens(steps, round_to=page), max_requests=2)
        assert_close(rh.run_trace(runner, steps), ref, dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_graphs(dtype):
    """Two prompt tokens, then 200 single-token steps of two requests side by side: steps of one shape are
    replayed as a captured graph, the states move on once per replay, the windows slide and give pages back."""
    cfg, page, w = model_of("A")
    reqs = requests(cfg, [202, 180], seed=6)
    ref = Reference(cfg, w, reqs, dtype)
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
    cfg, page, w = model_of("B")
    prompts = [gm.random_tokens(cfg, n, 50 + i) for i, n in enumerate([9, 30, 3, 17, 22])]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(pg.forward(cfg, w, ids)[-1].argmax()))
        want.append(ids[len(p):])
    runner = rh.make_runner(cfg, w, "float32", page, 64, max_requests=3, max_tokens_per_step=32)
    engine = PagedGenerateEngine(runner, chunk=8)
    got = engine.generate(prompts, new)
    assert got == want
    assert engine.scheduler.num_preemptions > 0
    runner.cache.check_invariants()


def test_trace_replay_and_prompt_command_on_a_model_folder(tmp_path):
    """`bin/trace_run` and `bin/run_prompt` on a folder written in the design's own format."""
    import json
    import os
    import subprocess
    import sys
    from litellmengine_b200.weights.safetensors_io import write_safetensors
    cfg, page, w = model_of("D")
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), {k: (v.to(torch.bfloat16) if v.dim() == 2 else v) for k, v in w.items()})
    toks = gm.random_tokens(cfg, 40, 8)
    ref = pg.forward(cfg, w, toks).numpy()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:25], "want": [3, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[25:], "want": [14]}], "end": ["a"]}]
    out = tmp_path / "out"
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32",
                          "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    spread = float(np.std(ref))
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for row, pos in ((got0[0], 3), (got0[1], 24), (got1[0], 39)):
        assert _spread_error(row, ref[pos], spread) < 1e-4
    # the prompt command: greedy tokens through the scheduler and the sampler
    prompt = toks[:17]
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(pg.forward(cfg, w, ids)[-1].argmax()))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "run_prompt"), "--model", str(folder), "--input-ids",
                           ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert proc.stdout.strip().split("\n")[-1] == ",".join(map(str, ids[len(prompt):]))


# ---- mechanisms alone -------------------------------------------------------------------------------
def _ops():
    from litellmengine_b200.csrc import ops
    return ops


def _i32(x):
    return torch.as_tensor(x, dtype=torch.int32, device=DEV)


def test_embedding_scale():
    ops = _ops()
    table = torch.randn(13, 24).to(torch.bfloat16)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    h = ops.embedding(_i32([3, 12, 0]), table.to(DEV), status, scale=7.25)
    assert torch.equal(h.cpu(), table[[3, 12, 0]].float() * 7.25)


@pytest.mark.parametrize("S", [1, 2, 3, 5])
@pytest.mark.parametrize("center", [True, False])
def test_streams_update_and_norm(S, center):
    """x_t <- sum_s mix[s, t] x_s + out[t] y, u = sum in[t] x_t, norm(u) w: against the plain formulas, with y as a
    product's k-splits, with picked rows, and as the plain residual stream (S = 1, no coefficients)."""
    ops = _ops()
    T, H, eps = 9, 52, 1e-5
    g = torch.Generator().manual_seed(S)
    xs = [torch.randn(T, H, generator=g, dtype=F64) * 3 + 1 for _ in range(S)]
    y = torch.randn(T, H, generator=g, dtype=F64)
    mix, out, inp = torch.randn(S, S, generator=g, dtype=F64), torch.randn(S, generator=g, dtype=F64), torch.randn(S, generator=g, dtype=F64)
    wn = 1 + 0.1 * torch.randn(H, generator=g, dtype=F64)
    new = pg.hyper_step(xs, y, inp, out, mix)
    u = pg.hyper_input(new, inp)
    ref = pg.layer_norm(u, wn, eps) if center else pg.rms_unit(u, eps) * wn
    f32 = lambda t: t.float().to(DEV).contiguous()
    streams = f32(torch.stack(xs))
    parts = torch.stack([y * 0.25, y * 0.5, y * 0.25]).float().to(DEV)
    got = ops.stream_norm(streams, ops.PartialSum(parts), f32(mix), f32(out), f32(inp), f32(wn), eps, center, torch.float32)
    assert (got.double().cpu() - ref).abs().max() < 2e-5
    assert (streams.double().cpu() - torch.stack(new)).abs().max() < 2e-5
    # picked rows, the sum of the streams (a model's final norm), nothing written back
    streams2 = f32(torch.stack(xs))
    rows = [7, 0, 3]
    got = ops.stream_norm(streams2, f32(y), f32(mix), f32(out), None, f32(wn), eps, center, torch.float32, rows=_i32(rows))
    u = sum(new)[rows]
    ref = pg.layer_norm(u, wn, eps) if center else pg.rms_unit(u, eps) * wn
    assert (got.double().cpu() - ref).abs().max() < 2e-5
    assert torch.equal(streams2.cpu(), torch.stack(xs).float())
    # a model's first layer: only stream 0 holds the embedding, the others are written on the way
    first = torch.full((S, T, H), 7.0, device=DEV)
    first[0] = f32(xs[0])
    got = ops.stream_norm(first, None, None, None, f32(inp), f32(wn), eps, center, torch.float32, fan=True)
    u = xs[0] * inp.sum()
    ref = pg.layer_norm(u, wn, eps) if center else pg.rms_unit(u, eps) * wn
    assert (got.double().cpu() - ref).abs().max() < 2e-5
    assert all(torch.equal(first[s2].cpu(), xs[0].float()) for s2 in range(S))
    if S == 1:      # the plain residual stream: x += y, norm(x)
        x = f32(xs[0])
        got = ops.stream_norm(x, f32(y), None, None, None, f32(wn), eps, center, torch.bfloat16)
        ref = pg.layer_norm(xs[0] + y, wn, eps) if center else pg.rms_unit(xs[0] + y, eps) * wn
        assert (got.double().cpu() - ref).abs().max() < 0.02
        assert (x.double().cpu() - (xs[0] + y)).abs().max() < 1e-5


def _paged(T, page, nkv, dk, dv, dtype, shuffle_seed=0):
    """One request of T tokens in slot 1 of 3, its pages scattered over a pool."""
    n = -(-T // page)
    pool = n + 5
    order = np.random.RandomState(shuffle_seed).permutation(pool)[:n]
    table = torch.full((3, n + 2), -1, dtype=torch.int32)
    table[1, :n] = torch.as_tensor(order, dtype=torch.int32)
    keys = torch.zeros(pool, nkv, page, dk, dtype=dtype, device=DEV)
    values = torch.zeros(pool, nkv, page, dv, dtype=dtype, device=DEV)
    return keys, values, table.to(DEV), order


def _fill(keys, values, order, page, k, v):
    for j in range(k.shape[0]):
        keys[order[j // page], :, j % page] = k[j].to(keys.dtype).to(DEV)
        values[order[j // page], :, j % page] = v[j].to(values.dtype).to(DEV)


@pytest.mark.parametrize("window", [None, 1, 7, 64, 65])
def test_attention_distance_bias_window_and_head_gate(window):
    """Random scores with a table that matters, and one key that would win by far placed just inside and just
    outside the window (which loses it), at a page's first and last place and at the sequence's first token."""
    ops = _ops()
    from litellmengine_b200.parts.attention import distance_bucket
    T, page, H, G, D, V, rows, far, scale = 150, 16, 4, 2, 24, 40, 10, 60.0, 0.3
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=F64) for n, d in ((H, D), (G, D), (G, V)))
    rel = torch.randn(rows, H, generator=g, dtype=F64) * 2
    gate = torch.randn(T, H, generator=g, dtype=F64)
    probes = [149, 148, 130, 100]
    if window is not None:          # a key that stands out, at the edge of the last queries' windows
        for i, off in zip(probes, (window - 1, window, window - 1, window)):
            j = i - off
            if j >= 0:
                k[j] = q[i, :G] * 4.0
    k[0] = q[120, :G] * 4.0          # the first token: seen by query 120 only without a window
    k[15], k[16] = q[140, :G] * 3.0, q[141, :G] * 3.0      # a page's last and first place
    count = int(math.ceil(far)) + 1 if window is None else min(int(math.ceil(far)) + 1, window)
    table = rel[[distance_bucket(n, rows, far) for n in range(count)]].float().to(DEV).contiguous()
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 0.05)):
        keys, values, block_table, order = _paged(T, page, G, D, V, dtype, 1)
        _fill(keys, values, order, page, k, v)
        out = torch.zeros(T, H * V + 8, dtype=dtype, device=DEV)
        gate_buf = torch.zeros(T, 3 + H, dtype=torch.float32, device=DEV)
        gate_buf[:, 3:] = gate.float().to(DEV)
        status = torch.zeros(2, dtype=torch.int32, device=DEV)
        ops.paged_attention_generic_kv(q.reshape(T, -1).to(dtype).to(DEV), keys, values, _i32(torch.arange(T)), _i32([0] * T),
                                       _i32([1]), block_table, H, G, D, V, page, window, scale, status, out, 8,
                                       gate=gate_buf, gate_off=3, dist_bias=table, gate_per_head=True)
        assert status.tolist() == [0, 0]
        kq, kk, kv = (t.to(dtype).double() for t in (q, k, v))
        ref_d = pg.attention_core(kq, kk, kv, rel, scale, far, window) * torch.sigmoid(gate)[:, :, None]
        got = out[:, 8:].double().cpu().view(T, H, V)
        assert (got - ref_d).abs().max() < tol, (window, dtype)


def test_distance_buckets_against_the_plain_rule():
    from litellmengine_b200.parts.attention import distance_bucket
    for rows, far in ((4, 9.0), (6, 16.0), (16, 240.0), (12, 100.0), (32, 1000.0)):
        got = [distance_bucket(n, rows, far) for n in range(int(far) + 50)]
        assert got == [pg.distance_bucket(n, rows, far) for n in range(int(far) + 50)]
        assert got[:rows // 2] == list(range(rows // 2)) and got[int(far)] == rows - 1 and max(got) == rows - 1
        assert all(b >= a for a, b in zip(got, got[1:]))


def _recurrent_setup(T, H, D, V, extra_cols, seed):
    g = torch.Generator().manual_seed(seed)
    width = 2 * H * D + 2 * H * V + extra_cols
    proj = torch.randn(T, width, generator=g, dtype=F64)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    return proj, offs


def _pieces(proj, offs, H, D, V):
    T = proj.shape[0]
    q = proj[:, :H * D].reshape(T, H, D).clone()
    k = proj[:, H * D:2 * H * D].reshape(T, H, D).clone()
    v = proj[:, 2 * H * D:2 * H * D + H * V].reshape(T, H, V).clone()
    return q, k, v, proj[:, offs[3]:offs[3] + H * V].clone()


def _scan_lists(portions, chunk):
    """Work lists of one entry per portion: (short items, chunk items, chains) as the step's prelude makes them."""
    short, chunks, chains = [], [], []
    at = 0
    for i, n in enumerate(portions):
        if chunk is None or n < chunk * 2:
            short.append((i, at, n, 0))
        else:
            first = len(chunks)
            for c0 in range(0, n, chunk):
                chunks.append((i, at + c0, min(chunk, n - c0), len(chunks)))
            chains.append((i, first, len(chunks) - first))
        at += n
    return short, chunks, chains


def _run_recurrence(mixer_kind, proj, offs, H, D, V, portions, chunk, dtype, **kw):
    """Feed one request's tokens portion by portion (each portion its own step, as the engine would) through the
    recurrence kernels: portions of one token through the decode kernel, others through the scan (in chunks
    when `chunk` is given and the portion is long enough).  Returns the outputs [T, H*V] and the state."""
    ops = _ops()
    T = proj.shape[0]
    normaliser = mixer_kind == "mlstm"
    head_floats = D * (V + 1) + 1 if normaliser else D * V
    state = torch.zeros(3, H, head_floats, dtype=torch.float32, device=DEV)
    out = torch.zeros(T, H * V, dtype=dtype, device=DEV)
    pd = proj.float().to(DEV).contiguous()
    at = 0
    for n in portions:
        rows = pd[at:at + n].clone()
        o = out[at:at + n]
        slot, q_start, q_len = _i32([2]), _i32([0]), _i32([n])
        positions = _i32(list(range(at, at + n)))
        if mixer_kind == "retention":
            decay, rot = kw["decay"], kw.get("rot")
            if n == 1:
                ops.recur_step(rows, offs, decay, (0, 1, 0), None, 0, "silu", kw["eps"], D ** -0.5, 1.0, o, 0, state, head_floats,
                               slot, q_start, 1, H, D, V, rotation=(rot[0], rot[1], positions) if rot else None)
                at += n
                continue
            if rot:
                ops.rotate_qk(rows, offs[0], offs[1], H, H, D, rot[1], rot[0], positions)
            alpha, a_tok, a_head, kscale, nfloor, norm_w, norm_stride, gate = decay, 0, 1, None, None, None, 0, "silu"
        else:
            gates = (kw["i_off"], kw["f_off"], kw["i_bias"], kw["f_bias"], kw["cap"])
            if n == 1:
                ops.recur_step(rows, offs, None, None, kw["norm_w"], V, "sigmoid", kw["eps"], D ** -0.5, 1.0, o, 0, state,
                               head_floats, slot, q_start, 1, H, D, V, gates=gates)
                at += n
                continue
            gt = ops.recur_gates(rows, gates[0], gates[1], gates[2], gates[3], gates[4], state, D * (V + 1), head_floats, slot,
                                 q_start, q_len, 1, H)
            alpha, a_tok, a_head, kscale, nfloor, norm_w, norm_stride, gate = gt[0], H, 1, gt[1], gt[2], kw["norm_w"], V, "sigmoid"
        short, chunks, chains = _scan_lists([n], chunk)
        scan = lambda items, cnt, mode, ss, sa: ops.recur_scan(
            rows, offs, alpha, a_tok, a_head, kscale, nfloor, norm_w, norm_stride, gate, kw["eps"], D ** -0.5, 1.0, o, 0, state,
            head_floats, slot, q_start, q_len, _i32(items), cnt, mode, ss, sa, H, D, V)
        if short:
            scan(short, len(short), ops.GLA_FULL, None, None)
        if chunks:
            cols = V + 1 if normaliser else V
            ss = torch.empty(len(chunks), H, D * cols, dtype=torch.float32, device=DEV)
            sa = torch.empty(len(chunks), H, D, dtype=torch.float32, device=DEV)
            scan(chunks, len(chunks), ops.GLA_LOCAL, ss, sa)
            ops.recur_chain(state, head_floats, ss, sa, _i32(chains), len(chains), slot, H, D, V, normaliser)
            scan(chunks, len(chunks), ops.GLA_OUT, ss, sa)
        at += n
    torch.cuda.synchronize()
    assert float(state[0].abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0, "another slot's state was touched"
    return out.double().cpu(), state[2].double().cpu()


CUTTINGS = [("whole", lambda T: [T], None), ("chunks of 16", lambda T: [T], 16),
            ("portions", lambda T: [2, 31, 1, 1, 64, 1] + [T - 100], None),
            ("portions in chunks", lambda T: [70, 3, T - 73], 16), ("decode", lambda T: [5] + [1] * (T - 5), None)]


@pytest.mark.parametrize("shape", [(3, 8, 16, 4), (2, 16, 8, 16), (1, 64, 64, 32), (2, 12, 20, 0), (2, 32, 48, 32)])
def test_retention_recurrence_in_every_cutting(shape):
    """Fixed decays per head (one head never forgets, one forgets at once), a rotation over a part of a head,
    over all of it and none; one pass, chunks, portions down to one token, the decode kernel; the state that is
    left behind is the plain code's in every cutting."""
    H, D, V, rot_dims = shape
    T, eps, base = 140, 1e-5, 300.0
    proj, offs = _recurrent_setup(T, H, D, V, 0, 5)
    q, k, v, gate = _pieces(proj, offs, H, D, V)
    decay = torch.tensor(([1.0, 0.0, 0.9] * H)[:H], dtype=F64)
    pos = torch.arange(T)
    qr, kr = (pg.rotate_half(t, pos, rot_dims, base) if rot_dims else t for t in (q, k))
    o, S = pg.retention_core(qr, kr * D ** -0.5, v, decay)
    ref = (pg.rms_unit(o, eps).reshape(T, H * V) * (gate * torch.sigmoid(gate)))
    inv = torch.pow(torch.tensor(base, dtype=F64), -2.0 * torch.arange(rot_dims // 2, dtype=F64) / max(rot_dims, 1))
    rot = (inv.float().to(DEV), rot_dims) if rot_dims else None
    for name, cut, chunk in CUTTINGS:
        got, state = _run_recurrence("retention", proj, offs, H, D, V, cut(T), chunk, torch.float32,
                                     decay=decay.float().to(DEV), rot=rot, eps=eps)
        assert (got - ref).abs().max() < 3e-4, name
        # the engine keeps the state without the keys' scale (it scales the finished sums)
        assert (state.view(H, D, V) * D ** -0.5 - S).abs().max() < 3e-4 * max(1.0, float(S.abs().max())), name


@pytest.mark.parametrize("shape", [(3, 8, 16), (2, 16, 8), (1, 64, 64), (2, 12, 20), (2, 32, 48), (1, 128, 128)])
def test_matrix_memory_recurrence_in_every_cutting(shape):
    """Exponential gates with a running maximum from 0: gates far out on both sides (the cap holds them), a
    normaliser below its floor at the first tokens and above it later; one pass, chunks, portions, decode."""
    H, D, V = shape
    T, eps, cap = 140, 1e-5, 5.0
    proj, offs = _recurrent_setup(T, H, D, V, 2 * H + 1, 6)
    i_off, f_off = offs[3] + H * V + 1, offs[3] + H * V + 1 + H
    proj[:, i_off:i_off + H] *= 6.0                       # far beyond the cap on both sides
    proj[:, f_off:f_off + H] = proj[:, f_off:f_off + H] * 3.0 + 2.0
    proj[:3, :2 * H * D] *= 0.05                          # first tokens: |n . q| below the floor
    q, k, v, gate = _pieces(proj, offs, H, D, V)
    g = torch.Generator().manual_seed(7)
    bi, bf = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    wn = 1 + 0.2 * torch.randn(H * V, generator=g, dtype=F64)
    ig, fg = pg.log_gates(proj[:, i_off:i_off + H] + bi, proj[:, f_off:f_off + H] + bf, cap)
    o, (S, n, mx) = pg.mlstm_core(q * D ** -0.5, k, v, ig, fg)
    ref = pg.rms_unit(o, eps).reshape(T, H * V) * wn * torch.sigmoid(gate)
    for name, cut, chunk in CUTTINGS:
        got, state = _run_recurrence("mlstm", proj, offs, H, D, V, cut(T), chunk, torch.float32, i_off=i_off, f_off=f_off,
                                     i_bias=bi.float().to(DEV), f_bias=bf.float().to(DEV), cap=cap, eps=eps,
                                     norm_w=wn.float().to(DEV))
        assert (got - ref).abs().max() < 5e-4, name
        scale = max(1.0, float(S.abs().max()))
        assert (state[:, :D * V].view(H, D, V) - S).abs().max() < 3e-4 * scale, name
        assert (state[:, D * V:D * V + D] - n).abs().max() < 3e-4 * scale, name
        assert (state[:, D * V + D] - mx).abs().max() < 1e-5, name


def test_router_groups_and_weights():
    """Scores made so that no choice is close: the best experts of the best groups, weights normalised and
    scaled; groups of one expert, no groups, top = experts."""
    ops = _ops()
    W = 24
    for E, top, groups, scale in ((12, 3, (4, 3), 1.5), (6, 2, (3, 1), 2.0), (6, 2, (6, 2), 1.0), (5, 2, None, 0.7), (4, 4, None, 1.0),
                                  (8, 3, (2, 1), 1.0)):
        g = torch.Generator().manual_seed(E * 10 + top)
        x = torch.randn(37, W, generator=g, dtype=F64)
        wr = torch.randn(E, W, generator=g, dtype=F64)
        r = {"experts": E, "top": top, "scale": scale}
        if groups:
            r["groups"] = {"count": groups[0], "keep": groups[1]}
        pick, weight = pg.route(x, wr, r)
        ref = torch.zeros(37, E, dtype=F64)
        ref.scatter_(1, pick, weight)
        dense, ids, wts = ops.moe_route(x.float().to(DEV), wr.float().to(DEV), top, groups, scale, lists=True)
        # a token whose choice hangs on scores closer than float32 resolves is no test of the rule
        s = torch.sigmoid(x @ wr.T)
        clear = (s[:, :, None] - s[:, None, :]).abs().add(torch.eye(E) * 9).amin(dim=(1, 2)) > 1e-4
        assert clear.sum() > 30
        assert (dense.double().cpu() - ref)[clear].abs().max() < 1e-5
        for t in torch.nonzero(clear).flatten().tolist():
            assert sorted(ids[t].tolist()) == sorted(pick[t].tolist())
        assert (wts.double().cpu().sum(-1)[clear] - scale).abs().max() < 1e-5


def test_expert_activation_and_routed_sum():
    """The whole feed-forward part against the plain code, clamps included (inputs beyond the limit on both sides)."""
    from litellmengine_b200.config.specs import FeedForwardSpec
    from litellmengine_b200.parts.feed_forward import RoutedExperts
    W, ff, E = 32, 24, 6
    g = torch.Generator().manual_seed(2)
    w = {"l0.mlp.router": torch.randn(E, W, generator=g, dtype=F64) * 0.5}
    for e in range(E):
        w[f"l0.mlp.e{e}.gate"] = torch.randn(ff, W, generator=g, dtype=F64) * 0.5
        w[f"l0.mlp.e{e}.up"] = torch.randn(ff, W, generator=g, dtype=F64) * 0.5
        w[f"l0.mlp.e{e}.down"] = torch.randn(W, ff, generator=g, dtype=F64) * 0.3
    mlp = {"expert": {"ff": ff, "limit": 1.1}, "router": {"experts": E, "top": 2, "scale": 1.7, "groups": {"count": 3, "keep": 2}}}
    x = torch.randn(50, W, generator=g, dtype=F64)
    ref = pg.moe(x, w, "l0.mlp", mlp)
    spec = FeedForwardSpec(kind="moe", intermediate_size=ff, params=(("experts", E), ("top", 2), ("groups", (3, 2)),
                                                                     ("route_scale", 1.7), ("limit", 1.1), ("expert_prefix", "e")))
    part = RoutedExperts(spec, W, torch.float32, DEV)
    part.load({n[len("l0.mlp."):]: t.float().to(DEV) for n, t in w.items()})
    for rows in (50, 3, 2):      # a prompt portion, decode steps (the last one reads only the chosen experts)
        got = _ops().as_tensor(part.forward(x[:rows].float().to(DEV).contiguous()))
        assert (got.double().cpu() - ref[:rows]).abs().max() < 2e-5
    # bfloat16: a prompt portion sorts its tokens by expert around the grouped product; a few tokens run the other ways
    wb = {n: t.to(torch.bfloat16).double() for n, t in w.items()}
    xb = x.to(torch.bfloat16).double()
    refb = pg.moe(xb, wb, "l0.mlp", mlp, act=pg.bf16_round)
    pick, _ = pg.route(xb, wb["l0.mlp.router"], mlp["router"])
    s_all = torch.sigmoid(xb @ wb["l0.mlp.router"].T)
    clear = (s_all[:, :, None] - s_all[:, None, :]).abs().add(torch.eye(E) * 9).amin(dim=(1, 2)) > 2e-3
    part16 = RoutedExperts(spec, W, torch.bfloat16, DEV)
    part16.load({n[len("l0.mlp."):]: (t.to(torch.bfloat16) if "router" not in n else t.float()).to(DEV) for n, t in w.items()})
    for rows in (50, 33, 3, 2):
        got = _ops().as_tensor(part16.forward(xb[:rows].to(torch.bfloat16).to(DEV).contiguous())).double().cpu()
        keep = clear[:rows]
        assert keep.sum() >= rows // 2
        assert (got - refb[:rows])[keep].abs().max() < 0.05 * float(refb.abs().max())


@pytest.mark.parametrize("d,window", [(64, None), (64, 70), (128, 33), (128, 200)])
def test_tensor_core_prompt_attention_with_distance_bias_and_head_gate(d, window):
    """The kernel that prompt portions of a bfloat16 run take (head sizes 64 and 128): a portion that starts in the
    middle of a page with keys before it, a table that matters, a key that would win placed just inside and just
    outside the window, a gate per head, the output as columns of a wider buffer; the step's single token goes
    through the general kernel by a row list."""
    ops = _ops()
    from litellmengine_b200.parts.attention import distance_bucket
    N, past, page, H, G, rows_, far, scale = 300, 37, 16, 4, 2, 12, 90.0, 0.2
    T = N - past
    g = torch.Generator().manual_seed(d + (window or 0))
    q, k, v = (torch.randn(N, n, d, generator=g, dtype=F64) for n in (H, G, G))
    rel = torch.randn(rows_, H, generator=g, dtype=F64) * 2
    gate = torch.randn(N, H, generator=g, dtype=F64)
    if window is not None:
        for i, off in ((299, window - 1), (298, window), (200, window - 1), (150, window)):
            k[i - off] = q[i, :G] * (2.0 if d == 64 else 1.4)
    q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    ref = pg.attention_core(q[past:], k, v, rel, scale, far, window, first_position=past) * torch.sigmoid(gate[past:])[:, :, None]
    count = int(math.ceil(far)) + 1 if window is None else min(int(math.ceil(far)) + 1, window)
    table = rel[[distance_bucket(n, rows_, far) for n in range(count)]].float().to(DEV).contiguous()
    table_t = (table.t() * math.log2(math.e)).contiguous()
    keys, values, block_table, order = _paged(N, page, G, d, d, torch.bfloat16, 2)
    cache = torch.zeros(keys.shape[0], 2, G, page, d, dtype=torch.bfloat16, device=DEV)
    _fill(cache[:, 0], cache[:, 1], order, page, k, v)
    qd = q[past:].reshape(T, -1).to(torch.bfloat16).to(DEV)
    out = torch.zeros(T, H * d + 16, dtype=torch.bfloat16, device=DEV)
    gate_buf = torch.zeros(T, 5 + H, dtype=torch.float32, device=DEV)
    gate_buf[:, 5:] = gate[past:].float().to(DEV)
    status = torch.zeros(2, dtype=torch.int32, device=DEV)
    # the portion is entry 0 (its last row left to the general kernel as if it were another entry's single token)
    tiles = _i32([(0, r0) for r0 in range(0, T - 1, ops.PREFILL_TILE_ROWS)])
    ops.paged_attention_prefill_biased(qd, out, 16, cache, tiles, tiles.shape[0], _i32([1]), _i32([0]), _i32([T - 1]), _i32([N - 1]),
                                       block_table, H, G, d, page, window, scale, status, dist_bias_t=table_t, head_gate=gate_buf,
                                       gate_off=5, out_scale=1.0)
    ops.paged_attention_generic_kv(qd, cache[:, 0], cache[:, 1], _i32(list(range(past, N))), _i32([0] * T), _i32([1]), block_table,
                                   H, G, d, d, page, window, scale, status, out, 16, gate=gate_buf, gate_off=5, dist_bias=table,
                                   gate_per_head=True, rows=_i32([T - 1, -1]))
    assert status.tolist() == [0, 0]
    got = out[:, 16:].double().cpu().view(T, H, d)
    assert (got - ref).abs().max() < 0.06
    assert float(out[:, :16].abs().max()) == 0.0
    # single tokens in the split-key decode kernel (the table joins its scores; the gate per head in the kernel after it)
    for splits in (1, 3):
        a = torch.zeros(T, H * d, dtype=torch.bfloat16, device=DEV)
        picked = [T - 1, 5, 150]
        ops.paged_attention_decode(qd, a, cache, _i32(picked + [-1]), 4, _i32(list(range(past, N))), _i32([0] * T), _i32([1]),
                                   block_table, H, G, d, page, window, scale, splits, status, dist_bias_t=table_t)
        out2 = torch.zeros(T, H * d + 16, dtype=torch.bfloat16, device=DEV)
        ops.gate_mul(a, gate_buf, 5, out2, 16, "sigmoid", 1.0, per_head=d)
        assert status.tolist() == [0, 0]
        got2 = out2[:, 16:].double().cpu().view(T, H, d)
        assert (got2[picked] - ref[picked]).abs().max() < 0.06, splits


def test_one_stream_without_connection_tensors_is_the_plain_residual():
    """`streams: 1` in a folder that stores no connection tensors: the model runs as one plainly added stream."""
    cfg, page, w = model_of("D")
    bare = {n: t for n, t in w.items() if ".hc" not in n}
    plain_cfg = {k: v for k, v in cfg.items() if k != "streams"}
    reqs = requests(cfg, [3, 41], seed=9)
    ref = Reference(plain_cfg, bare, reqs, "float32")
    steps = rh.trace_portions(reqs, seed=4)
    runner = rh.make_runner(cfg, bare, "float32", page, rh.peak_tokens(steps, round_to=page), max_requests=2)
    assert_close(rh.run_trace(runner, steps), ref, "float32", "one stream, no connection tensors")
