"""The Tobovik configuration reader, the plan it makes, and the host-side pieces the design added:
sizes that only stored tensors know, a stage that keeps pages and a state, the recurrence's work lists.
No GPU."""
import copy

import numpy as np
import pytest
import torch

import plain_tobovik as pt
import tobovik_models as tm


def test_plan_follows_the_layer_list_and_shares_weights():
    from litellmengine_b200.config import config_from_dict
    cfg = config_from_dict(tm.TOBO_A)
    plan = cfg.plan()
    assert [s.block for s in plan.order] == [0, 1, 1, 0]          # layers 1 and 3 run the tensors of 2 and 0
    assert [b.weight_prefix for b in plan.blocks] == ["l0", "l2"]
    assert plan.blocks[0].mixer.kind == "gla" and plan.blocks[0].feed_forward is None
    par = plan.blocks[1].mixer
    assert par.kind == "parallel" and [b.kind for b in par.branches] == ["gated_attention", "gla"]
    assert par.branch_scales == (1.25, 0.5)
    left = par.branches[0]
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim) == (4, 2, 16, 32)
    assert left.query_temperature == (0.4, 4) and left.qk_norm_scope == "projection" and left.bias
    assert dict(par.branches[1].params)["tau"] == 1.0
    assert plan.embedding_position.kind == "sinusoid_added" and not plan.tie_word_embeddings
    assert config_from_dict(cfg.to_dict()) == cfg


def test_tensor_names_and_shapes_are_the_designs():
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.parts.model import model_parameters
    for cfg, rank in ((tm.TOBO_A, tm.TOBO_A_RANK), (tm.TOBO_B, tm.TOBO_B_RANK), (tm.TOBO_C, tm.TOBO_C_RANK)):
        params = model_parameters(config_from_dict(cfg).plan())
        shapes = tm.tensor_shapes(cfg, rank)
        assert set(params) == set(shapes)
        for n, p in params.items():
            assert len(p.shape) == len(shapes[n]) and all(a in (-1, b) for a, b in zip(p.shape, shapes[n])), n
        # the rank of the decay projection is not in the file: it is whatever the tensors hold
        assert params["l0.mix.a1" if cfg is tm.TOBO_A else "l0.mix.right.a1"].shape[0] == -1


@pytest.mark.parametrize("change,message", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d["layers"][0].update(type="conv"), "not a mixer of this design"),
    (lambda d: d["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda d: d["layers"][2]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][2]["mlp"].update(kind="routed"), "not built"),
    (lambda d: d["layers"][1].update(weights_of=9), "must name a layer"),
    (lambda d: (d["layers"][0].update(weights_of=3)), "circle"),
])
def test_bad_configurations_are_refused_with_the_field_named(change, message):
    from litellmengine_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(tm.TOBO_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_a_size_only_the_tensor_knows():
    from litellmengine_b200.weights import DictSource, ParamSpec, RandomSource, WeightError, check_source
    params = {"a": ParamSpec((-1, 8)), "b": ParamSpec((4, -1))}
    check_source(params, DictSource({"a": torch.zeros(3, 8), "b": torch.zeros(4, 5)}))
    with pytest.raises(WeightError, match="wrong shape"):
        check_source(params, DictSource({"a": torch.zeros(3, 7), "b": torch.zeros(4, 5)}))
    with pytest.raises(ValueError, match="only known from stored weights"):
        RandomSource(params, 0, torch.float32).get("a")


def test_a_stage_keeps_pages_and_a_state():
    from litellmengine_b200.cache import CacheError, CacheManager, PagedNeed, StateNeed
    both = [PagedNeed(2, 16, None, 32), StateNeed((1, 8, 16))]
    c = CacheManager([StateNeed((3, 16, 8)), both, both, None], 4, 64, 3)
    assert sorted(c.stage_group) == [1, 2] and sorted(c.stage_state) == [0, 1, 2]
    assert len(c.groups) == 1 and c.groups[0].stages == [1, 2]
    with pytest.raises(CacheError, match="twice"):
        CacheManager([[StateNeed((1,)), StateNeed((2,))]], 4, 64, 3)


def test_recurrence_work_lists():
    from litellmengine_b200.parts.context import StepFacts
    from litellmengine_b200.parts.linear_attention import ScanWork
    work = ScanWork()
    C, F = work.CHUNK, work.CHUNKED_FROM
    q_len = np.array([1, F, 7, 2 * C * 3 + 5, F - 1], dtype=np.int64)
    facts = StepFacts(q_start=np.cumsum(q_len) - q_len, q_len=q_len, past=np.zeros(5, np.int64),
                      slot=np.arange(5, dtype=np.int32), num_tokens=int(q_len.sum()))
    out = {k: np.full(n, -7, np.int32) for k, n in work.sections(int(q_len.sum()), 5).items()}
    ns, nc, nh = work.fill(facts, out)
    assert (ns, nh) == (3, 2) and nc == F // C + 7
    short = out["short"][:4 * ns].reshape(ns, 4)
    assert short[:, 0].tolist() == [0, 2, 4] and short[:, 2].tolist() == [1, 7, F - 1]
    chunks = out["chunks"][:4 * nc].reshape(nc, 4)
    assert chunks[:, 3].tolist() == list(range(nc))                       # each chunk its own scratch
    for entry, first, n in out["chains"][:3 * nh].reshape(nh, 3).tolist():
        mine = chunks[first:first + n]
        assert (mine[:, 0] == entry).all() and int(mine[:, 2].sum()) == q_len[entry]
        assert mine[0, 1] == facts.q_start[entry] and (np.diff(mine[:, 1]) == C).all() and mine[:, 2].max() <= C


def test_plain_recurrence_carries_its_state():
    """The oracle's own consistency: a sequence in two calls with the state handed on equals one call."""
    g = torch.Generator().manual_seed(0)
    T, H, D, V = 23, 2, 5, 7
    q, k, la = (torch.randn(T, H, D, generator=g, dtype=torch.float64) for _ in range(3))
    v = torch.randn(T, H, V, generator=g, dtype=torch.float64)
    la = -la.abs()
    o, s = pt.gla_recurrence(q, k, v, la)
    o1, s1 = pt.gla_recurrence(q[:9], k[:9], v[:9], la[:9])
    o2, s2 = pt.gla_recurrence(q[9:], k[9:], v[9:], la[9:], s1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(s2, s)
    # closed form at the second token
    want = torch.einsum("hd,hd,hv->hv", q[1], torch.exp(la[1]) * k[0], v[0]) + torch.einsum("hd,hd,hv->hv", q[1], k[1], v[1])
    assert torch.allclose(o[1], want)
