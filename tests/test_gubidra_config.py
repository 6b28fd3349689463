"""The Gubidra configuration reader on the CPU: the plan it writes, the run order of a looped span, the
tensors the model asks for, what it refuses, and the distance table's rule."""
import copy

import pytest

import gubidra_models as gm
import plain_gubidra as pg
from litellmengine_b200.cache import PagedNeed, StateNeed
from litellmengine_b200.config import ConfigError, config_from_dict
from litellmengine_b200.parts.model import Model, model_parameters


@pytest.mark.parametrize("cfg", [gm.GUBI_A, gm.GUBI_B, gm.GUBI_C, gm.GUBI_D])
def test_plan_names_sizes_and_order(cfg):
    c = config_from_dict(cfg)
    plan = c.plan()
    assert [s.block for s in plan.order] == gm.run_order(cfg) == pg.run_order(cfg)
    assert plan.streams == (cfg.get("streams") or 0) and plan.embedding_scale == cfg["embedding"]["scale"]
    params = model_parameters(plan)
    shapes = gm.tensor_shapes(cfg)
    assert set(params) == set(shapes)
    for n, p in params.items():
        assert all(a in (-1, b) for a, b in zip(p.shape, shapes[n])), n
    assert config_from_dict(c.to_dict()).to_dict() == c.to_dict()
    kinds = {"attention": "gated_attention", "retention": "retention", "mlstm": "mlstm"}
    for b, e in zip(plan.blocks, cfg["layers"]):
        assert b.mixer.kind == kinds[e["type"]] and (b.feed_forward is None) == (e["mlp"] is None)
        assert b.arrangement == ("hyper_pre_norm" if cfg.get("streams") else "pre_norm")


def test_each_pass_of_a_loop_has_its_own_cache_and_state():
    model = Model(config_from_dict(gm.GUBI_A).plan(), dtype="float32", device="meta")
    needs = model.stage_needs()
    assert len(needs) == 6                                   # 0, then (1, 2) twice, then 3
    assert isinstance(needs[0], PagedNeed) and needs[0].window == 9 and needs[0].value_dim == 24
    assert needs[1] == needs[3] and isinstance(needs[1], StateNeed) and needs[1].shape == (3, 8 * 16)
    assert needs[2] == needs[4] and needs[2].shape == (2, 16 * 9 + 1)          # S, the normaliser, the maximum
    full = Model(config_from_dict(gm.GUBI_B).plan(), dtype="float32", device="meta").stage_needs()
    assert full[1].window is None and full[1].value_dim is None and full[2].window == 21


def _changed(cfg, path, value):
    d = copy.deepcopy(cfg)
    at = d
    for key in path[:-1]:
        at = at[key]
    if value is KeyError:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return d


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "convolution"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "scale"), KeyError),
    (("layers", 1, "mixer", "decay"), [0.5]), (("layers", 1, "mixer", "decay"), [0.5, 1.5, 0.2]), (("layers", 1, "mixer", "rot", "dims"), 5),
    (("layers", 1, "mixer", "rot", "dims"), 10), (("layers", 2, "mixer", "gate_cap"), 0.0), (("layers", 0, "mlp", "kind"), "dense"),
    (("layers", 0, "mlp", "router", "top"), 7), (("layers", 0, "mlp", "router", "groups", "count"), 4),
    (("layers", 0, "mlp", "router", "groups", "keep"), 0), (("loop", "stop"), 9), (("loop", "times"), 0), (("streams",), 9),
    (("norm", "eps"), 0.0), (("embedding", "scale"), "big"), (("vocab",), KeyError)])
def test_refused_configurations(path, value):
    with pytest.raises(ConfigError):
        config_from_dict(_changed(gm.GUBI_A, path, value))


def test_options_that_may_be_absent():
    d = _changed(_changed(_changed(gm.GUBI_A, ("loop",), KeyError), ("streams",), KeyError), ("layers", 0, "mixer", "mask"), KeyError)
    d = _changed(_changed(d, ("layers", 1, "mixer", "rot"), KeyError), ("layers", 0, "mlp", "router", "groups"), KeyError)
    plan = config_from_dict(d).plan()
    assert [s.block for s in plan.order] == [0, 1, 2, 3] and plan.streams == 0
    assert plan.blocks[0].mixer.window is None and plan.blocks[1].mixer.position.kind == "none"
    assert dict(plan.blocks[0].feed_forward.params)["groups"] is None
    rows_unknown = config_from_dict(_changed(gm.GUBI_A, ("layers", 0, "mixer", "bias_rows"), KeyError)).plan()
    assert rows_unknown.blocks[0].mixer.distance_bias == (-1, 40.0)           # only the stored table knows


def test_one_stream_may_come_without_connection_tensors():
    from litellmengine_b200.weights import DictSource
    from litellmengine_b200.weights.loader import WeightError, check_source
    w = gm.random_weights(gm.GUBI_D, 1)
    params = model_parameters(config_from_dict(gm.GUBI_D).plan())
    check_source(params, DictSource({n: t for n, t in w.items() if ".hc" not in n}))
    two = gm.random_weights(gm.GUBI_A, 1)
    with pytest.raises(WeightError):          # several streams need theirs
        check_source(model_parameters(config_from_dict(gm.GUBI_A).plan()), DictSource({n: t for n, t in two.items() if ".hc" not in n}))
