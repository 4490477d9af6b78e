"""Sugizen without a GPU: reading its configuration, the tensors it asks for, a model folder written
from a seed, and the cache's bookkeeping for a run with two kinds of state."""
import copy
import os

import pytest

from sugizen_configs import CONFIGS, MIXED


def test_configuration_reads_writes_and_refuses():
    import ultima_b200 as u
    from ultima_b200.config import SugizenConfig
    cfg = u.config_from_dict(MIXED)
    assert isinstance(cfg, SugizenConfig) and cfg.architecture == "Sugizen"
    assert [L.mixer.kind for L in cfg.layers] == [L["type"] for L in MIXED["layers"]]
    assert cfg.layers[2].mixer.kv_from == 0 and cfg.layers[3].mlp is None and cfg.layers[0].mixer.block == 24
    assert cfg.layers[0].mixer.rot.scaling == (8.0, 1.0, 3.0, 64.0)
    assert u.config_from_dict(cfg.to_dict()) == cfg
    for path, value in ((("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "heads"), 3), (("width",), 0),
                        (("layers", 2, "mixer", "kv_from"), 1), (("layers", 2, "mixer", "kv_from"), 2),
                        (("layers", 2, "mixer", "dim"), 48), (("layers", 1, "mlp", "kind"), "experts"),
                        (("layers", 0, "mixer", "rot", "dims"), 34), (("norm",), None)):
        bad = copy.deepcopy(MIXED)
        d = bad
        for k in path[:-1]:
            d = d[k]
        d[path[-1]] = value
        with pytest.raises(u.ConfigError):
            u.config_from_dict(bad)


def test_the_model_asks_for_the_tensors_its_layers_have():
    import ultima_b200 as u
    spec = u.model_spec_for(u.config_from_dict(MIXED))
    shapes = {s.name: tuple(s.shape) for s in spec.weight_specs()}
    assert shapes["embed"] == (300, 64) and shapes["head"] == (300, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (128, 64) and shapes["l0.mix.k"] == (64, 64) and shapes["l0.mix.v"] == (32, 64)
    assert shapes["l0.mix.g"] == (4, 64) and shapes["l0.mix.o"] == (64, 64) and shapes["l0.mix.q.norm"] == (32,)
    # a layer that reads another's keys and values has none of their tensors
    assert "l2.mix.q" in shapes and not any(n in shapes for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm"))
    assert shapes["l1.mix.a1"] == (5, 64) and shapes["l1.mix.a2"] == (96, 5) and shapes["l1.mix.g2"] == (160, 7)
    assert shapes["l1.mix.q.conv"] == (48, 3) and shapes["l1.mix.v.conv"] == (160, 3) and shapes["l1.mix.A_log"] == (4,)
    assert shapes["l1.mix.norm"] == (40,) and shapes["l1.mix.dt_bias"] == (96,) and shapes["l1.mix.b"] == (4, 64)
    # no feed-forward: no tensors of it and no second norm
    assert "l3.norm1" in shapes and not any(n.startswith("l3.mlp") or n == "l3.norm2" for n in shapes)
    assert [(r.layer, r.cache_from) for r in spec.runs] == [(0, None), (1, None), (2, 0), (3, None), (4, 0)]


def test_low_rank_sizes_come_from_the_stored_shapes(tmp_path):
    import json
    import ultima_b200 as u
    from ultima_b200.weights import check_weights
    cfg = u.config_from_dict(MIXED)
    d = str(tmp_path / "m")
    u.write_random_model(d, cfg, seed=3, dtype="bfloat16")
    with open(os.path.join(d, "config.json")) as f:
        stored = json.load(f)
    for L in stored["layers"]:
        L["mixer"].pop("decay_rank", None)
        L["mixer"].pop("gate_rank", None)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(stored, f)
    bare = u.config_from_dict(stored)
    assert bare.needs_tensor_shapes
    with pytest.raises(ValueError):
        u.model_spec_for(bare)
    read = u.config_from_dir(d)
    assert not read.needs_tensor_shapes and read.layers[1].mixer.decay_rank == 5 and read.layers[1].mixer.gate_rank == 7
    assert len(check_weights(d, u.model_spec_for(read).weight_specs())) == len(u.model_spec_for(cfg).weight_specs())


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_configuration_of_the_tests_builds(name):
    import ultima_b200 as u
    spec = u.model_spec_for(u.config_from_dict(CONFIGS[name]))
    assert len(spec.layers) == len(CONFIGS[name]["layers"]) and len(spec.weight_specs()) > 10


def test_a_run_with_two_states_gets_both_and_they_start_at_zero():
    import torch
    from ultima_b200.cache import Cache
    from ultima_b200.parts.base import KVNeed, StateNeed
    a, b = StateNeed((2, 3, 5), "float32"), StateNeed((1, 7), "float32")
    kv = KVNeed(2, 8, None, 4)
    cache = Cache([(a, b), kv, None, (a, b)], [None, None, 1, None], max_tokens=256, max_context=128, n_slots=3,
                  step_chunk=64, dtype=torch.float32, device="cpu")
    s0 = cache.acquire()
    rc = cache.run_cache(0, [t for t in map(torch.from_numpy, cache.tables([s0]))])
    assert [tuple(t.shape) for t in rc.states] == [(3, 2, 3, 5), (3, 1, 7)] and rc.state is rc.states[0]
    rc.states[0][s0].fill_(1.0)
    rc.states[1][s0].fill_(2.0)
    other = cache.run_cache(3, [])
    assert float(other.states[0].abs().sum()) == 0.0                 # the other run's state is its own
    cache.release(s0)
    assert cache.acquire() == s0                                      # the slot comes again ...
    assert float(cache.run_cache(0, []).states[0][s0].abs().sum()) == 0.0 and \
        float(cache.run_cache(0, []).states[1][s0].abs().sum()) == 0.0         # ... with its state cleared
    g = cache.kv_groups[0]
    assert tuple(g.k.shape[2:]) == (2, 64, 8) and tuple(g.v.shape[2:]) == (2, 64, 4)
    shared = cache.run_cache(2, [torch.zeros(1, 2, dtype=torch.int32)])
    assert shared.kv is not None and not shared.kv.owner and shared.kv.k.data_ptr() == g.k[0].data_ptr()
    # a run may name the same need twice (two convolutions over channels of one width): two arrays of one group
    twice = Cache([(a, a)], [None], 64, 64, 1, 64).run_cache(0, [])
    assert len(twice.states) == 2 and twice.states[0].data_ptr() != twice.states[1].data_ptr()
