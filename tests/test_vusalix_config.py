"""Vusalix without a GPU: the configuration read and written back, refusals that name the key, the model as data
(arrangements, parts, tensor names, cache needs), and a random model folder that the plain reader takes."""
import copy

import pytest

from vusalix_configs import CONFIGS, MIXED, PLAIN


def test_configuration_reads_and_writes_back():
    import ultima_b200 as u
    for name, raw in CONFIGS.items():
        cfg = u.config_from_dict(raw)
        assert cfg.architecture == "Vusalix" and len(cfg.layers) == len(raw["layers"])
        again = u.config_from_dict(cfg.to_dict())
        assert again == cfg, name
    cfg = u.config_from_dict(MIXED)
    assert cfg.streams == 3 and cfg.layers[1].mixer.window == 40 and cfg.layers[1].mixer.softcap == 15.0
    assert cfg.layers[2].mixer.scaling.factor == 8.0 and cfg.layers[0].mlp.groups == (4, 2) and cfg.layers[0].mlp.identity == 2
    assert cfg.layers[3].mlp is None and u.config_from_dict(PLAIN).streams is None


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "heads"), 5, "kv_heads"),
    (("layers", 2, "mixer", "rot", "dims"), 18, "rot.dims"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("norm",), 1e-5, "norm"), (("streams",), 0, "streams"), (("layers", 1, "mixer", "mask"), 7, "mask")])
def test_refusals_name_the_key(path, value, word):
    import ultima_b200 as u
    raw = copy.deepcopy(MIXED)
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(u.ConfigError) as e:
        u.config_from_dict(raw)
    assert word in str(e.value)


def test_the_bucket_count_comes_from_the_stored_table():
    import ultima_b200 as u
    raw = copy.deepcopy(MIXED)
    del raw["layers"][1]["mixer"]["buckets"]
    cfg = u.config_from_dict(raw)
    assert cfg.needs_tensor_shapes
    with pytest.raises(u.ConfigError):
        cfg.with_tensor_shapes({})
    full = cfg.with_tensor_shapes({"l1.mix.rel": (12, 4)})
    assert not full.needs_tensor_shapes and full.layers[1].mixer.buckets == 12


def test_the_model_as_data():
    import ultima_b200 as u
    from ultima_b200.arch import model_spec_for
    from ultima_b200.parts.base import KVNeed, StateNeed, build_part
    spec = model_spec_for(u.config_from_dict(MIXED))
    assert spec.streams == 3 and [L.arrangement.kind for L in spec.layers] == ["hyper_pre_norm"] * 3 + ["hyper_pre_norm_mixer_only"] * 2
    names = {w.name: tuple(w.shape) for w in spec.weight_specs()}
    assert names["l0.mix.a"] == (4, 64) and names["l0.mix.g"] == (160, 64) and names["l0.mix.dt_bias"] == (4,)
    assert names["l1.mix.rel"] == (12, 4) and names["l1.mix.sink"] == (4,) and names["l1.hc1.mix"] == (3, 3)
    assert names["l2.mix.dkv"] == (48, 64) and names["l2.mix.uk"] == (64, 32) and names["l2.mix.uv"] == (96, 32)
    assert names["l0.mlp.router"] == (8, 64) and names["l0.mlp.correction"] == (8,) and names["l0.mlp.e5.down"] == (64, 32)
    assert "l0.mlp.e6.gate" not in names and names["l0.mlp.shared.up"] == (48, 64) and "l2.mlp.shared.up" not in names
    assert "l3.norm2" not in names and "l3.hc2.in" not in names and names["l3.hc1.out"] == (3,)
    need = build_part("mixer", spec.layers[2].part("mixer")).cache_need()
    assert need == KVNeed(1, 48, 50, values_in_keys=True)
    assert build_part("mixer", spec.layers[1].part("mixer")).cache_need() == KVNeed(2, 32, 40, 16)
    delta = build_part("mixer", spec.layers[0].part("mixer")).cache_need()
    assert delta == (StateNeed((4, 24, 40), "float32"), StateNeed((2, 2 * 2 * 24 + 4 * 40), "float32"))
    plain = model_spec_for(u.config_from_dict(PLAIN))
    assert plain.streams == 0 and [L.arrangement.kind for L in plain.layers] == ["pre_norm", "pre_norm_mixer_only", "pre_norm"]


def test_a_random_folder_is_read_by_the_plain_reader(tmp_path):
    import plain_vusalix as P
    import ultima_b200 as u
    d = u.write_random_model(str(tmp_path / "m"), u.config_from_dict(PLAIN), seed=3, dtype="bfloat16")
    cfg, W = P.read_folder(d)
    assert cfg["architecture"] == "Vusalix" and W["l0.mix.rel"].shape == (6, 3) and W["l2.mix.dkv.norm"].shape == (24,)
    out = P.logits(cfg, W, [1, 2, 3, 4, 5])
    assert out.shape == (5, 130) and abs(out).max() > 0
    # the folder's own configuration, with the bucket count taken from the table when the key is absent
    import json, os
    raw = json.load(open(os.path.join(d, "config.json")))
    del raw["layers"][0]["mixer"]["buckets"]
    json.dump(raw, open(os.path.join(d, "config.json"), "w"))
    assert u.config_from_dir(d).layers[0].mixer.buckets == 6


def test_the_bench_models_are_configurations_of_equal_active_size():
    """The models that ``bench.py --only vusalix`` times: a Vusalix whose chosen and shared experts together have the dense
    models' inner size, and whose latent layers' key row is one the tensor-core attention takes."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    import ultima_b200 as u
    for z in bench.SUGIZEN_SIZES.values():
        cfg = u.config_from_dict(bench.vusalix_config(z))
        spec = u.model_spec_for(cfg)
        assert spec.streams == 2 and len(cfg.layers) == z["layers"]
        kinds = [L.kind for L in cfg.layers]
        assert set(kinds) == {"attention", "delta", "latent_attention"}
        for L in cfg.layers:
            f = L.mlp
            assert f.top * f.ff + f.shared_ff == z["ff"]
            if L.kind == "latent_attention":
                assert L.mixer.kv_rank + L.mixer.rot_dim == 256
