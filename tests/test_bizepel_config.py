"""Bizepel without a GPU: configuration reading and refusals, the model as data, tensor names, random folders."""
import copy
import json
import os

import pytest
import torch

import ultima_b200 as u
from ultima_b200.config import BizepelConfig, ConfigError, config_from_dict, config_from_dir
from ultima_b200.arch import model_spec_for

from bizepel_configs import CONFIGS, MIXED, ODD, PLAIN


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_configuration_reads_writes_and_reads_back(name):
    cfg = config_from_dict(CONFIGS[name])
    assert isinstance(cfg, BizepelConfig) and cfg.architecture == "Bizepel"
    again = config_from_dict(cfg.to_dict())
    assert again == cfg
    assert len(cfg.layers) == len(CONFIGS[name]["layers"])


def test_absent_keys_switch_their_mechanism_off():
    cfg = config_from_dict(PLAIN)
    assert cfg.canon_taps == 0 and cfg.side_dim == 0 and cfg.logit_scale == 1.0
    a = cfg.layers[0].mixer
    assert a.conv == 0 and a.window is None and a.keep_first == 0 and not a.v_mix and a.rot_dims == 8
    spec = model_spec_for(cfg)
    kinds = {r: ps.kind for r, ps in spec.layers[0].parts}
    assert kinds["mixer_filter"] == "none" and kinds["tail"] == "none" and "feed_forward" not in kinds
    odd = config_from_dict(ODD)
    assert odd.layers[1].mixer.rot_dims is None and odd.layers[1].mixer.keep_first == 0 and odd.layers[1].mlp.scale == 0.5
    assert odd.layers[2].mlp.groups == (3, 3) and odd.layers[1].mlp.groups is None


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), 0, "vocab"), (("norm",), None, "norm"), (("layers",), [], "layers"),
    (("layers", 1, "type"), "conv", "type"), (("layers", 1, "mixer", "heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "conv"), 17, "conv"),
    (("layers", 0, "mlp", "router", "top"), 9, "top"), (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "kind"), "glu", "kind"), (("canon", "taps"), 40, "taps"), (("layers", 2, "mixer", "state"), "x", "state"),
    (("layers", 3, "mixer", "vdim"), 8, "v_mix"),
])
def test_refusals_name_the_key(path, value, word):
    raw = copy.deepcopy(MIXED)
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_the_model_as_data_names_every_stored_tensor():
    spec = model_spec_for(config_from_dict(MIXED))
    names = {s.name: tuple(s.shape) for s in spec.weight_specs()}
    for n, shape in {"embed": (300, 64), "embed.norm": (64,), "side.embed": (300, 5 * 8), "final.norm": (64,),
                     "l0.mix.r": (48, 64), "l0.mix.w1": (5, 64), "l0.mix.w2": (48, 5), "l0.mix.w0": (48,), "l0.mix.a.b": (48,),
                     "l0.mix.norm": (48,), "l0.mlp.router": (6, 64), "l0.mlp.correction": (6,), "l0.mlp.e5.up": (24, 64),
                     "l0.mlp.shared.down": (64, 40), "l0.ls1": (64,), "l0.canon2": (64, 3), "l0.side.gate": (8, 64),
                     "l0.side.proj": (64, 8), "l0.side.norm": (64,), "l1.mix.q.b": (128,), "l1.mix.k.conv": (64, 3),
                     "l1.mix.v.conv": (32, 3), "l1.mix.q.norm": (32,), "l1.mix.vmix": (), "l1.mlp.up": (96, 64),
                     "l2.mix.in": (192, 64), "l2.mix.conv.b": (96,), "l2.mix.x": (6 + 20, 96), "l2.mix.dt": (96, 6),
                     "l2.mix.A_log": (96, 10), "l2.mix.D": (96,), "l4.mix.vmix": (), "l4.norm1": (64,)}.items():
        assert names.get(n) == shape, (n, names.get(n))
    assert "head.weight" not in names and "l4.norm2" not in names and "l4.ls2" not in names
    assert sum(1 for n in names if n == "side.embed") == 1
    # what a file may carry without the model having a use for it: the second sublayer's tensors of a layer without one
    assert set(spec.optional_tensors) == {"l4.norm2", "l4.canon2", "l4.ls2"}
    # the first layer that mixes values hands them out, the later ones blend
    mixes = [dict(L.parts)["mixer"].get("value_mix") for L in spec.layers]
    assert mixes == [None, "source", None, "blend", "blend"]


def test_a_general_delta_layer_takes_its_rank_from_the_stored_matrix(tmp_path):
    cfg = config_from_dict(MIXED)
    d = u.write_random_model(str(tmp_path / "m"), cfg, seed=3, dtype="bfloat16")
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    del raw["layers"][0]["mixer"]["decay_rank"]
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    assert config_from_dict(raw).needs_tensor_shapes
    with pytest.raises(ValueError):
        model_spec_for(config_from_dict(raw))
    assert config_from_dir(d).layers[0].mixer.decay_rank == 5
    assert config_from_dir(d) == cfg


def test_a_random_folder_reads_back_with_the_plain_reader_and_runs_in_the_plain_implementation(tmp_path):
    import plain_bizepel as P
    d = u.write_random_model(str(tmp_path / "m"), config_from_dict(PLAIN), seed=5, dtype="bfloat16")
    cfg, W = P.read_folder(d)
    spec = model_spec_for(config_from_dir(d))
    assert set(W) == {s.name for s in spec.weight_specs()}
    lg = P.logits(cfg, W, [1, 5, 7, 2, 9])
    assert lg.shape == (5, 130) and bool(torch.isfinite(torch.from_numpy(lg)).all())
    # causal: a prefix gives the same logits
    assert abs(P.logits(cfg, W, [1, 5, 7])[2] - lg[2]).max() < 1e-9
