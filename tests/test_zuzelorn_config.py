"""The Zuzelorn configuration class: what it reads, what it refuses, and the
model it describes (no GPU needed)."""
import copy

import pytest

from janas_b200.config import ConfigError, ZuzelornConfig, config_from_dict, known_architectures
from janas_b200.weights import expected_tensors
from zuzelorn_models import CONFIGS, tensor_shapes


def test_registered():
    assert "Zuzelorn" in known_architectures()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_list_matches_the_design(name):
    c = config_from_dict(CONFIGS[name])
    assert isinstance(c, ZuzelornConfig)
    assert c.to_dict()["layers"][0]["mixer"]["vdim"] == CONFIGS[name]["layers"][0]["mixer"]["vdim"]
    got = {n: tuple(s.shape) for n, s in expected_tensors(c.to_model_spec()).items() if not s.optional}
    assert got == {n: tuple(s) for n, s in tensor_shapes(CONFIGS[name]).items()}


def test_spec_describes_the_layers():
    spec = config_from_dict(CONFIGS["ZA"]).to_model_spec()
    assert [e.cache_of for e in spec.run_order] == [None, 0, None, 2]
    assert spec.position_table_name == "pos" and spec.logit_scale == 0.7
    l2 = spec.layers[2]
    assert l2.block == "sandwich" and l2.feed_forward is None and l2.ffn_norm is None
    assert l2.post_mixer_norm.kind == "dynamic_tanh"
    assert spec.layers[1].mixer.get("own_kv") is False and spec.layers[0].mixer.get("own_kv") is True
    assert spec.layers[0].mixer.get("v_head_dim") == 32
    spec.validate()


def bad(change):
    c = copy.deepcopy(CONFIGS["ZA"])
    change(c)
    with pytest.raises(ConfigError):
        config_from_dict(c)


def test_refusals():
    bad(lambda c: c["layers"][1]["mixer"].update(kv_from=3))             # a later layer
    bad(lambda c: c["layers"][3]["mixer"].update(kv_from=1))             # a layer that owns none
    bad(lambda c: c["layers"][1]["mixer"].update(vdim=16))               # other sizes than its source
    bad(lambda c: c["layers"][0].update(type="recurrent"))
    bad(lambda c: c["layers"][0]["mlp"].update(kind="routed"))
    bad(lambda c: c["layers"][0]["mixer"].update(heads=3))
    bad(lambda c: c.pop("width"))
    bad(lambda c: c["norm"].pop("eps"))


def test_random_model_folder(tmp_path):
    """The folder writer makes a model of the design that the loader accepts as a whole."""
    import torch
    from janas_b200.config import config_from_dir
    from janas_b200.weights import check_folder, list_folder, write_random_model
    c = config_from_dict(CONFIGS["ZD"])
    write_random_model(str(tmp_path), c, seed=3, dtype=torch.bfloat16)
    back = config_from_dir(str(tmp_path))
    assert back.to_dict() == c.to_dict()
    check_folder(str(tmp_path), expected_tensors(back.to_model_spec()))
    have = list_folder(str(tmp_path))
    assert have["l0.norm1.alpha"][1] == () and have["l2.mix.q"][1] == (6 * 24, 50) and "l2.mix.k" not in have
