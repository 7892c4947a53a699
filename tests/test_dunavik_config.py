"""The Dunavik configuration class: what it reads, what it refuses, and the model
it describes (no GPU needed)."""
import copy

import pytest

from janas_b200.config import ConfigError, DunavikConfig, config_from_dict, known_architectures
from janas_b200.weights import expected_tensors
from dunavik_models import CONFIGS, tensor_shapes
import plain_dunavik as pd


def test_registered():
    assert "Dunavik" in known_architectures()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_list_matches_the_design(name):
    c = config_from_dict(CONFIGS[name])
    assert isinstance(c, DunavikConfig)
    got = {n: tuple(s.shape) for n, s in expected_tensors(c.to_model_spec()).items() if not s.optional}
    assert got == {n: tuple(s) for n, s in tensor_shapes(CONFIGS[name]).items()}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_follows_the_loop(name):
    spec = config_from_dict(CONFIGS[name]).to_model_spec()
    assert [e.layer for e in spec.run_order] == pd.run_order(CONFIGS[name])
    lp = CONFIGS[name].get("loop")
    adds = [i for i, e in enumerate(spec.run_order) if e.add_embedding]
    if lp is None:
        assert adds == []
    else:
        span = lp["stop"] - lp["start"]
        assert adds == [lp["start"] + p * span for p in range(1, lp["times"])]
    assert all(e.cache_of is None for e in spec.run_order)


def test_spec_describes_the_layers():
    spec = config_from_dict(CONFIGS["DA"]).to_model_spec()
    assert spec.embedding_norm.kind == "layernorm" and spec.embedding_norm_name == "embed.norm"
    l0, l1, l2 = spec.layers[0], spec.layers[1], spec.layers[2]
    assert l0.block == "parallel" and l0.block_params["residual_mult"] == 0.5
    assert l0.mixer.kind == "latent_attention" and l0.mixer.get("kv_rank") == 40 and l0.mixer.get("rot_dim") == 8
    assert l0.mixer.get("position").kind == "rope_pairs"
    assert l1.mixer.kind == "sink_attention" and l1.mixer.get("window") == 37 and l1.mixer.get("softcap") == 20.0
    assert l1.mixer.get("q_temp_every") == 16 and l1.mixer.get("distance_slope_exponent") == 8.0
    assert l1.feed_forward.kind == "dense" and l1.feed_forward.get("activation") == "relu2"
    assert l1.ffn_norm is None and l2.feed_forward is None
    spec.validate()
    # what a layer leaves out is off: no window, no cap, no temperature
    plain = config_from_dict(CONFIGS["DB"]).to_model_spec().layers[2].mixer
    assert plain.get("window") == 0 and plain.get("softcap") is None and plain.get("q_temp_every") is None


def test_round_trip():
    for name, c in CONFIGS.items():
        d = config_from_dict(c).to_dict()
        assert config_from_dict(d).to_dict() == d
        assert d["layers"] == c["layers"] and d["residual_mult"] == c["residual_mult"]


def bad(change, name="DA"):
    c = copy.deepcopy(CONFIGS[name])
    change(c)
    with pytest.raises(ConfigError):
        config_from_dict(c)


def test_refusals():
    bad(lambda c: c["layers"][0].update(type="recurrent"))
    bad(lambda c: c["layers"][0]["mlp"].update(kind="routed"))
    bad(lambda c: c["layers"][1]["mixer"].update(heads=3))               # no multiple of kv_heads
    bad(lambda c: c["layers"][0]["mixer"].pop("kv_rank"))
    bad(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10))        # more than rot_dim
    bad(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3))         # odd
    bad(lambda c: c["layers"][0]["mixer"].update(kv_rank=510))           # rows beyond the kernels' 512
    bad(lambda c: c["layers"][1]["mixer"]["mask"].update(size=0))
    bad(lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0))
    bad(lambda c: c["loop"].update(stop=9))
    bad(lambda c: c["loop"].update(start=3, stop=1))
    bad(lambda c: c["loop"].update(times=0))
    bad(lambda c: c.pop("width"))
    bad(lambda c: c["norm"].pop("eps"))


def test_random_model_folder(tmp_path):
    """The folder writer makes a model of the design that the loader accepts as a whole."""
    import torch
    from janas_b200.config import config_from_dir
    from janas_b200.weights import check_folder, list_folder, write_random_model
    c = config_from_dict(CONFIGS["DB"])
    write_random_model(str(tmp_path), c, seed=3, dtype=torch.bfloat16)
    back = config_from_dir(str(tmp_path))
    assert back.to_dict() == c.to_dict()
    check_folder(str(tmp_path), expected_tensors(back.to_model_spec()))
    have = list_folder(str(tmp_path))
    assert have["l0.mix.dkv"][1] == (22 + 6, 50) and have["l0.mix.uk"][1] == (3 * 10, 22)
    assert have["embed.norm.b"][1] == (50,) and "l2.mlp.up" not in have
