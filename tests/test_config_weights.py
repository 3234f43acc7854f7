"""Configuration, registry and weight loading: what is accepted, and what the errors say."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import CONFIG_A, CONFIG_B
from mlx_lm_b200.config import ConfigError, get_architecture, get_model_classes, load_config, register_architecture
from mlx_lm_b200.models.gpt2 import ModelArgs, build
from mlx_lm_b200.parts import PagedKVSpec
from mlx_lm_b200.weights import WeightError, build_model, check_tensors, random_tensors, write_random_model


def test_args_from_config_keys():
    a = ModelArgs.from_dict(dict(CONFIG_A, some_unknown_key=3))
    assert (a.n_embd, a.n_head, a.head_dim, a.inner_width, a.n_ctx) == (64, 4, 16, 256, 128)
    b = ModelArgs.from_dict(CONFIG_B)
    assert (b.n_embd, b.n_head, b.head_dim, b.inner_width, b.layer_norm_epsilon) == (96, 3, 32, 320, 1e-6)
    assert b.num_key_value_heads == 3


def test_missing_keys_are_all_named():
    cfg = dict(CONFIG_A)
    del cfg["n_head"], cfg["vocab_size"]
    with pytest.raises(ConfigError) as e:
        ModelArgs.from_dict(cfg)
    assert "n_head" in str(e.value) and "vocab_size" in str(e.value)


@pytest.mark.parametrize("key,value,word", [("n_embd", 65, "divisible"), ("n_layer", 0, "n_layer"),
                                            ("activation_function", "swish", "gelu_new"),
                                            ("num_key_value_heads", 2, "num_key_value_heads"),
                                            ("layer_norm_epsilon", 0, "layer_norm_epsilon"), ("n_inner", -4, "n_inner")])
def test_bad_values_name_the_key(key, value, word):
    with pytest.raises(ConfigError) as e:
        ModelArgs.from_dict(dict(CONFIG_A, **{key: value}))
    assert word in str(e.value)


def test_registry():
    arch = get_architecture({"model_type": "gpt2"})
    assert arch.args_class is ModelArgs and arch.build is build
    assert get_model_classes({"model_type": "gpt2"}) == (build, ModelArgs)
    with pytest.raises(ValueError) as e:
        get_architecture({"model_type": "no_such_model"})
    assert "Model type no_such_model not supported" in str(e.value)
    with pytest.raises(ConfigError):
        register_architecture("gpt2", ModelArgs, build)


def test_description_follows_the_configuration():
    d = build(ModelArgs.from_dict(CONFIG_B))
    assert len(d.blocks) == 3 and [e.block for e in d.order] == [0, 1, 2]
    assert d.cache_specs() == {i: PagedKVSpec(3, 32, None) for i in range(3)}
    specs = {s.name: s.shape for s in d.param_specs()}
    assert specs["h.1.attn.c_attn.weight"] == (96, 288)          # HF Conv1D layout [in, out]
    assert specs["h.2.mlp.c_fc.weight"] == (96, 320) and specs["h.2.mlp.c_proj.weight"] == (320, 96)
    assert specs["wte.weight"] == (1000, 96) and specs["wpe.weight"] == (256, 96)
    assert "lm_head.weight" not in specs                          # tied head
    assert d.max_positions == 256
    assert set(d.kernel_libs()) >= {"embed", "norm", "attention"}


def test_generation_config_overrides_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(CONFIG_A, eos_token_id=1)))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 6]}))
    assert load_config(str(tmp_path))["eos_token_id"] == [5, 6]
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nowhere"))


def test_random_folder_round_trip(tmp_path):
    write_random_model(str(tmp_path), dict(CONFIG_B), seed=7)
    again = tmp_path / "again"
    write_random_model(str(again), dict(CONFIG_B), seed=7)
    a, b = load_file(str(tmp_path / "model.safetensors")), load_file(str(again / "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert all(t.dtype == torch.bfloat16 for t in a.values())
    other = random_tensors(build(ModelArgs.from_dict(CONFIG_B)), seed=8)
    assert not torch.equal(other["wte.weight"], a["wte.weight"])
    gains = a["h.0.ln_1.weight"].float()
    assert 0.05 < float(gains.std()) < 0.2 and abs(float(gains.mean()) - 1) < 0.1     # ln_gain_std = 0.1
    ones = random_tensors(build(ModelArgs.from_dict(CONFIG_A)), seed=1)["ln_f.weight"]
    assert torch.equal(ones.float(), torch.ones(64))
    assert abs(float(a["wte.weight"].float().std()) - 0.02) < 0.002


def test_dtypes_on_load():
    d = build(ModelArgs.from_dict(CONFIG_A))
    t = random_tensors(d, seed=0)
    t = {"transformer." + k: v for k, v in t.items()}                 # a prefix is accepted
    t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 4, 4)           # the mask buffer is dropped
    t["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    for dtype in (torch.bfloat16, torch.float32):
        m = build_model(dict(CONFIG_A), t, dtype=dtype, device="cpu")
        blk = m.description.blocks[0]
        assert blk.mixer.qkv.weight.dtype == dtype and blk.mixer.qkv.weight.shape == (192, 64)   # [out, in]
        assert blk.mixer.qkv.bias.dtype == torch.float32 and blk.norm_1.gain.dtype == torch.float32
        assert m.description.embedding.table.dtype == dtype
        assert m.description.head.linear.weight is m.description.embedding.table
        # the transposed copy equals the file's [in, out] tensor
        assert torch.equal(blk.mixer.qkv.weight.float().t(), t["transformer.h.0.attn.c_attn.weight"].float())


def test_one_error_lists_missing_unexpected_and_shapes():
    d = build(ModelArgs.from_dict(CONFIG_A))
    t = random_tensors(d, seed=0)
    del t["h.1.ln_2.bias"], t["wpe.weight"]
    t["h.0.attn.c_proj.weight"] = torch.zeros(64, 63)
    t["lm_head.weight"] = torch.zeros(512, 64)
    t["h.0.mlp.extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        check_tensors(d, t)
    msg = str(e.value)
    for word in ("missing (2)", "h.1.ln_2.bias", "wpe.weight", "unexpected (2)", "lm_head.weight", "h.0.mlp.extra",
                 "wrong shape (1)", "h.0.attn.c_proj.weight is (64, 63), expected (64, 64)"):
        assert word in msg, word


def test_custom_get_model_classes():
    """A caller may hand over its own (builder, args class) lookup, as mlx-lm's load_model allows
    (tests/test_utils.py:109-136 there)."""
    seen = []

    def mine(config):
        seen.append(config["model_type"])
        return build, ModelArgs

    t = random_tensors(build(ModelArgs.from_dict(CONFIG_A)), seed=0)
    m = build_model(dict(CONFIG_A, model_type="something_else"), t, dtype=torch.float32, device="cpu",
                    get_model_classes=mine)
    assert seen == ["something_else"] and len(m.layers) == 2


def test_no_safetensors(tmp_path):
    from mlx_lm_b200.weights import read_safetensors
    with pytest.raises(FileNotFoundError) as e:
        read_safetensors(str(tmp_path))
    assert "No safetensors found" in str(e.value)
