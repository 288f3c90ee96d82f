"""Configuration, registry, safetensors IO, weight errors, random weights (no GPU)."""

from __future__ import annotations

import json

import pytest
import torch

from research_2_b200.config import ConfigError, GPT2Config, architecture, known_architectures, load_config
from research_2_b200.config.engine_options import EngineOptions
from research_2_b200.models import gpt2 as gpt2_model
from research_2_b200.weights import (
    WeightError, check_and_select, load_weights, read_file, write_file, write_model_folder,
)
from tests.helpers import TINY_A, TINY_B


def test_registry_knows_gpt2_and_names_unknown():
    assert "GPT2LMHeadModel" in known_architectures()
    assert architecture("GPT2LMHeadModel").name == "GPT2LMHeadModel"
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*GPT2LMHeadModel"):
        architecture("LlamaForCausalLM")


def test_config_reads_every_key():
    a = GPT2Config.from_json(TINY_A["config"])
    b = GPT2Config.from_json(TINY_B["config"])
    assert (a.n_layer, a.n_embd, a.n_head, a.head_dim, a.n_inner, a.vocab_size, a.n_positions) == (2, 64, 4, 16, 256, 512, 128)
    assert (b.n_layer, b.n_embd, b.n_head, b.head_dim, b.n_inner, b.vocab_size, b.n_positions) == (3, 96, 3, 32, 320, 1031, 256)
    assert a.activation_function == "gelu_new" and b.activation_function == "gelu"
    assert a.layer_norm_epsilon == 1e-5 and b.layer_norm_epsilon == 1e-6
    assert a.attention_scale(1) == pytest.approx(16**-0.5)
    assert b.attention_scale(2) == pytest.approx(32**-0.5 / 3)
    assert a.eos_token_id == 511 and b.eos_token_id is None
    assert a.n_kv_heads == a.n_head


def test_config_defaults_follow_the_keys_meaning():
    data = {k: v for k, v in TINY_A["config"].items() if k not in ("n_inner", "activation_function", "scale_attn_weights")}
    cfg = GPT2Config.from_json(data)
    assert cfg.n_inner == 4 * cfg.n_embd and cfg.activation_function == "gelu_new" and cfg.scale_attn_weights


@pytest.mark.parametrize("change,match", [
    ({"n_head": 5}, "n_embd .* not a multiple of n_head"),
    ({"activation_function": "relu"}, "activation_function 'relu' is not supported"),
    ({"n_positions": 0}, "'n_positions' must be >= 1"),
    ({"layer_norm_epsilon": -1.0}, "layer_norm_epsilon"),
    ({"tie_word_embeddings": False}, "tie_word_embeddings=false"),
    ({"eos_token_id": 9999}, "eos_token_id"),
    ({"n_layer": "two"}, "'n_layer' must be an integer"),
])
def test_config_errors_name_the_key(change, match):
    with pytest.raises(ConfigError, match=match):
        GPT2Config.from_json(dict(TINY_A["config"], **change))


def test_config_missing_key_is_named():
    data = dict(TINY_A["config"])
    del data["n_embd"]
    with pytest.raises(ConfigError, match="required key 'n_embd' is missing"):
        GPT2Config.from_json(data)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B["config"]))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "GPT2LMHeadModel" and cfg.n_inner == 320
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B["config"], architectures=["Nope"])))
    with pytest.raises(ConfigError, match="unknown architecture"):
        load_config(tmp_path)
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path / "absent")


def test_engine_options_validation():
    opts = EngineOptions(max_requests=4, block_size=8).validated(256)
    assert opts.max_seq_len == 256 and opts.num_slabs == 4 * 32 and opts.max_batch_reqs == 4 and opts.capture is True
    assert EngineOptions(dtype="float32").validated(64).capture is False
    for bad in (dict(dtype="fp8"), dict(max_seq_len=999), dict(max_batch_tokens=0), dict(order="lifo"), dict(reserve_ratio=2.0)):
        with pytest.raises(ConfigError):
            EngineOptions(**bad).validated(256)


def test_safetensors_roundtrip_against_the_library(tmp_path):
    from safetensors.torch import load_file, save_file

    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
        "d": torch.randn(2, 2, 2).to(torch.float16),
    }
    write_file(tmp_path / "ours.safetensors", tensors)
    theirs = load_file(str(tmp_path / "ours.safetensors"))
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    ours = read_file(tmp_path / "theirs.safetensors")
    for name, t in tensors.items():
        assert theirs[name].dtype == t.dtype and torch.equal(theirs[name], t)
        assert ours[name].dtype == t.dtype and torch.equal(ours[name], t)


def test_random_weights_are_deterministic_and_follow_the_distributions():
    cfg = GPT2Config.from_json(TINY_B["config"])
    w1 = gpt2_model.random_weights(cfg, 2, std=0.05)
    w2 = gpt2_model.random_weights(cfg, 2, std=0.05)
    w3 = gpt2_model.random_weights(cfg, 3, std=0.05)
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert not torch.equal(w1["wte.weight"], w3["wte.weight"])
    assert w1["wte.weight"].std().item() == pytest.approx(0.05, rel=0.05)
    assert w1["h.0.attn.c_attn.bias"].std().item() == pytest.approx(0.01, rel=0.2)
    assert w1["h.1.ln_1.weight"].mean().item() == pytest.approx(1.0, abs=0.02)
    assert w1["ln_f.bias"].abs().max().item() < 0.2
    assert w1["h.2.mlp.c_fc.weight"].shape == (96, 320) and w1["h.2.attn.c_attn.weight"].shape == (96, 288)


def test_model_folder_is_read_back_in_its_stored_precision(tiny_a_dir, tiny_b_dir):
    for folder, want in ((tiny_a_dir, torch.float32), (tiny_b_dir, torch.bfloat16)):
        arch, cfg = load_config(folder)
        tensors = load_weights(folder, arch.weight_spec(cfg))
        assert len(tensors) == 2 + 12 * cfg.n_layer + 2
        assert all(t.dtype == want for t in tensors.values())


def test_transformer_prefix_and_ignorable_buffers(tmp_path):
    arch = architecture("GPT2LMHeadModel")
    cfg = arch.parse_config(TINY_A["config"])
    tensors = {"transformer." + k: v for k, v in arch.random_weights(cfg, 0).items()}
    tensors["lm_head.weight"] = tensors["transformer.wte.weight"]
    tensors["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
    tensors["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    got = check_and_select(tensors, arch.weight_spec(cfg))
    assert "wte.weight" in got and len(got) == 2 + 12 * cfg.n_layer + 2


def test_a_stored_head_that_differs_from_the_token_table_is_an_error():
    """GPT-2 ties its head to wte: a checkpoint whose lm_head.weight holds other values is not that model."""
    arch = architecture("GPT2LMHeadModel")
    cfg = arch.parse_config(TINY_A["config"])
    tensors = arch.random_weights(cfg, 0)
    tensors["lm_head.weight"] = tensors["wte.weight"].clone()
    tensors["lm_head.weight"][3, 5] += 0.25
    with pytest.raises(WeightError, match=r"lm_head\.weight: tied to wte\.weight but its values differ") as err:
        check_and_select(tensors, arch.weight_spec(cfg))
    assert len(err.value.wrong) == 1 and not err.value.missing and not err.value.unexpected
    tensors["lm_head.weight"] = tensors["wte.weight"][:-1]
    with pytest.raises(WeightError, match="tied to wte.weight of shape"):
        check_and_select(tensors, arch.weight_spec(cfg))


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    arch = architecture("GPT2LMHeadModel")
    cfg = arch.parse_config(TINY_A["config"])
    tensors = arch.random_weights(cfg, 0)
    del tensors["h.1.ln_2.bias"]
    del tensors["wpe.weight"]
    tensors["h.0.mlp.c_fc.weight"] = torch.zeros(64, 255)
    tensors["h.0.attn.c_proj.weight"] = torch.zeros(64, 64, dtype=torch.int32)
    tensors["h.7.extra.weight"] = torch.zeros(3)
    write_file(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as info:
        load_weights(tmp_path, arch.weight_spec(cfg))
    err = info.value
    assert len(err.missing) == 2 and any("wpe.weight or transformer.wpe.weight" in m for m in err.missing)
    assert err.unexpected == ["h.7.extra.weight"]
    assert len(err.wrong) == 2
    text = str(err)
    assert "missing (2)" in text and "unexpected (1)" in text and "wrong (2)" in text
    assert "h.0.mlp.c_fc.weight: expected shape (64, 256), got (64, 255)" in text
    assert "h.0.attn.c_proj.weight: expected a floating-point tensor" in text


def test_missing_file_is_a_weight_error(tmp_path):
    arch = architecture("GPT2LMHeadModel")
    with pytest.raises(WeightError, match="no .safetensors file"):
        load_weights(tmp_path, arch.weight_spec(arch.parse_config(TINY_A["config"])))
