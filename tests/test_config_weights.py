"""Configuration, registry and checkpoint loading (no device needed)."""

import json
import os

import pytest
import torch

import tesseract_b200.models  # noqa: F401  (registers the architecture and the parts)
from tesseract_b200.config import (ConfigError, EngineConfig, NoArchitectureError,
                                   UnsupportedArchitectureError, load_model_description, resolve_architecture)
from tesseract_b200.models import LlamaConfig, expected_tensors
from tesseract_b200.weights import (SafetensorsError, SafetensorsSource, WeightError, check_and_load,
                                    write_safetensors)
from tesseract_b200.weights.random_init import random_tensors, write_random_model
from tests.helpers import TINY


def test_llama_config_reads_every_key():
    cfg = LlamaConfig.from_dict(dict(TINY["b"], torch_dtype="bfloat16"))
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 3, 1)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings) == (32, 320, 384, 256)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 500000.0 and not cfg.tie_word_embeddings
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.eos_token_id == (383,)           # a single integer becomes a list of one
    assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_llama_config_defaults_and_relaxations():
    raw = dict(TINY["a"])
    raw.pop("head_dim")
    raw.pop("rope_scaling")
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.head_dim == 16 and cfg.rope_scaling is None
    # head_dim need not multiply back to hidden_size
    assert LlamaConfig.from_dict(TINY["c"]).head_dim * 6 != TINY["c"]["hidden_size"]


@pytest.mark.parametrize("change, message", [
    ({"hidden_act": "gelu"}, "SiLU"),
    ({"attention_bias": True}, "bias"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"torch_dtype": "float16"}, "torch_dtype"),
    ({"vocab_size": 0}, "positive"),
    ({"eos_token_id": [999]}, "eos_token_id"),
    ({"model_type": "qwen"}, "model_type"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 4096}}, "original rope context"),
])
def test_llama_config_rejects(change, message):
    with pytest.raises(ConfigError, match=message):
        LlamaConfig.from_dict(dict(TINY["a"], **change))


def test_llama_config_missing_key():
    raw = dict(TINY["a"])
    raw.pop("intermediate_size")
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(raw)


def test_registry_dispatch():
    assert resolve_architecture(TINY["a"]).name == "LlamaForCausalLM"
    with pytest.raises(NoArchitectureError):
        resolve_architecture({"architectures": []})
    with pytest.raises(UnsupportedArchitectureError, match="Qwen"):
        resolve_architecture({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"})


def test_spec_carries_every_size():
    arch = resolve_architecture(TINY["b"])
    spec = arch.build_spec(arch.read_config(TINY["b"]))
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    mixer = spec.layers[1].mixer
    assert mixer.kind == "attention" and mixer.params["num_kv_heads"] == 1 and mixer.params["head_dim"] == 32
    assert mixer.children["position"].params["scaling"]["factor"] == 8.0
    assert spec.layers[0].feed_forward.params["intermediate_size"] == 320
    assert spec.final_norm.params["eps"] == 1e-6
    assert spec.head.weights["weight"] == "lm_head.weight"
    tied = resolve_architecture(TINY["a"]).build_spec(LlamaConfig.from_dict(TINY["a"]))
    assert tied.head.weights["weight"] == tied.embedding.weights["table"]


def test_engine_config_invariants():
    EngineConfig().validate()
    for bad in (dict(max_running=0), dict(max_batch_tokens=4, max_running=8), dict(prefill_chunk_tokens=0),
                dict(kv_capacity_tokens=2, max_running=8), dict(page_size=24), dict(dtype="float16")):
        with pytest.raises(ValueError):
            EngineConfig(**bad).validate()


def test_random_model_round_trip(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), dict(TINY["a"], torch_dtype="bfloat16"), seed=3)
    arch, cfg, spec = load_model_description(folder)
    tensors = check_and_load(folder, expected_tensors(spec), arch.ignorable_tensors(cfg))
    assert len(tensors) == 2 + 2 * 9        # tied head: embedding, final norm, nine per layer
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    again = random_tensors(dict(TINY["a"], torch_dtype="bfloat16"), seed=3)
    other = random_tensors(dict(TINY["a"], torch_dtype="bfloat16"), seed=4)
    name = "model.layers.1.mlp.down_proj.weight"
    assert torch.equal(tensors[name], again[name]) and not torch.equal(tensors[name], other[name])
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    assert abs(norm.mean().item() - 1.0) < 0.05      # norm scales are 1 + N(0, 0.02)
    # the file is a plain safetensors file that the reference wheel reads too
    from safetensors.torch import load_file
    theirs = load_file(os.path.join(folder, "model.safetensors"))
    assert set(theirs) == set(tensors) and all(torch.equal(theirs[k], tensors[k]) for k in tensors)


def test_stored_dtype_is_kept(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), dict(TINY["a"], torch_dtype="float32"), seed=0)
    arch, cfg, spec = load_model_description(folder)
    tensors = check_and_load(folder, expected_tensors(spec))
    assert all(t.dtype == torch.float32 for t in tensors.values())


def test_weight_error_lists_everything(tmp_path):
    folder = str(tmp_path / "m")
    config = dict(TINY["a"], torch_dtype="bfloat16")
    tensors = random_tensors(config, seed=0)
    tensors.pop("model.layers.0.mlp.up_proj.weight")
    tensors.pop("model.norm.weight")
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(7, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    arch, cfg, spec = load_model_description(folder)
    with pytest.raises(WeightError) as info:
        check_and_load(folder, expected_tensors(spec), arch.ignorable_tensors(cfg))
    err = info.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.extra.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (32, 64), (7, 64))]
    assert err.wrong_dtype[0][0] == "model.layers.1.input_layernorm.weight"
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [7, 64], expected [32, 64]"):
        assert piece in text


def test_ignorable_tensors(tmp_path):
    folder = str(tmp_path / "m")
    config = dict(TINY["a"], torch_dtype="bfloat16")
    tensors = random_tensors(config, seed=0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()       # tied: may be present
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    arch, cfg, spec = load_model_description(folder)
    assert len(check_and_load(folder, expected_tensors(spec), arch.ignorable_tensors(cfg))) == 20


def test_safetensors_container_errors(tmp_path):
    path = tmp_path / "model.safetensors"
    path.write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsSource(str(tmp_path))
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(len(header).to_bytes(8, "little") + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not match shape"):
        SafetensorsSource(str(tmp_path))
    with pytest.raises(SafetensorsError, match="neither"):
        SafetensorsSource(str(tmp_path / "nowhere"))


def test_sharded_checkpoint(tmp_path):
    a = {"p": torch.arange(6, dtype=torch.float32).view(2, 3)}
    b = {"q": torch.ones(4, dtype=torch.bfloat16)}
    write_safetensors(str(tmp_path / "s1.safetensors"), a)
    write_safetensors(str(tmp_path / "s2.safetensors"), b)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"p": "s1.safetensors", "q": "s2.safetensors"}}))
    source = SafetensorsSource(str(tmp_path))
    assert source.names() == ["p", "q"] and torch.equal(source.tensor("p"), a["p"])
    assert source.tensor("q").dtype == torch.bfloat16
