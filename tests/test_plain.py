"""The plain implementation itself, and host-side restatements the engine shares formulas with."""

import math
import os

import numpy as np
import pytest
import torch

from tesseract_b200.parts.rotary import rotary_inverse_frequencies
from tesseract_b200.sampling import SplitMix64, sample_top_p_host
from tests.helpers import REL, TINY, random_tokens
from tests.plain import llama


def test_rope_frequencies_match_the_engine_and_the_three_bands():
    scaling = TINY["b"]["rope_scaling"]
    ours = rotary_inverse_frequencies(32, 500000.0, scaling)
    plain = llama.rope_inverse_frequencies(32, 500000.0, scaling)
    assert np.array_equal(ours, plain) and ours.dtype == np.float32
    base = llama.rope_inverse_frequencies(32, 500000.0, None)
    wavelength = 2 * math.pi / base
    high, low = 64 / 4.0, 64 / 1.0
    assert np.allclose(ours[wavelength < high], base[wavelength < high])
    assert np.allclose(ours[wavelength > low], base[wavelength > low] / 8.0)
    middle = (wavelength >= high) & (wavelength <= low)
    assert middle.any() and ((ours[middle] < base[middle]) & (ours[middle] > base[middle] / 8.0)).all()
    assert np.array_equal(rotary_inverse_frequencies(16, 10000.0, None), llama.rope_inverse_frequencies(16, 10000.0, None))


def test_splitmix64_known_values():
    # first outputs of SplitMix64 seeded with 0 (published test vector of the generator)
    rng = SplitMix64(0)
    assert [rng.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    a, b = SplitMix64(7), llama.SplitMix64(7)
    for _ in range(5):
        u = a.unit_f64()
        assert u == b.unit_f64() and 0.0 <= u < 1.0


def test_host_sampler_matches_the_plain_restatement():
    rng = np.random.default_rng(0)
    for trial in range(200):
        logits = rng.normal(size=50).astype(np.float32) * 3
        t, p, u = float(rng.uniform(0.2, 2.0)), float(rng.uniform(0.05, 1.0)), float(rng.uniform())
        assert sample_top_p_host(logits, t, p, u) == llama.sample_host(logits, t, p, u)
    assert sample_top_p_host(np.array([-1, 4, 4, 3], dtype=np.float32), 0.0, 1.0, 0.0) == 1     # lowest id on ties
    # a tiny top_p keeps only the most likely token
    assert sample_top_p_host(np.array([0, 5, 1], dtype=np.float32), 1.0, 1e-6, 0.999) == 1


def test_plain_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    y = llama.rms_norm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=torch.float64))
    one = torch.ones(1, 1, dtype=torch.float64)
    out = llama.swiglu(one * 2.0, one, one * 3.0, one * 0.5)
    assert math.isclose(out.item(), 2.0 / (1 + math.exp(-2.0)) * 6.0 * 0.5)


def test_plain_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nh, nkv, d = 9, 4, 2, 8
    q, k, v = (torch.randn(T, h, d, dtype=torch.float64) for h in (nh, nkv, nkv))
    out = llama.attention(q, k, v, 0.3)
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))            # the first row sees one key
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0.0, 9.0
    assert torch.allclose(llama.attention(q, k2, v2, 0.3)[:5], out[:5])        # later keys never reach earlier rows
    # one score made to stand out: the row returns that key's value
    q3, k3 = q.clone(), k.clone()
    q3[8, 1] = 0.0
    q3[8, 1, 0] = 100.0
    k3[:, 0, 0] = 0.0
    k3[2, 0, 0] = 10.0
    assert torch.allclose(llama.attention(q3, k3, v, 1.0)[8, 1], v[2, 0], atol=1e-9)
    windowed = llama.attention(q3, k3, v, 1.0, window=3)
    assert not torch.allclose(windowed[8, 1], v[2, 0], atol=1e-3)             # key 2 is outside the last three


def test_plain_forward_prefix_property_and_rounding_mode(tmp_path):
    from tesseract_b200.weights.random_init import write_random_model

    folder = write_random_model(str(tmp_path / "m"), dict(TINY["b"], torch_dtype="bfloat16"), seed=2)
    config, tensors = llama.load_folder(folder)
    tokens = random_tokens(config["vocab_size"], 40, seed=1)
    full = llama.forward(config, tensors, tokens)
    assert full.shape == (40, config["vocab_size"]) and torch.isfinite(full).all()
    assert torch.allclose(llama.forward(config, tensors, tokens[:13]), full[:13], atol=1e-12)
    f32 = llama.forward(config, tensors, tokens, dtype=torch.float32)
    rounded = llama.forward(config, tensors, tokens, dtype=torch.float32, round_to=torch.bfloat16)
    scale = full.abs().max().item()
    assert (f32 - full).abs().max().item() < 1e-5 * scale
    assert 1e-5 * scale < (rounded - full).abs().max().item() < REL["bfloat16"] * scale


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_the_two_plain_models_agree(tmp_path, name):
    """tests/plain/llama.py (whole sequences, torch) against tests/plain/llama_scalar.cpp (token by token, scalar
    loops, its own key/value list and its own frequency recipe): two implementations written apart from the same
    formulas.  The reference itself cannot be built here (Rust, GPU-only kernels), so this pair, not an output of
    the reference, is what anchors the plain model: with and without frequency scaling, tied and untied head,
    grouped heads, head sizes that do not multiply back to the width."""
    import shutil
    import struct
    import subprocess

    from tesseract_b200.weights.random_init import write_random_model

    compiler = shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        pytest.skip("no C++ compiler")
    source = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain", "llama_scalar.cpp")
    binary = str(tmp_path / "llama_scalar")
    subprocess.run([compiler, "-O2", "-std=c++17", "-o", binary, source], check=True)
    folder = write_random_model(str(tmp_path / "m"), dict(TINY[name], torch_dtype="float32"), seed=4)
    config, tensors = llama.load_folder(folder)
    tokens = random_tokens(config["vocab_size"], 70, seed=9)
    nh, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    d = config.get("head_dim") or config["hidden_size"] // nh
    scaling = config.get("rope_scaling")
    tied = bool(config.get("tie_word_embeddings"))
    with open(tmp_path / "model.bin", "wb") as out:
        out.write(struct.pack("<11i", config["num_hidden_layers"], config["hidden_size"], nh, nkv, d,
                              config["intermediate_size"], config["vocab_size"], int(tied), int(scaling is not None),
                              scaling["original_max_position_embeddings"] if scaling else 0, len(tokens)))
        out.write(struct.pack("<5d", config["rms_norm_eps"], config["rope_theta"],
                              *([scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]]
                                if scaling else [1.0, 1.0, 1.0])))
        out.write(np.asarray(tokens, dtype="<i4").tobytes())
        names = ["model.embed_tokens.weight"]
        for layer in range(config["num_hidden_layers"]):
            p = f"model.layers.{layer}"
            names += [f"{p}.input_layernorm.weight", f"{p}.self_attn.q_proj.weight", f"{p}.self_attn.k_proj.weight",
                      f"{p}.self_attn.v_proj.weight", f"{p}.self_attn.o_proj.weight",
                      f"{p}.post_attention_layernorm.weight", f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight",
                      f"{p}.mlp.down_proj.weight"]
        names += ["model.norm.weight"] + ([] if tied else ["lm_head.weight"])
        for tensor_name in names:
            out.write(tensors[tensor_name].to(torch.float32).contiguous().numpy().astype("<f4").tobytes())
    subprocess.run([binary, str(tmp_path / "model.bin"), str(tmp_path / "logits.bin")], check=True)
    scalar = np.fromfile(tmp_path / "logits.bin", dtype="<f8").reshape(len(tokens), config["vocab_size"])
    whole = llama.forward(config, tensors, tokens).numpy()
    # float64 both: what is left is the order of summation and one unit in the last place of a 32-bit frequency
    assert np.abs(scalar - whole).max() <= 1e-6 * np.abs(whole).max()
    assert (scalar.argmax(axis=1) == whole.argmax(axis=1)).all()
