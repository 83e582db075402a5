"""Weights: random-weights folders, reading by name, and the one error that lists everything (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import jax_llm_examples_b200 as J
from jax_llm_examples_b200.config import resolve
from jax_llm_examples_b200.weights import load_tensors, random_tensors


def _specs(name):
    arch = resolve(J.preset(name))
    cfg = arch.parse_config(J.preset(name))
    return arch, cfg, arch.tensor_specs(cfg)


def test_random_model_folder_round_trip(tmp_path):
    folder = J.write_random_model(tmp_path / "m", J.preset("tiny_b"), seed=1)
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 96
    arch, cfg, specs = _specs("tiny_b")
    t = load_tensors(folder, specs, arch.canonical_name, torch.bfloat16)
    assert set(t) == set(specs)
    assert t["model.layers.1.feed_forward.experts.gate_up_proj"].shape == (8, 96, 128)
    assert t["model.layers.0.feed_forward.gate_proj.weight"].shape == (192, 96)
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    # seeded: the same folder again is identical; another seed is not
    again = J.write_random_model(tmp_path / "m2", J.preset("tiny_b"), seed=1)
    other = J.write_random_model(tmp_path / "m3", J.preset("tiny_b"), seed=2)
    a, b, c = (load_file(str(f / "model.safetensors")) for f in (folder, again, other))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002
    assert torch.all(a["model.norm.weight"] == 1)


def test_norm_noise_and_a_tensor_does_not_depend_on_the_others():
    _, _, specs = _specs("tiny_a")
    t = random_tensors(specs, seed=0, norm_noise=0.1)
    g = t["model.layers.2.input_layernorm.weight"].float()
    assert 0.03 < float(g.std()) < 0.2 and abs(float(g.mean()) - 1) < 0.1
    one = random_tensors({k: v for k, v in specs.items() if k == "lm_head.weight"}, seed=0)
    assert torch.equal(one["lm_head.weight"], t["lm_head.weight"])


def test_stored_precision_is_kept(tmp_path):
    folder = J.write_random_model(tmp_path / "m", J.preset("tiny_a"), seed=0)
    path = str(folder / "model.safetensors")
    t = load_file(path)
    t["model.layers.0.feed_forward.router.weight"] = t["model.layers.0.feed_forward.router.weight"].float()
    save_file(t, path)
    arch, cfg, specs = _specs("tiny_a")
    bf = load_tensors(folder, specs, arch.canonical_name, torch.bfloat16)
    assert bf["model.layers.0.feed_forward.router.weight"].dtype == torch.float32  # stored 32-bit stays so
    assert bf["model.layers.1.feed_forward.router.weight"].dtype == torch.bfloat16
    f32 = load_tensors(folder, specs, arch.canonical_name, torch.float32)
    assert all(v.dtype == torch.float32 for v in f32.values())
    assert torch.equal(f32["lm_head.weight"], bf["lm_head.weight"].float())  # widening is exact


def test_prefix_and_foreign_tensors(tmp_path):
    folder = J.write_random_model(tmp_path / "m", J.preset("tiny_a"), seed=0)
    path = str(folder / "model.safetensors")
    t = {"language_model." + k: v for k, v in load_file(path).items()}
    t["vision_model.patch_embedding.weight"] = torch.zeros(3, 3)
    t["multi_modal_projector.linear_1.weight"] = torch.zeros(2, 2)
    save_file(t, path)
    arch, cfg, specs = _specs("tiny_a")
    assert set(load_tensors(folder, specs, arch.canonical_name, torch.bfloat16)) == set(specs)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = J.write_random_model(tmp_path / "m", J.preset("tiny_a"), seed=0)
    path = str(folder / "model.safetensors")
    t = load_file(path)
    del t["model.layers.3.self_attn.o_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    t["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    t["model.layers.2.feed_forward.experts.down_proj"] = torch.zeros(4, 64, 128)
    save_file(t, path)
    arch, cfg, specs = _specs("tiny_a")
    with pytest.raises(J.WeightError) as e:
        load_tensors(folder, specs, arch.canonical_name, torch.bfloat16)
    err = e.value
    assert sorted(err.missing) == ["model.layers.3.self_attn.o_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert len(err.wrong_shape) == 2
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "expected [32, 64], found [16, 64]",
                  "model.layers.2.feed_forward.experts.down_proj: expected [4, 128, 64], found [4, 64, 128]"):
        assert piece in msg, piece


def test_tied_embeddings_need_no_lm_head(tmp_path):
    d = J.preset("tiny_a", tie_word_embeddings=True)
    folder = J.write_random_model(tmp_path / "m", d, seed=0)
    assert "lm_head.weight" not in load_file(str(folder / "model.safetensors"))
    arch = resolve(d)
    cfg = arch.parse_config(d)
    assert "lm_head.weight" not in load_tensors(folder, arch.tensor_specs(cfg), arch.canonical_name, torch.bfloat16)


def test_missing_folder_and_file(tmp_path):
    arch, cfg, specs = _specs("tiny_a")
    with pytest.raises(FileNotFoundError):
        load_tensors(tmp_path, specs, arch.canonical_name, torch.bfloat16)
