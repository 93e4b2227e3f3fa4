"""Weights by tensor name: one error that lists everything wrong; random-weights mode; storage dtypes."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from oxr_inference_b200.parts.base import Runtime
from oxr_inference_b200.parts.decoder import DecoderModel
from oxr_inference_b200.config import resolve_architecture
from oxr_inference_b200.weights import WeightError, load_weights, shape_only_model, write_random_model
from util import TINY_A, TINY_B


def _host_model(raw, dtype=torch.float32):
    arch = resolve_architecture(raw)
    spec = arch.model_spec(arch.config_from_dict(raw, None))
    rt = Runtime(device=torch.device("cpu"), dtype=dtype, max_positions=8, status=torch.zeros(4, dtype=torch.int32))
    return DecoderModel(spec, rt)


def test_random_model_folder_has_every_tensor_with_its_shape(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "b", seed=5)
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 96
    t = load_file(str(folder / "model.safetensors"))
    assert t["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert t["model.layers.0.self_attn.k_proj.weight"].shape == (64, 96)
    assert t["model.layers.1.self_attn.q_norm.weight"].shape == (32,)
    assert t["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert t["lm_head.weight"].shape == (509, 96) and t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert len(t) == 3 * 11 + 3
    norm = t["model.layers.0.input_layernorm.weight"].float()
    assert 0.5 < norm.mean() < 1.5 and t["model.embed_tokens.weight"].float().std() < 0.03
    # tied: no separate head
    t_a = load_file(str(write_random_model(TINY_A, tmp_path / "a", seed=5) / "model.safetensors"))
    assert "lm_head.weight" not in t_a


def test_values_depend_on_seed_and_name_only(tmp_path):
    a = load_file(str(write_random_model(TINY_A, tmp_path / "1", seed=1) / "model.safetensors"))
    b = load_file(str(write_random_model(TINY_A, tmp_path / "2", seed=1) / "model.safetensors"))
    c = load_file(str(write_random_model(TINY_A, tmp_path / "3", seed=2) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    wider = dict(TINY_A, num_hidden_layers=3)
    d = load_file(str(write_random_model(wider, tmp_path / "4", seed=1) / "model.safetensors"))
    assert torch.equal(a["model.layers.1.mlp.up_proj.weight"], d["model.layers.1.mlp.up_proj.weight"])


def test_loads_fused_projections_by_name_and_keeps_dtypes(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "b", seed=0)
    stored = load_file(str(folder / "model.safetensors"))
    model = _host_model(TINY_B, torch.bfloat16)
    load_weights(model, folder)
    attn = model.blocks[1].mixer
    assert attn.qkv.weight.dtype == torch.bfloat16 and attn.qkv.weight.shape == (192 + 64 + 64, 96)
    assert torch.equal(attn.qkv.weight[:192], stored["model.layers.1.self_attn.q_proj.weight"])
    assert torch.equal(attn.qkv.weight[192:256], stored["model.layers.1.self_attn.k_proj.weight"])
    assert torch.equal(attn.qkv.weight[256:], stored["model.layers.1.self_attn.v_proj.weight"])
    ff = model.blocks[2].feed_forward
    # gate and up rows alternate in groups of 8: rows 16j .. 16j+7 are gate 8j .. 8j+7, the next 8 the matching up rows
    both = ff.gate_up.weight.view(-1, 2, 8, 96)
    assert ff.gate_up.interleave == 8 and ff.gate_up.weight.shape == (320, 96)
    assert torch.equal(both[:, 0].reshape(160, 96), stored["model.layers.2.mlp.gate_proj.weight"])
    assert torch.equal(both[:, 1].reshape(160, 96), stored["model.layers.2.mlp.up_proj.weight"])
    # small vectors are kept in fp32 whatever the path
    assert attn.q_norm.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
    assert torch.equal(attn.q_norm, stored["model.layers.1.self_attn.q_norm.weight"].float())
    # a float32 engine widens everything
    m32 = _host_model(TINY_B, torch.float32)
    load_weights(m32, folder)
    assert m32.blocks[0].mixer.qkv.weight.dtype == torch.float32 and m32.embedding.weight.dtype == torch.float32


def test_a_tensor_stored_in_32_bit_stays_32_bit(tmp_path):
    folder = write_random_model(TINY_A, tmp_path / "a", seed=0, dtype="float32")
    model = _host_model(TINY_A, torch.bfloat16)
    load_weights(model, folder)
    assert model.embedding.weight.dtype == torch.float32
    assert model.blocks[0].feed_forward.down.weight.dtype == torch.float32


def test_reference_prefix_and_tied_head_copy_are_accepted(tmp_path):
    folder = write_random_model(TINY_A, tmp_path / "a", seed=0)
    t = load_file(str(folder / "model.safetensors"))
    renamed = {"llm." + k: v for k, v in t.items()}  # the reference's files (oxr_runtime/weight_names.py:11)
    renamed["llm.lm_head.weight"] = t["model.embed_tokens.weight"].clone()  # a tied checkpoint that still carries the head
    save_file(renamed, str(folder / "model.safetensors"))
    load_weights(_host_model(TINY_A), folder)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "b", seed=0)
    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.0.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.7.mlp.up_proj.weight"] = torch.zeros(2, 2)
    t["visual.patch_embed.weight"] = torch.zeros(1)
    t["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(64, 95)
    t["lm_head.weight"] = torch.zeros(508, 96)
    save_file(t, str(folder / "model.safetensors"))
    model = _host_model(TINY_B)
    with pytest.raises(WeightError) as info:
        load_weights(model, folder)
    e = info.value
    assert e.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.mlp.up_proj.weight", "visual.patch_embed.weight"]
    assert len(e.wrong_shape) == 2 and "[64, 95]" in str(e) and "[64, 96]" in str(e) and "lm_head.weight" in str(e)
    for word in ("missing (2)", "unexpected (2)", "wrong shape (2)"):
        assert word in str(e)
    assert model.embedding.weight is None, "nothing may be copied before the whole checkpoint has been checked"


def test_sharded_checkpoint(tmp_path):
    folder = write_random_model(TINY_A, tmp_path / "a", seed=0)
    t = load_file(str(folder / "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    index = {"weight_map": {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, k in enumerate(names)}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    model = _host_model(TINY_A)
    load_weights(model, folder)
    assert torch.equal(model.embedding.weight, t["model.embed_tokens.weight"].float())
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(WeightError, match="absent"):
        load_weights(_host_model(TINY_A), folder)


def test_shape_only_model_lists_names():
    named = shape_only_model(TINY_A).named_parameters()
    assert "model.layers.1.self_attn.o_proj.weight" in named and "lm_head.weight" not in named
    assert named["model.layers.0.self_attn.q_norm.weight"][2].role == "vector"


def test_stacked_tensors_of_mixed_dtype_are_kept_in_32_bit_whatever_their_order():
    """q/k/v (or gate/up) share one buffer. If any of them is stored in 32-bit the buffer is 32-bit, and the values of
    all of them are exact, whichever came first."""
    import torch

    from oxr_inference_b200.parts.base import Runtime
    from oxr_inference_b200.parts.linear import StackedLinear

    rt = Runtime(device=torch.device("cpu"), dtype=torch.bfloat16, max_positions=8, status=torch.zeros(4, dtype=torch.int32))
    a32 = torch.randn(4, 8)
    b16 = torch.randn(6, 8).bfloat16()
    for order in (("a", "b"), ("b", "a")):
        lin = StackedLinear(rt, 8, {"a": 4, "b": 6})
        for name in order:
            lin.assign(name, a32 if name == "a" else b16)
        assert lin.weight.dtype == torch.float32
        assert torch.equal(lin.weight[:4], a32) and torch.equal(lin.weight[4:], b16.float())
    lin = StackedLinear(rt, 8, {"a": 4, "b": 6})
    lin.assign("a", a32.bfloat16())
    lin.assign("b", b16)
    assert lin.weight.dtype == torch.bfloat16
