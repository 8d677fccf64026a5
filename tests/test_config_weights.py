"""Configuration, registry, safetensors reading and weight errors (no GPU)."""
import copy
import json

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from vosti_b200.config import (ConfigError, Qwen3Config, known_architectures, model_spec_from_config,
                               model_spec_from_dir, register_architecture)
from vosti_b200.models import expected_weights
from vosti_b200.weights import (SafetensorsError, WeightError, WeightSpec, draw_tensors, load_weights,
                                open_model_shards, write_random_model, write_safetensors)


def test_config_reads_every_size_from_its_keys():
    cfg = Qwen3Config.from_dict(TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (3, 96, 6, 2, 32, 256, 512)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.tie_word_embeddings is False
    spec = cfg.to_model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    assert spec.layers[0].mixer["head_dim"] == 32 and spec.layers[0].norm["eps"] == 1e-5
    assert spec.layers[0].mixer["scale"] == pytest.approx(32 ** -0.5)
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", ["head_dim", "rms_norm_eps", "rope_theta", "num_key_value_heads",
                                 "tie_word_embeddings", "sliding_window", "rope_scaling", "hidden_act"])
def test_config_has_no_defaults(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        model_spec_from_config(raw)


@pytest.mark.parametrize("key,value", [
    ("num_attention_heads", 5), ("head_dim", 15), ("hidden_act", "gelu"), ("attention_bias", True),
    ("use_sliding_window", True), ("sliding_window", 128), ("rope_scaling", {"rope_type": "llama3"}),
    ("rms_norm_eps", 0.0), ("vocab_size", -1), ("tie_word_embeddings", "yes"), ("model_type", "llama"),
    ("hidden_size", True), ("attention_dropout", 0.1), ("rope_theta", float("inf"))])
def test_config_rejects_bad_values(key, value):
    raw = dict(TINY_A)
    raw[key] = value
    with pytest.raises(ConfigError):
        model_spec_from_config(raw)


def test_registry_names_the_architecture():
    assert "Qwen3ForCausalLM" in known_architectures()
    raw = dict(TINY_A, architectures=["SomethingElse"])
    with pytest.raises(ConfigError, match="unknown architecture 'SomethingElse'.*Qwen3ForCausalLM"):
        model_spec_from_config(raw)
    with pytest.raises(ConfigError, match="exactly one"):
        model_spec_from_config({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="already registered"):
        register_architecture("Qwen3ForCausalLM", lambda raw: None)


def test_expected_weights_names_and_shapes():
    names = expected_weights(model_spec_from_config(TINY_B))
    assert names["model.layers.2.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    assert names["model.layers.0.self_attn.k_proj.weight"].shape == (2 * 32, 96)
    assert names["model.layers.1.self_attn.q_norm.weight"].shape == (32,)
    assert names["model.layers.1.mlp.down_proj.weight"].shape == (96, 256)
    assert names["lm_head.weight"].shape == (512, 96) and names["model.norm.weight"].shape == (96,)
    assert len(names) == 2 + 1 + 3 * 11
    tied = expected_weights(model_spec_from_config(TINY_A))
    assert "lm_head.weight" not in tied


def test_random_model_folder_roundtrip(tmp_path):
    folder = write_random_model(tmp_path / "m", TINY_A, seed=7)
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 64
    spec = model_spec_from_dir(folder)
    expected = expected_weights(spec)
    tensors = load_weights(folder, expected, device="cpu", dtype=torch.bfloat16)
    assert set(tensors) == set(expected)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    again = draw_tensors(expected, seed=7)
    assert all(torch.equal(tensors[n], again[n]) for n in expected)            # seed decides
    other = draw_tensors(expected, seed=8)
    assert not torch.equal(tensors["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    norm = tensors["model.layers.0.self_attn.q_norm.weight"].float()
    assert abs(norm.mean().item() - 1.0) < 0.2
    wide = load_weights(folder, expected, device="cpu", dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in wide.values())
    assert torch.equal(wide["model.norm.weight"], tensors["model.norm.weight"].float())


def test_resident_dtypes(tmp_path):
    """bf16 stays bf16; a tensor stored in 32-bit stays 32-bit; integer tables become int32."""
    tensors = {"a": torch.randn(4, 4).bfloat16(), "b": torch.randn(4), "c": torch.arange(6, dtype=torch.int64)}
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    expected = {"a": WeightSpec((4, 4)), "b": WeightSpec((4,)), "c": WeightSpec((6,), integer=True)}
    got = load_weights(tmp_path / "m", expected, device="cpu", dtype=torch.bfloat16)
    assert [got[k].dtype for k in "abc"] == [torch.bfloat16, torch.float32, torch.int32]
    assert torch.equal(got["b"], tensors["b"]) and got["c"].tolist() == list(range(6))
    wide = load_weights(tmp_path / "m", expected, device="cpu", dtype=torch.float32)
    assert [wide[k].dtype for k in "abc"] == [torch.float32, torch.float32, torch.int32]


def test_floating_tensors_stored_in_another_dtype_are_refused_not_rounded(tmp_path):
    """F16 and F64 are listed in the one error beside the other faults
    (python/vosti_kernels/checkpoint.py:61-62 takes BF16 only; F32 is kept here as stored)."""
    from vosti_b200.weights import check_tensors
    tensors = {"a": torch.randn(4, 4).half(), "b": torch.randn(4).double(), "c": torch.randn(2).bfloat16(),
               "i": torch.arange(3, dtype=torch.int16)}
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    expected = {"a": WeightSpec((4, 4)), "b": WeightSpec((4,)), "c": WeightSpec((3,)), "i": WeightSpec((3,), integer=True)}
    for dtype in (torch.bfloat16, torch.float32):
        with pytest.raises(WeightError) as caught:
            load_weights(tmp_path / "m", expected, device="cpu", dtype=dtype)
        assert caught.value.wrong_dtype == [("a", "F16"), ("b", "F64")]
        assert caught.value.wrong_shape == [("c", (2,), (3,))]
        assert "a is stored as F16" in str(caught.value) and "BF16 or F32" in str(caught.value)
    with pytest.raises(WeightError) as caught:
        check_tensors(tensors, expected)
    assert [name for name, _ in caught.value.wrong_dtype] == ["a", "b"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    spec = model_spec_from_config(TINY_A)
    expected = expected_weights(spec)
    tensors = draw_tensors(expected, seed=0)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(32, 64).bfloat16()
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    with pytest.raises(WeightError) as caught:
        load_weights(tmp_path / "m", expected, device="cpu", dtype=torch.bfloat16)
    err = caught.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (32, 64), (64, 64))]
    text = str(err)
    for fragment in ("missing (2)", "unexpected (1)", "model.norm.weight", "has [32, 64], expected [64, 64]"):
        assert fragment in text


def test_tied_checkpoint_may_carry_a_head(tmp_path):
    from vosti_b200.models import build_model
    model = build_model(model_spec_from_config(TINY_A))
    expected = model.expected_weights()
    tensors = draw_tensors(expected, seed=0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    got = load_weights(tmp_path / "m", expected, device="cpu", dtype=torch.bfloat16, ignore=model.ignorable_weights(),
                       aliases=model.tied_weights())
    assert "lm_head.weight" not in got


def test_tied_checkpoint_with_a_different_head_is_refused(tmp_path):
    """`tie_word_embeddings: true` says the head is the embedding table; a folder whose
    lm_head.weight differs from it contradicts its own configuration
    (python/vosti_kernels/model_families/qwen3/physical.py:131-134)."""
    from vosti_b200.models import build_model
    from vosti_b200.weights import check_tensors
    model = build_model(model_spec_from_config(TINY_A))
    expected = model.expected_weights()
    tensors = draw_tensors(expected, seed=0)
    head = tensors["model.embed_tokens.weight"].clone()
    head[3, 5] += 1.0
    tensors["lm_head.weight"] = head
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
    with pytest.raises(WeightError) as caught:
        load_weights(tmp_path / "m", expected, device="cpu", dtype=torch.bfloat16, ignore=model.ignorable_weights(),
                     aliases=model.tied_weights())
    assert caught.value.conflicts == [("lm_head.weight", "model.embed_tokens.weight", "holds different values")]
    assert "lm_head.weight must equal model.embed_tokens.weight" in str(caught.value)
    with pytest.raises(WeightError):
        check_tensors(tensors, expected, ignore=model.ignorable_weights(), aliases=model.tied_weights())
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"][:-1]
    with pytest.raises(WeightError, match="has shape"):
        check_tensors(tensors, expected, ignore=model.ignorable_weights(), aliases=model.tied_weights())


def test_sharded_folder_and_broken_files(tmp_path):
    tensors = {"x": torch.ones(2, 3).bfloat16(), "y": torch.zeros(5).bfloat16()}
    folder = tmp_path / "m"
    folder.mkdir()
    write_safetensors(folder / "s1.safetensors", {"x": tensors["x"]})
    write_safetensors(folder / "s2.safetensors", {"y": tensors["y"]})
    (folder / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    got = load_weights(folder, {"x": WeightSpec((2, 3)), "y": WeightSpec((5,))}, device="cpu", dtype=torch.bfloat16)
    assert torch.equal(got["x"], tensors["x"])
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../evil.safetensors"}}))
    with pytest.raises(SafetensorsError):
        open_model_shards(folder)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(SafetensorsError, match="neither"):
        open_model_shards(empty)
    truncated = tmp_path / "t"
    truncated.mkdir()
    blob = (folder / "s1.safetensors").read_bytes()
    (truncated / "model.safetensors").write_bytes(blob[:-4])
    with pytest.raises(SafetensorsError):
        open_model_shards(truncated)
    (truncated / "model.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError):
        open_model_shards(truncated)
