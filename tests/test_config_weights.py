"""Configuration, registry and weight loading (CPU)."""
import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import helpers
from tinyinfer_b200.config import (EngineConfig, Qwen3Config, known_architectures, load_config,
                                   lookup_architecture, parse_dtype)
from tinyinfer_b200.weights import WeightError, load_weights, random_tensors, write_random_model
import tinyinfer_b200.models  # noqa: F401


def test_config_reads_its_own_keys_and_defaults():
    cfg = Qwen3Config.from_dict(helpers.TINY_BW)
    assert cfg.resolved_head_dim == 32 and cfg.hidden_size // cfg.num_attention_heads == 16
    spec = cfg.model_spec()
    assert [l.mixer.window for l in spec.layers] == [None, 40, None]
    assert spec.layers[0].mixer.scale == 32 ** -0.5
    assert spec.layers[0].mixer.position.theta == 1e6 and spec.layers[0].mixer_norm.eps == 1e-5
    assert not spec.tie_embeddings and spec.vocab_size == 389
    # head_dim falls back to hidden // heads; rope_theta to rope_scaling's, then to 10000
    d = {k: v for k, v in helpers.TINY_A.items() if k not in ("head_dim", "rope_theta")}
    assert Qwen3Config.from_dict(d).resolved_head_dim == 16
    assert Qwen3Config.from_dict(d).rope_theta == 10000.0
    assert Qwen3Config.from_dict(dict(d, rope_scaling={"rope_theta": 77.0})).rope_theta == 77.0
    # use_sliding_window + max_window_layers
    spec = Qwen3Config.from_dict(helpers.TINY_D).model_spec()
    assert [l.mixer.window for l in spec.layers] == [None, 96]
    # a round trip through to_dict
    again = Qwen3Config.from_dict(Qwen3Config.from_dict(helpers.TINY_BW).to_dict())
    assert again.model_spec() == Qwen3Config.from_dict(helpers.TINY_BW).model_spec()


@pytest.mark.parametrize("change,word", [
    (dict(num_key_value_heads=3), "multiple"), (dict(head_dim=15), "even"),
    (dict(hidden_act="gelu"), "hidden_act"), (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(layer_types=["sliding_attention", "full_attention"]), "sliding_window"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(vocab_size=0), "vocab_size")])
def test_config_refuses(change, word):
    with pytest.raises(ValueError, match=word):
        Qwen3Config.from_dict(dict(helpers.TINY_A, **change))


def test_config_missing_keys_are_listed():
    d = {k: v for k, v in helpers.TINY_A.items() if k not in ("intermediate_size", "vocab_size")}
    with pytest.raises(ValueError, match="intermediate_size") as e:
        Qwen3Config.from_dict(d)
    assert "vocab_size" in str(e.value)


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(KeyError, match="Qwen3ForCausalLM"):
        lookup_architecture("LlamaForCausalLM")
    (tmp_path / "config.json").write_text(json.dumps(dict(helpers.TINY_A, architectures=["Nope"])))
    with pytest.raises(KeyError, match="Nope"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in helpers.TINY_A.items() if k != "architectures"}))
    with pytest.raises(ValueError, match="architectures"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY_A))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and isinstance(cfg, Qwen3Config)


def test_engine_config_checks():
    EngineConfig().validate()
    for bad in (dict(max_num_seqs=0), dict(max_num_batched_tokens=0), dict(gpu_memory_utilization=0.0),
                dict(gpu_memory_utilization=1.5), dict(dtype="float16"), dict(kvcache_block_size=0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad).validate()
    assert parse_dtype("bf16") == "bfloat16" and parse_dtype("fp32") == "float32"
    with pytest.raises(ValueError):
        parse_dtype("int8")


def cpu_model(folder):
    arch, cfg = load_config(folder)
    return arch.model_factory(cfg, torch.float32, torch.device("cpu"))


def test_random_folder_loads_and_is_reproducible(tmp_path):
    cfg = Qwen3Config.from_dict(helpers.TINY_BW)
    a = write_random_model(tmp_path / "a", cfg, seed=7)
    b = write_random_model(tmp_path / "b", cfg, seed=7)
    c = write_random_model(tmp_path / "c", cfg, seed=8, dtype="bfloat16")
    ta, tb, tc = (load_file(str(p / "model.safetensors")) for p in (a, b, c))
    assert set(ta) == set(tb) and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"].float())
    assert tc["lm_head.weight"].dtype == torch.bfloat16
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    model = cpu_model(a)
    report = load_weights(model, a)
    assert sorted(report.loaded) == sorted(ta) and not report.skipped_tied
    # packed q, k, v rows in that order; gate then up; norm weights stay float32
    attn = model.blocks[1].mixer
    p = "model.layers.1.self_attn."
    assert torch.equal(attn.w_qkv, torch.cat([ta[p + "q_proj.weight"], ta[p + "k_proj.weight"], ta[p + "v_proj.weight"]]))
    ffn = model.blocks[2].feed_forward
    assert torch.equal(ffn.w_gate_up[:176], ta["model.layers.2.mlp.gate_proj.weight"])
    assert attn.q_norm.dtype == torch.float32 and model.final_norm.weight.dtype == torch.float32
    # a bfloat16 model keeps matrices in bfloat16 and norm weights in float32
    arch, cfgc = load_config(c)
    m16 = arch.model_factory(cfgc, torch.bfloat16, torch.device("cpu"))
    load_weights(m16, c)
    assert m16.embedding.dtype == torch.bfloat16 and m16.blocks[0].mixer_norm.weight.dtype == torch.float32


def test_tied_and_untied_heads(tmp_path):
    tied = write_random_model(tmp_path / "t", Qwen3Config.from_dict(helpers.TINY_A), seed=1)
    tensors = load_file(str(tied / "model.safetensors"))
    assert "lm_head.weight" not in tensors
    model = cpu_model(tied)
    load_weights(model, tied)
    assert model.head is model.embedding
    # a tied model's folder may still carry a head: it is skipped, not an error
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    save_file(tensors, str(tied / "model.safetensors"))
    report = load_weights(cpu_model(tied), tied)
    assert report.skipped_tied == ["lm_head.weight"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(tmp_path / "m", Qwen3Config.from_dict(helpers.TINY_BW), seed=1)
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.0.self_attn.k_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 175)
    tensors["model.norm.weight"] = torch.zeros(95)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(cpu_model(folder), folder)
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.k_proj.weight", "lm_head.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [n for n, _, _ in err.wrong_shape] == ["model.layers.2.mlp.down_proj.weight", "model.norm.weight"]
    text = str(err)
    for word in ("missing", "unexpected", "wrong shapes", "k_proj", "inv_freq", "(96, 175)", "(96, 176)"):
        assert word in text
    with pytest.raises(FileNotFoundError):
        load_weights(cpu_model(folder), tmp_path)


def test_random_tensors_follow_the_expected_names():
    cfg = Qwen3Config.from_dict(helpers.TINY_A)
    t = random_tensors(cfg, 0)
    assert abs(float(t["model.norm.weight"].mean()) - 1.0) < 0.1
    assert abs(float(t["model.embed_tokens.weight"].std()) - 0.02) < 0.005
