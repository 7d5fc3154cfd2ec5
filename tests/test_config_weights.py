"""Configuration, registry, safetensors reading/writing and weight errors (no GPU)."""

import json
import os
import struct

import pytest
import torch

from helpers import TINY, seeded_state, write_model_dir
from stride_b200.config import (ConfigError, EngineConfig, LlamaConfig, config_from_dict, load_config, preset,
                                registered_architectures)
from stride_b200.engine.loading import _declarations, write_random_model
from stride_b200.weights import (DictSource, RandomSource, SafetensorsSource, TensorDecl, WeightFileError,
                                 WeightMismatchError, check_source, load_weights, save_file)


def test_tiny_configs_are_read_with_every_field():
    a, b = config_from_dict(TINY["A"]), config_from_dict(TINY["B"])
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (a.intermediate_size, a.vocab_size, a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings) == (192, 256, 10000.0, 1e-5, False)
    assert a.rope_scaling is None and a.max_position_embeddings == 256 and a.group == 2
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (3, 96, 3, 1, 32)
    assert b.tie_word_embeddings and b.rms_norm_eps == 1e-6 and b.rope_theta == 500000.0
    s = b.rope_scaling
    assert (s.rope_type, s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == ("llama3", 8.0, 1.0, 4.0, 64)
    spec = b.to_model_spec()
    assert spec.head_name is None and len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.prefix == "model.layers.1.self_attn." and spec.layers[1].mixer.scale == 32 ** -0.5
    assert spec.layers[2].mixer_norm.eps == 1e-6 and spec.layers[0].feed_forward.intermediate == 256


def test_defaults_follow_the_reference_and_required_keys_are_required():
    d = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_attention_heads": 4, "num_hidden_layers": 1,
         "vocab_size": 10, "intermediate_size": 8}
    c = config_from_dict(d)
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta, c.max_position_embeddings) == (4, 16, 1e-5, 10000.0, 8192)
    for key in ("hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size", "intermediate_size"):
        bad = dict(d)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            config_from_dict(bad)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "do not divide"), ({"hidden_act": "gelu"}, "hidden_act"), ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"), ({"vocab_size": 0}, "vocab_size"),
    ({"hidden_size": "64"}, "hidden_size"), ({"head_dim": 15}, "even"), ({"architectures": ["GPT2LMHeadModel"]}, "LlamaForCausalLM"),
    ({"architectures": [], "model_type": "other"}, "names no architecture"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_bad_configs_are_refused(change, match):
    d = dict(TINY["A"])
    d.update(change)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(d)


def test_what_config_json_leaves_out_is_settled_as_the_reference_does():
    """No ``architectures``: placed by ``model_type``. No ``tie_word_embeddings`` or ``attention_bias``: the
    checkpoint's contents decide (python/stride_worker/model.py:127-128,159-169); a key that is given stands."""
    d = {k: v for k, v in TINY["A"].items() if k not in ("architectures", "tie_word_embeddings")}
    assert type(config_from_dict(d)) is LlamaConfig
    names = {"model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.q_proj.bias"}
    c = config_from_dict(d, tensor_names=names)
    assert c.tie_word_embeddings and c.attention_bias
    c = config_from_dict(d, tensor_names=(names - {"model.layers.0.self_attn.q_proj.bias"}) | {"lm_head.weight"})
    assert not c.tie_word_embeddings and not c.attention_bias
    given = dict(d, tie_word_embeddings=False, attention_bias=False)
    c = config_from_dict(given, tensor_names=names)
    assert not c.tie_word_embeddings and not c.attention_bias
    assert not config_from_dict(d).tie_word_embeddings, "without a checkpoint the default of the reference stands"


def test_registry_and_round_trip(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    c = config_from_dict(TINY["B"])
    assert config_from_dict(c.to_dict()) == c
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "nowhere"))
    legacy = dict(TINY["B"])
    legacy["rope_scaling"] = dict(legacy["rope_scaling"])
    legacy["rope_scaling"]["type"] = legacy["rope_scaling"].pop("rope_type")
    assert config_from_dict(legacy).rope_scaling == c.rope_scaling


def test_parameter_and_cache_arithmetic_of_the_named_shapes():
    c8, c70, c3 = (config_from_dict(preset(n)) for n in ("llama3.1-8b", "llama3.1-70b", "llama3.2-3b"))
    assert c8.total_params() == 8_030_261_248          # the published 8.03e9
    assert c70.total_params(with_norms=False) == 70_552_387_584
    assert c8.kv_bytes_per_token(2) == 128 * 1024 and c70.kv_bytes_per_token(2) == 320 * 1024   # README.md:118-119 of the reference
    assert c3.tie_word_embeddings and c3.kv_bytes_per_token(2) == 114_688


def test_engine_config_is_validated():
    assert EngineConfig().block_size == 16 and EngineConfig().max_batch_tokens == 2048
    assert EngineConfig().max_queued == 1024 and EngineConfig().max_batch_seqs == 256 and EngineConfig().max_model_len == 8192
    for bad in ({"dtype": "float16"}, {"block_size": 0}, {"activation_reserve": 1.0}, {"max_batch_seqs": 0}, {"max_queued": 0}):
        with pytest.raises(ValueError):
            EngineConfig(**bad)


# ------------------------------------------------------------------------ weights
def test_safetensors_round_trip_with_the_reference_package(tmp_path):
    from safetensors.torch import load_file, save_file as their_save
    g = torch.Generator().manual_seed(0)
    tensors = {"b.weight": torch.randn(3, 5, generator=g).bfloat16(), "a": torch.randn(7, generator=g),
               "ids": torch.arange(6, dtype=torch.int32).view(2, 3), "scalar": torch.tensor(2.5), "empty": torch.zeros(0, 4)}
    save_file(tensors, str(tmp_path / "ours.safetensors"), metadata={"k": "v"})
    theirs = load_file(str(tmp_path / "ours.safetensors"))
    assert set(theirs) == set(tensors) and all(torch.equal(theirs[k], v) and theirs[k].dtype == v.dtype for k, v in tensors.items())
    their_save(tensors, str(tmp_path / "model.safetensors"))
    src = SafetensorsSource(str(tmp_path))
    assert sorted(src.names()) == sorted(set(tensors) | set())  # both files are shards of this folder
    assert all(torch.equal(src.read(k), v) for k, v in tensors.items())
    assert src.describe("b.weight") == ((3, 5), torch.bfloat16)


def test_shards_follow_the_index_file(tmp_path):
    save_file({"x": torch.ones(2)}, str(tmp_path / "part-1.safetensors"))
    save_file({"y": torch.zeros(3)}, str(tmp_path / "part-2.safetensors"))
    save_file({"z": torch.zeros(3)}, str(tmp_path / "stray.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "part-1.safetensors", "y": "part-2.safetensors"}}))
    assert sorted(SafetensorsSource(str(tmp_path)).names()) == ["x", "y"]
    with pytest.raises(FileNotFoundError, match="no .safetensors"):
        SafetensorsSource(str(tmp_path / "empty"))


def test_broken_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="too short"):
        SafetensorsSource(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsSource(str(tmp_path))
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(WeightFileError, match="offsets"):
        SafetensorsSource(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_misshapen_tensors():
    cfg = config_from_dict(TINY["A"])
    declared = _declarations(cfg)
    state = seeded_state(TINY["A"], 1)
    check_source(DictSource(state), declared, cfg.to_model_spec().ignorable_tensors)
    state["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # ignorable, as in the reference
    check_source(DictSource(state), declared, cfg.to_model_spec().ignorable_tensors)
    del state["model.layers.1.mlp.up_proj.weight"], state["model.norm.weight"]
    state["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    state["model.layers.7.mlp.up_proj.weight"] = torch.zeros(1)
    state["lm_head.weight"] = torch.zeros(255, 64)
    state["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 64, dtype=torch.int32)
    with pytest.raises(WeightMismatchError) as e:
        check_source(DictSource(state), declared, cfg.to_model_spec().ignorable_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias", "model.layers.7.mlp.up_proj.weight"]
    assert [w[0] for w in err.wrong_shape] == ["lm_head.weight"] and err.wrong_shape[0][1:] == ((255, 64), (256, 64))
    assert [w[0] for w in err.wrong_kind] == ["model.layers.0.self_attn.k_proj.weight"]
    text = str(err)
    for name in err.missing + err.unexpected + ["lm_head.weight", "[255, 64]", "[256, 64]"]:
        assert name in text


def test_a_tied_model_must_not_carry_a_head_and_an_untied_one_must():
    tied = _declarations(config_from_dict(TINY["B"]))
    assert "lm_head.weight" not in tied
    state = seeded_state(TINY["B"], 1)
    state["lm_head.weight"] = torch.zeros(384, 96)
    with pytest.raises(WeightMismatchError, match="unexpected"):
        check_source(DictSource(state), tied)
    untied = seeded_state(TINY["A"], 1)
    del untied["lm_head.weight"]
    with pytest.raises(WeightMismatchError, match="missing"):
        check_source(DictSource(untied), _declarations(config_from_dict(TINY["A"])))


def test_element_types_on_load():
    declared = {"m": TensorDecl((2, 2)), "v": TensorDecl((2,), "vector"), "t": TensorDecl((3,), "table")}
    state = {"m": torch.ones(2, 2), "v": torch.ones(2, dtype=torch.bfloat16), "t": torch.arange(3)}
    bf = load_weights(DictSource(state), declared, torch.bfloat16, "cpu")
    assert (bf["m"].dtype, bf["v"].dtype, bf["t"].dtype) == (torch.bfloat16, torch.float32, torch.int32)
    state["v"] = torch.tensor([1.0000001, 2.0])      # stored in 32 bits: kept as it is
    f = load_weights(DictSource(state), declared, torch.bfloat16, "cpu")
    assert torch.equal(f["v"], state["v"])
    assert load_weights(DictSource(state), declared, torch.float32, "cpu")["m"].dtype == torch.float32


def test_random_weights_are_seeded_and_written_as_a_model_folder(tmp_path):
    cfg = config_from_dict(TINY["B"])
    a = write_random_model(cfg, 5, str(tmp_path / "a"), vector_jitter=0.1)
    b = write_random_model(cfg, 5, str(tmp_path / "b"), vector_jitter=0.1)
    c = write_random_model(cfg, 6, str(tmp_path / "c"), stored_dtype="float32")
    sa, sb, sc = SafetensorsSource(a), SafetensorsSource(b), SafetensorsSource(c)
    assert sorted(sa.names()) == sorted(_declarations(cfg))
    assert all(torch.equal(sa.read(n), sb.read(n)) for n in sa.names())
    assert not torch.equal(sa.read("model.embed_tokens.weight").float(), sc.read("model.embed_tokens.weight"))
    assert sc.describe("model.norm.weight")[1] == torch.float32 and torch.equal(sc.read("model.norm.weight"), torch.ones(96))
    w = sa.read("model.layers.1.mlp.down_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert load_config(a) == cfg
    src = RandomSource(_declarations(cfg), 5, vector_jitter=0.1)
    order1 = [src.read(n) for n in sorted(src.names())]
    order2 = [src.read(n) for n in sorted(src.names(), reverse=True)][::-1]
    assert all(torch.equal(x, y) for x, y in zip(order1, order2)), "a tensor's values depend on the order of reads"


def test_the_memory_plan_subtracts_weights_and_reserve_and_refuses_what_cannot_run():
    """crates/stride-model/src/memory.rs:67-121 on one device: the cache is what weights and the reserve leave."""
    from stride_b200.config import B200_MEMORY_BYTES, PlanError, plan_memory
    c8 = config_from_dict(preset("llama3.1-8b"))
    plan = plan_memory(c8, "bfloat16", block_size=16, activation_fraction=0.15)
    matrices = c8.total_params(with_norms=False)
    assert plan.weight_bytes == matrices * 2 + (c8.total_params() - matrices) * 4
    after = B200_MEMORY_BYTES - plan.weight_bytes
    assert plan.activation_reserve_bytes == int(after * 0.15) and plan.kv_bytes == after - plan.activation_reserve_bytes
    assert plan.kv_bytes_per_token == 131072 and plan.num_blocks == plan.kv_bytes // (131072 * 16)
    assert plan.max_context() == plan.num_blocks * 16
    assert plan.concurrent_sequences(8192) == plan.num_blocks // 512 and plan.concurrent_sequences(0) == 0
    assert plan.concurrent_sequences(8193) == plan.num_blocks // 513
    assert "pages of 16" in plan.describe()
    # the 70B shape in bfloat16 leaves tens of GiB of pages on one B200; in float32 its weights alone do not fit
    c70 = config_from_dict(preset("llama3.1-70b"))
    p70 = plan_memory(c70, "bfloat16")
    assert 130 < p70.weight_bytes / 2**30 < 133 and p70.kv_bytes_per_token == 327680 and p70.total_kv_tokens > 90_000
    with pytest.raises(PlanError, match="weights need"):
        plan_memory(c70, "float32")
    with pytest.raises(PlanError, match="one page"):
        plan_memory(c8, "bfloat16", memory_bytes=plan.weight_bytes + 1_000_000)
    with pytest.raises(PlanError):
        plan_memory(c8, "float16")
    with pytest.raises(PlanError):
        plan_memory(c8, activation_fraction=1.0)
    # a larger reserve or a float32 cache leaves fewer pages
    assert plan_memory(c8, activation_fraction=0.5).num_blocks < plan.num_blocks
    assert plan_memory(c8, "float32").kv_bytes_per_token == 262144


def test_the_plan_command_line(capsys):
    from stride_b200.cli import main
    assert main(["plan", "--preset", "llama3.2-3b", "--context", "4096"]) == 0
    out = capsys.readouterr().out
    assert "llama3.2-3b in bfloat16" in out and "requests of 4096" in out and "114688 bytes a token" in out
    assert main(["plan", "--preset", "llama3.1-70b", "--dtype", "float32"]) == 1
    assert "does not fit" in capsys.readouterr().err
