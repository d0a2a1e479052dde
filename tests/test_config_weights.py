"""Configuration, registry and weight loading: what is read, what is refused, and how errors read (CPU only)."""
from __future__ import annotations

import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from cuinfer_b200.models.qwen3 import Qwen3Config
from cuinfer_b200.config import (ConfigError, EngineConfig, get_architecture, known_architectures,
                                 load_model_config, register_architecture, unregister_architecture)
from cuinfer_b200.parts import DecoderModel
from cuinfer_b200.weights import Checkpoint, WeightError, WeightStore, write_random_model, write_safetensors


def test_config_reads_every_key_and_defaults():
    cfg = Qwen3Config.from_dict(TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 8, 2)
    assert (cfg.head_dim, cfg.q_size, cfg.kv_size) == (32, 256, 64)
    assert cfg.intermediate_size == 320 and cfg.vocab_size == 1000
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    assert cfg.eos_token_ids == (7, 9) and cfg.max_model_len == 768
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert Qwen3Config.from_dict(raw).head_dim == 64 // 4      # hidden_size // heads when absent
    assert Qwen3Config.from_dict(Qwen3Config.from_dict(TINY_B).to_dict()) == cfg


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta",
                                 "max_position_embeddings", "tie_word_embeddings"])
def test_config_missing_key_is_named(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("change, word", [
    ({"use_sliding_window": True}, "sliding"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"factor": 2.0}}, "rope_scaling"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"torch_dtype": "float16"}, "data type"), ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"), ({"vocab_size": 0}, "positive"), ({"hidden_size": "64"}, "integer"),
])
def test_config_refuses_what_is_not_built(change, word):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(raw)


def test_registry_maps_name_to_model_and_refuses_unknown(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    arch = get_architecture("Qwen3ForCausalLM")
    spec = arch.spec(arch.parse(TINY_A))
    assert len(spec.layers) == 2 and spec.lm_head_name is None and spec.layers[0].mixer.head_dim == 16
    with pytest.raises(ConfigError, match="unsupported model architecture.*LlamaForCausalLM"):
        get_architecture("LlamaForCausalLM")
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["Nope"])))
    with pytest.raises(ConfigError, match="Nope"):
        load_model_config(str(tmp_path))
    with pytest.raises(ConfigError, match="cannot open"):
        load_model_config(str(tmp_path / "missing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="invalid model config"):
        load_model_config(str(tmp_path))


def test_registry_takes_a_new_architecture():
    register_architecture("ToyForCausalLM", Qwen3Config.from_dict, get_architecture("Qwen3ForCausalLM").spec)
    try:
        assert get_architecture("ToyForCausalLM").parse(dict(TINY_A, architectures=["ToyForCausalLM"])).hidden_size == 64
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", None, None)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_generation_config_overrides_eos(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [11, 12]}))
    _, cfg = load_model_config(str(tmp_path))
    assert cfg.eos_token_ids == (11, 12)


def test_engine_config_ranges():
    EngineConfig(model_path="x")
    for bad in (dict(gpu_memory_utilization=0.0), dict(gpu_memory_utilization=0.99), dict(block_size=0),
                dict(max_num_seqs=0), dict(max_num_scheduled_tokens=-1), dict(dtype="float16"), dict(num_blocks=0),
                dict(enable_prefix_caching=True)):
        with pytest.raises(ConfigError):
            EngineConfig(model_path="x", **bad)


# ---- weights ---------------------------------------------------------------------------------------

def _store(folder, dtype=torch.float32):
    return WeightStore(folder, dtype, "cpu")


def _model(cfg, dtype=torch.float32):
    arch = get_architecture("Qwen3ForCausalLM")
    return DecoderModel(arch.spec(arch.parse(cfg)), dtype)


def test_random_model_round_trip_and_determinism(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, 5, gain_std=0.1)
    b = write_random_model(str(tmp_path / "b"), TINY_B, 5, gain_std=0.1)
    c = write_random_model(str(tmp_path / "c"), TINY_B, 6, gain_std=0.1)
    ca, cb, cc = Checkpoint(a), Checkpoint(b), Checkpoint(c)
    names = sorted(ca.names())
    assert names == sorted(t.name for t in _model(TINY_B).tensors())
    assert "lm_head.weight" in names                       # untied
    assert all(torch.equal(ca.tensor(n), cb.tensor(n)) for n in names)
    assert not torch.equal(ca.tensor("model.embed_tokens.weight"), cc.tensor("model.embed_tokens.weight"))
    from safetensors.torch import load_file            # the file format, checked against the library reader
    lib = load_file(os.path.join(a, "model.safetensors"))
    assert all(torch.equal(lib[n], ca.tensor(n)) for n in names)
    tied = write_random_model(str(tmp_path / "t"), TINY_A, 0)
    assert "lm_head.weight" not in Checkpoint(tied).names()
    _, cfg = load_model_config(tied)
    assert cfg.hidden_size == 64


def test_precision_rule(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0, dtype="bfloat16")
    # store one gain in 32 bits beside the bfloat16 rest
    ck = Checkpoint(folder)
    tensors = {n: ck.tensor(n) for n in ck.names()}
    ck.close()
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["extra.int_table"] = torch.arange(6, dtype=torch.int64).reshape(2, 3)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    from cuinfer_b200.parts import TensorSpec
    bf = _store(folder, torch.bfloat16)
    assert bf.get(TensorSpec("model.norm.weight", (64,), keep_stored_precision=True)).dtype == torch.float32
    assert bf.get(TensorSpec("model.layers.0.input_layernorm.weight", (64,), keep_stored_precision=True)).dtype == torch.bfloat16
    assert bf.get(TensorSpec("model.embed_tokens.weight", (256, 64))).dtype == torch.bfloat16
    assert bf.get(TensorSpec("extra.int_table", (2, 3))).dtype == torch.int32
    f32 = _store(folder, torch.float32)
    assert f32.get(TensorSpec("model.embed_tokens.weight", (256, 64))).dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    ck = Checkpoint(folder)
    tensors = {n: ck.tensor(n) for n in ck.names()}
    ck.close()
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.layers.0.self_attn.q_norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(48, 64)
    tensors["model.layers.1.self_attn.v_proj.weight"] = torch.zeros(32, 64, dtype=torch.int32)   # right shape, integers
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    store = _store(folder)
    with pytest.raises(WeightError) as err:
        store.check(_model(TINY_A).tensors())
    msg = str(err.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.down_proj.weight" in msg and "q_norm.weight" in msg
    assert "unexpected (1)" in msg and "q_proj.bias" in msg
    assert "wrong shape or dtype (2)" in msg and "k_proj.weight: expected [32, 64], got [48, 64]" in msg
    assert "v_proj.weight: expected a floating dtype, got torch.int32" in msg
    # and the other way round: a part that asks for an integer table refuses a floating tensor in its place
    from cuinfer_b200.parts.spec import TensorSpec
    with pytest.raises(WeightError, match="model.norm.weight: expected an integer dtype, got torch.float32"):
        _store(folder).check([TensorSpec("model.norm.weight", (64,), integer=True)] +
                             [TensorSpec(n, tuple(t.shape), integer=not t.is_floating_point) for n, t in tensors.items()
                              if n != "model.norm.weight"])


@pytest.mark.parametrize("damage, word", [
    (lambda raw: raw[:4], "shorter"),
    (lambda raw: struct.pack("<Q", 1 << 40) + raw[8:], "header size"),
    (lambda raw: raw[:8] + b"{" * (struct.unpack("<Q", raw[:8])[0]) + raw[8 + struct.unpack("<Q", raw[:8])[0]:], "header"),
])
def test_damaged_file_is_reported(tmp_path, damage, word):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    path = os.path.join(folder, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(damage(raw))
    with pytest.raises(WeightError, match=word):
        Checkpoint(folder)


def test_bad_offsets_dtype_and_missing_file(tmp_path):
    def write(header, payload=b"\0" * 16):
        blob = json.dumps(header).encode()
        (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(blob)) + blob + payload)
    write({"x": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}})
    with pytest.raises(WeightError, match="data_offsets"):
        Checkpoint(str(tmp_path))
    write({"x": {"dtype": "F64", "shape": [2], "data_offsets": [0, 16]}})
    with pytest.raises(WeightError, match="unsupported safetensors dtype F64"):
        Checkpoint(str(tmp_path))
    with pytest.raises(WeightError, match="cannot open"):
        Checkpoint(str(tmp_path / "nowhere"))
    # the same name twice in a header: an error (csrc/model/checkpoint.cpp:121-124), not "the last one wins"
    entry = '{"dtype": "F32", "shape": [2], "data_offsets": [%d, %d]}'
    blob = ('{"x": ' + entry % (0, 8) + ', "y": ' + entry % (8, 16) + ', "x": ' + entry % (8, 16) + '}').encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(blob)) + blob + b"\0" * 16)
    with pytest.raises(WeightError, match="duplicate tensor 'x'"):
        Checkpoint(str(tmp_path))


def test_sharded_checkpoint(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    ck = Checkpoint(folder)
    tensors = {n: ck.tensor(n) for n in ck.names()}
    ck.close()
    os.remove(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(folder, "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(folder, "s2.safetensors"), {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    sharded = Checkpoint(folder)
    assert sorted(sharded.names()) == names
    assert all(torch.equal(sharded.tensor(n), tensors[n]) for n in names)
    index["weight_map"]["ghost"] = "s1.safetensors"
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh)
    with pytest.raises(WeightError, match="ghost"):
        Checkpoint(folder)


def test_counter_generator_is_a_function_of_seed_name_and_index(tmp_path):
    """The generator behind device-side random weights, on the host: element i depends on (seed, name, i) only —
    a prefix of a longer draw is the shorter draw, another name or seed gives other values — the moments are those
    of a normal, and a folder without tensors names its recipe instead."""
    from cuinfer_b200.weights import counter_normal, random_tensors
    from cuinfer_b200.weights.random_init import RANDOM_MARKER

    a = counter_normal(77, 5000, 0.0, 1.0)
    assert torch.equal(a[:1234], counter_normal(77, 1234, 0.0, 1.0))
    assert not torch.equal(a, counter_normal(78, 5000, 0.0, 1.0))
    big = counter_normal(5, 400000, 0.0, 1.0)
    assert abs(float(big.mean())) < 0.01 and abs(float(big.std()) - 1.0) < 0.01 and 4.0 < float(big.abs().max()) <= 6.0
    assert torch.equal(counter_normal(5, 100, 1.0, 0.1, 2.0), ((1.0 + 0.1 * counter_normal(5, 100, 0.0, 1.0).double()).float() * 2.0))
    t1 = random_tensors(TINY_A, 3, generator="counter", gain_std=0.1, gains={"q_norm": 2.0})
    t2 = random_tensors(TINY_A, 3, generator="counter", gain_std=0.1, gains={"q_norm": 2.0})
    assert all(torch.equal(t1[k], t2[k]) for k in t1)
    assert abs(float(t1["model.layers.0.self_attn.q_norm.weight"].mean()) - 2.0) < 0.2
    folder = write_random_model(str(tmp_path / "m"), TINY_A, 3, generator="counter", materialize=False, dtype="bfloat16")
    assert sorted(os.listdir(folder)) == ["config.json", RANDOM_MARKER]
    with pytest.raises(ValueError, match="generator='counter'"):
        write_random_model(str(tmp_path / "n"), TINY_A, 3, materialize=False)
