"""Configuration (typed reading, registry) and weight loading errors."""
import json
import os

import pytest
import torch

import tiny_configs
from chibillm_b200.config import (ConfigError, Qwen3Config, find_architecture, load_config,
                                  register_architecture, registered_architectures,
                                  unregister_architecture)
from chibillm_b200.engine.model import DecoderModel
from chibillm_b200.parts import Runtime
from chibillm_b200.weights import (Checkpoint, SafetensorsError, WeightError, load_weights,
                                   random_tensors, write_random_model, write_safetensors)

CPU = Runtime(torch.device("cpu"), torch.bfloat16, None)


def test_reads_the_reference_fixture_keys():
    """The keys of the reference's own fixture (tests/fixtures/qwen3_0_6b_config.json)."""
    obj = {"architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "bos_token_id": 151643,
           "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 1024,
           "intermediate_size": 3072, "max_position_embeddings": 40960, "model_type": "qwen3",
           "num_attention_heads": 16, "num_hidden_layers": 28, "num_key_value_heads": 8,
           "rms_norm_eps": 1e-6, "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None,
           "tie_word_embeddings": True, "torch_dtype": "bfloat16", "use_sliding_window": False,
           "vocab_size": 151936}
    c = Qwen3Config.from_dict(obj)
    assert (c.query_width, c.kv_width, c.queries_per_kv_head) == (2048, 1024, 2)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-6 and c.tie_word_embeddings
    spec = c.model_spec()
    assert len(spec.layers) == 28 and len(spec.run_order) == 28
    attn = spec.layers[0].mixer
    assert attn.scale == pytest.approx(128 ** -0.5) and attn.window is None
    assert attn.qk_norm.size == 128 and attn.position.rotary_dim == 128
    assert Qwen3Config.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "max_position_embeddings",
                                 "rms_norm_eps", "rope_theta"])
def test_missing_and_bad_keys_are_named(key):
    obj = tiny_configs.get("A")
    del obj[key]
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(obj)
    assert e.value.code == "missing_field" and key in str(e.value)
    for bad in (0, -3, "x", True):
        obj[key] = bad
        with pytest.raises(ConfigError) as e:
            Qwen3Config.from_dict(obj)
        assert e.value.code == "invalid_field" and key in str(e.value)


@pytest.mark.parametrize("key,value,code", [
    ("model_type", "llama", "unsupported_model_type"), ("hidden_act", "gelu", "unsupported_configuration"),
    ("attention_bias", True, "unsupported_configuration"),
    ("rope_scaling", {"type": "yarn"}, "unsupported_configuration"),
    ("torch_dtype", "float16", "unsupported_configuration"),
    ("quantization_config", {"bits": 4}, "unsupported_configuration"),
    ("num_key_value_heads", 3, "invalid_geometry"), ("head_dim", 15, "invalid_geometry"),
    ("eos_token_id", 256, "invalid_geometry")])
def test_unsupported_values(key, value, code):
    obj = tiny_configs.get("A")
    obj[key] = value
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(obj)
    assert e.value.code == code and key in str(e.value)


def test_windows_per_layer():
    c = Qwen3Config.from_dict(tiny_configs.get("C"))
    assert c.layer_windows == (None, 24, None, 24)
    assert [l.mixer.window for l in c.model_spec().layers] == [None, 24, None, 24]
    obj = tiny_configs.get("D128")
    assert Qwen3Config.from_dict(obj).layer_windows == (None, 200)
    assert Qwen3Config.from_dict(Qwen3Config.from_dict(tiny_configs.get("C")).to_dict()).layer_windows == (None, 24, None, 24)


def test_optional_keys():
    obj = tiny_configs.get("B")
    for k in ("bos_token_id", "eos_token_id", "tie_word_embeddings", "torch_dtype"):
        obj.pop(k)
    c = Qwen3Config.from_dict(obj)
    assert c.eos_token_id is None and c.tie_word_embeddings is False
    obj["hidden_size"], obj["num_attention_heads"] = 96, 8
    obj.pop("head_dim")
    assert Qwen3Config.from_dict(obj).head_dim == 12
    obj.pop("rope_theta")
    obj["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "default"}
    assert Qwen3Config.from_dict(obj).rope_theta == 5e5


def test_registry(tmp_path):
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert find_architecture({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert find_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError) as e:
        find_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert e.value.code == "unsupported_architecture" and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        find_architecture({})
    # another architecture is one entry of the table
    register_architecture("ToyForCausalLM", Qwen3Config.from_dict, Qwen3Config.model_spec, model_type="toy")
    try:
        obj = tiny_configs.get("A")
        obj["architectures"] = ["ToyForCausalLM"]
        (tmp_path / "config.json").write_text(json.dumps(obj))
        arch, config, spec = load_config(str(tmp_path))
        assert arch.name == "ToyForCausalLM" and spec.hidden_size == 64
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", Qwen3Config.from_dict, Qwen3Config.model_spec)
    finally:
        unregister_architecture("ToyForCausalLM")
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError) as e:
        load_config(str(tmp_path))
    assert e.value.code == "invalid_json"
    with pytest.raises(ConfigError) as e:
        load_config(str(tmp_path / "nowhere"))
    assert e.value.code == "file_read_failed"


# ------------------------------------------------------------------ weights
def _model_and_tensors(name="A", seed=0):
    cfg = tiny_configs.get(name)
    spec = Qwen3Config.from_dict(cfg).model_spec()
    model = DecoderModel(spec, CPU)
    return cfg, model, dict(random_tensors(model, seed, torch.bfloat16))


def _write(tmp_path, cfg, tensors):
    d = tmp_path / "m"
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), tensors.items())
    return str(d)


def test_round_trip_and_dtypes(tmp_path):
    cfg, model, tensors = _model_and_tensors("B")
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()      # one tensor stored in 32-bit
    folder = _write(tmp_path, cfg, tensors)
    loaded = load_weights(model, folder, CPU)
    assert set(loaded) == set(tensors)
    assert loaded["model.norm.weight"].dtype == torch.float32                # stays 32-bit
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert all(torch.equal(loaded[n].float(), t.float()) for n, t in tensors.items())
    rt32 = Runtime(torch.device("cpu"), torch.float32, None)
    model32 = DecoderModel(model.spec, rt32)
    assert all(t.dtype == torch.float32 for t in load_weights(model32, folder, rt32).values())
    # q, k, v and gate, up are stacked in the order of the checkpoint
    blk = model.blocks[0]
    p = "model.layers.0."
    assert torch.equal(blk.mixer.qkv, torch.cat([tensors[p + f"self_attn.{n}_proj.weight"] for n in "qkv"]))
    assert torch.equal(blk.feed_forward.gate_up, torch.cat([tensors[p + "mlp.gate_proj.weight"],
                                                            tensors[p + "mlp.up_proj.weight"]]))


def test_one_error_lists_everything(tmp_path):
    cfg, model, tensors = _model_and_tensors("A")
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.int32)
    tensors["stray.tensor"] = torch.zeros(3, dtype=torch.bfloat16)
    tensors["model.layers.7.input_layernorm.weight"] = torch.zeros(64, dtype=torch.bfloat16)
    folder = _write(tmp_path, cfg, tensors)
    with pytest.raises(WeightError) as e:
        load_weights(model, folder, CPU)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.down_proj.weight", "model.norm.weight"]
    assert sorted(err.unexpected) == ["model.layers.7.input_layernorm.weight", "stray.tensor"]
    assert err.wrong_shape == ["model.layers.0.self_attn.q_proj.weight"]
    assert err.wrong_dtype == ["model.layers.0.self_attn.k_norm.weight"]
    text = str(err)
    for name in err.missing + err.unexpected + err.wrong_shape + err.wrong_dtype:
        assert name in text
    assert "stored [64, 63], expected [64, 64]" in text


def test_tied_and_untied_output(tmp_path):
    # tied and no output matrix in the file: the embedding table is used
    cfg, model, tensors = _model_and_tensors("A")
    assert "lm_head.weight" not in tensors
    load_weights(model, _write(tmp_path, cfg, tensors), CPU)
    assert model.output is model.embedding
    # tied, but the file has an output matrix: the file's contents decide
    tensors["lm_head.weight"] = torch.ones(256, 64, dtype=torch.bfloat16)
    load_weights(model, _write(tmp_path, cfg, tensors), CPU)
    assert model.output is not model.embedding and float(model.output[0, 0]) == 1.0
    # untied and absent: missing
    cfg_b, model_b, tensors_b = _model_and_tensors("B")
    del tensors_b["lm_head.weight"]
    with pytest.raises(WeightError) as e:
        load_weights(model_b, _write(tmp_path, cfg_b, tensors_b), CPU)
    assert e.value.missing == ["lm_head.weight"]


def test_random_model_folder_is_reproducible(tmp_path):
    a = write_random_model(tiny_configs.get("C"), str(tmp_path / "a"), seed=4)
    b = write_random_model(tiny_configs.get("C"), str(tmp_path / "b"), seed=4)
    c = write_random_model(tiny_configs.get("C"), str(tmp_path / "c"), seed=5)
    ca, cb, cc = (Checkpoint.open_model(x) for x in (a, b, c))
    assert sorted(ca.names()) == sorted(cb.names())
    assert all(torch.equal(ca.read(n), cb.read(n)) for n in ca.names())
    assert not torch.equal(ca.read("model.embed_tokens.weight"), cc.read("model.embed_tokens.weight"))
    emb = ca.read("model.embed_tokens.weight").float()
    assert 0.015 < float(emb.std()) < 0.025 and abs(float(emb.mean())) < 0.002
    norm = ca.read("model.layers.0.self_attn.q_norm.weight").float()
    assert float(norm.min()) >= 0.9 - 1e-2 and float(norm.max()) <= 1.1 + 1e-2
    assert json.load(open(os.path.join(a, "config.json")))["sliding_window"] == 24


def test_safetensors_header_checks(tmp_path):
    import struct
    good = tmp_path / "good.safetensors"
    write_safetensors(str(good), [("a", torch.arange(6, dtype=torch.float32).view(2, 3)),
                                  ("b", torch.ones(4, dtype=torch.bfloat16))])
    from chibillm_b200.weights import SafetensorsFile
    f = SafetensorsFile(str(good))
    assert torch.equal(f.read("a"), torch.arange(6, dtype=torch.float32).view(2, 3))

    def write_raw(name, header, data):
        blob = json.dumps(header).encode()
        p = tmp_path / name
        p.write_bytes(struct.pack("<Q", len(blob)) + blob + data)
        return str(p)

    cases = {
        "gap": ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8),
        "short": ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}, b"\0" * 4),
        "outside": ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4),
        "trailing": ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8),
        "dtype": ({"a": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4),
    }
    for name, (header, data) in cases.items():
        with pytest.raises(SafetensorsError):
            SafetensorsFile(write_raw(name + ".safetensors", header, data))
    (tmp_path / "tiny.safetensors").write_bytes(b"\1\2")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(tmp_path / "tiny.safetensors"))
    (tmp_path / "huge.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(tmp_path / "huge.safetensors"))


def test_checkpoint_discovery(tmp_path):
    t = {"x": torch.ones(2, dtype=torch.bfloat16), "y": torch.zeros(3, dtype=torch.bfloat16)}
    d1 = tmp_path / "sharded"
    d1.mkdir()
    write_safetensors(str(d1 / "s1.safetensors"), [("x", t["x"])])
    write_safetensors(str(d1 / "s2.safetensors"), [("y", t["y"])])
    with pytest.raises(SafetensorsError) as e:
        Checkpoint.open_model(str(d1))
    assert "ambiguous_checkpoint" in str(e.value)
    (d1 / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    ck = Checkpoint.open_model(str(d1))
    assert sorted(ck.names()) == ["x", "y"] and torch.equal(ck.read("y"), t["y"])
    (d1 / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "s1.safetensors"}}))
    write_safetensors(str(d1 / "s1.safetensors"), [("x", t["x"]), ("z", t["y"])])
    with pytest.raises(SafetensorsError):
        Checkpoint.open_model(str(d1))
    d2 = tmp_path / "single"
    d2.mkdir()
    write_safetensors(str(d2 / "weights.safetensors"), t.items())
    assert sorted(Checkpoint.open_model(str(d2)).names()) == ["x", "y"]
    with pytest.raises(SafetensorsError):
        Checkpoint.open_model(str(tmp_path / "nowhere"))
