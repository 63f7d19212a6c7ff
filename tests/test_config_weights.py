"""Configuration, registry, safetensors files and weight errors (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from airun_b200.config import (ConfigError, Qwen3Config, load_config, lookup_architecture,
                               registered_architectures)
from airun_b200.engine.model import DecoderModel
from airun_b200.weights import (DictSource, SafetensorsError, SafetensorsFolder, WeightError, check_source,
                                load_tensors, random_tensors, write_model_folder, write_safetensors)
from helpers import TINY


def test_defaults_and_derived_sizes():
    c = Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], vocab_size=1000, hidden_size=128,
                                   num_hidden_layers=2, num_attention_heads=8, intermediate_size=256))
    assert c.num_key_value_heads == 8 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.max_position_embeddings == 4096
    assert not c.tie_word_embeddings and c.layer_windows == ()
    assert c.q_dim == 128 and c.kv_dim == 128 and c.gqa_ratio == 1
    assert c.kv_bytes_per_token(2) == 2 * 128 * 2 * 2


def test_8b_shape_cache_bytes():
    c = Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096,
                                   num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                                   head_dim=128, intermediate_size=12288))
    assert c.kv_bytes_per_token(2) == 147456          # 144 KiB per token in bfloat16
    assert c.attn_scale == 128 ** -0.5


def test_1_7b_shape_matches_the_reference_config_tests():
    """crates/airun-core/src/config.rs:977-991: q_dim 2048, kv_dim 1024, two query heads per KV head,
    16 MiB of 16-bit keys and values per layer at 4,096 tokens, 28 layers."""
    c = Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=2048,
                                   num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                                   head_dim=128, intermediate_size=6144, tie_word_embeddings=True))
    assert (c.q_dim, c.kv_dim, c.gqa_ratio) == (2048, 1024, 2)
    assert c.kv_bytes_per_token(2) * 4096 == 28 * 16 * 1024 * 1024
    with pytest.raises(ConfigError):                                     # config.rs:994-1006: 5 KV heads do not divide 16
        Qwen3Config.from_dict(dict(c.to_dict(), num_key_value_heads=5))


def test_missing_keys_are_all_named():
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], hidden_size=64))
    msg = str(e.value)
    for k in ("vocab_size", "num_hidden_layers", "num_attention_heads", "intermediate_size"):
        assert k in msg


def test_every_problem_is_listed():
    bad = dict(TINY["A"]["cfg"], num_key_value_heads=3, head_dim=15, rope_scaling={"type": "yarn"},
               attention_bias=True, hidden_act="gelu")
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(bad)
    msg = str(e.value)
    for frag in ("multiple of num_key_value_heads", "head_dim", "rope_scaling", "attention_bias", "hidden_act"):
        assert frag in msg


def test_rotary_constants_in_a_dictionary():
    """Newer config.json files keep rope_theta inside ``rope_parameters``; the plain type is read,
    a top-level rope_theta wins, and every scaling rule is refused."""
    base = {k: v for k, v in TINY["A"]["cfg"].items() if k != "rope_theta"}
    assert Qwen3Config.from_dict(dict(base, rope_parameters={"rope_type": "default", "rope_theta": 5e5})).rope_theta == 5e5
    assert Qwen3Config.from_dict(dict(base, rope_theta=777.0, rope_parameters={"rope_theta": 5e5})).rope_theta == 777.0
    assert Qwen3Config.from_dict(dict(base, rope_scaling={"rope_type": "default"})).rope_theta == 10000.0
    for bad in ({"rope_type": "yarn", "factor": 4.0}, {"type": "linear", "factor": 2.0}, {"rope_type": "default", "factor": 2.0}):
        with pytest.raises(ConfigError, match="rope_scaling"):
            Qwen3Config.from_dict(dict(base, rope_scaling=bad))


def test_windows_from_layer_types_and_max_window_layers():
    c = Qwen3Config.from_dict(TINY["C"]["cfg"])
    assert c.layer_windows == (0, 24, 0, 24)
    d = dict(TINY["C"]["cfg"])
    del d["layer_types"]
    d["max_window_layers"] = 3
    assert Qwen3Config.from_dict(d).layer_windows == (0, 0, 0, 24)
    d["use_sliding_window"] = False
    assert Qwen3Config.from_dict(d).layer_windows == ()


def test_round_trip_and_registry(tmp_path):
    for name, spec in TINY.items():
        c = Qwen3Config.from_dict(spec["cfg"])
        assert Qwen3Config.from_dict(c.to_dict()) == c
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError) as e:
        lookup_architecture("NoSuchModel")
    assert "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_layer_specs_carry_every_constant():
    c = Qwen3Config.from_dict(TINY["C"]["cfg"])
    specs = c.layer_specs()
    assert len(specs) == 4
    assert specs[1].mixer_args["window"] == 24 and specs[0].mixer_args["window"] == 0
    assert specs[0].mixer_args["position_args"] == dict(rotary_dim=48, theta=500000.0)
    assert specs[0].norm_args == dict(size=80, eps=3e-6)
    assert specs[0].ffn_args == dict(hidden_size=80, intermediate_size=176)


def _model(name="A"):
    cfg = Qwen3Config.from_dict(TINY[name]["cfg"])
    return cfg, DecoderModel(cfg, torch.float32, "cpu")


def test_weight_names_of_the_architecture():
    cfg, m = _model("B")
    names = {s.name for s in m.weight_specs()}
    assert "model.embed_tokens.weight" in names and "lm_head.weight" in names and "model.norm.weight" in names
    for l in range(3):
        for suffix in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                       "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                       "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight",
                       "mlp.up_proj.weight", "mlp.down_proj.weight"):
            assert f"model.layers.{l}.{suffix}" in names
    shapes = {s.name: s.shape for s in m.weight_specs()}
    assert shapes["model.layers.0.self_attn.q_proj.weight"] == (256, 96)       # heads*head_dim != hidden
    assert shapes["model.layers.0.self_attn.k_proj.weight"] == (32, 96)
    assert shapes["model.layers.0.self_attn.o_proj.weight"] == (96, 256)
    _, tied = _model("A")
    assert "lm_head.weight" not in {s.name for s in tied.weight_specs()}


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    cfg, m = _model("A")
    t = random_tensors(m.weight_specs(), 1)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 10, dtype=torch.bfloat16)
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    with pytest.raises(WeightError) as e:
        m.load(DictSource(t))
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (10, 10), (64, 64))]
    msg = str(err)
    for frag in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[10, 10]", "[64, 64]"):
        assert frag in msg


def test_tied_model_ignores_a_stored_head_and_untied_needs_it():
    cfg, m = _model("A")
    t = random_tensors(m.weight_specs(), 1)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    m.load(DictSource(t))
    assert m.head.weight is m.embedding.table          # the table itself, not a copy
    cfgb, mb = _model("B")
    tb = random_tensors(mb.weight_specs(), 1)
    del tb["lm_head.weight"]
    with pytest.raises(WeightError) as e:
        mb.load(DictSource(tb))
    assert e.value.missing == ["lm_head.weight"]


def test_storage_types():
    cfg, m = _model("A")
    specs = m.weight_specs()
    t = random_tensors(specs, 1)
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.norm.weight"].dtype == torch.float32
    bf = load_tensors(specs, DictSource(t), torch.bfloat16, "cpu")
    assert bf["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert bf["model.layers.0.input_layernorm.weight"].dtype == torch.float32     # stored in 32-bit, stays so
    f32 = load_tensors(specs, DictSource(t), torch.float32, "cpu")
    assert f32["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    assert torch.equal(f32["model.layers.0.mlp.down_proj.weight"],
                       t["model.layers.0.mlp.down_proj.weight"].float())
    from airun_b200.weights.loader import WeightSpec, stored_dtype
    assert stored_dtype(WeightSpec("t", (4,), storage="as_stored"), torch.int64, torch.bfloat16) == torch.int32
    assert stored_dtype(WeightSpec("t", (4,), storage="as_stored"), torch.float32, torch.bfloat16) == torch.float32
    assert stored_dtype(WeightSpec("t", (4,), storage="as_stored"), torch.bfloat16, torch.bfloat16) == torch.bfloat16


def test_random_weights_are_seeded_and_independent_of_order():
    cfg, m = _model("A")
    specs = m.weight_specs()
    a = random_tensors(specs, 5)
    b = random_tensors(list(reversed(specs)), 5)
    c = random_tensors(specs, 6)
    for n in a:
        assert torch.equal(a[n], b[n])
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002
    nw = a["model.layers.0.input_layernorm.weight"]
    assert abs(float(nw.mean()) - 1.0) < 0.05 and 0.05 < float(nw.std()) < 0.15


def test_model_folder_round_trip(tmp_path):
    cfg, m = _model("B")
    d = str(tmp_path / "m")
    write_model_folder(d, cfg, m.weight_specs(), seed=9)
    assert load_config(d) == cfg
    folder = SafetensorsFolder(d)
    want = random_tensors(m.weight_specs(), 9)
    assert set(folder.names()) == set(want)
    for n in want:
        assert torch.equal(folder.read(n), want[n])
    from safetensors.torch import load_file          # an independent reader agrees
    other = load_file(os.path.join(d, "model.safetensors"))
    for n in want:
        assert torch.equal(other[n], want[n])
    m.load(folder)
    folder.close()


def test_broken_safetensors_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # payload truncated
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFolder(str(tmp_path))
    assert "truncated" in str(e.value)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)         # count does not match the span
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    hdr = json.dumps({"a": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    os.unlink(p)
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))


def test_sharded_folder(tmp_path):
    write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.arange(4.0)})
    write_safetensors(str(tmp_path / "s2.safetensors"), {"b": torch.arange(3, dtype=torch.int64)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    f = SafetensorsFolder(str(tmp_path))
    assert sorted(f.names()) == ["a", "b"]
    assert torch.equal(f.read("b"), torch.arange(3, dtype=torch.int64))
    f.close()


def test_inspect_subcommand_describes_a_folder_and_says_whether_it_loads(tmp_path, capsys):
    """``airun inspect`` (options of crates/airun-cli/src/inspect.rs:10-36) needs no GPU."""
    from airun_b200.cli import main
    cfg, m = _model("B")
    good = str(tmp_path / "good")
    write_model_folder(good, cfg, m.weight_specs(), seed=4)
    assert main(["inspect", good]) == 0
    out = capsys.readouterr().out
    assert "Qwen3ForCausalLM" in out and "every tensor the architecture wants is there" in out
    assert main(["inspect", good, "--tensors", "--json"]) == 0
    rep = json.loads(capsys.readouterr().out)
    want = random_tensors(m.weight_specs(), 4)
    assert rep["loadable"] and rep["tensor_count"] == len(want) and rep["config"]["hidden_size"] == cfg.hidden_size
    assert {t["name"]: tuple(t["shape"]) for t in rep["tensors"]} == {n: tuple(t.shape) for n, t in want.items()}
    assert rep["tensor_bytes"] == sum(t.numel() * t.element_size() for t in want.values())
    assert main(["inspect", good, "--values", "model.norm.weight", "--count", "3"]) == 0
    out = capsys.readouterr().out
    first = [float(x) for x in out.splitlines()[1].split(":")[1].split()]
    assert first == pytest.approx(want["model.norm.weight"][:3].tolist(), rel=1e-5) and "std" in out
    with pytest.raises(SystemExit):
        main(["inspect", good, "--values", "nobody"])
    # a folder that cannot be loaded: one tensor gone, one too many, one of the wrong shape
    bad = str(tmp_path / "bad")
    os.makedirs(bad)
    with open(os.path.join(bad, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    t = dict(want)
    del t["model.layers.1.mlp.up_proj.weight"]
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    t["model.norm.weight"] = torch.ones(5)
    write_safetensors(os.path.join(bad, "model.safetensors"), t)
    assert main(["inspect", bad]) == 1
    out = capsys.readouterr().out
    assert "NOT loadable" in out
    for frag in ("model.layers.1.mlp.up_proj.weight", "model.layers.0.extra.weight", "model.norm.weight"):
        assert frag in out


def test_gpu_subcommand_with_and_without_devices(monkeypatch, capsys):
    """``airun gpu`` (crates/airun-cli/src/gpu.rs:8-95) against a stand-in for the CUDA runtime."""
    from types import SimpleNamespace
    from airun_b200.cli import main
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert main(["gpu"]) == 0 and "No CUDA device found" in capsys.readouterr().out
    props = [SimpleNamespace(name="NVIDIA B200", major=10, minor=0, total_memory=192 << 30, multi_processor_count=148,
                             max_threads_per_multi_processor=2048, L2_cache_size=126 << 20),
             SimpleNamespace(name="Something older", major=9, minor=0, total_memory=80 << 30, multi_processor_count=132)]
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 2)
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda i: props[i])
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda i: (100 << 30, props[i].total_memory))
    assert main(["gpu"]) == 0
    out = capsys.readouterr().out
    assert "GPU 0 - NVIDIA B200\n" in out and "148 SMs" in out and "UNSUPPORTED" in out.split("GPU 1")[1]
    assert main(["gpu", "--json"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert [d["supported"] for d in rep["devices"]] == [True, False] and rep["devices"][0]["l2_bytes"] == 126 << 20


def test_random_weights_are_a_function_of_seed_name_and_index():
    """Counter-based: the host fill has the moments of a normal variate, equals the tests' own statement
    of the generator, and a tensor does not depend on which other tensors are made."""
    from airun_b200.weights.loader import fill_random_host, tensor_key
    from helpers import plain_random_tensor, plain_random_weights
    z = fill_random_host(400_000, tensor_key(1, "t"), "normal", 1.0)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01 and float(np.abs(z).max()) <= 6.0
    assert 2.8 < float(((z - z.mean()) ** 4).mean() / z.var() ** 2) < 3.1
    assert not np.array_equal(z[:1000], fill_random_host(1000, tensor_key(2, "t"), "normal", 1.0))
    assert not np.array_equal(z[:1000], fill_random_host(1000, tensor_key(1, "u"), "normal", 1.0))
    cfg = Qwen3Config.from_dict(TINY["B"]["cfg"])
    m = DecoderModel(cfg, torch.float32, "cpu")
    ours = random_tensors(m.weight_specs(), 77)
    mine = plain_random_weights(TINY["B"]["cfg"], 77)
    assert set(ours) == set(mine)
    for n in ours:
        assert ours[n].dtype == mine[n].dtype and torch.equal(ours[n], mine[n]), n
    i = fill_random_host(1000, tensor_key(1, "t"), "int", 0.0)
    assert i.dtype == np.int32 and i.min() >= 0 and i.max() < 2 ** 15


def test_weights_are_packed_into_one_allocation():
    """Every tensor the parts hold moves into one arena, 256-byte aligned, unchanged, and tensors that shared
    memory (a tied head and the table, the q rows of the stacked q/k/v matrix) still share it."""
    cfg = Qwen3Config.from_dict(TINY["A"]["cfg"])                      # tied head
    m = DecoderModel(cfg, torch.float32, "cpu")
    m.load(DictSource(random_tensors(m.weight_specs(), 1)))
    mx, ffn = m.layers[0].mixer, m.layers[1].ffn
    before = [t.clone() for t in (mx.w_qkv, mx.w_q, mx.w_o, ffn.w_gu, ffn.w_down, m.final_norm.weight, mx.pos.inv_freq,
                                  m.embedding.table)]
    import unittest.mock
    with unittest.mock.patch.object(torch.cuda, "empty_cache", lambda: None):
        m.pack_weights()
    after = (mx.w_qkv, mx.w_q, mx.w_o, ffn.w_gu, ffn.w_down, m.final_norm.weight, mx.pos.inv_freq, m.embedding.table)
    lo, hi = m.weight_arena.data_ptr(), m.weight_arena.data_ptr() + m.weight_arena.numel()
    for b, a in zip(before, after):
        assert torch.equal(a, b) and a.dtype == b.dtype
        assert lo <= a.data_ptr() and a.data_ptr() + a.numel() * a.element_size() <= hi
    for t in (mx.w_qkv, mx.w_o, ffn.w_gu, ffn.w_down, m.final_norm.weight, m.embedding.table):
        assert t.data_ptr() % 256 == 0
    assert mx.w_q.data_ptr() == mx.w_qkv.data_ptr() and m.head.weight.data_ptr() == m.embedding.table.data_ptr()
