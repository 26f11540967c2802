"""Configuration, registry, safetensors and weight binding: what is accepted and how refusals read."""
import json
import os
import struct

import pytest
import torch

from tiny_configs import TINY_A, TINY_B
from velomind_b200.config import ConfigError, LlamaConfig, read_config_json, register_architecture, resolve, unregister_architecture
from velomind_b200.engine.model import DecoderModel, weight_table
from velomind_b200.models.llama import llama_plan
from velomind_b200.weights import SafetensorsError, WeightError, load_file, load_weights, save_file, write_random_model
from velomind_b200.weights.safetensors_io import parse_header


def test_llama_config_reads_every_key():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.vocab_size, a.hidden_size, a.intermediate_size, a.num_hidden_layers) == (256, 64, 192, 2)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (4, 2, 16)
    assert a.rms_norm_eps == 1e-5 and a.rope_theta == 10000.0 and a.tie_word_embeddings
    assert a.eos_token_ids == (2,) and a.bos_token_id == 1 and a.max_position_embeddings == 512
    b = LlamaConfig.from_dict(TINY_B)
    assert (b.num_attention_heads, b.num_key_value_heads, b.head_dim, b.tie_word_embeddings) == (3, 1, 32, False)
    assert b.eos_token_ids == (7, 9) and b.queries_per_kv_head == 3
    assert LlamaConfig.from_dict(a.to_dict()) == a


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=f"missing required key '{key}'"):
        LlamaConfig.from_dict(d)


def test_bad_values_and_unsupported_options():
    for patch, pattern in [({"num_key_value_heads": 3}, "divisible"), ({"hidden_size": 66}, "divisible"),
                           ({"vocab_size": "many"}, "must be an integer"), ({"rms_norm_eps": -1}, "must be > 0"),
                           ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"),
                           ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
                           ({"eos_token_id": 999}, "outside the vocabulary"), ({"tie_word_embeddings": "yes"}, "true or false")]:
        d = dict(TINY_A, **patch)
        with pytest.raises(ConfigError, match=pattern):
            LlamaConfig.from_dict(d)
    zero_kv = dict(TINY_A, num_key_value_heads=0)        # the reference reads 0 as "as many as heads"
    assert LlamaConfig.from_dict(zero_kv).num_key_value_heads == 4
    explicit = dict(TINY_A, head_dim=32)
    assert LlamaConfig.from_dict(explicit).head_dim == 32


def test_registry_chooses_by_architecture_name(tmp_path):
    assert resolve(TINY_A).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="not registered; registered: .*LlamaForCausalLM"):
        resolve(dict(TINY_A, architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in TINY_A.items() if k != "architectures"})
    register_architecture("AliasForTest", LlamaConfig.from_dict, llama_plan)
    try:
        assert resolve(dict(TINY_A, architectures=["AliasForTest"])).plan is llama_plan
    finally:
        unregister_architecture("AliasForTest")
    with pytest.raises(ConfigError, match="no such file"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))


def test_plan_has_no_sizes_of_its_own():
    plan = llama_plan(LlamaConfig.from_dict(TINY_B))
    table = weight_table(plan)
    assert table["model.layers.2.self_attn.q_proj.weight"].shape == (96, 96)
    assert table["model.layers.0.self_attn.k_proj.weight"].shape == (32, 96)
    assert table["model.layers.1.mlp.down_proj.weight"].shape == (96, 160)
    assert table["lm_head.weight"].shape == (320, 96) and table["lm_head.weight"].alias_of is None
    tied = weight_table(llama_plan(LlamaConfig.from_dict(TINY_A)))
    assert tied["lm_head.weight"].alias_of == "model.embed_tokens.weight"
    assert len(table) == 3 * 9 + 3


def test_safetensors_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(4).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16),
               "i": torch.arange(6, dtype=torch.int64).reshape(2, 3), "e": torch.zeros(0, 4), "s": torch.tensor(3.5)}
    path = str(tmp_path / "t.safetensors")
    save_file(tensors, path)
    back = load_file(path)
    assert back["a"].dtype == torch.float32 and torch.equal(back["a"], tensors["a"])
    assert back["b"].dtype == torch.bfloat16 and torch.equal(back["b"], tensors["b"])
    assert back["c"].dtype == torch.float16 and torch.equal(back["c"], tensors["c"])
    assert back["i"].dtype == torch.int32 and back["i"].tolist() == [[0, 1, 2], [3, 4, 5]]
    assert back["e"].shape == (0, 4) and back["s"].shape == () and float(back["s"]) == 3.5


def _file(tmp_path, header: bytes, payload: bytes = b"") -> str:
    p = str(tmp_path / "x.safetensors")
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + payload)
    return p


def test_safetensors_refusals(tmp_path):
    ok = {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    assert "t" in parse_header(json.dumps(ok).encode(), 8)
    cases = [
        (b'{"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "t": {"dtype": "F32", "shape": [2], "data_offsets": [8, 16]}}', 16, "duplicate key"),
        (b'{"t": {"dtype": "F64", "shape": [2], "data_offsets": [0, 16]}}', 16, "unsupported dtype"),
        (b'{"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}', 8, "needs 12 bytes"),
        (b'{"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}', 4, "truncated"),
        (b'{"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}', 12, "overlap"),
        (b'{"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 8]}}', 8, "bad shape"),
        (b'{"t": [1, 2]}', 8, "not an object"),
        (b'{"t": ', 8, "malformed"),
        (b'[1]', 8, "not a JSON object"),
        (b"[" * 100000, 8, "malformed"),
    ]
    for blob, n, pattern in cases:
        with pytest.raises(SafetensorsError, match=pattern):
            parse_header(blob, n)
    with pytest.raises(SafetensorsError, match="shorter than"):
        p = str(tmp_path / "short"); open(p, "wb").write(b"abc"); load_file(p)
    with pytest.raises(SafetensorsError, match="not plausible"):
        load_file(_file(tmp_path, b"", b""))
    p = str(tmp_path / "huge"); open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="not plausible"):
        load_file(p)


def test_weight_errors_list_everything_at_once(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    table = weight_table(llama_plan(LlamaConfig.from_dict(TINY_A)))
    good = load_weights(folder, table)
    assert good["lm_head.weight"] is good["model.embed_tokens.weight"]          # tied means shared
    assert good["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16    # kept as stored
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    del tensors["model.norm.weight"], tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    tensors["stray.tensor"] = torch.zeros(1)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(folder, table)
    msg = str(e.value)
    assert "missing (2): " in msg and "model.norm.weight" in msg and "model.layers.1.mlp.up_proj.weight" in msg
    assert "unexpected (1): stray.tensor" in msg
    assert "model.layers.0.self_attn.q_proj.weight: expected [64, 64], found [64, 32]" in msg
    assert "wrong dtype (1)" in msg and "input_layernorm" in msg
    # untied model without a head: the head is missing, nothing stands in
    folder_b = write_random_model(str(tmp_path / "b"), TINY_B, seed=1)
    tb = load_file(os.path.join(folder_b, "model.safetensors"))
    del tb["lm_head.weight"]
    save_file(tb, os.path.join(folder_b, "model.safetensors"))
    with pytest.raises(WeightError, match="missing \\(1\\): lm_head.weight"):
        load_weights(folder_b, weight_table(llama_plan(LlamaConfig.from_dict(TINY_B))))
    with pytest.raises(WeightError, match="no such file"):
        load_weights(str(tmp_path), table)


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    a = load_file(os.path.join(write_random_model(str(tmp_path / "a"), TINY_A, seed=3), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(str(tmp_path / "b"), TINY_A, seed=3), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(str(tmp_path / "c"), TINY_A, seed=4), "model.safetensors"))
    more = dict(TINY_A, num_hidden_layers=3)
    d = load_file(os.path.join(write_random_model(str(tmp_path / "d"), more, seed=3), "model.safetensors"))
    assert "lm_head.weight" not in a                       # tied: stored once
    for k in a:
        assert torch.equal(a[k], b[k]) and torch.equal(a[k], d[k])
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    norm = a["model.norm.weight"].float()
    assert (norm - 1).abs().max() <= 0.1 + 1e-2 and abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 2e-3
    assert json.load(open(tmp_path / "a" / "config.json"))["hidden_size"] == 64


def test_a_layer_can_run_twice_and_share_a_cache():
    from velomind_b200.parts.spec import ScheduleEntry
    import dataclasses
    plan = llama_plan(LlamaConfig.from_dict(TINY_A))
    plan2 = dataclasses.replace(plan, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)))
    model = DecoderModel(plan2)
    needs = model.cache_needs()
    assert needs[0] is not None and needs[2] is not None and needs[3] is None
    assert model.cache_shares() == [None, None, None, 1]
    assert len(model.weight_table()) == len(weight_table(plan))       # weights are per layer, not per run
    with pytest.raises(ValueError, match="does not come before"):
        DecoderModel(dataclasses.replace(plan, schedule=(ScheduleEntry(0, cache_of=1), ScheduleEntry(1))))
