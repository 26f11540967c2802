"""Configuration, registry, safetensors and weight binding: what is accepted and how refusals read (no GPU needed)."""
import json
import os
import struct

import numpy as np
import pytest

import plain_llama as P
import st_files
import velomind_b200 as vm
from tiny_configs import TINY_A, TINY_B


def test_llama_config_reads_every_key():
    a = vm.describe_config(TINY_A)
    t = a["typed"]
    assert (t["vocab_size"], t["hidden_size"], t["intermediate_size"], t["num_hidden_layers"]) == (256, 64, 192, 2)
    assert (t["num_attention_heads"], t["num_key_value_heads"], t["head_dim"]) == (4, 2, 16)
    assert t["rms_norm_eps"] == 1e-5 and t["rope_theta"] == 10000.0 and t["tie_word_embeddings"] is True
    assert a["stop_tokens"] == [2] and a["bos_token"] == 1 and a["max_positions"] == 512
    b = vm.describe_config(TINY_B)
    tb = b["typed"]
    assert (tb["num_attention_heads"], tb["num_key_value_heads"], tb["head_dim"], tb["tie_word_embeddings"]) == (3, 1, 32, False)
    assert b["stop_tokens"] == [7, 9]
    assert vm.describe_config(t)["typed"] == t                       # the typed configuration reads back as itself


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(vm.ConfigError, match=f"missing required key '{key}'"):
        vm.describe_config(d)


def test_bad_values_and_unsupported_options():
    for patch, pattern in [({"num_key_value_heads": 3}, "divisible"), ({"hidden_size": 66}, "divisible"),
                           ({"vocab_size": "many"}, "must be an integer"), ({"rms_norm_eps": -1}, "must be > 0"),
                           ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"),
                           ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
                           ({"eos_token_id": 999}, "outside the vocabulary"), ({"tie_word_embeddings": "yes"}, "true or false"),
                           ({"sliding_window": 128}, "sliding_window"), ({"num_hidden_layers": 2.5}, "must be an integer")]:
        with pytest.raises(vm.ConfigError, match=pattern):
            vm.describe_config(dict(TINY_A, **patch))
    zero_kv = dict(TINY_A, num_key_value_heads=0)        # the reference reads 0 as "as many as heads"
    assert vm.describe_config(zero_kv)["typed"]["num_key_value_heads"] == 4
    assert vm.describe_config(dict(TINY_A, head_dim=32))["typed"]["head_dim"] == 32
    assert vm.describe_config(dict(TINY_A, rope_scaling=None, attention_bias=False, hidden_act="silu"))["hidden_size"] == 64


def test_registry_chooses_by_architecture_name(tmp_path):
    assert vm.describe_config(TINY_A)["architecture"] == "LlamaForCausalLM"
    assert "LlamaForCausalLM" in vm.registered_architectures()
    with pytest.raises(vm.ConfigError, match="not registered; registered: .*LlamaForCausalLM"):
        vm.describe_config(dict(TINY_A, architectures=["NoSuchModel"]))
    with pytest.raises(vm.ConfigError, match="architectures"):
        vm.describe_config({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(vm.ConfigError, match="no such file"):
        vm.check_model_folder(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(vm.ConfigError, match="not valid JSON"):
        vm.check_model_folder(str(tmp_path))


def test_plan_has_no_sizes_of_its_own():
    """Every size of the parts comes from config.json: another configuration, other shapes, layer by layer."""
    table = vm.weight_table(TINY_B)
    assert table["model.layers.2.self_attn.q_proj.weight"]["shape"] == [96, 96]
    assert table["model.layers.0.self_attn.k_proj.weight"]["shape"] == [32, 96]
    assert table["model.layers.1.mlp.down_proj.weight"]["shape"] == [96, 160]
    assert table["lm_head.weight"]["shape"] == [320, 96] and table["lm_head.weight"]["alias_of"] is None
    assert vm.weight_table(TINY_A)["lm_head.weight"]["alias_of"] == "model.embed_tokens.weight"
    assert len(table) == 3 * 9 + 3
    blocks = vm.describe_config(TINY_B)["blocks"]
    assert len(blocks) == 3 and blocks[0]["mixer"]["kind"] == "grouped_query_attention" and blocks[0]["arrangement"] == "prenorm"
    assert blocks[1]["mixer"]["args"]["kv_heads"] == 1 and blocks[1]["feed_forward"]["args"]["intermediate"] == 160
    assert blocks[2]["mixer_norm"]["args"]["eps"] == 1e-6 and blocks[2]["mixer"]["args"]["position"]["args"]["theta"] == 100000.0


def test_safetensors_keeps_dtypes_as_stored(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a": rng.standard_normal((3, 5)).astype(np.float32), "b": rng.standard_normal(4).astype(np.float32),
               "c": rng.standard_normal((2, 2)).astype(np.float16), "i": np.arange(6, dtype=np.int64).reshape(2, 3),
               "e": np.zeros((0, 4), dtype=np.float32), "s": np.array(3.5, dtype=np.float32)}
    path = str(tmp_path / "t.safetensors")
    st_files.write(path, tensors, bf16=("b",))
    info = vm.safetensors_info(path)
    assert {k: v["dtype"] for k, v in info.items()} == {"a": "F32", "b": "BF16", "c": "F16", "i": "I64", "e": "F32", "s": "F32"}
    assert info["i"]["shape"] == [2, 3] and info["e"]["shape"] == [0, 4] and info["s"]["shape"] == []
    back = P.read_safetensors(path)                       # the plain reader agrees on the values
    assert np.array_equal(back["a"], tensors["a"]) and back["i"].tolist() == [[0, 1, 2], [3, 4, 5]]


def _file(tmp_path, header: bytes, payload: bytes = b"") -> str:
    p = str(tmp_path / "x.safetensors")
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + payload)
    return p


def test_safetensors_refusals(tmp_path):
    ok = {"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    assert vm.check_safetensors_header(json.dumps(ok).encode(), 8) == 1
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
        with pytest.raises(vm.WeightError, match=pattern):
            vm.check_safetensors_header(blob, n)
    with pytest.raises(vm.WeightError, match="shorter than"):
        p = str(tmp_path / "short"); open(p, "wb").write(b"abc"); vm.safetensors_info(p)
    with pytest.raises(vm.WeightError, match="not plausible"):
        vm.safetensors_info(_file(tmp_path, b"", b""))
    p = str(tmp_path / "huge"); open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(vm.WeightError, match="not plausible"):
        vm.safetensors_info(p)


def test_weight_errors_list_everything_at_once(tmp_path):
    folder = vm.write_random_model(str(tmp_path / "m"), TINY_A, seed=0)
    vm.check_model_folder(folder)
    path = os.path.join(folder, "model.safetensors")
    info = vm.safetensors_info(path)
    assert "lm_head.weight" not in info                                          # tied: stored once, the table stands in
    assert info["model.layers.0.mlp.up_proj.weight"]["dtype"] == "BF16"          # kept as stored
    tensors = P.read_safetensors(path)
    names = set(tensors)
    del tensors["model.norm.weight"], tensors["model.layers.1.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = np.zeros((64, 32), dtype=np.float32)
    tensors["model.layers.0.input_layernorm.weight"] = np.zeros(64, dtype=np.int32)
    tensors["stray.tensor"] = np.zeros(1, dtype=np.float32)
    st_files.write(path, tensors, bf16=tuple(n for n in names if n in tensors and tensors[n].dtype == np.float32))
    with pytest.raises(vm.WeightError) as e:
        vm.check_model_folder(folder)
    msg = str(e.value)
    assert "missing (2): " in msg and "model.norm.weight" in msg and "model.layers.1.mlp.up_proj.weight" in msg
    assert "unexpected (1): stray.tensor" in msg
    assert "model.layers.0.self_attn.q_proj.weight: expected [64, 64], found [64, 32]" in msg
    assert "wrong dtype (1)" in msg and "input_layernorm" in msg
    # untied model without a head: the head is missing, nothing stands in
    folder_b = vm.write_random_model(str(tmp_path / "b"), TINY_B, seed=1)
    tb = P.read_safetensors(os.path.join(folder_b, "model.safetensors"))
    del tb["lm_head.weight"]
    st_files.write(os.path.join(folder_b, "model.safetensors"), tb)
    with pytest.raises(vm.WeightError, match="missing \\(1\\): lm_head.weight"):
        vm.check_model_folder(folder_b)
    os.remove(os.path.join(folder_b, "model.safetensors"))
    with pytest.raises(vm.WeightError, match="no such file"):
        vm.check_model_folder(folder_b)
    open(os.path.join(folder_b, "model.safetensors.index.json"), "w").write("{}")
    with pytest.raises(vm.WeightError, match="sharded checkpoint"):
        vm.check_model_folder(folder_b)


def test_random_weights_depend_on_seed_and_name_only(tmp_path):
    def read(name, config, seed):
        return P.read_safetensors(os.path.join(vm.write_random_model(str(tmp_path / name), config, seed=seed), "model.safetensors"))
    a, b, c = read("a", TINY_A, 3), read("b", TINY_A, 3), read("c", TINY_A, 4)
    d = read("d", dict(TINY_A, num_hidden_layers=3), 3)
    assert "lm_head.weight" not in a                       # tied: stored once
    for k in a:
        assert np.array_equal(a[k], b[k]) and np.array_equal(a[k], d[k])
    assert not np.array_equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert np.abs(a["model.norm.weight"] - 1).max() <= 0.1 + 1e-2 and abs(float(a["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert abs(float(a["model.embed_tokens.weight"].mean())) < 2e-3
    assert json.load(open(tmp_path / "a" / "config.json"))["hidden_size"] == 64
    f32 = vm.write_random_model(str(tmp_path / "f32"), TINY_A, seed=3, dtype="float32")
    assert vm.safetensors_info(os.path.join(f32, "model.safetensors"))["model.norm.weight"]["dtype"] == "F32"
    with pytest.raises(ValueError, match="bfloat16 or float32"):
        vm.write_random_model(str(tmp_path / "f16"), TINY_A, dtype="float16")


def test_a_schedule_is_checked(tmp_path, monkeypatch):
    """The order in which layers run is data; a run may read the cache of a run BEFORE it that owns one, nothing else."""
    import toy_plugin
    toy_plugin.load(str(tmp_path))
    looped = dict(TINY_A, architectures=["LoopedLlamaForCausalLM"], schedule=[[0, -1], [1, -1], [0, -1], [1, 1]])
    d = vm.describe_config(looped)
    assert d["runs"] == 4 and d["layers"] == 2
    assert len(vm.weight_table(looped)) == len(vm.weight_table(TINY_A))        # weights are per layer, not per run
    folder = vm.write_random_model(str(tmp_path / "looped"), looped, seed=1)
    vm.check_model_folder(folder)
    bad = dict(looped, schedule=[[0, 1], [1, -1]])
    with pytest.raises(vm.ConfigError, match="does not come before"):
        vm.write_random_model(str(tmp_path / "bad"), bad, seed=1)
    with pytest.raises(vm.ConfigError, match="names layer 5"):
        vm.write_random_model(str(tmp_path / "bad2"), dict(looped, schedule=[[5, -1]]), seed=1)
