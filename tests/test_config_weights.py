"""Configuration, registry, weight files and their errors, the random-weights mode: the host
library's own code (config/, weights/), through its C interface, on the CPU."""
import json
import os

import pytest
import torch

from helpers import TINY_A, TINY_B, model_folder, plain_weights, write_safetensors
from libllm_b200.config import (describe_model, known_architectures, load_config, parse_config, parse_llama_config,
                                register_architecture)
from libllm_b200.errors import ConfigError, InvalidArgError, WeightsError
from libllm_b200.weights import check_weights, create_random_model, read_safetensors_header, tensor_needs_of


def test_config_reads_its_own_keys():
    c = parse_llama_config(TINY_B)
    assert (c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"]) == (96, 3, 3, 1)
    assert (c["head_dim"], c["intermediate_size"], c["vocab_size"]) == (32, 256, 512)
    assert c["rope_theta"] == 500000.0 and c["rms_norm_eps"] == 1e-6 and not c["tie_word_embeddings"]
    assert c["rope_scaling"]["factor"] == 8.0 and c["rope_scaling"]["original_max_position_embeddings"] == 64
    assert c["eos_token_id"] == [3, 11]
    assert parse_config(c) == c                      # the normal form is a fixed point


def test_config_defaults_and_errors():
    base = dict(TINY_A)
    del base["num_key_value_heads"], base["head_dim"], base["rope_theta"]
    c = parse_llama_config(base)
    assert c["num_key_value_heads"] == 4 and c["head_dim"] == 16 and c["rope_theta"] == 10000.0
    assert c["attention_bias"] is False and c["eos_token_id"] == 7
    for key in ("hidden_size", "num_attention_heads", "intermediate_size", "rms_norm_eps", "num_hidden_layers",
                "vocab_size", "max_position_embeddings"):
        bad = dict(TINY_A)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            parse_llama_config(bad)
    for change, pattern in [(dict(hidden_size=65, head_dim=None), "invalid hidden_size"),
                            (dict(num_key_value_heads=3), "multiple"),
                            (dict(hidden_act="gelu"), "hidden_act"),
                            (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_scaling"),
                            (dict(vocab_size="256"), "integer"),
                            (dict(vocab_size=256.5), "integer"),
                            (dict(rms_norm_eps=0), "positive"),
                            (dict(tie_word_embeddings="yes"), "true or false"),
                            (dict(eos_token_id=9999), "eos_token_id"),
                            (dict(head_dim=15), "even")]:
        bad = dict(TINY_A, **change)
        with pytest.raises(ConfigError, match=pattern):
            parse_llama_config(bad)


def test_registry_maps_names_to_models(tmp_path):
    assert "llama" in known_architectures()
    with pytest.raises(ConfigError, match="unexpected model type 'mamba'.*llama"):
        parse_config(dict(TINY_A, model_type="mamba"))
    with pytest.raises(ConfigError, match="registered already"):
        register_architecture("llama", None, None)
    with pytest.raises(ConfigError, match="registered already"):
        register_architecture("llama", lambda d: d, lambda d: d)
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, model_type="nope")))
    with pytest.raises(ConfigError, match="unexpected model type"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))
    assert load_config(model_folder("A"))["model_type"] == "llama"
    d = describe_model(TINY_B)
    spec = d["spec"]
    assert len(spec["layers"]) == 3 and [e["layer"] for e in spec["schedule"]] == [0, 1, 2]
    assert spec["head"] == "lm_head.weight" and spec["layers"][1]["mixer"]["n_kv_heads"] == 1
    assert spec["layers"][2]["mixer"]["position"]["scaling"]["factor"] == 8.0 and spec["stop_tokens"] == [3, 11]
    assert describe_model(TINY_A)["spec"]["head"] is None
    assert "gemm_tc" in d["kernel_families"] and "gemm_tc" not in describe_model(TINY_B, "float32")["kernel_families"]


def test_an_architecture_registered_from_outside_is_described_by_its_own_functions():
    def parse(d):
        if "width" not in d:
            raise KeyError("width")
        return dict(model_type=d["model_type"], width=int(d["width"]), vocab_size=int(d.get("vocab_size", 11)))

    def describe(c):
        n = lambda name: dict(kind="rmsnorm", size=c["width"], eps=1e-5, weight=name)
        layer = dict(kind="prenorm", mixer_norm=n("l.n1"), ff_norm=n("l.n2"),
                     mixer=dict(kind="attention", hidden=c["width"], n_heads=2, n_kv_heads=1, head_dim=16, position=None,
                                q="l.q", k="l.k", v="l.v", o="l.o"),
                     ff=dict(kind="swiglu", hidden=c["width"], intermediate=24, gate="l.g", up="l.u", down="l.d"))
        return dict(name="two_runs", vocab_size=c["vocab_size"], hidden=c["width"], embedding="emb", layers=[layer],
                    schedule=[0, dict(layer=0, cache_from=0)], final_norm=n("fn"), head=None, max_positions=128)

    register_architecture("test_two_runs", parse, describe, replace=True)
    assert "test_two_runs" in known_architectures()
    d = describe_model(dict(model_type="test_two_runs", width=32))
    assert [n["name"] for n in d["tensor_needs"]] == ["emb", "l.n1", "l.q", "l.k", "l.v", "l.o", "l.n2", "l.g", "l.u", "l.d", "fn"]
    assert d["spec"]["schedule"] == [dict(layer=0, cache_from=None), dict(layer=0, cache_from=0)]
    with pytest.raises(ConfigError, match="KeyError.*width"):
        describe_model(dict(model_type="test_two_runs"))
    bad = lambda c: dict(describe(c), schedule=[dict(layer=0, cache_from=0)])
    register_architecture("test_bad_schedule", parse, bad, replace=True)
    with pytest.raises(ConfigError, match="does not run before it"):
        describe_model(dict(model_type="test_bad_schedule", width=32))


def test_safetensors_header_and_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "d": torch.randn(4).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    h = read_safetensors_header(path)
    assert sorted(h) == ["a", "b", "c", "d"]
    assert h["a"] == dict(dtype="BF16", shape=[3, 5], nbytes=30) and h["b"]["dtype"] == "I64" and h["d"]["dtype"] == "F16"
    # what the library writes, other readers read: the random-weights folder through the safetensors package
    folder = model_folder("A")
    from safetensors import safe_open
    w = plain_weights(folder)
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as g:
        assert sorted(g.keys()) == sorted(w)
        assert torch.equal(g.get_tensor("model.norm.weight").double(), w["model.norm.weight"])


def test_truncated_and_broken_files(tmp_path):
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"a": torch.zeros(100)})
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-10])
    with pytest.raises(WeightsError, match="truncated"):
        read_safetensors_header(path)
    open(path, "wb").write(data[:4])
    with pytest.raises(WeightsError, match="truncated"):
        read_safetensors_header(path)
    open(path, "wb").write(data[:8] + b"[" + data[9:])
    with pytest.raises(WeightsError, match="invalid header"):
        read_safetensors_header(path)
    with pytest.raises(WeightsError, match="neither"):
        check_weights(str(tmp_path / "nothing"), [])


def tensors_like(config, seed):
    g = torch.Generator().manual_seed(seed)
    return {n["name"]: (0.02 * torch.randn(n["shape"], generator=g)).to(torch.bfloat16) for n in tensor_needs_of(config)}


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    needs = tensor_needs_of(TINY_A)
    tensors = tensors_like(TINY_A, 1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        check_weights(str(tmp_path), needs)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.extra.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    msg = str(err)
    assert 'tensor "model.norm.weight" not found' in msg and "invalid shape: (32, 64) expected, but (64, 64) found" in msg
    assert "rotary_emb.inv_freq" in msg and "2 missing, 2 unexpected, 1 with a wrong shape" in msg
    # patterns of tensors that may lie in the files unused (the architecture's description names them)
    ignore = describe_model(TINY_A)["spec"]["ignore_tensors"]
    assert "lm_head.weight" in ignore
    with pytest.raises(WeightsError) as e:
        check_weights(str(tmp_path), needs, ignore)
    assert e.value.unexpected == ["model.extra.weight"]


def test_unexpected_tensors_alone_are_an_error_or_a_warning(tmp_path):
    needs = tensor_needs_of(TINY_A)
    tensors = tensors_like(TINY_A, 1)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()      # a tied checkpoint's copy
    tensors["model.extra.weight"] = torch.zeros(2)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    ignore = describe_model(TINY_A)["spec"]["ignore_tensors"]
    with pytest.raises(WeightsError) as e:
        check_weights(str(tmp_path), needs, ignore)
    assert e.value.unexpected == ["model.extra.weight"] and e.value.missing == []
    report = check_weights(str(tmp_path), needs, ignore, strict=False)
    assert report["unexpected"] == ["model.extra.weight"] and report["ignored"] == ["lm_head.weight"]


def test_tied_model_needs_no_head_and_untied_needs_it(tmp_path):
    assert "lm_head.weight" not in [n["name"] for n in tensor_needs_of(TINY_A)]
    needs_b = tensor_needs_of(TINY_B)
    t = tensors_like(TINY_B, 1)
    del t["lm_head.weight"]
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightsError) as e:
        check_weights(str(tmp_path), needs_b)
    assert e.value.missing == ["lm_head.weight"]


def test_random_model_folder_is_seeded_and_complete(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    create_random_model(a, TINY_B, 5)
    create_random_model(b, TINY_B, 5)
    create_random_model(c, TINY_B, 6)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(a, "config.json")))["num_hidden_layers"] == 3
    check_weights(a, tensor_needs_of(TINY_B))
    wa, wb, wc = plain_weights(a), plain_weights(b), plain_weights(c)
    for n in wa:
        assert torch.equal(wa[n], wb[n])
    assert not torch.equal(wa["lm_head.weight"], wc["lm_head.weight"])
    w = wa["model.layers.0.mlp.down_proj.weight"]
    assert read_safetensors_header(os.path.join(a, "model.safetensors"))["lm_head.weight"]["dtype"] == "BF16"
    assert abs(float(w.std()) - 0.02) < 2e-3 and abs(float(w.mean())) < 1e-3
    # a tensor's values depend on the seed and its name alone: two tensors of one shape differ
    assert not torch.equal(wa["model.layers.0.mlp.gate_proj.weight"], wa["model.layers.0.mlp.up_proj.weight"])
    nw = wa["model.norm.weight"]
    assert float(nw.min()) >= 0.9 - 1e-2 and float(nw.max()) <= 1.1 + 1e-2 and float(nw.std()) > 0.01
    create_random_model(str(tmp_path / "f32"), TINY_A, 5, dtype="float32")
    assert read_safetensors_header(str(tmp_path / "f32" / "model.safetensors"))["model.norm.weight"]["dtype"] == "F32"
    with pytest.raises(InvalidArgError, match="dtype"):
        create_random_model(str(tmp_path / "bad"), TINY_A, 5, dtype="int8")


def test_sharded_folder(tmp_path):
    t = tensors_like(TINY_A, 2)
    names = list(t)
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: t[n] for n in names[:7]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[7:]})
    idx = {"weight_map": {n: ("s1.safetensors" if i < 7 else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(idx))
    report = check_weights(str(tmp_path), tensor_needs_of(TINY_A))
    assert sorted(report["names"]) == sorted(names)
    # a tensor stored in two shards, and a shard that is named but missing
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[6:]})
    with pytest.raises(WeightsError, match="stored twice"):
        check_weights(str(tmp_path), tensor_needs_of(TINY_A))
    os.unlink(str(tmp_path / "s1.safetensors"))
    with pytest.raises(WeightsError, match="shard files .* are missing: s1.safetensors"):
        check_weights(str(tmp_path), tensor_needs_of(TINY_A))
