"""Configuration, registry, weight files and their errors, the random-weights mode."""
import json
import os

import pytest
import torch

from helpers import TINY_A, TINY_B, model_folder
from libllm_b200.config import (LlamaConfig, architecture_for, known_architectures, load_config,
                                parse_llama_config, register_architecture)
from libllm_b200.errors import ConfigError, WeightsError
from libllm_b200.weights import SafetensorsFile, StateMap, TensorNeed, write_safetensors
from libllm_b200.weights.random_model import create_random_model, random_tensors, tensor_needs_of


def test_config_reads_its_own_keys():
    c = parse_llama_config(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 256, 512)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-6 and not c.tie_word_embeddings
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert c.eos_token_ids == (3, 11)


def test_config_defaults_and_errors():
    base = dict(TINY_A)
    del base["num_key_value_heads"], base["head_dim"], base["rope_theta"]
    c = parse_llama_config(base)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.rope_theta == 10000.0
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
                            (dict(eos_token_id=9999), "eos_token_id"),
                            (dict(head_dim=15), "even")]:
        bad = dict(TINY_A, **change)
        with pytest.raises(ConfigError, match=pattern):
            parse_llama_config(bad)


def test_registry_maps_names_to_models(tmp_path):
    assert "llama" in known_architectures()
    with pytest.raises(ConfigError, match="unexpected model type 'mamba'.*llama"):
        architecture_for("mamba")
    with pytest.raises(ConfigError, match="registered already"):
        register_architecture("llama", None, None)
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, model_type="nope")))
    with pytest.raises(ConfigError, match="unexpected model type"):
        load_config(str(tmp_path))
    assert load_config(model_folder("A")).model_type == "llama"
    spec = architecture_for("llama").describe(parse_llama_config(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.head == "lm_head.weight" and spec.layers[1].mixer.n_kv_heads == 1
    assert architecture_for("llama").describe(parse_llama_config(TINY_A)).head is None


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "d": torch.randn(4).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t)
    f = SafetensorsFile(path)
    assert sorted(f.names()) == ["a", "b", "c", "d"]
    for k, v in t.items():
        assert f.dtype(k) == v.dtype and f.shape(k) == tuple(v.shape) and torch.equal(f.tensor(k), v)
    f.close()
    # the reader of the safetensors package reads the same bytes
    from safetensors import safe_open
    with safe_open(path, "pt") as g:
        assert torch.equal(g.get_tensor("a"), t["a"])


def test_truncated_and_broken_files(tmp_path):
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {"a": torch.zeros(100)})
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-10])
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(path)
    open(path, "wb").write(data[:4])
    with pytest.raises(WeightsError, match="truncated"):
        SafetensorsFile(path)
    with pytest.raises(WeightsError, match="neither"):
        StateMap.from_folder(str(tmp_path / "nothing"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config, needs = tensor_needs_of(TINY_A)
    tensors = random_tensors(TINY_A, 1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 64, dtype=torch.bfloat16)
    with pytest.raises(WeightsError) as e:
        StateMap.from_tensors(tensors).check(needs)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 64), (64, 64))]
    msg = str(err)
    assert 'tensor "model.norm.weight" not found' in msg and "invalid shape: (32, 64) expected, but (64, 64) found" in msg
    assert "rotary_emb.inv_freq" in msg


def test_tied_model_may_carry_an_unused_head_and_untied_needs_it():
    _, needs_a = tensor_needs_of(TINY_A)
    assert "lm_head.weight" not in [n.name for n in needs_a]
    _, needs_b = tensor_needs_of(TINY_B)
    t = random_tensors(TINY_B, 1)
    del t["lm_head.weight"]
    with pytest.raises(WeightsError) as e:
        StateMap.from_tensors(t).check(needs_b)
    assert e.value.missing == ["lm_head.weight"]


def test_precision_of_fetched_tensors():
    sm = StateMap.from_tensors({"m16": torch.ones(2, 2, dtype=torch.float16), "m32": torch.ones(2, 2),
                                "v32": torch.ones(2), "v16": torch.ones(2, dtype=torch.bfloat16),
                                "tab": torch.arange(4, dtype=torch.int64)})
    bf = torch.bfloat16
    assert sm.fetch(TensorNeed("m16", (2, 2)), bf, "cpu").dtype == bf
    assert sm.fetch(TensorNeed("m32", (2, 2)), bf, "cpu").dtype == bf             # a matrix product's operand
    assert sm.fetch(TensorNeed("v32", (2,), role="vector"), bf, "cpu").dtype == torch.float32   # stored in 32-bit: stays
    assert sm.fetch(TensorNeed("v16", (2,), role="vector"), bf, "cpu").dtype == bf
    assert sm.fetch(TensorNeed("tab", (4,), role="table"), bf, "cpu").dtype == torch.int32
    assert sm.fetch(TensorNeed("m16", (2, 2)), torch.float32, "cpu").dtype == torch.float32
    with pytest.raises(WeightsError, match="invalid shape"):
        sm.fetch(TensorNeed("m16", (3, 2)), bf, "cpu")
    assert sm.fetch(TensorNeed("gone", (1,), optional=True), bf, "cpu") is None


def test_random_model_folder_is_seeded_and_complete(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    create_random_model(a, TINY_B, 5)
    create_random_model(b, TINY_B, 5)
    create_random_model(c, TINY_B, 6)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(a, "config.json")))["num_hidden_layers"] == 3
    sa, sb, sc = (StateMap.from_folder(x) for x in (a, b, c))
    _, needs = tensor_needs_of(TINY_B)
    sa.check(needs)
    for n in sa.names():
        assert torch.equal(sa.raw(n), sb.raw(n))
    assert not torch.equal(sa.raw("lm_head.weight"), sc.raw("lm_head.weight"))
    w = sa.raw("model.layers.0.mlp.down_proj.weight").float()
    assert sa.stored_dtype("lm_head.weight") == torch.bfloat16 and abs(float(w.std()) - 0.02) < 2e-3
    nw = sa.raw("model.norm.weight").float()
    assert float(nw.min()) >= 0.9 - 1e-2 and float(nw.max()) <= 1.1 + 1e-2 and float(nw.std()) > 0.01


def test_sharded_folder(tmp_path):
    t = random_tensors(TINY_A, 2)
    names = list(t)
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: t[n] for n in names[:7]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: t[n] for n in names[7:]})
    idx = {"weight_map": {n: ("s1.safetensors" if i < 7 else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(idx))
    sm = StateMap.from_folder(str(tmp_path))
    sm.check(tensor_needs_of(TINY_A)[1])
    assert torch.equal(sm.raw(names[-1]), t[names[-1]])
