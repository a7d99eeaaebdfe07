"""Configuration, registry, weight loading errors and random-weights mode (CPU)."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import TINY_A, TINY_B, TINY_C, TINY_D, model_folder

from prism_b200.config.model_config import ConfigError
from prism_b200.models.qwen2 import Qwen2Config
from prism_b200.model_registry import build_model, registered_architectures, resolve
from prism_b200.weights.loader import WeightError, load_model_folder
from prism_b200.weights.random_init import file_tensors, write_model_folder


def test_config_reads_every_key_and_defaults():
    c = Qwen2Config.from_dict(TINY_C)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (389, 80, 176, 4)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 3, 48)
    assert c.rms_norm_eps == 3e-6 and c.rope_theta == 50000.0 and c.attention_bias is False
    assert [c.layer_window(i) for i in range(4)] == [None, None, 24, 24]
    d = Qwen2Config.from_dict(dict(vocab_size=10, hidden_size=32, intermediate_size=8, num_hidden_layers=1,
                                   num_attention_heads=4, architectures=["Qwen2ForCausalLM"]))
    assert d.num_key_value_heads == 4 and d.head_dim == 8 and d.rms_norm_eps == 1e-6 and d.rope_theta == 10000.0
    assert d.max_position_embeddings == 4096 and d.tie_word_embeddings is False and d.layer_window(0) is None
    # end-of-sequence ids: none, one, or a list (all kept)
    assert d.eos_token_id == ()
    assert Qwen2Config.from_dict(dict(TINY_A, eos_token_id=7)).eos_token_id == (7,)
    several = Qwen2Config.from_dict(dict(TINY_A, eos_token_id=[151645, 151643]))
    assert several.eos_token_id == (151645, 151643) and several.to_dict()["eos_token_id"] == [151645, 151643]
    _, m = build_model(dict(TINY_A, eos_token_id=[5, 9]))
    assert m.spec.eos_token_id == (5, 9)


@pytest.mark.parametrize("patch,word", [
    (dict(hidden_size=None), "hidden_size"),
    (dict(num_attention_heads=5, head_dim=None), "not divisible"),
    (dict(num_key_value_heads=3), "num_key_value_heads"),
    (dict(rope_scaling={"type": "yarn", "factor": 2}), "rope_scaling"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(head_dim=15), "even"),
])
def test_config_errors(patch, word):
    raw = dict(TINY_A)
    for k, v in patch.items():
        if v is None:
            raw.pop(k, None)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(raw)


def test_an_architecture_is_a_module_that_registers_itself():
    """Nothing outside ``prism_b200/models/qwen2.py`` names the architecture: the registry, the loader, the
    random-weights mode and the generic configuration module hold no architecture name."""
    import prism_b200
    root = os.path.dirname(prism_b200.__file__)
    for rel in ("model_registry.py", "config/model_config.py", "config/engine_config.py", "weights/random_init.py",
                "weights/loader.py", "weights/pool.py", "models/decoder.py", "engine/runner.py", "engine/llm.py"):
        with open(os.path.join(root, rel)) as f:
            text = f.read()
        assert "Qwen2" not in text and "qwen2" not in text, rel
    with pytest.raises(ConfigError, match="architectures"):
        write_model_folder({k: v for k, v in TINY_A.items() if k != "architectures"}, 0, "/nonexistent")


def test_sizes_no_kernel_takes_are_refused_when_the_model_is_built():
    """A head size beyond the attention kernels' limit is a configuration error at build time, not a kernel
    error at the first step; a shape that only the slow shape-generic kernel takes in bfloat16 is said so
    once, when the weights are bound."""
    with pytest.raises(ConfigError, match="head_dim 258"):
        build_model(dict(TINY_A, head_dim=258))
    build_model(dict(TINY_A, head_dim=256))
    import prism_b200.parts.attention as att
    att._warned.clear()
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        odd = write_model_folder(dict(TINY_A, hidden_size=72, head_dim=18), 0, d)         # head_dim 18: no multiple of 16
        with pytest.warns(RuntimeWarning, match="shape-generic kernel"):
            load_model_folder(odd, "cpu", torch.bfloat16)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            load_model_folder(odd, "cpu", torch.float32)                     # float32 has one kernel: nothing to say
            load_model_folder(model_folder("A"), "cpu", torch.bfloat16)      # head_dim 16: the tensor-core kernels
            load_model_folder(model_folder("D"), "cpu", torch.bfloat16)      # head_dim 64


def test_registry():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve(TINY_A).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="not registered.*Qwen2ForCausalLM"):
        resolve(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in TINY_A.items() if k != "architectures"})
    cfg, model = build_model(TINY_B)
    assert len(model.layers) == 3 and model.spec.vocab_size == 320
    # layer plan is data: per-layer parts take their constants as parameters
    _, mc = build_model(TINY_C)
    assert [l.mixer.window for l in mc.layers] == [None, None, 24, 24]
    assert mc.layers[0].mixer.qkv_bias is False and mc.layers[0].mixer_norm.eps == 3e-6


def test_load_tied_head_shares_storage_and_dtypes_are_kept():
    cfg, model, pool = load_model_folder(model_folder("A"), "cpu", torch.bfloat16)
    assert pool["head.weight"].data_ptr() == pool["embedding.weight"].data_ptr()
    assert all(t.dtype == torch.bfloat16 for t in pool.tensors.values() if t is not None)
    assert pool["layers.1.mixer.qkv_w"].shape == (4 * 16 + 2 * 2 * 16, 64)
    # fusion order: q rows, then k rows, then v rows; gate rows then up rows
    raw = load_file(os.path.join(model_folder("A"), "model.safetensors"))
    p = "model.layers.1."
    want = torch.cat([raw[p + "self_attn.q_proj.weight"], raw[p + "self_attn.k_proj.weight"],
                      raw[p + "self_attn.v_proj.weight"]])
    assert torch.equal(pool["layers.1.mixer.qkv_w"], want)
    assert torch.equal(pool["layers.1.feed_forward.gate_up_w"],
                       torch.cat([raw[p + "mlp.gate_proj.weight"], raw[p + "mlp.up_proj.weight"]]))
    # a float32 engine upcasts everything exactly
    _, _, pool32 = load_model_folder(model_folder("A"), "cpu", torch.float32)
    assert pool32["layers.1.mixer.qkv_w"].dtype == torch.float32
    assert torch.equal(pool32["layers.1.mixer.qkv_w"], want.float())


def test_tensor_stored_in_32bit_stays_so(tmp_path):
    d = write_model_folder(TINY_B, 3, str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["model.norm.weight"] = t["model.norm.weight"].float()
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].float()
    save_file(t, path)
    _, _, pool = load_model_folder(d, "cpu", torch.bfloat16)
    assert pool["final_norm.weight"].dtype == torch.float32
    assert pool["layers.0.feed_forward.down_w"].dtype == torch.float32
    assert pool["layers.1.feed_forward.down_w"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_model_folder(TINY_B, 3, str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.self_attn.k_proj.bias"]
    del t["model.layers.2.mlp.up_proj.weight"]
    t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(32)
    t["model.norm.weight"] = torch.zeros(97)
    t["model.layers.0.rotary_emb.inv_freq"] = torch.zeros(16)        # tolerated
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_model_folder(d, "cpu", torch.float32)
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.k_proj.bias", "model.layers.2.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert err.wrong_shape == [("model.norm.weight", (97,), (96,))]
    msg = str(err)
    for word in ("k_proj.bias", "up_proj.weight", "q_norm", "[97]", "[96]"):
        assert word in msg


def test_no_safetensors_and_no_config(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_model_folder(str(tmp_path), "cpu", torch.float32)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(TINY_A, f)
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model_folder(str(tmp_path), "cpu", torch.float32)


def test_untied_model_rejects_missing_head_and_tied_head_in_the_file_must_be_the_embedding(tmp_path):
    d = write_model_folder(TINY_B, 3, str(tmp_path / "b"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    head = t.pop("lm_head.weight")
    save_file(t, path)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model_folder(d, "cpu", torch.float32)
    a = write_model_folder(TINY_A, 0, str(tmp_path / "a"))
    ta = load_file(os.path.join(a, "model.safetensors"))
    ta["lm_head.weight"] = ta["model.embed_tokens.weight"].clone()      # the embedding over again: accepted
    save_file(ta, os.path.join(a, "model.safetensors"))
    _, _, pool = load_model_folder(a, "cpu", torch.float32)
    assert pool["head.weight"].data_ptr() == pool["embedding.weight"].data_ptr()
    ta["lm_head.weight"][3, 5] += 0.5                                   # one element off: not a tied model's file
    save_file(ta, os.path.join(a, "model.safetensors"))
    with pytest.raises(WeightError, match="lm_head.weight is stored although it is tied to model.embed_tokens.weight"):
        load_model_folder(a, "cpu", torch.float32)
    ta["lm_head.weight"] = torch.zeros(255, 64)
    save_file(ta, os.path.join(a, "model.safetensors"))
    with pytest.raises(WeightError, match="another shape"):
        load_model_folder(a, "cpu", torch.float32)


def test_dtypes_the_loader_refuses(tmp_path):
    """Weights are bf16, fp16 or fp32 in the file; 64-bit floats and integers are an error, not a cast."""
    d = write_model_folder(TINY_A, 0, str(tmp_path / "a"))
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["model.norm.weight"] = t["model.norm.weight"].double()
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].to(torch.int32)
    t["model.layers.1.mlp.down_proj.weight"] = t["model.layers.1.mlp.down_proj.weight"].half()      # fine
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_model_folder(d, "cpu", torch.bfloat16)
    assert len(e.value.other) == 2 and "F64" in str(e.value) and "I32" in str(e.value)


def test_random_weights_are_a_function_of_config_and_seed(tmp_path):
    a = load_file(os.path.join(write_model_folder(TINY_B, 7, str(tmp_path / "x")), "model.safetensors"))
    b = load_file(os.path.join(write_model_folder(TINY_B, 7, str(tmp_path / "y")), "model.safetensors"))
    c = load_file(os.path.join(write_model_folder(TINY_B, 8, str(tmp_path / "z")), "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    _, model = build_model(TINY_B)
    names = [n for n, _, _ in file_tensors(model)]
    assert names[0] == "model.embed_tokens.weight" and names[-1] == "lm_head.weight"
    assert set(names) == set(a.keys())
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 2e-3 and abs(float(w.mean())) < 1e-3
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 2e-2
    with open(tmp_path / "x" / "config.json") as f:
        assert json.load(f)["architectures"] == ["Qwen2ForCausalLM"]


def _split_into_shards(folder, with_index):
    """Rewrite model.safetensors as two shards: the q/k/v of every layer land in different files."""
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    names = sorted(t)
    a = {n: t[n] for i, n in enumerate(names) if i % 2 == 0}
    b = {n: t[n] for i, n in enumerate(names) if i % 2 == 1}
    os.remove(path)
    save_file(a, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file(b, os.path.join(folder, "model-00002-of-00002.safetensors"))
    if with_index:
        wm = {n: "model-00001-of-00002.safetensors" for n in a}
        wm.update({n: "model-00002-of-00002.safetensors" for n in b})
        with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": wm}, f)
    return t


@pytest.mark.parametrize("with_index", [True, False])
def test_sharded_folder_loads_like_a_single_file(tmp_path, with_index):
    d = write_model_folder(TINY_B, 5, str(tmp_path / "m"))
    _, _, whole = load_model_folder(d, "cpu", torch.bfloat16)
    whole = {k: v.clone() for k, v in whole.tensors.items() if v is not None}
    _split_into_shards(d, with_index)
    _, _, pool = load_model_folder(d, "cpu", torch.bfloat16)
    assert set(whole) == {k for k, v in pool.tensors.items() if v is not None}
    assert all(torch.equal(pool[k], v) for k, v in whole.items())


def test_tensor_in_two_shards_is_an_error(tmp_path):
    d = write_model_folder(TINY_B, 5, str(tmp_path / "m"))
    t = _split_into_shards(d, with_index=False)
    extra = load_file(os.path.join(d, "model-00002-of-00002.safetensors"))
    extra["model.norm.weight"] = t["model.norm.weight"]
    extra["model.embed_tokens.weight"] = t["model.embed_tokens.weight"]
    save_file(extra, os.path.join(d, "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightError) as e:
        load_model_folder(d, "cpu", torch.bfloat16)
    assert "more than one shard" in str(e.value) and "model.norm.weight" in str(e.value)


def test_half_precision_files_are_kept_in_bf16_and_float32_engine_upcasts(tmp_path):
    d = write_model_folder(TINY_A, 2, str(tmp_path / "m"))
    path = os.path.join(d, "model.safetensors")
    t = {k: v.to(torch.float16) for k, v in load_file(path).items()}
    save_file(t, path)
    _, _, pool = load_model_folder(d, "cpu", torch.bfloat16)
    assert all(v.dtype == torch.bfloat16 for v in pool.tensors.values() if v is not None)
    assert torch.equal(pool["final_norm.weight"], t["model.norm.weight"].to(torch.bfloat16))
    _, _, pool32 = load_model_folder(d, "cpu", torch.float32)
    assert torch.equal(pool32["final_norm.weight"], t["model.norm.weight"].float())
