"""Checkpoint-directory ingestion: the reference's `check_supported` unit tests
(ferrotensor-graph/src/model_builder.rs:766-870) restated, the directory rules of
ferrotensor-loader/src/lib.rs:452-503, and a model built from files on the GPU."""

import copy
import json

import numpy as np
import pytest
import torch

from ferrotensor_b200 import loader as ld
from ferrotensor_b200.checkpoint import write_safetensors


def _qwen2_5_config():
    """The config.json of Qwen2.5-0.5B as the reference's test holds it (model_builder.rs:770-797)."""
    return {"architectures": ["Qwen2ForCausalLM"], "attention_dropout": 0.0, "bos_token_id": 151643,
            "eos_token_id": 151643, "hidden_act": "silu", "hidden_size": 896, "initializer_range": 0.02,
            "intermediate_size": 4864, "max_position_embeddings": 32768, "max_window_layers": 24,
            "model_type": "qwen2", "num_attention_heads": 14, "num_hidden_layers": 24,
            "num_key_value_heads": 2, "rms_norm_eps": 1e-06, "rope_theta": 1000000.0,
            "sliding_window": 32768, "tie_word_embeddings": True, "torch_dtype": "bfloat16",
            "use_cache": True, "use_sliding_window": False, "vocab_size": 151936}


def _check_with(changes):
    c = _qwen2_5_config()
    c.update(changes)
    ld.check_supported(c)
    return c


def test_qwen2_5_config_is_supported():
    cfg = ld.model_config_from_json(_check_with({}))
    assert (cfg.hidden, cfg.ffn, cfg.heads, cfg.kv_heads, cfg.layers, cfg.vocab) == (896, 4864, 14, 2, 24, 151936)
    assert cfg.head_dim == 64 and cfg.tied and cfg.theta == 1e6 and abs(cfg.eps - 1e-6) < 1e-12
    c = _check_with({"rope_theta": None, "rope_parameters": {"rope_type": "default", "rope_theta": 1000000.0}})
    assert ld.model_config_from_json(c).theta == 1e6
    _check_with({"use_sliding_window": None, "sliding_window": 4096})
    _check_with({"rope_scaling": {"rope_theta": 1000000.0}})
    # defaults: no eps, no KV heads, no theta
    c = {k: v for k, v in _qwen2_5_config().items() if k not in ("rms_norm_eps", "num_key_value_heads", "rope_theta")}
    cfg = ld.model_config_from_json(c)
    assert abs(cfg.eps - 1e-5) < 1e-12 and cfg.kv_heads == 14 and cfg.theta == 10000.0


@pytest.mark.parametrize("changes,message", [
    ({"hidden_act": "gelu_pytorch_tanh"},
     'hidden_act "gelu_pytorch_tanh" is not supported: the MLP computes SiLU (silu) only'),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}},
     'rope_scaling type "llama3" is not supported: RoPE runs unscaled'),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}},
     'rope_scaling type "linear" is not supported: RoPE runs unscaled'),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6}},
     'rope_parameters type "yarn" is not supported: RoPE runs unscaled'),
    ({"use_sliding_window": True},
     "sliding_window 32768 is not supported: attention always covers the whole sequence"),
    ({"rope_scaling": {"factor": 4.0}},
     'rope_scaling type "unnamed" is not supported: RoPE runs unscaled'),
])
def test_unsupported_config_features_are_named(changes, message):
    with pytest.raises(ld.BuildError) as e:
        _check_with(changes)
    assert str(e.value) == message


def _tiny(tied=False, bias=False):
    from ferrotensor_b200.config import WORKLOADS, init_weights
    w = copy.deepcopy(WORKLOADS["tiny"])
    w.model.tied, w.model.qkv_bias = tied, bias
    weights = init_weights(w.model, 3, f16_base=False)
    c = w.model
    cfg = {"hidden_size": c.hidden, "intermediate_size": c.ffn, "num_attention_heads": c.heads,
           "num_hidden_layers": c.layers, "vocab_size": c.vocab, "num_key_value_heads": c.kv_heads,
           "rms_norm_eps": c.eps, "rope_theta": c.theta, "hidden_act": "silu", "model_type": "llama",
           "tie_word_embeddings": tied, "head_dim": c.head_dim}
    return w, weights, cfg


def _write_dir(path, weights, cfg, shards=1):
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    arrays = {k: v.numpy() for k, v in weights.items()}
    if shards == 1:
        write_safetensors(path / "model.safetensors", arrays)
        return
    names = sorted(arrays)
    wm = {}
    for s in range(shards):
        part = {n: arrays[n] for n in names[s::shards]}
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(path / fname, part)
        wm.update({n: fname for n in part})
    (path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))


@pytest.mark.parametrize("shards", [1, 3])
def test_directory_round_trip(tmp_path, shards):
    w, weights, cfg = _tiny(tied=True, bias=True)
    _write_dir(tmp_path / "m", weights, cfg, shards)
    mc, got, raw = ld.load_model_dir(tmp_path / "m")
    assert mc.tied and mc.qkv_bias and raw["model_type"] == "llama"
    assert (mc.hidden, mc.ffn, mc.layers, mc.heads, mc.kv_heads, mc.vocab, mc.head_dim) == \
        (w.model.hidden, w.model.ffn, w.model.layers, w.model.heads, w.model.kv_heads, w.model.vocab, w.model.head_dim)
    assert set(got) == set(weights)
    for k in weights:
        assert torch.equal(got[k], weights[k]), k


def test_half_precision_files_and_directory_rules(tmp_path):
    from safetensors.torch import save_file
    w, weights, cfg = _tiny()
    d = tmp_path / "bf16"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    save_file({k: (v.bfloat16() if v.dim() == 2 else v.half()) for k, v in weights.items()},
              str(d / "consolidated.safetensors"))
    mc, got, _ = ld.load_model_dir(d)
    assert not mc.tied and not mc.qkv_bias
    for k, v in weights.items():
        exp = v.bfloat16().float() if v.dim() == 2 else v.half().float()
        assert torch.equal(got[k], exp), k
    # no weights at all
    e = tmp_path / "empty"
    e.mkdir()
    (e / "config.json").write_text(json.dumps(cfg))
    with pytest.raises(ld.LoaderError, match="no model.safetensors, consolidated.safetensors"):
        ld.load_model_dir(e)
    # a shard name that leaves the directory
    (e / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../evil.safetensors"}}))
    with pytest.raises(ld.LoaderError, match="not a relative path inside the model directory"):
        ld.load_model_dir(e)
    (e / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(ld.LoaderError, match="weight_map lists no weights"):
        ld.load_model_dir(e)
    # a tensor whose shape contradicts the config
    bad = dict(weights)
    bad["model.norm.weight"] = torch.ones(w.model.hidden + 1)
    _write_dir(tmp_path / "bad", bad, cfg)
    with pytest.raises(ld.BuildError, match="model.norm.weight has shape"):
        ld.load_model_dir(tmp_path / "bad")


@pytest.mark.gpu
def test_model_from_files_steps_like_model_from_memory(cuda_ctx, tmp_path):
    from ferrotensor_b200.config import init_adapters, synthetic_batch
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    w, weights, cfg = _tiny(tied=True, bias=True)
    _write_dir(tmp_path / "m", weights, cfg, shards=2)
    mc, loaded, _ = ld.load_model_dir(tmp_path / "m")
    adapters = init_adapters(w.model, w.lora, 9, b_std=0.02)
    ids, tg, mk = synthetic_batch(w, 2)
    grads = []
    for conf, wts in ((w.model, weights), (mc, loaded)):
        model = LoraModel(cuda_ctx, conf, w.lora, wts, adapters, f16_base=False)
        tr = Trainer(model, AdamW(0.0)).with_grad_accum_steps(2)
        model.zero_grad()
        tr._run_chunk(ids, tg, mk)
        stats = tr._collect()
        grads.append((model.grads.clone(), [s.loss for s in stats]))
        model.close()
    assert torch.equal(grads[0][0], grads[1][0]) and grads[0][1] == grads[1][1]
