"""Adapter / training-state files: the reference's own unit tests for this format
(ferrotensor-trainer/src/checkpoint.rs:618-918) restated against the Python host, plus an
independent reader (the `safetensors` package) over the files this library writes."""

import json
import os

import numpy as np
import pytest

from ferrotensor_b200 import checkpoint as ck


def _checkpoint_at(step, values):
    """checkpoint.rs:789-817"""
    ts = ck.TrainingState.new(100)
    ts.step = step

    def state(seed):
        data = (np.float32(seed) + np.arange(values, dtype=np.float32) * np.float32(1e-3)).astype(np.float32)
        return ck.OptimizerTensorState([values // 4, 4], data)
    adam = ck.AdamWCheckpoint(5e-4, 0.9, 0.999, 1e-8, 0.0, float(step),
                              {"layers.0.q_proj.lora_a": state(0.25), "layers.0.q_proj.lora_b": state(-0.5)},
                              {"layers.0.q_proj.lora_a": state(1e-6), "layers.0.q_proj.lora_b": state(2e-6)})
    return ck.TrainingCheckpoint(ts, adam, None)


def test_metadata_keeps_lora_settings_and_trained_modules_apart():
    lora = ck.LoraMetadata(8, 16.0, ["q_proj", "v_proj"], None)
    m = lora.to_map()
    assert m["format"] == "ferrotensor-lora" and "trained_modules" not in m
    assert m["alpha"] == "16" and m["rank"] == "8" and m["target_modules"] == "q_proj,v_proj"
    assert ck.LoraMetadata.from_map(m) == lora
    w = ck.LoraMetadata.trained_weights("attn")
    m = w.to_map()
    assert m["format"] == "ferrotensor-weights" and m["trained_modules"] == "attn"
    assert ck.LoraMetadata.from_map(m) == w
    old = {"format": "ferrotensor-lora", "rank": "4", "alpha": "8", "target_modules": "q_proj"}
    assert ck.LoraMetadata.from_map(old).trained_modules is None
    assert ck.LoraMetadata.from_map({"rank": "x"}) is None


def test_resume_validation():
    s = ck.TrainingState.new(10)
    s.task, s.train_modules, s.sequence_length, s.model_path = "sft", "lora", 128, "/models/a"
    s.validate_resume("lora", "sft", 128, "/models/a")
    with pytest.raises(ck.CheckpointError, match="task"):
        s.validate_resume("lora", "pretrain", 128, "/models/a")
    with pytest.raises(ck.CheckpointError, match="sequence_length"):
        s.validate_resume("lora", "sft", 64, "/models/a")
    with pytest.raises(ck.CheckpointError, match="model_path"):
        s.validate_resume("lora", "sft", 128, "/models/b")


def test_training_checkpoint_roundtrip_preserves_resume_state(tmp_path):
    path = tmp_path / "resume.state.json"
    ts = ck.TrainingState.new(100)
    ts.step, ts.epoch, ts.task, ts.train_modules, ts.sequence_length = 42, 1, "pretrain", "lora", 128
    ts.model_path, ts.dataset_path, ts.grad_accum_steps, ts.fp16 = "/models/tiny", "./data/train.bin", 8, True
    cp = ck.TrainingCheckpoint(ts, ck.AdamWCheckpoint(1e-4, 0.9, 0.999, 1e-8, 0.01, 42.0),
                               ck.GradScalerCheckpoint(1024.0, 2.0, 0.5, 2000, 3, False, True))
    cp.save(path)
    text = path.read_text()
    # serde's layout: externally tagged optimizer enum, f32 printed with the shortest digits
    obj = json.loads(text)
    assert list(obj) == ["training_state", "optimizer_state", "grad_scaler_state"]
    assert obj["optimizer_state"]["AdamW"]["lr"] == 0.0001 and '"lr": 0.0001' in text
    assert "q4_weights" not in obj["training_state"]
    back = ck.TrainingCheckpoint.load(path)
    assert back.training_state.step == 42 and back.training_state.task == "pretrain"
    back.training_state.validate_resume("lora", "pretrain", 128, "/models/tiny")
    assert back.optimizer_state.t == 42.0 and back.grad_scaler_state.scale == 1024.0
    assert not ck.moments_path(path).exists()      # no moments: no second file


def test_moments_round_trip_through_safetensors_bit_for_bit(tmp_path):
    path = tmp_path / "moments.state.json"
    cp = _checkpoint_at(7, 40_000)
    cp.save(path)
    assert ck.moments_path(path).name == "moments.state.safetensors"
    assert len(path.read_text()) < 4_000
    assert ck.moments_path(path).stat().st_size >= 4 * 40_000 * 4
    back = ck.TrainingCheckpoint.load(path)
    a, b = cp.optimizer_state, back.optimizer_state
    assert b.t == 7.0
    for orig, got in ((a.m_states, b.m_states), (a.v_states, b.v_states)):
        assert set(orig) == set(got)
        for name, t in orig.items():
            assert got[name].shape == t.shape
            assert np.array_equal(got[name].data.view(np.uint32), t.data.view(np.uint32)), name


def test_moments_from_another_step_are_rejected(tmp_path):
    path = tmp_path / "mismatch.state.json"
    _checkpoint_at(5, 400).save(path)
    stale = ck.moments_path(path).read_bytes()
    _checkpoint_at(6, 400).save(path)
    ck.moments_path(path).write_bytes(stale)
    with pytest.raises(ck.CheckpointError) as e:
        ck.TrainingCheckpoint.load(path)
    assert "step 5" in str(e.value) and "step 6" in str(e.value)


def test_inline_json_checkpoints_still_load(tmp_path):
    path = tmp_path / "inline.state.json"
    cp = _checkpoint_at(3, 8)
    path.write_text(json.dumps(cp._json_obj(True)))
    back = ck.TrainingCheckpoint.load(path)
    assert not ck.moments_path(path).exists()
    name = "layers.0.q_proj.lora_b"
    assert np.array_equal(back.optimizer_state.m_states[name].data, cp.optimizer_state.m_states[name].data)


def test_adapter_file_layout_and_independent_reader(tmp_path):
    """The container as the reference's safetensors crate writes it: u64 header length, JSON header
    padded to 8 bytes, tensors in name order; read back by the `safetensors` package."""
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(0)
    tensors = {"model.layers.0.self_attn.q_proj.lora_B.weight": rng.standard_normal((4, 24), dtype=np.float32),
               "model.layers.0.self_attn.q_proj.lora_A.weight": rng.standard_normal((24, 4), dtype=np.float32)}
    path = tmp_path / "adapter.safetensors"
    ck.save_lora_checkpoint(path, tensors, ck.LoraMetadata(4, 8.0, ["q_proj"]))
    raw = path.read_bytes()
    n = int.from_bytes(raw[:8], "little")
    assert n % 8 == 0
    header = json.loads(raw[8:8 + n])
    assert header["__metadata__"] == {"format": "ferrotensor-lora", "rank": "4", "alpha": "8",
                                      "target_modules": "q_proj"}
    a, b = "model.layers.0.self_attn.q_proj.lora_A.weight", "model.layers.0.self_attn.q_proj.lora_B.weight"
    assert header[a]["data_offsets"] == [0, 384] and header[b]["data_offsets"] == [384, 768]
    assert header[a] == {"dtype": "F32", "shape": [24, 4], "data_offsets": [0, 384]}
    other = st.load_file(str(path))
    for k, v in tensors.items():
        assert np.array_equal(other[k], v)
    # and the other way: a file written by the package, with F16 and BF16 tensors, loads as f32
    import torch
    from safetensors.torch import save_file
    t16 = torch.randn(8, 4).half()
    tb = torch.randn(4, 8).bfloat16()
    save_file({"x.lora_A.weight": t16, "x.lora_B.weight": tb}, str(tmp_path / "half.safetensors"),
              metadata={"format": "ferrotensor-lora", "rank": "4", "alpha": "8.5", "target_modules": "x"})
    cp = ck.load_lora_checkpoint(tmp_path / "half.safetensors")
    assert cp.metadata == ck.LoraMetadata(4, 8.5, ["x"])
    assert np.array_equal(cp.tensors["x.lora_A.weight"][1], t16.float().numpy())
    assert np.array_equal(cp.tensors["x.lora_B.weight"][1], tb.float().numpy())
    assert not os.path.exists(str(path) + ".tmp")


def test_resolve_checkpoint_is_all_or_nothing():
    z = np.zeros((4, 2), np.float32)
    new = "model.layers.0.mlp.gate_proj.lora_A.weight"
    old = "model.layers.0.feed_forward.gate_proj.lora_A.weight"
    assert ck.legacy_llama_name(new) == old and ck.legacy_llama_name("lm_head.lora_A.weight") is None
    assert ck.resolve_checkpoint(ck.LoraCheckpoint({old: ([4, 2], z)}, None), {new: [4, 2]}) == {new: old}
    with pytest.raises(ck.CheckpointError, match="both"):
        ck.resolve_checkpoint(ck.LoraCheckpoint({old: ([4, 2], z), new: ([4, 2], z)}, None), {new: [4, 2]})
    with pytest.raises(ck.CheckpointError, match="no tensor"):
        ck.resolve_checkpoint(ck.LoraCheckpoint({}, None), {new: [4, 2]})
    with pytest.raises(ck.CheckpointError, match="shape"):
        ck.resolve_checkpoint(ck.LoraCheckpoint({new: ([2, 4], z.T)}, None), {new: [4, 2]})
    with pytest.raises(ck.CheckpointError, match="does not have"):
        ck.resolve_checkpoint(ck.LoraCheckpoint({new: ([4, 2], z), "extra": ([1], z[:1, 0])}, None), {new: [4, 2]})
    assert ck.reference_tensor_name("model.layers.3.self_attn.v_proj.lora_b") == \
        "model.layers.3.self_attn.v_proj.lora_B.weight"
    assert ck.host_tensor_name("lm_head.lora_A.weight") == "lm_head.lora_a"


@pytest.mark.gpu
def test_resume_continues_bit_for_bit(cuda_ctx, tmp_path):
    """Two steps, save, rebuild everything from the files, one more step == three steps straight."""
    import copy
    import torch
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights, synthetic_batch
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    w = copy.deepcopy(WORKLOADS["tiny"])
    weights = init_weights(w.model, 5, f16_base=w.f16_base)
    adapters = init_adapters(w.model, w.lora, 5, b_std=0.02)
    batches = [synthetic_batch(w, 2, seed=10 + i) for i in range(3)]

    def fresh():
        model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=w.f16_base)
        return model, Trainer(model, AdamW(1e-2, weight_decay=0.0)).with_grad_accum_steps(2).with_clip_grad_norm(1.0)

    model, tr = fresh()
    for ids, tg, mk in batches:
        tr.train_arrays(ids, tg, mk)
    straight = model.params.clone()
    model.close()

    model, tr = fresh()
    for ids, tg, mk in batches[:2]:
        tr.train_arrays(ids, tg, mk)
    ts = ck.TrainingState.new(3)
    ts.step, ts.lr, ts.sequence_length = 2, 1e-2, w.seq_len
    tr.save_adapter(tmp_path / "adapter.safetensors")
    tr.save_training_checkpoint(tmp_path / "adapter.state.json", ts)
    model.close()
    assert (tmp_path / "adapter.state.safetensors").exists()

    model, tr = fresh()
    n = tr.load_adapter(tmp_path / "adapter.safetensors")
    assert n == len(model.adapter_names())
    state = tr.load_training_checkpoint(tmp_path / "adapter.state.json")
    assert state.step == 2 and tr.optimizer.t == 2.0
    tr.train_arrays(*batches[2])
    assert torch.equal(model.params, straight)
    cp = ck.load_lora_checkpoint(tmp_path / "adapter.safetensors")
    assert cp.metadata.rank == w.lora.rank and cp.metadata.target_modules == list(w.lora.target_modules)
    assert all(k.endswith((".lora_A.weight", ".lora_B.weight")) for k in cp.tensors)
    model.close()


# ---- optimizer-state matching (ferrotensor-autograd/src/lib.rs:1668-1703 and its tests :1940-2062),
# ---- old Llama-block names (ferrotensor-graph/src/lfm.rs:234-255, :775-813)

def _moment(shape):
    return ck.OptimizerTensorState(shape=list(shape), data=np.full(int(np.prod(shape)), 0.5, np.float32))


def _saved_state(params):
    return ck.AdamWCheckpoint(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, t=3.0,
                              m_states={n: _moment(s) for n, s in params},
                              v_states={n: _moment(s) for n, s in params})


def test_saved_moments_match_the_same_parameters():
    shapes = {"a.weight": (2, 3), "b.weight": (4,)}
    matched, report = ck.match_moments(shapes, _saved_state([("a.weight", (2, 3)), ("b.weight", (4,))]))
    assert matched == ["a.weight", "b.weight"]
    assert (report.matched, report.missing, report.unused) == (2, 0, 0)


def test_saved_moments_of_other_parameters_match_none():
    shapes = {"x.weight": (2, 3), "y.weight": (4,)}
    matched, report = ck.match_moments(shapes, _saved_state([("a.weight", (2, 3)), ("b.weight", (4,))]))
    assert matched == []
    assert (report.matched, report.missing, report.unused) == (0, 2, 2)


def test_partial_overlap_reports_both_sides():
    shapes = {"a.weight": (2,), "b.weight": (2,), "c.weight": (2,)}
    matched, report = ck.match_moments(shapes, _saved_state([("a.weight", (2,)), ("old.weight", (2,))]))
    assert matched == ["a.weight"]
    assert (report.matched, report.missing, report.unused) == (1, 2, 1)


def test_a_moment_with_only_one_half_is_not_applied():
    state = _saved_state([("a.weight", (2,))])
    state.v_states.clear()
    matched, report = ck.match_moments({"a.weight": (2,)}, state)
    assert matched == [] and (report.missing, report.unused) == (1, 1)


def test_a_moment_of_the_wrong_shape_is_an_error():
    with pytest.raises(ck.CheckpointError) as e:
        ck.match_moments({"a.weight": (2, 3)}, _saved_state([("a.weight", (3, 2))]))
    assert "a.weight" in str(e.value) and "shape" in str(e.value)
    state = _saved_state([("a.weight", (2, 3))])       # the shape agrees, the value count does not
    state.v_states["a.weight"].data = state.v_states["a.weight"].data[:-1]
    with pytest.raises(ck.CheckpointError):
        ck.match_moments({"a.weight": (2, 3)}, state)


def test_llama_block_names_map_to_the_old_names():
    pairs = [("model.layers.3.input_layernorm.weight", "model.layers.3.operator_norm.weight"),
             ("model.layers.3.post_attention_layernorm.weight", "model.layers.3.ffn_norm.weight"),
             ("model.layers.0.mlp.gate_proj.lora_A.weight", "model.layers.0.feed_forward.gate_proj.lora_A.weight"),
             ("model.layers.11.mlp.down_proj.weight", "model.layers.11.feed_forward.down_proj.weight")]
    for new, old in pairs:
        assert ck.legacy_llama_name(new) == old
    for name in ["model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.q_proj.lora_A.weight",
                 "model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"]:
        assert ck.legacy_llama_name(name) is None, name


def test_moments_under_old_names_are_renamed_before_matching():
    new = "model.layers.0.mlp.gate_proj.lora_A.weight"
    old = "model.layers.0.feed_forward.gate_proj.lora_A.weight"
    keep = "model.layers.0.self_attn.q_proj.lora_A.weight"
    state = _saved_state([(old, (4, 2)), (keep, (4, 2))])
    assert ck.upgrade_optimizer_names(state, [new, keep]) == 2          # one name, both moments
    assert set(state.m_states) == {new, keep} and set(state.v_states) == {new, keep}
    assert ck.upgrade_optimizer_names(state, [new, keep]) == 0
    matched, report = ck.match_moments({new: (4, 2), keep: (4, 2)}, state)
    assert matched == sorted([new, keep]) and report.unused == 0


@pytest.mark.gpu
def test_optimizer_state_loads_as_the_reference_loads_it(cuda_ctx, tmp_path):
    """`AdamW::load_state` semantics on the device buffers: a file whose moments belong to other
    parameters leaves the optimizer untouched; a partial match restores the hyper-parameters and
    step count, copies the matched moments and zeroes the others; old Llama-block names are
    renamed first; a moment of the wrong shape is an error and nothing changes."""
    import copy
    import json
    import torch
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights, synthetic_batch
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer
    w = copy.deepcopy(WORKLOADS["tiny"])
    weights = init_weights(w.model, 5, f16_base=w.f16_base)
    adapters = init_adapters(w.model, w.lora, 5, b_std=0.02)
    model = LoraModel(cuda_ctx, w.model, w.lora, weights, adapters, f16_base=w.f16_base)
    tr = Trainer(model, AdamW(1e-2, weight_decay=0.0)).with_grad_accum_steps(2)
    tr.train_arrays(*synthetic_batch(w, 2, seed=3))
    path = tmp_path / "run.state.json"
    tr.save_training_checkpoint(path, ck.TrainingState.new(3))
    cp = ck.TrainingCheckpoint.load(path)
    a = cp.optimizer_state
    names = sorted(a.m_states)
    assert names and all(float(np.abs(a.m_states[n].data).max()) > 0 for n in names)
    m_dev, v_dev = model.named_moments()
    host_of = {ck.reference_tensor_name(n): n for n in m_dev}

    def write(state):
        ck.TrainingCheckpoint(optimizer_state=state, training_state=cp.training_state).save(tmp_path / "edit.state.json")
        return tmp_path / "edit.state.json"

    def reset():
        tr.optimizer.lr, tr.optimizer.t = 7e-3, 9.0
        for t in list(m_dev.values()) + list(v_dev.values()):
            t.fill_(0.25)

    # (a) nothing matches: untouched
    other = copy.deepcopy(a)
    other.m_states = {"x." + n: s for n, s in a.m_states.items()}
    other.v_states = {"x." + n: s for n, s in a.v_states.items()}
    reset()
    tr.load_training_checkpoint(write(other))
    assert tr.last_optimizer_load.matched == 0 and tr.last_optimizer_load.unused == len(names)
    assert tr.optimizer.lr == 7e-3 and tr.optimizer.t == 9.0
    assert all(float(t.min()) == 0.25 and float(t.max()) == 0.25 for t in m_dev.values())

    # (b) one parameter lost its second moment, one is stored under its old name
    part = copy.deepcopy(a)
    dropped = next(n for n in names if ".self_attn." in n)
    del part.v_states[dropped]
    renamed = next(n for n in names if ".mlp." in n)
    old = ck.legacy_llama_name(renamed)
    part.m_states[old] = part.m_states.pop(renamed)
    part.v_states[old] = part.v_states.pop(renamed)
    reset()
    tr.load_training_checkpoint(write(part))
    rep = tr.last_optimizer_load
    assert (rep.matched, rep.missing, rep.unused) == (len(names) - 1, 1, 1)
    assert tr.optimizer.lr == a.lr and tr.optimizer.t == a.t
    assert not m_dev[host_of[dropped]].any() and not v_dev[host_of[dropped]].any()
    got = m_dev[host_of[renamed]].cpu().numpy().reshape(-1)
    assert np.array_equal(got, np.asarray(a.m_states[renamed].data, np.float32).reshape(-1))

    # (c) a moment of the wrong shape: an error, nothing changed
    bad = copy.deepcopy(a)
    s = bad.v_states[names[-1]]
    s.shape = list(reversed(s.shape)) if len(s.shape) == 2 and s.shape[0] != s.shape[1] else [int(np.prod(s.shape))]
    reset()
    with pytest.raises(ck.CheckpointError):
        tr.load_training_checkpoint(write(bad))
    assert tr.optimizer.lr == 7e-3 and tr.optimizer.t == 9.0
    assert all(float(t.min()) == 0.25 and float(t.max()) == 0.25 for t in v_dev.values())
    model.close()
