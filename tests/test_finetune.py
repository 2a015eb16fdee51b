"""The caller of the step: tokenizer rules (ferrotensor-loader/src/tokenizer.rs tests :753-793
restated), dataset formats and command-line defaults of `train` (ferrotensor-cli/src/main.rs
tests :2070-2134, :2434-2483, :2599-2627 restated), and on the GPU a whole run from a model
directory and a text dataset to a saved adapter, with a resume that lands on the same bits."""

import copy
import json
import math

import numpy as np
import pytest

from ferrotensor_b200 import finetune as ft
from ferrotensor_b200 import tokenizer as tk
from ferrotensor_b200.checkpoint import LoraMetadata


def _chatml_vocab_json(plain=False):
    vocab = {"<|endoftext|>": 0, "<|im_start|>": 1, "<|im_end|>": 2, "Hi": 3}
    if plain:
        return {"model": {"vocab": vocab}}
    return {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
            "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
            "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "<|endoftext|>"}}


def _load(tmp_path, tag, tok_json, config=None):
    d = tmp_path / tag
    d.mkdir()
    (d / "tokenizer.json").write_text(json.dumps(tok_json))
    if config is not None:
        (d / "tokenizer_config.json").write_text(config)
    return tk.Tokenizer.from_file(d / "tokenizer.json")


def test_declared_bos_token_replaces_the_chatml_guess(tmp_path):
    guessed = _load(tmp_path, "none", _chatml_vocab_json())
    assert guessed.hf_tokenizer is not None and guessed.bos_token_id == 1
    for tag, config, bos in [("string", '{"bos_token": "<|endoftext|>"}', 0),
                             ("object", '{"bos_token": {"content": "<|endoftext|>", "special": true}}', 0),
                             ("null", '{"bos_token": null}', 1), ("unknown", '{"bos_token": "<s>"}', 1)]:
        tok = _load(tmp_path, tag, _chatml_vocab_json(), config)
        assert (tok.bos_token_id, tok.eos_token_id, tok.pad_token_id) == (bos, 2, 0), config
        assert tok.encode("Hi Hi") == guessed.encode("Hi Hi") == [3, 3]


def test_plain_vocabulary_reader(tmp_path):
    guessed = _load(tmp_path, "plain", _chatml_vocab_json(plain=True))
    assert guessed.hf_tokenizer is None and guessed.encode("Hi") == [1, 3]
    assert guessed.encode_continuation("Hi Hi") == [3, 3]
    declared = _load(tmp_path, "declared", _chatml_vocab_json(plain=True), '{"bos_token": "<|endoftext|>"}')
    assert declared.encode("Hi") == [0, 3] and declared.decode([1, 3, 2]) == "<|im_start|>Hi"
    with pytest.raises(tk.TokenizerError, match="used by more than one token"):
        _load(tmp_path, "dup", {"model": {"vocab": {"a": 1, "b": 1}}})
    with pytest.raises(tk.TokenizerError, match="vocabulary is empty"):
        _load(tmp_path, "empty", {"model": {"vocab": {}}})
    with pytest.raises(tk.TokenizerError, match="cannot load the Nonsense tokenizer"):
        _load(tmp_path, "typed", {"model": {"type": "Nonsense", "vocab": {"a": 1}}})


def test_byte_level_tokenizer_and_chat_prompt(tmp_path):
    tok = _load(tmp_path, "bytes", tk.byte_level_tokenizer_json())
    assert (tok.bos_token_id, tok.eos_token_id, tok.pad_token_id) == (1, 2, 0)
    text = "Hi é\n<s>"
    assert tok.encode(text) == [b + 3 for b in text.encode()] and tok.decode(tok.encode(text)) == text
    assert tk.chat_prompt(None, "q") == "<|im_start|>user\nq<|im_end|>\n<|im_start|>assistant\n"
    assert tk.conversation_prompt("s", ["a", "b", "c"]) == (
        "<|im_start|>system\ns<|im_end|>\n<|im_start|>user\na<|im_end|>\n<|im_start|>assistant\nb<|im_end|>\n"
        "<|im_start|>user\nc<|im_end|>\n<|im_start|>assistant\n")
    ex = ft.build_sft_example(tok, "q", "ab", None, True, 256)
    prompt = tok.encode_chat(None, "q")
    assert ex.input_ids == (prompt + [ord("a") + 3, ord("b") + 3])
    assert ex.target_ids[-1] == tok.eos_token_id and sum(ex.loss_mask) == 3
    raw = ft.build_sft_example(tok, "q", "ab", None, False, 256)
    assert raw.input_ids == [ord("q") + 3, ord("a") + 3] and raw.target_ids == [ord("a") + 3, ord("b") + 3]
    assert ft.build_sft_example(tok, "a long prompt", "x", None, True, 8) is None


def test_dataset_formats(tmp_path):
    tok = _load(tmp_path, "bytes", tk.byte_level_tokenizer_json())
    rows = [{"prompt": "2+2?", "response": "4"}, {"prompt": "x" * 300, "response": "y"},
            {"prompt": "hi", "response": "there", "system": "be brief"}]
    (tmp_path / "a.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n\n")
    (tmp_path / "a.json").write_text(json.dumps(rows))
    for name in ("a.jsonl", "a.json"):
        ds = ft.load_dataset(tmp_path / name, "sft", 128, tok)
        assert len(ds) == 2                                   # the 300-byte prompt does not fit
        assert ds.examples()[1].input_ids[:len(tok.encode_chat("be brief", "hi"))] == tok.encode_chat("be brief", "hi")
    assert len(ft.load_dataset(tmp_path / "a.jsonl", "sft", 128, tok, max_samples=1)) == 1
    (tmp_path / "ids.jsonl").write_text(json.dumps({"prompt_ids": [1, 5, 6], "response_ids": [7, 2]}) + "\n")
    ds = ft.load_dataset(tmp_path / "ids.jsonl", "sft", 16)   # already tokenised: no tokenizer needed
    assert ds.examples()[0].loss_mask == [0, 0, 1, 1]
    with pytest.raises(ft.Unmet, match="need a tokenizer.json"):
        ft.load_dataset(tmp_path / "a.jsonl", "sft", 64)
    with pytest.raises(ft.Unmet, match="line 1: expected"):
        (tmp_path / "bad.jsonl").write_text("{not json\n")
        ft.load_dataset(tmp_path / "bad.jsonl", "sft", 64, tok)
    with pytest.raises(ft.Unmet, match="use --task pretrain"):
        (tmp_path / "t.txt").write_text("some text\n")
        ft.load_dataset(tmp_path / "t.txt", "sft", 64, tok)
    with pytest.raises(ft.Unmet, match="does not exist"):
        ft.load_dataset(tmp_path / "missing.jsonl", "sft", 64, tok)
    with pytest.raises(ft.Unmet, match="at least 2"):
        ft.load_dataset(tmp_path / "a.jsonl", "sft", 1, tok)
    with pytest.raises(ft.Unmet, match="produced no usable examples"):
        ft.load_dataset(tmp_path / "a.jsonl", "sft", 4, tok)
    # pretrain: token files, token arrays, text lines
    (tmp_path / "t.bin").write_bytes(np.arange(1, 8, dtype="<u4").tobytes())
    (tmp_path / "t.json").write_text(json.dumps(list(range(1, 8))))
    for name in ("t.bin", "t.json"):
        assert [e.input_ids for e in ft.load_dataset(tmp_path / name, "pretrain", 4).examples()] == [[1, 2, 3], [4, 5, 6]]
    (tmp_path / "lines.json").write_text(json.dumps(["abc", "", "de"]))
    (tmp_path / "lines.txt").write_text("abc\n\nde\n")
    for name in ("lines.json", "lines.txt"):
        ds = ft.load_dataset(tmp_path / name, "pretrain", 8, tok)
        assert [e.input_ids + e.target_ids[-1:] for e in ds.examples()] == [[b + 3 for b in b"abcde"]]
    with pytest.raises(ft.Unmet, match=r"must be \[token ids\]"):
        (tmp_path / "odd.json").write_text('{"a": 1}')
        ft.load_dataset(tmp_path / "odd.json", "pretrain", 8, tok)


def test_command_line_defaults_and_helpers(tmp_path):
    a = ft.parse_args(["--model", "m", "--data", "d.jsonl"])
    assert (a.task, a.seq_len, a.out, a.lr, a.warmup_steps, a.epochs, a.max_steps) == ("sft", 256, "outputs/run", 2e-4, 10, 1, None)
    assert (a.batch_size, a.grad_accum, a.grad_clip, a.weight_decay) == (1, 4, 1.0, 0.0)
    assert (a.lora_rank, a.lora_alpha, a.lora_targets) == (8, 16.0, ["q_proj", "k_proj", "v_proj", "o_proj"])
    assert (a.log_every, a.save_every, a.eval_every, a.eval_samples, a.seed, a.train_modules) == (10, 0, 0, 64, 0, "lora")
    b = ft.parse_args(["--model", "m", "--dataset", "d.bin", "--task", "pretrain", "--seq-len", "64", "--max-steps", "7",
                       "--lora-targets", "q_proj, down_proj", "--lite", "--json", "--checkpoint-blocks"])
    assert (b.data, b.task, b.seq_len, b.max_steps, b.lora_targets) == ("d.bin", "pretrain", 64, 7, ["q_proj", "down_proj"])
    assert b.lite and b.json and b.checkpoint_blocks
    with pytest.raises(SystemExit):
        ft.parse_args(["--model", "m"])
    with pytest.raises(SystemExit):
        ft.parse_args(["--model", "m", "--data", "d", "--lr", "fast"])
    assert ft.state_path_for("out/lora_adapters.safetensors").as_posix() == "out/lora_adapters.safetensors.state.json"
    ft.check_resume_file(None, "lora")
    ft.check_resume_file(LoraMetadata(8, 16.0, ["q_proj"]), "lora")
    with pytest.raises(ft.Unmet, match="resume with --train-modules attn"):
        ft.check_resume_file(LoraMetadata.trained_weights("attn"), "lora")
    s = ft.TrainSummary(3, None, float("nan"), None, 1.5, 10, 0.25, "o", None)
    d = json.loads(s.to_json())
    assert list(d) == ["steps", "first_loss", "final_loss", "eval_loss_before", "eval_loss_after",
                       "measured_peak_mib", "seconds", "out_dir", "adapter"]
    assert d["final_loss"] is None and d["first_loss"] is None and d["eval_loss_after"] == 1.5 and d["adapter"] is None


def test_cli_parses_eval_and_generate_flags():
    from ferrotensor_b200 import cli
    a = cli._parser().parse_args(["eval", "--model", "m", "--dataset", "d.jsonl", "--lora", "a.safetensors", "--json"])
    assert (a.command, a.data, a.lora, a.json, a.task, a.seq_len) == ("eval", "d.jsonl", "a.safetensors", True, "sft", 256)
    g = cli._parser().parse_args(["infer", "--model", "m"])
    assert (g.prompt, g.max_new_tokens, g.temperature, g.top_k, g.top_p, g.seed, g.raw) == ("Hello!", 128, 0.7, 50, 0.9, None, False)
    with pytest.raises(SystemExit):
        cli._parser().parse_args(["eval", "--model", "m"])
    assert cli._json_line({"loss": float("nan"), "n": 1}) == '{"loss": null, "n": 1}'


def test_requests_that_cannot_be_met(tmp_path):
    base = dict(model=str(tmp_path), data=str(tmp_path / "d.jsonl"))
    with pytest.raises(ft.Unmet, match="must be positive"):
        ft.train(ft.TrainArgs(**base, batch_size=0))
    with pytest.raises(ft.Unmet, match="only `lora`"):
        ft.train(ft.TrainArgs(**base, train_modules="attn"))


# ---- a whole run on the device ----------------------------------------------------------------
def _model_dir(tmp_path):
    from ferrotensor_b200.config import WORKLOADS, init_weights
    from tests.test_loader import _write_dir
    w = copy.deepcopy(WORKLOADS["smollm2-135m"])
    w.model.layers, w.model.vocab = 2, 512
    c = w.model
    cfg = {"hidden_size": c.hidden, "intermediate_size": c.ffn, "num_attention_heads": c.heads,
           "num_hidden_layers": c.layers, "vocab_size": c.vocab, "num_key_value_heads": c.kv_heads,
           "rms_norm_eps": c.eps, "rope_theta": c.theta, "hidden_act": "silu", "model_type": "llama",
           "tie_word_embeddings": True, "head_dim": c.head_dim}
    weights = init_weights(c, 5, f16_base=False)
    weights.pop("lm_head.weight", None)
    d = tmp_path / "model"
    _write_dir(d, weights, cfg)
    (d / "tokenizer.json").write_text(json.dumps(tk.byte_level_tokenizer_json()))
    rng = np.random.default_rng(0)
    words = ["red", "green", "blue", "cyan", "pink", "grey"]
    rows = [{"prompt": f"colour {i % 6}?", "response": words[i % 6] + " " * int(rng.integers(0, 3))} for i in range(16)]
    (tmp_path / "train.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (tmp_path / "eval.jsonl").write_text("\n".join(json.dumps(r) for r in rows[:6]))
    return d


class _Stop(Exception):
    pass


@pytest.mark.gpu
def test_run_saves_resumes_and_lands_on_the_same_bits(cuda_ctx, tmp_path, monkeypatch, capsys):
    from ferrotensor_b200 import checkpoint as ck
    from ferrotensor_b200 import trainer as tr_mod
    model_dir = _model_dir(tmp_path)

    def args(out, **kw):
        return ft.TrainArgs(model=str(model_dir), data=str(tmp_path / "train.jsonl"), out=str(tmp_path / out),
                            seq_len=96, lr=5e-3, warmup_steps=2, max_steps=6, batch_size=2, grad_accum=2,
                            lora_targets=["q_proj", "v_proj", "down_proj"], log_every=1, seed=3, **kw)

    whole = ft.train(args("whole", eval_data=str(tmp_path / "eval.jsonl"), eval_every=4, sample_prompt="colour 2?"))
    assert capsys.readouterr().out.endswith("\n")            # the sampled reply went to stdout
    assert whole.steps == 6 and whole.final_loss < whole.first_loss and whole.eval_loss_after < whole.eval_loss_before
    assert whole.measured_peak_mib > 0 and whole.adapter == str(tmp_path / "whole" / "lora_adapters.safetensors")
    lines = [json.loads(l) for l in (tmp_path / "whole" / "metrics.jsonl").read_text().splitlines()]
    assert [l["step"] for l in lines if "loss" in l] == [1, 2, 3, 4, 5, 6]
    assert [l["step"] for l in lines if "eval_loss" in l] == [0, 4, 6]
    assert all(math.isfinite(l["grad_norm"]) and l["lr"] > 0 for l in lines if "loss" in l)
    state = ck.TrainingState.load(tmp_path / "whole" / "training_state.json")
    assert (state.step, state.total_steps, state.batch_size, state.grad_accum_steps, state.sequence_length,
            state.task, state.seed) == (6, 6, 2, 2, 96, "sft", 3)
    saved = ck.load_lora_checkpoint(whole.adapter)
    assert (saved.metadata.rank, saved.metadata.alpha, saved.metadata.target_modules) == (8, 16.0, ["q_proj", "v_proj", "down_proj"])
    assert len(saved) == 2 * 2 * 3

    # eval and generate read the adapter's settings from the file the run wrote
    from ferrotensor_b200 import cli
    capsys.readouterr()
    common = ["--model", str(model_dir), "--json"]
    assert cli.main(["eval", *common, "--data", str(tmp_path / "eval.jsonl"), "--seq-len", "96", "--lora", whole.adapter]) == 0
    with_lora = json.loads(capsys.readouterr().out)
    assert with_lora["examples"] == 6 and with_lora["tokens"] > 0
    assert abs(with_lora["loss"] - whole.eval_loss_after) < 1e-5 and with_lora["perplexity"] == pytest.approx(math.exp(with_lora["loss"]), rel=1e-5)
    assert cli.main(["eval", *common, "--data", str(tmp_path / "eval.jsonl"), "--seq-len", "96"]) == 0
    base_only = json.loads(capsys.readouterr().out)
    assert abs(base_only["loss"] - whole.eval_loss_before) < 1e-5
    assert cli.main(["generate", *common, "--lora", whole.adapter, "--prompt", "colour 2?", "--temperature", "0",
                     "--max-new-tokens", "8"]) == 0
    cap = capsys.readouterr()
    reply = json.loads(cap.out)
    assert reply["prompt_tokens"] > 20 and 0 <= reply["new_tokens"] <= 8 and reply["kv_cache"] is True
    assert reply["text"] + "\n" in cap.err and "prompt +" in cap.err
    assert cli.main(["eval", *common, "--data", str(tmp_path / "missing.jsonl")]) == 2
    capsys.readouterr()

    # the same run stopped right after the save at step 3 ...
    original = tr_mod.Trainer.save_training_checkpoint
    def save_then_stop(self, path, training_state):
        original(self, path, training_state)
        raise _Stop()
    monkeypatch.setattr(tr_mod.Trainer, "save_training_checkpoint", save_then_stop)
    with pytest.raises(_Stop):
        ft.train(args("halves", save_every=3))
    monkeypatch.setattr(tr_mod.Trainer, "save_training_checkpoint", original)
    first = tmp_path / "halves" / "lora_adapters.safetensors"
    assert ck.TrainingCheckpoint.load(ft.state_path_for(first)).training_state.step == 3
    # ... and resumed: the data order, the schedule, the moments and the step counter continue
    resumed = ft.train(args("halves2", resume=str(first)))
    assert resumed.steps == 6
    again = ck.load_lora_checkpoint(resumed.adapter)
    for name, (shape, arr) in saved.tensors.items():
        assert np.array_equal(arr.view(np.uint32), again.tensors[name][1].view(np.uint32)), name
    a, b = (ck.TrainingCheckpoint.load(ft.state_path_for(p)).optimizer_state for p in (whole.adapter, resumed.adapter))
    assert a.t == b.t == 6.0
    for name, st in a.m_states.items():
        assert np.array_equal(np.asarray(st.data, np.float32), np.asarray(b.m_states[name].data, np.float32)), name

    # resume refuses another sequence length
    with pytest.raises(ck.CheckpointError, match="sequence_length"):
        ft.train(dataclass_replace(args("halves3", resume=str(first)), seq_len=128))


def dataclass_replace(obj, **kw):
    import dataclasses
    return dataclasses.replace(obj, **kw)


@pytest.mark.parametrize("n,world", [(1007, 2), (1007, 3), (9, 4), (3, 4)])
def test_equal_shards_close_the_same_number_of_windows(n, world):
    """Data-parallel ranks must issue the same number of collectives: with an odd dataset,
    examples the trainer would drop scattered through it, every rank still gets the same
    number of trainable examples, hence the same number of accumulation windows."""
    from ferrotensor_b200.data import TrainingExample
    from ferrotensor_b200.finetune import equal_shard, trainable_example
    rng = np.random.default_rng(n * 31 + world)
    examples = []
    for i in range(n):
        kind = rng.integers(0, 10)
        if kind == 0:      # too short
            ex = TrainingExample([i % 50], [1], [1])
        elif kind == 1:    # nothing supervised
            ex = TrainingExample([1, 2, 3], [2, 3, 4], [0, 0, 0])
        else:
            ex = TrainingExample([1, 2, 3, i % 50], [2, 3, i % 50, 5], [0, 1, 1, 1])
        examples.append(ex)
    shards = [equal_shard(examples, world, r) for r in range(world)]
    assert len({len(s) for s in shards}) == 1
    assert all(trainable_example(e) for s in shards for e in s)
    kept = [e for e in examples if trainable_example(e)]
    assert sum(len(s) for s in shards) == len(kept) // world * world
    # disjoint, round-robin over the kept examples
    for r, s in enumerate(shards):
        assert [id(e) for e in s] == [id(kept[i]) for i in range(r, len(kept) // world * world, world)]
    micro_per_step = 8
    windows = {-(-len(s) // micro_per_step) for s in shards}
    assert len(windows) == 1
