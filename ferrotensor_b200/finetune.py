"""`train`: the caller of the step, from a model directory and a dataset file to a saved adapter.

The counterpart of `ferrotensor train` for LoRA on Llama-style models
(ferrotensor-cli/src/main.rs:1566-2033, flags :305-457): same flags and defaults, same dataset
formats (`load_dataset`, main.rs:988-1054), same step arithmetic (sequences per optimizer step =
batch size x grad accum, warm-up then cosine to lr/10, data order from the seed and the epoch,
resume skipping the micro-batches already seen), same files written (the adapter, its
`.state.json` and `.state.safetensors`, `training_state.json`, `metrics.jsonl`) and the same
`--json` summary.  Every float of the step is computed on the device by libft_cuda.

    python -m ferrotensor_b200.finetune --model DIR --data train.jsonl --out outputs/run

Several GPUs: launch under `python -m torch.distributed.run --nproc-per-node N`; each rank then
trains on its shard of the data (distributed.rs:222-227) and the gradients are averaged by one
NCCL all-reduce per optimizer step, where the reference exchanges them through files.

Not carried over, each an error rather than a silent difference: `--q4-weights`,
`--train-modules` other than `lora`, `--memory-report`, `--profile`.  One flag is added: `--gemm f16|f16x2|f32`, the arithmetic of
the matrix products (f16 operands with f32 accumulation on the tensor cores by default; `f32`
is the exact f32 path, which `--f32-weights` always takes).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

import numpy as np

from .data import DataLoader, TextDataset, sft_example_from_tokens, supervised_tokens
from .tokenizer import Tokenizer
from .trainer import shard_indices


class Unmet(RuntimeError):
    """A request that cannot be met as asked (exit code 2 in the reference, main.rs:107-110)."""


# ---- datasets (main.rs:988-1098) -------------------------------------------------------------
def build_sft_example(tokenizer: Tokenizer, prompt: str, response: str, system: Optional[str],
                      use_chat_template: bool, max_len: int):
    """data.rs:263-300: with the ChatML template the prompt is the chat prompt and the response
    ends with EOS, so that the model learns where to stop; the response never gets special
    tokens of its own."""
    if use_chat_template:
        response_tokens = tokenizer.encode_continuation(response) + [tokenizer.eos_token_id]
        prompt_tokens = tokenizer.encode_chat(system, prompt)
    else:
        prompt_tokens, response_tokens = tokenizer.encode(prompt), tokenizer.encode_continuation(response)
    return sft_example_from_tokens(prompt_tokens, response_tokens, max_len)


def _sft_rows(rows, where, tokenizer, chat, seq_len) -> TextDataset:
    ds = TextDataset()
    for n, row in rows:
        if not isinstance(row, dict):
            raise Unmet(f'{where}{n}: expected {{"prompt": ..., "response": ...}}')
        if "prompt_ids" in row and "response_ids" in row:
            # already tokenised text: the same length rules, no tokenizer needed
            ex = sft_example_from_tokens(list(row["prompt_ids"]), list(row["response_ids"]), seq_len)
        elif isinstance(row.get("prompt"), str) and isinstance(row.get("response"), str):
            if tokenizer is None:
                raise Unmet(f"{where}{n}: text examples need a tokenizer.json in the model directory")
            ex = build_sft_example(tokenizer, row["prompt"], row["response"], row.get("system"), chat, seq_len)
        else:
            raise Unmet(f'{where}{n}: expected {{"prompt": ..., "response": ...}}')
        if ex is not None:
            ds.add_example(ex)
    return ds


def load_dataset(path, task: str, seq_len: int, tokenizer: Optional[Tokenizer] = None,
                 chat_template: bool = True, max_samples: Optional[int] = None) -> TextDataset:
    path = Path(path)
    if not path.is_file():
        raise Unmet(f"dataset file {path} does not exist")
    if seq_len < 2:
        raise Unmet("--seq-len must be at least 2")
    ext = path.suffix.lower().lstrip(".")

    def need_tokenizer():
        if tokenizer is None:
            raise Unmet(f"{path}: text needs a tokenizer.json in the model directory")
        return tokenizer

    def lines_to_windows(lines):
        tok = need_tokenizer()
        return TextDataset.pack_sequences([tok.encode(l) for l in lines if l.strip()], seq_len)

    if task == "sft":
        if ext in ("txt", "bin"):
            raise Unmet('SFT expects .json/.jsonl with {"prompt", "response"}; use --task pretrain for .txt/.bin')
        if ext == "json":
            try:
                rows = json.loads(path.read_text())
                if not isinstance(rows, list):
                    raise ValueError("not an array")
            except ValueError as e:
                raise Unmet(f'{path}: expected a JSON array of {{"prompt", "response"}} objects: {e}') from e
            ds = _sft_rows(enumerate(rows), f"{path}: item ", tokenizer, chat_template, seq_len)
        else:
            rows = []
            for n, line in enumerate(path.read_text().splitlines(), 1):
                if not line.strip():
                    continue
                try:
                    rows.append((n, json.loads(line)))
                except ValueError as e:
                    raise Unmet(f'{path}: line {n}: expected {{"prompt": ..., "response": ...}}: {e}') from e
            ds = _sft_rows(rows, f"{path}: line ", tokenizer, chat_template, seq_len)
    elif task == "pretrain":
        if ext == "bin":
            ds = TextDataset.from_token_bin(path, seq_len)
        elif ext == "json":
            try:
                content = json.loads(path.read_text())
            except ValueError:
                content = None
            if isinstance(content, list) and all(isinstance(t, int) and not isinstance(t, bool) and 0 <= t < 2**32
                                                 for t in content):
                ds = TextDataset.from_packed_tokens(content, seq_len)
            elif isinstance(content, list) and all(isinstance(t, str) for t in content):
                ds = lines_to_windows(content)
            else:
                raise Unmet('pretrain .json must be [token ids] or ["text", ...]')
        else:
            ds = lines_to_windows(path.read_text().splitlines())
    else:
        raise Unmet(f"unknown task {task!r}")
    if max_samples is not None:
        first = TextDataset()
        for ex in ds.examples()[:max_samples]:
            first.add_example(ex)
        ds = first
    if ds.is_empty():
        raise Unmet(f"{path} produced no usable examples (empty, or every prompt is longer than --seq-len {seq_len})")
    return ds


# ---- arguments (main.rs:222-457) -------------------------------------------------------------
@dataclass
class TrainArgs:
    model: str = ""
    data: str = ""
    f32_weights: bool = False
    task: str = "sft"
    seq_len: int = 256
    max_samples: Optional[int] = None
    no_chat_template: bool = False
    out: str = "outputs/run"
    save_lora: Optional[str] = None
    resume: Optional[str] = None
    lr: float = 2e-4
    warmup_steps: int = 10
    epochs: int = 1
    max_steps: Optional[int] = None
    batch_size: int = 1
    grad_accum: int = 4
    grad_clip: float = 1.0
    weight_decay: float = 0.0
    lora_rank: int = 8
    lora_alpha: float = 16.0
    lora_targets: List[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj"])
    train_modules: str = "lora"
    log_every: int = 10
    save_every: int = 0
    eval_data: Optional[str] = None
    eval_every: int = 0
    eval_samples: int = 64
    seed: int = 0
    lite: bool = False
    json: bool = False
    sample_prompt: Optional[str] = None
    checkpoint_blocks: bool = False
    gemm: str = "f16"
    device: int = 0
    max_chunk: Optional[int] = None     # sequences per device micro-batch; None = all that fit the window
    dist_timeout: int = 600             # seconds a rank waits for its peers (the reference's max_wait)


@dataclass
class TrainSummary:
    """main.rs:1546-1563; a loss that was never measured is NaN and prints as null."""
    steps: int
    first_loss: Optional[float]
    final_loss: float
    eval_loss_before: Optional[float]
    eval_loss_after: Optional[float]
    measured_peak_mib: int
    seconds: float
    out_dir: str
    adapter: Optional[str]

    def to_json(self) -> str:
        def num(x):
            return None if x is None or (isinstance(x, float) and not math.isfinite(x)) else x
        return json.dumps({"steps": self.steps, "first_loss": num(self.first_loss), "final_loss": num(self.final_loss),
                           "eval_loss_before": num(self.eval_loss_before), "eval_loss_after": num(self.eval_loss_after),
                           "measured_peak_mib": self.measured_peak_mib, "seconds": self.seconds,
                           "out_dir": self.out_dir, "adapter": self.adapter})


def state_path_for(adapter) -> Path:
    """`x.safetensors` -> `x.safetensors.state.json`, beside it (main.rs:1537-1543)."""
    adapter = Path(adapter)
    return adapter.with_name((adapter.name or "lora_adapters.safetensors") + ".state.json")


def check_resume_file(metadata, train_modules: str) -> None:
    """A LoRA run resumes from an adapter file, never from saved base weights (main.rs:881-901)."""
    trained = getattr(metadata, "trained_modules", None) if metadata is not None else None
    if trained is not None:
        raise Unmet(f"it holds base weights trained with --train-modules {trained}, not a LoRA adapter; "
                    f"resume with --train-modules {trained}")


def _log(*parts) -> None:
    print(*parts, file=sys.stderr, flush=True)


# ---- the run (main.rs:1566-2033) -------------------------------------------------------------
def _pick_chunk(model, micro_per_step: int, seq_len: int, bucket: int) -> int:
    """Sequences per device micro-batch: the largest power of two up to the accumulation window
    whose workspace fits in 70 % of the free device memory."""
    import torch
    free, _ = torch.cuda.mem_get_info()
    padded = -(-seq_len // bucket) * bucket
    chunk = 1
    while chunk * 2 <= micro_per_step and model.workspace_bytes(chunk * 2, padded) <= 0.7 * free:
        chunk *= 2
    return chunk


def trainable_example(ex) -> bool:
    """What `Trainer.train_batch` keeps (ferrotensor-trainer/src/lib.rs:371-422): at least two
    positions and one supervised token."""
    return min(len(ex.input_ids), len(ex.target_ids)) >= 2 and any(ex.loss_mask)


def equal_shard(examples, world: int, rank: int):
    """This rank's examples for data-parallel training.  Every rank must close the same number
    of accumulation windows, since each closed window is one collective: examples the trainer
    would drop are removed BEFORE sharding (so no rank drops any later), the round-robin shards
    (distributed.rs:222-227) are cut to the common length, and with that the step count derived
    from the shard is the same on every rank."""
    kept = [ex for ex in examples if trainable_example(ex)]
    per_rank = len(kept) // world
    return [kept[i] for i in shard_indices(per_rank * world, world, rank)]


def train(args: TrainArgs) -> TrainSummary:
    import torch
    from . import checkpoint as ck
    from .config import LoRaConfig, init_adapters
    from .engine import CudaContext, GemmMode
    from .loader import load_model_dir
    from .model import LoraModel
    from .trainer import AdamW, Trainer, WarmupCosineScheduler, shard_indices

    if args.lite:                       # explicit flags win; only defaults are replaced
        if args.seq_len == 256:
            args.seq_len = 128
        if args.lora_rank == 8:
            args.lora_rank, args.lora_alpha = 4, 8.0
        if args.grad_accum == 4:
            args.grad_accum = 8
    if args.batch_size <= 0 or args.grad_accum <= 0 or args.lora_rank <= 0:
        raise Unmet("--batch-size, --grad-accum and --lora-rank must be positive")
    if args.train_modules.lower() != "lora":
        raise Unmet(f"--train-modules {args.train_modules}: only `lora` is built on this device path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    distributed = world > 1
    if distributed and args.resume is not None:
        raise Unmet("--resume is not supported with --world-size > 1 yet")
    is_root = rank == 0
    device = int(os.environ.get("LOCAL_RANK", args.device)) if distributed else args.device
    if distributed:
        import datetime
        import torch.distributed as dist
        torch.cuda.set_device(device)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", device),
                                    timeout=datetime.timedelta(seconds=args.dist_timeout))

    model_dir = Path(args.model)
    cfg, weights, _raw = load_model_dir(model_dir)
    tok_path = model_dir / "tokenizer.json"
    tokenizer = Tokenizer.from_file(tok_path) if tok_path.is_file() else None
    pad_id = tokenizer.pad_token_id if tokenizer is not None else 0
    chat = not args.no_chat_template
    dataset = load_dataset(args.data, args.task, args.seq_len, tokenizer, chat, args.max_samples)
    eval_ds = None
    if args.eval_data is not None:
        eval_ds = load_dataset(args.eval_data, args.task, args.seq_len, tokenizer, chat, args.eval_samples)
    for ds in (dataset, eval_ds):
        for ex in (ds.examples() if ds is not None else ()):
            if max(max(ex.input_ids), max(ex.target_ids)) >= cfg.vocab:
                raise Unmet(f"a token id in the data is not below the model's vocabulary size {cfg.vocab}")

    lora = LoRaConfig(args.lora_rank, args.lora_alpha, tuple(args.lora_targets))
    meta = ck.LoraMetadata(args.lora_rank, args.lora_alpha, list(args.lora_targets))
    ctx = CudaContext(device)
    modes = {"f16": GemmMode.F16, "f16x2": GemmMode.F16X2, "f32": GemmMode.F32}
    if args.gemm not in modes:
        raise Unmet(f"--gemm {args.gemm}: one of f16, f16x2, f32")
    ctx.set_gemm_mode(GemmMode.F32 if args.f32_weights else modes[args.gemm])
    adapters = init_adapters(cfg, lora, args.seed)
    model = LoraModel(ctx, cfg, lora, weights, adapters, f16_base=not args.f32_weights,
                      checkpoint_blocks=args.checkpoint_blocks)
    if args.checkpoint_blocks:
        _log("block checkpointing: on")
    if args.sample_prompt is None:
        del weights
    elif tokenizer is None:
        raise Unmet("--sample-prompt needs a tokenizer.json in the model directory")
    n_params = sum(t.numel() for t in model.named_lora_params().values())
    if n_params == 0:
        raise Unmet(f"--lora-targets {','.join(args.lora_targets)} matches no linear of the model")

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    adapter_path = Path(args.save_lora) if args.save_lora else out_dir / "lora_adapters.safetensors"
    state_path = state_path_for(adapter_path)

    if distributed:                     # each rank trains on a disjoint slice of equal length
        shard = TextDataset()
        for ex in equal_shard(dataset.examples(), world, rank):
            shard.add_example(ex)
        dataset = shard

    micro_per_step = args.batch_size * args.grad_accum
    steps_per_epoch = max(-(-len(dataset) // micro_per_step), 1)
    total_steps = max(args.max_steps if args.max_steps is not None else steps_per_epoch * max(args.epochs, 1), 1)
    warmup = min(args.warmup_steps, max(total_steps - 1, 0))

    optimizer = AdamW(args.lr, weight_decay=args.weight_decay)
    scheduler = WarmupCosineScheduler(args.lr, args.lr * 0.1, warmup, total_steps)
    trainer = (Trainer(model, optimizer).with_grad_accum_steps(micro_per_step)
               .with_clip_grad_norm(args.grad_clip).with_lr_scheduler(scheduler))
    trainer.max_chunk = args.max_chunk or _pick_chunk(model, micro_per_step, args.seq_len, trainer.length_bucket)
    if distributed:
        from .distributed import Communicator
        trainer.with_distributed(world, rank, Communicator.from_torch_distributed(
            ctx, max_wait_s=float(args.dist_timeout)))

    start_step = 0
    if args.resume is not None:
        resume = Path(args.resume)
        cp = ck.load_lora_checkpoint(resume)
        if cp.is_empty():
            raise Unmet(f"{resume} holds no tensors")
        try:
            check_resume_file(cp.metadata, args.train_modules)
        except Unmet as e:
            raise Unmet(f"{resume}: {e}") from e
        n = trainer.load_adapter(resume)
        resume_state = state_path_for(resume)
        if resume_state.is_file():
            ts = ck.TrainingCheckpoint.load(resume_state).training_state
            ts.validate_resume(args.train_modules, args.task, args.seq_len, str(args.model))
            trainer.load_training_checkpoint(resume_state)
            start_step, args.seed = ts.step, ts.seed
            trainer.set_optimizer_steps(start_step)
        _log(f"resume: {resume} ({n} tensors), continuing at step {start_step}")
    trainer.dropout_seed = args.seed     # attention-dropout masks follow the run seed (restored on resume)

    _log(f"data:   {len(dataset)} examples ({args.task} task), {supervised_tokens(dataset)} supervised tokens, "
         f"seq-len {args.seq_len}")
    _log(f"train:  lora ({n_params} trainable params), lr {args.lr} warmup {warmup} cosine, "
         f"{total_steps} steps x {micro_per_step} sequences")

    metrics = open(out_dir / "metrics.jsonl", "a") if is_root else open(os.devnull, "w")

    def metric(obj) -> None:
        metrics.write(json.dumps(obj) + "\n")
        metrics.flush()

    def evaluate(label: str, step: int) -> Optional[float]:
        if eval_ds is None:
            return None
        loss, tokens = trainer.evaluate(eval_ds, args.eval_samples)
        _log(f"eval {label}: loss {loss:.4f} ppl {math.exp(loss) if math.isfinite(loss) else float('nan'):.3f} "
             f"({tokens} tokens)")
        metric({"step": step, "eval_loss": None if not math.isfinite(loss) else loss})
        return loss

    eval_before = evaluate("before", start_step)

    def save(step: int, best: Optional[float]) -> None:
        if not is_root:
            return
        trainer.save_adapter(adapter_path)
        state = ck.TrainingState(
            step=step, total_steps=total_steps, best_loss=best, lr=args.lr, epoch=step // steps_per_epoch,
            batch_size=args.batch_size, grad_accum_steps=args.grad_accum, sequence_length=args.seq_len, fp16=False,
            train_modules=args.train_modules, task=args.task, model_path=str(args.model), dataset_path=str(args.data),
            seed=args.seed)
        state.save(out_dir / "training_state.json")
        trainer.save_training_checkpoint(state_path, state)

    _log("  step |   loss | grad norm |       lr | tok/s | s/step")
    loader = DataLoader(dataset, args.batch_size, not distributed, pad_id).with_seed(args.seed)
    step = start_step
    skip_micro, micro_seen = start_step * micro_per_step, 0
    win_loss, win_tok, win_seq = 0.0, 0, 0
    win_start = run_start = time.perf_counter()
    best: Optional[float] = None
    first_loss: Optional[float] = None
    last_loss, last_norm, last_lr = float("nan"), 0.0, 0.0
    epoch, done = 0, False
    while not done and step < total_steps:       # a resume at or past the last step only saves
        loader.set_epoch(epoch)
        loader.reset()
        any_batch = False
        for batch in loader:
            any_batch = True
            if micro_seen < skip_micro:
                micro_seen += batch.batch_size
                continue
            micro_seen += batch.batch_size
            for s in trainer.train_batch(batch):
                win_loss += float(s.loss) * s.tokens
                win_tok += s.tokens
                win_seq += 1
                if s.grad_norm is not None:
                    last_norm = s.grad_norm
                if s.lr is not None:
                    last_lr = s.lr
                if not s.optimizer_step:
                    continue
                step += 1
                if step % max(args.log_every, 1) == 0 or step == total_steps:
                    loss = float(np.float32(win_loss / max(win_tok, 1)))
                    secs = time.perf_counter() - win_start
                    steps_in_win = win_seq / micro_per_step
                    _log(f"{step:6d} | {loss:6.4f} | {last_norm:9.3f} | {last_lr:8.2e} | "
                         f"{win_tok / max(secs, 1e-6):5.0f} | {secs / max(steps_in_win, 1e-6):6.2f}")
                    metric({"step": step, "loss": loss, "grad_norm": last_norm, "lr": last_lr, "tokens": win_tok,
                            "seconds": secs, "elapsed": time.perf_counter() - run_start})
                    if first_loss is None:
                        first_loss = loss
                    last_loss = loss
                    best = loss if best is None else min(best, loss)
                    win_loss, win_tok, win_seq = 0.0, 0, 0
                    win_start = time.perf_counter()
                if args.save_every > 0 and step % args.save_every == 0 and step < total_steps:
                    save(step, best)
                if eval_ds is not None and args.eval_every > 0 and step % args.eval_every == 0 and step < total_steps:
                    evaluate(f"@ {step}", step)
                if step >= total_steps:
                    done = True
                    break
            if done:
                break
        if not any_batch or (epoch + 1 >= max(args.epochs, 1) and args.max_steps is None):
            break
        epoch += 1

    ctx.synchronize()
    elapsed = time.perf_counter() - run_start
    save(step, best)
    _log(f"done:   {step} steps in {elapsed:.1f}s; train loss "
         f"{'n/a' if first_loss is None else format(first_loss, '.4f')} -> {last_loss:.4f}")
    if is_root:
        _log(f"saved:  {adapter_path} (+ {state_path})")
        _log(f"metrics: {out_dir / 'metrics.jsonl'}")
    eval_after = evaluate("after", step)
    metrics.close()
    if args.sample_prompt is not None:
        # a quick sanity check: a greedy reply of up to 96 tokens to the prompt in the ChatML template
        from . import generate as gen
        adapters_now = {n: t.detach().clone() for n, t in model.named_lora_params().items()}
        infer = gen.InferenceModel(ctx, cfg, weights, lora, adapters_now, f16_base=not args.f32_weights)
        prompt = gen.Prompt.chatml(tokenizer, _raw, tokenizer.encode_chat(None, args.sample_prompt))
        _log(f"sample ({args.sample_prompt!r}):")
        out_stream = sys.stderr if args.json else sys.stdout

        def emit(text: str) -> None:
            out_stream.write(text)
            out_stream.flush()
        gen.generate_tokens(infer, prompt, 96, gen.Sampler(0.0, 0, 1.0), gen.DecodeCache(infer, len(prompt.ids) + 96),
                            tokenizer.decode, emit)
        emit("\n")
    peak_mib = -(-torch.cuda.max_memory_allocated(device) // (1 << 20))
    model.close()
    return TrainSummary(step, first_loss, last_loss, eval_before, eval_after, int(peak_mib), elapsed, str(out_dir),
                        str(adapter_path) if is_root else None)


# ---- command line ----------------------------------------------------------------------------
def parse_args(argv=None) -> TrainArgs:
    d = TrainArgs()
    ap = argparse.ArgumentParser(prog="python -m ferrotensor_b200.finetune",
                                 description="LoRA fine-tuning of a Llama-style model directory on one or more B200s")
    ap.add_argument("--model", required=True, metavar="DIR", help="model directory (config.json, *.safetensors, "
                    "tokenizer.json when the data is text)")
    ap.add_argument("--f32-weights", action="store_true", help="store frozen base weights as f32 instead of f16")
    ap.add_argument("--data", "--dataset", required=True, metavar="FILE", help="dataset file (see --task)")
    ap.add_argument("--task", choices=("sft", "pretrain"), default=d.task)
    ap.add_argument("--seq-len", type=int, default=d.seq_len, help="maximum tokens per example")
    ap.add_argument("--max-samples", type=int, default=None, help="use only the first N examples")
    ap.add_argument("--no-chat-template", action="store_true", help="do not wrap SFT prompts in ChatML")
    ap.add_argument("--out", default=d.out, metavar="DIR")
    ap.add_argument("--save-lora", default=None, metavar="FILE")
    ap.add_argument("--resume", default=None, metavar="FILE")
    ap.add_argument("--lr", type=float, default=d.lr)
    ap.add_argument("--warmup-steps", type=int, default=d.warmup_steps)
    ap.add_argument("--epochs", type=int, default=d.epochs)
    ap.add_argument("--max-steps", type=int, default=None)
    ap.add_argument("--batch-size", type=int, default=d.batch_size)
    ap.add_argument("--grad-accum", type=int, default=d.grad_accum)
    ap.add_argument("--grad-clip", type=float, default=d.grad_clip)
    ap.add_argument("--weight-decay", type=float, default=d.weight_decay)
    ap.add_argument("--lora-rank", type=int, default=d.lora_rank)
    ap.add_argument("--lora-alpha", type=float, default=d.lora_alpha)
    ap.add_argument("--lora-targets", default=",".join(d.lora_targets),
                    help="comma-separated projections that get adapters")
    ap.add_argument("--train-modules", default=d.train_modules)
    ap.add_argument("--log-every", type=int, default=d.log_every)
    ap.add_argument("--save-every", type=int, default=d.save_every)
    ap.add_argument("--eval-data", default=None, metavar="FILE")
    ap.add_argument("--eval-every", type=int, default=d.eval_every)
    ap.add_argument("--eval-samples", type=int, default=d.eval_samples)
    ap.add_argument("--seed", type=int, default=d.seed)
    ap.add_argument("--sample-prompt", default=None, help="generate from this prompt after training")
    ap.add_argument("--lite", action="store_true", help="seq-len 128, rank 4, grad-accum 8 unless set")
    ap.add_argument("--checkpoint-blocks", action="store_true",
                    help="recompute each decoder block during backward instead of keeping its activations")
    ap.add_argument("--gemm", choices=("f16", "f16x2", "f32"), default=d.gemm)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--max-chunk", type=int, default=None, help="sequences per device micro-batch")
    ap.add_argument("--dist-timeout", type=int, default=d.dist_timeout,
                    help="seconds a rank waits for its peers before it fails")
    ap.add_argument("--json", action="store_true", help="print one JSON summary to stdout when the run ends")
    ns = ap.parse_args(argv)
    kw = vars(ns)
    kw["lora_targets"] = [t.strip() for t in ns.lora_targets.split(",") if t.strip()]
    return TrainArgs(**kw)


def main(argv=None) -> int:
    """Exit codes as the reference's (main.rs:599-640): 0 done, 1 failed, 2 cannot be met as asked."""
    args = parse_args(argv)
    from .checkpoint import CheckpointError
    from .loader import BuildError, LoaderError
    from .tokenizer import TokenizerError
    try:
        summary = train(args)
    except (Unmet, BuildError) as e:
        _log(f"error: {e}")
        return 2
    except (CheckpointError, LoaderError, TokenizerError, OSError) as e:
        _log(f"error: {e}")
        return 1
    if args.json:
        print(summary.to_json())
    return 0


if __name__ == "__main__":
    sys.exit(main())
