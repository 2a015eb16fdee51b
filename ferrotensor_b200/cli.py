"""`train`, `eval` and `generate` on the `cuda` device, with the reference's flags.

    python -m ferrotensor_b200.cli train    --model DIR --data train.jsonl ...   (finetune.py)
    python -m ferrotensor_b200.cli eval     --model DIR --data held_out.jsonl [--lora FILE] [--json]
    python -m ferrotensor_b200.cli generate --model DIR [--lora FILE] --prompt "..." [--json]

`eval` (ferrotensor-cli/src/main.rs:1139-1178) prints the token-weighted held-out loss and its
perplexity; `generate` (:1181-1262) streams a reply to the prompt through the KV cache and
reports prompt tokens, new tokens, prefill time and decode speed.  Both read the adapter's rank,
alpha and target projections from the metadata of the file `train` wrote.  Exit codes: 0 done,
1 failed, 2 the request cannot be met as asked.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
import time
from pathlib import Path
from typing import Dict, Optional, Tuple

import numpy as np

from .finetune import Unmet, _log, load_dataset
from .tokenizer import Tokenizer


def _adapter_from_file(path, cfg) -> Tuple["LoRaConfig", Dict[str, "torch.Tensor"]]:
    """The LoRA settings and tensors of an adapter file, under the host model's names; every
    tensor must belong to a linear of `cfg` with the right shape (checkpoint.rs:229-282)."""
    import torch
    from . import checkpoint as ck
    from .config import LINEARS, LoRaConfig
    cp = ck.load_lora_checkpoint(path)
    if cp.is_empty():
        raise Unmet(f"{path} holds no tensors")
    meta = cp.metadata
    if meta is None:
        raise Unmet(f"{path} has no LoRA metadata (rank/alpha/targets); it was not written by the train command")
    if getattr(meta, "trained_modules", None):
        raise Unmet(f"{path} holds base weights trained with --train-modules {meta.trained_modules}, not a LoRA adapter")
    lora = LoRaConfig(int(meta.rank), float(meta.alpha), tuple(meta.target_modules))
    expected = {}
    for l in range(cfg.layers):
        for name, (out, inp) in cfg.linear_shapes().items():
            if lora.targeted(name):
                pre = f"model.layers.{l}.{name}"
                expected[f"{pre}.lora_A.weight"] = [inp, lora.rank]
                expected[f"{pre}.lora_B.weight"] = [lora.rank, out]
    sources = ck.resolve_checkpoint(cp, expected)
    adapters = {ck.host_tensor_name(n): torch.from_numpy(np.ascontiguousarray(cp.tensors[key][1], dtype=np.float32))
                for n, key in sources.items()}
    return lora, adapters


def _load_base(model_dir):
    from .loader import load_model_dir
    model_dir = Path(model_dir)
    cfg, weights, raw = load_model_dir(model_dir)
    tok_path = model_dir / "tokenizer.json"
    tokenizer = Tokenizer.from_file(tok_path) if tok_path.is_file() else None
    return cfg, weights, raw, tokenizer


def run_eval(args) -> dict:
    from .config import LoRaConfig
    from .engine import CudaContext, GemmMode
    from .model import LoraModel
    from .trainer import AdamW, Trainer
    cfg, weights, _raw, tokenizer = _load_base(args.model)
    ds = load_dataset(args.data, args.task, args.seq_len, tokenizer, not args.no_chat_template, args.max_samples)
    lora, adapters = (LoRaConfig(0, 0.0, ()), None)
    if args.lora:
        lora, adapters = _adapter_from_file(args.lora, cfg)
        _log(f"lora:   {args.lora} ({len(adapters)} tensors)")
    ctx = CudaContext(args.device)
    modes = {"f16": GemmMode.F16, "f16x2": GemmMode.F16X2, "f32": GemmMode.F32}
    ctx.set_gemm_mode(GemmMode.F32 if args.f32_weights else modes[args.gemm])
    model = LoraModel(ctx, cfg, lora, weights, adapters, f16_base=not args.f32_weights)
    trainer = Trainer(model, AdamW(0.0))
    t0 = time.perf_counter()
    loss, tokens = trainer.evaluate(ds)
    seconds = time.perf_counter() - t0
    model.close()
    return {"examples": len(ds), "tokens": tokens, "loss": loss,
            "perplexity": math.exp(loss) if math.isfinite(loss) else float("nan"), "seconds": seconds}


def run_generate(args, emit) -> dict:
    from . import generate as gen
    from .engine import CudaContext, GemmMode
    if not (0.0 <= args.top_p <= 1.0) or args.temperature < 0.0:
        raise Unmet("--top-p must be in [0, 1] and --temperature >= 0")
    cfg, weights, raw, tokenizer = _load_base(args.model)
    if tokenizer is None:
        raise Unmet(f"{args.model} has no tokenizer.json")
    lora, adapters = None, None
    if args.lora:
        lora, adapters = _adapter_from_file(args.lora, cfg)
        _log(f"lora:   {args.lora} ({len(adapters)} tensors)")
    ctx = CudaContext(args.device)
    ctx.set_gemm_mode(GemmMode.F32 if args.f32_weights else GemmMode.F16)
    model = gen.InferenceModel(ctx, cfg, weights, lora, adapters, f16_base=not args.f32_weights)
    if args.raw:
        prompt = gen.Prompt.raw(tokenizer, raw, tokenizer.encode(args.prompt))
    else:
        prompt = gen.Prompt.chatml(tokenizer, raw, tokenizer.encode_chat(args.system, args.prompt))
    max_new = args.max_new_tokens
    limit = raw.get("max_position_embeddings")
    if limit is not None:
        fits = gen.new_tokens_within(int(limit), len(prompt.ids), max_new)
        if fits is None:
            raise Unmet(f"the prompt is {len(prompt.ids)} tokens, longer than the model's {limit} positions")
        if fits < max_new:
            _log(f"lowered --max-new-tokens from {max_new} to {fits} to fit the model's {limit} positions")
            max_new = fits
    sampler = gen.Sampler(args.temperature, args.top_k, args.top_p, args.seed)
    cache = gen.DecodeCache(model, len(prompt.ids) + max_new, int(limit) if limit is not None else None)
    pieces = []

    def on_text(delta: str) -> None:
        pieces.append(delta)
        emit(delta)
    decoded = gen.generate_tokens(model, prompt, max_new, sampler, cache, tokenizer.decode, on_text)
    emit("\n")
    speed = decoded.decode_tokens_per_second()
    _log(f"[{len(prompt.ids)} prompt + {decoded.new_tokens} new tokens, prefill {decoded.prefill_seconds:.2f}s, "
         f"{'no decode step' if speed is None else format(speed, '.1f') + ' tok/s'}, kv cache on]")
    return {"text": "".join(pieces), "prompt_tokens": len(prompt.ids), "new_tokens": decoded.new_tokens,
            "tokens_per_second": speed, "prefill_seconds": decoded.prefill_seconds, "kv_cache": True}


def _json_line(obj: dict) -> str:
    return json.dumps({k: (None if isinstance(v, float) and not math.isfinite(v) else v) for k, v in obj.items()})


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="python -m ferrotensor_b200.cli")
    sub = ap.add_subparsers(dest="command", required=True)
    sub.add_parser("train", aliases=["finetune"], add_help=False,
                   help="LoRA fine-tuning (flags: python -m ferrotensor_b200.finetune --help)")

    def model_flags(p):
        p.add_argument("--model", required=True, metavar="DIR")
        p.add_argument("--f32-weights", action="store_true")
        p.add_argument("--lora", default=None, metavar="FILE", help="adapter written by train")
        p.add_argument("--device", type=int, default=0)
        p.add_argument("--json", action="store_true")

    ev = sub.add_parser("eval", help="held-out loss and perplexity")
    model_flags(ev)
    ev.add_argument("--data", "--dataset", required=True, metavar="FILE")
    ev.add_argument("--task", choices=("sft", "pretrain"), default="sft")
    ev.add_argument("--seq-len", type=int, default=256)
    ev.add_argument("--max-samples", type=int, default=None)
    ev.add_argument("--no-chat-template", action="store_true")
    ev.add_argument("--gemm", choices=("f16", "f16x2", "f32"), default="f16")
    ge = sub.add_parser("generate", aliases=["infer"], help="a reply to one prompt")
    model_flags(ge)
    ge.add_argument("--prompt", default="Hello!")
    ge.add_argument("--system", default=None)
    ge.add_argument("--raw", action="store_true", help="feed the prompt to the model verbatim")
    ge.add_argument("--max-new-tokens", type=int, default=128)
    ge.add_argument("--temperature", type=float, default=0.7)
    ge.add_argument("--top-k", type=int, default=50)
    ge.add_argument("--top-p", type=float, default=0.9)
    ge.add_argument("--seed", type=int, default=None)
    return ap


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("train", "finetune"):
        from .finetune import main as train_main
        return train_main(argv[1:])
    args = _parser().parse_args(argv)
    from .checkpoint import CheckpointError
    from .loader import BuildError, LoaderError
    from .tokenizer import TokenizerError
    try:
        if args.command == "eval":
            s = run_eval(args)
            if args.json:
                print(_json_line(s))
            else:
                print(f"eval: {s['examples']} examples, {s['tokens']} tokens, loss {s['loss']:.4f}, "
                      f"perplexity {s['perplexity']:.3f} ({s['seconds']:.1f}s)")
        else:
            stream = sys.stderr if args.json else sys.stdout

            def emit(text: str) -> None:
                stream.write(text)
                stream.flush()
            s = run_generate(args, emit)
            if args.json:
                print(_json_line(s))
    except (Unmet, BuildError) as e:
        _log(f"error: {e}")
        return 2
    except (CheckpointError, LoaderError, TokenizerError, OSError) as e:
        _log(f"error: {e}")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
