#!/usr/bin/env python3
"""Benchmark of the LoRA fine-tuning step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--micro-batch B]
    python bench.py --impl reference ...      # the reference's CPU restatement on host cores

One "step" is one optimizer step over the workload's global batch: forward, masked CE,
backward over every micro-batch, gradient mean over ranks (NCCL), global norm, clipping,
AdamW.  Prints ONE JSON line (rank 0).  `value` times the step with its inputs already in
HBM; `e2e` times the same step through `Trainer.train_arrays` with host arrays (pinned
host -> device copies of ids/targets/weights and the read-back of the row losses and the
gradient norm inside the timed region).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "lora_step_tokens_per_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["cuda", "reference"], default="cuda")
    ap.add_argument("--workload", default="smollm2-1.7b")
    ap.add_argument("--micro-batch", type=int, default=8, help="sequences per micro-batch")
    ap.add_argument("--mode", choices=["f16", "f16x2", "f32"], default="f16")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="override the workload's global batch (profiling of a reduced case; "
                         "the line then says so in config and is not the headline)")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: device-timed loop only")
    ap.add_argument("--cpu-sample-tokens", type=int, default=0)
    ap.add_argument("--kernel-times", action="store_true",
                    help="time every launch of one extra step by kernel name (CUDA events) and "
                         "add the table to the JSON line as kernel_ms")
    return ap.parse_args()


PARITY_RULES = {
    "f16": "|err| <= 5e-3*max|e| + 2e-2*|e| and relative L2 <= 8e-3 per tensor against the f32 CPU "
           "oracle (f16 tensor-core operands, f32 accumulation)",
    "f16x2": "1e-4 + 1e-3*|e| against the f32 CPU oracle (the reference's own rule; operands "
             "split into two f16 halves)",
    "f32": "1e-4 + 1e-3*|e| against the f32 CPU oracle (the reference's own rule; f32 FMA)",
}


def workload_config(w, world, micro_batch, mode, reduced):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": w.name, "global_batch": w.global_batch, "seq_len": w.seq_len,
            "micro_batch_sequences": micro_batch, "parallelism": f"dp{world}",
            "lora_rank": w.lora.rank, "checkpoint_blocks": w.checkpoint_blocks,
            "reduced_case": reduced,
            "l2": "inputs larger than L2 (weights and activations of one step exceed 126 MB)",
            "gemm_operands": "f16 activations x f16 weights, f32 accumulate" if mode != "f32" else "f32",
            "parity_rule": PARITY_RULES[mode]}


def resolve_mode(args, w):
    return args.mode if w.f16_base else "f32"


def local_micro_batch(args, w, world):
    return max(1, min(args.micro_batch, w.global_batch // world))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d.get("hbm_gbs"), "tflops": d.get("bf16_tflops_sustained"),
                "tflops_burst": d.get("bf16_tflops"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1400.0, "tflops_burst": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                clocks.append(float(f[1]))
                maxes.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = sorted(c for c in clocks if c > 0.5 * max(clocks)) or sorted(clocks)
        return {"sm_mhz": busy[len(busy) // 2], "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
                "samples": len(clocks)}


# ---------------------------------------------------------------------------------------
# the reference's CPU restatement, timed on the host cores
# ---------------------------------------------------------------------------------------

def cpu_step_tokens_per_s(workload, weights_cpu, adapters_cpu, sample_tokens, repeats=1, warmup=0,
                          budget_s=150.0):
    """One sequence of `sample_tokens` positions of the workload through the CPU oracle
    (forward, loss, autograd backward, clip, AdamW), all host threads.  At most `repeats`
    timed steps; after three, no further step starts once `budget_s` seconds of timed work
    have passed (a slow host must still finish within minutes).  Returns
    (tokens/s, cores, median seconds per step, steps timed)."""
    import numpy as np
    import torch
    from ferrotensor_b200.config import head_weight, synthetic_batch
    from oracle import lora_step as ol
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = workload
    c = w.model
    ocfg = ol.OracleConfig(vocab=c.vocab, hidden=c.hidden, layers=c.layers, heads=c.heads,
                           kv_heads=c.kv_heads, ffn=c.ffn, eps=c.eps, theta=c.theta,
                           head_dim=c.head_dim, tied=c.tied, qkv_bias=c.qkv_bias,
                           lora_rank=w.lora.rank, lora_alpha=w.lora.alpha,
                           lora_targets=tuple(w.lora.target_modules), f16_base=w.f16_base)
    p = dict(weights_cpu)
    p.update(adapters_cpu)
    p["lm_head.weight"] = head_weight(c, weights_cpu, w.f16_base)
    ids, tg, mk = synthetic_batch(w, 1)
    ids, tg, mk = ids[:, :sample_tokens], tg[:, :sample_tokens], mk[:, :sample_tokens]
    if not mk.any():
        mk[:, -1] = 1
    hp = ol.AdamParams(lr=w.lr, weight_decay=w.weight_decay)
    state = {}
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        ol.lora_step(ocfg, p, [[(ids.astype(np.int64), tg.astype(np.int64), mk)]], hp, state,
                     clip_grad_norm=w.clip)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
            if len(times) >= 3 and sum(times) > budget_s:
                break
    n_timed = len(times)
    times.sort()
    sec = times[len(times) // 2]
    return sample_tokens / sec, cores, sec, n_timed


def default_cpu_sample(workload):
    """Positions of the one sequence the CPU leg steps through: the whole sequence, capped at
    1024 positions (a 4096-position sequence of the oracle keeps every layer's [heads, S, S]
    score matrix for its backward pass, tens of GB).  The same on every box."""
    return min(workload.seq_len, 1024)


def run_reference(args):
    """`--impl reference`: the reference's own CPU statement of the step (the PyTorch model of
    its gradient-fixture generator, parametrised to the workload), on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights
    import copy
    w = copy.deepcopy(WORKLOADS[args.workload])
    reduced = bool(args.global_batch) and args.global_batch != w.global_batch
    if args.global_batch:
        w.global_batch = args.global_batch
    world = max(1, args.gpus)
    sample = args.cpu_sample_tokens or default_cpu_sample(w)
    weights = init_weights(w.model, w.seed, device="cpu", f16_base=w.f16_base)
    adapters = init_adapters(w.model, w.lora, w.seed, device="cpu", b_std=w.adapter_b_std)
    tps, cores, sec, n_timed = cpu_step_tokens_per_s(w, weights, adapters, sample, repeats=args.steps,
                                                     warmup=1)
    desc = (f"one sequence of {sample} of {w.seq_len} positions per step, median of {n_timed} "
            f"steps after one warm-up step (no further step starts after 150 s of timed work); "
            f"tokens/s of the sample (a full {w.global_batch}x{w.seq_len} step is that many "
            f"sequences, extrapolated linearly)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(w, world, local_micro_batch(args, w, world), resolve_mode(args, w),
                                  reduced),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc,
                         "steps_timed": n_timed},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------
# the CUDA arm
# ---------------------------------------------------------------------------------------

def run_cuda(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from ferrotensor_b200.config import (WORKLOADS, gemm_flops, init_adapters, init_weights,
                                         step_flops, synthetic_batch)
    from ferrotensor_b200.distributed import Communicator
    from ferrotensor_b200.engine import CudaContext, GemmMode
    from ferrotensor_b200.model import LoraModel
    from ferrotensor_b200.trainer import AdamW, Trainer, batch_targets_weights, shard_indices

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with: python -m torch.distributed.run "
                             "--nproc-per-node N bench.py --gpus N ...")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import copy
    w = copy.deepcopy(WORKLOADS[args.workload])
    reduced = bool(args.global_batch) and args.global_batch != w.global_batch
    if args.global_batch:
        w.global_batch = args.global_batch
    assert w.global_batch % world == 0, "global batch must divide over the ranks"
    ctx = CudaContext(local)
    mode_name = resolve_mode(args, w)
    mode = {"f16": GemmMode.F16, "f16x2": GemmMode.F16X2, "f32": GemmMode.F32}[mode_name]
    ctx.set_gemm_mode(mode)
    # the gradient exchange runs inside the library (NCCL on the context's stream);
    # torch.distributed only carries the communicator id, the barriers and the max over ranks
    comm = Communicator.from_torch_distributed(ctx, max_wait_s=120.0) if world > 1 else None

    weights = init_weights(w.model, w.seed, device=f"cuda:{local}", f16_base=w.f16_base)
    adapters = init_adapters(w.model, w.lora, w.seed, device=f"cuda:{local}", b_std=w.adapter_b_std)
    model = LoraModel(ctx, w.model, w.lora, weights, adapters, f16_base=w.f16_base,
                      checkpoint_blocks=w.checkpoint_blocks)
    want_cpu = rank == 0 and world == 1 and not args.no_cpu_baseline
    weights_cpu = adapters_cpu = None
    if want_cpu:
        weights_cpu = {k: v.cpu() for k, v in weights.items()}
        adapters_cpu = {k: v.cpu() for k, v in adapters.items()}
    del weights, adapters
    torch.cuda.empty_cache()

    # this rank's sequences (round-robin over the global batch, as the reference shards)
    ids, tg, mk = synthetic_batch(w, w.global_batch)
    mine = shard_indices(w.global_batch, world, rank)
    ids, tg, mk = ids[mine], tg[mine], mk[mine]
    n_local = len(mine)
    mb = local_micro_batch(args, w, world)
    tokens_per_step = w.global_batch * w.seq_len

    trainer = Trainer(model, AdamW(w.lr, weight_decay=w.weight_decay)) \
        .with_grad_accum_steps(n_local).with_clip_grad_norm(w.clip)
    if world > 1:
        trainer.with_distributed(world, rank, comm)
    trainer.max_chunk = mb

    # ---- device-resident form of one step --------------------------------------------------
    dev = ctx.device
    resident = []
    for r0 in range(0, n_local, mb):
        i, t, m = ids[r0:r0 + mb], tg[r0:r0 + mb], mk[r0:r0 + mb]
        rt, rw, tok = batch_targets_weights(t, m, w.model.vocab)
        resident.append((
            torch.from_numpy(np.ascontiguousarray(i).view(np.int32).reshape(-1)).to(dev),
            torch.from_numpy(rt.view(np.int32).reshape(-1)).to(dev),
            torch.from_numpy(rw.reshape(-1)).to(dev),
            torch.empty(i.size, device=dev, dtype=torch.float32), i.shape[0],
            torch.from_numpy(np.maximum(tok, 1).astype(np.float32)).to(dev)))
    # self-check of the first timed step, kept on the device until the timed region is over:
    # [sum over this rank's sequences of the sequence loss, pre-clip gradient norm, applied flag]
    check_dev = torch.zeros(3, device=dev, dtype=torch.float64)

    def resident_step(capture=False):
        model.zero_grad()
        for d_ids, d_tg, d_w, row_loss, n, d_tok in resident:
            model.forward_backward(d_ids, d_tg, d_w, n, w.seq_len, 1.0 / n_local, row_loss)
            if capture:
                check_dev[0] += (row_loss.view(n, -1).sum(dim=1) / d_tok).sum().double()
        trainer.optimizer.t += 1.0
        model.allreduce_apply_gradients(comm, w.clip, trainer.optimizer.params())
        if capture:
            check_dev[1:3] = model.norm_out[:2].double()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, first=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(steps):
            (first if first is not None and k == 0 else fn)()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        resident_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count()
    ms_total = timed(resident_step, args.steps, first=lambda: resident_step(True))
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps
    value = tokens_per_step / (ms_step * 1e-3)

    # ---- the step checks itself: loss and pre-clip norm of the first timed step, and whether
    # every rank holds the same parameters after the last one -----------------------------------
    chk = check_dev.clone()
    words = model.params.view(torch.int32).to(torch.int64)
    fingerprint = torch.stack([words.sum(), (words * (torch.arange(words.numel(), device=dev) % 8191 + 1)).sum()])
    fp_min, fp_max = fingerprint.clone(), fingerprint.clone()
    if world > 1:
        dist.all_reduce(chk[0:1], op=dist.ReduceOp.SUM)
        dist.all_reduce(fp_min, op=dist.ReduceOp.MIN)
        dist.all_reduce(fp_max, op=dist.ReduceOp.MAX)
    check = {"loss_step1": float(chk[0].item()) / w.global_batch,
             "grad_norm_step1": float(chk[1].item()),
             "update_applied_step1": bool(chk[2].item() != 0.0),
             "params_equal_across_ranks": bool(torch.equal(fp_min, fp_max)),
             "params_fingerprint": [int(v) for v in fingerprint.tolist()],
             "what": "mean sequence loss and pre-clip global gradient norm of the first timed "
                     "step (after the warm-up steps' updates); two integer checksums of the "
                     "parameter bits after the last step, min == max over ranks"}

    # ---- roofline of the dominant kernel: the tensor-core GEMM, timed inside a step ------------
    ctx.profile(True)
    resident_step()
    ctx.synchronize()
    gemm_bytes = ctx.profile_bytes()
    fused_ms, fused_flops, fused_launches = ctx.profile_read_fused()
    gemm_ms, gemm_flops_done, gemm_launches = ctx.profile_read()
    ctx.profile(False)
    # DRAM traffic per launch: the launches' algorithmic bytes (operands once, results once) times
    # the ratio dram bytes / algorithmic bytes that one ncu capture of the 8192 x 8192 x 2048
    # launch gave (344 MB / 335 MB); the full step is too large to capture with all metrics
    traffic = gemm_bytes / gemm_launches * (344.0 / 335.0) if gemm_launches else None

    kernel_ms = None
    if args.kernel_times:
        ctx.profile(2)
        resident_step()
        rep = ctx.profile_report()
        ctx.profile(0)
        kernel_ms = {k: {"launches": n, "ms": round(ms, 3)}
                     for k, (n, ms) in sorted(rep.items(), key=lambda kv: -kv[1][1])}

    # ---- end to end through the trainer with host inputs ---------------------------------------
    def e2e_step():
        trainer.train_arrays(ids, tg, mk)

    if args.skip_e2e:
        ms_e2e, e2e_value, h2d, d2h = None, None, 0, 0
    else:
        e2e_step()
        trainer.h2d_bytes = trainer.d2h_bytes = 0
        ms_e2e = timed(e2e_step, args.steps) / args.steps
        e2e_value = tokens_per_step / (ms_e2e * 1e-3)
        h2d = trainer.h2d_bytes // args.steps
        d2h = trainer.d2h_bytes // args.steps
    ctx.synchronize()

    if rank != 0:
        if comm is not None:
            comm.close()
        if world > 1:
            dist.destroy_process_group()
        return
    peaks = measured_peaks()
    executed = gemm_flops_done / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    # algorithmic FLOPs of this rank's share of the step's dense contractions (frozen projections
    # and head forward + input gradient, adapters forward + two gradients)
    gemm_alg = gemm_flops(w, tokens_per_step) / world
    achieved = gemm_alg / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    flops_step = step_flops(w, tokens_per_step)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": mode_name,
        "data": "synthetic",
        "config": workload_config(w, world, mb, mode_name, reduced),
        "check": check,
        "step_roofline": {"algorithmic_tflop_per_step": flops_step / 1e12,
                          "achieved_tflops": flops_step / (ms_step * 1e-3) / 1e12 / world,
                          "peak_tflops": peaks["tflops"],
                          "frac": flops_step / (ms_step * 1e-3) / 1e12 / world / peaks["tflops"],
                          "peak_source": peaks["source"]},
        "roofline": {"bound": "tensor", "kernel": "k_gemm_tc (tcgen05 f16)", "achieved": achieved,
                     "achieved_executed": executed,
                     "flops": "achieved = algorithmic FLOPs (2MNK of the frozen projections and "
                              "the rank-r adapter products) / summed launch time; "
                              "achieved_executed counts what the launches ran (adapter tail "
                              "padded to 64 columns, pre-tiles, checkpoint replays)",
                     "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["tflops"] if peaks["tflops"] else None,
                     "traffic": traffic, "traffic_unit": "bytes per launch: the launches' algorithmic bytes x 1.027, an estimate "
                                     "(ncu gave dram/algorithmic ratios of 1.04, 1.34 and 0.69 on "
                                     "the three captured shapes, profiles/k_gemm_tc_ncu_full.md)",
                     "peak_source": peaks["source"] + " (sustained)",
                     "launches_per_step": gemm_launches, "kernel_ms_per_step": gemm_ms,
                     # some launches also do elementwise work of the step in their epilogues
                     # (RoPE of q|k|v, SwiGLU forward, SwiGLU backward): their time contains what
                     # used to be separate HBM-bound kernels, so the two groups are also given apart
                     "fused_epilogue_launches": {
                         "launches_per_step": fused_launches, "kernel_ms_per_step": fused_ms,
                         "executed_tflops": fused_flops / (fused_ms * 1e-3) / 1e12 if fused_ms > 0 else None,
                         "what": "q|k|v projection + RoPE + f16 rounding; gate|up projection + "
                                 "SwiGLU; down projection's input gradient + SwiGLU backward"},
                     "plain_launches": {
                         "launches_per_step": gemm_launches - fused_launches,
                         "kernel_ms_per_step": gemm_ms - fused_ms,
                         "executed_tflops": (gemm_flops_done - fused_flops) / ((gemm_ms - fused_ms) * 1e-3) / 1e12
                         if gemm_ms > fused_ms else None}},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if kernel_ms is not None:
        out["kernel_ms"] = kernel_ms
    if want_cpu:
        sample = args.cpu_sample_tokens or default_cpu_sample(w)
        tps, cores, sec, _ = cpu_step_tokens_per_s(w, weights_cpu, adapters_cpu, sample, repeats=3,
                                                   warmup=1)
        out["cpu_baseline"] = {
            "value": tps, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one sequence of {sample} of {w.seq_len} positions per step, median of 3 "
                      f"steps after one warm-up step ({sec:.1f} s per step); a full step is "
                      f"extrapolated linearly"}
    print(json.dumps(out))
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
