"""Kernel micro-benchmarks through the public engine calls, at shapes chosen on the command line.

    python -m ferrotensor_b200.microbench gemm --m 8192 --n 8192 --k 2048
    python -m ferrotensor_b200.microbench attention --batch 8 --seq 1024 --heads 32 --kv-heads 32
    python -m ferrotensor_b200.microbench matvec --k 2048 --n 8192
    python -m ferrotensor_b200.microbench decode --batch 8 --seq 4096
    python -m ferrotensor_b200.microbench sustained --seconds 4       # GEMM under the power cap, beside cuBLAS
    python -m ferrotensor_b200.microbench step --layers 2             # one micro-batch of a cut-down benchmark model

Each case holds a few hundred MB on the device at most, which makes it the right target for a
profiler capture of one kernel (the training step keeps tens of GB resident).  Times come from
the library's per-kernel CUDA-event profiler, one line per kernel name.
"""

from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from .engine import AttentionOptions, ComputeEngine, CudaContext, DType, GemmMode, UnifiedTensor


def _dev_f32(ctx, shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = torch.randn(int(np.prod(shape)), device="cuda", generator=g) * scale
    return UnifiedTensor(t.view(torch.uint8), list(shape), DType.F32)


def _report(ctx, what, extra):
    rep = ctx.profile_report()
    ctx.profile(0)
    out = {"case": what, **extra, "kernels": {}}
    for name, (launches, ms) in rep.items():
        out["kernels"][name] = {"launches": launches, "ms_per_launch": ms / max(launches, 1)}
    print(json.dumps(out))
    return out


def gemm(args):
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    ctx.set_gemm_mode(GemmMode.F16)
    a = _dev_f32(ctx, [args.m, args.k], 1.0, 1)
    g = torch.Generator(device="cuda").manual_seed(2)
    b = UnifiedTensor((torch.randn(args.n * args.k, device="cuda", generator=g) * 0.05).half()
                      .view(torch.uint8), [args.n, args.k], DType.FP16)
    out = UnifiedTensor.empty(ctx, [args.m, args.n])
    for _ in range(args.warmup):
        eng.matmul_bt_f16b(ctx, a, b, out)
    ctx.profile(2)
    for _ in range(args.iters):
        eng.matmul_bt_f16b(ctx, a, b, out)
    ctx.synchronize()
    rep = _report(ctx, "gemm", {"m": args.m, "n": args.n, "k": args.k})
    for name, v in rep["kernels"].items():
        if name.startswith("k_gemm_tc"):
            tf = 2.0 * args.m * args.n * args.k / (v["ms_per_launch"] * 1e-3) / 1e12
            print(f"{name}: {v['ms_per_launch'] * 1e3:.1f} us, {tf:.0f} TFLOP/s")


def attention(args):
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    ctx.set_gemm_mode(GemmMode.F16)
    b, s, h, hk, d = args.batch, args.seq, args.heads, args.kv_heads, 64
    q = _dev_f32(ctx, [b, s, h, d], 1.0, 1)
    k = _dev_f32(ctx, [b, s, hk, d], 1.0, 2)
    v = _dev_f32(ctx, [b, s, hk, d], 1.0, 3)
    go = _dev_f32(ctx, [b, s, h, d], 1e-3, 4)
    out = UnifiedTensor.empty(ctx, [b, s, h, d])
    stats = UnifiedTensor.empty(ctx, [b * h * s * 2])
    gq = UnifiedTensor.empty(ctx, [b, s, h, d])
    gk = UnifiedTensor.empty(ctx, [b, s, hk, d])
    gv = UnifiedTensor.empty(ctx, [b, s, hk, d])
    opts = AttentionOptions(causal=True)

    def once():
        eng.flash_attention_v2_with_stats(ctx, q, k, v, out, stats, opts)
        if not args.forward_only:
            eng.flash_attention_v2_backward_with_stats(ctx, q, k, v, out, go, gq, gk, gv, stats, opts)

    for _ in range(args.warmup):
        once()
    ctx.profile(2)
    for _ in range(args.iters):
        once()
    ctx.synchronize()
    rep = _report(ctx, "attention", {"batch": b, "seq": s, "heads": h, "kv_heads": hk})
    fwd_flop = 4.0 * b * h * s * s * d / 2          # causal: half of the score matrix
    for name, mult in (("k_attn_fwd_tc", 1.0), ("k_attn_bwd_dq_tc2", 1.5), ("k_attn_bwd_dkv_tc2", 2.0)):
        if name in rep["kernels"]:
            ms = rep["kernels"][name]["ms_per_launch"]
            print(f"{name}: {ms * 1e3:.1f} us, {fwd_flop * mult / (ms * 1e-3) / 1e12:.0f} TFLOP/s")


def matvec(args):
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    k, n = args.k, args.n
    x = _dev_f32(ctx, [1, k], 1.0, 1)
    g = torch.Generator(device="cuda").manual_seed(2)
    # a few different weight matrices in turn so that the 126 MB L2 does not serve the reads
    ws = [UnifiedTensor((torch.randn(k * n, device="cuda", generator=g) * 0.05).half().view(torch.uint8),
                        [k, n], DType.FP16) for _ in range(args.copies)]
    out = UnifiedTensor.empty(ctx, [1, n])
    for i in range(args.warmup):
        eng.matmul_f16b(ctx, x, ws[i % len(ws)], out)
    ctx.profile(2)
    for i in range(args.iters):
        eng.matmul_f16b(ctx, x, ws[i % len(ws)], out)
    ctx.synchronize()
    rep = _report(ctx, "matvec", {"k": k, "n": n})
    ms = sum(v["ms_per_launch"] for v in rep["kernels"].values())
    print(f"matvec f16 weights {k} x {n}: {ms * 1e3:.1f} us, {k * n * 2 / (ms * 1e-3) / 1e9:.0f} GB/s of weights")


def decode(args):
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    b, s, h, hk, d = args.batch, args.seq, args.heads, args.kv_heads, 64
    q = _dev_f32(ctx, [b, 1, h, d], 1.0, 1)
    caches = [(_dev_f32(ctx, [b, s, hk, d], 1.0, 2 + 2 * i), _dev_f32(ctx, [b, s, hk, d], 1.0, 3 + 2 * i))
              for i in range(args.copies)]
    out = UnifiedTensor.empty(ctx, [b, 1, h, d])
    opts = AttentionOptions(causal=True, causal_offset=s - 1)
    for i in range(args.warmup):
        eng.flash_attention_v2_with(ctx, q, *caches[i % len(caches)], out, opts)
    ctx.profile(2)
    for i in range(args.iters):
        eng.flash_attention_v2_with(ctx, q, *caches[i % len(caches)], out, opts)
    ctx.synchronize()
    rep = _report(ctx, "decode", {"batch": b, "seq": s, "heads": h, "kv_heads": hk})
    ms = sum(v["ms_per_launch"] for v in rep["kernels"].values())
    byts = 2.0 * b * s * hk * d * 4
    print(f"decode attention: {ms * 1e3:.1f} us, {byts / (ms * 1e-3) / 1e9:.0f} GB/s of K and V")


def _sample_clocks(stop, acc, device):
    import subprocess
    import time
    while not stop.is_set():
        out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits",
                              "-i", str(device)], capture_output=True, text=True).stdout.strip().split(",")
        try:
            acc.append((float(out[0]), float(out[1])))
        except (ValueError, IndexError):
            pass
        time.sleep(0.2)


def step(args):
    """One micro-batch (forward, loss, backward) and the optimizer update of a benchmark
    workload's architecture cut to `--layers` blocks: every kernel of the training step at the
    shapes of the full model, with a few GB on the device instead of tens."""
    import copy
    from .config import WORKLOADS, init_adapters, init_weights, synthetic_batch
    from .model import LoraModel
    from .trainer import AdamW, batch_targets_weights
    ctx = CudaContext(0)
    ctx.set_gemm_mode(GemmMode.F16)
    w = copy.deepcopy(WORKLOADS[args.workload])
    w.model.layers = args.layers
    weights = init_weights(w.model, w.seed, device="cuda:0", f16_base=True)
    adapters = init_adapters(w.model, w.lora, w.seed, device="cuda:0", b_std=w.adapter_b_std)
    model = LoraModel(ctx, w.model, w.lora, weights, adapters, f16_base=True,
                      checkpoint_blocks=w.checkpoint_blocks)
    del weights, adapters
    torch.cuda.empty_cache()
    ids, tg, mk = synthetic_batch(w, args.batch)
    rt, rw, _ = batch_targets_weights(tg, mk, w.model.vocab)
    d_ids = torch.from_numpy(np.ascontiguousarray(ids).view(np.int32).reshape(-1)).cuda()
    d_tg = torch.from_numpy(rt.view(np.int32).reshape(-1)).cuda()
    d_w = torch.from_numpy(rw.reshape(-1)).cuda()
    row_loss = torch.empty(ids.size, device="cuda", dtype=torch.float32)
    opt = AdamW(w.lr, weight_decay=w.weight_decay)

    def once():
        model.zero_grad()
        model.forward_backward(d_ids, d_tg, d_w, args.batch, w.seq_len, 1.0 / args.batch, row_loss)
        opt.t += 1.0
        model.apply_gradients(1.0, w.clip, opt.params())
    for _ in range(args.warmup):
        once()
    ctx.profile(2)
    for _ in range(args.iters):
        once()
    ctx.synchronize()
    _report(ctx, "step", {"workload": w.name, "layers": args.layers, "sequences": args.batch,
                          "seq_len": w.seq_len, "loss": float(row_loss.sum().item()) / ids.size})
    model.close()


def sustained(args):
    """Each product back to back for `--seconds`, long enough for the power cap to settle the clock:
    this library's tensor-core GEMM (f32 activations rounded to f16 by its conversion kernel, f32
    result) and torch.matmul on the same f16 operands (cuBLAS, f16 result), with the median SM
    clock and board power of the second half of each run.  The GEMM's own time comes from the
    library's per-kernel events, cuBLAS's from events around each batch of launches."""
    import threading
    import time
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    ctx.set_gemm_mode(GemmMode.F16)
    shapes = [(8192, 8192, 2048), (8192, 2048, 8192), (8192, 2048, 2048), (8192, 16384, 2048), (8192, 6144, 2048),
              (8192, 8192, 8192)] if not args.shape else [tuple(args.shape)]
    per = 200
    for m, n, k in shapes:
        g = torch.Generator(device="cuda").manual_seed(1)
        a32 = torch.randn(m * k, device="cuda", generator=g)
        b16 = (torch.randn(n * k, device="cuda", generator=g) * 0.05).half()
        a = UnifiedTensor(a32.view(torch.uint8), [m, k], DType.F32)
        b = UnifiedTensor(b16.view(torch.uint8), [n, k], DType.FP16)
        out = UnifiedTensor.empty(ctx, [m, n])
        a16, bt = a32.view(m, k).half(), b16.view(n, k)
        flop = 2.0 * m * n * k
        row = {"case": "sustained", "m": m, "n": n, "k": k, "seconds": args.seconds}

        def run(batch):
            acc, stop = [], threading.Event()
            th = threading.Thread(target=_sample_clocks, args=(stop, acc, 0))
            th.start()
            t0, last = time.time(), None
            while time.time() - t0 < args.seconds:
                last = batch()
            stop.set()
            th.join()
            tail = acc[len(acc) // 2:] or [(float("nan"), float("nan"))]
            return last, float(np.median([c for c, _ in tail])), float(np.median([w for _, w in tail]))

        def ours():
            ctx.profile(2)
            for _ in range(per):
                eng.matmul_bt_f16b(ctx, a, b, out)
            ctx.synchronize()
            rep = ctx.profile_report()
            ctx.profile(0)
            cnt, ms = next((v for name, v in rep.items() if name.startswith("k_gemm_tc")), (0, 0.0))
            return flop * cnt / (ms * 1e-3) / 1e12 if ms else float("nan")

        def cublas():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(per):
                torch.matmul(a16, bt.t())
            e1.record()
            torch.cuda.synchronize()
            return flop * per / (e0.elapsed_time(e1) * 1e-3) / 1e12

        for name, fn in (("library", ours), ("cublas", cublas)):
            fn()
            tf, mhz, watts = run(fn)
            row[name] = {"tflops": round(tf, 1), "sm_mhz": mhz, "watts": watts}
        print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=2048)
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--seq", type=int, default=1024)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=32)
    a.add_argument("--forward-only", action="store_true")
    mv = sub.add_parser("matvec")
    mv.add_argument("--k", type=int, default=2048)
    mv.add_argument("--n", type=int, default=8192)
    mv.add_argument("--copies", type=int, default=8)
    dc = sub.add_parser("decode")
    dc.add_argument("--batch", type=int, default=8)
    dc.add_argument("--seq", type=int, default=4096)
    dc.add_argument("--heads", type=int, default=32)
    dc.add_argument("--kv-heads", type=int, default=32)
    dc.add_argument("--copies", type=int, default=3)
    su = sub.add_parser("sustained")
    su.add_argument("--seconds", type=float, default=4.0)
    su.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), default=None)
    st = sub.add_parser("step")
    st.add_argument("--workload", default="smollm2-1.7b")
    st.add_argument("--layers", type=int, default=2)
    st.add_argument("--batch", type=int, default=8)
    for p in (g, a, mv, dc, st):
        p.add_argument("--iters", type=int, default=5)
        p.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    {"gemm": gemm, "attention": attention, "matvec": matvec, "decode": decode, "sustained": sustained,
     "step": step}[args.case](args)


if __name__ == "__main__":
    main()
