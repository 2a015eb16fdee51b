"""Data parallelism through the C ABI on real GPUs: `ft_comm_*` and
`ft_model_allreduce_apply_gradients` (ferrotensor-trainer/src/distributed.rs:107-185,
src/lib.rs:318-358: every rank averages, then performs the identical update).

Each rank is a child process on its own GPU (needs at least two; skipped otherwise).  The
communicator id travels through a file in a shared directory, as the reference's gradient
files do.  NVLS is switched off for these processes: a rank that leaves must not hold a
multicast binding.  Nothing here faults or hangs a GPU: the failure case is a rank that never
joins, which the host-side deadline of `ft_comm_create` turns into an error code.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import lora_step as ol

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

_RANK_SCRIPT = r"""
import json, os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch
rank, world, sync_dir, steps = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4])
torch.cuda.set_device(rank)
from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights, synthetic_batch
from ferrotensor_b200.distributed import Communicator
from ferrotensor_b200.engine import CudaContext, GemmMode
from ferrotensor_b200.model import LoraModel
from ferrotensor_b200.trainer import AdamW, Trainer, shard_indices
import copy
w = copy.deepcopy(WORKLOADS["tiny"])
w.global_batch = 4
ctx = CudaContext(rank)
ctx.set_gemm_mode(GemmMode.F32)
weights = init_weights(w.model, w.seed, norm_jitter=0.25)
adapters = init_adapters(w.model, w.lora, w.seed, b_std=w.adapter_b_std)
model = LoraModel(ctx, w.model, w.lora, weights, adapters, f16_base=False)
comm = Communicator.from_sync_dir(ctx, world, rank, sync_dir, max_wait_s=60.0)
ids, tg, mk = synthetic_batch(w, w.global_batch)
mine = shard_indices(w.global_batch, world, rank)
tr = (Trainer(model, AdamW(w.lr, weight_decay=w.weight_decay)).with_grad_accum_steps(len(mine))
      .with_clip_grad_norm(0.05).with_distributed(world, rank, comm))
tr.length_bucket = 16
norms = []
for _ in range(steps):
    stats = tr.train_arrays(ids[mine], tg[mine], mk[mine])
    assert stats[-1].optimizer_step
    norms.append(stats[-1].grad_norm)
ctx.synchronize()
np.save(os.path.join(sync_dir, f"params_rank{{rank}}.npy"), model.params.cpu().numpy())
np.save(os.path.join(sync_dir, f"grads_rank{{rank}}.npy"), model.grads.cpu().numpy())
with open(os.path.join(sync_dir, f"norms_rank{{rank}}.json"), "w") as f:
    json.dump(norms, f)
names = model.adapter_names()
slices = {{n: model._slices[n] for n in names}}
if rank == 0:
    with open(os.path.join(sync_dir, "slices.json"), "w") as f:
        json.dump(slices, f)
comm.close()
model.close()
print("rank", rank, "done")
"""

_LONELY_SCRIPT = r"""
import sys, time
sys.path.insert(0, {root!r})
import torch
torch.cuda.set_device(0)
from ferrotensor_b200._lib import FT_ERR_COMM, FtError
from ferrotensor_b200.distributed import Communicator
from ferrotensor_b200.engine import CudaContext
ctx = CudaContext(0)
t0 = time.monotonic()
try:
    Communicator(ctx, 2, 0, Communicator.unique_id(), max_wait_s=3.0)   # rank 1 never comes
except FtError as e:
    dt = time.monotonic() - t0
    assert e.code == FT_ERR_COMM, e
    assert "timed out" in str(e), e
    assert dt < 30.0, dt
    # the context is still usable afterwards
    x = torch.ones(8, device="cuda")
    ctx.synchronize()
    assert float(x.sum()) == 8.0
    print("timed out as it should after", round(dt, 1), "s")
    sys.exit(0)
sys.exit("ft_comm_create returned although rank 1 never joined")
"""


def _gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _env():
    env = dict(os.environ)
    env.update(NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    return env


@pytest.mark.parametrize("world", [2, 4])
def test_n_rank_step_equals_the_one_rank_oracle(tmp_path, world):
    """Two optimizer steps of the tiny workload (4 sequences, clipping active) on `world` GPUs:
    all ranks end with bit-identical parameters, and those equal the oracle's `world`-rank step
    (sum of the ranks' gradients x 1/world, global norm, clip, AdamW) within the step tolerance."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT.format(root=str(ROOT)))
    steps = 2
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), str(tmp_path), str(steps)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=_env())
             for r in range(world)]
    outs = [p.communicate(timeout=600)[0].decode() for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    params = [np.load(tmp_path / f"params_rank{r}.npy") for r in range(world)]
    grads = [np.load(tmp_path / f"grads_rank{r}.npy") for r in range(world)]
    for r in range(1, world):
        assert np.array_equal(params[0].view(np.uint32), params[r].view(np.uint32)), f"rank {r} parameters differ"
        assert np.array_equal(grads[0].view(np.uint32), grads[r].view(np.uint32)), f"rank {r} summed gradients differ"
    norms = [json.loads((tmp_path / f"norms_rank{r}.json").read_text()) for r in range(world)]
    assert all(n == norms[0] for n in norms)

    # the oracle's world-rank run of the same two steps
    import copy
    from ferrotensor_b200.config import WORKLOADS, init_adapters, init_weights, synthetic_batch
    from ferrotensor_b200.trainer import shard_indices
    w = copy.deepcopy(WORKLOADS["tiny"])
    w.global_batch = 4
    weights = init_weights(w.model, w.seed, norm_jitter=0.25)
    adapters = init_adapters(w.model, w.lora, w.seed, b_std=w.adapter_b_std)
    ocfg = ol.OracleConfig(vocab=w.model.vocab, hidden=w.model.hidden, layers=w.model.layers,
                           heads=w.model.heads, kv_heads=w.model.kv_heads, ffn=w.model.ffn,
                           eps=w.model.eps, theta=w.model.theta, lora_rank=w.lora.rank,
                           lora_alpha=w.lora.alpha, lora_targets=tuple(w.lora.target_modules))
    p = {k: v.clone() for k, v in {**weights, **adapters}.items()}
    ids, tg, mk = synthetic_batch(w, w.global_batch)
    mbs = [[(ids[shard_indices(4, world, r)].astype(np.int64), tg[shard_indices(4, world, r)].astype(np.int64),
             mk[shard_indices(4, world, r)])] for r in range(world)]
    hp = ol.AdamParams(lr=w.lr, weight_decay=w.weight_decay)
    state = {}
    exp_norms = []
    for _ in range(steps):
        _, _, norm, *_ = ol.lora_step(ocfg, p, mbs, hp, state, clip_grad_norm=0.05, world=world)
        exp_norms.append(float(norm))
    assert np.allclose(norms[0], exp_norms, rtol=1e-3, atol=1e-5), (norms[0], exp_norms)
    assert exp_norms[0] > 0.05      # clipping was active
    slices = json.loads((tmp_path / "slices.json").read_text())
    for name, (off, rows, cols) in slices.items():
        got = params[0][off:off + rows * cols].reshape(rows, cols)
        e = p[name].numpy()
        assert np.all(np.abs(got - e) <= 1e-5 + 1e-4 * np.abs(e)), name


def test_a_rank_that_never_joins_times_out_on_the_host(tmp_path):
    """`ft_comm_create` for a world of two where the second rank never starts: the host-side
    deadline ends the call with FT_ERR_COMM (the reference: "timed out waiting for ..." after
    `max_wait`, distributed.rs:124-126); no kernel was launched and the GPU stays usable."""
    if _gpus() < 1:
        pytest.skip("needs a GPU")
    script = tmp_path / "lonely.py"
    script.write_text(_LONELY_SCRIPT.format(root=str(ROOT)))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300,
                       env=_env())
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
