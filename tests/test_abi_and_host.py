"""CPU-only checks: the C-ABI library loads and exports what include/ft_cuda.h declares,
and the host-side integer logic matches the oracle's restatement of the reference."""

import ctypes
import re
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import lora_step as ol

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from ferrotensor_b200 import _build, _lib
    _build.build()
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "ft_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ft_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lib, n), f"{n} declared in ft_cuda.h but not exported"


def test_every_prototype_is_declared_in_header(lib):
    from ferrotensor_b200 import _lib
    declared = set(declared_symbols())
    for n in list(_lib.PROTOTYPES) + list(_lib.STRING_GETTERS):
        assert n in declared, f"{n} bound in python but missing from ft_cuda.h"


def test_struct_layouts_match_header(tmp_path):
    """ctypes mirrors against the header itself: sizes and a few offsets printed by a C program."""
    import subprocess
    from ferrotensor_b200 import _lib
    assert ctypes.sizeof(_lib.FtAdamParams) == 32       # training.rs:15-32: 6 floats + 2 pad
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "ft_cuda.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(FtAdamParams), sizeof(FtAttnParams), '
                   'sizeof(FtModelConfig), offsetof(FtAttnParams, seed_lo), offsetof(FtAttnParams, mask_stride), '
                   'offsetof(FtModelConfig, attention_dropout)); return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    A, M = _lib.FtAttnParams, _lib.FtModelConfig
    assert got == [ctypes.sizeof(_lib.FtAdamParams), ctypes.sizeof(A), ctypes.sizeof(M), A.seed_lo.offset,
                   A.mask_stride.offset, M.attention_dropout.offset]
    assert ctypes.sizeof(A) == 18 * 4 and ctypes.sizeof(M) == 17 * 4


def test_build_info_lists_the_tensor_core_kernel(lib):
    info = lib.ft_build_info().decode()
    assert "sm_100a" in info and "tcgen05" in info


def test_no_gpu_call_fails_loudly(lib):
    """Without a device the context cannot be created and the error says why; nothing
    falls back to a CPU path."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from ferrotensor_b200.engine import CudaContext
    from ferrotensor_b200._lib import FtError
    with pytest.raises(FtError):
        CudaContext(0)
    h = ctypes.c_void_p()
    rc = lib.ft_ctx_create(0, None, ctypes.byref(h))
    assert rc != 0 and lib.ft_last_error()


def test_product_does_not_import_the_oracle():
    for f in (ROOT / "ferrotensor_b200").rglob("*.py"):
        src = f.read_text()
        assert "import oracle" not in src and "from oracle" not in src, f


def test_pad_chunk_and_targets_match_oracle():
    from ferrotensor_b200 import trainer as tr
    rng = np.random.default_rng(0)
    chunk = []
    for _ in range(5):
        n = int(rng.integers(2, 70))
        ids = rng.integers(0, 50, n).tolist()
        tgt = rng.integers(0, 60, n).tolist()      # some targets >= vocab (50)
        msk = rng.integers(0, 2, n).tolist()
        chunk.append((ids, tgt, msk))
    ids, tgt, msk = tr.pad_chunk(chunk, 32)
    oi, ot, om = ol.pad_chunk(chunk, 32)
    assert ids.tolist() == oi and tgt.tolist() == ot and msk.tolist() == om
    t, w, tokens = tr.batch_targets_weights(tgt, msk, 50)
    et, ew, etok = ol.batch_targets_weights(np.array(ot).reshape(-1).tolist(),
                                            np.array(om).reshape(-1).tolist(), 5, 50)
    assert t.reshape(-1).tolist() == et.tolist()
    assert w.reshape(-1).tobytes() == ew.tobytes()   # bit-exact f32 weights
    assert tokens.tolist() == etok


def test_scheduler_and_sharding_match_reference_values():
    from ferrotensor_b200 import trainer as tr
    s = tr.WarmupCosineScheduler(1.0, 0.1, 4, 14)
    lrs = []
    for _ in range(15):
        lrs.append(s.get_lr())
        s.step()
    assert lrs[:5] == [0.0, 0.25, 0.5, 0.75, 1.0]
    assert abs(lrs[9] - 0.55) < 1e-6 and lrs[14] == pytest.approx(0.1)
    for i in range(15):
        assert lrs[i] == ol.warmup_cosine_lr(i, 1.0, 0.1, 4, 14)
    assert tr.shard_indices(7, 3, 1) == [1, 4] == ol.shard_indices(7, 3, 1)


def test_workload_flops_match_published_table():
    from ferrotensor_b200.config import WORKLOADS, step_flops
    per_token = {n: step_flops(w, 1) / 1e9 for n, w in WORKLOADS.items()}
    assert per_token["smollm2-1.7b"] == pytest.approx(7.306, abs=2e-3)
    assert per_token["smollm2-135m"] == pytest.approx(0.574, abs=2e-3)
    assert per_token["smollm2-360m"] == pytest.approx(1.583, abs=2e-3)
    assert per_token["qwen2-0.5b"] == pytest.approx(2.599, abs=2e-3)


def test_synthetic_batches_are_seeded_and_rank_sliced():
    from ferrotensor_b200.config import WORKLOADS, synthetic_batch
    w = WORKLOADS["smollm2-360m"]
    a = synthetic_batch(w, 4)
    b = synthetic_batch(w, 2, first=2)
    assert np.array_equal(a[0][2:], b[0]) and np.array_equal(a[2][2:], b[2])
    ids, tgt, msk = a
    assert ids.max() < w.model.vocab and np.array_equal(ids[:, 1:], tgt[:, :-1])
    zeros = (msk == 0).sum(axis=1) / w.seq_len
    assert (zeros >= 0.09).all() and (zeros <= 0.41).all()


_DP_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
from ferrotensor_b200.trainer import Trainer, AdamW, StepStats
rank, world = int(sys.argv[1]), 2
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT={port!r}, RANK=str(rank), WORLD_SIZE="2")
dist.init_process_group("gloo", rank=rank, world_size=world)

class GlooComm:
    # stands in for distributed.Communicator on a machine without GPUs: same protocol
    # (world_size, rank, allreduce_sum, wait), the sum carried by gloo
    def __init__(self, world, rank):
        self.world_size, self.rank, self.waits = world, rank, 0
    def allreduce_sum(self, t):
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    def wait(self, timeout_s=0.0):
        self.waits += 1

class FakeModel:
    # stands in for the device model: a flat gradient buffer and a recorder; its
    # allreduce_apply_gradients does what ft_model_allreduce_apply_gradients does
    def __init__(self):
        self.ctx = None
        self.grads = torch.arange(8, dtype=torch.float32) * (rank + 1)
        self.norm_out = torch.tensor([1.0, 1.0, 0.0, 0.0])
        self.seen = None
    def allreduce_apply_gradients(self, comm, max_norm, adam):
        world = comm.world_size if comm is not None else 1
        if world > 1:
            comm.allreduce_sum(self.grads)
        self.seen = (self.grads * (1.0 / world)).clone()

m = FakeModel()
comm = GlooComm(world, rank)
t = Trainer(m, AdamW(1e-3)).with_distributed(world, rank, comm)
s = StepStats()
t.apply_gradients(s)
assert comm.waits == 1
expect = torch.arange(8, dtype=torch.float32) * 1.5      # mean of 1x and 2x
assert torch.equal(m.seen, expect), (m.seen, expect)
assert s.optimizer_step and t.optimizer.t == 1.0
dist.destroy_process_group()
print("ok", rank)
"""


def test_gradient_mean_over_two_gloo_ranks(tmp_path):
    """World-size-2 run of the trainer's cross-rank step on CPU: sum over ranks followed by
    the 1/world factor equals the reference's mean (distributed.rs:135-172)."""
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = str(s.getsockname()[1])
    script = tmp_path / "dp.py"
    script.write_text(_DP_SCRIPT.format(root=str(ROOT), port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT) for r in range(2)]
    outs = [p.communicate(timeout=120)[0].decode() for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o


def test_communicator_argument_errors():
    """ft_comm_create rejects what FileGradSyncConfig::new rejects (distributed.rs:31-44), with
    the same words, before it touches the context or NCCL."""
    import ctypes as C
    from ferrotensor_b200 import _lib
    lib = _lib.load()
    out = C.c_void_p()
    fake_ctx = C.c_void_p(1)   # never dereferenced: the argument checks come first
    assert lib.ft_comm_create(fake_ctx, 0, 0, None, 1000, C.byref(out)) == 1
    assert "world_size must be >= 1" in _lib.last_error()
    assert lib.ft_comm_create(fake_ctx, 2, 2, None, 1000, C.byref(out)) == 1
    assert "rank 2 is out of range for world_size 2" in _lib.last_error()
    assert lib.ft_comm_create(fake_ctx, 2, -1, None, 1000, C.byref(out)) == 1
    assert lib.ft_comm_create(fake_ctx, 2, 1, None, 0, C.byref(out)) == 1
    assert "timeout_ms" in _lib.last_error()
    assert lib.ft_comm_create(None, 2, 1, None, 1000, C.byref(out)) == 1
    assert lib.ft_comm_unique_id(None) == 1
    assert lib.ft_comm_wait(None, 10) == 1
    assert lib.ft_comm_allreduce_sum(None, None, 4) == 1
    assert lib.ft_comm_destroy(None) == 0
    assert lib.ft_model_allreduce_apply_gradients(None, None, 1.0, None, None) == 1


def test_host_side_world_validation():
    from ferrotensor_b200.distributed import validate_world
    from ferrotensor_b200.trainer import AdamW, Trainer
    validate_world(2, 1)
    with pytest.raises(ValueError, match="world_size must be >= 1"):
        validate_world(0, 0)
    with pytest.raises(ValueError, match="rank 2 is out of range for world_size 2"):
        validate_world(2, 2)

    class M:
        ctx = None
    with pytest.raises(ValueError, match="communicator is required"):
        Trainer(M(), AdamW(1e-3)).with_distributed(2, 0)
