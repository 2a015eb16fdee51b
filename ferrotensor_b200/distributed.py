"""Data-parallel gradient exchange: the host side of `ft_comm_*`.

Counterpart of `FileGradSyncConfig` + `average_grads_file_sync`
(ferrotensor-trainer/src/distributed.rs:17-69,107-185): world size, rank and a wait limit;
the exchange itself is one NCCL all-reduce inside libft_cuda on the context's stream.
The 128-byte communicator id made by rank 0 travels over any host channel; two are offered
here: an initialised `torch.distributed` group, or a file in a shared directory (the
reference's `sync_dir`).
"""

from __future__ import annotations

import ctypes as C
import os
import time
from pathlib import Path
from typing import Optional

from . import _lib
from ._lib import FtError, call


def validate_world(world_size: int, rank: int) -> None:
    """`FileGradSyncConfig::new` (distributed.rs:31-44)."""
    if world_size == 0:
        raise ValueError("world_size must be >= 1")
    if rank >= world_size or rank < 0:
        raise ValueError(f"rank {rank} is out of range for world_size {world_size}")


class Communicator:
    """One rank of a data-parallel group.  `max_wait_s` bounds the creation and every later
    wait, as the reference's `max_wait` does (default there: 600 s)."""

    def __init__(self, ctx, world_size: int, rank: int, comm_id: Optional[bytes],
                 max_wait_s: float = 600.0):
        validate_world(world_size, rank)
        self.ctx, self.world_size, self.rank = ctx, world_size, rank
        self.max_wait_ms = max(1, int(max_wait_s * 1000))
        handle = C.c_void_p()
        buf = None
        if world_size > 1:
            if comm_id is None or len(comm_id) != _lib.FT_COMM_ID_BYTES:
                raise ValueError(f"comm_id must be {_lib.FT_COMM_ID_BYTES} bytes")
            buf = C.create_string_buffer(bytes(comm_id), _lib.FT_COMM_ID_BYTES)
        call("ft_comm_create", ctx.handle, world_size, rank, buf, self.max_wait_ms, C.byref(handle))
        self.handle = handle

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(_lib.FT_COMM_ID_BYTES)
        call("ft_comm_unique_id", buf)
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, ctx, max_wait_s: float = 600.0) -> "Communicator":
        """Rank and world of the initialised default process group; rank 0's id is broadcast
        through it (host objects, so a gloo group serves as well)."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(), dist.get_rank()
        box = [cls.unique_id() if rank == 0 and world > 1 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        return cls(ctx, world, rank, box[0], max_wait_s)

    @classmethod
    def from_sync_dir(cls, ctx, world_size: int, rank: int, sync_dir, max_wait_s: float = 600.0,
                      name: str = "comm_id.bin") -> "Communicator":
        """The id as a file in a directory every rank can read (written atomically by rank 0,
        awaited by the others up to `max_wait_s`)."""
        validate_world(world_size, rank)
        path = Path(sync_dir) / name
        if world_size > 1:
            if rank == 0:
                path.parent.mkdir(parents=True, exist_ok=True)
                tmp = path.with_name(f".{path.name}.tmp.{os.getpid()}")
                tmp.write_bytes(cls.unique_id())
                os.replace(tmp, path)
            deadline = time.monotonic() + max_wait_s
            while not path.exists():
                if time.monotonic() > deadline:
                    raise FtError(_lib.FT_ERR_COMM, f"timed out waiting for {path}")
                time.sleep(0.025)
            comm_id = path.read_bytes()
        else:
            comm_id = None
        return cls(ctx, world_size, rank, comm_id, max_wait_s)

    def allreduce_sum(self, tensor) -> None:
        """In-place sum of a contiguous f32 device tensor over the ranks."""
        call("ft_comm_allreduce_sum", self.handle, C.c_void_p(tensor.data_ptr()), tensor.numel())

    def wait(self, timeout_s: float = 0.0) -> None:
        """Block until the last collective has finished on the device; raises FtError
        (FT_ERR_COMM) after the limit, with the communicator aborted."""
        call("ft_comm_wait", self.handle, int(timeout_s * 1000))

    def close(self) -> None:
        if self.handle:
            call("ft_comm_destroy", self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
