"""The training step on the `cuda` device: the counterpart of `ferrotensor_trainer::Trainer`
(ferrotensor-trainer/src/lib.rs:113-503), `AdamW` / `WarmupCosineScheduler`
(ferrotensor-autograd/src/lib.rs:1482-1552,1763-1805) and the data-parallel gradient mean
(ferrotensor-trainer/src/distributed.rs:107-185, there through files; here one NCCL
all-reduce of the flat gradient buffer inside the library, `distributed.Communicator`).

Host side = integer bookkeeping only (padding, targets, loss weights); every float of the
step is computed by libft_cuda kernels.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ._lib import FT_MASKED_CE_SKIP, FtAdamParams
from .model import LoraModel

MASKED_CE_SKIP = FT_MASKED_CE_SKIP


@dataclass
class StepStats:
    """ferrotensor-trainer/src/lib.rs:44-59"""
    loss: float = 0.0
    tokens: int = 0
    optimizer_step: bool = False
    grad_norm: Optional[float] = None
    lr: Optional[float] = None


@dataclass
class Batch:
    """The fields of the reference's data-loader batch the step reads
    (ferrotensor-trainer/src/data.rs): per-sequence padded ids/targets, attention mask
    (1 = real token) and loss mask (1 = supervised)."""
    padded_input_ids: Sequence[Sequence[int]]
    padded_target_ids: Sequence[Sequence[int]]
    attention_mask: Sequence[Sequence[int]]
    loss_masks: Sequence[Sequence[int]]
    input_ids: Optional[Sequence[Sequence[int]]] = None     # unpadded, as the data loader read them
    target_ids: Optional[Sequence[Sequence[int]]] = None
    max_seq_len: int = 0

    @property
    def batch_size(self) -> int:
        return len(self.padded_input_ids)


class AdamW:
    """Hyper-parameters and step counter; the update itself runs on the device.
    Defaults as `AdamW::new`: betas (0.9, 0.999), eps 1e-8, weight decay 0.01."""

    def __init__(self, lr: float, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay = weight_decay
        self.t = 0.0

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def params(self) -> FtAdamParams:
        return FtAdamParams(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.t)


class WarmupCosineScheduler:
    """Linear warm-up from 0 to `peak_lr`, cosine decay to `min_lr`; f32 arithmetic."""

    def __init__(self, peak_lr: float, min_lr: float, warmup_steps: int, total_steps: int):
        self.peak_lr, self.min_lr = np.float32(peak_lr), np.float32(min_lr)
        self.warmup_steps, self.total_steps = warmup_steps, total_steps
        self.current = 0

    def get_lr(self) -> float:
        f = np.float32
        if self.current < self.warmup_steps:
            return float(self.peak_lr * (f(self.current) / f(self.warmup_steps)))
        if self.current >= self.total_steps:
            return float(self.min_lr)
        progress = f(self.current - self.warmup_steps) / f(self.total_steps - self.warmup_steps)
        cosine = (f(1.0) + np.cos(f(np.pi) * progress, dtype=f)) / f(2.0)
        return float(self.min_lr + (self.peak_lr - self.min_lr) * cosine)

    def step(self) -> None:
        self.current += 1

    def current_step(self) -> int:
        return self.current


def shard_indices(n: int, world_size: int, rank: int) -> List[int]:
    """Round-robin data sharding (distributed.rs:222-227)."""
    return [i for i in range(n) if i % world_size == rank]


def pad_chunk(chunk, length_bucket: int):
    """Right-pad (ids, targets, mask) triples to a common multiple of `length_bucket`: ids
    and targets with the sequence's own last input id, masks with 0 (lib.rs:431-450)."""
    longest = max(min(len(i), len(t)) for i, t, _ in chunk)
    padded = -(-longest // length_bucket) * length_bucket
    n = len(chunk)
    ids = np.empty((n, padded), dtype=np.uint32)
    tgt = np.empty((n, padded), dtype=np.uint32)
    msk = np.zeros((n, padded), dtype=np.uint8)
    for r, (i, t, m) in enumerate(chunk):
        ln = min(len(i), len(t))
        pad = i[ln - 1] if ln else 0
        ids[r, :ln], ids[r, ln:] = i[:ln], pad
        tgt[r, :ln], tgt[r, ln:] = t[:ln], pad
        k = min(ln, len(m))
        msk[r, :k] = m[:k]
    return ids, tgt, msk


def batch_targets_weights(targets: np.ndarray, masks: np.ndarray, vocab: int):
    """Row targets (MASKED_CE_SKIP when unsupervised or out of vocabulary), row weights
    1/tokens(sequence) in f32, and the supervised-token count of each sequence
    (lib.rs:689-716).  `targets`, `masks` are [sequences, seq_len]."""
    sup = (masks != 0) & (targets < vocab)
    tokens = sup.sum(axis=1)
    tgt = np.where(sup, targets, np.uint32(MASKED_CE_SKIP)).astype(np.uint32)
    inv = np.zeros(len(tokens), dtype=np.float32)
    nz = tokens > 0
    inv[nz] = np.float32(1.0) / tokens[nz].astype(np.float32)
    wts = np.where(sup, inv[:, None], np.float32(0.0)).astype(np.float32)
    return tgt, wts, tokens


class Trainer:
    def __init__(self, model: LoraModel, optimizer: AdamW):
        self.model = model
        self.optimizer = optimizer
        self.ctx = model.ctx
        self.clip_grad_norm: Optional[float] = None
        self.grad_accum_steps = 1
        self.step_in_accum = 0
        self.lr_scheduler: Optional[WarmupCosineScheduler] = None
        self.length_bucket = 32
        self.max_chunk: Optional[int] = None   # memory bound on sequences per micro-batch
        self.world_size, self.rank = 1, 0
        self.comm = None                       # distributed.Communicator when world_size > 1
        self.optimizer_step_count = 0
        self.keep_logits = False
        self.last_logits: Optional[torch.Tensor] = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.dropout_seed = 0                  # run seed of the attention-dropout masks
        self._pending: List[Tuple[torch.Tensor, np.ndarray, int, int]] = []  # pinned row losses

    # builder-style setters, as the reference's `with_*`
    def with_grad_accum_steps(self, n: int) -> "Trainer":
        self.grad_accum_steps = max(1, n)
        return self

    def with_clip_grad_norm(self, max_norm: Optional[float]) -> "Trainer":
        self.clip_grad_norm = max_norm
        return self

    def with_lr_scheduler(self, s: WarmupCosineScheduler) -> "Trainer":
        self.lr_scheduler = s
        return self

    def with_dropout_seed(self, seed: int) -> "Trainer":
        self.dropout_seed = int(seed)
        return self

    def attention_dropout_seed(self) -> int:
        """The seed of the next forward pass's dropout masks: run seed, rank, optimizer step and
        position in the accumulation window (lib.rs:185-197); layers derive their own from it."""
        from .dropout import attention_dropout_seed
        return attention_dropout_seed(self.dropout_seed, self.rank if self.world_size > 1 else 0,
                                      self.optimizer_step_count, self.step_in_accum)

    def with_distributed(self, world_size: int, rank: int, comm=None) -> "Trainer":
        """Average gradients over `world_size` ranks through `comm`
        (`distributed.Communicator`, one per rank)."""
        from .distributed import validate_world
        validate_world(world_size, rank)
        if world_size > 1 and comm is None:
            raise ValueError("with_distributed: a communicator is required when world_size > 1")
        if comm is not None and (comm.world_size, comm.rank) != (world_size, rank):
            raise ValueError("with_distributed: the communicator was created for another rank/world")
        self.world_size, self.rank, self.comm = world_size, rank, comm
        return self

    def set_optimizer_steps(self, steps: int) -> None:
        """Restore the optimizer-step counter on resume and advance the LR schedule to match
        (lib.rs:204-213)."""
        if self.lr_scheduler is not None:
            while self.lr_scheduler.current_step() < steps:
                self.lr_scheduler.step()
        self.optimizer_step_count = steps

    # ---- one forward/backward over a chunk of sequences -----------------------------------
    def _run_chunk(self, ids: np.ndarray, tgt: np.ndarray, msk: np.ndarray) -> None:
        n, s = ids.shape
        dev = self.ctx.device
        row_tgt, row_w, tokens = batch_targets_weights(tgt, msk, self.model.cfg.vocab)
        packed = np.concatenate([ids.reshape(-1).view(np.int32), row_tgt.reshape(-1).view(np.int32),
                                 row_w.reshape(-1).view(np.int32)])
        host = torch.from_numpy(packed).pin_memory()
        devbuf = host.to(dev, non_blocking=True)
        self.h2d_bytes += packed.nbytes
        rows = n * s
        d_ids, d_tgt = devbuf[:rows], devbuf[rows:2 * rows]
        d_w = devbuf[2 * rows:].view(torch.float32)
        row_loss = torch.empty(rows, device=dev, dtype=torch.float32)
        logits = None
        if self.keep_logits:
            logits = torch.empty((n, s, self.model.cfg.vocab), device=dev, dtype=torch.float32)
        seed = 1.0 / self.grad_accum_steps
        if self.step_in_accum == 0:
            self.model.zero_grad()
        if self.model.cfg.attention_dropout > 0.0:
            self.model.set_dropout_seed(self.attention_dropout_seed())
        self.model.forward_backward(d_ids, d_tgt, d_w, n, s, seed, row_loss, logits)
        self.last_logits = logits
        # row losses travel to pinned host memory asynchronously; they are summed per
        # sequence in f64 on the host, as the reference does, once the window closes
        host_loss = torch.empty(rows, dtype=torch.float32, pin_memory=True)
        host_loss.copy_(row_loss, non_blocking=True)
        self.d2h_bytes += rows * 4
        self._pending.append((host_loss, tokens, n, s))

    def _collect(self) -> List[StepStats]:
        out: List[StepStats] = []
        self.ctx.synchronize()
        for host_loss, tokens, n, s in self._pending:
            host = host_loss.numpy().reshape(n, s).astype(np.float64).sum(axis=1)
            for r in range(n):
                t = int(tokens[r])
                out.append(StepStats(loss=float(np.float32(host[r] / max(t, 1))), tokens=t))
        self._pending.clear()
        return out

    def apply_gradients(self, stats: StepStats) -> None:
        """Mean over ranks -> global norm -> skip if non-finite -> clip -> LR schedule ->
        AdamW (lib.rs:296-360); norm, skip and clip are decided on the device."""
        prev_lr = self.optimizer.lr
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
            lr = self.lr_scheduler.get_lr()
            self.optimizer.set_lr(lr)
            stats.lr = lr
        self.optimizer.t += 1.0
        # sum over the ranks (NCCL, inside the library) with 1/world folded into the update
        self.model.allreduce_apply_gradients(self.comm if self.world_size > 1 else None,
                                             self.clip_grad_norm, self.optimizer.params())
        if self.comm is not None and self.world_size > 1:
            self.comm.wait()   # a peer that never joined ends here as FtError, not as a hang
        norm, applied = self.model.norm_out[:2].tolist()
        self.d2h_bytes += 8
        stats.grad_norm = norm
        if applied == 0.0:
            # non-finite norm: the device skipped the update.  The reference returns before the
            # schedule advances (lib.rs:330-352): undo the host-side counters, schedule included.
            self.optimizer.t -= 1.0
            if self.lr_scheduler is not None:
                self.lr_scheduler.current -= 1
                self.optimizer.set_lr(prev_lr)
            stats.lr = None
            return
        self.optimizer_step_count += 1
        stats.optimizer_step = True

    def train_chunk(self, chunk) -> List[StepStats]:
        ids, tgt, msk = pad_chunk(chunk, self.length_bucket)
        self._run_chunk(ids, tgt, msk)
        self.step_in_accum += len(chunk)
        out: List[StepStats] = []
        if self.step_in_accum >= self.grad_accum_steps:
            self.step_in_accum = 0
            out = self._close_window()
        return out

    def _close_window(self) -> List[StepStats]:
        applied = StepStats()
        self.apply_gradients(applied)
        window = self._collect()
        last = window[-1] if window else StepStats()
        if not window:
            window.append(last)
        last.optimizer_step, last.grad_norm, last.lr = (applied.optimizer_step, applied.grad_norm,
                                                        applied.lr)
        return window

    def train_batch(self, batch: Batch) -> List[StepStats]:
        """Train on every sequence of `batch` (lib.rs:371-422): padding is stripped by the
        attention mask, sequences without supervised tokens are dropped, chunks stop at the
        accumulation boundary.  Stats are returned when an optimizer step closes a window
        (one entry per sequence of the window)."""
        seqs = []
        for ids, tgt, attn, lm in zip(batch.padded_input_ids, batch.padded_target_ids,
                                      batch.attention_mask, batch.loss_masks):
            valid = 0
            for flag in attn:
                if flag != 1:
                    break
                valid += 1
            ids, tgt, lm = ids[:valid], tgt[:valid], lm[:valid]
            if len(ids) < 2 or len(tgt) == 0 or not any(lm):
                continue
            seqs.append((ids, tgt, lm))
        out: List[StepStats] = []
        rest = seqs
        while rest:
            room = max(self.grad_accum_steps - self.step_in_accum, 1)
            take = min(room, len(rest))
            if self.max_chunk:
                take = min(take, self.max_chunk)
            out.extend(self.train_chunk(rest[:take]))
            rest = rest[take:]
        return out

    # ---- evaluation (ferrotensor-cli/src/main.rs:1111-1137) ---------------------------------
    def evaluate(self, dataset, limit: Optional[int] = None, chunk: int = 8) -> Tuple[float, int]:
        """Token-weighted mean loss over (at most `limit`) examples of `dataset` and the number
        of supervised tokens it covers; (nan, 0) when nothing is supervised.  Forward only:
        gradients and the accumulation window are untouched."""
        examples = list(dataset.examples())[:limit] if limit is not None else list(dataset.examples())
        seqs = [(e.input_ids, e.target_ids, e.loss_mask) for e in examples
                if min(len(e.input_ids), len(e.target_ids)) >= 1 and any(e.loss_mask)]
        dev = self.ctx.device
        loss_sum, tokens_total = 0.0, 0
        for c0 in range(0, len(seqs), max(chunk, 1)):
            ids, tgt, msk = pad_chunk(seqs[c0:c0 + chunk], self.length_bucket)
            n, s = ids.shape
            row_tgt, row_w, tokens = batch_targets_weights(tgt, msk, self.model.cfg.vocab)
            d_ids = torch.from_numpy(ids.reshape(-1).view(np.int32)).to(dev)
            d_tgt = torch.from_numpy(row_tgt.reshape(-1).view(np.int32)).to(dev)
            d_w = torch.from_numpy(row_w.reshape(-1)).to(dev)
            row_loss = torch.empty(n * s, device=dev, dtype=torch.float32)
            self.model.forward_loss(d_ids, d_tgt, d_w, n, s, row_loss)
            self.ctx.synchronize()
            per_seq = row_loss.cpu().numpy().reshape(n, s).astype(np.float64).sum(axis=1)
            for r in range(n):
                t = int(tokens[r])
                if t > 0:
                    loss_sum += float(np.float32(per_seq[r] / t)) * t
                    tokens_total += t
        if tokens_total == 0:
            return float("nan"), 0
        return float(np.float32(loss_sum / tokens_total)), tokens_total

    # ---- checkpoint / resume in the reference's file formats (trainer/checkpoint.rs, ----------
    # ---- cli main.rs:1799-1841: adapter file + `x.state.json` + `x.state.safetensors`) ---------
    def save_adapter(self, path) -> None:
        """The adapters as F32 safetensors with rank/alpha/target_modules in the header."""
        from . import checkpoint as ck
        lora = self.model.lora
        meta = ck.LoraMetadata(lora.rank, lora.alpha, list(lora.target_modules))
        tensors = {ck.reference_tensor_name(n): t.detach().cpu().numpy()
                   for n, t in self.model.named_lora_params().items()}
        ck.save_lora_checkpoint(path, tensors, meta)

    def load_adapter(self, path) -> int:
        """All-or-nothing restore of the adapters (checkpoint.rs:214-297); returns the count."""
        from . import checkpoint as ck
        cp = ck.load_lora_checkpoint(path)
        params = self.model.named_lora_params()
        expected = {ck.reference_tensor_name(n): list(t.shape) for n, t in params.items()}
        sources = ck.resolve_checkpoint(cp, expected)
        adapters = {ck.host_tensor_name(n): torch.from_numpy(np.ascontiguousarray(cp.tensors[key][1]))
                    for n, key in sources.items()}
        self.model.load_adapters(adapters)
        return len(adapters)

    def optimizer_checkpoint(self):
        """`AdamW::save_state` (autograd/lib.rs:1577-1625): hyper-parameters, t, and both moments
        of every trainable tensor under its reference name."""
        from . import checkpoint as ck
        o = self.optimizer
        m, v = self.model.named_moments()
        def states(d):
            return {ck.reference_tensor_name(n): ck.OptimizerTensorState(list(t.shape), t.detach().cpu().numpy().ravel())
                    for n, t in d.items()}
        return ck.AdamWCheckpoint(o.lr, o.beta1, o.beta2, o.eps, o.weight_decay, o.t, states(m), states(v))

    def save_training_checkpoint(self, state_path, training_state) -> None:
        from . import checkpoint as ck
        ck.TrainingCheckpoint(training_state, self.optimizer_checkpoint(), None).save(state_path)

    def load_training_checkpoint(self, state_path):
        """Restores the optimizer from a training checkpoint as `AdamW::load_state` does
        (ferrotensor-autograd/src/lib.rs:1623-1703, CLI resume: main.rs:1724): moments stored
        under old Llama-block names are renamed first; a parameter takes its saved state when
        BOTH moments are stored under its name; a moment that does not fit its parameter is an
        error and nothing is changed; when no parameter matches the optimizer is left as it was;
        otherwise the hyper-parameters and step count are restored too and parameters without
        saved state start from zero moments.  Returns the TrainingState; the match counts are
        left in `self.last_optimizer_load`."""
        from . import checkpoint as ck
        cp = ck.TrainingCheckpoint.load(state_path)
        a = cp.optimizer_state
        self.last_optimizer_load = None
        if a is not None:
            m, v = self.model.named_moments()
            ref_of = {n: ck.reference_tensor_name(n) for n in m}
            ck.upgrade_optimizer_names(a, list(ref_of.values()))
            shapes = {ref_of[n]: tuple(t.shape) for n, t in m.items()}
            matched, report = ck.match_moments(shapes, a)      # raises before anything changes
            self.last_optimizer_load = report
            if matched:
                taken = set(matched)
                for dst, src in ((m, a.m_states), (v, a.v_states)):
                    for n, t in dst.items():
                        r = ref_of[n]
                        if r in taken:
                            s_ = src[r]
                            t.copy_(torch.from_numpy(np.asarray(s_.data, np.float32).reshape(s_.shape)))
                        else:
                            t.zero_()
                o = self.optimizer
                o.lr, o.beta1, o.beta2, o.eps, o.weight_decay, o.t = (a.lr, a.beta1, a.beta2, a.eps,
                                                                      a.weight_decay, a.t)
        return cp.training_state

    def train_arrays(self, ids: np.ndarray, tgt: np.ndarray, msk: np.ndarray) -> List[StepStats]:
        """`train_batch` for already rectangular uint32/uint8 arrays [sequences, seq_len]
        whose length is a multiple of the length bucket (the benchmark's input form)."""
        out: List[StepStats] = []
        n = ids.shape[0]
        r = 0
        while r < n:
            room = max(self.grad_accum_steps - self.step_in_accum, 1)
            take = min(room, n - r)
            if self.max_chunk:
                take = min(take, self.max_chunk)
            self._run_chunk(ids[r:r + take], tgt[r:r + take], msk[r:r + take])
            self.step_in_accum += take
            r += take
            if self.step_in_accum >= self.grad_accum_steps:
                self.step_in_accum = 0
                out.extend(self._close_window())
        return out
