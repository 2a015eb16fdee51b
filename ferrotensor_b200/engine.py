"""Host-side mirror of the reference's operator surface for the `cuda` device.

`ComputeEngine`, `UnifiedTensor` and `CudaContext` carry the names, argument order and
error behaviour of `ferrotensor_backend::{ComputeEngine, UnifiedTensor, WgpuContext}`
(ferrotensor-backend/src/engine/*.rs, tensor.rs, context.rs) so that code written
against the reference's engine reads the same here.  Every method is one call into
libft_cuda.so; torch only owns the device memory and the stream.
"""

from __future__ import annotations

import ctypes as C
import enum
import math
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import FtAdamParams, FtAttnParams, FtError, call

MASKED_CE_SKIP = _lib.FT_MASKED_CE_SKIP
SUM_SQUARES_CHUNK = _lib.FT_SUM_SQUARES_CHUNK


class DType(enum.Enum):
    """ferrotensor-backend/src/tensor.rs:18-29"""
    F32 = "f32"
    FP16 = "f16"
    U32 = "u32"

    def size_bytes(self) -> int:
        return 2 if self is DType.FP16 else 4


class GemmMode(enum.IntEnum):
    F32 = _lib.FT_GEMM_F32
    F16 = _lib.FT_GEMM_F16
    F16X2 = _lib.FT_GEMM_F16X2


class CudaContext:
    """One device + one stream; the counterpart of `WgpuContext` (context.rs:164-237).

    Work is enqueued in program order and runs asynchronously until `synchronize` or a
    read-back, exactly like the reference's pending-encoder queue."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise FtError(-1, "no CUDA device: the cuda engine has no CPU fallback")
        _lib.load()
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = torch.cuda.current_stream(self.device)
        handle = C.c_void_p()
        # torch's default stream is the legacy NULL stream: hand the library cudaStreamLegacy
        # (handle value 1) so that its kernels are ordered with torch's copies and NCCL calls
        raw = self.stream.cuda_stream or 1
        call("ft_ctx_create", device, C.c_void_p(raw), C.byref(handle))
        self.handle = handle
        self.gemm_mode = GemmMode.F32
        self.uploads = 0
        self.readbacks = 0

    def flush(self) -> None:
        call("ft_ctx_flush", self.handle)

    def synchronize(self) -> None:
        call("ft_ctx_synchronize", self.handle)

    def set_gemm_mode(self, mode: GemmMode) -> None:
        call("ft_ctx_set_gemm_mode", self.handle, int(mode))
        self.gemm_mode = GemmMode(int(mode))

    def profile(self, enable) -> None:
        """1/True: bracket every tensor-core GEMM launch with CUDA events (`profile_read`);
        2: every launch, by kernel name (`profile_report`); 0/False: off."""
        call("ft_ctx_profile", self.handle, int(enable))

    def profile_report(self):
        """{kernel name: (launches, total ms)} since the last report (mode 2)."""
        buf = C.create_string_buffer(1 << 16)
        call("ft_ctx_profile_report", self.handle, buf, len(buf))
        out = {}
        for line in buf.value.decode().splitlines():
            name, n, ms = line.rsplit(" ", 2)
            out[name] = (int(n), float(ms))
        return out

    def profile_read(self):
        """(kernel ms, algorithmic FLOPs, launches) of the GEMM launches since the last read."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_uint64()
        call("ft_ctx_profile_read", self.handle, C.byref(ms), C.byref(fl), C.byref(n))
        return ms.value, fl.value, n.value

    def profile_read_fused(self):
        """The same for the GEMM launches whose epilogue also does RoPE or SwiGLU (read before
        `profile_read`, which closes the interval)."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_uint64()
        call("ft_ctx_profile_read_fused", self.handle, C.byref(ms), C.byref(fl), C.byref(n))
        return ms.value, fl.value, n.value

    def profile_bytes(self) -> float:
        """Algorithmic bytes of the GEMM launches timed so far (read before `profile_read`)."""
        b = C.c_double()
        call("ft_ctx_profile_bytes", self.handle, C.byref(b))
        return b.value

    def launch_count(self) -> int:
        n = C.c_uint64()
        call("ft_ctx_launch_count", self.handle, C.byref(n))
        return n.value

    def adapter_info(self) -> str:
        p = torch.cuda.get_device_properties(self.device)
        return f"{p.name} (sm_{p.major}{p.minor}, {p.multi_processor_count} SMs, CUDA)"

    def close(self) -> None:
        if self.handle:
            call("ft_ctx_destroy", self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def _numel(shape: Sequence[int]) -> int:
    return int(math.prod(shape)) if len(shape) else 1


class UnifiedTensor:
    """Device buffer + shape + dtype (tensor.rs:57-65).  Clones made by `reshaped` share
    the buffer."""

    def __init__(self, storage: torch.Tensor, shape: Sequence[int], dtype: DType):
        self.storage = storage
        self.shape = list(shape)
        self.dtype = dtype

    # -- constructors -------------------------------------------------------------------
    @staticmethod
    def _alloc(ctx: CudaContext, shape, dtype: DType, zero=False) -> "UnifiedTensor":
        n = _numel(shape)
        nbytes = (n * dtype.size_bytes() + 3) // 4 * 4
        fn = torch.zeros if zero else torch.empty
        return UnifiedTensor(fn(max(nbytes, 4), dtype=torch.uint8, device=ctx.device), shape, dtype)

    @staticmethod
    def new(ctx: CudaContext, data, shape) -> "UnifiedTensor":
        host = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        assert host.size == _numel(shape), "UnifiedTensor::new: data length does not match shape"
        t = UnifiedTensor._alloc(ctx, shape, DType.F32)
        t.write_data(ctx, host.tobytes())
        return t

    @staticmethod
    def empty(ctx: CudaContext, shape) -> "UnifiedTensor":
        return UnifiedTensor._alloc(ctx, shape, DType.F32)

    @staticmethod
    def empty_with_dtype(ctx: CudaContext, shape, dtype: DType) -> "UnifiedTensor":
        return UnifiedTensor._alloc(ctx, shape, dtype)

    @staticmethod
    def zeros(ctx: CudaContext, shape) -> "UnifiedTensor":
        return UnifiedTensor._alloc(ctx, shape, DType.F32, zero=True)

    @staticmethod
    def from_bytes(ctx: CudaContext, data: bytes, shape) -> "UnifiedTensor":
        """Raw 32-bit words (the reference uploads u32 targets this way)."""
        assert len(data) == _numel(shape) * 4
        t = UnifiedTensor._alloc(ctx, shape, DType.U32)
        t.write_data(ctx, data)
        return t

    @staticmethod
    def from_f32_as_f16(ctx: CudaContext, data, shape) -> "UnifiedTensor":
        host = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        assert host.size == _numel(shape)
        t = UnifiedTensor._alloc(ctx, shape, DType.FP16)
        call("ft_upload_f32_as_f16", ctx.handle, t.ptr, host.ctypes.data_as(C.c_void_p), host.size)
        ctx.uploads += 1
        return t

    @staticmethod
    def from_f32_transposed(ctx: CudaContext, data, shape, dtype: DType = DType.F32):
        """`data` is [rows, cols] = `shape`; the tensor holds its transpose [cols, rows]."""
        rows, cols = shape
        host = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(rows, cols))
        t = UnifiedTensor._alloc(ctx, [cols, rows], dtype)
        call("ft_upload_f32_transposed", ctx.handle, t.ptr, host.ctypes.data_as(C.c_void_p),
             rows, cols, 1 if dtype is DType.FP16 else 0)
        ctx.uploads += 1
        return t

    # -- access ---------------------------------------------------------------------------
    @property
    def ptr(self) -> C.c_void_p:
        return C.c_void_p(self.storage.data_ptr())

    def numel(self) -> int:
        return _numel(self.shape)

    def size_in_bytes(self) -> int:
        return self.numel() * self.dtype.size_bytes()

    def reshaped(self, new_shape) -> "UnifiedTensor":
        assert _numel(new_shape) == self.numel(), "reshaped: element count differs"
        return UnifiedTensor(self.storage, new_shape, self.dtype)

    def write_data(self, ctx: CudaContext, data: bytes) -> None:
        assert len(data) <= self.storage.numel(), "write_data: buffer too small"
        buf = (C.c_char * len(data)).from_buffer_copy(data)
        call("ft_upload", ctx.handle, self.ptr, buf, len(data))
        ctx.uploads += 1

    def to_vec(self, ctx: CudaContext) -> np.ndarray:
        """Read back as f32 (f16 tensors are widened), waiting for the device."""
        n = self.numel()
        if self.dtype is DType.FP16:
            host = np.empty(n, dtype=np.float16)
        elif self.dtype is DType.U32:
            host = np.empty(n, dtype=np.uint32)
        else:
            host = np.empty(n, dtype=np.float32)
        call("ft_download", ctx.handle, host.ctypes.data_as(C.c_void_p), self.ptr, host.nbytes)
        ctx.readbacks += 1
        return host.astype(np.float32) if self.dtype is DType.FP16 else host


class AttentionOptions:
    """engine/attention.rs:581-594"""

    def __init__(self, causal=False, causal_offset=0, window=0, dropout_prob=0.0, seed=0):
        self.causal = causal
        self.causal_offset = causal_offset
        self.window = window
        self.dropout_prob = dropout_prob
        self.seed = seed


class AdamParams:
    """engine/training.rs:15-32"""

    def __init__(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, t=1.0):
        self.lr, self.beta1, self.beta2 = lr, beta1, beta2
        self.eps, self.weight_decay, self.t = eps, weight_decay, t

    def c(self) -> FtAdamParams:
        return FtAdamParams(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.t)


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise FtError(1, msg)


class ComputeEngine:
    """The kernel methods the LoRA step calls (ferrotensor-backend/src/engine/*.rs)."""

    def __init__(self, ctx: CudaContext):
        self.ctx = ctx

    # ---- matmul.rs:94-156
    def matmul(self, ctx, a, b, out):
        m, k, n = a.shape[0], a.shape[1], b.shape[1]
        _require(b.shape[0] == k and out.numel() == m * n, "matmul: shape mismatch")
        call("ft_matmul", ctx.handle, a.ptr, b.ptr, out.ptr, m, k, n)

    def matmul_bt(self, ctx, a, b, out):
        m, k, n = a.shape[0], a.shape[1], b.shape[0]
        _require(b.shape[1] == k and out.numel() == m * n, "matmul_bt: shape mismatch")
        call("ft_matmul_bt", ctx.handle, a.ptr, b.ptr, out.ptr, m, k, n)

    def matmul_at(self, ctx, a, b, out):
        m, k, n = a.shape[1], a.shape[0], b.shape[1]
        _require(b.shape[0] == k and out.numel() == m * n, "matmul_at: shape mismatch")
        call("ft_matmul_at", ctx.handle, a.ptr, b.ptr, out.ptr, m, k, n)

    def matmul_f16b(self, ctx, a, b, out):
        _require(b.dtype is DType.FP16, "matmul_f16b: b must be FP16")
        m, k, n = a.shape[0], a.shape[1], b.shape[1]
        _require(b.shape[0] == k and out.numel() == m * n, "matmul_f16b: shape mismatch")
        call("ft_matmul_f16b", ctx.handle, a.ptr, b.ptr, out.ptr, m, k, n)

    def matmul_bt_f16b(self, ctx, a, b, out):
        _require(b.dtype is DType.FP16, "matmul_bt_f16b: b must be FP16")
        m, k, n = a.shape[0], a.shape[1], b.shape[0]
        _require(b.shape[1] == k and out.numel() == m * n, "matmul_bt_f16b: shape mismatch")
        call("ft_matmul_bt_f16b", ctx.handle, a.ptr, b.ptr, out.ptr, m, k, n)

    # ---- attention.rs:15-83
    def _rotate(self, ctx, tensor, head_dim, pos, theta, inverse):
        shape = tensor.shape
        if len(shape) <= 1:
            seq_len, tokens = 1, 1
        elif len(shape) == 2:
            seq_len, tokens = shape[0], shape[0]
        else:
            seq_len, tokens = shape[1], shape[0] * shape[1]
        total = tensor.numel()
        heads = total // max(tokens * head_dim, 1)
        call("ft_rope_theta", ctx.handle, tensor.ptr, total, head_dim, seq_len, heads, pos,
             float(theta), 1 if inverse else 0)

    def rope(self, ctx, tensor, head_dim, pos):
        self._rotate(ctx, tensor, head_dim, pos, 10000.0, False)

    def rope_theta(self, ctx, tensor, head_dim, pos, theta):
        self._rotate(ctx, tensor, head_dim, pos, theta, False)

    def rope_theta_inverse(self, ctx, tensor, head_dim, pos, theta):
        self._rotate(ctx, tensor, head_dim, pos, theta, True)

    # ---- norm.rs:9-99
    def rms_norm(self, ctx, x, w, out):
        self.rms_norm_eps(ctx, x, w, out, 1e-5)

    def rms_norm_eps(self, ctx, x, w, out, eps):
        size = x.shape[-1]
        _require(w.numel() == size and out.numel() == x.numel(), "rms_norm: shape mismatch")
        call("ft_rms_norm_eps", ctx.handle, x.ptr, w.ptr, out.ptr, x.numel() // size, size,
             float(eps))

    def rms_norm_backward(self, ctx, x, w, grad_out, grad_x, grad_w, eps):
        size = x.shape[-1]
        _require(grad_out.numel() == x.numel() and grad_x.numel() == x.numel(),
                 "rms_norm_backward: shape mismatch")
        gw = grad_w.ptr if grad_w is not None else None
        call("ft_rms_norm_backward", ctx.handle, x.ptr, w.ptr, grad_out.ptr, grad_x.ptr, gw,
             x.numel() // size, size, float(eps))

    # ---- elementwise.rs, training.rs:161-205, mod.rs:399-428
    def add(self, ctx, a, b, out):
        _require(a.numel() == b.numel() == out.numel(), "add: shape mismatch")
        call("ft_add", ctx.handle, a.ptr, b.ptr, out.ptr, a.numel())

    def add_backward(self, ctx, grad_out, grad_a, grad_b):
        call("ft_add_backward", ctx.handle, grad_out.ptr, grad_a.ptr, grad_b.ptr, grad_out.numel())

    def gradient_scale(self, ctx, grad, scale):
        call("ft_gradient_scale", ctx.handle, grad.ptr, grad.numel(), float(scale))

    def clip_grad_by_norm(self, ctx, grad, scale):
        call("ft_clip_grad_by_norm", ctx.handle, grad.ptr, grad.numel(), float(scale))

    def copy_tensor(self, ctx, src, dst, dst_offset_bytes=0):
        _require(src.size_in_bytes() + dst_offset_bytes <= dst.size_in_bytes(),
                 "copy_tensor: destination too small")
        call("ft_copy", ctx.handle, src.ptr, dst.ptr, dst_offset_bytes, src.size_in_bytes())

    def silu_gate_fused(self, ctx, up, gate, out):
        """out = silu(up) * gate - the first operand goes through SiLU."""
        _require(up.numel() == gate.numel() == out.numel(), "silu_gate_fused: shape mismatch")
        call("ft_silu_gate_fused", ctx.handle, up.ptr, gate.ptr, out.ptr, out.numel())

    def silu_gate_backward(self, ctx, up, gate, grad_out, grad_up, grad_gate):
        call("ft_silu_gate_backward", ctx.handle, up.ptr, gate.ptr, grad_out.ptr, grad_up.ptr,
             grad_gate.ptr, grad_out.numel())

    # ---- attention.rs:139-441
    @staticmethod
    def _attn_params(q, k, opts: AttentionOptions, lse_saved=False, mask=None) -> FtAttnParams:
        _require(len(q.shape) == 4 and len(k.shape) == 4, "attention: q and k must be 4-D")
        b, sq, h, d = q.shape
        _, sk, hkv, _ = k.shape
        seed = int(opts.seed) & 0xFFFFFFFFFFFFFFFF
        strides = [0, 0, 0, 0]
        if mask is not None and len(mask.shape) == 4:
            # broadcast strides of a [batch, heads, seq_q, seq_k] mask: size-1 dimensions get 0
            mb, mh, mq, mk = mask.shape
            for dim, want, name in ((mb, b, "batch"), (mh, h, "heads"), (mq, sq, "seq_q"), (mk, sk, "seq_k")):
                _require(dim in (1, want), f"attention mask: {name} dimension is {dim}, expected 1 or {want}")
            strides = [mk * mq * mh if mb > 1 else 0, mk * mq if mh > 1 else 0, mk if mq > 1 else 0,
                       1 if mk > 1 else 0]
        return FtAttnParams(b, h, sq, sk, d, hkv, 1 if opts.causal else 0, opts.causal_offset,
                            opts.window, 0.0, float(opts.dropout_prob), 1 if lse_saved else 0,
                            seed & 0xFFFFFFFF, seed >> 32, (C.c_uint32 * 4)(*strides))

    def flash_attention_v2(self, ctx, q, k, v, out, causal, dropout_prob=0.0, seed=0, mask=None):
        """attention.rs:112-135: the positional form."""
        self.flash_attention_v2_with(ctx, q, k, v, out,
                                     AttentionOptions(causal=causal, dropout_prob=dropout_prob, seed=seed), mask)

    def flash_attention_v2_with(self, ctx, q, k, v, out, opts, mask=None):
        p = self._attn_params(q, k, opts, mask=mask)
        call("ft_flash_attention_v2", ctx.handle, q.ptr, k.ptr, v.ptr, out.ptr, None,
             mask.ptr if mask is not None else None, C.byref(p))

    def flash_attention_v2_with_stats(self, ctx, q, k, v, out, stats, opts, mask=None):
        p = self._attn_params(q, k, opts, mask=mask)
        _require(stats.numel() == p.batch * p.heads * p.seq_q * 2, "attention: stats size")
        call("ft_flash_attention_v2", ctx.handle, q.ptr, k.ptr, v.ptr, out.ptr, stats.ptr,
             mask.ptr if mask is not None else None, C.byref(p))

    def flash_attention_v2_backward_with(self, ctx, q, k, v, out, grad_out, grad_q, grad_k,
                                         grad_v, opts, mask=None):
        p = self._attn_params(q, k, opts, mask=mask)
        call("ft_flash_attention_v2_backward", ctx.handle, q.ptr, k.ptr, v.ptr, out.ptr,
             grad_out.ptr, grad_q.ptr, grad_k.ptr, grad_v.ptr, None,
             mask.ptr if mask is not None else None, C.byref(p))

    def flash_attention_v2_backward_with_stats(self, ctx, q, k, v, out, grad_out, grad_q, grad_k,
                                               grad_v, stats, opts, mask=None):
        p = self._attn_params(q, k, opts, lse_saved=True, mask=mask)
        call("ft_flash_attention_v2_backward", ctx.handle, q.ptr, k.ptr, v.ptr, out.ptr,
             grad_out.ptr, grad_q.ptr, grad_k.ptr, grad_v.ptr, stats.ptr,
             mask.ptr if mask is not None else None, C.byref(p))

    # ---- training.rs:54-77,207-290
    def masked_cross_entropy(self, ctx, logits, targets, grad, row_loss):
        rows = logits.numel() // logits.shape[-1]
        ones = UnifiedTensor.new(ctx, np.ones(rows, dtype=np.float32), [rows])
        self.masked_cross_entropy_weighted(ctx, logits, targets, ones, grad, row_loss)

    def masked_cross_entropy_weighted(self, ctx, logits, targets, weights, grad, row_loss):
        vocab = logits.shape[-1]
        rows = logits.numel() // vocab
        _require(targets.numel() == rows and weights.numel() == rows and
                 grad.numel() == logits.numel() and row_loss.numel() == rows,
                 "masked_cross_entropy: shape mismatch")
        call("ft_masked_cross_entropy_weighted", ctx.handle, logits.ptr, targets.ptr, weights.ptr,
             grad.ptr, row_loss.ptr, rows, vocab)

    # ---- misc.rs:20-34
    def argmax_rows(self, ctx, input, out_idx):
        n = input.shape[-1] if input.shape else 1
        n = max(n, 1)
        rows = input.numel() // n
        _require(out_idx.numel() == rows, "argmax_rows: one index per row")
        call("ft_argmax_rows", ctx.handle, input.ptr, out_idx.ptr, rows, n)

    def sum_squares_partial(self, ctx, x, out, offset) -> int:
        n = C.c_size_t()
        call("ft_sum_squares_partial", ctx.handle, x.ptr, x.numel(), out.ptr, offset, C.byref(n))
        return n.value

    def adamw_update(self, ctx, weight, grad, m, v, params: AdamParams):
        p = params.c()
        call("ft_adamw_update", ctx.handle, weight.ptr, grad.ptr, m.ptr, v.ptr, weight.numel(),
             C.byref(p))

    # ---- ferrotensor-autograd/src/lib.rs:1159-1179 (a host loop in the reference)
    def embedding_gather(self, ctx, table, ids, out):
        vocab, hidden = table.shape
        call("ft_embedding_gather", ctx.handle, table.ptr, ids.ptr, out.ptr, ids.numel(), vocab,
             hidden)
