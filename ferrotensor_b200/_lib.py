"""ctypes binding of libft_cuda.so (declared in include/ft_cuda.h).

The library is the product: there is no fallback.  If it is missing, or a call fails,
an exception is raised.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libft_cuda.so"

FT_OK = 0
FT_MASKED_CE_SKIP = 0xFFFFFFFF
FT_SUM_SQUARES_CHUNK = 4096
FT_GEMM_F32, FT_GEMM_F16, FT_GEMM_F16X2 = 0, 1, 2
FT_LINEARS = 7
FT_ERR_COMM = 5
FT_COMM_ID_BYTES = 128


class FtError(RuntimeError):
    """A libft_cuda call returned non-zero (the reference would have panicked)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libft_cuda error {code}: {message}")
        self.code = code


class FtAttnParams(C.Structure):
    _fields_ = [
        ("batch", C.c_uint32), ("heads", C.c_uint32), ("seq_q", C.c_uint32),
        ("seq_k", C.c_uint32), ("head_dim", C.c_uint32), ("kv_heads", C.c_uint32),
        ("causal", C.c_uint32), ("causal_offset", C.c_uint32), ("window", C.c_uint32),
        ("scale", C.c_float), ("dropout_prob", C.c_float), ("lse_saved", C.c_uint32),
        ("seed_lo", C.c_uint32), ("seed_hi", C.c_uint32), ("mask_stride", C.c_uint32 * 4),
    ]


class FtAdamParams(C.Structure):
    _fields_ = [
        ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
        ("weight_decay", C.c_float), ("t", C.c_float), ("_pad", C.c_float * 2),
    ]


class FtModelConfig(C.Structure):
    _fields_ = [
        ("vocab", C.c_int), ("hidden", C.c_int), ("layers", C.c_int), ("heads", C.c_int),
        ("kv_heads", C.c_int), ("head_dim", C.c_int), ("ffn", C.c_int),
        ("eps", C.c_float), ("theta", C.c_float),
        ("qkv_bias", C.c_int), ("lora_rank", C.c_int), ("lora_alpha", C.c_float),
        ("lora_mask", C.c_int), ("lora_head", C.c_int), ("f16_base", C.c_int),
        ("checkpoint_blocks", C.c_int), ("attention_dropout", C.c_float),
    ]


_P = C.c_void_p
_I = C.c_int
_Z = C.c_size_t
_F = C.c_float

# name -> argtypes; every function returns int except the two string getters
PROTOTYPES = {
    "ft_ctx_create": [_I, _P, C.POINTER(_P)],
    "ft_ctx_destroy": [_P],
    "ft_ctx_flush": [_P],
    "ft_ctx_synchronize": [_P],
    "ft_ctx_status": [_P, C.POINTER(_I)],
    "ft_ctx_debug_words": [_P, C.POINTER(_I)],
    "ft_ctx_profile": [_P, _I],
    "ft_ctx_profile_report": [_P, C.c_char_p, _Z],
    "ft_ctx_profile_read": [_P, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_uint64)],
    "ft_ctx_profile_read_fused": [_P, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_uint64)],
    "ft_ctx_profile_bytes": [_P, C.POINTER(C.c_double)],
    "ft_ctx_set_gemm_mode": [_P, _I],
    "ft_ctx_set_gemm_tile_m": [_P, _I],
    "ft_ctx_launch_count": [_P, C.POINTER(C.c_uint64)],
    "ft_tensor_alloc": [_P, _Z, C.POINTER(_P)],
    "ft_tensor_free": [_P, _P],
    "ft_tensor_zero": [_P, _P, _Z],
    "ft_upload": [_P, _P, _P, _Z],
    "ft_download": [_P, _P, _P, _Z],
    "ft_upload_f32_as_f16": [_P, _P, _P, _Z],
    "ft_upload_f32_transposed": [_P, _P, _P, _Z, _Z, _I],
    "ft_convert_f32_to_f16": [_P, _P, _P, _Z],
    "ft_transpose_f32": [_P, _P, _P, _Z, _Z, _I],
    "ft_matmul": [_P, _P, _P, _P, _I, _I, _I],
    "ft_matmul_bt": [_P, _P, _P, _P, _I, _I, _I],
    "ft_matmul_at": [_P, _P, _P, _P, _I, _I, _I],
    "ft_matmul_f16b": [_P, _P, _P, _P, _I, _I, _I],
    "ft_matmul_bt_f16b": [_P, _P, _P, _P, _I, _I, _I],
    "ft_rope_theta": [_P, _P, _Z, _I, _I, _I, _I, _F, _I],
    "ft_rms_norm_eps": [_P, _P, _P, _P, _I, _I, _F],
    "ft_rms_norm_backward": [_P, _P, _P, _P, _P, _P, _I, _I, _F],
    "ft_rms_norm_backward_noalloc": [_P, _P, _P, _P, _P, _P, _I, _I, _F],
    "ft_add": [_P, _P, _P, _P, _Z],
    "ft_add_backward": [_P, _P, _P, _P, _Z],
    "ft_gradient_scale": [_P, _P, _Z, _F],
    "ft_copy": [_P, _P, _P, _Z, _Z],
    "ft_silu_gate_fused": [_P, _P, _P, _P, _Z],
    "ft_silu_gate_backward": [_P, _P, _P, _P, _P, _P, _Z],
    "ft_flash_attention_v2": [_P, _P, _P, _P, _P, _P, _P, C.POINTER(FtAttnParams)],
    "ft_flash_attention_v2_backward": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                       C.POINTER(FtAttnParams)],
    "ft_masked_cross_entropy_weighted": [_P, _P, _P, _P, _P, _P, _I, _I],
    "ft_sum_squares_partial": [_P, _P, _Z, _P, _Z, C.POINTER(_Z)],
    "ft_clip_grad_by_norm": [_P, _P, _Z, _F],
    "ft_adamw_update": [_P, _P, _P, _P, _P, _Z, C.POINTER(FtAdamParams)],
    "ft_embedding_gather": [_P, _P, _P, _P, _I, _I, _I],
    "ft_argmax_rows": [_P, _P, _P, _I, _I],
    "ft_model_create": [_P, C.POINTER(FtModelConfig), C.POINTER(_P)],
    "ft_model_destroy": [_P],
    "ft_model_trainable_count": [_P, C.POINTER(_Z)],
    "ft_model_adapter_offset": [_P, _I, _I, _I, C.POINTER(_Z), C.POINTER(_I), C.POINTER(_I)],
    "ft_model_set_embedding": [_P, _P, _P, _P],
    "ft_model_set_layer": [_P, _I, _P, _P, C.POINTER(_P), C.POINTER(_P)],
    "ft_model_set_state": [_P, _P, _P, _P, _P],
    "ft_model_prepare": [_P],
    "ft_model_params_changed": [_P],
    "ft_model_workspace_bytes": [_P, _I, _I, C.POINTER(_Z)],
    "ft_model_set_workspace": [_P, _P, _Z],
    "ft_model_forward_backward": [_P, _P, _P, _P, _I, _I, _F, _P, _P],
    "ft_model_forward_loss": [_P, _P, _P, _P, _I, _I, _P, _P],
    "ft_model_set_dropout_seed": [_P, C.c_uint64],
    "ft_model_zero_grad": [_P],
    "ft_model_apply_gradients": [_P, _F, _F, C.POINTER(FtAdamParams), _P],
    "ft_comm_unique_id": [_P],
    "ft_comm_create": [_P, _I, _I, _P, _I, C.POINTER(_P)],
    "ft_comm_destroy": [_P],
    "ft_comm_info": [_P, C.POINTER(_I), C.POINTER(_I)],
    "ft_comm_allreduce_sum": [_P, _P, _Z],
    "ft_comm_wait": [_P, _I],
    "ft_model_allreduce_apply_gradients": [_P, _P, _F, C.POINTER(FtAdamParams), _P],
}
STRING_GETTERS = ("ft_last_error", "ft_build_info")

_lib = None


def load() -> C.CDLL:
    """Load libft_cuda.so and declare every prototype.  Raises if the library is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FtError(-1, f"{LIB_PATH} is missing: build it with "
                          "`python -m ferrotensor_b200._build` (needs nvcc)")
    lib = C.CDLL(str(LIB_PATH))
    for name, args in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    for name in STRING_GETTERS:
        fn = getattr(lib, name)
        fn.argtypes = []
        fn.restype = C.c_char_p
    _lib = lib
    return lib


def last_error() -> str:
    return load().ft_last_error().decode(errors="replace")


def check(code: int) -> None:
    if code != FT_OK:
        raise FtError(code, last_error())


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise FtError on failure."""
    check(getattr(load(), name)(*args))
