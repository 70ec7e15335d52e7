"""ctypes binding of ``libcleave_b200.so`` (declared in ``include/cleave_b200.h``).

There is no fallback: if the shared library is missing or a launch fails, the call raises.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcleave_b200.so")

F16, BF16 = 0, 1
OK = 0
ERR_UNSUPPORTED = 2
ERR_DEVICE_TIMEOUT = 6


class Cb200Error(RuntimeError):
    """A C-ABI call returned a non-zero ``cb200_status``."""

    def __init__(self, status: int, message: str):
        super().__init__(f"cleave_b200: status {status}: {message}")
        self.status = status


class AttnDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("kv_indptr", C.c_void_p), ("kv_indices", C.c_void_p), ("kv_last_page_len", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("batch", C.c_int32), ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("page_size", C.c_int32), ("num_pages", C.c_int32),
        ("num_kv_indices", C.c_int32), ("kv_len", C.c_int32), ("q_rows", C.c_int32),
        ("dtype", C.c_int32), ("max_ctas", C.c_int32), ("sm_scale", C.c_float),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("w1", C.c_void_p), ("gamma", C.c_void_p), ("y", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("op", C.c_int32), ("dtype", C.c_int32),
        ("split_k", C.c_int32), ("max_ctas", C.c_int32), ("eps", C.c_float), ("addend", C.c_void_p), ("dependent_launch", C.c_int32),
        ("x2", C.c_void_p), ("w2", C.c_void_p), ("k2", C.c_int32), ("ldx", C.c_int32),
        ("ldy", C.c_int32), ("n_peers", C.c_int32), ("y_peers", C.c_void_p * 7),
    ]


class GemmPlanInfo(C.Structure):
    _fields_ = [("tile_m", C.c_int32), ("tile_n", C.c_int32), ("split", C.c_int32), ("kind", C.c_int32),
                ("grid", C.c_int32), ("estimate_us", C.c_float)]


class MlaPrefillArgs(C.Structure):
    _fields_ = [
        ("q_nope", C.c_void_p), ("q_pe", C.c_void_p), ("ckv_cache", C.c_void_p), ("kpe_cache", C.c_void_p),
        ("qo_indptr", C.c_void_p), ("kv_indptr", C.c_void_p), ("kv_indices", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("batch", C.c_int32), ("total_q", C.c_int32), ("num_heads", C.c_int32), ("ckv_dim", C.c_int32),
        ("kpe_dim", C.c_int32), ("num_pages", C.c_int32), ("num_kv_indices", C.c_int32), ("dtype", C.c_int32),
        ("sm_scale", C.c_float),
    ]


class SplitCombineArgs(C.Structure):
    _fields_ = [
        ("num", C.c_void_p), ("den", C.c_void_p), ("out", C.c_void_p), ("outer", C.c_int64), ("inner", C.c_int64),
        ("splits", C.c_int32), ("den_inner", C.c_int32), ("dtype", C.c_int32),
    ]


class AttnUnnormaliseArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p), ("lse", C.c_void_p), ("o_part", C.c_void_p), ("l_part", C.c_void_p),
        ("kv_heads", C.c_int32), ("group", C.c_int32), ("splits", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("shift", C.c_float),
    ]


class MatmulRowsumArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("y", C.c_void_p), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("dtype", C.c_int32),
    ]


class MatmulMatmulArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("q_len", C.c_int32), ("kv_len", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("impl", C.c_int32),
    ]


MM_IMPL = {"auto": 0, "scores_first": 1, "chain": 2}


class LoraArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("y", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("r", C.c_int32), ("dtype", C.c_int32),
    ]


GEMM_MATMUL, GEMM_RMSNORM, GEMM_SWIGLU = 0, 1, 2


class MlaDecodeArgs(C.Structure):
    _fields_ = [
        ("q_nope", C.c_void_p), ("q_pe", C.c_void_p), ("ckv_cache", C.c_void_p), ("kpe_cache", C.c_void_p),
        ("kv_indptr", C.c_void_p), ("kv_indices", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("ckv_dim", C.c_int32), ("kpe_dim", C.c_int32),
        ("page_size", C.c_int32), ("num_pages", C.c_int32), ("num_kv_indices", C.c_int32),
        ("kv_len", C.c_int32), ("dtype", C.c_int32), ("max_ctas", C.c_int32), ("impl", C.c_int32),
        ("sm_scale", C.c_float), ("kv_start", C.c_void_p), ("kv_lens", C.c_void_p),
    ]


class AttnPrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("q_len", C.c_int32), ("kv_len", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
        ("score_mode", C.c_int32), ("qk_norm", C.c_int32), ("norm_eps", C.c_float),
    ]


SCORE_SOFTMAX, SCORE_LINEAR = 0, 1


class AttnPrefillRaggedArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("qo_indptr", C.c_void_p), ("kv_indptr", C.c_void_p),
        ("kv_indices", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("batch", C.c_int32), ("total_q", C.c_int32), ("total_kv", C.c_int32),
        ("num_qo_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("dtype", C.c_int32),
        ("causal", C.c_int32), ("sm_scale", C.c_float), ("num_kv_indices", C.c_int32),
    ]


MLA_IMPL = {"auto": 0, "mma_sync": 1, "tcgen05": 2}

_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (``python -c 'import __graft_entry__ as g; g.build()'``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with cleave_b200/csrc/build.sh "
                "(there is no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        L.cb200_version.restype = C.c_int
        L.cb200_peer_scatter_cols.restype = C.c_int
        L.cb200_peer_scatter_cols.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]
        L.cb200_set_small_problem_limit.restype = C.c_int
        L.cb200_set_small_problem_limit.argtypes = [C.c_int]
        L.cb200_strerror.restype = C.c_char_p
        L.cb200_strerror.argtypes = [C.c_int]
        L.cb200_last_cuda_error.restype = C.c_int
        L.cb200_sm_count.restype = C.c_int
        L.cb200_workspace_status.restype = C.c_int
        L.cb200_workspace_status.argtypes = [C.c_void_p, C.c_void_p]
        L.cb200_attn_decode_workspace_bytes.restype = C.c_size_t
        L.cb200_attn_decode_workspace_bytes.argtypes = [C.POINTER(AttnDecodeArgs)]
        L.cb200_attn_decode.restype = C.c_int
        L.cb200_attn_decode.argtypes = [C.POINTER(AttnDecodeArgs), C.c_void_p]
        L.cb200_attn_decode_static_scratch_max_bytes.restype = C.c_size_t
        L.cb200_attn_decode_static_scratch.restype = C.c_int
        L.cb200_attn_decode_static_scratch.argtypes = [C.POINTER(AttnDecodeArgs), C.c_void_p]
        L.cb200_attn_decode_static_scratch_status.restype = C.c_int
        L.cb200_attn_decode_static_scratch_status.argtypes = [C.c_void_p]
        L.cb200_workspace_reset.restype = C.c_int
        L.cb200_workspace_reset.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.cb200_gemm_workspace_bytes.restype = C.c_size_t
        L.cb200_gemm_workspace_bytes.argtypes = [C.POINTER(GemmArgs)]
        L.cb200_gemm_effective_split.restype = C.c_int
        L.cb200_gemm_effective_split.argtypes = [C.POINTER(GemmArgs)]
        L.cb200_gemm_plan.restype = C.c_int
        L.cb200_gemm_plan.argtypes = [C.POINTER(GemmArgs), C.POINTER(GemmPlanInfo)]
        L.cb200_gemm.restype = C.c_int
        L.cb200_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        L.cb200_mla_prefill_workspace_bytes.restype = C.c_size_t
        L.cb200_mla_prefill_workspace_bytes.argtypes = [C.POINTER(MlaPrefillArgs)]
        L.cb200_mla_prefill.restype = C.c_int
        L.cb200_mla_prefill.argtypes = [C.POINTER(MlaPrefillArgs), C.c_void_p]
        L.cb200_split_combine.restype = C.c_int
        L.cb200_split_combine.argtypes = [C.POINTER(SplitCombineArgs), C.c_void_p]
        L.cb200_attn_unnormalise.restype = C.c_int
        L.cb200_attn_unnormalise.argtypes = [C.POINTER(AttnUnnormaliseArgs), C.c_void_p]
        L.cb200_matmul_rowsum_workspace_bytes.restype = C.c_size_t
        L.cb200_matmul_rowsum_workspace_bytes.argtypes = [C.POINTER(MatmulRowsumArgs)]
        L.cb200_matmul_rowsum.restype = C.c_int
        L.cb200_matmul_rowsum.argtypes = [C.POINTER(MatmulRowsumArgs), C.c_void_p]
        L.cb200_matmul_matmul_workspace_bytes.restype = C.c_size_t
        L.cb200_matmul_matmul_workspace_bytes.argtypes = [C.POINTER(MatmulMatmulArgs)]
        L.cb200_matmul_matmul_uses_chain.restype = C.c_int
        L.cb200_matmul_matmul_uses_chain.argtypes = [C.POINTER(MatmulMatmulArgs)]
        L.cb200_matmul_matmul.restype = C.c_int
        L.cb200_matmul_matmul.argtypes = [C.POINTER(MatmulMatmulArgs), C.c_void_p]
        L.cb200_lora_workspace_bytes.restype = C.c_size_t
        L.cb200_lora_workspace_bytes.argtypes = [C.POINTER(LoraArgs)]
        L.cb200_lora.restype = C.c_int
        L.cb200_lora.argtypes = [C.POINTER(LoraArgs), C.c_void_p]
        L.cb200_mla_decode_workspace_bytes.restype = C.c_size_t
        L.cb200_mla_decode_workspace_bytes.argtypes = [C.POINTER(MlaDecodeArgs)]
        L.cb200_mla_decode.restype = C.c_int
        L.cb200_mla_decode.argtypes = [C.POINTER(MlaDecodeArgs), C.c_void_p]
        L.cb200_attn_prefill_workspace_bytes.restype = C.c_size_t
        L.cb200_attn_prefill_workspace_bytes.argtypes = [C.POINTER(AttnPrefillArgs)]
        L.cb200_attn_prefill.restype = C.c_int
        L.cb200_attn_prefill.argtypes = [C.POINTER(AttnPrefillArgs), C.c_void_p]
        L.cb200_attn_prefill_ragged_workspace_bytes.restype = C.c_size_t
        L.cb200_attn_prefill_ragged_workspace_bytes.argtypes = [C.POINTER(AttnPrefillRaggedArgs)]
        L.cb200_attn_prefill_ragged.restype = C.c_int
        L.cb200_attn_prefill_ragged.argtypes = [C.POINTER(AttnPrefillRaggedArgs), C.c_void_p]
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        L = lib()
        msg = L.cb200_strerror(status).decode()
        if status == 5:
            msg += f" [cuda error {L.cb200_last_cuda_error()}]"
        raise Cb200Error(status, msg)
