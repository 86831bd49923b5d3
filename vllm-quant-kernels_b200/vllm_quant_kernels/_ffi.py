"""ctypes binding of libvqk.so (the C ABI declared in include/vqk.h).

The library is the only compute path: if it is missing or the device is not a
B200 the calls raise, nothing falls back to torch or to the CPU.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvqk.so")

MODE_W8A16, MODE_W8A8, MODE_FP8, MODE_MXFP8, MODE_MXFP4 = range(5)
F16, BF16, F32 = range(3)
RECORD_BYTES = 1024
RECORD_CAP = 126
COMM_ID_BYTES = 128
PEER_HANDLE_BYTES = 64
PEER_MAX_RANKS = 8
STATIC_MAX_ROWS = 64
STATIC_MAX_VOCAB = 262144

# every symbol include/vqk.h declares
SYMBOLS = (
    "vqk_version", "vqk_strerror", "vqk_last_cuda_error", "vqk_device_error", "vqk_device_error_clear",
    "vqk_quantize_weight", "vqk_quantize_act",
    "vqk_lm_head_create", "vqk_lm_head_destroy", "vqk_lm_head_workspace_bytes", "vqk_lm_head_forward",
    "vqk_lm_head_set_kernel_events", "vqk_lm_head_set_debug_times", "vqk_lm_head_set_post_ops",
    "vqk_sample_workspace_bytes", "vqk_sample", "vqk_sample_static", "vqk_sample_finalize", "vqk_topk_threshold",
    "vqk_comm_unique_id", "vqk_comm_create", "vqk_comm_allgather", "vqk_comm_destroy",
    "vqk_peer_create", "vqk_peer_connect", "vqk_peer_connect_pointers", "vqk_peer_local_buffer",
    "vqk_peer_set_wait_limit", "vqk_lm_head_step_sharded_workspace_bytes", "vqk_lm_head_step_sharded",
    "vqk_lm_head_step_host_workspace_bytes", "vqk_lm_head_step_host",
    "vqk_peer_exchange_finalize", "vqk_peer_destroy",
)


class VqkError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"libvqk: {what} (status {status})")


class SampleParams(ctypes.Structure):
    """vqk_sample_params"""
    _fields_ = [
        ("temperature", c_void_p), ("seeds", c_void_p), ("top_k", c_void_p), ("top_p", c_void_p),
        ("topk_threshold", c_void_p), ("vocab_offset", c_int64), ("vocab_total", c_int64),
        ("logprobs", c_void_p),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is not built. Run `python vllm-quant-kernels_b200/build.py` "
            "(nvcc, sm_100a). There is no Triton, torch or CPU fallback for these operators.")
    L = ctypes.CDLL(LIB_PATH)
    L.vqk_version.restype = c_int
    L.vqk_strerror.restype = c_char_p
    L.vqk_strerror.argtypes = [c_int]
    L.vqk_last_cuda_error.restype = c_int
    L.vqk_device_error.restype = c_int
    L.vqk_quantize_weight.argtypes = [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    L.vqk_quantize_act.argtypes = [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    L.vqk_lm_head_create.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64, POINTER(c_void_p)]
    L.vqk_lm_head_destroy.argtypes = [c_void_p]
    L.vqk_lm_head_workspace_bytes.restype = c_int64
    L.vqk_lm_head_workspace_bytes.argtypes = [c_void_p, c_int64, c_int]
    L.vqk_lm_head_forward.argtypes = [
        c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, POINTER(SampleParams),
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    L.vqk_lm_head_set_kernel_events.argtypes = [c_void_p, c_void_p, c_void_p]
    L.vqk_lm_head_set_debug_times.argtypes = [c_void_p, c_void_p]
    L.vqk_lm_head_set_post_ops.argtypes = [c_void_p, c_float, c_float]
    L.vqk_sample_workspace_bytes.restype = c_int64
    L.vqk_sample_workspace_bytes.argtypes = [c_int64, c_int64]
    L.vqk_sample.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int64, POINTER(SampleParams), c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int64, c_void_p]
    L.vqk_sample_static.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int64, POINTER(SampleParams), c_void_p, c_void_p,
                                    c_void_p]
    L.vqk_sample_finalize.argtypes = [c_void_p, c_int, c_int64, POINTER(SampleParams), c_void_p, c_void_p, c_void_p]
    L.vqk_topk_threshold.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    L.vqk_comm_unique_id.argtypes = [c_void_p]
    L.vqk_comm_create.argtypes = [c_void_p, c_int, c_int, POINTER(c_void_p)]
    L.vqk_comm_allgather.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    L.vqk_comm_destroy.argtypes = [c_void_p]
    L.vqk_peer_create.argtypes = [c_int, c_int, c_int64, POINTER(c_void_p), c_void_p]
    L.vqk_peer_connect.argtypes = [c_void_p, c_void_p]
    L.vqk_peer_exchange_finalize.argtypes = [c_void_p, c_void_p, c_int64, POINTER(SampleParams), c_void_p, c_void_p,
                                             c_void_p]
    L.vqk_peer_destroy.argtypes = [c_void_p]
    L.vqk_device_error_clear.restype = c_int
    L.vqk_peer_connect_pointers.argtypes = [c_void_p, POINTER(c_void_p)]
    L.vqk_peer_local_buffer.restype = c_void_p
    L.vqk_peer_local_buffer.argtypes = [c_void_p]
    L.vqk_peer_set_wait_limit.argtypes = [c_void_p, c_int64]
    L.vqk_lm_head_step_sharded_workspace_bytes.restype = c_int64
    L.vqk_lm_head_step_sharded_workspace_bytes.argtypes = [c_void_p, c_int64]
    L.vqk_lm_head_step_sharded.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, POINTER(SampleParams), c_void_p, c_void_p,
        c_void_p, c_int64, c_void_p]
    L.vqk_lm_head_step_host_workspace_bytes.restype = c_int64
    L.vqk_lm_head_step_host_workspace_bytes.argtypes = [c_void_p, c_int64]
    L.vqk_lm_head_step_host.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, POINTER(SampleParams), c_void_p, c_void_p,
        c_void_p, c_int64, c_void_p]
    for name in SYMBOLS:
        fn = getattr(L, name)
        if fn.restype is c_int and name not in ("vqk_version", "vqk_last_cuda_error", "vqk_device_error"):
            fn.restype = c_int
    _lib = L
    return L


def check(rc: int) -> None:
    if rc == 0:
        return
    L = lib()
    what = L.vqk_strerror(rc).decode()
    if rc == -3:
        what += f" (cudaError {L.vqk_last_cuda_error()})"
    raise VqkError(rc, what)
