"""ctypes binding of ``libpypto_b200.so`` (the C ABI declared in ``include/pypto_b200.h``).

There is no CPU fallback: if the library is missing or does not load, every
operator raises ``BackendUnavailable``.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libpypto_b200.so")


class BackendUnavailable(RuntimeError):
    """The CUDA library is not built / not loadable, or no CUDA device is present."""


class PtoError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[pypto_b200 status {status}] {message}")
        self.status = status


PTO_FP32, PTO_BF16, PTO_FP16, PTO_INT32, PTO_INT64, PTO_FP8E4M3, PTO_UINT8 = range(7)


class ChipTensor(C.Structure):
    _fields_ = [("addr", C.c_uint64), ("start_offset", C.c_uint64), ("shapes", C.c_uint32 * 5),
                ("ndims", C.c_uint32), ("dtype", C.c_uint32), ("reserved", C.c_uint32)]


class TaskArgs(C.Structure):
    _fields_ = [("tensors", C.POINTER(ChipTensor)), ("n_tensors", C.c_uint32),
                ("scalars", C.POINTER(C.c_uint64)), ("n_scalars", C.c_uint32)]


_i, _i64, _sz, _p, _f = C.c_int, C.c_int64, C.c_size_t, C.c_void_p, C.c_float
_u64p, _i32p = C.POINTER(C.c_uint64), C.POINTER(C.c_int32)

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "pto_last_error": (C.c_char_p, []),
    "pto_version": (C.c_char_p, []),
    "pto_worker_create": (_i, [_i, C.POINTER(_p)]),
    "pto_worker_destroy": (_i, [_p]),
    "pto_malloc": (_i, [_p, _sz, _u64p]),
    "pto_free": (_i, [_p, C.c_uint64]),
    "pto_copy_to": (_i, [_p, C.c_uint64, _p, _sz]),
    "pto_copy_from": (_i, [_p, _p, C.c_uint64, _sz]),
    "pto_copy_to_async": (_i, [_p, C.c_uint64, _p, _sz]),
    "pto_copy_from_async": (_i, [_p, _p, C.c_uint64, _sz]),
    "pto_synchronize": (_i, [_p]),
    "pto_worker_stream": (_p, [_p]),
    "pto_device_status": (_i, [_p, _i32p]),
    "pto_worker_scratch": (_i, [_p, _sz, _u64p, C.POINTER(_sz)]),
    "pto_register_callable": (_i, [_p, C.c_char_p, _i32p]),
    "pto_unregister_callable": (_i, [_p, C.c_int32]),
    "pto_run": (_i, [_p, C.c_int32, C.POINTER(TaskArgs)]),
    "pto_op_list": (C.POINTER(C.c_char), []),
    "pto_register_kernel_image": (_i, [_p, _p, _sz, C.c_char_p, _i32p]),
    "pto_run_kernel": (_i, [_p, C.c_int32, C.POINTER(TaskArgs), C.c_uint32, C.c_uint32]),
    "pto_paged_attention_scratch_bytes": (_sz, [_i, _i, _i, _i]),
    "pto_paged_attention": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _f, _p, _sz, _p]),
    "pto_paged_attention_static": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _i64, _i, _f, _p, _p]),
    "pto_pack_weight": (_i, [_p, _i, _p, _i, _i, _p]),
    "pto_cast": (_i, [_p, _i, _p, _i, _i64, _p]),
    "pto_cast_zero": (_i, [_p, _i, _p, _i, _i64, _p, _sz, _p]),
    "pto_linear": (_i, [_p, _p, _p, _i, _i, _i, _i, _p, _p]),
    "pto_ffn_swiglu_workspace_bytes": (_sz, [_i, _i]),
    "pto_ffn_swiglu": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p, _sz, _i, _p, _p]),
    "pto_ffn_act_workspace_bytes": (_sz, [_i, _i]),
    "pto_ffn_act": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _i, C.c_float, _p, _sz, _i, _p, _p]),
    "pto_ffn_swiglu_f32_workspace_bytes": (_sz, [_i, _i, _i]),
    "pto_ffn_swiglu_f32": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p, _sz, _i, _p, _p]),
    "pto_rms_norm": (_i, [_p, _i, _p, _p, _i, _i64, _i, _f, _p]),
    "pto_rms_norm_ex": (_i, [_p, _i, _p, _p, _i, _i64, _i, _f, _p, _p, _sz, _p]),
    "pto_rope_kv_append": (_i, [_p, _p, _p, _p, _i, _p, _i, _p, _p, _p, _i, _i, _i, _i, _i, _i64, _p, _p]),
    "pto_swiglu_act": (_i, [_p, _p, _i64, _i, _p]),
    "pto_llama_mini": (_i, [_p] * 13 + [_i, _i, _i, _p]),
    "pto_set_trace": (_i, [_i]),
    "pto_get_trace": (_i, []),
    "pto_last_run_ms": (_i, [_p, C.POINTER(C.c_float)]),
    "pto_moe_topk": (_i, [_p, _p, _i, _i, _i, _i, _p, _p, _p]),
    "pto_quantize_rows": (_i, [_p, _i, _p, _p, _i64, _i, _p]),
    "pto_moe_dispatch_plan": (_i, [_p, _i, _i, _p, _p, _p, _p, _p, _p, _p]),
    "pto_moe_recv_plan": (_i, [_p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "pto_moe_gather_rows": (_i, [C.POINTER(_p), C.POINTER(_p), C.POINTER(_i), _i, _p, _i, _i64, _i64, _p, _p]),
    "pto_moe_move_rows": (_i, [C.POINTER(_p), C.POINTER(_i64), C.POINTER(_p), C.POINTER(_i64), C.POINTER(_i), _i, _p,
                               _i, _i64, _i64, _p, _p]),
    "pto_moe_gather_f32": (_i, [_p, _p, _i64, _i64, _p, _p, _p]),
    "pto_scale_rows": (_i, [_p, _p, _i, _p, _i, _i64, _i, _p, _p]),
    "pto_moe_expert_gemm": (_i, [_i, _p, _p, _i, _i, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p]),
    "pto_moe_combine": (_i, [_p, _p, _p, _i, _i, _i, _i64, _p, _p, _p]),
    "pto_moe_push_rows": (_i, [_p, _i, _p, _i, _i, _p, _p, _p, _i, _i, _i64, _i64, _p, _p, _p]),
    "pto_moe_wait_flags": (_i, [_p, _i, _i, _p, _p]),
    "pto_matmul_mx": (_i, [_p, _p, _i, _p, _p, _i, _p, _p, _i, _i, _i, _p, _p]),
    "pto_transpose_u8": (_i, [_p, _p, _i64, _i64, _p]),
    "pto_comm_unique_id": (_i, [_p]),
    "pto_comm_init": (_i, [_i, _i, _p, _i, C.POINTER(_p)]),
    "pto_comm_destroy": (_i, [_p]),
    "pto_comm_rank": (_i, [_p]),
    "pto_comm_size": (_i, [_p]),
    "pto_comm_nccl_version": (_i, []),
    "pto_all_to_all": (_i, [_p, _p, _p, _sz, _p]),
    "pto_all_to_all_v": (_i, [_p, _p, C.POINTER(_i64), _p, C.POINTER(_i64), _sz, _p]),
    "pto_paged_gather": (_i, [_p, _i64, _i64, _i, _p, _i64, _p, _i64, _i, _i64, _i64, _p, _p, _p]),
}

class MoeLayerDesc(C.Structure):
    _fields_ = [("hidden", C.c_int), ("inter", C.c_int), ("n_experts", C.c_int), ("topk", C.c_int),
                ("max_tokens", C.c_int), ("gate_packed", C.c_void_p), ("bias", C.c_void_p), ("w_gu", C.c_void_p),
                ("s_gu", C.c_void_p), ("w_d", C.c_void_p), ("s_d", C.c_void_p), ("sh_w_gu", C.c_void_p),
                ("sh_s_gu", C.c_void_p), ("sh_w_d", C.c_void_p), ("sh_s_d", C.c_void_p), ("comm", C.c_void_p)]


SIGNATURES.update({
    "pto_moe_layer_create": (_i, [C.POINTER(MoeLayerDesc), C.POINTER(_p)]),
    "pto_moe_layer_destroy": (_i, [_p]),
    "pto_moe_layer_forward": (_i, [_p, _p, _i, _p, _p, _p, _p, _p, C.POINTER(C.c_float), _p]),
    "pto_moe_layer_status": (_i, [_p, _i32p, _p]),
    "pto_moe_layer_peer_exchange": (_i, [_p]),
})

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Load the library once; raise BackendUnavailable if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise BackendUnavailable(
                f"{LIB_PATH} is missing: build it with `python -m pypto_b200.build` "
                "(there is no CPU fallback)")
        try:
            lib = C.CDLL(LIB_PATH)
        except OSError as e:  # pragma: no cover - depends on the machine
            raise BackendUnavailable(f"cannot load {LIB_PATH}: {e}") from e
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the export is missing
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise PtoError(status, load().pto_last_error().decode(errors="replace"))


def op_names() -> list[str]:
    raw = load().pto_op_list()
    names, cur, i = [], bytearray(), 0
    while True:
        c = raw[i]
        i += 1
        if c == b"\0":
            if not cur:
                break
            names.append(cur.decode())
            cur = bytearray()
        else:
            cur += c
    return names
