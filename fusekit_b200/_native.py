"""ctypes binding of ``libfusekit_cuda.so`` (declared in ``include/fusekit_cuda.h``).

This is the module a FuseKit host imports in place of ``_fusekit_runtime_native``
(python_runtime/src/lib.rs:1939-1971).  It fails loudly when the library is missing
or a call returns an error; there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FUSEKIT_CUDA_LIB") or os.path.join(_HERE, "libfusekit_cuda.so")

(TASK_STEP_INIT, TASK_EMBED_LOOKUP_DECODE, TASK_RMSNORM_QKV, TASK_QK_NORM_ROPE_STORE, TASK_SDPA_DECODE,
 TASK_LINEAR_RESIDUAL, TASK_RMSNORM_GATEUP_ACT, TASK_FINAL_RMSNORM_LM_HEAD, TASK_ARGMAX_FINALIZE,
 TASK_ALLREDUCE, TASK_RESIDUAL_ADD, TASK_RMSNORM_ROWS, TASK_ROPE_STORE_ROWS, TASK_ARGMAX_ROWS, TASK_KV_STORE_QUANT,
 TASK_SDPA_DECODE_QUANT) = range(16)
ACT_SWIGLU, ACT_GEGLU_TANH = 0, 1


class RoleBinding(C.Structure):
    """Mirror of ``fk_role_binding``: one role string of a task graph and the address / weight id behind it."""
    _fields_ = [("role", C.c_char_p), ("value", C.c_uint64)]


class FusekitError(RuntimeError):
    pass


class Task(C.Structure):
    """Mirror of ``fk_task``: one entry of the per-token dispatch list."""
    _fields_ = [("kind", C.c_int32), ("layer", C.c_int32), ("buf", C.c_uint64 * 12),
                ("iarg", C.c_int32 * 8), ("farg", C.c_float * 4)]

    @staticmethod
    def make(kind: int, layer: int = -1, buf=None, iarg=None, farg=None) -> "Task":
        t = Task()
        t.kind, t.layer = kind, layer
        for i, v in (buf or {}).items():
            t.buf[i] = int(v or 0)
        for i, v in enumerate(iarg or []):
            t.iarg[i] = int(v)
        for i, v in enumerate(farg or []):
            t.farg[i] = float(v)
        return t


_lib = None


def lib():
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FusekitError(f"{LIB_PATH} is missing: run fusekit_b200.build.build() (nvcc, sm_100a); there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    u64, i64, i32, u32, f32, vp, sz = C.c_uint64, C.c_int64, C.c_int, C.c_uint32, C.c_float, C.c_void_p, C.c_size_t
    P = C.POINTER
    sig = {
        "fk_open": [i32, P(u64)], "fk_close": [u64], "fk_info": [u64, C.c_char_p, sz], "fk_kernel_names": [C.c_char_p, sz],
        "fk_alloc": [u64, sz, P(u64)], "fk_free": [u64, u64], "fk_upload": [u64, u64, vp, sz], "fk_download": [u64, vp, u64, sz],
        "fk_memset": [u64, u64, i32, sz], "fk_sync": [u64], "fk_kv_cache_alloc": [u64, i32, i32, i32, P(u64), P(u64)],
        "fk_weight_alloc": [u64, i64, i64, i32, P(u64)], "fk_weight_upload_rows": [u64, u64, i64, i64, vp, vp, vp],
        "fk_weight_synth_rows": [u64, u64, i64, i64, u64, f32, i64, i64, i64], "fk_weight_finalize": [u64, u64],
        "fk_weight_set_rows": [u64, u64, i32, i32, i32], "fk_weight_pair": [u64, u64, u64, P(u64)],
        "fk_weight_dequant": [u64, u64, i64, i64, vp], "fk_weight_nbytes": [u64, u64, P(u64)],
        "fk_synth_normal_bf16": [u64, u64, u64, u64, u64, f32, f32],
        "fk_launch": [u64, P(Task)], "fk_launch_batch": [u64, P(Task), i32], "fk_smoke": [u64, vp, vp, vp, i32],
        "fk_state_set": [u64, u32, u32], "fk_state_get": [u64, P(u32), P(u32), P(u32)],
        "fk_peer_arena_export": [u64, C.c_void_p, C.c_size_t], "fk_peer_arena_open": [u64, C.c_void_p, i32, i32],
        "fk_peer_arena_loopback": [u64, i32, i32, u32], "fk_peer_arena_close": [u64],
        "fk_graph_capture": [u64, P(Task), i32, P(u64)],
        "fk_comm_check": [u64],
        "fk_weight_plan": [u64, u64, P(i32), P(i32), P(i32)],
        "fk_tasks_from_json": [C.c_char_p, P(RoleBinding), i32, P(Task), i32, P(i32)],
        "fk_graph_capture_json": [u64, C.c_char_p, P(RoleBinding), i32, P(u64)], "fk_graph_launch": [u64, u64, P(C.c_double)],
        "fk_graph_launch_async": [u64, u64], "fk_wait": [u64, P(C.c_double)],
        "fk_graph_profile_nodes": [u64, u64, i32, P(C.c_double), i32, P(i32)], "fk_graph_node_count": [u64, u64, P(i32)],
        "fk_time_tasks": [u64, P(Task), i32, i32, P(C.c_double)],
        "fk_step": [u64, u64, u32, u32, P(u32), P(C.c_double)],
        "fk_decode_chunk": [u64, u64, u32, u32, i32, vp, P(C.c_double)],
        "fk_decode_chunk_host": [u64, u64, u32, u32, i32, vp, P(C.c_double)],
        "fk_decode_chunk_rows": [u64, u64, u32, vp, i32, i32, vp, P(C.c_double)],
        "fk_debug_timeline": [u64, u64],
        "fk_sdpa_decode_noalloc": [vp, vp, vp, vp, i32, i32, i32, i32, u32, f32, vp], "fk_comm_unique_id": [vp, sz], "fk_comm_init": [u64, vp, i32, i32],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = C.c_int32
    L.fk_last_error.restype = C.c_char_p
    L.fk_version.restype = C.c_char_p
    _lib = L
    return L


def check(status: int, what: str = "") -> None:
    if status != 0:
        raise FusekitError(f"{what or 'fusekit call'} failed ({status}): {lib().fk_last_error().decode(errors='replace')}")
