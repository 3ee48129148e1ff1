"""CPU checks of the drop-in boundary: the library loads, exports every symbol the header declares,
and refuses to work without a CUDA device (no silent fallback)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fusekit_cuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for must in ("fk_open", "fk_alloc", "fk_upload", "fk_download", "fk_graph_capture", "fk_graph_launch",
                 "fk_decode_chunk", "fk_decode_chunk_host", "fk_step", "fk_launch", "fk_launch_batch", "fk_smoke",
                 "fk_graph_profile_nodes", "fk_kv_cache_alloc", "fk_comm_init", "fk_last_error", "fk_version"):
        assert must in syms
    assert len(syms) >= 30


def test_library_exports_every_declared_symbol():
    from fusekit_b200 import _native as N
    lib = N.lib()
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_task_struct_layout_matches_the_header():
    from fusekit_b200 import _native as N
    # int32 kind, int32 layer, u64 buf[12], int32 iarg[8], float farg[4]
    assert C.sizeof(N.Task) == 4 + 4 + 12 * 8 + 8 * 4 + 4 * 4
    assert N.Task.buf.offset == 8 and N.Task.iarg.offset == 104 and N.Task.farg.offset == 136
    text = open(HEADER).read()
    for i, name in enumerate(["STEP_INIT", "EMBED_LOOKUP_DECODE", "RMSNORM_QKV", "QK_NORM_ROPE_STORE", "SDPA_DECODE",
                              "LINEAR_RESIDUAL", "RMSNORM_GATEUP_ACT", "FINAL_RMSNORM_LM_HEAD", "ARGMAX_FINALIZE",
                              "ALLREDUCE", "RESIDUAL_ADD"]):
        assert re.search(rf"FK_TASK_{name} = {i}\b", text), name
        assert getattr(N, f"TASK_{name}") == i


def test_no_device_means_a_loud_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from fusekit_b200 import _native as N
    from fusekit_b200.runtime import Runtime
    with pytest.raises(N.FusekitError, match="fk_open"):
        Runtime(0)
    assert b"cuda" in N.lib().fk_last_error().lower()


def test_bad_handle_is_a_value_error():
    from fusekit_b200 import _native as N
    lib = N.lib()
    p = C.c_uint64()
    assert lib.fk_alloc(12345, 64, C.byref(p)) == -1
    assert b"invalid handle" in lib.fk_last_error()
    buf = C.create_string_buffer(512)
    assert lib.fk_kernel_names(buf, 512) == 0 and b"fusekit_rmsnorm_qkv" in buf.value


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "fusekit_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower() or f == "build.py", f"{f} mentions the oracle"
