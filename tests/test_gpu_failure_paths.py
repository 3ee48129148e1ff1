"""Failure paths that reach the host without faulting or hanging the GPU: a bounded device wait that runs out, and
bad seeds refused before anything is launched (reference analogue: strict dispatch falls back instead of running a
task list it cannot trust, python/fusekit_runtime/__init__.py:2889-2895)."""
import ctypes as C

import numpy as np
import pytest

from fusekit_b200 import _native as N
from fusekit_b200.model_spec import CONFIGS
from fusekit_b200.runtime import DecodeEngine, Runtime

pytestmark = pytest.mark.gpu


def test_peer_exchange_wait_runs_out_and_the_status_reaches_the_host():
    """Two 'ranks' whose arenas both live on this GPU; rank 1 never runs, so rank 0's wait for its flag gives up after
    2000 polls, the kernel sets error bit 0x8000 and returns.  The error word reaches fk_state_get and makes
    fk_decode_chunk fail with FK_ERR_DEVICE; fk_state_set clears it and the handle stays usable."""
    rt = Runtime(0)
    try:
        N.check(rt.L.fk_peer_arena_loopback(rt.h, 0, 2, 2000), "fk_peer_arena_loopback")
        buf = rt.to_device(np.arange(3584, dtype=np.float32))
        task = N.Task.make(N.TASK_ALLREDUCE, 0, {0: buf}, [3584, 0])
        rt.state_set(0, 0)
        rt.launch(task)                                    # returns: the wait is bounded
        _, _, err = rt.state_get()
        assert err & 0x8000, hex(err)
        arr = (N.Task * 1)(task)
        g = C.c_uint64()
        N.check(rt.L.fk_graph_capture(rt.h, arr, 1, C.byref(g)), "fk_graph_capture")
        out = np.zeros(1, np.uint32)
        st = rt.L.fk_decode_chunk(rt.h, g.value, 0, 0, 1, out.ctypes.data, None)
        assert st == -5 and b"0x8000" in rt.L.fk_last_error()
        rt.state_set(0, 0)                                 # a new state starts with a clean error word
        assert rt.state_get()[2] == 0
        a = np.arange(256, dtype=np.uint16)
        assert np.array_equal(rt.smoke(a, a).shape, a.shape)      # the context still runs kernels
    finally:
        rt.close()


def test_seed_token_outside_the_embedding_table_is_refused_on_the_host():
    spec = CONFIGS["tiny-qwen"]
    eng = DecodeEngine(spec, 64)
    try:
        eng.load_synthetic(); eng.capture()
        with pytest.raises(N.FusekitError, match="outside the embedding table"):
            eng.decode_chunk(0, spec.vocab, 1)
        with pytest.raises(N.FusekitError, match="outside the embedding table"):
            eng.rt.state_set(spec.vocab + 5, 0)
        toks, _ = eng.decode_chunk(0, spec.vocab - 1, 2)   # the last row of the table is fine
        assert len(toks) == 2 and all(int(t) < spec.vocab for t in toks)
    finally:
        eng.close()


def test_close_releases_device_memory():
    """Opening and closing handles (with weights, graphs and loopback arenas) does not accumulate device memory."""
    import torch
    free0 = None
    for i in range(4):
        eng = DecodeEngine(CONFIGS["tiny-qwen"], 64)
        eng.load_synthetic(); eng.capture(); eng.decode_chunk(0, 3, 2)
        N.check(eng.rt.L.fk_peer_arena_loopback(eng.rt.h, 0, 2, 100), "loopback")
        eng.close()
        torch.cuda.synchronize()
        free, _ = torch.cuda.mem_get_info()
        if i == 0:
            free0 = free
    assert free >= free0 - (8 << 20), (free0, free)


FAKE_NCCL_WORKER = r"""
import ctypes as C, os, sys
sys.path.insert(0, {root!r})
from fusekit_b200 import _native as N
from fusekit_b200.model_spec import CONFIGS
from fusekit_b200.runtime import DecodeEngine, comm_unique_id
fake = C.CDLL(os.environ["FK_NCCL_LIB"], mode=C.RTLD_GLOBAL)
eng = DecodeEngine(CONFIGS["tiny-qwen"], 64, device=0, tp_rank=0, tp_size=2)
eng.comm_init(comm_unique_id())
eng.load_synthetic(); eng.prefill_kv_synthetic(8)
toks, _ = eng.decode_chunk(8, 3, 4)                       # collectives are no-ops here: only the control flow matters
assert len(toks) == 4 and fake.fake_nccl_allreduce_count() > 0
assert eng.rt.L.fk_comm_check(eng.rt.h) == 0
fake.fake_nccl_set_async_error(6)                         # ncclRemoteError: a peer went away
out = (C.c_uint32 * 4)()
st = eng.rt.L.fk_decode_chunk(eng.rt.h, eng.graph, 12, int(toks[-1]), 4, out, None)
assert st == -4 and b"aborted" in eng.rt.L.fk_last_error(), (st, eng.rt.L.fk_last_error())
assert fake.fake_nccl_abort_count() == 1
st = eng.rt.L.fk_decode_chunk(eng.rt.h, eng.graph, 12, int(toks[-1]), 4, out, None)      # refused before anything is launched
assert st == -3 and fake.fake_nccl_abort_count() == 1, (st, eng.rt.L.fk_last_error())
assert eng.rt.L.fk_comm_check(eng.rt.h) == -3
eng.close()
print("fake-nccl ok")
"""


def test_communicator_error_aborts_and_reaches_the_host(tmp_path):
    """The library polls ncclCommGetAsyncError while it waits; on an asynchronous error it aborts the communicator, returns
    FK_ERR_NCCL and refuses further replays.  The failure is injected on the host through a stand-in libnccl (no collective
    runs, no GPU fault); a child process so the stand-in is the first NCCL the library loads."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    so = tmp_path / "libfakenccl.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so), os.path.join(root, "tests", "fake_nccl.c")])
    script = tmp_path / "worker.py"
    script.write_text(FAKE_NCCL_WORKER.format(root=root))
    env = dict(os.environ, FK_NCCL_LIB=str(so))
    p = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "fake-nccl ok" in p.stdout, (p.stdout + p.stderr)[-3000:]
