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
