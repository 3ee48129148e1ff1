"""The allocation-free attention entry point against the regular SDPA task.

Some hosts may not call the CUDA allocator while decoding: an engine that sizes every device buffer once at start-up
and treats any later cudaMalloc as a bug (it stalls the device and may fail when memory is nearly full), or a plug-in
that works only on buffers another framework hands it.  fk_sdpa_decode_noalloc serves them with scratch that is part
of the library image.  This file sorts last so a failure here cannot hide another test's result.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from fusekit_b200 import _native as N
from fusekit_b200.model_spec import stream_id
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _close(got, want, what):
    a, b = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
    # the tolerance of the other attention tests: 1e-2 max-abs (scaled by magnitude), 1e-3 relative RMS
    assert np.max(np.abs(a - b)) <= 1e-2 * max(1.0, np.abs(b).max()), what
    assert np.sqrt(np.mean((a - b) ** 2)) <= 1e-3 * np.sqrt(np.mean(b ** 2)), what


# (28, 4, 128, 700): the 7B shape; (14, 2, 64, 300) and (8, 4, 256, 300): the other head sizes; (8, 1, 128, 32256) sits
# at the limit of the built-in scratch: 8 heads * 1008 chunks * 130 floats = 1 048 320 of 1 048 576 floats
@pytest.mark.parametrize("nq,nkv,hd,cap,positions", [(28, 4, 128, 700, (600, 37)), (14, 2, 64, 300, (299, 5)), (8, 4, 256, 300, (150, 299)),
                                                     (8, 1, 128, 32256, (32255, 100))])
def test_noalloc_sdpa_matches_the_regular_entry_point_twice(runtime, nq, nkv, hd, cap, positions):
    rt = runtime
    scale = 1.0 / math.sqrt(hd)
    q = O.fill_normal_bf16(stream_id(3, "na.q"), 0, nq * hd, 0.0, 1.0)
    ck = O.fill_normal_bf16(stream_id(3, "na.k"), 0, nkv * cap * hd, 0.0, 1.0)
    cv = O.fill_normal_bf16(stream_id(3, "na.v"), 0, nkv * cap * hd, 0.0, 1.0)
    qd, kd, vd = rt.to_device(q), rt.to_device(ck), rt.to_device(cv)
    ref_out, new_out = rt.alloc(nq * hd * 2), rt.alloc(nq * hd * 2)
    chunks = (cap + 31) // 32
    part, cnt = rt.alloc(nq * chunks * (hd + 2) * 4), rt.alloc(nkv * 4)
    side = torch.cuda.Stream()                              # the second call of each shape goes to a stream of the caller's
    for n, pos in enumerate(positions):                     # two calls in a row share the built-in scratch
        rt.state_set(0, pos)
        rt.launch(N.Task.make(N.TASK_SDPA_DECODE, 0, {0: qd, 1: kd, 2: vd, 3: ref_out, 4: part, 5: cnt}, [nq, nkv, hd, cap], [scale]))
        want = rt.download(ref_out, (nq * hd,), np.uint16)
        N.check(rt.L.fk_memset(rt.h, new_out, 0, nq * hd * 2), "memset")
        rt.sync()
        stream = C.c_void_p(side.cuda_stream) if n == 1 else None
        N.check(rt.L.fk_sdpa_decode_noalloc(qd, kd, vd, new_out, nq, nkv, hd, cap, pos, scale, stream), "fk_sdpa_decode_noalloc")
        torch.cuda.synchronize()                            # the call only queued work
        got = rt.download(new_out, (nq * hd,), np.uint16)
        _close(got, want, f"vs the regular entry point, pos {pos}")
        _close(got, O.sdpa_decode(q, ck, cv, nq, nkv, hd, cap, min(pos + 1, cap), scale), f"vs the oracle, pos {pos}")
        assert np.any(got != 0)
    for p in (qd, kd, vd, ref_out, new_out, part, cnt):
        N.check(rt.L.fk_free(rt.h, p), "fk_free")


def test_noalloc_sdpa_refuses_oversized_shapes(runtime):
    rt = runtime
    p = rt.alloc(4096)
    # 64 heads * ceil(8192/32) chunks * 258 floats = 4.2 M floats > 1 Mi floats of built-in scratch
    assert rt.L.fk_sdpa_decode_noalloc(p, p, p, p, 64, 8, 256, 8192, 0, 1.0, None) == -1
    assert b"exceeds the built-in scratch" in rt.L.fk_last_error()
    assert rt.L.fk_sdpa_decode_noalloc(None, p, p, p, 8, 8, 64, 64, 0, 1.0, None) == -1
    # a position beyond 2^31 - 1 is refused on the host (nothing is launched)
    assert rt.L.fk_sdpa_decode_noalloc(p, p, p, p, 8, 8, 64, 64, 0x80000000, 1.0, None) == -1
    assert b"exceeds 2^31 - 1" in rt.L.fk_last_error()
