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


def test_noalloc_sdpa_matches_the_regular_entry_point_twice(runtime):
    rt = runtime
    nq, nkv, hd, cap = 28, 4, 128, 700
    scale = 1.0 / math.sqrt(hd)
    q = O.fill_normal_bf16(stream_id(3, "na.q"), 0, nq * hd, 0.0, 1.0)
    ck = O.fill_normal_bf16(stream_id(3, "na.k"), 0, nkv * cap * hd, 0.0, 1.0)
    cv = O.fill_normal_bf16(stream_id(3, "na.v"), 0, nkv * cap * hd, 0.0, 1.0)
    qd, kd, vd = rt.to_device(q), rt.to_device(ck), rt.to_device(cv)
    ref_out, new_out = rt.alloc(nq * hd * 2), rt.alloc(nq * hd * 2)
    chunks = (cap + 31) // 32
    part, cnt = rt.alloc(nq * chunks * (hd + 2) * 4), rt.alloc(nkv * 4)
    for pos in (600, 37):                                   # two calls in a row share the built-in scratch
        rt.state_set(0, pos)
        rt.launch(N.Task.make(N.TASK_SDPA_DECODE, 0, {0: qd, 1: kd, 2: vd, 3: ref_out, 4: part, 5: cnt}, [nq, nkv, hd, cap], [scale]))
        want = rt.download(ref_out, (nq * hd,), np.uint16)
        N.check(rt.L.fk_memset(rt.h, new_out, 0, nq * hd * 2), "memset")
        rt.sync()
        N.check(rt.L.fk_sdpa_decode_noalloc(qd, kd, vd, new_out, nq, nkv, hd, cap, pos, scale, None), "fk_sdpa_decode_noalloc")
        torch.cuda.synchronize()                            # the call only queued work on the default stream
        got = rt.download(new_out, (nq * hd,), np.uint16)
        a, b = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(want).astype(np.float64)
        # both entry points compute the same split-K attention with different chunking: bf16 outputs agree within the
        # tolerance the other attention tests use (1e-2 max-abs, 1e-3 relative RMS)
        assert np.max(np.abs(a - b)) <= 1e-2 * max(1.0, np.abs(b).max()), pos
        assert np.sqrt(np.mean((a - b) ** 2)) <= 1e-3 * np.sqrt(np.mean(b ** 2)), pos
        assert np.any(got != 0)


def test_noalloc_sdpa_refuses_oversized_shapes(runtime):
    rt = runtime
    p = rt.alloc(4096)
    # 64 heads * ceil(8192/32) chunks * 258 floats = 4.2 M floats > 1 Mi floats of built-in scratch
    assert rt.L.fk_sdpa_decode_noalloc(p, p, p, p, 64, 8, 256, 8192, 0, 1.0, None) == -1
    assert b"exceeds the built-in scratch" in rt.L.fk_last_error()
    assert rt.L.fk_sdpa_decode_noalloc(None, p, p, p, 8, 8, 64, 64, 0, 1.0, None) == -1
