"""Time the quantised projection with 1..16 activation rows on one weight shape.

    python -m fusekit_b200.qmm_bench [K N] [--weights 8] [--repeats 20] [--rows 1,2,4,8,16] [--gateup]

Synthetic 4-bit weights (`--weights` distinct ones, launched back to back so that together they exceed L2), CUDA-event
time per launch.  One row runs the batch-1 kernel, several rows the `fusekit_qmm` counterpart (reference: the M > 1
tiles of src/codegen/msl.rs:2318-2439).  `--gateup` times the norm-first gate/up + SwiGLU task instead (N outputs from a
pair of N x K weights; reference: fusekit_qmm_t_swiglu_pair_impl, msl.rs:2489).
"""
from __future__ import annotations

import argparse
import ctypes as C

from . import _native as N
from .model_spec import stream_id
from .runtime import Runtime


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("shape", nargs="*", type=int, default=[3584, 18944], help="K N")
    ap.add_argument("--weights", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=20)
    ap.add_argument("--rows", default="1,2,4,8,16")
    ap.add_argument("--gateup", action="store_true")
    a = ap.parse_args(argv)
    if len(a.shape) != 2:
        ap.error("shape is K N")
    k, n = a.shape
    rt = Runtime(0)
    ws = []
    def synth(tag):
        w = rt.weight_alloc(n, k, 4)
        rt.weight_synth_rows(w, 0, n, stream_id(3, tag), 0.02, k, 0, 0)
        return w

    for i in range(a.weights):
        if a.gateup:
            ws.append(rt.weight_pair(synth(f"qmm_bench.g{i}"), synth(f"qmm_bench.u{i}")))
        else:
            ws.append(synth(f"qmm_bench.{i}"))
            rt.weight_finalize(ws[-1])
    nw = rt.alloc(k * 2)
    rt.synth_normal(nw, stream_id(5, "qmm_bench.nw"), 0, k, 1.0, 0.02)
    x = rt.alloc(16 * k * 2)
    rt.synth_normal(x, stream_id(5, "qmm_bench.x"), 0, 16 * k, 0.0, 1.0)
    y = rt.alloc(16 * n * 2)
    nbytes = (n * k // 2 + n * (k // 64) * 4) * (2 if a.gateup else 1)
    for m in [int(v) for v in a.rows.split(",")]:
        if a.gateup:
            tasks = [N.Task.make(N.TASK_RMSNORM_GATEUP_ACT, 0, {0: x, 1: nw, 2: w, 4: y}, [k, n, 0, m], [1e-6]) for w in ws]
        else:
            tasks = [N.Task.make(N.TASK_LINEAR_RESIDUAL, 0, {0: x, 1: w, 3: y}, [k, n, m]) for w in ws]
        arr = (N.Task * len(tasks))(*tasks)
        secs = C.c_double()
        N.check(rt.L.fk_time_tasks(rt.h, arr, len(tasks), a.repeats, C.byref(secs)), "fk_time_tasks")
        us = secs.value / len(ws) * 1e6
        print(f"K={k} N={n} rows={m}: {us:.1f} us per launch, weights at {nbytes / us / 1e3:.0f} GB/s, {m / us * 1e6:.0f} rows/s", flush=True)
    rt.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
