"""In-kernel phase timeline of one decoded token: ``python -m fusekit_b200.timeline [config] [--ctx N] [--bits B]``.

Every block of the streamed kernels writes ``globaltimer`` stamps per phase into a buffer set with
``fk_debug_timeline``; this tool decodes three tokens, keeps the stamps of the last one and prints, per task kind,
where the time between two task boundaries goes.  It is a tuning aid (reference counterpart: the per-command GPU
times of ``profile_icb_commands``, python_runtime/src/lib.rs:821-869, which cannot see inside a kernel)."""
from __future__ import annotations

import argparse
import collections

import numpy as np

from . import _native as N
from .model_spec import CONFIGS
from .runtime import DecodeEngine

NAMES = {1: "embed", 2: "rmsnorm_qkv", 3: "qk_norm_rope_store", 4: "sdpa", 5: "linear", 6: "gateup", 7: "head"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("config", nargs="?", default="qwen2.5-7b", choices=sorted(CONFIGS))
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--bits", type=int, default=4)
    args = ap.parse_args()
    spec = CONFIGS[args.config].with_bits(args.bits)
    eng = DecodeEngine(spec, args.ctx + 64)
    eng.load_synthetic(); eng.prefill_kv_synthetic(args.ctx)
    rt, tasks = eng.rt, eng.build_dispatches()
    n, per_task = len(tasks), 4096                              # u64 entries per task slice
    buf = rt.alloc(n * per_task * 8)
    N.check(rt.L.fk_debug_timeline(rt.h, buf), "fk_debug_timeline")
    eng.capture()
    for rep in range(3):
        rt.L.fk_memset(rt.h, buf, 0, n * per_task * 8); rt.sync()
        _, secs = eng.decode_chunk(args.ctx + rep, 3, 1)
    tl = rt.download(buf, (n, per_task // 8, 8), np.uint64).astype(np.int64)
    print(f"{args.config} q{args.bits} ctx {args.ctx}: token {secs * 1e6:.1f} us on the device, {n} tasks, one kernel per task")
    agg = collections.defaultdict(list)
    prev_end = None
    for j, t in enumerate(tasks):
        a = tl[j]; a = a[a[:, 0] > 0]
        if not len(a):
            continue
        key = NAMES.get(t.kind, str(t.kind)) + (f"[{t.iarg[0]}->{t.iarg[1]}]" if t.kind == 5 else "")
        start = a[:, 0].min()
        # slots: 0 kernel start, 1 dependency met, 2 activations staged, 3 (6 for attention) end
        end = a[:, 6 if t.kind == 4 else 3]; end = end[end > 0].max()
        dep = np.median(a[:, 1]); staged = np.median(a[:, 2][a[:, 2] > 0]) if (a[:, 2] > 0).any() else dep
        base = prev_end if prev_end is not None else start
        agg[key].append(((end - base) / 1e3, (dep - base) / 1e3, (staged - dep) / 1e3, (end - staged) / 1e3))
        prev_end = end
    print(f"{'task':28s} {'n':>3s} {'total':>7s} {'prev end->dep met':>18s} {'stage':>7s} {'units+epilogue':>15s}   (us)")
    for k, v in agg.items():
        m = np.array(v).mean(0)
        print(f"{k:28s} {len(v):3d} {m[0]:7.2f} {m[1]:18.2f} {m[2]:7.2f} {m[3]:15.2f}")
    eng.close()


if __name__ == "__main__":
    main()
