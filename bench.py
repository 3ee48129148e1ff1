#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tokens/s of the Qwen2.5-7B-shaped 4-bit (group 64)
decoder at context 512, through the captured CUDA graph of libfusekit_cuda.so.

    python bench.py --gpus N --steps K --warmup W            (N > 1 under torchrun: N replicas + the 32B tensor-parallel run)
    python bench.py --impl reference ...                      (CPU oracle port on the host cores)
    python bench.py --workload qwen32b-q4-ctx4096 --tp        (N ranks form one tensor-parallel group)

A step is one decode chunk of 64 tokens (the reference's FK_CHUNK) with on-device token feedback.
`value` is device-timed (CUDA events on the library's stream, weights/KV resident in HBM); `e2e` is
wall-clock through DecodeEngine.decode_chunk with the seed token uploaded from pinned host memory
and the token history read back every chunk.  Synthetic data: seeded random-init weights and an
N(0,1) KV pre-fill, as the benchmark configs define.  Inputs (4 GB of weights) exceed the 126 MB L2,
so no explicit flush is needed between iterations.

With more than one rank the headline line stays the replica measurement (batch-1 decode does not
shard into independent units); the ranks then also run the 32B-shaped model tensor-parallel over all
of them and the line carries that as `tp` (tok/s of the one stream, roofline fraction, whether every
rank produced the same tokens).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

CHUNK = 64
WORKLOADS = {
    # name: (config, bits, ctx)
    "qwen7b-q4-ctx512": ("qwen2.5-7b", 4, 512),
    "qwen7b-q4-ctx32": ("qwen2.5-7b", 4, 32),
    "qwen7b-q8-ctx512": ("qwen2.5-7b", 8, 512),
    "qwen7b-bf16-ctx512": ("qwen2.5-7b", 16, 512),
    "gemma4b-q4-ctx4096": ("gemma3-4b", 4, 4096),
    "qwen32b-q4-ctx4096": ("qwen2.5-32b", 4, 4096),
    "qwen0.5b-q4-ctx32": ("qwen2.5-0.5b", 4, 32),
}
TP_WORKLOAD = "qwen32b-q4-ctx4096"
METRIC = "batch-1 decode tok/s, 7B-shaped int4 ctx512"      # other --workload values are named in config.workload
KIND_NAMES = ["step_init", "embed_lookup_decode", "rmsnorm_qkv", "qk_norm_rope_store", "sdpa_decode", "linear_residual",
              "rmsnorm_gateup_act", "final_rmsnorm_lm_head", "argmax_finalize", "allreduce", "residual_add"]


def ncu_traffic() -> dict:
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of each kernel kind, from the ncu captures summarised
    under profiles/ (one `kernel_name bytes` pair per line)."""
    out, p = {}, os.path.join(ROOT, "profiles", "dram_traffic_per_launch.txt")
    if os.path.exists(p):
        for ln in open(p):
            f = ln.split()
            if len(f) >= 2 and not ln.startswith("#"):
                try:
                    out[f[0]] = float(f[1])
                except ValueError:
                    pass
    return out


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu: int):
        self.gpu, self.lines, self.proc = gpu, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_oracle_check(config: str, bits: int, ctx: int, gpu_tokens, seed_token: int, budget_s: float):
    """The CPU oracle port (all host threads) walked along the GPU's own first tokens of the same workload: its rate is
    the CPU baseline, and every token is compared with the GPU's (a flip inside two bf16 ulps of the oracle's winning
    logit counts as a near-tie, anything wider as a mismatch)."""
    from fusekit_b200.model_spec import CONFIGS
    from oracle import oracle as O
    cores = O.set_num_threads(host_cores())
    spec = CONFIGS[config].with_bits(bits)
    m = O.Model(O.model_config(spec, ctx + 64))
    m.prefill_kv(ctx)
    t0 = time.perf_counter()
    m.step(seed_token, ctx)                      # one token to size the sample (its KV row is rewritten below)
    t1 = time.perf_counter() - t0
    n = int(max(1, min(len(gpu_tokens), budget_s / max(t1, 1e-3))))
    t0 = time.perf_counter()
    mism, ties = O.compare_greedy(gpu_tokens[:n], m, seed_token, ctx)
    secs = time.perf_counter() - t0
    m.close()
    return n / secs, n, cores, mism, ties


def run_reference(args, rank: int):
    """Reference arm: the reference's Metal/MLX path cannot run here, so the CPU port of its kernel
    math (the oracle) is timed on the host cores.  A step is one decoded token of the same workload."""
    if rank != 0:
        return
    config, bits, ctx = WORKLOADS[args.workload]
    from fusekit_b200.model_spec import CONFIGS
    from oracle import oracle as O
    cores = O.set_num_threads(host_cores())      # all host cores, whatever OMP_NUM_THREADS the launcher exported
    spec = CONFIGS[config].with_bits(bits)
    m = O.Model(O.model_config(spec, ctx + args.steps + args.warmup + 8))
    m.prefill_kv(ctx)
    tok, pos = 3, ctx
    for _ in range(args.warmup):
        tok, _, _ = m.step(tok, pos); pos += 1
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok, _, _ = m.step(tok, pos); pos += 1
    dt = time.perf_counter() - t0
    val = args.steps / dt
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": f"int{bits}" if bits != 16 else "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "step": "1 decoded token on the CPU"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} greedy tokens of {args.workload} after {args.warmup} warm-up tokens, OpenMP over output rows on {cores} threads"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def make_tp_engine(spec, cap, local, rank, world, dist):
    """One tensor-parallel slice per rank, with the exchange the library offers: peer-memory (CUDA IPC arenas, default
    where the GPUs can map each other) or the NCCL all-reduce captured in the graph (FK_PEER=0)."""
    from fusekit_b200.runtime import DecodeEngine, comm_unique_id
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    eng = DecodeEngine(spec, cap, device=local, tp_rank=rank, tp_size=world)
    peer = False
    if os.environ.get("FK_PEER", "1") != "0":
        handles = [None] * world
        dist.all_gather_object(handles, eng.peer_export())
        peer = eng.peer_open(handles)
        flags = [None] * world
        dist.all_gather_object(flags, bool(peer))
        peer = all(flags)
    if not peer:
        uid = [comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        eng.comm_init(uid[0])
        eng.peer_disable()
    return eng, peer


def timed_chunks(eng, ctx, warmup, steps, barrier, sampler=None):
    tok, first = 3, None
    for i in range(warmup):
        out, _ = eng.decode_chunk(ctx + i * CHUNK, tok, CHUNK)
        if first is None:
            first = out.copy()
    if sampler:
        sampler.start()
    barrier()
    dev_s, t0 = 0.0, time.perf_counter()
    last = None
    for i in range(steps):
        out, s = eng.decode_chunk(ctx + i * CHUNK, tok, CHUNK)
        tok = int(out[-1]); dev_s += s; last = out
    eng.rt.sync()
    wall_s = time.perf_counter() - t0
    barrier()
    return dev_s, wall_s, first, last, tok


def run_batch(args, local: int):
    """Benchmark configuration 5 at batch M: M independent sequences advanced together on one GPU, every projection
    reading its weights once per step for all rows.  `value` counts the tokens of all sequences; the first tokens of
    sequence 0 are compared with a batch-1 CPU oracle run of that sequence (the same bounded sample is the CPU baseline)."""
    import torch
    from fusekit_b200.batch import BatchDecodeEngine
    from fusekit_b200.model_spec import CONFIGS
    config, bits, ctx = WORKLOADS[args.workload]
    spec = CONFIGS[config].with_bits(bits)
    M = args.batch
    cap = ctx + CHUNK * max(args.steps, args.warmup) + 8
    eng = BatchDecodeEngine(spec, cap, M, device=local, qmm={"auto": 0, "tcgen05": 1, "mma": 2}[args.qmm])
    eng.load_synthetic(); eng.prefill_kv_synthetic(ctx); eng.capture()
    seeds = np.array([3 + 7 * m for m in range(M)], np.uint32)
    first = None
    for i in range(max(args.warmup, 1)):
        out, _ = eng.decode_chunk(ctx + i * CHUNK, seeds, CHUNK)
        first = out if first is None else first
    sampler = ClockSampler(local); sampler.start()
    torch.cuda.synchronize(); eng.rt.sync()
    dev_s, t0, tok = 0.0, time.perf_counter(), seeds
    for i in range(args.steps):
        out, s = eng.decode_chunk(ctx + i * CHUNK, tok, CHUNK)
        tok, dev_s = out[-1], dev_s + s
    eng.rt.sync()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop()
    steps_total = args.steps * CHUNK
    wbytes = spec.weight_bytes_per_token()
    kv = spec.kv_bytes_per_token(ctx + CHUNK * args.steps // 2) * M
    peak, peak_kind = measured_peak()
    cpu_baseline, parity = None, None
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        cores = O.set_num_threads(host_cores())
        m0 = O.Model(O.model_config(spec, ctx + 64))
        hd = spec.head_dim
        for l in range(spec.n_layers):           # sequence 0's pre-fill, the streams the engine used
            k = np.zeros((spec.n_kv, ctx + 64, hd), np.uint16); v = np.zeros_like(k)
            for hh in range(spec.n_kv):
                k[hh, :ctx] = O.fill_normal_bf16(BatchDecodeEngine.cache_stream(spec, l, "k", 0), hh * 1048576 * hd, ctx * hd, 0.0, 1.0).reshape(ctx, hd)
                v[hh, :ctx] = O.fill_normal_bf16(BatchDecodeEngine.cache_stream(spec, l, "v", 0), hh * 1048576 * hd, ctx * hd, 0.0, 1.0).reshape(ctx, hd)
            m0.set_cache(l, k, v)
        t1 = time.perf_counter(); m0.step(int(seeds[0]), ctx); t1 = time.perf_counter() - t1
        n = int(max(1, min(CHUNK, args.cpu_budget / max(t1, 1e-3))))
        t1 = time.perf_counter()
        mism, ties = O.compare_greedy(first[:n, 0], m0, int(seeds[0]), ctx)
        secs = time.perf_counter() - t1
        m0.close()
        cpu_baseline = {"value": n / secs, "unit": "tok/s", "cores": cores, "kind": "port",
                        "sample": f"{n} tokens of one sequence of {args.workload} on the CPU oracle ({cores} threads): the CPU decodes sequences one at a time"}
        parity = {"tokens_compared": n, "mismatches": len(mism), "near_ties": len(ties)}
        if mism:
            raise SystemExit(f"bench: batch row 0 differs from the CPU oracle beyond a near-tie: {mism}")
    nodes = len(eng.tasks)
    eng.close()
    tps = steps_total * M / dev_s
    print(json.dumps({
        "metric": f"batch-{M} decode tok/s (all sequences), {args.workload}", "value": tps, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4", "data": "synthetic",
        "config": {"workload": args.workload, "batch": M, "tokens_per_step": CHUNK * M, "ctx_start": ctx, "graph_nodes_per_token": nodes,
                   "projection_kernel": args.qmm, "l2": "inputs (weights) larger than L2"},
        "e2e": {"value": steps_total * M / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 80, "d2h_bytes_per_step": CHUNK * M * 4 + 84},
        "gpu_launches": nodes * steps_total, "clocks": clocks,
        "per_sequence_tok_s": steps_total / dev_s,
        "roofline": {"bound": "hbm", "kernel": "whole step (weights once per step + every sequence's KV)", "achieved": (wbytes + kv) * steps_total / dev_s / 1e9,
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": (wbytes + kv) * steps_total / dev_s / 1e9 / peak,
                     "bytes_per_launch": wbytes + kv, "weight_stream_gbs": wbytes * steps_total / dev_s / 1e9, "traffic": None},
        "cpu_baseline": cpu_baseline, "parity_checked": parity is not None and not parity["mismatches"], "parity": parity,
    }), flush=True)


def main():
    global CHUNK
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fusekit", choices=["fusekit", "reference"])
    ap.add_argument("--workload", default="qwen7b-q4-ctx512", choices=sorted(WORKLOADS))
    ap.add_argument("--chunk", type=int, default=CHUNK, help="tokens per step (64 = the reference's FK_CHUNK); smaller for profiler captures")
    ap.add_argument("--tp", action="store_true", help="N ranks form one tensor-parallel group (one stream) instead of N replicas")
    ap.add_argument("--no-tp-extra", action="store_true", help="with N > 1 replicas, skip the additional 32B tensor-parallel run")
    ap.add_argument("--batch", type=int, default=1, help="independent sequences decoded together (2..16: the batch decode engine, one GPU)")
    ap.add_argument("--qmm", default="auto", choices=["auto", "tcgen05", "mma"], help="kernel of the several-row projections in batch decode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--profile-nodes", type=int, default=5, help="repeats of the per-kernel timing pass (0 = skip)")
    args = ap.parse_args()
    CHUNK = args.chunk
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    if args.batch > 1:
        if rank == 0:
            run_batch(args, local)
        return

    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from fusekit_b200.model_spec import CONFIGS
    from fusekit_b200.runtime import DecodeEngine
    config, bits, ctx = WORKLOADS[args.workload]
    spec = CONFIGS[config].with_bits(bits)
    cap = ctx + CHUNK * max(args.steps, args.warmup) + 8
    peer = False
    if args.tp and world > 1:
        eng, peer = make_tp_engine(spec, cap, local, rank, world, dist)
    else:
        eng = DecodeEngine(spec, cap, device=local)      # N > 1: N independent replicas, one per GPU
    eng.load_synthetic()
    eng.prefill_kv_synthetic(ctx)
    eng.capture()
    nodes = len(eng.replay)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        eng.rt.sync()

    def max_over_ranks(*vals):
        t = torch.tensor(list(vals), dtype=torch.float64, device=f"cuda:{local}")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    sampler = ClockSampler(local)
    dev_s, wall_s, first_chunk, _, tok = timed_chunks(eng, ctx, max(args.warmup, 1), args.steps, barrier, sampler)
    clocks = sampler.stop()
    dev_s, wall_s = max_over_ranks(dev_s, wall_s)
    streams = 1 if args.tp else world
    tokens = args.steps * CHUNK * streams
    peak, peak_kind = measured_peak()

    # per-kernel timing: all launches of one kernel kind (one per layer, each touching its own layer's weights, so
    # every launch reads cold data) back to back between two CUDA events on the library's stream
    roofline = None
    shares = {}
    if args.profile_nodes > 0 and rank == 0 and not (args.tp and world > 1):
        traffic = ncu_traffic()
        eng.rt.state_set(tok, ctx + CHUNK)
        by_kind = {}
        for t in eng.tasks:
            by_kind.setdefault(t.kind, []).append(t)
        per_kind = {k: eng.time_tasks(v, args.profile_nodes) / len(v) for k, v in by_kind.items()}
        # a kernel kind may cover shapes of different size (o_proj and down_proj): time them apart
        lin = by_kind.get(5, [])
        subs = {}
        for t in lin:
            subs.setdefault((t.iarg[0], t.iarg[1]), []).append(t)
        lin_times = {shape: eng.time_tasks(v, args.profile_nodes) / len(v) for shape, v in subs.items()}
        tot = sum(per_kind[k] * len(v) for k, v in by_kind.items())
        H, I = spec.hidden, spec.inter
        algo_by_kind = {6: 2 * spec.linear_bytes(H, I) - 2 * H - 2 * I,            # gate+up weights, x once, one T[I] out
                        7: spec.linear_bytes(H, spec.vocab) - 2 * spec.vocab,      # no logits are written
                        2: spec.linear_bytes(H, (spec.n_q + 2 * spec.n_kv) * spec.head_dim)}
        shares = {}
        for k, v in by_kind.items():
            e = {"launches": len(v), "avg_us": 1e6 * per_kind[k], "share": per_kind[k] * len(v) / tot}
            if k in algo_by_kind:
                e["gbs"] = algo_by_kind[k] / per_kind[k] / 1e9; e["frac_of_peak"] = e["gbs"] / peak
            shares[KIND_NAMES[k]] = e
        for (kk, nn), tsec in lin_times.items():
            gbs = spec.linear_bytes(kk, nn, True) / tsec / 1e9
            shares[f"linear_residual[{kk}->{nn}]"] = {"launches": len(subs[(kk, nn)]), "avg_us": 1e6 * tsec, "gbs": gbs, "frac_of_peak": gbs / peak}
        cands = {k: per_kind[k] * len(by_kind[k]) for k in algo_by_kind if k in per_kind}
        for (kk, nn), tsec in lin_times.items():
            cands[("lin", kk, nn)] = tsec * len(subs[(kk, nn)])
        dom = max(cands, key=cands.get)
        if isinstance(dom, tuple):
            algo, avg, name = spec.linear_bytes(dom[1], dom[2], True), lin_times[(dom[1], dom[2])], f"fusekit_linear_residual[{dom[1]}->{dom[2]}]"
        else:
            algo, avg, name = algo_by_kind[dom], per_kind[dom], "fusekit_" + KIND_NAMES[dom]
        ach = algo / avg / 1e9
        roofline = {"bound": "hbm", "kernel": name, "achieved": ach, "peak": peak, "peak_kind": peak_kind,
                    "unit": "GB/s", "frac": ach / peak, "bytes_per_launch": algo, "avg_launch_us": avg * 1e6,
                    "traffic": traffic.get(name) if args.workload == "qwen7b-q4-ctx512" else None}

    cpu_baseline, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, n, cores, mism, ties = cpu_oracle_check(config, bits, ctx, first_chunk, 3, args.cpu_budget)
        cpu_baseline = {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port",
                        "sample": f"{n} tokens of {args.workload} on the CPU oracle (OpenMP over output rows, {cores} threads), walked along the GPU's token stream"}
        parity = {"tokens_compared": n, "mismatches": len(mism), "near_ties": len(ties)}
        if mism:
            raise SystemExit(f"bench: GPU tokens differ from the CPU oracle beyond a near-tie: {mism}")

    info = eng.rt.info()
    eng.close()

    # ---- N > 1 replicas: the same ranks also run the 32B-shaped model tensor-parallel over all of them
    tp = None
    if dist is not None and not args.tp and not args.no_tp_extra:
        tcfg, tbits, tctx = WORKLOADS[TP_WORKLOAD]
        tspec = CONFIGS[tcfg].with_bits(tbits)
        tsteps, twarm = max(2, min(args.steps, 4)), 2
        teng, tpeer = make_tp_engine(tspec, tctx + CHUNK * max(tsteps, twarm) + 8, local, rank, world, dist)
        teng.load_synthetic(); teng.prefill_kv_synthetic(tctx); teng.capture()

        def tbarrier():
            dist.barrier(); torch.cuda.synchronize(); teng.rt.sync()

        tdev, twall, _, tlast, _ = timed_chunks(teng, tctx, twarm, tsteps, tbarrier)
        tdev, twall = max_over_ranks(tdev, twall)
        gathered = [None] * world
        dist.all_gather_object(gathered, [int(v) for v in tlast])
        tnodes = len(teng.replay)
        teng.close()
        tps = tsteps * CHUNK / tdev
        bpt = tspec.bytes_per_token(tctx + CHUNK * tsteps // 2)
        tp = {"workload": TP_WORKLOAD, "tensor_parallel": world, "tok_s": tps, "e2e_tok_s": tsteps * CHUNK / twall, "steps": tsteps, "warmup": twarm,
              "roofline_frac": bpt * tps / 1e9 / peak / world, "bytes_per_token": bpt, "allreduce": "peer" if tpeer else "nccl",
              "graph_nodes_per_token": tnodes, "tokens_equal_across_ranks": all(g == gathered[0] for g in gathered)}

    if rank == 0:
        tps = tokens / dev_s
        bpt = spec.bytes_per_token(ctx + CHUNK * args.steps // 2)
        tpd = world if args.tp else 1
        line = {
            "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "strong" if args.tp else "weak", "vs_baseline": None,
            "dtype": f"int{bits}" if bits != 16 else "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_step": CHUNK, "batch": 1, "ctx_start": ctx, "graph_nodes_per_token": nodes,
                       "l2": "inputs (weights) larger than L2", "replicas": streams, "tensor_parallel": tpd,
                       "allreduce": ("peer" if peer else "nccl") if args.tp and world > 1 else None, "pdl": info.get("pdl")},
            "e2e": {"value": tokens / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 80, "d2h_bytes_per_step": CHUNK * 4 + 80},
            "gpu_launches": nodes * CHUNK * args.steps,
            "clocks": clocks,
            "token_roofline": {"bytes_per_token": bpt, "achieved_gbs": bpt * (tps / streams) / 1e9, "peak": peak, "peak_kind": peak_kind,
                               "frac": bpt * (tps / streams) / 1e9 / peak / tpd, "frac_of_8tbs": bpt * (tps / streams) / 8e12 / tpd},
            "roofline": roofline, "kernel_shares": shares, "cpu_baseline": cpu_baseline,
            "parity_checked": parity is not None and not parity["mismatches"], "parity": parity,
        }
        if tp is not None:
            line["tp"] = tp
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
