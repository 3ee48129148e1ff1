#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tokens/s of the Qwen2.5-7B-shaped 4-bit (group 64)
decoder at context 512, through the captured CUDA graph of libfusekit_cuda.so.

    python bench.py --gpus N --steps K --warmup W            (N > 1 under torchrun: N replicas)
    python bench.py --impl reference ...                      (CPU oracle port on the host cores)

A step is one decode chunk of 64 tokens (the reference's FK_CHUNK) with on-device token feedback.
`value` is device-timed (CUDA events on the library's stream, weights/KV resident in HBM); `e2e` is
wall-clock through DecodeEngine.decode_chunk with the seed token uploaded from pinned host memory
and the token history read back every chunk.  Synthetic data: seeded random-init weights and an
N(0,1) KV pre-fill, as the benchmark configs define.  Inputs (4 GB of weights) exceed the 126 MB L2,
so no explicit flush is needed between iterations.
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
    # name: (config, bits, ctx, metric tag)
    "qwen7b-q4-ctx512": ("qwen2.5-7b", 4, 512),
    "qwen7b-q4-ctx32": ("qwen2.5-7b", 4, 32),
    "qwen7b-q8-ctx512": ("qwen2.5-7b", 8, 512),
    "qwen7b-bf16-ctx512": ("qwen2.5-7b", 16, 512),
    "gemma4b-q4-ctx4096": ("gemma3-4b", 4, 4096),
    "qwen32b-q4-ctx4096": ("qwen2.5-32b", 4, 4096),
    "qwen0.5b-q4-ctx32": ("qwen2.5-0.5b", 4, 32),
}
METRIC = "batch-1 decode tok/s, 7B-shaped int4 ctx512"      # BASELINE.json metric; other --workload values are named in config.workload
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
NCU_TRAFFIC = {"fusekit_rmsnorm_gateup_act": 81.8e6 + 2.2e6, "fusekit_final_rmsnorm_lm_head": 315.9e6 + 0.4e6}
KIND_NAMES = ["step_init", "embed_lookup_decode", "rmsnorm_qkv", "qk_norm_rope_store", "sdpa_decode", "linear_residual",
              "rmsnorm_gateup_act", "final_rmsnorm_lm_head", "argmax_finalize", "allreduce", "residual_add"]


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


def cpu_oracle_rate(config: str, bits: int, ctx: int, budget_s: float, tokens: int | None = None):
    """Tokens/s of the CPU oracle port (all host threads) on a bounded sample of the same workload."""
    from fusekit_b200.model_spec import CONFIGS
    from oracle import oracle as O
    from tests.helpers import oracle_config
    spec = CONFIGS[config].with_bits(bits)
    m = O.Model(oracle_config(spec, ctx + 64))
    m.prefill_kv(ctx)
    _, t1 = m.greedy(3, ctx, 1)
    n = tokens if tokens is not None else int(max(1, min(16, budget_s / max(t1, 1e-3))))
    toks, secs = m.greedy(3, ctx + 1, n)
    m.close()
    return n / secs, n, O.num_threads()


def run_reference(args, rank: int):
    """Reference arm: the reference's Metal/MLX path cannot run here, so the CPU port of its kernel
    math (the oracle) is timed on the host cores.  A step is one decoded token of the same workload."""
    if rank != 0:
        return
    config, bits, ctx = WORKLOADS[args.workload]
    from fusekit_b200.model_spec import CONFIGS
    from oracle import oracle as O
    from tests.helpers import oracle_config
    spec = CONFIGS[config].with_bits(bits)
    m = O.Model(oracle_config(spec, ctx + args.steps + args.warmup + 8))
    m.prefill_kv(ctx)
    tok, pos = 3, ctx
    for _ in range(args.warmup):
        tok, _, _ = m.step(tok, pos); pos += 1
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok, _, _ = m.step(tok, pos); pos += 1
    dt = time.perf_counter() - t0
    val = args.steps / dt
    cores = O.num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": f"int{bits}" if bits != 16 else "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "step": "1 decoded token on the CPU"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} greedy tokens of {args.workload} after {args.warmup} warm-up tokens, OpenMP over output rows"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    ap.add_argument("--persistent", default="auto", choices=["auto", "on", "off"], help="run a token as one persistent kernel (auto: when the task list allows)")
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
    if args.tp and world > 1:
        from fusekit_b200.runtime import comm_unique_id
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        uid = [comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        eng = DecodeEngine(spec, cap, device=local, tp_rank=rank, tp_size=world)
        eng.comm_init(uid[0])
        peer = False
        # peer-memory all-reduce where the GPUs can map each other's arenas: measured faster than the library collective
        # from 4 ranks up (FK_PEER=1 / 0 forces it on / off)
        if os.environ.get("FK_PEER", "1" if world >= 4 else "0") != "0":
            handles = [None] * world
            dist.all_gather_object(handles, eng.peer_export())
            peer = eng.peer_open(handles)
    else:
        eng = DecodeEngine(spec, cap, device=local)      # N > 1: N independent replicas, one per GPU
    eng.load_synthetic()
    eng.prefill_kv_synthetic(ctx)
    eng.capture({"auto": None, "on": True, "off": False}[args.persistent])
    nodes = len(eng.replay)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        eng.rt.sync()

    tok = 3
    for i in range(args.warmup):
        out, _ = eng.decode_chunk(ctx + i * CHUNK, tok, CHUNK)
    sampler = ClockSampler(local)
    sampler.start()
    barrier()
    dev_s, t0 = 0.0, time.perf_counter()
    for i in range(args.steps):
        out, s = eng.decode_chunk(ctx + i * CHUNK, tok, CHUNK)
        tok = int(out[-1]); dev_s += s
    eng.rt.sync()
    wall_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop()
    times = torch.tensor([dev_s, wall_s], dtype=torch.float64, device=f"cuda:{local}")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, wall_s = float(times[0]), float(times[1])
    streams = 1 if args.tp else world
    tokens = args.steps * CHUNK * streams
    peak, peak_kind = measured_peak()

    # per-kernel timing: all launches of one kernel kind (one per layer, each touching its own layer's weights, so
    # every launch reads cold data) back to back between two CUDA events on the library's stream
    roofline = None
    shares = {}
    if args.profile_nodes > 0 and rank == 0:
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
        shares = {KIND_NAMES[k]: {"launches": len(v), "avg_us": 1e6 * per_kind[k], "share": per_kind[k] * len(v) / tot} for k, v in by_kind.items()}
        for (kk, nn), tsec in lin_times.items():
            shares[f"linear_residual[{kk}->{nn}]"] = {"launches": len(subs[(kk, nn)]), "avg_us": 1e6 * tsec}
        H, I = spec.hidden, spec.inter
        algo_by_kind = {6: 2 * spec.linear_bytes(H, I) - 2 * H - 2 * I,            # gate+up weights, x once, one T[I] out
                        7: spec.linear_bytes(H, spec.vocab) - 2 * spec.vocab,      # no logits are written
                        2: spec.linear_bytes(H, (spec.n_q + 2 * spec.n_kv) * spec.head_dim)}
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
                    "traffic": NCU_TRAFFIC.get(name)}
        if eng.persistent:
            # the timed region is launches of one kernel, the persistent token kernel: its roofline is the token's.  The
            # per-task figures above (same tasks, one kernel each) stay in kernel_shares as the breakdown.
            bpl = spec.bytes_per_token(ctx + CHUNK * args.steps // 2)
            avg = dev_s / (args.steps * CHUNK)
            roofline = {"bound": "hbm", "kernel": "fusekit_decode_token", "achieved": bpl / avg / 1e9, "peak": peak, "peak_kind": peak_kind,
                        "unit": "GB/s", "frac": bpl / avg / 1e9 / peak, "bytes_per_launch": bpl, "avg_launch_us": avg * 1e6,
                        "traffic": NCU_TRAFFIC.get("fusekit_decode_token"), "per_task_dominant": roofline}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, n, cores = cpu_oracle_rate(config, bits, ctx, args.cpu_budget)
        cpu_baseline = {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port",
                        "sample": f"{n} greedy tokens of {args.workload} on the CPU oracle (OpenMP over output rows)"}

    if rank == 0:
        tps = tokens / dev_s
        bpt = spec.bytes_per_token(ctx + CHUNK * args.steps // 2)
        line = {
            "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True, "scaling": "strong" if args.tp else "weak", "vs_baseline": None,
            "dtype": f"int{bits}" if bits != 16 else "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_step": CHUNK, "batch": 1, "ctx_start": ctx, "graph_nodes_per_token": nodes,
                       "l2": "inputs (weights) larger than L2", "persistent_kernel": eng.persistent, "replicas": streams, "tensor_parallel": world if args.tp else 1, "allreduce": ("peer" if (args.tp and world > 1 and peer) else "nccl") if args.tp and world > 1 else None, "pdl": eng.rt.info().get("pdl")},
            "e2e": {"value": tokens / wall_s, "unit": "tok/s", "h2d_bytes_per_step": 80, "d2h_bytes_per_step": CHUNK * 4 + 80},
            "gpu_launches": nodes * CHUNK * args.steps,
            "clocks": clocks,
            "token_roofline": {"bytes_per_token": bpt, "achieved_gbs": bpt * (tps / streams) / 1e9, "peak": peak, "peak_kind": peak_kind,
                               "frac": bpt * (tps / streams) / 1e9 / peak / (world if args.tp else 1), "frac_of_8tbs": bpt * (tps / streams) / 8e12 / (world if args.tp else 1)},
            "roofline": roofline, "kernel_shares": shares, "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
