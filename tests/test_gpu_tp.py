"""Tensor-parallel decode on 2 GPUs against the single-rank oracle: with the library all-reduce (NCCL, captured in the
graph), with the stand-alone peer-memory all-reduce kernel, and with the exchange fused into the projection kernels (no
all-reduce task at all).  Skipped where fewer than two CUDA devices are visible."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    from fusekit_b200.model_spec import CONFIGS
    from fusekit_b200.runtime import DecodeEngine, comm_unique_id
    spec, ctx, steps = CONFIGS["tiny-qwen"], 20, 16
    uid = [comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    eng = DecodeEngine(spec, 64, device=rank, tp_rank=rank, tp_size=world)
    eng.comm_init(uid[0])
    if mode == "peer":
        os.environ["FK_TP_EXCHANGE"] = "allreduce"
    if mode in ("peer", "fused"):
        handles = [None] * world
        dist.all_gather_object(handles, eng.peer_export())
        assert eng.peer_open(handles), "peer arenas could not be mapped"
    eng.load_synthetic(); eng.prefill_kv_synthetic(ctx)
    from fusekit_b200 import _native as N
    kinds = [t.kind for t in eng.build_dispatches()]
    assert (N.TASK_ALLREDUCE in kinds) == (mode != "fused"), kinds
    toks, secs = eng.decode_chunk(ctx, 3, steps)
    toks2, _ = eng.decode_chunk(ctx + steps, int(toks[-1]), 4)          # a second chunk: the exchange sequence numbers carry on
    toks = np.concatenate([toks, toks2])
    gathered = [None] * world
    dist.all_gather_object(gathered, [int(t) for t in toks])
    assert all(g == gathered[0] for g in gathered), gathered        # every rank decodes the same stream
    if rank == 0:
        from oracle import oracle as O
        from tests.helpers import compare_greedy, oracle_config
        m = O.Model(oracle_config(spec, 64)); m.prefill_kv(ctx)
        mism, ties = compare_greedy(toks, m, 3, ctx, tie_ulps=4.0)
        assert not mism and len(ties) <= 2, (mism, ties)
    dist.barrier(); eng.close(); dist.destroy_process_group()
    print("rank", rank, "ok")
""")


@pytest.mark.parametrize("mode", ["nccl", "peer", "fused"])
def test_two_rank_tensor_parallel_decode(tmp_path, mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    port = 29700 + os.getpid() % 2000 + {"nccl": 0, "peer": 1, "fused": 2}[mode]
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", mode], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-3000:]
