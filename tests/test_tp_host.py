"""CPU tests of the tensor-parallel host logic: shard plans, and a world-size-2 gloo run in which every rank
computes its column/row slices with the oracle and the all-reduced partial sums reproduce the full projections."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from fusekit_b200.model_spec import CONFIGS, stream_id, tensor_name
from fusekit_b200.runtime import check_tp, linear_plan, vector_plan
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shards_tile_the_full_tensors(world):
    spec = CONFIGS["qwen2.5-32b"]
    check_tp(spec, world)
    full = {name: (segs, kg, k0, k) for name, segs, kg, k0, k, _ in linear_plan(spec, 0, 1) if name.startswith("layers.0.") or name == "lm_head"}
    cover = {}
    for r in range(world):
        for name, segs, kg, k0, k, _ in linear_plan(spec, r, world):
            if not (name.startswith("layers.0.") or name == "lm_head"):
                continue
            assert kg == full[name][1]
            for leaf, row0, n in segs:
                cover.setdefault((name, leaf), []).append((row0, n, k0, k))
    for (name, leaf), parts in cover.items():
        segs, kg, _, kfull = full[name]
        nfull = dict((lf, n) for lf, _, n in segs)[leaf]
        if name.endswith((".o", ".down")):            # row-split: K is cut into `world` whole-group slices, all rows kept
            assert sorted(p[2] for p in parts) == [i * kfull // world for i in range(world)]
            assert all(p[3] == kfull // world and p[3] % 64 == 0 and p[1] == nfull for p in parts)
        else:                                         # column-split: output rows are cut, K kept
            assert sorted(p[0] for p in parts) == [i * nfull // world for i in range(world)]
            assert all(p[1] == nfull // world and p[3] == kfull for p in parts)
    # KV heads divide evenly and each rank keeps whole heads
    hd = spec.head_dim
    for name, leaf, layer, idx0, n, mean, std in vector_plan(spec, world - 1, world):
        if leaf == "k_bias":
            assert n == spec.n_kv // world * hd and idx0 == (world - 1) * n


def test_invalid_degrees_are_refused():
    with pytest.raises(ValueError):
        check_tp(CONFIGS["qwen2.5-7b"], 8)            # 4 kv heads cannot be split 8 ways
    with pytest.raises(ValueError):
        check_tp(CONFIGS["gemma3-4b"], 2)


WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from fusekit_b200.model_spec import CONFIGS, stream_id, tensor_name
    from fusekit_b200.runtime import linear_plan
    from oracle import oracle as O
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
    rank, world = dist.get_rank(), 2
    spec = CONFIGS["tiny-qwen"]
    H, hd = spec.hidden, spec.head_dim
    plan = dict((name, (segs, kg, k0, k)) for name, segs, kg, k0, k, _ in linear_plan(spec, rank, world))
    # the exchange step of a row-split projection: fp32 partial sums all-reduced over the ranks
    for name, xlen in (("layers.0.o", spec.n_q * hd), ("layers.0.down", spec.inter)):
        segs, kg, k0, k = plan[name]
        leaf, row0, n = segs[0]
        s = stream_id(spec.seed, tensor_name(0, leaf))
        x = O.fill_normal_bf16(stream_id(1, "tp.x." + leaf), 0, xlen, 0.0, 1.0)
        w = O.gen_weight(s, n, k, spec.bits, k_global=kg, row0=row0, k0=k0)
        part = torch.from_numpy(O.linear_acc(w, O.bf16_to_f32(x[k0:k0 + k])).copy())
        dist.all_reduce(part)
        full = O.linear_acc(O.gen_weight(s, n, kg, spec.bits), O.bf16_to_f32(x))
        assert np.allclose(part.numpy(), full, rtol=1e-5, atol=1e-5), name
    # the argmax exchange of the vocabulary-sharded head: max over ranks of (sortable key, inverted index)
    segs, kg, k0, k = plan["lm_head"]
    leaf, row0, n = segs[0]
    xf = O.bf16_to_f32(O.fill_normal_bf16(stream_id(1, "tp.head.x"), 0, H, 0.0, 1.0))
    s = stream_id(spec.seed, "lm_head")
    lg = O.f32_to_bf16(O.linear_acc(O.gen_weight(s, n, k, spec.bits, k_global=kg, row0=row0), xf))
    best = O.argmax_bf16(lg)
    bits = int(lg[best]); key = (~bits & 0xffff) if bits & 0x8000 else (bits ^ 0x8000)
    packed = torch.tensor([(key << 32) | (0xffffffff - (row0 + best))], dtype=torch.int64)
    dist.all_reduce(packed, op=dist.ReduceOp.MAX)
    winner = 0xffffffff - (int(packed[0]) & 0xffffffff)
    full_lg = O.f32_to_bf16(O.linear_acc(O.gen_weight(s, spec.vocab, H, spec.bits), xf))
    assert winner == O.argmax_bf16(full_lg), (winner, O.argmax_bf16(full_lg))
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_rank_exchange_reproduces_the_full_projections(tmp_path):
    port = 29500 + os.getpid() % 2000
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-2000:]
