"""Regenerates tests/golden/*.npz.  Run from the repository root:  python tests/golden/make_golden.py

The reference project ships no golden vectors for its decode kernels and cannot run on Linux, so
these fixtures pin the CPU oracle against drift and against an independent float64 NumPy
restatement: every file stores the seeded INPUTS, the C oracle's OUTPUT bits and, where the op is
not pure integer work, a float64 result computed without the oracle.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O            # noqa: E402
from fusekit_b200.model_spec import CONFIGS, stream_id   # noqa: E402
from tests.helpers import oracle_config   # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def qmatvec_case(bits, n=48, k=256, seed=7):
    w = O.gen_weight(stream_id(seed, f"golden.w{bits}"), n, k, bits)
    x = O.fill_normal_bf16(stream_id(seed, "golden.x"), 0, k, 0.0, 1.0)
    res = O.fill_normal_bf16(stream_id(seed, "golden.res"), 0, n, 0.0, 1.0)
    y = O.qmatvec(w, x, res)
    deq = O.bf16_to_f32(w.dense) if bits == 16 else O.np_dequant(w)
    y64 = deq.astype(np.float64) @ O.bf16_to_f32(x).astype(np.float64) + O.bf16_to_f32(res)
    d = dict(x=x, res=res, y=y, y64=y64, deq=deq)
    if bits == 16:
        d["dense"] = w.dense
    else:
        d.update(packed=w.packed, scales=w.scales, biases=w.biases)
    np.savez_compressed(os.path.join(OUT, f"qmatvec_q{bits}.npz"), **d)


def pointwise_case(seed=11):
    h = 320
    x = O.fill_normal_bf16(stream_id(seed, "golden.nx"), 0, h, 0.0, 1.5)
    w = O.fill_normal_bf16(stream_id(seed, "golden.nw"), 0, h, 1.0, 0.02)
    y = O.rmsnorm(x, w, 1e-6)
    g = O.bf16_to_f32(O.fill_normal_bf16(stream_id(seed, "golden.g"), 0, 512, 0.0, 2.0))
    u = O.bf16_to_f32(O.fill_normal_bf16(stream_id(seed, "golden.u"), 0, 512, 0.0, 2.0))
    v = O.fill_normal_bf16(stream_id(seed, "golden.rope"), 0, 4 * 64, 0.0, 1.0)
    np.savez_compressed(os.path.join(OUT, "pointwise.npz"), x=x, w=w, rms=y, g=g, u=u,
                        swiglu=O.act(g, u, 0), geglu=O.act(g, u, 1), rope_in=v,
                        rope_out=O.rope(v, 4, 64, 1234, 1e6), rope_pos=np.array([1234]))


def sdpa_case(seed=13):
    nq, nkv, hd, cap, kv_len = 4, 2, 64, 160, 137
    q = O.fill_normal_bf16(stream_id(seed, "golden.q"), 0, nq * hd, 0.0, 1.0)
    ck = O.fill_normal_bf16(stream_id(seed, "golden.ck"), 0, nkv * cap * hd, 0.0, 1.0)
    cv = O.fill_normal_bf16(stream_id(seed, "golden.cv"), 0, nkv * cap * hd, 0.0, 1.0)
    out = O.sdpa_decode(q, ck, cv, nq, nkv, hd, cap, kv_len, hd ** -0.5)
    out64 = O.np_sdpa(q, ck, cv, nq, nkv, hd, cap, kv_len, hd ** -0.5)
    np.savez_compressed(os.path.join(OUT, "sdpa.npz"), q=q, ck=ck, cv=cv, out=out, out64=out64,
                        shape=np.array([nq, nkv, hd, cap, kv_len]))


def model_case(name, ctx, steps):
    spec = CONFIGS[name]
    cap = ctx + steps + 8
    m = O.Model(oracle_config(spec, cap))
    m.prefill_kv(ctx)
    tok, toks, hid0 = 3, [], None
    for i in range(steps):
        tok, hid, _ = m.step(tok, ctx + i, want_hidden=(i == 0))
        if i == 0:
            hid0 = hid
        toks.append(tok)
    np.savez_compressed(os.path.join(OUT, f"model_{name}.npz"), tokens=np.array(toks, np.uint32), hidden0=hid0,
                        ctx=np.array([ctx]), capacity=np.array([cap]), first_token=np.array([3]))


if __name__ == "__main__":
    for b in (4, 8, 16):
        qmatvec_case(b)
    pointwise_case()
    sdpa_case()
    model_case("tiny-qwen", 20, 24)
    model_case("tiny-gemma", 37, 24)
    print("golden fixtures written to", OUT)
