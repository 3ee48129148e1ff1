"""Quantised KV cache: the RoPE + quantising store and the attention over packed keys / values against the oracle's
restatement of src/codegen/kernels/rope_kv_cache_store_decode_quant.rs and sdpa_decode_quant.rs, then whole decode steps."""
import math

import numpy as np
import pytest

from fusekit_b200 import _native as N
from fusekit_b200.model_spec import CONFIGS, stream_id
from fusekit_b200.runtime import DecodeEngine
from oracle import oracle as O
from tests.helpers import assert_close_bf16, compare_greedy, oracle_config

T = N.Task.make


def normal(name, n, std=1.0):
    return O.fill_normal_bf16(stream_id(11, name), 0, n, 0.0, std)


def deq_rows(packed, sc, bi, rows, hd, bits):
    per, ng = 32 // bits, hd // 64
    p = packed.reshape(rows, hd // per)
    q = np.stack([(p >> (j * bits)) & ((1 << bits) - 1) for j in range(per)], axis=-1).reshape(rows, hd).astype(np.float32)
    s = np.repeat(O.bf16_to_f32(sc).reshape(rows, ng), 64, axis=1); b = np.repeat(O.bf16_to_f32(bi).reshape(rows, ng), 64, axis=1)
    return q * s + b


def test_oracle_quantiser_properties():
    """Edge-anchored rule: the edge of larger magnitude is represented exactly (up to the T rounding of scale and bias), every
    value lies within half a step, constant groups give all-equal codes."""
    rng = np.random.default_rng(1)
    for bits in (4, 8):
        x = rng.standard_normal(256).astype(np.float32) * 3
        p, s, b = O.kv_quantize_row(x, bits)
        d = deq_rows(p, s, b, 1, 256, bits)[0]
        step = np.repeat([(x[g * 64:(g + 1) * 64].max() - x[g * 64:(g + 1) * 64].min()) / (2 ** bits - 1) for g in range(4)], 64)
        # within one step: re-anchoring the grid at the edge (scale = edge / q0) stretches it by up to half a code at the far
        # end, and rounding scale and bias to bf16 costs another 2^-9 relative of the scale times the code and of the edge
        assert np.all(np.abs(d - x) <= 1.0 * step + (2 ** bits) * step * 2.0 ** -8 + np.abs(x).max() * 2.0 ** -7)
        assert np.mean(np.abs(d - x) <= 0.5 * step) > 0.6
    p, s, b = O.kv_quantize_row(np.full(64, 2.5, np.float32), 4)
    assert len(set(((p[i // 8] >> ((i % 8) * 4)) & 15) for i in range(64))) == 1


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 64), (28, 4, 128), (8, 4, 256)])
@pytest.mark.parametrize("pos,cap", [(0, 64), (37, 64), (200, 96)])
def test_quantising_store_matches_the_oracle(runtime, bits, nq, nkv, hd, pos, cap):
    rt, theta = runtime, 1e6
    q, k, v = normal("kq.q", nq * hd), normal("kq.k", nkv * hd), normal("kq.v", nkv * hd)
    rows, per, ng = nkv * cap, 32 // bits, hd // 64
    bufs = {0: rt.to_device(q), 1: rt.to_device(k), 2: rt.to_device(v), 3: rt.alloc(rows * hd * bits // 8), 4: rt.alloc(rows * hd * bits // 8),
            5: rt.alloc(rows * ng * 2), 6: rt.alloc(rows * ng * 2), 7: rt.alloc(rows * ng * 2), 8: rt.alloc(rows * ng * 2)}
    rt.state_set(0, pos)
    rt.launch(T(N.TASK_KV_STORE_QUANT, 0, bufs, [nq, nkv, hd, cap, bits], [0.0, theta]))
    assert_close_bf16(rt.download(bufs[0], (nq * hd,), np.uint16), O.rope(q, nq, hd, pos, theta), "q rope")
    row = pos % cap
    kr = O.rope_f32(k, nkv, hd, pos, theta).reshape(nkv, hd)
    vf = O.bf16_to_f32(v).reshape(nkv, hd)
    gp = {n: rt.download(bufs[i], (rows, hd // per) if i < 5 else (rows, ng), np.uint32 if i < 5 else np.uint16) for n, i in
          (("kp", 3), ("vp", 4), ("ks", 5), ("kb", 6), ("vs", 7), ("vb", 8))}
    for hh in range(nkv):
        r = hh * cap + row
        wp, ws, wb = O.kv_quantize_row(vf[hh], bits)                      # v has no rotation: bit-exact
        assert np.array_equal(gp["vp"][r], wp) and np.array_equal(gp["vs"][r], ws) and np.array_equal(gp["vb"][r], wb), ("v", hh)
        # k: the device's sincosf may differ from libm in the last bit, which can move a code by one step: compare dequantised
        wp, ws, wb = O.kv_quantize_row(kr[hh], bits)
        got = deq_rows(gp["kp"][r], gp["ks"][r], gp["kb"][r], 1, hd, bits)[0]
        want = deq_rows(wp, ws, wb, 1, hd, bits)[0]
        step = (kr[hh].max() - kr[hh].min()) / (2 ** bits - 1)
        assert np.abs(got - want).max() <= 1.01 * step and np.mean(got != want) <= 0.05, ("k", hh)
    others = np.ones(rows, bool); others[[hh * cap + row for hh in range(nkv)]] = False
    assert not gp["kp"][others].any() and not gp["vs"][others].any()      # only the row of this position is written
    for p in bufs.values():
        N.check(rt.L.fk_free(rt.h, p), "fk_free")


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 64), (28, 4, 128), (8, 4, 256)])
@pytest.mark.parametrize("pos,cap", [(0, 64), (63, 64), (100, 200), (700, 512)])
def test_quantised_attention_matches_the_oracle(runtime, bits, nq, nkv, hd, pos, cap):
    rt = runtime
    rows, per, ng = nkv * cap, 32 // bits, hd // 64
    rng = np.random.default_rng(pos + hd + bits)
    kp = rng.integers(0, 2 ** 32, (rows, hd // per), dtype=np.uint64).astype(np.uint32); vp = rng.integers(0, 2 ** 32, (rows, hd // per), dtype=np.uint64).astype(np.uint32)
    sc = lambda n: O.f32_to_bf16((rng.standard_normal((rows, ng)) * (0.3 if bits == 4 else 0.02)).astype(np.float32))
    ks, kb, vs, vb = sc(0), sc(1), sc(2), sc(3)
    q = normal(f"qa.q{nq}", nq * hd)
    kv_len, scale = min(pos + 1, cap), 1.0 / math.sqrt(hd)
    want = O.sdpa_decode_quant(q, kp, ks, kb, vp, vs, vb, nq, nkv, hd, cap, kv_len, scale, bits)
    chunks = (cap + 31) // 32
    bufs = {0: rt.to_device(q), 1: rt.to_device(kp), 2: rt.to_device(vp), 3: rt.alloc(nq * hd * 2), 4: rt.alloc(nq * chunks * (hd + 2) * 4), 5: rt.alloc(nkv * 4),
            6: rt.to_device(ks), 7: rt.to_device(kb), 8: rt.to_device(vs), 9: rt.to_device(vb)}
    rt.state_set(0, pos)
    task = T(N.TASK_SDPA_DECODE_QUANT, 0, bufs, [nq, nkv, hd, cap, bits], [scale])
    rt.launch(task)
    got = rt.download(bufs[3], (nq * hd,), np.uint16)
    assert_close_bf16(got, want, f"quantised sdpa q{bits} kv_len {kv_len}")
    rt.launch(task)                                                       # the ticket counters reset themselves
    assert np.array_equal(rt.download(bufs[3], (nq * hd,), np.uint16), got)
    for p in bufs.values():
        N.check(rt.L.fk_free(rt.h, p), "fk_free")


@pytest.mark.gpu
@pytest.mark.parametrize("name,bits,kv_bits", [("tiny-qwen", 4, 4), ("tiny-qwen", 4, 8), ("tiny-qwen", 8, 8), ("qwen2.5-0.5b", 4, 8)])
def test_decode_with_a_quantised_cache_matches_the_oracle(name, bits, kv_bits):
    """Whole decode steps with the cache kept quantised on both sides, starting from an empty cache."""
    spec = CONFIGS[name].with_bits(bits)
    steps, cap = 24, 64
    m = O.Model(oracle_config(spec, cap)); m.set_kv_quant(kv_bits)
    eng = DecodeEngine(spec, cap, kv_bits=kv_bits)
    try:
        eng.load_synthetic()
        kinds = [t.kind for t in eng.build_dispatches()]
        assert N.TASK_KV_STORE_QUANT in kinds and N.TASK_SDPA_DECODE_QUANT in kinds and N.TASK_SDPA_DECODE not in kinds
        got, _ = eng.decode_chunk(0, 5, steps)
        mism, ties = compare_greedy(got, m, 5, 0, tie_ulps=4.0 if name.startswith("tiny") else 2.0)
        assert not mism and len(ties) <= 3, (mism, ties)
    finally:
        eng.close(); m.close()


def test_quantised_cache_is_refused_where_it_is_not_wired():
    with pytest.raises(ValueError):
        DecodeEngine.__new__(DecodeEngine).__init__(CONFIGS["tiny-gemma"], 64, kv_bits=4)
    from fusekit_b200 import task_graph as TG
    with pytest.raises(ValueError):
        TG.emit(CONFIGS["tiny-qwen"], 64, tp_rank=0, tp_size=2, kv_bits=4)
    g = TG.emit(CONFIGS["tiny-qwen"], 64, kv_bits=8)
    assert [t["kind"] for t in g["tasks"]].count(TG.K_KVQ) == CONFIGS["tiny-qwen"].n_layers
