"""CPU tests of the oracle: the C restatement against an independent NumPy/torch restatement and
against the committed fixtures.  (The reference holds no golden vectors for this path.)"""
import os

import numpy as np
import pytest
import torch

from fusekit_b200.model_spec import CONFIGS, stream_id
from oracle import oracle as O
from tests.helpers import oracle_config

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_bf16_round_trip_matches_torch():
    rng = np.random.default_rng(0)
    f = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-6, 6, 4096),
                        np.array([0.0, -0.0, 1.0, 3.3895314e38, 1.0039062, 1.0117188, np.inf, -np.inf], np.float32)])
    want = torch.from_numpy(f).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = O.f32_to_bf16(f)
    assert np.array_equal(got, want)
    got_c = np.array([O.lib().fko_f32_to_bf16(float(v)) for v in f[:512]], np.uint16)
    assert np.array_equal(got_c, want[:512])
    assert np.array_equal(O.bf16_to_f32(want), torch.from_numpy(want.view(np.int16)).view(torch.bfloat16).float().numpy())


def test_generator_is_deterministic_and_near_normal():
    s = stream_id(1, "probe")
    a = O.bf16_to_f32(O.fill_normal_bf16(s, 0, 200000, 0.0, 1.0))
    b = O.bf16_to_f32(O.fill_normal_bf16(s, 0, 200000, 0.0, 1.0))
    assert np.array_equal(a, b)
    assert abs(a.mean()) < 0.01 and abs(a.std() - 1.0) < 0.01
    assert abs(((a - a.mean()) ** 4).mean() / a.var() ** 2 - 3.0) < 0.15       # kurtosis of a normal
    c = O.bf16_to_f32(O.fill_normal_bf16(s, 1000, 16, 0.0, 1.0))
    assert np.array_equal(c, a[1000:1016])                                       # index-addressed
    assert O.stream_id("lm_head") ^ 0 == stream_id(0, "lm_head") ^ (stream_id(0, "") ^ O.stream_id(""))


def test_python_stream_ids_match_c():
    for seed in (0, 7, 20240531):
        for l, fmt in ((3, "layers.%d.q_proj"), (0, "lm_head"), (11, "layers.%d.cache_k")):
            name = fmt % l if "%d" in fmt else fmt
            assert O.tensor_stream(seed, fmt, l) == stream_id(seed, name)


@pytest.mark.parametrize("bits", [4, 8])
def test_quantizer_layout_and_error_bound(bits):
    n, k = 32, 512
    s = stream_id(3, f"w{bits}")
    w = O.gen_weight(s, n, k, bits)
    assert w.packed.shape == (n, k * bits // 32) and w.scales.shape == (n, k // 64)
    deq_c, deq_np = O.dequant(w), O.np_dequant(w)
    assert np.array_equal(deq_c.view(np.uint32), deq_np.view(np.uint32))        # bit-exact dequant
    # the generated fp32 weights are 0.02 * z(stream, row*k + col)
    z = np.array([[O.lib().fko_unit_normal(s, r * k + c) for c in range(k)] for r in range(4)], np.float32)
    src = np.float32(0.02) * z
    sc = np.repeat(O.bf16_to_f32(w.scales[:4]), 64, axis=1)
    bi = np.repeat(O.bf16_to_f32(w.biases[:4]), 64, axis=1)
    qmax = (1 << bits) - 1
    # half a step, plus the bf16 rounding of the scale (felt at q = qmax) and of the bias
    assert np.all(np.abs(deq_c[:4] - src) <= 0.5 * sc + qmax * sc * 2.0 ** -8 + np.abs(bi) * 2.0 ** -8 + 1e-7)
    q = O.np_unpack(w.packed, bits)
    assert q.min() == 0 and q.max() == (1 << bits) - 1                          # every group spans the range
    # LSB-first: element j of a word sits at bit j*bits
    word = int(w.packed[0, 0])
    assert [(word >> (j * bits)) & ((1 << bits) - 1) for j in range(32 // bits)] == list(q[0, :32 // bits])


def test_tensor_parallel_slices_are_slices_of_the_full_tensor():
    s = stream_id(5, "slice")
    full = O.gen_weight(s, 64, 256, 4)
    rows = O.gen_weight(s, 16, 256, 4, k_global=256, row0=32)
    cols = O.gen_weight(s, 64, 128, 4, k_global=256, k0=128)
    assert np.array_equal(rows.packed, full.packed[32:48]) and np.array_equal(rows.scales, full.scales[32:48])
    assert np.array_equal(cols.packed, full.packed[:, 16:]) and np.array_equal(cols.biases, full.biases[:, 2:])


@pytest.mark.parametrize("bits", [4, 8, 16])
def test_qmatvec_against_fixture_and_float64(bits):
    g = np.load(os.path.join(GOLD, f"qmatvec_q{bits}.npz"))
    if bits == 16:
        w = O.QWeight(48, 256, 16, None, None, None, dense=g["dense"])
        deq = O.bf16_to_f32(w.dense)
    else:
        w = O.QWeight(48, 256, bits, g["packed"], g["scales"], g["biases"])
        deq = O.dequant(w)
        assert np.array_equal(deq.view(np.uint32), g["deq"].view(np.uint32))
    y = O.qmatvec(w, g["x"], g["res"])
    assert np.array_equal(y, g["y"])                                             # drift pin
    y64 = deq.astype(np.float64) @ O.bf16_to_f32(g["x"]).astype(np.float64) + O.bf16_to_f32(g["res"])
    assert np.allclose(y64, g["y64"], rtol=0, atol=1e-12)
    # one bf16 rounding of an fp32 sum: within half an ulp (2^-9 relative) plus fp32 accumulation noise
    assert np.all(np.abs(O.bf16_to_f32(y) - y64) <= np.abs(y64) * 2.0 ** -8 + 1e-4)


def test_pointwise_fixture_and_numpy_restatement():
    g = np.load(os.path.join(GOLD, "pointwise.npz"))
    rms = O.rmsnorm(g["x"], g["w"], 1e-6)
    assert np.array_equal(rms.view(np.uint32), g["rms"].view(np.uint32))
    rms_np = O.np_rmsnorm(g["x"], g["w"], 1e-6)
    assert np.mean(rms != rms_np) < 0.02 and np.max(np.abs(rms - rms_np)) <= 2.0 ** -7 * np.max(np.abs(rms))
    assert np.array_equal(O.bf16_to_f32(O.f32_to_bf16(rms)), rms)               # outputs are T-exact
    sw, ge = O.act(g["g"], g["u"], 0), O.act(g["g"], g["u"], 1)
    assert np.array_equal(sw, g["swiglu"]) and np.array_equal(ge, g["geglu"])
    for got, want in ((sw, O.np_swiglu(g["g"], g["u"])), (ge, O.np_geglu_tanh(g["g"], g["u"]))):
        d = np.abs(O.bf16_to_f32(got) - O.bf16_to_f32(want))
        assert np.mean(d > 0) < 0.02 and np.all(d <= np.abs(O.bf16_to_f32(want)) * 2.0 ** -7 + 1e-30)
    x = g["g"][:8].astype(np.float64)
    ref = 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3))) * g["u"][:8]
    assert np.allclose(O.bf16_to_f32(ge[:8]), ref, rtol=0.03, atol=1e-2)         # it is GELU-tanh(g)*u up to the per-op bf16 roundings
    r = O.rope(g["rope_in"], 4, 64, int(g["rope_pos"][0]), 1e6)
    assert np.array_equal(r, g["rope_out"])
    v = O.bf16_to_f32(g["rope_in"]).reshape(4, 64).astype(np.float64)
    d = np.arange(32)
    ang = 1234 * np.exp2(-(d / 32) * np.log2(1e6))
    want = np.concatenate([v[:, :32] * np.cos(ang) - v[:, 32:] * np.sin(ang), v[:, 32:] * np.cos(ang) + v[:, :32] * np.sin(ang)], axis=1)
    assert np.allclose(O.bf16_to_f32(r).reshape(4, 64), want, rtol=2.0 ** -7, atol=2e-3)


def test_rope_position_zero_is_identity():
    v = O.fill_normal_bf16(stream_id(2, "r0"), 0, 128, 0.0, 1.0)
    assert np.array_equal(O.rope(v, 2, 64, 0, 1e4), v)


def test_sdpa_fixture_and_float64_softmax():
    g = np.load(os.path.join(GOLD, "sdpa.npz"))
    nq, nkv, hd, cap, kv_len = (int(v) for v in g["shape"])
    out = O.sdpa_decode(g["q"], g["ck"], g["cv"], nq, nkv, hd, cap, kv_len, hd ** -0.5)
    assert np.array_equal(out, g["out"])
    want = O.np_sdpa(g["q"], g["ck"], g["cv"], nq, nkv, hd, cap, kv_len, hd ** -0.5)
    assert np.allclose(want, g["out64"], atol=1e-12)
    assert np.all(np.abs(O.bf16_to_f32(out) - want) <= np.abs(want) * 2.0 ** -8 + 2e-4)
    one = O.sdpa_decode(g["q"], g["ck"], g["cv"], nq, nkv, hd, cap, 1, hd ** -0.5)   # a single key: output = V[0]
    V = g["cv"].reshape(nkv, cap, hd)
    assert np.array_equal(one.reshape(nq, hd)[0], V[0, 0]) and np.array_equal(one.reshape(nq, hd)[nq - 1], V[nkv - 1, 0])


def test_argmax_rounds_to_bf16_and_prefers_lowest_index():
    lg = O.f32_to_bf16(np.array([-1.0, 2.0, 2.0, -3.0, 2.0], np.float32))
    assert O.argmax_bf16(lg) == 1
    assert O.argmax_bf16(O.f32_to_bf16(np.array([-5.0, -2.0, -2.0], np.float32))) == 1
    a = np.array([1.0, 1.001], np.float32)            # equal once rounded to bf16
    assert O.argmax_bf16(O.f32_to_bf16(a)) == 0


@pytest.mark.parametrize("name", ["tiny-qwen", "tiny-gemma"])
def test_model_fixture(name):
    g = np.load(os.path.join(GOLD, f"model_{name}.npz"))
    spec, ctx, cap = CONFIGS[name], int(g["ctx"][0]), int(g["capacity"][0])
    m = O.Model(oracle_config(spec, cap))
    m.prefill_kv(ctx)
    tok, toks = int(g["first_token"][0]), []
    for i in range(len(g["tokens"])):
        tok, hid, lg = m.step(tok, ctx + i, want_hidden=(i == 0), want_logits=(i == 0))
        if i == 0:
            assert np.array_equal(hid, g["hidden0"])
            assert tok == O.argmax_bf16(lg)
        toks.append(tok)
    assert toks == list(g["tokens"])
    assert len(set(toks)) > 1                           # the greedy stream is not degenerate


def test_ring_cache_rows_and_kv_len():
    spec = CONFIGS["tiny-gemma"]                        # window 16, every 3rd layer global
    m = O.Model(oracle_config(spec, 64))
    assert [m.layer_sliding(l) for l in range(3)] == [True, True, False]
    assert [m.layer_cap(l) for l in range(3)] == [16, 16, 64]
    assert m.layer_theta(0) == spec.theta_local and m.layer_theta(2) == spec.theta
    m.prefill_kv(40)
    k0 = m.vec(0, 7, 2 * 16 * 64).reshape(2, 16, 64).copy()
    want = O.fill_normal_bf16(stream_id(spec.seed, "layers.0.cache_k"), (0 * 1048576 + 37) * 64, 64, 0.0, 1.0)
    assert np.array_equal(k0[0, 37 % 16], want)         # position 37 lives at ring row 5
    m.step(1, 40)                                       # position 40 overwrites row 8
    k_after = m.vec(0, 7, 2 * 16 * 64).reshape(2, 16, 64)
    assert not np.array_equal(k_after[0, 8], k0[0, 8])
