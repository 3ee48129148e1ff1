"""GPU parity of each decode kernel against the CPU oracle, called through the C ABI."""
import ctypes as C
import math

import numpy as np
import pytest

from fusekit_b200 import _native as N
from fusekit_b200.model_spec import stream_id
from oracle import oracle as O
from tests.helpers import assert_close_bf16, bf

pytestmark = pytest.mark.gpu
T = N.Task.make


def dev_weight(rt, w: O.QWeight, rope_rows=None, finalize=True) -> int:
    """Upload MLX-layout tensors; `rope_rows=(head_dim, n_rot_rows)` asks for the RoPE-pair tile order."""
    wid = rt.weight_alloc(w.n, w.k, w.bits)
    if w.bits == 16:
        rt.weight_upload_rows(wid, 0, w.dense)
    else:
        rt.weight_upload_rows(wid, 0, w.packed, w.scales, w.biases)
    if rope_rows and rt.tiled:
        rt.weight_set_rows(wid, 1, *rope_rows)
    if finalize:
        rt.weight_finalize(wid)
    return wid


def gateup_bufs(rt, wg: O.QWeight, wu: O.QWeight) -> dict:
    if rt.tiled:
        return {2: rt.weight_pair(dev_weight(rt, wg, finalize=False), dev_weight(rt, wu, finalize=False)), 3: 0}
    return {2: dev_weight(rt, wg), 3: dev_weight(rt, wu)}


def normal(name, n, std=1.0, mean=0.0, seed=99):
    return O.fill_normal_bf16(stream_id(seed, name), 0, n, mean, std)


def test_smoke_add_is_exact(runtime):
    a, b = normal("sa", 1024), normal("sb", 1024)
    got = runtime.smoke(a, b)
    assert np.array_equal(got, O.f32_to_bf16(bf(a) + bf(b)))      # max abs err 0.0, as the reference's smoke reports


@pytest.mark.parametrize("bits", [4, 8, 16])
def test_device_generator_and_dequant_are_bit_exact(runtime, bits):
    n, k, kg, row0, k0 = 40, 320, 640, 17, 192
    s = stream_id(4, f"gen{bits}")
    ref = O.gen_weight(s, n, k, bits, k_global=kg, row0=row0, k0=k0)
    wid = runtime.weight_alloc(n + 8, k, bits)
    runtime.weight_synth_rows(wid, 8, n, s, 0.02, kg, row0, k0)      # rows land at dst row 8
    runtime.weight_synth_rows(wid, 0, 8, s, 0.02, kg, 0, k0)
    runtime.weight_finalize(wid)
    got = runtime.weight_dequant(wid, 8, n, k)
    want = bf(ref.dense) if bits == 16 else O.dequant(ref)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    up = dev_weight(runtime, ref)                                    # uploaded MLX-layout tensors dequantise identically
    assert np.array_equal(runtime.weight_dequant(up, 0, n, k).view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("bits", [4, 8])
def test_repacked_layouts_dequantise_bit_exactly(runtime, bits):
    """Bit-exact dequantised weights out of the streaming layout: plain rows with ragged N and K, RoPE-pair
    row order, and the gate/up interleave."""
    rt = runtime
    for n, k, rope in ((100, 896, None), (48, 4864, None), ((4 + 2 * 2) * 64, 320, (64, (4 + 2) * 64))):
        w = O.gen_weight(stream_id(8, f"rp{bits}.{n}.{k}"), n, k, bits)
        wid = dev_weight(rt, w, rope_rows=rope)
        assert np.array_equal(rt.weight_dequant(wid, 0, n, k).view(np.uint32), O.dequant(w).view(np.uint32)), (n, k, rope)
        assert np.array_equal(rt.weight_dequant(wid, n - 7, 7, k).view(np.uint32), O.dequant(w)[n - 7:].view(np.uint32))
    wg, wu = O.gen_weight(stream_id(8, f"pg{bits}"), 40, 576, bits), O.gen_weight(stream_id(8, f"pu{bits}"), 40, 576, bits)
    pid = gateup_bufs(rt, wg, wu)[2]
    assert np.array_equal(rt.weight_dequant(pid, 0, 40, 576).view(np.uint32), O.dequant(wg).view(np.uint32))
    assert np.array_equal(rt.weight_dequant(pid, 40, 40, 576).view(np.uint32), O.dequant(wu).view(np.uint32))


def test_device_normal_fill_matches_oracle(runtime):
    s = stream_id(4, "vec")
    p = runtime.alloc(5000 * 2)
    runtime.synth_normal(p, s, 123, 5000, 1.0, 0.02)
    assert np.array_equal(runtime.download(p, (5000,), np.uint16), O.fill_normal_bf16(s, 123, 5000, 1.0, 0.02))


SHAPES = [(896, 1152), (896, 100), (4864, 896), (3584, 512), (18944, 96), (2560, 64), (64, 8), (5120, 72)]


@pytest.mark.parametrize("bits", [4, 8, 16])
@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("residual", [False, True])
def test_linear_residual(runtime, bits, k, n, residual):
    w = O.gen_weight(stream_id(1, f"lin{bits}.{k}.{n}"), n, k, bits)
    x, res = normal(f"x{k}", k), normal(f"r{n}", n)
    want = O.qmatvec(w, x, res if residual else None)
    xd, yd = runtime.to_device(x), runtime.alloc(n * 2)
    rd = runtime.to_device(res) if residual else 0
    runtime.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: xd, 1: dev_weight(runtime, w), 2: rd, 3: yd}, [k, n]))
    assert_close_bf16(runtime.download(yd, (n,), np.uint16), want, f"linear q{bits} {k}->{n}")


@pytest.mark.parametrize("m", [2, 5, 8, 13, 16])
@pytest.mark.parametrize("k,n", [(896, 1152), (896, 100), (4864, 896), (3584, 4736), (18944, 96), (64, 8), (512, 4800), (256, 9600), (320, 17088), (128, 34304)])
@pytest.mark.parametrize("residual", [False, True])
def test_linear_residual_rows(runtime, m, k, n, residual):
    """2..16 activation rows through one weight: row i equals the one-row task's result for x[i] (the oracle of a batch)."""
    w = O.gen_weight(stream_id(1, f"qmm.{k}.{n}"), n, k, 4)
    x, res = normal(f"qx{k}.{m}", m * k).reshape(m, k), normal(f"qr{n}.{m}", m * n).reshape(m, n)
    want = np.stack([O.qmatvec(w, x[i], res[i] if residual else None) for i in range(m)])
    xd, yd = runtime.to_device(x), runtime.alloc(m * n * 2)
    rd = runtime.to_device(res) if residual else 0
    runtime.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: xd, 1: dev_weight(runtime, w), 2: rd, 3: yd}, [k, n, m]))
    got = runtime.download(yd, (m, n), np.uint16)
    for i in range(m):
        assert_close_bf16(got[i], want[i], f"qmm row {i}/{m} {k}->{n}")
    assert runtime.state_get()[2] == 0


@pytest.mark.parametrize("m", [2, 8, 16, 17, 32])
@pytest.mark.parametrize("k,n", [(896, 1152), (896, 100), (4864, 896), (3584, 4736), (64, 8), (320, 1088)])
@pytest.mark.parametrize("residual", [False, True])
def test_linear_residual_rows_tcgen05(runtime, m, k, n, residual):
    """The same product on the 5th-generation tensor cores (weight rows on the MMA's M axis, activation rows on N,
    accumulators in tensor memory): up to 32 rows, each equal to the one-row task's result."""
    w = O.gen_weight(stream_id(1, f"qmm.{k}.{n}"), n, k, 4)
    x, res = normal(f"qx{k}.{m}", m * k).reshape(m, k), normal(f"qr{n}.{m}", m * n).reshape(m, n)
    want = np.stack([O.qmatvec(w, x[i], res[i] if residual else None) for i in range(m)])
    xd, yd = runtime.to_device(x), runtime.alloc(m * n * 2)
    rd = runtime.to_device(res) if residual else 0
    runtime.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: xd, 1: dev_weight(runtime, w), 2: rd, 3: yd}, [k, n, m, 0, 0, 1]))
    got = runtime.download(yd, (m, n), np.uint16)
    for i in range(m):
        assert_close_bf16(got[i], want[i], f"tcgen05 qmm row {i}/{m} {k}->{n}")
    assert runtime.state_get()[2] == 0


@pytest.mark.parametrize("m", [2, 7, 16])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("h,inter", [(896, 4864), (256, 100), (3584, 1024), (512, 19200)])
def test_rmsnorm_gateup_act_rows(runtime, m, act, h, inter):
    """2..16 activation rows through the norm-first gate/up task: row i equals the one-row task's result for x[i]."""
    rt = runtime
    if not rt.tiled:
        pytest.skip("streamed weight layout only")
    wg = O.gen_weight(stream_id(3, f"qg.{h}.{inter}"), inter, h, 4)
    wu = O.gen_weight(stream_id(3, f"qu.{h}.{inter}"), inter, h, 4)
    x, nw = normal(f"qgx{m}", m * h, 40.0).reshape(m, h), normal("qgnw", h, 0.02, 1.0)
    want = []
    for i in range(m):
        nf = O.rmsnorm(x[i], nw, 1e-6)
        want.append(O.act(O.linear_acc(wg, nf), O.linear_acc(wu, nf), act))
    out = rt.alloc(m * inter * 2)
    rt.launch(T(N.TASK_RMSNORM_GATEUP_ACT, 0, {0: rt.to_device(x), 1: rt.to_device(nw), **gateup_bufs(rt, wg, wu), 4: out},
                [h, inter, act, m], [1e-6]))
    got = rt.download(out, (m, inter), np.uint16)
    bufs = {1: rt.to_device(nw), **gateup_bufs(rt, wg, wu)}
    one = rt.alloc(inter * 2)
    for i in range(m):
        # The sum of squares is added in another order than the oracle's, so 1/rms can differ in its last bit; now and then
        # that flips one normalised activation by a bf16 ulp, which moves every output a little and a third of them across
        # a rounding boundary (seen at H = 3584: relative RMS 2.2e-3, the one-row kernel showing the very same deviation).
        # Hence the wider bound against the oracle, and the tight one against the one-row kernel, which shares the order.
        assert_close_bf16(got[i], want[i], f"gateup rows {i}/{m} act{act} {h}->{inter}", rel_rms_tol=4e-3)
        rt.launch(T(N.TASK_RMSNORM_GATEUP_ACT, 0, {0: rt.to_device(x[i].copy()), **bufs, 4: one}, [h, inter, act], [1e-6]))
        # two kernels with different summation orders, each within the bar of the oracle: against each other they get twice
        # the relative-RMS bound
        assert_close_bf16(got[i], rt.download(one, (inter,), np.uint16), f"gateup rows {i}/{m} against the one-row kernel", rel_rms_tol=2e-3)
    assert rt.state_get()[2] == 0


def test_linear_residual_rows_refusals(runtime):
    rt = runtime
    w8 = O.gen_weight(stream_id(1, "qmm8"), 16, 64, 8)
    with pytest.raises(N.FusekitError, match="4-bit"):
        rt.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: rt.alloc(4 * 64 * 2), 1: dev_weight(rt, w8), 3: rt.alloc(4 * 16 * 2)}, [64, 16, 4]))
    w4 = O.gen_weight(stream_id(1, "qmm4"), 16, 64, 4)
    with pytest.raises(N.FusekitError, match="at most 16"):
        rt.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: rt.alloc(17 * 64 * 2), 1: dev_weight(rt, w4), 3: rt.alloc(17 * 16 * 2)}, [64, 16, 17]))


@pytest.mark.parametrize("bits", [4, 8, 16])
@pytest.mark.parametrize("h,nq,nkv,hd,pos,cap", [(896, 14, 2, 64, 37, 64), (512, 4, 2, 128, 700, 512), (256, 2, 1, 256, 5, 16)])
def test_rmsnorm_qkv_rope_store(runtime, bits, h, nq, nkv, hd, pos, cap):
    n = (nq + 2 * nkv) * hd
    w = O.gen_weight(stream_id(2, f"qkv{bits}.{h}"), n, h, bits)
    x, nw, lb = normal("qx", h, 1.3), normal("qnw", h, 0.02, 1.0), normal("qb", n, 0.02)
    theta, eps = 1e6, 1e-6
    w.lin_bias = lb
    nf = O.rmsnorm(x, nw, eps)
    acc = O.linear_acc(w, nf)
    y = O.f32_to_bf16(acc)
    q = O.rope(y[:nq * hd], nq, hd, pos, theta)
    kk = O.rope(y[nq * hd:(nq + nkv) * hd], nkv, hd, pos, theta)
    v = y[(nq + nkv) * hd:]
    rt = runtime
    ck, cv, qd = rt.alloc(nkv * cap * hd * 2), rt.alloc(nkv * cap * hd * 2), rt.alloc(nq * hd * 2)
    rt.state_set(0, pos)
    rt.launch(T(N.TASK_RMSNORM_QKV, 0, {0: rt.to_device(x), 1: rt.to_device(nw), 2: dev_weight(rt, w, rope_rows=(hd, (nq + nkv) * hd)),
                                        3: rt.to_device(lb), 4: qd, 5: ck, 6: cv}, [h, nq, nkv, hd, cap, 1], [eps, theta]))
    row = pos % cap
    assert_close_bf16(rt.download(qd, (nq * hd,), np.uint16), q, "q")
    gk = rt.download(ck, (nkv, cap, hd), np.uint16)
    gv = rt.download(cv, (nkv, cap, hd), np.uint16)
    assert_close_bf16(gk[:, row].reshape(-1), kk, "k row")
    assert_close_bf16(gv[:, row].reshape(-1), v, "v row")
    mask = np.ones(cap, bool); mask[row] = False
    assert not gk[:, mask].any() and not gv[:, mask].any()           # only the write row is touched
    # without sinks the raw projections come back
    ko, vo = rt.alloc(nkv * hd * 2), rt.alloc(nkv * hd * 2)
    rt.launch(T(N.TASK_RMSNORM_QKV, 0, {0: rt.to_device(x), 1: rt.to_device(nw), 2: dev_weight(rt, w), 3: rt.to_device(lb),
                                        4: qd, 7: ko, 8: vo}, [h, nq, nkv, hd, cap, 0], [eps, theta]))
    assert_close_bf16(rt.download(qd, (nq * hd,), np.uint16), y[:nq * hd], "raw q")
    assert_close_bf16(rt.download(ko, (nkv * hd,), np.uint16), y[nq * hd:(nq + nkv) * hd], "raw k")


@pytest.mark.parametrize("variant", [0, 1, 2, 4])   # by shape, FMA cluster, global partials + ticket, tensor-core cluster
@pytest.mark.parametrize("nq,nkv,hd", [(14, 2, 64), (28, 4, 128), (8, 4, 256), (5, 1, 128), (1, 1, 64), (40, 8, 128)])
@pytest.mark.parametrize("pos,cap", [(0, 64), (62, 64), (63, 64), (64, 200), (136, 200), (199, 200), (1000, 96), (1030, 2100), (3000, 2100)])
def test_sdpa_decode(runtime, nq, nkv, hd, pos, cap, variant):
    if variant == 1 and hd == 256 and nq // nkv > 2:
        pytest.skip("the FMA cluster kernel takes at most two q heads per kv head at head_dim 256")
    if cap > 1000 and (nq, nkv) not in ((28, 4), (40, 8)):
        pytest.skip("long caches are exercised on the benchmark shapes only")
    rt = runtime
    q = normal(f"sq{nq}", nq * hd)
    ck, cv = normal(f"sk{hd}", nkv * cap * hd), normal(f"sv{hd}", nkv * cap * hd)
    kv_len = min(pos + 1, cap)
    scale = 1.0 / math.sqrt(hd)
    want = O.sdpa_decode(q, ck, cv, nq, nkv, hd, cap, kv_len, scale)
    chunks = (cap + 31) // 32
    out, part, cnt = rt.alloc(nq * hd * 2), rt.alloc(nq * chunks * (hd + 2) * 4), rt.alloc(nkv * 4)
    task = T(N.TASK_SDPA_DECODE, 0, {0: rt.to_device(q), 1: rt.to_device(ck), 2: rt.to_device(cv), 3: out, 4: part, 5: cnt},
             [nq, nkv, hd, cap, variant], [scale])
    rt.state_set(0, pos)
    rt.launch(task)
    got = rt.download(out, (nq * hd,), np.uint16)
    assert_close_bf16(got, want, f"sdpa kv_len {kv_len} variant {variant}")
    rt.launch(task)                                                   # the ticket counters reset themselves
    assert np.array_equal(rt.download(out, (nq * hd,), np.uint16), got)
    assert not rt.download(cnt, (nkv,), np.uint32).any()


@pytest.mark.parametrize("variant", [0, 2, 4])
@pytest.mark.parametrize("nq,nkv,hd", [(28, 4, 128), (40, 8, 128), (8, 4, 256)])
@pytest.mark.parametrize("pos", [4095, 4096, 4351, 5000])
def test_sdpa_decode_at_benchmark_capacity(runtime, nq, nkv, hd, pos, variant):
    """The capacities the 4096-token benchmark configurations run at (4096 + decoded tokens; the reference's own kernel
    stopped at 4096 keys, sdpa_decode.rs:76): last position before 4096, the first after, the last row of the cache and
    a wrapped ring position."""
    rt, cap = runtime, 4352
    q = normal(f"bq{nq}", nq * hd)
    ck, cv = normal(f"bk{hd}", nkv * cap * hd), normal(f"bv{hd}", nkv * cap * hd)
    kv_len, scale = min(pos + 1, cap), 1.0 / math.sqrt(hd)
    want = O.sdpa_decode(q, ck, cv, nq, nkv, hd, cap, kv_len, scale)
    chunks = (cap + 31) // 32
    out, part, cnt = rt.alloc(nq * hd * 2), rt.alloc(nq * chunks * (hd + 2) * 4), rt.alloc(nkv * 4)
    bufs = [rt.to_device(q), rt.to_device(ck), rt.to_device(cv)]
    task = T(N.TASK_SDPA_DECODE, 0, {0: bufs[0], 1: bufs[1], 2: bufs[2], 3: out, 4: part, 5: cnt}, [nq, nkv, hd, cap, variant], [scale])
    rt.state_set(0, pos)
    rt.launch(task)
    assert_close_bf16(rt.download(out, (nq * hd,), np.uint16), want, f"sdpa capacity {cap} kv_len {kv_len} variant {variant}")
    for p in bufs + [out, part, cnt]:
        N.check(rt.L.fk_free(rt.h, p), "fk_free")


@pytest.mark.parametrize("bits", [4, 8, 16])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("h,inter", [(896, 4864), (256, 100)])
def test_rmsnorm_gateup_act(runtime, bits, act, h, inter):
    rt = runtime
    wg = O.gen_weight(stream_id(3, f"g{bits}.{h}"), inter, h, bits)
    wu = O.gen_weight(stream_id(3, f"u{bits}.{h}"), inter, h, bits)
    x, nw = normal("gx", h, 40.0), normal("gnw", h, 0.02, 1.0)       # large activations exercise the tails
    nf = O.rmsnorm(x, nw, 1e-6)
    want = O.act(O.linear_acc(wg, nf), O.linear_acc(wu, nf), act)
    out = rt.alloc(inter * 2)
    rt.launch(T(N.TASK_RMSNORM_GATEUP_ACT, 0, {0: rt.to_device(x), 1: rt.to_device(nw), **gateup_bufs(rt, wg, wu), 4: out},
                [h, inter, act], [1e-6]))
    assert_close_bf16(rt.download(out, (inter,), np.uint16), want, f"gateup act{act}")


def test_pending_norm_prologue(runtime):
    """Gemma-shaped residual advance fused into the next kernel's prologue: x' = T(x + rmsnorm(y, w_post))."""
    rt, h, inter = runtime, 320, 128
    wg, wu = O.gen_weight(stream_id(3, "pg"), inter, h, 4), O.gen_weight(stream_id(3, "pu"), inter, h, 4)
    x, y, wp, nw = normal("px", h), normal("py", h, 3.0), normal("pw", h, 0.02, 1.0), normal("pn", h, 0.02, 1.0)
    hnew = O.f32_to_bf16(bf(x) + O.rmsnorm(y, wp, 1e-6))
    nf = O.rmsnorm(hnew, nw, 1e-6)
    want = O.act(O.linear_acc(wg, nf), O.linear_acc(wu, nf), 1)
    out, hout = rt.alloc(inter * 2), rt.alloc(h * 2)
    rt.launch(T(N.TASK_RMSNORM_GATEUP_ACT, 0, {0: rt.to_device(x), 1: rt.to_device(nw), **gateup_bufs(rt, wg, wu), 4: out,
                                               9: rt.to_device(y), 10: rt.to_device(wp), 11: hout}, [h, inter, 1], [1e-6]))
    got_h = rt.download(hout, (h,), np.uint16)
    assert np.mean(got_h != hnew) < 0.02
    assert_close_bf16(got_h, hnew, "advanced residual")
    assert_close_bf16(rt.download(out, (inter,), np.uint16), want, "gateup after pending norm")


@pytest.mark.parametrize("bits", [4, 8, 16])
def test_final_head_argmax(runtime, bits):
    rt, h, v = runtime, 896, 5000
    w = O.gen_weight(stream_id(5, f"head{bits}"), v, h, bits)
    x, nw = normal("hx", h, 2.0), normal("hnw", h, 0.02, 1.0)
    nf = O.rmsnorm(x, nw, 1e-6)
    want_logits = O.f32_to_bf16(O.linear_acc(w, nf))
    lg, scr, cnt = rt.alloc(v * 2), rt.alloc(8192), rt.alloc(4)
    rt.state_set(7, 11)
    rt.launch(T(N.TASK_FINAL_RMSNORM_LM_HEAD, -1, {0: rt.to_device(x), 1: rt.to_device(nw), 2: dev_weight(rt, w), 3: lg, 4: scr, 5: cnt},
                [h, v, 0, 1], [1e-6]))
    got = rt.download(lg, (v,), np.uint16)
    assert_close_bf16(got, want_logits, "logits")
    tok, off, err = rt.state_get()
    assert err == 0 and off == 12                                     # the state advanced on the device
    assert tok == O.argmax_bf16(got)                                  # argmax of the T-rounded logits, lowest index on ties
    top = np.sort(bf(want_logits))[-2:]
    if top[1] - top[0] > 0.02:
        assert tok == O.argmax_bf16(want_logits)


def test_argmax_tie_breaks_to_lowest_index(runtime):
    rt, h, v = runtime, 64, 300
    # identical rows -> identical logits everywhere: the winner must be index 0 (+ vocab offset)
    row = O.gen_weight(stream_id(6, "tie"), 1, h, 16)
    w = O.QWeight(v, h, 16, None, None, None, dense=np.repeat(row.dense, v, axis=0))
    x, nw = normal("tx", h), normal("tnw", h, 0.02, 1.0)
    scr, cnt = rt.alloc(8192), rt.alloc(4)
    rt.state_set(0, 0)
    rt.launch(T(N.TASK_FINAL_RMSNORM_LM_HEAD, -1, {0: rt.to_device(x), 1: rt.to_device(nw), 2: dev_weight(rt, w), 4: scr, 5: cnt},
                [h, v, 1000, 1], [1e-6]))
    assert rt.state_get()[0] == 1000


def test_qk_norm_rope_store(runtime):
    rt, nq, nkv, hd, cap, pos = runtime, 4, 2, 256, 16, 37
    q, k, v = normal("nq", nq * hd, 2.0), normal("nk", nkv * hd, 2.0), normal("nv", nkv * hd)
    wq, wk = normal("wq", hd, 0.02, 1.0), normal("wk", hd, 0.02, 1.0)
    def hn(vec, heads, w):
        return np.concatenate([O.f32_to_bf16(O.rmsnorm(vec[i * hd:(i + 1) * hd], w, 1e-6)) for i in range(heads)])
    want_q = O.rope(hn(q, nq, wq), nq, hd, pos, 1e4)
    want_k = O.rope(hn(k, nkv, wk), nkv, hd, pos, 1e4)
    qd, ck, cv = rt.to_device(q), rt.alloc(nkv * cap * hd * 2), rt.alloc(nkv * cap * hd * 2)
    rt.state_set(0, pos)
    rt.launch(T(N.TASK_QK_NORM_ROPE_STORE, 0, {0: qd, 1: rt.to_device(k), 2: rt.to_device(v), 3: rt.to_device(wq), 4: rt.to_device(wk), 5: ck, 6: cv},
                [nq, nkv, hd, cap], [1e-6, 1e4]))
    assert_close_bf16(rt.download(qd, (nq * hd,), np.uint16), want_q, "q")
    row = pos % cap
    assert_close_bf16(rt.download(ck, (nkv, cap, hd), np.uint16)[:, row].reshape(-1), want_k, "k")
    assert np.array_equal(rt.download(cv, (nkv, cap, hd), np.uint16)[:, row].reshape(-1), v)


def test_embed_lookup(runtime):
    rt, vocab, h = runtime, 50, 96
    table = normal("emb", vocab * h, 0.02)
    out = rt.alloc(h * 2)
    rt.state_set(31, 0)
    rt.launch(T(N.TASK_EMBED_LOOKUP_DECODE, -1, {0: rt.to_device(table), 1: out}, [h, 1], [50.5]))
    want = O.f32_to_bf16(bf(table.reshape(vocab, h)[31]) * np.float32(50.5))
    assert np.array_equal(rt.download(out, (h,), np.uint16), want)


def test_bad_arguments_are_refused(runtime):
    rt = runtime
    with pytest.raises(N.FusekitError, match="weight missing"):
        rt.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: rt.alloc(64), 1: 9999, 3: rt.alloc(64)}, [64, 8]))
    w = O.gen_weight(stream_id(1, "bad"), 8, 64, 4)
    with pytest.raises(N.FusekitError, match="shape mismatch"):
        rt.launch(T(N.TASK_LINEAR_RESIDUAL, 0, {0: rt.alloc(64), 1: dev_weight(rt, w), 3: rt.alloc(64)}, [128, 8]))
    with pytest.raises(N.FusekitError, match="unknown task kind"):
        rt.launch(T(77))
    wid = C.c_uint64()
    assert rt.L.fk_weight_alloc(rt.h, 8, 100, 4, C.byref(wid)) == -1     # k must be a multiple of the group size
