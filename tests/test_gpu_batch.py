"""Batch decode of M independent sequences against M batch-1 oracle runs (the reference has no batch of sequences:
python/fusekit_runtime/dispatch.py:2268-2289; each row is defined as what the one-row path gives for that sequence)."""
import numpy as np
import pytest

from fusekit_b200.batch import BatchDecodeEngine, PrefillEngine
from fusekit_b200.model_spec import CONFIGS
from oracle import oracle as O
from tests.helpers import compare_greedy, oracle_config

pytestmark = pytest.mark.gpu


def oracle_for_sequence(spec, cap, ctx, m):
    """A batch-1 oracle whose caches hold sequence m's pre-fill (the same streams the engine fills on the device)."""
    model = O.Model(oracle_config(spec, cap))
    hd = spec.head_dim
    for l in range(spec.n_layers):
        k = np.zeros((spec.n_kv, cap, hd), np.uint16); v = np.zeros_like(k)
        for hh in range(spec.n_kv):
            idx0 = hh * 1048576 * hd
            k[hh, :ctx] = O.fill_normal_bf16(BatchDecodeEngine.cache_stream(spec, l, "k", m), idx0, ctx * hd, 0.0, 1.0).reshape(ctx, hd)
            v[hh, :ctx] = O.fill_normal_bf16(BatchDecodeEngine.cache_stream(spec, l, "v", m), idx0, ctx * hd, 0.0, 1.0).reshape(ctx, hd)
        model.set_cache(l, k, v)
    return model


@pytest.mark.parametrize("rows,qmm", [(2, 2), (5, 2), (16, 2), (16, 1), (7, 1)])       # qmm: 2 = mma.sync projections, 1 = tcgen05
def test_batch_decode_rows_match_batch1_oracle_runs(rows, qmm):
    spec, ctx, steps, cap = CONFIGS["tiny-qwen"], 20, 12, 64
    eng = BatchDecodeEngine(spec, cap, rows, qmm=qmm)
    try:
        eng.load_synthetic(); eng.prefill_kv_synthetic(ctx)
        seeds = np.array([3 + 7 * m for m in range(rows)], np.uint32)
        toks, secs = eng.decode_chunk(ctx, seeds, steps)
        assert toks.shape == (steps, rows) and secs > 0
        toks2, _ = eng.decode_chunk(ctx + steps, toks[-1], 3)          # a second chunk continues every sequence
        allt = np.concatenate([toks, toks2])
        for m in range(rows):
            model = oracle_for_sequence(spec, cap, ctx, m)
            mism, ties = compare_greedy(allt[:, m], model, int(seeds[m]), ctx, tie_ulps=4.0)
            assert not mism and len(ties) <= 2, (m, mism, ties)
            model.close()
        assert len({tuple(allt[:, m]) for m in range(rows)}) > 1         # the sequences really differ
    finally:
        eng.close()


def test_batch_engine_refuses_unsupported_models():
    with pytest.raises(ValueError):
        BatchDecodeEngine(CONFIGS["tiny-gemma"], 64, 4)
    with pytest.raises(ValueError):
        BatchDecodeEngine(CONFIGS["tiny-qwen"].with_bits(8), 64, 4)
    with pytest.raises(ValueError):
        BatchDecodeEngine(CONFIGS["tiny-qwen"], 64, 17)


@pytest.mark.parametrize("rows,qmm", [(8, 2), (16, 2), (5, 1)])
def test_chunked_prefill_matches_the_oracle_stepping_the_prompt(rows, qmm):
    """A 37-token prompt through the prefill engine in chunks of `rows` consecutive positions: the prediction after every
    position equals the oracle's when it steps the same prompt token by token, the caches agree with the oracle's within the
    stage tolerance, and the batch-1 engine decodes on from those caches."""
    from fusekit_b200.model_spec import stream_id
    from fusekit_b200.runtime import DecodeEngine
    from tests.helpers import assert_close_bf16
    spec, cap = CONFIGS["tiny-qwen"], 96
    prompt = [O.uniform_u32(stream_id(spec.seed, "prompt"), i, spec.vocab) for i in range(37)]
    m = O.Model(oracle_config(spec, cap))
    want = [m.step(t, i)[0] for i, t in enumerate(prompt)]
    dec = DecodeEngine(spec, cap)
    try:
        dec.load_synthetic()
        pre = PrefillEngine(spec, cap, rows, runtime=dec.rt, qmm=qmm, caches=dec.cache)
        pre.load_synthetic()
        got = pre.prefill(prompt)
        flips = [i for i in range(len(prompt)) if int(got[i]) != want[i]]
        assert len(flips) <= 2, (flips, got, want)             # near-ties of the toy head; the caches below are the stronger check
        hd = spec.head_dim
        for l in range(spec.n_layers):
            k = dec.rt.download(dec.cache[l][0], (spec.n_kv, cap, hd), np.uint16)[:, :len(prompt)]
            v = dec.rt.download(dec.cache[l][1], (spec.n_kv, cap, hd), np.uint16)[:, :len(prompt)]
            n = spec.n_kv * cap * hd
            ok_, ov = m.vec(l, 7, n).reshape(spec.n_kv, cap, hd)[:, :len(prompt)], m.vec(l, 8, n).reshape(spec.n_kv, cap, hd)[:, :len(prompt)]
            assert_close_bf16(k.reshape(-1), ok_.reshape(-1), f"cache_k layer {l}", rel_rms_tol=5e-3)
            assert_close_bf16(v.reshape(-1), ov.reshape(-1), f"cache_v layer {l}", rel_rms_tol=5e-3)
        # decode continues from the prefilled caches on the batch-1 engine
        nxt, _ = dec.decode_chunk(len(prompt), int(got[-1]), 8)
        m2 = O.Model(oracle_config(spec, cap))
        for i, t in enumerate(prompt):
            m2.step(t, i)
        mism, ties = compare_greedy(nxt, m2, int(got[-1]), len(prompt), tie_ulps=4.0)
        assert not mism and len(ties) <= 2, (mism, ties)
    finally:
        dec.close()
