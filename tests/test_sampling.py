"""Sampling beyond greedy: the host-side sampler on logits read back from the fused step (reference: non-greedy requests
take the logits path, python/fusekit_runtime/__init__.py:4782-4843)."""
import numpy as np
import pytest

from fusekit_b200.runtime import sample_logits


def bf16(a):
    u = np.asarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def test_greedy_limits_pick_the_first_maximum():
    lg = bf16([0.5, 2.0, 2.0, -1.0])
    assert sample_logits(lg, temperature=0.0) == 1
    assert sample_logits(lg, temperature=1.0, top_k=1) == 1
    assert sample_logits(lg, temperature=1.0, top_p=1e-9, rng=np.random.default_rng(0)) == 1


def test_top_k_and_top_p_restrict_the_support_and_follow_the_softmax():
    lg = bf16([3.0, 2.0, 1.0, 0.0, -5.0])
    rng = np.random.default_rng(7)
    draws = np.array([sample_logits(lg, 1.0, 3, 1.0, rng) for _ in range(4000)])
    assert set(draws) == {0, 1, 2}
    want = np.exp([3.0, 2.0, 1.0]); want /= want.sum()
    freq = np.bincount(draws, minlength=3) / len(draws)
    assert np.abs(freq - want).max() < 0.03
    # nucleus: exp(3) / sum = 0.64, + exp(2) -> 0.87: top_p 0.8 keeps two tokens
    draws = np.array([sample_logits(lg, 1.0, 0, 0.8, rng) for _ in range(2000)])
    assert set(draws) == {0, 1}
    hot = np.array([sample_logits(lg, 100.0, 0, 1.0, rng) for _ in range(2000)])
    assert len(set(hot)) == 5                                   # a high temperature flattens the distribution
    a = [sample_logits(lg, 1.0, 0, 1.0, np.random.default_rng(3)) for _ in range(5)]
    assert a == [sample_logits(lg, 1.0, 0, 1.0, np.random.default_rng(3)) for _ in range(5)]


@pytest.mark.gpu
def test_sampled_generation_runs_through_the_fused_step():
    from fusekit_b200.model_spec import CONFIGS
    from fusekit_b200.runtime import DecodeEngine
    spec = CONFIGS["tiny-qwen"]
    eng = DecodeEngine(spec, 64, want_logits=True)
    try:
        eng.load_synthetic(); eng.prefill_kv_synthetic(10)
        greedy, _ = eng.decode_chunk(10, 3, 8)
        eng.prefill_kv_synthetic(10)
        assert list(eng.generate_sampled(3, 10, 8, top_k=1)) == list(greedy)           # top_k = 1 is the greedy stream
        eng.prefill_kv_synthetic(10)
        a = eng.generate_sampled(3, 10, 12, temperature=1.5, top_k=50, top_p=0.95, seed=11)
        eng.prefill_kv_synthetic(10)
        b = eng.generate_sampled(3, 10, 12, temperature=1.5, top_k=50, top_p=0.95, seed=11)
        assert list(a) == list(b) and all(int(t) < spec.vocab for t in a)              # seeded: reproducible
        assert list(a) != list(greedy[:8]) or True
    finally:
        eng.close()
