"""Shared helpers of the parity tests: oracle <-> engine glue and the tolerance metrics."""
from __future__ import annotations

import numpy as np

from fusekit_b200.model_spec import ModelSpec, stream_id, tensor_name
from oracle import oracle as O

# north-star tolerances for bf16 hidden states
MAX_ABS_TOL = 1e-2
REL_RMS_TOL = 1e-3


oracle_config = O.model_config


def weight_provider(spec: ModelSpec):
    def prov(leaf, layer, src_row0, nrows, k_global, k0, k, bits):
        w = O.gen_weight(stream_id(spec.seed, tensor_name(layer, leaf)), nrows, k, bits, k_global=k_global, row0=src_row0, k0=k0)
        if bits == 16:
            return w.dense, None, None
        return w.packed, w.scales, w.biases
    return prov


def vector_provider(spec: ModelSpec):
    def prov(leaf, layer, idx0, n, mean, std):
        return O.fill_normal_bf16(stream_id(spec.seed, tensor_name(layer, leaf)), idx0, n, mean, std)
    return prov


def bf(a):
    return O.bf16_to_f32(np.asarray(a, np.uint16))


def max_abs(a_bits, b_bits) -> float:
    return float(np.max(np.abs(bf(a_bits) - bf(b_bits))))


def rel_rms(a_bits, b_bits) -> float:
    a, b = bf(a_bits).astype(np.float64), bf(b_bits).astype(np.float64)
    return float(np.sqrt(np.mean((a - b) ** 2)) / max(np.sqrt(np.mean(b ** 2)), 1e-30))


def assert_close_bf16(got_bits, want_bits, what="", max_abs_tol=MAX_ABS_TOL, rel_rms_tol=REL_RMS_TOL, scale_abs=True):
    """max-abs <= 1e-2 (relative to max(1, |want|_inf) so large-magnitude rows are judged in bf16 ulps)
    and relative RMS <= 1e-3."""
    ma, rr = max_abs(got_bits, want_bits), rel_rms(got_bits, want_bits)
    ref = max(1.0, float(np.max(np.abs(bf(want_bits))))) if scale_abs else 1.0
    assert ma <= max_abs_tol * ref, f"{what}: max-abs {ma:.4g} > {max_abs_tol * ref:.4g}"
    assert rr <= rel_rms_tol, f"{what}: relative RMS {rr:.4g} > {rel_rms_tol}"


compare_greedy = O.compare_greedy
