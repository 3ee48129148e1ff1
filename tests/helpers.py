"""Shared helpers of the parity tests: oracle <-> engine glue and the tolerance metrics."""
from __future__ import annotations

import json
import os

import numpy as np

from fusekit_b200.model_spec import ModelSpec, stream_id, tensor_name
from oracle import oracle as O
from fusekit_b200 import checkpoint as CK

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


def export_oracle_model(model, spec, path: str):
    """Write the tensors of a CPU oracle model as an mlx-lm style checkpoint directory (config.json + model.safetensors):
    the fixture generator of the ingestion tests, and a way to hand a synthetic model to other tools."""
    os.makedirs(path, exist_ok=True)
    H, hd = spec.hidden, spec.head_dim
    t: dict = {}
    pre = "model."

    def put_linear(base, w):
        if w.bits == 16:
            t[base + ".weight"] = (w.dense, "BF16")
        else:
            t[base + ".weight"] = (w.packed, "U32"); t[base + ".scales"] = (w.scales, "BF16"); t[base + ".biases"] = (w.biases, "BF16")

    def norm(v):
        if spec.arch != "gemma3":
            return v
        f = (np.asarray(v, np.uint16).astype(np.uint32) << 16).view(np.float32) - np.float32(1.0)     # stored weight = effective - 1
        return CK.f32_to_bf16_bits(f)

    t[pre + "embed_tokens.weight"] = (model.vec(-1, 0, spec.vocab * H).reshape(spec.vocab, H), "BF16")
    t[pre + "norm.weight"] = (norm(model.vec(-1, 1, H)), "BF16")
    put_linear("lm_head", model.linear(-1, 0))
    names = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    for l in range(spec.n_layers):
        for i, leaf in enumerate(names):
            w = model.linear(l, i)
            put_linear(f"{pre}layers.{l}.{CK._W[leaf]}", w)
            if spec.qkv_bias and i < 3:
                t[f"{pre}layers.{l}.{CK._W[leaf]}.bias"] = (w.lin_bias, "BF16")
        t[f"{pre}layers.{l}.input_layernorm.weight"] = (norm(model.vec(l, 0, H)), "BF16")
        if spec.arch == "qwen2":
            t[f"{pre}layers.{l}.post_attention_layernorm.weight"] = (norm(model.vec(l, 1, H)), "BF16")
        else:
            for which, leaf, n in ((2, "post_attention_norm", H), (3, "pre_feedforward_norm", H), (4, "post_feedforward_norm", H),
                                   (5, "q_norm", hd), (6, "k_norm", hd)):
                t[f"{pre}layers.{l}.{CK._V[leaf]}"] = (norm(model.vec(l, which, n)), "BF16")
    cfg = {"model_type": "qwen2" if spec.arch == "qwen2" else "gemma3_text", "hidden_size": H, "num_hidden_layers": spec.n_layers,
           "num_attention_heads": spec.n_q, "num_key_value_heads": spec.n_kv, "head_dim": hd, "intermediate_size": spec.inter,
           "vocab_size": spec.vocab, "rms_norm_eps": spec.eps, "rope_theta": spec.theta, "tie_word_embeddings": False,
           "torch_dtype": "bfloat16"}
    if spec.arch == "gemma3":
        cfg.update({"sliding_window": spec.window, "sliding_window_pattern": spec.global_every, "rope_local_base_freq": spec.theta_local})
    if spec.bits != 16:
        cfg["quantization"] = {"group_size": 64, "bits": spec.bits}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    CK.write_safetensors(os.path.join(path, "model.safetensors"), t, {"format": "mlx"})
