"""Real-checkpoint ingestion: config.json / safetensors reader on the CPU, and on the GPU an engine loaded from a
checkpoint directory whose tensors are the CPU oracle's (dequantised weights bit-exact, greedy tokens equal)."""
import json
import os

import numpy as np
import pytest

from fusekit_b200 import checkpoint as CK
from fusekit_b200.model_spec import CONFIGS
from oracle import oracle as O
from tests.helpers import compare_greedy, export_oracle_model, oracle_config


def test_reader_agrees_with_the_safetensors_library(tmp_path):
    """A file written by the safetensors package (bf16 through torch) reads back identically through SafetensorsFile, and a
    file written by write_safetensors loads in the safetensors package."""
    import torch
    from safetensors.torch import load_file, save_file
    g = torch.Generator().manual_seed(5)
    t = {"a.weight": torch.randint(0, 2 ** 31 - 1, (6, 8), generator=g, dtype=torch.int32),
         "a.scales": torch.randn(6, 2, generator=g).to(torch.bfloat16), "b": torch.randn(3, 5, generator=g).to(torch.float16),
         "c": torch.randn(7, generator=g)}
    p = str(tmp_path / "lib.safetensors")
    save_file(t, p, metadata={"format": "mlx"})
    f = CK.SafetensorsFile(p)
    assert sorted(f.names()) == sorted(t) and f.meta == {"format": "mlx"}
    assert np.array_equal(f.get("a.weight"), t["a.weight"].numpy())
    assert f.dtype("a.scales") == "BF16" and np.array_equal(f.get("a.scales"), t["a.scales"].view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(f.get("b"), t["b"].numpy()) and np.array_equal(f.get("c"), t["c"].numpy())
    f.close()
    p2 = str(tmp_path / "mine.safetensors")
    CK.write_safetensors(p2, {"w": (np.arange(12, dtype=np.uint32).reshape(3, 4), "U32"),
                              "s": (t["a.scales"].view(torch.int16).numpy().view(np.uint16), "BF16")}, {"format": "mlx"})
    back = load_file(p2)
    assert torch.equal(back["s"], t["a.scales"]) and back["w"].shape == (3, 4)


def test_reader_refuses_damaged_files(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    CK.write_safetensors(p, {"w": (np.zeros((4, 4), np.uint32), "U32")})
    raw = bytearray(open(p, "rb").read())
    open(p, "wb").write(raw[:-8])                                   # truncated payload
    with pytest.raises(ValueError, match="inconsistent offsets"):
        CK.SafetensorsFile(p)
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(ValueError, match="not a safetensors file"):
        CK.SafetensorsFile(p)


def test_spec_from_config_lookup_order():
    """Flat configs, text_config sub-objects and `*_text` sub-objects (src/fusion/ir.rs:626-700)."""
    flat = {"model_type": "qwen2", "hidden_size": 896, "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2,
            "intermediate_size": 4864, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "quantization": {"group_size": 64, "bits": 4}}
    s = CK.spec_from_config(flat)
    ref = CONFIGS["qwen2.5-0.5b"]
    assert (s.arch, s.n_layers, s.hidden, s.n_q, s.n_kv, s.head_dim, s.inter, s.vocab, s.bits) == \
           (ref.arch, ref.n_layers, ref.hidden, ref.n_q, ref.n_kv, ref.head_dim, ref.inter, ref.vocab, 4)
    nested = {"model_type": "gemma3", "quantization": {"group_size": 64, "bits": 8},
              "text_config": {"model_type": "gemma3_text", "hidden_size": 2560, "num_hidden_layers": 34, "num_attention_heads": 8,
                              "num_key_value_heads": 4, "head_dim": 256, "intermediate_size": 10240, "vocab_size": 262144,
                              "sliding_window": 1024, "sliding_window_pattern": 6, "rope_local_base_freq": 10000.0}}
    g = CK.spec_from_config(nested)
    ref = CONFIGS["gemma3-4b"]
    assert (g.arch, g.head_dim, g.window, g.global_every, g.bits, g.vocab) == ("gemma3", 256, 1024, 6, 8, ref.vocab)
    sub = {"model_type": "gemma3", "language": {"model_type": "gemma3_text", **nested["text_config"]}}
    assert CK.spec_from_config(sub).hidden == 2560 and CK.spec_from_config(sub).bits == 16
    with pytest.raises(ValueError, match="missing hidden_size"):
        CK.spec_from_config({"model_type": "qwen2"})
    with pytest.raises(ValueError, match="group size"):
        CK.spec_from_config({**flat, "quantization": {"group_size": 32, "bits": 4}})
    with pytest.raises(ValueError, match="no decode path"):
        CK.spec_from_config({**flat, "model_type": "mamba"})


def _export(tmp_path, name, bits):
    spec = CONFIGS[name].with_bits(bits)
    m = O.Model(oracle_config(spec, 64))
    d = str(tmp_path / f"{name}-q{bits}")
    export_oracle_model(m, spec, d)
    return spec, m, d


@pytest.mark.parametrize("name,bits", [("tiny-qwen", 4), ("tiny-gemma", 8)])
def test_checkpoint_directory_round_trip_on_the_cpu(tmp_path, name, bits):
    """Exported oracle tensors come back through Checkpoint's providers exactly, including tensor-parallel slices, fp16
    scales are converted and flagged, a tied head falls back to the embedding."""
    spec, m, d = _export(tmp_path, name, bits)
    ck = CK.Checkpoint(d)
    s = ck.spec
    assert (s.arch, s.n_layers, s.hidden, s.n_q, s.n_kv, s.head_dim, s.inter, s.vocab, s.bits, s.window, s.global_every) == \
           (spec.arch, spec.n_layers, spec.hidden, spec.n_q, spec.n_kv, spec.head_dim, spec.inter, spec.vocab, bits, spec.window, spec.global_every)
    assert not ck.tied and ck.embed_bits == 16 and ck.prefix == "model."
    wp, vp = ck.weight_provider(), ck.vector_provider()
    H, I = spec.hidden, spec.inter
    w = m.linear(1, 6)                                               # down_proj of layer 1
    p, sc, bi = wp("down_proj", 1, 0, H, I, 0, I, bits)
    assert np.array_equal(p, w.packed) and np.array_equal(sc, w.scales) and np.array_equal(bi, w.biases)
    p, sc, bi = wp("down_proj", 1, 0, H, I, I // 2, I // 2, bits)    # second half of the input columns (row-split shard)
    assert np.array_equal(p, w.packed[:, w.packed.shape[1] // 2:]) and np.array_equal(sc, w.scales[:, w.scales.shape[1] // 2:])
    wq = m.linear(0, 0)
    p, sc, bi = wp("q_proj", 0, spec.head_dim, spec.head_dim, H, 0, H, bits)     # one head's rows
    assert np.array_equal(p, wq.packed[spec.head_dim:2 * spec.head_dim])
    assert np.array_equal(vp("input_norm", 0, 0, H, 1.0, 0.02), m.vec(0, 0, H))   # Gemma: stored as weight - 1, read back as 1 + w
    assert np.array_equal(vp("final_norm", -1, 0, H, 1.0, 0.02), m.vec(-1, 1, H))
    assert np.array_equal(vp("embed_tokens", -1, H, 2 * H, 0.0, 0.02), m.vec(-1, 0, 3 * H)[H:])
    if spec.qkv_bias:
        assert np.array_equal(vp("k_bias", 1, 0, spec.n_kv * spec.head_dim, 0.0, 0.02), m.linear(1, 1).lin_bias)
    else:
        assert np.array_equal(vp("q_norm", 2, 0, spec.head_dim, 1.0, 0.02), m.vec(2, 5, spec.head_dim))
    assert not ck.lossy
    ck.close()


def test_fp16_scales_are_converted_and_flagged_and_tied_heads_resolve(tmp_path):
    spec, m, d = _export(tmp_path, "tiny-qwen", 4)
    f = CK.SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {}
    for n in f.names():
        a, tag = f.get(n).copy(), f.dtype(n)
        if n.startswith("lm_head"):
            continue                                                  # tie the head: no lm_head tensors
        if n.endswith(".scales"):
            a, tag = (a.astype(np.uint32) << 16).view(np.float32).astype(np.float16), "F16"
        t[n] = (a, tag)
    # a tied head needs a quantised embedding: replace the bf16 table by the head's packed rows
    head = m.linear(-1, 0)
    t["model.embed_tokens.weight"] = (head.packed, "U32")
    t["model.embed_tokens.scales"] = ((head.scales.astype(np.uint32) << 16).view(np.float32).astype(np.float16), "F16")
    t["model.embed_tokens.biases"] = (head.biases, "BF16")
    f.close()
    CK.write_safetensors(os.path.join(d, "model.safetensors"), t)
    ck = CK.Checkpoint(d)
    assert ck.tied and ck.embed_bits == 4
    p, sc, bi = ck.weight_provider()("lm_head", -1, 0, spec.vocab, spec.hidden, 0, spec.hidden, 4)
    assert np.array_equal(p, head.packed) and np.array_equal(bi, head.biases)
    assert "model.embed_tokens.scales" in ck.lossy
    e = ck.embed_provider()
    assert e["bits"] == 4 and np.array_equal(e["packed"], head.packed)
    # bf16 -> fp16 -> bf16 keeps a bf16 value whenever fp16 can hold it (these scales are small normal numbers)
    assert np.array_equal(e["scales"], head.scales)
    ck.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name,bits", [("tiny-qwen", 4), ("tiny-qwen", 8), ("tiny-gemma", 4), ("tiny-qwen", 16)])
def test_engine_loaded_from_a_checkpoint_matches_the_oracle(tmp_path, name, bits):
    spec, m, d = _export(tmp_path, name, bits)
    eng, ck = CK.load_engine(d, 64)
    try:
        for wname, (layer, which, rows) in {"layers.0.o": (0, 3, 16), "layers.1.down": (1, 6, 16), "lm_head": (-1, 0, 32)}.items():
            ref = m.linear(layer, which)
            got = eng.rt.weight_dequant(eng.W[wname], 0, rows, ref.k)
            if ref.bits == 16:
                want = O.bf16_to_f32(np.ascontiguousarray(ref.dense[:rows]))
            else:
                want = O.dequant(O.QWeight(rows, ref.k, ref.bits, np.ascontiguousarray(ref.packed[:rows]),
                                           np.ascontiguousarray(ref.scales[:rows]), np.ascontiguousarray(ref.biases[:rows])))
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), wname
        ctx = 0
        got, _ = eng.decode_chunk(ctx, 5, 8)
        mism, ties = compare_greedy(got, m, 5, ctx, tie_ulps=4.0)
        assert not mism and len(ties) <= 1, (mism, ties)
    finally:
        eng.close(); ck.close()


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
def test_quantised_embedding_gather_is_exact(runtime, bits):
    """x = T((q * s + b) * scale) for a quantised embedding row (embed_lookup_decode.rs:79-93), against NumPy."""
    from fusekit_b200 import _native as N
    from fusekit_b200.model_spec import stream_id
    rt, V, H, scale = runtime, 300, 256, 16.0
    w = O.gen_weight(stream_id(9, f"emb{bits}"), V, H, bits)
    out = rt.alloc(H * 2)
    task = N.Task.make(N.TASK_EMBED_LOOKUP_DECODE, -1, {0: rt.to_device(w.packed), 1: out, 2: rt.to_device(w.scales), 3: rt.to_device(w.biases)},
                       [H, 1, V, bits], [scale])
    deq = O.dequant(w)
    for tok in (0, 17, V - 1):
        rt.state_set(tok, 0)
        rt.launch(task)
        want = O.f32_to_bf16((deq[tok] * np.float32(scale)).astype(np.float32))
        assert np.array_equal(rt.download(out, (H,), np.uint16), want), tok
