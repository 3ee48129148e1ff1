"""Real-checkpoint ingestion: an mlx-lm style model directory (``config.json`` + ``*.safetensors``) into a DecodeEngine.

What is read, and where the reference defines it:

* ``config.json`` -> :class:`ModelSpec` with the lookup order of ``ModelMeta::from_value`` (src/fusion/ir.rs:626-749): the
  text model's numbers come from ``text_config`` (or a sub-object whose ``model_type`` ends in ``_text``) and fall back to
  the root; ``head_dim`` defaults to hidden / heads; ``quantization.{bits, group_size}`` lives at the root.
* tensor names ``<prefix>layers.<i>.<relpath>`` with the relpaths of ``LayerParamKind::relpath``
  (src/codegen/kernels/mod.rs:4907-4939): ``self_attn.q_proj.{weight,scales,biases,bias}``, ``mlp.down_proj.weight`` ...;
  ``<prefix>embed_tokens.*``, ``<prefix>norm.weight`` and ``lm_head.*`` (absent when the head is tied to the embedding).
* MLX-affine layout (src/fusion/ir.rs:236-247): ``weight`` uint32 ``[N, K*bits/32]`` LSB-first, ``scales`` / ``biases``
  ``[N, K/group]``; a quantised embedding is gathered row-wise with the same rule (embed_lookup_decode.rs:79-93).

The safetensors container is parsed here directly (8-byte little-endian header length, JSON header, raw tensor bytes): bf16
tensors are handed out as their uint16 bit patterns, which NumPy-based loaders cannot express.

Scales and biases must be bf16, the activation type of this runtime.  Checkpoints that store them as fp16 are converted with
round-to-nearest-even and flagged in ``Checkpoint.lossy`` (their dequantised weights are then not bit-identical to MLX's).
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np

from .model_spec import ModelSpec

_DT = {"U32": (np.uint32, 4), "I32": (np.int32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4),
       "U8": (np.uint8, 1), "I64": (np.int64, 8), "U16": (np.uint16, 2)}


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors come back as NumPy views (bf16 as uint16 bits)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n > size - 8 or n > (100 << 20):
            raise ValueError(f"{path}: header length {n} exceeds the file")
        self.header = json.loads(self._f.read(n).decode("utf-8"))
        self.meta = self.header.pop("__metadata__", {})
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        for name, e in self.header.items():
            b, en = e["data_offsets"]
            if e["dtype"] not in _DT:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            want = int(np.prod(e["shape"], dtype=np.int64)) * _DT[e["dtype"]][1]
            if b < 0 or en < b or self._base + en > size or en - b != want:
                raise ValueError(f"{path}: tensor {name} has inconsistent offsets or shape")

    def names(self):
        return list(self.header)

    def dtype(self, name: str) -> str:
        return self.header[name]["dtype"]

    def get(self, name: str) -> np.ndarray:
        e = self.header[name]
        dt, _ = _DT[e["dtype"]]
        b, en = e["data_offsets"]
        return np.frombuffer(self._mm, dtype=dt, count=(en - b) // np.dtype(dt).itemsize, offset=self._base + b).reshape(e["shape"])

    def close(self):
        try:
            self._mm.close()
        except BufferError:          # arrays handed out by get() still view the mapping: it goes when they do
            pass
        self._f.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None):
    """Write ``{name: (array, dtype_tag)}`` as one safetensors file; ``dtype_tag`` names the stored type ("BF16" for uint16
    bit patterns of bf16 values).  Used by the tests and by tools that export models."""
    header, off, blobs = {}, 0, []
    for name, (arr, tag) in tensors.items():
        a = np.ascontiguousarray(arr)
        if tag not in _DT or a.dtype.itemsize != _DT[tag][1]:
            raise ValueError(f"{name}: array of {a.dtype} cannot be stored as {tag}")
        raw = a.tobytes()
        header[name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw); blobs.append(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h))); f.write(h)
        for raw in blobs:
            f.write(raw)


def f16_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float16).astype(np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def spec_from_config(cfg: dict, name: str = "checkpoint") -> ModelSpec:
    """config.json -> ModelSpec (lookup order of ModelMeta::from_value, src/fusion/ir.rs:626-749)."""
    text = cfg.get("text_config")
    if text is None:
        text = next((v for v in cfg.values() if isinstance(v, dict) and str(v.get("model_type", "")).endswith("_text")), cfg)

    def pick(k, default=None):
        v = text.get(k, cfg.get(k, default))
        return default if v is None else v

    def need(k):
        v = pick(k)
        if v is None:
            raise ValueError(f"config missing {k}")
        return v

    hidden, n_q, layers = int(need("hidden_size")), int(need("num_attention_heads")), int(need("num_hidden_layers"))
    n_kv = int(pick("num_key_value_heads", n_q))
    head_dim = int(pick("head_dim", hidden // n_q))
    q = cfg.get("quantization") or {}
    bits = int(q.get("bits", 16)) if q else 16
    group = int(q.get("group_size", 64)) if q else 64
    if bits not in (4, 8, 16):
        raise ValueError(f"{bits}-bit weights are not supported (4, 8 or unquantised)")
    if bits != 16 and group != 64:
        raise ValueError(f"quantisation group size {group} is not supported (64)")
    mt = str(cfg.get("model_type", text.get("model_type", "unknown")))
    if mt.startswith("qwen2"):
        arch = "qwen2"
    elif mt.startswith("gemma3"):
        arch = "gemma3"
    else:
        raise ValueError(f"model_type {mt!r} has no decode path here (qwen2*, gemma3*)")
    window, every = 0, 1
    if arch == "gemma3":
        window = int(pick("sliding_window", 0) or 0)
        every = int(pick("sliding_window_pattern", 6) or 1) if window else 1
    theta = float(pick("rope_theta", 1e6 if arch == "qwen2" else 1e6))
    return ModelSpec(name=name, arch=arch, n_layers=layers, hidden=hidden, n_q=n_q, n_kv=n_kv, head_dim=head_dim,
                     inter=int(need("intermediate_size")), vocab=int(need("vocab_size")), bits=bits,
                     eps=float(pick("rms_norm_eps", 1e-6)), theta=theta, theta_local=float(pick("rope_local_base_freq", 1e4)),
                     window=window, global_every=every)


_W = {"q_proj": "self_attn.q_proj", "k_proj": "self_attn.k_proj", "v_proj": "self_attn.v_proj", "o_proj": "self_attn.o_proj",
      "gate_proj": "mlp.gate_proj", "up_proj": "mlp.up_proj", "down_proj": "mlp.down_proj"}
_V = {"input_norm": "input_layernorm.weight", "post_attention_norm": "post_attention_layernorm.weight",
      "pre_feedforward_norm": "pre_feedforward_layernorm.weight", "post_feedforward_norm": "post_feedforward_layernorm.weight",
      "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight",
      "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias", "v_bias": "self_attn.v_proj.bias"}


class Checkpoint:
    """A model directory: config.json plus one or more safetensors shards."""

    def __init__(self, path: str):
        self.dir = path
        with open(os.path.join(path, "config.json")) as f:
            self.config = json.load(f)
        self.spec = spec_from_config(self.config, os.path.basename(os.path.normpath(path)))
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        idx = os.path.join(path, "model.safetensors.index.json")
        shards = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        if os.path.exists(idx):
            with open(idx) as f:
                shards = sorted(set(json.load(f)["weight_map"].values()))
        if not shards:
            raise FileNotFoundError(f"{path}: no .safetensors files")
        for s in shards:
            sf = SafetensorsFile(os.path.join(path, s))
            self.files.append(sf)
            for n in sf.names():
                self.where[n] = sf
        emb = [n for n in self.where if n.endswith("embed_tokens.weight")]
        if len(emb) != 1:
            raise ValueError(f"{path}: expected one embed_tokens.weight, found {emb}")
        self.prefix = emb[0][: -len("embed_tokens.weight")]          # "model." or "language_model.model."
        self.head_prefix = self.prefix[: -len("model.")] if self.prefix.endswith("model.") else ""
        self.tied = (self.head_prefix + "lm_head.weight") not in self.where
        self.lossy: list[str] = []                                  # tensors converted from fp16 / fp32 to bf16
        self.embed_bits = self.spec.bits if (self.prefix + "embed_tokens.scales") in self.where else 16
        # Gemma-family RMSNorm multiplies by (1 + weight); the runtime takes the effective weight
        self.norm_offset = 1.0 if self.spec.arch == "gemma3" else 0.0

    def has(self, name: str) -> bool:
        return name in self.where

    def raw(self, name: str) -> np.ndarray:
        if name not in self.where:
            raise KeyError(f"{self.dir}: tensor {name} not found")
        return self.where[name].get(name)

    def bf16(self, name: str) -> np.ndarray:
        """A floating tensor as bf16 bit patterns."""
        sf = self.where.get(name)
        if sf is None:
            raise KeyError(f"{self.dir}: tensor {name} not found")
        dt, a = sf.dtype(name), sf.get(name)
        if dt == "BF16":
            return a
        if dt in ("F16", "F32"):
            if name not in self.lossy:
                self.lossy.append(name)
            return f16_to_bf16_bits(a) if dt == "F16" else f32_to_bf16_bits(a)
        raise ValueError(f"{name}: dtype {dt} is not a floating type")

    def _linear_base(self, leaf: str, layer: int) -> str:
        if leaf == "lm_head":
            return (self.prefix + "embed_tokens") if self.tied else (self.head_prefix + "lm_head")
        return f"{self.prefix}layers.{layer}.{_W[leaf]}"

    def weight_provider(self):
        """For DecodeEngine.load_from: rows [src_row0, src_row0 + nrows) and input columns [k0, k0 + k) of a projection."""
        def prov(leaf, layer, src_row0, nrows, k_global, k0, k, bits):
            base = self._linear_base(leaf, layer)
            w = self.raw(base + ".weight")
            if bits == 16:
                if self.where[base + ".weight"].dtype(base + ".weight") != "BF16":
                    w = self.bf16(base + ".weight")
                if w.shape[1] != k_global:
                    raise ValueError(f"{base}.weight: {w.shape[1]} input columns, config says {k_global}")
                return np.ascontiguousarray(w[src_row0:src_row0 + nrows, k0:k0 + k]), None, None
            per = 32 // bits
            if w.dtype != np.uint32 or w.shape[1] * per != k_global:
                raise ValueError(f"{base}.weight: expected uint32 [N, {k_global * bits // 32}], found {w.dtype} {w.shape}")
            s, b = self.bf16(base + ".scales"), self.bf16(base + ".biases")
            if s.shape != (w.shape[0], k_global // 64) or b.shape != s.shape:
                raise ValueError(f"{base}: scales/biases must be [N, K/64]")
            rows = slice(src_row0, src_row0 + nrows)
            return (np.ascontiguousarray(w[rows, k0 // per:(k0 + k) // per]), np.ascontiguousarray(s[rows, k0 // 64:(k0 + k) // 64]),
                    np.ascontiguousarray(b[rows, k0 // 64:(k0 + k) // 64]))
        return prov

    def vector_provider(self):
        def prov(leaf, layer, idx0, n, mean, std):
            if leaf == "embed_tokens":
                if self.embed_bits != 16:
                    raise ValueError("the embedding is quantised: use embed_provider")
                a = self.bf16(self.prefix + "embed_tokens.weight").reshape(-1)
            elif leaf == "final_norm":
                a = self._norm(self.prefix + "norm.weight")
            elif leaf.endswith("_norm"):
                a = self._norm(f"{self.prefix}layers.{layer}.{_V[leaf]}")
            else:
                a = self.bf16(f"{self.prefix}layers.{layer}.{_V[leaf]}").reshape(-1)
            return np.ascontiguousarray(a[idx0:idx0 + n])
        return prov

    def _norm(self, name: str) -> np.ndarray:
        a = self.bf16(name).reshape(-1)
        if self.norm_offset == 0.0:
            return a
        f = (a.astype(np.uint32) << 16).view(np.float32) + np.float32(self.norm_offset)
        return f32_to_bf16_bits(f)

    def embed_provider(self):
        """Quantised embedding rows (None for a bf16 table)."""
        if self.embed_bits == 16:
            return None
        base = self.prefix + "embed_tokens"
        return {"bits": self.embed_bits, "packed": self.raw(base + ".weight"), "scales": self.bf16(base + ".scales"),
                "biases": self.bf16(base + ".biases")}

    def close(self):
        for f in self.files:
            f.close()


def load_engine(path: str, capacity: int, device: int = 0, tp_rank: int = 0, tp_size: int = 1, **kw):
    """Open a checkpoint directory and return (engine, checkpoint) with all tensors resident on the GPU."""
    from .runtime import DecodeEngine
    ck = Checkpoint(path)
    eng = DecodeEngine(ck.spec, capacity, device=device, tp_rank=tp_rank, tp_size=tp_size, **kw)
    eng.load_from(ck.weight_provider(), ck.vector_provider(), ck.embed_provider())
    return eng, ck
