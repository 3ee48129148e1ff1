"""Decoder shapes of the benchmark configs and the naming of their seeded tensors.

The reference learns these from ``config.json`` (``ModelMeta::from_config_file``,
src/fusion/ir.rs:604-749) and from the traced graph; capture needs MLX, so the five
benchmark shapes are stated here directly.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class ModelSpec:
    name: str
    arch: str                 # "qwen2" | "gemma3"
    n_layers: int
    hidden: int
    n_q: int
    n_kv: int
    head_dim: int
    inter: int
    vocab: int
    bits: int = 4             # 4 / 8 affine group-64, 16 = plain bf16
    eps: float = 1e-6
    theta: float = 1e6        # RoPE base of global-attention layers
    theta_local: float = 1e4  # RoPE base of sliding-window layers
    window: int = 0           # sliding window (0: every layer global)
    global_every: int = 1     # with a window: every Nth layer is global
    seed: int = 20240531

    @property
    def qkv_bias(self) -> bool:
        return self.arch == "qwen2"

    @property
    def act(self) -> int:
        return 1 if self.arch == "gemma3" else 0

    def is_sliding(self, layer: int) -> bool:
        return self.window > 0 and ((layer + 1) % self.global_every != 0)

    def layer_capacity(self, layer: int, capacity: int) -> int:
        return self.window if self.is_sliding(layer) else capacity

    def layer_theta(self, layer: int) -> float:
        return self.theta_local if self.is_sliding(layer) else self.theta

    def with_bits(self, bits: int) -> "ModelSpec":
        return replace(self, bits=bits)

    # ---- algorithmic bytes (what a decode step must read from HBM) ----
    def linear_bytes(self, k: int, n: int, residual: bool = False) -> int:
        """bytes(qmatvec K->N) = N*K*bits/8 + 2*N*(K/64)*2 + 2K + 2N (+2N with a residual)."""
        w = n * k * self.bits // 8 + (0 if self.bits == 16 else 2 * n * (k // 64) * 2)
        return w + 2 * k + 2 * n + (2 * n if residual else 0)

    def weight_bytes_per_token(self) -> int:
        h, i, qkv = self.hidden, self.inter, (self.n_q + 2 * self.n_kv) * self.head_dim
        per_layer = (self.linear_bytes(h, qkv) + self.linear_bytes(self.n_q * self.head_dim, h, True)
                     + 2 * self.linear_bytes(h, i) + self.linear_bytes(i, h, True))
        return self.n_layers * per_layer + self.linear_bytes(h, self.vocab)

    def kv_bytes_per_token(self, ctx: int) -> int:
        tot = 0
        for l in range(self.n_layers):
            n = min(ctx, self.window) if self.is_sliding(l) else ctx
            tot += 2 * self.n_kv * self.head_dim * 2 * n
        return tot

    def bytes_per_token(self, ctx: int) -> int:
        return self.weight_bytes_per_token() + self.kv_bytes_per_token(ctx)


CONFIGS = {
    # Qwen2.5-0.5B-shaped (CPU-reference-sized parity config)
    "qwen2.5-0.5b": ModelSpec("qwen2.5-0.5b", "qwen2", 24, 896, 14, 2, 64, 4864, 151936),
    # Qwen2.5-7B-shaped (headline metric)
    "qwen2.5-7b": ModelSpec("qwen2.5-7b", "qwen2", 28, 3584, 28, 4, 128, 18944, 152064),
    # Gemma-3-4B-shaped: GeGLU-tanh, sliding window 1024 on 5 of every 6 layers
    "gemma3-4b": ModelSpec("gemma3-4b", "gemma3", 34, 2560, 8, 4, 256, 10240, 262144, window=1024, global_every=6),
    # Qwen2.5-32B-shaped (tensor-parallel config)
    "qwen2.5-32b": ModelSpec("qwen2.5-32b", "qwen2", 64, 5120, 40, 8, 128, 27648, 152064),
    # tiny shapes for fast parity tests (not benchmark configs)
    "tiny-qwen": ModelSpec("tiny-qwen", "qwen2", 2, 256, 4, 2, 64, 512, 1024),
    "tiny-gemma": ModelSpec("tiny-gemma", "gemma3", 3, 256, 4, 2, 64, 512, 1024, window=16, global_every=3),
}


# ---- tensor naming / stream ids (FNV-1a 64 of the name, xor a mix of the seed) ----
def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def stream_id(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & MASK64
    return h ^ _mix64(seed)


def tensor_name(layer: int, leaf: str) -> str:
    return leaf if layer < 0 else f"layers.{layer}.{leaf}"
