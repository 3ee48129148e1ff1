"""ctypes binding of the CPU oracle (``fk_oracle.c``) plus a NumPy restatement
of the small ops used to cross-check it.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; the
shipped package never imports it.  PARITY UNPINNED: the reference repository
holds no golden vectors or known-answer tests for the decode path and its
Metal/MLX code cannot run on Linux, so the oracle follows the reference's
emitter sources (cited per function in ``fk_oracle.c``) and is pinned only by
the self-generated fixtures under ``tests/golden``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libfk_oracle.so")


def build(force: bool = False) -> str:
    """Compile ``fk_oracle.c`` with the committed Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "fk_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


class Linear(C.Structure):
    _fields_ = [("n", C.c_int64), ("k", C.c_int64), ("bits", C.c_int),
                ("packed", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
                ("dense", C.c_void_p), ("lin_bias", C.c_void_p)]


class Config(C.Structure):
    _fields_ = [("arch", C.c_int), ("n_layers", C.c_int), ("hidden", C.c_int), ("n_q", C.c_int),
                ("n_kv", C.c_int), ("head_dim", C.c_int), ("inter", C.c_int), ("vocab", C.c_int),
                ("bits", C.c_int), ("eps", C.c_float), ("theta", C.c_float), ("theta_local", C.c_float),
                ("window", C.c_int), ("global_every", C.c_int), ("capacity", C.c_int),
                ("seed", C.c_uint64), ("tp_rank", C.c_int), ("tp_size", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_LIB_PATH)
    u64, i64, f32, vp, i32, u32 = C.c_uint64, C.c_int64, C.c_float, C.c_void_p, C.c_int, C.c_uint32
    L.fko_stream_id.restype = u64; L.fko_stream_id.argtypes = [C.c_char_p]
    L.fko_tensor_stream.restype = u64; L.fko_tensor_stream.argtypes = [u64, C.c_char_p, i32]
    L.fko_unit_normal.restype = f32; L.fko_unit_normal.argtypes = [u64, u64]
    L.fko_uniform_u32.restype = u32; L.fko_uniform_u32.argtypes = [u64, u64, u32]
    L.fko_fill_normal_bf16.restype = None; L.fko_fill_normal_bf16.argtypes = [u64, u64, u64, f32, f32, vp]
    L.fko_gen_qweight.restype = None
    L.fko_gen_qweight.argtypes = [u64, f32, i64, i64, i64, i64, i64, i32, vp, vp, vp]
    L.fko_gen_dense_weight.restype = None
    L.fko_gen_dense_weight.argtypes = [u64, f32, i64, i64, i64, i64, i64, vp]
    L.fko_dequant.restype = None; L.fko_dequant.argtypes = [vp, vp, vp, i64, i64, i32, vp]
    L.fko_qmatvec.restype = None; L.fko_qmatvec.argtypes = [C.POINTER(Linear), vp, vp, vp]
    L.fko_linear_apply.restype = None; L.fko_linear_apply.argtypes = [C.POINTER(Linear), vp, vp, vp, vp]
    L.fko_rmsnorm.restype = None; L.fko_rmsnorm.argtypes = [vp, vp, i64, f32, vp]
    L.fko_rope.restype = None; L.fko_rope.argtypes = [vp, i32, i32, u32, f32]
    L.fko_sdpa_decode.restype = None
    L.fko_sdpa_decode.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, f32, vp]
    L.fko_act.restype = None; L.fko_act.argtypes = [vp, vp, i64, i32, vp]
    L.fko_argmax_bf16.restype = u32; L.fko_argmax_bf16.argtypes = [vp, i64]
    L.fko_model_create.restype = vp; L.fko_model_create.argtypes = [C.POINTER(Config)]
    L.fko_model_free.restype = None; L.fko_model_free.argtypes = [vp]
    L.fko_model_prefill_kv.restype = None; L.fko_model_prefill_kv.argtypes = [vp, i64]
    L.fko_model_linear.restype = C.POINTER(Linear); L.fko_model_linear.argtypes = [vp, i32, i32]
    L.fko_model_vec.restype = vp; L.fko_model_vec.argtypes = [vp, i32, i32]
    L.fko_model_layer_cap.restype = i64; L.fko_model_layer_cap.argtypes = [vp, i32]
    L.fko_model_layer_sliding.restype = i32; L.fko_model_layer_sliding.argtypes = [vp, i32]
    L.fko_model_layer_theta.restype = f32; L.fko_model_layer_theta.argtypes = [vp, i32]
    L.fko_model_embed_scale.restype = f32; L.fko_model_embed_scale.argtypes = [vp]
    L.fko_decode_step.restype = u32; L.fko_decode_step.argtypes = [vp, u32, u32, vp, vp]
    L.fko_layer_step.restype = None; L.fko_layer_step.argtypes = [vp, i32, vp, u32]
    L.fko_head_step.restype = u32; L.fko_head_step.argtypes = [vp, vp, vp]
    L.fko_decode_greedy.restype = C.c_double; L.fko_decode_greedy.argtypes = [vp, u32, u32, i32, vp]
    L.fko_num_threads.restype = i32
    L.fko_kv_quantize_row.restype = None; L.fko_kv_quantize_row.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    L.fko_rope_f32.restype = None; L.fko_rope_f32.argtypes = [vp, i32, i32, u32, f32, vp]
    L.fko_sdpa_decode_quant.restype = None; L.fko_sdpa_decode_quant.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, f32, i32, i32, vp]
    L.fko_model_set_kv_quant.restype = None; L.fko_model_set_kv_quant.argtypes = [vp, i32, i32]
    L.fko_set_num_threads.restype = None; L.fko_set_num_threads.argtypes = [i32]
    L.fko_f32_to_bf16.restype = C.c_uint16; L.fko_f32_to_bf16.argtypes = [f32]
    L.fko_bf16_to_f32.restype = f32; L.fko_bf16_to_f32.argtypes = [C.c_uint16]
    _lib = L
    return L


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


# ----------------------------------------------------------------- bf16 helpers
def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def stream_id(name: str) -> int:
    return int(lib().fko_stream_id(name.encode()))


def tensor_stream(seed: int, fmt: str, layer: int = 0) -> int:
    return int(lib().fko_tensor_stream(seed, fmt.encode(), layer))


def fill_normal_bf16(stream: int, idx0: int, n: int, mean: float, std: float) -> np.ndarray:
    out = np.empty(n, np.uint16)
    lib().fko_fill_normal_bf16(stream, idx0, n, mean, std, _p(out))
    return out


def uniform_u32(stream: int, idx: int, modulo: int) -> int:
    return int(lib().fko_uniform_u32(stream, idx, modulo))


@dataclass
class QWeight:
    n: int
    k: int
    bits: int
    packed: np.ndarray | None      # uint32 [n, k*bits/32]
    scales: np.ndarray | None      # bf16 bits [n, k/64]
    biases: np.ndarray | None
    dense: np.ndarray | None = None      # bf16 bits [n, k] when bits == 16
    lin_bias: np.ndarray | None = None   # bf16 bits [n]

    def as_struct(self) -> Linear:
        return Linear(self.n, self.k, self.bits, _p(self.packed), _p(self.scales), _p(self.biases),
                      _p(self.dense), _p(self.lin_bias))

    @property
    def nbytes(self) -> int:
        if self.bits == 16:
            return self.dense.nbytes
        return self.packed.nbytes + self.scales.nbytes + self.biases.nbytes


def gen_weight(stream: int, n: int, k: int, bits: int, k_global: int | None = None, row0: int = 0,
               k0: int = 0, std: float = 0.02) -> QWeight:
    kg = k if k_global is None else k_global
    if bits == 16:
        d = np.empty((n, k), np.uint16)
        lib().fko_gen_dense_weight(stream, std, kg, row0, n, k0, k, _p(d))
        return QWeight(n, k, 16, None, None, None, dense=d)
    packed = np.empty((n, k * bits // 32), np.uint32)
    sc = np.empty((n, k // 64), np.uint16)
    bi = np.empty((n, k // 64), np.uint16)
    lib().fko_gen_qweight(stream, std, kg, row0, n, k0, k, bits, _p(packed), _p(sc), _p(bi))
    return QWeight(n, k, bits, packed, sc, bi)


def dequant(w: QWeight) -> np.ndarray:
    out = np.empty((w.n, w.k), np.float32)
    lib().fko_dequant(_p(w.packed), _p(w.scales), _p(w.biases), w.n, w.k, w.bits, _p(out))
    return out


def qmatvec(w: QWeight, x_bf16: np.ndarray, residual: np.ndarray | None = None) -> np.ndarray:
    y = np.empty(w.n, np.uint16)
    s = w.as_struct()
    lib().fko_qmatvec(C.byref(s), _p(x_bf16), _p(residual), _p(y))
    return y


def linear_acc(w: QWeight, x_f32: np.ndarray) -> np.ndarray:
    acc = np.empty(w.n, np.float32)
    s = w.as_struct()
    lib().fko_linear_apply(C.byref(s), _p(np.ascontiguousarray(x_f32, np.float32)), None, None, _p(acc))
    return acc


def rmsnorm(x_bf16: np.ndarray, w_bf16: np.ndarray, eps: float) -> np.ndarray:
    y = np.empty(x_bf16.size, np.float32)
    lib().fko_rmsnorm(_p(x_bf16), _p(w_bf16), x_bf16.size, eps, _p(y))
    return y


def rope(v_bf16: np.ndarray, n_heads: int, hd: int, pos: int, theta: float) -> np.ndarray:
    v = v_bf16.copy()
    lib().fko_rope(_p(v), n_heads, hd, pos, theta)
    return v


def sdpa_decode(q, ck, cv, n_q, n_kv, hd, capacity, kv_len, scale) -> np.ndarray:
    out = np.empty(n_q * hd, np.uint16)
    lib().fko_sdpa_decode(_p(q), _p(ck), _p(cv), n_q, n_kv, hd, capacity, kv_len, scale, _p(out))
    return out


def act(gate_acc: np.ndarray, up_acc: np.ndarray, kind: int) -> np.ndarray:
    y = np.empty(gate_acc.size, np.uint16)
    lib().fko_act(_p(np.ascontiguousarray(gate_acc, np.float32)), _p(np.ascontiguousarray(up_acc, np.float32)),
                  gate_acc.size, kind, _p(y))
    return y


def kv_quantize_row(x_f32: np.ndarray, bits: int, group: int = 64):
    """One cache row quantised with the reference's edge-anchored rule: (packed u32, scales bf16, biases bf16)."""
    x = np.ascontiguousarray(x_f32, np.float32)
    packed = np.zeros(x.size * bits // 32, np.uint32); sc = np.zeros(x.size // group, np.uint16); bi = np.zeros(x.size // group, np.uint16)
    lib().fko_kv_quantize_row(_p(x), x.size, group, bits, _p(packed), _p(sc), _p(bi))
    return packed, sc, bi


def rope_f32(v_bf16: np.ndarray, n_heads: int, hd: int, pos: int, theta: float) -> np.ndarray:
    out = np.empty(n_heads * hd, np.float32)
    lib().fko_rope_f32(_p(np.ascontiguousarray(v_bf16, np.uint16)), n_heads, hd, pos, theta, _p(out))
    return out


def sdpa_decode_quant(q, kp, ks, kb, vp, vs, vb, n_q, n_kv, hd, capacity, kv_len, scale, bits, group=64) -> np.ndarray:
    out = np.empty(n_q * hd, np.uint16)
    lib().fko_sdpa_decode_quant(_p(q), _p(kp), _p(ks), _p(kb), _p(vp), _p(vs), _p(vb), n_q, n_kv, hd, capacity, kv_len, scale, group, bits, _p(out))
    return out


def argmax_bf16(logits: np.ndarray) -> int:
    return int(lib().fko_argmax_bf16(_p(logits), logits.size))


def num_threads() -> int:
    return int(lib().fko_num_threads())


def set_num_threads(n: int) -> int:
    """Pin the OpenMP thread count of the oracle (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().fko_set_num_threads(int(n))
    return num_threads()


def model_config(spec, capacity: int, tp_rank: int = 0, tp_size: int = 1) -> "Config":
    """Oracle configuration of a model shape (any object with the fields of fusekit_b200.model_spec.ModelSpec)."""
    return Config(arch=1 if spec.arch == "gemma3" else 0, n_layers=spec.n_layers, hidden=spec.hidden, n_q=spec.n_q,
                  n_kv=spec.n_kv, head_dim=spec.head_dim, inter=spec.inter, vocab=spec.vocab, bits=spec.bits,
                  eps=spec.eps, theta=spec.theta, theta_local=spec.theta_local, window=spec.window,
                  global_every=spec.global_every, capacity=capacity, seed=spec.seed, tp_rank=tp_rank, tp_size=tp_size)


class Model:
    """Whole-model oracle: seeded weights + a greedy decode loop on the CPU."""

    def __init__(self, cfg: Config):
        self.cfg = cfg
        self._h = lib().fko_model_create(C.byref(cfg))
        if not self._h:
            raise RuntimeError("fko_model_create failed")

    def close(self):
        if self._h:
            lib().fko_model_free(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def set_kv_quant(self, bits: int, group: int = 64):
        """Switch to a quantised KV cache (empty): store and attention follow the reference's quantised kernels."""
        lib().fko_model_set_kv_quant(self._h, bits, group)

    def prefill_kv(self, ctx: int):
        lib().fko_model_prefill_kv(self._h, ctx)

    def linear(self, layer: int, which: int) -> QWeight:
        s = lib().fko_model_linear(self._h, layer, which).contents
        def arr(ptr, shape, dt):
            if not ptr:
                return None
            n = int(np.prod(shape))
            buf = (C.c_byte * (n * np.dtype(dt).itemsize)).from_address(ptr)
            return np.frombuffer(buf, dtype=dt).reshape(shape)
        if s.bits == 16:
            return QWeight(s.n, s.k, 16, None, None, None, dense=arr(s.dense, (s.n, s.k), np.uint16),
                           lin_bias=arr(s.lin_bias, (s.n,), np.uint16))
        return QWeight(s.n, s.k, s.bits, arr(s.packed, (s.n, s.k * s.bits // 32), np.uint32),
                       arr(s.scales, (s.n, s.k // 64), np.uint16), arr(s.biases, (s.n, s.k // 64), np.uint16),
                       lin_bias=arr(s.lin_bias, (s.n,), np.uint16))

    def vec(self, layer: int, which: int, n: int) -> np.ndarray | None:
        ptr = lib().fko_model_vec(self._h, layer, which)
        if not ptr:
            return None
        buf = (C.c_byte * (n * 2)).from_address(ptr)
        return np.frombuffer(buf, dtype=np.uint16)       # a writable view of the oracle's own memory

    def set_cache(self, layer: int, k_bits: np.ndarray, v_bits: np.ndarray):
        """Overwrite a layer's K/V cache (bf16 bits, [n_kv, capacity, head_dim])."""
        n = k_bits.size
        self.vec(layer, 7, n)[:] = np.asarray(k_bits, np.uint16).reshape(-1)
        self.vec(layer, 8, n)[:] = np.asarray(v_bits, np.uint16).reshape(-1)

    def layer_cap(self, l): return int(lib().fko_model_layer_cap(self._h, l))
    def layer_sliding(self, l): return bool(lib().fko_model_layer_sliding(self._h, l))
    def layer_theta(self, l): return float(lib().fko_model_layer_theta(self._h, l))
    def embed_scale(self): return float(lib().fko_model_embed_scale(self._h))

    def step(self, tok: int, pos: int, want_hidden=False, want_logits=False):
        c = self.cfg
        hid = np.empty((c.n_layers + 1, c.hidden), np.uint16) if want_hidden else None
        lg = np.empty(c.vocab, np.uint16) if want_logits else None
        nxt = lib().fko_decode_step(self._h, tok, pos, _p(hid), _p(lg))
        return int(nxt), hid, lg

    def layer_step(self, layer: int, x_bf16: np.ndarray, pos: int) -> np.ndarray:
        """Layer `layer` applied to a given residual stream (teacher-forced per-layer check)."""
        x = np.ascontiguousarray(x_bf16, np.uint16).copy()
        lib().fko_layer_step(self._h, layer, _p(x), pos)
        return x

    def head_step(self, x_bf16: np.ndarray):
        lg = np.empty(self.cfg.vocab, np.uint16)
        tok = lib().fko_head_step(self._h, _p(np.ascontiguousarray(x_bf16, np.uint16)), _p(lg))
        return int(tok), lg

    def greedy(self, first_tok: int, pos0: int, steps: int):
        out = np.empty(steps, np.uint32)
        secs = lib().fko_decode_greedy(self._h, first_tok, pos0, steps, _p(out))
        return out, float(secs)


def compare_greedy(got_tokens, oracle_model, first_tok: int, pos0: int, tie_ulps: float = 2.0, stats: dict | None = None):
    """Walk the oracle along the GPU's token stream.  Returns (mismatches, ties): a mismatch where the
    oracle's own margin between its winner and the GPU's token is at most `tie_ulps` bf16 ulps of the logit
    is a near-tie (random-init logits are almost flat; the reference itself documents token flips
    from reordered fp32 sums); anything larger is a real mismatch.  `stats`, when given, receives
    ``ambiguous_steps``: the steps at which the oracle's own runner-up lies within `tie_ulps` ulps of its winner,
    i.e. the only steps at which a near-tie can occur at all."""
    tok, mism, ties, amb = first_tok, [], [], 0
    for i, g in enumerate(int(t) for t in got_tokens):
        want, _, lg = oracle_model.step(tok, pos0 + i, want_logits=True)
        l = bf16_to_f32(np.asarray(lg, np.uint16))
        ulp = 2.0 ** (np.floor(np.log2(max(abs(float(l[want])), 1e-30))) - 7)
        if stats is not None:
            top2 = np.partition(l, -2)[-2:]
            amb += int(float(top2[1] - top2[0]) <= tie_ulps * ulp)
        if want != g:
            margin = float(l[want] - l[g])
            (ties if margin <= tie_ulps * ulp else mism).append((i, want, g, margin, ulp))
        tok = g
    if stats is not None:
        stats["ambiguous_steps"] = amb
    return mism, ties



# ====================================================== NumPy restatement ==
# An independent second statement of the small ops (vectorised, float32 with
# explicit bf16 rounding).  Summation order differs from the C oracle, so the
# matvec/sdpa comparisons use a tolerance; the integer/byte work (unpack,
# dequant) and the elementwise chains must agree exactly.
def np_unpack(packed: np.ndarray, bits: int) -> np.ndarray:
    per = 32 // bits
    sh = (np.arange(per, dtype=np.uint32) * bits)
    q = (packed[..., None] >> sh) & np.uint32((1 << bits) - 1)
    return q.reshape(packed.shape[0], -1)


def np_dequant(w: QWeight) -> np.ndarray:
    q = np_unpack(w.packed, w.bits).astype(np.float32)
    s = np.repeat(bf16_to_f32(w.scales), 64, axis=1)
    b = np.repeat(bf16_to_f32(w.biases), 64, axis=1)
    return (q * s).astype(np.float32) + b


def np_round(a):
    return bf16_to_f32(f32_to_bf16(np.asarray(a, np.float32)))


def np_rmsnorm(x_bf16, w_bf16, eps):
    x = bf16_to_f32(x_bf16)
    ss = np.float32(np.sum((x * x).astype(np.float64)))
    r = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(x.size)) + np.float32(eps), dtype=np.float32)
    return np_round(bf16_to_f32(w_bf16) * np_round(x * r))


def np_swiglu(gate_acc, up_acc):
    g, u = np_round(gate_acc), np_round(up_acc)
    sg = np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))
    return f32_to_bf16((sg * g) * u)


def np_geglu_tanh(gate_acc, up_acc):
    g, u = np_round(gate_acc), np_round(up_acc)
    g3 = np_round(np_round(g * g) * g)
    t2 = np_round(g + np_round(np.float32(0.044715) * g3))
    t3 = np_round(np.float32(0.7978845608028654) * t2)
    t4 = np_round(np.tanh(np.clip(t3, -20.0, 20.0), dtype=np.float32))
    t7 = np_round(np_round(np.float32(0.5) * g) * np_round(np.float32(1.0) + t4))
    return f32_to_bf16(t7 * u)


def np_sdpa(q, ck, cv, n_q, n_kv, hd, capacity, kv_len, scale):
    qf = bf16_to_f32(q).reshape(n_q, hd).astype(np.float64)
    K = bf16_to_f32(ck).reshape(n_kv, capacity, hd)[:, :kv_len].astype(np.float64)
    V = bf16_to_f32(cv).reshape(n_kv, capacity, hd)[:, :kv_len].astype(np.float64)
    out = np.empty((n_q, hd))
    for h in range(n_q):
        kvh = h // (n_q // n_kv)
        s = (K[kvh] @ qf[h]) * scale
        p = np.exp(s - s.max()); p /= p.sum()
        out[h] = p @ V[kvh]
    return out.reshape(-1)
