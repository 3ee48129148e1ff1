"""Host side of the decode path: binds model tensors to device buffers, builds the
per-token dispatch list, captures it once as a CUDA graph and replays it per token.

It mirrors the reference's ``Dispatcher`` (python/fusekit_runtime/dispatch.py:
``_build_dispatches`` :3163-3611, ``_ensure_icb`` :3864-4024, ``_try_run_single``
:4380-4548) and the greedy chunk loop of ``_fast_generate_step``
(python/fusekit_runtime/__init__.py:4782-5139), with the Metal indirect command buffer
replaced by a graph that the native library owns.  Everything numeric happens in
``libfusekit_cuda.so``; this module only does bookkeeping.
"""
from __future__ import annotations

import ctypes as C
import json
import math

import numpy as np

from . import _native as N
from . import task_graph
from .model_spec import ModelSpec, stream_id, tensor_name

FK_CHUNK = 64          # tokens pre-submitted per chunk (reference FK_CHUNK, dispatch.py:1103)


def _bf16_round(v: float) -> float:
    u = int(np.array([v], np.float32).view(np.uint32)[0])
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return float(np.array([u], np.uint32).view(np.float32)[0])


class Runtime:
    """Thin owner of one ``fk_handle`` (reference: ``load_dispatcher`` handle, lib.rs:115)."""

    def __init__(self, device: int = 0):
        self.L = N.lib()
        h = C.c_uint64()
        N.check(self.L.fk_open(device, C.byref(h)), "fk_open")
        self.h = h.value
        self.device = device

    def close(self):
        if self.h:
            self.L.fk_close(self.h)
            self.h = 0

    def info(self) -> dict:
        buf = C.create_string_buffer(1024)
        N.check(self.L.fk_info(self.h, buf, len(buf)), "fk_info")
        return json.loads(buf.value.decode())

    def alloc(self, nbytes: int) -> int:
        p = C.c_uint64()
        N.check(self.L.fk_alloc(self.h, nbytes, C.byref(p)), "fk_alloc")
        return p.value

    def upload(self, dptr: int, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        N.check(self.L.fk_upload(self.h, dptr, arr.ctypes.data, arr.nbytes), "fk_upload")

    def to_device(self, arr: np.ndarray) -> int:
        p = self.alloc(arr.nbytes)
        self.upload(p, arr)
        return p

    def download(self, dptr: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype)
        N.check(self.L.fk_download(self.h, out.ctypes.data, dptr, out.nbytes), "fk_download")
        return out

    def sync(self):
        N.check(self.L.fk_sync(self.h), "fk_sync")

    def smoke(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        out = np.empty_like(a)
        N.check(self.L.fk_smoke(self.h, a.ctypes.data, b.ctypes.data, out.ctypes.data, a.size), "fk_smoke")
        return out

    # ---- weights
    def weight_alloc(self, n: int, k: int, bits: int) -> int:
        w = C.c_uint64()
        N.check(self.L.fk_weight_alloc(self.h, n, k, bits, C.byref(w)), "fk_weight_alloc")
        return w.value

    def weight_upload_rows(self, wid: int, row0: int, packed, scales=None, biases=None):
        packed = np.ascontiguousarray(packed)
        sp = np.ascontiguousarray(scales).ctypes.data if scales is not None else None
        bp = np.ascontiguousarray(biases).ctypes.data if biases is not None else None
        N.check(self.L.fk_weight_upload_rows(self.h, wid, row0, packed.shape[0], packed.ctypes.data, sp, bp), "fk_weight_upload_rows")

    def weight_synth_rows(self, wid, dst_row0, nrows, stream, std, k_global, src_row0, k0):
        N.check(self.L.fk_weight_synth_rows(self.h, wid, dst_row0, nrows, stream, std, k_global, src_row0, k0), "fk_weight_synth_rows")

    def weight_finalize(self, wid):
        N.check(self.L.fk_weight_finalize(self.h, wid), "fk_weight_finalize")

    def weight_set_rows(self, wid, kind: int, head_dim: int, n_rot_rows: int):
        N.check(self.L.fk_weight_set_rows(self.h, wid, kind, head_dim, n_rot_rows), "fk_weight_set_rows")

    def weight_pair(self, gate: int, up: int) -> int:
        out = C.c_uint64()
        N.check(self.L.fk_weight_pair(self.h, gate, up, C.byref(out)), "fk_weight_pair")
        return out.value

    @property
    def tiled(self) -> bool:
        """True when weights are repacked into the streaming layout (default)."""
        import os
        return os.environ.get("FK_LAYOUT", "") != "mlx"

    def weight_dequant(self, wid, row0, nrows, k) -> np.ndarray:
        out = np.empty((nrows, k), np.float32)
        N.check(self.L.fk_weight_dequant(self.h, wid, row0, nrows, out.ctypes.data), "fk_weight_dequant")
        return out

    def synth_normal(self, dptr, stream, idx0, n, mean, std):
        N.check(self.L.fk_synth_normal_bf16(self.h, dptr, stream, idx0, n, mean, std), "fk_synth_normal_bf16")

    # ---- launches
    def launch(self, task: N.Task):
        N.check(self.L.fk_launch(self.h, C.byref(task)), "fk_launch")

    def launch_batch(self, tasks):
        arr = (N.Task * len(tasks))(*tasks)
        N.check(self.L.fk_launch_batch(self.h, arr, len(tasks)), "fk_launch_batch")

    def state_set(self, token: int, offset: int):
        N.check(self.L.fk_state_set(self.h, token, offset), "fk_state_set")

    def state_get(self):
        t, o, e = C.c_uint32(), C.c_uint32(), C.c_uint32()
        N.check(self.L.fk_state_get(self.h, C.byref(t), C.byref(o), C.byref(e)), "fk_state_get")
        return t.value, o.value, e.value


def linear_plan(spec: ModelSpec, rank: int = 0, world: int = 1):
    """(name, [(leaf, src_row0, nrows)], k_global, k0, k, layer) for every weight object of tensor-parallel rank
    `rank`: q/k/v, gate/up and the lm_head are split by output rows (whole heads), o/down by input columns
    (whole quantisation groups), so a rank's tensors are exact slices of the full model's."""
    hd, H = spec.head_dim, spec.hidden
    nq, nkv, I, V = spec.n_q // world, spec.n_kv // world, spec.inter // world, spec.vocab // world
    r = rank
    plan = []
    for l in range(spec.n_layers):
        plan.append((f"layers.{l}.qkv", [("q_proj", r * nq * hd, nq * hd), ("k_proj", r * nkv * hd, nkv * hd),
                                         ("v_proj", r * nkv * hd, nkv * hd)], H, 0, H, l))
        plan.append((f"layers.{l}.o", [("o_proj", 0, H)], spec.n_q * hd, r * nq * hd, nq * hd, l))
        plan.append((f"layers.{l}.gate", [("gate_proj", r * I, I)], H, 0, H, l))
        plan.append((f"layers.{l}.up", [("up_proj", r * I, I)], H, 0, H, l))
        plan.append((f"layers.{l}.down", [("down_proj", 0, H)], spec.inter, r * I, I, l))
    plan.append(("lm_head", [("lm_head", r * V, V)], H, 0, H, -1))
    return plan


def vector_plan(spec: ModelSpec, rank: int = 0, world: int = 1):
    """(name, leaf, layer, idx0, n, mean, std) for every bf16 vector/table of rank `rank` (norms and the embedding
    are replicated, the q/k/v biases follow their heads)."""
    hd, H = spec.head_dim, spec.hidden
    nq, nkv = spec.n_q // world, spec.n_kv // world
    r = rank
    out = [("embed_tokens", "embed_tokens", -1, 0, spec.vocab * H, 0.0, 0.02), ("final_norm", "final_norm", -1, 0, H, 1.0, 0.02)]
    for l in range(spec.n_layers):
        out.append((f"layers.{l}.input_norm", "input_norm", l, 0, H, 1.0, 0.02))
        out.append((f"layers.{l}.post_attention_norm", "post_attention_norm", l, 0, H, 1.0, 0.02))
        if spec.arch == "qwen2":
            out.append((f"layers.{l}.q_bias", "q_bias", l, r * nq * hd, nq * hd, 0.0, 0.02))
            out.append((f"layers.{l}.k_bias", "k_bias", l, r * nkv * hd, nkv * hd, 0.0, 0.02))
            out.append((f"layers.{l}.v_bias", "v_bias", l, r * nkv * hd, nkv * hd, 0.0, 0.02))
        else:
            for leaf, n in (("pre_feedforward_norm", H), ("post_feedforward_norm", H), ("q_norm", hd), ("k_norm", hd)):
                out.append((f"layers.{l}.{leaf}", leaf, l, 0, n, 1.0, 0.02))
    return out


def check_tp(spec: ModelSpec, world: int):
    if spec.n_kv % world or spec.n_q % world or spec.inter % world or spec.vocab % world:
        raise ValueError("tensor-parallel degree must divide heads, intermediate size and vocabulary")
    if (spec.inter // world) % 64 or (spec.n_q // world * spec.head_dim) % 64:
        raise ValueError("row-split shards must keep whole quantisation groups of 64")
    if world > 1 and spec.arch != "qwen2":
        raise ValueError("tensor parallelism is wired for the Qwen-shaped layer only")


class DecodeEngine:
    """One model instance (or one tensor-parallel slice of it) resident on a GPU."""

    def __init__(self, spec: ModelSpec, capacity: int, device: int = 0, tp_rank: int = 0, tp_size: int = 1,
                 want_logits: bool = False, runtime: Runtime | None = None, kv_bits: int = 0, fuse_attention: bool | None = None):
        check_tp(spec, tp_size)
        self.kv_bits = kv_bits           # 4 / 8: quantised KV cache (reference: the *_quant cache kernels); 0: bf16
        if kv_bits and (kv_bits not in (4, 8) or spec.arch != "qwen2" or tp_size > 1):
            raise ValueError("the quantised KV cache is wired for Qwen-shaped layers on one GPU, 4 or 8 bits")
        self.spec, self.capacity, self.rank, self.world = spec, capacity, tp_rank, tp_size
        self.rt = runtime or Runtime(device)
        self.want_logits = want_logits
        # attention in the tail of the QKV kernel (no sdpa task): Qwen-shaped layers on one GPU, streaming layout, bf16 cache.  Off
        # unless asked for (FK_ATTEND=1): its two grid-wide hand-offs through global memory cost more than the launch they save
        # (689 against 780 tok/s on the 7B shape at context 512)
        import os
        can_fuse = (spec.arch == "qwen2" and not kv_bits and self.rt.tiled and spec.head_dim in (64, 128) and spec.n_q // spec.n_kv <= 8)
        can_fuse = can_fuse and tp_size == 1
        self.fuse_attention = can_fuse and (os.environ.get("FK_ATTEND", "0") == "1" if fuse_attention is None else bool(fuse_attention))
        s = spec
        self.nq, self.nkv, self.inter, self.vocab = s.n_q // tp_size, s.n_kv // tp_size, s.inter // tp_size, s.vocab // tp_size
        self.W: dict[str, int] = {}      # name -> fk_weight id
        self.V: dict[str, int] = {}      # name -> device address of a bf16 vector
        self.cache: list[tuple[int, int, int]] = []     # (k, v, capacity) per layer
        self.graph = 0
        self.embed_bits = 16             # 4 / 8: the embedding table is quantised (load_from with an embed provider)
        self._alloc_buffers()

    # ------------------------------------------------------------------ buffers
    def _alloc_buffers(self):
        s, rt, H = self.spec, self.rt, self.spec.hidden
        L = s.n_layers
        self.X = rt.alloc((L + 1) * H * 2)            # residual stream at each layer input (+ final)
        self.HB = rt.alloc(L * H * 2)                 # residual stream after attention
        self.q_buf = rt.alloc(self.nq * s.head_dim * 2)
        self.k_buf = rt.alloc(self.nkv * s.head_dim * 2)
        self.v_buf = rt.alloc(self.nkv * s.head_dim * 2)
        self.sdpa_buf = rt.alloc(self.nq * s.head_dim * 2)
        self.act_buf = rt.alloc(self.inter * 2)
        self.act_digits = rt.alloc(self.inter * 3 + 16 + (self.inter // 32 + 1) * 8)      # the same vector as staged digits + per-group pairs
        self.o_buf = rt.alloc(H * 2)                  # Gemma: o_proj output before its post-norm
        self.d_buf = rt.alloc(L * H * 2)              # Gemma: down_proj output before its post-norm
        self.part_f32 = rt.alloc(H * 4)               # tensor-parallel partial sums (o_proj)
        self.part_f32_b = rt.alloc(H * 4)             # tensor-parallel partial sums (down_proj)
        max_cap = max(s.layer_capacity(l, self.capacity) for l in range(L))
        chunks = (max_cap + 31) // 32
        self.sdpa_part = rt.alloc(self.nq * chunks * (s.head_dim + 2) * 4)
        self.sdpa_counter = rt.alloc(max(self.nkv, 1) * 4)
        # attention as the tail of the QKV kernel: 64 bytes of hand-off counters + one partial per block (<= 512) and q head (<= 8)
        self.attend_scratch = rt.alloc(64 + 512 * 8 * (s.head_dim + 2) * 4)
        self.argmax_scratch = rt.alloc(8 * 1024)
        self.head_counter = rt.alloc(4)
        self.logits = rt.alloc(self.vocab * 2) if self.want_logits else 0
        self.cacheq: list[dict] = []                   # quantised caches: packed words + scales / biases per layer
        for l in range(L):
            cap = s.layer_capacity(l, self.capacity)
            if self.kv_bits:
                rows, ng = self.nkv * cap, s.head_dim // 64
                nb = rows * s.head_dim * self.kv_bits // 8
                self.cacheq.append({"k": rt.alloc(nb), "v": rt.alloc(nb), "k_scales": rt.alloc(rows * ng * 2), "k_biases": rt.alloc(rows * ng * 2),
                                    "v_scales": rt.alloc(rows * ng * 2), "v_biases": rt.alloc(rows * ng * 2)})
                self.cache.append((0, 0, cap))
                continue
            k, v = C.c_uint64(), C.c_uint64()
            N.check(rt.L.fk_kv_cache_alloc(rt.h, self.nkv, cap, s.head_dim, C.byref(k), C.byref(v)), "fk_kv_cache_alloc")
            self.cache.append((k.value, v.value, cap))

    def x_ptr(self, l: int) -> int:
        return self.X + l * self.spec.hidden * 2

    def hb_ptr(self, l: int) -> int:
        return self.HB + l * self.spec.hidden * 2

    def d_ptr(self, l: int) -> int:
        return self.d_buf + l * self.spec.hidden * 2

    # ------------------------------------------------------------------ tensors
    def _linear_plan(self):
        return linear_plan(self.spec, self.rank, self.world)

    def _vector_plan(self):
        return vector_plan(self.spec, self.rank, self.world)

    def load_synthetic(self):
        """Generate every tensor on the device from its named stream (seeded, bit-identical to the
        documented CPU generator)."""
        s, rt = self.spec, self.rt
        for name, segs, k_global, k0, k, layer in self._linear_plan():
            wid = rt.weight_alloc(sum(n for _, _, n in segs), k, s.bits)
            row = 0
            for leaf, src_row0, n in segs:
                rt.weight_synth_rows(wid, row, n, stream_id(s.seed, tensor_name(layer, leaf)), 0.02, k_global, src_row0, k0)
                row += n
            self._finish_weight(name, wid)
        self._load_vectors(lambda leaf, layer, idx0, n, mean, std, dst: rt.synth_normal(
            dst, stream_id(s.seed, tensor_name(layer, leaf)), idx0, n, mean, std))
        rt.sync()

    def load_from(self, weight_provider, vector_provider, embed=None):
        """Upload host tensors in MLX-affine layout.  ``weight_provider(leaf, layer, src_row0, nrows,
        k_global, k0, k, bits) -> (packed_or_dense, scales, biases)``; ``vector_provider(leaf, layer,
        idx0, n, mean, std) -> uint16 array``; ``embed``: None for a bf16 embedding table served by the vector
        provider, or ``{"bits", "packed", "scales", "biases"}`` for a quantised one (fusekit_b200.checkpoint)."""
        s, rt = self.spec, self.rt
        for name, segs, k_global, k0, k, layer in self._linear_plan():
            wid = rt.weight_alloc(sum(n for _, _, n in segs), k, s.bits)
            row = 0
            for leaf, src_row0, n in segs:
                p, sc, bi = weight_provider(leaf, layer, src_row0, n, k_global, k0, k, s.bits)
                rt.weight_upload_rows(wid, row, p, sc, bi)
                row += n
            self._finish_weight(name, wid)
        if embed is not None:
            self.embed_bits = int(embed["bits"])
            self.V["embed_tokens"] = rt.to_device(np.ascontiguousarray(embed["packed"], np.uint32))
            self.V["embed_tokens.scales"] = rt.to_device(np.ascontiguousarray(embed["scales"], np.uint16))
            self.V["embed_tokens.biases"] = rt.to_device(np.ascontiguousarray(embed["biases"], np.uint16))
        self._load_vectors(lambda leaf, layer, idx0, n, mean, std, dst: rt.upload(dst, vector_provider(leaf, layer, idx0, n, mean, std)))
        rt.sync()

    def _finish_weight(self, name: str, wid: int):
        """Choose the tile row order the consuming kernel wants, then freeze the weight."""
        s, rt = self.spec, self.rt
        paired = rt.tiled
        if name.endswith(".qkv") and s.arch == "qwen2" and paired and not self.kv_bits:
            rt.weight_set_rows(wid, 1, s.head_dim, (self.nq + self.nkv) * s.head_dim)
        if paired and (name.endswith(".gate") or name.endswith(".up")):
            self.W[name] = wid                       # frozen together once both halves exist
            g, u = name.rsplit(".", 1)[0] + ".gate", name.rsplit(".", 1)[0] + ".up"
            if g in self.W and u in self.W:
                self.W[name.rsplit(".", 1)[0] + ".gateup"] = rt.weight_pair(self.W.pop(g), self.W.pop(u))
            return
        rt.weight_finalize(wid)
        self.W[name] = wid

    def _load_vectors(self, fill):
        s, rt = self.spec, self.rt
        for name, leaf, layer, idx0, n, mean, std in self._vector_plan():
            if leaf in ("q_bias", "k_bias", "v_bias") or name in self.V:
                continue
            self.V[name] = rt.alloc(n * 2)
            fill(leaf, layer, idx0, n, mean, std, self.V[name])
        if s.arch == "qwen2":          # q|k|v biases concatenated like the fused weight rows
            hd = s.head_dim
            for l in range(s.n_layers):
                nq, nkv = self.nq * hd, self.nkv * hd
                p = rt.alloc((nq + 2 * nkv) * 2)
                fill("q_bias", l, self.rank * nq, nq, 0.0, 0.02, p)
                fill("k_bias", l, self.rank * nkv, nkv, 0.0, 0.02, p + nq * 2)
                fill("v_bias", l, self.rank * nkv, nkv, 0.0, 0.02, p + (nq + nkv) * 2)
                self.V[f"layers.{l}.qkv_bias"] = p

    def prefill_kv_synthetic(self, ctx: int):
        """Fill positions [0, ctx) of every cache with N(0,1) values keyed by (layer, global kv head,
        position); ring caches keep the last `window` positions at row p % window."""
        s, rt, hd = self.spec, self.rt, self.spec.head_dim
        for l, (ck, cv, cap) in enumerate(self.cache):
            sk, sv = stream_id(s.seed, f"layers.{l}.cache_k"), stream_id(s.seed, f"layers.{l}.cache_v")
            for hh in range(self.nkv):
                gh = self.rank * self.nkv + hh
                p0 = max(0, ctx - cap) if s.is_sliding(l) else 0
                segs = []
                p = p0
                while p < ctx:                     # contiguous runs of rows inside the ring
                    row = p % cap if s.is_sliding(l) else p
                    run = min(ctx - p, cap - row)
                    segs.append((p, row, run)); p += run
                for p, row, run in segs:
                    idx0 = (gh * 1048576 + p) * hd
                    off = (hh * cap + row) * hd * 2
                    rt.synth_normal(ck + off, sk, idx0, run * hd, 0.0, 1.0)
                    rt.synth_normal(cv + off, sv, idx0, run * hd, 0.0, 1.0)
        rt.sync()

    def upload_kv(self, layer: int, k: np.ndarray, v: np.ndarray):
        ck, cv, _ = self.cache[layer]
        self.rt.upload(ck, k); self.rt.upload(cv, v)

    # ------------------------------------------------------------------ dispatch list
    def task_graph(self) -> dict:
        """This engine's decode step as a v2 ``task_graph.json`` document (see task_graph.emit)."""
        return task_graph.emit(self.spec, self.capacity, self.rank, self.world,
                               fused_weights=self.rt.tiled, want_logits=self.want_logits, embed_bits=getattr(self, "embed_bits", 16), tp_exchange=getattr(self, "tp_exchange", "allreduce"), kv_bits=getattr(self, "kv_bits", 0),
                               fuse_attention=getattr(self, "fuse_attention", False), act_digits=self._act_digits())

    def _act_digits(self) -> bool:
        """Whether gate/up can leave down_proj's activations as staged digits: one GPU, Qwen-shaped, 4/8-bit streaming layout, and
        the gate/up weight of every layer launched with whole tiles per warp (asked of the library: fk_weight_plan)."""
        import os
        s = self.spec
        if getattr(self, "_act_digits_ok", None) is not None:
            return self._act_digits_ok
        if not getattr(self, "W", None) or "layers.0.gateup" not in self.W:
            return False                     # asked before the weights exist: no digits, and no verdict cached
        ok = (s.arch == "qwen2" and getattr(self, "world", 1) == 1 and s.bits in (4, 8) and getattr(self.rt, "tiled", False)
              and s.inter % 64 == 0 and os.environ.get("FK_ACT_DIGITS", "1") != "0" and hasattr(self.rt, "L") and bool(getattr(self, "act_digits", 0)))
        if ok:
            for l in range(s.n_layers):
                g, w, ls = C.c_int32(), C.c_int32(), C.c_int32()
                wid = self.W.get(f"layers.{l}.gateup")
                if not wid or self.rt.L.fk_weight_plan(self.rt.h, wid, C.byref(g), C.byref(w), C.byref(ls)) != 0 or ls.value != 0:
                    ok = False
                    break
                tiles = (2 * s.inter + 15) // 16
                if -(-tiles // (g.value * w.value)) * w.value * 8 > 1024:
                    ok = False
                    break
        self._act_digits_ok = ok
        return ok

    def _resolve(self, role: str) -> int:
        """Device address (or fk_weight id) behind one role string of the task graph."""
        p = role.split(".")
        if p[0] == "param":
            return self.W["lm_head"] if p[1] == "lm_head" else self.V[".".join(p[1:])]
        if p[0] == "layer_param":
            l, rel = int(p[1]), ".".join(p[2:])
            w = {"self_attn.qkv_proj": "qkv", "self_attn.o_proj": "o", "mlp.gate_up_proj": "gateup", "mlp.gate_proj": "gate",
                 "mlp.up_proj": "up", "mlp.down_proj": "down"}
            v = {"input_layernorm.weight": "input_norm", "self_attn.qkv_proj.bias": "qkv_bias", "post_attention_layernorm.weight": "post_attention_norm",
                 "pre_feedforward_layernorm.weight": "pre_feedforward_norm", "post_feedforward_layernorm.weight": "post_feedforward_norm",
                 "self_attn.q_norm.weight": "q_norm", "self_attn.k_norm.weight": "k_norm"}
            return self.W[f"layers.{l}.{w[rel]}"] if rel in w else self.V[f"layers.{l}.{v[rel]}"]
        if p[0].startswith("layer_cache_") and getattr(self, "kv_bits", 0):
            return self.cacheq[int(p[1])][p[0][len("layer_cache_"):]]
        if p[0] == "layer_cache_k":
            return self.cache[int(p[1])][0]
        if p[0] == "layer_cache_v":
            return self.cache[int(p[1])][1]
        if p[0] == "global_scratch":
            if p[1] == "x_in":
                return self.x_ptr(int(p[2]))
            return {"sdpa_partials": self.sdpa_part, "sdpa_counter": self.sdpa_counter, "argmax_scratch": self.argmax_scratch, "attend_scratch": getattr(self, "attend_scratch", 0),
                    "head_counter": self.head_counter, "logits": self.logits, "tp_partial_a": self.part_f32, "tp_partial_b": self.part_f32_b}[p[1]]
        if p[0] == "layer_scratch":
            if p[1].isdigit():
                return {"h_attn": self.hb_ptr, "out_buf": self.d_ptr}[p[2]](int(p[1]))
            return {"q_buf": self.q_buf, "k_buf": self.k_buf, "v_buf": self.v_buf, "sdpa_buf": self.sdpa_buf, "silu_up": self.act_buf,
                    "o_buf": self.o_buf, "silu_up_digits": getattr(self, "act_digits", 0)}[p[1]]
        raise KeyError(f"unknown task-graph role {role!r}")

    def dispatches_from(self, graph: dict) -> list:
        """Resolve a task graph document (from task_graph.emit or read back from JSON) to the fk_task list, in
        decode_pipeline order (the reference's replay order, src/codegen/task_graph_json.rs:1619-1664)."""
        if graph.get("version") != task_graph.VERSION:
            raise ValueError(f"task graph version {graph.get('version')} (this runtime reads {task_graph.VERSION})")
        if graph.get("active_m", 1) != 1:
            raise ValueError("only batch-1 decode graphs are dispatchable")
        if not graph["decode_capabilities"]["dispatchable"]:
            raise ValueError("task graph is not dispatchable: " + "; ".join(graph["decode_capabilities"]["reasons"]))
        by_id = {t["id"]: t for t in graph["tasks"]}
        out = []
        for tid in graph["decode_pipeline"]:
            t = by_id[tid]
            bufs = {slot: self._resolve(role) for slot, role in task_graph.task_slots(t).items()}
            out.append(N.Task.make(t["kind"], t.get("layer_idx", -1), bufs, t["iargs"], t["fargs"]))
        return out

    def role_table(self, graph: dict) -> list:
        """(role, address-or-weight-id) for every explicit binding of the document: the table the library's own JSON reader
        (fk_tasks_from_json / fk_graph_capture_json) resolves role strings through."""
        roles = sorted({b["role"] for t in graph["tasks"] for b in t["extra_bindings"] if b["slot"] < 100})
        return [(r, self._resolve(r)) for r in roles]

    def dispatches_from_json(self, text: str, table=None) -> list:
        """The fk_task list of a task_graph.json text as the library parses it (no Python between the file and the records)."""
        import json
        table = self.role_table(json.loads(text)) if table is None else table
        L = N.lib()
        arr = (N.RoleBinding * max(1, len(table)))(*[N.RoleBinding(r.encode(), int(v)) for r, v in table])
        n = C.c_int32()
        N.check(L.fk_tasks_from_json(text.encode(), arr, len(table), None, 0, C.byref(n)), "fk_tasks_from_json")
        out = (N.Task * max(1, n.value))()
        N.check(L.fk_tasks_from_json(text.encode(), arr, len(table), out, n.value, C.byref(n)), "fk_tasks_from_json")
        return list(out)[: n.value]

    def capture_json(self, text: str) -> int:
        """Capture the decode step straight from a task_graph.json text (reference: load_dispatcher + build_icb,
        python_runtime/src/lib.rs:115-169, 459-570)."""
        import json
        table = self.role_table(json.loads(text))
        arr = (N.RoleBinding * len(table))(*[N.RoleBinding(r.encode(), int(v)) for r, v in table])
        g = C.c_uint64()
        N.check(self.rt.L.fk_graph_capture_json(self.rt.h, text.encode(), arr, len(table), C.byref(g)), "fk_graph_capture_json")
        self.tasks = self.replay = self.dispatches_from_json(text, table)
        self.graph = g.value
        return self.graph

    def build_dispatches(self) -> list:
        """The per-token kernel list in replay order (reference order: embed -> per layer RmsNormQkv,
        SDPA, LinearResidual, gate/up chain, LinearResidual -> final head -> argmax;
        src/codegen/task_graph_json.rs:1619-1664, dispatch.py:3163-3611)."""
        return self.dispatches_from(self.task_graph())

    # ------------------------------------------------------------------ replay
    def capture(self) -> int:
        """Capture the per-token task list once as a CUDA graph (reference: build_icb, lib.rs:459-570)."""
        self.tasks = self.replay = self.build_dispatches()
        arr = (N.Task * len(self.replay))(*self.replay)
        g = C.c_uint64()
        N.check(self.rt.L.fk_graph_capture(self.rt.h, arr, len(self.replay), C.byref(g)), "fk_graph_capture")
        self.graph = g.value
        return self.graph

    def run_eager(self, token: int, offset: int):
        """One token through the task list without a graph (verification path)."""
        self.rt.state_set(token, offset)
        self.rt.launch_batch(self.build_dispatches())
        return self.rt.state_get()[0]

    def decode_chunk(self, base_offset: int, seed_token: int, count: int):
        """`count` greedy tokens with on-device token feedback; returns (tokens, gpu_seconds)."""
        if not self.graph:
            self.capture()
        out = np.empty(count, np.uint32)
        secs = C.c_double()
        N.check(self.rt.L.fk_decode_chunk(self.rt.h, self.graph, base_offset, seed_token, count, out.ctypes.data, C.byref(secs)), "fk_decode_chunk")
        return out, secs.value

    def generate(self, seed_token: int, base_offset: int, max_tokens: int, chunk: int = FK_CHUNK):
        """Greedy loop in chunks of `chunk` tokens (reference: _fast_generate_step)."""
        toks, secs, tok, off = [], 0.0, seed_token, base_offset
        while len(toks) < max_tokens:
            n = min(chunk, max_tokens - len(toks))
            out, t = self.decode_chunk(off, tok, n)
            toks.extend(int(v) for v in out); secs += t; tok = int(out[-1]); off += n
        return np.array(toks, np.uint32), secs

    def generate_sampled(self, seed_token: int, base_offset: int, max_tokens: int, temperature: float = 1.0, top_k: int = 0,
                         top_p: float = 1.0, seed: int = 0):
        """Sampling beyond greedy, the way the reference does it: the fused step still runs on the GPU, the logits of every
        step come back to the host and the sampler picks the next token there (the reference hands logits to mlx-lm's
        sampler whenever the request is not greedy, python/fusekit_runtime/__init__.py:4782-4843).  Needs an engine created
        with want_logits=True.  Returns the sampled tokens."""
        if not self.logits:
            raise N.FusekitError("sampling needs an engine created with want_logits=True")
        rng = np.random.default_rng(seed)
        toks, tok = [], int(seed_token)
        for i in range(max_tokens):
            self.decode_chunk(base_offset + i, tok, 1)
            tok = sample_logits(self.last_logits(), temperature, top_k, top_p, rng)
            toks.append(tok)
        return np.array(toks, np.uint32)

    def profile_nodes(self, repeats: int = 3):
        if not self.graph:
            self.capture()
        n = len(self.replay)
        out = (C.c_double * n)()
        cnt = C.c_int()
        N.check(self.rt.L.fk_graph_profile_nodes(self.rt.h, self.graph, repeats, out, n, C.byref(cnt)), "fk_graph_profile_nodes")
        return [(self.replay[i].kind, self.replay[i].layer, out[i]) for i in range(n)]

    def time_tasks(self, tasks, repeats: int = 5) -> float:
        """Seconds per pass of `tasks` launched back to back (CUDA events on the library's stream)."""
        arr = (N.Task * len(tasks))(*tasks)
        secs = C.c_double()
        N.check(self.rt.L.fk_time_tasks(self.rt.h, arr, len(tasks), repeats, C.byref(secs)), "fk_time_tasks")
        return secs.value

    def hidden_states(self) -> np.ndarray:
        """Residual stream after every layer of the last decoded token, [n_layers, H] bf16 bits."""
        s = self.spec
        return self.rt.download(self.x_ptr(1), (s.n_layers, s.hidden), np.uint16)

    def residual_stream(self) -> np.ndarray:
        """Embedding output followed by the residual stream after every layer, [n_layers + 1, H]."""
        s = self.spec
        return self.rt.download(self.x_ptr(0), (s.n_layers + 1, s.hidden), np.uint16)

    def last_logits(self) -> np.ndarray:
        if not self.logits:
            raise N.FusekitError("engine was created without want_logits")
        return self.rt.download(self.logits, (self.vocab,), np.uint16)

    def comm_init(self, unique_id: bytes):
        _ensure_nccl_path()
        buf = C.create_string_buffer(unique_id, 128)
        N.check(self.rt.L.fk_comm_init(self.rt.h, buf, self.rank, self.world), "fk_comm_init")

    def peer_export(self) -> bytes:
        """This rank's arena for the peer-memory all-reduce as a 64-byte IPC handle (gather them in rank order)."""
        buf = C.create_string_buffer(64)
        N.check(self.rt.L.fk_peer_arena_export(self.rt.h, buf, 64), "fk_peer_arena_export")
        return buf.raw

    def peer_open(self, handles) -> bool:
        """Map the peers' arenas (`handles`: one 64-byte handle per rank, in rank order).  Returns False, leaving the
        library collective in charge, where peer mapping is not possible."""
        blob = C.create_string_buffer(b"".join(handles), 64 * len(handles))
        try:
            N.check(self.rt.L.fk_peer_arena_open(self.rt.h, blob, self.rank, self.world), "fk_peer_arena_open")
        except N.FusekitError:
            return False
        # with the arenas mapped the exchange is fused into the projection kernels (FK_TP_EXCHANGE=allreduce keeps one
        # all-reduce task per row-split projection, served by the stand-alone peer kernel)
        import os
        if self.rt.tiled and os.environ.get("FK_TP_EXCHANGE", "peer") == "peer":
            self.tp_exchange = "peer"
        return True

    def peer_disable(self):
        """Drop the peer mappings (some rank could not map them): the library collective takes over."""
        self.tp_exchange = "allreduce"
        N.check(self.rt.L.fk_peer_arena_close(self.rt.h), "fk_peer_arena_close")

    def close(self):
        self.rt.close()


def sample_logits(logits_bf16: np.ndarray, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, rng=None) -> int:
    """One token from bf16 logits (bit patterns): temperature scaling, then top-k and nucleus (top-p) filtering, then a draw.
    temperature <= 0 or top_k == 1 is the greedy choice with ties to the lowest index, like the on-device argmax."""
    x = (np.asarray(logits_bf16, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    if temperature <= 0.0 or top_k == 1:
        return int(np.argmax(x))                  # first maximum = lowest index
    x = x / temperature
    order = np.argsort(-x, kind="stable")
    if top_k and top_k > 0:
        order = order[:top_k]
    p = np.exp(x[order] - x[order[0]])
    p /= p.sum()
    if top_p < 1.0:
        keep = int(np.searchsorted(np.cumsum(p), top_p, side="left")) + 1      # smallest prefix whose mass reaches top_p
        order, p = order[:keep], p[:keep] / p[:keep].sum()
    rng = rng or np.random.default_rng()
    return int(order[int(rng.choice(len(order), p=p))])


def _ensure_nccl_path():
    """Point the library at the NCCL shipped in the Python environment unless FK_NCCL_LIB is already set."""
    import importlib.util
    import os
    if os.environ.get("FK_NCCL_LIB"):
        return
    spec = importlib.util.find_spec("nvidia")
    for base in (list(spec.submodule_search_locations) if spec and spec.submodule_search_locations else []):
        cand = os.path.join(base, "nccl", "lib", "libnccl.so.2")
        if os.path.exists(cand):
            os.environ["FK_NCCL_LIB"] = cand
            return


def comm_unique_id() -> bytes:
    _ensure_nccl_path()
    buf = C.create_string_buffer(128)
    N.check(N.lib().fk_comm_unique_id(buf, 128), "fk_comm_unique_id")
    return buf.raw


def attach(spec: ModelSpec, capacity: int, device: int = 0, **kw) -> DecodeEngine:
    """Counterpart of ``fusekit_runtime.attach`` (python/fusekit_runtime/__init__.py:3101-3156):
    returns an engine whose decode calls run on the CUDA runtime."""
    return DecodeEngine(spec, capacity, device, **kw)
