"""Batch decode: M independent sequences (2..16), each with its own KV cache, advanced one token per step on one GPU.

Benchmark configuration 5 asks for batch 16 on the 32B shape.  The reference has no counterpart -- its M > 1 kernels serve
consecutive positions of one sequence (python/fusekit_runtime/dispatch.py:2268-2289) -- so row m of every tensor is defined
as what the batch-1 path produces for sequence m alone, and that is what the tests check (M batch-1 runs of the CPU restatement).

A step replays, per layer: RMSNorm of the M rows -> QKV projection of all rows (+bias) -> RoPE and the K/V store into each
sequence's cache -> attention per sequence -> o_proj + residual -> norm-first gate/up + SwiGLU -> down_proj + residual; then
the final norm, the lm_head for all rows and one argmax per row, all captured in one CUDA graph.  Every projection reads its
weights once for the M rows (the quantised matrix product of fk_qmm.cuh / fk_qmm_tc.cuh).  Qwen-shaped layers with 4-bit
weights only.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _native as N
from .model_spec import ModelSpec, stream_id, tensor_name
from .runtime import Runtime


class BatchDecodeEngine:
    consecutive = False          # rows are independent sequences; PrefillEngine makes them consecutive positions of one

    def __init__(self, spec: ModelSpec, capacity: int, rows: int, device: int = 0, runtime: Runtime | None = None, qmm: int = 0,
                 caches=None):
        if spec.arch != "qwen2" or spec.bits != 4:
            raise ValueError("batch decode is wired for Qwen-shaped layers with 4-bit weights")
        if not 2 <= rows <= 16:
            raise ValueError("rows must be in 2..16")
        self.spec, self.capacity, self.rows, self.qmm = spec, capacity, rows, qmm
        self.rt = runtime or Runtime(device)
        s, rt, M, H, hd = spec, self.rt, rows, spec.hidden, spec.head_dim
        self.nqkv = (s.n_q + 2 * s.n_kv) * hd
        L = s.n_layers
        self.X = rt.alloc((L + 1) * M * H * 2)            # residual stream entering each layer (+ final), [M, H] each
        self.HB = rt.alloc(L * M * H * 2)
        self.xn = rt.alloc(M * H * 2)
        self.qkv = rt.alloc(M * self.nqkv * 2)
        self.q = rt.alloc(M * s.n_q * hd * 2)
        self.sdpa = rt.alloc(M * s.n_q * hd * 2)
        self.act = rt.alloc(M * s.inter * 2)
        self.logits = rt.alloc(M * s.vocab * 2)
        self.counter = rt.alloc(4)
        chunks = (capacity + 31) // 32
        self.sdpa_part, self.sdpa_counter = rt.alloc(64), rt.alloc(64)      # unused by the cluster kernel, required by the task
        self.cache = []
        for l in range(L):
            if caches is not None:              # caches owned by another engine on the same runtime: (k, v, ...) per layer
                self.cache.append((caches[l][0], caches[l][1]))
                continue
            n = (1 if self.consecutive else M) * s.n_kv * capacity * hd * 2
            self.cache.append((rt.alloc(n), rt.alloc(n)))
        self.W: dict[str, int] = {}
        self.V: dict[str, int] = {}
        self.graph = 0

    def x_ptr(self, l): return self.X + l * self.rows * self.spec.hidden * 2
    def hb_ptr(self, l): return self.HB + l * self.rows * self.spec.hidden * 2

    # ------------------------------------------------------------------ tensors (same seeded streams as DecodeEngine)
    def load_synthetic(self):
        s, rt, hd, H, M = self.spec, self.rt, self.spec.head_dim, self.spec.hidden, self.rows

        def synth(name, segs, k):
            wid = rt.weight_alloc(sum(n for _, _, n in segs), k, 4)
            row = 0
            for leaf, layer, n in segs:
                rt.weight_synth_rows(wid, row, n, stream_id(s.seed, tensor_name(layer, leaf)), 0.02, k, 0, 0)
                row += n
            return wid

        def vec(name, leaf, layer, n, mean, std):
            p = rt.alloc(n * 2)
            rt.synth_normal(p, stream_id(s.seed, tensor_name(layer, leaf)), 0, n, mean, std)
            self.V[name] = p
            return p

        for l in range(s.n_layers):
            w = synth("qkv", [("q_proj", l, s.n_q * hd), ("k_proj", l, s.n_kv * hd), ("v_proj", l, s.n_kv * hd)], H)
            rt.weight_finalize(w); self.W[f"layers.{l}.qkv"] = w
            w = synth("o", [("o_proj", l, H)], s.n_q * hd); rt.weight_finalize(w); self.W[f"layers.{l}.o"] = w
            g, u = synth("g", [("gate_proj", l, s.inter)], H), synth("u", [("up_proj", l, s.inter)], H)
            self.W[f"layers.{l}.gateup"] = rt.weight_pair(g, u)
            w = synth("d", [("down_proj", l, H)], s.inter); rt.weight_finalize(w); self.W[f"layers.{l}.down"] = w
            vec(f"layers.{l}.input_norm", "input_norm", l, H, 1.0, 0.02)
            vec(f"layers.{l}.post_attention_norm", "post_attention_norm", l, H, 1.0, 0.02)
            # q | k | v biases, one copy per sequence: the projection adds them like a residual, T(acc + bias)
            rep = rt.alloc(M * self.nqkv * 2)
            for m in range(M):
                off, base = 0, rep + m * self.nqkv * 2
                for leaf, n in (("q_bias", s.n_q * hd), ("k_bias", s.n_kv * hd), ("v_bias", s.n_kv * hd)):
                    rt.synth_normal(base + off * 2, stream_id(s.seed, tensor_name(l, leaf)), 0, n, 0.0, 0.02)
                    off += n
            self.V[f"layers.{l}.qkv_bias_rows"] = rep
        w = synth("head", [("lm_head", -1, s.vocab)], H); rt.weight_finalize(w); self.W["lm_head"] = w
        vec("embed_tokens", "embed_tokens", -1, s.vocab * H, 0.0, 0.02)
        vec("final_norm", "final_norm", -1, H, 1.0, 0.02)
        rt.sync()

    @staticmethod
    def cache_stream(spec: ModelSpec, layer: int, which: str, seq: int) -> int:
        return stream_id(spec.seed, f"layers.{layer}.cache_{which}.seq{seq}")

    def prefill_kv_synthetic(self, ctx: int):
        """Positions [0, ctx) of every sequence's caches from N(0,1) streams keyed by (layer, k|v, sequence)."""
        s, rt, hd, cap = self.spec, self.rt, self.spec.head_dim, self.capacity
        for l, (ck, cv) in enumerate(self.cache):
            for m in range(self.rows):
                sk, sv = self.cache_stream(s, l, "k", m), self.cache_stream(s, l, "v", m)
                for hh in range(s.n_kv):
                    off = ((m * s.n_kv + hh) * cap) * hd * 2
                    idx0 = (hh * 1048576) * hd
                    rt.synth_normal(ck + off, sk, idx0, ctx * hd, 0.0, 1.0)
                    rt.synth_normal(cv + off, sv, idx0, ctx * hd, 0.0, 1.0)
        rt.sync()

    # ------------------------------------------------------------------ dispatch list
    def build_dispatches(self) -> list:
        s, M, H, hd, I = self.spec, self.rows, self.spec.hidden, self.spec.head_dim, self.spec.inter
        T, q = N.Task.make, self.qmm
        tasks = [T(N.TASK_EMBED_LOOKUP_DECODE, -1, {0: self.V["embed_tokens"], 1: self.x_ptr(0)}, [H, M, s.vocab], [1.0])]
        scale = 1.0 / math.sqrt(hd)
        for l in range(s.n_layers):
            ck, cv = self.cache[l]
            tasks += [
                T(N.TASK_RMSNORM_ROWS, l, {0: self.x_ptr(l), 1: self.V[f"layers.{l}.input_norm"], 2: self.xn}, [H, M], [s.eps]),
                T(N.TASK_LINEAR_RESIDUAL, l, {0: self.xn, 1: self.W[f"layers.{l}.qkv"], 2: self.V[f"layers.{l}.qkv_bias_rows"], 3: self.qkv},
                  [H, self.nqkv, M, 0, 0, q]),
                T(N.TASK_ROPE_STORE_ROWS, l, {0: self.qkv, 1: self.q, 5: ck, 6: cv}, [s.n_q, s.n_kv, hd, self.capacity, M, int(self.consecutive)], [0.0, s.theta]),
                T(N.TASK_SDPA_DECODE, l, {0: self.q, 1: ck, 2: cv, 3: self.sdpa, 4: self.sdpa_part, 5: self.sdpa_counter},
                  [s.n_q, s.n_kv, hd, self.capacity, 0, M, int(self.consecutive)], [scale]),
                T(N.TASK_LINEAR_RESIDUAL, l, {0: self.sdpa, 1: self.W[f"layers.{l}.o"], 2: self.x_ptr(l), 3: self.hb_ptr(l)}, [s.n_q * hd, H, M, 0, 0, q]),
                # the norm runs once for all blocks; the gate/up product takes the rows as they are (no norm weight bound)
                T(N.TASK_RMSNORM_ROWS, l, {0: self.hb_ptr(l), 1: self.V[f"layers.{l}.post_attention_norm"], 2: self.xn}, [H, M], [s.eps]),
                T(N.TASK_RMSNORM_GATEUP_ACT, l, {0: self.xn, 2: self.W[f"layers.{l}.gateup"], 4: self.act}, [H, I, 0, M], [s.eps]),
                T(N.TASK_LINEAR_RESIDUAL, l, {0: self.act, 1: self.W[f"layers.{l}.down"], 2: self.hb_ptr(l), 3: self.x_ptr(l + 1)}, [I, H, M, 0, 0, q]),
            ]
        L = s.n_layers
        tasks += [
            T(N.TASK_RMSNORM_ROWS, -1, {0: self.x_ptr(L), 1: self.V["final_norm"], 2: self.xn}, [H, M], [s.eps]),
            T(N.TASK_LINEAR_RESIDUAL, -1, {0: self.xn, 1: self.W["lm_head"], 3: self.logits}, [H, s.vocab, M, 0, 0, q]),
            T(N.TASK_ARGMAX_ROWS, -1, {0: self.logits, 5: self.counter}, [s.vocab, M, M if self.consecutive else 1]),
        ]
        return tasks

    def capture(self) -> int:
        self.tasks = self.build_dispatches()
        arr = (N.Task * len(self.tasks))(*self.tasks)
        g = C.c_uint64()
        N.check(self.rt.L.fk_graph_capture(self.rt.h, arr, len(self.tasks), C.byref(g)), "fk_graph_capture")
        self.graph = g.value
        return self.graph

    def decode_chunk(self, base_offset: int, seed_tokens, count: int):
        """`count` greedy steps of all sequences; returns (tokens [count, rows], gpu_seconds)."""
        if not self.graph:
            self.capture()
        seeds = np.ascontiguousarray(seed_tokens, np.uint32)
        if seeds.shape != (self.rows,):
            raise ValueError("one seed token per sequence")
        out = np.empty((count, self.rows), np.uint32)
        secs = C.c_double()
        N.check(self.rt.L.fk_decode_chunk_rows(self.rt.h, self.graph, base_offset, seeds.ctypes.data, self.rows, count,
                                               out.ctypes.data, C.byref(secs)), "fk_decode_chunk_rows")
        return out, secs.value

    def weight_bytes(self) -> int:
        n = C.c_uint64(); tot = 0
        for w in self.W.values():
            N.check(self.rt.L.fk_weight_nbytes(self.rt.h, w, C.byref(n)), "fk_weight_nbytes"); tot += n.value
        return tot

    def close(self):
        self.rt.close()


class PrefillEngine(BatchDecodeEngine):
    """Chunked prefill (and verify rows): the M rows of a step are M consecutive positions of ONE sequence.

    Reference: the prefill path keeps its M > 1 trace shapes for prompt chunks and speculative verify rows
    (src/commands/patch.rs:112-152, python/fusekit_runtime/__init__.py:2535-2592, 2825-2850).  Row m of a chunk sits at
    position offset + m, its K/V rows go into the one shared cache before attention, and it attends keys 0 .. offset + m
    (causal); every row's greedy prediction comes back, so the same step serves prompt ingestion (the last row's prediction
    is the first generated token) and the verification of M drafted tokens.  Pass `caches` (and `runtime`) of a DecodeEngine
    to fill the caches that engine then decodes from."""
    consecutive = True

    def prefill(self, tokens, base_offset: int = 0):
        """Run `tokens` through the model in chunks of `rows` positions starting at `base_offset`; returns the greedy
        prediction after every position, [len(tokens)].  A last partial chunk is padded with token 0: the padded rows write
        cache rows beyond the prompt, which later positions overwrite before anything attends them."""
        toks = [int(t) for t in tokens]
        M, preds = self.rows, []
        for c0 in range(0, len(toks), M):
            chunk = toks[c0:c0 + M]
            if base_offset + c0 + M > self.capacity:
                raise ValueError("prefill chunk reaches beyond the cache capacity")
            out, _ = self.decode_chunk(base_offset + c0, np.array(chunk + [0] * (M - len(chunk)), np.uint32), 1)
            preds.extend(int(t) for t in out[0][:len(chunk)])
        return np.array(preds, np.uint32)
