"""The compiler -> runtime contract of the decode path: a ``task_graph.json`` in the reference's v2 shape.

The reference writes this file from its fused task graph (src/codegen/task_graph_json.rs:33-226) and its runtime
reads it back (src/runtime/plan.rs:39-164, python/fusekit_runtime/dispatch.py:318-329).  Capture needs MLX, so here
the graph is produced from the model shape: one task per fused decode kernel, buffers named by the reference's
role strings (``slot_role_key``, src/codegen/kernels/mod.rs:5531-5576), in replay order (embed -> per layer
RmsNormQkv, SDPA, LinearResidual, gate/up chain, LinearResidual -> final head; task_graph_json.rs:1619-1664).
``DecodeEngine.build_dispatches`` resolves exactly this structure to device addresses, so the JSON is the list the
GPU replays, not a description on the side.
"""
from __future__ import annotations

import math

from .model_spec import ModelSpec

VERSION = 2
KINDS = ["step_init", "embed_lookup_decode", "rmsnorm_qkv", "qk_norm_rope_store", "sdpa_decode", "linear_residual",
         "rmsnorm_gateup_act", "final_rmsnorm_lm_head", "argmax_finalize", "allreduce", "residual_add", "rmsnorm_rows",
         "rope_store_rows", "argmax_rows", "kv_store_quant", "sdpa_decode_quant"]
KERNEL = {k: "fusekit_" + k for k in KINDS}
(K_STEP, K_EMBED, K_QKV, K_QKNORM, K_SDPA, K_LIN, K_GATEUP, K_HEAD, K_ARGMAX, K_ALLREDUCE, K_RESADD, K_NORMROWS, K_ROPEROWS,
 K_ARGMAXROWS, K_KVQ, K_SDPAQ) = range(16)


def _bf16_round(v: float) -> float:
    import struct
    u = struct.unpack("<I", struct.pack("<f", v))[0]
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return struct.unpack("<f", struct.pack("<I", u))[0]


def emit(spec: ModelSpec, capacity: int, tp_rank: int = 0, tp_size: int = 1, fused_weights: bool = True,
         want_logits: bool = False, embed_bits: int = 16, tp_exchange: str = "allreduce", kv_bits: int = 0,
         fuse_attention: bool = False, act_digits: bool = False) -> dict:
    """Build the v2 task graph of one decode step for `spec` (one tensor-parallel rank of it).

    `fused_weights`: weights in the streaming layout (gate/up paired, residual add after an all-reduce fused into the next
    norm-first kernel); False describes the generic kernels on MLX-layout rows.
    `tp_exchange`: how the partial rows of the row-split projections meet -- "allreduce": an all-reduce task after each
    (library collective or the stand-alone peer kernel); "peer": no task of its own, the projection pushes its partial rows
    into every rank's arena and the next norm-first kernel sums them (exchange site 2l for o_proj, 2l + 1 for down_proj of
    layer l, 2L for the argmax keys of the vocabulary-sharded head).
    `kv_bits`: 4 or 8 = quantised KV cache (Qwen-shaped layers, one GPU): the QKV task writes raw projections, a
    kv_store_quant task rotates and quantises, sdpa_decode_quant attends the packed cache
    (src/codegen/kernels/rope_kv_cache_store_decode_quant.rs, sdpa_decode_quant.rs).
    `fuse_attention`: Qwen-shaped layers with the streaming layout and a bf16 cache: no sdpa_decode task, the QKV task attends
    the cache in its tail (iarg 7, slot 7 = attention output, slot 8 = scratch, farg 2 = scale).
    `act_digits`: one GPU, Qwen-shaped layers, 4/8-bit streaming layout: the gate/up task also leaves its output as the integer
    digits down_proj stages (slot 5 of both tasks, `layer_scratch.silu_up_digits`), so down_proj copies instead of converting."""
    s, hd, H = spec, spec.head_dim, spec.hidden
    nq, nkv, inter, vocab = s.n_q // tp_size, s.n_kv // tp_size, s.inter // tp_size, s.vocab // tp_size
    tp = tp_size > 1
    fused = fused_weights
    peer = tp and tp_exchange == "peer"
    if kv_bits and (kv_bits not in (4, 8) or s.arch != "qwen2" or tp):
        raise ValueError("the quantised KV cache is wired for Qwen-shaped layers on one GPU, 4 or 8 bits")
    attend = bool(fuse_attention) and s.arch == "qwen2" and fused and not kv_bits and not tp and hd in (64, 128) and s.n_q // s.n_kv <= 8
    if peer and not fused:
        raise ValueError("the fused peer exchange needs the streaming weight layout")
    if peer and 2 * s.n_layers + 1 > 160:
        raise ValueError("the fused peer exchange has 160 sites: at most 79 layers")
    tasks: list[dict] = []

    def add(kind, layer, bufs, iargs, fargs=()):
        tasks.append({"kind": kind, "layer": layer, "bufs": {int(k): v for k, v in bufs.items() if v}, "iargs": [int(v) for v in iargs],
                      "fargs": [float(v) for v in fargs]})

    x = lambda l: f"global_scratch.x_in.{l}"           # residual stream entering layer l (l = n_layers: final)
    hb = lambda l: f"layer_scratch.{l}.h_attn"
    lp = lambda l, rel: f"layer_param.{l}.{rel}"
    gateup = (lambda l: {2: lp(l, "mlp.gate_up_proj")}) if fused else (lambda l: {2: lp(l, "mlp.gate_proj"), 3: lp(l, "mlp.up_proj")})
    emb_scale = _bf16_round(math.sqrt(H)) if s.arch == "gemma3" else 1.0      # embed_lookup_decode.rs OUTPUT_SCALE
    if embed_bits in (4, 8):      # quantised embedding rows, dequantised in the gather (embed_lookup_decode.rs:40-61 signature)
        add(K_EMBED, -1, {0: "param.embed_tokens", 1: x(0), 2: "param.embed_tokens.scales", 3: "param.embed_tokens.biases"},
            [H, 1, s.vocab, embed_bits], [emb_scale])
    else:
        add(K_EMBED, -1, {0: "param.embed_tokens", 1: x(0)}, [H, 1, s.vocab], [emb_scale])
    scale = 1.0 / math.sqrt(hd)
    for l in range(s.n_layers):
        cap, theta = s.layer_capacity(l, capacity), s.layer_theta(l)
        ck, cv = f"layer_cache_k.{l}", f"layer_cache_v.{l}"
        if s.arch == "qwen2":
            x_in, pend, pull = x(l), {}, 0
            if tp and l > 0 and fused and peer:            # x[l] = T(sum of the ranks' down_proj partials + h[l-1])
                x_in, pend, pull = hb(l - 1), {11: x(l)}, 2 * (l - 1) + 2
            elif tp and l > 0 and fused:                   # x[l] = T(all-reduced down_proj + h[l-1])
                x_in, pend = hb(l - 1), {9: "global_scratch.tp_partial_b", 11: x(l)}
            if kv_bits:
                cq = {n: f"layer_cache_{n}.{l}" for n in ("k", "v", "k_scales", "k_biases", "v_scales", "v_biases")}
                add(K_QKV, l, {0: x_in, 1: lp(l, "input_layernorm.weight"), 2: lp(l, "self_attn.qkv_proj"), 3: lp(l, "self_attn.qkv_proj.bias"),
                               4: "layer_scratch.q_buf", 7: "layer_scratch.k_buf", 8: "layer_scratch.v_buf"}, [H, nq, nkv, hd, cap, 0], [s.eps, theta])
                add(K_KVQ, l, {0: "layer_scratch.q_buf", 1: "layer_scratch.k_buf", 2: "layer_scratch.v_buf", 3: cq["k"], 4: cq["v"], 5: cq["k_scales"],
                               6: cq["k_biases"], 7: cq["v_scales"], 8: cq["v_biases"]}, [nq, nkv, hd, cap, kv_bits], [0.0, theta])
            elif attend:
                add(K_QKV, l, {0: x_in, 1: lp(l, "input_layernorm.weight"), 2: lp(l, "self_attn.qkv_proj"), 3: lp(l, "self_attn.qkv_proj.bias"),
                               4: "layer_scratch.q_buf", 5: ck, 6: cv, 7: "layer_scratch.sdpa_buf", 8: "global_scratch.attend_scratch", **pend},
                    [H, nq, nkv, hd, cap, 1, pull, 1], [s.eps, theta, 1.0 / math.sqrt(hd)])
            else:
                add(K_QKV, l, {0: x_in, 1: lp(l, "input_layernorm.weight"), 2: lp(l, "self_attn.qkv_proj"), 3: lp(l, "self_attn.qkv_proj.bias"),
                               4: "layer_scratch.q_buf", 5: ck, 6: cv, **pend}, [H, nq, nkv, hd, cap, 1, pull], [s.eps, theta])
        else:
            x_in, pend = x(l), {}
            if l > 0:                                      # Gemma: x[l] = T(h[l-1] + rmsnorm(down_out[l-1]))
                x_in, pend = hb(l - 1), {9: f"layer_scratch.{l-1}.out_buf", 10: lp(l - 1, "post_feedforward_layernorm.weight"), 11: x(l)}
            add(K_QKV, l, {0: x_in, 1: lp(l, "input_layernorm.weight"), 2: lp(l, "self_attn.qkv_proj"), 4: "layer_scratch.q_buf",
                           7: "layer_scratch.k_buf", 8: "layer_scratch.v_buf", **pend}, [H, nq, nkv, hd, cap, 0], [s.eps, theta])
            add(K_QKNORM, l, {0: "layer_scratch.q_buf", 1: "layer_scratch.k_buf", 2: "layer_scratch.v_buf", 3: lp(l, "self_attn.q_norm.weight"),
                              4: lp(l, "self_attn.k_norm.weight"), 5: ck, 6: cv}, [nq, nkv, hd, cap], [s.eps, theta])
        if kv_bits:
            add(K_SDPAQ, l, {0: "layer_scratch.q_buf", 1: cq["k"], 2: cq["v"], 3: "layer_scratch.sdpa_buf", 4: "global_scratch.sdpa_partials",
                             5: "global_scratch.sdpa_counter", 6: cq["k_scales"], 7: cq["k_biases"], 8: cq["v_scales"], 9: cq["v_biases"]},
                [nq, nkv, hd, cap, kv_bits], [scale])
        elif not attend:
            add(K_SDPA, l, {0: "layer_scratch.q_buf", 1: ck, 2: cv, 3: "layer_scratch.sdpa_buf", 4: "global_scratch.sdpa_partials",
                            5: "global_scratch.sdpa_counter"}, [nq, nkv, hd, cap], [scale])
        ko = nq * hd
        if s.arch == "qwen2" and not tp:
            add(K_LIN, l, {0: "layer_scratch.sdpa_buf", 1: lp(l, "self_attn.o_proj"), 2: x(l), 3: hb(l)}, [ko, H])
            dig = {5: "layer_scratch.silu_up_digits"} if (act_digits and fused and s.bits in (4, 8) and inter % 64 == 0) else {}
            add(K_GATEUP, l, {0: hb(l), 1: lp(l, "post_attention_layernorm.weight"), **gateup(l), 4: "layer_scratch.silu_up", **dig}, [H, inter, s.act], [s.eps])
            add(K_LIN, l, {0: "layer_scratch.silu_up", 1: lp(l, "mlp.down_proj"), 2: hb(l), 3: x(l + 1), **dig}, [inter, H])
        elif s.arch == "qwen2" and peer:
            # row-split o/down with the exchange fused in: the projection pushes fp32 partial rows to every rank (site in i3),
            # the next norm-first kernel waits for all ranks, sums in rank order and adds the residual (site in its last iarg)
            add(K_LIN, l, {0: "layer_scratch.sdpa_buf", 1: lp(l, "self_attn.o_proj")}, [ko, H, 0, 2 * l + 1])
            add(K_GATEUP, l, {0: x(l), 11: hb(l), 1: lp(l, "post_attention_layernorm.weight"), **gateup(l), 4: "layer_scratch.silu_up"},
                [H, inter, s.act, 0, 2 * l + 1], [s.eps])
            add(K_LIN, l, {0: "layer_scratch.silu_up", 1: lp(l, "mlp.down_proj")}, [inter, H, 0, 2 * l + 2])
        elif s.arch == "qwen2":
            # row-split o/down: fp32 partial -> all-reduce over the ranks; the residual add rides in the next norm-first
            # kernel's prologue (streamed weights) or in a small kernel (generic weights)
            pa, pb = "global_scratch.tp_partial_a", "global_scratch.tp_partial_b"
            add(K_LIN, l, {0: "layer_scratch.sdpa_buf", 1: lp(l, "self_attn.o_proj"), 4: pa}, [ko, H])
            add(K_ALLREDUCE, l, {0: pa}, [H, 0])
            if not fused:
                add(K_RESADD, l, {0: pa, 1: x(l), 2: hb(l)}, [H])
            gin = {0: x(l), 9: pa, 11: hb(l)} if fused else {0: hb(l)}
            add(K_GATEUP, l, {**gin, 1: lp(l, "post_attention_layernorm.weight"), **gateup(l), 4: "layer_scratch.silu_up"}, [H, inter, s.act], [s.eps])
            add(K_LIN, l, {0: "layer_scratch.silu_up", 1: lp(l, "mlp.down_proj"), 4: pb}, [inter, H])
            add(K_ALLREDUCE, l, {0: pb}, [H, 0])
            if not fused:
                add(K_RESADD, l, {0: pb, 1: hb(l), 2: x(l + 1)}, [H])
        else:
            # Gemma-shaped: o_proj plain; post-attention norm + residual + pre-ffn norm in the gate/up prologue
            add(K_LIN, l, {0: "layer_scratch.sdpa_buf", 1: lp(l, "self_attn.o_proj"), 3: "layer_scratch.o_buf"}, [ko, H])
            add(K_GATEUP, l, {0: x(l), 1: lp(l, "pre_feedforward_layernorm.weight"), **gateup(l), 4: "layer_scratch.silu_up",
                              9: "layer_scratch.o_buf", 10: lp(l, "post_attention_layernorm.weight"), 11: hb(l)}, [H, inter, s.act], [s.eps])
            add(K_LIN, l, {0: "layer_scratch.silu_up", 1: lp(l, "mlp.down_proj"), 3: f"layer_scratch.{l}.out_buf"}, [inter, H])
    L = s.n_layers
    x_fin, pend = x(L), {}
    if s.arch == "gemma3":
        x_fin, pend = hb(L - 1), {9: f"layer_scratch.{L-1}.out_buf", 10: lp(L - 1, "post_feedforward_layernorm.weight"), 11: x(L)}
    elif tp and fused and peer:
        x_fin, pend = hb(L - 1), {11: x(L)}
    elif tp and fused:
        x_fin, pend = hb(L - 1), {9: "global_scratch.tp_partial_b", 11: x(L)}
    add(K_HEAD, -1, {0: x_fin, 1: "param.final_norm", 2: "param.lm_head", 3: "global_scratch.logits" if want_logits else None,
                     4: "global_scratch.argmax_scratch", 5: "global_scratch.head_counter", **pend},
        [H, vocab, tp_rank * vocab, 0 if tp else 1] + ([2 * (L - 1) + 2, 2 * L + 1] if (tp and fused and peer) else []), [s.eps])
    if tp and not (fused and peer):
        add(K_ALLREDUCE, -1, {0: "global_scratch.argmax_scratch"}, [1, 1])
        add(K_ARGMAX, -1, {4: "global_scratch.argmax_scratch"}, [1])

    # ---- v2 envelope: tasks with bindings, a linear event chain, layer groups, the decode pipeline
    out_slots = {K_EMBED: [1], K_QKV: [4, 5, 6, 7, 8, 11], K_QKNORM: [0, 5, 6], K_SDPA: [3, 4, 5], K_LIN: [3, 4], K_GATEUP: [4, 5, 11],
                 K_HEAD: [3, 4, 5, 11], K_ARGMAX: [], K_ALLREDUCE: [0], K_RESADD: [2], K_KVQ: [0, 3, 4, 5, 6, 7, 8], K_SDPAQ: [3, 4, 5]}
    jtasks, groups = [], {}
    for i, t in enumerate(tasks):
        ins, outs, extra = [], [], []
        for slot, role in sorted(t["bufs"].items()):
            if role.startswith(("param.", "layer_param.")):
                ins.append({"role": "external", "tensor_id": len(ins), "source_path": "model." + role.split(".", 1)[1], "role_name": role})
            elif slot in out_slots[t["kind"]]:
                outs.append({"role": "scratch", "scratch_id": slot, "role_name": role})
            else:
                ins.append({"role": "scratch", "scratch_id": slot, "role_name": role})
            extra.append({"slot": slot, "role": role})
        if t["kind"] not in (K_ALLREDUCE, K_RESADD):
            extra += [{"slot": 100, "role": "token_id_in" if t["kind"] == K_EMBED else "layer_offset"}]
        if t["kind"] in (K_HEAD, K_ARGMAX):
            extra += [{"slot": 101, "role": "next_token_out"}]
        jt = {"id": i, "fusion_id": i, "kernel": KERNEL[KINDS[t["kind"]]], "kind": t["kind"], "grid_threads": [0, 1, 1], "threadgroup": [0, 1, 1],
              "inputs": ins, "outputs": outs, "extra_bindings": extra, "depends_on": [i - 1] if i else [], "trigger_event": i,
              "iargs": t["iargs"], "fargs": t["fargs"]}
        if t["layer"] >= 0:
            jt["layer_idx"] = t["layer"]
        jtasks.append(jt)
        region = "embed" if t["kind"] == K_EMBED else (f"layer.{t['layer']}" if t["layer"] >= 0 else "post")
        groups.setdefault(region, []).append(i)
    return {
        "version": VERSION, "active_m": 1, "tasks": jtasks,
        "events": [{"id": i, "num_triggers": 1, "fires": [i + 1] if i + 1 < len(jtasks) else []} for i in range(len(jtasks))],
        "scratch_buffers": [], "initial_tasks": [0], "model_params": [],
        "layer_groups": [{"region": r, "task_ids": ids} for r, ids in groups.items()],
        "decode_pipeline": list(range(len(jtasks))),
        "decode_capabilities": {"dispatchable": True, "reasons": []},
        "target": {"chip": "b200", "arch": "sm_100a", "tensor_parallel": tp_size, "rank": tp_rank, "bits": s.bits,
                   "launch": "grid and block sizes are chosen by the runtime from the SM count (plan_shape)"},
    }


def task_slots(jtask: dict) -> dict:
    """slot -> role of a serialised task (the explicit extra_bindings below slot 100)."""
    return {b["slot"]: b["role"] for b in jtask["extra_bindings"] if b["slot"] < 100}


def write(path, graph: dict):
    """Serialise like the reference does (pretty-printed JSON, task_graph_json.rs:260-270)."""
    import json
    with open(path, "w") as f:
        json.dump(graph, f, indent=2)


def read(path) -> dict:
    import json
    with open(path) as f:
        return json.load(f)


# ------------------------------------------------------------------ lowering a graph the reference wrote
# A task_graph.json written by the reference for a real model names Metal kernels with a fusion-id suffix
# (`fusekit_rmsnorm_qkv_f12`) and carries no shapes: they are constants of the generated shader source.  The per-token list
# it replays has a fixed family order (src/codegen/task_graph_json.rs:1619-1664; python/fusekit_runtime/dispatch.py:3163-3611):
# step_init, embed, per layer [rmsnorm_qkv, sdpa_decode, linear_residual (o_proj), chain (norm -> gate, up -> activation),
# linear_residual (down_proj)], final head, argmax scan / finalize, optional history capture.  Lowering = check that order,
# take the shapes from the model's config.json (checkpoint.spec_from_config), emit this build's graph for them, and say which
# of the reference's parameter roles feed each role of the lowered graph (q|k|v rows concatenated, gate/up paired).
_REF_FAMILIES = ("step_init", "embed_lookup_decode", "rmsnorm_qkv", "sdpa_decode", "linear_residual", "chain", "final_rmsnorm_lm_head",
                 "argmax_logits_scan", "argmax_logits_finalize", "history_capture")
_REF_SKIP = ("step_init", "argmax_logits_scan", "argmax_logits_finalize", "history_capture")     # fused into neighbours here


def reference_family(kernel: str) -> str:
    """`fusekit_<family>[_f<id>][_partial|_combine]` -> family; raises on a kernel this build has no lowering for."""
    import re
    m = re.fullmatch(r"fusekit_([a-z0-9_]+?)(?:_f\d+)?(?:_(?:partial|combine))?", kernel)
    name = m.group(1) if m else ""
    if name not in _REF_FAMILIES:
        raise ValueError(f"no lowering for reference kernel {kernel!r}")
    return name


def lower_reference(doc: dict, spec: ModelSpec, capacity: int, **emit_kw) -> tuple[dict, dict]:
    """Lower a task graph written by the reference (Qwen-shaped default decode list) to this build's graph for `spec`.

    Returns (graph, sources): `graph` is emit(spec, capacity, ...); `sources[role]` lists, in row order, the reference's
    parameter roles (`layer_param.<i>.self_attn.q_proj` ...) whose `weight` / `scales` / `biases` tensors make up that role of
    the lowered graph.  Raises ValueError when the document is not a dispatchable v2 batch-1 graph, when its per-layer kernel
    order is not the one listed above, or when a projection the lowered graph needs is bound nowhere in the layer."""
    if doc.get("version") != VERSION or doc.get("active_m", 1) != 1:
        raise ValueError("reference graph: version 2 and active_m 1 expected")
    if not doc.get("decode_capabilities", {}).get("dispatchable", False):
        raise ValueError("reference graph is not dispatchable")
    if spec.arch != "qwen2":
        raise ValueError("the lowering covers the Qwen-shaped default dispatch list")
    by_id = {t["id"]: t for t in doc["tasks"]}
    per_layer: dict[int, list] = {}
    head_seen = embed_seen = False
    for tid in doc["decode_pipeline"]:
        t = by_id[tid]
        fam = reference_family(t["kernel"])
        if fam in _REF_SKIP:
            continue
        if fam == "embed_lookup_decode":
            embed_seen = True
        elif fam == "final_rmsnorm_lm_head":
            head_seen = True
        else:
            if "layer_idx" not in t:
                raise ValueError(f"reference task {tid} ({t['kernel']}) carries no layer_idx")
            fams = per_layer.setdefault(int(t["layer_idx"]), [])
            if not (fam == "sdpa_decode" and fams and fams[-1][0] == "sdpa_decode"):      # partial + combine count once
                fams.append((fam, t))
    if not embed_seen or not head_seen:
        raise ValueError("reference graph lacks the embed lookup or the final head")
    if sorted(per_layer) != list(range(spec.n_layers)):
        raise ValueError(f"reference graph has layers {sorted(per_layer)[:3]}..., the model {spec.n_layers}")
    want = ["rmsnorm_qkv", "sdpa_decode", "linear_residual", "chain", "linear_residual"]
    sources: dict[str, list] = {"param.embed_tokens": ["param.embed_tokens"], "param.final_norm": ["param.final_norm"], "param.lm_head": ["param.lm_head"]}
    for l in range(spec.n_layers):
        got = [f for f, _ in per_layer[l]]
        if got != want:
            raise ValueError(f"layer {l}: kernel order {got}, expected {want}")
        bound = set()
        for _, t in per_layer[l]:
            for b in list(t.get("extra_bindings", [])) + [{"role": x.get("role_name", "")} for x in t.get("inputs", [])]:
                r = b.get("role", "")
                if r.startswith(f"layer_param.{l}."):
                    rel = r[len(f"layer_param.{l}."):]
                    for suffix in (".weight", ".scales", ".biases", ".bias"):
                        if rel.endswith(suffix):
                            rel = rel[: -len(suffix)]
                            break
                    bound.add(rel)
        need = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]
        missing = [n for n in need if n not in bound]
        if missing:
            raise ValueError(f"layer {l}: the reference graph binds no {missing}")
        lp = f"layer_param.{l}."
        sources[lp + "self_attn.qkv_proj"] = [lp + "self_attn.q_proj", lp + "self_attn.k_proj", lp + "self_attn.v_proj"]
        sources[lp + "self_attn.qkv_proj.bias"] = [lp + "self_attn.q_proj.bias", lp + "self_attn.k_proj.bias", lp + "self_attn.v_proj.bias"]
        sources[lp + "self_attn.o_proj"] = [lp + "self_attn.o_proj"]
        sources[lp + "mlp.gate_up_proj"] = [lp + "mlp.gate_proj", lp + "mlp.up_proj"]
        sources[lp + "mlp.down_proj"] = [lp + "mlp.down_proj"]
        sources[lp + "input_layernorm.weight"] = [lp + "input_layernorm.weight"]
        sources[lp + "post_attention_layernorm.weight"] = [lp + "post_attention_layernorm.weight"]
    return emit(spec, capacity, **emit_kw), sources
