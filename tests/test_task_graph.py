"""Host-side checks of the task_graph.json document (reference schema: src/codegen/task_graph_json.rs:33-226) and
of its resolution to the fk_task list, without a GPU: a stand-in engine hands out fake addresses."""
import json

import pytest

from fusekit_b200 import task_graph as TG
from fusekit_b200.model_spec import CONFIGS
from fusekit_b200.runtime import DecodeEngine, linear_plan, vector_plan

V2_KEYS = {"version", "active_m", "tasks", "events", "scratch_buffers", "initial_tasks", "model_params", "layer_groups",
           "decode_pipeline", "decode_capabilities"}
TASK_KEYS = {"id", "fusion_id", "kernel", "grid_threads", "threadgroup", "inputs", "outputs", "extra_bindings", "depends_on", "trigger_event"}


class _Names(dict):
    """name -> fake address, remembering what was asked for."""
    def __init__(self, known):
        super().__init__()
        self.known, self.asked = set(known), []

    def __missing__(self, k):
        if k not in self.known:
            raise KeyError(k)
        self.asked.append(k)
        self[k] = 0x1000 + 16 * len(self.asked)
        return self[k]


def _fake_engine(spec, world=1, rank=0, fused=True):
    e = DecodeEngine.__new__(DecodeEngine)
    e.spec, e.capacity, e.rank, e.world, e.want_logits = spec, 1024, rank, world, False
    wn = {p[0] for p in linear_plan(spec, rank, world)}
    if fused:
        wn = {n for n in wn if not n.endswith((".gate", ".up"))} | {f"layers.{l}.gateup" for l in range(spec.n_layers)}
    vn = {p[0] for p in vector_plan(spec, rank, world) if not p[0].endswith(("q_bias", "k_bias", "v_bias"))}
    if spec.arch == "qwen2":
        vn |= {f"layers.{l}.qkv_bias" for l in range(spec.n_layers)}
    e.W, e.V = _Names(wn), _Names(vn)
    e.cache = [(0x100000 + 2 * l, 0x100001 + 2 * l, spec.layer_capacity(l, 1024)) for l in range(spec.n_layers)]
    e.X, e.HB, e.d_buf = 0x200000, 0x300000, 0x400000
    for i, n in enumerate(["q_buf", "k_buf", "v_buf", "sdpa_buf", "act_buf", "o_buf", "part_f32", "part_f32_b", "sdpa_part",
                           "sdpa_counter", "argmax_scratch", "head_counter"]):
        setattr(e, n, 0x500000 + 256 * i)
    e.logits = 0

    class _Rt:
        tiled = fused
    e.rt = _Rt()
    return e


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_schema_and_json_round_trip(name):
    spec = CONFIGS[name]
    g = TG.emit(spec, 1024)
    assert V2_KEYS <= set(g) and g["version"] == 2 and g["active_m"] == 1
    assert g["initial_tasks"] == [0] and g["decode_capabilities"] == {"dispatchable": True, "reasons": []}
    per_layer = 5 if spec.arch == "qwen2" else 6
    assert len(g["tasks"]) == 2 + per_layer * spec.n_layers == len(g["decode_pipeline"]) == len(g["events"])
    for i, t in enumerate(g["tasks"]):
        assert TASK_KEYS <= set(t) and t["id"] == i and t["kernel"].startswith("fusekit_")
        assert t["depends_on"] == ([i - 1] if i else [])
        assert ("layer_idx" in t) == (0 < i < len(g["tasks"]) - 1)
        for b in t["inputs"] + t["outputs"]:
            assert b["role"] in ("external", "scratch") and b["role_name"]
    assert [r["region"] for r in g["layer_groups"]] == ["embed"] + [f"layer.{l}" for l in range(spec.n_layers)] + ["post"]
    assert sorted(i for r in g["layer_groups"] for i in r["task_ids"]) == g["decode_pipeline"]
    assert json.loads(json.dumps(g)) == g
    # the reference's replay order inside a layer (task_graph_json.rs:1619-1664)
    kinds = [t["kernel"][8:] for t in g["tasks"] if t.get("layer_idx") == 0]
    want = ["rmsnorm_qkv", "sdpa_decode", "linear_residual", "rmsnorm_gateup_act", "linear_residual"]
    if spec.arch != "qwen2":
        want.insert(1, "qk_norm_rope_store")
    assert kinds == want


@pytest.mark.parametrize("name,world,fused", [("qwen2.5-7b", 1, True), ("qwen2.5-7b", 2, True), ("qwen2.5-7b", 2, False),
                                               ("gemma3-4b", 1, True), ("tiny-qwen", 1, False), ("tiny-gemma", 1, True)])
def test_every_role_resolves_and_every_tensor_is_used(name, world, fused):
    spec = CONFIGS[name]
    e = _fake_engine(spec, world, world - 1, fused)
    g = json.loads(json.dumps(e.task_graph()))
    tasks = e.dispatches_from(g)
    assert len(tasks) == len(g["tasks"])
    assert set(e.W.asked) == e.W.known and set(e.V.asked) == e.V.known
    # data flow: every buffer a task reads from the residual stream was written by an earlier task
    written = set()
    for t in g["tasks"]:
        outs = {b["role_name"] for b in t["outputs"]}
        for b in t["inputs"]:
            if b["role"] == "scratch" and b["role_name"].startswith(("global_scratch.x_in", "layer_scratch")) and b["role_name"] not in outs:
                assert b["role_name"] in written, (t["id"], t["kernel"], b["role_name"])
        written |= outs
    # iargs carry this rank's slice of the shape
    head = tasks[-1] if world == 1 else tasks[-3]
    assert head.iarg[1] == spec.vocab // world and head.iarg[2] == (world - 1) * (spec.vocab // world)


def test_reader_refuses_what_it_cannot_dispatch():
    e = _fake_engine(CONFIGS["tiny-qwen"])
    g = e.task_graph()
    with pytest.raises(ValueError):
        e.dispatches_from({**g, "version": 1})
    with pytest.raises(ValueError):
        e.dispatches_from({**g, "active_m": 16})
    with pytest.raises(ValueError):
        e.dispatches_from({**g, "decode_capabilities": {"dispatchable": False, "reasons": ["unsupported kernel"]}})
    bad = json.loads(json.dumps(g))
    bad["tasks"][1]["extra_bindings"][0]["role"] = "layer_scratch.nonesuch"
    with pytest.raises(KeyError):
        e.dispatches_from(bad)


def test_fused_peer_exchange_graph_has_no_allreduce_tasks():
    """Tensor parallel with the exchange fused in: five tasks per layer as on one GPU, the row-split projections carry a
    push site, the norm-first kernels after them the matching pull site, the head pulls the last down_proj and exchanges
    the argmax keys itself."""
    spec = CONFIGS["qwen2.5-32b"]
    g = TG.emit(spec, 4352, tp_rank=3, tp_size=8, tp_exchange="peer")
    kinds = [t["kind"] for t in g["tasks"]]
    assert TG.K_ALLREDUCE not in kinds and TG.K_ARGMAX not in kinds and TG.K_RESADD not in kinds
    assert len(kinds) == 2 + 5 * spec.n_layers
    L = spec.n_layers
    lin = [t for t in g["tasks"] if t["kind"] == TG.K_LIN]
    assert [t["iargs"][3] for t in lin] == [s + 1 for s in range(2 * L)]                    # sites 0 .. 2L-1 in order
    gu = [t for t in g["tasks"] if t["kind"] == TG.K_GATEUP]
    assert [t["iargs"][4] for t in gu] == [2 * l + 1 for l in range(L)]
    qkv = [t for t in g["tasks"] if t["kind"] == TG.K_QKV]
    assert [t["iargs"][6] for t in qkv] == [0] + [2 * l + 2 for l in range(L - 1)]
    head = g["tasks"][-1]
    assert head["kind"] == TG.K_HEAD and head["iargs"][3] == 0 and head["iargs"][4:6] == [2 * L, 2 * L + 1]
    with pytest.raises(ValueError):
        TG.emit(spec, 4352, tp_rank=0, tp_size=8, fused_weights=False, tp_exchange="peer")


def _records(tasks):
    return [bytes(t) for t in tasks]


@pytest.mark.parametrize("name,world,mode,kvb", [("qwen2.5-7b", 1, "allreduce", 0), ("gemma3-4b", 1, "allreduce", 0), ("qwen2.5-32b", 8, "peer", 0),
                                                   ("qwen2.5-7b", 2, "allreduce", 0), ("tiny-qwen", 1, "allreduce", 8)])
def test_library_json_reader_matches_the_python_resolution(name, world, mode, kvb):
    """The C-ABI reader (fk_tasks_from_json) turns the document text + a role table into byte-identical fk_task records to the
    Python resolution, pretty-printed or compact."""
    spec = CONFIGS[name]
    e = _fake_engine(spec, world, world - 1, True)
    e.tp_exchange, e.kv_bits = mode, kvb
    if kvb:
        e.cacheq = [{k: 0x700000 + 64 * l + i for i, k in enumerate(["k", "k_scales", "k_biases", "v", "v_scales", "v_biases"])} for l in range(spec.n_layers)]
    g = e.task_graph()
    want = _records(e.dispatches_from(g))
    for text in (json.dumps(g, indent=2), json.dumps(g, separators=(",", ":"))):
        got = _records(e.dispatches_from_json(text))
        assert got == want


def test_library_json_reader_refusals():
    from fusekit_b200 import _native as N
    e = _fake_engine(CONFIGS["tiny-qwen"])
    g = e.task_graph()
    table = e.role_table(g)
    for bad, word in (({**g, "version": 1}, "version"), ({**g, "active_m": 16}, "active_m"),
                      ({**g, "decode_capabilities": {"dispatchable": False, "reasons": []}}, "dispatchable"),
                      ({**g, "decode_pipeline": [9999]}, "names no task")):
        with pytest.raises(N.FusekitError, match=word):
            e.dispatches_from_json(json.dumps(bad), table)
    with pytest.raises(N.FusekitError, match="not a JSON object"):
        e.dispatches_from_json('{"version": 2, "tasks": [', table)
    with pytest.raises(N.FusekitError, match="layer_scratch.q_buf"):
        e.dispatches_from_json(json.dumps(g), [(r, v) for r, v in table if r != "layer_scratch.q_buf"])
    worse = json.loads(json.dumps(g)); worse["tasks"][0]["kind"] = 99
    with pytest.raises(N.FusekitError, match="kind"):
        e.dispatches_from_json(json.dumps(worse), table)


def test_attention_fused_into_the_qkv_task():
    """fuse_attention: four tasks per Qwen-shaped layer, the QKV task carries the attention output, scratch and scale; shapes
    the tail does not cover (Gemma's per-head norms, a quantised cache) keep their attention task."""
    spec = CONFIGS["qwen2.5-7b"]
    g = TG.emit(spec, 1024, fuse_attention=True)
    kinds = [t["kind"] for t in g["tasks"]]
    assert TG.K_SDPA not in kinds and len(kinds) == 2 + 4 * spec.n_layers
    qkv = g["tasks"][1]
    assert qkv["kind"] == TG.K_QKV and qkv["iargs"][7] == 1 and abs(qkv["fargs"][2] - spec.head_dim ** -0.5) < 1e-7
    slots = TG.task_slots(qkv)
    assert slots[7] == "layer_scratch.sdpa_buf" and slots[8] == "global_scratch.attend_scratch"
    assert TG.K_SDPA in [t["kind"] for t in TG.emit(CONFIGS["gemma3-4b"], 1024, fuse_attention=True)["tasks"]]
    assert TG.K_SDPAQ in [t["kind"] for t in TG.emit(CONFIGS["tiny-qwen"], 64, kv_bits=8, fuse_attention=True)["tasks"]]
    e = _fake_engine(spec)
    e.fuse_attention, e.attend_scratch = True, 0x600000
    assert _records(e.dispatches_from_json(json.dumps(e.task_graph()))) == _records(e.build_dispatches())


def _reference_style_graph(spec, split_sdpa=True, drop=None, swap=False):
    """A document shaped like the reference's own output for a Qwen-shaped model: suffixed kernel names, no shapes, one role per
    tensor, the replay order of task_graph_json.rs:1619-1664."""
    tasks, fid = [], [0]

    def add(name, layer=None, roles=()):
        fid[0] += 1
        t = {"id": len(tasks), "fusion_id": fid[0], "kernel": name if name in ("fusekit_step_init", "fusekit_history_capture") else f"{name}_f{fid[0]}",
             "grid_threads": [64, 1, 1], "threadgroup": [64, 1, 1], "inputs": [], "outputs": [],
             "extra_bindings": [{"slot": 3 + i, "role": r} for i, r in enumerate(roles)], "depends_on": [], "trigger_event": len(tasks)}
        if layer is not None:
            t["layer_idx"] = layer
        tasks.append(t)

    add("fusekit_step_init")
    add("fusekit_embed_lookup_decode", roles=["param.embed_tokens"])
    for l in range(spec.n_layers):
        lp = f"layer_param.{l}."
        qkv = [lp + f"self_attn.{p}_proj.{s}" for p in "qkv" for s in ("weight", "scales", "biases", "bias")] + [lp + "input_layernorm.weight"]
        fams = [("fusekit_rmsnorm_qkv", qkv), ("fusekit_sdpa_decode", ["layer_cache_k", "layer_cache_v"]),
                ("fusekit_linear_residual", [lp + "self_attn.o_proj.weight", lp + "self_attn.o_proj.scales", lp + "self_attn.o_proj.biases"]),
                ("fusekit_chain", [lp + f"mlp.{p}_proj.{s}" for p in ("gate", "up") for s in ("weight", "scales", "biases")] + [lp + "post_attention_layernorm.weight"]),
                ("fusekit_linear_residual", [lp + f"mlp.down_proj.{s}" for s in ("weight", "scales", "biases")])]
        if swap and l == 1:
            fams[2], fams[3] = fams[3], fams[2]
        for name, roles in fams:
            if drop and l == 0:
                roles = [r for r in roles if drop not in r]
            add(name, l, roles)
            if name == "fusekit_sdpa_decode" and split_sdpa:            # the runtime's partial / combine split
                tasks[-1]["kernel"] += "_partial"
                add(name, l, []); tasks[-1]["kernel"] += "_combine"
    add("fusekit_final_rmsnorm_lm_head", roles=["param.final_norm", "param.lm_head"])
    add("fusekit_argmax_logits_scan"); add("fusekit_argmax_logits_finalize")
    return {"version": 2, "active_m": 1, "tasks": tasks, "events": [], "scratch_buffers": [], "initial_tasks": [0], "model_params": [],
            "layer_groups": [], "decode_pipeline": list(range(len(tasks))), "decode_capabilities": {"dispatchable": True, "reasons": []}}


def test_lowering_of_a_reference_written_graph():
    """The reference's own dialect (suffixed Metal kernel names, no shapes) lowers to this build's graph once the model shape is
    known; a wrong family order, a missing projection or an unknown kernel are refused."""
    spec = CONFIGS["tiny-qwen"]
    for split in (True, False):
        g, src = TG.lower_reference(_reference_style_graph(spec, split), spec, 256)
        assert g == TG.emit(spec, 256)
        assert src["layer_param.1.self_attn.qkv_proj"] == [f"layer_param.1.self_attn.{p}_proj" for p in "qkv"]
        assert src["layer_param.0.mlp.gate_up_proj"] == ["layer_param.0.mlp.gate_proj", "layer_param.0.mlp.up_proj"]
        roles = {b["role"] for t in g["tasks"] for b in t["extra_bindings"] if b["role"].startswith(("param.", "layer_param."))}
        assert roles <= set(src)               # every parameter role of the lowered graph has its sources named
    assert TG.reference_family("fusekit_chain_f1234") == "chain" and TG.reference_family("fusekit_sdpa_decode_f7_combine") == "sdpa_decode"
    with pytest.raises(ValueError, match="kernel order"):
        TG.lower_reference(_reference_style_graph(spec, swap=True), spec, 256)
    with pytest.raises(ValueError, match="v_proj"):
        TG.lower_reference(_reference_style_graph(spec, drop="v_proj"), spec, 256)
    bad = _reference_style_graph(spec); bad["tasks"][3]["kernel"] = "fusekit_moe_router_f9"
    with pytest.raises(ValueError, match="no lowering"):
        TG.lower_reference(bad, spec, 256)
    with pytest.raises(ValueError, match="layers"):
        TG.lower_reference(_reference_style_graph(spec), CONFIGS["qwen2.5-0.5b"], 256)


def test_library_json_reader_tolerates_formatting_and_rejects_garbage():
    """Whitespace, escapes in strings, unknown extra keys, exponents in numbers: accepted.  Truncated text, wrong value types, deep
    nesting: refused with FK_ERR_VALUE, never a crash."""
    import ctypes as C
    from fusekit_b200 import _native as N
    e = _fake_engine(CONFIGS["tiny-qwen"])
    g = e.task_graph()
    table = e.role_table(g)
    want = _records(e.dispatches_from(g))
    noisy = json.loads(json.dumps(g))
    noisy['comment "quoted" \n'] = {"nested": [1, 2.5e0, -3, True, None, "\u00e9\t"]}
    noisy["tasks"][0]["fargs"] = [float(x) for x in noisy["tasks"][0]["fargs"]]
    text = json.dumps(noisy, indent=1).replace("\n", "\r\n\t ")
    assert _records(e.dispatches_from_json(text, table)) == want
    L = N.lib()
    arr = (N.RoleBinding * len(table))(*[N.RoleBinding(r.encode(), int(v)) for r, v in table])
    n = C.c_int32()
    full = json.dumps(g)
    for bad in (full[: len(full) // 2], "[]", "null", "{" * 200 + "}" * 200, full.replace('"decode_pipeline": [', '"decode_pipeline": {', 1),
                full.replace('"version": 2', '"version": "2"', 1), ""):
        st = L.fk_tasks_from_json(bad.encode(), arr, len(table), None, 0, C.byref(n))
        assert st == -1, (st, bad[:40])
    assert L.fk_tasks_from_json(None, arr, len(table), None, 0, C.byref(n)) == -1
    # a too small output array is refused, the count is still reported
    out = (N.Task * 1)()
    assert L.fk_tasks_from_json(full.encode(), arr, len(table), out, 1, C.byref(n)) == -1 and n.value == len(g["tasks"])
