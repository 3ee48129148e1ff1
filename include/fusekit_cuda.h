/*
 * fusekit_cuda.h -- C ABI of the B200 decode runtime (libfusekit_cuda.so).
 *
 * This is the boundary a FuseKit host binds in place of its Metal dispatcher
 * module `_fusekit_runtime_native` (python_runtime/src/lib.rs:1939-1971 in the
 * FuseKit tree).  Every entry point names the reference function it replaces.
 * The library owns device memory, the bf16 KV cache, the per-token kernel list
 * and its CUDA-graph replay; there is no CPU fallback and no PyTorch type in
 * any signature.  All calls return 0 on success or a negative fk_status; the
 * text of the last failure on the calling thread is in fk_last_error().
 * A handle is used from one host thread at a time (the reference serialises
 * every call behind one mutex, lib.rs:112).
 */
#ifndef FUSEKIT_CUDA_H
#define FUSEKIT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t fk_status;
enum {
    FK_OK = 0,
    FK_ERR_VALUE = -1,    /* bad handle / argument / range (reference: PyValueError, lib.rs:1977-1985) */
    FK_ERR_CUDA = -2,     /* a CUDA runtime call failed */
    FK_ERR_STATE = -3,    /* call made in the wrong order */
    FK_ERR_NCCL = -4,     /* collective backend failure */
    FK_ERR_DEVICE = -5    /* a kernel reported an error status word */
};

typedef uint64_t fk_handle;   /* index into a process-global table that only grows (lib.rs:112, 152-168) */
typedef uint64_t fk_graph;    /* captured per-token kernel list (reference: ICB id, lib.rs:559-569) */
typedef uint64_t fk_weight;   /* a linear layer's weights in the library's HBM layout */
typedef uint64_t fk_dptr;     /* raw device address returned by fk_alloc */

/* ---- task kinds: one per fused decode task of the reference task graph --- */
enum {
    FK_TASK_STEP_INIT = 0,             /* fusekit_step_init, src/codegen/kernels/mod.rs:542-579 */
    FK_TASK_EMBED_LOOKUP_DECODE = 1,   /* kernels/embed_lookup_decode.rs:17-104 */
    FK_TASK_RMSNORM_QKV = 2,           /* kernels/rmsnorm_qkv.rs:53-736 (with QkvDecodeSinks: RoPE + KV store) */
    FK_TASK_QK_NORM_ROPE_STORE = 3,    /* single.rs:4222-4311 + 4335-4485 + kv_cache_store_decode.rs (Gemma-shaped) */
    FK_TASK_SDPA_DECODE = 4,           /* kernels/sdpa_decode.rs:697-715, 992-1046 (partial + combine) */
    FK_TASK_LINEAR_RESIDUAL = 5,       /* kernels/linear_residual.rs:17-388; residual optional (QmvFanout single target) */
    FK_TASK_RMSNORM_GATEUP_ACT = 6,    /* fused_chain.rs:2902-3552 / qmv_swiglu.rs (SwiGLU or GeGLU-tanh tail) */
    FK_TASK_FINAL_RMSNORM_LM_HEAD = 7, /* final_rmsnorm_lm_head.rs:144-360 + direct argmax msl.rs:1674-1890 */
    FK_TASK_ARGMAX_FINALIZE = 8,       /* argmax_logits_finalize.rs:16-115 (+ history capture) */
    FK_TASK_ALLREDUCE = 9,             /* no reference counterpart: tensor-parallel sum over ranks */
    FK_TASK_RESIDUAL_ADD = 10,         /* no reference counterpart: y = T(sum + residual) after FK_TASK_ALLREDUCE */
    FK_TASK_RMSNORM_ROWS = 11,         /* batch of sequences: RMSNorm of every row (kernels/mod.rs:4464-4472 arithmetic; the reference
                                          never batches independent sequences, python/fusekit_runtime/dispatch.py:2268-2289) */
    FK_TASK_ROPE_STORE_ROWS = 12,      /* batch: RoPE on q / k and the cache store of every sequence (rmsnorm_qkv.rs:635-697) */
    FK_TASK_ARGMAX_ROWS = 13,          /* batch: greedy token of every sequence + position advance (argmax_logits_scan.rs:83-124) */
    FK_TASK_KV_STORE_QUANT = 14,       /* kernels/rope_kv_cache_store_decode_quant.rs (fused form rmsnorm_qkv.rs:435-612): RoPE + quantised KV store */
    FK_TASK_SDPA_DECODE_QUANT = 15,    /* kernels/sdpa_decode_quant.rs:301-680: attention over the quantised cache */
    FK_TASK_KIND_COUNT = 16
};

/* activation selector for FK_TASK_RMSNORM_GATEUP_ACT */
enum { FK_ACT_SWIGLU = 0, FK_ACT_GEGLU_TANH = 1 };

/*
 * One entry of the per-token dispatch list (reference: the (kernel, buffers,
 * grid, threadgroup) tuples that dispatch.py:3163-3611 builds and build_icb
 * encodes).  `buf` holds device addresses from fk_alloc / fk_kv_cache_alloc or
 * fk_weight ids; unused slots are 0.  Slot meaning per kind:
 *
 * EMBED_LOOKUP_DECODE  buf0 table T[V,H]  buf1 x_out T[rows,H]            i0 H  i1 rows  i2 V (rows of the table; 0 = unchecked)   f0 scale
 *                      with V given, fk_state_set / fk_decode_chunk refuse a seed token >= V and an id >= V arriving on the
 *                      device reads row 0 and sets error bit 0x20000.  i3 = 4 or 8: a quantised table -- buf0 packed u32
 *                      [V, H*bits/32], buf2 scales T[V, H/64], buf3 biases T[V, H/64], x = T((q*s + b) * scale)
 *                      (embed_lookup_decode.rs:79-93); i3 = 0 or 16: buf0 is the T[V,H] table
 * RMSNORM_QKV          buf0 x T[H]  buf1 norm_w  buf2 weight(qkv rows: q|k|v)  buf3 lin_bias|0
 *                      buf4 q_out  buf5 cache_k  buf6 cache_v  buf7 k_out|0  buf8 v_out|0
 *                      buf9 pending_y|0  buf10 pending_norm_w  buf11 h_out   (Gemma: x <- T(x + rmsnorm(pending_y)));
 *                      with buf10 = 0, buf9 is an fp32 all-reduced projection: x <- T(buf9 + x) (tensor parallel)
 *                      i0 H  i1 n_q  i2 n_kv  i3 head_dim  i4 capacity  i5 sinks(1 = RoPE + cache store)
 *                      i6 pull site + 1 (0 = none): x <- T(sum over ranks of the partial rows pushed to that exchange site + x),
 *                      written to buf11 (tensor parallel with the exchange fused in, see LINEAR_RESIDUAL i3)
 *                      i7 = 1: decode attention over the cache as the kernel's tail (streaming layout, sinks, head_dim 64 / 128,
 *                      <= 8 q heads per kv head; replaces the SDPA_DECODE task that would follow, sdpa_decode.rs:697-715, 992-1046):
 *                      buf7 = attention output T[n_q * head_dim], buf8 = scratch, 16-byte aligned, zero before first use:
 *                      64 bytes of hand-off counters + 512 * 8 * (head_dim + 2) floats of partials;  f2 = attention scale
 *                      f0 eps  f1 rope_theta
 * QK_NORM_ROPE_STORE   buf0 q(in/out)  buf1 k_in  buf2 v_in  buf3 q_norm_w  buf4 k_norm_w  buf5 cache_k  buf6 cache_v
 *                      i0 n_q  i1 n_kv  i2 head_dim  i3 capacity   f0 eps  f1 rope_theta
 * SDPA_DECODE          buf0 q  buf1 cache_k  buf2 cache_v  buf3 out  buf4 partials(f32)  buf5 counter(u32)
 *                      i5 sequences M (0 / 1: one)
 *                      i0 n_q  i1 n_kv  i2 head_dim  i3 capacity  i4 kernel choice (0 = by shape and capacity, 1 = cluster,
 *                      2 = global partials + ticket, 4 = tensor-core cluster)   f0 scale
 *                      partials: n_q * ceil(capacity / 32) * (head_dim + 2) floats; counter: n_kv words, zero before first use
 * LINEAR_RESIDUAL      buf0 x T[K]  buf1 weight  buf2 residual|0  buf3 y_out T[N]  buf4 y_f32_out|0   i0 K  i1 N
 *                      buf5 (optional, one row): x as staged digits, written by RMSNORM_GATEUP_ACT buf5 (then buf0 is not read)
 *                      i2 activation rows M (0 or 1: one row).  M = 2..16: x is T[M, K], residual and y_out are T[M, N], row m
 *                      is the result the one-row task gives for x[m] (reference: the fusekit_qmm tiles for M > 1,
 *                      src/codegen/msl.rs:2318-2439, chosen in kernels/mod.rs:1442-1473); streamed 4-bit weights only
 *                      i3 push site + 1 (0 = none; no reference counterpart): a row-split projection of a tensor-parallel layer
 *                      stores its fp32 partial rows into every rank's peer arena (fk_peer_arena_open) and the last block
 *                      publishes a flag; buf3 / buf4 may then be 0.  The norm-first task that follows names the same site as
 *                      its pull site, waits (bounded) for all ranks and sums in rank order.  Sites are numbered from 0 in task
 *                      order, at most 160, each written once per token
 *                      i5 kernel of the M > 1 form: 0 = default, 1 = tcgen05 (M <= 32), 2 = mma.sync (M <= 16)
 * RMSNORM_GATEUP_ACT   buf0 x  buf1 norm_w  buf2 weight(gate)  buf3 weight(up)  buf4 act_out T[I]
 *                      buf9..11 pending (as RMSNORM_QKV)     i0 H  i1 I  i2 act   f0 eps
 *                      i3 activation rows M (0 or 1: one row).  M = 2..16: x is T[M, H], act_out is T[M, I], every row normalised
 *                      by its own RMS (buf1 = 0: the rows are normalised already, e.g. by RMSNORM_ROWS, and only the product and
 *                      the activation run); paired 4-bit weights, no pending inputs (reference: fusekit_qmm_t_swiglu_pair_impl, msl.rs:2489)
 *                      i4 pull site + 1 (as RMSNORM_QKV i6)
 *                      buf5 (optional, one row, 4/8-bit): the activation vector once more as the integer digits the next
 *                      projection of the same bit width stages -- 3 bytes per activation, then (16-byte aligned) 8 bytes per
 *                      group of 64 (4-bit) / 32 (8-bit) -- for LINEAR_RESIDUAL buf5; needs whole tiles per warp (fk_weight_plan:
 *                      lsplit 0) and I a multiple of 64.  No counterpart in the reference (its kernels read T activations).
 * FINAL_RMSNORM_LM_HEAD buf0 x  buf1 norm_w  buf2 weight(head)  buf3 logits_out|0  buf4 argmax scratch(u64)
 *                      buf5 counter(u32)  buf9..11 pending     i0 H  i1 V(local)  i2 vocab_offset  i3 finalize(1/0)   f0 eps
 *                      i4 pull site + 1 (as RMSNORM_QKV i6); i5 argmax site + 1: a vocabulary-sharded head pushes its best key
 *                      to every rank, takes the maximum over the ranks and advances the decode state itself
 * ARGMAX_FINALIZE      buf4 argmax scratch  i0 entries
 * ALLREDUCE            buf0 f32 buffer   i0 count
 * RESIDUAL_ADD         buf0 sum f32[N]  buf1 residual T[N]  buf2 y_out T[N]   i0 N
 * RMSNORM_ROWS         buf0 x T[M,H]  buf1 norm_w T[H]  buf2 y_out T[M,H]   i0 H  i1 M   f0 eps
 * ROPE_STORE_ROWS      buf0 qkv T[M,(n_q+2n_kv)*hd] (bias added)  buf1 q_out T[M,n_q*hd]  buf5 cache_k  buf6 cache_v
 *                      (caches [M, n_kv, capacity, hd])   i0 n_q  i1 n_kv  i2 head_dim  i3 capacity  i4 M   f1 rope_theta
 * ARGMAX_ROWS          buf0 logits T[M,V]  buf5 counter(u32, zero before first use)   i0 V  i1 M
 *                      token[m] of the decode state and history[step * M + m] receive sequence m's token
 * KV_STORE_QUANT       buf0 q T[n_q*hd] (raw projection in, rotated out)  buf1 k_in T[n_kv*hd]  buf2 v_in T[n_kv*hd]  (RMSNORM_QKV
 *                      without sinks)  buf3 cache_k packed u32 [n_kv, capacity, hd*bits/32]  buf4 cache_v packed  buf5 k scales
 *                      buf6 k biases  buf7 v scales  buf8 v biases (T[n_kv, capacity, hd/64])
 *                      i0 n_q  i1 n_kv  i2 head_dim  i3 capacity  i4 bits (4 / 8)   f1 rope_theta
 * SDPA_DECODE_QUANT    buf0 q  buf1 cache_k packed  buf2 cache_v packed  buf3 out  buf4 partials(f32)  buf5 counter(u32)
 *                      buf6 k scales  buf7 k biases  buf8 v scales  buf9 v biases   i0 n_q  i1 n_kv  i2 head_dim  i3 capacity
 *                      i4 bits   f0 scale      (partials and counter as SDPA_DECODE)
 *                      ROPE_STORE_ROWS i5 = 1, SDPA_DECODE i6 = 1: the M rows are consecutive positions offset .. offset + M - 1 of
 *                      ONE sequence (a prefill chunk, or verify rows of speculative decoding; reference: the M > 1 trace
 *                      shapes, python/fusekit_runtime/__init__.py:2825-2850, src/commands/patch.rs:112-152) sharing one cache
 *                      [n_kv, capacity, hd]; row m attends keys 0 .. offset + m.  ARGMAX_ROWS i2: positions the step advances
 *                      by (default 1; M for such a chunk)
 * Batch decode (M = 2..16 independent sequences at one position): EMBED with i1 = M, LINEAR_RESIDUAL / RMSNORM_GATEUP_ACT
 * with their row counts, SDPA_DECODE with i5 = M (q and out T[M, n_q*hd], caches [M, n_kv, capacity, hd]).
 */
typedef struct fk_task {
    int32_t  kind;
    int32_t  layer;
    uint64_t buf[12];
    int32_t  iarg[8];
    float    farg[4];
} fk_task;

/* ---- lifetime and introspection ------------------------------------------ */
/* replaces load_dispatcher (lib.rs:115-169): binds a device, creates the stream and decode state */
fk_status fk_open(int device, fk_handle *out);
fk_status fk_close(fk_handle h);
/* replaces version / dispatcher_info / kernel_names (lib.rs:1879, 193, 222); JSON text into `buf` */
const char *fk_version(void);
fk_status fk_info(fk_handle h, char *buf, size_t cap);
fk_status fk_kernel_names(char *buf, size_t cap);
const char *fk_last_error(void);

/* ---- device memory (reference: alloc_uniform lib.rs:1657, register_host_buffer lib.rs:1681; the
 *      reference wraps unified host memory zero-copy, a discrete GPU needs explicit copies) ------ */
fk_status fk_alloc(fk_handle h, size_t nbytes, fk_dptr *out);
fk_status fk_free(fk_handle h, fk_dptr p);
fk_status fk_upload(fk_handle h, fk_dptr dst, const void *src, size_t nbytes);
fk_status fk_download(fk_handle h, void *dst, fk_dptr src, size_t nbytes);
fk_status fk_memset(fk_handle h, fk_dptr dst, int byte, size_t nbytes);
fk_status fk_sync(fk_handle h);
/* bf16 KV cache of one layer, layout [n_kv, capacity, head_dim] (sdpa_decode.rs:300-304), zero-filled */
fk_status fk_kv_cache_alloc(fk_handle h, int n_kv, int capacity, int head_dim, fk_dptr *k_out, fk_dptr *v_out);

/* ---- weights --------------------------------------------------------------
 * MLX-affine layout at the boundary (src/fusion/ir.rs:236-247): packed u32 [N, K*bits/32] LSB-first,
 * scales/biases bf16 [N, K/64]; bits 16 = dense bf16 [N,K].  Rows may be filled from several host
 * tensors (q|k|v concatenation).  fk_weight_finalize freezes the object before first use. */
fk_status fk_weight_alloc(fk_handle h, int64_t n, int64_t k, int bits, fk_weight *out);
fk_status fk_weight_upload_rows(fk_handle h, fk_weight w, int64_t dst_row0, int64_t nrows,
                                const void *packed_or_dense, const void *scales, const void *biases);
/* synthetic rows generated on the device, bit-identical to the documented counter-based generator:
 * value(row, col) = std * z(stream, (src_row0 + r) * k_global + k0 + c), quantised per group of 64 */
fk_status fk_weight_synth_rows(fk_handle h, fk_weight w, int64_t dst_row0, int64_t nrows, uint64_t stream,
                               float std, int64_t k_global, int64_t src_row0, int64_t k0);
/* Row order inside the library's 16-row tiles, chosen before fk_weight_finalize: 0 = plain, 1 = RoPE pairs
 * (the first n_rot_rows rows are heads of head_dim; dims d and d + head_dim/2 of a head share a lane so the
 * fused QKV kernel rotates them in registers -- required for RMSNORM_QKV with sinks). */
fk_status fk_weight_set_rows(fk_handle h, fk_weight w, int kind, int head_dim, int n_rot_rows);
/* Freezes the object; 4- and 8-bit rows are repacked into the streaming layout (16 rows x 8 groups per
 * 4608-byte unit, lane-ordered) and the MLX-layout copy is released. */
fk_status fk_weight_finalize(fk_handle h, fk_weight w);
/* Interleaves a gate and an up projection (same shape, not yet finalized) into one weight whose tiles hold
 * 8 gate rows and the 8 matching up rows; consumes both inputs.  RMSNORM_GATEUP_ACT takes it in buf2 (buf3 0). */
fk_status fk_weight_pair(fk_handle h, fk_weight gate, fk_weight up, fk_weight *out);
/* dequantised fp32 [nrows, K] of rows [row0, row0+nrows) -- the bit-exactness probe */
fk_status fk_weight_dequant(fk_handle h, fk_weight w, int64_t row0, int64_t nrows, float *host_out);
fk_status fk_weight_nbytes(fk_handle h, fk_weight w, uint64_t *out);
/* out[i] = bf16(mean + std * z(stream, idx0 + i)) written at a device address */
fk_status fk_synth_normal_bf16(fk_handle h, fk_dptr dst, uint64_t stream, uint64_t idx0, uint64_t n, float mean, float std);

/* ---- eager launches (reference: dispatch_kernel lib.rs:397, dispatch_batch lib.rs:1722,
 *      smoke_dispatch lib.rs:238 = elementwise_add_bf16 over n values) ------------------------- */
fk_status fk_launch(fk_handle h, const fk_task *task);
fk_status fk_launch_batch(fk_handle h, const fk_task *tasks, int n);
fk_status fk_smoke(fk_handle h, const uint16_t *a, const uint16_t *b, uint16_t *out, int n);

/* ---- decode state (reference: the token/offset/kv_len uniforms that step_decode pokes,
 *      lib.rs:884-1012, and the device-side counters of fusekit_step_init) -------------------- */
fk_status fk_state_set(fk_handle h, uint32_t token, uint32_t offset);
fk_status fk_state_get(fk_handle h, uint32_t *token, uint32_t *offset, uint32_t *error_word);

/* ---- per-token graph (reference: build_icb lib.rs:459-570, execute_icb lib.rs:718-760,
 *      submit_icb_async / wait_pending_icb lib.rs:659-715, profile_icb_commands lib.rs:821-869) - */
fk_status fk_graph_capture(fk_handle h, const fk_task *tasks, int n, fk_graph *out);
/* The file-level boundary: a v2 task_graph.json (src/codegen/task_graph_json.rs:33-226; reader src/runtime/plan.rs:39-164 and
 * load_dispatcher, python_runtime/src/lib.rs:115-169) parsed inside the library.  The caller supplies the table that maps
 * every role string of the document (slot_role_key, src/codegen/kernels/mod.rs:5531-5576: param.*, layer_param.<i>.*,
 * layer_cache_k.<i>, layer_scratch.*, global_scratch.*) to a device address or fk_weight id; tasks come out in
 * decode_pipeline order.  fk_tasks_from_json with tasks_out = NULL only counts; it needs no device. */
typedef struct fk_role_binding { const char *role; uint64_t value; } fk_role_binding;
fk_status fk_tasks_from_json(const char *json_text, const fk_role_binding *roles, int n_roles, fk_task *tasks_out, int cap, int *n_out);
fk_status fk_graph_capture_json(fk_handle h, const char *json_text, const fk_role_binding *roles, int n_roles, fk_graph *out);
fk_status fk_graph_launch(fk_handle h, fk_graph g, double *gpu_seconds);
fk_status fk_graph_launch_async(fk_handle h, fk_graph g);
fk_status fk_wait(fk_handle h, double *gpu_seconds);
fk_status fk_graph_profile_nodes(fk_handle h, fk_graph g, int repeats, double *seconds_out, int cap, int *n_out);
fk_status fk_graph_node_count(fk_handle h, fk_graph g, int *n_out);
/* CUDA-event time of `n` tasks launched back to back, averaged over `repeats` passes after one warm-up pass
 * (reference: execute_icb_range returns the GPU seconds of a command range, lib.rs:769) */
fk_status fk_time_tasks(fk_handle h, const fk_task *tasks, int n, int repeats, double *seconds_per_pass);

/* one token: write token/offset, replay, read the argmax back (step_decode, lib.rs:884-1012) */
fk_status fk_step(fk_handle h, fk_graph g, uint32_t token, uint32_t offset, uint32_t *next_token, double *gpu_seconds);
/* `count` tokens pre-submitted, token feedback on the device, one wait; out_history[count] on the host
 * (decode_chunk_gpu_chain, lib.rs:1275-1420) */
fk_status fk_decode_chunk(fk_handle h, fk_graph g, uint32_t base_offset, uint32_t seed_token, int count,
                          uint32_t *out_history, double *gpu_seconds);
/* `rows` independent sequences decoded together (a graph of the batch tasks): sequence m starts from seed_tokens[m], all at
 * base_offset; out_history[step * rows + m].  No reference counterpart (its M > 1 means positions of one sequence). */
fk_status fk_decode_chunk_rows(fk_handle h, fk_graph g, uint32_t base_offset, const uint32_t *seed_tokens, int rows, int count,
                               uint32_t *out_history, double *gpu_seconds);
/* same result with a host round trip per token (decode_chunk_host_loop, lib.rs:1129-1257) */
fk_status fk_decode_chunk_host(fk_handle h, fk_graph g, uint32_t base_offset, uint32_t seed_token, int count,
                               uint32_t *out_history, double *gpu_seconds);

/*
 * Split-K GQA decode attention that allocates nothing.  It has no counterpart in the reference: it exists for
 * hosts that must not touch the device allocator on their decode path -- a runtime that pre-sizes all device
 * memory at start-up and forbids later cudaMalloc calls (they synchronise the device and can fail under memory
 * pressure), or a host that only holds buffers handed to it by another framework.  q [n_q*head_dim], cache_k /
 * cache_v [n_kv, capacity, head_dim] and out [n_q*head_dim] are bf16 device buffers of the caller; `pos` is the
 * position being decoded (keys 0..min(pos+1, capacity)-1 are attended; pos > 2^31 - 1 is refused); `stream` is a cudaStream_t (0 = default)
 * and the call returns once the work is queued.  The split-K partial sums live in a fixed 4 MiB array inside the
 * library image, so the shape is limited to  n_q * ceil(capacity/32) * (head_dim+2) <= 1048576 floats  and at most
 * 64 kv heads; larger shapes are refused with FK_ERR_VALUE.  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress); make that call before any stream capture.  All calls on a device share the array:
 * two calls whose kernels overlap on the GPU (different streams) race; calls queued on one stream are safe.
 */
fk_status fk_sdpa_decode_noalloc(const void *q, const void *cache_k, const void *cache_v, void *out,
                                 int n_q, int n_kv, int head_dim, int capacity, uint32_t pos, float scale, void *stream);

/* tuning aid (no reference counterpart): while `buf` is non-zero the streamed kernels write per-block phase
 * timestamps ([grid][8] u64 nanoseconds: start, dependency met, activations staged, rows done) into it; a graph
 * captured while it is set gives task j the slice starting at entry j * 4096 (reference: profile_icb_commands,
 * lib.rs:821-869, times each command; this shows where inside a command the time goes).
 * `python -m fusekit_b200.timeline` prints it. */
fk_status fk_debug_timeline(fk_handle h, fk_dptr buf);

/* ---- peer-memory all-reduce for tensor parallelism (no reference counterpart).  Every rank exports a small arena as a
 *      64-byte CUDA IPC handle, the host gathers the handles (any transport) and every rank opens them in rank order;
 *      from then on FK_TASK_ALLREDUCE payloads of up to 32 KB are exchanged by peer stores and flags inside one small
 *      kernel (bit-identical on all ranks) instead of the library collective, which stays the fallback. ------------- */
fk_status fk_peer_arena_export(fk_handle h, void *handle64, size_t cap);
fk_status fk_peer_arena_open(fk_handle h, const void *handles /* world x 64 bytes */, int rank, int world);
/* unmaps the peers' arenas; all-reduce tasks launched afterwards use the library collective again (graphs captured
 * before keep the kernels they were captured with and must not be replayed) */
fk_status fk_peer_arena_close(fk_handle h);
/* diagnostic (no reference counterpart): the same exchange with all `world` arenas on this one GPU and the given number
 * of polls per wait; the other ranks never write, so an all-reduce task gives up after spin_limit polls and sets error
 * bit 0x8000 in the device state (fk_decode_chunk then returns FK_ERR_DEVICE; fk_state_set clears the word) */
fk_status fk_peer_arena_loopback(fk_handle h, int rank, int world, uint32_t spin_limit);

/* ---- tensor parallelism (no reference counterpart; NCCL over NVLink) ------ */
fk_status fk_comm_unique_id(void *id128, size_t cap);          /* rank 0 makes the 128-byte id */
fk_status fk_comm_init(fk_handle h, const void *id128, int rank, int world);
/* Poll the communicator for an asynchronous error (ncclCommGetAsyncError); on one the communicator is aborted and
 * FK_ERR_NCCL returned, afterwards FK_ERR_STATE.  fk_wait / fk_decode_chunk[_rows] poll the same way while they wait, so a
 * rank whose peer died returns instead of blocking; FK_COMM_TIMEOUT_MS (environment, off by default) bounds the wait with a
 * collective in flight.  No counterpart in the reference (single device). */
fk_status fk_comm_check(fk_handle h);
/* The launch shape the runtime uses for a finalized weight in the streaming layout: blocks, warps per block, and log2 of the
 * warps that share a row tile (0: a warp owns whole tiles).  Reference analogue: kernel_grid_threads / kernel_threadgroup
 * (src/codegen/kernels/mod.rs:5648-5700, 6218-7567), which the host also queries before building its dispatch list. */
fk_status fk_weight_plan(fk_handle h, fk_weight w, int *grid, int *warps, int *lsplit);

#ifdef __cplusplus
}
#endif
#endif /* FUSEKIT_CUDA_H */
