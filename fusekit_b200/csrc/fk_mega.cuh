// Persistent decode kernel: one cooperative launch runs the whole task list of a token.
//
// The reference replays its fused task graph as one dispatch per task, ordered by events with trigger counts
// (src/codegen/task_graph_json.rs:33-226; python/fusekit_runtime/dispatch.py:3163-3611).  At batch 1 on this GPU a
// task moves a few megabytes, so the time between two tasks (launch, ramp-up, drain) is as long as the task.  Here the
// tasks of a token become records that one resident grid (one block of 16 warps per SM) walks in order:
//   * every warp's weight ring runs on across task boundaries -- when a warp has issued its last unit of task i it
//     goes on to its first units of the next streamed task, so HBM keeps streaming through the barrier and the
//     activation staging of the next task;
//   * a task boundary is a grid barrier (one atomic arrive per block on a monotone counter + a bounded acquire
//     spin), the device-side form of the reference's event with `num_triggers` = number of blocks;
//   * attention splits the keys of a kv head over up to FK_MEGA_PARTS blocks that write (m, l, o) partials; the last
//     of them to arrive (a ticket, no waiting) folds the partials (sdpa_decode.rs:992-1046);
//   * a task runs its code once per token and layer, so code size is time: one call site per staging routine, one
//     instance of the streaming loop with the epilogue chosen inside, rolled loops in attention.
// Co-residency of the grid is guaranteed by the cooperative launch attribute; every wait is bounded and a block
// that gives up sets FkState.error, drains its own copies in flight and leaves.
#pragma once
#include "fk_kernels.cuh"
#include "fk_stream.cuh"

#define FK_MEGA_WARPS 16
#define FK_MEGA_PARTS 16            // blocks that may share one kv head's keys
#define FK_MEGA_KEYBLOCK 64         // keys per block are a multiple of this (one pass of the attention tiles)
#define FK_MEGA_SPIN_LIMIT (1u << 22)

struct MegaSync { unsigned int count, seq, pad[30]; };
struct MegaWeight { const uint4 *units; int ntiles, nsb; };     // what a producer needs of a streamed task

struct alignas(16) MegaOp {
    int kind, widx;             // FK_TASK_* kind; index into the weight table or -1
    int pad0, pad1;
    union { EmbedArgs emb; SQkvArgs qkv; SdpaArgs sdpa; SLinArgs lin; SGateUpArgs gu; SHeadArgs head; } u;
};
#define FK_MEGA_OP_BYTES 288
union alignas(16) MegaSlot { MegaOp op; unsigned char raw[FK_MEGA_OP_BYTES]; };      // records sit at a fixed stride
static_assert(sizeof(MegaSlot) == FK_MEGA_OP_BYTES, "MegaOp grew past its slot");

// shared memory: [op slots 2 x 288][flags 64][bars 512][zero 256][red 192][warp stream state 1024][weight table][xsi][fold][activations | attention scratch][ring]
struct MegaLayout { size_t wtab, xsi, fold, act, ring, total; };
__host__ __device__ inline MegaLayout mega_layout(int nweights, int max_nsb, int bits, size_t attn_bytes) {
    MegaLayout L;
    size_t b = 2 * FK_MEGA_OP_BYTES + 64 + 512 + 256 + 192 + 1024;
    L.wtab = b; b += (size_t)nweights * sizeof(MegaWeight);
    b = (b + 15) & ~(size_t)15;
    L.xsi = b; b += (size_t)stream_groups(max_nsb) * 8;
    L.fold = b; b += 2 * FK_CHUNK_TILES * FK_STREAM_MAXWARPS * 16 * 4;
    b = (b + 15) & ~(size_t)15;
    size_t act = (size_t)stream_groups(max_nsb) * xs_group_bytes(bits);
    if (attn_bytes > act) act = attn_bytes;
    L.act = b; b += act;
    b = (b + 127) & ~(size_t)127;
    L.ring = b; b += (size_t)FK_MEGA_WARPS * FK_STAGES * FK_UNIT_BYTES;
    L.total = b + 128;
    return L;
}

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void red_release_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Producer that walks the weight table: the ring of a warp is one continuous stream over all streamed tasks.
struct MegaStream {
    uint64_t *bars; uint4 *ring; Cursor prod; int consumed, issued, widx, nweights; const MegaWeight *wtab;
    __device__ __forceinline__ void seek() {       // move on to the next task that has units for this warp
        while (!prod.valid() && widx + 1 < nweights) {
            ++widx;
            prod.init(wtab[widx].ntiles, wtab[widx].nsb, blockIdx.x, gridDim.x, threadIdx.x >> 5, blockDim.x >> 5);
        }
    }
    __device__ __forceinline__ bool valid() const { return prod.valid(); }
    __device__ __forceinline__ void issue(int stage) {
        if ((threadIdx.x & 31) == 0) {
            mbar_expect_tx(bars + stage, FK_UNIT_BYTES);
            bulk_g2s(ring + (size_t)stage * FK_UNIT_VEC, wtab[widx].units + prod.unit_index() * FK_UNIT_VEC, FK_UNIT_BYTES, bars + stage);
        }
        ++issued;
        prod.advance();
        seek();
    }
    __device__ __forceinline__ void drained() {}
    __device__ __forceinline__ unsigned long long *tl() const { return nullptr; }
    // between tasks the state sits in shared memory (one record per warp), so it holds no registers during attention and staging
    __device__ __forceinline__ void save(int *w) const {
        if ((threadIdx.x & 31) == 0) { w[0] = consumed; w[1] = issued; w[2] = widx; w[3] = prod.chunk; w[4] = prod.tq; w[5] = prod.sbv; w[6] = prod.left; w[7] = prod.ntl; w[8] = prod.nsb; w[9] = prod.nb; }
        __syncwarp();
    }
    __device__ __forceinline__ void load(const int *w, uint64_t *bars_, uint4 *ring_, const MegaWeight *wtab_, int nweights_) {
        bars = bars_; ring = ring_; wtab = wtab_; nweights = nweights_;
        consumed = w[0]; issued = w[1]; widx = w[2]; prod.chunk = w[3]; prod.tq = w[4]; prod.sbv = w[5]; prod.left = w[6]; prod.ntl = w[7]; prod.nsb = w[8]; prod.nb = w[9];
        prod.nwarps = blockDim.x >> 5; prod.wid = threadIdx.x >> 5; prod.block = blockIdx.x; prod.grid = gridDim.x;
        prod.lw = 31 - __clz(prod.nwarps); prod.inv_nsb = __frcp_rn((float)prod.nsb);
    }
    // bounded wait for the copies still in flight (a block that leaves early must not exit under its own TMA writes)
    __device__ __forceinline__ void drain() {
        while (consumed < issued) { mbar_wait(bars + (consumed & (FK_STAGES - 1)), (uint32_t)(consumed >> 1) & 1u); ++consumed; }
    }
};

struct MegaCtl { unsigned int target; int dead; };

// Grid barrier: every block arrives (also one that has given up, so the others are not held), then waits for the
// count of this boundary unless it has given up.  Returns false, for the whole block, when the block is to leave.
__device__ __forceinline__ bool mega_barrier(MegaSync *sync, volatile MegaCtl *ctl, FkState *st) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int target = ctl->target + gridDim.x;
        ctl->target = target;
        red_release_add(&sync->count, 1u);          // release: the block's writes, ordered before this by the block barrier above
        unsigned int it = 0;
        while (ctl->dead == 0 && (int)(ld_acquire_u32(&sync->count) - target) < 0) {
            if (++it > FK_MEGA_SPIN_LIMIT || ((it & 1023u) == 0 && *(volatile uint32_t *)&st->error != 0u)) { ctl->dead = 1; atomicOr(&st->error, 0x1000u); }
        }
    }
    __syncthreads();
    return ctl->dead == 0;
}

__device__ __forceinline__ void mega_stamp(unsigned long long *tl, int op, int slot) {
    if (tl && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); tl[((size_t)op * gridDim.x + blockIdx.x) * 8 + slot] = t; }
}

// keys per participating block and number of participating blocks of a kv head
__device__ __forceinline__ void mega_attn_split(int kv_len, int &kpc, int &n_active, int parts = FK_MEGA_PARTS) {
    const int per = (kv_len + parts - 1) / parts;
    kpc = ((per + FK_MEGA_KEYBLOCK - 1) / FK_MEGA_KEYBLOCK) * FK_MEGA_KEYBLOCK;
    n_active = (kv_len + kpc - 1) / kpc;
}

// the K and V rows block (kv head, rank) will read in the attention task, pulled into L2 one task early (one thread)
__device__ __forceinline__ void mega_attn_prefetch(const FkState *st, const SdpaArgs &a) {
    const int kvh = blockIdx.x / FK_MEGA_PARTS, rank = blockIdx.x % FK_MEGA_PARTS;
    if (kvh >= a.n_kv) return;
    const int kv_len = (int)min(st->offset + 1u, (uint32_t)a.capacity);
    int kpc, n_active; mega_attn_split(kv_len, kpc, n_active);
    if (rank >= n_active) return;
    const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
    const size_t off = ((size_t)kvh * a.capacity + k_begin) * a.hd;
    const uint32_t bytes = (uint32_t)(k_end - k_begin) * a.hd * 2;          // rows are multiples of 16 bytes, the caches 256-byte aligned
    l2_prefetch(a.ck + off, bytes); l2_prefetch(a.cv + off, bytes);
}

// ---- attention, written for size: a task runs this code once per token and layer, so rolled loops over shared-memory
// tiles beat unrolled register blocking (the instruction fetch of straight-line code costs more than its execution).
#define FK_ATT_KEYS 64              // keys per pass (two 32-key groups)
template <int HD> struct AttLayout {
    static constexpr int KSTRIDE = HD * 2 + 16;                 // bytes per K row: 16-byte reads of 32 rows hit distinct banks
    static constexpr int q = 0;                                  // float [G][HD]
    __host__ __device__ static constexpr int k(int G) { return G * HD * 4; }                    // bf16 [64][HD + 8]
    __host__ __device__ static constexpr int v(int G) { return k(G) + FK_ATT_KEYS * KSTRIDE; }  // bf16 [64][HD]
    __host__ __device__ static constexpr int s(int G) { return v(G) + FK_ATT_KEYS * HD * 2; }   // float [G][64] scores, then [G][2] group maxima
    __host__ __device__ static constexpr int mrg(int G) { return s(G) + G * (FK_ATT_KEYS + 2) * 4; }   // float [G][2][HD + 2] half partials
    __host__ __device__ static constexpr int bytes(int G) { return mrg(G) + G * 2 * (HD + 2) * 4 + 16; }
};
__host__ __device__ inline size_t mega_attn2_bytes(int G, int hd) { return hd == 128 ? AttLayout<128>::bytes(G) : AttLayout<64>::bytes(G); }

// Block (kv head, rank) of the split: partial (m, l, o[HD]) per q head over keys [rank * kpc, ...) in fp32
// (sdpa_decode.rs:697-715), written to part[(kvh * PARTS + rank)][g][HD + 2]; the last block of a kv head to arrive
// (ticket) folds the partials into out = T(o / l) (sdpa_decode.rs:992-1046).
template <int HD>
__device__ __noinline__ void sdpa_tiles_block(const FkState *st, const SdpaArgs &a, unsigned char *scr, int kvh, int rank, int parts,
                                              unsigned long long *tl, int opi) {
    using L = AttLayout<HD>;
    constexpr int DPL = HD / 32, CH = HD / 8;                    // output dims per lane; 16-byte chunks per row
    const int G = a.n_q / a.n_kv, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nthreads = blockDim.x;
    if (kvh >= a.n_kv) return;
    const int kv_len = (int)min((a.pos_override >= 0 ? (uint32_t)a.pos_override : st->offset) + 1u, (uint32_t)a.capacity);
    int kpc, n_active; mega_attn_split(kv_len, kpc, n_active, parts);
    if (rank >= n_active) return;
    const int stride = HD + 2;
    float *qs = reinterpret_cast<float *>(scr + L::q);
    unsigned char *kt = scr + L::k(G), *vt = scr + L::v(G);
    float *sc = reinterpret_cast<float *>(scr + L::s(G)), *smax = sc + G * FK_ATT_KEYS;
    float *mrg = reinterpret_cast<float *>(scr + L::mrg(G));
    const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
    const uint16_t *K = a.ck + (size_t)kvh * a.capacity * HD, *V = a.cv + (size_t)kvh * a.capacity * HD;
    for (int i = tid; i < G * HD; i += nthreads) qs[i] = bf2f(__ldcg(a.q + kvh * G * HD + i));
    // this warp's (head, key group) item: scores for 32 keys, then p * V over the same 32 keys
    const int item_g = wid >> 1, item_kg = wid & 1;
    const bool has_item = item_g < G;
    float m_run = -INFINITY, l_run = 0.0f, o[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[j] = 0.0f;
    mega_stamp(tl, opi, 4);
#pragma unroll 1
    for (int kb = k_begin; kb < k_end; kb += FK_ATT_KEYS) {
        __syncthreads();                                        // q staged / previous pass done with the tiles
#pragma unroll 2
        for (int i = tid; i < FK_ATT_KEYS * CH; i += nthreads) {        // K and V tiles: rows past the end are zero
            const int row = i / CH, c = i - row * CH;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
            if (kb + row < k_end) {
                kv = __ldcg(reinterpret_cast<const uint4 *>(K + (size_t)(kb + row) * HD) + c);
                vv = __ldcg(reinterpret_cast<const uint4 *>(V + (size_t)(kb + row) * HD) + c);
            }
            *reinterpret_cast<uint4 *>(kt + row * L::KSTRIDE + c * 16) = kv;
            *reinterpret_cast<uint4 *>(vt + row * HD * 2 + c * 16) = vv;
        }
        __syncthreads();
        if (has_item) {                                         // scores: lane = key
            const int key = item_kg * 32 + lane;
            const unsigned char *kr = kt + key * L::KSTRIDE;
            const float *qg = qs + item_g * HD;
            float dot = 0.0f;
#pragma unroll 2
            for (int c = 0; c < CH; ++c) {
                const uint4 kv = *reinterpret_cast<const uint4 *>(kr + c * 16);
                const float4 q0 = *reinterpret_cast<const float4 *>(qg + c * 8), q1 = *reinterpret_cast<const float4 *>(qg + c * 8 + 4);
                dot = fmaf(q0.x, bf_lo(kv.x), dot); dot = fmaf(q0.y, bf_hi(kv.x), dot); dot = fmaf(q0.z, bf_lo(kv.y), dot); dot = fmaf(q0.w, bf_hi(kv.y), dot);
                dot = fmaf(q1.x, bf_lo(kv.z), dot); dot = fmaf(q1.y, bf_hi(kv.z), dot); dot = fmaf(q1.z, bf_lo(kv.w), dot); dot = fmaf(q1.w, bf_hi(kv.w), dot);
            }
            const float sv = (kb + key < k_end) ? dot * a.scale : -INFINITY;
            sc[item_g * FK_ATT_KEYS + key] = sv;
            const float mx = warp_max(sv);
            if (lane == 0) smax[item_g * 2 + item_kg] = mx;
        }
        __syncthreads();
        if (has_item) {                                         // online softmax step and p * V: lane = output dims
            const float m_pass = fmaxf(smax[item_g * 2], smax[item_g * 2 + 1]);      // finite: the pass holds a valid key
            const float m_new = fmaxf(m_run, m_pass);
            const float alpha = expf(m_run - m_new);            // 0 on the first pass
            const float sv = sc[item_g * FK_ATT_KEYS + item_kg * 32 + lane];
            const float pl = sv == -INFINITY ? 0.0f : expf(sv - m_new);
            l_run = fmaf(l_run, alpha, warp_sum(pl)); m_run = m_new;
#pragma unroll
            for (int j = 0; j < DPL; ++j) o[j] *= alpha;
            const unsigned char *vb = vt + (size_t)(item_kg * 32) * HD * 2 + lane * DPL * 2;
#pragma unroll 4
            for (int kk = 0; kk < 32; ++kk) {
                const float pk = __shfl_sync(0xffffffffu, pl, kk);
                if (DPL == 4) {
                    const uint2 vv = *reinterpret_cast<const uint2 *>(vb + kk * HD * 2);
                    o[0] = fmaf(pk, bf_lo(vv.x), o[0]); o[1] = fmaf(pk, bf_hi(vv.x), o[1]); o[2] = fmaf(pk, bf_lo(vv.y), o[2]); o[3] = fmaf(pk, bf_hi(vv.y), o[3]);
                } else {
                    const uint32_t vv = *reinterpret_cast<const uint32_t *>(vb + kk * HD * 2);
                    o[0] = fmaf(pk, bf_lo(vv), o[0]); o[1] = fmaf(pk, bf_hi(vv), o[1]);
                }
            }
        }
    }
    mega_stamp(tl, opi, 5);
    // the two key groups of a head merge through shared memory; warp 2g then owns head g's block partial
    if (has_item) {
        float *w = mrg + (item_g * 2 + item_kg) * stride;
        if (lane == 0) { w[0] = m_run; w[1] = l_run; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) w[2 + lane * DPL + j] = o[j];
    }
    __syncthreads();
    if (has_item && item_kg == 0) {
        const float *w0 = mrg + (item_g * 2) * stride, *w1 = w0 + stride;
        const float M = fmaxf(w0[0], w1[0]);
        const float e0 = w0[0] == -INFINITY ? 0.0f : expf(w0[0] - M), e1 = w1[0] == -INFINITY ? 0.0f : expf(w1[0] - M);
        float *dst = a.part + ((size_t)(kvh * parts + rank) * G + item_g) * stride;
        if (lane == 0) { dst[0] = M; dst[1] = fmaf(w0[1], e0, w1[1] * e1); }
#pragma unroll
        for (int j = 0; j < DPL; ++j) dst[2 + lane * DPL + j] = fmaf(w0[2 + lane * DPL + j], e0, w1[2 + lane * DPL + j] * e1);
    }
    mega_stamp(tl, opi, 6);
    // ticket: the last block of this kv head folds the partials
    __shared__ int is_last;
    __syncthreads();
    if (tid == 0) {
        uint32_t t;     // release: the block's partial, ordered before this by the block barrier; acquire: the other blocks' partials
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(a.counter + kvh) : "memory");
        is_last = (t == (uint32_t)(n_active - 1));
        if (is_last) a.counter[kvh] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    // merge weights e^(m_r - M) / L per (partial, head) into shared memory (the score area is free now), then every
    // thread sums its outputs over the partials straight from L2, eight loads in flight at a time
    const float *src = a.part + (size_t)kvh * parts * G * stride;
    float *wgt = sc;                                            // [n_active][G], n_active * G <= 16 * 8 <= G * 64 floats
    if (tid < G) {
        float M = -INFINITY;
        for (int r = 0; r < n_active; ++r) M = fmaxf(M, __ldcg(src + (size_t)(r * G + tid) * stride));
        float Lsum = 0.0f;
        for (int r = 0; r < n_active; ++r) {
            const float mr = __ldcg(src + (size_t)(r * G + tid) * stride);
            const float e = mr == -INFINITY ? 0.0f : expf(mr - M);
            wgt[r * G + tid] = e; Lsum = fmaf(__ldcg(src + (size_t)(r * G + tid) * stride + 1), e, Lsum);
        }
        const float inv = __fdiv_rn(1.0f, Lsum);
        for (int r = 0; r < n_active; ++r) wgt[r * G + tid] *= inv;
    }
    __syncthreads();
#pragma unroll 1
    for (int i = tid; i < G * HD; i += nthreads) {
        const int g = i / HD, d = i - g * HD;
        float O = 0.0f;
#pragma unroll 8
        for (int r = 0; r < n_active; ++r) O = fmaf(__ldcg(src + (size_t)(r * G + g) * stride + 2 + d), wgt[r * G + g], O);
        a.out[(kvh * G + g) * HD + d] = f2bf(O);
    }
}

// The same attention as a kernel of its own (one kernel per task): grid (parts, kv heads), 16 warps per block.  Chosen
// for long caches, where many blocks per kv head beat the eight of the cluster kernel.
#define FK_TILES_WARPS 16
__host__ __device__ inline int sdpa_tiles_parts(int capacity) { const int p = (capacity + FK_MEGA_KEYBLOCK - 1) / FK_MEGA_KEYBLOCK; return p < FK_MEGA_PARTS ? p : FK_MEGA_PARTS; }
template <int HD>
__global__ void __launch_bounds__(FK_TILES_WARPS * 32) k_sdpa_tiles(const FkState *st, SdpaArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    unsigned char *scr = smem_stream;
    const int parts = (int)gridDim.x, kvh = blockIdx.y, rank = blockIdx.x;
    pdl_launch_dependents();                     // attention leaves most SMs idle: the next projection may start prefetching now
    if (threadIdx.x == 0) {                      // every cache row but the newest was written by earlier tokens: pull this block's rows into L2
        const int kv_len = (int)min((a.pos_override >= 0 ? (uint32_t)a.pos_override : st->offset) + 1u, (uint32_t)a.capacity);
        int kpc, n_active; mega_attn_split(kv_len, kpc, n_active, parts);
        if (rank < n_active) {
            const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
            const size_t off = ((size_t)kvh * a.capacity + k_begin) * HD;
            l2_prefetch(a.ck + off, (uint32_t)(k_end - k_begin) * HD * 2); l2_prefetch(a.cv + off, (uint32_t)(k_end - k_begin) * HD * 2);
        }
    }
    pdl_wait();
    sdpa_tiles_block<HD>(st, a, scr, kvh, rank, parts, a.tl, 0);
}

// the epilogue of whichever streamed task is running (one instance of the streaming loop serves them all)
struct EpiAny {
    int kind; EpiQkv qkv; EpiLinear lin; EpiGateUp gu; EpiHead head;
    __device__ __forceinline__ EpiAny(const MegaOp &op, uint32_t pos) : kind(op.kind), qkv(op.u.qkv, pos), lin(op.u.lin), gu(op.u.gu), head(op.u.head) {}
    __device__ __forceinline__ void prefetch(int tile, int g) {
        if (kind == FK_TASK_RMSNORM_QKV) qkv.prefetch(tile, g); else if (kind == FK_TASK_LINEAR_RESIDUAL) lin.prefetch(tile, g);
    }
    __device__ __forceinline__ void operator()(int tile, int g, float lo, float hi) {
        if (kind == FK_TASK_RMSNORM_QKV) qkv(tile, g, lo, hi);
        else if (kind == FK_TASK_LINEAR_RESIDUAL) lin(tile, g, lo, hi);
        else if (kind == FK_TASK_RMSNORM_GATEUP_ACT) gu(tile, g, lo, hi);
        else head(tile, g, lo, hi);
    }
};

// The persistent kernel.  `ops` is the token's task list, `wtab` the streamed weights in task order.
template <int BITS>
__global__ void __launch_bounds__(FK_MEGA_WARPS * 32, 1)
k_decode_token(FkState *st, const MegaSlot *ops, int nops, const MegaWeight *wtab_g, int nweights, MegaSync *sync, int max_nsb,
               int attn_bytes, int barriers_per_launch, unsigned long long *timeline) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    unsigned char *base = smem_stream;
    const MegaLayout L = mega_layout(nweights, max_nsb, BITS, (size_t)attn_bytes);
    MegaSlot *opbuf = reinterpret_cast<MegaSlot *>(base);
    volatile MegaCtl *ctl = reinterpret_cast<volatile MegaCtl *>(base + 2 * FK_MEGA_OP_BYTES);
    StreamSmem sm;
    sm.bars = reinterpret_cast<uint64_t *>(base + 2 * FK_MEGA_OP_BYTES + 64);            // 512 bytes: 16 warps x 2 stages x 8, then 16 x 8 for wbest
    unsigned long long *wbest = reinterpret_cast<unsigned long long *>(sm.bars + FK_MEGA_WARPS * FK_STAGES);
    sm.zero = reinterpret_cast<uint4 *>(base + 2 * FK_MEGA_OP_BYTES + 64 + 512);
    sm.red = reinterpret_cast<float *>(base + 2 * FK_MEGA_OP_BYTES + 64 + 512 + 256);
    int *wstate = reinterpret_cast<int *>(base + 2 * FK_MEGA_OP_BYTES + 64 + 512 + 256 + 192) + (threadIdx.x >> 5) * 16;     // this warp's producer record
    MegaWeight *wtab = reinterpret_cast<MegaWeight *>(base + L.wtab);
    sm.xsi = reinterpret_cast<float2 *>(base + L.xsi);
    sm.fold = reinterpret_cast<float *>(base + L.fold);
    sm.xs = reinterpret_cast<uint2 *>(base + L.act);
    sm.ring = reinterpret_cast<uint4 *>(base + L.ring);
    float *attn_scr = reinterpret_cast<float *>(base + L.act);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    // ---- set-up: weight table and first task record into shared memory, barriers, ring prefill
    for (int i = threadIdx.x; i < nweights * (int)(sizeof(MegaWeight) / 4); i += blockDim.x) reinterpret_cast<uint32_t *>(wtab)[i] = reinterpret_cast<const uint32_t *>(wtab_g)[i];
    for (int i = threadIdx.x; i < FK_MEGA_OP_BYTES / 16; i += blockDim.x) reinterpret_cast<uint4 *>(opbuf)[i] = reinterpret_cast<const uint4 *>(ops)[i];
    for (int i = threadIdx.x; i < 2 * FK_CHUNK_TILES * FK_STREAM_MAXWARPS * 16; i += blockDim.x) sm.fold[i] = 0.0f;
    if (threadIdx.x == 0) { ctl->target = *(volatile unsigned int *)&sync->seq * (unsigned int)barriers_per_launch * gridDim.x; ctl->dead = 0; }
    uint64_t *wbars = sm.bars + wid * FK_STAGES;
    uint4 *wring = sm.ring + (size_t)wid * FK_STAGES * FK_UNIT_VEC;
    if (lane == 0) { for (int s = 0; s < FK_STAGES; ++s) mbar_init(wbars + s, 1); mbar_fence_init(); }
    __syncthreads();
    {
        MegaStream ms;
        ms.bars = wbars; ms.ring = wring; ms.consumed = 0; ms.issued = 0; ms.widx = -1; ms.nweights = nweights; ms.wtab = wtab;
        ms.prod.left = 0; ms.prod.chunk = 0; ms.prod.tq = 0; ms.prod.sbv = 0; ms.prod.ntl = 0; ms.prod.nsb = 1; ms.prod.nb = 0; ms.prod.lw = 4; ms.prod.inv_nsb = 1.0f;
        ms.seek();
        for (int s = 0; s < FK_STAGES && ms.valid(); ++s) ms.issue(s);
        ms.save(wstate);
    }

    bool ok = true;
    unsigned long long best = 0ull;
    for (int i = 0; i < nops && ok; ++i) {
        const MegaOp &op = opbuf[i & 1].op;
        // the next record travels while this task runs; the block-wide synchronisations inside the task publish it
        if (i + 1 < nops && wid == FK_MEGA_WARPS - 1 && lane < FK_MEGA_OP_BYTES / 16)
            reinterpret_cast<uint4 *>(&opbuf[(i + 1) & 1])[lane] = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const unsigned char *>(ops) + (size_t)(i + 1) * FK_MEGA_OP_BYTES) + lane);
        mega_stamp(timeline, i, 0);
        // One call site per staging routine and one instance of the streaming loop: a task executes its code once, so
        // the kernel is kept small enough for the instruction cache to hold a layer's worth of it.
        const int kind = op.kind;
        const bool streams = op.widx >= 0;
        bool sync_after = true;
        if (kind == FK_TASK_EMBED_LOOKUP_DECODE) {
            // every block writes the same row: a block only ever reads its own copy before the next barrier
            const EmbedArgs &a = op.u.emb;
            const uint32_t tok = st->token[0];
            for (int j = threadIdx.x; j < a.h; j += blockDim.x) a.x[j] = f2bf(bf2f(a.table[(size_t)tok * a.h + j]) * a.scale);
            __threadfence_block();
            __syncthreads();
            sync_after = false;
        } else if (kind == FK_TASK_SDPA_DECODE) {
            const SdpaArgs &a = op.u.sdpa;
            const int kvh = blockIdx.x / FK_MEGA_PARTS, rank = blockIdx.x % FK_MEGA_PARTS;
            if (a.hd == 128) sdpa_tiles_block<128>(st, a, reinterpret_cast<unsigned char *>(attn_scr), kvh, rank, FK_MEGA_PARTS, timeline, i);
            else sdpa_tiles_block<64>(st, a, reinterpret_cast<unsigned char *>(attn_scr), kvh, rank, FK_MEGA_PARTS, timeline, i);
        } else if (streams) {
            const TiledW *W;
            if (kind == FK_TASK_LINEAR_RESIDUAL) {
                const SLinArgs &a = op.u.lin;
                W = &a.P.W;
                stage_plain<BITS, 5>(sm, a.x, a.k, a.P.W.nsb);
            } else {
                // the three norm-first tasks differ only in where their arguments sit
                const uint16_t *x, *nw; int h; float eps;
                if (kind == FK_TASK_RMSNORM_QKV) { const SQkvArgs &a = op.u.qkv; W = &a.P.W; x = a.x; nw = a.norm_w; h = a.h; eps = a.eps; }
                else if (kind == FK_TASK_RMSNORM_GATEUP_ACT) { const SGateUpArgs &a = op.u.gu; W = &a.P.W; x = a.x; nw = a.norm_w; h = a.h; eps = a.eps; }
                else { const SHeadArgs &a = op.u.head; W = &a.P.W; x = a.x; nw = a.norm_w; h = a.h; eps = a.eps; }
                stage_rmsnorm<BITS, false>(sm, x, nw, h, W->nsb, eps, nullptr, nullptr, nullptr, nullptr, nullptr);     // lists with pending norms or all-reduce inputs are refused at build time
            }
            mega_stamp(timeline, i, 1);
            if (kind == FK_TASK_RMSNORM_QKV && threadIdx.x == 0 && i + 1 < nops) {      // the staging above synchronised the block: the next record is in
                const MegaOp &nx = opbuf[(i + 1) & 1].op;
                if (nx.kind == FK_TASK_SDPA_DECODE) mega_attn_prefetch(st, nx.u.sdpa);
            }
            EpiAny epi(op, st->offset);
            { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ok = stream_consume<BITS>(ms, *W, 0, sm, epi); ms.save(wstate); }
            if (kind == FK_TASK_FINAL_RMSNORM_LM_HEAD) {
                best = warp_max_u64(epi.head.best);
                if (lane == 0) wbest[wid] = best;
                __syncthreads();
                if (threadIdx.x == 0) {
                    for (int w = 1; w < FK_MEGA_WARPS; ++w) best = wbest[w] > best ? wbest[w] : best;
                    op.u.head.scratch[blockIdx.x] = best;
                }
            }
        }
        if (!ok) { atomicOr(&st->error, 0x2000u); ctl->dead = 1; }      // a ring wait expired in this warp: the block gives up at the boundary
        mega_stamp(timeline, i, 2);
        if (sync_after) ok = mega_barrier(sync, ctl, st);               // block-uniform from here on
        mega_stamp(timeline, i, 3);
        if (ok && op.kind == FK_TASK_FINAL_RMSNORM_LM_HEAD && blockIdx.x == 0 && wid == 0) {
            const SHeadArgs &a = op.u.head;
            unsigned long long b = 0ull;
            for (int j = lane; j < (int)gridDim.x; j += 32) { const unsigned long long v = __ldcg(a.scratch + j); b = v > b ? v : b; }
            b = warp_max_u64(b);
            if (lane == 0) {
                if (a.finalize) s_finalize_token(st, a.history, b); else a.scratch[0] = b;
                sync->seq = *(volatile unsigned int *)&sync->seq + 1u;      // every block read seq before its first arrive
            }
        }
    }
    if (!ok) { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ms.drain(); }
}
