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
//   * attention splits the keys of a kv head over up to FK_MEGA_PARTS blocks, writes (m, l, o) partials, and the
//     o_proj staging of every block folds them (sdpa_decode.rs:992-1046) -- no second barrier, no ticket.
// Co-residency of the grid is guaranteed by the cooperative launch attribute; every wait is bounded and a block
// that gives up sets FkState.error, drains its own copies in flight and leaves.
#pragma once
#include "fk_kernels.cuh"
#include "fk_stream.cuh"

#define FK_MEGA_WARPS 16
#define FK_MEGA_PARTS 8             // blocks that may share one kv head's keys
#define FK_MEGA_KEYBLOCK 128        // keys per block are a multiple of this (16 warps x 8 keys)
#define FK_MEGA_SPIN_LIMIT (1u << 22)

struct MegaSync { unsigned int count, seq, pad[30]; };
struct MegaWeight { const uint4 *units; int ntiles, nsb; };     // what a producer needs of a streamed task

struct MegaAttn {               // o_proj input folded from attention partials instead of read from x
    const float *part; uint16_t *out; int n_q, n_kv, hd, capacity;
};
struct alignas(16) MegaOp {
    int kind, widx;             // FK_TASK_* kind; index into the weight table or -1
    int attn_fold, pad0;
    MegaAttn attn;
    union { EmbedArgs emb; SQkvArgs qkv; SdpaArgs sdpa; SLinArgs lin; SGateUpArgs gu; SHeadArgs head; } u;
};
#define FK_MEGA_OP_BYTES 288
union alignas(16) MegaSlot { MegaOp op; unsigned char raw[FK_MEGA_OP_BYTES]; };      // records sit at a fixed stride
static_assert(sizeof(MegaSlot) == FK_MEGA_OP_BYTES, "MegaOp grew past its slot");

// shared memory: [op slots 2 x 288][flags 64][bars 512][zero 256][red 192][warp stream state 1024][weight table][xsi][fold][activations | attention scratch][ring]
__host__ __device__ inline size_t mega_attn_scratch_bytes(int G, int hd) { return sizeof(float) * (size_t)(G * (hd + 16) + (FK_MEGA_WARPS / 2) * G * (hd + 2) + G * (hd + 2) + 64); }
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
        if ((threadIdx.x & 31) == 0) { w[0] = consumed; w[1] = issued; w[2] = widx; w[3] = prod.chunk; w[4] = prod.tq; w[5] = prod.sbv; w[6] = prod.left; w[7] = prod.ntl; w[8] = prod.nsb; }
        __syncwarp();
    }
    __device__ __forceinline__ void load(const int *w, uint64_t *bars_, uint4 *ring_, const MegaWeight *wtab_, int nweights_) {
        bars = bars_; ring = ring_; wtab = wtab_; nweights = nweights_;
        consumed = w[0]; issued = w[1]; widx = w[2]; prod.chunk = w[3]; prod.tq = w[4]; prod.sbv = w[5]; prod.left = w[6]; prod.ntl = w[7]; prod.nsb = w[8];
        prod.nwarps = blockDim.x >> 5; prod.wid = threadIdx.x >> 5; prod.block = blockIdx.x; prod.grid = gridDim.x;
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
        __threadfence();
        red_release_add(&sync->count, 1u);
        unsigned int it = 0;
        while (ctl->dead == 0 && (int)(ld_acquire_u32(&sync->count) - target) < 0) {
            if (++it > FK_MEGA_SPIN_LIMIT || ((it & 1023u) == 0 && *(volatile uint32_t *)&st->error != 0u)) { ctl->dead = 1; atomicOr(&st->error, 0x1000u); }
        }
        __threadfence();
    }
    __syncthreads();
    return ctl->dead == 0;
}

__device__ __forceinline__ void mega_stamp(unsigned long long *tl, int op, int slot) {
    if (tl && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); tl[((size_t)op * gridDim.x + blockIdx.x) * 8 + slot] = t; }
}

// keys per participating block and number of participating blocks of a kv head
__device__ __forceinline__ void mega_attn_split(int kv_len, int &kpc, int &n_active) {
    const int per = (kv_len + FK_MEGA_PARTS - 1) / FK_MEGA_PARTS;
    kpc = ((per + FK_MEGA_KEYBLOCK - 1) / FK_MEGA_KEYBLOCK) * FK_MEGA_KEYBLOCK;
    n_active = (kv_len + kpc - 1) / kpc;
}

// Attention partials of block (kv head, rank): online softmax per warp over 8-key blocks (four lanes per key for the
// scores, head_dim/32 output dims per lane for p*V), warps merged pairwise through shared memory, the block's
// (m, l, o[hd]) per q head written to part[(kvh * PARTS + rank)][g][hd + 2].
template <int HD, int MAXG>
__device__ __forceinline__ void mega_sdpa(const FkState *st, const SdpaArgs &a, float *scr, unsigned long long *tl, int opi) {
    constexpr int DPL = HD / 32, KV4 = HD / 32, KPW = 8, CW = FK_MEGA_WARPS;
    const int G = a.n_q / a.n_kv, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int kvh = blockIdx.x / FK_MEGA_PARTS, rank = blockIdx.x % FK_MEGA_PARTS;
    if (kvh >= a.n_kv) return;
    const uint32_t pos = st->offset;
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    int kpc, n_active; mega_attn_split(kv_len, kpc, n_active);
    if (rank >= n_active) return;
    const int stride = HD + 2;
    constexpr int QS = HD + 16, QP = HD / 4 + 4;
    float *qs = scr;                              // [G][4][HD/4 + 4]
    float *wpart = qs + G * QS;                   // [CW/2][G][HD+2]
    const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
    const uint16_t *K = a.ck + (size_t)kvh * a.capacity * HD, *V = a.cv + (size_t)kvh * a.capacity * HD;
    const int part = lane & 3, kl = lane >> 2;
    uint4 kreg[KV4]; uint4 vraw[KPW];
    for (int i = tid; i < G * HD; i += CW * 32) { const int g = i / HD, d = i - g * HD; qs[g * QS + (d / (HD / 4)) * QP + d % (HD / 4)] = bf2f(__ldcg(a.q + kvh * G * HD + i)); }
    float m[MAXG], l[MAXG], o[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) { m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[g][j] = 0.0f; }
    __syncthreads();
    mega_stamp(tl, opi, 4);
    for (int kb = k_begin + wid * KPW; kb < k_end; kb += CW * KPW) {
        const int key = kb + kl;
        const bool valid = key < k_end;
        {   // rows past the end are clamped to the last valid row (their scores are masked below): no predicated loads,
            // so all K and V requests of the block are in flight together
            const int kc = min(key, k_end - 1);
            const uint4 *kr = reinterpret_cast<const uint4 *>(K + (size_t)kc * HD + part * (HD / 4));
#pragma unroll
            for (int c = 0; c < KV4; ++c) kreg[c] = __ldcg(kr + c);
#pragma unroll
            for (int kk = 0; kk < KPW; ++kk) {
                const uint16_t *vr = V + (size_t)min(kb + kk, k_end - 1) * HD;
                uint4 r = make_uint4(0, 0, 0, 0);
                if (DPL == 4) { const uint2 v = __ldcg(reinterpret_cast<const uint2 *>(vr) + lane); r.x = v.x; r.y = v.y; }
                else if (DPL == 2) r.x = __ldcg(reinterpret_cast<const uint32_t *>(vr) + lane);
                else r = __ldcg(reinterpret_cast<const uint4 *>(vr) + lane);
                vraw[kk] = r;
            }
        }
        float dot[MAXG];
#pragma unroll
        for (int g = 0; g < MAXG; ++g) dot[g] = 0.0f;
#pragma unroll
        for (int c = 0; c < KV4; ++c) {
            const uint4 v = kreg[c];
            const float kf[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
            const float *qp = qs + part * QP + c * 8;
#pragma unroll
            for (int g = 0; g < MAXG; ++g) if (g < G) {
                const float4 q0 = *reinterpret_cast<const float4 *>(qp + g * QS), q1 = *reinterpret_cast<const float4 *>(qp + g * QS + 4);
                dot[g] = fmaf(q0.x, kf[0], dot[g]); dot[g] = fmaf(q0.y, kf[1], dot[g]); dot[g] = fmaf(q0.z, kf[2], dot[g]); dot[g] = fmaf(q0.w, kf[3], dot[g]);
                dot[g] = fmaf(q1.x, kf[4], dot[g]); dot[g] = fmaf(q1.y, kf[5], dot[g]); dot[g] = fmaf(q1.z, kf[6], dot[g]); dot[g] = fmaf(q1.w, kf[7], dot[g]);
            }
        }
        float p[MAXG];
#pragma unroll
        for (int g = 0; g < MAXG; ++g) if (g < G) {
            float d = dot[g];
            d += __shfl_xor_sync(0xffffffffu, d, 1); d += __shfl_xor_sync(0xffffffffu, d, 2);
            const float s = valid ? d * a.scale : -INFINITY;
            float mb = s;
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 4)); mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 8));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
            const float mn = fmaxf(m[g], mb);                 // finite: the block holds at least one valid key
            const float alpha = expf(m[g] - mn);
            p[g] = valid ? expf(s - mn) : 0.0f;
            float ls = p[g];
            ls += __shfl_xor_sync(0xffffffffu, ls, 4); ls += __shfl_xor_sync(0xffffffffu, ls, 8); ls += __shfl_xor_sync(0xffffffffu, ls, 16);
            l[g] = fmaf(l[g], alpha, ls); m[g] = mn;
#pragma unroll
            for (int j = 0; j < DPL; ++j) o[g][j] *= alpha;
        }
#pragma unroll
        for (int kk = 0; kk < KPW; ++kk) {
#pragma unroll
            for (int g = 0; g < MAXG; ++g) if (g < G) {
                const float pk = __shfl_sync(0xffffffffu, p[g], kk * 4);
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    const uint32_t wv = j < 2 ? vraw[kk].x : j < 4 ? vraw[kk].y : j < 6 ? vraw[kk].z : vraw[kk].w;
                    o[g][j] = fmaf(pk, (j & 1) ? bf_hi(wv) : bf_lo(wv), o[g][j]);
                }
            }
        }
    }
    mega_stamp(tl, opi, 5);
    // pairwise merge of the warps: the upper half writes, the lower half folds, halving until warp 0 holds the block's sums
    for (int half = CW / 2; half >= 1; half >>= 1) {
        if (wid >= half && wid < 2 * half) {
#pragma unroll
            for (int g = 0; g < MAXG; ++g) if (g < G) {
                float *w = wpart + ((wid - half) * G + g) * stride;
                if (lane == 0) { w[0] = m[g]; w[1] = l[g]; }
#pragma unroll
                for (int j = 0; j < DPL; ++j) w[2 + lane * DPL + j] = o[g][j];
            }
        }
        __syncthreads();
        if (wid < half) {
#pragma unroll
            for (int g = 0; g < MAXG; ++g) if (g < G) {
                const float *w = wpart + (wid * G + g) * stride;
                const float m2 = w[0], l2 = w[1];
                const float mn = fmaxf(m[g], m2);
                const float e1 = m[g] == -INFINITY ? 0.0f : expf(m[g] - mn), e2 = m2 == -INFINITY ? 0.0f : expf(m2 - mn);
                l[g] = fmaf(l[g], e1, l2 * e2); m[g] = mn;
#pragma unroll
                for (int j = 0; j < DPL; ++j) o[g][j] = fmaf(o[g][j], e1, w[2 + lane * DPL + j] * e2);
            }
        }
        __syncthreads();
    }
    mega_stamp(tl, opi, 6);
    if (wid == 0) {
#pragma unroll
        for (int g = 0; g < MAXG; ++g) if (g < G) {
            float *w = a.part + ((size_t)(kvh * FK_MEGA_PARTS + rank) * G + g) * stride;
            if (lane == 0) { w[0] = m[g]; w[1] = l[g]; }
#pragma unroll
            for (int j = 0; j < DPL; ++j) w[2 + lane * DPL + j] = o[g][j];
        }
    }
}

// o_proj staging: every block folds the attention partials into x = T(o / l) (sdpa_decode.rs:992-1046) and stages its
// digits; block 0 also publishes x.
template <int BITS>
__device__ __forceinline__ void stage_attn(const StreamSmem &sm, const FkState *st, const MegaAttn &A, int nsb) {
    const int k = A.n_q * A.hd, nblk = k >> 3, G = A.n_q / A.n_kv, stride = A.hd + 2;
    stage_pad<BITS>(sm, k, nsb);
    const int kv_len = (int)min(st->offset + 1u, (uint32_t)A.capacity);
    int kpc, n_active; mega_attn_split(kv_len, kpc, n_active);
    for (int b0 = 0; b0 < nblk; b0 += blockDim.x) {
        const int blk = b0 + threadIdx.x;
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.0f;
        if (blk < nblk) {
            const int head = (blk * 8) / A.hd, d0 = blk * 8 - head * A.hd, kvh = head / G, g = head - kvh * G;
            const float *p0 = A.part + ((size_t)(kvh * FK_MEGA_PARTS) * G + g) * stride;
            const size_t rs = (size_t)G * stride;
            // all (m, l) pairs first, then the outputs four partials at a time: unconditional loads (inactive partials
            // re-read partial 0 and get weight 0), so each batch is one round trip
            float2 ml[FK_MEGA_PARTS];
#pragma unroll
            for (int r = 0; r < FK_MEGA_PARTS; ++r) ml[r] = __ldcg(reinterpret_cast<const float2 *>(p0 + (r < n_active ? r : 0) * rs));
            float M = -INFINITY;
#pragma unroll
            for (int r = 0; r < FK_MEGA_PARTS; ++r) if (r < n_active) M = fmaxf(M, ml[r].x);
            float L = 0.0f;
#pragma unroll
            for (int h4 = 0; h4 < FK_MEGA_PARTS; h4 += 4) {
                if (h4 >= n_active) break;
                float2 o[4][4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 *po = reinterpret_cast<const float2 *>(p0 + (h4 + q < n_active ? h4 + q : 0) * rs + 2 + d0);     // 8-byte aligned: stride and d0 are even
                    o[q][0] = __ldcg(po); o[q][1] = __ldcg(po + 1); o[q][2] = __ldcg(po + 2); o[q][3] = __ldcg(po + 3);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float e = (h4 + q < n_active && ml[h4 + q].x != -INFINITY) ? expf(ml[h4 + q].x - M) : 0.0f;
                    L = fmaf(ml[h4 + q].y, e, L);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { f[2 * j] = fmaf(o[q][j].x, e, f[2 * j]); f[2 * j + 1] = fmaf(o[q][j].y, e, f[2 * j + 1]); }
                }
            }
            const float inv = __fdiv_rn(1.0f, L);
            uint16_t ob16[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { ob16[j] = f2bf(f[j] * inv); f[j] = bf2f(ob16[j]); }
            if (blockIdx.x == 0 && A.out)
                *reinterpret_cast<uint4 *>(A.out + (size_t)blk * 8) = make_uint4(ob16[0] | ((uint32_t)ob16[1] << 16), ob16[2] | ((uint32_t)ob16[3] << 16),
                                                                                 ob16[4] | ((uint32_t)ob16[5] << 16), ob16[6] | ((uint32_t)ob16[7] << 16));
        }
        if (b0 < nblk) store_block<BITS>(sm, blk, f, blk < nblk);
    }
    __syncthreads();
}

// The persistent kernel.  `ops` is the token's task list, `wtab` the streamed weights in task order.
template <int BITS>
__global__ void __launch_bounds__(FK_MEGA_WARPS * 32, 1)
k_decode_token(FkState *st, const MegaSlot *ops, int nops, const MegaWeight *wtab_g, int nweights, MegaSync *sync, int max_nsb,
               int attn_bytes, int barriers_per_launch, unsigned long long *timeline, int dbg) {
    extern __shared__ unsigned char smem_stream[];
    unsigned char *base = (unsigned char *)(((uintptr_t)smem_stream + 127) & ~(uintptr_t)127);
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
        ms.prod.left = 0; ms.prod.chunk = 0; ms.prod.tq = 0; ms.prod.sbv = 0; ms.prod.ntl = 0; ms.prod.nsb = 1;
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
        bool sync_after = true;
        switch (op.kind) {
        case FK_TASK_EMBED_LOOKUP_DECODE: {
            // every block writes the same row: a block only ever reads its own copy before the next barrier
            const EmbedArgs &a = op.u.emb;
            const uint32_t tok = st->token[0];
            for (int j = threadIdx.x; j < a.h; j += blockDim.x) a.x[j] = f2bf(bf2f(a.table[(size_t)tok * a.h + j]) * a.scale);
            __threadfence_block();
            __syncthreads();
            sync_after = false;
            break;
        }
        case FK_TASK_RMSNORM_QKV: {
            const SQkvArgs &a = op.u.qkv;
            stage_rmsnorm<BITS>(sm, a.x, a.norm_w, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, nullptr, a.pend_sum);
            mega_stamp(timeline, i, 1);
            EpiQkv epi(a, st->offset);
            { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ok = stream_consume<BITS>(ms, a.P.W, 0, sm, epi); ms.save(wstate); }
            break;
        }
        case FK_TASK_SDPA_DECODE: {
            const SdpaArgs &a = op.u.sdpa;
            for (int rep = 0; rep <= dbg; ++rep) {       // dbg > 0 (tuning): repeat the task to see it with warm instruction caches
                if (rep) __syncthreads();
                if (a.hd == 128) mega_sdpa<128, 8>(st, a, attn_scr, timeline, i); else mega_sdpa<64, 8>(st, a, attn_scr, timeline, i);
            }
            break;
        }
        case FK_TASK_LINEAR_RESIDUAL: {
            const SLinArgs &a = op.u.lin;
            if (op.attn_fold) stage_attn<BITS>(sm, st, op.attn, a.P.W.nsb); else stage_plain<BITS>(sm, a.x, a.k, a.P.W.nsb);
            mega_stamp(timeline, i, 1);
            EpiLinear epi(a);
            { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ok = stream_consume<BITS>(ms, a.P.W, 0, sm, epi); ms.save(wstate); }
            break;
        }
        case FK_TASK_RMSNORM_GATEUP_ACT: {
            const SGateUpArgs &a = op.u.gu;
            stage_rmsnorm<BITS>(sm, a.x, a.norm_w, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, nullptr, a.pend_sum);
            mega_stamp(timeline, i, 1);
            EpiGateUp epi(a);
            { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ok = stream_consume<BITS>(ms, a.P.W, 0, sm, epi); ms.save(wstate); }
            break;
        }
        case FK_TASK_FINAL_RMSNORM_LM_HEAD: {
            const SHeadArgs &a = op.u.head;
            stage_rmsnorm<BITS>(sm, a.x, a.norm_w, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, nullptr, a.pend_sum);
            mega_stamp(timeline, i, 1);
            EpiHead epi(a);
            { MegaStream ms; ms.load(wstate, wbars, wring, wtab, nweights); ok = stream_consume<BITS>(ms, a.P.W, 0, sm, epi); ms.save(wstate); }
            best = warp_max_u64(epi.best);
            if (lane == 0) wbest[wid] = best;
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < FK_MEGA_WARPS; ++w) best = wbest[w] > best ? wbest[w] : best;
                a.scratch[blockIdx.x] = best;
            }
            break;
        }
        default: break;
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
