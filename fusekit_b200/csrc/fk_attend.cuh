// Decode attention as the tail of the fused RMSNorm -> QKV -> RoPE -> KV-store kernel.
//
// Reference: the QKV task is followed by the split-K attention tasks (partial + combine, src/codegen/kernels/sdpa_decode.rs:
// 697-715, 992-1046); as kernels of their own they cost a launch gap, a prologue and a cluster hand-off per layer -- more than
// the attention arithmetic of a short context.  Here the blocks of the QKV kernel, which are all resident (one or two per SM),
// carry on after their last row: a grid-wide hand-off (every q, k, v row of this token is written), then block b takes kv head
// b / P and the b % P-th slice of its keys (P = blocks / kv heads), leaves an (m, l, o) partial per q head in global memory,
// a second hand-off, and every block merges the partials for its slice of the output vector.  The arithmetic of a slice is the
// tensor-core form of k_sdpa_mma (S = q K^T and O^T = V^T P^T on mma.m16n8k16, p split into hi + lo bf16 terms).
//
// Hand-offs are counters in global memory: a block's thread 0 fences and adds one after the block's __syncthreads, then polls
// (bounded) until all blocks have arrived.  That is safe here because a block never waits for a block that is not running:
// the grid fits the SMs, earlier kernels do not depend on this one, and programmatic dependents cannot start before every
// block of this grid has started.  The last block to leave resets the counters, so a launch always finds them zero.  When a
// wait runs out the block sets error bit 0x80000 and carries on (wrong values, no hang).
//
// Measured (B200, 7B-shaped q4, context 512): the tail costs ~16 us -- every hand-off is a fence, an atomic and a poll through
// L2 (~2.5 us), and q, the partials and the merge each add an L2 round trip -- where the separate cluster kernel costs 9 us
// including its launch gap: 689 against 780 tok/s.  So the tail is built, tested and OFF by default (FK_ATTEND=1 or
// DecodeEngine(fuse_attention=True) turn it on); the cluster kernel folds through distributed shared memory instead.
//
// Key rows older than this token are fetched (V tile into shared memory, K rows into registers) BEFORE the first hand-off:
// only the newest cache row depends on the other blocks; the warp that owns it fetches its block again afterwards.
#pragma once
#include "fk_kernels.cuh"

#define FK_ATT_SPIN (1u << 21)
#define FK_ATTEND_MAX_BLOCKS 512       // the scratch holds 64 bytes of counters + 512 blocks x 8 heads x (head_dim + 2) floats

struct QkvAttend {
    uint16_t *out;          // T[n_q * head_dim], null: no attention tail
    float *part;            // [blocks][G][head_dim + 2] partials
    unsigned int *ctr;      // [4] hand-off counters, zero between launches
    float scale;
};

__device__ __forceinline__ bool grid_handoff(unsigned int *ctr, unsigned int target) {
    bool ok = true;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(ctr, 1u);
        unsigned int v = 0, it = 0;
        do { asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory"); } while (v < target && ++it < FK_ATT_SPIN);
        ok = v >= target;
    }
    __syncthreads();
    return ok;          // meaningful on thread 0
}

// `tiles`: per-warp areas of at least SdpaMmaLayout<HD>::WTILE bytes, `stride_w` apart (a warp's own ring slots: free once the
// warp's stream has ended); `qs`: 8 rows of SdpaMmaLayout<HD>::QSTRIDE bytes, free once every warp of the block is past the
// first hand-off (the staged activations).
template <int HD>
__device__ __noinline__ void qkv_attend(const QkvAttend at, FkState *st, const uint16_t *q, const uint16_t *ck, const uint16_t *cv,
                                        int n_q, int n_kv, int capacity, uint32_t pos, unsigned char *tiles, int stride_w, unsigned char *qs) {
    using L = SdpaMmaLayout<HD>;
    constexpr int KS = HD / 16, KV4 = HD / 32;
    const int tid = threadIdx.x, NT = blockDim.x, nw = NT >> 5, lane = tid & 31, wid = tid >> 5, g = lane >> 2, t = lane & 3;
    const int G = n_q / n_kv, nblk = (int)gridDim.x, P = nblk / n_kv, b = (int)blockIdx.x;
    const bool active = b < P * n_kv;
    const int kvh = active ? b / P : 0, part = active ? b - kvh * P : 0;
    const int kv_len = (int)min(pos + 1u, (uint32_t)capacity);
    const int kpc = ((kv_len + P * FK_SDPA_MK - 1) / (P * FK_SDPA_MK)) * FK_SDPA_MK;
    const int k_begin = part * kpc, k_end = active ? min(kv_len, k_begin + kpc) : 0;
    const int stride = HD + 2;
    unsigned char *vt = tiles + (size_t)wid * stride_w;
    const uint16_t *K = ck + (size_t)kvh * capacity * HD, *V = cv + (size_t)kvh * capacity * HD;
    uint4 kr[2][KV4];
    auto load_v_tile = [&](int kb) {
#pragma unroll
        for (int i = 0; i < FK_SDPA_MK * (HD / 8) / 32; ++i) {
            const int idx = lane + 32 * i, row = idx / (HD / 8), c = idx - row * (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (kb + row < k_end) v = __ldcg(reinterpret_cast<const uint4 *>(V + (size_t)(kb + row) * HD) + c);
            *reinterpret_cast<uint4 *>(vt + row * L::VSTRIDE + c * 16) = v;
        }
    };
    auto load_k = [&](int kb, int nb) {
        const int key = min(kb + 8 * nb + g, k_end - 1);
        const uint4 *kp = reinterpret_cast<const uint4 *>(K + (size_t)key * HD + t * (HD / 4));
#pragma unroll
        for (int c = 0; c < KV4; ++c) kr[nb][c] = __ldcg(kp + c);
    };
    const int kb0 = k_begin + wid * FK_SDPA_MK;
    const int newest = (int)(pos % (uint32_t)capacity);
    const bool pre = kb0 < k_end;
    if (pre) { load_v_tile(kb0); load_k(kb0, 0); load_k(kb0, 1); }
    bool ok = grid_handoff(at.ctr + 0, (unsigned int)nblk);
    if (pre && newest >= kb0 && newest < kb0 + FK_SDPA_MK) { load_v_tile(kb0); load_k(kb0, 0); load_k(kb0, 1); }
    for (int i = tid; i < G * HD / 2; i += NT) {             // q of this kv head's heads as bf16 rows
        const int gg = (2 * i) / HD, d = 2 * i - gg * HD;
        *reinterpret_cast<uint32_t *>(qs + gg * L::QSTRIDE + d * 2) = __ldcg(reinterpret_cast<const uint32_t *>(q + (size_t)kvh * G * HD) + i);
    }
    __syncthreads();
    uint32_t aq[KS][2];
    const uint32_t *qrow = reinterpret_cast<const uint32_t *>(qs + g * L::QSTRIDE + t * (HD / 2));
#pragma unroll
    for (int s = 0; s < KS; ++s) { aq[s][0] = g < G ? qrow[2 * s] : 0u; aq[s][1] = g < G ? qrow[2 * s + 1] : 0u; }
    float m = -INFINITY, l = 0.0f, oacc[KS][4];
#pragma unroll
    for (int mb = 0; mb < KS; ++mb) { oacc[mb][0] = oacc[mb][1] = oacc[mb][2] = oacc[mb][3] = 0.0f; }
    for (int kb = kb0; kb < k_end; kb += nw * FK_SDPA_MK) {
        if (kb != kb0) { load_v_tile(kb); load_k(kb, 0); load_k(kb, 1); }
        float sacc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.0f;
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                const uint4 q4 = kr[nb][s >> 1];
                const uint32_t w0 = (s & 1) ? q4.z : q4.x, w1 = (s & 1) ? q4.w : q4.y;
                mma_bf16_f32(sacc[nb], aq[s][0], 0u, aq[s][1], 0u, w0, w1);
            }
        }
        float sv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = kb + (i >> 1) * 8 + 2 * t + (i & 1);
            sv[i] = key < k_end ? sacc[i >> 1][i & 1] * at.scale : -INFINITY;
        }
        float mb4 = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mb4 = fmaxf(mb4, __shfl_xor_sync(0xffffffffu, mb4, 1)); mb4 = fmaxf(mb4, __shfl_xor_sync(0xffffffffu, mb4, 2));
        const float mn = fmaxf(m, mb4);
        const float alpha = expf(m - mn);
        float p[4], ls = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { p[i] = sv[i] == -INFINITY ? 0.0f : expf(sv[i] - mn); ls += p[i]; }
        ls += __shfl_xor_sync(0xffffffffu, ls, 1); ls += __shfl_xor_sync(0xffffffffu, ls, 2);
        l = fmaf(l, alpha, ls); m = mn;
        const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), al1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
        for (int mb = 0; mb < KS; ++mb) { oacc[mb][0] *= al0; oacc[mb][1] *= al1; oacc[mb][2] *= al0; oacc[mb][3] *= al1; }
        const uint32_t ph0 = pack_bf16(p[0], p[1]), ph1 = pack_bf16(p[2], p[3]);
        const uint32_t pl0 = pack_bf16(p[0] - bf_lo(ph0), p[1] - bf_hi(ph0)), pl1 = pack_bf16(p[2] - bf_lo(ph1), p[3] - bf_hi(ph1));
        __syncwarp();
        const int mat = lane >> 3, r = lane & 7;
        const uint32_t vaddr = (uint32_t)__cvta_generic_to_shared(vt + ((mat >> 1) * 8 + r) * L::VSTRIDE + (mat & 1) * 16);
#pragma unroll
        for (int mb = 0; mb < KS; ++mb) {
            uint32_t a0, a1, a2, a3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(vaddr + mb * 32));
            mma_bf16_f32(oacc[mb], a0, a1, a2, a3, ph0, ph1);
            mma_bf16_f32(oacc[mb], a0, a1, a2, a3, pl0, pl1);
        }
        __syncwarp();
    }
    // the warp's partial (m, l, o[HD]) per head goes where its tile was; the block folds its warps and leaves one partial in
    // global memory
    float *wp = reinterpret_cast<float *>(vt);
    if (t == 0 && g < G) { wp[g * stride] = m; wp[g * stride + 1] = l; }
#pragma unroll
    for (int mb = 0; mb < KS; ++mb) {
        const int h0 = 2 * t, h1 = 2 * t + 1, d = 16 * mb + g;
        if (h0 < G) { wp[h0 * stride + 2 + d] = oacc[mb][0]; wp[h0 * stride + 2 + d + 8] = oacc[mb][2]; }
        if (h1 < G) { wp[h1 * stride + 2 + d] = oacc[mb][1]; wp[h1 * stride + 2 + d + 8] = oacc[mb][3]; }
    }
    __syncthreads();
    const int nwp = min(nw, max(0, (k_end - k_begin + FK_SDPA_MK - 1) / FK_SDPA_MK));
    float *mine = at.part + (size_t)b * G * stride;
    if (active) for (int i = tid; i < G * stride; i += NT) {
        const int gg = i / stride, c = i - gg * stride;        // c: 0 = m, 1 = l, 2 + d = o[d]
        float M = -INFINITY;
        for (int w = 0; w < nwp; ++w) M = fmaxf(M, reinterpret_cast<const float *>(tiles + (size_t)w * stride_w)[gg * stride]);
        float acc = 0.0f;
        for (int w = 0; w < nwp; ++w) {
            const float *pw = reinterpret_cast<const float *>(tiles + (size_t)w * stride_w) + gg * stride;
            const float e = pw[0] == -INFINITY ? 0.0f : expf(pw[0] - M);
            acc = fmaf(c == 0 ? 0.0f : pw[c], e, acc);
        }
        __stcg(mine + i, c == 0 ? M : acc);
    }
    ok = grid_handoff(at.ctr + 1, (unsigned int)nblk) && ok;
    // merge: the output vector is dealt to the blocks; a warp takes one output at a time, its lanes the key slices
    const int total = n_q * HD, per = (total + nblk - 1) / nblk, np = min(P, (kv_len + kpc - 1) / kpc);
    const int o_begin = b * per, o_end = min(total, o_begin + per);
    for (int o = o_begin + wid; o < o_end; o += nw) {
        const int head = o / HD, d = o - head * HD, hk = head / G, gg = head - hk * G;
        const float *base = at.part + ((size_t)hk * P * G + gg) * stride;
        float M = -INFINITY;
        for (int p2 = lane; p2 < np; p2 += 32) M = fmaxf(M, __ldcg(base + (size_t)p2 * G * stride));
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, s));
        float Ls = 0.0f, O = 0.0f;
        for (int p2 = lane; p2 < np; p2 += 32) {
            const float *pp = base + (size_t)p2 * G * stride;
            const float mp = __ldcg(pp), e = mp == -INFINITY ? 0.0f : expf(mp - M);
            Ls = fmaf(__ldcg(pp + 1), e, Ls); O = fmaf(__ldcg(pp + 2 + d), e, O);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) { Ls += __shfl_xor_sync(0xffffffffu, Ls, s); O += __shfl_xor_sync(0xffffffffu, O, s); }
        if (lane == 0) at.out[o] = f2bf(O * __fdiv_rn(1.0f, Ls));
    }
    if (tid == 0) {
        if (!ok) atomicOr(&st->error, 0x80000u);
        if (atomicAdd(at.ctr + 2, 1u) == (unsigned int)nblk - 1u) { at.ctr[0] = 0u; at.ctr[1] = 0u; at.ctr[2] = 0u; __threadfence(); }
    }
}
