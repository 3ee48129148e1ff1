// Quantised matrix product for up to 16 activation rows: Y[M, N] = T(X[M, K] . dequant(W)^T + residual), 4-bit weights.
//
// Reference: the M > 1 tiles `fusekit_qmm_*` (src/codegen/msl.rs:2318-2439, 3821-4332; selection kernels/mod.rs:1442-1473),
// used by the reference for prefill chunks and multi-token verify rows; a batch of independent decode rows has no
// reference implementation: row m of the result is checked against the batch-1 matvec of x[m].
//
// The weights stream exactly as in the batch-1 engine (same units of 16 rows x 8 groups, one TMA copy each, a ring per
// warp).  The arithmetic is mma.sync.m16n8k16 on bf16 with exact products: a nibble q becomes the bf16 number 128 + q
// with one shift and one LOP3 per two weights ((w >> 4m) & 0x000F000F | 0x43004300), the activations are bf16 already,
// so every product (128 + q) * x is exact in the fp32 accumulator; per quantisation group the accumulator is flushed as
// s * D + (b - 128 s) * sum(x), which is s * sum(q x) + b * sum(x).  Weight rows are the 16 MMA rows, activation rows the
// columns (two column blocks for more than 8 rows).  K is walked in chunks of one unit (512 activations) shared by the
// warps of a block: the chunk's activations sit in shared memory in B-operand order (a lane's eight k values permuted
// 0,4,1,5,2,6,3,7 to match the nibble pairs above) with the per-group sums beside them.
//
// A block holds 8 tiles (one per warp), so a chunk of activations staged once serves 128 weight rows.  A weight of few
// tiles is split along K instead: `kparts` blocks share a set of 8 tiles, each walks its share of the chunks, writes its
// fp32 partial sums to a scratch area and takes a ticket; the block that draws the last ticket adds the partials in
// part order (the same order whichever block that is) and writes the rows.
#pragma once
#include "fk_stream.cuh"

#define FK_QMM_WARPS 8
#define FK_QMM_MAXM 16
#define FK_QMM_KC 512                               // activations per chunk = per unit at 4 bits
#define FK_QMM_XSTRIDE (FK_QMM_KC * 2 + 64)         // bytes per activation row of a chunk: 16-byte reads of a quarter warp hit distinct banks
#define FK_QMM_CHUNK (FK_QMM_MAXM * FK_QMM_XSTRIDE) // bytes per staged chunk
#define FK_QMM_PART_FLOATS (FK_QMM_WARPS * 8 * 32)  // partial sums one block leaves in the scratch area

// scratch: gridDim.x * FK_QMM_PART_FLOATS floats; counters: one per set of 8 tiles, zero before the launch and after it
// GATEUP form: W holds gate/up row pairs (tile rows g = gate, g + 8 = up of output tile * 8 + g), x is normalised on the
// way into shared memory (norm_w, eps; norm_w == nullptr: x is normalised already), y[m][n] takes the activation (act: 0 SwiGLU, 1 GeGLU-tanh); n = outputs per row.
struct QmmArgs { const uint16_t *x; TiledW W; const uint16_t *residual; uint16_t *y; float *scratch; unsigned int *counters; int m, k, n, kparts;
                 const uint16_t *norm_w; float eps; int act; };

__host__ __device__ inline size_t qmm_smem_bytes() {
    return 256 /*bars*/ + 2 * (size_t)(FK_QMM_CHUNK + FK_QMM_MAXM * 8 * 4 /*group sums*/) + (size_t)FK_QMM_WARPS * FK_STAGES * FK_UNIT_BYTES + 128;
}

template <bool GATEUP>
__global__ void __launch_bounds__(FK_QMM_WARPS * 32, 2) k_qmm4(FkState *st, QmmArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    __shared__ int s_last;
    __shared__ float s_r[FK_QMM_MAXM];                                      // GATEUP: 1 / rms of each activation row
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_stream);
    unsigned char *xs = smem_stream + 256;                                             // [2][16][XSTRIDE]
    float *sx = reinterpret_cast<float *>(xs + 2 * (size_t)FK_QMM_CHUNK);               // [2][16][8]
    uint4 *ring = reinterpret_cast<uint4 *>(reinterpret_cast<unsigned char *>(sx) + 2 * FK_QMM_MAXM * 8 * 4);
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, g = lane >> 2, t = lane & 3;
    const int nsb = a.W.nsb, ntiles = a.W.ntiles, nbs = a.m > 8 ? 2 : 1;
    const int S = a.kparts, kp = (int)blockIdx.x % S, bset = (int)blockIdx.x / S, nsets = (int)gridDim.x / S;
    uint64_t *wbar = bars + wid * FK_STAGES;
    uint4 *wring = ring + (size_t)wid * FK_STAGES * FK_UNIT_VEC;
    if (lane == 0) { for (int s = 0; s < FK_STAGES; ++s) mbar_init(wbar + s, 1); mbar_fence_init(); }
    __syncwarp();
    const int stride = nsets * FK_QMM_WARPS, first = bset * FK_QMM_WARPS + wid;
    const int rounds = (ntiles + stride - 1) / stride;                       // of the block (1 when K is split): every warp walks them all
    const int ss0 = (int)((long long)kp * nsb / S), ss1 = (int)((long long)(kp + 1) * nsb / S);   // this block's chunks of K
    const int total = first < ntiles ? ((ntiles - 1 - first) / stride + 1) * (ss1 - ss0) : 0;      // units of this warp
    int issued = 0, consumed = 0, ptile = first, psb = ss0;
    bool ok = true, announced = false;
    auto issue = [&]() {
        if (lane == 0) {
            const int s = issued & (FK_STAGES - 1);
            mbar_expect_tx(wbar + s, FK_UNIT_BYTES);
            bulk_g2s(wring + (size_t)s * FK_UNIT_VEC, a.W.units + ((size_t)ptile * nsb + psb) * FK_UNIT_VEC, FK_UNIT_BYTES, wbar + s);
        }
        if (++psb == ss1) { psb = ss0; ptile += stride; }
        ++issued;
    };
    while (issued < FK_STAGES && issued < total) issue();                    // weights are constants: fetched before the wait below
    pdl_wait();
    // norm_w == nullptr: the rows come in normalised already (a separate RMSNorm kernel ran once for all blocks)
    const bool norm = GATEUP && a.norm_w != nullptr;
    if (norm) {                                                              // RMSNorm scale of every row, over the whole of K
        if (tid < FK_QMM_MAXM && tid >= a.m) s_r[tid] = 0.0f;
        for (int mm = wid; mm < a.m; mm += FK_QMM_WARPS) {
            float ss = 0.0f;
            const uint4 *xr = reinterpret_cast<const uint4 *>(a.x + (size_t)mm * a.k);
            for (int v0 = lane; v0 < (a.k >> 3); v0 += 32 * 8) {         // eight loads in flight per lane
                uint4 xv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) xv[u] = v0 + 32 * u < (a.k >> 3) ? __ldcg(xr + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float f[8]; unpack8(xv[u], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) s_r[mm] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.k), a.eps)));
        }
        __syncthreads();
    }
    // Staging of chunk `ss`: item = 8 consecutive k of one row, four items per thread (two when 8 rows are enough).  The
    // loads are separate from the permute + store so that the arithmetic of a step sits between the two.
    const int items = nbs * 8 * (FK_QMM_KC / 8);
    auto stage_load = [&](int ss, uint4 (&v)[4], uint4 &wv) {
        if (norm) {                                                          // a thread's four items share their k range: one vector of norm weights
            const int k0 = ss * FK_QMM_KC + (tid & 63) * 8;
            wv = k0 < a.k ? __ldg(reinterpret_cast<const uint4 *>(a.norm_w + k0)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + q * FK_QMM_WARPS * 32, m = idx >> 6, item = idx & 63;
            const int k0 = ss * FK_QMM_KC + item * 8;
            v[q] = make_uint4(0, 0, 0, 0);
            if (idx < items && m < a.m && k0 < a.k) v[q] = __ldcg(reinterpret_cast<const uint4 *>(a.x + (size_t)m * a.k + k0));
        }
    };
    auto stage_store = [&](int buf, const uint4 (&v)[4], const uint4 &wv) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + q * FK_QMM_WARPS * 32, m = idx >> 6, item = idx & 63;
            uint32_t h[4] = {v[q].x, v[q].y, v[q].z, v[q].w};            // (x0,x1) (x2,x3) (x4,x5) (x6,x7)
            if (norm) {                                                  // y = T(w * T(x * r)), two roundings as in the one-row kernel
                float f[8], wf[8]; unpack8(v[q], f); unpack8(wv, wf);
                const float r = s_r[m & (FK_QMM_MAXM - 1)];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = (uint32_t)f2bf(wf[2 * j] * rT(f[2 * j] * r)) | ((uint32_t)f2bf(wf[2 * j + 1] * rT(f[2 * j + 1] * r)) << 16);
            }
            float s8 = bf_lo(h[0]) + bf_hi(h[0]) + bf_lo(h[1]) + bf_hi(h[1]) + bf_lo(h[2]) + bf_hi(h[2]) + bf_lo(h[3]) + bf_hi(h[3]);
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1); s8 += __shfl_xor_sync(0xffffffffu, s8, 2); s8 += __shfl_xor_sync(0xffffffffu, s8, 4);
            if (idx < items) {
                uint4 o;                                                 // B-operand order 0,4 | 1,5 | 2,6 | 3,7
                o.x = (h[0] & 0xffffu) | (h[2] << 16); o.y = (h[0] >> 16) | (h[2] & 0xffff0000u);
                o.z = (h[1] & 0xffffu) | (h[3] << 16); o.w = (h[1] >> 16) | (h[3] & 0xffff0000u);
                *reinterpret_cast<uint4 *>(xs + (size_t)buf * FK_QMM_CHUNK + (size_t)m * FK_QMM_XSTRIDE + item * 16) = o;
                if ((item & 7) == 0) sx[(buf * FK_QMM_MAXM + m) * 8 + (item >> 3)] = s8;
            }
        }
    };
    for (int r = 0; r < rounds; ++r) {
        const int tile = first + r * stride;
        const bool have = tile < ntiles;
        float acc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) { acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.0f; }
        uint4 nxt[4], nxw = make_uint4(0, 0, 0, 0);                      // the next chunk on its way
        stage_load(ss0, nxt, nxw); stage_store(0, nxt, nxw);
        __syncthreads();
        for (int ss = ss0; ss < ss1; ++ss) {
            const int buf = (ss - ss0) & 1;
            if (ss + 1 < ss1) stage_load(ss + 1, nxt, nxw);                   // loaded under this step's arithmetic, stored after it
            if (have && ok) {
                const int s = consumed & (FK_STAGES - 1);
                if (!mbar_wait(wbar + s, (uint32_t)(consumed >> 1) & 1u)) ok = false;
                if (ok) {
                    const uint4 *u = wring + (size_t)s * FK_UNIT_VEC;
                    const unsigned char *xb = xs + (size_t)buf * FK_QMM_CHUNK;
                    const float *sums = sx + buf * FK_QMM_MAXM * 8;
#pragma unroll 4
                    for (int j = 0; j < 8; ++j) {
                        const uint4 w = u[j * 32 + lane];                // {word A row g, word B row g, word A row g+8, word B row g+8}
                        float d[2][4];
#pragma unroll
                        for (int nb = 0; nb < 2; ++nb) { d[nb][0] = d[nb][1] = d[nb][2] = d[nb][3] = 0.0f; }
#pragma unroll
                        for (int wd = 0; wd < 2; ++wd) {                 // word A: k = 64 j + 8 t .., word B: 32 further on
                            const uint32_t w0 = wd ? w.y : w.x, w8 = wd ? w.w : w.z;
                            const int item = j * 8 + wd * 4 + t;
                            const uint32_t p0 = (w0 & 0x000F000Fu) | 0x43004300u, q0 = (w8 & 0x000F000Fu) | 0x43004300u;
                            const uint32_t p1 = ((w0 >> 4) & 0x000F000Fu) | 0x43004300u, q1 = ((w8 >> 4) & 0x000F000Fu) | 0x43004300u;
                            const uint32_t p2 = ((w0 >> 8) & 0x000F000Fu) | 0x43004300u, q2 = ((w8 >> 8) & 0x000F000Fu) | 0x43004300u;
                            const uint32_t p3 = ((w0 >> 12) & 0x000F000Fu) | 0x43004300u, q3 = ((w8 >> 12) & 0x000F000Fu) | 0x43004300u;
#pragma unroll
                            for (int nb = 0; nb < 2; ++nb) {
                                if (nb < nbs) {
                                    const uint4 xv = *reinterpret_cast<const uint4 *>(xb + (size_t)(nb * 8 + g) * FK_QMM_XSTRIDE + item * 16);
                                    mma_bf16(d[nb], p0, q0, p1, q1, xv.x, xv.y);      // nibble pairs (0,4) and (1,5)
                                    mma_bf16(d[nb], p2, q2, p3, q3, xv.z, xv.w);      // (2,6) and (3,7)
                                }
                            }
                        }
                        // scales and biases of rows g, g+8 for group j sit with lane (g, j / 2) of the unit's tail
                        const uint4 sb4 = u[256 + (g << 2) + (j >> 1)];
                        const float s0 = (j & 1) ? bf_hi(sb4.x) : bf_lo(sb4.x), s8 = (j & 1) ? bf_hi(sb4.y) : bf_lo(sb4.y);
                        const float b0 = (j & 1) ? bf_hi(sb4.z) : bf_lo(sb4.z), b8 = (j & 1) ? bf_hi(sb4.w) : bf_lo(sb4.w);
                        const float e0 = fmaf(-128.0f, s0, b0), e8 = fmaf(-128.0f, s8, b8);
#pragma unroll
                        for (int nb = 0; nb < 2; ++nb) {
                            if (nb < nbs) {
                                const float x0 = sums[(nb * 8 + 2 * t) * 8 + j], x1 = sums[(nb * 8 + 2 * t + 1) * 8 + j];
                                acc[nb][0] = fmaf(s0, d[nb][0], fmaf(e0, x0, acc[nb][0])); acc[nb][1] = fmaf(s0, d[nb][1], fmaf(e0, x1, acc[nb][1]));
                                acc[nb][2] = fmaf(s8, d[nb][2], fmaf(e8, x0, acc[nb][2])); acc[nb][3] = fmaf(s8, d[nb][3], fmaf(e8, x1, acc[nb][3]));
                            }
                        }
                    }
                    __syncwarp();
                    if (issued < total) issue();                         // refill the stage just drained
                    else if (!announced) { announced = true; pdl_launch_dependents(); }   // all of this warp's units are on their way
                    ++consumed;
                }
            }
            if (ss + 1 < ss1) stage_store(buf ^ 1, nxt, nxw);                  // the other buffer was last read in step ss - 1
            __syncthreads();                                             // chunk ss is no longer read, chunk ss + 1 is in place
        }
        // val[nb * 4 + i]: rows g (i = 0, 1) and g + 8 (i = 2, 3) of the tile against activation rows nb * 8 + 2 t + (i & 1)
        auto finish = [&](const float (&val)[8]) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const int m = (v >> 2) * 8 + 2 * t + (v & 1);
                if (GATEUP) {
                    const int out = tile * 8 + g;
                    if (!(v & 2) && out < a.n && m < a.m)
                        a.y[(size_t)m * a.n + out] = a.act == 1 ? s_act_geglu(val[v], val[v + 2]) : s_act_swiglu(val[v], val[v + 2]);
                } else {
                    const int row = tile * 16 + g + ((v & 2) ? 8 : 0);
                    if (row < a.n && m < a.m) {
                        float o = val[v];
                        if (a.residual) o += bf2f(__ldcg(a.residual + (size_t)m * a.n + row));
                        a.y[(size_t)m * a.n + row] = f2bf(o);
                    }
                }
            }
        };
        if (S == 1) {
            if (have) {
                const float val[8] = {acc[0][0], acc[0][1], acc[0][2], acc[0][3], acc[1][0], acc[1][1], acc[1][2], acc[1][3]};
                finish(val);
            }
        } else {                                                         // K split over S blocks (one round)
            float *mine = a.scratch + ((size_t)blockIdx.x * FK_QMM_WARPS + wid) * 256;
#pragma unroll
            for (int v = 0; v < 8; ++v) __stcg(mine + v * 32 + lane, acc[v >> 2][v & 3]);
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int ticket = atomicAdd(a.counters + bset, 1u);
                s_last = ticket == (unsigned int)(S - 1);
                if (s_last) a.counters[bset] = 0u;                       // every block of the set has arrived: ready for the next launch
            }
            __syncthreads();
            if (s_last && have) {
                __threadfence();
                float sum[8];
#pragma unroll
                for (int v = 0; v < 8; ++v) sum[v] = 0.0f;
                for (int p = 0; p < S; ++p) {                            // part order, whichever block does the adding
                    const float *src = a.scratch + ((size_t)(bset * S + p) * FK_QMM_WARPS + wid) * 256;
#pragma unroll
                    for (int v = 0; v < 8; ++v) sum[v] += __ldcg(src + v * 32 + lane);
                }
                finish(sum);
            }
        }
    }
    if (!ok) {                                                               // a wait ran out: give the copies in flight one more bounded wait each
        while (consumed < issued) { mbar_wait(wbar + (consumed & (FK_STAGES - 1)), (uint32_t)(consumed >> 1) & 1u); ++consumed; }
        if (lane == 0) atomicOr(&st->error, 0x10000u);
    }
}
