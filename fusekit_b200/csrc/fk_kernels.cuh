// Decode kernels, generic-shape edition: one warp per output row (or row pair), 128-bit weight
// loads, in-register dequant with the group-factored form  s * sum(x*q) + b * sum(x), fp32
// accumulation, warp-shuffle reduction.  These are the parity baseline and the fallback for
// shapes the streamed kernels (fk_stream.cuh) do not take.
//
// Programmatic dependent launch order: the projection kernels here wait for their predecessor first and only then let
// their successor start.  A kernel that triggers after its own wait guarantees that everything before it in the stream
// has completed by the time its successor is launched, which is what lets the attention kernels read the decode
// position and prefetch old cache rows ahead of their own wait.
#pragma once
#include "fk_common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

// ---------------------------------------------------------------- activations in shared memory
// x is staged per block as fp32 in a swizzled order so that a lane reading the 32 (or 16, 8)
// activations that belong to its 128-bit weight chunk hits 8 distinct bank groups.
__device__ __forceinline__ int xs_idx(int e) {
    return (e & ~31) | ((((e >> 2) & 7) ^ ((e >> 5) & 7)) << 2) | (e & 3);
}

struct Smem {
    float *xs;      // [K] swizzled fp32 activations
    float *xs16;    // [K/16] sums of 16 consecutive activations
    float *red;     // [40] reduction scratch
};
__device__ __forceinline__ Smem carve(float *base, int k) {
    Smem s; s.xs = base; s.xs16 = base + k; s.red = s.xs16 + (k >> 4); return s;
}
__host__ __device__ inline size_t smem_bytes_for(int k) { return (size_t)(k + (k >> 4) + 48) * sizeof(float); }

__device__ __forceinline__ void fill_xs16(const Smem &sm, int k) {
    for (int i = threadIdx.x; i < (k >> 4); i += blockDim.x) {
        float t = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) t += sm.xs[xs_idx(i * 16 + j)];
        sm.xs16[i] = t;
    }
}

// plain staging: xs = float(x)
__device__ __forceinline__ void stage_x(const Smem &sm, const uint16_t *x, int k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) sm.xs[xs_idx(i)] = bf2f(x[i]);
    __syncthreads();
    fill_xs16(sm, k);
    __syncthreads();
}

// RMSNorm staging: xs = float(T(w * T(x * r))), r = 1/sqrt(mean(x^2) + eps): two roundings to T
// (src/codegen/kernels/mod.rs:4464-4472; rmsnorm_qkv.rs:325).  With a pending tensor the residual
// stream is first advanced, x' = T(x + rmsnorm(pending, pending_w)) -- the Gemma-shaped
// post-attention / post-feed-forward norms -- and block 0 publishes x' to h_out.
__device__ __forceinline__ void stage_norm(const Smem &sm, const uint16_t *x, const uint16_t *w, int h, float eps,
                                           const uint16_t *pending, const uint16_t *pending_w, uint16_t *h_out) {
    if (pending) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < h; i += blockDim.x) { float v = bf2f(pending[i]); ss = fmaf(v, v, ss); }
        ss = block_sum(ss, sm.red);
        const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)h), eps)));
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float n = rT(bf2f(pending_w[i]) * rT(bf2f(pending[i]) * r));
            uint16_t hv = f2bf(bf2f(x[i]) + n);
            sm.xs[xs_idx(i)] = bf2f(hv);
            if (blockIdx.x == 0 && h_out) h_out[i] = hv;
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) sm.xs[xs_idx(i)] = bf2f(x[i]);
    }
    __syncthreads();
    float ss = 0.0f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) { float v = sm.xs[xs_idx(i)]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, sm.red);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)h), eps)));
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        const int p = xs_idx(i);
        sm.xs[p] = rT(bf2f(w[i]) * rT(sm.xs[p] * r));
    }
    __syncthreads();
    fill_xs16(sm, h);
    __syncthreads();
}

// ---------------------------------------------------------------- one row, one warp
template <int BITS>
__device__ __forceinline__ float warp_dot(const WView &W, long long row, const Smem &sm, int lane) {
    const int k = (int)W.k;
    float acc = 0.0f;
    if (BITS == 4) {
        const uint4 *wr = reinterpret_cast<const uint4 *>(W.w + row * (k >> 3));
        const uint16_t *sr = W.s + row * (k >> 6), *br = W.b + row * (k >> 6);
        for (int c = lane; c < (k >> 5); c += 32) {
            const uint4 v = __ldg(wr + c);
            const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
            const int sw = c & 7;
            float p = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 xa = *reinterpret_cast<const float4 *>(sm.xs + c * 32 + (((2 * i) ^ sw) << 2));
                const float4 xb = *reinterpret_cast<const float4 *>(sm.xs + c * 32 + (((2 * i + 1) ^ sw) << 2));
                const uint32_t u = wd[i];
                p = fmaf(xa.x, (float)(u & 15u), p);         p = fmaf(xa.y, (float)((u >> 4) & 15u), p);
                p = fmaf(xa.z, (float)((u >> 8) & 15u), p);  p = fmaf(xa.w, (float)((u >> 12) & 15u), p);
                p = fmaf(xb.x, (float)((u >> 16) & 15u), p); p = fmaf(xb.y, (float)((u >> 20) & 15u), p);
                p = fmaf(xb.z, (float)((u >> 24) & 15u), p); p = fmaf(xb.w, (float)(u >> 28), p);
            }
            const float s = bf2f(__ldg(sr + (c >> 1))), b = bf2f(__ldg(br + (c >> 1)));
            acc = fmaf(s, p, acc);
            acc = fmaf(b, sm.xs16[2 * c] + sm.xs16[2 * c + 1], acc);
        }
    } else if (BITS == 8) {
        const uint4 *wr = reinterpret_cast<const uint4 *>(W.w + row * (k >> 2));
        const uint16_t *sr = W.s + row * (k >> 6), *br = W.b + row * (k >> 6);
        for (int c = lane; c < (k >> 4); c += 32) {
            const uint4 v = __ldg(wr + c);
            const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
            const int base = (c >> 1) * 32, sw = (c >> 1) & 7, f0 = (c & 1) * 4;
            float p = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 xa = *reinterpret_cast<const float4 *>(sm.xs + base + (((f0 + i) ^ sw) << 2));
                const uint32_t u = wd[i];
                p = fmaf(xa.x, (float)(u & 255u), p);         p = fmaf(xa.y, (float)((u >> 8) & 255u), p);
                p = fmaf(xa.z, (float)((u >> 16) & 255u), p); p = fmaf(xa.w, (float)(u >> 24), p);
            }
            const float s = bf2f(__ldg(sr + (c >> 2))), b = bf2f(__ldg(br + (c >> 2)));
            acc = fmaf(s, p, acc);
            acc = fmaf(b, sm.xs16[c], acc);
        }
    } else {
        const uint4 *wr = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(W.w) + row * k);
        for (int c = lane; c < (k >> 3); c += 32) {
            const uint4 v = __ldg(wr + c);
            const int base = (c >> 2) * 32, sw = (c >> 2) & 7, f0 = (c & 3) * 2;
            const float4 xa = *reinterpret_cast<const float4 *>(sm.xs + base + (((f0) ^ sw) << 2));
            const float4 xb = *reinterpret_cast<const float4 *>(sm.xs + base + (((f0 + 1) ^ sw) << 2));
            acc = fmaf(xa.x, bf_lo(v.x), acc); acc = fmaf(xa.y, bf_hi(v.x), acc);
            acc = fmaf(xa.z, bf_lo(v.y), acc); acc = fmaf(xa.w, bf_hi(v.y), acc);
            acc = fmaf(xb.x, bf_lo(v.z), acc); acc = fmaf(xb.y, bf_hi(v.z), acc);
            acc = fmaf(xb.z, bf_lo(v.w), acc); acc = fmaf(xb.w, bf_hi(v.w), acc);
        }
    }
    return warp_sum(acc);
}

// ---------------------------------------------------------------- activations (pointwise tails)
// SwiGLU: g,u rounded to T first, y = T(((1/(1+exp(-g)))*g)*u) (src/codegen/msl.rs:1286-1294)
__device__ __forceinline__ uint16_t act_swiglu(float ga, float ua) {
    const float g = rT(ga), u = rT(ua);
    const float sg = __fdiv_rn(1.0f, 1.0f + expf(-g));
    return f2bf((sg * g) * u);
}
// GeGLU-tanh: the traced chain 0.5*g*(1+tanh(0.79788456*(g+0.044715*g^3)))*u with a rounding to T
// after every op, the cube as two multiplies and tanh(clamp(x,-20,20))
// (src/codegen/kernels/fused_chain.rs:2497-2565, 2715-2729)
__device__ __forceinline__ uint16_t act_geglu_tanh(float ga, float ua) {
    const float g = rT(ga), u = rT(ua);
    const float g3 = rT(rT(g * g) * g);
    const float t2 = rT(g + rT(0.044715f * g3));
    const float t3 = rT(0.7978845608028654f * t2);
    const float t4 = rT(tanhf(fminf(fmaxf(t3, -20.0f), 20.0f)));
    const float t7 = rT(rT(0.5f * g) * rT(1.0f + t4));
    return f2bf(t7 * u);
}

// half-split RoPE angle: inv = exp2(-(d/half)*log2(theta)), ang = float(pos)*inv
// (src/codegen/kernels/rope_q_decode.rs:93-114; rmsnorm_qkv.rs:273, 635-643)
__device__ __forceinline__ void rope_pair(float lo, float hi, int d, int half, uint32_t pos, float log2theta,
                                          uint16_t *o_lo, uint16_t *o_hi) {
    const float e = __fmul_rn(-__fdiv_rn((float)d, (float)half), log2theta);
    const float ang = __fmul_rn((float)pos, exp2f(e));
    float s, c; sincosf(ang, &s, &c);
    *o_lo = f2bf(__fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
    *o_hi = f2bf(__fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
}

// ================================================================ kernels
struct EmbedArgs { const uint16_t *table; uint16_t *x; int h, rows; float scale; int vocab; const uint16_t *qs, *qb; int bits; };
// x[row,:] = T(embed[token[row],:] * scale) (src/codegen/kernels/embed_lookup_decode.rs:95-98); with a quantised table
// (bits 4 / 8: `table` holds the packed u32 words, qs / qb the group scales and biases) the row is dequantised on the fly,
// x = T((float(q) * s + b) * scale), one rounding (embed_lookup_decode.rs:79-93).  A token id outside the table (vocab > 0)
// reads row 0 instead and raises error bit 0x20000: the host refuses such seeds, this guards the ids that arrive through
// the device-side feedback.
__global__ void k_embed_lookup(FkState *st, EmbedArgs a) {
    pdl_launch_dependents(); pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.h * a.rows) return;
    const int row = i / a.h, d = i - row * a.h;
    uint32_t tok = st->token[row];
    if (a.vocab > 0 && tok >= (uint32_t)a.vocab) { if (d == 0) atomicOr(&st->error, 0x20000u); tok = 0; }
    if (a.bits == 4 || a.bits == 8) {
        const int lanes = 32 / a.bits, nwords = a.h / lanes, ngroups = a.h >> 6;
        const uint32_t word = reinterpret_cast<const uint32_t *>(a.table)[(size_t)tok * nwords + d / lanes];
        const uint32_t q = (word >> ((d % lanes) * a.bits)) & ((1u << a.bits) - 1u);
        const float sc = bf2f(a.qs[(size_t)tok * ngroups + (d >> 6)]), bi = bf2f(a.qb[(size_t)tok * ngroups + (d >> 6)]);
        a.x[i] = f2bf(__fmul_rn(__fadd_rn(__fmul_rn((float)q, sc), bi), a.scale));
        return;
    }
    a.x[i] = f2bf(__fmul_rn(bf2f(a.table[(size_t)tok * a.h + d]), a.scale));
}

struct QkvArgs {
    const uint16_t *x, *norm_w; WView W; const uint16_t *lin_bias;
    uint16_t *q_out, *cache_k, *cache_v, *k_out, *v_out;
    const uint16_t *pending, *pending_w; uint16_t *h_out;
    int h, n_q, n_kv, hd, capacity, sinks; float eps, log2theta;
};
// RMSNorm -> Q,K,V matvec (+bias) -> RoPE on Q/K pairs -> K/V written into the live cache
// (src/codegen/kernels/rmsnorm_qkv.rs:616-726).  Without sinks the raw projections are written.
template <int BITS>
__global__ void __launch_bounds__(256) k_rmsnorm_qkv(const FkState *st, QkvArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.h);
    pdl_wait(); pdl_launch_dependents();
    stage_norm(sm, a.x, a.norm_w, a.h, a.eps, a.pending, a.pending_w, a.h_out);
    const int lane = threadIdx.x & 31, half = a.hd >> 1;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
    const int nqk = (a.n_q + a.n_kv) * a.hd, nq_rows = a.n_q * a.hd, nk_rows = a.n_kv * a.hd;
    const int units = (nqk + nk_rows) >> 1;
    const uint32_t pos = st->offset;
    const int wrow = (int)(pos % (uint32_t)a.capacity);
    for (int u = gw; u < units; u += nw) {
        int r0, r1;
        const bool rot = a.sinks && u < (nqk >> 1);
        if (rot) { const int head = u / half, d = u - head * half; r0 = head * a.hd + d; r1 = r0 + half; }
        else { r0 = 2 * u; r1 = r0 + 1; }
        float a0 = warp_dot<BITS>(a.W, r0, sm, lane);
        float a1 = warp_dot<BITS>(a.W, r1, sm, lane);
        if (lane != 0) continue;
        if (a.lin_bias) { a0 += bf2f(a.lin_bias[r0]); a1 += bf2f(a.lin_bias[r1]); }
        uint16_t o0, o1;
        if (rot) rope_pair(rT(a0), rT(a1), r0 % a.hd, half, pos, a.log2theta, &o0, &o1);
        else { o0 = f2bf(a0); o1 = f2bf(a1); }
        const int rr[2] = {r0, r1}; const uint16_t oo[2] = {o0, o1};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int r = rr[j];
            if (r < nq_rows) a.q_out[r] = oo[j];
            else if (r < nqk) {
                const int kr = r - nq_rows, kh = kr / a.hd, d = kr - kh * a.hd;
                if (a.sinks) a.cache_k[((size_t)kh * a.capacity + wrow) * a.hd + d] = oo[j]; else a.k_out[kr] = oo[j];
            } else {
                const int vr = r - nqk, kh = vr / a.hd, d = vr - kh * a.hd;
                if (a.sinks) a.cache_v[((size_t)kh * a.capacity + wrow) * a.hd + d] = oo[j]; else a.v_out[vr] = oo[j];
            }
        }
    }
}

struct QkNormArgs {
    uint16_t *q; const uint16_t *k_in, *v_in, *w_qn, *w_kn; uint16_t *cache_k, *cache_v;
    int n_q, n_kv, hd, capacity; float eps, log2theta;
};
// Gemma-shaped tail of the QKV stage: per-head RMSNorm on q and k (src/codegen/kernels/single.rs:4222-4311),
// RoPE (single.rs:4335-4485), K/V stored into the cache (kv_cache_store_decode.rs).  One block per head.
__global__ void k_qk_norm_rope_store(const FkState *st, QkNormArgs a) {
    __shared__ float red[40]; __shared__ float hv[512];
    pdl_launch_dependents(); pdl_wait();
    const int head = blockIdx.x, d = threadIdx.x, half = a.hd >> 1;
    const bool is_q = head < a.n_q; const int kh = head - a.n_q;
    const uint16_t *src = is_q ? a.q + head * a.hd : a.k_in + kh * a.hd;
    const uint16_t *w = is_q ? a.w_qn : a.w_kn;
    const uint32_t pos = st->offset; const int wrow = (int)(pos % (uint32_t)a.capacity);
    float v = d < a.hd ? bf2f(src[d]) : 0.0f;
    const float ss = block_sum(v * v, red);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.hd), a.eps)));
    if (d < a.hd) hv[d] = rT(bf2f(w[d]) * rT(v * r));
    __syncthreads();
    if (d < half) {
        uint16_t o0, o1; rope_pair(hv[d], hv[d + half], d, half, pos, a.log2theta, &o0, &o1);
        if (is_q) { a.q[head * a.hd + d] = o0; a.q[head * a.hd + d + half] = o1; }
        else {
            uint16_t *dst = a.cache_k + ((size_t)kh * a.capacity + wrow) * a.hd;
            dst[d] = o0; dst[d + half] = o1;
        }
    }
    if (!is_q && d < a.hd) a.cache_v[((size_t)kh * a.capacity + wrow) * a.hd + d] = a.v_in[kh * a.hd + d];
}

struct KvQuantArgs {
    uint16_t *q; const uint16_t *k_in, *v_in; uint32_t *kp, *vp; uint16_t *ks, *kb, *vs, *vb;
    int n_q, n_kv, hd, capacity, bits; float log2theta;
};
// RoPE + store into a quantised cache (src/codegen/kernels/rope_kv_cache_store_decode_quant.rs; the fused form
// rmsnorm_qkv.rs:435-612): q heads are rotated and rounded to T in place; a k head is rotated in fp32 from its T-rounded
// projection and quantised unrounded, a v head is quantised from its T values.  Per group of 64: min / max, the edge of
// larger magnitude anchors the grid (negative scale when that is the maximum), q0 = round(edge / scale), scale = edge / q0
// and bias = edge unless q0 is 0, q = clamp(round((x - bias) / scale)); scales and biases stored as T.  One block per head.
__global__ void k_rope_quant_store(const FkState *st, KvQuantArgs a) {
    __shared__ float row[512]; __shared__ float wmin[16], wmax[16];
    pdl_launch_dependents(); pdl_wait();
    const int head = blockIdx.x, d = threadIdx.x, half = a.hd >> 1, lane = d & 31, wid = d >> 5;
    const uint32_t pos = st->offset; const int wrow = (int)(pos % (uint32_t)a.capacity);
    if (head < a.n_q) {
        if (d < half) {
            uint16_t o0, o1; rope_pair(bf2f(a.q[head * a.hd + d]), bf2f(a.q[head * a.hd + d + half]), d, half, pos, a.log2theta, &o0, &o1);
            a.q[head * a.hd + d] = o0; a.q[head * a.hd + d + half] = o1;
        }
        return;
    }
    const bool is_v = head >= a.n_q + a.n_kv; const int kh = head - a.n_q - (is_v ? a.n_kv : 0);
    if (is_v) { if (d < a.hd) row[d] = bf2f(a.v_in[kh * a.hd + d]); }
    else if (d < half) {
        const float e = __fmul_rn(-__fdiv_rn((float)d, (float)half), a.log2theta);
        const float ang = __fmul_rn((float)pos, exp2f(e));
        float sn, cs; sincosf(ang, &sn, &cs);
        const float lo = bf2f(a.k_in[kh * a.hd + d]), hi = bf2f(a.k_in[kh * a.hd + d + half]);
        row[d] = __fsub_rn(__fmul_rn(lo, cs), __fmul_rn(hi, sn)); row[d + half] = __fadd_rn(__fmul_rn(hi, cs), __fmul_rn(lo, sn));
    }
    __syncthreads();
    const float x = d < a.hd ? row[d] : 0.0f;
    float mn = d < a.hd ? x : INFINITY, mx = d < a.hd ? x : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); }
    if (lane == 0) { wmin[wid] = mn; wmax[wid] = mx; }
    __syncthreads();
    const int grp = d >> 6;                                  // group of 64 = two warps
    const float vmin = fminf(wmin[2 * grp], wmin[2 * grp + 1]), vmax = fmaxf(wmax[2 * grp], wmax[2 * grp + 1]);
    const int mask = (1 << a.bits) - 1;
    const float scale_abs = fmaxf(__fdiv_rn(__fsub_rn(vmax, vmin), (float)mask), 1.0e-7f);
    const bool lo_anchor = fabsf(vmin) > fabsf(vmax);
    float scale = lo_anchor ? scale_abs : -scale_abs;
    const float edge = lo_anchor ? vmin : vmax;
    const float q0 = roundf(__fdiv_rn(edge, scale));
    const bool at_zero = q0 == 0.0f;
    if (!at_zero) scale = __fdiv_rn(edge, q0);
    const float bias = at_zero ? 0.0f : edge;
    const float inv = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    int qi = (int)roundf(__fmul_rn(__fsub_rn(x, bias), inv)); qi = qi < 0 ? 0 : (qi > mask ? mask : qi);
    const int per = 32 / a.bits;
    uint32_t word = d < a.hd ? ((uint32_t)qi << ((d % per) * a.bits)) : 0u;
    for (int o = 1; o < per; o <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, o);
    const size_t crow = (size_t)kh * a.capacity + wrow;
    if (d < a.hd && (d % per) == 0) (is_v ? a.vp : a.kp)[crow * (a.hd / per) + d / per] = word;
    if (d < a.hd && (d & 63) == 0) {
        (is_v ? a.vs : a.ks)[crow * (a.hd >> 6) + grp] = f2bf(scale);
        (is_v ? a.vb : a.kb)[crow * (a.hd >> 6) + grp] = f2bf(bias);
    }
}

struct SdpaArgs {
    const uint16_t *q, *ck, *cv; uint16_t *out; float *part; uint32_t *counter;
    int n_q, n_kv, hd, capacity, chunk; float scale; unsigned long long *tl;
    int pos_override;       // >= 0: decode position given by the caller instead of the device-resident state
    int rows;               // > 1: independent sequences (grid.z), each with its own q / out row and its own cache [n_kv, capacity, hd]
    int consecutive;        // with rows > 1: the rows are consecutive positions of ONE sequence (prefill chunk / verify rows): row m
                            // sits at position offset + m and attends the shared cache up to and including its own row
};
__device__ __forceinline__ void sd_stamp(unsigned long long *tl, int slot) {
    if (tl && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); tl[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + slot] = t; }
}
#define FK_SDPA_KEYS 32        // keys per block
#define FK_SDPA_MAXG 8         // q heads sharing one kv head
#define FK_SDPA_THREADS 256
__host__ __device__ inline size_t sdpa_smem_bytes(int G, int hd, int chunks) {
    return sizeof(float) * (size_t)(G * hd + G * FK_SDPA_KEYS + 2 * G + (FK_SDPA_THREADS / hd) * G * hd + G * chunks + 16);
}
// Split-K GQA decode attention.  Block (chunk, kv head) scores 32 keys against every q head of the group, so
// K/V are read once per group: s = dot(q,k)*scale, partial (m, l, o[hd]) in fp32 (sdpa_decode.rs:697-715).
// The last block of a kv head to finish merges the chunks and writes T(o * (1/l)) (sdpa_decode.rs:992-1046)
// -- a ticket counter, no waiting.  kv_len = min(pos+1, capacity).  head_dim in {64, 128, 256}.
__global__ void __launch_bounds__(FK_SDPA_THREADS) k_sdpa_decode(const FkState *st, SdpaArgs a) {
    extern __shared__ float sm[];
    const int G = a.n_q / a.n_kv, hd = a.hd, kvh = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
    const int nparts = FK_SDPA_THREADS / hd;               // key slices of the PV phase
    float *qs = sm;                                        // [G][hd]
    float *sc = qs + G * hd;                               // [G][KEYS]
    float *ml = sc + G * FK_SDPA_KEYS;                     // [G][2]
    float *op = ml + 2 * G;                                // [nparts][G][hd]
    float *wc = op + nparts * G * hd;                      // [G][chunks] merge weights
    __shared__ int is_last;
    sd_stamp(a.tl, 0);
    pdl_launch_dependents(); pdl_wait();
    const uint32_t pos = a.pos_override >= 0 ? (uint32_t)a.pos_override : st->offset;
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    const int n_active = (kv_len + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS;
    if (chunk >= n_active) return;
    const int k0 = chunk * FK_SDPA_KEYS, bs = min(FK_SDPA_KEYS, kv_len - k0);
    const uint16_t *K = a.ck + ((size_t)kvh * a.capacity + k0) * hd, *V = a.cv + ((size_t)kvh * a.capacity + k0) * hd;
    // V values of this thread's (dim, key slice), fetched before the score phase so the latency overlaps it
    const int vd = tid % hd, vpart = tid / hd, kpp = FK_SDPA_KEYS / nparts;
    uint16_t vreg[FK_SDPA_KEYS];
#pragma unroll
    for (int i = 0; i < FK_SDPA_KEYS; ++i) vreg[i] = 0;
    if (hd == 128) {
#pragma unroll
        for (int i = 0; i < 16; ++i) { const int key = vpart * 16 + i; if (key < bs) vreg[i] = __ldg(V + (size_t)key * hd + vd); }
    } else if (hd == 64) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const int key = vpart * 8 + i; if (key < bs) vreg[i] = __ldg(V + (size_t)key * hd + vd); }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) { if (i < bs) vreg[i] = __ldg(V + (size_t)i * hd + vd); }
    }
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) qs[i] = bf2f(a.q[kvh * G * hd + i]);
    __syncthreads();
    sd_stamp(a.tl, 1);
    {   // scores: 8 threads per key, each over head_dim/8 dims
        const int key = tid >> 3, part = tid & 7, dpp = hd >> 3;
        float dot[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) dot[g] = 0.0f;
        if (key < bs) {
            const uint4 *kr = reinterpret_cast<const uint4 *>(K + (size_t)key * hd + part * dpp);
            for (int c = 0; c < (dpp >> 3); ++c) {
                const uint4 v = __ldg(kr + c);
                const float kf[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
                const float *qp = qs + part * dpp + c * 8;
#pragma unroll
                for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) dot[g] = fmaf(qp[g * hd + j], kf[j], dot[g]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) {
            float d = dot[g];
            d += __shfl_xor_sync(0xffffffffu, d, 1); d += __shfl_xor_sync(0xffffffffu, d, 2); d += __shfl_xor_sync(0xffffffffu, d, 4);
            if (part == 0) sc[g * FK_SDPA_KEYS + key] = key < bs ? d * a.scale : -INFINITY;
        }
    }
    __syncthreads();
    sd_stamp(a.tl, 2);
    const int lane = tid & 31, wid = tid >> 5;
    if (wid < G) {      // softmax pieces of head `wid` over the 32 keys
        const float s0 = sc[wid * FK_SDPA_KEYS + lane];
        const float m = warp_max(s0);
        const float p0 = lane < bs ? expf(s0 - m) : 0.0f;
        sc[wid * FK_SDPA_KEYS + lane] = p0;
        const float l = warp_sum(p0);
        if (lane == 0) { ml[2 * wid] = m; ml[2 * wid + 1] = l; }
    }
    __syncthreads();
    {   // o[g][d] over this thread's key slice
        float o[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) o[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < FK_SDPA_KEYS; ++i) {
            if (i < kpp) {
                const float v = bf2f(vreg[i]); const int key = vpart * kpp + i;
#pragma unroll
                for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) o[g] = fmaf(sc[g * FK_SDPA_KEYS + key], v, o[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) op[(vpart * G + g) * hd + vd] = o[g];
    }
    __syncthreads();
    const int stride = hd + 2;
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) {
        float o = 0.0f;
        for (int q = 0; q < nparts; ++q) o += op[q * G * hd + i];
        const int g = i / hd, d = i - g * hd;
        float *p = a.part + ((size_t)(kvh * G + g) * a.chunk + chunk) * stride;
        if (n_active == 1) a.out[(kvh * G + g) * hd + d] = f2bf(o * __fdiv_rn(1.0f, ml[2 * g + 1]));
        else { p[2 + d] = o; if (d == 0) { p[0] = ml[2 * g]; p[1] = ml[2 * g + 1]; } }
    }
    if (n_active == 1) return;
    sd_stamp(a.tl, 3);
    __threadfence();
    __syncthreads();
    sd_stamp(a.tl, 4);
    if (tid == 0) {
        const uint32_t t = atomicAdd(a.counter + kvh, 1u);
        is_last = (t == (uint32_t)(n_active - 1));
        if (is_last) a.counter[kvh] = 0u;
    }
    __syncthreads();
    sd_stamp(a.tl, 5);
    if (!is_last) return;
    __threadfence();
    if (wid < G) {      // merge weights w_c = exp(m_c - M) and the normaliser, one warp per head
        const float *p = a.part + (size_t)(kvh * G + wid) * a.chunk * stride;
        float M = -INFINITY;
        for (int c = lane; c < n_active; c += 32) M = fmaxf(M, __ldcg(p + (size_t)c * stride));
        M = warp_max(M);
        float L = 0.0f;
        for (int c = lane; c < n_active; c += 32) {
            const float w = expf(__ldcg(p + (size_t)c * stride) - M);
            wc[wid * a.chunk + c] = w;
            L = fmaf(__ldcg(p + (size_t)c * stride + 1), w, L);
        }
        L = warp_sum(L);
        if (lane == 0) ml[2 * wid + 1] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) {
        const int g = i / hd, d = i - g * hd;
        const float *p = a.part + (size_t)(kvh * G + g) * a.chunk * stride + 2 + d;
        float O = 0.0f;
        for (int c = 0; c < n_active; ++c) O = fmaf(__ldcg(p + (size_t)c * stride), wc[g * a.chunk + c], O);
        a.out[(kvh * G + g) * hd + d] = f2bf(O * __fdiv_rn(1.0f, ml[2 * g + 1]));
    }
    __syncthreads();
    sd_stamp(a.tl, 6);
}

struct SdpaQArgs {
    const uint16_t *q; const uint32_t *kp, *vp; const uint16_t *ks, *kb, *vs, *vb; uint16_t *out; float *part; uint32_t *counter;
    int n_q, n_kv, hd, capacity, chunk; float scale;
};
// Split-K GQA decode attention over a QUANTISED cache: packed words [n_kv, capacity, hd * bits / 32] with T scales and biases
// [n_kv, capacity, hd / 64] per cache row; keys and values are dequantised in registers, float(q) * s + b
// (src/codegen/kernels/sdpa_decode_quant.rs:301-372 scores, 429-470 weighted values, 506-680 the split form).  Same
// decomposition as k_sdpa_decode: 32 keys per block, partial (m, l, o) per chunk, the last block of a kv head merges.
template <int BITS>
__global__ void __launch_bounds__(FK_SDPA_THREADS) k_sdpa_decode_q(const FkState *st, SdpaQArgs a) {
    extern __shared__ float sm[];
    const int G = a.n_q / a.n_kv, hd = a.hd, kvh = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
    const int nparts = FK_SDPA_THREADS / hd;               // key slices of the PV phase
    float *qs = sm;                                        // [G][hd]
    float *sc = qs + G * hd;                               // [G][KEYS]
    float *ml = sc + G * FK_SDPA_KEYS;                     // [G][2]
    float *op = ml + 2 * G;                                // [nparts][G][hd]
    float *wc = op + nparts * G * hd;                      // [G][chunks] merge weights
    __shared__ int is_last;
    pdl_launch_dependents(); pdl_wait();
    const uint32_t pos = st->offset;
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    const int n_active = (kv_len + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS;
    if (chunk >= n_active) return;
    const int k0 = chunk * FK_SDPA_KEYS, bs = min(FK_SDPA_KEYS, kv_len - k0);
    constexpr int PER = 32 / BITS; constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int nw = hd / PER, ng = hd >> 6;                 // packed words and quantisation groups per cache row
    const size_t row0 = (size_t)kvh * a.capacity + k0;     // first cache row of this block
    // V values of this thread's (dim, key slice), fetched before the score phase so the latency overlaps it
    const int vd = tid % hd, vpart = tid / hd, kpp = FK_SDPA_KEYS / nparts;
    float vreg[FK_SDPA_KEYS];                           // dequantised V values of this thread's (dim, key slice)
#pragma unroll
    for (int i = 0; i < FK_SDPA_KEYS; ++i) {
        vreg[i] = 0.0f;
        const int key = vpart * kpp + i;
        if (i < kpp && key < bs) {
            const uint32_t w = __ldg(a.vp + (row0 + key) * nw + vd / PER);
            const float sc = bf2f(__ldg(a.vs + (row0 + key) * ng + (vd >> 6))), bi = bf2f(__ldg(a.vb + (row0 + key) * ng + (vd >> 6)));
            vreg[i] = __fadd_rn(__fmul_rn((float)((w >> ((vd % PER) * BITS)) & MASK), sc), bi);
        }
    }
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) qs[i] = bf2f(a.q[kvh * G * hd + i]);
    __syncthreads();
    {   // scores: 8 threads per key, each over head_dim/8 dims
        const int key = tid >> 3, part = tid & 7, dpp = hd >> 3;
        float dot[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) dot[g] = 0.0f;
        if (key < bs) {
            // every key element is float(q) * s + b with the row's T scale and bias of its group (sdpa_decode_quant.rs:301-372)
            const int d0 = part * dpp;
            const float sc = bf2f(__ldg(a.ks + (row0 + key) * ng + (d0 >> 6))), bi = bf2f(__ldg(a.kb + (row0 + key) * ng + (d0 >> 6)));
            const uint32_t *kw = a.kp + (row0 + key) * nw + d0 / PER;
            for (int c = 0; c < dpp / PER; ++c) {
                const uint32_t w = __ldg(kw + c);
                const float *qp = qs + d0 + c * PER;
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const float kf = __fadd_rn(__fmul_rn((float)((w >> (j * BITS)) & MASK), sc), bi);
#pragma unroll
                    for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) dot[g] = fmaf(qp[g * hd + j], kf, dot[g]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) {
            float d = dot[g];
            d += __shfl_xor_sync(0xffffffffu, d, 1); d += __shfl_xor_sync(0xffffffffu, d, 2); d += __shfl_xor_sync(0xffffffffu, d, 4);
            if (part == 0) sc[g * FK_SDPA_KEYS + key] = key < bs ? d * a.scale : -INFINITY;
        }
    }
    __syncthreads();
    const int lane = tid & 31, wid = tid >> 5;
    if (wid < G) {      // softmax pieces of head `wid` over the 32 keys
        const float s0 = sc[wid * FK_SDPA_KEYS + lane];
        const float m = warp_max(s0);
        const float p0 = lane < bs ? expf(s0 - m) : 0.0f;
        sc[wid * FK_SDPA_KEYS + lane] = p0;
        const float l = warp_sum(p0);
        if (lane == 0) { ml[2 * wid] = m; ml[2 * wid + 1] = l; }
    }
    __syncthreads();
    {   // o[g][d] over this thread's key slice
        float o[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) o[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < FK_SDPA_KEYS; ++i) {
            if (i < kpp) {
                const float v = vreg[i]; const int key = vpart * kpp + i;
#pragma unroll
                for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) o[g] = fmaf(sc[g * FK_SDPA_KEYS + key], v, o[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) op[(vpart * G + g) * hd + vd] = o[g];
    }
    __syncthreads();
    const int stride = hd + 2;
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) {
        float o = 0.0f;
        for (int q = 0; q < nparts; ++q) o += op[q * G * hd + i];
        const int g = i / hd, d = i - g * hd;
        float *p = a.part + ((size_t)(kvh * G + g) * a.chunk + chunk) * stride;
        if (n_active == 1) a.out[(kvh * G + g) * hd + d] = f2bf(o * __fdiv_rn(1.0f, ml[2 * g + 1]));
        else { p[2 + d] = o; if (d == 0) { p[0] = ml[2 * g]; p[1] = ml[2 * g + 1]; } }
    }
    if (n_active == 1) return;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t t = atomicAdd(a.counter + kvh, 1u);
        is_last = (t == (uint32_t)(n_active - 1));
        if (is_last) a.counter[kvh] = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (wid < G) {      // merge weights w_c = exp(m_c - M) and the normaliser, one warp per head
        const float *p = a.part + (size_t)(kvh * G + wid) * a.chunk * stride;
        float M = -INFINITY;
        for (int c = lane; c < n_active; c += 32) M = fmaxf(M, __ldcg(p + (size_t)c * stride));
        M = warp_max(M);
        float L = 0.0f;
        for (int c = lane; c < n_active; c += 32) {
            const float w = expf(__ldcg(p + (size_t)c * stride) - M);
            wc[wid * a.chunk + c] = w;
            L = fmaf(__ldcg(p + (size_t)c * stride + 1), w, L);
        }
        L = warp_sum(L);
        if (lane == 0) ml[2 * wid + 1] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * hd; i += FK_SDPA_THREADS) {
        const int g = i / hd, d = i - g * hd;
        const float *p = a.part + (size_t)(kvh * G + g) * a.chunk * stride + 2 + d;
        float O = 0.0f;
        for (int c = 0; c < n_active; ++c) O = fmaf(__ldcg(p + (size_t)c * stride), wc[g * a.chunk + c], O);
        a.out[(kvh * G + g) * hd + d] = f2bf(O * __fdiv_rn(1.0f, ml[2 * g + 1]));
    }
    __syncthreads();
}

// ---------------------------------------------------------------- cluster SDPA
#define FK_SDPA_CL 8            // CTAs per kv head (portable cluster size); they split the keys
#define FK_SDPA_CLMAX 16        // the tensor-core kernel also runs as a cluster of 16 (non-portable size) when few kv heads leave SMs idle
#define FK_SDPA_CW 16           // warps per CTA
#define FK_SDPA_KPW 8           // keys per warp iteration (4 lanes per key)
__host__ __device__ inline size_t sdpa_cl_smem_bytes(int G, int hd) {
    return sizeof(float) * (size_t)(G * (hd + 16) + FK_SDPA_CW * G * (hd + 2) + G * (hd + 2) + FK_SDPA_CW * G + G + 16);
}
// Split-K GQA decode attention on a thread-block cluster: the CTAs of a cluster share one kv head and take
// contiguous key ranges; inside a CTA every warp runs an online softmax over 8-key blocks, four lanes per key for
// the scores (s = dot(q,k)*scale in fp32) and head_dim/32 output dims per lane for p*V, with running (m, l, o)
// (sdpa_decode.rs:1064-1211).  K and V rows of a block are requested together, and the first block before the
// dependency wait: every cache row but the newest was written by earlier tokens.  Warp partials merge through
// shared memory, CTA partials through distributed shared memory (sdpa_decode.rs:992-1046 combine),
// out = T(o * (1/l)).  No global scratch, no spinning.
template <int HD, int MAXG>
__global__ void __launch_bounds__(FK_SDPA_CW * 32) k_sdpa_cluster(const FkState *st, SdpaArgs a) {
    extern __shared__ float sm[];
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int DPL = HD / 32;                 // output dims per lane
    constexpr int KV4 = HD / 32;                 // uint4 per quarter row (HD/4 dims * 2 B / 16)
    constexpr int NT = FK_SDPA_CW * 32;
    const int G = a.n_q / a.n_kv, kvh = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int rank = (int)cluster.block_rank(), CL = (int)cluster.num_blocks();
    const int stride = HD + 2;
    constexpr int QS = HD + 16, QP = HD / 4 + 4; // q rows padded per quarter so the four lanes of a key hit distinct banks
    float *qs = sm;                              // [G][4][HD/4 + 4]
    float *wpart = qs + G * QS;                  // [CW][G][HD+2]
    float *cpart = wpart + FK_SDPA_CW * G * stride;   // [G][HD+2]   read by the other CTAs of the cluster
    float *wexp = cpart + G * stride;            // [CW][G] merge weights of the warp partials
    sd_stamp(a.tl, 0);
    pdl_launch_dependents();                     // attention occupies few SMs: the next projection may start prefetching now
    const uint32_t pos = st->offset;             // advanced by the previous token's head kernel, not by the QKV kernel in flight
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    const int newest = (int)(pos % (uint32_t)a.capacity);
    const int kpc = ((kv_len + CL * FK_SDPA_KPW - 1) / (CL * FK_SDPA_KPW)) * FK_SDPA_KPW;
    const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
    const uint16_t *K = a.ck + (size_t)kvh * a.capacity * HD, *V = a.cv + (size_t)kvh * a.capacity * HD;
    const int part = lane & 3, kl = lane >> 2;
    uint4 kreg[KV4]; uint4 vraw[FK_SDPA_KPW];    // V rows: DPL bf16 per lane, in the low words of vraw
    auto load_k = [&](int kb, int skip) {
        const int key = kb + kl;
        const uint4 *kr = reinterpret_cast<const uint4 *>(K + (size_t)key * HD + part * (HD / 4));
#pragma unroll
        for (int c = 0; c < KV4; ++c) kreg[c] = (key < k_end && key != skip) ? __ldg(kr + c) : make_uint4(0, 0, 0, 0);
    };
    auto load_v_row = [&](int row) -> uint4 {
        uint4 r = make_uint4(0, 0, 0, 0);
        if (DPL == 4) { const uint2 v = *(reinterpret_cast<const uint2 *>(V + (size_t)row * HD) + lane); r.x = v.x; r.y = v.y; }
        else if (DPL == 2) r.x = *(reinterpret_cast<const uint32_t *>(V + (size_t)row * HD) + lane);
        else r = *(reinterpret_cast<const uint4 *>(V + (size_t)row * HD) + lane);
        return r;
    };
    auto load_v = [&](int kb, int skip) {
#pragma unroll
        for (int kk = 0; kk < FK_SDPA_KPW; ++kk) vraw[kk] = (kb + kk < k_end && kb + kk != skip) ? load_v_row(kb + kk) : make_uint4(0, 0, 0, 0);
    };
    int kb = k_begin + wid * FK_SDPA_KPW;
    if (kb < k_end) { load_k(kb, newest); load_v(kb, newest); }
    pdl_wait();
    for (int i = tid; i < G * HD; i += NT) { const int g = i / HD, d = i - g * HD; qs[g * QS + (d / (HD / 4)) * QP + d % (HD / 4)] = bf2f(a.q[kvh * G * HD + i]); }
    float m[MAXG], l[MAXG], o[MAXG][DPL];
#pragma unroll
    for (int g = 0; g < MAXG; ++g) { m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < DPL; ++j) o[g][j] = 0.0f; }
    if (kb < k_end && newest >= kb && newest < kb + FK_SDPA_KPW && newest < k_end) {       // the row the QKV kernel just wrote
        if (kb + kl == newest) load_k(kb, -1);
#pragma unroll
        for (int kk = 0; kk < FK_SDPA_KPW; ++kk) if (kb + kk == newest) vraw[kk] = load_v_row(newest);
    }
    __syncthreads();
    sd_stamp(a.tl, 1);
    for (bool first = true; kb < k_end; kb += FK_SDPA_CW * FK_SDPA_KPW, first = false) {
        const bool valid = kb + kl < k_end;
        if (!first) { load_k(kb, -1); load_v(kb, -1); }
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
        if (first) sd_stamp(a.tl, 5);
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
        if (first) sd_stamp(a.tl, 7);
#pragma unroll
        for (int kk = 0; kk < FK_SDPA_KPW; ++kk) {
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
    sd_stamp(a.tl, 2);
#pragma unroll
    for (int g = 0; g < MAXG; ++g) if (g < G) {
        float *w = wpart + (wid * G + g) * stride;
        if (lane == 0) { w[0] = m[g]; w[1] = l[g]; }
#pragma unroll
        for (int j = 0; j < DPL; ++j) w[2 + lane * DPL + j] = o[g][j];
    }
    __syncthreads();
    // fold the warps of this CTA: weights e^(m_w - M) once per (warp, head), then every thread sums its outputs
    const int nwp = min(FK_SDPA_CW, (k_end - k_begin + FK_SDPA_KPW - 1) / FK_SDPA_KPW);      // warps that saw keys
    if (tid < G) {
        float M = -INFINITY;
        for (int w = 0; w < nwp; ++w) M = fmaxf(M, wpart[(w * G + tid) * stride]);
        float L = 0.0f;
        for (int w = 0; w < nwp; ++w) {
            const float *pw = wpart + (w * G + tid) * stride;
            const float e = pw[0] == -INFINITY ? 0.0f : expf(pw[0] - M);
            wexp[w * G + tid] = e; L = fmaf(pw[1], e, L);
        }
        cpart[tid * stride] = M; cpart[tid * stride + 1] = L;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += NT) {
        const int g = i / HD, d = i - g * HD;
        float O = 0.0f;
        for (int w = 0; w < nwp; ++w) O = fmaf(wpart[(w * G + g) * stride + 2 + d], wexp[w * G + g], O);
        cpart[g * stride + 2 + d] = O;
    }
    sd_stamp(a.tl, 3);
    cluster.sync();
    sd_stamp(a.tl, 4);
    const int total = G * HD, per = (total + CL - 1) / CL;
    for (int i = rank * per + tid; i < min(total, (rank + 1) * per); i += NT) {      // fold the CTAs: this CTA's slice of outputs
        const int g = i / HD, d = i - g * HD;
        float mm[FK_SDPA_CL], ll[FK_SDPA_CL], oo[FK_SDPA_CL];
#pragma unroll
        for (int r = 0; r < FK_SDPA_CL; ++r) {
            if (r < CL) { const float *rp = cluster.map_shared_rank(cpart, r) + g * stride; mm[r] = rp[0]; ll[r] = rp[1]; oo[r] = rp[2 + d]; }
            else { mm[r] = -INFINITY; ll[r] = 0.0f; oo[r] = 0.0f; }
        }
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < FK_SDPA_CL; ++r) M = fmaxf(M, mm[r]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int r = 0; r < FK_SDPA_CL; ++r) { const float e = mm[r] == -INFINITY ? 0.0f : expf(mm[r] - M); L = fmaf(ll[r], e, L); O = fmaf(oo[r], e, O); }
        a.out[(kvh * G + g) * HD + d] = f2bf(O * __fdiv_rn(1.0f, L));
    }
    cluster.sync();                                      // peers may still be reading this CTA's partial
    sd_stamp(a.tl, 6);
}

// ---------------------------------------------------------------- tensor-core cluster SDPA
// Same split as k_sdpa_cluster (cluster of 8 CTAs per kv head, contiguous key ranges, online softmax per warp, warp ->
// CTA -> cluster fold), but a warp iteration takes 16 keys on mma.sync.m16n8k16 (bf16, fp32 accumulate):
//   S[head][key]   = q K^T      -- A = q (heads padded to 16 rows, kept in registers), B = K rows straight from global
//                                  (a lane owns 32 contiguous dims of its key; the dims are relabelled identically in A)
//   O^T[dim][head] = V^T P^T    -- A = V^T through ldmatrix.trans from a per-warp shared-memory tile, B = P^T, which is
//                                  exactly the layout S came out in; p is split into two bf16 terms (hi + lo), so the
//                                  products carry 16 significant bits of p (sdpa_decode.rs:697-715 accumulates p*v in fp32)
// A lane then handles one head instead of looping over the group: ~150 instructions per 16 keys instead of ~2200.
#define FK_SDPA_MK 16
__device__ __forceinline__ void mma_bf16_f32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16); }
template <int HD> struct SdpaMmaLayout {
    static constexpr int QSTRIDE = HD * 2 + 16;                  // bytes per q row (bf16)
    static constexpr int VSTRIDE = HD * 2 + 16;                  // bytes per V tile row: ldmatrix rows hit distinct banks
    static constexpr int WTILE = FK_SDPA_MK * VSTRIDE;           // bytes of a warp's V tile; later its [G][HD+2] fp32 partial
    __host__ __device__ static constexpr int q() { return 0; }
    __host__ __device__ static constexpr int tiles() { return 8 * QSTRIDE; }
    __host__ __device__ static constexpr int cpart() { return tiles() + FK_SDPA_CW * WTILE; }
    __host__ __device__ static constexpr int wexp(int G) { return cpart() + (G * HD + FK_SDPA_CLMAX) * 4; }      // after the received o slices
    __host__ __device__ static constexpr int fexp(int G) { return wexp(G) + FK_SDPA_CLMAX * G * 2 * 4; }              // [16][G] factors + [G] maxima + [G] 1 / l
    __host__ __device__ static constexpr int bytes(int G) { return fexp(G) + (16 * G + 2 * G) * 4 + 64; }
};
__host__ __device__ inline size_t sdpa_mma_smem_bytes(int G, int hd) { return hd == 256 ? SdpaMmaLayout<256>::bytes(G) : hd == 128 ? SdpaMmaLayout<128>::bytes(G) : SdpaMmaLayout<64>::bytes(G); }
template <int HD>
__global__ void __launch_bounds__(FK_SDPA_CW * 32) k_sdpa_mma(const FkState *st, SdpaArgs a) {
    extern __shared__ __align__(128) unsigned char smem_att[];
    using L = SdpaMmaLayout<HD>;
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int NT = FK_SDPA_CW * 32, KS = HD / 16, KV4 = HD / 32;      // k16 steps over head_dim; uint4 per lane per key row
    const int G = a.n_q / a.n_kv, kvh = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rank = (int)cluster.block_rank(), CL = (int)cluster.num_blocks();
    const int stride = HD + 2;
    unsigned char *qs = smem_att + L::q();
    unsigned char *vt = smem_att + L::tiles() + wid * L::WTILE;                  // this warp's tile
    float *cpart = reinterpret_cast<float *>(smem_att + L::cpart());          // [G][HD+2], read by the other CTAs of the cluster
    float *wexp = reinterpret_cast<float *>(smem_att + L::wexp(G));           // [CW][G]
    sd_stamp(a.tl, 0);
    pdl_launch_dependents();
    auto started = cluster.barrier_arrive();     // waited for before the first remote store: every CTA of the cluster is running by then
    const uint32_t pos = (a.pos_override >= 0 ? (uint32_t)a.pos_override : st->offset) + (a.consecutive ? blockIdx.z : 0u);
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    const int kpc = ((kv_len + CL * FK_SDPA_MK - 1) / (CL * FK_SDPA_MK)) * FK_SDPA_MK;
    const int k_begin = rank * kpc, k_end = min(kv_len, k_begin + kpc);
    const size_t row = blockIdx.z, seq = a.consecutive ? 0 : row;     // row of a batch: its own q and output; sequence: its own cache
    a.q += row * (size_t)a.n_q * HD; a.out += row * (size_t)a.n_q * HD;
    const uint16_t *K = a.ck + (seq * a.n_kv + kvh) * (size_t)a.capacity * HD, *V = a.cv + (seq * a.n_kv + kvh) * (size_t)a.capacity * HD;
    if (tid == 0 && k_begin < k_end && a.rows <= 1) {           // every row but the newest predates the QKV kernel in flight: warm L2 meanwhile (one sequence: its cache fits L2)
        const uint32_t bytes = (uint32_t)(k_end - k_begin) * HD * 2;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(K + (size_t)k_begin * HD), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(V + (size_t)k_begin * HD), "r"(bytes) : "memory");
    }
    // K rows of both 8-key halves are requested together up to head_dim 128 (one round trip), one half at a time above
    constexpr bool QREG = HD <= 128;
    constexpr int NKR = QREG ? 2 : 1;
    uint4 kr[NKR][KV4];
    auto load_v_tile = [&](int kb) {             // V rows of a 16-key block into this warp's tile (rows past the end are zero)
#pragma unroll
        for (int i = 0; i < FK_SDPA_MK * (HD / 8) / 32; ++i) {
            const int idx = lane + 32 * i, row = idx / (HD / 8), c = idx - row * (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (kb + row < k_end) v = __ldcg(reinterpret_cast<const uint4 *>(V + (size_t)(kb + row) * HD) + c);
            *reinterpret_cast<uint4 *>(vt + row * L::VSTRIDE + c * 16) = v;
        }
    };
    // the same tile by asynchronous copies (no registers, nothing waits until cp.async.wait_all): rows past the end are zero-filled
    auto load_v_tile_async = [&](int kb) {
#pragma unroll
        for (int i = 0; i < FK_SDPA_MK * (HD / 8) / 32; ++i) {
            const int idx = lane + 32 * i, row = idx / (HD / 8), c = idx - row * (HD / 8);
            const bool in = kb + row < k_end;
            const uint4 *src = reinterpret_cast<const uint4 *>(V + (size_t)(in ? kb + row : k_begin) * HD) + c;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(vt + row * L::VSTRIDE + c * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
        }
    };
    auto load_k = [&](int kb, int nb, int slot) {
        const int key = min(kb + 8 * nb + g, k_end - 1);                  // clamped: masked below
        const uint4 *kp = reinterpret_cast<const uint4 *>(K + (size_t)key * HD + t * (HD / 4));
#pragma unroll
        for (int c = 0; c < KV4; ++c) kr[slot][c] = __ldcg(kp + c);
    };
    // The warp's first key block is fetched before the dependency wait: every cache row but the one of the token being
    // decoded was written by earlier tokens.  The block that holds that newest row is fetched again after the wait.
    const int kb0 = k_begin + wid * FK_SDPA_MK;
    const int newest = (int)(pos % (uint32_t)a.capacity);
    const bool pre = QREG && kb0 < k_end && !a.consecutive;      // several new rows in one cache: nothing is fetched early
    // Nothing here may wait for the early fetch: the V tile goes by asynchronous copies, the K rows stay unread in registers, so
    // the wait for the previous kernel and the round trip for q run under the same memory latency instead of after it.
    if (pre) { load_v_tile_async(kb0); load_k(kb0, 0, 0); load_k(kb0, 1, NKR - 1); }
    pdl_wait();
    if (pre && newest >= kb0 && newest < kb0 + FK_SDPA_MK) {
        asm volatile("cp.async.wait_all;" ::: "memory");          // the stale copy of the newest row must have landed before it is overwritten
        load_v_tile_async(kb0); load_k(kb0, 0, 0); load_k(kb0, 1, NKR - 1);
    }
    for (int i = tid; i < G * HD / 2; i += NT) {             // q as bf16 rows
        const int gg = (2 * i) / HD, d = 2 * i - gg * HD;
        *reinterpret_cast<uint32_t *>(qs + gg * L::QSTRIDE + d * 2) = __ldcg(reinterpret_cast<const uint32_t *>(a.q + kvh * G * HD) + i);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    sd_stamp(a.tl, 1);
    // A fragments of q: row g (rows >= G and 8..15 are zero); in registers up to head_dim 128, re-read from shared memory above
    uint32_t aq[QREG ? KS : 1][2];
    const uint32_t *qrow = reinterpret_cast<const uint32_t *>(qs + g * L::QSTRIDE + t * (HD / 2));      // the lane's HD/4 dims are contiguous
    if (QREG) {
#pragma unroll
        for (int s = 0; s < (QREG ? KS : 1); ++s) { aq[s][0] = g < G ? qrow[2 * s] : 0u; aq[s][1] = g < G ? qrow[2 * s + 1] : 0u; }
    }
    float m = -INFINITY, l = 0.0f, oacc[KS][4];
#pragma unroll
    for (int mb = 0; mb < KS; ++mb) { oacc[mb][0] = oacc[mb][1] = oacc[mb][2] = oacc[mb][3] = 0.0f; }
    for (int kb = kb0; kb < k_end; kb += FK_SDPA_CW * FK_SDPA_MK) {
        // V goes by asynchronous copies and is waited for only where it is needed (after the scores): the K rows, the scores and
        // the softmax run under its latency.  (With a synchronous tile store in front, every iteration paid two memory round trips
        // in a row: 69 us per layer for 16 sequences at context 4096.)
        if (!(pre && kb == kb0)) {
            load_v_tile_async(kb);
            if (QREG) { load_k(kb, 0, 0); load_k(kb, 1, NKR - 1); }
        }
        float sacc[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            if (!QREG) load_k(kb, nb, 0);
            sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.0f;
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                const uint4 q4 = kr[QREG ? nb : 0][s >> 1];
                const uint32_t w0 = (s & 1) ? q4.z : q4.x, w1 = (s & 1) ? q4.w : q4.y;
                uint32_t x0, x1;
                if (QREG) { x0 = aq[QREG ? s : 0][0]; x1 = aq[QREG ? s : 0][1]; }
                else { x0 = g < G ? qrow[2 * s] : 0u; x1 = g < G ? qrow[2 * s + 1] : 0u; }
                mma_bf16_f32(sacc[nb], x0, 0u, x1, 0u, w0, w1);
            }
        }
        // lane (g, t): scores of head g for keys kb + {2t, 2t+1, 8+2t, 9+2t}
        float sv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = kb + (i >> 1) * 8 + 2 * t + (i & 1);
            sv[i] = key < k_end ? sacc[i >> 1][i & 1] * a.scale : -INFINITY;
        }
        float mb4 = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
        mb4 = fmaxf(mb4, __shfl_xor_sync(0xffffffffu, mb4, 1)); mb4 = fmaxf(mb4, __shfl_xor_sync(0xffffffffu, mb4, 2));
        const float mn = fmaxf(m, mb4);                                       // finite: the block holds a valid key
        const float alpha = expf(m - mn);
        float p[4], ls = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { p[i] = sv[i] == -INFINITY ? 0.0f : expf(sv[i] - mn); ls += p[i]; }
        ls += __shfl_xor_sync(0xffffffffu, ls, 1); ls += __shfl_xor_sync(0xffffffffu, ls, 2);
        l = fmaf(l, alpha, ls); m = mn;
        // the O^T accumulators of this lane belong to heads 2t and 2t+1
        const float al0 = __shfl_sync(0xffffffffu, alpha, (2 * t) * 4), al1 = __shfl_sync(0xffffffffu, alpha, (2 * t + 1) * 4);
#pragma unroll
        for (int mb = 0; mb < KS; ++mb) { oacc[mb][0] *= al0; oacc[mb][1] *= al1; oacc[mb][2] *= al0; oacc[mb][3] *= al1; }
        // P^T as the B operand (k = key, n = head): hi + lo bf16 terms of p
        const uint32_t ph0 = pack_bf16(p[0], p[1]), ph1 = pack_bf16(p[2], p[3]);
        const uint32_t pl0 = pack_bf16(p[0] - bf_lo(ph0), p[1] - bf_hi(ph0)), pl1 = pack_bf16(p[2] - bf_lo(ph1), p[3] - bf_hi(ph1));
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncwarp();                                                         // the tile is written
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
        __syncwarp();                                                         // before the next block overwrites the tile
    }
    sd_stamp(a.tl, 2);
    // the warp's partial (m, l, o[HD]) per head goes where its tile was
    float *wp = reinterpret_cast<float *>(vt);
    if (t == 0 && g < G) { wp[g * stride] = m; wp[g * stride + 1] = l; }
#pragma unroll
    for (int mb = 0; mb < KS; ++mb) {
        const int h0 = 2 * t, h1 = 2 * t + 1, d = 16 * mb + g;
        if (h0 < G) { wp[h0 * stride + 2 + d] = oacc[mb][0]; wp[h0 * stride + 2 + d + 8] = oacc[mb][2]; }
        if (h1 < G) { wp[h1 * stride + 2 + d] = oacc[mb][1]; wp[h1 * stride + 2 + d + 8] = oacc[mb][3]; }
    }
    __syncthreads();
    // Fold the warps of this CTA and push the result to the CTA that owns the output: CTA r of the cluster writes outputs
    // [r * per, (r + 1) * per) and receives, from every CTA, that slice of o plus (m, l) of every head (distributed shared
    // memory stores).  One cluster barrier, then a local fold; nobody reads remote memory afterwards, so a CTA may exit as
    // soon as its own outputs are written.
    const unsigned char *tiles = smem_att + L::tiles();
    const int nwp = min(FK_SDPA_CW, max(0, (k_end - k_begin + FK_SDPA_MK - 1) / FK_SDPA_MK));        // warps that saw keys
    const int total = G * HD, per = (total + CL - 1) / CL;
    float *recv_o = cpart;                                   // [CL][per]
    float *recv_ml = wexp;                                   // [CL][G][2]
    // the factors exp(m_w - M) depend on (warp, head) only: one thread per pair computes them once, the element loop below is
    // then multiply-adds (an expf per element and source made the two folds the longest phases of the kernel at short contexts)
    float *fexp = reinterpret_cast<float *>(smem_att + L::fexp(G));          // [16][G], then M[G], then 1 / l [G]
    float *fmax = fexp + 16 * G;
    if (tid < nwp * G) {
        const int w = tid / G, gg = tid - w * G;
        float M = -INFINITY;
        for (int w2 = 0; w2 < nwp; ++w2) M = fmaxf(M, reinterpret_cast<const float *>(tiles + w2 * L::WTILE)[gg * stride]);
        const float mw = reinterpret_cast<const float *>(tiles + w * L::WTILE)[gg * stride];
        fexp[w * G + gg] = mw == -INFINITY ? 0.0f : expf(mw - M);
        if (w == 0) fmax[gg] = M;
    }
    if (nwp == 0 && tid < G) fmax[tid] = -INFINITY;
    __syncthreads();
    cluster.barrier_wait(std::move(started));
    for (int i = tid; i < total + G; i += NT) {              // i >= total: the (m, l) pair of head i - total
        const int gg = i < total ? i / HD : i - total, d = i < total ? i - gg * HD : -1;
        float acc = 0.0f;
        for (int w = 0; w < nwp; ++w) {
            const float *pw = reinterpret_cast<const float *>(tiles + w * L::WTILE) + gg * stride;
            acc = fmaf(d < 0 ? pw[1] : pw[2 + d], fexp[w * G + gg], acc);
        }
        if (d >= 0) {
            const int dst = i / per;
            cluster.map_shared_rank(recv_o, dst)[rank * per + (i - dst * per)] = acc;
        } else {
            const float M = fmax[gg];
            for (int dst = 0; dst < CL; ++dst) { float *q2 = cluster.map_shared_rank(recv_ml, dst) + (rank * G + gg) * 2; q2[0] = M; q2[1] = acc; }
        }
    }
    sd_stamp(a.tl, 3);
    cluster.sync();
    sd_stamp(a.tl, 4);
    if (tid < CL * G) {                                      // factor of (source CTA, head), once
        const int rr = tid / G, gg = tid - rr * G;
        float M = -INFINITY;
        for (int r2 = 0; r2 < CL; ++r2) M = fmaxf(M, recv_ml[(r2 * G + gg) * 2]);
        const float mr = recv_ml[(rr * G + gg) * 2];
        fexp[rr * G + gg] = mr == -INFINITY ? 0.0f : expf(mr - M);
    }
    __syncthreads();
    if (tid < G) {
        float Ls = 0.0f;
        for (int rr = 0; rr < CL; ++rr) Ls = fmaf(recv_ml[(rr * G + tid) * 2 + 1], fexp[rr * G + tid], Ls);
        fmax[G + tid] = __fdiv_rn(1.0f, Ls);
    }
    __syncthreads();
    for (int il = tid; il < per; il += NT) {
        const int i = rank * per + il;
        if (i >= total) break;
        const int gg = i / HD, d = i - gg * HD;
        float O = 0.0f;
        for (int rr = 0; rr < CL; ++rr) O = fmaf(recv_o[rr * per + il], fexp[rr * G + gg], O);
        a.out[(kvh * G + gg) * HD + d] = f2bf(O * fmax[G + gg]);
    }
    sd_stamp(a.tl, 6);
}

// ---------------------------------------------------------------- peer-memory all-reduce (tensor parallel, one process per GPU)
// The row-split projections of a tensor-parallel layer end in an all-reduce of one hidden vector (10-32 KB); a library
// all-reduce costs ~23 us of latency for that, 129 times per token.  Here every rank owns an arena that its peers map
// through CUDA IPC: a rank stores its partial into its slot of every peer's arena (plain peer stores over NVLink), then a
// flag per (source rank, block); each rank polls its own arena only and sums the slots in rank order, so all ranks get
// bit-identical results.  Slots and flags alternate by the parity of a per-block sequence number: a rank can be at most
// one all-reduce ahead of a peer, because it needs that peer's push to finish the one in between.  Waits are bounded.
template <typename T, bool IS_MAX>
__global__ void __launch_bounds__(256) k_allreduce_peer(T *buf, int n, PeerMap P, FkState *st) {
    __shared__ unsigned int seq_s; __shared__ int bad;
    pdl_wait();                                  // buf is the previous kernel's output
    unsigned char *own = P.base[P.rank];
    const int b = blockIdx.x, nb = gridDim.x;
    if (threadIdx.x == 0) {
        unsigned int *cnt = reinterpret_cast<unsigned int *>(own + PeerArena::counter(b));
        seq_s = *cnt + 1u; *cnt = seq_s; bad = 0;
    }
    __syncthreads();
    const unsigned int seq = seq_s; const int par = (int)(seq & 1u);
    const int per = (n + nb - 1) / nb, lo = b * per, hi = min(n, lo + per);
    // 1. my slice into my slot of every rank's arena (my own included)
    for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) {
        const T v = buf[i];
        for (int p = 0; p < P.world; ++p) reinterpret_cast<T *>(P.base[p] + PeerArena::slot(par, P.rank))[i] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();       // one fence per block orders all of the block's peer stores
    __syncthreads();
    // 2. tell every rank that slice b of this rank is in; 3. wait for slice b of every rank
    if ((int)threadIdx.x < P.world) {
        const int p = (int)threadIdx.x;
        unsigned int *remote = reinterpret_cast<unsigned int *>(P.base[p] + PeerArena::flag(par, P.rank, b));
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(seq) : "memory");
        const unsigned int *mine = reinterpret_cast<const unsigned int *>(own + PeerArena::flag(par, p, b));
        unsigned int it = 0, v;
        do {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        } while ((int)(v - seq) < 0 && ++it < P.spin_limit);
        if ((int)(v - seq) < 0) { bad = 1; atomicOr(&st->error, 0x8000u); }
    }
    __syncthreads();
    if (bad) return;
    // 4. the slots in rank order
    for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) {
        T acc = __ldcg(reinterpret_cast<const T *>(own + PeerArena::slot(par, 0)) + i);
        for (int p = 1; p < P.world; ++p) {
            const T v = __ldcg(reinterpret_cast<const T *>(own + PeerArena::slot(par, p)) + i);
            acc = IS_MAX ? (v > acc ? v : acc) : (T)(acc + v);
        }
        buf[i] = acc;
    }
}

struct LinArgs { const uint16_t *x; WView W; const uint16_t *residual; uint16_t *y; float *y_f32; int k, n; };
// y = T(acc + float(residual)), one rounding (src/codegen/msl.rs:2759-2775); residual optional
template <int BITS>
__global__ void __launch_bounds__(256) k_linear_residual(const FkState *st, LinArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.k);
    pdl_wait(); pdl_launch_dependents();
    stage_x(sm, a.x, a.k);
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
    for (int r = gw; r < a.n; r += nw) {
        float acc = warp_dot<BITS>(a.W, r, sm, lane);
        if (lane != 0) continue;
        if (a.y_f32) a.y_f32[r] = acc;
        if (a.residual) acc += bf2f(a.residual[r]);
        if (a.y) a.y[r] = f2bf(acc);
    }
}

struct GateUpArgs {
    const uint16_t *x, *norm_w; WView Wg, Wu; uint16_t *act_out;
    const uint16_t *pending, *pending_w; uint16_t *h_out;
    int h, inter, act; float eps;
};
// RMSNorm -> gate & up matvec -> activation tail in registers, only the activation is written
// (src/codegen/kernels/fused_chain.rs:2902-3552; qmv_swiglu.rs:20-246)
template <int BITS>
__global__ void __launch_bounds__(256) k_rmsnorm_gateup_act(const FkState *st, GateUpArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.h);
    pdl_wait(); pdl_launch_dependents();
    stage_norm(sm, a.x, a.norm_w, a.h, a.eps, a.pending, a.pending_w, a.h_out);
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
    for (int r = gw; r < a.inter; r += nw) {
        const float g = warp_dot<BITS>(a.Wg, r, sm, lane);
        const float u = warp_dot<BITS>(a.Wu, r, sm, lane);
        if (lane == 0) a.act_out[r] = a.act == 1 ? act_geglu_tanh(g, u) : act_swiglu(g, u);
    }
}

struct HeadArgs {
    const uint16_t *x, *norm_w; WView W; uint16_t *logits; unsigned long long *scratch; uint32_t *counter;
    const uint16_t *pending, *pending_w; uint16_t *h_out; uint32_t *history;
    int h, v, vocab_offset, finalize; float eps;
};
// advance the device-side decode state after the argmax (argmax_logits_finalize.rs:97-105 history
// append; kernels/mod.rs:542-579 offset advance; next_token_out aliases token_id_in)
__device__ __forceinline__ void finalize_token(FkState *st, uint32_t *history, unsigned long long best) {
    const uint32_t next = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
    st->token[0] = next;
    if (history && st->hist_counter < st->hist_cap) history[st->hist_counter] = next;
    st->hist_counter += 1;
    st->offset += 1;
    st->epoch += 1;
}
// final RMSNorm -> lm_head matvec -> argmax without a logits round trip: values are rounded to T
// before the compare and ties go to the lowest index (final_rmsnorm_lm_head.rs:250-326;
// msl.rs:1805-1838).  Per-block best keys land in `scratch`; the last block folds them.
template <int BITS>
__global__ void __launch_bounds__(256) k_final_head(FkState *st, HeadArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.h);
    __shared__ unsigned long long wbest[8]; __shared__ int is_last;
    pdl_wait(); pdl_launch_dependents();
    stage_norm(sm, a.x, a.norm_w, a.h, a.eps, a.pending, a.pending_w, a.h_out);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int gw = blockIdx.x * (blockDim.x >> 5) + wid, nw = gridDim.x * (blockDim.x >> 5);
    unsigned long long best = 0ull;
    for (int r = gw; r < a.v; r += nw) {
        const float acc = warp_dot<BITS>(a.W, r, sm, lane);
        const uint16_t t = f2bf(acc);
        if (lane == 0 && a.logits) a.logits[r] = t;
        const unsigned long long key = argmax_key(t, (uint32_t)(r + a.vocab_offset));
        best = key > best ? key : best;
    }
    if (lane == 0) wbest[wid] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = wbest[i] > best ? wbest[i] : best;
        a.scratch[blockIdx.x] = best;
        __threadfence();
        const uint32_t t = atomicAdd(a.counter, 1u);
        is_last = (t == gridDim.x - 1);
        if (is_last) *a.counter = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (wid == 0) {
        unsigned long long b = 0ull;
        for (int i = lane; i < (int)gridDim.x; i += 32) { const unsigned long long v = __ldcg(a.scratch + i); b = v > b ? v : b; }
        b = warp_max_u64(b);
        if (lane == 0) {
            if (a.finalize) finalize_token(st, a.history, b);
            else a.scratch[0] = b;      // vocab-sharded head: the rank's best key, folded across ranks next
        }
    }
}

// fold `entries` per-block (or per-rank) keys and advance the state (argmax_logits_finalize.rs:68-105)
__global__ void k_argmax_finalize(FkState *st, const unsigned long long *scratch, int entries, uint32_t *history) {
    pdl_wait(); pdl_launch_dependents();
    unsigned long long b = 0ull;
    for (int i = threadIdx.x; i < entries; i += 32) { const unsigned long long v = scratch[i]; b = v > b ? v : b; }
    b = warp_max_u64(b);
    if (threadIdx.x == 0) finalize_token(st, history, b);
}

// y = T(sum + float(residual)) after a tensor-parallel all-reduce
__global__ void k_residual_add(const float *sum, const uint16_t *residual, uint16_t *y, int n) {
    pdl_wait(); pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = f2bf(sum[i] + (residual ? bf2f(residual[i]) : 0.0f));
}

// ---------------------------------------------------------------- several independent sequences per step (batch decode)
// The reference never batches independent sequences (python/fusekit_runtime/dispatch.py:2268-2289): its M > 1 kernels serve
// consecutive positions of one sequence.  Here row m of every tensor belongs to sequence m, all sequences sit at the same
// position, and each has its own KV cache; the result of row m is what the one-row path gives for that sequence alone.
struct NormRowsArgs { const uint16_t *x, *w; uint16_t *y; int h, rows; float eps; };
// y[m, :] = T(w * T(x[m, :] * r_m)), r_m = 1 / sqrt(mean(x[m]^2) + eps): the two roundings of the fused kernels
// (src/codegen/kernels/mod.rs:4464-4472), one block per row
__global__ void __launch_bounds__(1024) k_rmsnorm_rows(const FkState *st, NormRowsArgs a) {
    __shared__ float red[40];
    pdl_wait(); pdl_launch_dependents();
    const uint16_t *x = a.x + (size_t)blockIdx.x * a.h; uint16_t *y = a.y + (size_t)blockIdx.x * a.h;
    // eight values per thread and round in registers between the two passes (h a multiple of 8: the rows are 16-byte aligned)
    const int nv = a.h / 8;
    uint4 keep = make_uint4(0, 0, 0, 0);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(x) + i);
        if (i == (int)threadIdx.x) keep = v;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float lo = bf_lo(w[j]), hi = bf_hi(w[j]); ss = fmaf(lo, lo, ss); ss = fmaf(hi, hi, ss); }
    }
    for (int i = nv * 8 + threadIdx.x; i < a.h; i += blockDim.x) { const float v = bf2f(__ldcg(x + i)); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.h), a.eps)));
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const uint4 v = i == (int)threadIdx.x ? keep : __ldcg(reinterpret_cast<const uint4 *>(x) + i);
        const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(a.w) + i);
        const uint32_t xs[4] = {v.x, v.y, v.z, v.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf_lo(ws[j]) * rT(bf_lo(xs[j]) * r), bf_hi(ws[j]) * rT(bf_hi(xs[j]) * r));
        reinterpret_cast<uint4 *>(y)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (int i = nv * 8 + threadIdx.x; i < a.h; i += blockDim.x) y[i] = f2bf(bf2f(a.w[i]) * rT(bf2f(__ldcg(x + i)) * r));
}
struct RopeRowsArgs { const uint16_t *qkv; uint16_t *q_out, *cache_k, *cache_v; int n_q, n_kv, hd, capacity, rows; float log2theta; int consecutive; };
// RoPE on the q and k heads of every sequence's raw projection row (q | k | v, bias already added), k and v into that
// sequence's cache row of the current position (src/codegen/kernels/rmsnorm_qkv.rs:635-697): block (head, sequence)
__global__ void k_rope_store_rows(const FkState *st, RopeRowsArgs a) {
    pdl_wait(); pdl_launch_dependents();
    const int head = blockIdx.x, m = blockIdx.y, d = threadIdx.x, half = a.hd >> 1;
    // independent sequences share the position and have a cache each; consecutive rows of one sequence share the cache
    const uint32_t pos = st->offset + (a.consecutive ? (uint32_t)m : 0u); const int wrow = (int)(pos % (uint32_t)a.capacity);
    const size_t seq = a.consecutive ? 0 : (size_t)m;
    const int nrow = (a.n_q + 2 * a.n_kv) * a.hd;
    const uint16_t *src = a.qkv + (size_t)m * nrow + (size_t)head * a.hd;
    if (d >= half) return;
    if (head < a.n_q + a.n_kv) {
        uint16_t o0, o1; rope_pair(bf2f(src[d]), bf2f(src[d + half]), d, half, pos, a.log2theta, &o0, &o1);
        uint16_t *dst = head < a.n_q ? a.q_out + ((size_t)m * a.n_q + head) * a.hd
                                     : a.cache_k + ((seq * a.n_kv + (head - a.n_q)) * a.capacity + wrow) * a.hd;
        dst[d] = o0; dst[d + half] = o1;
    } else {
        uint16_t *dst = a.cache_v + ((seq * a.n_kv + (head - a.n_q - a.n_kv)) * a.capacity + wrow) * a.hd;
        dst[d] = src[d]; dst[d + half] = src[d + half];
    }
}
struct ArgmaxRowsArgs { const uint16_t *logits; uint32_t *counter, *history; int v, rows, advance; };
// greedy token of every sequence from its T-rounded logits, ties to the lowest index (argmax_logits_scan.rs:83-124); the
// block that finishes last advances the shared position.  history[step * rows + m] receives sequence m's token.
__global__ void __launch_bounds__(1024) k_argmax_rows(FkState *st, ArgmaxRowsArgs a) {
    __shared__ unsigned long long wbest[32];
    pdl_wait(); pdl_launch_dependents();
    const int m = blockIdx.x, lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const uint16_t *lg = a.logits + (size_t)m * a.v;
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < a.v; i += blockDim.x) { const unsigned long long key = argmax_key(__ldcg(lg + i), (uint32_t)i); best = key > best ? key : best; }
    best = warp_max_u64(best);
    if (lane == 0) wbest[wid] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = wbest[i] > best ? wbest[i] : best;
        const uint32_t next = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
        st->token[m] = next;
        const uint32_t step = st->hist_counter;
        if (a.history && (step + 1) * (uint32_t)a.rows <= st->hist_cap) a.history[step * a.rows + m] = next;
        __threadfence();
        if (atomicAdd(a.counter, 1u) == (uint32_t)a.rows - 1u) { *a.counter = 0u; st->hist_counter = step + 1; st->offset += (uint32_t)a.advance; st->epoch += 1; }
    }
}

// smoke kernel: out = T(float(a) + float(b)) (metal/elementwise.metal:11-20 elementwise_add_bf16)
__global__ void k_add_bf16(const uint16_t *a, const uint16_t *b, uint16_t *out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}
