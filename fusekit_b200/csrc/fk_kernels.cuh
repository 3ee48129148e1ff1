// Decode kernels, generic-shape edition: one warp per output row (or row pair), 128-bit weight
// loads, in-register dequant with the group-factored form  s * sum(x*q) + b * sum(x), fp32
// accumulation, warp-shuffle reduction.  These are the parity baseline and the fallback for
// shapes the streamed kernels (fk_stream.cuh) do not take.
#pragma once
#include "fk_common.cuh"

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
struct EmbedArgs { const uint16_t *table; uint16_t *x; int h, rows; float scale; };
// x[row,:] = T(embed[token[row],:] * scale) (src/codegen/kernels/embed_lookup_decode.rs:95-98)
__global__ void k_embed_lookup(const FkState *st, EmbedArgs a) {
    pdl_launch_dependents(); pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.h * a.rows) return;
    const int row = i / a.h, d = i - row * a.h;
    a.x[i] = f2bf(__fmul_rn(bf2f(a.table[(size_t)st->token[row] * a.h + d]), a.scale));
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
    pdl_launch_dependents(); pdl_wait();
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

struct SdpaArgs {
    const uint16_t *q, *ck, *cv; uint16_t *out; float *part; uint32_t *counter;
    int n_q, n_kv, hd, capacity, chunk; float scale;
};
#define FK_SDPA_KEYS 64        // keys per block (the reference's BLOCK, sdpa_decode.rs:35-55)
#define FK_SDPA_MAXG 8         // q heads sharing one kv head
// Split-K GQA decode attention.  Block (chunk, kv head) scores 64 keys against every q head of the
// group, so K/V are read once per group: s = dot(q,k)*scale, partial (m, l, o[hd]) in fp32
// (sdpa_decode.rs:697-715).  The last block of a kv head to finish merges the chunks and writes
// T(o * (1/l)) (sdpa_decode.rs:992-1046) -- a ticket counter, no waiting.  kv_len = min(pos+1, capacity).
__global__ void k_sdpa_decode(const FkState *st, SdpaArgs a) {
    extern __shared__ float sm[];
    const int G = a.n_q / a.n_kv, hd = a.hd, kvh = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
    float *qs = sm;                        // [G][hd]
    float *sc = qs + G * hd;               // [G][64]
    float *ml = sc + G * FK_SDPA_KEYS;     // [G][2]
    __shared__ int is_last;
    pdl_launch_dependents(); pdl_wait();
    const uint32_t pos = st->offset;
    const int kv_len = (int)min(pos + 1u, (uint32_t)a.capacity);
    const int n_active = (kv_len + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS;
    if (chunk >= n_active) return;
    const int k0 = chunk * FK_SDPA_KEYS, bs = min(FK_SDPA_KEYS, kv_len - k0);
    for (int i = tid; i < G * hd; i += blockDim.x) qs[i] = bf2f(a.q[kvh * G * hd + i]);
    __syncthreads();
    const uint16_t *K = a.ck + ((size_t)kvh * a.capacity + k0) * hd, *V = a.cv + ((size_t)kvh * a.capacity + k0) * hd;
    if (tid < bs) {
        float dot[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) dot[g] = 0.0f;
        const uint4 *kr = reinterpret_cast<const uint4 *>(K + (size_t)tid * hd);
        for (int c = 0; c < (hd >> 3); ++c) {
            const uint4 v = __ldg(kr + c);
            const float kf[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
#pragma unroll
            for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) {
#pragma unroll
                for (int j = 0; j < 8; ++j) dot[g] = fmaf(qs[g * hd + c * 8 + j], kf[j], dot[g]);
            }
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) sc[g * FK_SDPA_KEYS + tid] = dot[g] * a.scale;
    }
    __syncthreads();
    const int lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
    for (int g = wid; g < G; g += nw) {
        const float s0 = lane < bs ? sc[g * FK_SDPA_KEYS + lane] : -INFINITY;
        const float s1 = lane + 32 < bs ? sc[g * FK_SDPA_KEYS + lane + 32] : -INFINITY;
        const float m = warp_max(fmaxf(s0, s1));
        const float p0 = lane < bs ? expf(s0 - m) : 0.0f, p1 = lane + 32 < bs ? expf(s1 - m) : 0.0f;
        sc[g * FK_SDPA_KEYS + lane] = p0; sc[g * FK_SDPA_KEYS + lane + 32] = p1;
        const float l = warp_sum(p0 + p1);
        if (lane == 0) { ml[2 * g] = m; ml[2 * g + 1] = l; }
    }
    __syncthreads();
    const int stride = hd + 2;
    if (tid < hd) {
        float o[FK_SDPA_MAXG];
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) o[g] = 0.0f;
        for (int i = 0; i < bs; ++i) {
            const float v = bf2f(__ldg(V + (size_t)i * hd + tid));
#pragma unroll
            for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) o[g] = fmaf(sc[g * FK_SDPA_KEYS + i], v, o[g]);
        }
#pragma unroll
        for (int g = 0; g < FK_SDPA_MAXG; ++g) if (g < G) {
            float *p = a.part + ((size_t)(kvh * G + g) * a.chunk + chunk) * stride;
            p[2 + tid] = o[g];
            if (tid == 0) { p[0] = ml[2 * g]; p[1] = ml[2 * g + 1]; }
        }
    }
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
    if (tid < hd) {
        for (int g = 0; g < G; ++g) {
            const float *p = a.part + (size_t)(kvh * G + g) * a.chunk * stride;
            float M = -INFINITY;
            for (int c = 0; c < n_active; ++c) M = fmaxf(M, __ldcg(p + (size_t)c * stride));
            float L = 0.0f, O = 0.0f;
            for (int c = 0; c < n_active; ++c) {
                const float w = expf(__ldcg(p + (size_t)c * stride) - M);
                L = fmaf(__ldcg(p + (size_t)c * stride + 1), w, L);
                O = fmaf(__ldcg(p + (size_t)c * stride + 2 + tid), w, O);
            }
            a.out[(kvh * G + g) * hd + tid] = f2bf(O * __fdiv_rn(1.0f, L));
        }
    }
}

struct LinArgs { const uint16_t *x; WView W; const uint16_t *residual; uint16_t *y; float *y_f32; int k, n; };
// y = T(acc + float(residual)), one rounding (src/codegen/msl.rs:2759-2775); residual optional
template <int BITS>
__global__ void __launch_bounds__(256) k_linear_residual(const FkState *st, LinArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.k);
    pdl_launch_dependents(); pdl_wait();
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
    pdl_launch_dependents(); pdl_wait();
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
}
// final RMSNorm -> lm_head matvec -> argmax without a logits round trip: values are rounded to T
// before the compare and ties go to the lowest index (final_rmsnorm_lm_head.rs:250-326;
// msl.rs:1805-1838).  Per-block best keys land in `scratch`; the last block folds them.
template <int BITS>
__global__ void __launch_bounds__(256) k_final_head(FkState *st, HeadArgs a) {
    extern __shared__ float smem_raw[];
    const Smem sm = carve(smem_raw, a.h);
    __shared__ unsigned long long wbest[8]; __shared__ int is_last;
    pdl_launch_dependents(); pdl_wait();
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
    pdl_launch_dependents(); pdl_wait();
    unsigned long long b = 0ull;
    for (int i = threadIdx.x; i < entries; i += 32) { const unsigned long long v = scratch[i]; b = v > b ? v : b; }
    b = warp_max_u64(b);
    if (threadIdx.x == 0) finalize_token(st, history, b);
}

// y = T(sum + float(residual)) after a tensor-parallel all-reduce
__global__ void k_residual_add(const float *sum, const uint16_t *residual, uint16_t *y, int n) {
    pdl_launch_dependents(); pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = f2bf(sum[i] + (residual ? bf2f(residual[i]) : 0.0f));
}

// smoke kernel: out = T(float(a) + float(b)) (metal/elementwise.metal:11-20 elementwise_add_bf16)
__global__ void k_add_bf16(const uint16_t *a, const uint16_t *b, uint16_t *out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(bf2f(a[i]) + bf2f(b[i]));
}
