/*
 * fk_oracle.c -- CPU restatement of FuseKit's fused-decode kernel math.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker (and the timed CPU
 * baseline) for the CUDA decode path; nothing in the shipped library links,
 * imports or calls it.  PARITY UNPINNED: the reference repository holds no
 * golden vectors, known-answer tests or numeric fixtures for this path (its
 * unit tests assert IR structure and emitted text only) and neither its
 * Metal kernels nor MLX can run on Linux, so this restatement is anchored on
 * the reference's emitter sources alone.  Each function cites the reference
 * file:line it follows (paths are relative to the FuseKit source tree).
 *
 * Conventions: T = bf16 (round-to-nearest-even), all arithmetic inside a
 * "kernel" is fp32, libm supplies exp/cos/sin/tanh (the reference's Metal
 * fast:: intrinsics are not reproduced), summation order is fixed (16
 * interleaved partial sums, then a sequential fold) so results do not depend
 * on compiler or thread count.  Build with -ffp-contract=off.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef uint16_t bf16_t;

/* ------------------------------------------------------------------ bf16 */
static inline float bf2f(bf16_t h) {
    uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}
static inline bf16_t f2bf(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (bf16_t)(u >> 16);
}
static inline float rT(float f) { return bf2f(f2bf(f)); }

float fko_bf16_to_f32(uint16_t h) { return bf2f(h); }
uint16_t fko_f32_to_bf16(float f) { return f2bf(f); }

/* --------------------------------------------- counter-based data source
 * Integer-only so a GPU generator can reproduce it bit for bit: a splitmix64
 * finaliser over (stream, index, lane), twelve 16-bit uniforms summed
 * (Irwin-Hall) to a unit-variance near-normal deviate.                    */
static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline uint64_t draw64(uint64_t stream, uint64_t idx, uint64_t lane) {
    return mix64(mix64(stream ^ (idx * 0xD1342543DE82EF95ull)) + lane);
}
static inline float unit_normal(uint64_t stream, uint64_t idx) {
    int32_t s = 0;
    for (uint64_t lane = 0; lane < 3; ++lane) {
        uint64_t h = draw64(stream, idx, lane);
        s += (int32_t)(h & 0xffff) + (int32_t)((h >> 16) & 0xffff)
           + (int32_t)((h >> 32) & 0xffff) + (int32_t)((h >> 48) & 0xffff);
    }
    return (float)(s - 393210) * (1.0f / 65536.0f);   /* exact in fp32 */
}
uint64_t fko_stream_id(const char *name) {            /* FNV-1a 64 */
    uint64_t h = 0xcbf29ce484222325ull;
    for (const unsigned char *p = (const unsigned char *)name; *p; ++p) {
        h ^= *p; h *= 0x100000001b3ull;
    }
    return h;
}
float fko_unit_normal(uint64_t stream, uint64_t idx) { return unit_normal(stream, idx); }
uint32_t fko_uniform_u32(uint64_t stream, uint64_t idx, uint32_t modulo) {
    return (uint32_t)(draw64(stream, idx, 0) % (uint64_t)modulo);
}

/* out[i] = T(mean + std * z(stream, idx0 + i)), product and sum rounded separately */
void fko_fill_normal_bf16(uint64_t stream, uint64_t idx0, uint64_t n, float mean, float std, bf16_t *out) {
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float v = std * unit_normal(stream, idx0 + (uint64_t)i);
        v = mean + v;
        out[i] = f2bf(v);
    }
}

/* ------------------------------------------------- MLX-affine quantizer
 * Layout follows src/fusion/ir.rs:236-247 and scripts/poc_int4_gemv.py:16-44:
 *   packed u32 [N, K*bits/32], element j of a row at bit (j % (32/bits))*bits
 *   of word j / (32/bits) (LSB first); scales, biases T [N, K/64];
 *   w = q * scale + bias.
 * Quantizer rule (the benchmark definition): per group of 64,
 *   scale = (max - min) / (2^bits - 1), bias = min, both rounded to T, and
 *   q = clamp(rint((w - bias) / scale)) computed with the rounded values.
 * The weight block is rows [row0,row0+nrows) x cols [k0,k0+kcount) of a
 * global [*, k_global] tensor w = std * z(stream, row*k_global + col).     */
void fko_gen_qweight(uint64_t stream, float std, int64_t k_global, int64_t row0, int64_t nrows,
                     int64_t k0, int64_t kcount, int bits,
                     uint32_t *packed, bf16_t *scales, bf16_t *biases) {
    const int per_word = 32 / bits;
    const int qmax = (1 << bits) - 1;
    const int64_t words = kcount / per_word, groups = kcount / 64;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < nrows; ++r) {
        float w[64];
        uint32_t *prow = packed + r * words;
        memset(prow, 0, (size_t)words * 4);
        for (int64_t g = 0; g < groups; ++g) {
            float mx = -INFINITY, mn = INFINITY;
            for (int j = 0; j < 64; ++j) {
                uint64_t idx = (uint64_t)((row0 + r) * k_global + k0 + g * 64 + j);
                w[j] = std * unit_normal(stream, idx);
                mx = w[j] > mx ? w[j] : mx; mn = w[j] < mn ? w[j] : mn;
            }
            float sc = (mx - mn) / (float)qmax;
            bf16_t sb = f2bf(sc), bb = f2bf(mn);
            float s = bf2f(sb), b = bf2f(bb);
            scales[r * groups + g] = sb; biases[r * groups + g] = bb;
            for (int j = 0; j < 64; ++j) {
                float qf = (s != 0.0f) ? rintf((w[j] - b) / s) : 0.0f;
                int q = qf < 0.0f ? 0 : (qf > (float)qmax ? qmax : (int)qf);
                int64_t e = g * 64 + j;
                prow[e / per_word] |= (uint32_t)q << ((e % per_word) * bits);
            }
        }
    }
}
/* dense T weights for the unquantized variant */
void fko_gen_dense_weight(uint64_t stream, float std, int64_t k_global, int64_t row0, int64_t nrows,
                          int64_t k0, int64_t kcount, bf16_t *out) {
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < nrows; ++r)
        for (int64_t c = 0; c < kcount; ++c)
            out[r * kcount + c] = f2bf(std * unit_normal(stream, (uint64_t)((row0 + r) * k_global + k0 + c)));
}

/* fp32 dequantised matrix; q*s is exact in fp32 so q*s+b has one rounding
 * (src/codegen/kernels/mod.rs:2850-2908 q4, :3053-3093 q8). */
void fko_dequant(const uint32_t *packed, const bf16_t *scales, const bf16_t *biases,
                 int64_t n, int64_t k, int bits, float *out) {
    const int per_word = 32 / bits; const uint32_t mask = (1u << bits) - 1u;
    const int64_t words = k / per_word, groups = k / 64;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n; ++r)
        for (int64_t c = 0; c < k; ++c) {
            uint32_t q = (packed[r * words + c / per_word] >> ((c % per_word) * bits)) & mask;
            float p = (float)q * bf2f(scales[r * groups + c / 64]);
            out[r * k + c] = p + bf2f(biases[r * groups + c / 64]);
        }
}

/* ------------------------------------------------------------ linear op */
typedef struct {
    int64_t n, k; int bits;                 /* bits 4, 8, or 16 (dense T) */
    const uint32_t *packed; const bf16_t *scales, *biases;   /* bits 4/8 */
    const bf16_t *dense;                                      /* bits 16  */
    const bf16_t *lin_bias;                                   /* optional [n] */
} fko_linear;

/* fp32 dot of row r with x (x given as fp32 values that are already T-exact).
 * acc += x[k] * (q*s+b)  (src/codegen/kernels/mod.rs:1984-2007). */
static float row_dot(const fko_linear *L, int64_t r, const float *x) {
    float part[16]; for (int i = 0; i < 16; ++i) part[i] = 0.0f;
    const int64_t k = L->k;
    if (L->bits == 16) {
        const bf16_t *w = L->dense + r * k;
        for (int64_t c = 0; c < k; c += 16)
            for (int i = 0; i < 16; ++i) { float p = x[c + i] * bf2f(w[c + i]); part[i] = part[i] + p; }
    } else {
        const int bits = L->bits, per_word = 32 / bits; const uint32_t mask = (1u << bits) - 1u;
        const int64_t words = k / per_word, groups = k / 64;
        const uint32_t *pw = L->packed + r * words;
        const bf16_t *ps = L->scales + r * groups, *pb = L->biases + r * groups;
        for (int64_t g = 0; g < groups; ++g) {
            const float s = bf2f(ps[g]), b = bf2f(pb[g]);
            for (int c = 0; c < 64; c += 16)
                for (int i = 0; i < 16; ++i) {
                    int64_t e = g * 64 + c + i;
                    uint32_t q = (pw[e / per_word] >> ((e % per_word) * bits)) & mask;
                    float wv = (float)q * s; wv = wv + b;
                    float p = x[e] * wv; part[i] = part[i] + p;
                }
        }
    }
    float acc = 0.0f; for (int i = 0; i < 16; ++i) acc = acc + part[i];
    return acc;
}

/* y[r] = T(acc + bias[r] + residual[r]); bias added in fp32 before the single
 * rounding (src/codegen/kernels/rmsnorm_qkv.rs:420-423), residual likewise
 * (src/codegen/msl.rs:2759-2775).  acc_out (optional) receives fp32 acc+bias. */
void fko_linear_apply(const fko_linear *L, const float *x, const bf16_t *residual, bf16_t *y, float *acc_out) {
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < L->n; ++r) {
        float acc = row_dot(L, r, x);
        if (L->lin_bias) acc = acc + bf2f(L->lin_bias[r]);
        if (acc_out) acc_out[r] = acc;
        if (residual) acc = acc + bf2f(residual[r]);
        if (y) y[r] = f2bf(acc);
    }
}
/* convenience for tests: x given as T */
void fko_qmatvec(const fko_linear *L, const bf16_t *x, const bf16_t *residual, bf16_t *y) {
    float *xf = (float *)malloc(sizeof(float) * (size_t)L->k);
    for (int64_t i = 0; i < L->k; ++i) xf[i] = bf2f(x[i]);
    fko_linear_apply(L, xf, residual, y, NULL);
    free(xf);
}

/* ---------------------------------------------------------------- RMSNorm
 * ss = sum x^2 (fp32), r = 1/sqrt(ss/H + eps), y = float(T(w * T(x*r))) -- two
 * roundings to T (src/codegen/kernels/mod.rs:4464-4472; rmsnorm_qkv.rs:325). */
void fko_rmsnorm(const bf16_t *x, const bf16_t *w, int64_t h, float eps, float *y) {
    float part[16]; for (int i = 0; i < 16; ++i) part[i] = 0.0f;
    int64_t c = 0;
    for (; c + 16 <= h; c += 16)
        for (int i = 0; i < 16; ++i) { float v = bf2f(x[c + i]); float p = v * v; part[i] = part[i] + p; }
    for (int i = 0; c < h; ++c, ++i) { float v = bf2f(x[c]); float p = v * v; part[i] = part[i] + p; }
    float ss = 0.0f; for (int i = 0; i < 16; ++i) ss = ss + part[i];
    float mean = ss / (float)h;
    float r = 1.0f / sqrtf(mean + eps);
    for (int64_t i = 0; i < h; ++i) {
        float t = rT(bf2f(x[i]) * r);
        y[i] = rT(bf2f(w[i]) * t);
    }
}

/* ------------------------------------------------------------------- RoPE
 * half-split pairs (d, d+hd/2): inv = exp2(-(d/half)*log2(theta)), log2(theta)
 * in f64 then cast to f32 (rmsnorm_qkv.rs:273); ang = float(pos)*inv;
 * lo' = T(lo*c - hi*s), hi' = T(hi*c + lo*s) (rmsnorm_qkv.rs:635-643;
 * rope_q_decode.rs:93-114).  In place on a T vector of n_heads*hd. */
void fko_rope(bf16_t *v, int n_heads, int hd, uint32_t pos, float theta) {
    const int half = hd / 2; const float l2t = (float)log2((double)theta);
    for (int h = 0; h < n_heads; ++h)
        for (int d = 0; d < half; ++d) {
            float e = -((float)d / (float)half); e = e * l2t;
            float inv = exp2f(e);
            float ang = (float)pos * inv;
            float c = cosf(ang), s = sinf(ang);
            float lo = bf2f(v[h * hd + d]), hi = bf2f(v[h * hd + d + half]);
            float a = lo * c, b = hi * s; float o_lo = a - b;
            float p = hi * c, q = lo * s; float o_hi = p + q;
            v[h * hd + d] = f2bf(o_lo); v[h * hd + d + half] = f2bf(o_hi);
        }
}

/* ------------------------------------------------------------ SDPA decode
 * per q head: 64-key blocks, s = dot(q,k)*scale, running (m,l,o) with exp,
 * out = T(o * (1/l)) (sdpa_decode.rs:1064-1211); kv_head = head/(nq/nkv)
 * (sdpa_decode.rs:736); cache layout [n_kv, capacity, hd] (sdpa_decode.rs:300-304). */
void fko_sdpa_decode(const bf16_t *q, const bf16_t *ck, const bf16_t *cv, int n_q, int n_kv, int hd,
                     int64_t capacity, int64_t kv_len, float scale, bf16_t *out) {
    #pragma omp parallel for schedule(static)
    for (int h = 0; h < n_q; ++h) {
        const int kvh = h / (n_q / n_kv);
        const bf16_t *K = ck + (int64_t)kvh * capacity * hd, *V = cv + (int64_t)kvh * capacity * hd;
        float qf[512], o[512], sblk[64];
        for (int d = 0; d < hd; ++d) { qf[d] = bf2f(q[h * hd + d]); o[d] = 0.0f; }
        float m = -INFINITY, l = 0.0f;
        for (int64_t blk = 0; blk < kv_len; blk += 64) {
            int bs = (int)((kv_len - blk) < 64 ? (kv_len - blk) : 64);
            float mb = -INFINITY;
            for (int i = 0; i < bs; ++i) {
                const bf16_t *kr = K + (blk + i) * hd; float dot = 0.0f;
                for (int d = 0; d < hd; ++d) { float p = qf[d] * bf2f(kr[d]); dot = dot + p; }
                sblk[i] = dot * scale; mb = sblk[i] > mb ? sblk[i] : mb;
            }
            float mn = m > mb ? m : mb;
            float alpha = expf(m - mn);
            float lb = 0.0f;
            for (int i = 0; i < bs; ++i) { sblk[i] = expf(sblk[i] - mn); lb = lb + sblk[i]; }
            l = l * alpha; l = l + lb;
            for (int d = 0; d < hd; ++d) {
                float c = 0.0f;
                for (int i = 0; i < bs; ++i) { float p = sblk[i] * bf2f(V[(blk + i) * hd + d]); c = c + p; }
                o[d] = o[d] * alpha; o[d] = o[d] + c;
            }
            m = mn;
        }
        float inv_l = 1.0f / l;
        for (int d = 0; d < hd; ++d) out[h * hd + d] = f2bf(o[d] * inv_l);
    }
}

/* ------------------------------------------------------------ quantised KV cache
 * One cache row (a head's k after RoPE, kept in fp32, or its v rounded to T) is quantised per group of `group` values with
 * the edge-anchored affine rule of src/codegen/kernels/rmsnorm_qkv.rs:560-590 (the same in
 * rope_kv_cache_store_decode_quant.rs): scale_abs = max((max - min) / (2^bits - 1), 1e-7); the edge of larger magnitude
 * anchors the grid (scale negative when that is the maximum); q0 = round(edge / scale), and unless q0 is 0 the scale
 * becomes edge / q0 and the bias the edge, so the edge is represented exactly; q = clamp(round((x - bias) / scale)).
 * scales and biases are stored as T.  round() is round-half-away-from-zero (Metal's round). */
void fko_kv_quantize_row(const float *x, int n, int group, int bits, uint32_t *packed, bf16_t *scales, bf16_t *biases) {
    const int mask = (1 << bits) - 1, per = 32 / bits;
    for (int i = 0; i < n / per; ++i) packed[i] = 0u;
    for (int g = 0; g < n / group; ++g) {
        float vmin = INFINITY, vmax = -INFINITY;
        for (int d = 0; d < group; ++d) { float v = x[g * group + d]; vmin = v < vmin ? v : vmin; vmax = v > vmax ? v : vmax; }
        float scale_abs = (vmax - vmin) / (float)mask; if (scale_abs < 1.0e-7f) scale_abs = 1.0e-7f;
        const int lo = fabsf(vmin) > fabsf(vmax);
        float scale = lo ? scale_abs : -scale_abs;
        const float edge = lo ? vmin : vmax;
        const float q0 = roundf(edge / scale);
        const int at_zero = (q0 == 0.0f);
        if (!at_zero) scale = edge / q0;
        const float bias = at_zero ? 0.0f : edge;
        const float inv = (scale != 0.0f) ? (1.0f / scale) : 0.0f;
        for (int d = 0; d < group; ++d) {
            const int idx = g * group + d;
            float t = x[idx] - bias; t = t * inv;
            int qi = (int)roundf(t); qi = qi < 0 ? 0 : (qi > mask ? mask : qi);
            packed[idx / per] |= ((uint32_t)qi & (uint32_t)mask) << ((idx % per) * bits);
        }
        scales[g] = f2bf(scale); biases[g] = f2bf(bias);
    }
}
/* RoPE of T-rounded heads with the rotated values left in fp32 (the quantising store reads them unrounded,
 * rmsnorm_qkv.rs:516-525) */
void fko_rope_f32(const bf16_t *v, int n_heads, int hd, uint32_t pos, float theta, float *out) {
    const int half = hd / 2; const float l2t = (float)log2((double)theta);
    for (int h = 0; h < n_heads; ++h)
        for (int d = 0; d < half; ++d) {
            float e = -((float)d / (float)half); e = e * l2t;
            float inv = exp2f(e);
            float ang = (float)pos * inv;
            float c = cosf(ang), s = sinf(ang);
            float lo = bf2f(v[h * hd + d]), hi = bf2f(v[h * hd + d + half]);
            float a = lo * c, b = hi * s; out[h * hd + d] = a - b;
            float p = hi * c, q = lo * s; out[h * hd + d + half] = p + q;
        }
}
static inline float kv_deq(const uint32_t *packed, const bf16_t *sc, const bf16_t *bi, int64_t row, int d, int hd, int group, int bits) {
    const int per = 32 / bits; const uint32_t mask = (1u << bits) - 1u;
    const uint32_t w = packed[row * (hd / per) + d / per];
    const float q = (float)((w >> ((d % per) * bits)) & mask);
    float t = q * bf2f(sc[row * (hd / group) + d / group]);
    return t + bf2f(bi[row * (hd / group) + d / group]);
}
/* SDPA over a quantised cache: every key / value element is float(q) * s + b with the T scales and biases
 * (sdpa_decode_quant.rs:301-372, 429-470); everything else as fko_sdpa_decode */
void fko_sdpa_decode_quant(const bf16_t *q, const uint32_t *kp, const bf16_t *ks, const bf16_t *kb, const uint32_t *vp, const bf16_t *vs,
                           const bf16_t *vb, int n_q, int n_kv, int hd, int64_t capacity, int64_t kv_len, float scale, int group, int bits,
                           bf16_t *out) {
    #pragma omp parallel for schedule(static)
    for (int h = 0; h < n_q; ++h) {
        const int kvh = h / (n_q / n_kv);
        float qf[512], o[512], sblk[64];
        for (int d = 0; d < hd; ++d) { qf[d] = bf2f(q[h * hd + d]); o[d] = 0.0f; }
        float m = -INFINITY, l = 0.0f;
        for (int64_t blk = 0; blk < kv_len; blk += 64) {
            int bs = (int)((kv_len - blk) < 64 ? (kv_len - blk) : 64);
            float mb = -INFINITY;
            for (int i = 0; i < bs; ++i) {
                const int64_t row = (int64_t)kvh * capacity + blk + i; float dot = 0.0f;
                for (int d = 0; d < hd; ++d) { float p = qf[d] * kv_deq(kp, ks, kb, row, d, hd, group, bits); dot = dot + p; }
                sblk[i] = dot * scale; mb = sblk[i] > mb ? sblk[i] : mb;
            }
            float mn = m > mb ? m : mb;
            float alpha = expf(m - mn);
            float lb = 0.0f;
            for (int i = 0; i < bs; ++i) { sblk[i] = expf(sblk[i] - mn); lb = lb + sblk[i]; }
            l = l * alpha; l = l + lb;
            for (int d = 0; d < hd; ++d) {
                float c = 0.0f;
                for (int i = 0; i < bs; ++i) { float p = sblk[i] * kv_deq(vp, vs, vb, (int64_t)kvh * capacity + blk + i, d, hd, group, bits); c = c + p; }
                o[d] = o[d] * alpha; o[d] = o[d] + c;
            }
            m = mn;
        }
        float inv_l = 1.0f / l;
        for (int d = 0; d < hd; ++d) out[h * hd + d] = f2bf(o[d] * inv_l);
    }
}

/* ------------------------------------------------------------ activations
 * SwiGLU: g=float(T(gate)), u=float(T(up)), y=T(((1/(1+exp(-g)))*g)*u)
 * (src/codegen/msl.rs:1286-1294). */
static inline bf16_t act_swiglu(float gate_acc, float up_acc) {
    float g = rT(gate_acc), u = rT(up_acc);
    float sg = 1.0f / (1.0f + expf(-g));
    float t = sg * g; t = t * u;
    return f2bf(t);
}
/* GeGLU-tanh: the traced pointwise chain gelu_approx(gate)*up evaluated op by
 * op in fp32 with a rounding to T after every op, cube expanded to multiplies
 * and tanh(clamp(x,-20,20)) (src/codegen/kernels/fused_chain.rs:2497-2565,
 * 2715-2729).  Chain: 0.5*g * (1 + tanh(0.7978845608*(g + 0.044715*g^3))) * u */
static inline bf16_t act_geglu_tanh(float gate_acc, float up_acc) {
    float g = rT(gate_acc), u = rT(up_acc);
    float g2 = rT(g * g), g3 = rT(g2 * g);
    float t1 = rT(0.044715f * g3);
    float t2 = rT(g + t1);
    float t3 = rT(0.7978845608028654f * t2);
    float cl = t3 < -20.0f ? -20.0f : (t3 > 20.0f ? 20.0f : t3);
    float t4 = rT(tanhf(cl));
    float t5 = rT(1.0f + t4);
    float t6 = rT(0.5f * g);
    float t7 = rT(t6 * t5);
    return f2bf(t7 * u);
}
void fko_act(const float *gate_acc, const float *up_acc, int64_t n, int kind, bf16_t *y) {
    for (int64_t i = 0; i < n; ++i) y[i] = kind ? act_geglu_tanh(gate_acc[i], up_acc[i]) : act_swiglu(gate_acc[i], up_acc[i]);
}

/* ------------------------------------------------------------------ argmax
 * compare on T-rounded logits, ties -> lowest index (msl.rs:1805-1838;
 * argmax_logits_decode.rs:57-59). */
uint32_t fko_argmax_bf16(const bf16_t *logits, int64_t n) {
    float best = -INFINITY; uint32_t bi = 0;
    for (int64_t i = 0; i < n; ++i) { float v = bf2f(logits[i]); if (v > best) { best = v; bi = (uint32_t)i; } }
    return bi;
}

/* =============================================================== model ==
 * A decoder laid out as the benchmark configs describe; weights generated
 * from named streams so any backend can rebuild the same tensors.          */
typedef struct {
    int arch;                 /* 0 = Qwen2-shaped, 1 = Gemma3-shaped */
    int n_layers, hidden, n_q, n_kv, head_dim, inter, vocab;
    int bits;                 /* 4, 8, 16 */
    float eps, theta, theta_local;
    int window, global_every; /* sliding window size (0 = none); every Nth layer global */
    int capacity;             /* KV capacity of global layers */
    uint64_t seed;
    /* tensor-parallel slice of the model held by this instance */
    int tp_rank, tp_size;
} fko_config;

typedef struct {
    fko_linear q, k, v, o, gate, up, down;
    bf16_t *w_in, *w_post;            /* Qwen: input / post-attention norms   */
    bf16_t *w_postattn, *w_preffn, *w_postffn, *w_qn, *w_kn;   /* Gemma extras */
    bf16_t *ck, *cv; int64_t cap; int sliding; float theta;
    /* quantised cache (fko_model_set_kv_quant): packed words [n_kv, cap, hd*bits/32], scales / biases [n_kv, cap, hd/group] */
    uint32_t *kp, *vp; bf16_t *ks, *kb, *vs, *vb;
} fko_layer;

typedef struct {
    fko_config c; fko_layer *L; bf16_t *embed; bf16_t *w_final; fko_linear head;
    float embed_scale;
    int kv_bits, kv_group;    /* 0: bf16 cache */
} fko_model;

static uint64_t sid(uint64_t seed, const char *fmt, int layer) {
    char name[128]; snprintf(name, sizeof name, fmt, layer);
    return fko_stream_id(name) ^ mix64(seed);
}
uint64_t fko_tensor_stream(uint64_t seed, const char *fmt, int layer) { return sid(seed, fmt, layer); }

static void make_linear(fko_linear *L, uint64_t stream, int64_t k_global, int64_t row0, int64_t n,
                        int64_t k0, int64_t k, int bits) {
    memset(L, 0, sizeof *L); L->n = n; L->k = k; L->bits = bits;
    if (bits == 16) {
        bf16_t *d = (bf16_t *)malloc((size_t)n * k * 2); fko_gen_dense_weight(stream, 0.02f, k_global, row0, n, k0, k, d); L->dense = d;
    } else {
        uint32_t *p = (uint32_t *)malloc((size_t)n * k * bits / 8);
        bf16_t *s = (bf16_t *)malloc((size_t)n * (k / 64) * 2), *b = (bf16_t *)malloc((size_t)n * (k / 64) * 2);
        fko_gen_qweight(stream, 0.02f, k_global, row0, n, k0, k, bits, p, s, b);
        L->packed = p; L->scales = s; L->biases = b;
    }
}
static bf16_t *make_vec(uint64_t stream, int64_t idx0, int64_t n, float mean, float std) {
    bf16_t *v = (bf16_t *)malloc((size_t)n * 2); fko_fill_normal_bf16(stream, (uint64_t)idx0, (uint64_t)n, mean, std, v); return v;
}
static void free_linear(fko_linear *L) {
    free((void *)L->packed); free((void *)L->scales); free((void *)L->biases); free((void *)L->dense); free((void *)L->lin_bias);
}

/* KV pre-fill: positions [0, ctx) of every layer's cache get N(0,1) values
 * (index = ((layer_kvhead_global * position_space) ...) by global kv head so a
 * tensor-parallel slice sees the same numbers as the full model). */
static void prefill_layer(fko_model *M, int l, int64_t ctx) {
    fko_layer *Y = &M->L[l]; const fko_config *c = &M->c;
    const int nkv_loc = c->n_kv / c->tp_size, hd = c->head_dim;
    uint64_t sk = sid(c->seed, "layers.%d.cache_k", l), sv = sid(c->seed, "layers.%d.cache_v", l);
    for (int h = 0; h < nkv_loc; ++h) {
        int gh = c->tp_rank * nkv_loc + h;
        for (int64_t p = 0; p < ctx; ++p) {
            /* ring caches keep the last `cap` positions at row p % cap */
            if (Y->sliding && p < ctx - Y->cap) continue;
            int64_t row = Y->sliding ? (p % Y->cap) : p;
            uint64_t idx0 = ((uint64_t)gh * 1048576ull + (uint64_t)p) * (uint64_t)hd;
            fko_fill_normal_bf16(sk, idx0, (uint64_t)hd, 0.0f, 1.0f, Y->ck + ((int64_t)h * Y->cap + row) * hd);
            fko_fill_normal_bf16(sv, idx0, (uint64_t)hd, 0.0f, 1.0f, Y->cv + ((int64_t)h * Y->cap + row) * hd);
        }
    }
}
void fko_model_prefill_kv(fko_model *M, int64_t ctx) { for (int l = 0; l < M->c.n_layers; ++l) prefill_layer(M, l, ctx); }

fko_model *fko_model_create(const fko_config *cfg) {
    fko_model *M = (fko_model *)calloc(1, sizeof *M); M->c = *cfg;
    const fko_config *c = &M->c;
    const int H = c->hidden, hd = c->head_dim, tp = c->tp_size, rk = c->tp_rank;
    const int nq = c->n_q / tp, nkv = c->n_kv / tp, I = c->inter / tp;
    M->L = (fko_layer *)calloc((size_t)c->n_layers, sizeof(fko_layer));
    M->embed = make_vec(sid(c->seed, "embed_tokens", 0), 0, (int64_t)c->vocab * H, 0.0f, 0.02f);
    M->w_final = make_vec(sid(c->seed, "final_norm", 0), 0, H, 1.0f, 0.02f);
    /* Gemma-family embedding scale sqrt(H) held in T (embed_lookup_decode.rs:95-98 OUTPUT_SCALE) */
    M->embed_scale = c->arch == 1 ? rT(sqrtf((float)H)) : 1.0f;
    int64_t vs = c->vocab / tp;
    make_linear(&M->head, sid(c->seed, "lm_head", 0), H, (int64_t)rk * vs, vs, 0, H, c->bits);
    for (int l = 0; l < c->n_layers; ++l) {
        fko_layer *Y = &M->L[l];
        make_linear(&Y->q, sid(c->seed, "layers.%d.q_proj", l), H, (int64_t)rk * nq * hd, (int64_t)nq * hd, 0, H, c->bits);
        make_linear(&Y->k, sid(c->seed, "layers.%d.k_proj", l), H, (int64_t)rk * nkv * hd, (int64_t)nkv * hd, 0, H, c->bits);
        make_linear(&Y->v, sid(c->seed, "layers.%d.v_proj", l), H, (int64_t)rk * nkv * hd, (int64_t)nkv * hd, 0, H, c->bits);
        make_linear(&Y->o, sid(c->seed, "layers.%d.o_proj", l), (int64_t)c->n_q * hd, 0, H, (int64_t)rk * nq * hd, (int64_t)nq * hd, c->bits);
        make_linear(&Y->gate, sid(c->seed, "layers.%d.gate_proj", l), H, (int64_t)rk * I, I, 0, H, c->bits);
        make_linear(&Y->up, sid(c->seed, "layers.%d.up_proj", l), H, (int64_t)rk * I, I, 0, H, c->bits);
        make_linear(&Y->down, sid(c->seed, "layers.%d.down_proj", l), c->inter, 0, H, (int64_t)rk * I, I, c->bits);
        Y->w_in = make_vec(sid(c->seed, "layers.%d.input_norm", l), 0, H, 1.0f, 0.02f);
        if (c->arch == 0) {
            Y->w_post = make_vec(sid(c->seed, "layers.%d.post_attention_norm", l), 0, H, 1.0f, 0.02f);
            /* Qwen2.5-shaped attention carries q/k/v biases, added in fp32 before rounding
             * (rmsnorm_qkv.rs:179-192, 631-634) */
            Y->q.lin_bias = make_vec(sid(c->seed, "layers.%d.q_bias", l), (int64_t)rk * nq * hd, (int64_t)nq * hd, 0.0f, 0.02f);
            Y->k.lin_bias = make_vec(sid(c->seed, "layers.%d.k_bias", l), (int64_t)rk * nkv * hd, (int64_t)nkv * hd, 0.0f, 0.02f);
            Y->v.lin_bias = make_vec(sid(c->seed, "layers.%d.v_bias", l), (int64_t)rk * nkv * hd, (int64_t)nkv * hd, 0.0f, 0.02f);
        } else {
            Y->w_postattn = make_vec(sid(c->seed, "layers.%d.post_attention_norm", l), 0, H, 1.0f, 0.02f);
            Y->w_preffn = make_vec(sid(c->seed, "layers.%d.pre_feedforward_norm", l), 0, H, 1.0f, 0.02f);
            Y->w_postffn = make_vec(sid(c->seed, "layers.%d.post_feedforward_norm", l), 0, H, 1.0f, 0.02f);
            Y->w_qn = make_vec(sid(c->seed, "layers.%d.q_norm", l), 0, hd, 1.0f, 0.02f);
            Y->w_kn = make_vec(sid(c->seed, "layers.%d.k_norm", l), 0, hd, 1.0f, 0.02f);
        }
        Y->sliding = (c->window > 0) && ((l + 1) % c->global_every != 0);
        Y->cap = Y->sliding ? c->window : c->capacity;
        Y->theta = Y->sliding ? c->theta_local : c->theta;
        Y->ck = (bf16_t *)calloc((size_t)nkv * Y->cap * hd, 2);
        Y->cv = (bf16_t *)calloc((size_t)nkv * Y->cap * hd, 2);
    }
    return M;
}
/* switch the model to a quantised KV cache (bits 4 / 8, group 64); the caches start empty */
void fko_model_set_kv_quant(fko_model *M, int bits, int group) {
    const int nkv = M->c.n_kv / M->c.tp_size, hd = M->c.head_dim;
    M->kv_bits = bits; M->kv_group = group;
    for (int l = 0; l < M->c.n_layers; ++l) {
        fko_layer *Y = &M->L[l];
        const size_t rows = (size_t)nkv * Y->cap;
        Y->kp = (uint32_t *)calloc(rows * hd * bits / 32, 4); Y->vp = (uint32_t *)calloc(rows * hd * bits / 32, 4);
        Y->ks = (bf16_t *)calloc(rows * hd / group, 2); Y->kb = (bf16_t *)calloc(rows * hd / group, 2);
        Y->vs = (bf16_t *)calloc(rows * hd / group, 2); Y->vb = (bf16_t *)calloc(rows * hd / group, 2);
    }
}
void fko_model_free(fko_model *M) {
    if (!M) return;
    for (int l = 0; l < M->c.n_layers; ++l) {
        fko_layer *Y = &M->L[l];
        free(Y->kp); free(Y->vp); free(Y->ks); free(Y->kb); free(Y->vs); free(Y->vb);
        free_linear(&Y->q); free_linear(&Y->k); free_linear(&Y->v); free_linear(&Y->o);
        free_linear(&Y->gate); free_linear(&Y->up); free_linear(&Y->down);
        free(Y->w_in); free(Y->w_post); free(Y->w_postattn); free(Y->w_preffn); free(Y->w_postffn);
        free(Y->w_qn); free(Y->w_kn); free(Y->ck); free(Y->cv);
    }
    free(M->L); free(M->embed); free(M->w_final); free_linear(&M->head); free(M);
}

/* accessors so a test can upload the very same tensors to another backend */
const fko_linear *fko_model_linear(const fko_model *M, int layer, int which) {
    if (layer < 0) return &M->head;
    const fko_layer *Y = &M->L[layer];
    switch (which) { case 0: return &Y->q; case 1: return &Y->k; case 2: return &Y->v; case 3: return &Y->o;
                     case 4: return &Y->gate; case 5: return &Y->up; default: return &Y->down; }
}
const bf16_t *fko_model_vec(const fko_model *M, int layer, int which) {
    if (layer < 0) return which == 0 ? M->embed : M->w_final;
    const fko_layer *Y = &M->L[layer];
    switch (which) { case 0: return Y->w_in; case 1: return Y->w_post; case 2: return Y->w_postattn; case 3: return Y->w_preffn;
                     case 4: return Y->w_postffn; case 5: return Y->w_qn; case 6: return Y->w_kn; case 7: return Y->ck; default: return Y->cv; }
}
int64_t fko_model_layer_cap(const fko_model *M, int layer) { return M->L[layer].cap; }
int fko_model_layer_sliding(const fko_model *M, int layer) { return M->L[layer].sliding; }
float fko_model_layer_theta(const fko_model *M, int layer) { return M->L[layer].theta; }
float fko_model_embed_scale(const fko_model *M) { return M->embed_scale; }

/* per-head RMSNorm in place over hd (Gemma q_norm/k_norm; single.rs:4222-4311 HEAD_MAJOR) */
static void head_norm(bf16_t *v, int n_heads, int hd, const bf16_t *w, float eps) {
    float y[512];
    for (int h = 0; h < n_heads; ++h) {
        fko_rmsnorm(v + h * hd, w, hd, eps, y);
        for (int d = 0; d < hd; ++d) v[h * hd + d] = f2bf(y[d]);
    }
}

/* One layer applied in place to the residual stream x (T[H]) of the token at `pos`; writes the
 * layer's K/V row into its cache.  Order of ops: scripts/debug_qwen2_layer0_forced.py:70-103
 * (Qwen2 shape), scripts/debug_gemma4_layer0.py:126-157 minus v_norm/per-layer inputs (Gemma shape).
 * Single rank only (tp_size 1). */
void fko_layer_step(fko_model *M, int l, bf16_t *x, uint32_t pos) {
    const fko_config *c = &M->c; const int H = c->hidden, hd = c->head_dim, nq = c->n_q, nkv = c->n_kv, I = c->inter;
    bf16_t *h = (bf16_t *)malloc((size_t)H * 2), *tmp = (bf16_t *)malloc((size_t)H * 2);
    float *nf = (float *)malloc(sizeof(float) * (size_t)(H > I ? H : I));
    bf16_t *q = (bf16_t *)malloc((size_t)nq * hd * 2), *k = (bf16_t *)malloc((size_t)nkv * hd * 2), *v = (bf16_t *)malloc((size_t)nkv * hd * 2);
    bf16_t *a = (bf16_t *)malloc((size_t)nq * hd * 2), *s = (bf16_t *)malloc((size_t)I * 2);
    float *ga = (float *)malloc(sizeof(float) * (size_t)I), *ua = (float *)malloc(sizeof(float) * (size_t)I);
    float *af = (float *)malloc(sizeof(float) * (size_t)(nq * hd > I ? nq * hd : I));
    const float scale = 1.0f / sqrtf((float)hd);          /* sdpa_decode.rs:248-252 */
    fko_layer *Y = &M->L[l];
    fko_rmsnorm(x, Y->w_in, H, c->eps, nf);
    fko_linear_apply(&Y->q, nf, NULL, q, NULL);
    fko_linear_apply(&Y->k, nf, NULL, k, NULL);
    fko_linear_apply(&Y->v, nf, NULL, v, NULL);
    if (c->arch == 1) { head_norm(q, nq, hd, Y->w_qn, c->eps); head_norm(k, nkv, hd, Y->w_kn, c->eps); }
    /* cache row = pos % capacity; kv_len = min(pos+1, capacity)
     * (rope_kv_cache_store_decode.rs:95; python/fusekit_runtime/dispatch.py:2324-2354) */
    int64_t row = (int64_t)pos % Y->cap, kv_len = (int64_t)pos + 1 < Y->cap ? (int64_t)pos + 1 : Y->cap;
    if (M->kv_bits) {       /* quantised cache: k rotated in fp32 and quantised unrounded, v quantised from its T values */
        const int G = M->kv_group, B = M->kv_bits, nw = hd * B / 32, ng = hd / G;
        float *kr = (float *)malloc(sizeof(float) * (size_t)nkv * hd), *vr = (float *)malloc(sizeof(float) * (size_t)nkv * hd);
        fko_rope_f32(k, nkv, hd, pos, Y->theta, kr);
        for (int i = 0; i < nkv * hd; ++i) vr[i] = bf2f(v[i]);
        fko_rope(q, nq, hd, pos, Y->theta);
        for (int hh = 0; hh < nkv; ++hh) {
            const int64_t r = (int64_t)hh * Y->cap + row;
            fko_kv_quantize_row(kr + hh * hd, hd, G, B, Y->kp + r * nw, Y->ks + r * ng, Y->kb + r * ng);
            fko_kv_quantize_row(vr + hh * hd, hd, G, B, Y->vp + r * nw, Y->vs + r * ng, Y->vb + r * ng);
        }
        free(kr); free(vr);
        fko_sdpa_decode_quant(q, Y->kp, Y->ks, Y->kb, Y->vp, Y->vs, Y->vb, nq, nkv, hd, Y->cap, kv_len, scale, G, B, a);
    } else {
    fko_rope(q, nq, hd, pos, Y->theta); fko_rope(k, nkv, hd, pos, Y->theta);
    for (int hh = 0; hh < nkv; ++hh) {
        memcpy(Y->ck + ((int64_t)hh * Y->cap + row) * hd, k + hh * hd, (size_t)hd * 2);
        memcpy(Y->cv + ((int64_t)hh * Y->cap + row) * hd, v + hh * hd, (size_t)hd * 2);
    }
    fko_sdpa_decode(q, Y->ck, Y->cv, nq, nkv, hd, Y->cap, kv_len, scale, a);
    }
    for (int i = 0; i < nq * hd; ++i) af[i] = bf2f(a[i]);
    if (c->arch == 0) {
        fko_linear_apply(&Y->o, af, x, h, NULL);                    /* h = T(Wo a + x) */
        fko_rmsnorm(h, Y->w_post, H, c->eps, nf);
    } else {
        fko_linear_apply(&Y->o, af, NULL, tmp, NULL);               /* o = T(Wo a) */
        fko_rmsnorm(tmp, Y->w_postattn, H, c->eps, nf);
        for (int i = 0; i < H; ++i) h[i] = f2bf(bf2f(x[i]) + nf[i]); /* h = T(x + norm(o)) */
        fko_rmsnorm(h, Y->w_preffn, H, c->eps, nf);
    }
    fko_linear_apply(&Y->gate, nf, NULL, NULL, ga);
    fko_linear_apply(&Y->up, nf, NULL, NULL, ua);
    fko_act(ga, ua, I, c->arch == 1, s);
    for (int i = 0; i < I; ++i) af[i] = bf2f(s[i]);
    if (c->arch == 0) {
        fko_linear_apply(&Y->down, af, h, x, NULL);                 /* x = T(Wd s + h) */
    } else {
        fko_linear_apply(&Y->down, af, NULL, tmp, NULL);
        fko_rmsnorm(tmp, Y->w_postffn, H, c->eps, nf);
        for (int i = 0; i < H; ++i) x[i] = f2bf(bf2f(h[i]) + nf[i]);
    }
    free(h); free(tmp); free(nf); free(q); free(k); free(v); free(a); free(s); free(ga); free(ua); free(af);
}

/* One decode step for token `tok` at position `pos`.
 * hidden_out (optional): [n_layers+1, H] T -- the residual stream after each layer, then the
 * final-normed vector.  logits_out (optional): [vocab] T. */
uint32_t fko_decode_step(fko_model *M, uint32_t tok, uint32_t pos, bf16_t *hidden_out, bf16_t *logits_out) {
    const fko_config *c = &M->c; const int H = c->hidden;
    bf16_t *x = (bf16_t *)malloc((size_t)H * 2);
    float *nf = (float *)malloc(sizeof(float) * (size_t)H);
    /* embed: x = T(embed[tok] * scale) (embed_lookup_decode.rs:95-98) */
    for (int i = 0; i < H; ++i) x[i] = f2bf(bf2f(M->embed[(int64_t)tok * H + i]) * M->embed_scale);
    for (int l = 0; l < c->n_layers; ++l) {
        fko_layer_step(M, l, x, pos);
        if (hidden_out) memcpy(hidden_out + (int64_t)l * H, x, (size_t)H * 2);
    }
    fko_rmsnorm(x, M->w_final, H, c->eps, nf);
    if (hidden_out) for (int i = 0; i < H; ++i) hidden_out[(int64_t)c->n_layers * H + i] = f2bf(nf[i]);
    bf16_t *logits = logits_out ? logits_out : (bf16_t *)malloc((size_t)c->vocab * 2);
    fko_linear_apply(&M->head, nf, NULL, logits, NULL);
    uint32_t next = fko_argmax_bf16(logits, c->vocab);
    if (!logits_out) free(logits);
    free(x); free(nf);
    return next;
}
/* logits of the head for a given residual stream (final norm + lm_head) */
uint32_t fko_head_step(fko_model *M, const bf16_t *x, bf16_t *logits_out) {
    const fko_config *c = &M->c; const int H = c->hidden;
    float *nf = (float *)malloc(sizeof(float) * (size_t)H);
    fko_rmsnorm(x, M->w_final, H, c->eps, nf);
    fko_linear_apply(&M->head, nf, NULL, logits_out, NULL);
    free(nf);
    return fko_argmax_bf16(logits_out, c->vocab);
}

/* greedy loop: tokens[i+1] = step(tokens[i], pos0+i); returns seconds spent */
double fko_decode_greedy(fko_model *M, uint32_t first_tok, uint32_t pos0, int steps, uint32_t *out_tokens) {
    double t0 = 0.0, t1 = 0.0;
#ifdef _OPENMP
    t0 = omp_get_wtime();
#endif
    uint32_t tok = first_tok;
    for (int i = 0; i < steps; ++i) { tok = fko_decode_step(M, tok, pos0 + (uint32_t)i, NULL, NULL); out_tokens[i] = tok; }
#ifdef _OPENMP
    t1 = omp_get_wtime();
#endif
    return t1 - t0;
}
/* thread count of the OpenMP loops, whatever OMP_NUM_THREADS said at start-up (results do not depend on it) */
void fko_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
int fko_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
