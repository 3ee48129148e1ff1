// Device-side synthetic weights (bit-identical to the documented counter-based generator), the
// fp32 dequantisation probe and layout utilities.  Integer hashing plus single IEEE operations, so
// a CPU restatement of the same formulas produces the same bits.
#pragma once
#include "fk_common.cuh"

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ uint64_t draw64(uint64_t stream, uint64_t idx, uint64_t lane) {
    return mix64(mix64(stream ^ (idx * 0xD1342543DE82EF95ull)) + lane);
}
// twelve 16-bit uniforms summed (Irwin-Hall): unit variance, exact in fp32
__device__ __forceinline__ float unit_normal(uint64_t stream, uint64_t idx) {
    int s = 0;
#pragma unroll
    for (uint64_t lane = 0; lane < 3; ++lane) {
        const uint64_t h = draw64(stream, idx, lane);
        s += (int)(h & 0xffff) + (int)((h >> 16) & 0xffff) + (int)((h >> 32) & 0xffff) + (int)((h >> 48) & 0xffff);
    }
    return __fmul_rn((float)(s - 393210), 1.0f / 65536.0f);
}

__global__ void k_synth_normal_bf16(uint16_t *out, uint64_t stream, uint64_t idx0, uint64_t n, float mean, float std) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(__fadd_rn(mean, __fmul_rn(std, unit_normal(stream, idx0 + i))));
}

// One thread per group of 64: scale = (max-min)/(2^bits-1), bias = min, both rounded to bf16;
// q = clamp(rint((w - bias)/scale)) with the rounded values; LSB-first packing
// (layout: src/fusion/ir.rs:236-247).
__global__ void k_synth_qweight(uint32_t *packed, uint16_t *scales, uint16_t *biases, long long k, int bits,
                                long long dst_row0, long long nrows, uint64_t stream, float std,
                                long long k_global, long long src_row0, long long k0) {
    const long long groups = k >> 6;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= nrows * groups) return;
    const long long r = gid / groups, g = gid - r * groups;
    const uint64_t base = (uint64_t)((src_row0 + r) * k_global + k0 + g * 64);
    float mx = -INFINITY, mn = INFINITY;
    for (int j = 0; j < 64; ++j) {
        const float w = __fmul_rn(std, unit_normal(stream, base + j));
        mx = fmaxf(mx, w); mn = fminf(mn, w);
    }
    const int qmax = (1 << bits) - 1;
    const uint16_t sb = f2bf(__fdiv_rn(__fsub_rn(mx, mn), (float)qmax)), bb = f2bf(mn);
    const float s = bf2f(sb), b = bf2f(bb);
    const long long row = dst_row0 + r;
    scales[row * groups + g] = sb; biases[row * groups + g] = bb;
    const int per_word = 32 / bits, words = 64 / per_word;
    uint32_t *dst = packed + row * (k / per_word) + g * words;
    for (int wd = 0; wd < words; ++wd) {
        uint32_t acc = 0u;
        for (int j = 0; j < per_word; ++j) {
            const float w = __fmul_rn(std, unit_normal(stream, base + wd * per_word + j));
            const float qf = (s != 0.0f) ? rintf(__fdiv_rn(__fsub_rn(w, b), s)) : 0.0f;
            const int q = qf < 0.0f ? 0 : (qf > (float)qmax ? qmax : (int)qf);
            acc |= (uint32_t)q << (j * bits);
        }
        dst[wd] = acc;
    }
}
__global__ void k_synth_dense(uint16_t *out, long long k, long long dst_row0, long long nrows, uint64_t stream, float std,
                              long long k_global, long long src_row0, long long k0) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * k) return;
    const long long r = i / k, c = i - r * k;
    out[(dst_row0 + r) * k + c] = f2bf(__fmul_rn(std, unit_normal(stream, (uint64_t)((src_row0 + r) * k_global + k0 + c))));
}

// fp32 dequantised rows: q*s is exact in fp32, so q*s+b carries one rounding
// (src/codegen/kernels/mod.rs:2850-2908 q4, :3053-3093 q8)
__global__ void k_dequant(const uint32_t *packed, const uint16_t *scales, const uint16_t *biases, long long k, int bits,
                          long long row0, long long nrows, float *out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * k) return;
    const long long r = i / k, c = i - r * k, row = row0 + r;
    if (bits == 16) { out[i] = bf2f(reinterpret_cast<const uint16_t *>(packed)[row * k + c]); return; }
    const int per_word = 32 / bits; const uint32_t mask = (1u << bits) - 1u;
    const uint32_t q = (packed[row * (k / per_word) + c / per_word] >> ((c % per_word) * bits)) & mask;
    out[i] = __fadd_rn(__fmul_rn((float)q, bf2f(scales[row * (k >> 6) + (c >> 6)])), bf2f(biases[row * (k >> 6) + (c >> 6)]));
}
