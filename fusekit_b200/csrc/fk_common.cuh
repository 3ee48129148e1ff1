// Shared device-side types and helpers of the sm_100a decode kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define FK_MAX_ROWS 16          // independent sequences decoded together (batch rows)
#define FK_WARP 32

// Device-resident decode state: the reference's per-step uniforms (token_id_in aliased with
// next_token_out, layer_offset / kv_len derived from `offset`) advanced on the device so a chunk
// of tokens replays with no host round trip (src/codegen/kernels/mod.rs:542-579;
// python/fusekit_runtime/dispatch.py:4070-4072).
struct FkState {
    uint32_t token[FK_MAX_ROWS];
    uint32_t offset;            // position of the token being decoded
    uint32_t hist_counter;      // tokens appended to history so far
    uint32_t error;             // non-zero: a kernel refused its arguments
    uint32_t hist_cap;
};

// A linear layer's weights as the kernels see them (MLX-affine rows, group 64).
struct WView {
    const uint32_t *w;          // packed u32 words (bits 4/8) or bf16 pairs (bits 16)
    const uint16_t *s;          // bf16 scales [n, k/64]
    const uint16_t *b;          // bf16 biases [n, k/64]
    long long n, k;
    int bits;
};

__device__ __forceinline__ float bf2f(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint16_t f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float rT(float f) { return bf2f(f2bf(f)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

// block-wide sum over `nwarps` warps through a small shared array (>= 33 floats)
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0f;
    if (wid == 0) { t = warp_sum(t); if (lane == 0) red[32] = t; }
    __syncthreads();
    return red[32];
}

// Programmatic dependent launch: let the next kernel in the stream start its weight prefetch while
// this one still runs, and wait for the previous kernel's results before touching activations.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Sortable key of a T-rounded logit with ties to the lowest index: monotone map of the bf16 bits
// (src/codegen/kernels/argmax_logits_scan.rs:118-122) in the high word, inverted index in the low.
__device__ __forceinline__ unsigned long long argmax_key(uint16_t bits, uint32_t idx) {
    uint32_t k = (bits & 0x8000u) ? (uint32_t)(uint16_t)~bits : (uint32_t)(bits ^ 0x8000u);
    return ((unsigned long long)k << 32) | (unsigned long long)(0xffffffffu - idx);
}
