// Shared device-side types and helpers of the sm_100a decode kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

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
    uint32_t epoch;             // tokens finalised since the handle was opened; never reset (fk_state_set keeps it), so all
                                // tensor-parallel ranks agree on it: the sequence number of the fused peer exchanges
};
#define FK_STATE_SET_BYTES offsetof(FkState, epoch)      // what fk_state_set overwrites

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

// ---------------------------------------------------------------- peer arenas of the tensor-parallel exchange
#define FK_PEER_MAX 8
#define FK_PEER_BLOCKS 8                    // blocks of an all-reduce; block b of every rank works on slice b
#define FK_PEER_SLOT_BYTES (64 * 1024)      // bytes of a (site, source rank) slot: 16 Ki fp32 for the all-reduce kernel, 8 Ki (value, sequence) pairs for a fused exchange
#define FK_PEER_SITES 162                   // 2 parities of the all-reduce kernel + up to 160 fused exchange sites (2 per layer + argmax)
#define FK_PEER_SITE0 2
#define FK_PEER_SPIN_LIMIT (1u << 22)
struct PeerArena {
    // byte offsets inside a rank's arena.  Sites 0 and 1 are the two parities of the stand-alone all-reduce kernel; sites
    // from FK_PEER_SITE0 on belong to the exchanges fused into the projection kernels (one site per row-split projection of
    // the task list plus one for the argmax), so a site is written once per token and needs no parity.
    __host__ __device__ static size_t slot(int site, int src) { return ((size_t)site * FK_PEER_MAX + src) * FK_PEER_SLOT_BYTES; }
    __host__ __device__ static size_t flags0() { return (size_t)FK_PEER_SITES * FK_PEER_MAX * FK_PEER_SLOT_BYTES; }
    __host__ __device__ static size_t flag(int site, int src, int block) { return flags0() + (((size_t)site * FK_PEER_MAX + src) * FK_PEER_BLOCKS + block) * 128; }
    __host__ __device__ static size_t counter(int block) { return flag(FK_PEER_SITES, 0, 0) + (size_t)block * 128; }
    __host__ __device__ static size_t xsum(int site) { return counter(FK_PEER_BLOCKS) + (size_t)site * (FK_PEER_SLOT_BYTES / 2); }   // the summed vector of a site, local use
    __host__ __device__ static size_t bytes() { return xsum(FK_PEER_SITES); }
};
struct PeerMap { unsigned char *base[FK_PEER_MAX]; int rank, world; unsigned int spin_limit; };     // base[r]: rank r's arena as mapped in this process; spin_limit: polls before a wait gives up

// One fused exchange as a kernel sees it.  A slot holds (value, sequence number) pairs, 8 bytes each and written with one
// 8-byte store, so a pair is either old or new as a whole and needs no fence, flag or ticket (the scheme of low-latency
// collectives).  Producer side (a row-split projection): every finished fp32 partial row goes, paired with the token's
// sequence number, into this rank's slot of `site` in every rank's arena (plain peer stores).  Consumer side (the next
// norm-first kernel): read the pairs of all source ranks from this rank's own arena until their sequence numbers match
// (bounded), and add the values in rank order -- the same order on every rank, so all ranks hold bit-identical sums.  A site
// is written once per token, so the previous token's pairs (sequence number - 1) can never be mistaken for this token's.
struct PeerXchg { PeerMap map; int site; };      // site < 0: no exchange
__device__ __forceinline__ void peer_store_pair(const PeerXchg &x, int index, uint32_t value_bits, uint32_t seq) {
    for (int p = 0; p < x.map.world; ++p) {
        uint2 *dst = reinterpret_cast<uint2 *>(x.map.base[p] + PeerArena::slot(x.site, x.map.rank)) + index;
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(value_bits), "r"(seq) : "memory");
    }
}
// two pairs (16 bytes) of source rank `src` as they are now (the caller checks the sequence numbers)
__device__ __forceinline__ uint4 peer_peek_pairs(const PeerXchg &x, int src, int index) {
    const uint4 *p = reinterpret_cast<const uint4 *>(x.map.base[x.map.rank] + PeerArena::slot(x.site, src)) + (index >> 1);
    uint4 w;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(p) : "memory");
    return w;
}
// the same, polled until both pairs carry `seq`; false if the wait ran out
__device__ __forceinline__ bool peer_wait_pairs(const PeerXchg &x, int src, int index, uint32_t seq, uint4 &w) {
    unsigned int it = 0;
    while ((w.y != seq || w.w != seq) && ++it < x.map.spin_limit) w = peer_peek_pairs(x, src, index);
    return w.y == seq && w.w == seq;
}
__device__ __forceinline__ bool peer_load_pairs(const PeerXchg &x, int src, int index, uint32_t seq, uint32_t &v0, uint32_t &v1) {
    uint4 w = peer_peek_pairs(x, src, index);
    const bool ok = peer_wait_pairs(x, src, index, seq, w);
    v0 = w.x; v1 = w.z;
    return ok;
}
