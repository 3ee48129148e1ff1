// Streamed batch-1 quantized matvec engine for sm_100a.
//
// HBM layout ("tiled"): a linear layer is cut into units of 16 output rows x 8 quantisation groups
// (512 weights per row at 4 bit, 256 at 8 bit).  A unit is 4608 contiguous bytes already in the order
// the consuming warp reads them: for each group j, one 16-byte vector per lane holding two packed words
// of tile row g and two of row g+8 (g = lane/4), then one 16-byte vector per lane with the four scales
// and four biases that lane applies.  One cp.async.bulk (TMA, 1-D) moves a unit into a per-warp ring in
// shared memory; a warp then needs one conflict-free LDS.128 per group.
//
// Arithmetic: integer tensor cores, exact.  The activations of a quantisation group (bf16, 8 significant bits)
// are scaled by a power of two so the largest lands in [2^19, 2^20), rounded to integers (exact for everything
// within 2^-12 of the group maximum, +-2^-20 of it below) and split into three balanced 7-bit digits (all signed,
// v = d0 + 128 d1 + 16384 d2).  Packed nibbles become bytes four at a time: w & 0x0F0F0F0F are the even nibbles,
// (w >> 4) & 0x0F0F0F0F the odd ones; 8-bit weights are used as stored.  mma.sync.m16n8k32 (u8 x s8, s32 accumulate)
// forms sum(q * digit) exactly.  The three digits of a group share their k slots, so they sit in three columns of ONE
// B operand (lanes with lane / 4 = 0, 1, 2 load digit 0, 1, 2): two MMAs per 4-bit group, one per 8-bit group, no zeroed
// operands; the lane that owns a column folds its digits exactly, scales by the group's power of two and the row's
// scale, adds b * sum(x_g), and the parts meet in the warp sum at the end of the row tile.  The tensor pipe is the
// dot-product unit because unpack + convert + FMA on the CUDA cores costs >2 issue slots per weight, more than an SM has
// at HBM speed.
// History of the mapping (7B-shaped q4, tok/s on one B200): fp16 MMA after unpacking 600; groups on the eight columns with
// zero vectors loaded from shared memory 741 (shared-memory bandwidth bound: 24 four-wavefront loads per unit); the same
// with each lane loading only its own group's digits and selecting zeros 777 (48 MMAs per unit, tensor pipe 38 %,
// math_pipe_throttle the top stall); digits on the columns 794 (16 MMAs per unit, memory-bound).  Two 8-bit digits
// (16-bit activations, the rounding loss of a group added back times the mean weight code) ran 6 % faster than the three-
// digit form of its day and stayed inside the per-stage tolerance, but its 64-token greedy check showed a flip three bf16
// ulps wide: not kept.
//
// Scheduling: blocks of 16 warps, one per SM (8 warps, two per SM, for weights with many rounds of tiles), each warp with
// its own ring and mbarriers.  With at least one row tile per warp in the grid a warp owns whole tiles (all of K); otherwise
// 2, 4, 8 or 16 warps of a block split K of a tile and fold their sums through shared memory in warp order (deterministic,
// no global round trip).  Rings are filled before griddepcontrol.wait: weights do not depend on the previous kernel, so
// under programmatic dependent launch a block of the next kernel that lands on an SM slot freed by this one streams its
// weights while this kernel finishes.  (L2 prefetches -- of the next kernel's first units, of the rest of a warp's run, of
// the unit a few fetches ahead -- were each measured and dropped: all slower.)
#pragma once
#include "fk_common.cuh"
#include "fk_attend.cuh"

#define FK_UNIT_VEC 288                 // uint4 per unit: 8 groups x 32 lanes + 32 scale/bias vectors (also the ring slot size)
#define FK_UNIT_BYTES (FK_UNIT_VEC * 16)
// bf16 weights use the same machinery with units of 16 rows x 128 activations: 8 mma.m16n8k16 A fragments of 32 lanes
// x 16 bytes = 256 vectors, no scale/bias tail
__host__ __device__ inline int unit_vec(int bits) { return bits == 16 ? 256 : FK_UNIT_VEC; }
__host__ __device__ inline int unit_k(int bits) { return bits == 4 ? 512 : bits == 8 ? 256 : 128; }      // activations covered by a unit
#define FK_STREAM_MAXWARPS 16         // blocks run 8 warps (two blocks per SM) or 16 (one per SM, large activations)
#define FK_STAGES 2                     // ring depth per warp
#define FK_ZERO_BYTES 256               // zero vectors (the bf16 engine's B operand outside column 0)
#define FK_WAIT_LIMIT (1u << 24)        // bounded mbarrier wait; on expiry the kernel flags an error and leaves
#ifndef FK_J_UNROLL
#define FK_J_UNROLL 8                   // unroll factor of the group loop inside a unit (code size against scheduling freedom)
#endif
#ifndef FK_ROLLED_UPTO
#define FK_ROLLED_UPTO 2                // runs of at most this many units per warp take the rolled (small-code) unit arithmetic
#endif
#define FK_STR(x) #x
#define FK_UNROLL(n) _Pragma(FK_STR(unroll n))

enum { FK_ROWS_PLAIN = 0, FK_ROWS_ROPE_PAIRS = 1, FK_ROWS_GATE_UP = 2 };

struct TiledW {
    const uint4 *units;     // [ntiles][nsb][FK_UNIT_VEC]
    int ntiles, nsb;        // row tiles of 16, super-blocks of 8 groups
    int n, k, bits;         // logical shape (rows after pairing/interleave)
    int rows_kind, hd, n_rot;   // row order inside tiles (see tile_row)
};

// source row of tile row r (0..15): plain order; RoPE pairs (rows 0-7 = dims d..d+7 of a head, rows 8-15 =
// the same dims + head_dim/2) for the first n_rot rows; gate/up interleave (rows 0-7 gate, 8-15 up).
__host__ __device__ inline long long tile_row(int kind, int hd, int n_rot, int tile, int r) {
    if (kind == FK_ROWS_ROPE_PAIRS && tile < n_rot / 16) {
        const int tph = hd / 16, head = tile / tph, c = tile - head * tph;
        return (long long)head * hd + c * 8 + (r & 7) + (r >= 8 ? hd / 2 : 0);
    }
    if (kind == FK_ROWS_GATE_UP) return (long long)tile * 8 + (r & 7);     // which matrix: r >= 8 -> up
    return (long long)tile * 16 + r;
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: returns false if the barrier never completed
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < FK_WAIT_LIMIT; ++i) if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// D[16x8] += A[16x32] * B[32x8], 8-bit operands, s32 accumulators.  B signed for the top digit only.
__device__ __forceinline__ void imma_us(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D[16x8] += A[16x16] * B[16x8], bf16 operands, fp32 accumulators
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// shared-memory loads by 32-bit address: the choice between a group's digits and the zero vectors is then a SEL on an
// address, where a choice between two generic pointers compiled to a divergent branch per group
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr)); return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr)); return v;
}

// ------------------------------------------------------------------ shared-memory plan of a streamed kernel
struct StreamSmem {
    uint64_t *bars;     // [warps * stages]
    uint4 *zero;        // FK_ZERO_BYTES of zeros
    float2 *xsi;        // [groups] (sum of the group's activations, 1 / power-of-two scale of its integer digits)
    float *red;         // [48]
    float *fold;        // [2][16 warps][16] per-warp row sums of a round
    uint2 *xs;          // [groups][3 digits][4 lanes][1 or 2] activation digits in MMA B-operand order
    uint4 *ring;        // [warps * stages * FK_UNIT_VEC]
};
__host__ __device__ inline int stream_groups(int nsb) { return nsb * 8; }
// bytes of staged activations per group: 4-bit 3 digits x 4 x 16, 8-bit 3 x 4 x 8, bf16 weights: the bf16 values themselves
__host__ __device__ inline int xs_group_bytes(int bits) { return bits == 4 ? 192 : bits == 8 ? 96 : 32; }      // bf16: a group is one k16 step, 4 lanes x {b0, b1}
__host__ __device__ inline size_t stream_smem_bytes(int nsb, int stages, int warps, int bits) {
    size_t b = 512 /*bars*/ + FK_ZERO_BYTES + (size_t)stream_groups(nsb) * 8 + 192 /*red*/ + 2 * FK_STREAM_MAXWARPS * 16 * 4 /*fold: two rounds of per-warp row sums*/;
    b = (b + 15) & ~(size_t)15;
    b += (size_t)stream_groups(nsb) * xs_group_bytes(bits);    // xs
    b = (b + 127) & ~(size_t)127;
    b += (size_t)warps * stages * FK_UNIT_BYTES;
    return b + 128;
}
// `base` is the kernel's dynamic shared memory (declared 128-byte aligned).  Offsets only, no integer casts: the compiler
// must keep seeing shared-memory pointers, or every access becomes a generic load with 64-bit address arithmetic.
__device__ __forceinline__ StreamSmem stream_carve(unsigned char *base, int nsb, int stages, int bits) {
    StreamSmem s;
    size_t o = 0;
    s.bars = (uint64_t *)(base + o); o += 512;
    s.zero = (uint4 *)(base + o); o += FK_ZERO_BYTES;
    s.xsi = (float2 *)(base + o); o += (size_t)stream_groups(nsb) * 8;
    s.red = (float *)(base + o); o += 192;
    s.fold = (float *)(base + o); o += 2 * FK_STREAM_MAXWARPS * 16 * 4;
    o = (o + 15) & ~(size_t)15;
    s.xs = (uint2 *)(base + o); o += (size_t)stream_groups(nsb) * xs_group_bytes(bits);
    o = (o + 127) & ~(size_t)127;
    s.ring = (uint4 *)(base + o);
    return s;
}

// Activation staging.  A thread owns blocks of 8 consecutive activations (one 16-byte load), keeps them in
// registers, and writes their three digits in MMA B-operand order:
//   4-bit: a packed word covers the block; its even nibbles unpack into one A register and its odd nibbles into the
//          other, so each digit is stored as bytes (x0,x2,x4,x6 | x1,x3,x5,x7); a group is 64 activations (8 threads);
//          lane t of the MMA reads {word A pair, word B pair} = 16 bytes per digit, word B being 32 activations on.
//   8-bit: a packed word covers 4 activations in order; a group (one MMA k-extent) is 32 activations (4 threads);
//          lane t reads {word A, word B} = 8 bytes per digit, word B being 16 activations on.
// Group maximum (for the scale) and group sum are reduced with shuffles across the threads of a group.
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
    f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 255) | ((uint32_t)(b & 255) << 8) | ((uint32_t)(c & 255) << 16) | ((uint32_t)(d & 255) << 24);
}
// `xsw` / `xsi`: where the digits and the (sum, 1 / scale) pairs go -- the kernel's shared memory, or a global buffer of the
// same layout that a later kernel copies in (the gate/up kernel prepares down_proj's activations that way).
template <int BITS>
__device__ __forceinline__ void store_block_to(uint32_t *xsw, float2 *xsi, int blk, const float (&f)[8], bool valid) {
    if (BITS == 16) {       // bf16 weights: the activations are bf16 already; lane t of k16 step s reads {x[2t], x[2t+1]} and {x[2t+8], x[2t+9]}
        if (!valid) return;
        uint32_t *dst = xsw + (size_t)(blk >> 1) * 8 + (blk & 1);
#pragma unroll
        for (int t = 0; t < 4; ++t) dst[2 * t] = (uint32_t)f2bf(f[2 * t]) | ((uint32_t)f2bf(f[2 * t + 1]) << 16);
        return;
    }
    float s8 = 0.0f, m8 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { s8 += f[i]; m8 = fmaxf(m8, fabsf(f[i])); }
    if (!valid) { s8 = 0.0f; m8 = 0.0f; }
    constexpr int TPG = BITS == 4 ? 8 : 4;          // threads per group
#pragma unroll
    for (int o = 1; o < TPG; o <<= 1) { s8 += __shfl_xor_sync(0xffffffffu, s8, o); m8 = fmaxf(m8, __shfl_xor_sync(0xffffffffu, m8, o)); }
    // scale = 2^(XB - exponent(max)): the largest activation becomes an integer in [2^19, 2^20), so that v + 8256 (the offset of
    // the balanced digits below) stays under 2^21 and the top digit fits s8
    constexpr int XB = 19;
    int e = m8 > 0.0f ? (int)((__float_as_uint(m8) >> 23) & 0xffu) - 127 : XB;
    e = e < -100 ? -100 : (e > 100 ? 100 : e);
    const float scale = __uint_as_float((uint32_t)(127 + XB - e) << 23), inv = __uint_as_float((uint32_t)(127 - XB + e) << 23);
    if (!valid) return;
    // three 7-bit digits of the integers: byte 0 of xi, xi >> 7, xi >> 14, gathered four at a time with byte permutes and masked
    // as a word.  Balanced: v + 64 + 64 * 128 is split and 64 taken off the two low digits again, so every digit is signed and
    // centred -- the partial sums that different lanes accumulate (low digits / top digit) then both have random signs.  (With
    // unsigned low digits the low-digit sums grow with K and the fp32 accumulation noise with them: three times as many
    // one-ulp flips per stage against the CPU restatement.)
    uint32_t x0[8], x7[8], x14[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { const int v = __float2int_rn(f[i] * scale) + 8256; x0[i] = (uint32_t)v; x7[i] = (uint32_t)(v >> 7); x14[i] = (uint32_t)(v >> 14); }
    auto bytes4 = [](uint32_t a, uint32_t b, uint32_t c, uint32_t d) {      // byte 0 of a, b, c, d
        return __byte_perm(__byte_perm(a, b, 0x0040u), __byte_perm(c, d, 0x0040u), 0x5410u);
    };
    auto low7 = [](uint32_t w) {                 // per byte: (w & 127) - 64 as s8 (flip bit 6, copy it into bit 7)
        const uint32_t t = (w & 0x7f7f7f7fu) ^ 0x40404040u;
        return t | ((t & 0x40404040u) << 1);
    };
    if (BITS == 4) {
        const int grp = blk >> 3, bb = blk & 7;
        // [digit][lane t = bb & 3]{word A even, word B even, word A odd, word B odd}: the even nibbles of both words feed one MMA,
        // the odd nibbles the other
        uint32_t *dst = xsw + (size_t)grp * 48 + (bb & 3) * 4 + (bb >> 2);
        dst[0] = low7(bytes4(x0[0], x0[2], x0[4], x0[6])); dst[2] = low7(bytes4(x0[1], x0[3], x0[5], x0[7]));
        dst[16] = low7(bytes4(x7[0], x7[2], x7[4], x7[6])); dst[18] = low7(bytes4(x7[1], x7[3], x7[5], x7[7]));
        dst[32] = bytes4(x14[0], x14[2], x14[4], x14[6]); dst[34] = bytes4(x14[1], x14[3], x14[5], x14[7]);
        if (bb == 0) xsi[grp] = make_float2(s8, inv);
    } else {
        const int k0 = blk * 8, grp = k0 >> 5, o = k0 & 31, half = o >> 4, t = (o >> 2) & 3;
        uint32_t *dst = xsw + (size_t)grp * 24 + t * 2 + half;   // [digit][lane][A|B] as words
#pragma unroll
        for (int q = 0; q < 2; ++q) {                    // the two 4-blocks of this thread: lanes t and t+1
            dst[2 * q] = low7(bytes4(x0[4 * q], x0[4 * q + 1], x0[4 * q + 2], x0[4 * q + 3]));
            dst[8 + 2 * q] = low7(bytes4(x7[4 * q], x7[4 * q + 1], x7[4 * q + 2], x7[4 * q + 3]));
            dst[16 + 2 * q] = bytes4(x14[4 * q], x14[4 * q + 1], x14[4 * q + 2], x14[4 * q + 3]);
        }
        if ((blk & 3) == 0) xsi[blk >> 2] = make_float2(s8, inv);
    }
}
template <int BITS>
__device__ __forceinline__ void store_block(const StreamSmem &sm, int blk, const float (&f)[8], bool valid) {
    store_block_to<BITS>(reinterpret_cast<uint32_t *>(sm.xs), sm.xsi, blk, f, valid);
}
// zero vectors, padded tail of xs / xsum (k rounded up to whole units)
template <int BITS>
__device__ __forceinline__ void stage_pad(const StreamSmem &sm, int k, int nsb) {
    const int per_group = BITS == 4 ? 64 : BITS == 8 ? 32 : 16, groups = stream_groups(nsb), g0 = k / per_group;
    constexpr int V = BITS == 4 ? 24 : BITS == 8 ? 12 : 4;          // uint2 per group
    for (int i = threadIdx.x; i < FK_ZERO_BYTES / 16; i += blockDim.x) sm.zero[i] = make_uint4(0, 0, 0, 0);
    for (int i = g0 * V + threadIdx.x; i < groups * V; i += blockDim.x) sm.xs[i] = make_uint2(0, 0);
    for (int i = g0 + threadIdx.x; i < groups; i += blockDim.x) sm.xsi[i] = make_float2(0.0f, 0.0f);
}
__device__ __forceinline__ void stamp_raw(unsigned long long *tl, int slot) {
    if (tl && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); tl[blockIdx.x * 8 + slot] = t; }
}
#define FK_STAGE_MAXB 4          // 8-blocks per thread held in registers during staging (h <= 8 * 256 * 4)
// MAXB: 8-blocks per thread requested together (one round trip); longer inputs take more rounds.  Small on purpose:
// every unrolled copy is code the kernel carries, and a kernel's launch-to-launch cost grows with its size.
template <int BITS, int MAXB>
__device__ __forceinline__ void stage_plain(const StreamSmem &sm, const uint16_t *x, int k, int nsb) {
    const int nblk = k >> 3;
    for (int b0 = 0; b0 < nblk; b0 += MAXB * blockDim.x) {
        uint4 v[MAXB];
#pragma unroll
        for (int i = 0; i < MAXB; ++i) {          // all loads in flight before the first use
            const int blk = b0 + i * blockDim.x + threadIdx.x;
            v[i] = blk < nblk ? __ldcg(reinterpret_cast<const uint4 *>(x + (size_t)blk * 8)) : make_uint4(0, 0, 0, 0);
        }
        // one copy of the conversion code, the held vectors rotated through v[0]: this code runs once per launch, so its size
        // (instruction fetch) counts as much as its instruction count
#pragma unroll 1
        for (int i = 0; i < MAXB; ++i) {
            const int blk = b0 + i * blockDim.x + threadIdx.x;
            if (b0 + i * (int)blockDim.x >= nblk) break;   // uniform across the block
            float f[8]; unpack8(v[0], f);
            store_block<BITS>(sm, blk, f, blk < nblk);
#pragma unroll
            for (int j = 0; j + 1 < MAXB; ++j) v[j] = v[j + 1];
        }
    }
    __syncthreads();
}
// RMSNorm (two roundings to T, src/codegen/kernels/mod.rs:4464-4472; rmsnorm_qkv.rs:325), optionally after advancing the
// residual stream with a pending post-norm, x' = T(x + rmsnorm(pending) * w_p) (Gemma-shaped layers); block 0
// publishes x' to h_out.  One round of global loads: x, w (and the pending pair) stay in registers.
// The norm weights are constants: a kernel fetches its thread's share before griddepcontrol.wait (a first touch per token
// comes from HBM), so only the activations are loaded on the critical path after it.
struct NormW { uint4 v[FK_STAGE_MAXB]; };
__device__ __forceinline__ void norm_w_load(NormW &nw, const uint16_t *w, int h) {
    const int nblk = h >> 3;
#pragma unroll
    for (int i = 0; i < FK_STAGE_MAXB; ++i) {
        const int blk = i * blockDim.x + threadIdx.x;
        nw.v[i] = blk < nblk ? __ldg(reinterpret_cast<const uint4 *>(w + (size_t)blk * 8)) : make_uint4(0, 0, 0, 0);
    }
}
template <int BITS, bool PEND = true>
__device__ __forceinline__ void stage_rmsnorm(const StreamSmem &sm, const uint16_t *x, const NormW &nwv, int h, int nsb, float eps,
                                              const uint16_t *pending, const uint16_t *pending_w, uint16_t *h_out,
                                              unsigned long long *tl = nullptr, const float *pend_sum = nullptr,
                                              const PeerXchg *pull = nullptr, FkState *st = nullptr) {
    const int nblk = h >> 3;
    uint4 xv[FK_STAGE_MAXB];
    const uint4 (&wv)[FK_STAGE_MAXB] = nwv.v;
#pragma unroll
    for (int i = 0; i < FK_STAGE_MAXB; ++i) {
        const int blk = i * blockDim.x + threadIdx.x;
        xv[i] = blk < nblk ? __ldcg(reinterpret_cast<const uint4 *>(x + (size_t)blk * 8)) : make_uint4(0, 0, 0, 0);
    }
    if (PEND && pull && pull->site >= 0) {
        // Tensor parallel, fused exchange: x' = T(sum over ranks of the partial rows + residual x).  Two steps, so that the cost
        // does not grow with the number of ranks: (A) the blocks of this kernel share the sum -- a block takes a slice of the
        // vector, one thread per (element pair, source rank) fetches the pushed (value, sequence) pairs, the ranks are added in
        // rank order through shared memory, and the rounded pair goes, with the sequence number, into this GPU's summed vector
        // of the site; (B) every block reads the whole summed vector from there.  Waits are bounded: on expiry the error word is
        // set and the values are wrong, nothing hangs.
        const uint32_t seq = st->epoch + 1u;
        const int world = pull->map.world, couples = h >> 1;
        const int per_block = (couples + (int)gridDim.x - 1) / (int)gridDim.x, c0 = (int)blockIdx.x * per_block;
        const int c1 = c0 + per_block < couples ? c0 + per_block : couples, pass = 256 / world;
        unsigned char *own = pull->map.base[pull->map.rank];
        uint2 *xsum = reinterpret_cast<uint2 *>(own + PeerArena::xsum(pull->site));
        float2 *part = reinterpret_cast<float2 *>(sm.fold);            // [pass][world]; the fold buffer is free until the unit loop
        bool ok = true;
        for (int base = c0; base < c1; base += pass) {
            const int n = c1 - base < pass ? c1 - base : pass;
            if ((int)threadIdx.x < n * world) {
                const int e = (int)threadIdx.x / world, p = (int)threadIdx.x - e * world;
                uint32_t v0, v1;
                ok = peer_load_pairs(*pull, p, 2 * (base + e), seq, v0, v1) && ok;
                part[e * world + p] = make_float2(__uint_as_float(v0), __uint_as_float(v1));
            }
            __syncthreads();
            if ((int)threadIdx.x < n) {
                const int ce = base + (int)threadIdx.x;
                float s0 = 0.0f, s1 = 0.0f;
                for (int p = 0; p < world; ++p) { const float2 v = part[threadIdx.x * world + p]; s0 += v.x; s1 += v.y; }
                const uint32_t xr = __ldcg(reinterpret_cast<const uint32_t *>(x) + ce);
                const uint32_t o = (uint32_t)f2bf(s0 + bf_lo(xr)) | ((uint32_t)f2bf(s1 + bf_hi(xr)) << 16);
                asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(xsum + ce), "r"(o), "r"(seq) : "memory");
                if (h_out) reinterpret_cast<uint32_t *>(h_out)[ce] = o;
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < FK_STAGE_MAXB; ++i) {
            const int blk = i * blockDim.x + threadIdx.x;
            if (blk < nblk) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; j += 2) {          // two (pair, sequence) entries per 16-byte load
                    const uint4 *src = reinterpret_cast<const uint4 *>(xsum + blk * 4 + j);
                    uint4 w; unsigned int it = 0;
                    do {
                        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
                    } while ((w.y != seq || w.w != seq) && ++it < pull->map.spin_limit);
                    ok = ok && w.y == seq && w.w == seq;
                    o[j] = w.x; o[j + 1] = w.z;
                }
                xv[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        if (!ok) atomicOr(&st->error, 0x8000u);
    } else if (PEND && pend_sum) {     // tensor parallel: x' = T(all-reduced projection + residual x); block 0 publishes it
#pragma unroll
        for (int i = 0; i < FK_STAGE_MAXB; ++i) {
            const int blk = i * blockDim.x + threadIdx.x;
            if (blk < nblk) {
                const float4 s0 = __ldcg(reinterpret_cast<const float4 *>(pend_sum + (size_t)blk * 8)), s1 = __ldcg(reinterpret_cast<const float4 *>(pend_sum + (size_t)blk * 8 + 4));
                float f[8]; unpack8(xv[i], f);
                const uint16_t o0 = f2bf(s0.x + f[0]), o1 = f2bf(s0.y + f[1]), o2 = f2bf(s0.z + f[2]), o3 = f2bf(s0.w + f[3]);
                const uint16_t o4 = f2bf(s1.x + f[4]), o5 = f2bf(s1.y + f[5]), o6 = f2bf(s1.z + f[6]), o7 = f2bf(s1.w + f[7]);
                xv[i] = make_uint4(o0 | ((uint32_t)o1 << 16), o2 | ((uint32_t)o3 << 16), o4 | ((uint32_t)o5 << 16), o6 | ((uint32_t)o7 << 16));
                if (blockIdx.x == 0 && h_out) *reinterpret_cast<uint4 *>(h_out + (size_t)blk * 8) = xv[i];
            }
        }
    }
    if (PEND && pending) {
        uint4 pv[FK_STAGE_MAXB], pw[FK_STAGE_MAXB];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < FK_STAGE_MAXB; ++i) {
            const int blk = i * blockDim.x + threadIdx.x;
            pv[i] = pw[i] = make_uint4(0, 0, 0, 0);
            if (blk < nblk) { pv[i] = __ldcg(reinterpret_cast<const uint4 *>(pending + (size_t)blk * 8)); pw[i] = *reinterpret_cast<const uint4 *>(pending_w + (size_t)blk * 8); }
            float f[8]; unpack8(pv[i], f);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
        }
        ss = block_sum(ss, sm.red);
        const float rp = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)h), eps)));
#pragma unroll
        for (int i = 0; i < FK_STAGE_MAXB; ++i) {
            const int blk = i * blockDim.x + threadIdx.x;
            float f[8], pf[8], wf[8]; unpack8(xv[i], f); unpack8(pv[i], pf); unpack8(pw[i], wf);
            uint16_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = f2bf(f[j] + rT(wf[j] * rT(pf[j] * rp)));
            xv[i] = make_uint4(o[0] | ((uint32_t)o[1] << 16), o[2] | ((uint32_t)o[3] << 16), o[4] | ((uint32_t)o[5] << 16), o[6] | ((uint32_t)o[7] << 16));
            if (blk < nblk && blockIdx.x == 0 && h_out) *reinterpret_cast<uint4 *>(h_out + (size_t)blk * 8) = xv[i];
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < FK_STAGE_MAXB; ++i) {
        float f[8]; unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
    }
    stamp_raw(tl, 4);
    ss = block_sum(ss, sm.red);
    stamp_raw(tl, 5);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)h), eps)));
    uint4 wl[FK_STAGE_MAXB];
#pragma unroll
    for (int i = 0; i < FK_STAGE_MAXB; ++i) wl[i] = wv[i];
#pragma unroll 1
    for (int i = 0; i < FK_STAGE_MAXB; ++i) {             // one copy of the conversion code (see stage_plain)
        const int blk = i * blockDim.x + threadIdx.x;
        if (i * (int)blockDim.x >= nblk) break;            // uniform across the block
        float f[8], wf[8]; unpack8(xv[0], f); unpack8(wl[0], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = rT(wf[j] * rT(f[j] * r));
        store_block<BITS>(sm, blk, f, blk < nblk);
#pragma unroll
        for (int j = 0; j + 1 < FK_STAGE_MAXB; ++j) { xv[j] = xv[j + 1]; wl[j] = wl[j + 1]; }
    }
    __syncthreads();
}

// ------------------------------------------------------------------ one unit: 16 rows x 8 groups
// Shared-memory loads at [address + immediate]: the unit loop is fully unrolled, so every offset inside a ring slot or a
// super-block of digits is a compile-time constant and costs no address arithmetic.
template <int OFF> __device__ __forceinline__ uint4 lds128o(uint32_t addr) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF)); return v;
}
template <int OFF> __device__ __forceinline__ uint2 lds64o(uint32_t addr) {
    uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF)); return v;
}
// first MMA of a chain: the accumulator starts at zero (constant-zero inputs instead of cleared registers)
__device__ __forceinline__ void imma_us0(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// bf16 weights: eight k16 steps; the activations sit in B column 0 (lanes with g == 0), so D[:, 0] = W x lands in the lanes
// with t == 0 and the other lanes add zeros.  `ub`: shared address of this lane's first vector of the unit.
__device__ __forceinline__ void unit_compute_bf16(uint32_t ub, const StreamSmem &sm, int sb, int lane, float &acc_lo, float &acc_hi) {
    const int g = lane >> 2, t = lane & 3;
    float c[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
    const uint2 *z2 = reinterpret_cast<const uint2 *>(sm.zero);
#pragma unroll
    for (int s8 = 0; s8 < 8; ++s8) {
        const uint4 w = lds128(ub + (uint32_t)s8 * 512u);
        const uint2 b = (g == 0) ? sm.xs[(size_t)(sb * 8 + s8) * 4 + t] : z2[t];
        mma_bf16(c[s8 & 1], w.x, w.y, w.z, w.w, b.x, b.y);
    }
    acc_lo += c[0][0] + c[1][0]; acc_hi += c[0][2] + c[1][2];
}
// 4- and 8-bit units, digits on the accumulator columns (8 bits: one MMA per 32-activation group, eight per unit instead of 24).  The three digits of a group's activations share their k slots, so they can
// sit in three columns of ONE B operand: lanes with lane / 4 = 0, 1, 2 load digit 0, 1, 2 of group J (the other lanes load
// digit 0 again; their columns are never read), and two MMAs per group -- even nibbles, then the odd nibbles shifted down --
// leave sum(q * digit_c) of rows g, g + 8 in columns 0..2: 16 MMAs per unit instead of 48 and no zeroed operands.  All digits
// go in as s8 (balanced digits, see store_block).  Column c belongs to lane t = c / 2: t = 0 folds
// d0 + 128 d1 (< 2^24), t = 1 holds 16384 d2, t = 2, 3 contribute zero through their multipliers; each lane scales its part
// by the group's power of two and the row's scale and the parts meet in the warp sum over t at the end of the row tile.
template <int BITS>
__device__ __forceinline__ void unit_compute_qc(uint32_t ub, const StreamSmem &sm, int sb, int lane, float &acc_lo, float &acc_hi) {
    const int g = lane >> 2, t = lane & 3;
    // staged digits: [group][digit][lane t]{...}; a group is one MMA k extent at 8 bits (32 activations), two at 4 bits (64)
    constexpr uint32_t GB = BITS == 4 ? 192u : 96u, DB = GB / 3, LB = BITS == 4 ? 16u : 8u;
    const uint32_t xb = smem_u32(sm.xs) + (uint32_t)sb * (8u * GB) + (uint32_t)(g < 3 ? g : 0) * DB + (uint32_t)t * LB;
    const int mulA = t == 0 ? 1 : (t == 1 ? 16384 : 0), mulB = t == 0 ? 128 : 0;
    const float fA = (float)mulA, fB = (float)mulB;
    const uint32_t xi = smem_u32(sm.xsi) + (uint32_t)sb * 64u;          // (sum, 1 / scale) of the eight groups
    const uint32_t sv = ub + 4096u - (uint32_t)t * 16u;                 // the scale / bias vectors of rows g, g + 8: lanes (g, 0..3)
    const uint2 s0 = lds64o<0>(sv), s1 = lds64o<16>(sv), s2 = lds64o<32>(sv), s3 = lds64o<48>(sv);
    const uint4 i01 = lds128o<0>(xi), i23 = lds128o<16>(xi), i45 = lds128o<32>(xi), i67 = lds128o<48>(xi);
    constexpr uint32_t M = 0x0F0F0F0Fu;
#define FK_GC(J, SV, INV, HALF)                                                                                              \
    {                                                                                                                        \
        const uint4 w = lds128o<J * 512>(ub);                                                                                \
        int d[4];                                                                                                            \
        float flo, fhi;                                                                                                      \
        const float inv = __uint_as_float(INV);                                                                              \
        if (BITS == 4) {                                                                                                     \
            const uint4 x = lds128o<J * 192>(xb);                                                                            \
            imma_us0(d, w.x & M, w.z & M, w.y & M, w.w & M, x.x, x.y);                                                       \
            imma_us(d, (w.x >> 4) & M, (w.z >> 4) & M, (w.y >> 4) & M, (w.w >> 4) & M, x.z, x.w);                            \
            flo = (float)(d[0] * mulA + d[1] * mulB) * inv; fhi = (float)(d[2] * mulA + d[3] * mulB) * inv;                  \
        } else {        /* sums up to 255 * 64 * 32: the top digit's factor is applied in fp32 */                            \
            const uint2 x = lds64o<J * 96>(xb);                                                                              \
            imma_us0(d, w.x, w.z, w.y, w.w, x.x, x.y);                                                                       \
            flo = fmaf((float)d[1], fB, (float)d[0] * fA) * inv; fhi = fmaf((float)d[3], fB, (float)d[2] * fA) * inv;        \
        }                                                                                                                    \
        acc_lo = fmaf(HALF ? bf_hi(SV.x) : bf_lo(SV.x), flo, acc_lo);                                                        \
        acc_hi = fmaf(HALF ? bf_hi(SV.y) : bf_lo(SV.y), fhi, acc_hi);                                                        \
    }
    FK_GC(0, s0, i01.y, 0) FK_GC(1, s0, i01.w, 1) FK_GC(2, s1, i23.y, 0) FK_GC(3, s1, i23.w, 1)
    FK_GC(4, s2, i45.y, 0) FK_GC(5, s2, i45.w, 1) FK_GC(6, s3, i67.y, 0) FK_GC(7, s3, i67.w, 1)
#undef FK_GC
    // b * sum(x) of the lane's own two groups (2t, 2t + 1), as laid out in its own vector
    const uint4 own = lds128o<4096>(ub);
    const uint4 xo = lds128(xi + (uint32_t)t * 16u);
    const float X0 = __uint_as_float(xo.x), X1 = __uint_as_float(xo.z);
    acc_lo = fmaf(bf_lo(own.z), X0, acc_lo); acc_lo = fmaf(bf_hi(own.z), X1, acc_lo);
    acc_hi = fmaf(bf_lo(own.w), X0, acc_hi); acc_hi = fmaf(bf_hi(own.w), X1, acc_hi);
}

// The same unit with the group loop rolled (two groups per iteration, addresses computed): a sixth of the code.  A warp whose
// whole run is one or two units executes the unit code once, cold -- there the instruction fetch of the unrolled form costs
// more than its address arithmetic saves.
template <int BITS>
__device__ __noinline__ float2 unit_compute_qc_rolled(uint32_t ub, uint32_t xs0, uint32_t xi0, int sb, int lane, float acc_lo, float acc_hi) {
    const int g = lane >> 2, t = lane & 3;
    constexpr uint32_t GB = BITS == 4 ? 192u : 96u, DB = GB / 3, LB = BITS == 4 ? 16u : 8u;
    uint32_t xb = xs0 + (uint32_t)sb * (8u * GB) + (uint32_t)(g < 3 ? g : 0) * DB + (uint32_t)t * LB;
    const int mulA = t == 0 ? 1 : (t == 1 ? 16384 : 0), mulB = t == 0 ? 128 : 0;
    const float fA = (float)mulA, fB = (float)mulB;
    uint32_t xi = xi0 + (uint32_t)sb * 64u, sv = ub + 4096u - (uint32_t)t * 16u, wb = ub;
    constexpr uint32_t M = 0x0F0F0F0Fu;
    float lo = acc_lo, hi = acc_hi;
#pragma unroll 1
    for (int j = 0; j < 4; ++j, xb += 2 * GB, xi += 16, sv += 16, wb += 1024) {
        const uint2 s2 = lds64(sv);
        const uint4 iv = lds128(xi);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 w = lds128(wb + h * 512u);
            int d[4];
            float flo, fhi;
            const float inv = __uint_as_float(h ? iv.w : iv.y);
            if (BITS == 4) {
                const uint4 x = lds128(xb + h * GB);
                imma_us0(d, w.x & M, w.z & M, w.y & M, w.w & M, x.x, x.y);
                imma_us(d, (w.x >> 4) & M, (w.z >> 4) & M, (w.y >> 4) & M, (w.w >> 4) & M, x.z, x.w);
                flo = (float)(d[0] * mulA + d[1] * mulB) * inv; fhi = (float)(d[2] * mulA + d[3] * mulB) * inv;
            } else {
                const uint2 x = lds64(xb + h * GB);
                imma_us0(d, w.x, w.z, w.y, w.w, x.x, x.y);
                flo = fmaf((float)d[1], fB, (float)d[0] * fA) * inv; fhi = fmaf((float)d[3], fB, (float)d[2] * fA) * inv;
            }
            lo = fmaf(h ? bf_hi(s2.x) : bf_lo(s2.x), flo, lo);
            hi = fmaf(h ? bf_hi(s2.y) : bf_lo(s2.y), fhi, hi);
        }
    }
    const uint4 own = lds128(ub + 4096u);
    const uint4 xo = lds128(xi0 + (uint32_t)sb * 64u + (uint32_t)t * 16u);
    const float X0 = __uint_as_float(xo.x), X1 = __uint_as_float(xo.z);
    lo = fmaf(bf_lo(own.z), X0, lo); lo = fmaf(bf_hi(own.z), X1, lo);
    hi = fmaf(bf_lo(own.w), X0, hi); hi = fmaf(bf_hi(own.w), X1, hi);
    return make_float2(lo, hi);
}

template <int BITS>
__device__ __forceinline__ void unit_compute(uint32_t ub, const StreamSmem &sm, int sb, int lane, float &acc_lo, float &acc_hi) {
    if constexpr (BITS == 16) unit_compute_bf16(ub, sm, sb, lane, acc_lo, acc_hi);
    else unit_compute_qc<BITS>(ub, sm, sb, lane, acc_lo, acc_hi);
}

// ------------------------------------------------------------------ per-warp unit stream
// Work split.  The host picks `lsplit`: S = 2^lsplit warps of a block share one row tile and split its K range (S = 1: a
// warp owns whole tiles).  A block of W warps works on W / S tiles per round: block b, round r takes tiles
// (r * grid + b) * (W / S) + [0, W / S); warp w handles tile slot w / S, part w % S, i.e. super-blocks
// [part * nsb / S, (part + 1) * nsb / S) of that tile -- a run of units that is contiguous in memory.  The parts of a tile
// are summed in part order through shared memory by the part-0 warp (deterministic), which then runs the epilogue.
struct StreamPlan {
    TiledW W;
    int stages;             // ring depth per warp (FK_STAGES)
    int lsplit;             // log2 of the warps sharing a tile
    unsigned long long *timeline;   // optional [grid][8] phase timestamps (ns) for tuning; null in normal use
};
__device__ __forceinline__ void stamp(const StreamPlan &p, int slot) {
    if (p.timeline && threadIdx.x == 0) {
        unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.timeline[blockIdx.x * 8 + slot] = t;
    }
}
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_a(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s_a(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// bounded wait on a barrier given by shared address: returns false if it never completed
__device__ __forceinline__ bool mbar_wait_a(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < FK_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
// A warp's ring and its walk over the runs: the producer fetches the same sequence of units the consumer takes, FK_STAGES
// units ahead.  `fetched` / `consumed` count units since the barriers were initialised: they name the ring slot
// (count % FK_STAGES) and the barrier phase.
struct WarpStream {
    const uint4 *src;           // next unit to fetch
    size_t jump;                // vectors from the end of a run to the start of the next run of this warp
    uint32_t bar, ring;         // shared addresses of stage 0's barrier and slot
    int p_tile, p_left;         // producer: tile of the run being fetched (>= ntiles: nothing left), units left in it
    int cnt, tstep, ntiles;     // units per run, tile stride between rounds
    int uvec, fetched, consumed;
    bool announced;
    __device__ __forceinline__ bool valid() const { return p_tile < ntiles; }
    __device__ __forceinline__ void issue() {
        const uint32_t s = (uint32_t)fetched & (FK_STAGES - 1);
        if ((threadIdx.x & 31) == 0) {
            mbar_expect_tx_a(bar + s * 8u, (uint32_t)uvec * 16u);
            bulk_g2s_a(ring + s * (uint32_t)FK_UNIT_BYTES, src, (uint32_t)uvec * 16u, bar + s * 8u);
        }
        ++fetched; src += uvec;
        if (--p_left == 0) { p_tile += tstep; p_left = cnt; src += jump; }
    }
    // everything this warp needs is in flight: let the next kernel start
    __device__ __forceinline__ void drained() {
        if (announced) return;
        announced = true; pdl_launch_dependents();
    }
};
// before griddepcontrol.wait: barriers up, ring filled with the warp's first units
__device__ __forceinline__ void stream_begin(WarpStream &ws, const StreamPlan &p, const StreamSmem &sm) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int ls = p.lsplit, part = wid & ((1 << ls) - 1), slot = wid >> ls, tpb = nw >> ls, nsb = p.W.nsb;
    const int sb0 = (part * nsb) >> ls, sb1 = ((part + 1) * nsb) >> ls;
    ws.uvec = unit_vec(p.W.bits); ws.cnt = sb1 - sb0; ws.ntiles = p.W.ntiles; ws.tstep = (int)gridDim.x * tpb;
    ws.p_tile = ws.cnt > 0 ? (int)blockIdx.x * tpb + slot : ws.ntiles; ws.p_left = ws.cnt;
    if (ws.p_tile > ws.ntiles) ws.p_tile = ws.ntiles;
    ws.src = p.W.units + ((size_t)ws.p_tile * nsb + sb0) * ws.uvec;
    ws.jump = ((size_t)ws.tstep * nsb - (size_t)ws.cnt) * ws.uvec;
    ws.bar = smem_u32(sm.bars + wid * FK_STAGES); ws.ring = smem_u32(sm.ring + (size_t)wid * FK_STAGES * FK_UNIT_VEC);
    ws.fetched = ws.consumed = 0; ws.announced = false;
    if (lane == 0) { for (int s = 0; s < FK_STAGES; ++s) mbar_init(sm.bars + wid * FK_STAGES + s, 1); mbar_fence_init(); }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < FK_STAGES; ++s) if (ws.valid()) ws.issue();
}

// Walk the block's rounds of the weight; `epi(tile, g, v_lo, v_hi)` receives the finished sums of tile rows g and g + 8 on
// lanes with (lane & 3) == 0 of the warp that owns (or folds) the tile.  Returns false if a barrier wait expired.
// Every warp of the block must call this: the warps sharing a tile meet at a named barrier once per round.
template <int BITS, class Epi>
__device__ __forceinline__ bool stream_run(WarpStream &ws, const StreamPlan &p, const StreamSmem &sm, Epi &epi) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5, g = lane >> 2, t = lane & 3;
    const int ls = p.lsplit, S = 1 << ls, part = wid & (S - 1), slot = wid >> ls, tpb = nw >> ls, nsb = p.W.nsb;
    const int sb0 = (part * nsb) >> ls, ntiles = p.W.ntiles;
    const uint32_t lane_off = (uint32_t)lane * 16u;
    bool ok = true;
    if (!ws.valid()) ws.drained();
    // what the epilogue of this lane's first tile needs from global memory (residual, bias) or from slow math (RoPE
    // angle) is fetched now, under the wait for the first unit, instead of after the last one
    if (t == 0 && part == 0 && (int)blockIdx.x * tpb + slot < ntiles) epi.prefetch((int)blockIdx.x * tpb + slot, g);
    int round = 0;
    for (int tb = (int)blockIdx.x * tpb; tb < ntiles; tb += ws.tstep, ++round) {
        const int tile = tb + slot;
        float acc_lo = 0.0f, acc_hi = 0.0f;
        if (tile < ntiles && ok) {
            int sb = sb0;
            for (int n = ws.cnt; n > 0; --n, ++sb) {
                const uint32_t s = (uint32_t)ws.consumed & (FK_STAGES - 1);
                if (!mbar_wait_a(ws.bar + s * 8u, ((uint32_t)ws.consumed / FK_STAGES) & 1u)) { ok = false; break; }
                if (BITS != 16 && ws.cnt <= FK_ROLLED_UPTO) {
                    const float2 r2 = unit_compute_qc_rolled<BITS == 16 ? 4 : BITS>(ws.ring + s * (uint32_t)FK_UNIT_BYTES + lane_off, smem_u32(sm.xs), smem_u32(sm.xsi), sb, lane, acc_lo, acc_hi);
                    acc_lo = r2.x; acc_hi = r2.y;
                } else
                    unit_compute<BITS>(ws.ring + s * (uint32_t)FK_UNIT_BYTES + lane_off, sm, sb, lane, acc_lo, acc_hi);
                __syncwarp();
                ++ws.consumed;
                if (ws.valid()) { ws.issue(); if (!ws.valid()) ws.drained(); }      // refill the stage just drained
            }
            acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 1); acc_lo += __shfl_xor_sync(0xffffffffu, acc_lo, 2);
            acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 1); acc_hi += __shfl_xor_sync(0xffffffffu, acc_hi, 2);
        }
        if (S == 1) { if (t == 0 && tile < ntiles) epi(tile, g, acc_lo, acc_hi); continue; }
        // the parts of a tile through shared memory (two buffers: a warp may be one round ahead of the folding warp)
        float *fold = sm.fold + ((round & 1) * FK_STREAM_MAXWARPS + slot * S) * 16;
        if (t == 0) { fold[part * 16 + g] = acc_lo; fold[part * 16 + 8 + g] = acc_hi; }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(S * 32) : "memory");
        if (part == 0 && t == 0 && tile < ntiles) {
            float lo = 0.0f, hi = 0.0f;
            for (int q = 0; q < S; ++q) { lo += fold[q * 16 + g]; hi += fold[q * 16 + 8 + g]; }
            epi(tile, g, lo, hi);
        }
    }
    return ok;
}

// ------------------------------------------------------------------ repack / probe kernels
struct SrcW { const uint32_t *w; const uint16_t *s, *b; };
// one thread per destination vector; sources are MLX-affine rows (src/fusion/ir.rs:236-247)
__global__ void k_repack_tiled(SrcW a, SrcW bsrc, uint4 *dst, long long n_src, int k, int bits, int ntiles, int nsb,
                               int rows_kind, int hd, int n_rot) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)ntiles * nsb * FK_UNIT_VEC) return;
    const int e = (int)(idx % FK_UNIT_VEC); const long long unit = idx / FK_UNIT_VEC;
    const int tile = (int)(unit / nsb), sb = (int)(unit % nsb);
    const int per_word = 32 / bits, kpg = bits == 4 ? 64 : 32;       // activations per nibble group
    const int words_per_row = k / per_word, groups_per_row = k / 64;
    const int lane = e & 31, g = lane >> 2, t = lane & 3;
    const long long r0 = tile_row(rows_kind, hd, n_rot, tile, g), r1 = tile_row(rows_kind, hd, n_rot, tile, g + 8);
    const SrcW &s0 = a, &s1 = (rows_kind == FK_ROWS_GATE_UP) ? bsrc : a;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (e < 256) {
        const int j = e >> 5;
        const int kA = sb * 8 * kpg + j * kpg + per_word * t, kB = kA + kpg / 2;
        if (r0 < n_src) { if (kA < k) out.x = s0.w[r0 * words_per_row + kA / per_word]; if (kB < k) out.y = s0.w[r0 * words_per_row + kB / per_word]; }
        if (r1 < n_src) { if (kA < k) out.z = s1.w[r1 * words_per_row + kA / per_word]; if (kB < k) out.w = s1.w[r1 * words_per_row + kB / per_word]; }
    } else {
        uint32_t sv[4] = {0, 0, 0, 0}, bv[4] = {0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int kk = (sb * 8 + 2 * t + q) * kpg;            // first activation of nibble group 2t+q
            if (kk < k) {
                const int gi = kk / 64;
                if (r0 < n_src) { sv[q] = s0.s[r0 * groups_per_row + gi]; bv[q] = s0.b[r0 * groups_per_row + gi]; }
                if (r1 < n_src) { sv[2 + q] = s1.s[r1 * groups_per_row + gi]; bv[2 + q] = s1.b[r1 * groups_per_row + gi]; }
            }
        }
        out.x = sv[0] | (sv[1] << 16); out.y = sv[2] | (sv[3] << 16); out.z = bv[0] | (bv[1] << 16); out.w = bv[2] | (bv[3] << 16);
    }
    dst[idx] = out;
}

// bf16 rows [n_src][k] -> units of 16 rows x 128 activations as mma.m16n8k16 A fragments: vector (step s, lane (g, t)) =
// {W[r0][k..k+1], W[r1][k..k+1], W[r0][k+8..k+9], W[r1][k+8..k+9]} with k = sb * 128 + 16 s + 2 t, r0/r1 = tile rows g, g + 8
__global__ void k_repack_tiled16(const uint16_t *a, const uint16_t *bsrc, uint4 *dst, long long n_src, int k, int ntiles, int nsb,
                                 int rows_kind, int hd, int n_rot) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)ntiles * nsb * 256) return;
    const int e = (int)(idx & 255); const long long unit = idx >> 8;
    const int tile = (int)(unit / nsb), sb = (int)(unit % nsb);
    const int s8 = e >> 5, lane = e & 31, g = lane >> 2, t = lane & 3;
    const long long r0 = tile_row(rows_kind, hd, n_rot, tile, g), r1 = tile_row(rows_kind, hd, n_rot, tile, g + 8);
    const uint16_t *s0 = a, *s1 = (rows_kind == FK_ROWS_GATE_UP) ? bsrc : a;
    const int kk = sb * 128 + s8 * 16 + 2 * t;
    auto pair = [&](const uint16_t *src, long long r, int kq) -> uint32_t {
        if (r >= n_src || kq >= k) return 0u;
        return (uint32_t)src[r * k + kq] | ((uint32_t)src[r * k + kq + 1] << 16);
    };
    dst[idx] = make_uint4(pair(s0, r0, kk), pair(s1, r1, kk), pair(s0, r0, kk + 8), pair(s1, r1, kk + 8));
}
__global__ void k_dequant_tiled16(TiledW W, int which, long long row0, long long nrows, float *out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)W.ntiles * W.nsb * 256) return;
    const int e = (int)(idx & 255); const long long unit = idx >> 8;
    const int tile = (int)(unit / W.nsb), sb = (int)(unit % W.nsb);
    const int s8 = e >> 5, lane = e & 31, g = lane >> 2, t = lane & 3;
    const uint4 w = W.units[(size_t)unit * 256 + e];
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int r = g + ((q & 1) ? 8 : 0);
        if (W.rows_kind == FK_ROWS_GATE_UP && ((r >= 8) != (which == 1))) continue;
        const long long src = tile_row(W.rows_kind, W.hd, W.n_rot, tile, r);
        if (src < row0 || src >= row0 + nrows) continue;
        const int kk = sb * 128 + s8 * 16 + 2 * t + ((q >= 2) ? 8 : 0);
        if (kk < W.k) out[(src - row0) * W.k + kk] = bf_lo(words[q]);
        if (kk + 1 < W.k) out[(src - row0) * W.k + kk + 1] = bf_hi(words[q]);
    }
}

// fp32 dequantised values scattered back to source order: out[(row - row0) * k + col] for rows of matrix `which`
// (0 = first / only source, 1 = the up matrix of a gate/up pair)
__global__ void k_dequant_tiled(TiledW W, int which, long long row0, long long nrows, float *out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)W.ntiles * W.nsb * 256) return;
    const int e = (int)(idx & 255); const long long unit = idx >> 8;
    const int tile = (int)(unit / W.nsb), sb = (int)(unit % W.nsb);
    const int j = e >> 5, lane = e & 31, g = lane >> 2, t = lane & 3;
    const int per_word = 32 / W.bits, kpg = W.bits == 4 ? 64 : 32;
    const uint4 *u = W.units + (size_t)unit * FK_UNIT_VEC;
    const uint4 w = u[j * 32 + lane];
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    const int jl = j >> 1;                                   // the lane (t = j/2) holding this group's scale pair
    const uint4 sb4 = u[256 + (g << 2) + jl];
    const uint32_t mask = (1u << W.bits) - 1u;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int r = g + (q >= 2 ? 8 : 0);
        if (W.rows_kind == FK_ROWS_GATE_UP && ((r >= 8) != (which == 1))) continue;
        const long long src = tile_row(W.rows_kind, W.hd, W.n_rot, tile, r);
        if (src < row0 || src >= row0 + nrows) continue;
        const uint32_t sp = (q >= 2) ? sb4.y : sb4.x, bp = (q >= 2) ? sb4.w : sb4.z;
        const float s = (j & 1) ? bf_hi(sp) : bf_lo(sp), b = (j & 1) ? bf_hi(bp) : bf_lo(bp);
        const int kbase = sb * 8 * kpg + j * kpg + per_word * t + ((q & 1) ? kpg / 2 : 0);
        for (int i = 0; i < per_word; ++i) {
            const int kk = kbase + i;
            if (kk < W.k) out[(src - row0) * W.k + kk] = __fadd_rn(__fmul_rn((float)((words[q] >> (i * W.bits)) & mask), s), b);
        }
    }
}

// ================================================================ streamed kernels

struct SLinArgs { const uint16_t *x; StreamPlan P; const uint16_t *residual; uint16_t *y; float *y_f32; int k, n; PeerXchg push;
                  const uint4 *xdig; const uint2 *xdig_xsi; };       // x once more, already as digits + (sum, 1 / scale) pairs (see SGateUpArgs)
// staging by copy: the digits of all k activations (3 bytes each) and the per-group pairs, prepared by the producing kernel
template <int BITS>
__device__ __forceinline__ void stage_copy(const StreamSmem &sm, const uint4 *dig, const uint2 *xsi, int k) {
    const int n16 = (k * 3) >> 4, np = k / (BITS == 4 ? 64 : 32);              // 16-byte vectors of digits; (sum, inv) pairs
    uint4 *xs = reinterpret_cast<uint4 *>(sm.xs); uint2 *xp = reinterpret_cast<uint2 *>(sm.xsi);
    for (int i0 = 0; i0 < n16; i0 += 8 * (int)blockDim.x) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { const int i = i0 + u * (int)blockDim.x + (int)threadIdx.x; v[u] = i < n16 ? __ldcg(dig + i) : make_uint4(0, 0, 0, 0); }
#pragma unroll
        for (int u = 0; u < 8; ++u) { const int i = i0 + u * (int)blockDim.x + (int)threadIdx.x; if (i < n16) xs[i] = v[u]; }
    }
    for (int i = threadIdx.x; i < np; i += blockDim.x) xp[i] = __ldcg(xsi + i);
    __syncthreads();
}
// Epilogues are functors: prefetch(tile, g) is called once per lane (lanes with (lane & 3) == 0) for the first tile the
// lane will finish, before the streaming loop; operator() gets the finished sums of tile rows g and g + 8.

// y = T(acc + float(residual)) (src/codegen/msl.rs:2759-2775); residual optional; optional fp32 copy of acc
struct EpiLinear {
    const SLinArgs &a; float res[2]; int ptile; uint32_t seq;
    __device__ __forceinline__ EpiLinear(const SLinArgs &a_, uint32_t seq_) : a(a_), ptile(-1), seq(seq_) { res[0] = res[1] = 0.0f; }
    __device__ __forceinline__ void prefetch(int tile, int g) {
        ptile = tile;
#pragma unroll
        for (int q = 0; q < 2; ++q) { const int r = tile * 16 + g + 8 * q; res[q] = (a.residual && r < a.n) ? bf2f(__ldcg(a.residual + r)) : 0.0f; }
    }
    __device__ __forceinline__ void operator()(int tile, int g, float lo, float hi) {
        if (tile != ptile) prefetch(tile, g);
        const float v[2] = {lo, hi};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int r = tile * 16 + g + 8 * q;
            if (r >= a.n) continue;
            if (a.y_f32) a.y_f32[r] = v[q];
            if (a.y) a.y[r] = f2bf(v[q] + res[q]);
            if (a.push.site >= 0) peer_store_pair(a.push, r, __float_as_uint(v[q]), seq);     // row-split projection: the fp32 partial goes to every rank
        }
    }
};
template <int BITS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS) k_s_linear(FkState *st, SLinArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    const StreamSmem sm = stream_carve(smem_stream, a.P.W.nsb, a.P.stages, BITS);
    stamp(a.P, 0);
    WarpStream ws; stream_begin(ws, a.P, sm);
    stage_pad<BITS>(sm, a.k, a.P.W.nsb);
    pdl_wait();
    stamp(a.P, 1);
    bool copied = false;
    if constexpr (BITS != 16) if (a.xdig) { stage_copy<BITS>(sm, a.xdig, a.xdig_xsi, a.k); copied = true; }
    if (!copied) stage_plain<BITS, (WARPS == 16 ? 5 : 2)>(sm, a.x, a.k, a.P.W.nsb);
    stamp(a.P, 2);
    EpiLinear epi(a, st->epoch + 1u);
    if (!stream_run<BITS>(ws, a.P, sm, epi)) atomicOr(&st->error, 0x100u);
    pdl_launch_dependents();
    __syncthreads(); stamp(a.P, 3);
}

struct SQkvArgs {
    const uint16_t *x, *norm_w; StreamPlan P; const uint16_t *lin_bias;
    uint16_t *q_out, *cache_k, *cache_v, *k_out, *v_out;
    const uint16_t *pending, *pending_w; uint16_t *h_out;
    int h, n_q, n_kv, hd, capacity, sinks; float eps, log2theta; const float *pend_sum; PeerXchg pull;
    QkvAttend att;          // att.out != null: decode attention over the cache as the kernel's tail (fk_attend.cuh)
};
// cos and sin of the RoPE angle of dim d at position pos: inv = exp2(-(d / half) * log2(theta)) (rope_kv_cache_store_decode.rs)
__device__ __forceinline__ void rope_angle(int d, int half, uint32_t pos, float log2theta, float *c, float *s) {
    const float e = __fmul_rn(-__fdiv_rn((float)d, (float)half), log2theta);
    const float ang = __fmul_rn((float)pos, exp2f(e));
    sincosf(ang, s, c);
}
__device__ __forceinline__ void rope_apply(float lo, float hi, float c, float s, uint16_t *o_lo, uint16_t *o_hi) {
    *o_lo = f2bf(__fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)));
    *o_hi = f2bf(__fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s)));
}
__device__ __forceinline__ void rope_rotate(float lo, float hi, int d, int half, uint32_t pos, float log2theta, uint16_t *o_lo, uint16_t *o_hi) {
    float c, s; rope_angle(d, half, pos, log2theta, &c, &s);
    rope_apply(lo, hi, c, s, o_lo, o_hi);
}
// RMSNorm -> QKV (+bias) -> RoPE -> K/V into the live cache (src/codegen/kernels/rmsnorm_qkv.rs:616-726).  With sinks the
// weight rows are tiled as RoPE pairs, so a lane owns dims d and d + head_dim/2 of one head.
struct EpiQkv {
    const SQkvArgs &a; uint32_t pos; int wrow, ptile; float b0, b1, cs, sn;
    __device__ __forceinline__ EpiQkv(const SQkvArgs &a_, uint32_t pos_) : a(a_), pos(pos_), wrow((int)(pos_ % (uint32_t)a_.capacity)), ptile(-1), b0(0.0f), b1(0.0f), cs(1.0f), sn(0.0f) {}
    __device__ __forceinline__ int nrows() const { return (a.n_q + 2 * a.n_kv) * a.hd; }
    __device__ __forceinline__ void store(int r, uint16_t v) const {
        const int nq_rows = a.n_q * a.hd, nqk = (a.n_q + a.n_kv) * a.hd;
        if (r < nq_rows) a.q_out[r] = v;
        else if (r < nqk) {
            const int kr = r - nq_rows, kh = kr / a.hd, d = kr - kh * a.hd;
            if (a.sinks) a.cache_k[((size_t)kh * a.capacity + wrow) * a.hd + d] = v; else a.k_out[kr] = v;
        } else if (r < nrows()) {
            const int vr = r - nqk, kh = vr / a.hd, d = vr - kh * a.hd;
            if (a.sinks) a.cache_v[((size_t)kh * a.capacity + wrow) * a.hd + d] = v; else a.v_out[vr] = v;
        }
    }
    __device__ __forceinline__ void prefetch(int tile, int g) {
        ptile = tile;
        const int r0 = (int)tile_row(a.P.W.rows_kind, a.hd, a.P.W.n_rot, tile, g), r1 = (int)tile_row(a.P.W.rows_kind, a.hd, a.P.W.n_rot, tile, g + 8);
        b0 = (a.lin_bias && r0 < nrows()) ? bf2f(a.lin_bias[r0]) : 0.0f;
        b1 = (a.lin_bias && r1 < nrows()) ? bf2f(a.lin_bias[r1]) : 0.0f;
        if (a.sinks && tile < a.P.W.n_rot / 16) rope_angle(r0 % a.hd, a.hd >> 1, pos, a.log2theta, &cs, &sn);
    }
    __device__ __forceinline__ void operator()(int tile, int g, float lo, float hi) {
        if (tile != ptile) prefetch(tile, g);
        const int r0 = (int)tile_row(a.P.W.rows_kind, a.hd, a.P.W.n_rot, tile, g), r1 = (int)tile_row(a.P.W.rows_kind, a.hd, a.P.W.n_rot, tile, g + 8);
        lo += b0; hi += b1;
        if (a.sinks && tile < a.P.W.n_rot / 16) {
            uint16_t o0, o1; rope_apply(rT(lo), rT(hi), cs, sn, &o0, &o1);
            store(r0, o0); store(r1, o1);
        } else { store(r0, f2bf(lo)); store(r1, f2bf(hi)); }
    }
};
// ATT: the instance that can carry the attention tail (a kernel of its own, so that the call does not cost the plain form
// registers or a stack frame)
template <int BITS, int WARPS, bool PEND = false, bool ATT = false>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS) k_s_rmsnorm_qkv(FkState *st, SQkvArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    const StreamSmem sm = stream_carve(smem_stream, a.P.W.nsb, a.P.stages, BITS);
    stamp(a.P, 0);
    WarpStream ws; stream_begin(ws, a.P, sm);
    stage_pad<BITS>(sm, a.h, a.P.W.nsb);
    NormW nwv; norm_w_load(nwv, a.norm_w, a.h);
    pdl_wait();
    stamp(a.P, 1);
    stage_rmsnorm<BITS, PEND>(sm, a.x, nwv, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, a.P.timeline, a.pend_sum, &a.pull, st);
    stamp(a.P, 2);
    const uint32_t pos = st->offset;
    EpiQkv epi(a, pos);
    if (!stream_run<BITS>(ws, a.P, sm, epi)) atomicOr(&st->error, 0x200u);
    pdl_launch_dependents();
    if constexpr (ATT) if (a.att.out) {        // a warp's ring slots are its own again; the staged activations are dead after the first hand-off
        unsigned char *tiles = reinterpret_cast<unsigned char *>(sm.ring);
        constexpr int stride_w = FK_STAGES * (BITS == 16 ? 256 : FK_UNIT_VEC) * 16;
        if (a.hd == 128) qkv_attend<128>(a.att, st, a.q_out, a.cache_k, a.cache_v, a.n_q, a.n_kv, a.capacity, pos, tiles, stride_w, tiles + SdpaMmaLayout<128>::WTILE);
        else qkv_attend<64>(a.att, st, a.q_out, a.cache_k, a.cache_v, a.n_q, a.n_kv, a.capacity, pos, tiles, stride_w, tiles + SdpaMmaLayout<64>::WTILE);
    }
    __syncthreads(); stamp(a.P, 3);
}

struct SGateUpArgs {
    const uint16_t *x, *norm_w; StreamPlan P; uint16_t *act_out;
    const uint16_t *pending, *pending_w; uint16_t *h_out;
    int h, inter, act; float eps; const float *pend_sum; PeerXchg pull;
    // optional: the activation vector again as the integer digits the next projection (down_proj, same bit width) stages --
    // [groups][digits] in the shared-memory layout of store_block, then the (sum, 1 / scale) pairs -- so that its 112+ blocks
    // copy 3 bytes per activation instead of each converting all of them (2.9 us of staging per layer on the 7B shape)
    uint32_t *dig_out; float2 *dig_xsi;
};
__device__ __forceinline__ uint16_t s_act_swiglu(float ga, float ua) {
    const float g = rT(ga), u = rT(ua);
    return f2bf((__fdiv_rn(1.0f, 1.0f + expf(-g)) * g) * u);
}
__device__ __forceinline__ uint16_t s_act_geglu(float ga, float ua) {
    const float g = rT(ga), u = rT(ua);
    const float g3 = rT(rT(g * g) * g);
    const float t2 = rT(g + rT(0.044715f * g3));
    const float t3 = rT(0.7978845608028654f * t2);
    const float t4 = rT(tanhf(fminf(fmaxf(t3, -20.0f), 20.0f)));
    return f2bf(rT(rT(0.5f * g) * rT(1.0f + t4)) * u);
}
// RMSNorm -> gate & up -> activation tail in registers (src/codegen/kernels/fused_chain.rs:2902-3552; msl.rs:1286-1294).
// The paired weight interleaves 8 gate rows with the 8 matching up rows per tile, so a lane holds both.
struct EpiGateUp {
    const SGateUpArgs &a; uint16_t *stash;       // stash: the block's own outputs, [round][warp][8], for the digit pass (or null)
    __device__ __forceinline__ EpiGateUp(const SGateUpArgs &a_, uint16_t *stash_) : a(a_), stash(stash_) {}
    __device__ __forceinline__ void prefetch(int, int) {}
    __device__ __forceinline__ void operator()(int tile, int g, float gate, float up) {
        const int r = tile * 8 + g;
        const uint16_t v = a.act == 1 ? s_act_geglu(gate, up) : s_act_swiglu(gate, up);
        if (r < a.inter) a.act_out[r] = v;
        if (stash) {                              // whole tiles per warp (no K split): tile = (round * grid + block) * warps + warp
            const int nw = (int)blockDim.x >> 5, lt = tile - (int)blockIdx.x * nw, span = (int)gridDim.x * nw, round = lt / span;
            stash[(round * nw + (lt - round * span)) * 8 + g] = r < a.inter ? v : (uint16_t)0;
        }
    }
};
// after the last round: the stashed outputs of this block, eight (one tile) per thread, as digits in global memory
template <int BITS>
__device__ __forceinline__ void gateup_digits(const SGateUpArgs &a, const uint16_t *stash) {
    const int nw = (int)blockDim.x >> 5, ntiles = a.P.W.ntiles, span = (int)gridDim.x * nw, first = (int)blockIdx.x * nw;
    const int rounds = first < ntiles ? (ntiles - first + span - 1) / span : 0, total = rounds * nw;
    // whole warps take 32 tiles at a time (store_block_to shuffles across the warp: every lane of a warp that enters takes part);
    // warps with nothing to do skip the pass
    for (int i0 = (int)(threadIdx.x & ~31u); i0 < total; i0 += (int)blockDim.x) {
        const int i = i0 + (int)(threadIdx.x & 31u), round = i / nw, tile = (round * (int)gridDim.x + (int)blockIdx.x) * nw + (i - round * nw);
        const bool valid = i < total && tile < ntiles && tile * 8 < a.inter;
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = valid ? bf2f(stash[i * 8 + j]) : 0.0f;
        store_block_to<BITS>(a.dig_out, a.dig_xsi, valid ? tile : 0, f, valid);
    }
}
template <int BITS, int WARPS, bool PEND = false>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS) k_s_gateup(FkState *st, SGateUpArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    const StreamSmem sm = stream_carve(smem_stream, a.P.W.nsb, a.P.stages, BITS);
    stamp(a.P, 0);
    WarpStream ws; stream_begin(ws, a.P, sm);
    stage_pad<BITS>(sm, a.h, a.P.W.nsb);
    if (BITS != 16 && a.dig_out) for (int i = threadIdx.x; i < 2 * FK_STREAM_MAXWARPS * 16; i += blockDim.x) sm.fold[i] = 0.0f;
    NormW nwv; norm_w_load(nwv, a.norm_w, a.h);
    pdl_wait();
    stamp(a.P, 1);
    stage_rmsnorm<BITS, PEND>(sm, a.x, nwv, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, a.P.timeline, a.pend_sum, &a.pull, st);
    stamp(a.P, 2);
    uint16_t *stash = (BITS != 16 && a.dig_out) ? reinterpret_cast<uint16_t *>(sm.fold) : nullptr;     // the fold buffer is idle without a K split
    EpiGateUp epi(a, stash);
    if (!stream_run<BITS>(ws, a.P, sm, epi)) atomicOr(&st->error, 0x400u);
    pdl_launch_dependents();
    __syncthreads();
    if constexpr (BITS != 16) if (stash) gateup_digits<BITS>(a, stash);
    stamp(a.P, 3);
}

struct SHeadArgs {
    const uint16_t *x, *norm_w; StreamPlan P; uint16_t *logits; unsigned long long *scratch; uint32_t *counter;
    const uint16_t *pending, *pending_w; uint16_t *h_out; uint32_t *history;
    int h, v, vocab_offset, finalize; float eps; const float *pend_sum; PeerXchg pull, amax;
};
__device__ __forceinline__ void s_finalize_token(FkState *st, uint32_t *history, unsigned long long best) {
    const uint32_t next = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
    st->token[0] = next;
    if (history && st->hist_counter < st->hist_cap) history[st->hist_counter] = next;
    st->hist_counter += 1;
    st->offset += 1;
    st->epoch += 1;
}
struct EpiHead {
    const SHeadArgs &a; unsigned long long best;
    __device__ __forceinline__ EpiHead(const SHeadArgs &a_) : a(a_), best(0ull) {}
    __device__ __forceinline__ void prefetch(int, int) {}
    __device__ __forceinline__ void operator()(int tile, int g, float lo, float hi) {
        const float v[2] = {lo, hi};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int r = tile * 16 + g + 8 * q;
            if (r >= a.v) continue;
            const uint16_t tb = f2bf(v[q]);
            if (a.logits) a.logits[r] = tb;
            const unsigned long long key = argmax_key(tb, (uint32_t)(r + a.vocab_offset));
            best = key > best ? key : best;
        }
    }
};
// final RMSNorm -> lm_head -> argmax on T-rounded logits, ties to the lowest index, no logits round trip
// (final_rmsnorm_lm_head.rs:250-326; msl.rs:1805-1838); the last block folds the per-block keys and advances the state
template <int BITS, int WARPS, bool PEND = false>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS) k_s_head(FkState *st, SHeadArgs a) {
    extern __shared__ __align__(128) unsigned char smem_stream[];
    const StreamSmem sm = stream_carve(smem_stream, a.P.W.nsb, a.P.stages, BITS);
    __shared__ unsigned long long wbest[WARPS]; __shared__ int is_last;
    stamp(a.P, 0);
    WarpStream ws; stream_begin(ws, a.P, sm);
    stage_pad<BITS>(sm, a.h, a.P.W.nsb);
    NormW nwv; norm_w_load(nwv, a.norm_w, a.h);
    pdl_wait();
    stamp(a.P, 1);
    stage_rmsnorm<BITS, PEND>(sm, a.x, nwv, a.h, a.P.W.nsb, a.eps, a.pending, a.pending_w, a.h_out, a.P.timeline, a.pend_sum, &a.pull, st);
    stamp(a.P, 2);
    EpiHead epi(a);
    const bool ok = stream_run<BITS>(ws, a.P, sm, epi);
    unsigned long long best = epi.best;
    pdl_launch_dependents();
    if (!ok) atomicOr(&st->error, 0x800u);
    stamp(a.P, 3);
    best = warp_max_u64(best);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) wbest[wid] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < WARPS; ++i) best = wbest[i] > best ? wbest[i] : best;
        a.scratch[blockIdx.x] = best;
        __threadfence();
        const uint32_t tk = atomicAdd(a.counter, 1u);
        is_last = (tk == gridDim.x - 1);
        if (is_last) *a.counter = 0u;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (wid == 0) {
        unsigned long long b = 0ull;
        for (int i = lane; i < (int)gridDim.x; i += 32) { const unsigned long long v = __ldcg(a.scratch + i); b = v > b ? v : b; }
        b = warp_max_u64(b);
        if (a.amax.site >= 0) {
            // vocabulary-sharded head: this rank's best key goes to every rank (two (word, sequence) pairs), then every rank
            // takes the maximum of all keys (the same on every rank) and advances its own decode state
            const uint32_t seq = st->epoch + 1u;
            if (lane == 0) {
                peer_store_pair(a.amax, 0, (uint32_t)(b & 0xffffffffull), seq);
                peer_store_pair(a.amax, 1, (uint32_t)(b >> 32), seq);
                unsigned long long best = 0ull; bool ok = true;
                for (int p = 0; p < a.amax.map.world; ++p) {
                    uint32_t lo, hi;
                    ok = peer_load_pairs(a.amax, p, 0, seq, lo, hi) && ok;
                    const unsigned long long v = ((unsigned long long)hi << 32) | lo;
                    best = v > best ? v : best;
                }
                if (!ok) atomicOr(&st->error, 0x8000u);
                s_finalize_token(st, a.history, best);
            }
            return;
        }
        if (lane == 0) { if (a.finalize) s_finalize_token(st, a.history, b); else a.scratch[0] = b; }
    }
}
