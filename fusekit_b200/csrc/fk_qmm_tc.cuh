// Quantised matrix product on the 5th-generation tensor cores (tcgen05): Y[M, N] = T(X[M, K] . dequant(W)^T + residual),
// 4-bit weights, M = 2 .. 32 activation rows.
//
// Reference: the M > 1 tiles `fusekit_qmm_*` (src/codegen/msl.rs:2318-2439, 3821-4332); like the mma.sync form in
// fk_qmm.cuh, row m of the result is what the one-row matvec gives for x[m].
//
// Mapping.  A CTA owns 128 weight rows -- the M axis of one tcgen05.mma (cta_group::1, kind::f16, bf16 operands, fp32
// accumulators in tensor memory) -- and all activation rows, which sit on the MMA's N axis (16 or 32).  K is walked one
// quantisation group (64 activations) at a time:
//   * threads 0..127 (thread r <-> weight row r) turn the group's nibbles into the bf16 numbers 128 + q, one shift and one
//     LOP3 per two weights ((w >> 4m) & 0x000F000F | 0x43004300), and store them as the A operand in the canonical K-major
//     shared-memory layout (8 x 16-byte core matrices, no swizzle); the activations of the group go beside them as the B
//     operand with the same permutation of k inside every 8 (0,4,1,5,2,6,3,7: the order the nibble pairs come out in);
//   * one thread of warp 4 issues four tcgen05.mma (K = 16 each) into one of two accumulator tiles in tensor memory and
//     commits them to an mbarrier; every product (128 + q) * x is exact in the fp32 accumulator;
//   * the same 128 threads read the finished tile back (tcgen05.ld, a thread owns its row's M values) and add
//     s * D + (b - 128 s) * sum(x_group) to the row's running results in registers, which is s * sum(q x) + b * sum(x).
// Two stages of operands and accumulators overlap the dequantisation of group g + 1 with the MMAs of group g and the
// read-back of group g - 1.  Every wait is bounded; on expiry the kernel sets error bit 0x40000, skips the rest of its work,
// frees its tensor memory and returns.
#pragma once
#include "fk_stream.cuh"

#define FK_TC_ROWS 128
#define FK_TC_MAXM 32
#define FK_TC_THREADS 160
#define FK_TC_SPIN (1u << 22)
#define FK_TC_A_BYTES (FK_TC_ROWS * 64 * 2)          // one stage of the A operand: 128 rows x 64 k, bf16
#define FK_TC_B_BYTES (FK_TC_MAXM * 64 * 2)

struct QmmTcArgs { const uint16_t *x; TiledW W; const uint16_t *residual; uint16_t *y; int m, k, n; };

__host__ __device__ inline size_t qmm_tc_smem_bytes() { return 2 * (size_t)(FK_TC_A_BYTES + FK_TC_B_BYTES) + 4 * FK_TC_MAXM * 4 + 64 + 128; }

// shared-memory matrix descriptor, K-major, no swizzle: start address, leading-dimension offset (between core matrices along
// K), stride-dimension offset (between groups of 8 rows), all in units of 16 bytes; bit 46: descriptor version of sm_100
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < FK_TC_SPIN; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
template <int NB>       // activation rows on the MMA's N axis: 16 or 32
__global__ void __launch_bounds__(FK_TC_THREADS) k_qmm_tc(FkState *st, QmmTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_tc[];
    unsigned char *sA = smem_tc;                                        // [2][128 rows x 64 k] canonical layout
    unsigned char *sB = sA + 2 * FK_TC_A_BYTES;                         // [2][NB rows x 64 k]
    // group sums of the activations, [4][FK_TC_MAXM]: a fast thread may stage group g + 3 while a slow one still reads group g
    // (it cannot reach g + 4: that needs the slow thread's operands of group g + 2), so four slots never collide
    float *xsum = reinterpret_cast<float *>(sB + 2 * FK_TC_B_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(xsum + 4 * FK_TC_MAXM);      // full[2], done[2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4);
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int nsb = a.W.nsb, G = a.k >> 6;
    const uint32_t full0 = smem_u32(bars), done0 = smem_u32(bars + 2);
    if (tid == 0) {
        mbar_init(bars + 0, FK_TC_ROWS); mbar_init(bars + 1, FK_TC_ROWS); mbar_init(bars + 2, 1); mbar_init(bars + 3, 1);
        mbar_fence_init();
    }
    if (wid == 4) {             // one warp allocates 64 columns of tensor memory: two accumulator tiles of up to 32 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_wait();
    bool ok = true;
    if (wid == 4) {
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, A and B bf16, both K-major, N = NB, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(FK_TC_ROWS >> 4) << 24);
            for (int g = 0; g < G && ok; ++g) {
                const int s = g & 1;
                if (!tc_wait(full0 + s * 8, (uint32_t)(g >> 1) & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t abase = smem_u32(sA + s * FK_TC_A_BYTES), bbase = smem_u32(sB + s * FK_TC_B_BYTES);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t ad = tc_smem_desc(abase + ks * 256, 128, 1024), bd = tc_smem_desc(bbase + ks * 256, 128, 1024);
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                 ::"r"(tmem + (uint32_t)s * 32u), "l"(ad), "l"(bd), "r"(idesc), "r"(ks) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(done0 + s * 8) : "memory");
            }
            if (!ok) atomicOr(&st->error, 0x40000u);
        }
    } else {
        const int r = tid, rt = (int)blockIdx.x * 8 + (r >> 4), rr = r & 15, gq = rr & 7, hi = rr >> 3;
        const bool row_ok = rt < a.W.ntiles;
        float acc[NB];
#pragma unroll
        for (int m = 0; m < NB; ++m) acc[m] = 0.0f;
        auto epilogue = [&](int g) {
            const int s = g & 1;
            // full[s] first: it makes the group sums written by the other producer threads visible; then the MMAs of the group
            if (!tc_wait(full0 + s * 8, (uint32_t)(g >> 1) & 1u) || !tc_wait(done0 + s * 8, (uint32_t)(g >> 1) & 1u)) { ok = false; return; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t d[NB];
            const uint32_t taddr = tmem + ((uint32_t)(wid * 32) << 16) + (uint32_t)s * 32u;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                           "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]) : "r"(taddr) : "memory");
            if (NB == 32)
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(d[NB - 16]), "=r"(d[NB - 15]), "=r"(d[NB - 14]), "=r"(d[NB - 13]), "=r"(d[NB - 12]), "=r"(d[NB - 11]), "=r"(d[NB - 10]), "=r"(d[NB - 9]),
                               "=r"(d[NB - 8]), "=r"(d[NB - 7]), "=r"(d[NB - 6]), "=r"(d[NB - 5]), "=r"(d[NB - 4]), "=r"(d[NB - 3]), "=r"(d[NB - 2]), "=r"(d[NB - 1]) : "r"(taddr + 16u) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            // scale and bias of (row, group): the unit's tail vector of lane (gq, t = j / 2), half j % 2
            float sc = 0.0f, bi = 0.0f;
            if (row_ok) {
                const int sb = g >> 3, j = g & 7;
                const uint4 sb4 = __ldg(a.W.units + ((size_t)rt * nsb + sb) * FK_UNIT_VEC + 256 + gq * 4 + (j >> 1));
                const uint32_t sw = hi ? sb4.y : sb4.x, bw = hi ? sb4.w : sb4.z;
                sc = (j & 1) ? bf_hi(sw) : bf_lo(sw); bi = (j & 1) ? bf_hi(bw) : bf_lo(bw);
            }
            const float tb = bi - 128.0f * sc;
#pragma unroll
            for (int m = 0; m < NB; ++m) acc[m] = fmaf(tb, xsum[(g & 3) * FK_TC_MAXM + m], fmaf(sc, __uint_as_float(d[m]), acc[m]));
        };
        for (int g = 0; g < G && ok; ++g) {
            const int s = g & 1, sb = g >> 3, j = g & 7;
            // ---- A operand: this row's 64 nibbles of the group as bf16 128 + q, chunk c = packed word c = k 8c .. 8c + 7
            unsigned char *A = sA + s * FK_TC_A_BYTES + (r >> 3) * 1024 + (r & 7) * 16;
            const uint4 *u = a.W.units + ((size_t)rt * nsb + sb) * FK_UNIT_VEC + j * 32 + gq * 4;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint4 v = row_ok ? __ldg(u + t) : make_uint4(0, 0, 0, 0);
                const uint32_t wa = hi ? v.z : v.x, wb = hi ? v.w : v.y;            // words t and t + 4 of the row
                *reinterpret_cast<uint4 *>(A + t * 128) = make_uint4((wa & 0x000F000Fu) | 0x43004300u, ((wa >> 4) & 0x000F000Fu) | 0x43004300u,
                                                                     ((wa >> 8) & 0x000F000Fu) | 0x43004300u, ((wa >> 12) & 0x000F000Fu) | 0x43004300u);
                *reinterpret_cast<uint4 *>(A + (t + 4) * 128) = make_uint4((wb & 0x000F000Fu) | 0x43004300u, ((wb >> 4) & 0x000F000Fu) | 0x43004300u,
                                                                           ((wb >> 8) & 0x000F000Fu) | 0x43004300u, ((wb >> 12) & 0x000F000Fu) | 0x43004300u);
            }
            // ---- B operand: chunk (activation row m, 8 consecutive k) per thread, k permuted like the nibble pairs; group sums
#pragma unroll
            for (int q = 0; q < NB / 16; ++q) {
                const int idx = r + q * 128, m = idx >> 3, c = idx & 7;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (m < a.m) v = __ldcg(reinterpret_cast<const uint4 *>(a.x + (size_t)m * a.k + (size_t)g * 64 + c * 8));
                float f[8]; unpack8(v, f);
                float sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
                sum += __shfl_xor_sync(0xffffffffu, sum, 1); sum += __shfl_xor_sync(0xffffffffu, sum, 2); sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (c == 0) xsum[(g & 3) * FK_TC_MAXM + m] = sum;
                *reinterpret_cast<uint4 *>(sB + s * FK_TC_B_BYTES + (m >> 3) * 1024 + c * 128 + (m & 7) * 16) =
                    make_uint4(__byte_perm(v.x, v.z, 0x5410u), __byte_perm(v.x, v.z, 0x7632u), __byte_perm(v.y, v.w, 0x5410u), __byte_perm(v.y, v.w, 0x7632u));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // the MMA reads the operands through the async proxy
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full0 + s * 8) : "memory");
            if (g >= 1) epilogue(g - 1);
        }
        if (ok && G >= 1) epilogue(G - 1);
        if (!ok) atomicOr(&st->error, 0x40000u);
        const int row = (int)blockIdx.x * FK_TC_ROWS + r;
        if (ok && row < a.n) {
            for (int m = 0; m < a.m; ++m) {
                const float res = a.residual ? bf2f(__ldcg(a.residual + (size_t)m * a.n + row)) : 0.0f;
                float v = 0.0f;
#pragma unroll
                for (int mm = 0; mm < NB; ++mm) if (mm == m) v = acc[mm];
                a.y[(size_t)m * a.n + row] = f2bf(v + res);
            }
        }
    }
    pdl_launch_dependents();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u) : "memory");
}

// ================================================================ warp-specialised form (M <= 16)
// The same mapping (128 weight rows on the MMA's M axis, the activation rows on N, 128 + q operands, per-group read-back),
// restructured so that nothing waits on a memory round trip:
//   warp 13      : streams the weights -- the 8 units (16 rows x 512 k each) of one super-block per stage, by 1-D TMA into a ring;
//   warps 0 .. 7 : producers; warp w turns its unit of the stage into the rows 16 w .. 16 w + 15 of the A operand, one group
//                  (64 k) at a time, into a ring of four 16 KB operand tiles; together they also stage the activations of a
//                  super-block (B operands of its 8 groups, fetched one super-block ahead) and the group sums;
//   warp 12      : one thread issues the MMAs of a group (4 x K = 16) into one of four 16-column accumulators in tensor memory
//                  and commits them to the barriers that free the operand tile and hand the accumulator over;
//   warps 8 .. 11: read an accumulator back (thread r <-> weight row r), release it, and add s * D + (b - 128 s) * sum(x_group);
//                  scales and biases come from the units' tail vectors, requested one super-block ahead.
// K can be split over `kparts` CTAs per 128-row tile: each leaves fp32 partials in the scratch area and takes a ticket; the last
// one adds the parts in part order (so the result does not depend on which CTA is last) and writes the rows.
// Every wait is bounded; on expiry error bit 0x40000 is set and the CTA winds down (tensor memory freed).
//
// Measured (B200, 16 rows, us per launch; one-row matvec / mma.sync k_qmm4 / this kernel / the one-CTA-per-tile form above):
//   5120 -> 55296: 26.6 / 65.8 / 157 / 201      27648 -> 5120: 23.8 / 38.2 / 103 / 687      5120 -> 5120: 6.3 / 12.7 / 33.5 / 128
// With its stages switched off one at a time (5120 -> 55296, 161 us): no read-back arithmetic 159, no read-back at all 161, no
// MMAs 151, no proxy fence in the producers 140, no conversion and operand stores 118, none of these 104.  Per-group
// timestamps of one CTA: a producer warp needs ~0.5 us per group (a 16 KB operand tile per 64 k: load, 28 ALU operations,
// four 16-byte stores, proxy fence, hand-off), the issuing thread ~0.3 us per group for waits, four MMAs and the commit;
// the commit reaches the read-back warps within 0.1 us and the read-back keeps up.  Two, four or eight tiles in flight, one
// or three commits per group, suspending or spinning waits: no change -- the pipeline is not latency-bound, its stages are
// simply too fine: a group is 4 KB of weights, and each hand-off costs as much as moving them.  A weight-streaming product
// with 16 rows expands its operand fourfold through shared memory for MMAs that take nanoseconds; the register-operand
// mma.sync form has no hand-offs and stays the default.
#define FK_TC2_PW 8                     // producer warps
#define FK_TC2_THREADS (14 * 32)
#define FK_TC2_RS 2                     // weight ring stages (one super-block of 8 units each)
#ifndef FK_TC2_NA
#define FK_TC2_NA 4                     // A operand tiles
#endif
#ifndef FK_TC2_NT
#define FK_TC2_NT 4                     // accumulators in tensor memory
#endif
static_assert(FK_TC2_NA == FK_TC2_NT, "an operand tile and its accumulator share one completion barrier");
#define FK_TC2_STAGE_BYTES (8 * FK_UNIT_BYTES)
#define FK_TC2_BSTAGE (8 * 2048)        // B operands of the 8 groups of a super-block (16 rows x 64 k, bf16)

struct QmmTc2Args { const uint16_t *x; TiledW W; const uint16_t *residual; uint16_t *y; float *scratch; unsigned int *counters; int m, k, n, kparts; };

__host__ __device__ inline size_t qmm_tc2_smem_bytes() {
    return (size_t)FK_TC2_RS * FK_TC2_STAGE_BYTES + (size_t)FK_TC2_NA * FK_TC_A_BYTES + 2 * (size_t)FK_TC2_BSTAGE + 2 * 8 * 16 * 4 /*group sums*/ + 256 /*barriers*/ + 1024;
}

__global__ void __launch_bounds__(FK_TC2_THREADS, 1) k_qmm_tc2(FkState *st, QmmTc2Args a) {
    extern __shared__ __align__(1024) unsigned char smem_tc2[];
    unsigned char *ring = smem_tc2;                                                     // [RS][8 units][4608]
    unsigned char *sA = ring + FK_TC2_RS * FK_TC2_STAGE_BYTES;                           // [NA][16 KB]   (1024-byte aligned: 73728 = 72 * 1024)
    unsigned char *sB = sA + FK_TC2_NA * FK_TC_A_BYTES;                                  // [2][8 groups][2 KB]
    float *xsum = reinterpret_cast<float *>(sB + 2 * FK_TC2_BSTAGE);                     // [2][8][16]
    uint64_t *bars = reinterpret_cast<uint64_t *>(xsum + 2 * 8 * 16);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + (2 * FK_TC2_RS + 2 * FK_TC2_NA + 4 + 2 * FK_TC2_NT));
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    // barriers: wfull[RS] wempty[RS] afull[NA] aempty[NA] bfull[2] bempty[2] tfull[NT] tempty[NT]
    const uint32_t b0 = smem_u32(bars);
    const uint32_t wfull = b0, wempty = b0 + 8 * FK_TC2_RS, afull = wempty + 8 * FK_TC2_RS, aempty = afull + 8 * FK_TC2_NA,
                   bfull = aempty + 8 * FK_TC2_NA, bempty = bfull + 16, tfull = bempty + 16, tempty = tfull + 8 * FK_TC2_NT;
    if (tid == 0) {
        for (int s = 0; s < FK_TC2_RS; ++s) { mbar_init(bars + s, 1); mbar_init(bars + FK_TC2_RS + s, FK_TC2_PW); }
        for (int s = 0; s < FK_TC2_NA; ++s) { mbar_init(bars + 2 * FK_TC2_RS + s, FK_TC2_PW); mbar_init(bars + 2 * FK_TC2_RS + FK_TC2_NA + s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(bars + 2 * FK_TC2_RS + 2 * FK_TC2_NA + s, FK_TC2_PW); mbar_init(bars + 2 * FK_TC2_RS + 2 * FK_TC2_NA + 2 + s, 4); }
        for (int s = 0; s < FK_TC2_NT; ++s) { mbar_init(bars + 2 * FK_TC2_RS + 2 * FK_TC2_NA + 4 + s, 1); mbar_init(bars + 2 * FK_TC2_RS + 2 * FK_TC2_NA + 4 + FK_TC2_NT + s, 4); }
        mbar_fence_init();
    }
    if (wid == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const int nsb = a.W.nsb, S = a.kparts, tile128 = (int)blockIdx.x / S, kp = (int)blockIdx.x - tile128 * S;
    const int sb0 = (int)((long long)kp * nsb / S), sb1 = (int)((long long)(kp + 1) * nsb / S), nit = sb1 - sb0;
    const int tile0 = tile128 * 8;                     // first 16-row tile of this CTA
    bool ok = true;
    if (wid == 13) {
        // ---------------------------------------------------------------- weight stream (constants: no dependency wait)
        if (lane == 0) {
            int nvalid = a.W.ntiles - tile0; nvalid = nvalid > 8 ? 8 : nvalid;
            for (int it = 0; it < nit && ok; ++it) {
                const int s = it % FK_TC2_RS;
                if (it >= FK_TC2_RS && !tc_wait(wempty + 8 * s, (uint32_t)(it / FK_TC2_RS - 1) & 1u)) { ok = false; break; }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(wfull + 8 * s), "r"((uint32_t)nvalid * FK_UNIT_BYTES) : "memory");
                for (int u = 0; u < nvalid; ++u)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_u32(ring + ((size_t)s * 8 + u) * FK_UNIT_BYTES)), "l"(a.W.units + ((size_t)(tile0 + u) * nsb + sb0 + it) * FK_UNIT_VEC),
                                   "r"((uint32_t)FK_UNIT_BYTES), "r"(wfull + 8 * s) : "memory");
            }
            if (!ok) atomicOr(&st->error, 0x40000u);
        }
    } else if (wid == 12) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(FK_TC_ROWS >> 4) << 24);
            // One thread issues everything, so its instruction count per group bounds the kernel: the group loop is unrolled -- with 8
            // groups per super-block and 4 operand tiles / accumulators, the tile, the accumulator and both barrier parities of group
            // j are compile-time constants -- and the descriptors are constants plus an offset in their address field (16-byte units).
            const uint64_t ad0 = tc_smem_desc(smem_u32(sA), 128, 1024), bd0 = tc_smem_desc(smem_u32(sB), 128, 1024);
            for (int it = 0; it < nit && ok; ++it) {
                const int bs = it & 1;
                if (!tc_wait(bfull + 8 * bs, (uint32_t)(it >> 1) & 1u)) { ok = false; break; }
                const uint64_t bdi = bd0 + (uint64_t)(bs * (FK_TC2_BSTAGE >> 4));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    constexpr int NA = FK_TC2_NA, NT = FK_TC2_NT;
                    const int ab = j % NA, tb = j % NT;
                    if (!tc_wait(afull + 8 * ab, (uint32_t)(j / NA) & 1u)) { ok = false; break; }
                    if ((it > 0 || j >= NT) && !tc_wait(tempty + 8 * tb, (uint32_t)(j / NT + 1) & 1u)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adj = ad0 + (uint64_t)(ab * (FK_TC_A_BYTES >> 4)), bdj = bdi + (uint64_t)(j * (2048 >> 4));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                                     ::"r"(tmem + (uint32_t)tb * 16u), "l"(adj + (uint64_t)(ks * 16)), "l"(bdj + (uint64_t)(ks * 16)), "r"(idesc), "r"(ks) : "memory");
                    // one commit per group (a commit costs the issuing thread about as much as the group's four MMAs): its barrier
                    // hands the accumulator to the read-back warps AND frees the operand tile for the producers (same index, NA == NT);
                    // the B stage needs no commit of its own -- by the time the producers restage it they have waited for a later group
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tfull + 8 * tb) : "memory");
                }
            }
            if (!ok) atomicOr(&st->error, 0x40000u);
        }
    } else if (wid < FK_TC2_PW) {
        // ---------------------------------------------------------------- producers
        pdl_wait();
        const int g = lane >> 2, t = lane & 3;
        uint4 xv[4];
        auto x_load = [&](int sb) {          // this thread's four 8-activation chunks of super-block sb (row m = idx / 64, chunk idx % 64)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int idx = tid + q * 256, m = idx >> 6, cc = idx & 63, k = sb * 512 + cc * 8;
                xv[q] = (m < a.m && k < a.k) ? __ldcg(reinterpret_cast<const uint4 *>(a.x + (size_t)m * a.k + k)) : make_uint4(0, 0, 0, 0);
            }
        };
        if (nit > 0) x_load(sb0);
        for (int it = 0; it < nit && ok; ++it) {
            const int s = it % FK_TC2_RS, bs = it & 1;
            // B operands and group sums of this super-block (held in registers since the previous one)
            if (it >= 2 && !tc_wait(bempty + 8 * bs, (uint32_t)(it / 2 - 1) & 1u)) { ok = false; break; }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int idx = tid + q * 256, m = idx >> 6, cc = idx & 63, j = cc >> 3, c = cc & 7;
                const uint4 v = xv[q];
                float f[8]; unpack8(v, f);
                float sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
                sum += __shfl_xor_sync(0xffffffffu, sum, 1); sum += __shfl_xor_sync(0xffffffffu, sum, 2); sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (c == 0) xsum[(bs * 8 + j) * 16 + m] = sum;
                *reinterpret_cast<uint4 *>(sB + bs * FK_TC2_BSTAGE + j * 2048 + (m >> 3) * 1024 + c * 128 + (m & 7) * 16) =
                    make_uint4(__byte_perm(v.x, v.z, 0x5410u), __byte_perm(v.x, v.z, 0x7632u), __byte_perm(v.y, v.w, 0x5410u), __byte_perm(v.y, v.w, 0x7632u));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bfull + 8 * bs) : "memory");
            if (it + 1 < nit) x_load(sb0 + it + 1);
            // the warp's unit of this stage, group by group, into the rows 16 w .. 16 w + 15 of an operand tile
            if (!tc_wait(wfull + 8 * s, (uint32_t)(it / FK_TC2_RS) & 1u)) { ok = false; break; }
            const bool unit_ok = tile0 + wid < a.W.ntiles;
            const uint32_t ub = smem_u32(ring + ((size_t)s * 8 + wid) * FK_UNIT_BYTES) + (uint32_t)lane * 16u;
            for (int j = 0; j < 8; ++j) {
                const int gi = it * 8 + j, ab = gi % FK_TC2_NA;
                if (gi >= FK_TC2_NA && !tc_wait(tfull + 8 * ab, (uint32_t)(gi / FK_TC2_NA - 1) & 1u)) { ok = false; break; }
                uint4 v = make_uint4(0, 0, 0, 0);
                if (unit_ok) v = lds128(ub + (uint32_t)j * 512u);
                // lane (g, t): v.x / v.y = words A (k 8t ..) and B (k 32 + 8t ..) of row g, v.z / v.w of row g + 8
                unsigned char *A0 = sA + ab * FK_TC_A_BYTES + (2 * wid) * 1024 + g * 16;
                const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t w = ws[q];
                    unsigned char *dst = A0 + (q >> 1) * 1024 + ((q & 1) * 4 + t) * 128;
                    *reinterpret_cast<uint4 *>(dst) = make_uint4((w & 0x000F000Fu) | 0x43004300u, ((w >> 4) & 0x000F000Fu) | 0x43004300u,
                                                                 ((w >> 8) & 0x000F000Fu) | 0x43004300u, ((w >> 12) & 0x000F000Fu) | 0x43004300u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(afull + 8 * ab) : "memory");
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(wempty + 8 * s) : "memory");
        }
        if (!ok && lane == 0) atomicOr(&st->error, 0x40000u);
    } else {
        // ---------------------------------------------------------------- read-back: thread r <-> weight row r
        pdl_wait();
        const int r = tid - FK_TC2_PW * 32, ew = r >> 5, rt = tile0 + (r >> 4), rr = r & 15, gq = rr & 7, hi = rr >> 3;
        const bool row_ok = rt < a.W.ntiles;
        float acc[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) acc[m] = 0.0f;
        uint4 sv[4], svn[4];
        auto s_load = [&](int sb, uint4 (&dst)[4]) {
            const uint4 *p = a.W.units + ((size_t)rt * nsb + sb) * FK_UNIT_VEC + 256 + gq * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = row_ok ? __ldg(p + q) : make_uint4(0, 0, 0, 0);
        };
        if (nit > 0) s_load(sb0, sv);
        for (int it = 0; it < nit && ok; ++it) {
            const int bs = it & 1;
            if (it + 1 < nit) s_load(sb0 + it + 1, svn);
            if (!tc_wait(bfull + 8 * bs, (uint32_t)(it >> 1) & 1u)) { ok = false; break; }       // the group sums are written
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int gi = it * 8 + j, tb = gi % FK_TC2_NT;
                if (!tc_wait(tfull + 8 * tb, (uint32_t)(gi / FK_TC2_NT) & 1u)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t d[16];
                const uint32_t taddr = tmem + ((uint32_t)(ew * 32) << 16) + (uint32_t)tb * 16u;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                               "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]) : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tempty + 8 * tb) : "memory");
                const uint4 s4 = sv[j >> 1];
                const uint32_t sw = hi ? s4.y : s4.x, bw = hi ? s4.w : s4.z;
                const float sc = (j & 1) ? bf_hi(sw) : bf_lo(sw), bi = (j & 1) ? bf_hi(bw) : bf_lo(bw);
                const float tbias = bi - 128.0f * sc;
                const float4 *xs4 = reinterpret_cast<const float4 *>(xsum + (bs * 8 + j) * 16);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 xq = xs4[q];
                    acc[4 * q + 0] = fmaf(tbias, xq.x, fmaf(sc, __uint_as_float(d[4 * q + 0]), acc[4 * q + 0]));
                    acc[4 * q + 1] = fmaf(tbias, xq.y, fmaf(sc, __uint_as_float(d[4 * q + 1]), acc[4 * q + 1]));
                    acc[4 * q + 2] = fmaf(tbias, xq.z, fmaf(sc, __uint_as_float(d[4 * q + 2]), acc[4 * q + 2]));
                    acc[4 * q + 3] = fmaf(tbias, xq.w, fmaf(sc, __uint_as_float(d[4 * q + 3]), acc[4 * q + 3]));
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bempty + 8 * bs) : "memory");
#pragma unroll
            for (int q = 0; q < 4; ++q) sv[q] = svn[q];
        }
        if (!ok && lane == 0) atomicOr(&st->error, 0x40000u);
        // ---- results: directly, or through the scratch area when K is split
        const int row = tile0 * 16 + r;
        if (S == 1) {
            if (ok && row < a.n)
#pragma unroll
                for (int m = 0; m < 16; ++m) if (m < a.m) {
                    const float res = a.residual ? bf2f(__ldcg(a.residual + (size_t)m * a.n + row)) : 0.0f;
                    a.y[(size_t)m * a.n + row] = f2bf(acc[m] + res);
                }
        } else {
            float *mine = a.scratch + (size_t)blockIdx.x * (16 * FK_TC_ROWS);
#pragma unroll
            for (int m = 0; m < 16; ++m) __stcg(mine + m * FK_TC_ROWS + r, acc[m]);
            __threadfence();
            asm volatile("bar.sync 2, 128;" ::: "memory");                  // the four read-back warps
            if (r == 0) {
                const unsigned int ticket = atomicAdd(a.counters + tile128, 1u);
                s_last = ticket == (unsigned int)(S - 1);
                if (s_last) a.counters[tile128] = 0u;
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (s_last) {
                __threadfence();
                if (row < a.n) {
                    const float *base = a.scratch + (size_t)tile128 * S * (16 * FK_TC_ROWS);
#pragma unroll
                    for (int m = 0; m < 16; ++m) if (m < a.m) {
                        float v = 0.0f;
                        for (int p = 0; p < S; ++p) v += __ldcg(base + (size_t)p * (16 * FK_TC_ROWS) + m * FK_TC_ROWS + r);
                        const float res = a.residual ? bf2f(__ldcg(a.residual + (size_t)m * a.n + row)) : 0.0f;
                        a.y[(size_t)m * a.n + row] = f2bf(v + res);
                    }
                }
            }
        }
    }
    pdl_launch_dependents();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (wid == 12) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(64u) : "memory");
}
