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
