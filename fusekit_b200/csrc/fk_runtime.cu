// libfusekit_cuda.so -- host runtime behind include/fusekit_cuda.h: handle table, device memory,
// weight objects, eager launches, CUDA-graph capture/replay of the per-token task list, decode
// chunk loops and the NCCL hook for tensor parallelism.  No PyTorch, no CPU fallback.
#include "../../include/fusekit_cuda.h"
#include "fk_common.cuh"
#include "fk_kernels.cuh"
#include "fk_synth.cuh"
#include "fk_stream.cuh"
#include "fk_qmm.cuh"
#include "fk_qmm_tc.cuh"
#include "fk_json.h"
#include <chrono>
#include <thread>

#include <dlfcn.h>
#include <math.h>
#include <mutex>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <string>
#include <vector>

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";
static fk_status fail(fk_status code, const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof g_err, fmt, ap); va_end(ap);
    return code;
}
#define CU(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) return fail(FK_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

// ------------------------------------------------------------------ NCCL (loaded on demand)
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
struct Nccl {
    void *dl = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
static Nccl g_nccl;
static fk_status nccl_load() {
    if (g_nccl.dl) return FK_OK;
    const char *names[] = {getenv("FK_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) { if (n && (g_nccl.dl = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break; }
    if (!g_nccl.dl) return fail(FK_ERR_NCCL, "cannot load libnccl.so.2 (set FK_NCCL_LIB): %s", dlerror());
    g_nccl.GetUniqueId = (int (*)(ncclUniqueId *))dlsym(g_nccl.dl, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(ncclComm_t *, int, ncclUniqueId, int))dlsym(g_nccl.dl, "ncclCommInitRank");
    g_nccl.AllReduce = (int (*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(g_nccl.dl, "ncclAllReduce");
    g_nccl.CommDestroy = (int (*)(ncclComm_t))dlsym(g_nccl.dl, "ncclCommDestroy");
    g_nccl.GetErrorString = (const char *(*)(int))dlsym(g_nccl.dl, "ncclGetErrorString");
    g_nccl.CommAbort = (int (*)(ncclComm_t))dlsym(g_nccl.dl, "ncclCommAbort");
    g_nccl.CommGetAsyncError = (int (*)(ncclComm_t, int *))dlsym(g_nccl.dl, "ncclCommGetAsyncError");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce) return fail(FK_ERR_NCCL, "libnccl lacks required symbols");
    return FK_OK;
}

// ------------------------------------------------------------------ objects
struct Weight {
    long long n = 0, k = 0; int bits = 0; bool finalized = false;
    uint32_t *w = nullptr; uint16_t *s = nullptr, *b = nullptr;       // MLX-affine rows (until repacked)
    size_t w_bytes = 0, sb_bytes = 0;
    // tiled layout (fk_stream.cuh): set by fk_weight_finalize / fk_weight_pair for 4- and 8-bit weights
    bool tiled = false; uint4 *units = nullptr; int ntiles = 0, nsb = 0; size_t unit_bytes = 0;
    int rows_kind = FK_ROWS_PLAIN, hd = 0, n_rot = 0;
    WView view() const { WView v; v.w = w; v.s = s; v.b = b; v.n = n; v.k = k; v.bits = bits; return v; }
    TiledW tview() const { TiledW t; t.units = units; t.ntiles = ntiles; t.nsb = nsb; t.n = (int)n; t.k = (int)k; t.bits = bits;
                           t.rows_kind = rows_kind; t.hd = hd; t.n_rot = n_rot; return t; }
};
struct Graph {
    std::vector<fk_task> tasks;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
};
struct Ctx {
    int device = 0; bool open = false;
    cudaStream_t stream = nullptr; cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    FkState *state = nullptr; uint32_t *history = nullptr; uint32_t hist_cap = 0;
    uint32_t *pinned = nullptr;                 // host staging for state / history
    std::vector<Weight> weights; std::vector<Graph> graphs; std::vector<void *> allocs;
    bool pending = false; bool pdl = true; int sm_count = 148;
    float *qmm_scratch = nullptr; unsigned int *qmm_counters = nullptr;   // K-split partial sums and tickets of the several-row projection
    bool use_tiled = true; int stages = FK_STAGES; int force_warps = 0; int force_split = -1; bool qmm_tc = false; int wide_upto = 3; bool sdpa_cluster = true; bool sdpa_mma = true; int sdpa_cl = 0;
    ncclComm_t comm = nullptr; int rank = 0, world = 1;
    bool comm_lost = false; long comm_timeout_ms = 0;
    unsigned long long *timeline = nullptr; int timeline_task = 0;      // tuning aid: per-task slices of 512 x 8 stamps
    long long launches = 0;
    uint32_t vocab = 0;                         // rows of the embedding table of the last embed task seen (0 = unknown)
    std::vector<void *> ipc_open; std::vector<unsigned char *> loop_arenas;      // peer mappings / loopback arenas to release
    unsigned char *arena = nullptr; PeerMap peers; bool peer_ready = false;      // peer-memory all-reduce
};
static std::mutex g_mu;
static std::vector<Ctx *> g_ctx;
#define FK_HIST_CAP 8192

static Ctx *get(fk_handle h) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (h == 0 || h > g_ctx.size() || !g_ctx[h - 1]->open) return nullptr;
    return g_ctx[h - 1];
}
#define CTX(h)                                                          \
    Ctx *c = get(h);                                                    \
    if (!c) return fail(FK_ERR_VALUE, "invalid handle %llu", (unsigned long long)(h)); \
    CU(cudaSetDevice(c->device))

// opt in to the full 227 KB of shared memory per block (minus the kernel's static part)
template <typename K> static cudaError_t big_smem(K kern) {
    cudaFuncAttributes fa; cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - (int)fa.sharedSizeBytes);
}

extern "C" const char *fk_last_error(void) { return g_err; }
extern "C" const char *fk_version(void) { return "fusekit-b200 0.1 (sm_100a)"; }

extern "C" fk_status fk_open(int device, fk_handle *out) {
    if (!out) return fail(FK_ERR_VALUE, "out is null");
    int ndev = 0; CU(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(FK_ERR_VALUE, "device %d out of range (%d visible)", device, ndev);
    CU(cudaSetDevice(device));
    cudaDeviceProp prop; CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(FK_ERR_STATE, "device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
    Ctx *c = new Ctx(); c->device = device; c->sm_count = prop.multiProcessorCount;
    CU(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    CU(cudaEventCreate(&c->ev0)); CU(cudaEventCreate(&c->ev1));
    CU(cudaMalloc(&c->state, sizeof(FkState))); CU(cudaMemset(c->state, 0, sizeof(FkState)));
    c->hist_cap = FK_HIST_CAP;
    CU(cudaMalloc(&c->qmm_scratch, sizeof(float) * 2 * c->sm_count * FK_QMM_PART_FLOATS));
    CU(cudaMalloc(&c->qmm_counters, sizeof(unsigned int) * 2 * c->sm_count)); CU(cudaMemset(c->qmm_counters, 0, sizeof(unsigned int) * 2 * c->sm_count));
    CU(cudaMalloc(&c->history, sizeof(uint32_t) * c->hist_cap)); CU(cudaMemset(c->history, 0, sizeof(uint32_t) * c->hist_cap));
    CU(cudaMallocHost(&c->pinned, sizeof(uint32_t) * (c->hist_cap + 64)));
    const char *e = getenv("FK_PDL"); if (e && e[0] == '0') c->pdl = false;
    e = getenv("FK_COMM_TIMEOUT_MS"); if (e) c->comm_timeout_ms = atol(e);
    e = getenv("FK_LAYOUT"); if (e && !strcmp(e, "mlx")) c->use_tiled = false;
    e = getenv("FK_SDPA"); if (e && !strcmp(e, "ticket")) c->sdpa_cluster = false;
    if (e && !strcmp(e, "mma")) c->sdpa_mma = true;
    if (e && !strcmp(e, "fma")) c->sdpa_mma = false;
    e = getenv("FK_SDPA_CL"); if (e && (atoi(e) == 1 || atoi(e) == 2 || atoi(e) == 4 || atoi(e) == 8 || atoi(e) == 16)) c->sdpa_cl = atoi(e);      // CTAs per kv head of the tensor-core attention
    e = getenv("FK_WARPS"); if (e) c->force_warps = atoi(e);
    e = getenv("FK_WIDE_UPTO"); if (e) c->wide_upto = atoi(e);      // 16-warp blocks for weights of up to this many tiles per warp of the machine
    e = getenv("FK_QMM_TC"); if (e && e[0] == '1') c->qmm_tc = true;     // several-row projections on tcgen05 by default
    e = getenv("FK_SPLIT"); if (e) c->force_split = atoi(e);        // log2 of the warps sharing a row tile (tuning)
#define BIG4(K) CU(big_smem(K<4, 8>)); CU(big_smem(K<4, 16>)); CU(big_smem(K<8, 8>)); CU(big_smem(K<8, 16>)); CU(big_smem(K<16, 8>)); CU(big_smem(K<16, 16>))
#define BIG4P(K) CU(big_smem(K<4, 8, true>)); CU(big_smem(K<4, 16, true>)); CU(big_smem(K<8, 8, true>)); CU(big_smem(K<8, 16, true>)); CU(big_smem(K<16, 8, true>)); CU(big_smem(K<16, 16, true>))
#define BIG4A(K) CU(big_smem(K<4, 8, false, true>)); CU(big_smem(K<4, 16, false, true>)); CU(big_smem(K<8, 8, false, true>)); CU(big_smem(K<8, 16, false, true>)); CU(big_smem(K<16, 8, false, true>)); CU(big_smem(K<16, 16, false, true>))
    BIG4A(k_s_rmsnorm_qkv);
    BIG4(k_s_linear); BIG4(k_s_rmsnorm_qkv); BIG4(k_s_gateup); BIG4(k_s_head); BIG4P(k_s_rmsnorm_qkv); BIG4P(k_s_gateup); BIG4P(k_s_head);
    CU(big_smem(k_sdpa_mma<64>)); CU(big_smem(k_sdpa_mma<128>)); CU(big_smem(k_sdpa_mma<256>));
    CU(cudaFuncSetAttribute(k_sdpa_mma<64>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CU(cudaFuncSetAttribute(k_sdpa_mma<128>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CU(cudaFuncSetAttribute(k_sdpa_mma<256>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    CU(big_smem(k_qmm4<false>)); CU(big_smem(k_qmm4<true>)); CU(big_smem(k_qmm_tc<32>)); CU(big_smem(k_qmm_tc2));
    CU(big_smem(k_sdpa_decode)); CU(big_smem(k_sdpa_decode_q<4>)); CU(big_smem(k_sdpa_decode_q<8>)); CU(big_smem(k_sdpa_cluster<64, 8>)); CU(big_smem(k_sdpa_cluster<128, 8>)); CU(big_smem(k_sdpa_cluster<256, 2>));
    CU(big_smem(k_rmsnorm_qkv<4>)); CU(big_smem(k_rmsnorm_qkv<8>)); CU(big_smem(k_rmsnorm_qkv<16>));
    CU(big_smem(k_linear_residual<4>)); CU(big_smem(k_linear_residual<8>)); CU(big_smem(k_linear_residual<16>));
    CU(big_smem(k_rmsnorm_gateup_act<4>)); CU(big_smem(k_rmsnorm_gateup_act<8>)); CU(big_smem(k_rmsnorm_gateup_act<16>));
    CU(big_smem(k_final_head<4>)); CU(big_smem(k_final_head<8>)); CU(big_smem(k_final_head<16>));
    c->open = true;
    std::lock_guard<std::mutex> lk(g_mu);
    g_ctx.push_back(c); *out = g_ctx.size();
    return FK_OK;
}

extern "C" fk_status fk_close(fk_handle h) {
    CTX(h);
    cudaStreamSynchronize(c->stream);
    for (auto &g : c->graphs) { if (g.exec) cudaGraphExecDestroy(g.exec); if (g.graph) cudaGraphDestroy(g.graph); }
    for (auto &w : c->weights) { cudaFree(w.w); cudaFree(w.s); cudaFree(w.b); cudaFree(w.units); }
    for (void *p : c->allocs) cudaFree(p);
    if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    for (void *p : c->ipc_open) cudaIpcCloseMemHandle(p);
    for (unsigned char *p : c->loop_arenas) cudaFree(p);
    if (c->arena) cudaFree(c->arena);
    c->ipc_open.clear(); c->loop_arenas.clear(); c->arena = nullptr; c->peer_ready = false; c->comm = nullptr;
    cudaFree(c->qmm_scratch); cudaFree(c->qmm_counters);
    cudaFree(c->state); cudaFree(c->history); cudaFreeHost(c->pinned);
    cudaEventDestroy(c->ev0); cudaEventDestroy(c->ev1); cudaStreamDestroy(c->stream);
    c->graphs.clear(); c->weights.clear(); c->allocs.clear(); c->open = false;
    return FK_OK;
}

extern "C" fk_status fk_info(fk_handle h, char *buf, size_t cap) {
    CTX(h);
    if (!buf || cap == 0) return fail(FK_ERR_VALUE, "buf is null");
    cudaDeviceProp prop; CU(cudaGetDeviceProperties(&prop, c->device));
    size_t fr = 0, tot = 0; CU(cudaMemGetInfo(&fr, &tot));
    snprintf(buf, cap, "{\"device\": %d, \"name\": \"%s\", \"sm\": %d, \"cc\": \"%d.%d\", \"mem_total\": %zu, \"mem_free\": %zu, "
             "\"weights\": %zu, \"graphs\": %zu, \"pdl\": %s, \"rank\": %d, \"world\": %d, \"kernel_launches\": %lld}",
             c->device, prop.name, prop.multiProcessorCount, prop.major, prop.minor, tot, fr, c->weights.size(), c->graphs.size(),
             c->pdl ? "true" : "false", c->rank, c->world, c->launches);
    return FK_OK;
}
static const char *kKernelNames[FK_TASK_KIND_COUNT] = {
    "fusekit_step_init", "fusekit_embed_lookup_decode", "fusekit_rmsnorm_qkv", "fusekit_qk_norm_rope_store",
    "fusekit_sdpa_decode", "fusekit_linear_residual", "fusekit_rmsnorm_gateup_act", "fusekit_final_rmsnorm_lm_head",
    "fusekit_argmax_finalize", "fusekit_allreduce", "fusekit_residual_add", "fusekit_rmsnorm_rows", "fusekit_rope_store_rows",
    "fusekit_argmax_rows", "fusekit_kv_store_quant", "fusekit_sdpa_decode_quant"};
extern "C" fk_status fk_kernel_names(char *buf, size_t cap) {
    if (!buf || cap == 0) return fail(FK_ERR_VALUE, "buf is null");
    std::string s;
    for (int i = 0; i < FK_TASK_KIND_COUNT; ++i) { if (i) s += ","; s += kKernelNames[i]; }
    snprintf(buf, cap, "%s", s.c_str());
    return FK_OK;
}

// ------------------------------------------------------------------ memory
extern "C" fk_status fk_alloc(fk_handle h, size_t nbytes, fk_dptr *out) {
    CTX(h);
    if (!out || nbytes == 0) return fail(FK_ERR_VALUE, "fk_alloc: bad arguments");
    void *p = nullptr; CU(cudaMalloc(&p, (nbytes + 255) & ~(size_t)255));
    CU(cudaMemsetAsync(p, 0, nbytes, c->stream));
    c->allocs.push_back(p); *out = (fk_dptr)p;
    return FK_OK;
}
extern "C" fk_status fk_free(fk_handle h, fk_dptr p) {
    CTX(h);
    for (size_t i = 0; i < c->allocs.size(); ++i)
        if (c->allocs[i] == (void *)p) { CU(cudaStreamSynchronize(c->stream)); CU(cudaFree((void *)p)); c->allocs.erase(c->allocs.begin() + i); return FK_OK; }
    return fail(FK_ERR_VALUE, "fk_free: address not owned by this handle");
}
extern "C" fk_status fk_upload(fk_handle h, fk_dptr dst, const void *src, size_t n) {
    CTX(h);
    if (!dst || !src) return fail(FK_ERR_VALUE, "fk_upload: null pointer");
    CU(cudaMemcpyAsync((void *)dst, src, n, cudaMemcpyHostToDevice, c->stream)); CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}
extern "C" fk_status fk_download(fk_handle h, void *dst, fk_dptr src, size_t n) {
    CTX(h);
    if (!dst || !src) return fail(FK_ERR_VALUE, "fk_download: null pointer");
    CU(cudaMemcpyAsync(dst, (const void *)src, n, cudaMemcpyDeviceToHost, c->stream)); CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}
extern "C" fk_status fk_memset(fk_handle h, fk_dptr dst, int byte, size_t n) {
    CTX(h); CU(cudaMemsetAsync((void *)dst, byte, n, c->stream)); return FK_OK;
}
extern "C" fk_status fk_sync(fk_handle h) { CTX(h); CU(cudaStreamSynchronize(c->stream)); return FK_OK; }
extern "C" fk_status fk_kv_cache_alloc(fk_handle h, int n_kv, int capacity, int head_dim, fk_dptr *k_out, fk_dptr *v_out) {
    if (n_kv <= 0 || capacity <= 0 || head_dim <= 0 || (head_dim & 7)) return fail(FK_ERR_VALUE, "fk_kv_cache_alloc: bad shape");
    const size_t bytes = (size_t)n_kv * capacity * head_dim * 2;
    fk_status s = fk_alloc(h, bytes, k_out); if (s) return s;
    return fk_alloc(h, bytes, v_out);
}

// ------------------------------------------------------------------ weights
static Weight *get_w(Ctx *c, fk_weight w) { return (w == 0 || w > c->weights.size()) ? nullptr : &c->weights[w - 1]; }

extern "C" fk_status fk_weight_alloc(fk_handle h, int64_t n, int64_t k, int bits, fk_weight *out) {
    CTX(h);
    if (!out || n <= 0 || k <= 0 || (k % 64) || (bits != 4 && bits != 8 && bits != 16)) return fail(FK_ERR_VALUE, "fk_weight_alloc: need n>0, k%%64==0, bits in {4,8,16}");
    Weight w; w.n = n; w.k = k; w.bits = bits;
    w.w_bytes = (size_t)n * k * bits / 8; w.sb_bytes = bits == 16 ? 0 : (size_t)n * (k / 64) * 2;
    CU(cudaMalloc(&w.w, w.w_bytes));
    if (w.sb_bytes) { CU(cudaMalloc(&w.s, w.sb_bytes)); CU(cudaMalloc(&w.b, w.sb_bytes)); }
    c->weights.push_back(w); *out = c->weights.size();
    return FK_OK;
}
extern "C" fk_status fk_weight_upload_rows(fk_handle h, fk_weight wid, int64_t r0, int64_t nr, const void *packed, const void *scales, const void *biases) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w) return fail(FK_ERR_VALUE, "bad weight id");
    if (w->finalized) return fail(FK_ERR_STATE, "weight already finalized");
    if (r0 < 0 || nr <= 0 || r0 + nr > w->n || !packed) return fail(FK_ERR_VALUE, "row range out of bounds");
    const size_t rb = (size_t)w->k * w->bits / 8, gb = (size_t)(w->k / 64) * 2;
    CU(cudaMemcpyAsync((char *)w->w + r0 * rb, packed, nr * rb, cudaMemcpyHostToDevice, c->stream));
    if (w->bits != 16) {
        if (!scales || !biases) return fail(FK_ERR_VALUE, "scales/biases required");
        CU(cudaMemcpyAsync((char *)w->s + r0 * gb, scales, nr * gb, cudaMemcpyHostToDevice, c->stream));
        CU(cudaMemcpyAsync((char *)w->b + r0 * gb, biases, nr * gb, cudaMemcpyHostToDevice, c->stream));
    }
    CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}
extern "C" fk_status fk_weight_synth_rows(fk_handle h, fk_weight wid, int64_t r0, int64_t nr, uint64_t stream, float std, int64_t k_global, int64_t src_row0, int64_t k0) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w) return fail(FK_ERR_VALUE, "bad weight id");
    if (w->finalized) return fail(FK_ERR_STATE, "weight already finalized");
    if (r0 < 0 || nr <= 0 || r0 + nr > w->n) return fail(FK_ERR_VALUE, "row range out of bounds");
    if (w->bits == 16) {
        const long long tot = nr * w->k;
        k_synth_dense<<<(unsigned)((tot + 255) / 256), 256, 0, c->stream>>>((uint16_t *)w->w, w->k, r0, nr, stream, std, k_global, src_row0, k0);
    } else {
        const long long tot = nr * (w->k / 64);
        k_synth_qweight<<<(unsigned)((tot + 127) / 128), 128, 0, c->stream>>>(w->w, w->s, w->b, w->k, w->bits, r0, nr, stream, std, k_global, src_row0, k0);
    }
    CU(cudaGetLastError());
    return FK_OK;
}
static fk_status repack(Ctx *c, Weight *dstw, const Weight *a, const Weight *b2) {
    const int kpu = unit_k(a->bits);                             // activations per unit
    dstw->ntiles = (int)((dstw->n + 15) / 16); dstw->nsb = (int)((a->k + kpu - 1) / kpu);
    dstw->unit_bytes = (size_t)dstw->ntiles * dstw->nsb * unit_vec(a->bits) * 16;
    CU(cudaMalloc(&dstw->units, dstw->unit_bytes));
    if (a->bits == 16) {
        const long long tot16 = (long long)dstw->ntiles * dstw->nsb * 256;
        k_repack_tiled16<<<(unsigned)((tot16 + 255) / 256), 256, 0, c->stream>>>((const uint16_t *)a->w, (const uint16_t *)(b2 ? b2->w : a->w), dstw->units, a->n,
                                                                                 (int)a->k, dstw->ntiles, dstw->nsb, dstw->rows_kind, dstw->hd, dstw->n_rot);
        CU(cudaGetLastError());
        CU(cudaStreamSynchronize(c->stream));
        dstw->tiled = true;
        return FK_OK;
    }
    SrcW sa{a->w, a->s, a->b}, sb{b2 ? b2->w : a->w, b2 ? b2->s : a->s, b2 ? b2->b : a->b};
    const long long tot = (long long)dstw->ntiles * dstw->nsb * FK_UNIT_VEC;
    k_repack_tiled<<<(unsigned)((tot + 255) / 256), 256, 0, c->stream>>>(sa, sb, dstw->units, a->n, (int)a->k, a->bits, dstw->ntiles, dstw->nsb,
                                                                        dstw->rows_kind, dstw->hd, dstw->n_rot);
    CU(cudaGetLastError());
    CU(cudaStreamSynchronize(c->stream));
    dstw->tiled = true;
    return FK_OK;
}
static void drop_rows(Weight *w) { cudaFree(w->w); cudaFree(w->s); cudaFree(w->b); w->w = nullptr; w->s = w->b = nullptr; }

extern "C" fk_status fk_weight_set_rows(fk_handle h, fk_weight wid, int kind, int head_dim, int n_rot_rows) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w) return fail(FK_ERR_VALUE, "bad weight id");
    if (w->finalized) return fail(FK_ERR_STATE, "weight already finalized");
    if (kind != FK_ROWS_PLAIN && kind != FK_ROWS_ROPE_PAIRS) return fail(FK_ERR_VALUE, "row order must be plain (0) or rope pairs (1)");
    if (kind == FK_ROWS_ROPE_PAIRS && (head_dim <= 0 || head_dim % 16 || n_rot_rows % head_dim || n_rot_rows > w->n)) return fail(FK_ERR_VALUE, "rope pairs need head_dim % 16 == 0 and whole heads");
    w->rows_kind = kind; w->hd = head_dim; w->n_rot = n_rot_rows;
    return FK_OK;
}
extern "C" fk_status fk_weight_finalize(fk_handle h, fk_weight wid) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w) return fail(FK_ERR_VALUE, "bad weight id");
    if (w->finalized) return FK_OK;
    if (c->use_tiled) {
        fk_status s = repack(c, w, w, nullptr); if (s) return s;
        drop_rows(w);
    } else { w->rows_kind = FK_ROWS_PLAIN; }
    w->finalized = true;
    return FK_OK;
}
extern "C" fk_status fk_weight_pair(fk_handle h, fk_weight gate, fk_weight up, fk_weight *out) {
    CTX(h); Weight *g = get_w(c, gate), *u = get_w(c, up);
    if (!g || !u || !out || gate == up) return fail(FK_ERR_VALUE, "bad weight ids");
    if (g->finalized || u->finalized) return fail(FK_ERR_STATE, "pair the weights before finalizing them");
    if (g->n != u->n || g->k != u->k || g->bits != u->bits) return fail(FK_ERR_VALUE, "gate and up must have one shape");
    if (!c->use_tiled) return fail(FK_ERR_STATE, "pairing needs the streaming layout");
    Weight p; p.n = 2 * g->n; p.k = g->k; p.bits = g->bits; p.rows_kind = FK_ROWS_GATE_UP;
    fk_status s = repack(c, &p, g, u); if (s) return s;
    p.finalized = true; p.w_bytes = g->w_bytes + u->w_bytes; p.sb_bytes = g->sb_bytes + u->sb_bytes;
    drop_rows(g); drop_rows(u); g->finalized = u->finalized = true; g->n = u->n = 0;      // consumed
    g = u = nullptr;
    c->weights.push_back(p); *out = c->weights.size();
    return FK_OK;
}
extern "C" fk_status fk_weight_dequant(fk_handle h, fk_weight wid, int64_t row0, int64_t nrows, float *host_out) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w || !host_out || row0 < 0 || nrows <= 0) return fail(FK_ERR_VALUE, "fk_weight_dequant: bad arguments");
    // a gate/up pair is addressed as rows [0, n/2) = gate, [n/2, n) = up
    const long long half = w->rows_kind == FK_ROWS_GATE_UP ? w->n / 2 : w->n;
    const int which = (w->rows_kind == FK_ROWS_GATE_UP && row0 >= half) ? 1 : 0;
    const long long r0 = which ? row0 - half : row0;
    if (r0 + nrows > half) return fail(FK_ERR_VALUE, "fk_weight_dequant: row range out of bounds");
    float *d = nullptr; const long long tot = nrows * w->k;
    CU(cudaMalloc(&d, tot * 4));
    if (w->tiled) {
        const long long th = (long long)w->ntiles * w->nsb * 256;
        if (w->bits == 16) k_dequant_tiled16<<<(unsigned)((th + 255) / 256), 256, 0, c->stream>>>(w->tview(), which, r0, nrows, d);
        else k_dequant_tiled<<<(unsigned)((th + 255) / 256), 256, 0, c->stream>>>(w->tview(), which, r0, nrows, d);
    } else {
        k_dequant<<<(unsigned)((tot + 255) / 256), 256, 0, c->stream>>>(w->w, w->s, w->b, w->k, w->bits, row0, nrows, d);
    }
    cudaError_t e = cudaMemcpyAsync(host_out, d, tot * 4, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(d);
    CU(e);
    return FK_OK;
}
extern "C" fk_status fk_weight_nbytes(fk_handle h, fk_weight wid, uint64_t *out) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w || !out) return fail(FK_ERR_VALUE, "bad weight id");
    *out = w->tiled ? w->unit_bytes : w->w_bytes + 2 * w->sb_bytes;
    return FK_OK;
}
extern "C" fk_status fk_synth_normal_bf16(fk_handle h, fk_dptr dst, uint64_t stream, uint64_t idx0, uint64_t n, float mean, float std) {
    CTX(h);
    if (!dst || n == 0) return fail(FK_ERR_VALUE, "fk_synth_normal_bf16: bad arguments");
    k_synth_normal_bf16<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>((uint16_t *)dst, stream, idx0, n, mean, std);
    CU(cudaGetLastError());
    return FK_OK;
}

// ------------------------------------------------------------------ launches
template <typename... KA, typename... A>
static cudaError_t launch(Ctx *c, void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, A... args) {
    cudaLaunchConfig_t cfg; memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = c->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = c->pdl ? 1 : 0;
    c->launches++;
    return cudaLaunchKernelEx(&cfg, kern, KA(args)...);
}
template <typename... KA, typename... A>
static cudaError_t launch_cluster(Ctx *c, void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, int cluster_x, A... args) {
    cudaLaunchConfig_t cfg; memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = c->stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cluster_x; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = c->pdl ? 2 : 1;
    c->launches++;
    return cudaLaunchKernelEx(&cfg, kern, KA(args)...);
}
// the several-row projection: 8 tiles per block; a weight with fewer sets of 8 tiles than block slots has K split over
// several blocks per set
static cudaError_t launch_qmm(Ctx *c, const Weight *w, QmmArgs &qa, bool gateup) {
    const int sets = (w->ntiles + FK_QMM_WARPS - 1) / FK_QMM_WARPS, slots = 2 * c->sm_count;
    int kparts = 1, qg = sets < slots ? sets : slots;
    if (sets * 10 < slots * 9) { kparts = slots / sets; if (kparts > w->nsb) kparts = w->nsb; qg = sets * kparts; }
    qa.kparts = kparts;
    if (gateup) return launch(c, k_qmm4<true>, dim3(qg), dim3(FK_QMM_WARPS * 32), qmm_smem_bytes(), c->state, qa);
    return launch(c, k_qmm4<false>, dim3(qg), dim3(FK_QMM_WARPS * 32), qmm_smem_bytes(), c->state, qa);
}
#define BITS_SWITCH(bits, CALL)                  \
    switch (bits) {                              \
        case 4: { constexpr int B = 4; CALL; break; }   \
        case 8: { constexpr int B = 8; CALL; break; }   \
        default: { constexpr int B = 16; CALL; break; } \
    }

static int grid_for(Ctx *c, long long units, int warps_per_block) {
    long long blocks = (units + warps_per_block - 1) / warps_per_block;
    const long long cap = (long long)c->sm_count * 4;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

// Work split of a streamed kernel.  Blocks have 8 warps and sit two to an SM when their shared memory (ring +
// staged activations) allows, else 16 warps and one per SM.  While there are fewer row tiles than warps in the grid, the
// K range of a tile is split over 2, 4, ... warps of one block (never more parts than super-blocks, rounded up to a power
// of two); a block then works on warps / parts tiles per round (fk_stream.cuh).
struct Shape { int grid, warps, lsplit; size_t smem; };
static Shape plan_shape(Ctx *c, const Weight *w) {
    Shape s;
    s.warps = 8;
    s.smem = stream_smem_bytes(w->nsb, c->stages, 8, w->bits);
    int per_sm = 2;
    // 16-warp blocks (one per SM) stage the activations once per SM instead of twice; weights with many rounds of tiles per
    // block (the lm_head) run faster with two 8-warp blocks per SM
    const bool few_rounds = (long long)w->ntiles <= (long long)c->wide_upto * c->sm_count * 16;
    if (s.smem > 113 * 1024 || c->force_warps == 16 || (c->force_warps == 0 && few_rounds)) {
        per_sm = 1;
        const size_t wide = stream_smem_bytes(w->nsb, c->stages, 16, w->bits);
        if (wide <= 226 * 1024) { s.warps = 16; s.smem = wide; }          // else: 8 warps, one block per SM (very long K)
    }
    const int slots = c->sm_count * per_sm;
    const long long total_warps = (long long)slots * s.warps;
    // the split with the shortest critical path: rounds of the busiest block x units of a warp per round, plus half a unit per
    // round for the fold when a tile is shared (a whole tile per warp leaves up to half the warps idle in the last round when
    // tiles / warps is 1.5, and a weight with few tiles of long K wants as many parts as it takes to reach every SM)
    (void)total_warps;
    int ls = 0; double best = 1e30;
    for (int l = 0; (1 << l) <= s.warps && ((1 << l) < 2 * w->nsb || l == 0); ++l) {
        const int S = 1 << l, tpb_l = s.warps >> l;
        const long long rounds_l = (w->ntiles + tpb_l - 1) / tpb_l, grid_l = rounds_l < slots ? rounds_l : slots;
        const double cost = (double)((rounds_l + grid_l - 1) / grid_l) * ((w->nsb + S - 1) / S + (S > 1 ? 0.5 : 0.0));
        if (cost < best - 1e-9) { best = cost; ls = l; }
    }
    if (c->force_split >= 0) { ls = c->force_split; while ((1 << ls) > s.warps) --ls; }
    s.lsplit = ls;
    const int tpb = s.warps >> ls, rounds = (w->ntiles + tpb - 1) / tpb;
    s.grid = rounds < slots ? rounds : slots;
    if (s.grid < 1) s.grid = 1;
    return s;
}
static Weight *get_w(Ctx *c, fk_weight w);
// the tiled weight a task streams, if any
static Weight *task_stream_weight(Ctx *c, const fk_task *t) {
    if (!t) return nullptr;
    Weight *w = nullptr;
    switch (t->kind) {
    case FK_TASK_RMSNORM_QKV: case FK_TASK_RMSNORM_GATEUP_ACT: case FK_TASK_FINAL_RMSNORM_LM_HEAD: w = get_w(c, t->buf[2]); break;
    case FK_TASK_LINEAR_RESIDUAL: w = get_w(c, t->buf[1]); break;
    default: break;
    }
    return (w && w->tiled) ? w : nullptr;
}
static Shape make_plan(Ctx *c, const Weight *w, StreamPlan *p, const Weight *next) {
    const Shape sh = plan_shape(c, w);
    p->W = w->tview(); p->stages = c->stages; p->lsplit = sh.lsplit;
    p->timeline = c->timeline ? c->timeline + (size_t)c->timeline_task * 512 * 8 : nullptr;
    return sh;
}
// launch a streamed kernel template instance for (bits, warps).  (One kernel shared by all four task kinds was tried
// to keep the code warm in the instruction caches between launches; it ran slower in the graph, 558 against 626 tok/s.)
#define STREAM_LAUNCH(KERN, w, sh, ...)                                                                                  \
    do {                                                                                                                 \
        if ((w)->bits == 4 && (sh).warps == 8) e = launch(c, KERN<4, 8>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);        \
        else if ((w)->bits == 4) e = launch(c, KERN<4, 16>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                     \
        else if ((w)->bits == 8 && (sh).warps == 8) e = launch(c, KERN<8, 8>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);   \
        else if ((w)->bits == 8) e = launch(c, KERN<8, 16>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                     \
        else if ((sh).warps == 8) e = launch(c, KERN<16, 8>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);                    \
        else e = launch(c, KERN<16, 16>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                                        \
    } while (0)
// norm-first kernels: the variant with the pending-norm / all-reduce prologue is a kernel of its own
#define STREAM_LAUNCH_P(KERN, pend, w, sh, ...)                                                                          \
    do {                                                                                                                 \
        if (pend) {                                                                                                      \
            if ((w)->bits == 4 && (sh).warps == 8) e = launch(c, KERN<4, 8, true>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);        \
            else if ((w)->bits == 4) e = launch(c, KERN<4, 16, true>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                     \
            else if ((w)->bits == 8 && (sh).warps == 8) e = launch(c, KERN<8, 8, true>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);   \
            else if ((w)->bits == 8) e = launch(c, KERN<8, 16, true>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                     \
            else if ((sh).warps == 8) e = launch(c, KERN<16, 8, true>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);                    \
            else e = launch(c, KERN<16, 16, true>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                                        \
        } else {                                                                                                         \
            if ((w)->bits == 4 && (sh).warps == 8) e = launch(c, KERN<4, 8, false>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);       \
            else if ((w)->bits == 4) e = launch(c, KERN<4, 16, false>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                    \
            else if ((w)->bits == 8 && (sh).warps == 8) e = launch(c, KERN<8, 8, false>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);  \
            else if ((w)->bits == 8) e = launch(c, KERN<8, 16, false>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                    \
            else if ((sh).warps == 8) e = launch(c, KERN<16, 8, false>, dim3((sh).grid), dim3(256), (sh).smem, __VA_ARGS__);                   \
            else e = launch(c, KERN<16, 16, false>, dim3((sh).grid), dim3(512), (sh).smem, __VA_ARGS__);                                       \
        }                                                                                                                \
    } while (0)
#define BITS48(bits, CALL) do { if ((bits) == 4) { constexpr int B = 4; CALL; } else { constexpr int B = 8; CALL; } } while (0)


// the fused peer exchange named by a task argument (0 = none, n > 0 = exchange site n - 1 of the task list)
static fk_status make_xchg(Ctx *c, int site_plus1, PeerXchg *x, const char *what) {
    memset(x, 0, sizeof *x); x->site = -1;
    if (site_plus1 <= 0) return FK_OK;
    if (!c->peer_ready) return fail(FK_ERR_STATE, "%s: a peer exchange site needs fk_peer_arena_open first", what);
    if (FK_PEER_SITE0 + site_plus1 - 1 >= FK_PEER_SITES) return fail(FK_ERR_VALUE, "%s: exchange site %d beyond the %d sites of an arena", what, site_plus1 - 1, FK_PEER_SITES - FK_PEER_SITE0);
    x->map = c->peers; x->site = FK_PEER_SITE0 + site_plus1 - 1;
    return FK_OK;
}
static fk_status run_task(Ctx *c, const fk_task &t, const Weight *nextw = nullptr) {
    const uint64_t *b = t.buf; const int32_t *i = t.iarg; const float *f = t.farg;
    cudaError_t e = cudaSuccess;
    switch (t.kind) {
    case FK_TASK_STEP_INIT: return FK_OK;     // offset/token advance is fused into the argmax finalisation
    case FK_TASK_EMBED_LOOKUP_DECODE: {
        if (!b[0] || !b[1] || i[0] <= 0 || i[1] <= 0 || i[1] > FK_MAX_ROWS) return fail(FK_ERR_VALUE, "embed: bad arguments");
        if (i[2] < 0) return fail(FK_ERR_VALUE, "embed: negative vocabulary size");
        if (i[3] != 0 && i[3] != 16 && ((i[3] != 4 && i[3] != 8) || !b[2] || !b[3] || (i[0] & 63))) return fail(FK_ERR_VALUE, "embed: a quantised table needs bits 4 or 8, scales, biases and H %% 64 == 0");
        EmbedArgs a{(const uint16_t *)b[0], (uint16_t *)b[1], i[0], i[1], f[0], i[2], (const uint16_t *)b[2], (const uint16_t *)b[3], i[3] == 16 ? 0 : i[3]};
        if (i[2] > 0) c->vocab = (uint32_t)i[2];        // seeds are checked against it in fk_state_set / fk_decode_chunk
        e = launch(c, k_embed_lookup, dim3((i[0] * i[1] + 255) / 256), dim3(256), 0, c->state, a);
        break;
    }
    case FK_TASK_RMSNORM_QKV: {
        Weight *w = get_w(c, b[2]);
        if (!w || !w->finalized) return fail(FK_ERR_VALUE, "rmsnorm_qkv: weight missing or not finalized");
        const int H = i[0], nq = i[1], nkv = i[2], hd = i[3], cap = i[4], sinks = i[5];
        if (w->k != H || w->n != (long long)(nq + 2 * nkv) * hd || (hd & 1) || cap <= 0) return fail(FK_ERR_VALUE, "rmsnorm_qkv: shape mismatch");
        if (sinks ? (!b[5] || !b[6]) : (!b[7] || !b[8])) return fail(FK_ERR_VALUE, "rmsnorm_qkv: output buffers missing");
        QkvArgs a{(const uint16_t *)b[0], (const uint16_t *)b[1], w->view(), (const uint16_t *)b[3], (uint16_t *)b[4], (uint16_t *)b[5],
                  (uint16_t *)b[6], (uint16_t *)b[7], (uint16_t *)b[8], (const uint16_t *)b[9], (const uint16_t *)b[10], (uint16_t *)b[11],
                  H, nq, nkv, hd, cap, sinks, f[0], (float)log2((double)f[1])};
        if (w->tiled) {
            if (sinks && (w->rows_kind != FK_ROWS_ROPE_PAIRS || w->hd != hd || w->n_rot != (nq + nkv) * hd)) return fail(FK_ERR_VALUE, "rmsnorm_qkv: weight rows must be laid out as RoPE pairs (fk_weight_set_rows)");
            if (!sinks && w->rows_kind != FK_ROWS_PLAIN) return fail(FK_ERR_VALUE, "rmsnorm_qkv without sinks takes plain row order");
            SQkvArgs sa{a.x, a.norm_w, StreamPlan(), a.lin_bias, a.q_out, a.cache_k, a.cache_v, a.k_out, a.v_out, a.pending, a.pending_w, a.h_out,
                        H, nq, nkv, hd, cap, sinks, a.eps, a.log2theta, nullptr, PeerXchg(), QkvAttend{nullptr, nullptr, nullptr, 0.0f}};
            if (i[7]) {         // attention as the kernel's tail: buf7 = attention output, buf8 = scratch (64 bytes of counters, then partials)
                if (!sinks || !b[7] || !b[8] || (b[8] & 15) || (hd != 64 && hd != 128) || nkv <= 0 || nq % nkv || nq / nkv > 8 || !(f[2] > 0.0f))
                    return fail(FK_ERR_VALUE, "rmsnorm_qkv with attention: needs the cache sinks, head_dim 64 or 128, at most 8 q heads per kv head, output, scratch and scale");
                sa.k_out = sa.v_out = nullptr;
                sa.att = QkvAttend{(uint16_t *)b[7], (float *)(b[8] + 64), (unsigned int *)b[8], f[2]};
            }
            { fk_status xs = make_xchg(c, i[6], &sa.pull, "rmsnorm_qkv"); if (xs) return xs; }
            if (sa.pull.site >= 0 && (b[9] || b[10] || H * 8 > FK_PEER_SLOT_BYTES)) return fail(FK_ERR_VALUE, "rmsnorm_qkv: a pulled exchange excludes pending inputs and needs H <= %d", FK_PEER_SLOT_BYTES / 8);
            if (b[9] && !b[10]) { sa.pending = nullptr; sa.pend_sum = (const float *)b[9]; }      // fp32 all-reduced projection + residual
            if (H > 8 * 256 * FK_STAGE_MAXB) return fail(FK_ERR_VALUE, "rmsnorm_qkv: hidden size above %d", 8 * 256 * FK_STAGE_MAXB);
            const Shape sh = make_plan(c, w, &sa.P, nextw);
            if (sa.att.out && (sh.grid > c->sm_count * (sh.warps == 8 ? 2 : 1) || sh.grid < nkv || sh.grid > FK_ATTEND_MAX_BLOCKS))
                return fail(FK_ERR_VALUE, "rmsnorm_qkv with attention: %d blocks do not fit the device at once (or fewer blocks than kv heads)", sh.grid);
            const bool pend = sa.pending || sa.pend_sum || sa.pull.site >= 0;
            if (sa.att.out) {
                if (pend) return fail(FK_ERR_VALUE, "rmsnorm_qkv with attention takes no pending inputs");
#define QKV_ATT(BITS_, WARPS_) launch(c, k_s_rmsnorm_qkv<BITS_, WARPS_, false, true>, dim3(sh.grid), dim3(WARPS_ * 32), sh.smem, c->state, sa)
                if (w->bits == 4) e = sh.warps == 8 ? QKV_ATT(4, 8) : QKV_ATT(4, 16);
                else if (w->bits == 8) e = sh.warps == 8 ? QKV_ATT(8, 8) : QKV_ATT(8, 16);
                else e = sh.warps == 8 ? QKV_ATT(16, 8) : QKV_ATT(16, 16);
#undef QKV_ATT
                break;
            }
            STREAM_LAUNCH_P(k_s_rmsnorm_qkv, pend, w, sh, c->state, sa);
            break;
        }
        if (i[7]) return fail(FK_ERR_VALUE, "rmsnorm_qkv with attention needs weights in the streaming layout");
        if (b[9] && !b[10]) return fail(FK_ERR_VALUE, "rmsnorm_qkv: the fused all-reduce residual needs 4/8-bit streamed weights");
        const int grid = grid_for(c, w->n / 2, 8);
        BITS_SWITCH(w->bits, e = launch(c, k_rmsnorm_qkv<B>, dim3(grid), dim3(256), smem_bytes_for(H), (const FkState *)c->state, a));
        break;
    }
    case FK_TASK_QK_NORM_ROPE_STORE: {
        const int nq = i[0], nkv = i[1], hd = i[2], cap = i[3];
        if (hd > 512 || (hd & 1) || !b[0] || !b[1] || !b[2] || !b[5] || !b[6]) return fail(FK_ERR_VALUE, "qk_norm_rope_store: bad arguments");
        QkNormArgs a{(uint16_t *)b[0], (const uint16_t *)b[1], (const uint16_t *)b[2], (const uint16_t *)b[3], (const uint16_t *)b[4],
                     (uint16_t *)b[5], (uint16_t *)b[6], nq, nkv, hd, cap, f[0], (float)log2((double)f[1])};
        e = launch(c, k_qk_norm_rope_store, dim3(nq + nkv), dim3((hd + 31) / 32 * 32), 0, (const FkState *)c->state, a);
        break;
    }
    case FK_TASK_SDPA_DECODE: {
        const int nq = i[0], nkv = i[1], hd = i[2], cap = i[3];
        if (nkv <= 0 || nq % nkv || nq / nkv > FK_SDPA_MAXG || (hd != 64 && hd != 128 && hd != 256) || !b[4] || !b[5]) return fail(FK_ERR_VALUE, "sdpa: unsupported shape (group <= 8, head_dim in {64,128,256})");
        const int chunks = (cap + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS, G = nq / nkv;
        SdpaArgs a{(const uint16_t *)b[0], (const uint16_t *)b[1], (const uint16_t *)b[2], (uint16_t *)b[3], (float *)b[4], (uint32_t *)b[5],
                   nq, nkv, hd, cap, chunks, f[0], c->timeline ? c->timeline + (size_t)c->timeline_task * 512 * 8 : nullptr, -1};
        const int variant = i[4];      // 0 = by shape, 1 = FMA cluster kernel, 2 = global-partials kernel, 4 = tensor-core cluster kernel
        if (i[5] > 1) {                // several sequences, each with its own cache: the tensor-core cluster kernel with the batch on grid.z
            if (i[5] > FK_MAX_ROWS || G > 8) return fail(FK_ERR_VALUE, "sdpa: at most %d sequences", FK_MAX_ROWS);
            a.rows = i[5]; a.consecutive = i[6] ? 1 : 0;
            const size_t smem = sdpa_mma_smem_bytes(G, hd);
            // one CTA of this kernel fills an SM (16 warps x 128 registers), so the CTAs of all sequences should fit the SMs at
            // once: 8 per kv head only while rows x kv heads x 8 does, down to one CTA that walks a whole cache (16 sequences of
            // the 32B shape: 128 CTAs; with 8 per kv head the 1024 CTAs took eight waves, 157 us a layer)
            int cl = FK_SDPA_CL;
            while (cl > 1 && cl * nkv * i[5] > c->sm_count) cl >>= 1;
            if (c->sdpa_cl > 0) cl = c->sdpa_cl;
            const dim3 cgrid(cl, nkv, i[5]), cblock(FK_SDPA_CW * 32);
            if (hd == 64) e = launch_cluster(c, k_sdpa_mma<64>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            else if (hd == 128) e = launch_cluster(c, k_sdpa_mma<128>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            else e = launch_cluster(c, k_sdpa_mma<256>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            break;
        }
        // tensor-core cluster kernel: the default up to head_dim 128; at 256 (two q heads per kv head in the Gemma shape)
        // the FMA kernel below is faster (11.0 against 12.1 us), so it runs only when asked for
        if (G <= 8 && (variant == 4 || (variant == 0 && hd <= 128 && c->sdpa_mma && c->sdpa_cluster))) {
            const size_t smem = sdpa_mma_smem_bytes(G, hd);
            // CTAs per kv head: 8 even for short caches (measured at 513 keys: 6.9 us with 8, 7.7 with 4, 10.6 with 2, 13.1 with 1)
            // 16 when few kv heads would leave most SMs idle on a long cache (a tensor-parallel slice of the 32B shape: 1 to 4 kv heads)
            const int cl = c->sdpa_cl > 0 ? c->sdpa_cl : ((nkv * 16 <= c->sm_count / 2 && cap >= 2048) ? FK_SDPA_CLMAX : FK_SDPA_CL);
            const dim3 cgrid(cl, nkv), cblock(FK_SDPA_CW * 32);
            if (hd == 64) e = launch_cluster(c, k_sdpa_mma<64>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            else if (hd == 128) e = launch_cluster(c, k_sdpa_mma<128>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            else e = launch_cluster(c, k_sdpa_mma<256>, cgrid, cblock, smem, cl, (const FkState *)c->state, a);
            break;
        }
        if (variant != 2 && c->sdpa_cluster && (hd != 256 || G <= 2)) {
            const size_t smem = sdpa_cl_smem_bytes(G, hd);
            const dim3 cgrid(FK_SDPA_CL, nkv), cblock(FK_SDPA_CW * 32);
            if (hd == 64) e = launch_cluster(c, k_sdpa_cluster<64, 8>, cgrid, cblock, smem, FK_SDPA_CL, (const FkState *)c->state, a);
            else if (hd == 128) e = launch_cluster(c, k_sdpa_cluster<128, 8>, cgrid, cblock, smem, FK_SDPA_CL, (const FkState *)c->state, a);
            else e = launch_cluster(c, k_sdpa_cluster<256, 2>, cgrid, cblock, smem, FK_SDPA_CL, (const FkState *)c->state, a);
            break;
        }
        const size_t smem = sdpa_smem_bytes(G, hd, chunks);
        if (smem > 200 * 1024) return fail(FK_ERR_VALUE, "sdpa: capacity too large for the merge table");
        e = launch(c, k_sdpa_decode, dim3(chunks, nkv), dim3(FK_SDPA_THREADS), smem, (const FkState *)c->state, a);
        break;
    }
    case FK_TASK_LINEAR_RESIDUAL: {
        Weight *w = get_w(c, b[1]);
        if (!w || !w->finalized) return fail(FK_ERR_VALUE, "linear_residual: weight missing or not finalized");
        if (w->k != i[0] || w->n != i[1] || !b[0] || (!b[3] && !b[4] && i[3] <= 0)) return fail(FK_ERR_VALUE, "linear_residual: shape mismatch");
        if (i[2] > 1) {                                    // 2..16 activation rows: the quantised matrix product
            if (!w->tiled || w->bits != 4 || w->rows_kind != FK_ROWS_PLAIN || !b[3] || b[4])
                return fail(FK_ERR_VALUE, "linear_residual with several rows takes streamed 4-bit weights in plain row order and a T output");
            if ((i[5] == 1 || (i[5] == 0 && c->qmm_tc)) && i[2] <= 16) {       // the warp-specialised tcgen05 form (i5: 1 = ask for it, 2 = mma.sync)
                const int t128 = (w->ntiles + 7) / 8;
                int kparts = t128 < c->sm_count ? c->sm_count / t128 : 1;
                if (kparts > w->nsb) kparts = w->nsb;
                if (kparts < 1) kparts = 1;
                QmmTc2Args ta{(const uint16_t *)b[0], w->tview(), (const uint16_t *)b[2], (uint16_t *)b[3], c->qmm_scratch, c->qmm_counters, i[2], i[0], i[1], kparts};
                e = launch(c, k_qmm_tc2, dim3((unsigned)(t128 * kparts)), dim3(FK_TC2_THREADS), qmm_tc2_smem_bytes(), c->state, ta);
                break;
            }
            if (i[5] == 1 || (i[5] == 0 && c->qmm_tc)) {             // 17 .. 32 rows: one CTA per 128 weight rows, all of K
                if (i[2] > FK_TC_MAXM) return fail(FK_ERR_VALUE, "linear_residual: the tcgen05 form takes at most %d activation rows", FK_TC_MAXM);
                QmmTcArgs ta{(const uint16_t *)b[0], w->tview(), (const uint16_t *)b[2], (uint16_t *)b[3], i[2], i[0], i[1]};
                const dim3 tgrid((unsigned)((w->ntiles + 7) / 8)), tblock(FK_TC_THREADS);
                e = launch(c, k_qmm_tc<32>, tgrid, tblock, qmm_tc_smem_bytes(), c->state, ta);
                break;
            }
            if (i[2] > FK_QMM_MAXM) return fail(FK_ERR_VALUE, "linear_residual: at most %d activation rows", FK_QMM_MAXM);
            QmmArgs qa{(const uint16_t *)b[0], w->tview(), (const uint16_t *)b[2], (uint16_t *)b[3], c->qmm_scratch, c->qmm_counters,
                       i[2], i[0], i[1], 1, nullptr, 0.0f, 0};
            e = launch_qmm(c, w, qa, false);
            break;
        }
        LinArgs a{(const uint16_t *)b[0], w->view(), (const uint16_t *)b[2], (uint16_t *)b[3], (float *)b[4], i[0], i[1]};
        if (w->tiled) {
            if (w->rows_kind != FK_ROWS_PLAIN) return fail(FK_ERR_VALUE, "linear_residual takes plain row order");
            SLinArgs sa{a.x, StreamPlan(), a.residual, a.y, a.y_f32, i[0], i[1], PeerXchg(), nullptr, nullptr};
            if (b[5]) {           // the activations once more as digits (written by the gate/up task): digits, then the (sum, 1 / scale) pairs
                if (w->bits == 16 || (b[5] & 15) || i[0] % 64) return fail(FK_ERR_VALUE, "linear_residual: staged digits need 4/8-bit weights, K a multiple of 64 and a 16-byte aligned buffer");
                sa.xdig = (const uint4 *)b[5]; sa.xdig_xsi = (const uint2 *)(b[5] + (((uint64_t)i[0] * 3 + 15) & ~(uint64_t)15));
            }
            { fk_status xs = make_xchg(c, i[3], &sa.push, "linear_residual"); if (xs) return xs; }
            if (sa.push.site >= 0 && i[1] * 8 > FK_PEER_SLOT_BYTES) return fail(FK_ERR_VALUE, "linear_residual: a pushed exchange needs N <= %d", FK_PEER_SLOT_BYTES / 8);
            const Shape sh = make_plan(c, w, &sa.P, nextw);
            STREAM_LAUNCH(k_s_linear, w, sh, c->state, sa);
            break;
        }
        if (i[3] > 0) return fail(FK_ERR_VALUE, "linear_residual: the fused peer exchange needs streamed weights");
        const int grid = grid_for(c, w->n, 8);
        BITS_SWITCH(w->bits, e = launch(c, k_linear_residual<B>, dim3(grid), dim3(256), smem_bytes_for(i[0]), (const FkState *)c->state, a));
        break;
    }
    case FK_TASK_RMSNORM_GATEUP_ACT: {
        Weight *wg = get_w(c, b[2]), *wu = get_w(c, b[3]);
        if (wg && wg->tiled && wg->rows_kind == FK_ROWS_GATE_UP) {       // paired gate/up weight (fk_weight_pair)
            if (wg->k != i[0] || wg->n != 2LL * i[1] || !b[4]) return fail(FK_ERR_VALUE, "gateup: shape mismatch");
            if (i[3] > 1) {                                // 2..16 activation rows
                if (i[3] > FK_QMM_MAXM) return fail(FK_ERR_VALUE, "gateup: at most %d activation rows", FK_QMM_MAXM);
                if (wg->bits != 4 || b[9] || b[10] || b[11]) return fail(FK_ERR_VALUE, "gateup with several rows takes 4-bit weights and no pending inputs");
                QmmArgs qa{(const uint16_t *)b[0], wg->tview(), nullptr, (uint16_t *)b[4], c->qmm_scratch, c->qmm_counters,
                           i[3], i[0], i[1], 1, (const uint16_t *)b[1], f[0], i[2]};
                e = launch_qmm(c, wg, qa, true);
                break;
            }
            SGateUpArgs sa{(const uint16_t *)b[0], (const uint16_t *)b[1], StreamPlan(), (uint16_t *)b[4],
                           (const uint16_t *)b[9], (const uint16_t *)b[10], (uint16_t *)b[11], i[0], i[1], i[2], f[0], nullptr, PeerXchg(), nullptr, nullptr};
            { fk_status xs = make_xchg(c, i[4], &sa.pull, "gateup"); if (xs) return xs; }
            if (sa.pull.site >= 0 && (b[9] || b[10] || i[0] * 8 > FK_PEER_SLOT_BYTES)) return fail(FK_ERR_VALUE, "gateup: a pulled exchange excludes pending inputs and needs H <= %d", FK_PEER_SLOT_BYTES / 8);
            if (b[9] && !b[10]) { sa.pending = nullptr; sa.pend_sum = (const float *)b[9]; }
            if (i[0] > 8 * 256 * FK_STAGE_MAXB) return fail(FK_ERR_VALUE, "gateup: hidden size above %d", 8 * 256 * FK_STAGE_MAXB);
            const Shape sh = make_plan(c, wg, &sa.P, nextw);
            if (b[5]) {           // also leave the activations as digits for the next projection (buf5: 3 bytes per activation, then 8 per group)
                const int rounds = (wg->ntiles + sh.grid * sh.warps - 1) / (sh.grid * sh.warps);
                if (wg->bits == 16 || sh.lsplit != 0 || i[1] % 64 || (b[5] & 15) || rounds * sh.warps * 8 > 2 * FK_STREAM_MAXWARPS * 16 * 2)
                    return fail(FK_ERR_VALUE, "gateup: digits for the next projection need 4/8-bit weights, whole tiles per warp (fk_weight_plan), I a multiple of 64 and at most %d outputs per block", 2 * FK_STREAM_MAXWARPS * 16 * 2);
                sa.dig_out = (uint32_t *)b[5]; sa.dig_xsi = (float2 *)(b[5] + (((uint64_t)i[1] * 3 + 15) & ~(uint64_t)15));
            }
            STREAM_LAUNCH_P(k_s_gateup, (sa.pending || sa.pend_sum || sa.pull.site >= 0), wg, sh, c->state, sa);
            break;
        }
        if (!wg || !wu || !wg->finalized || !wu->finalized) return fail(FK_ERR_VALUE, "gateup: weights missing or not finalized");
        if (wg->tiled || wu->tiled) return fail(FK_ERR_VALUE, "gateup: pair the gate and up weights with fk_weight_pair");
        if (wg->k != i[0] || wu->k != i[0] || wg->n != i[1] || wu->n != i[1] || wg->bits != wu->bits) return fail(FK_ERR_VALUE, "gateup: shape mismatch");
        GateUpArgs a{(const uint16_t *)b[0], (const uint16_t *)b[1], wg->view(), wu->view(), (uint16_t *)b[4],
                     (const uint16_t *)b[9], (const uint16_t *)b[10], (uint16_t *)b[11], i[0], i[1], i[2], f[0]};
        const int grid = grid_for(c, wg->n, 8);
        BITS_SWITCH(wg->bits, e = launch(c, k_rmsnorm_gateup_act<B>, dim3(grid), dim3(256), smem_bytes_for(i[0]), (const FkState *)c->state, a));
        break;
    }
    case FK_TASK_FINAL_RMSNORM_LM_HEAD: {
        Weight *w = get_w(c, b[2]);
        if (!w || !w->finalized) return fail(FK_ERR_VALUE, "lm_head: weight missing or not finalized");
        if (w->k != i[0] || w->n != i[1] || !b[4] || !b[5]) return fail(FK_ERR_VALUE, "lm_head: shape mismatch");
        HeadArgs a{(const uint16_t *)b[0], (const uint16_t *)b[1], w->view(), (uint16_t *)b[3], (unsigned long long *)b[4], (uint32_t *)b[5],
                   (const uint16_t *)b[9], (const uint16_t *)b[10], (uint16_t *)b[11], c->history, i[0], i[1], i[2], i[3], f[0]};
        if (w->tiled) {
            if (w->rows_kind != FK_ROWS_PLAIN) return fail(FK_ERR_VALUE, "lm_head takes plain row order");
            SHeadArgs sa{a.x, a.norm_w, StreamPlan(), a.logits, a.scratch, a.counter, a.pending, a.pending_w, a.h_out, a.history,
                         a.h, a.v, a.vocab_offset, a.finalize, a.eps, nullptr, PeerXchg(), PeerXchg()};
            { fk_status xs = make_xchg(c, i[4], &sa.pull, "lm_head"); if (xs) return xs; xs = make_xchg(c, i[5], &sa.amax, "lm_head"); if (xs) return xs; }
            if (sa.pull.site >= 0 && (b[9] || b[10] || i[0] * 8 > FK_PEER_SLOT_BYTES)) return fail(FK_ERR_VALUE, "lm_head: a pulled exchange excludes pending inputs and needs H <= %d", FK_PEER_SLOT_BYTES / 8);
            if (b[9] && !b[10]) { sa.pending = nullptr; sa.pend_sum = (const float *)b[9]; }
            if (i[0] > 8 * 256 * FK_STAGE_MAXB) return fail(FK_ERR_VALUE, "lm_head: hidden size above %d", 8 * 256 * FK_STAGE_MAXB);
            const Shape sh = make_plan(c, w, &sa.P, nextw);
            STREAM_LAUNCH_P(k_s_head, (sa.pending || sa.pend_sum || sa.pull.site >= 0), w, sh, c->state, sa);
            break;
        }
        const int grid = grid_for(c, w->n, 8);
        BITS_SWITCH(w->bits, e = launch(c, k_final_head<B>, dim3(grid), dim3(256), smem_bytes_for(i[0]), c->state, a));
        break;
    }
    case FK_TASK_ARGMAX_FINALIZE: {
        if (!b[4] || i[0] <= 0) return fail(FK_ERR_VALUE, "argmax_finalize: bad arguments");
        e = launch(c, k_argmax_finalize, dim3(1), dim3(32), 0, c->state, (const unsigned long long *)b[4], i[0], c->history);
        break;
    }
    case FK_TASK_ALLREDUCE: {
        if (c->peer_ready && i[0] > 0 && (size_t)i[0] * (i[1] == 1 ? 8 : 4) <= FK_PEER_SLOT_BYTES) {      // peer stores + flags instead of the library collective
            const int nbk = FK_PEER_BLOCKS;         // every call uses all blocks: one sequence number per block stays in step on all ranks
            if (i[1] == 1) e = launch(c, k_allreduce_peer<unsigned long long, true>, dim3(nbk), dim3(256), 0, (unsigned long long *)b[0], i[0], c->peers, c->state);
            else e = launch(c, k_allreduce_peer<float, false>, dim3(nbk), dim3(256), 0, (float *)b[0], i[0], c->peers, c->state);
            break;
        }
        if (c->comm_lost) return fail(FK_ERR_STATE, "the communicator was aborted after an error; open a new context");
        if (!c->comm) return fail(FK_ERR_STATE, "allreduce task without fk_comm_init");
        const int dtype = i[1] == 1 ? 5 /* ncclUint64 */ : 7 /* ncclFloat32 */, op = i[1] == 1 ? 2 /* ncclMax */ : 0 /* ncclSum */;
        int r = g_nccl.AllReduce((const void *)b[0], (void *)b[0], (size_t)i[0], dtype, op, c->comm, c->stream);
        if (r != 0) return fail(FK_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error");
        break;
    }
    case FK_TASK_RESIDUAL_ADD: {
        if (!b[0] || !b[2] || i[0] <= 0) return fail(FK_ERR_VALUE, "residual_add: bad arguments");
        e = launch(c, k_residual_add, dim3((i[0] + 255) / 256), dim3(256), 0, (const float *)b[0], (const uint16_t *)b[1], (uint16_t *)b[2], i[0]);
        break;
    }
    case FK_TASK_RMSNORM_ROWS: {
        if (!b[0] || !b[1] || !b[2] || i[0] <= 0 || i[1] <= 0 || i[1] > FK_MAX_ROWS) return fail(FK_ERR_VALUE, "rmsnorm_rows: bad arguments");
        NormRowsArgs a{(const uint16_t *)b[0], (const uint16_t *)b[1], (uint16_t *)b[2], i[0], i[1], f[0]};
        if (i[0] % 8 || (b[0] | b[1] | b[2]) % 16) return fail(FK_ERR_VALUE, "rmsnorm_rows: hidden size must be a multiple of 8 and the buffers 16-byte aligned");
        e = launch(c, k_rmsnorm_rows, dim3(i[1]), dim3(i[0] >= 8192 ? 1024 : i[0] >= 2048 ? 512 : 256), 0, (const FkState *)c->state, a);
        break;
    }
    case FK_TASK_ROPE_STORE_ROWS: {
        const int nq = i[0], nkv = i[1], hd = i[2], cap = i[3], rows = i[4];
        if (!b[0] || !b[1] || !b[5] || !b[6] || nq <= 0 || nkv <= 0 || hd <= 0 || (hd & 1) || hd > 2048 || cap <= 0 || rows <= 0 || rows > FK_MAX_ROWS)
            return fail(FK_ERR_VALUE, "rope_store_rows: bad arguments");
        RopeRowsArgs a{(const uint16_t *)b[0], (uint16_t *)b[1], (uint16_t *)b[5], (uint16_t *)b[6], nq, nkv, hd, cap, rows, (float)log2((double)f[1]), i[5] ? 1 : 0};
        e = launch(c, k_rope_store_rows, dim3(nq + 2 * nkv, rows), dim3((hd / 2 + 31) / 32 * 32), 0, (const FkState *)c->state, a);
        break;
    }
    case FK_TASK_ARGMAX_ROWS: {
        if (!b[0] || !b[5] || i[0] <= 0 || i[1] <= 0 || i[1] > FK_MAX_ROWS) return fail(FK_ERR_VALUE, "argmax_rows: bad arguments");
        ArgmaxRowsArgs a{(const uint16_t *)b[0], (uint32_t *)b[5], c->history, i[0], i[1], i[2] > 0 ? i[2] : 1};
        e = launch(c, k_argmax_rows, dim3(i[1]), dim3(1024), 0, c->state, a);
        break;
    }
    case FK_TASK_KV_STORE_QUANT: {
        const int nq = i[0], nkv = i[1], hd = i[2], cap = i[3], bits = i[4];
        if (!b[0] || !b[1] || !b[2] || !b[3] || !b[4] || !b[5] || !b[6] || !b[7] || !b[8] || nq <= 0 || nkv <= 0 || (hd != 64 && hd != 128 && hd != 256) ||
            cap <= 0 || (bits != 4 && bits != 8)) return fail(FK_ERR_VALUE, "kv_store_quant: bad arguments (head_dim in {64,128,256}, bits 4 or 8)");
        KvQuantArgs a{(uint16_t *)b[0], (const uint16_t *)b[1], (const uint16_t *)b[2], (uint32_t *)b[3], (uint32_t *)b[4], (uint16_t *)b[5],
                      (uint16_t *)b[6], (uint16_t *)b[7], (uint16_t *)b[8], nq, nkv, hd, cap, bits, (float)log2((double)f[1])};
        e = launch(c, k_rope_quant_store, dim3(nq + 2 * nkv), dim3(hd), 0, (const FkState *)c->state, a);
        break;
    }
    case FK_TASK_SDPA_DECODE_QUANT: {
        const int nq = i[0], nkv = i[1], hd = i[2], cap = i[3], bits = i[4];
        if (nkv <= 0 || nq % nkv || nq / nkv > FK_SDPA_MAXG || (hd != 64 && hd != 128 && hd != 256) || (bits != 4 && bits != 8) ||
            !b[0] || !b[1] || !b[2] || !b[3] || !b[4] || !b[5] || !b[6] || !b[7] || !b[8] || !b[9]) return fail(FK_ERR_VALUE, "sdpa_decode_quant: bad arguments");
        const int chunks = (cap + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS, G = nq / nkv;
        SdpaQArgs a{(const uint16_t *)b[0], (const uint32_t *)b[1], (const uint32_t *)b[2], (const uint16_t *)b[6], (const uint16_t *)b[7],
                    (const uint16_t *)b[8], (const uint16_t *)b[9], (uint16_t *)b[3], (float *)b[4], (uint32_t *)b[5], nq, nkv, hd, cap, chunks, f[0]};
        const size_t smem = sdpa_smem_bytes(G, hd, chunks);
        if (smem > 200 * 1024) return fail(FK_ERR_VALUE, "sdpa_decode_quant: capacity too large for the merge table");
        if (bits == 4) e = launch(c, k_sdpa_decode_q<4>, dim3(chunks, nkv), dim3(FK_SDPA_THREADS), smem, (const FkState *)c->state, a);
        else e = launch(c, k_sdpa_decode_q<8>, dim3(chunks, nkv), dim3(FK_SDPA_THREADS), smem, (const FkState *)c->state, a);
        break;
    }
    default: return fail(FK_ERR_VALUE, "unknown task kind %d", t.kind);
    }
    if (e != cudaSuccess) return fail(FK_ERR_CUDA, "launch of %s failed: %s", kKernelNames[t.kind], cudaGetErrorString(e));
    return FK_OK;
}


// the next streamed weight after task j (looking a few tasks ahead; wrapping to the start of the list when the
// list is replayed token after token)
static const Weight *next_stream_weight(Ctx *c, const fk_task *tasks, int n, int j, bool wrap) {
    for (int d = 1; d <= 4; ++d) {
        int q = j + d;
        if (q >= n) { if (!wrap) return nullptr; q -= n; if (q >= n) return nullptr; }
        Weight *w = task_stream_weight(c, &tasks[q]);
        if (w) return w;
    }
    return nullptr;
}

extern "C" fk_status fk_launch(fk_handle h, const fk_task *task) {
    CTX(h);
    if (!task) return fail(FK_ERR_VALUE, "task is null");
    fk_status s = run_task(c, *task); if (s) return s;
    CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}
extern "C" fk_status fk_launch_batch(fk_handle h, const fk_task *tasks, int n) {
    CTX(h);
    if (!tasks || n <= 0) return fail(FK_ERR_VALUE, "empty task list");
    for (int j = 0; j < n; ++j) { fk_status s = run_task(c, tasks[j], next_stream_weight(c, tasks, n, j, false)); if (s) return s; }
    CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}
extern "C" fk_status fk_smoke(fk_handle h, const uint16_t *a, const uint16_t *b, uint16_t *out, int n) {
    CTX(h);
    if (!a || !b || !out || n <= 0) return fail(FK_ERR_VALUE, "fk_smoke: bad arguments");
    uint16_t *d = nullptr; CU(cudaMalloc(&d, (size_t)n * 6));
    cudaError_t e = cudaMemcpyAsync(d, a, (size_t)n * 2, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d + n, b, (size_t)n * 2, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) { k_add_bf16<<<(n + 255) / 256, 256, 0, c->stream>>>(d, d + n, d + 2 * n, n); e = cudaGetLastError(); c->launches++; }
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, d + 2 * n, (size_t)n * 2, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(d);
    CU(e);
    return FK_OK;
}

// ------------------------------------------------------------------ state
static fk_status set_state(Ctx *c, uint32_t token, uint32_t offset) {
    if (c->vocab && token >= c->vocab) return fail(FK_ERR_VALUE, "token id %u is outside the embedding table (%u rows)", token, c->vocab);
    FkState *s = (FkState *)c->pinned; memset(s, 0, sizeof(FkState));
    s->token[0] = token; s->offset = offset; s->hist_counter = 0; s->error = 0; s->hist_cap = c->hist_cap;
    CU(cudaMemcpyAsync(c->state, s, FK_STATE_SET_BYTES, cudaMemcpyHostToDevice, c->stream));      // the epoch counter stays
    return FK_OK;
}
extern "C" fk_status fk_state_set(fk_handle h, uint32_t token, uint32_t offset) {
    CTX(h); fk_status s = set_state(c, token, offset); if (s) return s;
    CU(cudaStreamSynchronize(c->stream)); return FK_OK;
}
extern "C" fk_status fk_state_get(fk_handle h, uint32_t *token, uint32_t *offset, uint32_t *err) {
    CTX(h);
    CU(cudaMemcpyAsync(c->pinned, c->state, sizeof(FkState), cudaMemcpyDeviceToHost, c->stream)); CU(cudaStreamSynchronize(c->stream));
    const FkState *s = (const FkState *)c->pinned;
    if (token) *token = s->token[0]; if (offset) *offset = s->offset; if (err) *err = s->error;
    return FK_OK;
}

// ------------------------------------------------------------------ graph
static Graph *get_g(Ctx *c, fk_graph g) { return (g == 0 || g > c->graphs.size()) ? nullptr : &c->graphs[g - 1]; }

extern "C" fk_status fk_graph_capture(fk_handle h, const fk_task *tasks, int n, fk_graph *out) {
    CTX(h);
    if (!tasks || n <= 0 || !out) return fail(FK_ERR_VALUE, "empty task list");
    Graph g; g.tasks.assign(tasks, tasks + n);
    CU(cudaStreamSynchronize(c->stream));
    CU(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    fk_status s = FK_OK;
    for (int j = 0; j < n && s == FK_OK; ++j) { c->timeline_task = j; s = run_task(c, tasks[j], next_stream_weight(c, tasks, n, j, true)); }
    c->timeline_task = 0;
    cudaError_t e = cudaStreamEndCapture(c->stream, &g.graph);
    if (s) { if (g.graph) cudaGraphDestroy(g.graph); return s; }
    CU(e);
    CU(cudaGraphInstantiate(&g.exec, g.graph, 0));
    CU(cudaGraphUpload(g.exec, c->stream));
    c->graphs.push_back(g); *out = c->graphs.size();
    return FK_OK;
}
// ------------------------------------------------------------------ waiting with a communicator attached
// A rank whose peer died would wait in cudaStreamSynchronize for ever: the collective kernel never completes.  With a
// communicator the wait polls the stream and ncclCommGetAsyncError instead; on an asynchronous error (or after
// FK_COMM_TIMEOUT_MS without progress, off by default) the communicator is aborted, which ends its kernels, the stream is
// drained and the call returns FK_ERR_NCCL.  The context then refuses further token replays (its graphs hold collective
// nodes of the dead communicator).  Reference analogue: strict dispatch / fallback on a failed submit
// (python/fusekit_runtime/__init__.py:2889-2895).
static fk_status comm_check(Ctx *c) {
    if (!c->comm || !g_nccl.CommGetAsyncError) return FK_OK;
    int async = 0;
    const int r = g_nccl.CommGetAsyncError(c->comm, &async);
    if (r == 0 && (async == 0 || async == 7 /* ncclInProgress */)) return FK_OK;
    const int code = r != 0 ? r : async;
    if (g_nccl.CommAbort) g_nccl.CommAbort(c->comm); else if (g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    c->comm = nullptr; c->comm_lost = true;
    return fail(FK_ERR_NCCL, "communicator error (%s); communicator aborted", g_nccl.GetErrorString ? g_nccl.GetErrorString(code) : "async error");
}
static fk_status stream_wait(Ctx *c) {
    if (!c->comm) { CU(cudaStreamSynchronize(c->stream)); return FK_OK; }
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned spins = 0;; ++spins) {
        const cudaError_t q = cudaStreamQuery(c->stream);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) { CU(q); }
        fk_status s = comm_check(c);
        if (s) { cudaStreamSynchronize(c->stream); return s; }
        if (c->comm_timeout_ms > 0 && (spins & 255) == 255) {
            const long ms = (long)std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            if (ms > c->comm_timeout_ms) {
                if (g_nccl.CommAbort) g_nccl.CommAbort(c->comm);
                c->comm = nullptr; c->comm_lost = true;
                cudaStreamSynchronize(c->stream);
                return fail(FK_ERR_NCCL, "no progress for %ld ms with a collective in flight; communicator aborted", ms);
            }
        }
        if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    return comm_check(c);          // an error raised while the last kernels drained
}
// the launch shape the runtime will use for a streamed weight: blocks, warps per block, log2 of the warps sharing a row tile
extern "C" fk_status fk_weight_plan(fk_handle h, fk_weight wid, int *grid, int *warps, int *lsplit) {
    CTX(h); Weight *w = get_w(c, wid);
    if (!w || !w->finalized || !w->tiled) return fail(FK_ERR_VALUE, "fk_weight_plan: a finalized weight in the streaming layout is needed");
    const Shape sh = plan_shape(c, w);
    if (grid) *grid = sh.grid; if (warps) *warps = sh.warps; if (lsplit) *lsplit = sh.lsplit;
    return FK_OK;
}
extern "C" fk_status fk_comm_check(fk_handle h) { CTX(h); if (c->comm_lost) return fail(FK_ERR_STATE, "the communicator was aborted after an error"); return comm_check(c); }

// ------------------------------------------------------------------ task_graph.json behind the C ABI
// The file-level boundary of the reference: load_dispatcher(metallib, task_graph) reads the document and the host resolves
// every role string to a live buffer (python_runtime/src/lib.rs:115-169; src/runtime/plan.rs:39-164, 409-431).  Here the
// library parses the v2 document itself and the caller supplies the role -> address (or weight id) table, so a host without
// Python can replay a graph: tasks are taken in `decode_pipeline` order, `kind`, `layer_idx`, `iargs`, `fargs` as written
// by the emitter, and every explicit binding below slot 100 must be in the table.
extern "C" fk_status fk_tasks_from_json(const char *json_text, const fk_role_binding *roles, int n_roles, fk_task *tasks_out, int cap, int *n_out) {
    if (!json_text || (!roles && n_roles > 0) || n_roles < 0 || !n_out) return fail(FK_ERR_VALUE, "fk_tasks_from_json: null argument");
    JParser jp(json_text); JVal doc;
    if (!jp.parse(doc) || doc.kind != JVal::OBJ) return fail(FK_ERR_VALUE, "task graph: not a JSON object (%s)", jp.err.c_str());
    const JVal *ver = doc.get("version"), *am = doc.get("active_m"), *tasks = doc.get("tasks"), *pipe = doc.get("decode_pipeline"), *caps = doc.get("decode_capabilities");
    if (!ver || !ver->is_int() || (int)ver->num != 2) return fail(FK_ERR_VALUE, "task graph: version %d (this runtime reads 2)", ver && ver->kind == JVal::NUM ? (int)ver->num : -1);
    if (am && am->is_int() && (int)am->num != 1) return fail(FK_ERR_VALUE, "task graph: active_m %d (only batch-1 decode graphs are dispatchable)", (int)am->num);
    if (caps) { const JVal *d = caps->get("dispatchable"); if (d && d->kind == JVal::BOOL && !d->b) return fail(FK_ERR_VALUE, "task graph is marked not dispatchable"); }
    if (!tasks || tasks->kind != JVal::ARR || !pipe || pipe->kind != JVal::ARR) return fail(FK_ERR_VALUE, "task graph: tasks / decode_pipeline missing");
    std::map<long long, const JVal *> by_id;
    for (const JVal &t : tasks->arr) { const JVal *id = t.get("id"); if (id && id->is_int()) by_id[(long long)id->num] = &t; }
    std::map<std::string, uint64_t> table;
    for (int r = 0; r < n_roles; ++r) if (roles[r].role) table[roles[r].role] = roles[r].value;
    *n_out = (int)pipe->arr.size();
    if (!tasks_out) return FK_OK;                       // size query
    if (cap < *n_out) return fail(FK_ERR_VALUE, "tasks_out holds %d entries, %d needed", cap, *n_out);
    for (size_t j = 0; j < pipe->arr.size(); ++j) {
        const JVal &idv = pipe->arr[j];
        if (!idv.is_int() || !by_id.count((long long)idv.num)) return fail(FK_ERR_VALUE, "decode_pipeline[%zu] names no task", j);
        const JVal &t = *by_id[(long long)idv.num];
        fk_task &o = tasks_out[j]; memset(&o, 0, sizeof o);
        const JVal *kind = t.get("kind"), *layer = t.get("layer_idx"), *ia = t.get("iargs"), *fa = t.get("fargs"), *eb = t.get("extra_bindings");
        if (!kind || !kind->is_int() || kind->num < 0 || kind->num >= FK_TASK_KIND_COUNT) return fail(FK_ERR_VALUE, "task %lld: missing or unknown kind", (long long)idv.num);
        o.kind = (int32_t)kind->num; o.layer = layer && layer->is_int() ? (int32_t)layer->num : -1;
        if (ia && ia->kind == JVal::ARR) { if (ia->arr.size() > 8) return fail(FK_ERR_VALUE, "task %lld: more than 8 iargs", (long long)idv.num);
                                            for (size_t q = 0; q < ia->arr.size(); ++q) o.iarg[q] = (int32_t)ia->arr[q].num; }
        if (fa && fa->kind == JVal::ARR) { if (fa->arr.size() > 4) return fail(FK_ERR_VALUE, "task %lld: more than 4 fargs", (long long)idv.num);
                                            for (size_t q = 0; q < fa->arr.size(); ++q) o.farg[q] = (float)fa->arr[q].num; }
        if (eb && eb->kind == JVal::ARR) for (const JVal &bnd : eb->arr) {
            const JVal *slot = bnd.get("slot"), *role = bnd.get("role");
            if (!slot || !slot->is_int() || !role || role->kind != JVal::STR) return fail(FK_ERR_VALUE, "task %lld: malformed binding", (long long)idv.num);
            if (slot->num >= 100) continue;             // uniforms the runtime owns (token_id_in, layer_offset, next_token_out)
            if (slot->num < 0 || slot->num >= 12) return fail(FK_ERR_VALUE, "task %lld: buffer slot %d out of range", (long long)idv.num, (int)slot->num);
            auto it = table.find(role->str);
            if (it == table.end()) return fail(FK_ERR_VALUE, "task %lld: role '%s' is not in the binding table", (long long)idv.num, role->str.c_str());
            o.buf[(int)slot->num] = it->second;
        }
    }
    return FK_OK;
}
extern "C" fk_status fk_graph_capture_json(fk_handle h, const char *json_text, const fk_role_binding *roles, int n_roles, fk_graph *out) {
    int n = 0;
    fk_status s = fk_tasks_from_json(json_text, roles, n_roles, nullptr, 0, &n); if (s) return s;
    if (n <= 0) return fail(FK_ERR_VALUE, "task graph: empty decode_pipeline");
    std::vector<fk_task> tasks((size_t)n);
    s = fk_tasks_from_json(json_text, roles, n_roles, tasks.data(), n, &n); if (s) return s;
    return fk_graph_capture(h, tasks.data(), n, out);
}
extern "C" fk_status fk_graph_node_count(fk_handle h, fk_graph gid, int *n_out) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g || !n_out) return fail(FK_ERR_VALUE, "bad graph id");
    size_t n = 0; CU(cudaGraphGetNodes(g->graph, nullptr, &n)); *n_out = (int)n;
    return FK_OK;
}
extern "C" fk_status fk_graph_launch_async(fk_handle h, fk_graph gid) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g) return fail(FK_ERR_VALUE, "bad graph id");
    if (c->pending) return fail(FK_ERR_STATE, "a launch is already pending; call fk_wait");
    CU(cudaEventRecord(c->ev0, c->stream));
    CU(cudaGraphLaunch(g->exec, c->stream));
    CU(cudaEventRecord(c->ev1, c->stream));
    c->pending = true;
    return FK_OK;
}
extern "C" fk_status fk_wait(fk_handle h, double *gpu_seconds) {
    CTX(h);
    if (!c->pending) return fail(FK_ERR_STATE, "nothing pending");
    c->pending = false;
    { fk_status s = stream_wait(c); if (s) return s; }
    float ms = 0.0f; CU(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    if (gpu_seconds) *gpu_seconds = ms * 1e-3;
    return FK_OK;
}
extern "C" fk_status fk_graph_launch(fk_handle h, fk_graph gid, double *gpu_seconds) {
    fk_status s = fk_graph_launch_async(h, gid); if (s) return s;
    return fk_wait(h, gpu_seconds);
}
extern "C" fk_status fk_graph_profile_nodes(fk_handle h, fk_graph gid, int repeats, double *seconds_out, int cap, int *n_out) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g || !seconds_out || repeats <= 0) return fail(FK_ERR_VALUE, "bad arguments");
    const int n = (int)g->tasks.size();
    if (n_out) *n_out = n;
    if (cap < n) return fail(FK_ERR_VALUE, "seconds_out holds %d entries, %d needed", cap, n);
    // each task alone between two events, state restored afterwards (profile_icb_commands, lib.rs:821-869)
    CU(cudaMemcpyAsync(c->pinned + 32, c->state, sizeof(FkState), cudaMemcpyDeviceToHost, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    for (int j = 0; j < n; ++j) {
        double best = 1e30;
        for (int r = 0; r < repeats; ++r) {
            CU(cudaMemcpyAsync(c->state, c->pinned + 32, sizeof(FkState), cudaMemcpyHostToDevice, c->stream));
            CU(cudaEventRecord(c->ev0, c->stream));
            fk_status s = run_task(c, g->tasks[j], next_stream_weight(c, g->tasks.data(), n, j, true)); if (s) return s;
            CU(cudaEventRecord(c->ev1, c->stream));
            CU(cudaEventSynchronize(c->ev1));
            float ms = 0.0f; CU(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
            if (ms * 1e-3 < best) best = ms * 1e-3;
        }
        seconds_out[j] = best;
    }
    CU(cudaMemcpyAsync(c->state, c->pinned + 32, sizeof(FkState), cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}

// CUDA-event time of a list of tasks launched back to back on the library's stream, averaged over `repeats` passes
// (reference: execute_icb_range returns GPU seconds for a command range, lib.rs:769); the decode state is restored.
extern "C" fk_status fk_time_tasks(fk_handle h, const fk_task *tasks, int n, int repeats, double *seconds_per_pass) {
    CTX(h);
    if (!tasks || n <= 0 || repeats <= 0 || !seconds_per_pass) return fail(FK_ERR_VALUE, "bad arguments");
    CU(cudaMemcpyAsync(c->pinned + 32, c->state, sizeof(FkState), cudaMemcpyDeviceToHost, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    for (int j = 0; j < n; ++j) { fk_status s = run_task(c, tasks[j], next_stream_weight(c, tasks, n, j, true)); if (s) return s; }   // warm-up pass
    CU(cudaEventRecord(c->ev0, c->stream));
    for (int r = 0; r < repeats; ++r)
        for (int j = 0; j < n; ++j) { fk_status s = run_task(c, tasks[j], next_stream_weight(c, tasks, n, j, true)); if (s) return s; }
    CU(cudaEventRecord(c->ev1, c->stream));
    CU(cudaEventSynchronize(c->ev1));
    float ms = 0.0f; CU(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    *seconds_per_pass = ms * 1e-3 / repeats;
    CU(cudaMemcpyAsync(c->state, c->pinned + 32, sizeof(FkState), cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    return FK_OK;
}

extern "C" fk_status fk_step(fk_handle h, fk_graph gid, uint32_t token, uint32_t offset, uint32_t *next_token, double *gpu_seconds) {
    return fk_decode_chunk(h, gid, offset, token, 1, next_token, gpu_seconds);
}
extern "C" fk_status fk_decode_chunk(fk_handle h, fk_graph gid, uint32_t base_offset, uint32_t seed_token, int count,
                                     uint32_t *out_history, double *gpu_seconds) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g) return fail(FK_ERR_VALUE, "bad graph id");
    if (count <= 0 || (uint32_t)count > c->hist_cap) return fail(FK_ERR_VALUE, "count must be in 1..%u", c->hist_cap);
    if (c->pending) return fail(FK_ERR_STATE, "a launch is pending; call fk_wait");
    if (c->comm_lost) return fail(FK_ERR_STATE, "the communicator was aborted after an error; open a new context");
    fk_status s = set_state(c, seed_token, base_offset); if (s) return s;
    CU(cudaEventRecord(c->ev0, c->stream));
    for (int j = 0; j < count; ++j) CU(cudaGraphLaunch(g->exec, c->stream));
    CU(cudaEventRecord(c->ev1, c->stream));
    uint32_t *hist = c->pinned + 64;
    CU(cudaMemcpyAsync(hist, c->history, sizeof(uint32_t) * count, cudaMemcpyDeviceToHost, c->stream));
    CU(cudaMemcpyAsync(c->pinned + 32, c->state, sizeof(FkState), cudaMemcpyDeviceToHost, c->stream));
    s = stream_wait(c); if (s) return s;
    float ms = 0.0f; CU(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    if (gpu_seconds) *gpu_seconds = ms * 1e-3;
    if (out_history) memcpy(out_history, hist, sizeof(uint32_t) * count);
    const FkState *st = (const FkState *)(c->pinned + 32);
    if (st->error) return fail(FK_ERR_DEVICE, "device error word 0x%x", st->error);
    return FK_OK;
}
// `rows` independent sequences at one position: the graph holds the batch tasks, sequence m starts from seed_tokens[m];
// out_history[step * rows + m] is the token sequence m produced at step `step`
extern "C" fk_status fk_decode_chunk_rows(fk_handle h, fk_graph gid, uint32_t base_offset, const uint32_t *seed_tokens, int rows, int count,
                                          uint32_t *out_history, double *gpu_seconds) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g) return fail(FK_ERR_VALUE, "bad graph id");
    if (!seed_tokens || rows <= 0 || rows > FK_MAX_ROWS) return fail(FK_ERR_VALUE, "rows must be in 1..%d", FK_MAX_ROWS);
    if (count <= 0 || (uint64_t)count * rows > c->hist_cap) return fail(FK_ERR_VALUE, "count * rows must be in 1..%u", c->hist_cap);
    if (c->pending) return fail(FK_ERR_STATE, "a launch is pending; call fk_wait");
    for (int m = 0; m < rows; ++m)
        if (c->vocab && seed_tokens[m] >= c->vocab) return fail(FK_ERR_VALUE, "token id %u is outside the embedding table (%u rows)", seed_tokens[m], c->vocab);
    FkState *s0 = (FkState *)c->pinned; memset(s0, 0, sizeof(FkState));
    for (int m = 0; m < rows; ++m) s0->token[m] = seed_tokens[m];
    s0->offset = base_offset; s0->hist_cap = c->hist_cap;
    CU(cudaMemcpyAsync(c->state, s0, FK_STATE_SET_BYTES, cudaMemcpyHostToDevice, c->stream));
    CU(cudaEventRecord(c->ev0, c->stream));
    for (int j = 0; j < count; ++j) CU(cudaGraphLaunch(g->exec, c->stream));
    CU(cudaEventRecord(c->ev1, c->stream));
    uint32_t *hist = c->pinned + 64;
    CU(cudaMemcpyAsync(hist, c->history, sizeof(uint32_t) * count * rows, cudaMemcpyDeviceToHost, c->stream));
    CU(cudaMemcpyAsync(c->pinned + 32, c->state, sizeof(FkState), cudaMemcpyDeviceToHost, c->stream));
    { fk_status s = stream_wait(c); if (s) return s; }
    float ms = 0.0f; CU(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    if (gpu_seconds) *gpu_seconds = ms * 1e-3;
    if (out_history) memcpy(out_history, hist, sizeof(uint32_t) * count * rows);
    const FkState *st = (const FkState *)(c->pinned + 32);
    if (st->error) return fail(FK_ERR_DEVICE, "device error word 0x%x", st->error);
    return FK_OK;
}
extern "C" fk_status fk_decode_chunk_host(fk_handle h, fk_graph gid, uint32_t base_offset, uint32_t seed_token, int count,
                                          uint32_t *out_history, double *gpu_seconds) {
    CTX(h); Graph *g = get_g(c, gid);
    if (!g || count <= 0 || !out_history) return fail(FK_ERR_VALUE, "bad arguments");
    uint32_t tok = seed_token; double tot = 0.0;
    for (int j = 0; j < count; ++j) {
        double t = 0.0;
        fk_status s = fk_decode_chunk(h, gid, base_offset + j, tok, 1, &tok, &t); if (s) return s;
        out_history[j] = tok; tot += t;
    }
    if (gpu_seconds) *gpu_seconds = tot;
    return FK_OK;
}

// ------------------------------------------------------------------ allocation-free attention entry point
// Scratch of fk_sdpa_decode_noalloc: split-K partials (m, l, o[head_dim] per q head and 32-key chunk) followed by one
// arrival counter per kv head.  It lives in the library image, so every GPU that loads the library carries these
// 4 MiB + 256 B until the process exits, and every call on a device shares them.
#define FK_NOALLOC_PART_FLOATS (1u << 20)
#define FK_NOALLOC_MAX_KV 64
static __device__ __align__(256) unsigned char g_noalloc_scratch[FK_NOALLOC_PART_FLOATS * 4 + FK_NOALLOC_MAX_KV * 4];
static void *g_noalloc_ptr[64];             // device address of the scratch, per device ordinal (host-side cache)
static std::mutex g_noalloc_mu;

extern "C" fk_status fk_sdpa_decode_noalloc(const void *q, const void *cache_k, const void *cache_v, void *out,
                                            int n_q, int n_kv, int head_dim, int capacity, uint32_t pos, float scale, void *stream) {
    if (!q || !cache_k || !cache_v || !out) return fail(FK_ERR_VALUE, "fk_sdpa_decode_noalloc: null pointer");
    if (n_kv <= 0 || n_q <= 0 || n_q % n_kv || n_q / n_kv > FK_SDPA_MAXG || (head_dim != 64 && head_dim != 128 && head_dim != 256) || capacity <= 0)
        return fail(FK_ERR_VALUE, "fk_sdpa_decode_noalloc: unsupported shape (group <= 8, head_dim in {64,128,256})");
    if (pos > 0x7fffffffu) return fail(FK_ERR_VALUE, "fk_sdpa_decode_noalloc: pos %u exceeds 2^31 - 1", pos);
    const int chunks = (capacity + FK_SDPA_KEYS - 1) / FK_SDPA_KEYS, G = n_q / n_kv;
    const size_t need = (size_t)n_q * chunks * (head_dim + 2);
    if (need > FK_NOALLOC_PART_FLOATS || n_kv > FK_NOALLOC_MAX_KV)
        return fail(FK_ERR_VALUE, "fk_sdpa_decode_noalloc: n_q * ceil(capacity/32) * (head_dim+2) = %zu floats exceeds the built-in scratch of %u floats (or more than %d kv heads)",
                    need, FK_NOALLOC_PART_FLOATS, FK_NOALLOC_MAX_KV);
    const size_t smem = sdpa_smem_bytes(G, head_dim, chunks);
    if (smem > 200 * 1024) return fail(FK_ERR_VALUE, "fk_sdpa_decode_noalloc: capacity too large for the merge table");
    int dev = 0; CU(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(FK_ERR_VALUE, "device ordinal %d out of range", dev);
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {
            // first call on this device: resolve the device address of the array (its name is only a host-side handle)
            // and raise the kernel's shared-memory limit; neither allocates
            void *p = nullptr;
            CU(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            CU(big_smem(k_sdpa_decode));
            g_noalloc_ptr[dev] = p;
        }
        scratch = g_noalloc_ptr[dev];
    }
    cudaStream_t st = (cudaStream_t)stream;
    float *part = (float *)scratch;
    uint32_t *counters = (uint32_t *)((unsigned char *)scratch + (size_t)FK_NOALLOC_PART_FLOATS * 4);
    CU(cudaMemsetAsync(counters, 0, FK_NOALLOC_MAX_KV * 4, st));       // the arrival counters must start at zero
    SdpaArgs a{(const uint16_t *)q, (const uint16_t *)cache_k, (const uint16_t *)cache_v, (uint16_t *)out, part, counters,
               n_q, n_kv, head_dim, capacity, chunks, scale, nullptr, (int)pos};
    k_sdpa_decode<<<dim3(chunks, n_kv), dim3(FK_SDPA_THREADS), smem, st>>>((const FkState *)nullptr, a);
    CU(cudaGetLastError());
    return FK_OK;
}

// tuning aid: per-block phase timestamps of the next streamed launches land in `dptr` ([grid][8] u64), 0 = off
extern "C" fk_status fk_debug_timeline(fk_handle h, fk_dptr dptr) { CTX(h); c->timeline = (unsigned long long *)dptr; return FK_OK; }

// ------------------------------------------------------------------ tensor parallel
extern "C" fk_status fk_peer_arena_export(fk_handle h, void *handle64, size_t cap) {
    CTX(h);
    if (!handle64 || cap < sizeof(cudaIpcMemHandle_t)) return fail(FK_ERR_VALUE, "handle buffer must hold 64 bytes");
    if (!c->arena) {
        CU(cudaMalloc(&c->arena, PeerArena::bytes()));
        CU(cudaMemset(c->arena, 0, PeerArena::bytes()));
        CU(cudaDeviceSynchronize());
    }
    cudaIpcMemHandle_t hd; CU(cudaIpcGetMemHandle(&hd, c->arena));
    memcpy(handle64, &hd, sizeof hd);
    return FK_OK;
}
extern "C" fk_status fk_peer_arena_open(fk_handle h, const void *handles, int rank, int world) {
    CTX(h);
    if (!handles || world < 2 || world > FK_PEER_MAX || rank < 0 || rank >= world) return fail(FK_ERR_VALUE, "fk_peer_arena_open: 2..%d ranks", FK_PEER_MAX);
    if (!c->arena) return fail(FK_ERR_STATE, "call fk_peer_arena_export first");
    memset(&c->peers, 0, sizeof c->peers);
    c->peers.rank = rank; c->peers.world = world; c->peers.spin_limit = FK_PEER_SPIN_LIMIT;
    for (int r = 0; r < world; ++r) {
        if (r == rank) { c->peers.base[r] = c->arena; continue; }
        cudaIpcMemHandle_t hd; memcpy(&hd, (const unsigned char *)handles + (size_t)r * sizeof hd, sizeof hd);
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (void *q : c->ipc_open) cudaIpcCloseMemHandle(q);       // nothing stays mapped after a failed open
            c->ipc_open.clear(); memset(&c->peers, 0, sizeof c->peers);
            return fail(FK_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d: %s", r, cudaGetErrorString(e));
        }
        c->ipc_open.push_back(p);
        c->peers.base[r] = (unsigned char *)p;
    }
    c->rank = rank; c->world = world; c->peer_ready = true;
    return FK_OK;
}
extern "C" fk_status fk_peer_arena_close(fk_handle h) {
    CTX(h);
    CU(cudaStreamSynchronize(c->stream));
    for (void *p : c->ipc_open) cudaIpcCloseMemHandle(p);
    for (unsigned char *p : c->loop_arenas) cudaFree(p);
    c->ipc_open.clear(); c->loop_arenas.clear(); c->peer_ready = false; memset(&c->peers, 0, sizeof c->peers);
    return FK_OK;
}
// Diagnostic form of the peer exchange on ONE GPU: every "rank" gets an arena of its own in this device's memory, so an
// all-reduce task runs with ranks that never write.  With a small spin_limit the bounded wait of the exchange gives up
// after that many polls, the kernel sets error bit 0x8000 and returns; nothing hangs.
extern "C" fk_status fk_peer_arena_loopback(fk_handle h, int rank, int world, uint32_t spin_limit) {
    CTX(h);
    if (world < 2 || world > FK_PEER_MAX || rank < 0 || rank >= world || spin_limit == 0) return fail(FK_ERR_VALUE, "fk_peer_arena_loopback: 2..%d ranks, spin_limit > 0", FK_PEER_MAX);
    if (c->peer_ready) return fail(FK_ERR_STATE, "peer arenas are already open on this handle");
    memset(&c->peers, 0, sizeof c->peers);
    c->peers.rank = rank; c->peers.world = world; c->peers.spin_limit = spin_limit;
    for (int r = 0; r < world; ++r) {
        unsigned char *p = nullptr;
        CU(cudaMalloc(&p, PeerArena::bytes())); c->loop_arenas.push_back(p);
        CU(cudaMemset(p, 0, PeerArena::bytes()));
        c->peers.base[r] = p;
    }
    CU(cudaDeviceSynchronize());
    c->rank = rank; c->world = world; c->peer_ready = true;
    return FK_OK;
}
extern "C" fk_status fk_comm_unique_id(void *id128, size_t cap) {
    if (!id128 || cap < sizeof(ncclUniqueId)) return fail(FK_ERR_VALUE, "id buffer must hold 128 bytes");
    fk_status s = nccl_load(); if (s) return s;
    ncclUniqueId id; int r = g_nccl.GetUniqueId(&id);
    if (r != 0) return fail(FK_ERR_NCCL, "ncclGetUniqueId failed (%d)", r);
    memcpy(id128, &id, sizeof id);
    return FK_OK;
}
extern "C" fk_status fk_comm_init(fk_handle h, const void *id128, int rank, int world) {
    CTX(h);
    if (!id128 || world < 1 || rank < 0 || rank >= world) return fail(FK_ERR_VALUE, "fk_comm_init: bad arguments");
    fk_status s = nccl_load(); if (s) return s;
    ncclUniqueId id; memcpy(&id, id128, sizeof id);
    int r = g_nccl.CommInitRank(&c->comm, world, id, rank);
    if (r != 0) return fail(FK_ERR_NCCL, "ncclCommInitRank: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error");
    c->rank = rank; c->world = world;
    return FK_OK;
}
