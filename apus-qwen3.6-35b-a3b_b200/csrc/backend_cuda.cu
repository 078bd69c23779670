/*
 * backend_cuda.cu — C-ABI implementation of include/backend_cuda.h.
 *
 * Host side of the CUDA backend: context, HBM weight residency (the CPU
 * engine's NVMe expert cache, c/cache.h, has no counterpart here — a 67 GiB
 * checkpoint fits in one B200's 180 GB), workspace arena, kernel launches.
 * Shaped after c/backend_metal.mm: one process-wide context, one op mutex,
 * pointer-keyed weight cache, env-var knobs read at enable time, 0 / nonzero
 * return convention.  There is no CPU path in this file: without a usable
 * device every compute entry point fails.
 */
#include "../../include/backend_cuda.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "decode_fused.cuh"
#include "router_certify.cuh"
#include "decode_gemv.cuh"
#include "dispatch.cuh"
#include "ep_window.cuh"
#include "misc_kernels.cuh"
#include "prefill_gemm.cuh"
#include "pair_gemm.cuh"
#include "router.cuh"
#include "slab_loader.h"

using namespace apus;

constexpr int ROUTER_SMALL_MAX_T = 64;

/* ------------------------------------------------------------------------ */
/* context                                                                   */
/* ------------------------------------------------------------------------ */

struct DevBuf {
    void *ptr = nullptr;
    size_t bytes = 0;
};

struct Arena {
    char *base = nullptr;
    size_t cap = 0;
    size_t off = 0;
    /* Chunks this arena has outgrown.  A captured CUDA graph keeps the
     * addresses it was captured with (kernel arguments, tensor maps by value),
     * so an outgrown chunk is never freed while the backend is enabled: a
     * replay of an older capture still finds its memory. */
    std::vector<void *> retired;
    void reset() { off = 0; }
    void *take(size_t bytes) {
        size_t o = (off + 255) & ~(size_t)255;
        if (o + bytes > cap) return nullptr;
        off = o + bytes;
        return base + o;
    }
};

struct ApusCudaLayer {
    ApusCudaMoeCfg cfg;
    size_t e_begin = 0, e_end = 0;
    uint16_t *rtr_w = nullptr, *exp_gu = nullptr, *exp_d = nullptr;
    uint16_t *sh_g = nullptr, *sh_u = nullptr, *sh_d = nullptr,
             *sh_gate = nullptr;
    float wmin = 0.0f;          /* smallest nonzero |rtr_w| (0 = unknown) */
    float wmin_gate = 0.0f;     /* the same for the shared-gate row */
    float *d_wnorm = nullptr;   /* [E + 1] router row norms (rounded up), [E] = max */
    size_t bytes = 0;
    PrefillMaps *maps = nullptr; /* tensor maps for the tcgen05 path */
};

struct Ctx {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    cudaStream_t stream = nullptr;
    std::unordered_map<const void *, DevBuf> wcache;
    std::unordered_map<const void *, ApusCudaLayer *> layers;  /* host-ptr key */
    uint64_t budget = ~0ull;
    uint64_t bytes_resident = 0, bytes_uploaded = 0, launches = 0;
    Arena ws;      /* block workspace */
    Arena io;      /* host-pointer staging */
    int *d_status = nullptr;
    unsigned int *d_scratch_u32 = nullptr;
    unsigned int *d_router_counters = nullptr;   /* [ROUTER_SMALL_MAX_T], self-resetting */
    float *d_router_logits = nullptr;            /* [ROUTER_SMALL_MAX_T][1024] */
    int router_certify = 1;      /* many tokens: fast logits + exact chains for candidates */
    unsigned int *d_rc_stats = nullptr;          /* [0] exact chains run so far */
    int decode_max_t = 4;        /* above this the tcgen05 grouped GEMM runs */
    int fused_max_t = 4;         /* up to this the one-kernel decode path runs */
    /* scratch of the fused decode kernel */
    float *d_df_logits = nullptr;
    uint16_t *d_df_sgl = nullptr, *d_df_act = nullptr, *d_df_sa = nullptr;
    unsigned int *d_df_sync = nullptr;
    unsigned long long *d_df_timeline = nullptr;   /* [sm_count][DF_MARKS] */
    bool df_timeline_valid = false;
    size_t df_act_elems = 0, df_sa_elems = 0;
    int last_block_launches = 0;
    int last_block_path = 0;
    bool hooks_filled = false;
    size_t ep_rows_hint = 0;     /* rows the next experts_dev call expects (0: its R) */
    /* host-pointer block call with many tokens: two halves, the second half's
     * upload and the first half's download beside the other half's kernels */
    long host_split_t = 4096;    /* APUS_CUDA_HOST_SPLIT_T: from this many tokens (0: never) */
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_io[5] = {};   /* start, in[2], done[2] */
    /* ordering of calls that arrive on different streams */
    cudaStream_t cur_stream = nullptr, last_stream = nullptr;
    cudaEvent_t last_ev = nullptr;
    bool have_last = false, cur_capturing = false;
    /* optional per-stage CUDA events inside the block (benchmarks) */
    bool stage_timing = false;
    cudaEvent_t ev[16] = {};
    int n_ev = 0;
    int ev_stage[16] = {};
};

namespace apus { bool g_apus_use_pdl = true; }

static Ctx *g_ctx = nullptr;
static std::recursive_mutex g_mu;
static char g_err[512] = "";

ApusCudaBlockHooks apus_cuda_block_hooks = {nullptr};

/* The engine's three-slot table (c/backend_metal.h:79-88), when the engine is
 * linked into this process; absent (NULL address) otherwise. */
extern "C" {
typedef struct {
    int (*bf16_gemv)(const uint16_t *, const uint16_t *, uint16_t *, size_t,
                     size_t);
    int (*bf16_gemm)(const uint16_t *, const uint16_t *, uint16_t *, size_t,
                     size_t, size_t);
    int (*bf16_matvec_f32)(const uint16_t *, const uint16_t *, float *, size_t,
                           size_t);
} ApusBackendHooksView;
extern ApusBackendHooksView apus_backend_hooks __attribute__((weak));
}

static int fail(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return 1;
}
#define CU_OK(call)                                                        \
    do {                                                                   \
        cudaError_t e_ = (call);                                           \
        if (e_ != cudaSuccess)                                             \
            return fail("%s: %s (%s:%d)", #call, cudaGetErrorString(e_),   \
                        __FILE__, __LINE__);                               \
    } while (0)

static long env_long(const char *name, long dflt) {
    const char *e = getenv(name);
    return (e && *e) ? atol(e) : dflt;
}

static int ctx_init() {
    if (g_ctx) return 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0)
        return fail("no CUDA device (%s)", cudaGetErrorString(e));
    int dev = (int)env_long("APUS_CUDA_DEVICE", -1);
    if (dev < 0) {
        /* one process per GPU under a multi-rank launcher */
        dev = (int)env_long("LOCAL_RANK", 0);
        if (dev >= n) dev = dev % n;
    }
    if (dev >= n) return fail("APUS_CUDA_DEVICE=%d but %d device(s)", dev, n);
    CU_OK(cudaSetDevice(dev));
    cudaDeviceProp prop;
    CU_OK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        return fail("device %d is sm_%d%d; this backend is built for sm_100a",
                    dev, prop.major, prop.minor);
    Ctx *c = new Ctx();
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    /* experiments: run the persistent kernels on fewer SMs */
    if (env_long("APUS_CUDA_SMS", 0) > 0 && env_long("APUS_CUDA_SMS", 0) < c->sm_count)
        c->sm_count = (int)env_long("APUS_CUDA_SMS", 0);
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    CU_OK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    CU_OK(cudaMalloc(&c->d_status, 256));
    CU_OK(cudaMemset(c->d_status, 0, 256));
    c->d_scratch_u32 = reinterpret_cast<unsigned int *>(c->d_status) + 16;
    CU_OK(cudaMalloc(&c->d_router_counters, ROUTER_SMALL_MAX_T * 4));
    CU_OK(cudaMemset(c->d_router_counters, 0, ROUTER_SMALL_MAX_T * 4));
    CU_OK(cudaMalloc(&c->d_router_logits,
                     (size_t)ROUTER_SMALL_MAX_T * 1024 * sizeof(float)));
    long mb = env_long("APUS_CUDA_DENSE_MB", -1);
    c->budget = mb < 0 ? ~0ull : (uint64_t)mb << 20;
    c->decode_max_t = (int)env_long("APUS_CUDA_DECODE_MAX_T", 4);
    c->router_certify = (int)env_long("APUS_CUDA_ROUTER_CERTIFY", 1);
    CU_OK(cudaMalloc(&c->d_rc_stats, 64));
    CU_OK(cudaMemset(c->d_rc_stats, 0, 64));
    c->fused_max_t = (int)env_long("APUS_CUDA_FUSED_MAX_T", DF_MAX_T);
    if (c->fused_max_t > DF_MAX_T) c->fused_max_t = DF_MAX_T;
    CU_OK(cudaMalloc(&c->d_df_logits, (size_t)DF_MAX_T * 1024 * sizeof(float)));
    CU_OK(cudaMalloc(&c->d_df_sgl, 64));
    CU_OK(cudaMalloc(&c->d_df_sync, 64));
    CU_OK(cudaMemset(c->d_df_sync, 0, 64));
    CU_OK(cudaMalloc(&c->d_df_timeline,
                     (size_t)c->sm_count * DF_MARKS * sizeof(unsigned long long)));
    g_apus_use_pdl = env_long("APUS_CUDA_PDL", 1) != 0;
    g_pg_overlap = (int)env_long("APUS_CUDA_GEMM_OVERLAP", 1);
    g_pg_dynamic = (int)env_long("APUS_CUDA_GEMM_DYNAMIC", 3);
    g_pg_direct = (int)env_long("APUS_CUDA_GEMM_DIRECT", 1);
    g_pp_enable = (int)env_long("APUS_CUDA_PAIR", 1);
    g_pp_min_rows = (int)env_long("APUS_CUDA_PAIR_MIN_ROWS", 192);
    g_pp_gather = (int)env_long("APUS_CUDA_PAIR_GATHER", 0);
    g_pp_solo_below = (int)env_long("APUS_CUDA_PAIR_SOLO_BELOW", 160);
    c->host_split_t = env_long("APUS_CUDA_HOST_SPLIT_T", 4096);
    g_ctx = c;
    return 0;
}

static int arena_reserve(Arena &a, size_t bytes) {
    if (a.cap >= bytes) return 0;
    /* growing inside a capture would need a device-wide synchronisation,
     * which a capturing stream does not allow */
    if (g_ctx && g_ctx->cur_capturing)
        return fail("workspace too small for this call inside a stream capture: "
                    "call apus_cuda_reserve for the largest shape before capturing");
    CU_OK(cudaDeviceSynchronize());
    if (a.base) a.retired.push_back(a.base);
    a.base = nullptr;
    a.cap = 0;
    size_t want = bytes + (bytes >> 2) + (1u << 20);
    CU_OK(cudaMalloc((void **)&a.base, want));
    a.cap = want;
    a.off = 0;
    return 0;
}
static void arena_free(Arena &a) {
    if (a.base) cudaFree(a.base);
    for (void *p : a.retired) cudaFree(p);
    a.retired.clear();
    a.base = nullptr;
    a.cap = a.off = 0;
}

/* All device-pointer entry points share one workspace, one status word and
 * the counters of the one-kernel decode path, whatever stream they are given.
 * A call that arrives on another stream than the call before it is ordered
 * behind that call with an event, so two callers on two streams get serial,
 * correct results instead of a silent race.  Inside a stream capture nothing
 * is recorded or waited for (a capture must not depend on work outside it):
 * replays of captured graphs are ordered by their caller. */
static int order_begin(Ctx *c, cudaStream_t st) {
    c->cur_stream = st;
    c->cur_capturing = false;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    c->cur_capturing = cs != cudaStreamCaptureStatusNone;
    if (c->cur_capturing) return 0;
    if (c->have_last && c->last_stream != st)
        CU_OK(cudaStreamWaitEvent(st, c->last_ev, 0));
    return 0;
}
static void order_end(Ctx *c, cudaStream_t st) {
    if (c->cur_capturing) return;
    if (!c->last_ev &&
        cudaEventCreateWithFlags(&c->last_ev, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    if (cudaEventRecord(c->last_ev, st) == cudaSuccess) {
        c->last_stream = st;
        c->have_last = true;
    } else {
        cudaGetLastError();
    }
}
/* brackets one device-pointer entry point */
struct Ordered {
    Ctx *c;
    cudaStream_t st;
    int rc;
    Ordered(Ctx *c_, cudaStream_t st_) : c(c_), st(st_), rc(order_begin(c_, st_)) {}
    ~Ordered() { order_end(c, st); }
};

#define LAUNCHED()                                                         \
    do {                                                                   \
        g_ctx->launches++;                                                 \
        g_ctx->last_block_launches++;                                      \
        cudaError_t e_ = cudaGetLastError();                               \
        if (e_ != cudaSuccess)                                             \
            return fail("kernel launch: %s (%s:%d)", cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                               \
    } while (0)

/* stage marks: an event before the first stage and after every stage */
static void stage_mark(Ctx *c, int stage, cudaStream_t st) {
    if (!c->stage_timing || c->n_ev >= 16) return;
    if (!c->ev[c->n_ev]) cudaEventCreate(&c->ev[c->n_ev]);
    cudaEventRecord(c->ev[c->n_ev], st);
    c->ev_stage[c->n_ev] = stage;
    c->n_ev++;
}

static cudaStream_t g_mark_stream = nullptr;
static void mark_cb(int stage) {
    if (g_ctx) stage_mark(g_ctx, stage, g_mark_stream);
}

/* ------------------------------------------------------------------------ */
/* lifecycle                                                                 */
/* ------------------------------------------------------------------------ */

static int hook_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y,
                     size_t O, size_t K) {
    return apus_cuda_bf16_gemv(w, x, y, O, K);
}
static int hook_gemm(const uint16_t *w, const uint16_t *x, uint16_t *y,
                     size_t M, size_t O, size_t K) {
    return apus_cuda_bf16_gemm(w, x, y, M, O, K);
}
static int hook_matvec(const uint16_t *w, const uint16_t *x, float *y,
                       size_t O, size_t K) {
    return apus_cuda_bf16_matvec_f32(w, x, y, O, K);
}

extern "C" int apus_cuda_enable(char *err, size_t errcap) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) {
        if (err && errcap) snprintf(err, errcap, "%s", g_err);
        return -1;
    }
    if (&apus_backend_hooks) {
        apus_backend_hooks.bf16_gemv =
            getenv("APUS_CUDA_NO_GEMV") ? nullptr : hook_gemv;
        apus_backend_hooks.bf16_gemm =
            getenv("APUS_CUDA_NO_GEMM") ? nullptr : hook_gemm;
        apus_backend_hooks.bf16_matvec_f32 =
            getenv("APUS_CUDA_NO_MATVEC") ? nullptr : hook_matvec;
    }
    apus_cuda_block_hooks.moe_block =
        getenv("APUS_CUDA_NO_MOE") ? nullptr : apus_cuda_moe_block;
    g_ctx->hooks_filled = true;
    return 0;
}

static void layer_free(ApusCudaLayer *L) {
    if (!L) return;
    void *ptrs[] = {L->rtr_w, L->exp_gu, L->exp_d, L->sh_g,
                    L->sh_u,  L->sh_d,   L->sh_gate};
    for (void *p : ptrs)
        if (p) cudaFree(p);
    if (L->d_wnorm) cudaFree(L->d_wnorm);
    if (L->maps) prefill_maps_free(L->maps);
    if (g_ctx && g_ctx->bytes_resident >= L->bytes)
        g_ctx->bytes_resident -= L->bytes;
    delete L;
}

extern "C" void apus_cuda_disable(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (&apus_backend_hooks)
        memset(&apus_backend_hooks, 0, sizeof apus_backend_hooks);
    apus_cuda_block_hooks.moe_block = nullptr;
    Ctx *c = g_ctx;
    if (!c) return;
    cudaDeviceSynchronize();
    for (auto &kv : c->wcache) cudaFree(kv.second.ptr);
    for (auto &kv : c->layers) layer_free(kv.second);
    arena_free(c->ws);
    arena_free(c->io);
    if (c->last_ev) cudaEventDestroy(c->last_ev);
    if (c->d_status) cudaFree(c->d_status);
    if (c->d_router_counters) cudaFree(c->d_router_counters);
    if (c->d_rc_stats) cudaFree(c->d_rc_stats);
    if (c->d_df_logits) cudaFree(c->d_df_logits);
    if (c->d_df_sgl) cudaFree(c->d_df_sgl);
    if (c->d_df_sync) cudaFree(c->d_df_sync);
    if (c->d_df_timeline) cudaFree(c->d_df_timeline);
    if (c->d_df_act) cudaFree(c->d_df_act);
    if (c->d_df_sa) cudaFree(c->d_df_sa);
    if (c->d_router_logits) cudaFree(c->d_router_logits);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->s_in) cudaStreamDestroy(c->s_in);
    if (c->s_out) cudaStreamDestroy(c->s_out);
    for (auto &e : c->ev_io)
        if (e) cudaEventDestroy(e);
    g_ctx = nullptr;
    delete c;
}

extern "C" int apus_cuda_is_enabled(void) {
    return g_ctx && g_ctx->hooks_filled;
}
extern "C" uint64_t apus_cuda_bytes_resident(void) {
    return g_ctx ? g_ctx->bytes_resident : 0;
}
extern "C" uint64_t apus_cuda_bytes_uploaded(void) {
    return g_ctx ? g_ctx->bytes_uploaded : 0;
}
extern "C" uint64_t apus_cuda_launches(void) {
    return g_ctx ? g_ctx->launches : 0;
}
extern "C" const char *apus_cuda_last_error(void) { return g_err; }

/* ------------------------------------------------------------------------ */
/* per-matmul entry points (host pointers)                                   */
/* ------------------------------------------------------------------------ */

static void *weight_buf(Ctx *c, const void *ptr, size_t bytes) {
    auto it = c->wcache.find(ptr);
    if (it != c->wcache.end()) {
        if (it->second.bytes >= bytes) return it->second.ptr;
        /* same key, larger view: replace the copy */
        cudaFree(it->second.ptr);
        c->bytes_resident -= it->second.bytes;
        c->wcache.erase(it);
    }
    if (c->bytes_resident + bytes > c->budget) {
        fail("weight budget exhausted (APUS_CUDA_DENSE_MB)");
        return nullptr;
    }
    void *d = nullptr;
    if (cudaMalloc(&d, bytes) != cudaSuccess) {
        fail("cudaMalloc(%zu) for a weight failed", bytes);
        cudaGetLastError();
        return nullptr;
    }
    if (cudaMemcpy(d, ptr, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        fail("weight upload failed");
        cudaFree(d);
        return nullptr;
    }
    c->bytes_resident += bytes;
    c->bytes_uploaded += bytes;
    c->wcache.emplace(ptr, DevBuf{d, bytes});
    return d;
}

static int dense_op(const uint16_t *w, const uint16_t *x, void *y, size_t M,
                    size_t O, size_t K, bool f32_out) {
    if (!M || !O || !K) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    Ordered ord(c, c->stream);
    if (ord.rc) return 1;
    const uint16_t *dw = (const uint16_t *)weight_buf(c, w, O * K * 2);
    if (!dw) return 1;
    size_t xb = M * K * 2, yb = M * O * (f32_out ? 4 : 2);
    if (arena_reserve(c->io, xb + yb + 1024)) return 1;
    c->io.reset();
    uint16_t *dx = (uint16_t *)c->io.take(xb);
    void *dy = c->io.take(yb);
    CU_OK(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, c->stream));
    long total = (long)(M * O);
    int blocks = (int)((total + 127) / 128);
    if (blocks > c->sm_count * 16) blocks = c->sm_count * 16;
    if (f32_out)
        exact_matvec_f32_kernel<<<blocks, 128, 0, c->stream>>>(
            dw, dx, (float *)dy, (long)O, (int)K);
    else
        exact_gemm_kernel<<<blocks, 128, 0, c->stream>>>(
            dw, dx, (uint16_t *)dy, (long)M, (long)O, (int)K);
    LAUNCHED();
    CU_OK(cudaMemcpyAsync(y, dy, yb, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int apus_cuda_bf16_gemv(const uint16_t *w, const uint16_t *x,
                                   uint16_t *y, size_t O, size_t K) {
    return dense_op(w, x, y, 1, O, K, false);
}
extern "C" int apus_cuda_bf16_gemm(const uint16_t *w, const uint16_t *x,
                                   uint16_t *y, size_t M, size_t O, size_t K) {
    return dense_op(w, x, y, M, O, K, false);
}
extern "C" int apus_cuda_bf16_matvec_f32(const uint16_t *w, const uint16_t *x,
                                         float *y, size_t O, size_t K) {
    return dense_op(w, x, y, 1, O, K, true);
}

/* ------------------------------------------------------------------------ */
/* router / dispatch launches                                                */
/* ------------------------------------------------------------------------ */

template <int TT>
static int launch_router_tt(Ctx *c, const uint16_t *dx, const uint16_t *dwr,
                            int T, int E, int K, int topk, float wmin,
                            int32_t *didx, uint16_t *dw, uint16_t *dlogits,
                            const uint16_t *extra_row, uint16_t *extra_out,
                            cudaStream_t st) {
    size_t smem = ((size_t)TT * K + (size_t)TT * E) * sizeof(float);
    if (smem > (size_t)c->smem_optin)
        return fail("router tile does not fit shared memory (K=%d E=%d)", K, E);
    CU_OK(cudaFuncSetAttribute(router_topk_kernel<TT>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem));
    int grid = (T + TT - 1) / TT;
    launch_k(router_topk_kernel<TT>, dim3(grid), dim3(ROUTER_THREADS), smem, st, dx, dwr, T, E, K, topk, wmin, didx, dw, dlogits, extra_row, extra_out);
    LAUNCHED();
    return 0;
}

/* optional inputs of the certified many-token path */
struct RouterAux {
    const float *wnorm;     /* [E + 1] row norms of the router matrix */
    float wmin_extra;       /* smallest nonzero |extra_row| */
    float *approx_ws;       /* fp32 workspace, at least T*E*4 bytes */
    size_t approx_bytes;    /* its size: up to four [T, E] slabs are used */
};

static int launch_router(Ctx *c, const uint16_t *dx, const uint16_t *dwr, int T,
                         int E, int K, int topk, float wmin, int32_t *didx,
                         uint16_t *dw, uint16_t *dlogits,
                         const uint16_t *extra_row, uint16_t *extra_out,
                         cudaStream_t st, const RouterAux *aux = nullptr) {
    if (E < 1 || E > 1024 || topk < 1 || topk > 32 || topk > E || K < 1)
        return fail("router: unsupported E=%d topk=%d K=%d", E, topk, K);
    /* many tokens: fast logits on the tensor cores, exact chains only for the
     * experts that can still reach the top_k (router_certify.cuh) */
    if (c->router_certify && aux && aux->wnorm && aux->approx_ws && dlogits &&
        T > ROUTER_SMALL_MAX_T && E % PG_BM == 0 && K % 256 == 0 &&
        (((uintptr_t)dwr | (uintptr_t)dx | (uintptr_t)extra_row) & 15) == 0 &&
        router_certify_smem(E, K) <= (size_t)c->smem_optin) {
        int ksplit = dense_logits_ksplit(c->sm_count, T, E, K);
        while (ksplit > 1 && (size_t)ksplit * T * E * 4 > aux->approx_bytes) ksplit /= 2;
        if (run_dense_logits(c->sm_count, c->smem_optin, dwr, dx, T, E, K, ksplit,
                             aux->approx_ws, c->d_status, st,
                             &c->last_block_launches))
            return fail("%s", prefill_last_error());
        c->launches++;
        CertifyArgs ca;
        memset(&ca, 0, sizeof ca);
        ca.approx = aux->approx_ws;
        ca.nslab = ksplit;
        ca.x = dx;
        ca.w = dwr;
        ca.extra_row = extra_row;
        ca.wnorm = aux->wnorm;
        ca.T = T; ca.E = E; ca.K = K; ca.topk = topk;
        ca.wmin = wmin;
        ca.wmin_extra = aux->wmin_extra;
        /* the sequential chain errs by at most (K-1)u times the sum of the
         * term magnitudes; the tensor cores are granted eight times that */
        ca.cbound = 9.1f * (float)K * 5.9604645e-8f;   /* = debug_fast_logits' *cbound */
        ca.logits = nullptr;        /* nobody reads the merged logits */
        ca.idx_out = didx;
        ca.w_out = dw;
        ca.extra_out = extra_out;
        ca.status = c->d_status;
        ca.stats = c->d_rc_stats;
        const size_t smem = router_certify_smem(E, K);
        static size_t set_smem = 0;
        if (smem > set_smem) {
            CU_OK(cudaFuncSetAttribute(router_certify_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
            set_smem = smem;
        }
        launch_k(router_certify_kernel, dim3((T + RC_TT - 1) / RC_TT), dim3(RC_THREADS),
                 smem, st, ca);
        LAUNCHED();
        return 0;
    }
    /* few tokens: rows spread over many small CTAs, everything in flight at
     * once (latency path) */
    if (T <= ROUTER_SMALL_MAX_T && (K & 7) == 0 &&
        (((uintptr_t)dwr | (uintptr_t)extra_row) & 15) == 0) {
        const int rows = E + (extra_row ? 1 : 0);
        /* four tokens and one chain warp per CTA: two chain warps over eight
         * tokens measured slower (33 against 24 us at 32 tokens) */
        constexpr int tok = 4;
        const size_t smem = router_small_smem(E, K, tok);
        if (smem <= (size_t)c->smem_optin) {
            static size_t set_smem = 48 * 1024;
            auto kern = router_small_kernel<tok>;
            if (smem > set_smem) {
                CU_OK(cudaFuncSetAttribute(
                    kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                set_smem = smem;
            }
            dim3 grid((rows + ROUTER_SMALL_ROWS - 1) / ROUTER_SMALL_ROWS, (T + tok - 1) / tok);
            launch_k(kern, dim3(grid), dim3(ROUTER_SMALL_THREADS), smem, st, dx, dwr, T, E, K,
                     topk, wmin, aux ? aux->wmin_extra : 0.0f, didx, dw, dlogits, extra_row,
                     extra_out, c->d_router_logits, c->d_router_counters, c->d_status);
            LAUNCHED();
            return 0;
        }
    }
    /* many tokens: TMA-staged router tiles, then one warp per token */
    if (T > ROUTER_SMALL_MAX_T && dlogits && E % 256 == 0 && K % RL_BK == 0 &&
        (((uintptr_t)dwr | (uintptr_t)dx) & 15) == 0) {
        PFN_encodeTiled_local enc = tensor_map_encoder();
        if (!enc) return fail("%s", prefill_last_error());
        CUtensorMap map_w;
        if (encode_2d(enc, &map_w, dwr, (size_t)E, (size_t)K))
            return fail("%s", prefill_last_error());
        /* the token tile sets the L2 traffic (T/TT copies of the matrix);
         * take the largest one that still gives every SM a CTA */
        const int tt = T >= 32 * c->sm_count ? 32 : (T >= 16 * c->sm_count ? 16 : 8);
        const int rows = tt == 8 ? 128 : 256;
        const size_t xb = ((size_t)tt * RL_XPITCH * 4 + 1023) & ~(size_t)1023;
        const size_t smem = RL_STAGES * ((size_t)rows * RL_BK * 2 + xb) + 1024 + 64;
        dim3 grid((T + tt - 1) / tt, E / rows);
#define RL_LAUNCH(TTV, ROWSV)                                                   \
        do {                                                                    \
            static bool set_ = false;                                           \
            if (!set_) {                                                        \
                CU_OK(cudaFuncSetAttribute(                                     \
                    router_logits_kernel<TTV, ROWSV>,                           \
                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
                set_ = true;                                                    \
            }                                                                   \
            launch_k(router_logits_kernel<TTV, ROWSV>, grid, dim3(ROWSV + 32),  \
                     smem, st, map_w, dx, T, E, K, wmin, dlogits, extra_row,    \
                     extra_out, c->d_status);                                   \
        } while (0)
        if (tt == 32) RL_LAUNCH(32, 256);
        else if (tt == 16) RL_LAUNCH(16, 256);
        else RL_LAUNCH(8, 128);
#undef RL_LAUNCH
        LAUNCHED();
        launch_k(router_select_kernel, dim3((T + 7) / 8), dim3(256),
                 (size_t)8 * E * sizeof(float), st, dlogits, T, E, topk, didx, dw);
        LAUNCHED();
        return 0;
    }
    /* one token per CTA keeps the chain latency low for moderate T;
     * large T: eight chains per thread amortise the weight reads */
    if (T <= 2 * c->sm_count)
        return launch_router_tt<1>(c, dx, dwr, T, E, K, topk, wmin, didx, dw,
                                   dlogits, extra_row, extra_out, st);
    size_t smem8 = ((size_t)8 * K + (size_t)8 * E) * sizeof(float);
    if (smem8 <= (size_t)c->smem_optin)
        return launch_router_tt<8>(c, dx, dwr, T, E, K, topk, wmin, didx, dw,
                                   dlogits, extra_row, extra_out, st);
    return launch_router_tt<1>(c, dx, dwr, T, E, K, topk, wmin, didx, dw,
                               dlogits, extra_row, extra_out, st);
}

static size_t dispatch_scratch_bytes(size_t A, size_t E) {
    size_t units = (A + DISPATCH_UNIT - 1) / DISPATCH_UNIT;
    return units * E * sizeof(int32_t);
}

/* tp (optional, in/out): tile lists wanted with the dispatch.  The one-CTA
 * kernel builds them in the same launch and leaves tp->on set; the three-pass
 * form clears it and the caller launches build_tiles_kernel. */
static int launch_dispatch(Ctx *c, const int32_t *didx, int A, int E,
                           DispatchOut o, int32_t *unit_hist,
                           cudaStream_t st, DispatchKey kx = DispatchKey{0, 1},
                           TilePlan *tp = nullptr) {
    if (E < 1 || E > 1024) return fail("dispatch: unsupported E=%d", E);
    if (A <= DISPATCH_SMALL_MAX) {
        const size_t smem = (size_t)32 * E * sizeof(int);
        static bool attr_set = false;
        if (!attr_set) {
            CU_OK(cudaFuncSetAttribute(dispatch_small_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       32 * 1024 * (int)sizeof(int)));
            attr_set = true;
        }
        TilePlan none;
        memset(&none, 0, sizeof none);
        launch_k(dispatch_small_kernel, dim3(1), dim3(1024), smem, st, didx, A, E, kx, o,
                 c->d_status, tp ? *tp : none);
        LAUNCHED();
        return 0;
    }
    if (tp) tp->on = 0;
    int units = (A + DISPATCH_UNIT - 1) / DISPATCH_UNIT;
    int blocks = (units + DISPATCH_WARPS - 1) / DISPATCH_WARPS;
    size_t smem = (size_t)DISPATCH_WARPS * E * sizeof(int);
    launch_k(dispatch_hist_kernel, dim3(blocks), dim3(DISPATCH_WARPS * 32), smem, st, didx, A, E, kx, unit_hist, c->d_status);
    LAUNCHED();
    launch_k(dispatch_scan_kernel, dim3(1), dim3(1024), 0, st, unit_hist, units, E, o);
    LAUNCHED();
    launch_k(dispatch_permute_kernel, dim3(blocks), dim3(DISPATCH_WARPS * 32), smem, st, didx, A, E, kx, unit_hist, o);
    LAUNCHED();
    return 0;
}

/* ------------------------------------------------------------------------ */
/* router / dispatch, host pointers                                          */
/* ------------------------------------------------------------------------ */

static int min_nonzero(Ctx *c, const uint16_t *d, size_t n, float *out,
                       cudaStream_t st) {
    unsigned int inf = 0x7f800000u;
    CU_OK(cudaMemcpyAsync(c->d_scratch_u32, &inf, 4, cudaMemcpyHostToDevice, st));
    bf16_min_nonzero_kernel<<<c->sm_count * 2, 256, 0, st>>>(d, n,
                                                             c->d_scratch_u32);
    LAUNCHED();
    unsigned int bits = 0;
    CU_OK(cudaMemcpyAsync(&bits, c->d_scratch_u32, 4, cudaMemcpyDeviceToHost, st));
    CU_OK(cudaStreamSynchronize(st));
    float f;
    memcpy(&f, &bits, 4);
    *out = (bits >= 0x7f800000u) ? 0.0f : f;
    return 0;
}

/* what the router kernels need to know about a layer's router weights: the
 * smallest nonzero magnitudes (fused multiply-add guard) and the row norms
 * (error bound of the fast logits) */
static int layer_router_stats(Ctx *c, ApusCudaLayer *L) {
    const size_t E = L->cfg.experts, H = L->cfg.hidden;
    if (min_nonzero(c, L->rtr_w, E * H, &L->wmin, c->stream) ||
        min_nonzero(c, L->sh_gate, H, &L->wmin_gate, c->stream))
        return 1;
    if (!L->d_wnorm) CU_OK(cudaMalloc(&L->d_wnorm, (E + 1) * sizeof(float)));
    CU_OK(cudaMemsetAsync(L->d_wnorm, 0, (E + 1) * sizeof(float), c->stream));
    row_norm_kernel<<<(unsigned)((E * 32 + 255) / 256), 256, 0, c->stream>>>(
        L->rtr_w, (int)E, (int)H, L->d_wnorm);
    LAUNCHED();
    CU_OK(cudaStreamSynchronize(c->stream));
    return 0;
}

static int route_host(const uint16_t *x, const uint16_t *wg, int32_t *idx,
                      uint16_t *w, uint16_t *logits, size_t T, size_t E,
                      size_t K, size_t topk) {
    if (!T || !E || !K || !topk) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    Ordered ord(c, c->stream);
    if (ord.rc) return 1;
    size_t need = T * K * 2 + E * K * 2 + T * topk * 6 + T * E * 2 + 4096;
    if (arena_reserve(c->io, need)) return 1;
    c->io.reset();
    uint16_t *dx = (uint16_t *)c->io.take(T * K * 2);
    uint16_t *dwr = (uint16_t *)c->io.take(E * K * 2);
    int32_t *didx = (int32_t *)c->io.take(T * topk * 4);
    uint16_t *dw = (uint16_t *)c->io.take(T * topk * 2);
    uint16_t *dl = (uint16_t *)c->io.take(T * E * 2);
    CU_OK(cudaMemcpyAsync(dx, x, T * K * 2, cudaMemcpyHostToDevice, c->stream));
    CU_OK(cudaMemcpyAsync(dwr, wg, E * K * 2, cudaMemcpyHostToDevice, c->stream));
    float wmin = 0.0f;
    if (min_nonzero(c, dwr, E * K, &wmin, c->stream)) return 1;
    if (launch_router(c, dx, dwr, (int)T, (int)E, (int)K, (int)topk, wmin, didx,
                      w ? dw : nullptr, dl, nullptr, nullptr, c->stream))
        return 1;
    CU_OK(cudaMemcpyAsync(idx, didx, T * topk * 4, cudaMemcpyDeviceToHost,
                          c->stream));
    if (w)
        CU_OK(cudaMemcpyAsync(w, dw, T * topk * 2, cudaMemcpyDeviceToHost,
                              c->stream));
    if (logits)
        CU_OK(cudaMemcpyAsync(logits, dl, T * E * 2, cudaMemcpyDeviceToHost,
                              c->stream));
    CU_OK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int apus_cuda_moe_route(const uint16_t *x, const uint16_t *wg,
                                   int32_t *idx, uint16_t *w, uint16_t *logits,
                                   size_t T, size_t E, size_t K, size_t topk) {
    return route_host(x, wg, idx, w, logits, T, E, K, topk);
}
extern "C" int apus_cuda_moe_route_topn(const uint16_t *x, const uint16_t *wg,
                                        int32_t *idx, size_t n, size_t E,
                                        size_t K) {
    return route_host(x, wg, idx, nullptr, nullptr, 1, E, K, n);
}

extern "C" int apus_cuda_moe_dispatch(const int32_t *idx, size_t T, size_t topk,
                                      size_t E, int32_t *counts,
                                      int32_t *offsets, int32_t *perm) {
    size_t A = T * topk;
    if (!A || !E) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    Ordered ord(c, c->stream);
    if (ord.rc) return 1;
    size_t need = A * 8 + (2 * E + 1) * 4 + dispatch_scratch_bytes(A, E) + 4096;
    if (arena_reserve(c->io, need)) return 1;
    c->io.reset();
    int32_t *didx = (int32_t *)c->io.take(A * 4);
    DispatchOut o;
    memset(&o, 0, sizeof o);
    o.counts = (int32_t *)c->io.take(E * 4);
    o.offsets = (int32_t *)c->io.take((E + 1) * 4);
    o.perm = (int32_t *)c->io.take(A * 4);
    int32_t *uh = (int32_t *)c->io.take(dispatch_scratch_bytes(A, E));
    CU_OK(cudaMemcpyAsync(didx, idx, A * 4, cudaMemcpyHostToDevice, c->stream));
    CU_OK(cudaMemsetAsync(c->d_status, 0, 4, c->stream));
    if (launch_dispatch(c, didx, (int)A, (int)E, o, uh, c->stream)) return 1;
    CU_OK(cudaMemcpyAsync(counts, o.counts, E * 4, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(cudaMemcpyAsync(offsets, o.offsets, (E + 1) * 4, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(cudaMemcpyAsync(perm, o.perm, A * 4, cudaMemcpyDeviceToHost, c->stream));
    int st = 0;
    CU_OK(cudaMemcpyAsync(&st, c->d_status, 4, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(cudaStreamSynchronize(c->stream));
    if (st) return fail("dispatch: expert id out of range (status %d)", st);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* layers                                                                    */
/* ------------------------------------------------------------------------ */

static int cfg_check(const ApusCudaMoeCfg *c) {
    if (!c) return fail("null config");
    if (!c->hidden || !c->experts || !c->moe_inter || !c->shared_inter ||
        !c->top_k)
        return fail("zero dimension in MoE config");
    if (c->hidden % 8 || c->moe_inter % 8 || c->shared_inter % 8)
        return fail("hidden, moe_inter and shared_inter must be multiples of 8");
    if (c->experts > 1024 || c->top_k > 32 || c->top_k > c->experts)
        return fail("unsupported experts=%zu top_k=%zu", c->experts, c->top_k);
    return 0;
}

extern "C" int apus_cuda_layer_create(const ApusCudaMoeCfg *cfg,
                                      const ApusCudaMoeW *w,
                                      size_t expert_begin, size_t expert_end,
                                      ApusCudaLayer **out) {
    if (!out) return fail("null out");
    *out = nullptr;
    if (cfg_check(cfg)) return 1;
    if (expert_begin > expert_end || expert_end > cfg->experts)
        return fail("bad expert range [%zu,%zu)", expert_begin, expert_end);
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    const size_t H = cfg->hidden, E = cfg->experts, I = cfg->moe_inter,
                 Is = cfg->shared_inter;
    const size_t ne = expert_end - expert_begin;
    ApusCudaLayer *L = new ApusCudaLayer();
    L->cfg = *cfg;
    L->e_begin = expert_begin;
    L->e_end = expert_end;
    struct Item { uint16_t **dst; size_t elems; const uint16_t *src; };
    Item items[] = {
        {&L->rtr_w, E * H, w ? w->rtr_w : nullptr},
        {&L->exp_gu, ne * 2 * I * H,
         w && w->exp_gu ? w->exp_gu + expert_begin * 2 * I * H : nullptr},
        {&L->exp_d, ne * H * I,
         w && w->exp_d ? w->exp_d + expert_begin * H * I : nullptr},
        {&L->sh_g, Is * H, w ? w->sh_g : nullptr},
        {&L->sh_u, Is * H, w ? w->sh_u : nullptr},
        {&L->sh_d, H * Is, w ? w->sh_d : nullptr},
        {&L->sh_gate, H, w ? w->sh_gate : nullptr},
    };
    for (auto &it : items) {
        size_t bytes = it.elems * 2;
        if (!bytes) continue;
        if (c->bytes_resident + L->bytes + bytes > c->budget) {
            layer_free(L);
            return fail("weight budget exhausted (APUS_CUDA_DENSE_MB)");
        }
        if (cudaMalloc((void **)it.dst, bytes) != cudaSuccess) {
            cudaGetLastError();
            layer_free(L);
            return fail("cudaMalloc(%zu) for layer weights failed", bytes);
        }
        L->bytes += bytes;
        if (it.src) {
            if (cudaMemcpy(*it.dst, it.src, bytes, cudaMemcpyHostToDevice) !=
                cudaSuccess) {
                layer_free(L);
                return fail("layer weight upload failed");
            }
            c->bytes_uploaded += bytes;
        }
    }
    c->bytes_resident += L->bytes;
    L->maps = nullptr;
    if (w && w->rtr_w) {
        if (layer_router_stats(c, L)) {
            layer_free(L);
            return 1;
        }
    }
    *out = L;
    return 0;
}

extern "C" void apus_cuda_layer_destroy(ApusCudaLayer *layer) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (g_ctx) cudaDeviceSynchronize();
    layer_free(layer);
}

extern "C" void *apus_cuda_layer_tensor(ApusCudaLayer *L, int which,
                                        size_t *elems) {
    if (!L) return nullptr;
    const size_t H = L->cfg.hidden, E = L->cfg.experts, I = L->cfg.moe_inter,
                 Is = L->cfg.shared_inter, ne = L->e_end - L->e_begin;
    void *p = nullptr;
    size_t n = 0;
    switch (which) {
        case 1: p = L->rtr_w; n = E * H; break;
        case 2: p = L->exp_gu; n = ne * 2 * I * H; break;
        case 3: p = L->exp_d; n = ne * H * I; break;
        case 4: p = L->sh_g; n = Is * H; break;
        case 5: p = L->sh_u; n = Is * H; break;
        case 6: p = L->sh_d; n = H * Is; break;
        case 7: p = L->sh_gate; n = H; break;
        default: break;
    }
    if (elems) *elems = n;
    return p;
}

extern "C" int apus_cuda_layer_refresh(ApusCudaLayer *L) {
    if (!L) return fail("null layer");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    /* set-up call: whatever stream filled the tensor, wait for it */
    CU_OK(cudaDeviceSynchronize());
    return layer_router_stats(g_ctx, L);
}

extern "C" int apus_cuda_layer_upload(ApusCudaLayer *L, int which,
                                      const uint16_t *src, size_t first,
                                      size_t n) {
    size_t elems = 0;
    uint16_t *dst = (uint16_t *)apus_cuda_layer_tensor(L, which, &elems);
    if (!dst || !src || !n || first > elems || n > elems - first)
        return fail("layer_upload: bad tensor id or range");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    /* set-up call: synchronous, whatever stream used the tensor before */
    CU_OK(cudaDeviceSynchronize());
    CU_OK(cudaMemcpy(dst + first, src, n * 2, cudaMemcpyHostToDevice));
    g_ctx->bytes_uploaded += n * 2;
    if (which == 1 || which == 7) return layer_router_stats(g_ctx, L);
    return 0;
}

extern "C" int apus_cuda_layer_load_slabs(ApusCudaLayer *L, const char *container_dir,
                                          int layer_index) {
    if (!L || !container_dir || layer_index < 0) return fail("layer_load_slabs: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    if (L->e_end == L->e_begin) return 0;
    CU_OK(cudaDeviceSynchronize());
    char err[400] = "";
    const long long n = load_layer_slabs(container_dir, layer_index, L->e_begin, L->e_end,
                                         L->cfg.hidden, L->cfg.moe_inter, L->exp_gu, L->exp_d,
                                         err, sizeof err);
    if (n < 0) return fail("layer_load_slabs: %s", err);
    g_ctx->bytes_uploaded += (uint64_t)n;
    return 0;
}

/* ||x_t||_2 with the margin router_certify_kernel applies (one warp per row) */
__global__ void __launch_bounds__(256)
dbg_xnorm_kernel(const uint16_t *__restrict__ x, int T, int K, float *__restrict__ out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    float ss = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float v = bf16_f32(x[(size_t)warp * K + k]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) out[warp] = sqrtf(ss) * 1.001f;
}
__global__ void __launch_bounds__(256)
dbg_sum_slabs_kernel(const float *__restrict__ slabs, int nslab, size_t n,
                     float *__restrict__ out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        float p[RC_MAX_SLABS];
        for (int sl = 0; sl < RC_MAX_SLABS; sl++) p[sl] = sl < nslab ? slabs[sl * n + i] : 0.0f;
        out[i] = (p[0] + p[1]) + (p[2] + p[3]);     /* the certify kernel's order */
    }
}

extern "C" int apus_cuda_debug_fast_logits(const uint16_t *x, const uint16_t *wg,
                                           size_t T, size_t E, size_t K,
                                           float *fast, float *xnorm,
                                           float *wnorm, float *cbound) {
    if (!x || !wg || !fast || !xnorm || !wnorm || !cbound || !T || !E || !K)
        return fail("debug_fast_logits: bad args");
    if (E % PG_BM || K % 256) return fail("debug_fast_logits: E %% 128 or K %% 256");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    Ordered ord(c, c->stream);
    if (ord.rc) return 1;
    cudaStream_t st = c->stream;
    const size_t need = T * K * 2 + E * K * 2 + (RC_MAX_SLABS + 1) * T * E * 4 +
                        (T + E + 1) * 4 + 8192;
    if (arena_reserve(c->io, need)) return 1;
    c->io.reset();
    uint16_t *dx = (uint16_t *)c->io.take(T * K * 2);
    uint16_t *dw = (uint16_t *)c->io.take(E * K * 2);
    float *slabs = (float *)c->io.take(RC_MAX_SLABS * T * E * 4);
    float *dfast = (float *)c->io.take(T * E * 4);
    float *dxn = (float *)c->io.take(T * 4);
    float *dwn = (float *)c->io.take((E + 1) * 4);
    CU_OK(cudaMemcpyAsync(dx, x, T * K * 2, cudaMemcpyHostToDevice, st));
    CU_OK(cudaMemcpyAsync(dw, wg, E * K * 2, cudaMemcpyHostToDevice, st));
    CU_OK(cudaMemsetAsync(dwn, 0, (E + 1) * 4, st));
    CU_OK(cudaMemsetAsync(c->d_status, 0, 4, st));
    /* the same K split the block's router would choose for this shape */
    const int ksplit = dense_logits_ksplit(c->sm_count, (int)T, (int)E, (int)K);
    int launches = 0;
    if (run_dense_logits(c->sm_count, c->smem_optin, dw, dx, (int)T, (int)E, (int)K,
                         ksplit, slabs, c->d_status, st, &launches))
        return fail("%s", prefill_last_error());
    dbg_sum_slabs_kernel<<<c->sm_count * 4, 256, 0, st>>>(slabs, ksplit, T * E, dfast);
    dbg_xnorm_kernel<<<(unsigned)((T * 32 + 255) / 256), 256, 0, st>>>(dx, (int)T, (int)K, dxn);
    row_norm_kernel<<<(unsigned)((E * 32 + 255) / 256), 256, 0, st>>>(dw, (int)E, (int)K, dwn);
    LAUNCHED();
    CU_OK(cudaMemcpyAsync(fast, dfast, T * E * 4, cudaMemcpyDeviceToHost, st));
    CU_OK(cudaMemcpyAsync(xnorm, dxn, T * 4, cudaMemcpyDeviceToHost, st));
    CU_OK(cudaMemcpyAsync(wnorm, dwn, (E + 1) * 4, cudaMemcpyDeviceToHost, st));
    int stw = 0;
    CU_OK(cudaMemcpyAsync(&stw, c->d_status, 4, cudaMemcpyDeviceToHost, st));
    CU_OK(cudaStreamSynchronize(st));
    if (stw) return fail("debug_fast_logits: device status %d", stw);
    *cbound = 9.1f * (float)K * 5.9604645e-8f;
    return 0;
}

/* ------------------------------------------------------------------------ */
/* the block                                                                 */
/* ------------------------------------------------------------------------ */

struct BlockBufs {
    int32_t *idx;
    uint16_t *rw, *sgl, *logits;
    DispatchOut d;
    int32_t *unit_hist;
    uint16_t *act, *sa, *eo, *sy, *xg;
    void *tiles;           /* prefill tile lists */
    size_t total;
};

static size_t al256(size_t b) { return (b + 255) & ~(size_t)255; }
static int fused_scratch(Ctx *c, const ApusCudaMoeCfg &cfg);

/* carve (or just size, when a.base == NULL) the block's workspace */
static int block_layout(const ApusCudaMoeCfg &c, size_t T, Arena *a,
                        BlockBufs *b, bool prefill) {
    const size_t H = c.hidden, E = c.experts, I = c.moe_inter,
                 Is = c.shared_inter, TK = c.top_k, A = T * TK;
    size_t sz[] = {
        A * 4,                         /* idx */
        A * 2,                         /* rw */
        T * 2,                         /* sgl */
        T * E * 2,                     /* router logits */
        E * 4, (E + 1) * 4, A * 4, A * 4,            /* counts offsets perm pos */
        (A + E) * 4, (A + E) * 4, (A + E) * 4, 256,  /* groups, n_groups */
        dispatch_scratch_bytes(A, E),  /* unit_hist */
        A * I * 2, T * Is * 2, A * H * 2, T * H * 2, /* act sa eo sy */
        prefill ? A * H * 2 : 0,       /* xg */
        prefill ? prefill_tiles_bytes_for(c, A, T) : 0,
    };
    size_t total = 0;
    for (size_t s : sz) total += al256(s) + 256;
    b->total = total;
    if (!a) return 0;
    a->reset();
    void *p[sizeof sz / sizeof sz[0]];
    for (size_t i = 0; i < sizeof sz / sizeof sz[0]; i++) {
        p[i] = sz[i] ? a->take(sz[i]) : nullptr;
        if (sz[i] && !p[i]) return fail("workspace arena too small");
    }
    b->idx = (int32_t *)p[0];
    b->rw = (uint16_t *)p[1];
    b->sgl = (uint16_t *)p[2];
    b->logits = (uint16_t *)p[3];
    b->d.counts = (int32_t *)p[4];
    b->d.offsets = (int32_t *)p[5];
    b->d.perm = (int32_t *)p[6];
    b->d.pos = (int32_t *)p[7];
    b->d.grp_expert = (int32_t *)p[8];
    b->d.grp_first = (int32_t *)p[9];
    b->d.grp_n = (int32_t *)p[10];
    b->d.n_groups = (int32_t *)p[11];
    b->unit_hist = (int32_t *)p[12];
    b->act = (uint16_t *)p[13];
    b->sa = (uint16_t *)p[14];
    b->eo = (uint16_t *)p[15];
    b->sy = (uint16_t *)p[16];
    b->xg = (uint16_t *)p[17];
    b->tiles = p[18];
    return 0;
}

extern "C" int apus_cuda_reserve(const ApusCudaMoeCfg *cfg, size_t T) {
    if (cfg_check(cfg) || !T) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    BlockBufs b;
    block_layout(*cfg, T, nullptr, &b, true);
    g_ctx->cur_capturing = false;
    if (fused_scratch(g_ctx, *cfg)) return 1;
    return arena_reserve(g_ctx->ws, b.total + al256(T * cfg->hidden * 2) + 256);
}

static int decode_smem_bytes(const ApusCudaMoeCfg &c, bool down) {
    size_t H = c.hidden, Imax = c.moe_inter > c.shared_inter ? c.moe_inter
                                                             : c.shared_inter;
    size_t stage = down ? DOWN_ROWS * Imax : 2 * H;
    size_t xrow = down ? Imax : H;
    return (int)((DEC_WARPS * DEC_STAGES * stage + GROUP_TOKENS * xrow) * 2 +
                 DEC_WARPS * DEC_STAGES * 8 + 128);
}

/* routed and/or shared experts through the grouped-GEMV kernels.  x [T,H];
 * TK slots per token; routed outputs go to eo_out in flat assignment order;
 * expert ids in the group list are relative to expert_base. */
static int run_decode_experts(Ctx *c, ApusCudaLayer *L, const uint16_t *dx,
                              int T, int TK, int expert_base, BlockBufs &b,
                              bool do_shared, uint16_t *eo_out,
                              cudaStream_t st) {
    const ApusCudaMoeCfg &cfg = L->cfg;
    DecodeArgs a;
    memset(&a, 0, sizeof a);
    a.T = T;
    a.H = (int)cfg.hidden;
    a.I = (int)cfg.moe_inter;
    a.Is = (int)cfg.shared_inter;
    a.TK = TK;
    a.expert_begin = expert_base;
    a.x = dx;
    a.exp_gu = L->exp_gu;
    a.exp_d = L->exp_d;
    a.sh_g = L->sh_g;
    a.sh_u = L->sh_u;
    a.sh_d = L->sh_d;
    a.perm = b.d.perm;
    a.grp_expert = b.d.grp_expert;
    a.grp_first = b.d.grp_first;
    a.grp_n = b.d.grp_n;
    a.n_groups = b.d.n_groups;
    a.act = b.act;
    a.sa = b.sa;
    a.eo = eo_out;
    a.sy = b.sy;
    a.do_shared = do_shared ? 1 : 0;
    a.status = c->d_status;
    int s1 = decode_smem_bytes(cfg, false), s2 = decode_smem_bytes(cfg, true);
    if (s1 > c->smem_optin || s2 > c->smem_optin)
        return fail("decode kernels need %d/%d B shared memory (> %d)", s1, s2,
                    c->smem_optin);
    if (cfg.hidden % DOWN_ROWS) return fail("hidden must be a multiple of 8");
    static int set1 = 0, set2 = 0;
    if (s1 > set1) {
        CU_OK(cudaFuncSetAttribute(decode_gate_up_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, s1));
        set1 = s1;
    }
    if (s2 > set2) {
        CU_OK(cudaFuncSetAttribute(decode_down_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, s2));
        set2 = s2;
    }
    launch_k(decode_gate_up_kernel, dim3(c->sm_count), dim3(DEC_THREADS), s1, st, a);
    LAUNCHED();
    stage_mark(c, APUS_CUDA_STAGE_GATE_UP, st);
    launch_k(decode_down_kernel, dim3(c->sm_count), dim3(DEC_THREADS), s2, st, a);
    LAUNCHED();
    stage_mark(c, APUS_CUDA_STAGE_DOWN, st);
    return 0;
}

static int run_finalize(Ctx *c, const ApusCudaMoeCfg &cfg, int T,
                        const uint16_t *eo, const int32_t *pos,
                        const uint16_t *rw, const uint16_t *sy,
                        const uint16_t *sgl, uint16_t *d_out,
                        const ApusCudaMoeTrace *tr, cudaStream_t st,
                        const uint16_t *res = nullptr, uint16_t *res_out = nullptr) {
    FinalizeArgs f;
    memset(&f, 0, sizeof f);
    f.res = res;
    f.res_out = res_out;
    f.T = T;
    f.H = (int)cfg.hidden;
    f.TK = (int)cfg.top_k;
    f.eo = eo;
    f.pos = pos;
    f.rw = rw;
    f.sy = sy;
    f.sgl = sgl;
    f.out = d_out;
    f.tr_routed = tr ? tr->moe_routed : nullptr;
    f.tr_shared = tr ? tr->moe_shared : nullptr;
    f.tr_out = tr ? tr->moe_out : nullptr;
    long total = (long)T * (cfg.hidden / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > c->sm_count * 8) blocks = c->sm_count * 8;
    launch_k(moe_finalize_kernel, dim3(blocks), dim3(256), 0, st, f);
    LAUNCHED();
    return 0;
}


/* scratch of the one-kernel path, sized by the layer shape */
static int fused_scratch(Ctx *c, const ApusCudaMoeCfg &cfg) {
    const size_t need_act = (size_t)DF_MAX_A * cfg.moe_inter,
                 need_sa = (size_t)DF_MAX_T * cfg.shared_inter;
    if (c->df_act_elems >= need_act && c->df_sa_elems >= need_sa) return 0;
    if (c->cur_capturing)
        return fail("decode scratch missing inside a stream capture: call "
                    "apus_cuda_reserve before capturing");
    CU_OK(cudaDeviceSynchronize());
    /* outgrown buffers stay allocated until disable (older captures) */
    if (c->d_df_act) c->ws.retired.push_back(c->d_df_act);
    if (c->d_df_sa) c->ws.retired.push_back(c->d_df_sa);
    c->d_df_act = c->d_df_sa = nullptr;
    CU_OK(cudaMalloc(&c->d_df_act, need_act * 2));
    CU_OK(cudaMalloc(&c->d_df_sa, need_sa * 2));
    c->df_act_elems = need_act;
    c->df_sa_elems = need_sa;
    return 0;
}

/* The one-kernel path for a handful of tokens (cooperative launch). */
/* the two neighbours of the block folded into it (apus_cuda_moe_layer_dev) */
struct Residual {
    const uint16_t *res = nullptr, *ln_w = nullptr;
    uint16_t *res_out = nullptr;
};

static int run_fused_decode(Ctx *c, ApusCudaLayer *L, const uint16_t *d_ln2,
                            uint16_t *d_out, int T, const ApusCudaMoeTrace *tr,
                            cudaStream_t st, const Residual *rz = nullptr) {
    const ApusCudaMoeCfg &cfg = L->cfg;
    const int H = (int)cfg.hidden, I = (int)cfg.moe_inter,
              Is = (int)cfg.shared_inter, E = (int)cfg.experts,
              TK = (int)cfg.top_k;
    if (fused_scratch(c, cfg)) return 1;
    FusedArgs a;
    memset(&a, 0, sizeof a);
    a.T = T; a.H = H; a.I = I; a.Is = Is; a.E = E; a.TK = TK;
    a.stages = 3;
    size_t smem = decode_fused_smem(T, H, I, Is, E, TK, 3);
    if (smem > (size_t)c->smem_optin) {
        a.stages = 2;
        smem = decode_fused_smem(T, H, I, Is, E, TK, 2);
    }
    a.wmin = L->wmin;
    a.wmin_gate = L->wmin_gate;
    a.x = d_ln2;
    if (rz) {
        a.res = rz->res;
        a.ln_w = rz->ln_w;
        a.res_out = rz->res_out;
    }
    a.rtr_w = L->rtr_w; a.exp_gu = L->exp_gu; a.exp_d = L->exp_d;
    a.sh_g = L->sh_g; a.sh_u = L->sh_u; a.sh_d = L->sh_d; a.sh_gate = L->sh_gate;
    a.logits_ws = c->d_df_logits; a.sgl_ws = c->d_df_sgl;
    a.act_ws = c->d_df_act; a.sa_ws = c->d_df_sa; a.sync = c->d_df_sync;
    a.out = d_out;
    a.idx_out = tr ? tr->rtr_idx : nullptr;
    a.w_out = tr ? tr->rtr_w : nullptr;
    a.tr_routed = tr ? tr->moe_routed : nullptr;
    a.tr_shared = tr ? tr->moe_shared : nullptr;
    a.tr_out = tr ? tr->moe_out : nullptr;
    a.status = c->d_status;
    a.timeline = c->stage_timing ? c->d_df_timeline : nullptr;
    c->df_timeline_valid = c->stage_timing;
    static size_t set_smem = 0;
    if (smem > set_smem) {
        CU_OK(cudaFuncSetAttribute(decode_fused_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
        set_smem = smem;
    }
    cudaLaunchConfig_t cfgl = {};
    cfgl.gridDim = dim3(c->sm_count);
    cfgl.blockDim = dim3(DF_THREADS);
    cfgl.dynamicSmemBytes = smem;
    cfgl.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfgl.attrs = attr;
    cfgl.numAttrs = 1;
    CU_OK(cudaLaunchKernelEx(&cfgl, decode_fused_kernel, a));
    LAUNCHED();
    return 0;
}

static bool fused_supported(Ctx *c, const ApusCudaMoeCfg &cfg, size_t T) {
    if ((int)T > c->fused_max_t || T * cfg.top_k > DF_MAX_A) return false;
    if (cfg.experts > 1024 || cfg.hidden / 8 > 2 * (size_t)c->sm_count) return false;
    if (cfg.moe_inter * 2 > DF_STAGE_BYTES / 8 || cfg.shared_inter * 2 > DF_STAGE_BYTES / 8)
        return false;                      /* eight down rows per stage */
    if (cfg.hidden * 4 > DF_STAGE_BYTES) return false;   /* a gate+up row pair */
    size_t smem = decode_fused_smem((int)T, (int)cfg.hidden, (int)cfg.moe_inter,
                                    (int)cfg.shared_inter, (int)cfg.experts,
                                    (int)cfg.top_k, 2);
    return smem <= (size_t)c->smem_optin;
}

static int block_dev_locked(ApusCudaLayer *L, const uint16_t *d_ln2,
                            uint16_t *d_out, size_t T,
                            const ApusCudaMoeTrace *d_tr, cudaStream_t st,
                            const Residual *rz = nullptr) {
    Ctx *c = g_ctx;
    const ApusCudaMoeCfg &cfg = L->cfg;
    if (L->e_begin != 0 || L->e_end != cfg.experts)
        return fail("moe_block needs all experts resident; use the "
                    "expert-parallel entry points for a partial layer");
    c->last_block_launches = 0;
    c->df_timeline_valid = false;
    if (fused_supported(c, cfg, T)) {
        c->last_block_path = APUS_CUDA_PATH_FUSED;
        return run_fused_decode(c, L, d_ln2, d_out, (int)T, d_tr, st, rz);
    }
    const bool prefill = (int)T > c->decode_max_t && prefill_supported(cfg);
    BlockBufs b;
    block_layout(cfg, T, nullptr, &b, prefill);
    /* with the neighbours folded in, the normalised input lives behind the
     * block's own buffers */
    const size_t ln_bytes = rz ? al256(T * cfg.hidden * 2) + 256 : 0;
    if (arena_reserve(c->ws, b.total + ln_bytes)) return 1;
    if (block_layout(cfg, T, &c->ws, &b, prefill)) return 1;
    if (rz) {
        uint16_t *ln = (uint16_t *)c->ws.take(T * cfg.hidden * 2);
        if (!ln) return fail("workspace arena too small");
        const size_t smem = 4 * cfg.hidden * sizeof(float);
        if (smem > 48 * 1024) {
            if (smem > (size_t)c->smem_optin) return fail("rmsnorm: hidden too large");
            CU_OK(cudaFuncSetAttribute(rmsnorm_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        }
        rmsnorm_kernel<<<(unsigned)((T + 3) / 4), 128, smem, st>>>(rz->res, rz->ln_w, ln, (int)T,
                                                                   (int)cfg.hidden);
        LAUNCHED();
        d_ln2 = ln;
    }
    const int Ti = (int)T, E = (int)cfg.experts, H = (int)cfg.hidden,
              TK = (int)cfg.top_k;
    c->n_ev = 0;
    stage_mark(c, -1, st);
    /* the fast logits live in the combine buffer, which is written much later */
    RouterAux aux = {L->d_wnorm, L->wmin_gate, reinterpret_cast<float *>(b.eo),
                     (size_t)Ti * TK * H * 2};
    if (launch_router(c, d_ln2, L->rtr_w, Ti, E, H, TK, L->wmin, b.idx, b.rw,
                      b.logits, L->sh_gate, b.sgl, st,
                      (size_t)E * 4 <= (size_t)TK * H * 2 ? &aux : nullptr))
        return 1;
    stage_mark(c, APUS_CUDA_STAGE_ROUTER, st);
    if (prefill) {
        /* token groups feed the grouped-GEMV kernels only */
        b.d.grp_expert = nullptr;
        b.d.grp_first = nullptr;
        b.d.grp_n = nullptr;
        b.d.n_groups = nullptr;
    }
    /* many rows per expert: the kernels in which two SMs share a tile */
    const bool pair = prefill && pair_supported(cfg, c->sm_count, c->smem_optin) &&
                      (size_t)Ti * TK >= (size_t)g_pp_min_rows * E;
    c->last_block_path = pair ? APUS_CUDA_PATH_GEMM_2SM
                              : (prefill ? APUS_CUDA_PATH_GEMM : APUS_CUDA_PATH_GEMV);
    TilePlan plan;
    memset(&plan, 0, sizeof plan);
    if (prefill && !pair) plan = prefill_tile_plan(cfg, Ti, true, Ti * TK, b.tiles);
    if (launch_dispatch(c, b.idx, Ti * TK, E, b.d, b.unit_hist, st, DispatchKey{0, 1},
                        prefill && !pair ? &plan : nullptr))
        return 1;
    stage_mark(c, APUS_CUDA_STAGE_DISPATCH, st);
    if (pair) {
        const int before = c->last_block_launches;
        g_mark_stream = st;
        if (run_pair_experts(c->sm_count, c->smem_optin, L->maps, cfg, (int)L->e_begin,
                             d_ln2, Ti, Ti * TK, TK, true, b.d, b.xg, b.act, b.sa, b.eo,
                             b.sy, b.tiles, c->d_status, st, &c->last_block_launches,
                             mark_cb))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
    } else if (prefill) {
        const int before = c->last_block_launches;
        g_mark_stream = st;
        if (run_prefill_experts(c->sm_count, c->smem_optin, L->maps, cfg,
                                (int)L->e_begin, d_ln2, Ti, Ti * TK, TK, true, b.d,
                                b.xg, b.act, b.sa, b.eo, b.sy, b.tiles,
                                c->d_status, st, &c->last_block_launches,
                                mark_cb, plan.on ? &plan : nullptr))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
    } else {
        if (run_decode_experts(c, L, d_ln2, Ti, TK, 0, b, true, b.eo, st)) return 1;
    }
    if (run_finalize(c, cfg, Ti, b.eo, nullptr, b.rw, b.sy, b.sgl, d_out, d_tr, st,
                     rz ? rz->res : nullptr, rz ? rz->res_out : nullptr))
        return 1;
    stage_mark(c, APUS_CUDA_STAGE_FINALIZE, st);
    if (d_tr && d_tr->rtr_idx)
        CU_OK(cudaMemcpyAsync(d_tr->rtr_idx, b.idx, T * TK * 4,
                              cudaMemcpyDeviceToDevice, st));
    if (d_tr && d_tr->rtr_w)
        CU_OK(cudaMemcpyAsync(d_tr->rtr_w, b.rw, T * TK * 2,
                              cudaMemcpyDeviceToDevice, st));
    return 0;
}

extern "C" int apus_cuda_moe_block_dev(ApusCudaLayer *layer,
                                       const uint16_t *d_ln2, uint16_t *d_out,
                                       size_t T, const ApusCudaMoeTrace *d_tr,
                                       void *stream) {
    if (!T) return 0;      /* the engine's loops over T run zero times (c/layer.h:589) */
    if (!layer || !d_ln2 || !d_out) return fail("moe_block_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(g_ctx, st);
    if (ord.rc) return 1;
    if (layer->maps == nullptr && prefill_supported(layer->cfg) &&
        (int)T > g_ctx->decode_max_t) {
        layer->maps = prefill_maps_create(layer->cfg, layer->exp_gu,
                                          layer->exp_d, layer->sh_g,
                                          layer->sh_u, layer->sh_d,
                                          layer->e_end - layer->e_begin);
        if (!layer->maps) return fail("%s", prefill_last_error());
    }
    return block_dev_locked(layer, d_ln2, d_out, T, d_tr, st);
}

static int layer_dev(ApusCudaLayer *layer, const uint16_t *d_res, const uint16_t *d_ln_w,
                     uint16_t *d_res_out, size_t T, const ApusCudaMoeTrace *d_tr,
                     cudaStream_t st) {
    if (layer->maps == nullptr && prefill_supported(layer->cfg) &&
        (int)T > g_ctx->decode_max_t) {
        layer->maps = prefill_maps_create(layer->cfg, layer->exp_gu, layer->exp_d, layer->sh_g,
                                          layer->sh_u, layer->sh_d,
                                          layer->e_end - layer->e_begin);
        if (!layer->maps) return fail("%s", prefill_last_error());
    }
    Residual rz;
    rz.res = d_res;
    rz.ln_w = d_ln_w;
    rz.res_out = d_res_out;
    return block_dev_locked(layer, nullptr, nullptr, T, d_tr, st, &rz);
}

extern "C" int apus_cuda_moe_layer_dev(ApusCudaLayer *layer, const uint16_t *d_res,
                                       const uint16_t *d_ln_w, uint16_t *d_res_out, size_t T,
                                       const ApusCudaMoeTrace *d_tr, void *stream) {
    if (!layer || !d_res || !d_res_out || !T) return fail("moe_layer_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(g_ctx, st);
    if (ord.rc) return 1;
    return layer_dev(layer, d_res, d_ln_w, d_res_out, T, d_tr, st);
}

extern "C" int apus_cuda_moe_stack_dev(ApusCudaLayer *const *layers,
                                       const uint16_t *const *d_ln_w, size_t n_layers,
                                       uint16_t *d_res, size_t T, void *stream) {
    if (!layers || !n_layers || !d_res || !T) return fail("moe_stack_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(g_ctx, st);
    if (ord.rc) return 1;
    int launches = 0;
    for (size_t l = 0; l < n_layers; l++) {
        if (!layers[l]) return fail("moe_stack_dev: layer %zu is null", l);
        /* in place: a layer reads the stream's row (t, h) only in the thread
         * that then writes it, after everything else of the layer */
        if (layer_dev(layers[l], d_res, d_ln_w ? d_ln_w[l] : nullptr, d_res, T, nullptr, st))
            return 1;
        launches += g_ctx->last_block_launches;
    }
    g_ctx->last_block_launches = launches;
    return 0;
}

extern "C" int apus_cuda_stage_timing(int enable) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    g_ctx->stage_timing = enable != 0;
    g_ctx->n_ev = 0;
    return 0;
}
extern "C" int apus_cuda_last_stage_ms(float *ms, int cap) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!g_ctx || !ms) return -1;
    for (int i = 0; i < cap; i++) ms[i] = 0.0f;
    if (g_ctx->df_timeline_valid) {
        /* the one-kernel path: phase boundaries from the device's global
         * timer, each taken as the latest CTA to reach it */
        if (cudaDeviceSynchronize() != cudaSuccess) return -1;
        const int G = g_ctx->sm_count;
        std::vector<unsigned long long> tl((size_t)G * DF_MARKS);
        if (cudaMemcpy(tl.data(), g_ctx->d_df_timeline,
                       tl.size() * sizeof(unsigned long long),
                       cudaMemcpyDeviceToHost) != cudaSuccess)
            return -1;
        unsigned long long t0 = ~0ull, end[DF_MARKS] = {};
        for (int b = 0; b < G; b++) {
            if (tl[(size_t)b * DF_MARKS] < t0) t0 = tl[(size_t)b * DF_MARKS];
            for (int k = 1; k < DF_MARKS; k++)
                if (tl[(size_t)b * DF_MARKS + k] > end[k])
                    end[k] = tl[(size_t)b * DF_MARKS + k];
        }
        auto span = [&](int k0, int k1) {
            unsigned long long a0 = k0 == 0 ? t0 : end[k0];
            return end[k1] > a0 ? (float)((end[k1] - a0) * 1e-6) : 0.0f;
        };
        if (cap > APUS_CUDA_STAGE_ROUTER) ms[APUS_CUDA_STAGE_ROUTER] = span(0, 3);
        if (cap > APUS_CUDA_STAGE_GATE_UP) ms[APUS_CUDA_STAGE_GATE_UP] = span(3, 4);
        if (cap > APUS_CUDA_STAGE_DISPATCH) ms[APUS_CUDA_STAGE_DISPATCH] = span(4, 5);
        if (cap > APUS_CUDA_STAGE_DOWN) ms[APUS_CUDA_STAGE_DOWN] = span(5, 6);
        if (cap > APUS_CUDA_STAGE_FINALIZE) ms[APUS_CUDA_STAGE_FINALIZE] = span(6, 7);
        return DF_MARKS - 1;
    }
    if (g_ctx->n_ev < 2) return 0;
    if (cudaEventSynchronize(g_ctx->ev[g_ctx->n_ev - 1]) != cudaSuccess)
        return -1;
    for (int i = 1; i < g_ctx->n_ev; i++) {
        float t = 0.0f;
        cudaEventElapsedTime(&t, g_ctx->ev[i - 1], g_ctx->ev[i]);
        int sidx = g_ctx->ev_stage[i];
        if (sidx >= 0 && sidx < cap) ms[sidx] += t;
    }
    return g_ctx->n_ev - 1;
}

extern "C" int apus_cuda_fused_timeline(unsigned long long *out, int cap) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!g_ctx || !out || !g_ctx->df_timeline_valid) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    int n = g_ctx->sm_count * DF_MARKS;
    if (n > cap) n = cap;
    if (cudaMemcpy(out, g_ctx->d_df_timeline, (size_t)n * sizeof(unsigned long long),
                   cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    return n;
}

/* phase boundaries of the certified router's first CTA in its last launch:
 * out[0..3] = start, candidates known, chains done, end (ns, low 32 bits of the
 * global timer), out[4] = chains that CTA walked */
extern "C" int apus_cuda_router_timeline(unsigned int *out) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!g_ctx || !out) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    unsigned int v[16];
    if (cudaMemcpy(v, g_ctx->d_rc_stats, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -1;
    for (int i = 0; i < 5; i++) out[i] = v[2 + i];
    return 0;
}

extern "C" long apus_cuda_router_exact_chains(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!g_ctx) return -1;
    unsigned int n = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpy(&n, g_ctx->d_rc_stats, sizeof n, cudaMemcpyDeviceToHost) !=
        cudaSuccess)
        return -1;
    return (long)n;
}

extern "C" int apus_cuda_last_block_launches(void) {
    return g_ctx ? g_ctx->last_block_launches : 0;
}
extern "C" int apus_cuda_last_block_path(void) {
    return g_ctx ? g_ctx->last_block_path : -1;
}
extern "C" int apus_cuda_last_block_status(void) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (!g_ctx) return -1;
    int st = -1;
    if (cudaMemcpy(&st, g_ctx->d_status, 4, cudaMemcpyDeviceToHost) !=
        cudaSuccess)
        return -1;
    if (st) cudaMemset(g_ctx->d_status, 0, 4);
    return st;
}

extern "C" int apus_cuda_moe_block(const ApusCudaMoeCfg *cfg,
                                   const ApusCudaMoeW *w, const uint16_t *ln2,
                                   uint16_t *moe_out, size_t T,
                                   const ApusCudaMoeTrace *tr) {
    if (cfg_check(cfg)) return 1;
    if (!T) return 0;      /* no token: nothing is written, as in c/layer.h:570-651 */
    if (!w || !w->rtr_w || !w->sh_g || !w->sh_u || !w->sh_d || !w->sh_gate || !ln2 ||
        !moe_out)
        return fail("moe_block: null argument");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    ApusCudaLayer *L = nullptr;
    auto it = c->layers.find(w->rtr_w);
    if (it != c->layers.end()) {
        L = it->second;
        if (memcmp(&L->cfg, cfg, sizeof *cfg) != 0)
            return fail("moe_block: layer key reused with a different shape");
    } else {
        /* experts as host arrays, unless the layer was registered from the
         * weight container (apus_cuda_register_layer_slabs) */
        if (!w->exp_gu || !w->exp_d)
            return fail("moe_block: exp_gu / exp_d are NULL and the layer is not "
                        "registered (apus_cuda_register_layer_slabs)");
        if (apus_cuda_layer_create(cfg, w, 0, cfg->experts, &L)) return 1;
        c->layers.emplace(w->rtr_w, L);
    }
    const size_t H = cfg->hidden, TK = cfg->top_k;
    Ordered ord(c, c->stream);
    if (ord.rc) return 1;
    size_t need = 2 * T * H * 2 + T * TK * 6 + 3 * T * H * 2 + 8192;
    if (arena_reserve(c->io, need)) return 1;
    c->io.reset();
    uint16_t *dx = (uint16_t *)c->io.take(T * H * 2);
    uint16_t *dout = (uint16_t *)c->io.take(T * H * 2);
    ApusCudaMoeTrace dtr;
    memset(&dtr, 0, sizeof dtr);
    if (tr) {
        if (tr->rtr_idx) dtr.rtr_idx = (int32_t *)c->io.take(T * TK * 4);
        if (tr->rtr_w) dtr.rtr_w = (uint16_t *)c->io.take(T * TK * 2);
        if (tr->moe_routed) dtr.moe_routed = (uint16_t *)c->io.take(T * H * 2);
        if (tr->moe_shared) dtr.moe_shared = (uint16_t *)c->io.take(T * H * 2);
    }
    /* rows [r0, r0 + n) of the call: upload on s_up, block on the library's
     * stream, download on s_dn (all three the same stream for a small call) */
    auto download = [&](size_t r0, size_t n, cudaStream_t s_dn) -> int {
        CU_OK(cudaMemcpyAsync(moe_out + r0 * H, dout + r0 * H, n * H * 2,
                              cudaMemcpyDeviceToHost, s_dn));
        if (!tr) return 0;
        if (tr->rtr_idx)
            CU_OK(cudaMemcpyAsync(tr->rtr_idx + r0 * TK, dtr.rtr_idx + r0 * TK, n * TK * 4,
                                  cudaMemcpyDeviceToHost, s_dn));
        if (tr->rtr_w)
            CU_OK(cudaMemcpyAsync(tr->rtr_w + r0 * TK, dtr.rtr_w + r0 * TK, n * TK * 2,
                                  cudaMemcpyDeviceToHost, s_dn));
        if (tr->moe_routed)
            CU_OK(cudaMemcpyAsync(tr->moe_routed + r0 * H, dtr.moe_routed + r0 * H,
                                  n * H * 2, cudaMemcpyDeviceToHost, s_dn));
        if (tr->moe_shared)
            CU_OK(cudaMemcpyAsync(tr->moe_shared + r0 * H, dtr.moe_shared + r0 * H,
                                  n * H * 2, cudaMemcpyDeviceToHost, s_dn));
        return 0;
    };
    auto part_trace = [&](size_t r0) {
        ApusCudaMoeTrace t = dtr;
        if (t.rtr_idx) t.rtr_idx += r0 * TK;
        if (t.rtr_w) t.rtr_w += r0 * TK;
        if (t.moe_routed) t.moe_routed += r0 * H;
        if (t.moe_shared) t.moe_shared += r0 * H;
        return t;
    };
    const bool split = c->host_split_t > 0 && T >= (size_t)c->host_split_t;
    if (!split) {
        CU_OK(cudaMemcpyAsync(dx, ln2, T * H * 2, cudaMemcpyHostToDevice, c->stream));
        if (apus_cuda_moe_block_dev(L, dx, dout, T, tr ? &dtr : nullptr, c->stream))
            return 1;
        if (download(0, T, c->stream)) return 1;
    } else {
        /* A token's result does not depend on which other tokens share the call,
         * so two half calls give the same bits; the PCIe copies of one half run
         * beside the kernels of the other. */
        if (!c->s_in) {
            CU_OK(cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking));
            CU_OK(cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking));
            for (auto &e : c->ev_io) CU_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        const size_t r1 = T / 2, cut[3] = {0, r1, T};
        CU_OK(cudaEventRecord(c->ev_io[0], c->stream));       /* earlier work owns dx, dout */
        CU_OK(cudaStreamWaitEvent(c->s_in, c->ev_io[0], 0));
        CU_OK(cudaStreamWaitEvent(c->s_out, c->ev_io[0], 0));
        for (int k = 0; k < 2; k++) {
            CU_OK(cudaMemcpyAsync(dx + cut[k] * H, ln2 + cut[k] * H,
                                  (cut[k + 1] - cut[k]) * H * 2, cudaMemcpyHostToDevice,
                                  c->s_in));
            CU_OK(cudaEventRecord(c->ev_io[1 + k], c->s_in));
        }
        for (int k = 0; k < 2; k++) {
            const size_t r0 = cut[k], n = cut[k + 1] - cut[k];
            CU_OK(cudaStreamWaitEvent(c->stream, c->ev_io[1 + k], 0));
            ApusCudaMoeTrace tk = part_trace(r0);
            if (apus_cuda_moe_block_dev(L, dx + r0 * H, dout + r0 * H, n, tr ? &tk : nullptr,
                                        c->stream))
                return 1;
            CU_OK(cudaEventRecord(c->ev_io[3 + k], c->stream));
            CU_OK(cudaStreamWaitEvent(c->s_out, c->ev_io[3 + k], 0));
            if (download(r0, n, c->s_out)) return 1;
        }
        CU_OK(cudaStreamSynchronize(c->s_out));
    }
    int st = 0;
    CU_OK(cudaMemcpyAsync(&st, c->d_status, 4, cudaMemcpyDeviceToHost, c->stream));
    CU_OK(cudaStreamSynchronize(c->stream));
    if (tr && tr->moe_out) memcpy(tr->moe_out, moe_out, T * H * 2);
    if (st) {
        cudaMemset(c->d_status, 0, 4);
        return fail("moe_block: device status %d (a bounded wait gave up or "
                    "an index was out of range)", st);
    }
    return 0;
}


/* A layer whose routed experts never exist as host arrays (the engine's tiered
 * mode leaves exp_gu / exp_d NULL and resolves experts from its store,
 * c/model.h:499-503, c/cache.h:1498-1545): registered under the residency key
 * w->rtr_w with the experts read from the weight container, then served by
 * apus_cuda_moe_block like any other layer. */
extern "C" int apus_cuda_register_layer_slabs(const ApusCudaMoeCfg *cfg, const ApusCudaMoeW *w,
                                              const char *container_dir, int layer_index) {
    if (cfg_check(cfg)) return 1;
    if (!w || !w->rtr_w || !w->sh_g || !w->sh_u || !w->sh_d || !w->sh_gate || !container_dir)
        return fail("register_layer_slabs: null argument");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    if (c->layers.count(w->rtr_w)) return 0;           /* already resident */
    /* router, shared expert and gate from the host; expert tensors allocated only */
    ApusCudaMoeW w0 = *w;
    w0.exp_gu = nullptr;
    w0.exp_d = nullptr;
    ApusCudaLayer *L = nullptr;
    if (apus_cuda_layer_create(cfg, &w0, 0, cfg->experts, &L)) return 1;
    if (apus_cuda_layer_load_slabs(L, container_dir, layer_index)) {
        layer_free(L);
        return 1;
    }
    c->layers.emplace(w->rtr_w, L);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* expert parallelism                                                        */
/* ------------------------------------------------------------------------ */

static int ensure_maps(ApusCudaLayer *L) {
    if (L->maps || !prefill_supported(L->cfg)) return 0;
    L->maps = prefill_maps_create(L->cfg, L->exp_gu, L->exp_d, L->sh_g, L->sh_u,
                                  L->sh_d, L->e_end - L->e_begin);
    if (!L->maps) return fail("%s", prefill_last_error());
    return 0;
}

extern "C" int apus_cuda_ep_route_dev(ApusCudaLayer *L, const uint16_t *d_x,
                                      size_t T, int32_t *d_idx, uint16_t *d_w,
                                      uint16_t *d_sgl, void *stream) {
    if (!L || !d_x || !d_idx || !d_w || !d_sgl || !T)
        return fail("ep_route_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const size_t E = L->cfg.experts;
    if (arena_reserve(c->ws, T * E * 18 + 8192)) return 1;
    c->ws.reset();
    uint16_t *logits = (uint16_t *)c->ws.take(T * E * 2);
    RouterAux aux = {L->d_wnorm, L->wmin_gate, (float *)c->ws.take(T * E * 16),
                     T * E * 16};
    return launch_router(c, d_x, L->rtr_w, (int)T, (int)E, (int)L->cfg.hidden,
                         (int)L->cfg.top_k, L->wmin, d_idx, d_w, logits,
                         L->sh_gate, d_sgl, st, &aux);
}

/* gather kernel for the pack step: send_e[p] = idx[perm[p]] */
__global__ void ep_gather_ids_kernel(const int32_t *__restrict__ idx,
                                     const int32_t *__restrict__ perm, int A,
                                     int32_t *__restrict__ out) {
    pdl_enter();
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < A;
         p += gridDim.x * blockDim.x)
        out[p] = idx[perm[p]];
}

extern "C" int apus_cuda_ep_pack_dev(const uint16_t *d_x, const int32_t *d_idx,
                                     size_t T, size_t topk, size_t H, size_t E,
                                     size_t n_ranks, uint16_t *d_send_x,
                                     int32_t *d_send_e, int32_t *d_send_counts,
                                     int32_t *d_pos, void *stream) {
    const size_t A = T * topk;
    if (!d_x || !d_idx || !d_send_x || !d_send_e || !d_send_counts || !d_pos ||
        !A || !n_ranks || E % n_ranks || H % 8)
        return fail("ep_pack_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const size_t need = dispatch_scratch_bytes(A, n_ranks) + A * 4 +
                        (n_ranks + 1) * 4 + 4096;
    if (arena_reserve(c->ws, need)) return 1;
    c->ws.reset();
    DispatchOut o;
    memset(&o, 0, sizeof o);
    o.counts = d_send_counts;
    o.offsets = (int32_t *)c->ws.take((n_ranks + 1) * 4);
    o.perm = (int32_t *)c->ws.take(A * 4);
    o.pos = d_pos;
    int32_t *uh = (int32_t *)c->ws.take(dispatch_scratch_bytes(A, n_ranks));
    if (launch_dispatch(c, d_idx, (int)A, (int)n_ranks, o, uh, st,
                        DispatchKey{0, (int)(E / n_ranks)}))
        return 1;
    long total = (long)A * (long)(H / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > c->sm_count * 16) blocks = c->sm_count * 16;
    launch_k(gather_rows_kernel, dim3(blocks), dim3(256), 0, st, d_x, o.perm,
             (int)A, (int)H, (int)topk, d_send_x, (const int32_t *)nullptr);
    LAUNCHED();
    launch_k(ep_gather_ids_kernel, dim3((unsigned)((A + 255) / 256)), dim3(256),
             0, st, d_idx, o.perm, (int)A, d_send_e);
    LAUNCHED();
    return 0;
}

/* peer (expert parallelism, pull form): the rows are loaded from and the
 * outputs stored to other GPUs' memory; d_x and d_y are then unused. */
struct SharedWork {            /* the shared expert of the rank's own tokens, in the same */
    const uint16_t *x;         /* launches as the routed experts: x [T,H] -> y [T,H] */
    size_t T;
    uint16_t *y;
};
static int experts_core(ApusCudaLayer *L, const uint16_t *d_x, const int32_t *d_e, size_t R,
                        uint16_t *d_y, void *stream, const PeerRows *peer,
                        const SharedWork *sh = nullptr) {
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const size_t ne = L->e_end - L->e_begin;
    if (!ne) return fail("experts_dev: no routed experts resident");
    ApusCudaMoeCfg cx = L->cfg;       /* the shape dispatch and tiling see */
    cx.experts = ne;
    cx.top_k = 1;
    const bool prefill = ((int)R > c->decode_max_t || peer) && prefill_supported(L->cfg);
    if (peer && !prefill)
        return fail("experts over peer memory need the tensor-core path (hidden and "
                    "moe_inter multiples of 128, shared_inter == moe_inter)");
    if (prefill && ensure_maps(L)) return 1;
    BlockBufs b;
    block_layout(cx, R, nullptr, &b, prefill);
    if (arena_reserve(c->ws, b.total)) return 1;
    if (block_layout(cx, R, &c->ws, &b, prefill)) return 1;
    if (peer) {
        d_x = b.xg;          /* a valid local address for the unused token maps */
        d_y = b.eo;
    }
    if (sh && (!prefill || sh->T > R)) return fail("experts: shared work needs the GEMM path");
    const uint16_t *x_in = sh ? sh->x : d_x;
    const int T_in = sh ? (int)sh->T : (int)R;
    uint16_t *sy = sh ? sh->y : b.sy;
    if (prefill) {
        b.d.grp_expert = nullptr;
        b.d.grp_first = nullptr;
        b.d.grp_n = nullptr;
        b.d.n_groups = nullptr;
    }
    const size_t rows_expected = c->ep_rows_hint ? c->ep_rows_hint : R;
    c->ep_rows_hint = 0;
    const bool pair = prefill && pair_supported(L->cfg, c->sm_count, c->smem_optin) &&
                      rows_expected >= (size_t)g_pp_min_rows * ne;
    TilePlan plan;
    memset(&plan, 0, sizeof plan);
    if (prefill && !pair) plan = prefill_tile_plan(cx, T_in, sh != nullptr, (int)R, b.tiles);
    /* stage marks (apus_cuda_stage_timing): dispatch, gather, gate_up, down */
    c->n_ev = 0;
    stage_mark(c, -1, st);
    g_mark_stream = st;
    if (launch_dispatch(c, d_e, (int)R, (int)ne, b.d, b.unit_hist, st,
                        DispatchKey{(int)L->e_begin, 1, peer ? (int)ne : 0},
                        prefill && !pair ? &plan : nullptr))
        return 1;
    stage_mark(c, APUS_CUDA_STAGE_DISPATCH, st);
    if (pair) {
        const int before = c->last_block_launches;
        if (run_pair_experts(c->sm_count, c->smem_optin, L->maps, cx, 0, x_in, T_in, (int)R,
                             peer ? (int)L->cfg.top_k : 1, sh != nullptr, b.d, b.xg, b.act,
                             b.sa, d_y, sy, b.tiles, c->d_status, st, &c->last_block_launches,
                             mark_cb, peer))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
        return 0;
    }
    if (prefill) {
        const int before = c->last_block_launches;
        if (run_prefill_experts(c->sm_count, c->smem_optin, L->maps, cx, 0, x_in,
                                T_in, (int)R, peer ? (int)L->cfg.top_k : 1, sh != nullptr, b.d,
                                b.xg, b.act, b.sa, d_y, sy, b.tiles, c->d_status, st,
                                &c->last_block_launches, mark_cb,
                                plan.on ? &plan : nullptr, peer))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
        return 0;
    }
    return run_decode_experts(c, L, d_x, (int)R, 1, 0, b, false, d_y, st);
}

extern "C" int apus_cuda_experts_dev(ApusCudaLayer *L, const uint16_t *d_x,
                                     const int32_t *d_e, size_t R,
                                     uint16_t *d_y, void *stream) {
    if (!L || !d_x || !d_e || !d_y) return fail("experts_dev: bad args");
    if (!R) return 0;
    return experts_core(L, d_x, d_e, R, d_y, stream, nullptr);
}

extern "C" int apus_cuda_ep_finish_dev(ApusCudaLayer *L, const uint16_t *d_x,
                                       size_t T, const uint16_t *d_y_sorted,
                                       const int32_t *d_pos,
                                       const uint16_t *d_w,
                                       const uint16_t *d_sgl, uint16_t *d_out,
                                       const ApusCudaMoeTrace *d_tr,
                                       void *stream) {
    if (!L || !d_x || !d_y_sorted || !d_pos || !d_w || !d_sgl || !d_out || !T)
        return fail("ep_finish_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const ApusCudaMoeCfg &cfg = L->cfg;
    /* shared expert only: a dispatch result with no routed rows */
    ApusCudaMoeCfg cx = cfg;
    cx.top_k = 1;
    const bool prefill = (int)T > c->decode_max_t && prefill_supported(cfg);
    if (prefill && ensure_maps(L)) return 1;
    BlockBufs b;
    block_layout(cx, T, nullptr, &b, prefill);
    if (arena_reserve(c->ws, b.total)) return 1;
    if (block_layout(cx, T, &c->ws, &b, prefill)) return 1;
    CU_OK(cudaMemsetAsync(b.d.counts, 0, cfg.experts * 4, st));
    CU_OK(cudaMemsetAsync(b.d.offsets, 0, (cfg.experts + 1) * 4, st));
    CU_OK(cudaMemsetAsync(b.d.n_groups, 0, 4, st));
    if (prefill) {
        const int before = c->last_block_launches;
        if (run_prefill_experts(c->sm_count, c->smem_optin, L->maps, cfg,
                                (int)L->e_begin, d_x, (int)T, 0, 1, true, b.d,
                                b.xg, b.act, b.sa, b.eo, b.sy, b.tiles,
                                c->d_status, st, &c->last_block_launches,
                                nullptr))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
    } else {
        if (run_decode_experts(c, L, d_x, (int)T, 1, 0, b, true, b.eo, st))
            return 1;
    }
    return run_finalize(c, cfg, (int)T, d_y_sorted, d_pos, d_w, b.sy, d_sgl,
                        d_out, d_tr, st);
}

/* ---- expert parallelism through peer memory (ep_window.cuh) ------------- */
struct ApusCudaEpWindow {
    EpwLayout l;
    EpwPeers peers;
    bool opened[EPW_MAX_RANKS];      /* mapped with cudaIpcOpenMemHandle */
    int me;
    int topk, E;
    unsigned char *base;
    uint16_t *y;                     /* [n*cap][H] expert outputs by slot */
    int32_t *offsets, *perm, *counts;
    int32_t *uh;                     /* dispatch scratch */
    unsigned int *counter;           /* [2] finished-CTA counters */
    uint32_t *d_epoch;               /* step number for calls made with epoch 0 */
    unsigned long long *tbl;         /* [2][EPW_MAX_RANKS] addresses of every rank's xs, by */
    bool tbl_ready;
};

extern "C" int apus_cuda_ep_window_create(size_t max_tokens, size_t topk, size_t H,
                                          size_t E, size_t n_ranks, size_t rank,
                                          ApusCudaEpWindow **out) {
    if (!out || !max_tokens || !topk || !H || H % 8 || !n_ranks ||
        n_ranks > EPW_MAX_RANKS || rank >= n_ranks || !E || E % n_ranks)
        return fail("ep_window_create: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    ApusCudaEpWindow *w = new ApusCudaEpWindow();
    memset(w, 0, sizeof *w);
    const size_t cap = max_tokens * topk;
    w->l = epw_layout((int)n_ranks, (int)cap, (int)H, (int)max_tokens);
    w->me = (int)rank;
    w->topk = (int)topk;
    w->E = (int)E;
    const size_t A = cap;
    const size_t local = n_ranks * cap * H * 2 + (n_ranks + 1) * 4 + A * 4 +
                         n_ranks * 4 + 2 * EPW_MAX_RANKS * 8 +
                         dispatch_scratch_bytes(A, n_ranks) + 8192;
    unsigned char *loc = nullptr;
    if (cudaMalloc(&w->base, w->l.total) != cudaSuccess ||
        cudaMalloc(&loc, local) != cudaSuccess) {
        if (w->base) cudaFree(w->base);
        delete w;
        return fail("ep_window_create: out of device memory (%zu + %zu bytes)",
                    w->l.total, local);
    }
    cudaMemset(w->base, 0, w->l.total);
    cudaMemset(loc, 0, local);
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t o = 0;
    w->y = (uint16_t *)(loc + o);        o = up(o + n_ranks * cap * H * 2);
    w->offsets = (int32_t *)(loc + o);   o = up(o + (n_ranks + 1) * 4);
    w->perm = (int32_t *)(loc + o);      o = up(o + A * 4);
    w->counts = (int32_t *)(loc + o);    o = up(o + n_ranks * 4);
    w->counter = (unsigned int *)(loc + o); o = up(o + 8);
    w->d_epoch = (uint32_t *)(loc + o);  o = up(o + 4);
    w->tbl = (unsigned long long *)(loc + o); o = up(o + 2 * EPW_MAX_RANKS * 8);
    w->uh = (int32_t *)(loc + o);
    w->peers.base[rank] = w->base;
    CU_OK(cudaDeviceSynchronize());
    *out = w;
    return 0;
}

extern "C" void apus_cuda_ep_window_destroy(ApusCudaEpWindow *w) {
    if (!w) return;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    cudaDeviceSynchronize();
    for (int r = 0; r < w->l.n; r++)
        if (w->opened[r]) cudaIpcCloseMemHandle(w->peers.base[r]);
    if (w->y) cudaFree(w->y);           /* first address of the local allocation */
    if (w->base) cudaFree(w->base);
    delete w;
}

extern "C" size_t apus_cuda_ep_window_handle_bytes(void) {
    return sizeof(cudaIpcMemHandle_t);
}

extern "C" int apus_cuda_ep_window_handle(ApusCudaEpWindow *w, void *out) {
    if (!w || !out) return fail("ep_window_handle: bad args");
    cudaIpcMemHandle_t h;
    CU_OK(cudaIpcGetMemHandle(&h, w->base));
    memcpy(out, &h, sizeof h);
    return 0;
}

extern "C" int apus_cuda_ep_window_attach(ApusCudaEpWindow *w, size_t peer,
                                          const void *handle) {
    if (!w || !handle || peer >= (size_t)w->l.n || (int)peer == w->me)
        return fail("ep_window_attach: bad args");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    CU_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    w->peers.base[peer] = (unsigned char *)p;
    w->opened[peer] = true;
    w->tbl_ready = false;
    return 0;
}

extern "C" int apus_cuda_ep_window_attach_local(ApusCudaEpWindow *w, size_t peer,
                                                ApusCudaEpWindow *other) {
    if (!w || !other || peer >= (size_t)w->l.n || other->l.total != w->l.total)
        return fail("ep_window_attach_local: bad args");
    w->peers.base[peer] = other->base;
    w->tbl_ready = false;
    return 0;
}

static int epw_ready(ApusCudaEpWindow *w, const char *what) {
    if (!w) return fail("%s: no window", what);
    for (int r = 0; r < w->l.n; r++)
        if (!w->peers.base[r]) return fail("%s: peer %d not attached", what, r);
    return 0;
}

extern "C" int apus_cuda_ep_push_dev(ApusCudaEpWindow *w, const uint16_t *d_x,
                                     const int32_t *d_idx, size_t T, uint32_t epoch,
                                     int32_t *d_pos, void *stream) {
    if (epw_ready(w, "ep_push_dev")) return 1;
    const size_t A = T * w->topk;
    if (!d_x || !d_idx || !d_pos || !T || A > (size_t)w->l.cap)
        return fail("ep_push_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    DispatchOut o;
    memset(&o, 0, sizeof o);
    o.counts = w->counts;
    o.offsets = w->offsets;
    o.perm = w->perm;
    o.pos = d_pos;
    if (launch_dispatch(c, d_idx, (int)A, w->l.n, o, w->uh, st,
                        DispatchKey{0, w->E / w->l.n}))
        return 1;
    /* two CTAs per SM: every CTA ends with a system-scope fence and a turn at
     * one counter, so few CTAs with several rows each beat many small ones */
    long total = (long)A * (w->l.H / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > c->sm_count * 2) blocks = c->sm_count * 2;
    launch_k(epw_push_kernel, dim3(blocks), dim3(256), 0, st, d_x, d_idx,
             (const int32_t *)w->perm, (const int32_t *)w->offsets, (int)A, w->topk,
             w->l, w->peers, w->me, epoch, w->counter, w->d_epoch);
    LAUNCHED();
    return 0;
}

/* which: 0 = pushes of all sources have landed here; 1 = all returns have */
extern "C" int apus_cuda_ep_wait_dev(ApusCudaEpWindow *w, int which, uint32_t epoch,
                                     void *stream) {
    if (epw_ready(w, "ep_wait_dev")) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    Ordered ord(c, (cudaStream_t)stream);
    if (ord.rc) return 1;
    const uint32_t *flags =
        reinterpret_cast<const uint32_t *>(w->base + (which ? w->l.fbk : w->l.fin));
    launch_k(epw_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, flags, w->l.n,
             epoch, c->d_status, (const uint32_t *)w->d_epoch);
    LAUNCHED();
    return 0;
}

extern "C" int apus_cuda_ep_window_experts_dev(ApusCudaEpWindow *w, ApusCudaLayer *L,
                                               void *stream) {
    if (epw_ready(w, "ep_window_experts_dev")) return 1;
    {
        /* of the n * cap slots about cap hold a row (what one rank sends in all) */
        std::lock_guard<std::recursive_mutex> lk(g_mu);
        if (g_ctx) g_ctx->ep_rows_hint = (size_t)w->l.cap;
    }
    return apus_cuda_experts_dev(L, (const uint16_t *)(w->base + w->l.rx),
                                 (const int32_t *)(w->base + w->l.re),
                                 (size_t)w->l.n * w->l.cap, w->y, stream);
}

extern "C" int apus_cuda_ep_return_dev(ApusCudaEpWindow *w, uint32_t epoch,
                                       void *stream) {
    if (epw_ready(w, "ep_return_dev")) return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    Ordered ord(c, (cudaStream_t)stream);
    if (ord.rc) return 1;
    launch_k(epw_return_kernel, dim3(c->sm_count * 2), dim3(256), 0, (cudaStream_t)stream,
             (const uint16_t *)w->y, w->l, w->peers, w->me, epoch, w->counter + 1,
             (const uint32_t *)w->d_epoch);
    LAUNCHED();
    return 0;
}

/* ---- the pull form of the step (ep_window.cuh) ---- */
/* Touches the window and d_x only (no shared workspace), so it is not ordered
 * against the library's other calls: it may run beside the router on a second
 * stream.  The caller orders it after its previous step's combine and before
 * apus_cuda_ep_publish_dev(..., d_x = NULL, ...). */
extern "C" int apus_cuda_ep_publish_rows_dev(ApusCudaEpWindow *w, const uint16_t *d_x,
                                             size_t T, void *stream) {
    if (epw_ready(w, "ep_publish_rows_dev")) return 1;
    if (!d_x || !T || T > (size_t)w->l.tokens) return fail("ep_publish_rows_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    long total = (long)T * (w->l.H / 8) * w->l.n;
    int blocks = (int)((total + 255) / 256);
    if (blocks > c->sm_count * 2) blocks = c->sm_count * 2;
    epw_publish_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(d_x, (int)T, w->l,
                                                                      w->peers, w->me);
    LAUNCHED();
    return 0;
}

extern "C" int apus_cuda_ep_publish_dev(ApusCudaEpWindow *w, const uint16_t *d_x,
                                        const int32_t *d_idx, size_t T, uint32_t epoch,
                                        void *stream) {
    if (epw_ready(w, "ep_publish_dev")) return 1;
    if (!d_idx || !T || T > (size_t)w->l.tokens)
        return fail("ep_publish_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    long total = d_x ? (long)T * (w->l.H / 8) * w->l.n : (long)w->l.cap * w->l.n;
    int blocks = (int)((total + 255) / 256);
    if (blocks > c->sm_count * 2) blocks = c->sm_count * 2;
    /* ids only: a few hundred KB; every CTA ends with a system-scope fence and a
     * turn at one counter, so a handful of CTAs is quicker than hundreds */
    if (!d_x && blocks > 4 * w->l.n) blocks = 4 * w->l.n;
    launch_k(epw_publish_kernel, dim3(blocks), dim3(256), 0, st, d_x, d_idx, (int)T, w->topk,
             w->l, w->peers, w->me, epoch, w->counter, w->d_epoch);
    LAUNCHED();
    return 0;
}

extern "C" int apus_cuda_ep_pull_experts_dev(ApusCudaEpWindow *w, ApusCudaLayer *L,
                                             uint32_t epoch, const uint16_t *d_x, size_t T,
                                             uint16_t *d_sy, void *stream) {
    if (epw_ready(w, "ep_pull_experts_dev")) return 1;
    if (!L || (size_t)w->l.H != L->cfg.hidden || (size_t)w->topk != L->cfg.top_k ||
        (d_x && (!d_sy || !T || T > (size_t)w->l.tokens)))
        return fail("ep_pull_experts_dev: bad args");
    cudaStream_t st = (cudaStream_t)stream;
    {
        std::lock_guard<std::recursive_mutex> lk(g_mu);
        if (ctx_init()) return 1;
        Ctx *c = g_ctx;
        Ordered ord(c, st);
        if (ord.rc) return 1;
        if (!w->tbl_ready) {
            if (c->cur_capturing)
                return fail("ep_pull_experts_dev: run one step before capturing a graph");
            unsigned long long h[2 * EPW_MAX_RANKS] = {0};
            for (int r = 0; r < w->l.n; r++) {
                h[r] = (unsigned long long)(uintptr_t)(w->base + w->l.xs +
                                                       (size_t)r * w->l.tokens * w->l.H * 2);
                h[EPW_MAX_RANKS + r] = (unsigned long long)(uintptr_t)(w->peers.base[r] + w->l.by);
            }
            CU_OK(cudaMemcpyAsync(w->tbl, h, sizeof h, cudaMemcpyHostToDevice, st));
            CU_OK(cudaStreamSynchronize(st));
            w->tbl_ready = true;
        }
        /* of the n * cap slots about cap hold a resident expert; the dispatch
         * skips the others */
        c->ep_rows_hint = (size_t)w->l.cap;
    }
    PeerRows pr = {w->tbl, w->tbl + EPW_MAX_RANKS, w->l.cap};
    SharedWork sh = {d_x, T, d_sy};
    if (experts_core(L, nullptr, (const int32_t *)(w->base + w->l.ids),
                     (size_t)w->l.n * w->l.cap, nullptr, stream, &pr,
                     d_x ? &sh : nullptr))
        return 1;
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    /* a plain launch: it starts only when the GEMMs before it have ended */
    epw_signal_kernel<<<1, 32, 0, st>>>(w->l, w->peers, w->me, epoch,
                                        (const uint32_t *)w->d_epoch);
    LAUNCHED();
    return 0;
}

/* The shared expert of the rank's own tokens: d_sy [T,H] BF16 (c/layer.h:350-353). */
extern "C" int apus_cuda_ep_shared_dev(ApusCudaLayer *L, const uint16_t *d_x, size_t T,
                                       uint16_t *d_sy, void *stream) {
    if (!L || !d_x || !d_sy || !T) return fail("ep_shared_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const ApusCudaMoeCfg &cfg = L->cfg;
    ApusCudaMoeCfg cx = cfg;
    cx.top_k = 1;
    const bool prefill = (int)T > c->decode_max_t && prefill_supported(cfg);
    if (prefill && ensure_maps(L)) return 1;
    BlockBufs b;
    block_layout(cx, T, nullptr, &b, prefill);
    if (arena_reserve(c->ws, b.total)) return 1;
    if (block_layout(cx, T, &c->ws, &b, prefill)) return 1;
    CU_OK(cudaMemsetAsync(b.d.counts, 0, cfg.experts * 4, st));
    CU_OK(cudaMemsetAsync(b.d.offsets, 0, (cfg.experts + 1) * 4, st));
    CU_OK(cudaMemsetAsync(b.d.n_groups, 0, 4, st));
    if (prefill) {
        const int before = c->last_block_launches;
        if (run_prefill_experts(c->sm_count, c->smem_optin, L->maps, cfg,
                                (int)L->e_begin, d_x, (int)T, 0, 1, true, b.d, b.xg,
                                b.act, b.sa, b.eo, d_sy, b.tiles, c->d_status, st,
                                &c->last_block_launches, nullptr))
            return fail("%s", prefill_last_error());
        c->launches += (uint64_t)(c->last_block_launches - before);
        return 0;
    }
    if (run_decode_experts(c, L, d_x, (int)T, 1, 0, b, true, b.eo, st)) return 1;
    CU_OK(cudaMemcpyAsync(d_sy, b.sy, T * cfg.hidden * 2, cudaMemcpyDeviceToDevice, st));
    return 0;
}

/* out = rnd(rnd(sum_j w_j * y_j) + rnd(sy * rnd(sigmoid(sgl)))) with the returned
 * rows of the window as y (c/layer.h:349,356-360). */
extern "C" int apus_cuda_ep_combine_dev(ApusCudaEpWindow *w, ApusCudaLayer *L, size_t T,
                                        const int32_t *d_pos, const uint16_t *d_w,
                                        const uint16_t *d_sy, const uint16_t *d_sgl,
                                        uint16_t *d_out, void *stream) {
    if (epw_ready(w, "ep_combine_dev")) return 1;
    if (!L || !T || !d_w || !d_sy || !d_sgl || !d_out ||
        T * L->cfg.top_k > (size_t)w->l.cap)
        return fail("ep_combine_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    Ordered ord(c, (cudaStream_t)stream);
    if (ord.rc) return 1;
    return run_finalize(c, L->cfg, (int)T, (const uint16_t *)(w->base + w->l.by), d_pos,
                        d_w, d_sy, d_sgl, d_out, nullptr, (cudaStream_t)stream);
}

/* ------------------------------------------------------------------------ */
/* stages on device pointers                                                 */
/* ------------------------------------------------------------------------ */

extern "C" int apus_cuda_route_dev(ApusCudaLayer *L, const uint16_t *d_x,
                                   size_t T, int32_t *d_idx, uint16_t *d_w,
                                   void *stream) {
    if (!L || !d_x || !d_idx || !T) return fail("route_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    const size_t E = L->cfg.experts;
    if (arena_reserve(c->ws, T * E * 18 + 8192)) return 1;
    c->ws.reset();
    uint16_t *logits = (uint16_t *)c->ws.take(T * E * 2);
    RouterAux aux = {L->d_wnorm, 0.0f, (float *)c->ws.take(T * E * 16), T * E * 16};
    return launch_router(c, d_x, L->rtr_w, (int)T, (int)E, (int)L->cfg.hidden,
                         (int)L->cfg.top_k, L->wmin, d_idx, d_w, logits, nullptr,
                         nullptr, st, &aux);
}

extern "C" int apus_cuda_dispatch_dev(const int32_t *d_idx, size_t T,
                                      size_t topk, size_t E, int32_t *d_counts,
                                      int32_t *d_offsets, int32_t *d_perm,
                                      void *stream) {
    size_t A = T * topk;
    if (!d_idx || !A || !E) return fail("dispatch_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    c->last_block_launches = 0;
    cudaStream_t st = (cudaStream_t)stream;
    Ordered ord(c, st);
    if (ord.rc) return 1;
    size_t need = dispatch_scratch_bytes(A, E) + 1024;
    if (arena_reserve(c->io, need)) return 1;
    c->io.reset();
    DispatchOut o;
    memset(&o, 0, sizeof o);
    o.counts = d_counts;
    o.offsets = d_offsets;
    o.perm = d_perm;
    int32_t *uh = (int32_t *)c->io.take(dispatch_scratch_bytes(A, E));
    return launch_dispatch(c, d_idx, (int)A, (int)E, o, uh, st);
}

extern "C" int apus_cuda_rmsnorm_dev(const uint16_t *d_x, const uint16_t *d_w,
                                     uint16_t *d_y, size_t T, size_t N,
                                     void *stream) {
    if (!d_x || !d_y || !T || !N) return fail("rmsnorm_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    size_t smem = 4 * N * sizeof(float);
    if (smem > 48 * 1024) {
        if (smem > (size_t)g_ctx->smem_optin) return fail("rmsnorm: N too large");
        CU_OK(cudaFuncSetAttribute(rmsnorm_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    }
    rmsnorm_kernel<<<(unsigned)((T + 3) / 4), 128, smem, st>>>(d_x, d_w, d_y,
                                                               (int)T, (int)N);
    LAUNCHED();
    return 0;
}

template <int M>
static int launch_gemv_stream(Ctx *c, const uint16_t *w, const uint16_t *x, uint16_t *y,
                              size_t O, size_t K, cudaStream_t st) {
    const size_t smem = (size_t)M * K * sizeof(float);
    if (smem > (size_t)c->smem_optin) return fail("gemv_dev: M * K too large");
    if (smem > 48 * 1024)
        CU_OK(cudaFuncSetAttribute(gemv_stream_kernel<M>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    size_t blocks = (O + 15) / 16;                 /* 8 warps x 2 rows per CTA pass */
    const size_t cap = (size_t)c->sm_count * (smem > 64 * 1024 ? 1 : (smem > 24 * 1024 ? 3 : 6));
    if (blocks > cap) blocks = cap;
    gemv_stream_kernel<M><<<(unsigned)blocks, 256, smem, st>>>(w, x, y, (long)O, (int)K);
    return 0;
}

extern "C" int apus_cuda_bf16_gemv_dev(const uint16_t *d_w, const uint16_t *d_x,
                                       uint16_t *d_y, size_t M, size_t O, size_t K,
                                       void *stream) {
    if (!d_w || !d_x || !d_y || !M || !O || !K) return fail("gemv_dev: bad args");
    if (M > 8 || K % 256 || (((uintptr_t)d_w) & 15))
        return fail("gemv_dev: needs M <= 8, K a multiple of 256, 16-byte aligned weights");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    Ctx *c = g_ctx;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = 1;
    switch (M) {
        case 1: rc = launch_gemv_stream<1>(c, d_w, d_x, d_y, O, K, st); break;
        case 2: rc = launch_gemv_stream<2>(c, d_w, d_x, d_y, O, K, st); break;
        case 3: rc = launch_gemv_stream<3>(c, d_w, d_x, d_y, O, K, st); break;
        case 4: rc = launch_gemv_stream<4>(c, d_w, d_x, d_y, O, K, st); break;
        case 5: rc = launch_gemv_stream<5>(c, d_w, d_x, d_y, O, K, st); break;
        case 6: rc = launch_gemv_stream<6>(c, d_w, d_x, d_y, O, K, st); break;
        case 7: rc = launch_gemv_stream<7>(c, d_w, d_x, d_y, O, K, st); break;
        default: rc = launch_gemv_stream<8>(c, d_w, d_x, d_y, O, K, st); break;
    }
    if (rc) return 1;
    LAUNCHED();
    return 0;
}

extern "C" int apus_cuda_resadd_dev(const uint16_t *d_a, const uint16_t *d_b,
                                    uint16_t *d_out, size_t n, void *stream) {
    if (!d_a || !d_b || !d_out || !n) return fail("resadd_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)g_ctx->sm_count * 16) blocks = g_ctx->sm_count * 16;
    resadd_kernel<<<(unsigned)blocks, 256, 0, st>>>(d_a, d_b, d_out, n);
    LAUNCHED();
    return 0;
}

/* ------------------------------------------------------------------------ */
/* synthetic tensors                                                         */
/* ------------------------------------------------------------------------ */

extern "C" void apus_synth_fill_host(uint16_t *dst, size_t n, uint64_t seed,
                                     uint32_t layer, uint32_t tensor_id,
                                     uint64_t first, double sigma) {
    const uint64_t key = apus_synth_key(seed, layer, tensor_id);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++)
        dst[i] = apus_synth_bf16(key, first + (uint64_t)i, sigma);
}

extern "C" int apus_synth_fill_dev(uint16_t *d_dst, size_t n, uint64_t seed,
                                   uint32_t layer, uint32_t tensor_id,
                                   uint64_t first, double sigma, void *stream) {
    if (!d_dst || !n) return fail("synth_fill_dev: bad args");
    std::lock_guard<std::recursive_mutex> lk(g_mu);
    if (ctx_init()) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t key = apus_synth_key(seed, layer, tensor_id);
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)g_ctx->sm_count * 32) blocks = g_ctx->sm_count * 32;
    synth_fill_kernel<<<(unsigned)blocks, 256, 0, st>>>(d_dst, n, key, first,
                                                        sigma);
    LAUNCHED();
    return 0;
}

/* ------------------------------------------------------------------------ */
/* dispatch without any allocation                                           */
/* ------------------------------------------------------------------------ */

/* Scratch for apus_cuda_dispatch_dev_static: the per-unit histograms of the
 * three-pass dispatch plus one status word.  It is part of the library image,
 * so every GPU that loads the library carries this 1 MiB until the process
 * exits, whether or not the entry point is ever called. */
#define APUS_STATIC_SCRATCH_INTS 262144u
static __device__ __align__(256) int32_t
    g_dispatch_static_scratch[APUS_STATIC_SCRATCH_INTS + 64];

/* Device address of the array above, per device.  The array's name is only a
 * host-side handle here; the address a kernel can use comes from
 * cudaGetSymbolAddress, asked once per device with that device current. */
static int32_t *g_dispatch_static_addr[64] = {};
static std::mutex g_dispatch_static_mu;

extern "C" int apus_cuda_dispatch_dev_static(const int32_t *d_idx, size_t T,
                                             size_t topk, size_t E,
                                             int32_t *d_counts,
                                             int32_t *d_offsets,
                                             int32_t *d_perm, void *stream) {
    const size_t A = T * topk;
    /* g_mu guards the error text (and nothing else here: this entry point
     * touches none of the context's state) */
    std::lock_guard<std::recursive_mutex> lk_err(g_mu);
    if (!d_idx || !d_counts || !d_offsets || !d_perm || !A || !E)
        return fail("dispatch_dev_static: bad args");
    if (E > 1024) return fail("dispatch_dev_static: unsupported E=%zu", E);
    if (A > 0x7fffffffu) return fail("dispatch_dev_static: T*topk too large");
    const size_t units = (A + DISPATCH_UNIT - 1) / DISPATCH_UNIT;
    if (A > (size_t)DISPATCH_SMALL_MAX && units * E > APUS_STATIC_SCRATCH_INTS)
        return fail("dispatch_dev_static: ceil(T*topk/256)*E = %zu exceeds the "
                    "built-in scratch of %u entries; use apus_cuda_dispatch_dev",
                    units * E, APUS_STATIC_SCRATCH_INTS);
    int dev = -1;
    CU_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64)
        return fail("dispatch_dev_static: device ordinal %d not supported", dev);
    int32_t *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_dispatch_static_mu);
        if (!g_dispatch_static_addr[dev]) {
            void *p = nullptr;
            CU_OK(cudaGetSymbolAddress(&p, g_dispatch_static_scratch));
            g_dispatch_static_addr[dev] = static_cast<int32_t *>(p);
        }
        scratch = g_dispatch_static_addr[dev];
    }
    cudaStream_t st = (cudaStream_t)stream;
    int *status = reinterpret_cast<int *>(scratch + APUS_STATIC_SCRATCH_INTS);
    CU_OK(cudaMemsetAsync(status, 0, sizeof(int), st));
    DispatchOut o;
    memset(&o, 0, sizeof o);
    o.counts = d_counts;
    o.offsets = d_offsets;
    o.perm = d_perm;
    const int Ai = (int)A, Ei = (int)E;
    if (A <= (size_t)DISPATCH_SMALL_MAX) {
        CU_OK(cudaFuncSetAttribute(dispatch_small_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   32 * 1024 * (int)sizeof(int)));
        TilePlan none;
        memset(&none, 0, sizeof none);
        launch_k(dispatch_small_kernel, dim3(1), dim3(1024), (size_t)32 * E * sizeof(int), st, d_idx, Ai, Ei, DispatchKey{0, 1}, o, status, none);
    } else {
        const int blocks = (int)((units + DISPATCH_WARPS - 1) / DISPATCH_WARPS);
        const size_t smem = (size_t)DISPATCH_WARPS * E * sizeof(int);
        launch_k(dispatch_hist_kernel, dim3(blocks), dim3(DISPATCH_WARPS * 32), smem, st, d_idx, Ai, Ei, DispatchKey{0, 1}, scratch, status);
        launch_k(dispatch_scan_kernel, dim3(1), dim3(1024), 0, st, scratch, (int)units, Ei, o);
        launch_k(dispatch_permute_kernel, dim3(blocks), dim3(DISPATCH_WARPS * 32), smem, st, d_idx, Ai, Ei, DispatchKey{0, 1}, scratch, o);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail("dispatch_dev_static: launch failed: %s",
                    cudaGetErrorString(e));
    return 0;
}
