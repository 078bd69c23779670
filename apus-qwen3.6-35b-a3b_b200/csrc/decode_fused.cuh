/*
 * decode_fused.cuh — the whole MoE block for one to four tokens in ONE
 * cooperative kernel (c/layer.h:333-370 end to end): router chains, softmax /
 * top-k, the routed and shared experts' gate/up rows with SwiGLU, one grid-wide
 * barrier, the down rows, and the weighted combine + shared gate + add.
 *
 * At this size the block is a 57 MB weight stream that should take ~9 us, and
 * every kernel boundary, dependent global round trip and idle SM shows.  So:
 *
 *  - one launch; 148 persistent CTAs (one per SM), 8 warps each;
 *  - the first ceil((E+1)/8) CTAs walk the exact router chains (eight rows per
 *    CTA, one lane per (row, token), rows pulled in by bulk copies) while all
 *    the others already stream and reduce their share of the shared expert's
 *    gate/up rows, which do not depend on routing;
 *  - the logits meet in global memory behind a release/acquire counter; every
 *    CTA then runs the (cheap, bit-exact) softmax/top-k itself instead of
 *    waiting for a second broadcast;
 *  - expert rows arrive through per-warp rings of cp.async.bulk copies (no
 *    multicast); each CTA owns a contiguous slice of the flattened (expert,
 *    row) space;
 *  - the down phase gives each CTA a slice of the output columns across ALL
 *    selected experts, so the combine is local and no second barrier is
 *    needed; its first weight copies are issued before the barrier wait.
 *
 * CTAs wait on one another (router counter, barrier), which is only legal
 * because the launch is cooperative (all CTAs co-resident).  Every wait is
 * bounded: on a timeout the CTA records a status code and drains to the exit.
 * The counters are reset by the last CTA to leave, so the kernel can be
 * replayed from a CUDA graph.
 */
#pragma once
#include <climits>

#include "common.cuh"
#include "decode_gemv.cuh"
#include "router.cuh"

namespace apus {

constexpr int DF_THREADS = 256;
constexpr int DF_WARPS = 8;
constexpr int DF_MAX_T = 4;
constexpr int DF_MAX_A = 32;            /* T * top_k */
constexpr int DF_STAGE_BYTES = 8192;    /* a gate+up row pair, or 8 down rows */

struct FusedArgs {
    int T, H, I, Is, E, TK, stages;
    float wmin, wmin_gate;              /* smallest nonzero |w|: router, shared-gate row */
    const uint16_t *x;                  /* [T, H] block input; or, with res set, unused */
    /* the two steps either side of the block folded in (c/layer.h:386,388):
     * res [T,H] is the residual stream, the block input is rmsnorm(res, 1 + ln_w)
     * (c/attn.h:175-186, every CTA computes it for itself: 4 KB per token and
     * one sequential chain per token, no exchange), and res_out = rnd(res + moe_out) */
    const uint16_t *res, *ln_w;
    uint16_t *res_out;
    const uint16_t *rtr_w, *exp_gu, *exp_d, *sh_g, *sh_u, *sh_d, *sh_gate;
    /* global scratch owned by the backend */
    float *logits_ws;                   /* [DF_MAX_T][E] */
    uint16_t *sgl_ws;                   /* [DF_MAX_T] */
    uint16_t *act_ws;                   /* [DF_MAX_A][I] */
    uint16_t *sa_ws;                    /* [DF_MAX_T][Is] */
    unsigned int *sync;                 /* [0] router done, [1] barrier, [2] exits */
    /* outputs */
    uint16_t *out;                      /* [T, H] */
    int32_t *idx_out;                   /* [T, TK] (optional) */
    uint16_t *w_out;                    /* [T, TK] (optional) */
    uint16_t *tr_routed, *tr_shared, *tr_out;
    int *status;
    /* optional phase timeline: [grid][DF_MARKS] global-timer nanoseconds */
    unsigned long long *timeline;
};
constexpr int DF_MARKS = 8;
__device__ __forceinline__ void df_mark(const FusedArgs &a, int k) {
    if (a.timeline && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        a.timeline[(size_t)blockIdx.x * DF_MARKS + k] = t;
    }
}

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
/* thread 0 of a CTA: wait until *p >= target; false on timeout */
__device__ __forceinline__ bool spin_until(const unsigned int *p,
                                           unsigned int target) {
    for (uint32_t i = 0; i < (1u << 21); i++) {
        if (ld_acquire(p) >= target) return true;
        if (i > 32) __nanosleep(40);
    }
    return false;
}

/* butterfly-reduce N independent values at once (the shuffles of different
 * values overlap; a value-at-a-time reduction would serialise 5 shuffle
 * latencies per value) */
template <int N>
__device__ __forceinline__ void warp_sum_n(float (&v)[N]) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < N; i++) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
}

/* eight weight rows (contiguous, K each) against NT selected activation rows */
template <int NT>
__device__ __forceinline__ void df_down8(const uint16_t *ws, const uint16_t *src,
                                         const int *rows, int K, int lane,
                                         float (&acc)[8 * 4]) {
    float a[8 * NT];
#pragma unroll
    for (int i = 0; i < 8 * NT; i++) a[i] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        float xf[NT][8];
#pragma unroll
        for (int n = 0; n < NT; n++)
            unpack8(*reinterpret_cast<const uint4 *>(src + (size_t)rows[n] * K + k),
                    xf[n]);
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float wf[8];
            unpack8(*reinterpret_cast<const uint4 *>(ws + (size_t)r * K + k), wf);
#pragma unroll
            for (int n = 0; n < NT; n++)
#pragma unroll
                for (int j = 0; j < 8; j++)
                    a[r * NT + n] = fmaf(wf[j], xf[n][j], a[r * NT + n]);
        }
    }
    warp_sum_n<8 * NT>(a);
#pragma unroll
    for (int r = 0; r < 8; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) acc[r * 4 + n] = a[r * NT + n];
}

/* gate and up rows against NT selected token rows; reduced */
template <int NT>
__device__ __forceinline__ void df_gate_up(const uint16_t *gs, const uint16_t *us,
                                           const uint16_t *xs, int stride,
                                           const int *rows, int K, int lane,
                                           float (&ag)[4], float (&au)[4]) {
    float a[2 * NT];
#pragma unroll
    for (int i = 0; i < 2 * NT; i++) a[i] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        float gf[8], uf[8];
        unpack8(*reinterpret_cast<const uint4 *>(gs + k), gf);
        unpack8(*reinterpret_cast<const uint4 *>(us + k), uf);
#pragma unroll
        for (int n = 0; n < NT; n++) {
            float xf[8];
            unpack8(*reinterpret_cast<const uint4 *>(xs + (size_t)rows[n] * stride + k),
                    xf);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                a[n] = fmaf(gf[j], xf[j], a[n]);
                a[NT + n] = fmaf(uf[j], xf[j], a[NT + n]);
            }
        }
    }
    warp_sum_n<2 * NT>(a);
#pragma unroll
    for (int n = 0; n < NT; n++) {
        ag[n] = a[n];
        au[n] = a[NT + n];
    }
}
__device__ __forceinline__ void df_gate_up_n(int nt, const uint16_t *gs,
                                             const uint16_t *us, const uint16_t *xs,
                                             int stride, const int *rows, int K,
                                             int lane, float (&ag)[4],
                                             float (&au)[4]) {
    switch (nt) {
        case 1: df_gate_up<1>(gs, us, xs, stride, rows, K, lane, ag, au); break;
        case 2: df_gate_up<2>(gs, us, xs, stride, rows, K, lane, ag, au); break;
        case 3: df_gate_up<3>(gs, us, xs, stride, rows, K, lane, ag, au); break;
        default: df_gate_up<4>(gs, us, xs, stride, rows, K, lane, ag, au); break;
    }
}
__device__ __forceinline__ void df_down8_n(int nt, const uint16_t *ws,
                                           const uint16_t *src, const int *rows,
                                           int K, int lane, float (&acc)[32]) {
    switch (nt) {
        case 1: df_down8<1>(ws, src, rows, K, lane, acc); break;
        case 2: df_down8<2>(ws, src, rows, K, lane, acc); break;
        case 3: df_down8<3>(ws, src, rows, K, lane, acc); break;
        default: df_down8<4>(ws, src, rows, K, lane, acc); break;
    }
}


/* xs[t][:] = rmsnorm(res[t][:], 1 + ln_w) for t < T, bit for bit the engine's
 * (c/attn.h:175-186): the sum of squares is one ascending fp32 chain (lane 0 of
 * warp t walks it over the row staged in shared memory, operands converted on
 * the fly: the dependent add is the critical path), then y = rnd((x*rs)*(1+w)).
 * All threads call it; ends with a CTA barrier. */
__device__ __forceinline__ void df_rmsnorm_to_smem(const FusedArgs &a, uint16_t *xs) {
    const int T = a.T, H = a.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int c = tid; c < T * (H / 8); c += DF_THREADS)
        reinterpret_cast<uint4 *>(xs)[c] = ldg16(a.res + (size_t)c * 8);
    __syncthreads();
    if (warp < T) {
        uint16_t *row = xs + (size_t)warp * H;
        /* the gains are asked for before the chain starts, so that their trip
         * from L2 hides behind it: 16 bytes a lane and round, H / 256 rounds */
        const int nj = H / 256;
        const bool vec = H % 256 == 0 && nj <= 8;
        uint4 lw[8];
#pragma unroll
        for (int j = 0; j < 8; j++)
            lw[j] = (vec && a.ln_w && j < nj) ? ldg16(a.ln_w + (size_t)(lane + 32 * j) * 8)
                                              : make_uint4(0, 0, 0, 0);
        float ss = 0.0f;
        if (lane == 0) {
            const uint4 *r4 = reinterpret_cast<const uint4 *>(row);
            /* four rows of eight ahead: the shared-memory loads and the squares
             * stay off the chain of dependent adds */
#pragma unroll 4
            for (int i = 0; i < H / 8; i++) {
                const uint4 v = r4[i];
                const float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                                    bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
                float q[8];
#pragma unroll
                for (int j = 0; j < 8; j++) q[j] = __fmul_rn(f[j], f[j]);
#pragma unroll
                for (int j = 0; j < 8; j++) ss = __fadd_rn(ss, q[j]);
            }
        }
        ss = __shfl_sync(0xffffffffu, ss, 0);
        const float rs =
            __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)H), 1e-6f)));
        if (vec) {
            uint4 *r4 = reinterpret_cast<uint4 *>(row);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (j < nj) {
                    const uint4 v = r4[lane + 32 * j];
                    const uint32_t xw[4] = {v.x, v.y, v.z, v.w};
                    const uint32_t gw[4] = {lw[j].x, lw[j].y, lw[j].z, lw[j].w};
                    uint32_t o[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float g0 = __fadd_rn(1.0f, bf16lo(gw[q])),
                                    g1 = __fadd_rn(1.0f, bf16hi(gw[q]));
                        const float y0 = __fmul_rn(__fmul_rn(bf16lo(xw[q]), rs), g0),
                                    y1 = __fmul_rn(__fmul_rn(bf16hi(xw[q]), rs), g1);
                        o[q] = (uint32_t)bf16_bits(y0) | ((uint32_t)bf16_bits(y1) << 16);
                    }
                    r4[lane + 32 * j] = make_uint4(o[0], o[1], o[2], o[3]);
                }
            }
        } else {
            for (int i = lane; i < H; i += 32) {
                const float g = __fadd_rn(1.0f, a.ln_w ? bf16_f32(__ldg(a.ln_w + i)) : 0.0f);
                row[i] = bf16_bits(__fmul_rn(__fmul_rn(bf16_f32(row[i]), rs), g));
            }
        }
    }
    __syncthreads();
}

/* A warp's private ring of bulk copies.  issue() is called by lane 0 only. */
struct WarpRing {
    unsigned char *base;     /* stages * DF_STAGE_BYTES */
    uint64_t *bars;
    int stages;
    int issued, consumed;
    __device__ __forceinline__ void issue(const void *src0, uint32_t b0,
                                          const void *src1, uint32_t b1) {
        const int s = issued % stages;
        unsigned char *dst = base + (size_t)s * DF_STAGE_BYTES;
        mbar_expect_tx(&bars[s], b0 + b1);
        bulk_g2s(dst, src0, b0, &bars[s]);
        if (b1) bulk_g2s(dst + b0, src1, b1, &bars[s]);
    }
    __device__ __forceinline__ bool wait() {
        const int s = consumed % stages;
        return mbar_wait(&bars[s], (uint32_t)(consumed / stages) & 1u);
    }
    __device__ __forceinline__ const unsigned char *cur() const {
        return base + (size_t)(consumed % stages) * DF_STAGE_BYTES;
    }
};

/*
 * Dynamic shared memory:
 *   ring   [DF_WARPS][stages][8 KB]      (router CTAs first use it for their
 *                                          eight rows and the fp32 tokens)
 *   xs     uint16 [T][H]                  tokens (phase A/B); then
 *          uint16 [A][I] + [T][Is]        activations (phase C)   (union)
 *   ps     float  [T][E]                  logits -> probabilities
 *   ytab   uint16 [A + T][16]             down outputs of this CTA's columns
 *   small tables and barriers
 */
__global__ void __launch_bounds__(DF_THREADS, 1)
decode_fused_kernel(FusedArgs a) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char df_smem[];
    const int T = a.T, H = a.H, I = a.I, Is = a.Is, E = a.E, TK = a.TK;
    const int A = T * TK;
    const int G = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    unsigned char *ring_all = df_smem;
    const size_t ring_bytes = (size_t)DF_WARPS * a.stages * DF_STAGE_BYTES;
    const size_t un_bytes_x = (size_t)T * H * 2;
    const size_t un_bytes_a = ((size_t)A * I + (size_t)T * Is) * 2;
    const size_t un_bytes = un_bytes_x > un_bytes_a ? un_bytes_x : un_bytes_a;
    uint16_t *xs = reinterpret_cast<uint16_t *>(df_smem + ring_bytes);
    float *ps = reinterpret_cast<float *>(df_smem + ring_bytes + ((un_bytes + 127) & ~(size_t)127));
    uint16_t *ytab = reinterpret_cast<uint16_t *>(ps + (size_t)T * E);
    uint64_t *bars = reinterpret_cast<uint64_t *>(
        (reinterpret_cast<uintptr_t>(ytab + (size_t)(DF_MAX_A + DF_MAX_T) * 16) + 7) & ~(uintptr_t)7);
    uint64_t *rbar = bars + DF_WARPS * 3;          /* router rows barrier */
    __shared__ int s_idx[DF_MAX_A];
    __shared__ uint16_t s_w[DF_MAX_A];
    __shared__ uint16_t s_sgl[DF_MAX_T];
    __shared__ int s_uexp[DF_MAX_A];               /* unique experts */
    __shared__ unsigned int s_umask[DF_MAX_A];     /* assignments of each */
    __shared__ int s_U;
    __shared__ int s_dead;
    __shared__ unsigned int s_xmin;

    if (tid == 0) {
        for (int i = 0; i < DF_WARPS * 3; i++) mbar_init(&bars[i], 1);
        mbar_init(rbar, 1);
        mbar_fence_init();
        s_dead = 0;
        s_xmin = 0x7f800000u;
    }
    __syncthreads();

    WarpRing ring;
    ring.base = ring_all + (size_t)warp * a.stages * DF_STAGE_BYTES;
    ring.bars = bars + warp * 3;
    ring.stages = a.stages;
    ring.issued = 0;
    ring.consumed = 0;

    df_mark(a, 0);                          /* start */
    const int nR = (E + 1 + 7) / 8;        /* router CTAs */
    const bool is_router = (int)blockIdx.x < nR;
    const uint32_t rowb = (uint32_t)H * 2u;

    /* ---------------- router chains (first nR CTAs) ---------------- */
    if (is_router) {
        const int r0 = blockIdx.x * 8;
        const int nrows = min(8, E + 1 - r0);
        const int pitch = H * 2 + 16;
        unsigned char *rows_s = ring_all;
        float *xf = reinterpret_cast<float *>(ring_all + 8 * pitch);
        const int xpitch = H + 8;        /* floats: tokens on different banks */
        if (tid == 0) {
            mbar_expect_tx(rbar, (uint32_t)nrows * rowb);
            for (int r = 0; r < nrows; r++) {
                const uint16_t *src = (r0 + r == E) ? a.sh_gate
                                                    : a.rtr_w + (size_t)(r0 + r) * H;
                bulk_g2s(rows_s + (size_t)r * pitch, src, rowb, rbar);
            }
        }
        unsigned int xmin = 0x7f800000u;
        /* with the norm folded in, the block input is computed here (every CTA
         * does, the router CTAs first of all: their chains start from it) */
        if (a.res) df_rmsnorm_to_smem(a, xs);
        for (int c = tid; c < T * (H / 8); c += DF_THREADS) {
            const uint4 v = a.res ? reinterpret_cast<const uint4 *>(xs)[c]
                                  : ldg16(a.x + (size_t)c * 8);
            const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
            const int tt = c / (H / 8), cc = c - tt * (H / 8);
            float4 *d = reinterpret_cast<float4 *>(xf + (size_t)tt * xpitch + cc * 8);
            d[0] = make_float4(bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y));
            d[1] = make_float4(bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w));
#pragma unroll
            for (int q = 0; q < 4; q++) {
                unsigned int lo = (wds[q] << 16) & 0x7fffffffu;
                unsigned int hi = wds[q] & 0x7fff0000u;
                if (lo != 0 && lo < xmin) xmin = lo;
                if (hi != 0 && hi < xmin) xmin = hi;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, o));
        if (lane == 0) atomicMin(&s_xmin, xmin);
        __syncthreads();
        /* the fused form is exact while the smallest product is a normal
         * number; the shared-gate row has its own smallest weight */
        const double xmn = (double)__uint_as_float(s_xmin);
        const bool use_fma = (a.wmin > 0.0f) && ((double)a.wmin * xmn >= 7.52316384526264e-37);
        const bool use_fma_gate =
            (a.wmin_gate > 0.0f) && ((double)a.wmin_gate * xmn >= 7.52316384526264e-37);
        const bool arrived = mbar_wait(rbar, 0);      /* every warp waits */
        if (!arrived) {
            set_status(a.status, ST_MBAR_TIMEOUT);
            s_dead = 1;
        }
        if (warp == 0) {
            const int r = lane / T, t = lane - r * T;
            if (arrived && r < nrows) {
                const uint16_t *wrow =
                    reinterpret_cast<const uint16_t *>(rows_s + (size_t)r * pitch);
                const bool fma_row = (r0 + r != E) ? use_fma : use_fma_gate;
                const float acc =
                    fma_row ? small_chain<true>(wrow, xf + (size_t)t * xpitch, H)
                            : small_chain<false>(wrow, xf + (size_t)t * xpitch, H);
                const uint16_t code = bf16_bits(acc);
                if (r0 + r == E)
                    a.sgl_ws[t] = code;
                else
                    a.logits_ws[(size_t)t * E + r0 + r] = bf16_f32(code);
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence();
                red_release_add(&a.sync[0], 1u);
            }
        }
        fence_proxy_async();  /* generic writes above, bulk copies next */
        __syncthreads();      /* the ring region is free again */
    }

    df_mark(a, 1);                          /* router chains done (router CTAs) */
    /* ---------------- phase A: tokens to shared; shared gate/up ---------------- */
    if (a.res) {
        if (!is_router) df_rmsnorm_to_smem(a, xs);    /* router CTAs hold it already */
    } else {
        for (int c = tid; c < T * (H / 8); c += DF_THREADS)
            reinterpret_cast<uint4 *>(xs)[c] = ldg16(a.x + (size_t)c * 8);
    }
    __syncthreads();
    {
        /* The shared expert's rows go to the CTAs that have no router chains to
         * walk (they would otherwise idle until the logits arrive); a router CTA
         * that also took a share reached the selection 2-3 us after everyone
         * else and held up the grid barrier by as much. */
        const bool spare = G > nR;
        const int Gs = spare ? G - nR : G, bs = spare ? (int)blockIdx.x - nR : (int)blockIdx.x;
        const int lo = bs < 0 ? 0 : (int)((long)Is * bs / Gs);
        const int hi = bs < 0 ? 0 : (int)((long)Is * (bs + 1) / Gs);
        const int n_my = (lo + warp < hi) ? (hi - lo - warp + DF_WARPS - 1) / DF_WARPS : 0;
        if (lane == 0)
            for (; ring.issued < n_my && ring.issued < a.stages; ring.issued++) {
                const int row = lo + warp + ring.issued * DF_WARPS;
                ring.issue(a.sh_g + (size_t)row * H, rowb, a.sh_u + (size_t)row * H, rowb);
            }
        ring.issued = min(n_my, a.stages);
        const int rows[4] = {0, 1, 2, 3};
        for (int j = 0; j < n_my; j++) {
            const bool ok = !s_dead && ring.wait();
            if (!ok && !s_dead) {
                set_status(a.status, ST_MBAR_TIMEOUT);
                s_dead = 1;
            }
            const int row = lo + warp + j * DF_WARPS;
            if (ok) {
                const uint16_t *gs = reinterpret_cast<const uint16_t *>(ring.cur());
                float ag[4] = {0, 0, 0, 0}, au[4] = {0, 0, 0, 0};
                df_gate_up_n(T, gs, gs + H, xs, H, rows, H, lane, ag, au);
                if (lane < T) {
                    float g = 0.f, u = 0.f;
#pragma unroll
                    for (int n = 0; n < 4; n++)
                        if (lane == n) { g = ag[n]; u = au[n]; }
                    a.sa_ws[(size_t)lane * Is + row] =
                        silu_mul_bits(bf16_round(g), bf16_round(u));
                }
            }
            __syncwarp();
            ring.consumed++;
            if (!s_dead && ring.issued < n_my) {
                if (lane == 0) {
                    const int r2 = lo + warp + ring.issued * DF_WARPS;
                    ring.issue(a.sh_g + (size_t)r2 * H, rowb, a.sh_u + (size_t)r2 * H, rowb);
                }
                ring.issued++;
            }
        }
    }

    df_mark(a, 2);                          /* shared gate/up done */
    /* ---------------- routing result ---------------- */
    if (tid == 0 && !s_dead) {
        if (!spin_until(&a.sync[0], (unsigned)nR)) {
            set_status(a.status, ST_SCHED_TIMEOUT);
            s_dead = 1;
        }
    }
    __syncthreads();
    if (!s_dead) {
        for (int i = tid; i < T * E; i += DF_THREADS) ps[i] = __ldcg(&a.logits_ws[i]);
        if (tid < T) s_sgl[tid] = __ldcg(&a.sgl_ws[tid]);
    }
    __syncthreads();
    __shared__ int s_scratch[32];
    if (T == 1 && E <= DF_THREADS && TK <= 16) {
        /* one token: the whole CTA shares the softmax / selection */
        if (!s_dead)               /* uniform: s_dead is read after a barrier */
            router_softmax_topk_cta256(ps, E, TK, s_scratch, s_idx, s_w);
    } else if (!s_dead && warp < T) {
        router_softmax_topk(ps + (size_t)warp * E, E, TK, lane, s_idx + warp * TK,
                            s_w + warp * TK);
    }
    __syncthreads();
    if (blockIdx.x == 0 && tid < A) {
        if (a.idx_out) a.idx_out[tid] = s_idx[tid];
        if (a.w_out) a.w_out[tid] = s_w[tid];
    }
    /* unique experts and who uses them (A <= 32: one warp) */
    if (warp == 0) {
        const int e = lane < A ? s_idx[lane] : -1 - lane;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const bool leader = lane < A && (__ffs(peers) - 1) == lane;
        const unsigned leaders = __ballot_sync(0xffffffffu, leader);
        if (leader) {
            const int u = __popc(leaders & ((1u << lane) - 1u));
            s_uexp[u] = e;
            s_umask[u] = peers;
        }
        if (lane == 0) s_U = __popc(leaders);
    }
    __syncthreads();
    const int U = s_dead ? 0 : s_U;

    df_mark(a, 3);                          /* logits seen, softmax/top-k done */
    /* ---------------- phase B: routed gate/up ---------------- */
    {
        const long N = (long)U * I;
        const long lo = N * blockIdx.x / G, hi = N * (blockIdx.x + 1) / G;
        const long first = lo + warp;
        const int n_my = first < hi ? (int)((hi - first + DF_WARPS - 1) / DF_WARPS) : 0;
        ring.issued = ring.consumed;            /* ring is drained */
        const int base_c = ring.consumed;
        auto item_src = [&](int j, const uint16_t *&g, const uint16_t *&u) {
            const long it = first + (long)j * DF_WARPS;
            const int uu = (int)(it / I), row = (int)(it - (long)uu * I);
            const uint16_t *b = a.exp_gu + (size_t)s_uexp[uu] * 2 * I * H;
            g = b + (size_t)row * H;
            u = b + (size_t)(I + row) * H;
        };
        int issued_j = 0;
        if (lane == 0)
            for (; issued_j < n_my && issued_j < a.stages; issued_j++) {
                const uint16_t *g, *u;
                item_src(issued_j, g, u);
                ring.issue(g, rowb, u, rowb);
                ring.issued++;
            }
        issued_j = min(n_my, a.stages);
        ring.issued = base_c + issued_j;
        for (int j = 0; j < n_my; j++) {
            const bool ok = !s_dead && ring.wait();
            if (!ok && !s_dead) {
                set_status(a.status, ST_MBAR_TIMEOUT);
                s_dead = 1;
            }
            if (ok) {
                const long it = first + (long)j * DF_WARPS;
                const int uu = (int)(it / I), row = (int)(it - (long)uu * I);
                unsigned m = s_umask[uu];
                int rows[4] = {0, 0, 0, 0}, asg[4] = {0, 0, 0, 0}, nt = 0;
                while (m && nt < 4) {
                    const int aidx = __ffs(m) - 1;
                    m &= m - 1;
                    asg[nt] = aidx;
                    rows[nt] = aidx / TK;
                    nt++;
                }
                const uint16_t *gs = reinterpret_cast<const uint16_t *>(ring.cur());
                float ag[4] = {0, 0, 0, 0}, au[4] = {0, 0, 0, 0};
                df_gate_up_n(nt, gs, gs + H, xs, H, rows, H, lane, ag, au);
                if (lane < nt) {
                    float g = 0.f, u = 0.f;
                    int an = 0;
#pragma unroll
                    for (int n = 0; n < 4; n++)
                        if (lane == n) { g = ag[n]; u = au[n]; an = asg[n]; }
                    a.act_ws[(size_t)an * I + row] =
                        silu_act_bits(bf16_round(g), bf16_round(u));
                }
            }
            __syncwarp();
            ring.consumed++;
            if (!s_dead && issued_j < n_my) {
                if (lane == 0) {
                    const uint16_t *g, *u;
                    item_src(issued_j, g, u);
                    ring.issue(g, rowb, u, rowb);
                }
                issued_j++;
                ring.issued++;
            }
        }
    }

    df_mark(a, 4);                          /* routed gate/up done */
    /* ---------------- phase C set-up: first down copies, then the barrier ------- */
    const int HB = H / 8;
    const int b_lo = (int)((long)HB * blockIdx.x / G);
    const int b_hi = (int)((long)HB * (blockIdx.x + 1) / G);
    const int nb = b_hi - b_lo;                    /* 8-row blocks of this CTA (<= 2) */
    const int n_items = (U + 1) * nb;              /* expert-major, block-minor */
    const int n_my_c = warp < n_items ? (n_items - warp + DF_WARPS - 1) / DF_WARPS : 0;
    auto down_src = [&](int j, const uint16_t *&src, uint32_t &bytes) {
        const int it = warp + j * DF_WARPS;
        const int uu = it / nb, b = b_lo + (it - uu * nb);
        if (uu == U) {
            src = a.sh_d + (size_t)b * 8 * Is;
            bytes = (uint32_t)(8 * Is * 2);
        } else {
            src = a.exp_d + ((size_t)s_uexp[uu] * H + (size_t)b * 8) * I;
            bytes = (uint32_t)(8 * I * 2);
        }
    };
    int issued_c = 0;
    {
        const int base_c = ring.consumed;
        if (lane == 0 && !s_dead)
            for (; issued_c < n_my_c && issued_c < a.stages; issued_c++) {
                const uint16_t *src;
                uint32_t bytes;
                down_src(issued_c, src, bytes);
                ring.issued = base_c + issued_c;
                ring.issue(src, bytes, nullptr, 0);
            }
        issued_c = s_dead ? 0 : min(n_my_c, a.stages);
        ring.issued = base_c + issued_c;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        red_release_add(&a.sync[1], 1u);
        if (!s_dead && !spin_until(&a.sync[1], (unsigned)G)) {
            set_status(a.status, ST_SCHED_TIMEOUT);
            s_dead = 1;
        }
    }
    __syncthreads();

    df_mark(a, 5);                          /* barrier passed */
    /* activations of every assignment, and the shared activations */
    uint16_t *as = xs;
    uint16_t *sas = xs + (size_t)A * I;
    if (!s_dead) {
        for (int c = tid; c < A * (I / 8); c += DF_THREADS)
            reinterpret_cast<uint4 *>(as)[c] =
                __ldcg(reinterpret_cast<const uint4 *>(a.act_ws) + c);
        for (int c = tid; c < T * (Is / 8); c += DF_THREADS)
            reinterpret_cast<uint4 *>(sas)[c] =
                __ldcg(reinterpret_cast<const uint4 *>(a.sa_ws) + c);
    }
    __syncthreads();

    /* ---------------- phase C: down rows of this CTA's columns ---------------- */
    for (int j = 0; j < n_my_c; j++) {
        const bool ok = !s_dead && j < issued_c && ring.wait();
        if (!ok && !s_dead) {
            set_status(a.status, ST_MBAR_TIMEOUT);
            s_dead = 1;
        }
        if (ok) {
            const int it = warp + j * DF_WARPS;
            const int uu = it / nb, bl = it - uu * nb;
            const uint16_t *ws = reinterpret_cast<const uint16_t *>(ring.cur());
            int rows[4] = {0, 1, 2, 3}, nt, K;
            const uint16_t *src;
            int slot0;                          /* ytab row of rows[0] ... */
            int slots[4] = {0, 0, 0, 0};
            if (uu == U) {
                nt = T; K = Is; src = sas;
                for (int n = 0; n < 4; n++) slots[n] = DF_MAX_A + n;
            } else {
                unsigned m = s_umask[uu];
                nt = 0; K = I; src = as;
                while (m && nt < 4) {
                    const int aidx = __ffs(m) - 1;
                    m &= m - 1;
                    rows[nt] = aidx;
                    slots[nt] = aidx;
                    nt++;
                }
            }
            (void)slot0;
            float acc[32];
            df_down8_n(nt, ws, src, rows, K, lane, acc);
            if (lane < nt) {
                int sl = 0;
#pragma unroll
                for (int n = 0; n < 4; n++)
                    if (lane == n) sl = slots[n];
                uint32_t pk[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float v0 = 0.f, v1 = 0.f;
#pragma unroll
                    for (int n = 0; n < 4; n++)
                        if (lane == n) {
                            v0 = acc[(2 * q) * 4 + n];
                            v1 = acc[(2 * q + 1) * 4 + n];
                        }
                    pk[q] = pack_bf16(v0, v1);
                }
                *reinterpret_cast<uint4 *>(ytab + sl * 16 + bl * 8) =
                    make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
        __syncwarp();
        ring.consumed++;
        if (!s_dead && issued_c < n_my_c) {
            if (lane == 0) {
                const uint16_t *src;
                uint32_t bytes;
                down_src(issued_c, src, bytes);
                ring.issue(src, bytes, nullptr, 0);
            }
            issued_c++;
            ring.issued++;
        }
    }
    __syncthreads();

    df_mark(a, 6);                          /* down rows done */
    /* ---------------- combine (c/layer.h:350,356-361), this CTA's columns ------- */
    if (!s_dead && tid < T * nb * 8) {
        const int t = tid / (nb * 8), hl = tid - t * (nb * 8);
        float acc = 0.0f;
        for (int s = 0; s < TK; s++)
            acc = __fadd_rn(acc, __fmul_rn(bf16_f32(s_w[t * TK + s]),
                                           bf16_f32(ytab[(t * TK + s) * 16 + hl])));
        const float routed = bf16_round(acc);
        const float sgat = bf16_round(sigmoid_f32(bf16_f32(s_sgl[t])));
        const float shared =
            bf16_round(__fmul_rn(bf16_f32(ytab[(DF_MAX_A + t) * 16 + hl]), sgat));
        const uint16_t o = bf16_bits(__fadd_rn(routed, shared));
        const size_t at = (size_t)t * H + (size_t)b_lo * 8 + hl;
        if (a.out) a.out[at] = o;
        if (a.res_out)                          /* c/layer.h:230-234,388 */
            a.res_out[at] = bf16_bits(__fadd_rn(bf16_f32(__ldg(a.res + at)), bf16_f32(o)));
        if (a.tr_out) a.tr_out[at] = o;
        if (a.tr_routed) a.tr_routed[at] = bf16_bits(routed);
        if (a.tr_shared) a.tr_shared[at] = bf16_bits(shared);
    }

    /* last CTA out resets the counters for the next launch */
    __syncthreads();
    df_mark(a, 7);                          /* combine done */
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(&a.sync[2], 1u);
        if (old == (unsigned)G - 1) {
            a.sync[0] = 0;
            a.sync[1] = 0;
            __threadfence();
            a.sync[2] = 0;
        }
    }
}

inline size_t decode_fused_smem(int T, int H, int I, int Is, int E, int TK,
                                int stages) {
    const size_t A = (size_t)T * TK;
    size_t ring = (size_t)DF_WARPS * stages * DF_STAGE_BYTES;
    size_t ux = (size_t)T * H * 2, ua = (A * I + (size_t)T * Is) * 2;
    size_t un = ((ux > ua ? ux : ua) + 127) & ~(size_t)127;
    size_t ps = (size_t)T * E * 4;
    size_t yt = (size_t)(DF_MAX_A + DF_MAX_T) * 16 * 2;
    return ring + un + ps + yt + (DF_WARPS * 3 + 1) * 8 + 64;
}

}  // namespace apus
