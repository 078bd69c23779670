/*
 * router_certify.cuh — exact expert selection at a fraction of the exact
 * router's cost (c/moe.h:321-371 decides with BF16-rounded logits whose every
 * bit depends on a 2048-step sequential fp32 chain per expert, c/moe.h:289-291).
 *
 * Only the top_k experts of a token matter, and an expert far below the
 * top_k-th cannot become one because of rounding.  So:
 *
 *   1. fast logits a[t][e] for all experts come from the tensor cores (any
 *      summation order, prefill_gemm.cuh MODE 2);
 *   2. this kernel bounds how far the fast and the exact value of a pair can
 *      be apart:  |a - z| <= B(t,e) = cbound * ||x_t||_2 * ||w_e||_2
 *      (both are fp32 summations of the same exactly representable products;
 *      a summation of n terms in any order errs by at most about n*u times the
 *      sum of their magnitudes, which Cauchy-Schwarz bounds by the norms;
 *      cbound leaves the tensor cores eight times the worst case of the
 *      sequential chain);
 *   3. with a8 the top_k-th largest fast logit, every expert with
 *          a + B(t,e)  >=  a8 - Bmax(t) - spacing
 *      is a CANDIDATE (spacing = one BF16 step at that magnitude, so that two
 *      values further apart than it cannot round to the same code).  Any
 *      other expert's exact rounded logit is strictly below those of top_k
 *      experts, whatever the rounding did: it cannot be selected;
 *   4. candidates (about top_k + 2 of 256 at the real dimensions) and the
 *      shared-gate row get their exact chain, one lane each; everything else
 *      keeps its rounded fast logit, which only enters the softmax
 *      denominator (and cancels in the renormalised weights);
 *   5. the kernel checks |a - z| <= B on every pair it evaluates exactly and
 *      records ST_BOUND_VIOLATED if the assumption ever fails.
 *
 * The engine's softmax / top-k (router_softmax_topk, one warp per token) then
 * runs in the same kernel on the merged logits: ids are bit-exact by
 * construction, weights see exact logits for every selected expert.
 */
#pragma once
#include <climits>

#include "common.cuh"
#include "decode_gemv.cuh"
#include "router.cuh"

namespace apus {

constexpr int RC_TT = 8;            /* tokens per CTA (6 with deeper prefetch measured the same) */
constexpr int RC_THREADS = 256;      /* one warp per token in the first phase */
constexpr int RC_XPAD = 4;          /* floats between token rows: rows on
                                     * different bank groups */
constexpr int RC_CW = 4;            /* warps that walk chains: 128 pairs in one round (8 tokens
                                     * give 86 on average; a second round doubles the latency) */
constexpr int RC_BLK = 32;          /* weights per staged row block */
constexpr int RC_AHEAD = 2;         /* row blocks requested ahead of the one in use (4 ahead
                                     * measured the same: the chain is bound by its
                                     * dependent adds and shared-memory reads, ~12 cycles a
                                     * step, not by the copies) */
constexpr int RC_NBUF = RC_AHEAD + 1;
constexpr int RC_WPITCH = RC_BLK * 2 + 16;   /* bytes per staged row block */
constexpr int ST_BOUND_VIOLATED = 5;
constexpr int RC_MAX_SLABS = 4;     /* K slices of the fast-logit GEMM */

struct CertifyArgs {
    const float *approx;            /* [nslab][T, E]: the fast logits are the sum */
    int nslab;
    const uint16_t *x, *w;          /* [T, K], [E, K] */
    const uint16_t *extra_row;      /* [K] shared-gate row (optional) */
    const float *wnorm;             /* [E + 1]: ||w_e||_2 rounded up; [E] = their max */
    int T, E, K, topk;
    float wmin, wmin_extra;         /* smallest nonzero |w| (0 = unknown) */
    float cbound;                   /* see above */
    uint16_t *logits;               /* [T, E] merged BF16 logit codes out (optional) */
    int32_t *idx_out;               /* [T, topk] selection */
    uint16_t *w_out;                /* [T, topk] renormalised weights (optional) */
    uint16_t *extra_out;            /* [T] */
    int *status;
    unsigned int *stats;            /* [0] += exact chains run (optional) */
};

/* order-preserving integer key of a float (larger float -> larger int) */
__device__ __forceinline__ int rc_float_key(float f) {
    const int b = __float_as_int(f);
    return b >= 0 ? b : (b ^ 0x7fffffff);
}

/* Operands of RC_BLK steps of one exact chain: BF16 weights and fp32 tokens
 * from shared memory.  The chain is bound by instruction issue and by the
 * latency of the dependent add, so the tokens are kept converted (one shift or
 * mask per weight is all that remains beside the add) and the operands of the
 * next block are fetched while the current block's adds run. */
struct RcOperands {
    uint4 w[RC_BLK / 8];
    float4 x[RC_BLK / 4];
};
__device__ __forceinline__ void rc_fetch(RcOperands &o, const unsigned char *__restrict__ w,
                                         const float *__restrict__ x) {
#pragma unroll
    for (int c = 0; c < RC_BLK / 8; c++) {
        o.w[c] = *reinterpret_cast<const uint4 *>(w + c * 16);
        o.x[2 * c] = *reinterpret_cast<const float4 *>(x + c * 8);
        o.x[2 * c + 1] = *reinterpret_cast<const float4 *>(x + c * 8 + 4);
    }
}
template <bool FMA>
__device__ __forceinline__ float rc_steps(const RcOperands &o, float acc) {
#pragma unroll
    for (int c = 0; c < RC_BLK / 8; c++) {
        float wf[8];
        unpack8(o.w[c], wf);
        const float xf[8] = {o.x[2 * c].x,     o.x[2 * c].y,     o.x[2 * c].z,
                             o.x[2 * c].w,     o.x[2 * c + 1].x, o.x[2 * c + 1].y,
                             o.x[2 * c + 1].z, o.x[2 * c + 1].w};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (FMA)
                acc = __fmaf_rn(wf[j], xf[j], acc);
            else
                acc = __fadd_rn(acc, __fmul_rn(wf[j], xf[j]));
        }
    }
    return acc;
}
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)),
                 "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

/* One chain per lane over the warp's 32 staged rows (see the kernel's note).
 * rows[32]: the lanes' weight rows; wb: this warp's RC_NBUF buffers; x: this
 * lane's token in fp32.  Integer work issues at half the rate of the adds, so
 * the loop keeps running pointers instead of computing addresses. */
template <bool FMA>
__device__ __forceinline__ float rc_walk(const uint16_t *const *rows, unsigned char *wb,
                                         const float *__restrict__ xr, int K, int lane) {
    constexpr int LPR = RC_BLK / 8;            /* lanes per row in a copy instruction */
    constexpr int RPI = 32 / LPR;              /* rows per copy instruction */
    constexpr int NCP = 32 / RPI;              /* copy instructions per block */
    constexpr size_t BUF = (size_t)32 * RC_WPITCH;
    const int nblk = K / RC_BLK;
    const uint16_t *src[NCP];
#pragma unroll
    for (int i = 0; i < NCP; i++) src[i] = rows[RPI * i + lane / LPR] + (lane % LPR) * 8;
    unsigned char *const dst0 = wb + (size_t)(lane / LPR) * RC_WPITCH + (lane % LPR) * 16;
    unsigned char *const wend = wb + RC_NBUF * BUF;
    unsigned char *dst = dst0;                 /* where the next block goes */
    auto issue = [&]() {
#pragma unroll
        for (int i = 0; i < NCP; i++) {
            cp_async16(dst + (size_t)i * RPI * RC_WPITCH, src[i]);
            src[i] += RC_BLK;
        }
        dst += BUF;
        if (dst >= wend) dst -= RC_NBUF * BUF;
    };
    for (int b = 0; b < RC_AHEAD; b++) {
        if (b < nblk) issue();
        cp_async_commit();
    }
    const unsigned char *wl = wb + (size_t)lane * RC_WPITCH;   /* the block in use */
    const unsigned char *const wlend = wl + RC_NBUF * BUF;
    float z = 0.0f;
#pragma unroll 1
    for (int b = 0; b < nblk; b++) {
        cp_async_wait<RC_AHEAD - 1>();     /* block b has landed (my copies) */
        __syncwarp();                      /* ... and everyone else's; block b - 1 is
                                            * read out everywhere, so its buffer can
                                            * take block b + AHEAD */
        if (b + RC_AHEAD < nblk) issue();
        cp_async_commit();
        RcOperands o;
        rc_fetch(o, wl, xr);
        z = rc_steps<FMA>(o, z);
        wl += BUF;
        if (wl >= wlend) wl -= RC_NBUF * BUF;
        xr += RC_BLK;
    }
    return z;
}

/*
 * grid = ceil(T / RC_TT), block = RC_THREADS.  K % 256 == 0, E % 32 == 0,
 * E <= 1024.  Dynamic shared memory:
 *   xs    float  [RC_TT][K + RC_XPAD]   tokens
 *   af    float  [RC_TT][E]             fast logits
 *   pairs uint16 [RC_TT * (E + 1)]      (token << 11 | row); 16-bit so that TWO
 *                                        CTAs fit the SM's shared memory (one
 *                                        CTA per SM left the chain warps' idle
 *                                        phases uncovered: 7 waves of 22 us)
 *   wn    float  [E + 1]                row norms
 *   wbuf  [RC_CW][RC_NBUF][32][80 B]    staged weight blocks of the chain warps
 *
 * The chains: a warp takes 32 pairs, one per lane.  A lane reading its own
 * weight row 16 bytes at a time would cost the load unit one tag look-up per
 * lane and instruction; instead the warp copies each 32-weight block of its 32
 * rows into shared memory cooperatively (four lanes per row, cp.async, three
 * blocks in flight) and every lane then reads its row from there.
 */
__global__ void __launch_bounds__(RC_THREADS, 2)
router_certify_kernel(CertifyArgs a) {
    /* the next kernel may be scheduled; this kernel's own wait for the fast-logit
     * GEMM comes after the tokens are staged (they are the GEMM's input, complete
     * before it started) */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(16) unsigned char rc_smem[];
    const int T = a.T, E = a.E, K = a.K;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.x * RC_TT;
    const int nt = min(RC_TT, T - t0);
    const int xp = K + RC_XPAD;
    float *xs = reinterpret_cast<float *>(rc_smem);
    float *af = xs + (size_t)RC_TT * xp;
    uint16_t *pairs = reinterpret_cast<uint16_t *>(af + (size_t)RC_TT * E);
    float *wn = reinterpret_cast<float *>(
        (reinterpret_cast<uintptr_t>(pairs + (size_t)RC_TT * (E + 1)) + 15) & ~(uintptr_t)15);
    unsigned char *wbuf = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(wn + E + 1) + 15) & ~(uintptr_t)15);
    __shared__ const uint16_t *s_rowptr[RC_CW][32];
    __shared__ int s_npairs;
    __shared__ unsigned int s_xmin;
    __shared__ float s_xnorm[RC_TT];
    auto mark = [&](int k) {
        /* phase boundaries of CTA 0 (global timer, ns) for the profiling notes */
        if (a.stats && blockIdx.x == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            a.stats[2 + k] = (unsigned int)t;
        }
    };
    mark(0);
    if (tid == 0) {
        s_npairs = 0;
        s_xmin = 0x7f800000u;
    }
    for (int e = tid; e <= E; e += RC_THREADS) wn[e] = __ldg(&a.wnorm[e]);
    __syncthreads();

    /* ---- per token (one warp each, round robin): stage x, norm, fast logits,
     *      the top_k-th of them, the candidates ---- */
    for (int tl = warp; tl < nt; tl += RC_THREADS / 32) {
        const int t = t0 + tl;
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        unsigned int xmin = 0x7f800000u;
        /* every load of a batch is issued before the first is used */
        for (int k0 = 0; k0 < K; k0 += 2048) {
            uint4 xv[8];
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int k = k0 + c * 256 + lane * 8;
                xv[c] = k < K ? ldg16(a.x + (size_t)t * K + k) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int k = k0 + c * 256 + lane * 8;
                if (k >= K) continue;
                float f[8];
                unpack8(xv[c], f);
                float4 *d = reinterpret_cast<float4 *>(xs + (size_t)tl * xp + k);
                d[0] = make_float4(f[0], f[1], f[2], f[3]);
                d[1] = make_float4(f[4], f[5], f[6], f[7]);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    ss[j & 3] = fmaf(f[j], f[j], ss[j & 3]);
                    const unsigned int m = __float_as_uint(f[j]) & 0x7fffffffu;
                    if (m != 0 && m < xmin) xmin = m;
                }
            }
        }
        float s2 = warp_sum((ss[0] + ss[1]) + (ss[2] + ss[3]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, o));
        /* an upper bound of the norm: the fp32 sum of squares is within a
         * relative K*2^-23 of the truth */
        const float xnorm = sqrtf(s2) * 1.001f;
        if (lane == 0) {
            s_xnorm[tl] = xnorm;
            atomicMin(&s_xmin, xmin);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int e0 = 0; e0 < E; e0 += 256) {
            float av[8];
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int e = e0 + c * 32 + lane;
                float part[RC_MAX_SLABS];
#pragma unroll
                for (int sl = 0; sl < RC_MAX_SLABS; sl++)
                    part[sl] = (e < E && sl < a.nslab)
                                   ? __ldg(&a.approx[((size_t)sl * T + t) * E + e])
                                   : 0.0f;
                av[c] = (part[0] + part[1]) + (part[2] + part[3]);
            }
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int e = e0 + c * 32 + lane;
                if (e >= E) continue;
                af[(size_t)tl * E + e] = av[c];
                if (a.logits)
                    a.logits[(size_t)t * E + e] = bf16_bits(av[c]);   /* unless replaced below */
            }
        }
        __syncwarp();
        /* top_k-th largest fast logit (with multiplicity) */
        float a8 = 0.0f;
        unsigned int taken = 0;              /* bit i: my entry lane + 32*i is out */
        for (int i = 0; i < a.topk; i++) {
            int bk = INT_MIN, be = 0x7fffffff;
            for (int e = lane, j = 0; e < E; e += 32, j++) {
                if ((taken >> j) & 1u) continue;
                const int k = rc_float_key(af[(size_t)tl * E + e]);
                if (k > bk) { bk = k; be = e; }
            }
            const int wk = __reduce_max_sync(0xffffffffu, bk);
            const int we = (int)__reduce_min_sync(0xffffffffu,
                                                  bk == wk ? (unsigned)be : 0x7fffffffu);
            if (we < E) {
                a8 = af[(size_t)tl * E + we];
                if (lane == (we & 31)) taken |= 1u << (we >> 5);
            }
        }
        const float cb = a.cbound * xnorm;
        const float bmax = cb * wn[E];
        /* one BF16 step at the magnitude of the values compared, rounded up */
        const float spacing = (fabsf(a8) + bmax) * (1.0f / 64.0f) + 1e-30f;
        const float thr = a8 - bmax - spacing;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            const float v = af[(size_t)tl * E + e];
            const bool cand = v + cb * wn[e] >= thr;
            const unsigned m = __ballot_sync(0xffffffffu, cand);
            int base = 0;
            if (lane == 0 && m) base = atomicAdd(&s_npairs, __popc(m));
            base = __shfl_sync(0xffffffffu, base, 0);
            if (cand)
                pairs[base + __popc(m & ((1u << lane) - 1u))] = (uint16_t)((tl << 11) | e);
        }
        if (a.extra_row && lane == 0)
            pairs[atomicAdd(&s_npairs, 1)] = (uint16_t)((tl << 11) | E);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");   /* warps without a token */
    __syncthreads();
    mark(1);

    /* ---- exact chains, one lane per pair ---- */
    const int npairs = s_npairs;
    const double xmn = (double)__uint_as_float(s_xmin);
    const bool fma_ok = (a.wmin > 0.0f) && ((double)a.wmin * xmn >= 7.52316384526264e-37) &&
                        (!a.extra_row || ((a.wmin_extra > 0.0f) &&
                                          ((double)a.wmin_extra * xmn >= 7.52316384526264e-37)));
    if (warp < RC_CW) {
        unsigned char *wb = wbuf + (size_t)warp * RC_NBUF * 32 * RC_WPITCH;
        for (int base = warp * 32; base < npairs; base += RC_CW * 32) {
            const int p = base + lane;
            const bool valid = p < npairs;
            const int pr = pairs[valid ? p : base], tl = pr >> 11, e = pr & 0x7ff;
            const uint16_t *wrow = (e == E) ? a.extra_row : a.w + (size_t)e * K;
            __syncwarp();                     /* the previous round is done with these */
            s_rowptr[warp][lane] = wrow;
            __syncwarp();
            const float *xr = xs + (size_t)tl * xp;
            /* the two forms are separate instantiations of the whole loop: a
             * branch inside it would put both on the critical path */
            const float z = fma_ok ? rc_walk<true>(s_rowptr[warp], wb, xr, K, lane)
                                   : rc_walk<false>(s_rowptr[warp], wb, xr, K, lane);
            if (valid) {
                const int t = t0 + tl;
                if (e == E) {
                    a.extra_out[t] = bf16_bits(z);
                } else {
                    if (a.logits) a.logits[(size_t)t * E + e] = bf16_bits(z);
                    const float bound = a.cbound * s_xnorm[tl] * wn[e];
                    if (!(fabsf(z - af[(size_t)tl * E + e]) <= bound))
                        set_status(a.status, ST_BOUND_VIOLATED);
                    af[(size_t)tl * E + e] = bf16_round(z);    /* the exact logit */
                }
            }
        }
    }
    if (a.stats && tid == 0) atomicAdd(&a.stats[0], (unsigned)npairs);

    /* ---- softmax / top-k on the merged logits, one warp per token ---- */
    __syncthreads();
    mark(2);
    if (a.stats && blockIdx.x == 0 && tid == 0) a.stats[6] = (unsigned)npairs;
    for (int tl = warp; tl < nt; tl += RC_THREADS / 32) {
        float *pt = af + (size_t)tl * E;
        for (int e = lane; e < E; e += 32) pt[e] = bf16_round(pt[e]);
        __syncwarp();
        const int t = t0 + tl;
        router_softmax_topk(pt, E, a.topk, lane, a.idx_out + (size_t)t * a.topk,
                            a.w_out ? a.w_out + (size_t)t * a.topk : nullptr);
    }
    __syncthreads();
    mark(3);
}

inline size_t router_certify_smem(int E, int K) {
    return (size_t)RC_TT * (K + RC_XPAD) * 4 + (size_t)RC_TT * E * 4 +
           (size_t)RC_TT * (E + 1) * 2 + 16 + (size_t)(E + 1) * 4 + 16 +
           (size_t)RC_CW * RC_NBUF * 32 * RC_WPITCH;
}

/* ||w_e||_2 per row, rounded up; out[E] = the largest.  One warp per row. */
__global__ void __launch_bounds__(256)
row_norm_kernel(const uint16_t *__restrict__ w, int E, int K, float *__restrict__ out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= E) return;
    float ss = 0.f;
    for (int k = lane; k < K; k += 32) {
        const float v = bf16_f32(w[(size_t)warp * K + k]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float n = sqrtf(ss) * 1.001f;
    if (lane == 0) {
        out[warp] = n;
        atomicMax(reinterpret_cast<unsigned int *>(out + E), __float_as_uint(n));
    }
}

}  // namespace apus
