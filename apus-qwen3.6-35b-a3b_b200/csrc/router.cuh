/*
 * router.cuh — fused router: BF16 logits -> fp32 softmax -> top-k (lowest
 * index wins ties) -> renormalised BF16 weights, for a tile of tokens per CTA.
 *
 * Replaces apus_moe_route (c/moe.h:357-371) and its helpers
 * apus_moe_router_probs (c/moe.h:321-335) / apus_moe_router_select
 * (c/moe.h:339-355).  Selected ids must be bit-identical to the CPU engine's,
 * and the engine rounds its logits to BF16 before the softmax, so one fp32
 * ulp in a logit can flip a BF16 code and with it a selection.  The logit of
 * (token, expert) is therefore accumulated exactly as the CPU anchor does it
 * (c/bf16.h:285-294): one chain per (token, expert), k strictly ascending,
 * one rounding for the product and one for the add.
 *
 * Fast path: a product of two BF16 values has at most 16 significant bits,
 * so it is exact in fp32 whenever it does not underflow below 2^-133; then
 * rn(w*x) == w*x and fma(w, x, acc) == rn(rn(w*x) + acc) bit for bit.  The CTA
 * checks (smallest nonzero |w| of the router matrix, supplied by the host) x
 * (smallest nonzero |x| of its token tile) >= 2^-120 and takes the FMA chain;
 * otherwise it runs the literal multiply-then-add chain.
 *
 * Softmax: max by value; q_e = exp(l_e - m) evaluated in fp64 and rounded to
 * fp32 (glibc's expf is correctly rounded in all but vanishingly rare cases,
 * so this tracks it; a last-bit difference can only move a weight, never a
 * selection, because distinct BF16 logits give probabilities many ulps
 * apart and equal logits give equal probabilities on both sides); the
 * denominator is the ascending sequential fp32 sum; p_e = q_e / s; selection
 * on p with strict '>' from -inf; renormalisation sum in selection order.
 */
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace apus {

__device__ __forceinline__ void tma_load_2d_rl(void *dst, const CUtensorMap *map,
                                               int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::"
        "complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

constexpr int ROUTER_THREADS = 288;   /* 256 expert chains + a warp for the extra row */

template <int TT, bool FMA>
__device__ __forceinline__ void router_chains(const uint16_t *__restrict__ wrow,
                                              const float *__restrict__ xs,
                                              int K, float (&acc)[TT]) {
    /* wrow: this thread's expert row; xs: [TT][K] fp32 in shared memory */
    const bool vec = ((K & 7) == 0) && ((((uintptr_t)wrow) & 15) == 0);
    int k = 0;
    if (vec) {
#pragma unroll 2
        for (; k < K; k += 8) {
            uint4 wv = ldg16(wrow + k);
            float wf[8];
            wf[0] = bf16lo(wv.x); wf[1] = bf16hi(wv.x);
            wf[2] = bf16lo(wv.y); wf[3] = bf16hi(wv.y);
            wf[4] = bf16lo(wv.z); wf[5] = bf16hi(wv.z);
            wf[6] = bf16lo(wv.w); wf[7] = bf16hi(wv.w);
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const float4 xa =
                    *reinterpret_cast<const float4 *>(xs + (size_t)t * K + k);
                const float4 xb = *reinterpret_cast<const float4 *>(
                    xs + (size_t)t * K + k + 4);
                const float xf[8] = {xa.x, xa.y, xa.z, xa.w,
                                     xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (FMA)
                        acc[t] = __fmaf_rn(wf[j], xf[j], acc[t]);
                    else
                        acc[t] = __fadd_rn(acc[t], __fmul_rn(wf[j], xf[j]));
                }
            }
        }
    } else {
        for (; k < K; k++) {
            float wf = bf16_f32(__ldg(wrow + k));
#pragma unroll
            for (int t = 0; t < TT; t++) {
                float xf = xs[(size_t)t * K + k];
                if (FMA)
                    acc[t] = __fmaf_rn(wf, xf, acc[t]);
                else
                    acc[t] = __fadd_rn(acc[t], __fmul_rn(wf, xf));
            }
        }
    }
}

/* One warp turns a token's E BF16-valued logits (fp32 in shared memory,
 * overwritten) into the selection and the renormalised weights, exactly in
 * the order of c/moe.h:321-371. */
__device__ __forceinline__ void router_softmax_topk(float *p, int E, int topk,
                                                    int lane,
                                                    int32_t *__restrict__ idx_out,
                                                    uint16_t *__restrict__ w_out) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, p[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    for (int e = lane; e < E; e += 32)
        p[e] = (float)exp((double)__fsub_rn(p[e], m));
    __syncwarp();
    float s = 0.0f;
    if (lane == 0)
        for (int e = 0; e < E; e++) s = __fadd_rn(s, p[e]);
    s = __shfl_sync(0xffffffffu, s, 0);
    for (int e = lane; e < E; e += 32) p[e] = __fdiv_rn(p[e], s);
    __syncwarp();

    /* Selection.  Probabilities are non-negative, so their fp32 bit patterns
     * order like unsigned integers.  Each round: the warp-wide maximum
     * pattern (one redux), then the lowest index holding it (a second redux)
     * -- the strict '>' scan from -inf of the CPU loop, which keeps the lowest
     * index on ties.  A selected entry is overwritten with -inf (negative as
     * an integer) and can never win again. */
    int my_e = 0;
    float my_p = 0.0f;
    for (int i = 0; i < topk; i++) {
        int bb = -1, be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const int v = __float_as_int(p[e]);
            if (v > bb) { bb = v; be = e; }
        }
        const int wb = __reduce_max_sync(0xffffffffu, bb);
        int we;
        if (wb < 0) {          /* nothing left above -inf: CPU leaves best = 0 */
            we = 0;
        } else {
            we = (int)__reduce_min_sync(0xffffffffu,
                                        bb == wb ? (unsigned)be : 0x7fffffffu);
        }
        const float wp = wb < 0 ? p[0] : __int_as_float(wb);
        if (lane == i) { my_e = we; my_p = wp; }
        if (lane == (we & 31)) p[we] = -INFINITY;
        __syncwarp();
    }
    if (w_out) {
        float sw = 0.0f;
        for (int i = 0; i < topk; i++)
            sw = __fadd_rn(sw, __shfl_sync(0xffffffffu, my_p, i));
        if (lane < topk) w_out[lane] = bf16_bits(__fdiv_rn(my_p, sw));
    }
    if (lane < topk) idx_out[lane] = my_e;
}

/* The same arithmetic as router_softmax_topk, spread over a 256-thread CTA
 * for one token when latency matters (E <= 256): one expert per thread for the
 * exponentials, the division and the selection rounds; the denominator is
 * still the single ascending chain of c/moe.h:328-332 (thread 0).  Every
 * thread of the CTA must call it; results land in idx_out / w_out (shared or
 * global).  scratch: >= 2*16 ints of shared memory. */
__device__ __forceinline__ void router_softmax_topk_cta256(
    float *p /* [E] shared */, int E, int topk, int *scratch,
    int32_t *idx_out, uint16_t *w_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *fs = reinterpret_cast<float *>(scratch);
    /* max (value only) */
    float m = tid < E ? p[tid] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) fs[warp] = m;
    __syncthreads();
    m = fs[0];
#pragma unroll
    for (int w = 1; w < 8; w++) m = fmaxf(m, fs[w]);
    __syncthreads();
    float q = 0.0f;
    if (tid < E) {
        q = (float)exp((double)__fsub_rn(p[tid], m));
        p[tid] = q;
    }
    __syncthreads();
    if (tid == 0) {
        float s = 0.0f;
        for (int e = 0; e < E; e++) s = __fadd_rn(s, p[e]);
        fs[0] = s;
    }
    __syncthreads();
    const float s = fs[0];
    const float pr = tid < E ? __fdiv_rn(q, s) : -INFINITY;
    int myv = __float_as_int(pr);            /* >= 0 for a probability */
    if (tid >= E) myv = -1;
    __syncthreads();
    /* selection rounds: warp maxima to shared, everyone resolves the winner */
    float my_p = 0.0f;
    int my_e = 0;
    for (int i = 0; i < topk; i++) {
        const int wb = __reduce_max_sync(0xffffffffu, myv);
        const unsigned we = __reduce_min_sync(0xffffffffu,
                                              myv == wb ? (unsigned)tid : 0x7fffffffu);
        int *buf = scratch + (i & 1) * 16;
        if (lane == 0) {
            buf[warp] = wb;
            buf[8 + warp] = (int)we;
        }
        __syncthreads();
        int bb = buf[0], be = buf[8];
#pragma unroll
        for (int w = 1; w < 8; w++) {
            const int vb = buf[w], ve = buf[8 + w];
            if (vb > bb || (vb == bb && ve < be)) { bb = vb; be = ve; }
        }
        if (bb < 0) { be = 0; }              /* nothing left: CPU leaves best = 0 */
        if (tid == i) { my_e = be; my_p = __int_as_float(bb); }
        if (tid == be) myv = -1;
    }
    /* renormalisation in selection order (thread i holds pick i) */
    float *pk = fs;                           /* reuse: picks' probabilities */
    __syncthreads();
    if (tid < topk) pk[tid] = my_p;
    __syncthreads();
    if (tid < topk) {
        float sw = 0.0f;
        for (int i = 0; i < topk; i++) sw = __fadd_rn(sw, pk[i]);
        if (w_out) w_out[tid] = bf16_bits(__fdiv_rn(my_p, sw));
        idx_out[tid] = my_e;
    }
    __syncthreads();
}

/*
 * grid = ceil(T / TT); block = 256.  Dynamic shared memory:
 *   xs   float [TT][K]
 *   ps   float [TT][E]      logits, then exps, then probabilities
 * wmin = smallest nonzero |w| over the router matrix (0 = unknown: always
 * take the literal multiply-then-add chain).  topk == 0 is not allowed;
 * w_out may be NULL (ids only, c/moe.h:373-383); logits_out may be NULL.
 * extra_row [K] (optional) is one more weight row scored against every token
 * with the same exact chain, its BF16 result written to extra_out[t]: the
 * block uses it for the shared expert's gate logit (c/layer.h:355), which
 * then costs no launch and no extra latency.
 */
template <int TT>
__global__ void __launch_bounds__(ROUTER_THREADS)
router_topk_kernel(const uint16_t *__restrict__ x,
                   const uint16_t *__restrict__ wr, int T, int E, int K,
                   int topk, float wmin, int32_t *__restrict__ idx_out,
                   uint16_t *__restrict__ w_out,
                   uint16_t *__restrict__ logits_out,
                   const uint16_t *__restrict__ extra_row,
                   uint16_t *__restrict__ extra_out) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *xs = reinterpret_cast<float *>(smem_raw);
    float *ps = xs + (size_t)TT * K;
    __shared__ unsigned int s_xmin;

    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * TT;
    if (tid == 0) s_xmin = 0x7f800000u;
    __syncthreads();

    /* stage the token tile as fp32; track the smallest nonzero |x| */
    unsigned int xmin = 0x7f800000u;
    for (int i = tid; i < TT * K; i += ROUTER_THREADS) {
        int t = i / K, k = i - t * K;
        float v = 0.0f;
        if (t0 + t < T) {
            uint16_t c = x[(size_t)(t0 + t) * K + k];
            v = bf16_f32(c);
            unsigned int a = ((unsigned int)c << 16) & 0x7fffffffu;
            if (a != 0 && a < xmin) xmin = a;
        }
        xs[i] = v;
    }
    atomicMin(&s_xmin, xmin);
    __syncthreads();
    const double prod_floor = 7.52316384526264e-37;   /* 2^-120 */
    const bool use_fma =
        (wmin > 0.0f) &&
        ((double)wmin * (double)__uint_as_float(s_xmin) >= prod_floor);

    /* one chain per (token, expert) */
    const int rows = E + (extra_row ? 1 : 0);
    for (int e = tid; e < rows; e += ROUTER_THREADS) {
        float acc[TT];
#pragma unroll
        for (int t = 0; t < TT; t++) acc[t] = 0.0f;
        if (e == E) {
            router_chains<TT, false>(extra_row, xs, K, acc);
#pragma unroll
            for (int t = 0; t < TT; t++)
                if (t0 + t < T) extra_out[t0 + t] = bf16_bits(acc[t]);
            continue;
        }
        const uint16_t *wrow = wr + (size_t)e * K;
        if (use_fma)
            router_chains<TT, true>(wrow, xs, K, acc);
        else
            router_chains<TT, false>(wrow, xs, K, acc);
#pragma unroll
        for (int t = 0; t < TT; t++) {
            uint16_t code = bf16_bits(acc[t]);
            ps[(size_t)t * E + e] = bf16_f32(code);
            if (logits_out && t0 + t < T)
                logits_out[(size_t)(t0 + t) * E + e] = code;
        }
    }
    __syncthreads();

    /* one warp per token: softmax, selection, renormalisation */
    const int warp = tid >> 5, lane = tid & 31;
    for (int t = warp; t < TT; t += ROUTER_THREADS / 32) {
        if (t0 + t >= T) break;
        router_softmax_topk(ps + (size_t)t * E, E, topk, lane,
                            idx_out + (size_t)(t0 + t) * topk,
                            w_out ? w_out + (size_t)(t0 + t) * topk : nullptr);
    }
}

/* One exact chain over a router row and a token, both in shared memory.  The
 * dependent add (or fused multiply-add) per k is the critical path, so the
 * loop body holds nothing else that touches `acc`: FMA and literal
 * multiply-then-add are separate instantiations, and 64 k of operands are
 * loaded ahead of the 64 chain steps that consume them. */
template <bool FMA>
__device__ __forceinline__ float small_chain(const uint16_t *__restrict__ wrow,
                                             const float *__restrict__ xs,
                                             int K) {
    float acc = 0.0f;
    int k = 0;
#pragma unroll 2
    for (; k + 64 <= K; k += 64) {
        uint4 wv[8];
        float4 xv[16];
#pragma unroll
        for (int c = 0; c < 8; c++) {
            wv[c] = *reinterpret_cast<const uint4 *>(wrow + k + c * 8);
            xv[2 * c] = *reinterpret_cast<const float4 *>(xs + k + c * 8);
            xv[2 * c + 1] = *reinterpret_cast<const float4 *>(xs + k + c * 8 + 4);
        }
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float wf[8] = {bf16lo(wv[c].x), bf16hi(wv[c].x), bf16lo(wv[c].y),
                                 bf16hi(wv[c].y), bf16lo(wv[c].z), bf16hi(wv[c].z),
                                 bf16lo(wv[c].w), bf16hi(wv[c].w)};
            const float xf[8] = {xv[2 * c].x,     xv[2 * c].y,     xv[2 * c].z,
                                 xv[2 * c].w,     xv[2 * c + 1].x, xv[2 * c + 1].y,
                                 xv[2 * c + 1].z, xv[2 * c + 1].w};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (FMA)
                    acc = __fmaf_rn(wf[j], xf[j], acc);
                else
                    acc = __fadd_rn(acc, __fmul_rn(wf[j], xf[j]));
            }
        }
    }
    for (; k < K; k++) {       /* K % 64 tail (K is a multiple of 8) */
        const float wf = bf16_f32(wrow[k]);
        if (FMA)
            acc = __fmaf_rn(wf, xs[k], acc);
        else
            acc = __fadd_rn(acc, __fmul_rn(wf, xs[k]));
    }
    return acc;
}

/*
 * Latency path for few tokens.  grid = (ceil(rows / 8), ceil(T / TOK)), block
 * = 128: a CTA pulls eight router rows into shared memory with one bulk copy
 * each (all in flight at once, so the 1 MiB router matrix arrives spread over
 * 32 SMs instead of trickling through one) and stages TOK tokens as fp32;
 * the lanes of TOK/4 warps walk one exact chain each (lane = row * 4 + token),
 * and the BF16 logits go to global memory.  The CTA that arrives last for a
 * token (one atomic counter per token, which it resets for the next call) runs
 * that token's softmax / top-k on one of its warps.  No CTA ever waits on
 * another.  Requires K % 8 == 0 and a 16-byte-aligned router matrix.
 * Dynamic shared memory: 8 * (K*2 + 16) + TOK * ((K + 4) + E) * 4 bytes.
 */
constexpr int ROUTER_SMALL_ROWS = 8;
constexpr int ROUTER_SMALL_THREADS = 128;

/* TOK tokens per CTA: 4 (one chain warp) or 8 (two, on different schedulers) */
inline size_t router_small_smem(int E, int K, int tok) {
    return (size_t)ROUTER_SMALL_ROWS * (K * 2 + 16) + (size_t)tok * (K + 4) * 4 +
           (size_t)tok * E * 4;
}

template <int ROUTER_SMALL_TOK>
__global__ void __launch_bounds__(ROUTER_SMALL_THREADS)
router_small_kernel(const uint16_t *__restrict__ x,
                    const uint16_t *__restrict__ wr, int T, int E, int K,
                    int topk, float wmin, float wmin_extra,
                    int32_t *__restrict__ idx_out,
                    uint16_t *__restrict__ w_out,
                    uint16_t *__restrict__ logits_out,
                    const uint16_t *__restrict__ extra_row,
                    uint16_t *__restrict__ extra_out,
                    float *__restrict__ logits_ws,     /* [T][E] fp32 */
                    unsigned int *__restrict__ counters, /* [T], zero between calls */
                    int *status) {
    /* the next kernel may be scheduled; the wait for the previous one comes
     * after the router rows (constants) have been requested */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int pitch = K * 2 + 16;                 /* bytes; de-conflicts banks */
    const int xpitch = K + 4;                     /* floats; likewise for the tokens */
    unsigned char *rows_s = smem_raw;
    float *xs = reinterpret_cast<float *>(smem_raw + ROUTER_SMALL_ROWS * pitch);
    float *ps = xs + (size_t)ROUTER_SMALL_TOK * xpitch;
    __shared__ __align__(8) uint64_t bar;
    __shared__ unsigned int s_xmin;
    __shared__ int s_last[ROUTER_SMALL_TOK];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.y * ROUTER_SMALL_TOK;
    const int nt = min(ROUTER_SMALL_TOK, T - t0);
    const int rows_total = E + (extra_row ? 1 : 0);
    const int r0 = blockIdx.x * ROUTER_SMALL_ROWS;
    const int nrows = min(ROUTER_SMALL_ROWS, rows_total - r0);

    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        s_xmin = 0x7f800000u;
        mbar_expect_tx(&bar, (uint32_t)nrows * (uint32_t)K * 2u);
        for (int r = 0; r < nrows; r++) {
            const uint16_t *src = (r0 + r == E) ? extra_row
                                                : wr + (size_t)(r0 + r) * K;
            bulk_g2s(rows_s + (size_t)r * pitch, src, (uint32_t)K * 2u, &bar);
        }
    }
    if (tid < ROUTER_SMALL_TOK) s_last[tid] = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");   /* the tokens may be its output */
    __syncthreads();
    unsigned int xmin = 0x7f800000u;
    const int c8 = K / 8;
    for (int c = tid; c < nt * c8; c += ROUTER_SMALL_THREADS) {
        const int tt = c / c8, cc = c - tt * c8;
        const uint4 v = ldg16(x + (size_t)(t0 + tt) * K + (size_t)cc * 8);
        const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
        float4 *d = reinterpret_cast<float4 *>(xs + (size_t)tt * xpitch + cc * 8);
        d[0] = make_float4(bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y));
        d[1] = make_float4(bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w));
#pragma unroll
        for (int q = 0; q < 4; q++) {
            unsigned int a = (wds[q] << 16) & 0x7fffffffu;
            unsigned int b = wds[q] & 0x7fff0000u;
            if (a != 0 && a < xmin) xmin = a;
            if (b != 0 && b < xmin) xmin = b;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, o));
    if (lane == 0) atomicMin(&s_xmin, xmin);
    __syncthreads();
    if (warp < ROUTER_SMALL_TOK / 4) {
        const double xmn = (double)__uint_as_float(s_xmin);
        const bool use_fma = (wmin > 0.0f) && ((double)wmin * xmn >= 7.52316384526264e-37);
        const bool use_fma_x =
            (wmin_extra > 0.0f) && ((double)wmin_extra * xmn >= 7.52316384526264e-37);
        const bool arrived = mbar_wait(&bar, 0);
        if (!arrived) set_status(status, ST_MBAR_TIMEOUT);
        const int r = lane >> 2, tt = warp * 4 + (lane & 3);
        if (arrived && r < nrows && tt < nt) {
            const uint16_t *wrow =
                reinterpret_cast<const uint16_t *>(rows_s + (size_t)r * pitch);
            const float *xr = xs + (size_t)tt * xpitch;
            const bool fma_row = (r0 + r != E) ? use_fma : use_fma_x;
            const float acc = fma_row ? small_chain<true>(wrow, xr, K)
                                      : small_chain<false>(wrow, xr, K);
            const uint16_t code = bf16_bits(acc);
            const int t = t0 + tt;
            if (r0 + r == E) {
                extra_out[t] = code;
            } else {
                logits_ws[(size_t)t * E + r0 + r] = bf16_f32(code);
                if (logits_out) logits_out[(size_t)t * E + r0 + r] = code;
            }
        }
        /* the last CTA of a token finishes that token */
        __threadfence();
        __syncwarp();
        if (lane < 4 && warp * 4 + lane < nt)
            s_last[warp * 4 + lane] =
                atomicAdd(&counters[t0 + warp * 4 + lane], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += ROUTER_SMALL_THREADS / 32) {
        if (!s_last[tt]) continue;
        const int t = t0 + tt;
        float *p = ps + (size_t)tt * E;
        __threadfence();
        for (int e = lane; e < E; e += 32)
            p[e] = __ldcg(&logits_ws[(size_t)t * E + e]);
        __syncwarp();
        if (lane == 0) counters[t] = 0;
        router_softmax_topk(p, E, topk, lane, idx_out + (size_t)t * topk,
                            w_out ? w_out + (size_t)t * topk : nullptr);
    }
}

constexpr int RL_STAGES = 3;
constexpr int RL_BK = 64;
constexpr int RL_XPITCH = RL_BK + 4;   /* floats; keeps 4 token groups on
                                        * different banks */

/* One 64-k block of router_logits_kernel's register tile (4 experts x TT/4
 * tokens per thread); FMA and literal multiply-then-add are separate
 * instantiations so neither chain carries the other's instructions. */
template <int TT, bool FMA>
__device__ __forceinline__ void logits_kblock(const unsigned char *__restrict__ st,
                                              const float *__restrict__ xs,
                                              int er0, int tg,
                                              float (&acc)[4][TT / 4]) {
    constexpr int TPT = TT / 4;
#pragma unroll 2
    for (int c = 0; c < 8; c++) {
        float wf[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = er0 + i;
            const uint4 wv = *reinterpret_cast<const uint4 *>(
                st + (r >> 7) * 16384 + (r & 127) * 128 + ((c ^ (r & 7)) << 4));
            wf[i][0] = bf16lo(wv.x); wf[i][1] = bf16hi(wv.x);
            wf[i][2] = bf16lo(wv.y); wf[i][3] = bf16hi(wv.y);
            wf[i][4] = bf16lo(wv.z); wf[i][5] = bf16hi(wv.z);
            wf[i][6] = bf16lo(wv.w); wf[i][7] = bf16hi(wv.w);
        }
#pragma unroll
        for (int j = 0; j < TPT; j++) {
            const float *xp = xs + (j * 4 + tg) * RL_XPITCH + c * 8;
            const float4 xa = *reinterpret_cast<const float4 *>(xp);
            const float4 xb = *reinterpret_cast<const float4 *>(xp + 4);
            const float xf[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int kk = 0; kk < 8; kk++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (FMA)
                        acc[i][j] = __fmaf_rn(wf[i][kk], xf[kk], acc[i][j]);
                    else
                        acc[i][j] = __fadd_rn(acc[i][j],
                                              __fmul_rn(wf[i][kk], xf[kk]));
                }
        }
    }
}

/*
 * Throughput path for many tokens, in two kernels.
 *
 * router_logits_kernel<TT, ROWS>: grid = (ceil(T/TT), E/ROWS), block = ROWS+32.
 * A CTA scores ROWS experts (128 or 256) against TT tokens (8, 16 or 32).
 * Its slice of the router matrix streams through a three-stage shared-memory
 * ring of [ROWS x 64 k] tiles loaded by TMA (128-byte swizzle, no multicast);
 * the token tile's k-slice rides in the same ring as fp32.
 *
 * Shared memory serves one 128-byte wavefront per cycle whether or not the
 * lanes of a load want the same address, so a thread that owned one expert
 * and read every token's x by broadcast would spend four wavefronts per four
 * FMAs.  Instead each thread owns a 4-expert x (TT/4)-token register tile
 * (lane = 8 expert groups x 4 token groups): per eight k it loads 4 weight
 * vectors and TT/4 x vectors and issues 32*(TT/4) FMAs, every chain still
 * strictly ascending in k.  Every token tile re-reads the whole router matrix
 * from L2, so TT also sets the L2 traffic (T/TT MiB at the real dims): the host
 * picks the largest TT that still fills the SMs.  Lanes 0..TT-1 of the last
 * warp score the optional extra row (the shared expert's gate).  BF16 logits
 * go to logits_out [T, E].  Requires E % ROWS == 0, K % 64 == 0.
 *
 * router_select_kernel: one warp per token turns the logits into ids and
 * weights (router_softmax_topk).
 */

template <int TT, int ROWS>
__global__ void __launch_bounds__(ROWS + 32)
router_logits_kernel(const __grid_constant__ CUtensorMap map_w,   /* [E, K] box {64,128} */
                     const uint16_t *__restrict__ x, int T, int E, int K,
                     float wmin, uint16_t *__restrict__ logits_out,
                     const uint16_t *__restrict__ extra_row,
                     uint16_t *__restrict__ extra_out, int *status) {
    pdl_enter();
    static_assert(TT <= 32 && TT % 4 == 0, "token tile");
    constexpr int THREADS = ROWS + 32;
    constexpr int TPT = TT / 4;          /* tokens per thread */
    constexpr int EPT = 4;               /* experts per thread */
    /* ROWS experts / (8 expert groups * EPT) warps do the chains */
    constexpr int CHAIN_WARPS = ROWS / 32;
    extern __shared__ unsigned char rl_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(rl_smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int W_BYTES = ROWS * RL_BK * 2;
    constexpr int X_BYTES = TT * RL_XPITCH * 4;
    constexpr int STAGE = W_BYTES + ((X_BYTES + 1023) & ~1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + RL_STAGES * STAGE);
    __shared__ unsigned int s_xmin;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = blockIdx.x * TT;
    const int e0 = blockIdx.y * ROWS;
    const int nkb = K / RL_BK;
    if (tid == 0) {
        for (int s = 0; s < RL_STAGES; s++) mbar_init(&full[s], 1);
        mbar_fence_init();
        s_xmin = 0x7f800000u;
    }
    __syncthreads();

    auto issue = [&](int kb) {   /* thread 0 */
        const int s = kb % RL_STAGES;
        unsigned char *st = smem + (size_t)s * STAGE;
        mbar_expect_tx(&full[s], W_BYTES);
#pragma unroll
        for (int b = 0; b < ROWS / 128; b++)
            tma_load_2d_rl(st + b * 16384, &map_w, kb * RL_BK, e0 + b * 128,
                           &full[s]);
    };
    /* The token tile's k-slice for a stage: a thread fetches one 16-byte
     * piece into registers early (x_fetch), so the global-load latency hides
     * behind the chains, and widens it into the stage afterwards (x_store). */
    constexpr int XV = TT * RL_BK / 8;             /* 16-byte pieces per stage */
    static_assert(XV <= THREADS, "token tile too large for one piece per thread");
    uint4 xr = make_uint4(0, 0, 0, 0);
    auto x_fetch = [&](int kb) {
        xr = make_uint4(0, 0, 0, 0);
        if (tid < XV) {
            const int t = tid >> 3, j = tid & 7;
            if (t0 + t < T)
                xr = ldg16(x + (size_t)(t0 + t) * K + kb * RL_BK + j * 8);
        }
    };
    auto x_store = [&](int kb) {
        if (tid < XV) {
            const int s = kb % RL_STAGES;
            float *xs = reinterpret_cast<float *>(smem + (size_t)s * STAGE + W_BYTES);
            float4 *d = reinterpret_cast<float4 *>(xs + (tid >> 3) * RL_XPITCH +
                                                   (tid & 7) * 8);
            d[0] = make_float4(bf16lo(xr.x), bf16hi(xr.x), bf16lo(xr.y), bf16hi(xr.y));
            d[1] = make_float4(bf16lo(xr.z), bf16hi(xr.z), bf16lo(xr.w), bf16hi(xr.w));
        }
    };
    if (tid == 0)
        for (int kb = 0; kb < RL_STAGES && kb < nkb; kb++) issue(kb);
    for (int kb = 0; kb < RL_STAGES && kb < nkb; kb++) {
        x_fetch(kb);
        x_store(kb);
    }
    /* from here on the piece for stage kb+STAGES is fetched a whole k-block
     * before it is stored (xr_hold carries it across one iteration) */
    uint4 xr_hold = make_uint4(0, 0, 0, 0);
    if (RL_STAGES < nkb) {
        x_fetch(RL_STAGES);
        xr_hold = xr;
    }

    /* smallest nonzero |x| of the token tile (FMA-exactness guard) */
    unsigned int xmin = 0x7f800000u;
    for (int i = tid; i < TT * (K / 8); i += THREADS) {
        const int t = i / (K / 8), c = i - t * (K / 8);
        if (t0 + t < T) {
            const uint4 v = ldg16(x + (size_t)(t0 + t) * K + (size_t)c * 8);
            const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                unsigned int a = (wds[q] << 16) & 0x7fffffffu;
                unsigned int b = wds[q] & 0x7fff0000u;
                if (a != 0 && a < xmin) xmin = a;
                if (b != 0 && b < xmin) xmin = b;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        xmin = min(xmin, __shfl_xor_sync(0xffffffffu, xmin, o));
    if (lane == 0) atomicMin(&s_xmin, xmin);
    __syncthreads();
    const bool use_fma =
        (wmin > 0.0f) &&
        ((double)wmin * (double)__uint_as_float(s_xmin) >= 7.52316384526264e-37);

    /* register tile: experts er0..er0+3 (rows inside the CTA's slice), tokens
     * tg, tg+4, tg+8, ... */
    float acc[EPT][TPT];
#pragma unroll
    for (int i = 0; i < EPT; i++)
#pragma unroll
        for (int j = 0; j < TPT; j++) acc[i][j] = 0.0f;
    float acc_extra = 0.0f;
    const bool is_chain = warp < CHAIN_WARPS;
    const int er0 = warp * 32 + (lane >> 2) * EPT;
    const int tg = lane & 3;
    const bool is_extra = extra_row && blockIdx.y == 0 && warp == CHAIN_WARPS &&
                          lane < TT;
    bool ok = true;
    for (int kb = 0; kb < nkb; kb++) {
        const int s = kb % RL_STAGES;
        const uint4 xr_store = xr_hold;              /* piece for kb+STAGES */
        if (kb + RL_STAGES + 1 < nkb) {
            x_fetch(kb + RL_STAGES + 1);
            xr_hold = xr;
        }
        if (ok && !mbar_wait(&full[s], (uint32_t)(kb / RL_STAGES) & 1u)) {
            ok = false;
            set_status(status, ST_MBAR_TIMEOUT);
        }
        const unsigned char *st = smem + (size_t)s * STAGE;
        const float *xs = reinterpret_cast<const float *>(st + W_BYTES);
        if (ok && is_chain) {
            if (use_fma)
                logits_kblock<TT, true>(st, xs, er0, tg, acc);
            else
                logits_kblock<TT, false>(st, xs, er0, tg, acc);
        } else if (ok && is_extra) {
            /* lane t: the extra row against token t (literal chain) */
            float a = acc_extra;
            uint4 ev[RL_BK / 8];
#pragma unroll
            for (int c = 0; c < RL_BK / 8; c++)
                ev[c] = ldg16(extra_row + kb * RL_BK + c * 8);
#pragma unroll
            for (int c = 0; c < RL_BK / 8; c++) {
                const float ef[8] = {bf16lo(ev[c].x), bf16hi(ev[c].x),
                                     bf16lo(ev[c].y), bf16hi(ev[c].y),
                                     bf16lo(ev[c].z), bf16hi(ev[c].z),
                                     bf16lo(ev[c].w), bf16hi(ev[c].w)};
#pragma unroll
                for (int j = 0; j < 8; j++)
                    a = __fadd_rn(a, __fmul_rn(ef[j],
                                               xs[lane * RL_XPITCH + c * 8 + j]));
            }
            acc_extra = a;
        }
        __syncthreads();            /* everyone is done with stage s */
        if (kb + RL_STAGES < nkb) {
            if (tid == 0 && ok) issue(kb + RL_STAGES);
            xr = xr_store;
            x_store(kb + RL_STAGES);
        }
    }
    if (!ok) return;
    if (is_chain) {
#pragma unroll
        for (int j = 0; j < TPT; j++) {
            const int t = t0 + j * 4 + tg;
            if (t < T) {
                /* four consecutive experts: one 8-byte store */
                uint2 v;
                v.x = pack_bf16(acc[0][j], acc[1][j]);
                v.y = pack_bf16(acc[2][j], acc[3][j]);
                *reinterpret_cast<uint2 *>(logits_out + (size_t)t * E + e0 + er0) = v;
            }
        }
    } else if (is_extra) {
        if (t0 + lane < T) extra_out[t0 + lane] = bf16_bits(acc_extra);
    }
}

__global__ void __launch_bounds__(256)
router_select_kernel(const uint16_t *__restrict__ logits, int T, int E,
                     int topk, int32_t *__restrict__ idx_out,
                     uint16_t *__restrict__ w_out) {
    pdl_enter();
    extern __shared__ float sel_smem[];   /* [8][E] */
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + warp;
    if (t >= T) return;
    float *p = sel_smem + (size_t)warp * E;
    for (int e = lane; e < E; e += 32) p[e] = bf16_f32(logits[(size_t)t * E + e]);
    __syncwarp();
    router_softmax_topk(p, E, topk, lane, idx_out + (size_t)t * topk,
                        w_out ? w_out + (size_t)t * topk : nullptr);
}

/* smallest nonzero |w| over n BF16 codes, as fp32 bits (min-reduced into
 * *out, which the host initialises to +inf bits). */
__global__ void bf16_min_nonzero_kernel(const uint16_t *__restrict__ w,
                                        size_t n, unsigned int *out) {
    unsigned int m = 0x7f800000u;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        unsigned int a = ((unsigned int)w[i] << 16) & 0x7fffffffu;
        if (a != 0 && a < m) m = a;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        m = min(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMin(out, m);
}

}  // namespace apus
