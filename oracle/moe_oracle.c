/*
 * oracle/moe_oracle.c — TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of the reference engine's MoE-block arithmetic, used
 * only as the checker: tests, the smoke check and the CPU-baseline leg of the
 * benchmark load it; the CUDA library never does.  Every function names the
 * reference site whose arithmetic it restates (paths are relative to the
 * reference project).  The contract restated here: BF16 storage, fp32
 * arithmetic, every dot product accumulated sequentially in ascending k with
 * a separate multiply and add (no FMA; build with -ffp-contract=off), and an
 * RNE narrowing at each point where the reference materialises BF16.
 *
 * Parity pinned: this file is checked bit-for-bit against the reference's own
 * compiled code (oracle/_ref/libapus_ref.so) and against the reference's
 * golden vectors and known-answer tests (tests/golden/).
 *
 * Threads (OpenMP) only ever split independent outputs; each output's
 * accumulation order is fixed, so results are identical at any thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* --- c/bf16.h:261-274 : exact widen, RNE narrow with NaN pass-through ---- */
static inline float widen(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t narrow(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(u >> 16);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
ORC_API float orc_bf16_f32(uint16_t b) { return widen(b); }
ORC_API uint16_t orc_bf16_bits(float f) { return narrow(f); }
ORC_API int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* --- c/bf16.h:285-300 : GEMV / GEMM scalar anchor ------------------------
 * y[m,o] = rnd(sum_k f32(W[o,k]) * f32(x[m,k])), k ascending, mul then add.
 * Eight activation rows share one pass over a weight row (independent
 * chains; the per-output order is untouched). */
typedef float v8f __attribute__((vector_size(32)));

static void gemm_rows(const uint16_t *w, const uint16_t *x, uint16_t *y,
                      size_t M, size_t O, size_t K) {
    if (M == 1) {
        /* GEMV: chains for independent output rows, interleaved by 8. */
#pragma omp parallel for schedule(static)
        for (size_t ob = 0; ob < (O + 7) / 8; ob++) {
            size_t o0 = ob * 8, n = O - o0 < 8 ? O - o0 : 8;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t k = 0; k < K; k++) {
                float xv = widen(x[k]);
                for (size_t r = 0; r < n; r++) {
                    float p = widen(w[(o0 + r) * K + k]) * xv;
                    acc[r] = acc[r] + p;
                }
            }
            for (size_t r = 0; r < n; r++) y[o0 + r] = narrow(acc[r]);
        }
        return;
    }
    /* x transposed and widened to [K][Mp] so eight rows are one vector. */
    size_t Mp = (M + 7) & ~(size_t)7;
    float *xt = aligned_alloc(64, K * Mp * sizeof(float));
    for (size_t k = 0; k < K; k++)
        for (size_t m = 0; m < Mp; m++)
            xt[k * Mp + m] = m < M ? widen(x[m * K + k]) : 0.0f;
#pragma omp parallel for schedule(static)
    for (size_t o = 0; o < O; o++) {
        const uint16_t *wr = w + o * K;
        for (size_t mb = 0; mb < Mp; mb += 32) {
            size_t nv = (Mp - mb) / 8 < 4 ? (Mp - mb) / 8 : 4;
            v8f acc[4];
            for (size_t v = 0; v < 4; v++)
                acc[v] = (v8f){0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t k = 0; k < K; k++) {
                float wv = widen(wr[k]);
                v8f wb = {wv, wv, wv, wv, wv, wv, wv, wv};
                const float *xr = xt + k * Mp + mb;
                for (size_t v = 0; v < nv; v++) {
                    v8f xv;
                    memcpy(&xv, xr + v * 8, 32);
                    v8f p = wb * xv;
                    acc[v] = acc[v] + p;
                }
            }
            for (size_t v = 0; v < nv; v++)
                for (size_t l = 0; l < 8; l++) {
                    size_t m = mb + v * 8 + l;
                    if (m < M) y[m * O + o] = narrow(acc[v][l]);
                }
        }
    }
    free(xt);
}

ORC_API void orc_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y,
                           size_t O, size_t K) {
    gemm_rows(w, x, y, 1, O, K);
}
ORC_API void orc_bf16_gemm(const uint16_t *w, const uint16_t *x, uint16_t *y,
                           size_t M, size_t O, size_t K) {
    gemm_rows(w, x, y, M, O, K);
}

/* --- c/moe.h:151-160 : fp32-out matvec, no narrowing ---------------------- */
ORC_API void orc_matvec_f32(const uint16_t *w, const uint16_t *x, float *y,
                            size_t O, size_t K) {
    for (size_t o = 0; o < O; o++) {
        float acc = 0.0f;
        for (size_t k = 0; k < K; k++) {
            float p = widen(w[o * K + k]) * widen(x[k]);
            acc = acc + p;
        }
        y[o] = acc;
    }
}

/* --- c/moe.h:312-314 : sigmoid -------------------------------------------- */
static inline float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

/* --- c/moe.h:321-355 : fp32 softmax over bf16 logits, then top-n ----------
 * max by ascending scan with strict '>'; exps and their sum ascending;
 * selection = n passes, strict '>' against -inf, so the lowest index wins a
 * tie and the picks come out in descending-probability order. */
static void router_from_logits(const uint16_t *logits, size_t E, size_t n,
                               int32_t *idx, float *probs) {
    float m = widen(logits[0]);
    for (size_t e = 1; e < E; e++) {
        float a = widen(logits[e]);
        if (a > m) m = a;
    }
    float s = 0.0f;
    for (size_t e = 0; e < E; e++) {
        probs[e] = expf(widen(logits[e]) - m);
        s = s + probs[e];
    }
    for (size_t e = 0; e < E; e++) probs[e] = probs[e] / s;
    uint8_t *sel = calloc(E, 1);
    for (size_t i = 0; i < n; i++) {
        size_t best = 0;
        float bv = -INFINITY;
        for (size_t e = 0; e < E; e++)
            if (!sel[e] && probs[e] > bv) {
                bv = probs[e];
                best = e;
            }
        sel[best] = 1;
        idx[i] = (int32_t)best;
    }
    free(sel);
}

/* Logits for one token, one thread (used under an outer parallel loop). */
static void logits_one(const uint16_t *x, const uint16_t *wg, uint16_t *lg,
                       size_t E, size_t K) {
    for (size_t e0 = 0; e0 < E; e0 += 8) {
        size_t n = E - e0 < 8 ? E - e0 : 8;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t k = 0; k < K; k++) {
            float xv = widen(x[k]);
            for (size_t r = 0; r < n; r++) {
                float p = widen(wg[(e0 + r) * K + k]) * xv;
                acc[r] = acc[r] + p;
            }
        }
        for (size_t r = 0; r < n; r++) lg[e0 + r] = narrow(acc[r]);
    }
}

/* --- c/moe.h:357-371 : route = bf16 logits -> softmax -> top-k -> renorm --
 * renormalisation sum runs in selection order; weights narrowed to BF16. */
static void route_one(const uint16_t *x, const uint16_t *wg, int32_t *idx,
                      uint16_t *w, size_t E, size_t K, size_t topk,
                      uint16_t *logits_out) {
    uint16_t *lg = malloc(E * 2);
    float *probs = malloc(E * sizeof(float));
    logits_one(x, wg, lg, E, K);
    router_from_logits(lg, E, topk, idx, probs);
    if (w) {
        float sw = 0.0f;
        for (size_t i = 0; i < topk; i++) sw = sw + probs[idx[i]];
        for (size_t i = 0; i < topk; i++) w[i] = narrow(probs[idx[i]] / sw);
    }
    if (logits_out) memcpy(logits_out, lg, E * 2);
    free(lg);
    free(probs);
}
ORC_API void orc_moe_route(const uint16_t *x, const uint16_t *wg,
                           int32_t *idx, uint16_t *w, size_t E, size_t K,
                           size_t topk) {
    route_one(x, wg, idx, w, E, K, topk, NULL);
}
/* --- c/moe.h:373-383 : first n picks, no weights -------------------------- */
ORC_API void orc_moe_route_topn(const uint16_t *x, const uint16_t *wg,
                                int32_t *idx, size_t n, size_t E, size_t K) {
    route_one(x, wg, idx, NULL, E, K, n, NULL);
}
/* Batched router with optional logits capture: T independent tokens. */
ORC_API void orc_moe_route_batch(const uint16_t *x, const uint16_t *wg,
                                 int32_t *idx, uint16_t *w, uint16_t *logits,
                                 size_t T, size_t E, size_t K, size_t topk) {
#pragma omp parallel for schedule(dynamic, 4)
    for (size_t t = 0; t < T; t++)
        route_one(x + t * K, wg, idx + t * topk, w + t * topk, E, K, topk,
                  logits ? logits + t * E : NULL);
}

/* --- c/moe.h:387-395 : routed activation, TWO roundings ------------------- */
ORC_API void orc_moe_silu_act(const uint16_t *gu, uint16_t *act, size_t I) {
    for (size_t i = 0; i < I; i++) {
        float g = widen(gu[i]);
        uint16_t a1 = narrow(g * sigmoidf_(g));
        act[i] = narrow(widen(a1) * widen(gu[I + i]));
    }
}
/* --- c/moe.h:438-445 : shared activation, ONE rounding -------------------- */
ORC_API void orc_moe_silu_mul(const uint16_t *g, const uint16_t *u,
                              uint16_t *y, size_t I) {
    for (size_t i = 0; i < I; i++) {
        float gv = widen(g[i]);
        float sil = gv * sigmoidf_(gv);
        y[i] = narrow(sil * widen(u[i]));
    }
}
/* --- c/moe.h:487-495 : weighted combine, slots ascending, single rnd ------ */
ORC_API void orc_moe_combine(const uint16_t *y, const uint16_t *w,
                             uint16_t *out, size_t k, size_t N) {
    for (size_t n = 0; n < N; n++) {
        float acc = 0.0f;
        for (size_t e = 0; e < k; e++) {
            float p = widen(w[e]) * widen(y[e * N + n]);
            acc = acc + p;
        }
        out[n] = narrow(acc);
    }
}
/* --- c/attn.h:175-186 : RMSNorm, (1+w) gain, single rounding -------------- */
ORC_API void orc_rmsnorm(const uint16_t *x, const uint16_t *w, uint16_t *y,
                         size_t N) {
    float ss = 0.0f;
    for (size_t i = 0; i < N; i++) {
        float v = widen(x[i]);
        float p = v * v;
        ss = ss + p;
    }
    float rs = 1.0f / sqrtf(ss / (float)N + 1e-6f);
    for (size_t i = 0; i < N; i++) {
        float a = widen(x[i]) * rs;
        float g = 1.0f + (w ? widen(w[i]) : 0.0f);
        y[i] = narrow(a * g);
    }
}
/* --- c/layer.h:230-234 : residual add ------------------------------------- */
ORC_API void orc_resadd(const uint16_t *a, const uint16_t *b, uint16_t *out,
                        size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = narrow(widen(a[i]) + widen(b[i]));
}

/* --- c/layer.h:599-606,614-620 : the dispatch order the batched body implies
 * For e ascending, t ascending, slot j ascending: the r-th row of expert e's
 * gathered batch is flat assignment a = t*TK + j.  That is a stable counting
 * sort of the flat assignments by expert id. */
ORC_API void orc_dispatch(const int32_t *idx, size_t T, size_t TK, size_t E,
                          int32_t *counts, int32_t *offsets, int32_t *perm) {
    for (size_t e = 0; e < E; e++) counts[e] = 0;
    for (size_t a = 0; a < T * TK; a++) counts[idx[a]]++;
    offsets[0] = 0;
    for (size_t e = 0; e < E; e++) offsets[e + 1] = offsets[e] + counts[e];
    int32_t *cur = malloc(E * sizeof(int32_t));
    memcpy(cur, offsets, E * sizeof(int32_t));
    for (size_t a = 0; a < T * TK; a++) perm[cur[idx[a]]++] = (int32_t)a;
    free(cur);
}

/* --- c/layer.h:333-370 (per token) == c/layer.h:570-651 (batched) ---------
 * The whole block for T tokens.  Realised expert-major like the batched body
 * (each routed expert's two linears once over its gathered rows); every row
 * is bitwise what the per-token body produces because each output element's
 * arithmetic is independent of the batch it sits in. */
ORC_API void orc_moe_block(size_t H, size_t E, size_t I, size_t Is, size_t TK,
                           const uint16_t *rtr_w, const uint16_t *exp_gu,
                           const uint16_t *exp_d, const uint16_t *sh_g,
                           const uint16_t *sh_u, const uint16_t *sh_d,
                           const uint16_t *sh_gate, const uint16_t *ln2,
                           uint16_t *moe_out, size_t T, int32_t *tr_idx,
                           uint16_t *tr_w, uint16_t *tr_routed,
                           uint16_t *tr_shared) {
    size_t A = T * TK;
    int32_t *idx = malloc(A * sizeof(int32_t));
    uint16_t *rw = malloc(A * 2);
    orc_moe_route_batch(ln2, rtr_w, idx, rw, NULL, T, E, H, TK);

    /* shared expert: c/layer.h:351-360 / 593-597,626-635 */
    uint16_t *sg = malloc(T * Is * 2), *su = malloc(T * Is * 2);
    uint16_t *sa = malloc(T * Is * 2), *sy = malloc(T * H * 2);
    uint16_t *sgl = malloc(T * 2);
    gemm_rows(sh_g, ln2, sg, T, Is, H);
    gemm_rows(sh_u, ln2, su, T, Is, H);
    orc_moe_silu_mul(sg, su, sa, T * Is);
    gemm_rows(sh_d, sa, sy, T, H, Is);
    gemm_rows(sh_gate, ln2, sgl, T, 1, H);

    /* routed experts over the dispatch order */
    int32_t *counts = malloc(E * sizeof(int32_t));
    int32_t *offsets = malloc((E + 1) * sizeof(int32_t));
    int32_t *perm = malloc(A * sizeof(int32_t));
    orc_dispatch(idx, T, TK, E, counts, offsets, perm);
    uint16_t *eo = malloc(A * H * 2);
    size_t maxc = 0;
    for (size_t e = 0; e < E; e++)
        if ((size_t)counts[e] > maxc) maxc = (size_t)counts[e];
    uint16_t *xg = malloc((maxc ? maxc : 1) * H * 2);
    uint16_t *gu = malloc((maxc ? maxc : 1) * 2 * I * 2);
    uint16_t *act = malloc((maxc ? maxc : 1) * I * 2);
    uint16_t *eb = malloc((maxc ? maxc : 1) * H * 2);
    for (size_t e = 0; e < E; e++) {
        size_t cnt = (size_t)counts[e];
        if (!cnt) continue;
        const int32_t *rows = perm + offsets[e];
        for (size_t r = 0; r < cnt; r++)
            memcpy(xg + r * H, ln2 + (size_t)(rows[r] / (int32_t)TK) * H,
                   H * 2);
        gemm_rows(exp_gu + e * 2 * I * H, xg, gu, cnt, 2 * I, H);
        for (size_t r = 0; r < cnt; r++)
            orc_moe_silu_act(gu + r * 2 * I, act + r * I, I);
        gemm_rows(exp_d + e * H * I, act, eb, cnt, H, I);
        for (size_t r = 0; r < cnt; r++)
            memcpy(eo + (size_t)rows[r] * H, eb + r * H, H * 2);
    }

    /* per-token tail: c/layer.h:350,356-361 / 625-649 */
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < T; t++) {
        uint16_t sgat = narrow(1.0f / (1.0f + expf(-widen(sgl[t]))));
        uint16_t *routed = malloc(H * 2);
        orc_moe_combine(eo + t * TK * H, rw + t * TK, routed, TK, H);
        for (size_t i = 0; i < H; i++) {
            uint16_t shared = narrow(widen(sy[t * H + i]) * widen(sgat));
            moe_out[t * H + i] = narrow(widen(routed[i]) + widen(shared));
            if (tr_shared) tr_shared[t * H + i] = shared;
        }
        if (tr_routed) memcpy(tr_routed + t * H, routed, H * 2);
        free(routed);
    }
    if (tr_idx) memcpy(tr_idx, idx, A * sizeof(int32_t));
    if (tr_w) memcpy(tr_w, rw, A * 2);
    free(idx); free(rw); free(sg); free(su); free(sa); free(sy); free(sgl);
    free(counts); free(offsets); free(perm); free(eo); free(xg); free(gu);
    free(act); free(eb);
}
