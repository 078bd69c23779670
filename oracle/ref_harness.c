/*
 * oracle/ref_harness.c — TEST INFRASTRUCTURE, not product code.
 *
 * One translation unit that pulls in the reference engine's own headers
 * (from the read-only reference checkout, via -I; nothing is copied) with all
 * five *_IMPLEMENTATION macros defined, so the file-static MoE functions
 * apus_layer_moe (c/layer.h:333-370) and apus_layer_moe_batch
 * (c/layer.h:570-651) are callable, and re-exports them plus the per-op
 * kernels through a plain C ABI for ctypes.  Built by oracle/Makefile into
 * oracle/_ref/libapus_ref.so with the reference's own flags.
 *
 * On x86-64 the reference's hot path (AVX2 rows over its pthread pool) is
 * bitwise its scalar anchor, so this one library is both the parity oracle
 * of record and the timed CPU baseline.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load this library.
 */
#define APUS_BF16_IMPLEMENTATION
#define APUS_GDN_IMPLEMENTATION
#define APUS_ATTN_IMPLEMENTATION
#define APUS_MOE_IMPLEMENTATION
#define APUS_LAYER_IMPLEMENTATION
#include "bf16.h"
#include "gdn.h"
#include "attn.h"
#include "moe.h"
#include "layer.h"

#include <string.h>

#define REF_API __attribute__((visibility("default")))

REF_API int ref_pool_threads(void) { return apus_pool_threads(); }
REF_API int ref_have_avx2(void) {
#if APUS_X86
    return apus_x86_have_avx2();
#else
    return 0;
#endif
}

REF_API float ref_bf16_f32(uint16_t b) { return apus_bf16_f32(b); }
REF_API uint16_t ref_bf16_bits(float x) { return apus_bf16_bits(x); }

REF_API void ref_bf16_gemv_scalar(const uint16_t *w, const uint16_t *x,
                                  uint16_t *y, size_t O, size_t K) {
    apus_bf16_gemv_scalar(w, x, y, O, K);
}
REF_API void ref_bf16_gemm_scalar(const uint16_t *w, const uint16_t *x,
                                  uint16_t *y, size_t M, size_t O, size_t K) {
    apus_bf16_gemm_scalar(w, x, y, M, O, K);
}
/* Hot wrappers: these consult apus_backend_hooks first (c/bf16.h:199-231). */
REF_API void ref_bf16_gemv_hot(const uint16_t *w, const uint16_t *x,
                               uint16_t *y, size_t O, size_t K) {
    ApusScratchMark mk = apus_scratch_mark();
    apus_bf16_gemv_hot(w, x, y, O, K);
    apus_scratch_reset(mk);
}
REF_API void ref_bf16_gemm_hot(const uint16_t *w, const uint16_t *x,
                               uint16_t *y, size_t M, size_t O, size_t K) {
    ApusScratchMark mk = apus_scratch_mark();
    apus_bf16_gemm_hot(w, x, y, M, O, K);
    apus_scratch_reset(mk);
}
REF_API void ref_matvec_f32(const uint16_t *w, const uint16_t *x, float *y,
                            size_t O, size_t K) {
    apus_moe_matvec_f32(w, x, y, O, K);
}
REF_API void ref_matvec_f32_hot(const uint16_t *w, const uint16_t *x,
                                float *y, size_t O, size_t K) {
    ApusScratchMark mk = apus_scratch_mark();
    apus_moe_matvec_f32_hot(w, x, y, O, K);
    apus_scratch_reset(mk);
}

REF_API void ref_moe_route(const uint16_t *x, const uint16_t *wg,
                           int32_t *idx, uint16_t *w, size_t E, size_t K,
                           size_t topk) {
    ApusScratchMark mk = apus_scratch_mark();
    apus_moe_route(x, wg, idx, w, E, K, topk);
    apus_scratch_reset(mk);
}
REF_API void ref_moe_route_topn(const uint16_t *x, const uint16_t *wg,
                                int32_t *idx, size_t n, size_t E, size_t K) {
    ApusScratchMark mk = apus_scratch_mark();
    apus_moe_route_topn(x, wg, idx, n, E, K);
    apus_scratch_reset(mk);
}
REF_API void ref_moe_silu_act(const uint16_t *gu, uint16_t *act, size_t I) {
    apus_moe_silu_act(gu, act, I);
}
REF_API void ref_moe_silu_mul(const uint16_t *g, const uint16_t *u,
                              uint16_t *y, size_t I) {
    apus_moe_silu_mul(g, u, y, I);
}
REF_API void ref_moe_combine(const uint16_t *y, const uint16_t *w,
                             uint16_t *out, size_t k, size_t N) {
    apus_moe_combine(y, w, out, k, N);
}
REF_API void ref_rmsnorm(const uint16_t *x, const uint16_t *w, uint16_t *y,
                         size_t N) {
    apus_attn_rmsnorm(x, w, y, N);
}
REF_API void ref_resadd(const uint16_t *a, const uint16_t *b, uint16_t *out,
                        size_t n) {
    apus_layer_resadd(a, b, out, n);
}

/* The MoE block.  batched=0: T calls of the per-token body (the decode
 * path); batched=1: one call of the T>1 prefill body.  Trace pointers may be
 * NULL.  Arguments mirror ApusLayerCfg / ApusLayerW / ApusLayerTrace MoE
 * fields (c/layer.h:129-130,150-156,186-188). */
REF_API void ref_moe_block(size_t H, size_t E, size_t I, size_t Is, size_t TK,
                           const uint16_t *rtr_w, const uint16_t *exp_gu,
                           const uint16_t *exp_d, const uint16_t *sh_g,
                           const uint16_t *sh_u, const uint16_t *sh_d,
                           const uint16_t *sh_gate, const uint16_t *ln2,
                           uint16_t *moe_out, size_t T, int batched,
                           int32_t *tr_idx, uint16_t *tr_w,
                           uint16_t *tr_routed, uint16_t *tr_shared) {
    ApusLayerCfg c;
    ApusLayerW w;
    ApusLayerTrace tr;
    memset(&c, 0, sizeof c);
    memset(&w, 0, sizeof w);
    memset(&tr, 0, sizeof tr);
    c.hidden = H;
    c.experts = E;
    c.moe_inter = I;
    c.shared_inter = Is;
    c.top_k = TK;
    w.rtr_w = rtr_w;
    w.exp_gu = exp_gu;
    w.exp_d = exp_d;
    w.sh_g = sh_g;
    w.sh_u = sh_u;
    w.sh_d = sh_d;
    w.sh_gate = sh_gate;
    tr.rtr_idx = tr_idx;
    tr.rtr_w = tr_w;
    tr.moe_routed = tr_routed;
    tr.moe_shared = tr_shared;
    ApusScratchMark mk = apus_scratch_mark();
    if (batched) {
        apus_layer_moe_batch(&c, &w, ln2, moe_out, T, &tr);
    } else {
        for (size_t t = 0; t < T; t++) {
            ApusScratchMark m2 = apus_scratch_mark();
            apus_layer_moe(&c, &w, ln2 + t * H, moe_out + t * H, &tr, t);
            apus_scratch_reset(m2);
        }
    }
    apus_scratch_reset(mk);
}

/* Drop-in check: install a backend's three hook functions into the
 * reference's own table (c/bf16.h:248, c/backend_metal.h:79-88), after which
 * every ref_*_hot / ref_moe_block call above dispatches through them exactly
 * as the engine would.  NULL clears a slot. */
REF_API void ref_set_hooks(
    int (*gemv)(const uint16_t *, const uint16_t *, uint16_t *, size_t,
                size_t),
    int (*gemm)(const uint16_t *, const uint16_t *, uint16_t *, size_t,
                size_t, size_t),
    int (*matvec)(const uint16_t *, const uint16_t *, float *, size_t,
                  size_t)) {
    apus_backend_hooks.bf16_gemv = gemv;
    apus_backend_hooks.bf16_gemm = gemm;
    apus_backend_hooks.bf16_matvec_f32 = matvec;
}
