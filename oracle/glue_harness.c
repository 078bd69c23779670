/*
 * oracle/glue_harness.c — TEST INFRASTRUCTURE, not product code.
 *
 * A small host program that plays the engine: one translation unit with the
 * reference engine's own headers (from the reference checkout via -I, all
 * five *_IMPLEMENTATION macros, nothing copied) plus the engine-side glue of
 * the CUDA backend (include/apus_cuda_glue.h), linked against libapus_cuda.so
 * the way the engine's `-cuda` binary would be.  It defines the engine's hook
 * table apus_backend_hooks (c/bf16.h:248), so apus_cuda_enable fills the real
 * thing.  Built by oracle/Makefile into oracle/_ref/glue_test (and, without
 * the CUDA library and with the glue's weak stubs, oracle/_ref/glue_test_cpu).
 *
 *   glue_test block H E I Is K T t0   weights and tokens from the seeded
 *       generator; runs the engine's apus_layer_moe_batch on the CPU and the
 *       shim apus_layer_moe_cuda into a trace at row offset t0; prints one
 *       JSON object with the comparison.
 *   glue_test slots      enables the backend and prints which hook slots are
 *       filled (the APUS_CUDA_NO_* knobs leave a slot NULL).
 *   glue_test budget O K the engine's apus_bf16_gemv_hot on an O x K weight
 *       with the backend enabled: prints whether the hook produced the result
 *       (launch counter moved) and whether it is bitwise the scalar anchor.
 *       Under APUS_CUDA_DENSE_MB=1 a large weight makes the hook return
 *       nonzero and the engine falls back (c/backend_metal.h:65-67).
 *   glue_test topn E K n the predictor's router truncation (c/pilot.h:280-284)
 *       through apus_moe_route_topn_cuda against the engine's apus_moe_route_topn.
 *   glue_test stubs      (glue_test_cpu) apus_cuda_enable must fail with
 *       "not compiled in" and the shim must return 1.
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

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/backend_cuda.h"
#ifdef GLUE_CPU_ONLY
#define APUS_CUDA_GLUE_WEAK_STUBS
#endif
#include "../include/apus_cuda_glue.h"
#include "../apus-qwen3.6-35b-a3b_b200/csrc/synth.h"

static uint16_t *fill(size_t n, uint32_t tensor, double sigma) {
    uint16_t *p = malloc(n * 2);
    const uint64_t key = apus_synth_key(11, 0, tensor);
    for (size_t i = 0; i < n; i++) p[i] = apus_synth_bf16(key, i, sigma);
    return p;
}

static int cmd_block(int argc, char **argv) {
    if (argc < 9) return 2;
    ApusLayerCfg c;
    memset(&c, 0, sizeof c);
    c.hidden = (size_t)atol(argv[2]);
    c.experts = (size_t)atol(argv[3]);
    c.moe_inter = (size_t)atol(argv[4]);
    c.shared_inter = (size_t)atol(argv[5]);
    c.top_k = (size_t)atol(argv[6]);
    const size_t T = (size_t)atol(argv[7]), t0 = (size_t)atol(argv[8]);
    const size_t H = c.hidden, E = c.experts, I = c.moe_inter, Is = c.shared_inter,
                 K = c.top_k, TT = T + t0;
    ApusLayerW w;
    memset(&w, 0, sizeof w);
    w.rtr_w = fill(E * H, APUS_SYNTH_RTR_W, 0.05);
    w.exp_gu = fill(E * 2 * I * H, APUS_SYNTH_EXP_GU, 0.05);
    w.exp_d = fill(E * H * I, APUS_SYNTH_EXP_D, 0.05);
    w.sh_g = fill(Is * H, APUS_SYNTH_SH_G, 0.05);
    w.sh_u = fill(Is * H, APUS_SYNTH_SH_U, 0.05);
    w.sh_d = fill(H * Is, APUS_SYNTH_SH_D, 0.05);
    w.sh_gate = fill(H, APUS_SYNTH_SH_GATE, 0.05);
    uint16_t *x = fill(T * H, APUS_SYNTH_X, 1.0);
    /* CPU: the engine's own batched body */
    uint16_t *out_cpu = calloc(T * H, 2);
    ApusLayerTrace ta;
    memset(&ta, 0, sizeof ta);
    ta.rtr_idx = calloc(T * K, 4);
    ta.rtr_w = calloc(T * K, 2);
    ta.moe_routed = calloc(T * H, 2);
    ta.moe_shared = calloc(T * H, 2);
    ta.moe_out = calloc(T * H, 2);
    apus_layer_moe_batch(&c, &w, x, out_cpu, T, &ta);
    /* GPU through the shim, trace rows at offset t0 of a longer trace */
    char err[256] = "";
    if (apus_cuda_enable(err, sizeof err)) {
        printf("{\"error\": \"%s\"}\n", err);
        return 1;
    }
    uint16_t *out_gpu = calloc(T * H, 2);
    ApusLayerTrace tb;
    memset(&tb, 0, sizeof tb);
    tb.rtr_idx = malloc(TT * K * 4);
    tb.rtr_w = malloc(TT * K * 2);
    tb.moe_routed = malloc(TT * H * 2);
    tb.moe_shared = malloc(TT * H * 2);
    tb.moe_out = malloc(TT * H * 2);
    memset(tb.rtr_idx, 0xEE, TT * K * 4);
    memset(tb.moe_out, 0xEE, TT * H * 2);
    const int rc = apus_layer_moe_cuda(&c, &w, x, out_gpu, T, &tb, t0);
    int idx_exact = !memcmp(ta.rtr_idx, tb.rtr_idx + t0 * K, T * K * 4);
    int w_diff = 0;
    for (size_t i = 0; i < T * K; i++)
        if (ta.rtr_w[i] != tb.rtr_w[t0 * K + i]) w_diff++;
    double max_abs = 0, num = 0, den = 0, max_routed = 0, max_shared = 0;
    for (size_t i = 0; i < T * H; i++) {
        const double a = apus_bf16_f32(out_gpu[i]), b = apus_bf16_f32(out_cpu[i]);
        if (fabs(a - b) > max_abs) max_abs = fabs(a - b);
        num += (a - b) * (a - b);
        den += b * b;
        const double r = fabs(apus_bf16_f32(tb.moe_routed[t0 * H + i]) -
                              apus_bf16_f32(ta.moe_routed[i]));
        const double s = fabs(apus_bf16_f32(tb.moe_shared[t0 * H + i]) -
                              apus_bf16_f32(ta.moe_shared[i]));
        if (r > max_routed) max_routed = r;
        if (s > max_shared) max_shared = s;
    }
    /* rows before t0 untouched; trace out row == returned row */
    int before_untouched = 1;
    for (size_t i = 0; i < t0 * H; i++)
        if (tb.moe_out[i] != 0xEEEE) before_untouched = 0;
    for (size_t i = 0; i < t0 * K; i++)
        if ((uint32_t)tb.rtr_idx[i] != 0xEEEEEEEEu) before_untouched = 0;
    const int trace_out_equal = !memcmp(tb.moe_out + t0 * H, out_gpu, T * H * 2);
    printf("{\"rc\": %d, \"idx_exact\": %d, \"w_codes_differing\": %d, "
           "\"max_abs\": %.6g, \"rel_l2\": %.6g, \"max_abs_routed\": %.6g, "
           "\"max_abs_shared\": %.6g, \"rows_before_t0_untouched\": %d, "
           "\"trace_out_equals_out\": %d, \"launches\": %llu}\n",
           rc, idx_exact, w_diff, max_abs, sqrt(num / (den + 1e-30)), max_routed,
           max_shared, before_untouched, trace_out_equal,
           (unsigned long long)apus_cuda_launches());
    apus_cuda_disable();
    return 0;
}

static int cmd_slots(void) {
    char err[256] = "";
    if (apus_cuda_enable(err, sizeof err)) {
        printf("{\"error\": \"%s\"}\n", err);
        return 1;
    }
    printf("{\"gemv\": %d, \"gemm\": %d, \"matvec\": %d, \"moe\": %d, \"enabled\": %d}\n",
           apus_backend_hooks.bf16_gemv != NULL, apus_backend_hooks.bf16_gemm != NULL,
           apus_backend_hooks.bf16_matvec_f32 != NULL,
           apus_cuda_block_hooks.moe_block != NULL, apus_cuda_is_enabled());
    apus_cuda_disable();
    const int cleared = !apus_backend_hooks.bf16_gemv && !apus_backend_hooks.bf16_gemm &&
                        !apus_backend_hooks.bf16_matvec_f32 &&
                        !apus_cuda_block_hooks.moe_block;
    return cleared ? 0 : 3;
}

static int cmd_budget(int argc, char **argv) {
    if (argc < 4) return 2;
    const size_t O = (size_t)atol(argv[2]), K = (size_t)atol(argv[3]);
    char err[256] = "";
    if (apus_cuda_enable(err, sizeof err)) {
        printf("{\"error\": \"%s\"}\n", err);
        return 1;
    }
    uint16_t *wt = fill(O * K, APUS_SYNTH_RTR_W, 0.05), *x = fill(K, APUS_SYNTH_X, 1.0);
    uint16_t *y = calloc(O, 2), *ys = calloc(O, 2);
    const unsigned long long l0 = apus_cuda_launches();
    ApusScratchMark mk = apus_scratch_mark();
    apus_bf16_gemv_hot(wt, x, y, O, K);     /* hook first, CPU if it declines */
    apus_scratch_reset(mk);
    const unsigned long long l1 = apus_cuda_launches();
    apus_bf16_gemv_scalar(wt, x, ys, O, K);
    printf("{\"hook_took_it\": %d, \"bitwise_scalar\": %d, \"bytes_resident\": %llu}\n",
           l1 > l0, !memcmp(y, ys, O * 2), (unsigned long long)apus_cuda_bytes_resident());
    apus_cuda_disable();
    return 0;
}

/* the predictor's router truncation through the glue against the engine's own */
static int cmd_topn(int argc, char **argv) {
    if (argc < 5) return 2;
    const size_t E = (size_t)atol(argv[2]), K = (size_t)atol(argv[3]), n = (size_t)atol(argv[4]);
    char err[256] = "";
    if (apus_cuda_enable(err, sizeof err)) {
        printf("{\"error\": \"%s\"}\n", err);
        return 1;
    }
    uint16_t *wg = fill(E * K, APUS_SYNTH_RTR_W, 0.05), *x = fill(K, APUS_SYNTH_X, 1.0);
    int32_t a[64], b[64];
    apus_moe_route_topn(x, wg, a, n, E, K);
    const int rc = apus_moe_route_topn_cuda(x, wg, b, n, E, K);
    printf("{\"rc\": %d, \"equal\": %d, \"launches\": %llu}\n", rc,
           !memcmp(a, b, n * sizeof(int32_t)), (unsigned long long)apus_cuda_launches());
    apus_cuda_disable();
    return 0;
}

static int cmd_stubs(void) {
    char err[256] = "";
    const int rc = apus_cuda_enable(err, sizeof err);
    ApusLayerCfg c;
    ApusLayerW w;
    memset(&c, 0, sizeof c);
    memset(&w, 0, sizeof w);
    const int shim = apus_layer_moe_cuda(&c, &w, NULL, NULL, 1, NULL, 0) +
                     apus_store_moe_cuda(&c, &w, NULL, NULL, 1, NULL) - 1;
    int32_t ids[8];
    const int topn = apus_moe_route_topn_cuda(NULL, NULL, ids, 8, 16, 16);
    printf("{\"enable_rc\": %d, \"err\": \"%s\", \"shim_rc\": %d, \"topn_rc\": %d, "
           "\"enabled\": %d}\n",
           rc, err, shim, topn, apus_cuda_is_enabled());
    return 0;
}

int main(int argc, char **argv) {
    if (argc < 2) return 2;
    if (!strcmp(argv[1], "block")) return cmd_block(argc, argv);
    if (!strcmp(argv[1], "slots")) return cmd_slots();
    if (!strcmp(argv[1], "budget")) return cmd_budget(argc, argv);
    if (!strcmp(argv[1], "stubs")) return cmd_stubs();
    if (!strcmp(argv[1], "topn")) return cmd_topn(argc, argv);
    return 2;
}
