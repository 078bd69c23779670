/*
 * apus_cuda_glue.h — the engine-side glue for the CUDA backend: the few lines
 * the apus-qwen engine adds to dispatch its MoE block into libapus_cuda.
 * Header-only C11, included by the engine AFTER its own layer.h (it uses
 * ApusLayerCfg / ApusLayerW / ApusLayerTrace, c/layer.h:113-189) and after
 * backend_cuda.h.
 *
 *   apus_layer_moe_cuda()    the shim called on the first line of
 *                            apus_layer_moe (c/layer.h:333) and
 *                            apus_layer_moe_batch (c/layer.h:570):
 *                                if (!apus_layer_moe_cuda(c, w, ln2, moe_out,
 *                                                         T, tr, t0)) return;
 *                            It returns 1 when the block hook is not installed
 *                            (the CPU code then runs as before) and 0 when the
 *                            GPU produced moe_out and the trace rows.
 *
 *   APUS_CUDA_GLUE_WEAK_STUBS  define it in ONE translation unit (the engine
 *                            does so in its bf16 TU, next to the Metal stubs,
 *                            c/bf16.h:243-259) to get weak definitions of the
 *                            lifecycle entry points and of the block hook
 *                            table, so a binary built without the CUDA library
 *                            still links and says "not compiled in".
 *
 * Error policy: the engine silently falls back to its CPU kernel when one of
 * the three per-matmul hooks returns nonzero (c/backend_metal.h:65-67).  The
 * block operator is different: once the hook is installed, a failure is a hard
 * error (message, exit status 2) — there is no silent CPU path for the block.
 */
#ifndef APUS_CUDA_GLUE_H
#define APUS_CUDA_GLUE_H

#include <stdio.h>
#include <stdlib.h>

#include "backend_cuda.h"

#ifdef APUS_CUDA_GLUE_WEAK_STUBS
__attribute__((weak)) int apus_cuda_enable(char *err, size_t errcap) {
    if (err && errcap) snprintf(err, errcap, "cuda backend not compiled in");
    return -1;
}
__attribute__((weak)) void apus_cuda_disable(void) {}
__attribute__((weak)) int apus_cuda_is_enabled(void) { return 0; }
__attribute__((weak)) uint64_t apus_cuda_bytes_resident(void) { return 0; }
__attribute__((weak)) uint64_t apus_cuda_bytes_uploaded(void) { return 0; }
__attribute__((weak)) uint64_t apus_cuda_launches(void) { return 0; }
__attribute__((weak)) const char *apus_cuda_last_error(void) {
    return "cuda backend not compiled in";
}
__attribute__((weak)) int apus_cuda_moe_route_topn(const uint16_t *x, const uint16_t *wg,
                                                   int32_t *idx, size_t n, size_t E,
                                                   size_t K) {
    (void)x; (void)wg; (void)idx; (void)n; (void)E; (void)K;
    return 1;
}
__attribute__((weak)) ApusCudaBlockHooks apus_cuda_block_hooks;
#endif

/* ln2 [T,H] -> moe_out [T,H]; tr (optional) is the caller's trace with room
 * for its whole sequence, this call's rows starting at token t0 (the
 * per-token body passes T = 1 and its token index, c/layer.h:362-369; the
 * batched body passes t0 = 0, c/layer.h:636-650). */
static inline int apus_layer_moe_cuda(const ApusLayerCfg *c, const ApusLayerW *w,
                                      const uint16_t *ln2, uint16_t *moe_out,
                                      size_t T, ApusLayerTrace *tr, size_t t0) {
    if (!apus_cuda_block_hooks.moe_block) return 1;
    ApusCudaMoeCfg cc = { c->hidden, c->experts, c->moe_inter,
                          c->shared_inter, c->top_k };
    ApusCudaMoeW ww = { w->rtr_w, w->exp_gu, w->exp_d, w->sh_g, w->sh_u,
                        w->sh_d, w->sh_gate };
    ApusCudaMoeTrace tt = { 0, 0, 0, 0, 0 };
    if (tr) {
        const size_t H = c->hidden, K = c->top_k;
        tt.rtr_idx    = tr->rtr_idx    ? tr->rtr_idx    + t0 * K : NULL;
        tt.rtr_w      = tr->rtr_w      ? tr->rtr_w      + t0 * K : NULL;
        tt.moe_routed = tr->moe_routed ? tr->moe_routed + t0 * H : NULL;
        tt.moe_shared = tr->moe_shared ? tr->moe_shared + t0 * H : NULL;
        tt.moe_out    = tr->moe_out    ? tr->moe_out    + t0 * H : NULL;
    }
    if (apus_cuda_block_hooks.moe_block(&cc, &ww, ln2, moe_out, T,
                                        tr ? &tt : NULL)) {
        fprintf(stderr, "cuda moe_block: %s\n", apus_cuda_last_error());
        exit(2);                      /* hard error: no silent CPU path */
    }
    return 0;
}

/* The tiered mirrors (c/cache.h:1498 apus_store_moe, :1659 apus_store_prefill)
 * call this on their first line, exactly as the eager functions call the shim
 * above: in tiered mode w->exp_gu / exp_d are NULL, and the layer must have been
 * registered once at load with apus_cuda_register_layer_slabs (experts read from
 * the container the store would have streamed from).  rtr_idx, when the store's
 * router_actual hook wants the selection (c/cache.h:1510-1512), comes back
 * through tr.  Returns 1 when the block hook is not installed. */
static inline int apus_store_moe_cuda(const ApusLayerCfg *c, const ApusLayerW *w,
                                      const uint16_t *ln2, uint16_t *moe_out, size_t T,
                                      ApusLayerTrace *tr) {
    return apus_layer_moe_cuda(c, w, ln2, moe_out, T, tr, 0);
}

/* The prefetch predictor's deeper truncation of the router (c/pilot.h:280-284):
 * ids of the first n experts in selection order.  Returns 0 when the backend
 * produced them, 1 otherwise (the caller then runs apus_moe_route_topn). */
static inline int apus_moe_route_topn_cuda(const uint16_t *x, const uint16_t *wg,
                                           int32_t *idx, size_t n, size_t E, size_t K) {
    if (!apus_cuda_is_enabled()) return 1;
    return apus_cuda_moe_route_topn(x, wg, idx, n, E, K) ? 1 : 0;
}

#endif /* APUS_CUDA_GLUE_H */
