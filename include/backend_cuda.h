/*
 * backend_cuda.h — CUDA (NVIDIA B200, sm_100a) backend for the MoE block of
 * the apus-qwen engine.  Pure C11 interface; the implementation is
 * backend_cuda.cu.  It sits beside the engine's c/backend_metal.h and keeps
 * that header's conventions: plain pointers and sizes, BF16 as uint16_t
 * codes, row-major tensors, `0` = "produced the result", nonzero =
 * "unsupported / failed" (c/backend_metal.h:65-67), host buffers owned by the
 * caller, weights never written or freed by the backend.
 *
 * Two layers of entry points:
 *
 *  1. The engine's three per-matmul hooks (c/backend_metal.h:79-86), host
 *     pointers, synchronous.  Their kernels accumulate in the engine's
 *     normative order (ascending k, one fp32 rounding per step), so a taken
 *     hook is bit-identical to the engine's x86 CPU dispatch.
 *
 *  2. The MoE block as ONE operator (router -> top-k -> dispatch -> routed
 *     SwiGLU experts + shared expert -> weighted combine), which is what
 *     c/layer.h:333-370 (one token) and c/layer.h:570-651 (T tokens) assemble
 *     from 21 separate matmul calls.  Host-pointer form for the drop-in,
 *     device-pointer form (weights resident in HBM) for serving and
 *     benchmarks.
 *
 * Numerics of the block operator: router logits, softmax, selection and
 * renormalisation follow c/moe.h:321-371 exactly (selected expert ids and the
 * dispatch permutation are bit-exact); expert products accumulate in fp32 in
 * a different order than the CPU anchor and keep every BF16 rounding point of
 * c/moe.h:25-55 and c/layer.h:356-361, so outputs agree to BF16 tolerance
 * (max-abs 2e-2, relative L2 1e-2), not bitwise.
 *
 * There is no CPU fallback inside this library: if no usable GPU is present
 * every compute entry point returns nonzero and apus_cuda_enable fails.
 *
 * Threading: entry points serialise on one mutex per process (the engine may
 * call hooks from its forward thread and its prefetch-prediction thread at
 * the same time, c/backend_metal.mm:202-207).
 */
#ifndef APUS_BACKEND_CUDA_H
#define APUS_BACKEND_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------
 * Lifecycle and counters — mirror apus_metal_enable / _disable / _is_enabled
 * and the three counters (c/backend_metal.h:95-104).
 * ---------------------------------------------------------------------- */

/* Initialise the device (APUS_CUDA_DEVICE, default 0), create the stream and
 * the weight-residency table, and, when the engine's hook table
 * `apus_backend_hooks` is linked into the process, fill its three slots
 * (APUS_CUDA_NO_GEMV / _NO_GEMM / _NO_MATVEC leave a slot NULL, as
 * c/backend_metal.mm:490-495 does for Metal).  Also fills
 * apus_cuda_block_hooks unless APUS_CUDA_NO_MOE is set.  Returns 0 on
 * success; -1 with a message in err otherwise.  Idempotent. */
int  apus_cuda_enable(char *err, size_t errcap);
/* Zero the hook tables and release every device allocation (weight cache,
 * registered layers created through the host-pointer path, workspaces).
 * Call before freeing model weights. */
void apus_cuda_disable(void);
int  apus_cuda_is_enabled(void);

/* Weight bytes resident in HBM / copied host->device so far / kernels
 * launched so far.  (Metal's "wrapped" zero-copy counter has no CUDA
 * counterpart: every weight is a copy in HBM.) */
uint64_t apus_cuda_bytes_resident(void);
uint64_t apus_cuda_bytes_uploaded(void);
uint64_t apus_cuda_launches(void);
/* Text of the last error recorded by any entry point ("" if none). */
const char *apus_cuda_last_error(void);

/* ------------------------------------------------------------------------
 * Per-matmul entry points — same signatures and layouts as the hook slots
 * (c/backend_metal.h:80-85) and as the direct entry points
 * apus_metal_bf16_gemv / _gemm / _matvec_f32 (c/backend_metal.h:109-114).
 * w [O,K], x [M,K], y [M,O]; HOST pointers; synchronous.  The weight pointer
 * is the residency key: first sight uploads O*K*2 bytes, later calls reuse
 * the copy (stable-pointer rule, c/backend_metal.h:42-48).  Budget:
 * APUS_CUDA_DENSE_MB (default: unlimited); past it the call returns 1.
 * Zero dimensions return 1 (c/backend_metal.mm:323).
 * ---------------------------------------------------------------------- */
int apus_cuda_bf16_gemv(const uint16_t *w, const uint16_t *x, uint16_t *y,
                        size_t O, size_t K);
int apus_cuda_bf16_gemm(const uint16_t *w, const uint16_t *x, uint16_t *y,
                        size_t M, size_t O, size_t K);
int apus_cuda_bf16_matvec_f32(const uint16_t *w, const uint16_t *x, float *y,
                              size_t O, size_t K);

/* ------------------------------------------------------------------------
 * Router and dispatch on their own (host pointers; for kernel-level tests
 * and for the engine's second caller of the router, c/pilot.h:282-288).
 * ---------------------------------------------------------------------- */

/* apus_moe_route (c/moe.h:357-371) over T tokens: x [T,K], wg [E,K] ->
 * idx [T,topk] (selection order), w [T,topk] BF16.  logits [T,E] BF16 is
 * optional (NULL to skip).  E <= 1024, topk <= 32, topk <= E. */
int apus_cuda_moe_route(const uint16_t *x, const uint16_t *wg, int32_t *idx,
                        uint16_t *w, uint16_t *logits, size_t T, size_t E,
                        size_t K, size_t topk);
/* apus_moe_route_topn (c/moe.h:373-383): first n ids, no weights. */
int apus_cuda_moe_route_topn(const uint16_t *x, const uint16_t *wg,
                             int32_t *idx, size_t n, size_t E, size_t K);
/* The dispatch order c/layer.h:599-606,614-620 implies: stable counting sort
 * of the flat assignments a = t*topk + j by expert id.  idx [T*topk] ->
 * counts [E], offsets [E+1], perm [T*topk]. */
int apus_cuda_moe_dispatch(const int32_t *idx, size_t T, size_t topk,
                           size_t E, int32_t *counts, int32_t *offsets,
                           int32_t *perm);

/* ------------------------------------------------------------------------
 * The MoE block operator.
 * ---------------------------------------------------------------------- */

/* MoE fields of ApusLayerCfg (c/layer.h:115,129-130). */
typedef struct {
    size_t hidden;        /* H  (2048) */
    size_t experts;       /* E  (256)  */
    size_t moe_inter;     /* I  (512)  */
    size_t shared_inter;  /* Is (512)  */
    size_t top_k;         /* 8 */
} ApusCudaMoeCfg;

/* MoE fields of ApusLayerW (c/layer.h:150-156). */
typedef struct {
    const uint16_t *rtr_w;    /* [E, H] */
    const uint16_t *exp_gu;   /* [E, 2I, H] fused gate|up */
    const uint16_t *exp_d;    /* [E, H, I] */
    const uint16_t *sh_g;     /* [Is, H] */
    const uint16_t *sh_u;     /* [Is, H] */
    const uint16_t *sh_d;     /* [H, Is] */
    const uint16_t *sh_gate;  /* [1, H] */
} ApusCudaMoeW;

/* MoE fields of ApusLayerTrace (c/layer.h:186-188); every member optional. */
typedef struct {
    int32_t  *rtr_idx;      /* [T, top_k] */
    uint16_t *rtr_w;        /* [T, top_k] */
    uint16_t *moe_routed;   /* [T, H] */
    uint16_t *moe_shared;   /* [T, H] */
    uint16_t *moe_out;      /* [T, H] */
} ApusCudaMoeTrace;

/* Host-pointer block operator: argument meaning identical to
 * apus_layer_moe_batch (c/layer.h:570-573).  The layer's weights are uploaded
 * on first sight of w->rtr_w (the residency key) and stay in HBM until
 * apus_cuda_disable (exp_gu / exp_d may be NULL for a layer registered with
 * apus_cuda_register_layer_slabs).  Synchronous: moe_out and the trace rows are complete on
 * return.  T == 0 writes nothing and succeeds, as the engine's loops over T do.
 * From APUS_CUDA_HOST_SPLIT_T tokens (default 4096; 0: never) the call runs as
 * two half calls whose PCIe copies overlap the other half's kernels: the same
 * bits, since a token's result does not depend on its neighbours.
 * Returns 0, or nonzero with apus_cuda_last_error() set. */
int apus_cuda_moe_block(const ApusCudaMoeCfg *c, const ApusCudaMoeW *w,
                        const uint16_t *ln2, uint16_t *moe_out, size_t T,
                        const ApusCudaMoeTrace *tr);

/* The engine's tiered mode keeps no expert arrays on the host (exp_gu / exp_d
 * are NULL, c/model.h:499-503) and resolves experts from its NVMe store inside
 * the mirrors apus_store_moe / apus_store_prefill (c/cache.h:1498-1545,
 * 1659-1779).  With every expert resident in HBM that store has nothing left to
 * do: register each layer once — router, shared expert and gate from the host
 * pointers of w, the routed experts read from the weight container's slabs
 * (apus_cuda_layer_load_slabs) — and apus_cuda_moe_block then serves it under
 * the same key w->rtr_w with exp_gu / exp_d NULL.  Idempotent per key. */
int apus_cuda_register_layer_slabs(const ApusCudaMoeCfg *c, const ApusCudaMoeW *w,
                                   const char *container_dir, int layer_index);

/* Second hook table, for the block operator.  Kept apart from the engine's
 * three-slot table so that table's layout is untouched.  The engine-side
 * glue tests `apus_cuda_block_hooks.moe_block` at the top of apus_layer_moe
 * and apus_layer_moe_batch. */
typedef struct {
    int (*moe_block)(const ApusCudaMoeCfg *c, const ApusCudaMoeW *w,
                     const uint16_t *ln2, uint16_t *moe_out, size_t T,
                     const ApusCudaMoeTrace *tr);
} ApusCudaBlockHooks;
extern ApusCudaBlockHooks apus_cuda_block_hooks;

/* ---- device-resident form ------------------------------------------------ */

typedef struct ApusCudaLayer ApusCudaLayer;   /* one layer's MoE weights in HBM */

/* Allocate HBM for one layer's MoE weights and, if w is not NULL, upload
 * them.  Experts [expert_begin, expert_end) are made resident (pass 0, E for
 * all of them); router, shared expert and shared gate always are.  With
 * w == NULL the tensors are left uninitialised for apus_cuda_layer_tensor +
 * a device-side fill. */
int apus_cuda_layer_create(const ApusCudaMoeCfg *c, const ApusCudaMoeW *w,
                           size_t expert_begin, size_t expert_end,
                           ApusCudaLayer **out);
void apus_cuda_layer_destroy(ApusCudaLayer *layer);
/* Device pointer and element count of one tensor of the layer: which = 1
 * rtr_w, 2 exp_gu (first resident expert), 3 exp_d, 4 sh_g, 5 sh_u, 6 sh_d,
 * 7 sh_gate. */
void *apus_cuda_layer_tensor(ApusCudaLayer *layer, int which, size_t *elems);
/* Call after writing rtr_w through apus_cuda_layer_tensor: rescans the
 * router weights for the magnitude bound the router kernel's fast path
 * depends on. */
int apus_cuda_layer_refresh(ApusCudaLayer *layer);
/* Copy n BF16 elements from host memory into tensor `which` of the layer,
 * starting at element `first` of the resident part (ids as for
 * apus_cuda_layer_tensor).  Synchronous set-up call; the engine's eager load
 * fills exp_gu / exp_d expert by expert like this (c/model.h:505-537).
 * Writing rtr_w or sh_gate refreshes the router statistics. */
int apus_cuda_layer_upload(ApusCudaLayer *layer, int which, const uint16_t *src,
                           size_t first, size_t n);
/* Fill exp_gu / exp_d of the layer's resident expert range straight from the
 * engine's weight container in `container_dir`: the manifest apus.index.json
 * (format_version 2) locates each expert's slab {gate_up [2I,H] | down [H,I]}
 * by {layer, expert, shard, offset, nbytes} (c/cache.h:13-23); each slab is
 * read once into pinned staging and copied to HBM.  Takes the place of the
 * engine's eager load, which concatenates all experts of a layer into two host
 * arrays first (c/model.h:505-537); a rank of an expert-parallel server reads
 * only its own experts.  Router, shared expert and shared gate still come
 * through apus_cuda_layer_create / _upload.  Synchronous.  Nonzero with
 * apus_cuda_last_error() set on a missing or malformed manifest, a version
 * other than 2, a missing record or a slab of the wrong size. */
int apus_cuda_layer_load_slabs(ApusCudaLayer *layer, const char *container_dir,
                               int layer_index);

/* The block on device pointers: d_ln2 [T,H] -> d_out [T,H]; d_tr members are
 * device pointers (or NULL).  Enqueued on `stream` (a cudaStream_t; NULL is the
 * CUDA default stream, as everywhere in this header); does not synchronise.
 *
 * Path selection: T <= APUS_CUDA_FUSED_MAX_T (default and maximum 4) runs the
 * whole block as one cooperative kernel; larger T runs router -> dispatch ->
 * tcgen05 grouped GEMMs (gate/up, down) -> combine when the shape fits the MMA
 * tiles (H, I, Is multiples of 128, Is == I), else the grouped-GEMV kernels.
 * APUS_CUDA_DECODE_MAX_T (default 4) is the largest T that still takes the
 * grouped-GEMV kernels on a shape the GEMM supports.  From a mean of
 * APUS_CUDA_PAIR_MIN_ROWS (default 192) rows per expert on, and H a multiple of
 * 256, the two GEMMs run with a pair of SMs per tile (cta_group::2: tokens
 * 256 per pair, each SM loading half of the weight tile); APUS_CUDA_PAIR=0
 * keeps the one-SM kernels.
 *
 * Shared state.  Every device-pointer entry point of this header (the block,
 * the expert-parallel steps, route_dev, dispatch_dev) works in ONE per-process
 * workspace with one status word, whatever stream it is given.  The library
 * therefore orders a call behind the previous call when it arrives on a
 * different stream (an event wait on the device; no host synchronisation), so
 * calls from two streams or two threads are serialised on the GPU, not raced.
 * Inside a stream capture no such event is recorded or waited for: graphs
 * captured from these calls must be replayed in one stream order by the caller.
 *
 * Workspace growth.  The arena grows on demand; growth synchronises the device
 * and is refused (nonzero return) while `stream` is capturing.  Call
 * apus_cuda_reserve for the largest T first to keep both out of a timed region
 * or a capture.  An outgrown arena is kept allocated until apus_cuda_disable,
 * so a graph captured earlier stays valid after later, larger calls. */
int apus_cuda_moe_block_dev(ApusCudaLayer *layer, const uint16_t *d_ln2,
                            uint16_t *d_out, size_t T,
                            const ApusCudaMoeTrace *d_tr, void *stream);
/* The block with the two steps either side of it folded in (c/layer.h:386-388):
 *     d_res_out = rnd(d_res + moe_block(rmsnorm(d_res, gain 1 + d_ln_w)))
 * d_res [T,H] is the residual stream after the attention half, d_ln_w [H] the
 * post-attention norm's gain offsets (NULL = zero).  Norm and add are bit for
 * bit the engine's (c/attn.h:175-186, c/layer.h:230-234).  Up to
 * APUS_CUDA_FUSED_MAX_T tokens all of it is the one cooperative kernel (every
 * CTA normalises the tokens for itself; the add is in the combine): no extra
 * launch.  Above, the norm is one launch of its own and the add is part of the
 * combine kernel.  d_res_out may equal d_res.  d_tr->moe_out receives the
 * block's own output. */
int apus_cuda_moe_layer_dev(ApusCudaLayer *layer, const uint16_t *d_res,
                            const uint16_t *d_ln_w, uint16_t *d_res_out, size_t T,
                            const ApusCudaMoeTrace *d_tr, void *stream);
/* n_layers of the above back to back on one residual stream, in place:
 * d_res <- d_res + moe_l(rmsnorm(d_res, 1 + d_ln_w[l])) for l = 0 .. n_layers-1
 * (d_ln_w NULL, or an entry NULL = zero gain offsets).  The MoE half of a
 * decode step over a stack of layers as one call (and one CUDA graph when
 * captured). */
int apus_cuda_moe_stack_dev(ApusCudaLayer *const *layers, const uint16_t *const *d_ln_w,
                            size_t n_layers, uint16_t *d_res, size_t T, void *stream);
/* Grow the workspace arena for blocks of up to T tokens of this shape (and
 * allocate the one-kernel path's scratch for it). */
int apus_cuda_reserve(const ApusCudaMoeCfg *c, size_t T);
/* Kernels one apus_cuda_moe_block_dev call launched last time (for the
 * benchmark's launch count). */
int apus_cuda_last_block_launches(void);
/* Which kernels the last apus_cuda_moe_block[_dev] call took (-1: none yet). */
enum {
    APUS_CUDA_PATH_FUSED = 0,      /* one cooperative kernel (a handful of tokens) */
    APUS_CUDA_PATH_GEMV = 1,       /* grouped-GEMV kernels (shapes the MMA tiles do not fit) */
    APUS_CUDA_PATH_GEMM = 2,       /* tcgen05 grouped GEMM, one SM per tile */
    APUS_CUDA_PATH_GEMM_2SM = 3    /* tcgen05 grouped GEMM, a pair of SMs per tile */
};
int apus_cuda_last_block_path(void);
/* Per-stage device times of the block (benchmarks): with timing enabled,
 * apus_cuda_moe_block_dev brackets each stage with CUDA events on the stream
 * it launches on; apus_cuda_last_stage_ms waits for the last call's events
 * and fills ms[stage] (milliseconds, indexed by the enum below), returning
 * the number of intervals measured or -1. */
enum {
    APUS_CUDA_STAGE_ROUTER = 0,    /* fused router + top-k + shared-gate logit */
    APUS_CUDA_STAGE_DISPATCH = 1,  /* histogram, scan, stable permute */
    APUS_CUDA_STAGE_GATHER = 2,    /* prefill: permuted activation rows */
    APUS_CUDA_STAGE_GATE_UP = 3,   /* gate/up products + SwiGLU */
    APUS_CUDA_STAGE_DOWN = 4,      /* down products */
    APUS_CUDA_STAGE_FINALIZE = 5,  /* weighted combine + shared + add */
    APUS_CUDA_STAGE_COUNT = 6
};
int apus_cuda_stage_timing(int enable);
int apus_cuda_last_stage_ms(float *ms, int cap);
/* Diagnostic for the one-kernel path (T <= 4): with stage timing enabled each
 * CTA stamps the device's global timer (ns) at its eight phase boundaries;
 * this copies out[cta*8 + mark] for the last call and returns the number of
 * values written, or -1 if the last call did not take that path. */
int apus_cuda_fused_timeline(unsigned long long *out, int cap);
/* Diagnostic for the many-token router: it scores every expert with a fast
 * tensor-core product and walks the engine's exact sequential chain
 * (c/moe.h:289-291) only for the experts whose fast logit, widened by a proven
 * error bound, can still reach the top_k.  Returns how many exact chains have
 * run since enable (256 per token would be the plain exact router), -1 when
 * not enabled.  APUS_CUDA_ROUTER_CERTIFY=0 selects the plain exact router. */
long apus_cuda_router_exact_chains(void);
/* Diagnostic: phase boundaries of the many-token router's first CTA in its
 * last launch, out[0..3] = start, candidates known, exact chains done, end
 * (nanoseconds, low 32 bits of the device's global timer), out[4] = chains that
 * CTA walked.  Returns 0, or -1 when not enabled. */
int apus_cuda_router_timeline(unsigned int *out);
/* Diagnostic for the same router (host pointers, synchronous): the fast
 * tensor-core logits of every (token, expert) pair, fast [T,E] fp32, summed
 * over the K slices as the router does, together with the three factors of
 * the error bound it relies on: |fast - exact chain| <= cbound * xnorm[t] *
 * wnorm[e] (wnorm [E+1], the last entry the largest).  Tests compare this
 * with the engine's exact fp32 chain on every pair.  E % 128 == 0,
 * K % 256 == 0. */
int apus_cuda_debug_fast_logits(const uint16_t *x, const uint16_t *wg, size_t T,
                                size_t E, size_t K, float *fast, float *xnorm,
                                float *wnorm, float *cbound);

/* Device-side status word of the last block call: 0 = ok; nonzero = a
 * bounded wait inside a kernel gave up (the context stays usable). */
int apus_cuda_last_block_status(void);

/* ---- expert parallelism -----------------------------------------------------
 * Net-new: the reference engine is one process (no counterpart beyond the
 * math of c/layer.h:570-651).  A rank holds experts [begin, end) of every
 * layer (apus_cuda_layer_create) plus the replicated router, shared expert and
 * shared gate, and owns a slice of the tokens.  One block step on a rank:
 *
 *   1. apus_cuda_ep_route_dev   router on the rank's tokens -> idx, w, sgl
 *   2. apus_cuda_ep_pack_dev    stable sort of the T*topk assignments by
 *                               owning rank; packs the rows to send
 *   3. all-to-all of (row, expert id) — the caller's collective (NCCL)
 *   4. apus_cuda_experts_dev    the resident experts on the received rows
 *   5. all-to-all of the BF16 expert outputs back — the caller's collective
 *   6. apus_cuda_ep_finish_dev  shared expert on the rank's tokens, weighted
 *                               combine in slot order, gate, add
 *
 * Every assignment's expert output is rounded to BF16 exactly where the
 * single-GPU block rounds it, and step 6 combines in the same slot order, so
 * the result equals apus_cuda_moe_block_dev bit for bit at any rank count.
 * All pointers are device pointers; calls enqueue on `stream` and do not
 * synchronise. */

/* d_x [T,H] -> d_idx [T,topk], d_w [T,topk] BF16, d_sgl [T] BF16 (the shared
 * gate logit, c/layer.h:355). */
int apus_cuda_ep_route_dev(ApusCudaLayer *layer, const uint16_t *d_x, size_t T,
                           int32_t *d_idx, uint16_t *d_w, uint16_t *d_sgl,
                           void *stream);
/* Owner of expert e is e / (E / n_ranks).  Outputs, all in send order p (rank
 * 0's rows first, inside a rank by token then slot): d_send_x [T*topk, H] (the
 * token row of assignment p), d_send_e [T*topk] (its global expert id),
 * d_send_counts [n_ranks], d_pos [T*topk] (send position of flat assignment
 * t*topk + j). */
int apus_cuda_ep_pack_dev(const uint16_t *d_x, const int32_t *d_idx, size_t T,
                          size_t topk, size_t H, size_t E, size_t n_ranks,
                          uint16_t *d_send_x, int32_t *d_send_e,
                          int32_t *d_send_counts, int32_t *d_pos, void *stream);
/* d_y[r] = rnd(Wd[e_r] . act(Wgu[e_r] . d_x[r])) for R rows, e_r = d_e[r] a
 * global id inside the layer's resident range (c/layer.h:346-348 per row).
 * R == 0 is a no-op. */
int apus_cuda_experts_dev(ApusCudaLayer *layer, const uint16_t *d_x,
                          const int32_t *d_e, size_t R, uint16_t *d_y,
                          void *stream);
/* d_y_sorted [T*topk, H]: expert outputs in send order; d_pos from step 2;
 * d_w, d_sgl from step 1.  Writes d_out [T,H] (and the trace rows). */
int apus_cuda_ep_finish_dev(ApusCudaLayer *layer, const uint16_t *d_x, size_t T,
                            const uint16_t *d_y_sorted, const int32_t *d_pos,
                            const uint16_t *d_w, const uint16_t *d_sgl,
                            uint16_t *d_out, const ApusCudaMoeTrace *d_tr,
                            void *stream);

/* ---- expert parallelism without a collective library on the data path ------
 * Net-new (no reference counterpart).  Steps 2, 3 and 5 above as kernels that
 * store straight into the peers' memory over NVLink, with no host
 * synchronisation inside a step.  Every rank creates one window (a device
 * allocation holding, per source rank, a region of max_tokens*topk rows and
 * their expert ids, plus the rows returned to it), publishes its CUDA IPC
 * handle, and attaches every peer's.  One block step with epoch e (a counter
 * the caller increments per step, the same on all ranks, starting at 1):
 *
 *   apus_cuda_ep_route_dev          idx, w, sgl of the rank's tokens
 *   apus_cuda_ep_push_dev           rows and ids into the owners' windows;
 *                                   d_pos as in apus_cuda_ep_pack_dev
 *   apus_cuda_ep_shared_dev         shared expert (overlaps the peers' pushes)
 *   apus_cuda_ep_wait_dev(0, e)     every source's push has landed here
 *   apus_cuda_ep_window_experts_dev resident experts on the received rows
 *   apus_cuda_ep_return_dev         outputs into the senders' windows
 *   apus_cuda_ep_wait_dev(1, e)     every peer's return has landed here
 *   apus_cuda_ep_combine_dev        weighted sum in slot order, gate, add
 *
 * With epoch 0 in every call the step number is kept on the device (a push opens
 * the next step), so the eight calls can be captured once in a CUDA graph and
 * replayed.
 * All ranks must run the same sequence of steps.  Waits are bounded (about two
 * seconds); one that runs out sets apus_cuda_last_block_status() to 6 and the
 * step's output is not valid, but the context stays usable.  The result equals
 * apus_cuda_moe_block_dev bit for bit, as for the collective-based steps. */
typedef struct ApusCudaEpWindow ApusCudaEpWindow;
int apus_cuda_ep_window_create(size_t max_tokens, size_t topk, size_t H, size_t E,
                               size_t n_ranks, size_t rank, ApusCudaEpWindow **out);
void apus_cuda_ep_window_destroy(ApusCudaEpWindow *w);
/* size of the opaque handle a rank publishes (a CUDA IPC memory handle) */
size_t apus_cuda_ep_window_handle_bytes(void);
int apus_cuda_ep_window_handle(ApusCudaEpWindow *w, void *out_handle);
/* map the window of rank `peer` (another process on this node) */
int apus_cuda_ep_window_attach(ApusCudaEpWindow *w, size_t peer, const void *handle);
/* the same for a window created in this process (several ranks per process) */
int apus_cuda_ep_window_attach_local(ApusCudaEpWindow *w, size_t peer,
                                     ApusCudaEpWindow *other);
int apus_cuda_ep_push_dev(ApusCudaEpWindow *w, const uint16_t *d_x,
                          const int32_t *d_idx, size_t T, uint32_t epoch,
                          int32_t *d_pos, void *stream);
int apus_cuda_ep_wait_dev(ApusCudaEpWindow *w, int which, uint32_t epoch, void *stream);
int apus_cuda_ep_window_experts_dev(ApusCudaEpWindow *w, ApusCudaLayer *layer,
                                    void *stream);
int apus_cuda_ep_return_dev(ApusCudaEpWindow *w, uint32_t epoch, void *stream);
int apus_cuda_ep_shared_dev(ApusCudaLayer *layer, const uint16_t *d_x, size_t T,
                            uint16_t *d_sy, void *stream);
int apus_cuda_ep_combine_dev(ApusCudaEpWindow *w, ApusCudaLayer *layer, size_t T,
                             const int32_t *d_pos, const uint16_t *d_w,
                             const uint16_t *d_sy, const uint16_t *d_sgl,
                             uint16_t *d_out, void *stream);

/* The same step with each row crossing NVLink once per direction and no
 * exchange kernel around the experts ("pull" form; net-new as well).  A rank
 * stores its token rows and expert ids into every rank's window (with top-8
 * over at most 8 ranks nearly every rank needs nearly every token); the expert
 * ranks gather the rows they need from their own copy while sorting them for
 * the GEMMs, and the down GEMM's epilogue stores every output row straight into
 * the source rank's window, where its combine reads it (d_pos NULL: flat order
 * t * topk + j).
 *
 *   apus_cuda_ep_route_dev          idx, w, sgl of the rank's tokens
 *   apus_cuda_ep_publish_dev        rows and ids into every rank's window, flag
 *   apus_cuda_ep_wait_dev(0, e)     every source has published
 *   apus_cuda_ep_pull_experts_dev   resident ids kept and sorted, rows gathered,
 *                                   gate_up, down with remote stores (the shared
 *                                   expert of the own tokens rides along), flag
 *   apus_cuda_ep_wait_dev(1, e)     every peer's outputs have landed here
 *   apus_cuda_ep_combine_dev        with d_pos = NULL
 *
 * Same epoch rules, waits, status codes and bit-for-bit result as above.  Needs
 * the tensor-core path (hidden, moe_inter multiples of 128).  Before capturing
 * the step in a graph, run it once (the first call stores the peers' addresses
 * on the device). */
int apus_cuda_ep_publish_dev(ApusCudaEpWindow *w, const uint16_t *d_x,
                             const int32_t *d_idx, size_t T, uint32_t epoch,
                             void *stream);
/* The rows need nothing from the router: a caller may store them with this call
 * on a second stream while apus_cuda_ep_route_dev runs, and then pass d_x = NULL
 * to apus_cuda_ep_publish_dev (ids and flag only).  This call uses no shared
 * workspace and is the one device-pointer call the library does not order
 * against the others; the caller makes it start after its previous step's
 * combine and end before the publish (events, or a fork and join inside a
 * captured graph). */
int apus_cuda_ep_publish_rows_dev(ApusCudaEpWindow *w, const uint16_t *d_x, size_t T,
                                  void *stream);
/* d_x [T,H] (optional): the rank's own token rows; their shared expert then
 * runs inside the same GEMM launches and lands in d_sy [T,H], instead of in a
 * call to apus_cuda_ep_shared_dev. */
int apus_cuda_ep_pull_experts_dev(ApusCudaEpWindow *w, ApusCudaLayer *layer,
                                  uint32_t epoch, const uint16_t *d_x, size_t T,
                                  uint16_t *d_sy, void *stream);

/* ---- stages of the block, device pointers (kernel-level tests) ---------- */
int apus_cuda_route_dev(ApusCudaLayer *layer, const uint16_t *d_x, size_t T,
                        int32_t *d_idx, uint16_t *d_w, void *stream);
int apus_cuda_dispatch_dev(const int32_t *d_idx, size_t T, size_t topk,
                           size_t E, int32_t *d_counts, int32_t *d_offsets,
                           int32_t *d_perm, void *stream);

/* Same result as apus_cuda_dispatch_dev, for callers that must not touch the
 * device allocator.  (No counterpart in the reference engine, which has no
 * device memory at all.)  Who needs it: a serving loop that has handed every
 * free byte of HBM to its own pool, so a cudaMalloc from a library would fail
 * or fragment it; code running between the begin and end of a section where
 * allocation is forbidden by its owner; latency-critical paths where an
 * allocator call means an implicit device synchronisation.  This entry point
 * calls no cudaMalloc, cudaFree or other allocating routine: the per-unit
 * histogram scratch the three-pass dispatch needs lives in a 1 MiB array
 * built into the library (every GPU that loads the library holds it until the
 * process exits).  The caller still supplies d_idx and the three outputs.
 *
 * Limit: ceil(T*topk/256) * E <= 262144 (e.g. T*topk up to 262144 at E=256);
 * larger problems are refused with an error, not truncated.  E <= 1024.
 *
 * The first call on each device looks up the array's device address (with
 * that device current) and should therefore be made once, outside any stream
 * capture, before the calls that matter.  `stream` is used as given (NULL =
 * the default stream); the call enqueues and returns without synchronising.
 * All calls share the one array, and it keeps whatever the last call left
 * there; the kernels overwrite every entry they later read and the status
 * word is cleared on each call, but two calls whose kernels overlap on the
 * GPU (different streams, no ordering between them) race on it.  Expert ids
 * outside [0, E) are skipped silently here. */
int apus_cuda_dispatch_dev_static(const int32_t *d_idx, size_t T, size_t topk,
                                  size_t E, int32_t *d_counts,
                                  int32_t *d_offsets, int32_t *d_perm,
                                  void *stream);

/* ---- the two steps either side of the block (c/layer.h:386,388) --------- */
/* y = rmsnorm(x, gain 1+w) per row (c/attn.h:175-186; w NULL = zero gain
 * offset); out = rnd(a + b) (c/layer.h:230-234).  Device pointers. */
int apus_cuda_rmsnorm_dev(const uint16_t *d_x, const uint16_t *d_w,
                          uint16_t *d_y, size_t T, size_t N, void *stream);
int apus_cuda_resadd_dev(const uint16_t *d_a, const uint16_t *d_b,
                         uint16_t *d_out, size_t n, void *stream);

/* ---- the engine's largest dense product as a weight stream -------------- */
/* y[m,o] = rnd(sum_k W[o,k] x[m,k]) on DEVICE pointers, W [O,K], x [M,K],
 * y [M,O], M <= 8, K a multiple of 256: the bandwidth-bound form of the
 * bf16_gemv / bf16_gemm hooks for resident weights and activations (the
 * output head is 248320 x 2048, 1 GB of weights per token, c/model.h:667-688).
 * fp32 accumulation in a lane-strided order, so the result agrees with the
 * engine's sequential chain to BF16 tolerance, not bitwise; callers that need
 * the chain's exact bits (the router) use the host-pointer entry points. */
int apus_cuda_bf16_gemv_dev(const uint16_t *d_w, const uint16_t *d_x, uint16_t *d_y,
                            size_t M, size_t O, size_t K, void *stream);

/* ---- synthetic tensors (benchmarks and tests) ---------------------------- */
/* Fill n BF16 elements with the counter-based approximately-normal stream
 * (seed, layer, tensor_id), element index starting at first, scaled by
 * sigma.  Host and device versions produce identical bits. */
void apus_synth_fill_host(uint16_t *dst, size_t n, uint64_t seed,
                          uint32_t layer, uint32_t tensor_id, uint64_t first,
                          double sigma);
int apus_synth_fill_dev(uint16_t *d_dst, size_t n, uint64_t seed,
                        uint32_t layer, uint32_t tensor_id, uint64_t first,
                        double sigma, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* APUS_BACKEND_CUDA_H */
