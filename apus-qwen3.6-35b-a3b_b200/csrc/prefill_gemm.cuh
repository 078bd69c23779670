/*
 * prefill_gemm.cuh — the expert products for large token counts: a grouped
 * BF16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
 * tensor memory), fed by TMA, over the token rows dispatch has permuted into
 * expert-contiguous order.
 *
 * Replaces the per-expert loop of the CPU engine's batched body
 * (c/layer.h:599-621: gather rows -> gate_up GEMM -> apus_moe_silu_act per row
 * -> down GEMM -> scatter rows back) and its shared-expert GEMMs
 * (c/layer.h:593-596).
 *
 * Orientation ("swap A/B"): the WEIGHT rows are the MMA's M dimension (always
 * a full 128), the expert's TOKEN rows are N (16..128, rounded up to 16), so a
 * cold expert with a handful of rows still issues full-height MMAs and the
 * kernel degrades gracefully into a pure weight stream:
 *
 *   gate_up:  Dg[128 x N] = Wg[i0:i0+128, :] . X[r0:r0+N, :]^T     K = H
 *             Du[128 x N] = Wu[i0:i0+128, :] . X[r0:r0+N, :]^T
 *             epilogue in registers: g = rnd(Dg), u = rnd(Du);
 *             routed act = rnd(rnd(silu(g)) * u)   (c/moe.h:387-395)
 *             shared sa  = rnd(silu(g) * u)        (c/moe.h:438-445)
 *   down:     D[128 x N]  = Wd[h0:h0+128, :] . ACT[r0:r0+N, :]^T   K = I
 *             epilogue: y = rnd(D), stored at row perm[r] of the flat
 *             assignment-ordered buffer (the engine's eo, c/layer.h:618)
 *
 * One persistent CTA per SM, 10 warps: warp 0 picks tiles and issues TMA loads into a
 * shared-memory ring (128B-swizzled K-major tiles, no multicast), warp 1
 * issues the MMAs and owns the 512 TMEM columns (two accumulator stages), warps
 * 2-9 drain accumulators (tcgen05.ld, two warps per TMEM lane quarter) and run
 * the epilogue while the next tile's MMAs proceed.  Every wait is bounded; a
 * wait that runs out raises an abort flag, records a status code, and every
 * role falls through to the common exit where TMEM is released.
 *
 * A third mode of the same kernel multiplies one dense weight matrix with
 * every token row and stores the fp32 accumulators as they are: the router's
 * fast logits (router_certify.cuh).
 */
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "../../include/backend_cuda.h"
#include "common.cuh"
#include "decode_gemv.cuh"
#include "dispatch.cuh"

namespace apus {

constexpr int PG_BM = 128;        /* weight rows per tile (MMA M) */
constexpr int PG_BN_GU = 128;     /* token rows per gate_up tile (MMA N, max) */
constexpr int PG_BN_DN = 256;     /* token rows per down tile: one accumulator
                                   * per tile, so twice the columns fit TMEM and
                                   * every weight tile is fetched half as often */
constexpr int PG_BN_MIN = 32;     /* narrowest token box of a routed tile */
constexpr int PG_BN = PG_BN_MIN;  /* sizing of the tile lists (the finest one) */
constexpr int PG_BK = 64;         /* K elements per stage = one 128B swizzle row */
constexpr int PG_EPI_WARPS = 8;   /* two per TMEM lane quarter */
constexpr int PG_THREADS = 64 + PG_EPI_WARPS * 32;
constexpr int PG_TILE_BYTES = PG_BM * PG_BK * 2;   /* 16 KB */
constexpr int PG_CLAIM_KB = 8;     /* k-blocks before a tile's end at which the next is claimed */
constexpr int PG_TQ = 4;          /* tile queue entries */
constexpr int PG_STAGES = 4;      /* 48 KB per stage in both kernels */
constexpr int PG_TMEM_COLS = 512;

static char g_prefill_err[256] = "";
inline const char *prefill_last_error() { return g_prefill_err; }

/* ---- PTX wrappers ---------------------------------------------------------- */
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map,
                                            int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::"
        "complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *holder, uint32_t cols) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
            smem_u32(holder)),
        "r"(cols)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::
                     : "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                     taddr),
                 "r"(cols)
                 : "memory");
}
/* D[tmem] (+)= A[smem] * B[smem], BF16 in, fp32 accumulate */
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc,
                                          uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/* arrive on an mbarrier once every MMA issued so far by this thread is done */
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 "
        "[%0];" ::"r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
        "%30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
          "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
/* one accumulator column: 32 lanes x 32 bits */
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];"
                 : "=r"(r)
                 : "r"(taddr)
                 : "memory");
    return r;
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

/* K-major, 128-byte-swizzled operand tile [rows x 64 BF16]: rows are 128 B,
 * eight-row groups are 1024 B apart (SBO), descriptor version 1 (sm_100),
 * layout type 2 = SWIZZLE_128B.  The tile base must be 1024-byte aligned;
 * stepping K by 16 elements advances the start address by 32 bytes. */
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;                 /* LBO (unused for swizzled K-major) */
    d |= (uint64_t)(1024 >> 4) << 32;       /* SBO */
    d |= (uint64_t)1 << 46;                 /* descriptor version */
    d |= (uint64_t)2 << 61;                 /* SWIZZLE_128B */
    return d;
}
/* kind::f16 instruction descriptor: D fp32, A/B BF16, both K-major */
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(PG_BM >> 4) << 24);
}

/* wait on an mbarrier unless the CTA has aborted; a timeout aborts it */
__device__ __forceinline__ bool pg_wait(uint64_t *bar, uint32_t parity,
                                        volatile int *abort_flag, int *status,
                                        int code) {
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < APUS_WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 256) {
            __nanosleep(32);
            if (*abort_flag) return false;
        }
    }
    *abort_flag = 1;
    set_status(status, code);
    return false;
}

inline size_t prefill_max_ntiles(size_t A, size_t T, size_t E) {
    return A / PG_BN + E + (T + PG_BN_GU - 1) / PG_BN_GU + 1;
}
inline size_t prefill_tiles_bytes_for(const ApusCudaMoeCfg &c, size_t A,
                                      size_t T) {
    size_t nt = prefill_max_ntiles(A, T, c.experts);
    size_t m1 = (c.moe_inter > c.shared_inter ? c.moe_inter : c.shared_inter) / PG_BM;
    size_t m2 = c.hidden / PG_BM;
    return (nt * m1 + nt * m2) * sizeof(int4) + 256 + (2 * (c.experts + 2) + 2) * sizeof(int);
}

/* xg[p, :] = x[perm[p] / TK, :] — the rows of c/layer.h:603-605's memcpy.
 * n_valid (optional): how many of the A slots hold an assignment (empty slots
 * have no entry in perm). */
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint16_t *__restrict__ x,
                   const int32_t *__restrict__ perm, int A, int H, int TK,
                   uint16_t *__restrict__ xg, const int32_t *__restrict__ n_valid) {
    pdl_enter();
    const int c8 = H / 8;
    if (n_valid) A = min(A, max(*n_valid, 0));
    const long total = (long)A * c8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int p = (int)(i / c8), c = (int)(i - (long)p * c8);
        const int tok = perm[p] / TK;
        reinterpret_cast<uint4 *>(xg)[i] =
            ldg16(x + (size_t)tok * H + (size_t)c * 8);
    }
}

/* The block's rows live in other GPUs' memory (expert parallelism by peer
 * loads and stores; net-new, the reference engine is one process).  The flat
 * assignment a = s * cap + t * TK + j names slot j of token t of source rank
 * s; src[s] is the address of that rank's token rows [tokens, H] (this GPU's
 * copy of them, or the rank's own memory) and dst[s] the address of its buffer
 * of returned expert outputs [cap, H], mapped into this process. */
struct PeerRows {
    const unsigned long long *src;   /* device table [ranks] */
    const unsigned long long *dst;   /* device table [ranks] */
    int cap;
};

/* xg[p, :] = token row of assignment perm[p], loaded from its source rank
 * (NVLink reads for the remote ones). */
__global__ void __launch_bounds__(256)
gather_rows_peer_kernel(const unsigned long long *__restrict__ src, int cap,
                        const int32_t *__restrict__ perm, int A, int H, int TK,
                        uint16_t *__restrict__ xg, const int32_t *__restrict__ n_valid) {
    pdl_enter();
    const int c8 = H / 8;
    if (n_valid) A = min(A, max(*n_valid, 0));
    /* one row per 256-thread pass when H = 2048: consecutive rows of a CTA come
     * from whatever sources the sort put side by side */
    const long total = (long)A * c8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int p = (int)(i / c8), c = (int)(i - (long)p * c8);
        const int a = perm[p];
        const int s = a / cap, tok = (a - s * cap) / TK;
        const uint16_t *row = reinterpret_cast<const uint16_t *>(__ldg(src + s));
        reinterpret_cast<uint4 *>(xg)[i] = ldg16(row + (size_t)tok * H + (size_t)c * 8);
    }
}

/* ---- the grouped GEMM -------------------------------------------------------- */
struct GemmParams {
    const int4 *tiles;
    const int *n_tiles;
    int K;                 /* reduction length */
    int E;                 /* v == E: shared expert */
    int e_begin;           /* first resident expert */
    int rows_per_expert;   /* rows of the routed A tensor per expert */
    int up_off;            /* gate_up: row offset of the up half (I) */
    uint16_t *out_routed;  /* act [A, ld_routed]  or  eo [A, ld_routed] */
    uint16_t *out_shared;  /* sa [T, ld_shared]   or  sy [T, ld_shared] */
    int ld_routed, ld_shared;
    const int32_t *perm;   /* down: sorted position -> flat assignment */
    /* down, expert parallelism: routed output row a goes to row a % peer_cap of
     * the buffer at peer_dst[a / peer_cap] (another GPU's memory) instead of
     * row a of out_routed.  Null: off. */
    const unsigned long long *peer_dst;
    int peer_cap;
    int *status;
    /* Overlap of the two expert kernels.  When `done` is set, every epilogue
     * warp of the gate_up kernel counts a finished tile on done[expert] after
     * its stores, and the down kernel does not wait for the whole gate_up
     * kernel (programmatic dependent launch lets its CTAs start on SMs whose
     * gate_up CTA has run out of tiles) but, tile by tile, for done[expert] to
     * reach need[expert] * (epilogue warps).  The gate_up kernel never waits
     * on the down kernel, and all of its CTAs are resident before the first
     * down CTA can be, so the wait cannot hold up what it waits for. */
    int *done;
    const int *need;
    /* Tiles are handed out in list order by an atomic counter when `sched` is
     * set (CTA i starts with tile i): a CTA that starts late, because its SM
     * was still busy with the tail of the kernel before, simply takes fewer
     * tiles.  Null: tile i + k * gridDim.x belongs to CTA i. */
    int *sched;
    /* gate_up with up to 64 tokens (direct_tk = top_k, else 0): no gathered
     * copy of the rows.  Every routed tile multiplies its weights with ALL
     * direct_T tokens of the block input (one box; the MMA is as cheap for 32
     * columns as for 2), and the epilogue picks, for each of the expert's rows,
     * the column of that row's token. */
    int direct_tk, direct_T;
    int bn_rows;           /* token rows a routed tile's TMA box fetches (<= BN):
                            * experts with a handful of rows should not pull a
                            * full-width box of their neighbours' rows through L2 */
    /* MODE 2 (one dense weight matrix against every token row, fp32 out):
     * tiles are generated from the index, no list */
    int dense_T, dense_mt, dense_ntiles, dense_ksplit;
    float *out_f32;        /* [dense_ksplit][dense_T, ld_f32]: one slab per K slice */
    int ld_f32;
};

/* the tile with this index: from the list, or (MODE 2) generated: token tile
 * major, then weight-row tile, then K slice (in .x); p.K is the slice length */
template <int MODE>
__device__ __forceinline__ int4 pg_tile(const GemmParams &p, int tile) {
    if (MODE != 2) return __ldg(&p.tiles[tile]);
    const int ks = tile % p.dense_ksplit, r = tile / p.dense_ksplit;
    const int n = r / p.dense_mt, m = r - n * p.dense_mt;
    return make_int4(ks, m, n * PG_BN_GU, min(PG_BN_GU, p.dense_T - n * PG_BN_GU));
}

/* MODE 0: gate_up + SwiGLU;  1: down;  2: dense, fp32 accumulators stored as
 * they are (the router's fast logits) */
template <int MODE>
__global__ void __launch_bounds__(PG_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap mapA,     /* routed W */
                    const __grid_constant__ CUtensorMap mapAs,    /* shared g | d */
                    const __grid_constant__ CUtensorMap mapAs2,   /* shared u */
                    const __grid_constant__ CUtensorMap mapB,     /* xg | act */
                    const __grid_constant__ CUtensorMap mapBs,    /* x  | sa */
                    GemmParams p) {
    /* The next kernel may be scheduled now.  This kernel's own wait for the
     * previous one comes after the prologue below (barriers, TMEM), which
     * touches nothing the previous kernel writes. */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr bool GATE_UP = MODE == 0;
    constexpr int STAGES = PG_STAGES;
    constexpr int BN = MODE == 1 ? PG_BN_DN : PG_BN_GU;
    constexpr int A_TILES = GATE_UP ? 2 : 1;
    constexpr int B_OFF = A_TILES * PG_TILE_BYTES;        /* B tile offset */
    constexpr int B_BYTES = BN * PG_BK * 2;
    constexpr int STAGE_BYTES = B_OFF + B_BYTES;           /* 48 KB */

    extern __shared__ unsigned char pg_smem_raw[];
    /* 1024-byte alignment for the swizzled tiles */
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(pg_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + STAGES;
    uint64_t *tfull = bars + 2 * STAGES, *tempty = bars + 2 * STAGES + 2;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);
    /* tile queue: the producer warp decides which tile comes next and tells
     * the MMA warp and the epilogue warps through a small ring */
    uint64_t *tqf = bars + 2 * STAGES + 5, *tqe = tqf + PG_TQ;
    volatile int *tq = reinterpret_cast<volatile int *>(tqe + PG_TQ);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], PG_EPI_WARPS * 32);
        }
        for (int s = 0; s < PG_TQ; s++) {
            mbar_init(&tqf[s], 1);
            mbar_init(&tqe[s], 1 + PG_EPI_WARPS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_holder, PG_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    /* the down kernel of an overlapped pair does not wait for the whole gate_up
     * kernel: its producer waits per expert instead */
    if (!(MODE == 1 && p.done)) asm volatile("griddepcontrol.wait;" ::: "memory");
    const int n_tiles = MODE == 2 ? p.dense_ntiles : *p.n_tiles;
    const int num_kb = p.K / PG_BK;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (lane == 0) {
            uint32_t kiter = 0;
            bool alive = true;
            bool all_ready = false;
            /* Which tile comes next: the counter is asked while the last
             * k-blocks of the current tile are being requested — late, so that
             * a CTA claims no tile long before it can start it, yet early
             * enough for the answer (an L2 round trip) to be there.  Nothing
             * reads `claim` until the tile's loads are all out: the first
             * instruction that does would stall this lane for the round trip. */
            const bool dyn = MODE != 2 && p.sched != nullptr;
            const int kclaim = num_kb > PG_CLAIM_KB ? num_kb - PG_CLAIM_KB : 0;
            int tile = blockIdx.x;
            for (uint32_t qi = 0; alive; qi++) {
                const int qs = qi % PG_TQ;
                if (!pg_wait(&tqe[qs], ((qi / PG_TQ) & 1u) ^ 1u, abort_flag, p.status,
                             ST_MBAR_TIMEOUT))
                    break;
                tq[qs] = tile;
                mbar_arrive(&tqf[qs]);
                if (tile >= n_tiles) break;
                const int4 t = pg_tile<MODE>(p, tile);
                const bool shared = MODE == 2 || t.x == p.E;
                const int kb0 = MODE == 2 ? t.x * num_kb : 0;   /* K slice */
                const CUtensorMap *ma = shared ? &mapAs : &mapA;
                const CUtensorMap *ma2 = shared ? &mapAs2 : &mapA;
                const CUtensorMap *mb = shared ? &mapBs : &mapB;
                const int arow =
                    (shared ? 0 : (t.x - p.e_begin) * p.rows_per_expert) + t.y * PG_BM;
                const int arow2 = shared ? arow : arow + p.up_off;
                const int brows = (MODE == 2 || shared) ? BN : p.bn_rows;   /* box of mb */
                const int brow = (MODE == 0 && p.direct_tk && !shared) ? 0 : t.z;
                if (MODE == 1 && p.done && !all_ready) {
                    /* This expert's activations must be complete and visible.
                     * Once the whole gate_up kernel is through, no tile asks
                     * again (a look at the counter is an L2 round trip). */
                    const int e = shared ? p.E : t.x;
                    const int need = __ldg(&p.need[e]) * PG_EPI_WARPS;
                    const int need_all = __ldg(&p.need[p.E + 1]) * PG_EPI_WARPS;
                    bool ready = false;
                    for (uint32_t i = 0; i < APUS_WAIT_LIMIT && !*abort_flag; i++) {
                        int v, va;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];"
                                     : "=r"(va)
                                     : "l"(p.done + p.E + 1)
                                     : "memory");
                        if (va >= need_all) { all_ready = true; ready = true; break; }
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];"
                                     : "=r"(v)
                                     : "l"(p.done + e)
                                     : "memory");
                        if (v >= need) { ready = true; break; }
                        __nanosleep(100);
                    }
                    if (!ready) {
                        *abort_flag = 1;
                        set_status(p.status, ST_SCHED_TIMEOUT);
                        alive = false;
                        break;
                    }
                    /* generic-proxy writes of other SMs, then TMA (async proxy) reads */
                    asm volatile("fence.proxy.async;" ::: "memory");
                }
                int claim = tile;
                auto request = [&](int kb) -> bool {
                    const int s = kiter % STAGES;
                    const uint32_t ph = (kiter / STAGES) & 1u;
                    if (!pg_wait(&empty[s], ph ^ 1u, abort_flag, p.status,
                                 ST_MBAR_TIMEOUT))
                        return false;
                    unsigned char *st = smem + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], (uint32_t)(B_OFF + brows * PG_BK * 2));
                    tma_load_2d(st, ma, (kb0 + kb) * PG_BK, arow, &full[s]);
                    if (GATE_UP)
                        tma_load_2d(st + PG_TILE_BYTES, ma2, kb * PG_BK, arow2,
                                    &full[s]);
                    tma_load_2d(st + B_OFF, mb, (kb0 + kb) * PG_BK, brow, &full[s]);
                    kiter++;
                    return true;
                };
                int kb = 0;
                for (; alive && kb <= kclaim; kb++) alive = request(kb);
                if (dyn) claim = atomicAdd(p.sched, 1);
                for (; alive && kb < num_kb; kb++) alive = request(kb);
                tile = claim + (int)gridDim.x;
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer ---------------- */
        if (lane == 0) {
            uint32_t kiter = 0;
            bool alive = true;
            for (int it = 0; alive; it++) {
                const int qs = it % PG_TQ;
                if (!pg_wait(&tqf[qs], (uint32_t)(it / PG_TQ) & 1u, abort_flag, p.status,
                             ST_MBAR_TIMEOUT))
                    break;
                const int tile = tq[qs];
                mbar_arrive(&tqe[qs]);
                if (tile >= n_tiles) break;
                const int4 t = pg_tile<MODE>(p, tile);
                const int acc = it & 1;
                const uint32_t aph = (uint32_t)(it >> 1) & 1u;
                const int ncols = (MODE == 0 && p.direct_tk && t.x != p.E) ? p.direct_T : t.w;
                const int n = ((ncols + 15) >> 4) << 4;
                const uint32_t idesc = umma_idesc(n);
                if (!pg_wait(&tempty[acc], aph ^ 1u, abort_flag, p.status,
                             ST_TMEM_TIMEOUT)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)acc * 256u;
                for (int kb = 0; kb < num_kb; kb++, kiter++) {
                    const int s = kiter % STAGES;
                    const uint32_t ph = (kiter / STAGES) & 1u;
                    if (!pg_wait(&full[s], ph, abort_flag, p.status,
                                 ST_MBAR_TIMEOUT)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t da = umma_smem_desc(sa);
                    const uint64_t db = umma_smem_desc(sa + B_OFF);
#pragma unroll
                    for (int k = 0; k < PG_BK / 16; k++) {
                        const uint32_t accum = (kb | k) ? 1u : 0u;
                        /* +32 bytes per 16-element K step (encoded >> 4) */
                        umma_bf16(d0, da + 2u * k, db + 2u * k, idesc, accum);
                        if (GATE_UP) {
                            const uint64_t da2 = umma_smem_desc(sa + PG_TILE_BYTES);
                            umma_bf16(d0 + 128u, da2 + 2u * k, db + 2u * k, idesc,
                                      accum);
                        }
                    }
                    umma_commit(&empty[s]);    /* frees the stage when done */
                }
                if (alive) umma_commit(&tfull[acc]);
            }
        }
    } else {
        /* ---------------- epilogue (warps 2..9) ---------------- */
        /* A warp may only touch the TMEM lanes of its quarter (warp % 4); two
         * warps share a quarter and split the 32-column chunks between them. */
        const int q = warp & 3;                 /* TMEM lane quarter */
        const int half = (warp - 2) >> 2;       /* which chunks of the tile */
        const int row = q * 32 + lane;          /* row inside the tile */
        bool alive = true;
        for (int it = 0; alive; it++) {
            const int qs = it % PG_TQ;
            if (!pg_wait(&tqf[qs], (uint32_t)(it / PG_TQ) & 1u, abort_flag, p.status,
                         ST_MBAR_TIMEOUT))
                break;
            const int tile = tq[qs];
            __syncwarp();
            if (lane == 0) mbar_arrive(&tqe[qs]);
            if (tile >= n_tiles) break;
            const int4 t = pg_tile<MODE>(p, tile);
            const bool shared = MODE == 2 || t.x == p.E;
            const int acc = it & 1;
            const uint32_t aph = (uint32_t)(it >> 1) & 1u;
            if (!pg_wait(&tfull[acc], aph, abort_flag, p.status,
                         ST_TMEM_TIMEOUT)) {
                alive = false;
                break;
            }
            tc_fence_after();
            const uint32_t taddr =
                tmem_base + (uint32_t)acc * 256u + ((uint32_t)(q * 32) << 16);
            uint16_t *out = shared ? p.out_shared : p.out_routed;
            const int ld = shared ? p.ld_shared : p.ld_routed;
            const int col = t.y * PG_BM + row;
            if (MODE == 0 && p.direct_tk && !shared) {
                /* row n of this expert belongs to token perm[.] / top_k: its
                 * accumulator column is the token's index */
                if (half == 0) {
                    for (int n = 0; n < t.w; n++) {
                        const int tok = __ldg(&p.perm[t.z + n]) / p.direct_tk;
                        const uint32_t g1 = tmem_ld1(taddr + (uint32_t)tok);
                        const uint32_t u1 = tmem_ld1(taddr + 128u + (uint32_t)tok);
                        tmem_ld_wait();
                        float gv = __uint_as_float(g1), uv = __uint_as_float(u1);
                        bf16_round2(gv, uv);
                        out[(size_t)(t.z + n) * ld + col] =
                            (uint16_t)silu_act_pack2(gv, uv, 0.0f, 0.0f);
                    }
                }
            } else
            for (int c0 = half * 32; c0 < t.w; c0 += 64) {
                uint32_t g[32];
                tmem_ld32(taddr + (uint32_t)c0, g);
                if (GATE_UP) {
                    uint32_t u[32];
                    tmem_ld32(taddr + 128u + (uint32_t)c0, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const int n = c0 + j;
                        if (n < t.w) {
                            float g0 = __uint_as_float(g[j]), g1 = __uint_as_float(g[j + 1]),
                                  u0 = __uint_as_float(u[j]), u1 = __uint_as_float(u[j + 1]);
                            bf16_round2(g0, g1);
                            bf16_round2(u0, u1);
                            const uint32_t pk = shared ? silu_mul_pack2(g0, u0, g1, u1)
                                                       : silu_act_pack2(g0, u0, g1, u1);
                            out[(size_t)(t.z + n) * ld + col] = (uint16_t)pk;
                            if (n + 1 < t.w)
                                out[(size_t)(t.z + n + 1) * ld + col] = (uint16_t)(pk >> 16);
                        }
                    }
                } else if (MODE == 2) {
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < t.w)
                            p.out_f32[((size_t)t.x * p.dense_T + t.z + c0 + j) * p.ld_f32 +
                                      col] = __uint_as_float(g[j]);
                } else {
                    /* output row of each of this chunk's 32 columns: one load
                     * per lane, handed round by shuffle */
                    int my_orow = 0;
                    if (c0 + lane < t.w)
                        my_orow = shared ? t.z + c0 + lane
                                         : __ldg(&p.perm[t.z + c0 + lane]);
                    if (p.peer_dst && !shared) {
                        /* each output row has its own home: the address travels
                         * by shuffle instead of the row number */
                        unsigned long long my_row = 0;
                        if (c0 + lane < t.w) {
                            const int s = my_orow / p.peer_cap;
                            my_row = __ldg(p.peer_dst + s) +
                                     (unsigned long long)(my_orow - s * p.peer_cap) * ld * 2ull;
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            uint16_t *r0 = reinterpret_cast<uint16_t *>(
                                __shfl_sync(0xffffffffu, my_row, j));
                            uint16_t *r1 = reinterpret_cast<uint16_t *>(
                                __shfl_sync(0xffffffffu, my_row, j + 1));
                            const uint32_t pk = pack_bf16_rn(__uint_as_float(g[j]),
                                                             __uint_as_float(g[j + 1]));
                            if (c0 + j < t.w) r0[col] = (uint16_t)pk;
                            if (c0 + j + 1 < t.w) r1[col] = (uint16_t)(pk >> 16);
                        }
                        continue;
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const int orow0 = __shfl_sync(0xffffffffu, my_orow, j);
                        const int orow1 = __shfl_sync(0xffffffffu, my_orow, j + 1);
                        const uint32_t pk =
                            pack_bf16_rn(__uint_as_float(g[j]), __uint_as_float(g[j + 1]));
                        if (c0 + j < t.w) out[(size_t)orow0 * ld + col] = (uint16_t)pk;
                        if (c0 + j + 1 < t.w)
                            out[(size_t)orow1 * ld + col] = (uint16_t)(pk >> 16);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&tempty[acc]);
            if (MODE == 0 && p.done) {
                /* this warp's share of the tile is stored: make it visible, count it */
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    atomicAdd(p.done + (shared ? p.E : t.x), 1);
                    atomicAdd(p.done + p.E + 1, 1);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, PG_TMEM_COLS);
    }
}

/* ---- host side ---------------------------------------------------------------- */
typedef CUresult (*PFN_encodeTiled_local)(
    CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
    CUtensorMapFloatOOBfill);

struct PrefillMaps {
    PFN_encodeTiled_local encode = nullptr;
    CUtensorMap w_gu, sh_g, sh_u, w_d, sh_d;
};

/* cuTensorMapEncodeTiled through the runtime's driver entry-point lookup (the
 * library does not link libcuda, so it loads on machines without a driver) */
inline PFN_encodeTiled_local tensor_map_encoder() {
    static PFN_encodeTiled_local cached = nullptr;
    if (cached) return cached;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault,
                                &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "cuTensorMapEncodeTiled is not available from the driver");
        return nullptr;
    }
    cached = (PFN_encodeTiled_local)fn;
    return cached;
}

inline bool prefill_supported(const ApusCudaMoeCfg &c) {
    return c.hidden % PG_BM == 0 && c.moe_inter % PG_BM == 0 &&
           c.shared_inter % PG_BM == 0 && c.hidden % PG_BK == 0 &&
           c.moe_inter % PG_BK == 0 && c.shared_inter % PG_BK == 0 &&
           c.shared_inter == c.moe_inter && c.experts <= 1024;
}

/* rows x cols BF16, row-major; box = 128 rows x 64 columns, 128B swizzle */
inline int encode_2d(PFN_encodeTiled_local enc, CUtensorMap *m, const void *base,
                     size_t rows, size_t cols, int box_rows = PG_BM) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)PG_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base),
                     dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "cuTensorMapEncodeTiled failed (%d) rows=%zu cols=%zu", (int)r,
                 rows, cols);
        return 1;
    }
    return 0;
}

inline PrefillMaps *prefill_maps_create(const ApusCudaMoeCfg &c,
                                        const uint16_t *exp_gu,
                                        const uint16_t *exp_d,
                                        const uint16_t *sh_g,
                                        const uint16_t *sh_u,
                                        const uint16_t *sh_d, size_t n_experts) {
    PFN_encodeTiled_local fn = tensor_map_encoder();
    if (!fn) return nullptr;
    PrefillMaps *m = new PrefillMaps();
    m->encode = fn;
    const size_t H = c.hidden, I = c.moe_inter, Is = c.shared_inter;
    int bad = 0;
    if (n_experts) {
        bad |= encode_2d(m->encode, &m->w_gu, exp_gu, n_experts * 2 * I, H);
        bad |= encode_2d(m->encode, &m->w_d, exp_d, n_experts * H, I);
    } else {
        /* no routed experts resident: alias the shared maps (never read) */
        bad |= encode_2d(m->encode, &m->w_gu, sh_g, Is, H);
        bad |= encode_2d(m->encode, &m->w_d, sh_d, H, Is);
    }
    bad |= encode_2d(m->encode, &m->sh_g, sh_g, Is, H);
    bad |= encode_2d(m->encode, &m->sh_u, sh_u, Is, H);
    bad |= encode_2d(m->encode, &m->sh_d, sh_d, H, Is);
    if (bad) {
        delete m;
        return nullptr;
    }
    return m;
}
inline void prefill_maps_free(PrefillMaps *m) { delete m; }

/* Set when the backend is enabled: the two expert kernels overlap through
 * per-expert counters (0: plain kernel boundary); tiles handed out by an atomic
 * counter (bit 0: gate_up kernel, bit 1: down kernel). */
inline int g_pg_overlap = 1;
inline int g_pg_dynamic = 3;
inline int g_pg_direct = 1;      /* up to 32 tokens: no gathered copy of the rows */

inline int pg_smem_bytes(bool gate_up) {
    (void)gate_up;
    return PG_STAGES * 3 * PG_TILE_BYTES + 1024 /* alignment slack */ +
           256 /* barriers */;
}

/* Tile shapes and list storage for A routed rows and T tokens (the shared
 * expert runs over them when do_shared) */
inline TilePlan prefill_tile_plan(const ApusCudaMoeCfg &c, int T, bool do_shared, int A,
                                  void *tiles_ws) {
    const int H = (int)c.hidden, I = (int)c.moe_inter, Is = (int)c.shared_inter,
              E = (int)c.experts;
    TilePlan p;
    memset(&p, 0, sizeof p);
    p.on = 1;
    p.T = do_shared ? T : 0;
    p.m_gu = I / PG_BM;
    p.m_gu_sh = Is / PG_BM;
    p.m_dn = H / PG_BM;
    /* token box of the routed tiles: about twice the mean row count of an
     * expert, so that nearly every expert is one tile and a tile does not pull
     * rows it will not use through L2 */
    int want = PG_BN_MIN;
    while (want < PG_BN_DN && (long)want * E < 2L * A) want *= 2;
    p.bn_gu = want < PG_BN_GU ? want : PG_BN_GU;
    p.bn_dn = want < PG_BN_DN ? want : PG_BN_DN;
    p.bn_sh_gu = PG_BN_GU;
    p.bn_sh_dn = PG_BN_DN;
    const size_t nt = prefill_max_ntiles((size_t)A, (size_t)T, (size_t)E);
    const size_t m1 = (size_t)(p.m_gu > p.m_gu_sh ? p.m_gu : p.m_gu_sh);
    TileLists &tl = p.tl;
    tl.gu = reinterpret_cast<int4 *>(tiles_ws);
    tl.dn = tl.gu + nt * m1;
    tl.n_gu = reinterpret_cast<int *>(tl.dn + nt * p.m_dn);
    tl.n_dn = tl.n_gu + 1;
    tl.done = tl.n_gu + 16;
    tl.need = tl.done + (E + 2);
    tl.sched = tl.need + (E + 2);
    return p;
}

/* Routed + shared experts through the tensor-core path.  x [T,H] is the block
 * input; d holds the dispatch results; xg/act/sa/eo/sy are workspace. */
inline int run_prefill_experts(int sm_count, int smem_optin, PrefillMaps *maps,
                               const ApusCudaMoeCfg &c, int e_begin,
                               const uint16_t *x, int T, int A, int TK,
                               bool do_shared,
                               const DispatchOut &d, uint16_t *xg, uint16_t *act,
                               uint16_t *sa, uint16_t *eo, uint16_t *sy,
                               void *tiles_ws, int *status, cudaStream_t st,
                               int *launches, void (*mark)(int stage),
                               const TilePlan *built = nullptr,
                               const PeerRows *peer = nullptr) {
    const int H = (int)c.hidden, I = (int)c.moe_inter, Is = (int)c.shared_inter,
              E = (int)c.experts;
    if (!maps) {
        snprintf(g_prefill_err, sizeof g_prefill_err, "tensor maps missing");
        return 1;
    }
    const int s1 = pg_smem_bytes(true), s2 = pg_smem_bytes(false);
    if (s1 > smem_optin || s2 > smem_optin) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "grouped GEMM needs %d B shared memory", s1);
        return 1;
    }
    /* tile lists: built by the dispatch kernel already, or here */
    TilePlan plan = prefill_tile_plan(c, T, do_shared, A, tiles_ws);
    if (built) {
        plan = *built;
    } else {
        launch_k(build_tiles_kernel, dim3(1), dim3(1024), 0, st, (const int32_t *)d.counts,
                 (const int32_t *)d.offsets, E, plan);
        (*launches)++;
    }
    const TileLists tl = plan.tl;
    const int bn_gu = plan.bn_gu, bn_dn = plan.bn_dn;
    const int m_gu = plan.m_gu, m_gu_sh = plan.m_gu_sh, m_dn = plan.m_dn;
    (void)m_gu; (void)m_gu_sh; (void)m_dn;
    const bool overlap = g_pg_overlap != 0;
    const int dynamic = g_pg_dynamic;
    /* a handful of tokens: the gate_up kernel reads the block input itself */
    const bool direct = A > 0 && T <= 2 * PG_BN_MIN && g_pg_direct != 0 && !peer;
    const int box_gu = direct ? (T <= PG_BN_MIN ? PG_BN_MIN : 2 * PG_BN_MIN) : bn_gu;
    /* permuted activation rows */
    if (A > 0 && !direct) {
        long total = (long)A * (H / 8);
        int blocks = (int)((total + 255) / 256);
        if (blocks > sm_count * 16) blocks = sm_count * 16;
        if (peer)
            launch_k(gather_rows_peer_kernel, dim3(blocks), dim3(256), 0, st, peer->src,
                     peer->cap, (const int32_t *)d.perm, A, H, TK, xg,
                     (const int32_t *)(d.offsets + E));
        else
            launch_k(gather_rows_kernel, dim3(blocks), dim3(256), 0, st, x, d.perm, A, H,
                     TK, xg, (const int32_t *)(d.offsets + E));
        (*launches)++;
    }
    if (mark) mark(APUS_CUDA_STAGE_GATHER);
    /* activation-side tensor maps (buffers move with the workspace) */
    CUtensorMap m_xg, m_x, m_act, m_sa;
    int bad = 0;
    bad |= encode_2d(maps->encode, &m_xg, (A > 0 && !direct) ? (const void *)xg : (const void *)x,
                     (size_t)(direct ? T : (A > 0 ? A : 1)), H, box_gu);
    bad |= encode_2d(maps->encode, &m_x, x, (size_t)(T > 0 ? T : 1), H);
    bad |= encode_2d(maps->encode, &m_act, A > 0 ? (const void *)act : (const void *)sa,
                     (size_t)(A > 0 ? A : 1), I, bn_dn);
    bad |= encode_2d(maps->encode, &m_sa, do_shared ? (const void *)sa : (const void *)x,
                     (size_t)(do_shared && T > 0 ? T : 1), Is, PG_BN_DN);
    if (bad) return 1;

    cudaFuncSetAttribute(grouped_gemm_kernel<0>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, s1);
    cudaFuncSetAttribute(grouped_gemm_kernel<1>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, s2);
    GemmParams p1;
    memset(&p1, 0, sizeof p1);
    p1.tiles = tl.gu;
    p1.n_tiles = tl.n_gu;
    p1.K = H;
    p1.E = E;
    p1.e_begin = e_begin;
    p1.rows_per_expert = 2 * I;
    p1.up_off = I;
    p1.out_routed = act;
    p1.out_shared = sa;
    p1.ld_routed = I;
    p1.ld_shared = Is;
    p1.status = status;
    p1.bn_rows = box_gu;
    p1.done = overlap ? tl.done : nullptr;
    p1.need = tl.need;
    p1.perm = d.perm;
    p1.direct_tk = direct ? TK : 0;
    p1.direct_T = T;
    p1.sched = (dynamic & 1) ? tl.sched : nullptr;
    launch_k(grouped_gemm_kernel<0>, dim3(sm_count), dim3(PG_THREADS), s1, st, maps->w_gu, maps->sh_g, maps->sh_u, m_xg, m_x, p1);
    (*launches)++;
    if (mark) mark(APUS_CUDA_STAGE_GATE_UP);
    GemmParams p2 = p1;
    p2.tiles = tl.dn;
    p2.n_tiles = tl.n_dn;
    p2.K = I;   /* == Is is required below */
    p2.rows_per_expert = H;
    p2.up_off = 0;
    p2.out_routed = eo;
    p2.out_shared = sy;
    p2.ld_routed = H;
    p2.ld_shared = H;
    p2.perm = d.perm;
    p2.direct_tk = 0;
    p2.peer_dst = peer ? peer->dst : nullptr;
    p2.peer_cap = peer ? peer->cap : 0;
    p2.bn_rows = bn_dn;
    p2.sched = (dynamic & 2) ? tl.sched + 1 : nullptr;
    if (Is != I) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "tensor-core path needs shared_inter == moe_inter");
        return 1;
    }
    launch_k(grouped_gemm_kernel<1>, dim3(sm_count), dim3(PG_THREADS), s2, st, maps->w_d, maps->sh_d, maps->sh_d, m_act, m_sa, p2);
    (*launches)++;
    if (mark) mark(APUS_CUDA_STAGE_DOWN);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(g_prefill_err, sizeof g_prefill_err, "grouped GEMM launch: %s",
                 cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

/* How many K slices the dense logits GEMM uses for T tokens: few token tiles
 * would leave most SMs idle behind a long serial K loop. */
inline int dense_logits_ksplit(int sm_count, int T, int E, int K) {
    const int tiles = ((T + PG_BN_GU - 1) / PG_BN_GU) * (E / PG_BM);
    int s = 1;
    while (s < 4 && tiles * s * 2 <= sm_count && (K / PG_BK) % (s * 2) == 0) s *= 2;
    return s;
}

/* out[s][T, E] = x[T, Ks] . w[E, Ks]^T per K slice s on the tensor cores, fp32,
 * any summation order: the router's fast logits are the sum of the slabs.
 * E % 128 == 0, K % 64 == 0. */
inline int run_dense_logits(int sm_count, int smem_optin, const uint16_t *w,
                            const uint16_t *x, int T, int E, int K, int ksplit,
                            float *out, int *status, cudaStream_t st, int *launches) {
    PFN_encodeTiled_local enc = tensor_map_encoder();
    if (!enc) return 1;
    const int smem = PG_STAGES * 2 * PG_TILE_BYTES + 1024 + 256;
    if (smem > smem_optin || E % PG_BM || K % PG_BK) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "dense logits GEMM: unsupported shape E=%d K=%d", E, K);
        return 1;
    }
    CUtensorMap m_w, m_x;
    if (encode_2d(enc, &m_w, w, (size_t)E, (size_t)K) ||
        encode_2d(enc, &m_x, x, (size_t)T, (size_t)K))
        return 1;
    static bool set_ = false;
    if (!set_) {
        cudaFuncSetAttribute(grouped_gemm_kernel<2>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        set_ = true;
    }
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.K = K / ksplit;
    p.E = E;
    p.dense_T = T;
    p.dense_mt = E / PG_BM;
    p.dense_ksplit = ksplit;
    p.dense_ntiles = ((T + PG_BN_GU - 1) / PG_BN_GU) * p.dense_mt * ksplit;
    p.out_f32 = out;
    p.ld_f32 = E;
    p.status = status;
    const int grid = p.dense_ntiles < sm_count ? p.dense_ntiles : sm_count;
    launch_k(grouped_gemm_kernel<2>, dim3(grid), dim3(PG_THREADS), (size_t)smem, st,
             m_w, m_w, m_w, m_x, m_x, p);
    (*launches)++;
    return 0;
}

}  // namespace apus
