/*
 * pair_gemm.cuh — the expert products for thousands of tokens: a grouped BF16
 * GEMM in which TWO SMs work on one tile (tcgen05.mma.cta_group::2).
 *
 * Replaces, like prefill_gemm.cuh, the per-expert loop of the CPU engine's
 * batched body (c/layer.h:599-621) and its shared-expert GEMMs
 * (c/layer.h:593-596); this is the form for many rows per expert, where the
 * one-SM kernel is held back by the operand bytes every SM has to pull through
 * L2 (48 KB per 64-deep k-block for a 128 x 128(x2) tile).
 *
 * Orientation: the expert's TOKEN rows are the MMA's M dimension, 256 per pair
 * of CTAs (128 per CTA, one TMEM lane each), the WEIGHT rows are N = 256, of
 * which each CTA of the pair loads one half into its own shared memory; the
 * pair's MMA reads both halves.  Per k-block a CTA pulls 16 KB of tokens and
 * 16 KB of weights for 128 x 256 outputs: two thirds of the bytes per flop of
 * the one-SM kernel, and an expert with up to 256 rows reads its weights once.
 *
 *   gate_up:  N = 128 gate rows (CTA 0's half) | the 128 matching up rows
 *             (CTA 1's half), so every thread finds g and u of the same
 *             (token, i) in its own TMEM lane:
 *             act = rnd(rnd(silu(rnd g)) * rnd u)   routed  (c/moe.h:387-395)
 *             sa  = rnd(silu(rnd g) * rnd u)        shared  (c/moe.h:438-445)
 *   down:     N = 256 output columns h0..h0+255 (128 per CTA);
 *             y = rnd(D) stored at row perm[r] of the flat assignment-ordered
 *             buffer (the engine's eo, c/layer.h:618) or row t of sy.
 *
 * A thread owns one token row, so its outputs are contiguous: 16-byte stores.
 *
 * The kernel is bound by the bytes an SM can take in from L2 (about 38 bytes
 * per clock measured), so a tile's rows are split evenly between the two CTAs
 * and each CTA fetches a token box just tall enough for its share (32, 64, 96
 * or 128 rows): an expert with 100 rows costs each CTA 16 KB of weights and
 * 8 KB of tokens per k-block instead of 32 KB.  (The MMA always spans 256
 * rows; rows past a CTA's share hold stale data whose results are not stored.)
 *
 * One persistent cluster of two CTAs per SM pair, 10 warps per CTA: warp 0
 * issues TMA loads (no multicast: each CTA loads its own operands; the
 * completion bytes of both CTAs are counted on the leader's barrier), warp 1 of
 * the leader CTA issues the MMAs and both warps 1 own their CTA's 512 TMEM
 * columns (two accumulator stages), warps 2-9 drain the accumulators.  Stage
 * and accumulator hand-backs from the MMA to both CTAs are tcgen05.commit with
 * a cluster mask.  Every wait is bounded; a wait that runs out raises the
 * CTA's abort flag and records a status code, and every role falls through to
 * the common exit (cluster barrier, TMEM release).
 */
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "dispatch.cuh"
#include "prefill_gemm.cuh"

namespace apus {

constexpr int PP_BM = 128;          /* token rows per CTA (256 per pair) */
constexpr int PP_BN = 256;          /* weight rows per tile (128 per CTA) */
constexpr int PP_BK = 64;
constexpr int PP_HALF_BYTES = 128 * PP_BK * 2;       /* 16 KB */
constexpr int PP_STAGE_BYTES = 2 * PP_HALF_BYTES;    /* tokens | weights */
constexpr int PP_STAGES = 6;
constexpr int PP_EPI_WARPS = 8;
constexpr int PP_THREADS = 64 + PP_EPI_WARPS * 32;
/* gate_up only: six more warps that fetch the token rows themselves, so that no
 * permuted copy of the block input is needed */
constexpr int PP_GATHER_WARPS = 6;    /* == PP_STAGES: warp w serves stage w */
constexpr int PP_THREADS_GU = PP_THREADS + PP_GATHER_WARPS * 32;
constexpr int PP_TMEM_COLS = 512;
constexpr uint32_t PP_PEER_MASK = 0xFEFFFFFFu;      /* cluster address of CTA 0's copy */

/* down with outputs stored into peers' memory: a 32-row x 128-byte staging tile
 * per epilogue warp, so that a row leaves as 128 contiguous bytes */
constexpr int PP_STAGING_BYTES = PP_EPI_WARPS * 4096;
inline int pp_smem_bytes(bool staging = false) {
    /* after the stages and the barriers: the down epilogue's staging tiles, or
     * the gate_up gather warps' token tables (6 x 128 ints) */
    return PP_STAGES * PP_STAGE_BYTES + 1024 + 256 + (staging ? PP_STAGING_BYTES : 3072);
}

/* token-side tensor maps: the same tensor with boxes of 32, 64, 96, 128 rows */
struct PairMaps {
    CUtensorMap m[4];
};
/* rows of a c-row tile that CTA `rank` owns: the first ceil(c/2) or the rest */
__host__ __device__ __forceinline__ int pp_rows_of(int c, int rank) {
    const int n0 = (c + 1) >> 1;
    return rank ? c - n0 : n0;
}

struct PairParams {
    const int4 *tiles;       /* {expert or E, n-tile, first row, rows <= 256} */
    const int *n_tiles;
    int K;
    int E, e_begin;
    int rows_per_expert;     /* weight rows per expert in the routed tensor */
    int up_off;              /* gate_up: offset of the up rows (I) */
    uint16_t *out_routed, *out_shared;
    int ld_routed, ld_shared;
    const int32_t *perm;     /* down: sorted position -> flat assignment */
    /* down, expert parallelism: routed output row a is row a % peer_cap of the
     * buffer at peer_dst[a / peer_cap], in another GPU's memory (null: off) */
    const unsigned long long *peer_dst;
    int peer_cap;
    int *status;
    /* gate_up: token rows of the routed tiles fetched straight from the block
     * input by index (row perm[p] / gather_tk), four rows per TMA instruction,
     * instead of from a permuted copy */
    int gather_tk;           /* 0: off */
    /* gate_up: token rows fetched by the kernel's own gather warps with plain
     * loads (row perm[p] / wgather_tk of x for a routed tile, row p for the shared
     * expert) and written into the stage in the layout the TMA would have
     * produced; the TMA producer then loads weights only.  0: off */
    int wgather_tk;
    const uint16_t *x;       /* [T, K] block input (wgather) */
};

__device__ __forceinline__ uint32_t pp_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void pp_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
/* TMA tile load into this CTA's shared memory; completion bytes counted on the
 * LEADER CTA's barrier at the same offset (no multicast) */
__device__ __forceinline__ void pp_tma_load(void *dst, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::"
        "complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & PP_PEER_MASK), "r"(x),
        "r"(y)
        : "memory");
}
/* Four arbitrary rows of a 2-D tensor (64 columns of each) into four consecutive
 * 128-byte rows of this CTA's shared memory; the tensor map's box is 64 x 1.
 * Completion bytes go to the leader CTA's barrier, as for pp_tma_load. */
__device__ __forceinline__ void pp_tma_gather4(void *dst, const CUtensorMap *map, int x,
                                               int r0, int r1, int r2, int r3,
                                               uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::"
        "complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & PP_PEER_MASK), "r"(x),
        "r"(r0), "r"(r1), "r"(r2), "r"(r3)
        : "memory");
}
__device__ __forceinline__ void pp_tmem_alloc(uint32_t *holder, uint32_t cols) {
    asm volatile(
        "tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
            smem_u32(holder)),
        "r"(cols)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pp_tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void pp_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
/* arrive, once every MMA issued so far is done, on the barrier at this offset
 * in BOTH CTAs of the pair */
__device__ __forceinline__ void pp_commit_both(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster."
        "multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
        "h"(mask)
        : "memory");
}
/* arrive on the leader CTA's copy of a barrier */
__device__ __forceinline__ void pp_arrive_leader(uint64_t *bar) {
    asm volatile(
        "{\n\t"
        ".reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, 0;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t"
        "}\n" ::"r"(smem_u32(bar))
        : "memory");
}
/* barrier wait that also acquires what the PEER CTA's threads wrote before
 * their (cluster-scope release) arrivals */
__device__ __forceinline__ bool pp_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool pp_wait_cluster(uint64_t *bar, uint32_t parity,
                                                volatile int *abort_flag, int *status,
                                                int code) {
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < APUS_WAIT_LIMIT; i++) {
        if (pp_try_wait_cluster(bar, parity)) return true;
        if (i > 256) {
            __nanosleep(32);
            if (*abort_flag) return false;
        }
    }
    *abort_flag = 1;
    set_status(status, code);
    return false;
}
/* kind::f16 instruction descriptor: D fp32, A/B BF16, both K-major, M x N */
__device__ __forceinline__ uint32_t pp_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
/* 32 bytes (one whole sector) per store: a thread owns a row, so a warp's store
 * touches 32 rows whatever its width; half as many, complete sectors */
__device__ __forceinline__ void st32(uint16_t *p, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
                 "r"(v[7])
                 : "memory");
}

/* MODE 0: gate_up + SwiGLU;  MODE 1: down */
template <int MODE>
__global__ void __launch_bounds__(MODE == 0 ? PP_THREADS_GU : PP_THREADS, 1)
pair_gemm_kernel(const __grid_constant__ PairMaps mapA,        /* xg | act   (tokens) */
                 const __grid_constant__ PairMaps mapAs,       /* x  | sa */
                 const __grid_constant__ CUtensorMap mapB,     /* routed weights */
                 const __grid_constant__ CUtensorMap mapBs,    /* shared g | d */
                 const __grid_constant__ CUtensorMap mapBs2,   /* shared u */
                 const __grid_constant__ CUtensorMap mapG,     /* block input, 64 x 1 boxes */
                 PairParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int STAGES = PP_STAGES;
    extern __shared__ unsigned char pp_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(pp_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * PP_STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + STAGES;
    uint64_t *tfull = bars + 2 * STAGES, *tempty = tfull + 2;
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = pp_cta_rank();
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            /* the producer's expect_tx arrival, plus the stage's gather warp of
             * each CTA when they bring the token rows */
            mbar_init(&full[s], 1 + (MODE == 0 && p.wgather_tk ? 2 : 0));
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], 2 * PP_EPI_WARPS);   /* the epilogue warps of both CTAs */
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 1) pp_tmem_alloc(tmem_holder, PP_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    pp_cluster_sync();       /* the peer's barriers exist before anything signals them */
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int n_tiles = *p.n_tiles;
    const int num_kb = p.K / PP_BK;

    if (warp == 0) {
        /* ---------------- TMA producer (both CTAs; the whole warp when the
         *                  token rows are gathered by index) ---------------- */
        uint32_t kiter = 0;
        bool alive = true;
        /* operand coordinates of a tile for this CTA */
        struct Ops {
            const CUtensorMap *ma, *mb;
            int arow, brow, n_mine, n0, n1;
            bool mine, shared;
        };
        auto ops_of = [&](const int4 t) -> Ops {
            Ops o;
            o.shared = t.x == p.E;
            /* this CTA's share of the tile's rows and the box that covers it */
            o.n0 = pp_rows_of(t.w, 0);
            o.n1 = pp_rows_of(t.w, 1);
            o.n_mine = rank ? o.n1 : o.n0;
            const int hb_mine = (o.n_mine + 31) >> 5;
            o.ma = o.shared ? &mapAs.m[hb_mine ? hb_mine - 1 : 0]
                            : &mapA.m[hb_mine ? hb_mine - 1 : 0];
            if (MODE == 0) {
                o.mb = o.shared ? (rank ? &mapBs2 : &mapBs) : &mapB;
                o.brow = (o.shared ? 0
                                   : (t.x - p.e_begin) * p.rows_per_expert +
                                         (rank ? p.up_off : 0)) +
                         t.y * 128;
            } else {
                o.mb = o.shared ? &mapBs : &mapB;
                o.brow = (o.shared ? 0 : (t.x - p.e_begin) * p.rows_per_expert) +
                         t.y * PP_BN + (int)rank * 128;
            }
            o.arow = t.z + (rank ? o.n0 : 0);
            /* a CTA without a row of the tile skips the token load */
            o.mine = o.n_mine > 0;
            return o;
        };
        for (int tile = pair; alive && tile < n_tiles; tile += npairs) {
            const Ops o = ops_of(__ldg(&p.tiles[tile]));
            const bool gath = MODE == 0 && p.gather_tk > 0 && !o.shared;
            const bool wg = MODE == 0 && p.wgather_tk > 0;   /* rows come from the gather warps */
            /* lane l fetches rows 4l .. 4l+3 of this CTA's share */
            int g4[4] = {0, 0, 0, 0};
            const int ng_mine = (o.n_mine + 3) >> 2;
            if (gath && lane < ng_mine) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int rr = 4 * lane + j;
                    if (rr < o.n_mine) g4[j] = __ldg(&p.perm[o.arow + rr]) / p.gather_tk;
                }
            }
            const uint32_t bytes_all =
                (uint32_t)(2 * PP_HALF_BYTES) +
                (wg ? 0u : gath ? (uint32_t)(((o.n0 + 3) >> 2) + ((o.n1 + 3) >> 2)) * 4u * PP_BK * 2u
                      : (uint32_t)(((o.n0 + 31) >> 5) + ((o.n1 + 31) >> 5)) * 32u * PP_BK * 2u);
            for (int kb = 0; alive && kb < num_kb; kb++, kiter++) {
                const int s = kiter % STAGES;
                const uint32_t ph = (kiter / STAGES) & 1u;
                int ok = 1;
                if (lane == 0)
                    ok = pg_wait(&empty[s], ph ^ 1u, abort_flag, p.status, ST_MBAR_TIMEOUT) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    alive = false;
                    break;
                }
                unsigned char *st = smem + (size_t)s * PP_STAGE_BYTES;
                if (lane == 0) {
                    if (rank == 0) mbar_expect_tx(&full[s], bytes_all);
                    if (!gath && !wg && o.mine)
                        pp_tma_load(st, o.ma, kb * PP_BK, o.arow, &full[s]);
                    pp_tma_load(st + PP_HALF_BYTES, o.mb, kb * PP_BK, o.brow, &full[s]);
                }
                if (gath && lane < ng_mine)
                    pp_tma_gather4(st + (size_t)lane * 4 * PP_BK * 2, &mapG, kb * PP_BK, g4[0],
                                   g4[1], g4[2], g4[3], &full[s]);
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issuer (leader CTA only) ---------------- */
        if (rank == 0 && lane == 0) {
            uint32_t kiter = 0;
            bool alive = true;
            const uint32_t idesc = pp_idesc(2 * PP_BM, PP_BN);
            int it = 0;
            for (int tile = pair; alive && tile < n_tiles; tile += npairs, it++) {
                const int acc = it & 1;
                const uint32_t aph = (uint32_t)(it >> 1) & 1u;
                if (!pg_wait(&tempty[acc], aph ^ 1u, abort_flag, p.status, ST_TMEM_TIMEOUT))
                    break;
                tc_fence_after();
                const uint32_t d0 = tmem_base + (uint32_t)acc * 256u;
                for (int kb = 0; kb < num_kb; kb++, kiter++) {
                    const int s = kiter % STAGES;
                    const uint32_t ph = (kiter / STAGES) & 1u;
                    if (!pp_wait_cluster(&full[s], ph, abort_flag, p.status, ST_MBAR_TIMEOUT)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * PP_STAGE_BYTES);
                    const uint64_t da = umma_smem_desc(sa);
                    const uint64_t db = umma_smem_desc(sa + PP_HALF_BYTES);
#pragma unroll
                    for (int k = 0; k < PP_BK / 16; k++)
                        pp_mma(d0, da + 2u * k, db + 2u * k, idesc, (kb | k) ? 1u : 0u);
                    pp_commit_both(&empty[s]);       /* frees the stage in both CTAs */
                }
                if (alive) pp_commit_both(&tfull[acc]);
            }
        }
    } else if (MODE == 0 && warp >= 2 + PP_EPI_WARPS) {
        /* ---------------- gather warps (gate_up, both CTAs) ----------------
         * Per k-block the CTA's 128 rows x 128 bytes are fetched as 16-byte
         * units and land at (unit ^ (row & 7)) of their row — the 128-byte
         * swizzle the MMA's descriptor expects.  Generic-proxy writes become
         * visible to the tensor core through fence.proxy.async in the writer,
         * before the warp's arrival on the leader CTA's full barrier. */
        if (p.wgather_tk > 0) {
            /* One warp per pipeline stage: warp w brings the rows of every
             * PP_GATHER_WARPS-th k-block into stage w, so that a warp has one
             * k-block of cp.async in flight at a time (fence.proxy.async waits
             * for all of a thread's outstanding copies: issuing ahead within a
             * thread buys nothing) while the CTA has six.  Eight lanes share a
             * row (16 bytes each, one whole 128-byte line), four rows an
             * instruction, 32 instructions a k-block. */
            const int gw = warp - 2 - PP_EPI_WARPS, sub = lane >> 3, ch = lane & 7;
            int *tok = reinterpret_cast<int *>(smem + (size_t)STAGES * PP_STAGE_BYTES + 256) +
                       gw * PP_BM;
            const int my_tiles = pair < n_tiles ? (n_tiles - pair + npairs - 1) / npairs : 0;
            const uint32_t total = (uint32_t)my_tiles * (uint32_t)num_kb;
            int cur = -1, n_mine = 0;
            const uint32_t st0 = smem_u32(smem + (size_t)gw * PP_STAGE_BYTES);
            for (uint32_t it = (uint32_t)gw; it < total; it += PP_GATHER_WARPS) {
                const int tile_of = (int)(it / (uint32_t)num_kb),
                          kb = (int)(it - (uint32_t)tile_of * (uint32_t)num_kb);
                if (tile_of != cur) {
                    cur = tile_of;
                    const int4 t = __ldg(&p.tiles[pair + tile_of * npairs]);
                    const int n0 = pp_rows_of(t.w, 0);
                    n_mine = rank ? t.w - n0 : n0;
                    __syncwarp();
                    for (int g = lane; g < n_mine; g += 32) {
                        const int r = t.z + (rank ? n0 : 0) + g;
                        tok[g] = t.x == p.E ? r : __ldg(&p.perm[r]) / p.wgather_tk;
                    }
                    __syncwarp();
                }
                const uint32_t ph = (it / STAGES) & 1u;
                int ok = 1;
                if (lane == 0)
                    ok = pg_wait(&empty[gw], ph ^ 1u, abort_flag, p.status, ST_MBAR_TIMEOUT) ? 1
                                                                                             : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint16_t *col = p.x + (size_t)kb * PP_BK + ch * 8;
#pragma unroll 8
                for (int j = 0; j < PP_BM / 4; j++) {
                    const int g = j * 4 + sub;
                    if (g < n_mine)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                                         st0 + (uint32_t)(g * 128 + ((ch ^ (g & 7)) << 4))),
                                     "l"(col + (size_t)tok[g] * p.K)
                                     : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) pp_arrive_leader(&full[gw]);
            }
        }
    } else {
        /* ---------------- epilogue (warps 2..9, both CTAs) ---------------- */
        const int q = warp & 3;                 /* TMEM lane quarter of this warp */
        const int half = (warp - 2) >> 2;       /* which columns of the tile */
        const int rl = q * 32 + lane;           /* this thread's row among the CTA's rows */
        int it = 0;
        for (int tile = pair; tile < n_tiles; tile += npairs, it++) {
            const int4 t = __ldg(&p.tiles[tile]);
            const bool shared = t.x == p.E;
            const int acc = it & 1;
            const uint32_t aph = (uint32_t)(it >> 1) & 1u;
            const int n_mine = pp_rows_of(t.w, (int)rank);
            const int r = (rank ? pp_rows_of(t.w, 0) : 0) + rl;   /* row inside the tile */
            const bool valid = rl < n_mine;
            int orow = t.z + r;                 /* gate_up, and the shared expert */
            if (MODE == 1 && !shared && valid) orow = __ldg(&p.perm[t.z + r]);
            if (!pg_wait(&tfull[acc], aph, abort_flag, p.status, ST_TMEM_TIMEOUT)) break;
            tc_fence_after();
            const uint32_t taddr =
                tmem_base + (uint32_t)acc * 256u + ((uint32_t)(q * 32) << 16);
            uint16_t *out = shared ? p.out_shared : p.out_routed;
            const int ld = shared ? p.ld_shared : p.ld_routed;
            /* a warp whose rows are all past the tile's end has nothing to read */
            const bool any = q * 32 < n_mine;
            if (MODE == 0) {
                for (int c0 = half * 64; any && c0 < half * 64 + 64; c0 += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + (uint32_t)c0, g);
                    tmem_ld32(taddr + 128u + (uint32_t)c0, u);
                    tmem_ld_wait();
                    if (valid) {
                        uint16_t *dst = out + (size_t)orow * ld + t.y * 128 + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            uint32_t pk[8];
#pragma unroll
                            for (int h = 0; h < 8; h++) {
                                float g0 = __uint_as_float(g[j + 2 * h]),
                                      g1 = __uint_as_float(g[j + 2 * h + 1]),
                                      u0 = __uint_as_float(u[j + 2 * h]),
                                      u1 = __uint_as_float(u[j + 2 * h + 1]);
                                bf16_round2(g0, g1);
                                bf16_round2(u0, u1);
                                pk[h] = shared ? silu_mul_pack2(g0, u0, g1, u1)
                                               : silu_act_pack2(g0, u0, g1, u1);
                            }
                            st32(dst + j, pk);
                        }
                    }
                }
            } else {
                /* the row's home: this GPU's buffer, or the source rank's */
                uint16_t *out_row = out + (size_t)orow * ld;
                if (p.peer_dst && !shared && valid) {
                    const int s = orow / p.peer_cap;
                    out_row = reinterpret_cast<uint16_t *>(__ldg(p.peer_dst + s)) +
                              (size_t)(orow - s * p.peer_cap) * ld;
                }
                if (p.peer_dst && !shared) {
                    /* A thread owns a row, so a warp's store would touch 32 rows
                     * with 32 bytes each: fine for local memory, where L2 merges
                     * sectors, poor as NVLink packets.  The warp turns its 32 x 64
                     * chunk round in shared memory (16-byte units, XOR-swizzled by
                     * row) and stores it as 128 contiguous bytes per row, four
                     * rows an instruction. */
                    unsigned char *stg = smem + (size_t)STAGES * PP_STAGE_BYTES + 256 +
                                         (size_t)(warp - 2) * 4096;
                    const unsigned long long my_row =
                        valid ? (unsigned long long)reinterpret_cast<uintptr_t>(out_row) : 0ull;
                    for (int c0 = half * 128; any && c0 < half * 128 + 128; c0 += 64) {
                        uint32_t v[32], v2[32];
                        tmem_ld32(taddr + (uint32_t)c0, v);
                        tmem_ld32(taddr + (uint32_t)c0 + 32u, v2);
                        tmem_ld_wait();
#pragma unroll
                        for (int h8 = 0; h8 < 8; h8++) {
                            const uint32_t *f = h8 < 4 ? v + 8 * h8 : v2 + 8 * (h8 - 4);
                            uint4 q4;
                            q4.x = pack_bf16_rn(__uint_as_float(f[0]), __uint_as_float(f[1]));
                            q4.y = pack_bf16_rn(__uint_as_float(f[2]), __uint_as_float(f[3]));
                            q4.z = pack_bf16_rn(__uint_as_float(f[4]), __uint_as_float(f[5]));
                            q4.w = pack_bf16_rn(__uint_as_float(f[6]), __uint_as_float(f[7]));
                            *reinterpret_cast<uint4 *>(stg + lane * 128 +
                                                       ((h8 ^ (lane & 7)) << 4)) = q4;
                        }
                        __syncwarp();
#pragma unroll
                        for (int it = 0; it < 8; it++) {
                            const int rr = it * 4 + (lane >> 3), ch = lane & 7;
                            const unsigned long long rp = __shfl_sync(0xffffffffu, my_row, rr);
                            const uint4 q4 = *reinterpret_cast<const uint4 *>(
                                stg + rr * 128 + ((ch ^ (rr & 7)) << 4));
                            if (rp)
                                *reinterpret_cast<uint4 *>(
                                    reinterpret_cast<unsigned char *>((uintptr_t)rp) +
                                    (size_t)(t.y * PP_BN + c0) * 2 + (ch << 4)) = q4;
                        }
                        __syncwarp();
                    }
                } else
                for (int c0 = half * 128; any && c0 < half * 128 + 128; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (valid) {
                        uint16_t *dst = out_row + t.y * PP_BN + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            uint32_t pk[8];
#pragma unroll
                            for (int h = 0; h < 8; h++)
                                pk[h] = pack_bf16_rn(__uint_as_float(v[j + 2 * h]),
                                                     __uint_as_float(v[j + 2 * h + 1]));
                            st32(dst + j, pk);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) pp_arrive_leader(&tempty[acc]);
        }
    }
    /* neither CTA may leave (or free its tensor memory) while the other can
     * still signal its barriers or have MMAs in flight into its TMEM */
    tc_fence_before();
    __syncthreads();
    pp_cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        pp_tmem_dealloc(tmem_base, PP_TMEM_COLS);
    }
}

/* ---- host side ---------------------------------------------------------------- */
inline int g_pp_enable = 1;          /* APUS_CUDA_PAIR=0: never take this path */
inline int g_pp_min_rows = 192;      /* mean rows per resident expert from which it is taken */
inline int g_pp_solo_below = 160;    /* APUS_CUDA_PAIR_SOLO_BELOW: see build_hybrid_tiles_kernel
                                      * (0: every chunk to the pair kernels) */
inline int g_pp_gather = 0;          /* APUS_CUDA_PAIR_GATHER: how gate_up gets its token rows.
                                      * 0: permuted copy + TMA (fastest measured);
                                      * 1: TMA gather4 from the block input (2.4x slower:
                                      *    32 four-row requests per k-block);
                                      * 2: the kernel's gather warps, cp.async into the
                                      *    swizzled stage (gate_up 1.4x slower, no copy) */

inline bool pair_supported(const ApusCudaMoeCfg &c, int sm_count, int smem_optin) {
    return g_pp_enable && prefill_supported(c) && c.hidden % PP_BN == 0 &&
           sm_count >= 2 && pp_smem_bytes() <= smem_optin;
}

/* tile shapes of this path for the common tile-list builder */
inline TilePlan pair_tile_plan(const ApusCudaMoeCfg &c, int T, bool do_shared, int A,
                               void *tiles_ws) {
    TilePlan p = prefill_tile_plan(c, T, do_shared, A, tiles_ws);
    p.m_gu = (int)c.moe_inter / 128;
    p.m_gu_sh = (int)c.shared_inter / 128;
    p.m_dn = (int)c.hidden / PP_BN;
    p.bn_gu = p.bn_dn = p.bn_sh_gu = p.bn_sh_dn = 2 * PP_BM;
    return p;
}


/* ---- tile lists for the two-SM path ------------------------------------------
 * The pair's MMA always spans 256 token rows, so a tile with few rows wastes
 * tensor work (and, under the power cap, clock).  An expert's rows are therefore
 * cut into chunks of 256; a last chunk of at least `solo_below` rows still goes
 * to the pair kernels, a smaller remainder goes to the one-SM kernels of
 * prefill_gemm.cuh, whose MMA is exactly as wide as the rows it is given.
 * Four lists: pair gate_up / down (shared-expert tiles first), one-SM gate_up /
 * down (remainders only).  One CTA of 1024 threads, thread e = expert e. */
struct HybridLists {
    int4 *pair_gu, *pair_dn, *solo_gu, *solo_dn;
    int *n_pair_gu, *n_pair_dn, *n_solo_gu, *n_solo_dn;
    int *sched;              /* two counters of the one-SM kernels' tile hand-out */
};
struct HybridPlan {
    int T;                   /* tokens of the shared expert (0: none) */
    int m_gu, m_gu_sh, m_dn; /* pair N-tiles: gate_up, shared gate_up, down */
    int sm_gu, sm_dn;        /* one-SM weight-row tiles: gate_up, down */
    int solo_bn_gu, solo_bn_dn;   /* token rows per one-SM tile */
    int solo_below;          /* remainders below this many rows go to the one-SM kernels */
    HybridLists l;
};

__global__ void __launch_bounds__(1024)
build_hybrid_tiles_kernel(const int32_t *__restrict__ counts,
                          const int32_t *__restrict__ offsets, int E, HybridPlan hp) {
    pdl_enter();
    __shared__ int wt[3][32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cnt = tid < E ? counts[tid] : 0, off = tid < E ? offsets[tid] : 0;
    const int full = cnt / (2 * PP_BM), rem = cnt - full * 2 * PP_BM;
    const bool rem_pair = rem > 0 && rem >= hp.solo_below;   /* never a tile without rows */
    const int n_pair = full + (rem_pair ? 1 : 0);             /* 256-row chunks */
    const int solo = rem_pair ? 0 : rem;                      /* rows for the one-SM kernels */
    const int n_sg = (solo + hp.solo_bn_gu - 1) / hp.solo_bn_gu;
    const int n_sd = (solo + hp.solo_bn_dn - 1) / hp.solo_bn_dn;
    int inc[3] = {n_pair, n_sg, n_sd};
#pragma unroll
    for (int d = 1; d < 32; d <<= 1)
#pragma unroll
        for (int q = 0; q < 3; q++) {
            const int v = __shfl_up_sync(0xffffffffu, inc[q], d);
            if (lane >= d) inc[q] += v;
        }
    if (lane == 31)
        for (int q = 0; q < 3; q++) wt[q][warp] = inc[q];
    __syncthreads();
    int base[3] = {0, 0, 0}, total[3] = {0, 0, 0};
    for (int w = 0; w < 32; w++)
        for (int q = 0; q < 3; q++) {
            if (w < warp) base[q] += wt[q][w];
            total[q] += wt[q][w];
        }
    const int first_p = base[0] + inc[0] - n_pair, first_sg = base[1] + inc[1] - n_sg,
              first_sd = base[2] + inc[2] - n_sd;
    const int nts = (hp.T + 2 * PP_BM - 1) / (2 * PP_BM);
    const int sh_gu = nts * hp.m_gu_sh, sh_dn = nts * hp.m_dn;
    const HybridLists &l = hp.l;
    if (tid < E) {
        for (int n = 0; n < n_pair; n++) {
            const int rows = min(2 * PP_BM, cnt - n * 2 * PP_BM), r0 = off + n * 2 * PP_BM;
            for (int m = 0; m < hp.m_gu; m++)
                l.pair_gu[(size_t)sh_gu + (size_t)(first_p + n) * hp.m_gu + m] =
                    make_int4(tid, m, r0, rows);
            for (int m = 0; m < hp.m_dn; m++)
                l.pair_dn[(size_t)sh_dn + (size_t)(first_p + n) * hp.m_dn + m] =
                    make_int4(tid, m, r0, rows);
        }
        const int s0 = off + full * 2 * PP_BM;
        for (int m = 0; m < hp.sm_gu; m++)
            for (int n = 0; n < n_sg; n++)
                l.solo_gu[(size_t)first_sg * hp.sm_gu + (size_t)m * n_sg + n] = make_int4(
                    tid, m, s0 + n * hp.solo_bn_gu, min(hp.solo_bn_gu, solo - n * hp.solo_bn_gu));
        for (int m = 0; m < hp.sm_dn; m++)
            for (int n = 0; n < n_sd; n++)
                l.solo_dn[(size_t)first_sd * hp.sm_dn + (size_t)m * n_sd + n] = make_int4(
                    tid, m, s0 + n * hp.solo_bn_dn, min(hp.solo_bn_dn, solo - n * hp.solo_bn_dn));
    }
    for (int i = tid; i < sh_gu; i += blockDim.x) {
        const int n = i / hp.m_gu_sh, m = i - n * hp.m_gu_sh;
        l.pair_gu[i] = make_int4(E, m, n * 2 * PP_BM, min(2 * PP_BM, hp.T - n * 2 * PP_BM));
    }
    for (int i = tid; i < sh_dn; i += blockDim.x) {
        const int n = i / hp.m_dn, m = i - n * hp.m_dn;
        l.pair_dn[i] = make_int4(E, m, n * 2 * PP_BM, min(2 * PP_BM, hp.T - n * 2 * PP_BM));
    }
    if (tid == 0) {
        *l.n_pair_gu = sh_gu + total[0] * hp.m_gu;
        *l.n_pair_dn = sh_dn + total[0] * hp.m_dn;
        *l.n_solo_gu = total[1] * hp.sm_gu;
        *l.n_solo_dn = total[2] * hp.sm_dn;
        l.sched[0] = 0;
        l.sched[1] = 0;
    }
}

/* xg rows of the one-SM lists only (the SM pairs fetch their rows themselves):
 * every gate_up tile of weight-row tile 0 names one run of rows. */
__global__ void __launch_bounds__(256)
gather_solo_rows_kernel(const uint16_t *__restrict__ x, const int32_t *__restrict__ perm,
                        const int4 *__restrict__ tiles, const int *__restrict__ n_tiles, int H,
                        int TK, uint16_t *__restrict__ xg) {
    pdl_enter();
    const int n = *n_tiles, c8 = H / 8;
    for (int i = blockIdx.x; i < n; i += gridDim.x) {
        const int4 t = tiles[i];
        if (t.y != 0) continue;
        for (int j = threadIdx.x; j < t.w * c8; j += blockDim.x) {
            const int r = t.z + j / c8, c = j % c8;
            const int tok = perm[r] / TK;
            reinterpret_cast<uint4 *>(xg)[(size_t)r * c8 + c] =
                ldg16(x + (size_t)tok * H + (size_t)c * 8);
        }
    }
}

/* list storage inside the block's tile workspace (prefill_tiles_bytes_for) */
inline bool hybrid_plan(const ApusCudaMoeCfg &c, int T, bool do_shared, int A, void *ws,
                        size_t ws_bytes, HybridPlan *out) {
    const int H = (int)c.hidden, I = (int)c.moe_inter, Is = (int)c.shared_inter,
              E = (int)c.experts;
    HybridPlan p;
    memset(&p, 0, sizeof p);
    p.T = do_shared ? T : 0;
    p.m_gu = I / 128;
    p.m_gu_sh = Is / 128;
    p.m_dn = H / PP_BN;
    p.sm_gu = I / PG_BM;
    p.sm_dn = H / PG_BM;
    p.solo_bn_gu = PG_BN_GU;
    p.solo_bn_dn = PG_BN_DN;
    p.solo_below = g_pp_solo_below;
    const size_t chunks = (size_t)A / (2 * PP_BM) + E + (size_t)T / (2 * PP_BM) + 1;
    const size_t n_pg = chunks * (size_t)(p.m_gu > p.m_gu_sh ? p.m_gu : p.m_gu_sh),
                 n_pd = chunks * p.m_dn, n_sg = (size_t)E * 2 * p.sm_gu,
                 n_sd = (size_t)E * p.sm_dn;
    if ((n_pg + n_pd + n_sg + n_sd) * sizeof(int4) + 64 > ws_bytes) return false;
    p.l.pair_gu = reinterpret_cast<int4 *>(ws);
    p.l.pair_dn = p.l.pair_gu + n_pg;
    p.l.solo_gu = p.l.pair_dn + n_pd;
    p.l.solo_dn = p.l.solo_gu + n_sg;
    p.l.n_pair_gu = reinterpret_cast<int *>(p.l.solo_dn + n_sd);
    p.l.n_pair_dn = p.l.n_pair_gu + 1;
    p.l.n_solo_gu = p.l.n_pair_gu + 2;
    p.l.n_solo_dn = p.l.n_pair_gu + 3;
    p.l.sched = p.l.n_pair_gu + 4;
    *out = p;
    return true;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pair(void (*kernel)(KArgs...), int grid, int threads, size_t smem,
                               cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_apus_use_pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

/* Routed + shared experts through the two-SM kernels.  Same contract as
 * run_prefill_experts; the tile lists come from build_tiles_kernel with
 * pair_tile_plan's shapes. */
inline int run_pair_experts(int sm_count, int smem_optin, PrefillMaps *maps,
                            const ApusCudaMoeCfg &c, int e_begin, const uint16_t *x, int T,
                            int A, int TK, bool do_shared, const DispatchOut &d,
                            uint16_t *xg, uint16_t *act, uint16_t *sa, uint16_t *eo,
                            uint16_t *sy, void *tiles_ws, int *status, cudaStream_t st,
                            int *launches, void (*mark)(int stage),
                            const PeerRows *peer = nullptr) {
    const int H = (int)c.hidden, I = (int)c.moe_inter, Is = (int)c.shared_inter,
              E = (int)c.experts;
    if (!maps) {
        snprintf(g_prefill_err, sizeof g_prefill_err, "tensor maps missing");
        return 1;
    }
    const int smem = pp_smem_bytes(), smem_dn = pp_smem_bytes(peer != nullptr);
    if (smem_dn > smem_optin || Is != I) {
        snprintf(g_prefill_err, sizeof g_prefill_err,
                 "two-SM grouped GEMM: %d B shared memory, shared_inter == moe_inter", smem);
        return 1;
    }
    HybridPlan plan;
    if (!hybrid_plan(c, T, do_shared, A, tiles_ws,
                     prefill_tiles_bytes_for(c, (size_t)A, (size_t)T), &plan)) {
        snprintf(g_prefill_err, sizeof g_prefill_err, "tile workspace too small");
        return 1;
    }
    launch_k(build_hybrid_tiles_kernel, dim3(1), dim3(1024), 0, st,
             (const int32_t *)d.counts, (const int32_t *)d.offsets, E, plan);
    (*launches)++;
    const HybridLists tl = plan.l;
    const bool solo = plan.solo_below > 0 && A > 0;
    /* the one-SM kernels read the permuted copy, so it is made whenever they run */
    const bool gather = g_pp_gather == 1 && !solo && !peer;
    /* the SM pairs' gather warps read the block input themselves; a permuted
     * copy is made of the one-SM lists' rows only */
    const bool wgather = g_pp_gather == 2 && !peer && A > 0;
    if (wgather && solo) {
        launch_k(gather_solo_rows_kernel, dim3(sm_count * 4), dim3(256), 0, st, x,
                 (const int32_t *)d.perm, (const int4 *)tl.solo_gu, (const int *)tl.n_solo_gu, H,
                 TK, xg);
        (*launches)++;
    }
    if (A > 0 && !gather && !wgather) {
        long total = (long)A * (H / 8);
        int blocks = (int)((total + 255) / 256);
        if (blocks > sm_count * 16) blocks = sm_count * 16;
        if (peer)
            launch_k(gather_rows_peer_kernel, dim3(blocks), dim3(256), 0, st, peer->src,
                     peer->cap, (const int32_t *)d.perm, A, H, TK, xg,
                     (const int32_t *)(d.offsets + E));
        else
            launch_k(gather_rows_kernel, dim3(blocks), dim3(256), 0, st, x, d.perm, A, H, TK,
                     xg, (const int32_t *)(d.offsets + E));
        (*launches)++;
    }
    if (mark) mark(APUS_CUDA_STAGE_GATHER);
    PairMaps m_xg, m_x, m_act, m_sa;
    CUtensorMap m_g;
    int bad = encode_2d(maps->encode, &m_g, x, (size_t)(T > 0 ? T : 1), H, 1);
    for (int h = 0; h < 4; h++) {
        const int box = 32 * (h + 1);
        bad |= encode_2d(maps->encode, &m_xg.m[h],
                         A > 0 && !gather ? (const void *)xg : (const void *)x,
                         (size_t)(A > 0 && !gather ? A : (T > 0 ? T : 1)), H, box);
        bad |= encode_2d(maps->encode, &m_x.m[h], x, (size_t)(T > 0 ? T : 1), H, box);
        bad |= encode_2d(maps->encode, &m_act.m[h],
                         A > 0 ? (const void *)act : (const void *)sa, (size_t)(A > 0 ? A : 1),
                         I, box);
        bad |= encode_2d(maps->encode, &m_sa.m[h],
                         do_shared ? (const void *)sa : (const void *)x,
                         (size_t)(do_shared && T > 0 ? T : 1), Is, box);
    }
    if (bad) return 1;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(pair_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem);
        cudaFuncSetAttribute(pair_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             pp_smem_bytes(true) <= smem_optin ? pp_smem_bytes(true) : smem);
        attr_set = true;
    }
    const int grid = sm_count & ~1;
    PairParams p1;
    memset(&p1, 0, sizeof p1);
    p1.tiles = tl.pair_gu;
    p1.n_tiles = tl.n_pair_gu;
    p1.K = H;
    p1.E = E;
    p1.e_begin = e_begin;
    p1.rows_per_expert = 2 * I;
    p1.up_off = I;
    p1.out_routed = act;
    p1.out_shared = sa;
    p1.ld_routed = I;
    p1.ld_shared = Is;
    p1.perm = d.perm;
    p1.status = status;
    /* the one-SM kernels for the small remainders */
    CUtensorMap s_xg, s_act;
    GemmParams g1;
    memset(&g1, 0, sizeof g1);
    if (solo) {
        const int s1 = pg_smem_bytes(true);
        if (encode_2d(maps->encode, &s_xg, xg, (size_t)A, H, PG_BN_GU) ||
            encode_2d(maps->encode, &s_act, act, (size_t)A, I, PG_BN_DN))
            return 1;
        cudaFuncSetAttribute(grouped_gemm_kernel<0>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, s1);
        cudaFuncSetAttribute(grouped_gemm_kernel<1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, s1);
        g1.tiles = tl.solo_gu;
        g1.n_tiles = tl.n_solo_gu;
        g1.K = H;
        g1.E = E;
        g1.e_begin = e_begin;
        g1.rows_per_expert = 2 * I;
        g1.up_off = I;
        g1.out_routed = act;
        g1.out_shared = sa;
        g1.ld_routed = I;
        g1.ld_shared = Is;
        g1.status = status;
        g1.bn_rows = PG_BN_GU;
        g1.perm = d.perm;
        g1.sched = tl.sched;
    }
    p1.gather_tk = gather && A > 0 ? TK : 0;
    p1.wgather_tk = wgather ? TK : 0;
    p1.x = x;
    launch_pair(pair_gemm_kernel<0>, grid, PP_THREADS_GU, (size_t)smem, st, m_xg, m_x, maps->w_gu, maps->sh_g,
                maps->sh_u, m_g, p1);
    (*launches)++;
    if (solo) {
        launch_k(grouped_gemm_kernel<0>, dim3(sm_count), dim3(PG_THREADS),
                 (size_t)pg_smem_bytes(true), st, maps->w_gu, maps->sh_g, maps->sh_u, s_xg,
                 s_xg, g1);
        (*launches)++;
    }
    if (mark) mark(APUS_CUDA_STAGE_GATE_UP);
    PairParams p2 = p1;
    p2.tiles = tl.pair_dn;
    p2.n_tiles = tl.n_pair_dn;
    p2.K = I;
    p2.rows_per_expert = H;
    p2.up_off = 0;
    p2.out_routed = eo;
    p2.out_shared = sy;
    p2.ld_routed = H;
    p2.ld_shared = H;
    p2.gather_tk = 0;
    p2.wgather_tk = 0;
    p2.peer_dst = peer ? peer->dst : nullptr;
    p2.peer_cap = peer ? peer->cap : 0;
    launch_pair(pair_gemm_kernel<1>, grid, PP_THREADS, (size_t)smem_dn, st, m_act, m_sa, maps->w_d, maps->sh_d,
                maps->sh_d, m_g, p2);
    (*launches)++;
    if (solo) {
        GemmParams g2 = g1;
        g2.tiles = tl.solo_dn;
        g2.n_tiles = tl.n_solo_dn;
        g2.K = I;
        g2.rows_per_expert = H;
        g2.up_off = 0;
        g2.out_routed = eo;
        g2.out_shared = sy;
        g2.ld_routed = H;
        g2.ld_shared = H;
        g2.bn_rows = PG_BN_DN;
        g2.sched = tl.sched + 1;
        g2.peer_dst = p2.peer_dst;
        g2.peer_cap = p2.peer_cap;
        launch_k(grouped_gemm_kernel<1>, dim3(sm_count), dim3(PG_THREADS),
                 (size_t)pg_smem_bytes(false), st, maps->w_d, maps->sh_d, maps->sh_d, s_act,
                 s_act, g2);
        (*launches)++;
    }
    if (mark) mark(APUS_CUDA_STAGE_DOWN);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(g_prefill_err, sizeof g_prefill_err, "two-SM grouped GEMM launch: %s",
                 cudaGetErrorString(e));
        return 1;
    }
    return 0;
}

}  // namespace apus
