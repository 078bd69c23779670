/*
 * dispatch.cuh — token-to-expert dispatch: histogram, prefix sum, STABLE
 * permutation.
 *
 * The CPU engine never materialises a permutation; its batched body scans all
 * assignments once per expert (c/layer.h:599-606) and scatters results back
 * with a second scan (c/layer.h:614-620).  The order those loops imply is:
 * experts ascending; inside an expert, tokens ascending, then slots
 * ascending — i.e. a stable counting sort of the flat assignment index
 * a = t*topk + j by expert id.  These kernels produce exactly that order
 * (atomics are used for counts only, never for placement):
 *
 *   counts[e], offsets[e] (exclusive, offsets[E] = T*topk),
 *   perm[p]  = flat assignment sitting at sorted position p,
 *   pos[a]   = sorted position of flat assignment a (inverse of perm).
 *
 * Work unit = 256 consecutive assignments handled by one warp in 8 ordered
 * steps of 32; __match_any_sync ranks equal keys inside a step by lane, a
 * per-warp cursor carries the rank across steps, and a scan over
 * (expert, unit) gives every unit its base — so placement is deterministic
 * and stable at any grid size.
 *
 * The same pass also emits the token groups the decode kernels iterate:
 * every expert's rows cut into groups of at most GROUP_TOKENS.
 */
#pragma once
#include "common.cuh"

namespace apus {

constexpr int DISPATCH_UNIT = 256;      /* assignments per warp */
constexpr int DISPATCH_WARPS = 8;       /* warps per block */
constexpr int GROUP_TOKENS = 4;         /* rows per decode token group */

/* The sort key of an assignment is (idx - key_base) / key_div: plain expert
 * ids for the block (0, 1), expert ids local to a rank's slice (begin, 1), or
 * the owning rank under expert parallelism (0, experts per rank). */
struct DispatchKey {
    int base;
    int div;
    int lax;     /* > 0: ids outside [base, base + lax * div) are someone else's, skipped
                  * like empty slots (a rank sorting every rank's ids for its own experts) */
};
/* An id of -1 is an empty slot: skipped without complaint (key -2).  Any other
 * id outside the key range is an error (key -1 or >= E) unless the key is lax. */
__device__ __forceinline__ int dispatch_key(int raw, DispatchKey kx) {
    if (raw == -1) return -2;
    const int v = raw - kx.base;
    if (kx.lax > 0 && (v < 0 || v / kx.div >= kx.lax)) return -2;
    return v < 0 ? -1 : v / kx.div;
}

struct DispatchOut {
    int32_t *counts;     /* [E] */
    int32_t *offsets;    /* [E+1] */
    int32_t *perm;       /* [A] */
    int32_t *pos;        /* [A]  (may be NULL) */
    int32_t *grp_expert; /* [<= A] expert of each token group (may be NULL) */
    int32_t *grp_first;  /* [<= A] first sorted position of the group */
    int32_t *grp_n;      /* [<= A] rows in the group (1..GROUP_TOKENS) */
    int32_t *n_groups;   /* [1] */
};

/* ---- tile list --------------------------------------------------------------
 * One entry per (expert, weight-row tile, token-row tile): {v, m, row0, nrows}.
 * v == E is the shared expert (rows are token indices); otherwise row0 is a
 * position in dispatch order.  Tiles that share weights are adjacent, so when
 * an expert has several token tiles its weights come from HBM once and from
 * L2 afterwards. */
struct TileLists {
    int4 *gu;        /* gate_up tiles */
    int4 *dn;        /* down tiles */
    int *n_gu, *n_dn;
    /* per expert (index E: the shared expert): gate_up tiles finished so far
     * (counted once per epilogue warp) and how many there are */
    int *done, *need;
    /* next tile to hand out, one counter per expert kernel (gate_up, down) */
    int *sched;
};

/* What the tile lists are built from (host side fills it in) */
struct TilePlan {
    int on;                 /* 0: no tile lists wanted */
    int T;                  /* tokens the shared expert runs over (0: none) */
    int m_gu, m_gu_sh, m_dn;   /* weight-row tiles per expert: gate_up, shared gate_up, down */
    int bn_gu, bn_dn;       /* token rows per routed tile */
    int bn_sh_gu, bn_sh_dn; /* token rows per shared-expert tile */
    TileLists tl;
};

/* All 1024 threads of a one-CTA kernel call this with thread e < E holding
 * expert e's row count and first sorted position. */
__device__ __forceinline__ void build_tiles_body(int cnt, int off, int E, int T, int m_gu,
                                                 int m_gu_sh, int m_dn, int bn_gu,
                                                 int bn_dn, int bn_sh_gu, int bn_sh_dn,
                                                 TileLists tl) {
    __shared__ int warp_tot[2][32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nt_a = (cnt + bn_gu - 1) / bn_gu;
    const int nt_b = (cnt + bn_dn - 1) / bn_dn;
    int inc_a = nt_a, inc_b = nt_b;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int va = __shfl_up_sync(0xffffffffu, inc_a, d);
        int vb = __shfl_up_sync(0xffffffffu, inc_b, d);
        if (lane >= d) { inc_a += va; inc_b += vb; }
    }
    if (lane == 31) { warp_tot[0][warp] = inc_a; warp_tot[1][warp] = inc_b; }
    __syncthreads();
    int base_a = 0, total_a = 0, base_b = 0, total_b = 0;
    for (int w = 0; w < 32; w++) {
        if (w < warp) { base_a += warp_tot[0][w]; base_b += warp_tot[1][w]; }
        total_a += warp_tot[0][w];
        total_b += warp_tot[1][w];
    }
    const int first_a = base_a + inc_a - nt_a, first_b = base_b + inc_b - nt_b;
    /* The shared expert is dense over the tokens (always full-width tiles) and
     * its tiles come FIRST.  They are the expensive ones — wide MMAs fed from
     * L2 and a long epilogue — and at the end of the list they were the
     * kernel's tail: a few CTAs computing while HBM idles.  At the front they
     * run beside the routed tiles' weight stream. */
    const int nts_a = (T + bn_sh_gu - 1) / bn_sh_gu, nts_b = (T + bn_sh_dn - 1) / bn_sh_dn;
    const int sh_a = nts_a * m_gu_sh, sh_b = nts_b * m_dn;
    if (tid < E && cnt > 0) {
        for (int m = 0; m < m_gu; m++)
            for (int n = 0; n < nt_a; n++)
                tl.gu[(size_t)sh_a + (size_t)first_a * m_gu + (size_t)m * nt_a + n] =
                    make_int4(tid, m, off + n * bn_gu, min(bn_gu, cnt - n * bn_gu));
        for (int m = 0; m < m_dn; m++)
            for (int n = 0; n < nt_b; n++)
                tl.dn[(size_t)sh_b + (size_t)first_b * m_dn + (size_t)m * nt_b + n] =
                    make_int4(tid, m, off + n * bn_dn, min(bn_dn, cnt - n * bn_dn));
    }
    for (int i = tid; i < sh_a; i += blockDim.x) {
        int m = i / nts_a, n = i - m * nts_a;
        tl.gu[i] = make_int4(E, m, n * bn_sh_gu, min(bn_sh_gu, T - n * bn_sh_gu));
    }
    for (int i = tid; i < sh_b; i += blockDim.x) {
        int m = i / nts_b, n = i - m * nts_b;
        tl.dn[i] = make_int4(E, m, n * bn_sh_dn, min(bn_sh_dn, T - n * bn_sh_dn));
    }
    if (tid < E) {
        tl.done[tid] = 0;
        tl.need[tid] = nt_a * m_gu;
    }
    if (tid == 0) {
        tl.done[E] = 0;
        tl.need[E] = nts_a * m_gu_sh;
        tl.sched[0] = 0;
        tl.sched[1] = 0;
        tl.done[E + 1] = 0;                               /* all of them together */
        tl.need[E + 1] = total_a * m_gu + nts_a * m_gu_sh;
        *tl.n_gu = total_a * m_gu + nts_a * m_gu_sh;
        *tl.n_dn = total_b * m_dn + nts_b * m_dn;
    }
}

__global__ void __launch_bounds__(1024)
build_tiles_kernel(const int32_t *__restrict__ counts,
                   const int32_t *__restrict__ offsets, int E, TilePlan tp) {
    pdl_enter();
    const int tid = threadIdx.x;
    build_tiles_body(tid < E ? counts[tid] : 0, tid < E ? offsets[tid] : 0, E, tp.T, tp.m_gu,
                     tp.m_gu_sh, tp.m_dn, tp.bn_gu, tp.bn_dn, tp.bn_sh_gu, tp.bn_sh_dn,
                     tp.tl);
}

/* ---- small problems: one block does everything -------------------------- */
/* A <= 32 * DISPATCH_UNIT, E <= 1024; block = 1024 threads = 32 warps, each
 * warp owning one unit of up to 256 consecutive assignments.  Dynamic shared
 * memory: int [32][E] (per-warp histograms, then per-warp cursors). */
constexpr int DISPATCH_SMALL_MAX = 32 * DISPATCH_UNIT;

__global__ void __launch_bounds__(1024)
dispatch_small_kernel(const int32_t *__restrict__ idx, int A, int E,
                      DispatchKey kx, DispatchOut o, int *status, TilePlan tp) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ int sm[];          /* [32][E] */
    __shared__ int warp_tot[32];
    __shared__ int s_ngroups;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int *h = sm + warp * E;
    /* warps beyond the last unit hold no assignment: their histograms are
     * neither cleared nor summed (a handful of tokens is one unit) */
    const int units = (A + DISPATCH_UNIT - 1) / DISPATCH_UNIT;
    if (warp < units)
        for (int e = lane; e < E; e += 32) h[e] = 0;
    if (tid == 0) s_ngroups = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");   /* idx is the previous kernel's */
    __syncwarp();
    /* this warp's keys stay in registers for both passes */
    const int a_lo = warp * DISPATCH_UNIT;
    int keys[DISPATCH_UNIT / 32];
#pragma unroll
    for (int s = 0; s < DISPATCH_UNIT / 32; s++) {
        const int a = a_lo + s * 32 + lane;
        int k = (a < A) ? dispatch_key(idx[a], kx) : -1;
        if (a < A && (k == -1 || k >= E)) {
            set_status(status, ST_BAD_INDEX);
            k = -1;
        }
        keys[s] = k;
        if (k >= 0) atomicAdd(&h[k], 1);
    }
    __syncthreads();
    /* per expert: exclusive prefix over the 32 warps (in place) and total */
    int total = 0;
    for (int e = tid; e < E; e += 1024) {   /* E <= 1024: at most one e */
        int run = 0;
#pragma unroll 8
        for (int w = 0; w < units; w++) {
            int v = sm[w * E + e];
            sm[w * E + e] = run;
            run += v;
        }
        total = run;
    }
    int inc = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += v;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; w++) base += warp_tot[w];
    const int off = base + inc - total;
    if (tid < E) {
        o.counts[tid] = total;
        o.offsets[tid] = off;
        for (int w = 0; w < units; w++) sm[w * E + tid] += off;   /* cursors */
        if (o.grp_expert && total > 0) {
            int ng = (total + GROUP_TOKENS - 1) / GROUP_TOKENS;
            int g0 = atomicAdd(&s_ngroups, ng);
            /* group order is irrelevant to results */
            for (int g = 0; g < ng; g++) {
                o.grp_expert[g0 + g] = tid;
                o.grp_first[g0 + g] = off + g * GROUP_TOKENS;
                int left = total - g * GROUP_TOKENS;
                o.grp_n[g0 + g] = left < GROUP_TOKENS ? left : GROUP_TOKENS;
            }
        }
    }
    if (tid == 1023) o.offsets[E] = base + inc;   /* == number of valid keys */
    __syncthreads();
    if (tid == 0 && o.n_groups) *o.n_groups = s_ngroups;
    /* the grouped GEMMs' tile lists come out of the same counts: one launch less */
    if (tp.on)
        build_tiles_body(tid < E ? total : 0, tid < E ? off : 0, E, tp.T, tp.m_gu, tp.m_gu_sh,
                         tp.m_dn, tp.bn_gu, tp.bn_dn, tp.bn_sh_gu, tp.bn_sh_dn, tp.tl);
    /* stable placement inside each warp's unit */
#pragma unroll
    for (int s = 0; s < DISPATCH_UNIT / 32; s++) {
        const int a = a_lo + s * 32 + lane;
        const int k = keys[s];
        const bool ok = k >= 0;
        const unsigned act = __ballot_sync(0xffffffffu, ok);
        if (ok) {
            const unsigned peers = __match_any_sync(act, k);
            const int rank = __popc(peers & ((1u << lane) - 1u));
            const int dst = h[k] + rank;
            o.perm[dst] = a;
            if (o.pos) o.pos[a] = dst;
            __syncwarp(act);
            if (rank == 0) h[k] += __popc(peers);
        }
        __syncwarp();
    }
}

/* ---- large problems: three passes ---------------------------------------- */
/* pass 1: per-unit histograms, unit_hist[unit][e] */
__global__ void __launch_bounds__(DISPATCH_WARPS * 32)
dispatch_hist_kernel(const int32_t *__restrict__ idx, int A, int E,
                     DispatchKey kx, int32_t *__restrict__ unit_hist,
                     int *status) {
    pdl_enter();
    extern __shared__ int sm[];   /* [DISPATCH_WARPS][E] */
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = blockIdx.x * DISPATCH_WARPS + warp;
    int *h = sm + warp * E;
    for (int e = lane; e < E; e += 32) h[e] = 0;
    __syncwarp();
    const int a_lo = unit * DISPATCH_UNIT;
    if (a_lo < A) {
        const int a_hi = min(A, a_lo + DISPATCH_UNIT);
        for (int a = a_lo + lane; a < a_hi; a += 32) {
            int k = dispatch_key(idx[a], kx);
            if (k < 0 || k >= E) {
                if (k != -2) set_status(status, ST_BAD_INDEX);
                continue;
            }
            atomicAdd(&h[k], 1);
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32)
            unit_hist[(size_t)unit * E + e] = h[e];
    }
}

/* pass 2: one block of 1024 threads.  For each expert, exclusive prefix over
 * units (in place), totals -> counts; exclusive scan over experts -> offsets;
 * token groups.  Thread (part, e) first sums its quarter of the units, the
 * four partial sums meet in shared memory, then each thread rewrites its
 * quarter with running prefixes — four short chains of loads instead of one
 * long one.  E <= 256 takes this route; larger E the single-chain form. */
__global__ void __launch_bounds__(1024)
dispatch_scan_kernel(int32_t *__restrict__ unit_hist, int n_units, int E,
                     DispatchOut o) {
    pdl_enter();
    __shared__ int warp_tot[32];
    __shared__ int s_ngroups;
    __shared__ int part_sum[4][256];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_ngroups = 0;
    int total = 0;
    if (E <= 256) {
        const int e = tid & 255, part = tid >> 8;
        const int per = (n_units + 3) / 4;
        const int u_lo = part * per, u_hi = min(n_units, u_lo + per);
        int sum = 0;
        if (e < E) {
            for (int u0 = u_lo; u0 < u_hi; u0 += 8) {
                int v[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                    v[j] = (u0 + j < u_hi) ? unit_hist[(size_t)(u0 + j) * E + e] : 0;
#pragma unroll
                for (int j = 0; j < 8; j++) sum += v[j];
            }
        }
        part_sum[part][e] = sum;
        __syncthreads();
        int run = 0;
        for (int q = 0; q < part; q++) run += part_sum[q][e];
        if (e < E) {
            for (int u0 = u_lo; u0 < u_hi; u0 += 8) {
                int v[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                    v[j] = (u0 + j < u_hi) ? unit_hist[(size_t)(u0 + j) * E + e] : 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (u0 + j < u_hi) unit_hist[(size_t)(u0 + j) * E + e] = run;
                    run += v[j];
                }
            }
        }
        if (tid < E)
            total = part_sum[0][tid] + part_sum[1][tid] + part_sum[2][tid] +
                    part_sum[3][tid];
    } else if (tid < E) {
        for (int u0 = 0; u0 < n_units; u0 += 8) {
            int v[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                v[j] = (u0 + j < n_units)
                           ? unit_hist[(size_t)(u0 + j) * E + tid] : 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (u0 + j < n_units)
                    unit_hist[(size_t)(u0 + j) * E + tid] = total;
                total += v[j];
            }
        }
    }
    int inc = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += v;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; w++) base += warp_tot[w];
    const int off = base + inc - total;
    if (tid < E) {
        o.counts[tid] = total;
        o.offsets[tid] = off;
        if (o.grp_expert && total > 0) {
            int ng = (total + GROUP_TOKENS - 1) / GROUP_TOKENS;
            int g0 = atomicAdd(&s_ngroups, ng);
            for (int g = 0; g < ng; g++) {
                o.grp_expert[g0 + g] = tid;
                o.grp_first[g0 + g] = off + g * GROUP_TOKENS;
                int left = total - g * GROUP_TOKENS;
                o.grp_n[g0 + g] = left < GROUP_TOKENS ? left : GROUP_TOKENS;
            }
        }
    }
    if (tid == 1023) o.offsets[E] = base + inc;
    __syncthreads();
    if (tid == 0 && o.n_groups) *o.n_groups = s_ngroups;
}

/* pass 3: stable placement inside each unit */
__global__ void __launch_bounds__(DISPATCH_WARPS * 32)
dispatch_permute_kernel(const int32_t *__restrict__ idx, int A, int E,
                        DispatchKey kx, const int32_t *__restrict__ unit_hist,
                        DispatchOut o) {
    pdl_enter();
    extern __shared__ int sm[];   /* [DISPATCH_WARPS][E] cursors */
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = blockIdx.x * DISPATCH_WARPS + warp;
    const int a_lo = unit * DISPATCH_UNIT;
    if (a_lo >= A) return;
    int *cursor = sm + warp * E;
    for (int e = lane; e < E; e += 32)
        cursor[e] = o.offsets[e] + unit_hist[(size_t)unit * E + e];
    __syncwarp();
    const int a_hi = min(A, a_lo + DISPATCH_UNIT);
    for (int a0 = a_lo; a0 < a_hi; a0 += 32) {
        int a = a0 + lane;
        int k = (a < a_hi) ? dispatch_key(idx[a], kx) : -1;
        bool ok = (k >= 0 && k < E);
        unsigned act = __ballot_sync(0xffffffffu, ok);
        if (ok) {
            unsigned peers = __match_any_sync(act, k);
            int rank = __popc(peers & ((1u << lane) - 1u));
            int dst = cursor[k] + rank;
            o.perm[dst] = a;
            if (o.pos) o.pos[a] = dst;
            __syncwarp(act);
            if (rank == 0) cursor[k] += __popc(peers);
        }
        __syncwarp();
    }
}

}  // namespace apus
