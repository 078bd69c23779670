/*
 * decode_gemv.cuh — the bandwidth-bound expert path for small token counts:
 * grouped BF16 GEMV over the routed experts' and the shared expert's weights.
 *
 * Replaces, for T tokens at once, the per-slot loop of c/layer.h:344-349
 * (gate_up GEMV -> apus_moe_silu_act -> down GEMV) and the shared-expert
 * lines c/layer.h:351-354, reading each touched weight row from HBM exactly
 * once per token group:
 *
 *   gate_up kernel : for every (token group, row i):  g = rnd(Wg[i].x),
 *                    u = rnd(Wu[i].x);  routed: act = rnd(rnd(silu(g))*u)
 *                    (two roundings, c/moe.h:387-395);  shared:
 *                    sa = rnd(silu(g)*u) (one rounding, c/moe.h:438-445)
 *   down kernel    : for every (token group, row h):  y = rnd(Wd[h].act)
 *
 * Weight rows are contiguous in memory, so every work item is one or two 1-D
 * bulk copies (cp.async.bulk, no multicast) into a per-warp shared-memory
 * ring; a warp keeps DEC_STAGES-1 copies in flight while it reduces the
 * current rows with 16-byte shared loads and warp shuffles.  Each CTA owns a
 * contiguous slice of the flattened (group, row) space, so the whole grid
 * streams disjoint, contiguous weight ranges.  Dot products accumulate in
 * fp32 in lane-strided order (not the CPU anchor's sequential order): outputs
 * agree with the CPU engine to BF16 rounding, not bitwise.
 */
#pragma once
#include "common.cuh"
#include "dispatch.cuh"

namespace apus {

constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_STAGES = 3;
constexpr int DOWN_ROWS = 8;    /* weight rows per down-projection item */

struct DecodeArgs {
    int T, H, I, Is, TK;
    int expert_begin;            /* first expert resident on this GPU */
    const uint16_t *x;           /* [T, H] block input */
    const uint16_t *exp_gu;      /* resident experts, [e, 2I, H] */
    const uint16_t *exp_d;       /* resident experts, [e, H, I] */
    const uint16_t *sh_g, *sh_u; /* [Is, H] */
    const uint16_t *sh_d;        /* [H, Is] */
    const int32_t *perm;         /* [A] sorted position -> flat assignment */
    const int32_t *grp_expert, *grp_first, *grp_n, *n_groups;
    uint16_t *act;               /* [A, I] routed activations, sorted order */
    uint16_t *sa;                /* [T, Is] shared activations */
    uint16_t *eo;                /* [A, H] routed expert outputs, flat assignment order */
    uint16_t *sy;                /* [T, H] shared expert output */
    int do_shared;               /* 0: skip the shared expert's items */
    int *status;
};

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x);
    f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
    f[4] = bf16lo(v.z); f[5] = bf16hi(v.z);
    f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}

/* What an item index means.  Shared-expert groups (GROUP_TOKENS consecutive
 * tokens each) come first, then the routed token groups. */
struct ItemInfo {
    bool shared;
    int group;      /* index into the shared or the routed group list */
    int row;        /* row (gate_up) or row block (down) inside the group */
    int rows;       /* rows (or row blocks) per group of this kind */
};
__device__ __forceinline__ ItemInfo decode_item(long item, int n_sh_groups,
                                                int rows_sh, int rows_rt) {
    ItemInfo it;
    long sh_items = (long)n_sh_groups * rows_sh;
    if (item < sh_items) {
        it.shared = true;
        it.group = (int)(item / rows_sh);
        it.row = (int)(item - (long)it.group * rows_sh);
        it.rows = rows_sh;
    } else {
        long r = item - sh_items;
        it.shared = false;
        it.group = (int)(r / rows_rt);
        it.row = (int)(r - (long)it.group * rows_rt);
        it.rows = rows_rt;
    }
    return it;
}

template <int NT>
__device__ __forceinline__ void gate_up_rows(const uint16_t *gs,
                                             const uint16_t *us,
                                             const uint16_t *xs, int H,
                                             int lane, float (&ag)[4],
                                             float (&au)[4]) {
    for (int k = lane * 8; k < H; k += 256) {
        float gf[8], uf[8];
        unpack8(*reinterpret_cast<const uint4 *>(gs + k), gf);
        unpack8(*reinterpret_cast<const uint4 *>(us + k), uf);
#pragma unroll
        for (int n = 0; n < NT; n++) {
            float xf[8];
            unpack8(*reinterpret_cast<const uint4 *>(xs + (size_t)n * H + k),
                    xf);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                ag[n] = fmaf(gf[j], xf[j], ag[n]);
                au[n] = fmaf(uf[j], xf[j], au[n]);
            }
        }
    }
}

/* dynamic shared memory layout (both kernels):
 *   ring  : uint16 [DEC_WARPS][DEC_STAGES][stage_elems]
 *   xs    : uint16 [GROUP_TOKENS][x_elems]
 *   bars  : uint64 [DEC_WARPS][DEC_STAGES]
 */
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_gate_up_kernel(DecodeArgs a) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int H = a.H;
    const int stage_elems = 2 * H;
    uint16_t *ring = reinterpret_cast<uint16_t *>(smem_raw);
    uint16_t *xs = ring + (size_t)DEC_WARPS * DEC_STAGES * stage_elems;
    uint64_t *bars = reinterpret_cast<uint64_t *>(xs + (size_t)GROUP_TOKENS * H);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t *mybar = bars + warp * DEC_STAGES;
    uint16_t *myring = ring + (size_t)warp * DEC_STAGES * stage_elems;
    if (lane == 0)
        for (int s = 0; s < DEC_STAGES; s++) mbar_init(&mybar[s], 1);
    mbar_fence_init();
    __syncthreads();

    const int n_sh = a.do_shared ? (a.T + GROUP_TOKENS - 1) / GROUP_TOKENS : 0;
    const int n_rt = *a.n_groups;
    const long N = (long)n_sh * a.Is + (long)n_rt * a.I;
    const long lo = N * blockIdx.x / gridDim.x;
    const long hi = N * (blockIdx.x + 1) / gridDim.x;

    const long my_first = lo + warp;
    const int n_my = my_first < hi ? (int)((hi - my_first + DEC_WARPS - 1) / DEC_WARPS) : 0;
    const uint32_t row_bytes = (uint32_t)H * 2u;
    bool dead = false;

    auto issue = [&](int j) {
        /* lane 0 only */
        long item = my_first + (long)j * DEC_WARPS;
        ItemInfo it = decode_item(item, n_sh, a.Is, a.I);
        const uint16_t *g, *u;
        if (it.shared) {
            g = a.sh_g + (size_t)it.row * H;
            u = a.sh_u + (size_t)it.row * H;
        } else {
            int e = a.grp_expert[it.group] - a.expert_begin;
            const uint16_t *base = a.exp_gu + (size_t)e * 2 * a.I * H;
            g = base + (size_t)it.row * H;
            u = base + (size_t)(a.I + it.row) * H;
        }
        int s = j % DEC_STAGES;
        uint16_t *dst = myring + (size_t)s * stage_elems;
        mbar_expect_tx(&mybar[s], 2 * row_bytes);
        bulk_g2s(dst, g, row_bytes, &mybar[s]);
        bulk_g2s(dst + H, u, row_bytes, &mybar[s]);
    };

    int issued = min(DEC_STAGES, n_my);
    if (lane == 0)
        for (int j = 0; j < issued; j++) issue(j);
    int consumed = 0;

    long item = lo;
    while (item < hi) {   /* CTA-uniform loop over token-group segments */
        ItemInfo si = decode_item(item, n_sh, a.Is, a.I);
        const long seg_hi = min(hi, item - si.row + si.rows);
        int nt, first;
        if (si.shared) {
            first = si.group * GROUP_TOKENS;
            nt = min(GROUP_TOKENS, a.T - first);
        } else {
            first = a.grp_first[si.group];
            nt = a.grp_n[si.group];
        }
        /* stage the group's input rows */
        for (int i = tid; i < nt * (H / 8); i += DEC_THREADS) {
            int n = i / (H / 8), c = i - n * (H / 8);
            int tok = si.shared ? first + n : a.perm[first + n] / a.TK;
            reinterpret_cast<uint4 *>(xs + (size_t)n * H)[c] =
                ldg16(a.x + (size_t)tok * H + (size_t)c * 8);
        }
        __syncthreads();

        while (consumed < n_my &&
               my_first + (long)consumed * DEC_WARPS < seg_hi) {
            const int s = consumed % DEC_STAGES;
            const uint32_t parity = (uint32_t)(consumed / DEC_STAGES) & 1u;
            bool ok = consumed < issued ? mbar_wait(&mybar[s], parity) : false;
            if (!ok && !dead) {
                dead = true;
                set_status(a.status, ST_MBAR_TIMEOUT);
            }
            if (!dead) {
                const long my_item = my_first + (long)consumed * DEC_WARPS;
                const int row = (int)(my_item - (item - si.row));
                const uint16_t *gs = myring + (size_t)s * stage_elems;
                const uint16_t *us = gs + H;
                float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
                switch (nt) {
                    case 1: gate_up_rows<1>(gs, us, xs, H, lane, ag, au); break;
                    case 2: gate_up_rows<2>(gs, us, xs, H, lane, ag, au); break;
                    case 3: gate_up_rows<3>(gs, us, xs, H, lane, ag, au); break;
                    default: gate_up_rows<4>(gs, us, xs, H, lane, ag, au); break;
                }
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    ag[n] = warp_sum(ag[n]);
                    au[n] = warp_sum(au[n]);
                }
                if (lane < nt) {
                    float g = 0.f, u = 0.f;
#pragma unroll
                    for (int n = 0; n < 4; n++)
                        if (lane == n) { g = ag[n]; u = au[n]; }
                    g = bf16_round(g);
                    u = bf16_round(u);
                    if (si.shared)
                        a.sa[(size_t)(first + lane) * a.Is + row] =
                            silu_mul_bits(g, u);
                    else
                        a.act[(size_t)(first + lane) * a.I + row] =
                            silu_act_bits(g, u);
                }
            }
            __syncwarp();
            if (!dead && consumed + DEC_STAGES < n_my) {
                if (lane == 0) issue(consumed + DEC_STAGES);
                issued = consumed + DEC_STAGES + 1;
            }
            consumed++;
        }
        __syncthreads();
        item = seg_hi;
    }
}

template <int NT>
__device__ __forceinline__ void down_rows(const uint16_t *ws,
                                          const uint16_t *as, int I, int lane,
                                          float (&acc)[DOWN_ROWS][4]) {
    for (int k = lane * 8; k < I; k += 256) {
        float af[NT][8];
#pragma unroll
        for (int n = 0; n < NT; n++)
            unpack8(*reinterpret_cast<const uint4 *>(as + (size_t)n * I + k),
                    af[n]);
#pragma unroll
        for (int r = 0; r < DOWN_ROWS; r++) {
            float wf[8];
            unpack8(*reinterpret_cast<const uint4 *>(ws + (size_t)r * I + k),
                    wf);
#pragma unroll
            for (int n = 0; n < NT; n++)
#pragma unroll
                for (int j = 0; j < 8; j++)
                    acc[r][n] = fmaf(wf[j], af[n][j], acc[r][n]);
        }
    }
}

/* H must be a multiple of DOWN_ROWS.  Ring stage = DOWN_ROWS weight rows. */
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_down_kernel(DecodeArgs a) {
    pdl_enter();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int Imax = max(a.I, a.Is);
    const int stage_elems = DOWN_ROWS * Imax;
    uint16_t *ring = reinterpret_cast<uint16_t *>(smem_raw);
    uint16_t *as = ring + (size_t)DEC_WARPS * DEC_STAGES * stage_elems;
    uint64_t *bars =
        reinterpret_cast<uint64_t *>(as + (size_t)GROUP_TOKENS * Imax);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t *mybar = bars + warp * DEC_STAGES;
    uint16_t *myring = ring + (size_t)warp * DEC_STAGES * stage_elems;
    if (lane == 0)
        for (int s = 0; s < DEC_STAGES; s++) mbar_init(&mybar[s], 1);
    mbar_fence_init();
    __syncthreads();

    const int blocks = a.H / DOWN_ROWS;
    const int n_sh = a.do_shared ? (a.T + GROUP_TOKENS - 1) / GROUP_TOKENS : 0;
    const int n_rt = *a.n_groups;
    const long N = (long)(n_sh + n_rt) * blocks;
    const long lo = N * blockIdx.x / gridDim.x;
    const long hi = N * (blockIdx.x + 1) / gridDim.x;
    const long my_first = lo + warp;
    const int n_my = my_first < hi ? (int)((hi - my_first + DEC_WARPS - 1) / DEC_WARPS) : 0;
    bool dead = false;

    auto issue = [&](int j) {
        long item = my_first + (long)j * DEC_WARPS;
        ItemInfo it = decode_item(item, n_sh, blocks, blocks);
        const uint16_t *src;
        uint32_t bytes;
        if (it.shared) {
            src = a.sh_d + (size_t)it.row * DOWN_ROWS * a.Is;
            bytes = (uint32_t)(DOWN_ROWS * a.Is * 2);
        } else {
            int e = a.grp_expert[it.group] - a.expert_begin;
            src = a.exp_d + ((size_t)e * a.H + (size_t)it.row * DOWN_ROWS) * a.I;
            bytes = (uint32_t)(DOWN_ROWS * a.I * 2);
        }
        int s = j % DEC_STAGES;
        mbar_expect_tx(&mybar[s], bytes);
        bulk_g2s(myring + (size_t)s * stage_elems, src, bytes, &mybar[s]);
    };
    int issued = min(DEC_STAGES, n_my);
    if (lane == 0)
        for (int j = 0; j < issued; j++) issue(j);
    int consumed = 0;

    long item = lo;
    while (item < hi) {
        ItemInfo si = decode_item(item, n_sh, blocks, blocks);
        const long seg_hi = min(hi, item - si.row + si.rows);
        int nt, first, K;
        const uint16_t *asrc;
        if (si.shared) {
            first = si.group * GROUP_TOKENS;
            nt = min(GROUP_TOKENS, a.T - first);
            K = a.Is;
            asrc = a.sa + (size_t)first * a.Is;
        } else {
            first = a.grp_first[si.group];
            nt = a.grp_n[si.group];
            K = a.I;
            asrc = a.act + (size_t)first * a.I;
        }
        /* the group's activation rows are consecutive in sorted order */
        for (int i = tid; i < nt * (K / 8); i += DEC_THREADS)
            reinterpret_cast<uint4 *>(as)[i] = ldg16(asrc + (size_t)i * 8);
        __syncthreads();

        while (consumed < n_my &&
               my_first + (long)consumed * DEC_WARPS < seg_hi) {
            const int s = consumed % DEC_STAGES;
            const uint32_t parity = (uint32_t)(consumed / DEC_STAGES) & 1u;
            bool ok = consumed < issued ? mbar_wait(&mybar[s], parity) : false;
            if (!ok && !dead) {
                dead = true;
                set_status(a.status, ST_MBAR_TIMEOUT);
            }
            if (!dead) {
                const long my_item = my_first + (long)consumed * DEC_WARPS;
                const int blk = (int)(my_item - (item - si.row));
                const uint16_t *ws = myring + (size_t)s * stage_elems;
                float acc[DOWN_ROWS][4];
#pragma unroll
                for (int r = 0; r < DOWN_ROWS; r++)
#pragma unroll
                    for (int n = 0; n < 4; n++) acc[r][n] = 0.f;
                switch (nt) {
                    case 1: down_rows<1>(ws, as, K, lane, acc); break;
                    case 2: down_rows<2>(ws, as, K, lane, acc); break;
                    case 3: down_rows<3>(ws, as, K, lane, acc); break;
                    default: down_rows<4>(ws, as, K, lane, acc); break;
                }
                /* as rows are packed [nt][K] */
                uint32_t packed[4] = {0, 0, 0, 0};
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (n < nt) {
                        float v[DOWN_ROWS];
#pragma unroll
                        for (int r = 0; r < DOWN_ROWS; r++)
                            v[r] = warp_sum(acc[r][n]);
                        if (lane == n) {
                            packed[0] = pack_bf16(v[0], v[1]);
                            packed[1] = pack_bf16(v[2], v[3]);
                            packed[2] = pack_bf16(v[4], v[5]);
                            packed[3] = pack_bf16(v[6], v[7]);
                        }
                    }
                }
                if (lane < nt) {
                    /* routed rows go back to flat assignment order t*TK + j
                     * (the CPU engine's eo layout, c/layer.h:618) */
                    const size_t orow = si.shared
                                            ? (size_t)(first + lane)
                                            : (size_t)a.perm[first + lane];
                    uint16_t *dst = (si.shared ? a.sy : a.eo) + orow * a.H +
                                    (size_t)blk * DOWN_ROWS;
                    *reinterpret_cast<uint4 *>(dst) =
                        make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
            __syncwarp();
            if (!dead && consumed + DEC_STAGES < n_my) {
                if (lane == 0) issue(consumed + DEC_STAGES);
                issued = consumed + DEC_STAGES + 1;
            }
            consumed++;
        }
        __syncthreads();
        item = seg_hi;
    }
}

/*
 * Per-token tail (c/layer.h:350,356-361 == 625-649):
 *   routed = rnd(sum_j f32(w_j) * f32(y_j))   slots ascending, mul then add
 *   sgat   = rnd(sigmoid(f32(sgl)));  shared = rnd(f32(sy) * f32(sgat))
 *   out    = rnd(f32(routed) + f32(shared))
 * y_j is row t*TK + j of the expert outputs (flat assignment order), so the
 * sum runs in the CPU engine's slot order regardless of dispatch order.
 * One thread per 8 output columns.
 */
struct FinalizeArgs {
    int T, H, TK;
    const uint16_t *eo;      /* [A, H] flat assignment order ... */
    const int32_t *pos;      /* ... or, if not NULL, row pos[t*TK+j] of eo */
    const uint16_t *rw;      /* [T, TK] */
    const uint16_t *sy;      /* [T, H] (NULL: no shared expert term) */
    const uint16_t *sgl;     /* [T] shared-gate logits */
    uint16_t *out;           /* [T, H] (optional when res_out is set) */
    uint16_t *tr_routed, *tr_shared, *tr_out;   /* optional */
    /* the residual add after the block folded in (c/layer.h:230-234,388):
     * res_out = rnd(res + rnd(moe_out)) */
    const uint16_t *res;
    uint16_t *res_out;
};

__global__ void __launch_bounds__(256)
moe_finalize_kernel(FinalizeArgs a) {
    pdl_enter();
    const int cols8 = a.H / 8;
    const long total = (long)a.T * cols8;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int t = (int)(i / cols8), c = (int)(i - (long)t * cols8);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.0f;
        /* eight slots' rows are requested before the first is added (the sum
         * itself stays in slot order) */
        for (int s0 = 0; s0 < a.TK; s0 += 8) {
            uint4 yv[8];
            float wv[8];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int s = s0 + q;
                if (s < a.TK) {
                    const size_t flat = (size_t)t * a.TK + s;
                    const size_t row = a.pos ? (size_t)a.pos[flat] : flat;
                    yv[q] = ldg16(a.eo + row * a.H + (size_t)c * 8);
                    wv[q] = bf16_f32(a.rw[flat]);
                } else {
                    yv[q] = make_uint4(0, 0, 0, 0);
                    wv[q] = 0.0f;
                }
            }
#pragma unroll
            for (int q = 0; q < 8; q++) {
                if (s0 + q >= a.TK) break;
                float y[8];
                unpack8(yv[q], y);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    acc[j] = __fadd_rn(acc[j], __fmul_rn(wv[q], y[j]));
            }
        }
        float routed[8], shared[8], outv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) routed[j] = bf16_round(acc[j]);
        if (a.sy) {
            const float sgat =
                bf16_round(sigmoid_f32(bf16_f32(a.sgl[t])));
            float y[8];
            unpack8(ldg16(a.sy + (size_t)t * a.H + (size_t)c * 8), y);
#pragma unroll
            for (int j = 0; j < 8; j++)
                shared[j] = bf16_round(__fmul_rn(y[j], sgat));
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) shared[j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++)
            outv[j] = __fadd_rn(routed[j], shared[j]);
        const size_t o = (size_t)t * a.H + (size_t)c * 8;
        if (a.out)
            *reinterpret_cast<uint4 *>(a.out + o) =
                make_uint4(pack_bf16(outv[0], outv[1]), pack_bf16(outv[2], outv[3]),
                           pack_bf16(outv[4], outv[5]), pack_bf16(outv[6], outv[7]));
        if (a.res_out) {
            float r[8];
            unpack8(ldg16(a.res + o), r);
#pragma unroll
            for (int j = 0; j < 8; j++) r[j] = __fadd_rn(r[j], bf16_round(outv[j]));
            *reinterpret_cast<uint4 *>(a.res_out + o) =
                make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]),
                           pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
        }
        if (a.tr_out)
            *reinterpret_cast<uint4 *>(a.tr_out + o) = make_uint4(
                pack_bf16(outv[0], outv[1]), pack_bf16(outv[2], outv[3]),
                pack_bf16(outv[4], outv[5]), pack_bf16(outv[6], outv[7]));
        if (a.tr_routed)
            *reinterpret_cast<uint4 *>(a.tr_routed + o) = make_uint4(
                pack_bf16(routed[0], routed[1]), pack_bf16(routed[2], routed[3]),
                pack_bf16(routed[4], routed[5]), pack_bf16(routed[6], routed[7]));
        if (a.tr_shared)
            *reinterpret_cast<uint4 *>(a.tr_shared + o) = make_uint4(
                pack_bf16(shared[0], shared[1]), pack_bf16(shared[2], shared[3]),
                pack_bf16(shared[4], shared[5]), pack_bf16(shared[6], shared[7]));
    }
}

}  // namespace apus
