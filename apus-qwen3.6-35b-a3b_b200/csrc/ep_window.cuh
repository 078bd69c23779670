/*
 * Expert-parallel exchange through peer memory (NVLink loads and stores issued
 * by the kernels themselves; no collective library on the data path, no host
 * synchronisation inside a block step).
 *
 * Net-new: the reference engine is one process; what travels is the input of
 * its per-expert loop (c/layer.h:599-606: the rows of each expert) and its
 * output (c/layer.h:614-620: the rows scattered back to their slots).
 *
 * Every rank owns one window of device memory, mapped by all peers (CUDA IPC):
 *
 *   rx   [N][cap][H]  BF16   rows received, one region per source rank
 *   re   [N][cap]     int32  their global expert ids; -1 = empty slot
 *   hdr  [N][4]       int32  {rows sent, offset of those rows in the source's
 *                             send order, 0, 0}
 *   fin  [N]          uint32 epoch of the last complete push of each source
 *   by   [cap][H]     BF16   expert outputs returned for this rank's own
 *                            assignments, in its send order
 *   fbk  [N]          uint32 epoch of the last complete return of each peer
 *
 * cap = T_max * topk, the most rows one rank can send to one peer, so a push
 * never overflows and only rows that exist travel.  A step on rank s:
 *
 *   push    sort the T*topk assignments by owning rank (stable), then store
 *           each token row and its expert id straight into the owner's rx/re
 *           region s, pad re with -1, and — after a system-scope fence and a
 *           count of finished CTAs — the last CTA writes hdr and fin[s] = epoch
 *           into every peer's window (release).
 *   wait    one thread per source spins (bounded, acquire, system scope) until
 *           fin[src] has reached the epoch.
 *   experts the resident experts over all N*cap slots (empty ones skipped)
 *   return  each valid output row goes straight to by[] of the rank that sent
 *           the input row, at the position the source asked for; last CTA sets
 *           fbk[me] = epoch in every peer's window.
 *   wait    until fbk[peer] has reached the epoch for all peers; then the
 *           weighted sum in slot order as on one GPU.
 *
 * Reuse is safe without further flags: a rank starts step k+1 only after every
 * peer's return of step k, and a peer returns only after its expert kernels
 * have read rx; peers write by[] for step k+1 only after this rank's push of
 * step k+1, which follows its own read of by[] in stream order.
 *
 * The second form of the step ("pull") has no exchange kernel around the
 * experts; top-k of 8 over at most 8 ranks means nearly every rank needs
 * nearly every token, so the token rows are all-gathered instead of sent per
 * assignment (each row crosses a link once, not once per expert):
 *
 *   xs   [N][T_max][H] BF16   every rank's token rows, written by their owners
 *   ids  [N][cap]      int32  their expert ids (flat t * topk + j; -1 = none)
 *
 *   publish store x and the ids into region `me` of xs/ids of EVERY rank's
 *           window (its own included), then fin[me] = epoch everywhere.
 *   wait    as above.
 *   experts sort the ids of the resident experts (the dispatch skips everyone
 *           else's); the gather kernel reads
 *           each needed row from the local xs; gate_up as on one GPU; the down
 *           GEMM's epilogue stores every output row straight into by[] of the
 *           rank that owns the token, at the flat position t * topk + j its
 *           combine reads; one more launch (fence, fbk[me] = epoch in every
 *           peer) follows the GEMM.
 *   wait, combine as above, with no position table.
 *
 * Reuse: a rank overwrites region `me` of its peers' xs/ids for step k+1 only
 * after its combine of step k, which follows every peer's fbk of step k, which
 * follows that peer's last read of xs/ids.
 *
 * No kernel here waits on a kernel of the same GPU, so N windows in one process
 * on one GPU (the tests' emulation) work as long as all pushes are launched
 * before the first wait.
 */
#pragma once
#include "common.cuh"

namespace apus {

constexpr int EPW_MAX_RANKS = 8;
constexpr int ST_PEER_TIMEOUT = 6;      /* a peer's flag never reached the epoch */
constexpr uint32_t EPW_WAIT_POLLS = 1u << 21;   /* x ~1 us: about two seconds */

struct EpwLayout {
    size_t rx, re, hdr, fin, by, fbk, xs, ids, total;
    int cap, H, n, tokens;
};
inline EpwLayout epw_layout(int n, int cap, int H, int tokens) {
    EpwLayout l;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t o = 0;
    l.rx = o;  o = up(o + (size_t)n * cap * H * 2);
    l.re = o;  o = up(o + (size_t)n * cap * 4);
    l.hdr = o; o = up(o + (size_t)n * 16);
    l.fin = o; o = up(o + (size_t)n * 4);
    l.by = o;  o = up(o + (size_t)cap * H * 2);
    l.fbk = o; o = up(o + (size_t)n * 4);
    l.xs = o;  o = up(o + (size_t)n * tokens * H * 2);
    l.ids = o; o = up(o + (size_t)n * cap * 4);
    l.total = o;
    l.tokens = tokens;
    l.cap = cap;
    l.H = H;
    l.n = n;
    return l;
}

struct EpwPeers {
    unsigned char *base[EPW_MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

/* All CTAs call this after their last peer store.  Returns true in exactly one
 * CTA, the one that finished last, after which every CTA's stores are ordered
 * before whatever that CTA stores next (fence, counter, fence). */
__device__ __forceinline__ bool epw_last_cta(unsigned int *counter) {
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int old = atomicAdd(counter, 1u);
        s_last = old == gridDim.x - 1;
        if (s_last) *counter = 0;           /* ready for the next launch */
        __threadfence_system();
    }
    __syncthreads();
    return s_last != 0;
}

/* offsets[n+1]: send-order offsets per owner; perm[A]: send position -> flat
 * assignment t*TK + j.  grid-stride over (row, 16-byte chunk). */
__global__ void __launch_bounds__(256)
epw_push_kernel(const uint16_t *__restrict__ x, const int32_t *__restrict__ idx,
                const int32_t *__restrict__ perm, const int32_t *__restrict__ offsets,
                int A, int TK, EpwLayout l, EpwPeers peers, int me, uint32_t epoch,
                unsigned int *counter, uint32_t *d_epoch) {
    pdl_enter();
    /* epoch 0: the step number lives on the device (this push opens step
     * *d_epoch + 1), so that a captured CUDA graph can be replayed */
    if (epoch == 0) epoch = *d_epoch + 1;
    __shared__ int s_off[EPW_MAX_RANKS + 1];
    __shared__ unsigned char *s_base[EPW_MAX_RANKS];
    if (threadIdx.x <= l.n) s_off[threadIdx.x] = offsets[threadIdx.x];
    if (threadIdx.x < EPW_MAX_RANKS) s_base[threadIdx.x] = peers.base[threadIdx.x];
    __syncthreads();
    const int c8 = l.H / 8;
    const long stride = (long)gridDim.x * blockDim.x;
    const long first = (long)blockIdx.x * blockDim.x + threadIdx.x;
    /* Every CTA owns one contiguous run of the send order.  The send order is
     * destination-major, so at any moment different CTAs are storing to
     * different destinations: the NVLink stores to the peers and the local
     * copies proceed side by side instead of one destination after the other
     * (a grid-stride loop over the rows had all CTAs on the same destination:
     * 189 us for 32768 rows on two GPUs, half of them remote). */
    const int rows_per = (A + (int)gridDim.x - 1) / (int)gridDim.x;
    const int q_lo = min(A, (int)blockIdx.x * rows_per), q_hi = min(A, q_lo + rows_per);
    for (long i = (long)q_lo * c8 + threadIdx.x; i < (long)q_hi * c8; i += blockDim.x) {
        const int q = (int)(i / c8), c = (int)(i - (long)q * c8);
        int d = 0;
#pragma unroll
        for (int r = 1; r < EPW_MAX_RANKS; r++) d += (r < l.n && q >= s_off[r]) ? 1 : 0;
        const int slot = me * l.cap + (q - s_off[d]);
        const int a = perm[q];
        const uint4 v = ldg16(x + (size_t)(a / TK) * l.H + (size_t)c * 8);
        *reinterpret_cast<uint4 *>(s_base[d] + l.rx + ((size_t)slot * l.H + (size_t)c * 8) * 2) = v;
        if (c == 0) reinterpret_cast<int32_t *>(s_base[d] + l.re)[slot] = idx[a];
    }
    /* empty slots of my region in every peer */
    for (long i = first; i < (long)l.n * l.cap; i += stride) {
        const int d = (int)(i / l.cap), s = (int)(i - (long)d * l.cap);
        if (s >= s_off[d + 1] - s_off[d])
            reinterpret_cast<int32_t *>(s_base[d] + l.re)[me * l.cap + s] = -1;
    }
    if (epw_last_cta(counter) && threadIdx.x < l.n) {
        const int d = threadIdx.x;
        int32_t *h = reinterpret_cast<int32_t *>(s_base[d] + l.hdr) + me * 4;
        h[0] = s_off[d + 1] - s_off[d];
        h[1] = s_off[d];
        if (d == 0) *d_epoch = epoch;      /* every CTA has read it: this one is the last */
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(s_base[d] + l.fin) + me, epoch);
    }
}

/* flags[n] in this rank's own window.  One warp. */
__global__ void __launch_bounds__(32)
epw_wait_kernel(const uint32_t *flags, int n, uint32_t epoch, int *status,
                const uint32_t *d_epoch) {
    pdl_enter();
    if (epoch == 0) epoch = *d_epoch;
    if ((int)threadIdx.x >= n) return;
    for (uint32_t i = 0; i < EPW_WAIT_POLLS; i++) {
        const uint32_t v = ld_acquire_sys(flags + threadIdx.x);
        if ((int32_t)(v - epoch) >= 0) return;
        __nanosleep(1000);
    }
    set_status(status, ST_PEER_TIMEOUT);
}

/* y [N*cap][H]: expert outputs by slot.  Row i of source s goes to by[hdr[s].off
 * + i] of rank s. */
__global__ void __launch_bounds__(256)
epw_return_kernel(const uint16_t *__restrict__ y, EpwLayout l, EpwPeers peers, int me,
                  uint32_t epoch, unsigned int *counter, const uint32_t *d_epoch) {
    pdl_enter();
    if (epoch == 0) epoch = *d_epoch;
    __shared__ int s_cnt[EPW_MAX_RANKS + 1], s_dst[EPW_MAX_RANKS];
    __shared__ unsigned char *s_base[EPW_MAX_RANKS];
    if (threadIdx.x < EPW_MAX_RANKS) s_base[threadIdx.x] = peers.base[threadIdx.x];
    __syncthreads();
    if (threadIdx.x == 0) {
        const int32_t *h = reinterpret_cast<const int32_t *>(s_base[me] + l.hdr);
        int run = 0;
        for (int s = 0; s < l.n; s++) {
            s_cnt[s] = run;
            int cnt = h[s * 4];
            cnt = cnt < 0 ? 0 : (cnt > l.cap ? l.cap : cnt);
            run += cnt;
            s_dst[s] = h[s * 4 + 1];
        }
        s_cnt[l.n] = run;
    }
    __syncthreads();
    const int c8 = l.H / 8;
    /* one contiguous run of the (source-major) rows per CTA: see epw_push_kernel */
    const int n_rows = s_cnt[l.n];
    const int rows_per = (n_rows + (int)gridDim.x - 1) / (int)gridDim.x;
    const int r_lo = min(n_rows, (int)blockIdx.x * rows_per), r_hi = min(n_rows, r_lo + rows_per);
    for (long i = (long)r_lo * c8 + threadIdx.x; i < (long)r_hi * c8; i += blockDim.x) {
        const int r = (int)(i / c8), c = (int)(i - (long)r * c8);
        int s = 0;
#pragma unroll
        for (int k = 1; k < EPW_MAX_RANKS; k++) s += (k < l.n && r >= s_cnt[k]) ? 1 : 0;
        const int row = r - s_cnt[s];
        const int dst = s_dst[s] + row;
        if (dst < 0 || dst >= l.cap) continue;       /* a header that makes no sense */
        const uint4 v = ldg16(y + ((size_t)(s * l.cap + row) * l.H + (size_t)c * 8));
        *reinterpret_cast<uint4 *>(s_base[s] + l.by + ((size_t)dst * l.H + (size_t)c * 8) * 2) = v;
    }
    if (epw_last_cta(counter) && threadIdx.x < l.n)
        st_release_sys(reinterpret_cast<uint32_t *>(s_base[threadIdx.x] + l.fbk) + me, epoch);
}


/* Region `me` of xs and ids in every rank's window <- x [T,H], idx [T*TK] (-1
 * up to cap); then the push flag.  Every CTA owns one contiguous run of the
 * (destination, 16-byte chunk) list, so all destinations are written at once. */
__global__ void __launch_bounds__(256)
epw_publish_kernel(const uint16_t *__restrict__ x, const int32_t *__restrict__ idx, int T,
                   int TK, EpwLayout l, EpwPeers peers, int me, uint32_t epoch,
                   unsigned int *counter, uint32_t *d_epoch) {
    pdl_enter();
    if (epoch == 0) epoch = *d_epoch + 1;
    __shared__ unsigned char *s_base[EPW_MAX_RANKS];
    if (threadIdx.x < EPW_MAX_RANKS) s_base[threadIdx.x] = peers.base[threadIdx.x];
    __syncthreads();
    /* x == nullptr: the rows are there already (epw_publish_rows_kernel) */
    const long n16 = x ? (long)T * (l.H / 8) : 0;
    const long total = n16 * l.n;
    const long per = (total + gridDim.x - 1) / gridDim.x;
    const long lo = min(total, (long)blockIdx.x * per), hi = min(total, lo + per);
    const size_t region = (size_t)me * l.tokens * l.H * 2;
    /* four independent loads in flight per thread before the four stores */
    for (long j0 = lo + threadIdx.x; j0 < hi; j0 += 4L * blockDim.x) {
        uint4 v[4];
        int d[4];
        long i[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const long j = j0 + (long)u * blockDim.x;
            d[u] = j < hi ? (int)(j / n16) : -1;
            i[u] = j - (long)(d[u] < 0 ? 0 : d[u]) * n16;
            if (d[u] >= 0) v[u] = ldg16(x + (size_t)i[u] * 8);
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (d[u] >= 0)
                reinterpret_cast<uint4 *>(s_base[d[u]] + l.xs + region)[i[u]] = v[u];
    }
    const long ids_total = (long)l.cap * l.n;
    for (long j = (long)blockIdx.x * blockDim.x + threadIdx.x; j < ids_total;
         j += (long)gridDim.x * blockDim.x) {
        const int d = (int)(j / l.cap);
        const long i = j - (long)d * l.cap;
        reinterpret_cast<int32_t *>(s_base[d] + l.ids)[(size_t)me * l.cap + i] =
            i < (long)T * TK ? idx[i] : -1;
    }
    if (epw_last_cta(counter) && threadIdx.x < l.n) {
        if (threadIdx.x == 0) *d_epoch = epoch;
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(s_base[threadIdx.x] + l.fin) + me, epoch);
    }
}

/* The rows alone, no ids and no flag: needs nothing from the router, so it can
 * run beside it on another stream; the publish kernel proper (x = nullptr) must
 * follow it in device order. */
__global__ void __launch_bounds__(256)
epw_publish_rows_kernel(const uint16_t *__restrict__ x, int T, EpwLayout l, EpwPeers peers,
                        int me) {
    __shared__ unsigned char *s_base[EPW_MAX_RANKS];
    if (threadIdx.x < EPW_MAX_RANKS) s_base[threadIdx.x] = peers.base[threadIdx.x];
    __syncthreads();
    const long n16 = (long)T * (l.H / 8);
    const long total = n16 * l.n;
    const long per = (total + gridDim.x - 1) / gridDim.x;
    const long lo = min(total, (long)blockIdx.x * per), hi = min(total, lo + per);
    const size_t region = (size_t)me * l.tokens * l.H * 2;
    for (long j0 = lo + threadIdx.x; j0 < hi; j0 += 4L * blockDim.x) {
        uint4 v[4];
        int d[4];
        long i[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const long j = j0 + (long)u * blockDim.x;
            d[u] = j < hi ? (int)(j / n16) : -1;
            i[u] = j - (long)(d[u] < 0 ? 0 : d[u]) * n16;
            if (d[u] >= 0) v[u] = ldg16(x + (size_t)i[u] * 8);
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (d[u] >= 0)
                reinterpret_cast<uint4 *>(s_base[d[u]] + l.xs + region)[i[u]] = v[u];
    }
}

/* After the down GEMM whose epilogue stored into the peers: everything this GPU
 * wrote before this launch is ordered before the flags. */
__global__ void __launch_bounds__(32)
epw_signal_kernel(EpwLayout l, EpwPeers peers, int me, uint32_t epoch,
                  const uint32_t *d_epoch) {
    pdl_enter();
    if (epoch == 0) epoch = *d_epoch;
    __threadfence_system();
    if ((int)threadIdx.x < l.n)
        st_release_sys(reinterpret_cast<uint32_t *>(peers.base[threadIdx.x] + l.fbk) + me,
                       epoch);
}

}  // namespace apus
