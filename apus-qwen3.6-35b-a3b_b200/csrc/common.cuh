/*
 * common.cuh — BF16 code helpers, mbarrier / bulk-copy PTX wrappers with
 * bounded waits, and the device status word.  sm_100a only.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace apus {

/* ---- BF16 codes (c/bf16.h:261-274) -------------------------------------- */
__device__ __forceinline__ float bf16_f32(uint16_t b) {
    return __uint_as_float((uint32_t)b << 16);
}
/* RNE narrow; NaN passes through as the high half. */
__device__ __forceinline__ uint16_t bf16_bits(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(u >> 16);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
__device__ __forceinline__ float bf16_round(float f) {
    return bf16_f32(bf16_bits(f));
}
/* two packed codes in one 32-bit word: low half = element 0 */
__device__ __forceinline__ float bf16lo(uint32_t p) {
    return __uint_as_float(p << 16);
}
__device__ __forceinline__ float bf16hi(uint32_t p) {
    return __uint_as_float(p & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    return (uint32_t)bf16_bits(a) | ((uint32_t)bf16_bits(b) << 16);
}

/* sigmoid / silu in the written order of c/moe.h:312-314,390-393,441-443:
 * each operation one IEEE fp32 rounding, nothing contracted. */
__device__ __forceinline__ float sigmoid_f32(float z) {
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
}
/* routed activation: a1 = rnd(g*sigmoid(g)); act = rnd(f32(a1)*u) */
__device__ __forceinline__ uint16_t silu_act_bits(float g, float u) {
    float a1 = bf16_round(__fmul_rn(g, sigmoid_f32(g)));
    return bf16_bits(__fmul_rn(a1, u));
}
/* shared activation: y = rnd((g*sigmoid(g))*u), single rounding */
__device__ __forceinline__ uint16_t silu_mul_bits(float g, float u) {
    return bf16_bits(__fmul_rn(__fmul_rn(g, sigmoid_f32(g)), u));
}

/* ---- the same roundings for the tensor-core epilogues ----------------------
 * At thousands of tokens the gate/up GEMM is bound by its epilogue's
 * instruction count, not by the MMAs (37.7 M SwiGLU evaluations per 8192-token
 * block), so the epilogues narrow with the hardware conversion (cvt.rn: the
 * same round-to-nearest-even as the integer rule above for every finite value
 * and infinity; NaN payloads, outside the engine's contract, come out
 * canonical) two values at a time, and evaluate the sigmoid with ex2.approx /
 * rcp.approx (about 2 ulp of fp32 each, invisible after the BF16 narrowing in
 * all but ~1e-4 of the values, where the result moves by one BF16 step). */
__device__ __forceinline__ uint32_t pack_bf16_rn(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
/* both values narrowed to BF16 and widened again */
__device__ __forceinline__ void bf16_round2(float &a, float &b) {
    const uint32_t p = pack_bf16_rn(a, b);
    a = __uint_as_float(p << 16);
    b = __uint_as_float(p & 0xffff0000u);
}
__device__ __forceinline__ float silu_fast(float g) {
    return __fmul_rn(g, __fdividef(1.0f, __fadd_rn(1.0f, __expf(-g))));
}
/* two routed activations, packed: rnd(rnd(silu(g)) * u)  (g, u already BF16 values) */
__device__ __forceinline__ uint32_t silu_act_pack2(float g0, float u0, float g1, float u1) {
    float a0 = silu_fast(g0), a1 = silu_fast(g1);
    bf16_round2(a0, a1);
    return pack_bf16_rn(__fmul_rn(a0, u0), __fmul_rn(a1, u1));
}
/* two shared activations, packed: rnd(silu(g) * u), single rounding */
__device__ __forceinline__ uint32_t silu_mul_pack2(float g0, float u0, float g1, float u1) {
    return pack_bf16_rn(__fmul_rn(silu_fast(g0), u0), __fmul_rn(silu_fast(g1), u1));
}

/* ---- device status word --------------------------------------------------
 * Kernels never trap or spin without limit.  A wait that runs out records a
 * code here and the kernel returns; the host reads the word after the call. */
enum : int {
    ST_OK = 0,
    ST_MBAR_TIMEOUT = 1,     /* a bulk copy never signalled its barrier */
    ST_TMEM_TIMEOUT = 2,     /* an MMA commit never arrived */
    ST_BAD_INDEX = 3,        /* an expert id or row offset out of range */
    ST_SCHED_TIMEOUT = 4
};
__device__ __forceinline__ void set_status(int *status, int code) {
    if (status) atomicCAS(status, 0, code);
}

/* ---- shared-memory addresses, mbarriers, bulk copies --------------------- */
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(count)
                 : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile(
        "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
            smem_u32(bar)),
        "r"(bytes)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
/* Bounded wait: about a second at most, then give up.  Returns false on
 * timeout (the caller records a status code and unwinds). */
#ifndef APUS_WAIT_LIMIT
#define APUS_WAIT_LIMIT (1u << 22)
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < APUS_WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
/* 1-D bulk copy global -> shared, completion counted on an mbarrier.  Both
 * addresses 16-byte aligned, bytes a multiple of 16.  No multicast. */
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src,
                                         uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
/* L2 prefetch hint for a contiguous range (16-byte aligned, multiple of 16) */
__device__ __forceinline__ void bulk_prefetch_l2(const void *src,
                                                 uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

/* 16-byte read-only global load */
__device__ __forceinline__ uint4 ldg16(const void *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
}

/* Programmatic dependent launch: every kernel of the block begins with
 * pdl_enter(): it lets the next kernel in the stream be scheduled early (its
 * own prologue then overlaps this kernel's tail) and waits until the previous
 * kernel's memory is complete and visible.  Without the launch attribute both
 * instructions are no-ops. */
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* host: launch with the programmatic-stream-serialization attribute */
extern bool g_apus_use_pdl;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                            size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_apus_use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace apus
