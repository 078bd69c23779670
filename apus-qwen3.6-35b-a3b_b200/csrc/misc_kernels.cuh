/*
 * misc_kernels.cuh — the engine's per-matmul hooks in its normative
 * accumulation order, the two steps either side of the MoE block, and the
 * synthetic-tensor fill.
 */
#pragma once
#include "common.cuh"
#include "synth.h"

namespace apus {

/* One fp32 chain per output, k strictly ascending, product and sum each
 * rounded once (c/bf16.h:285-294).  The product of two BF16 values is exact
 * in fp32 unless it underflows, so the literal multiply-then-add is kept here
 * (these hooks are launch- and PCIe-bound; chain latency is what it is). */
__device__ __forceinline__ float exact_dot(const uint16_t *__restrict__ wrow,
                                           const uint16_t *__restrict__ xrow,
                                           int K) {
    float acc = 0.0f;
    int k = 0;
    if ((K & 7) == 0 && ((((uintptr_t)wrow) | ((uintptr_t)xrow)) & 15) == 0) {
        for (; k < K; k += 8) {
            uint4 wv = ldg16(wrow + k), xv = ldg16(xrow + k);
            acc = __fadd_rn(acc, __fmul_rn(bf16lo(wv.x), bf16lo(xv.x)));
            acc = __fadd_rn(acc, __fmul_rn(bf16hi(wv.x), bf16hi(xv.x)));
            acc = __fadd_rn(acc, __fmul_rn(bf16lo(wv.y), bf16lo(xv.y)));
            acc = __fadd_rn(acc, __fmul_rn(bf16hi(wv.y), bf16hi(xv.y)));
            acc = __fadd_rn(acc, __fmul_rn(bf16lo(wv.z), bf16lo(xv.z)));
            acc = __fadd_rn(acc, __fmul_rn(bf16hi(wv.z), bf16hi(xv.z)));
            acc = __fadd_rn(acc, __fmul_rn(bf16lo(wv.w), bf16lo(xv.w)));
            acc = __fadd_rn(acc, __fmul_rn(bf16hi(wv.w), bf16hi(xv.w)));
        }
    } else {
        for (; k < K; k++)
            acc = __fadd_rn(acc, __fmul_rn(bf16_f32(__ldg(wrow + k)),
                                           bf16_f32(__ldg(xrow + k))));
    }
    return acc;
}

/* y[m,o] = rnd(chain) — apus_bf16_gemv_hot / apus_bf16_gemm_hot
 * (c/bf16.h:199-231), row m of a GEMM bitwise its GEMV. */
__global__ void __launch_bounds__(128)
exact_gemm_kernel(const uint16_t *__restrict__ w, const uint16_t *__restrict__ x,
                  uint16_t *__restrict__ y, long M, long O, int K) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < M * O;
         i += (long)gridDim.x * blockDim.x) {
        long m = i / O, o = i - m * O;
        y[i] = bf16_bits(exact_dot(w + o * K, x + m * K, K));
    }
}
/* fp32-out matvec, no narrowing — apus_moe_matvec_f32_hot (c/moe.h:284-310) */
__global__ void __launch_bounds__(128)
exact_matvec_f32_kernel(const uint16_t *__restrict__ w,
                        const uint16_t *__restrict__ x, float *__restrict__ y,
                        long O, int K) {
    for (long o = (long)blockIdx.x * blockDim.x + threadIdx.x; o < O;
         o += (long)gridDim.x * blockDim.x)
        y[o] = exact_dot(w + o * K, x, K);
}

/* y[m,o] = rnd(sum_k W[o,k] x[m,k]) as a weight STREAM (the engine's largest
 * dense product per token is the output head, 248320 x 2048 = 1 GB of weights,
 * c/model.h:667-688): device pointers, one warp per pair of weight rows, 16-byte
 * coalesced loads with eight in flight per lane, the M <= 8 activation rows in
 * shared memory as fp32, lane-strided fp32 partial sums closed by shuffles.
 * The summation order differs from the engine's sequential chain, so the result
 * agrees to BF16 tolerance, not bitwise; the exact-order form is
 * exact_gemm_kernel behind the host-pointer hooks. */
template <int M>
__global__ void __launch_bounds__(256)
gemv_stream_kernel(const uint16_t *__restrict__ w, const uint16_t *__restrict__ x,
                   uint16_t *__restrict__ y, long O, int K) {
    extern __shared__ float gs_x[];          /* [M][K] */
    for (int i = threadIdx.x; i < M * K; i += blockDim.x) gs_x[i] = bf16_f32(x[i]);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long warp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
    for (long o0 = warp * 2; o0 < O; o0 += nwarps * 2) {
        const bool two = o0 + 1 < O;
        const uint16_t *r0 = w + o0 * K, *r1 = w + (two ? o0 + 1 : o0) * K;
        float a0[M], a1[M];
#pragma unroll
        for (int m = 0; m < M; m++) a0[m] = a1[m] = 0.0f;
#pragma unroll 4
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 v0 = ldg16(r0 + k), v1 = ldg16(r1 + k);
            const float f0[8] = {bf16lo(v0.x), bf16hi(v0.x), bf16lo(v0.y), bf16hi(v0.y),
                                 bf16lo(v0.z), bf16hi(v0.z), bf16lo(v0.w), bf16hi(v0.w)};
            const float f1[8] = {bf16lo(v1.x), bf16hi(v1.x), bf16lo(v1.y), bf16hi(v1.y),
                                 bf16lo(v1.z), bf16hi(v1.z), bf16lo(v1.w), bf16hi(v1.w)};
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float4 xa = *reinterpret_cast<const float4 *>(gs_x + (size_t)m * K + k);
                const float4 xb = *reinterpret_cast<const float4 *>(gs_x + (size_t)m * K + k + 4);
                const float xf[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    a0[m] = fmaf(f0[j], xf[j], a0[m]);
                    a1[m] = fmaf(f1[j], xf[j], a1[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; m++) {
            const float s0 = warp_sum(a0[m]), s1 = warp_sum(a1[m]);
            if (lane == 0) {
                y[(size_t)m * O + o0] = bf16_bits(s0);
                if (two) y[(size_t)m * O + o0 + 1] = bf16_bits(s1);
            }
        }
    }
}

/* RMSNorm with (1+w) gain, single rounding (c/attn.h:175-186): the sum of
 * squares is the ascending sequential fp32 chain; one warp per row, lane 0
 * walks the chain over the row staged in shared memory. */
__global__ void __launch_bounds__(128)
rmsnorm_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w,
               uint16_t *__restrict__ y, int T, int N) {
    extern __shared__ float rs_smem[];   /* [4][N] */
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float *row = rs_smem + (size_t)warp * N;
    for (int i = lane; i < N; i += 32)
        row[i] = bf16_f32(x[(size_t)t * N + i]);
    __syncwarp();
    /* the reference's sum of squares is one ascending fp32 chain; the dependent
     * add is the critical path, so operands come in vectors, sixteen steps per
     * iteration, and the next iteration's loads are hoisted above the adds */
    float ss = 0.0f;
    if (lane == 0) {
        int i = 0;
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
#pragma unroll 2
        for (; (N & 3) == 0 && i + 16 <= N; i += 16) {   /* rows stay 16-byte aligned */
            const float4 v[4] = {r4[i / 4], r4[i / 4 + 1], r4[i / 4 + 2], r4[i / 4 + 3]};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                ss = __fadd_rn(ss, __fmul_rn(v[q].x, v[q].x));
                ss = __fadd_rn(ss, __fmul_rn(v[q].y, v[q].y));
                ss = __fadd_rn(ss, __fmul_rn(v[q].z, v[q].z));
                ss = __fadd_rn(ss, __fmul_rn(v[q].w, v[q].w));
            }
        }
        for (; i < N; i++) ss = __fadd_rn(ss, __fmul_rn(row[i], row[i]));
    }
    ss = __shfl_sync(0xffffffffu, ss, 0);
    const float rs = __fdiv_rn(
        1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)N), 1e-6f)));
    for (int i = lane; i < N; i += 32) {
        float g = __fadd_rn(1.0f, w ? bf16_f32(w[i]) : 0.0f);
        y[(size_t)t * N + i] = bf16_bits(__fmul_rn(__fmul_rn(row[i], rs), g));
    }
}

/* out = rnd(f32(a) + f32(b))  (c/layer.h:230-234) */
__global__ void __launch_bounds__(256)
resadd_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b,
              uint16_t *__restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = bf16_bits(__fadd_rn(bf16_f32(a[i]), bf16_f32(b[i])));
}

__global__ void __launch_bounds__(256)
synth_fill_kernel(uint16_t *__restrict__ dst, size_t n, uint64_t key,
                  uint64_t first, double sigma) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        dst[i] = apus_synth_bf16(key, first + i, sigma);
}

}  // namespace apus
