/*
 * synth.h — counter-based synthetic tensor generator shared by host C/C++ and
 * CUDA device code, so a weight tensor can be produced directly in HBM (the
 * 40-layer stack is 64.7 GB) and reproduced bit-for-bit on the host for the
 * CPU checker without either side copying from the other.
 *
 * Element i of tensor (seed, layer, tensor_id) is an approximately normal
 * draw built only from integer arithmetic and exactly-rounded IEEE double
 * operations, so host and device agree on every bit:
 *
 *   key   = mix(mix(seed) ^ (layer << 8 | tensor_id))
 *   d_j   = mix(key + (3*i + j) * GAMMA),  j = 0..2      (splitmix64 stream;
 *           the reference's tests draw from the same generator,
 *           tests/m4a/test_moe.c:47-53)
 *   S     = sum of the twelve 16-bit fields of d_0, d_1, d_2
 *   z     = (S - 12*32767.5) / 65536          (Irwin-Hall(12): mean 0,
 *           variance 1 to 2e-10, support +-6 sigma)
 *   value = bf16_rne((float)(z * sigma))
 *
 * The narrowing is the reference's RNE rule (c/bf16.h:268-274).
 */
#ifndef APUS_SYNTH_H
#define APUS_SYNTH_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define APUS_SYNTH_FN __host__ __device__ static inline
#else
#define APUS_SYNTH_FN static inline
#endif

#define APUS_SYNTH_GAMMA 0x9E3779B97F4A7C15ull

/* tensor ids */
enum {
    APUS_SYNTH_X = 0,
    APUS_SYNTH_RTR_W = 1,
    APUS_SYNTH_EXP_GU = 2,
    APUS_SYNTH_EXP_D = 3,
    APUS_SYNTH_SH_G = 4,
    APUS_SYNTH_SH_U = 5,
    APUS_SYNTH_SH_D = 6,
    APUS_SYNTH_SH_GATE = 7,
    APUS_SYNTH_BIAS_PERM = 8
};

APUS_SYNTH_FN uint64_t apus_synth_mix(uint64_t z) {
    z += APUS_SYNTH_GAMMA;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

APUS_SYNTH_FN uint64_t apus_synth_key(uint64_t seed, uint32_t layer,
                                      uint32_t tensor_id) {
    return apus_synth_mix(apus_synth_mix(seed) ^
                          (((uint64_t)layer << 8) | (uint64_t)tensor_id));
}

APUS_SYNTH_FN uint32_t apus_synth_sum16(uint64_t d) {
    return (uint32_t)(d & 0xffff) + (uint32_t)((d >> 16) & 0xffff) +
           (uint32_t)((d >> 32) & 0xffff) + (uint32_t)(d >> 48);
}

/* approximately N(0,1), exactly reproducible */
APUS_SYNTH_FN double apus_synth_normal(uint64_t key, uint64_t i) {
    uint64_t c = key + (3ull * i) * APUS_SYNTH_GAMMA;
    uint32_t s = apus_synth_sum16(apus_synth_mix(c)) +
                 apus_synth_sum16(apus_synth_mix(c + APUS_SYNTH_GAMMA)) +
                 apus_synth_sum16(apus_synth_mix(c + 2 * APUS_SYNTH_GAMMA));
    return ((double)s - 393210.0) / 65536.0;
}

APUS_SYNTH_FN uint16_t apus_synth_bf16_rne(float f) {
    uint32_t u;
#if defined(__CUDA_ARCH__)
    u = __float_as_uint(f);
#else
    memcpy(&u, &f, 4);
#endif
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(u >> 16);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

APUS_SYNTH_FN uint16_t apus_synth_bf16(uint64_t key, uint64_t i,
                                       double sigma) {
    return apus_synth_bf16_rne((float)(apus_synth_normal(key, i) * sigma));
}

#endif /* APUS_SYNTH_H */
