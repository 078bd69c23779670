/*
 * oracle/synth_host.c — TEST INFRASTRUCTURE, not product code.
 *
 * Host-only build of the seeded synthetic tensor stream (the generator itself
 * is csrc/synth.h of the package, shared with the CUDA library, so both sides
 * draw from one definition).  It lets the benchmark's reference arm and the
 * CPU tests produce their inputs without loading the CUDA library.
 */
#include <stddef.h>
#include <stdint.h>

#include "../apus-qwen3.6-35b-a3b_b200/csrc/synth.h"

#define ORC_API __attribute__((visibility("default")))

ORC_API void orc_synth_fill(uint16_t *dst, size_t n, uint64_t seed,
                            uint32_t layer, uint32_t tensor_id, uint64_t first,
                            double sigma) {
    const uint64_t key = apus_synth_key(seed, layer, tensor_id);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++)
        dst[i] = apus_synth_bf16(key, first + (uint64_t)i, sigma);
}
