/* placeholder until the tcgen05 grouped GEMM lands */
#pragma once
#include "../../include/backend_cuda.h"
#include "dispatch.cuh"
namespace apus {
struct PrefillMaps;
inline bool prefill_supported(const ApusCudaMoeCfg &) { return false; }
inline PrefillMaps *prefill_maps_create(const ApusCudaMoeCfg &, const uint16_t *, const uint16_t *, const uint16_t *, const uint16_t *, const uint16_t *, size_t) { return nullptr; }
inline void prefill_maps_free(PrefillMaps *) {}
inline size_t prefill_tile_list_bytes(size_t, size_t, size_t) { return 0; }
inline const char *prefill_last_error() { return "prefill path not built"; }
inline int run_prefill_experts(int, int, PrefillMaps *, const ApusCudaMoeCfg &, const uint16_t *, const uint16_t *, const uint16_t *, const uint16_t *, const uint16_t *, const uint16_t *, int, DispatchOut, uint16_t *, uint16_t *, uint16_t *, uint16_t *, uint16_t *, int32_t *, int *, cudaStream_t, int *) { return 1; }
}
