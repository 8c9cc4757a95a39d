// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver
// entry point, so the library does not link libcuda), with a small per-thread cache: a decode or
// prefill loop calls with the same buffers and shapes step after step, and re-encoding two to four
// 128-byte descriptors per launch costs more host time than the launch itself on short kernels.
// An encoded map is a pure function of (base, dims, strides, box), so a cached copy never goes stale.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace rt {

// bf16 tiled map with 128-byte swizzle, 256-byte L2 promotion, no out-of-bounds fill.
// rank <= 4; dims / box have `rank` entries (innermost first), strides_bytes has rank - 1.
bool encode_bf16_map_cached(CUtensorMap* out, int rank, const void* base, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace rt
