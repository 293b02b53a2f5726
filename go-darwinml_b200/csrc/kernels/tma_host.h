// Host side of TMA: tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>

#include "../common.h"

namespace b200 {
namespace k {

// 4-D tiled map over 16-bit elements with 128-byte (default) or 64-byte swizzle.  dims / box are innermost first;
// strides (bytes) are for dims 1..3 and must be multiples of 16.
Status encode_tma_4d_16bit(CUtensorMap* map, const void* base, bool f16, const uint64_t dims[4], const uint64_t strides_bytes[3],
                           const uint32_t box[4], int swizzle_bytes = 128);

}  // namespace k
}  // namespace b200
