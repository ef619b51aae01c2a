// Host helper shared by the TMA-fed kernels: cached construction of 128-byte-swizzled tiled tensor maps.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace ocb {

// rank 2 or 3; dims / box innermost first; strides_bytes for dims 1.. ; the inner box extent must span 128 bytes.
bool get_tensor_map(CUtensorMap* out, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box, int elem_bytes);

}  // namespace ocb
