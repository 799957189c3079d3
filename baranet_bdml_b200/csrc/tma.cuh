// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled), reached
// through the runtime's driver-entry-point lookup so that the library does not
// link against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bn {

// dims[0] is the innermost (contiguous) dimension; strides_bytes[i] is the
// stride of dimension i+1 (rank-1 entries); box[i] the tile extent.
// Returns BN_OK or a failure code with the message recorded.
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

}  // namespace bn
