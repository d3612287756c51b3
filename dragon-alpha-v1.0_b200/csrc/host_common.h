// Declarations shared by the host translation units of the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*PFN_encodeIm2col)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                     cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);

namespace alpha {

// Records a printf-style message as the calling thread's last error and returns `code`.
int fail(int code, const char* fmt, ...);
// Counts one kernel launch and remembers the kernel family for alpha_conv_last_algo().
void note_launch(const char* algo);

}  // namespace alpha
