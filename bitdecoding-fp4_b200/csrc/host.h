// Host-side glue shared by the translation units of libbdfp4.so.
#pragma once

#include <cuda_runtime.h>

#include "../../include/bdfp4.h"

namespace bdfp4 {

// Records a failed CUDA call for bdfp4_last_cuda_error and maps it to a status code.
int cuda_status(cudaError_t error);

}  // namespace bdfp4
