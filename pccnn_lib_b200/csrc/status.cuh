// Sticky failure word shared by the operators whose kernels report through a status word (status.cu).
#pragma once

#include <cuda_runtime.h>

namespace pccnn {

enum : int { kOriginConvForward = 1, kOriginConvBackward = 2, kOriginWeightVar = 3 };

// Enqueues a one-thread kernel on `s` that copies a non-zero *status_dev (a word in the caller's workspace that
// the kernels before it may have set) into the process-wide pinned word, tagged with `origin`.
int publish_status(const int* status_dev, int origin, cudaStream_t s);

// Reads and clears the pinned word without synchronising.  Returns PCCNN_ERR_DEVICE (message set) if an earlier
// operator recorded a failure, PCCNN_OK otherwise.
int take_sticky_status(const char* who);

}  // namespace pccnn
