// Internal interface of the data-parallel communicator (comm.cu).
#pragma once

#include "common.cuh"

namespace ag {

// One kernel on `rank`'s stream: all-reduce (sum, rank order) of the gradient bucket over the
// peers' symmetric blocks, scaling by `scale`, and the SGD update of `values` (with
// `velocity` when use_momentum).  grads receives the reduced, scaled gradient.  The buckets
// hold n elements of dtype, are 16-byte aligned and padded to whole 16-byte packs.
// AG_ERR_LIMIT when the bucket exceeds the symmetric block, AG_ERR_UNSUPPORTED when the
// communicator's GPUs cannot address one another.
int comm_fused_update(ag_comm *comm, int rank, ag_dtype dtype, void *grads, void *values,
                      void *velocity, int64_t n, float scale, float lr, float momentum,
                      bool use_momentum);

}  // namespace ag
