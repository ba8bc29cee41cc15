// Device-side Lloyd k-means (see kmeans.cu for the arithmetic it pins).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// x_dev [n][d], cent_dev [k][d] (output), both on `device`.  assign_out_dev: optional [n] int32, the
// assignment of every vector to the FINAL centroids.  Synchronous.
void kmeans_device(int device, int d, int64_t n, const float* x_dev, int k, int niter, uint64_t seed, float* cent_dev,
                   int32_t* assign_out_dev);

}  // namespace b200
