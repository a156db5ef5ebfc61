// Host entry point of the KNN kernel.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace s3d {
int knn_launch(int K, const float *src, const float *query, const int32_t *src_offset,
               const int32_t *query_offset, int B, int64_t Nq, int32_t *ret_idx, float *ret_dist,
               cudaStream_t st);
}
