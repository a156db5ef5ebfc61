// Host entry points of the window builder.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace s3d {
int64_t window_build_workspace_bytes(int64_t N);
int window_build_launch(const int32_t *coords, const float *feats, int64_t N, int F, int stride,
                        int ws, int shift, int32_t *n2n, float *n_coords, int32_t *w_sizes,
                        int32_t *w2n, int64_t *counts, void *workspace, int64_t workspace_bytes,
                        cudaStream_t st);
}
