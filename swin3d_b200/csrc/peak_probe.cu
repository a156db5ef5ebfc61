// fp32 FMA throughput probe: the roofline denominator of the brute-force KNN, whose bit-exact distance
// expression keeps it on the CUDA cores (no GEMM formulation).  Every thread runs eight independent
// FFMA chains; one block of 1024 threads per SM slot.  The caller times the launch with CUDA events:
// flops = blocks * 1024 * iters * 8 chains * 2.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/swin3d_b200.h"

namespace s3d {

__global__ void __launch_bounds__(1024) ffma_probe_kernel(float *out, int iters, float a, float b)
{
    float x0 = threadIdx.x, x1 = x0 + 1.f, x2 = x0 + 2.f, x3 = x0 + 3.f, x4 = x0 + 4.f, x5 = x0 + 5.f, x6 = x0 + 6.f,
          x7 = x0 + 7.f;
#pragma unroll 4
    for (int i = 0; i < iters; ++i) {
        x0 = fmaf(x0, a, b); x1 = fmaf(x1, a, b); x2 = fmaf(x2, a, b); x3 = fmaf(x3, a, b);
        x4 = fmaf(x4, a, b); x5 = fmaf(x5, a, b); x6 = fmaf(x6, a, b); x7 = fmaf(x7, a, b);
    }
    out[blockIdx.x * (int64_t)blockDim.x + threadIdx.x] = ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7));
}

}  // namespace s3d

extern "C" int s3d_debug_ffma_probe(float *out, int blocks, int iters, void *stream)
{
    if (!out || blocks < 1 || iters < 1) return S3D_ERR_BAD_ARG;
    s3d::ffma_probe_kernel<<<blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(out, iters, 0.999f, 0.001f);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}
