// Row gather: dst[a][i][:] = src_a[idx[i]][:] for up to four per-voxel arrays sharing one index list,
// and row scatter: dst_a[idx[i]][:] = src[block(i)][a][i % block_rows][:], rows with idx < 0 skipped.
// Used by the multi-GPU window split to pack a rank's rows into its send buffer and to put the rows
// that arrived from the other ranks into voxel order.  HBM-bound byte work: one thread moves one 16-byte piece of a row, so
// a warp reads and writes whole 160- to 1280-byte rows in consecutive pieces.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/swin3d_b200.h"

namespace s3d {

struct GatherArgs {
    const uint4 *src[4];
    uint4 *dst;
    const int64_t *idx;
    int64_t n_rows;
    int64_t dst_array_stride;   // in 16-byte pieces
    int ppr;                    // 16-byte pieces per row
};

__global__ void __launch_bounds__(256) gather_rows_kernel(const GatherArgs a)
{
    const uint4 *src = a.src[blockIdx.y];
    uint4 *dst = a.dst + blockIdx.y * a.dst_array_stride;
    const int64_t total = a.n_rows * a.ppr;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = t / a.ppr;
        const int p = (int)(t - i * a.ppr);
        dst[t] = __ldg(src + __ldg(a.idx + i) * a.ppr + p);
    }
}

struct ScatterArgs {
    uint4 *dst[4];
    const uint4 *src;
    const int64_t *idx;
    int64_t n_rows, block_rows;
    int64_t block_stride, array_stride;   // in 16-byte pieces
    int ppr;
};

__global__ void __launch_bounds__(256) scatter_rows_kernel(const ScatterArgs a)
{
    uint4 *dst = a.dst[blockIdx.y];
    const uint4 *src = a.src + blockIdx.y * a.array_stride;
    const int64_t total = a.n_rows * a.ppr;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = t / a.ppr;
        const int p = (int)(t - i * a.ppr);
        const int64_t v = __ldg(a.idx + i);
        if (v < 0) continue;
        const int64_t b = i / a.block_rows, o = i - b * a.block_rows;
        dst[v * a.ppr + p] = __ldg(src + b * a.block_stride + o * a.ppr + p);
    }
}

}  // namespace s3d

extern "C" int s3d_scatter_rows(const void *src, int A, const int64_t *idx, int64_t n_rows, int64_t row_bytes,
                                int64_t block_rows, int64_t src_block_stride_bytes, int64_t src_array_stride_bytes,
                                void *const *dsts_host, void *stream)
{
    if (A < 1 || A > 4 || n_rows < 0 || row_bytes <= 0 || (row_bytes & 15) || block_rows <= 0 ||
        (src_block_stride_bytes & 15) || (src_array_stride_bytes & 15))
        return S3D_ERR_BAD_ARG;
    if (n_rows == 0) return S3D_OK;
    if (!dsts_host || !idx || !src || (reinterpret_cast<uintptr_t>(src) & 15)) return S3D_ERR_BAD_ARG;
    s3d::ScatterArgs a{};
    for (int i = 0; i < A; ++i) {
        if (!dsts_host[i] || (reinterpret_cast<uintptr_t>(dsts_host[i]) & 15)) return S3D_ERR_BAD_ARG;
        a.dst[i] = static_cast<uint4 *>(dsts_host[i]);
    }
    a.src = static_cast<const uint4 *>(src);
    a.idx = idx;
    a.n_rows = n_rows;
    a.block_rows = block_rows;
    a.block_stride = src_block_stride_bytes / 16;
    a.array_stride = src_array_stride_bytes / 16;
    a.ppr = (int)(row_bytes / 16);
    const int64_t total = n_rows * a.ppr;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = 148 * 16;
    if (blocks > cap) blocks = cap;
    dim3 grid((unsigned)blocks, (unsigned)A);
    s3d::scatter_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

extern "C" int s3d_gather_rows(const void *const *srcs_host, int A, const int64_t *idx, int64_t n_rows,
                               int64_t row_bytes, void *dst, int64_t dst_array_stride_bytes, void *stream)
{
    if (A < 1 || A > 4 || n_rows < 0 || row_bytes <= 0 || (row_bytes & 15) || (dst_array_stride_bytes & 15))
        return S3D_ERR_BAD_ARG;
    if (n_rows == 0) return S3D_OK;
    if (!srcs_host || !idx || !dst || (reinterpret_cast<uintptr_t>(dst) & 15)) return S3D_ERR_BAD_ARG;
    s3d::GatherArgs a{};
    for (int i = 0; i < A; ++i) {
        if (!srcs_host[i] || (reinterpret_cast<uintptr_t>(srcs_host[i]) & 15)) return S3D_ERR_BAD_ARG;
        a.src[i] = static_cast<const uint4 *>(srcs_host[i]);
    }
    a.dst = static_cast<uint4 *>(dst);
    a.idx = idx;
    a.n_rows = n_rows;
    a.dst_array_stride = dst_array_stride_bytes / 16;
    a.ppr = (int)(row_bytes / 16);
    const int64_t total = n_rows * a.ppr;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = 148 * 16;
    if (blocks > cap) blocks = cap;
    dim3 grid((unsigned)blocks, (unsigned)A);
    s3d::gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}
