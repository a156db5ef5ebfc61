// Debug entry points that evaluate the cRSE index function of every kernel family on caller-given
// inputs, so that each variant can be compared bit for bit with the reference's
// PositionEmbedding::set_qk_offset (Swin3D/src/attn/attn_utils.cuh:437-453):
//   variant 0  crse_index       (common.cuh)  generic fp32 / fp16-storage kernels
//   variant 1  crse_index_fast  (attn_tc.cuh) tiled tensor-core kernels
//   variant 2  crse_index_pc    (attn_tc.cuh) single-tile tensor-core kernels (constants precomputed)
#include "attn_kernels.cuh"
#include "attn_tc.cuh"

namespace s3d {

__device__ __forceinline__ int crse_index_variant(int variant, float cq, float ck, int L, bool last)
{
    if (variant == 1) return tc::crse_index_fast(cq, ck, L, last);
    if (variant == 2) return (int)tc::crse_index_pc(cq, ck, (float)(L / 2), (uint32_t)(last ? L - 1 : L));
    return crse_index(cq, ck, L, last);
}

__global__ void crse_index_values_kernel(const float *__restrict__ cq, const float *__restrict__ ck, int64_t n,
                                         int L, int last, int variant, int32_t *__restrict__ out)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = crse_index_variant(variant, cq[i], ck[i], L, last != 0);
}

__global__ void crse_indices_variant_kernel(const float *__restrict__ n_coords, const CrseMeta meta, int first_pos,
                                            int n, int variant, int32_t *__restrict__ out)
{
    const int D = meta.D;
    const int64_t total = (int64_t)n * n * D;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(t % D);
        const int64_t pr = t / D;
        const int j = (int)(pr % n), i = (int)(pr / n);
        out[t] = crse_index_variant(variant, n_coords[(int64_t)(first_pos + i) * D + d],
                                    n_coords[(int64_t)(first_pos + j) * D + d], meta.L[d], d == D - 1);
    }
}

int crse_index_values(const float *cq, const float *ck, int64_t n, int L, int last, int variant, int32_t *out,
                      cudaStream_t st)
{
    const int64_t blocks = (n + 255) / 256;
    crse_index_values_kernel<<<(unsigned)(blocks > 1184 ? 1184 : blocks), 256, 0, st>>>(cq, ck, n, L, last, variant, out);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

int crse_indices_dump_variant(const float *n_coords, const CrseMeta &meta, int first_pos, int n, int variant,
                              int32_t *out, cudaStream_t st)
{
    const int64_t total = (int64_t)n * n * meta.D;
    const int64_t blocks = (total + 255) / 256;
    crse_indices_variant_kernel<<<(unsigned)(blocks > 1184 ? 1184 : blocks), 256, 0, st>>>(n_coords, meta, first_pos, n,
                                                                                          variant, out);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

}  // namespace s3d
