// Host-side argument block and entry points of the attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace s3d {

// Further copies of a result array: every row the kernels write is also stored to the same row of
// these buffers (other GPUs' result arrays mapped into this process: plain peer stores).
struct Mirrors {
    int n;
    void *p[S3D_MAX_MIRRORS];
};

struct AttnArgs {
    const void *q, *k, *v, *tq, *tk, *tv;
    CrseMeta meta;
    const int32_t *w_sizes, *w2n, *n2n;
    const float *n_coords;
    int64_t N, W;
    int H, hd, dtype;
    void *out;        // forward: written; backward: read
    float *lse;       // forward: written; backward: read
    const void *dout; // backward only
    void *dq, *dk, *dv;
    float *dtq, *dtk, *dtv;
    Mirrors m_out, m_dq, m_dk, m_dv;   // forward: m_out; backward: m_dq, m_dk, m_dv
    int window_class;                  // forward: 0 mixed window sizes, 1 all <= 32 voxels, 2 all larger
};

// The last CUDA runtime error a launcher of this library ran into (cudaSuccess if none), for
// s3d_last_cuda_error_string(); S3D_ERR_LAUNCH alone does not say which one it was.
void note_cuda_error(cudaError_t e);

// Generic path (attn_scalar.cu).
int attn_scalar_forward(const AttnArgs &a, cudaStream_t st);
int attn_scalar_backward(const AttnArgs &a, cudaStream_t st);
int crse_indices_dump(const float *n_coords, const CrseMeta &meta, int first_pos, int n,
                      int32_t *out, cudaStream_t st);
// crse_debug.cu: the index function of each kernel family (variant 0, 1, 2) on given inputs.
int crse_indices_dump_variant(const float *n_coords, const CrseMeta &meta, int first_pos, int n, int variant,
                              int32_t *out, cudaStream_t st);
int crse_index_values(const float *cq, const float *ck, int64_t n, int L, int last, int variant, int32_t *out,
                      cudaStream_t st);

// Tensor-core path (attn_tc_fwd.cu): fp16 storage, head_dim 8, even head count.
bool attn_tc_supported(const AttnArgs &a);
int attn_tc_forward(const AttnArgs &a, cudaStream_t st);
int attn_tc_head_mode(const AttnArgs &a);                      // HDM_* of attn_tc.cuh for this call
bool attn_tc_fwd_small_supported(const AttnArgs &a);          // attn_tc_fwd_small.cu: windows <= 32 voxels
int attn_tc_forward_small(const AttnArgs &a, cudaStream_t st);
bool attn_tc_bwd_supported(const AttnArgs &a);
int attn_tc_backward(const AttnArgs &a, cudaStream_t st);   // dtq/dtk/dtv zeroed by the caller
bool attn_tc_bwd_small_supported(const AttnArgs &a);          // attn_tc_bwd_small.cu: windows <= 32 voxels
int attn_tc_backward_small(const AttnArgs &a, cudaStream_t st);

}  // namespace s3d
