/* swin3d_b200 -- C ABI of the B200 (sm_100a) library for Swin3D's sparse-voxel window attention
 * with contextual relative signal encoding (cRSE), its window builder, and the KNN used by
 * knn_down / Upsample.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name ends in _host.  The caller owns every
 *    buffer; the library allocates nothing, frees nothing and keeps no state between calls
 *    (the one exception, for the multi-GPU split, is the explicit pair s3d_peer_alloc / s3d_peer_free).
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  Calls only
 *    enqueue work; they never synchronise.
 *  - Return value: S3D_OK or an S3D_ERR_* code; s3d_status_string() names it.  Nothing here
 *    aborts the process (the reference's shape checks are host assert()s that abort).
 *  - dtype codes: S3D_F32 = 0, S3D_F16 = 1.  Accumulation is always fp32.
 *  - File:line citations name the interface of microsoft/Swin3D each entry point replaces.
 */
#ifndef SWIN3D_B200_H
#define SWIN3D_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define S3D_OK 0
#define S3D_ERR_BAD_ARG 1        /* null pointer, negative size, unknown dtype           */
#define S3D_ERR_UNSUPPORTED 2    /* head_dim, signal-dim count, K or window size not built */
#define S3D_ERR_LAUNCH 3         /* the CUDA runtime reported an error at launch           */
#define S3D_ERR_WORKSPACE 4      /* caller-provided workspace too small                    */
#define S3D_ERR_TOO_LARGE 5      /* input exceeds the fixed capacity of a *_static entry   */

#define S3D_F32 0
#define S3D_F16 1

#define S3D_MAX_SIGNAL_DIMS 9
#define S3D_KNN_MAX_K 64

const char *s3d_status_string(int status);

/* Library/ABI version (major*1000 + minor). */
int s3d_version(void);

/* Text of the last CUDA runtime error behind an S3D_ERR_LAUNCH of the single-tile attention
 * launchers ("no error" if none).  The reference reports launch errors through
 * C10_CUDA_KERNEL_LAUNCH_CHECK (Swin3D/src/attn/self_attn_aio_fwd.cu:448).                   */
const char *s3d_last_cuda_error_string(void);

/* ---------------------------------------------------------------------------------------------
 * Fused cRSE window attention, forward.
 * Replaces the pair  attn_cuda.cal_max_coffs + attn_cuda.self_attn_forward  and the host-side
 * normalisation (Swin3D/src/attn/self_attn_aio_fwd.h:11-26, Swin3D/src/attn/attn_api.cpp:20-23,
 * Swin3D/sparse_dl/attn/attn_coff.py:180-184) for IndexMode.INDIRECT + PosEmb.SEPARATE.
 *
 *  q,k,v        [N,H,hd] contiguous, ORIGINAL voxel order, dtype `dtype`; q already scaled.
 *  tq,tk,tv     flat tables, dtype `dtype`: concat over signal dims n of [L_n,H,hd].
 *  table_sizes_host  int32[D] on the HOST: elements per signal dim (L_n*H*hd).
 *  w_sizes,w2n  int32[W]: voxels per window, first sorted position of each window.
 *  n2n          int32[N]: sorted position -> voxel row.
 *  n_coords     float[N,D]: quantised signals in WINDOW-SORTED order.
 *  out          [N,H,hd] dtype `dtype`, original order: softmax-weighted values.
 *  lse          float[N,H], original order: log-sum-exp of each (voxel, head) score row.
 * Supported: hd in {8,16,32}; D in {3,6,9}; any H; any window size >= 1.
 * q, k, v, out and the tables (and dout, dq, dk, dv, dtq, dtk, dtv of the backward) must be
 * 16-byte aligned: S3D_ERR_BAD_ARG otherwise.
 */
int s3d_attn_fwd(const void *q, const void *k, const void *v,
                 const void *tq, const void *tk, const void *tv,
                 const int32_t *table_sizes_host, int D,
                 const int32_t *w_sizes, const int32_t *w2n, const int32_t *n2n,
                 const float *n_coords, int64_t N, int64_t W, int H, int hd, int dtype,
                 void *out, float *lse, void *stream);

/* Fused cRSE window attention, backward.
 * Replaces  attn_cuda.cal_exp_sum_grads + attn_cuda.self_attn_indir_backward  and the host-side
 * raw = norm*sum (Swin3D/src/attn/self_attn_aio_bwd.h:9-32, Swin3D/src/attn/attn_api.cpp:21,24,
 * Swin3D/sparse_dl/attn/attn_coff.py:219-224).
 *
 *  out, lse     the forward's outputs;  dout [N,H,hd] dtype `dtype`: upstream gradient.
 *  dq,dk,dv     [N,H,hd] dtype `dtype`, overwritten.
 *  dtq,dtk,dtv  float[sum table_sizes], overwritten (zeroed on `stream`, then accumulated).
 */
int s3d_attn_bwd(const void *q, const void *k, const void *v,
                 const void *tq, const void *tk, const void *tv,
                 const int32_t *table_sizes_host, int D,
                 const int32_t *w_sizes, const int32_t *w2n, const int32_t *n2n,
                 const float *n_coords, int64_t N, int64_t W, int H, int hd, int dtype,
                 const void *out, const float *lse, const void *dout,
                 void *dq, void *dk, void *dv, float *dtq, float *dtk, float *dtv,
                 void *stream);

/* The same two calls for one window set split over several GPUs: every row of out (forward) or of
 * dq, dk, dv (backward) that the call writes is ALSO stored to the same row of n_mirrors further
 * buffers of the same shape -- the result arrays of the other GPUs, mapped into this process
 * (s3d_ipc_open) -- by plain peer stores from inside the kernels, so that the exchange overlaps the
 * computation and no pack / collective / un-permute pass follows.  *_mirrors_host: HOST arrays of
 * n_mirrors <= S3D_MAX_MIRRORS device pointers, 16-byte aligned.  The caller orders the ranks
 * afterwards (any collective issued on the same stream, e.g. the all-reduce of the table
 * gradients: when it has completed on a rank, every rank's kernels have finished and their rows
 * are in place).  S3D_ERR_UNSUPPORTED for shapes served by kernels without mirrored stores (the
 * generic path and head_dim 16 with an even head count and large tables).
 * window_class (forward): 0 = windows of any size; 1 = the caller guarantees that every window of
 * this call has at most 32 voxels, 2 = that every window has more.  The forward runs one kernel for
 * each class and each walks the whole window list for its own windows; a caller that has the sizes
 * on the host (the multi-GPU split plans its ranges from them) passes the two classes in two calls
 * and saves both walks.  A window that breaks the guarantee is NOT processed.
 * The reference has no multi-GPU attention; this replaces nothing in it.                        */
#define S3D_MAX_MIRRORS 7
int s3d_attn_fwd_mirrored(const void *q, const void *k, const void *v,
                          const void *tq, const void *tk, const void *tv,
                          const int32_t *table_sizes_host, int D,
                          const int32_t *w_sizes, const int32_t *w2n, const int32_t *n2n,
                          const float *n_coords, int64_t N, int64_t W, int H, int hd, int dtype,
                          void *out, float *lse, int n_mirrors, void *const *out_mirrors_host,
                          int window_class, void *stream);
int s3d_attn_bwd_mirrored(const void *q, const void *k, const void *v,
                          const void *tq, const void *tk, const void *tv,
                          const int32_t *table_sizes_host, int D,
                          const int32_t *w_sizes, const int32_t *w2n, const int32_t *n2n,
                          const float *n_coords, int64_t N, int64_t W, int H, int hd, int dtype,
                          const void *out, const float *lse, const void *dout,
                          void *dq, void *dk, void *dv, float *dtq, float *dtk, float *dtv,
                          int n_mirrors, void *const *dq_mirrors_host, void *const *dk_mirrors_host,
                          void *const *dv_mirrors_host, void *stream);

/* Result arrays that other processes of this node can map: s3d_peer_alloc allocates `bytes` on the
 * current device (its own allocation, so that it can be exported) and writes the 64-byte CUDA IPC
 * memory handle of it to handle64_out; the owner releases it with s3d_peer_free once no peer maps
 * it any more.  s3d_ipc_open maps such an allocation of ANOTHER process into this process for the
 * current device, with peer access enabled on first use (*ptr_out = its base address);
 * s3d_ipc_close unmaps it.  These are the only calls of the library that allocate.             */
int s3d_peer_alloc(int64_t bytes, void **ptr_out, void *handle64_out);
int s3d_peer_free(void *ptr);
int s3d_ipc_open(const void *handle64, void **ptr_out);
int s3d_ipc_close(void *ptr);

/* fp32 FMA throughput probe (the roofline denominator of the KNN kernel, which stays on the CUDA cores
 * because its distance expression must match the reference bit for bit): launches `blocks` blocks
 * of 1024 threads, each thread running 8 independent chains of `iters` fused multiply-adds; the caller
 * times it.  out: float[blocks * 1024].  Replaces nothing in the reference.                      */
int s3d_debug_ffma_probe(float *out, int blocks, int iters, void *stream);

/* Debug switch: on != 0 routes every later attention call of this process to the generic kernels
 * (any window size, head_dim 8/16/32, fp32 arithmetic) instead of the tensor-core kernels, so that
 * the two implementations can be compared on the same GPU; returns the previous setting.
 * Replaces nothing in the reference.                                                          */
int s3d_debug_force_generic(int on);

/* Dump of the cRSE row indices idx[q,k,n] of one window (for bit-exact index tests).
 * Replaces nothing callable in the reference; it exposes PositionEmbedding::set_qk_offset
 * (Swin3D/src/attn/attn_utils.cuh:437-453).  idx_out: int32[n*n*D], n = w_sizes[window].    */
int s3d_debug_crse_indices(const float *n_coords, const int32_t *table_sizes_host, int D,
                           int H, int hd, int32_t first_pos, int32_t n, int32_t *idx_out,
                           void *stream);

/* The same dump through the index function of one kernel family, so that the code the tensor-core
 * kernels run is compared bit for bit too: variant 0 = generic kernels (as above), 1 = tiled
 * tensor-core kernels, 2 = single-tile tensor-core kernels.  All three restate
 * PositionEmbedding::set_qk_offset (Swin3D/src/attn/attn_utils.cuh:444-450).                 */
int s3d_debug_crse_indices_variant(const float *n_coords, const int32_t *table_sizes_host, int D,
                                   int H, int hd, int32_t first_pos, int32_t n, int variant,
                                   int32_t *idx_out, void *stream);

/* idx_out[i] = index of one signal dimension with L table rows for the coordinate pair
 * (cq[i], ck[i]) (device arrays of n floats), through variant 0, 1 or 2; last_dim != 0 applies
 * the clamp of the last signal dimension.  For sweeps over boundary values, NaN and infinities
 * (Swin3D/src/attn/attn_utils.cuh:444-450).                                                   */
int s3d_debug_crse_index_values(const float *cq, const float *ck, int64_t n, int L, int last_dim,
                                int variant, int32_t *idx_out, void *stream);

/* Row gather for the multi-GPU window split: dst[a][i][:] = src_a[idx[i]][:] for A <= 4 per-voxel
 * arrays that share one index list (rows of row_bytes, a multiple of 16; array a of the result
 * starts dst_array_stride_bytes after array a-1).  srcs_host: HOST array of A device pointers.
 * The reference has no multi-GPU code; within one GPU it scatters results through n2n_indices
 * inside its kernels (Swin3D/src/attn/attn_utils.cuh:391-409), which is what this un-permutation
 * undoes for rows that arrive from other ranks in window-sorted order.                        */
int s3d_gather_rows(const void *const *srcs_host, int A, const int64_t *idx, int64_t n_rows,
                    int64_t row_bytes, void *dst, int64_t dst_array_stride_bytes, void *stream);

/* Row scatter, the other half of the exchange: rows that arrived packed as
 * [block][array][block_rows] (one block per sending rank) go to their voxel rows,
 * dst_a[idx[i]][:] = src[i / block_rows][a][i % block_rows][:] for i < n_rows; rows with idx[i] < 0
 * (padding, and the receiving rank's own rows, which its kernels already wrote in place) are
 * skipped.  dsts_host: HOST array of A <= 4 device pointers; strides in bytes, multiples of 16.  */
int s3d_scatter_rows(const void *src, int A, const int64_t *idx, int64_t n_rows, int64_t row_bytes,
                     int64_t block_rows, int64_t src_block_stride_bytes, int64_t src_array_stride_bytes,
                     void *const *dsts_host, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Window builder.  Replaces BasicLayer.get_map_pair / get_window_mapping / get_index01 and
 * sparse_self_attention (Swin3D/modules/swin3d_layers.py:713-822 and :76-150), i.e. the
 * MinkowskiEngine pooling + insert_and_map + kernel_map + torch.sort + cumsum chain.
 *
 *  coords       int32[N,4] (batch, x, y, z), multiples of `stride` (the tensor stride).
 *  shift        window shift in voxels (0 or ws/2); window = floor((c + shift*stride)/(ws*stride)).
 *  feats        float[N,F] per-voxel signals: columns 0..2 = position inside the voxel in [0,1),
 *               columns 3.. = colour / normal signals (F = 3, 6 or 9).
 *  Outputs: n2n int32[N]; n_coords float[N,F] (cell + local xyz, then the other signals, sorted
 *  order); w_sizes, w2n int32[>=N] (first W valid);
 *  counts_out int64[4] = {W, M = sum w^2, max w, error word (1 = a coordinate or batch index is
 *  outside the key range: batch < 1024, |window index| < 16384)}.
 *  Windows come out in lexicographic (batch, wx, wy, wz) order, voxels inside a window in
 *  ascending cell id cx*ws^2 + cy*ws + cz.
 *  workspace: s3d_window_build_workspace_bytes(N) bytes.
 */
int64_t s3d_window_build_workspace_bytes(int64_t N);
int s3d_window_build(const int32_t *coords, const float *feats, int64_t N, int F,
                     int stride, int ws, int shift,
                     int32_t *n2n, float *n_coords, int32_t *w_sizes, int32_t *w2n,
                     int64_t *counts_out,
                     void *workspace, int64_t workspace_bytes, void *stream);

/* Window builder for callers that cannot allocate device memory (no counterpart in the
 * reference, whose builder allocates freely through PyTorch).  Same inputs, outputs and results as
 * s3d_window_build, but the scratch memory is a fixed 4.07 MiB array (the scratch layout of the largest accepted call) that is part of the library
 * image on every GPU that loads it, so neither the caller nor the library allocates anything: no
 * cudaMalloc, no cudaFree, no allocating library routine.  Meant for hosts whose memory is
 * frozen after start-up (an inference server that gave its arena every spare byte) or that
 * must not enter an allocator from the context they call from.
 *  - At most S3D_WINDOW_BUILD_STATIC_MAX_VOXELS voxels per call; more returns S3D_ERR_TOO_LARGE
 *    and launches nothing.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress
 *    with that device current) and caches it; make that first call before any stream capture.
 *  - All calls on one device share the one array: calls that overlap on the GPU (different
 *    streams, or threads) race and corrupt each other's results.  Serialise them.  The array
 *    keeps whatever the last call left; no call depends on it.
 */
#define S3D_WINDOW_BUILD_STATIC_MAX_VOXELS 131072
int s3d_window_build_static(const int32_t *coords, const float *feats, int64_t N, int F,
                            int stride, int ws, int shift,
                            int32_t *n2n, float *n_coords, int32_t *w_sizes, int32_t *w2n,
                            int64_t *counts_out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Brute-force KNN.  Replaces knn_cuda.knn_cuda (Swin3D/src/knn/knn_cuda_kernel.h:5-12,
 * Swin3D/src/knn/knn_api.cpp:4-6).
 *  src [Ns,3], query [Nq,3] float; src_offset, query_offset int32[B] cumulative scene ends.
 *  ret_idx int32[Nq,K] (row numbers into src), ret_dist float[Nq,K] SQUARED distances,
 *  ascending; selection and tie behaviour identical to the reference's max-heap scan.
 *  Slots without a candidate keep distance 2^31 and index 0.  1 <= K <= 64.
 */
int s3d_knn(int K, const float *src, const float *query, const int32_t *src_offset,
            const int32_t *query_offset, int B, int64_t Ns, int64_t Nq,
            int32_t *ret_idx, float *ret_dist, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Consumers of the KNN result (the callers either side of s3d_knn).
 *
 * s3d_knn_interpolate_fwd / _bwd replace the body of knn_linear_interpolation
 * (Swin3D/modules/swin3d_layers.py:53-73) after its KNN.apply call:
 *     w_i = 1/(dist_i + 1e-8);  w_i /= sum_j w_j;  out[q,:] = sum_i src_feat[idx[q,i],:] * w_i
 *  idx int32[Nq,K] and dist float[Nq,K] are KNN.apply's outputs (dist = sqrt of s3d_knn's
 *  ret_dist); src_feat [Ns,C], out/dout [Nq,C] in `dtype` (S3D_F32 or S3D_F16); 1 <= K <= 64;
 *  C a multiple of 4 (fp32) or 8 (fp16), rows 16-byte aligned.
 *  fp32 results follow the reference's operation order exactly; for fp16 the running sum is
 *  rounded to fp16 after every neighbour, as the reference's in-place += does.
 *  _bwd writes dsrc float[Ns,C] = the gradient w.r.t. src_feat (cleared by the call, accumulated
 *  in fp32); dist and the coordinates receive no gradient, as in the reference.
 *
 * s3d_knn_maxpool_fwd / _bwd replace gather + MaxPool1d(K) of GridKNNDownsample.forward
 * (swin3d_layers.py:302-309; query_knn_feature :28-50).  LayerNorm and the bias-free Linear of
 * that block act on each gathered row by itself, so the caller applies them once per SOURCE row
 * (g = linear(norm(src_feat)), [Ns,C]) and this call finishes the job:
 *     out[q,c] = max_i g[idx[q,i], c],   arg[q,c] = the source row that supplied it
 *  (first maximum wins on ties, NaN propagates, as MaxPool1d).  _bwd: dg float[Ns,C] (cleared by
 *  the call) receives dout[q,c] at row arg[q,c].
 */
int s3d_knn_interpolate_fwd(const int32_t *idx, const float *dist, const void *src_feat, void *out,
                            int64_t Nq, int K, int C, int dtype, void *stream);
int s3d_knn_interpolate_bwd(const int32_t *idx, const float *dist, const void *dout, float *dsrc,
                            int64_t Nq, int64_t Ns, int K, int C, int dtype, void *stream);
int s3d_knn_maxpool_fwd(const int32_t *idx, const void *g, void *out, int32_t *arg,
                        int64_t Nq, int K, int C, int dtype, void *stream);
int s3d_knn_maxpool_bwd(const int32_t *arg, const void *dout, float *dg,
                        int64_t Nq, int64_t Ns, int C, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SWIN3D_B200_H */
