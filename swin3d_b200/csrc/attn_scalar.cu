// Generic ("scalar") cRSE window-attention kernels: any window size, head_dim 8/16/32,
// 3/6/9 signal dimensions, fp32 or fp16 storage with fp32 arithmetic throughout.
//
// Semantics follow the reference kernels of microsoft/Swin3D
// (Swin3D/src/attn/self_attn_aio_fwd.cu:16-52,111-188, self_attn_aio_bwd.cu:14-113):
//   s_qk = sum_c ( q_c k_c + q_c * sum_n Tq[n,idx_n,h,c] + k_c * sum_n Tk[n,idx_n,h,c] )
//   out_q = sum_k softmax_k(s_qk) * ( v_k + sum_n Tv[n,idx_n,h,:] )
// but the structure is different: one warp owns a whole window, one lane owns one
// (query, head) row, the softmax is online, outputs are written once (no atomics), and the
// backward keeps the per-head table gradients in shared memory until the block retires.
#include "attn_kernels.cuh"
#include "common.cuh"

namespace s3d {

template <int D>
__device__ __forceinline__ void pair_rows(const float *cq, const float *__restrict__ ck,
                                          const CrseMeta &m, int *rows)
{
#pragma unroll
    for (int n = 0; n < D; ++n)
        rows[n] = m.rowbase[n] + crse_index(cq[n], __ldg(ck + n), m.L[n], n == D - 1);
}

// ---------------------------------------------------------------------------------------------
// Forward: warp per window, lane per (query, head).
template <typename T, int HD, int D>
__global__ void __launch_bounds__(128)
attn_fwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t W, int H,
                       T *__restrict__ out, float *__restrict__ lse)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int HC = H * HD;

    for (int64_t w = warp0; w < W; w += nwarps) {
        const int n = __ldg(w_sizes + w);
        const int base = __ldg(w2n + w);
        for (int item = lane; item < n * H; item += 32) {
            const int qi = item / H, h = item - qi * H;
            const int64_t qrow = __ldg(n2n + base + qi);
            float qv[HD], cq[D], acc[HD];
            load_vec<T, HD>(q + qrow * HC + h * HD, qv);
#pragma unroll
            for (int d = 0; d < D; ++d) cq[d] = __ldg(n_coords + (int64_t)(base + qi) * D + d);
#pragma unroll
            for (int c = 0; c < HD; ++c) acc[c] = 0.f;
            float mx = -INFINITY, l = 0.f;
            for (int kj = 0; kj < n; ++kj) {
                const int64_t krow = __ldg(n2n + base + kj);
                int rows[D];
                pair_rows<D>(cq, n_coords + (int64_t)(base + kj) * D, meta, rows);
                float kv[HD], bq[HD], bk[HD], bv[HD];
                load_vec<T, HD>(k + krow * HC + h * HD, kv);
#pragma unroll
                for (int c = 0; c < HD; ++c) bq[c] = bk[c] = bv[c] = 0.f;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    float t[HD];
                    const int64_t off = (int64_t)rows[d] * HC + h * HD;
                    load_vec<T, HD>(tq + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bq[c] += t[c];
                    load_vec<T, HD>(tk + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bk[c] += t[c];
                    load_vec<T, HD>(tv + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bv[c] += t[c];
                }
                float s = 0.f;
#pragma unroll
                for (int c = 0; c < HD; ++c) s += qv[c] * (kv[c] + bq[c]) + kv[c] * bk[c];
                float vv[HD];
                load_vec<T, HD>(v + krow * HC + h * HD, vv);
                const float mnew = fmaxf(mx, s);
                const float scale = __expf(mx - mnew);
                const float p = __expf(s - mnew);
                l = l * scale + p;
#pragma unroll
                for (int c = 0; c < HD; ++c) acc[c] = acc[c] * scale + p * (vv[c] + bv[c]);
                mx = mnew;
            }
            const float inv = 1.f / l;
#pragma unroll
            for (int c = 0; c < HD; ++c) acc[c] *= inv;
            store_vec<T, HD>(out + qrow * HC + h * HD, acc);
            lse[qrow * H + h] = mx + __logf(l);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Backward.  grid = (window chunks, H); one block works on one head so the three per-head
// table-gradient slices (3 * R * HD floats) fit in shared memory.  Inside a block every warp
// takes windows of the chunk; pass A runs with lane = query (dQ, dTq, dTv), pass B with
// lane = key (dK, dV, dTk).  Every quantity is recomputed from q,k,v,tables,lse.
template <typename T, int HD, int D>
__global__ void __launch_bounds__(128)
attn_bwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t W, int H, int windows_per_block,
                       const T *__restrict__ o, const float *__restrict__ lse,
                       const T *__restrict__ dout, T *__restrict__ dq, T *__restrict__ dk,
                       T *__restrict__ dv, float *__restrict__ dtq, float *__restrict__ dtk,
                       float *__restrict__ dtv)
{
    extern __shared__ float s_dt[];  // [3][R*HD]
    const int RH = meta.R * HD;
    for (int i = threadIdx.x; i < 3 * RH; i += blockDim.x) s_dt[i] = 0.f;
    __syncthreads();
    float *s_dtq = s_dt, *s_dtk = s_dt + RH, *s_dtv = s_dt + 2 * RH;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int h = blockIdx.y;
    const int HC = H * HD;
    const int64_t wbeg = (int64_t)blockIdx.x * windows_per_block;
    const int64_t wend = min(W, wbeg + (int64_t)windows_per_block);

    for (int64_t w = wbeg + warp; w < wend; w += nwarp) {
        const int n = __ldg(w_sizes + w);
        const int base = __ldg(w2n + w);
        // ---- pass A: lane = query ------------------------------------------------------------
        for (int qi = lane; qi < n; qi += 32) {
            const int64_t qrow = __ldg(n2n + base + qi);
            float qv[HD], gv[HD], cq[D], dqa[HD];
            load_vec<T, HD>(q + qrow * HC + h * HD, qv);
            load_vec<T, HD>(dout + qrow * HC + h * HD, gv);
            float delta = 0.f;
            {
                float ov[HD];
                load_vec<T, HD>(o + qrow * HC + h * HD, ov);
#pragma unroll
                for (int c = 0; c < HD; ++c) delta += ov[c] * gv[c];
            }
            const float L = __ldg(lse + qrow * H + h);
#pragma unroll
            for (int d = 0; d < D; ++d) cq[d] = __ldg(n_coords + (int64_t)(base + qi) * D + d);
#pragma unroll
            for (int c = 0; c < HD; ++c) dqa[c] = 0.f;
            for (int kj = 0; kj < n; ++kj) {
                const int64_t krow = __ldg(n2n + base + kj);
                int rows[D];
                pair_rows<D>(cq, n_coords + (int64_t)(base + kj) * D, meta, rows);
                float kv[HD], vv[HD], bq[HD], bk[HD], bv[HD];
                load_vec<T, HD>(k + krow * HC + h * HD, kv);
                load_vec<T, HD>(v + krow * HC + h * HD, vv);
#pragma unroll
                for (int c = 0; c < HD; ++c) bq[c] = bk[c] = bv[c] = 0.f;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    float t[HD];
                    const int64_t off = (int64_t)rows[d] * HC + h * HD;
                    load_vec<T, HD>(tq + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bq[c] += t[c];
                    load_vec<T, HD>(tk + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bk[c] += t[c];
                    load_vec<T, HD>(tv + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bv[c] += t[c];
                }
                float s = 0.f, dp = 0.f;
#pragma unroll
                for (int c = 0; c < HD; ++c) {
                    s += qv[c] * (kv[c] + bq[c]) + kv[c] * bk[c];
                    dp += gv[c] * (vv[c] + bv[c]);
                }
                const float p = __expf(s - L);
                const float ds = p * (dp - delta);
#pragma unroll
                for (int c = 0; c < HD; ++c) dqa[c] += ds * (kv[c] + bq[c]);
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int ro = rows[d] * HD;
#pragma unroll
                    for (int c = 0; c < HD; ++c) {
                        atomicAdd(s_dtq + ro + c, ds * qv[c]);
                        atomicAdd(s_dtv + ro + c, p * gv[c]);
                    }
                }
            }
            store_vec<T, HD>(dq + qrow * HC + h * HD, dqa);
        }
        // ---- pass B: lane = key --------------------------------------------------------------
        for (int kj = lane; kj < n; kj += 32) {
            const int64_t krow = __ldg(n2n + base + kj);
            float kv[HD], vv[HD], ck[D], dka[HD], dva[HD];
            load_vec<T, HD>(k + krow * HC + h * HD, kv);
            load_vec<T, HD>(v + krow * HC + h * HD, vv);
#pragma unroll
            for (int d = 0; d < D; ++d) ck[d] = __ldg(n_coords + (int64_t)(base + kj) * D + d);
#pragma unroll
            for (int c = 0; c < HD; ++c) dka[c] = dva[c] = 0.f;
            for (int qi = 0; qi < n; ++qi) {
                const int64_t qrow = __ldg(n2n + base + qi);
                int rows[D];
#pragma unroll
                for (int d = 0; d < D; ++d)
                    rows[d] = meta.rowbase[d] +
                              crse_index(__ldg(n_coords + (int64_t)(base + qi) * D + d), ck[d],
                                         meta.L[d], d == D - 1);
                float qv[HD], gv[HD], ov[HD], bq[HD], bk[HD], bv[HD];
                load_vec<T, HD>(q + qrow * HC + h * HD, qv);
                load_vec<T, HD>(dout + qrow * HC + h * HD, gv);
                load_vec<T, HD>(o + qrow * HC + h * HD, ov);
                const float L = __ldg(lse + qrow * H + h);
#pragma unroll
                for (int c = 0; c < HD; ++c) bq[c] = bk[c] = bv[c] = 0.f;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    float t[HD];
                    const int64_t off = (int64_t)rows[d] * HC + h * HD;
                    load_vec<T, HD>(tq + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bq[c] += t[c];
                    load_vec<T, HD>(tk + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bk[c] += t[c];
                    load_vec<T, HD>(tv + off, t);
#pragma unroll
                    for (int c = 0; c < HD; ++c) bv[c] += t[c];
                }
                float s = 0.f, dp = 0.f, delta = 0.f;
#pragma unroll
                for (int c = 0; c < HD; ++c) {
                    s += qv[c] * (kv[c] + bq[c]) + kv[c] * bk[c];
                    dp += gv[c] * (vv[c] + bv[c]);
                    delta += ov[c] * gv[c];
                }
                const float p = __expf(s - L);
                const float ds = p * (dp - delta);
#pragma unroll
                for (int c = 0; c < HD; ++c) {
                    dka[c] += ds * (qv[c] + bk[c]);
                    dva[c] += p * gv[c];
                }
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int ro = rows[d] * HD;
#pragma unroll
                    for (int c = 0; c < HD; ++c) atomicAdd(s_dtk + ro + c, ds * kv[c]);
                }
            }
            store_vec<T, HD>(dk + krow * HC + h * HD, dka);
            store_vec<T, HD>(dv + krow * HC + h * HD, dva);
        }
    }
    __syncthreads();
    // flush: element (row r, channel c) of this head lives at (r*H + h)*HD + c in the flat table
    for (int i = threadIdx.x; i < RH; i += blockDim.x) {
        const int r = i / HD, c = i - r * HD;
        const int64_t g = ((int64_t)r * H + h) * HD + c;
        const float a = s_dtq[i], b = s_dtk[i], cc = s_dtv[i];
        if (a != 0.f) atomicAdd(dtq + g, a);
        if (b != 0.f) atomicAdd(dtk + g, b);
        if (cc != 0.f) atomicAdd(dtv + g, cc);
    }
}

__global__ void crse_indices_kernel(const float *__restrict__ n_coords, const CrseMeta meta,
                                    int first_pos, int n, int32_t *__restrict__ out)
{
    const int D = meta.D;
    const int64_t total = (int64_t)n * n * D;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(t % D);
        const int64_t pr = t / D;
        const int j = (int)(pr % n), i = (int)(pr / n);
        out[t] = crse_index(n_coords[(int64_t)(first_pos + i) * D + d],
                            n_coords[(int64_t)(first_pos + j) * D + d], meta.L[d], d == D - 1);
    }
}

// ---------------------------------------------------------------------------------------------
template <typename T, int HD, int D>
static int launch_fwd(const AttnArgs &a, cudaStream_t st)
{
    if (a.W == 0) return S3D_OK;
    const int warps_per_block = 4;
    int64_t blocks = (a.W + warps_per_block - 1) / warps_per_block;
    const int64_t cap = 148 * 16;
    if (blocks > cap) blocks = cap;
    attn_fwd_scalar_kernel<T, HD, D><<<(unsigned)blocks, warps_per_block * 32, 0, st>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq, (const T *)a.tk,
        (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n, a.n_coords, a.W, a.H, (T *)a.out, a.lse);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <typename T, int HD, int D>
static int launch_bwd(const AttnArgs &a, cudaStream_t st)
{
    if (a.W == 0) return S3D_OK;
    const size_t smem = (size_t)3 * a.meta.R * HD * sizeof(float);
    if (smem > 200 * 1024) return S3D_ERR_UNSUPPORTED;
    auto kern = attn_bwd_scalar_kernel<T, HD, D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    // enough blocks to fill the machine a few times over, few enough that the per-block flush
    // of the table gradients stays small
    int64_t target_blocks = (148 * 8 + a.H - 1) / a.H;
    int64_t wpb = (a.W + target_blocks - 1) / target_blocks;
    if (wpb < 4) wpb = 4;
    const int64_t chunks = (a.W + wpb - 1) / wpb;
    dim3 grid((unsigned)chunks, (unsigned)a.H);
    kern<<<grid, 128, smem, st>>>((const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq,
                                  (const T *)a.tk, (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n,
                                  a.n_coords, a.W, a.H, (int)wpb, (const T *)a.out, a.lse,
                                  (const T *)a.dout, (T *)a.dq, (T *)a.dk, (T *)a.dv, a.dtq, a.dtk,
                                  a.dtv);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <typename T, int HD>
static int dispatch_d(const AttnArgs &a, bool bwd, cudaStream_t st)
{
    switch (a.meta.D) {
        case 3: return bwd ? launch_bwd<T, HD, 3>(a, st) : launch_fwd<T, HD, 3>(a, st);
        case 6: return bwd ? launch_bwd<T, HD, 6>(a, st) : launch_fwd<T, HD, 6>(a, st);
        case 9: return bwd ? launch_bwd<T, HD, 9>(a, st) : launch_fwd<T, HD, 9>(a, st);
        default: return S3D_ERR_UNSUPPORTED;
    }
}

template <typename T>
static int dispatch_hd(const AttnArgs &a, bool bwd, cudaStream_t st)
{
    switch (a.hd) {
        case 8: return dispatch_d<T, 8>(a, bwd, st);
        case 16: return dispatch_d<T, 16>(a, bwd, st);
        case 32: return dispatch_d<T, 32>(a, bwd, st);
        default: return S3D_ERR_UNSUPPORTED;
    }
}

int attn_scalar_forward(const AttnArgs &a, cudaStream_t st)
{
    return a.dtype == S3D_F16 ? dispatch_hd<__half>(a, false, st) : dispatch_hd<float>(a, false, st);
}

int attn_scalar_backward(const AttnArgs &a, cudaStream_t st)
{
    return a.dtype == S3D_F16 ? dispatch_hd<__half>(a, true, st) : dispatch_hd<float>(a, true, st);
}

int crse_indices_dump(const float *n_coords, const CrseMeta &meta, int first_pos, int n,
                      int32_t *out, cudaStream_t st)
{
    if (n <= 0) return S3D_OK;
    const int64_t total = (int64_t)n * n * meta.D;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 1184) blocks = 1184;
    crse_indices_kernel<<<blocks, 256, 0, st>>>(n_coords, meta, first_pos, n, out);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

}  // namespace s3d
