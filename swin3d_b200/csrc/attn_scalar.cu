// Generic ("scalar") cRSE window-attention kernels: any window size, head_dim 8/16/32,
// 3/6/9 signal dimensions, fp32 or fp16 storage with fp32 arithmetic throughout.
//
// Semantics follow the reference kernels of microsoft/Swin3D
// (Swin3D/src/attn/self_attn_aio_fwd.cu:16-52,111-188, self_attn_aio_bwd.cu:14-113):
//   s_qk = sum_c ( q_c k_c + q_c * sum_n Tq[n,idx_n,h,c] + k_c * sum_n Tk[n,idx_n,h,c] )
//   out_q = sum_k softmax_k(s_qk) * ( v_k + sum_n Tv[n,idx_n,h,:] )
// but the structure is different: a group of head_dim lanes (lane = channel) owns one
// (voxel, head) row, so rows of q, k, v and of the tables are read as coalesced pieces; the
// softmax is online, outputs are written once (no atomics), and the backward keeps the per-head
// table gradients in shared memory until the block retires.
#include "attn_kernels.cuh"
#include "common.cuh"

namespace s3d {

template <typename T> __device__ __forceinline__ float ldf(const T *p);
template <> __device__ __forceinline__ float ldf<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <typename T> __device__ __forceinline__ void stf(T *p, float x);
template <> __device__ __forceinline__ void stf<float>(float *p, float x) { *p = x; }
template <> __device__ __forceinline__ void stf<__half>(__half *p, float x) { *p = __float2half_rn(x); }

// Window that holds position p of the window-sorted voxel list: the last w with w2n[w] <= p.
__device__ __forceinline__ int64_t window_of(const int32_t *__restrict__ w2n, int64_t W, int p)
{
    int64_t lo = 0, hi = W - 1;
    while (lo < hi) {
        const int64_t mid = (lo + hi + 1) >> 1;
        if (__ldg(w2n + mid) <= p) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

// Sum over the HD lanes of a group (groups are aligned, so xor offsets below HD stay inside).
template <int HD>
__device__ __forceinline__ float group_sum(float x, unsigned gmask)
{
#pragma unroll
    for (int o = HD / 2; o > 0; o >>= 1) x += __shfl_xor_sync(gmask, x, o);
    return x;
}

// Table rows of the pair (query coordinates cq, key coordinates at ck) and the three sums of
// this lane's channel over the D looked-up rows.
template <typename T, int D>
__device__ __forceinline__ void pair_tables(const float *cq, const float *ck, const CrseMeta &m,
                                            const T *__restrict__ tq, const T *__restrict__ tk,
                                            const T *__restrict__ tv, int HC, int hc, int *rows,
                                            float &bq, float &bk, float &bv)
{
    bq = bk = bv = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        rows[d] = m.rowbase[d] + crse_index(cq[d], ck[d], m.L[d], d == D - 1);
        const int64_t off = (int64_t)rows[d] * HC + hc;
        bq += ldf(tq + off);
        bk += ldf(tk + off);
        bv += ldf(tv + off);
    }
}

// ---------------------------------------------------------------------------------------------
// Forward: a group of HD lanes (lane = channel) owns one (query, head) row and walks the keys of
// the query's window; every row of q, k, v and of the tables is read as one coalesced piece.
template <typename T, int HD, int D>
__global__ void __launch_bounds__(256)
attn_fwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t N, int64_t W, int H,
                       T *__restrict__ out, float *__restrict__ lse)
{
    constexpr int G = 32 / HD;
    const int lane = threadIdx.x & 31, c = lane % HD, gi = lane / HD;
    const unsigned gmask = HD == 32 ? 0xffffffffu : (((1u << (HD & 31)) - 1u) << (gi * HD));
    const int HC = H * HD;
    const int64_t group0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G + gi;
    const int64_t ngroups = (int64_t)gridDim.x * (blockDim.x >> 5) * G;

    for (int64_t item = group0; item < N * H; item += ngroups) {
        const int p = (int)(item / H), h = (int)(item - (int64_t)p * H);
        const int64_t w = window_of(w2n, W, p);
        const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
        const int64_t qrow = __ldg(n2n + p);
        const int hc = h * HD + c;
        const float qc = ldf(q + qrow * HC + hc);
        float cq[D];
#pragma unroll
        for (int d = 0; d < D; ++d) cq[d] = __ldg(n_coords + (int64_t)p * D + d);
        float acc = 0.f, mx = -INFINITY, l = 0.f;
        for (int kj = 0; kj < n; ++kj) {
            const int64_t krow = __ldg(n2n + base + kj);
            float ck[D];
#pragma unroll
            for (int d = 0; d < D; ++d) ck[d] = __ldg(n_coords + (int64_t)(base + kj) * D + d);
            const float kc = ldf(k + krow * HC + hc), vc = ldf(v + krow * HC + hc);
            int rows[D];
            float bq, bk, bv;
            pair_tables<T, D>(cq, ck, meta, tq, tk, tv, HC, hc, rows, bq, bk, bv);
            const float s = group_sum<HD>(qc * (kc + bq) + kc * bk, gmask);
            const float mnew = fmaxf(mx, s);
            const float scale = __expf(mx - mnew);
            const float pr = __expf(s - mnew);
            l = l * scale + pr;
            acc = acc * scale + pr * (vc + bv);
            mx = mnew;
        }
        stf(out + qrow * HC + hc, acc / l);
        if (c == 0) lse[qrow * H + h] = mx + __logf(l);
    }
}

// ---------------------------------------------------------------------------------------------
// Backward.  grid = (position chunks, H); one block works on one head so the three per-head
// table-gradient slices (3 * R * HD floats) fit in shared memory.  A group of HD lanes (lane =
// channel) takes one position of the window-sorted voxel list, first as a query (dQ, dTq, dTv over
// the keys of its window), then as a key (dK, dV, dTk over the queries).  Every quantity is
// recomputed from q, k, v, tables, out and lse; dP - delta is one sum, sum_c dO_c (v_c + B_c - o_c).
// The shared-memory adds of a group hit HD consecutive words, so they do not collide.
template <typename T, int HD, int D>
__global__ void __launch_bounds__(256)
attn_bwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t N, int64_t W, int H,
                       int positions_per_block,
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

    constexpr int G = 32 / HD;
    const int lane = threadIdx.x & 31, c = lane % HD, gi = lane / HD;
    const unsigned gmask = HD == 32 ? 0xffffffffu : (((1u << (HD & 31)) - 1u) << (gi * HD));
    const int h = blockIdx.y;
    const int HC = H * HD, hc = h * HD + c;
    const int group = (threadIdx.x >> 5) * G + gi, ngroup = (blockDim.x >> 5) * G;
    const int64_t pbeg = (int64_t)blockIdx.x * positions_per_block;
    const int64_t pend = min(N, pbeg + (int64_t)positions_per_block);

    for (int64_t pp = pbeg + group; pp < pend; pp += ngroup) {
        const int p = (int)pp;
        const int64_t w = window_of(w2n, W, p);
        const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
        const int64_t row = __ldg(n2n + p);
        float cp[D];
#pragma unroll
        for (int d = 0; d < D; ++d) cp[d] = __ldg(n_coords + (int64_t)p * D + d);
        // ---- position p as a query ---------------------------------------------------------------
        {
            const float qc = ldf(q + row * HC + hc), gc = ldf(dout + row * HC + hc);
            const float oc = ldf(o + row * HC + hc);
            const float L = __ldg(lse + row * H + h);
            float dqa = 0.f;
            for (int kj = 0; kj < n; ++kj) {
                const int64_t krow = __ldg(n2n + base + kj);
                float ck[D];
#pragma unroll
                for (int d = 0; d < D; ++d) ck[d] = __ldg(n_coords + (int64_t)(base + kj) * D + d);
                const float kc = ldf(k + krow * HC + hc), vc = ldf(v + krow * HC + hc);
                int rows[D];
                float bq, bk, bv;
                pair_tables<T, D>(cp, ck, meta, tq, tk, tv, HC, hc, rows, bq, bk, bv);
                const float s = group_sum<HD>(qc * (kc + bq) + kc * bk, gmask);
                const float e = group_sum<HD>(gc * (vc + bv - oc), gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
                dqa += ds * (kc + bq);
                const float aq = ds * qc, av = pr * gc;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    atomicAdd(s_dtq + rows[d] * HD + c, aq);
                    atomicAdd(s_dtv + rows[d] * HD + c, av);
                }
            }
            stf(dq + row * HC + hc, dqa);
        }
        // ---- position p as a key -----------------------------------------------------------------
        {
            const float kc = ldf(k + row * HC + hc), vc = ldf(v + row * HC + hc);
            float dka = 0.f, dva = 0.f;
            for (int qi = 0; qi < n; ++qi) {
                const int64_t qrow = __ldg(n2n + base + qi);
                float cq[D];
#pragma unroll
                for (int d = 0; d < D; ++d) cq[d] = __ldg(n_coords + (int64_t)(base + qi) * D + d);
                const float qc = ldf(q + qrow * HC + hc), gc = ldf(dout + qrow * HC + hc);
                const float oc = ldf(o + qrow * HC + hc);
                const float L = __ldg(lse + qrow * H + h);
                int rows[D];
                float bq, bk, bv;
                pair_tables<T, D>(cq, cp, meta, tq, tk, tv, HC, hc, rows, bq, bk, bv);
                const float s = group_sum<HD>(qc * (kc + bq) + kc * bk, gmask);
                const float e = group_sum<HD>(gc * (vc + bv - oc), gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
                dka += ds * (qc + bk);
                dva += pr * gc;
                const float ak = ds * kc;
#pragma unroll
                for (int d = 0; d < D; ++d) atomicAdd(s_dtk + rows[d] * HD + c, ak);
            }
            stf(dk + row * HC + hc, dka);
            stf(dv + row * HC + hc, dva);
        }
    }
    __syncthreads();
    // flush: element (row r, channel c) of this head lives at (r*H + h)*HD + c in the flat table
    for (int i = threadIdx.x; i < RH; i += blockDim.x) {
        const int r = i / HD, cc = i - r * HD;
        const int64_t g = ((int64_t)r * H + h) * HD + cc;
        const float a = s_dtq[i], b = s_dtk[i], e = s_dtv[i];
        if (a != 0.f) atomicAdd(dtq + g, a);
        if (b != 0.f) atomicAdd(dtk + g, b);
        if (e != 0.f) atomicAdd(dtv + g, e);
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
    if (a.W == 0 || a.N == 0) return S3D_OK;
    const int groups_per_block = 8 * (32 / HD);
    int64_t blocks = (a.N * a.H + groups_per_block - 1) / groups_per_block;
    const int64_t cap = 148 * 64;
    if (blocks > cap) blocks = cap;
    attn_fwd_scalar_kernel<T, HD, D><<<(unsigned)blocks, 256, 0, st>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq, (const T *)a.tk,
        (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n, a.n_coords, a.N, a.W, a.H, (T *)a.out, a.lse);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <typename T, int HD, int D>
static int launch_bwd(const AttnArgs &a, cudaStream_t st)
{
    if (a.W == 0 || a.N == 0) return S3D_OK;
    const size_t smem = (size_t)3 * a.meta.R * HD * sizeof(float);
    if (smem > 200 * 1024) return S3D_ERR_UNSUPPORTED;
    auto kern = attn_bwd_scalar_kernel<T, HD, D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    // enough blocks to fill the machine a few times over, few enough that the per-block flush
    // of the table gradients stays small
    const int64_t target_blocks = (148 * 8 + a.H - 1) / a.H;
    int64_t ppb = (a.N + target_blocks - 1) / target_blocks;
    const int groups_per_block = 8 * (32 / HD);
    if (ppb < groups_per_block) ppb = groups_per_block;
    const int64_t chunks = (a.N + ppb - 1) / ppb;
    dim3 grid((unsigned)chunks, (unsigned)a.H);
    kern<<<grid, 256, smem, st>>>((const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq,
                                  (const T *)a.tk, (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n,
                                  a.n_coords, a.N, a.W, a.H, (int)ppb, (const T *)a.out, a.lse,
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
