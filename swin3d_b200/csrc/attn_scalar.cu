// Generic ("scalar") cRSE window-attention kernels: any window size, head_dim 8/16/32,
// 3/6/9 signal dimensions, fp32 or fp16 storage with fp32 arithmetic throughout.
//
// Semantics follow the reference kernels of microsoft/Swin3D
// (Swin3D/src/attn/self_attn_aio_fwd.cu:16-52,111-188, self_attn_aio_bwd.cu:14-113):
//   s_qk = sum_c ( q_c k_c + q_c * sum_n Tq[n,idx_n,h,c] + k_c * sum_n Tk[n,idx_n,h,c] )
//   out_q = sum_k softmax_k(s_qk) * ( v_k + sum_n Tv[n,idx_n,h,:] )
// but the structure is different: a group of head_dim lanes (lane = channel) owns one
// (voxel, head) row, so rows of q, k, v and of the tables are read as coalesced pieces; the
// softmax is online, outputs are written once (no atomics), and the backward sums the scalar
// weights of every looked-up table row in per-group histograms and touches the global table
// gradient once per (voxel, head, touched row).
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

// The signal dimensions are dealt to the lanes of a group: lane c works out the table row of
// dimensions c, c + HD, ... (one per lane, two for lane 0 of an 8-lane group with 9 dimensions)
// and the group exchanges the rows by shuffles.
template <int HD, int D>
struct LaneDims {
    static constexpr int NDL = (D + HD - 1) / HD;
    float own[NDL];   // this voxel's coordinate in the lane's dimensions
    int L[NDL], rb[NDL], dim[NDL];
    bool last[NDL];

    __device__ __forceinline__ void init(const CrseMeta &m, int c)
    {
#pragma unroll
        for (int j = 0; j < NDL; ++j) {
            const int d = c + j * HD;
            const bool ok = d < D;
            dim[j] = ok ? d : 0;
            L[j] = m.L[dim[j]];
            rb[j] = m.rowbase[dim[j]];
            last[j] = d == D - 1;
        }
    }
    __device__ __forceinline__ void load(const float *__restrict__ coords_row, float (&x)[NDL]) const
    {
#pragma unroll
        for (int j = 0; j < NDL; ++j) x[j] = __ldg(coords_row + dim[j]);
    }
};

// Table rows of a pair and the three sums of this lane's channel over the D looked-up rows.
// oth: the other voxel's coordinate in this lane's dimensions; OWN_IS_QUERY says which side the
// lane's own voxel is on.
template <typename T, int HD, int D, bool OWN_IS_QUERY>
__device__ __forceinline__ void pair_tables(const LaneDims<HD, D> &ld, const float (&oth)[LaneDims<HD, D>::NDL],
                                            int gi, unsigned gmask,
                                            const T *__restrict__ tq, const T *__restrict__ tk,
                                            const T *__restrict__ tv, int HC, int hc,
                                            int (&mine)[LaneDims<HD, D>::NDL],
                                            float &bq, float &bk, float &bv)
{
    constexpr int NDL = LaneDims<HD, D>::NDL;
#pragma unroll
    for (int j = 0; j < NDL; ++j)
        mine[j] = ld.rb[j] + (OWN_IS_QUERY ? crse_index(ld.own[j], oth[j], ld.L[j], ld.last[j])
                                           : crse_index(oth[j], ld.own[j], ld.L[j], ld.last[j]));
    bq = bk = bv = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const int row = __shfl_sync(gmask, mine[d / HD], gi * HD + d % HD);
        const int64_t off = (int64_t)row * HC + hc;
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
        LaneDims<HD, D> ld;
        ld.init(meta, c);
        ld.load(n_coords + (int64_t)p * D, ld.own);
        float acc = 0.f, mx = -INFINITY, l = 0.f;
        // the next key's row number and coordinates are fetched one iteration ahead
        int64_t krow_n = __ldg(n2n + base);
        float oth_n[LaneDims<HD, D>::NDL];
        ld.load(n_coords + (int64_t)base * D, oth_n);
        for (int kj = 0; kj < n; ++kj) {
            const int64_t krow = krow_n;
            float oth[LaneDims<HD, D>::NDL];
#pragma unroll
            for (int j = 0; j < LaneDims<HD, D>::NDL; ++j) oth[j] = oth_n[j];
            const int nx = base + min(kj + 1, n - 1);
            krow_n = __ldg(n2n + nx);
            ld.load(n_coords + (int64_t)nx * D, oth_n);
            const float kc = ldf(k + krow * HC + hc), vc = ldf(v + krow * HC + hc);
            int mine[LaneDims<HD, D>::NDL];
            float bq, bk, bv;
            pair_tables<T, HD, D, true>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
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
// Backward.  A group of HD lanes (lane = channel) takes one (position, head) of the window-sorted
// voxel list, first as a query (dQ, dTq, dTv over the keys of its window), then as a key (dK, dV,
// dTk over the queries).  Every quantity is recomputed from q, k, v, tables, out and lse;
// dP - delta is one sum, sum_c dO_c (v_c + B_c - o_c).
//
// Table gradients: for a fixed query, dTq[r] = q * (sum of ds over the keys whose pair looks up
// row r), and likewise dTv[r] = dO * (sum of p) and, for a fixed key, dTk[r] = k * (sum of ds).
// So each group keeps two scalar histograms over the table rows in shared memory, updated by the
// lane that owns the signal dimension with a plain read-modify-write, and after the sweep adds
// (histogram entry) x (its row vector) to the global table gradient once per touched row.
// Histogram rows use a numbering in which every dimension owns L + 1 rows (index L, which through
// the reference's flat addressing names row 0 of the next dimension, gets a private slot), so lanes
// of different dimensions never touch the same word.
template <int D>
__device__ __forceinline__ int flat_row_of_slot(const CrseMeta &m, int slot)
{
    int d = 0;
#pragma unroll
    for (int i = 1; i < D; ++i) d += (slot >= m.rowbase[i] + i) ? 1 : 0;
    return slot - d;
}

// Adds x[slot] * (va, vb) to the rows of two global tables for every non-zero slot of the
// group's two histograms, and clears the histograms.  ta/tb may be the same pointer pair twice.
template <int HD, int D>
__device__ __forceinline__ void flush_hists(float *ha, float *hb, int n_slots, const CrseMeta &m,
                                            float *__restrict__ ta, float va,
                                            float *__restrict__ tb, float vb, bool use_b,
                                            int HC, int hc, int c, int gi, unsigned gmask)
{
    __syncwarp(gmask);
    for (int s0 = 0; s0 < n_slots; s0 += HD) {
        const int si = s0 + c;
        float a = 0.f, b = 0.f;
        if (si < n_slots) {
            a = ha[si];
            ha[si] = 0.f;
            if (use_b) {
                b = hb[si];
                hb[si] = 0.f;
            }
        }
        unsigned nz = __ballot_sync(gmask, a != 0.f || b != 0.f) >> (gi * HD);
        if (HD < 32) nz &= (1u << (HD & 31)) - 1u;
        while (nz) {
            const int j = __ffs(nz) - 1;
            nz &= nz - 1;
            const float aj = __shfl_sync(gmask, a, gi * HD + j);
            const float bj = __shfl_sync(gmask, b, gi * HD + j);
            const int64_t off = (int64_t)flat_row_of_slot<D>(m, s0 + j) * HC + hc;
            if (aj != 0.f) atomicAdd(ta + off, aj * va);
            if (use_b && bj != 0.f) atomicAdd(tb + off, bj * vb);
        }
    }
    __syncwarp(gmask);
}

template <typename T, int HD, int D>
__global__ void __launch_bounds__(256)
attn_bwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t N, int64_t W, int H, int slots_padded,
                       const T *__restrict__ o, const float *__restrict__ lse,
                       const T *__restrict__ dout, T *__restrict__ dq, T *__restrict__ dk,
                       T *__restrict__ dv, float *__restrict__ dtq, float *__restrict__ dtk,
                       float *__restrict__ dtv)
{
    extern __shared__ float s_hist[];  // [groups of the block][2][slots_padded]
    constexpr int G = 32 / HD;
    constexpr int NDL = LaneDims<HD, D>::NDL;
    const int lane = threadIdx.x & 31, c = lane % HD, gi = lane / HD;
    const unsigned gmask = HD == 32 ? 0xffffffffu : (((1u << (HD & 31)) - 1u) << (gi * HD));
    const int HC = H * HD;
    const int n_slots = meta.R + D;
    for (int i = threadIdx.x; i < (blockDim.x >> 5) * G * 2 * slots_padded; i += blockDim.x) s_hist[i] = 0.f;
    __syncthreads();
    float *ha = s_hist + (size_t)((threadIdx.x >> 5) * G + gi) * 2 * slots_padded;
    float *hb = ha + slots_padded;
    const int64_t group0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G + gi;
    const int64_t ngroups = (int64_t)gridDim.x * (blockDim.x >> 5) * G;

    LaneDims<HD, D> ld;
    ld.init(meta, c);
    bool mine_ok[NDL];
#pragma unroll
    for (int j = 0; j < NDL; ++j) mine_ok[j] = c + j * HD < D;

    for (int64_t item = group0; item < N * H; item += ngroups) {
        const int p = (int)(item / H), h = (int)(item - (int64_t)p * H);
        const int hc = h * HD + c;
        const int64_t w = window_of(w2n, W, p);
        const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
        const int64_t row = __ldg(n2n + p);
        ld.load(n_coords + (int64_t)p * D, ld.own);
        // ---- position p as a query ---------------------------------------------------------------
        {
            const float qc = ldf(q + row * HC + hc), gc = ldf(dout + row * HC + hc);
            const float oc = ldf(o + row * HC + hc);
            const float L = __ldg(lse + row * H + h);
            float dqa = 0.f;
            int64_t krow_n = __ldg(n2n + base);
            float oth_n[NDL];
            ld.load(n_coords + (int64_t)base * D, oth_n);
            for (int kj = 0; kj < n; ++kj) {
                const int64_t krow = krow_n;
                float oth[NDL];
#pragma unroll
                for (int j = 0; j < NDL; ++j) oth[j] = oth_n[j];
                const int nx = base + min(kj + 1, n - 1);
                krow_n = __ldg(n2n + nx);
                ld.load(n_coords + (int64_t)nx * D, oth_n);
                const float kc = ldf(k + krow * HC + hc), vc = ldf(v + krow * HC + hc);
                int mine[NDL];
                float bq, bk, bv;
                pair_tables<T, HD, D, true>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
                const float s = group_sum<HD>(qc * (kc + bq) + kc * bk, gmask);
                const float e = group_sum<HD>(gc * (vc + bv - oc), gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
                dqa += ds * (kc + bq);
#pragma unroll
                for (int j = 0; j < NDL; ++j)
                    if (mine_ok[j]) {
                        const int slot = mine[j] + ld.dim[j];
                        ha[slot] += ds;
                        hb[slot] += pr;
                    }
            }
            stf(dq + row * HC + hc, dqa);
            flush_hists<HD, D>(ha, hb, n_slots, meta, dtq, qc, dtv, gc, true, HC, hc, c, gi, gmask);
        }
        // ---- position p as a key -----------------------------------------------------------------
        {
            const float kc = ldf(k + row * HC + hc), vc = ldf(v + row * HC + hc);
            float dka = 0.f, dva = 0.f;
            int64_t qrow_n = __ldg(n2n + base);
            float oth_n[NDL];
            ld.load(n_coords + (int64_t)base * D, oth_n);
            for (int qi = 0; qi < n; ++qi) {
                const int64_t qrow = qrow_n;
                float oth[NDL];
#pragma unroll
                for (int j = 0; j < NDL; ++j) oth[j] = oth_n[j];
                const int nx = base + min(qi + 1, n - 1);
                qrow_n = __ldg(n2n + nx);
                ld.load(n_coords + (int64_t)nx * D, oth_n);
                const float qc = ldf(q + qrow * HC + hc), gc = ldf(dout + qrow * HC + hc);
                const float oc = ldf(o + qrow * HC + hc);
                const float L = __ldg(lse + qrow * H + h);
                int mine[NDL];
                float bq, bk, bv;
                pair_tables<T, HD, D, false>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
                const float s = group_sum<HD>(qc * (kc + bq) + kc * bk, gmask);
                const float e = group_sum<HD>(gc * (vc + bv - oc), gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
                dka += ds * (qc + bk);
                dva += pr * gc;
#pragma unroll
                for (int j = 0; j < NDL; ++j)
                    if (mine_ok[j]) ha[mine[j] + ld.dim[j]] += ds;
            }
            stf(dk + row * HC + hc, dka);
            stf(dv + row * HC + hc, dva);
            flush_hists<HD, D>(ha, hb, n_slots, meta, dtk, kc, dtk, 0.f, false, HC, hc, c, gi, gmask);
        }
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
    const int groups_per_block = 8 * (32 / HD);
    const int slots_padded = (a.meta.R + D + 31) / 32 * 32;
    const size_t smem = (size_t)groups_per_block * 2 * slots_padded * sizeof(float);
    if (smem > 227 * 1024) return S3D_ERR_UNSUPPORTED;
    auto kern = attn_bwd_scalar_kernel<T, HD, D>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    int64_t blocks = (a.N * a.H + groups_per_block - 1) / groups_per_block;
    const int64_t cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    kern<<<(unsigned)blocks, 256, smem, st>>>((const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq,
                                  (const T *)a.tk, (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n,
                                  a.n_coords, a.N, a.W, a.H, slots_padded, (const T *)a.out, a.lse,
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
