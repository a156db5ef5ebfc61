// Generic ("scalar") cRSE window-attention kernels: any window size, head_dim 8/16/32,
// 3/6/9 signal dimensions, fp32 or fp16 storage with fp32 arithmetic throughout.
//
// Semantics follow the reference kernels of microsoft/Swin3D
// (Swin3D/src/attn/self_attn_aio_fwd.cu:16-52,111-188, self_attn_aio_bwd.cu:14-113):
//   s_qk = sum_c ( q_c k_c + q_c * sum_n Tq[n,idx_n,h,c] + k_c * sum_n Tk[n,idx_n,h,c] )
//   out_q = sum_k softmax_k(s_qk) * ( v_k + sum_n Tv[n,idx_n,h,:] )
// but the structure is different: a group of head_dim / VEC lanes (VEC consecutive channels per
// lane) owns one (voxel, head) row, so rows of q, k, v and of the tables are read as coalesced pieces; the
// softmax is online, outputs are written once (no atomics), and the backward sums the scalar
// weights of every looked-up table row in per-group histograms and touches the global table
// gradient once per (voxel, head, touched row).
#include "attn_kernels.cuh"
#include "common.cuh"

namespace s3d {

// VEC consecutive channels of a row as floats (one 4-, 8- or 16-byte access).
template <typename T, int VEC> __device__ __forceinline__ void ldv(const T *p, float (&x)[VEC]);
template <> __device__ __forceinline__ void ldv<float, 1>(const float *p, float (&x)[1]) { x[0] = __ldg(p); }
template <> __device__ __forceinline__ void ldv<float, 2>(const float *p, float (&x)[2])
{
    const float2 a = __ldg(reinterpret_cast<const float2 *>(p));
    x[0] = a.x; x[1] = a.y;
}
template <> __device__ __forceinline__ void ldv<float, 4>(const float *p, float (&x)[4])
{
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
}
template <> __device__ __forceinline__ void ldv<__half, 1>(const __half *p, float (&x)[1]) { x[0] = __half2float(__ldg(p)); }
template <> __device__ __forceinline__ void ldv<__half, 2>(const __half *p, float (&x)[2])
{
    const float2 a = __half22float2(__ldg(reinterpret_cast<const __half2 *>(p)));
    x[0] = a.x; x[1] = a.y;
}
template <> __device__ __forceinline__ void ldv<__half, 4>(const __half *p, float (&x)[4])
{
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
template <typename T, int VEC> __device__ __forceinline__ void stv(T *p, const float (&x)[VEC]);
template <> __device__ __forceinline__ void stv<float, 1>(float *p, const float (&x)[1]) { *p = x[0]; }
template <> __device__ __forceinline__ void stv<float, 2>(float *p, const float (&x)[2])
{
    *reinterpret_cast<float2 *>(p) = make_float2(x[0], x[1]);
}
template <> __device__ __forceinline__ void stv<float, 4>(float *p, const float (&x)[4])
{
    *reinterpret_cast<float4 *>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
template <> __device__ __forceinline__ void stv<__half, 1>(__half *p, const float (&x)[1]) { *p = __float2half_rn(x[0]); }
template <> __device__ __forceinline__ void stv<__half, 2>(__half *p, const float (&x)[2])
{
    *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(x[0], x[1]);
}
template <> __device__ __forceinline__ void stv<__half, 4>(__half *p, const float (&x)[4])
{
    uint2 r;
    *reinterpret_cast<__half2 *>(&r.x) = __floats2half2_rn(x[0], x[1]);
    *reinterpret_cast<__half2 *>(&r.y) = __floats2half2_rn(x[2], x[3]);
    *reinterpret_cast<uint2 *>(p) = r;
}

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

// Sum over the LG lanes of a group (groups are aligned, so xor offsets below LG stay inside).
template <int LG>
__device__ __forceinline__ float group_sum(float x, unsigned gmask)
{
#pragma unroll
    for (int o = LG / 2; o > 0; o >>= 1) x += __shfl_xor_sync(gmask, x, o);
    return x;
}

template <int LG>
__device__ __forceinline__ unsigned group_mask(int gi)
{
    return LG == 32 ? 0xffffffffu : (((1u << (LG & 31)) - 1u) << (gi * LG));
}

// The signal dimensions are dealt to the LG lanes of a group: lane c works out the table row of
// dimensions c, c + LG, ... and the group exchanges the rows by shuffles.
template <int LG, int D>
struct LaneDims {
    static constexpr int NDL = (D + LG - 1) / LG;
    float own[NDL];   // this voxel's coordinate in the lane's dimensions
    int L[NDL], rb[NDL], dim[NDL];
    bool last[NDL], ok[NDL];

    __device__ __forceinline__ void init(const CrseMeta &m, int c)
    {
#pragma unroll
        for (int j = 0; j < NDL; ++j) {
            const int d = c + j * LG;
            ok[j] = d < D;
            dim[j] = ok[j] ? d : 0;
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

// Table rows of a pair and the three sums of this lane's channels over the D looked-up rows.
// oth: the other voxel's coordinate in this lane's dimensions; OWN_IS_QUERY says which side the
// lane's own voxel is on.  mine: the rows of the lane's own dimensions.
template <typename T, int LG, int D, int VEC, bool OWN_IS_QUERY>
__device__ __forceinline__ void pair_tables(const LaneDims<LG, D> &ld, const float (&oth)[LaneDims<LG, D>::NDL],
                                            int gi, unsigned gmask,
                                            const T *__restrict__ tq, const T *__restrict__ tk,
                                            const T *__restrict__ tv, int HC, int hc,
                                            int (&mine)[LaneDims<LG, D>::NDL],
                                            float (&bq)[VEC], float (&bk)[VEC], float (&bv)[VEC])
{
    constexpr int NDL = LaneDims<LG, D>::NDL;
#pragma unroll
    for (int j = 0; j < NDL; ++j)
        mine[j] = ld.rb[j] + (OWN_IS_QUERY ? crse_index(ld.own[j], oth[j], ld.L[j], ld.last[j])
                                           : crse_index(oth[j], ld.own[j], ld.L[j], ld.last[j]));
#pragma unroll
    for (int i = 0; i < VEC; ++i) bq[i] = bk[i] = bv[i] = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const int row = __shfl_sync(gmask, mine[d / LG], gi * LG + d % LG);
        const int64_t off = (int64_t)row * HC + hc;
        float a[VEC], b[VEC], e[VEC];
        ldv<T, VEC>(tq + off, a);
        ldv<T, VEC>(tk + off, b);
        ldv<T, VEC>(tv + off, e);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            bq[i] += a[i];
            bk[i] += b[i];
            bv[i] += e[i];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Forward: a group of LG = HD / VEC lanes (a lane holds VEC consecutive channels) owns one
// (query, head) row and walks the keys of the query's window; every row of q, k, v and of the
// tables is read as one coalesced piece.
template <typename T, int HD, int D, int VEC>
__global__ void __launch_bounds__(256)
attn_fwd_scalar_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                       const T *__restrict__ tq, const T *__restrict__ tk, const T *__restrict__ tv,
                       const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                       const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                       const float *__restrict__ n_coords, int64_t N, int64_t W, int H,
                       T *__restrict__ out, float *__restrict__ lse)
{
    constexpr int LG = HD / VEC, G = 32 / LG;
    constexpr int NDL = LaneDims<LG, D>::NDL;
    const int lane = threadIdx.x & 31, c = lane % LG, gi = lane / LG;
    const unsigned gmask = group_mask<LG>(gi);
    const int HC = H * HD;
    const int64_t group0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G + gi;
    const int64_t ngroups = (int64_t)gridDim.x * (blockDim.x >> 5) * G;
    LaneDims<LG, D> ld;
    ld.init(meta, c);

    // every lane of a warp runs the same number of items so that the warp stays together;
    // groups past the end repeat the last item without storing
    const int64_t items = N * H;
    for (int64_t it0 = group0 - gi; it0 < items; it0 += ngroups) {
        const bool live = it0 + gi < items;
        const int64_t item = live ? it0 + gi : items - 1;
        const int p = (int)(item / H), h = (int)(item - (int64_t)p * H);
        const int64_t w = window_of(w2n, W, p);
        const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
        const int64_t qrow = __ldg(n2n + p);
        const int hc = h * HD + c * VEC;
        float qc[VEC], acc[VEC];
        ldv<T, VEC>(q + qrow * HC + hc, qc);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
        ld.load(n_coords + (int64_t)p * D, ld.own);
        float mx = -INFINITY, l = 0.f;
        // the next key's row number and coordinates are fetched one iteration ahead
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
            float kc[VEC], vc[VEC], bq[VEC], bk[VEC], bv[VEC];
            ldv<T, VEC>(k + krow * HC + hc, kc);
            ldv<T, VEC>(v + krow * HC + hc, vc);
            int mine[NDL];
            pair_tables<T, LG, D, VEC, true>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
            float sp = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) sp += qc[i] * (kc[i] + bq[i]) + kc[i] * bk[i];
            const float s = group_sum<LG>(sp, gmask);
            const float mnew = fmaxf(mx, s);
            const float scale = __expf(mx - mnew);
            const float pr = __expf(s - mnew);
            l = l * scale + pr;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * scale + pr * (vc[i] + bv[i]);
            mx = mnew;
        }
        if (live) {
            const float inv = 1.f / l;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] *= inv;
            stv<T, VEC>(out + qrow * HC + hc, acc);
            if (c == 0) lse[qrow * H + h] = mx + __logf(l);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Backward.  A group of LG = HD / VEC lanes (a lane holds VEC consecutive channels) takes one (position, head) of the window-sorted
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

// Adds hist[slot] * (row vector) to the rows of two global tables for every non-zero slot of the
// group's two histograms, and clears the histograms.
template <int LG, int D, int VEC>
__device__ __forceinline__ void flush_hists(float *ha, float *hb, int n_slots, const CrseMeta &m,
                                            float *__restrict__ ta, const float (&va)[VEC],
                                            float *__restrict__ tb, const float (&vb)[VEC], bool use_b,
                                            int HC, int hc, int c, int gi, unsigned gmask)
{
    __syncwarp(gmask);
    for (int s0 = 0; s0 < n_slots; s0 += LG) {
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
        unsigned nz = __ballot_sync(gmask, a != 0.f || b != 0.f) >> (gi * LG);
        if (LG < 32) nz &= (1u << (LG & 31)) - 1u;
        while (nz) {
            const int j = __ffs(nz) - 1;
            nz &= nz - 1;
            const float aj = __shfl_sync(gmask, a, gi * LG + j);
            const float bj = __shfl_sync(gmask, b, gi * LG + j);
            const int64_t off = (int64_t)flat_row_of_slot<D>(m, s0 + j) * HC + hc;
            if (aj != 0.f) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) atomicAdd(ta + off + i, aj * va[i]);
            }
            if (use_b && bj != 0.f) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) atomicAdd(tb + off + i, bj * vb[i]);
            }
        }
    }
    __syncwarp(gmask);
}

template <typename T, int HD, int D, int VEC>
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
    constexpr int LG = HD / VEC, G = 32 / LG;
    constexpr int NDL = LaneDims<LG, D>::NDL;
    const int lane = threadIdx.x & 31, c = lane % LG, gi = lane / LG;
    const unsigned gmask = group_mask<LG>(gi);
    const int HC = H * HD;
    const int n_slots = meta.R + D;
    for (int i = threadIdx.x; i < (blockDim.x >> 5) * G * 2 * slots_padded; i += blockDim.x) s_hist[i] = 0.f;
    __syncthreads();
    float *ha = s_hist + (size_t)((threadIdx.x >> 5) * G + gi) * 2 * slots_padded;
    float *hb = ha + slots_padded;
    const int64_t group0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * G + gi;
    const int64_t ngroups = (int64_t)gridDim.x * (blockDim.x >> 5) * G;

    LaneDims<LG, D> ld;
    ld.init(meta, c);

    // every lane of a warp runs the same number of items; groups past the end repeat the last item
    // without storing or flushing
    const int64_t items = N * H;
    for (int64_t it0 = group0 - gi; it0 < items; it0 += ngroups) {
        const bool live = it0 + gi < items;
        const int64_t item = live ? it0 + gi : items - 1;
        const int p = (int)(item / H), h = (int)(item - (int64_t)p * H);
        const int hc = h * HD + c * VEC;
        const int64_t w = window_of(w2n, W, p);
        const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
        const int64_t row = __ldg(n2n + p);
        ld.load(n_coords + (int64_t)p * D, ld.own);
        // ---- position p as a query ---------------------------------------------------------------
        {
            float qc[VEC], gc[VEC], oc[VEC], dqa[VEC];
            ldv<T, VEC>(q + row * HC + hc, qc);
            ldv<T, VEC>(dout + row * HC + hc, gc);
            ldv<T, VEC>(o + row * HC + hc, oc);
#pragma unroll
            for (int i = 0; i < VEC; ++i) dqa[i] = 0.f;
            const float L = __ldg(lse + row * H + h);
            int64_t krow_n = __ldg(n2n + base);
            float oth_n[NDL];
            ld.load(n_coords + (int64_t)base * D, oth_n);
#pragma unroll(HD == 8 ? 2 : 1)
            for (int kj = 0; kj < n; ++kj) {
                const int64_t krow = krow_n;
                float oth[NDL];
#pragma unroll
                for (int j = 0; j < NDL; ++j) oth[j] = oth_n[j];
                const int nx = base + min(kj + 1, n - 1);
                krow_n = __ldg(n2n + nx);
                ld.load(n_coords + (int64_t)nx * D, oth_n);
                float kc[VEC], vc[VEC], bq[VEC], bk[VEC], bv[VEC];
                ldv<T, VEC>(k + krow * HC + hc, kc);
                ldv<T, VEC>(v + krow * HC + hc, vc);
                int mine[NDL];
                pair_tables<T, LG, D, VEC, true>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
                float sp = 0.f, ep = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    sp += qc[i] * (kc[i] + bq[i]) + kc[i] * bk[i];
                    ep += gc[i] * (vc[i] + bv[i] - oc[i]);
                }
                const float s = group_sum<LG>(sp, gmask);
                const float e = group_sum<LG>(ep, gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
#pragma unroll
                for (int i = 0; i < VEC; ++i) dqa[i] += ds * (kc[i] + bq[i]);
#pragma unroll
                for (int j = 0; j < NDL; ++j)
                    if (ld.ok[j]) {
                        const int slot = mine[j] + ld.dim[j];
                        ha[slot] += ds;
                        hb[slot] += pr;
                    }
            }
            if (live) stv<T, VEC>(dq + row * HC + hc, dqa);
            if (!live) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) qc[i] = gc[i] = 0.f;   // the repeated item adds zeros
            }
            flush_hists<LG, D, VEC>(ha, hb, n_slots, meta, dtq, qc, dtv, gc, true, HC, hc, c, gi, gmask);
        }
        // ---- position p as a key -----------------------------------------------------------------
        {
            float kc[VEC], vc[VEC], dka[VEC], dva[VEC];
            ldv<T, VEC>(k + row * HC + hc, kc);
            ldv<T, VEC>(v + row * HC + hc, vc);
#pragma unroll
            for (int i = 0; i < VEC; ++i) dka[i] = dva[i] = 0.f;
            int64_t qrow_n = __ldg(n2n + base);
            float oth_n[NDL];
            ld.load(n_coords + (int64_t)base * D, oth_n);
#pragma unroll(HD == 8 ? 2 : 1)
            for (int qi = 0; qi < n; ++qi) {
                const int64_t qrow = qrow_n;
                float oth[NDL];
#pragma unroll
                for (int j = 0; j < NDL; ++j) oth[j] = oth_n[j];
                const int nx = base + min(qi + 1, n - 1);
                qrow_n = __ldg(n2n + nx);
                ld.load(n_coords + (int64_t)nx * D, oth_n);
                float qc[VEC], gc[VEC], oc[VEC], bq[VEC], bk[VEC], bv[VEC];
                ldv<T, VEC>(q + qrow * HC + hc, qc);
                ldv<T, VEC>(dout + qrow * HC + hc, gc);
                ldv<T, VEC>(o + qrow * HC + hc, oc);
                const float L = __ldg(lse + qrow * H + h);
                int mine[NDL];
                pair_tables<T, LG, D, VEC, false>(ld, oth, gi, gmask, tq, tk, tv, HC, hc, mine, bq, bk, bv);
                float sp = 0.f, ep = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    sp += qc[i] * (kc[i] + bq[i]) + kc[i] * bk[i];
                    ep += gc[i] * (vc[i] + bv[i] - oc[i]);
                }
                const float s = group_sum<LG>(sp, gmask);
                const float e = group_sum<LG>(ep, gmask);
                const float pr = __expf(s - L);
                const float ds = pr * e;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    dka[i] += ds * (qc[i] + bk[i]);
                    dva[i] += pr * gc[i];
                }
#pragma unroll
                for (int j = 0; j < NDL; ++j)
                    if (ld.ok[j]) ha[mine[j] + ld.dim[j]] += ds;
            }
            if (live) {
                stv<T, VEC>(dk + row * HC + hc, dka);
                stv<T, VEC>(dv + row * HC + hc, dva);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) kc[i] = 0.f;
            }
            flush_hists<LG, D, VEC>(ha, hb, n_slots, meta, dtk, kc, dtk, kc, false, HC, hc, c, gi, gmask);
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
// Channels per lane, from measurements on a B200 (fp32, 9 signal dimensions): the forward is
// fastest with groups of 2 (head_dim 8) or 8 lanes (head_dim 16 and 32); the backward, whose
// histogram flush walks the table rows LG at a time, with groups of 8 or 16 lanes.
template <int HD> struct ScalarVec;
template <> struct ScalarVec<8> { static constexpr int FWD = 4, BWD = 1; };
template <> struct ScalarVec<16> { static constexpr int FWD = 2, BWD = 1; };
template <> struct ScalarVec<32> { static constexpr int FWD = 4, BWD = 4; };

template <typename T, int HD, int D, int VEC>
static int launch_fwd_v(const AttnArgs &a, cudaStream_t st)
{
    const int groups_per_block = 8 * (32 / (HD / VEC));
    int64_t blocks = (a.N * a.H + groups_per_block - 1) / groups_per_block;
    const int64_t cap = 148 * 64;
    if (blocks > cap) blocks = cap;
    attn_fwd_scalar_kernel<T, HD, D, VEC><<<(unsigned)blocks, 256, 0, st>>>(
        (const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq, (const T *)a.tk,
        (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n, a.n_coords, a.N, a.W, a.H, (T *)a.out, a.lse);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <typename T, int HD, int D>
static int launch_fwd(const AttnArgs &a, cudaStream_t st)
{
    if (a.W == 0 || a.N == 0) return S3D_OK;
    return launch_fwd_v<T, HD, D, ScalarVec<HD>::FWD>(a, st);
}

template <typename T, int HD, int D, int VEC>
static int launch_bwd_v(const AttnArgs &a, cudaStream_t st)
{
    constexpr int G = 32 / (HD / VEC);
    const int slots_padded = (a.meta.R + D + 31) / 32 * 32;
    const size_t per_group = (size_t)2 * slots_padded * sizeof(float);
    // as many warps per block (at most 8) as keep the histograms of a block near 100 KB
    int warps = (int)((100 * 1024) / (per_group * G));
    if (warps > 8) warps = 8;
    if (warps < 1) warps = 1;
    const size_t smem = per_group * G * warps;
    if (smem > 227 * 1024) return S3D_ERR_UNSUPPORTED;
    auto kern = attn_bwd_scalar_kernel<T, HD, D, VEC>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    const int groups_per_block = warps * G;
    int64_t blocks = (a.N * a.H + groups_per_block - 1) / groups_per_block;
    const int64_t cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    kern<<<(unsigned)blocks, warps * 32, smem, st>>>((const T *)a.q, (const T *)a.k, (const T *)a.v, (const T *)a.tq,
                                  (const T *)a.tk, (const T *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n,
                                  a.n_coords, a.N, a.W, a.H, slots_padded, (const T *)a.out, a.lse,
                                  (const T *)a.dout, (T *)a.dq, (T *)a.dk, (T *)a.dv, a.dtq, a.dtk,
                                  a.dtv);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <typename T, int HD, int D>
static int launch_bwd(const AttnArgs &a, cudaStream_t st)
{
    if (a.W == 0 || a.N == 0) return S3D_OK;
    return launch_bwd_v<T, HD, D, ScalarVec<HD>::BWD>(a, st);
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
