// Forward of the cRSE window attention for windows of at most 32 voxels, tensor-core path (fp16).
//
// The whole window is one 32 x 32 tile, so the softmax needs no running maximum across key tiles
// and nothing is ever rescaled: scores of all pairs first (lanes = queries, four keys per warp),
// exact row maxima through shared-memory atomics, then probabilities, histogram and P.V.
// The histogram reuses the shared memory of the P_q projection, which is dead once the scores
// exist; 105 KB of shared memory per block, two blocks of 8 warps per SM.
// Pair array: [key][query] 16-byte entries, row stride 33 (see attn_tc_small.cuh):
//   after the S0 GEMM   (q.k head 0, q.k head 1, -, -)              fp32
//   after the scores     (s head 0, s head 1, packed indices 0, 1)
//   after the softmax    (p half2, -, packed indices 0, 1)
// grid = (x, H/2) (head_dim 8) or (x, H) (head_dim 16).  Larger windows: attn_tc_fwd.cu.
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"

namespace s3d {
namespace tc {

constexpr int FS_NWARP = 8;
constexpr int FS_THREADS = FS_NWARP * 32;

struct FwdSmallSmem {
    int R16, Rp;
    int off_pq, off_pk, off_e, off_rows, off_c, off_misc, total;
};

__host__ __device__ inline FwdSmallSmem make_fwd_small_layout(int R)
{
    FwdSmallSmem L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    int off = 0;
    L.off_pq = off; off += L.R16 * QT * 4;                                   // P_q, later the histogram
    const int pk = 32 * L.Rp * 4;
    L.off_pk = off; off += pk > 18432 ? pk : 18432;                          // P_k, later the reduction buffer
    L.off_e = off; off += 32 * ES * 16;
    L.off_rows = off; off += 3 * 32 * 16 * 2;                                // Q, K, V rows
    L.off_c = off; off += 32 * 12 * 4;
    L.off_misc = off; off += 1024;
    L.total = off;
    return L;
}

struct FwdSmallParams {
    const __half *q, *k, *v, *tq, *tk, *tv;
    __half *out;
    float *lse;
    const int32_t *w_sizes, *w2n, *n2n;
    const float *n_coords;
    int64_t W;
    int H;
};

template <int D, int NPU /*projection units per warp*/, int NHU /*hist.T units per warp*/, bool HD16>
__global__ void __launch_bounds__(FS_THREADS, 2)
attn_fwd_small_kernel(const FwdSmallParams P, const CrseMeta meta)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const FwdSmallSmem L = make_fwd_small_layout(meta.R);
    uint32_t *s_pq = reinterpret_cast<uint32_t *>(smem + L.off_pq);
    uint32_t *s_hist = s_pq;
    uint32_t *s_pk = reinterpret_cast<uint32_t *>(smem + L.off_pk);
    uint4 *s_e = reinterpret_cast<uint4 *>(smem + L.off_e);
    __half *s_q = reinterpret_cast<__half *>(smem + L.off_rows);
    __half *s_k = s_q + 512, *s_v = s_q + 1024;
    float *s_c = reinterpret_cast<float *>(smem + L.off_c);
    float *s_max = reinterpret_cast<float *>(smem + L.off_misc);     // [32][2]
    int *s_row = reinterpret_cast<int *>(s_max + 64);                // [32]
    float *s_red = reinterpret_cast<float *>(smem + L.off_pk);       // [8][32][16], P_k is dead by then
    float *s_lsum = s_red + FS_NWARP * 512;                          // [8][32][2]

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int hp = blockIdx.y, H = P.H;
    const int HC = H * (HD16 ? 16 : 8), co = hp * 16;
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // projection units u = wid + 8 i : table = u / n_mt (0: Tq with Q, 1: Tk with K), tile = u % n_mt
    uint32_t ta[NPU][2][2];
#pragma unroll
    for (int i = 0; i < NPU; ++i) {
        const int u = wid + FS_NWARP * i;
        const int tab = u / n_mt, mt = u - tab * n_mt;
        const __half *T = tab == 0 ? P.tq : P.tk;
        const int r0 = table_row(meta, mt * 16 + g), r1 = table_row(meta, mt * 16 + g + 8);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            ta[i][h][0] = (tab < 2 && r0 >= 0) ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r0 * HC + co + h * 8 + 2 * t) : 0u;
            ta[i][h][1] = (tab < 2 && r1 >= 0) ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r1 * HC + co + h * 8 + 2 * t) : 0u;
        }
    }
    // hist.Tv units: k-step = wid + 8 i
    uint32_t tb[NHU][2][2];
#pragma unroll
    for (int i = 0; i < NHU; ++i) {
        const int ks = wid + FS_NWARP * i;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int ra = table_row(meta, ks * 16 + ht_krow(t, half, 0)), rb = table_row(meta, ks * 16 + ht_krow(t, half, 1));
                const __half lo = ra >= 0 ? P.tv[(int64_t)ra * HC + co + h * 8 + g] : __float2half(0.f);
                const __half hi = rb >= 0 ? P.tv[(int64_t)rb * HC + co + h * 8 + g] : __float2half(0.f);
                tb[i][h][half] = h2_as_u32(__halves2half2(lo, hi));
            }
    }

    for (int64_t w = blockIdx.x; w < P.W; w += gridDim.x) {
        const int n = __ldg(P.w_sizes + w);
        if (n > QT) continue;                       // larger windows: tiled kernel
        const int base = __ldg(P.w2n + w);
        __syncthreads();
        // ---- stage the window ---------------------------------------------------------------------
        float cx[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            cx[d] = lane < n ? __ldg(P.n_coords + (int64_t)(base + lane) * D + d) : 0.f;
            if (wid == 0) s_c[lane * 12 + d] = cx[d];
        }
        if (tid < 192) {
            const int i = tid / 6, r = tid - 6 * i, arr = r >> 1, hf = r & 1;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (i < n) {
                const int row = __ldg(P.n2n + base + i);
                if (r == 0) s_row[i] = row;
                const __half *src = arr == 0 ? P.q : (arr == 1 ? P.k : P.v);
                val = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)row * HC + co + hf * 8));
            }
            *reinterpret_cast<uint4 *>(s_q + arr * 512 + i * 16 + hf * 8) = val;
        } else {
            s_max[tid - 192] = -INFINITY;
        }
        __syncthreads();
        // ---- projections P_q (lane-major), P_k (tile-major); S0 = K.Q^T -------------------------------
#pragma unroll
        for (int i = 0; i < NPU; ++i) {
            const int u = wid + FS_NWARP * i;
            const int tab = u / n_mt, mt = u - tab * n_mt;
            if (tab == 0) project_unit<true>(ta[i], s_q, s_pq, mt, Rp, n, g, t);
            else if (tab == 1) project_unit<false>(ta[i], s_k, s_pk, mt, Rp, n, g, t);
        }
#pragma unroll
        for (int uu = 0; uu < 2; ++uu) {
            const int u = wid + FS_NWARP * uu, mt = u >> 3, j = u & 7;   // key rows 16mt.., query columns 4j..
            if (16 * mt < n && 4 * j < n) {
                const __half *ysrc = s_k + mt * 256;
                const uint32_t wv = *reinterpret_cast<const uint32_t *>(s_q + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 2 * t);
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 2 * t);
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 8 + 2 * t);
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 8 + 2 * t);
                float c[4];
                mma_k16_z(c, a0, a1, a2, a3, (g & 1) ? 0u : wv, (g & 1) ? wv : 0u);
                *reinterpret_cast<float2 *>(s_e + (16 * mt + g) * ES + 4 * j + t) = make_float2(c[0], c[1]);
                *reinterpret_cast<float2 *>(s_e + (16 * mt + g + 8) * ES + 4 * j + t) = make_float2(c[2], c[3]);
            }
        }
        __syncthreads();
        // ---- phase 1: keys wid, wid+8, wid+16, wid+24 ; lane = query: indices, 2*D look-ups, score ------
        float mloc0 = -INFINITY, mloc1 = -INFINITY;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = wid + FS_NWARP * k4;
            if (kk < n) {
                __half2 bq = __float2half2_rn(0.f), bk = bq;
                uint32_t w0 = 0, w1 = 0;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int idx = crse_index_fast(cx[d], s_c[kk * 12 + d], meta.L[d], d == D - 1);
                    const int row = meta.rowbase[d] + idx;
                    bq = __hadd2(bq, u32_as_h2(s_pq[row * QT + mypos]));
                    bk = __hadd2(bk, u32_as_h2(s_pk[kk * Rp + row]));
                    if (d < 5) w0 |= (uint32_t)idx << (IDX_BITS * d);
                    else w1 |= (uint32_t)idx << (IDX_BITS * (d - 5));
                }
                const float2 s0 = *reinterpret_cast<const float2 *>(s_e + kk * ES + lane);
                const float2 b = __half22float2(__hadd2(bq, bk));
                float sx = s0.x + b.x, sy = s0.y + b.y;
                if (HD16) sx = sy = sx + sy;          // one head: both halves carry the full score
                s_e[kk * ES + lane] = make_uint4(__float_as_uint(sx), __float_as_uint(sy), w0, w1);
                mloc0 = fmaxf(mloc0, sx);
                mloc1 = fmaxf(mloc1, sy);
            }
        }
        if (wid < n) {
            atomic_max_float(s_max + lane * 2, mloc0);
            atomic_max_float(s_max + lane * 2 + 1, mloc1);
        }
        __syncthreads();
        // ---- phase 1.5: probabilities; clear the histogram (the P_q storage) -------------------------------
        const float m0 = s_max[lane * 2], m1 = s_max[lane * 2 + 1];
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = wid + FS_NWARP * k4;
            uint32_t *e = reinterpret_cast<uint32_t *>(s_e + kk * ES + lane);
            uint32_t ph = 0u;
            if (kk < n) {
                const float p0 = exp2f((__uint_as_float(e[0]) - m0) * LOG2E);
                const float p1 = exp2f((__uint_as_float(e[1]) - m1) * LOG2E);
                l0 += p0;
                l1 += p1;
                ph = h2_as_u32(__floats2half2_rn(p0, p1));
            }
            e[0] = ph;      // zero for keys beyond the window: the P.V GEMM reads whole 16-key steps
        }
        for (int i = tid; i < L.R16 * QT / 4; i += FS_THREADS)
            reinterpret_cast<uint4 *>(s_hist)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        // ---- phase 2: histogram (a warp owns one or two signal dimensions) | warp 7: O = P.V -------------
        {
            int dA = -1, dB = -1;
            if (D <= FS_NWARP - 1) {
                if (wid < D) dA = wid;
            } else if (wid < D - 5) {
                dA = wid; dB = wid + 5;
            } else if (wid < 5) {
                dA = wid;
            }
            if (dA >= 0) {
                const int shA = IDX_BITS * (dA % 5), rbA = meta.rowbase[dA];
                const int shB = dB >= 0 ? IDX_BITS * (dB % 5) : 0, rbB = dB >= 0 ? meta.rowbase[dB] : 0;
                uint32_t *cell = s_hist + mypos;
                for (int kk0 = 0; kk0 < n; kk0 += 4) {
                    uint32_t pv[1][4];
                    int off2[2][4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool ok = kk0 + j < n;
                        const uint4 e = s_e[min(kk0 + j, QT - 1) * ES + lane];
                        pv[0][j] = ok ? e.x : 0u;
                        const int ia = ok ? ((dA < 5 ? e.z : e.w) >> shA) & ((1 << IDX_BITS) - 1) : 0;
                        const int ib = (ok && dB >= 0) ? ((dB < 5 ? e.z : e.w) >> shB) & ((1 << IDX_BITS) - 1) : 0;
                        off2[0][j] = (rbA + ia) * QT;
                        off2[1][j] = (rbB + ib) * QT;
                    }
                    if (dB >= 0) {
                        hist_add4<2, 1>(cell, 0, off2, pv, n - kk0);
                    } else {
                        int off1[1][4] = {{off2[0][0], off2[0][1], off2[0][2], off2[0][3]}};
                        hist_add4<1, 1>(cell, 0, off1, pv, n - kk0);
                    }
                }
            }
        }
        float part[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 2; ++i) part[h][i][0] = part[h][i][1] = part[h][i][2] = part[h][i][3] = 0.f;
        if (wid == FS_NWARP - 1) pair_gemm<0, false>(part, s_e, s_v, n, g, t);     // O[q] = sum_k p V[k]
        __syncthreads();
        // ---- O += hist . Tv (rows split over the warps), reduce, normalise, store --------------------------
#pragma unroll
        for (int i = 0; i < NHU; ++i) {
            const int ks = wid + FS_NWARP * i;
            if (ks < n_mt) ht_unit(part, s_hist, tb[i], ks, g, t);
        }
        store_part(s_red + wid * 512, part, g, t);       // P_k (aliased by s_red) is dead since phase 1
        s_lsum[(wid * QT + lane) * 2] = l0;
        s_lsum[(wid * QT + lane) * 2 + 1] = l1;
        __syncthreads();
        {
            const int qq = tid >> 3, ch = (tid & 7) * 2, h = ch >> 3;
            if (qq < n) {
                float a = 0.f, b = 0.f, ls = 0.f;
#pragma unroll
                for (int ww = 0; ww < FS_NWARP; ++ww) {
                    const float2 pr = *reinterpret_cast<const float2 *>(s_red + ww * 512 + qq * 16 + ch);
                    a += pr.x;
                    b += pr.y;
                    ls += s_lsum[(ww * QT + qq) * 2 + h];
                }
                const float inv = 1.f / ls;
                const int64_t row = s_row[qq];
                *reinterpret_cast<__half2 *>(P.out + row * HC + co + ch) = __floats2half2_rn(a * inv, b * inv);
                if (HD16) {
                    if (ch == 0) P.lse[row * H + hp] = s_max[qq * 2] + __logf(ls);
                } else if ((ch & 7) == 0) {
                    P.lse[row * H + 2 * hp + h] = s_max[qq * 2 + h] + __logf(ls);
                }
            }
        }
    }  // windows
}

template <int D, int NPU, int NHU, bool HD16>
static int launch_fwd_small(const FwdSmallParams &p, const CrseMeta &meta, cudaStream_t st)
{
    const FwdSmallSmem L = make_fwd_small_layout(meta.R);
    auto kern = attn_fwd_small_kernel<D, NPU, NHU, HD16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    int dev = 0, sms = 148, per_sm = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, FS_THREADS, L.total) != cudaSuccess || per_sm < 1)
        return S3D_ERR_LAUNCH;
    const int hp = HD16 ? p.H : p.H / 2;
    int gx = sms * per_sm / hp;
    if (gx > p.W) gx = (int)p.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, FS_THREADS, L.total, st>>>(p, meta);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

}  // namespace tc

bool attn_tc_fwd_small_supported(const AttnArgs &a)
{
    if (a.dtype != S3D_F16) return false;
    if (!(a.hd == 16 || (a.hd == 8 && !(a.H & 1)))) return false;
    const int Rint = a.meta.R + a.meta.D - 1;
    const int n_mt = (Rint + 15) / 16;
    if (2 * n_mt > 6 * tc::FS_NWARP) return false;
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;
    return tc::make_fwd_small_layout(Rint).total <= 227 * 1024;
}

// Windows of at most 32 voxels only; the others are left untouched.
int attn_tc_forward_small(const AttnArgs &a0, cudaStream_t st)
{
    if (a0.W == 0) return S3D_OK;
    AttnArgs a = a0;
    a.meta = tc::internal_meta(a0.meta);
    tc::FwdSmallParams p{};
    p.q = (const __half *)a.q; p.k = (const __half *)a.k; p.v = (const __half *)a.v;
    p.tq = (const __half *)a.tq; p.tk = (const __half *)a.tk; p.tv = (const __half *)a.tv;
    p.out = (__half *)a.out; p.lse = a.lse;
    p.w_sizes = a.w_sizes; p.w2n = a.w2n; p.n2n = a.n2n; p.n_coords = a.n_coords;
    p.W = a.W; p.H = a.H;
    const int n_mt = (a.meta.R + 15) / 16;
    const int npu = (2 * n_mt + tc::FS_NWARP - 1) / tc::FS_NWARP;   // <= 6
    const int nhu = (n_mt + tc::FS_NWARP - 1) / tc::FS_NWARP;       // <= 3
#define S3D_FS(DD, HH)                                                                        \
    if (npu <= 2 && nhu <= 1) return tc::launch_fwd_small<DD, 2, 1, HH>(p, a.meta, st);       \
    if (npu <= 4 && nhu <= 2) return tc::launch_fwd_small<DD, 4, 2, HH>(p, a.meta, st);       \
    return tc::launch_fwd_small<DD, 6, 3, HH>(p, a.meta, st);
#define S3D_FS_D(DD) if (a.hd == 16) { S3D_FS(DD, true) } else { S3D_FS(DD, false) }
    switch (a.meta.D) {
        case 3: S3D_FS_D(3)
        case 6: S3D_FS_D(6)
        case 9: S3D_FS_D(9)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_FS_D
#undef S3D_FS
}

}  // namespace s3d
