// Warp-level GEMM building blocks: one projection unit and the pair-array GEMMs of the single-tile
// (window of at most 32 voxels) kernels, one table-gradient unit and one hist.T unit for all kernels.
#pragma once
#include "attn_tc.cuh"

namespace s3d {
namespace tc {

constexpr int ES = 33;   // entry-row stride of the [32][ES] pair array (16-byte entries)

// One (table, 16-row tile) projection unit:  P^T[rows][(voxel, head)] = T . F^T  for the 32 voxels of
// the window, written lane-major ([row][qpos(voxel)]) or tile-major ([voxel][Rp]).
template <bool LANE_MAJOR>
__device__ __forceinline__ void project_unit(const uint32_t (&ta)[2][2], const __half *feat, uint32_t *dst,
                                             int mt, int Rp, int nvalid, int g, int t)
{
    uint32_t d0[8], d1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (4 * j < nvalid) {
            const uint32_t wv = *reinterpret_cast<const uint32_t *>(feat + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
            mma_k16_h(d0[j], d1[j], ta[0][0], ta[0][1], ta[1][0], ta[1][1], (g & 1) ? 0u : wv, (g & 1) ? wv : 0u);
        } else {
            d0[j] = 0u;
            d1[j] = 0u;
        }
    }
    if (LANE_MAJOR) {
        // 16-byte stores go out a quarter warp (rows g, g+1 ; t = 0..3) at a time: odd rows write their
        // upper half first so that the eight lanes of a quarter cover all 32 banks.
        uint32_t *r0 = dst + (mt * 16 + g) * QT + 4 * t;
        const bool od = g & 1;
        const int o0 = od ? 16 : 0, o1 = 16 - o0;
        const uint4 a0 = make_uint4(d0[0], d0[2], d0[4], d0[6]), a1 = make_uint4(d0[1], d0[3], d0[5], d0[7]);
        const uint4 b0 = make_uint4(d1[0], d1[2], d1[4], d1[6]), b1 = make_uint4(d1[1], d1[3], d1[5], d1[7]);
        *reinterpret_cast<uint4 *>(r0 + o0) = od ? a1 : a0;
        *reinterpret_cast<uint4 *>(r0 + o1) = od ? a0 : a1;
        *reinterpret_cast<uint4 *>(r0 + 8 * QT + o0) = od ? b1 : b0;
        *reinterpret_cast<uint4 *>(r0 + 8 * QT + o1) = od ? b0 : b1;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (4 * j < nvalid) {
                uint32_t *p = dst + (4 * j + t) * Rp + mt * 16 + g;
                p[0] = d0[j];
                p[8] = d1[j];
            }
    }
}

// Block-diagonal B fragments of a staged feature array ([32 voxels][16 halves] = two slots of 8
// channels) for the both-slots-in-one-instruction projections: n-tile j covers voxels 4j..4j+3.
// They depend on the window only, so a warp loads them once and uses them for all its units.
__device__ __forceinline__ void load_feat_bfrag(uint32_t (&bf)[8][2], const __half *feat, int nvalid, int g, int t)
{
    const bool od = g & 1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t wv = 4 * j < nvalid
            ? *reinterpret_cast<const uint32_t *>(feat + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t) : 0u;
        bf[j][0] = od ? 0u : wv;
        bf[j][1] = od ? wv : 0u;
    }
}

// project_unit with the B fragments supplied by the caller.
template <bool LANE_MAJOR>
__device__ __forceinline__ void project_unit_b(const uint32_t (&ta)[2][2], const uint32_t (&bf)[8][2], uint32_t *dst,
                                               int mt, int Rp, int nvalid, int g, int t)
{
    uint32_t d0[8], d1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (4 * j < nvalid) {
            mma_k16_h(d0[j], d1[j], ta[0][0], ta[0][1], ta[1][0], ta[1][1], bf[j][0], bf[j][1]);
        } else {
            d0[j] = 0u;
            d1[j] = 0u;
        }
    }
    if (LANE_MAJOR) {
        uint32_t *r0 = dst + (mt * 16 + g) * QT + 4 * t;
        const bool od = g & 1;
        const int o0 = od ? 16 : 0, o1 = 16 - o0;
        const uint4 a0 = make_uint4(d0[0], d0[2], d0[4], d0[6]), a1 = make_uint4(d0[1], d0[3], d0[5], d0[7]);
        const uint4 b0 = make_uint4(d1[0], d1[2], d1[4], d1[6]), b1 = make_uint4(d1[1], d1[3], d1[5], d1[7]);
        *reinterpret_cast<uint4 *>(r0 + o0) = od ? a1 : a0;
        *reinterpret_cast<uint4 *>(r0 + o1) = od ? a0 : a1;
        *reinterpret_cast<uint4 *>(r0 + 8 * QT + o0) = od ? b1 : b0;
        *reinterpret_cast<uint4 *>(r0 + 8 * QT + o1) = od ? b0 : b1;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (4 * j < nvalid) {
                uint32_t *p = dst + (4 * j + t) * Rp + mt * 16 + g;
                p[0] = d0[j];
                p[8] = d1[j];
            }
    }
}

// acc[head][m-tile] += A . B with A[m][kk] = field FIELD (0 = p, 1 = ds) of the pair entries and
// B[kk][c] = rows[kk][head*8 + c].  TRANSPOSED = false: m = query, kk = key (entry [kk][m]);
// TRANSPOSED = true: m = key, kk = query (entry [m][kk]).
template <int FIELD, bool TRANSPOSED>
__device__ __forceinline__ void pair_gemm(float (&acc)[2][2][4], const uint4 *s_e, const __half *rows, int nk, int g, int t)
{
    const uint32_t *e32 = reinterpret_cast<const uint32_t *>(s_e);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        if (16 * ks < nk) {
            uint32_t fa[2][2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int m = 16 * i + g + 8 * rr, ka = 16 * ks + 2 * t + 8 * kh;
                        const uint32_t u = TRANSPOSED ? e32[(m * ES + ka) * 4 + FIELD] : e32[(ka * ES + m) * 4 + FIELD];
                        const uint32_t w = TRANSPOSED ? e32[(m * ES + ka + 1) * 4 + FIELD] : e32[((ka + 1) * ES + m) * 4 + FIELD];
                        fa[0][i][2 * kh + rr] = pack_lo(u, w);
                        fa[1][i][2 * kh + rr] = pack_hi(u, w);
                    }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t yb[2];
#pragma unroll
                for (int kh = 0; kh < 2; ++kh) {
                    const int ka = 16 * ks + 2 * t + 8 * kh;
                    yb[kh] = h2_as_u32(__halves2half2(rows[ka * 16 + h * 8 + g], rows[(ka + 1) * 16 + h * 8 + g]));
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    mma_k16(acc[h][i], fa[h][i][0], fa[h][i][1], fa[h][i][2], fa[h][i][3], yb[0], yb[1]);
            }
        }
    }
}

// pair_gemm on a [32][ES] plane of 8-byte pair entries (two fields per entry).
template <int FIELD, bool TRANSPOSED>
__device__ __forceinline__ void pair_gemm2(float (&acc)[2][2][4], const uint2 *s_e, const __half *rows, int nk, int g, int t)
{
    const uint32_t *e32 = reinterpret_cast<const uint32_t *>(s_e);
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        if (16 * ks < nk) {
            uint32_t fa[2][2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int m = 16 * i + g + 8 * rr, ka = 16 * ks + 2 * t + 8 * kh;
                        const uint32_t u = TRANSPOSED ? e32[(m * ES + ka) * 2 + FIELD] : e32[(ka * ES + m) * 2 + FIELD];
                        const uint32_t w = TRANSPOSED ? e32[(m * ES + ka + 1) * 2 + FIELD] : e32[((ka + 1) * ES + m) * 2 + FIELD];
                        fa[0][i][2 * kh + rr] = pack_lo(u, w);
                        fa[1][i][2 * kh + rr] = pack_hi(u, w);
                    }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t yb[2];
#pragma unroll
                for (int kh = 0; kh < 2; ++kh) {
                    const int ka = 16 * ks + 2 * t + 8 * kh;
                    yb[kh] = h2_as_u32(__halves2half2(rows[ka * 16 + h * 8 + g], rows[(ka + 1) * 16 + h * 8 + g]));
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    mma_k16(acc[h][i], fa[h][i][0], fa[h][i][1], fa[h][i][2], fa[h][i][3], yb[0], yb[1]);
            }
        }
    }
}

// pair_gemm on a [32][ES] plane of 4-byte entries (one half2 per pair).
template <bool TRANSPOSED>
__device__ __forceinline__ void pair_gemm1(float (&acc)[2][2][4], const uint32_t *e32, const __half *rows, int nk, int g, int t)
{
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        if (16 * ks < nk) {
            uint32_t fa[2][2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int m = 16 * i + g + 8 * rr, ka = 16 * ks + 2 * t + 8 * kh;
                        const uint32_t u = TRANSPOSED ? e32[m * ES + ka] : e32[ka * ES + m];
                        const uint32_t w = TRANSPOSED ? e32[m * ES + ka + 1] : e32[(ka + 1) * ES + m];
                        fa[0][i][2 * kh + rr] = pack_lo(u, w);
                        fa[1][i][2 * kh + rr] = pack_hi(u, w);
                    }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t yb[2];
#pragma unroll
                for (int kh = 0; kh < 2; ++kh) {
                    const int ka = 16 * ks + 2 * t + 8 * kh;
                    yb[kh] = h2_as_u32(__halves2half2(rows[ka * 16 + h * 8 + g], rows[(ka + 1) * 16 + h * 8 + g]));
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    mma_k16(acc[h][i], fa[h][i][0], fa[h][i][1], fa[h][i][2], fa[h][i][3], yb[0], yb[1]);
            }
        }
    }
}

// B fragments (k = voxel, n = channel; [k-step][slot][b0, b1]) of a staged feature array for dt_unit_b.
__device__ __forceinline__ void load_dt_bfrag(uint32_t (&b)[2][2][2], const __half *xrows, int g, int t)
{
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int p0 = 16 * ks + 4 * t + 2 * half, p1 = p0 + 1;   // column -> voxel: (p >> 2) + 8 (p & 3)
                const int xa = (p0 >> 2) + 8 * (p0 & 3), xb = (p1 >> 2) + 8 * (p1 & 3);
                b[ks][h][half] = h2_as_u32(__halves2half2(xrows[xa * 16 + h * 8 + g], xrows[xb * 16 + h * 8 + g]));
            }
}

// dT[rows of tile mt][c] += sum over the 32 voxels of hist[row][voxel] * X[voxel][c]  (both heads).
__device__ __forceinline__ void dt_unit(float (&acc)[2][4], const uint32_t *hist, const __half *xrows, int mt, int g, int t)
{
    // lane (g,t): rows g, g+8 of the tile; columns 16ks+4t .. +3  <->  k = 2t, 2t+1, 2t+8, 2t+9.
    // Odd rows fetch the two k-steps in the opposite order: a quarter warp (rows g, g+1) then covers
    // all 32 banks with each 16-byte load.
    const bool od = g & 1;
    const uint32_t *hu = hist + (mt * 16 + g) * QT + 4 * t, *hw = hu + 8 * QT;
    const uint4 ua = *reinterpret_cast<const uint4 *>(hu + (od ? 16 : 0)), ub = *reinterpret_cast<const uint4 *>(hu + (od ? 0 : 16));
    const uint4 wa = *reinterpret_cast<const uint4 *>(hw + (od ? 16 : 0)), wb = *reinterpret_cast<const uint4 *>(hw + (od ? 0 : 16));
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        const bool first = (ks == 0) != od;
        const uint4 u = first ? ua : ub, w = first ? wa : wb;
        uint32_t b[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int p0 = 16 * ks + 4 * t + 2 * half, p1 = p0 + 1;   // column -> voxel: (p >> 2) + 8 (p & 3)
                const int xa = (p0 >> 2) + 8 * (p0 & 3), xb = (p1 >> 2) + 8 * (p1 & 3);
                b[h][half] = h2_as_u32(__halves2half2(xrows[xa * 16 + h * 8 + g], xrows[xb * 16 + h * 8 + g]));
            }
        mma_k16(acc[0], pack_lo(u.x, u.y), pack_lo(w.x, w.y), pack_lo(u.z, u.w), pack_lo(w.z, w.w), b[0][0], b[0][1]);
        mma_k16(acc[1], pack_hi(u.x, u.y), pack_hi(w.x, w.y), pack_hi(u.z, u.w), pack_hi(w.z, w.w), b[1][0], b[1][1]);
    }
}

// The same with the B fragments (k = voxel, n = channel; [k-step][slot][b0, b1]) supplied by the caller.
__device__ __forceinline__ void dt_unit_b(float (&acc)[2][4], const uint32_t *hist, const uint32_t (&b)[2][2][2], int mt, int g, int t)
{
    const bool od = g & 1;
    const uint32_t *hu = hist + (mt * 16 + g) * QT + 4 * t, *hw = hu + 8 * QT;
    const uint4 ua = *reinterpret_cast<const uint4 *>(hu + (od ? 16 : 0)), ub = *reinterpret_cast<const uint4 *>(hu + (od ? 0 : 16));
    const uint4 wa = *reinterpret_cast<const uint4 *>(hw + (od ? 16 : 0)), wb = *reinterpret_cast<const uint4 *>(hw + (od ? 0 : 16));
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
        const bool first = (ks == 0) != od;
        const uint4 u = first ? ua : ub, w = first ? wa : wb;
        mma_k16(acc[0], pack_lo(u.x, u.y), pack_lo(w.x, w.y), pack_lo(u.z, u.w), pack_lo(w.z, w.w), b[ks][0][0], b[ks][0][1]);
        mma_k16(acc[1], pack_hi(u.x, u.y), pack_hi(w.x, w.y), pack_hi(u.z, u.w), pack_hi(w.z, w.w), b[ks][1][0], b[ks][1][1]);
    }
}

// part[head][m-tile] += hist(16 rows of k-step ks) . T(16 rows)  for the 32 voxels (m) of the window.
// The fragment an mma lane (g,t) needs (four rows, one 16-byte column chunk g) would make the four
// t-lanes of a quarter warp hit the same banks; each lane therefore loads the conflict-free pattern
// (lane L: rows L/8 + 4i, chunk L%8, i.e. four rows x 128 bytes per instruction) and the registers
// are moved to their mma lane with shuffles.
__device__ __forceinline__ void ht_unit(float (&part)[2][2][4], const uint32_t *hist, const uint32_t (&tb)[2][2], int ks, int g, int t)
{
    const int lane = 4 * g + t, src = 8 * t + g;
    const uint32_t *hp = hist + (ks * 16 + (lane >> 3)) * QT + 4 * (lane & 7);
    uint4 y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = *reinterpret_cast<const uint4 *>(hp + 4 * i * QT);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        y[i].x = __shfl_sync(0xffffffffu, y[i].x, src);
        y[i].y = __shfl_sync(0xffffffffu, y[i].y, src);
        y[i].z = __shfl_sync(0xffffffffu, y[i].z, src);
        y[i].w = __shfl_sync(0xffffffffu, y[i].w, src);
    }
    // y[i] = row t + 4i, queries {g, g+8, g+16, g+24}
    mma_k16(part[0][0], pack_lo(y[0].x, y[1].x), pack_lo(y[0].y, y[1].y), pack_lo(y[2].x, y[3].x), pack_lo(y[2].y, y[3].y), tb[0][0], tb[0][1]);
    mma_k16(part[1][0], pack_hi(y[0].x, y[1].x), pack_hi(y[0].y, y[1].y), pack_hi(y[2].x, y[3].x), pack_hi(y[2].y, y[3].y), tb[1][0], tb[1][1]);
    mma_k16(part[0][1], pack_lo(y[0].z, y[1].z), pack_lo(y[0].w, y[1].w), pack_lo(y[2].z, y[3].z), pack_lo(y[2].w, y[3].w), tb[0][0], tb[0][1]);
    mma_k16(part[1][1], pack_hi(y[0].z, y[1].z), pack_hi(y[0].w, y[1].w), pack_hi(y[2].z, y[3].z), pack_hi(y[2].w, y[3].w), tb[1][0], tb[1][1]);
}

__device__ __forceinline__ void store_part(float *red, const float (&part)[2][2][4], int g, int t)
{
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int rr = 0; rr < 2; ++rr)
                *reinterpret_cast<float2 *>(red + (16 * i + g + 8 * rr) * 16 + h * 8 + 2 * t) =
                    make_float2(part[h][i][2 * rr], part[h][i][2 * rr + 1]);
}

}  // namespace tc
}  // namespace s3d
