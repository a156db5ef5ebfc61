// Building blocks of the factorised, tensor-core cRSE window-attention kernels (fp16 storage,
// head_dim 8, two heads per thread block packed as half2).
//
// Factorisation.  With P_q[r] = q . Tq[r] and P_k[r] = k . Tk[r] for every table row r (two small
// GEMMs per window and head), the score of a pair is
//     s_qk = q.k + sum_n P_q[row_n(q,k)] + sum_n P_k[row_n(q,k)]
// i.e. 2*D scalar look-ups instead of 2*D*hd multiply-adds, and the value term becomes
//     sum_k p_qk * sum_n Tv[row_n(q,k)] = hist_q . Tv,   hist_q[r] = sum_k p_qk [row_n(q,k) == r]
// a per-query histogram followed by one more small GEMM.  The GEMMs run on the tensor cores
// (mma.sync m16n8k8 / m16n8k16, fp16 in, fp32 accumulate); the look-ups and histogram updates
// are shared-memory traffic arranged to be bank-conflict free:
//   * per-query arrays (P_q, hist) are laid out [row][32 queries] with the query of lane l stored
//     in column pos(l) = (l%8)*4 + l/8, one 4-byte half2 (head 0, head 1) per entry.  A warp
//     whose lanes are queries therefore always hits 32 different banks whatever rows the lanes
//     select, and a 16-byte load at column 4g returns queries {g, g+8, g+16, g+24}: exactly the
//     rows of the two m16 tiles an mma lane (g, t) needs.
//   * the per-key array P_k is laid out [key][row] with a row stride == 8 (mod 32) words; lanes
//     (queries) read the same key at nearby rows.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "common.cuh"

namespace s3d {
namespace tc {

// A half2 of a result row, to this GPU's array and to the same place of every mirror (peer stores).
__device__ __forceinline__ void store_h2_mirrored(__half *base, const Mirrors &m, int64_t off, __half2 v)
{
    *reinterpret_cast<__half2 *>(base + off) = v;
    for (int i = 0; i < m.n; ++i) *reinterpret_cast<__half2 *>(static_cast<__half *>(m.p[i]) + off) = v;
}

constexpr int QT = 32;        // queries per tile (= lanes)
constexpr int KT = 16;        // keys per tile
constexpr int NWARP = 8;
constexpr int NTHREADS = NWARP * 32;
constexpr int IDX_BITS = 6;   // cRSE indices are packed 5 per 32-bit word, 6 bits each

__device__ __forceinline__ int qpos(int q) { return ((q & 7) << 2) | (q >> 3); }

__device__ __forceinline__ void mma_k8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
}

__device__ __forceinline__ void mma_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Both heads in one instruction: K index = (head, channel) = the 16 contiguous halves of a table or
// feature row, N index = (voxel, head) with a block-diagonal B operand.  fp16 accumulators come out
// as half2 (head 0, head 1) per (row, voxel): exactly the shared-memory entry format, no repacking.
__device__ __forceinline__ void mma_k16_h(uint32_t &d0, uint32_t &d1, uint32_t a0, uint32_t a1,
                                          uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    const uint32_t z = 0u;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8};\n"
                 : "=r"(d0), "=r"(d1)
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

// The same with the accumulators carried in (second plane of a head-dim-16 head pair).
__device__ __forceinline__ void mma_k16_ha(uint32_t &d0, uint32_t &d1, uint32_t a0, uint32_t a1,
                                           uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%0,%1};\n"
                 : "+r"(d0), "+r"(d1)
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same shape, fp32 accumulators, C = 0.
__device__ __forceinline__ void mma_k16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1)
{
    const float z = 0.f;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

// cRSE index with one unsigned clamp: cvt.rzi.u32 maps negatives (and NaN) to 0, so
// min(uint(rel), L) equals (int)fminf(fmaxf(0, rel), L) for every input.
__device__ __forceinline__ int crse_index_fast(float cq, float ck, int L, bool last_dim)
{
    const float rel = __fadd_rn(__fsub_rn(cq, ck), (float)(L / 2));
    const unsigned u = __float2uint_rz(rel);
    return (int)min(u, (unsigned)(last_dim ? L - 1 : L));
}

// The per-dimension constants of the cRSE index in the form the pair loops use them.  Passed as a
// kernel parameter, so that they are constant-bank operands and cost no instruction:
// half = (float)(L / 2), clamp = L (L - 1 for the last dimension, see crse_index in common.cuh).
struct PairConsts {
    float half[S3D_MAX_SIGNAL_DIMS];
    uint32_t clamp[S3D_MAX_SIGNAL_DIMS];
};

__host__ inline PairConsts make_pair_consts(const CrseMeta &m)
{
    PairConsts pc{};
    for (int d = 0; d < m.D; ++d) {
        pc.half[d] = (float)(m.L[d] / 2);
        pc.clamp[d] = (uint32_t)(d == m.D - 1 ? m.L[d] - 1 : m.L[d]);
    }
    return pc;
}

// crse_index_fast with the constants precomputed: same fp32 operations in the same order.
__device__ __forceinline__ uint32_t crse_index_pc(float cq, float ck, float half, uint32_t clamp)
{
    return min(__float2uint_rz(__fadd_rn(__fsub_rn(cq, ck), half)), clamp);
}

// exp2 of a non-positive argument: one MUFU instruction (flushes results below 2^-126 to zero).
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The coordinates of one staged voxel (rows of 12 floats, 16-byte aligned) as three broadcast
// 16-byte loads instead of one 4-byte load per signal dimension.
template <int D>
__device__ __forceinline__ void load_coords12(const float *row, float (&c)[D])
{
    float tmp[12];
    *reinterpret_cast<float4 *>(tmp) = *reinterpret_cast<const float4 *>(row);
    if (D > 4) *reinterpret_cast<float4 *>(tmp + 4) = *reinterpret_cast<const float4 *>(row + 4);
    if (D > 8) *reinterpret_cast<float4 *>(tmp + 8) = *reinterpret_cast<const float4 *>(row + 8);
#pragma unroll
    for (int d = 0; d < D; ++d) c[d] = tmp[d];
}

__device__ __forceinline__ uint32_t pack_lo(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x5410); }
__device__ __forceinline__ uint32_t pack_hi(uint32_t x, uint32_t y) { return __byte_perm(x, y, 0x7632); }

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// Orderable atomic max on a float held in shared memory (initialised to -inf).
__device__ __forceinline__ void atomic_max_float(float *addr, float v)
{
    if (v >= 0.f)
        atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else
        atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// Internal row numbering.  The reference's flat table addressing lets index L of signal dimension n
// fall on row 0 of dimension n+1.  Inside the kernels every dimension but the last therefore owns
// L+1 rows (its own L plus a private alias of the next dimension's row 0), so that the rows of
// different dimensions are disjoint and can be updated by different warps without a race.
// internal_meta() shifts rowbase[n] by n and grows R by D-1; table_row() maps an internal row back
// to the table row it stands for (two internal rows may name the same table row), -1 past the end.
__host__ inline CrseMeta internal_meta(const CrseMeta &m)
{
    CrseMeta r = m;
    for (int d = 0; d < m.D; ++d) r.rowbase[d] = m.rowbase[d] + d;
    r.R = m.R + m.D - 1;
    return r;
}

__device__ __forceinline__ int table_row(const CrseMeta &im, int r)
{
    int n = 0;
#pragma unroll
    for (int d = 1; d < S3D_MAX_SIGNAL_DIMS; ++d) n += (d < im.D && r >= im.rowbase[d]) ? 1 : 0;
    return r < im.R ? r - n : -1;
}

// Row numbering of the single-tile kernels.  Within a window the cRSE indices of a signal dimension
// rarely leave a narrow band around L/2 (voxels of a planar patch share one cell coordinate, colours
// lie in [0,1], normals vary slowly), so a window touches well under half of the table rows.  The
// rows are therefore numbered so that the bands ("centres") of all dimensions come first, followed by
// the remaining rows ("periphery") dimension by dimension; a window then touches few 16-row tiles,
// and every per-tile piece of work (projection, clearing, table-gradient and hist.T products) is
// skipped for tiles outside the index ranges of the window, which the producer warp derives from the
// minima and maxima of the coordinates (the index is monotone in both coordinates).  Skipping is
// exact: a skipped tile is neither written nor read.  As in internal_meta(), index L of a dimension
// but the last is a row of its own (an alias of row 0 of the next dimension).
struct PermMeta {
    int D, R;                                  // R = internal rows
    int n[S3D_MAX_SIGNAL_DIMS];                // index values of the dimension: L + 1 (L for the last)
    int c0[S3D_MAX_SIGNAL_DIMS], c1[S3D_MAX_SIGNAL_DIMS];       // centre = indices [c0, c1)
    int cbase[S3D_MAX_SIGNAL_DIMS], pbase[S3D_MAX_SIGNAL_DIMS]; // first internal row of the centre / periphery
    int tbase[S3D_MAX_SIGNAL_DIMS];            // first table row of the dimension
    int lut_stride;                            // entries per dimension of the index -> row table
};

__host__ inline PermMeta make_perm_meta(const CrseMeta &m)
{
    PermMeta p{};
    p.D = m.D;
    const int quant = m.D >= 6 ? m.L[3] / 8 : 0;             // colour / normal tables have 8 * quant rows
    int rows = 0, mx = 0;
    for (int d = 0; d < m.D; ++d) {
        const int L = m.L[d];
        p.n[d] = d == m.D - 1 ? L : L + 1;
        p.tbase[d] = m.rowbase[d];
        int half = d < 3 ? (quant > 0 ? quant : (L + 9) / 10) : (d >= 6 ? 2 : L / 4);
        if (half < 1) half = 1;
        p.c0[d] = L / 2 - half < 0 ? 0 : L / 2 - half;
        p.c1[d] = d < 3 ? L / 2 + half : L / 2 + half + 1;
        if (p.c1[d] > p.n[d]) p.c1[d] = p.n[d];
        p.cbase[d] = rows;
        rows += p.c1[d] - p.c0[d];
        if (p.n[d] > mx) mx = p.n[d];
    }
    for (int d = 0; d < m.D; ++d) {
        p.pbase[d] = rows;
        rows += p.n[d] - (p.c1[d] - p.c0[d]);
    }
    p.R = rows;
    p.lut_stride = (mx + 7) / 8 * 8;
    return p;
}

// internal row of (dimension, index)
__host__ __device__ __forceinline__ int perm_row(const PermMeta &p, int d, int idx)
{
    if (idx >= p.c0[d] && idx < p.c1[d]) return p.cbase[d] + idx - p.c0[d];
    return p.pbase[d] + (idx < p.c0[d] ? idx : idx - (p.c1[d] - p.c0[d]));
}

// table row an internal row stands for (-1 past the end); an alias row stands for row 0 of the next dimension
__device__ __forceinline__ int perm_table_row(const PermMeta &p, int r)
{
    if (r >= p.R || r < 0) return -1;
    for (int d = 0; d < p.D; ++d) {
        const int nc = p.c1[d] - p.c0[d];
        int idx = -1;
        if (r >= p.cbase[d] && r < p.cbase[d] + nc) idx = p.c0[d] + r - p.cbase[d];
        else if (r >= p.pbase[d] && r < p.pbase[d] + p.n[d] - nc) {
            const int rel = r - p.pbase[d];
            idx = rel < p.c0[d] ? rel : rel + nc;
        }
        if (idx >= 0) return p.tbase[d] + idx;      // idx == L: tbase[d] + L = tbase[d+1], row 0 of the next dimension
    }
    return -1;
}

// index -> internal row table in shared memory: lut[d * lut_stride + idx]
__device__ __forceinline__ void fill_perm_lut(uint16_t *lut, const PermMeta &p, int tid, int nthreads)
{
    for (int i = tid; i < p.D * p.lut_stride; i += nthreads) {
        const int d = i / p.lut_stride, idx = i - d * p.lut_stride;
        lut[i] = (uint16_t)(idx < p.n[d] ? perm_row(p, d, idx) : 0);
    }
}

// Order-preserving integer key of a finite float (for the warp-wide integer min / max reductions).
__device__ __forceinline__ int float_order_key(float x)
{
    const int i = __float_as_int(x);
    return i < 0 ? i ^ 0x7fffffff : i;
}
__device__ __forceinline__ float float_from_order_key(int k)
{
    return __int_as_float(k < 0 ? k ^ 0x7fffffff : k);
}

// Bit t set: 16-row tile t holds a row that the index range [lo, hi] of dimension d can reach.
// Warp-wide: lane l looks at the indices l and l + 32 through the index -> row table (at most 64
// index values per dimension) and the bits are OR-reduced; every lane returns the mask.
__device__ __forceinline__ uint32_t perm_tile_mask_warp(const uint16_t *lut_d, int n_d, int lo, int hi, int lane)
{
    uint32_t m = 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = lane + 32 * k;
        if (idx >= lo && idx <= hi && idx < n_d) m |= 1u << (lut_d[idx] >> 4);
    }
    return __reduce_or_sync(0xffffffffu, m);
}

// Head modes of the tiled kernels.  A thread block always works on two "slots" packed as half2:
//   HDM_PAIR8   head_dim 8 : slots = heads 2hp, 2hp+1, 8 channels each, one plane
//   HDM_SINGLE16 head_dim 16: slots = the two 8-channel halves of head hp (partial scores are summed)
//   HDM_PAIR16  head_dim 16: slots = heads 2hp, 2hp+1; their 16 channels are split into two PLANES of
//               8; contractions over channels accumulate over the planes, products whose result
//               is per channel are made once per plane.  Per-pair work (look-ups, histograms) is
//               that of one head_dim-8 pair, i.e. half of two HDM_SINGLE16 blocks.
constexpr int HDM_PAIR8 = 0, HDM_SINGLE16 = 1, HDM_PAIR16 = 2;

// Offset (in halves, inside a voxel or table row of H*hd channels) of the 8 channels of slot h, plane s.
template <int HDM>
__device__ __forceinline__ int slot_offset(int hp, int h, int s)
{
    return HDM == HDM_PAIR16 ? hp * 32 + h * 16 + s * 8 : hp * 16 + h * 8;
}

// A-operand fragment (16 table rows of tile mt x the 16 (slot, channel) of one plane).
template <int HDM>
__device__ __forceinline__ void load_table_a_frag(uint32_t (&a)[2][2], const __half *tab, const CrseMeta &im, int HC,
                                                  int hp, int s, int mt, int g, int t)
{
    const int r0 = table_row(im, mt * 16 + g), r1 = table_row(im, mt * 16 + g + 8);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int o = slot_offset<HDM>(hp, h, s) + 2 * t;
        a[h][0] = r0 >= 0 ? *reinterpret_cast<const uint32_t *>(tab + (int64_t)r0 * HC + o) : 0u;
        a[h][1] = r1 >= 0 ? *reinterpret_cast<const uint32_t *>(tab + (int64_t)r1 * HC + o) : 0u;
    }
}

// Table row (within a 16-row k-step) that k-slot (2t + 8*half + second) of an mma lane stands for in
// the hist . T products: slots {2t, 2t+1, 2t+8, 2t+9} <-> rows {t, t+4, t+8, t+12}.  This is the order
// in which the conflict-free histogram loads of ht_unit (attn_tc_small.cuh) deliver the rows.
__device__ __forceinline__ int ht_krow(int t, int half, int second) { return t + 8 * half + 4 * second; }

// B-operand fragment (k = the 16 table rows of k-step ks in ht_krow order, n = the 8 channels of
// slot h, plane s).
template <int HDM>
__device__ __forceinline__ void load_table_b_frag(uint32_t (&b)[2][2], const __half *tab, const CrseMeta &im, int HC,
                                                  int hp, int s, int ks, int g, int t)
{
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int ra = table_row(im, ks * 16 + ht_krow(t, half, 0)), rb = table_row(im, ks * 16 + ht_krow(t, half, 1));
            const int o = slot_offset<HDM>(hp, h, s) + g;
            const __half lo = ra >= 0 ? tab[(int64_t)ra * HC + o] : __float2half(0.f);
            const __half hi = rb >= 0 ? tab[(int64_t)rb * HC + o] : __float2half(0.f);
            b[h][half] = h2_as_u32(__halves2half2(lo, hi));
        }
}

// Histogram update  hist[a][row_j] += v[a][j]  for four voxels j of a tile at once, for NDIM signal
// dimensions (disjoint row ranges) and NARR histograms sharing the row index.  All loads are issued
// before any store, so the shared-memory latency is paid once per group instead of once per voxel;
// equal rows inside a group are chained in registers (later voxel wins the store, carrying the sum).
// `cell` points at this lane's column of histogram 0; `off[d][j]` = row * QT (words).
// Only the first `cnt` voxels of the group exist; the others are neither loaded into the chain nor
// stored (a dummy store could overwrite a concurrent update of an aliased row by another warp).
template <int NDIM, int NARR>
__device__ __forceinline__ void hist_add4(uint32_t *cell, int arr_stride, const int (&off)[NDIM][4],
                                          const uint32_t (&v)[NARR][4], int cnt)
{
    uint32_t c[NDIM][NARR][4];
#pragma unroll
    for (int d = 0; d < NDIM; ++d)
#pragma unroll
        for (int a = 0; a < NARR; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) c[d][a][j] = cell[a * arr_stride + off[d][j]];
#pragma unroll
    for (int d = 0; d < NDIM; ++d) {
        const bool e10 = off[d][1] == off[d][0];
        const bool e20 = off[d][2] == off[d][0], e21 = off[d][2] == off[d][1];
        const bool e30 = off[d][3] == off[d][0], e31 = off[d][3] == off[d][1], e32 = off[d][3] == off[d][2];
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            const __half2 s0 = __hadd2(u32_as_h2(c[d][a][0]), u32_as_h2(v[a][0]));
            const __half2 s1 = __hadd2(e10 ? s0 : u32_as_h2(c[d][a][1]), u32_as_h2(v[a][1]));
            const __half2 s2 = __hadd2(e21 ? s1 : (e20 ? s0 : u32_as_h2(c[d][a][2])), u32_as_h2(v[a][2]));
            const __half2 s3 = __hadd2(e32 ? s2 : (e31 ? s1 : (e30 ? s0 : u32_as_h2(c[d][a][3]))), u32_as_h2(v[a][3]));
            c[d][a][0] = h2_as_u32(s0); c[d][a][1] = h2_as_u32(s1);
            c[d][a][2] = h2_as_u32(s2); c[d][a][3] = h2_as_u32(s3);
        }
    }
#pragma unroll
    for (int d = 0; d < NDIM; ++d)
#pragma unroll
        for (int a = 0; a < NARR; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < cnt) cell[a * arr_stride + off[d][j]] = c[d][a][j];
}

// Work distribution of the tiled kernels.  A work item is (window, tile of 32 voxels); tile t of window w
// belongs to block (w + t) mod gridDim.x of its head pair, which spreads the tiles of large windows
// over the blocks (whole windows per block left the blocks 15-30 % out of balance where windows are
// few and of very different sizes).  The blocks find their items without any global bookkeeping:
// window sizes are read in chunks of WL_CHUNK, every thread of the first WL_CHUNK/32 warps looks at one
// window and the warp appends its items to its own segment of a list in shared memory, in window
// order (deterministic).  Entry: (window - chunk start) << 8 | tile.  A chunk whose items do not fit
// the list (windows of thousands of voxels) is walked directly instead (WorkItems::next).
constexpr int WL_CHUNK = 256, WL_SEG = 64;      // windows per chunk; list entries per warp segment
constexpr int WL_NSEG = WL_CHUNK / 32;
constexpr int WL_BYTES = WL_NSEG * WL_SEG * 2 + 64;

// s_list: uint16 [WL_NSEG][WL_SEG], s_cnt: int [WL_NSEG + 1] (the last entry: overflow flag, cleared by
// the caller before).  All threads of the block call this between two __syncthreads().  Windows of at
// most `skip_upto` voxels are left out.
__device__ __forceinline__ void build_work_list(const int32_t *__restrict__ w_sizes, int64_t W, int64_t c0,
                                                int skip_upto, uint16_t *s_list, int *s_cnt)
{
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    if (tid >= WL_CHUNK) return;
    const int nb = gridDim.x, b = blockIdx.x;
    const int64_t w = c0 + tid;
    const int n = w < W ? __ldg(w_sizes + w) : 0;
    const int tiles = n > skip_upto ? (n + QT - 1) / QT : 0;
    int t = (int)(((int64_t)b - w) % nb);
    if (t < 0) t += nb;
    int pos = 0;
    bool over = tiles > 256;
    while (__any_sync(0xffffffffu, t < tiles)) {
        const bool mine = t < tiles;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (mine) {
            const int at = pos + __popc(m & ((1u << lane) - 1u));
            if (at < WL_SEG) s_list[wid * WL_SEG + at] = (uint16_t)((tid << 8) | (t & 255));
        }
        pos += __popc(m);
        t += nb;
    }
    over = over || pos > WL_SEG;
    if (__any_sync(0xffffffffu, over) && lane == 0) s_cnt[WL_NSEG] = 1;
    if (lane == 0) s_cnt[wid] = pos;
}

// Next item of this block in the current chunk (every thread holds the same state: list position
// pos = segment * WL_SEG + index, or, when the list overflowed, the window and tile of a direct walk).
// -> true and (window, first voxel of the tile), false at the end of the chunk.
__device__ __forceinline__ bool next_work_item(const uint16_t *list, const int *cnt, const int32_t *__restrict__ w_sizes,
                                               int64_t W, int64_t c0, int skip_upto, int &pos, int &dw, int &dt,
                                               int64_t &win, int &x0)
{
    if (cnt[WL_NSEG] == 0) {
        while (pos < WL_NSEG * WL_SEG && (pos & (WL_SEG - 1)) >= cnt[pos / WL_SEG]) pos = (pos | (WL_SEG - 1)) + 1;
        if (pos >= WL_NSEG * WL_SEG) return false;
        const int e = list[pos++];
        win = c0 + (e >> 8);
        x0 = (e & 255) * QT;
        return true;
    }
    // direct walk: dw = window offset in the chunk, dt = next tile of that window for this block (-1: none yet)
    const int nb = gridDim.x, b = blockIdx.x;
    for (;;) {
        if (dw >= 0 && dw < WL_CHUNK && c0 + dw < W && dt >= 0) {
            const int n = __ldg(w_sizes + c0 + dw);
            const int tiles = n > skip_upto ? (n + QT - 1) / QT : 0;
            if (dt < tiles) {
                win = c0 + dw;
                x0 = dt * QT;
                dt += nb;
                return true;
            }
        }
        ++dw;
        if (dw >= WL_CHUNK || c0 + dw >= W) return false;
        dt = (int)(((int64_t)b - (c0 + dw)) % nb);
        if (dt < 0) dt += nb;
    }
}

// Shared-memory carve-up (byte offsets) for a table of R rows.
struct SmemLayout {
    int R16;      // rows rounded up to a multiple of 16
    int Rp;       // row stride (words) of the per-key array, == 8 (mod 32)
    int off_pq, off_hist, off_pk, off_s, off_idx, off_kv, off_kc, off_misc, total;
};

__host__ __device__ inline SmemLayout make_layout(int R, int n_rowq_arrays, int n_planes = 1, int n_warps = NWARP)
{
    const int kt = 2 * n_warps;                                  // keys per tile: two per warp
    SmemLayout L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    int off = 0;
    L.off_pq = off;   off += n_rowq_arrays * L.R16 * QT * 4;   // P_q (and dB in the backward)
    L.off_hist = off; off += n_rowq_arrays * L.R16 * QT * 4;   // histograms
    // the per-key array doubles as the cross-warp reduction buffer of the epilogue (2.25 KB per warp)
    const int red = n_warps * (QT * 16 + QT * 2) * 4;
    L.off_pk = off;   off += (kt * L.Rp * 4 > red) ? kt * L.Rp * 4 : red;
    L.off_s = off;    off += kt * QT * 8;                      // float2 scores / half2 probabilities
    L.off_idx = off;  off += kt * 2 * QT * 4;                  // packed cRSE indices
    L.off_kv = off;   off += n_planes * 2 * kt * 16 * 2;       // key and value rows of the tile, per plane
    L.off_kc = off;   off += kt * 12 * 4;                      // key coordinates, padded to 12
    L.off_misc = off; off += 1024 + WL_BYTES;
    L.total = off;
    return L;
}

}  // namespace tc
}  // namespace s3d
