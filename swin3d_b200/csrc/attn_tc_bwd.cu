// Fused backward of the cRSE window attention, tensor-core path (fp16 storage, head_dim 8 or 16).
//
// One templated kernel, launched twice per call:
//   SIDE 0  lanes = queries (x = q, y = k):  dQ, dTq, dTv
//   SIDE 1  lanes = keys    (x = k, y = q):  dK, dV, dTk
// Both sweeps recompute, per pair, s = q.k + sum_n P_q[row_n] + sum_n P_k[row_n], p = exp(s - lse),
// dP = dO.v + sum_n dB_q[row_n] (dB_q = dO_q . Tv^T) and ds = p (dP - delta_q), with the three
// projections P_q, P_k, dB produced by tensor-core GEMMs per window.  The x side owns per-voxel
// histograms  H0[x][row] += ds  (and, SIDE 0, H1[x][row] += p); they turn the table terms into GEMMs:
//   dX     += H0 . T0                 (T0 = Tq on SIDE 0, Tk on SIDE 1)
//   dT0    += H0^T . X0               (dTq += histQ^T.Q ; dTk += histK^T.K)
//   dTv    += H1^T . dO               (SIDE 0)
// Table gradients are accumulated in registers over every window a block processes and reach
// global memory once per block (atomicAdd of fp32), instead of once per pair, head and channel.
// grid = (x, head pairs or heads: head modes of attn_tc.cuh); one block per SM (16 warps).  With two
// planes (two heads of 16 channels per block) contractions over channels accumulate over the planes,
// per-channel products (dX, dT) are made once per plane; the y-side table fragments, used once per
// y tile, stay in registers, the x-side ones are fetched per item, and the x rows are staged a second
// time for the table-gradient GEMMs instead of being held in registers across the y loop.
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"

namespace s3d {
namespace tc {

constexpr int BW_NWARP = 16;
constexpr int BW_THREADS = BW_NWARP * 32;
// y voxels per tile: 32 (two per warp) where shared memory allows it, else 16
__host__ __device__ constexpr int bkt_of(int side) { return side == 0 ? 16 : 32; }

struct BwdSmem {
    int R16, Rp;
    int off_px, px_stride, off_hx, off_py, py_stride, off_s, off_dp, off_idx, off_yt, off_yc, off_misc, total;
};

__host__ __device__ inline BwdSmem make_bwd_layout(int R, int npx, int nh, int npy, int BKT, int n_planes = 1)
{
    BwdSmem L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    L.px_stride = L.R16 * QT * 4;
    L.py_stride = BKT * L.Rp * 4;
    int off = 0;
    const int px_bytes = npx * L.px_stride;
    L.off_px = off; off += px_bytes > 36864 ? px_bytes : 36864;   // doubles as the 34 KB reduction buffer
    L.off_hx = off; off += nh * L.px_stride;
    L.off_py = off; off += npy * L.py_stride;
    L.off_s = off;  off += BKT * QT * 8;     // float2 scores, then (p, ds) half2 pairs
    L.off_dp = off; off += BKT * QT * 8;     // float2 dO.v
    L.off_idx = off; off += BKT * 2 * QT * 4;
    L.off_yt = off; off += n_planes * 2 * BKT * 16 * 2;
    L.off_yc = off; off += BKT * 12 * 4;
    L.off_misc = off; off += 2048 + WL_BYTES;
    L.total = off;
    return L;
}

struct BwdParams {
    const __half *x0, *x1, *y0, *y1;   // feature rows [N][H][hd]: SIDE 0: q, dout, k, v ; SIDE 1: k, v, q, dout
    const __half *o;                   // forward output (for delta)
    const float *lse;
    const __half *t_px0, *t_px1, *t_py0, *t_py1;   // tables of the x / y projections
    __half *dx0, *dx1;                 // SIDE 0: dq, - ; SIDE 1: dk, dv
    float *dt0, *dt1;                  // SIDE 0: dtq, dtv ; SIDE 1: dtk, -
    const int32_t *w_sizes, *w2n, *n2n;
    const float *n_coords;
    int64_t W;
    int H;
    int skip_upto;   // windows with at most this many voxels are left to the single-sweep kernel
};

// Projection GEMM  P^T[row][(voxel, slot)] = T . F^T  for 8 n-tiles of 4 voxels, written either in the
// lane-major layout [row][32] (column = qpos(voxel)) or in the tile layout [voxel][Rp].  `feat` holds
// the staged rows plane by plane ([plane][plane_rows][16]); with two planes the channel contraction
// accumulates over them.  RESIDENT: the table fragments come from registers (`ta`, [unit][plane]);
// otherwise they are fetched from `tab` as they are needed.
template <int MTW, bool LANE_MAJOR, int HDM, bool RESIDENT, int MTA, int NPA>
__device__ __forceinline__ void project(const uint32_t (&ta)[MTA][NPA][2][2], const __half *tab, const CrseMeta &meta,
                                        int HC, int hp, const __half *feat, int plane_rows, uint32_t *dst,
                                        int n_mt, int Rp, int nvalid, int wid, int g, int t)
{
    constexpr int NT = 8;
    constexpr int NPL = HDM == HDM_PAIR16 ? 2 : 1;
    uint32_t b[NPL][NT][2];
#pragma unroll
    for (int pl = 0; pl < NPL; ++pl)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint32_t wv = 4 * j < nvalid ? *reinterpret_cast<const uint32_t *>(feat + pl * plane_rows * 16 + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t) : 0u;
            b[pl][j][0] = (g & 1) ? 0u : wv;
            b[pl][j][1] = (g & 1) ? wv : 0u;
        }
#pragma unroll
    for (int i = 0; i < MTW; ++i) {
        const int mt = wid + BW_NWARP * i;
        if (mt < n_mt) {
            uint32_t d0[NT], d1[NT];
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
                uint32_t af[2][2];
                if (!RESIDENT) {
                    load_table_a_frag<HDM>(af, tab, meta, HC, hp, pl, mt, g, t);
                } else {
                    af[0][0] = ta[i % MTA][pl % NPA][0][0]; af[0][1] = ta[i % MTA][pl % NPA][0][1];
                    af[1][0] = ta[i % MTA][pl % NPA][1][0]; af[1][1] = ta[i % MTA][pl % NPA][1][1];
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    if (4 * j < nvalid) {   // n-tiles made of padding voxels only are not computed
                        if (pl == 0) mma_k16_h(d0[j], d1[j], af[0][0], af[0][1], af[1][0], af[1][1], b[pl][j][0], b[pl][j][1]);
                        else mma_k16_ha(d0[j], d1[j], af[0][0], af[0][1], af[1][0], af[1][1], b[pl][j][0], b[pl][j][1]);
                    } else if (pl == 0) {
                        d0[j] = 0u;
                        d1[j] = 0u;
                    }
                }
            }
            if (LANE_MAJOR) {
                // odd rows of a quarter warp store their upper half first: the eight lanes cover all banks
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
                for (int j = 0; j < NT; ++j) {
                    if (4 * j < nvalid) {
                        uint32_t *p = dst + (4 * j + t) * Rp + mt * 16 + g;
                        p[0] = d0[j];
                        p[8] = d1[j];
                    }
                }
            }
        }
    }
}

// acc[head][m-tile] += E^T-tile . Y : rows = the 32 x of the item, k = the 16 y of the tile, E the
// p (WHICH = 1) or ds (WHICH = 0) half of the (p, ds) entries s_pd[y][x]; Y the staged y rows [32][16];
// one call covers the 16 y starting at `ybase`.
template <int WHICH>
__device__ __forceinline__ void dx_gemm(float (&acc)[2][2][4], const uint2 *s_pd, const __half *ysrc, int ybase, int g, int t)
{
    uint32_t fa[2][2][4];   // [head][m-tile][a0..a3]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int xx = 16 * i + g + 8 * rr, ya = ybase + 2 * t + 8 * kh;
                const uint2 e0 = s_pd[ya * QT + xx], e1 = s_pd[(ya + 1) * QT + xx];
                const uint32_t u = WHICH == 0 ? e0.y : e0.x, v2 = WHICH == 0 ? e1.y : e1.x;
                fa[0][i][2 * kh + rr] = pack_lo(u, v2);
                fa[1][i][2 * kh + rr] = pack_hi(u, v2);
            }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t yb[2];
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
            const int ya = ybase + 2 * t + 8 * kh;
            yb[kh] = h2_as_u32(__halves2half2(ysrc[ya * 16 + h * 8 + g], ysrc[(ya + 1) * 16 + h * 8 + g]));
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
            mma_k16(acc[h][i], fa[h][i][0], fa[h][i][1], fa[h][i][2], fa[h][i][3], yb[0], yb[1]);
    }
}

template <int D, int MTW, int SIDE, int HDM>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_tc_kernel(const BwdParams P, const CrseMeta meta)
{
    constexpr bool HD16 = HDM == HDM_SINGLE16;     // the two slots are halves of one head
    constexpr bool PAIR16 = HDM == HDM_PAIR16;     // two heads of 16 channels, two planes
    constexpr int NPL = PAIR16 ? 2 : 1;
    constexpr int MTP = PAIR16 ? 1 : MTW;          // resident table fragments only with one plane
    constexpr int BKT = bkt_of(SIDE);
    constexpr int NPX = SIDE == 0 ? 2 : 1;   // x-side projections: (P_q, dB) | (P_k)
    constexpr int NH = SIDE == 0 ? 2 : 1;    // x-side histograms:  (ds, p)   | (ds)
    constexpr int NPY = SIDE == 0 ? 1 : 2;   // y-side projections: (P_k)     | (P_q, dB)
    extern __shared__ __align__(16) unsigned char smem[];
    const BwdSmem L = make_bwd_layout(meta.R, NPX, NH, NPY, BKT, NPL);
    uint32_t *s_px = reinterpret_cast<uint32_t *>(smem + L.off_px);   // [NPX][R16][32]
    uint32_t *s_hx = reinterpret_cast<uint32_t *>(smem + L.off_hx);   // [NH][R16][32]
    uint32_t *s_py = reinterpret_cast<uint32_t *>(smem + L.off_py);   // [NPY][KT][Rp]
    float2 *s_s = reinterpret_cast<float2 *>(smem + L.off_s);         // [BKT][32]
    uint2 *s_pd = reinterpret_cast<uint2 *>(smem + L.off_s);          // same storage: (p, ds) half2 pairs
    float2 *s_dp = reinterpret_cast<float2 *>(smem + L.off_dp);       // [BKT][32]
    uint32_t *s_idx = reinterpret_cast<uint32_t *>(smem + L.off_idx); // [BKT][2][32]
    __half *s_y0 = reinterpret_cast<__half *>(smem + L.off_yt);       // [plane][BKT][16]
    __half *s_y1 = s_y0 + NPL * BKT * 16;                             // [plane][BKT][16]
    float *s_yc = reinterpret_cast<float *>(smem + L.off_yc);         // [BKT][12]
    float *s_ylse = reinterpret_cast<float *>(smem + L.off_misc);     // [BKT][2]          (SIDE 1)
    float *s_ydel = s_ylse + 2 * BKT;                                 // [plane][BKT][2]   (SIDE 1)
    float *s_xlse = s_ydel + 2 * 2 * BKT;                             // [32][2]           (SIDE 0)
    float *s_xdel = s_xlse + 64;                                      // [plane][32][2]    (SIDE 0)
    int *s_xrow = reinterpret_cast<int *>(s_xdel + 128);              // [32]
    uint16_t *s_wlist = reinterpret_cast<uint16_t *>(smem + L.off_misc + 2048);   // work list of the chunk
    int *s_wcnt = reinterpret_cast<int *>(s_wlist + WL_NSEG * WL_SEG);
    __half *s_x0 = reinterpret_cast<__half *>(smem + L.off_s);        // [plane][32][16] aliases s_s (set-up, table gradients)
    __half *s_x1 = reinterpret_cast<__half *>(smem + L.off_dp);       // [plane][32][16] aliases s_dp
    float *s_red = reinterpret_cast<float *>(smem + L.off_px);        // [16][32][16] aliases s_px (epilogue)
    float *s_red2 = s_red + BW_NWARP * QT * 16;                       // [32][16]

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int hp = blockIdx.y, H = P.H;
    const int HC = H * (HDM == HDM_PAIR8 ? 8 : 16);
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int pxw = L.px_stride / 4, pyw = L.py_stride / 4;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // ---- resident table fragments: those of the y side (used once per y tile) in every mode, those of
    //      the x side (used once per item) only with one plane --------------------------------------------
    uint32_t ta_py0[MTW][NPL][2][2], ta_py1[SIDE == 1 ? MTW : 1][NPL][2][2];
    uint32_t ta_px0[MTP][1][2][2], ta_px1[MTP][1][2][2];
    uint32_t t0B[MTP][2][2];   // B fragments (k = row, n = channel) of T0 for dX += H0 . T0
#pragma unroll
    for (int i = 0; i < MTW; ++i)
#pragma unroll
        for (int pl = 0; pl < NPL; ++pl) {
            const int mt = wid + BW_NWARP * i;
            load_table_a_frag<HDM>(ta_py0[i][pl], P.t_py0, meta, HC, hp, pl, mt, g, t);
            if (SIDE == 1) load_table_a_frag<HDM>(ta_py1[i % (SIDE == 1 ? MTW : 1)][pl], P.t_py1, meta, HC, hp, pl, mt, g, t);
        }
    if (!PAIR16) {
#pragma unroll
        for (int i = 0; i < MTP; ++i) {
            const int mt = wid + BW_NWARP * i;
            load_table_a_frag<HDM>(ta_px0[i][0], P.t_px0, meta, HC, hp, 0, mt, g, t);
            if (SIDE == 0) load_table_a_frag<HDM>(ta_px1[i][0], P.t_px1, meta, HC, hp, 0, mt, g, t);
            load_table_b_frag<HDM>(t0B[i], P.t_px0, meta, HC, hp, 0, mt, g, t);
        }
    }
    // table-gradient accumulators: [plane][hist][row tile of this warp][slot][c-frag]
    float dt_acc[NPL][NH][MTW][2][4];
#pragma unroll
    for (int pl = 0; pl < NPL; ++pl)
#pragma unroll
        for (int a = 0; a < NH; ++a)
#pragma unroll
            for (int i = 0; i < MTW; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    dt_acc[pl][a][i][h][0] = dt_acc[pl][a][i][h][1] = dt_acc[pl][a][i][h][2] = dt_acc[pl][a][i][h][3] = 0.f;
    // pair GEMMs dX += E^T . Y run in otherwise idle warps, one (product, plane) each:
    //   warp 15: ds . Y0 plane 0   warp 14: p . Y1 plane 0 (SIDE 1)   warps 13 / 12: the same for plane 1
    const int dx_which = (wid & 1) ? 0 : 1;
    const int dx_plane = wid >= BW_NWARP - 2 ? 0 : 1;
    const bool dx_warp = wid >= BW_NWARP - (PAIR16 ? 4 : 2) && (SIDE == 1 || dx_which == 0);

    for (int64_t c0 = 0; c0 < P.W; c0 += WL_CHUNK) {
        __syncthreads();            // every warp has left the item loop of the previous chunk
        if (tid == 0) s_wcnt[WL_NSEG] = 0;
        __syncthreads();
        build_work_list(P.w_sizes, P.W, c0, P.skip_upto, s_wlist, s_wcnt);
        __syncthreads();
        int it_pos = 0, it_dw = -1, it_dt = -1;
        int64_t w;
        int x0;
        while (next_work_item(s_wlist, s_wcnt, P.w_sizes, P.W, c0, P.skip_upto, it_pos, it_dw, it_dt, w, x0)) {
            const int n = __ldg(P.w_sizes + w), base = __ldg(P.w2n + w);
            const int nx = min(QT, n - x0);
            // ---- item set-up: x rows, x coordinates, projections of the x side, empty histograms --------
            __syncthreads();
            float cx[D];
#pragma unroll
            for (int d = 0; d < D; ++d)
                cx[d] = lane < nx ? __ldg(P.n_coords + (int64_t)(base + x0 + lane) * D + d) : 0.f;
            // y tiles are fetched into registers one tile ahead: row pieces (and, SIDE 1, the forward
            // output and lse of the rows) by the first 4*BKT*NPL threads, y coordinates one element per
            // thread starting from the upper half
            uint4 pf_val = make_uint4(0, 0, 0, 0), pf_o = make_uint4(0, 0, 0, 0);
            float pf_c = 0.f, pf_ls = 0.f;
            const int pf_e = (tid + BW_THREADS / 2) % BW_THREADS;
            static_assert(BKT * D <= BW_THREADS, "one y coordinate per thread");
            auto fetch_tile = [&](int yb) {
                const int nyb = min(BKT, n - yb);
                pf_val = make_uint4(0, 0, 0, 0);
                pf_o = make_uint4(0, 0, 0, 0);
                pf_c = 0.f;
                pf_ls = 0.f;
                if (tid < 4 * BKT * NPL) {
                    const int yi = (tid >> 2) % BKT, which = (tid >> 1) & 1, hf = tid & 1, pl = tid / (4 * BKT);
                    if (yi < nyb) {
                        const int row = __ldg(P.n2n + base + yb + yi);
                        const __half *src = which ? P.y1 : P.y0;
                        const int64_t goff = (int64_t)row * HC + slot_offset<HDM>(hp, hf, pl);
                        pf_val = __ldg(reinterpret_cast<const uint4 *>(src + goff));
                        if (SIDE == 1 && which == 1) {
                            pf_o = __ldg(reinterpret_cast<const uint4 *>(P.o + goff));
                            if (pl == 0) pf_ls = __ldg(P.lse + (int64_t)row * H + (HD16 ? hp : 2 * hp + hf));
                        }
                    }
                }
                if (pf_e < BKT * D && pf_e / D < nyb) pf_c = __ldg(P.n_coords + (int64_t)(base + yb + pf_e / D) * D + pf_e % D);
            };
            fetch_tile(0);
            // the global loads are issued first and consumed after the histograms have been cleared, so
            // that their latency overlaps the clearing
            const int st_xi = (tid >> 2) & 31, st_which = (tid >> 1) & 1, st_hf = tid & 1, st_pl = tid >> 7;
            const bool st_stage = tid < 128 * NPL, st_act = st_stage && st_xi < nx;
            uint4 st_val = make_uint4(0, 0, 0, 0), st_o = make_uint4(0, 0, 0, 0);
            float st_lse = 0.f;
            int st_row = 0;
            if (st_act) {
                st_row = __ldg(P.n2n + base + x0 + st_xi);
                const __half *src = st_which ? P.x1 : P.x0;
                const int64_t goff = (int64_t)st_row * HC + slot_offset<HDM>(hp, st_hf, st_pl);
                st_val = __ldg(reinterpret_cast<const uint4 *>(src + goff));
                if (SIDE == 0 && st_which == 1) {
                    st_o = __ldg(reinterpret_cast<const uint4 *>(P.o + goff));
                    if (st_pl == 0) st_lse = __ldg(P.lse + (int64_t)st_row * H + (HD16 ? hp : 2 * hp + st_hf));
                }
            }
            for (int i = tid; i < NH * L.R16 * QT / 4; i += BW_THREADS)
                reinterpret_cast<uint4 *>(s_hx)[i] = make_uint4(0, 0, 0, 0);
            if (st_stage) {
                if (st_act && st_which == 0 && st_hf == 0 && st_pl == 0) s_xrow[st_xi] = st_row;
                if (SIDE == 0 && st_which == 1) {
                    // delta[x][slot hf] = sum_c dO . O (this plane's 8 channels; zero beyond the tile) ; lse
                    const __half2 *a2 = reinterpret_cast<const __half2 *>(&st_val);
                    const __half2 *b2 = reinterpret_cast<const __half2 *>(&st_o);
                    float acc = 0.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float2 fa = __half22float2(a2[c]), fb = __half22float2(b2[c]);
                        acc += fa.x * fb.x + fa.y * fb.y;
                    }
                    s_xdel[st_pl * 64 + st_xi * 2 + st_hf] = acc;
                    if (st_pl == 0) s_xlse[st_xi * 2 + st_hf] = st_lse;
                }
                *reinterpret_cast<uint4 *>((st_which ? s_x1 : s_x0) + st_pl * 512 + st_xi * 16 + st_hf * 8) = st_val;
            }
            __syncthreads();
            float xlse[2] = {0.f, 0.f}, xdel[2] = {0.f, 0.f};
            if (SIDE == 0) {
                xlse[0] = s_xlse[lane * 2]; xlse[1] = s_xlse[lane * 2 + 1];
                xdel[0] = s_xdel[lane * 2]; xdel[1] = s_xdel[lane * 2 + 1];
                if (PAIR16) { xdel[0] += s_xdel[64 + lane * 2]; xdel[1] += s_xdel[64 + lane * 2 + 1]; }
                if (HD16) xdel[0] = xdel[1] = xdel[0] + xdel[1];   // delta of the whole head
            }
            // block-diagonal B fragments of X0^T / X1^T for the n-tile this warp multiplies in S0 / dPV0
            uint32_t xS[2][NPL][2];   // [X0 | X1][plane][b0, b1] for n-tile wid % 8
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int pl = 0; pl < NPL; ++pl) {
                    const __half *src = (a == 0 ? s_x0 : s_x1) + pl * 512;
                    const int j = wid & 7;
                    const uint32_t wv = *reinterpret_cast<const uint32_t *>(src + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                    xS[a][pl][0] = (g & 1) ? 0u : wv;
                    xS[a][pl][1] = (g & 1) ? wv : 0u;
                }
            // one-plane modes: B fragments (k = position, n = channel) of X0 / X1 for the table-gradient
            // GEMMs, kept in registers over the y loop (the staged rows are overwritten by it); with two
            // planes the rows are staged again after the loop instead
            constexpr int NHP = PAIR16 ? 1 : NH;
            uint32_t xTB[NHP][2][2][2];   // [hist][k-step][slot][b0,b1]
            if (!PAIR16) {
#pragma unroll
                for (int a = 0; a < NHP; ++a) {
                    // SIDE 0: hist 0 (ds) pairs with X0 = Q, hist 1 (p) with X1 = dO ; SIDE 1: hist 0 with X0 = K
                    const __half *src = a == 0 ? s_x0 : s_x1;
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                const int p0 = 16 * ks + 4 * t + 2 * half, p1 = p0 + 1;
                                const int xa = (p0 >> 2) + 8 * (p0 & 3), xb = (p1 >> 2) + 8 * (p1 & 3);
                                xTB[a][ks][h][half] = h2_as_u32(__halves2half2(src[xa * 16 + h * 8 + g], src[xb * 16 + h * 8 + g]));
                            }
                }
            }
            project<MTW, true, HDM, !PAIR16>(ta_px0, P.t_px0, meta, HC, hp, s_x0, 32, s_px, n_mt, Rp, nx, wid, g, t);
            if (SIDE == 0) project<MTW, true, HDM, !PAIR16>(ta_px1, P.t_px1, meta, HC, hp, s_x1, 32, s_px + pxw, n_mt, Rp, nx, wid, g, t);

            float dxa[2][2][4];   // [slot][m-tile][c-frag] of this warp's pair GEMM (see dx_warp)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i) dxa[h][i][0] = dxa[h][i][1] = dxa[h][i][2] = dxa[h][i][3] = 0.f;

            for (int y0 = 0; y0 < n; y0 += BKT) {
                const int ny = min(BKT, n - y0);
                __syncthreads();
                // ---- stage the y tile (fetched into registers one tile ahead) ----------------------------
                if (tid < 4 * BKT * NPL) {
                    const int yi = (tid >> 2) % BKT, which = (tid >> 1) & 1, hf = tid & 1, pl = tid / (4 * BKT);
                    if (SIDE == 1 && which == 1) {
                        const __half2 *a2 = reinterpret_cast<const __half2 *>(&pf_val);
                        const __half2 *b2 = reinterpret_cast<const __half2 *>(&pf_o);
                        float del = 0.f;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float2 fa = __half22float2(a2[c]), fb = __half22float2(b2[c]);
                            del += fa.x * fb.x + fa.y * fb.y;
                        }
                        s_ydel[pl * 2 * BKT + yi * 2 + hf] = del;      // zero beyond the tile (both rows are zero there)
                        if (pl == 0) s_ylse[yi * 2 + hf] = pf_ls;
                    }
                    *reinterpret_cast<uint4 *>((which ? s_y1 : s_y0) + pl * BKT * 16 + yi * 16 + hf * 8) = pf_val;
                }
                if (pf_e < BKT * D) s_yc[(pf_e / D) * 12 + pf_e % D] = pf_c;
                __syncthreads();
                if (y0 + BKT < n) fetch_tile(y0 + BKT);      // in flight while this tile is worked on
                // ---- y-side projections; S0 = Y0 . X0^T and dPV0 = Y1 . X1^T, one (m-tile, n-tile) per warp ----
                project<MTW, false, HDM, true>(ta_py0, P.t_py0, meta, HC, hp, s_y0, BKT, s_py, n_mt, Rp, ny, wid, g, t);
                if (SIDE == 1) project<MTW, false, HDM, true>(ta_py1, P.t_py1, meta, HC, hp, s_y1, BKT, s_py + pyw, n_mt, Rp, ny, wid, g, t);
                {
                    constexpr int PER = (BKT / 16) * 8;     // (m-tile, n-tile) units per product
#pragma unroll
                    for (int u0 = 0; u0 < 2 * PER; u0 += BW_NWARP) {
                        const int u = u0 + wid;
                        const int a = u / PER, r = u % PER, mt = r >> 3, j = r & 7;   // y rows 16mt.., x columns 4j..
                        if (16 * mt < ny && 4 * j < nx) {
                            float c[4];
#pragma unroll
                            for (int pl = 0; pl < NPL; ++pl) {
                                const __half *ysrc = (a == 0 ? s_y0 : s_y1) + pl * BKT * 16 + mt * 16 * 16;
                                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 2 * t);
                                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 2 * t);
                                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 8 + 2 * t);
                                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 8 + 2 * t);
                                const uint32_t b0 = a == 0 ? xS[0][pl][0] : xS[1][pl][0], b1 = a == 0 ? xS[0][pl][1] : xS[1][pl][1];
                                if (pl == 0) mma_k16_z(c, a0, a1, a2, a3, b0, b1);
                                else mma_k16(c, a0, a1, a2, a3, b0, b1);
                            }
                            float2 *dst = (a == 0 ? s_s : s_dp) + mt * 16 * QT;
                            dst[g * QT + 4 * j + t] = make_float2(c[0], c[1]);
                            dst[(g + 8) * QT + 4 * j + t] = make_float2(c[2], c[3]);
                        }
                    }
                }
                __syncthreads();
                // ---- phase 1: BKT/16 y per warp, lane = x: indices, 3*D look-ups, p and ds -------------
#pragma unroll
                for (int y2 = 0; y2 < BKT / BW_NWARP; ++y2) {
                    const int yy = (BKT / BW_NWARP) * wid + y2;
                    uint2 pd = make_uint2(0u, 0u);
                    if (yy < ny) {
                        __half2 b0 = __float2half2_rn(0.f), b1 = b0, b2 = b0;
                        uint32_t w0 = 0, w1 = 0;
                        float cyv[D];
                        load_coords12<D>(s_yc + yy * 12, cyv);
#pragma unroll
                        for (int d = 0; d < D; ++d) {
                            const float cy = cyv[d];
                            const int idx = SIDE == 0 ? crse_index_fast(cx[d], cy, meta.L[d], d == D - 1)
                                                      : crse_index_fast(cy, cx[d], meta.L[d], d == D - 1);
                            const int row = meta.rowbase[d] + idx;
                            b0 = __hadd2(b0, u32_as_h2(s_px[row * QT + mypos]));
                            b1 = __hadd2(b1, u32_as_h2(s_py[yy * Rp + row]));
                            if (SIDE == 0) b2 = __hadd2(b2, u32_as_h2(s_px[pxw + row * QT + mypos]));
                            else b2 = __hadd2(b2, u32_as_h2(s_py[pyw + yy * Rp + row]));
                            if (d < 5) w0 |= (uint32_t)idx << (IDX_BITS * d);
                            else w1 |= (uint32_t)idx << (IDX_BITS * (d - 5));
                        }
                        s_idx[(yy * 2 + 0) * QT + lane] = w0;
                        if (D > 5) s_idx[(yy * 2 + 1) * QT + lane] = w1;
                        const float2 bs = __half22float2(__hadd2(b0, b1));
                        const float2 bd = __half22float2(b2);
                        const float2 s0 = s_s[yy * QT + lane];
                        const float2 dp0 = s_dp[yy * QT + lane];
                        float ls0, ls1, de0, de1;
                        if (SIDE == 0) {
                            ls0 = xlse[0]; ls1 = xlse[1]; de0 = xdel[0]; de1 = xdel[1];
                        } else {
                            ls0 = s_ylse[yy * 2]; ls1 = s_ylse[yy * 2 + 1]; de0 = s_ydel[yy * 2]; de1 = s_ydel[yy * 2 + 1];
                            if (PAIR16) { de0 += s_ydel[2 * BKT + yy * 2]; de1 += s_ydel[2 * BKT + yy * 2 + 1]; }
                        }
                        if (HD16 && SIDE == 1) de0 = de1 = de0 + de1;
                        float sc0 = s0.x + bs.x, sc1 = s0.y + bs.y, dq0 = dp0.x + bd.x, dq1 = dp0.y + bd.y;
                        if (HD16) { sc0 = sc1 = sc0 + sc1; dq0 = dq1 = dq0 + dq1; }   // halves of one head add up
                        float p0 = exp2f((sc0 - ls0) * LOG2E);
                        float p1 = exp2f((sc1 - ls1) * LOG2E);
                        float ds0 = p0 * (dq0 - de0);
                        float ds1 = p1 * (dq1 - de1);
                        if (lane >= nx) { p0 = 0.f; p1 = 0.f; ds0 = 0.f; ds1 = 0.f; }   // padding lanes hold no voxel
                        pd.x = h2_as_u32(__floats2half2_rn(p0, p1));
                        pd.y = h2_as_u32(__floats2half2_rn(ds0, ds1));
                    }
                    s_pd[yy * QT + lane] = pd;   // replaces the score; zero for padded y
                }
                __syncthreads();
                // ---- phase 2: histogram updates, one signal dimension per warp, four y per step ----------
                if (wid < D) {
                    const int d = wid;
                    const int wsel = d / 5, sh = IDX_BITS * (d % 5);
                    const int rb = meta.rowbase[d];
                    uint32_t *cell = s_hx + mypos;
                    for (int y4 = 0; y4 < ny; y4 += 4) {
                        uint32_t vals[NH][4];
                        int off[1][4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int yy = y4 + j;
                            const uint2 pd = s_pd[yy * QT + lane];            // zero for padded y
                            vals[0][j] = pd.y;                                 // ds -> H0
                            if (NH == 2) vals[NH - 1][j] = pd.x;               // p  -> H1
                            const int idx = yy < ny ? (s_idx[(yy * 2 + wsel) * QT + lane] >> sh) & ((1 << IDX_BITS) - 1) : 0;
                            off[0][j] = (rb + idx) * QT;
                        }
                        hist_add4<1, NH>(cell, pxw, off, vals, ny - y4);
                    }
                }
                // ---- pair GEMMs on the tensor cores: dX += dS^T-tile . Y0 ; SIDE 1: dX1 += P^T-tile . Y1 ------
                if (dx_warp) {
                    if (dx_which == 0) {
                        const __half *ysrc = s_y0 + dx_plane * BKT * 16;
                        dx_gemm<0>(dxa, s_pd, ysrc, 0, g, t);
                        if (BKT > 16 && ny > 16) dx_gemm<0>(dxa, s_pd, ysrc, 16, g, t);
                    } else {
                        const __half *ysrc = s_y1 + dx_plane * BKT * 16;
                        dx_gemm<1>(dxa, s_pd, ysrc, 0, g, t);
                        if (BKT > 16 && ny > 16) dx_gemm<1>(dxa, s_pd, ysrc, 16, g, t);
                    }
                }
            }  // y tiles
            __syncthreads();
            if (PAIR16) {
                // the pair arrays are dead: stage the x rows again for the table-gradient GEMMs
                if (tid < 128 * NPL) {
                    const int xi = (tid >> 2) & 31, which = (tid >> 1) & 1, hf = tid & 1, pl = tid >> 7;
                    uint4 val = make_uint4(0, 0, 0, 0);
                    if (xi < nx && (which == 0 || NH == 2)) {
                        const __half *src = which ? P.x1 : P.x0;
                        val = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)s_xrow[xi] * HC + slot_offset<HDM>(hp, hf, pl)));
                    }
                    *reinterpret_cast<uint4 *>((which ? s_x1 : s_x0) + pl * 512 + xi * 16 + hf * 8) = val;
                }
                __syncthreads();
            }
            // ---- table gradients: dT[a][row][c] += sum_x H_a[row][x] X_a[x][c] --------------------------------
#pragma unroll
            for (int i = 0; i < MTW; ++i) {
                const int mt = wid + BW_NWARP * i;
                if (mt < n_mt) {
#pragma unroll
                    for (int a = 0; a < NH; ++a)
#pragma unroll
                        for (int pl = 0; pl < NPL; ++pl) {
                            uint32_t bf[2][2][2];   // [k-step][slot][b0, b1]
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                if (PAIR16) {
                                    const __half *src = (a == 0 ? s_x0 : s_x1) + pl * 512;
#pragma unroll
                                    for (int h = 0; h < 2; ++h)
#pragma unroll
                                        for (int half = 0; half < 2; ++half) {
                                            const int p0 = 16 * ks + 4 * t + 2 * half, p1 = p0 + 1;
                                            const int xa = (p0 >> 2) + 8 * (p0 & 3), xb = (p1 >> 2) + 8 * (p1 & 3);
                                            bf[ks][h][half] = h2_as_u32(__halves2half2(src[xa * 16 + h * 8 + g], src[xb * 16 + h * 8 + g]));
                                        }
                                } else {
                                    bf[ks][0][0] = xTB[a % NHP][ks][0][0]; bf[ks][0][1] = xTB[a % NHP][ks][0][1];
                                    bf[ks][1][0] = xTB[a % NHP][ks][1][0]; bf[ks][1][1] = xTB[a % NHP][ks][1][1];
                                }
                            }
                            dt_unit_b(dt_acc[pl][a][i], s_hx + a * pxw, bf, mt, g, t);
                        }
                }
            }
            // ---- per plane: dX += H0 . T0 (row range split over the warps), reduce, store ------------------------
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
                const int own0 = BW_NWARP - 1 - 2 * pl, own1 = BW_NWARP - 2 - 2 * pl;   // warps holding ds.Y0 / p.Y1 of this plane
                float part[2][2][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
#pragma unroll
                        for (int e = 0; e < 4; ++e) part[h][i][e] = (wid == own0) ? dxa[h][i][e] : 0.f;
#pragma unroll
                for (int i = 0; i < MTW; ++i) {
                    const int ks = wid + BW_NWARP * i;
                    if (ks < n_mt) {
                        uint32_t bf[2][2];
                        if (PAIR16) {
                            load_table_b_frag<HDM>(bf, P.t_px0, meta, HC, hp, pl, ks, g, t);
                        } else {
                            bf[0][0] = t0B[i % MTP][0][0]; bf[0][1] = t0B[i % MTP][0][1];
                            bf[1][0] = t0B[i % MTP][1][0]; bf[1][1] = t0B[i % MTP][1][1];
                        }
                        ht_unit(part, s_hx, bf, ks, g, t);
                    }
                }
                // every warp is done with s_px (phase 1 look-ups) before it becomes s_red, and with the
                // previous plane's reduction
                __syncthreads();
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const int xx = 16 * i + g + 8 * rr;
                            *reinterpret_cast<float2 *>(s_red + (wid * QT + xx) * 16 + h * 8 + 2 * t) =
                                make_float2(part[h][i][2 * rr], part[h][i][2 * rr + 1]);
                            if (SIDE == 1 && wid == own1)
                                *reinterpret_cast<float2 *>(s_red2 + xx * 16 + h * 8 + 2 * t) =
                                    make_float2(dxa[h][i][2 * rr], dxa[h][i][2 * rr + 1]);
                        }
                __syncthreads();
                {
                    const int xx = tid >> 4, ch = tid & 15;
                    if (xx < nx) {
                        float a = 0.f;
#pragma unroll
                        for (int ww = 0; ww < BW_NWARP; ++ww) a += s_red[(ww * QT + xx) * 16 + ch];
                        const int64_t o = (int64_t)s_xrow[xx] * HC + slot_offset<HDM>(hp, ch >> 3, pl) + (ch & 7);
                        P.dx0[o] = __float2half_rn(a);
                        if (SIDE == 1) P.dx1[o] = __float2half_rn(s_red2[xx * 16 + ch]);
                    }
                }
            }  // planes
        }  // items
    }      // chunks of windows

    // ---- flush the table gradients of this block ---------------------------------------------------------------
#pragma unroll
    for (int pl = 0; pl < NPL; ++pl)
#pragma unroll
        for (int a = 0; a < NH; ++a) {
            float *dst = a == 0 ? P.dt0 : P.dt1;
#pragma unroll
            for (int i = 0; i < MTW; ++i) {
                const int mt = wid + BW_NWARP * i;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int row = table_row(meta, mt * 16 + g + 8 * rr);   // aliases flush into the row they stand for
                        if (mt < n_mt && row >= 0) {
                            float *p = dst + (int64_t)row * HC + slot_offset<HDM>(hp, h, pl) + 2 * t;
                            atomicAdd(p, dt_acc[pl][a][i][h][2 * rr]);
                            atomicAdd(p + 1, dt_acc[pl][a][i][h][2 * rr + 1]);
                        }
                    }
            }
        }
}

template <int D, int MTW, int SIDE, int HDM>
static int launch_side(const BwdParams &p, const CrseMeta &meta, cudaStream_t st)
{
    const BwdSmem L = make_bwd_layout(meta.R, SIDE == 0 ? 2 : 1, SIDE == 0 ? 2 : 1, SIDE == 0 ? 1 : 2, bkt_of(SIDE),
                                      HDM == HDM_PAIR16 ? 2 : 1);
    auto kern = attn_bwd_tc_kernel<D, MTW, SIDE, HDM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    int dev = 0, sms = 148, per_sm = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, BW_THREADS, L.total) != cudaSuccess || per_sm < 1)
        return S3D_ERR_LAUNCH;
    const int hp = HDM == HDM_SINGLE16 ? p.H : p.H / 2;
    int gx = sms * per_sm / hp;
    if (gx > p.W) gx = (int)p.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, BW_THREADS, L.total, st>>>(p, meta);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <int D, int MTW, int HDM>
static int launch_both(const AttnArgs &a, int skip_upto, cudaStream_t st)
{
    BwdParams pq{};
    pq.skip_upto = skip_upto;
    pq.x0 = (const __half *)a.q;   pq.x1 = (const __half *)a.dout;
    pq.y0 = (const __half *)a.k;   pq.y1 = (const __half *)a.v;
    pq.o = (const __half *)a.out;  pq.lse = a.lse;
    pq.t_px0 = (const __half *)a.tq; pq.t_px1 = (const __half *)a.tv;
    pq.t_py0 = (const __half *)a.tk; pq.t_py1 = nullptr;
    pq.dx0 = (__half *)a.dq; pq.dx1 = nullptr;
    pq.dt0 = a.dtq; pq.dt1 = a.dtv;
    pq.w_sizes = a.w_sizes; pq.w2n = a.w2n; pq.n2n = a.n2n; pq.n_coords = a.n_coords;
    pq.W = a.W; pq.H = a.H;
    int rc = launch_side<D, MTW, 0, HDM>(pq, a.meta, st);
    if (rc != S3D_OK) return rc;
    BwdParams pk = pq;
    pk.x0 = (const __half *)a.k;   pk.x1 = (const __half *)a.v;
    pk.y0 = (const __half *)a.q;   pk.y1 = (const __half *)a.dout;
    pk.t_px0 = (const __half *)a.tk; pk.t_px1 = nullptr;
    pk.t_py0 = (const __half *)a.tq; pk.t_py1 = (const __half *)a.tv;
    pk.dx0 = (__half *)a.dk; pk.dx1 = (__half *)a.dv;
    pk.dt0 = a.dtk; pk.dt1 = nullptr;
    return launch_side<D, MTW, 1, HDM>(pk, a.meta, st);
}

template <int D, int MTW>
static int launch_mode(const AttnArgs &a, int hdm, int skip_upto, cudaStream_t st)
{
    switch (hdm) {
        case HDM_PAIR8: return launch_both<D, MTW, HDM_PAIR8>(a, skip_upto, st);
        case HDM_SINGLE16: return launch_both<D, MTW, HDM_SINGLE16>(a, skip_upto, st);
        default: return launch_both<D, MTW, HDM_PAIR16>(a, skip_upto, st);
    }
}

}  // namespace tc

bool attn_tc_bwd_supported(const AttnArgs &a)
{
    if (a.dtype != S3D_F16) return false;
    if (!(a.hd == 16 || (a.hd == 8 && !(a.H & 1)))) return false;
    const int Rint = a.meta.R + a.meta.D - 1;
    if (Rint > 16 * tc::BW_NWARP * 2) return false;
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;
    const int planes = attn_tc_head_mode(a) == tc::HDM_PAIR16 ? 2 : 1;
    if (tc::make_bwd_layout(Rint, 2, 2, 1, tc::bkt_of(0), planes).total > 227 * 1024) return false;
    if (tc::make_bwd_layout(Rint, 1, 1, 2, tc::bkt_of(1), planes).total > 227 * 1024) return false;
    return true;
}

// dtq, dtk, dtv must be zero on entry (the kernels accumulate into them).
int attn_tc_backward(const AttnArgs &a0, cudaStream_t st)
{
    if (a0.W == 0) return S3D_OK;
    AttnArgs a = a0;
    a.meta = tc::internal_meta(a0.meta);   // kernels work in the internal row numbering
    const int hdm = attn_tc_head_mode(a0);
    int skip_upto = 0;
    // the single-sweep kernel serves head pairs of 8 channels and single heads of 16, windows of any size
    if (hdm != tc::HDM_PAIR16 && attn_tc_bwd_small_supported(a0))
        return attn_tc_backward_small(a0, st);      // tile pairs: windows of any size
    if (a0.m_dq.n) return S3D_ERR_UNSUPPORTED;      // the two-sweep kernels have no mirrored stores
    const int n_mt = (a.meta.R + 15) / 16;
    const int mtw = (n_mt + tc::BW_NWARP - 1) / tc::BW_NWARP;
#define S3D_TC_BWD(DD)                                            \
    switch (mtw) {                                                \
        case 1: return tc::launch_mode<DD, 1>(a, hdm, skip_upto, st); \
        case 2: return tc::launch_mode<DD, 2>(a, hdm, skip_upto, st); \
        default: return S3D_ERR_UNSUPPORTED;                      \
    }
    switch (a.meta.D) {
        case 3: S3D_TC_BWD(3)
        case 6: S3D_TC_BWD(6)
        case 9: S3D_TC_BWD(9)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_TC_BWD
}

}  // namespace s3d
