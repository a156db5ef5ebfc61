// Backward of the cRSE window attention for windows of at most 32 voxels, tensor-core path
// (fp16 storage, head_dim 8): ONE sweep per window instead of a query sweep plus a key sweep.
//
// With the whole window in one 32 x 32 tile, the pair quantities (p, ds, packed cRSE indices) are
// computed once (lanes = queries, 3*D look-ups per pair) and kept in shared memory as a
// [key][query] array of 16-byte entries with a row stride of 33 entries, which can be read
// conflict-free both by rows (lanes = queries) and by columns (lanes = keys).  The query-side
// histograms (ds and p per query) are then built with lanes = queries, and the key-side histogram
// (ds per key) with lanes = keys from the stored entries -- no second set of projections and
// look-ups.  histK reuses the shared memory of the dead P_q projection, the cross-warp reduction
// buffer that of dB.  All table products are GEMMs (mma.sync m16n8k16); the (table, row-tile) units
// of the projection and table-gradient GEMMs are dealt round-robin to the 16 warps.
// grid = (x, H/2), one block per SM.  Larger windows go through attn_tc_bwd.cu.
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"

namespace s3d {
namespace tc {

#ifdef S3D_PHASE_CLOCK
__device__ unsigned int g_ablate_bwd;
__device__ unsigned long long g_phase_cycles_bwd[16];
#define S3D_KEEP(i) (!(ablate & (1u << (i))))
#define S3D_PHASE_DECL long long ph_t = clock64(); unsigned long long ph_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define S3D_PHASE_MARK(i) if (threadIdx.x == 0) { const long long now = clock64(); ph_acc[i] += (unsigned long long)(now - ph_t); ph_t = now; }
#define S3D_PHASE_FLUSH(base) if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) atomicAdd(&g_phase_cycles_bwd[(base) + i], ph_acc[i]); }
#else
#define S3D_KEEP(i) true
#define S3D_PHASE_DECL
#define S3D_PHASE_MARK(i)
#define S3D_PHASE_FLUSH(base)
#endif

constexpr int SM_NWARP = 16;
constexpr int SM_THREADS = SM_NWARP * 32;

struct SmallSmem {
    int R16, Rp;
    int off_pq, off_db, off_hq, off_hv, off_pk, off_e, off_rows, off_c, off_misc, total;
};

__host__ __device__ inline SmallSmem make_small_layout(int R)
{
    SmallSmem L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    const int lane_arr = L.R16 * QT * 4;
    int off = 0;
    L.off_pq = off; off += lane_arr;                               // P_q, later histK
    L.off_db = off; off += lane_arr > 38912 ? lane_arr : 38912;    // dB, later the 38 KB reduction buffer
    L.off_hq = off; off += lane_arr;
    L.off_hv = off; off += lane_arr;
    L.off_pk = off; off += 32 * L.Rp * 4;
    L.off_e = off; off += 32 * ES * 16;
    L.off_rows = off; off += 4 * 32 * 16 * 2;                      // Q, K, V, dO rows of the window
    L.off_c = off; off += 32 * 12 * 4;
    L.off_misc = off; off += 1024;
    L.total = off;
    return L;
}

struct SmallParams {
    const __half *q, *k, *v, *dout, *o;
    const float *lse;
    const __half *tq, *tk, *tv;
    __half *dq, *dk, *dv;
    float *dtq, *dtk, *dtv;
    const int32_t *w_sizes, *w2n, *n2n;
    const float *n_coords;
    int64_t W;
    int H;
};

template <int D, int NPU /*projection + dT units per warp*/, int NHU /*hist.T units per warp*/, bool HD16>
__global__ void __launch_bounds__(SM_THREADS, 1)
attn_bwd_small_kernel(const SmallParams P, const CrseMeta meta)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const SmallSmem L = make_small_layout(meta.R);
    uint32_t *s_pq = reinterpret_cast<uint32_t *>(smem + L.off_pq);
    uint32_t *s_db = reinterpret_cast<uint32_t *>(smem + L.off_db);
    uint32_t *s_hq = reinterpret_cast<uint32_t *>(smem + L.off_hq);
    uint32_t *s_hv = reinterpret_cast<uint32_t *>(smem + L.off_hv);
    uint32_t *s_hk = s_pq;                                              // histK reuses P_q
    uint32_t *s_pk = reinterpret_cast<uint32_t *>(smem + L.off_pk);
    uint4 *s_e = reinterpret_cast<uint4 *>(smem + L.off_e);             // [32][ES]
    __half *s_q = reinterpret_cast<__half *>(smem + L.off_rows);        // [32][16] each
    __half *s_k = s_q + 512, *s_v = s_q + 1024, *s_do = s_q + 1536;
    float *s_c = reinterpret_cast<float *>(smem + L.off_c);             // [32][12]
    float *s_lse = reinterpret_cast<float *>(smem + L.off_misc);        // [32][2]
    float *s_del = s_lse + 64;                                          // [32][2]
    int *s_row = reinterpret_cast<int *>(s_del + 64);                   // [32]
    float *s_red = reinterpret_cast<float *>(smem + L.off_db);          // [16][32][16]  (dB is dead by then)
    float *s_red_dk = s_red + SM_NWARP * 512;                           // [32][16]
    float *s_red_dv = s_red_dk + 512;                                   // [32][16]
    float *s_red_dq = s_red_dv + 512;                                   // [32][16]

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int hp = blockIdx.y, H = P.H;
    // head_dim 16: the block serves head hp; its two 8-channel halves stand in for the two heads
    const int HC = H * (HD16 ? 16 : 8), co = hp * 16;
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // ---- units of this warp: (table, row tile) for projections and table gradients -----------------
    // unit u = wid + 16 i ; table = u / n_mt (0: Tq with Q, 1: Tv with dO, 2: Tk with K), tile = u % n_mt
    uint32_t ta[NPU][2][2];
    float dt_acc[NPU][2][4];
#pragma unroll
    for (int i = 0; i < NPU; ++i) {
        const int u = wid + SM_NWARP * i;
        const int tab = u / n_mt, mt = u - tab * n_mt;
        const __half *T = tab == 0 ? P.tq : (tab == 1 ? P.tv : P.tk);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r0 = table_row(meta, mt * 16 + g), r1 = table_row(meta, mt * 16 + g + 8);
            const bool ok = tab < 3;
            ta[i][h][0] = (ok && r0 >= 0) ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r0 * HC + co + h * 8 + 2 * t) : 0u;
            ta[i][h][1] = (ok && r1 >= 0) ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r1 * HC + co + h * 8 + 2 * t) : 0u;
            dt_acc[i][h][0] = dt_acc[i][h][1] = dt_acc[i][h][2] = dt_acc[i][h][3] = 0.f;
        }
    }
    // hist.T units: v = wid + 16 i ; side = v / n_mt (0: histQ.Tq -> dQ, 1: histK.Tk -> dK), k-step = v % n_mt
    uint32_t tb[NHU][2][2];
#pragma unroll
    for (int i = 0; i < NHU; ++i) {
        const int v = wid + SM_NWARP * i;
        const int side = v / n_mt, ks = v - side * n_mt;
        const __half *T = side == 0 ? P.tq : P.tk;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int ra = table_row(meta, ks * 16 + ht_krow(t, half, 0)), rb = table_row(meta, ks * 16 + ht_krow(t, half, 1));
                const bool ok = side < 2;
                const __half lo = (ok && ra >= 0) ? T[(int64_t)ra * HC + co + h * 8 + g] : __float2half(0.f);
                const __half hi = (ok && rb >= 0) ? T[(int64_t)rb * HC + co + h * 8 + g] : __float2half(0.f);
                tb[i][h][half] = h2_as_u32(__halves2half2(lo, hi));
            }
    }

    S3D_PHASE_DECL
#ifdef S3D_PHASE_CLOCK
    const unsigned ablate = g_ablate_bwd;
#endif
    for (int64_t w = blockIdx.x; w < P.W; w += gridDim.x) {
        const int n = __ldg(P.w_sizes + w);
        if (n > QT) continue;                       // larger windows: two-sweep kernels
        const int base = __ldg(P.w2n + w);
        __syncthreads();
        S3D_PHASE_MARK(0)
        // ---- stage the window: Q, K, V, dO rows, delta, lse, coordinates; clear the histograms ----------
        float cx[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            cx[d] = lane < n ? __ldg(P.n_coords + (int64_t)(base + lane) * D + d) : 0.f;
            if (wid == 0) s_c[lane * 12 + d] = cx[d];
        }
        // the global loads are issued first and consumed after the histograms have been cleared, so
        // that their latency overlaps the clearing
        const int st_i = tid >> 3, st_arr = (tid >> 1) & 3, st_hf = tid & 1;
        const bool st_act = tid < 256 && st_i < n;
        uint4 st_val = make_uint4(0, 0, 0, 0), st_o = make_uint4(0, 0, 0, 0);
        float st_lse = 0.f;
        int st_row = 0;
        if (st_act) {
            st_row = __ldg(P.n2n + base + st_i);
            const __half *src = st_arr == 0 ? P.q : (st_arr == 1 ? P.k : (st_arr == 2 ? P.v : P.dout));
            st_val = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)st_row * HC + co + st_hf * 8));
            if (st_arr == 3) {
                st_o = __ldg(reinterpret_cast<const uint4 *>(P.o + (int64_t)st_row * HC + co + st_hf * 8));
                st_lse = __ldg(P.lse + (int64_t)st_row * H + (HD16 ? hp : 2 * hp + st_hf));
            }
        }
        for (int i = tid; i < 2 * L.R16 * QT / 4; i += SM_THREADS)
            reinterpret_cast<uint4 *>(s_hq)[i] = make_uint4(0, 0, 0, 0);     // histQ and histV are adjacent
        if (tid < 256) {
            if (st_act && st_arr == 0 && st_hf == 0) s_row[st_i] = st_row;
            if (st_arr == 3) {
                const __half2 *a2 = reinterpret_cast<const __half2 *>(&st_val);
                const __half2 *b2 = reinterpret_cast<const __half2 *>(&st_o);
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float2 fa = __half22float2(a2[c]), fb = __half22float2(b2[c]);
                    acc += fa.x * fb.x + fa.y * fb.y;
                }
                s_del[st_i * 2 + st_hf] = acc;         // zero beyond the window (both rows are zero there)
                s_lse[st_i * 2 + st_hf] = st_lse;
            }
            *reinterpret_cast<uint4 *>(s_q + st_arr * 512 + st_i * 16 + st_hf * 8) = st_val;
        }
        __syncthreads();
        S3D_PHASE_MARK(1)
        const float xlse0 = s_lse[lane * 2], xlse1 = s_lse[lane * 2 + 1];
        float xdel0 = s_del[lane * 2], xdel1 = s_del[lane * 2 + 1];
        if (HD16) xdel0 = xdel1 = xdel0 + xdel1;   // delta of the whole head
        // ---- projections P_q, dB (lane-major), P_k (tile-major); S0 = K.Q^T and dPV0 = V.dO^T ---------------
#pragma unroll
        for (int i = 0; i < NPU; ++i) {
            const int u = wid + SM_NWARP * i;
            const int tab = u / n_mt, mt = u - tab * n_mt;
            if (!S3D_KEEP(0)) continue;
            if (tab == 0) project_unit<true>(ta[i], s_q, s_pq, mt, Rp, n, g, t);
            else if (tab == 1) project_unit<true>(ta[i], s_do, s_db, mt, Rp, n, g, t);
            else if (tab == 2) project_unit<false>(ta[i], s_k, s_pk, mt, Rp, n, g, t);
        }
        {
            const int mt = wid >> 3, j = wid & 7;     // key rows 16mt.., query columns 4j..
            if (16 * mt < n && 4 * j < n && S3D_KEEP(1)) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    const __half *ysrc = (a == 0 ? s_k : s_v) + mt * 256;
                    const __half *xsrc = a == 0 ? s_q : s_do;
                    const uint32_t wv = *reinterpret_cast<const uint32_t *>(xsrc + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                    const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 2 * t);
                    const uint32_t a1 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 2 * t);
                    const uint32_t a2 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 8 + 2 * t);
                    const uint32_t a3 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 8 + 2 * t);
                    float c[4];
                    mma_k16_z(c, a0, a1, a2, a3, (g & 1) ? 0u : wv, (g & 1) ? wv : 0u);
                    float *e0 = reinterpret_cast<float *>(s_e + (16 * mt + g) * ES + 4 * j + t) + 2 * a;
                    float *e1 = reinterpret_cast<float *>(s_e + (16 * mt + g + 8) * ES + 4 * j + t) + 2 * a;
                    *reinterpret_cast<float2 *>(e0) = make_float2(c[0], c[1]);
                    *reinterpret_cast<float2 *>(e1) = make_float2(c[2], c[3]);
                }
            }
        }
        __syncthreads();
        S3D_PHASE_MARK(2)
        // ---- phase 1: two keys per warp, lane = query -----------------------------------------------------
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
            const int kk = 2 * wid + k2;
            uint4 ent = make_uint4(0u, 0u, 0u, 0u);
            if (kk < n && S3D_KEEP(2)) {
                __half2 b0 = __float2half2_rn(0.f), b1 = b0, b2 = b0;
                uint32_t w0 = 0, w1 = 0;
                float ckv[D];
                load_coords12<D>(s_c + kk * 12, ckv);
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int idx = crse_index_fast(cx[d], ckv[d], meta.L[d], d == D - 1);
                    const int row = meta.rowbase[d] + idx;
                    b0 = __hadd2(b0, u32_as_h2(s_pq[row * QT + mypos]));
                    b1 = __hadd2(b1, u32_as_h2(s_pk[kk * Rp + row]));
                    b2 = __hadd2(b2, u32_as_h2(s_db[row * QT + mypos]));
                    if (d < 5) w0 |= (uint32_t)idx << (IDX_BITS * d);
                    else w1 |= (uint32_t)idx << (IDX_BITS * (d - 5));
                }
                const float4 in = *reinterpret_cast<const float4 *>(s_e + kk * ES + lane);   // S0 (h0,h1), dPV0 (h0,h1)
                const float2 bs = __half22float2(__hadd2(b0, b1));
                const float2 bd = __half22float2(b2);
                float sc0 = in.x + bs.x, sc1 = in.y + bs.y, dq0 = in.z + bd.x, dq1 = in.w + bd.y;
                if (HD16) { sc0 = sc1 = sc0 + sc1; dq0 = dq1 = dq0 + dq1; }   // halves of one head add up
                float p0 = exp2f((sc0 - xlse0) * LOG2E);
                float p1 = exp2f((sc1 - xlse1) * LOG2E);
                float ds0 = p0 * (dq0 - xdel0);
                float ds1 = p1 * (dq1 - xdel1);
                if (lane >= n) { p0 = 0.f; p1 = 0.f; ds0 = 0.f; ds1 = 0.f; }
                ent.x = h2_as_u32(__floats2half2_rn(p0, p1));
                ent.y = h2_as_u32(__floats2half2_rn(ds0, ds1));
                ent.z = w0;
                ent.w = w1;
            }
            s_e[kk * ES + lane] = ent;
        }
        __syncthreads();
        S3D_PHASE_MARK(3)
        // ---- phase 2 (lanes = queries): histQ += ds, histV += p ; warps 13-15: dK, dV, dQ pair GEMMs ----------
        if (wid < D && S3D_KEEP(3)) {
            const int d = wid;
            const int sh = IDX_BITS * (d % 5);
            const int rb = meta.rowbase[d];
            uint32_t *cell = s_hq + mypos;
            for (int k4 = 0; k4 < n; k4 += 4) {
                uint32_t vals[2][4];
                int off[1][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 e = s_e[(k4 + j) * ES + lane];        // zero entries beyond the window
                    vals[0][j] = e.y;
                    vals[1][j] = e.x;
                    const int idx = ((d < 5 ? e.z : e.w) >> sh) & ((1 << IDX_BITS) - 1);
                    off[0][j] = (rb + idx) * QT;
                }
                hist_add4<1, 2>(cell, L.R16 * QT, off, vals, n - k4);
            }
        }
        float pg[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 2; ++i) pg[h][i][0] = pg[h][i][1] = pg[h][i][2] = pg[h][i][3] = 0.f;
        if (!S3D_KEEP(4)) {}
        else if (wid == 15) pair_gemm<1, false>(pg, s_e, s_k, n, g, t);        // dQ[q] += sum_k ds K[k]
        else if (wid == 14) pair_gemm<0, true>(pg, s_e, s_do, n, g, t);   // dV[k] += sum_q p  dO[q]
        else if (wid == 13) pair_gemm<1, true>(pg, s_e, s_q, n, g, t);    // dK[k] += sum_q ds Q[q]
        __syncthreads();
        S3D_PHASE_MARK(4)
        // ---- query side: dTq, dTv ; dQ partials ; clear histK (= P_q storage) ------------------------------------
#pragma unroll
        for (int i = 0; i < NPU; ++i) {
            const int u = wid + SM_NWARP * i;
            const int tab = u / n_mt, mt = u - tab * n_mt;
            if (!S3D_KEEP(5)) continue;
            if (tab == 0) dt_unit(dt_acc[i], s_hq, s_q, mt, g, t);
            else if (tab == 1) dt_unit(dt_acc[i], s_hv, s_do, mt, g, t);
        }
        float part[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 2; ++i) part[h][i][0] = part[h][i][1] = part[h][i][2] = part[h][i][3] = 0.f;
#pragma unroll
        for (int i = 0; i < NHU; ++i) {
            const int v = wid + SM_NWARP * i;
            if (v < n_mt && S3D_KEEP(6)) ht_unit(part, s_hq, tb[i], v, g, t);
        }
        for (int i = tid; i < L.R16 * QT / 4; i += SM_THREADS)
            reinterpret_cast<uint4 *>(s_hk)[i] = make_uint4(0, 0, 0, 0);
        store_part(s_red + wid * 512, part, g, t);            // dB (aliased by s_red) is dead since phase 1
        if (wid == 15) store_part(s_red_dq, pg, g, t);
        else if (wid == 14) store_part(s_red_dv, pg, g, t);
        else if (wid == 13) store_part(s_red_dk, pg, g, t);
        __syncthreads();
        S3D_PHASE_MARK(5)
        {
            const int xx = tid >> 4, ch = tid & 15;
            if (xx < n) {
                float a = s_red_dq[xx * 16 + ch];
#pragma unroll
                for (int ww = 0; ww < SM_NWARP; ++ww) a += s_red[ww * 512 + xx * 16 + ch];
                const int64_t row = s_row[xx];
                P.dq[row * HC + co + ch] = __float2half_rn(a);
                P.dv[row * HC + co + ch] = __float2half_rn(s_red_dv[xx * 16 + ch]);
            }
        }
        // ---- key side (lanes = keys): histK += ds, read column-wise from the pair array --------------------------
        if (wid < D && S3D_KEEP(7)) {
            const int d = wid;
            const int sh = IDX_BITS * (d % 5);
            const int rb = meta.rowbase[d];
            uint32_t *cell = s_hk + mypos;
            for (int q4 = 0; q4 < n; q4 += 4) {
                uint32_t vals[1][4];
                int off[1][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool ok = q4 + j < n && lane < n;
                    const uint4 e = s_e[lane * ES + min(q4 + j, QT - 1)];
                    vals[0][j] = ok ? e.y : 0u;
                    const int idx = ok ? ((d < 5 ? e.z : e.w) >> sh) & ((1 << IDX_BITS) - 1) : 0;
                    off[0][j] = (rb + idx) * QT;
                }
                hist_add4<1, 1>(cell, 0, off, vals, n - q4);
            }
        }
        __syncthreads();
        S3D_PHASE_MARK(6)
        // ---- dTk ; dK partials ---------------------------------------------------------------------------------------
#pragma unroll
        for (int i = 0; i < NPU; ++i) {
            const int u = wid + SM_NWARP * i;
            const int tab = u / n_mt, mt = u - tab * n_mt;
            if (tab == 2 && S3D_KEEP(5)) dt_unit(dt_acc[i], s_hk, s_k, mt, g, t);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 2; ++i) part[h][i][0] = part[h][i][1] = part[h][i][2] = part[h][i][3] = 0.f;
#pragma unroll
        for (int i = 0; i < NHU; ++i) {
            const int v = wid + SM_NWARP * i;
            if (v >= n_mt && v < 2 * n_mt && S3D_KEEP(6)) ht_unit(part, s_hk, tb[i], v - n_mt, g, t);
        }
        store_part(s_red + wid * 512, part, g, t);            // the previous contents were consumed before the last barrier
        __syncthreads();
        S3D_PHASE_MARK(7)
        {
            const int xx = tid >> 4, ch = tid & 15;
            if (xx < n) {
                float a = s_red_dk[xx * 16 + ch];
#pragma unroll
                for (int ww = 0; ww < SM_NWARP; ++ww) a += s_red[ww * 512 + xx * 16 + ch];
                P.dk[(int64_t)s_row[xx] * HC + co + ch] = __float2half_rn(a);
            }
        }
    }  // windows
    S3D_PHASE_FLUSH(0)

    // ---- flush the table gradients of this block ---------------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < NPU; ++i) {
        const int u = wid + SM_NWARP * i;
        const int tab = u / n_mt, mt = u - tab * n_mt;
        if (tab < 3) {
            float *dst = tab == 0 ? P.dtq : (tab == 1 ? P.dtv : P.dtk);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = table_row(meta, mt * 16 + g + 8 * rr);   // aliases flush into the row they stand for
                    if (row >= 0) {
                        float *p = dst + (int64_t)row * HC + co + h * 8 + 2 * t;
                        atomicAdd(p, dt_acc[i][h][2 * rr]);
                        atomicAdd(p + 1, dt_acc[i][h][2 * rr + 1]);
                    }
                }
        }
    }
}

template <int D, int NPU, int NHU, bool HD16>
static int launch_small(const SmallParams &p, const CrseMeta &meta, cudaStream_t st)
{
    const SmallSmem L = make_small_layout(meta.R);
    auto kern = attn_bwd_small_kernel<D, NPU, NHU, HD16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int hp = HD16 ? p.H : p.H / 2;
    int gx = sms / hp;
    if (gx > p.W) gx = (int)p.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, SM_THREADS, L.total, st>>>(p, meta);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

}  // namespace tc

#ifdef S3D_PHASE_CLOCK
extern "C" int s3d_debug_set_ablate_bwd(unsigned int mask)
{
    return cudaMemcpyToSymbol(tc::g_ablate_bwd, &mask, sizeof(mask)) == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

extern "C" int s3d_debug_phase_cycles_bwd(unsigned long long *out16, int reset)
{
    if (cudaMemcpyFromSymbol(out16, tc::g_phase_cycles_bwd, sizeof(unsigned long long) * 16) != cudaSuccess) return S3D_ERR_LAUNCH;
    if (reset) {
        unsigned long long z[16] = {0};
        if (cudaMemcpyToSymbol(tc::g_phase_cycles_bwd, z, sizeof(z)) != cudaSuccess) return S3D_ERR_LAUNCH;
    }
    return S3D_OK;
}
#endif

bool attn_tc_bwd_small_supported(const AttnArgs &a)
{
    if (a.dtype != S3D_F16) return false;
    if (!(a.hd == 16 || (a.hd == 8 && !(a.H & 1)))) return false;
    const int Rint = a.meta.R + a.meta.D - 1;
    const int n_mt = (Rint + 15) / 16;
    if (3 * n_mt > 5 * tc::SM_NWARP) return false;
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;
    return tc::make_small_layout(Rint).total <= 227 * 1024;
}

// Windows of at most 32 voxels; dtq, dtk, dtv must be zero on entry (accumulated into).
int attn_tc_backward_small(const AttnArgs &a0, cudaStream_t st)
{
    if (a0.W == 0) return S3D_OK;
    AttnArgs a = a0;
    a.meta = tc::internal_meta(a0.meta);   // kernels work in the internal row numbering
    tc::SmallParams p{};
    p.q = (const __half *)a.q; p.k = (const __half *)a.k; p.v = (const __half *)a.v;
    p.dout = (const __half *)a.dout; p.o = (const __half *)a.out; p.lse = a.lse;
    p.tq = (const __half *)a.tq; p.tk = (const __half *)a.tk; p.tv = (const __half *)a.tv;
    p.dq = (__half *)a.dq; p.dk = (__half *)a.dk; p.dv = (__half *)a.dv;
    p.dtq = a.dtq; p.dtk = a.dtk; p.dtv = a.dtv;
    p.w_sizes = a.w_sizes; p.w2n = a.w2n; p.n2n = a.n2n; p.n_coords = a.n_coords;
    p.W = a.W; p.H = a.H;
    const int n_mt = (a.meta.R + 15) / 16;
    const int npu = (3 * n_mt + tc::SM_NWARP - 1) / tc::SM_NWARP;   // <= 5
    const int nhu = (2 * n_mt + tc::SM_NWARP - 1) / tc::SM_NWARP;   // <= 3
#define S3D_SMALL(DD)                                                                   \
    if (a.hd == 16) {                                                                   \
        if (npu <= 2 && nhu <= 1) return tc::launch_small<DD, 2, 1, true>(p, a.meta, st);  \
        if (npu <= 3 && nhu <= 2) return tc::launch_small<DD, 3, 2, true>(p, a.meta, st);  \
        if (npu <= 4 && nhu <= 3) return tc::launch_small<DD, 4, 3, true>(p, a.meta, st);  \
        return tc::launch_small<DD, 5, 3, true>(p, a.meta, st);                          \
    }                                                                                   \
    if (npu <= 2 && nhu <= 1) return tc::launch_small<DD, 2, 1, false>(p, a.meta, st);  \
    if (npu <= 3 && nhu <= 2) return tc::launch_small<DD, 3, 2, false>(p, a.meta, st);  \
    if (npu <= 4 && nhu <= 3) return tc::launch_small<DD, 4, 3, false>(p, a.meta, st);  \
    return tc::launch_small<DD, 5, 3, false>(p, a.meta, st);
    switch (a.meta.D) {
        case 3: S3D_SMALL(3)
        case 6: S3D_SMALL(6)
        case 9: S3D_SMALL(9)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_SMALL
}

}  // namespace s3d
