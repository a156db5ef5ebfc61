// Backward of the cRSE window attention, tensor-core path (fp16 storage), for windows of any size:
// ONE sweep over the pairs instead of a query sweep plus a key sweep.
//
// A window of n voxels is cut into nt = ceil(n / 32) tiles of equal size (at most 32 voxels) and the
// work item is a tile pair (query tile i, key tile j): since p = exp(s - lse) needs nothing from the
// other key tiles, every tile pair is an independent 32 x 32 problem that adds its share to dQ of
// tile i, to dK and dV of tile j and to the table gradients.  The nt^2 items of a window run one after
// the other in the same block (j inner), and a share that is not the first one is added to the rows
// already written (read-modify-write of the fp16 rows in global memory by the block that wrote them).
// Windows of at most 32 voxels -- most of them -- are a single item.
//
// Block = 15 / 11 / 7 consumer warps (9 / 6 / 3 signal dimensions) + one producer warp, one block per SM, serving one head pair
// (head_dim 8) or one head (head_dim 16) for the windows x, x + gridDim.x, ...  The producer walks
// the block's items ahead of the consumers: row numbers, coordinates, lse and delta = dO.O by plain
// loads, the 32-byte Q, dO pieces of the query tile and K, V pieces of the key tile by the copy
// engine (cp.async.bulk) into the next stage of shared memory; stages are handed over through
// "full" / "empty" mbarriers.
// Per window (consumers, phases separated by a barrier among the consumer warps):
//   GEMM    P_q = Tq.Q^T, dB = Tv.dO^T (lane-major), P_k = Tk.K^T (key-major); a warp owns consecutive
//           (table, row tile) units, so it builds the B fragments of a feature array once per
//           table; S0 = K.Q^T, dPV0 = V.dO^T                                        [tensor cores]
//   scores  lane = query, keys dealt to the warps: D indices, 3*D look-ups, p = exp(s - lse),
//           ds = p (dP - delta); written to four [key][query] planes (p, ds, idx 0-4, idx 5-8) with
//           a row stride of 33, readable conflict-free by rows and by columns
//   clear   the three histograms (they reuse the storage of P_q, dB, P_k)
//   hist    warps 0..D-1: histQ += ds, histV += p for their dimension (lanes = queries);
//           the next (D+1)/2 warps: histK += ds for two dimensions each (lanes = keys, planes read
//           column-wise); one warp: dQ += dS.K, dK += dS^T.Q; one: dV = P^T.dO      [tensor cores]
//   GEMM    dTq += histQ^T.Q, dTv += histV^T.dO, dTk += histK^T.K (accumulated in registers over
//           all windows of the block), dQ += histQ.Tq, dK += histK.Tk                [tensor cores]
//   store   reduce the partial dQ, dK over the warps, write dQ, dK, dV
// grid = (x, H/2) or (x, H).
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"
#include "async_stage.cuh"

namespace s3d {
namespace tc {

// Debug build only (-DS3D_PHASE_CLOCK): cycles between the barriers of a window, summed over all
// windows and blocks (s3d_debug_phase_cycles_bwd), and switches that skip pieces of the kernel so
// that their cost can be measured (results are then wrong).  Compiled out otherwise.
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

constexpr int BS_STAGES = 2;

// Consumer warps per block: D for the query-side histograms, (D+1)/2 for the key side, one or two
// for the pair GEMMs, rounded so that consumers + producer fill whole groups of four warps (the
// register file is split over the four schedulers of an SM).
__host__ __device__ constexpr int bwd_small_warps(int D) { return D == 9 ? 15 : (D == 6 ? 11 : 7); }

struct SmallSmem {
    int R16, Rp;
    int off_pq, off_db, off_pk, off_s0, off_pl, off_rows, off_c, off_pg, off_ta, off_tb, off_lut, off_misc, total;
};

__host__ __device__ inline SmallSmem make_small_layout(int R, int nw, int lut_entries)
{
    SmallSmem L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    const int lane_arr = L.R16 * QT * 4;
    int off = 0;
    L.off_pq = off; off += lane_arr;                               // P_q, later histQ
    L.off_db = off; off += lane_arr;                               // dB, later histV
    const int pk = 32 * L.Rp * 4;
    L.off_pk = off; off += pk > lane_arr ? pk : lane_arr;          // P_k, later histK
    // S0/dPV0 and the planes are dead once the histograms exist; the partial dQ and dK of the hist.T
    // warps (2 * (nw/2) * 2 KB) are written over them
    const int part = 2 * (nw / 2) * 2048, s0pl = 32 * ES * 16 + 4 * 32 * ES * 4;
    L.off_s0 = off; off += 32 * ES * 16;                           // S0 and dPV0 of every pair
    L.off_pl = off; off += 4 * 32 * ES * 4;                        // planes p, ds, idx 0-4, idx 5-8
    if (part > s0pl) off += part - s0pl;
    L.off_rows = off; off += BS_STAGES * 4 * 32 * 16 * 2;          // Q, dO (query tile), K, V (key tile) rows, per stage
    L.off_c = off; off += BS_STAGES * 2 * 32 * 12 * 4;             // coordinates of the query and of the key tile
    L.off_pg = off; off += 3 * 2048;                               // dQ, dV, dK of the pair GEMMs
    L.off_ta = off; off += 3 * (L.R16 / 16) * 512;                 // Tq, Tv, Tk as A fragments of the projections
    L.off_tb = off; off += 2 * (L.R16 / 16) * 512;                 // Tq and Tk as B fragments of the hist.T products
    L.off_lut = off; off += (lut_entries * 2 + 15) / 16 * 16;      // index -> internal row, per dimension
    L.off_misc = off; off += 2048;
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

// The other GPUs' dq, dk, dv arrays of a split step (a kernel parameter of its own, after the others).
struct BwdMirrors {
    Mirrors dq, dk, dv;
};

// Set when a bounded wait of a kernel in this file ran out (it never should).
__device__ int g_bwd_small_async_error;

template <int D, int NPU /*projection + dT units per warp*/, int NHU /*hist.T units per warp*/, bool HD16,
          bool MIRROR /*also store the rows to other GPUs' arrays*/>
__global__ void __launch_bounds__((bwd_small_warps(D) + 1) * 32, 1)
attn_bwd_small_kernel(const SmallParams P, const PermMeta pm, const PairConsts pc, const __grid_constant__ BwdMirrors MM)
{
    constexpr int NW = bwd_small_warps(D);       // consumer warps
    constexpr int NT = NW * 32;
    constexpr int TG = NW / 3;                   // warps per table (projection and table-gradient units)
    constexpr int NKW = (D + 1) / 2;             // warps of the key-side histogram, two dimensions each
    constexpr int GEMM_WARP = D + NKW;           // dQ and dK pair GEMMs
    constexpr int DV_WARP = (D & 1) ? D + NKW - 1 : D + NKW + 1;   // dV: the key-side warp with one dimension, or a spare one
    static_assert(DV_WARP < NW && GEMM_WARP < NW, "not enough warps");
    constexpr int SG = NW / 2;                   // warps per hist.T side
    constexpr int KPW = (QT + NW - 1) / NW;      // keys per warp in the score phase
    extern __shared__ __align__(16) unsigned char smem[];
    const SmallSmem L = make_small_layout(pm.R, NW, pm.D * pm.lut_stride);
    uint32_t *s_pq = reinterpret_cast<uint32_t *>(smem + L.off_pq);
    uint32_t *s_db = reinterpret_cast<uint32_t *>(smem + L.off_db);
    uint32_t *s_pk = reinterpret_cast<uint32_t *>(smem + L.off_pk);
    uint32_t *s_hq = s_pq, *s_hv = s_db, *s_hk = s_pk;                  // the histograms reuse the projections
    float4 *s_s0 = reinterpret_cast<float4 *>(smem + L.off_s0);         // [32][ES] (S0 h0, S0 h1, dPV0 h0, dPV0 h1)
    uint32_t *s_P = reinterpret_cast<uint32_t *>(smem + L.off_pl);      // [32][ES] half2 p
    uint32_t *s_DS = s_P + 32 * ES, *s_W0 = s_DS + 32 * ES, *s_W1 = s_W0 + 32 * ES;
    __half *s_rows = reinterpret_cast<__half *>(smem + L.off_rows);     // [stage][Q,dO,K,V][32][16]
    float *s_cs = reinterpret_cast<float *>(smem + L.off_c);            // [stage][query tile, key tile][32][12]
    float *s_part = reinterpret_cast<float *>(smem + L.off_s0);         // [2][SG][32][16], over S0 and the planes
    uint4 *s_ta = reinterpret_cast<uint4 *>(smem + L.off_ta);           // [Tq, Tv, Tk][row tile][lane]
    float *s_pg = reinterpret_cast<float *>(smem + L.off_pg);           // [3][32][16]
    uint4 *s_tb = reinterpret_cast<uint4 *>(smem + L.off_tb);           // [Tq, Tk][k-step][lane]
    uint16_t *s_lut = reinterpret_cast<uint16_t *>(smem + L.off_lut);   // [dimension][index] -> internal row
    float *s_lses = reinterpret_cast<float *>(smem + L.off_misc);       // [stage][32][2]
    float *s_dels = s_lses + BS_STAGES * 64;                            // [stage][32][2]
    int *s_rowi = reinterpret_cast<int *>(s_dels + BS_STAGES * 64);     // [stage][query tile, key tile][32]
    int *s_n = s_rowi + BS_STAGES * 64;                                 // [stage][8]: nq, nk, j > 0, i > 0, used tiles ; nq = 0: no more items
    int *s_fail = s_n + BS_STAGES * 8;
    uint64_t *s_full = reinterpret_cast<uint64_t *>(smem + L.off_misc + 1792);   // [stage]
    uint64_t *s_empty = s_full + BS_STAGES;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int hp = blockIdx.y, H = P.H;
    // head_dim 16: the block serves head hp; its two 8-channel halves stand in for the two heads
    const int HC = H * (HD16 ? 16 : 8), co = hp * 16;

    if (tid == 0) {
        for (int s = 0; s < BS_STAGES; ++s) {
            mbar_init(s_full + s, 1);
            mbar_init(s_empty + s, NW);
        }
        *s_fail = 0;
        mbar_init_fence();
    }
    fill_perm_lut(s_lut, pm, tid, blockDim.x);
    // ---- this block's windows: a contiguous range of equal cost --------------------------------------------------
    // cost of a window = its number of tile pairs; every block scans all window sizes (a few hundred KB
    // from L2) and takes the range whose cumulative cost falls into its share, so the assignment is
    // balanced to within one window, needs no global counter and is the same on every run.
    {
        constexpr int NTA = (NW + 1) * 32;
        int64_t *s_seg = reinterpret_cast<int64_t *>(smem + L.off_pq);     // [NTA + 1] segment sums, then their exclusive scan
        int64_t *s_range = s_seg + NTA + 2;                                // [2] first window, one past the last
        const int64_t per = (P.W + NTA - 1) / NTA;
        const int64_t w0 = (int64_t)tid * per, w1 = w0 + per < P.W ? w0 + per : P.W;
        int64_t sum = 0;
        for (int64_t w = w0; w < w1; ++w) {
            const int nt = (__ldg(P.w_sizes + w) + QT - 1) / QT;
            sum += (int64_t)nt * nt;
        }
        s_seg[tid] = sum;
        __syncthreads();
        if (wid == 0) {                       // exclusive scan of the NTA segment sums by one warp
            int64_t carry = 0;
            for (int b0 = 0; b0 < NTA; b0 += 32) {
                const int64_t v = s_seg[b0 + lane];
                int64_t x = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int64_t y = __shfl_up_sync(0xffffffffu, x, o);
                    if (lane >= o) x += y;
                }
                s_seg[b0 + lane] = carry + x - v;
                carry += __shfl_sync(0xffffffffu, x, 31);
            }
            if (lane == 0) s_seg[NTA] = carry;
        }
        __syncthreads();
        const int64_t total = s_seg[NTA];
        // window index at which the cumulative cost reaches the target: first w with prefix(w) >= target
        const int64_t lo_t = total * blockIdx.x / gridDim.x, hi_t = total * (blockIdx.x + 1) / gridDim.x;
        const int64_t mine = s_seg[tid], next = tid + 1 < NTA ? s_seg[tid + 1] : total + 1;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int64_t target = k == 0 ? lo_t : hi_t;
            if (target >= total) {
                if (tid == 0) s_range[k] = P.W;
            } else if (mine <= target && target < next && w0 < w1) {
                int64_t acc = mine, w = w0;
                for (; w < w1; ++w) {
                    if (acc >= target) break;
                    const int nt = (__ldg(P.w_sizes + w) + QT - 1) / QT;
                    acc += (int64_t)nt * nt;
                }
                s_range[k] = w;
            }
        }
        __syncthreads();
    }
    const int64_t w_begin = reinterpret_cast<const int64_t *>(smem + L.off_pq)[(NW + 1) * 32 + 2];
    const int64_t w_end = reinterpret_cast<const int64_t *>(smem + L.off_pq)[(NW + 1) * 32 + 3];
    __syncthreads();

    if (wid == NW) {
        // ================================ producer warp ================================================
        // Software-pipelined so that no load is consumed right after it is issued: the sizes of the next
        // window are fetched when a window is opened, the row numbers and coordinates of the next item
        // (indexed by sorted position) at the end of the current iteration, and only lse / dO / O (indexed
        // by the row number) inside the iteration, under the tile-mask arithmetic.
        int64_t w = w_begin - 1;
        int n = 0, base = 0, nt = 0, ts = 0, ti = 0, tj = 0;
        int n_nx = 0, base_nx = 0;                         // sizes of window w + 1
        if (w_begin < w_end) {
            n_nx = __ldg(P.w_sizes + w_begin);
            base_nx = __ldg(P.w2n + w_begin);
        }
        bool have = false;
        int nq = 0, nk = 0, rowq = 0, rowk = 0;
        float cq[D], ck[D];
        // descriptor of the next item and the loads that depend on the sorted position only
        auto advance = [&]() {
            if (have && tj + 1 < nt) {
                ++tj;
            } else if (have && ti + 1 < nt) {
                ++ti;
                tj = 0;
            } else {
                ++w;
                have = w < w_end;
                if (have) {
                    n = n_nx;
                    base = base_nx;
                    if (w + 1 < w_end) {
                        n_nx = __ldg(P.w_sizes + w + 1);
                        base_nx = __ldg(P.w2n + w + 1);
                    }
                    nt = (n + QT - 1) / QT;
                    ts = nt > 0 ? (n + nt - 1) / nt : 0;      // equal tiles of at most QT voxels
                    ti = tj = 0;
                    have = n > 0;
                }
            }
            nq = have ? min(ts, n - ti * ts) : 0;
            nk = have ? min(ts, n - tj * ts) : 0;
            rowq = rowk = 0;
#pragma unroll
            for (int d = 0; d < D; ++d) cq[d] = ck[d] = 0.f;
            if (lane < nq) {
                const int pos = base + ti * ts + lane;
                rowq = __ldg(P.n2n + pos);
#pragma unroll
                for (int d = 0; d < D; ++d) cq[d] = __ldg(P.n_coords + (int64_t)pos * D + d);
            }
            if (lane < nk) {
                const int pos = base + tj * ts + lane;
                rowk = __ldg(P.n2n + pos);
#pragma unroll
                for (int d = 0; d < D; ++d) ck[d] = __ldg(P.n_coords + (int64_t)pos * D + d);
            }
        };
        advance();
        for (int it = 0;; ++it) {
            float ls0 = 0.f, ls1 = 0.f, de0 = 0.f, de1 = 0.f;
            uint4 gdo[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, go[2] = {gdo[0], gdo[0]};
            if (lane < nq) {
                if (HD16) {
                    ls0 = ls1 = __ldg(P.lse + (int64_t)rowq * H + hp);
                } else {
                    ls0 = __ldg(P.lse + (int64_t)rowq * H + 2 * hp);
                    ls1 = __ldg(P.lse + (int64_t)rowq * H + 2 * hp + 1);
                }
                const uint4 *gd = reinterpret_cast<const uint4 *>(P.dout + (int64_t)rowq * HC + co);
                const uint4 *gg = reinterpret_cast<const uint4 *>(P.o + (int64_t)rowq * HC + co);
                gdo[0] = __ldg(gd); gdo[1] = __ldg(gd + 1);
                go[0] = __ldg(gg); go[1] = __ldg(gg + 1);
            }
            // tiles this item can touch: index range of every dimension from the coordinate extrema
            uint32_t used = 0;
            {
                bool odd = false;           // a NaN or infinite coordinate: no range argument, use every tile
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    odd = odd || (lane < nq && !(fabsf(cq[d]) < INFINITY)) || (lane < nk && !(fabsf(ck[d]) < INFINITY));
                    const int kq = float_order_key(cq[d]), kk = float_order_key(ck[d]);
                    const float qmn = float_from_order_key(__reduce_min_sync(0xffffffffu, lane < nq ? kq : 0x7fffffff));
                    const float qmx = float_from_order_key(__reduce_max_sync(0xffffffffu, lane < nq ? kq : (int)0x80000000));
                    const float kmn = float_from_order_key(__reduce_min_sync(0xffffffffu, lane < nk ? kk : 0x7fffffff));
                    const float kmx = float_from_order_key(__reduce_max_sync(0xffffffffu, lane < nk ? kk : (int)0x80000000));
                    const int lo = (int)crse_index_pc(qmn, kmx, pc.half[d], pc.clamp[d]);
                    const int hi = (int)crse_index_pc(qmx, kmn, pc.half[d], pc.clamp[d]);
                    used |= perm_tile_mask_warp(s_lut + d * pm.lut_stride, pm.n[d], lo, hi, lane);
                }
                if (__any_sync(0xffffffffu, odd)) used = 0xffffffffu;
            }
            // delta[slot] = sum_c dO . O over the eight channels of the slot
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const __half2 *a2 = reinterpret_cast<const __half2 *>(&gdo[h]), *b2 = reinterpret_cast<const __half2 *>(&go[h]);
                float acc = 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float2 fa = __half22float2(a2[c]), fb = __half22float2(b2[c]);
                    acc += fa.x * fb.x + fa.y * fb.y;
                }
                if (h == 0) de0 = acc; else de1 = acc;
            }
            const int s = it % BS_STAGES;
            if (it >= BS_STAGES && !mbar_wait(s_empty + s, ((it / BS_STAGES) - 1) & 1)) {
                g_bwd_small_async_error = 1;
                nq = nk = 0;                              // tell the consumers to stop
            }
            __half *rq = s_rows + s * 2048;
            float *cs = s_cs + s * 768;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                cs[lane * 12 + d] = cq[d];
                cs[384 + lane * 12 + d] = ck[d];
            }
            s_rowi[s * 64 + lane] = rowq;
            s_rowi[s * 64 + 32 + lane] = rowk;
            s_lses[s * 64 + lane * 2] = ls0;
            s_lses[s * 64 + lane * 2 + 1] = ls1;
            s_dels[s * 64 + lane * 2] = de0;
            s_dels[s * 64 + lane * 2 + 1] = de1;
#pragma unroll
            for (int a = 0; a < 4; ++a)                   // rows beyond the tiles are zero
                if (lane >= (a < 2 ? nq : nk)) {
                    *reinterpret_cast<uint4 *>(rq + a * 512 + lane * 16) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4 *>(rq + a * 512 + lane * 16 + 8) = make_uint4(0, 0, 0, 0);
                }
            if (lane == 0) {
                s_n[s * 8] = nq;
                s_n[s * 8 + 1] = nk;
                s_n[s * 8 + 2] = tj > 0;
                s_n[s * 8 + 3] = ti > 0;
                s_n[s * 8 + 4] = (int)used;
            }
            async_proxy_fence();
            __syncwarp();
            if (lane == 0) mbar_arrive_expect_tx(s_full + s, (unsigned)((nq + nk) * 64));
            __syncwarp();
            if (lane < nq) {
                const int64_t off = (int64_t)rowq * HC + co;
                bulk_copy_g2s(rq + lane * 16, P.q + off, 32, s_full + s);
                bulk_copy_g2s(rq + 512 + lane * 16, P.dout + off, 32, s_full + s);
            }
            if (lane < nk) {
                const int64_t off = (int64_t)rowk * HC + co;
                bulk_copy_g2s(rq + 1024 + lane * 16, P.k + off, 32, s_full + s);
                bulk_copy_g2s(rq + 1536 + lane * 16, P.v + off, 32, s_full + s);
            }
            if (nq == 0) break;
            advance();                                    // the next item's position-indexed loads fly during the wait above
        }
        return;
    }

    // ==================================== consumer warps ===============================================
    const int g = lane >> 2, t = lane & 3;
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // (table, row tile) units of this warp, for the projections and the table gradients: the warps are
    // split into three groups, one per table -- 0 = Tq with Q (-> P_q, dTq), 1 = Tv with dO (-> dB, dTv),
    // 2 = Tk with K (-> P_k, dTk) -- so a warp builds the B fragments of one feature array only, and
    // the tiles are dealt round-robin inside a group (tile = wsub + TG i), so that the tiles a window
    // leaves out (see PermMeta) thin out every warp's share alike.
    const int tg = wid / TG, wsub = wid - tg * TG;
    // The A fragments of the table slices are built once per block and kept in shared memory (one
    // 16-byte load per unit and window); the table-gradient accumulators stay in registers.
    float dt_acc[NPU][2][4];
#pragma unroll
    for (int i = 0; i < NPU; ++i)
#pragma unroll
        for (int h = 0; h < 2; ++h) dt_acc[i][h][0] = dt_acc[i][h][1] = dt_acc[i][h][2] = dt_acc[i][h][3] = 0.f;
    for (int u = wid; u < 3 * n_mt; u += NW) {
        const int tab = u / n_mt, mt = u - tab * n_mt;
        const __half *T = tab == 0 ? P.tq : (tab == 1 ? P.tv : P.tk);
        const int r0 = perm_table_row(pm, mt * 16 + g), r1 = perm_table_row(pm, mt * 16 + g + 8);
        uint32_t f[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            f[h][0] = r0 >= 0 ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r0 * HC + co + h * 8 + 2 * t) : 0u;
            f[h][1] = r1 >= 0 ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r1 * HC + co + h * 8 + 2 * t) : 0u;
        }
        s_ta[u * 32 + lane] = make_uint4(f[0][0], f[0][1], f[1][0], f[1][1]);
    }
    // hist.T side of this warp: 0 = histQ.Tq -> dQ (warps [0, SG)), 1 = histK.Tk -> dK (warps [SG, 2 SG));
    // its k-steps are ws2 + SG i.  The B fragments of Tq and Tk for these products are built once per
    // block and kept in shared memory (one 16-byte load per unit instead of resident registers).
    const int side = wid / SG, ws2 = wid - side * SG;
    for (int u = wid; u < 2 * n_mt; u += NW) {
        const int sd = u / n_mt, ks = u - sd * n_mt;
        const __half *T = sd == 0 ? P.tq : P.tk;
        uint32_t f[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int ra = perm_table_row(pm, ks * 16 + ht_krow(t, half, 0));
                const int rb = perm_table_row(pm, ks * 16 + ht_krow(t, half, 1));
                const __half lo = ra >= 0 ? T[(int64_t)ra * HC + co + h * 8 + g] : __float2half(0.f);
                const __half hi = rb >= 0 ? T[(int64_t)rb * HC + co + h * 8 + g] : __float2half(0.f);
                f[h][half] = h2_as_u32(__halves2half2(lo, hi));
            }
        s_tb[u * 32 + lane] = make_uint4(f[0][0], f[0][1], f[1][0], f[1][1]);
    }
    S3D_PHASE_DECL
#ifdef S3D_PHASE_CLOCK
    const unsigned ablate = g_ablate_bwd;
#endif
    for (int it = 0;; ++it) {
        const int s = it % BS_STAGES;
        if (!mbar_wait(s_full + s, (it / BS_STAGES) & 1)) {
            *s_fail = 1;
            g_bwd_small_async_error = 2;
        }
        consumer_sync<NT>();          // the previous window's stores are over; the flag is settled
        S3D_PHASE_MARK(0)
        const int nq = s_n[s * 8], nk = s_n[s * 8 + 1];
        const bool add_q = s_n[s * 8 + 2] != 0, add_k = s_n[s * 8 + 3] != 0;   // not the first share of dQ / of dK, dV
        const uint32_t used = (uint32_t)s_n[s * 8 + 4];                        // tiles this item can touch
        if (nq == 0 || *s_fail) break;
        const __half *s_q = s_rows + s * 2048, *s_do = s_q + 512, *s_k = s_q + 1024, *s_v = s_q + 1536;
        const float *s_c = s_cs + s * 768, *s_ck = s_c + 384;
        const int *s_rowq = s_rowi + s * 64, *s_rowk = s_rowq + 32;
        const float *s_lse = s_lses + s * 64, *s_del = s_dels + s * 64;
        float cx[D];
        load_coords12<D>(s_c + lane * 12, cx);
        // ---- projections P_q, dB (lane-major), P_k (key-major); S0 = K.Q^T and dPV0 = V.dO^T -----------------
        if (tg < 3 && S3D_KEEP(0)) {
            uint32_t bf[8][2];
            load_feat_bfrag(bf, tg == 0 ? s_q : (tg == 1 ? s_do : s_k), tg == 2 ? nk : nq, g, t);
#pragma unroll
            for (int i = 0; i < NPU; ++i) {
                const int mt = wsub + TG * i;
                if (mt < n_mt && ((used >> mt) & 1u)) {
                    const uint4 f = s_ta[(tg * n_mt + mt) * 32 + lane];
                    const uint32_t taf[2][2] = {{f.x, f.y}, {f.z, f.w}};
                    if (tg == 0) project_unit_b<true>(taf, bf, s_pq, mt, Rp, nq, g, t);
                    else if (tg == 1) project_unit_b<true>(taf, bf, s_db, mt, Rp, nq, g, t);
                    else project_unit_b<false>(taf, bf, s_pk, mt, Rp, nk, g, t);
                }
            }
        }
        for (int u = wid; u < 32 && S3D_KEEP(1); u += NW) {
            const int a = u >> 4, mt = (u >> 3) & 1, j = u & 7;     // key rows 16mt.., query columns 4j..
            if (16 * mt < nk && 4 * j < nq) {
                const __half *ysrc = (a == 0 ? s_k : s_v) + mt * 256;
                const __half *xsrc = a == 0 ? s_q : s_do;
                const uint32_t wv = *reinterpret_cast<const uint32_t *>(xsrc + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 2 * t);
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 2 * t);
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 8 + 2 * t);
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 8 + 2 * t);
                float c[4];
                mma_k16_z(c, a0, a1, a2, a3, (g & 1) ? 0u : wv, (g & 1) ? wv : 0u);
                float *e0 = reinterpret_cast<float *>(s_s0 + (16 * mt + g) * ES + 4 * j + t) + 2 * a;
                float *e1 = reinterpret_cast<float *>(s_s0 + (16 * mt + g + 8) * ES + 4 * j + t) + 2 * a;
                *reinterpret_cast<float2 *>(e0) = make_float2(c[0], c[1]);
                *reinterpret_cast<float2 *>(e1) = make_float2(c[2], c[3]);
            }
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(1)
        // ---- scores: keys wid, wid + NW ; lane = query -------------------------------------------------------
        {
            const float xlse0 = s_lse[lane * 2] * LOG2E, xlse1 = s_lse[lane * 2 + 1] * LOG2E;
            float xdel0 = s_del[lane * 2], xdel1 = s_del[lane * 2 + 1];
            if (HD16) xdel0 = xdel1 = xdel0 + xdel1;   // delta of the whole head
            const uint32_t *pq_lane = s_pq + mypos, *db_lane = s_db + mypos;
#pragma unroll
            for (int j = 0; j < KPW; ++j) {
                const int kk = wid + NW * j;
                if (kk < QT) {
                    uint32_t pw = 0u, dsw = 0u, w0 = 0u, w1 = 0u;     // zero for keys beyond the window
                    if (kk < nk && S3D_KEEP(2)) {
                        float ck[D];
                        load_coords12<D>(s_ck + kk * 12, ck);
                        const uint32_t *pk_row = s_pk + kk * Rp;
                        __half2 b0 = __float2half2_rn(0.f), b1 = b0, b2 = b0;
#pragma unroll
                        for (int d = 0; d < D; ++d) {
                            const uint32_t idx = crse_index_pc(cx[d], ck[d], pc.half[d], pc.clamp[d]);
                            const uint32_t row = s_lut[d * pm.lut_stride + idx];
                            b0 = __hadd2(b0, u32_as_h2(pq_lane[row * QT]));
                            b1 = __hadd2(b1, u32_as_h2(pk_row[row]));
                            b2 = __hadd2(b2, u32_as_h2(db_lane[row * QT]));
                            if (d < 5) w0 |= idx << (IDX_BITS * d);
                            else w1 |= idx << (IDX_BITS * (d - 5));
                        }
                        const float4 in = s_s0[kk * ES + lane];          // S0 (h0,h1), dPV0 (h0,h1)
                        const float2 bs = __half22float2(__hadd2(b0, b1));
                        const float2 bd = __half22float2(b2);
                        float sc0 = in.x + bs.x, sc1 = in.y + bs.y, dq0 = in.z + bd.x, dq1 = in.w + bd.y;
                        if (HD16) { sc0 = sc1 = sc0 + sc1; dq0 = dq1 = dq0 + dq1; }   // halves of one head add up
                        float p0 = ex2_approx(fmaf(sc0, LOG2E, -xlse0));
                        float p1 = ex2_approx(fmaf(sc1, LOG2E, -xlse1));
                        float ds0 = p0 * (dq0 - xdel0);
                        float ds1 = p1 * (dq1 - xdel1);
                        if (lane >= nq) { p0 = 0.f; p1 = 0.f; ds0 = 0.f; ds1 = 0.f; }
                        pw = h2_as_u32(__floats2half2_rn(p0, p1));
                        dsw = h2_as_u32(__floats2half2_rn(ds0, ds1));
                    }
                    s_P[kk * ES + lane] = pw;
                    s_DS[kk * ES + lane] = dsw;
                    s_W0[kk * ES + lane] = w0;
                    s_W1[kk * ES + lane] = w1;
                }
            }
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(2)
        // ---- clear the three histograms (P_q, dB, P_k are dead) ------------------------------------------------
        for (int i = tid; i < L.R16 * QT / 4; i += NT)                       // 128 16-byte pieces per 16-row tile
            if ((used >> (i >> 7)) & 1u) {
                uint4 *h = reinterpret_cast<uint4 *>(s_hq) + i;              // the three arrays are adjacent
                h[0] = make_uint4(0, 0, 0, 0);
                h[L.R16 * QT / 4] = make_uint4(0, 0, 0, 0);
                h[2 * (L.R16 * QT / 4)] = make_uint4(0, 0, 0, 0);
            }
        consumer_sync<NT>();
        S3D_PHASE_MARK(3)
        // ---- histograms and pair GEMMs ------------------------------------------------------------------------
        if (wid < D) {
            // histQ += ds, histV += p ; lanes = queries, two keys per step
            if (S3D_KEEP(3)) {
                const int d = wid;
                const bool lo = d < 5;
                const int sh = IDX_BITS * (lo ? d : d - 5);
                const uint32_t *pcol = s_P + lane, *dcol = s_DS + lane, *wcol = (lo ? s_W0 : s_W1) + lane;
                const uint16_t *lut = s_lut + d * pm.lut_stride;
                uint32_t *cell = s_hq + mypos;
                const int hv = L.R16 * QT;                 // histV follows histQ
                uint32_t p0 = pcol[0], d0 = dcol[0], x0 = wcol[0];
                uint32_t p1 = pcol[ES], d1 = dcol[ES], x1 = wcol[ES];
                int kk = 0;
                for (; kk + 1 < nk; kk += 2) {
                    const uint32_t i0 = lut[(x0 >> sh) & ((1u << IDX_BITS) - 1u)], i1 = lut[(x1 >> sh) & ((1u << IDX_BITS) - 1u)];
                    uint32_t *a0 = cell + i0 * QT, *a1 = cell + i1 * QT;
                    const uint32_t q0 = a0[0], v0 = a0[hv], q1 = a1[0], v1 = a1[hv];
                    const uint32_t cp0 = p0, cd0 = d0, cp1 = p1, cd1 = d1;
                    const int k2 = min(kk + 2, QT - 1) * ES, k3 = min(kk + 3, QT - 1) * ES;
                    p0 = pcol[k2]; d0 = dcol[k2]; x0 = wcol[k2];
                    p1 = pcol[k3]; d1 = dcol[k3]; x1 = wcol[k3];
                    const bool same = a1 == a0;
                    const __half2 sq0 = __hadd2(u32_as_h2(q0), u32_as_h2(cd0));
                    const __half2 sv0 = __hadd2(u32_as_h2(v0), u32_as_h2(cp0));
                    const __half2 sq1 = __hadd2(same ? sq0 : u32_as_h2(q1), u32_as_h2(cd1));
                    const __half2 sv1 = __hadd2(same ? sv0 : u32_as_h2(v1), u32_as_h2(cp1));
                    a0[0] = h2_as_u32(sq0); a0[hv] = h2_as_u32(sv0);
                    a1[0] = h2_as_u32(sq1); a1[hv] = h2_as_u32(sv1);
                }
                if (kk < nk) {
                    const uint32_t i0 = lut[(x0 >> sh) & ((1u << IDX_BITS) - 1u)];
                    uint32_t *a0 = cell + i0 * QT;
                    a0[0] = h2_as_u32(__hadd2(u32_as_h2(a0[0]), u32_as_h2(d0)));
                    a0[hv] = h2_as_u32(__hadd2(u32_as_h2(a0[hv]), u32_as_h2(p0)));
                }
            }
        } else if (wid < D + NKW) {
            // histK += ds ; lanes = keys, the planes are read column-wise, two queries per step
            for (int d = 2 * (wid - D); d < 2 * (wid - D) + 2 && d < D && S3D_KEEP(7); ++d) {
                const bool lo = d < 5;
                const int sh = IDX_BITS * (lo ? d : d - 5);
                const uint32_t *drow = s_DS + lane * ES, *wrow = (lo ? s_W0 : s_W1) + lane * ES;
                const uint16_t *lut = s_lut + d * pm.lut_stride;
                uint32_t *cell = s_hk + mypos;
                uint32_t d0 = drow[0], x0 = wrow[0], d1 = drow[1], x1 = wrow[1];
                int qq = 0;
                for (; qq + 1 < nq; qq += 2) {
                    const uint32_t i0 = lut[(x0 >> sh) & ((1u << IDX_BITS) - 1u)], i1 = lut[(x1 >> sh) & ((1u << IDX_BITS) - 1u)];
                    uint32_t *a0 = cell + i0 * QT, *a1 = cell + i1 * QT;
                    const uint32_t c0 = a0[0], c1 = a1[0];
                    const uint32_t cd0 = d0, cd1 = d1;
                    const int q2 = min(qq + 2, QT - 1), q3 = min(qq + 3, QT - 1);
                    d0 = drow[q2]; x0 = wrow[q2];
                    d1 = drow[q3]; x1 = wrow[q3];
                    const __half2 s0 = __hadd2(u32_as_h2(c0), u32_as_h2(cd0));
                    const __half2 s1 = __hadd2(a1 == a0 ? s0 : u32_as_h2(c1), u32_as_h2(cd1));
                    a0[0] = h2_as_u32(s0);
                    a1[0] = h2_as_u32(s1);
                }
                if (qq < nq) {
                    const uint32_t i0 = lut[(x0 >> sh) & ((1u << IDX_BITS) - 1u)];
                    uint32_t *a0 = cell + i0 * QT;
                    a0[0] = h2_as_u32(__hadd2(u32_as_h2(a0[0]), u32_as_h2(d0)));
                }
            }
        }
        if (wid == GEMM_WARP || wid == DV_WARP) {
            float pg[2][2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                if (a == 1 && wid != GEMM_WARP) break;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i) pg[h][i][0] = pg[h][i][1] = pg[h][i][2] = pg[h][i][3] = 0.f;
                if (S3D_KEEP(4)) {
                    if (wid == DV_WARP) pair_gemm1<true>(pg, s_P, s_do, nq, g, t);         // dV[k]  = sum_q p  dO[q]
                    else if (a == 0) pair_gemm1<false>(pg, s_DS, s_k, nk, g, t);           // dQ[q] += sum_k ds K[k]
                    else pair_gemm1<true>(pg, s_DS, s_q, nq, g, t);                        // dK[k] += sum_q ds Q[q]
                }
                store_part(s_pg + (wid == DV_WARP ? 1 : 2 * a) * 512, pg, g, t);
            }
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(4)
        // ---- dTq, dTv, dTk ; dQ += histQ.Tq, dK += histK.Tk -------------------------------------------------------
        if (tg < 3 && S3D_KEEP(5)) {
            uint32_t xb[2][2][2];
            load_dt_bfrag(xb, tg == 0 ? s_q : (tg == 1 ? s_do : s_k), g, t);
            const uint32_t *hist = tg == 0 ? s_hq : (tg == 1 ? s_hv : s_hk);
#pragma unroll
            for (int i = 0; i < NPU; ++i) {
                const int mt = wsub + TG * i;
                if (mt < n_mt && ((used >> mt) & 1u)) dt_unit_b(dt_acc[i], hist, xb, mt, g, t);
            }
        }
        if (side < 2) {
            float part[2][2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i) part[h][i][0] = part[h][i][1] = part[h][i][2] = part[h][i][3] = 0.f;
#pragma unroll
            for (int i = 0; i < NHU; ++i) {
                const int ks = ws2 + SG * i;
                if (ks < n_mt && ((used >> ks) & 1u) && S3D_KEEP(6)) {
                    const uint4 f = s_tb[(side * n_mt + ks) * 32 + lane];
                    const uint32_t tbf[2][2] = {{f.x, f.y}, {f.z, f.w}};
                    ht_unit(part, side == 0 ? s_hq : s_hk, tbf, ks, g, t);
                }
            }
            store_part(s_part + (side * SG + ws2) * 512, part, g, t);
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(5)
        // ---- reduce and store dQ, dV (threads 0..255), dK (threads 256..511) ----------------------------------------
        for (int e = tid; e < 512; e += NT) {
            const int sd = e >> 8, xx = (e >> 3) & 31, ch = (e & 7) * 2;
            if (xx < (sd == 0 ? nq : nk)) {
                const float *pg = s_pg + (sd == 0 ? 0 : 2) * 512 + xx * 16 + ch;
                float a = pg[0], b = pg[1];
                const float *pp = s_part + sd * SG * 512 + xx * 16 + ch;
#pragma unroll
                for (int ww = 0; ww < SG; ++ww) {
                    const float2 pr = *reinterpret_cast<const float2 *>(pp + ww * 512);
                    a += pr.x;
                    b += pr.y;
                }
                // a later share of a large window is added to the rows this block wrote before
                const bool add = sd == 0 ? add_q : add_k;
                const int64_t o = (int64_t)(sd == 0 ? s_rowq : s_rowk)[xx] * HC + co + ch;
                // (the same thread writes every share of a row, to this GPU and to the mirrors: the last one stays)
                __half *dst = sd == 0 ? P.dq : P.dk;
                if (add) {
                    const float2 old = __half22float2(*reinterpret_cast<const __half2 *>(dst + o));
                    a += old.x;
                    b += old.y;
                }
                const __half2 r2 = __floats2half2_rn(a, b);
                *reinterpret_cast<__half2 *>(dst + o) = r2;
                __half2 dv2 = r2;
                if (sd == 1) {
                    float2 dvv = *reinterpret_cast<const float2 *>(s_pg + 512 + xx * 16 + ch);
                    if (add) {
                        const float2 old = __half22float2(*reinterpret_cast<const __half2 *>(P.dv + o));
                        dvv.x += old.x;
                        dvv.y += old.y;
                    }
                    dv2 = __floats2half2_rn(dvv.x, dvv.y);
                    *reinterpret_cast<__half2 *>(P.dv + o) = dv2;
                }
                if (MIRROR) {                        // the other GPUs' arrays (plain peer stores)
                    for (int m = 0; m < MM.dq.n; ++m) {
                        __half *mp = static_cast<__half *>(sd == 0 ? MM.dq.p[m] : MM.dk.p[m]);
                        *reinterpret_cast<__half2 *>(mp + o) = r2;
                        if (sd == 1) *reinterpret_cast<__half2 *>(static_cast<__half *>(MM.dv.p[m]) + o) = dv2;
                    }
                }
            }
        }
        // this warp is done with the stage
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + s);
    }  // windows
    S3D_PHASE_FLUSH(0)

    // ---- flush the table gradients of this block ---------------------------------------------------------------------
    if (tg < 3) {
        float *dst = tg == 0 ? P.dtq : (tg == 1 ? P.dtv : P.dtk);
#pragma unroll
        for (int i = 0; i < NPU; ++i) {
            const int mt = wsub + TG * i;
            if (mt < n_mt) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int row = perm_table_row(pm, mt * 16 + g + 8 * rr);   // aliases flush into the row they stand for
                        if (row >= 0) {
                            float *p = dst + (int64_t)row * HC + co + h * 8 + 2 * t;
                            atomicAdd(p, dt_acc[i][h][2 * rr]);
                            atomicAdd(p + 1, dt_acc[i][h][2 * rr + 1]);
                        }
                    }
            }
        }
    }
}

template <int D, int NPU, int NHU, bool HD16, bool MIRROR>
static int launch_small_m(const SmallParams &p, const BwdMirrors &mm, const CrseMeta &meta, const PermMeta &pm, cudaStream_t st)
{
    constexpr int NW = bwd_small_warps(D);
    const SmallSmem L = make_small_layout(pm.R, NW, pm.D * pm.lut_stride);
    auto kern = attn_bwd_small_kernel<D, NPU, NHU, HD16, MIRROR>;
    static int sms_of[64] = {0};     // 0: this instantiation has not been set up on the device yet
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return S3D_ERR_LAUNCH;
    if (sms_of[dev] == 0) {
        int sms = 0;
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        note_cuda_error(e);
        if (e != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
            return S3D_ERR_LAUNCH;
        sms_of[dev] = sms;
    }
    const int hp = HD16 ? p.H : p.H / 2;
    int gx = sms_of[dev] / hp;
    if (gx > p.W) gx = (int)p.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, (NW + 1) * 32, L.total, st>>>(p, pm, make_pair_consts(meta), mm);
    const cudaError_t le = cudaGetLastError();
    note_cuda_error(le);
    return le == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <int D, int NPU, int NHU, bool HD16>
static int launch_small(const SmallParams &p, const BwdMirrors &mm, const CrseMeta &meta, const PermMeta &pm, cudaStream_t st)
{
    return mm.dq.n ? launch_small_m<D, NPU, NHU, HD16, true>(p, mm, meta, pm, st)
                   : launch_small_m<D, NPU, NHU, HD16, false>(p, mm, meta, pm, st);
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
    const tc::PermMeta pm = tc::make_perm_meta(a.meta);
    const int n_mt = (pm.R + 15) / 16;
    const int nw = tc::bwd_small_warps(a.meta.D);
    if (n_mt > 32 || n_mt > 5 * (nw / 3) || n_mt > 4 * (nw / 2)) return false;     // the tile mask is one word
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;
    return tc::make_small_layout(pm.R, nw, pm.D * pm.lut_stride).total <= 227 * 1024;
}

// All windows; dtq, dtk, dtv must be zero on entry (accumulated into).
int attn_tc_backward_small(const AttnArgs &a0, cudaStream_t st)
{
    if (a0.W == 0) return S3D_OK;
    AttnArgs a = a0;
    const tc::PermMeta pm = tc::make_perm_meta(a0.meta);   // the kernel works in its own row numbering
    tc::SmallParams p{};
    p.q = (const __half *)a.q; p.k = (const __half *)a.k; p.v = (const __half *)a.v;
    p.dout = (const __half *)a.dout; p.o = (const __half *)a.out; p.lse = a.lse;
    p.tq = (const __half *)a.tq; p.tk = (const __half *)a.tk; p.tv = (const __half *)a.tv;
    p.dq = (__half *)a.dq; p.dk = (__half *)a.dk; p.dv = (__half *)a.dv;
    tc::BwdMirrors mm{a.m_dq, a.m_dk, a.m_dv};
    p.dtq = a.dtq; p.dtk = a.dtk; p.dtv = a.dtv;
    p.w_sizes = a.w_sizes; p.w2n = a.w2n; p.n2n = a.n2n; p.n_coords = a.n_coords;
    p.W = a.W; p.H = a.H;
    const int n_mt = (pm.R + 15) / 16;
    const int nw = tc::bwd_small_warps(a.meta.D);
    const int npu = (n_mt + nw / 3 - 1) / (nw / 3);   // <= 5
    const int nhu = (n_mt + nw / 2 - 1) / (nw / 2);   // <= 4
#define S3D_SMALL_H(DD, HH)                                                                  \
    if (npu <= 4 && nhu <= 3) return tc::launch_small<DD, 4, 3, HH>(p, mm, a.meta, pm, st);      \
    return tc::launch_small<DD, 5, 4, HH>(p, mm, a.meta, pm, st);
#define S3D_SMALL(DD) if (a.hd == 16) { S3D_SMALL_H(DD, true) } else { S3D_SMALL_H(DD, false) }
    switch (a.meta.D) {
        case 3: S3D_SMALL(3)
        case 6: S3D_SMALL(6)
        case 9: S3D_SMALL(9)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_SMALL
#undef S3D_SMALL_H
}

}  // namespace s3d
