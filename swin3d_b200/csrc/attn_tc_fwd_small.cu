// Forward of the cRSE window attention for windows of at most 32 voxels, tensor-core path (fp16).
//
// The whole window is one 32 x 32 tile, so the softmax needs no running maximum across key tiles
// and nothing is ever rescaled.  A block of D+1 warps (at least 8) serves one head pair (head_dim 8)
// or one head (head_dim 16) and walks the windows x, x + gridDim.x, ...; per window:
//   stage      Q, K, V rows of the head pair, the signal coordinates
//   GEMM       P_q = Tq.Q^T (lane-major), P_k = Tk.K^T (key-major), S0 = K.Q^T     [tensor cores]
//              the first half of the warps owns the Tq tiles, the second half the Tk tiles, so a
//              warp builds the block-diagonal B fragments of its feature array once per window
//   scores     lane = query, the keys dealt to the warps: D indices, 2*D look-ups, score; the
//              scores and the packed indices of a thread's (at most four) pairs stay in registers;
//              exact row maxima through shared-memory atomics
//   softmax    probabilities, row sums, pair entries written once: two [key][query] planes of
//              8-byte entries, (p, idx 0-4) and (idx 5-8, p), row stride 33 entries
//   histogram  warp d owns signal dimension d (rows of different dimensions are disjoint):
//              hist[row][q] += p, two keys per step, the next step's entries fetched before the
//              stores of this one; warp D: O = P.V                                    [tensor cores]
//   epilogue   O += hist.Tv (k-steps dealt to the warps) [tensor cores], reduce, normalise, store
// The histogram reuses the shared memory of P_q, which is dead once the scores exist; 108 KB of
// shared memory per block, two blocks per SM.
// grid = (x, H/2) (head_dim 8) or (x, H) (head_dim 16).  Larger windows: attn_tc_fwd.cu.
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"
#include "async_stage.cuh"

namespace s3d {
namespace tc {

// Debug build only (-DS3D_PHASE_CLOCK): cycles spent between the block-wide barriers of a window,
// summed over all windows and blocks by thread 0 of every block; read back with
// s3d_debug_phase_cycles().  Compiled out otherwise.
#ifdef S3D_PHASE_CLOCK
__device__ unsigned long long g_phase_cycles[16];
__device__ unsigned int g_ablate;      // bit i set: piece i of the kernel is skipped (results are then wrong)
#define S3D_KEEP(i) (!(ablate & (1u << (i))))
#define S3D_PHASE_DECL long long ph_t = clock64(); unsigned long long ph_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define S3D_PHASE_MARK(i) if (threadIdx.x == 0) { const long long now = clock64(); ph_acc[i] += (unsigned long long)(now - ph_t); ph_t = now; }
#define S3D_PHASE_FLUSH(base) if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) atomicAdd(&g_phase_cycles[(base) + i], ph_acc[i]); }
#else
#define S3D_KEEP(i) true
#define S3D_PHASE_DECL
#define S3D_PHASE_MARK(i)
#define S3D_PHASE_FLUSH(base)
#endif

constexpr int FS_STAGES = 2;      // windows staged ahead of the one being computed

struct FwdSmallSmem {
    int R16, Rp;
    int off_pq, off_pk, off_e, off_rows, off_c, off_misc, total;
};

__host__ __device__ inline FwdSmallSmem make_fwd_small_layout(int R, int nw)
{
    FwdSmallSmem L;
    L.R16 = (R + 15) / 16 * 16;
    L.Rp = (L.R16 + 31) / 32 * 32 + 8;
    int off = 0;
    L.off_pq = off; off += L.R16 * QT * 4;                                   // P_q, later the histogram
    const int pk = 32 * L.Rp * 4, red = nw * (QT * 16 + QT * 2) * 4;
    L.off_pk = off; off += pk > red ? pk : red;                              // P_k, later the reduction buffer
    L.off_e = off; off += 2 * 32 * ES * 8;                                   // pair entries, two planes
    L.off_rows = off; off += FS_STAGES * 3 * 32 * 16 * 2;                    // Q, K, V rows, per stage
    L.off_c = off; off += FS_STAGES * 32 * 12 * 4;                           // signal coordinates, per stage
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
    Mirrors m_out;
};

// Set when a bounded wait of a kernel in this file ran out (it never should); read and cleared by
// s3d_debug_async_error().
__device__ int g_fwd_small_async_error;

// Block = NW consumer warps + one producer warp.  The producer walks the block's windows
// (x, x + gridDim.x, ... of at most 32 voxels) ahead of the consumers: it finds the next window,
// reads its row numbers and coordinates and has the copy engine bring the 32-byte Q, K, V pieces
// of its voxels into the next stage of shared memory (cp.async.bulk, completion on the stage's
// "full" mbarrier); the consumers hand a stage back through its "empty" mbarrier.
template <int D, int NW, int NPU /*projection units per warp*/, int NHU /*hist.T units per warp*/, bool HD16>
__global__ void __launch_bounds__((NW + 1) * 32, 2)
attn_fwd_small_kernel(const __grid_constant__ FwdSmallParams P, const CrseMeta meta, const PairConsts pc)
{
    constexpr int NT = NW * 32;                  // consumer threads
    constexpr int HALF = NW / 2;                 // warps per projection table
    constexpr int KPW = (QT + NW - 1) / NW;      // keys per warp in the score phase
    static_assert(D < NW, "one warp per signal dimension plus one for P.V");
    extern __shared__ __align__(16) unsigned char smem[];
    const FwdSmallSmem L = make_fwd_small_layout(meta.R, NW);
    uint32_t *s_pq = reinterpret_cast<uint32_t *>(smem + L.off_pq);
    uint32_t *s_hist = s_pq;
    uint32_t *s_pk = reinterpret_cast<uint32_t *>(smem + L.off_pk);
    uint2 *s_elo = reinterpret_cast<uint2 *>(smem + L.off_e);        // [32][ES] (p, idx 0-4); S0 before
    uint2 *s_ehi = s_elo + 32 * ES;                                  // [32][ES] (idx 5-8, p)
    __half *s_rows = reinterpret_cast<__half *>(smem + L.off_rows);  // [stage][Q,K,V][32][16]
    float *s_cs = reinterpret_cast<float *>(smem + L.off_c);         // [stage][32][12]
    float *s_max = reinterpret_cast<float *>(smem + L.off_misc);     // [32][2]
    int *s_rowi = reinterpret_cast<int *>(s_max + 64);               // [stage][32]
    int *s_n = s_rowi + FS_STAGES * 32;                              // [stage] voxels of the window, 0: no more windows
    int *s_fail = s_n + FS_STAGES;
    uint64_t *s_full = reinterpret_cast<uint64_t *>(smem + L.off_misc + 768);   // [stage]
    uint64_t *s_empty = s_full + FS_STAGES;                                      // [stage]
    float *s_red = reinterpret_cast<float *>(smem + L.off_pk);       // [NW][32][16], P_k is dead by then
    float *s_lsum = s_red + NW * 512;                                // [NW][32][2]

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int hp = blockIdx.y, H = P.H;
    const int HC = H * (HD16 ? 16 : 8), co = hp * 16;

    if (tid == 0) {
        for (int s = 0; s < FS_STAGES; ++s) {
            mbar_init(s_full + s, 1);
            mbar_init(s_empty + s, NW);
        }
        *s_fail = 0;
        mbar_init_fence();
    }
    __syncthreads();

    if (wid == NW) {
        // ================================ producer warp ================================================
        int64_t w = (int64_t)blockIdx.x - gridDim.x;
        for (int it = 0;; ++it) {
            // next window of at most QT voxels among this block's windows, 32 candidates at a time
            int n = 0;
            for (;;) {
                const int64_t cand = w + (int64_t)(lane + 1) * gridDim.x;
                const int nn = cand < P.W ? __ldg(P.w_sizes + cand) : 0;
                const unsigned ok = __ballot_sync(0xffffffffu, nn >= 1 && nn <= QT);
                if (ok) {
                    const int j = __ffs(ok) - 1;
                    w += (int64_t)(j + 1) * gridDim.x;
                    n = __shfl_sync(0xffffffffu, nn, j);
                    break;
                }
                w += (int64_t)32 * gridDim.x;
                if (w + gridDim.x >= P.W) break;         // n stays 0: no more windows
            }
            int row = 0;
            float c[D];
#pragma unroll
            for (int d = 0; d < D; ++d) c[d] = 0.f;
            if (n > 0) {
                const int base = __ldg(P.w2n + w);
                if (lane < n) {
                    row = __ldg(P.n2n + base + lane);
#pragma unroll
                    for (int d = 0; d < D; ++d) c[d] = __ldg(P.n_coords + (int64_t)(base + lane) * D + d);
                }
            }
            const int s = it % FS_STAGES;
            if (it >= FS_STAGES && !mbar_wait(s_empty + s, ((it / FS_STAGES) - 1) & 1)) {
                g_fwd_small_async_error = 1;
                n = 0;                                    // tell the consumers to stop
            }
            __half *rq = s_rows + s * 1536;
            float *cs = s_cs + s * 384;
#pragma unroll
            for (int d = 0; d < D; ++d) cs[lane * 12 + d] = c[d];
            s_rowi[s * 32 + lane] = row;
            if (lane >= n) {                              // rows beyond the window are zero
#pragma unroll
                for (int a = 0; a < 3; ++a) {
                    *reinterpret_cast<uint4 *>(rq + a * 512 + lane * 16) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4 *>(rq + a * 512 + lane * 16 + 8) = make_uint4(0, 0, 0, 0);
                }
            }
            if (lane == 0) s_n[s] = n;
            async_proxy_fence();
            __syncwarp();
            if (lane == 0) mbar_arrive_expect_tx(s_full + s, (unsigned)(n * 96));
            __syncwarp();
            if (lane < n) {
                const int64_t off = (int64_t)row * HC + co;
                bulk_copy_g2s(rq + lane * 16, P.q + off, 32, s_full + s);
                bulk_copy_g2s(rq + 512 + lane * 16, P.k + off, 32, s_full + s);
                bulk_copy_g2s(rq + 1024 + lane * 16, P.v + off, 32, s_full + s);
            }
            if (n == 0) break;
        }
        return;
    }

    // ==================================== consumer warps ===============================================
    const int g = lane >> 2, t = lane & 3;
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // projection units: warps [0, HALF) own the Tq tiles wsub + HALF i, warps [HALF, 2 HALF) the Tk tiles
    const bool q_side = wid < HALF;
    const bool p_side = wid < 2 * HALF;
    const int wsub = q_side ? wid : wid - HALF;
    uint32_t ta[NPU][2][2];
#pragma unroll
    for (int i = 0; i < NPU; ++i) {
        const int mt = wsub + HALF * i;
        const __half *T = q_side ? P.tq : P.tk;
        const bool ok = p_side && mt < n_mt;
        const int r0 = ok ? table_row(meta, mt * 16 + g) : -1, r1 = ok ? table_row(meta, mt * 16 + g + 8) : -1;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            ta[i][h][0] = r0 >= 0 ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r0 * HC + co + h * 8 + 2 * t) : 0u;
            ta[i][h][1] = r1 >= 0 ? *reinterpret_cast<const uint32_t *>(T + (int64_t)r1 * HC + co + h * 8 + 2 * t) : 0u;
        }
    }
    // hist.Tv units: k-step = wid + NW i
    uint32_t tb[NHU][2][2];
#pragma unroll
    for (int i = 0; i < NHU; ++i) {
        const int ks = wid + NW * i;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int ra = ks < n_mt ? table_row(meta, ks * 16 + ht_krow(t, half, 0)) : -1;
                const int rb = ks < n_mt ? table_row(meta, ks * 16 + ht_krow(t, half, 1)) : -1;
                const __half lo = ra >= 0 ? P.tv[(int64_t)ra * HC + co + h * 8 + g] : __float2half(0.f);
                const __half hi = rb >= 0 ? P.tv[(int64_t)rb * HC + co + h * 8 + g] : __float2half(0.f);
                tb[i][h][half] = h2_as_u32(__halves2half2(lo, hi));
            }
    }
    S3D_PHASE_DECL
#ifdef S3D_PHASE_CLOCK
    const unsigned ablate = g_ablate;
#endif
    for (int it = 0;; ++it) {
        const int s = it % FS_STAGES;
        if (!mbar_wait(s_full + s, (it / FS_STAGES) & 1)) {
            *s_fail = 1;
            g_fwd_small_async_error = 2;
        }
        consumer_sync<NT>();          // the previous window's epilogue is over; the flag is settled
        S3D_PHASE_MARK(0)
        const int n = s_n[s];
        if (n == 0 || *s_fail) break;
        const __half *s_q = s_rows + s * 1536, *s_k = s_q + 512, *s_v = s_q + 1024;
        const float *s_c = s_cs + s * 384;
        const int *s_row = s_rowi + s * 32;
        float cx[D];
        load_coords12<D>(s_c + lane * 12, cx);
        if (tid < 64) s_max[tid] = -INFINITY;
        // ---- projections P_q (lane-major), P_k (key-major); S0 = K.Q^T ------------------------------
        if (p_side && S3D_KEEP(0)) {
            uint32_t bf[8][2];
            load_feat_bfrag(bf, q_side ? s_q : s_k, n, g, t);
#pragma unroll
            for (int i = 0; i < NPU; ++i) {
                const int mt = wsub + HALF * i;
                if (mt < n_mt) {
                    if (q_side) project_unit_b<true>(ta[i], bf, s_pq, mt, Rp, n, g, t);
                    else project_unit_b<false>(ta[i], bf, s_pk, mt, Rp, n, g, t);
                }
            }
        }
        for (int u = wid; u < 16 && S3D_KEEP(1); u += NW) {
            const int mt = u >> 3, j = u & 7;       // key rows 16mt.., query columns 4j..
            if (16 * mt < n && 4 * j < n) {
                const __half *ysrc = s_k + mt * 256;
                const uint32_t wv = *reinterpret_cast<const uint32_t *>(s_q + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 2 * t);
                const uint32_t a1 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 2 * t);
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(ysrc + g * 16 + 8 + 2 * t);
                const uint32_t a3 = *reinterpret_cast<const uint32_t *>(ysrc + (g + 8) * 16 + 8 + 2 * t);
                float c[4];
                mma_k16_z(c, a0, a1, a2, a3, (g & 1) ? 0u : wv, (g & 1) ? wv : 0u);
                *reinterpret_cast<float2 *>(s_elo + (16 * mt + g) * ES + 4 * j + t) = make_float2(c[0], c[1]);
                *reinterpret_cast<float2 *>(s_elo + (16 * mt + g + 8) * ES + 4 * j + t) = make_float2(c[2], c[3]);
            }
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(2)
        // ---- scores: keys wid, wid + NW, ... ; lane = query: indices, 2*D look-ups, score -------------
        float sreg[KPW][2];
        uint32_t wreg[KPW][2];
        float mloc0 = -INFINITY, mloc1 = -INFINITY;
        const uint32_t *pq_lane = s_pq + mypos;
#pragma unroll
        for (int j = 0; j < KPW; ++j) {
            const int kk = wid + NW * j;
            sreg[j][0] = sreg[j][1] = 0.f;
            wreg[j][0] = wreg[j][1] = 0u;
            if (kk < n && S3D_KEEP(2)) {
                float ck[D];
                load_coords12<D>(s_c + kk * 12, ck);
                const uint32_t *pk_row = s_pk + kk * Rp;
                __half2 bq = __float2half2_rn(0.f), bk = bq;
                uint32_t w0 = 0, w1 = 0;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const uint32_t idx = crse_index_pc(cx[d], ck[d], pc.half[d], pc.clamp[d]);
                    const uint32_t row = meta.rowbase[d] + idx;
                    bq = __hadd2(bq, u32_as_h2(pq_lane[row * QT]));
                    bk = __hadd2(bk, u32_as_h2(pk_row[row]));
                    if (d < 5) w0 |= idx << (IDX_BITS * d);
                    else w1 |= idx << (IDX_BITS * (d - 5));
                }
                const float2 s0 = *reinterpret_cast<const float2 *>(s_elo + kk * ES + lane);
                const float2 b = __half22float2(__hadd2(bq, bk));
                float sx = s0.x + b.x, sy = s0.y + b.y;
                if (HD16) sx = sy = sx + sy;          // one head: both halves carry the full score
                sreg[j][0] = sx;
                sreg[j][1] = sy;
                wreg[j][0] = w0;
                wreg[j][1] = w1;
                mloc0 = fmaxf(mloc0, sx);
                mloc1 = fmaxf(mloc1, sy);
            }
        }
        if (wid < n) {
            atomic_max_float(s_max + lane * 2, mloc0);
            atomic_max_float(s_max + lane * 2 + 1, mloc1);
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(3)
        // ---- probabilities, pair entries; clear the histogram (the P_q storage) ---------------------------
        const float m0 = s_max[lane * 2] * LOG2E, m1 = s_max[lane * 2 + 1] * LOG2E;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int j = 0; j < KPW; ++j) {
            const int kk = wid + NW * j;
            if (kk < QT && S3D_KEEP(3)) {
                uint32_t ph = 0u;                         // zero for keys beyond the window: P.V reads whole 16-key steps
                if (kk < n && lane < n) {
                    const float p0 = ex2_approx(fmaf(sreg[j][0], LOG2E, -m0));
                    const float p1 = ex2_approx(fmaf(sreg[j][1], LOG2E, -m1));
                    l0 += p0;
                    l1 += p1;
                    ph = h2_as_u32(__floats2half2_rn(p0, p1));
                }
                s_elo[kk * ES + lane] = make_uint2(ph, wreg[j][0]);
                s_ehi[kk * ES + lane] = make_uint2(wreg[j][1], ph);
            }
        }
        for (int i = tid; i < L.R16 * QT / 4 && S3D_KEEP(4); i += NT)
            reinterpret_cast<uint4 *>(s_hist)[i] = make_uint4(0, 0, 0, 0);
        consumer_sync<NT>();
        S3D_PHASE_MARK(4)
        // ---- histogram (warp d: signal dimension d) | warp D: O = P.V -----------------------------------------
        float part[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 2; ++i) part[h][i][0] = part[h][i][1] = part[h][i][2] = part[h][i][3] = 0.f;
        if (wid < D && S3D_KEEP(5)) {
            const int d = wid;
            const bool lo = d < 5;
            const int sh = IDX_BITS * (lo ? d : d - 5);
            // the half of a pair entry this dimension needs: (p, idx 0-4) or (idx 5-8, p)
            const uint2 *ecol = (lo ? s_elo : s_ehi) + lane;
            uint32_t *cell = s_hist + meta.rowbase[d] * QT + mypos;
            uint2 e0 = ecol[0], e1 = ecol[ES];              // keys beyond the window hold zero entries
            int kk = 0;
            for (; kk + 1 < n; kk += 2) {
                const uint32_t p0 = lo ? e0.x : e0.y, i0 = ((lo ? e0.y : e0.x) >> sh) & ((1u << IDX_BITS) - 1u);
                const uint32_t p1 = lo ? e1.x : e1.y, i1 = ((lo ? e1.y : e1.x) >> sh) & ((1u << IDX_BITS) - 1u);
                uint32_t *a0 = cell + i0 * QT, *a1 = cell + i1 * QT;
                const uint32_t c0 = *a0, c1 = *a1;
                e0 = ecol[min(kk + 2, QT - 1) * ES];
                e1 = ecol[min(kk + 3, QT - 1) * ES];
                const __half2 s0 = __hadd2(u32_as_h2(c0), u32_as_h2(p0));
                const __half2 s1 = __hadd2(a1 == a0 ? s0 : u32_as_h2(c1), u32_as_h2(p1));
                *a0 = h2_as_u32(s0);
                *a1 = h2_as_u32(s1);
            }
            if (kk < n) {
                const uint32_t p0 = lo ? e0.x : e0.y, i0 = ((lo ? e0.y : e0.x) >> sh) & ((1u << IDX_BITS) - 1u);
                uint32_t *a0 = cell + i0 * QT;
                *a0 = h2_as_u32(__hadd2(u32_as_h2(*a0), u32_as_h2(p0)));
            }
        } else if (wid == D && S3D_KEEP(6)) {
            pair_gemm2<0, false>(part, s_elo, s_v, n, g, t);  // O[q] = sum_k p V[k]
        }
        consumer_sync<NT>();
        S3D_PHASE_MARK(5)
        // ---- O += hist . Tv (k-steps split over the warps), reduce, normalise, store --------------------------
#pragma unroll
        for (int i = 0; i < NHU; ++i) {
            const int ks = wid + NW * i;
            if (ks < n_mt && S3D_KEEP(7)) ht_unit(part, s_hist, tb[i], ks, g, t);
        }
        store_part(s_red + wid * 512, part, g, t);       // P_k (aliased by s_red) is dead since the scores
        s_lsum[(wid * QT + lane) * 2] = l0;
        s_lsum[(wid * QT + lane) * 2 + 1] = l1;
        consumer_sync<NT>();
        S3D_PHASE_MARK(6)
        if (tid < 256 && S3D_KEEP(8)) {
            const int qq = tid >> 3, ch = (tid & 7) * 2, h = ch >> 3;
            if (qq < n) {
                float a = 0.f, b = 0.f, ls = 0.f;
#pragma unroll
                for (int ww = 0; ww < NW; ++ww) {
                    const float2 pr = *reinterpret_cast<const float2 *>(s_red + ww * 512 + qq * 16 + ch);
                    a += pr.x;
                    b += pr.y;
                    ls += s_lsum[(ww * QT + qq) * 2 + h];
                }
                const float inv = 1.f / ls;
                const int64_t row = s_row[qq];
                store_h2_mirrored(P.out, P.m_out, row * HC + co + ch, __floats2half2_rn(a * inv, b * inv));
                if (HD16) {
                    if (ch == 0) P.lse[row * H + hp] = s_max[qq * 2] + __logf(ls);
                } else if ((ch & 7) == 0) {
                    P.lse[row * H + 2 * hp + h] = s_max[qq * 2 + h] + __logf(ls);
                }
            }
        }
        // this warp is done with the stage (rows, coordinates, row numbers)
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty + s);
    }  // windows
    S3D_PHASE_FLUSH(0)
}

template <int D, int NW, int NPU, int NHU, bool HD16>
static int launch_fwd_small(const FwdSmallParams &p, const CrseMeta &meta, cudaStream_t st)
{
    const FwdSmallSmem L = make_fwd_small_layout(meta.R, NW);
    auto kern = attn_fwd_small_kernel<D, NW, NPU, NHU, HD16>;
    // blocks per SM of this instantiation, found once per device
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
    // the launch bounds keep two blocks' registers within an SM; shared memory (228 KB per SM, 1 KB
    // reserved per block) decides whether two fit
    const int per_sm = 2 * (L.total + 1024) <= 228 * 1024 ? 2 : 1;
    int gx = sms_of[dev] * per_sm / hp;
    if (gx > p.W) gx = (int)p.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, (NW + 1) * 32, L.total, st>>>(p, meta, make_pair_consts(meta));
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

static int fwd_small_warps(int D) { return D + 1 > 8 ? D + 1 : 8; }

}  // namespace tc

#ifdef S3D_PHASE_CLOCK
extern "C" int s3d_debug_set_ablate(unsigned int mask)
{
    return cudaMemcpyToSymbol(tc::g_ablate, &mask, sizeof(mask)) == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

extern "C" int s3d_debug_phase_cycles(unsigned long long *out16, int reset)
{
    if (cudaMemcpyFromSymbol(out16, tc::g_phase_cycles, sizeof(unsigned long long) * 16) != cudaSuccess) return S3D_ERR_LAUNCH;
    if (reset) {
        unsigned long long z[16] = {0};
        if (cudaMemcpyToSymbol(tc::g_phase_cycles, z, sizeof(z)) != cudaSuccess) return S3D_ERR_LAUNCH;
    }
    return S3D_OK;
}
#endif

bool attn_tc_fwd_small_supported(const AttnArgs &a)
{
    if (a.dtype != S3D_F16) return false;
    if (!(a.hd == 16 || (a.hd == 8 && !(a.H & 1)))) return false;
    const int Rint = a.meta.R + a.meta.D - 1;
    const int n_mt = (Rint + 15) / 16;
    const int nw = tc::fwd_small_warps(a.meta.D);
    if (n_mt > 6 * (nw / 2) || n_mt > 3 * nw) return false;
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;
    return tc::make_fwd_small_layout(Rint, nw).total <= 227 * 1024;
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
    p.out = (__half *)a.out; p.lse = a.lse; p.m_out = a.m_out;
    p.w_sizes = a.w_sizes; p.w2n = a.w2n; p.n2n = a.n2n; p.n_coords = a.n_coords;
    p.W = a.W; p.H = a.H;
    const int n_mt = (a.meta.R + 15) / 16;
    const int nw = tc::fwd_small_warps(a.meta.D);
    const int npu = (n_mt + nw / 2 - 1) / (nw / 2);   // <= 6
    const int nhu = (n_mt + nw - 1) / nw;             // <= 3
#define S3D_FS(DD, NWW, HH)                                                                       \
    if (npu <= 2 && nhu <= 1) return tc::launch_fwd_small<DD, NWW, 2, 1, HH>(p, a.meta, st);      \
    if (npu <= 4 && nhu <= 2) return tc::launch_fwd_small<DD, NWW, 4, 2, HH>(p, a.meta, st);      \
    return tc::launch_fwd_small<DD, NWW, 6, 3, HH>(p, a.meta, st);
#define S3D_FS_D(DD, NWW) if (a.hd == 16) { S3D_FS(DD, NWW, true) } else { S3D_FS(DD, NWW, false) }
    switch (a.meta.D) {
        case 3: S3D_FS_D(3, 8)
        case 6: S3D_FS_D(6, 8)
        case 9: S3D_FS_D(9, 10)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_FS_D
#undef S3D_FS
}

}  // namespace s3d
