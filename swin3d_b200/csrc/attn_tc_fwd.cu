// Fused forward of the cRSE window attention, tensor-core path (fp16 storage, head_dim 8 or 16).
//
// grid = (x, head pairs or heads, see the head modes in attn_tc.cuh): a block serves its two slots
// for the windows x, x+gridDim.x, ...  Work item = (window, tile of 32 queries); keys are streamed in
// tiles of two per warp (32 with 16 warps, 16 with 8) with an online softmax whose rescale happens
// once per key tile.  Per key tile:
//   GEMM    P_k = K.Tk^T (this tile's keys), S0 = K.Q^T                          [tensor cores]
//   phase 1 lane = query, each warp two keys: cRSE indices, 2*D look-ups, score, running max
//   phase 1.5 probabilities p = exp(s - m), row sums
//   phase 2 one signal dimension per warp (two with 8 warps): hist[row][q] += p, four keys per step
//           (no atomics: rows of different dimensions are disjoint, a warp owns its dimensions)
//           | last warp (and, with two planes, the one before it): O += P.V           [tensor cores]
// and per item:  P_q = Q.Tq^T before, O += hist.Tv after (once per plane)         [tensor cores]
// The Tk fragments (used once per key tile) stay in registers; Tq and Tv (used once per item) do
// too when the head mode has one plane and are fetched through L1/L2 otherwise.
// See attn_tc.cuh for the factorisation, the head modes and the shared-memory layouts.
#include "attn_kernels.cuh"
#include "attn_tc.cuh"
#include "attn_tc_small.cuh"

namespace s3d {
namespace tc {

template <int D, int MTW, int HDM, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 2 : 1)
attn_fwd_tc_kernel(const __half *__restrict__ q, const __half *__restrict__ k,
                   const __half *__restrict__ v, const __half *__restrict__ tq,
                   const __half *__restrict__ tk, const __half *__restrict__ tv,
                   const CrseMeta meta, const int32_t *__restrict__ w_sizes,
                   const int32_t *__restrict__ w2n, const int32_t *__restrict__ n2n,
                   const float *__restrict__ n_coords, int64_t W, int H, int skip_upto,
                   __half *__restrict__ out, float *__restrict__ lse, const __grid_constant__ Mirrors m_out)
{
    constexpr bool HD16 = HDM == HDM_SINGLE16;       // the two slots are halves of one head
    constexpr bool PAIR16 = HDM == HDM_PAIR16;       // two heads of 16 channels, two planes
    constexpr int NPL = PAIR16 ? 2 : 1;
    constexpr int MTP = PAIR16 ? 1 : MTW;            // resident table fragments only with one plane
    // NW warps per block: 8 (two blocks per SM) or, when the tables are too large for that, 16 (one
    // block per SM); a key tile holds two keys per warp
    constexpr int NWARP = NW, NTHREADS = NW * 32, KT = 2 * NW;
    extern __shared__ __align__(16) unsigned char smem[];
    const SmemLayout L = make_layout(meta.R, 1, NPL, NW);
    uint32_t *s_pq = reinterpret_cast<uint32_t *>(smem + L.off_pq);      // [R16][32] half2
    uint32_t *s_hist = reinterpret_cast<uint32_t *>(smem + L.off_hist);  // [R16][32] half2
    uint32_t *s_pk = reinterpret_cast<uint32_t *>(smem + L.off_pk);      // [KT][Rp] half2
    float2 *s_s = reinterpret_cast<float2 *>(smem + L.off_s);            // [KT][32] (slot 0, slot 1)
    uint32_t *s_idx = reinterpret_cast<uint32_t *>(smem + L.off_idx);    // [KT][2][32]
    __half *s_k = reinterpret_cast<__half *>(smem + L.off_kv);           // [plane][KT][16]
    __half *s_v = s_k + NPL * KT * 16;                                   // [plane][KT][16]
    float *s_kc = reinterpret_cast<float *>(smem + L.off_kc);            // [KT][12]
    float *s_mtile = reinterpret_cast<float *>(smem + L.off_misc);       // [32][2]
    float *s_alpha = s_mtile + 64;                                       // [32][2]
    int *s_qrow = reinterpret_cast<int *>(s_alpha + 64);                 // [32]
    uint16_t *s_wlist = reinterpret_cast<uint16_t *>(smem + L.off_misc + 1024);   // work list of the chunk
    int *s_wcnt = reinterpret_cast<int *>(s_wlist + WL_NSEG * WL_SEG);
    __half *s_q = reinterpret_cast<__half *>(smem + L.off_s);            // [plane][32][16], aliases s_s
    float *s_red = reinterpret_cast<float *>(smem + L.off_pk);           // [NW][32][16], aliases s_pk
    float *s_lsum = s_red + NWARP * QT * 16;                             // [NW][32][2]

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int hp = blockIdx.y;
    const int HC = H * (HDM == HDM_PAIR8 ? 8 : 16);
    const int n_mt = L.R16 / 16, Rp = L.Rp;
    const int mypos = qpos(lane);
    constexpr float LOG2E = 1.4426950408889634f;

    // ---- this block's table slices as mma fragments, resident in registers: Tk (used once per key
    //      tile) in every mode, Tq and Tv (used once per item) only with one plane -----------------------
    uint32_t tqA[MTP][2][2], tvB[MTP][2][2], tkA[MTW][NPL][2][2];
#pragma unroll
    for (int i = 0; i < MTW; ++i)
#pragma unroll
        for (int pl = 0; pl < NPL; ++pl) load_table_a_frag<HDM>(tkA[i][pl], tk, meta, HC, hp, pl, wid + NWARP * i, g, t);
    if (!PAIR16) {
#pragma unroll
        for (int i = 0; i < MTP; ++i) {
            const int mt = wid + NWARP * i;
            load_table_a_frag<HDM>(tqA[i], tq, meta, HC, hp, 0, mt, g, t);
            load_table_b_frag<HDM>(tvB[i], tv, meta, HC, hp, 0, mt, g, t);
        }
    }

    for (int64_t c0 = 0; c0 < W; c0 += WL_CHUNK) {
        __syncthreads();            // every warp has left the item loop of the previous chunk
        if (tid == 0) s_wcnt[WL_NSEG] = 0;
        __syncthreads();
        build_work_list(w_sizes, W, c0, skip_upto, s_wlist, s_wcnt);   // windows up to skip_upto: single-tile kernel
        __syncthreads();
        int it_pos = 0, it_dw = -1, it_dt = -1;
        int64_t w;
        int q0;
        while (next_work_item(s_wlist, s_wcnt, w_sizes, W, c0, skip_upto, it_pos, it_dw, it_dt, w, q0)) {
            const int n = __ldg(w_sizes + w), base = __ldg(w2n + w);
            const int nq = min(QT, n - q0);
            // ---- item set-up -------------------------------------------------------------------
            __syncthreads();  // previous item's epilogue has finished with s_red / s_qrow
            float cq[D];
#pragma unroll
            for (int d = 0; d < D; ++d)
                cq[d] = lane < nq ? __ldg(n_coords + (int64_t)(base + q0 + lane) * D + d) : 0.f;
            // key tiles are fetched into registers one tile ahead: K/V row pieces by the first
            // 4*KT*NPL threads, key coordinates one element per thread starting from the upper half
            uint4 pf_val = make_uint4(0, 0, 0, 0);
            float pf_c = 0.f;
            const int pf_e = (tid + NTHREADS / 2) % NTHREADS;
            static_assert(KT * D <= NTHREADS, "one key coordinate per thread");
            auto fetch_tile = [&](int kb) {
                const int nkb = min(KT, n - kb);
                pf_val = make_uint4(0, 0, 0, 0);
                pf_c = 0.f;
                if (tid < 4 * KT * NPL) {
                    const int ki = (tid >> 2) % KT, which = (tid >> 1) & 1, hf = tid & 1, pl = tid / (4 * KT);
                    if (ki < nkb) {
                        const int row = __ldg(n2n + base + kb + ki);
                        const __half *src = which ? v : k;
                        pf_val = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)row * HC + slot_offset<HDM>(hp, hf, pl)));
                    }
                }
                if (pf_e < KT * D && pf_e / D < nkb) pf_c = __ldg(n_coords + (int64_t)(base + kb + pf_e / D) * D + pf_e % D);
            };
            fetch_tile(0);
            // the row loads are issued first and stored after the histogram has been cleared, so that
            // their latency overlaps the clearing
            const int st_qi = (tid >> 1) & 31, st_hf = tid & 1, st_pl = tid >> 6;
            const bool st_stage = tid < 64 * NPL;
            uint4 st_val = make_uint4(0, 0, 0, 0);
            int st_row = 0;
            if (st_stage && st_qi < nq) {
                st_row = __ldg(n2n + base + q0 + st_qi);
                st_val = __ldg(reinterpret_cast<const uint4 *>(q + (int64_t)st_row * HC + slot_offset<HDM>(hp, st_hf, st_pl)));
            }
            for (int i = tid; i < L.R16 * QT / 4; i += NTHREADS)
                reinterpret_cast<uint4 *>(s_hist)[i] = make_uint4(0, 0, 0, 0);
            if (st_stage) {
                if (st_qi < nq && st_hf == 0 && st_pl == 0) s_qrow[st_qi] = st_row;
                *reinterpret_cast<uint4 *>(s_q + st_pl * 512 + st_qi * 16 + st_hf * 8) = st_val;
            }
            __syncthreads();
            // block-diagonal B fragments of Q^T: n-tile j <-> (queries 4j..4j+3) x (slot 0, slot 1)
            uint32_t qB[NPL][8][2];
            uint32_t qS[NPL][2];   // the n-tile of Q^T this warp multiplies with K for the plain q.k scores
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t wq = *reinterpret_cast<const uint32_t *>(s_q + pl * 512 + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                    qB[pl][j][0] = (g & 1) ? 0u : wq;
                    qB[pl][j][1] = (g & 1) ? wq : 0u;
                }
                const uint32_t wq = *reinterpret_cast<const uint32_t *>(s_q + pl * 512 + (4 * (wid & 7) + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                qS[pl][0] = (g & 1) ? 0u : wq;
                qS[pl][1] = (g & 1) ? wq : 0u;
            }
            // P_q^T[row][(q, slot)] = Tq . Q^T, fp16 accumulate, stored as it comes out
#pragma unroll
            for (int i = 0; i < MTW; ++i) {
                const int mt = wid + NWARP * i;
                if (mt < n_mt) {
                    uint32_t d0[8], d1[8];
#pragma unroll
                    for (int pl = 0; pl < NPL; ++pl) {
                        uint32_t af[2][2];
                        if (PAIR16) {
                            load_table_a_frag<HDM>(af, tq, meta, HC, hp, pl, mt, g, t);
                        } else {
                            af[0][0] = tqA[i % MTP][0][0]; af[0][1] = tqA[i % MTP][0][1];
                            af[1][0] = tqA[i % MTP][1][0]; af[1][1] = tqA[i % MTP][1][1];
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (pl == 0) mma_k16_h(d0[j], d1[j], af[0][0], af[0][1], af[1][0], af[1][1], qB[pl][j][0], qB[pl][j][1]);
                            else mma_k16_ha(d0[j], d1[j], af[0][0], af[0][1], af[1][0], af[1][1], qB[pl][j][0], qB[pl][j][1]);
                        }
                    }
                    // query 4j+t sits in column 4t + j/2 (j even) or 16 + 4t + j/2 (j odd); odd rows of a
                    // quarter warp store their upper half first so that the eight lanes cover all banks
                    uint32_t *r0 = s_pq + (mt * 16 + g) * QT + 4 * t;
                    const bool od = g & 1;
                    const int o0 = od ? 16 : 0, o1 = 16 - o0;
                    const uint4 a0 = make_uint4(d0[0], d0[2], d0[4], d0[6]), a1 = make_uint4(d0[1], d0[3], d0[5], d0[7]);
                    const uint4 b0 = make_uint4(d1[0], d1[2], d1[4], d1[6]), b1 = make_uint4(d1[1], d1[3], d1[5], d1[7]);
                    *reinterpret_cast<uint4 *>(r0 + o0) = od ? a1 : a0;
                    *reinterpret_cast<uint4 *>(r0 + o1) = od ? a0 : a1;
                    *reinterpret_cast<uint4 *>(r0 + 8 * QT + o0) = od ? b1 : b0;
                    *reinterpret_cast<uint4 *>(r0 + 8 * QT + o1) = od ? b0 : b1;
                }
            }
            float m_run[2] = {-INFINITY, -INFINITY};
            float l_part[2] = {0.f, 0.f};
            // P.V accumulators [slot][m-tile][c-frag]; meaningful in warp 7 (plane 0) and, with two
            // planes, warp 6 (plane 1)
            float oacc[2][2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 2; ++i) oacc[h][i][0] = oacc[h][i][1] = oacc[h][i][2] = oacc[h][i][3] = 0.f;
            const bool pv_warp = wid == NWARP - 1 || (PAIR16 && wid == NWARP - 2);
            const int pv_plane = NWARP - 1 - wid;

            for (int k0 = 0; k0 < n; k0 += KT) {
                const int nk = min(KT, n - k0);
                __syncthreads();  // P_q stored / previous key tile fully consumed
                // ---- stage the key tile (fetched into registers one tile ahead) ------------------------
                if (tid < 4 * KT * NPL) {
                    const int ki = (tid >> 2) % KT, which = (tid >> 1) & 1, hf = tid & 1, pl = tid / (4 * KT);
                    *reinterpret_cast<uint4 *>((which ? s_v : s_k) + pl * KT * 16 + ki * 16 + hf * 8) = pf_val;
                }
                if (tid >= NTHREADS - 32) {
                    s_mtile[(tid - (NTHREADS - 32)) * 2] = -INFINITY;
                    s_mtile[(tid - (NTHREADS - 32)) * 2 + 1] = -INFINITY;
                }
                if (pf_e < KT * D) s_kc[(pf_e / D) * 12 + pf_e % D] = pf_c;
                __syncthreads();
                if (k0 + KT < n) fetch_tile(k0 + KT);      // in flight while this tile is worked on
                // ---- P_k^T[row][(key, slot)] = Tk . K^T -> s_pk[key][row];  S0^T[key][(q, slot)] = K . Q^T ----
                {
#pragma unroll
                    for (int j = 0; j < KT / 4; ++j) {
                        uint32_t b0[NPL], b1[NPL];
#pragma unroll
                        for (int pl = 0; pl < NPL; ++pl) {
                            const uint32_t wk = *reinterpret_cast<const uint32_t *>(s_k + pl * KT * 16 + (4 * j + (g >> 1)) * 16 + (g & 1) * 8 + 2 * t);
                            b0[pl] = (g & 1) ? 0u : wk;
                            b1[pl] = (g & 1) ? wk : 0u;
                        }
#pragma unroll
                        for (int i = 0; i < MTW; ++i) {
                            const int mt = wid + NWARP * i;
                            if (mt < n_mt) {
                                uint32_t d0, d1;
                                mma_k16_h(d0, d1, tkA[i][0][0][0], tkA[i][0][0][1], tkA[i][0][1][0], tkA[i][0][1][1], b0[0], b1[0]);
                                if (PAIR16)
                                    mma_k16_ha(d0, d1, tkA[i][NPL - 1][0][0], tkA[i][NPL - 1][0][1], tkA[i][NPL - 1][1][0], tkA[i][NPL - 1][1][1], b0[NPL - 1], b1[NPL - 1]);
                                uint32_t *dst = s_pk + (4 * j + t) * Rp + mt * 16 + g;
                                dst[0] = d0;
                                dst[8] = d1;
                            }
                        }
                    }
                    {   // one (16 keys, 4 queries x 2 slots) tile of S0 per warp
                        const int smt = wid >> 3, sj = wid & 7;
                        float c[4];
#pragma unroll
                        for (int pl = 0; pl < NPL; ++pl) {
                            const __half *kp = s_k + pl * KT * 16 + smt * 256;
                            const uint32_t a0 = *reinterpret_cast<const uint32_t *>(kp + g * 16 + 2 * t);
                            const uint32_t a1 = *reinterpret_cast<const uint32_t *>(kp + (g + 8) * 16 + 2 * t);
                            const uint32_t a2 = *reinterpret_cast<const uint32_t *>(kp + g * 16 + 8 + 2 * t);
                            const uint32_t a3 = *reinterpret_cast<const uint32_t *>(kp + (g + 8) * 16 + 8 + 2 * t);
                            if (pl == 0) mma_k16_z(c, a0, a1, a2, a3, qS[pl][0], qS[pl][1]);
                            else mma_k16(c, a0, a1, a2, a3, qS[pl][0], qS[pl][1]);
                        }
                        s_s[(16 * smt + g) * QT + 4 * sj + t] = make_float2(c[0], c[1]);
                        s_s[(16 * smt + g + 8) * QT + 4 * sj + t] = make_float2(c[2], c[3]);
                    }
                }
                __syncthreads();
                // ---- phase 1: scores of this warp's two keys --------------------------------------
                float mloc[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int kk2 = 0; kk2 < 2; ++kk2) {
                    const int kk = 2 * wid + kk2;
                    if (kk < nk) {
                        __half2 bq = __float2half2_rn(0.f), bk = __float2half2_rn(0.f);
                        uint32_t w0 = 0, w1 = 0;
#pragma unroll
                        for (int d = 0; d < D; ++d) {
                            const int idx = crse_index_fast(cq[d], s_kc[kk * 12 + d], meta.L[d], d == D - 1);
                            const int row = meta.rowbase[d] + idx;
                            bq = __hadd2(bq, u32_as_h2(s_pq[row * QT + mypos]));
                            bk = __hadd2(bk, u32_as_h2(s_pk[kk * Rp + row]));
                            if (d < 5) w0 |= (uint32_t)idx << (IDX_BITS * d);
                            else w1 |= (uint32_t)idx << (IDX_BITS * (d - 5));
                        }
                        s_idx[(kk * 2 + 0) * QT + lane] = w0;
                        if (D > 5) s_idx[(kk * 2 + 1) * QT + lane] = w1;
                        const float2 b = __half22float2(__hadd2(bq, bk));
                        float2 s = s_s[kk * QT + lane];
                        s.x += b.x;
                        s.y += b.y;
                        if (HD16) s.x = s.y = s.x + s.y;   // one head: both halves carry the full score
                        s_s[kk * QT + lane] = s;
                        mloc[0] = fmaxf(mloc[0], s.x);
                        mloc[1] = fmaxf(mloc[1], s.y);
                    }
                }
                if (2 * wid < nk) {
                    atomic_max_float(s_mtile + lane * 2, mloc[0]);
                    atomic_max_float(s_mtile + lane * 2 + 1, mloc[1]);
                }
                __syncthreads();
                // ---- phase 1.5: probabilities with the updated running maximum -----------------------
                float alpha[2];
                bool unchanged = true;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float mnew = fmaxf(m_run[h], s_mtile[lane * 2 + h]);
                    alpha[h] = exp2f((m_run[h] - mnew) * LOG2E);   // 0 on the first tile (m_run = -inf)
                    unchanged = unchanged && (mnew == m_run[h]);
                    m_run[h] = mnew;
                    l_part[h] *= alpha[h];
                }
                if (wid == 0) {
                    s_alpha[lane * 2] = alpha[0];
                    s_alpha[lane * 2 + 1] = alpha[1];
                }
#pragma unroll
                for (int kk2 = 0; kk2 < 2; ++kk2) {
                    const int kk = 2 * wid + kk2;
                    uint32_t ph = 0;
                    if (kk < nk) {
                        const float2 s = s_s[kk * QT + lane];
                        const float p0 = exp2f((s.x - m_run[0]) * LOG2E);
                        const float p1 = exp2f((s.y - m_run[1]) * LOG2E);
                        l_part[0] += p0;
                        l_part[1] += p1;
                        ph = h2_as_u32(__floats2half2_rn(p0, p1));
                    }
                    reinterpret_cast<uint32_t *>(s_s + kk * QT + lane)[0] = ph;  // p replaces s
                }
                const int any_changed = __syncthreads_or((k0 > 0 && !unchanged) ? 1 : 0);
                // ---- rescale what was accumulated under the old maximum ------------------------------
                if (any_changed) {
                    const int c4 = tid & 7;  // 16-byte column: queries {c4, c4+8, c4+16, c4+24}
                    __half2 a[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        a[j] = __floats2half2_rn(s_alpha[(c4 + 8 * j) * 2], s_alpha[(c4 + 8 * j) * 2 + 1]);
                    for (int r = tid >> 3; r < L.R16; r += NTHREADS / 8) {
                        uint4 x = *reinterpret_cast<uint4 *>(s_hist + r * QT + 4 * c4);
                        x.x = h2_as_u32(__hmul2(u32_as_h2(x.x), a[0]));
                        x.y = h2_as_u32(__hmul2(u32_as_h2(x.y), a[1]));
                        x.z = h2_as_u32(__hmul2(u32_as_h2(x.z), a[2]));
                        x.w = h2_as_u32(__hmul2(u32_as_h2(x.w), a[3]));
                        *reinterpret_cast<uint4 *>(s_hist + r * QT + 4 * c4) = x;
                    }
                    if (pv_warp) {
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const float a0 = s_alpha[(16 * i + g) * 2 + h], a1 = s_alpha[(16 * i + g + 8) * 2 + h];
                                oacc[h][i][0] *= a0; oacc[h][i][1] *= a0;
                                oacc[h][i][2] *= a1; oacc[h][i][3] *= a1;
                            }
                    }
                    __syncthreads();
                }
                // ---- phase 2: histogram update; a warp owns one or two signal dimensions ----------------
                {
                    int dA = -1, dB = -1;
                    if (D <= NWARP - 2) {
                        if (wid < D) dA = wid;
                    } else if (wid < D - 5) {
                        dA = wid; dB = wid + 5;     // one index field from each packed word
                    } else if (wid < 5) {
                        dA = wid;
                    }
                    if (dA >= 0) {
                        const int shA = IDX_BITS * (dA % 5), wA = dA / 5, rbA = meta.rowbase[dA];
                        const int shB = dB >= 0 ? IDX_BITS * (dB % 5) : 0, wB = dB >= 0 ? dB / 5 : 0;
                        const int rbB = dB >= 0 ? meta.rowbase[dB] : 0;
                        uint32_t *cell = s_hist + mypos;
                        for (int kk0 = 0; kk0 < nk; kk0 += 4) {
                            uint32_t pv[1][4];
                            int off2[2][4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int kk = kk0 + j;
                                pv[0][j] = reinterpret_cast<const uint32_t *>(s_s + kk * QT + lane)[0];   // 0 for padded keys
                                const bool ok = kk < nk;
                                const int ia = ok ? (s_idx[(kk * 2 + wA) * QT + lane] >> shA) & ((1 << IDX_BITS) - 1) : 0;
                                off2[0][j] = (rbA + ia) * QT;
                                const int ib = (ok && dB >= 0) ? (s_idx[(kk * 2 + wB) * QT + lane] >> shB) & ((1 << IDX_BITS) - 1) : 0;
                                off2[1][j] = (rbB + ib) * QT;
                            }
                            if (dB >= 0) {
                                hist_add4<2, 1>(cell, 0, off2, pv, nk - kk0);
                            } else {
                                int off1[1][4] = {{off2[0][0], off2[0][1], off2[0][2], off2[0][3]}};
                                hist_add4<1, 1>(cell, 0, off1, pv, nk - kk0);
                            }
                        }
                    }
                }
                // ---- O += P.V on the tensor cores (warp 7; with two planes also warp 6) -----------------
                if (pv_warp) {
                    const __half *vp = s_v + pv_plane * KT * 16;
#pragma unroll
                    for (int ks = 0; ks < KT / 16; ++ks) {
                        if (16 * ks < nk) {
                            uint32_t pa[2][2][4];  // [slot][m-tile][a0..a3]
#pragma unroll
                            for (int i = 0; i < 2; ++i)
#pragma unroll
                                for (int kh = 0; kh < 2; ++kh)      // keys 2t.. / keys 2t+8..
#pragma unroll
                                    for (int rr = 0; rr < 2; ++rr) { // query 16i+g / 16i+g+8
                                        const int qq = 16 * i + g + 8 * rr, ka = 16 * ks + 2 * t + 8 * kh;
                                        const uint32_t x = reinterpret_cast<const uint32_t *>(s_s + ka * QT + qq)[0];
                                        const uint32_t y = reinterpret_cast<const uint32_t *>(s_s + (ka + 1) * QT + qq)[0];
                                        pa[0][i][2 * kh + rr] = pack_lo(x, y);
                                        pa[1][i][2 * kh + rr] = pack_hi(x, y);
                                    }
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t vb[2];
#pragma unroll
                                for (int kh = 0; kh < 2; ++kh) {
                                    const int ka = 16 * ks + 2 * t + 8 * kh;
                                    vb[kh] = h2_as_u32(__halves2half2(vp[ka * 16 + h * 8 + g], vp[(ka + 1) * 16 + h * 8 + g]));
                                }
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    mma_k16(oacc[h][i], pa[h][i][0], pa[h][i][1], pa[h][i][2], pa[h][i][3], vb[0], vb[1]);
                            }
                        }
                    }
                }
            }  // key tiles
            __syncthreads();
            // ---- per plane: O += hist . Tv (K split over the warps), reduce, normalise and store ------------
#pragma unroll
            for (int pl = 0; pl < NPL; ++pl) {
                float part[2][2][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
#pragma unroll
                        for (int e = 0; e < 4; ++e) part[h][i][e] = (wid == NWARP - 1 - pl) ? oacc[h][i][e] : 0.f;
#pragma unroll
                for (int i = 0; i < MTW; ++i) {
                    const int ks = wid + NWARP * i;
                    if (ks < n_mt) {
                        uint32_t bf[2][2];
                        if (PAIR16) {
                            load_table_b_frag<HDM>(bf, tv, meta, HC, hp, pl, ks, g, t);
                        } else {
                            bf[0][0] = tvB[i % MTP][0][0]; bf[0][1] = tvB[i % MTP][0][1];
                            bf[1][0] = tvB[i % MTP][1][0]; bf[1][1] = tvB[i % MTP][1][1];
                        }
                        ht_unit(part, s_hist, bf, ks, g, t);
                    }
                }
                // s_red aliases s_pk, which nobody reads after the last phase 1 (a barrier ago); the
                // second plane waits until the first one's reduction has been read
                if (pl > 0) __syncthreads();
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 2; ++i)
#pragma unroll
                        for (int rr = 0; rr < 2; ++rr) {
                            const int qq = 16 * i + g + 8 * rr;
                            *reinterpret_cast<float2 *>(s_red + (wid * QT + qq) * 16 + h * 8 + 2 * t) =
                                make_float2(part[h][i][2 * rr], part[h][i][2 * rr + 1]);
                        }
                if (pl == 0) {
                    s_lsum[(wid * QT + lane) * 2] = l_part[0];
                    s_lsum[(wid * QT + lane) * 2 + 1] = l_part[1];
                    if (wid == 0) {   // final maxima for the log-sum-exp
                        s_mtile[lane * 2] = m_run[0];
                        s_mtile[lane * 2 + 1] = m_run[1];
                    }
                }
                __syncthreads();
                {
                    const int qq = tid >> 3, ch = (tid & 7) * 2, h = ch >> 3;
                    if (qq < nq) {          // qq >= 32 (warps 8..15 of a 16-warp block) never passes: nq <= 32
                        float a = 0.f, b = 0.f, ls = 0.f;
#pragma unroll
                        for (int ww = 0; ww < NWARP; ++ww) {
                            const float2 pr = *reinterpret_cast<const float2 *>(s_red + (ww * QT + qq) * 16 + ch);
                            a += pr.x;
                            b += pr.y;
                            ls += s_lsum[(ww * QT + qq) * 2 + h];
                        }
                        const float inv = 1.f / ls;
                        const int64_t row = s_qrow[qq];
                        store_h2_mirrored(out, m_out, row * HC + slot_offset<HDM>(hp, h, pl) + (ch & 7),
                                          __floats2half2_rn(a * inv, b * inv));
                        if (pl == 0) {
                            if (HD16) {
                                if (ch == 0) lse[row * H + hp] = s_mtile[qq * 2] + __logf(ls);
                            } else if ((ch & 7) == 0) {
                                lse[row * H + 2 * hp + h] = s_mtile[qq * 2 + h] + __logf(ls);
                            }
                        }
                    }
                }
            }  // planes
        }  // items
    }      // chunks of windows
}

template <int D, int MTW, int HDM, int NW>
static int launch(const AttnArgs &a, int skip_upto, cudaStream_t st)
{
    constexpr int NTHREADS = NW * 32;
    const SmemLayout L = make_layout(a.meta.R, 1, HDM == HDM_PAIR16 ? 2 : 1, NW);
    auto kern = attn_fwd_tc_kernel<D, MTW, HDM, NW>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    const int hp = HDM == HDM_SINGLE16 ? a.H : a.H / 2;
    int dev = 0, sms = 148, per_sm = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NTHREADS, L.total) != cudaSuccess || per_sm < 1)
        return S3D_ERR_LAUNCH;
    // exactly one wave of resident blocks, shared evenly between the head pairs
    int gx = sms * per_sm / hp;
    if (gx > a.W) gx = (int)a.W;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)hp);
    kern<<<grid, NTHREADS, L.total, st>>>(
        (const __half *)a.q, (const __half *)a.k, (const __half *)a.v, (const __half *)a.tq,
        (const __half *)a.tk, (const __half *)a.tv, a.meta, a.w_sizes, a.w2n, a.n2n, a.n_coords, a.W,
        a.H, skip_upto, (__half *)a.out, a.lse, a.m_out);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

template <int D, int MTW, int NW>
static int launch_mode(const AttnArgs &a, int hdm, int skip_upto, cudaStream_t st)
{
    switch (hdm) {
        case HDM_PAIR8: return launch<D, MTW, HDM_PAIR8, NW>(a, skip_upto, st);
        case HDM_SINGLE16: return launch<D, MTW, HDM_SINGLE16, NW>(a, skip_upto, st);
        default: return launch<D, MTW, HDM_PAIR16, NW>(a, skip_upto, st);
    }
}

// Warps per block for a table of R (internal) rows: 16 (one block per SM, 32-key tiles, one signal
// dimension per warp in the histogram phase) whenever its shared memory fits, which measured 7 %
// faster than two 8-warp blocks per SM even where those fit; else 8.
static int warps_per_block(int R, int planes)
{
    return make_layout(R, 1, planes, 16).total <= 227 * 1024 ? 16 : 8;
}

}  // namespace tc

// Head mode of the tiled kernels for a call (see attn_tc.cuh).
int attn_tc_head_mode(const AttnArgs &a)
{
    if (a.hd == 8) return tc::HDM_PAIR8;
    return (a.H & 1) ? tc::HDM_SINGLE16 : tc::HDM_PAIR16;
}

bool attn_tc_supported(const AttnArgs &a)
{
    if (a.dtype != S3D_F16) return false;
    if (!(a.hd == 16 || (a.hd == 8 && !(a.H & 1)))) return false;
    const int Rint = a.meta.R + a.meta.D - 1;
    if (Rint > 16 * tc::NWARP * 3) return false;
    for (int d = 0; d < a.meta.D; ++d)
        if (a.meta.L[d] >= (1 << tc::IDX_BITS)) return false;   // idx may reach L
    if (tc::make_layout(Rint, 1, 2, 8).total > 227 * 1024) return false;
    return true;
}

int attn_tc_forward(const AttnArgs &a0, cudaStream_t st)
{
    if (a0.W == 0) return S3D_OK;
    AttnArgs a = a0;
    a.meta = tc::internal_meta(a0.meta);   // kernels work in the internal row numbering
    const int hdm = attn_tc_head_mode(a0);
    int skip_upto = 0;
    // the single-tile kernel serves head pairs of 8 channels and single heads of 16
    if (hdm != tc::HDM_PAIR16 && attn_tc_fwd_small_supported(a0)) {
        // window_class: the caller's word that every window has at most QT voxels (1) or more (2); each
        // kernel otherwise walks the whole list to find its own windows
        if (a0.window_class != 2) {
            const int rc = attn_tc_forward_small(a0, st);
            if (rc != S3D_OK) return rc;
        }
        if (a0.window_class == 1) return S3D_OK;
        skip_upto = tc::QT;
    }
    const int n_mt = (a.meta.R + 15) / 16;
    const int nw = tc::warps_per_block(a.meta.R, hdm == tc::HDM_PAIR16 ? 2 : 1);
    const int mtw = (n_mt + nw - 1) / nw;
#define S3D_TC_FWD(DD)                                            \
    switch (nw == 8 ? mtw : 10 + mtw) {                           \
        case 1: return tc::launch_mode<DD, 1, 8>(a, hdm, skip_upto, st); \
        case 2: return tc::launch_mode<DD, 2, 8>(a, hdm, skip_upto, st); \
        case 3: return tc::launch_mode<DD, 3, 8>(a, hdm, skip_upto, st); \
        case 11: return tc::launch_mode<DD, 1, 16>(a, hdm, skip_upto, st); \
        case 12: return tc::launch_mode<DD, 2, 16>(a, hdm, skip_upto, st); \
        default: return S3D_ERR_UNSUPPORTED;                      \
    }
    switch (a.meta.D) {
        case 3: S3D_TC_FWD(3)
        case 6: S3D_TC_FWD(6)
        case 9: S3D_TC_FWD(9)
        default: return S3D_ERR_UNSUPPORTED;
    }
#undef S3D_TC_FWD
}

}  // namespace s3d
