// Brute-force K-nearest-neighbour search, one scene per batch entry.
//
// Result semantics are those of the reference kernel (microsoft/Swin3D,
// Swin3D/src/knn/knn_cuda_kernel.cu:29-62,139-204): every query scans the source points of its
// own scene in ascending index order, keeps a K-entry max-heap that is replaced only by a
// strictly smaller distance, and heap-sorts at the end.  Reproducing that exact sequence per
// query (including the sift-down's behaviour on equal keys) is what makes indices bit-identical
// to the reference even when distances tie.
//
// What differs is the data path: a block of queries streams its scene's source points through
// shared memory in tiles (one read per point per block instead of one per thread) stored as four
// planes x, y, z, |p|^2, so that one broadcast 16-byte shared load returns a coordinate of four
// candidates.  The scan does not evaluate the reference's distance for every candidate: it
// evaluates a rounded lower bound of it (three packed two-candidate fma.f32x2 per pair of
// candidates, see "the filter" below) and compares the smallest of eight with a threshold derived
// from the heap root -- one compare per eight candidates in the common "none can be closer" case.
// Candidates that pass are parked in a small per-thread queue in shared memory and offered to the
// heap later, in index order, with the reference's own distance expression and against the then
// current root, by all lanes of the warp at the same time: the heap sees exactly the reference's
// sequence of replacements (a parked candidate that does not beat the root is dropped, as it would
// have been in its turn), but the divergent sift-downs of different lanes overlap instead of
// running one after the other.
#include <type_traits>

#include "common.cuh"
#include "knn_kernels.cuh"

namespace s3d {

constexpr int KNN_TILE = 768;          // source points per shared-memory tile (a multiple of KNN_STEP)
constexpr int KNN_STEP = 8;            // candidates per step of the scan

__device__ __forceinline__ void knn_sift_down(float *heap, int *idx, int start, int end)
{
    int curr = start;
    int child = curr * 2 + 1;
    while (child < end) {
        if (child + 1 < end && heap[child] < heap[child + 1]) child++;
        if (heap[curr] > heap[child]) return;
        const float tf = heap[curr]; heap[curr] = heap[child]; heap[child] = tf;
        const int ti = idx[curr]; idx[curr] = idx[child]; idx[child] = ti;
        curr = child;
        child = curr * 2 + 1;
    }
}

// fp32 squared distance.  The reference writes dx*dx + dy*dy + dz*dz and lets nvcc contract it;
// its compiled kernel (nvcc 12.9, default -fmad=true, sm_100) evaluates
// fma(dz,dz, fma(dx,dx, dy*dy)), established by comparing bit patterns of its output with the
// three possible contractions.  The expression is spelled with intrinsics so that it cannot
// drift with compiler versions; the GPU parity test re-checks it against the compiled reference.
__device__ __forceinline__ float knn_dist2(float dx, float dy, float dz)
{
    return __fmaf_rn(dz, dz, __fmaf_rn(dx, dx, __fmul_rn(dy, dy)));
}

// Two candidates per instruction: element 0 in the low half of the 64-bit register.
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// min of three that returns NaN when an input is NaN (a NaN bound must reach the exact test)
__device__ __forceinline__ float min3_nan(float a, float b, float c)
{
    float r;
    asm("min.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- the filter ---------------------------------------------------------------------------------
// The scan does not evaluate the reference's distance for every candidate.  It evaluates
//     bound = |p|^2 - 2 p.q        (three packed fma; |p|^2 is computed once per point per tile)
// and compares it with  thr = top - |q|^2 + margin.  In exact arithmetic bound + |q|^2 is the squared
// distance D.  Rounding: the stored |p|^2 and the three fma are each within one rounding of a value
// not larger than (|p| + |q|)^2, so |bound - (D - |q|^2)| < 7 eps (|p| + |q|)^2 (eps = 2^-24); the
// reference's own result d = fl(dz*dz + (dx*dx + dy*dy)) with rounded differences is within 5 eps D
// of D; |q|^2 as computed here is within 3 eps |q|^2.  With
//     margin = 32 eps (pmax + |q|)^2 + 16 eps top + 1e-36,   pmax >= |p| for every point seen so far,
// "bound >= thr" therefore implies d >= top, i.e. the reference would not have inserted the
// candidate.  Everything else (bound < thr, or a NaN) is parked and decided by the exact distance
// against the heap, so a loose margin only costs a few extra exact evaluations, never a result.
__device__ __forceinline__ float knn_threshold(float top, float sq, float pmax2)
{
    const float eps = 5.9604645e-8f;
    const float r = sqrtf(pmax2) + sqrtf(sq);
    const float margin = 32.f * eps * r * r + 16.f * eps * top + 1e-36f;   // the last term covers subnormal roundings
    const float thr = (top - sq) + margin;
    // non-finite magnitudes (coordinates beyond 1e19): no filtering, every candidate is decided exactly
    return (pmax2 < 1e37f && sq < 1e37f) ? thr : __int_as_float(0x7f800000);
}

// One thread owns NQ queries (g, g + NT, ...): a candidate read from shared memory serves all of
// them -- the broadcast loads are what the scan is otherwise bound by.
// QCAP: parked candidates per query; the queue is drained when a whole step may not fit.
// The heaps are thread-private arrays (local memory beyond a few entries; heaps in shared memory as
// [entry][thread] were measured at the same speed for K = 16: the cost there is the number of heap
// updates, K (1 + ln(N / K)) per query, each entered by a whole warp).
template <int KMAX, int NQ, int NT, int QCAP>
__global__ void __launch_bounds__(NT)
knn_kernel(int K, const float *__restrict__ src, const float *__restrict__ query,
           const int32_t *__restrict__ src_offset, const int32_t *__restrict__ query_offset,
           int B, int64_t Nq, int32_t *__restrict__ ret_idx, float *__restrict__ ret_dist)
{
    // planes x, y, z, |p|^2 of a tile; a step may read past the last point
    __shared__ __align__(16) float s_p[4][KNN_TILE + KNN_STEP];
    __shared__ int s_qi[NQ * QCAP * NT];       // parked candidates (source rows), [query][slot][thread]
    __shared__ int s_lo, s_hi;
    __shared__ unsigned s_pmax;                    // bits of the largest |p|^2 loaded so far

    const int64_t g0 = (int64_t)blockIdx.x * (NT * NQ) + threadIdx.x;

    float heap[NQ][KMAX];
    int hidx[NQ][KMAX];
    float qx[NQ], qy[NQ], qz[NQ], sq[NQ], thr[NQ];
    uint64_t a2[NQ], b2[NQ], c2[NQ];
    int s0[NQ], s1[NQ], qn[NQ];
    bool active[NQ];
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
#pragma unroll
        for (int i = 0; i < KMAX; ++i) {
            heap[r][i] = 2147483648.0f;  // (float)0x7fffffff
            hidx[r][i] = 0;
        }
        const int64_t g = g0 + (int64_t)r * NT;
        active[r] = g < Nq;
        qx[r] = qy[r] = qz[r] = 0.f;
        s0[r] = s1[r] = 0;
        qn[r] = 0;
        if (active[r]) {
            qx[r] = __ldg(query + g * 3);
            qy[r] = __ldg(query + g * 3 + 1);
            qz[r] = __ldg(query + g * 3 + 2);
            int b = 0;
            for (; b < B; ++b)
                if (g < __ldg(query_offset + b)) break;
            if (b >= B) b = B - 1;
            s0[r] = b > 0 ? __ldg(src_offset + b - 1) : 0;
            s1[r] = __ldg(src_offset + b);
        }
        a2[r] = pack2(-2.f * qx[r], -2.f * qx[r]);
        b2[r] = pack2(-2.f * qy[r], -2.f * qy[r]);
        c2[r] = pack2(-2.f * qz[r], -2.f * qz[r]);
        sq[r] = __fmaf_rn(qz[r], qz[r], __fmaf_rn(qy[r], qy[r], __fmul_rn(qx[r], qx[r])));
    }
    if (threadIdx.x == 0) { s_lo = 0x7fffffff; s_hi = 0; s_pmax = 0u; }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < NQ; ++r)
        if (active[r] && s1[r] > s0[r]) {
            atomicMin(&s_lo, s0[r]);
            atomicMax(&s_hi, s1[r]);
        }
    __syncthreads();
    const int lo = s_lo, hi = s_hi;
    float pmax2 = 0.f;

    // offer the parked candidates of every query to its heap, oldest first; every lane of the warp
    // takes part
    auto drain = [&]() {
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            const int most = __reduce_max_sync(0xffffffffu, qn[r]);
            const int *qi = s_qi + r * (QCAP * NT) + threadIdx.x;
            for (int e = 0; e < most; ++e) {
                if (e < qn[r]) {
                    // the reference's distance, from the source row
                    const int si = qi[e * NT];
                    const float *p = src + (int64_t)si * 3;
                    const float d = knn_dist2(__ldg(p) - qx[r], __ldg(p + 1) - qy[r], __ldg(p + 2) - qz[r]);
                    if (d < heap[r][0]) {
                        heap[r][0] = d;
                        hidx[r][0] = si;
                        knn_sift_down(heap[r], hidx[r], 0, K);
                    }
                }
            }
            qn[r] = 0;
            thr[r] = knn_threshold(heap[r][0], sq[r], pmax2);
        }
    };

    for (int t0 = lo; t0 < hi; t0 += KNN_TILE) {
        const int cnt = min(KNN_TILE, hi - t0);
        __syncthreads();
        {
            float mx = 0.f;
            for (int i = threadIdx.x; i < cnt; i += NT) {
                const float *p = src + (int64_t)(t0 + i) * 3;
                const float x = __ldg(p), y = __ldg(p + 1), z = __ldg(p + 2);
                const float n2 = __fmaf_rn(z, z, __fmaf_rn(y, y, __fmul_rn(x, x)));
                s_p[0][i] = x; s_p[1][i] = y; s_p[2][i] = z; s_p[3][i] = n2;
                mx = n2 > mx || n2 != n2 ? n2 : mx;                   // a NaN sticks
            }
            // |p|^2 >= 0: the unsigned order of the bits is the order of the values, NaN above infinity
            const unsigned wm = __reduce_max_sync(0xffffffffu, __float_as_uint(mx) & 0x7fffffffu);
            if ((threadIdx.x & 31) == 0) atomicMax(&s_pmax, wm);
        }
        __syncthreads();
        pmax2 = __uint_as_float(s_pmax);
        if (!(pmax2 == pmax2)) pmax2 = __int_as_float(0x7f800000);
        int jb[NQ], je[NQ];
        int jb_w = 0x7fffffff, je_w = 0;
#pragma unroll
        for (int r = 0; r < NQ; ++r) {
            thr[r] = knn_threshold(heap[r][0], sq[r], pmax2);
            // clip the tile to the query's own scene
            jb[r] = max(s0[r] - t0, 0);
            je[r] = min(s1[r] - t0, cnt);
            jb_w = min(jb_w, jb[r]);
            je_w = max(je_w, je[r]);
        }
        // every lane walks the same steps (queries of other scenes idle) so that the warp can drain together
        jb_w = __reduce_min_sync(0xffffffffu, jb_w);
        je_w = __reduce_max_sync(0xffffffffu, je_w);
        // KNN_STEP candidates per step and query: one test for "none can be closer than the heap root"
        // (the common case); the others are parked.  Steps start on a multiple of four points
        // (16-byte loads from the planes).  CLIP: the step may stick out of a query's scene.
        auto step = [&](int j, auto clip) {
            constexpr bool CLIP = decltype(clip)::value;
            ulonglong2 cx[KNN_STEP / 4], cy[KNN_STEP / 4], cz[KNN_STEP / 4], cn[KNN_STEP / 4];
#pragma unroll
            for (int u = 0; u < KNN_STEP / 4; ++u) {
                cx[u] = *reinterpret_cast<const ulonglong2 *>(&s_p[0][j + 4 * u]);
                cy[u] = *reinterpret_cast<const ulonglong2 *>(&s_p[1][j + 4 * u]);
                cz[u] = *reinterpret_cast<const ulonglong2 *>(&s_p[2][j + 4 * u]);
                cn[u] = *reinterpret_cast<const ulonglong2 *>(&s_p[3][j + 4 * u]);
            }
            float dd[NQ][KNN_STEP];
            bool some = false;
#pragma unroll
            for (int r = 0; r < NQ; ++r) {
#pragma unroll
                for (int u = 0; u < KNN_STEP / 4; ++u) {
                    unpack2(fma2(a2[r], cx[u].x, fma2(b2[r], cy[u].x, fma2(c2[r], cz[u].x, cn[u].x))),
                            dd[r][4 * u], dd[r][4 * u + 1]);
                    unpack2(fma2(a2[r], cx[u].y, fma2(b2[r], cy[u].y, fma2(c2[r], cz[u].y, cn[u].y))),
                            dd[r][4 * u + 2], dd[r][4 * u + 3]);
                }
                float m = min3_nan(dd[r][0], dd[r][1], dd[r][2]);
#pragma unroll
                for (int u = 3; u + 1 < KNN_STEP; u += 2) m = min3_nan(m, dd[r][u], dd[r][u + 1]);
                m = min3_nan(m, dd[r][KNN_STEP - 1], dd[r][KNN_STEP - 1]);
                some = some || !(m >= thr[r]);
            }
            // the whole warp enters the parking code together (or, mostly, not at all)
            if (__any_sync(0xffffffffu, some)) {
                bool full = false;
#pragma unroll
                for (int r = 0; r < NQ; ++r) {
                    int *qi = s_qi + r * (QCAP * NT) + threadIdx.x;
#pragma unroll
                    for (int u = 0; u < KNN_STEP; ++u) {
                        const bool inside = !CLIP || (j + u >= jb[r] && j + u < je[r]);
                        if (inside && !(dd[r][u] >= thr[r])) {
                            qi[qn[r] * NT] = t0 + j + u;
                            ++qn[r];
                        }
                    }
                    full = full || qn[r] > QCAP - KNN_STEP;
                }
                if (__any_sync(0xffffffffu, full)) drain();
            }
        };
        // all queries of the warp in one scene that covers the tile: no clipping except at the ends
        bool same = true;
#pragma unroll
        for (int r = 0; r < NQ; ++r) same = same && jb[r] == jb_w && je[r] == je_w;
        same = __all_sync(0xffffffffu, same);
        int j = jb_w & ~3;
        if (same) {
            if (j < jb_w) { step(j, std::true_type{}); j += KNN_STEP; }
            for (; j + KNN_STEP <= je_w; j += KNN_STEP) step(j, std::false_type{});
        }
        for (; j < je_w; j += KNN_STEP) step(j, std::true_type{});
    }
    drain();
#pragma unroll
    for (int r = 0; r < NQ; ++r) {
        if (!active[r]) continue;
        const int64_t g = g0 + (int64_t)r * NT;
        for (int i = K - 1; i > 0; --i) {
            const float tf = heap[r][0]; heap[r][0] = heap[r][i]; heap[r][i] = tf;
            const int ti = hidx[r][0]; hidx[r][0] = hidx[r][i]; hidx[r][i] = ti;
            knn_sift_down(heap[r], hidx[r], 0, i);
        }
        for (int i = 0; i < K; ++i) {
            ret_dist[g * K + i] = heap[r][i];
            ret_idx[g * K + i] = hidx[r][i];
        }
    }
}

template <int KMAX, int NQ, int NT, int QCAP>
static int knn_launch_as(int K, const float *src, const float *query, const int32_t *src_offset,
                         const int32_t *query_offset, int B, int64_t Nq, int32_t *ret_idx, float *ret_dist,
                         cudaStream_t st)
{
    const unsigned blocks = (unsigned)((Nq + NT * NQ - 1) / (NT * NQ));
    knn_kernel<KMAX, NQ, NT, QCAP><<<blocks, NT, 0, st>>>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

int knn_launch(int K, const float *src, const float *query, const int32_t *src_offset,
               const int32_t *query_offset, int B, int64_t Nq, int32_t *ret_idx, float *ret_dist,
               cudaStream_t st)
{
    if (Nq == 0) return S3D_OK;
    // few neighbours: the scan dominates, two queries per thread halve its shared-memory loads;
    // more neighbours: heap updates dominate, one query per thread keeps more warps resident
    // a short query list (a rank's share of a split call) does not fill the SMs with blocks of 256
    // queries: smaller blocks of one query per thread keep more warps resident (measured on 200 k to
    // 1.6 M queries: the smaller blocks win below about 300 k queries for K <= 4, 600 k for K <= 16)
    if (K <= 4) {
        if (Nq < 300000) return knn_launch_as<4, 1, 128, KNN_STEP + 4>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist, st);
        return knn_launch_as<4, 2, 128, KNN_STEP + 4>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist, st);
    }
    if (K <= 16) {
        if (Nq < 600000) return knn_launch_as<16, 1, 128, KNN_STEP + 4>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist, st);
        return knn_launch_as<16, 1, 256, KNN_STEP + 4>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist, st);
    }
    return knn_launch_as<64, 1, 256, KNN_STEP + 4>(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist, st);
}

}  // namespace s3d
