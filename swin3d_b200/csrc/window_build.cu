// Window builder: groups the voxels of a sparse batch into (shifted) cubic windows.
//
// It replaces the reference's chain of MinkowskiEngine pooling, insert_and_map, kernel_map,
// torch.sort and cumsum (microsoft/Swin3D, Swin3D/modules/swin3d_layers.py:713-822 and
// :76-150) with: one 64-bit key per voxel  (batch | wx | wy | wz | cell id),  a stable LSD
// radix sort of (key, voxel id), head flags where the window part of the key changes, and
// prefix sums.  Window of a voxel = floor((coord + shift*stride) / (ws*stride)) per axis;
// cell id = cx*ws^2 + cy*ws + cz  (meshgrid 'ij' order of swin3d_layers.py:724-730,779-786).
// Windows come out in lexicographic (batch, wx, wy, wz) order.
//
// All kernels are plain integer/byte work bound by HBM bandwidth: keys are read and written
// with coalesced accesses, digit ranking uses warp match + shared counters.  The batch and window
// fields of the key are packed as tightly as the batch at hand allows (a reduction finds their
// ranges first), so a typical batch sorts in four 8-bit passes instead of seven; the passes above
// the highest used bit exit at once, and passes whose digit is identical for every key are skipped
// on the device (no host round trip).
#include <climits>
#include <mutex>

#include "common.cuh"
#include "window_kernels.cuh"

namespace s3d {

constexpr int WB_THREADS = 256;
constexpr int WB_ITEMS = 8;
constexpr int WB_TILE = WB_THREADS * WB_ITEMS;  // keys per block in the radix passes
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 4;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

constexpr int CELL_BITS = 9, W_BITS = 15, B_BITS = 10;
constexpr int W_BIAS = 1 << (W_BITS - 1);
constexpr int NPASS = 8;

__device__ __forceinline__ int floor_div(int a, int b) { int q = a / b; return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q; }

// ---- keys ------------------------------------------------------------------------------------
struct VoxelWindow {
    int b, wx, wy, wz, cell;
};

__device__ __forceinline__ VoxelWindow voxel_window(const int32_t *__restrict__ coords, int64_t i, int stride, int ws, int shift)
{
    const int4 c = __ldg(reinterpret_cast<const int4 *>(coords) + i);  // b, x, y, z
    const int wstride = ws * stride;
    const int sx = c.y + shift * stride, sy = c.z + shift * stride, sz = c.w + shift * stride;
    VoxelWindow v;
    v.b = c.x;
    v.wx = floor_div(sx, wstride); v.wy = floor_div(sy, wstride); v.wz = floor_div(sz, wstride);
    const int cx = (sx - v.wx * wstride) / stride, cy = (sy - v.wy * wstride) / stride,
              cz = (sz - v.wz * wstride) / stride;
    v.cell = (cx * ws + cy) * ws + cz;
    return v;
}

// range[0..3] = min of (batch, wx, wy, wz), range[4..7] = max; also flags coordinates outside the
// supported range (batch < 2^10, |window index| < 2^14, cell id < 2^9)
__global__ void wb_range_kernel(const int32_t *__restrict__ coords, int64_t N, int stride, int ws, int shift,
                                int *__restrict__ range, int64_t *__restrict__ counts)
{
    int lo[4] = {INT_MAX, INT_MAX, INT_MAX, INT_MAX}, hi[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (int64_t)gridDim.x * blockDim.x) {
        const VoxelWindow v = voxel_window(coords, i, stride, ws, shift);
        const int f[4] = {v.b, v.wx, v.wy, v.wz};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            lo[k] = min(lo[k], f[k]);
            hi[k] = max(hi[k], f[k]);
        }
        const int bx = v.wx + W_BIAS, by = v.wy + W_BIAS, bz = v.wz + W_BIAS;
        bad = bad || v.b < 0 || v.b >= (1 << B_BITS) || bx < 0 || bx >= (1 << W_BITS) || by < 0 ||
              by >= (1 << W_BITS) || bz < 0 || bz >= (1 << W_BITS) || v.cell >= (1 << CELL_BITS);
    }
    // warp, then block, then one set of atomics per block
    __shared__ int s_lo[4], s_hi[4];
    if (threadIdx.x < 4) {
        s_lo[threadIdx.x] = INT_MAX;
        s_hi[threadIdx.x] = INT_MIN;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        lo[k] = __reduce_min_sync(0xffffffffu, lo[k]);
        hi[k] = __reduce_max_sync(0xffffffffu, hi[k]);
    }
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            atomicMin(s_lo + k, lo[k]);
            atomicMax(s_hi + k, hi[k]);
        }
    }
    __syncthreads();
    if (threadIdx.x < 4) {
        atomicMin(range + threadIdx.x, s_lo[threadIdx.x]);
        atomicMax(range + 4 + threadIdx.x, s_hi[threadIdx.x]);
    }
    if (bad) counts[3] = 1;  // coordinate outside the representable range
}

__device__ __forceinline__ int bits_for(int span) { return span > 0 ? 32 - __clz(span) : 0; }

// key = (batch - min | wx - min | wy - min | wz - min | cell), the first four fields as wide as their
// spans need.  live[p] = 1 for the radix passes that cover a used bit.
__global__ void wb_keys_kernel(const int32_t *__restrict__ coords, int64_t N, int stride, int ws,
                               int shift, const int *__restrict__ range, uint64_t *__restrict__ keys,
                               uint32_t *__restrict__ vals, int *__restrict__ live)
{
    const int wbx = bits_for(range[5] - range[1]), wby = bits_for(range[6] - range[2]), wbz = bits_for(range[7] - range[3]);
    const int wbb = bits_for(range[4] - range[0]);
    if (blockIdx.x == 0 && threadIdx.x < NPASS) {
        // spans are clamped by the range check (10 + 3*15 + 9 = 64 bits at most)
        const int total = min(64, wbb + wbx + wby + wbz + CELL_BITS);
        live[threadIdx.x] = 8 * threadIdx.x < total ? 1 : 0;
    }
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const VoxelWindow v = voxel_window(coords, i, stride, ws, shift);
    uint64_t key = (uint64_t)(uint32_t)(v.b - range[0]) & ((1ull << B_BITS) - 1);
    key = (key << wbx) | ((uint64_t)(uint32_t)(v.wx - range[1]) & ((1ull << W_BITS) - 1));
    key = (key << wby) | ((uint64_t)(uint32_t)(v.wy - range[2]) & ((1ull << W_BITS) - 1));
    key = (key << wbz) | ((uint64_t)(uint32_t)(v.wz - range[3]) & ((1ull << W_BITS) - 1));
    key = (key << CELL_BITS) | (uint32_t)(v.cell & ((1 << CELL_BITS) - 1));
    keys[i] = key;
    vals[i] = (uint32_t)i;
}

// ---- generic exclusive scan of uint32 (three kernels) ------------------------------------------
__device__ __forceinline__ uint32_t block_scan_incl(uint32_t x, uint32_t *s_warp, uint32_t &total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
        uint32_t v = lane < (SCAN_THREADS / 32) ? s_warp[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += y;
        }
        if (lane < (SCAN_THREADS / 32)) s_warp[lane] = v;
    }
    __syncthreads();
    total = s_warp[SCAN_THREADS / 32 - 1];
    const uint32_t prefix = warp > 0 ? s_warp[warp - 1] : 0;
    __syncthreads();
    return x + prefix;
}

// `gate`: optional flag in device memory; the kernel does nothing when it is zero (a radix pass that
// is known to have nothing to sort)
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tile_sums_kernel(const uint32_t *__restrict__ in, int64_t n, uint32_t *__restrict__ sums, const int *__restrict__ gate)
{
    if (gate && !*gate) return;
    __shared__ uint32_t s_warp[SCAN_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    uint32_t t = 0;
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS; ++j)
        if (base + j < n) t += in[base + j];
    uint32_t total;
    block_scan_incl(t, s_warp, total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

// single block: exclusive scan of sums[0..m) in place; sums[m] receives the grand total
__global__ void __launch_bounds__(SCAN_THREADS)
scan_sums_kernel(uint32_t *__restrict__ sums, int64_t m, const int *__restrict__ gate)
{
    if (gate && !*gate) return;
    __shared__ uint32_t s_warp[SCAN_THREADS / 32];
    uint32_t carry = 0;
    for (int64_t b0 = 0; b0 < m; b0 += SCAN_THREADS) {
        const int64_t i = b0 + threadIdx.x;
        const uint32_t x = i < m ? sums[i] : 0;
        uint32_t total;
        const uint32_t incl = block_scan_incl(x, s_warp, total);
        if (i < m) sums[i] = carry + incl - x;
        carry += total;
    }
    if (threadIdx.x == 0) sums[m] = carry;
}

__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(const uint32_t *__restrict__ in, int64_t n, const uint32_t *__restrict__ sums,
                  uint32_t *__restrict__ out_excl, const int *__restrict__ gate)
{
    if (gate && !*gate) return;
    __shared__ uint32_t s_warp[SCAN_THREADS / 32];
    const int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    uint32_t x[SCAN_ITEMS], t = 0;
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS; ++j) {
        x[j] = base + j < n ? in[base + j] : 0;
        t += x[j];
    }
    uint32_t total;
    const uint32_t incl = block_scan_incl(t, s_warp, total);
    uint32_t run = sums[blockIdx.x] + incl - t;
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS; ++j) {
        if (base + j < n) out_excl[base + j] = run;
        run += x[j];
    }
}

static void scan_excl_u32(const uint32_t *in, uint32_t *out, int64_t n, uint32_t *sums, cudaStream_t st,
                          const int *gate = nullptr)
{
    const int64_t tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    scan_tile_sums_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, st>>>(in, n, sums, gate);
    scan_sums_kernel<<<1, SCAN_THREADS, 0, st>>>(sums, tiles, gate);
    scan_apply_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, st>>>(in, n, sums, out, gate);
}

// ---- radix sort passes ---------------------------------------------------------------------------
struct SortBufs {
    uint64_t *keys[2];
    uint32_t *vals[2];
    int *cur;  // cur[p] = which buffer holds the input of pass p; cur[NPASS] = final buffer
};

__global__ void __launch_bounds__(WB_THREADS)
radix_hist_kernel(SortBufs b, int pass, int64_t N, int nblk, uint32_t *__restrict__ hist, const int *__restrict__ live)
{
    if (!live[pass]) return;
    __shared__ uint32_t s_h[256];
    s_h[threadIdx.x] = 0;
    __syncthreads();
    const uint64_t *keys = b.keys[b.cur[pass]];
    const int64_t base = (int64_t)blockIdx.x * WB_TILE;
#pragma unroll
    for (int j = 0; j < WB_ITEMS; ++j) {
        const int64_t i = base + j * WB_THREADS + threadIdx.x;
        if (i < N) atomicAdd(&s_h[(keys[i] >> (8 * pass)) & 255], 1u);
    }
    __syncthreads();
    hist[(int64_t)threadIdx.x * nblk + blockIdx.x] = s_h[threadIdx.x];
}

// Decide whether pass `pass` permutes anything: if one digit value holds all N keys the pass is
// the identity (the sort is stable) and is skipped.
__global__ void radix_decide_kernel(SortBufs b, int pass, int64_t N, int nblk,
                                    const uint32_t *__restrict__ excl, int *__restrict__ skip,
                                    const int *__restrict__ live)
{
    if (!live[pass]) {          // no used bit in this digit: nothing was counted, nothing moves
        if (threadIdx.x == 0) {
            skip[pass] = 1;
            b.cur[pass + 1] = b.cur[pass];
        }
        return;
    }
    __shared__ int s_uniform;
    if (threadIdx.x == 0) s_uniform = 0;
    __syncthreads();
    const int d = threadIdx.x;
    const uint32_t lo = excl[(int64_t)d * nblk];
    const uint32_t hi = d == 255 ? (uint32_t)N : excl[(int64_t)(d + 1) * nblk];
    if ((int64_t)(hi - lo) == N) s_uniform = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        skip[pass] = s_uniform;
        b.cur[pass + 1] = s_uniform ? b.cur[pass] : (b.cur[pass] ^ 1);
    }
}

__global__ void __launch_bounds__(WB_THREADS)
radix_scatter_kernel(SortBufs b, int pass, int64_t N, int nblk, const uint32_t *__restrict__ excl,
                     const int *__restrict__ skip)
{
    if (skip[pass]) return;
    __shared__ uint32_t s_run[256];
    const int src = b.cur[pass];
    const uint64_t *kin = b.keys[src];
    const uint32_t *vin = b.vals[src];
    uint64_t *kout = b.keys[src ^ 1];
    uint32_t *vout = b.vals[src ^ 1];
    s_run[threadIdx.x] = excl[(int64_t)threadIdx.x * nblk + blockIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t base = (int64_t)blockIdx.x * WB_TILE;
    for (int j = 0; j < WB_ITEMS; ++j) {
        const int64_t i = base + j * WB_THREADS + threadIdx.x;
        const bool valid = i < N;
        uint64_t key = 0;
        uint32_t val = 0;
        int digit = 256 + lane;  // unique per lane: invalid lanes match nobody
        if (valid) {
            key = kin[i];
            val = vin[i];
            digit = (int)((key >> (8 * pass)) & 255);
        }
        const uint32_t peers = __match_any_sync(0xffffffffu, digit);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        // warps take turns so that earlier keys get lower positions (stability)
        for (int wv = 0; wv < WB_THREADS / 32; ++wv) {
            uint32_t start = 0;
            if (warp == wv) {
                if (valid && lane == leader) {
                    start = s_run[digit];
                    s_run[digit] = start + __popc(peers);
                }
                start = __shfl_sync(0xffffffffu, start, leader);
                if (valid) {
                    kout[start + rank] = key;
                    vout[start + rank] = val;
                }
            }
            __syncthreads();
        }
    }
}

// ---- windows from sorted keys ------------------------------------------------------------------------
__global__ void wb_flags_kernel(SortBufs b, int64_t N, int ws, int F,
                                const float *__restrict__ feats, uint32_t *__restrict__ flags,
                                int32_t *__restrict__ n2n, float *__restrict__ n_coords)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const int fin = b.cur[NPASS];
    const uint64_t key = b.keys[fin][i];
    const uint32_t vid = b.vals[fin][i];
    const uint64_t win = key >> CELL_BITS;
    flags[i] = (i == 0 || (b.keys[fin][i - 1] >> CELL_BITS) != win) ? 1u : 0u;
    n2n[i] = (int32_t)vid;
    const int cell = (int)(key & ((1 << CELL_BITS) - 1));
    const int cz = cell % ws, cy = (cell / ws) % ws, cx = cell / (ws * ws);
    const float *f = feats + (int64_t)vid * F;
    float *o = n_coords + i * F;
    o[0] = (float)cx + __ldg(f);
    o[1] = (float)cy + __ldg(f + 1);
    o[2] = (float)cz + __ldg(f + 2);
    for (int j = 3; j < F; ++j) o[j] = __ldg(f + j);
}

__global__ void wb_heads_kernel(const uint32_t *__restrict__ flags, const uint32_t *__restrict__ excl,
                                int64_t N, int32_t *__restrict__ w2n, int64_t *__restrict__ counts)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    if (flags[i]) w2n[excl[i]] = (int32_t)i;
    if (i == N - 1) counts[0] = (int64_t)excl[i] + flags[i];
}

__global__ void wb_sizes_kernel(const int32_t *__restrict__ w2n, int64_t N,
                                int32_t *__restrict__ w_sizes, int64_t *__restrict__ counts)
{
    const int64_t W = counts[0];
    int64_t m = 0;
    int mx = 0;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < W;
         w += (int64_t)gridDim.x * blockDim.x) {
        const int32_t s = (int32_t)((w + 1 < W ? w2n[w + 1] : (int32_t)N) - w2n[w]);
        w_sizes[w] = s;
        m += (int64_t)s * s;
        mx = max(mx, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        m += __shfl_down_sync(0xffffffffu, m, o);
        mx = max(mx, __shfl_down_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(reinterpret_cast<unsigned long long *>(counts + 1), (unsigned long long)m);
        atomicMax(reinterpret_cast<long long *>(counts + 2), (long long)mx);
    }
}

__global__ void wb_init_kernel(int64_t *counts, int *cur, int *range)
{
    if (threadIdx.x < 4) {
        counts[threadIdx.x] = 0;
        range[threadIdx.x] = INT_MAX;
        range[4 + threadIdx.x] = INT_MIN;
    }
    if (threadIdx.x == 0) cur[0] = 0;
}

// ---- host ------------------------------------------------------------------------------------------------
static constexpr int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

struct WbLayout {
    int64_t keys0, keys1, vals0, vals1, hist, excl, sums, flags, cur, skip, total;
    int nblk;
};

static constexpr WbLayout wb_layout(int64_t N)
{
    WbLayout L{};
    const int64_t n = N < 1 ? 1 : N;
    L.nblk = (int)((n + WB_TILE - 1) / WB_TILE);
    const int64_t hist_n = (int64_t)256 * L.nblk;
    const int64_t scan_n = hist_n > n ? hist_n : n;
    int64_t off = 0;
    L.keys0 = off; off = align_up(off + n * 8, 256);
    L.keys1 = off; off = align_up(off + n * 8, 256);
    L.vals0 = off; off = align_up(off + n * 4, 256);
    L.vals1 = off; off = align_up(off + n * 4, 256);
    L.hist = off; off = align_up(off + hist_n * 4, 256);
    L.excl = off; off = align_up(off + scan_n * 4, 256);
    L.sums = off; off = align_up(off + ((scan_n + SCAN_TILE - 1) / SCAN_TILE + 2) * 4, 256);
    L.flags = off; off = align_up(off + n * 4, 256);
    L.cur = off; off = align_up(off + (NPASS + 1) * 4, 256);
    L.skip = off; off = align_up(off + NPASS * 4, 256);
    L.total = off;
    return L;
}

int64_t window_build_workspace_bytes(int64_t N) { return wb_layout(N).total; }

int window_build_launch(const int32_t *coords, const float *feats, int64_t N, int F, int stride,
                        int ws, int shift, int32_t *n2n, float *n_coords, int32_t *w_sizes,
                        int32_t *w2n, int64_t *counts, void *workspace, int64_t workspace_bytes,
                        cudaStream_t st)
{
    const WbLayout L = wb_layout(N);
    if (workspace_bytes < L.total) return S3D_ERR_WORKSPACE;
    char *ws_ptr = static_cast<char *>(workspace);
    SortBufs b;
    b.keys[0] = reinterpret_cast<uint64_t *>(ws_ptr + L.keys0);
    b.keys[1] = reinterpret_cast<uint64_t *>(ws_ptr + L.keys1);
    b.vals[0] = reinterpret_cast<uint32_t *>(ws_ptr + L.vals0);
    b.vals[1] = reinterpret_cast<uint32_t *>(ws_ptr + L.vals1);
    b.cur = reinterpret_cast<int *>(ws_ptr + L.cur);
    uint32_t *hist = reinterpret_cast<uint32_t *>(ws_ptr + L.hist);
    uint32_t *excl = reinterpret_cast<uint32_t *>(ws_ptr + L.excl);
    uint32_t *sums = reinterpret_cast<uint32_t *>(ws_ptr + L.sums);
    uint32_t *flags = reinterpret_cast<uint32_t *>(ws_ptr + L.flags);
    int *skip = reinterpret_cast<int *>(ws_ptr + L.skip);

    // the small arrays share one 256-byte slot of the workspace: cur[NPASS+1], range[8], live[NPASS]
    int *range = b.cur + 16, *live = b.cur + 24;
    wb_init_kernel<<<1, 32, 0, st>>>(counts, b.cur, range);
    if (N == 0) return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
    const unsigned nb = (unsigned)((N + 255) / 256);
    wb_range_kernel<<<nb < 148u * 8u ? nb : 148u * 8u, 256, 0, st>>>(coords, N, stride, ws, shift, range, counts);
    wb_keys_kernel<<<nb, 256, 0, st>>>(coords, N, stride, ws, shift, range, b.keys[0], b.vals[0], live);
    for (int pass = 0; pass < NPASS; ++pass) {
        radix_hist_kernel<<<L.nblk, WB_THREADS, 0, st>>>(b, pass, N, L.nblk, hist, live);
        scan_excl_u32(hist, excl, (int64_t)256 * L.nblk, sums, st, live + pass);
        radix_decide_kernel<<<1, 256, 0, st>>>(b, pass, N, L.nblk, excl, skip, live);
        radix_scatter_kernel<<<L.nblk, WB_THREADS, 0, st>>>(b, pass, N, L.nblk, excl, skip);
    }
    wb_flags_kernel<<<nb, 256, 0, st>>>(b, N, ws, F, feats, flags, n2n, n_coords);
    scan_excl_u32(flags, excl, N, sums, st);
    wb_heads_kernel<<<nb, 256, 0, st>>>(flags, excl, N, w2n, counts);
    wb_sizes_kernel<<<148 * 4, 256, 0, st>>>(w2n, N, w_sizes, counts);
    return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH;
}

}  // namespace s3d

// ---- window builder without any allocation by anybody -------------------------------------------------
// Some callers of this library cannot provide device scratch memory at the moment they need the
// window sets: code running while a memory pool is frozen (for instance a serving process that
// has handed every spare byte to its own arena and forbids driver allocations after start-up),
// or a host integration that may not call into an allocator from the thread or callback it runs
// on.  For them the scratch of the builder is a fixed array inside the library image.
//
// The array below is device memory that every GPU which loads this library keeps until the
// process exits.  Its name is only a host-side handle: passing `g_wb_static_scratch` itself to a
// kernel from host code would hand over a host address.  The device address is obtained with
// cudaGetSymbolAddress, once per device, with that device current, and cached.
namespace {

// The array is exactly as large as the scratch layout of the largest call the entry point accepts, so
// a change of the tile sizes or of the number of radix passes changes both together.
constexpr long long WB_STATIC_BYTES = s3d::wb_layout(S3D_WINDOW_BUILD_STATIC_MAX_VOXELS).total;
static_assert(WB_STATIC_BYTES > 0 && WB_STATIC_BYTES <= (5ll << 20), "static scratch of s3d_window_build_static: 5 MiB at most");
static_assert(s3d::wb_layout(S3D_WINDOW_BUILD_STATIC_MAX_VOXELS / 2).total <= WB_STATIC_BYTES, "the layout grows with the voxel count");
static __device__ __align__(256) unsigned char g_wb_static_scratch[WB_STATIC_BYTES];

constexpr int WB_MAX_DEVICES = 64;
void *g_wb_static_addr[WB_MAX_DEVICES] = {nullptr};
std::mutex g_wb_static_mutex;

// Device address of the scratch array on the current device (looked up on the first call per device).
int wb_static_scratch(void **out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= WB_MAX_DEVICES) return S3D_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_wb_static_mutex);
    if (g_wb_static_addr[dev] == nullptr) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_wb_static_scratch) != cudaSuccess || ptr == nullptr) return S3D_ERR_LAUNCH;
        g_wb_static_addr[dev] = ptr;
    }
    *out = g_wb_static_addr[dev];
    return S3D_OK;
}

}  // namespace

extern "C" int s3d_window_build_static(const int32_t *coords, const float *feats, int64_t N, int F, int stride,
                                       int ws, int shift, int32_t *n2n, float *n_coords, int32_t *w_sizes,
                                       int32_t *w2n, int64_t *counts_out, void *stream)
{
    if (N < 0 || stride < 1 || shift < 0 || F < 3 || F > 9) return S3D_ERR_BAD_ARG;
    if (ws < 1 || ws > 8) return S3D_ERR_UNSUPPORTED;
    if (N > S3D_WINDOW_BUILD_STATIC_MAX_VOXELS) return S3D_ERR_TOO_LARGE;
    if (s3d::window_build_workspace_bytes(N) > WB_STATIC_BYTES) return S3D_ERR_TOO_LARGE;
    if (!counts_out) return S3D_ERR_BAD_ARG;
    if (N > 0 && (!coords || !feats || !n2n || !n_coords || !w_sizes || !w2n)) return S3D_ERR_BAD_ARG;
    void *scratch = nullptr;
    const int rc = wb_static_scratch(&scratch);
    if (rc != S3D_OK) return rc;
    // Nothing in the scratch has to start at zero: every field the kernels read is written earlier
    // in the same call (keys, values, digit histograms, scans, flags, pass bookkeeping), so the
    // contents left behind by the previous call are simply overwritten.
    return s3d::window_build_launch(coords, feats, N, F, stride, ws, shift, n2n, n_coords, w_sizes, w2n,
                                    counts_out, scratch, WB_STATIC_BYTES, static_cast<cudaStream_t>(stream));
}
