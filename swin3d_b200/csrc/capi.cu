// extern "C" entry points of libswin3d_b200.so: argument validation and dispatch only.
// The declarations, with the reference interfaces they replace, are in include/swin3d_b200.h.
#include <string.h>
#include "attn_kernels.cuh"
#include <cstdint>
#include <initializer_list>
#include "knn_kernels.cuh"
#include "window_kernels.cuh"

#include <cstdlib>

using namespace s3d;

namespace s3d {
static int g_last_cuda_error = 0;
void note_cuda_error(cudaError_t e) { if (e != cudaSuccess) g_last_cuda_error = (int)e; }
}  // namespace s3d

namespace {

// Set through s3d_debug_force_generic(): routes every attention call of the process to the generic
// kernels (the tests cross-check the two implementations on the GPU with it).  Off by default; the
// product path reads one plain int.
int g_force_generic = 0;
bool force_scalar() { return g_force_generic != 0; }

int make_meta(const int32_t *table_sizes_host, int D, int H, int hd, CrseMeta &m)
{
    if (!table_sizes_host || H < 1) return S3D_ERR_BAD_ARG;
    if (D != 3 && D != 6 && D != 9) return S3D_ERR_UNSUPPORTED;
    if (hd != 8 && hd != 16 && hd != 32) return S3D_ERR_UNSUPPORTED;
    const int HC = H * hd;
    m.D = D;
    int rows = 0;
    for (int n = 0; n < S3D_MAX_SIGNAL_DIMS; ++n) { m.L[n] = 0; m.rowbase[n] = 0; }
    for (int n = 0; n < D; ++n) {
        if (table_sizes_host[n] <= 0 || table_sizes_host[n] % HC != 0) return S3D_ERR_BAD_ARG;
        m.L[n] = table_sizes_host[n] / HC;
        m.rowbase[n] = rows;
        rows += m.L[n];
    }
    m.R = rows;
    return S3D_OK;
}

}  // namespace

// The kernels read and write rows with 16-byte vector accesses.
static bool aligned16(std::initializer_list<const void *> ptrs)
{
    for (const void *p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) & 15) return false;
    return true;
}

extern "C" {

const char *s3d_status_string(int status)
{
    switch (status) {
        case S3D_OK: return "ok";
        case S3D_ERR_BAD_ARG: return "bad argument (null pointer, negative size, unknown dtype, table size not a multiple of H*hd, or a row/table pointer that is not 16-byte aligned)";
        case S3D_ERR_UNSUPPORTED: return "unsupported shape (head_dim must be 8, 16 or 32; signal dims 3, 6 or 9; K <= 64; window size <= 8)";
        case S3D_ERR_LAUNCH: return "CUDA launch error";
        case S3D_ERR_WORKSPACE: return "workspace too small";
        case S3D_ERR_TOO_LARGE: return "input larger than the fixed capacity of this *_static entry point (see its limit in swin3d_b200.h)";
        default: return "unknown status";
    }
}

int s3d_version(void) { return 1000; }

int s3d_debug_force_generic(int on)
{
    const int was = g_force_generic;
    g_force_generic = on ? 1 : 0;
    return was;
}

const char *s3d_last_cuda_error_string(void)
{
    return cudaGetErrorString(static_cast<cudaError_t>(s3d::g_last_cuda_error));
}

static int fill_mirrors(s3d::Mirrors &m, int n, void *const *host)
{
    m.n = 0;
    if (n == 0) return S3D_OK;
    if (n < 0 || n > S3D_MAX_MIRRORS || !host) return S3D_ERR_BAD_ARG;
    for (int i = 0; i < n; ++i) {
        if (!host[i] || (reinterpret_cast<uintptr_t>(host[i]) & 15)) return S3D_ERR_BAD_ARG;
        m.p[i] = host[i];
    }
    m.n = n;
    return S3D_OK;
}

static int attn_fwd_impl(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                         const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                         const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                         int H, int hd, int dtype, void *out, float *lse, int n_mirrors,
                         void *const *out_mirrors_host, int window_class, void *stream)
{
    if (N < 0 || W < 0 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    AttnArgs a{};
    const int rc = make_meta(table_sizes_host, D, H, hd, a.meta);
    if (rc != S3D_OK) return rc;
    if (N == 0 || W == 0) return S3D_OK;
    if (!q || !k || !v || !tq || !tk || !tv || !w_sizes || !w2n || !n2n || !n_coords || !out || !lse)
        return S3D_ERR_BAD_ARG;
    if (!aligned16({q, k, v, tq, tk, tv, out})) return S3D_ERR_BAD_ARG;
    a.q = q; a.k = k; a.v = v; a.tq = tq; a.tk = tk; a.tv = tv;
    a.w_sizes = w_sizes; a.w2n = w2n; a.n2n = n2n; a.n_coords = n_coords;
    a.N = N; a.W = W; a.H = H; a.hd = hd; a.dtype = dtype;
    a.out = out; a.lse = lse;
    const int mrc = fill_mirrors(a.m_out, n_mirrors, out_mirrors_host);
    if (mrc != S3D_OK) return mrc;
    if (window_class < 0 || window_class > 2) return S3D_ERR_BAD_ARG;
    a.window_class = window_class;
    if (!force_scalar() && attn_tc_supported(a)) return attn_tc_forward(a, static_cast<cudaStream_t>(stream));
    if (a.m_out.n) return S3D_ERR_UNSUPPORTED;
    return attn_scalar_forward(a, static_cast<cudaStream_t>(stream));
}

int s3d_attn_fwd(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                 const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                 const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                 int H, int hd, int dtype, void *out, float *lse, void *stream)
{
    return attn_fwd_impl(q, k, v, tq, tk, tv, table_sizes_host, D, w_sizes, w2n, n2n, n_coords, N, W, H, hd,
                         dtype, out, lse, 0, nullptr, 0, stream);
}

int s3d_attn_fwd_mirrored(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                          const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                          const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                          int H, int hd, int dtype, void *out, float *lse, int n_mirrors,
                          void *const *out_mirrors_host, int window_class, void *stream)
{
    return attn_fwd_impl(q, k, v, tq, tk, tv, table_sizes_host, D, w_sizes, w2n, n2n, n_coords, N, W, H, hd,
                         dtype, out, lse, n_mirrors, out_mirrors_host, window_class, stream);
}

int s3d_peer_alloc(int64_t bytes, void **ptr_out, void *handle64_out)
{
    if (bytes <= 0 || !ptr_out || !handle64_out) return S3D_ERR_BAD_ARG;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e == cudaSuccess) {
        cudaIpcMemHandle_t h;
        e = cudaIpcGetMemHandle(&h, p);
        if (e == cudaSuccess) {
            memcpy(handle64_out, &h, sizeof(h));
            *ptr_out = p;
            return S3D_OK;
        }
        cudaFree(p);
    }
    s3d::note_cuda_error(e);
    return S3D_ERR_LAUNCH;
}

int s3d_peer_free(void *ptr)
{
    if (!ptr) return S3D_ERR_BAD_ARG;
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) {
        s3d::note_cuda_error(e);
        return S3D_ERR_LAUNCH;
    }
    return S3D_OK;
}

int s3d_ipc_open(const void *handle64, void **ptr_out)
{
    if (!handle64 || !ptr_out) return S3D_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "CUDA IPC memory handles are 64 bytes");
    memcpy(&h, handle64, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        s3d::note_cuda_error(e);
        return S3D_ERR_LAUNCH;
    }
    *ptr_out = p;
    return S3D_OK;
}

int s3d_ipc_close(void *ptr)
{
    if (!ptr) return S3D_ERR_BAD_ARG;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) {
        s3d::note_cuda_error(e);
        return S3D_ERR_LAUNCH;
    }
    return S3D_OK;
}

static int attn_bwd_impl(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                         const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                         const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                         int H, int hd, int dtype, const void *out, const float *lse, const void *dout,
                         void *dq, void *dk, void *dv, float *dtq, float *dtk, float *dtv, int n_mirrors,
                         void *const *dq_m, void *const *dk_m, void *const *dv_m, void *stream)
{
    if (N < 0 || W < 0 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    AttnArgs a{};
    const int rc = make_meta(table_sizes_host, D, H, hd, a.meta);
    if (rc != S3D_OK) return rc;
    if (!dtq || !dtk || !dtv) return S3D_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t tbytes = (size_t)a.meta.R * H * hd * sizeof(float);
    if (cudaMemsetAsync(dtq, 0, tbytes, st) != cudaSuccess || cudaMemsetAsync(dtk, 0, tbytes, st) != cudaSuccess ||
        cudaMemsetAsync(dtv, 0, tbytes, st) != cudaSuccess)
        return S3D_ERR_LAUNCH;
    if (N == 0 || W == 0) return S3D_OK;
    if (!q || !k || !v || !tq || !tk || !tv || !w_sizes || !w2n || !n2n || !n_coords || !out || !lse ||
        !dout || !dq || !dk || !dv)
        return S3D_ERR_BAD_ARG;
    if (!aligned16({q, k, v, tq, tk, tv, out, dout, dq, dk, dv, dtq, dtk, dtv})) return S3D_ERR_BAD_ARG;
    a.q = q; a.k = k; a.v = v; a.tq = tq; a.tk = tk; a.tv = tv;
    a.w_sizes = w_sizes; a.w2n = w2n; a.n2n = n2n; a.n_coords = n_coords;
    a.N = N; a.W = W; a.H = H; a.hd = hd; a.dtype = dtype;
    a.out = const_cast<void *>(out); a.lse = const_cast<float *>(lse); a.dout = dout;
    a.dq = dq; a.dk = dk; a.dv = dv; a.dtq = dtq; a.dtk = dtk; a.dtv = dtv;
    if (fill_mirrors(a.m_dq, n_mirrors, dq_m) != S3D_OK || fill_mirrors(a.m_dk, n_mirrors, dk_m) != S3D_OK ||
        fill_mirrors(a.m_dv, n_mirrors, dv_m) != S3D_OK)
        return S3D_ERR_BAD_ARG;
    if (!force_scalar() && attn_tc_bwd_supported(a)) return attn_tc_backward(a, st);
    if (n_mirrors) return S3D_ERR_UNSUPPORTED;
    return attn_scalar_backward(a, st);
}

int s3d_attn_bwd(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                 const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                 const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                 int H, int hd, int dtype, const void *out, const float *lse, const void *dout,
                 void *dq, void *dk, void *dv, float *dtq, float *dtk, float *dtv, void *stream)
{
    return attn_bwd_impl(q, k, v, tq, tk, tv, table_sizes_host, D, w_sizes, w2n, n2n, n_coords, N, W, H, hd,
                         dtype, out, lse, dout, dq, dk, dv, dtq, dtk, dtv, 0, nullptr, nullptr, nullptr, stream);
}

int s3d_attn_bwd_mirrored(const void *q, const void *k, const void *v, const void *tq, const void *tk,
                          const void *tv, const int32_t *table_sizes_host, int D, const int32_t *w_sizes,
                          const int32_t *w2n, const int32_t *n2n, const float *n_coords, int64_t N, int64_t W,
                          int H, int hd, int dtype, const void *out, const float *lse, const void *dout,
                          void *dq, void *dk, void *dv, float *dtq, float *dtk, float *dtv, int n_mirrors,
                          void *const *dq_mirrors_host, void *const *dk_mirrors_host,
                          void *const *dv_mirrors_host, void *stream)
{
    return attn_bwd_impl(q, k, v, tq, tk, tv, table_sizes_host, D, w_sizes, w2n, n2n, n_coords, N, W, H, hd,
                         dtype, out, lse, dout, dq, dk, dv, dtq, dtk, dtv, n_mirrors, dq_mirrors_host,
                         dk_mirrors_host, dv_mirrors_host, stream);
}

int s3d_debug_crse_indices(const float *n_coords, const int32_t *table_sizes_host, int D, int H,
                           int hd, int32_t first_pos, int32_t n, int32_t *idx_out, void *stream)
{
    CrseMeta m;
    const int rc = make_meta(table_sizes_host, D, H, hd, m);
    if (rc != S3D_OK) return rc;
    if (n < 0 || first_pos < 0) return S3D_ERR_BAD_ARG;
    if (n == 0) return S3D_OK;
    if (!n_coords || !idx_out) return S3D_ERR_BAD_ARG;
    return crse_indices_dump(n_coords, m, first_pos, n, idx_out, static_cast<cudaStream_t>(stream));
}

int s3d_debug_crse_indices_variant(const float *n_coords, const int32_t *table_sizes_host, int D, int H,
                                   int hd, int32_t first_pos, int32_t n, int variant, int32_t *idx_out,
                                   void *stream)
{
    CrseMeta m;
    const int rc = make_meta(table_sizes_host, D, H, hd, m);
    if (rc != S3D_OK) return rc;
    if (n < 0 || first_pos < 0 || variant < 0 || variant > 2) return S3D_ERR_BAD_ARG;
    if (n == 0) return S3D_OK;
    if (!n_coords || !idx_out) return S3D_ERR_BAD_ARG;
    return crse_indices_dump_variant(n_coords, m, first_pos, n, variant, idx_out, static_cast<cudaStream_t>(stream));
}

int s3d_debug_crse_index_values(const float *cq, const float *ck, int64_t n, int L, int last_dim, int variant,
                                int32_t *idx_out, void *stream)
{
    if (n < 0 || L < 1 || variant < 0 || variant > 2) return S3D_ERR_BAD_ARG;
    if (n == 0) return S3D_OK;
    if (!cq || !ck || !idx_out) return S3D_ERR_BAD_ARG;
    return crse_index_values(cq, ck, n, L, last_dim, variant, idx_out, static_cast<cudaStream_t>(stream));
}

int64_t s3d_window_build_workspace_bytes(int64_t N) { return window_build_workspace_bytes(N); }

int s3d_window_build(const int32_t *coords, const float *feats, int64_t N, int F, int stride, int ws,
                     int shift, int32_t *n2n, float *n_coords, int32_t *w_sizes, int32_t *w2n,
                     int64_t *counts_out, void *workspace, int64_t workspace_bytes, void *stream)
{
    if (N < 0 || stride < 1 || shift < 0 || F < 3 || F > 3 + 2 * 3) return S3D_ERR_BAD_ARG;
    if (ws < 1 || ws > 8) return S3D_ERR_UNSUPPORTED;
    if (N >= (int64_t)1 << 31) return S3D_ERR_UNSUPPORTED;
    if (!counts_out || !workspace) return S3D_ERR_BAD_ARG;
    if (N > 0 && (!coords || !feats || !n2n || !n_coords || !w_sizes || !w2n)) return S3D_ERR_BAD_ARG;
    return window_build_launch(coords, feats, N, F, stride, ws, shift, n2n, n_coords, w_sizes, w2n,
                               counts_out, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int s3d_knn(int K, const float *src, const float *query, const int32_t *src_offset,
            const int32_t *query_offset, int B, int64_t Ns, int64_t Nq, int32_t *ret_idx,
            float *ret_dist, void *stream)
{
    if (K < 1 || K > S3D_KNN_MAX_K) return S3D_ERR_UNSUPPORTED;
    if (B < 1 || Ns < 0 || Nq < 0) return S3D_ERR_BAD_ARG;
    if (Nq == 0) return S3D_OK;
    if (!query || !src_offset || !query_offset || !ret_idx || !ret_dist || (Ns > 0 && !src))
        return S3D_ERR_BAD_ARG;
    return knn_launch(K, src, query, src_offset, query_offset, B, Nq, ret_idx, ret_dist,
                      static_cast<cudaStream_t>(stream));
}

}  // extern "C"
