// Consumers of the KNN result, fused so that the [Nq, K, C] gathered tensor is never materialised:
//
//  * inverse-distance interpolation (microsoft/Swin3D, Swin3D/modules/swin3d_layers.py:53-73):
//        w_i = 1/(dist_i + 1e-8),  w_i /= sum_j w_j,  out[q] = sum_i src_feat[idx[q,i]] * w_i
//    with the reference's operation order (weights in fp32, one rounded multiply and one rounded add
//    per neighbour; for fp16 features the running sum is rounded to fp16 after every neighbour, as
//    the reference's in-place `+=` on an fp16 tensor does).  Backward: scatter of dOut * w_i.
//  * neighbourhood max-pool (swin3d_layers.py:302-309): LayerNorm and the bias-free Linear act on
//    each gathered row separately, so they commute with the gather; what is left per query is
//    out[q][c] = max_i g[idx[q,i]][c] with g = linear(norm(src_feat)) evaluated once per SOURCE row.
//    The arg-max source row is kept for the backward scatter (first maximum wins, as MaxPool1d).
//
// Both are HBM-bound row gathers: a warp owns a query, lanes run over channels with 16-byte
// accesses; the scatter-adds of the backward are fp32 reductions in L2 (red.global.add).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace s3d {
namespace {

constexpr int KC_MAX_K = 64;
constexpr int KC_THREADS = 256;

template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    using Raw = float4;
    static __device__ __forceinline__ void unpack(const Raw &r, float (&f)[4]) { f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
    static __device__ __forceinline__ Raw pack(const float (&f)[4]) { return make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<__half> {
    static constexpr int N = 8;
    using Raw = uint4;
    static __device__ __forceinline__ void unpack(const Raw &r, float (&f)[8])
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(h[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    static __device__ __forceinline__ Raw pack(const float (&f)[8])
    {
        Raw r;
        __half2 *h = reinterpret_cast<__half2 *>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        return r;
    }
};

// Running sum of the reference: fp32 stays fp32, fp16 is rounded to fp16 after every neighbour.
template <typename T> __device__ __forceinline__ float round_acc(float x);
template <> __device__ __forceinline__ float round_acc<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_acc<__half>(float x) { return __half2float(__float2half_rn(x)); }

// Normalised inverse-distance weights of one query, every lane computes the same values.
__device__ __forceinline__ void interp_weights(const float *dist, int K, float (&w)[KC_MAX_K])
{
    float norm = 0.f;
#pragma unroll 4
    for (int i = 0; i < K; ++i) {
        w[i] = __fdiv_rn(1.0f, __fadd_rn(dist[i], 1e-8f));
        norm = __fadd_rn(norm, w[i]);
    }
#pragma unroll 4
    for (int i = 0; i < K; ++i) w[i] = __fdiv_rn(w[i], norm);
}

template <typename T, int KT /*0: runtime K*/>
__global__ void __launch_bounds__(KC_THREADS)
knn_interp_fwd_kernel(const int32_t *__restrict__ idx, const float *__restrict__ dist, const T *__restrict__ src,
                      T *__restrict__ out, int64_t Nq, int Krt, int C)
{
    constexpr int VN = Vec<T>::N;
    using Raw = typename Vec<T>::Raw;
    const int K = KT ? KT : Krt;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (KC_THREADS / 32) + (threadIdx.x >> 5);
    const int64_t nwarp = (int64_t)gridDim.x * (KC_THREADS / 32);
    const int CV = C / VN;   // C is a whole number of vectors (checked by the entry point)
    for (int64_t q = warp0; q < Nq; q += nwarp) {
        float w[KT ? KT : KC_MAX_K];
        int32_t id[KT ? KT : KC_MAX_K];
        {
            float norm = 0.f;
#pragma unroll 4
            for (int i = 0; i < K; ++i) {
                id[i] = __ldg(idx + q * K + i);
                w[i] = __fdiv_rn(1.0f, __fadd_rn(__ldg(dist + q * K + i), 1e-8f));
                norm = __fadd_rn(norm, w[i]);
            }
#pragma unroll 4
            for (int i = 0; i < K; ++i) w[i] = __fdiv_rn(w[i], norm);
        }
        for (int cv = lane; cv < CV; cv += 32) {
            float acc[VN];
#pragma unroll
            for (int j = 0; j < VN; ++j) acc[j] = 0.f;
#pragma unroll 4
            for (int i = 0; i < K; ++i) {
                const Raw r = __ldg(reinterpret_cast<const Raw *>(src + (int64_t)id[i] * C) + cv);
                float f[VN];
                Vec<T>::unpack(r, f);
#pragma unroll
                for (int j = 0; j < VN; ++j) acc[j] = round_acc<T>(__fadd_rn(acc[j], __fmul_rn(f[j], w[i])));
            }
            reinterpret_cast<Raw *>(out + q * C)[cv] = Vec<T>::pack(acc);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(KC_THREADS)
knn_interp_bwd_kernel(const int32_t *__restrict__ idx, const float *__restrict__ dist, const T *__restrict__ dout,
                      float *__restrict__ dsrc, int64_t Nq, int K, int C)
{
    constexpr int VN = Vec<T>::N;
    using Raw = typename Vec<T>::Raw;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (KC_THREADS / 32) + (threadIdx.x >> 5);
    const int64_t nwarp = (int64_t)gridDim.x * (KC_THREADS / 32);
    const int CV = C / VN;
    for (int64_t q = warp0; q < Nq; q += nwarp) {
        float w[KC_MAX_K];
        interp_weights(dist + q * K, K, w);
        for (int cv = lane; cv < CV; cv += 32) {
            float g[VN];
            Vec<T>::unpack(__ldg(reinterpret_cast<const Raw *>(dout + q * C) + cv), g);
            for (int i = 0; i < K; ++i) {
                float *dst = dsrc + (int64_t)__ldg(idx + q * K + i) * C + cv * VN;
#pragma unroll
                for (int j = 0; j < VN; j += 4)
                    atomicAdd(reinterpret_cast<float4 *>(dst + j),
                              make_float4(g[j] * w[i], g[j + 1] * w[i], g[j + 2] * w[i], g[j + 3] * w[i]));
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(KC_THREADS)
knn_maxpool_fwd_kernel(const int32_t *__restrict__ idx, const T *__restrict__ g, T *__restrict__ out,
                       int32_t *__restrict__ arg, int64_t Nq, int K, int C)
{
    constexpr int VN = Vec<T>::N;
    using Raw = typename Vec<T>::Raw;
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * (KC_THREADS / 32) + (threadIdx.x >> 5);
    const int64_t nwarp = (int64_t)gridDim.x * (KC_THREADS / 32);
    const int CV = C / VN;
    for (int64_t q = warp0; q < Nq; q += nwarp) {
        for (int cv = lane; cv < CV; cv += 32) {
            float best[VN] = {};
            int32_t who[VN] = {};
            for (int i = 0; i < K; ++i) {
                const int32_t s = __ldg(idx + q * K + i);
                float f[VN];
                Vec<T>::unpack(__ldg(reinterpret_cast<const Raw *>(g + (int64_t)s * C) + cv), f);
#pragma unroll
                for (int j = 0; j < VN; ++j)
                    if (i == 0 || f[j] > best[j] || f[j] != f[j]) {   // first maximum wins; NaN propagates
                        best[j] = f[j];
                        who[j] = s;
                    }
            }
            reinterpret_cast<Raw *>(out + q * C)[cv] = Vec<T>::pack(best);
#pragma unroll
            for (int j = 0; j < VN; j += 4)
                *reinterpret_cast<int4 *>(arg + q * C + cv * VN + j) = make_int4(who[j], who[j + 1], who[j + 2], who[j + 3]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(KC_THREADS)
knn_maxpool_bwd_kernel(const int32_t *__restrict__ arg, const T *__restrict__ dout, float *__restrict__ dg,
                       int64_t total, int C)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int c = (int)(e % C);
        atomicAdd(dg + (int64_t)__ldg(arg + e) * C + c, (float)dout[e]);
    }
}

int grid_for(int64_t warps_needed)
{
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t blocks = (warps_needed + KC_THREADS / 32 - 1) / (KC_THREADS / 32);
    const int64_t cap = (int64_t)sms * 8;     // 8 resident blocks of 256 threads per SM
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int last_status() { return cudaGetLastError() == cudaSuccess ? S3D_OK : S3D_ERR_LAUNCH; }

}  // namespace
}  // namespace s3d

using namespace s3d;

extern "C" int s3d_knn_interpolate_fwd(const int32_t *idx, const float *dist, const void *src_feat, void *out,
                                       int64_t Nq, int K, int C, int dtype, void *stream)
{
    if (Nq < 0 || K < 1 || K > KC_MAX_K || C < 1 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    if (Nq == 0) return S3D_OK;
    if (!idx || !dist || !src_feat || !out) return S3D_ERR_BAD_ARG;
    const int vn = dtype == S3D_F32 ? 4 : 8;
    if (C % vn != 0 || !aligned16(src_feat) || !aligned16(out)) return S3D_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = grid_for(Nq);
    if (dtype == S3D_F32) {
        if (K == 3)
            knn_interp_fwd_kernel<float, 3><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const float *)src_feat, (float *)out, Nq, K, C);
        else
            knn_interp_fwd_kernel<float, 0><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const float *)src_feat, (float *)out, Nq, K, C);
    } else {
        if (K == 3)
            knn_interp_fwd_kernel<__half, 3><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const __half *)src_feat, (__half *)out, Nq, K, C);
        else
            knn_interp_fwd_kernel<__half, 0><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const __half *)src_feat, (__half *)out, Nq, K, C);
    }
    return last_status();
}

extern "C" int s3d_knn_interpolate_bwd(const int32_t *idx, const float *dist, const void *dout, float *dsrc,
                                       int64_t Nq, int64_t Ns, int K, int C, int dtype, void *stream)
{
    if (Nq < 0 || Ns < 0 || K < 1 || K > KC_MAX_K || C < 1 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    if (Ns == 0) return S3D_OK;
    if (!dsrc) return S3D_ERR_BAD_ARG;
    const int vn = dtype == S3D_F32 ? 4 : 8;
    if (C % vn != 0 || !aligned16(dout) || !aligned16(dsrc)) return S3D_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(dsrc, 0, (size_t)Ns * C * sizeof(float), st) != cudaSuccess) return S3D_ERR_LAUNCH;
    if (Nq == 0) return S3D_OK;
    if (!idx || !dist || !dout) return S3D_ERR_BAD_ARG;
    const int grid = grid_for(Nq);
    if (dtype == S3D_F32)
        knn_interp_bwd_kernel<float><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const float *)dout, dsrc, Nq, K, C);
    else
        knn_interp_bwd_kernel<__half><<<grid, KC_THREADS, 0, st>>>(idx, dist, (const __half *)dout, dsrc, Nq, K, C);
    return last_status();
}

extern "C" int s3d_knn_maxpool_fwd(const int32_t *idx, const void *g, void *out, int32_t *arg,
                                   int64_t Nq, int K, int C, int dtype, void *stream)
{
    if (Nq < 0 || K < 1 || C < 1 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    if (Nq == 0) return S3D_OK;
    if (!idx || !g || !out || !arg) return S3D_ERR_BAD_ARG;
    const int vn = dtype == S3D_F32 ? 4 : 8;
    if (C % vn != 0 || !aligned16(g) || !aligned16(out) || !aligned16(arg)) return S3D_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = grid_for(Nq);
    if (dtype == S3D_F32)
        knn_maxpool_fwd_kernel<float><<<grid, KC_THREADS, 0, st>>>(idx, (const float *)g, (float *)out, arg, Nq, K, C);
    else
        knn_maxpool_fwd_kernel<__half><<<grid, KC_THREADS, 0, st>>>(idx, (const __half *)g, (__half *)out, arg, Nq, K, C);
    return last_status();
}

extern "C" int s3d_knn_maxpool_bwd(const int32_t *arg, const void *dout, float *dg,
                                   int64_t Nq, int64_t Ns, int C, int dtype, void *stream)
{
    if (Nq < 0 || Ns < 0 || C < 1 || (dtype != S3D_F32 && dtype != S3D_F16)) return S3D_ERR_BAD_ARG;
    if (Ns == 0) return S3D_OK;
    if (!dg) return S3D_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(dg, 0, (size_t)Ns * C * sizeof(float), st) != cudaSuccess) return S3D_ERR_LAUNCH;
    if (Nq == 0) return S3D_OK;
    if (!arg || !dout) return S3D_ERR_BAD_ARG;
    const int64_t total = Nq * C;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t want = (total + KC_THREADS - 1) / KC_THREADS;
    const int grid = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
    if (dtype == S3D_F32)
        knn_maxpool_bwd_kernel<float><<<grid, KC_THREADS, 0, st>>>(arg, (const float *)dout, dg, total, C);
    else
        knn_maxpool_bwd_kernel<__half><<<grid, KC_THREADS, 0, st>>>(arg, (const __half *)dout, dg, total, C);
    return last_status();
}
