// Shared device helpers for the swin3d_b200 kernels (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/swin3d_b200.h"

namespace s3d {

// Per-call description of the cRSE tables, passed to kernels by value.
// Signal dimension n owns L[n] rows of H*hd elements starting at row rowbase[n]; the flat
// element offset of (n, idx, h, c) is (rowbase[n] + idx) * H*hd + h*hd + c, which is the
// addressing of the reference (Swin3D/src/attn/attn_utils.cuh:441-451).
struct CrseMeta {
    int D;
    int R;  // total rows = sum L
    int L[S3D_MAX_SIGNAL_DIMS];
    int rowbase[S3D_MAX_SIGNAL_DIMS];
};

// cRSE row index of one signal dimension (Swin3D/src/attn/attn_utils.cuh:444-450):
// rel = cq - ck in fp32, plus L/2 (integer division), clamped to [0, (float)L], truncated.
// idx == L is reachable (the reference's upper bound L - 1e-10 rounds to L in fp32) and, through
// the flat addressing, selects row 0 of the next dimension; for the last dimension that would
// be past the table, so that one case is clamped to L-1.
__device__ __forceinline__ int crse_index(float cq, float ck, int L, bool last_dim)
{
    float rel = __fsub_rn(cq, ck);
    rel = __fadd_rn(rel, (float)(L / 2));
    rel = fminf(fmaxf(0.0f, rel), (float)L);
    int idx = (int)rel;
    if (last_dim && idx >= L) idx = L - 1;
    return idx;
}

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// Load HD consecutive elements (16-byte aligned when HD*sizeof(T) is a multiple of 16) as float.
template <typename T, int HD> __device__ __forceinline__ void load_vec(const T *p, float *dst);

template <> __device__ __forceinline__ void load_vec<float, 8>(const float *p, float *d)
{
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w; d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}
template <> __device__ __forceinline__ void load_vec<float, 16>(const float *p, float *d)
{
    load_vec<float, 8>(p, d);
    load_vec<float, 8>(p + 8, d + 8);
}
template <> __device__ __forceinline__ void load_vec<float, 32>(const float *p, float *d)
{
    load_vec<float, 16>(p, d);
    load_vec<float, 16>(p + 16, d + 16);
}
template <> __device__ __forceinline__ void load_vec<__half, 8>(const __half *p, float *d)
{
    const uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        d[2 * i] = f.x;
        d[2 * i + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void load_vec<__half, 16>(const __half *p, float *d)
{
    load_vec<__half, 8>(p, d);
    load_vec<__half, 8>(p + 8, d + 8);
}
template <> __device__ __forceinline__ void load_vec<__half, 32>(const __half *p, float *d)
{
    load_vec<__half, 16>(p, d);
    load_vec<__half, 16>(p + 16, d + 16);
}

template <typename T, int HD> __device__ __forceinline__ void store_vec(T *p, const float *s);
template <int HD> __device__ __forceinline__ void store_vec_f32(float *p, const float *s)
{
#pragma unroll
    for (int i = 0; i < HD / 4; ++i)
        reinterpret_cast<float4 *>(p)[i] = make_float4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
}
template <int HD> __device__ __forceinline__ void store_vec_f16(__half *p, const float *s)
{
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        uint4 r;
        __half2 *h = reinterpret_cast<__half2 *>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(s[8 * i + 2 * j], s[8 * i + 2 * j + 1]);
        reinterpret_cast<uint4 *>(p)[i] = r;
    }
}
template <> __device__ __forceinline__ void store_vec<float, 8>(float *p, const float *s) { store_vec_f32<8>(p, s); }
template <> __device__ __forceinline__ void store_vec<float, 16>(float *p, const float *s) { store_vec_f32<16>(p, s); }
template <> __device__ __forceinline__ void store_vec<float, 32>(float *p, const float *s) { store_vec_f32<32>(p, s); }
template <> __device__ __forceinline__ void store_vec<__half, 8>(__half *p, const float *s) { store_vec_f16<8>(p, s); }
template <> __device__ __forceinline__ void store_vec<__half, 16>(__half *p, const float *s) { store_vec_f16<16>(p, s); }
template <> __device__ __forceinline__ void store_vec<__half, 32>(__half *p, const float *s) { store_vec_f16<32>(p, s); }

}  // namespace s3d
