// Pieces shared by the tcgen05 GEMM kernels: the tile raster and the accumulator-row stores.
#pragma once
#include "common.cuh"

namespace fb {
namespace gemm_detail {

constexpr int kGroupM = 8;  // tile raster: columns of 8 M-tiles, for L2 reuse of B

struct TileCoord {
  int m, n;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
  int per_group = kGroupM * tiles_n;
  int group = t / per_group;
  int first_m = group * kGroupM;
  int gsize = min(tiles_m - first_m, kGroupM);
  int r = t - group * per_group;
  return TileCoord{first_m + r % gsize, r / gsize};
}

// the value an fp32 result takes once it is stored as TO
template <typename TO>
__device__ __forceinline__ float rounded_as(float v);
template <>
__device__ __forceinline__ float rounded_as<float>(float v) { return v; }
template <>
__device__ __forceinline__ float rounded_as<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <>
__device__ __forceinline__ float rounded_as<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename TO>
__device__ __forceinline__ void store_row_chunk(TO* p, const uint32_t (&v)[32], int valid, bool vec_ok,
                                                bool accumulate);

template <>
__device__ __forceinline__ void store_row_chunk<float>(float* p, const uint32_t (&v)[32], int valid, bool vec_ok,
                                                       bool accumulate) {
  if (vec_ok && valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 o = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                             __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
      if (accumulate) {
        float4 c = *reinterpret_cast<const float4*>(p + 4 * i);
        o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
      }
      *reinterpret_cast<float4*>(p + 4 * i) = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) p[i] = accumulate ? p[i] + __uint_as_float(v[i]) : __uint_as_float(v[i]);
  }
}

template <typename T2, typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half2, __half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat162, __nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// two fp32 values rounded to TO and packed (16-bit TO only; the float form exists so that templates compile)
template <typename TO>
__device__ __forceinline__ uint32_t pack_out(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_out<__half>(float a, float b) { return pack2<__half2, __half>(a, b); }
template <>
__device__ __forceinline__ uint32_t pack_out<__nv_bfloat16>(float a, float b) {
  return pack2<__nv_bfloat162, __nv_bfloat16>(a, b);
}
template <>
__device__ __forceinline__ uint32_t pack_out<float>(float a, float) { return __float_as_uint(a); }
__device__ __forceinline__ float2 unpack2(uint32_t u, __half) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
__device__ __forceinline__ float2 unpack2(uint32_t u, __nv_bfloat16) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

template <typename T, typename T2>
__device__ __forceinline__ void store_row_chunk16(T* p, const uint32_t (&v)[32], int valid, bool vec_ok,
                                                  bool accumulate) {
  if (vec_ok && valid == 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[8 * i + j]);
      if (accumulate) {
        uint4 c = *reinterpret_cast<const uint4*>(p + 8 * i);
        float2 c0 = unpack2(c.x, T()), c1 = unpack2(c.y, T()), c2 = unpack2(c.z, T()), c3 = unpack2(c.w, T());
        f[0] += c0.x; f[1] += c0.y; f[2] += c1.x; f[3] += c1.y;
        f[4] += c2.x; f[5] += c2.y; f[6] += c3.x; f[7] += c3.y;
      }
      uint4 o;
      o.x = pack2<T2, T>(f[0], f[1]);
      o.y = pack2<T2, T>(f[2], f[3]);
      o.z = pack2<T2, T>(f[4], f[5]);
      o.w = pack2<T2, T>(f[6], f[7]);
      *reinterpret_cast<uint4*>(p + 8 * i) = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < valid) {
        float f = __uint_as_float(v[i]);
        if (accumulate) f += static_cast<float>(p[i]);
        p[i] = static_cast<T>(f);
      }
    }
  }
}
template <>
__device__ __forceinline__ void store_row_chunk<__half>(__half* p, const uint32_t (&v)[32], int valid,
                                                        bool vec_ok, bool accumulate) {
  store_row_chunk16<__half, __half2>(p, v, valid, vec_ok, accumulate);
}
template <>
__device__ __forceinline__ void store_row_chunk<__nv_bfloat16>(__nv_bfloat16* p, const uint32_t (&v)[32],
                                                               int valid, bool vec_ok, bool accumulate) {
  store_row_chunk16<__nv_bfloat16, __nv_bfloat162>(p, v, valid, vec_ok, accumulate);
}

}  // namespace gemm_detail
}  // namespace fb
