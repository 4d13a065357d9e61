// Pieces shared by the attention kernels: tile sizes, launch parameters, the packed-fp32 and
// exponential helpers of the softmax, and the number of key tiles a query tile needs.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

#ifndef FB_ATTN_EMULATE_EVERY
#define FB_ATTN_EMULATE_EVERY 0
#endif

namespace fb {
namespace attn {

constexpr int BM = 128;        // query rows per tile (two tiles per CTA)
constexpr int BN = 128;        // keys per K/V tile
constexpr int kThreads = 384;  // warps 0-3, 4-7: softmax groups; warp 8: TMA; warp 9: MMA; 10-11 idle
constexpr int kRegsSoftmax = 208, kRegsOther = 72;  // per-thread register budgets after setmaxnreg
constexpr int kWarpTma = 8, kWarpMma = 9;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr int kEmulateEvery = FB_ATTN_EMULATE_EVERY;  // 0 = never; 2 = every other pair of P values

enum : unsigned { ST_ATTN_S = 0x201, ST_ATTN_P = 0x202, ST_ATTN_O = 0x203, ST_ATTN_KV = 0x204, ST_ATTN_Q = 0x205 };

struct AttnParams {
  int S_q, S_kv, n_pairs, causal;
  int normalized;  // 1: two passes over the keys, P divided by the complete row sum before it is rounded
  int64_t total_ctas;
  float scale_log2, scale;
  void* O;
  unsigned* status;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// packed fp32 pairs (one instruction for two lanes of the row)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.ftz.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return d;
}

__device__ __forceinline__ float2 add2_rm(float2 a, float2 b) {
  float2 d;
  asm("add.rm.ftz.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return d;
}
// 2^x for a pair of values on the FMA/ALU pipes instead of the special-function unit, which is
// the scarcest resource of the softmax (16 ex2 per clock per SM against 128x128 scores per
// tile).  x = n + f with n = floor(x) from a round-down add of 1.5*2^23, 2^f from a cubic
// (max relative error 9e-5, far below the 2^-9 of the 16-bit P it is rounded to), and n is
// added into the exponent field with integer arithmetic.
__device__ __forceinline__ float2 ex2_emulated(float2 x) {
  const float kMagic = 12582912.0f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -127.0f);
  x.y = fmaxf(x.y, -127.0f);
  const float2 t = add2_rm(x, make_float2(kMagic, kMagic));
  const float2 nf = add2(t, make_float2(-kMagic, -kMagic));
  const float2 f = fma2(nf, make_float2(-1.0f, -1.0f), x);
  float2 r = fma2(f, make_float2(0.077119089663028717f, 0.077119089663028717f),
                  make_float2(0.227564394474029541f, 0.227564394474029541f));
  r = fma2(r, f, make_float2(0.695146143436431885f, 0.695146143436431885f));
  r = fma2(r, f, make_float2(1.0f, 1.0f));
  r.x = __int_as_float(__float_as_int(r.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(r.y) + (__float_as_int(t.y) << 23));
  return r;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// number of key tiles query tile `m0` needs
__device__ __forceinline__ int kv_tiles_for(int m0, int S_q, int S_kv, int causal) {
  if (m0 >= S_q) return 0;
  int all = (S_kv + BN - 1) / BN;
  if (!causal) return all;
  int last_key = min(S_kv - 1, m0 + BM - 1 + (S_kv - S_q));  // visible to the tile's last row
  return min(all, last_key / BN + 1);
}

}  // namespace attn

}  // namespace fb
