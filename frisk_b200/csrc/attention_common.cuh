// Pieces shared by the attention kernels: tile sizes, launch parameters, the packed-fp32 and
// exponential helpers of the softmax, and the number of key tiles a query tile needs.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace fb {
namespace attn {

constexpr int BM = 128;        // query rows per tile (two tiles per CTA)
constexpr int BN = 128;        // keys per K/V tile
constexpr int kThreads = 384;  // warps 0-3, 4-7: softmax groups; warp 8: TMA; warps 9, 10: MMA of query tile 0, 1; 11 idle
constexpr int kRegsSoftmax = 208, kRegsOther = 72;  // per-thread register budgets after setmaxnreg
constexpr int kWarpTma = 8, kWarpMma = 9;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

enum : unsigned { ST_ATTN_S = 0x201, ST_ATTN_P = 0x202, ST_ATTN_O = 0x203, ST_ATTN_KV = 0x204, ST_ATTN_Q = 0x205 };

struct AttnParams {
  int S_q, S_kv, n_pairs, causal;
  int normalized;  // 1: two passes over the keys, P divided by the complete row sum before it is rounded
  int64_t total_items;  // work items: pairs of 128-row query tiles of one (batch, head)
  float scale_log2, scale;
  void* O;
  unsigned* status;
  unsigned* work;  // [0] next work item, [1] CTAs that have finished; both zero between launches
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The reference's exponential (benchmark/layout/execution/tiled_attention.py:511-513 emits
// ex2.approx.f32, and its qualification forbids .ftz): subnormal inputs and results are kept.
// Used by the normalised mode, which follows the reference's arithmetic to the letter.
__device__ __forceinline__ float ex2f_ieee_range(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
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
