// fp32 GEMM on the CUDA cores: C <- (clear_accum ? 0 : C) + op(A).op(B), fp32 throughout.
// Contract: `frisk.gemm` with f32 operands (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).
//
// 128x64 output tile per CTA, k-step 16, 256 threads each owning an 8x4 register tile.
// Global loads are 128-bit when the operand pitch and base allow it; the next k-step is
// fetched into registers while the current one is multiplied out of shared memory
// (two shared-memory buffers, one barrier per step).  Tiles are stored K-major in shared
// memory ([k][m] and [k][n]) whichever way the operand lies in global memory, so the
// inner product reads are broadcast/128-bit for all four transpose combinations.
#include "common.cuh"

namespace fb {
namespace {

constexpr int BM = 128, BN = 64, BK = 16, TM = 8, TN = 4, NT = 256;
constexpr int PAD = 4;

// Operand tile loader.  `KContig` = the global buffer is contiguous along K (A non-transposed,
// B transposed); otherwise it is contiguous along the tile's MN extent.
// EXT = tile extent along MN (BM or BN).  Each thread moves EXT*BK/NT floats.
template <int EXT, bool KContig>
struct TileLoader {
  static constexpr int kVecs = EXT * BK / 4 / NT;  // float4 per thread
  static_assert(EXT * BK % (4 * NT) == 0, "tile must split into float4 per thread");
  float4 reg[kVecs];

  // mn0: first MN index of the tile; k0: first K index; ext_mn / ext_k: logical extents
  __device__ __forceinline__ void load(const float* __restrict__ g, int64_t ld, int mn0, int k0, int ext_mn,
                                       int ext_k, bool vec_ok, int tid) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      int idx = tid + v * NT;
      int mn, k;
      if (KContig) {
        mn = idx / (BK / 4);
        k = (idx % (BK / 4)) * 4;
      } else {
        k = idx / (EXT / 4);
        mn = (idx % (EXT / 4)) * 4;
      }
      int gmn = mn0 + mn, gk = k0 + k;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (KContig) {
        const float* p = g + (int64_t)gmn * ld + gk;
        if (vec_ok && gmn < ext_mn && gk + 3 < ext_k) {
          val = __ldg(reinterpret_cast<const float4*>(p));
        } else if (gmn < ext_mn) {
          if (gk + 0 < ext_k) val.x = __ldg(p + 0);
          if (gk + 1 < ext_k) val.y = __ldg(p + 1);
          if (gk + 2 < ext_k) val.z = __ldg(p + 2);
          if (gk + 3 < ext_k) val.w = __ldg(p + 3);
        }
      } else {
        const float* p = g + (int64_t)gk * ld + gmn;
        if (vec_ok && gk < ext_k && gmn + 3 < ext_mn) {
          val = __ldg(reinterpret_cast<const float4*>(p));
        } else if (gk < ext_k) {
          if (gmn + 0 < ext_mn) val.x = __ldg(p + 0);
          if (gmn + 1 < ext_mn) val.y = __ldg(p + 1);
          if (gmn + 2 < ext_mn) val.z = __ldg(p + 2);
          if (gmn + 3 < ext_mn) val.w = __ldg(p + 3);
        }
      }
      reg[v] = val;
    }
  }
  __device__ __forceinline__ void store(float (*s)[EXT + PAD], int tid) const {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      int idx = tid + v * NT;
      if (KContig) {
        int mn = idx / (BK / 4);
        int k = (idx % (BK / 4)) * 4;
        s[k + 0][mn] = reg[v].x;
        s[k + 1][mn] = reg[v].y;
        s[k + 2][mn] = reg[v].z;
        s[k + 3][mn] = reg[v].w;
      } else {
        int k = idx / (EXT / 4);
        int mn = (idx % (EXT / 4)) * 4;
        *reinterpret_cast<float4*>(&s[k][mn]) = reg[v];
      }
    }
  }
};

template <bool TA, bool TB>
__global__ void __launch_bounds__(NT) gemm_simt_f32_kernel(const float* __restrict__ A,
                                                           const float* __restrict__ B, float* __restrict__ C,
                                                           int M, int N, int K, int64_t lda, int64_t ldb,
                                                           int64_t ldc, int accumulate, int vec_a, int vec_b,
                                                           int vec_c) {
  __shared__ __align__(16) float As[2][BK][BM + PAD];
  __shared__ __align__(16) float Bs[2][BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);  // 0..15 -> columns tx*4..
  const int ty = tid / (BN / TN);  // 0..15 -> rows ty*8..
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  TileLoader<BM, !TA> la;
  TileLoader<BN, TB> lb;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int ksteps = (K + BK - 1) / BK;
  la.load(A, lda, m0, 0, M, K, vec_a, tid);
  lb.load(B, ldb, n0, 0, N, K, vec_b, tid);
  la.store(As[0], tid);
  lb.store(Bs[0], tid);
  __syncthreads();

  for (int ks = 0; ks < ksteps; ++ks) {
    const int cur = ks & 1;
    if (ks + 1 < ksteps) {
      la.load(A, lda, m0, (ks + 1) * BK, M, K, vec_a, tid);
      lb.load(B, ldb, n0, (ks + 1) * BK, N, K, vec_b, tid);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
      float4 a0 = *reinterpret_cast<const float4*>(&As[cur][k][ty * TM]);
      float4 a1 = *reinterpret_cast<const float4*>(&As[cur][k][ty * TM + 4]);
      float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][k][tx * TN]);
      a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
      a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (ks + 1 < ksteps) {
      la.store(As[cur ^ 1], tid);
      lb.store(Bs[cur ^ 1], tid);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int r = m0 + ty * TM + i;
    if (r >= M) continue;
    int c = n0 + tx * TN;
    float* p = C + (int64_t)r * ldc + c;
    if (vec_c && c + 3 < N) {
      float4 o = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      if (accumulate) {
        float4 old = *reinterpret_cast<const float4*>(p);
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      *reinterpret_cast<float4*>(p) = o;
    } else {
#pragma unroll
      for (int j = 0; j < TN; ++j)
        if (c + j < N) p[j] = accumulate ? p[j] + acc[i][j] : acc[i][j];
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int launch_gemm_simt_f32(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const float* A, const float* B,
                         float* C, cudaStream_t s) {
  GemmDims g = resolve_dims(d);
  if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return FRISK_B200_E_UNSUPPORTED;
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((g.M + BM - 1) / BM));
  if (grid.y > 65535) return FRISK_B200_E_UNSUPPORTED;
  int vec_a = aligned16(A) && (g.lda % 4 == 0);
  int vec_b = aligned16(B) && (g.ldb % 4 == 0);
  int vec_c = aligned16(C) && (g.ldc % 4 == 0);
  int acc = d.clear_accum ? 0 : 1;
#define FB_LAUNCH(TA, TB)                                                                                   \
  gemm_simt_f32_kernel<TA, TB><<<grid, NT, 0, s>>>(A, B, C, (int)g.M, (int)g.N, (int)g.K, g.lda, g.ldb, g.ldc, \
                                                   acc, vec_a, vec_b, vec_c)
  if (d.trans_a) {
    if (d.trans_b) FB_LAUNCH(true, true); else FB_LAUNCH(true, false);
  } else {
    if (d.trans_b) FB_LAUNCH(false, true); else FB_LAUNCH(false, false);
  }
#undef FB_LAUNCH
  FB_CUDA(ctx, cudaGetLastError());
  return 0;
}

}  // namespace fb
