// fp32 GEMM on the tensor cores: every fp32 operand element is split exactly into three bf16
// terms (a = a1 + a2 + a3 up to 2^-26 |a|: 3 x 8 significant bits plus the signs), the nine
// products A_s . B_t are one bf16 GEMM with fp32 accumulation in tensor memory over the stacked
// operands [A1; A2; A3] (3M x K) and [B1; B2; B3] (3N x K), and the nine M x N blocks of that
// product are added smallest first.  Products of bf16 terms are exact in fp32, so the result has
// fp32-GEMM accuracy (relative Frobenius error a few 1e-7 against fp64, like the CUDA-core kernel)
// at tensor-core speed.  Same contract as the CUDA-core kernel: `frisk.gemm` with f32 operands,
// C <- (clear_accum ? 0 : C) + op(A).op(B) (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).
//
// Three launches on the caller's stream: split (both operands), the tcgen05 GEMM, the 9-block sum.
// Stacking keeps each operand's orientation: an operand stored [rows = MN][K] gets its planes one
// below the other, an operand stored [K][MN] gets them side by side (row pitch 3 MN), so all four
// transpose combinations reach the GEMM with the caller's flags unchanged.
#include <cuda_bf16.h>

#include "common.cuh"

namespace fb {
namespace {

struct SplitOperand {
  const float* src;
  __nv_bfloat16* dst;
  int64_t rows, cols, ld;       // as stored
  int64_t dst_ld, plane;        // destination row pitch and distance between planes (elements)
  int vec;                      // source rows 16-byte aligned and cols % 4 == 0
};

__device__ __forceinline__ void split3(float x, __nv_bfloat16& p0, __nv_bfloat16& p1, __nv_bfloat16& p2) {
  p0 = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(p0);   // exact
  p1 = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(p1);  // exact
  p2 = __float2bfloat16_rn(r2);
}

// grid.y selects the operand; four consecutive columns per thread
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const SplitOperand a, const SplitOperand b) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const SplitOperand& o = blockIdx.y == 0 ? a : b;
  const int64_t quads_per_row = (o.cols + 3) / 4;
  const int64_t total = o.rows * quads_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / quads_per_row, c = (i % quads_per_row) * 4;
    const float* s = o.src + r * o.ld + c;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const int n = (int)(o.cols - c < 4 ? o.cols - c : 4);
    if (o.vec && n == 4) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(s));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
      for (int j = 0; j < n; ++j) v[j] = __ldg(s + j);
    }
    __nv_bfloat16 p[3][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) split3(v[j], p[0][j], p[1][j], p[2][j]);
    __nv_bfloat16* d = o.dst + r * o.dst_ld + c;
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
      // destination rows are 16-byte aligned and c is a multiple of 4: 8-byte stores
      if (n == 4) {
        uint2 w;
        w.x = (uint32_t)__bfloat16_as_ushort(p[pl][0]) | ((uint32_t)__bfloat16_as_ushort(p[pl][1]) << 16);
        w.y = (uint32_t)__bfloat16_as_ushort(p[pl][2]) | ((uint32_t)__bfloat16_as_ushort(p[pl][3]) << 16);
        *reinterpret_cast<uint2*>(d + pl * o.plane) = w;
      } else {
        for (int j = 0; j < n; ++j) d[pl * o.plane + j] = p[pl][j];
      }
    }
  }
}

// C[i][j] <- (accumulate ? C[i][j] : 0) + sum over the nine blocks P[s*M + i][t*N + j], smallest terms first
__global__ void __launch_bounds__(256) sum9_kernel(const float* __restrict__ P, int64_t ldp, int64_t M, int64_t N,
                                                   float* __restrict__ C, int64_t ldc, int accumulate, int vec_c) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t quads = N / 4;  // N % 4 == 0 on this path
  const int64_t total = M * quads;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / quads, c = (i % quads) * 4;
    auto blk = [&](int s, int t) {
      return __ldcs(reinterpret_cast<const float4*>(P + ((int64_t)s * M + r) * ldp + (int64_t)t * N + c));
    };
    // order of magnitude of A_s.B_t is 2^(-8 (s + t)): add from s + t = 4 down to 0
    const float4 b22 = blk(2, 2), b21 = blk(2, 1), b12 = blk(1, 2), b20 = blk(2, 0), b02 = blk(0, 2),
                 b11 = blk(1, 1), b10 = blk(1, 0), b01 = blk(0, 1), b00 = blk(0, 0);
    float4 acc;
#define FB_SUM9(f) acc.f = ((((((((b22.f + b21.f) + b12.f) + b20.f) + b02.f) + b11.f) + b10.f) + b01.f) + b00.f)
    FB_SUM9(x); FB_SUM9(y); FB_SUM9(z); FB_SUM9(w);
#undef FB_SUM9
    float* dst = C + r * ldc + c;
    if (vec_c) {
      if (accumulate) {
        const float4 old = *reinterpret_cast<const float4*>(dst);
        acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w;
      }
      *reinterpret_cast<float4*>(dst) = acc;
    } else {
      const float v[4] = {acc.x, acc.y, acc.z, acc.w};
      for (int j = 0; j < 4; ++j) dst[j] = accumulate ? dst[j] + v[j] : v[j];
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int own_buffer(frisk_b200_ctx* ctx, int slot, size_t bytes) {
  StagingBuffer& b = ctx->stage[slot];
  if (b.ptr && b.bytes >= bytes) return 0;
  if (b.ptr) {
    FB_CUDA(ctx, cudaFree(b.ptr));
    b.ptr = nullptr;
    b.bytes = 0;
  }
  const size_t want = (bytes + 255) / 256 * 256;
  FB_CUDA(ctx, cudaMalloc(&b.ptr, want));
  b.bytes = want;
  return 0;
}

template <typename... Args>
int launch_pdl(frisk_b200_ctx* ctx, void (*kern)(Args...), unsigned grid_x, unsigned grid_y, cudaStream_t s,
               Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, grid_y);
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernels wait (griddepcontrol.wait) themselves
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, args...));
  return 0;
}

}  // namespace

// TMA wants 16-byte row pitches of the stacked bf16 operands and the sum works on whole float4s
bool f32_split_supported(const frisk_b200_gemm_desc& d) {
  if (d.dtype_ab != FRISK_B200_F32 || d.dtype_c != FRISK_B200_F32) return false;
  if (d.M % 8 || d.N % 8 || d.K % 8) return false;
  return 3 * d.M <= INT32_MAX && 3 * d.N <= INT32_MAX && d.K <= INT32_MAX;
}

// Worth the two extra passes only when the product is large next to them
bool f32_split_preferred(const frisk_b200_gemm_desc& d) {
  return f32_split_supported(d) && d.M >= 256 && d.N >= 256 && d.K >= 256;
}

int launch_gemm_f32_split(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const float* A, const float* B,
                          float* C, cudaStream_t s) {
  if (!f32_split_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  const GemmDims g = resolve_dims(d);
  const int64_t M = g.M, N = g.N, K = g.K;

  // context-owned scratch: the stacked operands, the 3M x 3N product, the GEMM's own tail scratch
  frisk_b200_gemm_desc t = {};
  t.M = 3 * M;
  t.N = 3 * N;
  t.K = K;
  t.dtype_ab = FRISK_B200_BF16;
  t.dtype_c = FRISK_B200_F32;
  t.trans_a = d.trans_a;
  t.trans_b = d.trans_b;
  t.clear_accum = 1;
  t.lda = d.trans_a ? 3 * M : K;
  t.ldb = d.trans_b ? K : 3 * N;
  t.ldc = 3 * N;
  t.algo = tcgen05_2cta_preferred(t) ? FRISK_B200_ALGO_TCGEN05_PAIR : FRISK_B200_ALGO_TCGEN05;
  const size_t tail = t.algo == FRISK_B200_ALGO_TCGEN05_PAIR ? tcgen05_2cta_workspace_bytes(t) : 0;
  void *pa, *pb, *pp, *ws = nullptr;
  size_t ws_bytes = 0;
  {
    std::lock_guard<std::recursive_mutex> lock(ctx->mu);
    int rc;
    if ((rc = own_buffer(ctx, 8, (size_t)3 * M * K * 2))) return rc;
    if ((rc = own_buffer(ctx, 9, (size_t)3 * N * K * 2))) return rc;
    if ((rc = own_buffer(ctx, 10, (size_t)9 * M * N * 4))) return rc;
    if (tail) {
      StagingBuffer& b = ctx->stage[5];
      if (!b.ptr || b.bytes < tail) {
        if ((rc = own_buffer(ctx, 5, tail))) return rc;
        FB_CUDA(ctx, cudaMemsetAsync(b.ptr, 0, b.bytes, s));  // tickets start at zero; every launch leaves them so
      }
      ws = b.ptr;
      ws_bytes = b.bytes;
    }
    pa = ctx->stage[8].ptr;
    pb = ctx->stage[9].ptr;
    pp = ctx->stage[10].ptr;
  }

  SplitOperand oa, ob;
  oa.src = A;
  oa.dst = static_cast<__nv_bfloat16*>(pa);
  oa.rows = d.trans_a ? K : M;
  oa.cols = d.trans_a ? M : K;
  oa.ld = g.lda;
  oa.dst_ld = t.lda;
  oa.plane = d.trans_a ? M : M * K;
  oa.vec = aligned16(A) && g.lda % 4 == 0;
  ob.src = B;
  ob.dst = static_cast<__nv_bfloat16*>(pb);
  ob.rows = d.trans_b ? N : K;
  ob.cols = d.trans_b ? K : N;
  ob.ld = g.ldb;
  ob.dst_ld = t.ldb;
  ob.plane = d.trans_b ? N * K : N;
  ob.vec = aligned16(B) && g.ldb % 4 == 0;
  const int64_t quads = std::max(oa.rows * ((oa.cols + 3) / 4), ob.rows * ((ob.cols + 3) / 4));
  const unsigned gx = (unsigned)std::min<int64_t>((quads + 255) / 256, (int64_t)ctx->num_sms * 8);
  int rc = launch_pdl(ctx, split_bf16x3_kernel, gx, 2u, s, oa, ob);
  if (rc) return rc;

  rc = t.algo == FRISK_B200_ALGO_TCGEN05_PAIR ? launch_gemm_tcgen05_2cta(ctx, t, pa, pb, pp, ws, ws_bytes, s)
                                              : launch_gemm_tcgen05(ctx, t, pa, pb, pp, s);
  if (rc) return rc;

  const int64_t out_quads = M * (N / 4);
  const unsigned gs = (unsigned)std::min<int64_t>((out_quads + 255) / 256, (int64_t)ctx->num_sms * 8);
  return launch_pdl(ctx, sum9_kernel, gs, 1u, s, static_cast<const float*>(pp), (int64_t)(3 * N), M, N, C, g.ldc,
                    d.clear_accum ? 0 : 1, (int)(aligned16(C) && g.ldc % 4 == 0));
}

}  // namespace fb
