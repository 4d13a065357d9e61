// What Frisk's IR can put next to a gemm on the same output: `frisk.fill` of C before an
// accumulating gemm and `frisk.reduce` of C along dim 1 after it (test/python/bind_test.py:44-53,
// reduce contract lib/Dialect/Frisk/IR/FriskOps.cpp:728-762: kinds add/mul/min/max, destination
// of the source's element type and one rank less).  The tcgen05 pair kernel folds both into its
// own epilogue and leaves one fp32 partial per (column tile, row); the kernels here finish that
// (fixed order over the column tiles, so the result is reproducible) and serve the GEMM kernels
// that have no fused form: a plain fill of C and a row reduction that reads C once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace fb {
namespace {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float reduce_identity(int kind) {
  return kind == FRISK_B200_REDUCE_MAX ? -INFINITY : kind == FRISK_B200_REDUCE_MIN ? INFINITY : 0.f;
}
__device__ __forceinline__ float reduce_combine(int kind, float a, float b) {
  return kind == FRISK_B200_REDUCE_MAX ? fmaxf(a, b) : kind == FRISK_B200_REDUCE_MIN ? fminf(a, b) : a + b;
}

// dst[row] = (clear ? id : dst[row]) (+) partials[0][row] (+) partials[1][row] ...
template <typename T>
__global__ void row_finalize_kernel(const float* __restrict__ partials, int tiles_n, int64_t M, int kind, int clear,
                                    T* __restrict__ dst) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float acc = clear ? reduce_identity(kind) : to_f(dst[row]);
  for (int t = 0; t < tiles_n; ++t) acc = reduce_combine(kind, acc, partials[(int64_t)t * M + row]);
  dst[row] = from_f<T>(acc);
}

// one CTA per row of C: 256 threads stride over the columns, fp32 accumulation, fixed tree
template <typename T>
__global__ void __launch_bounds__(256) row_reduce_kernel(const T* __restrict__ C, int64_t N, int64_t ldc, int kind,
                                                         int clear, T* __restrict__ dst) {
  const int64_t row = blockIdx.x;
  const T* p = C + row * ldc;
  float acc = reduce_identity(kind);
  for (int64_t j = threadIdx.x; j < N; j += 256) acc = reduce_combine(kind, acc, to_f(p[j]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = reduce_combine(kind, acc, __shfl_xor_sync(0xffffffffu, acc, o));
  __shared__ float warp_acc[8];
  if ((threadIdx.x & 31) == 0) warp_acc[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = clear ? reduce_identity(kind) : to_f(dst[row]);
#pragma unroll
    for (int w = 0; w < 8; ++w) r = reduce_combine(kind, r, warp_acc[w]);
    dst[row] = from_f<T>(r);
  }
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ C, int64_t M, int64_t N, int64_t ldc, float value) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  C[(i / N) * ldc + (i % N)] = from_f<T>(value);
}

}  // namespace

int launch_row_finalize(const float* partials, int tiles_n, int64_t M, int kind, int clear, void* dst, int dtype,
                        cudaStream_t s) {
  const unsigned blocks = (unsigned)((M + 255) / 256);
  if (dtype == FRISK_B200_F32)
    row_finalize_kernel<float><<<blocks, 256, 0, s>>>(partials, tiles_n, M, kind, clear, static_cast<float*>(dst));
  else if (dtype == FRISK_B200_F16)
    row_finalize_kernel<__half><<<blocks, 256, 0, s>>>(partials, tiles_n, M, kind, clear, static_cast<__half*>(dst));
  else
    row_finalize_kernel<__nv_bfloat16>
        <<<blocks, 256, 0, s>>>(partials, tiles_n, M, kind, clear, static_cast<__nv_bfloat16*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : FRISK_B200_E_CUDA;
}

int launch_row_reduce(const void* C, int64_t M, int64_t N, int64_t ldc, int kind, int clear, void* dst, int dtype,
                      cudaStream_t s) {
  if (M > INT32_MAX) return FRISK_B200_E_TOO_LARGE;
  const unsigned blocks = (unsigned)M;
  if (dtype == FRISK_B200_F32)
    row_reduce_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(C), N, ldc, kind, clear,
                                                     static_cast<float*>(dst));
  else if (dtype == FRISK_B200_F16)
    row_reduce_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(C), N, ldc, kind, clear,
                                                      static_cast<__half*>(dst));
  else
    row_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(C), N, ldc, kind,
                                                             clear, static_cast<__nv_bfloat16*>(dst));
  return cudaGetLastError() == cudaSuccess ? 0 : FRISK_B200_E_CUDA;
}

int launch_fill(void* C, int64_t M, int64_t N, int64_t ldc, float value, int dtype, cudaStream_t s) {
  const int64_t total = M * N;
  if ((total + 255) / 256 > INT32_MAX) return FRISK_B200_E_TOO_LARGE;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == FRISK_B200_F32)
    fill_kernel<float><<<blocks, 256, 0, s>>>(static_cast<float*>(C), M, N, ldc, value);
  else if (dtype == FRISK_B200_F16)
    fill_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<__half*>(C), M, N, ldc, value);
  else
    fill_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<__nv_bfloat16*>(C), M, N, ldc, value);
  return cudaGetLastError() == cudaSuccess ? 0 : FRISK_B200_E_CUDA;
}

}  // namespace fb
