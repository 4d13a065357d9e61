// C ABI of libfrisk_b200 (include/frisk_b200.h): context, host-side contract checks,
// kernel selection, and the host-buffer entry points.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace fb {

// ---------------------------------------------------------------- TMA descriptor encode
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
CUtensorMapDataType tmap_dtype(int dt) {
  switch (dt) {
    case FRISK_B200_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case FRISK_B200_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}
}  // namespace

namespace {
int encode_tiled(CUtensorMap* out, const TmapKey& k) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return 999;
  cuuint64_t dims[3] = {k.dims[0], k.dims[1], k.dims[2]};
  cuuint64_t strides[2] = {k.strides[0], k.strides[1]};
  cuuint32_t box[3] = {k.box[0], k.box[1], k.box[2]};
  cuuint32_t estr[3] = {1, 1, 1};
  return (int)fn(out, tmap_dtype(k.dtype), (cuuint32_t)k.rank, const_cast<void*>(k.base), dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, k.swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}
// A descriptor depends only on its key (it holds no reference to the memory besides the
// address), so a cached one stays valid however often the buffer's contents change.
int cached_tmap(frisk_b200_ctx* ctx, CUtensorMap* out, const TmapKey& k) {
  if (!ctx) return encode_tiled(out, k);
  std::lock_guard<std::mutex> lock(ctx->tmap_mu);
  ++ctx->tmap_clock;
  size_t oldest = 0;
  for (size_t i = 0; i < ctx->tmaps.size(); ++i) {
    if (ctx->tmaps[i].key == k) {
      ctx->tmaps[i].stamp = ctx->tmap_clock;
      *out = ctx->tmaps[i].map;
      return 0;
    }
    if (ctx->tmaps[i].stamp < ctx->tmaps[oldest].stamp) oldest = i;
  }
  const int rc = encode_tiled(out, k);
  if (rc) return rc;
  TmapEntry e{k, *out, ctx->tmap_clock};
  if (ctx->tmaps.size() < kTmapCacheEntries) ctx->tmaps.push_back(e); else ctx->tmaps[oldest] = e;
  return 0;
}
}  // namespace

int encode_tmap_2d(frisk_b200_ctx* ctx, CUtensorMap* out, int dtype, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                   bool swizzle128) {
  TmapKey k{base, {inner, outer, 1}, {outer_stride_bytes, 0}, {box_inner, box_outer, 1}, dtype, 2, swizzle128 ? 1 : 0};
  return cached_tmap(ctx, out, k);
}

int encode_tmap_3d(frisk_b200_ctx* ctx, CUtensorMap* out, int dtype, const void* base, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                   uint32_t b2, bool swizzle128) {
  TmapKey k{base, {d0, d1, d2}, {stride1_bytes, stride2_bytes}, {b0, b1, b2}, dtype, 3, swizzle128 ? 1 : 0};
  return cached_tmap(ctx, out, k);
}

// ---------------------------------------------------------------- small kernels
namespace {
template <typename T>
__global__ void convert_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // 8 elements per thread per step when everything is 16-byte aligned
  int64_t n8 = n / 8;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
    for (int64_t v = i; v < n8; v += stride) {
      float4 a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * v);
      float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * v + 1);
      T o[8] = {T(a.x), T(a.y), T(a.z), T(a.w), T(b.x), T(b.y), T(b.z), T(b.w)};
      reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<uint4*>(o);
    }
    for (int64_t k = n8 * 8 + i; k < n; k += stride) dst[k] = T(src[k]);
  } else {
    for (int64_t k = i; k < n; k += stride) dst[k] = T(src[k]);
  }
}
}  // namespace

namespace {
// dst[i] = round(slots[0][i] + slots[1][i] + ...), in slot order: the partial products the ranks of a
// K-split GEMM stored into this GPU's slots, summed and rounded in one pass over them
template <typename T>
__global__ void sum_slots_kernel(const float* __restrict__ slots, int n_slots, int64_t slot_elems,
                                 T* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n8 = n / 8;
  const bool vec = (reinterpret_cast<uintptr_t>(slots) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 &&
                   slot_elems % 4 == 0;
  if (vec) {
    for (int64_t v = i; v < n8; v += stride) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      for (int s = 0; s < n_slots; ++s) {
        const float4* p = reinterpret_cast<const float4*>(slots + (int64_t)s * slot_elems);
        const float4 x = __ldcs(p + 2 * v), y = __ldcs(p + 2 * v + 1);
        a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
        b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
      }
      T o[8] = {T(a.x), T(a.y), T(a.z), T(a.w), T(b.x), T(b.y), T(b.z), T(b.w)};
      reinterpret_cast<uint4*>(dst)[v] = *reinterpret_cast<uint4*>(o);
    }
  }
  for (int64_t k = (vec ? n8 * 8 : 0) + i; k < n; k += stride) {
    float acc = 0.f;
    for (int s = 0; s < n_slots; ++s) acc += slots[(int64_t)s * slot_elems + k];
    dst[k] = T(acc);
  }
}
}  // namespace

int launch_sum_slots(const float* slots, int n_slots, int64_t slot_elems, void* dst, int64_t n, int dtype,
                     cudaStream_t s) {
  if (n <= 0) return 0;
  int blocks = (int)((n / 8 + 255) / 256);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == FRISK_B200_F16)
    sum_slots_kernel<__half><<<blocks, 256, 0, s>>>(slots, n_slots, slot_elems, static_cast<__half*>(dst), n);
  else if (dtype == FRISK_B200_BF16)
    sum_slots_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(slots, n_slots, slot_elems, static_cast<__nv_bfloat16*>(dst), n);
  else
    return FRISK_B200_E_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? 0 : FRISK_B200_E_CUDA;
}

int launch_convert_f32(const float* src, void* dst, int64_t n, int dtype, cudaStream_t s) {
  if (n <= 0) return 0;
  int blocks = (int)((n / 8 + 255) / 256);
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == FRISK_B200_F16)
    convert_f32_kernel<__half><<<blocks, 256, 0, s>>>(src, static_cast<__half*>(dst), n);
  else if (dtype == FRISK_B200_BF16)
    convert_f32_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  else
    return FRISK_B200_E_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? 0 : FRISK_B200_E_CUDA;
}

// ---------------------------------------------------------------- helpers
namespace {

// (Re)allocates a context-owned buffer.  `zero`: fresh memory is cleared ON `s`, the stream
// the kernel that needs the zeroed control words is launched on (a clear on the legacy
// default stream would not be ordered before a kernel on a non-blocking stream).
int ensure_stage(frisk_b200_ctx* ctx, int slot, size_t bytes, bool zero, cudaStream_t s = nullptr) {
  StagingBuffer& b = ctx->stage[slot];
  if (b.bytes >= bytes && b.ptr) return 0;
  if (b.ptr) {
    FB_CUDA(ctx, cudaFree(b.ptr));
    b.ptr = nullptr;
    b.bytes = 0;
  }
  size_t want = (bytes + 255) / 256 * 256;
  FB_CUDA(ctx, cudaMalloc(&b.ptr, want));
  b.bytes = want;
  if (zero) FB_CUDA(ctx, cudaMemsetAsync(b.ptr, 0, want, s));
  return 0;
}

// Library-owned skinny-GEMM scratch: allocated (zeroed) on demand; its control prefix is
// cleared on the launch stream whenever the control layout differs from the last use.
int prepare_owned_skinny_ws(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, cudaStream_t s) {
  size_t need = skinny_workspace_bytes(d);
  void* before = ctx->stage[3].ptr;
  int rc = ensure_stage(ctx, 3, need, true, s);
  if (rc) return rc;
  uint64_t sig = (uint64_t)skinny_control_bytes(d) | (1ull << 63);
  if (ctx->stage[3].ptr != before) {
    ctx->ws_signature = sig;  // fresh and fully zeroed
  } else if (ctx->ws_signature != sig) {
    FB_CUDA(ctx, cudaMemsetAsync(ctx->stage[3].ptr, 0, skinny_control_bytes(d), s));
    ctx->ws_signature = sig;
  }
  return 0;
}

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" {

const char* frisk_b200_version(void) { return "frisk_b200 0.1 (sm_100a)"; }

const char* frisk_b200_strerror(int code) {
  switch (code) {
    case FRISK_B200_OK: return "ok";
    case FRISK_B200_E_GEMM_SHAPE: return "legacy-gemm-shape: A, B and C must be rank-2 with positive M, N, K and matching effective shapes";
    case FRISK_B200_E_GEMM_TYPE: return "legacy-gemm-type: A and B must share an element type; C must match it or be f32 for f16/bf16 inputs";
    case FRISK_B200_E_ALIGN: return "operand base address or row pitch is not 16-byte aligned";
    case FRISK_B200_E_OVERLAP: return "output overlaps an input";
    case FRISK_B200_E_WORKSPACE: return "workspace missing or too small";
    case FRISK_B200_E_UNSUPPORTED: return "no kernel for this element type / layout / algorithm";
    case FRISK_B200_E_ARG: return "invalid argument";
    case FRISK_B200_E_ATTN_SHAPE: return "shape outside the attention launch contract";
    case FRISK_B200_E_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
    case FRISK_B200_E_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case FRISK_B200_E_CUDA: return "CUDA call failed";
    default: return "unknown frisk_b200 status";
  }
}

int frisk_b200_ctx_create(frisk_b200_ctx** out, int device) {
  if (!out) return FRISK_B200_E_ARG;
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return FRISK_B200_E_CUDA;
  frisk_b200_ctx* ctx = new frisk_b200_ctx();
  ctx->device = device;
  auto fail = [&](cudaError_t e) {
    ctx->last_cuda = (int)e;
    delete ctx;
    return FRISK_B200_E_CUDA;
  };
  cudaError_t e;
  DeviceGuard guard(device);  // the caller's current device is put back on return
  if ((e = guard.error()) != cudaSuccess) return fail(e);
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return fail(e);
  if (prop.major != 10) {  // sm_100a code only: fail loudly on anything else
    delete ctx;
    return FRISK_B200_E_UNSUPPORTED;
  }
  ctx->num_sms = prop.multiProcessorCount;
  if ((e = cudaMalloc(&ctx->d_status, 256)) != cudaSuccess) return fail(e);
  if ((e = cudaMemset(ctx->d_status, 0, 256)) != cudaSuccess) return fail(e);
  if ((e = cudaMallocHost(&ctx->h_status, 256)) != cudaSuccess) return fail(e);
  ctx->h_status[0] = 0;
  if ((e = cudaStreamCreateWithFlags(&ctx->host_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
  if ((e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
  if ((e = cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
  for (auto& ev : ctx->ev)
    if ((e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming)) != cudaSuccess) return fail(e);
  *out = ctx;
  return 0;
}

int frisk_b200_ctx_destroy(frisk_b200_ctx* ctx) {
  if (!ctx) return FRISK_B200_E_ARG;
  DeviceGuard guard(ctx->device);
  cudaDeviceSynchronize();
  for (auto& b : ctx->stage)
    if (b.ptr) cudaFree(b.ptr);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  for (auto& ev : ctx->ev)
    if (ev) cudaEventDestroy(ev);
  if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  if (ctx->out_stream) cudaStreamDestroy(ctx->out_stream);
  delete ctx;
  return 0;
}

int frisk_b200_last_status(frisk_b200_ctx* ctx) { return ctx ? ctx->last_status : FRISK_B200_E_ARG; }
int frisk_b200_last_cuda(frisk_b200_ctx* ctx) { return ctx ? ctx->last_cuda : FRISK_B200_E_ARG; }

int frisk_b200_check(frisk_b200_ctx* ctx, void* stream) {
  if (!ctx) return FRISK_B200_E_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
  FB_CUDA(ctx, cudaStreamSynchronize(s));
  ctx->last_status = (int)ctx->h_status[0];
  if (ctx->last_status != 0) {
    cudaMemsetAsync(ctx->d_status, 0, sizeof(unsigned), s);
    cudaStreamSynchronize(s);
    return FRISK_B200_E_DEVICE_TIMEOUT;
  }
  return 0;
}

// ------------------------------------------------------------------------------ GEMM
int frisk_b200_gemm_validate(const frisk_b200_gemm_desc* d) {
  if (!d) return FRISK_B200_E_ARG;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) return FRISK_B200_E_GEMM_SHAPE;
  if (!dtype_ok(d->dtype_ab) || !dtype_ok(d->dtype_c)) return FRISK_B200_E_GEMM_TYPE;
  bool same = d->dtype_c == d->dtype_ab;
  bool low_f32 = (d->dtype_ab == FRISK_B200_F16 || d->dtype_ab == FRISK_B200_BF16) && d->dtype_c == FRISK_B200_F32;
  if (!same && !low_f32) return FRISK_B200_E_GEMM_TYPE;
  GemmDims g = resolve_dims(*d);
  int64_t a_cols = d->trans_a ? g.M : g.K, b_cols = d->trans_b ? g.K : g.N;
  if (g.lda < a_cols || g.ldb < b_cols || g.ldc < g.N) return FRISK_B200_E_GEMM_SHAPE;
  if (d->algo < FRISK_B200_ALGO_AUTO || d->algo > FRISK_B200_ALGO_F32_SPLIT) return FRISK_B200_E_ARG;
  return 0;
}

int frisk_b200_gemm_check_memrefs(int32_t a_rank, const int64_t* a_shape, int32_t a_dtype, int32_t b_rank,
                                  const int64_t* b_shape, int32_t b_dtype, int32_t c_rank, const int64_t* c_shape,
                                  int32_t c_dtype, int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                                  const char** message) {
  const char* msg = nullptr;
  int code = 0;
  auto fail = [&](int c, const char* text) {
    code = c;
    msg = text;
  };
  auto is_static = [](int rank, const int64_t* shape) {
    for (int i = 0; i < rank; ++i)
      if (shape[i] < 0) return false;
    return true;
  };
  if (!a_shape || !b_shape || !c_shape) {
    fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: A, B, and C must be memrefs");
  } else if (a_rank != 2 || b_rank != 2 || c_rank != 2) {
    fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: A, B, and C must have rank 2");
  } else if (!is_static(2, a_shape) || !is_static(2, b_shape) || !is_static(2, c_shape)) {
    fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: A, B, and C must have static shapes");
  } else if (m <= 0 || n <= 0 || k <= 0) {
    fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: M, N, and K must be positive");
  } else if (a_dtype != b_dtype) {
    fail(FRISK_B200_E_GEMM_TYPE, "legacy-gemm-type: A and B must have the same element type");
  } else if (!(c_dtype == a_dtype ||
               ((a_dtype == FRISK_B200_F16 || a_dtype == FRISK_B200_BF16) && c_dtype == FRISK_B200_F32))) {
    fail(FRISK_B200_E_GEMM_TYPE, "legacy-gemm-type: C must match A/B or be f32 for f16/bf16 inputs");
  } else {
    int64_t am = a_shape[trans_a ? 1 : 0], ak = a_shape[trans_a ? 0 : 1];
    int64_t bk = b_shape[trans_b ? 1 : 0], bn = b_shape[trans_b ? 0 : 1];
    if (am != m || ak != k || bk != k || bn != n)
      fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: effective A/B shapes must match M/N/K");
    else if (c_shape[0] != m || c_shape[1] != n)
      fail(FRISK_B200_E_GEMM_SHAPE, "legacy-gemm-shape: C shape must be MxN");
  }
  if (message) *message = msg;
  return code;
}

int frisk_b200_gemm_select(const frisk_b200_gemm_desc* d) {
  int rc = frisk_b200_gemm_validate(d);
  if (rc) return rc;
  if (d->algo != FRISK_B200_ALGO_AUTO) {
    if (d->algo == FRISK_B200_ALGO_SIMT_F32) return d->dtype_ab == FRISK_B200_F32 ? d->algo : FRISK_B200_E_UNSUPPORTED;
    if (d->algo == FRISK_B200_ALGO_F32_SPLIT) return f32_split_supported(*d) ? d->algo : FRISK_B200_E_UNSUPPORTED;
    if (d->algo == FRISK_B200_ALGO_SKINNY) return skinny_supported(*d) ? d->algo : FRISK_B200_E_UNSUPPORTED;
    if (d->algo == FRISK_B200_ALGO_TCGEN05 || d->algo == FRISK_B200_ALGO_TCGEN05_PAIR)
      return tcgen05_supported(*d) ? d->algo : FRISK_B200_E_UNSUPPORTED;
  }
  if (d->dtype_ab == FRISK_B200_F32) return f32_split_preferred(*d) ? FRISK_B200_ALGO_F32_SPLIT : FRISK_B200_ALGO_SIMT_F32;
  if (skinny_supported(*d)) return FRISK_B200_ALGO_SKINNY;
  if (tcgen05_supported(*d)) return tcgen05_2cta_preferred(*d) ? FRISK_B200_ALGO_TCGEN05_PAIR : FRISK_B200_ALGO_TCGEN05;
  return FRISK_B200_E_ALIGN;  // 16-bit operands whose pitch is not a multiple of 16 bytes
}

size_t frisk_b200_gemm_workspace_bytes(const frisk_b200_gemm_desc* d) {
  int algo = frisk_b200_gemm_select(d);
  if (algo == FRISK_B200_ALGO_SKINNY) return skinny_workspace_bytes(*d);
  if (algo == FRISK_B200_ALGO_TCGEN05_PAIR) return tcgen05_2cta_workspace_bytes(*d);
  return 0;
}

int frisk_b200_gemm(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* d, const void* A, const void* B, void* C,
                    void* workspace, size_t workspace_bytes, void* stream) {
  if (!ctx || !d || !A || !B || !C) return FRISK_B200_E_ARG;
  int algo = frisk_b200_gemm_select(d);
  if (algo < 0) return algo;
  GemmExtents e = gemm_extents(*d);
  if (ranges_overlap(C, e.c, A, e.a) || ranges_overlap(C, e.c, B, e.b)) return FRISK_B200_E_OVERLAP;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FB_DEVICE(ctx);
  switch (algo) {
    case FRISK_B200_ALGO_SIMT_F32:
      return launch_gemm_simt_f32(ctx, *d, static_cast<const float*>(A), static_cast<const float*>(B),
                                  static_cast<float*>(C), s);
    case FRISK_B200_ALGO_F32_SPLIT:
      return launch_gemm_f32_split(ctx, *d, static_cast<const float*>(A), static_cast<const float*>(B),
                                   static_cast<float*>(C), s);
    case FRISK_B200_ALGO_SKINNY: {
      size_t need = skinny_workspace_bytes(*d);
      if (!workspace) {
        // library-owned scratch: zeroed when (re)allocated, left clean by every launch
        std::lock_guard<std::recursive_mutex> lock(ctx->mu);
        (void)need;
        int rc = prepare_owned_skinny_ws(ctx, *d, s);
        if (rc) return rc;
        workspace = ctx->stage[3].ptr;
        workspace_bytes = ctx->stage[3].bytes;
      }
      return launch_gemm_skinny(ctx, *d, A, B, C, workspace, workspace_bytes, s);
    }
    case FRISK_B200_ALGO_TCGEN05:
      return launch_gemm_tcgen05(ctx, *d, A, B, C, s);
    case FRISK_B200_ALGO_TCGEN05_PAIR: {
      size_t need = tcgen05_2cta_workspace_bytes(*d);
      if (need && !workspace) {
        // library-owned scratch: zeroed when allocated, tickets are left at zero by every launch
        std::lock_guard<std::recursive_mutex> lock(ctx->mu);
        int rc = ensure_stage(ctx, 5, need, true, s);
        if (rc) return rc;
        workspace = ctx->stage[5].ptr;
        workspace_bytes = ctx->stage[5].bytes;
      }
      return launch_gemm_tcgen05_2cta(ctx, *d, A, B, C, workspace, workspace_bytes, s);
    }
  }
  return FRISK_B200_E_UNSUPPORTED;
}

int frisk_b200_gemm_host(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* d, const void* A, const void* B,
                         void* C) {
  if (!ctx || !d || !A || !B || !C) return FRISK_B200_E_ARG;
  int algo = frisk_b200_gemm_select(d);
  if (algo < 0) return algo;
  FB_DEVICE(ctx);
  GemmExtents e = gemm_extents(*d);
  std::lock_guard<std::recursive_mutex> lock(ctx->mu);
  int rc;
  if ((rc = ensure_stage(ctx, 0, e.a, false))) return rc;
  if ((rc = ensure_stage(ctx, 1, e.b, false))) return rc;
  if ((rc = ensure_stage(ctx, 2, e.c, false))) return rc;
  cudaStream_t s = ctx->host_stream, s2 = ctx->copy_stream, s3 = ctx->out_stream;
  if (algo == FRISK_B200_ALGO_SKINNY && (rc = prepare_owned_skinny_ws(ctx, *d, s))) return rc;
  if (size_t need = (algo == FRISK_B200_ALGO_TCGEN05_PAIR ? tcgen05_2cta_workspace_bytes(*d) : 0))
    if ((rc = ensure_stage(ctx, 5, need, true, s))) return rc;
  GemmDims g = resolve_dims(*d);
  const size_t es = dtype_size(d->dtype_ab), cs = dtype_size(d->dtype_c);

  // Row panels of A and C travel while other panels are multiplied: H2D on one stream, the
  // kernels on a second, D2H on a third, ordered by events (PCIe is full duplex, so the
  // copy-out of panel p overlaps the copy-in of panel p+1).  Only when A's rows are
  // contiguous in the buffer (trans_a = 0) and the problem is large enough to split.
  // Panel boundaries are multiples of 256 rows; four panels (more only add per-copy overheads).
  // Every panel runs the kernel chosen for the WHOLE problem (its scratch is the one prepared
  // above, and an explicit desc->algo is honoured); a last panel shorter than 256 rows is
  // merged into the one before it.
  int64_t bounds[8] = {0};
  int panels = 1;
  bounds[1] = g.M;
  if (!d->trans_a && algo != FRISK_B200_ALGO_SKINNY && g.M >= 1024 && e.a + e.c >= ((size_t)8 << 20)) {
    constexpr int want = 4;
    panels = 0;
    for (int i = 0; i < want; ++i) {
      int64_t end = g.M * (i + 1) / want;
      end = i + 1 == want ? g.M : std::min<int64_t>(g.M, (end + 255) / 256 * 256);
      if (end > bounds[panels]) bounds[++panels] = end;
    }
    if (panels > 1 && bounds[panels] - bounds[panels - 1] < 256) bounds[--panels] = g.M;
  }

  FB_CUDA(ctx, cudaMemcpyAsync(ctx->stage[1].ptr, B, e.b, cudaMemcpyHostToDevice, s2));
  for (int p = 0; p < panels; ++p) {
    const int64_t r0 = bounds[p], rows = bounds[p + 1] - r0;
    frisk_b200_gemm_desc dp = *d;
    dp.M = rows;
    dp.lda = g.lda;
    dp.ldb = g.ldb;
    dp.ldc = g.ldc;
    dp.algo = algo;
    const int algo_p = algo;
    // with trans_a the single panel is the whole (K x M) buffer
    const size_t a_off = d->trans_a ? 0 : (size_t)r0 * g.lda * es, a_bytes = panels == 1 ? e.a : operand_bytes(rows, g.K, g.lda, es);
    const size_t c_off = (size_t)r0 * g.ldc * cs, c_bytes = operand_bytes(rows, g.N, g.ldc, cs);
    unsigned char* dA = static_cast<unsigned char*>(ctx->stage[0].ptr) + a_off;
    unsigned char* dC = static_cast<unsigned char*>(ctx->stage[2].ptr) + c_off;
    FB_CUDA(ctx, cudaMemcpyAsync(dA, static_cast<const unsigned char*>(A) + a_off, a_bytes, cudaMemcpyHostToDevice, s2));
    if (!d->clear_accum)
      FB_CUDA(ctx, cudaMemcpyAsync(dC, static_cast<const unsigned char*>(C) + c_off, c_bytes, cudaMemcpyHostToDevice, s2));
    FB_CUDA(ctx, cudaEventRecord(ctx->ev[2 * p], s2));
    FB_CUDA(ctx, cudaStreamWaitEvent(s, ctx->ev[2 * p], 0));
    switch (algo_p) {
      case FRISK_B200_ALGO_SIMT_F32:
        rc = launch_gemm_simt_f32(ctx, dp, reinterpret_cast<const float*>(dA), static_cast<const float*>(ctx->stage[1].ptr),
                                  reinterpret_cast<float*>(dC), s);
        break;
      case FRISK_B200_ALGO_F32_SPLIT:
        rc = launch_gemm_f32_split(ctx, dp, reinterpret_cast<const float*>(dA), static_cast<const float*>(ctx->stage[1].ptr),
                                   reinterpret_cast<float*>(dC), s);
        break;
      case FRISK_B200_ALGO_SKINNY:
        rc = launch_gemm_skinny(ctx, dp, dA, ctx->stage[1].ptr, dC, ctx->stage[3].ptr, ctx->stage[3].bytes, s);
        break;
      case FRISK_B200_ALGO_TCGEN05_PAIR:
        rc = launch_gemm_tcgen05_2cta(ctx, dp, dA, ctx->stage[1].ptr, dC, ctx->stage[5].ptr, ctx->stage[5].bytes, s);
        break;
      default:
        rc = launch_gemm_tcgen05(ctx, dp, dA, ctx->stage[1].ptr, dC, s);
    }
    if (rc) return rc;
    FB_CUDA(ctx, cudaEventRecord(ctx->ev[2 * p + 1], s));
    FB_CUDA(ctx, cudaStreamWaitEvent(s3, ctx->ev[2 * p + 1], 0));
    FB_CUDA(ctx, cudaMemcpyAsync(static_cast<unsigned char*>(C) + c_off, dC, c_bytes, cudaMemcpyDeviceToHost, s3));
  }
  FB_CUDA(ctx, cudaEventRecord(ctx->ev[23], s3));
  FB_CUDA(ctx, cudaStreamWaitEvent(s, ctx->ev[23], 0));
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
  FB_CUDA(ctx, cudaStreamSynchronize(s));
  ctx->last_status = (int)ctx->h_status[0];
  if (ctx->last_status) {
    cudaMemsetAsync(ctx->d_status, 0, sizeof(unsigned), s);
    cudaStreamSynchronize(s);
    return FRISK_B200_E_DEVICE_TIMEOUT;
  }
  return 0;
}

// ------------------------------------------------------------------------------ attention
int frisk_b200_attention_validate(const frisk_b200_attn_desc* d) {
  if (!d) return FRISK_B200_E_ARG;
  if (d->B <= 0 || d->H <= 0 || d->S_q <= 0 || d->S_kv <= 0) return FRISK_B200_E_ATTN_SHAPE;
  if (d->D != 64 && d->D != 128) return FRISK_B200_E_ATTN_SHAPE;
  if (d->dtype_in != FRISK_B200_F16 && d->dtype_in != FRISK_B200_BF16) return FRISK_B200_E_UNSUPPORTED;
  if (d->dtype_out != d->dtype_in && d->dtype_out != FRISK_B200_F32) return FRISK_B200_E_UNSUPPORTED;
  if (d->causal && d->S_kv < d->S_q) return FRISK_B200_E_ATTN_SHAPE;
  if ((int64_t)d->B * d->H > INT32_MAX) return FRISK_B200_E_ATTN_SHAPE;
  if (!(d->scale == d->scale) || d->scale <= 0.f) return FRISK_B200_E_ARG;
  return 0;
}

size_t frisk_b200_attention_workspace_bytes(const frisk_b200_attn_desc* d) {
  (void)d;
  return 0;  // the 5th "scratch" argument of the reference ABI is unused there as well
}

int frisk_b200_attention_fwd(frisk_b200_ctx* ctx, const frisk_b200_attn_desc* d, const void* Q, const void* K,
                             const void* V, void* O, void* workspace, size_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  if (!ctx || !d || !Q || !K || !V || !O) return FRISK_B200_E_ARG;
  int rc = frisk_b200_attention_validate(d);
  if (rc) return rc;
  size_t es = dtype_size(d->dtype_in), os = dtype_size(d->dtype_out);
  size_t qb = (size_t)d->B * d->H * d->S_q * d->D * es, kb = (size_t)d->B * d->H * d->S_kv * d->D * es;
  size_t ob = (size_t)d->B * d->H * d->S_q * d->D * os;
  if (ranges_overlap(O, ob, Q, qb) || ranges_overlap(O, ob, K, kb) || ranges_overlap(O, ob, V, kb))
    return FRISK_B200_E_OVERLAP;
  for (const void* p : {Q, K, V, (const void*)O})
    if (reinterpret_cast<uintptr_t>(p) & 15u) return FRISK_B200_E_ALIGN;
  FB_DEVICE(ctx);
  return launch_attention_fwd(ctx, *d, Q, K, V, O, static_cast<cudaStream_t>(stream));
}

int frisk_b200_attention_fwd_host(frisk_b200_ctx* ctx, const frisk_b200_attn_desc* d, const void* Q,
                                  const void* K, const void* V, void* O) {
  if (!ctx || !d || !Q || !K || !V || !O) return FRISK_B200_E_ARG;
  int rc = frisk_b200_attention_validate(d);
  if (rc) return rc;
  FB_DEVICE(ctx);
  size_t es = dtype_size(d->dtype_in), os = dtype_size(d->dtype_out);
  size_t qb = (size_t)d->B * d->H * d->S_q * d->D * es, kb = (size_t)d->B * d->H * d->S_kv * d->D * es;
  size_t ob = (size_t)d->B * d->H * d->S_q * d->D * os;
  std::lock_guard<std::recursive_mutex> lock(ctx->mu);
  if ((rc = ensure_stage(ctx, 0, qb, false))) return rc;
  if ((rc = ensure_stage(ctx, 1, kb, false))) return rc;
  if ((rc = ensure_stage(ctx, 2, ob, false))) return rc;
  if ((rc = ensure_stage(ctx, 4, kb, false))) return rc;
  cudaStream_t s = ctx->host_stream, s2 = ctx->copy_stream;
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->stage[0].ptr, Q, qb, cudaMemcpyHostToDevice, s));
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->stage[1].ptr, K, kb, cudaMemcpyHostToDevice, s2));
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->stage[4].ptr, V, kb, cudaMemcpyHostToDevice, s));
  FB_CUDA(ctx, cudaEventRecord(ctx->ev[0], s2));
  FB_CUDA(ctx, cudaStreamWaitEvent(s, ctx->ev[0], 0));
  rc = launch_attention_fwd(ctx, *d, ctx->stage[0].ptr, ctx->stage[1].ptr, ctx->stage[4].ptr, ctx->stage[2].ptr, s);
  if (rc) return rc;
  FB_CUDA(ctx, cudaMemcpyAsync(O, ctx->stage[2].ptr, ob, cudaMemcpyDeviceToHost, s));
  FB_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(unsigned), cudaMemcpyDeviceToHost, s));
  FB_CUDA(ctx, cudaStreamSynchronize(s));
  ctx->last_status = (int)ctx->h_status[0];
  if (ctx->last_status) {
    cudaMemsetAsync(ctx->d_status, 0, sizeof(unsigned), s);
    cudaStreamSynchronize(s);
    return FRISK_B200_E_DEVICE_TIMEOUT;
  }
  return 0;
}

int frisk_b200_gemm_push(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* d, const void* A, const void* B,
                         float* const* targets, int32_t n_targets, int64_t rows_per_target, int64_t ld_target,
                         void* stream) {
  if (!ctx || !d || !A || !B || !targets) return FRISK_B200_E_ARG;
  int rc = frisk_b200_gemm_validate(d);
  if (rc) return rc;
  if (n_targets < 1 || n_targets > 8 || rows_per_target < 1 || rows_per_target * n_targets < d->M ||
      rows_per_target > INT32_MAX || ld_target < d->N)
    return FRISK_B200_E_ARG;
  PushTargets push{};
  for (int i = 0; i < n_targets; ++i) {
    if (!targets[i]) return FRISK_B200_E_ARG;
    if (reinterpret_cast<uintptr_t>(targets[i]) & 15u) return FRISK_B200_E_ALIGN;
    push.ptr[i] = targets[i];
  }
  push.n = n_targets;
  push.rows_per_target = (int)rows_per_target;
  push.ld = ld_target;
  FB_DEVICE(ctx);
  return launch_gemm_tcgen05_2cta_push(ctx, *d, A, B, push, static_cast<cudaStream_t>(stream));
}

// ---- gemm with the fill / row-reduce that Frisk's IR places on the same C
static int check_epilogue(const frisk_b200_gemm_desc* d, const frisk_b200_gemm_epilogue* e) {
  if (!d || !e) return FRISK_B200_E_ARG;
  int rc = frisk_b200_gemm_validate(d);
  if (rc) return rc;
  if (e->reduce_kind < FRISK_B200_REDUCE_NONE || e->reduce_kind > FRISK_B200_REDUCE_ADD) return FRISK_B200_E_UNSUPPORTED;
  if (e->reduce_kind != FRISK_B200_REDUCE_NONE && !e->reduce_dst) return FRISK_B200_E_ARG;
  if (!(e->fill_value == e->fill_value)) return FRISK_B200_E_ARG;  // NaN fill
  return 0;
}
static float round_fill(float v, int dtype) {
  if (dtype == FRISK_B200_F16) return __half2float(__float2half_rn(v));
  if (dtype == FRISK_B200_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}
int frisk_b200_gemm_fused_select(const frisk_b200_gemm_desc* d, const frisk_b200_gemm_epilogue* e) {
  int rc = check_epilogue(d, e);
  if (rc) return rc;
  int algo = frisk_b200_gemm_select(d);
  if (algo < 0) return algo;
  if (algo != FRISK_B200_ALGO_TCGEN05_PAIR) return 0;
  // a fused reduction needs the final value in registers: C must not be read back
  if (e->reduce_kind != FRISK_B200_REDUCE_NONE && !d->clear_accum && !e->fill_enable) return 0;
  return 1;
}
size_t frisk_b200_gemm_fused_workspace_bytes(const frisk_b200_gemm_desc* d, const frisk_b200_gemm_epilogue* e) {
  int fused = frisk_b200_gemm_fused_select(d, e);
  if (fused < 0) return 0;
  size_t base = (frisk_b200_gemm_workspace_bytes(d) + 255) / 256 * 256;
  if (fused == 1 && e->reduce_kind != FRISK_B200_REDUCE_NONE)
    base += (size_t)tcgen05_2cta_column_tiles(*d) * (size_t)d->M * sizeof(float);
  return base;
}
int frisk_b200_gemm_fused(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* d, const frisk_b200_gemm_epilogue* e,
                          const void* A, const void* B, void* C, void* workspace, size_t workspace_bytes,
                          void* stream) {
  if (!ctx || !A || !B || !C) return FRISK_B200_E_ARG;
  int fused = frisk_b200_gemm_fused_select(d, e);
  if (fused < 0) return fused;
  GemmExtents ext = gemm_extents(*d);
  GemmDims g = resolve_dims(*d);
  const size_t cs = dtype_size(d->dtype_c);
  if (ranges_overlap(C, ext.c, A, ext.a) || ranges_overlap(C, ext.c, B, ext.b)) return FRISK_B200_E_OVERLAP;
  if (e->reduce_kind != FRISK_B200_REDUCE_NONE &&
      (ranges_overlap(e->reduce_dst, (size_t)g.M * cs, C, ext.c) || ranges_overlap(e->reduce_dst, (size_t)g.M * cs, A, ext.a) ||
       ranges_overlap(e->reduce_dst, (size_t)g.M * cs, B, ext.b)))
    return FRISK_B200_E_OVERLAP;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  FB_DEVICE(ctx);
  const bool use_fill = e->fill_enable && !d->clear_accum;  // a fill before an overwriting gemm is dead
  const float fill = round_fill(e->fill_value, d->dtype_c);
  if (fused == 0) {
    int rc = 0;
    if (use_fill && (rc = launch_fill(C, g.M, g.N, g.ldc, fill, d->dtype_c, s))) return rc;
    if ((rc = frisk_b200_gemm(ctx, d, A, B, C, workspace, workspace_bytes, stream))) return rc;
    if (e->reduce_kind != FRISK_B200_REDUCE_NONE)
      rc = launch_row_reduce(C, g.M, g.N, g.ldc, e->reduce_kind, e->reduce_clear, e->reduce_dst, d->dtype_c, s);
    return rc;
  }
  const size_t tail = (tcgen05_2cta_workspace_bytes(*d) + 255) / 256 * 256;
  const int tiles_n = tcgen05_2cta_column_tiles(*d);
  const size_t part = e->reduce_kind != FRISK_B200_REDUCE_NONE ? (size_t)tiles_n * (size_t)g.M * sizeof(float) : 0;
  void* ws_tail = workspace;
  float* ws_part = nullptr;
  size_t ws_tail_bytes = 0;
  if (workspace) {
    if (workspace_bytes < tail + part) return FRISK_B200_E_WORKSPACE;
    ws_tail_bytes = tail;
    ws_part = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + tail);
  } else {
    std::lock_guard<std::recursive_mutex> lock(ctx->mu);
    int rc;
    if (tail) {
      if ((rc = ensure_stage(ctx, 5, tail, true, s))) return rc;
      ws_tail = ctx->stage[5].ptr;
      ws_tail_bytes = ctx->stage[5].bytes;
    }
    if (part) {
      if ((rc = ensure_stage(ctx, 6, part, false))) return rc;
      ws_part = static_cast<float*>(ctx->stage[6].ptr);
    }
  }
  if (!tail) ws_tail = nullptr;
  EpilogueArgs ea{};
  ea.has_fill = use_fill ? 1 : 0;
  ea.fill = fill;
  ea.reduce_kind = e->reduce_kind;
  ea.row_partials = ws_part;
  int rc = launch_gemm_tcgen05_2cta(ctx, *d, A, B, C, ws_tail, ws_tail_bytes, s, &ea);
  if (rc) return rc;
  if (e->reduce_kind != FRISK_B200_REDUCE_NONE)
    rc = launch_row_finalize(ws_part, tiles_n, g.M, e->reduce_kind, e->reduce_clear, e->reduce_dst, d->dtype_c, s);
  return rc;
}

int frisk_b200_sum_slots(frisk_b200_ctx* ctx, const float* slots, int32_t n_slots, int64_t slot_elems, void* dst,
                         int64_t count, int32_t dtype_dst, void* stream) {
  if (!ctx || !slots || !dst || count < 0 || n_slots < 1 || slot_elems < count) return FRISK_B200_E_ARG;
  FB_DEVICE(ctx);
  return launch_sum_slots(slots, n_slots, slot_elems, dst, count, dtype_dst, static_cast<cudaStream_t>(stream));
}

// ---- buffers other processes on this node can map (cudaIpc): the destinations of frisk_b200_gemm_push
int frisk_b200_peer_buffer_create(frisk_b200_ctx* ctx, size_t bytes, void** ptr, void* handle64) {
  if (!ctx || !ptr || !handle64 || bytes == 0) return FRISK_B200_E_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  FB_DEVICE(ctx);
  void* p = nullptr;
  FB_CUDA(ctx, cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // zero before the handle leaves this process
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    ctx->last_cuda = (int)e;
    return FRISK_B200_E_CUDA;
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return 0;
}
int frisk_b200_peer_buffer_open(frisk_b200_ctx* ctx, const void* handle64, void** ptr) {
  if (!ctx || !ptr || !handle64) return FRISK_B200_E_ARG;
  FB_DEVICE(ctx);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  FB_CUDA(ctx, cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int frisk_b200_peer_buffer_close(frisk_b200_ctx* ctx, void* ptr, int32_t owned) {
  if (!ctx || !ptr) return FRISK_B200_E_ARG;
  FB_DEVICE(ctx);
  if (owned) FB_CUDA(ctx, cudaFree(ptr)); else FB_CUDA(ctx, cudaIpcCloseMemHandle(ptr));
  return 0;
}

int frisk_b200_convert_f32(frisk_b200_ctx* ctx, const float* src, void* dst, int64_t count, int32_t dtype_dst,
                           void* stream) {
  if (!ctx || !src || !dst || count < 0) return FRISK_B200_E_ARG;
  FB_DEVICE(ctx);
  return launch_convert_f32(src, dst, count, dtype_dst, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
