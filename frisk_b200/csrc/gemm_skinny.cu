// Decode-shape ("skinny") GEMM: Y[M<=16, N] = X[M, K] . W[N, K]^T for fp16/bf16, fp32
// accumulation.  Contract: `frisk.gemm` with trans_a=0, trans_b=1
// (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).  The weight matrix is read exactly once, so
// the kernel is bound by HBM bandwidth; everything is arranged around keeping many 16-byte
// weight loads in flight.
//
// * K is split across CTAs (split s = blockIdx.x % S): a CTA stages only its K-slice of X
//   in shared memory (16 x K/S elements, rows padded by 64 bytes so that the fragment
//   reads below are bank-conflict free).
// * A warp owns one group of 8 weight rows at a time, taken from a per-split queue in the
//   workspace (an atomic counter), so all warps stay busy to the end of the stream.
// * HBM under load answers after 2-3 us, so ~128 KB per SM must be in flight to keep it busy:
//   more than registers can hold.  Each warp therefore streams its rows with cp.async (16
//   bytes per lane, one instruction = 512 contiguous bytes of one row, zero-filled past the
//   end of the slice) into a private ring of five 4 KB slots in shared memory and keeps four
//   256-wide k chunks in flight while it multiplies the oldest one.
// * The MMA wants lane (g, t) to supply row g.  Because a dot product does not care about the
//   order of k, the lane simply reads 16 bytes (8 consecutive k) of row g back from the slot
//   and feeds two m16n8k16 tensor-core MMAs with them as B fragments, with the matching 8
//   values of X rows g and g+8 as A fragments.  16-byte pieces are XOR-swizzled with the row
//   so that neither the cp.async writes nor these reads have bank conflicts.
// * With S > 1 a warp leaves its fp32 16x8 partial in the workspace and moves on (no fence, no
//   ticket: either would stall the warp's stream for a microsecond per row group); a second,
//   tiny kernel adds the S partials in split order (deterministic) and writes the rounded
//   output.  The id of the next row group is requested from the queue one chunk before it is
//   needed, so the atomic's round trip is hidden as well.
// All control words are left at zero when the kernel ends.
#include "common.cuh"

namespace fb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 8;               // k steps per chunk = rows per group
constexpr int kDepth = 5;                // ring slots per warp (kDepth - 1 chunks in flight)
constexpr int kStepK = 32;               // k covered by one warp step (4 lanes x 8 elements)
constexpr int kChunkK = kStepK * kUnroll;  // 256
constexpr int kRowPadBytes = 64;
constexpr int kCtlInts = 64;             // ctr[0..31], done = [32]
constexpr int kMaxSplit = 32;
constexpr int kSlotBytes = 8 * kChunkK * 2;                            // 8 rows x 512 bytes
constexpr int kRingBytes = kWarps * kDepth * kSlotBytes;               // 160 KB
constexpr int kFifoBytes = kWarps * 8 * 4;
constexpr size_t kMaxSmem = 232448 - 1024;                             // X slice + rings + fifos

struct SkinnyPlan {
  int S;            // K splits
  int kslice;       // elements per split (multiple of kChunkK)
  int ngroups;      // ceil(N / 8)
  size_t smem;      // dynamic shared bytes
  size_t off_partials, ws_bytes;
  int grid;
};

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// TO = output element type (T or float)
template <typename T, typename TO>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_skinny_kernel(const T* __restrict__ X, const T* __restrict__ W, TO* __restrict__ Y, int M, int N,
                       int K, int64_t ldx, int64_t ldw, int64_t ldy, int S, int kslice, int ngroups,
                       int accumulate, unsigned* __restrict__ ctl,
                       float* __restrict__ partials) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int s = blockIdx.x % S;
  const int kbeg = s * kslice;
  const int klen = max(0, min(K, kbeg + kslice) - kbeg);  // valid k in this slice (multiple of 8)
  const int pitch = kslice * (int)sizeof(T) + kRowPadBytes;

  const unsigned char* xs_lo = smem_raw + (size_t)g * pitch + (size_t)t * 8 * sizeof(T);
  const unsigned char* xs_hi = xs_lo + (size_t)8 * pitch;
  const int Npad = ngroups * 8;
  // this warp's ring of weight chunks and its queue of row groups in flight
  const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw)) + 16u * (uint32_t)pitch +
                        (uint32_t)(warp * kDepth) * kSlotBytes;
  volatile unsigned* fifo = reinterpret_cast<volatile unsigned*>(smem_raw + (size_t)16 * pitch + kRingBytes) + warp * 8;
  const int nchunks = (klen + kChunkK - 1) / kChunkK;

  // the queue: lane 0 requests an id early (the atomic's result is not touched until it is taken)
  unsigned requested = 0;
  auto request = [&]() {
    if (lane == 0) requested = atomicAdd(&ctl[s], 1u);
  };
  auto take = [&]() -> unsigned { return __shfl_sync(0xffffffffu, requested, 0); };

  if (nchunks > 0) {
    // ---- issue side: runs kDepth - 1 chunks ahead of the multiplication
    request();
    unsigned ng_issue = take(), pushed = 0;
    int c_issue = 0, slot_issue = 0;
    bool issue_live = ng_issue < (unsigned)ngroups;
    if (issue_live) {
      if (lane == 0) fifo[pushed & 7] = ng_issue;
      ++pushed;
    }
    auto issue_one = [&]() {
      if (issue_live) {
        const int k0 = c_issue * kChunkK + lane * 8;      // this lane's 16-byte piece
        const int bytes = k0 < klen ? 16 : 0;              // 0: the destination is zero-filled
        const T* src = W + kbeg + min(k0, klen - 8);
        const uint32_t dst = ring + (uint32_t)slot_issue * kSlotBytes;
        if (c_issue == nchunks - 1) request();  // answered while this chunk streams in
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {                // u = row within the group
          const int n_row = min((int)ng_issue * 8 + u, N - 1);
          cp_async16(dst + u * (kChunkK * 2) + (((lane ^ (u << 2)) & 31) << 4), src + (int64_t)n_row * ldw, bytes);
        }
        if (++c_issue == nchunks) {
          c_issue = 0;
          ng_issue = take();
          issue_live = ng_issue < (unsigned)ngroups;
          if (issue_live) {
            if (lane == 0) fifo[pushed & 7] = ng_issue;
            ++pushed;
          }
        }
      }
      cp_async_commit();  // also when nothing was issued: the group count stays in step
      slot_issue = slot_issue + 1 == kDepth ? 0 : slot_issue + 1;
    };
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) issue_one();

    // ---- stage this split's slice of X (rows >= M and k beyond the slice are zero) while the first
    // weight chunks are already on their way
    {
      const int vec_per_row = kslice / 8;
      for (int i = tid; i < 16 * vec_per_row; i += kThreads) {
        int r = i / vec_per_row, kv = (i % vec_per_row) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M && kv < klen) v = __ldg(reinterpret_cast<const uint4*>(X + (int64_t)r * ldx + kbeg + kv));
        *reinterpret_cast<uint4*>(smem_raw + (size_t)r * pitch + (size_t)kv * sizeof(T)) = v;
      }
    }
    __syncthreads();

    // ---- multiplication side
    unsigned popped = 0;
    int c = 0, slot = 0;
    float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
    while (popped < pushed) {
      issue_one();                 // refills the slot that was multiplied in the previous round
      cp_async_wait<kDepth - 1>();  // everything but the newest kDepth - 1 chunks has landed
      __syncwarp();
      const unsigned ng = fifo[popped & 7];
      const uint32_t base = ring + (uint32_t)slot * kSlotBytes + (uint32_t)g * (kChunkK * 2);
      const int k0 = c * kChunkK;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        size_t off = (size_t)(k0 + u * kStepK) * sizeof(T);
        uint4 xa = *reinterpret_cast<const uint4*>(xs_lo + off);
        uint4 xb = *reinterpret_cast<const uint4*>(xs_hi + off);
        const uint4 w = lds_v4(base + ((((u << 2) + t) ^ (g << 2)) << 4));
        mma16816<T>(acc0, xa.x, xb.x, xa.y, xb.y, w.x, w.y);
        mma16816<T>(acc1, xa.z, xb.z, xa.w, xb.w, w.z, w.w);
      }
      __syncwarp();  // every lane is done with the slot before it is refilled
      slot = slot + 1 == kDepth ? 0 : slot + 1;
      if (++c < nchunks) continue;
      c = 0;
      ++popped;

      // ---- the row group is complete
      float cc4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        cc4[i] = acc0[i] + acc1[i];
        acc0[i] = 0.f;
        acc1[i] = 0.f;
      }
      const int col = (int)ng * 8 + 2 * t;  // output columns col, col+1 ; rows g and g+8
      if (S > 1) {
        float* pp = partials + ((size_t)s * 16 + g) * Npad + col;
        __stcg(reinterpret_cast<float2*>(pp), make_float2(cc4[0], cc4[1]));
        __stcg(reinterpret_cast<float2*>(pp + (size_t)8 * Npad), make_float2(cc4[2], cc4[3]));
        continue;
      }
      {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          int r = g + 8 * h;
          if (r >= M) continue;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            int cc = col + jj;
            if (cc >= N) continue;
            TO* y = Y + (int64_t)r * ldy + cc;
            float v = cc4[2 * h + jj];
            if (accumulate) v += to_f32<TO>(*y);
            *y = from_f32<TO>(v);
          }
        }
      }
    }
    cp_async_wait<0>();
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the reduction grid may be scheduled

  // ---- leave the queue counters at zero for the next launch
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    unsigned d = atomicAdd(&ctl[32], 1u);
    if (d == gridDim.x - 1) {
      for (int i = 0; i < S; ++i) ctl[i] = 0;
      ctl[32] = 0;
      __threadfence();
    }
  }
}

// Y[r][n] = (accumulate ? Y[r][n] : 0) + sum over the splits, in split order, of partials[s][r][n]
template <typename TO>
__global__ void __launch_bounds__(256) skinny_reduce_kernel(const float* __restrict__ partials, int S, int Npad,
                                                            int M, int N, TO* __restrict__ Y, int64_t ldy,
                                                            int accumulate) {
  const int n = (blockIdx.x * 256 + threadIdx.x) * 2;
  const int r = blockIdx.y;
  // launched with programmatic stream serialization: the grid may be resident before the
  // streaming kernel has ended; its partial sums are visible after this wait
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (n >= N || r >= M) return;
  float2 acc = make_float2(0.f, 0.f);
  for (int ss = 0; ss < S; ++ss) {
    const float2 v = __ldcg(reinterpret_cast<const float2*>(partials + ((size_t)ss * 16 + r) * Npad + n));
    acc.x += v.x;
    acc.y += v.y;
  }
  TO* y = Y + (int64_t)r * ldy + n;
  if (accumulate) acc.x += to_f32<TO>(y[0]);
  y[0] = from_f32<TO>(acc.x);
  if (n + 1 < N) {
    if (accumulate) acc.y += to_f32<TO>(y[1]);
    y[1] = from_f32<TO>(acc.y);
  }
}

SkinnyPlan make_plan(const frisk_b200_gemm_desc& d, int num_sms) {
  SkinnyPlan p{};
  size_t es = dtype_size(d.dtype_ab);
  p.ngroups = (int)((d.N + 7) / 8);
  int S = 1;
  auto slice_of = [&](int s) { return (int)(((d.K + s - 1) / s + kChunkK - 1) / kChunkK * kChunkK); };
  auto smem_of = [&](int s) { return (size_t)16 * ((size_t)slice_of(s) * es + kRowPadBytes) + kRingBytes + kFifoBytes; };
  while (S < kMaxSplit && smem_of(S) > kMaxSmem) ++S;
  // enough warp-sized work items to keep every warp of the machine busy a few times over
  long want_items = (long)num_sms * kWarps * 4;
  // CTAs are bound to a split, so the splits should carry equal work: of the finer splits only those
  // whose slices cover K without a short last slice are taken
  auto even = [&](int s) { return (int64_t)slice_of(s) * (s - 1) < d.K && (int64_t)slice_of(s) * s - d.K < kChunkK; };
  for (int c = S + 1; c <= kMaxSplit && (long)p.ngroups * S < want_items && slice_of(c) >= 2 * kChunkK; ++c)
    if (even(c) && slice_of(c) < slice_of(S)) S = c;
  p.S = S;
  p.kslice = slice_of(S);
  p.smem = smem_of(S);
  p.grid = (num_sms / S) * S;
  if (p.grid < S) p.grid = S;
  p.off_partials = kCtlInts * sizeof(unsigned);  // queue counters, then the fp32 partials
  p.ws_bytes = p.off_partials + (S > 1 ? (size_t)S * 16 * p.ngroups * 8 * sizeof(float) : 0);
  return p;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, typename TO>
int launch_typed(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const SkinnyPlan& p, const void* A,
                 const void* B, void* C, void* ws, cudaStream_t s) {
  GemmDims g = resolve_dims(d);
  auto kern = gemm_skinny_kernel<T, TO>;
  // the opt-in is made once per device for the largest size any plan uses
  static PerDeviceOnce opt_in;
  int device = 0;
  FB_CUDA(ctx, cudaGetDevice(&device));
  if (opt_in(device, [&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem) == cudaSuccess ? 0 : 1;
      }))
    return FRISK_B200_E_CUDA;
  unsigned char* w = static_cast<unsigned char*>(ws);
  kern<<<p.grid, kThreads, p.smem, s>>>(static_cast<const T*>(A), static_cast<const T*>(B), static_cast<TO*>(C),
                                        (int)g.M, (int)g.N, (int)g.K, g.lda, g.ldb, g.ldc, p.S, p.kslice,
                                        p.ngroups, d.clear_accum ? 0 : 1, reinterpret_cast<unsigned*>(w),
                                        reinterpret_cast<float*>(w + p.off_partials));
  FB_CUDA(ctx, cudaGetLastError());
  if (p.S > 1) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.gridDim = dim3((unsigned)((p.ngroups * 8 / 2 + 255) / 256), (unsigned)g.M);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* parts = reinterpret_cast<const float*>(w + p.off_partials);
    int Sv = p.S, Npad = p.ngroups * 8, Mi = (int)g.M, Ni = (int)g.N, acc = d.clear_accum ? 0 : 1;
    TO* Yp = static_cast<TO*>(C);
    int64_t ldy = g.ldc;
    FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, skinny_reduce_kernel<TO>, parts, Sv, Npad, Mi, Ni, Yp, ldy, acc));
  }
  return 0;
}

}  // namespace

bool skinny_supported(const frisk_b200_gemm_desc& d) {
  if (d.dtype_ab != FRISK_B200_F16 && d.dtype_ab != FRISK_B200_BF16) return false;
  if (d.trans_a || !d.trans_b) return false;
  if (d.M < 1 || d.M > 16) return false;
  GemmDims g = resolve_dims(d);
  if (g.K % 8 || g.lda % 8 || g.ldb % 8) return false;
  if (g.N > (int64_t)INT32_MAX / 16 || g.K > INT32_MAX / 2) return false;
  // the K slice of X a CTA stages must fit shared memory with the deepest split there is
  // (K <= 65536 for 16-bit operands); deeper products go to the tcgen05 kernels
  if (make_plan(d, kNumSMsDefault).smem > kMaxSmem) return false;
  return true;
}

size_t skinny_workspace_bytes(const frisk_b200_gemm_desc& d) {
  return make_plan(d, kNumSMsDefault).ws_bytes;
}
size_t skinny_control_bytes(const frisk_b200_gemm_desc& d) { return make_plan(d, kNumSMsDefault).off_partials; }
uint64_t skinny_layout_signature(const frisk_b200_gemm_desc& d) {
  SkinnyPlan p = make_plan(d, kNumSMsDefault);
  return (static_cast<uint64_t>(p.ngroups) << 8) | static_cast<uint64_t>(p.S) | (1ull << 63);
}

// Also used by the fixed-capacity entry point, which passes its own scratch.
int launch_gemm_skinny(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                       void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!skinny_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  SkinnyPlan p = make_plan(d, kNumSMsDefault);
  if (!ws || ws_bytes < p.ws_bytes) return FRISK_B200_E_WORKSPACE;
  if (!aligned16(ws)) return FRISK_B200_E_ALIGN;
  bool out32 = d.dtype_c == FRISK_B200_F32;
  if (d.dtype_ab == FRISK_B200_F16)
    return out32 ? launch_typed<__half, float>(ctx, d, p, A, B, C, ws, s)
                 : launch_typed<__half, __half>(ctx, d, p, A, B, C, ws, s);
  return out32 ? launch_typed<__nv_bfloat16, float>(ctx, d, p, A, B, C, ws, s)
               : launch_typed<__nv_bfloat16, __nv_bfloat16>(ctx, d, p, A, B, C, ws, s);
}

}  // namespace fb

// ---------------------------------------------------------------------------------------
// Entry point that allocates nothing.
//
// Some users of this library are not allowed to allocate device memory at the moment they
// need a decode-shape GEMM: a serving process whose memory manager claimed all of HBM at
// start-up (a later cudaMalloc simply fails), or a latency-critical loop that cannot accept
// the device-wide synchronisation that cudaMalloc / cudaFree imply.  For them the split-K
// scratch of the skinny kernel lives in a fixed array in the library's device image.  It is
// part of the image, so every GPU that loads the library carries these bytes until the
// process exits; the size is therefore kept modest and larger problems are refused.
namespace fb {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: the 16 x 28672 x 8192 decode GEMM needs 7.0 MiB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address, so
// the address each device gave the array is looked up once (with that device current) and
// kept here.
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};

int static_scratch_for(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) return FRISK_B200_E_ARG;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return FRISK_B200_E_CUDA;
    g_static_ptr[device] = p;
  }
  *out = g_static_ptr[device];
  return 0;
}

}  // namespace
}  // namespace fb

extern "C" int frisk_b200_gemm_skinny_static(int device, const frisk_b200_gemm_desc* desc, const void* A,
                                             const void* B, void* C, void* stream) {
  using namespace fb;
  if (!desc || !A || !B || !C) return FRISK_B200_E_ARG;
  int rc = frisk_b200_gemm_validate(desc);
  if (rc) return rc;
  if (!skinny_supported(*desc)) return FRISK_B200_E_UNSUPPORTED;
  if (skinny_workspace_bytes(*desc) > kStaticScratchBytes) return FRISK_B200_E_TOO_LARGE;
  const GemmExtents ext = gemm_extents(*desc);
  if (ranges_overlap(C, ext.c, A, ext.a) || ranges_overlap(C, ext.c, B, ext.b)) return FRISK_B200_E_OVERLAP;
  DeviceGuard guard(device);  // the caller's current device is put back on return
  if (guard.error() != cudaSuccess) return FRISK_B200_E_CUDA;
  void* scratch = nullptr;
  if ((rc = static_scratch_for(device, &scratch))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call (possibly of another shape) left in it:
  // the queue counters at its start must be zero before the kernel runs.
  if (cudaMemsetAsync(scratch, 0, skinny_control_bytes(*desc), s) != cudaSuccess) return FRISK_B200_E_CUDA;
  return launch_gemm_skinny(nullptr, *desc, A, B, C, scratch, kStaticScratchBytes, s);
}
