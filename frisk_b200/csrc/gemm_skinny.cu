// Decode-shape ("skinny") GEMM on TMA + tcgen05: Y[M<=16, N] = X[M, K] . W[N, K]^T for fp16/bf16,
// fp32 accumulation.  Contract: `frisk.gemm` with trans_a=0, trans_b=1
// (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).  The weight matrix is read exactly once, so the
// kernel is bound by HBM bandwidth; the design is about keeping ~190 KB of weight loads in flight
// per SM with almost no instructions.
//
// * Roles are swapped with respect to the big GEMM: the WEIGHTS are the M operand of the MMA.  A
//   128-row x 64-k box of W (16 KB, one TMA instruction) and the matching 16 x 64 box of X (2 KB,
//   served by L2) make a k-block; a ring stage holds four of them, three stages = 192 KB of weights
//   in flight per SM; tcgen05.mma 128 x 16 x 16 accumulates Y^T for 128 output columns in 16
//   columns of tensor memory.
// * Work is cut stream-K fashion: the (128-row tile, group of four k-blocks) units are numbered
//   tile-major and CTA c takes the contiguous range [U*c/G, U*(c+1)/G), so every SM streams the same
//   number of bytes whatever N is (the N/8 shard of a multi-GPU run has 28 tiles for 148 SMs).  A
//   range is a sequence of segments (tile, k-group range).  A segment that covers a tile's whole K
//   is rounded and stored directly; otherwise the CTA leaves its fp32 partial in scratch and takes
//   the tile's ticket, and the contributor that draws the last ticket adds all partials of the tile
//   in contributor order (deterministic) and stores.  Nobody waits for another CTA.
// * warp 0: TMA producer; warp 1: MMA issuer; warps 2-5: epilogue (thread = output column).
// Every mbarrier wait is bounded (ptx.cuh); no TMA load uses cluster multicast.
#include "common.cuh"
#include "ptx.cuh"

namespace fb {
namespace {

constexpr int TN = 128;        // weight rows (output columns) per tile = MMA M
constexpr int TM = 16;         // activation rows = MMA N
constexpr int BK = 64;         // one 128-byte swizzle span
constexpr int UMMA_K = 16;
constexpr int KBS = 4;         // k-blocks per ring stage (fewer, larger stages stream faster than 12 x 18 KB)
constexpr int kStages = 3;
constexpr int kThreads = 192;
constexpr int kWBytes = TN * BK * 2;   // 16 KB
constexpr int kXBytes = TM * BK * 2;   // 2 KB
constexpr int kStageBytes = KBS * (kWBytes + kXBytes);
constexpr int kBarOffset = kStages * kStageBytes;
constexpr int kSmemTotal = kBarOffset + 512 + 1024;
constexpr int kPartialFloats = TM * TN;  // one fp32 partial: [16][128]

// Unit range of CTA c: [v[c], v[c + 1]).  Made on the host (the device has no 64-bit divider, and the
// epilogue looks several of these up on the path that ends the kernel) and passed by value.
struct RangeStarts {
  int v[kNumSMsDefault + 1];
};

// The segments (tile, k-group range) of a CTA's unit range, in the order they are processed: the
// partial segment of the LAST tile first, then the partial segment of the FIRST tile, then the whole
// tiles.  A tile shared with a neighbouring CTA is that neighbour's first (or second) segment too, so
// both halves are finished early in both CTAs' lives and their summation hides behind the streaming
// of the whole tiles; the last thing a CTA does is then a plain store.
struct Seg {
  int tile, kg0, kg1;
};
struct SegList {
  int u0, u1;
  int num_kg, first_tile, last_tile, n;
  bool head_p, tail_p;
  __device__ SegList(int a, int b, int nk) : u0(a), u1(b), num_kg(nk) {
    first_tile = u0 / nk;
    last_tile = (u1 - 1) / nk;
    head_p = first_tile != last_tile && (u0 % nk) != 0;
    tail_p = first_tile != last_tile && (u1 % nk) != 0;
    n = last_tile - first_tile + 1;
  }
  __device__ Seg get(int i) const {
    if (first_tile == last_tile)
      return Seg{first_tile, u0 - first_tile * num_kg, u1 - first_tile * num_kg};
    if (tail_p) {
      if (i == 0) return Seg{last_tile, 0, u1 - last_tile * num_kg};
      --i;
    }
    if (head_p) {
      if (i == 0) return Seg{first_tile, u0 - first_tile * num_kg, num_kg};
      --i;
    }
    return Seg{first_tile + (head_p ? 1 : 0) + i, 0, num_kg};
  }
};

template <typename TO>
__device__ __forceinline__ float load_as_f32(const TO* p);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_f32<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename TO>
__device__ __forceinline__ TO round_to(float v);
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half round_to<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 round_to<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename TO, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                           TO* __restrict__ Y, int M, int N, int num_kg, int64_t ldy, int accumulate,
                           const __grid_constant__ RangeStarts starts, float ctas_per_unit,
                           unsigned* __restrict__ tickets, float* __restrict__ partials,
                           unsigned* __restrict__ status) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;  // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint64_t* epi_bar = acc_empty + 2;         // [1] the four epilogue warps among themselves
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_word = tmem_slot + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int u_begin = starts.v[cta], u_end = starts.v[cta + 1];

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    mbar_init(epi_bar, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: this set-up may overlap the previous kernel of the
  // stream; nothing above touches global memory, everything below comes after that kernel's end.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const SegList segs(u_begin, u_end, num_kg);
      bool ok = true;
      for (int si = 0; si < segs.n && ok; ++si) {
        const Seg sg = segs.get(si);
        const int tile = sg.tile;
        for (int kg = sg.kg0; kg < sg.kg1; ++kg) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          unsigned char* sw = smem + stage * kStageBytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          // k-blocks past the end of K are zero-filled by TMA and add nothing
#pragma unroll
          for (int j = 0; j < KBS; ++j)
            tma_load_2d(sw + j * kWBytes, &tmap_w, &full_bar[stage], (kg * KBS + j) * BK, tile * TN);
#pragma unroll
          for (int j = 0; j < KBS; ++j)
            tma_load_2d(sw + KBS * kWBytes + j * kXBytes, &tmap_x, &full_bar[stage], (kg * KBS + j) * BK, 0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(TN, TM, BF16, false, false);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const SegList segs(u_begin, u_end, num_kg);
      for (int si = 0; si < segs.n && ok; ++si) {
        const Seg sg = segs.get(si);
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * TM;
        bool first = true;
        for (int kg = sg.kg0; kg < sg.kg1; ++kg) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sw = smem_u32(smem + stage * kStageBytes);
          const uint32_t sx = sw + KBS * kWBytes;
#pragma unroll
          for (int j = 0; j < KBS; ++j) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              umma_f16_ss(d_tmem, umma_desc_kmajor_sw128(sw + j * kWBytes + k * (UMMA_K * 2)),
                          umma_desc_kmajor_sw128(sx + j * kXBytes + k * (UMMA_K * 2)), idesc,
                          (first && j == 0 && k == 0) ? 0u : 1u);
            }
          }
          first = false;
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (thread = output column)
    const int quad = warp & 3;
    const int col_local = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0, epi_phase = 0;
    bool epi_ok = true;
    auto epi_sync = [&]() {
      mbar_arrive(epi_bar);
      if (epi_ok) epi_ok = mbar_wait(epi_bar, epi_phase, abort_flag, status, ST_TIMEOUT_MISC);
      epi_phase ^= 1;
    };
    auto store_column = [&](int tile, const float (&v)[TM]) {
      const int col = tile * TN + col_local;
      if (col >= N) return;
#pragma unroll
      for (int m = 0; m < TM; ++m) {
        if (m < M) {
          TO* y = Y + (int64_t)m * ldy + col;
          float r = v[m];
          if (accumulate) r += load_as_f32<TO>(y);
          *y = round_to<TO>(r);
        }
      }
    };
    const SegList segs(u_begin, u_end, num_kg);
    for (int si = 0; si < segs.n; ++si) {
      const Seg sg = segs.get(si);
      const int tile = sg.tile;
      const int t0 = tile * num_kg, t1 = t0 + num_kg;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, status, ST_TIMEOUT_ACC_FULL)) break;
      tc_fence_after_sync();
      uint32_t raw[TM];
      tmem_ld_32x32b_x16(tmem_base + acc * TM + (static_cast<uint32_t>(quad * 32) << 16), raw);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);  // the values are in registers: the accumulator is free
      float v[TM];
#pragma unroll
      for (int m = 0; m < TM; ++m) v[m] = __uint_as_float(raw[m]);
      if (sg.kg0 == 0 && sg.kg1 == num_kg) {
        store_column(tile, v);  // this CTA had the tile's whole K
      } else {
        // Contributors of this tile: the CTAs whose ranges meet [t0, t1), first to last.
        // (a float estimate, corrected against the table)
        int c_first = min(G - 1, (int)((float)t0 * ctas_per_unit)), c_last = min(G - 1, (int)((float)(t1 - 1) * ctas_per_unit));
        while (c_first + 1 < G && starts.v[c_first + 1] <= t0) ++c_first;
        while (c_first > 0 && starts.v[c_first] > t0) --c_first;
        while (c_last + 1 < G && starts.v[c_last + 1] < t1) ++c_last;
        while (c_last > 0 && starts.v[c_last] >= t1) --c_last;
        const int n_contrib = c_last - c_first + 1;
        // a CTA leaves at most two partials: slot 0 for the tile its range begins in, slot 1 for the tile it ends in
        const int my_slot = tile == segs.first_tile ? 0 : 1;
        float* mine = partials + ((size_t)cta * 2 + my_slot) * kPartialFloats + col_local;
#pragma unroll
        for (int m = 0; m < TM; ++m) __stcg(mine + m * TN, v[m]);
        epi_sync();  // all 128 columns of the partial are written ...
        if (warp == 2 && lane == 0) {
          __threadfence();  // ... and visible device-wide before the ticket is taken
          epi_word[si & 1] = atomicAdd(&tickets[tile], 1u);
        }
        epi_sync();
        const bool last = epi_ok && (epi_word[si & 1] == (unsigned)(n_contrib - 1));
        if (last) {
          __threadfence();
          float sum[TM];
#pragma unroll
          for (int m = 0; m < TM; ++m) sum[m] = 0.f;
          // contributor order, four contributors' loads in flight at a time (the additions stay in order)
          for (int c0 = c_first; c0 <= c_last; c0 += 4) {
            float part[4][TM];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int c = min(c0 + j, c_last);
              const int first_tile = starts.v[c] / num_kg;
              const float* p = partials + ((size_t)c * 2 + (first_tile == tile ? 0 : 1)) * kPartialFloats + col_local;
#pragma unroll
              for (int m = 0; m < TM; ++m) part[j][m] = __ldcg(p + m * TN);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (c0 + j <= c_last) {
#pragma unroll
                for (int m = 0; m < TM; ++m) sum[m] += part[j][m];
              }
          }
          store_column(tile, sum);
          if (warp == 2 && lane == 0) tickets[tile] = 0;  // clean for the next launch
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 32);
  }
}

struct SkinnyPlan {
  int tiles, num_kg, grid;
  long long units;  // < 2^31 (checked by skinny_supported)
  size_t ticket_bytes, ws_bytes;
};
SkinnyPlan make_plan(const frisk_b200_gemm_desc& d, int num_sms) {
  SkinnyPlan p{};
  p.tiles = (int)((d.N + TN - 1) / TN);
  p.num_kg = (int)((d.K + KBS * BK - 1) / (KBS * BK));
  p.units = (long long)p.tiles * p.num_kg;
  p.grid = (int)std::min<long long>(num_sms, p.units);
  p.ticket_bytes = ((size_t)p.tiles * sizeof(unsigned) + 255) / 256 * 256;
  // every CTA of the largest grid may leave two partials
  p.ws_bytes = p.ticket_bytes + (size_t)kNumSMsDefault * 2 * kPartialFloats * sizeof(float);
  return p;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TO, bool BF16>
int launch_typed(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                 void* ws, cudaStream_t s, int device, int num_sms, unsigned* status) {
  GemmDims g = resolve_dims(d);
  SkinnyPlan p = make_plan(d, std::min(num_sms, kNumSMsDefault));
  CUtensorMap tw, tx;
  int rc = encode_tmap_2d(ctx, &tw, d.dtype_ab, B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb * 2, BK, TN, true);
  if (!rc) rc = encode_tmap_2d(ctx, &tx, d.dtype_ab, A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda * 2, BK, TM, true);
  if (rc) {
    if (ctx) ctx->last_cuda = rc;
    return FRISK_B200_E_CUDA;
  }
  auto kern = gemm_skinny_kernel<TO, BF16>;
  static PerDeviceOnce opt_in;
  if (opt_in(device, [&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal) == cudaSuccess ? 0 : 1;
      }))
    return FRISK_B200_E_CUDA;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3((unsigned)p.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemTotal;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  unsigned char* w = static_cast<unsigned char*>(ws);
  TO* Yp = static_cast<TO*>(C);
  int Mi = (int)g.M, Ni = (int)g.N, nkb = p.num_kg, acc = d.clear_accum ? 0 : 1;
  int64_t ldy = g.ldc;
  RangeStarts starts{};
  for (int c = 0; c <= p.grid; ++c) starts.v[c] = (int)(p.units * c / p.grid);
  float ctas_per_unit = (float)p.grid / (float)p.units;
  unsigned* tickets = reinterpret_cast<unsigned*>(w);
  float* partials = reinterpret_cast<float*>(w + p.ticket_bytes);
  FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, tw, tx, Yp, Mi, Ni, nkb, ldy, acc, starts, ctas_per_unit, tickets, partials, status));
  return 0;
}

}  // namespace

bool skinny_supported(const frisk_b200_gemm_desc& d) {
  if (d.dtype_ab != FRISK_B200_F16 && d.dtype_ab != FRISK_B200_BF16) return false;
  if (d.trans_a || !d.trans_b) return false;
  if (d.M < 1 || d.M > TM) return false;
  GemmDims g = resolve_dims(d);
  if (g.lda % 8 || g.ldb % 8) return false;  // TMA: 16-byte pitches
  if (g.N > INT32_MAX - TN || g.K > INT32_MAX - KBS * BK) return false;
  if (((g.N + TN - 1) / TN) * ((g.K + KBS * BK - 1) / (KBS * BK)) > INT32_MAX / 2) return false;  // unit count fits an int
  return true;
}
size_t skinny_workspace_bytes(const frisk_b200_gemm_desc& d) { return make_plan(d, kNumSMsDefault).ws_bytes; }
size_t skinny_control_bytes(const frisk_b200_gemm_desc& d) { return make_plan(d, kNumSMsDefault).ticket_bytes; }

// `ctx` may be NULL (the entry that allocates nothing has no context): `status` then names the
// device word a wait that ran out is recorded in.
int launch_gemm_skinny(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                           void* ws, size_t ws_bytes, cudaStream_t s, unsigned* status) {
  if (!skinny_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  if (!ws || ws_bytes < skinny_workspace_bytes(d)) return FRISK_B200_E_WORKSPACE;
  if (!aligned16(ws)) return FRISK_B200_E_ALIGN;
  int device = 0;
  FB_CUDA(ctx, cudaGetDevice(&device));
  int num_sms = ctx ? ctx->num_sms : kNumSMsDefault;
  if (!ctx) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && n > 0) num_sms = n;
  }
  if (!status) status = ctx ? ctx->d_status : nullptr;
  if (!status) return FRISK_B200_E_ARG;
  const bool out32 = d.dtype_c == FRISK_B200_F32;
  if (d.dtype_ab == FRISK_B200_F16)
    return out32 ? launch_typed<float, false>(ctx, d, A, B, C, ws, s, device, num_sms, status)
                 : launch_typed<__half, false>(ctx, d, A, B, C, ws, s, device, num_sms, status);
  return out32 ? launch_typed<float, true>(ctx, d, A, B, C, ws, s, device, num_sms, status)
               : launch_typed<__nv_bfloat16, true>(ctx, d, A, B, C, ws, s, device, num_sms, status);
}

}  // namespace fb

// ---------------------------------------------------------------------------------------
// Entry point that allocates nothing.
//
// Some users of this library are not allowed to allocate device memory at the moment they
// need a decode-shape GEMM: a serving process whose memory manager claimed all of HBM at
// start-up (a later cudaMalloc simply fails), or a latency-critical loop that cannot accept
// the device-wide synchronisation that cudaMalloc / cudaFree imply.  For them the stream-K
// scratch of the skinny kernel lives in a fixed array in the library's device image.  It is
// part of the image, so every GPU that loads the library carries these bytes until the
// process exits; the size is therefore kept modest and larger problems are refused.
namespace fb {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: the 16 x 28672 x 8192 decode GEMM needs 2.3 MiB
constexpr size_t kStaticStatusBytes = 256;        // the device status word of these calls sits in front of the scratch

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes + kStaticStatusBytes];

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
  void* base = nullptr;
  if ((rc = static_scratch_for(device, &base))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned char* scratch = static_cast<unsigned char*>(base) + kStaticStatusBytes;
  // The array keeps whatever the previous call (possibly of another shape) left in it:
  // the tickets at its start must be zero before the kernel runs.
  if (cudaMemsetAsync(scratch, 0, skinny_control_bytes(*desc), s) != cudaSuccess) return FRISK_B200_E_CUDA;
  return launch_gemm_skinny(nullptr, *desc, A, B, C, scratch, kStaticScratchBytes, s, static_cast<unsigned*>(base));
}
