// fp16 / bf16 GEMM on the 5th-generation tensor cores (tcgen05), fp32 accumulation in
// tensor memory.  Contract: `frisk.gemm` with f16/bf16 operands and a C of the same type or
// f32 (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426,
// lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:26-44).
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0    TMA producer: A and B tiles -> 4-stage shared-memory ring (full/empty mbarriers)
//   warp 1    MMA issuer:   one thread issues tcgen05.mma (128 x BN x 16) per k16 slice,
//                           tcgen05.commit releases the stage / publishes the accumulator
//   warps 2-5 epilogue:     tcgen05.ld of the finished accumulator, conversion, global stores
// Two accumulators (2 x BN TMEM columns) let the epilogue of tile i overlap the main loop of
// tile i+1.
//
// Shared-memory operand images are the canonical 128-byte-swizzle layouts (rows of 64
// 16-bit elements, 1024-byte aligned stages): K-major for an operand that is contiguous
// along K in global memory, MN-major otherwise.  These are the images Frisk's layout
// inference proposes for 16-bit MMA operands
// (lib/Dialect/Frisk/Target/SM90/SM90GemmConstraints.cpp:121-138); TMA writes them directly.
// No TMA load uses cluster multicast.
#include <type_traits>

#include "common.cuh"

#include "gemm_common.cuh"
#include "ptx.cuh"

namespace fb {
namespace {
using namespace gemm_detail;

constexpr int BM = 128;
constexpr int BK = 64;       // one 128-byte swizzle span of 16-bit elements
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kThreads = 192;

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // barriers + alignment slack
  // TMA-store epilogue only: two [32 rows][128 bytes] output boxes per epilogue warp, 1024-byte aligned
  static constexpr int kOutOffset = kBarOffset + 1024;
  static constexpr int kOutWarpBytes = 2 * 32 * 128;
  static constexpr int kTotalOut = kOutOffset + 4 * kOutWarpBytes + 1024;
  static_assert(kTotalOut <= 232448, "the output boxes must fit next to the operand ring");
};

// Work items: the first n_full items are whole 128xBN tiles; the tiles that would form a
// partial last wave are cut into two 128x(BN/2) items each, so that the last wave takes half
// as long (see the host side for when this pays).
struct Item {
  int m0, n0, bn;
};
template <int BN>
__device__ __forceinline__ Item get_item(int idx, int n_full, int tiles_m, int tiles_n) {
  int t = idx, half = -1;
  if (idx >= n_full) {
    t = n_full + ((idx - n_full) >> 1);
    half = (idx - n_full) & 1;
  }
  TileCoord tc = tile_coord(t, tiles_m, tiles_n);
  Item it{tc.m * BM, tc.n * BN, BN};
  if (half >= 0) {
    it.n0 += half * (BN / 2);
    it.bn = BN / 2;
  }
  return it;
}

// A_MN / B_MN: the operand is contiguous along M / N in global memory (MN-major image).
// TMA_OUT: an overwriting store of an aligned C leaves through shared-memory boxes and TMA stores.
template <typename TO, int BN, bool BF16, bool A_MN, bool B_MN, bool TMA_OUT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_c, TO* __restrict__ C, int M, int N, int K, int64_t ldc, int accumulate, int vec_c,
                        int n_full, int n_items, unsigned* __restrict__ status) {
  using L = SmemLayout<BN>;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (TMA_OUT) tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: the set-up above may run while the kernel in front of
  // this one drains; nothing touches global memory before that kernel is complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_items && ok; t += gridDim.x) {
        const Item it = get_item<BN>(t, n_full, tiles_m, tiles_n);
        const int m0 = it.m0, n0 = it.n0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * L::kStageBytes;
          unsigned char* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kABytes + it.bn * (BK * 2));
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &full_bar[stage], m0 + j * 64, k0);
          } else {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          }
          if (B_MN) {
            for (int j = 0; j < it.bn / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &full_bar[stage], n0 + j * 64, k0);
          } else {
            // boxes of 128 rows: stacked 8-row groups, the same image as one taller box
            for (int j = 0; j < it.bn / 128; ++j)
              tma_load_2d(sb + j * (128 * BK * 2), &tmap_b, &full_bar[stage], k0, n0 + j * 128);
          }
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
      constexpr uint32_t idesc_full = umma_idesc_f16(BM, BN, BF16, A_MN, B_MN);
      constexpr uint32_t idesc_half = umma_idesc_f16(BM, BN / 2, BF16, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_items && ok; t += gridDim.x) {
        const uint32_t idesc = (t >= n_full) ? idesc_half : idesc_full;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = A_MN ? umma_desc_mnmajor_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                               : umma_desc_kmajor_sw128(sa + k * (UMMA_K * 2));
            uint64_t db = B_MN ? umma_desc_mnmajor_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                               : umma_desc_kmajor_sw128(sb + k * (UMMA_K * 2));
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are this warp's
    int box_sel = 0;            // which of the warp's two output boxes the next TMA store uses
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < n_items; t += gridDim.x) {
      const Item it = get_item<BN>(t, n_full, tiles_m, tiles_n);
      const int m0 = it.m0, n0 = it.n0;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, status, ST_TIMEOUT_ACC_FULL)) break;
      tc_fence_after_sync();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      if (TMA_OUT) {
        // a lane holds 128 bytes of ONE row; the warp writes its 32 rows as a 128-byte-swizzle box and one lane
        // hands the box to the TMA unit, which writes whole lines and clips at the edges of C
        constexpr int kUnitCols = 128 / (int)sizeof(TO);
        unsigned char* boxes = smem + L::kOutOffset + quad * L::kOutWarpBytes;
#pragma unroll 1
        for (int u = 0; u < it.bn / kUnitCols; ++u) {
          const int c0 = n0 + u * kUnitCols, r0 = m0 + quad * 32;
          if (c0 >= N || r0 >= M) break;  // wholly outside C (warp-uniform)
          uint32_t w[32];
          if (sizeof(TO) == 4) {
            tmem_ld_32x32b_x32(taddr + u * 32, w);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              uint32_t v[32];
              tmem_ld_32x32b_x32(taddr + u * 64 + hh * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                w[hh * 16 + i] = pack_out<TO>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
          }
          if (lane == 0) tma_store_wait_read<1>();  // the store before the last one used this box: it has been read
          __syncwarp();
          unsigned char* box = boxes + box_sel * (32 * 128);
          box_sel ^= 1;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_c, box, c0, r0);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < it.bn / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (row < M && col < N)
            store_row_chunk<TO>(C + (int64_t)row * ldc + col, v, min(32, N - col), vec_c != 0, accumulate != 0);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (TMA_OUT && lane == 0) tma_store_wait<0>();  // the boxes are read and written out before the CTA leaves
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // a wait ran out somewhere: give copies that are still in flight time to land
    unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TO, int BN, bool BF16, bool A_MN, bool B_MN>
int launch_cfg(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
               cudaStream_t s) {
  GemmDims g = resolve_dims(d);
  CUtensorMap ta, tb;
  int rc;
  // A: K-major -> dims {K, M}, box {64, 128};  MN-major (stored [K,M]) -> dims {M, K}, box {64, 64}
  if (A_MN)
    rc = encode_tmap_2d(ctx, &ta, d.dtype_ab, A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(ctx, &ta, d.dtype_ab, A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda * 2, BK, BM, true);
  if (rc) { if (ctx) ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }
  if (B_MN)
    rc = encode_tmap_2d(ctx, &tb, d.dtype_ab, B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(ctx, &tb, d.dtype_ab, B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb * 2, BK, 128, true);
  if (rc) { if (ctx) ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }

  // an overwriting store of a C whose base and row pitch are 16-byte aligned goes out through the TMA unit
  const bool tma_out = d.clear_accum && aligned16(C) && (g.ldc * sizeof(TO)) % 16 == 0;
  CUtensorMap tc = ta;  // unused otherwise
  if (tma_out) {
    const int out_dtype = sizeof(TO) == 4 ? FRISK_B200_F32 : (std::is_same<TO, __half>::value ? FRISK_B200_F16 : FRISK_B200_BF16);
    rc = encode_tmap_2d(ctx, &tc, out_dtype, C, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldc * sizeof(TO),
                        128 / sizeof(TO), 32, true);
    if (rc) { if (ctx) ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }
  }
  using L = SmemLayout<BN>;
  int tiles = (int)(((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN));
  int grid = tiles < ctx->num_sms ? tiles : ctx->num_sms;
  // A partial last wave of at most grid/2 tiles runs as twice as many half-width items: the
  // wave then costs half a tile time instead of a whole one.
  int rem = tiles % grid;
  int n_full = tiles, n_items = tiles;
  if (tiles > grid && rem > 0 && 2 * rem <= grid) {
    n_full = tiles - rem;
    n_items = n_full + 2 * rem;
  }
  int vec_c = aligned16(C) && (g.ldc * sizeof(TO)) % 16 == 0;
  auto launch = [&](auto kern, int smem_bytes, PerDeviceOnce& opt_in) -> int {
    if (opt_in(ctx->device, [&] {
          return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) == cudaSuccess ? 0 : 1;
        }))
      return FRISK_B200_E_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits (griddepcontrol.wait) itself
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TO* Cp = static_cast<TO*>(C);
    int Mi = (int)g.M, Ni = (int)g.N, Ki = (int)g.K, acc = d.clear_accum ? 0 : 1;
    int64_t ldc = g.ldc;
    unsigned* st = ctx->d_status;
    FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, Cp, Mi, Ni, Ki, ldc, acc, vec_c, n_full, n_items, st));
    return 0;
  };
  static PerDeviceOnce opt_in_plain, opt_in_tma;  // one pair per instantiation
  if (tma_out) return launch(gemm_tcgen05_kernel<TO, BN, BF16, A_MN, B_MN, true>, L::kTotalOut, opt_in_tma);
  return launch(gemm_tcgen05_kernel<TO, BN, BF16, A_MN, B_MN, false>, L::kTotal, opt_in_plain);
}

template <typename TO, int BN, bool BF16>
int launch_major(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                 cudaStream_t s) {
  bool a_mn = d.trans_a != 0;   // A stored [K,M]
  bool b_mn = d.trans_b == 0;   // B stored [K,N]
  if (a_mn) {
    if (b_mn) return launch_cfg<TO, BN, BF16, true, true>(ctx, d, A, B, C, s);
    return launch_cfg<TO, BN, BF16, true, false>(ctx, d, A, B, C, s);
  }
  if (b_mn) return launch_cfg<TO, BN, BF16, false, true>(ctx, d, A, B, C, s);
  return launch_cfg<TO, BN, BF16, false, false>(ctx, d, A, B, C, s);
}

}  // namespace

bool tcgen05_supported(const frisk_b200_gemm_desc& d) {
  if (d.dtype_ab != FRISK_B200_F16 && d.dtype_ab != FRISK_B200_BF16) return false;
  GemmDims g = resolve_dims(d);
  // TMA: 16-byte pitches; 32-bit coordinates
  if (g.lda % 8 || g.ldb % 8) return false;
  if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return false;
  return true;
}

int launch_gemm_tcgen05(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                        void* C, cudaStream_t s) {
  if (!tcgen05_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  const bool bf = d.dtype_ab == FRISK_B200_BF16;
  if (d.dtype_c == FRISK_B200_F32)
    return bf ? launch_major<float, 256, true>(ctx, d, A, B, C, s) : launch_major<float, 256, false>(ctx, d, A, B, C, s);
  if (bf) return launch_major<__nv_bfloat16, 256, true>(ctx, d, A, B, C, s);
  return launch_major<__half, 256, false>(ctx, d, A, B, C, s);
}

}  // namespace fb
