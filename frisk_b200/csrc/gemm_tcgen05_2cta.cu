// fp16 / bf16 GEMM on tcgen05 with CTA PAIRS (cta_group::2): a cluster of two CTAs on
// neighbouring SMs computes one 256 x 256 output tile.  Same contract as gemm_tcgen05.cu
// (`frisk.gemm`, lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).
//
// Why pairs: with one CTA per tile every tcgen05.mma 128x256x16 reads 12 KB of operands from
// shared memory while TMA writes the next stages into the same shared memory, and the
// two together exceed the 128 B/clk a shared memory delivers.  In a pair each CTA stages
// its own 128 rows of A and only HALF of the B tile (128 of the 256 columns); the MMA,
// issued by the leader CTA for both, reads each CTA's operands from that CTA's shared
// memory.  Per CTA that is 8 KB per MMA and 32 KB per k-block, so six ring stages fit
// where four did, and the accumulator of each CTA (its 128 rows x 256 columns) lives in
// that CTA's tensor memory.
//
// Nothing is multicast by TMA: every CTA loads exactly what it alone needs
// (cp.async.bulk.tensor with .cta_group::2 only so that the peer's copies can signal the
// leader's mbarrier).  tcgen05.commit multicasts barrier ARRIVALS to both CTAs.
//
//   warp 0    TMA producer (both CTAs)         warp 1   MMA issuer (leader CTA only)
//   warps 2-5 epilogue (both CTAs, own rows)
#include <cstdlib>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace fb {
namespace {
using namespace gemm_detail;

constexpr int BMC = 128;      // rows per CTA
constexpr int BM2 = 256;      // rows per pair
constexpr int BN2 = 256;      // columns per pair
constexpr int BNC = 128;      // B columns staged per CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kStages2 = 6;
constexpr int kThreads2 = 192;

struct Smem2 {
  static constexpr int kABytes = BMC * BK * 2;
  static constexpr int kBBytes = BNC * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages2 * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

// ---- cluster / cta_group::2 primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a shared-memory object of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is signalled on an mbarrier given as a shared::cluster address
// (it may live in the peer CTA); the destination is this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at the same shared-memory offset in every CTA of `mask` once all MMAs
// issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

template <typename TO, bool BF16, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads2, 1)
    gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             TO* __restrict__ C, int M, int N, int K, int64_t ldc, int accumulate, int vec_c,
                             unsigned* __restrict__ status) {
  using L = Smem2;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages2;
  uint64_t* acc_full = empty_bar + kStages2;  // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2] (the leader's is the one that is used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + BM2 - 1) / BM2, tiles_n = (N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages2; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);  // 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything crosses over
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        const int m0 = tc.m * BM2 + (int)rank * BMC;   // this CTA's rows of A (and of C)
        const int n0 = tc.n * BN2 + (int)rank * BNC;   // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * L::kStageBytes;
          unsigned char* sb = sa + L::kABytes;
          // the leader's barrier collects the bytes of both CTAs
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::kStageBytes);
          const uint32_t bar = mapa_u32(&full_bar[stage], 0);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BMC / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &tmap_a, bar, m0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BNC / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &tmap_b, bar, n0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          }
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BM2, BN2, BF16, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN2;
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
            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);  // both CTAs may refill this stage
          if (++stage == kStages2) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[acc], 3);  // both CTAs' epilogues may read their accumulator halves
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_acc_empty0 = mapa_u32(&acc_empty[0], 0), leader_acc_empty1 = mapa_u32(&acc_empty[1], 0);
    for (int t = pair; t < num_tiles; t += num_pairs) {
      TileCoord tc = tile_coord(t, tiles_m, tiles_n);
      const int m0 = tc.m * BM2 + (int)rank * BMC, n0 = tc.n * BN2;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, status, ST_TIMEOUT_ACC_FULL)) break;
      tc_fence_after_sync();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN2 + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN2 / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(taddr + c * 32, v);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N)
          store_row_chunk<TO>(C + (int64_t)row * ldc + col, v, min(32, N - col), vec_c != 0, accumulate != 0);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? leader_acc_empty1 : leader_acc_empty0);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's shared memory and barriers stay valid until both are done
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TO, bool BF16, bool A_MN, bool B_MN>
int launch_cfg2(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                cudaStream_t s) {
  GemmDims g = resolve_dims(d);
  CUtensorMap ta, tb;
  int rc;
  if (A_MN)
    rc = encode_tmap_2d(&ta, d.dtype_ab, A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(&ta, d.dtype_ab, A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda * 2, BK, BMC, true);
  if (rc) { ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }
  if (B_MN)
    rc = encode_tmap_2d(&tb, d.dtype_ab, B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(&tb, d.dtype_ab, B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb * 2, BK, BNC, true);
  if (rc) { ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }

  auto kern = gemm_tcgen05_2cta_kernel<TO, BF16, A_MN, B_MN>;
  FB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2::kTotal));
  int tiles = (int)(((g.M + BM2 - 1) / BM2) * ((g.N + BN2 - 1) / BN2));

  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads2);
  cfg.dynamicSmemBytes = Smem2::kTotal;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(2 * (ctx->num_sms / 2));
  int max_clusters = 0;
  FB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
  if (max_clusters < 1) return FRISK_B200_E_UNSUPPORTED;
  int pairs = tiles < max_clusters ? tiles : max_clusters;
  cfg.gridDim = dim3(2 * pairs);
  int vec_c = aligned16(C) && (g.ldc * sizeof(TO)) % 16 == 0;
  TO* Cp = static_cast<TO*>(C);
  int Mi = (int)g.M, Ni = (int)g.N, Ki = (int)g.K, acc = d.clear_accum ? 0 : 1;
  int64_t ldc = g.ldc;
  unsigned* st = ctx->d_status;
  FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, ta, tb, Cp, Mi, Ni, Ki, ldc, acc, vec_c, st));
  return 0;
}

template <typename TO, bool BF16>
int launch_major2(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                  cudaStream_t s) {
  bool a_mn = d.trans_a != 0, b_mn = d.trans_b == 0;
  if (a_mn) {
    if (b_mn) return launch_cfg2<TO, BF16, true, true>(ctx, d, A, B, C, s);
    return launch_cfg2<TO, BF16, true, false>(ctx, d, A, B, C, s);
  }
  if (b_mn) return launch_cfg2<TO, BF16, false, true>(ctx, d, A, B, C, s);
  return launch_cfg2<TO, BF16, false, false>(ctx, d, A, B, C, s);
}

}  // namespace

// The pair kernel pays when there are enough 256 x 256 tiles to fill the machine's CTA pairs.
bool tcgen05_2cta_preferred(const frisk_b200_gemm_desc& d) {
  if (const char* e = getenv("FRISK_B200_GEMM_PAIR")) return e[0] == '1';
  const int64_t tiles = ((d.M + BM2 - 1) / BM2) * ((d.N + BN2 - 1) / BN2);
  return tiles >= kNumSMsDefault / 2;
}

int launch_gemm_tcgen05_2cta(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                             void* C, cudaStream_t s) {
  if (!tcgen05_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  const bool bf = d.dtype_ab == FRISK_B200_BF16;
  if (d.dtype_c == FRISK_B200_F32)
    return bf ? launch_major2<float, true>(ctx, d, A, B, C, s) : launch_major2<float, false>(ctx, d, A, B, C, s);
  if (bf) return launch_major2<__nv_bfloat16, true>(ctx, d, A, B, C, s);
  return launch_major2<__half, false>(ctx, d, A, B, C, s);
}

}  // namespace fb
