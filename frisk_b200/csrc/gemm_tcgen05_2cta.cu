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

#include <type_traits>

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
constexpr size_t kTicketBytes = 1024;
constexpr int kMinKbAllHalved = 16;  // k-blocks a product needs before halving every tile's K pays for the fp32 hand-over
constexpr int kPairsAssumed = kNumSMsDefault / 2;  // CTA pairs the tail plan (and its workspace size) is made for

struct Smem2 {
  static constexpr int kABytes = BMC * BK * 2;
  static constexpr int kBBytes = BNC * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages2 * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
  // push mode only: one [32 rows][32 + 4 floats] transposition buffer per epilogue warp, behind the barriers
  static constexpr int kPushRowFloats = 36;
  static constexpr int kPushWarpBytes = 32 * kPushRowFloats * 4;
  static constexpr int kPushOffset = kBarOffset + 256;
  static constexpr int kTotalPush = kTotal + 4 * kPushWarpBytes;
  // TMA-store mode only: two [32 rows][128 bytes] output boxes per epilogue warp, 1024-byte aligned
  static constexpr int kOutOffset = kBarOffset + 1024;
  static constexpr int kOutWarpBytes = 2 * 32 * 128;
  static constexpr int kTotalOut = kOutOffset + 4 * kOutWarpBytes + 1024;
};
static_assert(Smem2::kTotalOut <= 232448, "the output boxes must fit next to the operand ring");

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

// Work items.  Items [0, n_full) are whole tiles.  The tiles that would form a partial last
// wave are each cut into two K halves (items n_full + 2*tail + half) that run side by side on
// two CTA pairs; each half leaves its fp32 accumulator in the workspace and takes a ticket,
// and the half that draws the second ticket adds the other half's values and writes C.
// Nothing waits on another CTA.
struct Item2 {
  int tile, kb0, kb1, tail, half;
};
__device__ __forceinline__ Item2 get_item2(int i, int n_full, int num_kb) {
  if (i < n_full) return Item2{i, 0, num_kb, -1, 0};
  const int u = i - n_full, tail = u >> 1, half = u & 1, mid = num_kb >> 1;
  return Item2{n_full + tail, half ? mid : 0, half ? num_kb : mid, tail, half};
}

// MODE: what the epilogue does with a finished tile.  Separate instantiations, so that the plain
// store keeps its register budget and code exactly as if the other two did not exist.
enum { kStore = 0, kPush = 1, kFused = 2, kStoreTma = 3, kStoreTmaWide = 4, kPushWide = 5 };
// kStoreTmaWide, kPushWide: deep-K products.  A work item is a 256 x 512 tile: both accumulators (all 512 tensor-memory columns)
// belong to ONE item, whose two 256-column halves share every A k-block, so per MMA each SM's shared memory takes
// 6 KB of TMA writes instead of 8.  The price is that the epilogue no longer overlaps the next item's MMAs, which a
// long K makes small.  Four stages of 48 KB instead of six of 32 KB.
constexpr int kWideN = 512;
constexpr int kStagesWide = 4;

template <typename TO, bool BF16, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kThreads2, 1)
    gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const __grid_constant__ CUtensorMap tmap_c, TO* __restrict__ C, int M, int N, int K, int64_t ldc, int accumulate, int vec_c,
                             int n_full, int n_items, float* __restrict__ partials,
                             unsigned* __restrict__ tickets, const PushTargets push, const EpilogueArgs epi,
                             unsigned* __restrict__ status) {
  using L = Smem2;
  constexpr bool WIDE = MODE == kStoreTmaWide || MODE == kPushWide;
  constexpr bool PUSH = MODE == kPush || MODE == kPushWide;
  constexpr bool TMA_OUT = MODE == kStoreTma || MODE == kStoreTmaWide;
  constexpr int TILE_N = WIDE ? kWideN : BN2;                       // columns of a work item
  constexpr int NST = WIDE ? kStagesWide : kStages2;                // ring depth
  constexpr int STAGE = WIDE ? L::kABytes + 2 * L::kBBytes : L::kStageBytes;
  static_assert(kStagesWide * (L::kABytes + 2 * L::kBBytes) <= L::kBarOffset, "the wide ring must fit in the ring area");
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages2;
  uint64_t* acc_full = empty_bar + kStages2;  // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2] (the leader's is the one that is used)
  uint64_t* epi_bar = acc_empty + 2;          // [1] the four epilogue warps of this CTA among themselves
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_word = tmem_slot + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + BM2 - 1) / BM2, tiles_n = (N + TILE_N - 1) / TILE_N;
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
    mbar_init(epi_bar, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (TMA_OUT) tma_prefetch_desc(&tmap_c);
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
  // Launched with programmatic stream serialization: the next kernel in the stream may take an SM as
  // soon as this CTA leaves it and run its own set-up (barriers, tensor memory) while our last wave
  // drains; nothing of that kernel touches global memory before its own wait below has seen the
  // kernel in front of it complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < n_items && ok; t += num_pairs) {
        const Item2 it = get_item2(t, n_full, num_kb);
        TileCoord tc = tile_coord(it.tile, tiles_m, tiles_n);
        const int m0 = tc.m * BM2 + (int)rank * BMC;   // this CTA's rows of A (and of C)
        const int n0 = tc.n * TILE_N + (int)rank * BNC;   // this CTA's half of the (first) B tile
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          unsigned char* sa = smem + stage * STAGE;
          unsigned char* sb = sa + L::kABytes;
          // the leader's barrier collects the bytes of both CTAs
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE);
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
          if (WIDE) {
            // this CTA's half of the second 256 columns (beyond N the TMA unit fills zeros)
            unsigned char* sb1 = sb + L::kBBytes;
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BNC / 64; ++j)
                tma_load_2d_pair(sb1 + j * (BK * 128), &tmap_b, bar, n0 + BN2 + j * 64, k0);
            } else {
              tma_load_2d_pair(sb1, &tmap_b, bar, k0, n0 + BN2);
            }
          }
          if (++stage == NST) {
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
      for (int t = pair; t < n_items && ok; t += num_pairs) {
        const Item2 it = get_item2(t, n_full, num_kb);
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, status, ST_TIMEOUT_ACC_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (WIDE ? 0 : acc * BN2);
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * STAGE);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = A_MN ? umma_desc_mnmajor_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                               : umma_desc_kmajor_sw128(sa + k * (UMMA_K * 2));
            uint64_t db = B_MN ? umma_desc_mnmajor_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                               : umma_desc_kmajor_sw128(sb + k * (UMMA_K * 2));
            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb > it.kb0 || k != 0) ? 1u : 0u);
            if (WIDE) {
              const uint32_t sb1 = sb + L::kBBytes;
              uint64_t db1 = B_MN ? umma_desc_mnmajor_sw128(sb1 + k * (UMMA_K * 128), BK * 128, 1024)
                                  : umma_desc_kmajor_sw128(sb1 + k * (UMMA_K * 2));
              umma_f16_ss_pair(d_tmem + BN2, da, db1, idesc, (kb > it.kb0 || k != 0) ? 1u : 0u);
            }
          }
          umma_commit_pair(&empty_bar[stage], 3);  // both CTAs may refill this stage
          if (++stage == NST) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[acc], 3);  // both CTAs' epilogues may read their accumulator halves
        if (WIDE) {
          acc_phase ^= 1;  // one accumulator (of 512 columns), used by every item
        } else if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows)
    const int quad = warp & 3;
    int box_sel = 0;  // which of the warp's two output boxes the next TMA store uses
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_acc_empty0 = mapa_u32(&acc_empty[0], 0), leader_acc_empty1 = mapa_u32(&acc_empty[1], 0);
    uint32_t epi_phase = 0;
    bool epi_ok = true;
    // bounded meeting point of this CTA's 128 epilogue threads
    auto epi_sync = [&]() {
      mbar_arrive(epi_bar);
      if (epi_ok) epi_ok = mbar_wait(epi_bar, epi_phase, abort_flag, status, ST_TIMEOUT_MISC);
      epi_phase ^= 1;
    };
    for (int t = pair; t < n_items; t += num_pairs) {
      const Item2 it = get_item2(t, n_full, num_kb);
      TileCoord tc = tile_coord(it.tile, tiles_m, tiles_n);
      const int m0 = tc.m * BM2 + (int)rank * BMC, n0 = tc.n * TILE_N;
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, status, ST_TIMEOUT_ACC_FULL)) break;
      tc_fence_after_sync();
      const int row_local = quad * 32 + lane;
      const int row = m0 + row_local;
      const uint32_t taddr = tmem_base + (WIDE ? 0 : acc * BN2) + (static_cast<uint32_t>(quad * 32) << 16);
      bool write_c = true;
      const float4* other = nullptr;
      if (it.tail >= 0) {  // (pushed K halves simply both add into the owner's buffer)
        // leave this K half in the workspace, then see whether the other half is already there
        // scratch layout per (tail tile, K half, CTA): [64 groups of 4 columns][128 rows] float4, so that
        // the 32 lanes of a warp (32 consecutive rows) write and read consecutive 16-byte words
        float4* mine = reinterpret_cast<float4*>(partials + (((size_t)it.tail * 2 + it.half) * 2 + rank) * (BMC * BN2)) + row_local;
        other = reinterpret_cast<const float4*>(partials + (((size_t)it.tail * 2 + (it.half ^ 1)) * 2 + rank) * (BMC * BN2)) + row_local;
#pragma unroll 1
        for (int c = 0; c < BN2 / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            __stcg(mine + (c * 8 + i) * BMC,
                   make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                               __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])));
        }
        __threadfence();
        epi_sync();
        if (warp == 2 && lane == 0) *epi_word = atomicAdd(&tickets[it.tail * 2 + rank], 1u);
        epi_sync();
        write_c = epi_ok && (*epi_word == 1u);
        if (write_c) __threadfence();
        epi_sync();  // everybody has read the ticket before the next item overwrites it
        if (write_c && warp == 2 && lane == 0) tickets[it.tail * 2 + rank] = 0;
      }
      float row_acc = 0.f;
      if (MODE == kFused)
        row_acc = epi.reduce_kind == FRISK_B200_REDUCE_MAX ? -INFINITY
                  : epi.reduce_kind == FRISK_B200_REDUCE_MIN ? INFINITY : 0.f;
      if (TMA_OUT && write_c) {
        // Plain store through shared memory: a lane holds 128 bytes of ONE row, the warp writes them as a
        // [32 rows][128 bytes] box in the 128-byte-swizzle image and one lane hands the box to the TMA unit,
        // which writes whole lines and clips the box at the edges of C.  Two boxes per warp alternate.
        constexpr int kUnitCols = 128 / (int)sizeof(TO);
        unsigned char* boxes = smem + L::kOutOffset + quad * L::kOutWarpBytes;
#pragma unroll 1
        for (int u = 0; u < TILE_N / kUnitCols; ++u) {
          const int c0 = n0 + u * kUnitCols, r0 = m0 + quad * 32;
          if (c0 >= N || r0 >= M) break;  // wholly outside C (warp-uniform)
          uint32_t w[32];
          if (sizeof(TO) == 4) {
            tmem_ld_32x32b_x32(taddr + u * 32, w);
            tmem_ld_wait();
            if (other != nullptr) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 o = __ldcg(other + (u * 8 + i) * BMC);
                w[4 * i] = __float_as_uint(__uint_as_float(w[4 * i]) + o.x);
                w[4 * i + 1] = __float_as_uint(__uint_as_float(w[4 * i + 1]) + o.y);
                w[4 * i + 2] = __float_as_uint(__uint_as_float(w[4 * i + 2]) + o.z);
                w[4 * i + 3] = __float_as_uint(__uint_as_float(w[4 * i + 3]) + o.w);
              }
            }
          } else {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              uint32_t v[32];
              tmem_ld_32x32b_x32(taddr + u * 64 + hh * 32, v);
              tmem_ld_wait();
              if (other != nullptr) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float4 o = __ldcg(other + ((u * 2 + hh) * 8 + i) * BMC);
                  v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + o.x);
                  v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + o.y);
                  v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + o.z);
                  v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + o.w);
                }
              }
#pragma unroll
              for (int i = 0; i < 16; ++i)
                w[hh * 16 + i] = pack_out<TO>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
          }
          // the store before the last one used this box: it has been read
          if (lane == 0) tma_store_wait_read<1>();
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
      } else if (write_c) {
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c * 32, v);
          tmem_ld_wait();
          if (other != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 o = __ldcg(other + (c * 8 + i) * BMC);
              v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + o.x);
              v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + o.y);
              v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + o.z);
              v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + o.w);
            }
          }
          const int col = n0 + c * 32;
          if (PUSH) {
            // split-K across GPUs: store this chunk into this rank's slot at the GPU that owns the row.
            // A thread holds 32 columns of ONE row; stored as they are, every 16-byte store would be
            // its own NVLink transaction (measured: 65 GB/s per GPU).  The warp therefore transposes
            // its 32 x 32 block through shared memory so that eight lanes write one full 128-byte
            // line of a row and one instruction writes four such lines.
            float* stage = reinterpret_cast<float*>(smem + L::kPushOffset) + quad * (32 * L::kPushRowFloats);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<float4*>(stage + lane * L::kPushRowFloats + 4 * i) =
                  make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                              __uint_as_float(v[4 * i + 3]));
            __syncwarp();
            const int piece = lane & 7, rsub = lane >> 3;
            const int gcol = col + piece * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rl = j * 4 + rsub;
              const int grow = m0 + quad * 32 + rl;
              const float4 x = *reinterpret_cast<const float4*>(stage + rl * L::kPushRowFloats + piece * 4);
              if (grow < M && gcol < N) {
                const int owner = grow / push.rows_per_target;
                float* dst = push.ptr[owner] + (int64_t)(grow - owner * push.rows_per_target) * push.ld + gcol;
                if (gcol + 4 <= N && (push.ld & 3) == 0) {
                  *reinterpret_cast<float4*>(dst) = x;
                } else {
                  const float xs[4] = {x.x, x.y, x.z, x.w};
                  for (int e = 0; e < 4 && gcol + e < N; ++e) dst[e] = xs[e];
                }
              }
            }
            __syncwarp();  // the buffer is rewritten for the next 32 columns
          } else if (row < M && col < N) {
            const int valid = min(32, N - col);
            if (MODE == kFused && epi.has_fill) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + epi.fill);
            }
            store_row_chunk<TO>(C + (int64_t)row * ldc + col, v, valid, vec_c != 0, accumulate != 0);
            if (MODE == kFused && epi.reduce_kind) {
              // over the values as they were stored (accumulate is off whenever a reduction is fused)
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float r = rounded_as<TO>(__uint_as_float(v[i]));
                if (i < valid)
                  row_acc = epi.reduce_kind == FRISK_B200_REDUCE_MAX   ? fmaxf(row_acc, r)
                            : epi.reduce_kind == FRISK_B200_REDUCE_MIN ? fminf(row_acc, r)
                                                                       : row_acc + r;
              }
            }
          }
        }
        if (MODE == kFused && epi.reduce_kind && row < M) epi.row_partials[(int64_t)tc.n * M + row] = row_acc;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? leader_acc_empty1 : leader_acc_empty0);
      if (WIDE) {
        acc_phase ^= 1;
      } else if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (TMA_OUT && lane == 0) tma_store_wait<0>();  // the boxes are read and written out before the CTA leaves
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

// Tail plan: `pairs` CTA pairs, `tiles` 256x256 tiles.  A partial last wave of at most pairs/2
// tiles is run as twice as many K halves.
struct TailPlan {
  int pairs, n_full, n_items, tail_tiles;
  size_t off_partials, bytes;
};
TailPlan make_tail_plan(const frisk_b200_gemm_desc& d, int pairs_available) {
  GemmDims g = resolve_dims(d);
  TailPlan t{};
  int tiles = (int)(((g.M + BM2 - 1) / BM2) * ((g.N + BN2 - 1) / BN2));
  t.pairs = tiles < pairs_available ? tiles : pairs_available;
  t.n_full = t.n_items = tiles;
  int rem = tiles % t.pairs;
  int num_kb = (int)((g.K + BK - 1) / BK);
  if (tiles > t.pairs && rem > 0 && 2 * rem <= t.pairs && num_kb >= 8) {
    t.tail_tiles = rem;
    t.n_full = tiles - rem;
    t.n_items = t.n_full + 2 * rem;
  } else if (2 * tiles <= pairs_available && num_kb >= kMinKbAllHalved) {
    // fewer tiles than half the pairs: EVERY tile runs as two K halves, so twice as many SMs work
    t.tail_tiles = tiles;
    t.n_full = 0;
    t.n_items = 2 * tiles;
    t.pairs = 2 * tiles;
  }
  // tickets live in a fixed-size prefix so that a scratch buffer reused for another shape never
  // finds old partial sums where it keeps tickets
  t.off_partials = kTicketBytes;
  t.bytes = t.tail_tiles ? t.off_partials + (size_t)t.tail_tiles * 2 * BM2 * BN2 * sizeof(float) : 0;
  return t;
}

template <typename TO, bool BF16, bool A_MN, bool B_MN, int MODE>
int launch_cfg2(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                void* ws, size_t ws_bytes, cudaStream_t s, const PushTargets* push_in = nullptr,
                const EpilogueArgs* epi_in = nullptr) {
  GemmDims g = resolve_dims(d);
  CUtensorMap ta, tb;
  int rc;
  if (A_MN)
    rc = encode_tmap_2d(ctx, &ta, d.dtype_ab, A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(ctx, &ta, d.dtype_ab, A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda * 2, BK, BMC, true);
  if (rc) { ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }
  if (B_MN)
    rc = encode_tmap_2d(ctx, &tb, d.dtype_ab, B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb * 2, 64, BK, true);
  else
    rc = encode_tmap_2d(ctx, &tb, d.dtype_ab, B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb * 2, BK, BNC, true);
  if (rc) { ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }

  CUtensorMap tc = ta;  // unused by the other modes
  if (MODE == kStoreTma || MODE == kStoreTmaWide) {
    // C as [M][N] with boxes of 32 rows x 128 bytes in the 128-byte-swizzle image the epilogue writes
    const int out_dtype = sizeof(TO) == 4 ? FRISK_B200_F32 : (std::is_same<TO, __half>::value ? FRISK_B200_F16 : FRISK_B200_BF16);
    rc = encode_tmap_2d(ctx, &tc, out_dtype, C, (uint64_t)g.N, (uint64_t)g.M, (uint64_t)g.ldc * sizeof(TO),
                        128 / sizeof(TO), 32, true);
    if (rc) { ctx->last_cuda = rc; return FRISK_B200_E_CUDA; }
  }

  auto kern = gemm_tcgen05_2cta_kernel<TO, BF16, A_MN, B_MN, MODE>;
  constexpr int kSmemBytes = (MODE == kPush || MODE == kPushWide) ? Smem2::kTotalPush
                             : (MODE == kStoreTma || MODE == kStoreTmaWide) ? Smem2::kTotalOut : Smem2::kTotal;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads2);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(2 * (ctx->num_sms / 2));
  // once per device and instantiation: the shared-memory opt-in and how many CTA pairs fit the device
  static PerDeviceOnce set_up;
  static std::atomic<int> pairs_on_device[kMaxDevices];
  if (ctx->device < 0 || ctx->device >= kMaxDevices) return FRISK_B200_E_ARG;
  if (set_up(ctx->device, [&] {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) return 1;
        pairs_on_device[ctx->device].store(n);
        return 0;
      }))
    return FRISK_B200_E_CUDA;
  int max_clusters = pairs_on_device[ctx->device].load();
  if (max_clusters < 1) return FRISK_B200_E_UNSUPPORTED;
  if (max_clusters > kPairsAssumed) max_clusters = kPairsAssumed;
  TailPlan tp = make_tail_plan(d, max_clusters);
  PushTargets push{};
  if (push_in) push = *push_in;
  EpilogueArgs epi{};
  if (epi_in) epi = *epi_in;
  if (MODE == kStoreTmaWide || MODE == kPushWide) {
    // 256 x 512 items, every one whole
    const int tiles_w = (int)(((g.M + BM2 - 1) / BM2) * ((g.N + kWideN - 1) / kWideN));
    tp.pairs = tiles_w < max_clusters ? tiles_w : max_clusters;
    tp.n_full = tp.n_items = tiles_w;
    tp.tail_tiles = 0;
    tp.bytes = 0;
  }
  if (tp.bytes && (MODE == kPush || MODE == kPushWide || !ws || ws_bytes < tp.bytes)) {
    // no scratch: run every tile whole
    tp.n_full = tp.n_items = tp.n_full + tp.tail_tiles;
    tp.tail_tiles = 0;
  }
  cfg.gridDim = dim3(2 * tp.pairs);
  cfg.numAttrs = 2;  // (the occupancy query above ran with the cluster attribute alone)
  unsigned* tickets = static_cast<unsigned*>(ws);
  float* partials = tp.tail_tiles ? reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + tp.off_partials) : nullptr;
  int vec_c = aligned16(C) && (g.ldc * sizeof(TO)) % 16 == 0;
  TO* Cp = static_cast<TO*>(C);
  int Mi = (int)g.M, Ni = (int)g.N, Ki = (int)g.K, acc = (d.clear_accum || epi.has_fill) ? 0 : 1;
  int64_t ldc = g.ldc;
  unsigned* st = ctx->d_status;
  int n_full = tp.n_full, n_items = tp.n_items;
  FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, Cp, Mi, Ni, Ki, ldc, acc, vec_c, n_full, n_items, partials,
                                  tickets, push, epi, st));
  return 0;
}

template <typename TO, bool BF16, int MODE>
int launch_major2(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                  void* ws, size_t ws_bytes, cudaStream_t s, const EpilogueArgs* epi) {
  bool a_mn = d.trans_a != 0, b_mn = d.trans_b == 0;
  if (a_mn) {
    if (b_mn) return launch_cfg2<TO, BF16, true, true, MODE>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr, epi);
    return launch_cfg2<TO, BF16, true, false, MODE>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr, epi);
  }
  if (b_mn) return launch_cfg2<TO, BF16, false, true, MODE>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr, epi);
  return launch_cfg2<TO, BF16, false, false, MODE>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr, epi);
}

}  // namespace

// The pair kernel pays when there are enough 256 x 256 tiles to fill the machine's CTA pairs.
// ... or so few that halving every tile's K doubles the SMs at work (the one-CTA kernel's 128 x 256 tiles
// would occupy at most as many SMs as there are tiles x 2).
bool tcgen05_2cta_preferred(const frisk_b200_gemm_desc& d) {
  const int64_t tiles = ((d.M + BM2 - 1) / BM2) * ((d.N + BN2 - 1) / BN2);
  if (tiles >= kNumSMsDefault / 2) return true;
  return 2 * tiles <= kPairsAssumed && (d.K + BK - 1) / BK >= kMinKbAllHalved;
}

// Split-K across GPUs: the same kernel, its epilogue storing every fp32 tile into this rank's slot at the row's owner.
int launch_gemm_tcgen05_2cta_push(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                                  const PushTargets& push, cudaStream_t s) {
  if (!tcgen05_supported(d) || d.dtype_c != FRISK_B200_F32) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  const bool a_mn = d.trans_a != 0, b_mn = d.trans_b == 0;
  if (a_mn || b_mn) return FRISK_B200_E_UNSUPPORTED;  // the K-split path keeps both operands K-contiguous
  // very deep K and several rounds of 256 x 512 items per CTA pair: the wide items (see kStoreTmaWide).  The push
  // of a wide item (512 KB per CTA to the row owners) does not hide behind the next item, so the bar is higher than
  // for a local store: 8192 x 8192 with K = 65536 per rank gains 6 %, with K = 16384 per rank it loses 2 %.
  const GemmDims g = resolve_dims(d);
  const int64_t tiles_w = ((g.M + BM2 - 1) / BM2) * ((g.N + kWideN - 1) / kWideN);
  if (g.K >= 32768 && tiles_w >= 4 * kPairsAssumed) {
    if (d.dtype_ab == FRISK_B200_BF16)
      return launch_cfg2<float, true, false, false, kPushWide>(ctx, d, A, B, nullptr, nullptr, 0, s, &push);
    return launch_cfg2<float, false, false, false, kPushWide>(ctx, d, A, B, nullptr, nullptr, 0, s, &push);
  }
  if (d.dtype_ab == FRISK_B200_BF16)
    return launch_cfg2<float, true, false, false, kPush>(ctx, d, A, B, nullptr, nullptr, 0, s, &push);
  return launch_cfg2<float, false, false, false, kPush>(ctx, d, A, B, nullptr, nullptr, 0, s, &push);
}

int tcgen05_2cta_column_tiles(const frisk_b200_gemm_desc& d) { return (int)((resolve_dims(d).N + BN2 - 1) / BN2); }

// Worst case over the number of CTA pairs the device grants (at most kPairsAssumed/2 tail tiles).
size_t tcgen05_2cta_workspace_bytes(const frisk_b200_gemm_desc& d) {
  GemmDims g = resolve_dims(d);
  const int64_t tiles = ((g.M + BM2 - 1) / BM2) * ((g.N + BN2 - 1) / BN2);
  const int64_t num_kb = (g.K + BK - 1) / BK;
  if (num_kb < 8) return 0;
  if (2 * tiles <= kPairsAssumed ? num_kb < kMinKbAllHalved : tiles <= kPairsAssumed) return 0;
  return kTicketBytes + (size_t)(kPairsAssumed / 2) * 2 * BM2 * BN2 * sizeof(float);
}

int launch_gemm_tcgen05_2cta(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                             void* C, void* ws, size_t ws_bytes, cudaStream_t s, const EpilogueArgs* epi) {
  if (!tcgen05_supported(d)) return FRISK_B200_E_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return FRISK_B200_E_ALIGN;
  const bool bf = d.dtype_ab == FRISK_B200_BF16;
  if (epi && (epi->has_fill || epi->reduce_kind)) {
    if (d.dtype_c == FRISK_B200_F32)
      return bf ? launch_major2<float, true, kFused>(ctx, d, A, B, C, ws, ws_bytes, s, epi)
                : launch_major2<float, false, kFused>(ctx, d, A, B, C, ws, ws_bytes, s, epi);
    if (bf) return launch_major2<__nv_bfloat16, true, kFused>(ctx, d, A, B, C, ws, ws_bytes, s, epi);
    return launch_major2<__half, false, kFused>(ctx, d, A, B, C, ws, ws_bytes, s, epi);
  }
  // an overwriting store of a C whose base and row pitch are 16-byte aligned goes out through the TMA unit
  const GemmDims g = resolve_dims(d);
  const size_t cs = dtype_size(d.dtype_c);
#ifndef FB_NO_TMA_STORE
  if (d.clear_accum && aligned16(C) && (g.ldc * cs) % 16 == 0) {
    // deep K and enough 256 x 512 items to keep every CTA pair busy for several rounds: the wide items
    const int64_t tiles_w = ((g.M + BM2 - 1) / BM2) * ((g.N + kWideN - 1) / kWideN);
    // (at 8192 x 8192 the wide items lose 2-7 % for K <= 4096, where the exposed epilogue outweighs the saved writes)
    if (g.K >= 8192 && tiles_w >= 4 * kPairsAssumed) {
      if (d.dtype_c == FRISK_B200_F32)
        return bf ? launch_major2<float, true, kStoreTmaWide>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr)
                  : launch_major2<float, false, kStoreTmaWide>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
      if (bf) return launch_major2<__nv_bfloat16, true, kStoreTmaWide>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
      return launch_major2<__half, false, kStoreTmaWide>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
    }
    if (d.dtype_c == FRISK_B200_F32)
      return bf ? launch_major2<float, true, kStoreTma>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr)
                : launch_major2<float, false, kStoreTma>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
    if (bf) return launch_major2<__nv_bfloat16, true, kStoreTma>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
    return launch_major2<__half, false, kStoreTma>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
  }
#endif
  if (d.dtype_c == FRISK_B200_F32)
    return bf ? launch_major2<float, true, kStore>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr)
              : launch_major2<float, false, kStore>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
  if (bf) return launch_major2<__nv_bfloat16, true, kStore>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
  return launch_major2<__half, false, kStore>(ctx, d, A, B, C, ws, ws_bytes, s, nullptr);
}

}  // namespace fb
