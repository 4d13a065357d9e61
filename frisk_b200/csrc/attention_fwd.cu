// Fused attention forward for sm_100a: O = softmax(scale * Q.K^T [+ causal mask]) . V over
// compact BHSD tensors, fp16/bf16 inputs, fp32 scores and statistics, probabilities rounded to
// the 16-bit input type before P.V.  Numerics contract:
// benchmark/layout/execution/tiled_attention.py:392,505-515,628-629 (scale applied to the fp32
// dot, exp through ex2, P rounded RNE before P.V, fp32 accumulation of P.V); launch contract:
// tiled_attention.py:52-61 (compact BHSD, q/k/v/out pointers).
//
// Unlike the reference's three-pass schedule (tiled_attention.py:697-698) this is a single
// pass with an online softmax, so K and V are read once per query tile:
//
//   * the kernel is persistent: one CTA per SM takes work items (TWO 128-row query tiles of one
//     (batch, head)) from an atomic counter, heavy items first, until none is left.  Barriers, tensor
//     memory and the K/V ring live across items, so the next item's Q, K and V are already on their
//     way, and its first scores are computed, while the softmax warps still store the last item's O;
//   * 128-key K/V tiles stream through a 2-stage TMA ring (K and V have separate full/empty mbarriers);
//   * warp 8 is the TMA producer; warps 9 and 10 issue the tcgen05.mma of query tile 0 and 1: S_q =
//     Q_q.K^T (SS form, both operands K-major, 128-byte swizzle) into tensor memory and O_q += P_q.V
//     (P read from tensor memory, V as an MN-major shared-memory operand);
//   * warps 0-3 and 4-7 are the two softmax groups: thread r owns row r of its query tile
//     (TMEM lane r), so row max / row sum need no shuffles.  The two groups alternate, so
//     the tensor core works on one tile's MMAs while the other group exponentiates;
//   * the running maximum is applied lazily: O is rescaled in tensor memory only when the
//     maximum grew by more than 2^8, which keeps P within bf16/fp16 range and makes most
//     iterations rescale-free;
//   * causal: key tiles wholly above the diagonal are never loaded; only tiles that touch the
//     diagonal (or the ragged end of the keys) are masked.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D); P_q aliases the first
// 64 columns of S_q (two 16-bit values per column).
// Every mbarrier wait is bounded (ptx.cuh); no TMA load uses cluster multicast.
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

#include "attention_common.cuh"

namespace fb {
namespace {
using namespace attn;

constexpr int kStagesKV = 2;
constexpr int kHeadChunk = 16;  // heads whose K and V are worked on together (they stay in L2: 16 x 2 MB at S = 4096)
template <int D>
struct AttnSmem {
  static constexpr int kTileBytes = BM * D * 2;       // one Q, K or V tile
  static constexpr int kQ = 0;                         // Q0, Q1
  static constexpr int kK = 2 * kTileBytes;            // K stages
  static constexpr int kV = kK + kStagesKV * kTileBytes;
  static constexpr int kBar = kV + kStagesKV * kTileBytes;
  // 16-bit outputs: one [32 rows][128 bytes] box per softmax warp for the TMA stores of O, 1024-byte aligned
  static constexpr int kOut = kBar + 1024;
  static constexpr int kTotal = kOut + 8 * (32 * 128) + 1024;
  static_assert(kTotal <= 232448, "the output boxes must fit next to the Q, K and V tiles");
};


template <bool BF16, int D, bool OUT_F32, bool NORM>
__global__ void __launch_bounds__(kThreads, 1)
    attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                         const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int kBoxes = D / 64;            // 64-element (128-byte) column blocks per tile
  constexpr int kBoxBytes = BM * 128;       // one [128 rows][128 B] block
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;              // [1]
  uint64_t* k_full = bars + 1;          // [2]
  uint64_t* k_empty = bars + 3;         // [2]
  uint64_t* v_full = bars + 5;          // [2]
  uint64_t* v_empty = bars + 7;         // [2]
  uint64_t* s_full = bars + 9;          // [2] per query tile
  uint64_t* p_ready = bars + 11;        // [2] first half of P_q (keys 0-63) written
  uint64_t* p_ready_hi = bars + 16;     // [2] second half written
  uint64_t* o_done = bars + 13;         // [2]
  uint64_t* turn = bars + 18;           // [2] hand-over of the exponential section between the two softmax groups
  uint64_t* item_full = bars + 20;      // [2] the producer has published the id of a work item
  uint64_t* item_empty = bars + 22;     // [2] every consumer has read it
  uint64_t* q_empty = bars + 24;        // [1] both MMA threads are done with the Q tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* item_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work items in the order they are handed out: heads in chunks of kHeadChunk (their K and V stay in L2
  // together); inside a chunk the heavy (late) query tiles of every head first, so that the machine
  // drains on light items.
  struct Item {
    int bh, m0, nq[2], n_max;
  };
  const int bh_total = (int)(p.total_items / p.n_pairs);
  auto decode = [&](int t) {
    const int per_chunk = kHeadChunk * p.n_pairs;
    const int chunk = t / per_chunk;
    const int within = t - chunk * per_chunk;
    const int heads_here = min(kHeadChunk, bh_total - chunk * kHeadChunk);
    const int pair = p.n_pairs - 1 - within / heads_here;
    Item it;
    it.bh = chunk * kHeadChunk + within % heads_here;
    it.m0 = pair * 2 * BM;
    it.nq[0] = kv_tiles_for(it.m0, p.S_q, p.S_kv, p.causal);
    it.nq[1] = kv_tiles_for(it.m0 + BM, p.S_q, p.S_kv, p.causal);
    it.n_max = max(it.nq[0], it.nq[1]);
    return it;
  };
  // Consumers (the two MMA threads, the softmax warps) learn the n-th item of this CTA from the producer:
  // returns its id, or -1 when the work has run out or a wait was abandoned.
  auto next_item = [&](int n, bool arrive) -> int {
    if (!mbar_wait(&item_full[n & 1], (n >> 1) & 1, abort_flag, p.status, ST_ATTN_Q)) return -1;
    const int t = item_slot[n & 1];
    if (arrive) mbar_arrive(&item_empty[n & 1]);
    return t;
  };
  // Normalised mode runs the key loop twice: pass 0 only gathers row maxima and row sums, pass 1
  // is the pass every mode has.  Barrier phases keep counting across passes and items.
  constexpr int first_pass = NORM ? 0 : 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);  // one arrival per MMA-issuing thread
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      mbar_init(&p_ready_hi[i], 128);
      mbar_init(&o_done[i], 1);
      mbar_init(&turn[i], 128);
      mbar_init(&item_full[i], 1);
      mbar_init(&item_empty[i], 10);  // two MMA threads, one lane of each of the eight softmax warps
    }
    mbar_init(q_empty, 2);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == kWarpMma) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // the TMA/MMA warpgroup hands registers to the two softmax warpgroups (a full row of S per thread)
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
  if (warp == kWarpTma) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int kt = 0, vt = 0;  // K / V tiles loaded so far, over all items (K is streamed once per pass)
      bool ok = true;
      for (int n = 0; ok; ++n) {
        // take the next item and tell the other roles (slot n & 1 was last used by item n - 2)
        if (n >= 2 && !mbar_wait(&item_empty[n & 1], ((n >> 1) & 1) ^ 1, abort_flag, p.status, ST_ATTN_Q)) break;
        int t = (int)atomicAdd(p.work, 1u);
        if (t >= (int)p.total_items) t = -1;
        item_slot[n & 1] = t;
        mbar_arrive(&item_full[n & 1]);
        if (t < 0) break;
        const Item it = decode(t);
        // the Q tiles of the item before are free when both MMA threads have issued their last S of it
        if (n > 0 && !mbar_wait(q_empty, (n - 1) & 1, abort_flag, p.status, ST_ATTN_Q)) break;
        mbar_expect_tx(q_full, 2 * L::kTileBytes);
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int b = 0; b < kBoxes; ++b)
            tma_load_3d(smem + L::kQ + q * L::kTileBytes + b * kBoxBytes, &tmap_q, q_full, b * 64, it.m0 + q * BM, it.bh);
        for (int pass = first_pass; pass < 2 && ok; ++pass) {
          for (int j = 0; j < it.n_max; ++j) {
            const int ks = kt % kStagesKV;
            if (!mbar_wait(&k_empty[ks], ((kt / kStagesKV) & 1) ^ 1, abort_flag, p.status, ST_ATTN_KV)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&k_full[ks], L::kTileBytes);
#pragma unroll
            for (int b = 0; b < kBoxes; ++b)
              tma_load_3d(smem + L::kK + ks * L::kTileBytes + b * kBoxBytes, &tmap_k, &k_full[ks], b * 64, j * BN, it.bh);
            ++kt;
            if (pass == 0) continue;  // the statistics pass needs no values
            const int vs = vt % kStagesKV;
            if (!mbar_wait(&v_empty[vs], ((vt / kStagesKV) & 1) ^ 1, abort_flag, p.status, ST_ATTN_KV)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&v_full[vs], L::kTileBytes);
#pragma unroll
            for (int b = 0; b < kBoxes; ++b)
              tma_load_3d(smem + L::kV + vs * L::kTileBytes + b * kBoxBytes, &tmap_v, &v_full[vs], b * 64, j * BN, it.bh);
            ++vt;
          }
        }
      }
    }
  } else if (warp == kWarpMma || warp == kWarpMma + 1) {
    // ------------------------------------------------------------------ MMA issuers, one thread per query tile
    // Each query tile has its own issuing thread (warps 9 and 10).  One thread for both tiles was the
    // kernel's bottleneck: besides the 32 MMAs of a key tile it has a dozen barrier waits, fences and commits
    // to execute, each a round trip of ~100 clocks for a single thread, and the two tiles' chains
    // (S -> softmax -> P.V -> next S) queued behind each other in it.  tcgen05 operations of ONE thread execute
    // in issue order, which is all the ordering a query tile needs (S_q(j+1) overwrites P_q(j) only after
    // P_q(j).V(j) has read it); the two tiles share only the read-only K and V stages, which each thread
    // releases with its own arrival (the empty barriers count two).
    const int mq = warp - kWarpMma;
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(BM, BN, BF16, false, false);
      constexpr uint32_t idesc_o = umma_idesc_f16(BM, D, BF16, false, true);
      const uint32_t sq = smem_u32(smem + L::kQ), sk = smem_u32(smem + L::kK), sv = smem_u32(smem + L::kV);
      // descriptors are built once; the k16 slices only add a constant to the start-address field
      const uint64_t dq = umma_desc_kmajor_sw128(sq + mq * L::kTileBytes);
      const uint64_t dk[2] = {umma_desc_kmajor_sw128(sk), umma_desc_kmajor_sw128(sk + L::kTileBytes)};
      const uint64_t dv[2] = {umma_desc_mnmajor_sw128(sv, kBoxBytes, 1024),
                              umma_desc_mnmajor_sw128(sv + L::kTileBytes, kBoxBytes, 1024)};
      const uint32_t t_sq = tmem_base + mq * 128;        // S_q; P_q aliases its first 64 columns (8 per k16 slice)
      const uint32_t t_oq = tmem_base + 256 + mq * 128;  // O_q
      int kt = 0, vt = 0;  // K / V tiles seen so far, over all items (ring positions; K is streamed once per pass)
      int steps = 0;       // (pass, key tile) steps of THIS query tile so far: the phase of s_full / p_ready
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int t = next_item(n, true);
        if (t < 0) break;
        const Item it = decode(t);
        const int n_mine = it.nq[mq], n_max = it.n_max;
        ok = mbar_wait(q_full, n & 1, abort_flag, p.status, ST_ATTN_Q);
        for (int pass = first_pass; pass < 2 && ok; ++pass) {
          const bool stats_pass = pass == 0;  // the pass that only gathers statistics issues no P.V
          // Per key tile and query tile the dependent chain is: softmax publishes P(j) -> P(j).V(j) -> S(j+1) ->
          // softmax.  Everything this thread can do off that chain is done off it: the wait for K(j+1) happens
          // before the wait for P(j), and the commits that release V(j), K(j+1) and publish O come after the
          // MMAs of S(j+1) have been issued (a commit covers everything issued before it, so they only fire a
          // little later than strictly possible).
          bool have_k = false;  // K(j) of the current pass is known to have landed
          for (int j = 0; j < n_max && ok; ++j, ++kt) {
            const int ks = kt % kStagesKV;
            if (!have_k) ok = mbar_wait(&k_full[ks], (kt / kStagesKV) & 1, abort_flag, p.status, ST_ATTN_KV);
            have_k = false;
            if (!ok) break;
            if (j < n_mine) {
              tc_fence_after_sync();
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t off = static_cast<uint64_t>(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
                umma_f16_ss(t_sq, dq + off, dk[ks] + off, idesc_s, kk != 0);
              }
              umma_commit(&s_full[mq]);
              umma_commit(&k_empty[ks]);  // this tile's use of the K stage ends when these MMAs have read it
              if (j > 0 && !stats_pass) {  // (deferred from the previous tile)
                umma_commit(&o_done[mq]);
                umma_commit(&v_empty[(vt - 1) % kStagesKV]);
              }
              if (pass == 1 && j == n_mine - 1) umma_commit(q_empty);  // this thread's last use of the Q tiles
            } else {
              mbar_arrive(&k_empty[ks]);  // a key tile only the other query tile needs
            }
            const int vs = vt % kStagesKV;
            if (j < n_mine) {
              // the next K tile, while the softmax group works on this one
              if (j + 1 < n_max) {
                ok = mbar_wait(&k_full[(kt + 1) % kStagesKV], ((kt + 1) / kStagesKV) & 1, abort_flag, p.status, ST_ATTN_KV);
                have_k = ok;
              }
              if (!stats_pass && ok) ok = mbar_wait(&v_full[vs], (vt / kStagesKV) & 1, abort_flag, p.status, ST_ATTN_KV);
              // O_q += P_q(j) . V(j).  The softmax group publishes P in two halves (64 keys each), so the first
              // four k16 slices start while the second half is still being exponentiated.  In the statistics
              // pass the two waits only tell that the softmax group is done with S_q.
              const uint32_t parity = steps & 1;
              ++steps;
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                if (ok) ok = mbar_wait(half ? &p_ready_hi[mq] : &p_ready[mq], parity, abort_flag, p.status, ST_ATTN_P);
                if (stats_pass) continue;
                if (!ok) break;
                tc_fence_after_sync();
#pragma unroll
                for (int kk = half * 4; kk < half * 4 + 4; ++kk)
                  umma_f16_ts(t_oq, t_sq + kk * 8, dv[vs] + static_cast<uint64_t>((kk * 2048) >> 4), idesc_o,
                              (j | kk) != 0);
              }
              if (!ok) break;
              if (!stats_pass && (j + 1 >= n_mine)) {  // no further S of this item follows: publish now
                umma_commit(&o_done[mq]);
                umma_commit(&v_empty[vs]);
              }
            } else if (!stats_pass) {
              ok = mbar_wait(&v_full[vs], (vt / kStagesKV) & 1, abort_flag, p.status, ST_ATTN_KV);
              if (ok) mbar_arrive(&v_empty[vs]);
            }
            if (!stats_pass) ++vt;
          }
        }
        if (ok && n_mine == 0) mbar_arrive(q_empty);  // (a query tile beyond the end of the sequence)
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // ------------------------------------------------------------------ softmax groups
    const int q = warp >> 2;         // query tile of this group
    const int quad = warp & 3;       // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + q * 128 + lane_addr;
    const uint32_t t_o = tmem_base + 256 + q * 128 + lane_addr;
    const int off = p.S_kv - p.S_q;
    int steps = 0;    // (pass, key tile) steps of this query tile so far, over all items: the phase of s_full
    int turns = 0;    // key-tile iterations so far: the phase of the turn barriers
    int pv_base = 0;  // key tiles whose P.V was issued for earlier items: the phase of o_done
    bool ok = true;

    for (int n = 0; ok; ++n) {
      const int item_id = next_item(n, lane == 0);
      if (item_id < 0) break;
      const Item it = decode(item_id);
      const int bh = it.bh, n_max = it.n_max;
      const int n_tiles = it.nq[q];
      const int m_tile = it.m0 + q * BM;
      const int g_row = m_tile + row;  // query index within the head
      float m_ref = -INFINITY;  // reference maximum (scaled, log2 units) the stored P and O are relative to
      float l_sum = 0.f;

      if (NORM) {
        // The reference's semantics (benchmark/layout/execution/tiled_attention.py:697-698,
        // tail_attention_reference.py:74-78): score = fp32(dot) * scale; subtract the maximum of the
        // WHOLE row; e = ex2((score - max) * log2e); p = e / (sum of e over the whole row), IEEE
        // division; p rounded to 16 bits; then P.V.  Pass 0 finds max and sum, pass 1 forms P.
        const float kLog2e = 1.44269504088896340736f;
        float m_run = -INFINITY, l_run = 0.f;
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait(&s_full[q], steps & 1, abort_flag, p.status, ST_ATTN_S)) {
              ok = false;
              break;
            }
            ++steps;
            tc_fence_after_sync();
            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, sr[c]);
            tmem_ld_wait();
            const int n0 = j * BN;
            int limit = p.S_kv - 1;
            if (p.causal) limit = min(limit, g_row + off);
            limit -= n0;
            if (pass == 0) {
              // S_q is in registers: the MMA warp may overwrite it
              tc_fence_before_sync();
              mbar_arrive(&p_ready[q]);
              mbar_arrive(&p_ready_hi[q]);
              float mx = -INFINITY;
#pragma unroll
              for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  float sc = (c * 32 + i > limit) ? -INFINITY : __fmul_rn(__uint_as_float(sr[c][i]), p.scale);
                  sr[c][i] = __float_as_uint(sc);
                  mx = fmaxf(mx, sc);
                }
              const float m_new = fmaxf(m_run, mx);
              float sum = 0.f;
              if (m_new != -INFINITY) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    sum += ex2f_ieee_range(__fmul_rn(__fsub_rn(__uint_as_float(sr[c][i]), m_new), kLog2e));
                const float carry = (m_run == -INFINITY) ? 0.f : l_run * ex2f_ieee_range(__fmul_rn(__fsub_rn(m_run, m_new), kLog2e));
                l_run = carry + sum;
                m_run = m_new;
              }
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  float pv[2];
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    const int col = c * 32 + 2 * i + e;
                    const float sc = __fmul_rn(__uint_as_float(sr[c][2 * i + e]), p.scale);
                    const float ex = (col > limit) ? 0.f : ex2f_ieee_range(__fmul_rn(__fsub_rn(sc, m_run), kLog2e));
                    pv[e] = __fdiv_rn(ex, l_run);
                  }
                  pk[i] = pack16<BF16>(pv[0], pv[1]);
                }
                tmem_st_32x32b_x16(t_s + c * 16, pk);
                if (c & 1) {
                  tmem_st_wait();
                  tc_fence_before_sync();
                  mbar_arrive(c == 1 ? &p_ready[q] : &p_ready_hi[q]);
                }
              }
            }
          }
        }
        l_sum = 1.0f;  // P is already normalised
      } else
      // The two softmax groups take turns: group 1 starts the arithmetic of its key tile j when group 0 has
      // finished that of its tile j (all 128 keys: handing over after the first 64 measured 3 % slower), and group 0
      // starts tile j+1 when group 1 has finished tile j.  Left alone the
      // two groups fall into step (they share the K/V ring and the tensor pipe), exponentiate at the same time
      // on the same four schedulers and then both sit idle while their MMAs run; taking turns, one group works
      // alone (a third faster) while the other group's P.V and next S are in flight.  A group with fewer key
      // tiles than the other keeps passing the turn on until the other is done.
      for (int j = 0; j < n_max; ++j) {
        const bool mine = j < n_tiles;
        uint32_t sr[4][32];
        if (mine) {
          if (!mbar_wait(&s_full[q], steps & 1, abort_flag, p.status, ST_ATTN_S)) {
            ok = false;
            break;
          }
          ++steps;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, sr[c]);
          tmem_ld_wait();
        }
        if (!mbar_wait(&turn[q], q == 0 ? ((turns & 1) ^ 1) : (turns & 1), abort_flag, p.status, ST_ATTN_S)) {
          ok = false;
          break;
        }
        ++turns;
        if (!mine) {
          mbar_arrive(&turn[q ^ 1]);
          continue;
        }

        const int n0 = j * BN;
        const bool needs_mask = (n0 + BN > p.S_kv) || (p.causal && (n0 + BN - 1 > m_tile + off));
        if (needs_mask) {
          int limit = p.S_kv - 1;
          if (p.causal) limit = min(limit, g_row + off);
          limit -= n0;  // columns > limit are hidden
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i > limit) sr[c][i] = 0xff800000u;  // -inf
        }
        // P = 2^(s*scale_log2 - m_ref) with packed fp32 FMAs, row sum in fp32, P rounded to 16 bits.
        // Two 32-key chunks at a time, interleaved pair by pair so that the special-function unit always has
        // independent work.  WITH_MAX also runs the row maximum of all 128 keys (four chains of three-input
        // max, two keys of every chunk per step) through the same loop: the maximum is a chain on the ALU, the
        // exponentials are bound by the special-function unit, and neither waits for the other.
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        float mxc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        auto exp_chunks = [&](int c0, float mref, uint32_t (&pa)[16], uint32_t (&pb)[16], float2& sum, auto with_max) {
          const float2 negm2 = make_float2(-mref, -mref);
          float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 xa = fma2(make_float2(__uint_as_float(sr[c0][2 * i]), __uint_as_float(sr[c0][2 * i + 1])), scale2, negm2);
            const float2 xb = fma2(make_float2(__uint_as_float(sr[c0 + 1][2 * i]), __uint_as_float(sr[c0 + 1][2 * i + 1])), scale2, negm2);
            if (decltype(with_max)::value) {
#pragma unroll
              for (int c = 0; c < 4; ++c)
                mxc[c] = max3f(mxc[c], __uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1]));
            }
            const float2 ea = make_float2(ex2f(xa.x), ex2f(xa.y));
            const float2 eb = make_float2(ex2f(xb.x), ex2f(xb.y));
            sa = add2(sa, ea);
            sb = add2(sb, eb);
            pa[i] = pack16<BF16>(ea.x, ea.y);
            pb[i] = pack16<BF16>(eb.x, eb.y);
          }
          sum = add2(sa, sb);
        };

        // Optimistic first half: the exponentials of keys 0-63 are taken relative to the reference maximum
        // the row already has, so they do not wait for the row maximum.  Only when the maximum turns out to
        // have grown by more than the threshold (rare after the first tiles; always on the first tile, whose
        // reference is -infinity) is O rescaled and the half recomputed.  The stale reference cannot overflow
        // what is kept: a value that would exceed 2^threshold is by construction one that triggers the
        // recomputation.
        uint32_t pk0[16], pk1[16];
        float2 sum01;
        exp_chunks(0, m_ref, pk0, pk1, sum01, std::true_type());
        const float mx = max3f(mxc[0], mxc[1], fmaxf(mxc[2], mxc[3]));
        float m_new = fmaxf(m_ref, mx * p.scale_log2);
        if (m_new == -INFINITY) m_new = 0.f;  // a row that sees no key yet: keep everything finite
        // lazy rescale: warp-uniform decision because the TMEM accesses are warp-collective
        const bool grow = (j > 0) && (m_new - m_ref > kRescaleThreshold);
        bool redo = j == 0;
        if (j == 0) {
          m_ref = m_new;
        } else if (__any_sync(0xffffffffu, grow)) {
          const float factor = ex2f(m_ref - m_new);
          m_ref = m_new;
          l_sum *= factor;
          redo = true;
          // O_q must be complete up to tile j-1 before it is scaled
          if (!mbar_wait(&o_done[q], (pv_base + j - 1) & 1, abort_flag, p.status, ST_ATTN_O)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st_32x32b_x32(t_o + c * 32, o);
          }
        }
        if (redo) exp_chunks(0, m_ref, pk0, pk1, sum01, std::false_type());
        // P is written back over S chunk by chunk; a half of P (64 keys) that is complete lets the MMA warp start on it
        tmem_st_32x32b_x16(t_s, pk0);
        tmem_st_32x32b_x16(t_s + 16, pk1);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&p_ready[q]);
        float2 sum23;
        exp_chunks(2, m_ref, pk0, pk1, sum23, std::false_type());
        tmem_st_32x32b_x16(t_s + 32, pk0);
        tmem_st_32x32b_x16(t_s + 48, pk1);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&p_ready_hi[q]);
        mbar_arrive(&turn[q ^ 1]);  // the other group's turn: its scores arrived while this one worked alone
        const float2 tot = add2(sum01, sum23);
        l_sum += tot.x + tot.y;
      }

      // ---- epilogue: O / l
      if (ok && n_tiles > 0) ok = mbar_wait(&o_done[q], (pv_base + n_tiles - 1) & 1, abort_flag, p.status, ST_ATTN_O);
      if (ok && n_tiles > 0) {
        tc_fence_after_sync();
        const float inv = 1.0f / l_sum;
        const bool valid = g_row < p.S_q;
        const size_t row_off = ((size_t)bh * p.S_q + (size_t)min(g_row, p.S_q - 1)) * D;
        uint32_t packed[32];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(t_o + c * 32, o);
          tmem_ld_wait();
          if (valid) {
            if (OUT_F32) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.O) + row_off + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                dst[i] = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                     __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
            }
          }
          if (!OUT_F32) {
            // the 32 scaled values of this lane's row, rounded: half of a 128-byte box row
#pragma unroll
            for (int i = 0; i < 16; ++i)
              packed[(c & 1) * 16 + i] = pack16<BF16>(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
            if (c & 1) {
              // A lane holds 128 bytes of ONE row: the warp writes its 32 rows as a 128-byte-swizzle box and one
              // lane hands it to the TMA unit, which writes whole lines and leaves out rows beyond S_q.
              unsigned char* box = smem + L::kOut + warp * (32 * 128);
              if (lane == 0) tma_store_wait_read<0>();  // the previous store from this box has read it
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                    make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              const int row0 = g_row - lane;
              if (lane == 0 && row0 < p.S_q) {
                tma_store_3d(&tmap_o, box, (c >> 1) * 64, row0, bh);
                tma_store_commit();
              }
            }
          }
        }
      }
      pv_base += n_tiles;
    }
  }

  // ------------------------------------------------------------------ teardown
  if (!OUT_F32 && warp < 8 && lane == 0) tma_store_wait<0>();  // the output boxes are read and written out
  if (*abort_flag) {
    unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  // the last CTA to leave puts the work counter back to zero for the next launch
  if (threadIdx.x == 0) {
    if (atomicAdd(p.work + 1, 1u) == gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
      __threadfence();
    }
  }
}

template <bool BF16, int D, bool OUT_F32, bool NORM>
int launch_cfg(frisk_b200_ctx* ctx, const frisk_b200_attn_desc& d, const void* Q, const void* K, const void* V,
               void* O, cudaStream_t s) {
  CUtensorMap tq, tk, tv;
  const int bh = d.B * d.H;
  const uint64_t row_bytes = (uint64_t)D * 2;
  int rc = encode_tmap_3d(ctx, &tq, d.dtype_in, Q, D, d.S_q, bh, row_bytes, row_bytes * d.S_q, 64, BM, 1, true);
  if (!rc) rc = encode_tmap_3d(ctx, &tk, d.dtype_in, K, D, d.S_kv, bh, row_bytes, row_bytes * d.S_kv, 64, BN, 1, true);
  if (!rc) rc = encode_tmap_3d(ctx, &tv, d.dtype_in, V, D, d.S_kv, bh, row_bytes, row_bytes * d.S_kv, 64, BN, 1, true);
  CUtensorMap to = tq;  // unused for fp32 outputs
  if (!rc && !OUT_F32)
    rc = encode_tmap_3d(ctx, &to, d.dtype_out, O, D, d.S_q, bh, row_bytes, row_bytes * d.S_q, 64, 32, 1, true);
  if (rc) {
    ctx->last_cuda = rc;
    return FRISK_B200_E_CUDA;
  }
  AttnParams p;
  p.S_q = d.S_q;
  p.S_kv = d.S_kv;
  p.n_pairs = (d.S_q + 2 * BM - 1) / (2 * BM);
  p.causal = d.causal ? 1 : 0;
  p.total_items = (int64_t)p.n_pairs * bh;
  p.scale_log2 = d.scale * 1.4426950408889634f;
  p.scale = d.scale;
  p.normalized = d.normalize_p ? 1 : 0;
  p.O = O;
  p.status = ctx->d_status;
  p.work = ctx->d_status + 16;  // work counter and exit counter of the persistent grid (zero between launches)
  if (p.total_items > INT32_MAX) return FRISK_B200_E_ATTN_SHAPE;
  auto kern = attention_fwd_kernel<BF16, D, OUT_F32, NORM>;
  using L = AttnSmem<D>;
  // setmaxnreg.inc waits (without a bound) until the CTA's own register pool holds what it
  // asks for: the registers the TMA/MMA warpgroup (128 threads) gives up must cover what the
  // two softmax warpgroups (256 threads) take, or the kernel would never start.  Checked
  // against the compiled register count before every launch.
  static PerDeviceOnce set_up;  // one per instantiation; a failed check is repeated (and fails) every call
  const int bad = set_up(ctx->device, [&] {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return (int)FRISK_B200_E_CUDA;
    if (fa.numRegs < kRegsOther || fa.numRegs > kRegsSoftmax ||
        (fa.numRegs - kRegsOther) * 128 < (kRegsSoftmax - fa.numRegs) * 256)
      return (int)FRISK_B200_E_UNSUPPORTED;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess)
      return (int)FRISK_B200_E_CUDA;
    return 0;
  });
  if (bad) return bad;
  const unsigned grid = (unsigned)std::min<int64_t>(p.total_items, ctx->num_sms);
  kern<<<grid, kThreads, L::kTotal, s>>>(tq, tk, tv, to, p);
  FB_CUDA(ctx, cudaGetLastError());
  return 0;
}

template <bool BF16, int D>
int launch_out(frisk_b200_ctx* ctx, const frisk_b200_attn_desc& d, const void* Q, const void* K, const void* V,
               void* O, cudaStream_t s) {
  if (d.normalize_p) {
    if (d.dtype_out == FRISK_B200_F32) return launch_cfg<BF16, D, true, true>(ctx, d, Q, K, V, O, s);
    return launch_cfg<BF16, D, false, true>(ctx, d, Q, K, V, O, s);
  }
  if (d.dtype_out == FRISK_B200_F32) return launch_cfg<BF16, D, true, false>(ctx, d, Q, K, V, O, s);
  return launch_cfg<BF16, D, false, false>(ctx, d, Q, K, V, O, s);
}

}  // namespace

int launch_attention_fwd(frisk_b200_ctx* ctx, const frisk_b200_attn_desc& d, const void* Q, const void* K,
                         const void* V, void* O, cudaStream_t s) {
  const bool bf = d.dtype_in == FRISK_B200_BF16;
  if (d.D == 128) return bf ? launch_out<true, 128>(ctx, d, Q, K, V, O, s) : launch_out<false, 128>(ctx, d, Q, K, V, O, s);
  if (d.D == 64) return bf ? launch_out<true, 64>(ctx, d, Q, K, V, O, s) : launch_out<false, 64>(ctx, d, Q, K, V, O, s);
  return FRISK_B200_E_ATTN_SHAPE;
}

}  // namespace fb
