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
//   * one CTA owns TWO 128-row query tiles of one (batch, head) and streams 128-key K/V tiles
//     through a 2-stage TMA ring (K and V have separate full/empty mbarriers);
//   * warp 8 is the TMA producer, warp 9 issues every tcgen05.mma: S_q = Q_q.K^T (SS form,
//     both operands K-major, 128-byte swizzle) into tensor memory and O_q += P_q.V (P read
//     from tensor memory, V as an MN-major shared-memory operand);
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
#include "common.cuh"
#include "ptx.cuh"

#include "attention_common.cuh"

namespace fb {
namespace {
using namespace attn;

constexpr int kStagesKV = 2;
#ifndef FB_ATTN_HEAD_CHUNK
#define FB_ATTN_HEAD_CHUNK 16
#endif
constexpr int kHeadChunk = FB_ATTN_HEAD_CHUNK;
template <int D>
struct AttnSmem {
  static constexpr int kTileBytes = BM * D * 2;       // one Q, K or V tile
  static constexpr int kQ = 0;                         // Q0, Q1
  static constexpr int kK = 2 * kTileBytes;            // K stages
  static constexpr int kV = kK + kStagesKV * kTileBytes;
  static constexpr int kBar = kV + kStagesKV * kTileBytes;
  static constexpr int kTotal = kBar + 256 + 1024;
};


template <bool BF16, int D, bool OUT_F32, bool NORM>
__global__ void __launch_bounds__(kThreads, 1)
    attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTA order: heads in chunks of kHeadChunk (their K and V stay in L2 together); inside a chunk the
  // heavy (late) query tiles of every head first, so that the machine drains on light CTAs
  const int bh_total = (int)(p.total_ctas / p.n_pairs);
  const int per_chunk = kHeadChunk * p.n_pairs;
  const int chunk = (int)blockIdx.x / per_chunk;
  const int within = (int)blockIdx.x - chunk * per_chunk;
  const int heads_here = min(kHeadChunk, bh_total - chunk * kHeadChunk);
  const int pair = p.n_pairs - 1 - within / heads_here;
  const int bh = chunk * kHeadChunk + within % heads_here;
  const int m0 = pair * 2 * BM;
  const int nq[2] = {kv_tiles_for(m0, p.S_q, p.S_kv, p.causal), kv_tiles_for(m0 + BM, p.S_q, p.S_kv, p.causal)};
  const int n_max = max(nq[0], nq[1]);
  // Normalised mode runs the key loop twice: pass 0 only gathers row maxima and row sums, pass 1
  // is the pass every mode has.  Barrier phases keep counting across the passes.
  constexpr int first_pass = NORM ? 0 : 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 128);
      mbar_init(&p_ready_hi[i], 128);
      mbar_init(&o_done[i], 1);
    }
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
    if (lane == 0 && n_max > 0) {
      mbar_expect_tx(q_full, 2 * L::kTileBytes);
#pragma unroll
      for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int b = 0; b < kBoxes; ++b)
          tma_load_3d(smem + L::kQ + q * L::kTileBytes + b * kBoxBytes, &tmap_q, q_full, b * 64, m0 + q * BM, bh);
      int kt = 0, vt = 0;  // K / V tiles loaded so far (K is streamed once per pass)
      bool ok = true;
      for (int pass = first_pass; pass < 2 && ok; ++pass) {
        for (int j = 0; j < n_max; ++j) {
          const int ks = kt % kStagesKV;
          if (!mbar_wait(&k_empty[ks], ((kt / kStagesKV) & 1) ^ 1, abort_flag, p.status, ST_ATTN_KV)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&k_full[ks], L::kTileBytes);
#pragma unroll
          for (int b = 0; b < kBoxes; ++b)
            tma_load_3d(smem + L::kK + ks * L::kTileBytes + b * kBoxBytes, &tmap_k, &k_full[ks], b * 64, j * BN, bh);
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
            tma_load_3d(smem + L::kV + vs * L::kTileBytes + b * kBoxBytes, &tmap_v, &v_full[vs], b * 64, j * BN, bh);
          ++vt;
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_max > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(BM, BN, BF16, false, false);
      constexpr uint32_t idesc_o = umma_idesc_f16(BM, D, BF16, false, true);
      const uint32_t sq = smem_u32(smem + L::kQ), sk = smem_u32(smem + L::kK), sv = smem_u32(smem + L::kV);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_ATTN_Q);
      tc_fence_after_sync();

      // One thread issues every MMA, and a 128x128x16 MMA runs for only 64 clocks, so the
      // instruction count per issue matters: descriptors are built once per tile and the k16
      // slices only add a compile-time constant to the start-address field (low word).
      const uint64_t dq0 = umma_desc_kmajor_sw128(sq), dq1 = umma_desc_kmajor_sw128(sq + L::kTileBytes);
      const uint64_t dk0 = umma_desc_kmajor_sw128(sk), dk1 = umma_desc_kmajor_sw128(sk + L::kTileBytes);
      const uint64_t dv0 = umma_desc_mnmajor_sw128(sv, kBoxBytes, 1024);
      const uint64_t dv1 = umma_desc_mnmajor_sw128(sv + L::kTileBytes, kBoxBytes, 1024);
      auto issue_s = [&](int q, int stage) {
        const uint32_t d_tmem = tmem_base + q * 128;
        const uint64_t da = q ? dq1 : dq0, db = stage ? dk1 : dk0;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk / 4) * kBoxBytes + (kk % 4) * 32) >> 4);
          umma_f16_ss(d_tmem, da + off, db + off, idesc_s, kk != 0);
        }
        umma_commit(&s_full[q]);
      };
      int v_waited = 0;  // V tiles [0, v_waited) are known to have landed
      auto ensure_v = [&](int j) {
        while (ok && v_waited <= j) {
          ok = mbar_wait(&v_full[v_waited % kStagesKV], (v_waited / kStagesKV) & 1, abort_flag, p.status,
                         ST_ATTN_KV);
          ++v_waited;
        }
        tc_fence_after_sync();
      };

      // O_q += P_q(j) . V(j).  The softmax group publishes P in two halves (64 keys each), so
      // the first four k16 slices start while the second half is still being exponentiated.
      int pass_index = 0;       // 0 for the first pass that runs, 1 for the second
      bool stats_pass = false;  // the pass that only gathers statistics issues no P.V
      auto issue_pv = [&](int q, int stage, int j) {
        const uint32_t d_tmem = tmem_base + 256 + q * 128;
        const uint32_t a_tmem = tmem_base + q * 128;  // P_q: 8 columns per k16 slice
        const uint64_t dv = stage ? dv1 : dv0;
        const uint32_t parity = (pass_index * nq[q] + j) & 1;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          // in the statistics pass this only learns that the softmax group is done with S_q
          if (ok) ok = mbar_wait(half ? &p_ready_hi[q] : &p_ready[q], parity, abort_flag, p.status, ST_ATTN_P);
          if (stats_pass) continue;
          if (half == 0) ensure_v(j);
          if (!ok) return;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = half * 4; kk < half * 4 + 4; ++kk)
            umma_f16_ts(d_tmem, a_tmem + kk * 8, dv + static_cast<uint64_t>((kk * 2048) >> 4), idesc_o,
                        (j | kk) != 0);
        }
        if (!stats_pass) umma_commit(&o_done[q]);
      };

      for (int pass = first_pass; pass < 2 && ok; ++pass, ++pass_index) {
        stats_pass = pass == 0;
        const int kbase = pass_index * n_max;  // K tiles consumed by the earlier pass
        for (int j = 0; j < n_max && ok; ++j) {
          const int stage = (kbase + j) % kStagesKV;  // K stage; V tiles only exist in the last pass: stage j % 2
          ok = mbar_wait(&k_full[stage], ((kbase + j) / kStagesKV) & 1, abort_flag, p.status, ST_ATTN_KV);
          if (!ok) break;
          tc_fence_after_sync();
          if (j < nq[0]) issue_s(0, stage);
          if (j >= 1 && j - 1 < nq[1]) {  // O1 += P1(j-1) . V(j-1)
            issue_pv(1, (j - 1) % kStagesKV, j - 1);
            if (!ok) break;
          }
          if (j >= 1 && !stats_pass) umma_commit(&v_empty[(j - 1) % kStagesKV]);  // both P.V of tile j-1 are issued
          if (j < nq[1]) issue_s(1, stage);
          umma_commit(&k_empty[stage]);  // both S of tile j are issued
          if (j < nq[0]) {               // O0 += P0(j) . V(j)
            issue_pv(0, j % kStagesKV, j);
            if (!ok) break;
          }
        }
        if (ok && n_max >= 1) {
          const int j = n_max - 1;
          if (j < nq[1]) issue_pv(1, j % kStagesKV, j);
          if (ok && !stats_pass) umma_commit(&v_empty[j % kStagesKV]);
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    // ------------------------------------------------------------------ softmax groups
    const int q = warp >> 2;         // query tile of this group
    const int quad = warp & 3;       // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;
    const int n_tiles = nq[q];
    const int m_tile = m0 + q * BM;
    const int g_row = m_tile + row;  // query index within the head
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_s = tmem_base + q * 128 + lane_addr;
    const uint32_t t_o = tmem_base + 256 + q * 128 + lane_addr;
    const int off = p.S_kv - p.S_q;

    float m_ref = -INFINITY;  // reference maximum (scaled, log2 units) the stored P and O are relative to
    float l_sum = 0.f;
    bool ok = true;

    if (NORM) {
      // The reference's semantics (benchmark/layout/execution/tiled_attention.py:697-698,
      // tail_attention_reference.py:74-78): score = fp32(dot) * scale; subtract the maximum of the
      // WHOLE row; e = ex2((score - max) * log2e); p = e / (sum of e over the whole row), IEEE
      // division; p rounded to 16 bits; then P.V.  Pass 0 finds max and sum, pass 1 forms P.
      const float kLog2e = 1.44269504088896340736f;
      float m_run = -INFINITY, l_run = 0.f;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < n_tiles; ++j) {
          if (!mbar_wait(&s_full[q], (pass * n_tiles + j) & 1, abort_flag, p.status, ST_ATTN_S)) {
            ok = false;
            break;
          }
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
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(&s_full[q], j & 1, abort_flag, p.status, ST_ATTN_S)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, sr[c]);
      tmem_ld_wait();

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
      // row maximum: four independent chains of three-input max
      float mxc[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        mxc[c] = max3f(__uint_as_float(sr[c][0]), __uint_as_float(sr[c][1]), __uint_as_float(sr[c][2]));
#pragma unroll
        for (int i = 3; i + 1 < 32; i += 2)
          mxc[c] = max3f(mxc[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
        mxc[c] = fmaxf(mxc[c], __uint_as_float(sr[c][31]));
      }
      const float mx = max3f(mxc[0], mxc[1], fmaxf(mxc[2], mxc[3]));
      float m_new = fmaxf(m_ref, mx * p.scale_log2);
      if (m_new == -INFINITY) m_new = 0.f;  // a row that sees no key yet: keep everything finite

      // lazy rescale: warp-uniform decision because the TMEM accesses are warp-collective
      const bool grow = (j > 0) && (m_new - m_ref > kRescaleThreshold);
      if (j == 0) {
        m_ref = m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        const float factor = ex2f(m_ref - m_new);
        m_ref = m_new;
        l_sum *= factor;
        // O_q must be complete up to tile j-1 before it is scaled
        if (!mbar_wait(&o_done[q], (j - 1) & 1, abort_flag, p.status, ST_ATTN_O)) {
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

      // P = 2^(s*scale_log2 - m_ref) with packed fp32 FMAs, row sum in fp32 (two packed
      // accumulators), P rounded to 16 bits and written back over S chunk by chunk
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 negm2 = make_float2(-m_ref, -m_ref);
      float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 x = fma2(make_float2(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), scale2, negm2);
          float2 e = make_float2(ex2f(x.x), ex2f(x.y));
          if (i & 1) sum_b = add2(sum_b, e); else sum_a = add2(sum_a, e);
          pk[i] = pack16<BF16>(e.x, e.y);
        }
        tmem_st_32x32b_x16(t_s + c * 16, pk);
        if (c & 1) {  // a half of P (64 keys) is complete: let the MMA warp start on it
          tmem_st_wait();
          tc_fence_before_sync();
          mbar_arrive(c == 1 ? &p_ready[q] : &p_ready_hi[q]);
        }
      }
      sum_a = add2(sum_a, sum_b);
      l_sum += sum_a.x + sum_a.y;
    }

    // ---- epilogue: O / l
    if (ok && n_tiles > 0 && mbar_wait(&o_done[q], (n_tiles - 1) & 1, abort_flag, p.status, ST_ATTN_O)) {
      tc_fence_after_sync();
      const float inv = 1.0f / l_sum;
      const bool valid = g_row < p.S_q;
      const size_t row_off = ((size_t)bh * p.S_q + (size_t)min(g_row, p.S_q - 1)) * D;
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
          } else {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.O) + row_off + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack16<BF16>(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
              v.y = pack16<BF16>(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
              v.z = pack16<BF16>(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
              v.w = pack16<BF16>(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
              dst[i] = v;
            }
          }
        }
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
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
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
  if (rc) {
    ctx->last_cuda = rc;
    return FRISK_B200_E_CUDA;
  }
  AttnParams p;
  p.S_q = d.S_q;
  p.S_kv = d.S_kv;
  p.n_pairs = (d.S_q + 2 * BM - 1) / (2 * BM);
  p.causal = d.causal ? 1 : 0;
  p.total_ctas = (int64_t)p.n_pairs * bh;
  p.scale_log2 = d.scale * 1.4426950408889634f;
  p.scale = d.scale;
  p.normalized = d.normalize_p ? 1 : 0;
  p.O = O;
  p.status = ctx->d_status;
  if (p.total_ctas > INT32_MAX) return FRISK_B200_E_ATTN_SHAPE;
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
  kern<<<(unsigned)p.total_ctas, kThreads, L::kTotal, s>>>(tq, tk, tv, p);
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
