// fp32 GEMM on the CUDA cores: C <- (clear_accum ? 0 : C) + op(A).op(B), fp32 throughout.
// Contract: `frisk.gemm` with f32 operands (lib/Dialect/Frisk/IR/FriskOps.cpp:406-426).
//
// One CTA of 256 threads per SM computes 64x64 output tiles.  The CTA is four "k-groups" of two
// warps; a pipeline stage holds 64 k of the A and B tiles in shared memory ([k][m] and [k][n],
// whichever way the operand lies in global memory) and k-group g multiplies rows [16g, 16g+16) of
// it, every thread owning an 8x8 register tile (two 4-row groups x two 4-column groups: the 32
// lanes of a 128-bit fragment read touch at most 128 distinct bytes, which the shared memory
// delivers in one cycle).  The four partial tiles are added through shared memory when a tile's
// k range ends.  Small CTA tiles keep the tile count above the SM count for the small problems
// this path serves; one CTA per SM leaves each thread up to 255 registers, so the next stage's
// operand fetches and the next k-step's fragments stay in flight across the multiply.
//
// Work is split stream-K style: unit = (tile, k-stage); the units are numbered tile-major and
// worker c takes the contiguous range [start(c), start(c+1)), so every SM multiplies the same
// number of k-stages whatever the tile count.  A tile whose k range is shared is finished by
// whichever contributor draws the last ticket: each contributor leaves its partial tile in its
// own slot, and the finisher adds the slots IN CONTRIBUTOR ORDER (bitwise reproducible).  No CTA
// waits for another.  A worker does its shared segments first and its whole tiles last, so
// the hand-over is not at the end of the kernel.
#include <type_traits>

#include "common.cuh"

namespace fb {
namespace {

constexpr int BT = 64;                 // tile edge (rows and columns)
constexpr int kTileFloats = BT * BT;   // 4096
constexpr int kMaxStreamTiles = 16384;  // tickets held by the context's scratch

template <int KG, int BKS_>
struct Cfg {
  static constexpr int NT = 64 * KG;       // threads
  static constexpr int BKS = BKS_;         // k per stage
  static constexpr int KPG = BKS / KG;     // k per k-group and stage
  static constexpr int kVec = BKS * BT / 4 / NT;                    // float4 per thread, operand and stage
  static constexpr int kStageFloats = 2 * BKS * BT;                 // A part then B part
  static constexpr int kRedFloats = KG * kTileFloats;               // reduction area
  static constexpr int kSmemFloats = kRedFloats > 2 * kStageFloats ? kRedFloats : 2 * kStageFloats;
  static constexpr int kEpi = kTileFloats / 4 / NT;                 // float4 per thread in the epilogue
  static_assert(BKS % KG == 0 && KPG % 4 == 0 && BKS % (NT / 16) == 0, "stage must split evenly");
};

struct Partition {
  unsigned q, r;        // W = G*q + r units: workers 0..r-1 take q+1, the rest q
  unsigned kb;          // k-stages per tile
  unsigned tiles_n;     // tiles along N
  __host__ __device__ unsigned start(unsigned c) const { return c * q + (c < r ? c : r); }
  __device__ unsigned worker_of(unsigned u) const {
    unsigned big = r * (q + 1);
    return u < big ? u / (q + 1) : r + (u - big) / q;
  }
};

// One operand's share of a stage per thread (kVec float4), fetched early and stored (transposed if
// the operand is contiguous along K) after the current stage has been multiplied.
// KContig: global buffer contiguous along K (A non-transposed, B transposed).  Then a warp reads
// 4 rows x 128 contiguous bytes per instruction (lane = row * 8 + k chunk) and scatters the four
// floats of each chunk to rows 4*kc..4*kc+3 of the [k][mn] image; element (k, mn) lives at column
// mn ^ 4*(k/4), which makes the scatter free of bank conflicts (8 chunk lanes -> 8 bank groups, 4
// row lanes -> 4 banks inside a group) and keeps 16-byte groups of mn together for the readers.
template <class C, bool KContig>
struct StageLoader {
  static_assert(C::BKS == 64 && C::NT == 256, "the K-contiguous mapping below is written for 64 k and 8 warps");
  float4 reg[C::kVec];
  const float* base;   // this thread's first element of the stage the fast path loads next
  int64_t step32;      // K-contiguous: 32 rows further; otherwise: 16 k further

  // k0: first k of the stage the next load_fast() fetches
  __device__ __forceinline__ void begin(const float* __restrict__ g, int64_t ld, int mn0, int k0, int tid) {
    if (KContig) {
      base = g + (int64_t)(mn0 + (tid >> 5) * 4 + ((tid & 31) >> 3)) * ld + k0 + 4 * (tid & 7);
      step32 = 32 * ld;
    } else {
      base = g + (int64_t)(k0 + (tid >> 4)) * ld + mn0 + (tid & 15) * 4;
      step32 = 16 * ld;
    }
  }
  // whole stage inside the operand, 16-byte aligned rows: no bounds logic
  __device__ __forceinline__ void load_fast() {
    if (KContig) {
      reg[0] = __ldg(reinterpret_cast<const float4*>(base));
      reg[1] = __ldg(reinterpret_cast<const float4*>(base + step32));
      reg[2] = __ldg(reinterpret_cast<const float4*>(base + 32));
      reg[3] = __ldg(reinterpret_cast<const float4*>(base + step32 + 32));
      base += C::BKS;
    } else {
#pragma unroll
      for (int v = 0; v < C::kVec; ++v) reg[v] = __ldg(reinterpret_cast<const float4*>(base + v * step32));
      base += 4 * step32;
    }
  }
  __device__ __forceinline__ void skip() { base += KContig ? (int64_t)C::BKS : 4 * step32; }

  __device__ __forceinline__ void load(const float* __restrict__ g, int64_t ld, int mn0, int k0, int ext_mn,
                                       int ext_k, bool vec_ok, int tid) {
    skip();
    if (KContig) {
      const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
      for (int v = 0; v < C::kVec; ++v) {
        const int mn = mn0 + warp * 4 + (lane >> 3) + 32 * (v & 1);
        const int kk = k0 + 4 * ((lane & 7) + 8 * (v >> 1));
        const float* p = g + (int64_t)mn * ld + kk;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (mn < ext_mn) {
          if (vec_ok && kk + 3 < ext_k) {
            val = __ldg(reinterpret_cast<const float4*>(p));
          } else {
            if (kk + 0 < ext_k) val.x = __ldg(p + 0);
            if (kk + 1 < ext_k) val.y = __ldg(p + 1);
            if (kk + 2 < ext_k) val.z = __ldg(p + 2);
            if (kk + 3 < ext_k) val.w = __ldg(p + 3);
          }
        }
        reg[v] = val;
      }
    } else {
      // thread -> four mn at (tid % 16) * 4, rows k = tid / 16 + v * (NT / 16)
      const int mn = mn0 + (tid & 15) * 4;
#pragma unroll
      for (int v = 0; v < C::kVec; ++v) {
        const int k = k0 + (tid >> 4) + v * (C::NT / 16);
        const float* p = g + (int64_t)k * ld + mn;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < ext_k) {
          if (vec_ok && mn + 3 < ext_mn) {
            val = __ldg(reinterpret_cast<const float4*>(p));
          } else {
            if (mn + 0 < ext_mn) val.x = __ldg(p + 0);
            if (mn + 1 < ext_mn) val.y = __ldg(p + 1);
            if (mn + 2 < ext_mn) val.z = __ldg(p + 2);
            if (mn + 3 < ext_mn) val.w = __ldg(p + 3);
          }
        }
        reg[v] = val;
      }
    }
  }
  // s: this operand's part of a stage, [BKS][64] floats
  __device__ __forceinline__ void store(float* s, int tid) const {
    if (KContig) {
      const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
      for (int v = 0; v < C::kVec; ++v) {
        const int mn = warp * 4 + (lane >> 3) + 32 * (v & 1);
        const int kc = (lane & 7) + 8 * (v >> 1);
        float* q = s + (4 * kc) * BT + (mn ^ (4 * kc));
        q[0 * BT] = reg[v].x;
        q[1 * BT] = reg[v].y;
        q[2 * BT] = reg[v].z;
        q[3 * BT] = reg[v].w;
      }
    } else {
#pragma unroll
      for (int v = 0; v < C::kVec; ++v)
        *reinterpret_cast<float4*>(s + ((tid >> 4) + v * (C::NT / 16)) * BT + (tid & 15) * 4) = reg[v];
    }
  }
};

struct SimtArgs {
  const float* A;
  const float* B;
  float* C;
  int M, N, K;
  int64_t lda, ldb, ldc;
  int accumulate, vec_a, vec_b, vec_c;
  Partition part;
  unsigned* tickets;   // one per tile, zero between launches
  float4* slots;       // two partial tiles per worker
};

struct Segment {
  unsigned tile, kb0, kb1;
  int m0, n0;
  bool fast;  // whole tile inside the operands and 16-byte aligned rows
};

template <bool TA, bool TB, class C>
__global__ void __launch_bounds__(C::NT, 1) gemm_simt_f32_kernel(const SimtArgs p) {
  constexpr int NT = C::NT, BKS = C::BKS, KG = C::NT / 64, KPG = C::KPG;
  extern __shared__ __align__(16) float smem[];
  __shared__ unsigned s_ticket;

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int grp = warp >> 1;            // k-group
  const int wm = (warp & 1) * 32;       // the warp's 32 rows of the tile
  const int ty = lane >> 3, tx = lane & 7;
  // fragment offsets inside a stage row
  const int a_off = wm + ty * 4;        // rows a_off..+3 and a_off+16..+19
  const int b_off = tx * 4;             // columns b_off..+3 and b_off+32..+35

  // fragment read pointers into the current buffer, one pair per group of four k: a K-contiguous operand was
  // stored with its 16-byte column groups permuted by the row's k/4 (see StageLoader)
  const float* fa[KPG / 4][2];
  const float* fb[KPG / 4][2];
#pragma unroll
  for (int j = 0; j < KPG / 4; ++j) {
    const int swa = !TA ? 4 * (grp * (KPG / 4) + j) : 0;
    const int swb = TB ? 4 * (grp * (KPG / 4) + j) : 0;
    const float* rows = smem + (grp * KPG) * BT;
    fa[j][0] = rows + (a_off ^ swa);
    fa[j][1] = rows + ((a_off + 16) ^ swa);
    fb[j][0] = rows + BKS * BT + (b_off ^ swb);
    fb[j][1] = rows + BKS * BT + ((b_off + 32) ^ swb);
  }
  // invariant between stages: the fragment pointers address the current buffer, `store_to` the other one,
  // `flip` = other - current
  float* store_to = smem + C::kStageFloats;
  int flip = C::kStageFloats;

  const Partition part = p.part;
  const unsigned kb = part.kb;
  const unsigned w_begin = part.start(blockIdx.x), w_end = part.start(blockIdx.x + 1);
  if (w_begin >= w_end) return;
  const unsigned t0 = w_begin / kb, t1 = (w_end - 1) / kb;
  const bool tail_partial = w_end != (t1 + 1) * kb;

  // segment list: shared tail segment, then the head segment (shared or not), then whole tiles
  const unsigned first_whole = t0 + 1, last_whole = (tail_partial || t1 == t0) ? (t1 == t0 ? t0 : t1 - 1) : t1;
  const int n_pre = (t1 != t0 && tail_partial) ? 2 : 1;
  const int n_seg = n_pre + (last_whole >= first_whole ? (int)(last_whole - first_whole + 1) : 0);
  auto segment = [&](int seg) {
    Segment s;
    if (n_pre == 2 && seg == 0) {
      s.tile = t1; s.kb0 = 0; s.kb1 = w_end - t1 * kb;
    } else if (seg == n_pre - 1) {
      s.tile = t0; s.kb0 = w_begin - t0 * kb; s.kb1 = (t1 == t0 ? w_end - t0 * kb : kb);
    } else {
      s.tile = first_whole + (unsigned)(seg - n_pre); s.kb0 = 0; s.kb1 = kb;
    }
    s.m0 = (int)(s.tile / part.tiles_n) * BT;
    s.n0 = (int)(s.tile % part.tiles_n) * BT;
    s.fast = p.vec_a && p.vec_b && s.m0 + BT <= p.M && s.n0 + BT <= p.N;
    return s;
  };

  StageLoader<C, !TA> la;
  StageLoader<C, TB> lb;
  // stage ks of segment s into registers; stages that are whole in K and inside the operands skip the bounds logic
  auto fetch = [&](const Segment& s, unsigned ks) {
    if (s.fast && (int)(ks + 1) * BKS <= p.K) {
      la.load_fast();
      lb.load_fast();
    } else {
      la.load(p.A, p.lda, s.m0, (int)ks * BKS, p.M, p.K, p.vec_a, tid);
      lb.load(p.B, p.ldb, s.n0, (int)ks * BKS, p.N, p.K, p.vec_b, tid);
    }
  };
  auto first_fetch = [&](const Segment& s) {
    la.begin(p.A, p.lda, s.m0, (int)s.kb0 * BKS, tid);
    lb.begin(p.B, p.ldb, s.n0, (int)s.kb0 * BKS, tid);
    fetch(s, s.kb0);
  };

  asm volatile("griddepcontrol.wait;" ::: "memory");  // operands and scratch of the kernel before this one
  Segment cur = segment(0);
  first_fetch(cur);

  for (int seg = 0; seg < n_seg; ++seg) {
    const bool whole = cur.kb0 == 0 && cur.kb1 == kb;
    Segment nxt = cur;
    if (seg + 1 < n_seg) nxt = segment(seg + 1);

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    __syncthreads();  // the reduction area of the previous segment is free
    la.store(store_to - flip, tid);
    lb.store(store_to - flip + BKS * BT, tid);
    __syncthreads();

    // one stage per iteration: fetch the next one (of this segment, or the first of the next segment), multiply
    // this one out of the current buffer, store the next one into the other buffer
#pragma unroll 1
    for (unsigned ks = cur.kb0; ks < cur.kb1; ++ks) {
      const bool more = ks + 1 < cur.kb1;
      if (more) fetch(cur, ks + 1);
      else if (seg + 1 < n_seg) first_fetch(nxt);
#pragma unroll
      for (int k = 0; k < KPG; ++k) {
        const float4 a0 = *reinterpret_cast<const float4*>(fa[k >> 2][0] + k * BT);
        const float4 a1 = *reinterpret_cast<const float4*>(fa[k >> 2][1] + k * BT);
        const float4 b0 = *reinterpret_cast<const float4*>(fb[k >> 2][0] + k * BT);
        const float4 b1 = *reinterpret_cast<const float4*>(fb[k >> 2][1] + k * BT);
        const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      if (more) {
        la.store(store_to, tid);
        lb.store(store_to + BKS * BT, tid);
      }
      // the other buffer becomes the current one (also after the last stage: the next segment's first stage
      // goes into whichever buffer is then current)
#pragma unroll
      for (int j = 0; j < KPG / 4; ++j) {
        fa[j][0] += flip; fa[j][1] += flip; fb[j][0] += flip; fb[j][1] += flip;
      }
      store_to -= flip;
      flip = -flip;
      __syncthreads();
    }
    if (seg + 1 == n_seg) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // the KG partial tiles meet in shared memory: group g writes red[g][64][64]
    {
      float* red = smem + grp * kTileFloats;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = a_off + (i >> 2) * 16 + (i & 3);
        *reinterpret_cast<float4*>(red + row * BT + b_off) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(red + row * BT + b_off + 32) =
            make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
    __syncthreads();
    float4 out[C::kEpi];
#pragma unroll
    for (int h = 0; h < C::kEpi; ++h) {
      const float4* r4 = reinterpret_cast<const float4*>(smem) + tid + h * NT;
      float4 sum = r4[0];
#pragma unroll
      for (int g = 1; g < KG; ++g) {
        const float4 v = r4[g * (kTileFloats / 4)];
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
      out[h] = sum;
    }

    bool finish = whole;
    if (!whole) {
      // leave the partial tile in this worker's slot (0: the segment that begins the range), take a ticket.
      // Release: every thread's stores, CTA barrier, then ONE fence and the ticket by thread 0 (the fence is
      // cumulative over what the barrier ordered before it); acquire the same way round.
      const unsigned slot = blockIdx.x * 2 + ((cur.tile * kb + cur.kb0 == w_begin) ? 0u : 1u);
      float4* dst = p.slots + (size_t)slot * (kTileFloats / 4);
#pragma unroll
      for (int h = 0; h < C::kEpi; ++h) __stcg(dst + tid + h * NT, out[h]);
      __syncthreads();
      const unsigned c_first = part.worker_of(cur.tile * kb), c_last = part.worker_of(cur.tile * kb + kb - 1);
      if (tid == 0) {
        __threadfence();
        unsigned old = atomicAdd(p.tickets + cur.tile, 1u);
        const bool last = old == c_last - c_first;
        if (last) {
          p.tickets[cur.tile] = 0;  // every contributor has drawn: clean for the next launch
          __threadfence();
        }
        s_ticket = last ? 1u : 0u;
      }
      __syncthreads();
      finish = s_ticket != 0;
      if (finish) {
#pragma unroll
        for (int h = 0; h < C::kEpi; ++h) out[h] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (unsigned c = c_first; c <= c_last; ++c) {
          const unsigned cslot = c * 2 + (part.start(c) >= cur.tile * kb ? 0u : 1u);
          const float4* src = p.slots + (size_t)cslot * (kTileFloats / 4);
          float4 v[C::kEpi];
#pragma unroll
          for (int h = 0; h < C::kEpi; ++h) v[h] = __ldcg(src + tid + h * NT);
#pragma unroll
          for (int h = 0; h < C::kEpi; ++h) {
            out[h].x += v[h].x; out[h].y += v[h].y; out[h].z += v[h].z; out[h].w += v[h].w;
          }
        }
      }
    }
    if (finish) {
#pragma unroll
      for (int h = 0; h < C::kEpi; ++h) {
        const int e = tid + h * NT;
        const int r = cur.m0 + (e >> 4), c = cur.n0 + (e & 15) * 4;
        if (r >= p.M || c >= p.N) continue;
        float* dst = p.C + (int64_t)r * p.ldc + c;
        float4 o = out[h];
        if (p.vec_c && c + 3 < p.N) {
          if (p.accumulate) {
            const float4 old = *reinterpret_cast<const float4*>(dst);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(dst) = o;
        } else {
          const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c + j < p.N) dst[j] = p.accumulate ? dst[j] + ov[j] : ov[j];
        }
      }
    }
    cur = nxt;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 256 threads, one CTA per SM, 64 k per stage: with up to 255 registers per thread the compiler keeps the
// next stage's operand fetches and the next k-step's fragments in flight across the multiply.
using SimtCfg = Cfg<4, 64>;

template <bool TA, bool TB>
int launch_one(frisk_b200_ctx* ctx, const SimtArgs& a, unsigned grid, cudaStream_t s) {
  static PerDeviceOnce once;
  constexpr int smem = SimtCfg::kSmemFloats * (int)sizeof(float);
  int rc = once(ctx->device, [&]() -> int {
    FB_CUDA(ctx, cudaFuncSetAttribute(gemm_simt_f32_kernel<TA, TB, SimtCfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      smem));
    return 0;
  });
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(SimtCfg::NT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits (griddepcontrol.wait) itself
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_simt_f32_kernel<TA, TB, SimtCfg>, a));
  FB_CUDA(ctx, cudaGetLastError());
  return 0;
}

}  // namespace

int launch_gemm_simt_f32(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const float* A, const float* B,
                         float* C, cudaStream_t s) {
  GemmDims g = resolve_dims(d);
  if (g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX) return FRISK_B200_E_UNSUPPORTED;
  const int64_t tiles_m = (g.M + BT - 1) / BT, tiles_n = (g.N + BT - 1) / BT;
  const int64_t tiles = tiles_m * tiles_n;
  const int64_t kb = std::max<int64_t>(1, (g.K + SimtCfg::BKS - 1) / SimtCfg::BKS);
  if (tiles <= 0 || tiles > (int64_t)1 << 30 || tiles * kb >= (int64_t)1 << 32) return FRISK_B200_E_UNSUPPORTED;

  // Few tiles: one worker per SM, k ranges shared (tickets + slots in context-owned scratch).  Many tiles:
  // one worker per tile, launched in tile order so that neighbours share operand panels in L2.
  const bool stream = tiles <= kMaxStreamTiles && tiles < (int64_t)ctx->num_sms * 16;
  const uint64_t W = (uint64_t)tiles * (uint64_t)kb;
  const unsigned G = stream ? (unsigned)std::min<uint64_t>(W, (uint64_t)ctx->num_sms) : (unsigned)tiles;

  SimtArgs a;
  a.A = A; a.B = B; a.C = C;
  a.M = (int)g.M; a.N = (int)g.N; a.K = (int)g.K;
  a.lda = g.lda; a.ldb = g.ldb; a.ldc = g.ldc;
  a.accumulate = d.clear_accum ? 0 : 1;
  a.vec_a = aligned16(A) && (g.lda % 4 == 0);
  a.vec_b = aligned16(B) && (g.ldb % 4 == 0);
  a.vec_c = aligned16(C) && (g.ldc % 4 == 0);
  a.part.q = (unsigned)(W / G);
  a.part.r = (unsigned)(W % G);
  a.part.kb = (unsigned)kb;
  a.part.tiles_n = (unsigned)tiles_n;
  a.tickets = nullptr;
  a.slots = nullptr;
  if (stream) {
    // scratch: tickets (zero between launches: the finisher of a tile clears its ticket), then two slots per SM
    const size_t ticket_bytes = (size_t)kMaxStreamTiles * sizeof(unsigned);
    const size_t need = ticket_bytes + (size_t)ctx->num_sms * 2 * kTileFloats * sizeof(float);
    std::lock_guard<std::recursive_mutex> lock(ctx->mu);
    StagingBuffer& b = ctx->stage[7];
    if (!b.ptr) {
      FB_CUDA(ctx, cudaMalloc(&b.ptr, need));
      b.bytes = need;
      FB_CUDA(ctx, cudaMemsetAsync(b.ptr, 0, ticket_bytes, s));
    }
    a.tickets = static_cast<unsigned*>(b.ptr);
    a.slots = reinterpret_cast<float4*>(static_cast<unsigned char*>(b.ptr) + ticket_bytes);
  }
  if (d.trans_a) return d.trans_b ? launch_one<true, true>(ctx, a, G, s) : launch_one<true, false>(ctx, a, G, s);
  return d.trans_b ? launch_one<false, true>(ctx, a, G, s) : launch_one<false, false>(ctx, a, G, s);
}

}  // namespace fb
