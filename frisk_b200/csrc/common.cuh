// Shared host-side declarations of libfrisk_b200: the context, error helpers and the
// per-kernel launch functions that api.cu dispatches to.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/frisk_b200.h"

namespace fb {

constexpr int kNumSMsDefault = 148;

struct StagingBuffer {
  void* ptr = nullptr;
  size_t bytes = 0;
};

// One encoded TMA descriptor and everything that determined it.  The context keeps the most
// recently used ones, so a caller that launches the same operands again (the normal case: a
// weight matrix, a preallocated activation buffer) pays the driver's encode call once.
struct TmapKey {
  const void* base;
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  int dtype, rank, swizzle;
  bool operator==(const TmapKey& o) const {
    return base == o.base && dtype == o.dtype && rank == o.rank && swizzle == o.swizzle && dims[0] == o.dims[0] &&
           dims[1] == o.dims[1] && dims[2] == o.dims[2] && strides[0] == o.strides[0] && strides[1] == o.strides[1] &&
           box[0] == o.box[0] && box[1] == o.box[1] && box[2] == o.box[2];
  }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  uint64_t stamp;
};
constexpr size_t kTmapCacheEntries = 64;
constexpr int kMaxDevices = 64;

// Per-kernel set-up that has to happen once per device (opting in to large dynamic shared
// memory, an occupancy query): `run` returns 0 on success, and then never runs again for
// that device.  Two threads may both run it the first time; the calls are idempotent.
struct PerDeviceOnce {
  std::atomic<int> done[kMaxDevices] = {};
  template <typename F>
  int operator()(int device, F&& run) {
    if (device < 0 || device >= kMaxDevices) return run();
    if (done[device].load(std::memory_order_acquire)) return 0;
    const int rc = run();
    if (rc == 0) done[device].store(1, std::memory_order_release);
    return rc;
  }
};

}  // namespace fb

struct frisk_b200_ctx {
  int device = 0;
  int num_sms = fb::kNumSMsDefault;
  int last_cuda = 0;
  int last_status = 0;
  uint64_t ws_signature = 0;     // layout of the control words last left in stage[3]
  unsigned* d_status = nullptr;  // device status word (first failing wait records its code)
  unsigned* h_status = nullptr;  // pinned mirror
  // staging for the *_host entry points and library-owned workspace
  fb::StagingBuffer stage[11];  // 0-2 A/B/C staging, 3 skinny scratch, 4 V staging, 5 GEMM tail scratch, 6 row partials,
                                // 7 fp32 stream-K scratch, 8-10 fp32-on-tensor-cores: stacked A, stacked B, 3M x 3N product
  cudaStream_t host_stream = nullptr;
  cudaStream_t copy_stream = nullptr;
  cudaStream_t out_stream = nullptr;
  cudaEvent_t ev[24] = {};
  std::recursive_mutex mu;  // recursive: the *_host entries hold it while a launcher takes it for its scratch
  std::mutex tmap_mu;
  std::vector<fb::TmapEntry> tmaps;  // encoded TMA descriptors, most recently used (see TmapKey)
  uint64_t tmap_clock = 0;
};

namespace fb {

inline size_t dtype_size(int dt) { return dt == FRISK_B200_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == FRISK_B200_F32 || dt == FRISK_B200_F16 || dt == FRISK_B200_BF16; }

#define FB_CUDA(ctx, expr)                          \
  do {                                              \
    cudaError_t e__ = (expr);                       \
    if (e__ != cudaSuccess) {                       \
      if (ctx) (ctx)->last_cuda = (int)e__;         \
      return FRISK_B200_E_CUDA;                     \
    }                                               \
  } while (0)

// Makes `device` current for the duration of an entry point and puts the caller's device back
// when it returns, so that a call never changes the calling thread's current device.
class DeviceGuard {
 public:
  explicit DeviceGuard(int device) {
    err_ = cudaGetDevice(&prev_);
    if (err_ == cudaSuccess && prev_ != device) {
      err_ = cudaSetDevice(device);
      switched_ = err_ == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (switched_) cudaSetDevice(prev_);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;
  cudaError_t error() const { return err_; }

 private:
  int prev_ = 0;
  bool switched_ = false;
  cudaError_t err_ = cudaSuccess;
};
#define FB_DEVICE(ctx)                   \
  fb::DeviceGuard device_guard__((ctx)->device); \
  FB_CUDA(ctx, device_guard__.error())

// resolved leading dimensions (elements)
struct GemmDims {
  int64_t M, N, K, lda, ldb, ldc;
};
inline GemmDims resolve_dims(const frisk_b200_gemm_desc& d) {
  GemmDims g{d.M, d.N, d.K, d.lda, d.ldb, d.ldc};
  if (g.lda == 0) g.lda = d.trans_a ? d.M : d.K;
  if (g.ldb == 0) g.ldb = d.trans_b ? d.K : d.N;
  if (g.ldc == 0) g.ldc = d.N;
  return g;
}

// ---- byte extents of the operands, for the output-overlaps-input refusal every entry makes
inline bool ranges_overlap(const void* a, size_t an, const void* b, size_t bn) {
  uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
  return a0 < b0 + bn && b0 < a0 + an;
}

inline size_t operand_bytes(int64_t rows, int64_t cols, int64_t ld, size_t es) {
  if (rows <= 0) return 0;
  return (size_t)((rows - 1) * ld + cols) * es;
}

struct GemmExtents {
  size_t a, b, c;
};
inline GemmExtents gemm_extents(const frisk_b200_gemm_desc& d) {
  GemmDims g = resolve_dims(d);
  size_t es = dtype_size(d.dtype_ab), cs = dtype_size(d.dtype_c);
  GemmExtents e;
  e.a = d.trans_a ? operand_bytes(g.K, g.M, g.lda, es) : operand_bytes(g.M, g.K, g.lda, es);
  e.b = d.trans_b ? operand_bytes(g.N, g.K, g.ldb, es) : operand_bytes(g.K, g.N, g.ldb, es);
  e.c = operand_bytes(g.M, g.N, g.ldc, cs);
  return e;
}


// ---- kernel launchers (one per .cu file) --------------------------------------------
int launch_gemm_simt_f32(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const float* A, const float* B,
                         float* C, cudaStream_t s);
// fp32 GEMM as nine bf16 tensor-core products of exactly split operands (gemm_f32_split.cu)
bool f32_split_supported(const frisk_b200_gemm_desc& d);
bool f32_split_preferred(const frisk_b200_gemm_desc& d);
int launch_gemm_f32_split(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const float* A, const float* B,
                          float* C, cudaStream_t s);

// Decode-shape GEMM (gemm_skinny.cu).  Its scratch begins with one ticket per 128-column tile; the
// kernel leaves them at zero, so they need clearing only when the scratch was last used with
// another layout (another kernel's partial sums may lie where this one keeps tickets):
// skinny_control_bytes is the size of that prefix and also identifies the layout.
size_t skinny_workspace_bytes(const frisk_b200_gemm_desc& d);
size_t skinny_control_bytes(const frisk_b200_gemm_desc& d);
bool skinny_supported(const frisk_b200_gemm_desc& d);
// `ctx` may be NULL (the entry that allocates nothing has no context): `status` then names the
// device word in which a wait that ran out is recorded.
int launch_gemm_skinny(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B, void* C,
                       void* ws, size_t ws_bytes, cudaStream_t s, unsigned* status = nullptr);

bool tcgen05_supported(const frisk_b200_gemm_desc& d);
int launch_gemm_tcgen05(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                        void* C, cudaStream_t s);

// Row blocks of the fp32 product are stored into up to 8 destination buffers instead of C:
// destination i receives rows [i*rows_per_target, (i+1)*rows_per_target) (it may be a peer
// GPU's memory, reached with plain stores over NVLink; never with TMA).
struct PushTargets {
  float* ptr[8];
  int n;                 // 0 = ordinary store to C
  int rows_per_target;
  int64_t ld;            // row pitch of every destination, in elements
};
// What the pair kernel does with a finished tile besides storing it (frisk.fill before, frisk.reduce
// along dim 1 after the gemm, on the same C).
struct EpilogueArgs {
  int has_fill;         // C_in is the constant `fill`; C is not read
  float fill;           // already rounded to C's element type
  int reduce_kind;      // FRISK_B200_REDUCE_*; over the ROUNDED values that are stored
  float* row_partials;  // [column tiles of 256][M] fp32, one partial per (tile column, row)
};
bool tcgen05_2cta_preferred(const frisk_b200_gemm_desc& d);
int launch_gemm_tcgen05_2cta_push(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                                  const PushTargets& push, cudaStream_t s);
int launch_sum_slots(const float* slots, int n_slots, int64_t slot_elems, void* dst, int64_t n, int dtype,
                     cudaStream_t s);
// scratch for the K-split tail wave (0 when every tile runs whole); tickets at its start must be zero
size_t tcgen05_2cta_workspace_bytes(const frisk_b200_gemm_desc& d);
int launch_gemm_tcgen05_2cta(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc& d, const void* A, const void* B,
                             void* C, void* ws, size_t ws_bytes, cudaStream_t s, const EpilogueArgs* epi = nullptr);
int tcgen05_2cta_column_tiles(const frisk_b200_gemm_desc& d);
// epilogue.cu
int launch_row_finalize(const float* partials, int tiles_n, int64_t M, int kind, int clear, void* dst, int dtype,
                        cudaStream_t s);
int launch_row_reduce(const void* C, int64_t M, int64_t N, int64_t ldc, int kind, int clear, void* dst, int dtype,
                      cudaStream_t s);
int launch_fill(void* C, int64_t M, int64_t N, int64_t ldc, float value, int dtype, cudaStream_t s);

int launch_attention_fwd(frisk_b200_ctx* ctx, const frisk_b200_attn_desc& d, const void* Q, const void* K,
                         const void* V, void* O, cudaStream_t s);

int launch_convert_f32(const float* src, void* dst, int64_t n, int dtype, cudaStream_t s);

// TMA descriptors, encoded through the driver entry point (no link-time libcuda dependency) and
// kept in the context's cache (ctx may be NULL: encode without caching)
int encode_tmap_2d(frisk_b200_ctx* ctx, CUtensorMap* out, int dtype, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                   bool swizzle128);
int encode_tmap_3d(frisk_b200_ctx* ctx, CUtensorMap* out, int dtype, const void* base, uint64_t d0, uint64_t d1,
                   uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                   uint32_t b2, bool swizzle128);

}  // namespace fb
