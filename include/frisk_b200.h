/*
 * libfrisk_b200 — C ABI of the B200 (sm_100a) GEMM / attention kernels that stand in
 * for the NVIDIA lowering of the Frisk dialect's `frisk.gemm` op and of its attention
 * graph.  Plain C: pointers and sizes only.  Device pointers are raw 64-bit device
 * addresses, as in the reference's launcher (benchmark/layout/execution/load_cubin.py:16,
 * run_execution.py:77).  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *
 * Return value of every int function: 0 = OK; negative = contract violation found on the
 * host before anything was launched (the reference raises ValueError at the same point,
 * ffi/ir.cpp:333-341, benchmark/layout/execution/async_host.py:4-10); positive = CUDA /
 * device-side status.  frisk_b200_strerror() turns a code into text whose prefix matches
 * the reference's message prefixes ("legacy-gemm-shape", "legacy-gemm-type").
 *
 * Ownership: the caller owns every operand buffer and the optional workspace; the
 * library owns only what hangs off the opaque context (cached TMA descriptors, staging
 * buffers of the *_host entry points).  Kernels launch on the caller's stream and never
 * synchronise, except the *_host entry points, which return after the result is in host
 * memory.  Inputs are read-only and may alias each other; the output must not overlap an
 * input (benchmark/layout/execution/tiled_execution.py:113-139).
 *
 * One context serves one stream of calls: the context holds scratch that its kernels share
 * (the attention kernel's work counter, the fp32 and skinny GEMMs' tickets and partial sums when
 * no workspace is passed, the device status word), so two calls on the same context must not
 * run on the GPU at the same time.  Use one context per concurrent stream.  Every entry point
 * leaves the calling thread's current device as it found it.
 */
#ifndef FRISK_B200_H
#define FRISK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct frisk_b200_ctx frisk_b200_ctx;

/* element types: the float types python/frisk/common/utils.py:156-170 can name */
enum { FRISK_B200_F32 = 0, FRISK_B200_F16 = 1, FRISK_B200_BF16 = 2 };

/* kernel selection for frisk_b200_gemm (AUTO picks by type and shape).  f32 operands: AUTO takes F32_SPLIT when
 * M, N and K are multiples of 8 and at least 256, else SIMT_F32.  F32_SPLIT and SIMT_F32 keep their scratch (stacked
 * bf16 operands and the 3M x 3N fp32 product; tickets and partial tiles) in the context, whatever `workspace` is. */
enum {
  FRISK_B200_ALGO_AUTO = 0,
  FRISK_B200_ALGO_SIMT_F32 = 1, /* fp32 CUDA-core GEMM                                   */
  FRISK_B200_ALGO_TCGEN05 = 2,  /* fp16/bf16 tcgen05 + TMEM + TMA ring, one CTA per tile */
  FRISK_B200_ALGO_SKINNY = 3,   /* M<=16: weights streamed by TMA into tcgen05, stream-K  */
  FRISK_B200_ALGO_TCGEN05_PAIR = 4, /* tcgen05 with CTA pairs (cta_group::2), 256x256 tiles */
  FRISK_B200_ALGO_F32_SPLIT = 5 /* fp32 operands split exactly into 3 bf16 terms, 9 tcgen05 products, fp32 sums */
};

/* error codes (negative: host-side contract checks) */
enum {
  FRISK_B200_OK = 0,
  FRISK_B200_E_GEMM_SHAPE = -1,    /* "legacy-gemm-shape: ..."  */
  FRISK_B200_E_GEMM_TYPE = -2,     /* "legacy-gemm-type: ..."   */
  FRISK_B200_E_ALIGN = -3,         /* pointer / pitch not 16-byte aligned                   */
  FRISK_B200_E_OVERLAP = -4,       /* output overlaps an input                              */
  FRISK_B200_E_WORKSPACE = -5,     /* workspace missing or too small                        */
  FRISK_B200_E_UNSUPPORTED = -6,   /* no kernel for this type / layout / algo combination   */
  FRISK_B200_E_ARG = -7,           /* null pointer, bad enum, bad context                   */
  FRISK_B200_E_ATTN_SHAPE = -8,    /* attention shape outside the launch contract           */
  FRISK_B200_E_TOO_LARGE = -9,     /* exceeds the fixed capacity of a no-allocation entry   */
  FRISK_B200_E_DEVICE_TIMEOUT = 1, /* a bounded device-side wait ran out (status word set)  */
  FRISK_B200_E_CUDA = 2            /* a CUDA runtime/driver call failed (see last_cuda)     */
};

/*
 * GEMM descriptor: the attributes of `frisk.gemm`
 * (include/Dialect/Frisk/IR/FriskOps.td:252-268: A, B, C, transA, transB, M, N, K, policy,
 * clear_accum) plus leading dimensions in ELEMENTS (0 = dense).
 * Buffers are dense row-major memrefs; transposes are flags, not strides
 * (lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:37-44):
 *   A buffer is [M,K] (trans_a=0) or [K,M] (trans_a=1)
 *   B buffer is [K,N] (trans_b=0) or [N,K] (trans_b=1)
 *   C buffer is [M,N].
 * C <- (clear_accum ? 0 : C) + op(A).op(B), fp32 accumulation, one rounding to dtype_c
 * (lib/Dialect/Frisk/IR/FriskOps.cpp:416-426).
 */
typedef struct frisk_b200_gemm_desc {
  int64_t M, N, K;
  int32_t trans_a, trans_b;
  int32_t clear_accum;
  int32_t dtype_ab; /* FRISK_B200_F32 / F16 / BF16: A and B share it */
  int32_t dtype_c;  /* == dtype_ab, or F32 for F16/BF16 inputs      */
  int64_t lda, ldb, ldc;
  int32_t policy; /* GemmWarpPolicy of the op; informational (kernels fix their own tiling) */
  int32_t algo;   /* FRISK_B200_ALGO_*                                                        */
} frisk_b200_gemm_desc;

/*
 * Attention-forward descriptor.  Q [B,H,S_q,D], K/V [B,H,S_kv,D], O [B,H,S_q,D], compact
 * BHSD (benchmark/layout/execution/tiled_attention.py:52-55).  O = softmax(scale * Q.K^T
 * [+ causal mask]).V with fp32 scores and statistics and P rounded to the 16-bit input
 * type before P.V (tiled_attention.py:628-629, tail_attention_reference.py:74-85).
 * causal: key j is visible to query i iff j <= i + S_kv - S_q.
 */
typedef struct frisk_b200_attn_desc {
  int32_t B, H, S_q, S_kv, D;
  float scale;
  int32_t causal;
  int32_t dtype_in;  /* F16 or BF16                      */
  int32_t dtype_out; /* == dtype_in, or F32              */
  /* 0: single pass, P rounded relative to a running maximum (fast path).
   * 1: the reference's semantics to the letter: two passes over the keys, every probability is
   *    divided by the COMPLETE row sum (IEEE division) before it is rounded to 16 bits
   *    (tiled_attention.py:697-698, tail_attention_reference.py:74-78); the reference's analytic
   *    fixtures then match bit for bit. */
  int32_t normalize_p;
} frisk_b200_attn_desc;

/* ---- context -------------------------------------------------------------------------
 * Replaces the reference's per-run module load (benchmark/layout/execution/load_cubin.py:6).
 * `device` is a CUDA ordinal; the context caches TMA descriptors and staging buffers. */
int frisk_b200_ctx_create(frisk_b200_ctx** out, int device);
int frisk_b200_ctx_destroy(frisk_b200_ctx* ctx);
/* Device status word of the last launch that was checked (0 = clean) and the last CUDA
 * error code seen by this context. */
int frisk_b200_last_status(frisk_b200_ctx* ctx);
int frisk_b200_last_cuda(frisk_b200_ctx* ctx);
const char* frisk_b200_strerror(int code);
const char* frisk_b200_version(void);

/* ---- GEMM ----------------------------------------------------------------------------
 * Host-only contract check: what ffi/ir.cpp:323-354 (create_gemm_op) does through
 * getLegacyGemmValidationError (lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:11-46).
 * Usable without a GPU. */
int frisk_b200_gemm_validate(const frisk_b200_gemm_desc* desc);
/* The same check over the memref SHAPES of the three operands, exactly the test
 * getLegacyGemmValidationError applies (rank 2, static (>= 0) extents, positive M/N/K,
 * A/B same type, C same type or f32 for f16/bf16, effective shapes match M/N/K, C is MxN).
 * `message`, when not NULL, receives the reference's message text (NULL when the check
 * passes).  Host-only. */
int frisk_b200_gemm_check_memrefs(int32_t a_rank, const int64_t* a_shape, int32_t a_dtype,
                                  int32_t b_rank, const int64_t* b_shape, int32_t b_dtype,
                                  int32_t c_rank, const int64_t* c_shape, int32_t c_dtype,
                                  int32_t trans_a, int32_t trans_b, int64_t m, int64_t n, int64_t k,
                                  const char** message);
/* Which kernel AUTO resolves to for this descriptor (FRISK_B200_ALGO_*), or a negative
 * error.  Host-only. */
int frisk_b200_gemm_select(const frisk_b200_gemm_desc* desc);
/* Bytes of caller-provided, ZERO-INITIALISED scratch this descriptor needs (0 = none).
 * The kernels leave their control words zero again, so one memset at allocation suffices
 * for repeated launches of the SAME descriptor; a scratch buffer that is reused with
 * another M/N/K must be zeroed again first (partial sums of the old shape may lie where
 * the new shape keeps control words).  Passing workspace = NULL to frisk_b200_gemm uses
 * scratch owned by the context, which does this bookkeeping itself; such calls must not
 * overlap on the GPU for one context. */
size_t frisk_b200_gemm_workspace_bytes(const frisk_b200_gemm_desc* desc);
/* Replaces the launch of the kernel the reference would have generated for a
 * `frisk.gemm` (benchmark/layout/execution/run_execution.py:84, load_cubin.py:18). */
int frisk_b200_gemm(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* desc, const void* A,
                    const void* B, void* C, void* workspace, size_t workspace_bytes,
                    void* stream);
/* Same op on HOST buffers: copies A, B (and C when it is read) to the device, runs, copies
 * C back and returns when C is valid.  The end-to-end path of the benchmark. */
int frisk_b200_gemm_host(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* desc, const void* A,
                         const void* B, void* C);
/* The decode-shape (M <= 16, trans_a = 0, trans_b = 1, fp16/bf16) GEMM for callers that must
 * not allocate device memory when they call: processes whose memory manager reserved all of
 * HBM at start-up, so a cudaMalloc made now would fail, and latency-critical loops that cannot
 * take the device-wide synchronisation of cudaMalloc / cudaFree.  It has no counterpart in the
 * reference (whose kernels need no scratch); it needs no context either, because creating one
 * allocates.  The kernel's stream-K scratch (tickets and fp32 partial sums) is a fixed 8 MiB array
 * inside the library's device image (every GPU that loads the library holds those 8 MiB until the
 * process exits).
 *  - Problems whose scratch (frisk_b200_gemm_workspace_bytes) exceeds 8 MiB are refused with
 *    FRISK_B200_E_TOO_LARGE; nothing is launched.
 *  - The first call on a device looks up that device's address of the array; make that first
 *    call outside any stream capture.  No call allocates or frees anything.
 *  - All calls on a device share the one array.  Each call clears the control words it needs
 *    on `stream` before its kernel, but two calls that overlap on the GPU (different streams)
 *    race on it: serialise them.
 * Results are bit-identical to frisk_b200_gemm with FRISK_B200_ALGO_SKINNY. */
int frisk_b200_gemm_skinny_static(int device, const frisk_b200_gemm_desc* desc, const void* A,
                                  const void* B, void* C, void* stream);

/* ---- attention forward -----------------------------------------------------------------
 * Replaces the launch of `frisk_execution` for the attention graph
 * (benchmark/layout/execution/tiled_attention.py:56-61: args q,k,v,out,scratch). */
int frisk_b200_attention_validate(const frisk_b200_attn_desc* desc);
size_t frisk_b200_attention_workspace_bytes(const frisk_b200_attn_desc* desc);
int frisk_b200_attention_fwd(frisk_b200_ctx* ctx, const frisk_b200_attn_desc* desc, const void* Q,
                             const void* K, const void* V, void* O, void* workspace,
                             size_t workspace_bytes, void* stream);
int frisk_b200_attention_fwd_host(frisk_b200_ctx* ctx, const frisk_b200_attn_desc* desc,
                                  const void* Q, const void* K, const void* V, void* O);

/* ---- split-K epilogue ------------------------------------------------------------------
 * After the fp32 partial products of a K-split GEMM have been summed across GPUs
 * (reduce-scatter), round this GPU's slice to the 16-bit output type.  No reference
 * counterpart: the reference has no multi-GPU path. */
int frisk_b200_convert_f32(frisk_b200_ctx* ctx, const float* src, void* dst, int64_t count,
                           int32_t dtype_dst, void* stream);

/* ---- fused split-K: GEMM whose fp32 result is STORED at the row-block owners ----------------
 * No reference counterpart (the reference is single-GPU).  The fp32 product of this rank's K
 * slice is not written to a local C: rows [i*rows_per_target, (i+1)*rows_per_target) are
 * stored, with 16-byte stores issued from the GEMM epilogue, into targets[i] (row pitch
 * ld_target elements).  A target may be another GPU's memory mapped into this process
 * (frisk_b200_peer_buffer_open): the exchange then travels over NVLink tile by tile while the
 * tensor cores work on the next tile.  Each rank points its targets at ITS OWN slot of the
 * owners' buffers; once every rank's kernel has finished (the caller places a cross-GPU
 * barrier on the stream) an owner sums its slots in slot order with frisk_b200_sum_slots, so
 * the result does not depend on timing.  Requirements: dtype_c = F32, trans_a = 0,
 * trans_b = 1, n_targets <= 8. */
int frisk_b200_gemm_push(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* desc, const void* A,
                         const void* B, float* const* targets, int32_t n_targets,
                         int64_t rows_per_target, int64_t ld_target, void* stream);
/* ---- what Frisk's IR can put next to a gemm on the same C --------------------------------
 * `frisk.fill` of C directly before an accumulating gemm and `frisk.reduce` of C along dim 1
 * directly after it (builders ffi/ir.cpp:439-456 and 457-470; ops
 * include/Dialect/Frisk/IR/FriskOps.td:400-423 and 425-453, reduce contract
 * lib/Dialect/Frisk/IR/FriskOps.cpp:728-762; the flow of test/python/bind_test.py:44-53).
 * frisk_b200_gemm_fused computes
 *     C <- (clear_accum ? 0 : fill_enable ? fill_value : C) + op(A).op(B)
 * (a fill before a gemm that overwrites C is dead: clear_accum wins)
 *     reduce_dst[i] <- (reduce_clear ? identity : reduce_dst[i]) (+) reduce_j C[i][j]
 * with the reduction taken over the values of C as stored (rounded to its element type) and
 * accumulated in fp32.  On the tcgen05 pair kernel both happen in the GEMM's epilogue (C is
 * not read for the fill; the reduction costs one fp32 per row and 256 columns, combined in a
 * fixed order); for the other kernels, and for a reduction after an accumulate that reads C,
 * the same result is produced by a fill kernel before and a row-reduction kernel after the
 * GEMM.  Kind `mul` of the reference has no kernel here (FRISK_B200_E_UNSUPPORTED). */
enum {
  FRISK_B200_REDUCE_NONE = 0,
  FRISK_B200_REDUCE_MAX = 1,
  FRISK_B200_REDUCE_MIN = 2,
  FRISK_B200_REDUCE_ADD = 3
};
typedef struct frisk_b200_gemm_epilogue {
  int32_t fill_enable;  /* C holds fill_value everywhere (it need not have been written) */
  float fill_value;     /* rounded to C's element type before use, as frisk.fill stores it */
  int32_t reduce_kind;  /* FRISK_B200_REDUCE_* */
  int32_t reduce_clear; /* 1: overwrite reduce_dst; 0: combine with what it holds */
  void* reduce_dst;     /* M elements of C's element type; may be NULL when reduce_kind is NONE */
} frisk_b200_gemm_epilogue;
/* 1 when the descriptor/epilogue pair runs fused in the GEMM epilogue, 0 when it is composed
 * from separate kernels, negative error code otherwise.  Host-only. */
int frisk_b200_gemm_fused_select(const frisk_b200_gemm_desc* desc, const frisk_b200_gemm_epilogue* epi);
size_t frisk_b200_gemm_fused_workspace_bytes(const frisk_b200_gemm_desc* desc,
                                             const frisk_b200_gemm_epilogue* epi);
/* workspace may be NULL: the context then owns the scratch (allocated on first use). */
int frisk_b200_gemm_fused(frisk_b200_ctx* ctx, const frisk_b200_gemm_desc* desc,
                          const frisk_b200_gemm_epilogue* epi, const void* A, const void* B, void* C,
                          void* workspace, size_t workspace_bytes, void* stream);

/* dst[i] = round(sum over s < n_slots of slots[s * slot_elems + i]), i < count, added in slot
 * order in fp32 and rounded once to the 16-bit type. */
int frisk_b200_sum_slots(frisk_b200_ctx* ctx, const float* slots, int32_t n_slots, int64_t slot_elems,
                         void* dst, int64_t count, int32_t dtype_dst, void* stream);
/* Device buffers that other processes of this node can map (cudaIpc): `handle64` is 64 bytes
 * to hand to the peers, which call _open.  _close frees (owned = 1) or unmaps (owned = 0). */
int frisk_b200_peer_buffer_create(frisk_b200_ctx* ctx, size_t bytes, void** ptr, void* handle64);
int frisk_b200_peer_buffer_open(frisk_b200_ctx* ctx, const void* handle64, void** ptr);
int frisk_b200_peer_buffer_close(frisk_b200_ctx* ctx, void* ptr, int32_t owned);

/* Checks the device status word after the stream has drained (synchronises `stream`).
 * Returns 0, FRISK_B200_E_DEVICE_TIMEOUT or FRISK_B200_E_CUDA. */
int frisk_b200_check(frisk_b200_ctx* ctx, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FRISK_B200_H */
