/*
 * pope_b200.h -- C ABI of libpope_b200.so: PoPE (polar positional embedding) attention
 * kernels for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a binding of the reference project (lucidrains/PoPE-pytorch) loads
 * in place of its two Triton modules.  Plain C: raw device pointers, sizes and element
 * strides; no C++ or framework types; no exceptions cross it.
 *
 * Conventions shared by every entry point
 *   - All tensor pointers are DEVICE pointers on the current CUDA device.  The caller owns
 *     and allocates every input, output and workspace; the operator entry points never allocate
 *     or free device memory and never synchronise the device.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Tensors are addressed as base + b*stride.b + h*stride.h + n*stride.n + feature, strides
 *     in ELEMENTS, innermost (feature / key) dimension contiguous.  Both the (b,h,n,d) and
 *     the (b,n,h,d) layouts of the reference are therefore zero-copy views.
 *   - `freqs` is an opaque fp32 table of phases, addressed as
 *     freqs[b*sf.b + h*sf.h + pos*sf.n + c], c < r; a stride of 0 broadcasts that axis
 *     (the encoding of PoPE_pytorch/triton_pope_flash_attn.py:237-245).  It has Nk rows;
 *     query i uses row (Nk - Nq + i)  (PoPE_pytorch/pope.py:64).
 *   - `bias` is fp32 (Hk, r): the per-key-head phase added to the key side only
 *     (PoPE_pytorch/pope.py:56).  Query head h reads key/value/bias head h % Hk
 *     (PoPE_pytorch/attention.py:44-45,118-120).
 *   - Return value: POPE_OK or a negative PopeStatus.  Argument errors are detected before
 *     anything is launched.
 *   - Thread-safe: any number of host threads may call concurrently, on the same or on different
 *     streams and devices.  State the library keeps per device for the life of the process:
 *       * one 4-byte sticky status word (see pope_b200_device_status), written only when a
 *         kernel's bounded wait gives up;
 *       * for pope_b200_attn_bwd on the tensor-core path, up to four (side stream + four events)
 *         sets created on first use.  A call borrows one set only while it ENQUEUES work: it
 *         forks the side stream off `stream` with an event, runs part of its kernels there and
 *         joins it back into `stream` before returning -- on error returns too -- so everything
 *         the call launches is ordered inside `stream` exactly like a single launch, and the
 *         sequence can be captured into a CUDA graph.  With all sets in use the call runs on
 *         `stream` alone.  No lock is held while the GPU executes;
 *       * the fixed scratch array of pope_b200_attn_fwd_noalloc (documented there).
 *     Kernel attributes (dynamic shared-memory opt-in) are set once per kernel and device.
 */
#ifndef POPE_B200_H_
#define POPE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define POPE_B200_ABI_VERSION 3

#if defined(__GNUC__)
#define POPE_API __attribute__((visibility("default")))
#else
#define POPE_API
#endif

typedef enum PopeStatus {
  POPE_OK = 0,
  POPE_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, Nq > Nk, r > d, H % Hk != 0 ... */
  POPE_ERR_UNSUPPORTED = -2,  /* shape / dtype outside what the kernels implement             */
  POPE_ERR_MISALIGNED = -3,   /* a pointer or stride breaks the documented alignment          */
  POPE_ERR_WORKSPACE = -4,    /* workspace missing or smaller than pope_b200_workspace_bytes   */
  POPE_ERR_CUDA = -5,         /* a CUDA runtime call failed (launch, attribute, symbol lookup) */
  POPE_ERR_ARCH = -6,         /* the current device is not compute capability 10.x            */
  POPE_ERR_TOO_LARGE = -7     /* the problem exceeds a fixed built-in capacity                */
} PopeStatus;

typedef enum PopeDtype { POPE_F32 = 0, POPE_BF16 = 1, POPE_F16 = 2 } PopeDtype;

typedef enum PopeOp {
  POPE_OP_SIM_FWD = 0, POPE_OP_SIM_BWD = 1, POPE_OP_ATTN_FWD = 2, POPE_OP_ATTN_BWD = 3, POPE_OP_DECODE_PAGED = 4
} PopeOp;

/* Element strides of the batch, head and row axes (innermost axis is contiguous). */
typedef struct PopeStride3 { int64_t b, h, n; } PopeStride3;

/* Problem geometry common to all operators. */
typedef struct PopeShape {
  int32_t B;   /* batch                                   */
  int32_t H;   /* query heads                             */
  int32_t Hk;  /* key/value heads, H % Hk == 0            */
  int32_t Nq;  /* query rows, Nq <= Nk                    */
  int32_t Nk;  /* key rows = rows of freqs                */
  int32_t d;   /* head dim                                */
  int32_t r;   /* rotated dims, 0 <= r <= d               */
  int32_t dtype; /* PopeDtype of q, k, v and their grads  */
} PopeShape;

/* The (freqs, bias) pair every operator takes -- PolarEmbedReturn, PoPE_pytorch/pope.py:18.
 * Optional factored form of the same table: when `positions` is not NULL the caller states that
 *   freqs[pos, c] == positions[pos * pos_stride_n + axis_of[c]] * inv_freqs[c]      (one fp32 multiply,
 * as PoPE.forward, PoPE_pytorch/pope.py:141, and AxialPoPE.forward, pope_nd.py:88-100, build it; axis_of
 * NULL = a single position axis), for a table without batch / head axes.  Kernels that derive their own
 * phase tables then recompute the phases from the 4-byte positions instead of loading the table; all other
 * kernels keep reading `freqs`, which must always be valid. */
typedef struct PopeEmbed {
  const float* freqs; PopeStride3 sf;      /* ignored when r == 0 */
  const float* bias;  int64_t bias_stride_h;
  const float* positions; int64_t pos_stride_n;   /* may be NULL */
  const float* inv_freqs;                         /* (r) */
  const int32_t* axis_of;                         /* (r), may be NULL */
} PopeEmbed;

/* ---- similarity: sim[b,h,i,j] = <q'_i, k'_j> --------------------------------------------
 * Replaces PoPESimilarityFunction.forward / _fwd_kernel, PoPE_pytorch/triton_pope.py:28-83,
 * 260-288.  `sim` has the dtype of q (triton_pope.py:273); ss = strides of (b, h, row). */
typedef struct PopeSimArgs {
  uint32_t struct_bytes;     /* sizeof(PopeSimArgs), checked */
  int32_t allow_tf32;        /* accepted; the kernels always meet the fp32 tolerance */
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  void* sim;     PopeStride3 ss;
  void* workspace; size_t workspace_bytes;  /* pope_b200_workspace_bytes(POPE_OP_SIM_FWD, &args); may be NULL when 0 */
} PopeSimArgs;

/* Replaces PoPESimilarityFunction.backward, PoPE_pytorch/triton_pope.py:290-362.
 * dq/dk are written (dtype of q).  dfreqs / dbias are optional fp32 ACCUMULATORS the caller
 * zero-fills: dfreqs uses the stride encoding of freqs (0 = summed over that axis),
 * dbias is (Hk, r) contiguous rows with stride dbias_stride_h. */
typedef struct PopeSimBwdArgs {
  uint32_t struct_bytes;
  int32_t allow_tf32;
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  const void* dsim; PopeStride3 sds;
  void* dq; PopeStride3 sdq;
  void* dk; PopeStride3 sdk;
  float* dfreqs; PopeStride3 sdf;   /* may be NULL */
  float* dbias; int64_t dbias_stride_h; /* may be NULL */
  void* workspace; size_t workspace_bytes;  /* pope_b200_workspace_bytes(POPE_OP_SIM_BWD, &args); may be NULL when 0 */
} PopeSimBwdArgs;

/* ---- attention ----------------------------------------------------------------------------
 * Replaces flash_attn_forward / _fwd_kernel, PoPE_pytorch/triton_pope_flash_attn.py:23-117,
 * 222-271.  out has q's dtype; lse is fp32 (B, H, Nq) contiguous.  mask is an optional
 * uint8/bool key-padding mask, nonzero = keep, addressed mask[b*mask_stride_b + j*mask_stride_n]
 * (PoPE_pytorch/attention.py:129-131).  The causal mask is top-left aligned (key j visible to
 * query i iff j <= i); a row with no visible key gives out = 0 and lse = -inf.
 * Small Nq against a long key range (decode) is split over the keys internally; that path
 * and the table-driven tensor-core path need `workspace` (size from
 * pope_b200_workspace_bytes(POPE_OP_ATTN_FWD, &args); may be NULL when that returns 0). */
typedef struct PopeAttnArgs {
  uint32_t struct_bytes;
  int32_t causal;
  float softmax_scale;
  int32_t reserved0;
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  const void* v; PopeStride3 sv;
  void* out;     PopeStride3 so;
  float* lse;
  const uint8_t* mask; int64_t mask_stride_b, mask_stride_n;
  void* workspace; size_t workspace_bytes;
} PopeAttnArgs;

/* Replaces flash_attn_backward / _bwd_preprocess / _bwd_kernel,
 * PoPE_pytorch/triton_pope_flash_attn.py:119-218, 273-335.  dq, dk, dv are written (q's dtype).
 * dfreqs / dbias as in PopeSimBwdArgs (caller zero-fills; NULL = not wanted). */
typedef struct PopeAttnBwdArgs {
  uint32_t struct_bytes;
  int32_t causal;
  float softmax_scale;
  int32_t reserved0;
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  const void* v; PopeStride3 sv;
  const void* out; PopeStride3 so;
  const void* dout; PopeStride3 sdo;
  const float* lse;
  const uint8_t* mask; int64_t mask_stride_b, mask_stride_n;
  void* dq; PopeStride3 sdq;
  void* dk; PopeStride3 sdk;
  void* dv; PopeStride3 sdv;
  float* dfreqs; PopeStride3 sdf;
  float* dbias; int64_t dbias_stride_h;
  void* workspace; size_t workspace_bytes;
} PopeAttnBwdArgs;

/* ---- the stand-alone transform ---------------------------------------------------------------
 * Replaces the pure-PyTorch body of apply_pope_to_qk, PoPE_pytorch/pope.py:37-86 (return_complex
 * excluded): q (B,H,Nq,d) and k (B,Hk,Nk,d) -> q_out (B,H,Nq,d+r), k_out (B,Hk,Nk,d+r) in fp32, the
 * rotated features as interleaved pairs (a cos, a sin) followed by the pass-through features
 * (:69-70, :77-78, :82-84).  One pass over the data.  freqs may carry batch / head strides (3-D and 4-D
 * tables, :53-56).  Output rows must start on 8-byte boundaries (even d + r and row strides). */
typedef struct PopeApplyArgs {
  uint32_t struct_bytes;
  int32_t reserved0;
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  float* q_out;  PopeStride3 sqo;
  float* k_out;  PopeStride3 sko;
} PopeApplyArgs;

/* Backward of the transform (autograd does it in the reference): dq_out / dk_out are the fp32 gradients
 * of the two outputs; dq, dk are written (dtype of q); dfreqs / dbias are optional fp32 ACCUMULATORS
 * the caller zero-fills, as in PopeSimBwdArgs. */
typedef struct PopeApplyBwdArgs {
  uint32_t struct_bytes;
  int32_t reserved0;
  PopeShape shape;
  PopeEmbed embed;
  const void* q; PopeStride3 sq;
  const void* k; PopeStride3 sk;
  const float* dq_out; PopeStride3 sdqo;
  const float* dk_out; PopeStride3 sdko;
  void* dq; PopeStride3 sdq;
  void* dk; PopeStride3 sdk;
  float* dfreqs; PopeStride3 sdf;
  float* dbias; int64_t dbias_stride_h;
} PopeApplyBwdArgs;

/* ---- decode over a paged key / value cache ------------------------------------------------------
 * (No counterpart in the reference, which recomputes attention over full K and V every step; this is
 * the step either side of the decode path in a serving loop: append the new token's k and v to a cache,
 * then attend the new query over everything cached.)
 *
 * Layout.  Keys and values live in fixed-size pages, k_pages / v_pages = [num_pages][Hk][page_size][d]
 * contiguous, dtype of q (bf16 or fp16); page_size is a multiple of 64.  page_table[b * max_pages_per_seq + i]
 * is the physical page that holds keys [i * page_size, (i + 1) * page_size) of sequence b; seq_lens[b] is
 * the number of keys sequence b holds.  Key j of a sequence sits at position j (row j of freqs); raw k is
 * cached, the transform is applied as the keys stream through shared memory, so a cache entry never
 * depends on the phase bias.  Which physical page a sequence gets next is the caller's policy: the
 * library only reads the table.  A page index outside [0, num_pages) is never dereferenced: it is
 * clamped, bit 1 of the device status word (pope_b200_device_status) is set and the results of that call
 * are invalid. */
typedef struct PopePagedKV {
  void* k_pages;
  void* v_pages;
  const int32_t* page_table;   /* (B, max_pages_per_seq), device */
  int32_t* seq_lens;           /* (B), device; read by decode, read and advanced by append */
  int32_t num_pages, page_size, max_pages_per_seq, reserved0;
} PopePagedKV;

/* Append n_new rows per sequence: k, v (B, Hk, n_new, d) with element strides, written at positions
 * [seq_lens[b], seq_lens[b] + n_new) of sequence b; the table must already map those positions.  With
 * `advance` nonzero seq_lens[b] += n_new afterwards (a second tiny launch on the same stream). */
typedef struct PopeKvAppendArgs {
  uint32_t struct_bytes;
  int32_t dtype;               /* PopeDtype: POPE_BF16 or POPE_F16 */
  int32_t B, Hk, d, n_new;
  int32_t advance, reserved0;
  PopePagedKV kv;
  const void* k; PopeStride3 sk;
  const void* v; PopeStride3 sv;
} PopeKvAppendArgs;

/* One query row per (batch, head) against the cached keys of its sequence: out = softmax(q' K'^T scale) V
 * with the query at the LAST cached position, seq_lens[b] - 1 (PoPE_pytorch/pope.py:64 and
 * triton_pope_flash_attn.py:54-55: positions are bottom-right aligned), no causal mask needed.
 * shape.Nq = 1; shape.Nk = an upper bound of every seq_lens[b] (it sizes the key split and the phase
 * table; freqs must have at least that many rows and no batch / head axes).  A sequence without keys
 * gives out = 0, lse = -inf.  lse (B, H) fp32 may be NULL.  Workspace: pope_b200_workspace_bytes(
 * POPE_OP_DECODE_PAGED, &args).  Kernel: the streaming decode kernel (copy-engine ring of 64-key tiles,
 * key ranges split over CTAs, split combine), tile addresses taken from the page table. */
typedef struct PopePagedDecodeArgs {
  uint32_t struct_bytes;
  float softmax_scale;
  PopeShape shape;
  PopeEmbed embed;
  PopePagedKV kv;
  const void* q; PopeStride3 sq;   /* (B, H, 1, d): batch and head strides are used */
  void* out;     PopeStride3 so;
  float* lse;
  void* workspace; size_t workspace_bytes;
} PopePagedDecodeArgs;

POPE_API int pope_b200_abi_version(void);
POPE_API const char* pope_b200_status_str(int status);

/* Name of the kernel family the last successful call ON THIS THREAD dispatched to
 * ("simt", "tcgen05", ...).  Diagnostic only. */
POPE_API const char* pope_b200_last_path(void);

/* Sticky device-side status of the tensor-core kernels on the current device: 0 = healthy,
 * bit 0 = a bounded wait inside a kernel gave up (its results are then invalid), bit 1 = a paged-cache call
 * met a page index or a position outside the cache (clamped / skipped; its results are invalid).
 * Diagnostic: this call synchronises the device. */
POPE_API int pope_b200_device_status(void);

/* Reset that word to 0 on the current device (synchronises the device).  POPE_OK or POPE_ERR_CUDA. */
POPE_API int pope_b200_clear_device_status(void);

/* Diagnostic, not an operator: launches one tiny kernel on `stream` whose only mbarrier is never
 * completed, waited on with the same bounded wait the real kernels use but a limit of a few
 * microseconds.  The kernel gives up, sets bit 0 of the status word, frees its tensor memory and
 * returns; the device stays healthy.  It exists so that the give-up path can be tested without
 * faulting or hanging a GPU.  Follow it with pope_b200_clear_device_status(). */
POPE_API int pope_b200_selftest_bounded_wait(void* stream);

/* Bytes of workspace the operator needs for these arguments (`args` points at the matching
 * Pope*Args struct; pointers inside it are not dereferenced).  0 = none. */
POPE_API size_t pope_b200_workspace_bytes(int op, const void* args);

POPE_API int pope_b200_sim_fwd(const PopeSimArgs* args, void* stream);
POPE_API int pope_b200_sim_bwd(const PopeSimBwdArgs* args, void* stream);
POPE_API int pope_b200_attn_fwd(const PopeAttnArgs* args, void* stream);
POPE_API int pope_b200_attn_bwd(const PopeAttnBwdArgs* args, void* stream);
POPE_API int pope_b200_apply_qk_fwd(const PopeApplyArgs* args, void* stream);
POPE_API int pope_b200_apply_qk_bwd(const PopeApplyBwdArgs* args, void* stream);
POPE_API int pope_b200_kv_append(const PopeKvAppendArgs* args, void* stream);
POPE_API int pope_b200_attn_decode_paged(const PopePagedDecodeArgs* args, void* stream);

/* ---- attention forward for callers that cannot allocate -----------------------------------------
 * (No counterpart in the reference: its wrappers always allocate through torch.)
 *
 * Same arguments and results as pope_b200_attn_fwd, but `workspace` / `workspace_bytes` are
 * ignored: the kernel's scratch (the position phase table and the expanded operand tiles of k)
 * lives in a fixed array inside the library instead.  Meant for hosts that may not touch a device allocator where they call us --
 * an inference loop whose memory plan is frozen, a plugin that is only ever handed input and
 * output buffers, a latency-critical thread that must not take the allocator's lock.  The call
 * itself performs no device allocation or free of any kind.
 *
 * Limits and rules
 *   - Only the tensor-core shapes are served (bf16/fp16, d in {64,96,128}, r % 16 == 0, Nq >= 64,
 *     16-byte aligned rows); anything else returns POPE_ERR_UNSUPPORTED.
 *   - The scratch a call needs is what pope_b200_workspace_bytes reports for the forward
 *     (4 Nk r bytes of table -- fp16 cos and sin -- rounded up to 256, plus
 *     2 (d + r) bytes per key row of every key head, rows padded to a multiple of 256);
 *     more than POPE_B200_NOALLOC_MAX_SCRATCH returns POPE_ERR_TOO_LARGE and launches nothing.  Every GPU that loads the library holds that many
 *     bytes until the process exits.
 *   - The first call on each device looks up the array's device address (a one-time runtime
 *     query made with that device current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array and each call rewrites the part it uses, so
 *     nothing is carried over between calls -- but two calls whose kernels overlap on the GPU
 *     (different streams, no ordering) race on it.  Serialise them. */
#define POPE_B200_NOALLOC_MAX_SCRATCH (16u << 20)
POPE_API int pope_b200_attn_fwd_noalloc(const PopeAttnArgs* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* POPE_B200_H_ */
