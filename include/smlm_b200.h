/* smlm_b200 - C ABI of the B200 (sm_100a) Segmented Multi-LoRA Multiplication path.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*), enqueues work on that stream and returns an
 * int status (SMLM_OK == 0) without synchronising and without allocating: all
 * scratch is caller-owned (see smlm_b200_plan_bytes).  `dtype` selects the 16-bit
 * storage type of activations and adapter weights; accumulation is always fp32.
 *
 * Weight layout follows the reference operator's `is_row_major` flag
 * (kernel_src/csrc/loquetier_ops.cc:294-303): 0 = column-major, i.e. the PEFT
 * layout A[r, h_in], B[h_out, r] that the reference's add_lora passes
 * (src/loquetier_src/kernel_utils.py:118-119); 1 = row-major, the math layout
 * A[h_in, r], B[r, h_out].
 *
 * Adapter weights are given as a device array of device addresses, exactly like the
 * reference's int64 pointer tensors (src/loquetier_src/models/mixed_lora.py:151-161).
 * Either the array has one entry per segment (`seg_ids == NULL`, what the reference
 * builds with `wa_ptrs[lora_ids]`, mixed_lora.py:182), or it is the per-adapter
 * table itself and `seg_ids[nseg]` holds each segment's adapter index, which saves
 * the gather.  `n_table` is the length of the array in both cases.
 */
#ifndef SMLM_B200_H_
#define SMLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SMLM_OK = 0,
  SMLM_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size */
  SMLM_ERR_DTYPE = 2,            /* dtype is neither SMLM_F16 nor SMLM_BF16 */
  SMLM_ERR_NO_KERNEL = 3,        /* shape outside the path: the small dimension must be a
                                    multiple of 8 and <= 128, the large one a multiple of 8
                                    (the reference's "No suitable kernel.", loquetier_ops.cc:318) */
  SMLM_ERR_MISALIGNED = 4,       /* a base pointer is not 16-byte aligned */
  SMLM_ERR_WORKSPACE = 5,        /* plan buffer too small */
  SMLM_ERR_CUDA = 6,             /* the CUDA runtime rejected a launch */
  SMLM_ERR_BAD_INDPTR = 7,       /* reported by smlm_b200_plan_status */
  SMLM_ERR_BAD_POINTER = 8,      /* reported by smlm_b200_plan_status */
  SMLM_ERR_BAD_INDEX = 9,        /* reported by smlm_b200_plan_status */
  SMLM_ERR_TIMEOUT = 10,         /* reported by smlm_b200_plan_status: a bounded wait in a kernel gave up */
  SMLM_ERR_STATIC_LIMIT = 11,    /* smlm_b200_wgrad_static: the problem needs more than the built-in scratch */
  SMLM_ERR_GROUPED_PLAN = 12     /* reported by smlm_b200_plan_status: a grouped plan reached a launch that cannot use it */
};

enum { SMLM_F16 = 0, SMLM_BF16 = 1 };

int smlm_b200_version(void);
const char* smlm_b200_status_string(int status);

/* Scratch bytes the reference asks its caller for, 60 per segment
 * (smlm_forward_tmp_size, kernel_src/csrc/smlm_forward/smlm_forward_cutlass.cuh:48-52;
 * bound as smlm_forward_cutlass_tmp_size, loquetier_ops.cc:372).  Kept so that the
 * reference's own size check (loquetier_ops.cc:304) holds; this library never
 * writes into that buffer. */
size_t smlm_b200_tmp_size(int num_problems);

/* For callers that have one weight pointer per segment and no adapter table (the arguments of the reference
 * operator, loquetier_ops.cc:277-281): ids_out[i] = index of the first segment whose pointer equals w_table[i].
 * Passing w_table as the adapter table (n_table = nseg) and ids_out as seg_ids to smlm_b200_plan_grouped and to the
 * compute call gathers the decode tokens of one adapter into one piece wherever they sit in the batch - what the
 * reference only gets from a batch sorted by adapter.  nseg <= 4096 for the grouped plan to apply. */
int smlm_b200_group_ids_from_pointers(const void* const* w_table, int nseg, int32_t* ids_out, void* stream);

/* Segment bookkeeping on the device: the run-length merge of the ordered requests of a step into
 * segments, bit-identical to the reference's host loop (src/loquetier_src/model_generation.py:267-283:
 * neighbours with the same adapter become one segment; `segment` = cumsum of the lengths with a
 * leading 0, int32).  req_ids / req_len: adapter id and token count per request in batch row order,
 * n entries.  Outputs have n (seg_ids, seg_len) and n + 1 (seg_indptr) entries; entries past the
 * number of segments are empty segments, so (seg_indptr, nseg = n) can be handed to smlm_b200_plan
 * without reading nseg_out[0] back.  Stream-ordered; can be captured in a CUDA graph. */
int smlm_b200_merge_segments(const int32_t* req_ids, const int32_t* req_len, int n, int32_t* seg_ids,
                             int32_t* seg_len, int32_t* seg_indptr, int32_t* nseg_out, void* stream);

/* Rows per piece the plan uses for a batch of T token rows (64 at most; a multiple of 8). */
int smlm_b200_piece_rows(int T);

/* Kernel choice for ranks above 32 in smlm_b200_fwd / smlm_b200_bwd_dx / smlm_b200_bwd.  No
 * reference counterpart (the reference has one CUTLASS grouped GEMM per product).  mode 0 (default):
 * the tcgen05 kernel with 128-row tiles is used for batches of long segments, the mma.sync kernel
 * with 64-row tiles otherwise; mode > 0: the tcgen05 kernel wherever it applies; mode < 0: never.
 * Process-wide; returns the previous mode.  Both kernels compute the same function (fp32
 * accumulation, V rounded to the storage type between the products). */
int smlm_b200_set_tensor_core_mode(int mode);

/* Tuning knob of the mma.sync fused kernel, for measurements: a piece (up to 64 rows of one segment)
 * is served by a cluster of 1..4 CTAs that split the hidden dimension; 0 (default) lets the library
 * choose per launch from the batch shape, 1..4 forces the split.  No reference counterpart.
 * Process-wide; returns the previous setting.  Results are the same function either way (sums over
 * the hidden dimension are cut differently). */
int smlm_b200_set_cluster_split(int split);

/* Bytes of the plan buffer for a batch of T token rows in nseg segments. */
size_t smlm_b200_plan_bytes(int T, int nseg);

/* Build the work list of a batch from its device-resident segment index pointer
 * seg_indptr[nseg + 1] (int32, the reference's `s`).  Replaces
 * precompute_smlm_forward_args (smlm_forward_cutlass.cuh:31-46, launched :76).
 * One plan serves every call on the same index pointer (shrink, expand, every
 * projection of a model step).  `plan` must be 16-byte aligned. */
int smlm_b200_plan(void* plan, size_t plan_bytes, const int32_t* seg_indptr, int nseg, int T, void* stream);

/* The same, for the forward entry points when they are called with an adapter table and seg_ids:
 * segments of at most 8 rows (decode tokens) are not given pieces of their own; their rows are grouped
 * by adapter, wherever they sit in the batch, so that the kernels fetch an adapter's panels once for all
 * of its decode tokens.  The reference gets this effect only when its batch assembler has sorted the
 * decode requests by adapter (src/loquetier_src/model_generation.py:186, 267-273); here the order of the
 * batch does not matter.  seg_ids[nseg] is the per-segment adapter index the compute call will also be
 * given, n_table the table size (tables above 4096 entries, or seg_ids == NULL, give the ordinary plan).
 * A grouped plan serves smlm_b200_gemm / smlm_b200_fwd / smlm_b200_bwd_dx with that seg_ids and table and
 * `grouped = 1`; the weight-gradient entry points need an ordinary plan (they record SMLM_ERR_GROUPED_PLAN
 * otherwise).  The tcgen05 kernels read the plan's list of 128-row pieces, which is never grouped.
 * Same buffer size as smlm_b200_plan. */
int smlm_b200_plan_grouped(void* plan, size_t plan_bytes, const int32_t* seg_indptr, const int32_t* seg_ids,
                           int nseg, int n_table, int T, void* stream);

/* Two plans in one launch: plan A as smlm_b200_plan_grouped builds it (ids_a may be NULL for an ordinary
 * plan), plan B as smlm_b200_plan builds it - typically the plan of all segments and the plan of the train
 * partitions of one step, which would otherwise cost two launches back to back. */
int smlm_b200_plan_pair(void* plan_a, size_t plan_a_bytes, const int32_t* indptr_a, const int32_t* ids_a, int nseg_a,
                        int n_table_a, int T_a, void* plan_b, size_t plan_b_bytes, const int32_t* indptr_b,
                        int nseg_b, int T_b, void* stream);

/* Synchronises the stream and reports what the device recorded in a plan: number
 * of pieces and SMLM_OK or one of the SMLM_ERR_BAD_* codes.  For tests and
 * debugging; the compute entry points never synchronise. */
int smlm_b200_plan_status(const void* plan, int* n_pieces, void* stream);

/* One segmented GEMM  Y[s_i:s_{i+1}] = scale_i * X[s_i:s_{i+1}] . W_i  (+ Y).
 * Stand-in for one call of the reference operator smlm_forward_cutlass(y, x, w_ptr,
 * s, tmp, is_row_major) (dispatch_smlm_forward_cutlass, loquetier_ops.cc:277-319;
 * smlm_forward, smlm_forward_cutlass.cuh:61-175): d_in >= d_out runs the shrink
 * kernel, d_in < d_out the expand kernel.  With seg_scale == NULL and
 * accumulate == 0 the result is the reference's (alpha 1, beta 0: rows inside
 * segments overwritten, other rows untouched).  `grouped` must be 1 when `plan` comes from
 * smlm_b200_plan_grouped (the launch then runs the kernel variant that knows gather pieces) and 0
 * otherwise; a grouped plan passed with 0 is refused piece by piece (SMLM_ERR_GROUPED_PLAN). */
int smlm_b200_gemm(void* y, const void* x, const void* const* w_table, const int32_t* seg_ids,
                   const float* seg_scale, void* plan, int n_table, int T, int nseg, int d_in, int d_out,
                   int dtype, int is_row_major, int accumulate, int grouped, void* stream);

/* Fused LoRA forward  v = x . A^T ;  y (+)= scale * v . B^T  for every segment:
 * the two operator calls of add_lora.forward (kernel_utils.py:114-120) and, with
 * seg_scale / accumulate, the scale and add of MixedLoraLinear.forward
 * (mixed_lora.py:214-217).  `v` [T, rank] is written in the storage type like the
 * reference's intermediate (kernel_utils.py:117) and is what the backward needs.
 *
 * `independent` = 1 is a promise by the caller about every kernel enqueued on `stream` since, and
 * including, the most recent launch of this library with independent = 0 (call them the open
 * kernels): this call reads nothing and writes nothing that an open kernel writes, and writes
 * nothing that an open kernel reads.  Typical use: q_proj, k_proj and v_proj of one layer, which
 * share their input and write different outputs.  An independent launch does not wait for its
 * predecessors at its start - its read phase overlaps their write phase, which is how both
 * directions of HBM are kept busy - so it can run alongside ALL open kernels, not only the
 * previous one: in a chain D (dependent), I1, I2 (independent) the kernel I2 may run while D is
 * still writing, hence a call that consumes D's output must be launched with independent = 0 even if
 * an unrelated independent launch sits between them.  An independent launch still completes after
 * the open kernels, so stream order holds for everything enqueued later.  With 0 the launch waits
 * for its predecessor like any kernel.  `grouped` as in smlm_b200_gemm. */
int smlm_b200_fwd(void* y, const void* x, void* v, const void* const* wa_table, const void* const* wb_table,
                  const int32_t* seg_ids, const float* seg_scale, void* plan, int n_table, int T, int nseg,
                  int h_in, int h_out, int rank, int dtype, int is_row_major, int accumulate, int independent,
                  int grouped, void* stream);

/* Bytes of the workspace the weight-gradient kernels need for a batch of T token
 * rows in npart partitions and one (h1 == 0) or two column counts.  The workspace
 * holds tickets and parked partial sums of partitions that are spread over several
 * CTAs.  Its head - smlm_b200_wgrad_ticket_bytes(...) bytes, the tickets - must be
 * zero when a launch starts; every launch leaves the tickets it used zeroed again.  So:
 * zero-fill the workspace once after allocation, and zero the head again whenever the
 * next call's shape (T, npart, rank, column counts, or the kinds selected by
 * smlm_b200_wgrad_select_multi) differs from the previous call's on the same workspace:
 * a different shape puts the boundary between tickets and parked sums elsewhere, and what
 * one shape parked lies where another expects tickets.  Launches that overlap in time must
 * not share a workspace. */
size_t smlm_b200_wgrad_workspace_bytes(int T, int npart, int rank, int h0, int h1);
size_t smlm_b200_wgrad_ticket_bytes(int T, int npart, int rank, int h0, int h1);

/* Per-partition weight gradient  G_p = scale_p * P[rows_p]^T . Q[rows_p]  with P
 * [T, rank] and Q [T, h]; G_p is [rank, h] (transposed == 0) or [h, rank]
 * (transposed == 1), of the storage type or fp32 (grad_fp32), overwritten or
 * accumulated into.  The dA / dB products of add_lora.backward
 * (kernel_utils.py:144-145).  `plan` is a plan built on part_indptr. */
int smlm_b200_wgrad(void* const* g_table, const void* p, const void* q, const int32_t* part_indptr,
                    const float* part_scale, void* plan, void* workspace, size_t workspace_bytes, int npart, int T,
                    int rank, int h, int dtype, int transposed, int accumulate, int grad_fp32, void* stream);

/* smlm_b200_wgrad for callers that cannot hand over device memory of their own.
 * (No counterpart in the reference: its backward is torch matmuls and allocates freely.)
 *
 * Who needs it: code that runs where allocating is not an option - a serving loop
 * that carved up all device memory at start-up and must not call the allocator on the
 * request path, a plugin that receives its buffers from a host application and owns
 * no allocator, an embedding framework whose caching pool must see every allocation.
 * Such callers can pass inputs and outputs but have nowhere to get the workspace of
 * smlm_b200_wgrad from.  This variant keeps the workspace in a fixed array inside the
 * library's device image instead and calls no allocating routine at all.
 *
 * Same arguments and results as smlm_b200_wgrad, minus the workspace.  Limits and rules:
 *  - the array is SMLM_STATIC_WGRAD_BYTES (16 MiB) and every GPU that loads the library
 *    holds it until the process exits; a problem whose workspace
 *    (smlm_b200_wgrad_workspace_bytes(T, npart, rank, h, 0)) is larger is refused with
 *    SMLM_ERR_STATIC_LIMIT before anything is launched;
 *  - the first call on each device looks up the array's device address (with that
 *    device current).  Make that first call outside any stream capture;
 *  - all calls on a device share the one array, which keeps the previous call's
 *    contents; the tickets, the only part that must start from zero, are cleared on
 *    `stream` at the start of every call.  Two calls that may run on the GPU at the
 *    same time (different streams, or graphs replayed concurrently) race on it - keep
 *    them ordered, or use smlm_b200_wgrad with separate workspaces. */
#define SMLM_STATIC_WGRAD_BYTES (16u << 20)
int smlm_b200_wgrad_static(void* const* g_table, const void* p, const void* q, const int32_t* part_indptr,
                           const float* part_scale, void* plan, int npart, int T, int rank, int h, int dtype,
                           int transposed, int accumulate, int grad_fp32, void* stream);

/* Both weight gradients of the backward in one launch:
 *   dB_p = scale_p * gO[rows_p]^T . V[rows_p]      dA_p = dV[rows_p]^T . X[rows_p]
 * (kernel_utils.py:144-145; dV is expected to carry the scale already, as
 * smlm_b200_bwd produces it).  Layout of dA / dB follows is_row_major like the
 * weights; part_ids (or NULL) selects the per-adapter entry of part_scale.
 * `independent` as in smlm_b200_fwd, with one more condition: the call must not share
 * its workspace with the previous kernel of the stream. */
int smlm_b200_wgrad_pair(void* const* dA_table, void* const* dB_table, const void* dv, const void* x,
                         const void* v, const void* go, const int32_t* part_indptr, const int32_t* part_ids,
                         const float* part_scale, void* plan, void* workspace, size_t workspace_bytes, int n_table,
                         int npart, int T, int h_in, int h_out, int rank, int dtype, int is_row_major,
                         int accumulate, int grad_fp32, int independent, void* stream);

/* First half of the backward: dV = scale * gO . B (written to dv [T, rank]) and
 * dX = dV . A for the rows of every train partition (kernel_utils.py:142-143), one
 * launch.  `plan` is built on the partition index pointer; `independent` and `grouped` as in
 * smlm_b200_fwd. */
int smlm_b200_bwd_dx(void* dx, void* dv, const void* go, const void* const* wa_table, const void* const* wb_table,
                     const int32_t* part_ids, const float* part_scale, void* plan, int n_table, int T, int npart,
                     int h_in, int h_out, int rank, int dtype, int is_row_major, int independent, int grouped,
                     void* stream);

/* Fine-tuning backward of the fused forward over the train partitions
 * part_indptr[npart + 1] (add_lora.backward, kernel_utils.py:129-147):
 *   dV = scale * gO . B     (written to dv [T, rank], storage type)
 *   dB_p = scale * gO^T . V   dA_p = dV^T . X   dX = dV . A
 * i.e. smlm_b200_bwd_dx followed by smlm_b200_wgrad_pair.
 * `plan` is a plan built on part_indptr.  wa_table / wb_table / part_ids follow
 * the forward's convention with partitions in the role of segments.  dX rows
 * outside the partitions are not written (the reference returns zeros there,
 * kernel_utils.py:136; the host wrapper clears them).  dA_table / dB_table are
 * device arrays of npart output addresses in the layout of A and B.  `workspace`:
 * smlm_b200_wgrad_workspace_bytes(T, npart, rank, h_out, h_in) bytes, see there. */
int smlm_b200_bwd(void* dx, void* const* dA_table, void* const* dB_table, void* dv, const void* go,
                  const void* x, const void* v, const void* const* wa_table, const void* const* wb_table,
                  const int32_t* part_ids, const float* part_scale, const int32_t* part_indptr, void* plan,
                  void* workspace, size_t workspace_bytes, int n_table, int T, int npart, int h_in, int h_out,
                  int rank, int dtype, int is_row_major, int accumulate_grads, int grad_fp32, void* stream);

/* ---- several projections of one layer per launch ----------------------------------------------
 * No reference counterpart: the reference calls its operator once per product and projection
 * (kernel_utils.py:118-119 inside MixedLoraLinear.forward, mixed_lora.py:198).  Projections that share
 * the batch - q/k/v or gate/up of a layer, or every LoRA target when their inputs are at hand - also
 * share the segment plan, the adapter ids, the rank and the scales, so their launches can be laid end
 * to end in one grid: short launches then stop paying a set-up and a drain each.  The function
 * computed is that of the single-projection entry points; how a sum over the hidden dimension is cut
 * over the CTAs of a cluster is chosen per launch, so v / dV can differ from a single-projection call
 * in the last bit of a sum.
 *
 * `projs` is a HOST array of nproj <= SMLM_MAX_PROJ descriptors; only the fields an entry point names
 * are read.  The projections must not depend on one another: none may read or write what another
 * writes.  `independent` is the promise of smlm_b200_fwd for the call as a whole. */
#define SMLM_MAX_PROJ 8
typedef struct smlm_b200_proj {
  const void* x;                 /* [T, h_in]      forward input                                   */
  void* y;                       /* [T, h_out]     forward output                                  */
  void* v;                       /* [T, rank]      forward intermediate (written by fwd)           */
  const void* go;                /* [T_ft, h_out]  gradient of y over the train rows               */
  void* dx;                      /* [T_ft, h_in]                                                   */
  void* dv;                      /* [T_ft, rank]   backward intermediate (written by bwd_dx)       */
  const void* const* wa_table;   /* adapter tables as in smlm_b200_fwd                             */
  const void* const* wb_table;
  void* const* dA_table;         /* per-partition gradient addresses as in smlm_b200_bwd           */
  void* const* dB_table;
  int h_in, h_out;
} smlm_b200_proj;

/* smlm_b200_fwd for every projection: reads x, wa_table, wb_table; writes y, v. */
int smlm_b200_fwd_multi(const smlm_b200_proj* projs, int nproj, const int32_t* seg_ids, const float* seg_scale,
                        void* plan, int n_table, int T, int nseg, int rank, int dtype, int is_row_major,
                        int accumulate, int independent, int grouped, void* stream);

/* smlm_b200_bwd_dx for every projection: reads go, wa_table, wb_table; writes dx, dv.  T is the number of
 * train rows the partition plan covers. */
int smlm_b200_bwd_dx_multi(const smlm_b200_proj* projs, int nproj, const int32_t* part_ids, const float* part_scale,
                           void* plan, int n_table, int T, int npart, int rank, int dtype, int is_row_major,
                           int independent, void* stream);

/* Workspace of smlm_b200_wgrad_pair_multi for these projections (h_in, h_out are read); same rules as
 * smlm_b200_wgrad_workspace_bytes. */
size_t smlm_b200_wgrad_multi_workspace_bytes(const smlm_b200_proj* projs, int nproj, int T, int npart, int rank);
/* The head of that workspace that has to be zero (see smlm_b200_wgrad_workspace_bytes), for the whole set; it covers
 * the head of every subset that smlm_b200_wgrad_select_multi may launch. */
size_t smlm_b200_wgrad_multi_ticket_bytes(const smlm_b200_proj* projs, int nproj, int T, int npart, int rank);

/* smlm_b200_wgrad_pair for every projection: reads dv, x, v, go; writes through dA_table, dB_table. */
int smlm_b200_wgrad_pair_multi(const smlm_b200_proj* projs, int nproj, const int32_t* part_indptr,
                               const int32_t* part_ids, const float* part_scale, void* plan, void* workspace,
                               size_t workspace_bytes, int n_table, int npart, int T, int rank, int dtype,
                               int is_row_major, int accumulate, int grad_fp32, int independent, void* stream);

/* The same launch for one kind of gradient only: `which` = SMLM_WGRAD_DB (dB = gO^T . V: reads v, go), SMLM_WGRAD_DA
 * (dA = dV^T . X: reads dv, x) or both.  dA needs nothing of the forward, so a step can launch it right behind
 * smlm_b200_bwd_dx_multi, let the forward run next to it as an independent launch, and keep only dB for the end.
 * Two such launches may share a workspace when they do not overlap in time. */
#define SMLM_WGRAD_DB 1
#define SMLM_WGRAD_DA 2
int smlm_b200_wgrad_select_multi(const smlm_b200_proj* projs, int nproj, int which, const int32_t* part_indptr,
                                 const int32_t* part_ids, const float* part_scale, void* plan, void* workspace,
                                 size_t workspace_bytes, int n_table, int npart, int T, int rank, int dtype,
                                 int is_row_major, int accumulate, int grad_fp32, int independent, void* stream);

/* ---- RMSNorm: the caller on either side of the q/k/v and gate/up projections ----------------- */

/* Replaces dispatch_rms_norm / rms_norm<T> (kernel_src/csrc/loquetier_ops.cc:326-358,
 * kernel_src/csrc/rms_norm/rms_norm_cutlass.cu:158-186) behind `loquetier.ops._kernels.rms_norm`:
 *   rms_out[row] = rsqrt(mean(x[row]^2) + eps)   (fp32, the reference's [rows, 1] tensor)
 *   out[row]     = T(float(x[row]) * rms_out[row] * float(w))
 * x, out [rows, cols] and w [cols] in the 16-bit `dtype`, 16-byte aligned; cols a multiple of 8
 * (otherwise SMLM_ERR_NO_KERNEL, the reference's "No suitable kernel.").  Runs on `stream` and does
 * not synchronise (the reference launches on the default stream and then synchronises `stream`). */
int smlm_b200_rms_norm(void* out, float* rms_out, const void* x, const void* w, int rows, int cols, float eps,
                       int dtype, void* stream);

/* Bytes of the workspace of smlm_b200_rms_norm_bwd (fp32 partial sums of dW, one row per CTA). */
size_t smlm_b200_rms_norm_bwd_workspace_bytes(int rows, int cols);

/* Backward of the above; replaces the torch expressions of rms_norm.backward
 * (src/loquetier_src/kernel_utils.py:166-176), which the reference runs as separate passes:
 *   dW = sum_rows(x * rms * gO)      dX = (gO * w - x * dot * rms^2 / cols) * rms,  dot = sum_cols(gO * w * x)
 * go, x, dx [rows, cols] and w in `dtype`; rms [rows] fp32 as written by the forward; dw [cols] in
 * `dtype`, or fp32 when dw_fp32 is set.  Sums are formed in fp32 in a fixed order.  The workspace needs
 * no initialisation.  rows must be positive. */
int smlm_b200_rms_norm_bwd(void* dx, void* dw, const void* go, const void* x, const void* w, const float* rms,
                           void* workspace, size_t workspace_bytes, int rows, int cols, int dtype, int dw_fp32,
                           void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMLM_B200_H_ */
