/*
 * splash_b200 — C ABI of the B200 (sm_100a) splash-attention path.
 *
 * The reference (primatrix/tokamax) has no C ABI: its splash attention is reached through two
 * Python interfaces (tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py
 * and tokamax/_src/ops/attention/api.py).  Each entry point below names the reference function it
 * stands in for, so a binding (ctypes, XLA custom call, pybind11 ...) can replace that function's
 * device work one-for-one.
 *
 * Conventions
 *   - Plain C types only.  Device buffers are raw pointers owned by the caller; the library
 *     allocates no device memory.  Scratch comes from the caller (splash_bwd_workspace_bytes).
 *   - Every call enqueues work on the given stream and returns without synchronising.
 *   - Return value: 0 (SPLASH_OK) or a negative SplashStatus.  Nothing aborts or throws.
 *   - Asynchronous kernel faults (a bounded wait that ran out) are reported through a
 *     caller-provided 4-word device error record, read back with splash_read_error.
 *   - Tensors are (batch, heads, seq, head_dim) with element strides; head_dim must be
 *     contiguous (stride 1), a multiple of 8 and at most 256 (q / k and v / o may differ; the
 *     e4m3 forward takes 128 only), and every other stride a multiple of 8 elements (16 bytes), so the
 *     reference's [heads, seq, dim] layout, the Op layout [batch, seq, heads, dim] and the
 *     head-sharded layout the context-parallel exchange produces are all consumed without copies.
 */
#ifndef SPLASH_B200_H_
#define SPLASH_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum SplashStatus {
  SPLASH_OK = 0,
  SPLASH_ERR_INVALID_ARGUMENT = -1, /* shapes / strides / block sizes the kernels do not take */
  SPLASH_ERR_UNSUPPORTED = -2,      /* valid for the reference, not built here (maps to NotImplementedError) */
  SPLASH_ERR_CUDA = -3,             /* a CUDA runtime / driver call failed */
  SPLASH_ERR_NO_DEVICE = -4,        /* no sm_100 device / driver entry point missing */
  SPLASH_ERR_KERNEL_TIMEOUT = -5,   /* a device-side bounded wait ran out (see error record) */
  SPLASH_ERR_OUT_OF_MEMORY = -6,    /* host allocation failed */
  SPLASH_ERR_TOO_LARGE = -7         /* size beyond a fixed built-in limit */
} SplashStatus;

typedef enum SplashDType {
  SPLASH_BF16 = 0,
  SPLASH_F32 = 1,
  SPLASH_F8E4M3 = 2
} SplashDType;

/* (batch, heads, seq, head_dim) view of device memory. */
typedef struct SplashTensor {
  void* data;
  int32_t dtype;      /* SplashDType */
  int64_t size[4];    /* batch, heads, seq, head_dim */
  int64_t stride[4];  /* element strides in the same order; stride[3] == 1 */
} SplashTensor;

/* In-kernel mask function for partially masked blocks; the counterpart of the reference's
 * `mask_function` + `q_sequence` (splash_attention_mask.py:177-244, CausalMask :247,
 * ChunkedCausalMask :303, LocalMask :363).  Every one of them keeps key j for query i iff
 * lo(i) <= j <= hi(i):
 *   CAUSAL : hi = i + offset
 *   LOCAL  : lo = i + offset - left (if has_left), hi = i + offset + right (if has_right)
 *   CHUNKED: lo = (i / chunk) * chunk, hi = i
 * where i = q_sequence[row] (row itself when q_sequence is NULL).
 * TABLE means: read the partial block from partial_mask_blocks instead. */
typedef enum SplashMaskKind {
  SPLASH_MASK_TABLE = 0,
  SPLASH_MASK_CAUSAL = 1,
  SPLASH_MASK_LOCAL = 2,
  SPLASH_MASK_CHUNKED = 3
} SplashMaskKind;

typedef struct SplashMaskFn {
  int32_t kind;       /* SplashMaskKind */
  int32_t offset;     /* CAUSAL, LOCAL */
  int32_t left;       /* LOCAL */
  int32_t right;      /* LOCAL */
  int32_t has_left;   /* LOCAL: 0 = unbounded */
  int32_t has_right;  /* LOCAL: 0 = unbounded */
  int32_t chunk;      /* CHUNKED */
} SplashMaskFn;

/* ------------------------------------------------------------------------------------------
 * MaskInfo builder (host).  Replaces `_process_mask`
 * (splash_attention_mask_info.py:357-570; process_mask / process_mask_dkv :573-574), including
 * `_generate_shard_metadata` (:183-228) and `_downcast_to_small_type` (:91-124).
 *
 * The mask is given as an expression tree in post-order (children before parents); the last
 * node is the root.  Leaves: FULL, CAUSAL, LOCAL, CHUNKED (evaluated analytically per block) and
 * DENSE (a row-major bool[Sq, Skv] host array).  Inner nodes: AND, OR.
 * ---------------------------------------------------------------------------------------- */
typedef enum SplashMaskNodeKind {
  SPLASH_NODE_FULL = 0,
  SPLASH_NODE_CAUSAL = 1,
  SPLASH_NODE_LOCAL = 2,
  SPLASH_NODE_CHUNKED = 3,
  SPLASH_NODE_DENSE = 4,
  SPLASH_NODE_AND = 5,
  SPLASH_NODE_OR = 6
} SplashMaskNodeKind;

typedef struct SplashMaskNode {
  int32_t kind;            /* SplashMaskNodeKind */
  int32_t left_child;      /* AND / OR: node indices */
  int32_t right_child;
  SplashMaskFn fn;         /* CAUSAL / LOCAL / CHUNKED parameters */
  const uint8_t* dense;    /* DENSE: bool[Sq*Skv], row-major */
} SplashMaskNode;

/* Result tables, all int32 on this side of the ABI (the Python layer applies the reference's
 * int8/int16 downcast rule, which only depends on the maximum value reported here).
 * A pointer is NULL exactly where the reference returns None. */
typedef struct SplashMaskInfoOut {
  int32_t* mask_next;            /* [n_entries] or NULL */
  int32_t* active_rows;          /* [n_entries] or NULL (static grid) */
  int32_t* active_cols;          /* [n_entries] or NULL */
  int32_t* block_mask;           /* [n_entries] or NULL (all-full mask) */
  int32_t* num_active_blocks;    /* [n_shards] or NULL */
  int8_t* partial_mask_blocks;   /* [n_partial, bq, bkv] ([n_partial, bkv, bq] for dkv) or NULL */
  int64_t n_entries;
  int32_t n_shards;
  int32_t n_partial;
  int32_t all_full;              /* 1: every field above is NULL (reference's early return) */
} SplashMaskInfoOut;

int splash_maskinfo_build(const SplashMaskNode* nodes, int32_t n_nodes, int64_t q_len,
                          int64_t kv_len, int32_t block_q, int32_t block_kv, int32_t is_dkv,
                          int32_t q_seq_shards, int32_t kv_seq_shards, int32_t return_dynamic_grid,
                          SplashMaskInfoOut* out);
void splash_maskinfo_free(SplashMaskInfoOut* out);

/* ------------------------------------------------------------------------------------------
 * Kernel schedule (host).  The device kernels walk 128x128 tiles.  This expands a block-level
 * classification (what MaskInfo encodes: 0 empty / 1 partial / 2 full per (block_q, block_kv)
 * block, plus the partial-block id) into per-CTA work lists.  It is the counterpart of the
 * index maps the reference derives from MaskInfo at call time
 * (splash_attention_kernel.py:663-696 forward, :1512-1592 backward; find_bounds,
 * splash_attention_mask_info.py:33-47).
 *
 *   kind 0 (forward): one row per pair of q tiles; entry = kv tile.
 *   kind 1 (dq)     : one row per q tile;          entry = kv tile.
 *   kind 2 (dkv)    : one row per kv tile;         entry = q tile.
 * Entry layout (4 x int32): [0] tile index along the walked axis, [1] state of sub-tile 0 in
 * bits 0-1 and of sub-tile 1 in bits 2-3 (0 skip, 1 partial, 2 full); bits 4 / 5, written by
 * splash_segment_schedule only: sub-tile 0 / 1 lies inside one segment (every token of its q tile
 * and of its kv tile carries the same id), so the kernels need not compare ids element by element;
 * [2]/[3] partial-block id of sub-tile 0/1 (-1 if none).
 * ---------------------------------------------------------------------------------------- */
typedef struct SplashScheduleOut {
  int32_t* row_ptr;   /* [n_rows + 1] */
  int32_t* entries;   /* [n_entries * 4] */
  int32_t n_rows;
  int64_t n_entries;
  int32_t* row_order; /* [n_rows]: rows by decreasing entry count (ties by row index) */
} SplashScheduleOut;

int splash_schedule_build(const int32_t* block_state, const int32_t* partial_id, int32_t n_q_blocks,
                          int32_t n_kv_blocks, int32_t block_q, int32_t block_kv, int32_t kind,
                          SplashScheduleOut* out);
void splash_schedule_free(SplashScheduleOut* out);

/* Device-resident schedule + mask data shared by the kernels. */
typedef struct SplashDeviceSchedule {
  const int32_t* row_ptr;            /* device, [n_rows + 1] */
  const int32_t* entries;            /* device, [n_entries * 4], 16-byte aligned */
  int32_t n_rows;
  const int8_t* partial_mask_blocks; /* device, [n_partial, pm_rows, pm_cols] or NULL */
  int32_t block_q;                   /* block shape the partial blocks were cut with */
  int32_t block_kv;
  int64_t n_entries;                 /* entries in the list (needed by splash_segment_schedule) */
  /* Per-batch-row specialisation written by splash_segment_schedule; zero / NULL otherwise. */
  const int32_t* row_end;            /* device, [batch, n_rows]: end of each row's entries; NULL:
                                        row r ends at row_ptr[r + 1] */
  int64_t entries_per_batch;         /* batch row b reads entries + b * entries_per_batch * 4 */
  /* Launch order of the rows, longest first, so that the last CTAs of a grid are the short ones
   * (SplashScheduleOut.row_order uploaded as is).  NULL: the kernels fall back to an order that
   * suits causal masks (forward / dq: last row first; dkv: first row first). */
  const int32_t* row_order;          /* device, [n_rows] or NULL */
} SplashDeviceSchedule;

/* ------------------------------------------------------------------------------------------
 * Segment-aware schedules (device).  With segment ids the reference masks element by element
 * only (splash_attention_kernel.py:262-278); tiles whose q and kv segment-id ranges do not
 * overlap contribute nothing, so they can be dropped before the kernels run.  This call filters
 * a schedule per batch row: it computes the [min, max] segment id of every 128-token tile and
 * writes, for each batch row, the entries that can still hold an unmasked pair (sub-tile states
 * are lowered to 0 where they cannot) and marks the sub-tiles that lie inside one segment (entry
 * bits 4 / 5).  Results are unchanged; only skipped work differs.
 *
 * `in` is a schedule of `kind` (0 forward, 1 dq, 2 dkv, as in splash_schedule_build) with
 * n_entries filled in.  `out` receives device pointers into `workspace`
 * (splash_segment_schedule_bytes bytes, 256-byte aligned) and is then passed to splash_fwd /
 * splash_bwd in place of `in`.  Enqueued on the stream; no host synchronisation.
 * ---------------------------------------------------------------------------------------- */
size_t splash_segment_schedule_bytes(int64_t batch, int64_t q_len, int64_t kv_len, int32_t n_rows,
                                     int64_t n_entries);
int splash_segment_schedule(const SplashDeviceSchedule* in, int32_t kind, const int32_t* q_segment_ids,
                            const int32_t* kv_segment_ids, int64_t batch, int64_t q_len, int64_t kv_len,
                            void* workspace, size_t workspace_bytes, SplashDeviceSchedule* out,
                            void* cuda_stream);

/* ------------------------------------------------------------------------------------------
 * Schedules for a mask that is data on the device (device).  Replaces `_process_dynamic_mask`
 * (splash_attention_mask_info.py:231-350; factories splash_attention_kernel.py:2134-2226) for the
 * kernels' purposes: nothing goes through the host, so a mask may change every call.
 *
 * splash_mask_tile_states: `mask` is [q_len, kv_len] bytes (0 = masked, anything else = keep; a
 * bool or int8 array), 16-byte aligned rows (`row_stride_bytes` a multiple of 16); writes the state
 * of every 128x128 tile (0 empty, 1 partial, 2 full) to `states` [q_len / 128, kv_len / 128].
 *
 * splash_dynamic_schedule: turns `states` into a schedule of `kind` (as in splash_schedule_build)
 * inside `workspace` (splash_dynamic_schedule_bytes bytes, 256-byte aligned): rows at a fixed
 * stride with `row_end` replicated for `batch` rows.  `partial_blocks` is what the attention
 * kernels read for partial tiles — the mask itself [q_len, kv_len] for kinds 0 and 1, its
 * transpose [kv_len, q_len] for kind 2 — registered as one partial block covering the whole mask.
 * The result cannot be passed to splash_segment_schedule (segment ids are still applied
 * element by element by the kernels).
 * ---------------------------------------------------------------------------------------- */
int splash_mask_tile_states(const void* mask, int64_t row_stride_bytes, int64_t q_len, int64_t kv_len,
                            int32_t* states, void* cuda_stream);
size_t splash_dynamic_schedule_bytes(int64_t q_len, int64_t kv_len, int32_t kind, int64_t batch);
int splash_dynamic_schedule(const int32_t* states, int64_t q_len, int64_t kv_len, int32_t kind, int64_t batch,
                            const void* partial_blocks, void* workspace, size_t workspace_bytes,
                            SplashDeviceSchedule* out, void* cuda_stream);

/* ------------------------------------------------------------------------------------------
 * Forward.  Replaces `_splash_attention_forward` + `flash_attention_kernel`
 * (splash_attention_kernel.py:550-995, :299-527): o = softmax(mask(scale * q k^T)) v with fp32
 * accumulation, plus logsumexp and max_logits (natural log, fp32 [batch, q_heads, q_len]).
 * q head h reads kv head h / (q_heads / kv_heads) (:675-682).
 * ---------------------------------------------------------------------------------------- */
/* Optional second destination of an output, for context parallelism (the Ulysses exchange fused
 * into the kernel that produces the tensor): besides its ordinary destination, every row of the
 * output is also stored — plain 16-byte stores over NVLink, no TMA, no multicast — into the buffer
 * of the rank that owns that row in the sequence-sharded layout [batch, all heads, rows_per_peer,
 * head_dim].  Sequence row s of local head h goes to rank s / rows_per_peer, at
 *   ptrs[rank] + base_bytes + 2 * (batch * stride_b + (head0 + h) * stride_h + (s % rows_per_peer) * stride_s).
 * `ptrs` is a device array with one entry per rank: the address at which that rank's buffer is mapped
 * in this process (symmetric memory / IPC; this rank's own buffer included).  The caller orders the
 * kernel between two barriers across the ranks: receive buffers free before, all stores landed after.
 * ptrs == NULL: no second destination.  The reference has no counterpart (its context-parallel
 * wrapper is ring attention, ring_attention_kernel.py:68-293). */
typedef struct SplashPeerOutput {
  const uint64_t* ptrs;
  int64_t base_bytes;
  int64_t rows_per_peer;
  int64_t stride_b, stride_h, stride_s;  /* elements */
  int32_t head0;
} SplashPeerOutput;

typedef struct SplashFwdArgs {
  SplashTensor q, k, v, o;          /* bf16 */
  float* logsumexp;                 /* may be NULL */
  float* max_logits;                /* may be NULL */
  const int32_t* q_segment_ids;     /* [batch, q_len] or NULL */
  const int32_t* kv_segment_ids;    /* [batch, kv_len] or NULL (both or neither) */
  const int32_t* q_sequence;        /* [q_len] or NULL (= arange) */
  SplashDeviceSchedule sched;       /* kind 0 */
  SplashMaskFn mask_fn;
  float scale;                      /* multiplies q k^T in fp32 */
  float mask_value;                 /* written to logsumexp / max_logits of rows with no work */
  uint32_t* error_record;           /* device, 4 words, zeroed by the caller */
  /* Attention sinks (splash_attention_kernel.py:375-395, base.py:96-104): one extra logit per q
   * head that joins the softmax of every row of that head without a value: the running maximum
   * starts at it and l at 1.  Device fp32 [q_heads], in the units of scale * q k^T; NULL: none. */
  const float* sinks;
  /* Fixed maximum (`max_logit_const` / `max_logit_value`, splash_attention_kernel.py:363-369,
   * :440-470): exp(logit - value) is used for every tile, no running maximum is computed and
   * max_logits returns the value.  Device fp32 [q_heads]; NULL: running maximum.  Logits far
   * above the value overflow, as in the reference. */
  const float* max_logit_value;
  /* attn_logits_soft_cap (splash_attention_kernel.py:202-296, base.py:92-94): logits become
   * cap * tanh(scale * q k^T / cap) before masking.  0 = off.  bf16 inputs only. */
  float soft_cap;
  /* Second destination of `o` in other ranks' memory; bf16 kernels with head dims up to 128 only
   * (SPLASH_ERR_UNSUPPORTED otherwise). */
  SplashPeerOutput o_peer;
} SplashFwdArgs;

int splash_fwd(const SplashFwdArgs* args, void* cuda_stream);

/* Forward for e4m3 inputs (inference prefill).  No counterpart in the reference, whose splash path
 * rejects everything but bf16 / f32 (pallas_mosaic_tpu_common.py:40-42); the contract is the bf16
 * forward above run on the dequantised tensors.
 * base.q / base.k / base.v are SPLASH_F8E4M3 (element strides multiples of 16), base.o is bf16.
 * Each scale array is fp32 [batch, heads, seq / 128]: the stored values of one 128-token tile of
 * one head times its scale are the real values.  Scales must be finite and >= 0.  Every other
 * field means what it means for splash_fwd (segment ids and sinks included; a soft cap and a fixed
 * maximum are not taken); logsumexp / max_logits refer to the dequantised logits.
 * flags: 0 keeps the probabilities in e4m3 for p v (fastest; output within a few percent of the
 * bf16 forward: relative L2 <= 3e-2); SPLASH_FP8_P_F16 keeps them 16 bits wide — q k^T on the e4m3
 * tiles, each V tile converted once to f16 in shared memory, p v as a 16-bit MMA — which meets the
 * bf16 forward's bound (max-abs <= 1e-2). */
typedef enum SplashFwdFp8Flags { SPLASH_FP8_P_F16 = 1 } SplashFwdFp8Flags;

typedef struct SplashFwdFp8Args {
  SplashFwdArgs base;
  const float* q_scale;             /* [batch, q_heads, q_len / 128] */
  const float* k_scale;             /* [batch, kv_heads, kv_len / 128] */
  const float* v_scale;             /* [batch, kv_heads, kv_len / 128] */
  uint32_t flags;                   /* SplashFwdFp8Flags */
} SplashFwdFp8Args;

int splash_fwd_fp8(const SplashFwdFp8Args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------------
 * Backward.  Replaces `_splash_attention_bwd` + `_splash_attention_bwd_dkv` +
 * `_flash_attention_dkv_kernel` (splash_attention_kernel.py:1871-1947, :1462-1868, :1234-1459):
 * di = sum(o * do), then dq (q-tile stationary) and dk/dv (kv-tile stationary, the q heads of a
 * kv head summed inside one CTA in fp32 — no atomics, bitwise repeatable).
 * Workspace: splash_bwd_workspace_bytes(batch, q_heads, q_len) bytes, 256-byte aligned.
 * ---------------------------------------------------------------------------------------- */
typedef struct SplashBwdArgs {
  SplashTensor q, k, v, o, d_o;     /* bf16 inputs */
  SplashTensor dq, dk, dv;          /* bf16 outputs */
  const float* logsumexp;           /* forward result, natural log */
  const int32_t* q_segment_ids;
  const int32_t* kv_segment_ids;
  const int32_t* q_sequence;
  SplashDeviceSchedule sched_dq;    /* kind 1 */
  SplashDeviceSchedule sched_dkv;   /* kind 2 */
  SplashMaskFn mask_fn;
  float scale;
  void* workspace;
  size_t workspace_bytes;
  uint32_t* error_record;
  uint32_t launch_mask;             /* 0 = everything; else bit 0 di pass, bit 1 dq kernel, bit 2
                                       dkv kernel (for timing / profiling one kernel alone; the di
                                       pass must have run on this workspace before bits 1 or 2) */
  float soft_cap;                   /* as in SplashFwdArgs; dS gains the factor 1 - tanh^2
                                       (base.py:159-163).  0 = off */
  uint32_t flags;                   /* SplashBwdFlags; 0 = split form */
  /* Second destinations of dq / dk / dv in other ranks' memory (see SplashPeerOutput; dk_peer and
   * dv_peer are laid out over all kv heads).  dk / dv rows leave from the epilogue of the kernel
   * that accumulates them, dq rows from the cast pass.  Fused form with head dims up to 128 only
   * (SPLASH_ERR_UNSUPPORTED otherwise). */
  SplashPeerOutput dq_peer, dk_peer, dv_peer;
} SplashBwdArgs;

/* SPLASH_BWD_FUSED_DQ: one kernel per (kv tile, kv head) forms all three gradients, five matmuls
 * per live block, as the reference's `_flash_attention_dkv_kernel` does with its dq partials
 * (splash_attention_kernel.py:1395-1410, reduced at :1864).  Here the partials are added into an
 * fp32 dQ image in the workspace by vector reductions and a last pass scales and casts it, so the
 * workspace is splash_bwd_fused_workspace_bytes and `sched_dq` is not read.  dK / dV are still
 * accumulated without atomics and repeat bit for bit; dQ's fp32 sums are formed in an order that
 * changes from run to run (differences in the last bits).  With this flag launch_mask bit 0 also
 * clears the image, bit 1 is the cast pass and bit 2 the fused kernel. */
typedef enum SplashBwdFlags {
  SPLASH_BWD_FUSED_DQ = 1
} SplashBwdFlags;

size_t splash_bwd_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len);
size_t splash_bwd_fused_workspace_bytes(int64_t batch, int64_t q_heads, int64_t q_len);
int splash_bwd(const SplashBwdArgs* args, void* cuda_stream);

/* Ring attention (ring_attention_kernel.py:150-158): folds one ring step's partial result
 * (o_i bf16 [n_rows, 128], its logsumexp lse_i [n_rows]) into the running fp32 pair in place:
 * lse_acc <- log(exp(lse_acc) + exp(lse_i)), o_acc <- the logsumexp-weighted mean.  Start with
 * o_acc = 0, lse_acc = -inf.  n_rows = batch * q_heads * q_len of contiguous rows. */
int splash_ring_merge(float* o_acc, float* lse_acc, const void* o_i, const float* lse_i, int64_t n_rows,
                      int64_t head_dim, void* cuda_stream);

/* ------------------------------------------------------------------------------------------
 * Context-parallel exchange by peer stores (sequence shard <-> head shard, the Ulysses all-to-all).
 * The reference has no all-to-all — its context-parallel wrapper is ring attention over
 * lax.ppermute (ring_attention_kernel.py:95-99) — so this stands where
 * `jax.lax.all_to_all(x, axis, split_axis=heads, concat_axis=seq)` would around the kernels.
 *
 * seq_to_head = 1: `src` is this rank's [batch, h_loc * world, s_loc, head_dim] (its sequence shard
 * of all heads); peer j receives heads [j * h_loc, (j + 1) * h_loc) at sequence offset
 * rank * s_loc of its [batch, h_loc, s_loc * world, head_dim] buffer.  seq_to_head = 0 is the
 * inverse.  `dst_ptrs` is a DEVICE array of `world` pointers to the ranks' receive buffers (peer
 * mappings of symmetric / IPC memory; entry `rank` is this rank's own buffer), every one laid out as
 * the kernels read it, so there is no pack or unpack pass.  Plain 16-byte loads and stores: no TMA,
 * no multicast.  The caller orders the ranks: a barrier before the call (receive buffers no longer
 * in use) and one after it (all pushes have landed); any stream-ordered collective does (the Python
 * layer uses a one-element NCCL all-reduce).  Tensors are contiguous; row_bytes =
 * head_dim * element size must be a multiple of 16. */
typedef struct SplashExchangeArgs {
  const void* src;
  void* const* dst_ptrs;   /* device memory: world pointers */
  int32_t world, rank;
  int32_t seq_to_head;
  int64_t batch, h_loc, s_loc, row_bytes;
  int64_t dst_base_bytes;  /* offset of the receive buffer inside each rank's mapped block (the same
                              on every rank for symmetric allocations; 0 if dst_ptrs point at the
                              buffers themselves); a multiple of 16 */
} SplashExchangeArgs;
int splash_exchange_push(const SplashExchangeArgs* args, void* cuda_stream);

/* Backward pass for callers that cannot obtain device memory at the point of the call.
 * (No counterpart in the reference; it exists only on this side of the boundary.)
 *
 * splash_bwd needs a scratch buffer for the per-row terms di and -logsumexp*log2(e).  Some
 * callers have no way to provide one when the backward runs: a plugin or custom-call handler that
 * is only handed its operand and result buffers by the runtime that invokes it; code that runs
 * after the process has handed all remaining device memory to another allocator; or a caller whose
 * allocator is not safe to enter from the thread or callback the backward is issued from.  This
 * variant takes the same SplashBwdArgs, ignores `workspace` / `workspace_bytes` (and always runs
 * the split form, whatever `flags` says: the fused form's dQ image would not fit), and keeps the
 * scratch in an array that is part of the loaded library image on every GPU: it performs no
 * cudaMalloc / cudaFree and calls nothing that allocates.
 *
 * Limit: batch * q_heads * q_len <= SPLASH_STATIC_SCRATCH_MAX_ROWS (the array is
 * 2 * 4 * SPLASH_STATIC_SCRATCH_MAX_ROWS bytes = 8 MiB, held by each GPU that loads the library
 * until the process exits).  Larger problems return SPLASH_ERR_TOO_LARGE and launch nothing.
 *
 * The first call on a device looks up the array's device address (once per device, with that
 * device current); make that first call outside any stream capture.  The array is shared by
 * every call on the device and keeps the previous call's contents; nothing in it has to start at
 * zero, because the di pass overwrites every row a call later reads.  Two calls whose kernels
 * can overlap on the same GPU (different streams without an ordering between them) race on the
 * array — order them, or use splash_bwd with separate workspaces. */
#define SPLASH_STATIC_SCRATCH_MAX_ROWS (1 << 20)
int splash_bwd_static_scratch(const SplashBwdArgs* args, void* cuda_stream);

/* Copies the 4-word device error record to host (synchronises the stream) and maps it to a
 * status: SPLASH_OK or SPLASH_ERR_KERNEL_TIMEOUT.  record_out may be NULL. */
int splash_read_error(const uint32_t* error_record, void* cuda_stream, uint32_t record_out[4]);

/* Diagnostic for the error path (no counterpart in the reference): launches one tiny kernel in
 * which a thread waits, through the same bounded wait the attention kernels use, on a barrier
 * nothing ever arrives on.  The wait gives up after `limit_cycles` SM cycles (1 .. 1e8, i.e. at
 * most some tens of milliseconds), the kernel writes {1, block, tag, thread} to the record and
 * returns; splash_read_error then reports SPLASH_ERR_KERNEL_TIMEOUT.  Lets an integration check
 * its handling of a device-side timeout without hanging anything. */
int splash_probe_bounded_wait(uint32_t* error_record, int64_t limit_cycles, uint32_t tag, void* cuda_stream);

/* XLA custom-call adapter (tokamax_b200/csrc/splash_xla_ffi.cc; stands where the reference calls
 * `pl.pallas_call`, splash_attention_kernel.py:888, :1840).  When the library is built with XLA's
 * "xla/ffi/api/ffi.h" on the include path it also exports the FFI handlers `SplashFwd` and
 * `SplashBwd` (XLA_FFI_DEFINE_HANDLER_SYMBOL) for jax.ffi.register_ffi_target;
 * splash_xla_ffi_compiled says whether it was (1) or not (0).  splash_xla_ffi_signature(0 | 1)
 * returns the forward / backward handler's operands, results and attributes in binding order as
 * "operands=name:kind,...;results=...;attrs=name:type,...;". */
int splash_xla_ffi_compiled(void);
const char* splash_xla_ffi_signature(int which);

/* Human-readable text for a SplashStatus.  Never NULL. */
const char* splash_status_str(int status);

/* Library / build identification: "splash_b200 <version> sm_100a". */
const char* splash_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SPLASH_B200_H_ */
