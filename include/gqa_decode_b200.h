/*
 * C ABI of the B200 (sm_100a) GQA decode-attention library.
 *
 * This is the boundary a binding of alityb/gqa-decode would call instead of its
 * CuTe-DSL JIT callables.  Every function takes plain pointers and sizes, returns an
 * int (0 = ok, negative = bad argument (GQA_ERR_*), positive = cudaError_t), never
 * throws, never exits, never allocates or frees device memory unless its comment says
 * so, and enqueues its work on the CUDA stream it is given without synchronising.
 * Device pointers must be 16-byte aligned and refer to the device that is current on
 * the calling thread.
 *
 * Citations `gqa_decode/...py:N` name the reference interface each entry replaces.
 */
#ifndef GQA_DECODE_B200_H_
#define GQA_DECODE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define GQA_DTYPE_BF16 0
#define GQA_DTYPE_FP16 1
#define GQA_DTYPE_E4M3 2

/* K/V memory layouts (rows of head_dim elements, every (sequence, KV head) slab contiguous
 * exactly like the reference's [Hkv, S, D] tensors, gqa_decode/gqa_decode.py:44) */
#define GQA_LAYOUT_PADDED 0 /* [batch, Hkv, max_seq_len, D]; batch = 1 is the reference layout */
#define GQA_LAYOUT_PACKED 1 /* sequence b holds [Hkv, len_b, D], sequences back to back */
/* Paged caches as serving engines hold them (the reference has only contiguous tensors): key r
 * of sequence b lives in page block_table[b * block_table_stride + r / page_size], row
 * r % page_size.  page_size is a multiple of 16 that divides, or is a multiple of, the tile
 * (gqa_decode_tile_rows()).  Entries of the table past a sequence's last page are ignored. */
#define GQA_LAYOUT_PAGED_HND 2 /* [num_pages, Hkv, page_size, D] */
#define GQA_LAYOUT_PAGED_NHD 3 /* [num_pages, page_size, Hkv, D] */

/* flags */
#define GQA_FLAG_SEPARATE_MERGE 1 /* run the merge as a second kernel instead of in-kernel */
#define GQA_FLAG_NO_MERGE 2       /* explicit splits only: write every partial, merge nothing */
#define GQA_FLAG_WORK_STEALING 8   /* balanced schedule: CTAs that finish their own share steal work
                                     chunks from others.  Off by default: on an otherwise idle GPU
                                     the static shares finish within a few percent of each other;
                                     useful when SMs are shared with other work.  With it the
                                     float32 summation order, hence the last bits of the result,
                                     depend on timing; without it results are bit-reproducible */
#define GQA_FLAG_FP8_EXACT_V 4    /* E4M3: round every dequantised V element to the 16-bit type like
                                     dequantize_kv_fp8 (gqa_decode/fp8_utils.py:54-55) instead of
                                     applying the V scale once to the fp32 output (default, faster) */
#define GQA_FLAG_CLEAR_WORKSPACE 16 /* zero the workspace's control words (one small memset node on the
                                     stream, after the arguments have been checked) before the
                                     launch: for a workspace whose contents are unknown, or that
                                     last served a launch of another geometry */
#define GQA_FLAG_TICKET_MERGE 64   /* find out that a group's partials are complete with atomic
                                     tickets.  Default for the static schedules is cheaper: partials
                                     announce themselves (a word that is not zero has arrived) and
                                     the CTA that writes a group's last partial polls for the rest,
                                     which needs the workspace's partial area to be all zero at
                                     launch (kernels leave it so); with tickets only the control
                                     words need to be zero */
#define GQA_FLAG_DEPENDENT_LAUNCH 32 /* launch with programmatic stream serialization: the kernel's
                                     prologue (and, for uniform lengths, its scheduling) overlaps the
                                     end of the previous kernel on the stream; it waits for that
                                     kernel before it reads any input or touches the workspace.
                                     Hides the launch gap between back-to-back steps */

/* errors */
#define GQA_ERR_ARG (-1)       /* null pointer, non-positive size, misaligned pointer */
#define GQA_ERR_SHAPE (-2)     /* unsupported head_dim / group size / dtype combination */
#define GQA_ERR_WORKSPACE (-3) /* workspace too small */
#define GQA_ERR_DRIVER (-4)    /* cuTensorMapEncodeTiled unavailable or failed */
#define GQA_ERR_LIMIT (-5)     /* size beyond a documented maximum */
#define GQA_ERR_INTERNAL (-6)  /* a self-check of the library failed (please report) */

/*
 * One decode step over a batch.  Replaces the argument lists of
 * gqa_decode_attention (gqa_decode/gqa_decode.py:672-681),
 * gqa_decode_attention_fp8 (:1900-1910) and gqa_decode_attention_persistent
 * (:1365-1371); batch/seq_lens/layout are additions (the reference is single-sequence).
 */
typedef struct gqa_decode_args {
  const void* q;            /* [batch, num_q_heads, head_dim], q_dtype (bf16 or fp16) */
  const void* k;            /* K cache, kv_dtype, layout above */
  const void* v;            /* V cache, same shape and type as k */
  void* out;                /* [batch, num_q_heads, head_dim] in q_dtype; may be NULL if out_f32 given */
  float* out_f32;           /* optional fp32 copy of the output (sequence-shard partials) */
  float* out_lse;           /* optional [batch, num_q_heads] natural-log sum-exp of the scaled scores */
  const int32_t* seq_lens;  /* device [batch] KV lengths, or NULL: every sequence has max_seq_len keys */
  const float* k_scale;     /* E4M3 only: device [batch * num_kv_heads] dequantisation scales */
  const float* v_scale;     /* E4M3 only: same */
  int32_t batch;
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;         /* 64, 128 or 256 (E4M3: 64 or 128) */
  int32_t max_seq_len;      /* rows per head slab (padded layout); bound on every length */
  int64_t total_rows;       /* rows of the whole K (= V) allocation, viewed as [rows, head_dim]
                               (paged: num_pages * num_kv_heads * page_size) */
  int32_t q_dtype;          /* GQA_DTYPE_BF16 | GQA_DTYPE_FP16 */
  int32_t kv_dtype;         /* q_dtype, or GQA_DTYPE_E4M3 */
  int32_t kv_layout;        /* GQA_LAYOUT_* */
  int32_t num_splits;       /* 0: balanced persistent schedule; K>0: K partials per (sequence, KV head) */
  int32_t num_ctas;         /* 0: one CTA per SM */
  int32_t flags;            /* GQA_FLAG_* */
  float softmax_scale;      /* 0: head_dim ** -0.5 (gqa_decode/gqa_decode.py:60) */
  void* workspace;          /* device scratch of gqa_decode_workspace_bytes(); reusable across calls */
  size_t workspace_bytes;
  void* stream;             /* cudaStream_t */
  const int32_t* block_table;  /* paged layouts: device [batch, block_table_stride] page numbers */
  int32_t page_size;           /* paged layouts: rows per page */
  int32_t block_table_stride;  /* paged layouts: table entries per sequence */
  uint64_t wait_limit_ns;      /* bound on every wait inside the kernel (a tile that never lands,
                                  a peer GPU's flag); on expiry a status bit is set and the
                                  kernel returns.  0: two seconds */
  uint64_t* debug_timestamps;  /* optional diagnostics: device buffer of 12 * num_ctas uint64; per
                                  CTA {prologue done, first load issued, first tile landed, start
                                  of the last segment's epilogue, end, start of the CTA's merge
                                  or 0} in %globaltimer ns, {SM id, tiles consumed}, then three
                                  more times of that merge and a spare word */
} gqa_decode_args_t;

/*
 * Bytes of device scratch a launch with these sizes needs (partials, tickets, status).
 *
 * Workspace contract.  The library keeps no record of workspaces.  A workspace holds
 * control words (status, tickets, counters) and partial results; what a launch uses of it
 * must be ZERO when the launch starts, and kernels leave it zero when they finish with
 * status 0 (the default in-kernel merge hands its partials back as zeros; launches with
 * GQA_FLAG_SEPARATE_MERGE, _NO_MERGE, _WORK_STEALING or _TICKET_MERGE need only the control
 * words zero and leave their partials behind).  Where control words and partials lie depends
 * on the launch geometry.  So: zero a workspace when it is created
 * (gqa_decode_workspace_reset), and set GQA_FLAG_CLEAR_WORKSPACE (or call
 * gqa_decode_workspace_reset) on the first launch after the geometry - batch, head counts,
 * head_dim, num_splits, num_ctas, workspace_bytes, the merge flags - changed and after a
 * launch that reported a non-zero status.  GQA_FLAG_CLEAR_WORKSPACE zeroes exactly what the
 * launch uses (tens of megabytes for the default merge, a few kilobytes otherwise).  A
 * workspace serves one launch at a time: launches that may overlap on the GPU need one each.
 */
int gqa_decode_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                               int32_t head_dim, int32_t num_splits, int32_t num_ctas,
                               size_t* bytes);


/*
 * Byte offsets inside a workspace for explicit splits (num_splits = K > 0): offsets[0]
 * status word, [1] tickets, [2] group table, [3] partial log-sum-exp [slots, G] fp32,
 * [4] partial outputs [slots, G, head_dim] fp32, [5] total bytes;
 * slot = (sequence * Hkv + kv_head) * K + split.  Lets a caller that asked for
 * GQA_FLAG_NO_MERGE read the partials (the reference's reduction="python" path,
 * gqa_decode/gqa_decode.py:753-756).
 */
int gqa_decode_workspace_layout(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                int32_t head_dim, int32_t num_splits, int32_t num_ctas,
                                size_t offsets[6]);

/* Zero a whole workspace on the stream.  Call once after allocating it and after any launch
 * that reported a non-zero status. */
int gqa_decode_workspace_reset(void* workspace, size_t workspace_bytes, void* stream);

/* Copy the status word back (synchronises the stream): 0 = ok, else OR of
 * 1 (consumer wait expired), 2 (producer wait expired), 4 (shared-memory misalignment),
 * 8 (a partial-slot index was out of range: the control words were not clean),
 * 16 (a peer GPU's flag never arrived: sequence exchange, head gather),
 * 32 (a partial never arrived at the CTA merging its group: the workspace was not clean). */
int gqa_decode_read_status(const void* workspace, void* stream, int32_t* status);

/* bf16 / fp16 K and V.  Replaces gqa_decode_attention, gqa_decode/gqa_decode.py:672-762
 * (DirectDecodeKernel :105, SplitKDecodeKernel :235, DoubleBufferSplitKKernel :1043,
 * ReductionKernel :419). */
int gqa_decode_attention(const gqa_decode_args_t* args);

/* Same kernel, always the balanced persistent schedule.  Replaces
 * gqa_decode_attention_persistent, gqa_decode/gqa_decode.py:1365-1446
 * (PersistentDecodeKernel :771). */
int gqa_decode_attention_persistent(const gqa_decode_args_t* args);

/*
 * Variant of gqa_decode_attention for callers that cannot hand the library a scratch
 * buffer.  (No counterpart in the reference: its host code allocates three partial
 * tensors per call with torch.)
 *
 * Who needs it: a serving engine that gave all of HBM to its own KV-cache pool at
 * start-up, so a later cudaMalloc would fail or fragment it; a latency-critical decode
 * loop that cannot accept the device-wide synchronisation an allocation may trigger;
 * a host-language binding (cgo, JNI, a plugin sandbox) that can pass the tensors it was
 * given but has no way to own and free a device buffer of its own.
 *
 * What it does: identical inputs, outputs and arithmetic to gqa_decode_attention
 * (bf16/fp16 K and V, any schedule), but the partials, tickets and status word live in a
 * fixed array of GQA_STATIC_SCRATCH_BYTES (16 MiB) that is part of the library image; every GPU
 * that loads the library keeps that much memory until the process exits.  args->workspace
 * and args->workspace_bytes are ignored.  The call performs no cudaMalloc, cudaFree or
 * any other allocation.
 *
 * Limits and rules:
 *  - if the launch cannot fit the array (explicit splits need batch*Hkv*K partial slots of
 *    G*(D+1)*4 bytes each, the balanced schedule batch*Hkv + num_ctas + 2 of them) the call
 *    returns GQA_ERR_LIMIT and launches nothing;
 *  - the first call on each device looks up the array's device address (once per
 *    device, with that device current); make that first call during set-up, before any
 *    stream capture is begun;
 *  - all calls on a device share the one array, which keeps whatever the previous call
 *    left: the entry clears the tickets and the status word on the stream before each
 *    launch (after the arguments have been checked: a rejected call touches nothing), and
 *    two calls that overlap on the GPU (different streams, or different host threads) race
 *    on it - serialise them;
 *  - gqa_decode_read_status cannot be pointed at the array; a caller that wants the
 *    status word uses the workspace-taking entry instead.
 */
#define GQA_STATIC_SCRATCH_BYTES (16u << 20)
int gqa_decode_attention_static_scratch(const gqa_decode_args_t* args);

/* E4M3 K and V with per-(sequence, KV head) fp32 scales.  Replaces
 * gqa_decode_attention_fp8, gqa_decode/gqa_decode.py:1900-2010
 * (FP8DirectDecodeKernel :1454, FP8SplitKDecodeKernel :1599). */
int gqa_decode_attention_fp8(const gqa_decode_args_t* args);

/*
 * LSE-weighted merge of normalised partials.  o_parts [num_parts, rows, head_dim] fp32,
 * lse_parts [num_parts, rows] (natural log, -inf = empty partial).  Writes
 * out [rows, head_dim] in out_dtype (may be NULL), out_f32 and out_lse (optional).
 * Replaces ReductionKernel / reduce_partials, gqa_decode/gqa_decode.py:419-495, :647-669;
 * also merges the (O, LSE) partials of sequence shards gathered from other GPUs.
 */
int gqa_merge_partials(const float* o_parts, const float* lse_parts, int32_t num_parts,
                       int64_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                       float* out_f32, float* out_lse, void* stream);

/*
 * Per-KV-head E4M3 quantisation on the GPU.  Replaces the tensor-op passes of
 * quantize_kv_fp8, gqa_decode/fp8_utils.py:8-43, for one cache tensor (call it for K and for
 * V): x [num_heads, elems_per_head] bf16/fp16 (a head's [S, D] slab flattened,
 * elems_per_head % 8 == 0), codes same shape uint8 (E4M3 bit patterns), scales [num_heads]
 * fp32 (multiply to dequantise), amax_scratch [num_heads] fp32 (overwritten).  Bit-identical
 * to the reference arithmetic.
 */
int gqa_quantize_kv_fp8(const void* x, int32_t x_dtype, int64_t num_heads, int64_t elems_per_head,
                        uint8_t* codes, float* scales, float* amax_scratch, void* stream);

/*
 * Head-sharded decode whose outputs are gathered on every rank inside the same kernel (no
 * counterpart in the reference, which is single-GPU; this is the hand-off a tensor-parallel
 * layer otherwise does with an all-gather after attention).  Rank r of `world` runs its KV
 * heads exactly as gqa_decode_attention[_fp8] would (args->num_q_heads / num_kv_heads are the
 * LOCAL head counts, args->out is ignored) and writes every final row with plain peer stores
 * into every rank's [batch, world * num_q_heads, head_dim] buffer at head offset
 * r * num_q_heads.  The last CTA then raises flag[epoch parity][r] = epoch on every peer
 * (release, system scope) and waits - bounded, status bit 16 on expiry - for every peer's
 * flag, so that when the kernel ends the gathered tensor in this rank's buffer is complete.
 * peer_out / peer_flags are HOST arrays of `world` device pointers as mapped in this process
 * (symmetric memory); flags are 2 * world uint32 per rank, zero before the first call;
 * epoch starts at 1 and grows by one per call, the same on all ranks.  Callers alternate
 * between two output buffers by epoch parity when consecutive steps may overlap across
 * ranks.  Needs the in-kernel merge and the static schedule (no GQA_FLAG_SEPARATE_MERGE,
 * _NO_MERGE, _WORK_STEALING); world <= 8.  No multicast, no NVLS: plain loads and stores.
 */
#define GQA_GATHER_HEADS 0    /* ranks own KV heads; outputs are gathered (described above) */
#define GQA_GATHER_SEQUENCE 1 /* ranks own contiguous key ranges of every head: rank r's
                                 normalised fp32 rows and log-sum-exps are pushed into every
                                 rank's receive area peer_out[p] (gqa_sequence_exchange_bytes(),
                                 zero-filled once when created) as they are produced, every value
                                 as an 8-byte word {float, epoch}: the data is its own arrival
                                 flag (peer_flags is not used).  At its end every CTA merges its
                                 share of the rows (LSE-weighted, the reference's reduce_partials
                                 algebra, gqa_decode/gqa_decode.py:661-669, across ranks) into
                                 args->out / out_f32 / out_lse of this rank, waiting - bounded,
                                 status bit 16 - for words that have not landed: one kernel per
                                 rank and step, the exchange overlaps the streaming */
typedef struct gqa_gather_args {
  void* const* peer_out;
  uint32_t* const* peer_flags;
  int32_t world;
  int32_t rank;
  uint32_t epoch;
  int32_t mode;               /* GQA_GATHER_* */
} gqa_gather_args_t;
int gqa_decode_attention_gather(const gqa_decode_args_t* args, const gqa_gather_args_t* gather);

/* Bytes of one rank's receive area for GQA_GATHER_SEQUENCE (rows = batch * num_q_heads):
 * 2 parity halves x world source ranks x (rows * head_dim + rows rounded up to even) 8-byte
 * words. */
size_t gqa_sequence_exchange_bytes(int32_t world, int64_t rows, int32_t head_dim);

/*
 * Append one token per sequence to E4M3 caches with fixed per-(sequence, head) scales: the
 * step a decode loop runs between two gqa_decode_attention_fp8 calls (the reference only
 * quantises whole caches, gqa_decode/fp8_utils.py:8-43).  Arithmetic of quantize_kv_fp8 with
 * amax = scale * 448; elements outside the head's range saturate at +-448 and are counted.
 * The token of sequence b is written to row positions[b] (normally the length before the
 * append); rows outside [0, max_seq_len) are skipped.
 */
typedef struct gqa_append_args {
  const void* k_new;           /* [batch, num_kv_heads, head_dim], src_dtype (bf16 or fp16) */
  const void* v_new;
  void* k_cache;               /* E4M3 codes: GQA_LAYOUT_PADDED or GQA_LAYOUT_PAGED_* */
  void* v_cache;
  const float* k_scale;        /* device [batch * num_kv_heads] */
  const float* v_scale;
  const int32_t* positions;    /* device [batch] */
  const int32_t* block_table;  /* paged layouts: device [batch, block_table_stride] */
  int32_t* saturated;          /* optional device counter, incremented per clamped element */
  int32_t batch;
  int32_t num_kv_heads;
  int32_t head_dim;            /* multiple of 4, at most 1024 */
  int32_t max_seq_len;         /* rows per head slab (padded), bound on positions */
  int32_t src_dtype;
  int32_t kv_layout;
  int32_t page_size;
  int32_t block_table_stride;
  void* stream;
} gqa_append_args_t;
int gqa_quantize_append_fp8(const gqa_append_args_t* args);

/*
 * Sequence-shard exchange over NVLink, fused with the merge (no counterpart in the
 * reference, which is single-GPU): every rank calls this once per decode step after its
 * local kernel wrote (local_o [rows, head_dim] fp32, local_lse [rows]).  peer_bufs is a
 * DEVICE array of `world` pointers: the receive buffer of every rank as mapped into this
 * process (symmetric memory of gqa_exchange_buffer_bytes() bytes, zero-filled once when
 * created).  The kernel pushes the local partial to all peers with plain peer stores,
 * signals them, waits (bounded by wait_limit_ns; 0 = two seconds) for all peers' partials and
 * writes the merged out / out_f32 / out_lse.  `epoch` must be > 0 and increase by one on
 * every call, on all ranks alike.  `status` (optional device word) gets bit 16 if a peer
 * never arrived; the outputs are then left untouched.
 * All ranks must be separate processes on separate GPUs of one NVLink domain.
 */
size_t gqa_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t head_dim);
int gqa_exchange_merge(const float* local_o, const float* local_lse, void* const* peer_bufs,
                       int32_t rank, int32_t world, uint32_t epoch, int64_t rows,
                       int32_t head_dim, void* out, int32_t out_dtype, float* out_f32,
                       float* out_lse, int32_t* status, uint64_t wait_limit_ns, void* stream);

/* One-wave split heuristic of the reference, gqa_decode/gqa_decode.py:80-102.
 * Returns the split count (>= 1) or a negative error. */
int gqa_select_num_splits(int32_t num_kv_heads, int32_t seq_len, int32_t block_seq,
                          int32_t target_blocks_per_sm, int32_t num_sms);

/* Keys per pipeline tile the kernels use for this configuration (schedule granularity). */
int gqa_decode_tile_rows(int32_t head_dim, int32_t kv_dtype);

/*
 * Host-side replay of the device scheduler, for inspection and tests: fills up to
 * `capacity` records of 9 int64 each {cta, seq, kv_head, row_begin, row_end, slot,
 * first_slot, n_parts, kv_row0} for the launch described by the arguments
 * (seq_lens is a HOST array here, or NULL).  Returns the number of segments, or a
 * negative error.  No GPU needed.
 */
int64_t gqa_schedule_dump(const int32_t* seq_lens_host, int32_t batch, int32_t num_kv_heads,
                          int32_t max_seq_len, int32_t tile_rows, int32_t num_ctas,
                          int32_t num_splits, int32_t kv_layout, int64_t* records,
                          int64_t capacity);

/* Same records produced by the device-side scheduler (warp-cooperative set-up) running on
 * the GPU; seq_lens is a DEVICE array, records a DEVICE buffer of capacity*9 int64,
 * count a DEVICE int64.  For tests. */
int gqa_schedule_dump_device(const int32_t* seq_lens, int32_t batch, int32_t num_kv_heads,
                             int32_t max_seq_len, int32_t tile_rows, int32_t num_ctas,
                             int32_t num_splits, int32_t kv_layout, int64_t* records,
                             int64_t capacity, int64_t* count, void* stream);

/* Library version string. */
const char* gqa_decode_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GQA_DECODE_B200_H_ */
