// extern "C" entry points of libgqa_decode_b200.so (declared in include/gqa_decode_b200.h).
// Host-side work per call: argument checks, two tensor-map encodes, one (or two) launches.
#include "../../include/gqa_decode_b200.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdlib>

#include "decode_kernel.cuh"
#include "fp8_path.cuh"
#include "exchange.cuh"
#include "quantize.cuh"

namespace gqa {

// ------------------------------------------------------------------ workspace layout
// [status, done_ctas | chunk deques | tickets | alloc | group table | partial LSE | partial O]
struct WorkspaceLayout {
  size_t status_off, done_off, deques_off, tickets_off, alloc_off, info_off, lse_off, o_off, total;
  long long slots;
};
static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }
static size_t slot_bytes(int G, int D) { return (size_t)G * (D + 1) * sizeof(float); }
static WorkspaceLayout layout_workspace(long long groups, int num_ctas, long long slots, int G,
                                        int D) {
  WorkspaceLayout w;
  w.status_off = 0;
  w.done_off = 4;
  w.deques_off = 256;
  w.tickets_off = up256(w.deques_off + (size_t)num_ctas * sizeof(unsigned long long));
  w.alloc_off = up256(w.tickets_off + (size_t)groups * sizeof(int));
  w.info_off = up256(w.alloc_off + (size_t)groups * sizeof(int));
  w.lse_off = up256(w.info_off + (size_t)groups * sizeof(int2));
  w.o_off = up256(w.lse_off + (size_t)slots * G * sizeof(float));
  w.total = up256(w.o_off + (size_t)slots * G * D * sizeof(float));
  w.slots = slots;
  return w;
}
// Largest slot count whose layout fits in `bytes` (0 if not even the fixed part fits).
static long long slots_that_fit(long long groups, int num_ctas, int G, int D, size_t bytes) {
  const WorkspaceLayout w0 = layout_workspace(groups, num_ctas, 0, G, D);
  if (bytes < w0.total + 512) return 0;
  long long s = (long long)((bytes - w0.total - 512) / slot_bytes(G, D));
  while (s > 0 && layout_workspace(groups, num_ctas, s, G, D).total > bytes) --s;
  return s;
}
// Slots a comfortably sized workspace offers the balanced schedule: one per group plus 64
// chunks per CTA (the chunk size adapts to whatever the caller really provides).
static long long default_balanced_slots(long long groups, int num_ctas) {
  return groups + 64ll * num_ctas + 1;
}

static int sm_count_or(int fallback) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return fallback;
  }
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return fallback;
  }
  return n;
}

// ------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// View K (or V) as a row-major matrix [total_rows, row_bytes] and describe boxes of
// [box_rows x 128 bytes] with the 128-byte swizzle.  Rows past total_rows read as zero.
// `row_elems` is the distance between consecutive rows in elements (head_dim, or
// Hkv * head_dim when the heads of a page row are interleaved).
// With `box_pieces` > 1 (a head's row is that many 128-byte pieces wide and a box spans them
// all) the view is 3-D instead, [pieces of the row][rows][128 bytes] - the piece index is the
// outermost coordinate although its stride is the smallest - so that ONE box brings the whole
// tile in, laid out in shared memory piece after piece exactly as separate 2-D boxes would be.
// Heads narrower than 128 bytes (E4M3 with head_dim 64) get boxes of their own width, unswizzled.
static int make_kv_map(CUtensorMap* tm, const void* base, int kv_dtype, long long row_elems,
                       long long total_rows, int box_rows, int box_pieces, int head_dim) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return GQA_ERR_DRIVER;
  const bool fp8 = kv_dtype == GQA_DTYPE_E4M3;
  const int esz = fp8 ? 1 : 2;
  CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                               : (kv_dtype == GQA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUresult r;
  if (box_pieces <= 1) {
    cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)total_rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_elems * esz};
    const bool narrow = head_dim * esz < 128;
    cuuint32_t box[2] = {(cuuint32_t)(narrow ? head_dim : 128 / esz), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE,
            narrow ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[3] = {(cuuint64_t)(128 / esz), (cuuint64_t)total_rows,
                          (cuuint64_t)(row_elems * esz / 128)};
    cuuint64_t strides[2] = {(cuuint64_t)row_elems * esz, 128};
    cuuint32_t box[3] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows, (cuuint32_t)box_pieces};
    cuuint32_t estr[3] = {1, 1, 1};
    r = enc(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? 0 : GQA_ERR_DRIVER;
}

// ------------------------------------------------------------------ dispatch
// Cost units charged per group by the balanced partition: starting and finishing a group
// costs about 1.5 us, i.e. two 32 KB tiles of streaming or one 64 KB tile.
static int group_overhead_for(int head_dim, int kv_dtype) {
  return (kv_dtype == GQA_DTYPE_E4M3 || head_dim == 256) ? 1 : 2;
}

// E4M3 tiles: 256 keys shared by 8 consumer warps, 32 keys each.  (Measured alternatives:
// 12 warps x 16 keys on 192-key tiles 17 % slower, 4 warps x 64 keys 8 % slower.)
constexpr int kFp8Warps = 8;
constexpr int kFp8Tile = 256;
static int tile_rows_for(int head_dim, int kv_dtype) {
  if (kv_dtype == GQA_DTYPE_E4M3) return (head_dim == 128 || head_dim == 64) ? kFp8Tile : 0;
  if (head_dim == 256) return 64;
  if (head_dim == 128) return 64;
  if (head_dim == 64) return 128;
  return 0;
}

template <class Tr>
static int launch_decode(const CUtensorMap& tk, const CUtensorMap& tv, DecodeParams prm,
                         int num_ctas, cudaStream_t stream, bool separate_merge, long long groups) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  int smem_cap = 0;
  e = cudaDeviceGetAttribute(&smem_cap, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e != cudaSuccess) return (int)e;
  const int grows = Tr::UPPER ? 16 : 8;
  int nst = kMaxStages;
  while (nst > 2 &&
         decode_smem_bytes(Tr::kStageBytes, nst, Tr::kMoStride, grows, Tr::kWarps) > (size_t)smem_cap)
    --nst;
  const size_t smem = decode_smem_bytes(Tr::kStageBytes, nst, Tr::kMoStride, grows, Tr::kWarps);
  if (smem > (size_t)smem_cap) return GQA_ERR_SHAPE;
  prm.num_stages = nst;
  static std::atomic<unsigned long long> configured{0};  // bit per device (first 64 devices)
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(decode_kernel<Tr>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             smem_cap);
    if (e != cudaSuccess) return (int)e;
    configured.fetch_or(bit, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)num_ctas);
  cfg.blockDim = dim3((unsigned)BlockShape<Tr>::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (prm.pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  e = cudaLaunchKernelEx(&cfg, decode_kernel<Tr>, tk, tv, prm);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  if (separate_merge) {
    merge_groups_kernel<typename Tr::Q, Tr::D>
        <<<(unsigned)groups, kMergeThreads, 0, stream>>>(prm);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// `own_scratch`: the call runs on the library's own scratch array (completion tickets, control
// words cleared on the stream once every check has passed).
static int run_decode(const gqa_decode_args_t* a, bool want_fp8, bool force_balanced,
                      const gqa_gather_args_t* gather = nullptr, bool own_scratch = false) {
  if (!a || !a->q || !a->k || !a->v || !a->workspace) return GQA_ERR_ARG;
  if ((!gather || gather->mode == GQA_GATHER_SEQUENCE) && !a->out && !a->out_f32) return GQA_ERR_ARG;
  if (gather) {
    if (gather->mode != GQA_GATHER_HEADS && gather->mode != GQA_GATHER_SEQUENCE) return GQA_ERR_ARG;
    if (gather->world < 1 || gather->world > kMaxPeers || gather->rank < 0 ||
        gather->rank >= gather->world || gather->epoch == 0 || !gather->peer_out ||
        !gather->peer_flags)
      return GQA_ERR_ARG;
    for (int p = 0; p < gather->world; ++p)
      if (!gather->peer_out[p] || !gather->peer_flags[p] || !aligned16(gather->peer_out[p]))
        return GQA_ERR_ARG;
    // the hand-off is part of the decode kernel's tail: it needs the in-kernel merge, and the
    // finished-CTA counter it uses is the work-stealing clean-up's
    if (a->flags & (GQA_FLAG_SEPARATE_MERGE | GQA_FLAG_NO_MERGE | GQA_FLAG_WORK_STEALING))
      return GQA_ERR_ARG;
  }
  if (a->batch <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->max_seq_len <= 0 ||
      a->total_rows <= 0 || a->num_splits < 0 || a->num_ctas < 0)
    return GQA_ERR_ARG;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out) ||
      !aligned16(a->out_f32) || !aligned16(a->workspace))
    return GQA_ERR_ARG;
  if (a->q_dtype != GQA_DTYPE_BF16 && a->q_dtype != GQA_DTYPE_FP16) return GQA_ERR_SHAPE;
  const bool fp8 = a->kv_dtype == GQA_DTYPE_E4M3;
  if (fp8 != want_fp8) return GQA_ERR_SHAPE;
  if (!fp8 && a->kv_dtype != a->q_dtype) return GQA_ERR_SHAPE;
  if (fp8 && (!a->k_scale || !a->v_scale)) return GQA_ERR_ARG;
  if (a->num_q_heads % a->num_kv_heads) return GQA_ERR_SHAPE;
  const int G = a->num_q_heads / a->num_kv_heads;
  if (G > 16) return GQA_ERR_SHAPE;
  const int D = a->head_dim;
  const int tile = tile_rows_for(D, a->kv_dtype);
  if (!tile) return GQA_ERR_SHAPE;
  if (a->kv_layout < GQA_LAYOUT_PADDED || a->kv_layout > GQA_LAYOUT_PAGED_NHD) return GQA_ERR_ARG;
  if (a->kv_layout == GQA_LAYOUT_PACKED && !a->seq_lens) return GQA_ERR_ARG;
  const bool paged = a->kv_layout >= GQA_LAYOUT_PAGED_HND;
  if (paged) {
    if (!a->block_table || a->page_size < 16 || a->page_size % 16 || a->block_table_stride <= 0)
      return GQA_ERR_ARG;
    if (a->page_size % tile && tile % a->page_size) return GQA_ERR_SHAPE;
    if ((long long)a->block_table_stride * a->page_size < a->max_seq_len) return GQA_ERR_ARG;
    if (a->total_rows % ((long long)a->num_kv_heads * a->page_size)) return GQA_ERR_ARG;
  }
  if (a->total_rows >= (1ll << 31)) return GQA_ERR_LIMIT;  // TMA coordinates are 32-bit
  const long long groups = (long long)a->batch * a->num_kv_heads;
  if (a->kv_layout == GQA_LAYOUT_PADDED && groups * a->max_seq_len > a->total_rows)
    return GQA_ERR_ARG;

  const int num_ctas = a->num_ctas > 0 ? a->num_ctas : sm_count_or(0);
  if (num_ctas <= 0) return (int)cudaErrorNoDevice;
  const int splits = force_balanced ? 0 : a->num_splits;
  const bool no_merge = (a->flags & GQA_FLAG_NO_MERGE) != 0;
  if (no_merge && splits == 0) return GQA_ERR_ARG;
  const bool separate = !no_merge && (a->flags & GQA_FLAG_SEPARATE_MERGE) != 0;
  const bool fused = !separate && !no_merge;
  const int overhead = group_overhead_for(D, a->kv_dtype);
  const long long tiles_per_group = ((long long)a->max_seq_len + tile - 1) / tile + overhead;

  // Partial slots: explicit splits need exactly groups*K; static balanced ranges one per group
  // and CTA (units are dealt one by one: equal shares to within a unit); with work stealing
  // the schedule takes what the workspace offers and sizes its chunks accordingly.
  const bool steal = fused && splits == 0 && (a->flags & GQA_FLAG_WORK_STEALING);
  WorkspaceLayout w;
  int chunk = 1;
  if (splits > 0) {
    w = layout_workspace(groups, num_ctas, groups * splits, G, D);
    if (a->workspace_bytes < w.total) return GQA_ERR_WORKSPACE;
  } else if (!steal) {
    const long long slots = groups + num_ctas + 2;
    w = layout_workspace(groups, num_ctas, slots, G, D);
    if (a->workspace_bytes < w.total) return GQA_ERR_WORKSPACE;
  } else {
    long long slots = slots_that_fit(groups, num_ctas, G, D, a->workspace_bytes);
    if (slots < groups + 2) return GQA_ERR_WORKSPACE;
    const long long cap = default_balanced_slots(groups, num_ctas);
    if (slots > cap) slots = cap;
    chunk = choose_chunk_tiles(groups, tiles_per_group, num_ctas, slots);
    if (max_slots(groups, 0, tiles_per_group, chunk) > slots) return GQA_ERR_WORKSPACE;
    w = layout_workspace(groups, num_ctas, slots, G, D);
  }

  CUtensorMap tk, tv;
  const int box_rows = paged && a->page_size < tile ? a->page_size : tile;
  // [rows, D] for every layout except page rows with interleaved heads: [pages * page_size, Hkv * D]
  const bool nhd = a->kv_layout == GQA_LAYOUT_PAGED_NHD;
  const long long row_elems = nhd ? (long long)a->num_kv_heads * D : D;
  const long long map_rows = nhd ? a->total_rows / a->num_kv_heads : a->total_rows;
  // 128-byte pieces of one head's row; a box spans all of them unless it is shorter than the
  // tile (small pages: the pieces of a tile then lie a whole tile apart in shared memory).
  const int row_pieces = D * (a->kv_dtype == GQA_DTYPE_E4M3 ? 1 : 2) / 128;
  // (bf16/fp16 D=128 has instantiations for 16- and 32-row pages whose stage layout takes one
  // box per page with all its pieces)
  const bool page_boxes = !fp8 && D == 128 && (box_rows == 16 || box_rows == 32);
  const int box_pieces = (box_rows == tile || page_boxes) ? row_pieces : 1;
  int r = make_kv_map(&tk, a->k, a->kv_dtype, row_elems, map_rows, box_rows, box_pieces, D);
  if (r) return r;
  r = make_kv_map(&tv, a->v, a->kv_dtype, row_elems, map_rows, box_rows, box_pieces, D);
  if (r) return r;

  char* ws = static_cast<char*>(a->workspace);
  DecodeParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.q = a->q;
  prm.out = a->out;
  prm.out_f32 = a->out_f32;
  prm.out_lse = a->out_lse;
  prm.k_scale = a->k_scale;
  prm.v_scale = a->v_scale;
  prm.status = reinterpret_cast<int*>(ws + w.status_off);
  prm.done_ctas = reinterpret_cast<int*>(ws + w.done_off);
  prm.deques = reinterpret_cast<unsigned long long*>(ws + w.deques_off);
  prm.tickets = reinterpret_cast<int*>(ws + w.tickets_off);
  prm.alloc = reinterpret_cast<int*>(ws + w.alloc_off);
  prm.group_info = reinterpret_cast<int2*>(ws + w.info_off);
  prm.part_lse = reinterpret_cast<float*>(ws + w.lse_off);
  prm.part_o = reinterpret_cast<float*>(ws + w.o_off);
  prm.sched.seq_lens = a->seq_lens;
  prm.sched.batch = a->batch;
  prm.sched.num_kv_heads = a->num_kv_heads;
  prm.sched.max_seq = a->max_seq_len;
  prm.sched.tile_rows = tile;
  prm.sched.num_ctas = num_ctas;
  prm.sched.num_splits = splits;
  prm.sched.layout = a->kv_layout;
  prm.sched.chunk_tiles = chunk;
  prm.sched.group_overhead = overhead;
  // stealing needs the in-kernel merge (partials are counted as they complete)
  prm.sched.steal = steal ? 1 : 0;
  // uniform lengths on the static balanced schedule: geometry and reciprocals from the host
  prepare_fast_schedule(prm.sched);
  prm.num_q_heads = a->num_q_heads;
  prm.group = G;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)D);
  prm.scale_log2 = scale * kLog2e;
  prm.fused_merge = fused ? 1 : 0;
  // Partials that announce themselves need every contributor of a group to be resident (or
  // finished) while the group's last CTA polls: guaranteed with at most one CTA per SM.
  prm.polled = (fused && !prm.sched.steal && !own_scratch && !(a->flags & GQA_FLAG_TICKET_MERGE) &&
                num_ctas <= sm_count_or(0))
                   ? 1
                   : 0;
  prm.no_merge = no_merge ? 1 : 0;
  prm.num_slots = (int)w.slots;
  prm.timestamps = reinterpret_cast<unsigned long long*>(a->debug_timestamps);
  prm.wait_limit_ns = a->wait_limit_ns ? a->wait_limit_ns : kDefaultWaitLimitNs;
  prm.pdl = (a->flags & GQA_FLAG_DEPENDENT_LAUNCH) ? 1 : 0;
  prm.block_table = paged ? a->block_table : nullptr;
  prm.page_size = paged ? a->page_size : 0;
  prm.table_stride = paged ? a->block_table_stride : 0;
  prm.box_rows = box_rows;
  prm.box_shift = 0;
  while ((1 << prm.box_shift) < box_rows) ++prm.box_shift;
  prm.page_shift = -1;
  if (paged && (a->page_size & (a->page_size - 1)) == 0)
    for (prm.page_shift = 0; (1 << prm.page_shift) < a->page_size;) ++prm.page_shift;

  if (gather) {
    for (int p = 0; p < gather->world; ++p) {
      prm.gather_out[p] = gather->peer_out[p];
      prm.gather_flags[p] = gather->peer_flags[p];
    }
    prm.gather_world = gather->world;
    prm.gather_rank = gather->rank;
    prm.gather_epoch = gather->epoch;
    prm.gather_mode = gather->mode;
    prm.gather_rows = (long long)a->batch * a->num_q_heads;
  }
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  if (own_scratch || (a->flags & GQA_FLAG_CLEAR_WORKSPACE)) {
    // control words always; the partial area too when the launch expects it to be zero
    cudaError_t e = cudaMemsetAsync(a->workspace, 0, prm.polled ? w.total : w.lse_off, st);
    if (e != cudaSuccess) return (int)e;
  }
  const bool upper = G > 8;
  const bool bf = a->q_dtype == GQA_DTYPE_BF16;
#define GQA_LAUNCH(...) \
  return launch_decode<__VA_ARGS__>(tk, tv, prm, num_ctas, st, separate, groups)
  if (fp8 && D == 64) {  // every element rounded like dequantize_kv_fp8, K and V alike
    if (bf) {
      if (upper) GQA_LAUNCH(KvFp8Dim64Traits<__nv_bfloat16, true>);
      GQA_LAUNCH(KvFp8Dim64Traits<__nv_bfloat16, false>);
    }
    if (upper) GQA_LAUNCH(KvFp8Dim64Traits<__half, true>);
    GQA_LAUNCH(KvFp8Dim64Traits<__half, false>);
  }
  if (fp8) {
    const bool exact_v = (a->flags & GQA_FLAG_FP8_EXACT_V) != 0;
    if (exact_v) {
      if (bf) {
        if (upper) GQA_LAUNCH(KvFp8Traits<__nv_bfloat16, kFp8Tile, true, true, kFp8Warps>);
        GQA_LAUNCH(KvFp8Traits<__nv_bfloat16, kFp8Tile, false, true, kFp8Warps>);
      }
      if (upper) GQA_LAUNCH(KvFp8Traits<__half, kFp8Tile, true, true, kFp8Warps>);
      GQA_LAUNCH(KvFp8Traits<__half, kFp8Tile, false, true, kFp8Warps>);
    }
    if (bf) {
      if (upper) GQA_LAUNCH(KvFp8Traits<__nv_bfloat16, kFp8Tile, true, false, kFp8Warps>);
      GQA_LAUNCH(KvFp8Traits<__nv_bfloat16, kFp8Tile, false, false, kFp8Warps>);
    }
    if (upper) GQA_LAUNCH(KvFp8Traits<__half, kFp8Tile, true, false, kFp8Warps>);
    GQA_LAUNCH(KvFp8Traits<__half, kFp8Tile, false, false, kFp8Warps>);
  }
  if (D == 256) {
    if (bf) {
      if (upper) GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 256, 64, true>);
      GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 256, 64, false>);
    }
    if (upper) GQA_LAUNCH(Kv16Traits<__half, 256, 64, true>);
    GQA_LAUNCH(Kv16Traits<__half, 256, 64, false>);
  }
  if (D == 128 && page_boxes) {
    if (box_rows == 16) {
      if (bf) {
        if (upper) GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, true, 4, 16>);
        GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, false, 4, 16>);
      }
      if (upper) GQA_LAUNCH(Kv16Traits<__half, 128, 64, true, 4, 16>);
      GQA_LAUNCH(Kv16Traits<__half, 128, 64, false, 4, 16>);
    }
    if (bf) {
      if (upper) GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, true, 4, 32>);
      GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, false, 4, 32>);
    }
    if (upper) GQA_LAUNCH(Kv16Traits<__half, 128, 64, true, 4, 32>);
    GQA_LAUNCH(Kv16Traits<__half, 128, 64, false, 4, 32>);
  }
  if (D == 128) {
    if (bf) {
      if (upper) GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, true>);
      GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 128, 64, false>);
    }
    if (upper) GQA_LAUNCH(Kv16Traits<__half, 128, 64, true>);
    GQA_LAUNCH(Kv16Traits<__half, 128, 64, false>);
  }
  if (bf) {
    if (upper) GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 64, 128, true>);
    GQA_LAUNCH(Kv16Traits<__nv_bfloat16, 64, 128, false>);
  }
  if (upper) GQA_LAUNCH(Kv16Traits<__half, 64, 128, true>);
  GQA_LAUNCH(Kv16Traits<__half, 64, 128, false>);
#undef GQA_LAUNCH
}

// ------------------------------------------------------------------ generic merge
template <typename Q>
__global__ void merge_rows_kernel(const float* __restrict__ o_parts,
                                  const float* __restrict__ lse_parts, int num_parts,
                                  long long rows, int D, Q* out, float* out_f32, float* out_lse) {
  const int D4 = D / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * D4) return;
  const long long row = idx / D4;
  const int d4 = (int)(idx % D4);
  float mx = -INFINITY;
  for (int p = 0; p < num_parts; ++p) mx = fmaxf(mx, lse_parts[(size_t)p * rows + row]);
  const float ms = (mx == -INFINITY) ? 0.f : mx;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
  for (int p = 0; p < num_parts; ++p) {
    const float w = fast_exp2((lse_parts[(size_t)p * rows + row] - ms) * kLog2e);
    const float4 o =
        reinterpret_cast<const float4*>(o_parts + ((size_t)p * rows + row) * D)[d4];
    acc.x += w * o.x;
    acc.y += w * o.y;
    acc.z += w * o.z;
    acc.w += w * o.w;
    wsum += w;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  acc.x *= inv;
  acc.y *= inv;
  acc.z *= inv;
  acc.w *= inv;
  if (out) {
    uint2 pk;
    pk.x = Mma16<Q>::pack(acc.x, acc.y);
    pk.y = Mma16<Q>::pack(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + row * D + 4 * d4) = pk;
  }
  if (out_f32) reinterpret_cast<float4*>(out_f32 + row * D)[d4] = acc;
  if (out_lse && d4 == 0) out_lse[row] = wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY;
}

// ------------------------------------------------------------------ scheduler dumps
static __host__ __device__ void put_record(long long* rec, int cta, const Segment& s) {
  rec[0] = cta;
  rec[1] = s.b;
  rec[2] = s.h;
  rec[3] = s.row_begin;
  rec[4] = s.row_end;
  rec[5] = s.slot;
  rec[6] = s.first_slot;
  rec[7] = s.n_parts;
  rec[8] = s.kv_row0;
}

constexpr int kDumpSegs = 64;  // segments replayed per batch of walk_static calls

__global__ void schedule_dump_kernel(SchedParams sp, long long* records, long long capacity,
                                     unsigned long long* count) {
  Walker wk;
  wk.init_warp(sp);
  long long t0, t1;
  if (!wk.static_range(blockIdx.x, t0, t1)) return;
  if (sp.num_splits > 0) wk.seek_unit_warp(t0);
  else wk.seek_warp(t0);
  if (threadIdx.x != 0) return;
  // walk the CTA's static range one segment at a time
  if (sp.num_splits > 0) {
    for (long long u = t0; u < t1; ++u) {
      Segment s;
      wk.next_unit(s);
      const unsigned long long i = atomicAdd(count, 1ull);
      if ((long long)i < capacity) put_record(records + 9 * i, blockIdx.x, s);
    }
    return;
  }
  long long t = t0;
  while (t < t1) {
    Segment s;
    long long tt1 = t + (wk.ntg - wk.ti);
    if (tt1 > t1) tt1 = t1;
    const long long n = wk.walk_static(blockIdx.x, t, tt1, &s, 1);
    if (n >= 1) {
      const unsigned long long i = atomicAdd(count, 1ull);
      if ((long long)i < capacity) put_record(records + 9 * i, blockIdx.x, s);
    }
    t = tt1;
  }
}

constexpr int kDumpOverhead = 2;  // group overhead units used by the schedule dumps
// the dumps replay the static schedule: one unit per chunk
static int default_chunk(int, int, int, int, int) { return 1; }

}  // namespace gqa

using namespace gqa;

extern "C" {

const char* gqa_decode_version(void) { return "gqa_decode_b200 0.1 (sm_100a)"; }

int gqa_decode_tile_rows(int32_t head_dim, int32_t kv_dtype) {
  const int t = tile_rows_for(head_dim, kv_dtype);
  return t ? t : GQA_ERR_SHAPE;
}

int gqa_decode_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                               int32_t head_dim, int32_t num_splits, int32_t num_ctas,
                               size_t* bytes) {
  if (!bytes || batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
      num_splits < 0 || num_ctas < 0 || num_q_heads % num_kv_heads)
    return GQA_ERR_ARG;
  // Without an explicit CTA count size for the SM count of the current device (or a
  // generous bound when no device is visible, e.g. when sizing buffers on a host-only box).
  const int ctas = num_ctas > 0 ? num_ctas : sm_count_or(1024);
  const long long groups = (long long)batch * num_kv_heads;
  // a workspace sized for the balanced schedule also has to serve explicit splits and back
  long long slots = default_balanced_slots(groups, ctas);
  if (groups * num_splits > slots) slots = groups * num_splits;
  *bytes = layout_workspace(groups, ctas, slots, num_q_heads / num_kv_heads, head_dim).total + 512;
  return 0;
}

int gqa_decode_workspace_layout(int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                int32_t head_dim, int32_t num_splits, int32_t num_ctas,
                                size_t offsets[6]) {
  if (!offsets || batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
      num_splits <= 0 || num_ctas < 0 || num_q_heads % num_kv_heads)
    return GQA_ERR_ARG;
  const int ctas = num_ctas > 0 ? num_ctas : sm_count_or(0);
  if (ctas <= 0) return (int)cudaErrorNoDevice;
  const long long groups = (long long)batch * num_kv_heads;
  const WorkspaceLayout w =
      layout_workspace(groups, ctas, groups * num_splits, num_q_heads / num_kv_heads, head_dim);
  offsets[0] = w.status_off;
  offsets[1] = w.tickets_off;
  offsets[2] = w.info_off;
  offsets[3] = w.lse_off;
  offsets[4] = w.o_off;
  offsets[5] = w.total;
  return 0;
}

int gqa_decode_workspace_reset(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < 512) return GQA_ERR_ARG;
  // Only the control words need to be zero, but how far they reach depends on the geometry
  // of the next launch, which is not known here: clear everything.
  cudaError_t e = cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream));
  return (int)e;
}

int gqa_decode_read_status(const void* workspace, void* stream, int32_t* status) {
  if (!workspace || !status) return GQA_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(st);
}

int gqa_decode_attention(const gqa_decode_args_t* args) { return run_decode(args, false, false); }

int gqa_decode_attention_persistent(const gqa_decode_args_t* args) {
  return run_decode(args, false, true);
}

int gqa_decode_attention_fp8(const gqa_decode_args_t* args) { return run_decode(args, true, false); }

int gqa_decode_attention_gather(const gqa_decode_args_t* args, const gqa_gather_args_t* gather) {
  if (!args || !gather) return GQA_ERR_ARG;
  return run_decode(args, args->kv_dtype == GQA_DTYPE_E4M3, false, gather);
}

// ---- entry for callers that cannot allocate: scratch inside the library image ----------
// The array's name is only a host-side handle in host code; kernels must be given the
// device address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) unsigned char g_static_scratch[GQA_STATIC_SCRATCH_BYTES];
static constexpr int kMaxScratchDevices = 64;
static std::atomic<void*> g_static_scratch_addr[kMaxScratchDevices];

int gqa_decode_attention_static_scratch(const gqa_decode_args_t* args) {
  if (!args) return GQA_ERR_ARG;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxScratchDevices) return GQA_ERR_LIMIT;
  void* base = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (!base) {
    // set-up, once per device, with that device current
    e = cudaGetSymbolAddress(&base, g_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!base) return GQA_ERR_DRIVER;
    g_static_scratch_addr[dev].store(base, std::memory_order_release);
  }
  if (args->batch <= 0 || args->num_q_heads <= 0 || args->num_kv_heads <= 0 ||
      args->head_dim <= 0 || args->num_splits < 0 || args->num_ctas < 0 ||
      args->num_q_heads % args->num_kv_heads)
    return GQA_ERR_ARG;
  const int ctas = args->num_ctas > 0 ? args->num_ctas : sm_count_or(0);
  if (ctas <= 0) return (int)cudaErrorNoDevice;
  const long long groups = (long long)args->batch * args->num_kv_heads;
  const int G = args->num_q_heads / args->num_kv_heads;
  // Explicit splits need groups*K partial slots, the balanced schedule one per group and CTA
  // (with work stealing at least one per group: its chunk size adapts to the room there is):
  // refuse what cannot fit the array.
  const long long need_slots = args->num_splits > 0 ? groups * args->num_splits
                               : (args->flags & GQA_FLAG_WORK_STEALING) ? groups + 2
                                                                        : groups + ctas + 2;
  const WorkspaceLayout w = layout_workspace(groups, ctas, need_slots, G, args->head_dim);
  if (w.total + 512 > (size_t)GQA_STATIC_SCRATCH_BYTES) return GQA_ERR_LIMIT;
  // The array still holds the previous call's bytes: deques, tickets and status must start
  // at zero (everything in front of the partial slots).  run_decode clears them on the stream
  // after its own checks, so a call that is rejected leaves the array - which a launch in
  // flight on another stream may be using - untouched.
  gqa_decode_args_t a = *args;
  a.workspace = base;
  a.workspace_bytes = GQA_STATIC_SCRATCH_BYTES;
  return run_decode(&a, false, false, nullptr, /*own_scratch=*/true);
}

int gqa_merge_partials(const float* o_parts, const float* lse_parts, int32_t num_parts,
                       int64_t rows, int32_t head_dim, void* out, int32_t out_dtype,
                       float* out_f32, float* out_lse, void* stream) {
  if (!o_parts || !lse_parts || num_parts <= 0 || rows <= 0 || head_dim <= 0 || head_dim % 4 ||
      (!out && !out_f32))
    return GQA_ERR_ARG;
  if (!aligned16(o_parts) || !aligned16(out) || !aligned16(out_f32)) return GQA_ERR_ARG;
  if (out && out_dtype != GQA_DTYPE_BF16 && out_dtype != GQA_DTYPE_FP16) return GQA_ERR_SHAPE;
  const long long work = rows * (head_dim / 4);
  const int block = 128;
  const unsigned grid = (unsigned)((work + block - 1) / block);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == GQA_DTYPE_FP16)
    merge_rows_kernel<__half><<<grid, block, 0, st>>>(o_parts, lse_parts, num_parts, rows,
                                                      head_dim, static_cast<__half*>(out),
                                                      out_f32, out_lse);
  else
    merge_rows_kernel<__nv_bfloat16><<<grid, block, 0, st>>>(
        o_parts, lse_parts, num_parts, rows, head_dim, static_cast<__nv_bfloat16*>(out), out_f32,
        out_lse);
  return (int)cudaGetLastError();
}

int gqa_quantize_kv_fp8(const void* x, int32_t x_dtype, int64_t num_heads, int64_t elems_per_head,
                        uint8_t* codes, float* scales, float* amax_scratch, void* stream) {
  if (!x || !codes || !scales || !amax_scratch || num_heads <= 0 || elems_per_head <= 0 ||
      elems_per_head % 8 || num_heads > 65535)
    return GQA_ERR_ARG;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 7)) return GQA_ERR_ARG;
  if (x_dtype != GQA_DTYPE_BF16 && x_dtype != GQA_DTYPE_FP16) return GQA_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, (size_t)num_heads * sizeof(float), st);
  if (e != cudaSuccess) return (int)e;
  // enough blocks per head to fill the GPU a few times over, at least 16 KB of input each
  long long per = elems_per_head / 8 / kQuantThreads / 4;
  const long long want = (long long)sm_count_or(148) * 8 / num_heads + 1;
  if (per > want) per = want;
  if (per < 1) per = 1;
  const dim3 grid((unsigned)per, (unsigned)num_heads);
  if (x_dtype == GQA_DTYPE_BF16) {
    amax_kernel<__nv_bfloat16><<<grid, kQuantThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), elems_per_head, amax_scratch);
    quantize_kernel<__nv_bfloat16><<<grid, kQuantThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), elems_per_head, amax_scratch, codes, scales);
  } else {
    amax_kernel<__half><<<grid, kQuantThreads, 0, st>>>(static_cast<const __half*>(x),
                                                        elems_per_head, amax_scratch);
    quantize_kernel<__half><<<grid, kQuantThreads, 0, st>>>(
        static_cast<const __half*>(x), elems_per_head, amax_scratch, codes, scales);
  }
  return (int)cudaGetLastError();
}

int gqa_quantize_append_fp8(const gqa_append_args_t* a) {
  if (!a || !a->k_new || !a->v_new || !a->k_cache || !a->v_cache || !a->k_scale || !a->v_scale ||
      !a->positions || a->batch <= 0 || a->num_kv_heads <= 0 || a->max_seq_len <= 0)
    return GQA_ERR_ARG;
  if (a->head_dim <= 0 || a->head_dim % 4 || a->head_dim > 1024) return GQA_ERR_SHAPE;
  if (a->src_dtype != GQA_DTYPE_BF16 && a->src_dtype != GQA_DTYPE_FP16) return GQA_ERR_SHAPE;
  const bool paged = a->kv_layout == GQA_LAYOUT_PAGED_HND || a->kv_layout == GQA_LAYOUT_PAGED_NHD;
  if (!paged && a->kv_layout != GQA_LAYOUT_PADDED) return GQA_ERR_ARG;
  if (paged && (!a->block_table || a->page_size <= 0 || a->block_table_stride <= 0 ||
                (long long)a->block_table_stride * a->page_size < a->max_seq_len))
    return GQA_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a->k_new) & 7) || (reinterpret_cast<uintptr_t>(a->v_new) & 7) ||
      (reinterpret_cast<uintptr_t>(a->k_cache) & 3) || (reinterpret_cast<uintptr_t>(a->v_cache) & 3))
    return GQA_ERR_ARG;
  AppendParams p;
  p.k_new = a->k_new;
  p.v_new = a->v_new;
  p.k_cache = static_cast<uint8_t*>(a->k_cache);
  p.v_cache = static_cast<uint8_t*>(a->v_cache);
  p.k_scale = a->k_scale;
  p.v_scale = a->v_scale;
  p.positions = a->positions;
  p.block_table = a->block_table;
  p.saturated = a->saturated;
  p.num_kv_heads = a->num_kv_heads;
  p.head_dim = a->head_dim;
  p.max_seq = a->max_seq_len;
  p.layout = a->kv_layout;
  p.page_size = a->page_size;
  p.table_stride = a->block_table_stride;
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  const unsigned grid = (unsigned)((long long)a->batch * a->num_kv_heads);
  if (a->src_dtype == GQA_DTYPE_BF16)
    append_quantize_kernel<__nv_bfloat16><<<grid, a->head_dim / 4, 0, st>>>(p);
  else
    append_quantize_kernel<__half><<<grid, a->head_dim / 4, 0, st>>>(p);
  return (int)cudaGetLastError();
}

size_t gqa_sequence_exchange_bytes(int32_t world, int64_t rows, int32_t head_dim) {
  if (world <= 0 || rows <= 0 || head_dim <= 0) return 0;
  return (size_t)2 * world * sequence_exchange_slot_words(rows, head_dim) * sizeof(uint2);
}

size_t gqa_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t head_dim) {
  if (world <= 0 || rows <= 0 || head_dim <= 0) return 0;
  return exchange_buffer_bytes(world, rows, head_dim);
}

int gqa_exchange_merge(const float* local_o, const float* local_lse, void* const* peer_bufs,
                       int32_t rank, int32_t world, uint32_t epoch, int64_t rows,
                       int32_t head_dim, void* out, int32_t out_dtype, float* out_f32,
                       float* out_lse, int32_t* status, uint64_t wait_limit_ns, void* stream) {
  if (!local_o || !local_lse || !peer_bufs || world <= 0 || world > kExchangeThreads ||
      rank < 0 || rank >= world || epoch == 0 || rows <= 0 || head_dim <= 0 || head_dim % 4 ||
      (!out && !out_f32))
    return GQA_ERR_ARG;
  if (!aligned16(local_o) || !aligned16(out) || !aligned16(out_f32)) return GQA_ERR_ARG;
  if (out && out_dtype != GQA_DTYPE_BF16 && out_dtype != GQA_DTYPE_FP16) return GQA_ERR_SHAPE;
  ExchangeParams p;
  p.local_o = local_o;
  p.local_lse = local_lse;
  p.peer_bufs = peer_bufs;
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.rows = rows;
  p.D = head_dim;
  p.out = out;
  p.out_fp16 = out_dtype == GQA_DTYPE_FP16;
  p.out_f32 = out_f32;
  p.out_lse = out_lse;
  p.status = status;
  p.wait_limit_ns = wait_limit_ns ? wait_limit_ns : kDefaultWaitLimitNs;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == GQA_DTYPE_FP16)
    exchange_merge_kernel<__half><<<world, kExchangeThreads, 0, st>>>(p);
  else
    exchange_merge_kernel<__nv_bfloat16><<<world, kExchangeThreads, 0, st>>>(p);
  return (int)cudaGetLastError();
}

int gqa_select_num_splits(int32_t num_kv_heads, int32_t seq_len, int32_t block_seq,
                          int32_t target_blocks_per_sm, int32_t num_sms) {
  if (num_kv_heads <= 0 || block_seq <= 0 || target_blocks_per_sm <= 0 || num_sms <= 0)
    return GQA_ERR_ARG;
  // Same one-wave rule as the reference: grid = num_sms * min(target, shared-memory cap),
  // splits = min(max(1, grid / Hkv), tiles).  The cap models two padded 16-bit tiles of
  // head_dim 128 (row pad 8, 16-byte rounded) against 228 KB, minus one block of slack.
  const long long tile = ((((long long)block_seq - 1) * (128 + 8) + 128) * 2 + 15) & ~15ll;
  long long cap = (228ll * 1024) / (2 * tile) - 1;
  if (cap < 1) cap = 1;
  const long long per_sm = target_blocks_per_sm < cap ? target_blocks_per_sm : cap;
  long long splits = (long long)num_sms * per_sm / num_kv_heads;
  if (splits < 1) splits = 1;
  long long tiles = ((long long)seq_len + block_seq - 1) / block_seq;
  if (tiles < 1) tiles = 1;
  return (int)(splits < tiles ? splits : tiles);
}

int64_t gqa_schedule_dump(const int32_t* seq_lens_host, int32_t batch, int32_t num_kv_heads,
                          int32_t max_seq_len, int32_t tile_rows, int32_t num_ctas,
                          int32_t num_splits, int32_t kv_layout, int64_t* records,
                          int64_t capacity) {
  if (batch <= 0 || num_kv_heads <= 0 || max_seq_len <= 0 || tile_rows <= 0 || num_ctas <= 0 ||
      num_splits < 0 || (capacity > 0 && !records))
    return GQA_ERR_ARG;
  SchedParams sp{seq_lens_host, batch,      num_kv_heads, max_seq_len, tile_rows,
                 num_ctas,      num_splits, kv_layout,
                 default_chunk(batch, num_kv_heads, max_seq_len, tile_rows, num_ctas), kDumpOverhead, 0};
  // Where the closed-form set-up applies (uniform lengths), the replay runs twice - general
  // path and closed form - and the two must agree segment for segment.
  SchedParams sp_fast = sp;
  prepare_fast_schedule(sp_fast);
  int64_t n = 0;
  for (int c = 0; c < num_ctas; ++c) {
    Walker wk;
    wk.init_serial(sp);
    long long t0, t1;
    if (!wk.static_range(c, t0, t1)) continue;
    if (num_splits > 0) wk.seek_unit_serial(t0);
    else wk.seek_serial(t0);
    Segment buf[kDumpSegs];
    // segments of one CTA are produced in batches so that no large buffer is needed
    long long got = wk.walk_static(c, t0, t1, buf, 0);  // count only
    Walker wk2;
    wk2.init_serial(sp);
    if (num_splits > 0) wk2.seek_unit_serial(t0);
    else wk2.seek_serial(t0);
    Segment* all = got <= kDumpSegs ? buf : new Segment[got];
    wk2.walk_static(c, t0, t1, all, got);
    if (sp_fast.fast) {
      Walker wf;
      wf.init_serial(sp_fast);
      long long f0, f1;
      if (!wf.static_range(c, f0, f1) || f0 != t0 || f1 != t1) return GQA_ERR_INTERNAL;
      wf.seek_serial(f0);
      Segment* again = new Segment[got > 0 ? got : 1];
      const long long got2 = wf.walk_static(c, f0, f1, again, got);
      bool same = got2 == got;
      for (long long i = 0; same && i < got; ++i)
        same = again[i].b == all[i].b && again[i].h == all[i].h && again[i].len == all[i].len &&
               again[i].row_begin == all[i].row_begin && again[i].row_end == all[i].row_end &&
               again[i].kv_row0 == all[i].kv_row0 && again[i].slot == all[i].slot &&
               again[i].first_slot == all[i].first_slot && again[i].n_parts == all[i].n_parts;
      delete[] again;
      if (!same) {
        if (all != buf) delete[] all;
        return GQA_ERR_INTERNAL;
      }
    }
    for (long long i = 0; i < got; ++i, ++n)
      if (n < capacity) put_record(reinterpret_cast<long long*>(records) + 9 * n, c, all[i]);
    if (all != buf) delete[] all;
  }
  return n;
}

int gqa_schedule_dump_device(const int32_t* seq_lens, int32_t batch, int32_t num_kv_heads,
                             int32_t max_seq_len, int32_t tile_rows, int32_t num_ctas,
                             int32_t num_splits, int32_t kv_layout, int64_t* records,
                             int64_t capacity, int64_t* count, void* stream) {
  if (batch <= 0 || num_kv_heads <= 0 || max_seq_len <= 0 || tile_rows <= 0 || num_ctas <= 0 ||
      num_splits < 0 || !records || !count)
    return GQA_ERR_ARG;
  SchedParams sp{seq_lens, batch,      num_kv_heads, max_seq_len, tile_rows,
                 num_ctas, num_splits, kv_layout,
                 default_chunk(batch, num_kv_heads, max_seq_len, tile_rows, num_ctas), kDumpOverhead, 0};
  prepare_fast_schedule(sp);  // uniform lengths: the device takes the closed-form set-up
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(count, 0, sizeof(int64_t), st);
  if (e != cudaSuccess) return (int)e;
  schedule_dump_kernel<<<num_ctas, 32, 0, st>>>(sp, reinterpret_cast<long long*>(records),
                                               capacity,
                                               reinterpret_cast<unsigned long long*>(count));
  return (int)cudaGetLastError();
}

}  // extern "C"
