// Persistent split-K decode-attention kernel for sm_100a.
//
// One CTA per SM.  The producer warp is the CTA's scheduler: it takes chunks of the tile
// line (its own range first, then chunks stolen from slower CTAs), and for every tile writes a
// small descriptor into shared memory and streams the K and V tile into a multi-stage
// ring with TMA (cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers).
// The other warps (4 or 8) are consumers: they follow the descriptors, each owns an equal
// slice of a tile's keys, computes
// S = Q K^T for the whole query group of the KV head with mma.sync (query heads
// padded to the 16-row MMA tile), keeps an online softmax in registers and
// accumulates O += P V, again on the tensor cores.  At the end of a segment the
// consumer warps combine their states through shared memory and write either the final output
// (the segment covered the whole (sequence, KV head) group) or one partial
// (normalised O in fp32 + log-sum-exp) into the workspace; the CTA that completes a
// group's last partial merges them (atomic ticket), so one launch does everything.
//
// Replaces the reference's DirectDecodeKernel / SplitKDecodeKernel /
// DoubleBufferSplitKKernel / PersistentDecodeKernel (gqa_decode/gqa_decode.py:105-232,
// :235-416, :1043-1320, :771-1040) and, through the in-kernel merge, its
// ReductionKernel (:419-495).
#pragma once
#include "ptx.cuh"
#include "schedule.cuh"

namespace gqa {

constexpr int kMaxConsumerWarps = 8;
constexpr int kMergeThreads = 128;  // block size of the stand-alone merge kernel
constexpr int kMaxStages = 8;
constexpr int kMaxPeers = 8;  // GPUs of one NVLink domain that can gather head-sharded outputs
constexpr int kDescRing = 32;  // tile descriptors kept in shared memory (>= 4 * kMaxStages)
constexpr int kTimestampWords = 12;  // diagnostics words per CTA (DecodeParams::timestamps)
constexpr int kDeferCap = 4;  // group merges a CTA puts off until its streaming is over (one is the rule)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

enum StatusBits : int {
  kStatusOk = 0,
  kStatusWaitFull = 1,    // a consumer gave up waiting for a tile
  kStatusWaitEmpty = 2,   // the producer gave up waiting for a free stage
  kStatusSmemAlign = 4,   // shared memory base not 1024-byte aligned
  kStatusSlotRange = 8,   // a partial slot index fell outside the workspace (write skipped)
  kStatusWaitExchange = 16,  // a peer GPU's flag never arrived (sequence exchange, head gather)
  kStatusWaitPartial = 32,   // a partial of a group never arrived at the CTA that merges the group
};

struct DecodeParams {
  const void* q;        // [batch, Hq, D], 16-bit
  void* out;            // [batch, Hq, D], same type as q (may be null if out_f32 is set)
  float* out_f32;       // optional [batch, Hq, D] fp32 copy of the final output
  float* out_lse;       // optional [batch, Hq] natural-log sum-exp of the scaled scores
  const float* k_scale; // FP8 only: [batch * Hkv]
  const float* v_scale; // FP8 only: [batch * Hkv]
  float* part_o;        // workspace: [slots, G, D] fp32 normalised partial outputs
  float* part_lse;      // workspace: [slots, G] natural-log sum-exp per partial
  int* tickets;         // workspace: [batch * Hkv] completion tickets, zero between launches
  int* alloc;           // workspace: [batch * Hkv] partials allocated per group, zero between launches
  unsigned long long* deques;  // workspace: [num_ctas] chunks taken {front: low 32, back: high 32}
  int* done_ctas;       // workspace: CTAs that finished (the last one cleans the deques)
  int* status;          // workspace: one word, OR of StatusBits
  int2* group_info;     // workspace: [batch * Hkv] {first_slot, n_parts}, written when the merge
                        // runs as a separate kernel
  SchedParams sched;
  int num_q_heads;
  int group;            // G = Hq / Hkv
  float scale_log2;     // softmax scale * log2(e)
  int fused_merge;      // 1: the partials of a group are merged inside this launch
  int polled;           // fused merge, static schedule: 1 = partials announce themselves (a word that
                        // is not zero has arrived; the partial area is all zero between launches
                        // and writers turn +0 into -0) and the CTA that writes a group's last
                        // partial polls for the others; 0 = completion tickets (atomics)
  int no_merge;         // 1: every segment is written as a partial and nothing is merged
  int num_stages;
  int num_slots;        // partial slots the workspace holds
  unsigned long long* timestamps;  // optional diagnostics: kTimestampWords per CTA, %globaltimer ns:
                                   // {prologue done, first load issued, first tile landed, start of
                                   // the last segment's epilogue, end, ticket drawn by the CTA's
                                   // last merging segment (0: it merged nothing), SM id, tile
                                   // descriptors consumed, then for the CTA's last polled merge
                                   // {log-sum-exps all there, thread 0's outputs fetched, thread 0's
                                   // row stored, 0}}; builds with
                                   // GQA_PROFILE_WAITS append, after those words of the whole grid,
                                   // per CTA {producer wait cycles, producer cycles, tiles posted,
                                   // consumer warp 0 wait-for-data cycles, consumer cycles}
  unsigned long long wait_limit_ns;  // every bounded wait gives up after this long
  int pdl;                  // 1: launched with programmatic stream serialization - the previous
                            // kernel of the stream may still be running until griddep_wait()
  // paged K/V (sched.layout >= kLayoutPagedHnd)
  const int* block_table;   // [batch, table_stride] page numbers
  int page_size;            // rows per page
  int table_stride;         // table entries per sequence
  int box_rows;             // rows per TMA box: min(tile, page_size), a power of two
  int box_shift;            // log2(box_rows)
  int page_shift;           // log2(page_size), or -1 when page_size is not a power of two
  // head-sharded launches that gather their outputs on every rank (gather_world > 0): final
  // rows go to every rank's [batch, gather_world * Hq, D] buffer by peer stores, at this rank's
  // head offset; the last CTA then raises this rank's flag on every peer and waits for theirs
  void* gather_out[kMaxPeers];
  unsigned* gather_flags[kMaxPeers];  // every rank's [2 parities][world] flag words
  int gather_world, gather_rank;
  unsigned gather_epoch;
  // gather_mode 1 (sequence sharding): gather_out[p] is rank p's receive area of 8-byte words
  // {float value, epoch}: [2 parities][source rank][rows * D outputs, rows log-sum-exps (padded
  // to an even count)].  Every rank's normalised fp32 rows and LSEs are pushed there as soon
  // as they exist; a word is valid once its tag equals the step's epoch, so the data is its
  // own arrival flag (no fence, no separate flag, no counter).  At the end of the kernel
  // every CTA merges its share of the rows from the `world` partials into out / out_f32 /
  // out_lse, waiting (bounded) for words that have not landed yet.
  int gather_mode;
  long long gather_rows;    // batch * Hq
};

// What the producer tells the consumers about the tile in a pipeline stage.
struct TileDesc {
  int b, h;         // sequence and KV head
  int valid;        // keys in this tile (0: no data was loaded - empty piece or end marker)
  int flags;        // kTileFirst | kTileLast | kTileEnd
  int ntg;          // tiles in the whole group
  int first_slot;   // first partial slot of the group
  int slot;         // slot of this segment's partial, or -1: allocate at the end of the segment
  int n_parts;      // partials of the group if known in advance (static schedules), else 0
};
enum TileFlags : int {
  kTileFirst = 1,
  kTileLast = 2,
  kTileEnd = 4,
  kTileShared = 8,  // other CTAs contribute partials to this tile's group
};

__host__ __device__ inline size_t decode_smem_bytes(int stage_bytes, int num_stages, int mo_stride,
                                                    int group_rows, int consumer_warps) {
  size_t b = 1024;  // alignment slack
  b += (size_t)stage_bytes * num_stages;
  b += (size_t)consumer_warps * group_rows * mo_stride * sizeof(float);
  b += (size_t)consumer_warps * group_rows * 2 * sizeof(float);
  b += 2 * kMaxStages * sizeof(uint64_t);
  b += kDescRing * sizeof(TileDesc);
  b += 128;  // flag words and the list of deferred merges (8 + 3 * kDeferCap ints)
  return b;
}

// ---------------------------------------------------------------------------
// Per-warp online-softmax state for a 16-row (padded) query group.
// Thread (lane) owns rows r0 = lane/4 and r0+8, and columns 2*(lane%4)+{0,1} of
// every 8-wide MMA tile.
// ---------------------------------------------------------------------------
template <int D, bool UPPER>
struct WarpState {
  float o[D / 8][4];
  float m[2];
  float l[2];
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// Online softmax over NB consecutive 16-key blocks held as 2*NB S fragments (fragment
// t covers keys key0 + 8t .. 8t+7); returns P packed for the PV MMAs (pa[blk][0..3]) and
// rescales O once when the running maximum moved.
template <typename TP, int D, bool UPPER, bool PARTIAL, int NB = 1>
__device__ __forceinline__ void softmax_block(float (&s)[2 * NB][4], WarpState<D, UPPER>& st,
                                              uint32_t (&pa)[NB][4], float scale_log2, int key0,
                                              int valid, int lane) {
  const int c = lane & 3;
#pragma unroll
  for (int t = 0; t < 2 * NB; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const bool dead = PARTIAL && (key0 + 8 * t + 2 * c + e >= valid);
      s[t][e] = dead ? -INFINITY : s[t][e] * scale_log2;
      if (UPPER) s[t][2 + e] = dead ? -INFINITY : s[t][2 + e] * scale_log2;
    }
  float alpha[2] = {1.f, 1.f};
#pragma unroll
  for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < 2 * NB; ++t) mx = fmaxf(mx, fmaxf(s[t][2 * r], s[t][2 * r + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mnew = fmaxf(st.m[r], mx);
    const float msafe = (mnew == -INFINITY) ? 0.f : mnew;
    alpha[r] = fast_exp2(st.m[r] - msafe);
    st.m[r] = mnew;
    float sum = 0.f;
#pragma unroll
    for (int t = 0; t < 2 * NB; ++t)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pv = fast_exp2(s[t][2 * r + e] - msafe);
        s[t][2 * r + e] = pv;
        sum += pv;
      }
    st.l[r] = st.l[r] * alpha[r] + sum;
  }
  const bool moved = alpha[0] != 1.f || (UPPER && alpha[1] != 1.f);
  if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      st.o[i][0] *= alpha[0];
      st.o[i][1] *= alpha[0];
      if (UPPER) {
        st.o[i][2] *= alpha[1];
        st.o[i][3] *= alpha[1];
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    pa[b][0] = Mma16<TP>::pack(s[2 * b][0], s[2 * b][1]);
    pa[b][2] = Mma16<TP>::pack(s[2 * b + 1][0], s[2 * b + 1][1]);
    pa[b][1] = UPPER ? Mma16<TP>::pack(s[2 * b][2], s[2 * b][3]) : 0u;
    pa[b][3] = UPPER ? Mma16<TP>::pack(s[2 * b + 1][2], s[2 * b + 1][3]) : 0u;
  }
}

// ---------------------------------------------------------------------------
// 16-bit K/V (bf16 or fp16): fragments come straight from the swizzled TMA tiles
// with ldmatrix.  A tile holds TILE rows; a row of D 16-bit elements is stored as
// D/64 separate boxes of [TILE x 128 B], each with the hardware 128-byte swizzle
// (16-byte chunk index XOR (row & 7)), which makes every ldmatrix phase hit eight
// different bank groups.
// With BOXROWS < TILE (paged caches whose pages are shorter than a tile) a tile arrives as
// TILE / BOXROWS boxes of [D/64 pieces x BOXROWS rows x 128 B] instead, one after the other:
// a row's pieces then lie BOXROWS * 128 bytes apart and the 16-key blocks of different pages
// a whole box apart (BOXROWS is a multiple of 16, so a block never straddles two boxes).
// ---------------------------------------------------------------------------
template <int D, int TILE, int BOXROWS>
__device__ __forceinline__ uint32_t tile_row_offset(int key) {
  if constexpr (BOXROWS == TILE) return (uint32_t)key * 128u;
  else return ((uint32_t)key / BOXROWS) * (uint32_t)((D / 64) * BOXROWS * 128) +
              ((uint32_t)key % BOXROWS) * 128u;
}

template <typename T16, int D, int TILE, bool UPPER, bool PARTIAL, int BOXROWS = TILE>
__device__ __forceinline__ void consume_block_16(uint32_t k_base, uint32_t v_base, int key0,
                                                 int valid, const uint32_t (&qa)[D / 16][4],
                                                 WarpState<D, UPPER>& st, float scale_log2,
                                                 int lane) {
  constexpr uint32_t kBoxBytes = BOXROWS * 128;
  float s[2][4];
#pragma unroll
  for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  // S = Q K^T : B operand = K rows (n = key, k = d contiguous)
#pragma unroll
  for (int ks = 0; ks < D / 16; ks += 2) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int key = key0 + 8 * j + (lane & 7);
      const int chunk = 2 * ks + (lane >> 3);
      const uint32_t addr = k_base + (chunk >> 3) * kBoxBytes + tile_row_offset<D, TILE, BOXROWS>(key) +
                            (((chunk & 7) ^ (key & 7)) << 4);
      uint32_t r[4];
      ldsm_x4(r, addr);
      Mma16<T16>::run(s[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r[0], r[1]);
      Mma16<T16>::run(s[j], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], r[2],
                      r[3]);
    }
  }
  uint32_t pa1[1][4];
  softmax_block<T16, D, UPPER, PARTIAL, 1>(s, st, pa1, scale_log2, key0, valid, lane);
  const uint32_t(&pa)[4] = pa1[0];
  // O += P V : B operand = V (k = key, n = d), transposed on load
  const int c = lane & 3;
#pragma unroll
  for (int nt = 0; nt < D / 8; nt += 2) {
    const int key = key0 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int chunk = nt + (lane >> 4);
    const uint32_t addr = v_base + (chunk >> 3) * kBoxBytes + tile_row_offset<D, TILE, BOXROWS>(key) +
                          (((chunk & 7) ^ (key & 7)) << 4);
    uint32_t r[4];
    ldsm_x4_trans(r, addr);
    if (PARTIAL) {
      // rows past the end of the sequence may hold anything (another head's data,
      // padding, NaN patterns): force them to zero so that 0 * V stays 0.
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k0 = key0 + 2 * c + (i & 1) * 8;
        if (k0 >= valid) r[i] = 0u;
        else if (k0 + 1 >= valid) r[i] &= 0x0000ffffu;
      }
    }
    Mma16<T16>::run(st.o[nt], pa[0], pa[1], pa[2], pa[3], r[0], r[1]);
    Mma16<T16>::run(st.o[nt + 1], pa[0], pa[1], pa[2], pa[3], r[2], r[3]);
  }
}

template <typename T16_, int D_, int TILE_, bool UPPER_, int WARPS_ = 4, int BOXROWS_ = TILE_>
struct Kv16Traits {
  static constexpr int kBoxRows = BOXROWS_;  // rows per TMA box: the tile, or a shorter page
  using Q = T16_;
  static constexpr int D = D_;
  static constexpr int TILE = TILE_;
  static constexpr bool UPPER = UPPER_;
  static constexpr int kWarps = WARPS_;  // consumer warps
  static constexpr int kGroups = 1;      // consumer groups taking turns on tiles
  static constexpr bool kFp8 = false;
  static constexpr int kBoxesPerTensor = D * 2 / 128;          // TMA boxes per K (or V) tile
  static constexpr int kBoxBytes = TILE * 128;
  static constexpr int kStageBytes = 2 * kBoxesPerTensor * kBoxBytes;
  static constexpr int kTxBytes = kStageBytes;                 // bytes the loads of a full tile bring
  static constexpr int kPieceBytes = 128;                      // bytes of one box row
  static constexpr int kBoxCols = 64;                          // elements per box row
  static constexpr int kMoStride = D + 8;  // floats per merge row; +8 keeps float2 stores conflict-free
  // float index of (merge row, column) inside a warp's block of merge rows
  __device__ static __forceinline__ int mo_index(int row, int col) { return row * kMoStride + col; }
  // partials the inline merge takes; groups with more go through merge_group_wide
  static constexpr int kMergeBatch = 8;
  struct Extra {};
  __device__ static __forceinline__ void begin_segment(Extra&, const DecodeParams&, int, int) {}
  __device__ static __forceinline__ float out_scale(const Extra&) { return 1.f; }
  // Process the NB 16-key blocks starting at key0 of the tile.
  template <bool PARTIAL, int NB>
  __device__ static __forceinline__ void consume(uint32_t k_base, uint32_t v_base, int key0,
                                                 int valid, const uint32_t (&qa)[D / 16][4],
                                                 WarpState<D, UPPER>& st, float scale_log2,
                                                 int lane, const Extra&) {
#pragma unroll
    for (int b = 0; b < NB; ++b)
      if (!PARTIAL || key0 + 16 * b < valid)
        consume_block_16<Q, D, TILE, UPPER, PARTIAL, kBoxRows>(k_base, v_base, key0 + 16 * b, valid,
                                                               qa, st, scale_log2, lane);
  }
  // Load the A fragments of Q for k-step ks: thread holds d = 16*ks + 2c + {0,1} and +8.
  __device__ static __forceinline__ void load_q(uint32_t (&qa)[D / 16][4], const Q* row0,
                                                const Q* row1, bool v0, bool v1, int c) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d = 16 * ks + 2 * c;
      qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(row0 + d) : 0u;
      qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(row0 + d + 8) : 0u;
      qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(row1 + d) : 0u;
      qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(row1 + d + 8) : 0u;
    }
  }
  // d index of accumulator element (n-tile nt, thread column c, element e).
  __device__ static __forceinline__ int out_col(int nt, int c, int e) { return 8 * nt + 2 * c + e; }
};

// ---------------------------------------------------------------------------
// Merge `n` partials of one group (rows = G query heads) and write the result.
// Executed by the 128 consumer threads of the CTA that completed the group.
// ---------------------------------------------------------------------------
// 8-byte words one source rank's partial occupies in a receive area of the sequence exchange
// (rows * D outputs, then the rows' log-sum-exps padded to an even count so that every
// source's block starts on a 16-byte boundary).
__host__ __device__ inline size_t sequence_exchange_slot_words(long long rows, int D) {
  return (size_t)rows * D + (size_t)((rows + 1) & ~1ll);
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.volatile.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
// Loads for polling words that other SMs or GPUs write: served by L2 (where such stores
// become visible), issued every time the statement is reached (the compiler may neither hoist
// nor merge an asm volatile), and ordinary weak loads to the hardware, so that dozens of them
// overlap.
__device__ __forceinline__ uint4 ld_poll_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_poll_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.cg.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

template <typename Q, int D>
__device__ __forceinline__ void store_final(const DecodeParams& prm, long long out_row, int d4,
                                            float4 v) {
  if (prm.gather_world > 0 && prm.gather_mode == 1) {
    // sequence shard: this rank's normalised fp32 row goes to every rank's receive area, every
    // value tagged with the epoch (two values per 16-byte store; an aligned 8-byte word
    // arrives whole, so a reader that sees the tag sees the value)
    const size_t slot = sequence_exchange_slot_words(prm.gather_rows, D);
    const size_t off = ((size_t)(prm.gather_epoch & 1u) * prm.gather_world + prm.gather_rank) * slot +
                       (size_t)out_row * D + 4 * d4;
    const uint32_t e = prm.gather_epoch;
    for (int p = 0; p < prm.gather_world; ++p) {
      uint2* dst = static_cast<uint2*>(prm.gather_out[p]) + off;
      st_volatile_v4(dst, __float_as_uint(v.x), e, __float_as_uint(v.y), e);
      st_volatile_v4(dst + 2, __float_as_uint(v.z), e, __float_as_uint(v.w), e);
    }
    return;
  }
  if (prm.gather_world > 0) {
    // row (b, head) of this rank is row (b, rank * Hq + head) of the gathered tensor
    const long long b = out_row / prm.num_q_heads, hd = out_row % prm.num_q_heads;
    const long long grow =
        (b * prm.gather_world + prm.gather_rank) * (long long)prm.num_q_heads + hd;
    uint2 pk;
    pk.x = Mma16<Q>::pack(v.x, v.y);
    pk.y = Mma16<Q>::pack(v.z, v.w);
    for (int p = 0; p < prm.gather_world; ++p)
      *reinterpret_cast<uint2*>(reinterpret_cast<Q*>(prm.gather_out[p]) + grow * D + 4 * d4) = pk;
  } else if (prm.out) {
    Q* o = reinterpret_cast<Q*>(prm.out) + out_row * D + 4 * d4;
    uint2 pk;
    pk.x = Mma16<Q>::pack(v.x, v.y);
    pk.y = Mma16<Q>::pack(v.z, v.w);
    *reinterpret_cast<uint2*>(o) = pk;
  }
  if (prm.out_f32) *reinterpret_cast<float4*>(prm.out_f32 + out_row * D + 4 * d4) = v;
}

// Natural-log sum-exp of a final row: to the caller's buffer, or (sequence shards) to every
// rank's receive area next to the row's output.
template <int D>
__device__ __forceinline__ void store_final_lse(const DecodeParams& prm, long long out_row, float lse) {
  if (prm.gather_world > 0 && prm.gather_mode == 1) {
    const size_t slot = sequence_exchange_slot_words(prm.gather_rows, D);
    const size_t off = ((size_t)(prm.gather_epoch & 1u) * prm.gather_world + prm.gather_rank) * slot +
                       (size_t)prm.gather_rows * D + out_row;
    for (int p = 0; p < prm.gather_world; ++p)
      st_volatile_v2(static_cast<uint2*>(prm.gather_out[p]) + off, __float_as_uint(lse), prm.gather_epoch);
    return;
  }
  if (prm.out_lse) prm.out_lse[out_row] = lse;
}

// One (row, 4-column slice) of a merged group from its partial values: weights
// e^(lse_i - max), normalised sum, final store.
template <typename Q, int D, int N>
__device__ __forceinline__ void merge_finish(const DecodeParams& prm, long long out_row, int d4,
                                             const float4 (&o)[N], const float (&l)[N]) {
  float mx = -INFINITY;
#pragma unroll
  for (int u = 0; u < N; ++u) mx = fmaxf(mx, l[u]);
  const float ms = (mx == -INFINITY) ? 0.f : mx;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float wsum = 0.f;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    const float w = fast_exp2((l[u] - ms) * kLog2e);
    acc.x += w * o[u].x;
    acc.y += w * o[u].y;
    acc.z += w * o[u].z;
    acc.w += w * o[u].w;
    wsum += w;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  acc.x *= inv;
  acc.y *= inv;
  acc.z *= inv;
  acc.w *= inv;
  store_final<Q, D>(prm, out_row, d4, acc);
  if (d4 == 0)
    store_final_lse<D>(prm, out_row, wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY);
}

// Up to kBatch partials: every thread fetches the handful of log-sum-exps it needs together
// with the outputs, so the whole merge costs one L2 round trip.
template <typename Q, int D, int kBatch>
__device__ __forceinline__ void merge_small(const DecodeParams& prm, int first_slot, int n,
                                            long long out_row0, int tid, int nthreads) {
  const int G = prm.group;
  constexpr int D4 = D / 4;
  const float* lse_g = prm.part_lse + (size_t)first_slot * G;  // [n, G], contiguous slots
  for (int idx = tid; idx < G * D4; idx += nthreads) {
    const int row = idx / D4, d4 = idx % D4;
    const float4* o_g =
        reinterpret_cast<const float4*>(prm.part_o + ((size_t)first_slot * G + row) * D) + d4;
    float4 o[kBatch];
    float l[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (u < n) {
        l[u] = ld_cg_f32(lse_g + (size_t)u * G + row);
        o[u] = ld_cg_f32x4(o_g + (size_t)u * G * D4);
      } else {
        l[u] = -INFINITY;
        o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    merge_finish<Q, D, kBatch>(prm, out_row0 + row, d4, o, l);
  }
}

// More than kBatch partials, completion-ticket mode, inline: a first pass over the
// log-sum-exps for the row's maximum, then the outputs kBatch at a time (one L2 round trip per
// batch).  Used inside the streaming loop, where an out-of-line call would cost the loop
// more than the merge gains.
template <typename Q, int D, int kBatch>
__device__ __forceinline__ void merge_rounds(const DecodeParams& prm, int first_slot, int n,
                                             long long out_row0, int tid, int nthreads) {
  const int G = prm.group;
  constexpr int D4 = D / 4;
  const float* lse_g = prm.part_lse + (size_t)first_slot * G;
  for (int idx = tid; idx < G * D4; idx += nthreads) {
    const int row = idx / D4, d4 = idx % D4;
    const float4* o_g =
        reinterpret_cast<const float4*>(prm.part_o + ((size_t)first_slot * G + row) * D) + d4;
    float mx = -INFINITY;
    for (int p = 0; p < n; ++p) mx = fmaxf(mx, ld_cg_f32(lse_g + (size_t)p * G + row));
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int p0 = 0; p0 < n; p0 += kBatch) {
      float4 o[kBatch];
      float w[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int p = p0 + u;
        if (p < n) {
          o[u] = ld_cg_f32x4(o_g + (size_t)p * G * D4);
          w[u] = fast_exp2((ld_cg_f32(lse_g + (size_t)p * G + row) - ms) * kLog2e);
        } else {
          o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          w[u] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        acc.x += w[u] * o[u].x;
        acc.y += w[u] * o[u].y;
        acc.z += w[u] * o[u].z;
        acc.w += w[u] * o[u].w;
        wsum += w[u];
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    store_final<Q, D>(prm, out_row0 + row, d4, acc);
    if (d4 == 0)
      store_final_lse<D>(prm, out_row0 + row, wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY);
  }
}

// Many partials, completion-ticket mode (a single long sequence spreads every group over about
// twenty CTAs): the same single round trip with kMergeWide partials per thread.  Kept out of
// line so that its hundred-odd live registers do not weigh on the register allocation of the
// streaming loop; the launch parameters are reached through their address in the parameter space.
// More than kMergeWide partials: a first pass finds the row's largest log-sum-exp, then the
// outputs come kMergeWide at a time.
#ifndef GQA_MERGE_WIDE
#define GQA_MERGE_WIDE 24
#endif
constexpr int kMergeWide = GQA_MERGE_WIDE;
template <typename Q, int D>
__device__ __noinline__ void merge_group_wide(const DecodeParams* __restrict__ prmp, int first_slot,
                                              int n, long long out_row0, int tid, int nthreads) {
  const DecodeParams& prm = *prmp;
  const int G = prm.group;
  constexpr int D4 = D / 4;
  const float* lse_g = prm.part_lse + (size_t)first_slot * G;
  for (int idx = tid; idx < G * D4; idx += nthreads) {
    const int row = idx / D4, d4 = idx % D4;
    const float4* o_g =
        reinterpret_cast<const float4*>(prm.part_o + ((size_t)first_slot * G + row) * D) + d4;
    if (n <= kMergeWide) {
      float4 o[kMergeWide];
      float l[kMergeWide];
#pragma unroll
      for (int u = 0; u < kMergeWide; ++u) {
        if (u < n) {
          l[u] = ld_cg_f32(lse_g + (size_t)u * G + row);
          o[u] = ld_cg_f32x4(o_g + (size_t)u * G * D4);
        } else {
          l[u] = -INFINITY;
          o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      merge_finish<Q, D, kMergeWide>(prm, out_row0 + row, d4, o, l);
      continue;
    }
    float mx = -INFINITY;
    for (int p0 = 0; p0 < n; p0 += 32) {
      float l[32];
#pragma unroll
      for (int u = 0; u < 32; ++u)
        l[u] = p0 + u < n ? ld_cg_f32(lse_g + (size_t)(p0 + u) * G + row) : -INFINITY;
#pragma unroll
      for (int u = 0; u < 32; ++u) mx = fmaxf(mx, l[u]);
    }
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int p0 = 0; p0 < n; p0 += kMergeWide) {
      float4 o[kMergeWide];
      float w[kMergeWide];
#pragma unroll
      for (int u = 0; u < kMergeWide; ++u) {
        const int p = p0 + u;
        if (p < n) {
          o[u] = ld_cg_f32x4(o_g + (size_t)p * G * D4);
          w[u] = fast_exp2((ld_cg_f32(lse_g + (size_t)p * G + row) - ms) * kLog2e);
        } else {
          o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          w[u] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < kMergeWide; ++u) {
        acc.x += w[u] * o[u].x;
        acc.y += w[u] * o[u].y;
        acc.z += w[u] * o[u].z;
        acc.w += w[u] * o[u].w;
        wsum += w[u];
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    store_final<Q, D>(prm, out_row0 + row, d4, acc);
    if (d4 == 0)
      store_final_lse<D>(prm, out_row0 + row, wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY);
  }
}

// A value stored into a polled partial: any bit pattern but zero (zero means "not here yet").
__device__ __forceinline__ float not_zero(float v) {
  return __float_as_uint(v) == 0u ? __uint_as_float(0x80000000u) : v;  // +0 -> -0
}
__device__ __forceinline__ float4 ld_poll_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_poll_f1(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// Merge of a group whose partials announce themselves (DecodeParams::polled), run by one
// designated contributor of the group once its own part is done.  All `nthreads` threads of
// named barrier 1 call it together.  A thread fetches its four columns and the log-sum-exp of
// up to kMergeWide partials at once and fetches again, until the time limit, whatever is
// still zero; in the usual case everything is there at the first look and the merge costs
// one L2 round trip, with no atomic and no fence on anybody's critical path.  The words are
// handed back as zeros for the next launch.
template <typename Q, int D, int kMergeWide>
__device__ __forceinline__ void merge_polled_body(const DecodeParams& prm, int first_slot, int n,
                                                  long long out_row0, int tid, int nthreads) {
  const int G = prm.group;
  constexpr int D4 = D / 4;
  float* lse_g = prm.part_lse + (size_t)first_slot * G;
  // Wait quietly: one thread per log-sum-exp word looks at it every few hundred nanoseconds
  // (a CTA that polled all its words with all its threads would take L2 bandwidth from the
  // CTAs it is waiting for).  Once the log-sum-exps are there the outputs are too, or nearly.
  for (int i = tid; i < n * G; i += nthreads) {
    const unsigned long long t0 = global_timer_ns();
    unsigned pause = 64;
    while (__float_as_uint(ld_poll_f1(lse_g + i)) == 0u) {
      if (global_timer_ns() - t0 > prm.wait_limit_ns) break;  // reported by the fetch below
      __nanosleep(pause);
      if (pause < 512) pause *= 2;
    }
  }
  bar_sync(1, nthreads);
  for (int idx = tid; idx < G * D4; idx += nthreads) {
    const int row = idx / D4, d4 = idx % D4;
    float* o_g = prm.part_o + ((size_t)first_slot * G + row) * D + 4 * d4;
    const size_t o_step = (size_t)G * D;  // floats between consecutive partials
    float mx = -INFINITY, wsum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool complete = true;
    for (int p0 = 0; p0 < n && complete; p0 += kMergeWide) {
      float4 o[kMergeWide];
      float l[kMergeWide];
      unsigned pending = n - p0 >= kMergeWide ? (kMergeWide == 32 ? 0xffffffffu : (1u << kMergeWide) - 1u)
                                              : (1u << (n - p0)) - 1u;
      const unsigned long long t0 = global_timer_ns();
      for (;;) {
#pragma unroll
        for (int u = 0; u < kMergeWide; ++u) {
          if ((pending >> u) & 1u) {
            l[u] = ld_poll_f1(lse_g + (size_t)(p0 + u) * G + row);
            o[u] = ld_poll_f4(o_g + (size_t)(p0 + u) * o_step);
          }
        }
#pragma unroll
        for (int u = 0; u < kMergeWide; ++u) {
          if (((pending >> u) & 1u) && __float_as_uint(l[u]) != 0u && __float_as_uint(o[u].x) != 0u &&
              __float_as_uint(o[u].y) != 0u && __float_as_uint(o[u].z) != 0u &&
              __float_as_uint(o[u].w) != 0u)
            pending &= ~(1u << u);
        }
        if (!pending) break;
        if (global_timer_ns() - t0 > prm.wait_limit_ns) {
          atomicOr(prm.status, kStatusWaitPartial);
          complete = false;
          break;
        }
        __nanosleep(100);
      }
      if (!complete) break;
      // running maximum across batches of partials (one batch is the usual case)
      float bm = -INFINITY;
#pragma unroll
      for (int u = 0; u < kMergeWide; ++u)
        if (p0 + u < n) bm = fmaxf(bm, l[u]);
      const float mnew = fmaxf(mx, bm);
      const float ms = (mnew == -INFINITY) ? 0.f : mnew;
      if (p0 > 0) {
        const float keep = fast_exp2((mx - ms) * kLog2e);
        acc.x *= keep;
        acc.y *= keep;
        acc.z *= keep;
        acc.w *= keep;
        wsum *= keep;
      }
      mx = mnew;
#pragma unroll
      for (int u = 0; u < kMergeWide; ++u) {
        if (p0 + u < n) {
          const float w = fast_exp2((l[u] - ms) * kLog2e);
          acc.x += w * o[u].x;
          acc.y += w * o[u].y;
          acc.z += w * o[u].z;
          acc.w += w * o[u].w;
          wsum += w;
        }
      }
    }
    if (!complete) continue;
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    store_final<Q, D>(prm, out_row0 + row, d4, acc);
    if (d4 == 0)
      store_final_lse<D>(prm, out_row0 + row, wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY);
    for (int p = 0; p < n; ++p) {
      *reinterpret_cast<float4*>(o_g + (size_t)p * o_step) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d4 == 0) lse_g[(size_t)p * G + row] = 0.f;
    }
  }
}
// The polled merge as it runs after a CTA's streaming, when the pipeline stages in shared
// memory are free: a thread copies its four columns and the log-sum-exp of every partial
// straight into shared memory with cp.async (no destination registers, so a short rolled loop
// puts dozens of copies in flight), waits once, and folds them together from shared memory.
// Code executed once per launch is cold in the instruction cache: two small loops cost a
// fraction of what an unrolled register version costs, and they need next to no registers.
// `stage` is 16-byte aligned scratch of `stage_bytes` bytes, private to the calling threads.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}
template <typename Q, int D>
__device__ __forceinline__ void merge_polled_staged(const DecodeParams& prm, int first_slot, int n,
                                                    long long out_row0, int tid, int nthreads,
                                                    uint8_t* stage, int stage_bytes) {
  const int G = prm.group;
  constexpr int D4 = D / 4;
  float* lse_g = prm.part_lse + (size_t)first_slot * G;
  // Wait quietly until every log-sum-exp is there (see merge_polled_body); the values go into
  // shared memory for everybody (read from L2 here, never again).
  float* lse_sm = reinterpret_cast<float*>(stage);  // [n][G]
  const int lse_bytes = (n * G * 4 + 15) & ~15;
  for (int i = tid; i < n * G; i += nthreads) {
    const unsigned long long t0 = global_timer_ns();
    unsigned pause = 64;
    float v;
    while (__float_as_uint(v = ld_poll_f1(lse_g + i)) == 0u) {
      if (global_timer_ns() - t0 > prm.wait_limit_ns) break;  // v stays 0: reported below
      __nanosleep(pause);
      if (pause < 512) pause *= 2;
    }
    lse_sm[i] = v;
  }
  bar_sync(1, nthreads);
  if (prm.timestamps && tid == 0) prm.timestamps[kTimestampWords * blockIdx.x + 8] = global_timer_ns();
  int cap = (stage_bytes - lse_bytes) / (nthreads * 16);  // partials per batch: 16 bytes per thread each
  if (cap > 64) cap = 64;
  float4* my_o = reinterpret_cast<float4*>(stage + lse_bytes) + tid;  // [cap][nthreads]
  const uint32_t my_o_addr = smem_u32(my_o);
  const size_t o_step = (size_t)G * D;  // floats between consecutive partials
  for (int idx = tid; idx < G * D4; idx += nthreads) {
    const int row = idx / D4, d4 = idx % D4;
    float* o_g = prm.part_o + ((size_t)first_slot * G + row) * D + 4 * d4;
    float mx = -INFINITY, wsum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool complete = true;
    for (int p = 0; p < n; ++p) {
      const float l = lse_sm[p * G + row];
      complete = complete && __float_as_uint(l) != 0u;
      mx = fmaxf(mx, l);
    }
    if (!complete) atomicOr(prm.status, kStatusWaitPartial);
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    for (int p0 = 0; p0 < n && complete; p0 += cap) {
      const int nb = n - p0 < cap ? n - p0 : cap;
      const unsigned long long t0 = global_timer_ns();
      for (;;) {
        for (int p = 0; p < nb; ++p)
          cp_async_16(my_o_addr + (uint32_t)p * nthreads * 16, o_g + (size_t)(p0 + p) * o_step);
        cp_async_wait_all();
        bool all_there = true;
        for (int p = 0; p < nb; ++p) {
          const float4 o = my_o[p * nthreads];
          all_there = all_there && __float_as_uint(o.x) != 0u && __float_as_uint(o.y) != 0u &&
                      __float_as_uint(o.z) != 0u && __float_as_uint(o.w) != 0u;
        }
        if (all_there) break;
        if (global_timer_ns() - t0 > prm.wait_limit_ns) {
          atomicOr(prm.status, kStatusWaitPartial);
          complete = false;
          break;
        }
        __nanosleep(200);
      }
      if (!complete) break;
      if (prm.timestamps && tid == 0 && idx == 0) prm.timestamps[kTimestampWords * blockIdx.x + 9] = global_timer_ns();
      for (int p = 0; p < nb; ++p) {
        const float w = fast_exp2((lse_sm[(p0 + p) * G + row] - ms) * kLog2e);
        const float4 o = my_o[p * nthreads];
        acc.x += w * o.x;
        acc.y += w * o.y;
        acc.z += w * o.z;
        acc.w += w * o.w;
        wsum += w;
      }
    }
    if (!complete) continue;
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    store_final<Q, D>(prm, out_row0 + row, d4, acc);
    if (d4 == 0)
      store_final_lse<D>(prm, out_row0 + row, wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY);
    if (prm.timestamps && tid == 0 && idx == 0) prm.timestamps[kTimestampWords * blockIdx.x + 10] = global_timer_ns();
    for (int p = 0; p < n; ++p) {
      *reinterpret_cast<float4*>(o_g + (size_t)p * o_step) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (d4 == 0) lse_g[(size_t)p * G + row] = 0.f;
    }
  }
}

// Sequence shards, end of the kernel: LSE-weighted merge of the `world` partials of this CTA's
// share of the rows (the algebra of merge_rows_kernel, i.e. of gqa_decode/gqa_decode.py:661-669
// one level up).  The partials sit in this rank's receive area as {value, epoch} words; a
// thread fetches all sources of its (row, 4 columns) at once and fetches again, until a time
// limit, whatever does not carry this step's epoch yet.  A row whose sources never all arrive
// is left unwritten and the status word gets kStatusWaitExchange.  All `nthreads` threads of
// named barrier 1 call it together.
template <typename Q, int D>
__device__ __noinline__ void merge_sequence_shards(const DecodeParams* __restrict__ prmp, int tid,
                                                   int nthreads) {
  const DecodeParams& prm = *prmp;
  constexpr int D4 = D / 4;
  const int w = prm.gather_world;
  const uint32_t e = prm.gather_epoch;
  const long long rows = prm.gather_rows;
  const size_t slot = sequence_exchange_slot_words(rows, D);
  const uint2* part =
      static_cast<const uint2*>(prm.gather_out[prm.gather_rank]) + (size_t)(e & 1u) * w * slot;
  const long long r0 = rows * blockIdx.x / gridDim.x, r1 = rows * (blockIdx.x + 1) / gridDim.x;
  // Wait quietly: one thread per (row of this CTA's share, source rank) looks at that row's
  // log-sum-exp word every few hundred nanoseconds.  (If every thread polled all its words,
  // two thousand threads would keep L2 busy with tens of loads each per poll - bandwidth the
  // CTAs that still stream, and whose rows everybody is waiting for, need.)
  for (long long i = tid; i < (r1 - r0) * w; i += nthreads) {
    const long long row = r0 + i / w;
    const uint2* word = part + (size_t)(i % w) * slot + (size_t)rows * D + row;
    const unsigned long long t0 = global_timer_ns();
    unsigned pause = 64;
    while (ld_poll_v2(word).y != e) {
      if (global_timer_ns() - t0 > prm.wait_limit_ns) break;  // reported by the fetch below
      __nanosleep(pause);
      if (pause < 512) pause *= 2;
    }
  }
  bar_sync(1, nthreads);
  for (long long idx = r0 * D4 + tid; idx < r1 * D4; idx += nthreads) {
    const long long row = idx / D4;
    const int d4 = (int)(idx % D4);
    float4 o[kMaxPeers];
    float l[kMaxPeers];
    unsigned pending = (1u << w) - 1u;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
      uint2 lw[kMaxPeers];
      uint4 a[kMaxPeers], b[kMaxPeers];
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if ((pending >> s) & 1u) {
          const uint2* src = part + (size_t)s * slot;
          lw[s] = ld_poll_v2(src + (size_t)rows * D + row);
          a[s] = ld_poll_v4(src + (size_t)row * D + 4 * d4);
          b[s] = ld_poll_v4(src + (size_t)row * D + 4 * d4 + 2);
        }
      }
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if (((pending >> s) & 1u) && lw[s].y == e && a[s].y == e && a[s].w == e && b[s].y == e &&
            b[s].w == e) {
          l[s] = __uint_as_float(lw[s].x);
          o[s] = make_float4(__uint_as_float(a[s].x), __uint_as_float(a[s].z),
                             __uint_as_float(b[s].x), __uint_as_float(b[s].z));
          pending &= ~(1u << s);
        }
      }
      if (!pending) break;
      if (global_timer_ns() - t0 > prm.wait_limit_ns) {
        atomicOr(prm.status, kStatusWaitExchange);
        break;
      }
      __nanosleep(200);
    }
    if (pending) continue;
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < kMaxPeers; ++s)
      if (s < w) mx = fmaxf(mx, l[s]);
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxPeers; ++s) {
      if (s < w) {
        const float wt = fast_exp2((l[s] - ms) * kLog2e);
        acc.x += wt * o[s].x;
        acc.y += wt * o[s].y;
        acc.z += wt * o[s].z;
        acc.w += wt * o[s].w;
        wsum += wt;
      }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    acc.x *= inv;
    acc.y *= inv;
    acc.z *= inv;
    acc.w *= inv;
    if (prm.out) {
      uint2 pk;
      pk.x = Mma16<Q>::pack(acc.x, acc.y);
      pk.y = Mma16<Q>::pack(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<Q*>(prm.out) + row * D + 4 * d4) = pk;
    }
    if (prm.out_f32) *reinterpret_cast<float4*>(prm.out_f32 + row * D + 4 * d4) = acc;
    if (prm.out_lse && d4 == 0)
      prm.out_lse[row] = wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY;
  }
}

// ---------------------------------------------------------------------------
// The kernel.
// ---------------------------------------------------------------------------
// Producer warps per CTA.  With 8 consumer warps the producer gets a whole warpgroup of
// its own (only one warp works) so that `setmaxnreg` can move registers from it to the
// two consumer warpgroups: 12 warps x 168 registers at launch become 56 for the producer
// warpgroup and 224 for the consumers.
template <class Tr>
struct BlockShape {
  static constexpr int kProducerWarps = Tr::kWarps == 8 ? 4 : 1;
  static constexpr int kThreads = (Tr::kWarps + kProducerWarps) * 32;
  static constexpr bool kRebalanceRegs = Tr::kWarps == 8;
};

// Stage index and use parity of the next tile (it % nst and (it / nst) & 1 without the
// divisions: both run once per tile on every warp's critical path).
__device__ __forceinline__ void next_stage(uint32_t& stage, uint32_t& parity, int nst) {
  if (++stage == (uint32_t)nst) {
    stage = 0;
    parity ^= 1u;
  }
}

// ------------------------------------------------------------------ producer
template <class Tr>
struct Producer {
  const CUtensorMap* tm_k;
  const CUtensorMap* tm_v;
  const DecodeParams* prm;
  TileDesc* sm_desc;
  volatile int* sm_published;
  uint32_t full0, empty0, stage_addr0;
  uint64_t policy;
  uint32_t it;        // tiles posted so far
  uint32_t stg, par;  // stage of tile `it` and the parity of its use: it % nst, (it / nst) & 1
  int nst, lane;
  bool dead;
  bool wait_grid;  // the previous kernel of the stream has not been waited for yet
  // paged layouts: 32 consecutive block-table entries of one sequence, one per lane
  int pg_seq, pg_base, pg_entry;
#ifdef GQA_PROFILE_WAITS
  long long wait_cycles;  // diagnostics build: cycles spent waiting for a free stage
#endif

  __device__ __forceinline__ void step() {
    ++it;
    next_stage(stg, par, nst);
  }
  // Wait for the stage of tile `it` to be free, publish its descriptor and start the
  // loads (or just signal when there is no data).  All lanes call it; lane 0 acts.
  // `piece` is the first 128-byte piece of the head's row (non-zero only for page rows with
  // interleaved heads).
  __device__ __forceinline__ void post(const TileDesc& d, long long row, int piece = 0) {
    if (dead) return;
    if (wait_grid) {
      griddep_wait();
      wait_grid = false;
    }
    const uint32_t s = stg, ph = par;
    int ok = 1;
#ifdef GQA_PROFILE_WAITS
    const long long w0 = clock64();
#endif
    if (lane == 0) ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, prm->wait_limit_ns) ? 1 : 0;
#ifdef GQA_PROFILE_WAITS
    wait_cycles += clock64() - w0;
#endif
    if (!__shfl_sync(0xffffffffu, ok, 0)) {
      if (lane == 0) atomicOr(prm->status, kStatusWaitEmpty);
      dead = true;
      return;
    }
    if (lane == 0) {
      // The descriptor ring is much deeper than the stage ring and is published before the
      // loads are issued: consumers read it (and fetch a new segment's queries) early.
      sm_desc[it % kDescRing] = d;
      __threadfence_block();
      *sm_published = (int)(it + 1);
      const uint32_t fb = full0 + 8 * s;
      if (d.valid > 0) {
        mbar_expect_tx(fb, Tr::kTxBytes);  // release: the descriptor is visible to waiters
        const uint32_t kdst = stage_addr0 + s * Tr::kStageBytes;
        const uint32_t vdst = kdst + Tr::kBoxesPerTensor * Tr::kBoxBytes;
        if constexpr (Tr::kBoxesPerTensor == 1) {
          tma_load_2d(kdst, tm_k, fb, piece * Tr::kBoxCols, (int)row, policy);
          tma_load_2d(vdst, tm_v, fb, piece * Tr::kBoxCols, (int)row, policy);
        } else {  // one box per tensor: all 128-byte pieces of the rows, piece after piece
          tma_load_3d(kdst, tm_k, fb, 0, (int)row, piece, policy);
          tma_load_3d(vdst, tm_v, fb, 0, (int)row, piece, policy);
        }
      } else {
        mbar_arrive(fb);
      }
      if (it == 0 && prm->timestamps) prm->timestamps[kTimestampWords * blockIdx.x + 1] = global_timer_ns();
    }
    __syncwarp();
    step();
  }

  // Paged layouts with pages of at least a tile: the tile starting at key `key0` of sequence
  // d.b lies inside one page; returns its first row in the tensor-map view (then post() as for
  // the other layouts).  The block table is read 32 entries at a time, one per lane.
  __device__ __forceinline__ int resolve_row(const TileDesc& d, int key0) {
    const int ps = prm->page_size, psh = prm->page_shift;
    const int pidx = psh >= 0 ? key0 >> psh : key0 / ps;
    if (d.b != pg_seq || pidx < pg_base || pidx >= pg_base + 32) {
      pg_seq = d.b;
      pg_base = pidx;
      const int e = pg_base + lane;
      pg_entry = e < prm->table_stride
                     ? __ldg(prm->block_table + (long long)d.b * prm->table_stride + e)
                     : 0;
    }
    const int page = __shfl_sync(0xffffffffu, pg_entry, pidx - pg_base);
    const int off = key0 - pidx * ps;
    return prm->sched.layout == kLayoutPagedHnd ? (page * prm->sched.num_kv_heads + d.h) * ps + off
                                                : page * ps + off;
  }

  // Paged layouts with pages shorter than a tile: the tile holds keys [key0, key0 + d.valid)
  // of sequence d.b, head d.h.
  // It is fetched as boxes of prm->box_rows rows, each inside one page; lane j resolves and
  // issues box j, and boxes that start past the last valid key are not fetched (consumers
  // mask those rows).  The block table is read 32 entries at a time, one per lane.
  __device__ __forceinline__ void post_paged(const TileDesc& d, int key0) {
    if (dead) return;
    if (wait_grid) {
      griddep_wait();
      wait_grid = false;
    }
    const uint32_t s = stg, ph = par;
    // (shifts instead of divisions: this runs once per tile on the producer's critical path)
    const int ps = prm->page_size, psh = prm->page_shift, bsh = prm->box_shift;
    const int nbox = (d.valid + (1 << bsh) - 1) >> bsh;
    const int last_key = key0 + d.valid - 1;
    const int pg_first = psh >= 0 ? key0 >> psh : key0 / ps;
    const int pg_last = psh >= 0 ? last_key >> psh : last_key / ps;
    if (d.b != pg_seq || pg_first < pg_base || pg_last >= pg_base + 32) {
      pg_seq = d.b;
      pg_base = pg_first;
      const int e = pg_base + lane;
      pg_entry = e < prm->table_stride
                     ? __ldg(prm->block_table + (long long)d.b * prm->table_stride + e)
                     : 0;
    }
    const int key = key0 + (lane << bsh);  // first key of this lane's box
    const int pidx = psh >= 0 ? key >> psh : key / ps;
    const int page = __shfl_sync(0xffffffffu, pg_entry, min(pidx - pg_base, 31));
    int ok = 1;
#ifdef GQA_PROFILE_WAITS
    const long long w0 = clock64();
#endif
    if (lane == 0) ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, prm->wait_limit_ns) ? 1 : 0;
#ifdef GQA_PROFILE_WAITS
    wait_cycles += clock64() - w0;
#endif
    if (!__shfl_sync(0xffffffffu, ok, 0)) {
      if (lane == 0) atomicOr(prm->status, kStatusWaitEmpty);
      dead = true;
      return;
    }
    const uint32_t fb = full0 + 8 * s;
    if (lane == 0) {
      sm_desc[it % kDescRing] = d;
      __threadfence_block();
      *sm_published = (int)(it + 1);
      mbar_expect_tx(fb, ((uint32_t)nbox << bsh) * (uint32_t)Tr::kPieceBytes * 2u * Tr::kBoxesPerTensor);
    }
    __syncwarp();
    if (lane < nbox) {
      const int off = key - pidx * ps;
      const bool hnd = prm->sched.layout == kLayoutPagedHnd;
      const int row = hnd ? (page * prm->sched.num_kv_heads + d.h) * ps + off : page * ps + off;
      const int col0 = hnd ? 0 : d.h * (Tr::kBoxCols * Tr::kBoxesPerTensor);
      if constexpr (Tr::kBoxRows < Tr::TILE) {
        // instantiation for one page size: a box brings all 128-byte pieces of the page's rows
        // (3-D view) and the boxes of a tile follow each other in the stage
        const uint32_t kdst = stage_addr0 + s * Tr::kStageBytes +
                              (uint32_t)lane * (Tr::kBoxesPerTensor * Tr::kBoxRows * 128);
        const uint32_t vdst = kdst + Tr::kBoxesPerTensor * Tr::kBoxBytes;
        const int piece0 = hnd ? 0 : d.h * Tr::kBoxesPerTensor;
        tma_load_3d(kdst, tm_k, fb, 0, row, piece0, policy);
        tma_load_3d(vdst, tm_v, fb, 0, row, piece0, policy);
      } else {
        const uint32_t kdst = stage_addr0 + s * Tr::kStageBytes + ((uint32_t)lane << bsh) * Tr::kPieceBytes;
        const uint32_t vdst = kdst + Tr::kBoxesPerTensor * Tr::kBoxBytes;
#pragma unroll
        for (int bx = 0; bx < Tr::kBoxesPerTensor; ++bx)
          tma_load_2d(kdst + bx * Tr::kBoxBytes, tm_k, fb, col0 + bx * Tr::kBoxCols, row, policy);
#pragma unroll
        for (int bx = 0; bx < Tr::kBoxesPerTensor; ++bx)
          tma_load_2d(vdst + bx * Tr::kBoxBytes, tm_v, fb, col0 + bx * Tr::kBoxCols, row, policy);
      }
    }
    __syncwarp();
    step();
  }
};

// A run of consecutive chunks [q, q + n) handed to a CTA.
struct ChunkRun {
  long long q;
  int n;  // 0: nothing left anywhere
};

// Chunk hand-out.  CTA c owns the chunk range [q0, q1).  Its first part is private: the
// owner walks it without any atomic and nobody else may touch it.  The rest is shared
// through one 64-bit word {taken from the front by the owner : low 32 bits, taken from
// the back by thieves : high 32 bits}; a grab is one atomicAdd and succeeds while
// front + back stays below the shared length.  The owner takes several chunks per atomic
// (a quarter of what is left), a thief one chunk from the CTA that has most left.
struct ChunkSource {
  long long q0, q1, shared0;  // own range and the start of its shared part
  bool private_left, own_left;

  __device__ __forceinline__ static long long shared_start(long long a, long long b, int steal) {
    // without stealing everything is private; with it the last 3/8 of the range is shared
    return steal ? b - ((b - a) * 3) / 8 : b;
  }
  __device__ __forceinline__ void init(const Walker& wk, int cta) {
    wk.cta_range(cta, q0, q1);
    shared0 = shared_start(q0, q1, wk.p.steal);
    private_left = shared0 > q0;
    own_left = q1 > shared0;
  }
  // Warp-cooperative; identical result on all lanes.
  __device__ __forceinline__ ChunkRun next(const Walker& wk, const DecodeParams& prm, int cta,
                                           int lane) {
    const unsigned full = 0xffffffffu;
    ChunkRun r{0, 0};
    if (private_left) {
      private_left = false;
      r.q = q0;
      r.n = (int)(shared0 - q0);
      return r;
    }
    if (own_left) {
      const long long ns = q1 - shared0;
      // ask for a quarter of the shared part at a time (at least one chunk)
      long long ask = ns / 4;
      if (ask < 1) ask = 1;
      unsigned long long old = 0;
      if (lane == 0) old = atomicAdd(prm.deques + cta, (unsigned long long)ask);
      old = __shfl_sync(full, old, 0);
      const long long lo = (long long)(old & 0xffffffffull), hi = (long long)(old >> 32);
      long long got = ns - hi - lo;
      if (got > ask) got = ask;
      if (got > 0) {
        r.q = shared0 + lo;
        r.n = (int)got;
        return r;
      }
      own_left = false;
    }
    if (!wk.p.steal) return r;
    for (int attempt = 0; attempt < 8; ++attempt) {
      long long best = 0;
      int victim = -1;
      for (int v = lane; v < (int)wk.parts; v += 32) {
        if (v == cta) continue;
        long long a, b;
        wk.cta_range(v, a, b);
        const long long vs = b - shared_start(a, b, 1);
        const unsigned long long w = __ldcg(prm.deques + v);
        const long long left = vs - (long long)(w & 0xffffffffull) - (long long)(w >> 32);
        if (left > best) {
          best = left;
          victim = v;
        }
      }
      for (int o = 16; o; o >>= 1) {
        const long long ob = __shfl_xor_sync(full, best, o);
        const int ov = __shfl_xor_sync(full, victim, o);
        if (ob > best || (ob == best && ov > victim)) {
          best = ob;
          victim = ov;
        }
      }
      if (best <= 0 || victim < 0) return r;
      long long a, b;
      wk.cta_range(victim, a, b);
      const long long vs = b - shared_start(a, b, 1);
      unsigned long long old = 0;
      if (lane == 0) old = atomicAdd(prm.deques + victim, 1ull << 32);
      old = __shfl_sync(full, old, 0);
      const long long lo = (long long)(old & 0xffffffffull), hi = (long long)(old >> 32);
      if (lo + hi < vs) {
        r.q = b - 1 - hi;
        r.n = 1;
        return r;
      }
    }
    return r;
  }
};

template <class Tr>
__global__ void __launch_bounds__(BlockShape<Tr>::kThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ DecodeParams prm) {
  using Q = typename Tr::Q;
  constexpr int D = Tr::D;
  constexpr int TILE = Tr::TILE;
  constexpr bool UPPER = Tr::UPPER;
  constexpr int kConsumerWarps = Tr::kWarps;
  constexpr int kConsumerThreads = kConsumerWarps * 32;
  static_assert(Tr::kGroups == 1, "every consumer warp takes its slice of every tile");
  constexpr int kWarpsPerGroup = kConsumerWarps;
  constexpr int kRowsPerWarp = TILE / kWarpsPerGroup;
  static_assert(kRowsPerWarp % 16 == 0, "each consumer warp works in 16-key blocks");
  constexpr int NB = kRowsPerWarp / 16;
  constexpr int kMoStride = Tr::kMoStride;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const int nst = prm.num_stages;
  const int G = prm.group;
  const int grows = UPPER ? 16 : 8;
  uint8_t* stage0 = smem;
  float* sm_o = reinterpret_cast<float*>(smem + (size_t)nst * Tr::kStageBytes);
  float* sm_ml = sm_o + (size_t)kConsumerWarps * grows * kMoStride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm_ml + kConsumerWarps * grows * 2);
  TileDesc* sm_desc = reinterpret_cast<TileDesc*>(bars + 2 * kMaxStages);
  int* sm_flag = reinterpret_cast<int*>(sm_desc + kDescRing);
  volatile int* sm_published = sm_flag + 1;
  volatile int* sm_deferred = sm_flag + 3;  // merges put off so far
  int* sm_defer_list = sm_flag + 8;         // kDeferCap x {first slot, partials, first output row}
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
  const uint32_t stage_addr0 = smem_u32(stage0);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int Hkv = prm.sched.num_kv_heads;

  if (tid == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kWarpsPerGroup);
    }
    *sm_published = 0;
    *sm_deferred = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  __syncthreads();
  // Nothing above touched global memory.  Under programmatic dependent launch the next
  // kernel of the stream may be scheduled from here on (its CTAs become resident as this
  // grid's CTAs leave their SMs) and this kernel must wait for the previous one before it
  // reads inputs that kernel may have written, or touches the workspace they share.
  if (prm.pdl) griddep_launch_dependents();
  if (prm.timestamps && tid == 0) prm.timestamps[kTimestampWords * blockIdx.x] = global_timer_ns();

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------ producer warp
    if (BlockShape<Tr>::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp != kConsumerWarps) return;
    // With uniform lengths and static ranges the schedule is pure arithmetic: it is worked
    // out while the previous kernel drains, and the wait moves to the first load.
    const bool wait_late = prm.pdl && !prm.sched.seq_lens && !prm.sched.steal;
    if (prm.pdl && !wait_late) griddep_wait();
    Walker wk;
    wk.init_warp(prm.sched);
    Producer<Tr> pr;
    pr.tm_k = &tm_k;
    pr.tm_v = &tm_v;
    pr.prm = &prm;
    pr.sm_desc = sm_desc;
    pr.sm_published = sm_published;
    pr.full0 = full0;
    pr.empty0 = empty0;
    pr.stage_addr0 = stage_addr0;
    pr.policy = l2_evict_first_policy();
    pr.it = 0;
    pr.stg = 0;
    pr.par = 0;
    pr.nst = nst;
    pr.lane = lane;
    pr.dead = false;
    pr.wait_grid = wait_late;
#ifdef GQA_PROFILE_WAITS
    pr.wait_cycles = 0;
    const long long pc0 = clock64();
#endif
    pr.pg_seq = -1;
    pr.pg_base = 0;
    pr.pg_entry = 0;
    // 0: rows addressed directly; 1: pages of at least a tile (one box per tile and tensor);
    // 2: smaller pages (several boxes per tile)
    const int paged = prm.sched.layout < kLayoutPagedHnd ? 0 : (prm.box_rows == TILE ? 1 : 2);
    const int nhd_pieces = prm.sched.layout == kLayoutPagedHnd ? 0 : Tr::kBoxesPerTensor;
    const int cta = blockIdx.x;
    TileDesc d;
    if (prm.sched.num_splits > 0) {
      // explicit split-K: a static run of (group, piece) units, one segment each
      long long u0, u1;
      wk.cta_range(cta, u0, u1);
      if (u1 > u0) wk.seek_unit_warp(u0);
      for (long long u = u0; u < u1 && !pr.dead; ++u) {
        Segment sg;
        wk.next_unit(sg);
        const int rows = sg.row_end - sg.row_begin;
        const int ntiles = (rows + TILE - 1) / TILE;
        d.b = sg.b;
        d.h = sg.h;
        d.ntg = ntiles;
        d.first_slot = sg.first_slot;
        d.slot = sg.slot;
        d.n_parts = sg.n_parts;
        if (ntiles == 0) {
          d.valid = 0;
          d.flags = kTileFirst | kTileLast | (sg.first_slot < u0 ? kTileShared : 0);
          pr.post(d, 0);
        }
        for (int t = 0; t < ntiles; ++t) {
          d.valid = min(TILE, rows - t * TILE);
          d.flags = (t == 0 ? kTileFirst : 0) | (t == ntiles - 1 ? kTileLast : 0) |
                    (sg.first_slot < u0 ? kTileShared : 0);
          if (paged == 2) pr.post_paged(d, sg.row_begin + t * TILE);
          else if (paged) pr.post(d, pr.resolve_row(d, sg.row_begin + t * TILE), d.h * nhd_pieces);
          else pr.post(d, sg.kv_row0 + sg.row_begin + (long long)t * TILE);
        }
      }
    } else {
      ChunkSource src;
      src.init(wk, cta);
      ChunkRun cur = src.next(wk, prm, cta, lane);
      long long t = 0, t_end = 0, tmp;
      if (cur.n > 0) {
        wk.chunk_tile_range(cur.q, t, tmp);
        wk.chunk_tile_range(cur.q + cur.n - 1, tmp, t_end);
        wk.seek_warp(t);
      }
      bool open = false;
      int cached_group = -1;  // group whose per-group descriptor fields are in `d`
      long long row0 = 0;
      while (cur.n > 0 && !pr.dead) {
        ChunkRun nxt{0, 0};
        bool contiguous = false;
        for (; t < t_end; ++t) {
          if (t == t_end - 1) {
            // only the last tile of a run needs to know whether the segment continues:
            // fetch the next run now (the ring is full, so the atomic's latency is hidden)
            nxt = src.next(wk, prm, cta, lane);
            contiguous = nxt.n > 0 && nxt.q == cur.q + cur.n;
          }
          if (wk.ti < 0) {  // a unit of the group's fixed overhead: nothing to load
            wk.advance();
            continue;
          }
          const int gi = wk.b * Hkv + wk.h;
          if (gi != cached_group) {
            // per-group values are computed once per group
            cached_group = gi;
            d.b = wk.b;
            d.h = wk.h;
            d.ntg = wk.ntg;
            row0 = wk.kv_row0();
            if (prm.sched.steal) {
              d.first_slot = wk.group_first_slot();
              d.slot = -1;
              d.n_parts = 0;
            } else {
              int index;
              wk.group_static_slots(cta, d.first_slot, d.n_parts, index);
              d.slot = d.first_slot + index;
            }
          }
          const bool last = (wk.ti == wk.ntg - 1) || (t == t_end - 1 && !contiguous);
          d.valid = min(TILE, wk.len - wk.ti * TILE);
          d.flags = (open ? 0 : kTileFirst) | (last ? kTileLast : 0) | kTileShared;
          if (paged == 2) pr.post_paged(d, wk.ti * TILE);
          else if (paged) pr.post(d, pr.resolve_row(d, wk.ti * TILE), d.h * nhd_pieces);
          else pr.post(d, row0 + (long long)wk.ti * TILE);
          open = !last;
          wk.advance();
        }
        if (nxt.n <= 0) break;
        wk.chunk_tile_range(nxt.q, t, tmp);
        wk.chunk_tile_range(nxt.q + nxt.n - 1, tmp, t_end);
        if (!contiguous) {
          wk.seek_warp(t);
          cached_group = -1;
        }
        cur = nxt;
      }
    }
    d.valid = 0;
    d.flags = kTileEnd;
    pr.post(d, 0);
#ifdef GQA_PROFILE_WAITS
    if (prm.timestamps && lane == 0) {
      unsigned long long* ts = prm.timestamps + kTimestampWords * gridDim.x + 5 * blockIdx.x;
      ts[0] = (unsigned long long)pr.wait_cycles;
      ts[1] = (unsigned long long)(clock64() - pc0);
      ts[2] = pr.it;
    }
#endif
    return;
  }

  // -------------------------------------------------------------- consumers
  if (BlockShape<Tr>::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
  if (prm.pdl) griddep_wait();
  const int r0 = lane >> 2, c = lane & 3;
  const int Hq = prm.num_q_heads;
  const bool dynamic = prm.sched.num_splits == 0 && prm.sched.steal;
  const bool polled = prm.polled != 0;

  // Sequences without keys own no tiles in the balanced schedule: their outputs are zeros.
  if (prm.sched.num_splits == 0 && prm.sched.seq_lens) {
    for (int b = blockIdx.x; b < prm.sched.batch; b += gridDim.x) {
      if (__ldg(prm.sched.seq_lens + b) > 0) continue;
      for (int idx = tid; idx < Hq * (D / 4); idx += kConsumerThreads) {
        const int row = idx / (D / 4), d4 = idx % (D / 4);
        store_final<Q, D>(prm, (long long)b * Hq + row, d4, make_float4(0.f, 0.f, 0.f, 0.f));
        if (d4 == 0) store_final_lse<D>(prm, (long long)b * Hq + row, -INFINITY);
      }
      if (!prm.fused_merge)
        for (int h = tid; h < Hkv; h += kConsumerThreads)
          prm.group_info[(long long)b * Hkv + h] = make_int2(0, 1);
    }
  }

  WarpState<D, UPPER> st;
  uint32_t qa[D / 16][4];
  typename Tr::Extra extra;
  int seg_tiles = 0;
#ifdef GQA_PROFILE_WAITS
  long long cons_wait = 0;  // diagnostics build: cycles this warp waited for data
  const long long cc0 = clock64();
#endif

  uint32_t s = 0, ph = 0;  // stage of tile `it` and the parity of its use
  uint32_t it = 0;  // descriptors consumed so far
  for (;; ++it, next_stage(s, ph, nst)) {
    // The descriptor is published before the tile's loads are even issued, so it is read
    // first: a new segment's query rows are then fetched while the tile is still in flight.
    bool ok = true;
    if (*sm_published <= (int)it) {
      const unsigned long long t0 = global_timer_ns();
      while (*sm_published <= (int)it) {
        if (global_timer_ns() - t0 > prm.wait_limit_ns) {
          ok = false;
          break;
        }
      }
    }
    __threadfence_block();
    const TileDesc d = sm_desc[it % kDescRing];
    if (!ok) {
      // the producer stopped: every consumer warp runs into this at the same descriptor
      if (lane == 0) atomicOr(prm.status, kStatusWaitFull);
      break;
    }
    if (d.flags & kTileEnd) break;
    const long long g = (long long)d.b * Hkv + d.h;
    const long long out_row0 = (long long)d.b * Hq + (long long)d.h * G;
    if (d.flags & kTileFirst) {
      const Q* qbase = reinterpret_cast<const Q*>(prm.q) + out_row0 * D;
      Tr::load_q(qa, qbase + (size_t)r0 * D, qbase + (size_t)(r0 + 8) * D, r0 < G,
                 UPPER && (r0 + 8 < G), c);
      Tr::begin_segment(extra, prm, d.b, d.h);
      st.reset();
      seg_tiles = 0;
    }
#ifdef GQA_PROFILE_WAITS
    const long long cw0 = clock64();
#endif
    if (!mbar_wait(full0 + 8 * s, ph, prm.wait_limit_ns)) {
      // every consumer warp waits on the same barrier, so all of them give up together
      if (lane == 0) atomicOr(prm.status, kStatusWaitFull);
      break;
    }
#ifdef GQA_PROFILE_WAITS
    cons_wait += clock64() - cw0;
#endif
    if (prm.timestamps && tid == 0 && it == 0)
      prm.timestamps[kTimestampWords * blockIdx.x + 2] = global_timer_ns();
    if (d.valid > 0) {
      ++seg_tiles;
      {
        const uint32_t kb = stage_addr0 + s * Tr::kStageBytes;
        const uint32_t vb = kb + Tr::kBoxesPerTensor * Tr::kBoxBytes;
        const int key0 = (warp % kWarpsPerGroup) * kRowsPerWarp;
        if (d.valid == TILE) {
          Tr::template consume<false, NB>(kb, vb, key0, d.valid, qa, st, prm.scale_log2, lane, extra);
        } else if (key0 < d.valid) {
          Tr::template consume<true, NB>(kb, vb, key0, d.valid, qa, st, prm.scale_log2, lane, extra);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);
    if (!(d.flags & kTileLast)) continue;

    // The next descriptor (normally published long ago) starts a new segment: pull its
    // query rows towards L1 now, so that their load does not wait behind this epilogue.
    if (*sm_published > (int)(it + 1)) {
      __threadfence_block();
      const TileDesc nd = sm_desc[(it + 1) % kDescRing];
      if ((nd.flags & kTileFirst) && tid < G * (D * 2 / 128)) {
        const char* qn = reinterpret_cast<const char*>(prm.q) +
                         ((long long)nd.b * Hq + (long long)nd.h * G) * D * 2 + (size_t)tid * 128;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(qn));
      }
    }

    // ---- end of a segment: combine the consumer warps' states ------------------------
    if (prm.timestamps && tid == 0) prm.timestamps[kTimestampWords * blockIdx.x + 3] = global_timer_ns();
#pragma unroll
    for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
      st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    if (c == 0) {
      sm_ml[(warp * grows + r0) * 2 + 0] = st.m[0];
      sm_ml[(warp * grows + r0) * 2 + 1] = st.l[0];
      if (UPPER) {
        sm_ml[(warp * grows + r0 + 8) * 2 + 0] = st.m[1];
        sm_ml[(warp * grows + r0 + 8) * 2 + 1] = st.l[1];
      }
    }
    // a partial needs a slot: static schedules know it, the stealing schedule takes the
    // group's next free one (the atomic overlaps the combine below)
    const bool direct =
        !prm.no_merge && (dynamic ? seg_tiles == d.ntg : d.n_parts == 1);
    if (tid == 0 && !direct) {
      int sl = d.slot >= 0 ? d.slot : d.first_slot + atomicAdd(prm.alloc + g, 1);
      if (sl < 0 || sl >= prm.num_slots) {  // cannot happen with clean control words; never write outside
        atomicOr(prm.status, kStatusSlotRange);
        sl = -1;
      }
      *sm_flag = sl;
    }
    bar_sync(1, kConsumerThreads);
#pragma unroll
    for (int r = 0; r < (UPPER ? 2 : 1); ++r) {
      const int row = r0 + 8 * r;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, sm_ml[(w * grows + row) * 2]);
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w)
        L += sm_ml[(w * grows + row) * 2 + 1] * fast_exp2(sm_ml[(w * grows + row) * 2] - Ms);
      const float f = L > 0.f ? fast_exp2(st.m[r] - Ms) / L * Tr::out_scale(extra) : 0.f;
      if (row < G) {
        float* dst = sm_o + (size_t)warp * grows * kMoStride;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
          *reinterpret_cast<float2*>(dst + Tr::mo_index(row, Tr::out_col(nt, c, 0))) =
              make_float2(st.o[nt][2 * r] * f, st.o[nt][2 * r + 1] * f);
        }
      }
    }
    const int slot = direct ? 0 : *sm_flag;
    bar_sync(1, kConsumerThreads);
    for (int idx = tid; idx < G * (D / 4); idx += kConsumerThreads) {
      const int row = idx / (D / 4), d4 = idx % (D / 4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(
            sm_o + (size_t)w * grows * kMoStride + Tr::mo_index(row, 4 * d4));
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      if (direct) {
        store_final<Q, D>(prm, out_row0 + row, d4, acc);
      } else if (slot >= 0) {
        if (polled) acc = make_float4(not_zero(acc.x), not_zero(acc.y), not_zero(acc.z), not_zero(acc.w));
        *reinterpret_cast<float4*>(prm.part_o + ((size_t)slot * G + row) * D + 4 * d4) = acc;
      }
    }
    if (tid < G) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, sm_ml[(w * grows + tid) * 2]);
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w)
        L += sm_ml[(w * grows + tid) * 2 + 1] * fast_exp2(sm_ml[(w * grows + tid) * 2] - Ms);
      const float lse = L > 0.f ? (Ms + fast_log2(L)) * kLn2 : -INFINITY;
      if (direct) {
        store_final_lse<D>(prm, out_row0 + tid, lse);
      } else if (slot >= 0) {
        prm.part_lse[(size_t)slot * G + tid] = polled ? not_zero(lse) : lse;
      }
    }
    if (!prm.fused_merge && tid == 0) {
      if (direct) prm.group_info[g] = make_int2(0, 1);
      else if (slot == d.first_slot) prm.group_info[g] = make_int2(d.first_slot, d.n_parts);
    }
    if (!direct && prm.fused_merge) {
      if (polled) {
        // The partial announces itself; one contributor merges the group.  Balanced schedule:
        // the CTA that wrote the group's FIRST partial - its share of the group is the end
        // of its range, so by then the partial of the CTA holding the group's tail (the start
        // of that CTA's range) is long there and the ones in between arrive at the same
        // moment; it merges after its last tile.  Explicit splits: the CTA holding the LAST
        // piece - the earlier pieces are its own, already written (merge on the spot), or a
        // lower CTA's (merge after the last tile).
        const bool mine = prm.sched.num_splits > 0 ? slot == d.first_slot + d.n_parts - 1
                                                   : slot == d.first_slot;
        if (mine && (d.flags & kTileShared)) {
          if (tid == 0) {
            const int at = *sm_deferred;  // never more than one per CTA
            if (at < kDeferCap) {
              sm_defer_list[3 * at] = d.first_slot;
              sm_defer_list[3 * at + 1] = d.n_parts;
              sm_defer_list[3 * at + 2] = (int)out_row0;
              *sm_deferred = at + 1;
            } else {
              atomicOr(prm.status, kStatusSlotRange);
            }
          }
        } else if (mine) {
          merge_polled_body<Q, D, 4>(prm, d.first_slot, d.n_parts, out_row0, tid, kConsumerThreads);
        }
      } else {
        // completion tickets: publish the partial, then count tiles covered (stealing
        // schedule) or partials (static schedules); whoever completes the group merges it.
        // The CTA barrier orders all threads' partial stores before thread 0's
        // release-acquire ticket, and the barrier after it hands the acquired view to the
        // other threads.
        bar_sync(1, kConsumerThreads);
        if (tid == 0) {
          const int add = dynamic ? seg_tiles : 1, want = dynamic ? d.ntg : d.n_parts;
          const int before = atom_add_acq_rel(prm.tickets + g, add);
          int n = 0;
          if (before + add == want) {
            n = dynamic ? atomicAdd(prm.alloc + g, 0) : d.n_parts;
            if (n < 0 || d.first_slot + n > prm.num_slots) {
              atomicOr(prm.status, kStatusSlotRange);
              n = 0;
            }
            prm.tickets[g] = 0;  // every contributor has arrived: leave the counters clean
            prm.alloc[g] = 0;
            if (n > 0 && prm.timestamps) prm.timestamps[kTimestampWords * blockIdx.x + 5] = global_timer_ns();
          }
          *sm_flag = n;
        }
        bar_sync(1, kConsumerThreads);
        const int n = *sm_flag;
        if (n > Tr::kMergeBatch)
          merge_rounds<Q, D, Tr::kMergeBatch>(prm, d.first_slot, n, out_row0, tid, kConsumerThreads);
        else if (n > 0)
          merge_small<Q, D, Tr::kMergeBatch>(prm, d.first_slot, n, out_row0, tid, kConsumerThreads);
      }
    }
    // sm_ml / sm_o / sm_flag are rewritten only after the next segment's barriers.
    bar_sync(1, kConsumerThreads);
  }

  // ---- the group merges that were put off (every consumer thread sees the same list: it was
  // last changed before the barrier that ended the last segment)
  {
    const int todo = *sm_deferred;
    if (todo > 0 && prm.timestamps && tid == 0)
      prm.timestamps[kTimestampWords * blockIdx.x + 5] = global_timer_ns();
    for (int e = 0; e < todo; ++e) {
      const int first_slot = sm_defer_list[3 * e], n = sm_defer_list[3 * e + 1];
      const long long row0 = sm_defer_list[3 * e + 2];
      // (the streaming loop is over and every tile has been consumed: the pipeline stages
      // serve as staging memory)
      merge_polled_staged<Q, D>(prm, first_slot, n, row0, tid, kConsumerThreads, stage0,
                                nst * Tr::kStageBytes);
    }
  }

#ifdef GQA_PROFILE_WAITS
  if (prm.timestamps && tid == 0) {
    unsigned long long* ts = prm.timestamps + kTimestampWords * gridDim.x + 5 * blockIdx.x;
    ts[3] = (unsigned long long)cons_wait;
    ts[4] = (unsigned long long)(clock64() - cc0);
  }
#endif
  if (prm.gather_world > 0 && prm.gather_mode == 1) {
    // sequence shards: every final row of this launch has been pushed to all ranks already
    merge_sequence_shards<Q, D>(&prm, tid, kConsumerThreads);
  } else if (prm.gather_world > 0) {
    // Hand-off of the gathered outputs: every thread's peer stores are fenced at system scope;
    // in the last CTA to get here, thread p raises this rank's flag on peer p (one fence, then
    // a plain system-scope store: eight release stores in a row would pay eight fences) and
    // waits, bounded, for peer p's flag of this epoch.  When the kernel ends, the whole
    // [batch, world * Hq, D] tensor is complete in this rank's buffer.
    __threadfence_system();
    bar_sync(1, kConsumerThreads);
    if (tid == 0) {
      const int before = atom_add_acq_rel(prm.done_ctas, 1);
      const int last = before == (int)gridDim.x - 1;
      if (last) *prm.done_ctas = 0;
      *sm_flag = last;
    }
    bar_sync(1, kConsumerThreads);
    const int w = prm.gather_world;
    const unsigned par = prm.gather_epoch & 1u;
    if (*sm_flag && tid < w) {
      __threadfence_system();
      st_relaxed_sys(prm.gather_flags[tid] + par * w + prm.gather_rank, prm.gather_epoch);
      // only the last CTA has to see the peers' flags before the kernel may end
      const unsigned* mine = prm.gather_flags[prm.gather_rank] + par * w + tid;
      const unsigned long long t0 = global_timer_ns();
      while (ld_acquire_sys(mine) != prm.gather_epoch) {
        if (global_timer_ns() - t0 > prm.wait_limit_ns) {
          atomicOr(prm.status, kStatusWaitExchange);
          break;
        }
        __nanosleep(100);
      }
    }
  }
  if (tid == 0) {
    if (prm.timestamps) {
      unsigned smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      prm.timestamps[kTimestampWords * blockIdx.x + 4] = global_timer_ns();
      prm.timestamps[kTimestampWords * blockIdx.x + 6] = smid;
      prm.timestamps[kTimestampWords * blockIdx.x + 7] = it;
    }
    // work stealing only: the last CTA to finish leaves the chunk deques clean for the
    // next launch
    if (dynamic) {
      __threadfence();
      if (atomicAdd(prm.done_ctas, 1) == (int)gridDim.x - 1) {
        for (int i = 0; i < prm.sched.num_ctas; ++i) prm.deques[i] = 0ull;
        *prm.done_ctas = 0;
      }
    }
  }
}

// Second-kernel merge (one CTA of 128 threads per (sequence, KV head) group), used when
// the in-kernel merge is switched off.
template <typename Q, int D>
__global__ void __launch_bounds__(kMergeThreads)
merge_groups_kernel(const __grid_constant__ DecodeParams prm) {
  const long long g = blockIdx.x;
  const int2 info = prm.group_info[g];
  if (info.y <= 1) return;  // written directly by the decode kernel
  const long long b = g / prm.sched.num_kv_heads, h = g % prm.sched.num_kv_heads;
  const long long out_row0 = b * prm.num_q_heads + h * prm.group;
  if (info.y <= 8) merge_small<Q, D, 8>(prm, info.x, info.y, out_row0, threadIdx.x, kMergeThreads);
  else merge_group_wide<Q, D>(&prm, info.x, info.y, out_row0, threadIdx.x, kMergeThreads);
}

}  // namespace gqa
