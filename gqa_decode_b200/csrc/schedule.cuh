// Work scheduler shared by host and device code.
//
// The KV cache of a batch is cut into tiles of `tile_rows` keys.  A "group" is one
// (sequence, KV head) pair; its tiles are consecutive.  Two policies hand tiles to
// the persistent CTAs:
//
//   balanced (num_splits == 0): all tiles of the batch, in (sequence, KV head, tile)
//     order, are divided into `num_ctas` contiguous ranges of equal size (+-1).  A CTA
//     therefore owns a few "segments" (maximal runs inside one group).  Ragged
//     lengths cost nothing: a long sequence simply spans more CTAs.  This replaces the
//     reference's PersistentDecodeKernel work loop (gqa_decode/gqa_decode.py:865,
//     :902-907) and its host-side sizing (:1408-1410), which recompiles per length
//     and handles one sequence only.
//
//   explicit (num_splits == K > 0): every group is cut into K chunks of
//     ceil(tiles/K) tiles, the classic split-K grid of the reference
//     (gqa_decode/gqa_decode.py:273-274, :1104-1105); units (group, chunk) are dealt to
//     CTAs in contiguous runs.
//
// Each segment produces one partial (normalised O, log-sum-exp) in a numbered slot.
// In balanced mode slot = cta + group: both indices grow monotonically along the
// tile order, so the sum is unique and a group's partials occupy consecutive slots.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define GQA_HD __host__ __device__ __forceinline__
#else
#define GQA_HD inline
#endif

namespace gqa {

enum KvLayout : int {
  kLayoutPadded = 0,  // K/V [batch, Hkv, max_seq, D]: head slab of (b,h) starts at row (b*Hkv+h)*max_seq
  kLayoutPacked = 1,  // K/V [sum_b Hkv*len_b, D]: sequence b holds [Hkv, len_b, D] after all earlier sequences
};

struct SchedParams {
  const int32_t* seq_lens;  // [batch] KV length per sequence; null = every sequence has max_seq keys
  int batch;
  int num_kv_heads;
  int max_seq;     // rows per head slab (padded layout) and upper bound of any length
  int tile_rows;   // keys per pipeline stage
  int num_ctas;    // persistent CTAs
  int num_splits;  // 0 = balanced, K > 0 = explicit split-K
  int layout;      // KvLayout
};

struct Segment {
  int b, h;                // sequence and KV head
  int len;                 // keys in the sequence
  int row_begin, row_end;  // key range [row_begin, row_end) handled by this segment (may be empty)
  long long kv_row0;       // row of key 0 of this (b,h) slab in the 2-D [rows, D] view of K and V
  int slot;                // partial slot written by this segment
  int first_slot;          // first slot of the group
  int n_parts;             // partials the group is made of (1 = the segment is the whole group)
};

struct Walker {
  SchedParams p;
  int cta;
  long long total;  // balanced: tiles in the batch; explicit: units in the batch
  long long parts;  // balanced: CTAs that actually receive tiles = min(num_ctas, total)
  long long rem;    // tiles (balanced) or units (explicit) this CTA still owns
  long long unit;   // explicit: next unit
  int b, h, ti;     // balanced cursor: sequence, head, first unprocessed tile of the group
  int len, ntg;     // length and tile count of sequence b
  long long tiles_before_group;
  long long rows_before_seq;

  GQA_HD int len_of(int bb) const {
    int l = p.max_seq;
    if (p.seq_lens) {
#if defined(__CUDA_ARCH__)
      l = __ldg(p.seq_lens + bb);
#else
      l = p.seq_lens[bb];
#endif
      if (l < 0) l = 0;
      if (p.layout == kLayoutPadded && l > p.max_seq) l = p.max_seq;
    }
    return l;
  }
  GQA_HD int tiles_of(int l) const { return (l + p.tile_rows - 1) / p.tile_rows; }
  GQA_HD long long cta_of_tile(long long t) const {
    // largest c with floor(c*total/parts) <= t.  parts <= total, so every one of the
    // `parts` ranges is non-empty and a group's CTAs are consecutive.
    return ((t + 1) * parts - 1) / total;
  }

  // Finish initialisation once `total`, the starting sequence and the sums over the
  // sequences before it are known.
  GQA_HD void seat_balanced(long long t0, long long t1, int b0, long long tiles_before,
                            long long rows_before) {
    rem = t1 - t0;
    b = b0;
    h = 0;
    ti = 0;
    len = 0;
    ntg = 0;
    tiles_before_group = tiles_before;
    rows_before_seq = rows_before;
    if (rem <= 0 || b0 >= p.batch) {
      rem = 0;
      return;
    }
    len = len_of(b);
    ntg = tiles_of(len);
    long long off = t0 - tiles_before;
    h = (int)(off / ntg);
    ti = (int)(off % ntg);
    tiles_before_group = tiles_before + (long long)h * ntg;
  }

  // Serial initialisation: usable from host code or from a single device thread.
  GQA_HD void init_serial(const SchedParams& sp, int cta_index) {
    p = sp;
    cta = cta_index;
    unit = 0;
    if (p.num_splits > 0) {
      total = (long long)p.batch * p.num_kv_heads * p.num_splits;
      unit = cta * total / p.num_ctas;
      rem = (cta + 1) * total / p.num_ctas - unit;
      b = (int)(unit / p.num_splits / p.num_kv_heads);
      parts = p.num_ctas;
      rows_before_seq = 0;
      for (int bb = 0; bb < b && bb < p.batch; ++bb) rows_before_seq += len_of(bb);
      h = ti = len = ntg = 0;
      tiles_before_group = 0;
      return;
    }
    long long n = 0;
    for (int bb = 0; bb < p.batch; ++bb) n += tiles_of(len_of(bb));
    total = n * p.num_kv_heads;
    parts = total < p.num_ctas ? total : p.num_ctas;
    long long t0 = 0, t1 = 0;
    if (cta < parts) {
      t0 = cta * total / parts;
      t1 = (cta + 1) * total / parts;
    }
    long long acc_t = 0, acc_r = 0;
    int b0 = 0;
    for (; b0 < p.batch; ++b0) {
      int l = len_of(b0);
      long long nt = (long long)tiles_of(l) * p.num_kv_heads;
      if (acc_t + nt > t0) break;
      acc_t += nt;
      acc_r += l;
    }
    seat_balanced(t0, t1, b0, acc_t, acc_r);
  }

#if defined(__CUDACC__)
  // Warp-cooperative initialisation: all 32 lanes of a warp call it together and end
  // with identical state.  Lengths are read 32 at a time and combined with shuffles,
  // so the cost is a few dependent L2 reads even for batches of thousands.
  __device__ __forceinline__ void init_warp(const SchedParams& sp, int cta_index) {
    p = sp;
    cta = cta_index;
    unit = 0;
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    if (p.num_splits > 0) {
      total = (long long)p.batch * p.num_kv_heads * p.num_splits;
      unit = cta * total / p.num_ctas;
      rem = (cta + 1) * total / p.num_ctas - unit;
      b = (int)(unit / p.num_splits / p.num_kv_heads);
      parts = p.num_ctas;
      long long r = 0;
      for (int bb = lane; bb < b && bb < p.batch; bb += 32) r += len_of(bb);
      for (int o = 16; o; o >>= 1) r += __shfl_xor_sync(full, r, o);
      rows_before_seq = r;
      h = ti = len = ntg = 0;
      tiles_before_group = 0;
      return;
    }
    long long n = 0;
    for (int bb = lane; bb < p.batch; bb += 32) n += tiles_of(len_of(bb));
    for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(full, n, o);
    total = n * p.num_kv_heads;
    parts = total < p.num_ctas ? total : p.num_ctas;
    long long t0 = 0, t1 = 0;
    if (cta < parts) {
      t0 = cta * total / parts;
      t1 = (cta + 1) * total / parts;
    }
    long long acc_t = 0, acc_r = 0;
    int b0 = p.batch;
    for (int base = 0; base < p.batch; base += 32) {
      int bb = base + lane;
      int l = bb < p.batch ? len_of(bb) : 0;
      long long nt = (long long)tiles_of(l) * p.num_kv_heads;
      long long it = nt, ir = l;  // inclusive scans over the 32 lanes
      for (int o = 1; o < 32; o <<= 1) {
        long long a = __shfl_up_sync(full, it, o);
        long long c = __shfl_up_sync(full, ir, o);
        if (lane >= o) {
          it += a;
          ir += c;
        }
      }
      unsigned hit = __ballot_sync(full, bb < p.batch && acc_t + it > t0);
      if (hit) {
        int first = __ffs(hit) - 1;
        long long et = __shfl_sync(full, it - nt, first);
        long long er = __shfl_sync(full, ir - l, first);
        acc_t += et;
        acc_r += er;
        b0 = base + first;
        break;
      }
      acc_t += __shfl_sync(full, it, 31);
      acc_r += __shfl_sync(full, ir, 31);
    }
    seat_balanced(t0, t1, b0, acc_t, acc_r);
  }
#endif

  // Produce the next segment of this CTA.  Called by single threads; no cross-lane ops.
  GQA_HD bool next(Segment& s) {
    if (rem <= 0) return false;
    const int T = p.tile_rows;
    if (p.num_splits > 0) {
      const int K = p.num_splits;
      long long g = unit / K;
      int sp = (int)(unit % K);
      int nb = (int)(g / p.num_kv_heads);
      while (b < nb) {
        rows_before_seq += len_of(b);
        ++b;
      }
      h = (int)(g % p.num_kv_heads);
      len = len_of(b);
      ntg = tiles_of(len);
      int cs = (ntg + K - 1) / K;
      long long tb = (long long)sp * cs;
      if (tb > ntg) tb = ntg;
      long long te = tb + cs;
      if (te > ntg) te = ntg;
      s.b = b;
      s.h = h;
      s.len = len;
      long long re = te * T;
      s.row_begin = tb == te ? 0 : (int)(tb * T);  // an empty chunk is reported as [0, 0)
      s.row_end = tb == te ? 0 : (int)(re < len ? re : len);
      s.slot = (int)unit;
      s.first_slot = (int)(g * K);
      s.n_parts = K;
      s.kv_row0 = p.layout == kLayoutPadded ? g * (long long)p.max_seq
                                            : rows_before_seq * p.num_kv_heads + (long long)h * len;
      ++unit;
      --rem;
      return true;
    }
    long long take = ntg - ti;
    if (take > rem) take = rem;
    long long g = (long long)b * p.num_kv_heads + h;
    s.b = b;
    s.h = h;
    s.len = len;
    s.row_begin = ti * T;
    long long re = (long long)(ti + take) * T;
    s.row_end = (int)(re < len ? re : len);
    long long cf = cta_of_tile(tiles_before_group);
    long long cl = cta_of_tile(tiles_before_group + ntg - 1);
    s.n_parts = (int)(cl - cf + 1);
    s.first_slot = (int)(cf + g);
    s.slot = (int)(cta + g);
    s.kv_row0 = p.layout == kLayoutPadded ? g * (long long)p.max_seq
                                          : rows_before_seq * p.num_kv_heads + (long long)h * len;
    rem -= take;
    ti += (int)take;
    if (ti == ntg) {
      tiles_before_group += ntg;
      ti = 0;
      if (++h == p.num_kv_heads) {
        h = 0;
        rows_before_seq += len;
        ++b;
        len = 0;
        ntg = 0;
        while (b < p.batch) {
          len = len_of(b);
          ntg = tiles_of(len);
          if (ntg) break;
          ++b;
        }
        if (b >= p.batch) rem = 0;
      }
    }
    return true;
  }
};

// Upper bound on partial slots for a launch.
GQA_HD long long max_slots(int batch, int num_kv_heads, int num_ctas, int num_splits) {
  long long groups = (long long)batch * num_kv_heads;
  return num_splits > 0 ? groups * num_splits : groups + num_ctas;
}

}  // namespace gqa
