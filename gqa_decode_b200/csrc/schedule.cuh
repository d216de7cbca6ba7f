// Work scheduler shared by host and device code.
//
// The KV cache of a batch is cut into tiles of `tile_rows` keys.  A "group" is one
// (sequence, KV head) pair; its tiles are consecutive.  All tiles of the batch, in
// (sequence, KV head, tile) order, form one line.  Every group additionally contributes
// `group_overhead` cost units in front of its tiles: starting and finishing a group
// (query load, cross-warp combine, output write) costs about as much as streaming a
// couple of tiles, and a partition that ignored it would hand a CTA that owns many
// one-tile groups twice the work of its neighbours.  The line is therefore measured in
// units; a unit is either a tile or a slice of a group's overhead.
//
//   balanced (num_splits == 0): the line is cut into M chunks of `chunk_tiles` units (one
//     unit per chunk unless CTAs steal work from each other: equal shares to within a unit) and
//     CTA c owns the chunk range [c*M/P, (c+1)*M/P), P = min(#CTAs, M).  A CTA works
//     through its own range from the front; consecutive chunks fuse into one running
//     segment, so an undisturbed CTA produces one partial per group it touches, exactly
//     like a static split.  A CTA that runs dry steals single chunks from the back of
//     other CTAs' ranges (kernel side, decode_kernel.cuh).  SMs do not stream at the same
//     speed - on B200 the slowest SM needs about 1.3x the time of the fastest for the same
//     bytes - so equal static shares leave most SMs idle while the slowest finishes.
//     Ragged lengths cost nothing: a long sequence simply spans more chunks.  This
//     replaces the reference's PersistentDecodeKernel work loop
//     (gqa_decode/gqa_decode.py:865, :902-907) and its host-side sizing (:1408-1410),
//     which recompiles per length and handles one sequence.
//
//   explicit (num_splits == K > 0): every group is cut into K pieces of ceil(tiles/K)
//     tiles, the classic split-K grid of the reference (gqa_decode/gqa_decode.py:273-274,
//     :1104-1105); units (group, piece) are dealt to CTAs in contiguous static runs.
//
// A "segment" is a run of tiles of one group processed by one CTA without interruption;
// it produces one partial (normalised O, log-sum-exp).  Partial slots of a group start at
// first_slot = (first CTA holding a tile of the group, or with stealing the chunk of the
// group's first tile) + group index: both terms grow along the line, so groups get disjoint
// slot ranges with room for one partial per CTA (per chunk).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define GQA_HD __host__ __device__ __forceinline__
#else
#define GQA_HD inline
#endif

namespace gqa {

// Quotient (and remainder) of non-negative line positions.  A 64-bit division is a long
// software routine on the GPU (the better part of a microsecond of dependent instructions,
// and a CTA's set-up performs a dozen before its first load can be issued); nearly every
// operand here fits 32 bits, where the division is a short inline sequence.
GQA_HD long long idiv(long long a, long long b) {
  if ((((unsigned long long)a | (unsigned long long)b) >> 32) == 0)
    return (long long)((unsigned)a / (unsigned)b);
  return a / b;
}
GQA_HD long long imod(long long a, long long b) {
  if ((((unsigned long long)a | (unsigned long long)b) >> 32) == 0)
    return (long long)((unsigned)a % (unsigned)b);
  return a % b;
}

// Division by a divisor known on the host: multiply-shift reciprocal (Granlund-Montgomery),
// exact for every 32-bit numerator.  Three instructions instead of a division routine.
struct FastDiv {
  unsigned mul, s1, s2;
};
GQA_HD unsigned fdiv(unsigned n, const FastDiv& f) {
  const unsigned t = (unsigned)(((unsigned long long)f.mul * n) >> 32);
  return (t + ((n - t) >> f.s1)) >> f.s2;
}
inline FastDiv make_fastdiv(unsigned d) {
  unsigned l = 0;
  while ((1ull << l) < d) ++l;
  FastDiv f;
  f.mul = (unsigned)((((1ull << l) - d) << 32) / d + 1);
  f.s1 = l < 1 ? l : 1;
  f.s2 = l < 1 ? 0 : l - 1;
  return f;
}

enum KvLayout : int {
  kLayoutPadded = 0,  // K/V [batch, Hkv, max_seq, D]: head slab of (b,h) starts at row (b*Hkv+h)*max_seq
  kLayoutPacked = 1,  // K/V [sum_b Hkv*len_b, D]: sequence b holds [Hkv, len_b, D] after all earlier sequences
  kLayoutPagedHnd = 2,  // K/V [num_pages, Hkv, page_size, D] + block table (rows resolved by the producer)
  kLayoutPagedNhd = 3,  // K/V [num_pages, page_size, Hkv, D] + block table
};

struct SchedParams {
  const int32_t* seq_lens;  // [batch] KV length per sequence; null = every sequence has max_seq keys
  int batch;
  int num_kv_heads;
  int max_seq;      // rows per head slab (padded layout) and upper bound of any length
  int tile_rows;    // keys per pipeline stage
  int num_ctas;     // persistent CTAs
  int num_splits;   // 0 = balanced, K > 0 = explicit split-K
  int layout;       // KvLayout
  int chunk_tiles;  // balanced: units per chunk (>= 1)
  int group_overhead;  // balanced: cost units charged per (sequence, KV head) group
  int steal;        // balanced: 1 = idle CTAs steal chunks (results then depend on timing in
                    // the last float32 bits), 0 = static ranges only (bit-reproducible)
  // Uniform lengths (seq_lens == null), balanced static schedule: the geometry is worked out
  // on the host, together with reciprocals of the divisors a CTA's set-up needs, so that the
  // set-up is a few dozen instructions instead of a scan and a dozen divisions.  Every
  // numerator stays below 2^32 (the host checks).  Same schedule as the general path.
  int fast;                   // 1: the fields below are valid
  int fast_parts;             // CTAs that own chunks
  long long fast_total;       // units in the batch
  long long fast_chunks;      // chunks
  FastDiv div_ung, div_hkv, div_chunk, div_chunks, div_parts;  // units per group, KV heads,
                              // units per chunk, chunks, owning CTAs
};

// One run of tiles inside one group, as reported by the host-side replay of the static
// schedule (and used by the explicit split mode on the device).
struct Segment {
  int b, h;                // sequence and KV head
  int len;                 // keys in the sequence
  int row_begin, row_end;  // key range [row_begin, row_end) handled by this segment (may be empty)
  long long kv_row0;       // row of key 0 of this (b,h) slab in the 2-D [rows, D] view of K and V
  int slot;                // partial slot written by this segment (static schedule)
  int first_slot;          // first slot of the group
  int n_parts;             // partials the group is made of in the static schedule
};

struct Walker {
  SchedParams p;
  long long total;     // balanced: units (tiles + group overheads) in the batch; explicit: split units
  long long n_chunks;  // balanced: M
  long long parts;     // balanced: CTAs that own chunks (P)
  // forward scan cursor: first sequence not yet passed, with the sums over earlier ones
  int sb;
  long long s_tiles_before, s_rows_before;
  // unit cursor (balanced)
  int b, h, ui;   // sequence, head, unit inside the group (overhead units first, then tiles)
  int len, ntg;   // length and tile count of sequence b
  int ti;         // tile inside the group (ui - overhead; negative inside the overhead)
  long long tiles_before_group, rows_before_seq;  // tiles_before_group counts units
  // explicit mode cursor
  long long unit;

  GQA_HD int len_of(int bb) const {
    int l = p.max_seq;
    if (p.seq_lens) {
#if defined(__CUDA_ARCH__)
      l = __ldg(p.seq_lens + bb);
#else
      l = p.seq_lens[bb];
#endif
      if (l < 0) l = 0;
      if (p.layout != kLayoutPacked && l > p.max_seq) l = p.max_seq;
    }
    return l;
  }
  GQA_HD int tiles_of(int l) const { return (l + p.tile_rows - 1) / p.tile_rows; }
  // cost units of one group of a sequence with l keys (0 for an empty sequence)
  GQA_HD int units_of(int l) const {
    const int t = tiles_of(l);
    return t ? t + (p.num_splits > 0 ? 0 : p.group_overhead) : 0;
  }
  GQA_HD int overhead() const { return p.num_splits > 0 ? 0 : p.group_overhead; }

  // ---- geometry ---------------------------------------------------------------
  GQA_HD void set_geometry(long long total_items) {
    total = total_items;
    sb = 0;
    s_tiles_before = s_rows_before = 0;
    b = h = ui = ti = len = ntg = 0;
    tiles_before_group = rows_before_seq = 0;
    unit = 0;
    if (p.num_splits > 0) {
      n_chunks = total;
      parts = p.num_ctas;
      return;
    }
    const long long c = p.chunk_tiles > 0 ? p.chunk_tiles : 1;
    n_chunks = idiv(total + c - 1, c);
    parts = n_chunks < p.num_ctas ? n_chunks : p.num_ctas;
  }
  GQA_HD long long chunk_tiles() const { return p.chunk_tiles > 0 ? p.chunk_tiles : 1; }
  // host-prepared geometry (SchedParams::fast)
  GQA_HD void set_geometry_fast() {
    total = p.fast_total;
    n_chunks = p.fast_chunks;
    parts = p.fast_parts;
    sb = 0;
    s_tiles_before = s_rows_before = 0;
    b = h = ui = ti = len = ntg = 0;
    tiles_before_group = rows_before_seq = 0;
    unit = 0;
  }
  // position on unit t0 in closed form (uniform lengths)
  GQA_HD void seat_fast(long long t0) {
    len = p.max_seq;
    ntg = tiles_of(len);
    const int ung = ntg + overhead();
    const unsigned gi = fdiv((unsigned)t0, p.div_ung);
    ui = (int)((unsigned)t0 - gi * (unsigned)ung);
    ti = ui - overhead();
    b = (int)fdiv(gi, p.div_hkv);
    h = (int)(gi - (unsigned)b * (unsigned)p.num_kv_heads);
    tiles_before_group = (long long)gi * ung;
    rows_before_seq = (long long)b * len;
    sb = b;
    s_tiles_before = (long long)b * p.num_kv_heads * ung;
    s_rows_before = rows_before_seq;
  }
  // chunk (balanced) or unit (explicit) range owned by CTA c
  GQA_HD void cta_range(int c, long long& q0, long long& q1) const {
    if (p.num_splits > 0) {
      q0 = idiv(c * total, p.num_ctas);
      q1 = idiv((c + 1) * total, p.num_ctas);
    } else if (c < parts) {
      if (p.fast) {
        q0 = fdiv((unsigned)(c * n_chunks), p.div_parts);
        q1 = fdiv((unsigned)((c + 1) * n_chunks), p.div_parts);
      } else {
        q0 = idiv(c * n_chunks, parts);
        q1 = idiv((c + 1) * n_chunks, parts);
      }
    } else {
      q0 = q1 = 0;
    }
  }
  // owner of chunk q: largest c with floor(c*M/P) <= q (P <= M: every owner has chunks)
  GQA_HD long long cta_of_chunk(long long q) const {
    if (p.fast) return fdiv((unsigned)((q + 1) * parts - 1), p.div_chunks);
    return idiv((q + 1) * parts - 1, n_chunks);
  }
  GQA_HD void chunk_tile_range(long long q, long long& t0, long long& t1) const {
    t0 = q * chunk_tiles();
    t1 = t0 + chunk_tiles();
    if (t1 > total) t1 = total;
  }
  GQA_HD long long group_index() const { return (long long)b * p.num_kv_heads + h; }
  GQA_HD long long kv_row0() const {
    if (p.layout >= kLayoutPagedHnd) return 0;  // paged: rows come from the block table
    return p.layout == kLayoutPadded ? group_index() * (long long)p.max_seq
                                     : rows_before_seq * p.num_kv_heads + (long long)h * len;
  }
  // slot bookkeeping of the current group (balanced)
  // (measured from the group's first tile unit: chunks that only hold its overhead produce
  // no partial)
  GQA_HD long long group_first_tile_unit() const { return tiles_before_group + overhead(); }
  // chunk that holds unit u
  GQA_HD long long chunk_of(long long u) const {
    return p.fast ? (long long)fdiv((unsigned)u, p.div_chunk) : idiv(u, chunk_tiles());
  }
  // Static ranges: a group's partials are numbered from (first CTA that holds a tile of it) +
  // (group index) - both grow along the line and a group has one partial per CTA it spans, so
  // the ranges are disjoint and groups + CTAs slots are enough.  Stealing: any chunk may end
  // up a partial of its own, so the numbering starts from the chunk of the group's first tile.
  GQA_HD int group_first_slot() const {
    const long long q = chunk_of(group_first_tile_unit());
    return (int)((p.steal ? q : cta_of_chunk(q)) + group_index());
  }
  GQA_HD int group_static_parts() const {
    return (int)(cta_of_chunk(chunk_of(group_first_tile_unit() + ntg - 1)) -
                 cta_of_chunk(chunk_of(group_first_tile_unit())) + 1);
  }
  GQA_HD int group_static_index(int cta) const {
    return (int)(cta - cta_of_chunk(chunk_of(group_first_tile_unit())));
  }
  // The three values above in one go (four divisions instead of seven): first slot of the
  // current group, how many partials the static schedule makes of it, and which of them CTA
  // `cta` writes.
  GQA_HD void group_static_slots(int cta, int& first_slot, int& n_parts, int& index) const {
    const long long u0 = group_first_tile_unit();
    const long long q_first = chunk_of(u0), q_last = chunk_of(u0 + ntg - 1);
    const long long c_first = cta_of_chunk(q_first), c_last = cta_of_chunk(q_last);
    first_slot = (int)(c_first + group_index());  // static ranges only, see group_first_slot()
    n_parts = (int)(c_last - c_first + 1);
    index = (int)(cta - c_first);
  }

  // ---- positioning on unit t0 of the line (balanced) ---------------------------------
  GQA_HD void seat(long long t0) {
    b = sb;
    h = ui = len = ntg = 0;
    ti = -overhead();
    tiles_before_group = s_tiles_before;
    rows_before_seq = s_rows_before;
    if (sb >= p.batch) return;
    len = len_of(b);
    ntg = tiles_of(len);
    const int ung = ntg + overhead();
    const long long off = t0 - s_tiles_before;
    h = (int)idiv(off, ung);
    ui = (int)(off - (long long)h * ung);
    ti = ui - overhead();
    tiles_before_group = s_tiles_before + (long long)h * ung;
  }
  GQA_HD void rewind_if_behind(long long t0) {
    if (t0 < s_tiles_before) {
      sb = 0;
      s_tiles_before = s_rows_before = 0;
    }
  }
  // advance the cursor by one unit; returns false when the line is exhausted
  GQA_HD bool advance() {
    ++ti;
    if (++ui < ntg + overhead()) return true;
    tiles_before_group += ntg + overhead();
    ui = 0;
    ti = -overhead();
    if (++h < p.num_kv_heads) return true;
    h = 0;
    rows_before_seq += len;
    ++b;
    len = ntg = 0;
    while (b < p.batch) {
      len = len_of(b);
      ntg = tiles_of(len);
      if (ntg) return true;
      ++b;
    }
    return false;
  }

  // Serial versions: usable from host code or from a single device thread.
  GQA_HD void init_serial(const SchedParams& sp) {
    p = sp;
    if (p.fast) {
      set_geometry_fast();
      return;
    }
    if (p.num_splits > 0) {
      set_geometry((long long)p.batch * p.num_kv_heads * p.num_splits);
      return;
    }
    long long n = 0;
    for (int bb = 0; bb < p.batch; ++bb) n += units_of(len_of(bb));
    set_geometry(n * p.num_kv_heads);
  }
  GQA_HD void seek_serial(long long t0) {
    if (p.fast) {
      seat_fast(t0);
      return;
    }
    rewind_if_behind(t0);
    for (; sb < p.batch; ++sb) {
      const int l = len_of(sb);
      const long long nt = (long long)units_of(l) * p.num_kv_heads;
      if (s_tiles_before + nt > t0) break;
      s_tiles_before += nt;
      s_rows_before += l;
    }
    seat(t0);
  }
  // explicit mode: position on unit u (units are visited in increasing order)
  GQA_HD void seek_unit_serial(long long u) {
    unit = u;
    const int nb = (int)idiv(idiv(u, p.num_splits), p.num_kv_heads);
    for (; sb < nb && sb < p.batch; ++sb) s_rows_before += len_of(sb);
    b = sb;
    rows_before_seq = s_rows_before;
  }

#if defined(__CUDACC__)
  // Warp-cooperative versions: all 32 lanes of a warp call them together and end with
  // identical state.  Lengths are read 32 at a time and combined with shuffles.
  __device__ __forceinline__ void init_warp(const SchedParams& sp) {
    p = sp;
    if (p.fast) {
      set_geometry_fast();
      return;
    }
    if (p.num_splits > 0) {
      set_geometry((long long)p.batch * p.num_kv_heads * p.num_splits);
      return;
    }
    const int lane = threadIdx.x & 31;
    long long n = 0;
    for (int bb = lane; bb < p.batch; bb += 32) n += units_of(len_of(bb));
    for (int o = 16; o; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    set_geometry(n * p.num_kv_heads);
  }
  __device__ __forceinline__ void seek_warp(long long t0) {
    if (p.fast) {
      seat_fast(t0);
      return;
    }
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    rewind_if_behind(t0);
    while (sb < p.batch) {
      const int bb = sb + lane;
      const int l = bb < p.batch ? len_of(bb) : 0;
      const long long nt = (long long)units_of(l) * p.num_kv_heads;
      long long it = nt, ir = l;  // inclusive scans over the 32 lanes
      for (int o = 1; o < 32; o <<= 1) {
        const long long a = __shfl_up_sync(full, it, o);
        const long long c = __shfl_up_sync(full, ir, o);
        if (lane >= o) {
          it += a;
          ir += c;
        }
      }
      const unsigned hit = __ballot_sync(full, bb < p.batch && s_tiles_before + it > t0);
      if (hit) {
        const int first = __ffs(hit) - 1;
        s_tiles_before += __shfl_sync(full, it - nt, first);
        s_rows_before += __shfl_sync(full, ir - l, first);
        sb += first;
        break;
      }
      s_tiles_before += __shfl_sync(full, it, 31);
      s_rows_before += __shfl_sync(full, ir, 31);
      sb += 32;
    }
    if (sb > p.batch) sb = p.batch;
    seat(t0);
  }
  __device__ __forceinline__ void seek_unit_warp(long long u) {
    const int lane = threadIdx.x & 31;
    unit = u;
    const int nb = (int)idiv(idiv(u, p.num_splits), p.num_kv_heads);
    long long r = 0;
    for (int bb = sb + lane; bb < nb && bb < p.batch; bb += 32) r += len_of(bb);
    for (int o = 16; o; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    s_rows_before += r;
    if (nb > sb) sb = nb < p.batch ? nb : p.batch;
    b = sb;
    rows_before_seq = s_rows_before;
  }
#endif

  // explicit mode: describe unit `unit` and move to the next one
  GQA_HD void next_unit(Segment& s) {
    const int T = p.tile_rows, K = p.num_splits;
    const long long g = idiv(unit, K);
    const int sp = (int)(unit - g * K);
    const int nb = (int)idiv(g, p.num_kv_heads);
    while (b < nb) {
      rows_before_seq += len_of(b);
      ++b;
    }
    h = (int)(g - (long long)nb * p.num_kv_heads);
    len = len_of(b);
    ntg = tiles_of(len);
    const int cs = (ntg + K - 1) / K;
    long long tb = (long long)sp * cs;
    if (tb > ntg) tb = ntg;
    long long te = tb + cs;
    if (te > ntg) te = ntg;
    s.b = b;
    s.h = h;
    s.len = len;
    const long long re = te * T;
    s.row_begin = tb == te ? 0 : (int)(tb * T);  // an empty piece is reported as [0, 0)
    s.row_end = tb == te ? 0 : (int)(re < len ? re : len);
    s.slot = (int)unit;
    s.first_slot = (int)(g * K);
    s.n_parts = K;
    s.kv_row0 = kv_row0();
    ++unit;
  }

  // Static schedule of CTA `cta` (no stealing), for inspection and tests.  Call
  // static_range() for the tile / unit range, seek to its start (serial or warp
  // version), then walk_static() fills `out` with up to `cap` segments and returns how
  // many the CTA has.
  GQA_HD bool static_range(int cta, long long& t0, long long& t1) const {
    long long q0, q1;
    cta_range(cta, q0, q1);
    if (q0 >= q1) return false;
    if (p.num_splits > 0) {
      t0 = q0;
      t1 = q1;
    } else {
      long long tmp;
      chunk_tile_range(q0, t0, tmp);
      chunk_tile_range(q1 - 1, tmp, t1);
    }
    return true;
  }
  GQA_HD long long walk_static(int cta, long long t0, long long t1, Segment* out, long long cap) {
    long long n = 0;
    if (p.num_splits > 0) {
      for (long long u = t0; u < t1; ++u, ++n) {
        Segment s;
        next_unit(s);
        if (n < cap) out[n] = s;
      }
      return n;
    }
    long long t = t0;
    while (t < t1) {
      if (ti < 0) {  // inside the group's overhead: no tile, nothing to report
        ++t;
        if (!advance()) break;
        continue;
      }
      long long take = ntg - ti;
      if (take > t1 - t) take = t1 - t;
      Segment s;
      s.b = b;
      s.h = h;
      s.len = len;
      s.row_begin = ti * p.tile_rows;
      const long long re = (long long)(ti + take) * p.tile_rows;
      s.row_end = (int)(re < len ? re : len);
      s.kv_row0 = kv_row0();
      s.first_slot = group_first_slot();
      s.n_parts = group_static_parts();
      s.slot = s.first_slot + group_static_index(cta);
      if (n < cap) out[n] = s;
      ++n;
      t += take;
      ui += (int)take - 1;
      ti += (int)take - 1;
      if (!advance()) break;
    }
    return n;
  }
};

// Host side: fill in SchedParams::fast and what goes with it where the closed-form set-up
// applies (uniform lengths, balanced static schedule, every numerator below 2^32).
inline void prepare_fast_schedule(SchedParams& sp) {
  sp.fast = 0;
  if (sp.seq_lens || sp.num_splits > 0 || sp.steal || sp.batch <= 0 || sp.num_kv_heads <= 0 ||
      sp.max_seq <= 0 || sp.tile_rows <= 0 || sp.num_ctas <= 0)
    return;
  const long long tiles = ((long long)sp.max_seq + sp.tile_rows - 1) / sp.tile_rows;
  const long long ung = tiles + sp.group_overhead;
  const long long total = (long long)sp.batch * sp.num_kv_heads * ung;
  const long long chunk = sp.chunk_tiles > 0 ? sp.chunk_tiles : 1;
  if (total * ((long long)sp.num_ctas + 1) >= (1ll << 31)) return;
  const long long chunks = (total + chunk - 1) / chunk;
  sp.fast = 1;
  sp.fast_total = total;
  sp.fast_chunks = chunks;
  sp.fast_parts = (int)(chunks < sp.num_ctas ? chunks : sp.num_ctas);
  sp.div_ung = make_fastdiv((unsigned)ung);
  sp.div_hkv = make_fastdiv((unsigned)sp.num_kv_heads);
  sp.div_chunk = make_fastdiv((unsigned)chunk);
  sp.div_chunks = make_fastdiv((unsigned)chunks);
  sp.div_parts = make_fastdiv((unsigned)sp.fast_parts);
}

// Upper bound on partial slots for a launch with chunk size `chunk_tiles`:
// one slot per chunk plus one per group.
GQA_HD long long max_slots(long long groups, int num_splits, long long max_units_per_group,
                           int chunk_tiles) {
  if (num_splits > 0) return groups * num_splits;
  const long long tiles = groups * max_units_per_group;
  return (tiles + chunk_tiles - 1) / chunk_tiles + groups + 1;
}

// Chunk size (tiles) for the balanced schedule: small enough that stealing evens out the
// tail (about 48 chunks per CTA, 4 to 16 tiles each), never more chunks than `slot_budget` allows.
GQA_HD int choose_chunk_tiles(long long groups, long long max_units_per_group, int num_ctas,
                              long long slot_budget) {
  const long long tiles = groups * max_units_per_group;
  // at least 4 tiles (about 3 us of streaming on one SM) so that the atomic that hands out
  // a chunk stays off the critical path
  long long c = tiles / ((long long)num_ctas * 48);
  if (c < 4) c = 4;
  if (c > 16) c = 16;
  const long long room = slot_budget - groups - 1;
  if (room > 0) {
    const long long need = (tiles + room - 1) / room;  // smallest chunk that fits the budget
    if (c < need) c = need;
  }
  return (int)c;
}

}  // namespace gqa
