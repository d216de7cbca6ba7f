// FP8-E4M3 K/V consumer for the persistent decode kernel.
//
// K and V tiles arrive as raw bytes ([TILE rows x 128 B], 128-byte swizzle).  Each
// thread pulls the bytes its MMA fragments need with plain shared loads and
// dequantises them in registers.  K always follows the reference's oracle exactly
// (gqa_decode/fp8_utils.py:54-55): float32(code) * scale[head] rounded to nearest in
// fp32, then rounded to nearest-even to the 16-bit MMA type.  The K scale is NOT
// folded into the score: the oracle's bf16 rounding of each dequantised element is
// part of the answer, and dropping it moves peaked softmax rows outside tolerance.
// V follows the same rule when EXACT_V is set; by default its scale is applied once to
// the accumulated output instead (see consume_block_fp8).
// Replaces FP8DirectDecodeKernel / FP8SplitKDecodeKernel
// (gqa_decode/gqa_decode.py:1454-1596, :1599-1803; dequant at :1565-1566, :1752-1753).
//
// Because the contraction index of an MMA may be permuted freely as long as A and B
// agree, the d axis is permuted so that a thread's 16-byte shared load feeds four
// k-steps of Q K^T (the Q fragments use the same permutation).  V is fetched with the
// byte-transposing ldmatrix (ldmatrix ... .m16n16 ... .trans ... .b8), which delivers four
// keys of one column per register, ready for two conversions into an MMA B fragment.
#pragma once
#include <type_traits>

#include "decode_kernel.cuh"

namespace gqa {

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// Four E4M3 codes in one 32-bit word (lowest byte first) -> two registers of two
// dequantised, rounded 16-bit values each (b0 = codes 0,1; b1 = codes 2,3).  Written as one
// PTX block on 16-bit sub-registers so that no separate shift / mask instructions are
// needed to split words and half2 pairs; the multiply is one packed fp32x2 operation
// (round-to-nearest per lane, the same result as two fmul.rn).
__device__ __forceinline__ void codes_word_to_f16x2_fwd(uint32_t w, uint32_t& h0, uint32_t& h1) {
  asm("{\n\t"
      ".reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t"
      "}"
      : "=r"(h0), "=r"(h1)
      : "r"(w));
}
template <typename T16>
__device__ __forceinline__ void dequant_word(uint32_t w, float scale, uint32_t& b0, uint32_t& b1) {
  float f0, f1, f2, f3;
  asm("{\n\t"
      ".reg .b16 lo, hi, a, b, c, d;\n\t"
      ".reg .b32 h0, h1;\n\t"
      "mov.b32 {lo, hi}, %4;\n\t"
      "cvt.rn.f16x2.e4m3x2 h0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 h1, hi;\n\t"
      "mov.b32 {a, b}, h0;\n\t"
      "mov.b32 {c, d}, h1;\n\t"
      "cvt.f32.f16 %0, a;\n\t"
      "cvt.f32.f16 %1, b;\n\t"
      "cvt.f32.f16 %2, c;\n\t"
      "cvt.f32.f16 %3, d;\n\t"
      "}"
      : "=f"(f0), "=f"(f1), "=f"(f2), "=f"(f3)
      : "r"(w));
  unsigned long long in0, in1, sc, p0, p1;
  asm("mov.b64 %0, {%1, %2};" : "=l"(in0) : "f"(f0), "f"(f1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(in1) : "f"(f2), "f"(f3));
  asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(scale));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p0) : "l"(in0), "l"(sc));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(p1) : "l"(in1), "l"(sc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(f0), "=f"(f1) : "l"(p0));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(f2), "=f"(f3) : "l"(p1));
  b0 = Mma16<T16>::pack(f0, f1);
  b1 = Mma16<T16>::pack(f2, f3);
}

// N words at once, written stage by stage (all first conversions, then all widenings, all
// multiplies, all roundings): long runs of independent instructions keep the slow
// conversion pipe fed instead of leaving each word's five-deep dependency chain exposed.
template <typename T16, int N>
__device__ __forceinline__ void dequant_words(const uint32_t (&w)[N], float scale,
                                              uint32_t (&b)[2 * N]) {
  uint32_t h[2 * N];
#pragma unroll
  for (int j = 0; j < N; ++j) codes_word_to_f16x2_fwd(w[j], h[2 * j], h[2 * j + 1]);
  float f[4 * N];
#pragma unroll
  for (int j = 0; j < 2 * N; ++j)
    asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.f32.f16 %0, a;\n\tcvt.f32.f16 %1, b;\n\t}"
        : "=f"(f[2 * j]), "=f"(f[2 * j + 1])
        : "r"(h[j]));
  unsigned long long sc;
  asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(scale));
#pragma unroll
  for (int j = 0; j < 2 * N; ++j) {
    unsigned long long in, pr;
    asm("mov.b64 %0, {%1, %2};" : "=l"(in) : "f"(f[2 * j]), "f"(f[2 * j + 1]));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(pr) : "l"(in), "l"(sc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(f[2 * j]), "=f"(f[2 * j + 1]) : "l"(pr));
  }
#pragma unroll
  for (int j = 0; j < 2 * N; ++j) b[j] = Mma16<T16>::pack(f[2 * j], f[2 * j + 1]);
}

// Four E4M3 codes in one word -> two f16x2 registers holding the codes' exact values.
__device__ __forceinline__ void codes_word_to_f16x2(uint32_t w, uint32_t& h0, uint32_t& h1) {
  asm("{\n\t"
      ".reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t"
      "}"
      : "=r"(h0), "=r"(h1)
      : "r"(w));
}

// EXACT_V = true : V is dequantised like K (oracle rounding) and P V runs in the query type.
// EXACT_V = false: V codes are widened to f16 (exact) and P V runs as an f16 MMA on the
//   unscaled codes; the per-head V scale multiplies the fp32 output once at the end.  This
//   skips the oracle's bf16 rounding of each dequantised V element (a relative 2^-9
//   perturbation averaged over the softmax weights, well inside the tolerance) and
//   removes three quarters of the conversion work.
template <typename T16, int TILE, bool UPPER, bool PARTIAL, bool EXACT_V, int NB>
__device__ __forceinline__ void consume_block_fp8(uint32_t k_base, uint32_t v_base, int key0,
                                                  int valid, const uint32_t (&qa)[8][4],
                                                  WarpState<128, UPPER>& st, float scale_log2,
                                                  int lane, float k_scale, float v_scale) {
  constexpr int D = 128;
  using TP = typename std::conditional<EXACT_V, T16, __half>::type;  // type of P and of the PV MMA
  const int n = lane >> 2, c = lane & 3;
  // NB blocks of 16 keys are processed together: their 2*NB score tiles are independent
  // MMA chains, which gives the scheduler conversion work to overlap with MMA latency.
  float s[2 * NB][4];
#pragma unroll
  for (int t = 0; t < 2 * NB; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
  // K: two score tiles (eight words) are dequantised per batch, stage by stage.
  constexpr int kBatch = 2;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int t0 = 0; t0 < 2 * NB; t0 += kBatch) {
      uint32_t ww[4 * kBatch], bb[8 * kBatch];
#pragma unroll
      for (int t = 0; t < kBatch; ++t) {
        const int key = key0 + 8 * (t0 + t) + n;
        const uint4 w = lds128(k_base + key * 128 + (((2 * c + i) ^ (key & 7)) << 4));
        ww[4 * t] = w.x, ww[4 * t + 1] = w.y, ww[4 * t + 2] = w.z, ww[4 * t + 3] = w.w;
      }
      dequant_words<T16, 4 * kBatch>(ww, k_scale, bb);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int ks = 4 * i + u;
#pragma unroll
        for (int t = 0; t < kBatch; ++t)
          Mma16<T16>::run(s[t0 + t], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], bb[8 * t + 2 * u],
                          bb[8 * t + 2 * u + 1]);
      }
    }
  }
  uint32_t pa[NB][4];
  softmax_block<TP, D, UPPER, PARTIAL, NB>(s, st, pa, scale_log2, key0, valid, lane);
  // O += P V.  V fragments come from the byte-transposing ldmatrix: the 16 row addresses of
  // a matrix are given in the order 0,1,8,9, 2,3,10,11, ... so that the four rows a thread
  // receives in one register (matrix rows 4c..4c+3) are keys 2c, 2c+1, 2c+8, 2c+9 - exactly
  // the k indices of its B fragment.  Register u of a load covers output columns
  // 32q + 8u + n: accumulator tile 4q + u, natural column order.
  const int mr = lane & 15;
  const int vkey = 2 * (mr >> 2) + (mr & 1) + 8 * ((mr >> 1) & 1);  // key of this lane's matrix row
  uint32_t live = 0xffffffffu;  // byte mask of the keys that exist (PARTIAL tiles)
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    if (PARTIAL) {
      const int k0 = key0 + 16 * b + 2 * c;
      live = (k0 < valid ? 0x000000ffu : 0u) | (k0 + 1 < valid ? 0x0000ff00u : 0u) |
             (k0 + 8 < valid ? 0x00ff0000u : 0u) | (k0 + 9 < valid ? 0xff000000u : 0u);
    }
    const int kk = key0 + 16 * b + vkey;
    const uint32_t row_addr = v_base + kk * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t w[4];
      ldsm8_x2_trans(w, row_addr + (((2 * q + (lane >> 4)) ^ (kk & 7)) << 4));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t b0, b1;
        const uint32_t codes = PARTIAL ? (w[u] & live) : w[u];
        if (EXACT_V) dequant_word<T16>(codes, v_scale, b0, b1);
        else codes_word_to_f16x2(codes, b0, b1);
        Mma16<TP>::run(st.o[4 * q + u], pa[b][0], pa[b][1], pa[b][2], pa[b][3], b0, b1);
      }
    }
  }
}

template <typename T16_, int TILE_, bool UPPER_, bool EXACT_V_ = false, int WARPS_ = 8>
struct KvFp8Traits {
  using Q = T16_;
  static constexpr int D = 128;
  static constexpr int TILE = TILE_;
  static constexpr bool UPPER = UPPER_;
  static constexpr int kWarps = WARPS_;  // consumer warps: two per SM sub-partition; with 256-key
                                         // tiles each owns 32 keys (two independent 16-key blocks)
  static constexpr int kGroups = 1;
  // Merge rows are unpadded (every byte counts: three 64 KB stages plus these rows just fit
  // into shared memory); an XOR of the 8-float column group with the row keeps the float2
  // stores of different rows on different banks.
  static constexpr int kMoStride = 128;
  __device__ static __forceinline__ int mo_index(int row, int col) {
    return row * kMoStride + (col ^ ((row & 7) << 3));
  }
  static constexpr int kMergeBatch = 8;      // partials merged per L2 round trip
  static constexpr bool kFp8 = true;
  static constexpr int kBoxesPerTensor = 1;
  static constexpr int kBoxRows = TILE_;  // small pages keep per-page 2-D boxes (rows are one piece)
  static constexpr int kBoxBytes = TILE * 128;
  static constexpr int kStageBytes = 2 * kBoxBytes;
  static constexpr int kTxBytes = kStageBytes;
  static constexpr int kPieceBytes = 128;
  static constexpr int kBoxCols = 128;
  struct Extra {
    float ks, vs;
  };
  __device__ static __forceinline__ void begin_segment(Extra& e, const DecodeParams& prm, int b,
                                                       int h) {
    const long long g = (long long)b * prm.sched.num_kv_heads + h;
    e.ks = __ldg(prm.k_scale + g);
    e.vs = __ldg(prm.v_scale + g);
  }
  template <bool PARTIAL, int NB>
  __device__ static __forceinline__ void consume(uint32_t k_base, uint32_t v_base, int key0,
                                                 int valid, const uint32_t (&qa)[8][4],
                                                 WarpState<128, UPPER>& st, float scale_log2,
                                                 int lane, const Extra& e) {
    consume_block_fp8<Q, TILE, UPPER, PARTIAL, EXACT_V_, NB>(k_base, v_base, key0, valid, qa, st,
                                                             scale_log2, lane, e.ks, e.vs);
  }
  // scale applied to the fp32 output when V was accumulated unscaled
  __device__ static __forceinline__ float out_scale(const Extra& e) { return EXACT_V_ ? 1.f : e.vs; }
  // k-step ks of thread column c covers d = 32c + 16(ks/4) + 4(ks%4) + {0,1 | 2,3}.
  __device__ static __forceinline__ void load_q(uint32_t (&qa)[8][4], const Q* row0, const Q* row1,
                                                bool v0, bool v1, int c) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d = 32 * c + 16 * (ks >> 2) + 4 * (ks & 3);
      qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(row0 + d) : 0u;
      qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(row0 + d + 2) : 0u;
      qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(row1 + d) : 0u;
      qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(row1 + d + 2) : 0u;
    }
  }
  // d index of accumulator element (n-tile nt, thread column c, element e).
  __device__ static __forceinline__ int out_col(int nt, int c, int e) { return 8 * nt + 2 * c + e; }
};

// ---------------------------------------------------------------------------
// E4M3 K/V with head_dim 64 (accepted by the reference's FP8 kernels,
// gqa_decode/gqa_decode.py:1466-1467).  Rows are 64 bytes, so the permuted fragment loads
// above do not apply; instead each consumer warp dequantises the 16 keys of a block exactly
// like dequantize_kv_fp8 (gqa_decode/fp8_utils.py:54-55: float32(code) * scale, rounded to the
// 16-bit type - K and V alike) into a scratch of its own behind the stage's raw bytes, laid out
// as the 128-byte-swizzled rows the 16-bit consumer reads, and then runs that consumer on it.
// Tiles of 256 keys: [256 x 64 B] for K and for V, unswizzled; eight consumer warps.
// ---------------------------------------------------------------------------
template <typename T16_, bool UPPER_, int TILE_ = 256, int WARPS_ = 8>
struct KvFp8Dim64Traits {
  using Q = T16_;
  static constexpr int D = 64;
  static constexpr int TILE = TILE_;
  static constexpr bool UPPER = UPPER_;
  static constexpr int kWarps = WARPS_;  // 32 keys (two blocks) per warp and tile
  static constexpr int kGroups = 1;
  static constexpr bool kFp8 = true;
  static constexpr int kBoxesPerTensor = 1;
  static constexpr int kBoxRows = TILE;
  static constexpr int kPieceBytes = 64;                 // bytes of one box row
  static constexpr int kBoxBytes = TILE * kPieceBytes;   // raw K (or V) bytes of a tile
  static constexpr int kTxBytes = 2 * kBoxBytes;
  static constexpr int kScratchBytes = 2 * 16 * 128;     // per warp: 16 keys of K, 16 of V, 16-bit
  static constexpr int kStageBytes = kTxBytes + kWarps * kScratchBytes;
  static constexpr int kBoxCols = 64;
  static constexpr int kMoStride = D + 8;
  __device__ static __forceinline__ int mo_index(int row, int col) { return row * kMoStride + col; }
  static constexpr int kMergeBatch = 8;
  struct Extra {
    float ks, vs;
  };
  __device__ static __forceinline__ void begin_segment(Extra& e, const DecodeParams& prm, int b,
                                                       int h) {
    const long long g = (long long)b * prm.sched.num_kv_heads + h;
    e.ks = __ldg(prm.k_scale + g);
    e.vs = __ldg(prm.v_scale + g);
  }
  __device__ static __forceinline__ float out_scale(const Extra&) { return 1.f; }
  // 16 rows of 64 codes at `src` (rows 64 bytes apart) -> 16 rows of 64 16-bit values at
  // `dst` (rows 128 bytes apart, 16-byte chunk c of row r at chunk position c ^ (r & 7)).
  // Lane l converts the 32 bytes of half (l & 1) of row (l >> 1).
  __device__ static __forceinline__ void dequant_rows(uint32_t src, uint32_t dst, float scale, int lane) {
    const int r = lane >> 1, h = lane & 1;
    const uint4 a = lds128(src + lane * 32), b = lds128(src + lane * 32 + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t o[16];
    dequant_words<Q, 8>(w, scale, o);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t at = dst + r * 128 + (((4 * h + c) ^ (r & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(at), "r"(o[4 * c]), "r"(o[4 * c + 1]),
                   "r"(o[4 * c + 2]), "r"(o[4 * c + 3])
                   : "memory");
    }
  }
  template <bool PARTIAL, int NB>
  __device__ static __forceinline__ void consume(uint32_t k_base, uint32_t v_base, int key0,
                                                 int valid, const uint32_t (&qa)[D / 16][4],
                                                 WarpState<D, UPPER>& st, float scale_log2,
                                                 int lane, const Extra& e) {
    // this warp's scratch sits behind the raw bytes of the stage; warp = key0 / (16 * NB)
    const uint32_t scratch = k_base + kTxBytes + (uint32_t)(key0 / (16 * NB)) * kScratchBytes;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const int k0 = key0 + 16 * b;
      if (PARTIAL && k0 >= valid) break;
      __syncwarp();  // the previous block's fragment loads are done with the scratch
      dequant_rows(k_base + k0 * kPieceBytes, scratch, e.ks, lane);
      dequant_rows(v_base + k0 * kPieceBytes, scratch + 16 * 128, e.vs, lane);
      __syncwarp();
      // the 16-bit consumer addresses rows as key * 128 from its base: rebase to the scratch
      consume_block_16<Q, D, TILE, UPPER, PARTIAL>(scratch - k0 * 128, scratch + 16 * 128 - k0 * 128, k0,
                                                   valid, qa, st, scale_log2, lane);
    }
  }
  __device__ static __forceinline__ void load_q(uint32_t (&qa)[D / 16][4], const Q* row0,
                                                const Q* row1, bool v0, bool v1, int c) {
    Kv16Traits<Q, D, TILE, UPPER>::load_q(qa, row0, row1, v0, v1, c);
  }
  __device__ static __forceinline__ int out_col(int nt, int c, int e) { return 8 * nt + 2 * c + e; }
};

}  // namespace gqa
