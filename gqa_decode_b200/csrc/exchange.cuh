// Cross-GPU exchange + merge of sequence-shard partials over NVLink, in one kernel.
//
// Every rank owns a receive buffer that all ranks can address (symmetric memory: the
// same allocation made on every GPU and mapped into every process).  Layout, in floats,
// after a header of 2 * world 32-bit flags (padded to 256 bytes):
//     [parity 0 | parity 1] x [source rank 0 .. world-1] x [rows * D outputs, rows LSEs]
// One launch with epoch e (odd/even selects the parity half):
//   CTA p pushes this rank's partial into peer p's buffer (slot = this rank) with plain
//   peer stores, fences, and sets peer p's flag[parity][this rank] = e (release, system
//   scope).  Then every CTA waits - bounded by wall-clock time - until all `world` flags of
//   this rank carry e (acquire, system scope) and merges its share of the rows from the
//   partials now sitting in local memory.  No multicast, no NVLS: plain loads and stores.
//
// Two parity halves make reuse safe without another barrier: a rank can start exchange
// e+1 (writing the other half) while a slower peer still merges exchange e, and nobody can
// reach e+2 before every peer has finished e, because e+1 needs every peer's e+1 push.
//
// The merge is the same LSE-weighted sum as merge_rows_kernel / the reference's
// reduce_partials (gqa_decode/gqa_decode.py:661-669).
#pragma once
#include "decode_kernel.cuh"

namespace gqa {

struct ExchangeParams {
  const float* local_o;    // [rows, D] this rank's normalised partial output
  const float* local_lse;  // [rows]
  void* const* peer_bufs;  // device array [world]: receive buffer of every rank, as mapped here
  int rank, world;
  unsigned epoch;          // > 0, incremented by the caller on every exchange
  long long rows;
  int D;
  void* out;               // [rows, D] bf16/fp16 or null
  int out_fp16;
  float* out_f32;          // optional
  float* out_lse;          // optional
  int* status;             // optional device word: |= kStatusWaitExchange on expiry
  unsigned long long wait_limit_ns;  // bound on the wait for the peers' flags
};
constexpr int kExchangeThreads = 256;

__host__ __device__ inline size_t exchange_header_bytes(int world) {
  return ((size_t)2 * world * sizeof(unsigned) + 255) & ~(size_t)255;
}
__host__ __device__ inline size_t exchange_slot_floats(long long rows, int D) {
  return (size_t)rows * (D + 1);
}
__host__ __device__ inline size_t exchange_buffer_bytes(int world, long long rows, int D) {
  return exchange_header_bytes(world) + 2 * (size_t)world * exchange_slot_floats(rows, D) * sizeof(float);
}

template <typename Q>
__global__ void __launch_bounds__(kExchangeThreads)
exchange_merge_kernel(const ExchangeParams p) {
  const int tid = threadIdx.x;
  const int peer = blockIdx.x;  // grid = world
  const int parity = p.epoch & 1u;
  const int D4 = p.D / 4;
  const size_t slot = exchange_slot_floats(p.rows, p.D);
  const size_t hdr = exchange_header_bytes(p.world);
  __shared__ int timed_out;
  if (tid == 0) timed_out = 0;

  // ---- 1. push this rank's partial into peer `peer`
  {
    char* base = static_cast<char*>(p.peer_bufs[peer]);
    float* dst = reinterpret_cast<float*>(base + hdr) + ((size_t)parity * p.world + p.rank) * slot;
    if (peer != p.rank) {
      float4* dst4 = reinterpret_cast<float4*>(dst);
      const float4* src4 = reinterpret_cast<const float4*>(p.local_o);
      for (long long i = tid; i < p.rows * D4; i += kExchangeThreads) dst4[i] = src4[i];
      float* dl = dst + (size_t)p.rows * p.D;
      for (long long i = tid; i < p.rows; i += kExchangeThreads) dl[i] = p.local_lse[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0)
      st_release_sys(reinterpret_cast<unsigned*>(base) + parity * p.world + p.rank, p.epoch);
  }

  // ---- 2. wait (bounded) until every rank's partial has landed here
  {
    const unsigned* flags =
        reinterpret_cast<const unsigned*>(p.peer_bufs[p.rank]) + parity * p.world;
    if (tid < p.world) {
      const unsigned long long t0 = global_timer_ns();
      while (ld_acquire_sys(flags + tid) != p.epoch) {
        if (global_timer_ns() - t0 > p.wait_limit_ns) {
          timed_out = 1;
          break;
        }
        __nanosleep(100);
      }
    }
    __syncthreads();
    if (timed_out) {
      if (tid == 0 && p.status) atomicOr(p.status, kStatusWaitExchange);
      return;
    }
  }

  // ---- 3. merge this CTA's share of the rows
  const float* mine = reinterpret_cast<const float*>(static_cast<const char*>(p.peer_bufs[p.rank]) + hdr) +
                      (size_t)parity * p.world * slot;
  const long long r_begin = p.rows * peer / p.world, r_end = p.rows * (peer + 1) / p.world;
  for (long long idx = r_begin * D4 + tid; idx < r_end * D4; idx += kExchangeThreads) {
    const long long row = idx / D4;
    const int d4 = (int)(idx % D4);
    float mx = -INFINITY;
    for (int s = 0; s < p.world; ++s) {
      const float l = s == p.rank ? p.local_lse[row] : __ldcg(mine + s * slot + (size_t)p.rows * p.D + row);
      mx = fmaxf(mx, l);
    }
    const float ms = (mx == -INFINITY) ? 0.f : mx;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int s = 0; s < p.world; ++s) {
      float l;
      float4 o;
      if (s == p.rank) {
        l = p.local_lse[row];
        o = reinterpret_cast<const float4*>(p.local_o + row * p.D)[d4];
      } else {
        l = __ldcg(mine + s * slot + (size_t)p.rows * p.D + row);
        o = __ldcg(reinterpret_cast<const float4*>(mine + s * slot + row * p.D) + d4);
      }
      const float w = fast_exp2((l - ms) * kLog2e);
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
    if (p.out) {
      uint2 pk;
      pk.x = Mma16<Q>::pack(acc.x, acc.y);
      pk.y = Mma16<Q>::pack(acc.z, acc.w);
      *reinterpret_cast<uint2*>(static_cast<Q*>(p.out) + row * p.D + 4 * d4) = pk;
    }
    if (p.out_f32) reinterpret_cast<float4*>(p.out_f32 + row * p.D)[d4] = acc;
    if (p.out_lse && d4 == 0) p.out_lse[row] = wsum > 0.f ? ms + fast_log2(wsum) * kLn2 : -INFINITY;
  }
}

}  // namespace gqa
