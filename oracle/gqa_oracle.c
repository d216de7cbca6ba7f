/*
 * C restatement of the reference's decode attention for large inputs.
 *
 * TEST INFRASTRUCTURE ONLY: loaded by tests/ (through oracle/c_oracle.py) to check the
 * CUDA path at the full benchmark sizes, where the PyTorch restatement
 * (oracle/gqa_oracle.py) would need tens of GB for its per-query-head gathers.  The
 * shipped library never links or loads this file.
 *
 * Parity status: pinned indirectly - tests/test_oracle_golden.py requires this code to
 * agree with the golden vectors produced by the reference implementation (within the
 * float32 rounding of the reference itself; accumulation here is float64).
 *
 * Algorithm followed: reference_gqa_decode, gqa_decode/gqa_decode.py:36-66
 *   kv head of query head h is h / (Hq / Hkv)                         (:58-59)
 *   score = (q . k) * D^-0.5                                           (:60-62)
 *   weights = softmax(score) over keys, out = weights . V              (:63-65)
 * and dequantize_kv_fp8, gqa_decode/fp8_utils.py:54-55
 *   value = bf16_round(float32(code) * scale[head]).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (m == 0) u = s;
    else {
      int sh = 0;
      while (!(m & 1024)) { m <<= 1; ++sh; }
      u = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023) << 13);
    }
  } else if (e == 31) u = s | 0x7f800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}
/* E4M3 (fn variant: no infinities, 0x7f/0xff are NaN), exact in float32 */
static inline float e4m3_to_f32(uint8_t c) {
  int s = c >> 7, e = (c >> 3) & 15, m = c & 7;
  float v;
  if (e == 15 && m == 7) v = NAN;
  else if (e == 0) v = ldexpf((float)m, -9);
  else v = ldexpf((float)(8 + m), e - 10);
  return s ? -v : v;
}

/* kv_kind: 0 = bf16 bits, 1 = fp16 bits, 2 = e4m3 codes with per-head scales (dequantised
 * with the reference's bf16 rounding).  q_kind: 0 bf16, 1 fp16.  K/V are [Hkv, S, D];
 * `head_stride` is the element distance between consecutive KV heads (S*D when
 * contiguous).  Writes out[Hq*D] (float64, not rounded) and lse[Hq] (natural log).
 * Query heads are spread over `threads` POSIX threads. */
typedef struct {
  const void *q, *k, *v;
  const float *k_scale, *v_scale;
  int q_kind, kv_kind, Hq, Hkv, D, h0, h1;
  long S, head_stride;
  double *out, *lse;
  int rc;
} job_t;

static inline double load_kv(const void* p, long i, int kind, float scale) {
  if (kind == 2) return bf16_to_f32(f32_to_bf16_rne(e4m3_to_f32(((const uint8_t*)p)[i]) * scale));
  uint16_t b = ((const uint16_t*)p)[i];
  return kind ? f16_to_f32(b) : bf16_to_f32(b);
}

static void* run_heads(void* arg) {
  job_t* j = (job_t*)arg;
  const int D = j->D, G = j->Hq / j->Hkv;
  const double scale = 1.0 / sqrt((double)D);
  double* qd = (double*)malloc(sizeof(double) * D);
  double* acc = (double*)malloc(sizeof(double) * D);
  if (!qd || !acc) { j->rc = -2; free(qd); free(acc); return 0; }
  for (int h = j->h0; h < j->h1; ++h) {
    const int kh = h / G;
    const float ks = j->kv_kind == 2 ? j->k_scale[kh] : 1.f, vs = j->kv_kind == 2 ? j->v_scale[kh] : 1.f;
    for (int d = 0; d < D; ++d) {
      uint16_t b = ((const uint16_t*)j->q)[(long)h * D + d];
      qd[d] = j->q_kind ? f16_to_f32(b) : bf16_to_f32(b);
      acc[d] = 0.0;
    }
    double m = -INFINITY, l = 0.0;
    for (long s = 0; s < j->S; ++s) {
      const long base = (long)kh * j->head_stride + s * D;
      double dot = 0.0;
      for (int d = 0; d < D; ++d) dot += qd[d] * load_kv(j->k, base + d, j->kv_kind, ks);
      const double sc = dot * scale;
      const double mn = sc > m ? sc : m;
      const double a = (m == -INFINITY) ? 0.0 : exp(m - mn);
      const double p = exp(sc - mn);
      for (int d = 0; d < D; ++d) acc[d] = acc[d] * a + p * load_kv(j->v, base + d, j->kv_kind, vs);
      l = l * a + p;
      m = mn;
    }
    for (int d = 0; d < D; ++d) j->out[(long)h * D + d] = l > 0 ? acc[d] / l : 0.0;
    if (j->lse) j->lse[h] = l > 0 ? m + log(l) : -INFINITY;
  }
  free(qd);
  free(acc);
  return 0;
}

int gqa_oracle_attend(const void* q, int q_kind, const void* k, const void* v, int kv_kind,
                      const float* k_scale, const float* v_scale, int Hq, int Hkv, long S, int D,
                      long head_stride, double* out, double* lse, int threads) {
  if (Hkv <= 0 || Hq % Hkv || S < 0 || D <= 0) return -1;
  if (threads < 1) threads = 1;
  if (threads > Hq) threads = Hq;
  if (threads > 256) threads = 256;
  job_t jobs[256];
  pthread_t tids[256];
  for (int t = 0; t < threads; ++t) {
    job_t j = {q, k, v, k_scale, v_scale, q_kind, kv_kind, Hq, Hkv, D,
               (int)((long)Hq * t / threads), (int)((long)Hq * (t + 1) / threads),
               S, head_stride, out, lse, 0};
    jobs[t] = j;
    if (pthread_create(&tids[t], 0, run_heads, &jobs[t])) return -3;
  }
  int rc = 0;
  for (int t = 0; t < threads; ++t) {
    pthread_join(tids[t], 0);
    if (jobs[t].rc) rc = jobs[t].rc;
  }
  return rc;
}

/* bf16_round(float32(code) * scale) for n codes: the dequantisation contract on its own. */
void gqa_oracle_dequant_e4m3(const uint8_t* codes, float scale, long n, uint16_t* out_bf16) {
  for (long i = 0; i < n; ++i) out_bf16[i] = f32_to_bf16_rne(e4m3_to_f32(codes[i]) * scale);
}
