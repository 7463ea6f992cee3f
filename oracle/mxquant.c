/* C restatement of the reference's MXFP8 quantiser.  TEST INFRASTRUCTURE ONLY: used by tests/ as a second,
 * independent checker next to oracle/reference_math.py:quantize_mx and by bench.py as the timed CPU baseline of
 * the quantiser; never linked into the product library.
 *
 * Follows warpy_kernels/gemm/sm89.py:65-93 (_store_mx: block = 32 consecutive columns of a row, integer amax of
 * sign-cleared fp32 bit patterns), warpy_kernels/ptx/common.py:546-565 (mx_scale) and
 * warpy_kernels/ptx/sm89.py:85-93 (pack_e4m3x2 = cvt.rn.satfinite.e4m3x2.f32: round to nearest even, saturate at
 * +-448).  PARITY UNPINNED against reference outputs (the reference has no CPU implementation and no golden
 * vectors for this arithmetic); pinned by hand-derived known answers and the reference test's two properties.
 */
#include <stdint.h>
#include <string.h>
#include <pthread.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> e4m3 code, RNE, saturating (NaN -> 0x7f). */
static inline uint8_t e4m3_rne_sat(float x) {
  const uint32_t bits = f2u(x);
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80);
  const uint32_t mag = bits & 0x7fffffffu;
  if (mag > 0x7f800000u) return (uint8_t)(sign | 0x7f);
  if (mag == 0) return sign;
  const int exp = (int)(mag >> 23) - 127;
  const uint64_t man = (uint64_t)(mag & 0x7fffffu) | 0x800000u;
  int shift = exp >= -6 ? 20 : 20 + (-6 - exp);
  if (shift > 40) shift = 40;
  uint64_t q = man >> shift;
  const uint64_t rem = man & (((uint64_t)1 << shift) - 1);
  const uint64_t half = (uint64_t)1 << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) q += 1;
  uint64_t code = exp >= -6 ? (((uint64_t)(exp + 7) - 1) << 3) + q : q;
  if (code > 0x7e) code = 0x7e;
  return (uint8_t)(sign | (uint8_t)code);
}

/* rows [r0, r1) of x [rows, cols] fp32 row-major (leading dimension ld). */
static void quantize_rows_f32(const float* x, int64_t r0, int64_t r1, int64_t cols, int64_t ld, uint8_t* q,
                              uint8_t* s) {
  const int64_t nblk = cols / 32;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nblk; ++b) {
      const float* p = x + r * ld + b * 32;
      uint32_t amax = 0;
      for (int i = 0; i < 32; ++i) {
        const uint32_t a = f2u(p[i]) & 0x7fffffffu;
        if (a > amax) amax = a;
      }
      int e = (int)((amax + 0x1fffffu) >> 23) - 8;
      if (e < 0) e = 0;
      if (e > 254) e = 254;
      int ie = 254 - e;
      if (ie < 1) ie = 1;
      const float inv = u2f((uint32_t)ie << 23);
      uint8_t* out = q + r * cols + b * 32;
      for (int i = 0; i < 32; ++i) out[i] = e4m3_rne_sat(p[i] * inv);
      s[r * nblk + b] = (uint8_t)e;
    }
  }
}

/* Same for bf16 input (raw 16-bit patterns); bf16 -> fp32 is exact. */
static void quantize_rows_bf16(const uint16_t* x, int64_t r0, int64_t r1, int64_t cols, int64_t ld, uint8_t* q,
                               uint8_t* s) {
  const int64_t nblk = cols / 32;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nblk; ++b) {
      const uint16_t* p = x + r * ld + b * 32;
      float v[32];
      uint32_t amax = 0;
      for (int i = 0; i < 32; ++i) {
        const uint32_t u = (uint32_t)p[i] << 16;
        v[i] = u2f(u);
        if ((u & 0x7fffffffu) > amax) amax = u & 0x7fffffffu;
      }
      int e = (int)((amax + 0x1fffffu) >> 23) - 8;
      if (e < 0) e = 0;
      if (e > 254) e = 254;
      int ie = 254 - e;
      if (ie < 1) ie = 1;
      const float inv = u2f((uint32_t)ie << 23);
      uint8_t* out = q + r * cols + b * 32;
      for (int i = 0; i < 32; ++i) out[i] = e4m3_rne_sat(v[i] * inv);
      s[r * nblk + b] = (uint8_t)e;
    }
  }
}

typedef struct {
  const void* x;
  int64_t r0, r1, cols, ld;
  uint8_t *q, *s;
  int bf16;
} job_t;

static void* worker(void* arg) {
  job_t* j = (job_t*)arg;
  if (j->bf16)
    quantize_rows_bf16((const uint16_t*)j->x, j->r0, j->r1, j->cols, j->ld, j->q, j->s);
  else
    quantize_rows_f32((const float*)j->x, j->r0, j->r1, j->cols, j->ld, j->q, j->s);
  return 0;
}

/* x [rows, cols] (fp32, or bf16 bit patterns when bf16 != 0), leading dimension ld elements ->
 * q [rows, cols] codes, s [rows, cols/32] scale bytes; rows are split over nthreads pthreads. */
void oracle_quantize_mx(const void* x, int bf16, int64_t rows, int64_t cols, int64_t ld, uint8_t* q, uint8_t* s,
                        int nthreads) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  pthread_t th[256];
  job_t jobs[256];
  const int64_t per = (rows + nthreads - 1) / nthreads;
  int started = 0;
  for (int t = 0; t < nthreads; ++t) {
    int64_t r0 = t * per, r1 = r0 + per;
    if (r1 > rows) r1 = rows;
    if (r0 >= r1) break;
    jobs[t] = (job_t){x, r0, r1, cols, ld, q, s, bf16};
    if (t == nthreads - 1 || r1 == rows) {
      worker(&jobs[t]); /* last slice on the calling thread */
      break;
    }
    pthread_create(&th[t], 0, worker, &jobs[t]);
    started = t + 1;
  }
  for (int t = 0; t < started; ++t) pthread_join(th[t], 0);
}
