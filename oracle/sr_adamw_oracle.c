/*
 * sr_adamw_oracle.c — TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement, for the CPU, of the optimizer-step arithmetic of RamTorch
 * (ramtorch/stochastic_optimizers/adamw.py).  It is the checker the CUDA kernels are compared
 * with and the CPU baseline the benchmark times.  Nothing in the product package may
 * import, link or execute it.
 *
 * Pinning: the fp32 update and the map (fp32 bits, r16) -> bf16 are pinned against outputs of
 * the reference's own AdamW.step / copy_stochastic_ executed on the CPU (fixtures under
 * tests/golden/, produced by tests/golden/make_golden.py).  The reference ships no golden
 * vectors of its own.  The random bit STREAM of the reference (torch.Generator) is not
 * reproduced: it is replaced by the counter-based Philox4x32-10 stream specified in
 * include/rt_b200.h, pinned here against the Random123 known-answer vectors.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/build_oracle.py).
 * -ffp-contract=off matters: the only fused operations are the explicit fmaf() calls.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/rt_b200.h"

/* ---------------------------------------------------------------- Philox4x32-10 */
/* Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3" (SC'11). */
#define PHILOX_M0 0xD2511F53u
#define PHILOX_M1 0xCD9E8D57u
#define PHILOX_W0 0x9E3779B9u
#define PHILOX_W1 0xBB67AE85u

void rto_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3];
  uint32_t k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    uint64_t p0 = (uint64_t)PHILOX_M0 * c0;
    uint64_t p1 = (uint64_t)PHILOX_M1 * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += PHILOX_W0;
    k1 += PHILOX_W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* The 16-bit draw of element i (index inside its tensor); include/rt_b200.h "Random bits". */
static inline uint32_t draw16_at(uint64_t seed, uint32_t tensor_id, uint32_t step,
                                 uint32_t stream, int64_t i);

/* RT_HYPER_SHARED_DRAWS: every stream reads the block of stream 0, two lanes further per stream. */
static inline uint32_t draw16(uint64_t seed, uint32_t tensor_id, uint32_t step,
                              uint32_t stream, int64_t i, int shared) {
  if (!shared) return draw16_at(seed, tensor_id, step, stream, i);
  return draw16_at(seed, tensor_id, step, 0, (i & ~(int64_t)7) | (((i & 7) + 2 * (int64_t)stream) & 7));
}

static inline uint32_t draw16_at(uint64_t seed, uint32_t tensor_id, uint32_t step,
                                 uint32_t stream, int64_t i) {
  uint32_t ctr[4] = {(uint32_t)((uint64_t)i >> 3), tensor_id, step, stream};
  uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t out[4];
  rto_philox4x32_10(ctr, key, out);
  uint32_t j = (uint32_t)(i & 7);
  uint32_t w = out[j >> 1];
  return (j & 1) ? (w >> 16) : (w & 0xFFFFu);
}

void rto_draws(uint64_t seed, uint32_t tensor_id, uint32_t step, uint32_t stream,
               int64_t index0, int64_t n, uint16_t* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    out[i] = (uint16_t)draw16(seed, tensor_id, step, stream, index0 + i, 0);
}

/* ---------------------------------------------------------------- bit helpers */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* copy_stochastic_, adamw.py:13-30: randint[0,65536) as int32, += bits(source) (wrapping
 * int32 add), &= 0xFFFF0000, then copy into the bf16 target (exact: low 16 bits are zero). */
static inline uint16_t sr_bf16(float x, uint32_t r16) {
  return (uint16_t)(((f2u(x) + r16) & 0xFFFF0000u) >> 16);
}

void rto_sr_round_bf16(uint16_t* target, const float* source, const uint16_t* rand16,
                       int64_t n) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) target[i] = sr_bf16(source[i], rand16[i]);
}

static inline float load_as_f32(const void* base, int dtype, int64_t i) {
  switch (dtype) {
    case RT_BF16: return u2f((uint32_t)((const uint16_t*)base)[i] << 16);
    case RT_F32:  return ((const float*)base)[i];
    default:      return (float)((const _Float16*)base)[i];
  }
}

/* Write-back of adamw.py:204-222: bf16 -> stochastic rounding, otherwise Tensor.copy_
 * (exact for fp32, round-to-nearest-even for fp16). */
static inline void store_from_f32(void* base, int dtype, int64_t i, float x, uint32_t r16) {
  switch (dtype) {
    case RT_BF16: ((uint16_t*)base)[i] = sr_bf16(x, r16); break;
    case RT_F32:  ((float*)base)[i] = x; break;
    default:      ((_Float16*)base)[i] = (_Float16)x; break;
  }
}

/* ---------------------------------------------------------------- the step */
/*
 * One AdamW.step body (adamw.py:160-222) over n contiguous elements, in place.
 *   index0    tensor-local index of element 0 (for the Philox counter)
 *   row_mean  NULL, or the per-element-row mean of the fp32 gradient already multiplied by
 *             nothing: g -= centralization * row_mean[i / row_len]   (adamw.py:179-184)
 *   rand_*    NULL (draw from Philox) or injected 16-bit draws, one per element
 *   f32_*     NULL or taps receiving p', m', v' before the write-back
 */
int rto_adamw_sr(void* p, const void* g, void* m, void* v, int64_t n,
                 int p_dtype, int g_dtype, int state_dtype, const rt_hyper* h,
                 uint64_t seed, uint32_t tensor_id, int64_t index0,
                 const float* row_mean, int64_t row_len,
                 const uint16_t* rand_p, const uint16_t* rand_m, const uint16_t* rand_v,
                 float* f32_p, float* f32_m, float* f32_v) {
  if (!p || !g || !m || !v || !h) return -1;
  if (n < 0) return -3;
  const int sr_p = (p_dtype == RT_BF16), sr_s = (state_dtype == RT_BF16);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float gi = load_as_f32(g, g_dtype, i);
    float mi = load_as_f32(m, state_dtype, i);
    float vi = load_as_f32(v, state_dtype, i);
    float pi = load_as_f32(p, p_dtype, i);
    if (row_mean) {
      /* grad.sub_(mean.mul_(c)), adamw.py:180-184 */
      float cm = row_mean[row_len > 0 ? (index0 + i) / row_len : 0] * h->centralization;
      gi = gi - cm;
    }
    /* ema.mul_(beta1).add_(grad, alpha=1-beta1): the add with alpha is a fused
     * multiply-add in ATen's vectorised CPU kernel (adamw.py:190). */
    float m1 = fmaf(h->one_minus_beta1, gi, mi * h->beta1);
    /* ema_sq.mul_(beta2).addcmul_(grad, grad, value=1-beta2) (adamw.py:191) */
    float v1 = fmaf(h->one_minus_beta2 * gi, gi, vi * h->beta2);
    /* p.mul_(1 - step_size*wd) (adamw.py:197-198) */
    float pw = h->apply_decay ? pi * h->decay : pi;
    float p1;
    if (h->flags & RT_HYPER_REFERENCE_ORDER) {
      /* denom = (sqrt(v) / bias_correction_sqrt).add_(eps) (adamw.py:193-195);
       * p.addcdiv_(m, denom, value=-step_size) (adamw.py:199-200), in the reference's order */
      float den = sqrtf(v1) / h->bias_correction2_sqrt + h->eps;
      p1 = pw + (h->neg_step_size * m1) / den;
    } else {
      /* the same two lines in the default order of include/rt_b200.h: the division by the bias
       * correction becomes a multiply-add, the division by denom a reciprocal and a multiply-add;
       * sqrtf, fmaf and 1.0f / x are correctly rounded here as on the GPU */
      float den = fmaf(sqrtf(v1), h->inv_bias_correction2_sqrt, h->eps);
      p1 = fmaf(h->neg_step_size * m1, 1.0f / den, pw);
    }
    if (f32_p) f32_p[i] = p1;
    if (f32_m) f32_m[i] = m1;
    if (f32_v) f32_v[i] = v1;
    int64_t gi_idx = index0 + i;
    uint32_t rp = 0, rm = 0, rv = 0;
    const int shared = (h->flags & RT_HYPER_SHARED_DRAWS) != 0;
    if (sr_p) rp = rand_p ? rand_p[i] : draw16(seed, tensor_id, h->step, 0, gi_idx, shared);
    if (sr_s) {
      rm = rand_m ? rand_m[i] : draw16(seed, tensor_id, h->step, 1, gi_idx, shared);
      rv = rand_v ? rand_v[i] : draw16(seed, tensor_id, h->step, 2, gi_idx, shared);
    }
    store_from_f32(p, p_dtype, i, p1, rp);
    store_from_f32(m, state_dtype, i, m1, rm);
    store_from_f32(v, state_dtype, i, v1, rv);
  }
  return 0;
}

/* Same scalars as rt_hyper_fill of the product library, restated independently
 * (adamw.py:173-188): Python-double arithmetic, then one rounding to fp32 each. */
void rto_hyper_fill(rt_hyper* out, double lr, double beta1, double beta2, double eps,
                    double weight_decay, double centralization, uint32_t step) {
  double bc1 = 1.0 - pow(beta1, (double)step);
  double bc2s = sqrt(1.0 - pow(beta2, (double)step));
  double ss = lr / bc1;
  memset(out, 0, sizeof(*out));
  out->beta1 = (float)beta1;
  out->one_minus_beta1 = (float)(1.0 - beta1);
  out->beta2 = (float)beta2;
  out->one_minus_beta2 = (float)(1.0 - beta2);
  out->bias_correction2_sqrt = (float)bc2s;
  out->eps = (float)eps;
  out->decay = (float)(1.0 - ss * weight_decay);
  out->neg_step_size = (float)(-ss);
  out->centralization = (float)centralization;
  out->apply_decay = weight_decay != 0.0;
  out->step = step;
  out->inv_bias_correction2_sqrt = (float)(1.0 / (double)out->bias_correction2_sqrt);
}

void rto_set_num_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int rto_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}
