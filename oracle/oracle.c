/*
 * CPU oracle for the fp16 HWC U-Net dispatch path of denox.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing on the product path may call into this
 * file; it exists so that the CUDA kernels can be checked against a plain
 * restatement of the reference arithmetic, and so that a CPU baseline can be
 * timed next to the GPU numbers.
 *
 * Parity status: the reference ships no golden vectors for this path (its
 * tests compare against PyTorch with unseeded random inputs), and its shaders
 * cannot run here (no Vulkan).  Bit-level parity is therefore UNPINNED; what is
 * pinned is the tolerance contract against PyTorch semantics
 * (test/__init__.py:48-49,97: allclose(rtol=1e-3, atol=1e-2)), which the tests
 * check through fixtures generated with PyTorch on CPU.
 *
 * Each function cites the reference file it restates (paths relative to the
 * reference project root).
 *
 * Tensors are HWC, IEEE binary16 stored as uint16_t:
 *   index(h, w, c) = (h * W + w) * C + c
 *   (common/src/denox/memory/tensor/ActivationLayout.hpp:38-40)
 * Convolution weights arrive in the ONNX order KCRS (= OIHW),
 *   index(k, c, r, s) = ((k * C + c) * 3 + r) * 3 + s
 *   (compiler/src/denox/compiler/frontend/onnx/details/ops/conv.cpp:211-219)
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---- binary16 helpers ------------------------------------------------- */

static inline float h2f(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) { /* round to nearest even */
  _Float16 v = (_Float16)f;
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}
/* value of f after one rounding to binary16 */
static inline float rh(float f) { return (float)(_Float16)f; }

ORC_API void orc_f16_to_f32(const uint16_t *src, float *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = h2f(src[i]);
}
ORC_API void orc_f32_to_f16_rne(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = f2h(src[i]);
}
/* The reference's own float->half used when a model carries fp32 weights:
 * truncates the mantissa and flushes results below the normal range to zero
 * (common/src/denox/memory/dtype/f16.cpp:6-20). */
ORC_API void orc_f32_to_f16_trunc(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t x;
    memcpy(&x, &src[i], 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007FFFFFu;
    int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    if (e <= 0) dst[i] = (uint16_t)sign;
    else if (e >= 31) dst[i] = (uint16_t)(sign | 0x7C00u);
    else dst[i] = (uint16_t)(sign | ((uint32_t)e << 10) | (mant >> 13));
  }
}

/* ---- 3x3 convolution --------------------------------------------------- */

enum { ORC_ACC_F32 = 0, ORC_ACC_F16 = 1, ORC_ACC_F16_FMA = 2 };

/* One K-phase of the implicit GEMM: acc[k] += sum_{r,s,c} in(y+r-1, x+s-1, c) * w[r][s][c][k]
 * with zero padding decided by a bounds test on the input coordinate
 * (direct_conv.comp:209-212) and k walked as (r, s, c)
 * (direct_conv.comp:198-202, 458-543).
 * `up` != 0 reads the operand through the nearest-neighbour map
 * src = dst / 2 (basic_upsample.comp:49-56), i.e. `in` is H/2 x W/2.
 * halo_top / halo_bot, when non-NULL, supply row -1 / row H of the (virtual,
 * full resolution for up==0; half resolution source row for up!=0) operand for
 * a row band cut out of a taller image; NULL means image border (zeros). */
static void conv_phase(float *acc, int K, const uint16_t *in, int C, int up, int H, int W, int y,
                       int x, const uint16_t *halo_top, const uint16_t *halo_bot, const float *wt,
                       int mode) {
  const int Ws = up ? W / 2 : W;
  for (int r = 0; r < 3; ++r) {
    const int iy = y + r - 1;
    const uint16_t *row;
    if (iy < 0) {
      if (!halo_top) continue;
      row = halo_top;
    } else if (iy >= H) {
      if (!halo_bot) continue;
      row = halo_bot;
    } else {
      row = in + (int64_t)(up ? iy / 2 : iy) * Ws * C;
    }
    for (int s = 0; s < 3; ++s) {
      const int ix = x + s - 1;
      if (ix < 0 || ix >= W) continue;
      const uint16_t *px = row + (int64_t)(up ? ix / 2 : ix) * C;
      const float *w = wt + (int64_t)((r * 3 + s) * C) * K;
      if (mode == ORC_ACC_F32) {
        for (int c = 0; c < C; ++c) {
          const float a = h2f(px[c]);
          const float *wk = w + (int64_t)c * K;
          for (int k = 0; k < K; ++k) acc[k] += a * wk[k];
        }
      } else if (mode == ORC_ACC_F16) {
        /* acc and product each rounded to binary16 (direct_conv.comp:481-543:
         * f16vec2 acc += f16vec2(b) * f16vec2(a), no contraction). */
        for (int c = 0; c < C; ++c) {
          const float a = h2f(px[c]);
          const float *wk = w + (int64_t)c * K;
          for (int k = 0; k < K; ++k) acc[k] = rh(acc[k] + rh(a * wk[k]));
        }
      } else {
        /* the same with the multiply-add contracted into one rounding */
        for (int c = 0; c < C; ++c) {
          const double a = h2f(px[c]);
          const float *wk = w + (int64_t)c * K;
          for (int k = 0; k < K; ++k) acc[k] = rh((float)((double)acc[k] + a * (double)wk[k]));
        }
      }
    }
  }
}

/* The activation on a finished sum, in binary16 as the reference applies it to its binary16 accumulator:
 * act 1 = max(0, x) (direct_conv.comp:559-590, direct_conv_cm.comp:1061-1070), act 2 = LeakyReLU
 * max(alpha * x, x) with alpha rounded to binary16 and the product rounded to binary16
 * (direct_conv_cm.comp:1071-1076, basic_activation.comp:26-34).  Of two zeros the positive one wins,
 * as in the max of IEEE 754-2019. */
static inline uint16_t activate_h(uint16_t xh, int act, float alpha) {
  const float x = h2f(xh);
  if (act == 1) return f2h(x > 0.0f ? x : 0.0f);
  if (act == 2) {
    const float a = rh(rh(alpha) * x); /* exact product of two binary16 values, one rounding */
    if (x > a || (x == a && !signbit(x))) return xh;
    return f2h(a);
  }
  return xh;
}

/* conv3x3, stride 1, padding 1, optional bias, optional ReLU, over the channel
 * concatenation [a, b] (a first: torch.cat((upsampled, skip), 1),
 * oidn_model.py:227-228).  Restates direct_conv.comp:82-775 for one operand
 * and the two-phase loop of concat_conv_cm.comp:1042-1127 (all of a's taps,
 * then all of b's, into one accumulator; weights split along C,
 * ConcatConvCMShader.cpp:832-873) for two.  ReLU is applied to the finished
 * sum (direct_conv.comp:559-590).  Cb == 0 / b == NULL selects the one-operand
 * form.  up_a != 0: `a` is H/2 x W/2 and is read through the 2x nearest map.
 * w_kcrs: [K][Ca+Cb][3][3] binary16.  bias: [K] binary16 or NULL. */
ORC_API int orc_conv3x3_act(const uint16_t *a, int Ca, int up_a, const uint16_t *b, int Cb, int H,
                            int W, const uint16_t *w_kcrs, const uint16_t *bias, int K, int act,
                            float alpha, int mode, uint16_t *out, const uint16_t *a_halo_top,
                            const uint16_t *a_halo_bot, const uint16_t *b_halo_top,
                            const uint16_t *b_halo_bot) {
  if (!a || !w_kcrs || !out || Ca <= 0 || K <= 0 || H <= 0 || W <= 0) return -1;
  if (up_a && ((H | W) & 1)) return -1;
  const int C = Ca + Cb;
  /* weights as float [r][s][c][k], one table per operand */
  float *wa = (float *)malloc(sizeof(float) * 9 * (size_t)Ca * K);
  float *wb = Cb ? (float *)malloc(sizeof(float) * 9 * (size_t)Cb * K) : NULL;
  for (int k = 0; k < K; ++k)
    for (int c = 0; c < C; ++c)
      for (int r = 0; r < 3; ++r)
        for (int s = 0; s < 3; ++s) {
          const float v = h2f(w_kcrs[(((int64_t)k * C + c) * 3 + r) * 3 + s]);
          if (c < Ca) wa[((int64_t)((r * 3 + s) * Ca + c)) * K + k] = v;
          else wb[((int64_t)((r * 3 + s) * Cb + (c - Ca))) * K + k] = v;
        }
#pragma omp parallel
  {
    float *acc = (float *)malloc(sizeof(float) * K);
#pragma omp for schedule(dynamic, 1)
    for (int y = 0; y < H; ++y) {
      for (int x = 0; x < W; ++x) {
        for (int k = 0; k < K; ++k) acc[k] = bias ? h2f(bias[k]) : 0.0f;
        conv_phase(acc, K, a, Ca, up_a, H, W, y, x, a_halo_top, a_halo_bot, wa, mode);
        if (Cb) conv_phase(acc, K, b, Cb, 0, H, W, y, x, b_halo_top, b_halo_bot, wb, mode);
        uint16_t *o = out + ((int64_t)y * W + x) * K;
        for (int k = 0; k < K; ++k) o[k] = activate_h(f2h(acc[k]), act, alpha);
      }
    }
    free(acc);
  }
  free(wa);
  free(wb);
  return 0;
}

/* The form without LeakyReLU: relu != 0 selects max(0, x). */
ORC_API int orc_conv3x3(const uint16_t *a, int Ca, int up_a, const uint16_t *b, int Cb, int H,
                        int W, const uint16_t *w_kcrs, const uint16_t *bias, int K, int relu,
                        int mode, uint16_t *out, const uint16_t *a_halo_top,
                        const uint16_t *a_halo_bot, const uint16_t *b_halo_top,
                        const uint16_t *b_halo_bot) {
  return orc_conv3x3_act(a, Ca, up_a, b, Cb, H, W, w_kcrs, bias, K, relu ? 1 : 0, 0.0f, mode, out,
                         a_halo_top, a_halo_bot, b_halo_top, b_halo_bot);
}

/* 2x2 / stride 2 max pool, floor output size, -inf start value
 * (basic_pool.comp:41-42, 44-82). out: (H/2) x (W/2) x C. */
ORC_API int orc_maxpool2x2(const uint16_t *in, int H, int W, int C, uint16_t *out) {
  const int H2 = H / 2, W2 = W / 2;
#pragma omp parallel for
  for (int y = 0; y < H2; ++y)
    for (int x = 0; x < W2; ++x)
      for (int c = 0; c < C; ++c) {
        float m = -INFINITY;
        for (int r = 0; r < 2; ++r)
          for (int s = 0; s < 2; ++s) {
            const float v = h2f(in[((int64_t)(2 * y + r) * W + (2 * x + s)) * C + c]);
            m = v > m ? v : m;
          }
        out[((int64_t)y * W2 + x) * C + c] = f2h(m);
      }
  return 0;
}

/* 2x nearest upsample: out[h2][w2] = in[h2/2][w2/2] (basic_upsample.comp:49-56). */
ORC_API int orc_upsample2x(const uint16_t *in, int H, int W, int C, uint16_t *out) {
  const int H2 = H * 2, W2 = W * 2;
#pragma omp parallel for
  for (int y = 0; y < H2; ++y)
    for (int x = 0; x < W2; ++x)
      memcpy(out + ((int64_t)y * W2 + x) * C, in + ((int64_t)(y / 2) * W + x / 2) * C,
             (size_t)C * 2);
  return 0;
}

/* channel concat, src0 then src1 (copy_transform.comp:53-64 run twice with
 * OUT_OFF = 0 and OUT_OFF = C0). */
ORC_API int orc_concat(const uint16_t *a, int Ca, const uint16_t *b, int Cb, int H, int W,
                       uint16_t *out) {
  const int C = Ca + Cb;
#pragma omp parallel for
  for (int64_t p = 0; p < (int64_t)H * W; ++p) {
    memcpy(out + p * C, a + p * Ca, (size_t)Ca * 2);
    memcpy(out + p * C + Ca, b + p * Cb, (size_t)Cb * 2);
  }
  return 0;
}

/* standalone ReLU, max(v, 0) in binary16 (basic_activation.comp:26-34). */
ORC_API int orc_relu(const uint16_t *in, int64_t n, uint16_t *out) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) {
    const float v = h2f(in[i]);
    out[i] = f2h(v > 0.0f ? v : 0.0f);
  }
  return 0;
}

/* standalone LeakyReLU (basic_activation.comp:29-30). */
ORC_API int orc_leaky_relu(const uint16_t *in, int64_t n, float alpha, uint16_t *out) {
#pragma omp parallel for
  for (int64_t i = 0; i < n; ++i) out[i] = activate_h(in[i], 2, alpha);
  return 0;
}

/* Spatial pad with edge replication (memory_pad.comp:71-72: the source coordinate is the
 * output coordinate minus the pad, clamped to the input extent).  out is
 * (H + top + bottom) x (W + left + right) x C. */
ORC_API int orc_pad_edge(const uint16_t *in, int H, int W, int C, int left, int right, int top,
                         int bottom, uint16_t *out) {
  const int OH = H + top + bottom, OW = W + left + right;
  if (H <= 0 || W <= 0 || left < 0 || right < 0 || top < 0 || bottom < 0) return -1;
#pragma omp parallel for
  for (int ho = 0; ho < OH; ++ho)
    for (int wo = 0; wo < OW; ++wo) {
      int hi = ho - top, wi = wo - left;
      hi = hi < 0 ? 0 : (hi > H - 1 ? H - 1 : hi);
      wi = wi < 0 ? 0 : (wi > W - 1 ? W - 1 : wi);
      memcpy(out + ((int64_t)ho * OW + wo) * C, in + ((int64_t)hi * W + wi) * C, (size_t)C * 2);
    }
  return 0;
}

/* Spatial slice: out[h][w] = in[h + top][w + left] (memory_slice.comp:59-66). */
ORC_API int orc_slice(const uint16_t *in, int H, int W, int C, int left, int top, int OH, int OW,
                      uint16_t *out) {
  if (left < 0 || top < 0 || left + OW > W || top + OH > H) return -1;
#pragma omp parallel for
  for (int h = 0; h < OH; ++h)
    memcpy(out + (int64_t)h * OW * C, in + ((int64_t)(h + top) * W + left) * C, (size_t)OW * C * 2);
  return 0;
}

/* Number of threads the parallel loops use from now on (n <= 0: leave as it is). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
  int n = 1;
#pragma omp parallel
  {
#pragma omp master
    n =
#ifdef _OPENMP
        __builtin_omp_get_num_threads();
#else
        1;
#endif
  }
  return n;
}
