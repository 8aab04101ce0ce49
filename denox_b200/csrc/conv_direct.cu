// "direct-conv": 3x3 convolution as an implicit GEMM on the CUDA cores with
// fp32 accumulation.  It is the variant that runs every shape (any channel
// count, any alignment) and the one a device without tcgen05 would get, the
// role direct_conv.comp plays next to direct_conv_cm.comp in the reference
// (compiler/src/denox/compiler/implement/shaders/shaders.cpp:22-30).
//
// One block = 8 x 16 output pixels x 32 output channels, one thread per pixel.
// The K loop walks operand a then operand b (concat_conv_cm.comp:1042-1127) in
// chunks of 8 channels; per chunk the 10 x 18 input halo and the 9 x 8 x 32
// weights are staged in shared memory.  Nearest upsampling of operand a is an
// address map in the loader (src = dst / 2, basic_upsample.comp:49-56); zero
// padding is a bounds test (direct_conv.comp:209-212).
#include "internal.h"

namespace dnxcu {
namespace {

constexpr int TW = 16, TH = 8, KT = 32, CC = 8;
constexpr int HW_ = TW + 2, HH_ = TH + 2;

struct Operand {
  const __half *ptr;       // H x W x C, or (H/2) x (W/2) x C when up
  const __half *halo_top;  // row -1, or nullptr
  const __half *halo_bot;  // row H, or nullptr
  int C;
  int up;
};

struct DirectArgs {
  Operand a, b;
  const __half *w;  // [chunk][tap][8][Kp]
  const __half *bias;
  __half *out;
  int H, W, K, Kp;
  int relu;      // 0 none, 1 max(x, 0), 2 max(x, alpha * x) in binary16 on the rounded sum
  __half alpha;
};

__global__ void __launch_bounds__(TW *TH) conv3x3_direct(DirectArgs g) {
  __shared__ float s_in[CC][HH_][HW_ + 1];
  __shared__ __align__(16) float s_w[9][CC][KT];

  const int tx = threadIdx.x % TW, ty = threadIdx.x / TW;
  const int x0 = blockIdx.x * TW, y0 = blockIdx.y * TH, k0 = blockIdx.z * KT;

  float acc[KT];
#pragma unroll
  for (int k = 0; k < KT; ++k) acc[k] = 0.0f;
  if (g.bias) {
#pragma unroll
    for (int k = 0; k < KT; ++k)
      if (k0 + k < g.K) acc[k] = __half2float(g.bias[k0 + k]);
  }

  int chunk = 0;
  for (int seg = 0; seg < 2; ++seg) {
    const Operand &op = seg == 0 ? g.a : g.b;
    if (op.C <= 0) continue;
    const int Ws = op.up ? g.W >> 1 : g.W;
    for (int c0 = 0; c0 < op.C; c0 += CC, ++chunk) {
      __syncthreads();
      // input halo tile: HH_ x HW_ pixels x 8 channels
      for (int i = threadIdx.x; i < HH_ * HW_ * CC; i += TW * TH) {
        const int c = i % CC;
        const int p = i / CC;
        const int px = p % HW_, py = p / HW_;
        const int iy = y0 + py - 1, ix = x0 + px - 1;
        float v = 0.0f;
        if (ix >= 0 && ix < g.W && c0 + c < op.C) {
          const __half *row = nullptr;
          if (iy < 0) row = (iy == -1) ? op.halo_top : nullptr;
          else if (iy >= g.H) row = (iy == g.H) ? op.halo_bot : nullptr;
          else row = op.ptr + (long long)(op.up ? iy >> 1 : iy) * Ws * op.C;
          if (row) v = __half2float(row[(long long)(op.up ? ix >> 1 : ix) * op.C + c0 + c]);
        }
        s_in[c][py][px] = v;
      }
      // weights of this chunk for output channels [k0, k0 + 32)
      const __half *wsrc = g.w + (long long)chunk * 9 * CC * g.Kp + k0;
      for (int i = threadIdx.x; i < 9 * CC * KT; i += TW * TH) {
        const int k = i % KT;
        const int tc = i / KT;  // tap * 8 + c
        s_w[tc / CC][tc % CC][k] = __half2float(wsrc[(long long)tc * g.Kp + k]);
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int s = 0; s < 3; ++s)
#pragma unroll
          for (int c = 0; c < CC; ++c) {
            const float a = s_in[c][ty + r][tx + s];
            const float4 *w4 = reinterpret_cast<const float4 *>(&s_w[r * 3 + s][c][0]);
#pragma unroll
            for (int k4 = 0; k4 < KT / 4; ++k4) {
              const float4 w = w4[k4];
              acc[4 * k4 + 0] = fmaf(a, w.x, acc[4 * k4 + 0]);
              acc[4 * k4 + 1] = fmaf(a, w.y, acc[4 * k4 + 1]);
              acc[4 * k4 + 2] = fmaf(a, w.z, acc[4 * k4 + 2]);
              acc[4 * k4 + 3] = fmaf(a, w.w, acc[4 * k4 + 3]);
            }
          }
    }
  }

  const int x = x0 + tx, y = y0 + ty;
  if (x >= g.W || y >= g.H) return;
  __half *o = g.out + ((long long)y * g.W + x) * g.K + k0;
#pragma unroll
  for (int k = 0; k < KT; ++k) {
    if (k0 + k < g.K) {
      float v = acc[k];
      if (g.relu == 1) v = fmaxf(v, 0.0f);
      __half h = __float2half_rn(v);
      if (g.relu == 2) h = __hmax(h, __hmul(g.alpha, h));
      o[k] = h;
    }
  }
}

inline int chunks(int c) { return (c + CC - 1) / CC; }
inline int kpad(int k) { return (k + KT - 1) / KT * KT; }

}  // namespace

size_t conv_direct_weight_bytes(const Variant &, int k, int ca, int cb) {
  return (size_t)(chunks(ca) + chunks(cb)) * 9 * CC * kpad(k) * 2;
}

// KCRS -> [chunk][tap][c8][Kp], operand a's chunks first, zero padded.
void conv_direct_prepare(const Variant &, const uint16_t *kcrs, int K, int ca, int cb, uint16_t *out) {
  const int C = ca + cb, Kp = kpad(K);
  const size_t n = (size_t)(chunks(ca) + chunks(cb)) * 9 * CC * Kp;
  for (size_t i = 0; i < n; ++i) out[i] = 0;
  for (int seg = 0; seg < 2; ++seg) {
    const int Cs = seg ? cb : ca, cbase = seg ? ca : 0, chbase = seg ? chunks(ca) : 0;
    for (int c = 0; c < Cs; ++c)
      for (int t = 0; t < 9; ++t)
        for (int k = 0; k < K; ++k)
          out[(((size_t)(chbase + c / CC) * 9 + t) * CC + c % CC) * Kp + k] =
              kcrs[((size_t)k * C + cbase + c) * 9 + t];
  }
}

int conv_direct_validate(const Variant &, const dnxcu_dispatch &d) {
  if (!d.in_a || !d.out || !d.weights || d.c_a <= 0 || d.c_out <= 0 || d.c_b < 0) return DNXCU_E_BAD_ARG;
  if (d.pc[0] == 0 || d.pc[1] == 0) return DNXCU_E_BAD_ARG;
  if (d.c_b > 0 && !d.in_b) return DNXCU_E_BAD_ARG;
  if ((d.flags & DNXCU_F_BIAS) && !d.bias) return DNXCU_E_BAD_ARG;
  if ((d.flags & DNXCU_F_UP2X_A) && ((d.pc[0] | d.pc[1]) & 1)) return DNXCU_E_BAD_ARG;
  if (d.flags & (DNXCU_F_POOL_OUT | DNXCU_F_NO_FULL_OUT)) return DNXCU_E_UNSUPPORTED;
  if (((uintptr_t)d.in_a | (uintptr_t)d.in_b | (uintptr_t)d.out | (uintptr_t)d.weights | (uintptr_t)d.bias) & 1)
    return DNXCU_E_MISALIGNED;
  return DNXCU_OK;
}

void conv_direct_grid(const Variant &, const dnxcu_dispatch &d, uint32_t g[3]) {
  g[0] = cdiv(d.pc[0], TW);
  g[1] = cdiv(d.pc[1], TH);
  g[2] = cdiv((uint32_t)d.c_out, KT);
}

int conv_direct_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s) {
  int st = conv_direct_validate(v, d);
  if (st) return st;
  DirectArgs g;
  g.a = {(const __half *)d.in_a, (const __half *)d.halo[0], (const __half *)d.halo[1], d.c_a,
         (d.flags & DNXCU_F_UP2X_A) ? 1 : 0};
  g.b = {(const __half *)d.in_b, (const __half *)d.halo[2], (const __half *)d.halo[3], d.c_b, 0};
  g.w = (const __half *)d.weights;
  g.bias = (d.flags & DNXCU_F_BIAS) ? (const __half *)d.bias : nullptr;
  g.out = (__half *)d.out;
  g.W = (int)d.pc[0];
  g.H = (int)d.pc[1];
  g.K = d.c_out;
  g.Kp = kpad(d.c_out);
  g.relu = (d.flags & DNXCU_F_LEAKY) ? 2 : ((d.flags & DNXCU_F_RELU) ? 1 : 0);
  g.alpha = __float2half_rn(d.leaky_alpha);
  uint32_t grid[3];
  conv_direct_grid(v, d, grid);
  conv3x3_direct<<<dim3(grid[0], grid[1], grid[2]), TW * TH, 0, s>>>(g);
  DNXCU_CUDA(cudaGetLastError());
  return DNXCU_OK;
}

}  // namespace dnxcu
