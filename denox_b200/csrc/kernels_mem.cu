// Bandwidth bound kernels: 2x2 max pool, 2x nearest upsample, channel concat,
// ReLU.  Each has a 128-bit form (channel counts multiple of 8, 16-byte aligned
// pointers) and a 2-byte form for everything else, like the reference's HWC8 /
// HWC split (basic_pool.comp:28-226).  All are grid-stride loops over 16-byte
// (or 2-byte) output items with consecutive threads on consecutive addresses.
#include "internal.h"

namespace dnxcu {
namespace {

__device__ __forceinline__ uint4 ldg16(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

__device__ __forceinline__ uint32_t hmax2u(uint32_t a, uint32_t b) {
  __half2 r = __hmax2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint4 hmax8(uint4 a, uint4 b) {
  return make_uint4(hmax2u(a.x, b.x), hmax2u(a.y, b.y), hmax2u(a.z, b.z), hmax2u(a.w, b.w));
}

// out[y][x][c] = max over the 2x2 window (basic_pool.comp:44-82), floor size.
__global__ void pool2x2_v8(const uint4 *__restrict__ in, uint4 *__restrict__ out, int H, int W, int C8) {
  const int H2 = H >> 1, W2 = W >> 1;
  const long long n = (long long)H2 * W2 * C8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const long long p = i / C8;
    const int x = (int)(p % W2), y = (int)(p / W2);
    const uint4 *r0 = in + ((long long)(2 * y) * W + 2 * x) * C8 + c;
    const uint4 *r1 = r0 + (long long)W * C8;
    uint4 a = ldg16(r0), b = ldg16(r0 + C8), d = ldg16(r1), e = ldg16(r1 + C8);
    out[i] = hmax8(hmax8(a, b), hmax8(d, e));
  }
}
__global__ void pool2x2_s(const __half *__restrict__ in, __half *__restrict__ out, int H, int W, int C) {
  const int H2 = H >> 1, W2 = W >> 1;
  const long long n = (long long)H2 * W2 * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const long long p = i / C;
    const int x = (int)(p % W2), y = (int)(p / W2);
    const __half *r0 = in + ((long long)(2 * y) * W + 2 * x) * C + c;
    const __half *r1 = r0 + (long long)W * C;
    out[i] = __hmax(__hmax(r0[0], r0[C]), __hmax(r1[0], r1[C]));
  }
}

// out[y][x] = in[y/2][x/2] (basic_upsample.comp:49-56); H, W are the INPUT extent.
__global__ void upsample2x_v8(const uint4 *__restrict__ in, uint4 *__restrict__ out, int H, int W, int C8) {
  const int W2 = W * 2;
  const long long n = (long long)H * 2 * W2 * C8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const long long p = i / C8;
    const int x = (int)(p % W2), y = (int)(p / W2);
    out[i] = ldg16(in + ((long long)(y >> 1) * W + (x >> 1)) * C8 + c);
  }
}
__global__ void upsample2x_s(const __half *__restrict__ in, __half *__restrict__ out, int H, int W, int C) {
  const int W2 = W * 2;
  const long long n = (long long)H * 2 * W2 * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const long long p = i / C;
    const int x = (int)(p % W2), y = (int)(p / W2);
    out[i] = in[((long long)(y >> 1) * W + (x >> 1)) * C + c];
  }
}

// out[p][0:Ca] = a[p], out[p][Ca:Ca+Cb] = b[p] (copy_transform.comp:53-64).
__global__ void concat_v8(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ out,
                          long long P, int Ca8, int Cb8) {
  const int C8 = Ca8 + Cb8;
  const long long n = P * C8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C8);
    const long long p = i / C8;
    out[i] = c < Ca8 ? ldg16(a + p * Ca8 + c) : ldg16(b + p * Cb8 + (c - Ca8));
  }
}
__global__ void concat_s(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ out,
                         long long P, int Ca, int Cb) {
  const int C = Ca + Cb;
  const long long n = P * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % C);
    const long long p = i / C;
    out[i] = c < Ca ? a[p * Ca + c] : b[p * Cb + (c - Ca)];
  }
}

// max(v, 0), or with LEAKY max(v, alpha * v) in binary16 (basic_activation.comp:26-34)
__device__ __forceinline__ uint32_t leaky2u(uint32_t a, __half2 alpha) {
  const __half2 v = *reinterpret_cast<__half2 *>(&a);
  __half2 r = __hmax2(v, __hmul2(alpha, v));
  return *reinterpret_cast<uint32_t *>(&r);
}
template <bool LEAKY>
__global__ void relu_v8(const uint4 *__restrict__ in, uint4 *__restrict__ out, long long n8, __half alpha) {
  const __half2 a2 = __half2half2(alpha);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = ldg16(in + i);
    if (LEAKY) out[i] = make_uint4(leaky2u(v.x, a2), leaky2u(v.y, a2), leaky2u(v.z, a2), leaky2u(v.w, a2));
    else out[i] = hmax8(v, make_uint4(0, 0, 0, 0));
  }
}
template <bool LEAKY>
__global__ void relu_s(const __half *__restrict__ in, __half *__restrict__ out, long long n, __half alpha) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    out[i] = LEAKY ? __hmax(in[i], __hmul(alpha, in[i])) : __hmax(in[i], __float2half(0.0f));
}

// out[p][0:C] = in[p][0:C], out[p][C:Cp] = 0: one thread per pixel and 8 channel piece of the output
// (2 byte loads: C is not a multiple of 8 when this runs; 16 byte stores).
__global__ void pad_channels(const unsigned short *__restrict__ in, uint4 *__restrict__ out, long long P, int C,
                             int Cp8) {
  const long long n = P * Cp8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % Cp8);
    const long long p = i / Cp8;
    const unsigned short *src = in + p * C + c8 * 8;
    unsigned int w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (c8 * 8 + e < C) w[e >> 1] |= (unsigned int)__ldg(src + e) << ((e & 1) * 16);
    out[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// The same by warps: the input of 32 consecutive pixels is 64 * C contiguous bytes that start on a 16 byte boundary
// when the tensor does, so a warp fetches them with 16 byte loads into its piece of shared memory (instead of up to
// nine 2 byte loads per pixel), picks the pieces apart there and writes the 32 * Cp8 output pieces with consecutive
// lanes on consecutive 16 bytes.  The last, partial group of pixels is fetched by 2 byte loads.
__global__ void pad_channels_warp(const unsigned short *__restrict__ in, uint4 *__restrict__ out, long long P, int C,
                                  int Cp8) {
  extern __shared__ uint4 pad_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  uint4 *s4 = pad_smem + (size_t)warp * 4 * C;  // 64 * C bytes per warp
  const unsigned short *s = reinterpret_cast<const unsigned short *>(s4);
  const uint4 *in16 = reinterpret_cast<const uint4 *>(in);
  const long long groups = (P + 31) / 32;
  for (long long w = (long long)blockIdx.x * wpb + warp; w < groups; w += (long long)gridDim.x * wpb) {
    const long long p0 = w * 32;
    const int np = (int)(P - p0 < 32 ? P - p0 : 32);
    if (np == 32) {
      for (int i = lane; i < 4 * C; i += 32) s4[i] = __ldg(in16 + w * 4 * C + i);
    } else {
      unsigned short *sw = reinterpret_cast<unsigned short *>(s4);
      for (int i = lane; i < np * C; i += 32) sw[i] = __ldg(in + p0 * C + i);
    }
    __syncwarp();
    for (int q = lane; q < np * Cp8; q += 32) {
      const int px = q / Cp8, c8 = q - px * Cp8;
      const unsigned short *src = s + px * C + c8 * 8;
      unsigned int wv[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (c8 * 8 + e < C) wv[e >> 1] |= (unsigned int)src[e] << ((e & 1) * 16);
      out[p0 * Cp8 + q] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    }
    __syncwarp();
  }
}

// Spatial pad by edge replication and spatial slice: one thread per output pixel and piece (16 bytes
// or one channel) of it.  T = uint4 (C % 8 == 0) or unsigned short.
//   pad:   out[ho][wo] = in[clamp(ho - top, 0, IH - 1)][clamp(wo - left, 0, IW - 1)]   (memory_pad.comp:71-72)
//   slice: out[h][w]   = in[h + top][w + left]                                         (memory_slice.comp:59-66)
template <class T, bool PAD>
__global__ void pad_or_slice(const T *__restrict__ in, T *__restrict__ out, int OH, int OW, int IH, int IW, int CT,
                             int left, int top) {
  const long long n = (long long)OH * OW * CT;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % CT);
    const long long p = i / CT;
    const int wo = (int)(p % OW), ho = (int)(p / OW);
    int hi, wi;
    if (PAD) {
      hi = min(max(ho - top, 0), IH - 1);
      wi = min(max(wo - left, 0), IW - 1);
    } else {
      hi = ho + top;
      wi = wo + left;
    }
    out[i] = in[((long long)hi * IW + wi) * CT + c];
  }
}

constexpr int kThreads = 256;

// Number of 16-byte (or 2-byte) items the dispatch writes.
long long item_count(const Variant &v, const dnxcu_dispatch &d) {
  const long long W = d.pc[0], H = d.pc[1];
  const int vec = v.p0;
  switch (v.kind) {
    case VK_POOL: return (H / 2) * (W / 2) * (d.c_a / vec);
    case VK_UPSAMPLE: return 4 * H * W * (d.c_a / vec);
    case VK_CONCAT: return H * W * ((d.c_a + d.c_b) / vec);
    case VK_RELU: return H * W * d.c_a / vec;
    case VK_PADC: return H * W * (d.c_out / 8);
    case VK_PAD_EDGE:
    case VK_SLICE: return H * W * (d.c_a / vec);
    default: return 0;
  }
}

int sm_count_cached() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

void mem_grid(const Variant &v, const dnxcu_dispatch &d, uint32_t g[3]) {
  const long long n = item_count(v, d);
  // whole waves of resident blocks: a multiple of the SM count, 8 blocks of 256 per SM at most
  const long long want = (n + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count_cached() * 8;
  long long blocks = want < cap ? want : cap;
  if (blocks < 1) blocks = 1;
  g[0] = (uint32_t)blocks;
  g[1] = g[2] = 1;
}

int mem_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s) {
  const int W = (int)d.pc[0], H = (int)d.pc[1];
  const int vec = v.p0;
  if (!d.in_a || !d.out || W <= 0 || H <= 0 || d.c_a <= 0) return DNXCU_E_BAD_ARG;
  if (v.kind == VK_CONCAT && (!d.in_b || d.c_b <= 0)) return DNXCU_E_BAD_ARG;
  if (vec == 8) {
    if (d.c_a % 8 || (v.kind == VK_CONCAT && d.c_b % 8)) {
      if (v.kind != VK_RELU || ((long long)H * W * d.c_a) % 8) return DNXCU_E_UNSUPPORTED;
    }
    if (((uintptr_t)d.in_a | (uintptr_t)d.out | (uintptr_t)d.in_b) & 15) return DNXCU_E_MISALIGNED;
  } else {
    if (((uintptr_t)d.in_a | (uintptr_t)d.out | (uintptr_t)d.in_b) & 1) return DNXCU_E_MISALIGNED;
  }
  if (v.kind == VK_POOL && (H < 2 || W < 2)) return DNXCU_E_BAD_ARG;
  if (v.kind == VK_PAD_EDGE || v.kind == VK_SLICE) {
    // W, H are the output extent here
    const bool pad = v.kind == VK_PAD_EDGE;
    const long long IW = pad ? (long long)W - d.pc_ext[0] - d.pc_ext[1] : d.pc_ext[2];
    const long long IH = pad ? (long long)H - d.pc_ext[2] - d.pc_ext[3] : d.pc_ext[3];
    if (IW <= 0 || IH <= 0) return DNXCU_E_BAD_ARG;
    if (!pad && ((long long)d.pc_ext[0] + W > IW || (long long)d.pc_ext[1] + H > IH)) return DNXCU_E_BAD_ARG;
    const int left = (int)d.pc_ext[0], top = pad ? (int)d.pc_ext[2] : (int)d.pc_ext[1];
    uint32_t gp[3];
    mem_grid(v, d, gp);
    if (vec == 8) {
      if (pad) pad_or_slice<uint4, true><<<gp[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, H, W, (int)IH, (int)IW, d.c_a / 8, left, top);
      else pad_or_slice<uint4, false><<<gp[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, H, W, (int)IH, (int)IW, d.c_a / 8, left, top);
    } else {
      if (pad) pad_or_slice<unsigned short, true><<<gp[0], kThreads, 0, s>>>((const unsigned short *)d.in_a, (unsigned short *)d.out, H, W, (int)IH, (int)IW, d.c_a, left, top);
      else pad_or_slice<unsigned short, false><<<gp[0], kThreads, 0, s>>>((const unsigned short *)d.in_a, (unsigned short *)d.out, H, W, (int)IH, (int)IW, d.c_a, left, top);
    }
    DNXCU_CUDA(cudaGetLastError());
    return DNXCU_OK;
  }
  if (v.kind == VK_PADC) {
    if (d.c_out < d.c_a || d.c_out % 8) return DNXCU_E_BAD_ARG;
    if (((uintptr_t)d.out & 15) || ((uintptr_t)d.in_a & 1)) return DNXCU_E_MISALIGNED;
    uint32_t gp[3];
    mem_grid(v, d, gp);
    const size_t warp_smem = (size_t)(kThreads / 32) * 64 * d.c_a;
    if (((uintptr_t)d.in_a & 15) == 0 && warp_smem <= 48 * 1024) {
      // (a grid of a few blocks per SM: every warp walks groups of 32 pixels)
      const long long groups = ((long long)H * W + 31) / 32;
      long long blocks = (groups + kThreads / 32 - 1) / (kThreads / 32);
      if (blocks > gp[0]) blocks = gp[0];
      pad_channels_warp<<<(unsigned)blocks, kThreads, warp_smem, s>>>((const unsigned short *)d.in_a, (uint4 *)d.out,
                                                                      (long long)H * W, d.c_a, d.c_out / 8);
    } else {
      pad_channels<<<gp[0], kThreads, 0, s>>>((const unsigned short *)d.in_a, (uint4 *)d.out, (long long)H * W, d.c_a,
                                              d.c_out / 8);
    }
    DNXCU_CUDA(cudaGetLastError());
    return DNXCU_OK;
  }
  uint32_t g[3];
  mem_grid(v, d, g);
  const long long P = (long long)H * W;
  switch (v.kind) {
    case VK_POOL:
      if (vec == 8) pool2x2_v8<<<g[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, H, W, d.c_a / 8);
      else pool2x2_s<<<g[0], kThreads, 0, s>>>((const __half *)d.in_a, (__half *)d.out, H, W, d.c_a);
      break;
    case VK_UPSAMPLE:
      if (vec == 8) upsample2x_v8<<<g[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, H, W, d.c_a / 8);
      else upsample2x_s<<<g[0], kThreads, 0, s>>>((const __half *)d.in_a, (__half *)d.out, H, W, d.c_a);
      break;
    case VK_CONCAT:
      if (vec == 8)
        concat_v8<<<g[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (const uint4 *)d.in_b, (uint4 *)d.out, P,
                                            d.c_a / 8, d.c_b / 8);
      else
        concat_s<<<g[0], kThreads, 0, s>>>((const __half *)d.in_a, (const __half *)d.in_b, (__half *)d.out, P,
                                           d.c_a, d.c_b);
      break;
    case VK_RELU: {
      const __half alpha = __float2half_rn(d.leaky_alpha);
      const bool leaky = d.flags & DNXCU_F_LEAKY;
      if (vec == 8) {
        if (leaky) relu_v8<true><<<g[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, P * d.c_a / 8, alpha);
        else relu_v8<false><<<g[0], kThreads, 0, s>>>((const uint4 *)d.in_a, (uint4 *)d.out, P * d.c_a / 8, alpha);
      } else {
        if (leaky) relu_s<true><<<g[0], kThreads, 0, s>>>((const __half *)d.in_a, (__half *)d.out, P * d.c_a, alpha);
        else relu_s<false><<<g[0], kThreads, 0, s>>>((const __half *)d.in_a, (__half *)d.out, P * d.c_a, alpha);
      }
      break;
    }
    default: return DNXCU_E_BAD_ARG;
  }
  DNXCU_CUDA(cudaGetLastError());
  return DNXCU_OK;
}

}  // namespace dnxcu
