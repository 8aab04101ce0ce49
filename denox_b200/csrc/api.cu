// C ABI: status strings, device capabilities, the variant table, dispatch
// validation / launch / cost, parameter re-layout.
#include "internal.h"
#include <string.h>
#include <stdio.h>
#include <atomic>
#include <new>

namespace dnxcu {

static thread_local int g_last_cuda_error = 0;
int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  cudaGetLastError();  // clear the sticky-free error so later calls start clean
  return DNXCU_E_CUDA;
}

// ---- SHA-256 ------------------------------------------------------------------
namespace {
const uint32_t Kc[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98,
    0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786,
    0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8,
    0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
    0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819,
    0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a,
    0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
    0xc67178f2};
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
void sha_block(uint32_t h[8], const unsigned char *p) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
  for (int i = 0; i < 64; ++i) {
    uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
    uint32_t t1 = hh + S1 + ch + Kc[i] + w[i];
    uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
    uint32_t t2 = S0 + mj;
    hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
}
}  // namespace

void sha256_hex(const void *data, size_t n, char out_hex[65]) {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  const unsigned char *p = (const unsigned char *)data;
  size_t i = 0;
  for (; i + 64 <= n; i += 64) sha_block(h, p + i);
  unsigned char tail[128];
  size_t r = n - i;
  memcpy(tail, p + i, r);
  tail[r++] = 0x80;
  size_t padded = r <= 56 ? 64 : 128;
  memset(tail + r, 0, padded - r);
  uint64_t bits = (uint64_t)n * 8;
  for (int k = 0; k < 8; ++k) tail[padded - 1 - k] = (unsigned char)(bits >> (8 * k));
  sha_block(h, tail);
  if (padded == 128) sha_block(h, tail + 64);
  for (int k = 0; k < 8; ++k) snprintf(out_hex + 8 * k, 9, "%08x", h[k]);
  out_hex[64] = 0;
}

// ---- bounded waits ------------------------------------------------------------
namespace {
constexpr unsigned long long kDefaultWaitCycles = 3000000000ull;  // about 1.5 s
std::atomic<unsigned long long> g_wait_limit_cycles{kDefaultWaitCycles};
}  // namespace
unsigned long long wait_limit_cycles() { return g_wait_limit_cycles.load(std::memory_order_relaxed); }

// ---- variant table ------------------------------------------------------------
// Digest of the kernel sources this library was built from (the build passes the SHA-256 of csrc/*.cu,
// csrc/*.h and the public header): part of every variant's identity, so a changed kernel invalidates the
// timings a benchmark database holds for it.
#ifndef DNXCU_SOURCE_DIGEST
#define DNXCU_SOURCE_DIGEST "unversioned-build"
#endif
static const char *kSourceRevision = DNXCU_SOURCE_DIGEST;

static const uint32_t CONV_BASE = DNXCU_F_RELU | DNXCU_F_BIAS | DNXCU_F_UP2X_A | DNXCU_F_LEAKY;
static const uint32_t CONV_ALL = CONV_BASE | DNXCU_F_POOL_OUT | DNXCU_F_NO_FULL_OUT;

static const Variant kVariants[] = {
    // id, op, family, config, flags, tcgen05, c_align, k_align, max_c_out | kind, p0..p3
    {{0, DNXCU_OP_CONV3X3, "direct-conv", "ACC=f32#TILE=16x8#KT=32", CONV_BASE, 0, 1, 1, 65536, 0}, VK_CONV_DIRECT, 0, 0, 0, 0},
    {{1, DNXCU_OP_CONV3X3, "direct-conv-tc", "R=1#KG=1#W=resident", CONV_BASE, 1, 1, 1, 256, 0}, VK_CONV_TC, 1, 1, 0, 0},
    {{2, DNXCU_OP_CONV3X3, "direct-conv-tc", "R=2#KG=1#W=resident", CONV_ALL, 1, 1, 1, 256, 0}, VK_CONV_TC, 2, 1, 0, 0},
    {{3, DNXCU_OP_CONV3X3, "direct-conv-tc", "R=4#KG=1#W=resident", CONV_ALL, 1, 1, 1, 128, 0}, VK_CONV_TC, 4, 1, 0, 0},
    {{4, DNXCU_OP_CONV3X3, "direct-conv-tc", "R=2#KG=1#W=stream3", CONV_ALL, 1, 1, 1, 256, 0}, VK_CONV_TC, 2, 1, 1, 3},
    {{5, DNXCU_OP_CONV3X3, "direct-conv-tc", "R=2#KG=2#W=stream3", CONV_ALL, 1, 1, 1, 256, 0}, VK_CONV_TC, 2, 2, 1, 3},
    {{6, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident", CONV_ALL, 1, 1, 1, 128, 0}, VK_CONV_TC, 0, 1, 0, 0},
    {{7, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident", CONV_ALL, 1, 1, 1, 128, 0}, VK_CONV_TC, 0, 2, 0, 0},
    {{8, DNXCU_OP_MAXPOOL2X2, "basic-pool", "VEC=8", 0, 0, 8, 1, 0, 0}, VK_POOL, 8, 0, 0, 0},
    {{9, DNXCU_OP_MAXPOOL2X2, "basic-pool", "VEC=1", 0, 0, 1, 1, 0, 0}, VK_POOL, 1, 0, 0, 0},
    {{10, DNXCU_OP_UPSAMPLE2X, "basic-upsample", "VEC=8", 0, 0, 8, 1, 0, 0}, VK_UPSAMPLE, 8, 0, 0, 0},
    {{11, DNXCU_OP_UPSAMPLE2X, "basic-upsample", "VEC=1", 0, 0, 1, 1, 0, 0}, VK_UPSAMPLE, 1, 0, 0, 0},
    {{12, DNXCU_OP_CONCAT, "copy-transform", "VEC=8", 0, 0, 8, 1, 0, 0}, VK_CONCAT, 8, 0, 0, 0},
    {{13, DNXCU_OP_CONCAT, "copy-transform", "VEC=1", 0, 0, 1, 1, 0, 0}, VK_CONCAT, 1, 0, 0, 0},
    {{14, DNXCU_OP_RELU, "basic-activation", "VEC=8", DNXCU_F_LEAKY, 0, 8, 1, 0, 0}, VK_RELU, 8, 0, 0, 0},
    {{15, DNXCU_OP_RELU, "basic-activation", "VEC=1", DNXCU_F_LEAKY, 0, 1, 1, 0, 0}, VK_RELU, 1, 0, 0, 0},
    {{16, DNXCU_OP_PAD_CHANNELS, "copy-transform", "PAD=8", 0, 0, 1, 8, 65536, 0}, VK_PADC, 1, 0, 0, 0},
    {{17, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=4#W=resident", CONV_ALL, 1, 1, 1, 128, 0}, VK_CONV_TC, 0, 4, 0, 0},
    {{18, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident#NSPLIT=2", CONV_ALL, 1, 1, 16, 256, 0}, VK_CONV_TC, 0, 2, 0, 2},
    {{19, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=4#W=resident#NSPLIT=2", CONV_ALL, 1, 1, 16, 256, 0}, VK_CONV_TC, 0, 4, 0, 2},
    {{20, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=4#W=resident#NSPLIT=3", CONV_ALL, 1, 1, 16, 256, 0}, VK_CONV_TC, 0, 4, 0, 3},
    {{21, DNXCU_OP_PAD_EDGE, "memory-pad", "VEC=8", 0, 0, 8, 1, 0, 0}, VK_PAD_EDGE, 8, 0, 0, 0},
    {{22, DNXCU_OP_PAD_EDGE, "memory-pad", "VEC=1", 0, 0, 1, 1, 0, 0}, VK_PAD_EDGE, 1, 0, 0, 0},
    {{23, DNXCU_OP_SLICE, "memory-slice", "VEC=8", 0, 0, 8, 1, 0, 0}, VK_SLICE, 8, 0, 0, 0},
    {{24, DNXCU_OP_SLICE, "memory-slice", "VEC=1", 0, 0, 1, 1, 0, 0}, VK_SLICE, 1, 0, 0, 0},
    {{25, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#PIPES=1", CONV_ALL, 1, 1, 1, 128, 0}, VK_CONV_TC, 0, 1, 2, 0},
    {{26, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident#NSPLIT=3", CONV_ALL, 1, 1, 16, 256, 0}, VK_CONV_TC, 0, 2, 0, 3},
    {{27, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident#NSPLIT=4", CONV_ALL, 1, 1, 16, 256, 0}, VK_CONV_TC, 0, 2, 0, 4},
    {{28, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#ER=2", CONV_ALL, 1, 8, 1, 128, 0}, VK_CONV_TC, 0, 1, 0, 0, 2},
    {{29, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#PIPES=1#ER=2", CONV_ALL, 1, 8, 1, 128, 0}, VK_CONV_TC, 0, 1, 2, 0, 2},
    {{30, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#CSPLIT=2", CONV_ALL, 1, 1, 8, 256, 0}, VK_CONV_TC, 0, 1, 0, 0, 0, 2},
    {{31, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#CSPLIT=3", CONV_ALL, 1, 1, 8, 256, 0}, VK_CONV_TC, 0, 1, 0, 0, 0, 3},
    {{32, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=1#W=resident#CSPLIT=4", CONV_ALL, 1, 1, 8, 256, 0}, VK_CONV_TC, 0, 1, 0, 0, 0, 4},
    {{33, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident#CSPLIT=2", CONV_ALL, 1, 1, 8, 256, 0}, VK_CONV_TC, 0, 2, 0, 0, 0, 2},
    {{34, DNXCU_OP_CONV3X3, "direct-conv-tc", "DY=stack#KG=2#W=resident#CSPLIT=4", CONV_ALL, 1, 1, 8, 256, 0}, VK_CONV_TC, 0, 2, 0, 0, 0, 4},
};
static const int kVariantCount = (int)(sizeof(kVariants) / sizeof(kVariants[0]));

const Variant *get_variant(int id) { return (id >= 0 && id < kVariantCount) ? &kVariants[id] : nullptr; }
int variant_count() { return kVariantCount; }

}  // namespace dnxcu

using namespace dnxcu;

extern "C" {

const char *dnxcu_status_string(int status) {
  switch (status) {
    case DNXCU_OK: return "ok";
    case DNXCU_E_BAD_ARG: return "bad argument";
    case DNXCU_E_UNSUPPORTED: return "variant does not support this dispatch";
    case DNXCU_E_MISALIGNED: return "misaligned pointer";
    case DNXCU_E_CUDA: return "CUDA call failed";
    case DNXCU_E_DEVICE: return "a kernel's bounded wait ran out";
    case DNXCU_E_NO_MEMORY: return "out of memory";
    case DNXCU_E_STATE: return "object in wrong state";
    case DNXCU_E_IO: return "file i/o failed";
    case DNXCU_E_LIMIT: return "capacity exceeded";
    default: return "unknown status";
  }
}

int dnxcu_last_cuda_error(void) { return g_last_cuda_error; }

int dnxcu_get_device_caps(int device, dnxcu_caps *caps) {
  if (!caps) return DNXCU_E_BAD_ARG;
  memset(caps, 0, sizeof(*caps));
  cudaDeviceProp p;
  DNXCU_CUDA(cudaGetDeviceProperties(&p, device));
  caps->device = device;
  caps->cc_major = p.major;
  caps->cc_minor = p.minor;
  caps->sm_count = p.multiProcessorCount;
  caps->max_threads_per_block = p.maxThreadsPerBlock;
  caps->tcgen05 = (p.major == 10) ? 1 : 0;
  caps->tmem_columns = caps->tcgen05 ? 512 : 0;
  caps->smem_per_block_optin = p.sharedMemPerBlockOptin;
  caps->l2_bytes = (uint64_t)p.l2CacheSize;
  caps->global_bytes = (uint64_t)p.totalGlobalMem;
  const size_t nlen = strnlen(p.name, sizeof(caps->name) - 1);
  memcpy(caps->name, p.name, nlen);
  caps->name[nlen] = 0;
  return DNXCU_OK;
}

int dnxcu_variant_count(void) { return kVariantCount; }
const dnxcu_variant_desc *dnxcu_variant(int id) {
  const Variant *v = get_variant(id);
  return v ? &v->desc : nullptr;
}
int dnxcu_find_variant(const char *family, const char *config) {
  if (!family || !config) return DNXCU_E_BAD_ARG;
  for (int i = 0; i < kVariantCount; ++i)
    if (!strcmp(kVariants[i].desc.family, family) && !strcmp(kVariants[i].desc.config, config)) return i;
  return DNXCU_E_BAD_ARG;
}
int dnxcu_variant_sha256(int id, char out_hex[65]) {
  const Variant *v = get_variant(id);
  if (!v || !out_hex) return DNXCU_E_BAD_ARG;
  char buf[512];
  int n = snprintf(buf, sizeof(buf), "%s\n%s\n%s\n", v->desc.family, v->desc.config, kSourceRevision);
  sha256_hex(buf, (size_t)n, out_hex);
  return DNXCU_OK;
}

int dnxcu_validate(const dnxcu_dispatch *d) {
  if (!d) return DNXCU_E_BAD_ARG;
  const Variant *v = get_variant(d->variant);
  if (!v) return DNXCU_E_BAD_ARG;
  if (d->flags & ~v->desc.allowed_flags) return DNXCU_E_UNSUPPORTED;
  if ((d->flags & DNXCU_F_RELU) && (d->flags & DNXCU_F_LEAKY)) return DNXCU_E_BAD_ARG;
  switch (v->kind) {
    case VK_CONV_DIRECT: return conv_direct_validate(*v, *d);
    case VK_CONV_TC: return conv_tc_validate(*v, *d);
    default:
      if (!d->in_a || !d->out || d->c_a <= 0 || !d->pc[0] || !d->pc[1]) return DNXCU_E_BAD_ARG;
      if (v->kind == VK_CONCAT && (!d->in_b || d->c_b <= 0)) return DNXCU_E_BAD_ARG;
      if (v->kind == VK_PAD_EDGE || v->kind == VK_SLICE) {
        const bool pad = v->kind == VK_PAD_EDGE;
        const long long iw = pad ? (long long)d->pc[0] - d->pc_ext[0] - d->pc_ext[1] : d->pc_ext[2];
        const long long ih = pad ? (long long)d->pc[1] - d->pc_ext[2] - d->pc_ext[3] : d->pc_ext[3];
        if (iw <= 0 || ih <= 0) return DNXCU_E_BAD_ARG;
        if (!pad && ((long long)d->pc_ext[0] + d->pc[0] > iw || (long long)d->pc_ext[1] + d->pc[1] > ih))
          return DNXCU_E_BAD_ARG;
      }
      if (v->kind == VK_PADC) {
        if (d->c_out < d->c_a || d->c_out % 8) return DNXCU_E_BAD_ARG;
        if (((uintptr_t)d->out & 15) || ((uintptr_t)d->in_a & 1)) return DNXCU_E_MISALIGNED;
        return DNXCU_OK;
      }
      if (v->p0 == 8) {
        if (v->kind == VK_RELU) {
          if (((uint64_t)d->pc[0] * d->pc[1] * d->c_a) % 8) return DNXCU_E_UNSUPPORTED;
        } else if (d->c_a % 8 || (v->kind == VK_CONCAT && d->c_b % 8)) {
          return DNXCU_E_UNSUPPORTED;
        }
        if (((uintptr_t)d->in_a | (uintptr_t)d->in_b | (uintptr_t)d->out) & 15) return DNXCU_E_MISALIGNED;
      }
      return DNXCU_OK;
  }
}

int dnxcu_launch(const dnxcu_dispatch *d, void *stream) {
  if (!d) return DNXCU_E_BAD_ARG;
  const Variant *v = get_variant(d->variant);
  if (!v) return DNXCU_E_BAD_ARG;
  if (d->flags & ~v->desc.allowed_flags) return DNXCU_E_UNSUPPORTED;
  if ((d->flags & DNXCU_F_RELU) && (d->flags & DNXCU_F_LEAKY)) return DNXCU_E_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  switch (v->kind) {
    case VK_CONV_DIRECT: return conv_direct_launch(*v, *d, s);
    case VK_CONV_TC: return conv_tc_launch(*v, *d, s);
    default: return mem_launch(*v, *d, s);
  }
}

int dnxcu_set_wait_limit_us(uint32_t us) {
  if (us == 0) {
    g_wait_limit_cycles.store(kDefaultWaitCycles, std::memory_order_relaxed);
    return DNXCU_OK;
  }
  int dev = 0, khz = 0;
  DNXCU_CUDA(cudaGetDevice(&dev));
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess || khz <= 0) khz = 1965000;
  g_wait_limit_cycles.store((unsigned long long)us * (unsigned long long)khz / 1000ull, std::memory_order_relaxed);
  return DNXCU_OK;
}

}  // extern "C"

// A planned dispatch.  Tensor core convs keep their launch parameters and encoded tensor maps; every other
// kernel family derives its launch from the dispatch record alone, which is kept as it is.
struct dnxcu_plan {
  dnxcu_dispatch d;
  const Variant *v = nullptr;
  ConvTcPlan *tc = nullptr;
};

extern "C" {

int dnxcu_plan_create(const dnxcu_dispatch *d, dnxcu_plan **out) {
  if (!d || !out) return DNXCU_E_BAD_ARG;
  int st = dnxcu_validate(d);
  if (st) return st;
  dnxcu_plan *p = new (std::nothrow) dnxcu_plan();
  if (!p) return DNXCU_E_NO_MEMORY;
  p->d = *d;
  p->v = get_variant(d->variant);
  if (p->v->kind == VK_CONV_TC) {
    st = conv_tc_plan(*p->v, *d, &p->tc);
    if (st) {
      delete p;
      return st;
    }
  }
  *out = p;
  return DNXCU_OK;
}

int dnxcu_plan_launch(const dnxcu_plan *p, void *stream) {
  if (!p || !p->v) return DNXCU_E_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  switch (p->v->kind) {
    case VK_CONV_DIRECT: return conv_direct_launch(*p->v, p->d, s);
    case VK_CONV_TC: return conv_tc_launch_plan(*p->tc, s);
    default: return mem_launch(*p->v, p->d, s);
  }
}

void dnxcu_plan_destroy(dnxcu_plan *p) {
  if (!p) return;
  if (p->tc) conv_tc_plan_free(p->tc);
  delete p;
}

int dnxcu_grid(const dnxcu_dispatch *d, uint32_t grid[3]) {
  if (!d || !grid) return DNXCU_E_BAD_ARG;
  const Variant *v = get_variant(d->variant);
  if (!v) return DNXCU_E_BAD_ARG;
  switch (v->kind) {
    case VK_CONV_DIRECT: conv_direct_grid(*v, *d, grid); break;
    case VK_CONV_TC: conv_tc_grid(*v, *d, grid); break;
    default: mem_grid(*v, *d, grid); break;
  }
  return DNXCU_OK;
}

// Unique tensor bytes in / out and flops, counted the way the reference fills
// memoryReads / memoryWrites / flops of a dispatch (DirectConvShaderCM.cpp:632-644,
// BasicPoolShader.cpp:603-604): no credit for padding, only tensors that cross HBM.
int dnxcu_cost(const dnxcu_dispatch *d, uint64_t *rd, uint64_t *wr, uint64_t *fl) {
  if (!d) return DNXCU_E_BAD_ARG;
  const Variant *v = get_variant(d->variant);
  if (!v) return DNXCU_E_BAD_ARG;
  const uint64_t W = d->pc[0], H = d->pc[1], P = W * H;
  uint64_t r = 0, w = 0, f = 0;
  switch (v->desc.op) {
    case DNXCU_OP_CONV3X3: {
      const uint64_t C = (uint64_t)d->c_a + d->c_b, K = d->c_out;
      const uint64_t pa = (d->flags & DNXCU_F_UP2X_A) ? P / 4 : P;
      r = 2 * (pa * d->c_a + P * d->c_b) + 2 * 9 * C * K;
      if (d->flags & DNXCU_F_BIAS) r += 2 * K;
      if (!(d->flags & DNXCU_F_NO_FULL_OUT)) w += 2 * P * K;
      if (d->flags & DNXCU_F_POOL_OUT) w += 2 * (P / 4) * K;
      f = 2 * P * 9 * C * K;
      break;
    }
    case DNXCU_OP_MAXPOOL2X2: r = 2 * P * d->c_a; w = 2 * (H / 2) * (W / 2) * d->c_a; break;
    case DNXCU_OP_UPSAMPLE2X: r = 2 * P * d->c_a; w = 8 * P * d->c_a; break;
    case DNXCU_OP_CONCAT: r = 2 * P * ((uint64_t)d->c_a + d->c_b); w = r; break;
    case DNXCU_OP_RELU: r = 2 * P * d->c_a; w = r; break;
    case DNXCU_OP_PAD_CHANNELS: r = 2 * P * d->c_a; w = 2 * P * d->c_out; break;
    case DNXCU_OP_PAD_EDGE:
      r = 2 * (uint64_t)(W - d->pc_ext[0] - d->pc_ext[1]) * (H - d->pc_ext[2] - d->pc_ext[3]) * d->c_a;
      w = 2 * P * d->c_a;
      break;
    case DNXCU_OP_SLICE: r = 2 * P * d->c_a; w = r; break;
    default: return DNXCU_E_BAD_ARG;
  }
  if (rd) *rd = r;
  if (wr) *wr = w;
  if (fl) *fl = f;
  return DNXCU_OK;
}

int dnxcu_prepare_weights(int variant, const void *kcrs_f16, int c_out, int c_a, int c_b, void *out, size_t *bytes) {
  const Variant *v = get_variant(variant);
  if (!v || v->desc.op != DNXCU_OP_CONV3X3 || c_out <= 0 || c_a <= 0 || c_b < 0 || !bytes) return DNXCU_E_BAD_ARG;
  const size_t need = v->kind == VK_CONV_TC ? conv_tc_weight_bytes(*v, c_out, c_a, c_b)
                                            : conv_direct_weight_bytes(*v, c_out, c_a, c_b);
  if (!out) {
    *bytes = need;
    return DNXCU_OK;
  }
  if (!kcrs_f16 || *bytes < need) return DNXCU_E_BAD_ARG;
  if (v->kind == VK_CONV_TC) conv_tc_prepare(*v, (const uint16_t *)kcrs_f16, c_out, c_a, c_b, (uint16_t *)out);
  else conv_direct_prepare(*v, (const uint16_t *)kcrs_f16, c_out, c_a, c_b, (uint16_t *)out);
  *bytes = need;
  return DNXCU_OK;
}

uint16_t dnxcu_f16_from_float(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u, mant = x & 0x007FFFFFu;
  const int32_t e = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  if (e <= 0) return (uint16_t)sign;
  if (e >= 31) return (uint16_t)(sign | 0x7C00u);
  return (uint16_t)(sign | ((uint32_t)e << 10) | (mant >> 13));
}

float dnxcu_f16_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
  if (e == 0) {
    if (m == 0) bits = sign;
    else {
      e = 1;
      while (!(m & 0x400)) { m <<= 1; --e; }
      m &= 0x3FF;
      bits = sign | ((e + 112) << 23) | (m << 13);
    }
  } else if (e == 31) {
    bits = sign | 0x7F800000u | (m << 13);
  } else {
    bits = sign | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

}  // extern "C"

#ifdef DNXCU_DEBUG_AIDS
// Development builds only (not part of the public header): hands the conv kernels a device buffer for their time
// line stamps, used while the environment variable DNXCU_TC_TRACE is 1; nullptr switches tracing off again.
namespace dnxcu {
int conv_tc_debug_trace_buffer(void *device_buffer, size_t bytes);
}
extern "C" DNXCU_API int dnxcu_debug_trace_buffer(void *device_buffer, size_t bytes) {
  return dnxcu::conv_tc_debug_trace_buffer(device_buffer, bytes);
}
#endif
