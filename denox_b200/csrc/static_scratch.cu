// conv3x3 (+bias, +ReLU) followed by a 2x2 max pool for callers that must not
// allocate device memory: the full resolution intermediate lives in a fixed,
// file-scope device array instead of a buffer from cudaMalloc.
#include "internal.h"

namespace dnxcu {
namespace {

// 8 MiB of binary16: the largest H x W x c_out intermediate this entry point takes.
constexpr size_t kScratchHalves = DNXCU_STATIC_SCRATCH_BYTES / 2;
static __device__ __align__(256) __half g_scratch[kScratchHalves];

constexpr int kMaxDevices = 64;
// Device address of g_scratch per device.  The symbol's name is only a host-side handle;
// the address a kernel can use comes from cudaGetSymbolAddress with that device current.
static void *g_scratch_addr[kMaxDevices] = {};

int scratch_for_current_device(void **out) {
  int dev = -1;
  DNXCU_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return DNXCU_E_LIMIT;
  if (!g_scratch_addr[dev]) {
    void *p = nullptr;
    DNXCU_CUDA(cudaGetSymbolAddress(&p, g_scratch));
    if (!p) return DNXCU_E_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DNXCU_OK;
}

}  // namespace
}  // namespace dnxcu

using namespace dnxcu;

extern "C" int dnxcu_conv3x3_pool_static(const void *in, int height, int width, int c_in, const void *weights,
                                         const void *bias, int c_out, uint32_t flags, void *out_pool, void *stream) {
  if (!in || !weights || !out_pool || height < 2 || width < 2 || c_in <= 0 || c_out <= 0) return DNXCU_E_BAD_ARG;
  if ((height | width) & 1) return DNXCU_E_BAD_ARG;
  if (flags & ~(DNXCU_F_RELU | DNXCU_F_BIAS)) return DNXCU_E_BAD_ARG;
  if ((flags & DNXCU_F_BIAS) && !bias) return DNXCU_E_BAD_ARG;
  if ((uint64_t)height * (uint64_t)width * (uint64_t)c_out > (uint64_t)kScratchHalves) return DNXCU_E_LIMIT;
  void *scratch = nullptr;
  int st = scratch_for_current_device(&scratch);
  if (st) return st;

  dnxcu_dispatch conv = {};
  conv.variant = dnxcu_find_variant("direct-conv", "ACC=f32#TILE=16x8#KT=32");  // runs every shape, never fuses the pool
  conv.flags = flags;
  conv.pc[0] = (uint32_t)width;
  conv.pc[1] = (uint32_t)height;
  conv.c_a = c_in;
  conv.c_out = c_out;
  conv.in_a = in;
  conv.out = scratch;
  conv.weights = weights;
  conv.bias = bias;
  st = dnxcu_launch(&conv, stream);
  if (st) return st;

  dnxcu_dispatch pool = {};
  pool.variant = dnxcu_find_variant("basic-pool", (c_out % 8 == 0 && ((uintptr_t)out_pool & 15) == 0) ? "VEC=8" : "VEC=1");
  pool.pc[0] = (uint32_t)width;
  pool.pc[1] = (uint32_t)height;
  pool.c_a = c_out;
  pool.in_a = scratch;
  pool.out = out_pool;
  return dnxcu_launch(&pool, stream);
}
