// Internal declarations shared by the translation units of libdnxcu.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include "dnxcu.h"

namespace dnxcu {

// Records a failing CUDA call for dnxcu_last_cuda_error and maps it to a status.
int cuda_fail(cudaError_t e);
#define DNXCU_CUDA(call)                                   \
  do {                                                     \
    cudaError_t _e = (call);                               \
    if (_e != cudaSuccess) return ::dnxcu::cuda_fail(_e);  \
  } while (0)

inline uint32_t cdiv(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

enum VariantKind {
  VK_CONV_DIRECT = 0,  // CUDA core implicit GEMM, fp32 accumulate
  VK_CONV_TC,          // tcgen05 / TMEM implicit GEMM, fp32 accumulate
  VK_POOL,
  VK_UPSAMPLE,
  VK_CONCAT,
  VK_RELU,
  VK_PADC,
  VK_PAD_EDGE,
  VK_SLICE,
};

struct Variant {
  dnxcu_variant_desc desc;
  VariantKind kind;
  // tuning parameters (meaning depends on kind)
  int p0, p1, p2, p3;
  int p4 = 0;
  int p5 = 0;
};

const Variant *get_variant(int id);
int variant_count();

// ---- per family entry points (each validates what only it knows) ----------
int conv_direct_validate(const Variant &v, const dnxcu_dispatch &d);
int conv_direct_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s);
void conv_direct_grid(const Variant &v, const dnxcu_dispatch &d, uint32_t g[3]);
size_t conv_direct_weight_bytes(const Variant &v, int k, int ca, int cb);
void conv_direct_prepare(const Variant &v, const uint16_t *kcrs, int k, int ca, int cb, uint16_t *out);

int conv_tc_validate(const Variant &v, const dnxcu_dispatch &d);
int conv_tc_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s);
// A tensor core conv dispatch planned once (launch parameters + encoded tensor maps), launched many times.
struct ConvTcPlan;
int conv_tc_plan(const Variant &v, const dnxcu_dispatch &d, ConvTcPlan **out);
int conv_tc_launch_plan(const ConvTcPlan &p, cudaStream_t s);
void conv_tc_plan_free(ConvTcPlan *p);
// Sets the per-kernel attributes of every tensor core kernel on the current device (idempotent).
int conv_tc_init_device();
void conv_tc_grid(const Variant &v, const dnxcu_dispatch &d, uint32_t g[3]);
size_t conv_tc_weight_bytes(const Variant &v, int k, int ca, int cb);
void conv_tc_prepare(const Variant &v, const uint16_t *kcrs, int k, int ca, int cb, uint16_t *out);

int mem_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s);
void mem_grid(const Variant &v, const dnxcu_dispatch &d, uint32_t g[3]);

// Limit of every bounded device-side wait in clock64 ticks (dnxcu_set_wait_limit_us).
unsigned long long wait_limit_cycles();

// SHA-256 (hex) of a byte string; used for variant identities and database keys.
void sha256_hex(const void *data, size_t n, char out_hex[65]);

}  // namespace dnxcu
