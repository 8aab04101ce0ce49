// "direct-conv-tc": 3x3 convolution (+bias, +ReLU, +2x2 max pool, over a concat
// of two operands, the first optionally read through a 2x nearest upsample) as
// an implicit GEMM on the sm_100a tensor cores: tcgen05.mma with fp32
// accumulators in tensor memory.  It replaces direct_conv_cm.comp and
// concat_conv_cm.comp of the reference
// (compiler/src/denox/compiler/implement/shaders/conv/), keeps their GEMM view
// (M = pixels, N = all output channels, K = taps x channels walked tap major,
// direct_conv_cm.comp:328-334) and their two phase concat (operand a's channels
// then operand b's into one accumulator, concat_conv_cm.comp:1042-1127).
//
// Shape of the computation
//   A persistent CTA (one per SM) walks work units.  A unit is a strip of 128
//   pixels in x times RB output rows.  Input rows stream through a ring of
//   shared memory slots (one slot = one input row of the strip: 130 pixels x
//   all channels), so every input row is fetched once per unit and reused by
//   the three vertical taps; the three horizontal taps are the same slot read
//   at a 16 byte offset.  One MMA covers M = 128 pixels of one output row.
//   R output rows form a pass: the pass walks the 9 taps once and issues, per
//   tap and per 16 channel step, R MMAs that share the weight tile.
//
// Shared memory operand layout (no swizzle, K major "core matrices" of 8 rows
// x 16 bytes): slot[chunk c8][pixel p][8 halves].  For an MMA the 8 row groups
// of M are 128 bytes apart (SBO) and the two 8 channel halves of a K=16 step
// are one chunk pitch apart (LBO).  Weights: w[tap][chunk c8][n][8 halves],
// SBO = 128, LBO = N*16.
//
// Warp roles (320 threads): warp 0 issues MMAs and owns the TMEM allocation,
// warp 1 moves weights with bulk async copies, warps 2-5 are the epilogue
// (TMEM -> registers -> ReLU / pool -> global), warps 6-9 fill the input slots
// with 16 byte cp.async (zero fill = conv padding; the upsample is the address
// map src = dst / 2, basic_upsample.comp:49-56).
//
// Every wait on an mbarrier is bounded: when a wait runs out the kernel raises
// a CTA wide abort flag, stores a code to the dispatch's device_status word
// and every role leaves its loop; TMEM is freed on that path too.
#include "internal.h"
#include <cuda.h>
#include <atomic>
#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace dnxcu {
namespace {

constexpr int STRIP = 128;        // pixels per MMA (M)
constexpr int SLOT_PX = 130;      // pixels used per slot row (strip + 1 left + 1 right)
constexpr int WH = 132;           // slot pixel pitch = TMA box width: two chunks = 4224 B, a multiple of 128
constexpr int CHUNK_PITCH = WH * 16;
constexpr int SW_PX = 136;                 // pixels per row of a swizzled block (the box of its tensor map)
constexpr int SW_BLOCK = SW_PX * 64;       // 32 channels x 136 pixels: 8704 bytes = 17 x 512
constexpr int SW_CHUNK = SW_BLOCK / 4;     // per 8 channel chunk of such a block
constexpr int HEADER_BYTES = 1024;
constexpr int MAX_SLOTS = 16;
constexpr int MAX_GROUPS = 4;
constexpr int MAX_DEPTH = 8;      // input rows a producer thread keeps in flight
constexpr int MAX_WST = 4;
constexpr int N_PRODUCER = 128;
constexpr int THREADS = 320;

// barrier indices inside the header
constexpr int BAR_FULL = 0;                   // [MAX_SLOTS] slot filled (4 producer warps arrive)
constexpr int BAR_EMPTY = BAR_FULL + MAX_SLOTS;   // [MAX_SLOTS] slot free (tcgen05.commit)
constexpr int BAR_TFULL = BAR_EMPTY + MAX_SLOTS;  // [2] accumulator set complete (tcgen05.commit)
constexpr int BAR_TEMPTY = BAR_TFULL + 2;         // [2] accumulator set drained (4 epilogue warps)
constexpr int BAR_WFULL = BAR_TEMPTY + 2;         // [MAX_WST] weight stage landed
constexpr int BAR_WEMPTY = BAR_WFULL + MAX_WST;   // [MAX_WST] weight stage consumed
constexpr int BAR_WRES = BAR_WEMPTY + MAX_WST;    // resident weights landed
constexpr int BAR_COUNT = BAR_WRES + 1;
static_assert(BAR_COUNT * 8 + 16 <= HEADER_BYTES, "header too small");
constexpr int OFF_TMEM_PTR = BAR_COUNT * 8;
constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;  // int abort flag, then the 64-bit wait limit

struct Seg {
  const __half *ptr;  // H x W x C (or (H/2) x (W/2) x C when up)
  const __half *top;  // row above the band or nullptr
  const __half *bot;  // row below the band or nullptr
  int C;              // channels
  int nch;            // 8 channel chunks after padding C to a multiple of 16
  int up;
  int tma;            // rows of this operand are fetched by TMA (tensor map below)
  int tbox;           // 8 channel chunks per TMA copy (box extent of the tensor map's chunk dimension)
  int rg;             // ragged operand (C not a multiple of 8, at most 16 channels): its rows are fetched as raw
                      // bytes by a bulk copy and re-laid into the chunk layout inside shared memory
  int sw;             // pixel major slot layout with 64 byte swizzled rows of 32 channels ("blocks") for this operand
  int dup;            // 2x upsampled operand whose tensor map has a pixel doubling dimension of stride 0: the copy
                      // engine writes every half resolution pixel twice, i.e. the upsampled row itself
};

struct TcArgs {
  // 4-D views of the operands for TMA: (8 channels, pixel x, 8 channel chunk, row y), so that a box of
  // (8, 132, 2, 1) lands in shared memory as [chunk][pixel][8 halves] — the MMA's K major core matrix order
  alignas(64) CUtensorMap tm_a;
  alignas(64) CUtensorMap tm_b;
  alignas(64) CUtensorMap tm_out;  // (channels, x, y) view of the full resolution output, box (K, 32, 1)
  // the halo rows of a row band (one row tensors of their own): a above, a below, b above, b below
  alignas(64) CUtensorMap tm_halo[4];
  Seg a, b;
  const __half *w;  // [9][nch_a + nch_b][N][8]
  const __half *bias;
  __half *out;
  __half *out_pool;
  int *status;
  int H, W, K, N, Ns;
  int os;  // halves between consecutive pixels of the outputs (= K unless the output channels are split over launches)
  int relu, pool, full_out;  // relu: an activation follows the sum (ReLU, or LeakyReLU when leaky is set)
  int leaky;                 // the activation is max(x, alpha * x) in binary16
  uint32_t alpha_h2;         // alpha as a binary16 pair
  int RB, S, nstrips, nunits;
  // Stacked form, "cut" units (cut_L > 0): the rows of all strips, strip after strip, are cut into cut_R ranges of
  // cut_L rows, one per pipeline of a CTA.  A range that crosses from one strip into the next makes two units;
  // those ranges (cut_nb of them, indices cut_x[], ascending) go to the first lanes, so unit u < lanes is the
  // first part of lane u's range and unit lanes + i the second part of lane i's.
  // The ranges are cut in a row count that has cut_pad extra rows between two strips, so a range that crosses
  // (two more halo rows and a restart of the pipeline) gets that many rows less.
  int cut_L, cut_R, cut_nb, cut_pad;
  short cut_x[32];
  int wstream, WST;
  int G;                 // K groups: 1 = rolling row window; > 1 = every pass loads its rows once per group
  int gc0[MAX_GROUPS];   // first 8 channel chunk of each group
  int gch[MAX_GROUPS];   // chunks in each group (even)
  int gmax;              // largest group
  int D;                 // producer depth (rows in flight per thread)
  int cpa;               // producer warps copy part of the rows (cp.async) besides TMA
  int NB;                // stacked form: accumulator blocks in the TMEM ring (per pipeline)
  int P;                 // stacked form: pipelines per CTA (1 or 2)
  int ER;                // stacked form: input rows per ring entry (1, or 2: one wait, one descriptor, one slot release per two rows)
  int xp;                // stacked form: operand a (2x upsampled) comes by TMA at half resolution and is expanded in shared memory
  uint32_t src_bytes;    // expand mode: bytes of one half resolution staging buffer (one per slot)
  int stage_pitch;       // stacked form: bytes per pixel row of an epilogue warp's staging tile, 0 = direct stores
  int stage2;            // stacked form: two staging tiles per epilogue warp (a row pair is staged in one go)
  int out_tma;           // stacked form: staged rows leave by one tensor copy per warp and row (shared -> global) from an
                         // unpadded, swizzled tile: 1 = 128 byte pixel rows (64 channels), 2 = 64 byte rows (32 channels)
  uint32_t stage_warp_bytes;  // staging bytes per epilogue warp
  uint32_t tmem_cols;
  int parts;       // launches of this dispatch that run side by side (output channel split): each plans for 1/parts of the SMs
  int ab;          // stacked form, one pipeline: two MMA warps issue alternate entries (see the kernel)
  int eteams;      // stacked form: epilogue teams per pipeline (2: one pipeline, the teams take alternate items)
  // Stacked form, the A operand of the K steps of an entry (16 channels each), in K order: start address offset from
  // the entry's slot row (>> 4, with the descriptor's leading byte offset bits), descriptor high word (stride byte
  // offset, version, swizzle mode) and start address step per horizontal tap (>> 4).  Two slot layouts exist:
  // [8 channel chunk][132 pixels][16 bytes] without swizzle, and, for operands of whole 32 channel blocks that
  // come by TMA, [block][136 pixels][64 bytes] with the 64 byte swizzle (pixel major: the copy engine moves one
  // box row per cycle, and these rows are four times as long).
  uint32_t kst_lo[16], kst_hi[16], kst_dx[16];
  // The TMA copies of an entry, per K group, worked out by the host: where the box lands in the slot row, which
  // operand, and its chunk or block coordinate.  (The feeding thread is a single thread: what it has to compute per
  // entry is time the slots wait.)
  struct Copy {
    uint32_t dst;
    short unit;
    unsigned char sg, pad;
  } cp[MAX_GROUPS][8];
  int ncp[MAX_GROUPS];
  uint32_t grp_tx[MAX_GROUPS];  // bytes the copies of one row of the group bring
  uint32_t row_bytes;  // bytes of one input row (of one K group) in a slot
  uint32_t seg_off[2]; // one K group: byte offset of each operand's area in the slot row
  int swmode;          // some operand uses the swizzled layout
  int shift;       // stacked form: the slots hold pixels x0 - 2 .. x0 + 129 instead of x0 - 1 .. x0 + 130 (a row that
                   // comes through a pixel doubling map starts on an even pixel), so the MMAs read one pixel further
  int cparts;      // stacked form: output channel parts inside ONE launch (blockIdx.y): part p computes channels
                   // [p * N, p * N + N) from its own weight blob; K is then the dispatch's whole channel count
  unsigned long long wait_limit;  // clock64 ticks after which a barrier wait gives up (see mbar_wait)
#ifdef DNXCU_DEBUG_AIDS
  int desc_swap;     // exchange the two descriptor strides
  long long *trace;  // per role time stamps of CTA 0 (nullptr = off)
  int switch_issue;  // the straight line form is chosen per row even with one K group
  int loop_issue;    // MMAs issued by the generic loops instead of the straight line code
  int skip;          // timing only, results wrong: 1 no input loads, 2 no MMAs, 4 no output stores
#endif
};

// Development aids (time line tracing, switching loads / MMAs / stores off for timing experiments) exist only in
// builds made with -DDNXCU_DEBUG_AIDS.  A normal build compiles them out: the macros below are constants, so no
// kernel carries the fields or the tests, and nothing reads the environment.
#ifdef DNXCU_DEBUG_AIDS
#define DBG_SKIP(g) ((g).skip)
#define DBG_DESC_SWAP(g) ((g).desc_swap)
#define DBG_SWITCH_ISSUE(g) ((g).switch_issue)
#define DBG_LOOP_ISSUE(g) ((g).loop_issue)
#define DBG_TRACE_ON(g) ((g).trace != nullptr)
#else
#define DBG_SKIP(g) 0
#define DBG_DESC_SWAP(g) 0
#define DBG_SWITCH_ISSUE(g) 0
#define DBG_LOOP_ISSUE(g) 0
#define DBG_TRACE_ON(g) false
#endif

// ---- PTX wrappers ---------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another ran out).
// SLEEP_NS > 0: back off between polls, so that a waiting warp does not take issue
// slots from the warps that share its scheduler (the MMA issuer above all).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code) {
  if (mbar_test_wait(bar, parity)) return true;  // the cheap probe: about half the cost of try_wait when it passes
  const unsigned long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    const bool done = mbar_try_wait(bar, parity);
    if (done || (it & 63u) == 1u) {  // after the first probe that came back empty handed, then every 64th
      if (!done && *abort_flag) return false;
      // The limit (clock64 ticks) sits in the header right behind the abort flag, written once at kernel start.
      // Its top bit marks a limit below a millisecond (test use): a probe may itself suspend the thread for
      // microseconds, so with such a limit a wait that was over it when it came true counts as run out too, and
      // the limit is honoured whatever the probe does.  With ordinary limits a wait that came true has succeeded.
      const unsigned long long raw = *reinterpret_cast<const volatile unsigned long long *>(abort_flag + 1);
      if (done && !(raw >> 63)) return true;
      if ((unsigned long long)clock64() - t0 > (raw & ~(1ull << 63))) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
      if (done) return true;
    }
  }
}
// After a wait ran out every role has left its loop, but copies into shared memory and MMAs that were started
// before may still be in flight.  The block stays for a fixed, bounded time (far longer than a copy or an MMA
// takes) before it frees its tensor memory and ends, so that nothing lands in memory it no longer owns.
__device__ __forceinline__ void abort_drain(volatile int *abort_flag) {
  if (*abort_flag) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
    __syncthreads();
  }
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// 4-D tiled TMA load, global -> shared, completion counted in bytes on an mbarrier.
// Brings a tensor map into the descriptor cache ahead of its first use.
__device__ __forceinline__ void tma_prefetch_map(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void *tmap, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], "
      "[%7];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void *tmap, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], "
      "[%6];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Zeroes `ncols` (a multiple of 16) columns of the calling warp's 32 TMEM lanes.
__device__ __forceinline__ void tc_zero_cols(uint32_t taddr, int ncols) {
  const uint32_t z = 0u;
  int c0 = 0;
#pragma unroll 1
  for (; c0 + 32 <= ncols; c0 += 32)
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
        "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr + (uint32_t)c0),
        "r"(z)
        : "memory");
  if (c0 < ncols)
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(
            taddr + (uint32_t)c0),
        "r"(z)
        : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hmax2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// The activation on a pair of finished, rounded sums: max(x, 0), or max(x, alpha * x) with the product rounded
// to binary16 (direct_conv_cm.comp:1061-1076).
__device__ __forceinline__ uint32_t activate_h2(uint32_t p, int leaky, uint32_t alpha_h2) {
  return leaky ? hmax2_u32(p, hmul2_u32(alpha_h2, p)) : hmax2_u32(p, 0u);
}
// The same on one fp32 sum; the result is the binary16 value as a float.
__device__ __forceinline__ float activate_f(float v, int leaky, uint32_t alpha_h2) {
  if (!leaky) return fmaxf(v, 0.0f);
  const __half h = __float2half_rn(v);
  const __half a = __ushort_as_half((unsigned short)(alpha_h2 & 0xffffu));
  return __half2float(__hmax(h, __hmul(a, h)));
}

// Debug time line: role `role` of CTA 0 stores clock64() at event `ev` of its n-th iteration.
#ifdef DNXCU_DEBUG_AIDS
constexpr int TRACE_ITERS = 64, TRACE_EVENTS = 6;
constexpr int TRACE_CTAS = 1024;
// behind the role stamps: CTA 0's kernel entry, set-up done, roles done (clock64), entry and end (globaltimer); then
// per CTA (the first TRACE_CTAS) its cycles from entry to roles done and its entry time (globaltimer)
constexpr int TRACE_EXTRA = 8 + 2 * TRACE_CTAS;
#endif
__device__ __forceinline__ void trace(const TcArgs &g, int role, int n, int ev) {
#ifdef DNXCU_DEBUG_AIDS
  if (g.trace && blockIdx.x == 0 && blockIdx.y == 0 && n < TRACE_ITERS) g.trace[(role * TRACE_ITERS + n) * TRACE_EVENTS + ev] = clock64();
#else
  (void)g; (void)role; (void)n; (void)ev;
#endif
}

struct Unit {
  int x0, y0, npass;
};
template <int R>
__device__ __forceinline__ Unit unit_of(const TcArgs &g, int u) {
  Unit t;
  const int strip = u % g.nstrips, rb = u / g.nstrips;
  t.x0 = strip * STRIP;
  t.y0 = rb * g.RB;
  int rows = g.H - t.y0;
  if (rows > g.RB) rows = g.RB;
  t.npass = (rows + R - 1) / R;
  return t;
}

__device__ __forceinline__ void cp_async_wait_dyn(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    case 4: cp_async_wait<4>(); break;
    case 5: cp_async_wait<5>(); break;
    case 6: cp_async_wait<6>(); break;
    default: cp_async_wait<7>(); break;
  }
}

// True when TMA fetches this operand's part of input row iy (otherwise the
// producer warps copy it): the operand has a tensor map and the row is not one
// of the separately stored halo rows of a row band.
__device__ __forceinline__ bool row_by_tma(const TcArgs &g, const Seg &s, int iy) {
  if (!s.tma && !s.rg) return false;
  // halo rows of a TMA operand come by TMA too (tensor maps of their own); a ragged operand's by the producer warps
  if (iy == -1 && s.top) return s.tma != 0;
  if (iy == g.H && s.bot) return s.tma != 0;
  return true;
}

// Tensor map and row coordinate for input row iy of operand sg (0: a, 1: b): the operand itself, or the one row
// tensor that holds the row above / below a row band.  `row` is the coordinate inside the operand (iy, or iy / 2
// for an operand read through the 2x upsample).
__device__ __forceinline__ bool banded(const TcArgs &g) { return g.a.top || g.a.bot || g.b.top || g.b.bot; }
__device__ __forceinline__ const void *tmap_of(const TcArgs &g, int sg, int iy, int row, int *y) {
  const Seg &s = sg ? g.b : g.a;
  if (iy == -1 && s.top) {
    *y = 0;
    return &g.tm_halo[sg * 2];
  }
  if (iy == g.H && s.bot) {
    *y = 0;
    return &g.tm_halo[sg * 2 + 1];
  }
  *y = row;
  return sg ? (const void *)&g.tm_b : (const void *)&g.tm_a;
}

// Raw byte span of a ragged operand's row for the strip starting at x0 (pixels x0-1 .. x0+128 clipped to the
// image): the first fetched pixel, the 16 byte aligned source address, the bytes in front of the first pixel
// and the copy size (a multiple of 16; the tensor's byte size is one too, so the copy stays inside it).
struct RawSpan {
  const unsigned char *src;
  int xs;          // first pixel fetched
  uint32_t lead;   // bytes between the aligned source address and pixel xs
  uint32_t bytes;  // copy size
};
__device__ __forceinline__ RawSpan raw_span(const TcArgs &g, const Seg &s, int iy, int x0) {
  RawSpan r;
  r.xs = max(x0 - 1, 0);
  const int xe = min(x0 + STRIP + 1, g.W);
  const size_t start = ((size_t)iy * g.W + r.xs) * (size_t)s.C * 2u;
  const unsigned char *p = reinterpret_cast<const unsigned char *>(s.ptr) + start;
  r.lead = (uint32_t)(reinterpret_cast<uintptr_t>(p) & 15u);
  r.src = p - r.lead;
  r.bytes = (r.lead + (uint32_t)(xe - r.xs) * (uint32_t)s.C * 2u + 15u) & ~15u;
  return r;
}

// TMA part of one ring entry: chunks [c_lo, c_hi) of input row iy, pixels x0-1 ..
// x0+130, two 8 channel chunks per copy.  Rows and pixels outside the tensor
// are zero filled by the copy engine (= the convolution's zero padding).
// Returns the bytes that will land.
template <bool ISSUE>
__device__ __forceinline__ uint32_t tma_row(const TcArgs &g, uint32_t slot_addr, int iy, int x0, int c_lo, int c_hi,
                                            uint32_t bar) {
  uint32_t bytes = 0;
  int chbase = 0;
#pragma unroll 1
  for (int sg = 0; sg < 2; ++sg) {
    const Seg &s = sg ? g.b : g.a;
    if (s.nch == 0) continue;
    const int lo = max(c_lo - chbase, 0), hi = min(c_hi - chbase, s.nch);
    if (hi > lo && s.tma && row_by_tma(g, s, iy)) {
      int y = iy;
      const void *tm = sg ? (const void *)&g.tm_b : (const void *)&g.tm_a;
      if (banded(g)) tm = tmap_of(g, sg, iy, iy, &y);
#pragma unroll 1
      for (int c = lo; c < hi; c += s.tbox) {
        if (ISSUE) tma_load_4d(slot_addr + (uint32_t)((chbase + c - c_lo) * CHUNK_PITCH), tm, 0, x0 - 1, c, y, bar);
        bytes += (uint32_t)s.tbox * CHUNK_PITCH;
      }
    }
    chbase += s.nch;
  }
  return bytes;
}

// Producer warp part of one ring entry: the operands (or halo rows) TMA does not
// cover, with 16 byte cp.async (2 byte loads for channel counts that are not a
// multiple of 8).  Chunk c of the operand list lands at slot chunk c - c_lo.
__device__ __forceinline__ void load_row(const TcArgs &g, uint32_t slot_addr, int iy, int x0, int tid, int nprod,
                                         int c_lo, int c_hi) {
  int chbase = 0;
#pragma unroll 1
  for (int sg = 0; sg < 2; ++sg) {
    const Seg &s = sg ? g.b : g.a;
    if (s.nch == 0) continue;
    const int lo = max(c_lo - chbase, 0), hi = min(c_hi - chbase, s.nch);
    if (hi > lo && !row_by_tma(g, s, iy)) {
      const int n = hi - lo;
      const int Ws = s.up ? g.W >> 1 : g.W;
      const __half *row = nullptr;
      if (iy < 0) row = (iy == -1) ? s.top : nullptr;
      else if (iy >= g.H) row = (iy == g.H) ? s.bot : nullptr;
      else row = s.ptr + (long long)(s.up ? iy >> 1 : iy) * Ws * s.C;
      const bool vec = (s.C & 7) == 0;
      const int nchv = s.C >> 3;
      const uint32_t dst0 = slot_addr + (uint32_t)((chbase + lo - c_lo) * CHUNK_PITCH);
      // a thread owns pixels tid, tid + nprod, ... and walks the chunks of each (no division in the loop)
#pragma unroll 1
      for (int px = tid; px < SLOT_PX; px += nprod) {
        const int ix = x0 - 1 + px;
        const bool inb = row != nullptr && ix >= 0 && ix < g.W;
        const __half *src = inb ? row + (long long)(s.up ? ix >> 1 : ix) * s.C + lo * 8 : s.ptr;
        uint32_t dst = dst0 + (uint32_t)(px * 16);
        if (vec) {
#pragma unroll 2
          for (int ch = 0; ch < n; ++ch) {
            const bool ok = inb && (lo + ch) < nchv;
            cp_async16(dst, ok ? (const void *)(src + ch * 8) : (const void *)s.ptr, ok ? 16u : 0u);
            dst += CHUNK_PITCH;
          }
        } else {
#pragma unroll 1
          for (int ch = 0; ch < n; ++ch) {
            uint32_t v[4] = {0u, 0u, 0u, 0u};
            if (inb) {
              const unsigned short *p = reinterpret_cast<const unsigned short *>(src + ch * 8);
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if ((lo + ch) * 8 + e < s.C) v[e >> 1] |= (uint32_t)__ldg(p + e) << ((e & 1) * 16);
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                         "r"(v[3])
                         : "memory");
            dst += CHUNK_PITCH;
          }
        }
      }
    }
    chbase += s.nch;
  }
}

// Epilogue of NC accumulator columns [c0, c0 + NC) for RSTEP output rows of one
// pixel: TMEM -> registers, (+bias), (ReLU), binary16, stores; with RSTEP == 2
// optionally the 2x2 max pool (vertical max in registers, horizontal max with
// the neighbouring lane; max commutes with the rounding, basic_pool.comp:44-82).
template <int NC, int RSTEP>
__device__ __forceinline__ void epilogue_block(const TcArgs &g, uint32_t t0, uint32_t t1, int c0, int x, int y,
                                               bool xin, int lane) {
  uint32_t v0[NC], v1[RSTEP == 2 ? NC : 1];
  if constexpr (NC == 32) {
    tc_ld32(t0 + (uint32_t)c0, v0);
    if constexpr (RSTEP == 2) tc_ld32(t1 + (uint32_t)c0, v1);
  } else {
    tc_ld16(t0 + (uint32_t)c0, v0);
    if constexpr (RSTEP == 2) tc_ld16(t1 + (uint32_t)c0, v1);
  }
  tc_wait_ld();
  const bool vec_out = (g.K & 7) == 0;
  const bool row1 = RSTEP == 2 && (y + 1 < g.H);
  const bool do_pool = RSTEP == 2 && g.pool;
  __half *o0 = g.out + ((long long)y * g.W + x) * g.K + c0;
  __half *o1 = o0 + (long long)g.W * g.K;
  __half *op = g.out_pool + ((long long)(y >> 1) * (g.W >> 1) + (x >> 1)) * g.K + c0;
  const bool st_full = g.full_out && xin && !(DBG_SKIP(g) & 4);
  const bool st_pool = do_pool && xin && !(lane & 1) && row1;
#pragma unroll
  for (int j8 = 0; j8 < NC; j8 += 8) {
    float f0[8], f1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float bj = 0.0f;
      if (g.bias && c0 + j8 + j < g.K) bj = __half2float(__ldg(g.bias + c0 + j8 + j));
      f0[j] = __uint_as_float(v0[j8 + j]) + bj;
      if (g.relu) f0[j] = activate_f(f0[j], g.leaky, g.alpha_h2);
      if constexpr (RSTEP == 2) {
        f1[j] = __uint_as_float(v1[j8 + j]) + bj;
        if (g.relu) f1[j] = activate_f(f1[j], g.leaky, g.alpha_h2);
      } else {
        f1[j] = 0.0f;
      }
    }
    const bool whole = vec_out && (c0 + j8 + 8 <= g.K);
    if (st_full) {
      if (whole) {
        *reinterpret_cast<uint4 *>(o0 + j8) =
            make_uint4(pack_h2(f0[0], f0[1]), pack_h2(f0[2], f0[3]), pack_h2(f0[4], f0[5]), pack_h2(f0[6], f0[7]));
        if (row1)
          *reinterpret_cast<uint4 *>(o1 + j8) =
              make_uint4(pack_h2(f1[0], f1[1]), pack_h2(f1[2], f1[3]), pack_h2(f1[4], f1[5]), pack_h2(f1[6], f1[7]));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c0 + j8 + j < g.K) {
            o0[j8 + j] = __float2half_rn(f0[j]);
            if (row1) o1[j8 + j] = __float2half_rn(f1[j]);
          }
      }
    }
    if (do_pool) {
      float pm[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float vmax = fmaxf(f0[j], f1[j]);
        pm[j] = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 1));
      }
      if (st_pool) {
        if (whole) {
          *reinterpret_cast<uint4 *>(op + j8) =
              make_uint4(pack_h2(pm[0], pm[1]), pack_h2(pm[2], pm[3]), pack_h2(pm[4], pm[5]), pack_h2(pm[6], pm[7]));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c0 + j8 + j < g.K) op[j8 + j] = __float2half_rn(pm[j]);
        }
      }
    }
  }
}

template <int R>
__global__ void __launch_bounds__(THREADS, 1) conv3x3_tc(const __grid_constant__ TcArgs g) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + OFF_ABORT);
  volatile uint32_t *tmem_ptr = reinterpret_cast<volatile uint32_t *>(smem + OFF_TMEM_PTR);
  auto bar = [&](int i) { return sbase + (uint32_t)i * 8u; };

  const int nch = g.a.nch + g.b.nch;
  const uint32_t wtap_bytes = (uint32_t)nch * g.N * 16u;        // one tap, all chunks
  const uint32_t wstage_bytes = (uint32_t)g.gmax * g.N * 16u;   // one (tap, group) block
  const uint32_t w_addr = sbase + HEADER_BYTES;
  const uint32_t wregion = g.wstream ? wstage_bytes * g.WST : wtap_bytes * 9u;
  const uint32_t slot_bytes = (uint32_t)g.gmax * CHUNK_PITCH;
  const uint32_t slots_addr = w_addr + ((wregion + 127u) & ~127u);
  const int S = g.S;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *reinterpret_cast<volatile unsigned long long *>(abort_flag + 1) = g.wait_limit;
    // a slot is full when the TMA bytes have landed (one arrival with the byte count by the
    // issuing thread) and, when producer warps copy part of the rows, those four warps arrived
    const uint32_t full_count = g.cpa ? 5u : 1u;
    for (int i = 0; i < MAX_SLOTS; ++i) {
      mbar_init(bar(BAR_FULL + i), full_count);
      mbar_init(bar(BAR_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_TFULL + i), 1);
      mbar_init(bar(BAR_TEMPTY + i), 4);
    }
    for (int i = 0; i < MAX_WST; ++i) {
      mbar_init(bar(BAR_WFULL + i), 1);
      mbar_init(bar(BAR_WEMPTY + i), 1);
    }
    mbar_init(bar(BAR_WRES), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + OFF_TMEM_PTR),
                 "r"(g.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  // Ring bookkeeping shared by the producer and the MMA issuer: entry number `pos`
  // (0, 1, 2, ... in load order) lives in slot pos % S with phase (pos / S) & 1.
  // G == 1: the entries of a unit are its input rows y0-1 .. y0+rows, loaded once
  //         and reused by up to three passes (rolling window).
  // G  > 1: every (pass, group) loads its own R + 2 rows (no reuse across passes).

  if (warp == 0) {
    // ---------------- MMA issue ----------------
    // The whole warp walks the loop (uniform control flow keeps the descriptors in
    // uniform registers); lane 0 alone issues the tcgen05 instructions.
    const bool issuer = lane == 0;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(g.N >> 3) << 17) | ((uint32_t)(STRIP >> 4) << 24);
    const uint32_t a_lbo = DBG_DESC_SWAP(g) ? 128u : (uint32_t)CHUNK_PITCH;
    const uint32_t a_sbo = DBG_DESC_SWAP(g) ? (uint32_t)CHUNK_PITCH : 128u;
    const uint32_t b_lbo = DBG_DESC_SWAP(g) ? 128u : (uint32_t)g.N * 16u;
    const uint32_t b_sbo = DBG_DESC_SWAP(g) ? (uint32_t)g.N * 16u : 128u;
    // descriptor = hi word (stride offset + version, constant) : lo word (start address + leading offset)
    const uint32_t a_hi = (a_sbo >> 4) | (1u << 14), b_hi = (b_sbo >> 4) | (1u << 14);
    const uint32_t a_lo0 = (a_lbo >> 4) << 16, b_lo0 = (b_lbo >> 4) << 16;
    const uint32_t kstep_a = (2u * CHUNK_PITCH) >> 4, kstep_b = (2u * (uint32_t)g.N * 16u) >> 4;
    bool ok = true;
    if (!g.wstream) ok = mbar_wait(bar(BAR_WRES), 0, abort_flag, g.status, 1);
    int pos_base = 0;  // ring position of the current unit's first entry (G == 1) / next entry (G > 1)
    int gpass = 0, gw = 0;
    for (int u = blockIdx.x; ok && u < g.nunits; u += gridDim.x) {
      const Unit t = unit_of<R>(g, u);
      int waited = 0;  // G == 1: entries of this unit already waited for
      for (int p = 0; ok && p < t.npass; ++p) {
        const int set = gpass & 1;
        if (issuer) trace(g, 0, gpass, 0);
        ok = mbar_wait(bar(BAR_TEMPTY + set), ((uint32_t)(gpass >> 1) & 1u) ^ 1u, abort_flag, g.status, 3);
        if (!ok) break;
        if (issuer) trace(g, 0, gpass, 1);
        for (int gi = 0; ok && gi < g.G; ++gi) {
          int first;  // ring position of input row (pass row 0, dy = 0)
          if (g.G == 1) {
            first = pos_base + p * R;
            const int need = p * R + R + 1;
            while (ok && waited <= need) {
              const int gg = pos_base + waited;
              ok = mbar_wait(bar(BAR_FULL + gg % S), (uint32_t)(gg / S) & 1u, abort_flag, g.status, 2);
              ++waited;
            }
          } else {
            first = pos_base;
            for (int q = 0; ok && q < R + 2; ++q) {
              const int gg = pos_base + q;
              ok = mbar_wait(bar(BAR_FULL + gg % S), (uint32_t)(gg / S) & 1u, abort_flag, g.status, 2);
            }
          }
          if (!ok) break;
          if (issuer) trace(g, 0, gpass, 2);
          tc_fence_after();
          uint32_t row_lo[R + 2];
#pragma unroll
          for (int q = 0; q < R + 2; ++q)
            row_lo[q] = (((slots_addr + (uint32_t)((first + q) % S) * slot_bytes) & 0x3FFFFu) >> 4) | a_lo0;
          const int nk16 = g.gch[gi] >> 1;
          const uint32_t wgrp = (uint32_t)g.gc0[gi] * g.N * 16u;
          // The tap loop is unrolled so that the row word (dy) and the pixel offset (dx) are
          // compile time: per MMA the issuing thread spends one add on the descriptor.
#pragma unroll
          for (int tap = 0; tap < 9; ++tap) {
            const int dy = tap / 3, dx = tap - dy * 3;
            uint32_t wb;
            int ws = 0;
            if (g.wstream) {
              if (!ok) continue;
              ws = gw % g.WST;
              ok = mbar_wait(bar(BAR_WFULL + ws), (uint32_t)(gw / g.WST) & 1u, abort_flag, g.status, 4);
              if (!ok) continue;
              tc_fence_after();
              wb = w_addr + (uint32_t)ws * wstage_bytes;
            } else {
              wb = w_addr + (uint32_t)tap * wtap_bytes + wgrp;
            }
            uint32_t b_lo = ((wb & 0x3FFFFu) >> 4) | b_lo0;
            uint32_t a_off = (uint32_t)dx;  // 16 bytes per pixel
            uint32_t acc = (gi | tap) == 0 ? 0u : 1u;
#pragma unroll 1
            for (int kc = 0; kc < nk16; ++kc) {
              if (issuer && !(DBG_SKIP(g) & 2)) {
                const uint64_t bdesc = ((uint64_t)b_hi << 32) | b_lo;
#pragma unroll
                for (int r = 0; r < R; ++r)
                  tc_mma(tmem_base + (uint32_t)((set * R + r) * g.Ns), ((uint64_t)a_hi << 32) | (row_lo[r + dy] + a_off),
                         bdesc, idesc, acc);
              }
              acc = 1u;
              b_lo += kstep_b;
              a_off += kstep_a;
            }
            if (g.wstream) {
              if (issuer) tc_commit(bar(BAR_WEMPTY + ws));
              ++gw;
            }
          }
          if (!ok) break;
          if (g.G > 1) {
            if (issuer)
              for (int q = 0; q < R + 2; ++q) tc_commit(bar(BAR_EMPTY + (pos_base + q) % S));
            pos_base += R + 2;
          }
        }
        if (!ok) break;
        if (issuer) {
          trace(g, 0, gpass, 3);
          tc_commit(bar(BAR_TFULL + set));
          if (g.G == 1) {
            const int nrel = (p == t.npass - 1) ? R + 2 : R;
            for (int q = 0; q < nrel; ++q) tc_commit(bar(BAR_EMPTY + (pos_base + p * R + q) % S));
          }
          trace(g, 0, gpass, 4);
        }
        ++gpass;
      }
      if (g.G == 1) pos_base += t.npass * R + 2;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- weights ----------------
    if (lane == 0) {
      const unsigned char *wsrc = reinterpret_cast<const unsigned char *>(g.w);
      if (!g.wstream) {
        mbar_expect_tx(bar(BAR_WRES), wtap_bytes * 9u);
        for (int tap = 0; tap < 9; ++tap)
          bulk_g2s(w_addr + (uint32_t)tap * wtap_bytes, wsrc + (size_t)tap * wtap_bytes, wtap_bytes, bar(BAR_WRES));
      } else {
        bool ok = true;
        int gw = 0;
        for (int u = blockIdx.x; ok && u < g.nunits; u += gridDim.x) {
          const Unit t = unit_of<R>(g, u);
          for (int p = 0; ok && p < t.npass; ++p)
            for (int gi = 0; ok && gi < g.G; ++gi) {
              const uint32_t bytes = (uint32_t)g.gch[gi] * g.N * 16u;
              const size_t goff = (size_t)g.gc0[gi] * g.N * 16u;
              for (int tap = 0; ok && tap < 9; ++tap) {
                const int ws = gw % g.WST;
                ok = mbar_wait<64>(bar(BAR_WEMPTY + ws), ((uint32_t)(gw / g.WST) & 1u) ^ 1u, abort_flag, g.status, 5);
                if (!ok) break;
                mbar_expect_tx(bar(BAR_WFULL + ws), bytes);
                bulk_g2s(w_addr + (uint32_t)ws * wstage_bytes, wsrc + (size_t)tap * wtap_bytes + goff, bytes,
                         bar(BAR_WFULL + ws));
                ++gw;
              }
            }
        }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------- epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int m = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    bool ok = true;
    int gpass = 0;
    for (int u = blockIdx.x; ok && u < g.nunits; u += gridDim.x) {
      const Unit t = unit_of<R>(g, u);
      const int x = t.x0 + m;
      const bool xin = x < g.W;
      for (int p = 0; ok && p < t.npass; ++p) {
        const int set = gpass & 1;
        if (threadIdx.x == 64) trace(g, 1, gpass, 0);
        ok = mbar_wait<64>(bar(BAR_TFULL + set), (uint32_t)(gpass >> 1) & 1u, abort_flag, g.status, 6);
        if (!ok) break;
        if (threadIdx.x == 64) trace(g, 1, gpass, 1);
        tc_fence_after();
        const int yb = t.y0 + p * R;
        constexpr int RSTEP = (R >= 2) ? 2 : 1;
#pragma unroll
        for (int r = 0; r < R; r += RSTEP) {
          const int y = yb + r;
          const uint32_t t0 = lane_addr + (uint32_t)((set * R + r) * g.Ns);
          const uint32_t t1 = t0 + (uint32_t)g.Ns;
          // rows past the image are computed but never stored
          const bool yin = xin && y < g.H;
          int c0 = 0;
#pragma unroll 1
          for (; c0 + 32 <= g.N; c0 += 32) epilogue_block<32, RSTEP>(g, t0, t1, c0, x, y, yin, lane);
          if (c0 < g.N) epilogue_block<16, RSTEP>(g, t0, t1, c0, x, y, yin, lane);
        }
        if (threadIdx.x == 64) trace(g, 1, gpass, 2);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BAR_TEMPTY + set));
        if (threadIdx.x == 64) trace(g, 1, gpass, 3);
        ++gpass;
      }
    }
  } else {
    // ---------------- input slots ----------------
    // Thread 0 of the producer warps issues the TMA copies of an entry and arrives on
    // the slot's barrier with their byte count.  When some rows need the producer warps
    // (upsampled operand, channel count not a multiple of 8, halo rows of a row band)
    // all 128 threads walk the entries: each keeps up to D rows of cp.async in flight
    // and signals entry pos - D + 1 after issuing entry pos.
    const int tid = threadIdx.x - 6 * 32;
    bool ok = true;
    int pos = 0;        // entries issued
    int signalled = 0;  // entries signalled full by the producer warps
    const int D = g.D;
    auto emit = [&](int iy, int x0, int c_lo, int c_hi) {
      const int slot = pos % S;
      if (tid == 0) trace(g, 2, pos, 0);
      ok = mbar_wait<64>(bar(BAR_EMPTY + slot), ((uint32_t)(pos / S) & 1u) ^ 1u, abort_flag, g.status, 7);
      if (!ok) return;
      if (tid == 0) trace(g, 2, pos, 1);
      const uint32_t slot_addr = slots_addr + (uint32_t)slot * slot_bytes;
      if (tid == 0) {
        const uint32_t fb = bar(BAR_FULL + slot);
        // announce the byte count first, then start the copies
        const uint32_t bytes = (DBG_SKIP(g) & 1) ? 0u : tma_row<false>(g, slot_addr, iy, x0, c_lo, c_hi, fb);
        if (bytes) {
          mbar_expect_tx(fb, bytes);
          tma_row<true>(g, slot_addr, iy, x0, c_lo, c_hi, fb);
        } else {
          mbar_arrive(fb);
        }
      }
      if (g.cpa) {
        if (!(DBG_SKIP(g) & 1)) load_row(g, slot_addr, iy, x0, tid, N_PRODUCER, c_lo, c_hi);
        cp_async_commit();
        if (tid == 0) trace(g, 2, pos, 2);
        ++pos;
        if (pos - signalled >= D) {
          cp_async_wait_dyn(D - 1);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(BAR_FULL + signalled % S));
          ++signalled;
        }
      } else {
        if (tid == 0) trace(g, 2, pos, 2);
        ++pos;
      }
    };
    if (g.cpa || tid == 0) {
      for (int u = blockIdx.x; ok && u < g.nunits; u += gridDim.x) {
        const Unit t = unit_of<R>(g, u);
        if (g.G == 1) {
          const int rows_in = t.npass * R + 2;
          for (int j = 0; ok && j < rows_in; ++j) emit(t.y0 - 1 + j, t.x0, 0, nch);
        } else {
          for (int p = 0; ok && p < t.npass; ++p)
            for (int gi = 0; ok && gi < g.G; ++gi)
              for (int q = 0; ok && q < R + 2; ++q)
                emit(t.y0 - 1 + p * R + q, t.x0, g.gc0[gi], g.gc0[gi] + g.gch[gi]);
        }
      }
      if (g.cpa) {
        cp_async_wait<0>();
        if (ok) {
          fence_proxy_async();
          __syncwarp();
          if (lane == 0)
            for (; signalled < pos; ++signalled) mbar_arrive(bar(BAR_FULL + signalled % S));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  abort_drain(abort_flag);
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(g.tmem_cols) : "memory");
  }
}

// Epilogue of the stacked kernel, specialised at compile time on what the dispatch
// needs (EPI bits: 1 bias, 2 ReLU, 4 pooled output, 8 full resolution output) so
// that no flag is tested per value.  Values are rounded to binary16 pairs first;
// ReLU and the 2x2 max then work on packed pairs (max commutes with the rounding).
constexpr int EPI_BIAS = 1, EPI_RELU = 2, EPI_POOL = 4, EPI_FULL = 8;

// What differs between the output channel parts of one launch (TcArgs::cparts): the part's first channel is
// folded into the pointers, K is the number of valid channels of the part.
struct OutPart {
  const __half *bias;
  __half *out;
  __half *out_pool;
  int K;
};

template <int NC, int EPI>
__device__ __forceinline__ void round_row(const TcArgs &g, const OutPart &o, const uint32_t (&v)[NC], int c0,
                                          uint32_t (&h)[NC / 2]) {
#pragma unroll
  for (int j = 0; j < NC; j += 2) {
    float lo = __uint_as_float(v[j]), hi = __uint_as_float(v[j + 1]);
    if (EPI & EPI_BIAS) {
      lo += (c0 + j < o.K) ? __half2float(__ldg(o.bias + c0 + j)) : 0.0f;
      hi += (c0 + j + 1 < o.K) ? __half2float(__ldg(o.bias + c0 + j + 1)) : 0.0f;
    }
    uint32_t p = pack_h2(lo, hi);
    if (EPI & EPI_RELU) p = activate_h2(p, g.leaky, g.alpha_h2);
    h[j / 2] = p;
  }
}

// Stores NC channels [c0, c0 + NC) of one pixel from packed pairs.
template <int NC>
__device__ __forceinline__ void store_row(int K, __half *o, const uint32_t (&h)[NC / 2], int c0) {
  if ((K & 7) == 0) {
#pragma unroll
    for (int j8 = 0; j8 < NC; j8 += 8)
      if (c0 + j8 + 8 <= K)
        *reinterpret_cast<uint4 *>(o + j8) = make_uint4(h[j8 / 2], h[j8 / 2 + 1], h[j8 / 2 + 2], h[j8 / 2 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < NC; ++j)
      if (c0 + j < K) {
        const uint32_t p = h[j / 2];
        reinterpret_cast<unsigned short *>(o)[j] = (unsigned short)((j & 1) ? (p >> 16) : (p & 0xffffu));
      }
  }
}

struct NoRelease {
  __device__ __forceinline__ void operator()() const {}
};
// `rel` runs as soon as the accumulators are in registers (a layer of at most 32 channels hands its TMEM blocks back
// there, before the conversion and the stores: the ring of blocks is what couples MMA and epilogue in thin layers).
template <int NC, int RSTEP, int EPI, class Rel = NoRelease>
__device__ __forceinline__ void epi_fast(const TcArgs &g, const OutPart &o, uint32_t t0, uint32_t t1, int c0, int x,
                                         int y, bool xin, int lane, Rel rel = Rel()) {
  uint32_t v0[NC], v1[RSTEP == 2 ? NC : 2];
  if constexpr (NC == 32) {
    tc_ld32(t0 + (uint32_t)c0, v0);
    if constexpr (RSTEP == 2) tc_ld32(t1 + (uint32_t)c0, v1);
  } else {
    tc_ld16(t0 + (uint32_t)c0, v0);
    if constexpr (RSTEP == 2) tc_ld16(t1 + (uint32_t)c0, v1);
  }
  tc_wait_ld();
  rel();
  if (DBG_SKIP(g) & 16) return;
  if (DBG_SKIP(g) & 4) xin = false;
  uint32_t h0[NC / 2], h1[RSTEP == 2 ? NC / 2 : 1];
  round_row<NC, EPI>(g, o, v0, c0, h0);
  if constexpr (RSTEP == 2) round_row<NC, EPI>(g, o, v1, c0, h1);
  const bool row1 = RSTEP == 2 && (y + 1 < g.H);
  if (EPI & EPI_FULL) {
    if (xin) {
      __half *o0 = o.out + ((long long)y * g.W + x) * g.os + c0;
      store_row<NC>(o.K, o0, h0, c0);
      if constexpr (RSTEP == 2) {
        if (row1) store_row<NC>(o.K, o0 + (long long)g.W * g.os, h1, c0);
      }
    }
  }
  if constexpr (RSTEP == 2 && (EPI & EPI_POOL) != 0) {
    uint32_t pm[NC / 2];
#pragma unroll
    for (int j = 0; j < NC / 2; ++j) {
      const uint32_t vm = hmax2_u32(h0[j], h1[j]);
      pm[j] = hmax2_u32(vm, __shfl_xor_sync(0xffffffffu, vm, 1));
    }
    if (xin && !(lane & 1) && row1)
      store_row<NC>(o.K, o.out_pool + ((long long)(y >> 1) * (g.W >> 1) + (x >> 1)) * g.os + c0, pm, c0);
  }
}

// ============================================================================
// Stacked form ("DY=stack"): one pass per INPUT row.  The three vertical taps are
// stacked along N: for input row j, horizontal tap dx and a 16 channel step, one
// MMA with N' = 3N multiplies the row's pixels with [W(r=2) | W(r=1) | W(r=0)] and
// adds into the accumulators of output rows j-1, j, j+1, which sit side by side
// in a ring of TMEM blocks.  The A tile (4 KB per MMA, the operand that bounds
// thin layers: its fetch from shared memory costs more than the math for N < 128)
// is read three times per input row instead of nine.
//   - block ring: output row number ob (counted over the CTA's whole life) uses
//     TMEM block ob % NB, columns [block * N, block * N + N)
//   - an output row is complete after input row y+1: commit -> tfull[block]
//   - every MMA accumulates: the epilogue zeroes a block (tcgen05.st) after its last
//     read and hands it back zeroed; all blocks are zeroed once at kernel start
//   - runs of blocks are split where the ring wraps and where N' would exceed 256
//   - an input slot is released as soon as its own row's MMAs are committed
// Warp roles (512 threads): warps 0..P-1 issue the MMAs of pipeline 0..P-1 (one thread
// each, or two that take alternate entries: the partner of a single pipeline's thread
// is in warp 15, the partners of two pipelines are in the producer warps 11 and 13 when
// every operand comes by TMA; warp 0 owns the TMEM allocation); warp 1 also moves the weights and, with one
// pipeline in expand mode, issues the TMA copies; warps 2..2+4P-1 are the epilogue teams
// (four warps per pipeline, one TMEM lane quarter each); warps 10-13 fill the input
// slots; warps 14, 15 hold the descriptor threads (one thread per pipeline), which work
// out, per entry, what the MMA thread needs and write it to shared memory.
constexpr int ST_THREADS = 512;
constexpr int ST_MAX_BLOCKS = 16;
constexpr int ST_BAR_FULL = 0;
constexpr int ST_BAR_EMPTY = ST_BAR_FULL + MAX_SLOTS;
constexpr int ST_BAR_TFULL = ST_BAR_EMPTY + MAX_SLOTS;
constexpr int ST_BAR_TEMPTY = ST_BAR_TFULL + ST_MAX_BLOCKS;
constexpr int ST_BAR_WRES = ST_BAR_TEMPTY + ST_MAX_BLOCKS;
constexpr int ST_BAR_RAW = ST_BAR_WRES + 1;  // [MAX_SLOTS] expand mode: TMA data of an entry landed (before the expansion)
constexpr int ST_BAR_COUNT = ST_BAR_RAW + MAX_SLOTS;
static_assert(ST_BAR_COUNT * 8 + 16 <= HEADER_BYTES, "header too small");
constexpr int ST_OFF_TMEM_PTR = ST_BAR_COUNT * 8;
constexpr int ST_OFF_ABORT = ST_OFF_TMEM_PTR + 4;   // int abort flag, then the 64-bit wait limit
constexpr int ST_OFF_TURN = ST_OFF_ABORT + 12;      // entries issued so far (two alternating MMA threads), one word per pipeline
static_assert(ST_OFF_TURN + 8 <= HEADER_BYTES, "header too small");
// entry descriptors, one per slot (index: pipeline's barrier offset + slot), written by the descriptor threads
constexpr int ST_SUBDESC_BYTES = 48;                  // one input row
constexpr int ST_DESC_BYTES = 2 * ST_SUBDESC_BYTES;   // an entry holds one or two input rows (TcArgs::ER)
constexpr int ST_OFF_DESC = HEADER_BYTES;
constexpr int ST_HEADER_BYTES = HEADER_BYTES + MAX_SLOTS * ST_DESC_BYTES;
static_assert(ST_HEADER_BYTES % 128 == 0, "weights must start on a 128 byte boundary");
// descriptor flag word: bits 0-3 K steps of 16, then
constexpr uint32_t DF_NR2 = 1u << 4, DF_PENULT = 1u << 6, DF_LAST = 1u << 7;

// The stacked kernel's MMA warps run their loop with all lanes (so that two of them can meet at a named
// barrier); only the lane with `leader` set issues.
__device__ __forceinline__ void tc_mma_e(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t leader) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, e;\n\t"
      "setp.ne.b32 p, 1, 0;\n\t"
      "setp.ne.b32 e, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(leader)
      : "memory");
}
__device__ __forceinline__ void tc_commit_e(uint32_t bar, uint32_t leader) {
  asm volatile(
      "{\n\t"
      ".reg .pred e;\n\t"
      "setp.ne.b32 e, %1, 0;\n\t"
      "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(bar),
      "r"(leader)
      : "memory");
}

struct StUnit {
  int x0, y0, rows_out;
};
__device__ __forceinline__ StUnit st_unit_of(const TcArgs &g, int u) {
  StUnit t;
  if (g.cut_L > 0) {
    const int second = u >= g.cut_R ? 1 : 0;
    const int lane = second ? u - g.cut_R : u;
    int r;
    if (lane < g.cut_nb) {
      r = g.cut_x[lane];
    } else {
      r = lane - g.cut_nb;  // the (lane - cut_nb)-th range that stays inside one strip
      for (int i = 0; i < g.cut_nb; ++i)
        if (g.cut_x[i] <= r) ++r;
    }
    const int Hp = g.H + g.cut_pad;
    const int v0 = r * g.cut_L, v1 = min(v0 + g.cut_L, g.nstrips * Hp - g.cut_pad);
    int s0 = v0 / Hp, y0 = v0 - s0 * Hp;       // first row of the range (one that starts in the padding starts the next strip)
    if (y0 >= g.H) { ++s0; y0 = 0; }
    int s1 = (v1 - 1) / Hp, y1 = (v1 - 1) - s1 * Hp;  // last row
    if (y1 >= g.H) y1 = g.H - 1;
    if (!second) {
      t.x0 = s0 * STRIP;
      t.y0 = y0;
      t.rows_out = (s1 == s0 ? y1 + 1 : g.H) - y0;
    } else {
      t.x0 = s1 * STRIP;
      t.y0 = 0;
      t.rows_out = y1 + 1;
    }
    return t;
  }
  const int strip = u % g.nstrips, rb = u / g.nstrips;
  t.x0 = strip * STRIP;
  t.y0 = rb * g.RB;
  t.rows_out = min(g.RB, g.H - t.y0);
  return t;
}

struct Run {
  uint32_t col;    // first TMEM column
  uint32_t boff;   // byte offset of the run's first weight row inside a stacked chunk, >> 4
  uint32_t idesc;  // instruction descriptor with this run's N'
  uint32_t acc;    // 1: in use (accumulates), 2: unused
};

// The MMAs of one input row (all horizontal taps, NK K steps, NR runs of TMEM blocks) as straight
// line code.  Every instruction gets descriptor registers of its own, so the issuing thread keeps
// several MMAs in flight; a loop that reuses the registers issues three times slower (measured).
template <int NK, int NR>
__device__ __forceinline__ void st_issue_row(const TcArgs &g, uint32_t hi, uint32_t row_lo, uint32_t b_lo, uint32_t wdx16,
                                             uint32_t kstep_b, const Run &r0, const Run &r1, uint32_t leader) {
#pragma unroll
  for (int dx = 0; dx < 3; ++dx) {
#pragma unroll
    for (int kc = 0; kc < NK; ++kc) {
      const uint32_t a = row_lo + g.kst_lo[kc] + (uint32_t)dx * g.kst_dx[kc];
      const uint64_t ahi = (uint64_t)g.kst_hi[kc] << 32;
      const uint32_t b = b_lo + (uint32_t)dx * wdx16 + (uint32_t)kc * kstep_b;
      tc_mma_e(r0.col, ahi | a, ((uint64_t)hi << 32) | (b + r0.boff), r0.idesc, leader);
      if (NR == 2) tc_mma_e(r1.col, ahi | a, ((uint64_t)hi << 32) | (b + r1.boff), r1.idesc, leader);
    }
  }
}
template <int V>
struct IntC {
  static constexpr int value = V;
};
template <int NR>
__device__ __forceinline__ bool st_issue_nk(const TcArgs &g, int nk, uint32_t hi, uint32_t row_lo, uint32_t b_lo,
                                            uint32_t wdx16, uint32_t kstep_b, const Run &r0, const Run &r1, uint32_t leader) {
  switch (nk) {
    case 1: st_issue_row<1, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 2: st_issue_row<2, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 3: st_issue_row<3, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 4: st_issue_row<4, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 5: st_issue_row<5, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 6: st_issue_row<6, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 7: st_issue_row<7, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    case 8: st_issue_row<8, NR>(g, hi, row_lo, b_lo, wdx16, kstep_b, r0, r1, leader); return true;
    default: return false;
  }
}

// ---- staged epilogue --------------------------------------------------------
// A thread owns one pixel after tcgen05.ld, so direct stores put 32 lanes on 32
// different cache lines (measured: about 170 cycles per store instruction, 2700 of the
// 3600 cycles of a two row item at 64 channels).  Instead each epilogue warp parks its
// 32 pixels x K channels in a padded shared memory tile (pitch K*2 + 16 bytes: conflict
// free for 16 byte accesses) and copies it out with consecutive lanes on consecutive 16
// byte pieces (512 contiguous bytes per instruction; HWC keeps the 32 pixels contiguous).
// The 2x2 max pool is taken while copying out, from the two staged rows.

// TMEM -> registers -> (+bias) -> binary16 pairs -> (ReLU) -> this lane's pixel row of the staging tile
template <int NC, int EPI>
__device__ __forceinline__ void stage_cols(const TcArgs &g, const OutPart &o, uint32_t taddr, int c0, uint32_t dst, uint32_t xr) {
  uint32_t v[NC];
  if constexpr (NC == 32) tc_ld32(taddr + (uint32_t)c0, v);
  else tc_ld16(taddr + (uint32_t)c0, v);
  tc_wait_ld();
  uint32_t h[NC / 2];
  round_row<NC, EPI>(g, o, v, c0, h);
#pragma unroll
  for (int j8 = 0; j8 < NC; j8 += 8)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + ((uint32_t)((c0 + j8) * 2) ^ xr)), "r"(h[j8 / 2]),
                 "r"(h[j8 / 2 + 1]), "r"(h[j8 / 2 + 2]), "r"(h[j8 / 2 + 3])
                 : "memory");
}

// The same for one chunk of two rows: both TMEM loads are under way before the thread waits for either.
template <int NC, int EPI, class Rel = NoRelease>
__device__ __forceinline__ void stage_cols2(const TcArgs &g, const OutPart &o, uint32_t taddr0, uint32_t taddr1, int c0,
                                            uint32_t dst0, uint32_t dst1, uint32_t xr, Rel rel = Rel()) {
  uint32_t v0[NC], v1[NC];
  if constexpr (NC == 32) {
    tc_ld32(taddr0 + (uint32_t)c0, v0);
    tc_ld32(taddr1 + (uint32_t)c0, v1);
  } else {
    tc_ld16(taddr0 + (uint32_t)c0, v0);
    tc_ld16(taddr1 + (uint32_t)c0, v1);
  }
  tc_wait_ld();
  rel();
  uint32_t h[NC / 2];
  round_row<NC, EPI>(g, o, v0, c0, h);
#pragma unroll
  for (int j8 = 0; j8 < NC; j8 += 8)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 + ((uint32_t)((c0 + j8) * 2) ^ xr)), "r"(h[j8 / 2]),
                 "r"(h[j8 / 2 + 1]), "r"(h[j8 / 2 + 2]), "r"(h[j8 / 2 + 3])
                 : "memory");
  round_row<NC, EPI>(g, o, v1, c0, h);
#pragma unroll
  for (int j8 = 0; j8 < NC; j8 += 8)
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst1 + ((uint32_t)((c0 + j8) * 2) ^ xr)), "r"(h[j8 / 2]),
                 "r"(h[j8 / 2 + 1]), "r"(h[j8 / 2 + 2]), "r"(h[j8 / 2 + 3])
                 : "memory");
}

__device__ __forceinline__ void sts16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// Copies `npx` staged pixels (K channels each) to `dst` (contiguous), lanes on consecutive 16 byte pieces.
__device__ __forceinline__ void copy_out(uint32_t tile, int pitch, int nck, int os8, int npx, __half *dst, int lane) {
  const int total = npx * nck;
  int px = lane / nck, ch = lane - px * nck;
  const int dpx = 32 / nck, dch = 32 - dpx * nck;
  uint4 *o = reinterpret_cast<uint4 *>(dst);
  // two pieces per lane and round: both loads are under way before the first store waits for its data (one at a
  // time, every piece pays the shared memory latency by itself; more at a time cost registers the epilogue lacks)
  for (int i = lane; i < total; i += 64) {
    const int at0 = px * os8 + ch;
    const uint4 v0 = lds16(tile + (uint32_t)(px * pitch + ch * 16));
    px += dpx;
    ch += dch;
    if (ch >= nck) { ch -= nck; ++px; }
    const bool two = i + 32 < total;
    const int at1 = px * os8 + ch;
    uint4 v1 = v0;
    if (two) v1 = lds16(tile + (uint32_t)(px * pitch + ch * 16));
    px += dpx;
    ch += dch;
    if (ch >= nck) { ch -= nck; ++px; }
    o[at0] = v0;
    if (two) o[at1] = v1;
  }
}

// A warp's staged row (32 pixels x K channels, swizzled like the tensor map says) to global memory through the
// copy engine; pixels right of the image are dropped by the copy.  (The channel coordinate is 0: 16 byte rule.)
__device__ __forceinline__ void tma_store_3d(const void *tmap, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap), "r"(src),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint4 hmax8_u(uint4 a, uint4 b) {
  return make_uint4(hmax2_u32(a.x, b.x), hmax2_u32(a.y, b.y), hmax2_u32(a.z, b.z), hmax2_u32(a.w, b.w));
}

// 2x2 max of two staged rows (tile0, tile1), `npx` input pixels -> npx / 2 pooled pixels at `dst`.
// (sw: 0 = padded tile, 1 / 2 = tile swizzled for the tensor copy, 128 / 64 byte pixel rows)
__device__ __forceinline__ void copy_out_pooled(uint32_t tile0, uint32_t tile1, int pitch, int nck, int os8, int npx,
                                                __half *dst, int lane, int sw) {
  const int total = (npx >> 1) * nck;
  int px = lane / nck, ch = lane - px * nck;
  const int dpx = 32 / nck, dch = 32 - dpx * nck;
  uint4 *o = reinterpret_cast<uint4 *>(dst);
  for (int i = lane; i < total; i += 32) {
    const int p0 = 2 * px, p1 = p0 + 1;
    const uint32_t x0 = sw == 1 ? (uint32_t)(p0 & 7) << 4 : sw == 2 ? (uint32_t)((p0 >> 1) & 3) << 4 : 0u;
    const uint32_t x1 = sw == 1 ? (uint32_t)(p1 & 7) << 4 : sw == 2 ? (uint32_t)((p1 >> 1) & 3) << 4 : 0u;
    const uint32_t off0 = (uint32_t)(p0 * pitch) + ((uint32_t)(ch * 16) ^ x0);
    const uint32_t off1 = (uint32_t)(p1 * pitch) + ((uint32_t)(ch * 16) ^ x1);
    const uint4 a = hmax8_u(lds16(tile0 + off0), lds16(tile0 + off1));
    const uint4 b = hmax8_u(lds16(tile1 + off0), lds16(tile1 + off1));
    o[px * os8 + ch] = hmax8_u(a, b);
    px += dpx;
    ch += dch;
    if (ch >= nck) { ch -= nck; ++px; }
  }
}

// P = 1 or 2 independent pipelines share the CTA's resident weights: each pipeline has
// its own MMA issuing warp, its own input slots, half of the TMEM ring, one epilogue
// team and its own work units.  The issuing thread's instruction stream, not the tensor
// pipe, limits one pipeline (about 3000 cycles per input row against 1250 cycles of MMA
// execution at 64 -> 64 channels), so two of them nearly double the rate.
constexpr int SRC_PX = 72;                 // half resolution pixels per TMA box in expand mode (66 used)
constexpr int SRC_PITCH = SRC_PX * 16;     // 1152 bytes per 8 channel chunk: a multiple of 128
constexpr int ST_PIPE_STRIDE = 8;  // barrier index stride between the pipelines (slots / blocks per pipeline <= 8 when P == 2)

template <int EPI>
__global__ void __launch_bounds__(ST_THREADS, 1) conv3x3_tc_stack(const __grid_constant__ TcArgs g) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + ST_OFF_ABORT);
  volatile uint32_t *tmem_ptr = reinterpret_cast<volatile uint32_t *>(smem + ST_OFF_TMEM_PTR);
  auto bar = [&](int i) { return sbase + (uint32_t)i * 8u; };

#ifdef DNXCU_DEBUG_AIDS
  if (g.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 0] = clock64();
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 3] = (long long)gt;
  }
#endif
#ifdef DNXCU_DEBUG_AIDS
  const long long dbg_entry = clock64();
  const int dbg_cta = (int)(blockIdx.x + gridDim.x * blockIdx.y);
  if (g.trace && threadIdx.x == 0 && dbg_cta < TRACE_CTAS) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 8 + TRACE_CTAS + dbg_cta] = (long long)gt;
  }
#endif
  const int nch = g.a.nch + g.b.nch;
  const int N = g.N, NB = g.NB, P = g.P;
  const uint32_t wdx_bytes = (uint32_t)nch * 3u * N * 16u;  // one horizontal tap: all chunks x 3N rows
  const uint32_t w_addr = sbase + ST_HEADER_BYTES;
  const uint32_t row_bytes = g.row_bytes;  // one input row (of one K group) in a slot
  const uint32_t slot_bytes = row_bytes * (uint32_t)g.ER;
  // (slots on a 1024 byte boundary of the shared memory window: swizzled rows repeat their pattern every 512 bytes)
  const uint32_t slots_addr0 = (w_addr + wdx_bytes * 3u + 1023u) & ~1023u;
  const int S = g.S;  // slots per pipeline
  const int unit_stride = (int)gridDim.x * P;
  const int nprod_warps = P == 2 ? 2 : 4;  // producer warps per pipeline
  // Output channel parts of one launch: blockIdx.y picks the part (always 0 when the launch has one part).
  // Pipeline p of CTA b starts at unit b + p * gridDim.x, so a launch with fewer units than pipelines spreads
  // over the SMs before any SM runs two units side by side.
  const int kofs = (int)blockIdx.y * N;
  OutPart part;
  part.K = min(N, g.K - kofs);
  part.bias = g.bias ? g.bias + kofs : nullptr;
  part.out = g.out ? g.out + kofs : nullptr;
  part.out_pool = g.out_pool ? g.out_pool + kofs : nullptr;

  if (warp == 2) {
    // barrier set-up by a whole warp (one barrier per lane and round) while warp 0 allocates tensor memory
    if (lane == 0) {
      *abort_flag = 0;
      *reinterpret_cast<volatile unsigned long long *>(abort_flag + 1) = g.wait_limit;
      *reinterpret_cast<volatile uint32_t *>(smem + ST_OFF_TURN) = 0u;
      *reinterpret_cast<volatile uint32_t *>(smem + ST_OFF_TURN + 4) = 0u;
    }
    // who completes a slot: the TMA bytes alone; or TMA bytes + the producer warps' cp.async part; or, in expand
    // mode, the producer warps alone after they have expanded the TMA data that landed on the raw barrier;
    // plus, always, the descriptor thread
    const uint32_t full_count = 1u + (g.xp ? (uint32_t)nprod_warps : (g.cpa ? (uint32_t)nprod_warps + 1u : 1u));
    for (int i = lane; i < ST_BAR_COUNT; i += 32) {
      if (i == ST_BAR_WRES) continue;  // warp 1's own
      uint32_t count = 1;
      if (i >= ST_BAR_FULL && i < ST_BAR_FULL + MAX_SLOTS) count = full_count;
      if (i >= ST_BAR_TEMPTY && i < ST_BAR_TEMPTY + ST_MAX_BLOCKS) count = 4;
      mbar_init(bar(i), count);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1 && lane == 0) {
    // ---------------- weights (resident), copies of at most 32 KB: started before anything else ----------------
    mbar_init(bar(ST_BAR_WRES), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t total = wdx_bytes * 3u;
    const unsigned char *wsrc = reinterpret_cast<const unsigned char *>(g.w) + (size_t)blockIdx.y * total;
    mbar_expect_tx(bar(ST_BAR_WRES), total);
    for (uint32_t off = 0; off < total; off += 32768u)
      bulk_g2s(w_addr + off, wsrc + off, min(32768u, total - off), bar(ST_BAR_WRES));
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + ST_OFF_TMEM_PTR),
                 "r"(g.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp == 3 && lane == 0) {
    // the first copy of every tensor map would otherwise wait for its descriptor (a launch of the small levels is
    // a chain of such latencies)
    if (g.a.tma) tma_prefetch_map(&g.tm_a);
    if (g.b.tma && g.b.nch > 0) tma_prefetch_map(&g.tm_b);
    if (g.a.tma && g.a.top) tma_prefetch_map(&g.tm_halo[0]);
    if (g.a.tma && g.a.bot) tma_prefetch_map(&g.tm_halo[1]);
    if (g.b.tma && g.b.top) tma_prefetch_map(&g.tm_halo[2]);
    if (g.b.tma && g.b.bot) tma_prefetch_map(&g.tm_halo[3]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base0 = *tmem_ptr;
#ifdef DNXCU_DEBUG_AIDS
  if (g.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 1] = clock64();
#endif

  // ---- expand mode: cursor over the (unit, input row, K group) entries of one pipeline, and the TMA issue of one entry
  struct XpCursor {
    int u, jj, gi, slot;
    uint32_t ephase, rphase;
    StUnit t;
    bool valid;
  };
  auto xp_start = [&](XpCursor &c, int pipe) {
    c.u = (int)blockIdx.x + pipe * (int)gridDim.x;
    c.jj = c.gi = c.slot = 0;
    c.ephase = 1;
    c.rphase = 0;
    c.valid = c.u < g.nunits;
    if (c.valid) c.t = st_unit_of(g, c.u);
  };
  auto xp_advance = [&](XpCursor &c) {
    if (++c.slot == S) { c.slot = 0; c.ephase ^= 1u; c.rphase ^= 1u; }
    if (++c.gi < g.G) return;
    c.gi = 0;
    if (++c.jj < c.t.rows_out + 2) return;
    c.jj = 0;
    c.u += unit_stride;
    c.valid = c.u < g.nunits;
    if (c.valid) c.t = st_unit_of(g, c.u);
  };
  // Waits for the entry's slot to be free, arms its raw barrier with the byte count and starts the copies:
  // operand a's half resolution row into the slot's staging buffer, operand b's row straight into the slot.
  const bool band = banded(g);
  auto xp_issue = [&](XpCursor &is, int pipe) -> bool {
    const int bofs = pipe * ST_PIPE_STRIDE;
    const uint32_t slots_addr = slots_addr0 + (uint32_t)(pipe * S) * slot_bytes;
    const int nca = g.a.nch;
    const int iy = is.t.y0 - 1 + is.jj;
    const bool a_eng = row_by_tma(g, g.a, iy), b_eng = g.b.nch > 0 && row_by_tma(g, g.b, iy);
    const bool in_image = iy >= 0 && iy < g.H;
    const int c_lo = g.gc0[is.gi], c_hi = c_lo + g.gch[is.gi];
    const int a_lo = min(c_lo, nca), a_hi = min(c_hi, nca);  // operand a's chunks in this group
    const int b_lo = max(c_lo, nca), b_hi = max(c_hi, nca);  // operand b's
    if (!mbar_wait<64>(bar(ST_BAR_EMPTY + bofs + is.slot), is.ephase, abort_flag, g.status, 7)) return false;
    const uint32_t slot_addr = slots_addr + (uint32_t)is.slot * slot_bytes;
    const uint32_t rb = bar(ST_BAR_RAW + bofs + is.slot);
    // what the copy engine brings for this entry: per operand a half resolution row (upsampled operand), the row
    // itself (plain operand), or its raw bytes (ragged operand, rows inside the image only)
    const bool a_raw = a_eng && g.a.rg && in_image && a_hi > a_lo;
    const bool b_raw = b_eng && g.b.rg && in_image && b_hi > b_lo;
    RawSpan ra = {nullptr, 0, 0, 0}, rbs = {nullptr, 0, 0, 0};
    if (a_raw) ra = raw_span(g, g.a, iy, is.t.x0);
    if (b_raw) rbs = raw_span(g, g.b, iy, is.t.x0);
    uint32_t bytes = 0;
    if (a_eng && g.a.tma) bytes += (uint32_t)(a_hi - a_lo) * (g.a.up ? (uint32_t)SRC_PITCH : (uint32_t)CHUNK_PITCH);
    if (b_eng && g.b.tma) bytes += (uint32_t)(b_hi - b_lo) * CHUNK_PITCH;
    bytes += ra.bytes + rbs.bytes;
    if (DBG_SKIP(g) & 1) bytes = 0;
    if (bytes) {
      mbar_expect_tx(rb, bytes);
      if (a_eng && g.a.tma) {
        // (the common case, no row band, keeps the operand's own map as a fixed address)
        if (!band) {
          if (g.a.up) {
            for (int c = a_lo; c < a_hi; c += 2)  // two chunks of the half resolution row, packed, at the first one's place
              tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), &g.tm_a, 0, (is.t.x0 >> 1) - 1, c, iy >> 1, rb);
          } else {
            for (int c = a_lo; c < a_hi; c += g.a.tbox)
              tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), &g.tm_a, 0, is.t.x0 - 1, c, iy, rb);
          }
        } else {
          int y;
          const void *tm = tmap_of(g, 0, iy, g.a.up ? iy >> 1 : iy, &y);
          if (g.a.up) {
            for (int c = a_lo; c < a_hi; c += 2)
              tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), tm, 0, (is.t.x0 >> 1) - 1, c, y, rb);
          } else {
            for (int c = a_lo; c < a_hi; c += g.a.tbox)
              tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), tm, 0, is.t.x0 - 1, c, y, rb);
          }
        }
      }
      if (b_eng && g.b.tma) {
        if (!band) {
          for (int c = b_lo; c < b_hi; c += g.b.tbox)
            tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), &g.tm_b, 0, is.t.x0 - 1, c - nca, iy, rb);
        } else {
          int y;
          const void *tm = tmap_of(g, 1, iy, iy, &y);
          for (int c = b_lo; c < b_hi; c += g.b.tbox)
            tma_load_4d(slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH), tm, 0, is.t.x0 - 1, c - nca, y, rb);
        }
      }
      if (a_raw) bulk_g2s(slot_addr + (uint32_t)((a_lo - c_lo) * CHUNK_PITCH), ra.src, ra.bytes, rb);
      if (b_raw) bulk_g2s(slot_addr + (uint32_t)((b_lo - c_lo) * CHUNK_PITCH), rbs.src, rbs.bytes, rb);
    } else {
      mbar_arrive(rb);
    }
    xp_advance(is);
    return true;
  };

  if (warp == 1 && lane == 0 && g.xp && P == 1) {
    // one pipeline: this thread has nothing else to do and feeds the expand mode's TMA copies
    XpCursor is;
    xp_start(is, 0);
    bool ok = true;
    while (ok && is.valid) ok = xp_issue(is, 0);
  }
  if (warp == 1) __syncwarp();

  // Two issuing threads on one pipeline (TcArgs::ab, one pipeline only): lane 0 of warp 0 takes the even entries,
  // lane 0 of warp 15 the odd ones.  A thread that issues tcgen05.mma gets nothing else done until the tensor pipe
  // has taken the instruction, so with one issuing thread the per entry work (slot wait, descriptor, commits) is
  // time the pipe idles; with two, one prepares its next entry while the other one issues, and the MMAs of
  // consecutive entries follow each other without a gap.  The hand-over is a counter in shared memory (entries
  // issued so far) that the thread whose turn it is next polls, bounded like every other wait; the order of the
  // MMAs, and with it the order of the additions into an accumulator, stays that of the entries.
  const bool ab = g.ab != 0;
  // (the partner thread sits in warp 15 with one pipeline; with two pipelines, which alternate only when every
  // operand comes by TMA, in the then idle producer warps 11 and 13)
  const bool ab_partner = ab && (P == 1 ? warp == 15 : (warp == 11 || warp == 13));
  if (warp < P || ab_partner) {
    // ---------------- MMA issue: one thread, one descriptor per entry ----------------
    // Everything that depends on where an entry sits in its unit (TMEM blocks, runs, barriers) was worked
    // out by the pipeline's descriptor thread and lies in shared memory when the slot's barrier completes;
    // this thread only waits, loads six vectors and issues.  It is the thread the kernel's speed hangs on.
    const int pipe = ab_partner ? (warp == 13 ? 1 : 0) : warp;
    const int me = ab_partner ? 1 : 0;  // which of the two alternating threads
    const int nw = ab ? 2 : 1;
    const uint32_t leader = 1u;
    const int bofs = pipe * ST_PIPE_STRIDE;
    const uint32_t a_hi = (128u >> 4) | (1u << 14), b_hi = a_hi;  // (the B operand's high word; A's comes from the K step table)
    const uint32_t kstep_b = 2u * 3u * N;
    bool ok = lane == 0 && mbar_wait(bar(ST_BAR_WRES), 0, abort_flag, g.status, 1);
    const bool tr = DBG_TRACE_ON(g) && blockIdx.x == 0 && lane == 0 && warp == 0;
    auto mma1 = [&](uint32_t d, uint32_t ahi, uint32_t alo, uint32_t blo, uint32_t idesc) {
      tc_mma_e(d, ((uint64_t)ahi << 32) | alo, ((uint64_t)b_hi << 32) | blo, idesc, leader);
    };
    // Waits until `want` entries have been issued (this thread's turn); gives up like mbar_wait does.
    volatile uint32_t *turn = reinterpret_cast<volatile uint32_t *>(smem + ST_OFF_TURN + 4 * pipe);
    auto my_turn = [&](uint32_t want) -> bool {
      if (*turn == want) return true;
      const unsigned long long t0 = clock64();
      for (uint32_t it = 1;; ++it) {
        if (*turn == want) return true;
        if ((it & 63u) == 0) {
          if (*abort_flag) return false;
          const unsigned long long limit =
              *reinterpret_cast<const volatile unsigned long long *>(abort_flag + 1) & ~(1ull << 63);
          if ((unsigned long long)clock64() - t0 > limit) {
            *abort_flag = 1;
            if (g.status) atomicCAS(g.status, 0, 11);
            return false;
          }
        }
      }
    };
    // The loop, instantiated per K step count: when all K groups have the same count, the choice of the
    // straight line form is made once here and not per row (NKC = 0: per row, by a switch).
    auto mma_loop = [&](auto NKC, auto ERC) {
      constexpr int NK = decltype(NKC)::value;
      constexpr int ERT = decltype(ERC)::value;  // input rows per entry
      int slot = me, pos = me;                    // (the ring has at least two slots)
      uint32_t fphase = 0;
      for (;;) {
        if (tr) trace(g, 0, pos >> (nw - 1), 0);
        if (!mbar_wait(bar(ST_BAR_FULL + bofs + slot), fphase, abort_flag, g.status, 2)) break;
        if (tr) trace(g, 0, pos >> (nw - 1), 1);
        const uint32_t da = sbase + ST_OFF_DESC + (uint32_t)(bofs + slot) * ST_DESC_BYTES;
        uint4 q[ERT][3];
#pragma unroll
        for (int r = 0; r < ERT; ++r) {
          q[r][0] = lds16(da + (uint32_t)(r * ST_SUBDESC_BYTES));
          q[r][1] = lds16(da + (uint32_t)(r * ST_SUBDESC_BYTES + 16));
          q[r][2] = lds16(da + (uint32_t)(r * ST_SUBDESC_BYTES + 32));
        }
        // the fresh accumulator block of each row has been read out and zeroed
        {
          bool blocks_ok = true;
#pragma unroll
          for (int r = 0; r < ERT; ++r)
            if (q[r][2].z) blocks_ok = blocks_ok && mbar_wait(q[r][2].z, q[r][2].w, abort_flag, g.status, 3);
          if (!blocks_ok) break;
        }
        // my turn: the other thread has issued the entry before this one
        if (ab && !my_turn((uint32_t)pos)) break;
        tc_fence_after();
        uint32_t allflags = 0;
#pragma unroll
        for (int r = 0; r < ERT; ++r) {
          const uint4 q0 = q[r][0], q1 = q[r][1], q2 = q[r][2];
          const uint32_t flags = q0.z;
          allflags |= flags;
          if (!(DBG_SKIP(g) & 2)) {
            const uint32_t row_lo = q0.x, b_lo = q0.y;
            const Run R0 = {q1.x, q1.y, q1.z, 1u}, R1 = {q1.w, q2.x, q2.y, 1u};
            if constexpr (NK > 0) {
              if (flags & DF_NR2) st_issue_row<NK, 2>(g, b_hi, row_lo, b_lo, wdx_bytes >> 4, kstep_b, R0, R1, leader);
              else st_issue_row<NK, 1>(g, b_hi, row_lo, b_lo, wdx_bytes >> 4, kstep_b, R0, R0, leader);
            } else {
              const int nk16 = (int)(flags & 15u);
              bool done = false;
              if (!DBG_LOOP_ISSUE(g))
                done = (flags & DF_NR2) ? st_issue_nk<2>(g, nk16, b_hi, row_lo, b_lo, wdx_bytes >> 4, kstep_b, R0, R1, leader)
                                        : st_issue_nk<1>(g, nk16, b_hi, row_lo, b_lo, wdx_bytes >> 4, kstep_b, R0, R0, leader);
              if (!done) {
                // more K steps than the straight line forms cover
                for (int dx = 0; dx < 3; ++dx)
                  for (int kc = 0; kc < nk16; ++kc) {
                    const uint32_t a = row_lo + g.kst_lo[kc & 15] + (uint32_t)dx * g.kst_dx[kc & 15];
                    const uint32_t b = b_lo + (uint32_t)dx * (wdx_bytes >> 4) + (uint32_t)kc * kstep_b;
                    mma1(R0.col, g.kst_hi[kc & 15], a, b + R0.boff, R0.idesc);
                    if (flags & DF_NR2) mma1(R1.col, g.kst_hi[kc & 15], a, b + R1.boff, R1.idesc);
                  }
              }
            }
          }
          if (tr) trace(g, 0, pos >> (nw - 1), 2);
          if (ab && r == ERT - 1) {
            // hand over: the other thread may issue the next entry; the commits below are this thread's own time
            tc_fence_before();
            *turn = (uint32_t)pos + 1u;
          }
          // the slot is free once the MMAs of its last row are done; an output row completed by this input row
          // is announced right behind that row's MMAs
          if (r == ERT - 1) tc_commit_e(bar(ST_BAR_EMPTY + bofs + slot), leader);
          if (q0.w) tc_commit_e(q0.w, leader);
        }
        if (tr) trace(g, 0, pos >> (nw - 1), 3);
        if (allflags & DF_LAST) break;
        if (ab && (allflags & DF_PENULT)) break;  // the other thread issues the last entry
        pos += nw;
        slot += nw;
        if (slot >= S) {
          slot -= S;
          fphase ^= 1u;
        }
      }
    };
    if (lane == 0 && ok && (int)blockIdx.x + pipe * (int)gridDim.x < g.nunits) {
      bool same = !DBG_LOOP_ISSUE(g) && !DBG_SWITCH_ISSUE(g);
      for (int gi = 1; gi < g.G; ++gi) same = same && g.gch[gi] == g.gch[0];
      const int nkfix = same ? (g.gch[0] >> 1) : 0;
      if (g.ER == 2) {
        // two rows per entry: one K group, at most six K steps (the plan refuses anything else)
        switch (nkfix) {
          case 1: mma_loop(IntC<1>{}, IntC<2>{}); break;
          case 2: mma_loop(IntC<2>{}, IntC<2>{}); break;
          case 3: mma_loop(IntC<3>{}, IntC<2>{}); break;
          case 4: mma_loop(IntC<4>{}, IntC<2>{}); break;
          case 5: mma_loop(IntC<5>{}, IntC<2>{}); break;
          default: mma_loop(IntC<6>{}, IntC<2>{}); break;
        }
      } else {
        switch (nkfix) {
          case 1: mma_loop(IntC<1>{}, IntC<1>{}); break;
          case 2: mma_loop(IntC<2>{}, IntC<1>{}); break;
          case 3: mma_loop(IntC<3>{}, IntC<1>{}); break;
          case 4: mma_loop(IntC<4>{}, IntC<1>{}); break;
          case 5: mma_loop(IntC<5>{}, IntC<1>{}); break;
          case 6: mma_loop(IntC<6>{}, IntC<1>{}); break;
          default: mma_loop(IntC<0>{}, IntC<1>{}); break;
        }
      }
    }
    __syncwarp();
  } else if (warp >= 2 && warp < 2 + 4 * P * g.eteams) {
    // ---------------- epilogue: teams of four warps ----------------
    // Two pipelines: one team each.  One pipeline: one team, or two teams that take alternate items (a team
    // needs about 3800 cycles for a row pair of 64 channels, two alternating MMA warps produce one in 2300).
    const int team = (warp - 2) >> 2;
    const int nteams = g.eteams;
    const int pipe = nteams == 2 ? 0 : team;
    const int myteam = nteams == 2 ? team : 0;
    const int bofs = pipe * ST_PIPE_STRIDE;
    const uint32_t tmem_base = tmem_base0 + (uint32_t)(pipe * NB * N);
    const int q = warp & 3;
    const int m = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const bool tr = DBG_TRACE_ON(g) && blockIdx.x == 0 && threadIdx.x == 64;
    const int pitch = g.stage_pitch;  // 0: no staging tile, direct stores
    const int nck = part.K >> 3;
    const int os8 = g.os >> 3;  // output pixel stride in 16 byte units (= nck unless the output channels are split)
    const int otma = g.out_tma;
    // (tiles that leave by tensor copy start on a 1024 byte boundary: the swizzle pattern is a function of the address)
    const uint32_t stage_region = slots_addr0 + (uint32_t)(P * S) * (slot_bytes + g.src_bytes);
    const uint32_t stage_base = (otma ? (stage_region + 1023u) & ~1023u : stage_region) + (uint32_t)(warp - 2) * g.stage_warp_bytes;
    const uint32_t xr = otma == 1 ? (uint32_t)(lane & 7) << 4 : otma == 2 ? (uint32_t)((lane >> 1) & 3) << 4 : 0u;
    bool ok = true;
    int item = 0;
    int blk = 0;
    uint32_t tphase = 0;  // parity of tfull[blk] for the current round of the ring
    // Every MMA accumulates, so a block is zero when the MMA thread gets it: all of them once here (this
    // completes the first phase of the block barriers), and each one again when it has been read out.
    if (myteam == 0) {
      for (int b = 0; b < NB; ++b) tc_zero_cols(lane_addr + (uint32_t)(b * N), N);
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        for (int b = 0; b < NB; ++b) mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b));
    }
    for (int u = (int)blockIdx.x + pipe * (int)gridDim.x; ok && u < g.nunits; u += unit_stride) {
      const StUnit t = st_unit_of(g, u);
      const int x = t.x0 + m;
      const bool xin = x < g.W;
      for (int i = 0; ok && i < t.rows_out; i += 2, ++item) {
        const int nrows = min(2, t.rows_out - i);
        // blocks and phases of this item's rows; the ring state advances for every item, taken or not
        const int b0 = blk;
        const uint32_t ph0 = tphase;
        if (++blk == NB) { blk = 0; tphase ^= 1u; }
        const int b1 = blk;
        const uint32_t ph1 = tphase;
        if (nrows == 2) {
          if (++blk == NB) { blk = 0; tphase ^= 1u; }
        }
        if (nteams == 2 && (item & 1) != myteam) continue;  // the other team's item
        if (tr) trace(g, 1, item >> 1, 0);
        ok = mbar_wait<64>(bar(ST_BAR_TFULL + bofs + b0), ph0, abort_flag, g.status, 6);
        if (ok && nrows == 2) ok = mbar_wait<64>(bar(ST_BAR_TFULL + bofs + b1), ph1, abort_flag, g.status, 6);
        if (!ok) break;
        if (tr) trace(g, 1, item >> 1, 1);
        tc_fence_after();
        const int y = t.y0 + i;
        const uint32_t t0 = lane_addr + (uint32_t)(b0 * N), t1 = lane_addr + (uint32_t)(b1 * N);
        if (pitch) {
          // staged: all TMEM reads first (the blocks are handed back before the copy-out)
          const uint32_t tile0 = stage_base, tile1 = stage_base + (uint32_t)(32 * pitch);
          const uint32_t mine = (uint32_t)(lane * pitch);
          const int xw = t.x0 + q * 32;                      // first pixel of this warp
          const int npx = max(0, min(32, g.W - xw));        // pixels of this warp inside the image
          // two tiles per warp (always with the fused pool, and where shared memory allows): a row pair is staged
          // in one go, its blocks go back, then both rows are copied out
          const bool both = g.stage2 && nrows == 2;
          if (!(DBG_SKIP(g) & 8)) {
            if (both) {
              if (otma) {  // (the copies of this warp's last item have read the tiles)
                if (lane == 0) bulk_wait_read();
                __syncwarp();
              }
              // last TMEM read of the item done: give the blocks back, zeroed (every MMA accumulates)
              auto release = [&]() {
                tc_zero_cols(t0, N);
                tc_zero_cols(t1, N);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                  mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b0));
                  mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b1));
                }
              };
              if (N == 32) {
                // one chunk: the blocks go back as soon as it is in registers, before the conversion
                stage_cols2<32, EPI>(g, part, t0, t1, 0, tile0 + mine, tile1 + mine, xr, release);
              } else if (N == 16) {
                stage_cols2<16, EPI>(g, part, t0, t1, 0, tile0 + mine, tile1 + mine, xr, release);
              } else {
                int c0 = 0;
#pragma unroll 1
                for (; c0 + 32 <= N; c0 += 32) stage_cols2<32, EPI>(g, part, t0, t1, c0, tile0 + mine, tile1 + mine, xr);
                if (c0 < N) stage_cols2<16, EPI>(g, part, t0, t1, c0, tile0 + mine, tile1 + mine, xr);
                release();
              }
              if (otma) fence_async_smem();  // (my rows of the tiles, for the copy engine; the warp meets below)
              __syncwarp();
              if (tr) trace(g, 1, item >> 1, 3);
              if (tr) trace(g, 1, item >> 1, 4);
              if (!(DBG_SKIP(g) & 4)) {
                if ((EPI & EPI_FULL) && otma) {
                  if (lane == 0 && npx > 0) {
                    tma_store_3d(&g.tm_out, tile0, 0, xw, y);
                    tma_store_3d(&g.tm_out, tile1, 0, xw, y + 1);
                    bulk_commit();
                  }
                } else if (EPI & EPI_FULL) {
                  copy_out(tile0, pitch, nck, os8, npx, part.out + ((long long)y * g.W + xw) * g.os, lane);
                  copy_out(tile1, pitch, nck, os8, npx, part.out + ((long long)(y + 1) * g.W + xw) * g.os, lane);
                }
                if (EPI & EPI_POOL)
                  copy_out_pooled(tile0, tile1, pitch, nck, os8, npx,
                                  part.out_pool + ((long long)(y >> 1) * (g.W >> 1) + (xw >> 1)) * g.os, lane, otma);
              }
              __syncwarp();
              if (tr) trace(g, 1, item >> 1, 5);
            } else {
              for (int r = 0; r < nrows; ++r) {
                const uint32_t tr_addr = r ? t1 : t0;
                if (otma) {
                  if (lane == 0) bulk_wait_read();
                  __syncwarp();
                }
                int c0 = 0;
#pragma unroll 1
                for (; c0 + 32 <= N; c0 += 32) stage_cols<32, EPI>(g, part, tr_addr, c0, tile0 + mine, xr);
                if (c0 < N) stage_cols<16, EPI>(g, part, tr_addr, c0, tile0 + mine, xr);
                if (otma) fence_async_smem();
                if (tr && r == 0) trace(g, 1, item >> 1, 3);
                if (r == nrows - 1) {
                  // last TMEM read of the item done: give the blocks back, zeroed (every MMA accumulates)
                  tc_zero_cols(t0, N);
                  if (nrows == 2) tc_zero_cols(t1, N);
                  tc_fence_before();
                  __syncwarp();
                  if (lane == 0) {
                    mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b0));
                    if (nrows == 2) mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b1));
                  }
                  if (tr) trace(g, 1, item >> 1, 4);
                } else {
                  __syncwarp();
                }
                // (a single row of a plan with the fused pool is a last row without partner: it has no pooled output)
                if ((EPI & EPI_FULL) && !(DBG_SKIP(g) & 4)) {
                  if (otma) {
                    if (lane == 0 && npx > 0) {
                      tma_store_3d(&g.tm_out, tile0, 0, xw, y + r);
                      bulk_commit();
                    }
                  } else {
                    copy_out(tile0, pitch, nck, os8, npx, part.out + ((long long)(y + r) * g.W + xw) * g.os, lane);
                  }
                }
                __syncwarp();
                if (tr && r == 0) trace(g, 1, item >> 1, 5);
              }
            }
          } else {
            tc_zero_cols(t0, N);
            if (nrows == 2) tc_zero_cols(t1, N);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b0));
              if (nrows == 2) mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b1));
            }
          }
          if (tr) trace(g, 1, item >> 1, 2);
          continue;
        }
        int c0 = (DBG_SKIP(g) & 8) ? N : 0;
        if (nrows == 2 && N <= 32 && c0 == 0) {
          // one chunk: the blocks go back as soon as it is in registers, before the conversion and the stores
          auto release = [&]() {
            tc_zero_cols(t0, N);
            tc_zero_cols(t1, N);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b0));
              mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b1));
            }
          };
          if (N == 32) epi_fast<32, 2, EPI>(g, part, t0, t1, 0, x, y, xin, lane, release);
          else epi_fast<16, 2, EPI>(g, part, t0, t1, 0, x, y, xin, lane, release);
          if (tr) trace(g, 1, item >> 1, 2);
          continue;
        }
        if (nrows == 2) {
#pragma unroll 1
          for (; c0 + 32 <= N; c0 += 32) epi_fast<32, 2, EPI>(g, part, t0, t1, c0, x, y, xin, lane);
          if (c0 < N) epi_fast<16, 2, EPI>(g, part, t0, t1, c0, x, y, xin, lane);
        } else {
#pragma unroll 1
          for (; c0 + 32 <= N; c0 += 32) epi_fast<32, 1, EPI>(g, part, t0, t1, c0, x, y, xin, lane);
          if (c0 < N) epi_fast<16, 1, EPI>(g, part, t0, t1, c0, x, y, xin, lane);
        }
        if (tr) trace(g, 1, item >> 1, 2);
        tc_zero_cols(t0, N);
        if (nrows == 2) tc_zero_cols(t1, N);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b0));
          if (nrows == 2) mbar_arrive(bar(ST_BAR_TEMPTY + bofs + b1));
        }
      }
    }
    if (g.out_tma && lane == 0) bulk_wait_all();  // (the staging tiles must outlive the copies that read them)
  } else if (warp >= 10 && warp < 14) {
    // ---------------- input slots ----------------
    // P == 2: warps 10, 11 feed pipeline 0 and warps 12, 13 pipeline 1; P == 1: all four feed pipeline 0.
    const int pipe = P == 2 ? (warp - 10) >> 1 : 0;
    const int bofs = pipe * ST_PIPE_STRIDE;
    const uint32_t slots_addr = slots_addr0 + (uint32_t)(pipe * S) * slot_bytes;
    const int nprod = nprod_warps * 32;
    const int tid = threadIdx.x - (10 + pipe * nprod_warps * (P == 2 ? 1 : 0)) * 32;
    bool ok = true;
    if (!g.cpa) {
      // everything comes by TMA: one thread per pipeline, one or two copies per entry
      if (tid == 0) {
        int slot = 0, pcount = 0;
        uint32_t phase = 1;  // parity to wait for on the empty barrier: first round passes
        const bool tr = DBG_TRACE_ON(g) && blockIdx.x == 0 && pipe == 0;
        for (int u = (int)blockIdx.x + pipe * (int)gridDim.x; ok && u < g.nunits; u += unit_stride) {
          const StUnit t = st_unit_of(g, u);
          for (int jj = 0; ok && jj < t.rows_out + 2; jj += g.ER) {
            for (int gi = 0; ok && gi < g.G; ++gi) {
              if (tr) trace(g, 2, pcount, 0);
              ok = mbar_wait<64>(bar(ST_BAR_EMPTY + bofs + slot), phase, abort_flag, g.status, 7);
              if (!ok) break;
              if (tr) trace(g, 2, pcount, 1);
              const uint32_t fb = bar(ST_BAR_FULL + bofs + slot);
              const uint32_t row_tx = g.grp_tx[gi];
              mbar_expect_tx(fb, row_tx * (uint32_t)g.ER);
              if (!(DBG_SKIP(g) & 1)) {
                // the entry's rows one after the other in the slot (rows past the image are zero filled by the copy)
                for (int r = 0; r < g.ER; ++r) {
                  const int iy = t.y0 - 1 + jj + r;
                  const uint32_t slot_addr = slots_addr + (uint32_t)slot * slot_bytes + (uint32_t)r * row_bytes;
                  // first pixel of the slot row: x0 - 1, or x0 - 2 when an operand comes through a pixel doubling
                  // map (whose rows start on an even pixel: half resolution pixel x0 / 2 - 1, row iy >> 1)
                  const int xs = t.x0 - 1 - g.shift, xh = (t.x0 >> 1) - 1;
                  const int ncp = g.ncp[gi];
#pragma unroll 1
                  for (int j = 0; j < ncp; ++j) {
                    const uint32_t dst = slot_addr + g.cp[gi][j].dst;
                    const int unit = g.cp[gi][j].unit, sg = g.cp[gi][j].sg;
                    const bool dup = sg == 0 && g.a.dup;
                    int y = dup ? iy >> 1 : iy;
                    const void *tm = sg ? (const void *)&g.tm_b : (const void *)&g.tm_a;
                    if (band) tm = tmap_of(g, sg, iy, y, &y);
                    if (dup) tma_load_5d(dst, tm, 0, 0, xh, unit, y, fb);
                    else tma_load_4d(dst, tm, 0, xs, unit, y, fb);
                  }
                }
              } else {
                // timing aid: nothing will land, so complete the transaction count by hand
                asm volatile("mbarrier.complete_tx.shared::cta.b64 [%0], %1;" ::"r"(fb), "r"(row_tx * (uint32_t)g.ER) : "memory");
              }
              if (tr) trace(g, 2, pcount, 2);
              ++pcount;
              if (++slot == S) {
                slot = 0;
                phase ^= 1u;
              }
            }
          }
        }
      }
    } else if (g.xp) {
      // Operand a is the 2x nearest upsample of a half resolution tensor (basic_upsample.comp:49-56:
      // src = dst / 2).  TMA fetches the half resolution row (66 pixels) into a staging buffer and operand
      // b's row straight into the slot; both land on the slot's raw barrier.  The producer warps then write
      // every source pixel to its two destination pixels inside shared memory and signal the slot.
      const int nca = g.a.nch;
      // Thread 0 of the producer warps (two pipelines) or lane 0 of the otherwise idle weights warp (one
      // pipeline) starts the TMA copies; it runs ahead of the expansion as far as free slots allow, so the copy
      // latency overlaps the expansion of earlier rows.
      const bool self_issue = P == 2;
      const bool meet = g.a.rg || g.b.rg;  // the producer threads of a pipeline meet at a named barrier per entry
      const int LA = S - 1 < 4 ? S - 1 : 4;
      XpCursor is, ex;
      xp_start(is, pipe);
      xp_start(ex, pipe);
      int ahead = 0;  // entries issued but not yet expanded (thread 0, self_issue only)
      int xcount = 0;
      while (ex.valid) {
        if (self_issue && tid == 0) {
          while (ok && is.valid && ahead < LA) {
            ok = xp_issue(is, pipe);
            ++ahead;
          }
        }
        // expand entry `ex`
        {
          const int iy = ex.t.y0 - 1 + ex.jj;
          const bool a_eng = row_by_tma(g, g.a, iy), b_eng = g.b.nch > 0 && row_by_tma(g, g.b, iy);
          const int c_lo = g.gc0[ex.gi], c_hi = c_lo + g.gch[ex.gi];
          const int a_lo = min(c_lo, nca), a_hi = min(c_hi, nca);
          const uint32_t slot_addr = slots_addr + (uint32_t)ex.slot * slot_bytes;
          const uint32_t rb = bar(ST_BAR_RAW + bofs + ex.slot);
          if (tid == 32 && pipe == 0) trace(g, 2, xcount, 0);
          if (ok) ok = mbar_wait<32>(rb, ex.rphase, abort_flag, g.status, 8);
          // The re-lay of a ragged operand meets at a named barrier, so there the producer threads of a pipeline
          // must leave this loop together: they vote, and a wait that ran out in one of them takes all of them
          // out.  Without a ragged operand every warp works on chunk pairs of its own and only its lanes vote.
          if (!meet) {
            ok = __all_sync(0xffffffffu, ok);
          } else {
            uint32_t all_ok;
            asm volatile(
                "{\n\t"
                ".reg .pred p, q;\n\t"
                "setp.ne.u32 p, %1, 0;\n\t"
                "bar.red.and.pred q, %2, %3, p;\n\t"
                "selp.u32 %0, 1, 0, q;\n\t"
                "}"
                : "=r"(all_ok)
                : "r"((uint32_t)ok), "r"(1 + pipe), "r"(nprod)
                : "memory");
            ok = all_ok != 0;
          }
          if (!ok) break;
          if (tid == 32 && pipe == 0) trace(g, 2, xcount, 1);
          // rows TMA does not cover (halo rows of a row band) come the old way; the raw barrier has completed,
          // so the slot is free (thread 0 waited for that before it armed the barrier)
          if (!(DBG_SKIP(g) & 1) && (!a_eng || (g.b.nch > 0 && !b_eng))) {
            load_row(g, slot_addr, iy, ex.t.x0, tid, nprod, c_lo, c_hi);
            cp_async_commit();
            cp_async_wait<0>();
          }
          if (a_eng && g.a.up && !(DBG_SKIP(g) & 1)) {
            // In place, a pair of chunks per warp: the copy left the pair's two half resolution rows packed
            // (2 x 72 pixels) at the start of the pair's 2 x 132 pixel area.  The lanes of a warp first load the
            // sources of all pixels of the pair, meet, then store; no other warp touches that pair, so the warps
            // of a pipeline expand different pairs side by side without meeting.
            static_assert(SLOT_PX <= 5 * 32, "five pixels per lane cover a slot row");
            for (int c = a_lo + 2 * (tid >> 5); c < a_hi; c += 2 * nprod_warps) {
              const uint32_t pair = slot_addr + (uint32_t)((c - c_lo) * CHUNK_PITCH);
              uint4 v[5][2];
#pragma unroll
              for (int i = 0; i < 5; ++i) {
                const int px = lane + i * 32;
                if (px < SLOT_PX) {
                  const uint32_t sp = pair + (uint32_t)(((px + 1) >> 1) * 16);
                  v[i][0] = lds16(sp);
                  v[i][1] = lds16(sp + (uint32_t)SRC_PITCH);
                }
              }
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 5; ++i) {
                const int px = lane + i * 32;
                if (px < SLOT_PX) {
                  const uint32_t dp = pair + (uint32_t)(px * 16);
                  sts16(dp, v[i][0]);
                  sts16(dp + (uint32_t)CHUNK_PITCH, v[i][1]);
                }
              }
            }
          }
          // Ragged operands (at most 16 channels, two chunks): the copy left the row's raw bytes, pixel after
          // pixel at C halves each, at the start of the operand's two chunk area.  Re-laid in place into
          // [chunk][pixel][8 halves] with zeros for the channels up to 16 and for pixels outside the image: every
          // thread gathers its pixels, the producer threads of the pipeline meet, then they store.
          if (!(DBG_SKIP(g) & 1)) {
#pragma unroll 1
            for (int sg = 0; sg < 2; ++sg) {
              const Seg &sgm = sg ? g.b : g.a;
              if (!sgm.rg || !(sg ? b_eng : a_eng)) continue;
              const int lo = sg ? max(c_lo, nca) : a_lo, hi = sg ? max(c_hi, nca) : a_hi;
              if (hi <= lo) continue;
              const uint32_t area = slot_addr + (uint32_t)((lo - c_lo) * CHUNK_PITCH);
              const bool in_image = iy >= 0 && iy < g.H;
              RawSpan rs = {nullptr, 0, 0, 0};
              if (in_image) rs = raw_span(g, sgm, iy, ex.t.x0);
              const int C = sgm.C;
              uint32_t wv[3][8];
#pragma unroll
              for (int i = 0; i < 3; ++i) {
#pragma unroll
                for (int e = 0; e < 8; ++e) wv[i][e] = 0u;
                const int px = tid + i * nprod;
                const int ix = ex.t.x0 - 1 + px;
                if (px < SLOT_PX && in_image && ix >= 0 && ix < g.W) {
                  const uint32_t sp = area + rs.lead + (uint32_t)((ix - rs.xs) * C * 2);
#pragma unroll
                  for (int e = 0; e < 16; ++e)
                    if (e < C) {
                      uint32_t hv;
                      asm volatile("ld.shared.u16 %0, [%1];" : "=r"(hv) : "r"(sp + (uint32_t)(2 * e)) : "memory");
                      wv[i][e >> 1] |= hv << ((e & 1) * 16);
                    }
                }
              }
              asm volatile("bar.sync %0, %1;" ::"r"(1 + pipe), "r"(nprod) : "memory");
#pragma unroll
              for (int i = 0; i < 3; ++i) {
                const int px = tid + i * nprod;
                if (px < SLOT_PX) {
                  const uint32_t dp = area + (uint32_t)(px * 16);
                  sts16(dp, make_uint4(wv[i][0], wv[i][1], wv[i][2], wv[i][3]));
                  sts16(dp + (uint32_t)CHUNK_PITCH, make_uint4(wv[i][4], wv[i][5], wv[i][6], wv[i][7]));
                }
              }
            }
          }
          if (tid == 32 && pipe == 0) trace(g, 2, xcount, 2);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(ST_BAR_FULL + bofs + ex.slot));
          if (tid == 32 && pipe == 0) trace(g, 2, xcount, 3);
          ++xcount;
          if (self_issue && tid == 0) --ahead;
          xp_advance(ex);
        }
      }
    } else {
      // some rows need the producer warps: all threads of the pipeline's producer warps walk the entries,
      // thread 0 also issues the TMA part; each thread keeps up to D rows of cp.async in flight
      int pos = 0, signalled = 0;
      const int D = g.D;
      for (int u = (int)blockIdx.x + pipe * (int)gridDim.x; ok && u < g.nunits; u += unit_stride) {
        const StUnit t = st_unit_of(g, u);
        for (int jj = 0; ok && jj < t.rows_out + 2; ++jj) {
          const int iy = t.y0 - 1 + jj;
          for (int gi = 0; ok && gi < g.G; ++gi) {
            const int c_lo = g.gc0[gi], c_hi = c_lo + g.gch[gi];
            const int slot = pos % S;
            ok = mbar_wait<64>(bar(ST_BAR_EMPTY + bofs + slot), ((uint32_t)(pos / S) & 1u) ^ 1u, abort_flag, g.status, 7);
            if (!ok) break;
            const uint32_t slot_addr = slots_addr + (uint32_t)slot * slot_bytes;
            if (tid == 0) {
              const uint32_t fb = bar(ST_BAR_FULL + bofs + slot);
              const uint32_t bytes = (DBG_SKIP(g) & 1) ? 0u : tma_row<false>(g, slot_addr, iy, t.x0, c_lo, c_hi, fb);
              if (bytes) {
                mbar_expect_tx(fb, bytes);
                tma_row<true>(g, slot_addr, iy, t.x0, c_lo, c_hi, fb);
              } else {
                mbar_arrive(fb);
              }
            }
            if (!(DBG_SKIP(g) & 1)) load_row(g, slot_addr, iy, t.x0, tid, nprod, c_lo, c_hi);
            cp_async_commit();
            ++pos;
            if (pos - signalled >= D) {
              cp_async_wait_dyn(D - 1);
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(ST_BAR_FULL + bofs + signalled % S));
              ++signalled;
            }
          }
        }
      }
      cp_async_wait<0>();
      if (ok) {
        fence_proxy_async();
        __syncwarp();
        if (lane == 0)
          for (; signalled < pos; ++signalled) mbar_arrive(bar(ST_BAR_FULL + bofs + signalled % S));
      }
    }
  } else if (warp >= 14 && warp - 14 < P && lane == 0) {
    // ---------------- entry descriptors: one thread per pipeline ----------------
    // Walks the same (unit, input row, K group) sequence as the producers, keeps the ring of TMEM blocks
    // and writes what the MMA thread needs for the entry into the slot's descriptor, then arrives on the
    // slot's barrier: the descriptor is visible when the barrier completes.
    const int pipe = warp - 14;
    const int bofs = pipe * ST_PIPE_STRIDE;
    const uint32_t tmem_base = tmem_base0 + (uint32_t)(pipe * NB * N);
    const uint32_t slots_addr = slots_addr0 + (uint32_t)(pipe * S) * slot_bytes;
    const uint32_t b_lo0 = (3u * N) << 16;  // leading offset = chunk pitch = 3N rows x 16 bytes, >> 4
    const uint32_t idesc0 = (1u << 4) | ((uint32_t)(STRIP >> 4) << 24);
    const bool two = 2 * N <= 256, three = 3 * N <= 256;
    const uint32_t N16 = (uint32_t)N;  // weight rows of one vertical tap, in 16 byte units of a chunk
    // instruction descriptors of runs of one, two and three blocks
    const uint32_t idesc_len[3] = {idesc0 | ((uint32_t)(N >> 3) << 17), idesc0 | ((uint32_t)((2 * N) >> 3) << 17),
                                   idesc0 | ((uint32_t)((3 * N) >> 3) << 17)};
    int slot = 0;
    uint32_t ephase = 1;  // parity to wait for on the empty barrier: first round passes
    int blkC = 0;
    uint32_t cphase = 0;  // parity to wait for on tempty[blkC]: the epilogue's first zeroing completes phase 0
    bool ok = true;
    [[maybe_unused]] int dcount = 0;
    for (int u = (int)blockIdx.x + pipe * (int)gridDim.x; ok && u < g.nunits; u += unit_stride) {
      const StUnit t = st_unit_of(g, u);
      const int rows_in = t.rows_out + 2;
      const bool last_unit = u + unit_stride >= g.nunits;
      int blkA = 0, blkB = 0;  // blocks of output rows jj-2, jj-1 (stack positions 0, 1); blkC: row jj (position 2)
      for (int jj = 0; ok && jj < rows_in; ++jj) {
        const bool vA = jj >= 2, vB = jj >= 1 && jj <= t.rows_out, vC = jj < t.rows_out;
        auto mk = [&](int sidx, int len, uint32_t acc) {
          Run r;
          const int blk = sidx == 0 ? blkA : (sidx == 1 ? blkB : blkC);
          r.col = tmem_base + (uint32_t)(blk * N);
          r.boff = (uint32_t)sidx * N16;
          r.idesc = idesc0 | ((uint32_t)((len * N) >> 3) << 17);
          r.acc = acc;
          return r;
        };
        // runs of neighbouring blocks one MMA can cover (every block starts zeroed, so all MMAs accumulate);
        // acc == 2: unused
        Run R0 = {0, 0, 0, 2}, R1 = R0, R2 = R0;
        const bool mAB_mid = blkB != 0 && two, mBC_mid = blkC != 0 && two && (!mAB_mid || three);
        if (vA && vB && vC && (mAB_mid || mBC_mid)) {
          // the rows in the middle of a unit (all but four), spelled out: this thread has about a thousand cycles
          // per entry when two MMA warps alternate, and the general form below takes most of them
          const uint32_t cA = tmem_base + (uint32_t)(blkA * N);
          if (mAB_mid && mBC_mid) {
            R0 = {cA, 0u, idesc_len[2], 1u};
          } else if (mAB_mid) {
            R0 = {cA, 0u, idesc_len[1], 1u};
            R1 = {tmem_base + (uint32_t)(blkC * N), 2u * N16, idesc_len[0], 1u};
          } else {
            R0 = {cA, 0u, idesc_len[0], 1u};
            R1 = {tmem_base + (uint32_t)(blkB * N), N16, idesc_len[1], 1u};
          }
        } else {
          const bool mAB = vA && vB && blkB != 0 && two;
          const bool mBC = vB && vC && blkC != 0 && two && (!mAB || three);
          if (mAB && mBC) {
            R0 = mk(0, 3, 1);
          } else if (mAB) {
            R0 = mk(0, 2, 1);
            if (vC) R1 = mk(2, 1, 1);
          } else if (mBC) {
            if (vA) { R0 = mk(0, 1, 1); R1 = mk(1, 2, 1); } else { R0 = mk(1, 2, 1); }
          } else {
            if (vA) R0 = mk(0, 1, 1);
            if (vB) { if (vA) R1 = mk(1, 1, 1); else R0 = mk(1, 1, 1); }
            if (vC) { if (vA && vB) R2 = mk(2, 1, 1); else if (vA || vB) R1 = mk(2, 1, 1); else R0 = mk(2, 1, 1); }
          }
        }
        if (R2.acc != 2) {
          // three separate runs need a block ring shorter than the plan ever makes: refuse instead of computing wrong
          *abort_flag = 1;
          if (g.status) atomicCAS(g.status, 0, 9);
          ok = false;
          break;
        }
        const uint32_t rowflags = R1.acc != 2 ? DF_NR2 : 0u;
        // with two rows per entry (one K group then) this row is the first or the second half of its entry: the
        // slot is waited for before the first half is described and handed over after the second
        const int sub = g.ER == 2 ? (jj & 1) : 0;
        for (int gi = 0; ok && gi < g.G; ++gi) {
          if (DBG_TRACE_ON(g) && blockIdx.x == 0 && pipe == 0) trace(g, 2, dcount, 4);
          if (sub == 0) {
            ok = mbar_wait<32>(bar(ST_BAR_EMPTY + bofs + slot), ephase, abort_flag, g.status, 7);
            if (!ok) break;
          }
          uint32_t flags = rowflags | (uint32_t)(g.gch[gi] >> 1);
          if (last_unit && jj == rows_in - 1 && gi == g.G - 1) flags |= DF_LAST;
          // the entry before the last one: the last entry of one of two alternating MMA warps
          if (last_unit && ((g.G > 1 && jj == rows_in - 1 && gi == g.G - 2) || (g.G == 1 && jj == rows_in - 2)))
            flags |= DF_PENULT;
          // (the slot row's address; layout, leading byte offset and the extra pixel of shifted rows are in the K step table)
          const uint32_t row_lo = ((slots_addr + (uint32_t)slot * slot_bytes + (uint32_t)sub * row_bytes) & 0x3FFFFu) >> 4;
          const uint32_t wgrp = (uint32_t)g.gc0[gi] * 3u * N16;  // group's first chunk, in 16 byte units
          const uint32_t b_lo = (((w_addr & 0x3FFFFu) >> 4) + wgrp) | b_lo0;
          const uint32_t tfbar = (gi == g.G - 1 && vA) ? bar(ST_BAR_TFULL + bofs + blkA) : 0u;
          const uint32_t da = sbase + ST_OFF_DESC + (uint32_t)(bofs + slot) * ST_DESC_BYTES + (uint32_t)(sub * ST_SUBDESC_BYTES);
          sts16(da, make_uint4(row_lo, b_lo, flags, tfbar));
          sts16(da + 16, make_uint4(R0.col, R0.boff, R0.idesc, R1.col));
          // The row's fresh TMEM block must have been read out and zeroed before the MMAs of the row start.  The MMA
          // thread waits for that itself, right before it issues (barrier and parity ride in the descriptor): this
          // thread runs several entries ahead of the MMAs, and a wait here would claim the block that much earlier
          // than it is needed, which a ring of eight blocks cannot afford.
          const bool fresh = gi == 0 && vC;
          sts16(da + 32, make_uint4(R1.boff, R1.idesc, fresh ? bar(ST_BAR_TEMPTY + bofs + blkC) : 0u, cphase));
          if (DBG_TRACE_ON(g) && blockIdx.x == 0 && pipe == 0) trace(g, 2, dcount++, 5);
          if (sub == g.ER - 1) {
            mbar_arrive(bar(ST_BAR_FULL + bofs + slot));
            if (++slot == S) {
              slot = 0;
              ephase ^= 1u;
            }
          }
        }
        blkA = blkB;
        blkB = blkC;
        if (vC) {
          if (++blkC == NB) {
            blkC = 0;
            cphase ^= 1u;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
#ifdef DNXCU_DEBUG_AIDS
  if (g.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
    unsigned long long gt;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 2] = clock64();
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 4] = (long long)gt;
  }
#endif
#ifdef DNXCU_DEBUG_AIDS
  if (g.trace && threadIdx.x == 0 && dbg_cta < TRACE_CTAS)
    g.trace[3 * TRACE_ITERS * TRACE_EVENTS + 8 + dbg_cta] = clock64() - dbg_entry;
#endif
  abort_drain(abort_flag);
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base0), "r"(g.tmem_cols) : "memory");
  }
}

// ---- host side --------------------------------------------------------------

#ifdef DNXCU_DEBUG_AIDS
long long *g_trace_buffer = nullptr;
inline bool dbg_env(const char *name) {
  const char *v = getenv(name);
  return v && v[0] == '1';
}
#else
inline bool dbg_env(const char *) { return false; }
#endif

inline int pad16(int c) { return (c + 15) / 16 * 16; }
inline int nch_of(int c) { return c > 0 ? pad16(c) / 8 : 0; }

struct Plan {
  TcArgs args;
  size_t smem;
  int grid;
  int grid_y;  // output channel parts inside the launch (stacked form), else 1
  int no_sw;   // stacked form: the swizzled slot layout did not fit (its K groups are whole 32 channel blocks): plan without
  int R;
};

// Output channel parts inside one launch ("CSPLIT=n", v.p5): channels per part, a multiple of 16, the same for
// every part (the last part may hold fewer valid channels; its weights are zero padded).
int csplit_of(const Variant &v) { return (v.p0 == 0 && v.p5 > 1) ? v.p5 : 1; }
int csplit_n(const Variant &v, int K) {
  const int want = csplit_of(v);
  return ((K + want - 1) / want + 15) / 16 * 16;
}

constexpr size_t SMEM_LIMIT = 232448;  // 227 KB opt-in per block on sm_100

// SM count of the current device (cached per device; the first query of each device may race with another
// thread's, both then store the same value).
int sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const bool cacheable = dev >= 0 && dev < 64;
  int n = cacheable ? cache[dev].load(std::memory_order_relaxed) : 0;
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (cacheable) cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// H x W x C binary16 tensor as (8, W, C/8, H) with strides (2, 2C, 16, 2WC) bytes; box (8, 132, 2, 1).
int make_tensor_map(CUtensorMap *tm, const void *ptr, int H, int W, int C, int box_chunks, int box_px = WH) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DNXCU_E_CUDA;
  const cuuint64_t dims[4] = {8, (cuuint64_t)W, (cuuint64_t)(C / 8), (cuuint64_t)H};
  const cuuint64_t strides[3] = {(cuuint64_t)C * 2, 16, (cuuint64_t)W * C * 2};
  const cuuint32_t box[4] = {8, (cuuint32_t)box_px, (cuuint32_t)box_chunks, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    // A host thread that has made no runtime call yet has no context bound, which this driver entry point wants:
    // bind the device's primary context (what any runtime call that touches the device does) and try once more.
    if ((r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) || cudaFree(nullptr) != cudaSuccess) break;
  }
  return r == CUDA_SUCCESS ? DNXCU_OK : DNXCU_E_CUDA;
}

// (H/2) x (W/2) x C binary16 tensor read through a 2x nearest upsample in x: rank 5 view (8, 2, W/2, C/8, H/2) whose
// second dimension has stride 0, so a box of (8, 2, 66, chunks, 1) lands in shared memory as 132 pixels of 8
// channels per chunk: every source pixel twice.  (The rows are doubled by reading row y >> 1.)
int make_tensor_map_dup(CUtensorMap *tm, const void *ptr, int H2, int W2, int C, int box_chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DNXCU_E_CUDA;
  const cuuint64_t dims[5] = {8, 2, (cuuint64_t)W2, (cuuint64_t)(C / 8), (cuuint64_t)H2};
  const cuuint64_t strides[4] = {0, (cuuint64_t)C * 2, 16, (cuuint64_t)W2 * C * 2};
  const cuuint32_t box[5] = {8, 2, (cuuint32_t)(WH / 2), (cuuint32_t)box_chunks, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void *>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if ((r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) || cudaFree(nullptr) != cudaSuccess) break;
  }
  return r == CUDA_SUCCESS ? DNXCU_OK : DNXCU_E_CUDA;
}
// Pixel major views for the swizzled slot layout: rows of 32 channels (64 bytes), box (32, 136, blocks, 1), 64 byte
// swizzle; the copy engine then moves a quarter of the box rows it moves for 16 byte rows.
int make_tensor_map_sw(CUtensorMap *tm, const void *ptr, int H, int W, int C, int box_blocks, bool dup) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DNXCU_E_CUDA;
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    if (!dup) {
      const cuuint64_t dims[4] = {32, (cuuint64_t)W, (cuuint64_t)(C / 32), (cuuint64_t)H};
      const cuuint64_t strides[3] = {(cuuint64_t)C * 2, 64, (cuuint64_t)W * C * 2};
      const cuuint32_t box[4] = {32, (cuuint32_t)SW_PX, (cuuint32_t)box_blocks, 1};
      r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {  // (H, W: extent of the half resolution tensor)
      const cuuint64_t dims[5] = {32, 2, (cuuint64_t)W, (cuuint64_t)(C / 32), (cuuint64_t)H};
      const cuuint64_t strides[4] = {0, (cuuint64_t)C * 2, 64, (cuuint64_t)W * C * 2};
      const cuuint32_t box[5] = {32, 2, (cuuint32_t)(SW_PX / 2), (cuuint32_t)box_blocks, 1};
      r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void *>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if ((r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) || cudaFree(nullptr) != cudaSuccess) break;
  }
  return r == CUDA_SUCCESS ? DNXCU_OK : DNXCU_E_CUDA;
}
// The full resolution output as (K channels, x, y): box (K, 32, 1) = one epilogue warp's pixels of a row; the
// swizzle mode is the one whose span is a pixel's K * 2 bytes (K = 64: 128 bytes, K = 32: 64 bytes).
int make_tensor_map_out(CUtensorMap *tm, const void *ptr, int H, int W, int K) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return DNXCU_E_CUDA;
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)W, (cuuint64_t)H};
  const cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)W * K * 2};
  const cuuint32_t box[3] = {(cuuint32_t)K, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = CUDA_SUCCESS;
  for (int attempt = 0; attempt < 2; ++attempt) {
    r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, K == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if ((r != CUDA_ERROR_INVALID_CONTEXT && r != CUDA_ERROR_NOT_INITIALIZED) || cudaFree(nullptr) != cudaSuccess) break;
  }
  return r == CUDA_SUCCESS ? DNXCU_OK : DNXCU_E_CUDA;
}
// Whether the driver takes such maps: assumed until an encoding has failed once (then the producer warps expand
// upsampled operands inside shared memory, as before).
std::atomic<bool> g_dup_maps_ok{true};

// One row tensor maps for the halo rows of a row band, per operand that is fetched by TMA: the same box as the
// operand's own map (a half resolution row for an operand read through the 2x upsample).
int encode_halo_maps(TcArgs &g, int W) {
  memset(g.tm_halo, 0, sizeof(g.tm_halo));
  for (int sg = 0; sg < 2; ++sg) {
    const Seg &s = sg ? g.b : g.a;
    if (!s.tma || s.nch == 0) continue;
    if (s.sw) {
      const int Ws = s.dup ? W / 2 : W;
      if (s.top && make_tensor_map_sw(&g.tm_halo[sg * 2], s.top, 1, Ws, s.C, s.tbox, s.dup != 0)) return DNXCU_E_CUDA;
      if (s.bot && make_tensor_map_sw(&g.tm_halo[sg * 2 + 1], s.bot, 1, Ws, s.C, s.tbox, s.dup != 0)) return DNXCU_E_CUDA;
      continue;
    }
    if (s.dup) {
      if (s.top && make_tensor_map_dup(&g.tm_halo[sg * 2], s.top, 1, W / 2, s.C, s.tbox)) return DNXCU_E_CUDA;
      if (s.bot && make_tensor_map_dup(&g.tm_halo[sg * 2 + 1], s.bot, 1, W / 2, s.C, s.tbox)) return DNXCU_E_CUDA;
      continue;
    }
    const int Ws = s.up ? W / 2 : W, chunks = s.up ? 2 : s.tbox, px = s.up ? SRC_PX : WH;
    if (s.top && make_tensor_map(&g.tm_halo[sg * 2], s.top, 1, Ws, s.C, chunks, px)) return DNXCU_E_CUDA;
    if (s.bot && make_tensor_map(&g.tm_halo[sg * 2 + 1], s.bot, 1, Ws, s.C, chunks, px)) return DNXCU_E_CUDA;
  }
  return DNXCU_OK;
}

// Plan of the stacked form: weights resident, one K group, TMEM ring of NB blocks.
// Expects pl.args filled up to the operand description (done by make_plan).
int make_plan_stack(const Variant &v, const dnxcu_dispatch &d, Plan &pl, bool encode) {
  TcArgs &g = pl.args;
  const int W = g.W, H = g.H;
  g.cparts = 1;
  if (csplit_of(v) > 1) {
    // every part stages whole 16 byte pieces of its channels and starts on a 16 byte boundary of the pixel
    if (g.K % 8) return DNXCU_E_UNSUPPORTED;
    g.N = csplit_n(v, g.K);
    g.cparts = (g.K + g.N - 1) / g.N;
    if (g.cparts < 2) return DNXCU_E_UNSUPPORTED;  // nothing to split: the plain variant covers it
    g.parts = g.cparts;
  }
  if (g.N > 128) return DNXCU_E_UNSUPPORTED;
  g.Ns = g.N;
  g.wstream = 0;
  // A 2x upsampled operand of whole chunks comes through a pixel doubling tensor map when the other operand comes
  // by TMA too: the copy engine writes the upsampled row, and nothing is left for the producer warps to do.
  if (g.a.up && (g.a.C % 8) == 0 && !g.b.rg && (g.b.nch == 0 || g.b.tma) && g_dup_maps_ok.load(std::memory_order_relaxed) &&
      !dbg_env("DNXCU_TC_NO_DUP")) {
    g.a.dup = 1;
    g.a.tma = 1;
    g.cpa = 0;
    g.shift = 1;
  }
  const int nch = g.a.nch + g.b.nch;
  // K groups cost nothing here (every input row is used once): a slot holds one group of one row
  g.G = v.p1 > 0 ? v.p1 : 1;
  if (g.G > MAX_GROUPS) g.G = MAX_GROUPS;
  if (g.G * 2 > nch) g.G = nch / 2;
  {
    int per = (nch + g.G - 1) / g.G;
    per += per & 1;
    int c = 0, gi = 0;
    for (; gi < MAX_GROUPS && c < nch; ++gi) {
      g.gc0[gi] = c;
      g.gch[gi] = (nch - c < per) ? nch - c : per;
      c += g.gch[gi];
    }
    g.G = gi;
    for (; gi < MAX_GROUPS; ++gi) g.gc0[gi] = g.gch[gi] = 0;
    g.gmax = per < nch ? per : nch;
  }
  // Two input rows per ring entry ("ER=2"): halves the per-entry work of the single-thread roles (slot wait,
  // descriptor, slot release), which is what bounds thin layers.  Only where every row comes by one plain TMA
  // copy per operand: one K group, no upsampled or ragged operand, no halo rows, an even number of rows, and
  // at most six K steps per row (the straight line MMA forms).
  const int ER = v.p4 == 2 ? 2 : 1;
  if (ER == 2 && (g.cpa || g.a.up || g.G != 1 || (H & 1) || nch / 2 > 6)) return DNXCU_E_UNSUPPORTED;
  g.ER = ER;
  // Slot layout per operand.  Everything by TMA, one input row per entry, an operand of whole 32 channel blocks:
  // pixel major rows with the 64 byte swizzle.  With K groups every operand must be of that kind, and the groups
  // are made of whole blocks.
  g.a.sw = g.b.sw = 0;
  if (!g.cpa && ER == 1 && !pl.no_sw && !dbg_env("DNXCU_TC_NO_SW")) {
    const bool a_sw = g.a.C % 32 == 0, b_sw = g.b.nch > 0 && g.b.C % 32 == 0;
    if (g.G == 1) {
      g.a.sw = a_sw;
      g.b.sw = b_sw;
    } else if (a_sw && (g.b.nch == 0 || b_sw)) {
      int per = (nch + g.G - 1) / g.G;
      per = (per + 3) / 4 * 4;
      int c = 0, gi = 0;
      for (; gi < MAX_GROUPS && c < nch; ++gi) {
        g.gc0[gi] = c;
        g.gch[gi] = (nch - c < per) ? nch - c : per;
        c += g.gch[gi];
      }
      g.G = gi;
      for (; gi < MAX_GROUPS; ++gi) g.gc0[gi] = g.gch[gi] = 0;
      g.gmax = per < nch ? per : nch;
      g.a.sw = 1;
      g.b.sw = g.b.nch > 0;
    }
  }
  g.swmode = (g.a.sw || g.b.sw) ? 1 : 0;
  // chunks (16 byte layout) or blocks (swizzled layout) per TMA copy: the operand's whole row when a slot holds all
  // channels, else two chunks / one block
  g.a.tbox = g.a.sw ? (g.G == 1 ? g.a.nch / 4 : 1) : ((g.G == 1) ? g.a.nch : 2);
  g.b.tbox = g.b.sw ? (g.G == 1 ? g.b.nch / 4 : 1) : ((g.G == 1 && g.b.nch) ? g.b.nch : 2);
  // the slot row and the K step table of an entry
  {
    const uint32_t hi16 = (128u >> 4) | (1u << 14);                 // 16 byte layout: stride 128 bytes, version 1
    const uint32_t hisw = (512u >> 4) | (1u << 14) | (4u << 29);    // swizzled: stride 512 bytes, version 1, 64 byte swizzle
    const uint32_t lbo16 = ((uint32_t)CHUNK_PITCH >> 4) << 16, lbosw = 1u << 16;
    const uint32_t sh16 = g.shift ? 1u : 0u, shsw = g.shift ? 4u : 0u;  // rows that start one pixel early
    for (int kc = 0; kc < 16; ++kc) {
      g.kst_lo[kc] = ((uint32_t)kc * ((2u * CHUNK_PITCH) >> 4) + sh16) | lbo16;
      g.kst_hi[kc] = hi16;
      g.kst_dx[kc] = 1;
    }
    g.seg_off[0] = g.seg_off[1] = 0;
    g.row_bytes = (uint32_t)g.gmax * CHUNK_PITCH;
    if (g.swmode && g.G > 1) {
      g.row_bytes = (uint32_t)g.gmax * SW_CHUNK;
      for (int kc = 0; kc < 16; ++kc) {
        g.kst_lo[kc] = ((((uint32_t)(kc >> 1) * SW_BLOCK + (uint32_t)(kc & 1) * 32u) >> 4) + shsw) | lbosw;
        g.kst_hi[kc] = hisw;
        g.kst_dx[kc] = 4;
      }
    } else if (g.swmode) {
      // swizzled areas first (they want 512 byte boundaries), then the 16 byte chunks
      uint32_t off = 0;
      if (g.a.sw) { g.seg_off[0] = off; off += (uint32_t)(g.a.nch / 4) * SW_BLOCK; }
      if (g.b.sw) { g.seg_off[1] = off; off += (uint32_t)(g.b.nch / 4) * SW_BLOCK; }
      if (!g.a.sw) { g.seg_off[0] = off; off += (uint32_t)g.a.nch * CHUNK_PITCH; }
      if (g.b.nch > 0 && !g.b.sw) { g.seg_off[1] = off; off += (uint32_t)g.b.nch * CHUNK_PITCH; }
      g.row_bytes = (off + 511u) & ~511u;
      int kc = 0;
      for (int sg = 0; sg < 2; ++sg) {
        const Seg &s = sg ? g.b : g.a;
        for (int j = 0; j < s.nch / 2 && kc < 16; ++j, ++kc) {
          if (s.sw) {
            g.kst_lo[kc] = (((g.seg_off[sg] + (uint32_t)(j >> 1) * SW_BLOCK + (uint32_t)(j & 1) * 32u) >> 4) + shsw) | lbosw;
            g.kst_hi[kc] = hisw;
            g.kst_dx[kc] = 4;
          } else {
            g.kst_lo[kc] = (((g.seg_off[sg] + (uint32_t)j * 2u * CHUNK_PITCH) >> 4) + sh16) | lbo16;
            g.kst_hi[kc] = hi16;
            g.kst_dx[kc] = 1;
          }
        }
      }
      if (nch / 2 > 16) return DNXCU_E_UNSUPPORTED;
    }
  }
  // the copies of an entry, per K group (used when everything comes by TMA)
  for (int gi = 0; gi < MAX_GROUPS; ++gi) {
    g.ncp[gi] = 0;
    g.grp_tx[gi] = 0;
    if (gi >= g.G) continue;
    const int c_lo = g.gc0[gi], c_hi = c_lo + g.gch[gi];
    for (int sg = 0; sg < 2; ++sg) {
      const Seg &s = sg ? g.b : g.a;
      const int first = sg ? g.a.nch : 0;
      const int lo = c_lo > first ? c_lo : first, hi = c_hi < first + s.nch ? c_hi : first + s.nch;
      if (hi <= lo) continue;
      const uint32_t per = s.sw ? (uint32_t)SW_CHUNK : (uint32_t)CHUNK_PITCH;
      uint32_t area;
      if (!g.swmode) area = (uint32_t)(lo - c_lo) * CHUNK_PITCH;
      else if (g.G == 1) area = g.seg_off[sg];
      else area = (uint32_t)(lo - c_lo) * SW_CHUNK;
      const int step = s.sw ? 4 * s.tbox : s.tbox;
      for (int c = lo; c < hi; c += step) {
        if (g.ncp[gi] >= 8) return DNXCU_E_UNSUPPORTED;
        TcArgs::Copy &cp = g.cp[gi][g.ncp[gi]++];
        cp.dst = area + (uint32_t)(c - lo) * per;
        cp.unit = (short)(s.sw ? (c - first) >> 2 : c - first);
        cp.sg = (unsigned char)sg;
        cp.pad = 0;
      }
      g.grp_tx[gi] += (uint32_t)(hi - lo) * per;
    }
  }
  const size_t wbytes = (size_t)9 * nch * g.N * 16;
  if (wbytes >= (1u << 20)) return DNXCU_E_UNSUPPORTED;
  const size_t wregion = (wbytes + 127) & ~(size_t)127;
  // Shared memory budget.  Wanted, in this order of importance: four input slots; the epilogue staging tiles
  // (4 warps per pipeline x 32 pixels x (K*2 + 16) bytes, two rows when pooling); expand mode for an upsampled
  // operand a (TMA at half resolution + one staging buffer per slot); a second pipeline (eight slots).
  // "fix-up" mode: the copy engine brings every row (a half resolution row of an upsampled operand, the raw
  // bytes of a ragged one, a plain operand's row as it is) and the producer warps put it right inside shared
  // memory.  Possible when at least one operand needs that and each operand is one of the three kinds.
  const bool a_up_ok = g.a.up && (g.a.C % 8) == 0;
  const bool a_kind_ok = a_up_ok || g.a.rg || (!g.a.up && g.a.tma);
  const bool b_kind_ok = g.b.nch == 0 || g.b.tma || g.b.rg;
  const bool xp_possible = !g.a.dup && (a_up_ok || g.a.rg || g.b.rg) && a_kind_ok && b_kind_ok &&
                           !dbg_env("DNXCU_TC_NO_EXPAND") && !dbg_env("DNXCU_TC_NO_TMA");
  uint32_t xp_src_bytes = 0;
  if (xp_possible) {
    int amax = 0;
    for (int gi = 0; gi < g.G; ++gi) {
      const int lo = g.gc0[gi] < g.a.nch ? g.gc0[gi] : g.a.nch;
      const int hi = g.gc0[gi] + g.gch[gi] < g.a.nch ? g.gc0[gi] + g.gch[gi] : g.a.nch;
      if (hi - lo > amax) amax = hi - lo;
    }
    xp_src_bytes = 0;  // the half resolution rows land in the slot itself and are expanded in place
    (void)amax;
  }
  const bool stage_possible = g.K % 8 == 0 && !dbg_env("DNXCU_TC_NO_STAGE");
  // Full resolution rows of 32 or 64 channels leave through the copy engine: one tensor copy per warp and row out
  // of an unpadded tile whose 16 byte pieces are swizzled the way the tensor map says (which keeps the staging
  // writes free of bank conflicts, as the padding does for the other shapes).
  const int out_tma = (stage_possible && g.full_out && g.cparts == 1 && g.parts == 1 && g.os == g.K && (g.K == 32 || g.K == 64) &&
                       !dbg_env("DNXCU_TC_NO_OTMA"))
                          ? (g.K == 64 ? 1 : 2)
                          : 0;
  const size_t stage_pitch = out_tma ? (size_t)g.K * 2 : (size_t)(g.cparts > 1 ? g.N : g.K) * 2 + 16;
  // two tiles per warp where a row pair is staged in one go: with the fused pool (which needs both rows), and for
  // thin layers, whose tiles are small and whose epilogue is what bounds them
  const bool two_tiles = g.pool || (g.N <= 32 && !dbg_env("DNXCU_TC_ONE_TILE"));
  const size_t stage_per_warp = (two_tiles ? 2 : 1) * 32 * stage_pitch;
  const size_t base_bytes = ST_HEADER_BYTES + wregion + 1024 + (out_tma ? 1024 : 0);  // (the slots start on a 1024 byte boundary, swizzled staging tiles too)
  const size_t plain_slot = (size_t)g.row_bytes * ER;
  // v.p2 == 2 ("PIPES=1"): one pipeline with a longer slot ring even where two would fit
  const bool p2_possible = 4 * g.N <= 256 && !dbg_env("DNXCU_TC_PIPES") && v.p2 != 2;
  // candidate configurations, best first: (pipelines, expand, staging)
  int P = 0;
  size_t slot_bytes = 0, stage_total = 0;
  int total_slots = 0;
  g.eteams = 1;
  // one pipeline: a second epilogue team when its staging tiles fit (the second row of `tries` entries)
  const int tries[16][4] = {{2, 1, 1, 1}, {1, 1, 1, 2}, {1, 1, 1, 1}, {2, 1, 0, 1}, {1, 1, 0, 2}, {2, 0, 1, 1}, {1, 0, 1, 2}, {1, 0, 1, 1},
                            {2, 0, 0, 1}, {1, 0, 0, 2}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
  const bool teams2_ok = ER == 1 && !dbg_env("DNXCU_TC_ONE_TEAM");
  for (int ti = 0; ti < 16 && P == 0; ++ti) {
    const int tp = tries[ti][0], txp = tries[ti][1], tst = tries[ti][2], tt = tries[ti][3];
    if (tp == 0) break;
    if (tt == 2 && (!teams2_ok || txp)) continue;  // (expand mode: the tiles would cost input slots, which count for more there)
    if (tp == 2 && !p2_possible) continue;
    {
      // two rows per entry keep four accumulator blocks in use at once: the ring must leave the epilogue room
      const int nb = tp == 2 ? (256 / g.N < ST_PIPE_STRIDE ? 256 / g.N : ST_PIPE_STRIDE)
                             : (512 / g.N < ST_MAX_BLOCKS ? 512 / g.N : ST_MAX_BLOCKS);
      if (ER == 2 && nb < 6) continue;
    }
    if (txp != (xp_possible ? 1 : 0) && txp == 1) continue;
    if (tst && !stage_possible) continue;
    const size_t sb = plain_slot + (txp ? xp_src_bytes : 0);
    const size_t st = tst ? (size_t)4 * tp * tt * stage_per_warp : 0;
    const int min_slots = ER == 2 ? 2 : (tp == 2 ? 3 : 4);  // two issuing threads pay for a shorter ring
    if (base_bytes + st + (size_t)min_slots * tp * sb > SMEM_LIMIT) continue;
    P = tp;
    g.eteams = tt;
    slot_bytes = sb;
    stage_total = st;
    total_slots = (int)((SMEM_LIMIT - base_bytes - st) / sb);
    g.xp = txp;
    g.src_bytes = txp ? xp_src_bytes : 0;
    g.stage_pitch = tst ? (int)stage_pitch : 0;
    g.stage2 = (tst && two_tiles) ? 1 : 0;
    g.out_tma = tst ? out_tma : 0;
    g.stage_warp_bytes = tst ? (uint32_t)stage_per_warp : 0;
  }
  if (P == 0 && g.swmode && !pl.no_sw) {
    pl.no_sw = 1;  // (groups of whole blocks can make the slots larger than the 16 byte layout would)
    return make_plan_stack(v, d, pl, encode);
  }
  if (P == 0) return DNXCU_E_UNSUPPORTED;
  if (g.xp) {
    g.cpa = 1;
    if (g.a.up) g.a.tma = 1;  // by TMA at half resolution
  } else {
    g.a.rg = g.b.rg = 0;  // without the fix-up mode ragged operands are loaded by the producer warps
  }
  g.nstrips = (W + STRIP - 1) / STRIP;
  g.P = P;
  if (P == 2) {
    g.NB = 256 / g.N;
    if (g.NB > ST_PIPE_STRIDE) g.NB = ST_PIPE_STRIDE;
    g.S = total_slots / 2 < ST_PIPE_STRIDE ? total_slots / 2 : ST_PIPE_STRIDE;
  } else {
    g.NB = 512 / g.N;
    if (g.NB > ST_MAX_BLOCKS) g.NB = ST_MAX_BLOCKS;
    g.S = total_slots < MAX_SLOTS ? total_slots : MAX_SLOTS;
  }
  // One pipeline: two MMA threads take alternate entries (each entry is one input row of one K group).  Not in
  // fix-up mode: there the producer warps' work in shared memory bounds the kernel, and a second polling thread
  // only takes shared memory cycles away from them (measured: 5-20 % slower).
  g.ab = (ER == 1 && g.S >= 2 && !g.xp && (P == 1 || !g.cpa) && !dbg_env("DNXCU_TC_ONE_ISSUER")) ? 1 : 0;
  uint32_t p2 = 32;
  while (p2 < (uint32_t)(P * g.NB * g.N)) p2 <<= 1;
  g.tmem_cols = p2;
  g.D = g.S - 1 < MAX_DEPTH ? g.S - 1 : MAX_DEPTH;
  pl.smem = ST_HEADER_BYTES + wregion + 1024 + (g.out_tma ? 1024 : 0) + (size_t)P * g.S * slot_bytes + stage_total;
  const int sms = g.parts > 1 ? (sm_count() / g.parts > 0 ? sm_count() / g.parts : 1) : sm_count();
  const int lanes = sms * P;
  double best = 1e30;
  int bestRB = 2;
  for (int rb = 2; rb <= 64; rb += 2) {
    const long long units = (long long)g.nstrips * ((H + rb - 1) / rb);
    const long long waves = (units + lanes - 1) / lanes;
    const double cost = (double)waves * (rb + 2.5);
    if (cost < best - 1e-9) {
      best = cost;
      bestRB = rb;
    }
  }
  g.RB = bestRB;
  g.nunits = g.nstrips * ((H + g.RB - 1) / g.RB);
  pl.grid = g.nunits < sms ? g.nunits : sms;  // spread first: a second unit per SM only when every SM has one
  g.cut_L = g.cut_R = g.cut_nb = g.cut_pad = 0;
  // More units than pipelines: blocks of RB rows leave the last wave partly empty and pay two halo rows per unit
  // (1088 rows x 15 strips on 148 SMs: 3 units of 38 rows + 6 halo rows where 110.3 rows are the fair share).
  // Instead cut the rows of all strips, laid end to end, into one range per pipeline: two halo rows per range,
  // four for the few ranges that cross into the next strip.  (Row pairs stay together where the pool or a two
  // row entry needs them.)
  if (g.nunits > lanes && !dbg_env("DNXCU_TC_NO_CUT")) {
    const int step = (g.pool || ER == 2 || (H & 1)) ? 2 : 1;
    const int pad = step == 2 ? 4 : 3;
    const int Hp = H + pad;
    const long long T = (long long)g.nstrips * Hp - pad;
    int L = (int)((T + lanes - 1) / lanes);
    L = (L + step - 1) / step * step;
    for (int attempt = 0; attempt < 8 && !g.cut_L; ++attempt, L += step) {
      const int R = (int)((T + L - 1) / L);
      if (R % P != 0 || R > lanes || L > H || L <= pad || (step == 2 && (H & 1))) continue;
      int nb = 0;
      bool fits = true;
      for (int r = 0; r < R && fits; ++r) {
        const long long v0 = (long long)r * L, v1 = v0 + L < T ? v0 + L : T;
        long long s0 = v0 / Hp;
        if (v0 - s0 * Hp >= H) ++s0;
        const long long s1 = (v1 - 1) / Hp;
        if (s1 != s0) {
          if (nb < 32) g.cut_x[nb] = (short)r;
          else fits = false;
          ++nb;
        }
      }
      if (!fits || R > 32767) continue;
      const double cost = (double)L + 2.5;
      if (cost >= best) break;
      g.cut_L = L;
      g.cut_R = R;
      g.cut_nb = nb;
      g.cut_pad = pad;
      g.nunits = R + nb;
      pl.grid = R / P;
    }
  }
  pl.grid_y = g.cparts;
  pl.R = 0;
  memset(&g.tm_a, 0, sizeof(g.tm_a));
  memset(&g.tm_b, 0, sizeof(g.tm_b));
  memset(g.tm_halo, 0, sizeof(g.tm_halo));
  memset(&g.tm_out, 0, sizeof(g.tm_out));
  if (encode) {
    if (g.out_tma && make_tensor_map_out(&g.tm_out, d.out, H, W, g.K)) return DNXCU_E_CUDA;
    if (g.a.sw) {
      if (make_tensor_map_sw(&g.tm_a, d.in_a, g.a.dup ? H / 2 : H, g.a.dup ? W / 2 : W, d.c_a, g.a.tbox, g.a.dup != 0)) return DNXCU_E_CUDA;
    } else if (g.a.dup) {
      if (make_tensor_map_dup(&g.tm_a, d.in_a, H / 2, W / 2, d.c_a, g.a.tbox)) {
        // this driver does not take a zero stride: plan again, with the expansion inside shared memory
        g_dup_maps_ok.store(false, std::memory_order_relaxed);
        g.a.dup = 0;
        g.a.tma = 0;
        g.cpa = 1;
        g.shift = 0;
        return make_plan_stack(v, d, pl, encode);
      }
    } else if (g.xp && g.a.up) {
      if (make_tensor_map(&g.tm_a, d.in_a, H / 2, W / 2, d.c_a, 2, SRC_PX)) return DNXCU_E_CUDA;
    } else if (g.a.tma && make_tensor_map(&g.tm_a, d.in_a, H, W, d.c_a, g.a.tbox)) {
      return DNXCU_E_CUDA;
    }
    if (g.b.sw) {
      if (make_tensor_map_sw(&g.tm_b, d.in_b, H, W, d.c_b, g.b.tbox, false)) return DNXCU_E_CUDA;
    } else if (g.b.tma && make_tensor_map(&g.tm_b, d.in_b, H, W, d.c_b, g.b.tbox)) {
      return DNXCU_E_CUDA;
    }
    if (encode_halo_maps(g, W)) return DNXCU_E_CUDA;
  }
  return DNXCU_OK;
}

// v.p0 = R (rows per pass), v.p1 = K groups, v.p2 = weight mode (0 resident, 1 streamed; stacked form: 2 = one
// pipeline only), v.p3 = weight stages (stacked form: output channel split)
int make_plan(const Variant &v, const dnxcu_dispatch &d, Plan &pl, bool encode, int os_override = 0, int parts = 1) {
  if (!d.in_a || !d.weights || d.c_a <= 0 || d.c_out <= 0 || d.c_b < 0) return DNXCU_E_BAD_ARG;
  if (d.pc[0] == 0 || d.pc[1] == 0) return DNXCU_E_BAD_ARG;
  if (d.c_b > 0 && !d.in_b) return DNXCU_E_BAD_ARG;
  if ((d.flags & DNXCU_F_BIAS) && !d.bias) return DNXCU_E_BAD_ARG;
  const int W = (int)d.pc[0], H = (int)d.pc[1];
  const bool up = d.flags & DNXCU_F_UP2X_A, pool = d.flags & DNXCU_F_POOL_OUT;
  const bool full = !(d.flags & DNXCU_F_NO_FULL_OUT);
  if ((d.flags & DNXCU_F_NO_FULL_OUT) && !pool) return DNXCU_E_BAD_ARG;
  if (full && !d.out) return DNXCU_E_BAD_ARG;
  if (pool && !d.out_pool) return DNXCU_E_BAD_ARG;
  if ((up || pool) && ((W | H) & 1)) return DNXCU_E_BAD_ARG;
  const int R = v.p0;  // 0 selects the stacked form
  if (pool && R == 1) return DNXCU_E_UNSUPPORTED;
  if (d.c_out > 256) return DNXCU_E_UNSUPPORTED;
  // 16 byte rules: vector loads of operands with C % 8 == 0, vector stores when K % 8 == 0, bulk weight copies
  if ((uintptr_t)d.weights & 15) return DNXCU_E_MISALIGNED;
  if ((d.c_a % 8 == 0) && (((uintptr_t)d.in_a | (uintptr_t)d.halo[0] | (uintptr_t)d.halo[1]) & 15))
    return DNXCU_E_MISALIGNED;
  if (d.c_b > 0 && (d.c_b % 8 == 0) && (((uintptr_t)d.in_b | (uintptr_t)d.halo[2] | (uintptr_t)d.halo[3]) & 15))
    return DNXCU_E_MISALIGNED;
  if ((d.c_out % 8 == 0) && (((uintptr_t)d.out | (uintptr_t)d.out_pool) & 15)) return DNXCU_E_MISALIGNED;
  if (((uintptr_t)d.in_a | (uintptr_t)d.in_b | (uintptr_t)d.out | (uintptr_t)d.out_pool | (uintptr_t)d.bias) & 1)
    return DNXCU_E_MISALIGNED;

  pl.grid_y = 1;
  pl.no_sw = 0;
  TcArgs &g = pl.args;
  g.a = {(const __half *)d.in_a, (const __half *)d.halo[0], (const __half *)d.halo[1], d.c_a, nch_of(d.c_a), up ? 1 : 0, 0, 2, 0, 0, 0};
  g.b = {(const __half *)d.in_b, (const __half *)d.halo[2], (const __half *)d.halo[3], d.c_b, nch_of(d.c_b), 0, 0, 2, 0, 0, 0};
  g.shift = 0;
  // TMA takes the operands whose pixels are whole 16 byte chunks at full resolution
  const bool allow_tma = !dbg_env("DNXCU_TC_NO_TMA");
  g.a.tma = allow_tma && !up && (d.c_a % 8 == 0);
  g.b.tma = allow_tma && d.c_b > 0 && (d.c_b % 8 == 0);
  // ragged operands of at most 16 channels (the 9 channel colour / albedo / normal input): raw row bytes by bulk
  // copy, re-laid in shared memory (stacked form).  Bulk copies move whole 16 byte pieces from 16 byte aligned
  // addresses, so the tensor must start on such an address and end on one.
  auto raggable = [&](const void *ptr, int C, bool upsampled) {
    return allow_tma && !upsampled && C > 0 && (C % 8) != 0 && C <= 16 && ((uintptr_t)ptr & 15) == 0 &&
           ((size_t)H * W * C * 2) % 16 == 0;
  };
  g.a.rg = raggable(d.in_a, d.c_a, up) ? 1 : 0;
  g.b.rg = raggable(d.in_b, d.c_b, false) ? 1 : 0;
  // the producer warps copy what the copy engine cannot: operands without a tensor map (halo rows of operands
  // with one come through one row tensor maps of their own)
  g.cpa = (!g.a.tma || (d.c_b > 0 && !g.b.tma)) ? 1 : 0;
  g.w = (const __half *)d.weights;
  g.bias = (d.flags & DNXCU_F_BIAS) ? (const __half *)d.bias : nullptr;
  g.out = (__half *)d.out;
  g.out_pool = (__half *)d.out_pool;
  g.status = d.device_status;
  g.H = H;
  g.W = W;
  g.K = d.c_out;
  g.os = os_override ? os_override : d.c_out;
  g.N = pad16(d.c_out);
  g.Ns = (g.N + 31) / 32 * 32;
  g.relu = (d.flags & (DNXCU_F_RELU | DNXCU_F_LEAKY)) ? 1 : 0;
  g.leaky = (d.flags & DNXCU_F_LEAKY) ? 1 : 0;
  {
    const uint32_t ah = __half_as_ushort(__float2half_rn(d.leaky_alpha));
    g.alpha_h2 = ah | (ah << 16);
  }
  g.pool = pool ? 1 : 0;
  g.full_out = full ? 1 : 0;
  g.wstream = v.p2 == 1 ? 1 : 0;
  g.parts = parts;
  g.WST = v.p3 > 0 ? v.p3 : 2;
  if (g.WST > MAX_WST) g.WST = MAX_WST;
  g.wait_limit = wait_limit_cycles();
  if (g.wait_limit < 2000000ull) g.wait_limit |= 1ull << 63;  // below about a millisecond: strict (see mbar_wait)
#ifdef DNXCU_DEBUG_AIDS
  g.desc_swap = dbg_env("DNXCU_TC_DESC_SWAP") ? 1 : 0;
  const char *sk = getenv("DNXCU_TC_SKIP");
  g.skip = sk ? atoi(sk) : 0;
  g.switch_issue = dbg_env("DNXCU_TC_SWITCH_ISSUE") ? 1 : 0;
  g.loop_issue = dbg_env("DNXCU_TC_LOOP_ISSUE") ? 1 : 0;
  // time line tracing writes to a buffer of its own, handed over by dnxcu_debug_trace_buffer (size checked there)
  g.trace = dbg_env("DNXCU_TC_TRACE") ? g_trace_buffer : nullptr;
#endif

  if (R == 0) return make_plan_stack(v, d, pl, encode);
  g.a.rg = g.b.rg = 0;  // the pass kernel loads ragged operands with its producer warps
  g.ER = 1;
  g.cparts = 1;
  g.ab = 0;
  g.eteams = 1;
  g.stage2 = 0;
  g.out_tma = 0;
  g.cut_L = g.cut_R = g.cut_nb = g.cut_pad = 0;
  uint32_t cols = 2u * R * g.Ns;
  if (cols > 512) return DNXCU_E_UNSUPPORTED;
  uint32_t p2 = 32;
  while (p2 < cols) p2 <<= 1;
  g.tmem_cols = p2;

  // K groups: contiguous runs of 8 channel chunks (even counts: one MMA takes two chunks)
  const int nch = g.a.nch + g.b.nch;
  g.G = v.p1 > 0 ? v.p1 : 1;
  if (g.G > MAX_GROUPS) g.G = MAX_GROUPS;
  if (g.G * 2 > nch) g.G = nch / 2;
  {
    int per = (nch + g.G - 1) / g.G;
    per += per & 1;
    int c = 0, gi = 0;
    for (; gi < MAX_GROUPS && c < nch; ++gi) {
      g.gc0[gi] = c;
      g.gch[gi] = (nch - c < per) ? nch - c : per;
      c += g.gch[gi];
    }
    g.G = gi;
    for (; gi < MAX_GROUPS; ++gi) g.gc0[gi] = g.gch[gi] = 0;
    g.gmax = per < nch ? per : nch;
  }

  const size_t wtap = (size_t)nch * g.N * 16;
  const size_t wstage = (size_t)g.gmax * g.N * 16;
  const size_t wregion = ((g.wstream ? wstage * g.WST : wtap * 9) + 127) & ~(size_t)127;
  if (wtap * 9 >= (1u << 20)) return DNXCU_E_UNSUPPORTED;  // mbarrier transaction count limit
  const size_t slot_bytes = (size_t)g.gmax * CHUNK_PITCH;
  if (HEADER_BYTES + wregion + (size_t)(R + 3) * slot_bytes > SMEM_LIMIT) return DNXCU_E_UNSUPPORTED;
  int S = (int)((SMEM_LIMIT - HEADER_BYTES - wregion) / slot_bytes);
  if (S > MAX_SLOTS) S = MAX_SLOTS;
  g.S = S;
  g.D = S - (R + 2);
  if (g.D > MAX_DEPTH) g.D = MAX_DEPTH;
  if (g.D < 1) g.D = 1;
  pl.smem = HEADER_BYTES + wregion + (size_t)S * slot_bytes;

  // rows per unit: whole waves of CTAs with little halo re-read
  g.nstrips = (W + STRIP - 1) / STRIP;
  const int sms = sm_count();
  const int step = (R > 2 ? R : 2);
  if (g.G > 1) {
    g.RB = R;  // nothing is reused across passes: the smallest unit balances best
  } else {
    double best = 1e30;
    int bestRB = step;
    for (int rb = step; rb <= 64; rb += step) {
      const long long units = (long long)g.nstrips * ((H + rb - 1) / rb);
      const long long waves = (units + sms - 1) / sms;
      const double cost = (double)waves * (rb + 2.5);
      if (cost < best - 1e-9) {
        best = cost;
        bestRB = rb;
      }
    }
    g.RB = bestRB;
  }
  g.nunits = g.nstrips * ((H + g.RB - 1) / g.RB);
  pl.grid = g.nunits < sms ? g.nunits : sms;
  pl.R = R;
  memset(&g.tm_a, 0, sizeof(g.tm_a));
  memset(&g.tm_b, 0, sizeof(g.tm_b));
  memset(g.tm_halo, 0, sizeof(g.tm_halo));
  if (encode) {
    if (g.a.tma && make_tensor_map(&g.tm_a, d.in_a, H, W, d.c_a, g.a.tbox)) return DNXCU_E_CUDA;
    if (g.b.tma && make_tensor_map(&g.tm_b, d.in_b, H, W, d.c_b, g.b.tbox)) return DNXCU_E_CUDA;
    if (encode_halo_maps(g, W)) return DNXCU_E_CUDA;
  }
  return DNXCU_OK;
}

// Raises the kernel's dynamic shared memory limit once per device (under a lock: callers on several threads).
template <class K>
int ensure_smem_attr(K kernel, std::atomic<bool> (&done)[64]) {
  int dev = 0;
  DNXCU_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && done[dev].load(std::memory_order_acquire)) return DNXCU_OK;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  DNXCU_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT));
  if (dev >= 0 && dev < 64) done[dev].store(true, std::memory_order_release);
  return DNXCU_OK;
}

template <int R>
int launch_r(const Plan &pl, cudaStream_t s, bool attr_only = false) {
  static std::atomic<bool> done[64];
  int st = ensure_smem_attr(conv3x3_tc<R>, done);
  if (st || attr_only) return st;
  conv3x3_tc<R><<<pl.grid, THREADS, pl.smem, s>>>(pl.args);
  DNXCU_CUDA(cudaGetLastError());
  return DNXCU_OK;
}

template <int EPI>
int launch_stack_epi(const Plan &pl, cudaStream_t s, bool attr_only = false) {
  static std::atomic<bool> done[64];
  int st = ensure_smem_attr(conv3x3_tc_stack<EPI>, done);
  if (st || attr_only) return st;
  conv3x3_tc_stack<EPI><<<dim3((unsigned)pl.grid, (unsigned)pl.grid_y), ST_THREADS, pl.smem, s>>>(pl.args);
  DNXCU_CUDA(cudaGetLastError());
  return DNXCU_OK;
}

int launch_stack(const Plan &pl, cudaStream_t s) {
  const TcArgs &g = pl.args;
  const int epi = (g.bias ? EPI_BIAS : 0) | (g.relu ? EPI_RELU : 0) | (g.pool ? EPI_POOL : 0) | (g.full_out ? EPI_FULL : 0);
  switch (epi) {
#define DNXCU_EPI_CASE(E) case E: return launch_stack_epi<E>(pl, s);
    DNXCU_EPI_CASE(8) DNXCU_EPI_CASE(9) DNXCU_EPI_CASE(10) DNXCU_EPI_CASE(11)
    DNXCU_EPI_CASE(4) DNXCU_EPI_CASE(5) DNXCU_EPI_CASE(6) DNXCU_EPI_CASE(7)
    DNXCU_EPI_CASE(12) DNXCU_EPI_CASE(13) DNXCU_EPI_CASE(14) DNXCU_EPI_CASE(15)
#undef DNXCU_EPI_CASE
    default: return DNXCU_E_BAD_ARG;
  }
}

// Output channel split of the stacked form (variant parameter p3 = parts): a layer whose weights do not fit
// in shared memory runs as several launches, each producing a run of output channels (a multiple of 16) with
// its own resident weights; the outputs interleave through the pixel stride.
int split_parts(const Variant &v, int K, int k0[8], int kp[8]) {
  const int want = (v.p0 == 0 && v.p3 > 1) ? v.p3 : 1;
  const int np = ((K + want - 1) / want + 15) / 16 * 16;
  int n = 0;
  for (int c = 0; c < K && n < 8; c += np, ++n) {
    k0[n] = c;
    kp[n] = K - c < np ? K - c : np;
  }
  return n;
}

}  // namespace

size_t conv_tc_weight_bytes(const Variant &v, int k, int ca, int cb) {
  int k0[8], kp[8];
  const int n = split_parts(v, k, k0, kp);
  if (csplit_of(v) > 1) {
    const int np = csplit_n(v, k);
    return (size_t)9 * (nch_of(ca) + nch_of(cb)) * np * 16 * ((k + np - 1) / np);
  }
  size_t total = 0;
  for (int p = 0; p < n; ++p) total += (size_t)9 * (nch_of(ca) + nch_of(cb)) * pad16(kp[p]) * 16;
  return total;
}

// KCRS -> the shared memory image of the MMA's B operand, operand a's chunks first, each operand's channel
// count padded to a multiple of 16 and the output channels to a multiple of 16, zero filled.  Plays the role
// of the RSCKC16 / KRSCK16 re-layouts of the reference (common/src/denox/memory/tensor/FilterLayout.hpp:74-78,104-108).
//   pass variants:    [tap][chunk c8][n][8]
//   stacked variants: [dx][chunk c8][3N rows][8], the rows of a chunk being the three vertical taps r = 2, 1, 0
//                     one after the other (matching output rows j-1, j, j+1 of input row j); one such blob per
//                     output channel part
void conv_tc_prepare(const Variant &v, const uint16_t *kcrs, int K, int ca, int cb, uint16_t *out) {
  const int C = ca + cb, nch = nch_of(ca) + nch_of(cb);
  const size_t total = conv_tc_weight_bytes(v, K, ca, cb) / 2;
  for (size_t i = 0; i < total; ++i) out[i] = 0;
  if (v.p0 == 0) {
    int k0[8], kp[8];
    int n = split_parts(v, K, k0, kp);
    const int cs_n = csplit_of(v) > 1 ? csplit_n(v, K) : 0;
    if (cs_n) {  // parts of one launch: every part cs_n channels wide
      n = 0;
      for (int c = 0; c < K && n < 8; c += cs_n, ++n) {
        k0[n] = c;
        kp[n] = K - c < cs_n ? K - c : cs_n;
      }
    }
    size_t off = 0;
    for (int p = 0; p < n; ++p) {
      const int N = cs_n ? cs_n : pad16(kp[p]);
      for (int seg = 0; seg < 2; ++seg) {
        const int Cs = seg ? cb : ca, cbase = seg ? ca : 0, chbase = seg ? nch_of(ca) : 0;
        for (int r = 0; r < 3; ++r)
          for (int sx = 0; sx < 3; ++sx)
            for (int c = 0; c < Cs; ++c)
              for (int k = 0; k < kp[p]; ++k)
                out[off + ((((size_t)sx * nch + chbase + c / 8) * 3 + (2 - r)) * N + k) * 8 + c % 8] =
                    kcrs[((size_t)(k0[p] + k) * C + cbase + c) * 9 + r * 3 + sx];
      }
      off += (size_t)9 * nch * N * 8;
    }
    return;
  }
  const int N = pad16(K);
  for (int seg = 0; seg < 2; ++seg) {
    const int Cs = seg ? cb : ca, cbase = seg ? ca : 0, chbase = seg ? nch_of(ca) : 0;
    for (int t = 0; t < 9; ++t)
      for (int c = 0; c < Cs; ++c)
        for (int k = 0; k < K; ++k)
          out[(((size_t)t * nch + chbase + c / 8) * N + k) * 8 + c % 8] = kcrs[((size_t)k * C + cbase + c) * 9 + t];
  }
}

namespace {
// The dispatch of one output channel part: pointers advanced to the part's first channel.
dnxcu_dispatch part_dispatch(const dnxcu_dispatch &d, int k0, int kp, size_t woff) {
  dnxcu_dispatch p = d;
  p.c_out = kp;
  if (p.out) p.out = (char *)p.out + (size_t)k0 * 2;
  if (p.out_pool) p.out_pool = (char *)p.out_pool + (size_t)k0 * 2;
  if (p.bias) p.bias = (const char *)p.bias + (size_t)k0 * 2;
  p.weights = (const char *)p.weights + woff;
  return p;
}
}  // namespace

int conv_tc_validate(const Variant &v, const dnxcu_dispatch &d) {
  if (d.c_out <= 0) return DNXCU_E_BAD_ARG;
  int k0[8], kp[8];
  const int n = split_parts(v, d.c_out, k0, kp);
  if (n == 1) {
    Plan pl;
    return make_plan(v, d, pl, false);
  }
  if (d.c_out % 16) return DNXCU_E_UNSUPPORTED;
  size_t woff = 0;
  for (int p = 0; p < n; ++p) {
    Plan pl;
    const dnxcu_dispatch dp = part_dispatch(d, k0[p], kp[p], woff);
    const int st = make_plan(v, dp, pl, false, d.c_out, n);
    if (st) return st;
    woff += (size_t)9 * (nch_of(d.c_a) + nch_of(d.c_b)) * pad16(kp[p]) * 16;
  }
  return DNXCU_OK;
}

void conv_tc_grid(const Variant &v, const dnxcu_dispatch &d, uint32_t g[3]) {
  int k0[8], kp[8];
  const int n = split_parts(v, d.c_out, k0, kp);
  Plan pl;
  g[0] = g[1] = g[2] = 1;
  const dnxcu_dispatch dp = n == 1 ? d : part_dispatch(d, k0[0], kp[0], 0);
  if (make_plan(v, dp, pl, false, n == 1 ? 0 : d.c_out, n) == DNXCU_OK) {
    g[0] = (uint32_t)pl.grid;
    g[1] = (uint32_t)pl.grid_y;
  }
  g[2] = (uint32_t)n;  // launches
}

// A dispatch planned once: launch parameters and encoded tensor maps of every part (one part unless the
// output channels are split).  Valid for the pointers and the shape it was made from.
struct ConvTcPlan {
  int n = 0;
  Plan part[8];
};

int conv_tc_plan(const Variant &v, const dnxcu_dispatch &d, ConvTcPlan **out) {
  if (d.c_out <= 0 || !out) return DNXCU_E_BAD_ARG;
  int k0[8], kp[8];
  const int n = split_parts(v, d.c_out, k0, kp);
  if (n > 1 && d.c_out % 16) return DNXCU_E_UNSUPPORTED;
  ConvTcPlan *cp = new (std::nothrow) ConvTcPlan();
  if (!cp) return DNXCU_E_NO_MEMORY;
  cp->n = n;
  size_t woff = 0;
  for (int p = 0; p < n; ++p) {
    const dnxcu_dispatch dp = n == 1 ? d : part_dispatch(d, k0[p], kp[p], woff);
    int st = make_plan(v, dp, cp->part[p], true, n == 1 ? 0 : d.c_out, n);
    if (!st && n > 1 && cp->part[p].R != 0) st = DNXCU_E_UNSUPPORTED;
    if (st) {
      delete cp;
      return st;
    }
    woff += (size_t)9 * (nch_of(d.c_a) + nch_of(d.c_b)) * pad16(kp[p]) * 16;
  }
  *out = cp;
  return DNXCU_OK;
}

void conv_tc_plan_free(ConvTcPlan *p) { delete p; }

namespace {

int launch_part(const Plan &pl, cudaStream_t s) {
  switch (pl.R) {
    case 0: return launch_stack(pl, s);
    case 1: return launch_r<1>(pl, s);
    case 2: return launch_r<2>(pl, s);
    case 4: return launch_r<4>(pl, s);
    default: return DNXCU_E_UNSUPPORTED;
  }
}

// Side streams for the launches of an output channel split: the parts are independent, each plans for its share
// of the SMs, and they run side by side between a fork and a join on the caller's stream (inside a stream
// capture this becomes parallel branches of the graph).  Every host thread has its own set per device, created
// on first use: two threads that launch split dispatches at the same time, or one that captures while another
// launches, never share a fork event or a side stream.
struct SideStreams {
  cudaStream_t stream[8] = {};
  cudaEvent_t fork = nullptr, join[8] = {};
  bool ready = false;
  ~SideStreams() {
    if (!ready) return;
    // at thread exit; errors (the context may be gone already) are of no interest here
    for (int i = 1; i < 8; ++i) {
      if (stream[i]) cudaStreamDestroy(stream[i]);
      if (join[i]) cudaEventDestroy(join[i]);
    }
    if (fork) cudaEventDestroy(fork);
    cudaGetLastError();
  }
};
constexpr int kSideDevices = 16;

int side_streams(int dev, SideStreams **out) {
  static thread_local SideStreams t_side[kSideDevices];
  if (dev < 0 || dev >= kSideDevices) return DNXCU_E_UNSUPPORTED;
  SideStreams &ss = t_side[dev];
  if (!ss.ready) {
    DNXCU_CUDA(cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming));
    for (int i = 1; i < 8; ++i) {
      DNXCU_CUDA(cudaStreamCreateWithFlags(&ss.stream[i], cudaStreamNonBlocking));
      DNXCU_CUDA(cudaEventCreateWithFlags(&ss.join[i], cudaEventDisableTiming));
    }
    ss.ready = true;
  }
  *out = &ss;
  return DNXCU_OK;
}

}  // namespace

int conv_tc_launch_plan(const ConvTcPlan &cp, cudaStream_t s) {
  const int n = cp.n;
  if (n == 1) return launch_part(cp.part[0], s);
  SideStreams *ss = nullptr;
  int dev = 0;
  DNXCU_CUDA(cudaGetDevice(&dev));
  int st = side_streams(dev, &ss);
  if (st) return st;
  // nothing below may fail between the fork and the join except the launches themselves
  DNXCU_CUDA(cudaEventRecord(ss->fork, s));
  for (int p = 1; p < n; ++p) DNXCU_CUDA(cudaStreamWaitEvent(ss->stream[p], ss->fork, 0));
  int result = DNXCU_OK;
  for (int p = 0; p < n; ++p) {
    st = launch_part(cp.part[p], p > 0 ? ss->stream[p] : s);
    if (st && !result) result = st;
  }
  // the join is made even after a failed launch, so that the side streams never stay forked
  for (int p = 1; p < n; ++p) {
    cudaEventRecord(ss->join[p], ss->stream[p]);
    cudaStreamWaitEvent(s, ss->join[p], 0);
  }
  return result;
}

int conv_tc_launch(const Variant &v, const dnxcu_dispatch &d, cudaStream_t s) {
  ConvTcPlan *cp = nullptr;
  int st = conv_tc_plan(v, d, &cp);
  if (st) return st;
  st = conv_tc_launch_plan(*cp, s);
  conv_tc_plan_free(cp);
  return st;
}

// One-time set-up of every kernel of this file on the current device (the dynamic shared memory limits), so that
// no launch has to do it later, e.g. inside a stream capture.
int conv_tc_init_device() {
  Plan none;
  memset(&none, 0, sizeof(none));
  int st = launch_r<1>(none, nullptr, true);
  if (!st) st = launch_r<2>(none, nullptr, true);
  if (!st) st = launch_r<4>(none, nullptr, true);
#define DNXCU_EPI_INIT(E) if (!st) st = launch_stack_epi<E>(none, nullptr, true);
  DNXCU_EPI_INIT(4) DNXCU_EPI_INIT(5) DNXCU_EPI_INIT(6) DNXCU_EPI_INIT(7)
  DNXCU_EPI_INIT(8) DNXCU_EPI_INIT(9) DNXCU_EPI_INIT(10) DNXCU_EPI_INIT(11)
  DNXCU_EPI_INIT(12) DNXCU_EPI_INIT(13) DNXCU_EPI_INIT(14) DNXCU_EPI_INIT(15)
#undef DNXCU_EPI_INIT
  return st;
}

#ifdef DNXCU_DEBUG_AIDS
int conv_tc_debug_trace_buffer(void *device_buffer, size_t bytes) {
  const size_t need = ((size_t)3 * TRACE_ITERS * TRACE_EVENTS + TRACE_EXTRA) * sizeof(long long);
  if (device_buffer && bytes < need) return DNXCU_E_BAD_ARG;
  g_trace_buffer = (long long *)device_buffer;
  return DNXCU_OK;
}
#endif

}  // namespace dnxcu
