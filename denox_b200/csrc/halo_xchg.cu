// Halo exchange of row band instances over peer memory (several GPUs of one node, or several bands on one
// device).  A 3x3 conv on a row band needs one row of each operand from the band above and the band below
// (the reference has no multi-device execution; the exchange step follows from its conv's 3x3 window,
// direct_conv.comp:209-212).  Each band keeps, per conv operand, two slabs in its OWN memory (the row above,
// the row below) and two flags.  One kernel per conv does both halves of the swap:
//   push: copy this band's first row into the upper neighbour's "row below" slab and its last row into the
//         lower neighbour's "row above" slab with plain 16 byte stores through peer pointers, make them
//         visible system wide, then store this band's running count into the neighbours' flags;
//   wait: spin (bounded) until this band's own flags hold that count, i.e. both neighbours have pushed.
// The conv that follows on the same stream reads only local memory.  No load ever targets a peer.
#include "internal.h"
#include "halo_xchg.h"

namespace dnxcu {
namespace {

__device__ __forceinline__ void copy16(uint4 *dst, const uint4 *src, unsigned n16, unsigned tid, unsigned nthreads) {
  for (unsigned i = tid; i < n16; i += nthreads) dst[i] = src[i];
}

__global__ void __launch_bounds__(512) halo_xchg(const XchgArgs a) {
  __shared__ int s_last;
  const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  if (a.mode & XCHG_PUSH) {
    for (int p = 0; p < a.npoints; ++p) {
      const XchgPoint &q = a.pt[p];
      if (q.peer_up_slab) copy16(q.peer_up_slab, q.send_top, q.n16, tid, nthreads);
      if (q.peer_down_slab) copy16(q.peer_down_slab, q.send_bottom, q.n16, tid, nthreads);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // the block's stores (ordered before this point by the barrier) become visible system wide before the block
    // is counted as done
    __threadfence_system();
    const unsigned ticket = atomicAdd(a.done, 1u);
    s_last = ticket == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last || threadIdx.x != 0) return;
  // the last block to finish: every block's stores are fenced and counted
  *a.done = 0;  // ready for the next launch (stream order: no other launch of this kernel overlaps on this band)
  __threadfence_system();
  unsigned count = *a.counter;
  if (a.mode & XCHG_PUSH) {
    count += 1;
    *a.counter = count;
    for (int p = 0; p < a.npoints; ++p) {
      const XchgPoint &q = a.pt[p];
      if (q.peer_up_flag) *reinterpret_cast<volatile unsigned *>(q.peer_up_flag) = count;
      if (q.peer_down_flag) *reinterpret_cast<volatile unsigned *>(q.peer_down_flag) = count;
    }
    __threadfence_system();
  }
  if (a.mode & XCHG_WAIT) {
    // After a wait of this instance has run out its frames are void until the host has read the status and
    // resynchronised the bands; waiting again for every later row would only add the limit once more per
    // exchange (16 exchanges per frame).
    if (a.status && *reinterpret_cast<volatile int *>(a.status) != 0) return;
    const unsigned long long t0 = clock64();
    for (int p = 0; p < a.npoints; ++p) {
      const XchgPoint &q = a.pt[p];
      for (int side = 0; side < 2; ++side) {
        const volatile unsigned *flag = side ? q.my_flag_bottom : q.my_flag_top;
        if (!flag) continue;
        // counts only grow; the signed difference keeps the comparison right across a wrap of the counter
        for (unsigned it = 0; (int)(*flag - count) < 0; ++it) {
          if ((it & 15u) == 15u && (unsigned long long)clock64() - t0 > a.wait_limit) {
            if (a.status) atomicCAS(a.status, 0, 10);
            return;  // bounded: the neighbour's row did not arrive; the output of this frame is undefined
          }
          __nanosleep(64);
        }
      }
    }
    __threadfence();  // the rows the flags announce are read by the next kernel on this stream
  }
}

}  // namespace

int halo_xchg_launch(const XchgArgs &a, cudaStream_t s) {
  if (a.npoints <= 0 || a.npoints > XCHG_MAX_POINTS || !a.done || !a.counter) return DNXCU_E_BAD_ARG;
  unsigned most = 0;
  for (int p = 0; p < a.npoints; ++p) most = a.pt[p].n16 > most ? a.pt[p].n16 : most;
  // enough blocks to keep several hundred 16 byte stores in flight per direction; one block when only waiting
  int blocks = (a.mode & XCHG_PUSH) ? (int)((most + 2047u) / 2048u) : 1;
  if (blocks < 1) blocks = 1;
  if (blocks > 16) blocks = 16;
  halo_xchg<<<blocks, 512, 0, s>>>(a);
  DNXCU_CUDA(cudaGetLastError());
  return DNXCU_OK;
}

}  // namespace dnxcu
