// Arguments of the halo exchange kernel (halo_xchg.cu) and its launcher.
#pragma once
#include "internal.h"

namespace dnxcu {

constexpr int XCHG_MAX_POINTS = 2;  // operands of one conv
constexpr unsigned XCHG_PUSH = 1u, XCHG_WAIT = 2u;

struct XchgPoint {
  const uint4 *send_top, *send_bottom;  // this band's first / last row of the operand (local)
  uint4 *peer_up_slab;                  // the upper neighbour's "row below" slab (peer memory), or nullptr
  uint4 *peer_down_slab;                // the lower neighbour's "row above" slab (peer memory), or nullptr
  unsigned *peer_up_flag, *peer_down_flag;       // the neighbours' flags for those slabs (peer memory)
  unsigned *my_flag_top, *my_flag_bottom;        // this band's flags (local), nullptr at an image border
  unsigned n16;                                  // 16 byte pieces per row
};

struct XchgArgs {
  XchgPoint pt[XCHG_MAX_POINTS];
  int npoints;
  unsigned mode;               // XCHG_PUSH | XCHG_WAIT
  unsigned *done;              // local: blocks finished (returns to 0 at the end of every launch)
  unsigned *counter;           // local: pushes made so far at this exchange
  int *status;                 // local: receives code 10 when the wait runs out
  unsigned long long wait_limit;
};

int halo_xchg_launch(const XchgArgs &a, cudaStream_t s);

}  // namespace dnxcu
