// Runtime: fuses the node list of a model into dispatches, and runs them.
// Stands in for the reference's implement -> select -> Model -> Instance chain
// on this path (compiler/src/denox/compiler/implement/implement.cpp:11-68,
// runtime/src/denox/runtime/model.cpp:637-659, instance.cpp:25-430).
#include "runtime.h"
#include "halo_xchg.h"
#include "select.h"
#include <string.h>
#include <unistd.h>
#include <map>
#include <memory>

using namespace dnxcu;

namespace dnxcu {

// ---- fusion -----------------------------------------------------------------
// Patterns (the first two exist in the reference, the last two are new):
//   conv -> relu                         DirectConvShaderCM.cpp:201-244
//   concat(a, b) -> conv                 ConcatConvCMShader.cpp:301-359
//   conv(+relu) -> maxpool 2x2           pool in the conv epilogue
//   upsample 2x -> [concat ->] conv      upsample as the conv's operand address map
// True when some variant that writes the pooled output from its epilogue accepts a conv with these channel
// counts and flags.  Acceptance depends on channels and weight size only, so a nominal extent is probed.
static bool fused_pool_variant_exists(int c_a, int c_b, int c_out, uint32_t flags) {
  dnxcu_dispatch d;
  memset(&d, 0, sizeof(d));
  d.flags = flags;
  d.pc[0] = d.pc[1] = 64;
  d.c_a = c_a;
  d.c_b = c_b;
  d.c_out = c_out;
  void *const probe = (void *)0x1000;  // passes the alignment rules, never dereferenced by validation
  d.in_a = probe;
  d.in_b = c_b > 0 ? probe : nullptr;
  d.out = (flags & DNXCU_F_NO_FULL_OUT) ? nullptr : probe;
  d.out_pool = probe;
  d.weights = probe;
  d.bias = (flags & DNXCU_F_BIAS) ? probe : nullptr;
  for (int id = 0; id < variant_count(); ++id) {
    const Variant *v = get_variant(id);
    if (v->desc.op != DNXCU_OP_CONV3X3 || !(v->desc.allowed_flags & DNXCU_F_POOL_OUT)) continue;
    d.variant = id;
    if (dnxcu_validate(&d) == DNXCU_OK) return true;
  }
  return false;
}

int build_fused_ops(const dnxcu_model_desc &desc, bool allow_tc, dnxcu_model &m) {
  if (desc.n_nodes <= 0 || desc.n_tensors <= 0 || !desc.nodes) return DNXCU_E_BAD_ARG;
  if (desc.input_tensor < 0 || desc.input_tensor >= desc.n_tensors || desc.output_tensor < 0 ||
      desc.output_tensor >= desc.n_tensors || desc.input_channels <= 0)
    return DNXCU_E_BAD_ARG;
  const int NT = desc.n_tensors, NN = desc.n_nodes;
  m.tensors.assign(NT, TensorInfo());
  m.n_model_tensors = NT;
  m.nodes.clear();
  m.ops.clear();
  m.input_tensor = desc.input_tensor;
  m.output_tensor = desc.output_tensor;
  m.input_channels = desc.input_channels;
  m.options = desc.options;
  std::vector<int> producer(NT, -1);
  std::vector<std::vector<int>> consumers(NT);
  std::vector<bool> defined(NT, false);
  defined[desc.input_tensor] = true;
  m.tensors[desc.input_tensor].channels = desc.input_channels;
  m.tensors[desc.input_tensor].level = 0;
  for (int i = 0; i < NN; ++i) {
    const dnxcu_node &n = desc.nodes[i];
    if (n.in0 < 0 || n.in0 >= NT || n.out < 0 || n.out >= NT || !defined[n.in0] || defined[n.out]) return DNXCU_E_BAD_ARG;
    const TensorInfo &t0 = m.tensors[n.in0];
    TensorInfo &to = m.tensors[n.out];
    consumers[n.in0].push_back(i);
    switch (n.kind) {
      case DNXCU_NODE_CONV:
        if (n.c_out <= 0 || !n.weights_kcrs) return DNXCU_E_BAD_ARG;
        to.channels = n.c_out;
        to.level = t0.level;
        break;
      case DNXCU_NODE_RELU:
      case DNXCU_NODE_LEAKY_RELU: to = t0; break;
      case DNXCU_NODE_MAXPOOL:
        to.channels = t0.channels;
        to.level = t0.level + 1;
        break;
      case DNXCU_NODE_UPSAMPLE:
        to.channels = t0.channels;
        to.level = t0.level - 1;
        break;
      case DNXCU_NODE_CONCAT: {
        if (n.in1 < 0 || n.in1 >= NT || !defined[n.in1]) return DNXCU_E_BAD_ARG;
        const TensorInfo &t1 = m.tensors[n.in1];
        if (t1.level != t0.level) return DNXCU_E_BAD_ARG;  // same H, W (ConcatConvCMShader.cpp:783-787)
        consumers[n.in1].push_back(i);
        to.channels = t0.channels + t1.channels;
        to.level = t0.level;
        break;
      }
      default: return DNXCU_E_BAD_ARG;
    }
    to.materialized = false;
    defined[n.out] = true;
    producer[n.out] = i;
    NodeRec rec;
    rec.kind = n.kind;
    rec.in0 = n.in0;
    rec.in1 = n.kind == DNXCU_NODE_CONCAT ? n.in1 : -1;
    rec.out = n.out;
    rec.c_out = n.c_out;
    rec.alpha = n.alpha;
    if (n.kind == DNXCU_NODE_CONV) {
      const size_t nw = (size_t)n.c_out * t0.channels * 9;
      rec.weights.assign((const uint16_t *)n.weights_kcrs, (const uint16_t *)n.weights_kcrs + nw);
      if (n.bias) {
        rec.has_bias = true;
        rec.bias.assign((const uint16_t *)n.bias, (const uint16_t *)n.bias + n.c_out);
      }
    }
    m.nodes.push_back(std::move(rec));
  }
  if (!defined[desc.output_tensor]) return DNXCU_E_BAD_ARG;

  const bool f_act = !(desc.options & DNXCU_OPT_NO_FUSE_ACTIVATION);
  const bool f_pool = !(desc.options & DNXCU_OPT_NO_FUSE_POOL) && allow_tc;
  const bool f_up = !(desc.options & DNXCU_OPT_NO_FUSE_UPSAMPLE);
  const bool f_cat = !(desc.options & DNXCU_OPT_NO_FUSE_CONCAT);
  auto sole = [&](int t, int node) {
    return consumers[t].size() == 1 && consumers[t][0] == node && t != desc.output_tensor;
  };

  std::vector<bool> absorbed(NN, false);
  struct ConvPlan {
    int a, b, up, relu_node, pool_node, out, out_pool;
    bool no_full;
  };
  std::map<int, ConvPlan> plans;
  for (int i = 0; i < NN; ++i) {
    const dnxcu_node &n = desc.nodes[i];
    if (n.kind != DNXCU_NODE_CONV) continue;
    ConvPlan p = {n.in0, -1, 0, -1, -1, n.out, -1, false};
    int pc = producer[p.a];
    if (f_cat && pc >= 0 && desc.nodes[pc].kind == DNXCU_NODE_CONCAT && sole(p.a, i)) {
      absorbed[pc] = true;
      p.a = desc.nodes[pc].in0;
      p.b = desc.nodes[pc].in1;
      const int pu = producer[p.a];
      if (f_up && pu >= 0 && desc.nodes[pu].kind == DNXCU_NODE_UPSAMPLE && sole(p.a, pc)) {
        absorbed[pu] = true;
        p.a = desc.nodes[pu].in0;
        p.up = 1;
      }
    } else if (f_up && pc >= 0 && desc.nodes[pc].kind == DNXCU_NODE_UPSAMPLE && sole(p.a, i)) {
      absorbed[pc] = true;
      p.a = desc.nodes[pc].in0;
      p.up = 1;
    }
    // conv -> ReLU | LeakyReLU (DirectConvShaderCM.cpp:201-244: both activations are fused)
    if (f_act && sole(p.out, consumers[p.out].empty() ? -1 : consumers[p.out][0]) &&
        (desc.nodes[consumers[p.out][0]].kind == DNXCU_NODE_RELU ||
         desc.nodes[consumers[p.out][0]].kind == DNXCU_NODE_LEAKY_RELU)) {
      p.relu_node = consumers[p.out][0];
      absorbed[p.relu_node] = true;
      p.out = desc.nodes[p.relu_node].out;
    }
    if (f_pool) {
      for (int c : consumers[p.out])
        if (desc.nodes[c].kind == DNXCU_NODE_MAXPOOL && p.pool_node < 0) p.pool_node = c;
      if (p.pool_node >= 0) {
        // The pool moves into the conv's epilogue only when a variant with that epilogue takes the conv
        // (channel counts, weight size): otherwise the conv keeps any variant, the CUDA core one included,
        // and basic-pool follows as a dispatch of its own, as in the reference's schedule.
        const int ca = m.tensors[p.a].channels, cb = p.b >= 0 ? m.tensors[p.b].channels : 0;
        uint32_t fl = DNXCU_F_POOL_OUT | (p.up ? DNXCU_F_UP2X_A : 0u) | (n.bias ? DNXCU_F_BIAS : 0u);
        if (p.relu_node >= 0)
          fl |= desc.nodes[p.relu_node].kind == DNXCU_NODE_RELU ? DNXCU_F_RELU : DNXCU_F_LEAKY;
        if (sole(p.out, p.pool_node)) fl |= DNXCU_F_NO_FULL_OUT;
        if (fused_pool_variant_exists(ca, cb, n.c_out, fl)) {
          absorbed[p.pool_node] = true;
          p.out_pool = desc.nodes[p.pool_node].out;
          p.no_full = sole(p.out, p.pool_node);
        } else {
          p.pool_node = -1;
        }
      }
    }
    plans[i] = p;
  }

  for (int i = 0; i < NN; ++i) {
    if (absorbed[i]) continue;
    const dnxcu_node &n = desc.nodes[i];
    FusedOp op;
    op.src_node = i;
    op.in_a = n.in0;
    op.out = n.out;
    op.c_a = m.tensors[n.in0].channels;
    op.level = m.tensors[n.in0].level;
    switch (n.kind) {
      case DNXCU_NODE_CONV: {
        const ConvPlan &p = plans[i];
        op.op = DNXCU_OP_CONV3X3;
        op.in_a = p.a;
        op.in_b = p.b;
        op.c_a = m.tensors[p.a].channels;
        op.c_b = p.b >= 0 ? m.tensors[p.b].channels : 0;
        op.c_out = n.c_out;
        op.level = m.tensors[n.out].level;
        op.out = p.out;
        op.out_pool = p.out_pool;
        op.name = "direct-conv";
        if (p.b >= 0) op.name = "concat-conv";
        if (p.up) { op.flags |= DNXCU_F_UP2X_A; op.name = "up" + op.name; }
        if (p.relu_node >= 0) {
          if (desc.nodes[p.relu_node].kind == DNXCU_NODE_RELU) {
            op.flags |= DNXCU_F_RELU;
            op.name += "+relu";
          } else {
            op.flags |= DNXCU_F_LEAKY;
            op.alpha = desc.nodes[p.relu_node].alpha;
            op.name += "+leaky";
          }
        }
        if (p.pool_node >= 0) { op.flags |= DNXCU_F_POOL_OUT; op.name += "+pool"; }
        if (p.no_full) op.flags |= DNXCU_F_NO_FULL_OUT;
        const size_t nw = (size_t)n.c_out * (op.c_a + op.c_b) * 9;
        op.weights_kcrs.assign((const uint16_t *)n.weights_kcrs, (const uint16_t *)n.weights_kcrs + nw);
        if (n.bias) {
          op.flags |= DNXCU_F_BIAS;
          op.bias.assign((const uint16_t *)n.bias, (const uint16_t *)n.bias + n.c_out);
        }
        break;
      }
      case DNXCU_NODE_RELU: op.op = DNXCU_OP_RELU; op.name = "basic-activation"; break;
      case DNXCU_NODE_LEAKY_RELU:
        op.op = DNXCU_OP_RELU;
        op.flags |= DNXCU_F_LEAKY;
        op.alpha = n.alpha;
        op.name = "basic-activation(leaky)";
        break;
      case DNXCU_NODE_MAXPOOL: op.op = DNXCU_OP_MAXPOOL2X2; op.name = "basic-pool"; break;
      case DNXCU_NODE_UPSAMPLE: op.op = DNXCU_OP_UPSAMPLE2X; op.name = "basic-upsample"; break;
      case DNXCU_NODE_CONCAT:
        op.op = DNXCU_OP_CONCAT;
        op.in_b = n.in1;
        op.c_b = m.tensors[n.in1].channels;
        op.name = "copy-transform";
        break;
    }
    if (!(op.flags & DNXCU_F_NO_FULL_OUT)) m.tensors[op.out].materialized = true;
    if (op.out_pool >= 0) m.tensors[op.out_pool].materialized = true;
    m.ops.push_back(std::move(op));
  }
  m.tensors[desc.input_tensor].materialized = true;

  // An input whose channel count is not a multiple of 8 (the 9 channel colour/albedo/normal image) cannot be
  // fetched in 16 byte pieces.  Like the reference's layout specialisation (HWC -> HWC8, specialization.cpp:183-340)
  // the schedule then starts with one copy into a tensor padded with zero channels, and the convs that read the
  // input get zero weights for the added channels.
  if (allow_tc && !(desc.options & DNXCU_OPT_NO_PAD_INPUT) && (desc.input_channels % 8) != 0) {
    const int C = desc.input_channels, Cp = (C + 15) / 16 * 16;
    const int padded = (int)m.tensors.size();
    TensorInfo ti;
    ti.channels = Cp;
    ti.level = 0;
    ti.materialized = true;
    m.tensors.push_back(ti);
    for (FusedOp &op : m.ops) {
      if (op.op != DNXCU_OP_CONV3X3) continue;
      const bool ina = op.in_a == desc.input_tensor, inb = op.in_b == desc.input_tensor;
      if (!ina && !inb) continue;
      const int ca = op.c_a, cb = op.c_b, Cold = ca + cb;
      const int nca = ina ? Cp : ca, ncb = inb ? Cp : cb, Cnew = nca + ncb;
      std::vector<uint16_t> w((size_t)op.c_out * Cnew * 9, 0);
      for (int k = 0; k < op.c_out; ++k)
        for (int c = 0; c < Cold; ++c) {
          const int cn = c < ca ? c : nca + (c - ca);
          for (int t = 0; t < 9; ++t) w[((size_t)k * Cnew + cn) * 9 + t] = op.weights_kcrs[((size_t)k * Cold + c) * 9 + t];
        }
      op.weights_kcrs.swap(w);
      if (ina) { op.in_a = padded; op.c_a = Cp; }
      if (inb) { op.in_b = padded; op.c_b = Cp; }
    }
    FusedOp pad;
    pad.op = DNXCU_OP_PAD_CHANNELS;
    pad.in_a = desc.input_tensor;
    pad.out = padded;
    pad.c_a = C;
    pad.c_out = Cp;
    pad.level = 0;
    pad.src_node = 0;
    pad.name = "copy-transform(pad)";
    m.ops.insert(m.ops.begin(), pad);
  }
  return DNXCU_OK;
}

// preference when no benchmark data exists: tensor core variants first,
// resident weights before streamed, then the CUDA core fallback; 128-bit before 2-byte.
static const int conv_pref[] = {6, 7, 17, 18, 19, 26, 20, 27, 25, 28, 29, 2, 3, 1, 4, 5, 0};

int variant_rank(int variant) {
  int r = 0;
  for (int id : conv_pref) {
    if (id == variant) return r;
    ++r;
  }
  const Variant *v = get_variant(variant);
  return 100 + (v && v->p0 == 8 ? 0 : 1);  // memory kernels: the 128-bit form first
}

void candidate_variants(const FusedOp &op, bool allow_tc, std::vector<int> &out) {
  out.clear();
  if (op.op == DNXCU_OP_CONV3X3) {
    for (int id : conv_pref) {
      const Variant *v = get_variant(id);
      if (!v || (op.flags & ~v->desc.allowed_flags)) continue;
      if (v->desc.needs_tcgen05 && !allow_tc) continue;
      out.push_back(id);
    }
    return;
  }
  for (int id = 0; id < variant_count(); ++id) {
    const Variant *v = get_variant(id);
    if (v->desc.op == op.op) out.push_back(id);
  }
}

}  // namespace dnxcu

// ---- instance -----------------------------------------------------------------

struct dnxcu_instance {
  const dnxcu_model *model = nullptr;
  int H = 0, W = 0;  // band extent at level 0 (what the schedule runs at)
  // Frames whose extent is not a multiple of the network's alignment: the caller's extent, the two
  // extra dispatches (edge pad in front, slice behind) and the caller-extent device buffers.
  int user_H = 0, user_W = 0;
  bool padded = false;
  dnxcu_dispatch pre = {}, post = {};
  void *user_in = nullptr, *user_out = nullptr;
  dnxcu_band band = {0, 0, 0};
  bool banded = false;
  std::vector<dnxcu::FusedOp> ops;        // this instance's schedule: the model's default, or what the cost
  std::vector<dnxcu::TensorInfo> tensors;  // driven selection chose for this extent
  std::vector<int> preset_variant;         // selection's variant per dispatch (empty: chosen per dispatch below)
  std::vector<void *> tensor_ptr;    // per tensor device pointer (nullptr if not materialized)
  std::vector<void *> owned;         // everything to cudaFree
  std::vector<dnxcu_dispatch> disp;  // with the instance's own input / output buffers
  std::vector<dnxcu_halo_point> halos;
  // Direct halo exchange over peer memory (row bands on several GPUs, or several bands on one device).
  // All slabs and flags of the band live in one allocation with a layout that depends only on the model,
  // the width and the band height, so neighbours address each other's slabs by offset.
  struct HaloSlot {
    size_t top_off, bot_off, flag_off;  // slab "row above", slab "row below", two flags (top, bottom)
    int dispatch;
  };
  std::vector<HaloSlot> halo_slots;     // one per entry of `halos`
  char *arena = nullptr;
  size_t arena_bytes = 0;
  uint64_t arena_layout = 0;            // hash of what determines the layout
  unsigned *xchg_ctl = nullptr;         // per dispatch: blocks-done counter, push counter
  char *peer_up = nullptr, *peer_down = nullptr;  // the neighbours' arenas as this device sees them
  bool peer_up_ipc = false, peer_down_ipc = false;
  bool connected = false, auto_exchange = false;
  std::vector<dnxcu::XchgArgs> xchg;    // per dispatch, npoints == 0: nothing to exchange
  std::vector<dnxcu_plan *> plans;   // one per dispatch, made from the instance's own buffers
  int *status = nullptr;
  cudaStream_t stream = nullptr;
  // cached graphs of the whole schedule, one per (input, output) pointer pair, most recently used first
  struct Graph {
    cudaGraphExec_t exec;
    const void *in;
    void *out;
  };
  std::vector<Graph> graphs;
  size_t graph_capacity = 4;
  std::vector<cudaEvent_t> events;

  ~dnxcu_instance() {
    if (peer_up_ipc && peer_up) cudaIpcCloseMemHandle(peer_up);
    if (peer_down_ipc && peer_down) cudaIpcCloseMemHandle(peer_down);
    for (Graph &g : graphs) cudaGraphExecDestroy(g.exec);
    for (dnxcu_plan *p : plans) dnxcu_plan_destroy(p);
    for (cudaEvent_t e : events) cudaEventDestroy(e);
    if (stream) cudaStreamDestroy(stream);
    for (void *p : owned) cudaFree(p);
  }
};

namespace {

int dev_alloc(dnxcu_instance &inst, size_t bytes, void **out) {
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    cuda_fail(e);
    return e == cudaErrorMemoryAllocation ? DNXCU_E_NO_MEMORY : DNXCU_E_CUDA;
  }
  inst.owned.push_back(p);
  *out = p;
  return DNXCU_OK;
}

// Enqueues dispatch i, substituting caller pointers for the model's input / output tensors.
int launch_one(dnxcu_instance &inst, int i, const void *in_override, void *out_override, cudaStream_t s) {
  const FusedOp &op = inst.ops[i];
  if (inst.connected && inst.auto_exchange && inst.xchg[i].npoints > 0) {
    // the neighbours' boundary rows of this conv's operands: push ours, wait for theirs
    dnxcu::XchgArgs a = inst.xchg[i];
    a.mode = XCHG_PUSH | XCHG_WAIT;
    a.wait_limit = wait_limit_cycles();
    int st = halo_xchg_launch(a, s);
    if (st) return st;
  }
  const int tin = inst.model->input_tensor, tout = inst.model->output_tensor;
  const bool sub_in = in_override && (op.in_a == tin || op.in_b == tin);
  const bool sub_out = out_override && (op.out == tout || op.out_pool == tout);
  if (!sub_in && !sub_out) return dnxcu_plan_launch(inst.plans[i], s);  // planned once at creation
  dnxcu_dispatch d = inst.disp[i];
  if (sub_in) {
    if (op.in_a == tin) d.in_a = in_override;
    if (op.in_b == tin) d.in_b = in_override;
  }
  if (sub_out) {
    if (op.out == tout) d.out = out_override;
    if (op.out_pool == tout) d.out_pool = out_override;
  }
  return dnxcu_launch(&d, s);
}

// Reads the instance's status word; a kernel's time-out code is reported once and then cleared, so that
// the frames after it are judged on their own.
int take_status(dnxcu_instance &inst, int hstatus) {
  if (!hstatus) return DNXCU_OK;
  cudaMemsetAsync(inst.status, 0, sizeof(int), inst.stream);
  cudaStreamSynchronize(inst.stream);
  return DNXCU_E_DEVICE;
}

}  // namespace

extern "C" {

int dnxcu_model_create(const dnxcu_model_desc *desc, const dnxcu_db *db, int device, dnxcu_model **out) {
  if (!desc || !out) return DNXCU_E_BAD_ARG;
  int st;
  bool allow_tc = !(desc->options & DNXCU_OPT_NO_TCGEN05);
  if (device >= 0) {
    dnxcu_caps caps;
    st = dnxcu_get_device_caps(device, &caps);
    if (st) return st;
    allow_tc = allow_tc && caps.tcgen05;
  }  // device < 0: no device at hand (compiling a model to a dnx file): every capability is assumed
  std::unique_ptr<dnxcu_model> m(new (std::nothrow) dnxcu_model());
  if (!m) return DNXCU_E_NO_MEMORY;
  st = build_fused_ops(*desc, allow_tc, *m);
  if (st) return st;
  m->device = device < 0 ? 0 : device;
  m->db = db;
  *out = m.release();
  return DNXCU_OK;
}

void dnxcu_model_destroy(dnxcu_model *m) { delete m; }
const char *dnxcu_last_error_message(void) { return error_text(); }

int dnxcu_model_create_from_onnx(const void *bytes, size_t n, const dnxcu_db *db, int device, uint32_t options,
                                 dnxcu_model **out) {
  if (!bytes || !out) return DNXCU_E_BAD_ARG;
  int st;
  bool allow_tc = !(options & DNXCU_OPT_NO_TCGEN05);
  if (device >= 0) {
    dnxcu_caps caps;
    st = dnxcu_get_device_caps(device, &caps);
    if (st) return st;
    allow_tc = allow_tc && caps.tcgen05;
  }
  std::unique_ptr<dnxcu_model> m(new (std::nothrow) dnxcu_model());
  if (!m) return DNXCU_E_NO_MEMORY;
  st = import_onnx(bytes, n, options, *m, allow_tc);
  if (st) return st;
  m->device = device < 0 ? 0 : device;
  m->db = db;
  *out = m.release();
  return DNXCU_OK;
}

int dnxcu_model_create_from_dnx(const void *bytes, size_t n, int device, dnxcu_model **out) {
  if (!bytes || !out) return DNXCU_E_BAD_ARG;
  std::unique_ptr<dnxcu_model> m(new (std::nothrow) dnxcu_model());
  if (!m) return DNXCU_E_NO_MEMORY;
  int st = read_dnx(bytes, n, *m, &m->dnx_align);
  if (st) return st;
  if (device >= 0) {
    dnxcu_caps caps;
    st = dnxcu_get_device_caps(device, &caps);
    if (st) return st;
    for (int v : m->dnx_variants)
      if (get_variant(v)->desc.needs_tcgen05 && !caps.tcgen05) return DNXCU_E_UNSUPPORTED;
  }
  m->device = device < 0 ? 0 : device;
  *out = m.release();
  return DNXCU_OK;
}

static int hand_out(const std::vector<uint8_t> &blob, void *out, size_t *bytes) {
  if (!out) {
    *bytes = blob.size();
    return DNXCU_OK;
  }
  if (*bytes < blob.size()) return DNXCU_E_BAD_ARG;
  memcpy(out, blob.data(), blob.size());
  *bytes = blob.size();
  return DNXCU_OK;
}

static int model_align(const std::vector<TensorInfo> &tensors) {
  int maxlevel = 0;
  for (const TensorInfo &t : tensors) maxlevel = t.level > maxlevel ? t.level : maxlevel;
  return 1 << maxlevel;
}

int dnxcu_model_write_dnx(const dnxcu_model *m, void *out, size_t *bytes) {
  if (!m || !bytes) return DNXCU_E_BAD_ARG;
  std::vector<int> variants;
  if (m->from_dnx) {
    variants = m->dnx_variants;
  } else {
    // no extent, no database: per dispatch the first variant of the preference order that takes it
    const int align = model_align(m->tensors);
    const int probe = 16 * align;
    for (const FusedOp &op : m->ops) {
      std::vector<int> cand;
      candidate_variants(op, !(m->options & DNXCU_OPT_NO_TCGEN05), cand);
      int chosen = -1;
      for (int id : cand) {
        const dnxcu_dispatch d = probe_dispatch(op, probe, probe, id);
        if (dnxcu_validate(&d) == DNXCU_OK) {
          chosen = id;
          break;
        }
      }
      if (chosen < 0) return DNXCU_E_UNSUPPORTED;
      variants.push_back(chosen);
    }
  }
  std::vector<uint8_t> blob;
  int st = write_dnx(*m, m->ops, m->tensors, variants, model_align(m->tensors), blob);
  if (st) return st;
  return hand_out(blob, out, bytes);
}

int dnxcu_instance_write_dnx(const dnxcu_instance *inst, void *out, size_t *bytes) {
  if (!inst || !bytes) return DNXCU_E_BAD_ARG;
  std::vector<int> variants;
  for (const dnxcu_dispatch &d : inst->disp) variants.push_back(d.variant);
  std::vector<uint8_t> blob;
  int st = write_dnx(*inst->model, inst->ops, inst->tensors, variants, model_align(inst->tensors), blob);
  if (st) return st;
  return hand_out(blob, out, bytes);
}

int dnxcu_model_io(const dnxcu_model *m, int *input_tensor, int *input_channels, int *output_tensor) {
  if (!m) return DNXCU_E_BAD_ARG;
  if (input_tensor) *input_tensor = m->input_tensor;
  if (input_channels) *input_channels = m->input_channels;
  if (output_tensor) *output_tensor = m->output_tensor;
  return DNXCU_OK;
}

int dnxcu_model_dispatch_count(const dnxcu_model *m) { return m ? (int)m->ops.size() : DNXCU_E_BAD_ARG; }
int dnxcu_instance_dispatch_count(const dnxcu_instance *inst) { return inst ? (int)inst->disp.size() : DNXCU_E_BAD_ARG; }

int dnxcu_select_min_cost(int n_nodes, int n_edges, const int32_t *src_off, const int32_t *srcs, const int32_t *dst_off,
                          const int32_t *dsts, const double *weight, const int32_t *inputs, int n_inputs,
                          const int32_t *outputs, int n_outputs, int min_dispatches, int32_t *chosen, int32_t *n_chosen,
                          double *cost) {
  if (n_nodes <= 0 || n_edges < 0 || !src_off || !dst_off || !weight || !inputs || !outputs || !chosen || !n_chosen ||
      n_inputs < 0 || n_outputs <= 0 || (n_edges > 0 && (!srcs || !dsts)))
    return DNXCU_E_BAD_ARG;
  HyperGraph g;
  g.n_nodes = n_nodes;
  for (int e = 0; e < n_edges; ++e) {
    if (src_off[e + 1] < src_off[e] || dst_off[e + 1] <= dst_off[e]) return DNXCU_E_BAD_ARG;
    HyperEdge he;
    he.src.assign(srcs + src_off[e], srcs + src_off[e + 1]);
    he.dst.assign(dsts + dst_off[e], dsts + dst_off[e + 1]);
    he.weight = weight[e];
    he.payload = e;
    g.edges.push_back(std::move(he));
  }
  const std::vector<int> in(inputs, inputs + n_inputs), out(outputs, outputs + n_outputs);
  if (min_dispatches && !prune_topological(g, in, out)) return DNXCU_E_UNSUPPORTED;
  std::vector<int> ch;
  double c = 0;
  if (!minimum_cost_subgraph(g, in, out, ch, &c)) return DNXCU_E_UNSUPPORTED;
  *n_chosen = (int32_t)ch.size();
  for (size_t i = 0; i < ch.size(); ++i) chosen[i] = g.edges[ch[i]].payload;
  if (cost) *cost = c;
  return DNXCU_OK;
}

int dnxcu_instance_create(const dnxcu_model *m, int height, int width, const dnxcu_band *band, dnxcu_instance **out) {
  if (!m || !out || height <= 0 || width <= 0) return DNXCU_E_BAD_ARG;
  int maxlevel = 0;
  for (const TensorInfo &t : m->tensors) {
    if (t.level < 0) return DNXCU_E_UNSUPPORTED;  // a tensor larger than the input
    if (t.level > maxlevel) maxlevel = t.level;
  }
  const int align = 1 << maxlevel;
  std::unique_ptr<dnxcu_instance> inst(new (std::nothrow) dnxcu_instance());
  if (!inst) return DNXCU_E_NO_MEMORY;
  inst->model = m;
  inst->user_W = width;
  inst->user_H = height;
  if (!band && ((height % align) || (width % align))) {
    // the reference's exported models wrap the net in pad (replicate, right and bottom) -> net -> slice
    // (oidn_model.py:334-347); here the instance does it
    if (m->tensors[m->output_tensor].level != 0) return DNXCU_E_UNSUPPORTED;
    inst->padded = true;
    height = (height + align - 1) / align * align;
    width = (width + align - 1) / align * align;
  }
  inst->W = width;
  inst->H = height;
  inst->band = {height, 0, height};
  if (band) {
    if (band->rows <= 0 || band->row0 < 0 || band->row0 + band->rows > band->image_h) return DNXCU_E_BAD_ARG;
    inst->band = *band;
    inst->H = band->rows;
    inst->banded = band->rows != band->image_h;
    if (inst->banded && ((band->rows | band->row0 | band->image_h) % align)) return DNXCU_E_BAD_ARG;
  }
  // every level must keep integral extents (the reference pads images to the
  // network's alignment for the same reason, oidn_model.py:334-347)
  if ((inst->H % align) || (width % align)) return DNXCU_E_UNSUPPORTED;
  const bool has_up = inst->banded && inst->band.row0 > 0;
  const bool has_down = inst->banded && inst->band.row0 + inst->band.rows < inst->band.image_h;

  dnxcu_caps caps;
  int st = dnxcu_get_device_caps(m->device, &caps);
  if (st) return st;
  const bool allow_tc = caps.tcgen05 && !(m->options & DNXCU_OPT_NO_TCGEN05);
  // the schedule: with a benchmark database, the cheapest sub-graph of all candidate dispatches at this extent
  // (row bands take the default schedule: every band must run the same dispatches)
  inst->ops = m->ops;
  inst->tensors = m->tensors;
  if (m->from_dnx) inst->preset_variant = m->dnx_variants;  // a compiled model: schedule and variants are the file's
  if (m->db && !band && !m->from_dnx) {
    std::vector<FusedOp> sel_ops;
    std::vector<TensorInfo> sel_tensors;
    std::vector<int> sel_variants;
    st = select_schedule(*m, m->db, allow_tc, inst->H, width, sel_ops, sel_tensors, sel_variants, nullptr);
    if (st) return st;
    inst->ops.swap(sel_ops);
    inst->tensors.swap(sel_tensors);
    inst->preset_variant.swap(sel_variants);
  }
  const std::vector<FusedOp> &ops = inst->ops;
  const std::vector<TensorInfo> &tensors = inst->tensors;

  DNXCU_CUDA(cudaSetDevice(m->device));
  DNXCU_CUDA(cudaStreamCreateWithFlags(&inst->stream, cudaStreamNonBlocking));
  st = dev_alloc(*inst, 256, (void **)&inst->status);
  if (st) return st;
  DNXCU_CUDA(cudaMemset(inst->status, 0, 256));

  const int NT = (int)tensors.size();
  inst->tensor_ptr.assign(NT, nullptr);
  for (int t = 0; t < NT; ++t) {
    const TensorInfo &ti = tensors[t];
    if (!ti.materialized) continue;
    const size_t bytes = (size_t)(inst->H >> ti.level) * (width >> ti.level) * ti.channels * 2;
    st = dev_alloc(*inst, bytes, &inst->tensor_ptr[t]);
    if (st) return st;
  }

  // kernel attributes now, so that no launch needs set-up work later (a launch may sit inside a stream capture)
  if (allow_tc && (st = conv_tc_init_device())) return st;

  inst->disp.resize(ops.size());
  inst->plans.assign(ops.size(), nullptr);
  if (inst->banded) {
    // lay out the halo arena: per conv operand a slab above and a slab below (256 byte aligned), then the flags
    size_t off = 0;
    uint64_t hsh = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { hsh = (hsh ^ v) * 1099511628211ull; };
    mix((uint64_t)width);
    mix((uint64_t)inst->H);
    for (size_t i = 0; i < ops.size(); ++i) {
      const FusedOp &op = ops[i];
      if (op.op != DNXCU_OP_CONV3X3) continue;
      for (int sgi = 0; sgi < 2; ++sgi) {
        const int t = sgi ? op.in_b : op.in_a;
        if (t < 0) continue;
        const TensorInfo &ti = tensors[t];
        const size_t row_bytes = (size_t)(width >> ti.level) * ti.channels * 2;
        const size_t slab = (row_bytes + 255) & ~(size_t)255;
        dnxcu_instance::HaloSlot hs;
        hs.dispatch = (int)i;
        hs.top_off = off;
        hs.bot_off = off + slab;
        hs.flag_off = 0;
        off += 2 * slab;
        inst->halo_slots.push_back(hs);
        mix((uint64_t)i * 4 + (uint64_t)sgi);
        mix((uint64_t)row_bytes);
      }
    }
    for (size_t e = 0; e < inst->halo_slots.size(); ++e) inst->halo_slots[e].flag_off = off + e * 8;
    off += (inst->halo_slots.size() * 8 + 255) & ~(size_t)255;
    inst->arena_bytes = off;
    inst->arena_layout = hsh;
    void *ar = nullptr, *ctl = nullptr;
    st = dev_alloc(*inst, off, &ar);
    if (st) return st;
    DNXCU_CUDA(cudaMemset(ar, 0, off));
    inst->arena = (char *)ar;
    st = dev_alloc(*inst, ops.size() * 2 * sizeof(unsigned), &ctl);
    if (st) return st;
    DNXCU_CUDA(cudaMemset(ctl, 0, ops.size() * 2 * sizeof(unsigned)));
    inst->xchg_ctl = (unsigned *)ctl;
  }
  size_t next_slot = 0;
  for (size_t i = 0; i < ops.size(); ++i) {
    const FusedOp &op = ops[i];
    dnxcu_dispatch d;
    memset(&d, 0, sizeof(d));
    d.flags = op.flags;
    d.pc[0] = (uint32_t)(width >> op.level);
    d.pc[1] = (uint32_t)(inst->H >> op.level);
    d.c_a = op.c_a;
    d.c_b = op.c_b;
    d.c_out = op.c_out;
    d.in_a = inst->tensor_ptr[op.in_a];
    d.in_b = op.in_b >= 0 ? inst->tensor_ptr[op.in_b] : nullptr;
    d.out = (op.flags & DNXCU_F_NO_FULL_OUT) ? nullptr : inst->tensor_ptr[op.out];
    d.out_pool = op.out_pool >= 0 ? inst->tensor_ptr[op.out_pool] : nullptr;
    d.device_status = inst->status;
    d.leaky_alpha = op.alpha;
    if (!d.in_a || (op.in_b >= 0 && !d.in_b)) return DNXCU_E_STATE;

    if (op.op == DNXCU_OP_CONV3X3) {
      // halo slabs of a row band: one row above and below per operand
      if (inst->banded) {
        for (int sgi = 0; sgi < 2; ++sgi) {
          const int t = sgi ? op.in_b : op.in_a;
          if (t < 0) continue;
          const TensorInfo &ti = tensors[t];
          const size_t row_bytes = (size_t)(width >> ti.level) * ti.channels * 2;
          const size_t th = (size_t)(inst->H >> ti.level);
          dnxcu_halo_point hp;
          memset(&hp, 0, sizeof(hp));
          hp.before_dispatch = (int)i;
          hp.tensor = t;
          hp.row_bytes = row_bytes;
          hp.send_top = inst->tensor_ptr[t];
          hp.send_bottom = (const char *)inst->tensor_ptr[t] + (th - 1) * row_bytes;
          const dnxcu_instance::HaloSlot &hs = inst->halo_slots[next_slot++];
          if (has_up) hp.recv_top = inst->arena + hs.top_off;
          if (has_down) hp.recv_bottom = inst->arena + hs.bot_off;
          d.halo[sgi * 2 + 0] = hp.recv_top;
          d.halo[sgi * 2 + 1] = hp.recv_bottom;
          inst->halos.push_back(hp);
        }
      }
      void *dbias = nullptr;
      if (!op.bias.empty()) {
        st = dev_alloc(*inst, op.bias.size() * 2, &dbias);
        if (st) return st;
        DNXCU_CUDA(cudaMemcpy(dbias, op.bias.data(), op.bias.size() * 2, cudaMemcpyHostToDevice));
        d.bias = dbias;
      }
    }

    // choose the variant: lowest database latency among those that accept the
    // dispatch (selection.cpp:43-123), else the first in preference order
    std::vector<int> cand;
    if (!inst->preset_variant.empty()) cand.push_back(inst->preset_variant[i]);  // the selection's choice
    else candidate_variants(op, allow_tc, cand);
    int chosen = -1;
    double best_ms = 0;
    d.weights = (const void *)0x1000;  // placeholder that passes the alignment checks
    for (int id : cand) {
      d.variant = id;
      if (dnxcu_validate(&d) != DNXCU_OK) continue;
      double ms = 0;
      int ns = 0;
      if (m->db && dnxcu_db_query(m->db, &d, &ms, nullptr, &ns) == DNXCU_OK && ns > 0) {
        if (chosen < 0 || best_ms == 0 || ms < best_ms) {
          chosen = id;
          best_ms = ms;
        }
      } else if (chosen < 0) {
        chosen = id;
      }
    }
    if (chosen < 0) return DNXCU_E_UNSUPPORTED;
    d.variant = chosen;
    d.weights = nullptr;
    if (op.op == DNXCU_OP_CONV3X3) {
      size_t bytes = 0;
      st = dnxcu_prepare_weights(chosen, nullptr, op.c_out, op.c_a, op.c_b, nullptr, &bytes);
      if (st) return st;
      std::vector<unsigned char> blob(bytes);
      if (!op.prepared.empty()) {
        if (op.prepared.size() != bytes) return DNXCU_E_STATE;
        blob = op.prepared;  // a dnx file carries the weights in the variant's layout already
      } else {
        st = dnxcu_prepare_weights(chosen, op.weights_kcrs.data(), op.c_out, op.c_a, op.c_b, blob.data(), &bytes);
        if (st) return st;
      }
      void *dw = nullptr;
      st = dev_alloc(*inst, bytes, &dw);
      if (st) return st;
      DNXCU_CUDA(cudaMemcpy(dw, blob.data(), bytes, cudaMemcpyHostToDevice));
      d.weights = dw;
    }
    inst->disp[i] = d;
    st = dnxcu_plan_create(&d, &inst->plans[i]);
    if (st) return st;
  }
  if (inst->padded) {
    const TensorInfo &ti = tensors[m->input_tensor], &to = tensors[m->output_tensor];
    st = dev_alloc(*inst, (size_t)inst->user_H * inst->user_W * ti.channels * 2, &inst->user_in);
    if (st) return st;
    st = dev_alloc(*inst, (size_t)inst->user_H * inst->user_W * to.channels * 2, &inst->user_out);
    if (st) return st;
    dnxcu_dispatch &p = inst->pre, &q = inst->post;
    p.variant = dnxcu_find_variant("memory-pad", ti.channels % 8 ? "VEC=1" : "VEC=8");
    p.pc[0] = (uint32_t)inst->W;
    p.pc[1] = (uint32_t)inst->H;
    p.c_a = ti.channels;
    p.pc_ext[1] = (uint32_t)(inst->W - inst->user_W);
    p.pc_ext[3] = (uint32_t)(inst->H - inst->user_H);
    p.in_a = inst->user_in;
    p.out = inst->tensor_ptr[m->input_tensor];
    q.variant = dnxcu_find_variant("memory-slice", to.channels % 8 ? "VEC=1" : "VEC=8");
    q.pc[0] = (uint32_t)inst->user_W;
    q.pc[1] = (uint32_t)inst->user_H;
    q.c_a = to.channels;
    q.pc_ext[2] = (uint32_t)inst->W;
    q.pc_ext[3] = (uint32_t)inst->H;
    q.in_a = inst->tensor_ptr[m->output_tensor];
    q.out = inst->user_out;
    if (p.variant < 0 || q.variant < 0 || !p.out || !q.in_a) return DNXCU_E_STATE;
    if ((st = dnxcu_validate(&p)) || (st = dnxcu_validate(&q))) return st;
  }
  inst->events.resize(inst->disp.size() + 1);
  for (cudaEvent_t &e : inst->events) DNXCU_CUDA(cudaEventCreate(&e));
  *out = inst.release();
  return DNXCU_OK;
}

void dnxcu_instance_destroy(dnxcu_instance *inst) {
  if (!inst) return;
  cudaSetDevice(inst->model->device);
  delete inst;
}

int dnxcu_instance_enqueue_range(dnxcu_instance *inst, int first, int last, void *stream) {
  if (!inst || first < 0 || last > (int)inst->disp.size() || first > last) return DNXCU_E_BAD_ARG;
  for (int i = first; i < last; ++i) {
    int st = launch_one(*inst, i, nullptr, nullptr, (cudaStream_t)stream);
    if (st) return st;
  }
  return DNXCU_OK;
}

int dnxcu_instance_enqueue(dnxcu_instance *inst, const void *dev_in, void *dev_out, void *stream) {
  if (!inst || !dev_in || !dev_out) return DNXCU_E_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  // The schedule is a fixed chain of launches: capture it once per (in, out) pointer pair and replay the
  // graph (one launch instead of one per dispatch).  Capturing records the launches on the instance's own
  // stream without running anything, so nothing here touches the caller's buffers or waits for the device.
  size_t hit = 0;
  while (hit < inst->graphs.size() && (inst->graphs[hit].in != dev_in || inst->graphs[hit].out != dev_out)) ++hit;
  if (hit == inst->graphs.size()) {
    // caller-extent frames: pad into the model's own input tensor first, slice out of its own output tensor last
    auto whole = [&]() -> int {
      int st = DNXCU_OK;
      if (inst->padded) {
        dnxcu_dispatch p = inst->pre;
        p.in_a = dev_in;
        st = dnxcu_launch(&p, inst->stream);
      }
      for (size_t i = 0; i < inst->disp.size() && !st; ++i)
        st = launch_one(*inst, (int)i, inst->padded ? nullptr : dev_in, inst->padded ? nullptr : dev_out, inst->stream);
      if (inst->padded && !st) {
        dnxcu_dispatch q = inst->post;
        q.out = dev_out;
        st = dnxcu_launch(&q, inst->stream);
      }
      return st;
    };
    cudaGraph_t gr = nullptr;
    // relaxed mode: only this instance's private stream is captured; other threads' CUDA calls are not its business
    DNXCU_CUDA(cudaStreamBeginCapture(inst->stream, cudaStreamCaptureModeRelaxed));
    int st = whole();
    cudaError_t e = cudaStreamEndCapture(inst->stream, &gr);
    if (st) {
      if (gr) cudaGraphDestroy(gr);
      return st;
    }
    if (e != cudaSuccess) return cuda_fail(e);
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, gr, 0);
    cudaGraphDestroy(gr);
    if (e != cudaSuccess) return cuda_fail(e);
    if (inst->graphs.size() >= inst->graph_capacity) {  // keep the most recently used pairs
      cudaGraphExecDestroy(inst->graphs.back().exec);
      inst->graphs.pop_back();
    }
    inst->graphs.insert(inst->graphs.begin(), dnxcu_instance::Graph{exec, dev_in, dev_out});
    hit = 0;
  } else if (hit > 0) {
    const dnxcu_instance::Graph g = inst->graphs[hit];
    inst->graphs.erase(inst->graphs.begin() + (long)hit);
    inst->graphs.insert(inst->graphs.begin(), g);
    hit = 0;
  }
  DNXCU_CUDA(cudaGraphLaunch(inst->graphs[0].exec, s));
  return DNXCU_OK;
}

int dnxcu_instance_graph_cache(dnxcu_instance *inst, int pairs) {
  if (!inst || pairs < 1 || pairs > 256) return DNXCU_E_BAD_ARG;
  inst->graph_capacity = (size_t)pairs;
  while (inst->graphs.size() > inst->graph_capacity) {
    cudaGraphExecDestroy(inst->graphs.back().exec);
    inst->graphs.pop_back();
  }
  return DNXCU_OK;
}

// Host in, host out, but stream ordered: the copies and the schedule are enqueued on the instance's own
// stream and the call returns.  Several instances used round robin overlap one frame's copies with another
// frame's kernels.  The host buffers must stay valid (and should be pinned) until dnxcu_instance_wait returns.
int dnxcu_instance_infer_async(dnxcu_instance *inst, const void *host_in, void *host_out) {
  if (!inst || !host_in || !host_out) return DNXCU_E_BAD_ARG;
  const dnxcu_model *m = inst->model;
  DNXCU_CUDA(cudaSetDevice(m->device));
  void *din = inst->padded ? inst->user_in : inst->tensor_ptr[m->input_tensor];
  void *dout = inst->padded ? inst->user_out : inst->tensor_ptr[m->output_tensor];
  if (!din || !dout) return DNXCU_E_STATE;
  const TensorInfo &ti = inst->tensors[m->input_tensor], &to = inst->tensors[m->output_tensor];
  const int fh = inst->padded ? inst->user_H : inst->H, fw = inst->padded ? inst->user_W : inst->W;
  const size_t in_bytes = (size_t)fh * fw * ti.channels * 2;
  const size_t out_bytes = (size_t)(fh >> to.level) * (fw >> to.level) * to.channels * 2;
  DNXCU_CUDA(cudaMemcpyAsync(din, host_in, in_bytes, cudaMemcpyHostToDevice, inst->stream));
  int st = dnxcu_instance_enqueue(inst, din, dout, inst->stream);
  if (st) return st;
  DNXCU_CUDA(cudaMemcpyAsync(host_out, dout, out_bytes, cudaMemcpyDeviceToHost, inst->stream));
  return DNXCU_OK;
}

int dnxcu_instance_wait(dnxcu_instance *inst) {
  if (!inst) return DNXCU_E_BAD_ARG;
  DNXCU_CUDA(cudaSetDevice(inst->model->device));
  DNXCU_CUDA(cudaStreamSynchronize(inst->stream));
  int hstatus = 0;
  DNXCU_CUDA(cudaMemcpy(&hstatus, inst->status, sizeof(int), cudaMemcpyDeviceToHost));
  return take_status(*inst, hstatus);
}

int dnxcu_instance_infer(dnxcu_instance *inst, const void *host_in, void *host_out) {
  if (!inst || !host_in || !host_out) return DNXCU_E_BAD_ARG;
  const dnxcu_model *m = inst->model;
  DNXCU_CUDA(cudaSetDevice(m->device));
  void *din = inst->padded ? inst->user_in : inst->tensor_ptr[m->input_tensor];
  void *dout = inst->padded ? inst->user_out : inst->tensor_ptr[m->output_tensor];
  if (!din || !dout) return DNXCU_E_STATE;
  const TensorInfo &ti = inst->tensors[m->input_tensor], &to = inst->tensors[m->output_tensor];
  const int fh = inst->padded ? inst->user_H : inst->H, fw = inst->padded ? inst->user_W : inst->W;
  const size_t in_bytes = (size_t)fh * fw * ti.channels * 2;
  const size_t out_bytes = (size_t)(fh >> to.level) * (fw >> to.level) * to.channels * 2;
  DNXCU_CUDA(cudaMemcpyAsync(din, host_in, in_bytes, cudaMemcpyHostToDevice, inst->stream));
  int st = dnxcu_instance_enqueue(inst, din, dout, inst->stream);
  if (st) return st;
  DNXCU_CUDA(cudaMemcpyAsync(host_out, dout, out_bytes, cudaMemcpyDeviceToHost, inst->stream));
  int hstatus = 0;
  DNXCU_CUDA(cudaMemcpyAsync(&hstatus, inst->status, sizeof(int), cudaMemcpyDeviceToHost, inst->stream));
  DNXCU_CUDA(cudaStreamSynchronize(inst->stream));
  return take_status(*inst, hstatus);
}

int dnxcu_instance_tensor(const dnxcu_instance *inst, int t, void **ptr, int *h, int *w, int *c) {
  if (!inst || t < 0 || t >= (int)inst->tensor_ptr.size()) return DNXCU_E_BAD_ARG;
  const TensorInfo &ti = inst->tensors[t];
  if (ptr) *ptr = inst->tensor_ptr[t];
  if (h) *h = inst->H >> ti.level;
  if (w) *w = inst->W >> ti.level;
  if (c) *c = ti.channels;
  return inst->tensor_ptr[t] ? DNXCU_OK : DNXCU_E_STATE;
}

int dnxcu_instance_io(const dnxcu_instance *inst, void **dev_in, void **dev_out) {
  if (!inst) return DNXCU_E_BAD_ARG;
  if (dev_in) *dev_in = inst->padded ? inst->user_in : inst->tensor_ptr[inst->model->input_tensor];
  if (dev_out) *dev_out = inst->padded ? inst->user_out : inst->tensor_ptr[inst->model->output_tensor];
  return DNXCU_OK;
}

int dnxcu_instance_extent(const dnxcu_instance *inst, int *h, int *w, int *h_run, int *w_run) {
  if (!inst) return DNXCU_E_BAD_ARG;
  if (h) *h = inst->padded ? inst->user_H : inst->H;
  if (w) *w = inst->padded ? inst->user_W : inst->W;
  if (h_run) *h_run = inst->H;
  if (w_run) *w_run = inst->W;
  return DNXCU_OK;
}

int dnxcu_instance_dispatch_info(const dnxcu_instance *inst, int i, dnxcu_dispatch_info *info) {
  if (!inst || !info || i < 0 || i >= (int)inst->disp.size()) return DNXCU_E_BAD_ARG;
  const FusedOp &op = inst->ops[i];
  const dnxcu_dispatch &d = inst->disp[i];
  memset(info, 0, sizeof(*info));
  const dnxcu_variant_desc *vd = dnxcu_variant(d.variant);
  std::string name = op.name;
  if (op.op == DNXCU_OP_CONV3X3 && vd && strcmp(vd->family, "direct-conv-tc") == 0) {
    const size_t pos = name.find("conv");
    if (pos != std::string::npos) name.insert(pos + 4, "-tc");
  }
  strncpy(info->name, name.c_str(), sizeof(info->name) - 1);
  info->variant = d.variant;
  info->src_node = op.src_node;
  dnxcu_grid(&d, info->grid);
  info->flags = d.flags;
  dnxcu_cost(&d, &info->bytes_read, &info->bytes_written, &info->flops);
  info->w = (int)d.pc[0];
  info->h = (int)d.pc[1];
  info->c_a = d.c_a;
  info->c_b = d.c_b;
  info->c_out = d.c_out;
  info->out_tensor = (op.flags & DNXCU_F_NO_FULL_OUT) ? op.out_pool : op.out;
  return DNXCU_OK;
}

int dnxcu_instance_bench(dnxcu_instance *inst, int warmup, int iters, dnxcu_dispatch_info *info, int n_info,
                         float *total_ms) {
  if (!inst || iters <= 0 || warmup < 0) return DNXCU_E_BAD_ARG;
  const int n = (int)inst->disp.size();
  if (info && n_info < n) return DNXCU_E_BAD_ARG;
  DNXCU_CUDA(cudaSetDevice(inst->model->device));
  for (int w = 0; w < warmup; ++w) {
    int st = dnxcu_instance_enqueue_range(inst, 0, n, inst->stream);
    if (st) return st;
  }
  std::vector<double> acc(n, 0.0);
  double total = 0;
  for (int it = 0; it < iters; ++it) {
    // An untimed frame goes first, so the device is busy while the host enqueues the timed one: otherwise the
    // intervals of dispatches shorter than a launch call (the small levels) measure the host, not the kernel.
    // (The reference times with device timestamps inside one recorded command buffer.)
    if (it > 0 || warmup == 0) {
      int st = dnxcu_instance_enqueue_range(inst, 0, n, inst->stream);
      if (st) return st;
    }
    DNXCU_CUDA(cudaEventRecord(inst->events[0], inst->stream));
    for (int i = 0; i < n; ++i) {
      int st = launch_one(*inst, i, nullptr, nullptr, inst->stream);
      if (st) return st;
      DNXCU_CUDA(cudaEventRecord(inst->events[i + 1], inst->stream));
    }
    DNXCU_CUDA(cudaStreamSynchronize(inst->stream));
    for (int i = 0; i < n; ++i) {
      float ms = 0;
      DNXCU_CUDA(cudaEventElapsedTime(&ms, inst->events[i], inst->events[i + 1]));
      acc[i] += ms;
      total += ms;
    }
  }
  if (info)
    for (int i = 0; i < n; ++i) {
      dnxcu_instance_dispatch_info(inst, i, &info[i]);
      info[i].ms = (float)(acc[i] / iters);
    }
  if (total_ms) *total_ms = (float)(total / iters);
  int hstatus = 0;
  DNXCU_CUDA(cudaMemcpy(&hstatus, inst->status, sizeof(int), cudaMemcpyDeviceToHost));
  return take_status(*inst, hstatus);
}

// ---- halo exchange over peer memory ----------------------------------------------

int dnxcu_instance_halo_export(const dnxcu_instance *inst, dnxcu_peer_handle *out) {
  if (!inst || !out) return DNXCU_E_BAD_ARG;
  if (!inst->banded || !inst->arena) return DNXCU_E_STATE;
  memset(out, 0, sizeof(*out));
  DNXCU_CUDA(cudaSetDevice(inst->model->device));
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) <= sizeof(out->ipc), "handle does not fit");
  DNXCU_CUDA(cudaIpcGetMemHandle(&h, inst->arena));
  memcpy(out->ipc, &h, sizeof(h));
  out->arena_bytes = inst->arena_bytes;
  out->layout = inst->arena_layout;
  out->device = inst->model->device;
  out->pid = (int64_t)getpid();
  out->local_ptr = (uint64_t)(uintptr_t)inst->arena;
  out->row0 = inst->band.row0;
  out->rows = inst->band.rows;
  return DNXCU_OK;
}

int dnxcu_instance_halo_connect(dnxcu_instance *inst, const dnxcu_peer_handle *up, const dnxcu_peer_handle *down,
                                int auto_exchange) {
  if (!inst) return DNXCU_E_BAD_ARG;
  if (!inst->banded || !inst->arena || inst->connected) return DNXCU_E_STATE;
  const bool has_up = inst->band.row0 > 0, has_down = inst->band.row0 + inst->band.rows < inst->band.image_h;
  if ((has_up && !up) || (has_down && !down)) return DNXCU_E_BAD_ARG;
  DNXCU_CUDA(cudaSetDevice(inst->model->device));
  // the neighbour must be the band directly above / below, of the same height and layout (same model, same width)
  auto check = [&](const dnxcu_peer_handle *p, bool above) -> int {
    if (p->arena_bytes != inst->arena_bytes || p->layout != inst->arena_layout || p->rows != inst->band.rows)
      return DNXCU_E_BAD_ARG;
    const int want_row0 = above ? inst->band.row0 - inst->band.rows : inst->band.row0 + inst->band.rows;
    return p->row0 == want_row0 ? DNXCU_OK : DNXCU_E_BAD_ARG;
  };
  auto open = [&](const dnxcu_peer_handle *p, char **base, bool *ipc) -> int {
    if (p->pid == (int64_t)getpid()) {
      // a band of this process: its pointer is usable as it is on the same device; another device of this
      // process needs peer access switched on
      if (p->device != inst->model->device) {
        cudaError_t e = cudaDeviceEnablePeerAccess(p->device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e);
        cudaGetLastError();
      }
      *base = (char *)(uintptr_t)p->local_ptr;
      *ipc = false;
      return DNXCU_OK;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, p->ipc, sizeof(h));
    void *ptr = nullptr;
    DNXCU_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    *base = (char *)ptr;
    *ipc = true;
    return DNXCU_OK;
  };
  int st;
  if (has_up && ((st = check(up, true)) || (st = open(up, &inst->peer_up, &inst->peer_up_ipc)))) return st;
  if (has_down && ((st = check(down, false)) || (st = open(down, &inst->peer_down, &inst->peer_down_ipc)))) return st;

  inst->xchg.assign(inst->disp.size(), dnxcu::XchgArgs());
  for (dnxcu::XchgArgs &a : inst->xchg) memset(&a, 0, sizeof(a));
  for (size_t e = 0; e < inst->halos.size(); ++e) {
    const dnxcu_halo_point &hp = inst->halos[e];
    const dnxcu_instance::HaloSlot &hs = inst->halo_slots[e];
    if (hp.row_bytes % 16) return DNXCU_E_UNSUPPORTED;
    dnxcu::XchgArgs &a = inst->xchg[hs.dispatch];
    if (a.npoints >= XCHG_MAX_POINTS) return DNXCU_E_LIMIT;
    dnxcu::XchgPoint &q = a.pt[a.npoints++];
    q.send_top = (const uint4 *)hp.send_top;
    q.send_bottom = (const uint4 *)hp.send_bottom;
    q.n16 = (unsigned)(hp.row_bytes / 16);
    // my first row is the upper neighbour's "row below"; my last row is the lower neighbour's "row above"
    q.peer_up_slab = has_up ? (uint4 *)(inst->peer_up + hs.bot_off) : nullptr;
    q.peer_up_flag = has_up ? (unsigned *)(inst->peer_up + hs.flag_off + 4) : nullptr;
    q.peer_down_slab = has_down ? (uint4 *)(inst->peer_down + hs.top_off) : nullptr;
    q.peer_down_flag = has_down ? (unsigned *)(inst->peer_down + hs.flag_off) : nullptr;
    q.my_flag_top = has_up ? (unsigned *)(inst->arena + hs.flag_off) : nullptr;
    q.my_flag_bottom = has_down ? (unsigned *)(inst->arena + hs.flag_off + 4) : nullptr;
    a.done = inst->xchg_ctl + 2 * hs.dispatch;
    a.counter = inst->xchg_ctl + 2 * hs.dispatch + 1;
    a.status = inst->status;
  }
  inst->connected = true;
  inst->auto_exchange = auto_exchange != 0;
  return DNXCU_OK;
}

int dnxcu_instance_halo_step(dnxcu_instance *inst, int dispatch, uint32_t mode, void *stream) {
  if (!inst || dispatch < 0 || dispatch >= (int)inst->disp.size() || !(mode & 3u) || (mode & ~3u)) return DNXCU_E_BAD_ARG;
  if (!inst->connected) return DNXCU_E_STATE;
  if (inst->xchg[dispatch].npoints == 0) return DNXCU_OK;
  dnxcu::XchgArgs a = inst->xchg[dispatch];
  a.mode = mode;
  a.wait_limit = wait_limit_cycles();
  return halo_xchg_launch(a, (cudaStream_t)stream);
}

int dnxcu_instance_halo_reset(dnxcu_instance *inst) {
  if (!inst) return DNXCU_E_BAD_ARG;
  if (!inst->banded || !inst->arena) return DNXCU_E_STATE;
  DNXCU_CUDA(cudaSetDevice(inst->model->device));
  DNXCU_CUDA(cudaDeviceSynchronize());
  const size_t flags_off = inst->halo_slots.empty() ? inst->arena_bytes : inst->halo_slots[0].flag_off;
  DNXCU_CUDA(cudaMemset(inst->arena + flags_off, 0, inst->arena_bytes - flags_off));
  DNXCU_CUDA(cudaMemset(inst->xchg_ctl, 0, inst->disp.size() * 2 * sizeof(unsigned)));
  DNXCU_CUDA(cudaDeviceSynchronize());
  return DNXCU_OK;
}

int dnxcu_instance_halo_auto(dnxcu_instance *inst, int on) {
  if (!inst) return DNXCU_E_BAD_ARG;
  if (!inst->connected) return DNXCU_E_STATE;
  inst->auto_exchange = on != 0;
  for (dnxcu_instance::Graph &g : inst->graphs) cudaGraphExecDestroy(g.exec);
  inst->graphs.clear();  // captured under the other setting
  return DNXCU_OK;
}

int dnxcu_instance_halo_count(const dnxcu_instance *inst) { return inst ? (int)inst->halos.size() : DNXCU_E_BAD_ARG; }
int dnxcu_instance_halo(const dnxcu_instance *inst, int e, dnxcu_halo_point *p) {
  if (!inst || !p || e < 0 || e >= (int)inst->halos.size()) return DNXCU_E_BAD_ARG;
  *p = inst->halos[e];
  return DNXCU_OK;
}

}  // extern "C"
