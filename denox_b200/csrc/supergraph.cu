// The hypergraph of candidate dispatches of a model ("SuperGraph") and the cost driven choice of a schedule.
//
// Every way this backend can compute a tensor of the model becomes a hyperedge: each node on its own, and each
// fusion pattern that applies (conv -> activation, concat -> conv, upsample -> [concat ->] conv, conv [->
// activation] -> max pool), each once per kernel variant that accepts the dispatch at the instance's extent.  The
// reference builds the same structure in implement() (compiler/src/denox/compiler/implement/implement.cpp:11-68:
// every IShader pattern match x every configuration becomes a SuperGraph edge), filters it by dispatch count
// (dce/prune_topological.cpp:86-152) and picks the cheapest sub-graph with the latencies of its benchmark
// database (selection/selection.cpp:23-270).  populate (compiler/src/denox/compiler/populate.cpp:23-256) walks
// the same filtered graph and adds its dispatches to the database.
#include "runtime.h"
#include "select.h"
#include <string.h>
#include <algorithm>

namespace dnxcu {
namespace {

struct GraphInfo {
  std::vector<int> producer;                // node that writes the tensor, -1 for the input
  std::vector<std::vector<int>> consumers;  // nodes that read the tensor
};

GraphInfo analyse(const dnxcu_model &m) {
  GraphInfo gi;
  const int NT = m.n_model_tensors;
  gi.producer.assign(NT, -1);
  gi.consumers.assign(NT, {});
  for (int i = 0; i < (int)m.nodes.size(); ++i) {
    const NodeRec &n = m.nodes[i];
    gi.producer[n.out] = i;
    gi.consumers[n.in0].push_back(i);
    if (n.kind == DNXCU_NODE_CONCAT) gi.consumers[n.in1].push_back(i);
  }
  return gi;
}

}  // namespace

// Validation probe of an op at the instance's extent (placeholders for the pointers: validation never
// dereferences them).
dnxcu_dispatch probe_dispatch(const FusedOp &op, int H, int W, int variant) {
  dnxcu_dispatch d;
  memset(&d, 0, sizeof(d));
  void *const probe = (void *)0x1000;
  d.variant = variant;
  d.flags = op.flags;
  d.pc[0] = (uint32_t)(W >> op.level);
  d.pc[1] = (uint32_t)(H >> op.level);
  d.c_a = op.c_a;
  d.c_b = op.c_b;
  d.c_out = op.c_out;
  d.leaky_alpha = op.alpha;
  d.in_a = probe;
  d.in_b = op.c_b > 0 ? probe : nullptr;
  d.out = (op.flags & DNXCU_F_NO_FULL_OUT) ? nullptr : probe;
  d.out_pool = (op.flags & DNXCU_F_POOL_OUT) ? probe : nullptr;
  d.weights = probe;
  d.bias = (op.flags & DNXCU_F_BIAS) ? probe : nullptr;
  return d;
}

int build_supergraph(const dnxcu_model &m, bool allow_tc, int H, int W, HyperGraph &g, std::vector<Candidate> &cands) {
  const int NT = m.n_model_tensors;
  const GraphInfo gi = analyse(m);
  const uint32_t opt = m.options;
  const bool f_act = !(opt & DNXCU_OPT_NO_FUSE_ACTIVATION);
  const bool f_pool = !(opt & DNXCU_OPT_NO_FUSE_POOL) && allow_tc;
  const bool f_up = !(opt & DNXCU_OPT_NO_FUSE_UPSAMPLE);
  const bool f_cat = !(opt & DNXCU_OPT_NO_FUSE_CONCAT);
  const bool ragged_in = (m.input_channels % 8) != 0;
  const bool pad_in = ragged_in && allow_tc && !(opt & DNXCU_OPT_NO_PAD_INPUT);
  const int padded = NT;  // tensor id of the zero padded copy of a ragged input
  const int Cp = (m.input_channels + 15) / 16 * 16;
  g.n_nodes = NT + 1;
  g.edges.clear();
  cands.clear();
  auto sole = [&](int t, int node) {
    return gi.consumers[t].size() == 1 && gi.consumers[t][0] == node && t != m.output_tensor;
  };
  // one edge per variant that takes the op at this extent
  auto add = [&](const FusedOp &op, const std::vector<int> &src, const std::vector<int> &dst) {
    for (int id = 0; id < variant_count(); ++id) {
      const Variant *v = get_variant(id);
      if (v->desc.op != op.op || (op.flags & ~v->desc.allowed_flags)) continue;
      if (v->desc.needs_tcgen05 && !allow_tc) continue;
      const dnxcu_dispatch d = probe_dispatch(op, H, W, id);
      if (dnxcu_validate(&d) != DNXCU_OK) continue;
      Candidate c;
      c.op = op;
      c.variant = id;
      cands.push_back(std::move(c));
      HyperEdge e;
      e.src = src;
      e.dst = dst;
      e.weight = kUnbenchmarkedMs;
      e.dispatches = 1;
      e.payload = (int)cands.size() - 1;
      g.edges.push_back(std::move(e));
    }
  };
  for (int i = 0; i < (int)m.nodes.size(); ++i) {
    const NodeRec &n = m.nodes[i];
    FusedOp base;
    base.src_node = i;
    base.in_a = n.in0;
    base.out = n.out;
    base.c_a = m.tensors[n.in0].channels;
    base.level = m.tensors[n.in0].level;
    switch (n.kind) {
      case DNXCU_NODE_RELU:
        base.op = DNXCU_OP_RELU;
        base.name = "basic-activation";
        add(base, {n.in0}, {n.out});
        break;
      case DNXCU_NODE_LEAKY_RELU:
        base.op = DNXCU_OP_RELU;
        base.flags = DNXCU_F_LEAKY;
        base.alpha = n.alpha;
        base.name = "basic-activation(leaky)";
        add(base, {n.in0}, {n.out});
        break;
      case DNXCU_NODE_MAXPOOL:
        base.op = DNXCU_OP_MAXPOOL2X2;
        base.name = "basic-pool";
        add(base, {n.in0}, {n.out});
        break;
      case DNXCU_NODE_UPSAMPLE:
        base.op = DNXCU_OP_UPSAMPLE2X;
        base.name = "basic-upsample";
        add(base, {n.in0}, {n.out});
        break;
      case DNXCU_NODE_CONCAT:
        base.op = DNXCU_OP_CONCAT;
        base.in_b = n.in1;
        base.c_b = m.tensors[n.in1].channels;
        base.name = "copy-transform";
        add(base, {n.in0, n.in1}, {n.out});
        break;
      case DNXCU_NODE_CONV: {
        // operand choices: the conv's own input; the two operands of a concat that feeds only this conv; either
        // with a 2x upsample in front of operand a read through the conv's address map
        struct Operands {
          int a, b, up;
        };
        std::vector<Operands> operands;
        operands.push_back({n.in0, -1, 0});
        const int pc = gi.producer[n.in0];
        if (f_cat && pc >= 0 && m.nodes[pc].kind == DNXCU_NODE_CONCAT && sole(n.in0, i)) {
          operands.push_back({m.nodes[pc].in0, m.nodes[pc].in1, 0});
          const int pu = gi.producer[m.nodes[pc].in0];
          if (f_up && pu >= 0 && m.nodes[pu].kind == DNXCU_NODE_UPSAMPLE && sole(m.nodes[pc].in0, pc))
            operands.push_back({m.nodes[pu].in0, m.nodes[pc].in1, 1});
        } else if (f_up && pc >= 0 && m.nodes[pc].kind == DNXCU_NODE_UPSAMPLE && sole(n.in0, i)) {
          operands.push_back({m.nodes[pc].in0, -1, 1});
        }
        // activation choices: none; the ReLU / LeakyReLU that alone reads the conv's output
        struct Act {
          int node;  // -1: none
        };
        std::vector<Act> acts;
        acts.push_back({-1});
        if (f_act && gi.consumers[n.out].size() == 1 && sole(n.out, gi.consumers[n.out][0])) {
          const int an = gi.consumers[n.out][0];
          if (m.nodes[an].kind == DNXCU_NODE_RELU || m.nodes[an].kind == DNXCU_NODE_LEAKY_RELU) acts.push_back({an});
        }
        for (const Operands &o : operands)
          for (const Act &act : acts) {
            const int out_t = act.node >= 0 ? m.nodes[act.node].out : n.out;
            // pool choices: none; the max pool that reads the result (the full result stays when others read it too)
            int pool_node = -1;
            if (f_pool)
              for (int c : gi.consumers[out_t])
                if (m.nodes[c].kind == DNXCU_NODE_MAXPOOL && pool_node < 0) pool_node = c;
            for (int with_pool = 0; with_pool <= (pool_node >= 0 ? 1 : 0); ++with_pool) {
              // a ragged network input can be read as it is or through its zero padded copy
              const bool a_is_in = o.a == m.input_tensor, b_is_in = o.b == m.input_tensor;
              const int pad_choices = (pad_in && (a_is_in || b_is_in)) ? 2 : 1;
              for (int use_pad = 0; use_pad < pad_choices; ++use_pad) {
                FusedOp op;
                op.op = DNXCU_OP_CONV3X3;
                op.src_node = i;
                op.in_a = (use_pad && a_is_in) ? padded : o.a;
                op.in_b = (use_pad && b_is_in) ? padded : o.b;
                op.c_a = (use_pad && a_is_in) ? Cp : m.tensors[o.a].channels;
                op.c_b = o.b >= 0 ? ((use_pad && b_is_in) ? Cp : m.tensors[o.b].channels) : 0;
                op.c_out = n.c_out;
                op.level = m.tensors[n.out].level;
                op.out = out_t;
                op.pad_a = use_pad && a_is_in;
                op.pad_b = use_pad && b_is_in;
                op.name = o.b >= 0 ? "concat-conv" : "direct-conv";
                if (o.up) {
                  op.flags |= DNXCU_F_UP2X_A;
                  op.name = "up" + op.name;
                }
                if (act.node >= 0) {
                  if (m.nodes[act.node].kind == DNXCU_NODE_RELU) {
                    op.flags |= DNXCU_F_RELU;
                    op.name += "+relu";
                  } else {
                    op.flags |= DNXCU_F_LEAKY;
                    op.alpha = m.nodes[act.node].alpha;
                    op.name += "+leaky";
                  }
                }
                if (n.has_bias) op.flags |= DNXCU_F_BIAS;
                std::vector<int> src, dst;
                src.push_back(op.in_a);
                if (op.in_b >= 0) src.push_back(op.in_b);
                if (with_pool) {
                  op.flags |= DNXCU_F_POOL_OUT;
                  op.out_pool = m.nodes[pool_node].out;
                  op.name += "+pool";
                  if (sole(out_t, pool_node)) {
                    op.flags |= DNXCU_F_NO_FULL_OUT;
                    dst.push_back(op.out_pool);
                  } else {
                    dst.push_back(out_t);
                    dst.push_back(op.out_pool);
                  }
                } else {
                  dst.push_back(out_t);
                }
                add(op, src, dst);
              }
            }
          }
        break;
      }
      default: return DNXCU_E_BAD_ARG;
    }
  }
  if (pad_in) {
    FusedOp pad;
    pad.op = DNXCU_OP_PAD_CHANNELS;
    pad.in_a = m.input_tensor;
    pad.out = padded;
    pad.c_a = m.input_channels;
    pad.c_out = Cp;
    pad.level = 0;
    pad.src_node = 0;
    pad.name = "copy-transform(pad)";
    const size_t before = g.edges.size();
    add(pad, {m.input_tensor}, {padded});
    // a layout change of the input, not an operation of the model: it does not count as a dispatch when the
    // topologies are compared by dispatch count, so reading the input raw or through the copy is decided by cost
    for (size_t e = before; e < g.edges.size(); ++e) g.edges[e].dispatches = 0;
  }
  return DNXCU_OK;
}

// The conv's weights for the op's operand layout: the model's KCRS weights, with zero weights for the channels
// a padded copy of the network input adds.
void fill_parameters(const dnxcu_model &m, FusedOp &op) {
  if (op.op != DNXCU_OP_CONV3X3) return;
  const NodeRec &n = m.nodes[op.src_node];
  const int ca_real = op.pad_a ? m.input_channels : op.c_a;
  const int cb_real = op.pad_b ? m.input_channels : op.c_b;
  const int Cold = ca_real + cb_real, Cnew = op.c_a + op.c_b;
  if (Cold == Cnew) {
    op.weights_kcrs = n.weights;
  } else {
    op.weights_kcrs.assign((size_t)op.c_out * Cnew * 9, 0);
    for (int k = 0; k < op.c_out; ++k)
      for (int c = 0; c < Cold; ++c) {
        const int cn = c < ca_real ? c : op.c_a + (c - ca_real);
        for (int t = 0; t < 9; ++t)
          op.weights_kcrs[((size_t)k * Cnew + cn) * 9 + t] = n.weights[((size_t)k * Cold + c) * 9 + t];
      }
  }
  if (n.has_bias) op.bias = n.bias;
}

int select_schedule(const dnxcu_model &m, const dnxcu_db *db, bool allow_tc, int H, int W, std::vector<FusedOp> &ops,
                    std::vector<TensorInfo> &tensors, std::vector<int> &variants, double *total_ms) {
  HyperGraph g;
  std::vector<Candidate> cands;
  int st = build_supergraph(m, allow_tc, H, W, g, cands);
  if (st) return st;
  const std::vector<int> inputs = {m.input_tensor}, outputs = {m.output_tensor};
  // only topologies with the fewest dispatches are candidates, unless the model asks for cost alone to decide
  if (!(m.options & DNXCU_OPT_SELECT_BY_COST_ONLY) && !prune_topological(g, inputs, outputs)) return DNXCU_E_UNSUPPORTED;
  for (HyperEdge &e : g.edges) {
    const Candidate &c = cands[e.payload];
    const dnxcu_dispatch d = probe_dispatch(c.op, H, W, c.variant);
    double ms = 0;
    int ns = 0;
    if (db && dnxcu_db_query(db, &d, &ms, nullptr, &ns) == DNXCU_OK && ns > 0 && ms > 0) e.weight = ms;
    else e.weight = kUnbenchmarkedMs + 1e-3 * variant_rank(c.variant);  // selection.cpp:21,116; ties by preference
  }
  prune_duplicate_edges(g);
  std::vector<int> chosen;
  double cost = 0;
  if (!minimum_cost_subgraph(g, inputs, outputs, chosen, &cost)) return DNXCU_E_UNSUPPORTED;
  if (total_ms) *total_ms = cost;
  ops.clear();
  variants.clear();
  tensors.assign(m.tensors.begin(), m.tensors.begin() + m.n_model_tensors);
  {
    TensorInfo padded;  // the zero padded copy of a ragged input: the entry behind the model's own tensors
    padded.channels = (m.input_channels + 15) / 16 * 16;
    padded.level = 0;
    tensors.push_back(padded);
  }
  for (TensorInfo &t : tensors) t.materialized = false;
  tensors[m.input_tensor].materialized = true;
  for (int e : chosen) {
    const Candidate &c = cands[g.edges[e].payload];
    FusedOp op = c.op;
    fill_parameters(m, op);
    if (!(op.flags & DNXCU_F_NO_FULL_OUT)) tensors[op.out].materialized = true;
    if (op.out_pool >= 0) tensors[op.out_pool].materialized = true;
    ops.push_back(std::move(op));
    variants.push_back(c.variant);
  }
  return DNXCU_OK;
}

}  // namespace dnxcu
