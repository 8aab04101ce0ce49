// Model (fused dispatch list) and instance (buffers + chosen variants) of the runtime.
#pragma once
#include "internal.h"
#include <string>
#include <vector>

namespace dnxcu {

struct TensorInfo {
  int channels = 0;
  int level = 0;  // resolution = image >> level
  bool materialized = false;
};

// One dispatch after fusion, before a variant is chosen.
struct FusedOp {
  int op = 0;  // dnxcu_op
  uint32_t flags = 0;
  int in_a = -1, in_b = -1, out = -1, out_pool = -1;  // tensor ids
  int c_a = 0, c_b = 0, c_out = 0;
  int level = 0;  // resolution level of the push constants
  int src_node = -1;
  float alpha = 0.0f;                  // slope of a (fused or standalone) LeakyReLU
  bool pad_a = false, pad_b = false;   // the operand is the zero padded copy of the ragged network input
  std::vector<unsigned char> prepared; // conv of a model read from a dnx file: the weights in the variant's layout
  std::vector<uint16_t> weights_kcrs;  // conv
  std::vector<uint16_t> bias;          // conv, may be empty
  std::string name;
};

// One node of the model as it was handed in (the un-fused graph an ONNX import yields), parameters included.
struct NodeRec {
  int kind = 0, in0 = -1, in1 = -1, out = -1, c_out = 0;
  float alpha = 0.0f;
  bool has_bias = false;
  std::vector<uint16_t> weights;  // conv: KCRS binary16
  std::vector<uint16_t> bias;
};

// A hyperedge's payload in the graph of candidate dispatches: the dispatch (without parameters) and its variant.
struct Candidate {
  FusedOp op;
  int variant = -1;
};

}  // namespace dnxcu

struct dnxcu_model {
  std::vector<dnxcu::TensorInfo> tensors;  // the model's tensors, then (if the default schedule uses it) the padded input
  int n_model_tensors = 0;
  std::vector<dnxcu::NodeRec> nodes;
  std::vector<dnxcu::FusedOp> ops;         // the default schedule: every fusion pattern that applies
  bool from_dnx = false;                   // read from a dnx file: `ops` is the file's schedule, variants fixed
  std::vector<int> dnx_variants;
  int dnx_align = 1;
  int input_tensor = -1, output_tensor = -1, input_channels = 0;
  uint32_t options = 0;
  int device = 0;
  const dnxcu_db *db = nullptr;
};

namespace dnxcu {
// Runs the fusion patterns over the node list.  Shared by model creation and
// by the database's populate step.
int build_fused_ops(const dnxcu_model_desc &desc, bool allow_tc, dnxcu_model &m);
// Candidate variants for a fused op in preference order.
void candidate_variants(const FusedOp &op, bool allow_tc, std::vector<int> &out);
// Position of a variant in that preference order (large for variants outside it).
int variant_rank(int variant);
}  // namespace dnxcu

namespace dnxcu {
struct HyperGraph;
// Every way to compute the model's tensors at extent H x W as hyperedges (supergraph.cu).
int build_supergraph(const dnxcu_model &m, bool allow_tc, int H, int W, HyperGraph &g, std::vector<Candidate> &cands);
// Cost driven schedule: dispatch list, tensor table (with what is materialised) and variant per dispatch.
int select_schedule(const dnxcu_model &m, const dnxcu_db *db, bool allow_tc, int H, int W, std::vector<FusedOp> &ops,
                    std::vector<TensorInfo> &tensors, std::vector<int> &variants, double *total_ms);
// Validation probe of an op at an extent (placeholder pointers).
dnxcu_dispatch probe_dispatch(const FusedOp &op, int H, int W, int variant);
// dnx container (dnx.cu): a schedule with its variants and parameters -> bytes, and back.
int write_dnx(const dnxcu_model &m, const std::vector<FusedOp> &ops, const std::vector<TensorInfo> &tensors,
              const std::vector<int> &variants, int align, std::vector<uint8_t> &out);
int read_dnx(const void *bytes, size_t n, dnxcu_model &m, int *align_out);
// ONNX subset import (onnx.cu): fills the model like dnxcu_model_create does from a node list.
int import_onnx(const void *bytes, size_t n, uint32_t options, dnxcu_model &m, bool allow_tc);
// Text of the last import failure on this thread.
void set_error_text(const std::string &s);
const char *error_text();
}  // namespace dnxcu
