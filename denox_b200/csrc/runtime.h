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
  std::vector<uint16_t> weights_kcrs;  // conv
  std::vector<uint16_t> bias;          // conv, may be empty
  std::string name;
};

}  // namespace dnxcu

struct dnxcu_model {
  std::vector<dnxcu::TensorInfo> tensors;
  std::vector<dnxcu::FusedOp> ops;
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
}  // namespace dnxcu
