// ONNX import for the subset of operators this backend runs: Conv (3x3, stride 1, size preserving), Relu,
// LeakyRelu, MaxPool (2x2, stride 2), Resize (nearest, x2), Concat (two inputs, channel axis).  Stands in for the
// reference's front end (compiler/src/denox/compiler/frontend/onnx/onnx.cpp:32-160 and details/ops/conv.cpp:9-306,
// max_pool.cpp:18-67, resize.cpp:24-136, concat.cpp:43-73, relu.cpp, leaky_relu.cpp:9-44) and keeps its
// acceptance rules: group = 1, dilation 1, symmetric padding (or SAME_*) that preserves the extent; MaxPool
// without auto_pad, ceil_mode or an indices output; Resize with mode nearest, asymmetric coordinates and constant
// integer scales that leave N and C alone; Concat of exactly two runtime tensors on the channel axis; weights
// arrive OIHW (conv.cpp:211-219), fp32 weights become binary16 by the reference's truncating conversion
// (common/src/denox/memory/dtype/f16.cpp:6-20).
//
// The reference parses with libprotobuf and generated classes; neither exists here, so this file reads the
// protobuf wire format directly (varints, length delimited fields) against the field numbers of onnx.proto.
#include "runtime.h"
#include <string.h>
#include <map>
#include <memory>
#include <string>

namespace dnxcu {

static thread_local std::string g_error_text;
void set_error_text(const std::string &s) { g_error_text = s; }
const char *error_text() { return g_error_text.c_str(); }

namespace {

struct Span {
  const uint8_t *p = nullptr;
  size_t n = 0;
  std::string str() const { return std::string((const char *)p, n); }
};

// One pass over the fields of a protobuf message.
struct Pb {
  const uint8_t *p, *end;
  bool bad = false;
  explicit Pb(Span s) : p(s.p), end(s.p + s.n) {}
  bool varint(uint64_t *v) {
    uint64_t x = 0;
    for (int shift = 0; shift < 64 && p < end; shift += 7) {
      const uint8_t b = *p++;
      x |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) {
        *v = x;
        return true;
      }
    }
    bad = true;
    return false;
  }
  // next field: number, wire type; value in `v` (varint / fixed) or `s` (length delimited)
  bool next(uint32_t *field, uint32_t *wire, uint64_t *v, Span *s) {
    if (p >= end || bad) return false;
    uint64_t tag;
    if (!varint(&tag)) return false;
    *field = (uint32_t)(tag >> 3);
    *wire = (uint32_t)(tag & 7);
    switch (*wire) {
      case 0: return varint(v);
      case 1:
        if (end - p < 8) return bad = true, false;
        memcpy(v, p, 8);
        p += 8;
        return true;
      case 5: {
        if (end - p < 4) return bad = true, false;
        uint32_t x;
        memcpy(&x, p, 4);
        *v = x;
        p += 4;
        return true;
      }
      case 2: {
        uint64_t len;
        if (!varint(&len) || len > (uint64_t)(end - p)) return bad = true, false;
        s->p = p;
        s->n = (size_t)len;
        p += len;
        return true;
      }
      default: return bad = true, false;
    }
  }
};

struct Tensor {  // TensorProto
  std::vector<int64_t> dims;
  int data_type = 0;
  Span raw;
  std::vector<float> floats;
  std::vector<int32_t> int32s;
  std::vector<int64_t> int64s;
  std::string name;
  bool external = false;
};

void packed_or_single(uint32_t wire, uint64_t v, Span s, int width, std::vector<uint64_t> &out) {
  if (wire == 2) {
    if (width == 0) {  // packed varints
      Pb q(s);
      uint64_t x;
      while (q.p < q.end && q.varint(&x)) out.push_back(x);
    } else {
      for (size_t i = 0; i + width <= s.n; i += width) {
        uint64_t x = 0;
        memcpy(&x, s.p + i, width);
        out.push_back(x);
      }
    }
  } else {
    out.push_back(v);
  }
}

bool parse_tensor(Span s, Tensor &t) {
  Pb pb(s);
  uint32_t f = 0, w = 0;
  uint64_t v = 0;
  Span sp;
  while (pb.next(&f, &w, &v, &sp)) {
    std::vector<uint64_t> tmp;
    switch (f) {
      case 1:
        packed_or_single(w, v, sp, 0, tmp);
        for (uint64_t x : tmp) t.dims.push_back((int64_t)x);
        break;
      case 2: t.data_type = (int)v; break;
      case 4:
        packed_or_single(w, v, sp, 4, tmp);
        for (uint64_t x : tmp) {
          float fl;
          const uint32_t b = (uint32_t)x;
          memcpy(&fl, &b, 4);
          t.floats.push_back(fl);
        }
        break;
      case 5:
        packed_or_single(w, v, sp, 0, tmp);
        for (uint64_t x : tmp) t.int32s.push_back((int32_t)x);
        break;
      case 7:
        packed_or_single(w, v, sp, 0, tmp);
        for (uint64_t x : tmp) t.int64s.push_back((int64_t)x);
        break;
      case 8: t.name = sp.str(); break;
      case 9: t.raw = sp; break;
      case 13: t.external = true; break;
      case 14: t.external = t.external || v == 1; break;
      default: break;
    }
  }
  return !pb.bad;
}

int64_t numel(const Tensor &t) {
  int64_t n = 1;
  for (int64_t d : t.dims) n *= d;
  return n;
}

// The tensor's values as float (FLOAT, FLOAT16, INT64, INT32).
bool tensor_floats(const Tensor &t, std::vector<float> &out) {
  const int64_t n = numel(t);
  out.clear();
  if (n < 0 || n > (1 << 28) || t.external) return false;
  switch (t.data_type) {
    case 1:  // FLOAT
      if (t.raw.n == (size_t)n * 4) {
        out.resize(n);
        memcpy(out.data(), t.raw.p, t.raw.n);
      } else if ((int64_t)t.floats.size() == n) {
        out = t.floats;
      } else {
        return false;
      }
      return true;
    case 10:  // FLOAT16: raw bytes, or one value per int32
      out.resize(n);
      if (t.raw.n == (size_t)n * 2) {
        for (int64_t i = 0; i < n; ++i) {
          uint16_t h;
          memcpy(&h, t.raw.p + 2 * i, 2);
          out[i] = dnxcu_f16_to_float(h);
        }
      } else if ((int64_t)t.int32s.size() == n) {
        for (int64_t i = 0; i < n; ++i) out[i] = dnxcu_f16_to_float((uint16_t)t.int32s[i]);
      } else {
        return false;
      }
      return true;
    case 7:  // INT64
      out.resize(n);
      if (t.raw.n == (size_t)n * 8) {
        for (int64_t i = 0; i < n; ++i) {
          int64_t x;
          memcpy(&x, t.raw.p + 8 * i, 8);
          out[i] = (float)x;
        }
      } else if ((int64_t)t.int64s.size() == n) {
        for (int64_t i = 0; i < n; ++i) out[i] = (float)t.int64s[i];
      } else {
        return false;
      }
      return true;
    default: return false;
  }
}

// Binary16 bits of the tensor: FLOAT16 as it is, FLOAT through the reference's truncating conversion.
bool tensor_halves(const Tensor &t, std::vector<uint16_t> &out) {
  const int64_t n = numel(t);
  if (t.data_type == 10 && t.raw.n == (size_t)n * 2 && !t.external) {
    out.resize(n);
    memcpy(out.data(), t.raw.p, t.raw.n);
    return true;
  }
  std::vector<float> f;
  if (!tensor_floats(t, f)) return false;
  out.resize(f.size());
  for (size_t i = 0; i < f.size(); ++i)
    out[i] = t.data_type == 10 ? (uint16_t)t.int32s[i] : dnxcu_f16_from_float(f[i]);
  return true;
}

struct Attr {
  std::string name, s;
  int64_t i = 0;
  float f = 0;
  std::vector<int64_t> ints;
  std::vector<float> floats;
  Tensor t;
  bool has_t = false;
};

bool parse_attr(Span s, Attr &a) {
  Pb pb(s);
  uint32_t f = 0, w = 0;
  uint64_t v = 0;
  Span sp;
  while (pb.next(&f, &w, &v, &sp)) {
    std::vector<uint64_t> tmp;
    switch (f) {
      case 1: a.name = sp.str(); break;
      case 2: {
        const uint32_t b = (uint32_t)v;
        memcpy(&a.f, &b, 4);
        break;
      }
      case 3: a.i = (int64_t)v; break;
      case 4: a.s = sp.str(); break;
      case 5: a.has_t = parse_tensor(sp, a.t); break;
      case 7:
        packed_or_single(w, v, sp, 4, tmp);
        for (uint64_t x : tmp) {
          float fl;
          const uint32_t b = (uint32_t)x;
          memcpy(&fl, &b, 4);
          a.floats.push_back(fl);
        }
        break;
      case 8:
        packed_or_single(w, v, sp, 0, tmp);
        for (uint64_t x : tmp) a.ints.push_back((int64_t)x);
        break;
      default: break;
    }
  }
  return !pb.bad;
}

struct Node {
  std::vector<std::string> in, out;
  std::string op, name, domain;
  std::vector<Attr> attrs;
  const Attr *attr(const char *n) const {
    for (const Attr &a : attrs)
      if (a.name == n) return &a;
    return nullptr;
  }
};

bool parse_node(Span s, Node &nd) {
  Pb pb(s);
  uint32_t f = 0, w = 0;
  uint64_t v = 0;
  Span sp;
  while (pb.next(&f, &w, &v, &sp)) {
    switch (f) {
      case 1: nd.in.push_back(sp.str()); break;
      case 2: nd.out.push_back(sp.str()); break;
      case 3: nd.name = sp.str(); break;
      case 4: nd.op = sp.str(); break;
      case 7: nd.domain = sp.str(); break;
      case 5: {
        Attr a;
        if (!parse_attr(sp, a)) return false;
        nd.attrs.push_back(std::move(a));
        break;
      }
      default: break;
    }
  }
  return !pb.bad;
}

// ValueInfoProto: name and, when the type is a tensor with a shape, the channel dimension (dim 1 of NCHW).
bool parse_value_info(Span s, std::string &name, int64_t *channels) {
  Pb pb(s);
  uint32_t f = 0, w = 0;
  uint64_t v = 0;
  Span sp;
  *channels = -1;
  while (pb.next(&f, &w, &v, &sp)) {
    if (f == 1) name = sp.str();
    if (f == 2) {  // TypeProto
      Pb ty(sp);
      Span tsp;
      while (ty.next(&f, &w, &v, &tsp))
        if (f == 1) {  // tensor_type
          Pb tt(tsp);
          Span shp;
          while (tt.next(&f, &w, &v, &shp))
            if (f == 2) {  // shape
              Pb sh(shp);
              Span dim;
              int idx = 0;
              while (sh.next(&f, &w, &v, &dim))
                if (f == 1) {
                  Pb d(dim);
                  Span dummy;
                  uint32_t df = 0, dw = 0;
                  uint64_t dv = 0;
                  while (d.next(&df, &dw, &dv, &dummy))
                    if (df == 1 && idx == 1) *channels = (int64_t)dv;
                  ++idx;
                }
            }
        }
    }
  }
  return !pb.bad;
}

int fail(const std::string &what) {
  set_error_text("ONNX import: " + what);
  return DNXCU_E_UNSUPPORTED;
}

}  // namespace

int import_onnx(const void *bytes, size_t n, uint32_t options, dnxcu_model &m, bool allow_tc) {
  set_error_text("");
  if (!bytes || n == 0) return DNXCU_E_BAD_ARG;
  Span graph;
  bool have_graph = false, have_opset = false, functions = false;
  {
    Pb pb(Span{(const uint8_t *)bytes, n});
    uint32_t f = 0, w = 0;
    uint64_t v = 0;
    Span sp;
    while (pb.next(&f, &w, &v, &sp)) {
      if (f == 7 && w == 2) {
        graph = sp;
        have_graph = true;
      }
      if (f == 8 && w == 2) {
        // OperatorSetIdProto: only the default domain (ai.onnx) is accepted (onnx.cpp:139-147)
        Pb os(sp);
        Span dom;
        std::string domain;
        uint32_t of = 0, ow = 0;
        uint64_t ov = 0;
        while (os.next(&of, &ow, &ov, &dom))
          if (of == 1) domain = dom.str();
        if (!domain.empty() && domain != "ai.onnx") return fail("unsupported operator set domain \"" + domain + "\"");
        have_opset = true;
      }
      if (f == 25) functions = true;
    }
    if (pb.bad) return fail("not a protobuf message");
  }
  if (functions) return fail("ONNX functions are not supported");
  if (!have_opset) return fail("missing opset_import");
  if (!have_graph) return fail("missing top-level graph");

  std::map<std::string, Tensor> inits;
  std::vector<Node> nodes;
  std::vector<std::pair<std::string, int64_t>> g_inputs, g_outputs;
  {
    Pb pb(graph);
    uint32_t f = 0, w = 0;
    uint64_t v = 0;
    Span sp;
    while (pb.next(&f, &w, &v, &sp)) {
      if (f == 1) {
        Node nd;
        if (!parse_node(sp, nd)) return fail("malformed node");
        nodes.push_back(std::move(nd));
      } else if (f == 5) {
        Tensor t;
        if (!parse_tensor(sp, t)) return fail("malformed initializer");
        if (t.external) return fail("initializer \"" + t.name + "\" uses external data");
        inits[t.name] = std::move(t);
      } else if (f == 15) {
        return fail("sparse initializers are not supported");
      } else if (f == 11 || f == 12) {
        std::string name;
        int64_t ch;
        if (!parse_value_info(sp, name, &ch)) return fail("malformed value info");
        (f == 11 ? g_inputs : g_outputs).push_back(std::make_pair(name, ch));
      }
    }
    if (pb.bad) return fail("malformed graph");
  }
  // runtime inputs: graph inputs that are not initializers (onnx.cpp:44-50)
  std::vector<std::pair<std::string, int64_t>> rt_in;
  for (auto &gi : g_inputs)
    if (!inits.count(gi.first)) rt_in.push_back(gi);
  if (rt_in.size() != 1 || g_outputs.size() != 1) return fail("exactly one runtime input and one output are supported");
  if (rt_in[0].second <= 0) return fail("the input's channel count must be a constant");

  // constants produced by Constant nodes (torch exports Resize scales this way)
  std::map<std::string, Tensor> consts;
  std::map<std::string, int> tid;   // runtime tensor name -> id
  std::vector<int> channels;
  std::vector<std::vector<uint16_t>> weight_store, bias_store;
  std::vector<dnxcu_node> out_nodes;
  tid[rt_in[0].first] = 0;
  channels.push_back((int)rt_in[0].second);
  auto new_tensor = [&](const std::string &name, int c) {
    tid[name] = (int)channels.size();
    channels.push_back(c);
    return (int)channels.size() - 1;
  };
  auto runtime = [&](const std::string &name) -> int {
    auto it = tid.find(name);
    return it == tid.end() ? -1 : it->second;
  };
  auto constant = [&](const std::string &name) -> const Tensor * {
    auto a = inits.find(name);
    if (a != inits.end()) return &a->second;
    auto b = consts.find(name);
    return b == consts.end() ? nullptr : &b->second;
  };
  for (const Node &nd : nodes) {
    const std::string where = "node \"" + (nd.name.empty() ? nd.op : nd.name) + "\": ";
    if (!nd.domain.empty() && nd.domain != "ai.onnx") return fail(where + "operator domain \"" + nd.domain + "\"");
    if (nd.op == "Constant") {
      const Attr *a = nd.attr("value");
      if (!a || !a->has_t || nd.out.size() != 1) return fail(where + "only tensor valued constants are supported");
      consts[nd.out[0]] = a->t;
      continue;
    }
    if (nd.op == "Identity" && nd.in.size() == 1 && nd.out.size() == 1) {
      if (const Tensor *c = constant(nd.in[0])) {
        consts[nd.out[0]] = *c;
        continue;
      }
      const int t = runtime(nd.in[0]);
      if (t < 0) return fail(where + "unknown input");
      tid[nd.out[0]] = t;
      continue;
    }
    dnxcu_node o;
    memset(&o, 0, sizeof(o));
    o.in1 = -1;
    if (nd.op == "Conv") {
      if (nd.in.size() < 2 || nd.in.size() > 3 || nd.out.size() != 1) return fail(where + "expects 2 or 3 inputs and 1 output");
      const int x = runtime(nd.in[0]);
      const Tensor *wt = constant(nd.in[1]);
      if (x < 0 || !wt) return fail(where + "needs a runtime input and constant weights");
      if (wt->dims.size() != 4) return fail(where + "weights must be OIHW");
      const int64_t K = wt->dims[0], C = wt->dims[1], R = wt->dims[2], S = wt->dims[3];
      const Attr *a;
      if ((a = nd.attr("group")) && a->i != 1) return fail(where + "group must be 1");
      if ((a = nd.attr("dilations")))
        for (int64_t d : a->ints)
          if (d != 1) return fail(where + "dilation must be 1");
      if ((a = nd.attr("strides")))
        for (int64_t d : a->ints)
          if (d != 1) return fail(where + "stride must be 1");
      if (R != 3 || S != 3) return fail(where + "only 3x3 kernels run on this backend");
      if ((a = nd.attr("kernel_shape")) && (a->ints.size() != 2 || a->ints[0] != 3 || a->ints[1] != 3))
        return fail(where + "kernel_shape does not match the weights");
      const Attr *ap = nd.attr("auto_pad"), *pads = nd.attr("pads");
      const std::string mode = ap ? ap->s : "NOTSET";
      if (mode == "NOTSET") {
        if (!pads || pads->ints.size() != 4) return fail(where + "padding must keep the extent (pads = 1)");
        for (int64_t p : pads->ints)
          if (p != 1) return fail(where + "padding must keep the extent (pads = 1)");
      } else if (mode != "SAME_UPPER" && mode != "SAME_LOWER") {
        return fail(where + "auto_pad " + mode + " does not keep the extent");
      }
      if (C != channels[x]) return fail(where + "weight channels do not match the input");
      weight_store.emplace_back();
      if (!tensor_halves(*wt, weight_store.back()) || (int64_t)weight_store.back().size() != K * C * 9)
        return fail(where + "weights must be float or float16 constants");
      o.kind = DNXCU_NODE_CONV;
      o.in0 = x;
      o.c_out = (int)K;
      o.weights_kcrs = weight_store.back().data();
      if (nd.in.size() == 3 && !nd.in[2].empty()) {
        const Tensor *bt = constant(nd.in[2]);
        bias_store.emplace_back();
        if (!bt || !tensor_halves(*bt, bias_store.back()) || (int64_t)bias_store.back().size() != K)
          return fail(where + "bias must be a constant of one value per output channel");
        o.bias = bias_store.back().data();
      }
      o.out = new_tensor(nd.out[0], (int)K);
    } else if (nd.op == "Relu" || nd.op == "LeakyRelu") {
      if (nd.in.size() != 1 || nd.out.size() != 1) return fail(where + "expects exactly 1 input and 1 output");
      const int x = runtime(nd.in[0]);
      if (x < 0) return fail(where + "only runtime tensors are supported");
      o.kind = nd.op == "Relu" ? DNXCU_NODE_RELU : DNXCU_NODE_LEAKY_RELU;
      o.in0 = x;
      if (nd.op == "LeakyRelu") {
        const Attr *a = nd.attr("alpha");
        o.alpha = a ? a->f : 0.01f;  // the operator's default slope
      }
      o.out = new_tensor(nd.out[0], channels[x]);
    } else if (nd.op == "MaxPool") {
      if (nd.in.size() != 1) return fail(where + "expects exactly 1 input");
      if (nd.out.size() != 1) return fail(where + "the indices output is not supported");
      const int x = runtime(nd.in[0]);
      if (x < 0) return fail(where + "only runtime tensors are supported");
      const Attr *a;
      if ((a = nd.attr("auto_pad")) && a->s != "NOTSET") return fail(where + "auto_pad is not supported");
      if ((a = nd.attr("ceil_mode")) && a->i != 0) return fail(where + "ceil_mode is not supported");
      a = nd.attr("kernel_shape");
      if (!a || a->ints.size() != 2 || a->ints[0] != 2 || a->ints[1] != 2) return fail(where + "only 2x2 windows run on this backend");
      a = nd.attr("strides");
      if (!a || a->ints.size() != 2 || a->ints[0] != 2 || a->ints[1] != 2) return fail(where + "stride must be 2");
      if ((a = nd.attr("pads")))
        for (int64_t p : a->ints)
          if (p != 0) return fail(where + "padding is not supported");
      if ((a = nd.attr("dilations")))
        for (int64_t d : a->ints)
          if (d != 1) return fail(where + "dilation must be 1");
      o.kind = DNXCU_NODE_MAXPOOL;
      o.in0 = x;
      o.out = new_tensor(nd.out[0], channels[x]);
    } else if (nd.op == "Resize" || nd.op == "Upsample") {
      if (nd.in.empty() || nd.out.size() != 1) return fail(where + "expects an input and 1 output");
      const int x = runtime(nd.in[0]);
      if (x < 0) return fail(where + "only runtime tensors are supported");
      const Attr *a;
      if ((a = nd.attr("mode")) && a->s != "nearest") return fail(where + "mode must be nearest");
      if ((a = nd.attr("coordinate_transformation_mode")) && a->s != "asymmetric")
        return fail(where + "coordinate_transformation_mode must be asymmetric");
      // scales: input 2 of Resize (opset >= 11), input 1 of Upsample / Resize-10
      const Tensor *sc = nullptr;
      for (size_t k = 1; k < nd.in.size() && !sc; ++k)
        if (!nd.in[k].empty()) {
          const Tensor *c = constant(nd.in[k]);
          if (c && numel(*c) == 4 && c->data_type == 1) sc = c;
        }
      std::vector<float> scales;
      if (!sc || !tensor_floats(*sc, scales) || scales.size() != 4) return fail(where + "scales must be a constant of 4 floats");
      if (scales[0] != 1.0f || scales[1] != 1.0f) return fail(where + "N and C must not be scaled");
      if (scales[2] != 2.0f || scales[3] != 2.0f) return fail(where + "only a 2x upsample runs on this backend");
      o.kind = DNXCU_NODE_UPSAMPLE;
      o.in0 = x;
      o.out = new_tensor(nd.out[0], channels[x]);
    } else if (nd.op == "Concat") {
      if (nd.in.size() != 2 || nd.out.size() != 1) return fail(where + "expects exactly 2 inputs and 1 output");
      const Attr *a = nd.attr("axis");
      if (!a || (a->i != 1 && a->i != -3)) return fail(where + "only the channel axis is supported");
      const int x = runtime(nd.in[0]), y = runtime(nd.in[1]);
      if (x < 0 || y < 0) return fail(where + "only runtime tensors are supported");
      o.kind = DNXCU_NODE_CONCAT;
      o.in0 = x;
      o.in1 = y;
      o.out = new_tensor(nd.out[0], channels[x] + channels[y]);
    } else {
      return fail(where + "operator " + nd.op + " is not supported");
    }
    out_nodes.push_back(o);
  }
  const int out_t = runtime(g_outputs[0].first);
  if (out_t < 0 || out_nodes.empty()) return fail("the graph output is not produced by a supported node");
  dnxcu_model_desc desc;
  memset(&desc, 0, sizeof(desc));
  desc.n_nodes = (int)out_nodes.size();
  desc.n_tensors = (int)channels.size();
  desc.nodes = out_nodes.data();
  desc.input_tensor = 0;
  desc.input_channels = channels[0];
  desc.output_tensor = out_t;
  desc.options = options;
  const int st = build_fused_ops(desc, allow_tc, m);
  if (st) set_error_text("ONNX import: the graph is not a valid model for this backend");
  return st;
}

}  // namespace dnxcu
