// dnx files: the compiled-model container of denox (dnx.fbs:1-195), written and read without the FlatBuffers
// library (flatbuf.h).  The writer plays the role of the reference's serialize step
// (compiler/src/denox/compiler/serialize/serialize.cpp:1-635): tensors with symbolic extents, one buffer per
// tensor, parameter tensors with initializers (weights already in the chosen variant's layout, as the reference
// stores its re-laid filters), one ComputeDispatch per kernel launch with its descriptor bindings in the order
// inputs, outputs, parameters, push constants {IN_W, IN_H}, symbolic work group count, and the symbolic
// expression list (SymIR, common/src/denox/symbolic/SymIR.hpp:10-70) over the two variables H and W.  The reader
// plays the role of runtime::Model::make (runtime/src/denox/runtime/model.cpp:80-245,392-659).
//
// What differs from a file the reference writes is the content of `shader_binaries`: where the reference stores
// SPIR-V words (first word 0x07230203), this backend stores a descriptor of the CUDA kernel variant and its
// specialisation (first word "DNXC"); `entry_point` is the variant family instead of "main".  A file whose
// binaries are SPIR-V cannot run here and is refused with DNXCU_E_UNSUPPORTED.
#include "runtime.h"
#include "flatbuf.h"
#include <string.h>
#include <map>
#include <new>

namespace dnxcu {
namespace {

constexpr uint32_t kBinaryMagic = 0x43584E44u;  // "DNXC"
constexpr uint32_t kSpirvMagic = 0x07230203u;
// dnx.fbs enums
enum { ST_U32 = 3, ST_U64 = 5, ST_F16 = 6 };
enum { SRC_NONE = 0, SRC_LITERAL = 1, SRC_SYMBOLIC = 2 };
enum { ACCESS_RO = 0, ACCESS_WO = 1 };
enum { FMT_UNKNOWN = 0, FMT_SSBO_HWC = 1 };
enum { OP_ADD = 1, OP_SUB = 2, OP_MUL = 3, OP_DIV = 4, OP_MOD = 5, OP_MIN = 6, OP_MAX = 7, OP_LHSC = 0x8000, OP_RHSC = 0x4000 };

#pragma pack(push, 1)
struct SymOpRaw {  // struct SymIROp of dnx.fbs: uint16 opcode, then two int64 at their natural alignment
  uint16_t opcode;
  uint8_t pad[6];
  int64_t lhs, rhs;
};
#pragma pack(pop)
static_assert(sizeof(SymOpRaw) == 24, "SymIROp is 24 bytes");

// ---- symbolic expressions over H (symbol 0) and W (symbol 1) --------------------------------------------------

struct Scalar {  // a ScalarSource: a literal or a symbol id
  bool symbolic = false;
  int64_t v = 0;
};
inline Scalar lit(int64_t v) { return Scalar{false, v}; }

struct SymBuilder {
  std::vector<SymOpRaw> ops;
  std::map<std::tuple<int, bool, int64_t, bool, int64_t>, int64_t> cache;
  static constexpr int kVars = 2;
  Scalar var(int i) const { return Scalar{true, i}; }
  Scalar emit(int opcode, Scalar a, Scalar b) {
    if (!a.symbolic && !b.symbolic) {
      switch (opcode) {
        case OP_ADD: return lit(a.v + b.v);
        case OP_SUB: return lit(a.v - b.v);
        case OP_MUL: return lit(a.v * b.v);
        case OP_DIV: return lit(b.v ? a.v / b.v : 0);
        default: return lit(0);
      }
    }
    const auto key = std::make_tuple(opcode, a.symbolic, a.v, b.symbolic, b.v);
    auto it = cache.find(key);
    if (it != cache.end()) return Scalar{true, it->second};
    SymOpRaw r;
    memset(&r, 0, sizeof(r));
    r.opcode = (uint16_t)(opcode | (a.symbolic ? 0 : OP_LHSC) | (b.symbolic ? 0 : OP_RHSC));
    r.lhs = a.v;
    r.rhs = b.v;
    ops.push_back(r);
    const int64_t sid = kVars + (int64_t)ops.size() - 1;
    cache[key] = sid;
    return Scalar{true, sid};
  }
  Scalar add(Scalar a, Scalar b) { return emit(OP_ADD, a, b); }
  Scalar mul(Scalar a, Scalar b) { return emit(OP_MUL, a, b); }
  Scalar div(Scalar a, Scalar b) { return emit(OP_DIV, a, b); }
};

void put_source(fb::Table &t, size_t type_slot, Scalar s, int dtype = ST_U64) {
  auto src = fb::make_table();
  if (s.symbolic) {
    src->scalar<uint32_t>(0, (uint32_t)s.v);  // SymRef.sid
    t.scalar<uint8_t>(type_slot, SRC_SYMBOLIC);
  } else {
    src->scalar<uint8_t>(0, (uint8_t)dtype);  // ScalarLiteral.dtype
    if (dtype == ST_U32) {
      const uint32_t v = (uint32_t)s.v;
      src->bytes(1, &v, 4);
    } else {
      const uint64_t v = (uint64_t)s.v;
      src->bytes(1, &v, 8);
    }
    t.scalar<uint8_t>(type_slot, SRC_LITERAL);
  }
  t.table(type_slot + 1, src);
}

// The stand-in for a shader binary: which kernel variant, specialised how.
std::vector<uint32_t> binary_blob(const Variant &v, const FusedOp &op) {
  std::vector<uint32_t> w;
  const std::string family = v.desc.family, config = v.desc.config;
  uint32_t alpha_bits;
  memcpy(&alpha_bits, &op.alpha, 4);
  w = {kBinaryMagic, 1u, (uint32_t)op.op, op.flags, (uint32_t)op.c_a, (uint32_t)op.c_b, (uint32_t)op.c_out, alpha_bits,
       (uint32_t)family.size(), (uint32_t)config.size()};
  auto put_str = [&](const std::string &s) {
    for (size_t i = 0; i < s.size(); i += 4) {
      uint32_t x = 0;
      memcpy(&x, s.data() + i, std::min<size_t>(4, s.size() - i));
      w.push_back(x);
    }
  };
  put_str(family);
  put_str(config);
  return w;
}

}  // namespace

int write_dnx(const dnxcu_model &m, const std::vector<FusedOp> &ops, const std::vector<TensorInfo> &tensors,
              const std::vector<int> &variants, int align, std::vector<uint8_t> &out) {
  if (ops.size() != variants.size()) return DNXCU_E_BAD_ARG;
  SymBuilder sym;
  const Scalar H = sym.var(0), W = sym.var(1);
  auto extent = [&](Scalar full, int level) { return level > 0 ? sym.div(full, lit(1ll << level)) : full; };

  // tensors: the activations the schedule materialises keep their ids' order; parameter tensors follow
  std::vector<int> dnx_id(tensors.size(), -1);
  std::vector<std::shared_ptr<fb::Table>> ftensors, fbuffers, finits, fdisp, fbins;
  auto add_tensor = [&](Scalar w, Scalar h, Scalar c, Scalar bytes, const std::string &name, int format) {
    auto info = fb::make_table();
    put_source(*info, 0, w, ST_U32);
    put_source(*info, 2, h, ST_U32);
    put_source(*info, 4, c, ST_U32);
    info->scalar<uint16_t>(6, (uint16_t)format);
    info->scalar<uint16_t>(7, 0);  // StorageBuffer
    info->scalar<uint8_t>(8, ST_F16);
    info->string(9, name);
    auto buf = fb::make_table();
    put_source(*buf, 0, bytes);
    buf->scalar<uint16_t>(2, 256);
    fbuffers.push_back(buf);
    auto t = fb::make_table();
    t->scalar<uint32_t>(0, (uint32_t)fbuffers.size() - 1);
    put_source(*t, 1, lit(0));
    put_source(*t, 3, bytes);
    t->table(5, info);
    ftensors.push_back(t);
    return (int)ftensors.size() - 1;
  };
  for (size_t t = 0; t < tensors.size(); ++t) {
    if (!tensors[t].materialized) continue;
    const Scalar w = extent(W, tensors[t].level), h = extent(H, tensors[t].level);
    const Scalar bytes = sym.mul(sym.mul(w, h), lit((int64_t)tensors[t].channels * 2));
    dnx_id[t] = add_tensor(w, h, lit(tensors[t].channels), bytes, "t" + std::to_string(ftensors.size()), FMT_SSBO_HWC);
  }
  if (dnx_id[m.input_tensor] < 0 || dnx_id[m.output_tensor] < 0) return DNXCU_E_STATE;

  bool any_tc = false;
  for (size_t i = 0; i < ops.size(); ++i) {
    const FusedOp &op = ops[i];
    const Variant *v = get_variant(variants[i]);
    if (!v || v->desc.op != op.op) return DNXCU_E_BAD_ARG;
    any_tc = any_tc || v->desc.needs_tcgen05;
    auto bin = fb::make_table();
    bin->vec<uint32_t>(0, binary_blob(*v, op));
    fbins.push_back(bin);

    std::vector<std::shared_ptr<fb::Table>> binds;
    auto bind = [&](int tensor, int access) {
      auto b = fb::make_table();
      b->scalar<uint16_t>(0, (uint16_t)binds.size());
      b->scalar<uint8_t>(1, (uint8_t)access);
      b->scalar<uint32_t>(2, (uint32_t)tensor);
      binds.push_back(b);
    };
    // inputs, outputs, parameters (the reference's binding order, ComputeDispatchBuilder.cpp:100-176)
    bind(dnx_id[op.in_a], ACCESS_RO);
    if (op.in_b >= 0) bind(dnx_id[op.in_b], ACCESS_RO);
    if (!(op.flags & DNXCU_F_NO_FULL_OUT)) bind(dnx_id[op.out], ACCESS_WO);
    if (op.out_pool >= 0) bind(dnx_id[op.out_pool], ACCESS_WO);
    if (op.op == DNXCU_OP_CONV3X3) {
      std::vector<unsigned char> blob = op.prepared;
      if (blob.empty()) {
        size_t bytes = 0;
        int st = dnxcu_prepare_weights(variants[i], nullptr, op.c_out, op.c_a, op.c_b, nullptr, &bytes);
        if (st) return st;
        blob.resize(bytes);
        st = dnxcu_prepare_weights(variants[i], op.weights_kcrs.data(), op.c_out, op.c_a, op.c_b, blob.data(), &bytes);
        if (st) return st;
      }
      const int wt = add_tensor(lit(0), lit(0), lit(0), lit((int64_t)blob.size()), "weights" + std::to_string(i), FMT_UNKNOWN);
      auto init = fb::make_table();
      init->scalar<uint32_t>(0, (uint32_t)wt);
      init->bytes(1, blob.data(), blob.size());
      finits.push_back(init);
      bind(wt, ACCESS_RO);
      if (op.flags & DNXCU_F_BIAS) {
        const int bt = add_tensor(lit(1), lit(1), lit(op.c_out), lit((int64_t)op.bias.size() * 2), "bias" + std::to_string(i), FMT_UNKNOWN);
        auto binit = fb::make_table();
        binit->scalar<uint32_t>(0, (uint32_t)bt);
        binit->bytes(1, op.bias.data(), op.bias.size() * 2);
        finits.push_back(binit);
        bind(bt, ACCESS_RO);
      }
    }
    auto set0 = fb::make_table();
    set0->scalar<uint16_t>(0, 0);
    set0->tables(1, binds);

    const Scalar pw = extent(W, op.level), ph = extent(H, op.level);
    auto pc = fb::make_table();
    pc->scalar<uint16_t>(0, 8);
    std::vector<std::shared_ptr<fb::Table>> fields;
    for (int f = 0; f < 2; ++f) {
      auto fld = fb::make_table();
      fld->scalar<uint8_t>(0, ST_U32);
      fld->scalar<uint16_t>(1, (uint16_t)(4 * f));
      put_source(*fld, 2, f ? ph : pw, ST_U32);  // IN_W at offset 0, IN_H at offset 4 (DirectConvShaderCM.cpp:628-630)
      fields.push_back(fld);
    }
    pc->tables(1, fields);

    // work units of the dispatch (strips of 128 pixels x pairs of rows for the convs, 2048 items otherwise); the
    // launcher sizes its persistent grid from these and the device's SM count
    const Scalar pix = sym.mul(pw, ph);
    const Scalar units = op.op == DNXCU_OP_CONV3X3
                             ? sym.mul(sym.div(sym.add(pw, lit(127)), lit(128)), sym.div(sym.add(ph, lit(1)), lit(2)))
                             : sym.div(sym.add(sym.mul(pix, lit(op.c_a > 0 ? op.c_a : 1)), lit(2047)), lit(2048));
    // algorithmic cost (dnxcu_cost's formulas with symbolic pixel counts)
    const int64_t C = (int64_t)op.c_a + op.c_b, K = op.c_out;
    Scalar rd = lit(0), wr = lit(0), fl = lit(0);
    if (op.op == DNXCU_OP_CONV3X3) {
      const Scalar pa = (op.flags & DNXCU_F_UP2X_A) ? sym.div(pix, lit(4)) : pix;
      rd = sym.add(sym.add(sym.mul(pa, lit(2ll * op.c_a)), sym.mul(pix, lit(2ll * op.c_b))), lit(18 * C * K));
      if (!(op.flags & DNXCU_F_NO_FULL_OUT)) wr = sym.mul(pix, lit(2 * K));
      if (op.flags & DNXCU_F_POOL_OUT) wr = sym.add(wr, sym.mul(sym.div(pix, lit(4)), lit(2 * K)));
      fl = sym.mul(pix, lit(18 * C * K));
    } else {
      rd = sym.mul(pix, lit(2ll * (op.c_a + op.c_b)));
      wr = op.op == DNXCU_OP_MAXPOOL2X2 ? sym.mul(sym.div(pix, lit(4)), lit(2ll * op.c_a))
           : op.op == DNXCU_OP_UPSAMPLE2X ? sym.mul(pix, lit(8ll * op.c_a))
           : op.op == DNXCU_OP_PAD_CHANNELS ? sym.mul(pix, lit(2ll * op.c_out))
                                            : rd;
    }
    auto info = fb::make_table();
    info->string(0, op.name);
    info->string(1, v->desc.config);
    info->string(2, std::string("dnxcu:") + v->desc.family);
    put_source(*info, 3, rd);
    put_source(*info, 5, wr);
    put_source(*info, 7, fl);

    auto disp = fb::make_table();
    disp->scalar<uint32_t>(0, (uint32_t)fbins.size() - 1);
    put_source(*disp, 1, units, ST_U32);
    put_source(*disp, 3, lit(1), ST_U32);
    put_source(*disp, 5, lit(1), ST_U32);
    disp->string(7, v->desc.family);
    disp->tables(8, {set0});
    disp->table(9, pc);
    disp->table(10, info);
    fdisp.push_back(disp);
  }

  auto model = fb::make_table();
  model->scalar<uint16_t>(0, 0);  // DNX_VERSION_1_0
  if (any_tc) model->vec<uint32_t>(1, std::vector<uint32_t>{0u});  // CooperativeMatrix: the tensor core variants
  auto minfo = fb::make_table();
  minfo->string(0, "dnxcu");
  char sha[65] = "";
  dnxcu_variant_sha256(0, sha);
  minfo->string(1, sha);
  minfo->string(2, "");
  model->table(2, minfo);
  model->tables(3, ftensors);
  model->tables(4, finits);
  model->vec<uint32_t>(5, std::vector<uint32_t>{(uint32_t)dnx_id[m.input_tensor]});
  model->vec<uint32_t>(6, std::vector<uint32_t>{(uint32_t)dnx_id[m.output_tensor]});
  model->tables(7, fbuffers);
  model->tables(8, fdisp);
  model->tables(9, fbins);
  auto symir = fb::make_table();
  symir->scalar<uint16_t>(0, (uint16_t)SymBuilder::kVars);
  symir->vec<SymOpRaw>(1, sym.ops, 8);
  model->table(10, symir);
  std::vector<std::shared_ptr<fb::Table>> names;
  auto name_of = [&](const char *n, Scalar s) {
    auto vn = fb::make_table();
    vn->string(0, n);
    put_source(*vn, 1, s);
    names.push_back(vn);
  };
  name_of("H", H);
  name_of("W", W);
  name_of("ALIGN", lit(align));
  model->tables(11, names);
  out = fb::finish(*model, "dnxx");
  return DNXCU_OK;
}

// ---- reader -------------------------------------------------------------------------------------------------

namespace {

struct SymEval {
  std::vector<int64_t> dp;
  bool ok = true;
  // SymIR::eval (common/src/denox/symbolic/SymIR.cpp:5-100)
  SymEval(const fb::View &symir, int64_t h, int64_t w) {
    const uint16_t vars = symir.scalar<uint16_t>(0);
    size_t n = 0;
    const size_t first = symir.vec(1, sizeof(SymOpRaw), &n);
    dp.assign(vars + n, 0);
    if (vars > 0) dp[0] = h;
    if (vars > 1) dp[1] = w;
    for (size_t pc = 0; pc < n; ++pc) {
      SymOpRaw r;
      memcpy(&r, symir.b.p + first + pc * sizeof(SymOpRaw), sizeof(r));
      const bool lc = r.opcode & OP_LHSC, rc = r.opcode & OP_RHSC;
      auto val = [&](bool is_const, int64_t x) -> int64_t {
        if (is_const) return x;
        if (x < 0 || (size_t)x >= vars + pc) {
          ok = false;
          return 0;
        }
        return dp[(size_t)x];
      };
      const int64_t a = val(lc, r.lhs), b = val(rc, r.rhs);
      int64_t v = 0;
      switch (r.opcode & 0x3fff) {
        case OP_ADD: v = a + b; break;
        case OP_SUB: v = a - b; break;
        case OP_MUL: v = a * b; break;
        case OP_DIV: v = b ? a / b : 0; break;
        case OP_MOD:
          v = b ? a % b : 0;
          if (v < 0) v += b;
          break;
        case OP_MIN: v = a < b ? a : b; break;
        case OP_MAX: v = a > b ? a : b; break;
        default: v = 0; break;
      }
      dp[vars + pc] = v;
    }
  }
  // value of the ScalarSource union at (type_slot, type_slot + 1) of `t`
  bool source(const fb::View &t, size_t type_slot, int64_t *out) const {
    const uint8_t kind = t.scalar<uint8_t>(type_slot);
    const fb::View src = t.table(type_slot + 1);
    if (!src.valid) return false;
    if (kind == SRC_SYMBOLIC) {
      const uint32_t sid = src.scalar<uint32_t>(0);
      if (sid >= dp.size()) return false;
      *out = dp[sid];
      return true;
    }
    if (kind == SRC_LITERAL) {
      size_t n = 0;
      const size_t p = src.vec(1, 1, &n);
      if (!p || n == 0 || n > 8) return false;
      uint64_t v = 0;
      memcpy(&v, src.b.p + p, n);
      *out = (int64_t)v;
      return true;
    }
    return false;
  }
};

int log2_exact(int64_t ratio) {
  int l = 0;
  while ((1ll << l) < ratio) ++l;
  return (1ll << l) == ratio ? l : -1;
}

}  // namespace

int read_dnx(const void *bytes, size_t n, dnxcu_model &m, int *align_out) {
  const fb::View model = fb::root(bytes, n, "dnxx");
  if (!model.valid) return DNXCU_E_BAD_ARG;
  const fb::View symir = model.table(10);
  if (!symir.valid) return DNXCU_E_BAD_ARG;
  // tensor extents are read off a probe evaluation: this backend's tensors are the frame extent shifted right
  // by a resolution level, which two evaluations at different extents pin down
  const int64_t PH = 1 << 12, PW = 1 << 13;
  const SymEval ev(symir, PH, PW);
  if (!ev.ok) return DNXCU_E_BAD_ARG;

  size_t nt = 0, nd = 0, ni = 0, nin = 0, nout = 0, nb = 0;
  model.vec(3, 4, &nt);
  model.vec(8, 4, &nd);
  model.vec(4, 4, &ni);
  model.vec(9, 4, &nb);
  const size_t pin = model.vec(5, 4, &nin), pout = model.vec(6, 4, &nout);
  if (nt == 0 || nd == 0 || nin != 1 || nout != 1) return DNXCU_E_UNSUPPORTED;
  m.tensors.assign(nt, TensorInfo());
  m.n_model_tensors = (int)nt;
  m.nodes.clear();
  m.ops.clear();
  m.from_dnx = true;
  m.dnx_variants.clear();
  std::vector<bool> is_param(nt, false);
  for (size_t t = 0; t < nt; ++t) {
    const fb::View tv = model.vec_table(3, t), info = tv.table(5);
    if (!tv.valid || !info.valid) return DNXCU_E_BAD_ARG;
    int64_t w = 0, h = 0, c = 0;
    if (!ev.source(info, 0, &w) || !ev.source(info, 2, &h) || !ev.source(info, 4, &c)) return DNXCU_E_BAD_ARG;
    if (info.scalar<uint16_t>(6) != FMT_SSBO_HWC) {
      is_param[t] = true;
      continue;
    }
    if (info.scalar<uint8_t>(8) != ST_F16 || w <= 0 || h <= 0 || c <= 0) return DNXCU_E_UNSUPPORTED;
    const int lw = log2_exact(PW / w), lh = log2_exact(PH / h);
    if (PW % w || PH % h || lw < 0 || lw != lh) return DNXCU_E_UNSUPPORTED;
    m.tensors[t].channels = (int)c;
    m.tensors[t].level = lw;
  }
  m.input_tensor = (int)model.b.rd<uint32_t>(pin);
  m.output_tensor = (int)model.b.rd<uint32_t>(pout);
  if (m.input_tensor < 0 || (size_t)m.input_tensor >= nt || (size_t)m.output_tensor >= nt) return DNXCU_E_BAD_ARG;
  m.input_channels = m.tensors[m.input_tensor].channels;
  m.tensors[m.input_tensor].materialized = true;

  std::map<uint32_t, std::pair<size_t, size_t>> init;  // tensor -> (position, bytes)
  for (size_t i = 0; i < ni; ++i) {
    const fb::View iv = model.vec_table(4, i);
    size_t len = 0;
    const size_t p = iv.vec(1, 1, &len);
    if (!iv.valid || !p) return DNXCU_E_BAD_ARG;
    init[iv.scalar<uint32_t>(0)] = std::make_pair(p, len);
  }

  for (size_t di = 0; di < nd; ++di) {
    const fb::View dv = model.vec_table(8, di);
    if (!dv.valid) return DNXCU_E_BAD_ARG;
    const uint32_t bin_id = dv.scalar<uint32_t>(0);
    if (bin_id >= nb) return DNXCU_E_BAD_ARG;
    const fb::View bv = model.vec_table(9, bin_id);
    size_t nw = 0;
    const size_t wp = bv.vec(0, 4, &nw);
    if (!wp || nw < 1) return DNXCU_E_BAD_ARG;
    const uint32_t *w = (const uint32_t *)(model.b.p + wp);
    uint32_t word0;
    memcpy(&word0, w, 4);
    if (word0 == kSpirvMagic) return DNXCU_E_UNSUPPORTED;  // a SPIR-V module: a file for the Vulkan runtime
    if (word0 != kBinaryMagic || nw < 10) return DNXCU_E_UNSUPPORTED;
    uint32_t hdr[10];
    memcpy(hdr, w, sizeof(hdr));
    if (hdr[1] != 1u) return DNXCU_E_UNSUPPORTED;
    const size_t flen = hdr[8], clen = hdr[9];
    if (flen > 256 || clen > 256 || 10 + (flen + 3) / 4 + (clen + 3) / 4 > nw) return DNXCU_E_BAD_ARG;
    const char *sp = (const char *)(w + 10);
    const std::string family(sp, flen), config(sp + (flen + 3) / 4 * 4, clen);
    const int variant = dnxcu_find_variant(family.c_str(), config.c_str());
    if (variant < 0) return DNXCU_E_UNSUPPORTED;  // a variant this build does not have
    if (dv.string(7) != family) return DNXCU_E_BAD_ARG;

    FusedOp op;
    op.op = (int)hdr[2];
    op.flags = hdr[3];
    op.c_a = (int)hdr[4];
    op.c_b = (int)hdr[5];
    op.c_out = (int)hdr[6];
    memcpy(&op.alpha, &hdr[7], 4);
    op.src_node = (int)di;
    op.name = dv.table(10).string(0);
    // bindings of set 0 in the order inputs, outputs, parameters
    const fb::View set0 = dv.vec_table(8, 0);
    size_t nbind = 0;
    set0.vec(1, 4, &nbind);
    std::vector<uint32_t> bt;
    for (size_t k = 0; k < nbind; ++k) {
      const fb::View b = set0.vec_table(1, k);
      const uint32_t t = b.scalar<uint32_t>(2, 0xffffffffu);
      if (!b.valid || t >= nt) return DNXCU_E_BAD_ARG;
      bt.push_back(t);
    }
    size_t k = 0;
    auto next = [&]() -> int { return k < bt.size() ? (int)bt[k++] : -1; };
    op.in_a = next();
    if (op.c_b > 0) op.in_b = next();
    if (!(op.flags & DNXCU_F_NO_FULL_OUT)) op.out = next();
    if (op.flags & DNXCU_F_POOL_OUT) op.out_pool = next();
    if (op.in_a < 0 || (op.c_b > 0 && op.in_b < 0) || (op.out < 0 && op.out_pool < 0)) return DNXCU_E_BAD_ARG;
    if (is_param[op.in_a] || (op.in_b >= 0 && is_param[op.in_b])) return DNXCU_E_BAD_ARG;
    if (op.op == DNXCU_OP_CONV3X3) {
      const int wt = next();
      auto it = wt >= 0 ? init.find((uint32_t)wt) : init.end();
      if (it == init.end()) return DNXCU_E_BAD_ARG;
      op.prepared.assign(model.b.p + it->second.first, model.b.p + it->second.first + it->second.second);
      size_t want = 0;
      if (dnxcu_prepare_weights(variant, nullptr, op.c_out, op.c_a, op.c_b, nullptr, &want) || want != op.prepared.size())
        return DNXCU_E_BAD_ARG;
      if (op.flags & DNXCU_F_BIAS) {
        const int bts = next();
        auto ib = bts >= 0 ? init.find((uint32_t)bts) : init.end();
        if (ib == init.end() || ib->second.second != (size_t)op.c_out * 2) return DNXCU_E_BAD_ARG;
        op.bias.resize(op.c_out);
        memcpy(op.bias.data(), model.b.p + ib->second.first, ib->second.second);
      }
    }
    // the dispatch's resolution level from its push constants {IN_W, IN_H}
    const fb::View pc = dv.table(9);
    int64_t pw = 0;
    const fb::View f0 = pc.vec_table(1, 0);
    if (!f0.valid || !ev.source(f0, 2, &pw) || pw <= 0 || PW % pw) return DNXCU_E_BAD_ARG;
    op.level = log2_exact(PW / pw);
    if (op.level < 0) return DNXCU_E_UNSUPPORTED;
    if (m.tensors[op.in_a].channels != op.c_a || (op.in_b >= 0 && m.tensors[op.in_b].channels != op.c_b))
      return DNXCU_E_BAD_ARG;
    if (op.out >= 0 && !(op.flags & DNXCU_F_NO_FULL_OUT)) m.tensors[op.out].materialized = true;
    if (op.out_pool >= 0) m.tensors[op.out_pool].materialized = true;
    if (op.flags & DNXCU_F_NO_FULL_OUT) op.out = op.out_pool;  // a tensor id for the unused slot (never bound)
    m.ops.push_back(std::move(op));
    m.dnx_variants.push_back(variant);
  }
  if (!m.tensors[m.output_tensor].materialized) return DNXCU_E_BAD_ARG;
  // ALIGN among the value names (the frame extents must be multiples of it)
  int align = 1;
  size_t nv = 0;
  model.vec(11, 4, &nv);
  for (size_t i = 0; i < nv; ++i) {
    const fb::View vn = model.vec_table(11, i);
    int64_t v = 0;
    if (vn.valid && vn.string(0) == "ALIGN" && ev.source(vn, 1, &v) && v > 0) align = (int)v;
  }
  if (align_out) *align_out = align;
  return DNXCU_OK;
}

}  // namespace dnxcu
