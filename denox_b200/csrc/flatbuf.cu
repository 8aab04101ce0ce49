// Minimal FlatBuffers writer and reader (see flatbuf.h).
#include "flatbuf.h"
#include <algorithm>

namespace dnxcu {
namespace fb {
namespace {

struct Out {
  std::vector<uint8_t> buf;
  void align(size_t a) {
    while (buf.size() % a) buf.push_back(0);
  }
  template <class T>
  size_t put(T v) {
    const size_t pos = buf.size();
    buf.resize(pos + sizeof(T));
    memcpy(buf.data() + pos, &v, sizeof(T));
    return pos;
  }
  template <class T>
  void patch(size_t pos, T v) { memcpy(buf.data() + pos, &v, sizeof(T)); }
  size_t put_bytes(const void *p, size_t n) {
    const size_t pos = buf.size();
    buf.resize(pos + n);
    if (n) memcpy(buf.data() + pos, p, n);
    return pos;
  }
};

size_t emit_table(Out &o, const Table &t);

// Emits a string / vector / table and returns the position a uoffset must point at.
size_t emit_object(Out &o, const Value &v) {
  switch (v.kind) {
    case Value::STRING: {
      o.align(4);
      const size_t pos = o.put<uint32_t>((uint32_t)v.str.size());
      o.put_bytes(v.str.data(), v.str.size());
      o.put<uint8_t>(0);
      return pos;
    }
    case Value::VEC_SCALAR: {
      // the element data must be aligned for its type; the count sits in the four bytes right in front of it
      const size_t a = std::max<size_t>(4, v.elem_align);
      o.align(4);
      while ((o.buf.size() + 4) % a) o.buf.push_back(0);
      const size_t pos = o.put<uint32_t>((uint32_t)(v.elem_size ? v.raw.size() / v.elem_size : 0));
      o.put_bytes(v.raw.data(), v.raw.size());
      return pos;
    }
    case Value::VEC_TABLE: {
      o.align(4);
      const size_t pos = o.put<uint32_t>((uint32_t)v.tables.size());
      const size_t first = o.buf.size();
      for (size_t i = 0; i < v.tables.size(); ++i) o.put<uint32_t>(0);
      for (size_t i = 0; i < v.tables.size(); ++i) {
        const size_t tp = emit_table(o, *v.tables[i]);
        const size_t fp = first + 4 * i;
        o.patch<uint32_t>(fp, (uint32_t)(tp - fp));
      }
      return pos;
    }
    case Value::TABLE: return emit_table(o, *v.table);
    default: return 0;
  }
}

size_t emit_table(Out &o, const Table &t) {
  // inline layout: the 4 byte offset to the vtable, then every present field, largest alignment first is not
  // required by the format; fields are simply placed in slot order at their natural alignment
  const size_t nslots = t.slots.size();
  std::vector<uint16_t> off(nslots, 0);
  size_t cur = 4;
  size_t max_align = 4;
  for (size_t i = 0; i < nslots; ++i) {
    const Value &v = t.slots[i];
    if (v.kind == Value::NONE) continue;
    const size_t sz = v.kind == Value::SCALAR ? v.raw.size() : 4;
    cur = (cur + sz - 1) / sz * sz;
    off[i] = (uint16_t)cur;
    cur += sz;
    max_align = std::max(max_align, sz);
  }
  const size_t tsize = cur;
  const size_t vsize = 4 + 2 * nslots;
  // the vtable directly in front of the table; the table itself aligned for its widest scalar
  o.align(2);
  while ((o.buf.size() + vsize) % max_align) o.buf.push_back(0);
  const size_t vpos = o.buf.size();
  o.put<uint16_t>((uint16_t)vsize);
  o.put<uint16_t>((uint16_t)tsize);
  for (size_t i = 0; i < nslots; ++i) o.put<uint16_t>(off[i]);
  const size_t tpos = o.buf.size();
  o.buf.resize(tpos + tsize, 0);
  o.patch<int32_t>(tpos, (int32_t)(tpos - vpos));
  for (size_t i = 0; i < nslots; ++i) {
    const Value &v = t.slots[i];
    if (v.kind == Value::SCALAR) memcpy(o.buf.data() + tpos + off[i], v.raw.data(), v.raw.size());
  }
  for (size_t i = 0; i < nslots; ++i) {
    const Value &v = t.slots[i];
    if (v.kind == Value::NONE || v.kind == Value::SCALAR) continue;
    const size_t target = emit_object(o, v);
    const size_t fp = tpos + off[i];
    o.patch<uint32_t>(fp, (uint32_t)(target - fp));
  }
  return tpos;
}

}  // namespace

std::vector<uint8_t> finish(const Table &root_table, const char identifier[4]) {
  Out o;
  o.put<uint32_t>(0);  // offset to the root table
  o.put_bytes(identifier, 4);
  const size_t tp = emit_table(o, root_table);
  o.patch<uint32_t>(0, (uint32_t)tp);
  o.align(8);
  return o.buf;
}

size_t View::field(size_t slot) const {
  if (!valid) return 0;
  const int32_t so = b.rd<int32_t>(pos);
  const int64_t vpos = (int64_t)pos - so;
  if (vpos < 0 || !b.ok((size_t)vpos, 4)) return 0;
  const uint16_t vsize = b.rd<uint16_t>((size_t)vpos);
  if (vsize < 4 || !b.ok((size_t)vpos, vsize)) return 0;
  const size_t entry = 4 + 2 * slot;
  if (entry + 2 > vsize) return 0;
  const uint16_t fo = b.rd<uint16_t>((size_t)vpos + entry);
  if (!fo) return 0;
  const size_t f = pos + fo;
  return b.ok(f, 1) ? f : 0;
}

static size_t follow(const Buf &b, size_t f) {
  if (!f || !b.ok(f, 4)) return 0;
  const uint32_t uo = b.rd<uint32_t>(f);
  const size_t target = f + uo;
  return (uo && b.ok(target, 4)) ? target : 0;
}

std::string View::string(size_t slot) const {
  const size_t t = follow(b, field(slot));
  if (!t) return std::string();
  const uint32_t len = b.rd<uint32_t>(t);
  if (!b.ok(t + 4, len)) return std::string();
  return std::string((const char *)b.p + t + 4, len);
}

View View::table(size_t slot) const {
  View v;
  v.b = b;
  const size_t t = follow(b, field(slot));
  v.pos = t;
  v.valid = t != 0;
  return v;
}

size_t View::vec(size_t slot, size_t elem_size, size_t *count) const {
  *count = 0;
  const size_t t = follow(b, field(slot));
  if (!t) return 0;
  const uint32_t len = b.rd<uint32_t>(t);
  if (elem_size && (size_t)len > (b.n - t - 4) / elem_size) return 0;
  *count = len;
  return t + 4;
}

View View::vec_table(size_t slot, size_t i) const {
  View v;
  v.b = b;
  size_t n = 0;
  const size_t first = vec(slot, 4, &n);
  if (!first || i >= n) return v;
  const size_t t = follow(b, first + 4 * i);
  v.pos = t;
  v.valid = t != 0;
  return v;
}

View root(const void *data, size_t n, const char *identifier) {
  View v;
  v.b.p = (const uint8_t *)data;
  v.b.n = n;
  if (!data || n < 8) return v;
  if (identifier && memcmp((const uint8_t *)data + 4, identifier, 4) != 0) return v;
  const uint32_t ro = v.b.rd<uint32_t>(0);
  if (!ro || !v.b.ok(ro, 4)) return v;
  v.pos = ro;
  v.valid = true;
  return v;
}

}  // namespace fb
}  // namespace dnxcu
