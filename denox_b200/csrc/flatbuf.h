// A minimal FlatBuffers codec: just what reading and writing denox's dnx files (dnx.fbs) and benchmark
// databases (db.fbs) needs, written against the published binary format (a table is a signed offset to its
// vtable followed by its inline fields; a vtable is [its size, the table's inline size, one 16-bit field offset
// per slot, 0 = absent]; strings, vectors and sub-tables are reached through unsigned 32-bit offsets relative to
// the offset's own position, always pointing forward; vectors start with a 32-bit element count).  The
// reference links the FlatBuffers library and flatc generated headers, neither of which exists here.
//
// Writer: an in-memory tree of values that is laid out front to back (every object behind the table that refers
// to it), each table directly behind its own vtable.
// Reader: bounds checked accessors; a malformed buffer yields "absent", never an out-of-range read.
#pragma once
#include <stdint.h>
#include <string.h>
#include <memory>
#include <string>
#include <vector>

namespace dnxcu {
namespace fb {

// ---- writer -------------------------------------------------------------------------------------------------

struct Table;

struct Value {
  enum Kind { NONE, SCALAR, STRING, BYTES, VEC_SCALAR, VEC_TABLE, TABLE } kind = NONE;
  // SCALAR: little endian bytes (1, 2, 4 or 8); VEC_SCALAR / BYTES: raw element bytes
  std::vector<uint8_t> raw;
  uint32_t elem_size = 1;   // VEC_SCALAR: bytes per element (structs included); its alignment is elem_align
  uint32_t elem_align = 1;
  std::string str;
  std::shared_ptr<Table> table;
  std::vector<std::shared_ptr<Table>> tables;
};

struct Table {
  std::vector<Value> slots;  // index = field id of the schema
  Value &at(size_t i) {
    if (slots.size() <= i) slots.resize(i + 1);
    return slots[i];
  }
  template <class T>
  void scalar(size_t i, T v) {
    Value &x = at(i);
    x.kind = Value::SCALAR;
    x.raw.resize(sizeof(T));
    memcpy(x.raw.data(), &v, sizeof(T));
  }
  void string(size_t i, const std::string &s) {
    Value &x = at(i);
    x.kind = Value::STRING;
    x.str = s;
  }
  void bytes(size_t i, const void *p, size_t n) {
    Value &x = at(i);
    x.kind = Value::VEC_SCALAR;
    x.elem_size = x.elem_align = 1;
    x.raw.assign((const uint8_t *)p, (const uint8_t *)p + n);
  }
  template <class T>
  void vec(size_t i, const std::vector<T> &v, uint32_t align = sizeof(T)) {
    Value &x = at(i);
    x.kind = Value::VEC_SCALAR;
    x.elem_size = sizeof(T);
    x.elem_align = align;
    x.raw.resize(v.size() * sizeof(T));
    if (!v.empty()) memcpy(x.raw.data(), v.data(), x.raw.size());
  }
  void table(size_t i, std::shared_ptr<Table> t) {
    Value &x = at(i);
    x.kind = Value::TABLE;
    x.table = std::move(t);
  }
  void tables(size_t i, std::vector<std::shared_ptr<Table>> t) {
    Value &x = at(i);
    x.kind = Value::VEC_TABLE;
    x.tables = std::move(t);
  }
};

inline std::shared_ptr<Table> make_table() { return std::make_shared<Table>(); }

// Serialises `root` as a finished buffer with the 4 character file identifier.
std::vector<uint8_t> finish(const Table &root, const char identifier[4]);

// ---- reader -------------------------------------------------------------------------------------------------

struct Buf {
  const uint8_t *p = nullptr;
  size_t n = 0;
  bool ok(size_t pos, size_t len) const { return pos <= n && len <= n - pos; }
  template <class T>
  T rd(size_t pos) const {
    T v{};
    if (ok(pos, sizeof(T))) memcpy(&v, p + pos, sizeof(T));
    return v;
  }
};

struct View {  // a table inside a buffer
  Buf b;
  size_t pos = 0;
  bool valid = false;
  // position of field `slot`'s inline data, 0 when absent
  size_t field(size_t slot) const;
  template <class T>
  T scalar(size_t slot, T dflt = T{}) const {
    const size_t f = field(slot);
    return f && b.ok(f, sizeof(T)) ? b.rd<T>(f) : dflt;
  }
  bool has(size_t slot) const { return field(slot) != 0; }
  std::string string(size_t slot) const;
  View table(size_t slot) const;
  // vectors: element count and position of element 0 (0 when absent or malformed)
  size_t vec(size_t slot, size_t elem_size, size_t *count) const;
  View vec_table(size_t slot, size_t i) const;
};

// Root table of a finished buffer; `identifier` (4 characters) is checked when given.
View root(const void *data, size_t n, const char *identifier);

}  // namespace fb
}  // namespace dnxcu
