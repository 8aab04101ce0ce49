// Benchmark database: which variant runs a given dispatch fastest on this device.
// Same role and life cycle as denox::Db + runtime::Db::bench in the reference
// (database/src/denox/db/Db.cpp:546-756, runtime/src/denox/runtime/db.cpp:71-175,
// 542-868): populate adds (dispatch, variant) candidates, bench samples the
// un-converged ones until the standard error of the mean is small, the file is
// replaced atomically, selection reads mean latencies.
//
// The file is a FlatBuffer of the reference's schema (db.fbs:1-139, root table Db, identifier "dbdb"), written
// and read with this library's own codec (flatbuf.h):
//   * Db.env: one BenchEnv per process that added samples (device, driver, source digest, start time);
//   * Db.shader_binaries: one ShaderBinary per variant identity: src_sha256 = the eight words of
//     dnxcu_variant_sha256 (which covers the kernel sources), spirv = a "DNXC" descriptor (magic, variant id)
//     where the reference keeps SPIR-V;
//   * Db.dispatches: one ComputeDispatch per (variant, extent, channels, flags): binary_id, the launch grid as
//     workgroup counts, push_constant = {IN_W, IN_H} as in the reference followed by {c_a, c_b, c_out, flags}
//     (specialisation constants of the reference's shaders are arguments here), hash = FNV-1a over the identity
//     and the push constant bytes (the grid is left out: it follows the SM count of the device at hand),
//     time = every Sample {timestamp ns, latency ns, env} with mean and standard deviation in ns, and
//     info = operation / family / config names, algorithmic bytes and flops, coopmat = needs tcgen05.
// Entries whose identity this build does not know are kept and written back untouched.
#include "runtime.h"
#include "select.h"
#include "flatbuf.h"
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <sys/utsname.h>
#include <time.h>
#include <algorithm>
#include <map>
#include <random>
#include <string>

using namespace dnxcu;

struct DbSample {  // db.fbs:62-66
  uint64_t timestamp_ns = 0, latency_ns = 0;
  uint32_t env = 0;
};

struct DbEnv {  // db.fbs:114-128
  std::string device, os, driver_version, commit_hash, version;
  uint64_t start_timestamp = 0;
  uint16_t clock_mode = 1 /* None: clocks are never touched */, l2_warmup = 0, jit_warmup = 1, iterations = 0;
};

struct DbEntry {
  int variant = -1;  // resolved against this build's table; -1 when the identity is unknown here
  std::string sha;   // variant identity
  uint32_t w = 0, h = 0, flags = 0;
  int c_a = 0, c_b = 0, c_out = 0;
  std::vector<DbSample> samples;
  // running statistics (Welford) over the samples, latency in ms (Db.cpp:733-754)
  long long n = 0;
  double mean = 0, m2 = 0;
  // what the file said about an entry of unknown identity (written back as read)
  std::string operation, family, config;
  uint32_t grid[3] = {0, 0, 0};
  uint64_t reads = 0, writes = 0, flops = 0;
  bool coopmat = false;
};

struct dnxcu_db {
  std::string path;
  std::vector<DbEntry> entries;
  std::map<std::string, int> index;
  std::vector<DbEnv> envs;
  int session_env = -1;  // index of this process's BenchEnv once it has added a sample
};

namespace {

std::string key_of(const std::string &sha, uint32_t w, uint32_t h, int ca, int cb, int cout, uint32_t flags) {
  char buf[200];
  snprintf(buf, sizeof(buf), "%s/%u/%u/%d/%d/%d/%u", sha.c_str(), w, h, ca, cb, cout, flags);
  return buf;
}

int key_of_dispatch(const dnxcu_dispatch &d, std::string &key, std::string *sha_out = nullptr) {
  char sha[65];
  if (dnxcu_variant_sha256(d.variant, sha) != DNXCU_OK) return DNXCU_E_BAD_ARG;
  // pointer-free key, like the reference's (sha, push constants, workgroup counts) key (db.fbs:93-102)
  key = key_of(sha, d.pc[0], d.pc[1], d.c_a, d.c_b, d.c_out, d.flags);
  if (sha_out) *sha_out = sha;
  return DNXCU_OK;
}

void describe(DbEntry &e);

int find_or_add(dnxcu_db &db, const dnxcu_dispatch &d, bool add, bool *added = nullptr) {
  std::string key, sha;
  if (key_of_dispatch(d, key, &sha)) return -1;
  auto it = db.index.find(key);
  if (it != db.index.end()) return it->second;
  if (!add) return -1;
  DbEntry e;
  e.variant = d.variant;
  e.sha = sha;
  e.w = d.pc[0];
  e.h = d.pc[1];
  e.flags = d.flags;
  e.c_a = d.c_a;
  e.c_b = d.c_b;
  e.c_out = d.c_out;
  describe(e);
  db.entries.push_back(e);
  db.index[key] = (int)db.entries.size() - 1;
  if (added) *added = true;
  return (int)db.entries.size() - 1;
}

void account(DbEntry &e, double ms) {
  e.n += 1;
  const double delta = ms - e.mean;
  e.mean += delta / (double)e.n;
  e.m2 += delta * (ms - e.mean);
}

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

// This process's BenchEnv, made when it adds its first sample (Db.cpp:758-786).
uint32_t session_env(dnxcu_db &db, int iterations) {
  if (db.session_env >= 0) return (uint32_t)db.session_env;
  DbEnv env;
  env.device = "unknown";
  int dev = 0;
  cudaDeviceProp prop;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaGetDeviceProperties(&prop, dev) == cudaSuccess) env.device = prop.name;
  cudaGetLastError();
  utsname un;
  if (uname(&un) == 0) env.os = std::string(un.sysname) + " " + un.release;
  int drv = 0;
  if (cudaDriverGetVersion(&drv) == cudaSuccess) env.driver_version = std::to_string(drv / 1000) + "." + std::to_string(drv % 1000 / 10);
  cudaGetLastError();
#ifdef DNXCU_SOURCE_DIGEST
  env.commit_hash = DNXCU_SOURCE_DIGEST;
#endif
  env.version = "dnxcu (" + std::to_string(variant_count()) + " variants)";
  env.start_timestamp = now_ns();
  env.iterations = (uint16_t)iterations;
  db.envs.push_back(env);
  db.session_env = (int)db.envs.size() - 1;
  return (uint32_t)db.session_env;
}

void add_sample(dnxcu_db &db, DbEntry &e, double ms, int iterations) {
  DbSample smp;
  smp.timestamp_ns = now_ns();
  smp.latency_ns = (uint64_t)llround(ms * 1e6);
  smp.env = session_env(db, iterations);
  e.samples.push_back(smp);
  account(e, (double)smp.latency_ns * 1e-6);  // what a reader of the file will see
}

uint64_t fnv1a(const void *p, size_t n, uint64_t h = 1469598103934665603ull) {
  for (size_t i = 0; i < n; ++i) h = (h ^ ((const uint8_t *)p)[i]) * 1099511628211ull;
  return h;
}

constexpr uint32_t kDbBinaryMagic = 0x43584E44u;  // "DNXC", as in this library's dnx files

const char *operation_name(int op) {
  switch (op) {
    case DNXCU_OP_CONV3X3: return "conv3x3";
    case DNXCU_OP_MAXPOOL2X2: return "maxpool2x2";
    case DNXCU_OP_UPSAMPLE2X: return "upsample2x";
    case DNXCU_OP_CONCAT: return "concat";
    case DNXCU_OP_RELU: return "activation";
    case DNXCU_OP_PAD_CHANNELS: return "pad-channels";
    case DNXCU_OP_PAD_EDGE: return "pad";
    case DNXCU_OP_SLICE: return "slice";
    default: return "unknown";
  }
}

// Launch grid and algorithmic cost of a known entry (pointer-free probe of the dispatch).
void describe(DbEntry &e) {
  const Variant *v = get_variant(e.variant);
  if (!v) return;
  e.operation = operation_name(v->desc.op);
  e.family = v->desc.family;
  e.config = v->desc.config;
  e.coopmat = v->desc.needs_tcgen05 != 0;
  dnxcu_dispatch d;
  memset(&d, 0, sizeof(d));
  d.variant = e.variant;
  d.flags = e.flags;
  d.pc[0] = e.w;
  d.pc[1] = e.h;
  d.c_a = e.c_a;
  d.c_b = e.c_b;
  d.c_out = e.c_out;
  // placeholder addresses: only shapes matter to the grid and the cost
  void *const somewhere = (void *)(uintptr_t)0x1000;
  d.in_a = d.weights = d.bias = somewhere;
  d.out = d.out_pool = somewhere;
  if (e.c_b) d.in_b = somewhere;
  if (dnxcu_grid(&d, e.grid) != DNXCU_OK) e.grid[0] = e.grid[1] = e.grid[2] = 0;
  if (dnxcu_cost(&d, &e.reads, &e.writes, &e.flops) != DNXCU_OK) e.reads = e.writes = e.flops = 0;
}

std::vector<uint8_t> serialise(const dnxcu_db &db) {
  using namespace fb;
  auto root_t = make_table();
  root_t->scalar<uint32_t>(0, 0);  // version (Db.cpp:484)
  std::vector<std::shared_ptr<Table>> envs;
  for (const DbEnv &e : db.envs) {
    auto t = make_table();
    t->string(0, e.device);
    t->string(1, e.os);
    t->string(2, e.driver_version);
    t->string(3, e.commit_hash);
    t->string(4, e.version);
    t->scalar<uint64_t>(5, e.start_timestamp);
    t->scalar<uint16_t>(6, e.clock_mode);
    t->scalar<uint16_t>(7, e.l2_warmup);
    t->scalar<uint16_t>(8, e.jit_warmup);
    t->scalar<uint16_t>(9, e.iterations);
    envs.push_back(t);
  }
  root_t->tables(1, envs);
  // one binary per identity, in order of first use
  std::map<std::string, uint32_t> binary_of;
  std::vector<std::shared_ptr<Table>> binaries, dispatches;
  for (const DbEntry &e : db.entries) {
    auto it = binary_of.find(e.sha);
    if (it == binary_of.end()) {
      it = binary_of.emplace(e.sha, (uint32_t)binaries.size()).first;
      std::vector<uint32_t> words(8, 0);
      for (int i = 0; i < 8 && (size_t)(i * 8 + 8) <= e.sha.size(); ++i)
        words[i] = (uint32_t)strtoul(e.sha.substr((size_t)i * 8, 8).c_str(), nullptr, 16);
      auto t = make_table();
      t->vec<uint32_t>(0, words);
      std::vector<uint32_t> blob;
      blob.push_back(kDbBinaryMagic);
      blob.push_back(e.variant < 0 ? 0xffffffffu : (uint32_t)e.variant);
      t->vec<uint32_t>(1, blob);
      binaries.push_back(t);
    }
    auto t = make_table();
    t->scalar<uint32_t>(0, it->second);
    t->scalar<uint32_t>(1, e.grid[0]);
    t->scalar<uint32_t>(2, e.grid[1]);
    t->scalar<uint32_t>(3, e.grid[2]);
    const uint32_t pc[6] = {e.w, e.h, (uint32_t)e.c_a, (uint32_t)e.c_b, (uint32_t)e.c_out, e.flags};
    t->bytes(4, pc, sizeof(pc));
    t->scalar<uint64_t>(5, fnv1a(pc, sizeof(pc), fnv1a(e.sha.data(), e.sha.size())));
    {
      auto tm = make_table();
      std::vector<std::shared_ptr<Table>> smp;
      for (const DbSample &x : e.samples) {
        auto st = make_table();
        st->scalar<uint64_t>(0, x.timestamp_ns);
        st->scalar<uint64_t>(1, x.latency_ns);
        st->scalar<uint32_t>(2, x.env);
        smp.push_back(st);
      }
      tm->tables(0, smp);
      tm->scalar<uint64_t>(1, (uint64_t)llround(e.mean * 1e6));
      tm->scalar<uint64_t>(2, e.n > 1 ? (uint64_t)llround(sqrt(e.m2 / (double)(e.n - 1)) * 1e6) : 0);
      t->table(7, tm);
    }
    {
      auto inf = make_table();
      inf->string(0, e.operation);
      inf->string(1, e.family);
      inf->string(2, e.config);
      inf->scalar<uint64_t>(3, e.reads);
      inf->scalar<uint64_t>(4, e.writes);
      inf->scalar<uint64_t>(5, e.flops);
      inf->scalar<uint8_t>(6, e.coopmat ? 1 : 0);
      t->table(8, inf);
    }
    dispatches.push_back(t);
  }
  root_t->tables(2, binaries);
  root_t->tables(3, dispatches);
  return finish(*root_t, "dbdb");
}

int deserialise(dnxcu_db &db, const std::vector<uint8_t> &bytes) {
  using namespace fb;
  const View r = root(bytes.data(), bytes.size(), "dbdb");
  if (!r.valid) return DNXCU_E_IO;
  size_t n_env = 0, n_bin = 0, n_disp = 0;
  r.vec(1, 4, &n_env);
  r.vec(2, 4, &n_bin);
  r.vec(3, 4, &n_disp);
  for (size_t i = 0; i < n_env; ++i) {
    const View t = r.vec_table(1, i);
    DbEnv e;
    e.device = t.string(0);
    e.os = t.string(1);
    e.driver_version = t.string(2);
    e.commit_hash = t.string(3);
    e.version = t.string(4);
    e.start_timestamp = t.scalar<uint64_t>(5);
    e.clock_mode = t.scalar<uint16_t>(6);
    e.l2_warmup = t.scalar<uint16_t>(7);
    e.jit_warmup = t.scalar<uint16_t>(8);
    e.iterations = t.scalar<uint16_t>(9);
    db.envs.push_back(e);
  }
  std::vector<std::string> shas(n_bin);
  for (size_t i = 0; i < n_bin; ++i) {
    const View t = r.vec_table(2, i);
    size_t nw = 0;
    const size_t p0 = t.vec(0, 4, &nw);
    if (!p0 || nw != 8) return DNXCU_E_IO;
    char hex[65];
    for (int k = 0; k < 8; ++k) snprintf(hex + 8 * k, 9, "%08x", t.b.rd<uint32_t>(p0 + 4 * (size_t)k));
    shas[i] = hex;
    // a database of the reference holds SPIR-V here: its timings say nothing about this library's kernels
    size_t nb = 0;
    const size_t b0 = t.vec(1, 4, &nb);
    if (!b0 || nb < 1 || t.b.rd<uint32_t>(b0) != kDbBinaryMagic) return DNXCU_E_IO;
  }
  std::map<std::string, int> variant_of;
  for (int v = 0; v < variant_count(); ++v) {
    char vs[65];
    dnxcu_variant_sha256(v, vs);
    variant_of[vs] = v;
  }
  for (size_t i = 0; i < n_disp; ++i) {
    const View t = r.vec_table(3, i);
    const uint32_t bid = t.scalar<uint32_t>(0, 0xffffffffu);
    if (bid >= n_bin) return DNXCU_E_IO;
    DbEntry e;
    e.sha = shas[bid];
    auto vit = variant_of.find(e.sha);
    e.variant = vit == variant_of.end() ? -1 : vit->second;
    size_t npc = 0;
    const size_t pc0 = t.vec(4, 1, &npc);
    if (!pc0 || npc != 24) return DNXCU_E_IO;
    uint32_t pc[6];
    for (int k = 0; k < 6; ++k) pc[k] = t.b.rd<uint32_t>(pc0 + 4 * (size_t)k);
    e.w = pc[0];
    e.h = pc[1];
    e.c_a = (int)pc[2];
    e.c_b = (int)pc[3];
    e.c_out = (int)pc[4];
    e.flags = pc[5];
    e.grid[0] = t.scalar<uint32_t>(1);
    e.grid[1] = t.scalar<uint32_t>(2);
    e.grid[2] = t.scalar<uint32_t>(3);
    const View tm = t.table(7);
    size_t ns = 0;
    tm.vec(0, 4, &ns);
    for (size_t k = 0; k < ns; ++k) {
      const View st = tm.vec_table(0, k);
      DbSample x;
      x.timestamp_ns = st.scalar<uint64_t>(0);
      x.latency_ns = st.scalar<uint64_t>(1);
      x.env = st.scalar<uint32_t>(2);
      e.samples.push_back(x);
      account(e, (double)x.latency_ns * 1e-6);
    }
    const View inf = t.table(8);
    e.operation = inf.string(0);
    e.family = inf.string(1);
    e.config = inf.string(2);
    e.reads = inf.scalar<uint64_t>(3);
    e.writes = inf.scalar<uint64_t>(4);
    e.flops = inf.scalar<uint64_t>(5);
    e.coopmat = inf.scalar<uint8_t>(6) != 0;
    const std::string key = key_of(e.sha, e.w, e.h, e.c_a, e.c_b, e.c_out, e.flags);
    if (db.index.count(key)) continue;  // a duplicate key: the first one stands
    db.index[key] = (int)db.entries.size();
    db.entries.push_back(std::move(e));
  }
  return DNXCU_OK;
}

double rel_sem(const DbEntry &e) {
  if (e.n < 2 || e.mean <= 0) return 1e30;
  const double var = e.m2 / (double)(e.n - 1);
  return sqrt(var / (double)e.n) / e.mean;
}

// deterministic fill so that timings do not depend on stale memory (denormals / NaNs slow some paths)
__global__ void fill_pattern(__half *p, long long n, unsigned seed) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    unsigned x = (unsigned)i * 2654435761u + seed;
    x ^= x >> 15;
    x *= 2246822519u;
    x ^= x >> 13;
    p[i] = __float2half((float)(x & 0xffff) * (1.0f / 65536.0f) - 0.25f);
  }
}

struct Bufs {
  std::vector<void *> ptrs;
  ~Bufs() {
    for (void *p : ptrs) cudaFree(p);
  }
  void *get(size_t bytes, unsigned seed, bool fill) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) return nullptr;
    ptrs.push_back(p);
    if (fill) fill_pattern<<<592, 256>>>((__half *)p, (long long)(bytes / 2), seed);
    return p;
  }
};

// Builds a runnable dispatch (own buffers, patterned weights) for an entry.
int materialise(const DbEntry &e, Bufs &bufs, dnxcu_dispatch &d) {
  memset(&d, 0, sizeof(d));
  d.variant = e.variant;
  d.flags = e.flags;
  d.pc[0] = e.w;
  d.pc[1] = e.h;
  d.c_a = e.c_a;
  d.c_b = e.c_b;
  d.c_out = e.c_out;
  const Variant *v = get_variant(e.variant);
  if (!v) return DNXCU_E_BAD_ARG;
  const size_t P = (size_t)e.w * e.h;
  size_t a_bytes = P * e.c_a * 2, out_bytes = 0;
  switch (v->desc.op) {
    case DNXCU_OP_CONV3X3:
      if (e.flags & DNXCU_F_UP2X_A) a_bytes /= 4;
      out_bytes = P * e.c_out * 2;
      break;
    case DNXCU_OP_MAXPOOL2X2: out_bytes = (size_t)(e.w / 2) * (e.h / 2) * e.c_a * 2; break;
    case DNXCU_OP_UPSAMPLE2X: out_bytes = 4 * P * e.c_a * 2; break;
    case DNXCU_OP_CONCAT: out_bytes = P * (e.c_a + e.c_b) * 2; break;
    case DNXCU_OP_PAD_CHANNELS: out_bytes = P * e.c_out * 2; break;
    default: out_bytes = P * e.c_a * 2; break;
  }
  d.in_a = bufs.get(a_bytes, 1u, true);
  if (e.c_b > 0) d.in_b = bufs.get(P * e.c_b * 2, 2u, true);
  if (!(e.flags & DNXCU_F_NO_FULL_OUT)) d.out = bufs.get(out_bytes, 0, false);
  if (e.flags & DNXCU_F_POOL_OUT) d.out_pool = bufs.get(out_bytes / 4, 0, false);
  if (!d.in_a || (e.c_b > 0 && !d.in_b)) return DNXCU_E_NO_MEMORY;
  if (v->desc.op == DNXCU_OP_CONV3X3) {
    const int C = e.c_a + e.c_b;
    std::vector<uint16_t> kcrs((size_t)e.c_out * C * 9);
    std::mt19937 rng(1234u);
    for (uint16_t &x : kcrs) x = dnxcu_f16_from_float(((float)(rng() & 0xffff) / 65536.0f - 0.5f) * 0.2f);
    size_t bytes = 0;
    int st = dnxcu_prepare_weights(e.variant, nullptr, e.c_out, e.c_a, e.c_b, nullptr, &bytes);
    if (st) return st;
    std::vector<unsigned char> blob(bytes);
    st = dnxcu_prepare_weights(e.variant, kcrs.data(), e.c_out, e.c_a, e.c_b, blob.data(), &bytes);
    if (st) return st;
    void *dw = bufs.get(bytes, 0, false);
    if (!dw) return DNXCU_E_NO_MEMORY;
    if (cudaMemcpy(dw, blob.data(), bytes, cudaMemcpyHostToDevice) != cudaSuccess) return DNXCU_E_CUDA;
    d.weights = dw;
    if (e.flags & DNXCU_F_BIAS) {
      d.bias = bufs.get((size_t)e.c_out * 2, 3u, true);
      if (!d.bias) return DNXCU_E_NO_MEMORY;
    }
  }
  return DNXCU_OK;
}

}  // namespace

extern "C" {

int dnxcu_db_open(const char *path, dnxcu_db **out) {
  if (!path || !out) return DNXCU_E_BAD_ARG;
  dnxcu_db *db = new (std::nothrow) dnxcu_db();
  if (!db) return DNXCU_E_NO_MEMORY;
  db->path = path;
  FILE *f = fopen(path, "rb");
  if (f) {
    std::vector<uint8_t> bytes;
    uint8_t chunk[65536];
    size_t got;
    while ((got = fread(chunk, 1, sizeof(chunk), f)) > 0) bytes.insert(bytes.end(), chunk, chunk + got);
    fclose(f);
    const int st = deserialise(*db, bytes);
    if (st) {
      delete db;
      return st;
    }
  }
  *out = db;
  return DNXCU_OK;
}

void dnxcu_db_close(dnxcu_db *db) { delete db; }
int dnxcu_db_size(const dnxcu_db *db) { return db ? (int)db->entries.size() : DNXCU_E_BAD_ARG; }

int dnxcu_db_atomic_writeback(dnxcu_db *db) {
  if (!db) return DNXCU_E_BAD_ARG;
  const std::string tmp = db->path + ".tmp";
  FILE *f = fopen(tmp.c_str(), "wb");
  if (!f) return DNXCU_E_IO;
  const std::vector<uint8_t> bytes = serialise(*db);
  const bool wrote = fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
  if (fflush(f) != 0 || fclose(f) != 0 || !wrote) return DNXCU_E_IO;
  if (rename(tmp.c_str(), db->path.c_str()) != 0) return DNXCU_E_IO;
  return DNXCU_OK;
}

// Every candidate dispatch of the model at this extent: each node alone, each fusion pattern, each variant that
// takes it; reduced, like the reference's populate (populate.cpp:41), to the topologies with the fewest
// dispatches unless the model asks for selection by cost alone.
static int populate_model(dnxcu_db &db, const dnxcu_model &m, bool allow_tc, int height, int width) {
  if (m.from_dnx || m.nodes.empty()) return DNXCU_E_STATE;  // a compiled model has no candidates left to choose from
  HyperGraph g;
  std::vector<Candidate> cands;
  int st = build_supergraph(m, allow_tc, height, width, g, cands);
  if (st) return st;
  if (!(m.options & DNXCU_OPT_SELECT_BY_COST_ONLY) && !prune_topological(g, {m.input_tensor}, {m.output_tensor}))
    return DNXCU_E_UNSUPPORTED;
  int added = 0;
  for (const HyperEdge &e : g.edges) {
    const Candidate &c = cands[e.payload];
    const dnxcu_dispatch d = probe_dispatch(c.op, height, width, c.variant);
    bool is_new = false;
    find_or_add(db, d, true, &is_new);
    if (is_new) ++added;
  }
  return added;
}

// The candidates are those the device can run (the reference prunes its configuration space with the device info
// the same way, DirectConvShaderCM.cpp:19-28); device < 0: no device at hand, every variant counts.
static int device_allows_tc(int device, uint32_t options, bool *allow_tc) {
  *allow_tc = !(options & DNXCU_OPT_NO_TCGEN05);
  if (device >= 0) {
    dnxcu_caps caps;
    int cst = dnxcu_get_device_caps(device, &caps);
    if (cst) return cst;
    *allow_tc = *allow_tc && caps.tcgen05;
    cudaSetDevice(device);  // launch geometry follows this device's SM count
  }
  return DNXCU_OK;
}

int dnxcu_db_populate(dnxcu_db *db, const dnxcu_model_desc *desc, int height, int width, int device) {
  if (!db || !desc || height <= 0 || width <= 0) return DNXCU_E_BAD_ARG;
  bool allow_tc;
  int st = device_allows_tc(device, desc->options, &allow_tc);
  if (st) return st;
  dnxcu_model m;
  st = build_fused_ops(*desc, allow_tc, m);
  if (st) return st;
  m.options = desc->options;
  return populate_model(*db, m, allow_tc, height, width);
}

int dnxcu_db_populate_model(dnxcu_db *db, const dnxcu_model *m, int height, int width, int device) {
  if (!db || !m || height <= 0 || width <= 0) return DNXCU_E_BAD_ARG;
  bool allow_tc;
  int st = device_allows_tc(device, m->options, &allow_tc);
  if (st) return st;
  return populate_model(*db, *m, allow_tc, height, width);
}

int dnxcu_db_query(const dnxcu_db *db, const dnxcu_dispatch *d, double *mean_ms, double *std_ms, int *samples) {
  if (!db || !d) return DNXCU_E_BAD_ARG;
  const int i = find_or_add(*const_cast<dnxcu_db *>(db), *d, false);
  if (i < 0 || db->entries[i].n == 0) return DNXCU_E_BAD_ARG;
  const DbEntry &e = db->entries[i];
  if (mean_ms) *mean_ms = e.mean;
  if (std_ms) *std_ms = e.n > 1 ? sqrt(e.m2 / (double)(e.n - 1)) : 0.0;
  if (samples) *samples = (int)e.n;
  return DNXCU_OK;
}

int dnxcu_db_add_result(dnxcu_db *db, const dnxcu_dispatch *d, const double *samples_ms, int n) {
  if (!db || !d || !samples_ms || n <= 0) return DNXCU_E_BAD_ARG;
  const int i = find_or_add(*db, *d, true);
  if (i < 0) return DNXCU_E_BAD_ARG;
  for (int k = 0; k < n; ++k) add_sample(*db, db->entries[i], samples_ms[k], 1);
  return DNXCU_OK;
}

int dnxcu_db_bench(dnxcu_db *db, int device, int min_samples, double max_relative_error, int max_rounds) {
  if (!db || min_samples < 1 || max_relative_error <= 0 || max_rounds < 1) return DNXCU_E_BAD_ARG;
  DNXCU_CUDA(cudaSetDevice(device));
  cudaStream_t s;
  DNXCU_CUDA(cudaStreamCreate(&s));
  cudaEvent_t e0, e1;
  DNXCU_CUDA(cudaEventCreate(&e0));
  DNXCU_CUDA(cudaEventCreate(&e1));
  int *dstatus = nullptr;
  DNXCU_CUDA(cudaMalloc(&dstatus, 256));
  DNXCU_CUDA(cudaMemset(dstatus, 0, 256));
  // one sample = kReps launches back to back between one event pair: launch latency and event resolution
  // weigh less than with single launches, so the variant picks are stable from run to run
  constexpr int kReps = 5;
  int status = DNXCU_OK;
  for (int round = 0; round < max_rounds && status == DNXCU_OK; ++round) {
    // un-converged entries, never sampled first, then by largest relative standard error (db.cpp:88-175)
    std::vector<int> todo;
    for (int i = 0; i < (int)db->entries.size(); ++i) {
      const DbEntry &e = db->entries[i];
      if (e.variant < 0) continue;
      if (e.n >= min_samples && rel_sem(e) <= max_relative_error) continue;
      todo.push_back(i);
    }
    if (todo.empty()) break;
    std::sort(todo.begin(), todo.end(), [&](int a, int b) {
      const DbEntry &x = db->entries[a], &y = db->entries[b];
      if ((x.n == 0) != (y.n == 0)) return x.n == 0;
      return rel_sem(x) > rel_sem(y);
    });
    for (int i : todo) {
      DbEntry &e = db->entries[i];
      Bufs bufs;
      dnxcu_dispatch d;
      int st = materialise(e, bufs, d);
      if (st == DNXCU_E_NO_MEMORY) continue;
      if (st) { status = st; break; }
      d.device_status = dstatus;
      dnxcu_plan *plan = nullptr;
      st = dnxcu_plan_create(&d, &plan);
      if (st == DNXCU_E_UNSUPPORTED) continue;  // an entry of another device's database
      if (st) { status = st; break; }
      st = dnxcu_plan_launch(plan, s);  // untimed first launch
      const int want = e.n == 0 ? min_samples : std::max(2, min_samples / 2);
      for (int k = 0; k < want && !st; ++k) {
        cudaEventRecord(e0, s);
        for (int r = 0; r < kReps && !st; ++r) st = dnxcu_plan_launch(plan, s);
        cudaEventRecord(e1, s);
        if (st) break;
        if (cudaEventSynchronize(e1) != cudaSuccess) { st = DNXCU_E_CUDA; break; }
        int hstatus = 0;
        if (cudaMemcpy(&hstatus, dstatus, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { st = DNXCU_E_CUDA; break; }
        if (hstatus) {
          // a bounded wait ran out inside the kernel: this is a failure, not a latency
          cudaMemset(dstatus, 0, sizeof(int));
          st = DNXCU_E_DEVICE;
          break;
        }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        ms /= (float)kReps;
        if (ms > 0 && ms < 100000.0f) add_sample(*db, e, ms, kReps);  // the reference drops ts1 <= ts0 and > 100 s (db.cpp:498-540)
      }
      cudaStreamSynchronize(s);
      dnxcu_plan_destroy(plan);
      if (st) { status = st; break; }
    }
    if (status == DNXCU_OK) status = dnxcu_db_atomic_writeback(db);
  }
  cudaFree(dstatus);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(s);
  return status;
}

}  // extern "C"
