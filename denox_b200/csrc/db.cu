// Benchmark database: which variant runs a given dispatch fastest on this device.
// Same role and life cycle as denox::Db + runtime::Db::bench in the reference
// (database/src/denox/db/Db.cpp:546-756, runtime/src/denox/runtime/db.cpp:71-175,
// 542-868): populate adds (dispatch, variant) candidates, bench samples the
// un-converged ones until the standard error of the mean is small, the file is
// replaced atomically, selection reads mean latencies.  The file is a text
// table (one entry per line) instead of a flatbuffer.
#include "runtime.h"
#include "select.h"
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <algorithm>
#include <map>
#include <random>
#include <string>

using namespace dnxcu;

struct DbEntry {
  int variant = -1;  // resolved against this build's table; -1 when the identity is unknown here
  std::string sha;   // variant identity
  uint32_t w = 0, h = 0, flags = 0;
  int c_a = 0, c_b = 0, c_out = 0;
  // running statistics (Welford), latency in ms (Db.cpp:733-754)
  long long n = 0;
  double mean = 0, m2 = 0;
};

struct dnxcu_db {
  std::string path;
  std::vector<DbEntry> entries;
  std::map<std::string, int> index;
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
  db.entries.push_back(e);
  db.index[key] = (int)db.entries.size() - 1;
  if (added) *added = true;
  return (int)db.entries.size() - 1;
}

void add_sample(DbEntry &e, double ms) {
  e.n += 1;
  const double delta = ms - e.mean;
  e.mean += delta / (double)e.n;
  e.m2 += delta * (ms - e.mean);
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
  FILE *f = fopen(path, "r");
  if (f) {
    char line[512];
    bool header_ok = false;
    while (fgets(line, sizeof(line), f)) {
      if (!header_ok) {
        if (strncmp(line, "dnxcu-db 1", 10) != 0) {
          fclose(f);
          delete db;
          return DNXCU_E_IO;
        }
        header_ok = true;
        continue;
      }
      DbEntry e;
      char sha[80];
      if (sscanf(line, "%64s %u %u %d %d %d %u %lld %lf %lf", sha, &e.w, &e.h, &e.c_a, &e.c_b, &e.c_out, &e.flags, &e.n,
                 &e.mean, &e.m2) != 10)
        continue;
      e.sha = sha;
      for (int v = 0; v < variant_count(); ++v) {
        char vs[65];
        dnxcu_variant_sha256(v, vs);
        if (e.sha == vs) e.variant = v;
      }
      db->index[key_of(e.sha, e.w, e.h, e.c_a, e.c_b, e.c_out, e.flags)] = (int)db->entries.size();
      db->entries.push_back(e);
    }
    fclose(f);
  }
  *out = db;
  return DNXCU_OK;
}

void dnxcu_db_close(dnxcu_db *db) { delete db; }
int dnxcu_db_size(const dnxcu_db *db) { return db ? (int)db->entries.size() : DNXCU_E_BAD_ARG; }

int dnxcu_db_atomic_writeback(dnxcu_db *db) {
  if (!db) return DNXCU_E_BAD_ARG;
  const std::string tmp = db->path + ".tmp";
  FILE *f = fopen(tmp.c_str(), "w");
  if (!f) return DNXCU_E_IO;
  fprintf(f, "dnxcu-db 1\n");
  for (const DbEntry &e : db->entries)
    fprintf(f, "%s %u %u %d %d %d %u %lld %.9g %.9g\n", e.sha.c_str(), e.w, e.h, e.c_a, e.c_b, e.c_out, e.flags, e.n,
            e.mean, e.m2);
  if (fflush(f) != 0 || fclose(f) != 0) return DNXCU_E_IO;
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
  for (int k = 0; k < n; ++k) add_sample(db->entries[i], samples_ms[k]);
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
        if (ms > 0 && ms < 100000.0f) add_sample(e, ms);  // the reference drops ts1 <= ts0 and > 100 s (db.cpp:498-540)
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
