// dnxcu-cli: the command line front door of the backend, with the reference CLI's verbs and flag spelling
// (cli/src/denox/cli/main.cpp:16-48, README.md "Setup benchmark database" .. "Compile ONNX -> DNX"):
//
//   dnxcu-cli populate gpu.db net.onnx --assume H=1080 W=1920 [--device N] [--cost-only]
//   dnxcu-cli bench gpu.db [--samples=10] [--relative-error=0.05] [--device N]
//   dnxcu-cli bench net.dnx --spec H=1080 W=1920 [--device N]
//   dnxcu-cli compile net.onnx -o net.dnx [--db gpu.db --assume H=1080 W=1920] [--device N]
//   dnxcu-cli infer net.dnx|net.onnx --input in.npy --output out.npy [--device N]
//   dnxcu-cli version | help
//
// Everything goes through the C ABI of include/dnxcu.h.  The reference's --type / --shape / --storage /
// --format / --use-descriptor-sets flags are accepted so that its scripts keep working; this backend has one
// answer to each (f16, H:W:C, ssbo, hwc, one set) and refuses anything else.  Images are .npy files of HWC
// binary16 (the reference reads PNG through libpng, which is not available here).
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <map>
#include <string>
#include <vector>
#include "dnxcu.h"

namespace {

struct Args {
  std::string verb;
  std::vector<std::string> positional;
  std::map<std::string, std::string> opt;       // --key=value / --key value
  std::map<std::string, std::string> assign;    // NAME=value after --assume / --spec
  bool cost_only = false;
};

[[noreturn]] void die(const std::string &msg) {
  fprintf(stderr, "dnxcu-cli: %s\n", msg.c_str());
  exit(2);
}

void check(int st, const char *what) {
  if (st >= 0) return;
  std::string msg = std::string(what) + ": " + dnxcu_status_string(st);
  const char *why = dnxcu_last_error_message();
  if (why && why[0]) msg += std::string(" (") + why + ")";
  if (st == DNXCU_E_CUDA) msg += " [cudaError " + std::to_string(dnxcu_last_cuda_error()) + "]";
  die(msg);
}

Args parse(int argc, char **argv) {
  Args a;
  if (argc < 2) {
    a.verb = "help";
    return a;
  }
  a.verb = argv[1];
  // flags of the reference CLI that take a list of NAME=value items; only one value each is meaningful here
  const std::map<std::string, std::string> fixed = {{"--type", "f16"}, {"--storage", "ssbo"}, {"--format", "hwc"}};
  for (int i = 2; i < argc; ++i) {
    std::string s = argv[i];
    auto items = [&](auto &&fn) {
      while (i + 1 < argc && argv[i + 1][0] != '-') fn(std::string(argv[++i]));
    };
    if (s == "--assume" || s == "--spec") {
      items([&](const std::string &kv) {
        const size_t eq = kv.find('=');
        if (eq == std::string::npos) die("expected NAME=value after " + s + ", got " + kv);
        a.assign[kv.substr(0, eq)] = kv.substr(eq + 1);
      });
    } else if (fixed.count(s)) {
      items([&](const std::string &kv) {
        const size_t eq = kv.find('=');
        const std::string v = eq == std::string::npos ? kv : kv.substr(eq + 1);
        if (v != fixed.at(s)) die(s + " " + kv + ": this backend runs " + fixed.at(s) + " tensors only");
      });
    } else if (s == "--shape") {
      items([&](const std::string &kv) {
        const size_t eq = kv.find('=');
        const std::string v = eq == std::string::npos ? kv : kv.substr(eq + 1);
        if (v != "H:W:C") die("--shape " + kv + ": extents are named H:W:C here");
      });
    } else if (s == "--use-descriptor-sets") {
      items([&](const std::string &) {});
    } else if (s == "--cost-only") {
      a.cost_only = true;
    } else if (s == "-o") {
      if (i + 1 >= argc) die("-o needs a file name");
      a.opt["output"] = argv[++i];
    } else if (s.rfind("--", 0) == 0) {
      const size_t eq = s.find('=');
      std::string key = s.substr(2, eq == std::string::npos ? std::string::npos : eq - 2), val;
      if (eq != std::string::npos) val = s.substr(eq + 1);
      else if (i + 1 < argc && (argv[i + 1][0] != '-' || (argv[i + 1][1] >= '0' && argv[i + 1][1] <= '9'))) val = argv[++i];
      if (key == "database") key = "db";
      a.opt[key] = val;
    } else {
      a.positional.push_back(s);
    }
  }
  return a;
}

int opt_int(const Args &a, const char *key, int dflt) {
  auto it = a.opt.find(key);
  return it == a.opt.end() || it->second.empty() ? dflt : atoi(it->second.c_str());
}
double opt_double(const Args &a, const char *key, double dflt) {
  auto it = a.opt.find(key);
  return it == a.opt.end() || it->second.empty() ? dflt : atof(it->second.c_str());
}
bool extent(const Args &a, int *h, int *w) {
  auto ih = a.assign.find("H"), iw = a.assign.find("W");
  if (ih == a.assign.end() || iw == a.assign.end()) return false;
  *h = atoi(ih->second.c_str());
  *w = atoi(iw->second.c_str());
  if (*h <= 0 || *w <= 0) die("H and W must be positive");
  return true;
}

std::vector<uint8_t> read_file(const std::string &path) {
  FILE *f = fopen(path.c_str(), "rb");
  if (!f) die("cannot open " + path);
  std::vector<uint8_t> data;
  uint8_t buf[1 << 16];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) data.insert(data.end(), buf, buf + n);
  fclose(f);
  return data;
}
void write_file(const std::string &path, const void *p, size_t n) {
  FILE *f = fopen(path.c_str(), "wb");
  if (!f || fwrite(p, 1, n, f) != n || fclose(f) != 0) die("cannot write " + path);
}
bool ends_with(const std::string &s, const char *suffix) {
  const size_t n = strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

// .npy (format 1.0 / 2.0) of a C-ordered binary16 array with three dimensions H, W, C
std::vector<uint16_t> read_npy(const std::string &path, int *h, int *w, int *c) {
  const std::vector<uint8_t> d = read_file(path);
  if (d.size() < 10 || memcmp(d.data(), "\x93NUMPY", 6) != 0) die(path + ": not a .npy file");
  size_t hlen, hoff;
  if (d[6] == 1) {
    hlen = d[8] | (d[9] << 8);
    hoff = 10;
  } else {
    if (d.size() < 12) die(path + ": truncated");
    hlen = d[8] | (d[9] << 8) | (d[10] << 16) | ((size_t)d[11] << 24);
    hoff = 12;
  }
  if (hoff + hlen > d.size()) die(path + ": truncated header");
  const std::string hdr((const char *)d.data() + hoff, hlen);
  if (hdr.find("'<f2'") == std::string::npos && hdr.find("'|f2'") == std::string::npos && hdr.find("float16") == std::string::npos)
    die(path + ": expected dtype float16 ('<f2')");
  if (hdr.find("'fortran_order': False") == std::string::npos) die(path + ": expected C order");
  const size_t sp = hdr.find("'shape': (");
  if (sp == std::string::npos || sscanf(hdr.c_str() + sp + 10, "%d, %d, %d", h, w, c) != 3) die(path + ": expected shape (H, W, C)");
  const size_t n = (size_t)*h * *w * *c;
  if (hoff + hlen + n * 2 != d.size()) die(path + ": size does not match its header");
  std::vector<uint16_t> out(n);
  memcpy(out.data(), d.data() + hoff + hlen, n * 2);
  return out;
}
void write_npy(const std::string &path, const uint16_t *data, int h, int w, int c) {
  char dict[128];
  snprintf(dict, sizeof(dict), "{'descr': '<f2', 'fortran_order': False, 'shape': (%d, %d, %d), }", h, w, c);
  std::string hdr = dict;
  while ((10 + hdr.size() + 1) % 64) hdr += ' ';
  hdr += '\n';
  std::vector<uint8_t> out = {0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0, (uint8_t)(hdr.size() & 0xff), (uint8_t)(hdr.size() >> 8)};
  out.insert(out.end(), hdr.begin(), hdr.end());
  const uint8_t *p = (const uint8_t *)data;
  out.insert(out.end(), p, p + (size_t)h * w * c * 2);
  write_file(path, out.data(), out.size());
}

dnxcu_model *load_model(const std::string &path, const dnxcu_db *db, int device, uint32_t options) {
  const std::vector<uint8_t> bytes = read_file(path);
  dnxcu_model *m = nullptr;
  if (ends_with(path, ".dnx")) check(dnxcu_model_create_from_dnx(bytes.data(), bytes.size(), device, &m), "reading the dnx file");
  else check(dnxcu_model_create_from_onnx(bytes.data(), bytes.size(), db, device, options, &m), "importing the ONNX file");
  return m;
}

int cmd_populate(const Args &a) {
  if (a.positional.size() != 2) die("usage: populate <gpu.db> <net.onnx> --assume H=.. W=..");
  int h, w;
  if (!extent(a, &h, &w)) die("populate needs --assume H=<height> W=<width>");
  const int device = opt_int(a, "device", 0);
  const uint32_t options = a.cost_only ? DNXCU_OPT_SELECT_BY_COST_ONLY : 0u;
  dnxcu_db *db = nullptr;
  check(dnxcu_db_open(a.positional[0].c_str(), &db), "opening the database");
  dnxcu_model *m = load_model(a.positional[1], nullptr, device, options);
  const int added = dnxcu_db_populate_model(db, m, h, w, device);
  check(added, "populate");
  dnxcu_model_destroy(m);
  check(dnxcu_db_atomic_writeback(db), "writing the database");
  printf("%d dispatches added, %d in the database\n", added, dnxcu_db_size(db));
  dnxcu_db_close(db);
  return 0;
}

int cmd_bench(const Args &a) {
  if (a.positional.size() != 1) die("usage: bench <gpu.db> | bench <net.dnx> --spec H=.. W=..");
  const int device = opt_int(a, "device", 0);
  const std::string &path = a.positional[0];
  if (ends_with(path, ".dnx") || ends_with(path, ".onnx")) {
    int h, w;
    if (!extent(a, &h, &w)) die("bench of a model needs --spec H=<height> W=<width>");
    dnxcu_model *m = load_model(path, nullptr, device, 0);
    dnxcu_instance *inst = nullptr;
    check(dnxcu_instance_create(m, h, w, nullptr, &inst), "creating the instance");
    const int n = dnxcu_instance_dispatch_count(inst);
    std::vector<dnxcu_dispatch_info> info(n);
    float total = 0;
    check(dnxcu_instance_bench(inst, 10, opt_int(a, "samples", 20), info.data(), n, &total), "benchmarking");
    printf("%-40s %-44s %10s %10s %10s\n", "dispatch", "variant", "ms", "GB/s", "TFLOP/s");
    for (const dnxcu_dispatch_info &d : info) {
      const dnxcu_variant_desc *v = dnxcu_variant(d.variant);
      printf("%-40s %-44s %10.4f %10.1f %10.1f\n", d.name, v ? v->config : "?", d.ms,
             (double)(d.bytes_read + d.bytes_written) / d.ms / 1e6, (double)d.flops / d.ms / 1e9);
    }
    printf("total %.4f ms per frame, %.1f frames/s\n", total, 1e3 / total);
    dnxcu_instance_destroy(inst);
    dnxcu_model_destroy(m);
    return 0;
  }
  dnxcu_db *db = nullptr;
  check(dnxcu_db_open(path.c_str(), &db), "opening the database");
  check(dnxcu_db_bench(db, device, opt_int(a, "samples", 10), opt_double(a, "relative-error", 0.05), opt_int(a, "rounds", 8)),
        "benchmarking the database");
  printf("%d dispatches in the database\n", dnxcu_db_size(db));
  dnxcu_db_close(db);
  return 0;
}

int cmd_compile(const Args &a) {
  if (a.positional.size() != 1 || !a.opt.count("output")) die("usage: compile <net.onnx> -o <net.dnx> [--db gpu.db --assume H=.. W=..]");
  const uint32_t options = a.cost_only ? DNXCU_OPT_SELECT_BY_COST_ONLY : 0u;
  std::vector<uint8_t> out;
  size_t n = 0;
  if (a.opt.count("db")) {
    // with a database the schedule is the cheapest one at the assumed extent: that needs the device
    int h, w;
    if (!extent(a, &h, &w)) die("compile with a database needs --assume H=<height> W=<width>");
    const int device = opt_int(a, "device", 0);
    dnxcu_db *db = nullptr;
    check(dnxcu_db_open(a.opt.at("db").c_str(), &db), "opening the database");
    dnxcu_model *m = load_model(a.positional[0], db, device, options);
    dnxcu_instance *inst = nullptr;
    check(dnxcu_instance_create(m, h, w, nullptr, &inst), "selecting the schedule");
    check(dnxcu_instance_write_dnx(inst, nullptr, &n), "serialising");
    out.resize(n);
    check(dnxcu_instance_write_dnx(inst, out.data(), &n), "serialising");
    printf("%d dispatches\n", dnxcu_instance_dispatch_count(inst));
    dnxcu_instance_destroy(inst);
    dnxcu_model_destroy(m);
    dnxcu_db_close(db);
  } else {
    dnxcu_model *m = load_model(a.positional[0], nullptr, -1, options);
    check(dnxcu_model_write_dnx(m, nullptr, &n), "serialising");
    out.resize(n);
    check(dnxcu_model_write_dnx(m, out.data(), &n), "serialising");
    printf("%d dispatches\n", dnxcu_model_dispatch_count(m));
    dnxcu_model_destroy(m);
  }
  write_file(a.opt.at("output"), out.data(), n);
  printf("%s: %zu bytes\n", a.opt.at("output").c_str(), n);
  return 0;
}

int cmd_infer(const Args &a) {
  if (a.positional.size() != 1 || !a.opt.count("input") || !a.opt.count("output"))
    die("usage: infer <net.dnx|net.onnx> --input in.npy --output out.npy");
  const int device = opt_int(a, "device", 0);
  int h, w, c;
  const std::vector<uint16_t> x = read_npy(a.opt.at("input"), &h, &w, &c);
  dnxcu_model *m = load_model(a.positional[0], nullptr, device, 0);
  int cin = 0, tout = 0;
  check(dnxcu_model_io(m, nullptr, &cin, &tout), "model");
  if (cin != c) die("the image has " + std::to_string(c) + " channels, the model takes " + std::to_string(cin));
  dnxcu_instance *inst = nullptr;
  check(dnxcu_instance_create(m, h, w, nullptr, &inst), "creating the instance");
  int oh, ow, oc;
  void *ptr;
  check(dnxcu_instance_tensor(inst, tout, &ptr, &oh, &ow, &oc), "output tensor");
  int fh, fw;
  check(dnxcu_instance_extent(inst, &fh, &fw, nullptr, nullptr), "extent");
  std::vector<uint16_t> y((size_t)fh * fw * oc);
  check(dnxcu_instance_infer(inst, x.data(), y.data()), "infer");
  write_npy(a.opt.at("output"), y.data(), fh, fw, oc);
  printf("%s: %d x %d x %d\n", a.opt.at("output").c_str(), fh, fw, oc);
  dnxcu_instance_destroy(inst);
  dnxcu_model_destroy(m);
  return 0;
}

int cmd_help() {
  puts("dnxcu-cli <command>\n"
       "  populate <gpu.db> <net.onnx> --assume H=<h> W=<w> [--device N] [--cost-only]\n"
       "      add every candidate dispatch of the model at that extent to the benchmark database\n"
       "  bench <gpu.db> [--samples=10] [--relative-error=0.05] [--rounds=8] [--device N]\n"
       "      time the database's dispatches until their latencies converge\n"
       "  bench <net.dnx|net.onnx> --spec H=<h> W=<w> [--samples=20] [--device N]\n"
       "      per dispatch timing of a model\n"
       "  compile <net.onnx> -o <net.dnx> [--db gpu.db --assume H=<h> W=<w>] [--cost-only] [--device N]\n"
       "      write the model's schedule (with a database: the cheapest at that extent) as a dnx file\n"
       "  infer <net.dnx|net.onnx> --input in.npy --output out.npy [--device N]\n"
       "      run one HWC float16 frame\n"
       "  version | help\n"
       "Accepted for compatibility with denox scripts: --type *=f16, --shape *=H:W:C, --storage *=ssbo,\n"
       "--format *=hwc, --use-descriptor-sets ...");
  return 0;
}

int cmd_version() {
  char sha[65] = "";
  dnxcu_variant_sha256(0, sha);
  printf("dnxcu-cli, %d kernel variants, build identity %.16s\n", dnxcu_variant_count(), sha);
  return 0;
}

}  // namespace

int main(int argc, char **argv) {
  const Args a = parse(argc, argv);
  if (a.verb == "populate") return cmd_populate(a);
  if (a.verb == "bench") return cmd_bench(a);
  if (a.verb == "compile") return cmd_compile(a);
  if (a.verb == "infer") return cmd_infer(a);
  if (a.verb == "version" || a.verb == "--version") return cmd_version();
  if (a.verb == "help" || a.verb == "--help" || a.verb == "-h") return cmd_help();
  die("unknown command \"" + a.verb + "\" (try: help)");
}
