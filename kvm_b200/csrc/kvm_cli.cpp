// kvm_exec: run bundle directories on the B200 executor from the command line, with the reference CLI's contract
// (mvm_exec.cu:1962-1982 options, :2252-2309 golden compare and result line), over the C ABI of include/kvm_b200.h only.
//
//   kvm_exec [options] bundle_dir...
//     --golden [--golden-tol R]   compare final buffers (relative L2 per buffer; i32 exact) and versions with <bundle_dir>/golden.json
//     --dump-bin DIR i,j,..       write the listed buffers (metadata index) widened to little-endian float32 to DIR/<index>.bin
//     --dump-buffers              print every buffer as text ("buffer <i>: v v v ...", what the reference's golden_check.py reads)
//     --trace-csv FILE            per-task timeline: task,start_ns,end_ns,smid
//     --workers N  --timeout-s N  --device N  --no-tensor-cores  --static | --dynamic  --steps N  --quiet  --check-ops
//
// Prints ONE result line on stdout:   OK|FAIL: <done>/<admitted> tasks, <ms> ms[, golden match|golden MISMATCH]
// (the reference's bench drivers parse exactly this line, bench/exec_vs_torch/run_gpt.py:79).  Exit 0 pass, 1 fail, 2 usage.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/kvm_b200.h"
#include "kvm_json.hpp"

static int g_log = 2;
#define KLOG(level, ...) do { if (g_log >= (level)) { fprintf(stderr, "kvm_exec: "); fprintf(stderr, __VA_ARGS__); fprintf(stderr, "\n"); } } while (0)

static void usage() {
  fprintf(stderr,
          "usage: kvm_exec [options] bundle_dir...\n"
          "  bundle_dir: tasks.bin successors.bin args.bin metadata.json (ABI v2)\n"
          "  --golden [--golden-tol R]  compare with <bundle_dir>/golden.json (single bundle): final buffers, versions\n"
          "  --dump-bin DIR i,j,..      write the listed buffers (metadata index, widened to little-endian f32) to DIR/<index>.bin\n"
          "  --dump-buffers             print buffers as text\n"
          "  --trace-csv FILE           per-task timeline\n"
          "  --workers N  --timeout-s N  --device N  --steps N (re-arm and run the program N times)\n"
          "  --no-tensor-cores          every GEMM on the bit-exact SIMT path\n"
          "  --static | --dynamic       per-worker programs planned at load | ready queue (default: decided from the bundle)\n"
          "  --quiet  --check-ops\n");
}

static bool read_file(const std::string& path, std::string& out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}

int main(int argc, char** argv) {
  KvmConfig cfg{};
  std::vector<std::string> dirs;
  const char* csv = nullptr;
  bool golden = false, dump = false;
  double golden_tol = 1e-6;
  std::string dump_dir;
  std::vector<int> dump_idx;
  int steps = 1;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto val = [&](long long lo, long long hi) -> long long {
      if (i + 1 >= argc) { usage(); exit(2); }
      char* e; errno = 0;
      const long long v = strtoll(argv[++i], &e, 10);
      if (e == argv[i] || *e || errno || v < lo || v > hi) { fprintf(stderr, "%s: integer in [%lld,%lld] expected, got '%s'\n", a.c_str(), lo, hi, argv[i]); exit(2); }
      return v;
    };
    if (a == "--workers") cfg.workers = (int)val(1, 1 << 20);
    else if (a == "--device") cfg.device = (int)val(0, 1023);
    else if (a == "--timeout-s") cfg.timeout_ms = (int)(val(1, 2000000) * 1000);
    else if (a == "--steps") steps = (int)val(1, 1 << 20);
    else if (a == "--no-tensor-cores") cfg.flags |= KVM_CFG_NO_TENSOR_CORES;
    else if (a == "--static") cfg.flags |= KVM_CFG_STATIC;
    else if (a == "--dynamic") cfg.flags |= KVM_CFG_DYNAMIC;
    else if (a == "--trace-csv") { if (i + 1 >= argc) { usage(); return 2; } csv = argv[++i]; }
    else if (a == "--golden") golden = true;
    else if (a == "--golden-tol") { if (i + 1 >= argc) { usage(); return 2; } golden_tol = atof(argv[++i]); }
    else if (a == "--dump-buffers") dump = true;
    else if (a == "--dump-bin") {
      if (i + 2 >= argc) { usage(); return 2; }
      dump_dir = argv[++i];
      for (char* p = argv[++i]; *p;) {
        char* e;
        const long v = strtol(p, &e, 10);
        if (e == p || v < 0) { usage(); return 2; }
        dump_idx.push_back((int)v);
        p = *e == ',' ? e + 1 : e;
      }
    }
    else if (a == "--quiet") g_log = 0;
    else if (a == "--check-ops") {
      for (int id = 0; id < 512; ++id) if (kvm_op_arity(id) >= 0) printf("%3d %-20s arity %d\n", id, kvm_op_name(id), kvm_op_arity(id));
      return 0;
    }
    else if (!a.empty() && a[0] == '-') { usage(); return 2; }
    else dirs.push_back(a);
  }
  if (dirs.empty()) { usage(); return 2; }
  if ((cfg.flags & KVM_CFG_STATIC) && (cfg.flags & KVM_CFG_DYNAMIC)) { KLOG(0, "--static and --dynamic exclude each other"); return 1; }
  if (golden && dirs.size() != 1) { KLOG(0, "--golden needs exactly one bundle directory"); return 1; }
  cfg.trace = (csv || golden) ? 1 : 0;

  KvmExec* h = nullptr;
  if (kvm_create(&cfg, &h) != 0 || !h) { KLOG(0, "cannot create the executor (no sm_100 GPU, or a CUDA error)"); return 1; }
  int rc = 1;
  do {
    bool loaded = true;
    for (auto& d : dirs)
      if (kvm_load_bundle_dir(h, d.c_str()) != 0) { KLOG(0, "%s", kvm_last_error(h)); loaded = false; break; }
    if (!loaded) break;
    KvmResult r{};
    const int status = steps > 1 ? kvm_run_steps(h, steps, &r) : kvm_run(h, &r);
    if (status != 0) KLOG(0, "%s", kvm_last_error(h));
    const bool ran_ok = status == 0 && r.status == 0 && r.done == r.admitted;
    const int nb = kvm_buffer_count(h);

    if (csv) {
      std::vector<uint64_t> s(r.admitted), e(r.admitted);
      std::vector<int32_t> sm(r.admitted);
      FILE* f = fopen(csv, "w");
      if (!f || kvm_trace(h, s.data(), e.data(), sm.data(), r.admitted) != 0) { KLOG(0, "--trace-csv: cannot write %s", csv); if (f) fclose(f); break; }
      fprintf(f, "task,start_ns,end_ns,smid\n");
      for (int i = 0; i < r.admitted; ++i) fprintf(f, "%d,%llu,%llu,%d\n", i, (unsigned long long)s[i], (unsigned long long)e[i], sm[i]);
      fclose(f);
    }

    auto read_buf = [&](int idx, std::vector<float>& out) {
      int32_t rows = 0, cols = 0, dt = 0;
      if (kvm_buffer_info(h, idx, &rows, &cols, &dt) != 0) return -1;
      out.resize((size_t)rows * cols);
      if (dt == KVM_I32) {           // raw integers, carried bit for bit in the float slots (as the reference's golden compare expects)
        if (kvm_read_buffer_raw(h, idx, out.data(), out.size() * 4, 0) != 0) return -1;
      } else if (kvm_read_buffer(h, idx, out.data(), out.size()) != 0) return -1;
      return (int)dt;
    };

    int golden_bad = 0;
    if (golden) {
      if (!ran_ok) { KLOG(0, "golden: skipped, the run failed"); }
      else {
        std::string text;
        if (!read_file(dirs[0] + "/golden.json", text)) { KLOG(0, "cannot read %s/golden.json", dirs[0].c_str()); break; }
        KvmJson g;
        try { g = KvmJsonParser(text).parse(); } catch (const std::exception& e) { KLOG(0, "golden.json: %s", e.what()); break; }
        long long values = 0, exact = 0;
        double worst = 0.0;
        if (const KvmJson* gb = g.get("buffers")) for (auto& kv : gb->o) {
          const int idx = kvm_buffer_index(h, kv.first.c_str());
          if (idx < 0) { KLOG(0, "golden: unknown buffer %s", kv.first.c_str()); ++golden_bad; continue; }
          std::vector<float> got;
          const int dt = read_buf(idx, got);
          if (dt < 0) { KLOG(0, "golden: cannot read buffer %s", kv.first.c_str()); ++golden_bad; continue; }
          if (got.size() != kv.second.a.size()) { KLOG(0, "golden: buffer %s has %zu values, golden %zu", kv.first.c_str(), got.size(), kv.second.a.size()); ++golden_bad; continue; }
          double num = 0, den = 0;
          size_t ndiff = 0;
          for (size_t i = 0; i < got.size(); ++i) {
            ++values;
            if (dt == KVM_I32) {
              int32_t gi; memcpy(&gi, &got[i], 4);
              if (gi == (int32_t)strtoll(kv.second.a[i].s.c_str(), nullptr, 10)) { ++exact; continue; }
              if (++ndiff <= 3) KLOG(0, "golden: %s[%zu] differs (i32)", kv.first.c_str(), i);
              ++golden_bad;
              continue;
            }
            const float want = (float)kv.second.a[i].n;
            if (memcmp(&got[i], &want, 4) == 0) { ++exact; den += (double)want * want; continue; }
            ++ndiff;
            num += ((double)got[i] - want) * ((double)got[i] - want);
            den += (double)want * want;
          }
          if (dt != KVM_I32) {
            const double rel = std::sqrt(num) / std::max(1e-30, std::sqrt(den));
            worst = std::max(worst, rel);
            if (!(rel <= golden_tol)) { KLOG(0, "golden: buffer %s: relative L2 error %.3g > %.3g (%zu of %zu elements differ)", kv.first.c_str(), rel, golden_tol, ndiff, got.size()); ++golden_bad; }
          }
        }
        if (const KvmJson* gv = g.get("versions")) for (auto& kv : gv->o) {
          const int id = kvm_variable_id(h, kv.first.c_str());
          int32_t got = -1;
          if (id >= 0) kvm_get_version(h, id, &got);
          if (got != (int32_t)kv.second.n) { KLOG(0, "golden: version %s = %d, golden %d", kv.first.c_str(), got, (int)kv.second.n); ++golden_bad; }
        }
        KLOG(2, "golden: %lld buffer values compared, %lld bitwise equal, worst buffer relative L2 error %.3g (tolerance %.3g)", values, exact, worst, golden_tol);
      }
    }
    if (dump) for (int i = 0; i < nb; ++i) {
      std::vector<float> v;
      const int dt = read_buf(i, v);
      printf("buffer %d:", i);
      for (float x : v) { if (dt == KVM_I32) { int32_t iv; memcpy(&iv, &x, 4); printf(" %d", iv); } else printf(" %.9g", x); }
      printf("\n");
    }
    bool dump_failed = false;
    for (int idx : dump_idx) {
      if (idx >= nb) { fprintf(stderr, "--dump-bin: buffer %d out of range (%d buffers)\n", idx, nb); kvm_destroy(h); return 2; }
      std::vector<float> v;
      const int dt = read_buf(idx, v);
      if (dt == KVM_I32) for (float& x : v) { int32_t iv; memcpy(&iv, &x, 4); x = (float)iv; }
      const std::string path = dump_dir + "/" + std::to_string(idx) + ".bin";
      FILE* f = fopen(path.c_str(), "wb");
      if (dt < 0 || !f || fwrite(v.data(), sizeof(float), v.size(), f) != v.size()) { fprintf(stderr, "--dump-bin: cannot write %s\n", path.c_str()); dump_failed = true; }
      if (f) fclose(f);
    }
    if (dump_failed) { kvm_destroy(h); return 2; }
    const bool pass = ran_ok && golden_bad == 0;
    printf("%s: %d/%d tasks, %.3f ms%s\n", pass ? "OK" : "FAIL", r.done, r.admitted, r.ms, golden ? (golden_bad || !ran_ok ? ", golden MISMATCH" : ", golden match") : "");
    rc = pass ? 0 : 1;
  } while (false);
  kvm_destroy(h);
  return rc;
}
