// Host side of the static-schedule path: turn the resident program into per-worker task lists with cross-worker dependency
// entries.  What it implements of the reference: mvm_static_plan / layout / emit (include/mvm_static.h:150-356: list schedule by
// estimated cost, earliest-finish placement, per-record watermark waits) and the feasibility rule of its CLI
// (mvm_exec.cu:2085-2110: every version wait must be ordered inside the bundle or met by the base versions).
//
// Planning order: ready tasks by (priority class, higher first; then submission index), each placed on the worker where it can
// start earliest (ties: the least loaded worker).  A task's dependency list holds, per worker that ran one of its predecessors,
// how many tasks that worker must have finished; identical lists are stored once.

#include <queue>
#include <unordered_map>

// Estimated duration of a task in microseconds: bytes over one SM's share of HBM for the memory-bound ops, FLOPs over one SM's
// tensor / FMA rate for the contractions, plus a fixed cost.  Only relative sizes matter (the plan balances the workers with it).
static double kvm_static_cost(const KvmExec* h, const KvmTaskDesc& d, const int32_t* a) {
  const double BPU = 40000.0;                 // bytes per microsecond per SM (HBM share)
  auto elems = [&](int e0, int e1) { return (double)(e1 > e0 ? e1 - e0 : 0); };
  switch (d.op_id) {
    case 0: return 0.2;
    case 134: case 301: return 8.0 + elems(a[6], a[7]) * a[8] * 2.0 / BPU;     // fixed part measured: prologue and hand-over of a streamed task
    case 135: case 300: { const double keys = a[10] > 0 ? (double)a[14] / a[10] : a[14]; return 14.0 + 2.0 * keys * a[13] * 2.0 / BPU; }
    case 136: return 8.0;                     // a few dependent round trips, measured
    case 58: case 57: return 2.0 + elems(a[d.op_id == 58 ? 2 : 3], a[d.op_id == 58 ? 3 : 4]) * a[d.op_id == 58 ? 4 : 5] * 4.0 / BPU;
    case 122: { const double m = std::min(128, a[8] - a[6]), n = std::min(256, a[9] - a[7]); return 5.0 + 2.0 * m * n * a[10] / 8.0e6; }
    case 34: case 114: { const int tm = (a[11] & 64) ? 256 : (a[11] & 32) ? 128 : 64, tn = (a[11] & 64) ? 128 : (a[11] & 32) ? 128 : 64;
      const double m = std::min(tm, a[8] - a[6]), n = std::min(tn, a[9] - a[7]); return 2.0 + 2.0 * m * n * a[10] / 0.2e6; }
    case 8: return 2.0 + 2.0 * (double)a[3] * a[4] * a[5] / 0.2e6;
    case 45: return 4.0 + 4.0 * 128.0 * (a[7] + 64.0) * a[11] / 3.0e6;
    case 47: return 4.0 + 5.0 * 128.0 * (a[9] + 64.0) * a[13] / 3.0e6;
    case 48: return 4.0 + 5.0 * 128.0 * std::max(64.0, (double)a[11] - a[10] - 64.0) * a[13] / 3.0e6;
    case 46: return 2.0 + elems(a[3], a[4]) * a[6] * a[7] * 4.0 / BPU;
    case 35: case 36: case 37: case 38: { const int r0 = a[d.op_id == 36 ? 4 : 6], r1 = a[d.op_id == 36 ? 5 : 7], dd = a[d.op_id == 36 ? 6 : 8];
      return 2.0 + elems(r0, r1) * dd * 10.0 / BPU; }
    case 39: return 2.0 + (double)a[6] * elems(a[8], a[9]) * 8.0 / BPU;
    case 61: return 2.0 + (double)a[2] * elems(a[3], a[4]) * 4.0 / BPU;
    case 51: case 53: case 127: { const int r0 = a[d.op_id == 51 ? 4 : 5], r1 = a[d.op_id == 51 ? 5 : 6], V = a[d.op_id == 51 ? 6 : 7]; return 2.0 + elems(r0, r1) * V * 6.0 / BPU; }
    case 54: case 115: return 2.0 + elems(a[6], a[7]) * 28.0 / BPU;
    case 55: return 1.5 + elems(a[3], a[4]) * 4.0 / BPU;
    case 32: return 2.0 + elems(a[4], a[5]) * a[7] * 8.0 / BPU;
    case 33: return 3.0 + (double)a[3] * 4.0 / BPU + elems(a[5], a[6]) * a[7] * 8.0 / BPU;
    case 40: case 41: case 42: case 113: case 117: case 126: case 96: case 97: case 98: case 123: case 59: {
      const int w = d.args_words;             // flat ops end with (..., e0, e1) or (e0, e1, acc / kind-dependent)
      double n = 0;
      for (int k = 0; k + 1 < w; ++k) if (a[k + 1] > a[k] && a[k] >= 0 && (double)a[k + 1] - a[k] > n && a[k + 1] < (1 << 30)) n = (double)a[k + 1] - a[k];
      return 1.5 + n * 12.0 / BPU; }
    default: return 3.0;
  }
  (void)h;
}

// Buffers some task of the batch may write.  Everything a task names counts as written unless the (op, argument) pair is known
// to be read-only; the streamed operands of decode (weights of gemv_bf16, caches of attn_decode_part, which only adds the one
// row its own copy leaves out) are what this is for.
static std::vector<char> kvm_written_buffers(const KvmExec* h) {
  std::vector<char> wr(h->bufs.size(), 0);
  for (const KvmTaskDesc& d : h->tasks) {
    const KvmOpInfo* op = kvm_find_op(d.op_id);
    if (!op) continue;
    const int32_t* a = h->args.data() + d.args_off;
    for (int j = 0; j < op->arity; ++j) {
      if (op->types[j] < 2 || a[j] < 0 || a[j] >= (int)wr.size()) continue;
      bool read_only = false;
      switch (d.op_id) {
        case 134: case 301: read_only = j != 4; break;                // x, x2, gamma, w, res
        case 135: case 300: read_only = j != 4; break;                // q, kc, vc, lens, knew, vnew, qk_gamma (kc / vc: own appended row only)
        case 136: read_only = j == 0; break;
        case 63: read_only = j != 2; break;
        case 58: read_only = j == 0; break;
        case 57: read_only = j == 0 || j == 2; break;
        case 36: read_only = j <= 1; break;
        case 98: read_only = j <= 1; break;
        default: break;
      }
      if (!read_only) wr[a[j]] = 1;
    }
  }
  return wr;
}

// Plan the resident program.  Returns 0 and fills `plan`, or KVM_E_STATE with the reason in h->error when the program cannot run
// statically (a version wait that nothing in the program and no base version satisfies).
static int kvm_plan_static(KvmExec* h, const std::vector<int>& base_versions, KvmStaticPlan& plan) {
  const int nt = (int)h->tasks.size(), W = h->workers;
  // a dependency list has one entry per worker at most, and the front warp holds 5 x 32 of them
  if (W > 160 || nt >= (1 << KVM_ST_WAIT_BITS)) { h->error = "static path: too many workers or tasks for the dependency encoding"; return KVM_E_STATE; }
  // predecessors: in-batch edges plus version waits turned into edges on their publisher
  std::vector<std::vector<int>> preds(nt);
  std::vector<int> indeg(nt, 0);
  for (int i = 0; i < nt; ++i) {
    const KvmTaskDesc& d = h->tasks[i];
    for (int k = 0; k < d.succ_cnt; ++k) preds[h->succ[d.succ_off + k]].push_back(i);
  }
  std::vector<std::vector<int>> extra_succ(nt);
  for (int i = 0; i < nt; ++i) {
    const KvmTaskDesc& d = h->tasks[i];
    if (d.wait_var < 0) continue;
    if (d.wait_var < (int)base_versions.size() && d.wait_ver <= base_versions[d.wait_var]) continue;      // met before the launch
    int pub = -1;
    for (int p = 0; p < nt; ++p) if (h->tasks[p].pub_var == d.wait_var && h->tasks[p].pub_ver == d.wait_ver) { pub = p; break; }
    if (pub < 0) {
      char m[160];
      snprintf(m, sizeof m, "static path: task %d waits for version %d of variable %d, which no task of the program publishes (the ready-queue path parks such tasks)", i, d.wait_ver, d.wait_var);
      h->error = m;
      return KVM_E_STATE;
    }
    preds[i].push_back(pub);
    extra_succ[pub].push_back(i);
  }
  for (int i = 0; i < nt; ++i) indeg[i] = (int)preds[i].size();

  std::vector<double> cost(nt), finish(nt, 0.0), avail(W, 0.0);
  std::vector<int> worker(nt, -1), pos(nt, 0), count(W, 0);
  for (int i = 0; i < nt; ++i) cost[i] = kvm_static_cost(h, h->tasks[i], h->args.data() + h->tasks[i].args_off);
  typedef std::pair<int, int> Key;      // (-priority class, index): smallest first
  std::priority_queue<Key, std::vector<Key>, std::greater<Key>> ready;
  auto cls = [&](int i) { const int p = h->tasks[i].priority; return p < 0 ? 0 : (p >> 3) >= KVM_NCLASS ? KVM_NCLASS - 1 : (p >> 3); };
  for (int i = 0; i < nt; ++i) if (!indeg[i]) ready.push({-cls(i), i});
  std::vector<std::vector<int>> lists(W);
  int placed = 0;
  const double comm = 1.5;                     // microseconds until another worker sees a progress word
  while (!ready.empty()) {
    const int t = ready.top().second;
    ready.pop();
    double dr = 0.0;                           // when the predecessors' results are there
    int crit = -1;
    for (int p : preds[t]) if (finish[p] > dr) { dr = finish[p]; crit = worker[p]; }
    int best = 0;
    double best_start = 1e300, best_avail = 1e300;
    for (int w = 0; w < W; ++w) {
      const double start = std::max(avail[w], w == crit ? dr : dr + (preds[t].empty() ? 0.0 : comm));
      if (start < best_start - 1e-9 || (start < best_start + 1e-9 && avail[w] < best_avail)) { best = w; best_start = start; best_avail = avail[w]; }
    }
    worker[t] = best; pos[t] = count[best]++;
    lists[best].push_back(t);
    finish[t] = best_start + cost[t];
    avail[best] = finish[t];
    ++placed;
    const KvmTaskDesc& d = h->tasks[t];
    for (int k = 0; k < d.succ_cnt; ++k) { const int s = h->succ[d.succ_off + k]; if (--indeg[s] == 0) ready.push({-cls(s), s}); }
    for (int s : extra_succ[t]) if (--indeg[s] == 0) ready.push({-cls(s), s});
  }
  if (placed != nt) { h->error = "static path: dependency cycle"; return KVM_E_STATE; }
  plan.makespan_us = 0.0;
  for (int w = 0; w < W; ++w) plan.makespan_us = std::max(plan.makespan_us, avail[w]);

  plan.prog.clear(); plan.prog_off.assign(W + 1, 0);
  for (int w = 0; w < W; ++w) { plan.prog_off[w] = (int)plan.prog.size(); plan.prog.insert(plan.prog.end(), lists[w].begin(), lists[w].end()); }
  plan.prog_off[W] = (int)plan.prog.size();

  // dependency lists: per worker the count it must have reached; own-worker entries stay in (they cost nothing at run time: a
  // worker's tasks finish in list order) so that the tasks of one phase share one list
  plan.waits.clear(); plan.wait_off.assign(nt, 0); plan.wait_cnt.assign(nt, 0);
  struct VecHash { size_t operator()(const std::vector<int>& v) const { size_t hh = 1469598103934665603ull; for (int x : v) { hh ^= (size_t)(unsigned)x; hh *= 1099511628211ull; } return hh; } };
  std::unordered_map<std::vector<int>, int, VecHash> seen;
  std::vector<int> need(W), touched;
  for (int t = 0; t < nt; ++t) {
    touched.clear();
    for (int p : preds[t]) {
      const int w = worker[p];
      if (need[w] == 0) touched.push_back(w);
      need[w] = std::max(need[w], pos[p] + 1);
    }
    std::sort(touched.begin(), touched.end());
    std::vector<int> lst;
    lst.reserve(touched.size());
    for (int w : touched) { lst.push_back((w << KVM_ST_WAIT_BITS) | need[w]); need[w] = 0; }
    auto it = seen.find(lst);
    if (it == seen.end()) {
      it = seen.emplace(lst, (int)plan.waits.size()).first;
      plan.waits.insert(plan.waits.end(), lst.begin(), lst.end());
    }
    plan.wait_off[t] = it->second; plan.wait_cnt[t] = (int)lst.size();
  }

  // streaming: which tasks may copy ahead of their dependencies, and whether the launch carries the stage ring at all
  plan.stream.assign(nt, 0);
  const std::vector<char> written = kvm_written_buffers(h);
  const int nb = (int)written.size();
  // A split-attention task reads its length counter ahead of time (the front warp sizes the copies with it).  That is the value
  // the task itself would read only if every task that may change the counter comes after the reader: for each written counter,
  // the readers that are direct predecessors of ALL its other users.
  std::vector<std::vector<int>> len_readers(nb), len_users(nb);
  for (int t = 0; t < nt; ++t) if (h->tasks[t].op_id == 135 || h->tasks[t].op_id == 300) { const int L = h->args[h->tasks[t].args_off + 3]; if (L >= 0 && L < nb && written[L]) len_readers[L].push_back(t); }
  for (int u = 0; u < nt; ++u) {
    const KvmTaskDesc& du = h->tasks[u];
    const KvmOpInfo* op = kvm_find_op(du.op_id);
    if (!op || du.op_id == 134 || du.op_id == 301 || du.op_id == 135 || du.op_id == 300) continue;
    const int32_t* au = h->args.data() + du.args_off;
    for (int j = 0; j < op->arity; ++j) if (op->types[j] >= 2 && au[j] >= 0 && au[j] < nb && !len_readers[au[j]].empty()) { len_users[au[j]].push_back(u); break; }
  }
  std::vector<char> len_ok(nt, 1), mark(nt, 0);
  for (int L = 0; L < nb; ++L) for (int u : len_users[L]) {
    for (int p : preds[u]) mark[p] = 1;
    for (int t : len_readers[L]) if (!mark[t]) len_ok[t] = 0;
    for (int p : preds[u]) mark[p] = 0;
  }
  bool any_stream = false, all_fit = true, any_rows = false;
  for (int t = 0; t < nt; ++t) {
    const KvmTaskDesc& d = h->tasks[t];
    const int32_t* a = h->args.data() + d.args_off;
    if (d.op_id == 134 || d.op_id == 301) {
      any_stream = true;
      if (d.op_id == 301) any_rows = true;
      const int K = a[8];
      if (K <= 0 || (K & 255) || K * 2 > KVM_ST_STAGE) all_fit = false;       // such a row does not stream through a stage: run the whole program without the ring
      if (a[3] >= 0 && a[3] < nb && !written[a[3]]) plan.stream[t] = 1;
    } else if (d.op_id == 135 || d.op_id == 300) {
      if (a[1] >= 0 && a[2] >= 0 && a[3] >= 0 && a[1] < nb && a[2] < nb && a[3] < nb && !written[a[1]] && !written[a[2]] && len_ok[t]) plan.stream[t] = 1;
    }
  }
  plan.ring = !(any_stream && all_fit) ? 0 : any_rows ? 2 : 1;
  return 0;
}
