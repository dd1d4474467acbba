// Host state and the C entry points (included by kvm_exec.cu).

#define KVM_CUDA(call)                                                                         \
  do {                                                                                         \
    cudaError_t e_ = (call);                                                                   \
    if (e_ != cudaSuccess) { h->error = std::string(#call) + ": " + cudaGetErrorString(e_); return KVM_E_CUDA; } \
  } while (0)

struct KvmOwned { void* p; size_t bytes; };

// Result of the host planner of the static-schedule path (kvm_static_host.inl).
struct KvmStaticPlan {
  std::vector<int> prog, prog_off, waits;
  std::vector<int> wait_off, wait_cnt, stream;      // per task
  int ring = 0;                                     // 0 no stream ring; 1 three stages (decode programs); 2 two stages and a large scratch (programs with gemv_bf16_rows)
  double makespan_us = 0.0;                         // the planner's estimate of one run
};

struct KvmExec {
  KvmConfig cfg{};
  int device = 0, sms = 0, workers = 0, smem_bytes = 0, nvars = 64;
  std::string error;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  // buffer table
  std::vector<KvmBuf> bufs;
  std::vector<KvmOwned> owned;
  KvmBuf* d_bufs = nullptr; size_t d_bufs_cap = 0; bool bufs_dirty = true;
  // tasks (all submitted batches, successor indices already global)
  std::vector<KvmTaskDesc> tasks;
  std::vector<int32_t> succ, args;
  std::vector<int4> aux;
  std::vector<CUtensorMap> tmaps;
  bool tasks_dirty = true;
  KvmTaskDesc* d_tasks = nullptr; int32_t* d_succ = nullptr; int32_t* d_args = nullptr; int4* d_aux = nullptr; void* d_tmaps = nullptr; int32_t* d_recs = nullptr;
  int *d_indeg = nullptr, *d_exec = nullptr, *d_ring = nullptr, *d_park_next = nullptr, *d_tsmid = nullptr, *d_claim = nullptr;
  unsigned long long *d_tstart = nullptr, *d_tend = nullptr;
  size_t task_cap = 0;
  // control words
  int* d_ctl = nullptr;          // [0] head [1] tail [2] done
  int* d_versions = nullptr; int* d_park_head = nullptr; int* d_ver_base = nullptr; int* d_ver_off = nullptr;
  KvmErrRec* d_err = nullptr;
  bool started = false, armed = false;
  bool has_gemv = false;         // a submitted task is a gemv_bf16: its shared-memory ring is worth more than the buffer-table cache
  bool own_stream = true;        // false after kvm_set_stream: the caller's stream is used and never destroyed here
  bool use_static = false;       // the resident program runs as per-worker lists (kvm_static.cuh); decided when the tasks are uploaded
  KvmStaticPlan splan;
  int *d_prog = nullptr, *d_prog_off = nullptr, *d_waits = nullptr, *d_progress = nullptr;
  std::vector<std::string> buf_names;              // by buffer index; "" where the caller gave none (kvm_load_bundle_dir fills them from metadata.json)
  std::map<std::string, int> var_ids;              // version variables by name (from metadata.json)
  KvmResult last{};
};

// Stacked GEMM tiles are opt-in (KVM_CFG_PAIR_TILES); the environment variable KVM_B200_PAIRING (0 or 1) overrides the
// flag for A/B measurements, KVM_B200_PAIR_DEPTH the queue depth from which tiles are stacked.
static bool kvm_feature_on(const char* env, int dflt) {
  const char* v = getenv(env);
  return v && *v ? atoi(v) != 0 : dflt != 0;
}

static void kvm_free_tasks(KvmExec* h) {
  for (void* p : {(void*)h->d_tasks, (void*)h->d_succ, (void*)h->d_args, (void*)h->d_aux, (void*)h->d_tmaps, (void*)h->d_indeg, (void*)h->d_exec, (void*)h->d_ring,
                  (void*)h->d_park_next, (void*)h->d_tsmid, (void*)h->d_tstart, (void*)h->d_tend, (void*)h->d_recs, (void*)h->d_claim, (void*)h->d_prog, (void*)h->d_prog_off,
                  (void*)h->d_waits, (void*)h->d_progress})
    if (p) cudaFree(p);
  h->d_prog = h->d_prog_off = h->d_waits = h->d_progress = nullptr;
  h->d_tasks = nullptr; h->d_succ = nullptr; h->d_args = nullptr; h->d_aux = nullptr; h->d_tmaps = nullptr; h->d_indeg = h->d_exec = h->d_ring = h->d_park_next = h->d_tsmid = nullptr;
  h->d_tstart = h->d_tend = nullptr; h->d_recs = nullptr; h->d_claim = nullptr; h->task_cap = 0;
}

extern "C" const char* kvm_err_name(int32_t code) {
  static const char* names[] = {
#define E(n) #n,
      KVM_ERRORS(E)
#undef E
  };
  if (code >= 0 && code < KVM_ERR_COUNT) return names[code];
  switch (code) {
    case KVM_OPE_BUF: return "E_BUF"; case KVM_OPE_DTYPE: return "E_DTYPE"; case KVM_OPE_RANGE: return "E_RANGE"; case KVM_OPE_SHAPE: return "E_SHAPE";
    case KVM_OPE_TOKEN: return "E_TOKEN"; case KVM_OPE_KVLEN: return "E_KVLEN"; case KVM_OPE_SMEM: return "E_SMEM";
    case KVM_E_ARG: return "KVM_E_ARG"; case KVM_E_CUDA: return "KVM_E_CUDA"; case KVM_E_BUNDLE: return "KVM_E_BUNDLE"; case KVM_E_STATE: return "KVM_E_STATE";
    case KVM_E_NOMEM: return "KVM_E_NOMEM"; case KVM_E_IO: return "KVM_E_IO";
  }
  return "UNKNOWN";
}
extern "C" int kvm_op_arity(int32_t op_id) { const KvmOpInfo* o = kvm_find_op(op_id); return o ? o->arity : -1; }
extern "C" const char* kvm_op_name(int32_t op_id) { const KvmOpInfo* o = kvm_find_op(op_id); return o ? o->name : nullptr; }
extern "C" const char* kvm_last_error(KvmExec* h) { return h ? h->error.c_str() : "null handle"; }

extern "C" int kvm_create(const KvmConfig* cfg, KvmExec** out) {
  if (!out) return KVM_E_ARG;
  *out = nullptr;
  KvmExec* h = new KvmExec();
  if (cfg) h->cfg = *cfg;
  h->device = h->cfg.device;
  auto fail = [&](const char* what, cudaError_t e) {
    fprintf(stderr, "kvm_create: %s: %s\n", what, cudaGetErrorString(e));
    if (h->ev0) cudaEventDestroy(h->ev0);
    if (h->ev1) cudaEventDestroy(h->ev1);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return KVM_E_CUDA;
  };
  cudaError_t e;
  if ((e = cudaSetDevice(h->device)) != cudaSuccess) return fail("cudaSetDevice", e);
  cudaDeviceProp prop;
  if ((e = cudaGetDeviceProperties(&prop, h->device)) != cudaSuccess) return fail("cudaGetDeviceProperties", e);
  if (prop.major != 10) { fprintf(stderr, "kvm_create: device %d is sm_%d%d; this library holds sm_100a code only\n", h->device, prop.major, prop.minor); delete h; return KVM_E_CUDA; }
  h->sms = prop.multiProcessorCount;
  h->workers = h->cfg.workers > 0 ? h->cfg.workers : h->sms;
  if (h->workers > h->sms) h->workers = h->sms;      // one CTA per SM: more could not be co-resident, and waiting CTAs need their peers running
  h->smem_bytes = (int)prop.sharedMemPerBlockOptin;
  h->nvars = h->cfg.num_vars > 0 ? h->cfg.num_vars : 64;
  if ((e = cudaFuncSetAttribute(kvm_exec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h->smem_bytes)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = kvm_static_set_smem(h->smem_bytes)) != cudaSuccess) return fail("cudaFuncSetAttribute", e);
  if ((e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail("cudaStreamCreate", e);
  if ((e = cudaEventCreate(&h->ev0)) != cudaSuccess || (e = cudaEventCreate(&h->ev1)) != cudaSuccess) return fail("cudaEventCreate", e);
  if ((e = cudaMalloc(&h->d_ctl, 64 * sizeof(int))) != cudaSuccess || (e = cudaMalloc(&h->d_versions, h->nvars * sizeof(int))) != cudaSuccess ||
      (e = cudaMalloc(&h->d_park_head, h->nvars * sizeof(int))) != cudaSuccess || (e = cudaMalloc(&h->d_ver_base, h->nvars * sizeof(int))) != cudaSuccess ||
      (e = cudaMalloc(&h->d_ver_off, h->nvars * sizeof(int))) != cudaSuccess || (e = cudaMalloc(&h->d_err, sizeof(KvmErrRec))) != cudaSuccess) {
    for (void* p : {(void*)h->d_ctl, (void*)h->d_versions, (void*)h->d_park_head, (void*)h->d_ver_base, (void*)h->d_ver_off, (void*)h->d_err}) if (p) cudaFree(p);
    return fail("cudaMalloc", e);
  }
  if ((e = cudaMemset(h->d_versions, 0, h->nvars * sizeof(int))) != cudaSuccess || (e = cudaMemset(h->d_err, 0, sizeof(KvmErrRec))) != cudaSuccess ||
      (e = cudaMemset(h->d_ctl, 0, 64 * sizeof(int))) != cudaSuccess) return fail("cudaMemset", e);
  if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail("init", e);
  *out = h;
  return 0;
}

extern "C" void kvm_destroy(KvmExec* h) {
  if (!h) return;
  cudaSetDevice(h->device);
  cudaStreamSynchronize(h->stream);
  for (auto& o : h->owned) cudaFree(o.p);
  kvm_free_tasks(h);
  for (void* p : {(void*)h->d_bufs, (void*)h->d_ctl, (void*)h->d_versions, (void*)h->d_park_head, (void*)h->d_ver_base, (void*)h->d_ver_off, (void*)h->d_err}) if (p) cudaFree(p);
  if (h->ev0) cudaEventDestroy(h->ev0);
  if (h->ev1) cudaEventDestroy(h->ev1);
  if (h->stream && h->own_stream) cudaStreamDestroy(h->stream);
  delete h;
}

static size_t kvm_elem_bytes(int dtype) { return dtype == KVM_BF16 ? 2 : 4; }

extern "C" int kvm_add_buffer(KvmExec* h, int32_t rows, int32_t cols, int32_t dtype, const KvmInit* init) {
  if (!h) return KVM_E_ARG;
  if (rows < 1 || cols < 1 || dtype < 0 || dtype > 2 || (long long)rows * cols > 2147483647LL) { h->error = "kvm_add_buffer: bad shape or dtype"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  const size_t n = (size_t)rows * cols, bytes = n * kvm_elem_bytes(dtype);
  void* p = nullptr;
  if (cudaMalloc(&p, bytes < 256 ? 256 : bytes) != cudaSuccess) { cudaGetLastError(); h->error = "kvm_add_buffer: out of device memory"; return KVM_E_NOMEM; }
  const int kind = init ? init->kind : KVM_INIT_FILL;
  const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
  if (kind == KVM_INIT_FILL) kvm_fill_kernel<<<blocks, 256, 0, h->stream>>>(p, n, dtype, init ? init->fill : 0.0);
  else if (kind == KVM_INIT_VALUES) {
    if (!init->data) { cudaFree(p); h->error = "kvm_add_buffer: VALUES init without data"; return KVM_E_ARG; }
    KVM_CUDA(cudaMemcpyAsync(p, init->data, bytes, cudaMemcpyHostToDevice, h->stream));
    KVM_CUDA(cudaStreamSynchronize(h->stream));
  } else if (kind == KVM_INIT_SEEDED) {
    if (dtype == KVM_I32 || (init->draws != 1 && init->draws != 4)) { cudaFree(p); h->error = "kvm_add_buffer: seeded init needs f32 or bf16 storage and draws 1 or 4"; return KVM_E_ARG; }
    kvm_seeded_kernel<<<blocks, 256, 0, h->stream>>>(p, n, init->seed, init->draws, init->bias, init->coef, dtype);
  } else if (kind != KVM_INIT_NONE) { cudaFree(p); h->error = "kvm_add_buffer: unknown init kind"; return KVM_E_ARG; }
  KVM_CUDA(cudaGetLastError());
  KvmBuf b{p, rows, cols, cols, dtype, {0, 0}};
  h->bufs.push_back(b);
  h->owned.push_back({p, bytes});
  h->bufs_dirty = true;
  return (int)h->bufs.size() - 1;
}

extern "C" int kvm_bind_buffer(KvmExec* h, void* dev_ptr, int32_t rows, int32_t cols, int32_t ld, int32_t dtype) {
  if (!h || !dev_ptr || rows < 1 || cols < 1 || ld < cols || dtype < 0 || dtype > 2) { if (h) h->error = "kvm_bind_buffer: bad argument"; return KVM_E_ARG; }
  KvmBuf b{dev_ptr, rows, cols, ld, dtype, {0, 0}};
  h->bufs.push_back(b);
  h->bufs_dirty = true;
  return (int)h->bufs.size() - 1;
}

// Sharing a buffer with an executor in another process on the same node (the inbox and flag words of the peer exchange ops):
// the owner exports a 64-byte handle of the buffer's allocation, the peer maps it and binds the pointer as one of its own
// table entries (kvm_bind_buffer).  Owned buffers are allocations of their own, so the handle addresses exactly the buffer.
extern "C" int kvm_ipc_export(KvmExec* h, int32_t idx, void* handle64) {
  if (!h || !handle64 || idx < 0 || idx >= (int)h->bufs.size()) { if (h) h->error = "kvm_ipc_export: bad argument"; return KVM_E_ARG; }
  bool owned = false;
  for (auto& o : h->owned) if (o.p == h->bufs[idx].p) owned = true;
  if (!owned) { h->error = "kvm_ipc_export: only buffers this executor allocated can be exported"; return KVM_E_ARG; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaSetDevice(h->device);
  KVM_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, h->bufs[idx].p));
  return 0;
}
extern "C" int kvm_ipc_open(KvmExec* h, const void* handle64, void** out) {
  if (!h || !handle64 || !out) { if (h) h->error = "kvm_ipc_open: bad argument"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle64, sizeof hd);
  KVM_CUDA(cudaIpcOpenMemHandle(out, hd, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
extern "C" int kvm_ipc_close(KvmExec* h, void* ptr) {
  if (!h || !ptr) return KVM_E_ARG;
  cudaSetDevice(h->device);
  KVM_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

extern "C" void* kvm_buffer_ptr(KvmExec* h, int32_t idx) { return (h && idx >= 0 && idx < (int)h->bufs.size()) ? h->bufs[idx].p : nullptr; }

static int kvm_buf_span(KvmExec* h, int idx, size_t bytes, size_t offset) {
  if (!h || idx < 0 || idx >= (int)h->bufs.size()) { if (h) h->error = "buffer index out of range"; return KVM_E_ARG; }
  const KvmBuf& b = h->bufs[idx];
  if (offset + bytes > (size_t)b.rows * b.ld * kvm_elem_bytes(b.dtype)) { h->error = "buffer copy out of range"; return KVM_E_ARG; }
  return 0;
}
extern "C" int kvm_write_buffer(KvmExec* h, int32_t idx, const void* host, size_t bytes, size_t offset) {
  if (int r = kvm_buf_span(h, idx, bytes, offset)) return r;
  cudaSetDevice(h->device);
  KVM_CUDA(cudaMemcpyAsync((char*)h->bufs[idx].p + offset, host, bytes, cudaMemcpyHostToDevice, h->stream));
  return 0;     // ordered before the next launch on the same stream; the source must stay valid until then (pinned) or is staged by CUDA (pageable)
}
extern "C" int kvm_read_buffer_raw(KvmExec* h, int32_t idx, void* host, size_t bytes, size_t offset) {
  if (int r = kvm_buf_span(h, idx, bytes, offset)) return r;
  cudaSetDevice(h->device);
  KVM_CUDA(cudaMemcpyAsync(host, (const char*)h->bufs[idx].p + offset, bytes, cudaMemcpyDeviceToHost, h->stream));
  KVM_CUDA(cudaStreamSynchronize(h->stream));
  return 0;
}
extern "C" int kvm_read_buffer(KvmExec* h, int32_t idx, float* out, size_t n) {
  if (!h || idx < 0 || idx >= (int)h->bufs.size() || !out) { if (h) h->error = "kvm_read_buffer: bad argument"; return KVM_E_ARG; }
  const KvmBuf& b = h->bufs[idx];
  if (b.ld != b.cols || n > (size_t)b.rows * b.cols) { h->error = "kvm_read_buffer: range"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  if (b.dtype == KVM_F32) { KVM_CUDA(cudaMemcpyAsync(out, b.p, n * 4, cudaMemcpyDeviceToHost, h->stream)); KVM_CUDA(cudaStreamSynchronize(h->stream)); return 0; }
  float* tmp = nullptr;
  KVM_CUDA(cudaMalloc(&tmp, n * 4));
  kvm_widen_kernel<<<(int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048), 256, 0, h->stream>>>(b.p, tmp, n, b.dtype);
  cudaError_t e = cudaMemcpyAsync(out, tmp, n * 4, cudaMemcpyDeviceToHost, h->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  cudaFree(tmp);
  KVM_CUDA(e);
  return 0;
}

extern "C" int kvm_set_version(KvmExec* h, int32_t var, int32_t version) {
  if (!h || var < 0 || var >= h->nvars || version < 0) { if (h) h->error = "kvm_set_version: bad variable"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  KVM_CUDA(cudaMemcpyAsync(h->d_versions + var, &version, 4, cudaMemcpyHostToDevice, h->stream));
  KVM_CUDA(cudaStreamSynchronize(h->stream));
  return 0;
}
extern "C" int kvm_get_version(KvmExec* h, int32_t var, int32_t* version) {
  if (!h || var < 0 || var >= h->nvars || !version) { if (h) h->error = "kvm_get_version: bad variable"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  KVM_CUDA(cudaMemcpyAsync(version, h->d_versions + var, 4, cudaMemcpyDeviceToHost, h->stream));
  KVM_CUDA(cudaStreamSynchronize(h->stream));
  return 0;
}

// The host check of MvmBundle::validate (mvm_exec.cu:141-208): first problem as text, "" if well formed.
static std::string kvm_validate(const KvmTaskDesc* t, int nt, const int32_t* succ, int ne, const int32_t* args, int na, int nbufs, int nvars) {
  char m[256];
  if (nt <= 0) return "empty bundle";
  std::vector<int> in(nt, 0);
  for (int i = 0; i < nt; ++i) {
    const KvmTaskDesc& d = t[i];
    const KvmOpInfo* op = kvm_find_op(d.op_id);
    if (!op) { snprintf(m, sizeof m, "task %d: bad op_id %d", i, d.op_id); return m; }
    if (d.args_words != op->arity) { snprintf(m, sizeof m, "task %d: %s takes %d args, got %d", i, op->name, op->arity, d.args_words); return m; }
    if (d.args_off < 0 || (long long)d.args_off + d.args_words > na) { snprintf(m, sizeof m, "task %d: args range", i); return m; }
    if (d.succ_off < 0 || d.succ_cnt < 0 || (long long)d.succ_off + d.succ_cnt > ne) { snprintf(m, sizeof m, "task %d: successor range", i); return m; }
    if (d.priority < 0 || d.priority >= 32) { snprintf(m, sizeof m, "task %d: priority %d outside [0,31]", i, d.priority); return m; }
    if (d.deadline_us < -1) { snprintf(m, sizeof m, "task %d: deadline_us", i); return m; }
    for (int v : {d.wait_var, d.pub_var}) if (v < -1 || v >= nvars) { snprintf(m, sizeof m, "task %d: version variable %d out of range", i, v); return m; }
    if ((d.wait_var >= 0 && d.wait_ver < 0) || (d.pub_var >= 0 && d.pub_ver < 1)) { snprintf(m, sizeof m, "task %d: wait_ver >= 0 and pub_ver >= 1 (0 is the initial state)", i); return m; }
    for (int j = 0; j < op->arity; ++j)
      if (op->types[j] >= 2) {
        const int b = args[d.args_off + j];
        if ((b == -1 && op->types[j] == 2) || b < -1 || b >= nbufs) { snprintf(m, sizeof m, "task %d: %s arg %d buffer index %d out of range", i, op->name, j, b); return m; }
      }
    for (int k = 0; k < d.succ_cnt; ++k) {
      const int s = succ[d.succ_off + k];
      if (s < 0 || s >= nt || s == i) { snprintf(m, sizeof m, "task %d: successor %d out of range", i, s); return m; }
      ++in[s];
    }
  }
  for (int i = 0; i < nt; ++i) if (in[i] != t[i].indegree) { snprintf(m, sizeof m, "task %d: indegree %d != in-edges %d", i, t[i].indegree, in[i]); return m; }
  std::vector<int> q, rem = in;
  q.reserve(nt);
  for (int i = 0; i < nt; ++i) if (!rem[i]) q.push_back(i);
  for (size_t x = 0; x < q.size(); ++x) {
    const KvmTaskDesc& d = t[q[x]];
    for (int k = 0; k < d.succ_cnt; ++k) if (--rem[succ[d.succ_off + k]] == 0) q.push_back(succ[d.succ_off + k]);
  }
  if ((int)q.size() != nt) return "dependency cycle";
  // version waits decidable inside the batch: publisher -> waiter edges must keep the graph acyclic
  std::vector<std::pair<int, int>> extra;
  for (int i = 0; i < nt; ++i) if (t[i].wait_var >= 0)
    for (int p = 0; p < nt; ++p) if (t[p].pub_var == t[i].wait_var && t[p].pub_ver <= t[i].wait_ver) {
      if (p == i) { snprintf(m, sizeof m, "task %d: waits for version %d of variable %d that it publishes itself", i, t[i].wait_ver, t[i].wait_var); return m; }
      extra.push_back({p, i});
    }
  if (!extra.empty()) {
    std::vector<int> deg = in;
    std::vector<std::vector<int>> xs(nt);
    for (auto& e : extra) { ++deg[e.second]; xs[e.first].push_back(e.second); }
    std::vector<int> st;
    int seen = 0;
    for (int i = 0; i < nt; ++i) if (!deg[i]) st.push_back(i);
    while (!st.empty()) {
      const int u = st.back(); st.pop_back(); ++seen;
      for (int k = 0; k < t[u].succ_cnt; ++k) { const int v = succ[t[u].succ_off + k]; if (--deg[v] == 0) st.push_back(v); }
      for (int v : xs[u]) if (--deg[v] == 0) st.push_back(v);
    }
    if (seen != nt) return "version-wait cycle: a task waits for a version that only a task depending on it can publish";
  }
  return "";
}

// The same check without a handle or a GPU: what a loader or a fuzzer calls before anything is created on a device.
extern "C" int kvm_validate_batch(const KvmTaskDesc* tasks, int32_t nt, const int32_t* succ, int32_t ne, const int32_t* args, int32_t na, int32_t nbufs, int32_t nvars,
                                  char* msg, size_t msg_len) {
  std::string problem;
  if (nt < 0 || ne < 0 || na < 0 || nbufs < 0 || nvars < 0 || (nt && !tasks) || (ne && !succ) || (na && !args)) problem = "bad argument";
  else problem = kvm_validate(tasks, nt, succ, ne, args, na, nbufs, nvars);
  if (msg && msg_len) snprintf(msg, msg_len, "%s", problem.c_str());
  return problem.empty() ? 0 : KVM_E_BUNDLE;
}

static int kvm_plan_tc(KvmExec* h, int first_task);   // kvm_gemm_host.inl: tensor maps of the tensor-core tasks
static int kvm_plan_static(KvmExec* h, const std::vector<int>& base_versions, KvmStaticPlan& plan);   // kvm_static_host.inl

extern "C" int kvm_submit(KvmExec* h, const KvmTaskDesc* tasks, int32_t nt, const int32_t* succ, int32_t ne, const int32_t* args, int32_t na) {
  if (!h || !tasks || nt <= 0 || ne < 0 || na < 0 || (ne && !succ) || (na && !args)) { if (h) h->error = "kvm_submit: bad argument"; return KVM_E_ARG; }
  if (h->started) { h->error = "kvm_submit: a run is in flight"; return KVM_E_STATE; }
  const std::string problem = kvm_validate(tasks, nt, succ, ne, args, na, (int)h->bufs.size(), h->nvars);
  if (!problem.empty()) { h->error = problem; return KVM_E_BUNDLE; }
  const int tbase = (int)h->tasks.size(), sbase = (int)h->succ.size(), abase = (int)h->args.size();
  for (int i = 0; i < nt; ++i) { KvmTaskDesc d = tasks[i]; d.succ_off += sbase; d.args_off += abase; h->tasks.push_back(d); }
  for (int i = 0; i < ne; ++i) h->succ.push_back(succ[i] + tbase);
  h->args.insert(h->args.end(), args, args + na);
  h->aux.resize(h->tasks.size(), make_int4(0, 0, 0, 0));
  h->tasks_dirty = true; h->armed = false;
  return kvm_plan_tc(h, tbase);
}

static bool kvm_read_file(const std::string& path, std::vector<char>& out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  fseek(f, 0, SEEK_END); long n = ftell(f); fseek(f, 0, SEEK_SET);
  out.resize(n > 0 ? n : 0);
  const bool ok = n <= 0 || fread(out.data(), 1, n, f) == (size_t)n;
  fclose(f);
  return ok;
}
extern "C" int kvm_submit_bundle_dir(KvmExec* h, const char* dir) {
  if (!h || !dir) return KVM_E_ARG;
  std::vector<char> t, s, a;
  const std::string d(dir);
  if (!kvm_read_file(d + "/tasks.bin", t) || !kvm_read_file(d + "/successors.bin", s) || !kvm_read_file(d + "/args.bin", a)) { h->error = "cannot read bundle files in " + d; return KVM_E_IO; }
  if (t.size() % sizeof(KvmTaskDesc) || s.size() % 4 || a.size() % 4) { h->error = "bundle file sizes are not whole records"; return KVM_E_BUNDLE; }
  return kvm_submit(h, (const KvmTaskDesc*)t.data(), (int)(t.size() / sizeof(KvmTaskDesc)), (const int32_t*)s.data(), (int)(s.size() / 4), (const int32_t*)a.data(), (int)(a.size() / 4));
}

// ---- bundle directory loader: what the reference CLI does with metadata.json (mvm_exec.cu:2055-2076,1915-1929) ----------------------
static uint16_t kvm_host_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);      // NaN stays NaN
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

extern "C" int kvm_load_bundle_dir(KvmExec* h, const char* dir) {
  if (!h || !dir) { if (h) h->error = "kvm_load_bundle_dir: bad argument"; return KVM_E_ARG; }
  if (h->started) { h->error = "kvm_load_bundle_dir: a run is in flight"; return KVM_E_STATE; }
  const std::string d(dir);
  std::vector<char> raw;
  if (!kvm_read_file(d + "/metadata.json", raw)) { h->error = "cannot read " + d + "/metadata.json"; return KVM_E_IO; }
  try {
    const std::string text(raw.begin(), raw.end());
    const KvmJson m = KvmJsonParser(text).parse();
    if (m.type != KvmJson::Obj) throw std::runtime_error("metadata.json is not an object");
    if (m.integer("abi_version", -1) != KVM_ABI_VERSION) throw std::runtime_error("abi_version " + std::to_string(m.integer("abi_version", -1)) + " != " + std::to_string(KVM_ABI_VERSION));
    const long long nt = m.integer("task_count", -1), ne = m.integer("edge_count", -1), nw = m.integer("args_words", -1);
    if (nt < 1 || ne < 0 || nw < 0) throw std::runtime_error("task_count / edge_count / args_words missing");
    std::vector<char> t, sc, ar;
    if (!kvm_read_file(d + "/tasks.bin", t) || !kvm_read_file(d + "/successors.bin", sc) || !kvm_read_file(d + "/args.bin", ar)) { h->error = "cannot read bundle files in " + d; return KVM_E_IO; }
    if ((long long)t.size() != nt * (long long)sizeof(KvmTaskDesc) || (long long)sc.size() != ne * 4 || (long long)ar.size() != nw * 4)
      throw std::runtime_error("tasks.bin / successors.bin / args.bin do not have the sizes metadata.json states");
    if (const KvmJson* bs = m.get("buffers")) {
      if (bs->type != KvmJson::Arr) throw std::runtime_error("buffers is not an array");
      for (const KvmJson& jb : bs->a) {
        const long long idx = jb.integer("index", -1), rows = jb.integer("rows", 0), cols = jb.integer("cols", 0), dtype = jb.integer("dtype", 0);
        const std::string name = jb.str("name");
        if (idx < 0 || rows < 1 || cols < 1 || rows * cols > 2147483647LL || dtype < 0 || dtype > 2) throw std::runtime_error("bad buffer entry '" + name + "'");
        if (idx < (long long)h->bufs.size()) {      // a buffer an earlier bundle of this handle declared: the shapes must agree
          const KvmBuf& b = h->bufs[idx];
          if (b.rows != rows || b.cols != cols || b.dtype != dtype) throw std::runtime_error("buffer " + std::to_string(idx) + " differs from an earlier bundle's");
          continue;
        }
        if (idx != (long long)h->bufs.size()) throw std::runtime_error("buffer indices must be dense and ascending");
        const size_t n = (size_t)(rows * cols);
        KvmInit init{};
        std::vector<char> data;
        const KvmJson* in = jb.get("init");
        const std::string kind = in ? in->str("kind") : "fill";
        if (!in || kind == "fill") { init.kind = KVM_INIT_FILL; init.fill = in ? in->num("value", 0.0) : 0.0; }
        else if (kind == "values") {
          const KvmJson& vals = in->need("values");
          if (vals.type != KvmJson::Arr || vals.a.size() != n) throw std::runtime_error("buffer '" + name + "': values do not match rows x cols");
          data.resize(n * kvm_elem_bytes((int)dtype));
          for (size_t i = 0; i < n; ++i) {
            if (vals.a[i].type != KvmJson::Num) throw std::runtime_error("buffer '" + name + "': a value is not a number");
            if (dtype == KVM_I32) ((int32_t*)data.data())[i] = (int32_t)strtoll(vals.a[i].s.c_str(), nullptr, 10);
            else if (dtype == KVM_BF16) ((uint16_t*)data.data())[i] = kvm_host_bf16((float)vals.a[i].n);
            else ((float*)data.data())[i] = (float)vals.a[i].n;
          }
          init.kind = KVM_INIT_VALUES; init.data = data.data();
        } else if (kind == "seeded") {
          init.kind = KVM_INIT_SEEDED; init.seed = in->u64("seed", 0); init.draws = (int)in->integer("draws", 1);
          init.bias = (float)in->num("bias", 0.0); init.coef = (float)in->num("coef", 1.0);
        } else if (kind == "file") {
          const std::string rel = in->str("path");
          if (rel.empty() || rel[0] == '/' || rel.find("..") != std::string::npos) throw std::runtime_error("buffer '" + name + "': file init needs a path inside the bundle directory");
          if (!kvm_read_file(d + "/" + rel, data)) { h->error = "cannot read " + d + "/" + rel; return KVM_E_IO; }
          if (data.size() != n * kvm_elem_bytes((int)dtype)) throw std::runtime_error("buffer '" + name + "': " + rel + " does not hold rows x cols elements");
          init.kind = KVM_INIT_VALUES; init.data = data.data();
        } else throw std::runtime_error("buffer '" + name + "': unknown init kind '" + kind + "'");
        const int r = kvm_add_buffer(h, (int)rows, (int)cols, (int)dtype, &init);
        if (r < 0) return r;
        h->buf_names.resize(h->bufs.size());
        h->buf_names[r] = name;
      }
    }
    if (const KvmJson* vs = m.get("variables")) for (const KvmJson& jv : vs->a) {
      const long long id = jv.integer("id", -1), base = jv.integer("base_version", 0);
      if (id < 0 || id >= h->nvars || base < 0) throw std::runtime_error("variable id or base_version out of range");
      h->var_ids[jv.str("name")] = (int)id;
      if (base) if (int r = kvm_set_version(h, (int)id, (int)base)) return r;
    }
    return kvm_submit(h, (const KvmTaskDesc*)t.data(), (int)nt, (const int32_t*)sc.data(), (int)ne, (const int32_t*)ar.data(), (int)nw);
  } catch (const std::exception& e) {
    h->error = d + ": " + e.what();
    return KVM_E_BUNDLE;
  }
}

extern "C" int kvm_buffer_count(KvmExec* h) { return h ? (int)h->bufs.size() : KVM_E_ARG; }
extern "C" int kvm_buffer_info(KvmExec* h, int32_t idx, int32_t* rows, int32_t* cols, int32_t* dtype) {
  if (!h || idx < 0 || idx >= (int)h->bufs.size()) { if (h) h->error = "kvm_buffer_info: index out of range"; return KVM_E_ARG; }
  if (rows) *rows = h->bufs[idx].rows;
  if (cols) *cols = h->bufs[idx].cols;
  if (dtype) *dtype = h->bufs[idx].dtype;
  return 0;
}
extern "C" const char* kvm_buffer_name(KvmExec* h, int32_t idx) { return (h && idx >= 0 && idx < (int)h->buf_names.size()) ? h->buf_names[idx].c_str() : ""; }
extern "C" int kvm_buffer_index(KvmExec* h, const char* name) {
  if (!h || !name) return KVM_E_ARG;
  for (size_t i = 0; i < h->buf_names.size(); ++i) if (h->buf_names[i] == name) return (int)i;
  return KVM_E_ARG;
}
extern "C" int kvm_variable_id(KvmExec* h, const char* name) {
  if (!h || !name) return KVM_E_ARG;
  auto it = h->var_ids.find(name);
  return it == h->var_ids.end() ? KVM_E_ARG : it->second;
}

extern "C" int kvm_clear_tasks(KvmExec* h) {
  if (!h) return KVM_E_ARG;
  if (h->started) { h->error = "kvm_clear_tasks: a run is in flight"; return KVM_E_STATE; }
  h->tasks.clear(); h->succ.clear(); h->args.clear(); h->aux.clear(); h->tmaps.clear();
  h->tasks_dirty = true; h->armed = false;
  return 0;
}

// Cells per class of the ready ring: every task is pushed once, a task that may yield (a wait for a peer's flag) up to six times more.
static int kvm_ring_cap(const KvmExec* h) {
  size_t extra = 0;
  for (const KvmTaskDesc& t : h->tasks) if (t.op_id == 303 || t.op_id == 304) extra += 6;
  return (int)(h->tasks.size() + extra);
}
static KvmDevState kvm_dev_state(KvmExec* h) {
  KvmDevState S{};
  S.tasks = h->d_tasks; S.succ = h->d_succ; S.args = h->d_args; S.nt = (int)h->tasks.size();
  S.indeg = h->d_indeg; S.exec_count = h->d_exec; S.ring = h->d_ring; S.ring_cap = kvm_ring_cap(h);
  S.head = (unsigned*)h->d_ctl + 8; S.tail = (unsigned*)h->d_ctl + 12; S.done = h->d_ctl + 2;      // head[4], tail[4]: 16-byte aligned, one sector
  S.bufs = h->d_bufs; S.nbufs = (int)h->bufs.size();
  S.versions = h->d_versions; S.nvars = h->nvars; S.ver_base = h->d_ver_base; S.ver_off = h->d_ver_off; S.park_head = h->d_park_head; S.park_next = h->d_park_next;
  S.err = h->d_err;
  S.t_start = h->d_tstart; S.t_end = h->d_tend; S.t_smid = h->d_tsmid; S.trace = h->cfg.trace;
  S.timeout_ns = (unsigned long long)(h->cfg.timeout_ms > 0 ? h->cfg.timeout_ms : 20000) * 1000000ull;
  S.cfg_flags = h->cfg.flags;
  S.tmaps = h->d_tmaps; S.task_aux = h->d_aux; S.recs = h->d_recs; S.claim = h->d_claim; S.buf_cache = kvm_feature_on("KVM_B200_BUFCACHE", h->has_gemv ? 0 : 1) ? 1 : 0;
  { const char* v = getenv("KVM_B200_PAIR_DEPTH"); S.pair_depth = v && *v ? atoi(v) : 2 * h->workers; }
  // overlapped GEMM pipeline: on unless tiles are stacked (that path owns both accumulators) or tensor cores are off; KVM_B200_ENGINE=0 for A/B measurements
  S.engine = !(h->cfg.flags & KVM_CFG_NO_TENSOR_CORES) && !kvm_feature_on("KVM_B200_PAIRING", (h->cfg.flags & KVM_CFG_PAIR_TILES) ? 1 : 0) && kvm_feature_on("KVM_B200_ENGINE", 1) ? 1 : 0;
  return S;
}

static KvmStaticState kvm_static_state(KvmExec* h) {
  KvmStaticState T{};
  T.D = kvm_dev_state(h);
  T.prog = h->d_prog; T.prog_off = h->d_prog_off; T.waits = h->d_waits; T.progress = h->d_progress;
  T.ring = h->splan.ring;
  return T;
}

// Which path runs the resident program.  KVM_CFG_STATIC / KVM_CFG_DYNAMIC force one; otherwise the static path is taken for
// programs of streaming decode tasks (gemv_bf16), where knowing a worker's next task lets the weights stream ahead of the
// dependencies.  The environment variable KVM_B200_STATIC (0 / 1) overrides the default for measurements.
static bool kvm_wants_static(KvmExec* h, bool has_gemv) {
  if (h->cfg.flags & KVM_CFG_STATIC) return true;
  if (h->cfg.flags & KVM_CFG_DYNAMIC) return false;
  return kvm_feature_on("KVM_B200_STATIC", has_gemv ? 1 : 0);
}

static void kvm_launch(KvmExec* h) {
  if (h->use_static) kvm_static_launch(kvm_static_state(h), h->workers, h->smem_bytes, h->stream);
  else { KvmDevState S = kvm_dev_state(h); kvm_exec_kernel<<<h->workers, KVM_EXEC_THREADS, h->smem_bytes, h->stream>>>(S); }
}

// Upload whatever changed since the last run, arm the counters and enqueue the roots.
static int kvm_prepare(KvmExec* h, bool keep_error = false) {
  cudaSetDevice(h->device);
  const size_t nt = h->tasks.size();
  if (nt == 0) { h->error = "nothing submitted"; return KVM_E_STATE; }
  if (h->bufs_dirty) {
    if (h->bufs.size() > h->d_bufs_cap) {
      if (h->d_bufs) cudaFree(h->d_bufs);
      h->d_bufs_cap = h->bufs.size() * 2 + 16;
      KVM_CUDA(cudaMalloc(&h->d_bufs, h->d_bufs_cap * sizeof(KvmBuf)));
    }
    KVM_CUDA(cudaMemcpyAsync(h->d_bufs, h->bufs.data(), h->bufs.size() * sizeof(KvmBuf), cudaMemcpyHostToDevice, h->stream));
    h->bufs_dirty = false;
  }
  if (h->tasks_dirty) {
    kvm_free_tasks(h);
    KVM_CUDA(cudaMalloc(&h->d_tasks, nt * sizeof(KvmTaskDesc)));
    KVM_CUDA(cudaMalloc(&h->d_succ, (h->succ.size() + 1) * 4));
    KVM_CUDA(cudaMalloc(&h->d_args, (h->args.size() + 1) * 4));
    KVM_CUDA(cudaMalloc(&h->d_aux, nt * sizeof(int4)));
    KVM_CUDA(cudaMalloc(&h->d_tmaps, (h->tmaps.size() + 1) * sizeof(CUtensorMap)));
    KVM_CUDA(cudaMalloc(&h->d_indeg, nt * 4)); KVM_CUDA(cudaMalloc(&h->d_exec, nt * 4)); KVM_CUDA(cudaMalloc(&h->d_ring, (size_t)kvm_ring_cap(h) * 4 * KVM_NCLASS)); KVM_CUDA(cudaMalloc(&h->d_park_next, nt * 4)); KVM_CUDA(cudaMalloc(&h->d_claim, nt * 4));
    if (h->cfg.trace) { KVM_CUDA(cudaMalloc(&h->d_tstart, nt * 8)); KVM_CUDA(cudaMalloc(&h->d_tend, nt * 8)); KVM_CUDA(cudaMalloc(&h->d_tsmid, nt * 4)); }
    KVM_CUDA(cudaMemcpyAsync(h->d_tasks, h->tasks.data(), nt * sizeof(KvmTaskDesc), cudaMemcpyHostToDevice, h->stream));
    if (!h->succ.empty()) {
      // device form of a successor entry: task index in the low 27 bits, above it the successor's priority class (2 bits) and
      // whether it waits on a version (1 bit), so that the releasing warp needs no look at the successor's descriptor
      if (nt >= (size_t)1 << KVM_SUCC_BITS) { h->error = "too many tasks for one launch"; return KVM_E_ARG; }
      std::vector<int32_t> enc(h->succ.size());
      for (size_t k = 0; k < enc.size(); ++k) {
        const KvmTaskDesc& d = h->tasks[h->succ[k]];
        const int cls = d.priority < 0 ? 0 : (d.priority >> 3) >= KVM_NCLASS ? KVM_NCLASS - 1 : (d.priority >> 3);
        enc[k] = h->succ[k] | (cls << KVM_SUCC_BITS) | ((d.wait_var >= 0 ? 1 : 0) << (KVM_SUCC_BITS + 2));
      }
      KVM_CUDA(cudaMemcpyAsync(h->d_succ, enc.data(), enc.size() * 4, cudaMemcpyHostToDevice, h->stream));
      KVM_CUDA(cudaStreamSynchronize(h->stream));      // `enc` is a local
    }
    if (!h->args.empty()) KVM_CUDA(cudaMemcpyAsync(h->d_args, h->args.data(), h->args.size() * 4, cudaMemcpyHostToDevice, h->stream));
    KVM_CUDA(cudaMemcpyAsync(h->d_aux, h->aux.data(), nt * sizeof(int4), cudaMemcpyHostToDevice, h->stream));
    h->has_gemv = false;
    for (const KvmTaskDesc& d : h->tasks) if (d.op_id == 134 || d.op_id == 301) h->has_gemv = true;
    h->use_static = false;
    if (kvm_wants_static(h, h->has_gemv)) {
      std::vector<int> base(h->nvars, 0);
      KVM_CUDA(cudaStreamSynchronize(h->stream));
      KVM_CUDA(cudaMemcpy(base.data(), h->d_versions, h->nvars * sizeof(int), cudaMemcpyDeviceToHost));
      const int r = kvm_plan_static(h, base, h->splan);
      if (r == 0) h->use_static = true;
      else if (h->cfg.flags & KVM_CFG_STATIC) return r;      // asked for explicitly: say why it cannot be done
    }
    if (h->use_static) {
      const KvmStaticPlan& P = h->splan;
      KVM_CUDA(cudaMalloc(&h->d_prog, (P.prog.size() + 1) * 4)); KVM_CUDA(cudaMalloc(&h->d_prog_off, P.prog_off.size() * 4));
      KVM_CUDA(cudaMalloc(&h->d_waits, (P.waits.size() + 1) * 4)); KVM_CUDA(cudaMalloc(&h->d_progress, (size_t)h->workers * 4));
      KVM_CUDA(cudaMemcpyAsync(h->d_prog, P.prog.data(), P.prog.size() * 4, cudaMemcpyHostToDevice, h->stream));
      KVM_CUDA(cudaMemcpyAsync(h->d_prog_off, P.prog_off.data(), P.prog_off.size() * 4, cudaMemcpyHostToDevice, h->stream));
      if (!P.waits.empty()) KVM_CUDA(cudaMemcpyAsync(h->d_waits, P.waits.data(), P.waits.size() * 4, cudaMemcpyHostToDevice, h->stream));
    }
    {   // one record per task for the workers: descriptor, argument words and path selector side by side (a single fetch per pop)
      std::vector<int32_t> recs(nt * (size_t)KVM_REC_WORDS, 0);
      for (size_t i = 0; i < nt; ++i) {
        int32_t* r = &recs[i * KVM_REC_WORDS];
        memcpy(r, &h->tasks[i], sizeof(KvmTaskDesc));
        const int ao = r[6], aw = r[7] < KVM_MAX_ARGS ? r[7] : KVM_MAX_ARGS;
        for (int k = 0; k < aw; ++k) r[16 + k] = h->args[(size_t)ao + k];
        memcpy(r + 16 + KVM_MAX_ARGS, &h->aux[i], sizeof(int4));
        if (h->use_static) { r[KVM_REC_WAIT_OFF] = h->splan.wait_off[i]; r[KVM_REC_WAIT_CNT] = h->splan.wait_cnt[i]; r[KVM_REC_STREAM] = h->splan.stream[i]; }
      }
      KVM_CUDA(cudaMalloc(&h->d_recs, recs.size() * 4));
      KVM_CUDA(cudaMemcpyAsync(h->d_recs, recs.data(), recs.size() * 4, cudaMemcpyHostToDevice, h->stream));
      KVM_CUDA(cudaStreamSynchronize(h->stream));      // `recs` is a local
    }
    if (!h->tmaps.empty()) KVM_CUDA(cudaMemcpyAsync(h->d_tmaps, h->tmaps.data(), h->tmaps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
    KVM_CUDA(cudaMemcpyAsync(h->d_ver_base, h->d_versions, h->nvars * sizeof(int), cudaMemcpyDeviceToDevice, h->stream));   // the versions these tasks were compiled against
    h->tasks_dirty = false; h->task_cap = nt;
  }
  KvmDevState S = kvm_dev_state(h);
  KVM_CUDA(cudaMemsetAsync(h->d_ctl, 0, 64 * sizeof(int), h->stream));
  if (!keep_error) KVM_CUDA(cudaMemsetAsync(h->d_err, 0, sizeof(KvmErrRec), h->stream));
  if (h->cfg.trace) { cudaMemsetAsync(h->d_tstart, 0, nt * 8, h->stream); cudaMemsetAsync(h->d_tend, 0, nt * 8, h->stream); }
  size_t arm_n = nt > (size_t)h->nvars ? nt : (size_t)h->nvars;
  if ((size_t)h->workers > arm_n) arm_n = h->workers;
  const int blocks = (int)((arm_n + 255) / 256);
  if (h->use_static) kvm_static_arm(kvm_static_state(h), h->workers, blocks, h->stream);
  else {
    kvm_arm_kernel<<<blocks, 256, 0, h->stream>>>(S);
    kvm_roots_kernel<<<blocks, 256, 0, h->stream>>>(S);
  }
  KVM_CUDA(cudaGetLastError());
  h->armed = true;
  return 0;
}

extern "C" int kvm_rearm(KvmExec* h) {
  if (!h) return KVM_E_ARG;
  if (h->started) { h->error = "kvm_rearm: a run is in flight"; return KVM_E_STATE; }
  return kvm_prepare(h);
}

extern "C" int kvm_set_stream(KvmExec* h, void* stream) {
  if (!h) return KVM_E_ARG;
  if (h->started) { h->error = "kvm_set_stream: a run is in flight"; return KVM_E_STATE; }
  cudaSetDevice(h->device);
  cudaStreamSynchronize(h->stream);
  if (h->own_stream && h->stream) cudaStreamDestroy(h->stream);
  h->stream = (cudaStream_t)stream;
  h->own_stream = false;
  return 0;
}

extern "C" int kvm_start(KvmExec* h) {
  if (!h) return KVM_E_ARG;
  bool chained = false;
  if (h->started) {
    // KVM_CFG_CHAIN: the next run is queued behind the previous one on the same stream without reading its result back
    // (segments of one token with collectives between them); the device's first error stays recorded across the chain.
    if (!(h->cfg.flags & KVM_CFG_CHAIN)) { h->error = "kvm_start: already started"; return KVM_E_STATE; }
    chained = true; h->armed = false;
  }
  cudaSetDevice(h->device);
  // buffers added or bound, or tasks submitted, after kvm_rearm: the device tables are stale, prepare again
  if (!h->armed || h->bufs_dirty || h->tasks_dirty) if (int r = kvm_prepare(h, chained)) return r;
  KVM_CUDA(cudaEventRecord(h->ev0, h->stream));
  kvm_launch(h);
  KVM_CUDA(cudaGetLastError());
  KVM_CUDA(cudaEventRecord(h->ev1, h->stream));
  h->started = true; h->armed = false;
  return 0;
}

extern "C" int kvm_close(KvmExec* h) {
  if (!h) return KVM_E_ARG;
  if (!h->started) { h->error = "kvm_close: nothing started"; return KVM_E_STATE; }
  return 0;          // every batch was resident before the launch: nothing to close
}

extern "C" int kvm_finish(KvmExec* h, KvmResult* res) {
  if (!h) return KVM_E_ARG;
  if (!h->started) { h->error = "kvm_finish: nothing started"; return KVM_E_STATE; }
  h->started = false;
  cudaSetDevice(h->device);
  KVM_CUDA(cudaStreamSynchronize(h->stream));
  int ctl[4]; KvmErrRec er;
  KVM_CUDA(cudaMemcpy(ctl, h->d_ctl, sizeof ctl, cudaMemcpyDeviceToHost));
  KVM_CUDA(cudaMemcpy(&er, h->d_err, sizeof er, cudaMemcpyDeviceToHost));
  KvmResult r{};
  r.status = er.code; r.done = ctl[2]; r.admitted = (int)h->tasks.size();
  r.err_task = er.code ? er.task : -1; r.err_a = er.a; r.err_b = er.b;
  cudaEventElapsedTime(&r.ms, h->ev0, h->ev1);
  if (h->cfg.trace && !h->tasks.empty()) {
    const size_t nt = h->tasks.size();
    std::vector<unsigned long long> s(nt), e(nt);
    cudaMemcpy(s.data(), h->d_tstart, nt * 8, cudaMemcpyDeviceToHost); cudaMemcpy(e.data(), h->d_tend, nt * 8, cudaMemcpyDeviceToHost);
    unsigned long long lo = ~0ull, hi = 0; double busy = 0;
    for (size_t i = 0; i < nt; ++i) if (e[i] > s[i] && s[i]) { busy += (double)(e[i] - s[i]); if (s[i] < lo) lo = s[i]; if (e[i] > hi) hi = e[i]; }
    if (hi > lo) r.busy_frac = (float)(busy / ((double)h->workers * (double)(hi - lo)));
  }
  if (er.code) {
    char m[200];
    snprintf(m, sizeof m, "device error %d (%s) at task %d, detail %d %d; %d/%d tasks done", er.code, kvm_err_name(er.code), er.task, er.a, er.b, r.done, r.admitted);
    h->error = m;
  } else if (r.done != r.admitted) {
    r.status = KVM_ERR_TIMEOUT; h->error = "run ended with unfinished tasks";
  }
  h->last = r;
  if (res) *res = r;
  return r.status;
}

extern "C" int kvm_run(KvmExec* h, KvmResult* res) {
  if (int r = kvm_start(h)) { if (res) { *res = KvmResult{}; res->status = r; } return r; }
  return kvm_finish(h, res);
}

extern "C" int kvm_run_steps(KvmExec* h, int32_t steps, KvmResult* res) {
  if (!h || steps < 1) return KVM_E_ARG;
  if (h->started) { h->error = "kvm_run_steps: a run is in flight"; return KVM_E_STATE; }
  if (int r = kvm_prepare(h)) return r;
  KVM_CUDA(cudaEventRecord(h->ev0, h->stream));
  for (int s = 0; s < steps; ++s) {
    if (s) if (int r = kvm_prepare(h, true)) return r;
    kvm_launch(h);
    KVM_CUDA(cudaGetLastError());
  }
  KVM_CUDA(cudaEventRecord(h->ev1, h->stream));
  h->started = true; h->armed = false;
  return kvm_finish(h, res);
}

extern "C" int kvm_task_counts(KvmExec* h, int32_t* exec_count, int32_t* observed, int32_t n) {
  if (!h || n < 0 || n > (int)h->tasks.size() || !h->d_exec) { if (h) h->error = "kvm_task_counts: bad argument or no run yet"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  if (exec_count) KVM_CUDA(cudaMemcpy(exec_count, h->d_exec, (size_t)n * 4, cudaMemcpyDeviceToHost));
  if (observed) {
    std::vector<int> rem(n);
    KVM_CUDA(cudaMemcpy(rem.data(), h->d_indeg, (size_t)n * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < n; ++i) observed[i] = h->tasks[i].indegree - rem[i];
  }
  return 0;
}
extern "C" int kvm_trace(KvmExec* h, uint64_t* start_ns, uint64_t* end_ns, int32_t* smid, int32_t n) {
  if (!h || !h->cfg.trace || n < 0 || n > (int)h->tasks.size() || !h->d_tstart) { if (h) h->error = "kvm_trace: tracing is off or no run yet"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  if (start_ns) KVM_CUDA(cudaMemcpy(start_ns, h->d_tstart, (size_t)n * 8, cudaMemcpyDeviceToHost));
  if (end_ns) KVM_CUDA(cudaMemcpy(end_ns, h->d_tend, (size_t)n * 8, cudaMemcpyDeviceToHost));
  if (smid) {
    KVM_CUDA(cudaMemcpy(smid, h->d_tsmid, (size_t)n * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < n; ++i) smid[i] &= 0xff;
  }
  return 0;
}
extern "C" int kvm_trace_detail(KvmExec* h, int32_t* detail, int32_t n) {
  if (!h || !h->cfg.trace || !detail || n < 0 || n > (int)h->tasks.size() || !h->d_tstart) { if (h) h->error = "kvm_trace_detail: tracing is off or no run yet"; return KVM_E_ARG; }
  cudaSetDevice(h->device);
  KVM_CUDA(cudaMemcpy(detail, h->d_tsmid, (size_t)n * 4, cudaMemcpyDeviceToHost));
  for (int i = 0; i < n; ++i) detail[i] = (int32_t)((uint32_t)detail[i] >> 8);
  return 0;
}
extern "C" int kvm_launch_info(KvmExec* h, int32_t* workers, int32_t* threads, int32_t* smem_bytes) {
  if (!h) return KVM_E_ARG;
  if (workers) *workers = h->workers;
  if (threads) *threads = h->use_static ? KVM_NT + 32 : KVM_EXEC_THREADS;
  if (smem_bytes) *smem_bytes = h->smem_bytes;
  return 0;
}

extern "C" int kvm_plan_info(KvmExec* h, int32_t* is_static, int32_t* stream_ring, float* planned_us) {
  if (!h) return KVM_E_ARG;
  if (h->tasks_dirty) { h->error = "kvm_plan_info: the program has not been prepared yet (kvm_rearm or a run does it)"; return KVM_E_STATE; }
  if (is_static) *is_static = h->use_static ? 1 : 0;
  if (stream_ring) *stream_ring = h->use_static && h->splan.ring ? 1 : 0;
  if (planned_us) *planned_us = h->use_static ? (float)h->splan.makespan_us : 0.0f;
  return 0;
}

extern "C" int kvm_tc_task_count(KvmExec* h) {
  if (!h) return KVM_E_ARG;
  int n = 0;
  for (auto& a : h->aux) n += a.x != 0;
  return n;
}

#include "kvm_gemm_host.inl"
#include "kvm_static_host.inl"
