// Exchange ops between executors on different GPUs of one node: plain peer stores into the other rank's inbox, a system-scope
// release of a flag word, and a bounded wait on the receiving side.  No multicast, no library call on peer memory.
// Semantics after the reference's put_signal and its inbox versions (include/mvm_ops_comm.def:5-11, include/mvm_dist.cuh:73-77).
#pragma once
#include "kvm_dev.cuh"

__device__ __forceinline__ void kvm_st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int kvm_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool kvm_span_ok(const KvmCtx& c, const KvmBuf& b, long long off, long long n) {
  if (off < 0 || n < 0 || b.ld != b.cols || off + n > (long long)b.rows * b.cols) { c.fail(KVM_OPE_RANGE, (int)off, (int)n); return false; }
  return true;
}

// peer_put_signal (302)
KVM_OP_FN void kvm_op_peer_put_signal(const KvmCtx& c, const int32_t* a) {
  KvmBuf src, dst, flag, seq;
  if (!kvm_buf(c, a[0], KVM_M_F32, src) || !kvm_buf(c, a[1], KVM_M_F32, dst) || !kvm_buf(c, a[5], KVM_M_I32, flag) || !kvm_buf(c, a[8], KVM_M_I32, seq, true)) return;
  const int so = a[2], d0 = a[3], n = a[4], var = a[6], ver = a[7], stride = a[9];
  if (n <= 0 || !kvm_span_ok(c, src, so, n) || !kvm_span_ok(c, dst, d0, n) || !kvm_span_ok(c, flag, var, 1)) { if (n <= 0) c.fail(KVM_OPE_RANGE, n); return; }
  const float* s = (const float*)src.p + so;
  float* d = (float*)dst.p + d0;
  if (!(((uintptr_t)s | (uintptr_t)d) & 15) && !(n & 3)) {
    for (int i = threadIdx.x; i < n / 4; i += KVM_NT) ((float4*)d)[i] = ((const float4*)s)[i];
  } else {
    for (int i = threadIdx.x; i < n; i += KVM_NT) d[i] = s[i];
  }
  __threadfence_system();                       // every writer: its stores are performed at system scope before the barrier
  kvm_sync();
  if (threadIdx.x == 0) {
    const int eff = ver + (seq.p ? ((const int*)seq.p)[0] * stride : 0);
    asm volatile("fence.sc.sys;" ::: "memory");
    kvm_st_release_sys((int*)flag.p + var, eff);
  }
}

// peer_wait_sum (303)
KVM_OP_FN void kvm_op_peer_wait_sum(const KvmCtx& c, const int32_t* a) {
  KvmBuf part, inbox, flag, out, res, seq;
  if (!kvm_buf(c, a[0], KVM_M_F32, part) || !kvm_buf(c, a[1], KVM_M_F32, inbox) || !kvm_buf(c, a[2], KVM_M_I32, flag) || !kvm_buf(c, a[3], KVM_M_F32, out) ||
      !kvm_buf(c, a[4], KVM_M_F32, res, true) || !kvm_buf(c, a[10], KVM_M_I32, seq, true)) return;
  const int n = a[5], row0 = a[6], rank = a[7], world = a[8], ver = a[9], stride = a[11];
  if (n <= 0 || world < 1 || world > 32 || rank < 0 || rank >= world || row0 < 0) { c.fail(KVM_OPE_RANGE, n, world); return; }
  if (!kvm_span_ok(c, part, 0, n) || !kvm_span_ok(c, out, 0, n) || (res.p && !kvm_span_ok(c, res, 0, n)) || !kvm_span_ok(c, flag, row0, world) ||
      !kvm_mat_ok(c, inbox, (long long)row0 + world, n)) return;
  int* ok = (int*)c.smem;
  kvm_sync();                                   // the previous task is done with the scratch
  if (threadIdx.x < 32) {
    const int eff = ver + (seq.p ? ((const int*)seq.p)[0] * stride : 0);
    const int p = threadIdx.x;
    bool met = !(p < world && p != rank);
    unsigned spins = 0;
    bool alive = true;
    while (alive) {
      if (!met && kvm_ld_acquire_sys((const int*)flag.p + row0 + p) >= eff) met = true;
      if (__all_sync(0xffffffffu, met)) break;
      if ((++spins & 255u) == 0 && (kvm_globaltimer() > c.deadline || *(volatile const int*)&c.err->code != 0)) alive = false;
      alive = __all_sync(0xffffffffu, alive);
    }
    if (!alive && !met) c.fail_any(KVM_ERR_TIMEOUT, row0 + p, eff);        // the peer's flag never came (first error wins)
    if (threadIdx.x == 0) *ok = alive ? 1 : 0;
  }
  kvm_sync();                                   // the acquiring warp's loads happen before everyone's reads of the inbox
  if (*ok == 0) return;
  const float* ib = (const float*)inbox.p;
  for (int i = threadIdx.x; i < n; i += KVM_NT) {
    float v = res.p ? ((const float*)res.p)[i] : 0.0f;
    bool first = !res.p;
    for (int p = 0; p < world; ++p) {
      const float t = p == rank ? ((const float*)part.p)[i] : __ldcg(ib + (size_t)(row0 + p) * inbox.ld + i);     // L2: what the peer wrote, never a stale L1 line of the last run
      v = first ? t : __fadd_rn(v, t);
      first = false;
    }
    ((float*)out.p)[i] = v;
  }
}
