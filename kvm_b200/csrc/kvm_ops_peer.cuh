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

#define KVM_MAX_YIELDS 6
// Bounded wait of warp 0 for flag[row0 + i] >= eff, i < count (count <= 32; lane i polls word i, `skip` is left out).  *ok (shared
// memory) = 1: every flag came; 0: give up.  On expiry of the launch's deadline the lane whose flag is missing records
// KVM_ERR_TIMEOUT.  Where the executor allows it (KvmCtx::yield_word) and other tasks are queued, the wait ends early with a yield:
// the task has written nothing and runs again later, so a flag that is late costs a trip through the queue, not a stalled worker.
__device__ __forceinline__ void kvm_peer_poll(const KvmCtx& c, const KvmBuf& flag, int row0, int count, int skip, int eff, int* ok) {
  if (threadIdx.x < 32) {
    const int p = threadIdx.x;
    bool met = !(p < count && p != skip);
    unsigned spins = 0;
    int verdict = 0;                               // 1 all flags, 2 timeout / error elsewhere, 3 yield
    while (verdict == 0) {
      if (!met && kvm_ld_acquire_sys((const int*)flag.p + row0 + p) >= eff) met = true;
      if (__all_sync(0xffffffffu, met)) { verdict = 1; break; }
      if ((++spins & 15u) == 0) {                     // a poll is a system-scope load of about a microsecond: look around every 16th
        int v = 0;
        if (threadIdx.x == 0) {
          if (kvm_globaltimer() > c.deadline || *(volatile const int*)&c.err->code != 0) v = 2;
          else if (c.yield_word) {
            unsigned h[4], t[4];
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "l"(c.q_head) : "memory");
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3]) : "l"(c.q_tail) : "memory");
            const bool queued = t[0] > h[0] || t[1] > h[1] || t[2] > h[2] || t[3] > h[3];
            if (queued && atomicAdd(c.yield_count, 1) < KVM_MAX_YIELDS) v = 3;
          }
        }
        verdict = __shfl_sync(0xffffffffu, v, 0);
      }
    }
    if (verdict == 2 && !met) c.fail_any(KVM_ERR_TIMEOUT, row0 + p, eff);        // the peer's flag never came (first error wins)
    if (threadIdx.x == 0) { *ok = verdict == 1 ? 1 : 0; if (verdict == 3) *c.yield_word = 1; }
  }
}

// peer_wait_sum (303)
KVM_OP_FN void kvm_op_peer_wait_sum(const KvmCtx& c, const int32_t* a) {
  KvmBuf part, inbox, flag, out, res, seq;
  if (!kvm_buf(c, a[0], KVM_M_F32, part) || !kvm_buf(c, a[1], KVM_M_F32, inbox) || !kvm_buf(c, a[2], KVM_M_I32, flag) || !kvm_buf(c, a[3], KVM_M_F32, out) ||
      !kvm_buf(c, a[4], KVM_M_F32, res, true) || !kvm_buf(c, a[10], KVM_M_I32, seq, true)) return;
  const int n = a[5], row0 = a[6], rank = a[7], world = a[8], ver = a[9], stride = a[11], po = a[12], oo = a[13];
  if (n <= 0 || world < 1 || world > 32 || rank < 0 || rank >= world || row0 < 0) { c.fail(KVM_OPE_RANGE, n, world); return; }
  if (!kvm_span_ok(c, part, po, n) || !kvm_span_ok(c, out, oo, n) || (res.p && !kvm_span_ok(c, res, 0, n)) || !kvm_span_ok(c, flag, row0, world) ||
      !kvm_mat_ok(c, inbox, (long long)row0 + world, n)) return;
  int* ok = (int*)c.smem;
  kvm_sync();                                   // the previous task is done with the scratch
  kvm_peer_poll(c, flag, row0, world, rank, ver + (seq.p ? ((const int*)seq.p)[0] * stride : 0), ok);
  kvm_sync();                                   // the acquiring warp's loads happen before everyone's reads of the inbox
  if (*ok == 0) return;
  // inbox rows are read from L2 (what the peer wrote, never a stale L1 line of the last run); rank order, one rounded add each
  const float* ib = (const float*)inbox.p;
  const float* pp = (const float*)part.p + po;
  float* op = (float*)out.p + oo;
  const float* rp = (const float*)res.p;
  if (!(n & 3) && !(inbox.ld & 3) && !(((uintptr_t)pp | (uintptr_t)op | (uintptr_t)ib | (uintptr_t)rp) & 15)) {
    for (int i = threadIdx.x; i < n / 4; i += KVM_NT) {
      float4 v = rp ? ((const float4*)rp)[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      bool first = !rp;
      for (int p = 0; p < world; ++p) {
        const float4 t = p == rank ? ((const float4*)pp)[i] : __ldcg((const float4*)(ib + (size_t)(row0 + p) * inbox.ld) + i);
        v = first ? t : make_float4(__fadd_rn(v.x, t.x), __fadd_rn(v.y, t.y), __fadd_rn(v.z, t.z), __fadd_rn(v.w, t.w));
        first = false;
      }
      ((float4*)op)[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < n; i += KVM_NT) {
      float v = rp ? rp[i] : 0.0f;
      bool first = !rp;
      for (int p = 0; p < world; ++p) {
        const float t = p == rank ? pp[i] : __ldcg(ib + (size_t)(row0 + p) * inbox.ld + i);
        v = first ? t : __fadd_rn(v, t);
        first = false;
      }
      op[i] = v;
    }
  }
}

// peer_wait (304)
KVM_OP_FN void kvm_op_peer_wait(const KvmCtx& c, const int32_t* a) {
  KvmBuf flag, seq;
  if (!kvm_buf(c, a[0], KVM_M_I32, flag) || !kvm_buf(c, a[4], KVM_M_I32, seq, true)) return;
  const int row0 = a[1], count = a[2], ver = a[3], stride = a[5];
  if (row0 < 0 || count < 1 || count > 32 || !kvm_span_ok(c, flag, row0, count)) { if (count < 1 || count > 32 || row0 < 0) c.fail(KVM_OPE_RANGE, row0, count); return; }
  int* ok = (int*)c.smem;
  kvm_sync();
  kvm_peer_poll(c, flag, row0, count, -1, ver + (seq.p ? ((const int*)seq.p)[0] * stride : 0), ok);
  kvm_sync();
  // The data that came with the flags is in L2; lines of it that this SM still holds in L1 from an earlier run are dropped by the
  // acquire above (system scope), so the tasks released by this one read what the peers stored.
}
