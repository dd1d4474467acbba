// State shared by the two executor kernels (ready-queue path: kvm_sched.cuh; static-schedule path: kvm_static.cuh): the device view
// of the resident program, memory-ordering helpers, first-error-wins failure, priority classes.
#pragma once
#include "kvm_dev.cuh"

struct KvmDevState {
  const KvmTaskDesc* tasks;
  const int32_t* succ;
  const int32_t* args;
  int nt;
  int* indeg;                 // remaining predecessors per task
  int* exec_count;            // times executed (exactly-once witness)
  int* ring;                  // ready rings, one per priority class: ring[c * nt + ticket] = task + 1 once filled
  unsigned* head;             // head[c]: next pop ticket of class c   (head and tail words share one 32-byte sector)
  unsigned* tail;             // tail[c]: next push ticket of class c
  int* done;                  // tasks finished
  const KvmBuf* bufs;
  int nbufs;
  int* versions;
  int nvars;
  const int* ver_base;        // versions when the submitted tasks were first armed (what they were compiled against)
  int* ver_off;               // versions now minus ver_base at arm time: a re-run is the next window of the same template
  int* park_head;             // per variable: head of the parked list (-1 empty)
  int* park_next;             // per task
  KvmErrRec* err;
  unsigned long long* t_start;  // trace (optional)
  unsigned long long* t_end;
  int* t_smid;
  int trace;
  unsigned long long timeout_ns;
  int cfg_flags;
  const void* tmaps;          // CUtensorMap table for tensor-core tasks
  const int4* task_aux;       // per task: tensor-map indices / path selector
  const int32_t* recs;        // per task KVM_REC_WORDS words: descriptor [0,16), argument words [16,36), path selector [36,40)
  int buf_cache;              // 1: copy the buffer table into shared memory at launch (off for graphs of streaming GEMVs, which want the space)
  int pair_depth;             // tiles are stacked only while at least this many tasks are queued (wide phases; narrow ones keep their parallelism)
  int* claim;                 // per task: 0 free, 1 taken (tensor-core GEMM tiles that may run stacked with a partner tile)
  int ring_cap;               // cells per class of the ready ring: nt, plus the bounded re-queues of tasks that may yield (peer waits)
  int engine;                 // 1: the ready-queue kernel's engine warps run the mainloops of the tensor-core GEMM tiles (overlapped with the previous tile's epilogue)
};
#define KVM_REC_WORDS 48
#define KVM_SUCC_BITS 27          // successor entry on the device: index | class << 27 | has-version-wait << 29


__device__ __forceinline__ int kvm_ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void kvm_st_release(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void kvm_st_relaxed(int* p, int v) { asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int kvm_ld_volatile_shared(const int* p) { return *(volatile const int*)p; }

__device__ __forceinline__ void kvm_dev_fail(const KvmDevState& S, int code, int task, int a = 0, int b = 0) {
  if (atomicCAS(&S.err->code, 0, code) == 0) { S.err->task = task; S.err->a = a; S.err->b = b; __threadfence_system(); }
}

// Priority classes: the ABI's 32 priorities (larger first, include/mvm_task_abi.h:16) fold into KVM_NCLASS rings, class = priority / 8.
// A pop looks at the classes from the highest down and claims a ticket only where one is known to be filled or about to be
// (head < tail, compare-and-swap), so no worker ever commits to a ticket that may stay empty.
#define KVM_NCLASS 4
__device__ __forceinline__ int kvm_class_of(int priority) { return priority < 0 ? 0 : (priority >> 3) >= KVM_NCLASS ? KVM_NCLASS - 1 : (priority >> 3); }

static __device__ void kvm_dispatch(const KvmCtx& c, int op, const int32_t* args, const int4& aux);

#define KVM_EXEC_SMEM_HDR 2048     // slots + control words at the start of dynamic shared memory
#define KVM_BUFCACHE_BYTES 32768    // shared-memory copy of the buffer table (up to 1024 buffers), after the header

