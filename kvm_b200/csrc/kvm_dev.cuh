// Device-side common definitions of the B200 executor: buffer table entry, per-task context, typed argument access, error
// reporting, storage-typed loads/stores and block reductions used by every op body.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kvm_b200.h"

#define KVM_NT 512                 // compute threads per worker CTA (16 warps)
#define KVM_NWARPS (KVM_NT / 32)
#define KVM_MAX_ARGS 20            // reference: MVM_MAX_ARGS (include/mvm_exec.cuh:58)

// Executor error codes: the reference's MVM_ERRORS list (include/mvm_exec.cuh:147-164), same order and meaning.
#define KVM_ERRORS(E) \
  E(OK) E(BAD_OP) E(BAD_ARITY) E(BAD_BUF_INDEX) E(BAD_BUF) E(BOUNDS) E(BAD_VAR) E(VERSION_GAP) E(WAIT_VIOLATION) E(DOUBLE_EXEC) \
  E(BAD_RECORD) E(BAD_TASK) E(SLOTS) E(POOL) E(BATCH_TOO_LARGE) E(TIMEOUT) E(QUEUE_OVERFLOW) E(BAD_CONFIG) E(PARK_STALL) \
  E(TASK_LIMIT) E(ALIAS_RECORD)
enum KvmErr {
#define E(n) KVM_ERR_##n,
  KVM_ERRORS(E)
#undef E
  KVM_ERR_COUNT
};
// Op-pack error codes (reference: MVM_GPT_ERRORS, include/mvm_ops_gpt.cuh:181-194).
enum { KVM_OPE_BUF = 1001, KVM_OPE_DTYPE = 1002, KVM_OPE_RANGE = 1003, KVM_OPE_SHAPE = 1004, KVM_OPE_TOKEN = 1005, KVM_OPE_KVLEN = 1006,
       KVM_OPE_SMEM = 1007 };

// Buffer table entry, 32 bytes like the reference's MvmBuf (include/mvm_task_abi.h:33-39).
struct KvmBuf {
  void* p;
  int32_t rows, cols, ld, dtype;
  int32_t reserved[2];
};
static_assert(sizeof(KvmBuf) == 32, "KvmBuf size");

struct KvmErrRec { int code, task, a, b; };

struct KvmCtx {
  const KvmBuf* bufs;
  int nbufs;
  int task;
  KvmErrRec* err;
  unsigned char* smem;        // op scratch (dynamic shared memory after the executor's own words)
  int smem_bytes;
  int cfg_flags;
  int* ctl;                   // executor control words in shared memory (ctl[0] = TMEM base address)
  const void* tmaps;          // tensor-map table of the tensor-core tasks
  int pair;                   // >= 0: the task runs together with this partner task (two stacked GEMM tiles), else -1
  // Yielding (ready-queue kernel only, else yield_word == nullptr): a task that would only wait for something outside the launch
  // (a peer's flag) while other tasks are queued may set *yield_word = 1 and return WITHOUT having written anything; the worker
  // then puts it back at the end of its queue instead of finishing it.  yield_count: per-task attempts word (bounds the re-queues),
  // q_head / q_tail: the ready queue's ticket words of the four classes.
  int* yield_word;
  int* yield_count;
  const unsigned* q_head;
  const unsigned* q_tail;
  unsigned long long deadline;   // %globaltimer value after which a task that waits for something outside the launch (a peer's flag) gives up
  float* rope_cache;          // shared memory, 66 floats kept over the tasks of a launch: [0] theta bits, [1] head dimension bits, [2..] the inverse frequencies of that pair (or nullptr)
  int engine;                 // 1: the kernel's engine warps run the mainloops of tensor-core GEMM tiles, the op body is their epilogue only
  unsigned gemm_seq;          // with engine: how many tensor-core GEMM tiles this CTA ran before this one (accumulator = gemm_seq & 1)

  // First error wins (reference: mvm_fail, include/mvm_exec.cuh:260-266).  `fail` is for errors every thread of the group sees
  // alike (argument checks): all call it with the same arguments and thread 0 records.  `fail_any` is for data-dependent
  // errors that only the thread that met the bad value knows about (a token id out of range in the row it happens to own).
  __device__ void fail(int code, int a = 0, int b = 0) const {
    if (threadIdx.x == 0) fail_any(code, a, b);
  }
  __device__ void fail_any(int code, int a = 0, int b = 0) const {
    if (atomicCAS(&err->code, 0, code) == 0) {
      err->task = task; err->a = a; err->b = b;
      __threadfence_system();
    }
  }
};

__device__ __forceinline__ float kvm_bits_f32(int32_t w) { return __int_as_float(w); }

// ---- storage-typed scalar access (f32 or bf16 storage; i32 buffers are accessed as int directly) -------------------------
__device__ __forceinline__ float kvm_ld(const KvmBuf& b, size_t i) {
  return b.dtype == KVM_BF16 ? __bfloat162float(((const __nv_bfloat16*)b.p)[i]) : ((const float*)b.p)[i];
}
__device__ __forceinline__ void kvm_st(const KvmBuf& b, size_t i, float v) {
  if (b.dtype == KVM_BF16) ((__nv_bfloat16*)b.p)[i] = __float2bfloat16_rn(v);
  else ((float*)b.p)[i] = v;
}
__device__ __forceinline__ float kvm_bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// The same with the storage type as a template argument, for loops whose memory parallelism must not depend on whether the compiler
// hoists the type test out of the loop (with the test inside, every load sits in a basic block of its own and waits for the one
// before it: measured 2.3x on the column reductions).
template <bool BF>
__device__ __forceinline__ float kvm_ldt(const void* p, size_t i) { return BF ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i]; }

// 8 consecutive elements starting at i (i % 8 == 0 and the base 16-byte aligned).
__device__ __forceinline__ void kvm_ld8(const KvmBuf& b, size_t i, float (&v)[8]) {
  if (b.dtype == KVM_BF16) {
    uint4 u = *(const uint4*)((const __nv_bfloat16*)b.p + i);
    const __nv_bfloat162* h = (const __nv_bfloat162*)&u;
#pragma unroll
    for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
  } else {
    float4 a = *(const float4*)((const float*)b.p + i), c = *(const float4*)((const float*)b.p + i + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  }
}
__device__ __forceinline__ void kvm_st8(const KvmBuf& b, size_t i, const float (&v)[8]) {
  if (b.dtype == KVM_BF16) {
    uint4 u;
    __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    *(uint4*)((__nv_bfloat16*)b.p + i) = u;
  } else {
    *(float4*)((float*)b.p + i) = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)((float*)b.p + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}
template <bool BF>
__device__ __forceinline__ void kvm_ld8t(const void* p, size_t i, float (&v)[8]) {
  if (BF) {
    uint4 u = *(const uint4*)((const __nv_bfloat16*)p + i);
    const __nv_bfloat162* h = (const __nv_bfloat162*)&u;
#pragma unroll
    for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
  } else {
    float4 a = *(const float4*)((const float*)p + i), c = *(const float4*)((const float*)p + i + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
  }
}
template <bool BF>
__device__ __forceinline__ void kvm_st8t(void* p, size_t i, const float (&v)[8]) {
  if (BF) {
    uint4 u;
    __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
    *(uint4*)((__nv_bfloat16*)p + i) = u;
  } else {
    *(float4*)((float*)p + i) = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)((float*)p + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}
__device__ __forceinline__ bool kvm_vec_ok(const KvmBuf& b) { return ((uintptr_t)b.p & 15) == 0; }

// ---- argument checking ------------------------------------------------------------------------------------------------------
// Mask bits for accepted dtypes.
#define KVM_M_F32 1
#define KVM_M_I32 2
#define KVM_M_BF16 4
#define KVM_M_FLT (KVM_M_F32 | KVM_M_BF16)

// Op bodies are inlined into the dispatcher.  For a per-op report of registers and spills from the compiler (-Xptxas -v), build once
// with -DKVM_OPS_NOINLINE: every op then is a function of its own (measured 3% slower on a training step, so not the default).
#ifdef KVM_OPS_NOINLINE
#define KVM_OP_FN static __device__ __noinline__
#else
#define KVM_OP_FN static __device__
#endif

// Fetch table entry `idx` (an argument word). Optional buffers: idx == -1 gives p == nullptr and returns true.
__device__ __forceinline__ bool kvm_buf(const KvmCtx& c, int idx, int mask, KvmBuf& out, bool optional = false) {
  if (idx == -1 && optional) { out.p = nullptr; out.rows = out.cols = out.ld = 0; out.dtype = 0; return true; }
  if (idx < 0 || idx >= c.nbufs) { c.fail(KVM_OPE_BUF, idx); return false; }
  out = c.bufs[idx];
  if (out.p == nullptr || !((1 << out.dtype) & mask)) { c.fail(KVM_OPE_DTYPE, idx, out.dtype); return false; }
  return true;
}
// A flat op needs a contiguous buffer holding at least n elements.
__device__ __forceinline__ bool kvm_flat_ok(const KvmCtx& c, const KvmBuf& b, long long n) {
  if (!b.p) return true;
  if (b.ld != b.cols || n > (long long)b.rows * b.cols) { c.fail(KVM_OPE_RANGE, (int)n, b.rows * b.cols); return false; }
  return true;
}
// A matrix op needs rows x cols inside the buffer.
__device__ __forceinline__ bool kvm_mat_ok(const KvmCtx& c, const KvmBuf& b, long long rows, long long cols) {
  if (!b.p) return true;
  if (rows > b.rows || cols > b.cols) { c.fail(KVM_OPE_RANGE, (int)rows, (int)cols); return false; }
  return true;
}

// ---- reductions (fixed order: deterministic for a given launch geometry) ----------------------------------------------------
__device__ __forceinline__ float kvm_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double kvm_warp_sum(double v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float kvm_warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Named barrier over the KVM_NT compute threads only (barrier 1; barrier 0 = whole CTA including the scheduler warp).
__device__ __forceinline__ void kvm_sync() { asm volatile("bar.sync 1, %0;" ::"n"(KVM_NT) : "memory"); }

// Block-wide sum; `red` is a KVM_NWARPS-element shared scratch. All compute threads get the result.
template <class T>
__device__ __forceinline__ T kvm_block_sum(T v, T* red) {
  v = kvm_warp_sum(v);
  kvm_sync();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  kvm_sync();
  T s = 0;
#pragma unroll
  for (int w = 0; w < KVM_NWARPS; ++w) s += red[w];
  return s;
}
__device__ __forceinline__ float kvm_block_max(float v, float* red) {
  v = kvm_warp_max(v);
  kvm_sync();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  kvm_sync();
  float s = red[0];
#pragma unroll
  for (int w = 1; w < KVM_NWARPS; ++w) s = fmaxf(s, red[w]);
  return s;
}

__device__ __forceinline__ unsigned long long kvm_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned kvm_smid() {
  unsigned r;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
  return r;
}
