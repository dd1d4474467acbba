// libkvm_b200.so: host side of the executor (bundle validation, device tables, launch, results) and the C ABI of
// include/kvm_b200.h.  Mirrors what the reference's MvmExec does around its persistent kernel (mvm_exec.cu:492-1677):
// own the device buffers, check a batch before it reaches the device, launch one persistent kernel, read back counters.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -shared (see kvm_b200/build.py).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "kvm_json.hpp"
#include "kvm_dispatch.cuh"
#include "kvm_sched.cuh"
#include "kvm_static_api.h"

// ---------------------------------------------------------------------------------------------------------------- registry
struct KvmOpInfo { const char* name; int id; const char* sig; int arity; unsigned char types[KVM_MAX_ARGS]; };   // type 0 i32, 1 f32, 2 buf, 3 buf?
static std::vector<KvmOpInfo> g_ops;
static const KvmOpInfo* kvm_find_op(int id) {
  if (g_ops.empty()) {
    const struct { const char* n; int id; const char* s; } raw[] = {
#define KVM_OP(name, id, sig) {#name, id, sig},
#include "../../include/kvm_ops.def"
#undef KVM_OP
    };
    for (auto& r : raw) {
      KvmOpInfo o{r.n, r.id, r.s, 0, {}};
      const char* p = r.s;
      while (*p) {
        const char* colon = strchr(p, ':');
        if (!colon) break;
        const char* end = strchr(colon, ',');
        std::string ty(colon + 1, end ? end - colon - 1 : strlen(colon + 1));
        o.types[o.arity++] = ty == "i32" ? 0 : ty == "f32" ? 1 : ty == "buf" ? 2 : 3;
        if (!end) break;
        p = end + 1;
      }
      g_ops.push_back(o);
    }
  }
  for (auto& o : g_ops) if (o.id == id) return &o;
  return nullptr;
}

// ---------------------------------------------------------------------------------------------------------------- init kernels
// Seeded init: SplitMix64 at counter i*draws+d, u = (z >> 40) * 2^-24, every step one rounded float32 operation
// (reference: runtime/initgen.py:1-58, device twin include/mvm_exec.cuh:1089-1115).  Bit-exact requirement.
__device__ __forceinline__ float kvm_seeded_u(unsigned long long seed, unsigned long long j) {
  unsigned long long z = seed + (j + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return __fmul_rn((float)(z >> 40), 1.0f / 16777216.0f);
}
__global__ void kvm_seeded_kernel(void* p, size_t n, unsigned long long seed, int draws, float bias, float coef, int dtype) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc;
    if (draws == 1) acc = kvm_seeded_u(seed, i);
    else {
      const unsigned long long j = i * (unsigned long long)draws;
      acc = __fadd_rn(__fadd_rn(kvm_seeded_u(seed, j), kvm_seeded_u(seed, j + 1)), __fadd_rn(kvm_seeded_u(seed, j + 2), kvm_seeded_u(seed, j + 3)));
    }
    const float v = __fmul_rn(__fsub_rn(acc, bias), coef);
    if (dtype == KVM_BF16) ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
    else ((float*)p)[i] = v;
  }
}
__global__ void kvm_fill_kernel(void* p, size_t n, int dtype, double value) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    if (dtype == KVM_I32) ((int*)p)[i] = (int)value;
    else if (dtype == KVM_BF16) ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn((float)value);
    else ((float*)p)[i] = (float)value;
  }
}
__global__ void kvm_widen_kernel(const void* p, float* out, size_t n, int dtype) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = dtype == KVM_I32 ? (float)((const int*)p)[i] : dtype == KVM_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// ---------------------------------------------------------------------------------------------------------------- host state
#include "kvm_host.inl"

// ---------------------------------------------------------------------------------------------------------------- read-back without allocation
// kvm_read_buffer widens bf16 / i32 storage to float32 in a temporary device buffer it gets from cudaMalloc and frees again.
// A serving loop that reads logits or sampled tokens back every decode step cannot afford that: cudaMalloc and cudaFree
// synchronise the whole device, which stalls every other stream (and any persistent executor running beside the reader).
// This variant widens into a fixed scratch array that lives in the library image instead: KVM_NOALLOC_MAX_ELEMS floats (4 MiB)
// per GPU that loads the library, held until the process exits.  It allocates nothing, but it is an ordinary blocking read:
// it launches on `stream`, copies, and synchronises that stream before it returns, so `stream` must not be capturing (and
// NULL means the legacy default stream: pass a non-blocking stream of your own when other streams should keep running).
//
// The array is shared by every call on that GPU and keeps whatever the last call left in it.  Nothing in it has to start at
// zero: each call overwrites exactly the n elements it then copies out and never reads beyond them.  Two calls whose device work
// overlaps on one GPU (different streams, or different host threads) race on the array; callers serialise them.
//
// In host code `kvm_noalloc_scratch` is only a stand-in for the symbol, not a device address, so the address is taken with
// cudaGetSymbolAddress, once per device, with that device current, by the first call on the device (which therefore should
// happen before any stream capture starts anywhere in the process); later calls reuse the cached pointer and do no set-up.
// The caller's current device is put back before the call returns.
static __device__ __align__(256) float kvm_noalloc_scratch[KVM_NOALLOC_MAX_ELEMS];
#define KVM_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[KVM_NOALLOC_MAX_DEVICES];
static char g_noalloc_error[256] = "";

extern "C" const char* kvm_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int kvm_read_f32_noalloc(int32_t device, const void* dev_src, int32_t dtype, size_t n, float* host_out, void* stream) {
  int prev_device = -1;
  auto done = [&](int code, const char* what, cudaError_t e) {
    if (code == 0) g_noalloc_error[0] = 0;
    else if (e != cudaSuccess) snprintf(g_noalloc_error, sizeof g_noalloc_error, "kvm_read_f32_noalloc: %s: %s", what, cudaGetErrorString(e));
    else snprintf(g_noalloc_error, sizeof g_noalloc_error, "kvm_read_f32_noalloc: %s", what);
    if (prev_device >= 0 && prev_device != device) cudaSetDevice(prev_device);
    return code;
  };
  if (device < 0 || device >= KVM_NOALLOC_MAX_DEVICES || !dev_src || !host_out || dtype < 0 || dtype > 2) return done(KVM_E_ARG, "bad device, pointer or dtype", cudaSuccess);
  if (n > (size_t)KVM_NOALLOC_MAX_ELEMS) {
    snprintf(g_noalloc_error, sizeof g_noalloc_error, "kvm_read_f32_noalloc: %zu elements exceed the fixed scratch of %u (KVM_NOALLOC_MAX_ELEMS); read in pieces or use kvm_read_buffer",
             n, (unsigned)KVM_NOALLOC_MAX_ELEMS);
    return KVM_E_ARG;
  }
  if (n == 0) return done(0, "", cudaSuccess);
  cudaError_t e = cudaGetDevice(&prev_device);
  if (e != cudaSuccess) { prev_device = -1; return done(KVM_E_CUDA, "cudaGetDevice", e); }
  if ((e = cudaSetDevice(device)) != cudaSuccess) return done(KVM_E_CUDA, "cudaSetDevice", e);
  if (!g_noalloc_ptr[device]) {      // set-up, once per device, with that device current
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, kvm_noalloc_scratch);
    if (e != cudaSuccess || !p) return done(KVM_E_CUDA, "cudaGetSymbolAddress(kvm_noalloc_scratch)", e);
    g_noalloc_ptr[device] = p;
  }
  float* scratch = g_noalloc_ptr[device];
  cudaStream_t st = (cudaStream_t)stream;
  const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
  kvm_widen_kernel<<<blocks, 256, 0, st>>>(dev_src, scratch, n, dtype);
  if ((e = cudaGetLastError()) != cudaSuccess) return done(KVM_E_CUDA, "kernel launch", e);
  if ((e = cudaMemcpyAsync(host_out, scratch, n * sizeof(float), cudaMemcpyDeviceToHost, st)) != cudaSuccess) return done(KVM_E_CUDA, "cudaMemcpyAsync", e);
  if ((e = cudaStreamSynchronize(st)) != cudaSuccess) return done(KVM_E_CUDA, "cudaStreamSynchronize", e);
  return done(0, "", cudaSuccess);
}
