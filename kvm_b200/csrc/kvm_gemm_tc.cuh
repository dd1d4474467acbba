// tcgen05 / TMEM / TMA GEMM tile path (placeholder while the SIMT executor is brought up).
#pragma once
#include "kvm_dev.cuh"
#include "kvm_ops_mm.cuh"
__device__ __forceinline__ void kvm_tc_init(int* ctl, unsigned char* smem) {}
__device__ __forceinline__ void kvm_tc_fini(int* ctl) {}
__device__ void kvm_op_matmul_mma_bf16(const KvmCtx& c, const int32_t* a, const int4& aux) {
  KvmMmArgs g;
  if (kvm_mm_args(c, a, 2, g)) kvm_mm_simt(c, g);
}
