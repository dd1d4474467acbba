// Translation unit of the static-schedule kernels (kvm_static.cuh) and their host-callable launchers.
#include "kvm_static.cuh"

cudaError_t kvm_static_set_smem(int bytes) { return cudaFuncSetAttribute(kvm_static_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes); }
void kvm_static_launch(const KvmStaticState& T, int workers, int smem_bytes, cudaStream_t stream) { kvm_static_kernel<<<workers, KVM_NT + 32, smem_bytes, stream>>>(T); }
void kvm_static_arm(const KvmStaticState& T, int workers, int blocks, cudaStream_t stream) { kvm_static_arm_kernel<<<blocks, 256, 0, stream>>>(T, workers); }
