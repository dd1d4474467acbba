// Host-callable entry points of the static-schedule kernels, which are compiled in a translation unit of their own
// (kvm_static.cu) beside the ready-queue kernel's (kvm_exec.cu).
#pragma once
#include <cuda_runtime.h>

#include "kvm_state.cuh"

#define KVM_ST_STAGE 65536             // bytes of one stream stage
#define KVM_ST_WAIT_BITS 20            // dependency entry: worker << 20 | tasks that worker must have finished

struct KvmStaticState {
  KvmDevState D;
  const int* prog;            // task indices, the workers' lists one after the other
  const int* prog_off;        // [workers + 1]
  const int* waits;           // dependency entries of all tasks (deduplicated lists)
  int* progress;              // [workers]: tasks finished by that worker (release stores)
  int ring;                   // 0: all shared memory is op scratch; 1: three 64 KB stream stages + 32 KB scratch (decode programs); 2: two stages + 96 KB scratch (programs with gemv_bf16_rows)
};

// record words beyond the ready-queue path's (descriptor 0..15, arguments 16..35, path selector 36..39)
#define KVM_REC_WAIT_OFF 40
#define KVM_REC_WAIT_CNT 41
#define KVM_REC_STREAM 42              // bit 0: streamed operand is constant during the launch (copies may run ahead of the dependencies)

cudaError_t kvm_static_set_smem(int bytes);
void kvm_static_launch(const KvmStaticState& T, int workers, int smem_bytes, cudaStream_t stream);
void kvm_static_arm(const KvmStaticState& T, int workers, int blocks, cudaStream_t stream);
