// The op dispatcher: one switch from op id to op body, expanded into each executor kernel that includes this header (the two
// kernels live in translation units of their own so that they compile side by side; a device function is private to its unit).
#pragma once
#include "kvm_dev.cuh"
#include "kvm_ops_flat.cuh"
#include "kvm_ops_rows.cuh"
#include "kvm_ops_mm.cuh"
#include "kvm_ops_attn.cuh"
#include "kvm_ops_decode.cuh"
#include "kvm_ops_peer.cuh"
#include "kvm_gemm_tc.cuh"
#include "kvm_attn_tc.cuh"
#include "kvm_state.cuh"

static __device__ void kvm_dispatch(const KvmCtx& c, int op, const int32_t* a, const int4& aux) {
  switch (op) {
    case 1: kvm_op_copy(c, a); break;
    case 2: kvm_op_add(c, a); break;
    case 3: kvm_op_scale(c, a); break;
    case 4: kvm_op_relu(c, a); break;
    case 5: kvm_op_sgd(c, a); break;
    case 6: kvm_op_predict(c, a); break;
    case 7: kvm_op_mse_grad(c, a); break;
    case 8: kvm_op_matmul(c, a); break;
    case 9: kvm_op_fill(c, a); break;
    case 10: kvm_op_spin(c, a); break;
    case 32: kvm_op_embedding_fwd(c, a); break;
    case 33: kvm_op_embedding_bwd(c, a); break;
    case 34: kvm_op_matmul_tile(c, a); break;
    case 35: kvm_op_layernorm_fwd(c, a); break;
    case 36: kvm_op_rmsnorm_fwd(c, a); break;
    case 37: kvm_op_layernorm_bwd_dx(c, a); break;
    case 38: kvm_op_rmsnorm_bwd_dx(c, a); break;
    case 39: kvm_op_norm_bwd_params(c, a); break;
    case 40: kvm_op_gelu_fwd(c, a); break;
    case 41: kvm_op_gelu_bwd(c, a); break;
    case 42: kvm_op_residual_add(c, a); break;
    case 43: kvm_op_rope_fwd(c, a); break;
    case 44: kvm_op_rope_bwd(c, a); break;
    case 45: if ((aux.x & 255) == 2 && !(c.cfg_flags & KVM_CFG_NO_TENSOR_CORES)) kvm_attn_fwd_tc(c, a, aux); else kvm_op_attn_fwd(c, a); break;
    case 46: kvm_op_attn_bwd_delta(c, a); break;
    case 47: if ((aux.x & 255) == 2 && !(c.cfg_flags & KVM_CFG_NO_TENSOR_CORES)) kvm_attn_dq_tc(c, a, aux); else kvm_op_attn_bwd_dq(c, a); break;
    case 48: if ((aux.x & 255) == 2 && !(c.cfg_flags & KVM_CFG_NO_TENSOR_CORES)) kvm_attn_dkv_tc(c, a, aux); else kvm_op_attn_bwd_dkv(c, a); break;
    case 49: kvm_op_kv_append(c, a); break;
    case 50: kvm_op_attn_decode(c, a); break;
    case 51: kvm_op_softmax_ce_fwd(c, a); break;
    case 52: kvm_op_softmax_ce_reduce(c, a); break;
    case 53: kvm_op_softmax_ce_bwd(c, a); break;
    case 54: kvm_op_adamw(c, a); break;
    case 55: kvm_op_gradnorm_partial(c, a); break;
    case 56: kvm_op_gradnorm_finish(c, a); break;
    case 57: kvm_op_sample(c, a); break;
    case 58: kvm_op_argmax(c, a); break;
    case 59: kvm_op_zero_buf(c, a); break;
    case 60: kvm_op_counter_inc(c, a); break;
    case 61: kvm_op_colsum(c, a); break;
    case 62: kvm_op_select_window(c, a); break;
    case 63: kvm_op_gather_rows(c, a); break;
    case 96: kvm_op_act_fwd(c, a); break;
    case 97: kvm_op_act_bwd(c, a); break;
    case 98: kvm_op_silu_mul_fwd(c, a); break;
    case 113: kvm_op_round_bf16(c, a); break;
    case 114: kvm_op_matmul_tile_bf16(c, a); break;
    case 115: kvm_op_adamw_lr(c, a); break;
    case 116: kvm_op_lr_schedule(c, a); break;
    case 117: kvm_op_scale_flat(c, a); break;
    case 118: kvm_op_add_rowtile(c, a); break;
    case 122: kvm_op_matmul_mma_bf16(c, a, aux); break;
    case 123: kvm_op_sgd_range(c, a); break;
    case 126: kvm_op_round_tf32(c, a); break;
    case 127: kvm_op_softmax_ce_fused(c, a); break;
    case 134: kvm_op_gemv_bf16(c, a); break;
    case 135: kvm_op_attn_decode_part(c, a); break;
    case 136: kvm_op_attn_decode_merge(c, a); break;
    case 300: kvm_op_attn_decode_part_qkn(c, a); break;
    case 301: kvm_op_gemv_bf16_rows(c, a); break;
    case 302: kvm_op_peer_put_signal(c, a); break;
    case 303: kvm_op_peer_wait_sum(c, a); break;
    case 304: kvm_op_peer_wait(c, a); break;
    default: c.fail(KVM_ERR_BAD_OP, op); break;
  }
}

