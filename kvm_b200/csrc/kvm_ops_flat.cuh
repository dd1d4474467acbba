// Memory-bound elementwise ops over a flat range [e0,e1): 128-bit accesses, two batches of loads in flight per thread.
// Reference semantics: runtime/ref_ops.py:17-60, runtime/ref_gpt.py:196-247, runtime/ref_extra.py:56-72,306-310,350-360.
#pragma once
#include "kvm_dev.cuh"

// out[i] = f(in0[i], in1[i], ...) for i in [e0,e1).  NI inputs; `out` may alias an input.  F: float(const float (&x)[NI]).
template <int NI, class F>
__device__ __forceinline__ void kvm_flat_map(const KvmBuf (&in)[NI], const KvmBuf& out, long long e0, long long e1, F f) {
  bool vec = (e0 & 7) == 0 && kvm_vec_ok(out);
#pragma unroll
  for (int k = 0; k < NI; ++k) vec = vec && kvm_vec_ok(in[k]);
  long long body = vec ? ((e1 - e0) & ~7LL) : 0;
  const long long step = (long long)KVM_NT * 8;
  long long i = e0 + (long long)threadIdx.x * 8;
  // two vectors per thread per trip: all loads issued before the first store
  for (; i + step + 8 <= e0 + body; i += 2 * step) {
    float a[NI][8], b[NI][8], ra[8], rb[8];
#pragma unroll
    for (int k = 0; k < NI; ++k) { kvm_ld8(in[k], i, a[k]); kvm_ld8(in[k], i + step, b[k]); }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float xa[NI], xb[NI];
#pragma unroll
      for (int k = 0; k < NI; ++k) { xa[k] = a[k][j]; xb[k] = b[k][j]; }
      ra[j] = f(xa); rb[j] = f(xb);
    }
    kvm_st8(out, i, ra); kvm_st8(out, i + step, rb);
  }
  for (; i + 8 <= e0 + body; i += step) {
    float a[NI][8], ra[8];
#pragma unroll
    for (int k = 0; k < NI; ++k) kvm_ld8(in[k], i, a[k]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float xa[NI];
#pragma unroll
      for (int k = 0; k < NI; ++k) xa[k] = a[k][j];
      ra[j] = f(xa);
    }
    kvm_st8(out, i, ra);
  }
  for (long long s = e0 + body + threadIdx.x; s < e1; s += KVM_NT) {
    float x[NI];
#pragma unroll
    for (int k = 0; k < NI; ++k) x[k] = kvm_ld(in[k], s);
    kvm_st(out, s, f(x));
  }
}

__device__ __forceinline__ bool kvm_range_ok(const KvmCtx& c, long long e0, long long e1) {
  if (e0 < 0 || e1 < e0) { c.fail(KVM_OPE_RANGE, (int)e0, (int)e1); return false; }
  return true;
}

__device__ __forceinline__ float kvm_gelu(float x) {
  return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float kvm_gelu_grad(float x) {
  float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
}
__device__ __forceinline__ float kvm_sigmoid(float x) {
  float e = expf(-fabsf(x));
  return x >= 0 ? 1.0f / (1.0f + e) : e / (1.0f + e);
}
__device__ __forceinline__ float kvm_silu(float x) { return x * kvm_sigmoid(x); }
__device__ __forceinline__ float kvm_act(int kind, float x) {
  switch (kind) {
    case 0: return x > 0 ? x : 0.0f;
    case 1: return kvm_silu(x);
    case 2: return tanhf(x);
    default: return kvm_sigmoid(x);
  }
}
__device__ __forceinline__ float kvm_act_grad(int kind, float x) {
  switch (kind) {
    case 0: return x > 0 ? 1.0f : 0.0f;
    case 1: { float s = kvm_sigmoid(x); return s * (1.0f + x * (1.0f - s)); }
    case 2: { float t = tanhf(x); return 1.0f - t * t; }
    default: { float s = kvm_sigmoid(x); return s * (1.0f - s); }
  }
}
__device__ __forceinline__ float kvm_tf32_round(float x) {
  unsigned u = __float_as_uint(x);
  if ((u & 0x7fffffffu) <= 0x7f800000u) u += 0x1000u;
  return __uint_as_float(u & 0xffffe000u);
}

// ---- core pack: n elements from 0 --------------------------------------------------------------------------------------------
KVM_OP_FN void kvm_op_copy(const KvmCtx& c, const int32_t* a) {
  KvmBuf s, d;
  if (!kvm_buf(c, a[0], 7, s) || !kvm_buf(c, a[1], 7, d)) return;
  long long n = a[2];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, s, n) || !kvm_flat_ok(c, d, n)) return;
  if (s.dtype != d.dtype) { c.fail(KVM_OPE_DTYPE, a[0], a[1]); return; }
  if (s.dtype == KVM_BF16) { for (long long i = threadIdx.x; i < n; i += KVM_NT) ((uint16_t*)d.p)[i] = ((const uint16_t*)s.p)[i]; }
  else { for (long long i = threadIdx.x; i < n; i += KVM_NT) ((uint32_t*)d.p)[i] = ((const uint32_t*)s.p)[i]; }
}
KVM_OP_FN void kvm_op_add(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[2], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, in[1]) || !kvm_buf(c, a[2], KVM_M_FLT, o)) return;
  long long n = a[3];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, in[0], n) || !kvm_flat_ok(c, in[1], n) || !kvm_flat_ok(c, o, n)) return;
  kvm_flat_map<2>(in, o, 0, n, [](const float (&x)[2]) { return __fadd_rn(x[0], x[1]); });
}
KVM_OP_FN void kvm_op_scale(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  float al = kvm_bits_f32(a[2]);
  long long n = a[3];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, in[0], n) || !kvm_flat_ok(c, o, n)) return;
  kvm_flat_map<1>(in, o, 0, n, [al](const float (&x)[1]) { return __fmul_rn(x[0], al); });
}
KVM_OP_FN void kvm_op_relu(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  long long n = a[2];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, in[0], n) || !kvm_flat_ok(c, o, n)) return;
  kvm_flat_map<1>(in, o, 0, n, [](const float (&x)[1]) { return x[0] > 0 ? x[0] : 0.0f; });
}
static __device__ void kvm_sgd_common(const KvmCtx& c, int wi, int gi, float lr, long long e0, long long e1) {
  KvmBuf in[2];
  if (!kvm_buf(c, wi, KVM_M_F32, in[0]) || !kvm_buf(c, gi, KVM_M_FLT, in[1])) return;
  if (!kvm_range_ok(c, e0, e1) || !kvm_flat_ok(c, in[0], e1) || !kvm_flat_ok(c, in[1], e1)) return;
  kvm_flat_map<2>(in, in[0], e0, e1, [lr](const float (&x)[2]) { return __fsub_rn(x[0], __fmul_rn(lr, x[1])); });
}
KVM_OP_FN void kvm_op_sgd(const KvmCtx& c, const int32_t* a) { kvm_sgd_common(c, a[0], a[1], kvm_bits_f32(a[2]), 0, a[3]); }
KVM_OP_FN void kvm_op_sgd_range(const KvmCtx& c, const int32_t* a) { kvm_sgd_common(c, a[0], a[1], kvm_bits_f32(a[2]), a[3], a[4]); }
KVM_OP_FN void kvm_op_predict(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], w, o;
  if (!kvm_buf(c, a[0], KVM_M_F32, in[0]) || !kvm_buf(c, a[1], KVM_M_F32, w) || !kvm_buf(c, a[2], KVM_M_F32, o)) return;
  long long n = a[3];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, in[0], n) || !kvm_flat_ok(c, o, n)) return;
  float w0 = ((const float*)w.p)[0];
  kvm_flat_map<1>(in, o, 0, n, [w0](const float (&x)[1]) { return __fmul_rn(w0, x[0]); });
}
// loss[0] = mean((p-t)^2), grad[0] = mean(2(p-t)x): float32 sums in index order (runtime/ref_ops.py:44-52), so one thread.
KVM_OP_FN void kvm_op_mse_grad(const KvmCtx& c, const int32_t* a) {
  KvmBuf p, t, x, l, g;
  if (!kvm_buf(c, a[0], KVM_M_F32, p) || !kvm_buf(c, a[1], KVM_M_F32, t) || !kvm_buf(c, a[2], KVM_M_F32, x) || !kvm_buf(c, a[3], KVM_M_F32, l) ||
      !kvm_buf(c, a[4], KVM_M_F32, g)) return;
  int n = a[5];
  if (n < 1 || !kvm_flat_ok(c, p, n) || !kvm_flat_ok(c, t, n) || !kvm_flat_ok(c, x, n)) { c.fail(KVM_OPE_RANGE, n); return; }
  if (threadIdx.x == 0) {
    float la = 0, ga = 0;
    for (int i = 0; i < n; ++i) {
      float d = __fsub_rn(((const float*)p.p)[i], ((const float*)t.p)[i]);
      la = __fadd_rn(la, __fmul_rn(d, d));
      ga = __fadd_rn(ga, __fmul_rn(__fmul_rn(2.0f, d), ((const float*)x.p)[i]));
    }
    ((float*)l.p)[0] = (float)((double)la / n);
    ((float*)g.p)[0] = (float)((double)ga / n);
  }
}
KVM_OP_FN void kvm_op_fill(const KvmCtx& c, const int32_t* a) {
  KvmBuf x;
  if (!kvm_buf(c, a[0], 7, x)) return;
  long long n = a[2];
  if (!kvm_range_ok(c, 0, n) || !kvm_flat_ok(c, x, n)) return;
  float v = kvm_bits_f32(a[1]);
  if (x.dtype == KVM_I32) { for (long long i = threadIdx.x; i < n; i += KVM_NT) ((int*)x.p)[i] = (int)v; }
  else { for (long long i = threadIdx.x; i < n; i += KVM_NT) kvm_st(x, i, v); }
}
KVM_OP_FN void kvm_op_spin(const KvmCtx& c, const int32_t* a) {
  if (threadIdx.x == 0) {
    unsigned long long t0 = kvm_globaltimer(), lim = (unsigned long long)(a[0] < 0 ? 0 : (a[0] > 1000000 ? 1000000 : a[0])) * 1000ull;
    while (kvm_globaltimer() - t0 < lim) __nanosleep(200);
  }
}

// ---- GPT / extra packs -----------------------------------------------------------------------------------------------------------
KVM_OP_FN void kvm_op_gelu_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  if (!kvm_range_ok(c, a[2], a[3]) || !kvm_flat_ok(c, in[0], a[3]) || !kvm_flat_ok(c, o, a[3])) return;
  kvm_flat_map<1>(in, o, a[2], a[3], [](const float (&x)[1]) { return kvm_gelu(x[0]); });
}
// dx (+)= f'(x) * dy with one float32 rounding of the product, then one of the sum (runtime/ref_gpt.py:202-206).
template <class G>
__device__ __forceinline__ void kvm_bwd_map(const KvmCtx& c, int xi, int dyi, int dxi, long long e0, long long e1, int acc, G grad) {
  KvmBuf in[3];
  if (!kvm_buf(c, xi, KVM_M_FLT, in[0]) || !kvm_buf(c, dyi, KVM_M_FLT, in[1]) || !kvm_buf(c, dxi, KVM_M_FLT, in[2])) return;
  if (!kvm_range_ok(c, e0, e1) || !kvm_flat_ok(c, in[0], e1) || !kvm_flat_ok(c, in[1], e1) || !kvm_flat_ok(c, in[2], e1)) return;
  if (acc) kvm_flat_map<3>(in, in[2], e0, e1, [grad](const float (&x)[3]) { return __fadd_rn(x[2], __fmul_rn(x[1], grad(x[0]))); });
  else {
    KvmBuf in2[2] = {in[0], in[1]};
    kvm_flat_map<2>(in2, in[2], e0, e1, [grad](const float (&x)[2]) { return __fmul_rn(x[1], grad(x[0])); });
  }
}
KVM_OP_FN void kvm_op_gelu_bwd(const KvmCtx& c, const int32_t* a) {
  kvm_bwd_map(c, a[0], a[1], a[2], a[3], a[4], a[5], [](float x) { return kvm_gelu_grad(x); });
}
KVM_OP_FN void kvm_op_act_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  int kind = a[2];
  if (kind < 0 || kind > 3) { c.fail(KVM_OPE_RANGE, kind); return; }
  if (!kvm_range_ok(c, a[3], a[4]) || !kvm_flat_ok(c, in[0], a[4]) || !kvm_flat_ok(c, o, a[4])) return;
  kvm_flat_map<1>(in, o, a[3], a[4], [kind](const float (&x)[1]) { return kvm_act(kind, x[0]); });
}
KVM_OP_FN void kvm_op_act_bwd(const KvmCtx& c, const int32_t* a) {
  int kind = a[3];
  if (kind < 0 || kind > 3) { c.fail(KVM_OPE_RANGE, kind); return; }
  kvm_bwd_map(c, a[0], a[1], a[2], a[4], a[5], a[6], [kind](float x) { return kvm_act_grad(kind, x); });
}
KVM_OP_FN void kvm_op_silu_mul_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[2], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, in[1]) || !kvm_buf(c, a[2], KVM_M_FLT, o)) return;
  if (!kvm_range_ok(c, a[3], a[4]) || !kvm_flat_ok(c, in[0], a[4]) || !kvm_flat_ok(c, in[1], a[4]) || !kvm_flat_ok(c, o, a[4])) return;
  kvm_flat_map<2>(in, o, a[3], a[4], [](const float (&x)[2]) { return kvm_silu(x[0]) * x[1]; });
}
KVM_OP_FN void kvm_op_residual_add(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[2], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, in[1]) || !kvm_buf(c, a[2], KVM_M_FLT, o)) return;
  if (!kvm_range_ok(c, a[3], a[4]) || !kvm_flat_ok(c, in[0], a[4]) || !kvm_flat_ok(c, in[1], a[4]) || !kvm_flat_ok(c, o, a[4])) return;
  kvm_flat_map<2>(in, o, a[3], a[4], [](const float (&x)[2]) { return __fadd_rn(x[0], x[1]); });
}
KVM_OP_FN void kvm_op_round_tf32(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_F32, in[0]) || !kvm_buf(c, a[1], KVM_M_F32, o)) return;
  if (!kvm_range_ok(c, a[2], a[3]) || !kvm_flat_ok(c, in[0], a[3]) || !kvm_flat_ok(c, o, a[3])) return;
  kvm_flat_map<1>(in, o, a[2], a[3], [](const float (&x)[1]) { return kvm_tf32_round(x[0]); });
}
// f32 -> bf16 narrows (RNE), bf16 -> f32 widens, f32 -> f32 emulates, bf16 -> bf16 copies (include/mvm_ops_extra.def:63-66).
KVM_OP_FN void kvm_op_round_bf16(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  if (!kvm_range_ok(c, a[2], a[3]) || !kvm_flat_ok(c, in[0], a[3]) || !kvm_flat_ok(c, o, a[3])) return;
  kvm_flat_map<1>(in, o, a[2], a[3], [](const float (&x)[1]) { return kvm_bf16_round(x[0]); });
}
KVM_OP_FN void kvm_op_scale_flat(const KvmCtx& c, const int32_t* a) {
  KvmBuf in[1], o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, in[0]) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  float al = kvm_bits_f32(a[2]);
  if (!kvm_range_ok(c, a[3], a[4]) || !kvm_flat_ok(c, in[0], a[4]) || !kvm_flat_ok(c, o, a[4])) return;
  kvm_flat_map<1>(in, o, a[3], a[4], [al](const float (&x)[1]) { return __fmul_rn(al, x[0]); });
}
KVM_OP_FN void kvm_op_zero_buf(const KvmCtx& c, const int32_t* a) {
  KvmBuf x;
  if (!kvm_buf(c, a[0], 7, x)) return;
  long long e0 = a[1], e1 = a[2];
  if (!kvm_range_ok(c, e0, e1) || !kvm_flat_ok(c, x, e1)) return;
  if (x.dtype == KVM_BF16) { for (long long i = e0 + threadIdx.x; i < e1; i += KVM_NT) ((uint16_t*)x.p)[i] = 0; }
  else { for (long long i = e0 + threadIdx.x; i < e1; i += KVM_NT) ((uint32_t*)x.p)[i] = 0; }
}
KVM_OP_FN void kvm_op_counter_inc(const KvmCtx& c, const int32_t* a) {
  KvmBuf x;
  if (!kvm_buf(c, a[0], KVM_M_I32, x)) return;
  if (!kvm_range_ok(c, a[1], a[2]) || !kvm_flat_ok(c, x, a[2])) return;
  for (long long i = a[1] + threadIdx.x; i < a[2]; i += KVM_NT) ((unsigned*)x.p)[i] += (unsigned)a[3];
}
// dst[i] = src[step[0]*stride + off + i], any 4-byte dtype (include/mvm_ops_gpt.def:86-88).
KVM_OP_FN void kvm_op_select_window(const KvmCtx& c, const int32_t* a) {
  KvmBuf s, st, d;
  if (!kvm_buf(c, a[0], KVM_M_F32 | KVM_M_I32, s) || !kvm_buf(c, a[1], KVM_M_I32, st) || !kvm_buf(c, a[2], KVM_M_F32 | KVM_M_I32, d)) return;
  if (s.dtype != d.dtype) { c.fail(KVM_OPE_DTYPE, a[0], a[2]); return; }
  long long i0 = a[3], i1 = a[4], base = (long long)((const int*)st.p)[0] * a[5] + a[6];
  if (!kvm_range_ok(c, i0, i1) || !kvm_flat_ok(c, d, i1)) return;
  if (base < 0 || s.ld != s.cols || base + i1 > (long long)s.rows * s.cols) { c.fail(KVM_OPE_RANGE, (int)base, (int)i1); return; }
  for (long long i = i0 + threadIdx.x; i < i1; i += KVM_NT) ((uint32_t*)d.p)[i] = ((const uint32_t*)s.p)[base + i];
}
