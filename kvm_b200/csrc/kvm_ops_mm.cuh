// GEMM tile ops, SIMT form: the bit-exact float32 path (matmul, matmul_tile) and the fallback of the bf16 tile ops for
// operands the tensor-core path cannot take (unaligned ld / base, f32 operands).  Accumulation is k-ascending with one
// rounded multiply and one rounded add per step, which is the reference's golden for every matmul flavour
// (runtime/ref_gpt.py:69-103, runtime/ref_extra.py:312-331), so results equal its CPU model bit for bit.
// The epilogue (shared with the tcgen05 path in kvm_gemm_tc.cuh) follows the reference order:
//   v = alpha*acc; + bias[n]; (flag 512: * gelu'(pre)) else (pre = v; flag 8: gelu); + res; (flag 4: out += v).
#pragma once
#include "kvm_dev.cuh"
#include "kvm_ops_flat.cuh"

struct KvmMmArgs {
  KvmBuf a, b, out, bias, res, pre;
  int m0, n0, M, N, K, flags;
  float alpha;
  int tm, tn;            // tile extent
  bool round_ops;        // operands rounded to bf16 on load
};

__device__ __forceinline__ float kvm_mm_epilogue(const KvmMmArgs& g, float acc, int m, int n) {
  float v = __fmul_rn(acc, g.alpha);
  if (g.bias.p) v = __fadd_rn(v, ((const float*)g.bias.p)[n]);
  if (g.flags & 512) v = v * kvm_gelu_grad(kvm_ld(g.pre, (size_t)m * g.pre.ld + n));
  else {
    if (g.pre.p) kvm_st(g.pre, (size_t)m * g.pre.ld + n, v);
    if (g.flags & 8) v = kvm_gelu(v);
  }
  if (g.res.p) v = __fadd_rn(v, kvm_ld(g.res, (size_t)m * g.res.ld + n));
  if (g.flags & 4) v = __fadd_rn(kvm_ld(g.out, (size_t)m * g.out.ld + n), v);
  return v;
}

// Decode and check the 13 argument words shared by matmul_tile / matmul_tile_bf16 / matmul_mma_bf16.
static __device__ bool kvm_mm_args(const KvmCtx& c, const int32_t* a, int kind /*0 f32 tile, 1 bf16 tile, 2 mma 128x256*/, KvmMmArgs& g) {
  const int opmask = kind == 0 ? KVM_M_F32 : KVM_M_FLT, omask = kind == 0 ? KVM_M_F32 : KVM_M_FLT;
  if (!kvm_buf(c, a[0], opmask, g.a) || !kvm_buf(c, a[1], opmask, g.b) || !kvm_buf(c, a[2], omask, g.out) || !kvm_buf(c, a[3], KVM_M_F32, g.bias, true) ||
      !kvm_buf(c, a[4], omask, g.res, true) || !kvm_buf(c, a[5], omask, g.pre, true)) return false;
  g.m0 = a[6]; g.n0 = a[7]; g.M = a[8]; g.N = a[9]; g.K = a[10]; g.flags = a[11]; g.alpha = kvm_bits_f32(a[12]);
  const int fl = g.flags;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.m0 < 0 || g.m0 >= g.M || g.n0 < 0 || g.n0 >= g.N) { c.fail(KVM_OPE_RANGE, g.m0, g.n0); return false; }
  const int allowed = kind == 2 ? (1 | 2 | 4 | 8) : (127 | 256 | 512 | 1024);
  if ((fl & ~allowed) || ((fl & 32) && (fl & 64)) || ((fl & 256) && (fl & 1024)) ||
      ((fl & 512) && (!g.pre.p || g.bias.p || g.res.p || (fl & (4 | 8 | 128))))) { c.fail(KVM_OPE_SHAPE, fl); return false; }
  if (kind == 2) { g.tm = 128; g.tn = 256; }
  else if (fl & 64) { g.tm = 256; g.tn = 128; }
  else if (fl & 32) { g.tm = 128; g.tn = 128; }
  else { g.tm = 64; g.tn = 64; }
  g.round_ops = kind != 0 || (fl & 128);
  const bool ta = fl & 1, tb = fl & 2;
  if (!kvm_mat_ok(c, g.a, ta ? g.K : g.M, ta ? g.M : g.K) || !kvm_mat_ok(c, g.b, tb ? g.N : g.K, tb ? g.K : g.N) || !kvm_mat_ok(c, g.out, g.M, g.N) ||
      !kvm_mat_ok(c, g.res, g.M, g.N) || !kvm_mat_ok(c, g.pre, g.M, g.N) || !kvm_flat_ok(c, g.bias, g.N)) return false;
  return true;
}

// SIMT tile: 64x64 sub-tiles, K staged through shared memory 32 at a time; thread = (row, 8 columns).
static __device__ void kvm_mm_simt(const KvmCtx& c, const KvmMmArgs& g) {
  float (*As)[65] = (float (*)[65])c.smem;                  // [32][65]: As[k][m]
  float (*Bs)[64] = (float (*)[64])(c.smem + 32 * 65 * 4);  // [32][64]: Bs[k][n]
  const bool ta = g.flags & 1, tb = g.flags & 2;
  const int m_end = min(g.m0 + g.tm, g.M), n_end = min(g.n0 + g.tn, g.N);
  const int row = threadIdx.x >> 3, cg = (threadIdx.x & 7) * 8;
  for (int mb = g.m0; mb < m_end; mb += 64)
    for (int nb = g.n0; nb < n_end; nb += 64) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
      for (int k0 = 0; k0 < g.K; k0 += 32) {
        kvm_sync();
        for (int e = threadIdx.x; e < 32 * 64; e += KVM_NT) {
          int kk, mm;
          if (ta) { kk = e >> 6; mm = e & 63; } else { mm = e >> 5; kk = e & 31; }
          float v = 0.0f;
          if (k0 + kk < g.K && mb + mm < m_end) {
            v = ta ? kvm_ld(g.a, (size_t)(k0 + kk) * g.a.ld + mb + mm) : kvm_ld(g.a, (size_t)(mb + mm) * g.a.ld + k0 + kk);
            if (g.round_ops) v = kvm_bf16_round(v);
          }
          As[kk][mm] = v;
          int kb, nn;
          if (tb) { nn = e >> 5; kb = e & 31; } else { kb = e >> 6; nn = e & 63; }
          float w = 0.0f;
          if (k0 + kb < g.K && nb + nn < n_end) {
            w = tb ? kvm_ld(g.b, (size_t)(nb + nn) * g.b.ld + k0 + kb) : kvm_ld(g.b, (size_t)(k0 + kb) * g.b.ld + nb + nn);
            if (g.round_ops) w = kvm_bf16_round(w);
          }
          Bs[kb][nn] = w;
        }
        kvm_sync();
        const int kmax = min(32, g.K - k0);
        for (int kk = 0; kk < kmax; ++kk) {
          const float x = As[kk][row];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(x, Bs[kk][cg + j]));
        }
      }
      const int m = mb + row;
      if (m < m_end)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int n = nb + cg + j;
          if (n < n_end) kvm_st(g.out, (size_t)m * g.out.ld + n, kvm_mm_epilogue(g, acc[j], m, n));
        }
    }
}

KVM_OP_FN void kvm_op_matmul_tile(const KvmCtx& c, const int32_t* a) {
  KvmMmArgs g;
  if (kvm_mm_args(c, a, 0, g)) kvm_mm_simt(c, g);
}
KVM_OP_FN void kvm_op_matmul_tile_bf16(const KvmCtx& c, const int32_t* a) {
  KvmMmArgs g;
  if (kvm_mm_args(c, a, 1, g)) kvm_mm_simt(c, g);
}
// out[m,n] = a[m,k] @ b[k,n] from element 0, contiguous (include/mvm_ops.def:14; runtime/ref_ops.py:55-64).
KVM_OP_FN void kvm_op_matmul(const KvmCtx& c, const int32_t* a) {
  KvmMmArgs g{};
  if (!kvm_buf(c, a[0], KVM_M_F32, g.a) || !kvm_buf(c, a[1], KVM_M_F32, g.b) || !kvm_buf(c, a[2], KVM_M_F32, g.out)) return;
  const int m = a[3], n = a[4], k = a[5];
  if (m < 1 || n < 1 || k < 1 || !kvm_flat_ok(c, g.a, (long long)m * k) || !kvm_flat_ok(c, g.b, (long long)k * n) || !kvm_flat_ok(c, g.out, (long long)m * n)) {
    c.fail(KVM_OPE_RANGE, m, n); return; }
  g.a.ld = k; g.b.ld = n; g.out.ld = n;
  g.M = m; g.N = n; g.K = k; g.m0 = 0; g.n0 = 0; g.tm = m; g.tn = n; g.alpha = 1.0f; g.flags = 0; g.round_ops = false;
  kvm_mm_simt(c, g);
}
