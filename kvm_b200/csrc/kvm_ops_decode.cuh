// Decode (serving) ops: KV-cache append, one-row attention over the cache (whole and split-context flash-decoding with
// optional fused RoPE + append), the bf16 weight-streaming GEMV with RMSNorm / SwiGLU prologue, and token sampling.
// Reference semantics: runtime/ref_gpt.py:367-410,485-545, runtime/ref_extra.py:398-498; layouts from
// include/mvm_ops_gpt.def:19-20 (cache [B*Hkv*Tmax, hd], row (b*Hkv+kvh)*Tmax+t) and include/mvm_ops_extra.def:79-95.
#pragma once
#include "kvm_dev.cuh"
#include "kvm_ops_flat.cuh"
#include "kvm_ops_rows.cuh"
#include "kvm_decode_stream.cuh"

#define KVM_ATTN_EMPTY_M (-3.4028234663852886e38f)

KVM_OP_FN void kvm_op_kv_append(const KvmCtx& c, const int32_t* a) {
  KvmBuf kn, vn, kc, vc, lens;
  if (!kvm_buf(c, a[0], KVM_M_FLT, kn) || !kvm_buf(c, a[1], KVM_M_FLT, vn) || !kvm_buf(c, a[2], KVM_M_FLT, kc) || !kvm_buf(c, a[3], KVM_M_FLT, vc) ||
      !kvm_buf(c, a[4], KVM_M_I32, lens)) return;
  const int b0 = a[5], b1 = a[6], nn = a[7], Hkv = a[8], hd = a[9], Tmax = a[10];
  if (b0 < 0 || b1 < b0 || nn <= 0 || Hkv <= 0 || hd <= 0 || Tmax <= 0 || !kvm_mat_ok(c, kn, (long long)b1 * nn, Hkv * hd) || !kvm_mat_ok(c, vn, (long long)b1 * nn, Hkv * hd) ||
      !kvm_mat_ok(c, kc, (long long)b1 * Hkv * Tmax, hd) || !kvm_mat_ok(c, vc, (long long)b1 * Hkv * Tmax, hd) || !kvm_flat_ok(c, lens, b1)) { c.fail(KVM_OPE_RANGE, b0, b1); return; }
  for (int bb = b0; bb < b1; ++bb) { const int L = ((const int*)lens.p)[bb]; if (L < 0 || L + nn > Tmax) { c.fail(KVM_OPE_KVLEN, bb, L); return; } }
  const long long per = (long long)nn * Hkv * hd;
  for (long long e = threadIdx.x; e < (long long)(b1 - b0) * per; e += KVM_NT) {
    const int bb = b0 + (int)(e / per), t = (int)((e % per) / (Hkv * hd)), h = (int)((e % (Hkv * hd)) / hd), cc = (int)(e % hd);
    const size_t row = (size_t)(bb * Hkv + h) * Tmax + ((const int*)lens.p)[bb] + t;
    kvm_st(kc, row * kc.ld + cc, kvm_ld(kn, (size_t)(bb * nn + t) * kn.ld + h * hd + cc));
    kvm_st(vc, row * vc.ld + cc, kvm_ld(vn, (size_t)(bb * nn + t) * vn.ld + h * hd + cc));
  }
}

// Partial attention of one GQA group (G <= 8 query heads sharing one kv head) over cache rows [j0,j1) of `base`.
// Warps take keys j0+warp, j0+warp+16, ...; lanes hold hd/32 (<= 4) columns.  Results (m, l, acc[hd]) per head are merged over
// the 16 warps in warp order through shared memory, then handed to `emit(g, m, l, acc_of_column)` per head.
//   qs: G*hd floats in shared memory (the query rows, already rotated)       ws: scratch of 16*G*(hd+2) floats
template <class Emit>
static __device__ void kvm_decode_group(const KvmBuf& kc, const KvmBuf& vc, size_t base, int j0, int j1, int G, int hd, float sc, const float* qs, float* ws, Emit emit) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nc = (hd + 31) / 32;
  float m[8], l[8], acc[8][4];
#pragma unroll
  for (int g = 0; g < 8; ++g) { m[g] = KVM_ATTN_EMPTY_M; l[g] = 0.0f;
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[g][t] = 0.0f; }
  for (int j = j0 + warp; j < j1; j += KVM_NWARPS) {
    float kr[4], vr[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int cc = lane + 32 * t;
      kr[t] = (t < nc && cc < hd) ? kvm_ld(kc, (base + j) * kc.ld + cc) : 0.0f;
      vr[t] = (t < nc && cc < hd) ? kvm_ld(vc, (base + j) * vc.ld + cc) : 0.0f;
    }
#pragma unroll
    for (int g = 0; g < 8; ++g) if (g < G) {
      float s = 0.0f;
#pragma unroll
      for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) s += qs[g * hd + lane + 32 * t] * kr[t];
      s = kvm_warp_sum(s) * sc;
      const float mn = fmaxf(m[g], s), corr = __expf(m[g] - mn), p = __expf(s - mn);
      l[g] = l[g] * corr + p;
#pragma unroll
      for (int t = 0; t < 4; ++t) acc[g][t] = acc[g][t] * corr + p * vr[t];
      m[g] = mn;
    }
  }
  const int stride = hd + 2;
  kvm_sync();
#pragma unroll
  for (int g = 0; g < 8; ++g) if (g < G) {
    float* w = ws + (size_t)(warp * G + g) * stride;
#pragma unroll
    for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) w[lane + 32 * t] = acc[g][t];
    if (lane == 0) { w[hd] = m[g]; w[hd + 1] = l[g]; }
  }
  kvm_sync();
  // merge over warps: thread (g, column)
  for (int e = threadIdx.x; e < G * hd; e += KVM_NT) {
    const int g = e / hd, cc = e % hd;
    float M = KVM_ATTN_EMPTY_M;
    for (int w = 0; w < KVM_NWARPS; ++w) if (ws[(size_t)(w * G + g) * stride + hd + 1] > 0.0f) M = fmaxf(M, ws[(size_t)(w * G + g) * stride + hd]);
    float L = 0.0f, A = 0.0f;
    for (int w = 0; w < KVM_NWARPS; ++w) {
      const float* r = ws + (size_t)(w * G + g) * stride;
      if (r[hd + 1] > 0.0f) { const float e2 = __expf(r[hd] - M); L += e2 * r[hd + 1]; A += e2 * r[cc]; }
    }
    emit(g, cc, M, L, A);
  }
}

// Vector form of the same partial attention for power-of-two head sizes (8..128) and 16-byte aligned cache rows: a key is
// handled by hd/8 lanes (each holds 8 contiguous columns of K and V, one 16-byte load each for bf16), so a warp covers 32/(hd/8)
// keys per step; two steps of loads are in flight before the first is consumed.  Every lane group keeps its own online-softmax
// state per head; groups are merged by shuffles, warps through shared memory as in kvm_decode_group, same emit contract.
template <int GT, class Emit>
static __device__ void kvm_decode_group_vec_t(const KvmBuf& kc, const KvmBuf& vc, size_t base, int j0, int j1, int G, int hd, float sc, const float* qs, float* ws, Emit emit) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int LPK = hd >> 3, KPI = 32 / LPK, slot = lane / LPK, c0 = (lane % LPK) * 8;
  float m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int g = 0; g < GT; ++g) { m[g] = KVM_ATTN_EMPTY_M; l[g] = 0.0f;
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[g][t] = 0.0f; }
  // contiguous key range per warp
  const int n = j1 - j0, per = (n + KVM_NWARPS - 1) / KVM_NWARPS, w0 = j0 + warp * per, w1 = min(j1, w0 + per);
  for (int jb = w0; jb < w1; jb += 2 * KPI) {
    float kr[2][8], vr[2][8];
    int jj[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      jj[u] = jb + u * KPI + slot;
      if (jj[u] < w1) { kvm_ld8(kc, (base + jj[u]) * kc.ld + c0, kr[u]); kvm_ld8(vc, (base + jj[u]) * vc.ld + c0, vr[u]); }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool live = jj[u] < w1;
#pragma unroll
      for (int g = 0; g < GT; ++g) if (g < G) {
        float s = 0.0f;
        if (live) {
          const float4 qa = *(const float4*)(qs + g * hd + c0), qb = *(const float4*)(qs + g * hd + c0 + 4);     // query columns of this lane (shared memory)
          s = qa.x * kr[u][0] + qa.y * kr[u][1] + qa.z * kr[u][2] + qa.w * kr[u][3] + qb.x * kr[u][4] + qb.y * kr[u][5] + qb.z * kr[u][6] + qb.w * kr[u][7];
        }
        for (int o = LPK >> 1; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (live) {
          s *= sc;
          const float mn = fmaxf(m[g], s), corr = __expf(m[g] - mn), p = __expf(s - mn);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int t = 0; t < 8; ++t) acc[g][t] = acc[g][t] * corr + p * vr[u][t];
          m[g] = mn;
        }
      }
    }
  }
  // merge the key slots of the warp (lanes with equal column range)
#pragma unroll
  for (int g = 0; g < GT; ++g) if (g < G) {
    for (int o = LPK; o < 32; o <<= 1) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o), lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo), ca = __expf(m[g] - mn), cb = __expf(mo - mn);
      l[g] = l[g] * ca + lo * cb;
#pragma unroll
      for (int t = 0; t < 8; ++t) acc[g][t] = acc[g][t] * ca + __shfl_xor_sync(0xffffffffu, acc[g][t], o) * cb;
      m[g] = mn;
    }
  }
  const int stride = hd + 2;
  kvm_sync();
#pragma unroll
  for (int g = 0; g < GT; ++g) if (g < G && slot == 0) {
    float* w = ws + (size_t)(warp * G + g) * stride;
#pragma unroll
    for (int t = 0; t < 8; ++t) w[c0 + t] = acc[g][t];
    if (lane == 0) { w[hd] = m[g]; w[hd + 1] = l[g]; }
  }
  kvm_sync();
  for (int e = threadIdx.x; e < G * hd; e += KVM_NT) {
    const int g = e / hd, cc = e % hd;
    float M = KVM_ATTN_EMPTY_M;
    for (int w = 0; w < KVM_NWARPS; ++w) if (ws[(size_t)(w * G + g) * stride + hd + 1] > 0.0f) M = fmaxf(M, ws[(size_t)(w * G + g) * stride + hd]);
    float L = 0.0f, A = 0.0f;
    for (int w = 0; w < KVM_NWARPS; ++w) {
      const float* r = ws + (size_t)(w * G + g) * stride;
      if (r[hd + 1] > 0.0f) { const float e2 = __expf(r[hd] - M); L += e2 * r[hd + 1]; A += e2 * r[cc]; }
    }
    emit(g, cc, M, L, A);
  }
}
template <class Emit>
static __device__ void kvm_decode_group_vec(const KvmBuf& kc, const KvmBuf& vc, size_t base, int j0, int j1, int G, int hd, float sc, const float* qs, float* ws, Emit emit) {
  if (G <= 1) kvm_decode_group_vec_t<1>(kc, vc, base, j0, j1, G, hd, sc, qs, ws, emit);
  else if (G <= 2) kvm_decode_group_vec_t<2>(kc, vc, base, j0, j1, G, hd, sc, qs, ws, emit);
  else if (G <= 4) kvm_decode_group_vec_t<4>(kc, vc, base, j0, j1, G, hd, sc, qs, ws, emit);
  else kvm_decode_group_vec_t<8>(kc, vc, base, j0, j1, G, hd, sc, qs, ws, emit);
}
__device__ __forceinline__ bool kvm_decode_vec_ok(const KvmBuf& kc, const KvmBuf& vc, int hd) {
  return hd >= 8 && hd <= 128 && (hd & (hd - 1)) == 0 && (kc.ld & 7) == 0 && (vc.ld & 7) == 0 && kvm_vec_ok(kc) && kvm_vec_ok(vc);
}

KVM_OP_FN void kvm_op_attn_decode(const KvmCtx& c, const int32_t* a) {
  KvmBuf q, kc, vc, lens, o;
  if (!kvm_buf(c, a[0], KVM_M_FLT, q) || !kvm_buf(c, a[1], KVM_M_FLT, kc) || !kvm_buf(c, a[2], KVM_M_FLT, vc) || !kvm_buf(c, a[3], KVM_M_I32, lens) ||
      !kvm_buf(c, a[4], KVM_M_FLT, o)) return;
  const int b = a[5], h = a[6], H = a[7], Hkv = a[8], hd = a[9], Tmax = a[10];
  const float sc = kvm_bits_f32(a[11]);
  if (b < 0 || h < 0 || h >= H || Hkv <= 0 || H % Hkv || hd <= 0 || hd > 128 || Tmax <= 0) { c.fail(KVM_OPE_SHAPE, h, hd); return; }
  if (!kvm_mat_ok(c, q, b + 1, H * hd) || !kvm_mat_ok(c, o, b + 1, H * hd) || !kvm_mat_ok(c, kc, (long long)(b + 1) * Hkv * Tmax, hd) ||
      !kvm_mat_ok(c, vc, (long long)(b + 1) * Hkv * Tmax, hd) || !kvm_flat_ok(c, lens, b + 1)) return;
  const int L = ((const int*)lens.p)[b], n = L + 1;
  if (L < 0 || n > Tmax) { c.fail(KVM_OPE_KVLEN, b, L); return; }
  float* qs = (float*)c.smem;
  float* ws = qs + 128;
  kvm_sync();
  for (int cc = threadIdx.x; cc < hd; cc += KVM_NT) qs[cc] = kvm_ld(q, (size_t)b * q.ld + h * hd + cc);
  kvm_sync();
  const size_t base = (size_t)(b * Hkv + h / (H / Hkv)) * Tmax;
  auto emit = [&](int, int cc, float, float Lsum, float A) { kvm_st(o, (size_t)b * o.ld + h * hd + cc, A / Lsum); };
  if (kvm_decode_vec_ok(kc, vc, hd)) kvm_decode_group_vec(kc, vc, base, 0, n, 1, hd, sc, qs, ws, emit);
  else kvm_decode_group(kc, vc, base, 0, n, 1, hd, sc, qs, ws, emit);
}

// What a split-attention task does before it looks at the cache: inverse frequencies, the appended key (optionally RMS-normalised,
// rotated, stored to the cache and kept as floats for the staged tile) and value, the rotated (optionally normalised) queries
// of the group.  Shared by the ready-queue form below and the ring form of the static path.  Whole compute group.
struct KvmPartPro {
  KvmBuf q, kc, vc, kn, vn, gam;      // gam.p == nullptr: no QK norm
  int b, kvh, G, hd, fl, p0;
  size_t base;
  float theta, eps;
  bool appends;
  float *qs, *inv, *kns, *vns, *rsq;  // shared memory: G*hd queries, hd/2 frequencies, hd + hd appended row, G + 1 reciprocal RMS values
  float* rope_cache;                  // KvmCtx::rope_cache
};
static __device__ void kvm_part_prologue(const KvmPartPro& P) {
  const int hd = P.hd, half = hd / 2, G = P.G, b = P.b, kvh = P.kvh, n = P.p0 + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (P.gam.p) {
    // reciprocal RMS per query head (warps 0..G-1) and of the appended key (warp G): float32 sums in a fixed lane / shuffle order
    if (warp <= G) {
      const bool key = warp == G;
      float ss = 0.0f;
      if (!key || P.kn.p)
        for (int i = lane; i < hd; i += 32) {
          const float t = key ? kvm_ld(P.kn, (size_t)b * P.kn.ld + kvh * hd + i) : kvm_ld(P.q, (size_t)b * P.q.ld + (kvh * G + warp) * hd + i);
          ss += t * t;
        }
      ss = kvm_warp_sum(ss);
      if (lane == 0) P.rsq[warp] = 1.0f / sqrtf(ss / hd + P.eps);
    }
    kvm_sync();
  }
  const float* gq = P.gam.p ? (const float*)P.gam.p : nullptr;
  const float* gk = P.gam.p ? (const float*)P.gam.p + P.gam.ld : nullptr;
  const float* inv = P.inv;
  if (P.fl & 1) {
    // theta^(-2i/hd) is a double-precision pow per frequency: computed once per (theta, head dimension) and launch, not per task
    float* rc = P.rope_cache;
    const bool hit = rc && __float_as_int(rc[0]) == __float_as_int(P.theta) && __float_as_int(rc[1]) == hd;
    if (rc) kvm_sync();                                      // every thread has looked at the key before anyone replaces it
    if (!hit) {
      float* dst = rc ? rc + 2 : P.inv;
      for (int i = threadIdx.x; i < half; i += KVM_NT) dst[i] = kvm_rope_inv(P.theta, i, hd);
      if (rc && threadIdx.x == 0) { rc[0] = P.theta; rc[1] = __int_as_float(hd); }
      kvm_sync();
    }
    if (rc) inv = rc + 2;
  }
  if (P.appends) {
    for (int i = threadIdx.x; i < half; i += KVM_NT) {
      float sn, co; sincosf(__fmul_rn((float)P.p0, inv[i]), &sn, &co);
      float x1 = kvm_ld(P.kn, (size_t)b * P.kn.ld + kvh * hd + i), x2 = kvm_ld(P.kn, (size_t)b * P.kn.ld + kvh * hd + i + half);
      if (gk) { x1 = x1 * P.rsq[G] * gk[i]; x2 = x2 * P.rsq[G] * gk[i + half]; }
      const float y1 = x1 * co - x2 * sn, y2 = x1 * sn + x2 * co;
      P.kns[i] = y1; P.kns[i + half] = y2;
      kvm_st(P.kc, (P.base + n - 1) * P.kc.ld + i, y1);
      kvm_st(P.kc, (P.base + n - 1) * P.kc.ld + i + half, y2);
    }
    for (int cc = threadIdx.x; cc < hd; cc += KVM_NT) {
      const float t = kvm_ld(P.vn, (size_t)b * P.vn.ld + kvh * hd + cc);
      P.vns[cc] = t;
      kvm_st(P.vc, (P.base + n - 1) * P.vc.ld + cc, t);
    }
  }
  for (int e = threadIdx.x; e < G * half; e += KVM_NT) {
    const int g = e / half, i = e % half, h = kvh * G + g;
    float x1 = kvm_ld(P.q, (size_t)b * P.q.ld + h * hd + i), x2 = kvm_ld(P.q, (size_t)b * P.q.ld + h * hd + i + half);
    if (gq) { x1 = x1 * P.rsq[g] * gq[i]; x2 = x2 * P.rsq[g] * gq[i + half]; }
    if (P.fl & 1) {
      float sn, co; sincosf(__fmul_rn((float)P.p0, inv[i]), &sn, &co);
      const float y1 = x1 * co - x2 * sn, y2 = x1 * sn + x2 * co;
      x1 = y1; x2 = y2;
      if (P.fl & 2) { x1 = kvm_bf16_round(x1); x2 = kvm_bf16_round(x2); }
    }
    P.qs[g * hd + i] = x1; P.qs[g * hd + i + half] = x2;
  }
}

// attn_decode_part (135) and, with qkn, its QK-norm extension attn_decode_part_qkn (300: two more arguments, qk_gamma and eps).
static __device__ void kvm_attn_decode_part_op(const KvmCtx& c, const int32_t* a, bool qkn) {
  KvmBuf q, kc, vc, lens, part, kn, vn, gam{};
  if (!kvm_buf(c, a[0], KVM_M_FLT, q) || !kvm_buf(c, a[1], KVM_M_FLT, kc) || !kvm_buf(c, a[2], KVM_M_FLT, vc) || !kvm_buf(c, a[3], KVM_M_I32, lens) ||
      !kvm_buf(c, a[4], KVM_M_F32, part) || !kvm_buf(c, a[5], KVM_M_FLT, kn, true) || !kvm_buf(c, a[6], KVM_M_FLT, vn, true)) return;
  if (qkn && !kvm_buf(c, a[18], KVM_M_F32, gam)) return;
  const int b = a[7], kvh = a[8], s = a[9], S = a[10], H = a[11], Hkv = a[12], hd = a[13], Tmax = a[14], fl = a[17];
  const float sc = kvm_bits_f32(a[15]), theta = kvm_bits_f32(a[16]);
  if (b < 0 || Hkv <= 0 || H % Hkv || kvh < 0 || kvh >= Hkv || s < 0 || s >= S || Tmax <= 0 || hd <= 0 || hd > 128 || (hd & 7) || H / Hkv > 8 ||
      !(fl == 0 || fl == 1 || fl == 3) || ((fl & 1) && (!kn.p || !vn.p))) { c.fail(KVM_OPE_SHAPE, hd, fl); return; }
  const int G = H / Hkv;
  if (!kvm_mat_ok(c, q, b + 1, H * hd) || !kvm_mat_ok(c, kc, (long long)(b + 1) * Hkv * Tmax, hd) || !kvm_mat_ok(c, vc, (long long)(b + 1) * Hkv * Tmax, hd) ||
      !kvm_flat_ok(c, lens, b + 1) || !kvm_mat_ok(c, part, (long long)(b + 1) * S * H, hd + 2) || !kvm_mat_ok(c, kn, b + 1, Hkv * hd) || !kvm_mat_ok(c, vn, b + 1, Hkv * hd) ||
      !kvm_mat_ok(c, gam, 2, hd)) return;
  const int p0 = ((const int*)lens.p)[b], n = p0 + 1;
  if (p0 < 0 || n > Tmax) { c.fail(KVM_OPE_KVLEN, b, p0); return; }
  const int chunk = (n + S - 1) / S, j0 = s * chunk, j1 = min(n, s * chunk + chunk);
  const size_t base = (size_t)(b * Hkv + kvh) * Tmax;
  KvmPartPro P;
  P.q = q; P.kc = kc; P.vc = vc; P.kn = kn; P.vn = vn; P.gam = gam;
  P.b = b; P.kvh = kvh; P.G = G; P.hd = hd; P.fl = fl; P.p0 = p0; P.base = base; P.theta = theta; P.eps = qkn ? kvm_bits_f32(a[19]) : 0.0f;
  P.rope_cache = c.rope_cache;
  P.appends = (fl & 1) && j0 <= n - 1 && n - 1 < j1;    // this split holds the newest key: it appends (rotated key), rounded to the cache dtype
  P.qs = (float*)(c.smem + KVM_AS_OFF_QS);                       // G*hd rotated queries
  P.inv = (float*)(c.smem + KVM_AS_OFF_INV);                     // hd/2 inverse frequencies
  P.kns = (float*)(c.smem + KVM_AS_OFF_KNEW);                    // the appended key (rotated) and value, float
  P.vns = (float*)(c.smem + KVM_AS_OFF_VNEW);
  P.rsq = (float*)(c.smem + KVM_AS_OFF_ML);                      // free until the softmax writes its (m, l) there
  float* ws = (float*)(c.smem + KVM_AS_OFF_SC);
  auto prologue = [&]() { kvm_part_prologue(P); };
  float* pp = (float*)part.p;
  auto emit = [&](int g, int cc, float M, float Lsum, float A) {
    const size_t row = ((size_t)(b * S + s) * H + kvh * G + g) * part.ld;
    pp[row + cc] = Lsum > 0.0f ? A : 0.0f;
    if (cc == 0) { pp[row + hd] = Lsum > 0.0f ? M : KVM_ATTN_EMPTY_M; pp[row + hd + 1] = Lsum; }
  };
  if (kvm_attn_part_stream(c, kc, vc, base, j0, j1, P.appends ? n - 1 - j0 : -1, G, hd, sc, prologue, emit)) return;
  kvm_sync();
  prologue();
  __threadfence_block();
  kvm_sync();
  if (kvm_decode_vec_ok(kc, vc, hd)) kvm_decode_group_vec(kc, vc, base, j0, j1, G, hd, sc, P.qs, ws, emit);
  else kvm_decode_group(kc, vc, base, j0, j1, G, hd, sc, P.qs, ws, emit);
}
KVM_OP_FN void kvm_op_attn_decode_part(const KvmCtx& c, const int32_t* a) { kvm_attn_decode_part_op(c, a, false); }
KVM_OP_FN void kvm_op_attn_decode_part_qkn(const KvmCtx& c, const int32_t* a) { kvm_attn_decode_part_op(c, a, true); }

KVM_OP_FN void kvm_op_attn_decode_merge(const KvmCtx& c, const int32_t* a) {
  KvmBuf part, o;
  if (!kvm_buf(c, a[0], KVM_M_F32, part) || !kvm_buf(c, a[1], KVM_M_FLT, o)) return;
  const int b = a[2], h0 = a[3], h1 = a[4], S = a[5], H = a[6], hd = a[7];
  if (b < 0 || h0 < 0 || h1 <= h0 || h1 > H || S <= 0 || hd <= 0 || !kvm_mat_ok(c, part, (long long)(b + 1) * S * H, hd + 2) || !kvm_mat_ok(c, o, b + 1, H * hd)) {
    c.fail(KVM_OPE_RANGE, h0, h1); return; }
  const float* pp = (const float*)part.p;
  for (int e = threadIdx.x; e < (h1 - h0) * hd; e += KVM_NT) {
    const int h = h0 + e / hd, cc = e % hd;
    float M = KVM_ATTN_EMPTY_M, L = 0.0f, A = 0.0f;
    for (int s0 = 0; s0 < S; s0 += 12) {       // twelve splits at a time: their loads are independent and issued together
      float ms[12], ls[12], as[12];
#pragma unroll
      for (int u = 0; u < 12; ++u) {
        const int s = s0 + u;
        const float* r = pp + ((size_t)(b * S + (s < S ? s : 0)) * H + h) * part.ld;
        ms[u] = r[hd]; ls[u] = s < S ? r[hd + 1] : 0.0f; as[u] = r[cc];
      }
#pragma unroll
      for (int u = 0; u < 12; ++u) if (ls[u] > 0.0f) {      // split order, as the reference merges
        const float mn = fmaxf(M, ms[u]), ca = __expf(M - mn), cb = __expf(ms[u] - mn);
        L = L * ca + ls[u] * cb; A = A * ca + as[u] * cb; M = mn;
      }
    }
    kvm_st(o, (size_t)b * o.ld + h * hd + cc, A / L);
  }
}

// out[0,n] = sum_k v[k] w[n,k] (+ res[0,n]), v = bf16(prologue(x)); w bf16 [>=n1, K], rows contiguous in K.
// The activation row is staged once per task in shared memory (as float); each warp then streams four weight rows at a
// time with 16-byte loads, two k-steps in flight, float32 accumulation in a fixed order, warp-shuffle reduction.
// One activation row: x / x2 / out / res are one-row views (row 0 of what they point to).
static __device__ void kvm_gemv_row(const KvmCtx& c, const KvmBuf& x, const KvmBuf& x2, const KvmBuf& gm, const KvmBuf& w, const KvmBuf& out, const KvmBuf& res, int n0, int n1, int K,
                                    int pro, float eps) {
  if (kvm_gemv_stream(c, x, x2, gm, w, out, res, n0, n1, K, pro, eps)) return;      // bulk-copy ring; the form below serves what does not fit
  float* vs = (float*)c.smem;
  float* red = vs + K;
  float rs = 1.0f;
  if (pro == 1) {
    float q = 0.0f;
    for (int k = threadIdx.x; k < K; k += KVM_NT) { const float t = kvm_ld(x, k); q += t * t; }
    q = kvm_block_sum(q, red);
    rs = 1.0f / sqrtf(q / K + eps);
  }
  kvm_sync();
  for (int k = threadIdx.x; k < K; k += KVM_NT) {
    const float t = kvm_ld(x, k);
    vs[k] = kvm_bf16_round(pro == 1 ? t * rs * ((const float*)gm.p)[k] : pro == 2 ? kvm_silu(t) * kvm_ld(x2, k) : t);
  }
  kvm_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w.p;
  // Work units = (group of 4 rows) x (slice of K): few rows are split along K so that all 16 warps stream weights;
  // the slices of a row are then added in slice order (fixed order, deterministic).
  const int rows = n1 - n0, RG = (rows + 3) / 4;
  int KS = 1;
  while (KS < 16 && RG * KS < 2 * KVM_NWARPS && (K / (KS * 2)) >= 512) KS *= 2;
  const int kslice = ((K / KS + 255) / 256) * 256;
  float* parts = red + 64;                       // [RG][KS][4]
  if ((K + 64 + RG * KS * 4) * 4 + 256 > c.smem_bytes) { c.fail(KVM_OPE_SMEM, K, rows); return; }
  for (int u = warp; u < RG * KS; u += KVM_NWARPS) {
    const int rg = u / KS, ks = u % KS, nb = n0 + rg * 4, nr = min(4, n1 - nb);
    const int kend = min(K, (ks + 1) * kslice);
    float acc[4] = {0, 0, 0, 0};
    for (int k = ks * kslice + lane * 8; k < kend; k += 512) {
      uint4 wv[4][2];
      const bool two = k + 256 < kend;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const __nv_bfloat16* row = wp + (size_t)(nb + (r < nr ? r : 0)) * w.ld;
        wv[r][0] = __ldcs((const uint4*)(row + k));
        wv[r][1] = two ? __ldcs((const uint4*)(row + k + 256)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int hstep = 0; hstep < 2; ++hstep) {
        if (hstep == 1 && !two) break;
        const float4 va = *(const float4*)(vs + k + hstep * 256), vb = *(const float4*)(vs + k + hstep * 256 + 4);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const __nv_bfloat162* hh = (const __nv_bfloat162*)&wv[r][hstep];
          const float2 f0 = __bfloat1622float2(hh[0]), f1 = __bfloat1622float2(hh[1]), f2 = __bfloat1622float2(hh[2]), f3 = __bfloat1622float2(hh[3]);
          acc[r] = fmaf(va.x, f0.x, acc[r]); acc[r] = fmaf(va.y, f0.y, acc[r]); acc[r] = fmaf(va.z, f1.x, acc[r]); acc[r] = fmaf(va.w, f1.y, acc[r]);
          acc[r] = fmaf(vb.x, f2.x, acc[r]); acc[r] = fmaf(vb.y, f2.y, acc[r]); acc[r] = fmaf(vb.z, f3.x, acc[r]); acc[r] = fmaf(vb.w, f3.y, acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float sum = kvm_warp_sum(acc[r]);
      if (lane == 0) parts[(rg * KS + ks) * 4 + r] = sum;
    }
  }
  kvm_sync();
  for (int i = threadIdx.x; i < rows; i += KVM_NT) {
    float sum = 0.0f;
    for (int ks = 0; ks < KS; ++ks) sum += parts[((i >> 2) * KS + ks) * 4 + (i & 3)];
    const int n = n0 + i;
    kvm_st(out, n, res.p ? __fadd_rn(sum, kvm_ld(res, n)) : sum);
  }
}

__device__ __forceinline__ KvmBuf kvm_row_view(const KvmBuf& b, int r) {
  KvmBuf v = b;
  if (b.p) { v.p = (char*)b.p + (size_t)r * b.ld * (b.dtype == KVM_BF16 ? 2 : 4); v.rows = 1; }
  return v;
}
// gemv_bf16 (134): row 0.  gemv_bf16_rows (301, an extension): rows r0..r1 of x / x2 / out / res, one after the other here (the
// static path's ring form reads the weights once for all rows; this form serves the ready queue and shapes the ring cannot take).
static __device__ void kvm_gemv_op(const KvmCtx& c, const int32_t* a, int r0, int r1) {
  KvmBuf x, x2, gm, w, out, res;
  if (!kvm_buf(c, a[0], KVM_M_FLT, x) || !kvm_buf(c, a[1], KVM_M_FLT, x2, true) || !kvm_buf(c, a[2], KVM_M_F32, gm, true) || !kvm_buf(c, a[3], KVM_M_BF16, w) ||
      !kvm_buf(c, a[4], KVM_M_FLT, out) || !kvm_buf(c, a[5], KVM_M_FLT, res, true)) return;
  const int n0 = a[6], n1 = a[7], K = a[8], pro = a[9];
  const float eps = kvm_bits_f32(a[10]);
  if (n0 < 0 || n1 <= n0 || K <= 0 || (K & 7) || pro < 0 || pro > 2 || (pro == 1 && !gm.p) || (pro == 2 && !x2.p) || (w.ld & 7) || !kvm_vec_ok(w) ||
      K * 4 + 256 > c.smem_bytes || r0 < 0 || r1 <= r0) { c.fail(KVM_OPE_SHAPE, K, pro); return; }
  if (!kvm_mat_ok(c, w, n1, K) || !kvm_mat_ok(c, x, r1, K) || !kvm_mat_ok(c, x2, r1, K) || !kvm_flat_ok(c, gm, K) || !kvm_mat_ok(c, out, r1, n1) || !kvm_mat_ok(c, res, r1, n1)) return;
  for (int r = r0; r < r1; ++r) {
    if (r > r0) kvm_sync();
    kvm_gemv_row(c, kvm_row_view(x, r), kvm_row_view(x2, r), gm, w, kvm_row_view(out, r), kvm_row_view(res, r), n0, n1, K, pro, eps);
  }
}
KVM_OP_FN void kvm_op_gemv_bf16(const KvmCtx& c, const int32_t* a) { kvm_gemv_op(c, a, 0, 1); }
KVM_OP_FN void kvm_op_gemv_bf16_rows(const KvmCtx& c, const int32_t* a) { kvm_gemv_op(c, a, a[11], a[12]); }

// ---- sampling: Philox-4x32-10 counter (row, ctr, 0, 0), key (seed, 0x9E3779B9) (runtime/ref_gpt.py:488-506) --------------------------
__device__ __forceinline__ float kvm_philox_uniform(unsigned seed, unsigned ctr, unsigned row) {
  unsigned c0 = row, c1 = ctr, c2 = 0, c3 = 0, k0 = seed, k1 = 0x9E3779B9u;
  for (int i = 0; i < 10; ++i) {
    const unsigned long long p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
    const unsigned n0 = (unsigned)(p1 >> 32) ^ c1 ^ k0, n1 = (unsigned)p1, n2 = (unsigned)(p0 >> 32) ^ c3 ^ k1, n3 = (unsigned)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ unsigned kvm_order_key(float x) { const unsigned b = __float_as_uint(x); return (b >> 31) ? ~b : (b ^ 0x80000000u); }

// temp <= 0: argmax. Otherwise inverse-CDF over softmax(logits/temp) restricted to the topk largest (ties kept), weights and
// running sum in double in index order by one thread (the reference's order; rows are short-lived serving rows).
KVM_OP_FN void kvm_op_sample(const KvmCtx& c, const int32_t* a) {
  KvmBuf lg, out, ctr;
  if (!kvm_buf(c, a[0], KVM_M_FLT, lg) || !kvm_buf(c, a[1], KVM_M_I32, out) || !kvm_buf(c, a[2], KVM_M_I32, ctr, true)) return;
  const int r0 = a[3], r1 = a[4], V = a[5], topk = a[7];
  const float temp = kvm_bits_f32(a[6]);
  if (r0 < 0 || r1 < r0 || V <= 0 || !kvm_mat_ok(c, lg, r1, V) || !kvm_flat_ok(c, out, r1)) { c.fail(KVM_OPE_RANGE, r0, r1); return; }
  if (temp <= 0.0f) { kvm_argmax_rows(c, lg, out, r0, r1, V); return; }
  const unsigned cv = ctr.p ? (unsigned)((const int*)ctr.p)[0] : 0u;
  unsigned* sh = (unsigned*)c.smem;
  for (int r = r0; r < r1; ++r) {
    // threshold key = topk-th largest order key, by bitwise binary search on the count of keys >= candidate (block-parallel counts)
    unsigned thr = 0;
    if (topk > 0 && topk < V) {
      for (int bit = 31; bit >= 0; --bit) {
        const unsigned cand = thr | (1u << bit);
        int cnt = 0;
        for (int k = threadIdx.x; k < V; k += KVM_NT) cnt += kvm_order_key(kvm_ld(lg, (size_t)r * lg.ld + k)) >= cand;
        const float tot = kvm_block_sum((float)cnt, (float*)sh);
        if ((int)tot >= topk) thr = cand;
      }
    }
    float mx = -INFINITY;
    for (int k = threadIdx.x; k < V; k += KVM_NT) { const float v = kvm_ld(lg, (size_t)r * lg.ld + k); if (v == v) mx = fmaxf(mx, v); }
    mx = kvm_block_max(mx, (float*)sh);
    if (threadIdx.x == 0) {
      double total = 0.0;
      for (int k = 0; k < V; ++k) { const float v = kvm_ld(lg, (size_t)r * lg.ld + k); if (v == v && kvm_order_key(v) >= thr) total += exp((double)__fsub_rn(v, mx) / (double)temp); }
      const double target = (double)kvm_philox_uniform((unsigned)a[8], cv, (unsigned)r) * total;
      double run = 0.0; int pick = -1, last = -1;
      for (int k = 0; k < V; ++k) {
        const float v = kvm_ld(lg, (size_t)r * lg.ld + k);
        if (v == v && kvm_order_key(v) >= thr) { run += exp((double)__fsub_rn(v, mx) / (double)temp); last = k; if (run > target) { pick = k; break; } }
      }
      ((int*)out.p)[r] = pick >= 0 ? pick : (last > 0 ? last : 0);
    }
    kvm_sync();
  }
}
