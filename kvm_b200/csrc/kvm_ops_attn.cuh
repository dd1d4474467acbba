// Causal attention (training) forward / backward, SIMT form: one warp per query (or key) row, lanes across 32 keys for the
// score and across the head dimension for the value products, online softmax in float32.  Reference semantics:
// runtime/ref_gpt.py:279-364 (128 rows per task, natural-log lse at (b*H+h)*T+t, GQA kv head = h/(H/Hkv), dk/dv summed over
// the whole group in head-then-query order).  This form serves any hd in {16,32,64,128} and any storage dtype; the tcgen05
// form in kvm_attn_tc.cuh takes the bf16 hd=64 / hd=128 cases.
#pragma once
#include "kvm_dev.cuh"

#define KVM_ATTN_ROWS 128

// dot of a row held in shared memory (broadcast reads) with a row in global memory
__device__ __forceinline__ float kvm_dot_row(const float* __restrict__ s, const KvmBuf& b, size_t off, int hd, bool vec) {
  float acc = 0.0f;
  if (vec) for (int k = 0; k < hd; k += 8) { float v[8]; kvm_ld8(b, off + k, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += s[k + j] * v[j]; }
  else for (int k = 0; k < hd; ++k) acc += s[k] * kvm_ld(b, off + k);
  return acc;
}
__device__ __forceinline__ bool kvm_attn_vec(const KvmBuf& b, int hd) { return (hd & 7) == 0 && (b.ld & 7) == 0 && kvm_vec_ok(b); }

static __device__ bool kvm_attn_geom(const KvmCtx& c, int b, int h, int r0, int T, int H, int Hkv, int hd) {
  if (!(hd == 16 || hd == 32 || hd == 64 || hd == 128) || T <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || b < 0 || r0 < 0 || r0 >= T || h < 0) {
    c.fail(KVM_OPE_SHAPE, hd, r0); return false; }
  return true;
}

KVM_OP_FN void kvm_op_attn_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf q, k, v, o, lse;
  if (!kvm_buf(c, a[0], KVM_M_FLT, q) || !kvm_buf(c, a[1], KVM_M_FLT, k) || !kvm_buf(c, a[2], KVM_M_FLT, v) || !kvm_buf(c, a[3], KVM_M_FLT, o) ||
      !kvm_buf(c, a[4], KVM_M_F32, lse)) return;
  const int b = a[5], h = a[6], q0 = a[7], T = a[8], H = a[9], Hkv = a[10], hd = a[11];
  const float sc = kvm_bits_f32(a[12]);
  if (!kvm_attn_geom(c, b, h, q0, T, H, Hkv, hd) || h >= H) { c.fail(KVM_OPE_SHAPE, h, H); return; }
  const long long R = (long long)(b + 1) * T;
  if (!kvm_mat_ok(c, q, R, H * hd) || !kvm_mat_ok(c, k, R, Hkv * hd) || !kvm_mat_ok(c, v, R, Hkv * hd) || !kvm_mat_ok(c, o, R, H * hd) ||
      !kvm_flat_ok(c, lse, R * H)) return;
  const int kvh = h / (H / Hkv), lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q1 = min(q0 + KVM_ATTN_ROWS, T);
  float* qs = (float*)c.smem + warp * 128;
  const bool kvec = kvm_attn_vec(k, hd);
  const int nc = (hd + 31) / 32;
  for (int gq = q0 + warp; gq < q1; gq += KVM_NWARPS) {
    __syncwarp();
    for (int cc = lane; cc < hd; cc += 32) qs[cc] = kvm_ld(q, (size_t)(b * T + gq) * q.ld + h * hd + cc);
    __syncwarp();
    float m = -INFINITY, l = 0.0f, acc[4] = {0, 0, 0, 0};
    for (int j0 = 0; j0 <= gq; j0 += 32) {
      const int j = j0 + lane;
      float s = -INFINITY;
      if (j <= gq) s = kvm_dot_row(qs, k, (size_t)(b * T + j) * k.ld + kvh * hd, hd, kvec) * sc;
      const float mn = fmaxf(m, kvm_warp_max(s));
      const float corr = __expf(m - mn), p = j <= gq ? __expf(s - mn) : 0.0f;
      l = l * corr + kvm_warp_sum(p);
#pragma unroll
      for (int t = 0; t < 4; ++t) acc[t] *= corr;
      const int nk = min(32, gq + 1 - j0);
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const size_t vo = (size_t)(b * T + j0 + jj) * v.ld + kvh * hd;
#pragma unroll
        for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) acc[t] += pj * kvm_ld(v, vo + lane + 32 * t);
      }
      m = mn;
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) kvm_st(o, (size_t)(b * T + gq) * o.ld + h * hd + lane + 32 * t, acc[t] / l);
    if (lane == 0) ((float*)lse.p)[(size_t)(b * H + h) * T + gq] = m + logf(l);
  }
}

KVM_OP_FN void kvm_op_attn_bwd_delta(const KvmCtx& c, const int32_t* a) {
  KvmBuf o, dO, delta;
  if (!kvm_buf(c, a[0], KVM_M_FLT, o) || !kvm_buf(c, a[1], KVM_M_FLT, dO) || !kvm_buf(c, a[2], KVM_M_F32, delta)) return;
  const int r0 = a[3], r1 = a[4], T = a[5], H = a[6], hd = a[7];
  if (r0 < 0 || r1 < r0 || T <= 0 || H <= 0 || hd <= 0 || !kvm_mat_ok(c, o, r1, H * hd) || !kvm_mat_ok(c, dO, r1, H * hd) ||
      !kvm_flat_ok(c, delta, (long long)((r1 + T - 1) / T) * H * T)) { c.fail(KVM_OPE_RANGE, r0, r1); return; }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if ((hd == 64 || hd == 128 || hd == 32) && (o.ld & 7) == 0 && (dO.ld & 7) == 0 && kvm_vec_ok(o) && kvm_vec_ok(dO)) {
    // vector form: an item is 8 consecutive columns of one row (hd/8 neighbouring lanes make up a head); four items per thread
    // are loaded before any of them is reduced, so the loads of a task overlap instead of queueing behind each other's stores
    const int cpr = H * hd / 8, lph = hd / 8;                 // items per row, lanes per head
    const long long items = (long long)(r1 - r0) * cpr;
    for (long long i0 = 0; i0 < items; i0 += 4LL * KVM_NT) {
      float ov[4][8], dv[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long it = i0 + (long long)u * KVM_NT + threadIdx.x;
        if (it < items) {
          const int r = r0 + (int)(it / cpr), cc = (int)(it % cpr) * 8;
          kvm_ld8(o, (size_t)r * o.ld + cc, ov[u]); kvm_ld8(dO, (size_t)r * dO.ld + cc, dv[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long it = i0 + (long long)u * KVM_NT + threadIdx.x;      // KVM_NT and cpr are multiples of hd/8: a head never straddles warps or steps
        float s = 0.0f;
        if (it < items) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s += ov[u][j] * dv[u][j];
        }
        for (int w = lph >> 1; w; w >>= 1) s += __shfl_xor_sync(0xffffffffu, s, w);
        if (it < items && (lane % lph) == 0) {
          const int r = r0 + (int)(it / cpr), h = (int)(it % cpr) / lph;
          ((float*)delta.p)[(size_t)((r / T) * H + h) * T + r % T] = s;
        }
      }
    }
    return;
  }
  for (int e = warp; e < (r1 - r0) * H; e += KVM_NWARPS) {
    const int r = r0 + e / H, h = e % H;
    float s = 0.0f;
    for (int cc = lane; cc < hd; cc += 32) s += kvm_ld(o, (size_t)r * o.ld + h * hd + cc) * kvm_ld(dO, (size_t)r * dO.ld + h * hd + cc);
    s = kvm_warp_sum(s);
    if (lane == 0) ((float*)delta.p)[(size_t)((r / T) * H + h) * T + r % T] = s;
  }
}

KVM_OP_FN void kvm_op_attn_bwd_dq(const KvmCtx& c, const int32_t* a) {
  KvmBuf q, k, v, dO, lse, delta, dq;
  if (!kvm_buf(c, a[0], KVM_M_FLT, q) || !kvm_buf(c, a[1], KVM_M_FLT, k) || !kvm_buf(c, a[2], KVM_M_FLT, v) || !kvm_buf(c, a[3], KVM_M_FLT, dO) ||
      !kvm_buf(c, a[4], KVM_M_F32, lse) || !kvm_buf(c, a[5], KVM_M_F32, delta) || !kvm_buf(c, a[6], KVM_M_FLT, dq)) return;
  const int b = a[7], h = a[8], q0 = a[9], T = a[10], H = a[11], Hkv = a[12], hd = a[13];
  const float sc = kvm_bits_f32(a[14]);
  if (!kvm_attn_geom(c, b, h, q0, T, H, Hkv, hd) || h >= H) { c.fail(KVM_OPE_SHAPE, h, H); return; }
  const long long R = (long long)(b + 1) * T;
  if (!kvm_mat_ok(c, q, R, H * hd) || !kvm_mat_ok(c, k, R, Hkv * hd) || !kvm_mat_ok(c, v, R, Hkv * hd) || !kvm_mat_ok(c, dO, R, H * hd) ||
      !kvm_mat_ok(c, dq, R, H * hd) || !kvm_flat_ok(c, lse, R * H) || !kvm_flat_ok(c, delta, R * H)) return;
  const int kvh = h / (H / Hkv), lane = threadIdx.x & 31, warp = threadIdx.x >> 5, q1 = min(q0 + KVM_ATTN_ROWS, T);
  float* qs = (float*)c.smem + warp * 256;
  float* ds_ = qs + 128;
  const bool kvec = kvm_attn_vec(k, hd), vvec = kvm_attn_vec(v, hd);
  const int nc = (hd + 31) / 32;
  for (int gq = q0 + warp; gq < q1; gq += KVM_NWARPS) {
    __syncwarp();
    for (int cc = lane; cc < hd; cc += 32) {
      qs[cc] = kvm_ld(q, (size_t)(b * T + gq) * q.ld + h * hd + cc);
      ds_[cc] = kvm_ld(dO, (size_t)(b * T + gq) * dO.ld + h * hd + cc);
    }
    __syncwarp();
    const float li = ((const float*)lse.p)[(size_t)(b * H + h) * T + gq], di = ((const float*)delta.p)[(size_t)(b * H + h) * T + gq];
    float acc[4] = {0, 0, 0, 0};
    for (int j0 = 0; j0 <= gq; j0 += 32) {
      const int j = j0 + lane;
      float dsv = 0.0f;
      if (j <= gq) {
        const float s = kvm_dot_row(qs, k, (size_t)(b * T + j) * k.ld + kvh * hd, hd, kvec);
        const float dp = kvm_dot_row(ds_, v, (size_t)(b * T + j) * v.ld + kvh * hd, hd, vvec);
        dsv = __expf(s * sc - li) * (dp - di);
      }
      const int nk = min(32, gq + 1 - j0);
      for (int jj = 0; jj < nk; ++jj) {
        const float d = __shfl_sync(0xffffffffu, dsv, jj);
        const size_t ko = (size_t)(b * T + j0 + jj) * k.ld + kvh * hd;
#pragma unroll
        for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) acc[t] += d * kvm_ld(k, ko + lane + 32 * t);
      }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) kvm_st(dq, (size_t)(b * T + gq) * dq.ld + h * hd + lane + 32 * t, acc[t] * sc);
  }
}

KVM_OP_FN void kvm_op_attn_bwd_dkv(const KvmCtx& c, const int32_t* a) {
  KvmBuf q, k, v, dO, lse, delta, dk, dv;
  if (!kvm_buf(c, a[0], KVM_M_FLT, q) || !kvm_buf(c, a[1], KVM_M_FLT, k) || !kvm_buf(c, a[2], KVM_M_FLT, v) || !kvm_buf(c, a[3], KVM_M_FLT, dO) ||
      !kvm_buf(c, a[4], KVM_M_F32, lse) || !kvm_buf(c, a[5], KVM_M_F32, delta) || !kvm_buf(c, a[6], KVM_M_FLT, dk) || !kvm_buf(c, a[7], KVM_M_FLT, dv)) return;
  const int b = a[8], kvh = a[9], k0 = a[10], T = a[11], H = a[12], hd = a[13];
  const float sc = kvm_bits_f32(a[14]);
  if (hd <= 0 || k.cols % hd) { c.fail(KVM_OPE_SHAPE, hd, k.cols); return; }
  const int Hkv = k.cols / hd;
  if (!kvm_attn_geom(c, b, kvh, k0, T, H, Hkv, hd) || kvh >= Hkv) { c.fail(KVM_OPE_SHAPE, kvh, Hkv); return; }
  const long long R = (long long)(b + 1) * T;
  if (!kvm_mat_ok(c, q, R, H * hd) || !kvm_mat_ok(c, k, R, (kvh + 1) * hd) || !kvm_mat_ok(c, v, R, (kvh + 1) * hd) || !kvm_mat_ok(c, dO, R, H * hd) ||
      !kvm_mat_ok(c, dk, R, (kvh + 1) * hd) || !kvm_mat_ok(c, dv, R, (kvh + 1) * hd) || !kvm_flat_ok(c, lse, R * H) || !kvm_flat_ok(c, delta, R * H)) return;
  const int G = H / Hkv, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, k1 = min(k0 + KVM_ATTN_ROWS, T);
  float* ks = (float*)c.smem + warp * 256;
  float* vs = ks + 128;
  const bool qvec = kvm_attn_vec(q, hd), ovec = kvm_attn_vec(dO, hd);
  const int nc = (hd + 31) / 32;
  for (int gk = k0 + warp; gk < k1; gk += KVM_NWARPS) {
    __syncwarp();
    for (int cc = lane; cc < hd; cc += 32) {
      ks[cc] = kvm_ld(k, (size_t)(b * T + gk) * k.ld + kvh * hd + cc);
      vs[cc] = kvm_ld(v, (size_t)(b * T + gk) * v.ld + kvh * hd + cc);
    }
    __syncwarp();
    float ak[4] = {0, 0, 0, 0}, av[4] = {0, 0, 0, 0};
    for (int h = kvh * G; h < (kvh + 1) * G; ++h)
      for (int g0 = gk; g0 < T; g0 += 32) {
        const int gq = g0 + lane;
        float p = 0.0f, dsv = 0.0f;
        if (gq < T) {
          const float s = kvm_dot_row(ks, q, (size_t)(b * T + gq) * q.ld + h * hd, hd, qvec);
          const float dp = kvm_dot_row(vs, dO, (size_t)(b * T + gq) * dO.ld + h * hd, hd, ovec);
          p = __expf(s * sc - ((const float*)lse.p)[(size_t)(b * H + h) * T + gq]);
          dsv = p * (dp - ((const float*)delta.p)[(size_t)(b * H + h) * T + gq]);
        }
        const int nq = min(32, T - g0);
        for (int jj = 0; jj < nq; ++jj) {
          const float pj = __shfl_sync(0xffffffffu, p, jj), dj = __shfl_sync(0xffffffffu, dsv, jj);
          const size_t qo = (size_t)(b * T + g0 + jj) * q.ld + h * hd, oo = (size_t)(b * T + g0 + jj) * dO.ld + h * hd;
#pragma unroll
          for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) { av[t] += pj * kvm_ld(dO, oo + lane + 32 * t); ak[t] += dj * kvm_ld(q, qo + lane + 32 * t); }
        }
      }
#pragma unroll
    for (int t = 0; t < 4; ++t) if (t < nc && lane + 32 * t < hd) {
      kvm_st(dk, (size_t)(b * T + gk) * dk.ld + kvh * hd + lane + 32 * t, ak[t] * sc);
      kvm_st(dv, (size_t)(b * T + gk) * dv.ld + kvh * hd + lane + 32 * t, av[t]);
    }
  }
}
