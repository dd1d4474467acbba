// Row-structured memory-bound ops: embeddings, normalisation forward/backward, column sums, rotary embedding,
// cross-entropy, AdamW, gradient norm, argmax.  Reference semantics: runtime/ref_gpt.py:44-66,107-193,250-275,414-482,
// runtime/ref_extra.py:333-360.  Sums run in float32 warp/block trees of fixed shape (deterministic per launch geometry);
// the reference's CPU model sums in double, so these agree to its documented 1e-5 relative tolerance, not bitwise.
#pragma once
#include "kvm_dev.cuh"

// ---- embeddings --------------------------------------------------------------------------------------------------------------
KVM_OP_FN void kvm_op_embedding_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf ids, wte, wpe, out;
  if (!kvm_buf(c, a[0], KVM_M_I32, ids) || !kvm_buf(c, a[1], KVM_M_FLT, wte) || !kvm_buf(c, a[2], KVM_M_FLT, wpe, true) ||
      !kvm_buf(c, a[3], KVM_M_FLT, out)) return;
  int r0 = a[4], r1 = a[5], T = a[6], d = a[7];
  if (r0 < 0 || r1 < r0 || T <= 0 || d <= 0 || !kvm_flat_ok(c, ids, r1) || !kvm_mat_ok(c, out, r1, d) || !kvm_mat_ok(c, wte, 0, d) ||
      !kvm_mat_ok(c, wpe, T, d)) { c.fail(KVM_OPE_RANGE, r0, r1); return; }
  const int* id = (const int*)ids.p;
  long long n = (long long)(r1 - r0) * d;
  for (long long e = threadIdx.x; e < n; e += KVM_NT) {
    int r = r0 + (int)(e / d), col = (int)(e % d), tok = id[r];
    float v = 0.0f;
    if (tok < 0 || tok >= wte.rows) c.fail_any(KVM_OPE_TOKEN, tok, r);
    else {
      v = kvm_ld(wte, (size_t)tok * wte.ld + col);
      if (wpe.p) v = __fadd_rn(v, kvm_ld(wpe, (size_t)(r % T) * wpe.ld + col));
    }
    kvm_st(out, (size_t)r * out.ld + col, v);
  }
}

// One task owns keys [v0,v1): rows with a key in range are compacted in ascending order into shared memory (block-wide
// ordered scan), then added row by row, each thread owning columns, so every element sums its rows in ascending order
// with one float32 add each (runtime/ref_gpt.py:55-66).
KVM_OP_FN void kvm_op_embedding_bwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf ids, dout, dt;
  if (!kvm_buf(c, a[0], KVM_M_I32, ids, true) || !kvm_buf(c, a[1], KVM_M_FLT, dout) || !kvm_buf(c, a[2], KVM_M_F32, dt)) return;
  int N = a[3], mod = a[4], v0 = a[5], v1 = a[6], d = a[7], acc = a[8];
  if (N < 0 || v0 < 0 || v1 < v0 || d <= 0 || (!ids.p && mod <= 0) || !kvm_mat_ok(c, dout, N, d) || !kvm_mat_ok(c, dt, v1, d) ||
      !kvm_flat_ok(c, ids, N)) { c.fail(KVM_OPE_RANGE, v0, v1); return; }
  float* tab = (float*)dt.p;
  if (!ids.p) {
    // positional table: key k collects rows k, k+mod, k+2*mod, ... in that (ascending) order; thread = (key, column)
    for (long long e = threadIdx.x; e < (long long)(v1 - v0) * d; e += KVM_NT) {
      const int key = v0 + (int)(e / d), col = (int)(e % d);
      const size_t o = (size_t)key * dt.ld + col;
      float sum = acc ? tab[o] : 0.0f;
      if (key < mod) for (int r = key; r < N; r += mod) sum = __fadd_rn(sum, kvm_ld(dout, (size_t)r * dout.ld + col));
      tab[o] = sum;
    }
    return;
  }
  if (!acc)
    for (long long e = threadIdx.x; e < (long long)(v1 - v0) * d; e += KVM_NT) tab[(size_t)(v0 + e / d) * dt.ld + e % d] = 0.0f;
  int* list = (int*)c.smem;                       // [cap] rows, then KVM_NWARPS+1 counters
  const int cap = (c.smem_bytes - 256) / 4;
  int* wcnt = list + cap;
  const int* id = (const int*)ids.p;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  kvm_sync();
  for (int base = 0; base < N;) {
    // fill the list with up to cap matching rows starting at `base`
    int filled = 0, next = base;
    while (next < N && filled + KVM_NT <= cap) {
      int r = next + threadIdx.x;
      int key = r < N ? (id ? id[r] : r % mod) : -1;
      bool hit = r < N && key >= v0 && key < v1;
      unsigned m = __ballot_sync(0xffffffffu, hit);
      if (lane == 0) wcnt[warp] = __popc(m);
      kvm_sync();
      int off = filled;
      for (int w = 0; w < warp; ++w) off += wcnt[w];
      if (hit) list[off + __popc(m & ((1u << lane) - 1))] = r;
      int tot = 0;
      for (int w = 0; w < KVM_NWARPS; ++w) tot += wcnt[w];
      kvm_sync();
      filled += tot; next += KVM_NT;
    }
    kvm_sync();
    for (int i = 0; i < filled; ++i) {
      int r = list[i], key = id ? id[r] : r % mod;
      for (int col = threadIdx.x; col < d; col += KVM_NT) {
        size_t o = (size_t)key * dt.ld + col;
        tab[o] = __fadd_rn(tab[o], kvm_ld(dout, (size_t)r * dout.ld + col));
      }
    }
    kvm_sync();
    base = next;
  }
}

KVM_OP_FN void kvm_op_add_rowtile(const KvmCtx& c, const int32_t* a) {
  KvmBuf x, pos, out;
  if (!kvm_buf(c, a[0], KVM_M_FLT, x) || !kvm_buf(c, a[1], KVM_M_FLT, pos) || !kvm_buf(c, a[2], KVM_M_FLT, out)) return;
  int r0 = a[3], r1 = a[4], T = a[5], d = a[6];
  if (r0 < 0 || r1 < r0 || T <= 0 || d <= 0 || !kvm_mat_ok(c, x, r1, d) || !kvm_mat_ok(c, out, r1, d) || !kvm_mat_ok(c, pos, T, d)) {
    c.fail(KVM_OPE_RANGE, r0, r1); return; }
  for (long long e = threadIdx.x; e < (long long)(r1 - r0) * d; e += KVM_NT) {
    int r = r0 + (int)(e / d), col = (int)(e % d);
    kvm_st(out, (size_t)r * out.ld + col, __fadd_rn(kvm_ld(x, (size_t)r * x.ld + col), kvm_ld(pos, (size_t)(r % T) * pos.ld + col)));
  }
}

KVM_OP_FN void kvm_op_gather_rows(const KvmCtx& c, const int32_t* a) {
  KvmBuf src, idx, dst;
  if (!kvm_buf(c, a[0], KVM_M_FLT, src) || !kvm_buf(c, a[1], KVM_M_I32, idx) || !kvm_buf(c, a[2], KVM_M_FLT, dst)) return;
  int r0 = a[3], r1 = a[4], d = a[5];
  if (r0 < 0 || r1 < r0 || d <= 0 || !kvm_flat_ok(c, idx, r1) || !kvm_mat_ok(c, dst, r1, d) || !kvm_mat_ok(c, src, 0, d)) {
    c.fail(KVM_OPE_RANGE, r0, r1); return; }
  for (long long e = threadIdx.x; e < (long long)(r1 - r0) * d; e += KVM_NT) {
    int r = r0 + (int)(e / d), col = (int)(e % d), i = ((const int*)idx.p)[r];
    float v = 0.0f;
    if (i < 0 || i >= src.rows) c.fail_any(KVM_OPE_TOKEN, i, r);
    else v = kvm_ld(src, (size_t)i * src.ld + col);
    kvm_st(dst, (size_t)r * dst.ld + col, v);
  }
}

// ---- normalisation: one warp per row -----------------------------------------------------------------------------------------
template <bool RMS>
static __device__ void kvm_norm_fwd(const KvmCtx& c, int xi, int gi, int bi, int oi, int mi, int ri, int r0, int r1, int d, float eps) {
  KvmBuf x, g, be, out, mean, rstd;
  if (!kvm_buf(c, xi, KVM_M_FLT, x) || !kvm_buf(c, gi, KVM_M_F32, g) || !kvm_buf(c, bi, KVM_M_F32, be, RMS) || !kvm_buf(c, oi, KVM_M_FLT, out) ||
      !kvm_buf(c, mi, KVM_M_F32, mean, RMS) || !kvm_buf(c, ri, KVM_M_F32, rstd)) return;
  if (r0 < 0 || r1 < r0 || d <= 0 || !kvm_mat_ok(c, x, r1, d) || !kvm_mat_ok(c, out, r1, d) || !kvm_flat_ok(c, g, d) || !kvm_flat_ok(c, be, d) ||
      !kvm_flat_ok(c, mean, r1) || !kvm_flat_ok(c, rstd, r1)) { c.fail(KVM_OPE_RANGE, r0, r1); return; }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* gp = (const float*)g.p;
  const float* bp = (const float*)be.p;
  const bool vec = (d & 7) == 0 && (x.ld & 7) == 0 && (out.ld & 7) == 0 && kvm_vec_ok(x) && kvm_vec_ok(out) && kvm_vec_ok(g) && (RMS || kvm_vec_ok(be));
  if (vec && d <= 1024) {
    // the row (up to four 8-element vectors per lane) is fetched once and stays in registers over the two reductions (gamma and
    // beta come from L1 as vectors); same per-lane summation order as the loops below
    for (int r = r0 + warp; r < r1; r += KVM_NWARPS) {
      const size_t xo = (size_t)r * x.ld, oo = (size_t)r * out.ld;
      float xv[4][8], s = 0.0f, q = 0.0f;
#pragma unroll
      for (int t = 0; t < 4; ++t) { const int k = lane * 8 + t * 256; if (k < d) kvm_ld8(x, xo + k, xv[t]); }
      if (!RMS) {
#pragma unroll
        for (int t = 0; t < 4; ++t) if (lane * 8 + t * 256 < d) {
#pragma unroll
          for (int j = 0; j < 8; ++j) s += xv[t][j];
        }
        s = kvm_warp_sum(s);
      }
      const float mu = RMS ? 0.0f : s / d;
#pragma unroll
      for (int t = 0; t < 4; ++t) if (lane * 8 + t * 256 < d) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float tt = xv[t][j] - mu; q += tt * tt; }
      }
      q = kvm_warp_sum(q);
      const float rs = 1.0f / sqrtf(q / d + eps);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int k = lane * 8 + t * 256;
        if (k < d) {
          float ov[8], gv[8], bv[8];
          kvm_ld8(g, k, gv);
          if (!RMS) kvm_ld8(be, k, bv);
#pragma unroll
          for (int j = 0; j < 8; ++j) ov[j] = (xv[t][j] - mu) * rs * gv[j] + (RMS ? 0.0f : bv[j]);
          kvm_st8(out, oo + k, ov);
        }
      }
      if (lane == 0) { ((float*)rstd.p)[r] = rs; if (!RMS) ((float*)mean.p)[r] = mu; }
    }
    return;
  }
  for (int r = r0 + warp; r < r1; r += KVM_NWARPS) {
    const size_t xo = (size_t)r * x.ld, oo = (size_t)r * out.ld;
    float s = 0.0f;
    if (!RMS) {
      if (vec) for (int k = lane * 8; k < d; k += 256) { float v[8]; kvm_ld8(x, xo + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[j]; }
      else for (int k = lane; k < d; k += 32) s += kvm_ld(x, xo + k);
      s = kvm_warp_sum(s);
    }
    const float mu = RMS ? 0.0f : s / d;
    float q = 0.0f;
    if (vec) for (int k = lane * 8; k < d; k += 256) { float v[8]; kvm_ld8(x, xo + k, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { float t = v[j] - mu; q += t * t; } }
    else for (int k = lane; k < d; k += 32) { float t = kvm_ld(x, xo + k) - mu; q += t * t; }
    q = kvm_warp_sum(q);
    const float rs = 1.0f / sqrtf(q / d + eps);
    if (vec) for (int k = lane * 8; k < d; k += 256) {
      float v[8], o[8]; kvm_ld8(x, xo + k, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (v[j] - mu) * rs * gp[k + j] + (RMS ? 0.0f : bp[k + j]);
      kvm_st8(out, oo + k, o);
    } else for (int k = lane; k < d; k += 32) kvm_st(out, oo + k, (kvm_ld(x, xo + k) - mu) * rs * gp[k] + (RMS ? 0.0f : bp[k]));
    if (lane == 0) { ((float*)rstd.p)[r] = rs; if (!RMS) ((float*)mean.p)[r] = mu; }
  }
}
KVM_OP_FN void kvm_op_layernorm_fwd(const KvmCtx& c, const int32_t* a) {
  kvm_norm_fwd<false>(c, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], kvm_bits_f32(a[9]));
}
KVM_OP_FN void kvm_op_rmsnorm_fwd(const KvmCtx& c, const int32_t* a) {
  kvm_norm_fwd<true>(c, a[0], a[1], -1, a[2], -1, a[3], a[4], a[5], a[6], kvm_bits_f32(a[7]));
}

template <bool RMS>
static __device__ void kvm_norm_bwd_dx(const KvmCtx& c, int xi, int dyi, int gi, int mi, int ri, int dxi, int r0, int r1, int d, int acc) {
  KvmBuf x, dy, g, mean, rstd, dx;
  if (!kvm_buf(c, xi, KVM_M_FLT, x) || !kvm_buf(c, dyi, KVM_M_FLT, dy) || !kvm_buf(c, gi, KVM_M_F32, g) || !kvm_buf(c, mi, KVM_M_F32, mean, RMS) ||
      !kvm_buf(c, ri, KVM_M_F32, rstd) || !kvm_buf(c, dxi, KVM_M_FLT, dx)) return;
  if (r0 < 0 || r1 < r0 || d <= 0 || !kvm_mat_ok(c, x, r1, d) || !kvm_mat_ok(c, dy, r1, d) || !kvm_mat_ok(c, dx, r1, d) || !kvm_flat_ok(c, g, d) ||
      !kvm_flat_ok(c, mean, r1) || !kvm_flat_ok(c, rstd, r1)) { c.fail(KVM_OPE_RANGE, r0, r1); return; }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* gp = (const float*)g.p;
  const bool vec = (d & 7) == 0 && d <= 1024 && (x.ld & 7) == 0 && (dy.ld & 7) == 0 && (dx.ld & 7) == 0 && kvm_vec_ok(x) && kvm_vec_ok(dy) && kvm_vec_ok(dx) && kvm_vec_ok(g);
  for (int r = r0 + warp; r < r1; r += KVM_NWARPS) {
    const float mu = RMS ? 0.0f : ((const float*)mean.p)[r], rs = ((const float*)rstd.p)[r];
    const size_t xo = (size_t)r * x.ld, yo = (size_t)r * dy.ld, oo = (size_t)r * dx.ld;
    float s1 = 0.0f, s2 = 0.0f;
    if (vec) {      // the row stays in registers between the two passes: up to four 8-element vectors of x and dy per lane
      float xv[4][8], gv[4][8];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int k = lane * 8 + t * 256;
        if (k < d) {
          float yv[8], gm[8];
          kvm_ld8(x, xo + k, xv[t]); kvm_ld8(dy, yo + k, yv); kvm_ld8(g, k, gm);
#pragma unroll
          for (int j = 0; j < 8; ++j) { gv[t][j] = yv[j] * gm[j]; xv[t][j] = (xv[t][j] - mu) * rs; s1 += gv[t][j]; s2 += gv[t][j] * xv[t][j]; }
        }
      }
      s1 = RMS ? 0.0f : kvm_warp_sum(s1) / d;
      s2 = kvm_warp_sum(s2) / d;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int k = lane * 8 + t * 256;
        if (k < d) {
          float o[8];
          if (acc) kvm_ld8(dx, oo + k, o);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float v = rs * (gv[t][j] - s1 - xv[t][j] * s2); o[j] = acc ? __fadd_rn(o[j], v) : v; }
          kvm_st8(dx, oo + k, o);
        }
      }
      continue;
    }
    for (int k = lane; k < d; k += 32) {
      float gs = kvm_ld(dy, yo + k) * gp[k], xh = (kvm_ld(x, xo + k) - mu) * rs;
      s1 += gs; s2 += gs * xh;
    }
    s1 = RMS ? 0.0f : kvm_warp_sum(s1) / d;
    s2 = kvm_warp_sum(s2) / d;
    for (int k = lane; k < d; k += 32) {
      float gs = kvm_ld(dy, yo + k) * gp[k], xh = (kvm_ld(x, xo + k) - mu) * rs;
      float v = rs * (gs - s1 - xh * s2);
      kvm_st(dx, oo + k, acc ? __fadd_rn(kvm_ld(dx, oo + k), v) : v);
    }
  }
}
KVM_OP_FN void kvm_op_layernorm_bwd_dx(const KvmCtx& c, const int32_t* a) { kvm_norm_bwd_dx<false>(c, a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9]); }
KVM_OP_FN void kvm_op_rmsnorm_bwd_dx(const KvmCtx& c, const int32_t* a) { kvm_norm_bwd_dx<true>(c, a[0], a[1], a[2], -1, a[3], a[4], a[5], a[6], a[7], a[8]); }

// Column sums over R rows for columns [c0,c1): thread = (row group, column), row groups reduced in fixed order through
// shared memory.  MODE 0: colsum of x; MODE 1: dgamma / dbeta of a norm layer.
template <int MODE, bool XB, bool YB>
static __device__ void kvm_colreduce_t(const KvmCtx& c, const KvmBuf& x, const KvmBuf& dy, const KvmBuf& mean, const KvmBuf& rstd, float* o1, float* o2,
                                       int R, int c0, int c1, int acc) {
  float* red = (float*)c.smem;                    // [2][KVM_NT]
  const void* xp = x.p;
  const void* yp = dy.p;
  const float* mp = (const float*)mean.p;
  const float* rp = (const float*)rstd.p;
  const size_t xld = x.ld, yld = MODE == 1 ? dy.ld : 0;
  for (int cb = c0; cb < c1; cb += 64) {
    const int w = min(64, c1 - cb), col = threadIdx.x & 63, rg = threadIdx.x >> 6, ngroups = KVM_NT / 64;
    float s1 = 0.0f, s2 = 0.0f;
    if (col < w) {
      // latency-bound (one short load per row): eight rows' loads are issued before the first is used; the sums run in row order
      int r = rg;
      for (; r + 7 * ngroups < R; r += 8 * ngroups) {
        float xv[8], gv[8], mu[8], rs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int rr = r + u * ngroups;
          xv[u] = kvm_ldt<XB>(xp, (size_t)rr * xld + cb + col);
          if (MODE == 1) {
            gv[u] = kvm_ldt<YB>(yp, (size_t)rr * yld + cb + col);
            mu[u] = mp ? mp[rr] : 0.0f;
            rs[u] = rp[rr];
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (MODE == 0) s1 += xv[u];
          else { s1 += gv[u] * (xv[u] - mu[u]) * rs[u]; s2 += gv[u]; }
        }
      }
      for (; r < R; r += ngroups) {
        if (MODE == 0) s1 += kvm_ldt<XB>(xp, (size_t)r * xld + cb + col);
        else {
          const float g = kvm_ldt<YB>(yp, (size_t)r * yld + cb + col);
          const float mu = mp ? mp[r] : 0.0f;
          s1 += g * (kvm_ldt<XB>(xp, (size_t)r * xld + cb + col) - mu) * rp[r];
          s2 += g;
        }
      }
    }
    kvm_sync();
    red[threadIdx.x] = s1; red[KVM_NT + threadIdx.x] = s2;
    kvm_sync();
    if (threadIdx.x < w) {
      float t1 = 0.0f, t2 = 0.0f;
      for (int g = 0; g < ngroups; ++g) { t1 += red[g * 64 + threadIdx.x]; t2 += red[KVM_NT + g * 64 + threadIdx.x]; }
      const int cc = cb + threadIdx.x;
      o1[cc] = acc ? __fadd_rn(o1[cc], t1) : t1;
      if (MODE == 1 && o2) o2[cc] = acc ? __fadd_rn(o2[cc], t2) : t2;
    }
  }
}
// Column sums over R rows for columns [c0,c1): thread = (row group, column), row groups reduced in fixed order through
// shared memory.  MODE 0: colsum of x; MODE 1: dgamma / dbeta of a norm layer.  One instance per storage type of x (and dy).
template <int MODE>
static __device__ void kvm_colreduce(const KvmCtx& c, const KvmBuf& x, const KvmBuf& dy, const KvmBuf& mean, const KvmBuf& rstd, float* o1, float* o2,
                              int R, int c0, int c1, int acc) {
  const bool xb = x.dtype == KVM_BF16, yb = MODE == 1 && dy.dtype == KVM_BF16;
  if (MODE == 0) {
    if (xb) kvm_colreduce_t<MODE, true, false>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
    else kvm_colreduce_t<MODE, false, false>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
  } else if (xb) {
    if (yb) kvm_colreduce_t<MODE, true, true>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
    else kvm_colreduce_t<MODE, true, false>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
  } else {
    if (yb) kvm_colreduce_t<MODE, false, true>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
    else kvm_colreduce_t<MODE, false, false>(c, x, dy, mean, rstd, o1, o2, R, c0, c1, acc);
  }
}
KVM_OP_FN void kvm_op_colsum(const KvmCtx& c, const int32_t* a) {
  KvmBuf x, out, none{};
  if (!kvm_buf(c, a[0], KVM_M_FLT, x) || !kvm_buf(c, a[1], KVM_M_F32, out)) return;
  int R = a[2], c0 = a[3], c1 = a[4];
  if (R < 0 || c0 < 0 || c1 < c0 || !kvm_mat_ok(c, x, R, c1) || !kvm_flat_ok(c, out, c1)) { c.fail(KVM_OPE_RANGE, c0, c1); return; }
  kvm_colreduce<0>(c, x, none, none, none, (float*)out.p, nullptr, R, c0, c1, a[5]);
}
KVM_OP_FN void kvm_op_norm_bwd_params(const KvmCtx& c, const int32_t* a) {
  KvmBuf x, dy, mean, rstd, dg, db;
  if (!kvm_buf(c, a[0], KVM_M_FLT, x) || !kvm_buf(c, a[1], KVM_M_FLT, dy) || !kvm_buf(c, a[2], KVM_M_F32, mean, true) || !kvm_buf(c, a[3], KVM_M_F32, rstd) ||
      !kvm_buf(c, a[4], KVM_M_F32, dg) || !kvm_buf(c, a[5], KVM_M_F32, db, true)) return;
  int R = a[6], d = a[7], c0 = a[8], c1 = a[9];
  if (R < 0 || c0 < 0 || c1 < c0 || c1 > d || !kvm_mat_ok(c, x, R, d) || !kvm_mat_ok(c, dy, R, d) || !kvm_flat_ok(c, mean, R) || !kvm_flat_ok(c, rstd, R) ||
      !kvm_flat_ok(c, dg, d) || !kvm_flat_ok(c, db, d)) { c.fail(KVM_OPE_RANGE, c0, c1); return; }
  kvm_colreduce<1>(c, x, dy, mean, rstd, (float*)dg.p, (float*)db.p, R, c0, c1, a[10]);
}

// ---- rotary embedding (pairs (i, i+hd/2); ang = f32(f32(pos) * f32(theta^(-2i/hd))), runtime/ref_gpt.py:250-262) ------------------
__device__ __forceinline__ float kvm_rope_inv(float theta, int i, int hd) { return (float)pow((double)theta, -(double)(float)(2 * i) / hd); }
static __device__ void kvm_rope(const KvmCtx& c, const int32_t* a, float sign) {
  KvmBuf x, out, pos;
  if (!kvm_buf(c, a[0], KVM_M_FLT, x) || !kvm_buf(c, a[1], KVM_M_FLT, out) || !kvm_buf(c, a[2], KVM_M_I32, pos, true)) return;
  int r0 = a[3], r1 = a[4], T = a[5], H = a[6], hd = a[7];
  float theta = kvm_bits_f32(a[8]);
  if (r0 < 0 || r1 < r0 || T <= 0 || H <= 0 || hd <= 0 || (hd & 1) || hd > 512 || !kvm_mat_ok(c, x, r1, H * hd) || !kvm_mat_ok(c, out, r1, H * hd)) {
    c.fail(KVM_OPE_RANGE, r0, r1); return; }
  const int half = hd / 2, p0 = pos.p ? ((const int*)pos.p)[0] : 0;
  float* inv = (float*)c.smem;
  kvm_sync();
  for (int i = threadIdx.x; i < half; i += KVM_NT) inv[i] = kvm_rope_inv(theta, i, hd);
  kvm_sync();
  long long n = (long long)(r1 - r0) * H * half;
  for (long long e = threadIdx.x; e < n; e += KVM_NT) {
    int i = (int)(e % half), h = (int)((e / half) % H), r = r0 + (int)(e / ((long long)half * H));
    float ang = __fmul_rn((float)((r % T) + p0), inv[i]), s, co;
    sincosf(ang, &s, &co);
    s *= sign;
    size_t o1 = (size_t)r * x.ld + h * hd + i, w1 = (size_t)r * out.ld + h * hd + i;
    float x1 = kvm_ld(x, o1), x2 = kvm_ld(x, o1 + half);
    kvm_st(out, w1, x1 * co - x2 * s);
    kvm_st(out, w1 + half, x1 * s + x2 * co);
  }
}
KVM_OP_FN void kvm_op_rope_fwd(const KvmCtx& c, const int32_t* a) { kvm_rope(c, a, 1.0f); }
KVM_OP_FN void kvm_op_rope_bwd(const KvmCtx& c, const int32_t* a) { kvm_rope(c, a, -1.0f); }

// ---- cross entropy: the block walks rows; per row one pass for (max, sum) and one for the gradient -------------------------------------
// MODE bit 0: forward (rowloss, lse); bit 1: backward (dlogits).
template <int MODE, bool LB, bool DB>      // storage types of the logits and of their gradient as template arguments: no type test inside the loops
static __device__ void kvm_ce_t(const KvmCtx& c, const KvmBuf& lg, const KvmBuf& tg, const KvmBuf& rl, const KvmBuf& ls, const KvmBuf& dl, int r0, int r1, int V,
                         int ignore, float f) {
  float* red = (float*)c.smem;
  const bool vec = (V & 7) == 0 && (lg.ld & 7) == 0 && kvm_vec_ok(lg) && (!(MODE & 2) || ((dl.ld & 7) == 0 && kvm_vec_ok(dl)));
  for (int r = r0; r < r1; ++r) {
    const int t = ((const int*)tg.p)[r];
    const size_t lo = (size_t)r * lg.ld;
    float lse;
    if (t != ignore && (t < 0 || t >= V)) { c.fail(KVM_OPE_TOKEN, t, r); return; }
    if (MODE & 1) {
      if (t == ignore) { if (threadIdx.x == 0) { ((float*)rl.p)[r] = 0.0f; ((float*)ls.p)[r] = 0.0f; } lse = 0.0f; }
      else {
        float m = -INFINITY, s = 0.0f;            // online (max, sum) per thread
        if (vec) for (int k = threadIdx.x * 8; k < V; k += KVM_NT * 8) {
          float v[8]; kvm_ld8t<LB>(lg.p, lo + k, v);
          float mm = v[0];
#pragma unroll
          for (int j = 1; j < 8; ++j) mm = fmaxf(mm, v[j]);
          if (mm > m) { s *= __expf(m - mm); m = mm; }
#pragma unroll
          for (int j = 0; j < 8; ++j) s += __expf(v[j] - m);
        } else for (int k = threadIdx.x; k < V; k += KVM_NT) {
          float v = kvm_ldt<LB>(lg.p, lo + k);
          if (v > m) { s *= __expf(m - v); m = v; }
          s += __expf(v - m);
        }
        float M = kvm_block_max(m, red);
        s = (m == -INFINITY) ? 0.0f : s * __expf(m - M);
        float S = kvm_block_sum(s, red);
        lse = M + logf(S);
        if (threadIdx.x == 0) { ((float*)ls.p)[r] = lse; ((float*)rl.p)[r] = lse - kvm_ld(lg, lo + t); }
      }
    } else lse = ((const float*)ls.p)[r];
    if (MODE & 2) {
      const size_t dq = (size_t)r * dl.ld;
      if (vec) for (int k = threadIdx.x * 8; k < V; k += KVM_NT * 8) {
        float v[8], o[8]; kvm_ld8t<LB>(lg.p, lo + k, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = t == ignore ? 0.0f : (__expf(v[j] - lse) - (k + j == t ? 1.0f : 0.0f)) * f;
        kvm_st8t<DB>(dl.p, dq + k, o);
      } else for (int k = threadIdx.x; k < V; k += KVM_NT)
        kvm_st(dl, dq + k, t == ignore ? 0.0f : (__expf(kvm_ldt<LB>(lg.p, lo + k) - lse) - (k == t ? 1.0f : 0.0f)) * f);
    }
  }
}
template <int MODE>
static __device__ void kvm_ce(const KvmCtx& c, const KvmBuf& lg, const KvmBuf& tg, const KvmBuf& rl, const KvmBuf& ls, const KvmBuf& dl, int r0, int r1, int V,
                       int ignore, float f) {
  const bool lb = lg.dtype == KVM_BF16, db = (MODE & 2) && dl.dtype == KVM_BF16;
  if (lb) { if (db) kvm_ce_t<MODE, true, true>(c, lg, tg, rl, ls, dl, r0, r1, V, ignore, f); else kvm_ce_t<MODE, true, false>(c, lg, tg, rl, ls, dl, r0, r1, V, ignore, f); }
  else { if (db) kvm_ce_t<MODE, false, true>(c, lg, tg, rl, ls, dl, r0, r1, V, ignore, f); else kvm_ce_t<MODE, false, false>(c, lg, tg, rl, ls, dl, r0, r1, V, ignore, f); }
}
static __device__ bool kvm_ce_args(const KvmCtx& c, const KvmBuf& lg, const KvmBuf& tg, const KvmBuf& rl, const KvmBuf& ls, const KvmBuf& dl, int r0, int r1, int V) {
  if (r0 < 0 || r1 < r0 || V <= 0 || !kvm_mat_ok(c, lg, r1, V) || !kvm_flat_ok(c, tg, r1) || !kvm_flat_ok(c, rl, r1) || !kvm_flat_ok(c, ls, r1) ||
      !kvm_mat_ok(c, dl, r1, V)) { c.fail(KVM_OPE_RANGE, r0, r1); return false; }
  return true;
}
KVM_OP_FN void kvm_op_softmax_ce_fwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf lg, tg, rl, ls, none{};
  if (!kvm_buf(c, a[0], KVM_M_FLT, lg) || !kvm_buf(c, a[1], KVM_M_I32, tg) || !kvm_buf(c, a[2], KVM_M_F32, rl) || !kvm_buf(c, a[3], KVM_M_F32, ls)) return;
  if (!kvm_ce_args(c, lg, tg, rl, ls, none, a[4], a[5], a[6])) return;
  kvm_ce<1>(c, lg, tg, rl, ls, none, a[4], a[5], a[6], a[7], 0.0f);
}
KVM_OP_FN void kvm_op_softmax_ce_bwd(const KvmCtx& c, const int32_t* a) {
  KvmBuf lg, tg, ls, loss, dl, none{};
  if (!kvm_buf(c, a[0], KVM_M_FLT, lg) || !kvm_buf(c, a[1], KVM_M_I32, tg) || !kvm_buf(c, a[2], KVM_M_F32, ls) || !kvm_buf(c, a[3], KVM_M_F32, loss) ||
      !kvm_buf(c, a[4], KVM_M_FLT, dl)) return;
  if (!kvm_ce_args(c, lg, tg, none, ls, dl, a[5], a[6], a[7]) || !kvm_flat_ok(c, loss, 2)) return;
  kvm_ce<2>(c, lg, tg, none, ls, dl, a[5], a[6], a[7], a[8], __fmul_rn(((const float*)loss.p)[1], kvm_bits_f32(a[9])));
}
KVM_OP_FN void kvm_op_softmax_ce_fused(const KvmCtx& c, const int32_t* a) {
  KvmBuf lg, tg, rl, ls, dl;
  if (!kvm_buf(c, a[0], KVM_M_FLT, lg) || !kvm_buf(c, a[1], KVM_M_I32, tg) || !kvm_buf(c, a[2], KVM_M_F32, rl) || !kvm_buf(c, a[3], KVM_M_F32, ls) ||
      !kvm_buf(c, a[4], KVM_M_FLT, dl)) return;
  if (a[8] != -1 || a[9] <= 0) { c.fail(KVM_OPE_RANGE, a[8], a[9]); return; }
  if (!kvm_ce_args(c, lg, tg, rl, ls, dl, a[5], a[6], a[7])) return;
  kvm_ce<3>(c, lg, tg, rl, ls, dl, a[5], a[6], a[7], -1, __fmul_rn((float)(1.0 / (double)a[9]), kvm_bits_f32(a[10])));
}
// loss[0] = mean rowloss over non-ignored rows, loss[1] = 1/count (runtime/ref_gpt.py:430-437); double sums, fixed tree.
KVM_OP_FN void kvm_op_softmax_ce_reduce(const KvmCtx& c, const int32_t* a) {
  KvmBuf rl, tg, loss;
  if (!kvm_buf(c, a[0], KVM_M_F32, rl) || !kvm_buf(c, a[1], KVM_M_I32, tg) || !kvm_buf(c, a[2], KVM_M_F32, loss)) return;
  int N = a[3], ign = a[4];
  if (N < 0 || !kvm_flat_ok(c, rl, N) || !kvm_flat_ok(c, tg, N) || !kvm_flat_ok(c, loss, 2)) { c.fail(KVM_OPE_RANGE, N); return; }
  double s = 0.0, cnt = 0.0;
  for (int r = threadIdx.x; r < N; r += KVM_NT)
    if (((const int*)tg.p)[r] != ign) { s += ((const float*)rl.p)[r]; cnt += 1.0; }
  double* red = (double*)c.smem;
  s = kvm_block_sum(s, red);
  cnt = kvm_block_sum(cnt, red);
  if (threadIdx.x == 0) {
    ((float*)loss.p)[0] = cnt > 0 ? (float)(s / cnt) : 0.0f;
    ((float*)loss.p)[1] = cnt > 0 ? (float)(1.0 / cnt) : 0.0f;
  }
}

// ---- optimiser ---------------------------------------------------------------------------------------------------------------------
// AdamW in the reference's strict float32 step order (runtime/ref_gpt.py:457-471): every operation below is one rounded
// float32 operation with no fused multiply-add, so p, m, v come out bit-identical to the CPU model.
static __device__ void kvm_adamw(const KvmCtx& c, const int32_t* a, bool lr_buf) {
  KvmBuf p, g, m, v, gs, st, lrb;
  if (!kvm_buf(c, a[0], KVM_M_F32, p) || !kvm_buf(c, a[1], KVM_M_FLT, g) || !kvm_buf(c, a[2], KVM_M_F32, m) || !kvm_buf(c, a[3], KVM_M_F32, v) ||
      !kvm_buf(c, a[4], KVM_M_F32, gs, true) || !kvm_buf(c, a[5], KVM_M_I32, st)) return;
  if (lr_buf && !kvm_buf(c, a[8], KVM_M_F32, lrb)) return;
  long long e0 = a[6], e1 = a[7];
  if (e0 < 0 || e1 < e0 || !kvm_flat_ok(c, p, e1) || !kvm_flat_ok(c, g, e1) || !kvm_flat_ok(c, m, e1) || !kvm_flat_ok(c, v, e1)) { c.fail(KVM_OPE_RANGE, (int)e0, (int)e1); return; }
  const int t = ((const int*)st.p)[0];
  if (t < 1) { c.fail(KVM_OPE_RANGE, t); return; }
  const float lr = lr_buf ? ((const float*)lrb.p)[0] : kvm_bits_f32(a[8]);
  const float b1 = kvm_bits_f32(a[9]), b2 = kvm_bits_f32(a[10]), eps = kvm_bits_f32(a[11]), wd = kvm_bits_f32(a[12]);
  float* sh = (float*)c.smem;
  kvm_sync();
  if (threadIdx.x == 0) {
    sh[0] = (float)(1.0 - (double)(float)pow((double)b1, (double)t));
    sh[1] = (float)(1.0 - (double)(float)pow((double)b2, (double)t));
  }
  kvm_sync();
  const float bc1 = sh[0], bc2 = sh[1], gsc = gs.p ? ((const float*)gs.p)[0] : 1.0f;
  const float omb1 = (float)(1.0 - (double)b1), omb2 = (float)(1.0 - (double)b2), lrwd = __fmul_rn(lr, wd);
  float* pp = (float*)p.p; float* mp = (float*)m.p; float* vp = (float*)v.p;
  auto upd = [&](float pi, float gi0, float mi0, float vi0, float& po, float& mo, float& vo) {
    float gi = __fmul_rn(gi0, gsc);
    mo = __fadd_rn(__fmul_rn(b1, mi0), __fmul_rn(omb1, gi));
    vo = __fadd_rn(__fmul_rn(b2, vi0), __fmul_rn(__fmul_rn(omb2, gi), gi));
    float decay = __fmul_rn(lrwd, pi);
    float step = __fdiv_rn(__fmul_rn(lr, __fdiv_rn(mo, bc1)), __fadd_rn(__fsqrt_rn(__fdiv_rn(vo, bc2)), eps));
    po = __fsub_rn(__fsub_rn(pi, decay), step);
  };
  const bool vec = (e0 & 7) == 0 && kvm_vec_ok(p) && kvm_vec_ok(g) && kvm_vec_ok(m) && kvm_vec_ok(v);
  long long body = vec ? ((e1 - e0) & ~7LL) : 0;
  for (long long i = e0 + (long long)threadIdx.x * 8; i + 8 <= e0 + body; i += (long long)KVM_NT * 8) {
    float P[8], G[8], M[8], Vv[8];
    kvm_ld8(p, i, P); kvm_ld8(g, i, G); kvm_ld8(m, i, M); kvm_ld8(v, i, Vv);
#pragma unroll
    for (int j = 0; j < 8; ++j) upd(P[j], G[j], M[j], Vv[j], P[j], M[j], Vv[j]);
    kvm_st8(p, i, P); kvm_st8(m, i, M); kvm_st8(v, i, Vv);
  }
  for (long long i = e0 + body + threadIdx.x; i < e1; i += KVM_NT) upd(pp[i], kvm_ld(g, i), mp[i], vp[i], pp[i], mp[i], vp[i]);
}
KVM_OP_FN void kvm_op_adamw(const KvmCtx& c, const int32_t* a) { kvm_adamw(c, a, false); }
KVM_OP_FN void kvm_op_adamw_lr(const KvmCtx& c, const int32_t* a) { kvm_adamw(c, a, true); }

KVM_OP_FN void kvm_op_lr_schedule(const KvmCtx& c, const int32_t* a) {
  KvmBuf st, lr;
  if (!kvm_buf(c, a[0], KVM_M_I32, st) || !kvm_buf(c, a[1], KVM_M_F32, lr)) return;
  int kind = a[2], warmup = a[4], total = a[5];
  if (kind < 0 || kind > 2) { c.fail(KVM_OPE_RANGE, kind); return; }
  if (threadIdx.x == 0) {
    double t = ((const int*)st.p)[0], base = kvm_bits_f32(a[3]), mr = kvm_bits_f32(a[6]);
    double warm = (warmup > 0 && t <= warmup) ? t / warmup : 1.0;
    double den = total - warmup > 1 ? total - warmup : 1;
    double prog = fmin(fmax((t - warmup) / den, 0.0), 1.0);
    double f = kind == 0 ? 1.0 : kind == 1 ? mr + (1 - mr) * 0.5 * (1 + cos(3.141592653589793 * prog)) : 1.0 - (1 - mr) * prog;
    ((float*)lr.p)[0] = (float)(base * warm * f);
  }
}

KVM_OP_FN void kvm_op_gradnorm_partial(const KvmCtx& c, const int32_t* a) {
  KvmBuf g, part;
  if (!kvm_buf(c, a[0], KVM_M_FLT, g) || !kvm_buf(c, a[1], KVM_M_F32, part)) return;
  int slot = a[2];
  long long e0 = a[3], e1 = a[4];
  if (slot < 0 || e0 < 0 || e1 < e0 || !kvm_flat_ok(c, g, e1) || !kvm_flat_ok(c, part, slot + 1)) { c.fail(KVM_OPE_RANGE, slot); return; }
  double s = 0.0;
  const bool vec = (e0 & 7) == 0 && kvm_vec_ok(g);
  long long body = vec ? ((e1 - e0) & ~7LL) : 0;
  for (long long i = e0 + (long long)threadIdx.x * 8; i + 8 <= e0 + body; i += (long long)KVM_NT * 8) {
    float v[8]; kvm_ld8(g, i, v);
    float q = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) q += v[j] * v[j];
    s += q;
  }
  for (long long i = e0 + body + threadIdx.x; i < e1; i += KVM_NT) { float v = kvm_ld(g, i); s += (double)v * v; }
  s = kvm_block_sum(s, (double*)c.smem);
  if (threadIdx.x == 0) ((float*)part.p)[slot] = (float)s;
}
KVM_OP_FN void kvm_op_gradnorm_finish(const KvmCtx& c, const int32_t* a) {
  KvmBuf part, out;
  if (!kvm_buf(c, a[0], KVM_M_F32, part) || !kvm_buf(c, a[2], KVM_M_F32, out)) return;
  int ns = a[1];
  float mx = kvm_bits_f32(a[3]);
  if (ns < 0 || !kvm_flat_ok(c, part, ns) || !kvm_flat_ok(c, out, 2)) { c.fail(KVM_OPE_RANGE, ns); return; }
  double s = 0.0;
  for (int i = threadIdx.x; i < ns; i += KVM_NT) s += ((const float*)part.p)[i];
  s = kvm_block_sum(s, (double*)c.smem);
  if (threadIdx.x == 0) {
    float n = (float)sqrt(s);
    ((float*)out.p)[0] = mx > 0 ? fminf(1.0f, __fdiv_rn(mx, __fadd_rn(n, 1e-6f))) : 1.0f;
    ((float*)out.p)[1] = n;
  }
}

// ---- argmax (lowest index on ties, NaN never wins; runtime/ref_gpt.py:508-514) -------------------------------------------------------
static __device__ void kvm_argmax_rows(const KvmCtx& c, const KvmBuf& lg, const KvmBuf& out, int r0, int r1, int V) {
  float* rv = (float*)c.smem;
  int* ri = (int*)(rv + KVM_NWARPS);
  for (int r = r0; r < r1; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int k = threadIdx.x; k < V; k += KVM_NT) {
      float v = kvm_ld(lg, (size_t)r * lg.ld + k);
      if (v > bv || (v == bv && k < bi)) { bv = v; bi = k; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    kvm_sync();
    if ((threadIdx.x & 31) == 0) { rv[threadIdx.x >> 5] = bv; ri[threadIdx.x >> 5] = bi; }
    kvm_sync();
    if (threadIdx.x == 0) {
      for (int w = 1; w < KVM_NWARPS; ++w) if (rv[w] > bv || (rv[w] == bv && ri[w] < bi)) { bv = rv[w]; bi = ri[w]; }
      ((int*)out.p)[r] = bi == 0x7fffffff ? 0 : bi;
    }
  }
}
KVM_OP_FN void kvm_op_argmax(const KvmCtx& c, const int32_t* a) {
  KvmBuf lg, out;
  if (!kvm_buf(c, a[0], KVM_M_FLT, lg) || !kvm_buf(c, a[1], KVM_M_I32, out)) return;
  if (a[2] < 0 || a[3] < a[2] || a[4] <= 0 || !kvm_mat_ok(c, lg, a[3], a[4]) || !kvm_flat_ok(c, out, a[3])) { c.fail(KVM_OPE_RANGE, a[2], a[3]); return; }
  kvm_argmax_rows(c, lg, out, a[2], a[3], a[4]);
}
