// Streaming forms of the decode ops: weights and cache rows travel global -> shared memory as bulk asynchronous copies
// (cp.async.bulk, completion counted on mbarriers) so that far more bytes are in flight per SM than register loads allow.
//   kvm_gemv_stream       rows [n0,n1) of a bf16 [N,K] weight matrix through a ring of up to 64 KB stages (whole rows)
//   kvm_attn_part_stream  all keys and values of one context split in one go, scores / softmax / PV from shared memory
// Numerics are those of the register-load forms in kvm_ops_decode.cuh (float32 accumulation, fixed order per launch geometry);
// op semantics: runtime/ref_extra.py:398-498 of the reference.  The mbarriers live in the op's own scratch: initialised at
// the start of the task, invalidated at its end.  Every wait is bounded; on expiry the task records KVM_ERR_TIMEOUT.
#pragma once
#include "kvm_dev.cuh"
#include "kvm_gemm_tc.cuh"
#include "kvm_ops_flat.cuh"

#define KVM_GS_UNITS 8                  // consumer warps of the streaming GEMV: unit = (row of the stage, part of K)
#define KVM_GS_STAGE_MAX 65536          // bytes of one stage (one bulk copy when the rows are contiguous)
#define KVM_GS_MAX_STAGES 4
#define KVM_STREAM_WAIT_NS 2000000000ull

__device__ __forceinline__ void kvm_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void kvm_mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void kvm_mbar_inval(uint32_t bar) { asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory"); }
// Wait on phase parity, bounded by wall time (2 s): returns false when the time ran out.
__device__ __forceinline__ bool kvm_mbar_wait_t(uint32_t bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63) == 63) {
      const unsigned long long t = kvm_globaltimer();
      if (!t0) t0 = t; else if (t - t0 > KVM_STREAM_WAIT_NS) return false;
    }
  }
}
__device__ __forceinline__ void kvm_stream_timeout(const KvmCtx& c, int where) {
  if (atomicCAS(&c.err->code, 0, KVM_ERR_TIMEOUT) == 0) { c.err->task = c.task; c.err->a = where; c.err->b = (int)threadIdx.x; }
}
__device__ __forceinline__ float kvm_bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float kvm_bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Streaming GEMV.  A stage holds R consecutive weight rows in full (R a power of two <= 8, R*K*2 <= 64 KB): one bulk copy when
// the rows are contiguous (ld == K), else one per row.  Warp 15 is the producer (one lane issues the copies and only waits for
// free stages); warps 0..7 consume: unit u = (row u / KP, part u % KP of K), KP = 8 / R, each lane 8 consecutive k per
// 256-wide block; the other warps only help with the prologue.  Per row the KP partial sums are added in part order.
// The activation row v = bf16(prologue(x)) is staged once as floats.  Returns false when the ring does not fit in the scratch
// (the caller then uses the register-load form).
static __device__ bool kvm_gemv_stream(const KvmCtx& c, const KvmBuf& x, const KvmBuf& x2, const KvmBuf& gm, const KvmBuf& w, const KvmBuf& out, const KvmBuf& res,
                                int n0, int n1, int K, int pro, float eps) {
  const int rows = n1 - n0;
  int R = KVM_GS_UNITS;
  while (R > 1 && R * K * 2 > KVM_GS_STAGE_MAX) R >>= 1;
  // at least three stages in flight where the scratch allows: smaller stages (fewer rows each) rather than a two-deep ring
  while (R > 1 && (c.smem_bytes - ((256 + K * 4 + 256 + ((rows + 7) & ~7) * (KVM_GS_UNITS / R) * 4 + 127) & ~127)) / ((R * K * 2 + 127) & ~127) < 3) R >>= 1;
  const int KP = KVM_GS_UNITS / R, stage_bytes = (R * K * 2 + 127) & ~127;
  const int plen = (((K + KP - 1) / KP) + 255) & ~255;                      // k extent of one part
  const int fixed = (256 + K * 4 + 256 + ((rows + 7) & ~7) * KP * 4 + 127) & ~127;
  int NS = stage_bytes > 0 ? (c.smem_bytes - fixed) / stage_bytes : 0;
  if (NS < 2 || R * K * 2 > KVM_GS_STAGE_MAX) return false;
  NS = min(NS, KVM_GS_MAX_STAGES);
  unsigned char* sm = c.smem;
  const uint32_t bar0 = kvm_smem_addr(sm);                 // full[s] at bar0 + 8 s, empty[s] at bar0 + 128 + 8 s
  float* vs = (float*)(sm + 256);
  float* red = vs + K;
  float* parts = red + 64;                                 // [rows][KP]
  unsigned char* stages = sm + fixed;
  const uint32_t stage0 = kvm_smem_addr(stages);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int NC = (rows + R - 1) / R;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w.p;
  const bool contiguous = w.ld == K;

  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // earlier plain accesses to this scratch come before the copies
  kvm_sync();
  bool ok = true;
  auto issue = [&](int ci) {                                       // producer lane only
    const int s = ci % NS, use = ci / NS;
    if (use > 0 && !kvm_mbar_wait_t(bar0 + 128 + 8 * s, (uint32_t)(use - 1) & 1)) { ok = false; return; }
    const int r0 = n0 + ci * R, nr = min(R, n1 - r0);
    kvm_mbar_expect_tx(bar0 + 8 * s, (uint32_t)(nr * K * 2));
    if (contiguous) kvm_bulk_g2s(stage0 + s * stage_bytes, wp + (size_t)r0 * w.ld, (uint32_t)(nr * K * 2), bar0 + 8 * s);
    else for (int r = 0; r < nr; ++r) kvm_bulk_g2s(stage0 + s * stage_bytes + r * K * 2, wp + (size_t)(r0 + r) * w.ld, (uint32_t)(K * 2), bar0 + 8 * s);
  };
  const bool producer = tid == (KVM_NWARPS - 1) * 32;
  int ni = 0;
  if (producer) {
    for (int s = 0; s < NS; ++s) { kvm_mbar_init(bar0 + 8 * s, 1); kvm_mbar_init(bar0 + 128 + 8 * s, KVM_GS_UNITS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (; ni < min(NS, NC); ++ni) issue(ni);                      // the weights start to stream while the prologue runs
  }
  __syncwarp();

  // ---- prologue: v = bf16(pro(x)) as floats in shared memory (all 16 warps)
  if (pro == 1 && K <= 16 * KVM_NT) {           // x and gamma fetched together and kept in registers over the block sum
    float xr[16], gr[16], q = 0.0f;
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int k = tid + u * KVM_NT;
      xr[u] = k < K ? kvm_ld(x, k) : 0.0f;
      gr[u] = k < K ? ((const float*)gm.p)[k] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) q += xr[u] * xr[u];
    q = kvm_block_sum(q, red);
    const float rs = 1.0f / sqrtf(q / K + eps);
#pragma unroll
    for (int u = 0; u < 16; ++u) { const int k = tid + u * KVM_NT; if (k < K) vs[k] = kvm_bf16_round(xr[u] * rs * gr[u]); }
  } else if (pro == 1) {
    float q = 0.0f;
    for (int k = tid; k < K; k += KVM_NT) { const float t = kvm_ld(x, k); vs[k] = t; q += t * t; }
    q = kvm_block_sum(q, red);
    const float rs = 1.0f / sqrtf(q / K + eps);
    for (int k = tid; k < K; k += KVM_NT) vs[k] = kvm_bf16_round(vs[k] * rs * ((const float*)gm.p)[k]);
  } else {
    // eight elements per thread at a time, all loads before the first store: a store to shared memory between two global loads
    // would keep the second from being issued early (the compiler cannot prove the pointers apart), one round trip per element
    for (int k0 = 0; k0 < K; k0 += 8 * KVM_NT) {
      float a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + tid + u * KVM_NT;
        a[u] = k < K ? kvm_ld(x, k) : 0.0f;
        b[u] = (pro == 2 && k < K) ? kvm_ld(x2, k) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + tid + u * KVM_NT;
        if (k < K) vs[k] = kvm_bf16_round(pro == 2 ? kvm_silu(a[u]) * b[u] : a[u]);
      }
    }
  }
  kvm_sync();

  if (producer) {
    for (; ni < NC && ok; ++ni) issue(ni);
  } else if (warp < KVM_GS_UNITS) {
    const int r = warp / KP, part = warp % KP, kb = part * plen, ke = min(K, kb + plen);
    for (int ci = 0; ci < NC; ++ci) {
      const int s = ci % NS;
      if (!kvm_mbar_wait_t(bar0 + 8 * s, (uint32_t)(ci / NS) & 1)) { ok = false; break; }
      if (ci * R + r < rows) {
        const unsigned char* st = stages + s * stage_bytes + (size_t)r * K * 2;
        float acc = 0.0f;
        for (int k = kb + lane * 8; k < ke; k += 256) {
          const uint4 wv = *(const uint4*)(st + k * 2);
          const float4 xa = *(const float4*)(vs + k), xb = *(const float4*)(vs + k + 4);
          acc = fmaf(xa.x, kvm_bf16lo(wv.x), acc); acc = fmaf(xa.y, kvm_bf16hi(wv.x), acc); acc = fmaf(xa.z, kvm_bf16lo(wv.y), acc); acc = fmaf(xa.w, kvm_bf16hi(wv.y), acc);
          acc = fmaf(xb.x, kvm_bf16lo(wv.z), acc); acc = fmaf(xb.y, kvm_bf16hi(wv.z), acc); acc = fmaf(xb.z, kvm_bf16lo(wv.w), acc); acc = fmaf(xb.w, kvm_bf16hi(wv.w), acc);
        }
        acc = kvm_warp_sum(acc);
        if (lane == 0) parts[(ci * R + r) * KP + part] = acc;
      }
      __syncwarp();
      if (lane == 0) kvm_mbar_arrive(bar0 + 128 + 8 * s);
    }
  }
  __syncwarp();
  if (!ok) kvm_stream_timeout(c, 134);
  kvm_sync();
  for (int i = tid; i < rows; i += KVM_NT) {
    float sum = 0.0f;
    for (int p = 0; p < KP; ++p) sum += parts[i * KP + p];
    kvm_st(out, n0 + i, res.p ? __fadd_rn(sum, kvm_ld(res, n0 + i)) : sum);
  }
  if (producer) for (int s = 0; s < NS; ++s) { kvm_mbar_inval(bar0 + 8 * s); kvm_mbar_inval(bar0 + 128 + 8 * s); }
  return true;
}

// ---- split-context decode attention from shared memory ------------------------------------------------------------------------
// One kv head, keys [j0,j1) of cache rows `base + j`, G = H/Hkv query heads (rotated queries in qs [G][hd], float).
// Keys and values (bf16, rows contiguous: ld == hd) arrive as two bulk copies.  If `newrow` >= 0 that key is the one this task
// appends: its rotated key / value (float, hd each, in knew / vnew shared arrays) is placed in the staged tiles by the threads
// and the copies leave it out.
//   scores   kvm_decode_scores: lanes = (key, head, pieces of the row), query values in registers, shuffle sums
//   softmax  over the whole split at once (warp g = query head g): p = exp(s - m) kept in shared memory as [key][8]
//   PV       thread = (key group, column pair): all G heads share one read of V; key groups are summed in group order
// emit(g, column, m, l, acc) as in kvm_decode_group.  Returns false when the split does not fit in shared memory.
// Scores of one split from the staged keys: s[key][g] = scale * q_g . k_key.  A key is spread over G*(hd/8)/CPL lanes: each lane
// owns one query head g and CPL 16-byte pieces (8 columns each) of the row, with its 8*CPL query values in registers (a small,
// fixed register footprint whatever G is); the lanes of one (key, g) are neighbours and add up by shuffles; a warp takes
// 32 / lanes-per-key consecutive keys per step.  Needs G and hd/8 to be powers of two and lanes-per-key <= 32.
template <int CPL>
__device__ __forceinline__ void kvm_decode_scores(const unsigned char* Ks, const float* qs, float* ps, int nk, int G, int hd, float sc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nch = hd >> 3, lpg = nch / CPL, lpk = G * lpg, KPW = 32 / lpk;         // lanes per (key, head), per key; keys per warp step
  const int sub = lane / lpk, li = lane % lpk, g = li / lpg, ch0 = (li % lpg) * CPL;
  float qr[CPL * 8];
#pragma unroll
  for (int j = 0; j < CPL; ++j) {
    const float4 qa = *(const float4*)(qs + g * hd + (ch0 + j) * 8), qb = *(const float4*)(qs + g * hd + (ch0 + j) * 8 + 4);
    qr[8 * j] = qa.x; qr[8 * j + 1] = qa.y; qr[8 * j + 2] = qa.z; qr[8 * j + 3] = qa.w; qr[8 * j + 4] = qb.x; qr[8 * j + 5] = qb.y; qr[8 * j + 6] = qb.z; qr[8 * j + 7] = qb.w;
  }
  for (int key0 = warp * KPW; key0 < nk; key0 += KVM_NWARPS * KPW) {
    const int key = key0 + sub, kk = min(key, nk - 1);
    const unsigned char* kp = Ks + (size_t)kk * hd * 2 + ch0 * 16;
    float sg = 0.0f;
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
      const uint4 kv = *(const uint4*)(kp + j * 16);
      sg = fmaf(qr[8 * j], kvm_bf16lo(kv.x), sg); sg = fmaf(qr[8 * j + 1], kvm_bf16hi(kv.x), sg); sg = fmaf(qr[8 * j + 2], kvm_bf16lo(kv.y), sg);
      sg = fmaf(qr[8 * j + 3], kvm_bf16hi(kv.y), sg); sg = fmaf(qr[8 * j + 4], kvm_bf16lo(kv.z), sg); sg = fmaf(qr[8 * j + 5], kvm_bf16hi(kv.z), sg);
      sg = fmaf(qr[8 * j + 6], kvm_bf16lo(kv.w), sg); sg = fmaf(qr[8 * j + 7], kvm_bf16hi(kv.w), sg);
    }
    for (int o = lpg >> 1; o; o >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, o);
    if (key < nk && (li % lpg) == 0) ps[key * 8 + g] = sg * sc;
  }
}

#define KVM_AS_QS 4096             // byte offsets in the op scratch: 64 barriers | qs [8][128] | inv [128] | knew [128] | vnew [128] | ml [16] | ...
#define KVM_AS_OFF_QS 64
#define KVM_AS_OFF_INV (64 + KVM_AS_QS)
#define KVM_AS_OFF_KNEW (KVM_AS_OFF_INV + 512)
#define KVM_AS_OFF_VNEW (KVM_AS_OFF_INV + 1024)
#define KVM_AS_OFF_ML (KVM_AS_OFF_INV + 1536)
#define KVM_AS_OFF_SC (KVM_AS_OFF_ML + 64)
#define KVM_ATTN_EMPTY_M_STREAM (-3.4028234663852886e38f)
// The part of the split attention that runs once the key / value tiles are on their way into shared memory: prologue (rotated
// queries, the appended key / value), scores, softmax over the split, PV, emit.  `sm` is the op scratch (queries, scores and
// reduction space at the KVM_AS_OFF_* offsets), Ks / Vs the staged tiles [nk][hd] bf16 wherever the caller keeps them;
// waitK() / waitV() block until the respective tile has landed and return false if the wait ran out.  Whole compute group;
// returns false if a wait ran out (the results are then not meaningful, the caller records the timeout).
template <int GT, class Pro, class WaitK, class WaitV, class Emit>
static __device__ bool kvm_attn_part_core(unsigned char* sm, unsigned char* Ks, unsigned char* Vs, int nk, int newrow, int G, int hd, float sc, Pro prologue, WaitK waitK,
                                   WaitV waitV, Emit emit) {
  const int ncp = hd >> 1, KQ = KVM_NT / ncp;
  const int off_sc = KVM_AS_OFF_SC, off_red = off_sc + ((nk + 3) & ~3) * 32;
  const float* qs = (const float*)(sm + KVM_AS_OFF_QS);
  const float* knew = (const float*)(sm + KVM_AS_OFF_KNEW);
  const float* vnew = (const float*)(sm + KVM_AS_OFF_VNEW);
  float* ml = (float*)(sm + KVM_AS_OFF_ML);                // m[8], l[8]
  float* ps = (float*)(sm + off_sc);
  float* red = (float*)(sm + off_red);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  bool ok = true;
  prologue();                                                      // queries (and the appended key / value) while the copies fly
  kvm_sync();
  if (newrow >= 0) for (int cc = tid; cc < hd; cc += KVM_NT) {     // the copies leave the appended row out: these bytes are the threads' alone
    ((__nv_bfloat16*)Ks)[(size_t)(nk - 1) * hd + cc] = __float2bfloat16_rn(knew[cc]);
    ((__nv_bfloat16*)Vs)[(size_t)(nk - 1) * hd + cc] = __float2bfloat16_rn(vnew[cc]);
  }
  kvm_sync();
  if (!waitK()) ok = false;

  // ---- scores (see kvm_decode_scores): the smallest number of pieces per lane that fits a key into one warp
  {
    const int slots = G * (hd >> 3);
    if (slots <= 32) kvm_decode_scores<1>(Ks, qs, ps, nk, G, hd, sc);
    else if (slots <= 64) kvm_decode_scores<2>(Ks, qs, ps, nk, G, hd, sc);
    else kvm_decode_scores<4>(Ks, qs, ps, nk, G, hd, sc);
  }
  kvm_sync();
  // ---- softmax over the split: 16/G warps per query head, each a quarter (or so) of the keys; p = exp(s - m) replaces s
  {
    const int wpg = KVM_NWARPS / G, g = warp % G, part = warp / G;
    float m = KVM_ATTN_EMPTY_M_STREAM;
    for (int j = part * 32 + lane; j < nk; j += wpg * 32) m = fmaxf(m, ps[j * 8 + g]);
    m = kvm_warp_max(m);
    if (lane == 0) red[warp] = m;
    kvm_sync();
    m = KVM_ATTN_EMPTY_M_STREAM;
    for (int p2 = 0; p2 < wpg; ++p2) m = fmaxf(m, red[g + G * p2]);
    float l = 0.0f;
    for (int j = part * 32 + lane; j < nk; j += wpg * 32) { const float p = __expf(ps[j * 8 + g] - m); ps[j * 8 + g] = p; l += p; }
    l = kvm_warp_sum(l);
    if (lane == 0) red[KVM_NWARPS + warp] = l;
    kvm_sync();
    if (warp < G && lane == 0) {
      float L = 0.0f;
      for (int p2 = 0; p2 < wpg; ++p2) L += red[KVM_NWARPS + warp + G * p2];
      ml[warp] = m; ml[8 + warp] = L;
    }
  }
  kvm_sync();
  if (!waitV()) ok = false;
  // ---- PV
  {
    const int kq = tid / ncp, c2 = tid % ncp;
    float acc[GT][2];
#pragma unroll
    for (int g = 0; g < GT; ++g) acc[g][0] = acc[g][1] = 0.0f;
#pragma unroll 4
    for (int j = kq; j < nk; j += KQ) {
      const uint32_t vv = *(const uint32_t*)(Vs + (size_t)j * hd * 2 + c2 * 4);
      const float v0 = kvm_bf16lo(vv), v1 = kvm_bf16hi(vv);
      float p[8];
      *(float4*)p = *(const float4*)(ps + j * 8);
      if (GT > 4) *(float4*)(p + 4) = *(const float4*)(ps + j * 8 + 4);
#pragma unroll
      for (int g = 0; g < GT; ++g) { acc[g][0] = fmaf(p[g], v0, acc[g][0]); acc[g][1] = fmaf(p[g], v1, acc[g][1]); }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) if (g < G) *(float2*)(red + ((size_t)kq * G + g) * hd + 2 * c2) = make_float2(acc[g][0], acc[g][1]);
  }
  kvm_sync();
  for (int e = tid; e < G * hd; e += KVM_NT) {
    const int g = e / hd, cc = e % hd;
    float A = 0.0f;
    for (int q = 0; q < KQ; ++q) A += red[((size_t)q * G + g) * hd + cc];
    emit(g, cc, ml[g], ml[8 + g], A);
  }
  return ok;
}
// Scratch bytes the core needs ahead of the tiles for a split of nk keys.
__device__ __forceinline__ int kvm_attn_part_scratch(int nk, int G, int hd) {
  const int KQ = KVM_NT / (hd >> 1);
  return (KVM_AS_OFF_SC + ((nk + 3) & ~3) * 32 + KQ * G * hd * 4 + 127) & ~127;
}

template <int GT, class Pro, class Emit>
static __device__ bool kvm_attn_part_stream_t(const KvmCtx& c, const KvmBuf& kc, const KvmBuf& vc, size_t base, int j0, int j1, int newrow, int G, int hd, float sc,
                                       Pro prologue, Emit emit) {
  const int nk = max(j1 - j0, 0);
  const int off_k = kvm_attn_part_scratch(nk, G, hd);
  const int tile = (nk * hd * 2 + 127) & ~127;
  if (off_k + 2 * tile > c.smem_bytes) return false;
  unsigned char* sm = c.smem;
  const uint32_t barK = kvm_smem_addr(sm), barV = barK + 8;
  unsigned char* Ks = sm + off_k;
  unsigned char* Vs = Ks + tile;
  const int tid = threadIdx.x;
  const int ncopy = newrow >= 0 ? nk - 1 : nk;             // the appended key is the last one of its split
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // earlier plain accesses to this scratch come before the copies
  kvm_sync();
  if (tid == 0) {
    kvm_mbar_init(barK, 1); kvm_mbar_init(barV, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async;" ::: "memory");       // rows appended by earlier tasks were written with plain stores
    const uint32_t bytes = (uint32_t)(ncopy * hd * 2);
    kvm_mbar_expect_tx(barK, bytes);
    if (bytes) kvm_bulk_g2s(kvm_smem_addr(Ks), (const __nv_bfloat16*)kc.p + (base + j0) * kc.ld, bytes, barK);
    kvm_mbar_expect_tx(barV, bytes);
    if (bytes) kvm_bulk_g2s(kvm_smem_addr(Vs), (const __nv_bfloat16*)vc.p + (base + j0) * vc.ld, bytes, barV);
  }
  const bool ok = kvm_attn_part_core<GT>(sm, Ks, Vs, nk, newrow, G, hd, sc, prologue, [&]() { return kvm_mbar_wait_t(barK, 0); }, [&]() { return kvm_mbar_wait_t(barV, 0); }, emit);
  if (!ok) kvm_stream_timeout(c, 135);
  kvm_sync();
  if (tid == 0) { kvm_mbar_inval(barK); kvm_mbar_inval(barV); }
  return true;
}

// Dispatch on the group size; false = not taken (layout, size or dtype outside what the streaming form handles).
template <class Pro, class Emit>
static __device__ bool kvm_attn_part_stream(const KvmCtx& c, const KvmBuf& kc, const KvmBuf& vc, size_t base, int j0, int j1, int newrow, int G, int hd, float sc,
                                     Pro prologue, Emit emit) {
  if (kc.dtype != KVM_BF16 || vc.dtype != KVM_BF16 || kc.ld != hd || vc.ld != hd || !kvm_vec_ok(kc) || !kvm_vec_ok(vc) || G > 8 || (G & (G - 1)) ||
      !(hd == 16 || hd == 32 || hd == 64 || hd == 128)) return false;
  if (G <= 1) return kvm_attn_part_stream_t<1>(c, kc, vc, base, j0, j1, newrow, G, hd, sc, prologue, emit);
  if (G <= 2) return kvm_attn_part_stream_t<2>(c, kc, vc, base, j0, j1, newrow, G, hd, sc, prologue, emit);
  if (G <= 4) return kvm_attn_part_stream_t<4>(c, kc, vc, base, j0, j1, newrow, G, hd, sc, prologue, emit);
  return kvm_attn_part_stream_t<8>(c, kc, vc, base, j0, j1, newrow, G, hd, sc, prologue, emit);
}
