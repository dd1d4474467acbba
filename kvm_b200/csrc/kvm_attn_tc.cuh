// Causal attention forward / backward on tcgen05 for bf16 storage with head dimension 64: 128 query (or key) rows per task
// as the op contract says (runtime/ref_gpt.py:14,279-364), 128-wide blocks of the other sequence axis streamed by TMA.
//   forward   S = Q K^T (M128 N128 K64) -> TMEM; softmax by all 16 warps straight from TMEM (thread = one row x 32 columns,
//             row maxima combined through shared memory), P written as bf16 into a swizzled K-major tile, O_blk = P V
//             (M128 N64 K128, V consumed MN-major from the tile TMA delivered) -> TMEM, accumulated in registers with the
//             online-softmax rescale; lse = m + log(l) in natural log.
//   dq        per key block: S, dP = dO V^T -> TMEM; dS = P (dP - delta) -> bf16 tile; dQ += dS K accumulates in TMEM.
//   dk, dv    per query block (and head of the GQA group): S^T = K Q^T, dP^T = V dO^T -> TMEM; P^T, dS^T -> bf16 tiles;
//             dV += P^T dO, dK += dS^T Q accumulate in TMEM.
// The same shared-memory tile serves as a K-major operand (contraction over the head dimension) and as an MN-major operand
// (contraction over the sequence axis): only the descriptor differs.  Replaces the mma.sync kernels of
// include/mvm_attn_bf16.cuh:1-12.  Waits are bounded as in kvm_gemm_tc.cuh.
#pragma once
#include "kvm_gemm_tc.cuh"

#define KVM_ATT_NBAR 12

__device__ __forceinline__ float kvm_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ void kvm_att_init(int* ctl) {      // thread 32 at kernel start
  for (int i = 0; i < KVM_ATT_NBAR; ++i) { kvm_mbar_init(kvm_bar_addr(ctl, KVM_CTL_ABAR + i), 1); ctl[KVM_CTL_ACNT + i] = 0; }
}
// 32 consecutive values of row r, logical columns [k0, k0+32) of a [128 x 128] bf16 tile stored K-major as two 64-column chunks
// of 128 rows x 128 bytes with the 128-byte swizzle (16-byte unit u of row r lives at unit u ^ (r & 7)).
__device__ __forceinline__ void kvm_store_tile_row32(unsigned char* tile, int r, int k0, const float (&v)[32]) {
  unsigned char* rowp = tile + (k0 >> 6) * 16384 + r * 128;
  const int u0 = (k0 & 63) >> 3;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    uint4 w;
    __nv_bfloat162* hh = (__nv_bfloat162*)&w;
#pragma unroll
    for (int j = 0; j < 4; ++j) hh[j] = __floats2bfloat162_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
    *(uint4*)(rowp + (((u0 + u) ^ (r & 7)) << 4)) = w;
  }
}
// 16 consecutive values of row r, logical columns [k0, k0+16), same tile layout.
__device__ __forceinline__ void kvm_store_tile_row16(unsigned char* tile, int r, int k0, const float (&v)[16]) {
  unsigned char* rowp = tile + (k0 >> 6) * 16384 + r * 128;
  const int u0 = (k0 & 63) >> 3;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    uint4 w;
    __nv_bfloat162* hh = (__nv_bfloat162*)&w;
#pragma unroll
    for (int j = 0; j < 4; ++j) hh[j] = __floats2bfloat162_rn(v[u * 8 + 2 * j], v[u * 8 + 2 * j + 1]);
    *(uint4*)(rowp + (((u0 + u) ^ (r & 7)) << 4)) = w;
  }
}
__device__ __forceinline__ void kvm_att_fail(const KvmCtx& c, int where) {
  if (atomicCAS(&c.err->code, 0, KVM_ERR_TIMEOUT) == 0) { c.err->task = c.task; c.err->a = where; c.err->b = (int)threadIdx.x; }
}
// S-type product: D[128 x 128] = A[128 x 64] B[128 x 64]^T, both K-major tiles of 128 rows x 128 bytes.
__device__ __forceinline__ void kvm_att_mma_qk(uint32_t tmem_d, uint32_t sa, uint32_t sb) {
  const uint32_t idesc = kvm_idesc_bf16(128, 128, false, false);
#pragma unroll
  for (int j = 0; j < 4; ++j) kvm_tc_mma_bf16(tmem_d, kvm_smem_desc(sa + j * 32, 16, 1024), kvm_smem_desc(sb + j * 32, 16, 1024), idesc, j ? 1u : 0u);
}
// PV-type product: D[128 x 64] (+)= A[128 x 128] B[128 x 64], A a K-major two-chunk tile, B an MN-major tile (128 k-rows x 128 bytes).
__device__ __forceinline__ void kvm_att_mma_pv(uint32_t tmem_d, uint32_t sa, uint32_t sb, bool accumulate) {
  const uint32_t idesc = kvm_idesc_bf16(128, 64, false, true);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    kvm_tc_mma_bf16(tmem_d, kvm_smem_desc(sa + (j >> 2) * 16384 + (j & 3) * 32, 16, 1024), kvm_smem_desc(sb + j * 2048, 8192, 1024), idesc, (accumulate || j) ? 1u : 0u);
}

#define KVM_LOG2E 1.4426950408889634f
#define KVM_LN2 0.6931471805599453f

// aux: x = 2 (tensor-core attention), y / z / w = tensor-map indices of q / k / v (box 64 x 128 over [rows, H*hd]).
KVM_OP_FN void kvm_attn_fwd_tc(const KvmCtx& c, const int32_t* a, const int4& aux) {
  KvmBuf o, lse;
  if (!kvm_buf(c, a[3], KVM_M_FLT, o) || !kvm_buf(c, a[4], KVM_M_F32, lse)) return;
  const int b = a[5], h = a[6], q0 = a[7], T = a[8], H = a[9], Hkv = a[10];
  const float sc2 = kvm_bits_f32(a[12]) * KVM_LOG2E;
  const int kvh = h / (H / Hkv), nb = q0 / 128 + 1;
  int* ctl = c.ctl;
  int* cnt = ctl + KVM_CTL_ACNT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, qd = warp & 3, cg = warp >> 2, row = qd * 32 + lane;
  const uint32_t s0 = kvm_smem_addr(c.smem), sQ = s0, sP = s0 + 81920;
  unsigned char* Pt = c.smem + 81920;
  float* red = (float*)(c.smem + 114688);          // [4][128] row maxima, then [4][128] row sums
  const char* tmQ = (const char*)c.tmaps + (size_t)aux.y * 128;
  const char* tmK = (const char*)c.tmaps + (size_t)aux.z * 128;
  const char* tmV = (const char*)c.tmaps + (size_t)aux.w * 128;
  enum { BQ = 0, BKV = 1, BE = 3, BS = 5, BO = 6 };
  auto bar = [&](int i) { return kvm_bar_addr(ctl, KVM_CTL_ABAR + i); };
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
  const int cQ = cnt[BQ], cKV0 = cnt[BKV], cKV1 = cnt[BKV + 1], cE0 = cnt[BE], cE1 = cnt[BE + 1], cS = cnt[BS], cO = cnt[BO];
  bool ok = true;
  if (tid == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");
    kvm_mbar_expect_tx(bar(BQ), 16384);
    kvm_tma_load_2d(sQ, tmQ, h * 64, b * T + q0, bar(BQ));
    for (int j = 0; j < min(nb, 2); ++j) {
      kvm_mbar_expect_tx(bar(BKV + j), 32768);
      kvm_tma_load_2d(s0 + 16384 + j * 32768, tmK, kvh * 64, b * T + j * 128, bar(BKV + j));
      kvm_tma_load_2d(s0 + 32768 + j * 32768, tmV, kvh * 64, b * T + j * 128, bar(BKV + j));
    }
  }
  if (tid == 32) {
    ok = kvm_mbar_wait(bar(BQ), cQ & 1) && kvm_mbar_wait(bar(BKV), cKV0 & 1);
    kvm_tc_fence_after();
    kvm_att_mma_qk(tmem, sQ, s0 + 16384);
    kvm_tc_commit(bar(BS));
  }
  float m_run = -INFINITY, l_part = 0.0f, oacc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) oacc[i] = 0.0f;
  for (int j = 0; j < nb; ++j) {
    __syncwarp();
    if (!kvm_mbar_wait(bar(BS), (cS + j) & 1)) ok = false;
    kvm_tc_fence_after();
    float s[32];
    kvm_tmem_ld32(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(cg * 32), s);
    float mloc = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      s[i] *= sc2;
      if (j == nb - 1 && cg * 32 + i > row) s[i] = -INFINITY;      // diagonal block: key index beyond the query
      mloc = fmaxf(mloc, s[i]);
    }
    red[cg * 128 + row] = mloc;
    kvm_sync();
    const float m_new = fmaxf(m_run, fmaxf(fmaxf(red[row], red[128 + row]), fmaxf(red[256 + row], red[384 + row])));
    const float alpha = kvm_ex2(m_run - m_new);
    float psum = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { s[i] = kvm_ex2(s[i] - m_new); psum += s[i]; }
    l_part = l_part * alpha + psum;
    kvm_store_tile_row32(Pt, row, cg * 32, s);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    kvm_tc_fence_before();
    kvm_sync();
    if (tid == 32) {
      kvm_tc_fence_after();
      kvm_att_mma_pv(tmem + 128, sP, s0 + 32768 + (j & 1) * 32768, false);
      kvm_tc_commit(bar(BE + (j & 1)));
      kvm_tc_commit(bar(BO));
      if (j + 1 < nb) {
        const int st = (j + 1) & 1;
        if (!kvm_mbar_wait(bar(BKV + st), ((st ? cKV1 : cKV0) + (j + 1) / 2) & 1)) ok = false;
        kvm_tc_fence_after();
        kvm_att_mma_qk(tmem, sQ, s0 + 16384 + st * 32768);
        kvm_tc_commit(bar(BS));
      }
    }
    if (tid == 0 && j + 2 < nb) {
      const int st = j & 1;
      if (!kvm_mbar_wait(bar(BE + st), ((st ? cE1 : cE0) + j / 2) & 1)) ok = false;
      kvm_mbar_expect_tx(bar(BKV + st), 32768);
      kvm_tma_load_2d(s0 + 16384 + st * 32768, tmK, kvh * 64, b * T + (j + 2) * 128, bar(BKV + st));
      kvm_tma_load_2d(s0 + 32768 + st * 32768, tmV, kvh * 64, b * T + (j + 2) * 128, bar(BKV + st));
    }
    __syncwarp();
    if (!kvm_mbar_wait(bar(BO), (cO + j) & 1)) ok = false;
    kvm_tc_fence_after();
    float t[16];
    kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(128 + cg * 16), t);
#pragma unroll
    for (int i = 0; i < 16; ++i) oacc[i] = oacc[i] * alpha + t[i];
    m_run = m_new;
    kvm_tc_fence_before();
  }
  if (!ok) kvm_att_fail(c, 45);
  red[512 + cg * 128 + row] = l_part;
  kvm_sync();
  const float l = red[512 + row] + red[640 + row] + red[768 + row] + red[896 + row], inv = 1.0f / l;
  const size_t orow = (size_t)(b * T + q0 + row) * o.ld + h * 64 + cg * 16;
  if (ok) {
    float v0[8], v1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { v0[i] = oacc[i] * inv; v1[i] = oacc[8 + i] * inv; }
    if ((o.ld & 7) == 0 && kvm_vec_ok(o)) { kvm_st8(o, orow, v0); kvm_st8(o, orow + 8, v1); }
    else for (int i = 0; i < 16; ++i) kvm_st(o, orow + i, oacc[i] * inv);
    if (cg == 0) ((float*)lse.p)[(size_t)(b * H + h) * T + q0 + row] = (m_run + log2f(l)) * KVM_LN2;
  }
  kvm_tc_fence_before();
  kvm_sync();
  if (tid == 0) {
    cnt[BQ] = cQ + 1; cnt[BKV] = cKV0 + (nb + 1) / 2; cnt[BKV + 1] = cKV1 + nb / 2; cnt[BE] = cE0 + (nb + 1) / 2; cnt[BE + 1] = cE1 + nb / 2;
    cnt[BS] = cS + nb; cnt[BO] = cO + nb;
  }
}

// dq for 128 query rows.  aux.y/z/w = maps of q / k / v; the dO map index travels in the high half of aux.x (aux.x = 2 | idx << 8).
// Shared memory: Q 16K, dO 16K, two stages of (K 16K, V 16K), dS tile 32K.  TMEM: S cols 0..127, dP 128..255, dQ 256..319.
KVM_OP_FN void kvm_attn_dq_tc(const KvmCtx& c, const int32_t* a, const int4& aux) {
  KvmBuf lse, delta, dq;
  if (!kvm_buf(c, a[4], KVM_M_F32, lse) || !kvm_buf(c, a[5], KVM_M_F32, delta) || !kvm_buf(c, a[6], KVM_M_FLT, dq)) return;
  const int b = a[7], h = a[8], q0 = a[9], T = a[10], H = a[11], Hkv = a[12];
  const float sc = kvm_bits_f32(a[14]), sc2 = sc * KVM_LOG2E;
  const int kvh = h / (H / Hkv), nb = q0 / 128 + 1;
  int* ctl = c.ctl;
  int* cnt = ctl + KVM_CTL_ACNT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, qd = warp & 3, cg = warp >> 2, row = qd * 32 + lane;
  const uint32_t s0 = kvm_smem_addr(c.smem), sQ = s0, sDO = s0 + 16384, sKV = s0 + 32768, sDS = s0 + 98304;
  unsigned char* DSt = c.smem + 98304;
  const char* tmQ = (const char*)c.tmaps + (size_t)aux.y * 128;
  const char* tmK = (const char*)c.tmaps + (size_t)aux.z * 128;
  const char* tmV = (const char*)c.tmaps + (size_t)aux.w * 128;
  const char* tmDO = (const char*)c.tmaps + (size_t)(aux.x >> 8) * 128;
  enum { BQ = 0, BKV = 1, BE = 3, BS = 5, BO = 6 };
  auto bar = [&](int i) { return kvm_bar_addr(ctl, KVM_CTL_ABAR + i); };
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
  const int cQ = cnt[BQ], cKV0 = cnt[BKV], cKV1 = cnt[BKV + 1], cE0 = cnt[BE], cE1 = cnt[BE + 1], cS = cnt[BS], cO = cnt[BO];
  bool ok = true;
  if (tid == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");
    kvm_mbar_expect_tx(bar(BQ), 32768);
    kvm_tma_load_2d(sQ, tmQ, h * 64, b * T + q0, bar(BQ));
    kvm_tma_load_2d(sDO, tmDO, h * 64, b * T + q0, bar(BQ));
    for (int j = 0; j < min(nb, 2); ++j) {
      kvm_mbar_expect_tx(bar(BKV + j), 32768);
      kvm_tma_load_2d(sKV + j * 32768, tmK, kvh * 64, b * T + j * 128, bar(BKV + j));
      kvm_tma_load_2d(sKV + 16384 + j * 32768, tmV, kvh * 64, b * T + j * 128, bar(BKV + j));
    }
  }
  if (tid == 32) {
    ok = kvm_mbar_wait(bar(BQ), cQ & 1) && kvm_mbar_wait(bar(BKV), cKV0 & 1);
    kvm_tc_fence_after();
    kvm_att_mma_qk(tmem, sQ, sKV);
    kvm_att_mma_qk(tmem + 128, sDO, sKV + 16384);
    kvm_tc_commit(bar(BS));
  }
  const size_t vrow = (size_t)(b * H + h) * T + q0 + row;
  const float li2 = ((const float*)lse.p)[vrow] * KVM_LOG2E, di = ((const float*)delta.p)[vrow];
  for (int j = 0; j < nb; ++j) {
    __syncwarp();
    if (!kvm_mbar_wait(bar(BS), (cS + j) & 1)) ok = false;
    kvm_tc_fence_after();
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {        // two halves of 16 columns: half the live registers
      float s[16], dp[16];
      const int c0 = cg * 32 + hf * 16;
      kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)c0, s);
      kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(128 + c0), dp);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p = (j == nb - 1 && c0 + i > row) ? 0.0f : kvm_ex2(s[i] * sc2 - li2);
        s[i] = p * (dp[i] - di);
      }
      kvm_store_tile_row16(DSt, row, c0, s);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    kvm_tc_fence_before();
    kvm_sync();
    if (tid == 32) {
      kvm_tc_fence_after();
      kvm_att_mma_pv(tmem + 256, sDS, sKV + (j & 1) * 32768, j > 0);        // dQ += dS K_j (K tile read MN-major)
      kvm_tc_commit(bar(BE + (j & 1)));
      if (j + 1 < nb) {
        const int st = (j + 1) & 1;
        if (!kvm_mbar_wait(bar(BKV + st), ((st ? cKV1 : cKV0) + (j + 1) / 2) & 1)) ok = false;
        kvm_tc_fence_after();
        kvm_att_mma_qk(tmem, sQ, sKV + st * 32768);
        kvm_att_mma_qk(tmem + 128, sDO, sKV + 16384 + st * 32768);
        kvm_tc_commit(bar(BS));
      } else kvm_tc_commit(bar(BO));
    }
    if (tid == 0 && j + 2 < nb) {
      const int st = j & 1;
      if (!kvm_mbar_wait(bar(BE + st), ((st ? cE1 : cE0) + j / 2) & 1)) ok = false;
      kvm_mbar_expect_tx(bar(BKV + st), 32768);
      kvm_tma_load_2d(sKV + st * 32768, tmK, kvh * 64, b * T + (j + 2) * 128, bar(BKV + st));
      kvm_tma_load_2d(sKV + 16384 + st * 32768, tmV, kvh * 64, b * T + (j + 2) * 128, bar(BKV + st));
    }
    kvm_tc_fence_before();
  }
  __syncwarp();
  if (!kvm_mbar_wait(bar(BO), cO & 1)) ok = false;
  kvm_tc_fence_after();
  if (!ok) kvm_att_fail(c, 47);
  float t[16];
  kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(256 + cg * 16), t);
  if (ok) {
    const size_t orow = (size_t)(b * T + q0 + row) * dq.ld + h * 64 + cg * 16;
    float v0[8], v1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { v0[i] = t[i] * sc; v1[i] = t[8 + i] * sc; }
    if ((dq.ld & 7) == 0 && kvm_vec_ok(dq)) { kvm_st8(dq, orow, v0); kvm_st8(dq, orow + 8, v1); }
    else for (int i = 0; i < 16; ++i) kvm_st(dq, orow + i, t[i] * sc);
  }
  kvm_tc_fence_before();
  kvm_sync();
  if (tid == 0) {
    cnt[BQ] = cQ + 1; cnt[BKV] = cKV0 + (nb + 1) / 2; cnt[BKV + 1] = cKV1 + nb / 2; cnt[BE] = cE0 + (nb + 1) / 2; cnt[BE + 1] = cE1 + nb / 2;
    cnt[BS] = cS + nb; cnt[BO] = cO + 1;
  }
}

// dk, dv for 128 key rows of kv head kvh: loops over the heads of the GQA group and the query blocks at or after the key block.
// Shared memory: K 16K, V 16K, two stages of (Q 16K, dO 16K), P^T tile 32K, dS^T tile 32K, lse / delta of the block 1K.
// TMEM: S^T cols 0..127, dP^T 128..255, dV 256..319, dK 320..383.
KVM_OP_FN void kvm_attn_dkv_tc(const KvmCtx& c, const int32_t* a, const int4& aux) {
  KvmBuf lse, delta, dk, dv, kb;
  if (!kvm_buf(c, a[1], KVM_M_FLT, kb) || !kvm_buf(c, a[4], KVM_M_F32, lse) || !kvm_buf(c, a[5], KVM_M_F32, delta) || !kvm_buf(c, a[6], KVM_M_FLT, dk) ||
      !kvm_buf(c, a[7], KVM_M_FLT, dv)) return;
  const int b = a[8], kvh = a[9], k0 = a[10], T = a[11], H = a[12];
  const float sc = kvm_bits_f32(a[14]), sc2 = sc * KVM_LOG2E;
  const int Hkv = kb.cols / 64, G = H / Hkv, kblk = k0 / 128, nqb = T / 128 - kblk, nit = G * nqb;
  int* ctl = c.ctl;
  int* cnt = ctl + KVM_CTL_ACNT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, qd = warp & 3, cg = warp >> 2, row = qd * 32 + lane;
  const uint32_t s0 = kvm_smem_addr(c.smem), sK = s0, sV = s0 + 16384, sQD = s0 + 32768, sPT = s0 + 98304, sDST = s0 + 131072;
  unsigned char* PTt = c.smem + 98304;
  unsigned char* DSTt = c.smem + 131072;
  float* vec = (float*)(c.smem + 163840);            // [2 stages][lse2 128 | delta 128]
  const char* tmQ = (const char*)c.tmaps + (size_t)aux.y * 128;
  const char* tmK = (const char*)c.tmaps + (size_t)aux.z * 128;
  const char* tmV = (const char*)c.tmaps + (size_t)aux.w * 128;
  const char* tmDO = (const char*)c.tmaps + (size_t)(aux.x >> 8) * 128;
  enum { BQ = 0, BKV = 1, BE = 3, BS = 5, BO = 6 };
  auto bar = [&](int i) { return kvm_bar_addr(ctl, KVM_CTL_ABAR + i); };
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
  const int cQ = cnt[BQ], cKV0 = cnt[BKV], cKV1 = cnt[BKV + 1], cE0 = cnt[BE], cE1 = cnt[BE + 1], cS = cnt[BS], cO = cnt[BO];
  bool ok = true;
  auto coords = [&](int it, int& hh, int& qrow) { hh = kvh * G + it / nqb; qrow = b * T + (kblk + it % nqb) * 128; };
  if (tid == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");
    kvm_mbar_expect_tx(bar(BQ), 32768);
    kvm_tma_load_2d(sK, tmK, kvh * 64, b * T + k0, bar(BQ));
    kvm_tma_load_2d(sV, tmV, kvh * 64, b * T + k0, bar(BQ));
    for (int it = 0; it < min(nit, 2); ++it) {
      int hh, qrow; coords(it, hh, qrow);
      kvm_mbar_expect_tx(bar(BKV + it), 32768);
      kvm_tma_load_2d(sQD + it * 32768, tmQ, hh * 64, qrow, bar(BKV + it));
      kvm_tma_load_2d(sQD + 16384 + it * 32768, tmDO, hh * 64, qrow, bar(BKV + it));
    }
  }
  if (tid == 32) {
    ok = kvm_mbar_wait(bar(BQ), cQ & 1) && kvm_mbar_wait(bar(BKV), cKV0 & 1);
    kvm_tc_fence_after();
    kvm_att_mma_qk(tmem, sK, sQD);                   // S^T = K Q^T
    kvm_att_mma_qk(tmem + 128, sV, sQD + 16384);      // dP^T = V dO^T
    kvm_tc_commit(bar(BS));
  }
  for (int it = 0; it < nit; ++it) {
    int hh, qrow; coords(it, hh, qrow);
    const bool diag = (it % nqb) == 0;
    float* vv = vec + (it & 1) * 256;
    if (tid < 128) {
      const size_t vi = (size_t)(b * H + hh) * T + (qrow - b * T) + tid;
      vv[tid] = ((const float*)lse.p)[vi] * KVM_LOG2E; vv[128 + tid] = ((const float*)delta.p)[vi];
    }
    kvm_sync();
    __syncwarp();
    if (!kvm_mbar_wait(bar(BS), (cS + it) & 1)) ok = false;
    kvm_tc_fence_after();
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {        // two halves of 16 columns: half the live registers
      float s[16], dp[16];
      const int c0 = cg * 32 + hf * 16;
      kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)c0, s);
      kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(128 + c0), dp);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int qi = c0 + i;                       // query index inside the block (column); row = key index inside the block
        const float p = (diag && qi < row) ? 0.0f : kvm_ex2(s[i] * sc2 - vv[qi]);
        s[i] = p;
        dp[i] = p * (dp[i] - vv[128 + qi]);
      }
      kvm_store_tile_row16(PTt, row, c0, s);
      kvm_store_tile_row16(DSTt, row, c0, dp);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    kvm_tc_fence_before();
    kvm_sync();
    if (tid == 32) {
      kvm_tc_fence_after();
      const uint32_t st_ = sQD + (it & 1) * 32768;
      kvm_att_mma_pv(tmem + 256, sPT, st_ + 16384, it > 0);       // dV += P^T dO  (dO tile read MN-major)
      kvm_att_mma_pv(tmem + 320, sDST, st_, it > 0);              // dK += dS^T Q  (Q tile read MN-major)
      kvm_tc_commit(bar(BE + (it & 1)));
      if (it + 1 < nit) {
        const int st = (it + 1) & 1;
        if (!kvm_mbar_wait(bar(BKV + st), ((st ? cKV1 : cKV0) + (it + 1) / 2) & 1)) ok = false;
        kvm_tc_fence_after();
        kvm_att_mma_qk(tmem, sK, sQD + st * 32768);
        kvm_att_mma_qk(tmem + 128, sV, sQD + 16384 + st * 32768);
        kvm_tc_commit(bar(BS));
      } else kvm_tc_commit(bar(BO));
    }
    if (tid == 0 && it + 2 < nit) {
      const int st = it & 1;
      int h2, qr2; coords(it + 2, h2, qr2);
      if (!kvm_mbar_wait(bar(BE + st), ((st ? cE1 : cE0) + it / 2) & 1)) ok = false;
      kvm_mbar_expect_tx(bar(BKV + st), 32768);
      kvm_tma_load_2d(sQD + st * 32768, tmQ, h2 * 64, qr2, bar(BKV + st));
      kvm_tma_load_2d(sQD + 16384 + st * 32768, tmDO, h2 * 64, qr2, bar(BKV + st));
    }
    kvm_tc_fence_before();
  }
  __syncwarp();
  if (!kvm_mbar_wait(bar(BO), cO & 1)) ok = false;
  kvm_tc_fence_after();
  if (!ok) kvm_att_fail(c, 48);
  float tv[16], tk[16];
  kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(256 + cg * 16), tv);
  kvm_tmem_ld16(tmem + ((uint32_t)(qd * 32) << 16) + (uint32_t)(320 + cg * 16), tk);
  if (ok) {
    const size_t kr = (size_t)(b * T + k0 + row) * dk.ld + kvh * 64 + cg * 16, vr = (size_t)(b * T + k0 + row) * dv.ld + kvh * 64 + cg * 16;
#pragma unroll
    for (int i = 0; i < 16; ++i) tk[i] *= sc;
    if ((dk.ld & 7) == 0 && (dv.ld & 7) == 0 && kvm_vec_ok(dk) && kvm_vec_ok(dv)) {
      float a0[8], a1[8], b0[8], b1[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { a0[i] = tk[i]; a1[i] = tk[8 + i]; b0[i] = tv[i]; b1[i] = tv[8 + i]; }
      kvm_st8(dk, kr, a0); kvm_st8(dk, kr + 8, a1); kvm_st8(dv, vr, b0); kvm_st8(dv, vr + 8, b1);
    } else for (int i = 0; i < 16; ++i) { kvm_st(dk, kr + i, tk[i]); kvm_st(dv, vr + i, tv[i]); }
  }
  kvm_tc_fence_before();
  kvm_sync();
  if (tid == 0) {
    cnt[BQ] = cQ + 1; cnt[BKV] = cKV0 + (nit + 1) / 2; cnt[BKV + 1] = cKV1 + nit / 2; cnt[BE] = cE0 + (nit + 1) / 2; cnt[BE + 1] = cE1 + nit / 2;
    cnt[BS] = cS + nit; cnt[BO] = cO + 1;
  }
}
