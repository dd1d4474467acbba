// bf16 GEMM tile on the 5th-generation tensor cores: 128 x 256 output tile per task (matmul_mma_bf16, op 122), operands
// staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a 4-stage shared-memory ring, products issued by one
// elected thread as tcgen05.mma (kind::f16, M128 N256 K16) into a float32 accumulator in TMEM, epilogue read back with
// tcgen05.ld by all 16 compute warps (bias, GELU, pre, residual, accumulate; f32 or bf16 stores).
//
// Operand layouts (flags 1 / 2 of the op = transposed A / B):
//   A [M,K] row-major        K-major   one TMA box 64(k) x 128(m)  -> 128 rows of 128 B, 8-row swizzle atoms, SBO 1024 B
//   A [K,M] row-major        MN-major  two boxes 64(m) x 64(k)     -> per box 64 k-rows of 128 B; LBO 8192 B, SBO 1024 B
//   B [N,K] row-major (tb)   K-major   one box 64(k) x 256(n)
//   B [K,N] row-major        MN-major  four boxes 64(n) x 64(k)
// Reference being replaced: the mma.sync m16n8k16 tile of include/mvm_mma_bf16.cuh:1-17 with the epilogue of
// include/mvm_ops_gpt.cuh:1435-1491; numerics contract runtime/ref_extra.py:312-331 (bf16 operands, float32 accumulation,
// one rounding per stored bf16 value).  Accumulation order differs from the k-ascending CPU model (tensor-core tree),
// which the reference allows for its own device path too.
//
// Every mbarrier wait is bounded: on expiry the task records KVM_ERR_TIMEOUT and falls through, so the kernel always ends.
#pragma once
#include "kvm_dev.cuh"
#include "kvm_ops_mm.cuh"

#define KVM_TC_STAGES 4
#define KVM_TC_BK 64
#define KVM_TC_A_BYTES (128 * 128)
#define KVM_TC_B_BYTES (256 * 128)
#define KVM_TC_STAGE_BYTES (KVM_TC_A_BYTES + KVM_TC_B_BYTES)
#define KVM_TC_SMEM (KVM_TC_STAGES * KVM_TC_STAGE_BYTES)
#define KVM_TC_SPIN_LIMIT (1u << 26)

// control words in the executor's shared-memory header (int index into ctl[])
#define KVM_CTL_TMEM 0
#define KVM_CTL_PROD_IT 1
#define KVM_CTL_MMA_IT 2
#define KVM_CTL_ACC_PH 3
#define KVM_CTL_YIELD 5          // ready-queue kernel: set by a task that wants to be put back into the queue instead of finished
#define KVM_CTL_BAR 8          // 8-byte aligned: full[4], empty[4], acc_full at ctl[8 + 2*i]
#define KVM_CTL_ABAR 9          // second barrier set (attention, paired GEMM tiles): indices 9.. in the ctl barrier array
#define KVM_CTL_ACNT 64         // completed-phase counts of the second set (ints)

__device__ __forceinline__ uint32_t kvm_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t kvm_bar_addr(int* ctl, int i) { return kvm_smem_addr(ctl + KVM_CTL_BAR + 2 * i); }

__device__ __forceinline__ void kvm_mbar_init(uint32_t bar, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void kvm_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait on phase parity. Returns false if the limit ran out.
__device__ __forceinline__ bool kvm_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < KVM_TC_SPIN_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void kvm_tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void kvm_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void kvm_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void kvm_tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void kvm_tc_mma_bf16(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc),
               "r"(accumulate)
               : "memory");
}
// 32 lanes x 32 consecutive columns of 32-bit words: thread (lane) gets its TMEM lane's columns [col, col+32).
__device__ __forceinline__ void kvm_tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = (uint32_t*)v;
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, "
      "%27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
        "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void kvm_tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = (uint32_t*)v;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                 "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (SM100 format): start address, leading / stride byte offsets in 16-byte units,
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t kvm_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: f32 accumulator, bf16 A and B, majorness bits, N >> 3, M >> 4.
__device__ __forceinline__ uint32_t kvm_idesc_bf16(int M, int N, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Whole CTA, once at kernel start: TMEM allocation (all 512 columns: one CTA per SM) and mbarrier initialisation.
__device__ __forceinline__ void kvm_att_init(int* ctl);
__device__ __forceinline__ void kvm_tc_init(int* ctl, unsigned char* smem) {
  (void)smem;
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(kvm_smem_addr(ctl + KVM_CTL_TMEM)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (threadIdx.x == 32) {
    for (int i = 0; i < 2 * KVM_TC_STAGES + 1; ++i) kvm_mbar_init(kvm_bar_addr(ctl, i), 1);
    for (int i = 21; i < 25; ++i) kvm_mbar_init(kvm_bar_addr(ctl, i), 1);          // accumulator full / empty of the overlapped pipeline
    ctl[KVM_CTL_PROD_IT] = 0; ctl[KVM_CTL_MMA_IT] = 0; ctl[KVM_CTL_ACC_PH] = 0;
    kvm_att_init(ctl);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  kvm_tc_fence_before();
}
__device__ __forceinline__ void kvm_tc_fini(int* ctl) {
  kvm_tc_fence_after();
  if (threadIdx.x < 32) {
    const uint32_t base = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(512) : "memory");
  }
}

// Vector epilogue of one thread: 32 consecutive columns [n, n+32) of row m. Falls back to scalar stores at the ragged edge.
__device__ __forceinline__ void kvm_tc_store32(const KvmMmArgs& g, const float (&acc)[32], int m, int n) {
  const int nvalid = min(32, g.N - n);
  if (nvalid <= 0) return;
  const bool simple = !(g.flags & 512);
  const bool vec = nvalid == 32 && (n & 7) == 0 && (g.out.ld & 7) == 0 && kvm_vec_ok(g.out) && (!g.res.p || ((g.res.ld & 7) == 0 && kvm_vec_ok(g.res))) &&
                   (!g.pre.p || ((g.pre.ld & 7) == 0 && kvm_vec_ok(g.pre))) && simple;
  if (!vec) {
    for (int j = 0; j < nvalid; ++j) kvm_st(g.out, (size_t)m * g.out.ld + n + j, kvm_mm_epilogue(g, acc[j], m, n + j));
    return;
  }
  const float* bias = (const float*)g.bias.p;
#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += 8) {
    float v[8], t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = acc[j0 + j] * g.alpha; if (bias) v[j] += bias[n + j0 + j]; }
    if (g.pre.p) kvm_st8(g.pre, (size_t)m * g.pre.ld + n + j0, v);
    if (g.flags & 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = kvm_gelu(v[j]);
    }
    if (g.res.p) { kvm_ld8(g.res, (size_t)m * g.res.ld + n + j0, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += t[j]; }
    if (g.flags & 4) { kvm_ld8(g.out, (size_t)m * g.out.ld + n + j0, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += t[j]; }
    kvm_st8(g.out, (size_t)m * g.out.ld + n + j0, v);
  }
}

// Epilogue of one 128 x 256 accumulator through shared memory, so that every global access is a whole contiguous row segment:
//   phase 1  warp (q = w & 3, cg = w >> 2) reads TMEM lanes 32q.. / columns 64cg.. and parks the raw float32 sums in a staging tile
//            (row pitch 1040 bytes: eight rows of one 16-byte column piece fall into different banks)
//   phase 2  thread = (row, 8 consecutive columns), a warp = one row of 256 columns: scale, bias, pre-activation / GELU, residual,
//            accumulate and the store (f32 or bf16) all touch 512 or 1024 contiguous bytes per warp instruction
// `stage` is the operand ring (free once the accumulator is complete).  Falls back to the element-wise epilogue for geometry the
// vector accesses cannot take.  Whole compute group; ends with the group in step (kvm_sync).
#define KVM_TC_EPI_PITCH 260          // floats per staged row
__device__ __forceinline__ bool kvm_tc_epi_vec_ok(const KvmMmArgs& g) {
  return (g.out.ld & 7) == 0 && kvm_vec_ok(g.out) && (g.n0 & 7) == 0 && (!g.res.p || ((g.res.ld & 7) == 0 && kvm_vec_ok(g.res))) &&
         (!g.pre.p || ((g.pre.ld & 7) == 0 && kvm_vec_ok(g.pre))) && (!g.bias.p || (((uintptr_t)g.bias.p & 15) == 0));
}
static __device__ void kvm_tc_epilogue_staged(const KvmCtx& c, const KvmMmArgs& g, uint32_t tmem_acc, int m_base, bool ok) {
  float* T = (float*)c.smem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = warp & 3, cgi = warp >> 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int col = cgi * 64 + h * 32;
    float acc[32];
    kvm_tmem_ld32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)col, acc);
    float* dst = T + (size_t)(q * 32 + lane) * KVM_TC_EPI_PITCH + col;
#pragma unroll
    for (int j = 0; j < 32; j += 4) *(float4*)(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
  }
  kvm_tc_fence_before();
  kvm_sync();
  if (ok) {
    const bool simple = !(g.flags & 512);
    const float* bias = (const float*)g.bias.p;
    for (int item = threadIdx.x; item < 128 * 32; item += KVM_NT) {
      const int r = item >> 5, cc = (item & 31) * 8, m = m_base + r, n = g.n0 + cc;
      if (m >= g.M || n >= g.N) continue;
      const float* src = T + (size_t)r * KVM_TC_EPI_PITCH + cc;
      float v[8];
      *(float4*)v = *(const float4*)src; *(float4*)(v + 4) = *(const float4*)(src + 4);
      if (n + 8 <= g.N && simple) {
        float t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= g.alpha;
        if (bias) { *(float4*)t = *(const float4*)(bias + n); *(float4*)(t + 4) = *(const float4*)(bias + n + 4);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += t[j]; }
        if (g.pre.p) kvm_st8(g.pre, (size_t)m * g.pre.ld + n, v);
        if (g.flags & 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = kvm_gelu(v[j]);
        }
        if (g.res.p) { kvm_ld8(g.res, (size_t)m * g.res.ld + n, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += t[j]; }
        if (g.flags & 4) { kvm_ld8(g.out, (size_t)m * g.out.ld + n, t);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += t[j]; }
        kvm_st8(g.out, (size_t)m * g.out.ld + n, v);
      } else {
        for (int j = 0; j < 8 && n + j < g.N; ++j) kvm_st(g.out, (size_t)m * g.out.ld + n + j, kvm_mm_epilogue(g, v[j], m, n + j));
      }
    }
  }
  kvm_sync();
}

// Two stacked tiles (rows m0.. and m0+128.., same 256 columns) as one 256 x 256 product: both read the same B stage, so a
// k-block moves 64 KB for two tiles instead of 96 KB, which is what the L2 -> shared-memory path of an SM can feed.
// Three 64 KB stages [A0 16K | A1 16K | B 32K]; two float32 accumulators in TMEM (columns 0..255 and 256..511).
// Barriers: the attention set (full 0..2, empty 3..5, accumulator 6) with their completed-phase counts in ctl[KVM_CTL_ACNT + i].
#define KVM_TCP_STAGES 3
#define KVM_TCP_STAGE_BYTES (2 * KVM_TC_A_BYTES + KVM_TC_B_BYTES)
static __device__ void kvm_mm_tc_pair(const KvmCtx& c, const KvmMmArgs& g, const int4& aux) {
  int* ctl = c.ctl;
  int* cnt = ctl + KVM_CTL_ACNT;
  auto bar = [&](int i) { return kvm_bar_addr(ctl, KVM_CTL_ABAR + i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool ta = g.flags & 1, tb = g.flags & 2;
  const int num_kb = (g.K + KVM_TC_BK - 1) / KVM_TC_BK;
  const uint32_t stage0 = kvm_smem_addr(c.smem);
  const char* tmA = (const char*)c.tmaps + (size_t)aux.y * 128;
  const char* tmB = (const char*)c.tmaps + (size_t)aux.z * 128;
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
  const int cA = cnt[6];
  bool ok = true;
  asm volatile("fence.proxy.async;" ::: "memory");
  if (warp == 0 && lane == 0) {                         // ---- TMA producer
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % KVM_TCP_STAGES, u = kb / KVM_TCP_STAGES;
      if (u > 0 && !kvm_mbar_wait(bar(3 + s), (uint32_t)(cnt[3 + s] + u - 1) & 1)) { ok = false; break; }
      const uint32_t full = bar(s), sa = stage0 + s * KVM_TCP_STAGE_BYTES, sb = sa + 2 * KVM_TC_A_BYTES;
      kvm_mbar_expect_tx(full, KVM_TCP_STAGE_BYTES);
      const int k0 = kb * KVM_TC_BK;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int m0 = g.m0 + t * 128;
        const uint32_t st = sa + t * KVM_TC_A_BYTES;
        if (!ta) kvm_tma_load_2d(st, tmA, k0, m0, full);
        else { kvm_tma_load_2d(st, tmA, m0, k0, full); kvm_tma_load_2d(st + 8192, tmA, m0 + 64, k0, full); }
      }
      if (tb) kvm_tma_load_2d(sb, tmB, k0, g.n0, full);
      else {
#pragma unroll
        for (int i = 0; i < 4; ++i) kvm_tma_load_2d(sb + i * 8192, tmB, g.n0 + 64 * i, k0, full);
      }
    }
  } else if (warp == 1 && lane == 0) {                  // ---- MMA issuer
    const uint32_t idesc = kvm_idesc_bf16(128, 256, ta, !tb);
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % KVM_TCP_STAGES, u = kb / KVM_TCP_STAGES;
      if (!kvm_mbar_wait(bar(s), (uint32_t)(cnt[s] + u) & 1)) { ok = false; break; }
      kvm_tc_fence_after();
      const uint32_t sa = stage0 + s * KVM_TCP_STAGE_BYTES, sb = sa + 2 * KVM_TC_A_BYTES;
#pragma unroll
      for (int j = 0; j < KVM_TC_BK / 16; ++j) {
        const uint64_t db = tb ? kvm_smem_desc(sb + j * 32, 16, 1024) : kvm_smem_desc(sb + j * 2048, 8192, 1024);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          const uint32_t st = sa + t * KVM_TC_A_BYTES;
          const uint64_t da = ta ? kvm_smem_desc(st + j * 2048, 8192, 1024) : kvm_smem_desc(st + j * 32, 16, 1024);
          kvm_tc_mma_bf16(tmem + t * 256, da, db, idesc, (kb | j) ? 1u : 0u);
        }
      }
      kvm_tc_commit(bar(3 + s));
    }
    kvm_tc_commit(bar(6));
  }
  __syncwarp();
  if (!kvm_mbar_wait(bar(6), (uint32_t)cA & 1)) ok = false;
  kvm_tc_fence_after();
  if (!ok && atomicCAS(&c.err->code, 0, KVM_ERR_TIMEOUT) == 0) { c.err->task = c.task; c.err->a = 1122; c.err->b = (int)threadIdx.x; }
  if (kvm_tc_epi_vec_ok(g)) {
#pragma unroll 1
    for (int t = 0; t < 2; ++t) kvm_tc_epilogue_staged(c, g, tmem + t * 256, g.m0 + t * 128, ok);
  } else {
    const int q = warp & 3, cgi = warp >> 2;
#pragma unroll 1
    for (int t = 0; t < 2; ++t) {
      const int m = g.m0 + t * 128 + q * 32 + lane;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int col = cgi * 64 + h * 32;
        float acc[32];
        kvm_tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * 256 + col), acc);
        if (ok && m < g.M) kvm_tc_store32(g, acc, m, g.n0 + col);
      }
    }
    kvm_tc_fence_before();
    kvm_sync();
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < KVM_TCP_STAGES; ++s) { const int uses = (num_kb - s + KVM_TCP_STAGES - 1) / KVM_TCP_STAGES; cnt[s] += uses; cnt[3 + s] += uses; }
    cnt[6] = cA + 1;
  }
}

static __device__ void kvm_tce_epilogue(const KvmCtx& c, const KvmMmArgs& g);
__device__ __forceinline__ void kvm_mbar_arrive_local(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
// aux.x = 1: tensor-core path planned by the host (aux.y / aux.z = tensor-map indices of A / B); else SIMT fallback.
KVM_OP_FN void kvm_op_matmul_mma_bf16(const KvmCtx& c, const int32_t* a, const int4& aux) {
  KvmMmArgs g;
  if (!kvm_mm_args(c, a, 2, g)) return;
  if (aux.x != 1 || (c.cfg_flags & KVM_CFG_NO_TENSOR_CORES)) { kvm_mm_simt(c, g); return; }
  if (c.engine) { kvm_tce_epilogue(c, g); return; }      // the engine warps run this tile's mainloop (ready-queue kernel)
  if (c.pair >= 0) { g.m0 &= ~255; kvm_mm_tc_pair(c, g, aux); return; }       // this task and its partner: rows m0.. and m0+128..
  int* ctl = c.ctl;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool ta = g.flags & 1, tb = g.flags & 2;
  const int num_kb = (g.K + KVM_TC_BK - 1) / KVM_TC_BK;
  const uint32_t stage0 = kvm_smem_addr(c.smem);       // 1024-byte aligned (the header is 1024 bytes of a 1024-aligned block)
  const char* tmA = (const char*)c.tmaps + (size_t)aux.y * 128;
  const char* tmB = (const char*)c.tmaps + (size_t)aux.z * 128;
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
  bool ok = true;
  asm volatile("fence.proxy.async;" ::: "memory");     // operands written by other tasks' plain stores are read here through TMA

  if (warp == 0 && lane == 0) {                         // ---- TMA producer
    uint32_t it = (uint32_t)ctl[KVM_CTL_PROD_IT];
    for (int kb = 0; kb < num_kb; ++kb, ++it) {
      const int s = it % KVM_TC_STAGES;
      const uint32_t ph = (it / KVM_TC_STAGES) & 1;
      if (!kvm_mbar_wait(kvm_bar_addr(ctl, KVM_TC_STAGES + s), ph ^ 1)) { ok = false; break; }
      const uint32_t full = kvm_bar_addr(ctl, s), sa = stage0 + s * KVM_TC_STAGE_BYTES, sb = sa + KVM_TC_A_BYTES;
      kvm_mbar_expect_tx(full, KVM_TC_STAGE_BYTES);
      const int k0 = kb * KVM_TC_BK;
      if (!ta) kvm_tma_load_2d(sa, tmA, k0, g.m0, full);
      else { kvm_tma_load_2d(sa, tmA, g.m0, k0, full); kvm_tma_load_2d(sa + 8192, tmA, g.m0 + 64, k0, full); }
      if (tb) kvm_tma_load_2d(sb, tmB, k0, g.n0, full);
      else {
#pragma unroll
        for (int i = 0; i < 4; ++i) kvm_tma_load_2d(sb + i * 8192, tmB, g.n0 + 64 * i, k0, full);
      }
    }
    ctl[KVM_CTL_PROD_IT] = (int)it;
  } else if (warp == 1 && lane == 0) {                  // ---- MMA issuer
    uint32_t it = (uint32_t)ctl[KVM_CTL_MMA_IT];
    const uint32_t idesc = kvm_idesc_bf16(128, 256, ta, !tb);
    for (int kb = 0; kb < num_kb; ++kb, ++it) {
      const int s = it % KVM_TC_STAGES;
      const uint32_t ph = (it / KVM_TC_STAGES) & 1;
      if (!kvm_mbar_wait(kvm_bar_addr(ctl, s), ph)) { ok = false; break; }
      kvm_tc_fence_after();
      const uint32_t sa = stage0 + s * KVM_TC_STAGE_BYTES, sb = sa + KVM_TC_A_BYTES;
#pragma unroll
      for (int j = 0; j < KVM_TC_BK / 16; ++j) {
        const uint64_t da = ta ? kvm_smem_desc(sa + j * 2048, 8192, 1024) : kvm_smem_desc(sa + j * 32, 16, 1024);
        const uint64_t db = tb ? kvm_smem_desc(sb + j * 32, 16, 1024) : kvm_smem_desc(sb + j * 2048, 8192, 1024);
        kvm_tc_mma_bf16(tmem, da, db, idesc, (kb | j) ? 1u : 0u);
      }
      kvm_tc_commit(kvm_bar_addr(ctl, KVM_TC_STAGES + s));       // frees the stage when these MMAs have read it
    }
    kvm_tc_commit(kvm_bar_addr(ctl, 2 * KVM_TC_STAGES));          // accumulator complete
    ctl[KVM_CTL_MMA_IT] = (int)it;
  }
  __syncwarp();
  // ---- epilogue: all 16 warps. Warp w owns TMEM lanes 32*(w%4).. and columns 64*(w/4)..
  const uint32_t acc_ph = (uint32_t)ctl[KVM_CTL_ACC_PH] & 1;
  if (!kvm_mbar_wait(kvm_bar_addr(ctl, 2 * KVM_TC_STAGES), acc_ph)) ok = false;
  kvm_tc_fence_after();
  if (!ok && atomicCAS(&c.err->code, 0, KVM_ERR_TIMEOUT) == 0) { c.err->task = c.task; c.err->a = 122; c.err->b = (int)threadIdx.x; }
  if (kvm_tc_epi_vec_ok(g)) kvm_tc_epilogue_staged(c, g, tmem, g.m0, ok);
  else {
    const int q = warp & 3, cgi = warp >> 2;
    const int m = g.m0 + q * 32 + lane;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = cgi * 64 + h * 32;
      float acc[32];
      kvm_tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)col, acc);
      if (ok && m < g.M) kvm_tc_store32(g, acc, m, g.n0 + col);
    }
    kvm_tc_fence_before();
    kvm_sync();
  }
  if (threadIdx.x == 0) ctl[KVM_CTL_ACC_PH] = (int)(acc_ph ^ 1);
}


// ---- the overlapped pipeline of the ready-queue kernel ---------------------------------------------------------------------------
// In the ready-queue kernel two extra warps run the mainloops (one thread issues the TMA loads, one the MMAs) for every tensor-core
// GEMM task as soon as it is staged, into one of TWO TMEM accumulators (columns 0..255 / 256..511), while the 16 compute warps are
// still draining the previous tile: tile n's epilogue overlaps tile n+1's mainloop and the first loads of tile n+2.
//   shared memory of the op scratch:  [0, KVM_TCE_STAGING)  epilogue staging (64 accumulator columns at a time)
//                                     [KVM_TCE_STAGING, + 3 x 48 KB)  operand ring of the engine
//   barriers (ctl barrier indices):   full[s] = s, empty[s] = 4 + s (s < 3), accumulator full[a] = 21 + a, accumulator empty[a] = 23 + a
// The engine only starts a tile while the compute group runs another tensor-core GEMM tile or has finished everything before it:
// any other op may use the whole scratch.
#define KVM_TCE_STAGES 3
#define KVM_TCE_STAGING 50176              // 49 KB: a multiple of 1024 (the ring's swizzled tiles start behind it), at least 128 rows x 68 floats
#define KVM_TCE_BAR_ACC_FULL 21
#define KVM_TCE_BAR_ACC_EMPTY 23
#define KVM_TCE_CHUNK 64                  // accumulator columns staged at a time
#define KVM_TCE_PITCH 68                  // floats per staged row (conflict-free 16-byte accesses)

// Bounded wait that also gives up when an error has been recorded anywhere (the other side may have left).
__device__ __forceinline__ bool kvm_mbar_wait_err(uint32_t bar, uint32_t parity, const KvmErrRec* err) {
  unsigned long long t0 = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 127u) == 127u) {
      if (*(volatile const int*)&err->code != 0) return false;
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (!t0) t0 = t; else if (t - t0 > 4000000000ull) return false;      // four seconds: the other side is not coming
    }
  }
}

// One tile's loads (engine producer thread).  `it` is the producer's running stage counter.
__device__ __forceinline__ bool kvm_tce_produce(int* ctl, uint32_t ring0, const void* tmaps, const int32_t* a, const int4& aux, uint32_t& it, const KvmErrRec* err) {
  const int m0 = a[6], n0 = a[7], K = a[10], fl = a[11];
  const bool ta = fl & 1, tb = fl & 2;
  const int num_kb = (K + KVM_TC_BK - 1) / KVM_TC_BK;
  const char* tmA = (const char*)tmaps + (size_t)aux.y * 128;
  const char* tmB = (const char*)tmaps + (size_t)aux.z * 128;
  asm volatile("fence.proxy.async;" ::: "memory");     // operands written by other tasks' plain stores are read here through TMA
  for (int kb = 0; kb < num_kb; ++kb, ++it) {
    const int s = it % KVM_TCE_STAGES;
    const uint32_t ph = (it / KVM_TCE_STAGES) & 1;
    if (it >= KVM_TCE_STAGES && !kvm_mbar_wait_err(kvm_bar_addr(ctl, 4 + s), ph ^ 1, err)) return false;
    const uint32_t full = kvm_bar_addr(ctl, s), sa = ring0 + s * KVM_TC_STAGE_BYTES, sb = sa + KVM_TC_A_BYTES;
    kvm_mbar_expect_tx(full, KVM_TC_STAGE_BYTES);
    const int k0 = kb * KVM_TC_BK;
    if (!ta) kvm_tma_load_2d(sa, tmA, k0, m0, full);
    else { kvm_tma_load_2d(sa, tmA, m0, k0, full); kvm_tma_load_2d(sa + 8192, tmA, m0 + 64, k0, full); }
    if (tb) kvm_tma_load_2d(sb, tmB, k0, n0, full);
    else {
#pragma unroll
      for (int i = 0; i < 4; ++i) kvm_tma_load_2d(sb + i * 8192, tmB, n0 + 64 * i, k0, full);
    }
  }
  return true;
}

// One tile's MMAs (engine MMA thread) into accumulator `g & 1`; `g` counts the tensor-core tiles of this CTA.
__device__ __forceinline__ bool kvm_tce_mma(int* ctl, uint32_t ring0, uint32_t tmem, const int32_t* a, uint32_t& it, uint32_t g, const KvmErrRec* err) {
  const int K = a[10], fl = a[11];
  const bool ta = fl & 1, tb = fl & 2;
  const int num_kb = (K + KVM_TC_BK - 1) / KVM_TC_BK;
  const uint32_t acc = g & 1u, use = g >> 1;
  if (use > 0 && !kvm_mbar_wait_err(kvm_bar_addr(ctl, KVM_TCE_BAR_ACC_EMPTY + acc), (use - 1) & 1, err)) return false;     // the tile before last has been drained
  kvm_tc_fence_after();
  const uint32_t idesc = kvm_idesc_bf16(128, 256, ta, !tb), d = tmem + acc * 256;
  for (int kb = 0; kb < num_kb; ++kb, ++it) {
    const int s = it % KVM_TCE_STAGES;
    const uint32_t ph = (it / KVM_TCE_STAGES) & 1;
    if (!kvm_mbar_wait_err(kvm_bar_addr(ctl, s), ph, err)) return false;
    kvm_tc_fence_after();
    const uint32_t sa = ring0 + s * KVM_TC_STAGE_BYTES, sb = sa + KVM_TC_A_BYTES;
#pragma unroll
    for (int j = 0; j < KVM_TC_BK / 16; ++j) {
      const uint64_t da = ta ? kvm_smem_desc(sa + j * 2048, 8192, 1024) : kvm_smem_desc(sa + j * 32, 16, 1024);
      const uint64_t db = tb ? kvm_smem_desc(sb + j * 32, 16, 1024) : kvm_smem_desc(sb + j * 2048, 8192, 1024);
      kvm_tc_mma_bf16(d, da, db, idesc, (kb | j) ? 1u : 0u);
    }
    kvm_tc_commit(kvm_bar_addr(ctl, 4 + s));
  }
  kvm_tc_commit(kvm_bar_addr(ctl, KVM_TCE_BAR_ACC_FULL + acc));
  return true;
}

// The compute group's share of a tile whose mainloop the engine runs: wait for the accumulator, drain it 64 columns at a time
// through the staging area (TMEM -> shared memory by (lane quarter, 16 columns) per warp; then thread = (row, 8 columns): every
// global access a whole row segment), hand the accumulator back.
static __device__ void kvm_tce_epilogue(const KvmCtx& c, const KvmMmArgs& g) {
  int* ctl = c.ctl;
  const uint32_t acc = c.gemm_seq & 1u, use = c.gemm_seq >> 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, q = warp & 3, cgi = warp >> 2;
  kvm_tc_fence_after();
  const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM) + acc * 256;
  bool ok = kvm_mbar_wait_err(kvm_bar_addr(ctl, KVM_TCE_BAR_ACC_FULL + acc), use & 1, c.err);
  kvm_tc_fence_after();
  if (!ok && atomicCAS(&c.err->code, 0, KVM_ERR_TIMEOUT) == 0) { c.err->task = c.task; c.err->a = 2122; c.err->b = (int)threadIdx.x; }
  if (kvm_tc_epi_vec_ok(g)) {
    float* T = (float*)c.smem;
    const bool simple = !(g.flags & 512);
    const float* bias = (const float*)g.bias.p;
#pragma unroll 1
    for (int ch = 0; ch < 256 / KVM_TCE_CHUNK; ++ch) {
      {
        float v[16];
        kvm_tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(ch * KVM_TCE_CHUNK + cgi * 16), v);
        float* dst = T + (size_t)(q * 32 + lane) * KVM_TCE_PITCH + cgi * 16;
#pragma unroll
        for (int j = 0; j < 16; j += 4) *(float4*)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
      if (ch == 256 / KVM_TCE_CHUNK - 1) kvm_tc_fence_before();
      kvm_sync();
      if (ch == 256 / KVM_TCE_CHUNK - 1 && threadIdx.x == 0 && ok) kvm_mbar_arrive_local(kvm_bar_addr(ctl, KVM_TCE_BAR_ACC_EMPTY + acc));      // every TMEM read of this tile is done
      if (ok) {
        for (int item = threadIdx.x; item < 128 * (KVM_TCE_CHUNK / 8); item += KVM_NT) {
          const int r = item >> 3, cc = (item & 7) * 8, m = g.m0 + r, n = g.n0 + ch * KVM_TCE_CHUNK + cc;
          if (m >= g.M || n >= g.N) continue;
          const float* src = T + (size_t)r * KVM_TCE_PITCH + cc;
          float v[8];
          *(float4*)v = *(const float4*)src; *(float4*)(v + 4) = *(const float4*)(src + 4);
          if (n + 8 <= g.N && simple) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= g.alpha;
            if (bias) { *(float4*)t = *(const float4*)(bias + n); *(float4*)(t + 4) = *(const float4*)(bias + n + 4);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += t[j]; }
            if (g.pre.p) kvm_st8(g.pre, (size_t)m * g.pre.ld + n, v);
            if (g.flags & 8) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = kvm_gelu(v[j]);
            }
            if (g.res.p) { kvm_ld8(g.res, (size_t)m * g.res.ld + n, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += t[j]; }
            if (g.flags & 4) { kvm_ld8(g.out, (size_t)m * g.out.ld + n, t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += t[j]; }
            kvm_st8(g.out, (size_t)m * g.out.ld + n, v);
          } else {
            for (int j = 0; j < 8 && n + j < g.N; ++j) kvm_st(g.out, (size_t)m * g.out.ld + n + j, kvm_mm_epilogue(g, v[j], m, n + j));
          }
        }
      }
      kvm_sync();
    }
  } else {
    const int m = g.m0 + q * 32 + lane;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int col = cgi * 64 + h * 32;
      float acc32[32];
      kvm_tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)col, acc32);
      if (ok && m < g.M) kvm_tc_store32(g, acc32, m, g.n0 + col);
    }
    kvm_tc_fence_before();
    kvm_sync();
    if (threadIdx.x == 0 && ok) kvm_mbar_arrive_local(kvm_bar_addr(ctl, KVM_TCE_BAR_ACC_EMPTY + acc));
  }
}
