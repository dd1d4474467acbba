// The static-schedule path: the resident program runs as per-worker task lists planned on the host (kvm_static_host.inl), with
// no ready queue, no dependency counters and no atomics on the task path.  What it implements of the reference: the static path
// of include/mvm_static.h:1-17,43-51 (list schedule -> per-worker records, cross-worker watermark waits) and its worker loop
// include/mvm_static.cuh:161-229 (fetch the next record ahead, poll the watermarks, dispatch, publish own progress).
//
// One CTA per SM as in the dynamic kernel: 16 compute warps + one FRONT warp.  The front warp walks the worker's list ahead of the
// compute group: it fetches task records into a four-slot shared-memory ring, polls the task's dependencies (pairs of
// (worker, tasks that worker must have finished), lanes in parallel over the pairs), and marks the slot ready.  A worker's
// progress word is one release store per finished task; nothing else is written to global memory for scheduling.
//
// Because a worker knows its next tasks, the front warp also STREAMS AHEAD: for decode GEMVs and split decode attention it
// issues the bulk copies of the task's weight rows / cache rows into a shared-memory stage ring as soon as stages are free,
// BEFORE the task's dependencies are resolved (weights and old cache rows do not change during a launch; the host marks a task
// whose streamed operand is written by some task of the batch, and its copies then wait for the dependencies like everything
// else).  The dependency wait then only gates the prologue and the arithmetic, so HBM keeps streaming across phase boundaries.
//
// Every wait is bounded (time limit); on expiry KVM_ERR_TIMEOUT is recorded, every CTA leaves, copies in flight are awaited.
#pragma once
#include "kvm_dispatch.cuh"
#include "kvm_static_api.h"

#define KVM_ST_SLOTS 4                 // record ring depth (tasks fetched ahead)
#define KVM_ST_HDR 3072                // header bytes: slots, control words, barriers
#define KVM_ST_ARRIVALS 16             // arrivals that free a stage: every compute warp, once it is done with the stage (or has nothing to do with it)

struct KvmStSlot {
  int task;
  int state;                  // 0 free, 1 fetched, 2 ready, 3 leave
  int go;
  int kind;                   // 0 generic op, 1 streamed gemv (one activation row, SIMT consumer), 2 streamed split attention, 3 streamed gemv on tensor cores (rows)
  int nchunks;                // stage uses of this task
  int R;                      // gemv: weight rows per stage (kind 3 keeps its chunk columns / row groups / k-chunks in j0 / j1 / newrow)
  int wait_off, wait_cnt;
  int32_t desc[16];
  int32_t args[KVM_MAX_ARGS];
  int4 aux;
  int prefetch;               // 1: copies may be issued before the dependencies are met
  int j0, j1, newrow;         // attention: key range of the split, index of the appended key inside it (-1 none)
  KvmBuf lb[7];               // streamed tasks: the buffer-table entries of the task's buffer arguments (argument j -> lb[j]), looked up once by the front warp
};
static_assert(sizeof(KvmStSlot) * KVM_ST_SLOTS + 128 * 4 + 64 + 288 + 128 <= KVM_ST_HDR, "static header too small");      // slots | control words | ... | rope cache (288) | ring barriers (128)

__device__ __forceinline__ bool kvm_mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

struct KvmRing {
  uint32_t bar0;              // full[s] at bar0 + 8 s, empty[s] at bar0 + 64 + 8 s
  unsigned char* base;        // stage s at base + s * KVM_ST_STAGE
  uint32_t base_addr;
  unsigned ns;                // stages: 3 (32 KB of op scratch beside them) or, for programs with gemv_bf16_rows, 2 (96 KB of scratch: the activations of eight rows)
};
__device__ __forceinline__ unsigned kvm_ring_slot(const KvmRing& r, unsigned it) { return r.ns == 2 ? (it & 1u) : it % 3u; }
__device__ __forceinline__ uint32_t kvm_ring_full(const KvmRing& r, unsigned it) { return r.bar0 + 8 * kvm_ring_slot(r, it); }
__device__ __forceinline__ uint32_t kvm_ring_empty(const KvmRing& r, unsigned it) { return r.bar0 + 64 + 8 * kvm_ring_slot(r, it); }
__device__ __forceinline__ uint32_t kvm_ring_parity(const KvmRing& r, unsigned it) { return (r.ns == 2 ? (it >> 1) : it / 3u) & 1u; }
__device__ __forceinline__ unsigned char* kvm_ring_stage(const KvmRing& r, unsigned it) { return r.base + kvm_ring_slot(r, it) * KVM_ST_STAGE; }

// Buffer argument j of a streamed task from the slot's own copy of the table entries (same checks as kvm_buf).
__device__ __forceinline__ bool kvm_buf_local(const KvmCtx& c, const KvmBuf* lb, const int32_t* a, int j, int mask, KvmBuf& out, bool optional = false) {
  const int idx = a[j];
  if (idx == -1 && optional) { out.p = nullptr; out.rows = out.cols = out.ld = 0; out.dtype = 0; return true; }
  if (idx < 0 || idx >= c.nbufs) { c.fail(KVM_OPE_BUF, idx); return false; }
  out = lb[j];
  if (out.p == nullptr || !((1 << out.dtype) & mask)) { c.fail(KVM_OPE_DTYPE, idx, out.dtype); return false; }
  return true;
}
__device__ __forceinline__ int kvm_ld_relaxed(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait for stage use `it` to land: lane 0 polls (bounded by the launch deadline and by an error recorded elsewhere), the verdict
// is the same for the whole warp.  All 32 lanes must call it.
__device__ __forceinline__ bool kvm_ring_wait_warp(const KvmRing& ring, unsigned it, unsigned long long deadline, const KvmErrRec* err) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    const uint32_t bar = kvm_ring_full(ring, it), par = kvm_ring_parity(ring, it);
    unsigned spins = 0;
    while (!kvm_mbar_test(bar, par)) {
      if ((++spins & 1023u) == 0 && (kvm_globaltimer() > deadline || *(volatile const int*)&err->code != 0)) { ok = 0; break; }      // an error elsewhere: the copies may never come
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ---- streamed GEMV, consumer side --------------------------------------------------------------------------------------------
// Stage use `cit + ci` holds rows n0 + ci*R .. of the weight matrix in full (R*K*2 bytes).  All sixteen warps consume: warp = (row r of the
// stage, part of K); the activation row v = bf16(prologue(x)) is staged once as bf16.  Partial sums are added in part order.
// Semantics as kvm_op_gemv_bf16 (runtime/ref_extra.py:398-415).  Always consumes its nchunks stage uses, also after an error.
KVM_OP_FN void kvm_gemv_ring(const KvmCtx& c, const int32_t* a, const KvmBuf* lb, const KvmRing& ring, unsigned cit, int R, int NC, unsigned long long deadline,
                                     unsigned long long t_task, int* stamp) {
  KvmBuf x, x2, gm, w, out, res;
  const int n0 = a[6], n1 = a[7], K = a[8], pro = a[9];
  const float eps = kvm_bits_f32(a[10]);
  bool ok = kvm_buf_local(c, lb, a, 0, KVM_M_FLT, x) && kvm_buf_local(c, lb, a, 1, KVM_M_FLT, x2, true) && kvm_buf_local(c, lb, a, 2, KVM_M_F32, gm, true) &&
            kvm_buf_local(c, lb, a, 3, KVM_M_BF16, w) && kvm_buf_local(c, lb, a, 4, KVM_M_FLT, out) && kvm_buf_local(c, lb, a, 5, KVM_M_FLT, res, true);
  const int rows = n1 - n0;
  const int KP = KVM_ST_ARRIVALS / R;
  const int fixed = ((K * 2 + 127) & ~127) + 256 + ((rows + 7) & ~7) * KP * 4;
  if (ok && (pro < 0 || pro > 2 || (pro == 1 && !gm.p) || (pro == 2 && !x2.p) || fixed > c.smem_bytes)) { c.fail(KVM_OPE_SHAPE, K, pro); ok = false; }
  if (ok) ok = kvm_mat_ok(c, x, 1, K) && kvm_mat_ok(c, x2, 1, K) && kvm_flat_ok(c, gm, K) && kvm_mat_ok(c, out, 1, n1) && kvm_mat_ok(c, res, 1, n1);
  __nv_bfloat16* vs = (__nv_bfloat16*)c.smem;
  float* red = (float*)(c.smem + ((K * 2 + 127) & ~127));
  float* parts = red + 64;                                 // [rows][KP]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  kvm_sync();                                              // the previous task is done with the scratch
  if (ok) {
    // ---- prologue: v = bf16(pro(x)) (all 16 warps)
    if (pro == 1 && K <= 16 * KVM_NT && x.dtype == KVM_F32 && kvm_vec_ok(x) && kvm_vec_ok(gm)) {
      // float32 row of up to 8192 values: four 16-byte loads of x and of gamma per thread, all in flight together (no storage-type
      // test between them: with one, every load waits for the one before it), the row stays in registers for the statistics
      float4 xr[4], gr[4];
      float q = 0.0f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = (tid + u * KVM_NT) * 4;
        xr[u] = k < K ? *(const float4*)((const float*)x.p + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        gr[u] = k < K ? *(const float4*)((const float*)gm.p + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) q += xr[u].x * xr[u].x + xr[u].y * xr[u].y + xr[u].z * xr[u].z + xr[u].w * xr[u].w;
      q = kvm_block_sum(q, red);
      const float rs = 1.0f / sqrtf(q / K + eps);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = (tid + u * KVM_NT) * 4;
        if (k < K) {
          *(__nv_bfloat162*)(vs + k) = __floats2bfloat162_rn(xr[u].x * rs * gr[u].x, xr[u].y * rs * gr[u].y);
          *(__nv_bfloat162*)(vs + k + 2) = __floats2bfloat162_rn(xr[u].z * rs * gr[u].z, xr[u].w * rs * gr[u].w);
        }
      }
    } else if (pro == 1 && K <= 16 * KVM_NT) {
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
      for (int u = 0; u < 16; ++u) { const int k = tid + u * KVM_NT; if (k < K) vs[k] = __float2bfloat16_rn(xr[u] * rs * gr[u]); }
    } else if (pro == 1) {
      float q = 0.0f;
      for (int k = tid; k < K; k += KVM_NT) { const float t = kvm_ld(x, k); q += t * t; }
      q = kvm_block_sum(q, red);
      const float rs = 1.0f / sqrtf(q / K + eps);
      for (int k = tid; k < K; k += KVM_NT) vs[k] = __float2bfloat16_rn(kvm_ld(x, k) * rs * ((const float*)gm.p)[k]);
    } else if (x.dtype == KVM_F32 && kvm_vec_ok(x) && (pro != 2 || (x2.dtype == KVM_F32 && kvm_vec_ok(x2)))) {
      // three 16-byte loads per input and thread in flight per round (a 12288-wide SwiGLU row is two rounds)
      for (int k0 = 0; k0 < K; k0 += 12 * KVM_NT) {
        float4 p[3], q[3];
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          const int k = k0 + (tid + u * KVM_NT) * 4;
          p[u] = k < K ? *(const float4*)((const float*)x.p + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          q[u] = (pro == 2 && k < K) ? *(const float4*)((const float*)x2.p + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          const int k = k0 + (tid + u * KVM_NT) * 4;
          if (k < K) {
            const float4 v = pro == 2 ? make_float4(kvm_silu(p[u].x) * q[u].x, kvm_silu(p[u].y) * q[u].y, kvm_silu(p[u].z) * q[u].z, kvm_silu(p[u].w) * q[u].w) : p[u];
            *(__nv_bfloat162*)(vs + k) = __floats2bfloat162_rn(v.x, v.y);
            *(__nv_bfloat162*)(vs + k + 2) = __floats2bfloat162_rn(v.z, v.w);
          }
        }
      }
    } else {
      for (int k0 = 0; k0 < K; k0 += 8 * KVM_NT) {
        float p[8], q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = k0 + tid + u * KVM_NT;
          p[u] = k < K ? kvm_ld(x, k) : 0.0f;
          q[u] = (pro == 2 && k < K) ? kvm_ld(x2, k) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = k0 + tid + u * KVM_NT;
          if (k < K) vs[k] = __float2bfloat16_rn(pro == 2 ? kvm_silu(p[u]) * q[u] : p[u]);
        }
      }
    }
  }
  kvm_sync();
  bool waited = true;
  unsigned long long t_pro = 0, t_wait = 0, t_first = 0;
  if (stamp && tid == 0) t_pro = kvm_globaltimer();
  {
    const int r = warp / KP, part = warp % KP;
    const int plen = (((K + KP - 1) / KP) + 255) & ~255, kb = part * plen, ke = min(K, kb + plen);
    for (int ci = 0; ci < NC; ++ci) {
      const unsigned it = cit + ci;
      unsigned long long tw = 0;
      if (stamp && tid == 0) tw = kvm_globaltimer();
      if (waited && !kvm_ring_wait_warp(ring, it, deadline, c.err)) waited = false;
      if (stamp && tid == 0) { const unsigned long long d = kvm_globaltimer() - tw; t_wait += d; if (ci == 0) t_first = d; }
      if (!waited) break;                                  // warp-uniform
      if (ok && r < R && ci * R + r < rows) {
        const unsigned char* st = kvm_ring_stage(ring, it) + (size_t)r * K * 2;
        float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
        int k = kb + lane * 8;
        for (; k + 256 < ke; k += 512) {                   // two 16-byte pieces of the row and of the activations in flight per trip
          const uint4 wa = *(const uint4*)(st + k * 2), wb = *(const uint4*)(st + (k + 256) * 2);
          const uint4 xa = *(const uint4*)(vs + k), xb = *(const uint4*)(vs + k + 256);
          acc0 = fmaf(kvm_bf16lo(xa.x), kvm_bf16lo(wa.x), acc0); acc1 = fmaf(kvm_bf16hi(xa.x), kvm_bf16hi(wa.x), acc1);
          acc2 = fmaf(kvm_bf16lo(xb.x), kvm_bf16lo(wb.x), acc2); acc3 = fmaf(kvm_bf16hi(xb.x), kvm_bf16hi(wb.x), acc3);
          acc0 = fmaf(kvm_bf16lo(xa.y), kvm_bf16lo(wa.y), acc0); acc1 = fmaf(kvm_bf16hi(xa.y), kvm_bf16hi(wa.y), acc1);
          acc2 = fmaf(kvm_bf16lo(xb.y), kvm_bf16lo(wb.y), acc2); acc3 = fmaf(kvm_bf16hi(xb.y), kvm_bf16hi(wb.y), acc3);
          acc0 = fmaf(kvm_bf16lo(xa.z), kvm_bf16lo(wa.z), acc0); acc1 = fmaf(kvm_bf16hi(xa.z), kvm_bf16hi(wa.z), acc1);
          acc2 = fmaf(kvm_bf16lo(xb.z), kvm_bf16lo(wb.z), acc2); acc3 = fmaf(kvm_bf16hi(xb.z), kvm_bf16hi(wb.z), acc3);
          acc0 = fmaf(kvm_bf16lo(xa.w), kvm_bf16lo(wa.w), acc0); acc1 = fmaf(kvm_bf16hi(xa.w), kvm_bf16hi(wa.w), acc1);
          acc2 = fmaf(kvm_bf16lo(xb.w), kvm_bf16lo(wb.w), acc2); acc3 = fmaf(kvm_bf16hi(xb.w), kvm_bf16hi(wb.w), acc3);
        }
        for (; k < ke; k += 256) {
          const uint4 wv = *(const uint4*)(st + k * 2);
          const uint4 xv = *(const uint4*)(vs + k);
          acc0 = fmaf(kvm_bf16lo(xv.x), kvm_bf16lo(wv.x), acc0); acc1 = fmaf(kvm_bf16hi(xv.x), kvm_bf16hi(wv.x), acc1);
          acc0 = fmaf(kvm_bf16lo(xv.y), kvm_bf16lo(wv.y), acc0); acc1 = fmaf(kvm_bf16hi(xv.y), kvm_bf16hi(wv.y), acc1);
          acc0 = fmaf(kvm_bf16lo(xv.z), kvm_bf16lo(wv.z), acc0); acc1 = fmaf(kvm_bf16hi(xv.z), kvm_bf16hi(wv.z), acc1);
          acc0 = fmaf(kvm_bf16lo(xv.w), kvm_bf16lo(wv.w), acc0); acc1 = fmaf(kvm_bf16hi(xv.w), kvm_bf16hi(wv.w), acc1);
        }
        const float sum = kvm_warp_sum((acc0 + acc1) + (acc2 + acc3));
        if (lane == 0) parts[(ci * R + r) * KP + part] = sum;
      }
      __syncwarp();
      if (lane == 0) kvm_mbar_arrive(kvm_ring_empty(ring, it));
    }
  }
  __syncwarp();
  if (stamp && tid == 0) {      // trace detail, one byte each in units of 0.2 us: prologue | stage loop (waits included) | waits for stages
    (void)t_first;
    stamp[0] = (int)min(255ull, (t_pro - t_task) / 200) | ((int)min(255ull, (kvm_globaltimer() - t_pro) / 200) << 8) | ((int)min(255ull, t_wait / 200) << 16);
  }
  if (!waited && *(volatile int*)&c.err->code == 0) kvm_stream_timeout(c, 1134);
  kvm_sync();
  if (ok && *(volatile int*)&c.err->code == 0)
    for (int i = tid; i < rows; i += KVM_NT) {
      float sum = 0.0f;
      for (int p = 0; p < KP; ++p) sum += parts[i * KP + p];
      kvm_st(out, n0 + i, res.p ? __fadd_rn(sum, kvm_ld(res, n0 + i)) : sum);
    }
}

// ---- streamed GEMV on tensor cores (gemv_bf16 with one activation row, gemv_bf16_rows with up to eight), consumer side --------------
// D[16 x 8] += A[16 x 16] B[16 x 8] (mma.sync m16n8k16, bf16 operands, float32 accumulate) with A = activations (rows = activation
// rows, at most eight of the sixteen used), B = the weight rows of a stage (columns).  A dot product does not care in which order k
// is visited, so both operands are read 16 bytes per thread from row-major [row][k] arrays at the SAME k offsets (thread t of a quad
// takes k = 8t .. 8t+7 of a 32-wide step, for two MMAs) instead of in the instruction's interleaved k layout.  Steps are taken in
// pairs: weight rows sit a multiple of 128 bytes apart, so an odd row reads the pair's steps in the other order (and swaps the
// registers back before the MMAs): the eight lanes of a quarter warp (two rows, four quads) then read eight different 16-byte
// bank groups.  The activations are staged as bf16 with a row pitch of 64 bytes mod 128 for the same reason.
//
// Two stage layouts, chosen by kvm_gemv_mma_layout from the shapes alone (the front warp and the consumers compute the same):
//   whole rows   a stage holds R <= 8 weight rows in full (KC = K, R*K*2 <= 64 KB, one bulk copy); every stage is a row group of
//                its own, its sums leave the registers when the stage is done; needs all of the M activation rows staged at once;
//   k chunks     a stage holds 8 weight rows x KC columns (KC < K, eight copies); stages run k-chunk outer, row group inner, the
//                accumulators of up to eight row groups stay in registers over the whole task, the activations are staged per k-chunk.
// All sixteen warps multiply (pairs of steps are dealt round robin); their partial sums are added in warp order at the end.
// Semantics per activation row as gemv_bf16 (runtime/ref_extra.py:398-415).  Always consumes its nchunks stage uses, also after an error.
#define KVM_MMA_PARTS_OFF 512
struct KvmMmaLayout {
  int R, KC, nkc, ng;       // weight rows and columns per stage, k-chunks, row groups
  int full_x;               // all k of the activations staged once
  int pitch;                // bytes per staged activation row
  int parts_off;            // byte offset of the partial sums [16 warps][ng][M][R] in the scratch
  int nchunks;
  bool ok;
};
__device__ __forceinline__ KvmMmaLayout kvm_gemv_mma_layout(int rows, int K, int M, int scratch_bytes) {
  KvmMmaLayout L;
  L.ok = false;
  const int row_pitch = K * 2 + 64;
  // whole rows
  L.R = K * 2 * 8 <= KVM_ST_STAGE ? 8 : KVM_ST_STAGE / (K * 2);
  if (L.R >= 1) {
    L.KC = K; L.nkc = 1; L.ng = (rows + L.R - 1) / L.R; L.full_x = 1; L.pitch = row_pitch;
    L.parts_off = M * row_pitch + KVM_MMA_PARTS_OFF;
    if (L.parts_off + 16 * L.ng * M * L.R * 4 <= scratch_bytes) { L.nchunks = L.ng; L.ok = true; return L; }
  }
  // k chunks
  L.R = 8; L.KC = 4096;
  while (L.KC > 0 && K % L.KC) L.KC -= 256;
  if (L.KC <= 0 || L.KC >= K) return L;
  L.nkc = K / L.KC; L.ng = (rows + 7) / 8;
  if (L.ng > 8) return L;
  L.full_x = M * row_pitch + KVM_MMA_PARTS_OFF + 16 * L.ng * M * 8 * 4 <= scratch_bytes;
  L.pitch = L.full_x ? row_pitch : L.KC * 2 + 64;
  L.parts_off = M * L.pitch + KVM_MMA_PARTS_OFF;
  if (L.parts_off + 16 * L.ng * M * 8 * 4 > scratch_bytes) return L;
  L.nchunks = L.nkc * L.ng; L.ok = true;
  return L;
}
__device__ __forceinline__ void kvm_mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
// v[j] = prologue value of 8 consecutive activations starting at column k of row u
__device__ __forceinline__ void kvm_mma_pro8(int pro, float (&v)[8], const float (&v2)[8], float rs) {
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = pro == 1 ? v[j] * rs * v2[j] : pro == 2 ? kvm_silu(v[j]) * v2[j] : v[j];
}
__device__ __forceinline__ uint4 kvm_pack_bf16x8(const float (&v)[8]) {
  uint4 pk;
  __nv_bfloat162* hh = (__nv_bfloat162*)&pk;
#pragma unroll
  for (int j = 0; j < 4; ++j) hh[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  return pk;
}
// Staging of the activations v = bf16(pro(x)) for the tensor-core consumer, functions of their own (registers of their own).
struct KvmStageX {
  KvmBuf x, x2, gm;
  unsigned char* xs;        // [M][pitch] bytes
  float* rsq;               // [8] reciprocal RMS per row, from [64] on reduction scratch
  int r0, M, K, pro, pitch;
  float eps;
};
// One activation row whose prologue loads all fit into registers: every load in flight at once, one pass.  false = not taken.
KVM_OP_FN bool kvm_stage_one_row(const KvmStageX& s) {
  const KvmBuf x = s.x, x2 = s.x2, gm = s.gm;
  const int K = s.K, pro = s.pro, tid = threadIdx.x;
  if (K > 3 * 8 * KVM_NT || (x.ld & 7) || !kvm_vec_ok(x) || (pro == 2 && ((x2.ld & 7) || !kvm_vec_ok(x2))) || (pro == 1 && !kvm_vec_ok(gm))) return false;
  float v[3][8], v2[3][8];
  const size_t xo = (size_t)s.r0 * x.ld, x2o = x2.p ? (size_t)s.r0 * x2.ld : 0;
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int k = (tid + j * KVM_NT) * 8;
    if (k < K) {
      kvm_ld8(x, xo + k, v[j]);
      if (pro == 2) kvm_ld8(x2, x2o + k, v2[j]);
      else if (pro == 1) { *(float4*)v2[j] = *(const float4*)((const float*)gm.p + k); *(float4*)(v2[j] + 4) = *(const float4*)((const float*)gm.p + k + 4); }
    }
  }
  float rs = 0.0f;
  if (pro == 1) {
    float q = 0.0f;
#pragma unroll
    for (int j = 0; j < 3; ++j) if ((tid + j * KVM_NT) * 8 < K)
#pragma unroll
      for (int u = 0; u < 8; ++u) q += v[j][u] * v[j][u];
    q = kvm_block_sum(q, s.rsq + 64);
    rs = 1.0f / sqrtf(q / K + s.eps);
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int k = (tid + j * KVM_NT) * 8;
    if (k < K) { kvm_mma_pro8(pro, v[j], v2[j], rs); *(uint4*)(s.xs + (size_t)k * 2) = kvm_pack_bf16x8(v[j]); }
  }
  return true;
}
// RMS statistics of up to eight rows: two warps per activation row.  Whole compute group.
KVM_OP_FN void kvm_stage_rms(const KvmStageX& s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, u = warp >> 1, hf = warp & 1, K = s.K;
  float q = 0.0f;
  if (u < s.M) for (int k = hf * (K / 2) + lane; k < (hf + 1) * (K / 2); k += 32) { const float v = kvm_ld(s.x, (size_t)(s.r0 + u) * s.x.ld + k); q += v * v; }
  q = kvm_warp_sum(q);
  if (lane == 0) s.rsq[64 + warp] = q;
  kvm_sync();
  if (tid < 8) s.rsq[tid] = tid < s.M ? 1.0f / sqrtf((s.rsq[64 + 2 * tid] + s.rsq[64 + 2 * tid + 1]) / K + s.eps) : 0.0f;
  kvm_sync();
}
// Columns [kb, kb + kn) of the M rows to column offset 0 of the staged rows (all 16 warps).
KVM_OP_FN void kvm_stage_rows(const KvmStageX& s, int kb, int kn) {
  const KvmBuf x = s.x, x2 = s.x2, gm = s.gm;
  const int pro = s.pro, r0 = s.r0;
  const bool vec_x = (x.ld & 7) == 0 && kvm_vec_ok(x), vec_x2 = x2.p && (x2.ld & 7) == 0 && kvm_vec_ok(x2), vec_g = gm.p && kvm_vec_ok(gm);
  for (int e = threadIdx.x; e < s.M * (kn / 8); e += KVM_NT) {
    const int u = e / (kn / 8), k0 = (e % (kn / 8)) * 8, k = kb + k0;
    float v[8], v2[8];
    if (vec_x) kvm_ld8(x, (size_t)(r0 + u) * x.ld + k, v);
    else for (int j = 0; j < 8; ++j) v[j] = kvm_ld(x, (size_t)(r0 + u) * x.ld + k + j);
    if (pro == 2) {
      if (vec_x2) kvm_ld8(x2, (size_t)(r0 + u) * x2.ld + k, v2);
      else for (int j = 0; j < 8; ++j) v2[j] = kvm_ld(x2, (size_t)(r0 + u) * x2.ld + k + j);
    } else if (pro == 1) {
      if (vec_g) { *(float4*)v2 = *(const float4*)((const float*)gm.p + k); *(float4*)(v2 + 4) = *(const float4*)((const float*)gm.p + k + 4); }
      else for (int j = 0; j < 8; ++j) v2[j] = ((const float*)gm.p)[k + j];
    }
    kvm_mma_pro8(pro, v, v2, pro == 1 ? s.rsq[u] : 0.0f);
    *(uint4*)(s.xs + (size_t)u * s.pitch + (size_t)k0 * 2) = kvm_pack_bf16x8(v);
  }
}
template <bool CHUNKED>      // the k-chunk layout (accumulators of eight row groups live over the task) or the whole-row layout, a function each
KVM_OP_FN void kvm_gemv_mma_ring_t(const KvmCtx& c, const int32_t* a, const KvmBuf* lb, bool has_rows, const KvmRing& ring, unsigned cit, unsigned long long deadline,
                                   unsigned long long t_task, int* stamp) {
  KvmBuf x, x2, gm, w, out, res;
  const int n0 = a[6], n1 = a[7], K = a[8], pro = a[9], r0 = has_rows ? a[11] : 0, r1 = has_rows ? a[12] : 1;
  const float eps = kvm_bits_f32(a[10]);
  bool ok = kvm_buf_local(c, lb, a, 0, KVM_M_FLT, x) && kvm_buf_local(c, lb, a, 1, KVM_M_FLT, x2, true) && kvm_buf_local(c, lb, a, 2, KVM_M_F32, gm, true) &&
            kvm_buf_local(c, lb, a, 3, KVM_M_BF16, w) && kvm_buf_local(c, lb, a, 4, KVM_M_FLT, out) && kvm_buf_local(c, lb, a, 5, KVM_M_FLT, res, true);
  const int rows = n1 - n0, M = r1 - r0;
  const KvmMmaLayout L = kvm_gemv_mma_layout(rows, K, M, c.smem_bytes);       // the front warp accepted the same layout
  const int R = L.R, KC = L.KC, ng = L.ng, nkc = L.nkc, pitch = L.pitch;
  if (ok && (pro < 0 || pro > 2 || (pro == 1 && !gm.p) || (pro == 2 && !x2.p) || !L.ok || CHUNKED != (L.nkc > 1))) { c.fail(KVM_OPE_SHAPE, K, pro); ok = false; }
  if (ok) ok = kvm_mat_ok(c, x, r1, K) && kvm_mat_ok(c, x2, r1, K) && kvm_flat_ok(c, gm, K) && kvm_mat_ok(c, out, r1, n1) && kvm_mat_ok(c, res, r1, n1);
  unsigned char* xs = c.smem;                              // [M][pitch]
  float* rsq = (float*)(c.smem + M * pitch);               // [8] reciprocal RMS per activation row, from [64] on reduction scratch
  float* parts = (float*)(c.smem + L.parts_off);           // [16 warps][ng][M][R]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  kvm_sync();                                              // the previous task is done with the scratch
  struct KvmStageX sx;
  sx.x = x; sx.x2 = x2; sx.gm = gm; sx.xs = xs; sx.rsq = rsq; sx.r0 = r0; sx.M = M; sx.K = K; sx.pro = pro; sx.pitch = pitch; sx.eps = eps;
  bool staged = false;
  if (ok && M == 1 && L.full_x) staged = kvm_stage_one_row(sx);
  if (ok && !staged && pro == 1) kvm_stage_rms(sx);
  if (ok && !staged && L.full_x) kvm_stage_rows(sx, 0, K);
  kvm_sync();
  unsigned long long t_pro = 0, t_wait = 0, t_first = 0;
  if (stamp && tid == 0) t_pro = kvm_globaltimer();
  bool waited = true;
  const int npairs = KC / 64;
  // one stage use: wait for it, multiply it into acc (x columns from xk0 of the staged rows), release it
  auto consume = [&](unsigned it, float (&acc)[4], int xk0) {
    unsigned long long tw = 0;
    if (stamp && tid == 0) tw = kvm_globaltimer();
    if (waited && !kvm_ring_wait_warp(ring, it, deadline, c.err)) waited = false;
    if (stamp && tid == 0) { const unsigned long long d = kvm_globaltimer() - tw; t_wait += d; if (it == cit) t_first = d; }
    if (!waited) return;                                   // warp-uniform; the warp still takes part in every barrier of the task
    if (ok) {
      const unsigned char* wrow = kvm_ring_stage(ring, it) + (size_t)g * KC * 2 + t * 16;
      const unsigned char* xrow = xs + (size_t)g * pitch + (size_t)xk0 * 2 + t * 16;
      const int odd = g & 1;
      float acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};                  // the two steps of a pair accumulate side by side
#pragma unroll 2
      for (int p = warp; p < npairs; p += KVM_NT / 32) {
        uint4 b0 = make_uint4(0, 0, 0, 0), b1 = b0, a0 = b0, a1 = b0;
        if (g < R) { b0 = *(const uint4*)(wrow + (2 * p + odd) * 64); b1 = *(const uint4*)(wrow + (2 * p + 1 - odd) * 64); }
        if (g < M) { a0 = *(const uint4*)(xrow + (2 * p) * 64); a1 = *(const uint4*)(xrow + (2 * p + 1) * 64); }
        const uint4 e0 = odd ? b1 : b0, e1 = odd ? b0 : b1;       // weights of step 2p and of step 2p + 1
        kvm_mma_bf16_16816(acc, a0.x, a0.y, e0.x, e0.y);
        kvm_mma_bf16_16816(acc2, a1.x, a1.y, e1.x, e1.y);
        kvm_mma_bf16_16816(acc, a0.z, a0.w, e0.z, e0.w);
        kvm_mma_bf16_16816(acc2, a1.z, a1.w, e1.z, e1.w);
      }
      acc[0] += acc2[0]; acc[1] += acc2[1]; acc[2] += acc2[2]; acc[3] += acc2[3];
    }
    __syncwarp();
    if (lane == 0) kvm_mbar_arrive(kvm_ring_empty(ring, it));
  };
  // thread (g, t) holds D[activation row g][weight rows 2t, 2t + 1]
  auto put_parts = [&](int rg, const float (&acc)[4]) {
    if (g < M) {
      float* pp = parts + (((size_t)warp * ng + rg) * M + g) * R;
      if (2 * t < R) pp[2 * t] = acc[0];
      if (2 * t + 1 < R) pp[2 * t + 1] = acc[1];
    }
  };
  if (!CHUNKED) {
    for (int rg = 0; rg < ng; ++rg) {
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      consume(cit + (unsigned)rg, acc, 0);
      put_parts(rg, acc);
    }
  } else {
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    for (int kc = 0; kc < nkc; ++kc) {
      if (!L.full_x) {
        if (kc) kvm_sync();                                // the consumers are done with the previous chunk's activations
        if (ok) kvm_stage_rows(sx, kc * KC, KC);
        kvm_sync();
      }
#pragma unroll
      for (int rg = 0; rg < 8; ++rg) if (rg < ng) consume(cit + (unsigned)(kc * ng + rg), acc[rg], L.full_x ? kc * KC : 0);
    }
#pragma unroll
    for (int rg = 0; rg < 8; ++rg) if (rg < ng) put_parts(rg, acc[rg]);
  }
  __syncwarp();
  if (stamp && tid == 0) {      // trace detail, one byte each in units of 0.2 us: prologue | stage loop (waits included) | waits for stages
    (void)t_first;
    stamp[0] = (int)min(255ull, (t_pro - t_task) / 200) | ((int)min(255ull, (kvm_globaltimer() - t_pro) / 200) << 8) | ((int)min(255ull, t_wait / 200) << 16);
  }
  if (!waited && *(volatile int*)&c.err->code == 0) kvm_stream_timeout(c, 1301);
  kvm_sync();
  if (ok && *(volatile int*)&c.err->code == 0)            // a warp that gave up has recorded the timeout before the barrier
    for (int e = tid; e < ng * M * R; e += KVM_NT) {
      const int rg = e / (M * R), u = (e / R) % M, nn = e % R, n = n0 + rg * R + nn;
      if (n >= n1) continue;
      float sum = 0.0f;
#pragma unroll
      for (int wv = 0; wv < KVM_NT / 32; ++wv) sum += parts[(((size_t)wv * ng + rg) * M + u) * R + nn];
      const size_t o = (size_t)(r0 + u) * out.ld + n;
      kvm_st(out, o, res.p ? __fadd_rn(sum, kvm_ld(res, (size_t)(r0 + u) * res.ld + n)) : sum);
    }
}

__device__ __forceinline__ void kvm_gemv_mma_ring(const KvmCtx& c, const int32_t* a, const KvmBuf* lb, bool has_rows, const KvmRing& ring, unsigned cit, int nkc,
                                                  unsigned long long deadline, unsigned long long t_task, int* stamp) {
  if (nkc > 1) kvm_gemv_mma_ring_t<true>(c, a, lb, has_rows, ring, cit, deadline, t_task, stamp);
  else kvm_gemv_mma_ring_t<false>(c, a, lb, has_rows, ring, cit, deadline, t_task, stamp);
}

// ---- streamed split attention, consumer side ----------------------------------------------------------------------------------
// Stage use `cit` holds the split's keys, `cit + 1` its values (the appended row left out).  Semantics as kvm_op_attn_decode_part
// (runtime/ref_extra.py:421-498); the front warp has validated the geometry before it issued the copies.
KVM_OP_FN void kvm_attn_part_ring(const KvmCtx& c, const int32_t* a, const KvmBuf* lb, bool qkn, const KvmRing& ring, unsigned cit, int j0, int j1, int newrow,
                                          unsigned long long deadline, unsigned long long t_task, int* stamp) {
  KvmBuf q, kc, vc, lens, part, kn, vn, gam{};
  bool ok = kvm_buf_local(c, lb, a, 0, KVM_M_FLT, q) && kvm_buf_local(c, lb, a, 1, KVM_M_FLT, kc) && kvm_buf_local(c, lb, a, 2, KVM_M_FLT, vc) &&
            kvm_buf_local(c, lb, a, 3, KVM_M_I32, lens) && kvm_buf_local(c, lb, a, 4, KVM_M_F32, part) && kvm_buf_local(c, lb, a, 5, KVM_M_FLT, kn, true) &&
            kvm_buf_local(c, lb, a, 6, KVM_M_FLT, vn, true);
  if (ok && qkn) ok = kvm_buf(c, a[18], KVM_M_F32, gam);
  const int b = a[7], kvh = a[8], s = a[9], S = a[10], H = a[11], Hkv = a[12], hd = a[13], Tmax = a[14], fl = a[17];
  const float sc = kvm_bits_f32(a[15]), theta = kvm_bits_f32(a[16]);
  const int G = H / Hkv;
  if (ok) ok = kvm_mat_ok(c, q, b + 1, H * hd) && kvm_mat_ok(c, part, (long long)(b + 1) * S * H, hd + 2) && kvm_mat_ok(c, kn, b + 1, Hkv * hd) && kvm_mat_ok(c, vn, b + 1, Hkv * hd) &&
            kvm_mat_ok(c, gam, 2, hd);
  if (ok && ((fl & 1) && (!kn.p || !vn.p))) { c.fail(KVM_OPE_SHAPE, hd, fl); ok = false; }
  const int p0 = ok ? ((const int*)lens.p)[b] : 0, nk = max(j1 - j0, 0);
  unsigned char* sm = c.smem;
  unsigned char* Ks = kvm_ring_stage(ring, cit);
  unsigned char* Vs = kvm_ring_stage(ring, cit + 1);
  auto wait_use = [&](unsigned it) {
    const uint32_t bar = kvm_ring_full(ring, it), par = kvm_ring_parity(ring, it);
    unsigned spins = 0;
    while (!kvm_mbar_test(bar, par)) if ((++spins & 1023u) == 0 && (kvm_globaltimer() > deadline || *(volatile int*)&c.err->code != 0)) return false;
    return true;
  };
  kvm_sync();                                              // the previous task is done with the scratch
  bool waited = true;
  if (ok) {
    KvmPartPro P;
    P.q = q; P.kc = kc; P.vc = vc; P.kn = kn; P.vn = vn; P.gam = gam;
    P.b = b; P.kvh = kvh; P.G = G; P.hd = hd; P.fl = fl; P.p0 = p0; P.base = (size_t)(b * Hkv + kvh) * Tmax; P.theta = theta; P.eps = qkn ? kvm_bits_f32(a[19]) : 0.0f;
    P.appends = newrow >= 0;
    P.rope_cache = c.rope_cache;
    P.qs = (float*)(sm + KVM_AS_OFF_QS); P.inv = (float*)(sm + KVM_AS_OFF_INV); P.kns = (float*)(sm + KVM_AS_OFF_KNEW); P.vns = (float*)(sm + KVM_AS_OFF_VNEW);
    P.rsq = (float*)(sm + KVM_AS_OFF_ML);
    unsigned long long t_wait = 0;
    auto prologue = [&]() {
      kvm_part_prologue(P);
      if (stamp && threadIdx.x == 0) stamp[0] = (int)min(255ull, (kvm_globaltimer() - t_task) / 100);      // trace detail, byte 0: start to end of the prologue (0.1 us)
    };
    float* pp = (float*)part.p;
    auto emit = [&](int g, int cc, float M, float Lsum, float A) {
      const size_t row = ((size_t)(b * S + s) * H + kvh * G + g) * part.ld;
      pp[row + cc] = Lsum > 0.0f ? A : 0.0f;
      if (cc == 0) { pp[row + hd] = Lsum > 0.0f ? M : KVM_ATTN_EMPTY_M_STREAM; pp[row + hd + 1] = Lsum; }
    };
    auto timed_wait = [&](unsigned it) {
      const unsigned long long t0 = stamp && threadIdx.x == 0 ? kvm_globaltimer() : 0;
      const bool r = wait_use(it);
      if (stamp && threadIdx.x == 0) t_wait += kvm_globaltimer() - t0;
      return r;
    };
    auto wk = [&]() { return timed_wait(cit); };
    auto wv = [&]() { return timed_wait(cit + 1); };
    if (G <= 1) waited = kvm_attn_part_core<1>(sm, Ks, Vs, nk, newrow, G, hd, sc, prologue, wk, wv, emit);
    else if (G <= 2) waited = kvm_attn_part_core<2>(sm, Ks, Vs, nk, newrow, G, hd, sc, prologue, wk, wv, emit);
    else if (G <= 4) waited = kvm_attn_part_core<4>(sm, Ks, Vs, nk, newrow, G, hd, sc, prologue, wk, wv, emit);
    else waited = kvm_attn_part_core<8>(sm, Ks, Vs, nk, newrow, G, hd, sc, prologue, wk, wv, emit);
    if (stamp && threadIdx.x == 0) stamp[0] |= (int)min(255ull, t_wait / 100) << 8;       // byte 1: waits for the keys and the values (0.1 us)
  } else {
    waited = wait_use(cit) && wait_use(cit + 1);
  }
  if (!waited && *(volatile int*)&c.err->code == 0) kvm_stream_timeout(c, 1135);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the appended row was written by threads; the next copies into these stages come after it
  kvm_sync();
  if (waited && (threadIdx.x & 31) == 0) { kvm_mbar_arrive(kvm_ring_empty(ring, cit)); kvm_mbar_arrive(kvm_ring_empty(ring, cit + 1)); }
}

// ---- front warp: stream geometry of a fetched task (lane 0) ---------------------------------------------------------------------
// Decides whether the task streams through the ring and with which chunking; every bound the copies rely on is checked here,
// a task that fails one runs as a generic op (whose own checks then report the error).
static __device__ void kvm_static_geometry(const KvmDevState& S, KvmStSlot& sl, int scratch_bytes) {
  sl.kind = 0; sl.nchunks = 0; sl.R = 1; sl.j0 = sl.j1 = 0; sl.newrow = -1;
  const int op = sl.desc[0];
  const int32_t* a = sl.args;
  if (op == 134 || op == 301) {
    const int wi = a[3], n0 = a[6], n1 = a[7], K = a[8], r0 = op == 301 ? a[11] : 0, r1 = op == 301 ? a[12] : 1;
    if (wi < 0 || wi >= S.nbufs || n0 < 0 || n1 <= n0 || K <= 0 || (K & 255) || r0 < 0 || r1 <= r0 || r1 - r0 > 8) return;
    const KvmBuf w = sl.lb[3];
    if (!w.p || w.dtype != KVM_BF16 || (w.ld & 7) || ((uintptr_t)w.p & 15) || n1 > w.rows || K > w.cols) return;
    // one activation row: the SIMT consumer over stages of whole rows (measured faster than mma.sync fragments at one row: the
    // legacy tensor path of this part issues an m16n8k16 every few hundred cycles per warp); several rows: the tensor-core consumer
    if (op == 134 && K * 2 <= KVM_ST_STAGE) {
      int R = KVM_ST_STAGE / (K * 2);
      if (R > KVM_ST_ARRIVALS) R = KVM_ST_ARRIVALS;
      if (((K * 2 + 127) & ~127) + 256 + ((n1 - n0 + 7) & ~7) * (KVM_ST_ARRIVALS / R) * 4 <= scratch_bytes) { sl.kind = 1; sl.R = R; sl.nchunks = (n1 - n0 + R - 1) / R; return; }
    }
    const KvmMmaLayout L = kvm_gemv_mma_layout(n1 - n0, K, r1 - r0, scratch_bytes);
    if (L.ok) { sl.kind = 3; sl.R = L.R; sl.j0 = L.KC; sl.j1 = L.ng; sl.newrow = L.nkc; sl.nchunks = L.nchunks; }      // j0 / j1 / newrow double as KC / row groups / k-chunks
  } else if (op == 135 || op == 300) {
    const int kci = a[1], vci = a[2], li = a[3], b = a[7], kvh = a[8], s = a[9], Sp = a[10], H = a[11], Hkv = a[12], hd = a[13], Tmax = a[14], fl = a[17];
    if (kci < 0 || kci >= S.nbufs || vci < 0 || vci >= S.nbufs || li < 0 || li >= S.nbufs) return;
    if (b < 0 || Hkv <= 0 || H <= 0 || H % Hkv || kvh < 0 || kvh >= Hkv || s < 0 || Sp <= 0 || s >= Sp || Tmax <= 0 || !(fl == 0 || fl == 1 || fl == 3)) return;
    const int G = H / Hkv;
    if (G > 8 || (G & (G - 1)) || !(hd == 16 || hd == 32 || hd == 64 || hd == 128)) return;
    const KvmBuf kc = sl.lb[1], vc = sl.lb[2], lens = sl.lb[3];
    if (!kc.p || !vc.p || !lens.p || kc.dtype != KVM_BF16 || vc.dtype != KVM_BF16 || lens.dtype != KVM_I32 || kc.ld != hd || vc.ld != hd || ((uintptr_t)kc.p & 15) || ((uintptr_t)vc.p & 15)) return;
    if ((long long)(b + 1) * Hkv * Tmax > kc.rows || (long long)(b + 1) * Hkv * Tmax > vc.rows || hd > kc.cols || hd > vc.cols || lens.ld != lens.cols || b >= lens.rows * lens.cols) return;
    const int p0 = ((const int*)lens.p)[b], n = p0 + 1;
    if (p0 < 0 || n > Tmax) return;
    const int chunk = (n + Sp - 1) / Sp, j0 = s * chunk, j1 = min(n, s * chunk + chunk), nk = max(j1 - j0, 0);
    if (nk * hd * 2 > KVM_ST_STAGE || kvm_attn_part_scratch(nk, G, hd) > scratch_bytes) return;
    sl.kind = 2; sl.nchunks = 2; sl.j0 = j0; sl.j1 = j1;
    sl.newrow = ((fl & 1) && j0 <= n - 1 && n - 1 < j1) ? n - 1 - j0 : -1;
  }
}

// Issue the copies of chunk `ci` of the task in `sl` as stage use `it` (front warp, lane 0; the stage is known to be free).
static __device__ void kvm_static_issue(const KvmDevState& S, const KvmStSlot& sl, const KvmRing& ring, unsigned it, int ci) {
  const uint32_t full = kvm_ring_full(ring, it), dst = ring.base_addr + kvm_ring_slot(ring, it) * KVM_ST_STAGE;
  const int32_t* a = sl.args;
  if (sl.kind == 3) {
    // stage = R weight rows x KC columns; chunk ci = (k-chunk, row group), row group inner
    const KvmBuf w = sl.lb[3];
    const int n0 = a[6], n1 = a[7], K = a[8], R = sl.R, KC = sl.j0, ng = sl.j1;
    const int kc = ci / ng, rg = ci % ng, r0 = n0 + rg * R, nr = min(R, n1 - r0);
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w.p + (size_t)kc * KC;
    kvm_mbar_expect_tx(full, (uint32_t)(nr * KC * 2));
    if (KC == K && w.ld == K) kvm_bulk_g2s(dst, wp + (size_t)r0 * w.ld, (uint32_t)(nr * K * 2), full);
    else for (int r = 0; r < nr; ++r) kvm_bulk_g2s(dst + r * KC * 2, wp + (size_t)(r0 + r) * w.ld, (uint32_t)(KC * 2), full);
  } else if (sl.kind == 1) {
    const KvmBuf w = sl.lb[3];
    const int n0 = a[6], n1 = a[7], K = a[8], R = sl.R;
    const int r0 = n0 + ci * R, nr = min(R, n1 - r0);
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w.p;
    kvm_mbar_expect_tx(full, (uint32_t)(nr * K * 2));
    if (w.ld == K) kvm_bulk_g2s(dst, wp + (size_t)r0 * w.ld, (uint32_t)(nr * K * 2), full);
    else for (int r = 0; r < nr; ++r) kvm_bulk_g2s(dst + r * K * 2, wp + (size_t)(r0 + r) * w.ld, (uint32_t)(K * 2), full);
  } else {
    const KvmBuf cb = sl.lb[ci == 0 ? 1 : 2];
    const int b = a[7], kvh = a[8], Hkv = a[12], hd = a[13], Tmax = a[14];
    const size_t base = (size_t)(b * Hkv + kvh) * Tmax;
    const int nk = max(sl.j1 - sl.j0, 0), ncopy = sl.newrow >= 0 ? nk - 1 : nk;
    const uint32_t bytes = (uint32_t)(ncopy * hd * 2);
    kvm_mbar_expect_tx(full, bytes);
    if (bytes) kvm_bulk_g2s(dst, (const __nv_bfloat16*)cb.p + (base + sl.j0) * cb.ld, bytes, full);
  }
}

__global__ void __launch_bounds__(KVM_NT + 32, 1) kvm_static_kernel(KvmStaticState T) {
  extern __shared__ __align__(1024) unsigned char kvm_smem[];
  const KvmDevState& S = T.D;
  KvmStSlot* slots = (KvmStSlot*)kvm_smem;
  int* ctl = (int*)(kvm_smem + KVM_ST_SLOTS * sizeof(KvmStSlot));          // as in the dynamic kernel: ctl[0] = TMEM base, tensor-core barriers from ctl[8]
  int* sctl = ctl + 96;                                                     // static path's own words: [0] consumer stage-use count, [1] tasks finished
  const uint32_t sbar = kvm_smem_addr(kvm_smem + KVM_ST_HDR - 128);         // stream ring barriers: full[3] | empty[3]
  const int tid = threadIdx.x;
  const bool is_front = tid >= KVM_NT;
  const int w = blockIdx.x;
  unsigned dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  if (tid < KVM_ST_SLOTS) { slots[tid].state = 0; slots[tid].task = -1; }
  if (tid == 0) { sctl[0] = 0; sctl[1] = 0; ((int*)(kvm_smem + KVM_ST_HDR - 128 - 288))[0] = 0; ((int*)(kvm_smem + KVM_ST_HDR - 128 - 288))[1] = 0; }
  kvm_tc_init(ctl, kvm_smem);
  const unsigned ring_ns = T.ring == 2 ? 2u : 3u;
  const int ring_bytes = (int)ring_ns * KVM_ST_STAGE;
  const bool use_ring = T.ring && dyn >= KVM_ST_HDR + ring_bytes + 32768;
  if (tid == 64 && use_ring) {
    for (int s = 0; s < 3; ++s) { kvm_mbar_init(sbar + 8 * s, 1); kvm_mbar_init(sbar + 64 + 8 * s, KVM_ST_ARRIVALS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  const int cache_bytes = (int)(((size_t)S.nbufs * sizeof(KvmBuf) + 1023) & ~(size_t)1023);
  const bool buf_cache = !use_ring && S.buf_cache && cache_bytes <= KVM_BUFCACHE_BYTES && dyn >= KVM_ST_HDR + KVM_BUFCACHE_BYTES + 192 * 1024;
  if (buf_cache) {
    const uint4* src = (const uint4*)S.bufs;
    uint4* dst = (uint4*)(kvm_smem + KVM_ST_HDR);
    for (int i = tid; i < S.nbufs * 2; i += KVM_NT + 32) dst[i] = src[i];
  }
  __syncthreads();
  const unsigned long long t_begin = kvm_globaltimer();
  const unsigned long long deadline = t_begin + S.timeout_ns;
  KvmRing ring;
  ring.bar0 = sbar;
  ring.ns = ring_ns;
  ring.base = kvm_smem + (use_ring ? dyn - ring_bytes : 0);
  ring.base_addr = kvm_smem_addr(ring.base);
  const int p_lo = T.prog_off[w], n = T.prog_off[w + 1] - p_lo;

  if (is_front) {
    const int lane = tid & 31;
    int fi = 0, ri = 0, ii = 0, ic = 0;        // next position to fetch / to mark ready / to stream; chunk inside the streamed task
    unsigned pit = 0;                          // stage uses issued
    int dep[5] = {-1, -1, -1, -1, -1}, dep_pos = -1;     // dependency entries of the task at `ri`
    bool stop = false;
    unsigned idle = 0;
    // one pass of the copy issuer: lane 0 issues chunks of the oldest tasks that still have copies to issue while stages are free
    auto stream_pass = [&]() -> bool {
      if (ii >= fi) return false;
      int lii = ii, lic = ic;
      unsigned lpit = pit;
      if (lane == 0) {
        for (int guard = 0; guard < 6 && lii < fi; ++guard) {
          KvmStSlot& sl = slots[lii % KVM_ST_SLOTS];
          if (sl.kind == 0) { ++lii; lic = 0; continue; }
          if (!(sl.prefetch || lii < ri)) break;             // constants may run ahead; anything else waits until the task is ready
          if (!(lpit < ring.ns || kvm_mbar_test(kvm_ring_empty(ring, lpit), kvm_ring_parity(ring, lpit) ^ 1u))) break;
          if (!sl.prefetch) asm volatile("fence.proxy.async;" ::: "memory");      // data other workers wrote with plain stores, read here by bulk copies
          kvm_static_issue(S, sl, ring, lpit, lic);
          ++lpit; ++lic;
          if (lic >= sl.nchunks) { ++lii; lic = 0; }
        }
      }
      lii = __shfl_sync(0xffffffffu, lii, 0); lic = __shfl_sync(0xffffffffu, lic, 0); lpit = __shfl_sync(0xffffffffu, lpit, 0);
      const bool moved = lii != ii || lic != ic;
      ii = lii; ic = lic; pit = lpit;
      return moved;
    };
    while (!stop && (ri < n || ii < n)) {
      bool progressed = false;
      // 1. fetch the next record into a free slot
      if (fi < n && kvm_ld_volatile_shared(&slots[fi % KVM_ST_SLOTS].state) == 0) {
        KvmStSlot& sl = slots[fi % KVM_ST_SLOTS];
        const int task = T.prog[p_lo + fi];
        const int32_t* rec = S.recs + (size_t)task * KVM_REC_WORDS;
        const int32_t w0 = rec[lane], w1 = lane < 16 ? rec[32 + lane] : 0;
        if (lane < 16) sl.desc[lane] = w0; else sl.args[lane - 16] = w0;
        if (lane < 4) sl.args[16 + lane] = w1; else if (lane < 8) ((int32_t*)&sl.aux)[lane - 4] = w1;
        if (lane == 8) sl.wait_off = w1;
        if (lane == 9) sl.wait_cnt = w1;
        if (lane == 10) sl.prefetch = w1 & 1;
        if (lane == 31) sl.task = task;
        __syncwarp();
        if (use_ring) {                                      // table entries of the buffer arguments of a streaming op, lanes in parallel
          const int op = sl.desc[0], nb = (op == 134 || op == 301) ? 6 : (op == 135 || op == 300) ? 7 : 0;
          if (lane < nb) {
            const int idx = sl.args[lane];
            KvmBuf e; e.p = nullptr; e.rows = e.cols = e.ld = 0; e.dtype = 0; e.reserved[0] = e.reserved[1] = 0;
            if (idx >= 0 && idx < S.nbufs) e = S.bufs[idx];
            sl.lb[lane] = e;
          }
          __syncwarp();
        }
        if (lane == 0) {
          if (use_ring) kvm_static_geometry(S, sl, (int)dyn - KVM_ST_HDR - ring_bytes); else { sl.kind = 0; sl.nchunks = 0; }
          sl.state = 1;
        }
        __syncwarp();
        ++fi; progressed = true;
      }
      // 2. stream ahead: chunks of the oldest tasks that still have copies to issue, as many as there are free stages
      if (stream_pass()) progressed = true;
      // 3. dependencies of the next task to become ready: its entries are held in registers (up to five per lane) and polled with
      //    plain loads, all in flight together; one acquire fence once they are all met
      if (ri < fi) {
        KvmStSlot& sl = slots[ri % KVM_ST_SLOTS];
        if (dep_pos != ri) {
          const int off = sl.wait_off, cnt = sl.wait_cnt;
#pragma unroll
          for (int j = 0; j < 5; ++j) dep[j] = lane + 32 * j < cnt ? T.waits[off + lane + 32 * j] : -1;
          dep_pos = ri;
        }
        int seen[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) seen[j] = dep[j] >= 0 ? kvm_ld_relaxed(&T.progress[dep[j] >> KVM_ST_WAIT_BITS]) : 0;
        // while those loads are in flight (an L2 round trip, longer when the memory system is saturated by the copies) keep
        // refilling stages: a freed stage must not wait for the poll
        if (ii < fi)
          for (int sp = 0; sp < 6; ++sp) if (stream_pass()) progressed = true;
        bool met = true;
#pragma unroll
        for (int j = 0; j < 5; ++j) if (dep[j] >= 0 && seen[j] < (dep[j] & ((1 << KVM_ST_WAIT_BITS) - 1))) met = false;
        if (__all_sync(0xffffffffu, met)) {
          __threadfence();                                   // acquire: what the finished predecessors wrote is visible to this CTA's compute group
          if (lane == 0) { S.indeg[sl.task] = 0; sl.state = 2; }     // every predecessor's completion was observed
          __syncwarp();
          ++ri; progressed = true;
        }
      }
      // 4. failure / stall
      if (!progressed) {
        if ((++idle & 63u) == 0) {
          int e = 0;
          if (lane == 0) e = *(volatile int*)&S.err->code;
          e = __shfl_sync(0xffffffffu, e, 0);
          if (e != 0) stop = true;
          else if (kvm_globaltimer() > deadline) {
            if (lane == 0) kvm_dev_fail(S, KVM_ERR_TIMEOUT, ri < n ? T.prog[p_lo + ri] : -1, ri, fi);
            stop = true;
          }
        }
      } else idle = 0;
    }
    // leave: the compute group takes slots in order; the first one that is not ready tells it to go
    if (stop) {
      if (lane == 0) {
        for (int k = 0; k < KVM_ST_SLOTS; ++k) {
          KvmStSlot& sl = slots[(ri + k) % KVM_ST_SLOTS];
          if (kvm_ld_volatile_shared(&sl.state) != 2) { sl.state = 3; break; }
        }
      }
    }
    sctl[2] = (int)pit;
  } else {
    KvmCtx c;
    c.nbufs = S.nbufs; c.err = S.err; c.cfg_flags = S.cfg_flags; c.ctl = ctl; c.tmaps = S.tmaps; c.pair = -1; c.engine = 0; c.gemm_seq = 0;
    c.rope_cache = (float*)(kvm_smem + KVM_ST_HDR - 128 - 288);
    c.yield_word = nullptr; c.yield_count = nullptr; c.q_head = c.q_tail = nullptr;      // program order: a waiting task waits in place
    c.deadline = deadline - S.timeout_ns / 8;      // a task's own wait gives up (and names itself) before the launch's stall limit does
    c.bufs = buf_cache ? (const KvmBuf*)(kvm_smem + KVM_ST_HDR) : S.bufs;
    const int used = KVM_ST_HDR + (buf_cache ? cache_bytes : 0);
    c.smem = kvm_smem + used;
    c.smem_bytes = (int)dyn - used - (use_ring ? ring_bytes : 0);
    unsigned cit = 0;
    int finished = 0;
    for (int i = 0; i < n; ++i) {
      KvmStSlot& sl = slots[i % KVM_ST_SLOTS];
      if (tid == 0) {
        unsigned polls = 0;
        int st;
        while ((st = kvm_ld_volatile_shared(&sl.state)) < 2) {
          if ((++polls & 1023u) == 0 && kvm_globaltimer() > deadline + S.timeout_ns) { st = 3; break; }      // the front warp always answers first
        }
        sl.go = st == 3 ? 0 : (*(volatile int*)&S.err->code == 0 ? 1 : 2);
      }
      kvm_sync();
      const int go = kvm_ld_volatile_shared(&sl.go);
      if (go == 0) break;
      const int task = sl.task;
      c.task = task;
      unsigned long long t_task = 0;
      if (tid == 0 && S.trace) { t_task = kvm_globaltimer(); S.t_start[task] = t_task; sctl[3] = 0; }
      const int op = sl.desc[0], kind = sl.kind, nch = sl.nchunks;
      if (kind == 1) kvm_gemv_ring(c, sl.args, sl.lb, ring, cit, sl.R, nch, deadline, t_task, S.trace ? sctl + 3 : nullptr);
      else if (kind == 3) kvm_gemv_mma_ring(c, sl.args, sl.lb, op == 301, ring, cit, sl.newrow, deadline, t_task, S.trace ? sctl + 3 : nullptr);
      else if (kind == 2) kvm_attn_part_ring(c, sl.args, sl.lb, op == 300, ring, cit, sl.j0, sl.j1, sl.newrow, deadline, t_task, S.trace ? sctl + 3 : nullptr);
      else if (op != 0 && go == 1) kvm_dispatch(c, op, sl.args, sl.aux);
      cit += (unsigned)nch;
      // Results that a later bulk copy or TMA load may read (cache rows appended by an attention split, operands of tensor-core ops)
      // need the writer's generic-to-async proxy fence.  A streamed GEMV writes activations only, which every consumer reads with
      // plain loads: it skips the fence (it waits for the task's global stores, about a microsecond per task).
      if (kind != 1 && kind != 3) asm volatile("fence.proxy.async;" ::: "memory");
      kvm_sync();
      if (tid == 0) {
        if (S.trace) { S.t_end[task] = kvm_globaltimer(); S.t_smid[task] = (int)kvm_smid() | (sctl[3] << 8); }     // bits 8.. : detail of a streamed task
        atomicAdd(&S.exec_count[task], 1);                   // no result needed: nothing waits for the old value
        const int pv = sl.desc[10];
        if (pv >= 0) {                                       // publish (include/mvm_task_abi.h:20-23): old + 1, else VERSION_GAP
          if (pv >= S.nvars) kvm_dev_fail(S, KVM_ERR_BAD_VAR, task, pv);
          else {
            __threadfence();                                 // the task's writes before its version
            const int ver = sl.desc[11] + S.ver_off[pv];
            if (atomicCAS(&S.versions[pv], ver - 1, ver) != ver - 1) kvm_dev_fail(S, KVM_ERR_VERSION_GAP, task, pv, ver);
          }
        }
        kvm_st_release(&T.progress[w], i + 1);               // release at gpu scope: the CTA's writes (ordered before this thread by the barrier) come first
        sctl[0] = (int)cit;
        sl.state = 0;
      }
      ++finished;
    }
    if (tid == 0) { sctl[1] = finished; atomicAdd(S.done, finished); }
  }
  __syncthreads();
  // copies issued but never consumed (an early exit): wait for them, bounded, before the shared memory goes away
  if (use_ring && tid == KVM_NT) {
    const unsigned pit = (unsigned)sctl[2], cit = (unsigned)sctl[0];
    for (unsigned it = cit; it < pit; ++it) {
      const uint32_t bar = kvm_ring_full(ring, it), par = kvm_ring_parity(ring, it);
      const unsigned long long t0 = kvm_globaltimer();
      unsigned spins = 0;
      while (!kvm_mbar_test(bar, par)) if ((++spins & 63u) == 0 && kvm_globaltimer() - t0 > 50000000ull) break;      // 50 ms: a bulk copy lands in microseconds
    }
  }
  __syncthreads();
  kvm_tc_fini(ctl);
}

// Arm kernel of the static path: progress words and witnesses cleared, version offsets taken.
__global__ void kvm_static_arm_kernel(KvmStaticState T, int workers) {
  const KvmDevState& S = T.D;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < S.nt) { S.indeg[i] = S.tasks[i].indegree; S.exec_count[i] = 0; }
  if (i < workers) T.progress[i] = 0;
  if (i < S.nvars) S.ver_off[i] = S.versions[i] - S.ver_base[i];
}
