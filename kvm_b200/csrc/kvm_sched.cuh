// The persistent executor kernel: one worker CTA per SM, each made of a scheduler warp and KVM_NT compute threads.
//
//   scheduler warp   claims ready-queue tickets, fetches the 16-word descriptor and the argument words of the next task into a
//                    two-entry shared-memory slot ring (so the next task is staged while the current one computes), and, when
//                    the compute group reports a task finished, publishes its version, decrements the dependency counters
//                    of its successors (lanes in parallel) and enqueues or parks the ones that reach zero.
//   compute group    waits for a full slot, dispatches the op body (SIMT ops use all 16 warps; tcgen05 GEMM / attention tasks
//                    split them into TMA-producer, MMA-issuer and epilogue roles), fences, and hands the slot back.
//
// What it implements of the reference (include/mvm_exec.cuh, include/mvm_sched.cuh): mvm_worker / mvm_run_task / mvm_post_task
// (:614-801), the successor release with continuation (:690-713), mvm_publish / park lists (:523-565), the ready queue
// (mvm_sched.cuh:107-246, here a ticketed ring: one atomic per push and per pop) and first-error-wins failure (:260-266).
// Admission differs by design: the whole batch is resident in HBM before launch (descriptor table, CSR successors, args),
// dependency counters are armed by a tiny kernel, so no admitter CTA is needed.
// Every wait has a time limit after which the kernel records KVM_ERR_TIMEOUT and all workers leave.
#pragma once
#include "kvm_state.cuh"

#define KVM_NSLOT 2               // tasks a worker holds at most: one running and one staged behind it (more slots let a worker hoard ready tasks while others idle)
struct KvmSlot {
  int task;                   // -1 = leave
  int state;                  // 0 free, 1 full, 2 finished (awaiting release)
  int pair;                   // partner task run together with `task` (stacked GEMM tiles), or -1
  int go;                     // written by compute thread 0 before the group's barrier: 0 leave, 1 run the op body, 2 skip it (an error is recorded)
  int seq;                    // fill counter for the engine warps: 2k - 1 while fill k is being written, 2k once it is complete
  int kind;                   // 1: a tensor-core GEMM tile whose mainloop the engine warps run; -1: leave; else 0
  int pad[2];
  int32_t desc[16];
  int32_t args[KVM_MAX_ARGS];
  int4 aux;
};

__device__ __forceinline__ void kvm_push_ready(const KvmDevState& S, int task) {
  const int c = kvm_class_of(S.tasks[task].priority);
  unsigned t = atomicAdd(&S.tail[c], 1u);
  if (t >= (unsigned)S.ring_cap) { kvm_dev_fail(S, KVM_ERR_QUEUE_OVERFLOW, task, (int)t); return; }
  kvm_st_release(&S.ring[(size_t)c * S.ring_cap + t], task + 1);
}
// Pop, highest class first.  Tickets are taken with atomicAdd (no compare-and-swap convoy when many workers are idle) but only
// where head < tail was just seen; a ticket that lost that race and points past the tail is HELD: the worker keeps polling its
// cell while it goes on serving the other classes, so a held ticket can never starve anyone.  held[c] = ring cell or -1.
// `min_depth`: a worker that is still running a task stages its next one only while at least that many tasks are queued
// (one for every worker): with fewer, the queued tasks are left to the idle workers instead of waiting behind a running one.
// Returns task or -1.
__device__ __forceinline__ int kvm_try_pop(const KvmDevState& S, int (&held)[KVM_NCLASS], unsigned min_depth, unsigned& depth_out) {
  depth_out = 0;
#pragma unroll
  for (int c = KVM_NCLASS - 1; c >= 0; --c)
    if (held[c] >= 0) {
      const int v = kvm_ld_acquire(&S.ring[held[c]]);
      if (v > 0) { held[c] = -1; return v - 1; }
    }
  unsigned t[4], h[4];
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "l"(S.head) : "memory");
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3]) : "l"(S.tail) : "memory");
  unsigned depth = 0;
#pragma unroll
  for (int c = 0; c < KVM_NCLASS; ++c) depth += t[c] > h[c] ? t[c] - h[c] : 0u;
  depth_out = depth;
  if (depth < min_depth) return -1;
#pragma unroll
  for (int c = KVM_NCLASS - 1; c >= 0; --c)
    if (held[c] < 0 && h[c] < t[c]) {
      const unsigned tk = atomicAdd(&S.head[c], 1u);
      if (tk >= (unsigned)S.ring_cap) continue;
      const int cell = (int)((size_t)c * S.ring_cap + tk);
      const int v = kvm_ld_acquire(&S.ring[cell]);
      if (v > 0) return v - 1;
      held[c] = cell;                      // its pusher is one store away, or the race was lost: look again next pass
    }
  return -1;
}

// Push `task` onto the parked list of `var` (lock-free stack).
__device__ __forceinline__ void kvm_park_push(const KvmDevState& S, int task, int var) {
  int old = *(volatile int*)&S.park_head[var];
  while (true) {
    S.park_next[task] = old;
    __threadfence();
    const int prev = atomicCAS(&S.park_head[var], old, task);
    if (prev == old) break;
    old = prev;
  }
}
// Re-examine the tasks parked on `var`: the list is detached atomically (so each waiter is in exactly one scanner's hands),
// satisfied waiters are enqueued, the rest pushed back; if the version moved meanwhile, look again.
static __device__ void kvm_scan_parked(const KvmDevState& S, int var) {
  for (int round = 0; round < 1024; ++round) {
    const int v0 = kvm_ld_acquire(&S.versions[var]);
    int list = atomicExch(&S.park_head[var], -1);
    bool reparked = false;
    while (list != -1) {
      const int nxt = S.park_next[list];
      if (v0 >= S.tasks[list].wait_ver + S.ver_off[var]) kvm_push_ready(S, list);
      else { kvm_park_push(S, list, var); reparked = true; }
      list = nxt;
    }
    __threadfence();
    if (!reparked || kvm_ld_acquire(&S.versions[var]) == v0) return;
  }
}
// Park, then look again: a publish that landed between the caller's check and the push is not lost (the Dekker pattern of
// the reference's mvm_release_task, include/mvm_exec.cuh:544-556).
__device__ __forceinline__ void kvm_park(const KvmDevState& S, int task, int var, int ver) {
  kvm_park_push(S, task, var);
  __threadfence();
  if (kvm_ld_acquire(&S.versions[var]) >= ver) kvm_scan_parked(S, var);
}
// A task whose predecessors have all finished: enqueue it, or park it on its version wait.
__device__ __forceinline__ void kvm_release_task(const KvmDevState& S, int task) {
  const int wv = S.tasks[task].wait_var;
  if (wv >= 0) {
    if (wv >= S.nvars) { kvm_dev_fail(S, KVM_ERR_BAD_VAR, task, wv); return; }
    const int want = S.tasks[task].wait_ver + S.ver_off[wv];
    if (kvm_ld_acquire(&S.versions[wv]) < want) { kvm_park(S, task, wv, want); return; }
  }
  kvm_push_ready(S, task);
}

// Arm kernel: dependency counters from the descriptors, roots into the ring, counters cleared.
__global__ void kvm_arm_kernel(KvmDevState S) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < S.nt) {
    S.indeg[i] = S.tasks[i].indegree;
    S.exec_count[i] = 0;
    S.claim[i] = 0;
    S.park_next[i] = -1;
  }
  for (int j = i; j < S.ring_cap; j += gridDim.x * blockDim.x)       // a class's ring holds every task once, plus the re-queues of tasks that may yield
#pragma unroll
    for (int c = 0; c < KVM_NCLASS; ++c) S.ring[(size_t)c * S.ring_cap + j] = 0;
  if (i < S.nvars) { S.park_head[i] = -1; S.ver_off[i] = S.versions[i] - S.ver_base[i]; }
}
__global__ void kvm_roots_kernel(KvmDevState S) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < S.nt && S.tasks[i].indegree == 0) kvm_release_task(S, i);
}

// The scheduler warp's share of finishing `task`: publish its version, then release its successors.
// The successors are taken eight per lane at a time and every step is done for all of them before the next one starts: the
// index loads, the counter decrements, the look at the ready ones' descriptors, and one ticket grab per priority class for the
// whole warp - so a fan-out of a few hundred costs the same handful of memory round trips as a fan-out of one.
// Returns a continuation task (>= 0) when the caller may run one directly, else -1.
#define KVM_REL_U 8
static __device__ int kvm_finish_task(const KvmDevState& S, int task, int so, int sc, int pv, int pver, bool want_cont) {
  const int lane = threadIdx.x & 31;
  __threadfence();             // pairs with the compute group's fence before it flagged the slot finished
  if (pv >= 0) {
    if (lane == 0) {
      if (pv >= S.nvars) kvm_dev_fail(S, KVM_ERR_BAD_VAR, task, pv);
      else {
        __threadfence();
        const int ver = pver + S.ver_off[pv];
        if (atomicCAS(&S.versions[pv], ver - 1, ver) != ver - 1) kvm_dev_fail(S, KVM_ERR_VERSION_GAP, task, pv, ver);
        __threadfence();
        kvm_scan_parked(S, pv);
      }
    }
    __syncwarp();
  }
  int cont = -1;
  for (int k0 = 0; k0 < sc; k0 += 32 * KVM_REL_U) {
    int s[KVM_REL_U], kind[KVM_REL_U];       // kind: -1 nothing, 0..3 enqueue in that class, 4 version wait
#pragma unroll
    for (int u = 0; u < KVM_REL_U; ++u) { const int k = k0 + u * 32 + lane; s[u] = k < sc ? S.succ[so + k] : -1; }
#pragma unroll
    for (int u = 0; u < KVM_REL_U; ++u) {
      kind[u] = -1;
      if (s[u] >= 0) {
        const int meta = s[u] >> KVM_SUCC_BITS;
        s[u] &= (1 << KVM_SUCC_BITS) - 1;
        const int old = atomicSub(&S.indeg[s[u]], 1);
        if (old == 1) kind[u] = (meta & 4) ? 4 : (meta & 3);
        else if (old <= 0) kvm_dev_fail(S, KVM_ERR_BAD_TASK, s[u], old);
      }
    }
    // One fence for the whole batch: whoever made a counter reach zero has seen every other predecessor's decrement, and those
    // came after their data; the ring cells below are then plain stores (their readers load with acquire).
    __threadfence();
    // the continuation: the first ready successor without a version wait (no queue hop)
#pragma unroll
    for (int u = 0; u < KVM_REL_U; ++u) {
      const unsigned mc = __ballot_sync(0xffffffffu, kind[u] >= 0 && kind[u] < 4 && want_cont && cont < 0);
      if (mc) {
        const int take = __ffs(mc) - 1;
        cont = __shfl_sync(0xffffffffu, s[u], take);
        if (lane == take) kind[u] = -1;
      }
    }
    // enqueue: one ticket grab per class for the warp
#pragma unroll
    for (int c = KVM_NCLASS - 1; c >= 0; --c) {
      int n = 0;
#pragma unroll
      for (int u = 0; u < KVM_REL_U; ++u) n += kind[u] == c;
      if (!__any_sync(0xffffffffu, n > 0)) continue;
      int incl = n;                                           // inclusive prefix sum over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      unsigned base = 0;
      if (lane == 0) base = atomicAdd(&S.tail[c], (unsigned)total);
      base = __shfl_sync(0xffffffffu, base, 0);
      unsigned t = base + (unsigned)(incl - n);
#pragma unroll
      for (int u = 0; u < KVM_REL_U; ++u)
        if (kind[u] == c) {
          if (t >= (unsigned)S.ring_cap) kvm_dev_fail(S, KVM_ERR_QUEUE_OVERFLOW, s[u], (int)t);
          else kvm_st_relaxed(&S.ring[(size_t)c * S.ring_cap + t], s[u] + 1);
          ++t;
        }
    }
#pragma unroll
    for (int u = 0; u < KVM_REL_U; ++u) if (kind[u] == 4) kvm_release_task(S, s[u]);     // version waits: check, park or enqueue
  }
  if (lane == 0) atomicAdd(S.done, 1);
  return cont;
}
#define KVM_EXEC_THREADS (KVM_NT + 96)      // 16 compute warps, the scheduler warp, two engine warps (TMA producer, MMA issuer)
__global__ void __launch_bounds__(KVM_EXEC_THREADS, 1) kvm_exec_kernel(KvmDevState S) {
  extern __shared__ __align__(1024) unsigned char kvm_smem[];
  KvmSlot* slots = (KvmSlot*)kvm_smem;                 // the slot ring
  int* ctl = (int*)(kvm_smem + KVM_NSLOT * sizeof(KvmSlot));   // ctl[0] = TMEM base, ctl[1..] scratch
  static_assert(KVM_NSLOT * sizeof(KvmSlot) + 96 * sizeof(int) + 288 <= KVM_EXEC_SMEM_HDR, "header too small");      // slots | control words | ... | rope cache (288)
  const int tid = threadIdx.x;
  const bool is_sched = tid >= KVM_NT && tid < KVM_NT + 32;
  const int engine_role = tid == KVM_NT + 32 ? 1 : tid == KVM_NT + 64 ? 2 : 0;      // one thread each: TMA producer, MMA issuer
  if (tid < KVM_NSLOT) { slots[tid].state = 0; slots[tid].task = -1; slots[tid].seq = 0; slots[tid].kind = 0; }
  if (tid == 0) ctl[KVM_CTL_YIELD] = 0;
  if (tid == 0) { ((int*)(kvm_smem + KVM_EXEC_SMEM_HDR - 288))[0] = 0; ((int*)(kvm_smem + KVM_EXEC_SMEM_HDR - 288))[1] = 0; }      // rope cache: no key yet
  unsigned dyn;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
  kvm_tc_init(ctl, kvm_smem);                          // TMEM allocation + mbarrier init (whole CTA)
  // The buffer table is copied into shared memory once per launch when it fits: every task starts by looking up its buffers, and
  // from here that is a shared-memory read instead of a round trip to L2.
  const int cache_bytes = (int)(((size_t)S.nbufs * sizeof(KvmBuf) + 1023) & ~(size_t)1023);      // whole KB: the op scratch keeps its 1024-byte alignment
  const bool buf_cache = S.buf_cache && cache_bytes <= KVM_BUFCACHE_BYTES && dyn >= KVM_EXEC_SMEM_HDR + KVM_BUFCACHE_BYTES + 192 * 1024;
  if (buf_cache) {
    const uint4* src = (const uint4*)S.bufs;
    uint4* dst = (uint4*)(kvm_smem + KVM_EXEC_SMEM_HDR);
    for (int i = tid; i < S.nbufs * 2; i += KVM_EXEC_THREADS) dst[i] = src[i];
  }
  __syncthreads();
  const unsigned long long t_begin = kvm_globaltimer();
  const int used_hdr = KVM_EXEC_SMEM_HDR + (buf_cache ? cache_bytes : 0);
  const bool engine_on = S.engine && (int)dyn - used_hdr >= KVM_TCE_STAGING + KVM_TCE_STAGES * KVM_TC_STAGE_BYTES;

  if (is_sched) {
    const int lane = tid & 31;
    int fill = 0;              // slot to fill next
    int drain = 0;             // slot whose completion is due next (tasks finish in slot order)
    int inflight = 0;          // slots handed to the compute group and not yet released
    int ticket = -1;           // >= 0 while this worker holds an unfilled ticket
    int held[KVM_NCLASS] = {-1, -1, -1, -1};
    int nfill = 0;             // slots filled so far (fill k goes to slot (k - 1) % KVM_NSLOT)

    int cont = -1;             // continuation ready to be staged
    bool stop = false;
    unsigned polls = 0;
    while (true) {
      bool progressed = false;
      // 1. a task that yielded: back to the end of its class's queue, nothing released, the exactly-once witness taken back
      if (inflight > 0 && kvm_ld_volatile_shared(&slots[drain].state) == 3) {
        __syncwarp();
        if (lane == 0) {
          const int t = slots[drain].task;
          atomicSub(&S.exec_count[t], 1);
          __threadfence();
          kvm_push_ready(S, t);
          slots[drain].state = 0;
        }
        __syncwarp();
        drain = (drain + 1) % KVM_NSLOT; --inflight; progressed = true;
      }
      // 1b. a finished task?
      if (inflight > 0 && kvm_ld_volatile_shared(&slots[drain].state) == 2) {
        __syncwarp();
        const int32_t* dd = slots[drain].desc;
        const bool wc = cont < 0 && ticket < 0 && !stop;
        const int c2 = kvm_finish_task(S, slots[drain].task, dd[1], dd[2], dd[10], dd[11], wc);
        if (c2 >= 0) cont = c2;
        const int pr = slots[drain].pair;
        if (pr >= 0) {                                       // the partner tile finished with it
          const int32_t w = lane < 16 ? ((const int32_t*)&S.tasks[pr])[lane] : 0;
          const int c4 = kvm_finish_task(S, pr, __shfl_sync(0xffffffffu, w, 1), __shfl_sync(0xffffffffu, w, 2), __shfl_sync(0xffffffffu, w, 10),
                                         __shfl_sync(0xffffffffu, w, 11), wc && cont < 0);
          if (c4 >= 0) cont = c4;
        }
        __syncwarp();
        if (lane == 0) slots[drain].state = 0;
        __syncwarp();
        drain = (drain + 1) % KVM_NSLOT; --inflight; progressed = true;
      }
      // 2. stage the next task if a slot is free
      if (!stop && inflight < KVM_NSLOT) {
        int task = -1;
        unsigned depth = 0;                 // tasks queued when this one was popped (0 for a continuation)
        if (cont >= 0) { task = cont; cont = -1; }
        else {
          int tk = -1, hold = 0;
          unsigned dp = 0;
          if (lane == 0) { tk = kvm_try_pop(S, held, inflight > 0 ? (unsigned)inflight * gridDim.x : 1u, dp); hold = (held[0] & held[1] & held[2] & held[3]) >= 0 ? 1 : ((held[0] >= 0) | (held[1] >= 0) | (held[2] >= 0) | (held[3] >= 0)); }
          task = __shfl_sync(0xffffffffu, tk, 0);
          ticket = __shfl_sync(0xffffffffu, hold, 0) ? 0 : -1;      // ticket >= 0 now only means: this worker holds a ticket (no continuation then)
          depth = __shfl_sync(0xffffffffu, dp, 0);
        }
        if (task >= 0) {
          // one fetch: the task's record holds descriptor, argument words and path selector side by side
          // the exactly-once witness is taken here (its round trip overlaps the record fetch), not by the compute group
          const int seen = lane == 0 ? atomicAdd(&S.exec_count[task], 1) : 0;
          const int32_t* rec = S.recs + (size_t)task * KVM_REC_WORDS;
          const int32_t w0 = rec[lane], w1 = lane < 8 ? rec[32 + lane] : 0;
          // Stacked GEMM tiles: a tensor-core tile whose partner (same product, rows 128 further or nearer; path selector word 3)
          // is ready too is run together with it as one 256 x 256 tile.  Either ticket may come first: whoever takes a tile's
          // claim word runs it; a ticket whose tile is already taken is dropped.
          int pair = -1;
          bool drop = false;
          const int ax = __shfl_sync(0xffffffffu, w1, 4), aw = __shfl_sync(0xffffffffu, w1, 7), opid = __shfl_sync(0xffffffffu, w0, 0);
          if (ax == 1 && aw > 0) {
            int v = 0;
            if (lane == 0) {
              if (atomicCAS(&S.claim[task], 0, 1) != 0) v = -2;
              else if (depth >= (unsigned)S.pair_depth && kvm_ld_acquire(&S.indeg[aw - 1]) == 0 && atomicCAS(&S.claim[aw - 1], 0, 1) == 0) v = aw;
            }
            v = __shfl_sync(0xffffffffu, v, 0);
            drop = v == -2;
            pair = v > 0 ? v - 1 : -1;
          }
          if (drop) { if (lane == 0) atomicSub(&S.exec_count[task], 1); progressed = true; continue; }      // not run here: its partner's worker runs it
          if (lane == 0) {
            if (seen != 0) kvm_dev_fail(S, KVM_ERR_DOUBLE_EXEC, task);
            if (pair >= 0) atomicAdd(&S.exec_count[pair], 1);      // counted only: the claim word is what makes a stacked tile run once
          }
          KvmSlot& sl = slots[fill];
          ++nfill;
          if (lane == 0) { *(volatile int*)&sl.seq = 2 * nfill - 1; __threadfence_block(); }
          __syncwarp();
          if (lane < 16) sl.desc[lane] = w0; else sl.args[lane - 16] = w0;
          if (lane < 4) sl.args[16 + lane] = w1; else if (lane < 8) ((int32_t*)&sl.aux)[lane - 4] = w1;
          if (lane == 31) { sl.task = task; sl.pair = pair; }
          if (lane == 30) sl.kind = (engine_on && pair < 0 && opid == 122 && ax == 1) ? 1 : 0;      // host-planned tensor-core tile: the engine warps run its mainloop
          __threadfence();       // gpu scope: the predecessors' data must be visible to this CTA's compute group (and its engine warps)
          __syncwarp();
          if (lane == 0) { *(volatile int*)&sl.seq = 2 * nfill; __threadfence_block(); sl.state = 1; }
          fill = (fill + 1) % KVM_NSLOT; ++inflight; progressed = true;
        }
      }
      // 3. termination / failure / stall
      if (!progressed) {
        // An idle worker mostly watches the queue (step 2); the global done / error words are looked at every 2nd idle pass: often
        // enough that a short launch (one segment of a tensor-parallel token) does not sit idle for microseconds before it ends.
        if ((++polls & 1u) == 0 || stop) {
          int d = 0, e = 0;
          if (lane == 0) { d = kvm_ld_acquire(S.done); e = *(volatile int*)&S.err->code; }
          d = __shfl_sync(0xffffffffu, d, 0); e = __shfl_sync(0xffffffffu, e, 0);
          if (d >= S.nt || e != 0) stop = true;
          if (stop && inflight == 0) break;
          if ((polls & 255u) == 0 && kvm_globaltimer() - t_begin > S.timeout_ns) {
            if (lane == 0) kvm_dev_fail(S, KVM_ERR_TIMEOUT, ticket, d, inflight);
            stop = true;
            if (inflight == 0) break;
          }
        }
      } else polls = 0;
    }
    // tell the compute group to leave: it consumes slots in order, `fill` is the next one it looks at
    if (lane == 0) {
      KvmSlot& sl = slots[fill];
      ++nfill;
      *(volatile int*)&sl.seq = 2 * nfill - 1; __threadfence_block();
      sl.task = -1; sl.kind = -1;
      __threadfence_block();
      *(volatile int*)&sl.seq = 2 * nfill; __threadfence_block();
      sl.state = 1;
    }
  } else if (tid >= KVM_NT) {
    // ---- engine warps: one thread issues the TMA loads, one the MMAs, of every tensor-core GEMM tile, in the order the slots are filled
    if (engine_role && engine_on) {
      const uint32_t ring0 = kvm_smem_addr(kvm_smem + used_hdr + KVM_TCE_STAGING);
      kvm_tc_fence_after();
      const uint32_t tmem = *(volatile uint32_t*)(ctl + KVM_CTL_TMEM);
      const unsigned long long t_limit = t_begin + 2 * S.timeout_ns;
      uint32_t it = 0, g = 0;
      bool prev_tile = false;            // the task before this one is one of the engine's tiles (it only uses the staging area)
      for (int k = 1;; ++k) {
        KvmSlot& sl = slots[(k - 1) % KVM_NSLOT];
        int sq;
        unsigned polls = 0;
        while ((sq = *(volatile int*)&sl.seq) < 2 * k) {
          if ((++polls & 1023u) == 0 && kvm_globaltimer() > t_limit) { sq = -1; break; }
        }
        if (sq < 0) break;                                   // the scheduler always posts the leave message first
        if (sq > 2 * k) { prev_tile = false; continue; }     // filled, run and recycled meanwhile: not a tile of ours (ours wait for us)
        const int kind = *(volatile int*)&sl.kind;
        int32_t a[12];
#pragma unroll
        for (int j = 6; j < 12; ++j) a[j] = *(volatile int32_t*)&sl.args[j];
        int4 aux;
        aux.x = 1; aux.y = *(volatile int*)&sl.aux.y; aux.z = *(volatile int*)&sl.aux.z; aux.w = 0;
        __threadfence_block();
        if (*(volatile int*)&sl.seq != 2 * k) { prev_tile = false; continue; }
        if (kind < 0) break;
        if (kind != 1) { prev_tile = false; continue; }
        bool ok = true;
        if (engine_role == 1) {
          if (!prev_tile && k > 1) {
            // whatever the compute group runs before this tile may use the whole scratch: wait until it has finished
            KvmSlot& pv = slots[(k - 2) % KVM_NSLOT];
            polls = 0;
            while (*(volatile int*)&pv.seq == 2 * (k - 1) && *(volatile int*)&pv.state == 1) {
              if ((++polls & 1023u) == 0 && (kvm_globaltimer() > t_limit || *(volatile int*)&S.err->code != 0)) { ok = false; break; }
            }
          }
          if (ok) ok = kvm_tce_produce(ctl, ring0, S.tmaps, a, aux, it, S.err);
        } else ok = kvm_tce_mma(ctl, ring0, tmem, a, it, g, S.err);
        if (!ok) { if (*(volatile int*)&S.err->code == 0) kvm_dev_fail(S, KVM_ERR_TIMEOUT, sl.task, 3122, engine_role); break; }
        ++g; prev_tile = true;
      }
    }
  } else {
    KvmCtx c;
    c.nbufs = S.nbufs; c.err = S.err; c.cfg_flags = S.cfg_flags; c.ctl = ctl; c.tmaps = S.tmaps;
    c.bufs = buf_cache ? (const KvmBuf*)(kvm_smem + KVM_EXEC_SMEM_HDR) : S.bufs;
    const int used = used_hdr;
    c.smem = kvm_smem + used; c.smem_bytes = (int)dyn - used;
    c.engine = engine_on ? 1 : 0; c.gemm_seq = 0;
    c.rope_cache = (float*)(kvm_smem + KVM_EXEC_SMEM_HDR - 288);
    c.yield_word = ctl + KVM_CTL_YIELD; c.q_head = S.head; c.q_tail = S.tail;
    c.deadline = t_begin + S.timeout_ns - S.timeout_ns / 8;      // a task's own wait gives up (and names itself) before the launch's stall limit does
    unsigned tiles = 0;
    int cur = 0;
    while (true) {
      KvmSlot& sl = slots[cur];
      // Whether this slot is taken, and whether its op body runs, is decided ONCE per CTA: thread 0 looks at the slot state and at
      // the device's error word and leaves its verdict in the slot's `go` word; after the barrier every thread branches on that
      // shared word only.  (A per-thread look at the global error word could split the group: the op bodies contain barriers
      // over all KVM_NT threads, so warps that skipped the body and warps that entered it would wait for each other forever.)
      if (tid == 0) {
        unsigned polls = 0;
        bool full = true;
        while (kvm_ld_volatile_shared(&sl.state) != 1) {
          if ((++polls & 1023u) == 0 && kvm_globaltimer() - t_begin > 2 * S.timeout_ns) { full = false; break; }   // the scheduler always answers first
        }
        sl.go = !full ? 0 : (*(volatile int*)&S.err->code == 0 ? 1 : 2);      // 0 leave, 1 run the op, 2 finish the task without running it
      }
      kvm_sync();
      const int go = kvm_ld_volatile_shared(&sl.go);
      if (go == 0) break;
      const int task = sl.task;
      if (task < 0) break;
      c.task = task; c.pair = sl.pair;
      if (tid == 0) {
        const int wv = sl.desc[8];
        if (wv >= 0 && wv < S.nvars && kvm_ld_acquire(&S.versions[wv]) < sl.desc[9] + S.ver_off[wv]) kvm_dev_fail(S, KVM_ERR_WAIT_VIOLATION, task, wv);
        if (S.trace) {
          S.t_start[task] = kvm_globaltimer(); S.t_smid[task] = (int)kvm_smid();
          if (c.pair >= 0) { S.t_start[c.pair] = S.t_start[task]; S.t_smid[c.pair] = S.t_smid[task]; }
        }
      }
      const int op = sl.desc[0];
      const bool tile = sl.kind == 1;
      c.gemm_seq = tiles;
      c.yield_count = S.claim + task;           // the claim word of a task that is not a stacked GEMM tile is free: it counts the task's yields
      if (op != 0 && go == 1) kvm_dispatch(c, op, sl.args, sl.aux);
      if (tile) ++tiles;
      // this task's generic-proxy writes (global results, shared scratch) ordered before any later TMA access to them
      asm volatile("fence.proxy.async;" ::: "memory");
      kvm_sync();                       // every thread's writes happen before thread 0's fence below (barrier, then a cumulative gpu-scope fence)
      if (tid == 0) {
        if (S.trace) { S.t_end[task] = kvm_globaltimer(); if (c.pair >= 0) S.t_end[c.pair] = S.t_end[task]; }
        __threadfence();
        const int y = ctl[KVM_CTL_YIELD];
        ctl[KVM_CTL_YIELD] = 0;
        sl.state = y ? 3 : 2;                    // 3: the task wrote nothing and wants to run again later
      }
      cur = (cur + 1) % KVM_NSLOT;
    }
  }
  __syncthreads();
  kvm_tc_fini(ctl);
}
