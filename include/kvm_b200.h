/* libkvm_b200.so: C ABI of the B200 executor for Magni VM task bundles (ABI v2).
 *
 * The reference has no FFI: its executor is a header-level C++ class (MvmExec, mvm_exec.cu:492-1677) driven by a CLI that
 * reads a bundle directory.  Each entry point below flattens one member of that class (cited beside it), with plain
 * pointers and sizes, so the CLI, a ctypes / cgo / JNI stub or a C++ host can bind it.  Return value: 0 = ok, negative =
 * host-side error (KVM_E_*), positive = device error code (executor codes 1..20 as in the reference's MVM_ERRORS,
 * include/mvm_exec.cuh:147-164; op codes 1001..1007 as in MVM_GPT_ERRORS, include/mvm_ops_gpt.cuh:181-194).
 * No exception crosses the boundary; kvm_last_error() gives the text of the last failure on a handle.
 */
#ifndef KVM_B200_H
#define KVM_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KVM_ABI_VERSION 2
#define KVM_NO_VAR (-1)

/* Task descriptor: sixteen int32 words, field for field the reference's MvmTaskDesc (include/mvm_task_abi.h:11-29). */
typedef struct KvmTaskDesc {
    int32_t op_id, succ_off, succ_cnt, indegree, priority, deadline_us, args_off, args_words;
    int32_t wait_var, wait_ver, pub_var, pub_ver, workload_id, flags, reserved0, reserved1;
} KvmTaskDesc;

enum { KVM_F32 = 0, KVM_I32 = 1, KVM_BF16 = 2 };            /* buffer dtypes, MvmBuf.dtype (include/mvm_task_abi.h:33-38) */
enum { KVM_INIT_FILL = 0, KVM_INIT_VALUES = 1, KVM_INIT_SEEDED = 2, KVM_INIT_NONE = 3 };

/* Host-side error codes (negative). */
enum { KVM_E_ARG = -1, KVM_E_CUDA = -2, KVM_E_BUNDLE = -3, KVM_E_STATE = -4, KVM_E_NOMEM = -5, KVM_E_IO = -6 };

typedef struct KvmConfig {
    int32_t device;        /* CUDA device ordinal */
    int32_t workers;       /* worker CTAs; 0 = one per SM */
    int32_t trace;         /* 1 = record per-task start/end timestamps and SM id */
    int32_t timeout_ms;    /* device-side stall limit; 0 = default (20000) */
    int32_t num_vars;      /* version variables; 0 = default (64) */
    int32_t flags;         /* KVM_CFG_* */
} KvmConfig;
enum { KVM_CFG_NO_TENSOR_CORES = 1, /* run every GEMM on the SIMT reference path (debugging / bit-exact f32) */
       KVM_CFG_PAIR_TILES = 2,      /* run two row-adjacent tensor-core GEMM tiles of one product as one 256 x 256 tile when both are ready */
       KVM_CFG_CHAIN = 4,           /* kvm_start may be called again before kvm_finish: the runs queue up on the stream (first device error is kept) */
       KVM_CFG_STATIC = 8,          /* run the resident program as per-worker programs planned on the host (no ready queue); refused if it cannot */
       KVM_CFG_DYNAMIC = 16         /* always the ready queue, even where the static path would be chosen */ };

/* Buffer initial value (mvm_exec.cu:1915-1929 buffer init kinds; `file` inits are read by the caller and passed as VALUES). */
typedef struct KvmInit {
    int32_t kind;          /* KVM_INIT_* */
    int32_t draws;         /* SEEDED: draws per element (1 uniform, 4 normal) */
    double  fill;          /* FILL: the value (integers for i32 buffers) */
    const void* data;      /* VALUES: rows*cols elements in the buffer's storage type (f32 / i32 / raw bf16) */
    uint64_t seed;         /* SEEDED */
    float   bias, coef;    /* SEEDED: value = (acc - bias) * coef */
} KvmInit;

typedef struct KvmResult {
    int32_t status;        /* 0 or the first device error code */
    int32_t done;          /* tasks finished */
    int32_t admitted;      /* tasks submitted */
    int32_t err_task;      /* task index of the first error, -1 if none */
    int32_t err_a, err_b;  /* two words of detail */
    float   ms;            /* device time of the persistent kernel (CUDA events) */
    float   busy_frac;     /* with trace: sum(end - start) / (workers * span); else 0 */
} KvmResult;

typedef struct KvmExec KvmExec;

/* MvmExec::MvmExec(cfg) (mvm_exec.cu:494-569): create the context, size the pools. */
int kvm_create(const KvmConfig* cfg, KvmExec** out);
/* ~MvmExec (mvm_exec.cu:570-578): frees every device buffer the handle allocated. */
void kvm_destroy(KvmExec* h);
/* MvmExec::add_buffer (mvm_exec.cu:582-591,1621-1651): allocate rows x cols of dtype, initialise on the device; returns the
 * buffer-table index (>= 0) or a negative error. */
int kvm_add_buffer(KvmExec* h, int32_t rows, int32_t cols, int32_t dtype, const KvmInit* init);
/* Same table entry over memory the caller owns (a device pointer, ld in elements): how an NCCL / framework tensor becomes a
 * task operand.  No reference counterpart (its buffers are always owned). */
int kvm_bind_buffer(KvmExec* h, void* dev_ptr, int32_t rows, int32_t cols, int32_t ld, int32_t dtype);
/* Device address of buffer idx (NULL on a bad index). */
void* kvm_buffer_ptr(KvmExec* h, int32_t idx);
/* Sharing a buffer with an executor in another process of the same node, for the peer exchange ops (peer_put_signal / peer_wait_sum,
 * include/kvm_ops.def; the reference takes peer pointers from CUDA P2P / IPC the same way, include/mvm_ops_comm.def:5-9):
 * the owner exports a 64-byte handle of a buffer it allocated, the peer maps it (kvm_ipc_open) and binds the pointer as a table
 * entry of its own (kvm_bind_buffer); kvm_ipc_close unmaps it after the peer's executor is destroyed. */
int kvm_ipc_export(KvmExec* h, int32_t idx, void* handle64);
int kvm_ipc_open(KvmExec* h, const void* handle64, void** dev_ptr);
int kvm_ipc_close(KvmExec* h, void* dev_ptr);
/* Raw host -> device / device -> host copies of [offset, offset+bytes) of a buffer's storage. */
int kvm_write_buffer(KvmExec* h, int32_t idx, const void* host, size_t bytes, size_t offset);
int kvm_read_buffer_raw(KvmExec* h, int32_t idx, void* host, size_t bytes, size_t offset);
/* MvmExec::read_buffer (mvm_exec.cu:1541-1554): n elements widened to float32 (i32 converted, bf16 widened exactly). */
int kvm_read_buffer(KvmExec* h, int32_t idx, float* out, size_t n);
/* Version variables (include/mvm_task_abi.h:20-23): base version before a run / value after it. */
int kvm_set_version(KvmExec* h, int32_t var, int32_t version);
int kvm_get_version(KvmExec* h, int32_t var, int32_t* version);
/* MvmBundle::validate + MvmExec::submit (mvm_exec.cu:141-208,742-793): append one compiled batch; successor indices are
 * batch-local.  The bundle is checked (op ids, arities, ranges, buffer indices, indegree == in-edges, acyclic) before any
 * of it reaches the device.
 * Where this differs from the reference: there a submitted batch is admitted and runs once.  Here the batches submitted since
 * the last kvm_clear_tasks form ONE resident program, and every kvm_start / kvm_run executes that whole program (re-armed, as
 * the next window of a template: version waits and publishes shift by what the variables have advanced since).  So
 * submit(A); run; submit(B); run executes A, then A and B.  To run B alone: kvm_clear_tasks between the two. */
int kvm_submit(KvmExec* h, const KvmTaskDesc* tasks, int32_t nt, const int32_t* succ, int32_t ne, const int32_t* args, int32_t na);
/* MvmBundle::validate (mvm_exec.cu:141-208) on its own: the same host check kvm_submit runs, without a handle, a CUDA context
 * or a GPU, against a buffer table of nbufs entries and nvars version variables.  Returns 0, or KVM_E_BUNDLE with the first
 * problem as text in msg (truncated to msg_len).  A malformed bundle is rejected here, before anything reaches a device. */
int kvm_validate_batch(const KvmTaskDesc* tasks, int32_t nt, const int32_t* succ, int32_t ne, const int32_t* args, int32_t na, int32_t nbufs, int32_t nvars,
                       char* msg, size_t msg_len);
/* Read tasks.bin / successors.bin / args.bin of a bundle directory (FRAMEWORK.md:62-71) and submit them; buffers must have
 * been added in metadata.json's order by the caller. */
int kvm_submit_bundle_dir(KvmExec* h, const char* dir);
/* What the reference CLI does with a bundle directory before it runs it (mvm_exec.cu:2055-2076, init kinds :1915-1929): read
 * metadata.json (abi_version 2), create every buffer it lists, in index order, with its init (fill / values / seeded / file, a
 * file path being relative to the directory), set the variables' base versions, then submit tasks.bin / successors.bin /
 * args.bin.  Buffers an earlier bundle of this handle already declared (same index) must have the same shape and are kept.
 * KVM_E_IO if a file cannot be read, KVM_E_BUNDLE (with the reason in kvm_last_error) if the metadata or the batch is malformed. */
int kvm_load_bundle_dir(KvmExec* h, const char* dir);
/* The buffer table as loaded: count, shape / dtype of an entry, and the names metadata.json gave (kvm_buffer_index: index of
 * a name, or KVM_E_ARG; kvm_buffer_name: "" for a buffer added without a name).  kvm_variable_id: id of a named version variable. */
int kvm_buffer_count(KvmExec* h);
int kvm_buffer_info(KvmExec* h, int32_t idx, int32_t* rows, int32_t* cols, int32_t* dtype);
const char* kvm_buffer_name(KvmExec* h, int32_t idx);
int kvm_buffer_index(KvmExec* h, const char* name);
int kvm_variable_id(KvmExec* h, const char* name);
/* MvmExec::start (mvm_exec.cu:724-738): launch the persistent kernel over the resident program (every batch submitted since
 * the last kvm_clear_tasks, see kvm_submit).  kvm_finish (mvm_exec.cu:1513-1539): wait, copy counters back.  kvm_run = both. */
int kvm_start(KvmExec* h);
/* MvmExec::close (mvm_exec.cu:1513-1520: no more batches will be admitted to the running launch).  Here every batch is resident
 * before the launch, so there is nothing to close: kept for callers written against start / close / finish; returns 0, or
 * KVM_E_STATE when no run was started. */
int kvm_close(KvmExec* h);
/* Run on the caller's CUDA stream (a cudaStream_t) from now on, so that launches order with the caller's own work - collectives
 * between segments of a tensor-parallel token - without host synchronisation.  No counterpart in the reference (its executor
 * owns one non-blocking stream, mvm_exec.cu:546).  The stream is not destroyed by kvm_destroy. */
int kvm_set_stream(KvmExec* h, void* stream);
int kvm_finish(KvmExec* h, KvmResult* res);
int kvm_run(KvmExec* h, KvmResult* res);
/* Re-arm the submitted tasks (dependency counters, queue, per-task records) so the same program runs again on the current
 * buffer contents and versions: the reference re-admits a one-step template per window (FRONTEND.md:201-213). */
int kvm_rearm(KvmExec* h);
/* Run the submitted program `steps` times back to back: re-arm + launch per step on the executor's stream with no host
 * synchronisation in between; res->ms is the device time of the whole sequence (CUDA events on that stream) and the
 * counters are those of the last step.  A device error in any step stops the following ones (they see the error word). */
int kvm_run_steps(KvmExec* h, int32_t steps, KvmResult* res);
/* Drop all submitted tasks (buffers and versions stay). */
int kvm_clear_tasks(KvmExec* h);
/* Per task of the last run: times executed and predecessor completions observed (the exactly-once witness and dependency
 * count the reference keeps in MvmTrace.exec_count, include/mvm_exec.cuh:167-176,733-736). Either pointer may be NULL. */
int kvm_task_counts(KvmExec* h, int32_t* exec_count, int32_t* observed, int32_t n);
/* With trace on: per task start / end (ns, %globaltimer) and SM id (MvmTrace, include/mvm_exec.cuh:167-176). */
int kvm_trace(KvmExec* h, uint64_t* start_ns, uint64_t* end_ns, int32_t* smid, int32_t n);
/* With trace on, static path: per streamed GEMV task three bytes of where its time went, each in units of 0.2 us (saturating):
 * bits 0-7 prologue, bits 8-15 the loop over the stages of weights (waits included), bits 16-23 the waits for stages alone;
 * for a streamed attention split: bits 0-7 prologue (0.1 us), bits 8-15 waits for keys and values (0.1 us); 0 for other tasks. */
int kvm_trace_detail(KvmExec* h, int32_t* detail, int32_t n);
/* Launch geometry of the persistent kernel: worker CTAs, threads per CTA, dynamic shared memory bytes. */
int kvm_launch_info(KvmExec* h, int32_t* workers, int32_t* threads, int32_t* smem_bytes);
/* Which path runs the prepared program: the ready queue (0) or per-worker lists planned on the host (1: the reference's static
 * path, include/mvm_static.h:1-17, mvm_exec.cu:1364-1502), whether that launch carries the shared-memory stream ring of the
 * decode ops, and the planner's estimate of one run in microseconds (0 on the ready-queue path).  Valid after kvm_rearm or a run. */
int kvm_plan_info(KvmExec* h, int32_t* is_static, int32_t* stream_ring, float* planned_us);
/* Number of submitted tasks the host planned onto the tcgen05 / TMA path (the rest run SIMT bodies). */
int kvm_tc_task_count(KvmExec* h);
const char* kvm_last_error(KvmExec* h);
/* Read n elements of device memory `dev_src` (storage type dtype: KVM_F32 / KVM_I32 / KVM_BF16) back as float32 WITHOUT allocating
 * anything: no counterpart in the reference (its read_buffer, like kvm_read_buffer here, may allocate).  For callers that must not
 * call cudaMalloc: a decode loop that reads logits / tokens every step while other streams (or a persistent executor) keep the
 * GPU busy - cudaMalloc and cudaFree synchronise the whole device and would stall them.  The widening uses a fixed scratch array
 * inside the library, KVM_NOALLOC_MAX_ELEMS floats (4 MiB) per GPU; larger n is refused with KVM_E_ARG and a message from
 * kvm_noalloc_last_error().  The first call on a device looks the array's address up (make that call before any stream capture
 * starts).  All calls on a GPU share the array: calls whose device work overlaps race, so serialise them.  `stream` is a
 * cudaStream_t the caller owns and that is NOT capturing (NULL = the legacy default stream, which waits for the blocking streams):
 * the call launches on it, copies, synchronises it and returns with the data in host_out.  The caller's current device is unchanged
 * on return. */
#define KVM_NOALLOC_MAX_ELEMS (1u << 20)
int kvm_read_f32_noalloc(int32_t device, const void* dev_src, int32_t dtype, size_t n, float* host_out, void* stream);
const char* kvm_noalloc_last_error(void);
const char* kvm_err_name(int32_t code);
/* Registry lookups (include/kvm_ops.def): arity of op id, or -1; name or NULL. */
int kvm_op_arity(int32_t op_id);
const char* kvm_op_name(int32_t op_id);

#ifdef __cplusplus
}
#endif
#endif
