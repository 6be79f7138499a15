/* etxb200 -- C ABI of the B200 (sm_100a) decode megakernel.
 *
 * The reference (cklxx/etx-megakernel) has no FFI: Python emits a HIP kernel plus a C++ host built on
 * etx/runtime/include/etx/host.h and runs the linked binary as a subprocess.  This library replaces that emitted
 * kernel + host with one hand-written persistent CUDA kernel behind plain C entry points, so the same program
 * surface (task graph -> plan -> session run) drives it through ctypes / cgo / JNI.  Every entry point returns an
 * int32 status (0 = OK, ETXB_E_* otherwise), never throws and never exits the process.
 *
 * Which reference interface each entry replaces (paths inside the reference project):
 *   etxb_create / etxb_bind   etx_host::alloc_args + setup      etx/runtime/include/etx/host.h:55-210
 *   etxb_set_step             vl_set_params (VlParams upload)   examples/vllm_llm/vl_tiles.hip:13-24, 92-95
 *   etxb_launch               etx_host::check_residency+launch  host.h:326-347
 *   etxb_wait                 etx_host::wait (watchdog)         host.h:351-417
 *   etxb_step                 etx_host::run                     host.h:518-531
 *   etxb_status               ctrl words + event dump           etx/runtime/include/etx/abi.h:101-105, host.h:564-580
 *   etxb_trace                ETX_TRACE_RAW per-task stamps     host.h:640-675
 *   etxb_decode_host          the host token loop               examples/vllm_llm/host.hip:819-894
 *   etxb_op_*                 one launch of a single tile type; the argument-block bytes are the tile's own
 *                             (etx/ops/gemv.py:80-94, etx/ops/topk.py:16-23, etx/ops/attnprep.py:11-15,
 *                              etx/importer/argblock.py:16-29)
 */
#ifndef ETXB200_H
#define ETXB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ETXB_VERSION 0x00010000

/* status codes */
enum {
  ETXB_OK = 0,
  ETXB_E_ARG = 1,        /* null pointer, bad size, unknown name */
  ETXB_E_PLAN = 2,       /* plan blob malformed or inconsistent (rejected before any launch) */
  ETXB_E_CUDA = 3,       /* a CUDA runtime call failed; etxb_last_error() has the text */
  ETXB_E_RESIDENCY = 4,  /* the persistent grid cannot be co-resident on this device */
  ETXB_E_TIMEOUT = 5,    /* a device wait ran past its deadline; the kernel returned, the context is usable */
  ETXB_E_ABORTED = 6,    /* host abort requested */
  ETXB_E_UNSUPPORTED = 7 /* shape outside what the tile supports (message says which) */
};

/* tile bodies (the `body` field of a plan's task type; the symbol names a graph links are mapped to these) */
enum {
  ETXB_BODY_NOP = 0,
  ETXB_BODY_PROLOGUE = 1,     /* vl_prologue       examples/vllm_llm/vl_tiles.hip:31-45 */
  ETXB_BODY_ARGMAX = 2,       /* vl_argmax         vl_tiles.hip:47-89 */
  ETXB_BODY_GEMV = 3,         /* dsl_gemv[_fold]   etx/ops/gemv.py:816-840 */
  ETXB_BODY_MOE_UP = 4,       /* dsl_moe_up[_fold] etx/ops/gemv.py:841-911 */
  ETXB_BODY_MOE_DOWN = 5,     /* dsl_moe_down      etx/ops/gemv.py:912-953 */
  ETXB_BODY_TOPK = 6,         /* dsl_topk          etx/ops/topk.py:35-156 */
  ETXB_BODY_ATTNPREP = 7,     /* dsl_attnprep      etx/ops/attnprep.py:86-211 */
  ETXB_BODY_ATTN = 8,         /* paged GQA decode attention, one (partition, kv head) per task */
  ETXB_BODY_ATTN_REDUCE = 9,  /* merge of the partitions of one q head */
  ETXB_BODY_SPLITK_PART = 10, /* demo: partial sums of a split-K reduction (etx/operators/splitk_sum.py) */
  ETXB_BODY_SPLITK_SUM = 11,
  ETXB_BODY_ATTN_FUSED = 12,  /* prep + split-KV attention + merge by the last task to finish, one phase (general and grouped form) */
  /* batched decode (several sequences per step; the reference's column batching, etx/ops/gemv.py:40-73, and request batching,
   * examples/vllm_llm/model.py:194-211): tensor-core tiles that read a weight row once for up to 8 tokens per pass */
  ETXB_BODY_NORM_COL = 13,    /* residual add (+ expert combine in ascending expert id) + RMSNorm of one column */
  ETXB_BODY_GEMV_NB = 14,     /* dsl_gemv with nb activation columns (dsl_gemv_rows_nb, etx/ops/gemv.py:176-289) */
  ETXB_BODY_ROUTE = 15,       /* softmax top-k of every column + per-expert token lists */
  ETXB_BODY_MOE_UP_G = 16,    /* expert-grouped gate+up: an expert's rows read once for all the tokens that selected it */
  ETXB_BODY_MOE_DOWN_G = 17,  /* expert-grouped down, scaled by the routing weight */
  ETXB_BODY_PROLOGUE_NB = 18, /* vl_prologue for column c of a batch */
  ETXB_BODY_ARGMAX_NB = 19,   /* vl_argmax for column c of a batch */
  /* the same three batched grids on the Blackwell tensor cores: tcgen05.mma, weights through TMA tensor copies, fp32 accumulators
   * in tensor memory (the library builds the tensor maps when the plan is bound) */
  ETXB_BODY_GEMV_TC = 20,
  ETXB_BODY_MOE_UP_TC = 21,
  ETXB_BODY_MOE_DOWN_TC = 22,
  ETXB_BODY_MLA_ATTN = 23,    /* absorbed multi-head latent attention of one head over the whole context (DeepSeek-V2 family) */
  ETXB_BODY_COUNT = 24
};

/* The per-step scalars and buffers of the prologue / argmax tiles: field for field the reference's VlParams
 * (examples/vllm_llm/vl_tiles.hip:13-24).  `tok` is the step index t: the prologue embeds token_in[t]; argmax
 * writes token_out[t] and, when write_next, token_in[t + 1], so a greedy run needs no device->host copy per token. */
typedef struct etxb_step_params {
  int32_t tok, pos, write_next, H, V, nrep;
  const void* embed;       /* bf16 [V][H] */
  void* resid;             /* bf16 [H] */
  int64_t* positions;      /* [1] */
  int32_t* seq_lens;       /* [1] */
  int64_t* slot_mapping;   /* [1] */
  const void* logits;      /* bf16 [V] */
  int32_t* token_in;       /* [steps + 2] */
  int32_t* token_out;      /* [steps + 1] */
  uint64_t* token_time;    /* [2 * (steps + 1)] globaltimer ns at prologue / argmax, may be null */
} etxb_step_params;

typedef struct etxb_status_t {
  int32_t ctrl;            /* bit0 host abort seen, bit1 wait deadline passed, bit2 bad task table entry */
  int32_t stuck_task;      /* task index (queue order) that gave up, -1 if none */
  int32_t stuck_event;     /* event word it waited for */
  int32_t stuck_value;     /* counter value seen */
  int32_t stuck_target;    /* value it needed */
  int32_t tasks_run;       /* tasks completed in the last step (only counted when tracing is on) */
  uint32_t epoch;          /* steps launched so far */
  float last_ms;           /* device time of the last etxb_step / etxb_wait, CUDA events */
  int32_t kernel_variant;  /* 0: the full kernel; 1..4: the lean decode kernel (grouped attention with 1, 2, 4, 8 q heads per task)
                              the library picked for this plan; option "full_kernel" = 1 forces 0 */
} etxb_status_t;

typedef struct etxb_device_info_t {
  int32_t sm_count, smem_per_block_optin, l2_bytes, cc_major, cc_minor;
  int32_t workers;         /* persistent CTAs the kernel will use (one per SM) */
  int32_t threads;         /* threads per CTA */
  int32_t smem_bytes;      /* dynamic shared memory per CTA */
  uint64_t hbm_bytes;
} etxb_device_info_t;

typedef struct etxb_session etxb_session;

int32_t etxb_version(void);
const char* etxb_last_error(void);   /* thread-local text of the last failure */
int32_t etxb_device_info(int device, etxb_device_info_t* out);

/* plan_blob: the serialized plan (layout in etx-megakernel_b200/csrc/etxb_abi.h, written by passes/plan.py).
 * The blob is copied; the caller may free it. */
int32_t etxb_create(const void* plan_blob, size_t bytes, int device, etxb_session** out);
/* Give a named plan tensor its device address.  The caller keeps ownership and must keep it alive. */
int32_t etxb_bind(etxb_session* s, const char* name, void* dev_ptr, size_t bytes);
int32_t etxb_set_step(etxb_session* s, const etxb_step_params* p);
/* Options: "timeout_ms" (device wait deadline), "trace" (0/1: per-task stamps + execution counts), "full_kernel" (0/1: run
 * the kernel that holds every tile even when the plan qualifies for the lean decode kernel; see etxb_status_t.kernel_variant). */
int32_t etxb_set_option(etxb_session* s, const char* key, int64_t value);
int32_t etxb_launch(etxb_session* s, void* cuda_stream);
/* The unfused baseline: the same step as one kernel launch PER GRID, in plan order on one stream (what the reference
 * builds with kernel.py:645-681 and runs with host.h:440-457 to state the gain of the single launch).  Same results;
 * refused (ETXB_E_UNSUPPORTED) when a grid waits for a grid that comes later in the plan. */
int32_t etxb_launch_unfused(etxb_session* s, void* cuda_stream);
int32_t etxb_wait(etxb_session* s, double timeout_s);

int32_t etxb_step(etxb_session* s, void* cuda_stream, double timeout_s);
int32_t etxb_status(etxb_session* s, etxb_status_t* out);

/* ---- sharded model: one rank (process + GPU) per shard, partial rows exchanged inside the kernel ------------------
 * The reference shards a program over devices with device-scoped events and multi-device plans
 * (etx/passes/plan.py:58-86 device_of_task, etx/runtime/include/etx/host.h:79-210 one event region per device); here
 * every rank runs the SAME single-device plan on its shard of the weights and the ranks meet at the row-parallel grids
 * the plan marks as exchanged (o_proj, MoE / MLP down).  A task of such a grid publishes the bf16 rows it wrote as
 * FLAGGED WORDS -- 4 bytes: the value in the low half, a 16-bit flag derived from the step in the high half -- into
 * row `rank` of the grid's [n_ranks][M] block in EVERY rank's exchange region: plain 4-byte stores, over NVLink for
 * the peers.  A store of 4 bytes is atomic, so value and flag arrive together: no fence, no remote counter, no
 * collective call.  The norm fold that follows (mode bit 0x1000, R = n_ranks) reads the block in its own rank's
 * memory, re-reads a word until its flag is this step's (bounded by the step's deadline like every wait), and adds
 * the ranks' rows in rank order, so every rank computes bit-identical hidden states.
 *
 * A region is one device allocation holding the blocks at offsets the caller chooses -- the same on every rank (the
 * argument blocks name them in `rows`).  etxb_exchange_alloc zeroes it and exports a 64-byte inter-process handle;
 * the caller passes the handles around (any transport) and opens the peers' with etxb_exchange_open.
 * etxb_set_exchange (once, before the first step) records this rank's region and the peers' mappings (peer_bases[r]
 * for r != rank; entry `rank` is ignored).  All ranks must run the same steps; a rank whose peers stop publishing
 * returns ETXB_E_TIMEOUT at its deadline.  Every rank must have finished its last step before any rank frees or
 * closes a region (a running peer still stores into it).  etxb_launch_unfused is refused on a sharded session, and
 * etxb_launch on a rank's plan that has no exchange set.
 * lm_head split by vocabulary: each rank's step parameters name its own V / n_ranks logits; after etxb_set_exchange,
 * etxb_set_option(s, "exchange_argmax_offset", off) names n_ranks x 16 bytes of every region where the argmax tile
 * exchanges the ranks' (maximum, global index) pairs as 8-byte (payload, step flag) stores and picks the same token
 * on every rank. */
#define ETXB_IPC_HANDLE_BYTES 64
int32_t etxb_exchange_alloc(int device, size_t bytes, void** dev_ptr, unsigned char* handle /*[64]*/);
int32_t etxb_exchange_free(int device, void* dev_ptr);
int32_t etxb_exchange_open(int device, const unsigned char* handle /*[64]*/, void** peer_ptr);
int32_t etxb_exchange_close(int device, void* peer_ptr);
int32_t etxb_set_exchange(etxb_session* s, int32_t rank, int32_t n_ranks, void* local_base, size_t bytes, void* const* peer_bases);
/* Copies 8 x uint64 per task of the last traced step: {taken, deps ready, body done, worker, 4 in-body marks}
 * (globaltimer ns; a mark a tile did not set is 0). */
int32_t etxb_trace(etxb_session* s, void* host_buf, size_t bytes);
int32_t etxb_exec_counts(etxb_session* s, int32_t* host_buf, size_t count);
int32_t etxb_destroy(etxb_session* s);

/* Greedy decode with HOST buffers: token ids come from and go back to host memory every step (one 8-byte H2D of
 * {token, position} through pinned memory and one 4-byte D2H per step, both inside the call).  tokens_in[n_in] are
 * fed first (teacher-forced); generation continues greedily until n_total steps ran.  tokens_out[n_total] receives
 * the argmax of every step.  start_pos is the position of tokens_in[0]. */
int32_t etxb_decode_host(etxb_session* s, const int32_t* tokens_in, int32_t n_in, int32_t n_total,
                         int32_t start_pos, int32_t* tokens_out, float* step_ms /* may be null */);

/* Stand-alone tile launches (tests, micro-benchmarks).  `argblock` is host memory holding the tile's argument block
 * (device pointers inside); ntasks tasks of the tile run on the persistent grid, task index = blockIdx-style `blk`.
 * form: ETXB_BODY_*.  The call is asynchronous on `cuda_stream`. */
int32_t etxb_op_launch(int device, int32_t body, const void* argblock, size_t bytes, int32_t ntasks,
                       const etxb_step_params* step /* may be null */, void* cuda_stream);

/* The fused attention phase with NO device allocation: its partial-result scratch lives in a fixed-size static
 * device array inside the library (about 2.1 MiB, held by every GPU that loads the library until the process exits).
 * No counterpart in the reference.  For callers that cannot allocate when they need attention (a plug-in that only
 * gets the host's buffers, a serving loop that pre-sized its pools, a caller whose free memory all went to the KV
 * cache).  `argblock`: an attn_fused block (etx-megakernel_b200/csrc/etxb_abi.h: etxb_attnf_args); its four scratch
 * pointers are ignored.  Limits: NH <= 64, max_parts <= 64 (context <= 2048), HD <= 128, else ETXB_E_UNSUPPORTED.
 * The first call on a device does the one-time set-up (symbol address, shared-memory limit): make it before any
 * stream capture.  All calls share the array; calls that overlap on the GPU race on it.  Asynchronous on the stream. */
int32_t etxb_attn_fused_static(int device, const void* argblock, size_t bytes, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
