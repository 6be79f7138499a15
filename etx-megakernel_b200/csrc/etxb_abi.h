// Device/host shared layouts of the B200 decode megakernel: plan blob, task table, kernel parameters and the
// argument blocks of the built-in tiles.
//
// The task descriptor {type, coord[4]} and the idea of per-worker static queues follow the reference runtime ABI
// (etx/runtime/include/etx/abi.h:33-41, 77-80); the event protocol does not: counters here only ever count UP and a
// consumer of step `epoch` waits for `epoch * arrivals_per_step`, so nothing is reset between steps (the reference
// re-initialises every counter per step, etx/runtime/include/etx/host.h:264-325).
#pragma once
#include <stdint.h>

#define ETXB_EV_STRIDE 32            // int32 words between event counters: one 128-byte line each (abi.h:7-12)
#define ETXB_CONSUMER_WARPS 16       // warps that run tile bodies
#define ETXB_CONSUMERS (ETXB_CONSUMER_WARPS * 32)
#define ETXB_THREADS (ETXB_CONSUMERS + 32)   // + one producer warp that streams weights with bulk async copies
#define ETXB_NWARPS ETXB_CONSUMER_WARPS
#define ETXB_MAX_ARGS 4              // tensor pointers a task type may name (Graph.call_device(args=[...]))
// shared memory of the persistent CTA
#ifndef ETXB_STAGE_BYTES
#define ETXB_STAGE_BYTES 24576       // one ring stage: whole weight rows, so a row is at most 24 KB (K <= 12288); 24 KB holds 6 / 3 / 1
#endif
                                     // rows of K = 2048 / 4096 / 12288 and 16 rows of K = 768 without a remainder
#ifndef ETXB_NSTAGE
#define ETXB_NSTAGE 6                // 144 KB of weights in flight per SM (measured against 5 x 32 KB: 0.8 % / 2.3 % faster on the MoE / dense model)
#endif
#define ETXB_RING_BYTES (ETXB_STAGE_BYTES * ETXB_NSTAGE)
#ifndef ETXB_GEN_BYTES
#define ETXB_GEN_BYTES 65536         // activations: fp32 scratch [0,32K), bf16 x [32K,56K), row results [56K,64K); attention tiles use all of it
#endif
#ifndef ETXB_XF_FLOATS
#define ETXB_XF_FLOATS 8192          // norm fold works on K <= 8192 floats
#endif
#ifndef ETXB_XB_OFF
#define ETXB_XB_OFF 32768
#endif
#ifndef ETXB_XB_ELEMS
#define ETXB_XB_ELEMS 12288          // streamed GEMV rows are at most 12288 elements long
#endif
#ifndef ETXB_G_OFF
#define ETXB_G_OFF 57344
#endif
#ifndef ETXB_G_FLOATS
#define ETXB_G_FLOATS 2048
#endif
#define ETXB_SCR_FLOATS 256
#define ETXB_CTX_BYTES 288           // one prefetched task context: 96-byte record + 192 bytes of argument block
#define ETXB_CTX_SLOTS 4
#define ETXB_SMEM_BYTES (ETXB_RING_BYTES + ETXB_GEN_BYTES + ETXB_SCR_FLOATS * 4 + 512 + ETXB_CTX_SLOTS * ETXB_CTX_BYTES)
#define ETXB_ATTN_PART 32            // KV positions per attention task
#define ETXB_MAX_PEERS 7           // ranks of a sharded model besides this one
#define ETXB_MAX_NB 8                // activation columns of the stand-alone batched GEMV kernel

// ---- plan blob ------------------------------------------------------------------------------------------------
// header, then sections in this order, each starting on an 8-byte boundary:
//   tensors   n_tensors x etxb_blob_tensor
//   types     n_types   x etxb_type
//   qbegin    (n_workers + 1) x int32       tasks are stored grouped by worker: worker w owns [qbegin[w], qbegin[w+1])
//   tasks     n_tasks   x etxb_task
//   evcount   n_events  x int32             arrivals one step delivers to each event counter
//   inwords   n_in      x int32             event indices, referenced by etxb_task.in_off / in_n
//   outwords  n_out     x int32
//   pool      pool_bytes                    argument blocks (tensor 0, "impargs"), device pointers already inside
#define ETXB_MAGIC 0x3030324258544555ull   // "UETXB200" little endian
struct etxb_blob_header {
  uint64_t magic;
  uint32_t version, n_workers, n_tasks, n_types, n_events, n_in, n_out, n_tensors, pool_bytes, flags;
  uint32_t reserved[4];
};
struct etxb_blob_tensor { char name[56]; uint64_t bytes; };

struct etxb_type {
  int32_t body;                 // ETXB_BODY_*
  int32_t cst[4];               // TaskGrid.consts: cst[0] = byte offset of the grid's argument block in args[0]
  int32_t args[ETXB_MAX_ARGS];  // plan tensor indices, -1 = unused
  int32_t flags;                // bit0: the tile streams weights through the ring
  int32_t stream_word;          // event the producer warp waits for before it reads the weight addresses of a task:
                                // -1 none (static weights: stream ahead freely), -2 the task's own in-events, >= 0 that event
  int32_t exchange;             // 1: a row-parallel GEMV / MoE-down grid of a sharded model -- every rank runs the same grid on its
                                // shard and a task publishes the rows it wrote, as flagged words, into the block its argument
                                // block names in `rows`, in every rank's exchange region (etxb_set_exchange); 0 otherwise
};

struct etxb_task {
  int32_t type;
  int32_t coord[4];
  int32_t in_off, in_n;         // events to wait for
  int32_t out_off, out_n;       // events to arrive on
  int32_t id;                   // index in program (graph) order, for traces and diagnostics
};

// Per-task record, in queue order, built by the host when the tensors are bound: everything the consumer loop needs of
// a task in one 96-byte read (the task table -> type table -> argument pointer chain resolved ahead of time).
struct etxb_rec {
  int32_t body, c0, c1, id, in_n, out_n, in_off, out_off;
  int32_t in_word[4], in_cnt[4], out_word[4];      // the first four of each list; longer lists continue in inwords / outwords
  uint64_t args;                                   // device address of the task's argument block
  int32_t stream_word;
  uint32_t mirror;                                 // exchanged task: bits 0..21 first 4-byte word (from the exchange region's base) of the
                                                   // flagged words it publishes, bits 22..31 how many (the rows it wrote); 0 = none
};

// ---- step parameters (the reference's VlParams, examples/vllm_llm/vl_tiles.hip:13-24) ---------------------------
struct etxb_stepv {
  int32_t tok, pos, write_next, H, V, nrep;
  const void* embed; void* resid; int64_t* positions; int32_t* seq_lens; int64_t* slot_mapping;
  const void* logits; int32_t* token_in; int32_t* token_out; uint64_t* token_time;
};

// ---- kernel parameters --------------------------------------------------------------------------------------
struct etxb_params {
  const etxb_task* tasks;
  const int32_t* qbegin;
  const etxb_type* types;
  const etxb_rec* recs;         // [n_tasks] in queue order
  void* const* type_args;       // [n_types][ETXB_MAX_ARGS] device pointers
  int32_t* events;              // counters, ETXB_EV_STRIDE words apart
  const int32_t* evcount;
  const int32_t* inwords;
  const int32_t* outwords;
  int32_t* ctrl;                // [0] status bits, [1] stuck task, [2] stuck event, [3] value, [4] target, [5] tasks run
  uint64_t* trace;              // 4 x u64 per task (by task id) or null
  int32_t* exec_count;          // per task id or null
  const int32_t* step_dev;      // optional {tok, pos} pair in device memory overriding step.tok/pos (host decode loop)
  unsigned long long timeout_ns;
  uint32_t epoch;
  int32_t n_workers;
  etxb_stepv step;
  // sharded model (etxb_set_exchange): this rank's exchange region and the other ranks' as mapped into this process;
  // the blocks of flagged rows sit at the same offsets in every rank's region.
  int32_t n_peers, rank;
  uint32_t xargmax, tc_on;                         // byte offset in a region of the [ranks][2] 8-byte (payload, flag) slots of the sharded
                                                   // argmax (lm_head split by vocabulary); 0 = every rank holds all logits
  unsigned char* xbase;
  unsigned char* xpeer[ETXB_MAX_PEERS];
};

// ctrl[0] bits
#define ETXB_CTRL_ABORT 1
#define ETXB_CTRL_TIMEOUT 2
#define ETXB_CTRL_BADTASK 4

// ---- argument blocks ----------------------------------------------------------------------------------------
// GEMV family: byte for byte the reference's 160-byte block (etx/ops/gemv.py:80-94), grid words at 144.
struct etxb_gemv_args {
  const void* W; const void* x; void* out; const int32_t* ids; const float* wts; int64_t estride;   // 0..47
  int32_t M, K, rpt, tpe;                                                                         // 48..63
  const void* rows; const void* resid_in; void* resid_out; const void* ln;                        // 64..95
  int32_t R; float eps; int32_t mode; int32_t E; const void* logits;                              // 96..119
  int32_t nb, sx, sout, srows, srin, srout;                                                       // 120..143
  uint32_t grid[3], nblocks;                                                                      // 144..159
};
// mode bits of the GEMV family.  0 plain; 1 norm fold (x = rmsnorm(bf16(resid_in + sum of R rows)), task 0 stores
// resid_out and x); 2 / 3 top-k fold without / with renormalisation (etx/ops/gemv.py:75-79).  Extensions used by the
// B200 builder: 0x100 bf16-round the routing weights (the oracle's numerics), 0x200 add a bf16 bias row taken from
// `wts` (plain form only; the reference passes biases through its DSL_EXT block).
#define ETXB_MODE_NORM 1
#define ETXB_MODE_TOPK 2
#define ETXB_MODE_TOPK_RENORM 3
#define ETXB_MODE_BF16_WTS 0x100
#define ETXB_MODE_BIAS 0x200
#define ETXB_MODE_SUM_SLOTS 0x400     // MoE down: the task covers every slot and writes their bf16 sum in ascending expert id
#define ETXB_MODE_FLAGGED 0x1000      // sharded model.  Norm fold: `rows` holds R rows of K flagged words (4 bytes: bf16 value | step flag
                                      // << 16) that the ranks publish; the fold re-reads a word until its flag is this step's.  Plain GEMV /
                                      // MoE down of an exchanged grid: `rows` names the [ranks][M] block of flagged words to publish into
#define ETXB_MODE_ROUTE_READY 0x800   // MoE down with the top-k fold: the gate/up tiles it waits for have published the routing in
                                      // ids / wts, so the consumer warps read it there (one load) instead of redoing the top-k;
                                      // the producer warp, which runs ahead of the gate/up phase, still derives it from the logits
// bits 16..23 of mode: expert slots per task of the MoE forms (0 = 1)
// bits 24..27 of mode (top-k fold): ns always-on experts stored after the E routed ones (DeepSeek's shared experts as
// experts E .. E + ns - 1): the fold picks R - ns experts from the logits and gives the last ns slots weight 1

// top-k: the reference's 64-byte block (etx/ops/topk.py:16-23), grid words at 48.
struct etxb_topk_args {
  const void* logits; float* wts; int32_t* ids; int32_t* tei; int32_t E, K, mode, nbsv;
  uint32_t grid[3], nblocks;
};

// attention prep: the reference's 112-byte block (etx/ops/attnprep.py:11-15), grid words at 96.
struct etxb_attnprep_args {
  void* qkv; const void* qw; const void* kw; const void* cos_sin; const int64_t* positions; void* kc; void* vc;
  const int64_t* slot_mapping; int32_t NH, NKV, HD; float eps; int32_t BS, X; int32_t pad[2];
  uint32_t grid[3], nblocks;
};

// decode attention + reduce (the reference imports vLLM's kernels for these: importer/spec.py:243-244; this block is
// this library's own): q rows are read from `q` with `q_stride` elements between heads.
struct etxb_attn_args {
  const void* q; const void* kc; const void* vc; const int32_t* block_tables; const int32_t* seq_lens;   // 0..39
  float* exp_sums; float* max_logits; float* tmp_out; void* out;                                         // 40..71
  float scale; int32_t NH, NKV, HD, BS, X, max_parts, max_blocks;                                        // 72..103
  int32_t pad[2];                                                                                        // 104..111
  uint32_t grid[3], nblocks;                                                                             // 112..127
};

// fused attention phase (this library's own): q/k norm + rope + cache write of the new position, split-KV attention over
// a partition of the context, and the merge of the partitions by the last task to finish (counters: monotonic int32,
// never reset).  General form (gq = 0): task blk = part * NKV + h covers 32 positions x the G q heads of kv head h, one
// counter per kv head.  Grouped form (gq > 0, head_dim 128, cache blocks of 16): task blk = part * (NH / gq) + group
// covers part_len = 128 positions x gq q heads, one counter per group.
struct etxb_attnf_args {
  void* qkv; const void* qw; const void* kw; const void* cos_sin; void* kc; void* vc;                            // 0..47
  const int32_t* block_tables; const int32_t* seq_lens; const int64_t* positions; const int64_t* slot_mapping;  // 48..79
  float* exp_sums; float* max_logits; float* tmp_out; void* out; int32_t* counters;                             // 80..119
  float scale, eps; int32_t NH, NKV, HD, BS, X, max_parts;                                                      // 120..151
  int32_t gq, part_len;   // 152..159: gq > 0 selects the grouped form (gq q heads x 128 positions per task, task = part * (NH / gq) + group);
                          // part_len: bits 0..15 = 128, bits 16..23 = a tag that tells the grids sharing the partial buffers apart (the layer),
                          // bit 24 = whole-sequence form: task = q group, walks every partition, partials in the idle weight ring
                          // (plans without streamed tiles only: the batched step)
  uint32_t grid[3], nblocks;                                                                                    // 160..175
};

// split-K demo (etx/operators/splitk_sum.py): parts[i][j] = sum of a chunk, out[i] = sum over j.
struct etxb_splitk_args { const float* in; float* parts; float* out; int32_t rows, cols, chunks, pad; uint32_t grid[3], nblocks; };
