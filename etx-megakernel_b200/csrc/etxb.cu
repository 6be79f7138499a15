// Host side of the C ABI declared in include/etxb200.h: plan blob validation and upload, session lifecycle,
// cooperative launch of the persistent kernel, bounded waiting, status / trace read-back, the host-buffer decode
// loop and single-tile launches.
//
// Takes over the reference's host launcher etx/runtime/include/etx/host.h (setup 79-210, launch 339-347, watchdog
// wait 351-417, event dump 545-587) and the token loop of examples/vllm_llm/host.hip:819-894.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <chrono>
#include <string>
#include <thread>
#include <vector>

#include "../../include/etxb200.h"
#include "etxb_kernel.cuh"
#include "etxb_gemv_nb.cuh"

static_assert(sizeof(etxb_gemv_args) == 160 && offsetof(etxb_gemv_args, grid) == 144, "GEMV block layout (etx/ops/gemv.py:80-94)");
static_assert(sizeof(etxb_topk_args) == 64 && offsetof(etxb_topk_args, grid) == 48, "top-k block layout (etx/ops/topk.py:16-23)");
static_assert(sizeof(etxb_attnprep_args) == 112 && offsetof(etxb_attnprep_args, grid) == 96, "attnprep block layout (etx/ops/attnprep.py:11-15)");
static_assert(sizeof(etxb_attnf_args) == 176 && offsetof(etxb_attnf_args, grid) == 160, "fused attention block layout");
static_assert(sizeof(etxb_attn_args) == 128 && offsetof(etxb_attn_args, grid) == 112, "attention block layout");
static_assert(ETXB_SMEM_BYTES + 256 <= 232448, "dynamic + static shared memory must fit the 227 KB a CTA may opt into");
static_assert(sizeof(etxb_task) == 40 && sizeof(etxb_type) == 48, "plan table layouts");
static_assert(sizeof(etxb_stepv) == sizeof(etxb_step_params), "step parameter layouts must agree");
static_assert(sizeof(etxb::etxb_route_args) == 88 && offsetof(etxb::etxb_route_args, grid) == 72, "route block layout");
static_assert(sizeof(etxb::etxb_mla_args) == 128 && offsetof(etxb::etxb_mla_args, grid) == 112 && offsetof(etxb::etxb_mla_args, tmp) == 88, "mla block layout");
static_assert(sizeof(etxb::etxb_batch_args) == 32 && offsetof(etxb::etxb_batch_args, grid) == 16, "column block layout");
static_assert(ETXB_NBR_OFF + 2 * ETXB_NB_ROWS * ETXB_NBC * 4 <= ETXB_GEN_BYTES && ETXB_NBP_OFF + ETXB_NBP_UNITS * 512 <= ETXB_NBR_OFF, "batched tiles fit the general region");

static thread_local std::string g_err;
static int32_t fail(int32_t code, const std::string& msg) { g_err = msg; return code; }
#define CU(call)                                                                                         \
  do {                                                                                                   \
    cudaError_t e_ = (call);                                                                             \
    if (e_ != cudaSuccess) return fail(ETXB_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)

struct etxb_session {
  int device = 0;
  etxb_blob_header h{};
  std::vector<etxb_blob_tensor> tensors;
  std::vector<etxb_type> types;
  std::vector<int32_t> qbegin, evcount, inwords, outwords;
  std::vector<etxb_task> tasks;
  std::vector<void*> tensor_ptr;       // device address of every plan tensor (index 0 = argument pool)
  // device copies
  etxb_task* d_tasks = nullptr; etxb_rec* d_recs = nullptr; etxb_rec* d_urecs = nullptr; int32_t* d_uqbegin = nullptr;
  bool grid_order_ok = true;
  int variant = 0;                     // kernel variant picked from the plan (select_variant); force_full overrides it
  bool force_full = false;
  int32_t* d_qbegin = nullptr; etxb_type* d_types = nullptr; void** d_type_args = nullptr;
  int32_t* d_events = nullptr; int32_t* d_evcount = nullptr; int32_t* d_inwords = nullptr; int32_t* d_outwords = nullptr;
  int32_t* d_ctrl = nullptr; uint64_t* d_trace = nullptr; int32_t* d_exec = nullptr; unsigned char* d_pool = nullptr;
  int32_t* h_ctrl = nullptr;           // pinned mirror
  int32_t* h_tok = nullptr;            // pinned staging of the host decode loop
  bool args_dirty = true, trace = false, launched = false;
  uint32_t epoch = 0;
  unsigned long long timeout_ns = 2000000000ull;
  etxb_stepv step{};
  cudaStream_t stream = nullptr, own_stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = 0.f;
  int workers = 0;
  // sharded model (etxb_set_exchange)
  std::vector<unsigned char> h_pool;   // host copy of the argument pool (the rows an exchanged task writes are derived from it)
  int n_ranks = 1, rank = 0;
  unsigned char* xbase = nullptr; size_t xbytes = 0;
  unsigned char* xpeer[ETXB_MAX_PEERS] = {};
  uint32_t xargmax = 0;                // byte offset of the sharded argmax block in a region (0: the lm_head is whole on every rank)
  bool has_exchange = false;           // the plan is one rank's step of a sharded model (some grid is marked exchanged)
  bool tc_on = false;                  // the plan has tensor-core tiles (tcgen05): the kernel allocates tensor memory
  void* d_maps = nullptr;              // their TMA tensor maps, one per grid (128 bytes each)
};

static int g_kernel_ready[64];

static int g_sm_count[64];

// ---- argument-block checks ----------------------------------------------------------------------------------------
// What the tiles take, checked on the host for every block that reaches the device (a plan's pool when the records are
// built, a single-tile launch's block): a block outside these limits would make a device loop that cannot advance or
// overrun a shared-memory region, so it is refused with ETXB_E_UNSUPPORTED before anything is launched.  The Python
// packers check the same limits earlier (ops/gemv.py check_shape, ops/attn.py check_fused).
static int32_t check_gemv_block(int body, const etxb_gemv_args& a) {
  char m[256];
  const int fold = a.mode & 0xff;
  const int spt = ((a.mode >> 16) & 0xff) ? ((a.mode >> 16) & 0xff) : 1;
  const char* why = nullptr;
  if (a.K <= 0 || a.K > ETXB_XB_ELEMS || (a.K % 8)) why = "0 < K <= 12288 and K % 8 == 0 (a row fills at most one 24 KB stage)";
  else if (a.M < 1 || a.rpt < 1) why = "M >= 1 and rpt >= 1";
  else if (body != ETXB_BODY_GEMV && a.tpe < 1) why = "tpe >= 1";
  else if (fold == ETXB_MODE_NORM && a.K > ETXB_XF_FLOATS) why = "a norm fold works on K <= 8192";
  else if (fold == ETXB_MODE_NORM && (a.R < 0 || a.R > 64)) why = "a norm fold adds 0 <= R <= 64 rows";
  else if (fold > 3) why = "mode & 0xff is 0 (plain), 1 (norm fold), 2 or 3 (top-k fold)";
  else if (fold >= 2 && (a.E < 1 || a.E > 256 || a.R < 1 || a.R > 16 || a.R > a.E || a.logits == nullptr)) why = "a top-k fold needs logits, 1 <= E <= 256 and 1 <= R <= min(16, E)";
  else if (body == ETXB_BODY_GEMV && (a.mode & (ETXB_MODE_SUM_SLOTS | 0xff0000))) why = "slot bits are for the MoE forms only";
  else if (fold >= 2 && ((a.mode >> 24) & 0xf) >= a.R) why = "the always-on experts (mode bits 24..27) leave at least one routed slot";
  else if (body == ETXB_BODY_MOE_UP && 2 * spt * a.rpt > ETXB_G_FLOATS) why = "gate + up results of a task: 2 * slots * rpt <= 2048";
  else if (body == ETXB_BODY_MOE_DOWN && ((long long)spt * a.K > ETXB_XB_ELEMS || spt * a.rpt > ETXB_G_FLOATS)) why = "down: slots * K <= 12288 activations and slots * rpt <= 2048 results per task";
  else if (body != ETXB_BODY_GEMV && spt > 16) why = "at most 16 expert slots per task";
  else if (body != ETXB_BODY_GEMV && ((long long)((a.nblocks + (uint32_t)a.tpe - 1) / (uint32_t)a.tpe) * spt > 16)) why = "slot groups x slots per task <= 16 slots";
  if (!why) return ETXB_OK;
  snprintf(m, sizeof m, "GEMV-family block (body %d, M=%d, K=%d, rpt=%d, tpe=%d, R=%d, E=%d, mode=0x%x) outside the tile: %s", body, a.M, a.K, a.rpt, a.tpe, a.R, a.E, a.mode, why);
  return fail(ETXB_E_UNSUPPORTED, m);
}
static int32_t check_attnf_block(const etxb_attnf_args& a) {
  const char* why = nullptr;
  if (a.NKV < 1 || a.NH < a.NKV || a.NH % a.NKV) why = "NH must be a positive multiple of NKV";
  else if (a.max_parts < 1 || a.X != 8 || (a.BS != 16 && a.BS != 32)) why = "max_parts >= 1, X = 8, BS 16 or 32";
  else if (a.gq != 0) {
    const int G = a.NH / a.NKV;
    if (!(a.gq == 1 || a.gq == 2 || a.gq == 4 || a.gq == 8) || G % a.gq) why = "gq is 1, 2, 4 or 8 and divides NH / NKV";
    else if (a.HD != 128 || a.BS != 16 || (a.part_len & 0xffff) != 128) why = "the grouped form is head_dim 128, cache blocks of 16, partitions of 128";
    else if (a.gq * a.max_parts > 4096) why = "gq * max_parts <= 4096";
    else if ((a.part_len >> 24) & ~1) why = "part_len bits 25..31 are zero";
    else if ((a.part_len >> 24) && (a.nblocks > (uint32_t)(a.NH / a.gq) || 65536 + (size_t)a.max_parts * a.gq * 130 * 4 > ETXB_RING_BYTES))
      why = "whole-sequence form: the grid is NH / gq tasks and 64 KB + max_parts * gq * 130 floats fit the idle weight ring";
    else if (a.nblocks > (uint32_t)(a.max_parts * (a.NH / a.gq))) why = "the grid is at most max_parts * NH / gq tasks";
  } else {
    const int G = a.NH / a.NKV;
    if (G + 2 > ETXB_CONSUMER_WARPS || G * a.HD > 2048 || a.HD % 32 || a.HD > 256) why = "general form: G + 2 <= 16, G * HD <= 2048, HD % 32 == 0";
    else if (G * a.max_parts > 8192) why = "G * max_parts <= 8192";
    else if (a.nblocks > (uint32_t)(a.max_parts * a.NKV)) why = "the grid is at most max_parts * NKV tasks";
  }
  if (!why) return ETXB_OK;
  char m[256];
  snprintf(m, sizeof m, "attn_fused block (NH=%d, NKV=%d, HD=%d, BS=%d, max_parts=%d, gq=%d) outside the tile: %s", a.NH, a.NKV, a.HD, a.BS, a.max_parts, a.gq, why);
  return fail(ETXB_E_UNSUPPORTED, m);
}
// the tiles of a batched step (several columns): the GEMV block with its column strides / the routing block
static int32_t check_batch_block(int body, const unsigned char* blk, size_t bytes) {
  const char* why = nullptr;
  char m[256];
  if (body == ETXB_BODY_ROUTE) {
    if (bytes < sizeof(etxb::etxb_route_args)) return fail(ETXB_E_ARG, "route tile: the argument block is 88 bytes");
    etxb::etxb_route_args a;
    memcpy(&a, blk, sizeof a);
    if (a.E < 1 || a.E > 256 || a.K < 1 || a.K > 16 || a.K > a.E) why = "1 <= K <= min(16, E), E <= 256";
    else if (a.nb < 1 || a.nb > 64 || a.nb * a.K > 2048 || a.cap < 1) why = "1 <= nb <= 64 columns, cap >= 1";
    else if (!a.logits || !a.wts || !a.ids || (a.elist != nullptr && !a.ecount)) why = "null pointer";
    if (!why) return ETXB_OK;
    snprintf(m, sizeof m, "route block (E=%d, K=%d, nb=%d, cap=%d) outside the tile: %s", a.E, a.K, a.nb, a.cap, why);
    return fail(ETXB_E_UNSUPPORTED, m);
  }
  if (body == ETXB_BODY_PROLOGUE_NB || body == ETXB_BODY_ARGMAX_NB) {
    if (bytes < sizeof(etxb::etxb_batch_args)) return fail(ETXB_E_ARG, "per-column prologue / argmax: the argument block is 32 bytes");
    etxb::etxb_batch_args a;
    memcpy(&a, blk, sizeof a);
    if (a.nb < 1 || a.nb > 64 || a.slot_span < 0) return fail(ETXB_E_UNSUPPORTED, "per-column prologue / argmax: 1 <= nb <= 64 columns");
    return ETXB_OK;
  }
  if (bytes < sizeof(etxb_gemv_args)) return fail(ETXB_E_ARG, "batched GEMV-family tile: the argument block is 160 bytes");
  etxb_gemv_args a;
  memcpy(&a, blk, sizeof a);
  if (a.K <= 0 || (a.K % 8) || a.M < 0) why = "K > 0, K % 8 == 0";
  else if (a.nb < 1 || a.nb > 64) why = "1 <= nb <= 64 columns";
  else if (body == ETXB_BODY_NORM_COL && (a.K > ETXB_XF_FLOATS || a.R < 0 || a.R > 64 || !a.resid_in || !a.x || !a.ln)) why = "norm of a column: K <= 8192, 0 <= R <= 64, resid_in / x / ln set";
  else if (body != ETXB_BODY_NORM_COL && body < ETXB_BODY_GEMV_TC && (size_t)a.K * 2 + ETXB_NB_PAD > ETXB_NBX_BYTES) why = "one token vector must fit the 40 KB activation stage";
  else if (body != ETXB_BODY_NORM_COL && (a.rpt < 1 || a.M < 1 || !a.W || !a.x || !a.out)) why = "rpt >= 1, M >= 1, W / x / out set";
  else if ((body == ETXB_BODY_MOE_UP_G || body == ETXB_BODY_MOE_DOWN_G) &&
           (a.tpe < 1 || a.R < 1 || a.R > 255 || !a.rows || !a.resid_in)) why = "expert-grouped tile: tpe >= 1, 1 <= R <= 255, token lists (rows) and their lengths (resid_in) set";
  else if ((body == ETXB_BODY_MOE_UP_TC || body == ETXB_BODY_MOE_DOWN_TC) && (a.R < 1 || a.R > 16 || a.nb * a.R > 1024 || !a.ids || a.E > 256))
    why = "share-scheduled expert tile: 1 <= R <= 16, nb * R <= 1024, E <= 256, the step's routing ids set";
  else if (body >= ETXB_BODY_GEMV_TC && (a.K % 64 || ((uintptr_t)a.W & 15))) why = "tensor-core tile: K % 64 == 0 and W 16-byte aligned (TMA tensor copies of 64-wide chunks)";
  else if (body == ETXB_BODY_GEMV_TC && a.tpe > 1 && (a.K % (64 * a.tpe) || !a.rows || !a.resid_in)) why = "split-K dense tile: K a multiple of 64 x the split, partial sums (rows) and arrival counters (resid_in) set";
  else if ((body == ETXB_BODY_MOE_UP_TC || body == ETXB_BODY_MOE_DOWN_TC) && (a.E < 1 || a.estride <= 0 || a.estride % a.K)) why = "tensor-core expert tile: E >= 1 and estride a multiple of K (the experts form one [E * rows][K] matrix)";
  if (!why) return ETXB_OK;
  snprintf(m, sizeof m, "batched block (body %d, M=%d, K=%d, rpt=%d, tpe=%d, R=%d, nb=%d) outside the tile: %s", body, a.M, a.K, a.rpt, a.tpe, a.R, a.nb, why);
  return fail(ETXB_E_UNSUPPORTED, m);
}

static int32_t check_mla_block(const unsigned char* blk, size_t bytes) {
  if (bytes < sizeof(etxb::etxb_mla_args)) return fail(ETXB_E_ARG, "mla_attn tile: the argument block is 128 bytes");
  etxb::etxb_mla_args a;
  memcpy(&a, blk, sizeof a);
  const char* why = nullptr;
  if (a.NH < 1 || a.C < 8 || a.C > 512 || (a.C & 7) || a.DR < 8 || a.DR > 64 || (a.DR & 7) || a.DN < 1 || a.DN + a.DR > 256 || a.C + a.DR > 640 || a.DV < 1)
    why = "C <= 512 and DR <= 64 (multiples of 8), DN + DR <= 256";
  else if (a.maxlen < 1 || a.maxlen > ETXB_MLA_MAXCTX) why = "1 <= maxlen <= 8192";
  else if (!a.qkv || !a.kvln || !a.cos_sin || !a.wkvb || !a.cache || !a.positions || !a.out || !a.tmp) why = "null pointer";
  else if (a.max_parts < 1 || a.max_parts > 64 || (long long)a.max_parts * ETXB_MLA_PART < a.maxlen) why = "max_parts partitions of 128 positions cover maxlen (at most 64)";
  else if (a.nblocks != (uint32_t)(a.NH * (a.max_parts + ETXB_MLA_FIN))) why = "the grid is (max_parts + 4) * NH tasks: the partitions, then four finishing tasks per head";
  if (!why) return ETXB_OK;
  char m[256];
  snprintf(m, sizeof m, "mla_attn block (NH=%d, C=%d, DN=%d, DR=%d, DV=%d, maxlen=%d) outside the tile: %s", a.NH, a.C, a.DN, a.DR, a.DV, a.maxlen, why);
  return fail(ETXB_E_UNSUPPORTED, m);
}

// A block of `body` at `blk` (`bytes` readable).  Tiles whose blocks carry no loop bound the device depends on pass.
static int32_t check_block(int body, const unsigned char* blk, size_t bytes) {
  if (body >= ETXB_BODY_NORM_COL && body <= ETXB_BODY_MOE_DOWN_TC) return check_batch_block(body, blk, bytes);
  if (body == ETXB_BODY_MLA_ATTN) return check_mla_block(blk, bytes);
  if (body == ETXB_BODY_GEMV || body == ETXB_BODY_MOE_UP || body == ETXB_BODY_MOE_DOWN) {
    if (bytes < sizeof(etxb_gemv_args)) return fail(ETXB_E_ARG, "GEMV-family tile: the argument block is 160 bytes");
    etxb_gemv_args a;
    memcpy(&a, blk, sizeof a);
    return check_gemv_block(body, a);
  }
  if (body == ETXB_BODY_ATTN_FUSED) {
    if (bytes < sizeof(etxb_attnf_args)) return fail(ETXB_E_ARG, "attn_fused tile: the argument block is 176 bytes");
    etxb_attnf_args a;
    memcpy(&a, blk, sizeof a);
    return check_attnf_block(a);
  }
  return ETXB_OK;
}

// Which kernel can run this plan?  The lean decode kernels hold only the tiles of a fused decode step; a plan qualifies
// when every grid is one of those tiles with its argument block in the pool (one block per grid) and the blocks stay
// inside what the lean forms cover: norm folds of at most one row (or the flagged rows of a sharded model), top-k folds over at most 128 experts, grouped
// attention (head_dim 128, cache blocks of 16, partitions of 128) with the same group size everywhere.
static int select_variant(const etxb_session* s, const std::vector<unsigned char>& pool) {
  int gq = 0;
  bool any_attn = false, any_mla = false;
  for (const etxb_type& ty : s->types) {
    const int b = ty.body;
    if (b == ETXB_BODY_NOP || b == ETXB_BODY_PROLOGUE || b == ETXB_BODY_ARGMAX) continue;
    if (b == ETXB_BODY_MLA_ATTN) { any_mla = true; continue; }
    if (!(b == ETXB_BODY_GEMV || b == ETXB_BODY_MOE_UP || b == ETXB_BODY_MOE_DOWN || b == ETXB_BODY_ATTN_FUSED)) return 0;
    if (ty.args[0] != 0 || ty.cst[1] != 0 || ty.cst[0] < 0) return 0;
    const size_t off = (size_t)ty.cst[0];
    if (b == ETXB_BODY_ATTN_FUSED) {
      if (off + sizeof(etxb_attnf_args) > pool.size()) return 0;
      etxb_attnf_args a;
      memcpy(&a, pool.data() + off, sizeof a);
      if (!(a.gq == 1 || a.gq == 2 || a.gq == 4 || a.gq == 8) || a.HD != 128 || a.BS != 16 || (a.part_len & 0xffff) != 128 || (a.part_len >> 24)) return 0;
      if (any_attn && a.gq != gq) return 0;
      gq = a.gq; any_attn = true;
    } else {
      if (off + sizeof(etxb_gemv_args) > pool.size()) return 0;
      etxb_gemv_args a;
      memcpy(&a, pool.data() + off, sizeof a);
      const int fold = a.mode & 0xff;
      if (fold == ETXB_MODE_NORM && a.R > 1 && !(a.mode & ETXB_MODE_FLAGGED)) return 0;
      if (fold >= 2 && a.E > 128) return 0;
    }
  }
  if (any_mla) return any_attn ? 0 : 10;                           // latent attention: its own lean kernel (no GQA grids beside it)
  if (!any_attn) gq = 1;                                           // no attention grid: any lean kernel will do
  return gq == 1 ? 1 : gq == 2 ? 2 : gq == 4 ? 3 : 4;
}

// The kernel variants: index 0 = the full kernel, 1..4 = the lean decode kernels for grouped attention with 1, 2, 4, 8
// q heads per task (etxb_kernel.cuh, run_body).
// Entries 5..9: the same five with the exchange code of a sharded session compiled in (launch_kernel adds 5).
// Entry 10: the lean decode kernel of a latent-attention model (no sharded form: such a session falls back to entry 5).
static const void* const g_kernels[11] = {(const void*)etxb::etxb_megakernel<0>, (const void*)etxb::etxb_megakernel<1>, (const void*)etxb::etxb_megakernel<2>,
                                          (const void*)etxb::etxb_megakernel<4>, (const void*)etxb::etxb_megakernel<8>,
                                          (const void*)etxb::etxb_megakernel<0, true>, (const void*)etxb::etxb_megakernel<1, true>,
                                          (const void*)etxb::etxb_megakernel<2, true>, (const void*)etxb::etxb_megakernel<4, true>,
                                          (const void*)etxb::etxb_megakernel<8, true>, (const void*)etxb::etxb_megakernel<ETXB_VARIANT_MLA>};
static int kernel_index(const etxb_session* s) {
  const int v = s->force_full ? 0 : s->variant;
  if (s->xbase == nullptr) return v;
  return (v >= 10 ? 0 : v) + 5;
}

static int32_t prepare_kernel(int device, int* workers_out) {
  CU(cudaSetDevice(device));
  if (device < 0 || device >= 64) return fail(ETXB_E_ARG, "device index out of range");
  if (!g_kernel_ready[device]) {                                   // once per device: attribute queries are slow
    int sms = 0;
    CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    for (const void* k : g_kernels) CU(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, ETXB_SMEM_BYTES));
    int per_sm = 0;
    CU(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, etxb::etxb_megakernel<0>, ETXB_THREADS, ETXB_SMEM_BYTES));
    if (per_sm < 1) return fail(ETXB_E_RESIDENCY, "the persistent CTA does not fit one SM of this device");
    g_sm_count[device] = sms;
    g_kernel_ready[device] = 1;
  }
  *workers_out = g_sm_count[device];
  return ETXB_OK;
}

extern "C" int32_t etxb_version(void) { return ETXB_VERSION; }
extern "C" const char* etxb_last_error(void) { return g_err.c_str(); }

extern "C" int32_t etxb_device_info(int device, etxb_device_info_t* out) {
  if (!out) return fail(ETXB_E_ARG, "null out");
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, device));
  int workers = 0;
  int32_t rc = prepare_kernel(device, &workers);
  if (rc) return rc;
  out->sm_count = prop.multiProcessorCount; out->smem_per_block_optin = (int32_t)prop.sharedMemPerBlockOptin;
  out->l2_bytes = prop.l2CacheSize; out->cc_major = prop.major; out->cc_minor = prop.minor;
  out->workers = workers; out->threads = ETXB_THREADS; out->smem_bytes = ETXB_SMEM_BYTES; out->hbm_bytes = prop.totalGlobalMem;
  return ETXB_OK;
}

// ---- plan blob ------------------------------------------------------------------------------------------------
static size_t al8(size_t x) { return (x + 7) & ~size_t(7); }

static int32_t parse_plan(etxb_session* s, const unsigned char* b, size_t n) {
  if (n < sizeof(etxb_blob_header)) return fail(ETXB_E_PLAN, "plan blob shorter than its header");
  memcpy(&s->h, b, sizeof(s->h));
  const etxb_blob_header& h = s->h;
  if (h.magic != ETXB_MAGIC) return fail(ETXB_E_PLAN, "plan blob: bad magic");
  if (h.version != 1) return fail(ETXB_E_PLAN, "plan blob: unsupported version");
  if (h.n_workers == 0 || h.n_workers > 4096 || h.n_types == 0 || h.n_tensors == 0) return fail(ETXB_E_PLAN, "plan blob: empty tables");
  size_t off = al8(sizeof(h));
  auto take = [&](void* dst, size_t bytes) -> bool {
    if (off + bytes > n) return false;
    if (bytes) memcpy(dst, b + off, bytes);
    off = al8(off + bytes);
    return true;
  };
  s->tensors.resize(h.n_tensors); s->types.resize(h.n_types); s->qbegin.resize(h.n_workers + 1); s->tasks.resize(h.n_tasks);
  s->evcount.resize(h.n_events); s->inwords.resize(h.n_in); s->outwords.resize(h.n_out);
  std::vector<unsigned char> pool(h.pool_bytes);
  if (!take(s->tensors.data(), h.n_tensors * sizeof(etxb_blob_tensor)) || !take(s->types.data(), h.n_types * sizeof(etxb_type)) ||
      !take(s->qbegin.data(), (h.n_workers + 1) * 4) || !take(s->tasks.data(), h.n_tasks * sizeof(etxb_task)) ||
      !take(s->evcount.data(), h.n_events * 4) || !take(s->inwords.data(), h.n_in * 4) || !take(s->outwords.data(), h.n_out * 4) ||
      !take(pool.data(), h.pool_bytes))
    return fail(ETXB_E_PLAN, "plan blob: truncated");
  // consistency: queues cover every task once, indices in range, arrivals per event == declared count
  if (s->qbegin[0] != 0 || s->qbegin[h.n_workers] != (int32_t)h.n_tasks) return fail(ETXB_E_PLAN, "plan blob: queues do not cover the task table");
  for (uint32_t w = 0; w < h.n_workers; ++w)
    if (s->qbegin[w] > s->qbegin[w + 1]) return fail(ETXB_E_PLAN, "plan blob: queue bounds not monotone");
  std::vector<int64_t> arrivals(h.n_events, 0);
  std::vector<char> seen(h.n_tasks, 0);
  for (const etxb_task& t : s->tasks) {
    if (t.type < 0 || t.type >= (int32_t)h.n_types) return fail(ETXB_E_PLAN, "plan blob: task type out of range");
    if (t.id < 0 || t.id >= (int32_t)h.n_tasks || seen[t.id]) return fail(ETXB_E_PLAN, "plan blob: task ids are not a permutation");
    seen[t.id] = 1;
    if (t.in_n < 0 || t.out_n < 0 || t.in_off < 0 || t.out_off < 0 || (uint64_t)t.in_off + t.in_n > h.n_in || (uint64_t)t.out_off + t.out_n > h.n_out)
      return fail(ETXB_E_PLAN, "plan blob: event list out of range");
    for (int i = 0; i < t.in_n; ++i)
      if (s->inwords[t.in_off + i] < 0 || s->inwords[t.in_off + i] >= (int32_t)h.n_events) return fail(ETXB_E_PLAN, "plan blob: wait on an unknown event");
    for (int i = 0; i < t.out_n; ++i) {
      const int32_t w = s->outwords[t.out_off + i];
      if (w < 0 || w >= (int32_t)h.n_events) return fail(ETXB_E_PLAN, "plan blob: arrival on an unknown event");
      ++arrivals[w];
    }
  }
  for (uint32_t e = 0; e < h.n_events; ++e)
    if (arrivals[e] != s->evcount[e]) {
      char m[160];
      snprintf(m, sizeof m, "plan blob: event %u gets %lld arrivals per step but declares %d", e, (long long)arrivals[e], s->evcount[e]);
      return fail(ETXB_E_PLAN, m);
    }
  for (const etxb_task& t : s->tasks)
    for (int i = 0; i < t.in_n; ++i)
      if (s->evcount[s->inwords[t.in_off + i]] <= 0) return fail(ETXB_E_PLAN, "plan blob: a task waits on an event nobody arrives on");
  for (const etxb_type& ty : s->types) {
    if (ty.body < 0 || ty.body >= ETXB_BODY_COUNT) return fail(ETXB_E_PLAN, "plan blob: unknown tile body");
    for (int k = 0; k < ETXB_MAX_ARGS; ++k)
      if (ty.args[k] >= (int32_t)h.n_tensors) return fail(ETXB_E_PLAN, "plan blob: type names an unknown tensor");
    if (ty.body >= ETXB_BODY_GEMV && ty.args[0] < 0) return fail(ETXB_E_PLAN, "plan blob: tile without an argument tensor");
  }
  if (pool.size() != s->tensors[0].bytes) return fail(ETXB_E_PLAN, "plan blob: tensor 0 must be the argument pool");
  if (h.pool_bytes < 192) pool.resize(192, 0);
  // upload
  CU(cudaSetDevice(s->device));
  auto up = [&](void** d, const void* src, size_t bytes) -> cudaError_t {
    cudaError_t e = cudaMalloc(d, bytes ? bytes : 8);
    if (e != cudaSuccess) return e;
    return bytes ? cudaMemcpy(*d, src, bytes, cudaMemcpyHostToDevice) : cudaSuccess;
  };
  CU(up((void**)&s->d_tasks, s->tasks.data(), h.n_tasks * sizeof(etxb_task)));
  CU(up((void**)&s->d_qbegin, s->qbegin.data(), s->qbegin.size() * 4));
  CU(up((void**)&s->d_types, s->types.data(), h.n_types * sizeof(etxb_type)));
  CU(up((void**)&s->d_evcount, s->evcount.data(), h.n_events * 4));
  CU(up((void**)&s->d_inwords, s->inwords.data(), h.n_in * 4));
  CU(up((void**)&s->d_outwords, s->outwords.data(), h.n_out * 4));
  s->variant = select_variant(s, pool);
  s->h_pool = pool;
  for (const etxb_type& ty : s->types) s->has_exchange = s->has_exchange || ty.exchange != 0;
  pool.resize(pool.size() + 256, 0);                               // the context prefetch reads 192 bytes from a block start
  CU(up((void**)&s->d_pool, pool.data(), pool.size()));
  CU(cudaMalloc((void**)&s->d_type_args, (size_t)h.n_types * ETXB_MAX_ARGS * sizeof(void*)));
  const size_t evbytes = (size_t)(h.n_events ? h.n_events : 1) * ETXB_EV_STRIDE * 4;
  CU(cudaMalloc((void**)&s->d_events, evbytes));
  CU(cudaMemset(s->d_events, 0, evbytes));
  CU(cudaMalloc((void**)&s->d_ctrl, 64));
  CU(cudaMemset(s->d_ctrl, 0, 64));
  CU(cudaMallocHost((void**)&s->h_ctrl, 64));
  CU(cudaMallocHost((void**)&s->h_tok, 64));
  s->tensor_ptr.assign(h.n_tensors, nullptr);
  s->tensor_ptr[0] = s->d_pool;
  return ETXB_OK;
}

extern "C" int32_t etxb_create(const void* plan_blob, size_t bytes, int device, etxb_session** out) {
  if (!plan_blob || !out) return fail(ETXB_E_ARG, "null argument");
  *out = nullptr;
  etxb_session* s = new etxb_session();
  s->device = device;
  int32_t rc = prepare_kernel(device, &s->workers);
  if (rc == ETXB_OK) rc = parse_plan(s, (const unsigned char*)plan_blob, bytes);
  if (rc == ETXB_OK && (int)s->h.n_workers > s->workers) rc = fail(ETXB_E_RESIDENCY, "plan wants more workers than the device has SMs");
  if (rc == ETXB_OK) {
    cudaError_t e = cudaStreamCreateWithFlags(&s->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&s->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&s->ev1);
    if (e != cudaSuccess) rc = fail(ETXB_E_CUDA, cudaGetErrorString(e));
  }
  if (rc != ETXB_OK) { std::string keep = g_err; etxb_destroy(s); g_err = keep; return rc; }
  *out = s;
  return ETXB_OK;
}

extern "C" int32_t etxb_destroy(etxb_session* s) {
  if (!s) return ETXB_OK;
  cudaSetDevice(s->device);
  if (s->launched) cudaDeviceSynchronize();
  void* ptrs[] = {s->d_tasks, s->d_recs, s->d_urecs, s->d_uqbegin, s->d_qbegin, s->d_types, s->d_type_args, s->d_events, s->d_evcount, s->d_inwords, s->d_outwords,
                  s->d_ctrl, s->d_trace, s->d_exec, s->d_pool, s->d_maps};
  for (void* p : ptrs) if (p) cudaFree(p);
  if (s->h_ctrl) cudaFreeHost(s->h_ctrl);
  if (s->h_tok) cudaFreeHost(s->h_tok);
  if (s->ev0) cudaEventDestroy(s->ev0);
  if (s->ev1) cudaEventDestroy(s->ev1);
  if (s->own_stream) cudaStreamDestroy(s->own_stream);
  delete s;
  return ETXB_OK;
}

extern "C" int32_t etxb_bind(etxb_session* s, const char* name, void* dev_ptr, size_t bytes) {
  if (!s || !name) return fail(ETXB_E_ARG, "null argument");
  for (size_t i = 0; i < s->tensors.size(); ++i)
    if (strncmp(s->tensors[i].name, name, sizeof(s->tensors[i].name)) == 0) {
      if (bytes < s->tensors[i].bytes) return fail(ETXB_E_ARG, std::string("bind ") + name + ": buffer smaller than the plan's tensor");
      s->tensor_ptr[i] = dev_ptr;
      s->args_dirty = true;
      return ETXB_OK;
    }
  return fail(ETXB_E_ARG, std::string("bind: the plan has no tensor named ") + name);
}

extern "C" int32_t etxb_set_step(etxb_session* s, const etxb_step_params* p) {
  if (!s || !p) return fail(ETXB_E_ARG, "null argument");
  memcpy(&s->step, p, sizeof(s->step));
  return ETXB_OK;
}

extern "C" int32_t etxb_set_option(etxb_session* s, const char* key, int64_t value) {
  if (!s || !key) return fail(ETXB_E_ARG, "null argument");
  if (!strcmp(key, "timeout_ms")) { s->timeout_ns = (unsigned long long)(value > 0 ? value : 1) * 1000000ull; return ETXB_OK; }
  if (!strcmp(key, "trace")) {
    CU(cudaSetDevice(s->device));
    s->trace = value != 0;
    if (s->trace && !s->d_trace) {
      CU(cudaMalloc((void**)&s->d_trace, (size_t)s->h.n_tasks * 64 + 64));
      CU(cudaMemset(s->d_trace, 0, (size_t)s->h.n_tasks * 64 + 64));
      CU(cudaMalloc((void**)&s->d_exec, (size_t)s->h.n_tasks * 4 + 4));
    }
    return ETXB_OK;
  }
  if (!strcmp(key, "full_kernel")) { s->force_full = value != 0; return ETXB_OK; }
  if (!strcmp(key, "exchange_argmax_offset")) {
    // sharded lm_head: where in every rank's region the [n_ranks] 16-byte argmax slots sit (after etxb_set_exchange)
    if (s->n_ranks < 2) return fail(ETXB_E_ARG, "exchange_argmax_offset: set the exchange first");
    if (value <= 0 || (value & 15) || (size_t)value + 16 * (size_t)s->n_ranks > s->xbytes) return fail(ETXB_E_ARG, "exchange_argmax_offset: 16-byte aligned, non-zero, n_ranks x 16 bytes inside the region");
    s->xargmax = (uint32_t)value;
    return ETXB_OK;
  }
  return fail(ETXB_E_ARG, std::string("unknown option ") + key);
}

// ---- sharded model: exchange regions ------------------------------------------------------------------------------
// One region per rank, allocated here so that it is its own device allocation (an inter-process handle names a whole
// allocation), zeroed, and exported as a 64-byte handle the other ranks' processes open.
static_assert(sizeof(cudaIpcMemHandle_t) == ETXB_IPC_HANDLE_BYTES, "handle size");

extern "C" int32_t etxb_exchange_alloc(int device, size_t bytes, void** dev_ptr, unsigned char* handle) {
  if (!dev_ptr || !handle || bytes == 0) return fail(ETXB_E_ARG, "bad argument");
  CU(cudaSetDevice(device));
  const size_t gran = size_t(2) << 20;
  const size_t sz = (bytes + gran - 1) / gran * gran;
  void* p = nullptr;
  CU(cudaMalloc(&p, sz));
  cudaError_t e = cudaMemset(p, 0, sz);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return fail(ETXB_E_CUDA, std::string("exchange_alloc: ") + cudaGetErrorString(e)); }
  memcpy(handle, &h, sizeof h);
  *dev_ptr = p;
  return ETXB_OK;
}
extern "C" int32_t etxb_exchange_free(int device, void* dev_ptr) {
  CU(cudaSetDevice(device));
  if (dev_ptr) CU(cudaFree(dev_ptr));
  return ETXB_OK;
}
extern "C" int32_t etxb_exchange_open(int device, const unsigned char* handle, void** peer_ptr) {
  if (!handle || !peer_ptr) return fail(ETXB_E_ARG, "null argument");
  CU(cudaSetDevice(device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  CU(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ETXB_OK;
}
extern "C" int32_t etxb_exchange_close(int device, void* peer_ptr) {
  CU(cudaSetDevice(device));
  if (peer_ptr) CU(cudaIpcCloseMemHandle(peer_ptr));
  return ETXB_OK;
}

extern "C" int32_t etxb_set_exchange(etxb_session* s, int32_t rank, int32_t n_ranks, void* local_base, size_t bytes, void* const* peer_bases) {
  if (!s || !local_base || (!peer_bases && n_ranks > 1)) return fail(ETXB_E_ARG, "null argument");
  if (n_ranks < 1 || n_ranks > ETXB_MAX_PEERS + 1 || rank < 0 || rank >= n_ranks) return fail(ETXB_E_ARG, "set_exchange: 1 <= n_ranks <= 8, 0 <= rank < n_ranks");
  if (s->epoch != 0 || s->launched || s->xbase != nullptr) return fail(ETXB_E_ARG, "set_exchange: once, before the first step");
  if (bytes < 4 || bytes > (size_t(1) << 24) || ((uintptr_t)local_base & 15)) return fail(ETXB_E_ARG, "set_exchange: a region is 16-byte aligned and at most 16 MiB");
  if (!s->has_exchange) return fail(ETXB_E_PLAN, "set_exchange: the plan marks no grid as exchanged");
  int q = 0;
  for (int r = 0; r < n_ranks; ++r) {
    if (r == rank) continue;
    if (!peer_bases[r] || ((uintptr_t)peer_bases[r] & 15)) return fail(ETXB_E_ARG, "set_exchange: a peer's region is missing or misaligned");
    s->xpeer[q++] = (unsigned char*)peer_bases[r];
  }
  s->xbase = (unsigned char*)local_base; s->xbytes = bytes; s->rank = rank; s->n_ranks = n_ranks;
  s->args_dirty = true;
  return ETXB_OK;
}

// What an exchanged task publishes: the rows it wrote, out[r0 .. r0 + n) of a plain GEMV or of a MoE-down grid that leaves
// one row vector (one slot, or every slot summed), go as flagged words to row `rank` of the [ranks][M] block the grid's
// argument block names in `rows`.  Returns (first word from the region's base) | n << 22.
static int32_t exchange_rows(const etxb_session* s, const etxb_type& ty, const etxb_task& t, uint32_t* mirror) {
  *mirror = 0;
  if (ty.body != ETXB_BODY_GEMV && ty.body != ETXB_BODY_MOE_DOWN) return fail(ETXB_E_UNSUPPORTED, "exchange: only GEMV and MoE-down grids can be exchanged");
  if (ty.args[0] != 0 || ty.cst[1] != 0 || ty.cst[0] < 0 || (size_t)ty.cst[0] + sizeof(etxb_gemv_args) > s->h_pool.size())
    return fail(ETXB_E_UNSUPPORTED, "exchange: the grid's argument block must be in the pool");
  etxb_gemv_args a;
  memcpy(&a, s->h_pool.data() + ty.cst[0], sizeof a);
  if (!(a.mode & ETXB_MODE_FLAGGED) || a.rows == nullptr) return fail(ETXB_E_ARG, "exchange: the grid's argument block must carry the flagged mode bit and name its block in `rows`");
  const int blk = t.coord[0];
  if (blk >= (int)a.nblocks || a.rpt <= 0) return ETXB_OK;
  int r0;
  if (ty.body == ETXB_BODY_GEMV) {
    if ((a.mode & 0xff) != 0) return fail(ETXB_E_UNSUPPORTED, "exchange: a folded GEMV writes no partial rows");
    r0 = blk * a.rpt;
  } else {
    const int spt = ((a.mode >> 16) & 0xff) ? ((a.mode >> 16) & 0xff) : 1;
    if (a.tpe <= 0 || blk / a.tpe != 0 || (!(a.mode & ETXB_MODE_SUM_SLOTS) && spt != 1))
      return fail(ETXB_E_UNSUPPORTED, "exchange: the MoE-down grid must leave one row vector (one slot, or every slot summed by the task)");
    r0 = (blk % a.tpe) * a.rpt;
  }
  const int r1 = std::min(a.M, r0 + a.rpt);
  if (r0 >= r1) return ETXB_OK;
  const unsigned char* block = (const unsigned char*)a.rows;
  if (block < s->xbase || block + (size_t)s->n_ranks * a.M * 4 > s->xbase + s->xbytes || ((block - s->xbase) & 15))
    return fail(ETXB_E_ARG, "exchange: an exchanged grid's block lies outside the exchange region");
  const size_t off = (size_t)(block - s->xbase) / 4 + (size_t)s->rank * a.M + r0;
  if (off >= (size_t(1) << 22) || (r1 - r0) >= 1024) return fail(ETXB_E_UNSUPPORTED, "exchange: row range does not fit the task record");
  *mirror = (uint32_t)off | ((uint32_t)(r1 - r0) << 22);
  return ETXB_OK;
}

typedef CUresult (*etxb_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int32_t build_tensor_maps(etxb_session* s) {
  std::vector<size_t> blocks;                                       // pool offsets of the argument blocks of tensor-core grids
  for (const etxb_type& ty : s->types)
    if (ty.body >= ETXB_BODY_GEMV_TC && ty.body <= ETXB_BODY_MOE_DOWN_TC) {
      if (ty.args[0] != 0 || ty.cst[0] < 0 || (size_t)ty.cst[0] + sizeof(etxb_gemv_args) > s->h_pool.size())
        return fail(ETXB_E_UNSUPPORTED, "a tensor-core grid keeps its argument block in the pool");
      blocks.push_back((size_t)ty.cst[0]);
    }
  s->tc_on = !blocks.empty();
  if (blocks.empty()) return ETXB_OK;
  static etxb_encode_fn encode = nullptr;
  if (!encode) {
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    CU(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return fail(ETXB_E_CUDA, "the driver does not offer cuTensorMapEncodeTiled");
    encode = (etxb_encode_fn)fn;
  }
  std::vector<CUtensorMap> maps(blocks.size());
  if (s->d_maps) { CU(cudaFree(s->d_maps)); s->d_maps = nullptr; }
  CU(cudaMalloc(&s->d_maps, maps.size() * sizeof(CUtensorMap)));
  size_t i = 0;
  for (const etxb_type& ty : s->types) {
    if (!(ty.body >= ETXB_BODY_GEMV_TC && ty.body <= ETXB_BODY_MOE_DOWN_TC)) continue;
    etxb_gemv_args a;
    memcpy(&a, s->h_pool.data() + ty.cst[0], sizeof a);
    const cuuint64_t rows = ty.body == ETXB_BODY_GEMV_TC ? (cuuint64_t)a.M : (cuuint64_t)a.E * (cuuint64_t)(a.estride / a.K);
    cuuint64_t gdim[2] = {(cuuint64_t)a.K, rows};
    cuuint64_t gstr[1] = {(cuuint64_t)a.K * 2};
    cuuint32_t box[2] = {64, ETXB_TC_ROWS};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)a.W, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      char m[160];
      snprintf(m, sizeof m, "cuTensorMapEncodeTiled failed (%d) for a [%llu][%d] bf16 weight tensor", (int)r, (unsigned long long)rows, a.K);
      return fail(ETXB_E_CUDA, m);
    }
    const void* dev = (const unsigned char*)s->d_maps + i * sizeof(CUtensorMap);
    CU(cudaMemcpy(s->d_pool + ty.cst[0] + offsetof(etxb_gemv_args, ln), &dev, sizeof dev, cudaMemcpyHostToDevice));
    ++i;
  }
  CU(cudaMemcpy(s->d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
  return ETXB_OK;
}

static int32_t upload_type_args(etxb_session* s) {
  std::vector<void*> ta((size_t)s->h.n_types * ETXB_MAX_ARGS, nullptr);
  for (size_t t = 0; t < s->types.size(); ++t)
    for (int k = 0; k < ETXB_MAX_ARGS; ++k) {
      const int idx = s->types[t].args[k];
      if (idx < 0) continue;
      if (!s->tensor_ptr[idx]) return fail(ETXB_E_ARG, std::string("tensor not bound: ") + s->tensors[idx].name);
      ta[t * ETXB_MAX_ARGS + k] = s->tensor_ptr[idx];
    }
  CU(cudaMemcpy(s->d_type_args, ta.data(), ta.size() * sizeof(void*), cudaMemcpyHostToDevice));
  // every argument block that lives in the plan's pool is checked against the tile's limits (a block in a tensor the
  // caller fills later cannot be read here: such a program is the caller's to check)
  for (const etxb_type& ty : s->types) {
    if (ty.args[0] != 0 || ty.cst[0] < 0 || (size_t)ty.cst[0] >= s->h_pool.size()) continue;
    int32_t rc = check_block(ty.body, s->h_pool.data() + ty.cst[0], s->h_pool.size() - (size_t)ty.cst[0]);
    if (rc) return rc;
  }
  // tensor-core tiles: one TMA tensor map per grid -- the weight tensor as a [rows][K] bf16 matrix, box 64 k x 128 rows,
  // 128-byte swizzle -- built here because only the library knows the driver entry point; its device address goes into
  // the `ln` field of the grid's argument block (in the device copy of the pool)
  {
    int32_t rc = build_tensor_maps(s);
    if (rc) return rc;
  }
  // per-task records in queue order (the consumer loop prefetches them)
  std::vector<etxb_rec> recs(s->tasks.size());
  for (size_t i = 0; i < s->tasks.size(); ++i) {
    const etxb_task& t = s->tasks[i];
    const etxb_type& ty = s->types[t.type];
    etxb_rec& r = recs[i];
    memset(&r, 0, sizeof r);
    r.body = ty.body; r.c0 = t.coord[0]; r.c1 = t.coord[1]; r.id = t.id;
    r.in_n = t.in_n; r.out_n = t.out_n; r.in_off = t.in_off; r.out_off = t.out_off;
    for (int k = 0; k < 4 && k < t.in_n; ++k) { r.in_word[k] = s->inwords[t.in_off + k]; r.in_cnt[k] = s->evcount[r.in_word[k]]; }
    for (int k = 0; k < 4 && k < t.out_n; ++k) r.out_word[k] = s->outwords[t.out_off + k];
    // tiles below the GEMV family take no argument block: point them at the pool so the 192-byte prefetch stays in bounds
    const bool has_block = ty.body >= ETXB_BODY_GEMV && ty.args[0] >= 0;
    r.args = has_block ? (uint64_t)(uintptr_t)ta[(size_t)t.type * ETXB_MAX_ARGS] + (uint64_t)ty.cst[0] + (uint64_t)t.coord[1] * (uint64_t)ty.cst[1]
                       : (uint64_t)(uintptr_t)s->d_pool;
    r.stream_word = ty.stream_word;
    if (s->xbase != nullptr && ty.exchange) {
      int32_t rc = exchange_rows(s, ty, t, &r.mirror);
      if (rc) return rc;
    }
  }
  if (!s->d_recs) CU(cudaMalloc((void**)&s->d_recs, recs.size() * sizeof(etxb_rec) + 96));
  CU(cudaMemcpy(s->d_recs, recs.data(), recs.size() * sizeof(etxb_rec), cudaMemcpyHostToDevice));
  // the same records grouped by grid (type), worker by worker, for the one-launch-per-grid baseline
  const uint32_t W = s->h.n_workers, NT = s->h.n_types;
  std::vector<etxb_rec> ug; ug.reserve(recs.size());
  std::vector<int32_t> uq((size_t)NT * (W + 1), 0);
  for (uint32_t t = 0; t < NT; ++t) {
    for (uint32_t w = 0; w < W; ++w) {
      uq[(size_t)t * (W + 1) + w] = (int32_t)ug.size();
      for (int32_t i = s->qbegin[w]; i < s->qbegin[w + 1]; ++i)
        if ((uint32_t)s->tasks[i].type == t) ug.push_back(recs[i]);
    }
    uq[(size_t)t * (W + 1) + W] = (int32_t)ug.size();
  }
  // launching grid by grid in type order is only a valid order when every producer's grid precedes its consumers'
  std::vector<int32_t> word_type(s->h.n_events, -1);
  for (const etxb_task& t : s->tasks)
    for (int k = 0; k < t.out_n; ++k) word_type[s->outwords[t.out_off + k]] = std::max(word_type[s->outwords[t.out_off + k]], t.type);
  s->grid_order_ok = true;
  for (const etxb_task& t : s->tasks)
    for (int k = 0; k < t.in_n; ++k)
      if (word_type[s->inwords[t.in_off + k]] >= t.type) s->grid_order_ok = false;
  if (!s->d_urecs) { CU(cudaMalloc((void**)&s->d_urecs, ug.size() * sizeof(etxb_rec) + 96)); CU(cudaMalloc((void**)&s->d_uqbegin, uq.size() * 4)); }
  CU(cudaMemcpy(s->d_urecs, ug.data(), ug.size() * sizeof(etxb_rec), cudaMemcpyHostToDevice));
  CU(cudaMemcpy(s->d_uqbegin, uq.data(), uq.size() * 4, cudaMemcpyHostToDevice));
  s->args_dirty = false;
  return ETXB_OK;
}

static void fill_params(etxb_session* s, etxb_params& p) {
  p.tasks = s->d_tasks; p.recs = s->d_recs; p.qbegin = s->d_qbegin; p.types = s->d_types; p.type_args = s->d_type_args;
  p.events = s->d_events; p.evcount = s->d_evcount; p.inwords = s->d_inwords; p.outwords = s->d_outwords;
  p.ctrl = s->d_ctrl; p.trace = s->trace ? s->d_trace : nullptr; p.exec_count = s->trace ? s->d_exec : nullptr;
  p.step_dev = nullptr; p.timeout_ns = s->timeout_ns; p.epoch = s->epoch; p.n_workers = (int32_t)s->h.n_workers;
  p.step = s->step;
  p.n_peers = s->n_ranks - 1; p.rank = s->rank; p.xargmax = s->xargmax; p.tc_on = s->tc_on ? 1u : 0u; p.xbase = s->xbase;
  for (int q = 0; q < ETXB_MAX_PEERS; ++q) p.xpeer[q] = s->xpeer[q];
}

static int32_t launch_kernel(const etxb_params& p, int grid, cudaStream_t st, int variant = 0) {
  void* kargs[] = {(void*)&p};
  CU(cudaLaunchCooperativeKernel(g_kernels[variant], dim3(grid), dim3(ETXB_THREADS), kargs, ETXB_SMEM_BYTES, st));
  return ETXB_OK;
}

extern "C" int32_t etxb_launch(etxb_session* s, void* cuda_stream) {
  if (!s) return fail(ETXB_E_ARG, "null session");
  CU(cudaSetDevice(s->device));
  if (s->has_exchange && s->xbase == nullptr) return fail(ETXB_E_ARG, "the plan is one rank of a sharded model: etxb_set_exchange comes before the first step");
  if (s->args_dirty) { int32_t rc = upload_type_args(s); if (rc) return rc; }
  s->stream = cuda_stream ? (cudaStream_t)cuda_stream : s->own_stream;
  if (s->trace && s->d_exec) CU(cudaMemsetAsync(s->d_exec, 0, (size_t)s->h.n_tasks * 4, s->stream));
  ++s->epoch;
  etxb_params p;
  fill_params(s, p);
  CU(cudaEventRecord(s->ev0, s->stream));
  int32_t rc = launch_kernel(p, (int)s->h.n_workers, s->stream, kernel_index(s));
  if (rc) return rc;
  CU(cudaEventRecord(s->ev1, s->stream));
  s->launched = true;
  return ETXB_OK;
}

// The unfused baseline (the reference's etx/codegen/kernel.py:645-681 and host.h:440-457): the same tiles and the same
// task records, but one kernel launch per grid, in grid order on one stream.  The in-events of a launch's tasks were
// all counted up by earlier launches, so nothing waits inside a launch; what is lost is what the single launch is
// for: weights streaming ahead across phase boundaries and the hand-off without a launch in between.
extern "C" int32_t etxb_launch_unfused(etxb_session* s, void* cuda_stream) {
  if (!s) return fail(ETXB_E_ARG, "null session");
  CU(cudaSetDevice(s->device));
  if (s->args_dirty) { int32_t rc = upload_type_args(s); if (rc) return rc; }
  if (!s->grid_order_ok) return fail(ETXB_E_UNSUPPORTED, "a grid waits for a grid that comes later in the plan: no launch-per-grid order");
  if (s->n_ranks > 1) return fail(ETXB_E_UNSUPPORTED, "a sharded session runs as the single launch only");   // (its grids wait for peers: launches of two ranks could not be ordered)
  s->stream = cuda_stream ? (cudaStream_t)cuda_stream : s->own_stream;
  if (s->trace && s->d_exec) CU(cudaMemsetAsync(s->d_exec, 0, (size_t)s->h.n_tasks * 4, s->stream));
  ++s->epoch;
  etxb_params p;
  fill_params(s, p);
  p.recs = s->d_urecs;
  CU(cudaEventRecord(s->ev0, s->stream));
  for (uint32_t t = 0; t < s->h.n_types; ++t) {
    p.qbegin = s->d_uqbegin + (size_t)t * (s->h.n_workers + 1);
    int32_t rc = launch_kernel(p, (int)s->h.n_workers, s->stream, kernel_index(s));
    if (rc) return rc;
  }
  CU(cudaEventRecord(s->ev1, s->stream));
  s->launched = true;
  return ETXB_OK;
}

static int32_t read_ctrl(etxb_session* s) {
  CU(cudaMemcpyAsync(s->h_ctrl, s->d_ctrl, 32, cudaMemcpyDeviceToHost, s->stream));
  CU(cudaStreamSynchronize(s->stream));
  return ETXB_OK;
}

// After a failed step the counters are inconsistent: bring every one to epoch * count and clear ctrl, so the next
// step starts clean (the reference forces a full host reset after a failed step, host.h:388).
static int32_t recover(etxb_session* s) {
  std::vector<int32_t> ev((size_t)s->h.n_events * ETXB_EV_STRIDE, 0);
  for (uint32_t e = 0; e < s->h.n_events; ++e) ev[(size_t)e * ETXB_EV_STRIDE] = (int32_t)(s->epoch * (uint32_t)s->evcount[e]);
  if (!ev.empty()) CU(cudaMemcpy(s->d_events, ev.data(), ev.size() * 4, cudaMemcpyHostToDevice));
  // The merge election of the general fused attention tile counts arrivals in the caller's counters buffer (one int32
  // per kv head, max_parts arrivals per step, elected when the count reaches a multiple of max_parts): a step abandoned
  // in the middle of an attention phase leaves them off a multiple, and every later step would then elect its merging
  // task too early.  Zero is a multiple: clear the counters of every fused attention grid of the pool.  (The grouped
  // form has no counters: its partials carry the step number, which only grows.)
  for (const etxb_type& ty : s->types) {
    if (ty.body != ETXB_BODY_ATTN_FUSED || ty.args[0] != 0 || ty.cst[0] < 0 || (size_t)ty.cst[0] + sizeof(etxb_attnf_args) > s->h_pool.size()) continue;
    etxb_attnf_args a;
    memcpy(&a, s->h_pool.data() + ty.cst[0], sizeof a);
    if (a.counters == nullptr || a.NKV < 1 || a.NH < 1) continue;
    const int n = a.gq > 0 ? a.NH / a.gq : a.NKV;
    if (n > 0) CU(cudaMemset(a.counters, 0, (size_t)n * 4));
  }
  CU(cudaMemset(s->d_ctrl, 0, 64));
  return ETXB_OK;
}

extern "C" int32_t etxb_wait(etxb_session* s, double timeout_s) {
  if (!s) return fail(ETXB_E_ARG, "null session");
  if (!s->launched) return ETXB_OK;
  CU(cudaSetDevice(s->device));
  const auto t0 = std::chrono::steady_clock::now();
  bool aborted = false;
  for (;;) {
    cudaError_t q = cudaEventQuery(s->ev1);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) return fail(ETXB_E_CUDA, std::string("kernel failed: ") + cudaGetErrorString(q));
    const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (!aborted && timeout_s > 0 && el > timeout_s) {             // host watchdog: ask the kernel to stop, keep waiting
      const int32_t one = ETXB_CTRL_ABORT;
      cudaStream_t side;
      CU(cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking));
      CU(cudaMemcpyAsync(s->d_ctrl, &one, 4, cudaMemcpyHostToDevice, side));
      CU(cudaStreamSynchronize(side));
      cudaStreamDestroy(side);
      aborted = true;
    }
    if (el > 50e-6) std::this_thread::yield();
  }
  CU(cudaEventElapsedTime(&s->last_ms, s->ev0, s->ev1));
  int32_t rc = read_ctrl(s);
  if (rc) return rc;
  s->launched = false;
  const int32_t c = s->h_ctrl[0];
  if (c == 0) return ETXB_OK;
  char m[200];
  snprintf(m, sizeof m, "step %u stopped: ctrl=%d task=%d event=%d value=%d target=%d", s->epoch, c, s->h_ctrl[1], s->h_ctrl[2], s->h_ctrl[3], s->h_ctrl[4]);
  std::string msg = m;
  recover(s);
  if (c & ETXB_CTRL_BADTASK) return fail(ETXB_E_PLAN, msg);
  if (c & ETXB_CTRL_TIMEOUT) return fail(ETXB_E_TIMEOUT, msg);
  return fail(ETXB_E_ABORTED, msg);
}

extern "C" int32_t etxb_step(etxb_session* s, void* cuda_stream, double timeout_s) {
  int32_t rc = etxb_launch(s, cuda_stream);
  if (rc) return rc;
  return etxb_wait(s, timeout_s);
}

extern "C" int32_t etxb_status(etxb_session* s, etxb_status_t* out) {
  if (!s || !out) return fail(ETXB_E_ARG, "null argument");
  out->ctrl = s->h_ctrl ? s->h_ctrl[0] : 0; out->stuck_task = s->h_ctrl && s->h_ctrl[0] ? s->h_ctrl[1] : -1;
  out->stuck_event = s->h_ctrl[2]; out->stuck_value = s->h_ctrl[3]; out->stuck_target = s->h_ctrl[4];
  out->tasks_run = 0; out->epoch = s->epoch; out->last_ms = s->last_ms;
  out->kernel_variant = s->force_full ? 0 : s->variant;
  if (s->trace && s->d_exec) {
    std::vector<int32_t> ex(s->h.n_tasks);
    CU(cudaSetDevice(s->device));
    CU(cudaMemcpy(ex.data(), s->d_exec, ex.size() * 4, cudaMemcpyDeviceToHost));
    for (int32_t v : ex) out->tasks_run += v;
  }
  return ETXB_OK;
}

extern "C" int32_t etxb_trace(etxb_session* s, void* host_buf, size_t bytes) {
  if (!s || !host_buf) return fail(ETXB_E_ARG, "null argument");
  if (!s->d_trace) return fail(ETXB_E_ARG, "tracing is off (set option trace=1 before the step)");
  if (bytes < (size_t)s->h.n_tasks * 64) return fail(ETXB_E_ARG, "trace buffer too small: 64 bytes per task");
  CU(cudaSetDevice(s->device));
  CU(cudaMemcpy(host_buf, s->d_trace, (size_t)s->h.n_tasks * 64, cudaMemcpyDeviceToHost));
  return ETXB_OK;
}

extern "C" int32_t etxb_exec_counts(etxb_session* s, int32_t* host_buf, size_t count) {
  if (!s || !host_buf) return fail(ETXB_E_ARG, "null argument");
  if (!s->d_exec) return fail(ETXB_E_ARG, "tracing is off (set option trace=1 before the step)");
  if (count < s->h.n_tasks) return fail(ETXB_E_ARG, "buffer too small: one int32 per task");
  CU(cudaSetDevice(s->device));
  CU(cudaMemcpy(host_buf, s->d_exec, (size_t)s->h.n_tasks * 4, cudaMemcpyDeviceToHost));
  return ETXB_OK;
}

extern "C" int32_t etxb_decode_host(etxb_session* s, const int32_t* tokens_in, int32_t n_in, int32_t n_total, int32_t start_pos,
                                    int32_t* tokens_out, float* step_ms) {
  if (!s || !tokens_in || !tokens_out || n_in < 1 || n_total < 1) return fail(ETXB_E_ARG, "bad argument");
  if (!s->step.token_in || !s->step.token_out) return fail(ETXB_E_ARG, "set_step must name token_in / token_out first");
  CU(cudaSetDevice(s->device));
  cudaStream_t st = s->own_stream;
  int32_t next = tokens_in[0];
  for (int t = 0; t < n_total; ++t) {
    const int32_t tok = t < n_in ? tokens_in[t] : next;
    s->h_tok[0] = tok;
    // slot 0 of token_in / token_out is reused every step: the host owns the sequence
    CU(cudaMemcpyAsync(s->step.token_in, s->h_tok, 4, cudaMemcpyHostToDevice, st));
    s->step.tok = 0; s->step.pos = start_pos + t; s->step.write_next = 0;
    int32_t rc = etxb_launch(s, st);
    if (rc) return rc;
    CU(cudaMemcpyAsync(s->h_tok + 8, s->step.token_out, 4, cudaMemcpyDeviceToHost, st));
    rc = etxb_wait(s, 60.0);
    if (rc) return rc;
    CU(cudaStreamSynchronize(st));
    next = s->h_tok[8];
    tokens_out[t] = next;
    if (step_ms) step_ms[t] = s->last_ms;
  }
  return ETXB_OK;
}

// ---- single-tile launches ---------------------------------------------------------------------------------------
struct OpCtx {
  etxb_task* d_tasks = nullptr; etxb_rec* d_recs = nullptr; int cap_tasks = 0; int32_t* d_qbegin = nullptr; etxb_type* d_type = nullptr; void** d_targs = nullptr;
  unsigned char* d_pool = nullptr; size_t cap_pool = 0; int32_t* d_ctrl = nullptr; int32_t* d_events = nullptr; int32_t* d_zero = nullptr;
  int workers = 0;
};
static OpCtx g_op[64];

extern "C" int32_t etxb_op_launch(int device, int32_t body, const void* argblock, size_t bytes, int32_t ntasks,
                                  const etxb_step_params* step, void* cuda_stream) {
  if (device < 0 || device >= 64 || body < 0 || body >= ETXB_BODY_COUNT || ntasks < 1) return fail(ETXB_E_ARG, "bad argument");
  if (body >= ETXB_BODY_GEMV && (!argblock || bytes < 16)) return fail(ETXB_E_ARG, "this tile needs an argument block");
  OpCtx& c = g_op[device];
  int32_t rc = prepare_kernel(device, &c.workers);
  if (rc) return rc;
  if (!(body == ETXB_BODY_GEMV && bytes >= sizeof(etxb_gemv_args) && ((const etxb_gemv_args*)argblock)->nb > 1)) {
    rc = check_block(body, (const unsigned char*)argblock, bytes);      // (the column-batched kernel checks its own limits below)
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)cuda_stream;
  if (body == ETXB_BODY_GEMV && bytes >= sizeof(etxb_gemv_args) && ((const etxb_gemv_args*)argblock)->nb > 1) {
    // column-batched GEMV (the sweep with M = 2, 4, 8 tokens): its own kernel, one CTA per task
    etxb_gemv_args d;
    memcpy(&d, argblock, sizeof d);
    if ((d.mode & 0xff) != 0) return fail(ETXB_E_UNSUPPORTED, "batched GEMV: plain form only");
    if (d.nb > 8 || d.K % 8) return fail(ETXB_E_UNSUPPORTED, "batched GEMV: nb must be 2 .. 8 and K a multiple of 8");
    const size_t smem = (size_t)d.nb * ((size_t)d.K * 2 + ETXB_NB_PAD) + (size_t)ETXB_NB_PART_FLOATS * 4;
    if (smem > 200 * 1024) return fail(ETXB_E_UNSUPPORTED, "batched GEMV: nb * K exceeds the activation stage (nb tokens x K bf16 in shared memory)");
    if (d.rpt > 1024) return fail(ETXB_E_UNSUPPORTED, "batched GEMV: more than 1024 rows per task");
    static int nb_ready[64];
    if (!nb_ready[device]) {
      CU(cudaFuncSetAttribute(etxb::etxb_gemv_nb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      nb_ready[device] = 1;
    }
    etxb::etxb_gemv_nb_kernel<<<ntasks, ETXB_NB_THREADS, smem, st>>>(d);
    CU(cudaGetLastError());
    return ETXB_OK;
  }
  if (!c.d_type) {
    CU(cudaMalloc((void**)&c.d_type, sizeof(etxb_type))); CU(cudaMalloc((void**)&c.d_targs, ETXB_MAX_ARGS * sizeof(void*)));
    CU(cudaMalloc((void**)&c.d_qbegin, 4097 * 4)); CU(cudaMalloc((void**)&c.d_ctrl, 64)); CU(cudaMemset(c.d_ctrl, 0, 64));
    CU(cudaMalloc((void**)&c.d_events, ETXB_EV_STRIDE * 4)); CU(cudaMemset(c.d_events, 0, ETXB_EV_STRIDE * 4));
    CU(cudaMalloc((void**)&c.d_zero, 64)); CU(cudaMemset(c.d_zero, 0, 64));
  }
  if (ntasks > c.cap_tasks) {
    if (c.d_tasks) { CU(cudaStreamSynchronize(st)); CU(cudaFree(c.d_tasks)); CU(cudaFree(c.d_recs)); }
    c.cap_tasks = ntasks + 1024;
    CU(cudaMalloc((void**)&c.d_tasks, (size_t)c.cap_tasks * sizeof(etxb_task)));
    CU(cudaMalloc((void**)&c.d_recs, (size_t)c.cap_tasks * sizeof(etxb_rec)));
  }
  const size_t need = bytes ? bytes : 16;
  if (need > c.cap_pool) {
    if (c.d_pool) { CU(cudaStreamSynchronize(st)); CU(cudaFree(c.d_pool)); }
    c.cap_pool = need + 4096;
    CU(cudaMalloc((void**)&c.d_pool, c.cap_pool));
  }
  const int W = c.workers;
  std::vector<etxb_task> tasks(ntasks);
  std::vector<etxb_rec> recs(ntasks);
  std::vector<int32_t> qb(W + 1, 0);
  // worker w runs tasks w, w + W, ...: store grouped by worker
  int n = 0;
  for (int w = 0; w < W; ++w) {
    qb[w] = n;
    for (int t = w; t < ntasks; t += W) {
      etxb_task& k = tasks[n++];
      memset(&k, 0, sizeof k);
      k.type = 0; k.coord[0] = t; k.id = t;
      etxb_rec& r = recs[n - 1];
      memset(&r, 0, sizeof r);
      r.body = body; r.c0 = t; r.id = t; r.args = (uint64_t)(uintptr_t)c.d_pool; r.stream_word = -1;
    }
  }
  qb[W] = n;
  etxb_type ty; memset(&ty, 0, sizeof ty);
  ty.body = body; for (int k = 0; k < ETXB_MAX_ARGS; ++k) ty.args[k] = -1; ty.args[0] = 0;
  ty.stream_word = -1;                                             // everything the weight addresses depend on precedes the launch
  void* targs[ETXB_MAX_ARGS] = {c.d_pool, nullptr, nullptr, nullptr};
  CU(cudaMemcpyAsync(c.d_tasks, tasks.data(), tasks.size() * sizeof(etxb_task), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c.d_recs, recs.data(), recs.size() * sizeof(etxb_rec), cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c.d_qbegin, qb.data(), qb.size() * 4, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c.d_type, &ty, sizeof ty, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(c.d_targs, targs, sizeof targs, cudaMemcpyHostToDevice, st));
  if (bytes) CU(cudaMemcpyAsync(c.d_pool, argblock, bytes, cudaMemcpyHostToDevice, st));
  etxb_params p; memset(&p, 0, sizeof p);
  p.tasks = c.d_tasks; p.recs = c.d_recs; p.qbegin = c.d_qbegin; p.types = c.d_type; p.type_args = c.d_targs; p.events = c.d_events;
  p.evcount = c.d_zero; p.inwords = c.d_zero; p.outwords = c.d_zero; p.ctrl = c.d_ctrl; p.timeout_ns = 2000000000ull;
  static uint32_t op_epoch[64];                                    // a new step number per launch: flags a tile derives from it never repeat
  p.epoch = ++op_epoch[device];
  p.n_workers = W;
  if (step) memcpy(&p.step, step, sizeof(p.step));
  return launch_kernel(p, W, st);
}

// ---- attention phase without any allocation ---------------------------------------------------------------------
// Some callers cannot allocate device memory at the point where they need attention: code running inside a region
// that forbids cudaMalloc (a real-time serving loop that pre-sized its pools, a plug-in that only receives the
// host's input and output buffers, a caller that already handed all free memory to its KV cache).  The fused
// attention tile needs scratch for the per-partition partial results; here that scratch is a file-scope device array
// of fixed size that every GPU loading this library holds until the process exits.
#define ETXB_STATIC_MAX_NH 64        // q heads
#define ETXB_STATIC_MAX_PARTS 64     // partitions of 32 positions: context <= 2048
#define ETXB_STATIC_MAX_HD 128
struct etxb_static_scratch {
  float tmp_out[ETXB_STATIC_MAX_NH * ETXB_STATIC_MAX_PARTS * ETXB_STATIC_MAX_HD];   // 2 MiB
  float exp_sums[ETXB_STATIC_MAX_NH * ETXB_STATIC_MAX_PARTS];
  float max_logits[ETXB_STATIC_MAX_NH * ETXB_STATIC_MAX_PARTS];
  int32_t counters[ETXB_STATIC_MAX_NH];
};
static __device__ __align__(256) unsigned char g_attn_scratch[sizeof(etxb_static_scratch)];
static etxb_static_scratch* g_attn_scratch_dev[64];   // device address of the array on each device, set once per device

namespace etxb {
__global__ void __launch_bounds__(ETXB_CONSUMERS, 1) etxb_attn_static_kernel(const etxb_attnf_args d, const etxb_stepv S) {
  extern __shared__ __align__(128) unsigned char st_smem[];
  Smem sm;
  sm.xs = (float*)st_smem;
  sm.scr = (float*)(st_smem + ETXB_GEN_BYTES);
  sm.ring = nullptr; sm.full = nullptr; sm.empty = nullptr; sm.prod = nullptr; sm.deadline = nullptr; sm.ctrl = nullptr; sm.stop = nullptr; sm.tr = nullptr; sm.tc = nullptr; sm.epoch = 0; sm.cur = 0;
  tile_attn_fused((const unsigned char*)&d, (int)blockIdx.x, sm, S);
}
}  // namespace etxb

// The fused attention phase (see etxb_attnf_args) with its partial-result scratch in the static array above.
// `argblock` is an etxb_attnf_args block as for the attn_fused tile; its exp_sums, max_logits, tmp_out and counters
// pointers are ignored.  Limits: NH <= 64, max_parts <= 64 (context <= 2048), HD <= 128; larger sizes are refused
// with ETXB_E_UNSUPPORTED.  Calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on a
// device looks the array's device address up (cudaGetSymbolAddress) and raises the kernel's shared-memory limit: make
// that first call before any stream capture.  Every call shares the one array: it keeps the previous call's
// partials, the election counters are cleared at the start of each call, and two calls that overlap on the GPU
// (different streams) race on it.  Asynchronous on `cuda_stream`.
extern "C" int32_t etxb_attn_fused_static(int device, const void* argblock, size_t bytes, void* cuda_stream) {
  if (!argblock || bytes < sizeof(etxb_attnf_args)) return fail(ETXB_E_ARG, "attn_fused_static: needs a 176-byte attn_fused argument block");
  if (device < 0 || device >= 64) return fail(ETXB_E_ARG, "device index out of range");
  etxb_attnf_args d;
  memcpy(&d, argblock, sizeof d);
  if (d.NKV < 1 || d.NH < d.NKV || d.NH % d.NKV) return fail(ETXB_E_ARG, "attn_fused_static: NH must be a multiple of NKV");
  const int G = d.NH / d.NKV;
  if (d.NH > ETXB_STATIC_MAX_NH || d.max_parts > ETXB_STATIC_MAX_PARTS || d.HD > ETXB_STATIC_MAX_HD || d.max_parts < 1) {
    char m[200];
    snprintf(m, sizeof m, "attn_fused_static: NH=%d, max_parts=%d, HD=%d exceed the static scratch (NH <= %d, max_parts <= %d, HD <= %d)",
             d.NH, d.max_parts, d.HD, ETXB_STATIC_MAX_NH, ETXB_STATIC_MAX_PARTS, ETXB_STATIC_MAX_HD);
    return fail(ETXB_E_UNSUPPORTED, m);
  }
  if (G + 2 > ETXB_CONSUMER_WARPS || G * d.HD > 2048 || d.HD % 32 || d.X != 8 || (d.BS != 16 && d.BS != 32) || G * d.max_parts > 8192)
    return fail(ETXB_E_UNSUPPORTED, "attn_fused_static: shape outside the fused attention tile (G + 2 <= 16, G * HD <= 2048, HD % 32 == 0, X = 8, BS 16 or 32)");
  if (d.gq != 0) return fail(ETXB_E_UNSUPPORTED, "attn_fused_static: the general form only (gq = 0)");
  if (d.nblocks != (uint32_t)(d.max_parts * d.NKV)) return fail(ETXB_E_ARG, "attn_fused_static: the grid must be max_parts * NKV tasks");
  CU(cudaSetDevice(device));
  const int smem = ETXB_GEN_BYTES + ETXB_SCR_FLOATS * 4;
  if (!g_attn_scratch_dev[device]) {                              // set-up, once per device, with that device current
    void* p = nullptr;
    CU(cudaGetSymbolAddress(&p, g_attn_scratch));
    CU(cudaFuncSetAttribute(etxb::etxb_attn_static_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    g_attn_scratch_dev[device] = (etxb_static_scratch*)p;
  }
  etxb_static_scratch* sc = g_attn_scratch_dev[device];
  cudaStream_t st = (cudaStream_t)cuda_stream;
  CU(cudaMemsetAsync(sc->counters, 0, sizeof(sc->counters), st));  // the merge election counts arrivals from zero
  d.tmp_out = sc->tmp_out; d.exp_sums = sc->exp_sums; d.max_logits = sc->max_logits; d.counters = sc->counters;
  etxb_stepv S;
  memset(&S, 0, sizeof S);                                        // no step buffers: position / slot / length come from the block's pointers
  etxb::etxb_attn_static_kernel<<<d.nblocks, ETXB_CONSUMERS, smem, st>>>(d, S);
  CU(cudaGetLastError());
  return ETXB_OK;
}
