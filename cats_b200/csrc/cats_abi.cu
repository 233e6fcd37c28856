// extern "C" entry points declared in include/cats_b200.h: argument checks, grid sizing and
// launches.  No allocation, no device synchronisation (except cats_read_counters), no exit().
#include "../../include/cats_b200.h"

#include <string.h>

#include <stdlib.h>

#include <mutex>

#include "cats_run.cuh"
#include "cats_stats.cuh"

namespace cats {

int g_use_pdl = 1;

// Per-device properties, queried once per device (no allocation involved).
const DevInfo& dev_info() {
  static DevInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (info[dev].sms == 0) {
    int sms = 0, smem = 0, khz = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
    info[dev].max_smem_optin = smem;
    info[dev].clock_khz = khz > 0 ? khz : 1965000;
    info[dev].sms = sms > 0 ? sms : 148;
  }
  return info[dev];
}

// the per-type launchers are instantiated in cats_inst_stage.cu / cats_inst_mega.cu
#define CATS_EXTERN_INST(T)                                                                         \
  extern template cudaError_t inst_gate<T>(const void*, const void*, WsPtrs, int, int, int, float,  \
                                           void*, uint8_t*, cudaStream_t);                          \
  extern template cudaError_t inst_updown<T>(int, const void*, const void*, const void*, WsPtrs,    \
                                             int, int, int, void*, int, void*, void*, const void*,  \
                                             float, void*, cudaStream_t);                           \
  extern template cudaError_t inst_rows_gemv<T>(const void*, const void*, int, int, int, void*,     \
                                                cudaStream_t);                                      \
  extern template cudaError_t inst_gate_tma<T>(const TmaPlan&, const void*, const void*, WsPtrs,    \
                                               int, int, int, float, void*, uint8_t*,               \
                                               cudaStream_t);                                       \
  extern template cudaError_t inst_updown_tma<T>(const TmaPlan&, const void*, const void*,          \
                                                 const void*, WsPtrs, int, int, int, void*, int,    \
                                                 void*, void*, const void*, float, cudaStream_t);   \
  extern template cudaError_t inst_mega<T>(const MegaPlan&, const MegaParams&, const MegaArgs&,     \
                                           WsPtrs, cudaStream_t);
CATS_EXTERN_INST(float)
CATS_EXTERN_INST(__half)
CATS_EXTERN_INST(__nv_bfloat16)
#undef CATS_EXTERN_INST

}  // namespace cats

namespace {

using namespace cats;

thread_local cudaError_t g_last_cuda = cudaSuccess;

int esize(int dtype) { return dtype == CATS_F32 ? 4 : 2; }
int vecn(int dtype) { return dtype == CATS_F32 ? 4 : 8; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(int B, int H, int I, int dtype) {
  if (dtype != CATS_F32 && dtype != CATS_F16 && dtype != CATS_BF16) return CATS_ERR_DTYPE;
  if (B < 1 || B > kMaxB || H < 1 || I < 1) return CATS_ERR_SHAPE;
  if (H % vecn(dtype) != 0) return CATS_ERR_SHAPE;
  return CATS_OK;
}

int check_ws(void* ws, size_t ws_bytes, int H, int I, WsPtrs* p) {
  if (!ws) return CATS_ERR_NULL;
  if (!aligned16(ws)) return CATS_ERR_ALIGN;
  if (ws_layout(ws, H, I, p) > ws_bytes) return CATS_ERR_WORKSPACE;
  return CATS_OK;
}

int cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return CATS_OK;
  g_last_cuda = e;
  return CATS_ERR_CUDA;
}

// FN<T>(args...) for the runtime dtype
#define CATS_DISPATCH(dtype, FN, ...)                                  \
  do {                                                                 \
    if ((dtype) == CATS_F32) return FN<float>(__VA_ARGS__);            \
    if ((dtype) == CATS_F16) return FN<__half>(__VA_ARGS__);           \
    return FN<__nv_bfloat16>(__VA_ARGS__);                             \
  } while (0)

// ---- tuning knobs (cats_set_option) ------------------------------------------------------------
struct Options {
  int use_tma = 1;     // TMA-fed kernels where the shape allows (else the direct-load kernels)
  int ring_kb = 200;   // shared-memory ring per TMA kernel
  int use_mega = 1;    // persistent cooperative kernel for cats_mlp / cats_mlp_stack
  int pair_ahead_rows = 16; // up-projection rows per segment that stage 1 of cats_mlp asks into L2
  int single_pair = 1; // cats_mlp with one token: the stage-1 / stage-2+3 kernel pair instead
  int bulk_flush = 1;  // persistent kernel: flush accumulators with TMA bulk reduces
  int mma_dot = 1;     // persistent kernel: gate / up dot products on the tensor cores (16-bit)
  int parts = 0;       // persistent kernel: parts per layer (0 = choose by the rows per CTA)
  int wait_ms = 1000;  // limit of every device-side wait (mbarrier, grid barrier, peer data)
  int l2_ahead_kb = 128;  // gate rows a stalled producer of the persistent kernel asks into L2, KB per CTA (0: off)
  int local_lists = 1; // tensor-parallel ranks with one part per layer: per-CTA lists, no list barrier
  int xchg = 0;        // tensor-parallel exchange: 0 = by the number of ranks, 1 = every CTA adds
                       // all ranks' partial sums, 2 = per-slice totals published by each CTA
};
Options& options() {
  static Options o = [] {
    Options v;
    if (const char* e = getenv("CATS_B200_TMA")) v.use_tma = atoi(e);
    if (const char* e = getenv("CATS_B200_RING_KB")) v.ring_kb = atoi(e);
    if (const char* e = getenv("CATS_B200_PDL")) g_use_pdl = atoi(e);
    if (const char* e = getenv("CATS_B200_MEGA")) v.use_mega = atoi(e);
    if (const char* e = getenv("CATS_B200_SINGLE_PAIR")) v.single_pair = atoi(e);
    if (const char* e = getenv("CATS_B200_PAIR_AHEAD_ROWS")) v.pair_ahead_rows = atoi(e);
    if (const char* e = getenv("CATS_B200_BULK_FLUSH")) v.bulk_flush = atoi(e);
    if (const char* e = getenv("CATS_B200_MMA_DOT")) v.mma_dot = atoi(e);
    if (const char* e = getenv("CATS_B200_PARTS")) v.parts = atoi(e);
    if (const char* e = getenv("CATS_B200_WAIT_MS")) v.wait_ms = atoi(e);
    if (const char* e = getenv("CATS_B200_XCHG")) v.xchg = atoi(e);
    if (const char* e = getenv("CATS_B200_LOCAL_LISTS")) v.local_lists = atoi(e);
    if (const char* e = getenv("CATS_B200_L2_AHEAD_KB")) v.l2_ahead_kb = atoi(e);
    return v;
  }();
  return o;
}

// The wait limit in units of 1024 clock cycles of the current device.
int wait_kcycles() {
  long long ms = options().wait_ms;
  if (ms < 1) ms = 1;
  if (ms > 60000) ms = 60000;
  const long long kc = ms * dev_info().clock_khz / 1024;
  return (int)(kc > 0x7fffffffLL ? 0x7fffffffLL : kc);
}

// Largest stage count <= smax (looking at most 3 below it) whose largest divisor <= 8 — the
// number of consumer warps that can stride over the ring — is biggest.
void pick_stages(int smax, int* S, int* cw) {
  *S = 0;
  *cw = 0;
  for (int cand = smax; cand >= 2 && cand >= smax - 3; --cand) {
    int d_best = 1;
    for (int d = 1; d <= kConsumerWarps; ++d)
      if (cand % d == 0) d_best = d;
    if (d_best > *cw) {
      *cw = d_best;
      *S = cand;
    }
  }
}

TmaPlan plan_gate_tma(int B, int H, int I, int dtype) {
  TmaPlan p;
  const Options& o = options();
  if (!o.use_tma || B > 4) return p;
  const size_t row_bytes = (size_t)H * esize(dtype);
  if (row_bytes % 16) return p;
  const size_t xbytes = (size_t)B * row_bytes;
  p.xs = xbytes <= 32 * 1024;
  size_t budget = (size_t)o.ring_kb * 1024;
  if (p.xs) budget = budget > xbytes + 32 * 1024 ? budget - xbytes : 32 * 1024;
  p.sr = (row_bytes <= 8192) ? 2 : 1;
  const size_t stage = p.sr * row_bytes;
  int smax = (int)(budget / stage);
  if (smax > 16) smax = 16;
  if (smax < 2) return p;
  pick_stages(smax, &p.S, &p.cw);
  p.pw = (stage < 16 * 1024 && p.S % 2 == 0) ? 2 : 1;
  p.grid = dev_info().sms;
  if (p.grid > I) p.grid = I;
  p.rmax = (I + p.grid - 1) / p.grid;
  p.smem = align_up(p.S * stage + 16 * (size_t)p.S + 4 * (size_t)p.rmax * batch_tile(B), 16) +
           (p.xs ? xbytes : 0);
  p.wait_kc = wait_kcycles();
  p.ok = p.smem + 2048 <= (size_t)dev_info().max_smem_optin;
  return p;
}

TmaPlan plan_updown_tma(int B, int H, int I, int dtype) {
  TmaPlan p;
  const Options& o = options();
  if (!o.use_tma || B > 4) return p;
  const size_t row_bytes = (size_t)H * esize(dtype);
  if (row_bytes % 16) return p;
  const int nvec = H / vecn(dtype);
  const int need = (nvec + kConsumerThreads - 1) / kConsumerThreads;
  p.nvt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  if (need > 8) return p;
  const size_t xbytes = (size_t)B * row_bytes;
  p.xs = xbytes <= 32 * 1024;
  size_t budget = (size_t)o.ring_kb * 1024;
  if (p.xs) budget = budget > xbytes + 32 * 1024 ? budget - xbytes : 32 * 1024;
  int smax = (int)(budget / row_bytes);
  if (smax > 32) smax = 32;
  if (smax < 2) return p;
  pick_stages(smax, &p.S, &p.cw);
  p.pw = (row_bytes < 16 * 1024 && p.S % 2 == 0) ? 2 : 1;
  p.grid = dev_info().sms;
  const int by_rows = (I + 7) / 8;
  if (p.grid > by_rows) p.grid = by_rows;
  p.cap = (I + p.grid - 1) / p.grid;
  p.smem = align_up(p.S * row_bytes + 16 * (size_t)p.S +
                        4 * (size_t)p.cap * (1 + batch_tile(B)), 16) +
           (p.xs ? xbytes : 0);
  p.wait_kc = wait_kcycles();
  p.ok = p.smem + 8192 <= (size_t)dev_info().max_smem_optin;
  return p;
}

// ---- persistent kernel ------------------------------------------------------------------------
MegaPlan plan_mega(int L, int B, int H, int I, int dtype, bool has_resid, bool tp = false) {
  MegaPlan p;
  const Options& o = options();
  if (!o.use_mega || !o.use_tma || B > 4 || L < 1 || L > kMegaMaxLayers) return p;
  if (L > 1 && !has_resid) return p;
  const size_t row_bytes = (size_t)H * esize(dtype);
  if (row_bytes % 16) return p;
  const int nvec = H / vecn(dtype);
  const int need = (nvec + kConsumerThreads - 1) / kConsumerThreads;
  if (need > 8) return p;
  p.nvt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  p.grid = dev_info().sms;
  if (p.grid > kMegaMaxGrid) p.grid = kMegaMaxGrid;
  // Parts per layer: three hide the list latency (publish, grid barrier, scan) of one part
  // behind the gate rows of the others, but that takes enough rows; a slice of a few rows per
  // CTA (tensor-parallel ranks) is quicker with one barrier chain per layer.
  // (measured on the Mistral shape, one GPU: 12 rows per CTA and layer: 16.7 us with one part,
  // 19.2 with three; 24 rows: 19.6 with two, 21.3 with three; from 48 rows up three are best)
  const int rows_per_cta = I / p.grid;
  p.parts = o.parts >= 1 && o.parts <= kParts ? o.parts
            : rows_per_cta < 18 ? 1 : rows_per_cta < 36 ? 2 : kParts;
  // Tensor-parallel ranks can work on per-CTA lists (no list barrier at all), which needs one
  // part per layer; with rows of at most 8 KB that beats two balanced parts up to 36 rows per CTA
  // (measured on one GPU with a rank's slice, H 4096: 3584 rows 22.0 us against 23.7, 1792 rows
  // 17.5 against 20.5; with 16 KB rows and a 12-stage ring two balanced parts stay ahead).
  if (tp && o.local_lists && !(o.parts >= 1 && o.parts <= kParts) && rows_per_cta < 36 &&
      row_bytes <= 8192)
    p.parts = 1;
  if (p.grid > I / p.parts) p.grid = I / p.parts;
  if (p.grid < 1) return p;
  const int half_rows = (I + p.parts - 1) / p.parts;
  p.rmax = (half_rows + p.grid - 1) / p.grid + 1;
  p.cap = p.rmax;
  const int bt = batch_tile(B);
  // staging area of the bulk-reduce flush: 32 vectors of fp32 per consumer warp (needs whole
  // warps of vectors: H a multiple of 32 vectors)
  p.bulk_flush = (o.bulk_flush && nvec % 32 == 0) ? 1 : 0;
  // tensor-core dot products: 16-bit weights, every warp's column range a whole number of
  // double steps (32 columns), partial sums of two groups in shared memory
  // (batches only: for one token the warp-per-row FMA path keeps up with HBM and needs no
  // barrier per group)
  p.mma_dot = (o.mma_dot && B >= 2 && dtype != CATS_F32 && H % (32 * kConsumerWarps) == 0) ? 1 : 0;
  const size_t stage = (p.bulk_flush ? 128 + (size_t)kConsumerWarps * 32 * vecn(dtype) * sizeof(float) : 0) +
                       (p.mma_dot ? sizeof(float) * 2 * kConsumerWarps * 8 * bt : 0);
  const size_t fixed = 16 + (size_t)B * (row_bytes + 16) + (has_resid ? (size_t)B * row_bytes : 0) +
                       kParts * (sizeof(float) * (size_t)p.rmax * bt + sizeof(int) * (size_t)p.cap +
                                 sizeof(float) * (size_t)p.cap * bt) + stage;
  const size_t limit = (size_t)dev_info().max_smem_optin;
  const size_t statics = 2048;  // static shared memory of the kernel + slack
  if (limit < fixed + statics + 2 * row_bytes + 1024) return p;
  int smax = (int)((limit - fixed - statics - 1024) / (row_bytes + 16 + 16));
  if (smax > 48) smax = 48;
  // Stage count: even (at least two producer threads), preferring, in this order, as many
  // dot-owner warps as possible (a divisor of S, at most 8), four producer threads (S a
  // multiple of 4; with two the copies are issued too slowly) and depth.
  for (int cand = smax; cand >= 2 && cand >= smax - 7; --cand) {
    if (cand & 1) continue;
    int cw = 1;
    for (int d = 1; d <= kConsumerWarps; ++d)
      if (cand % d == 0) cw = d;
    const int four = (cand % kMegaProducers == 0) ? 1 : 0;
    const int best_four = (p.S % kMegaProducers == 0) ? 1 : 0;
    if (p.S == 0 || cw > p.cw || (cw == p.cw && four > best_four)) {
      p.cw = cw;
      p.S = cand;
    }
  }
  if (p.mma_dot) {
    // the tensor-core path has no dot-owner warps: take the deepest ring that three or four
    // producer threads divide (an extra stage is worth about as much as the fourth producer)
    int best = 0, best_score = -1;
    for (int cand = smax; cand >= 8 && cand >= smax - 7; --cand) {
      const int np = cand % 4 == 0 ? 4 : cand % 3 == 0 ? 3 : 0;
      if (!np) continue;
      const int score = 2 * cand + (np == 4 ? 3 : 0);
      if (score > best_score) {
        best_score = score;
        best = cand;
      }
    }
    if (best) {
      p.S = best;
      p.cw = 1;
      for (int d = 1; d <= kConsumerWarps; ++d)
        if (best % d == 0) p.cw = d;
    }
  }
  if (p.S < 2) return p;
  if (p.S < 8) p.mma_dot = 0;  // a group of eight rows has to fit in the ring
  p.smem = align_up((size_t)p.S * (row_bytes + 16) + 8 * (size_t)(2 * p.S + 3 * kParts + 1), 16) + fixed;
  p.ok = p.smem + statics <= limit;
  return p;
}

cudaError_t do_mega(const MegaPlan& p, const MegaParams& P, MegaArgs A, WsPtrs ws, int dtype,
                    cudaStream_t st) {
  A.S = p.S;
  A.cw = p.cw;
  A.npw = (p.S % kMegaProducers == 0) ? kMegaProducers : (p.S % 3 == 0) ? 3 : 2;
  A.bulk_flush = p.bulk_flush;
  A.mma_dot = p.mma_dot;
  A.parts = p.parts;
  A.wait_kc = wait_kcycles();
  A.s_magic = (unsigned)(0x100000000ull / (unsigned)p.S) + 1u;
  // single GPU only: with the tensor-parallel exchange in the layer chain the look-ahead costs
  // more than it brings (two ranks, Mistral-7B shape: 34.3 us per layer with it, 32.1 without)
  A.pf_rows = (options().l2_ahead_kb > 0 && A.nranks == 0)
                  ? (int)((size_t)options().l2_ahead_kb * 1024 / ((size_t)A.H * esize(dtype)))
                  : 0;
  A.cap = p.cap;
  A.rmax = p.rmax;
  CATS_DISPATCH(dtype, inst_mega, p, P, A, ws, st);
}

// One layer, one token: which kernels cats_mlp launches.  The persistent kernel is a cooperative
// launch: it cannot overlap its start with the end of the kernel before it, and inside a decoder
// (attention kernels before and after every MLP) that costs more than its better streaming
// gains on a single layer.  The stage-1 / stage-2+3 pair is launched with programmatic dependent
// launch and runs a decoder's token 5-6 % faster (measured, Llama-2-7B and Mistral-7B shapes), so
// it is the default there; timed alone with an event pair per call the persistent kernel is
// 2-3 % ahead.  Stacks of layers (cats_mlp_stack) always take the persistent kernel.
bool single_layer_pair(int B, int H, int I, int dtype) {
  if (B != 1 || !options().single_pair || !options().use_tma) return false;
  return plan_gate_tma(B, H, I, dtype).ok && plan_updown_tma(B, H, I, dtype).ok;
}

// Dense tensor-core path: one row tile of at most 128 neurons per CTA and pass (two passes at the
// 70B shape), rings as deep as shared memory allows.
DensePlan plan_dense(int B, int H, int I, int dtype) {
  DensePlan p;
  // (H <= 8192: the tail keeps a token's row in the registers of 128 threads)
  if (dtype == CATS_F32 || B < 1 || B > 16 || H % 128 || I % 64 || H < 128 || H > 8192) return p;
  p.grid = dev_info().sms;
  if (p.grid > I / 8) p.grid = I / 8;
  if (p.grid < B) return p;                              // CTA b finishes token b
  const int rows = (I + p.grid - 1) / p.grid;            // most neurons any CTA owns
  const int tiles = (rows + 127) / 128;
  const int per_tile = (rows + tiles - 1) / tiles;
  p.box_rows = (per_tile + 7) / 8 * 8;
  if (p.box_rows > 128) p.box_rows = 128;
  const size_t limit = (size_t)dev_info().max_smem_optin - 4096;   // static shared memory + slack
  const size_t stf = 2 * 16384 + 4096;                             // one 36 KB stage
  p.Sf = (int)((limit - 1024) / stf);
  if (p.Sf > 16) p.Sf = 16;
  if (p.Sf < 2) return p;
  p.smemf = p.Sf * stf + 1024;
  p.wait_kc = wait_kcycles();
  p.ok = true;
  return p;
}

cudaError_t do_gate(const void* x, const void* Wg, WsPtrs ws, int B, int H, int I, int dtype,
                    float thr, void* gate_dense, uint8_t* flag_dense, cudaStream_t st,
                    const void* Wu_ahead = nullptr) {
  TmaPlan p = plan_gate_tma(B, H, I, dtype);
  if (Wu_ahead && options().pair_ahead_rows > 0) {
    p.pf_base = Wu_ahead;
    p.pf_n = options().pair_ahead_rows;
  }
  if (p.ok) CATS_DISPATCH(dtype, inst_gate_tma, p, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
  CATS_DISPATCH(dtype, inst_gate, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
}

cudaError_t do_updown(int mode, const void* x, const void* Wu, const void* WdT, WsPtrs ws, int B,
                      int H, int I, int dtype, void* out, int out_mode, void* resid, void* x_next,
                      const void* norm_w, float eps, void* inter_dense, cudaStream_t st) {
  if (mode == 3) {
    const TmaPlan p = plan_updown_tma(B, H, I, dtype);
    if (p.ok)
      CATS_DISPATCH(dtype, inst_updown_tma, p, x, Wu, WdT, ws, B, H, I, out, out_mode, resid,
                    x_next, norm_w, eps, st);
  }
  CATS_DISPATCH(dtype, inst_updown, mode, x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next,
                norm_w, eps, inter_dense, st);
}

int check_out_mode(int out_mode, const void* out, const void* resid, const void* x_next) {
  if (out_mode != CATS_OUT_STORE && out_mode != CATS_OUT_ACC_F32) return CATS_ERR_MODE;
  if (out_mode == CATS_OUT_ACC_F32 && (resid || x_next)) return CATS_ERR_MODE;
  if (x_next && !resid) return CATS_ERR_MODE;
  if (!out && !resid) return CATS_ERR_NULL;
  if (out && !aligned16(out)) return CATS_ERR_ALIGN;
  return CATS_OK;
}

}  // namespace

extern "C" {

int cats_abi_version(void) { return 1; }

const char* cats_status_string(int status) {
  switch (status) {
    case CATS_OK: return "ok";
    case CATS_ERR_DTYPE: return "unknown dtype (expected CATS_F32, CATS_F16 or CATS_BF16)";
    case CATS_ERR_SHAPE:
      return "bad shape (need 1 <= B <= 16, H >= 1, I >= 1 and rows that are a whole number of "
             "16-byte vectors)";
    case CATS_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case CATS_ERR_NULL: return "required pointer is NULL";
    case CATS_ERR_WORKSPACE: return "workspace is smaller than cats_workspace_bytes(B, H, I)";
    case CATS_ERR_CUDA: return "CUDA error at launch";
    case CATS_ERR_MODE: return "unsupported mode or flag combination";
    case CATS_ERR_STATIC_LIMIT:
      return "shape needs more scratch than the built-in array of cats_mlp_static holds "
             "(see cats_mlp_static_limit); use cats_mlp with a caller-provided workspace";
    default: return "unknown status";
  }
}

const char* cats_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda); }

int cats_sm_count(void) { return dev_info().sms; }

int cats_set_option(const char* name, int value) {
  if (!name) return CATS_ERR_NULL;
  if (!strcmp(name, "tma")) options().use_tma = value;
  else if (!strcmp(name, "ring_kb")) options().ring_kb = value;
  else if (!strcmp(name, "pdl")) g_use_pdl = value;
  else if (!strcmp(name, "mega")) options().use_mega = value;
  else if (!strcmp(name, "single_pair")) options().single_pair = value;
  else if (!strcmp(name, "pair_ahead_rows")) options().pair_ahead_rows = value;
  else if (!strcmp(name, "bulk_flush")) options().bulk_flush = value;
  else if (!strcmp(name, "mma_dot")) options().mma_dot = value;
  else if (!strcmp(name, "parts")) options().parts = value;
  else if (!strcmp(name, "wait_ms")) options().wait_ms = value;
  else if (!strcmp(name, "xchg")) options().xchg = value;
  else if (!strcmp(name, "local_lists")) options().local_lists = value;
  else if (!strcmp(name, "l2_ahead_kb")) options().l2_ahead_kb = value;
  else return CATS_ERR_MODE;
  return CATS_OK;
}

size_t cats_workspace_bytes(int B, int H, int I) {
  (void)B;
  if (H < 1 || I < 1) return 0;
  return ws_layout(nullptr, H, I, nullptr);
}

int cats_workspace_init(void* ws, size_t ws_bytes, void* stream) {
  if (!ws) return CATS_ERR_NULL;
  return cuda_status(cudaMemsetAsync(ws, 0, ws_bytes, static_cast<cudaStream_t>(stream)));
}

int cats_gate(const void* x, const void* Wg, void* ws, size_t ws_bytes, int B, int H, int I,
              int dtype, float threshold, void* gate_dense, uint8_t* flag_dense, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wg) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wg)) return CATS_ERR_ALIGN;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  return cuda_status(do_gate(x, Wg, p, B, H, I, dtype, threshold, gate_dense, flag_dense,
                             static_cast<cudaStream_t>(stream)));
}

int cats_compact(const void* values, const uint8_t* flags, void* ws, size_t ws_bytes, int B,
                 int H, int I, int dtype, float threshold, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!values) return CATS_ERR_NULL;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (dtype == CATS_F32)
    e = launch(k_compact<float>, dim3(1), dim3(1024), 0, st, (const float*)values, flags, p, B, I,
               threshold);
  else if (dtype == CATS_F16)
    e = launch(k_compact<__half>, dim3(1), dim3(1024), 0, st, (const __half*)values, flags, p, B,
               I, threshold);
  else
    e = launch(k_compact<__nv_bfloat16>, dim3(1), dim3(1024), 0, st,
               (const __nv_bfloat16*)values, flags, p, B, I, threshold);
  return cuda_status(e);
}

int cats_up(const void* x, const void* Wu, void* ws, size_t ws_bytes, int B, int H, int I,
            int dtype, void* inter_dense, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wu) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wu)) return CATS_ERR_ALIGN;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  return cuda_status(do_updown(1, x, Wu, nullptr, p, B, H, I, dtype, nullptr, CATS_OUT_STORE,
                               nullptr, nullptr, nullptr, 0.f, inter_dense,
                               static_cast<cudaStream_t>(stream)));
}

int cats_down(const void* WdT, void* ws, size_t ws_bytes, int B, int H, int I, int dtype,
              void* out, int out_mode, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!WdT || !out) return CATS_ERR_NULL;
  if (!aligned16(WdT)) return CATS_ERR_ALIGN;
  if ((s = check_out_mode(out_mode, out, nullptr, nullptr))) return s;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  return cuda_status(do_updown(2, nullptr, nullptr, WdT, p, B, H, I, dtype, out, out_mode,
                               nullptr, nullptr, nullptr, 0.f, nullptr,
                               static_cast<cudaStream_t>(stream)));
}

int cats_updown(const void* x, const void* Wu, const void* WdT, void* ws, size_t ws_bytes,
                int B, int H, int I, int dtype, void* out, int out_mode, void* resid,
                void* x_next, const void* norm_weight, float eps, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wu || !WdT) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wu) || !aligned16(WdT)) return CATS_ERR_ALIGN;
  if ((s = check_out_mode(out_mode, out, resid, x_next))) return s;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  return cuda_status(do_updown(3, x, Wu, WdT, p, B, H, I, dtype, out, out_mode, resid, x_next,
                               norm_weight, eps, nullptr, static_cast<cudaStream_t>(stream)));
}

int cats_mlp(const void* x, const void* Wg, const void* Wu, const void* WdT, void* ws,
             size_t ws_bytes, int B, int H, int I, int dtype, float threshold, void* out,
             int out_mode, void* resid, void* x_next, const void* norm_weight, float eps,
             void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wg || !Wu || !WdT) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(WdT)) return CATS_ERR_ALIGN;
  if ((s = check_out_mode(out_mode, out, resid, x_next))) return s;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_mode == CATS_OUT_STORE && !single_layer_pair(B, H, I, dtype)) {
    const MegaPlan mp = plan_mega(1, B, H, I, dtype, resid != nullptr);
    if (mp.ok) {
      MegaParams P;
      P.wg[0] = Wg;
      P.wu[0] = Wu;
      P.wdt[0] = WdT;
      P.nw[0] = norm_weight;
      P.thr[0] = threshold;
      MegaArgs A;
      memset(&A, 0, sizeof(A));
      A.L = 1; A.B = B; A.H = H; A.I = I; A.eps = eps;
      A.x_in = x; A.x_out = x_next; A.resid = resid; A.out_last = out;
      return cuda_status(do_mega(mp, P, A, p, dtype, st));
    }
  }
  cudaError_t e = do_gate(x, Wg, p, B, H, I, dtype, threshold, nullptr, nullptr, st, Wu);
  if (e != cudaSuccess) return cuda_status(e);
  return cuda_status(do_updown(3, x, Wu, WdT, p, B, H, I, dtype, out, out_mode, resid, x_next,
                               norm_weight, eps, nullptr, st));
}

int cats_mlp_dense(const void* x, const void* Wg, const void* Wu, const void* Wd, void* ws,
                   size_t ws_bytes, int B, int H, int I, int dtype, float threshold, void* out,
                   int out_mode, void* resid, void* x_next, const void* norm_weight, float eps,
                   void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wg || !Wu || !Wd) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(Wd)) return CATS_ERR_ALIGN;
  if ((s = check_out_mode(out_mode, out, resid, x_next))) return s;
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  const DensePlan dp = plan_dense(B, H, I, dtype);
  if (!dp.ok) return CATS_ERR_MODE;
  return cuda_status(inst_dense(dp, x, Wg, Wu, Wd, p, B, H, I, dtype, threshold, out, out_mode, resid,
                                x_next, norm_weight, eps, static_cast<cudaStream_t>(stream)));
}

int cats_mlp_stack_dense(int L, const void* const* Wg, const void* const* Wu, const void* const* Wd,
                         const float* thresholds, void* x_io, void* x_tmp, void* resid, void* ws,
                         size_t ws_bytes, int B, int H, int I, int dtype, float eps, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (L < 1) return CATS_ERR_SHAPE;
  if (!Wg || !Wu || !Wd || !thresholds || !x_io || !x_tmp || !resid) return CATS_ERR_NULL;
  if (!aligned16(x_io) || !aligned16(x_tmp) || !aligned16(resid)) return CATS_ERR_ALIGN;
  for (int l = 0; l < L; ++l) {
    if (!Wg[l] || !Wu[l] || !Wd[l]) return CATS_ERR_NULL;
    if (!aligned16(Wg[l]) || !aligned16(Wu[l]) || !aligned16(Wd[l])) return CATS_ERR_ALIGN;
  }
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  const DensePlan dp = plan_dense(B, H, I, dtype);
  if (!dp.ok) return CATS_ERR_MODE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // at most kDenseStackMaxLayers layers per launch; an odd-sized chunk leaves its result in x_io
  // as well (the kernel's last layer always writes x_io), so chunks chain without copies
  for (int l0 = 0; l0 < L; l0 += kDenseStackMaxLayers) {
    const int n = (L - l0 < kDenseStackMaxLayers) ? L - l0 : kDenseStackMaxLayers;
    cudaError_t e = inst_dense_stack(dp, n, Wg + l0, Wu + l0, Wd + l0, thresholds + l0, x_io, x_tmp,
                                     resid, p, B, H, I, dtype, eps, st);
    if (e != cudaSuccess) return cuda_status(e);
  }
  return CATS_OK;
}

int cats_dense_supported(int B, int H, int I, int dtype) {
  if (check_common(B, H, I, dtype)) return 0;
  return plan_dense(B, H, I, dtype).ok ? 1 : 0;
}

int cats_mlp_stack(int L, const void* const* Wg, const void* const* Wu, const void* const* WdT,
                   const float* thresholds, void* x_io, void* x_tmp, void* resid, void* ws,
                   size_t ws_bytes, int B, int H, int I, int dtype, float eps, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (L < 1) return CATS_ERR_SHAPE;
  if (!Wg || !Wu || !WdT || !thresholds || !x_io || !x_tmp || !resid) return CATS_ERR_NULL;
  if (!aligned16(x_io) || !aligned16(x_tmp) || !aligned16(resid)) return CATS_ERR_ALIGN;
  for (int l = 0; l < L; ++l) {
    if (!Wg[l] || !Wu[l] || !WdT[l]) return CATS_ERR_NULL;
    if (!aligned16(Wg[l]) || !aligned16(Wu[l]) || !aligned16(WdT[l])) return CATS_ERR_ALIGN;
  }
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I, &p))) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const MegaPlan mp = plan_mega(L, B, H, I, dtype, true);
  if (mp.ok) {
    MegaParams P;
    for (int l = 0; l < L; ++l) {
      P.wg[l] = Wg[l];
      P.wu[l] = Wu[l];
      P.wdt[l] = WdT[l];
      P.nw[l] = nullptr;
      P.thr[l] = thresholds[l];
    }
    MegaArgs A;
    memset(&A, 0, sizeof(A));
    A.L = L; A.B = B; A.H = H; A.I = I; A.eps = eps;
    A.x_in = x_io; A.x_out = x_io; A.resid = resid; A.out_last = nullptr;
    return cuda_status(do_mega(mp, P, A, p, dtype, st));
  }
  void* cur = x_io;
  void* nxt = x_tmp;
  for (int l = 0; l < L; ++l) {
    cudaError_t e = do_gate(cur, Wg[l], p, B, H, I, dtype, thresholds[l], nullptr, nullptr, st);
    if (e != cudaSuccess) return cuda_status(e);
    e = do_updown(3, cur, Wu[l], WdT[l], p, B, H, I, dtype, nullptr, CATS_OUT_STORE, resid, nxt,
                  nullptr, eps, nullptr, st);
    if (e != cudaSuccess) return cuda_status(e);
    void* t = cur;
    cur = nxt;
    nxt = t;
  }
  if (cur != x_io)
    return cuda_status(cudaMemcpyAsync(x_io, cur, (size_t)B * H * esize(dtype),
                                       cudaMemcpyDeviceToDevice, st));
  return CATS_OK;
}

// ---- tensor-parallel stack: compute and exchange in one persistent kernel per GPU --------------
size_t cats_tp_exchange_bytes(int H) { return H > 0 ? xchg_bytes(H) : 0; }

int cats_tp_exchange_alloc(int H, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64) return CATS_ERR_NULL;
  if (H <= 0) return CATS_ERR_SHAPE;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle is passed around as 64 bytes");
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, xchg_bytes(H));
  if (e == cudaSuccess) e = cudaMemset(d, 0, xchg_bytes(H));
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    if (d) cudaFree(d);
    return cuda_status(e);
  }
  memcpy(handle64, &h, 64);
  *ptr = d;
  return CATS_OK;
}

int cats_tp_exchange_open(const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) return CATS_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cuda_status(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int cats_tp_exchange_close(void* ptr) {
  return ptr ? cuda_status(cudaIpcCloseMemHandle(ptr)) : CATS_ERR_NULL;
}

int cats_tp_exchange_free(void* ptr) { return ptr ? cuda_status(cudaFree(ptr)) : CATS_ERR_NULL; }

int cats_tp_mlp_stack(int L, const void* const* Wg, const void* const* Wu, const void* const* WdT,
                      const float* thresholds, void* x_io, void* resid, void* ws, size_t ws_bytes,
                      int B, int H, int I_local, int dtype, float eps, int nranks, int rank,
                      void* const* exchange, void* stream) {
  int s = check_common(B, H, I_local, dtype);
  if (s) return s;
  if (L < 1 || nranks < 1 || nranks > kMaxRanks || rank < 0 || rank >= nranks || B > kMegaMaxB)
    return CATS_ERR_SHAPE;
  if (!Wg || !Wu || !WdT || !thresholds || !x_io || !resid || !exchange) return CATS_ERR_NULL;
  if (!aligned16(x_io) || !aligned16(resid)) return CATS_ERR_ALIGN;
  for (int l = 0; l < L; ++l) {
    if (!Wg[l] || !Wu[l] || !WdT[l]) return CATS_ERR_NULL;
    if (!aligned16(Wg[l]) || !aligned16(Wu[l]) || !aligned16(WdT[l])) return CATS_ERR_ALIGN;
  }
  for (int p = 0; p < nranks; ++p) {
    if (!exchange[p]) return CATS_ERR_NULL;
    if (((uintptr_t)exchange[p]) % 256) return CATS_ERR_ALIGN;
  }
  WsPtrs p;
  if ((s = check_ws(ws, ws_bytes, H, I_local, &p))) return s;
  const MegaPlan mp = plan_mega(L, B, H, I_local, dtype, true, true);
  // every rank has to run the same grid (the arrival counts are per source rank): one CTA per
  // SM, which needs at least that many rows per part
  if (!mp.ok || mp.grid != dev_info().sms) return CATS_ERR_MODE;
  MegaParams P;
  for (int l = 0; l < L; ++l) {
    P.wg[l] = Wg[l];
    P.wu[l] = Wu[l];
    P.wdt[l] = WdT[l];
    P.nw[l] = nullptr;
    P.thr[l] = thresholds[l];
  }
  MegaArgs A;
  memset(&A, 0, sizeof(A));
  A.L = L; A.B = B; A.H = H; A.I = I_local; A.eps = eps;
  A.x_in = x_io; A.x_out = x_io; A.resid = resid; A.out_last = nullptr;
  A.nranks = nranks; A.rank = rank;
  // up to two ranks a CTA reads at most twice what the totals would be and saves a hand-off
  A.xchg_all = options().xchg == 1 ? 1 : options().xchg == 2 ? 0 : (nranks <= 2 ? 1 : 0);
  A.local = (options().local_lists && mp.parts == 1) ? 1 : 0;
  for (int q = 0; q < nranks; ++q) A.xchg[q] = static_cast<unsigned char*>(exchange[q]);
  return cuda_status(do_mega(mp, P, A, p, dtype, static_cast<cudaStream_t>(stream)));
}

int cats_uses_persistent_kernel(int L, int B, int H, int I, int dtype) {
  if (check_common(B, H, I, dtype)) return 0;
  if (L == 1 && single_layer_pair(B, H, I, dtype)) return 0;
  return plan_mega(L, B, H, I, dtype, true).ok ? 1 : 0;
}

// ---- entry point for callers that cannot allocate device memory --------------------------------
// Scratch for cats_mlp_static lives in this file-scope array: it is part of the loaded module, so
// every GPU that loads the library carries it until the process exits, and nobody ever has to
// allocate it.  kStaticWsBytes is the documented limit of that entry point.
constexpr size_t kStaticWsBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

namespace {
// In host code `g_static_ws` is only a handle for the runtime, not an address a kernel can use:
// the device address has to be asked for, once per device, with that device current.
void* g_static_ws_dev[64];
bool g_static_ws_ready[64];
std::mutex g_static_ws_mutex;

int static_ws_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= 64) return CATS_ERR_SHAPE;
  std::lock_guard<std::mutex> lock(g_static_ws_mutex);
  if (!g_static_ws_ready[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_ws);
    if (e != cudaSuccess) return cuda_status(e);
    if (!ptr) return CATS_ERR_NULL;
    g_static_ws_dev[dev] = ptr;
    g_static_ws_ready[dev] = true;
  }
  *out = g_static_ws_dev[dev];
  return CATS_OK;
}
}  // namespace

size_t cats_mlp_static_limit(void) { return kStaticWsBytes; }

int cats_mlp_static(const void* x, const void* Wg, const void* Wu, const void* WdT, int B, int H,
                    int I, int dtype, float threshold, void* out, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  if (!x || !Wg || !Wu || !WdT || !out) return CATS_ERR_NULL;
  if (!aligned16(x) || !aligned16(Wg) || !aligned16(Wu) || !aligned16(WdT) || !aligned16(out))
    return CATS_ERR_ALIGN;
  // the size check comes first: a shape whose scratch does not fit is refused, never truncated
  if (ws_layout(nullptr, H, I, nullptr) > kStaticWsBytes) return CATS_ERR_STATIC_LIMIT;
  void* base = nullptr;
  if ((s = static_ws_for_current_device(&base))) return s;
  WsPtrs p;
  ws_layout(base, H, I, &p);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array still holds whatever the previous call (of any caller) left in it.  What the
  // kernels need to find zero is cleared here, in stream order: the completion ticket and the
  // fp32 accumulators of the B tokens.  The sticky status word is left alone.
  cudaError_t e = cudaMemsetAsync(p.hdr + HDR_TICKET, 0, sizeof(int), st);
  if (e == cudaSuccess) e = cudaMemsetAsync(p.acc32, 0, sizeof(float) * (size_t)B * H, st);
  if (e != cudaSuccess) return cuda_status(e);
  e = do_gate(x, Wg, p, B, H, I, dtype, threshold, nullptr, nullptr, st);
  if (e != cudaSuccess) return cuda_status(e);
  return cuda_status(do_updown(3, x, Wu, WdT, p, B, H, I, dtype, out, CATS_OUT_STORE, nullptr,
                               nullptr, nullptr, 0.f, nullptr, st));
}

int cats_mlp_static_status(int* device_status, void* stream) {
  if (!device_status) return CATS_ERR_NULL;
  void* base = nullptr;
  int s = static_ws_for_current_device(&base);
  if (s) return s;
  return cats_read_counters(base, nullptr, device_status, stream);
}

int cats_down_dense(const void* inter, const void* Wd, int B, int H, int I, int dtype, void* out,
                    void* stream) {
  // rows of Wd [H, I] have length I: the vector-width rule applies to I here
  int s = check_common(B, I, H, dtype);
  if (s) return s;
  if (!inter || !Wd || !out) return CATS_ERR_NULL;
  if (!aligned16(inter) || !aligned16(Wd)) return CATS_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto go = [&]() -> cudaError_t {
    CATS_DISPATCH(dtype, inst_rows_gemv, inter, Wd, B, I, H, out, st);
  };
  return cuda_status(go());
}

int cats_tail(const void* y, void* resid, void* x_next, const void* norm_weight, float eps, int B,
              int H, int dtype, void* stream) {
  if (dtype != CATS_F32 && dtype != CATS_F16 && dtype != CATS_BF16) return CATS_ERR_DTYPE;
  if (B < 1 || H < 1) return CATS_ERR_SHAPE;
  if (!y || !resid) return CATS_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (dtype == CATS_F32)
    e = launch(k_tail<float>, dim3(B), dim3(kThreads), 0, st, (const float*)y, (float*)resid,
               (float*)x_next, (const float*)norm_weight, eps, H);
  else if (dtype == CATS_F16)
    e = launch(k_tail<__half>, dim3(B), dim3(kThreads), 0, st, (const __half*)y, (__half*)resid,
               (__half*)x_next, (const __half*)norm_weight, eps, H);
  else
    e = launch(k_tail<__nv_bfloat16>, dim3(B), dim3(kThreads), 0, st, (const __nv_bfloat16*)y,
               (__nv_bfloat16*)resid, (__nv_bfloat16*)x_next, (const __nv_bfloat16*)norm_weight,
               eps, H);
  return cuda_status(e);
}

int cats_rope_cache(const void* qkv, const void* cos_table, const void* sin_table,
                    const long long* position, void* q_out, void* k_cache, void* v_cache, int B,
                    int n_heads, int n_kv_heads, int head_dim, int max_len, int dtype, void* stream) {
  if (dtype != CATS_F32 && dtype != CATS_F16 && dtype != CATS_BF16) return CATS_ERR_DTYPE;
  if (B < 1 || n_heads < 1 || n_kv_heads < 1 || head_dim < 2 || head_dim % 2 || max_len < 1)
    return CATS_ERR_SHAPE;
  if (!qkv || !cos_table || !sin_table || !position || !q_out || !k_cache || !v_cache)
    return CATS_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int warps = B * (n_heads + 2 * n_kv_heads);
  const dim3 grid((warps + kWarps - 1) / kWarps), block(kThreads);
  cudaError_t e;
  if (dtype == CATS_F32)
    e = launch(k_rope_cache<float>, grid, block, 0, st, (const float*)qkv, (const float*)cos_table,
               (const float*)sin_table, position, (float*)q_out, (float*)k_cache, (float*)v_cache, B,
               n_heads, n_kv_heads, head_dim, max_len);
  else if (dtype == CATS_F16)
    e = launch(k_rope_cache<__half>, grid, block, 0, st, (const __half*)qkv, (const __half*)cos_table,
               (const __half*)sin_table, position, (__half*)q_out, (__half*)k_cache, (__half*)v_cache,
               B, n_heads, n_kv_heads, head_dim, max_len);
  else
    e = launch(k_rope_cache<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)qkv,
               (const __nv_bfloat16*)cos_table, (const __nv_bfloat16*)sin_table, position,
               (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, B, n_heads,
               n_kv_heads, head_dim, max_len);
  return cuda_status(e);
}

int cats_transpose(const void* src, void* dst, int rows, int cols, int dtype, void* stream) {
  if (dtype != CATS_F32 && dtype != CATS_F16 && dtype != CATS_BF16) return CATS_ERR_DTYPE;
  if (rows < 1 || cols < 1) return CATS_ERR_SHAPE;
  if (!src || !dst) return CATS_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (esize(dtype) == 4)
    k_transpose<uint32_t><<<grid, block, 0, st>>>((const uint32_t*)src, (uint32_t*)dst, rows, cols);
  else
    k_transpose<uint16_t><<<grid, block, 0, st>>>((const uint16_t*)src, (uint16_t*)dst, rows, cols);
  return cuda_status(cudaGetLastError());
}

int cats_histogram(const void* values, size_t n, int dtype, const float* edges, int n_edges,
                   unsigned long long* counts, int take_abs, void* stream) {
  if (dtype != CATS_F32 && dtype != CATS_F16 && dtype != CATS_BF16) return CATS_ERR_DTYPE;
  if (n_edges < 2 || n_edges > kHistMaxEdges) return CATS_ERR_SHAPE;
  if (!edges || !counts || (!values && n)) return CATS_ERR_NULL;
  if (((uintptr_t)values) % esize(dtype)) return CATS_ERR_ALIGN;
  if (n == 0) return CATS_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = hist_smem_bytes(n_edges);
  const size_t per_block = (size_t)kHistThreads * 16 / esize(dtype) * 2;  // 2 vectors per thread
  size_t blocks = (n + per_block - 1) / per_block;
  if (blocks > (size_t)dev_info().sms) blocks = (size_t)dev_info().sms;  // one CTA per SM
  const dim3 grid((unsigned)blocks), block(kHistThreads);
  cudaError_t e;
#define CATS_HIST_LAUNCH(T)                                                                      \
  do {                                                                                           \
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(k_histogram<T>),                      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    if (e == cudaSuccess)                                                                        \
      k_histogram<T><<<grid, block, smem, st>>>((const T*)values, n, edges, n_edges, counts,     \
                                                take_abs);                                       \
  } while (0)
  if (dtype == CATS_F32) CATS_HIST_LAUNCH(float);
  else if (dtype == CATS_F16) CATS_HIST_LAUNCH(__half);
  else CATS_HIST_LAUNCH(__nv_bfloat16);
#undef CATS_HIST_LAUNCH
  if (e != cudaSuccess) return cuda_status(e);
  return cuda_status(cudaGetLastError());
}

int cats_histogram_threshold(const unsigned long long* counts, const float* edges, int n_edges,
                             float sparsity, float* threshold, void* stream) {
  if (n_edges < 2 || n_edges > kHistMaxEdges) return CATS_ERR_SHAPE;
  if (!counts || !edges || !threshold) return CATS_ERR_NULL;
  k_hist_threshold<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(counts, edges, n_edges, sparsity,
                                                                    threshold);
  return cuda_status(cudaGetLastError());
}

int cats_read_counters(const void* ws, int* n_active, int* device_status, void* stream) {
  if (!ws) return CATS_ERR_NULL;
  // header and segment counts sit at the start of the workspace whatever (H, I) are
  static_assert(sizeof(int) * kHdrInts % 256 == 0, "header must keep 256-byte alignment");
  int host[kHdrInts + kMaxSeg];
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(host, ws, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_status(e);
  int nseg = host[HDR_NSEG];
  if (nseg > kMaxSeg) nseg = kMaxSeg;
  long long n = 0;
  if (nseg < 0) n = host[HDR_NACTIVE];  // left by the persistent kernel (last layer's total)
  for (int c = 0; c < nseg; ++c) n += host[kHdrInts + c];
  if (n_active) *n_active = (int)n;
  if (device_status) *device_status = host[HDR_STATUS];
  return CATS_OK;
}

int cats_export_list(const void* ws, size_t ws_bytes, int B, int H, int I, int dtype,
                     int64_t* idx_out, void* val_out, void* stream) {
  int s = check_common(B, H, I, dtype);
  if (s) return s;
  WsPtrs p;
  if ((s = check_ws(const_cast<void*>(ws), ws_bytes, H, I, &p))) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int g = (I + kThreads - 1) / kThreads;
  if (g > dev_info().sms) g = dev_info().sms;
  cudaError_t e;
  if (dtype == CATS_F32)
    e = launch(k_export<float>, dim3(g), dim3(kThreads), 0, st, p, B, I, (long long*)idx_out,
               (float*)val_out);
  else if (dtype == CATS_F16)
    e = launch(k_export<__half>, dim3(g), dim3(kThreads), 0, st, p, B, I, (long long*)idx_out,
               (__half*)val_out);
  else
    e = launch(k_export<__nv_bfloat16>, dim3(g), dim3(kThreads), 0, st, p, B, I,
               (long long*)idx_out, (__nv_bfloat16*)val_out);
  return cuda_status(e);
}

}  // extern "C"
