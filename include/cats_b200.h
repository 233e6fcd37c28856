/*
 * cats_b200.h — C ABI of the B200 (sm_100a) CATS sparse-MLP decode kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, allocates nothing,
 * never synchronises the device and never terminates the process.  The return value is a
 * status code (CATS_OK == 0; negative values are argument errors detected on the host before
 * any launch; CATS_ERR_CUDA reports a failed launch).  `cats_status_string` turns it into text.
 *
 * Tensor layouts (row-major, contiguous):
 *   x        [B, H]   activations, B = batch * seq (decode: seq == 1), 1 <= B <= 16
 *   Wg, Wu   [I, H]   nn.Linear.weight layout of gate_proj / up_proj (one neuron per row)
 *   WdT      [I, H]   down_proj.weight transposed: intermediate-major, one neuron per row
 *   Wd       [H, I]   down_proj.weight as stored by nn.Linear (dense fallback only)
 *   out      [B, H]
 * All rows must be 16-byte aligned: base pointers 16-byte aligned and H * sizeof(element) a
 * multiple of 16 (H % 8 == 0 for fp16/bf16, H % 4 == 0 for fp32).
 *
 * Semantics replaced (reference = ScalingIntelligence/CATS):
 *   out = Wd * ( mask(SiLU(Wg x)) * (Wu x) ),  mask keeps v where |v| > threshold (strict) and
 *   zeroes it otherwise — experiments/models/sparse_silu/ugly_utils.py:896-899.
 */
#ifndef CATS_B200_H_
#define CATS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of x / weights / out */
enum { CATS_F32 = 0, CATS_F16 = 1, CATS_BF16 = 2 };

/* status codes */
enum {
  CATS_OK = 0,
  CATS_ERR_DTYPE = -1,      /* unknown dtype enum */
  CATS_ERR_SHAPE = -2,      /* B, H or I out of range, or H not a multiple of the 16-byte vector */
  CATS_ERR_ALIGN = -3,      /* a pointer is not 16-byte aligned */
  CATS_ERR_NULL = -4,       /* a required pointer is NULL */
  CATS_ERR_WORKSPACE = -5,  /* workspace too small for (B, H, I) */
  CATS_ERR_CUDA = -6,       /* CUDA runtime reported an error at launch; see cats_last_cuda_error */
  CATS_ERR_MODE = -7,       /* unknown mode / flag combination */
  CATS_ERR_STATIC_LIMIT = -8 /* cats_mlp_static: shape needs more scratch than its built-in array */
};

/* how cats_down / cats_updown / cats_mlp deliver the result */
enum {
  CATS_OUT_STORE = 0,     /* out[B,H] (element type = dtype) is overwritten                        */
  CATS_OUT_ACC_F32 = 1    /* out[B,H] is fp32 and the result is ADDED to it (caller pre-zeroes),   */
                          /* the convention of the reference's atomic ops                           */
};

/* ABI version of this header (bumped when a signature changes). */
int cats_abi_version(void);

/* Text for a status code. */
const char* cats_status_string(int status);

/* Text of the CUDA error behind the most recent CATS_ERR_CUDA on the calling thread. */
const char* cats_last_cuda_error(void);

/* Number of SMs of the current device (the persistent grids are sized from it). */
int cats_sm_count(void);

/*
 * Tuning knob, process-wide.  "tma" (0/1): use the TMA-fed kernels where the shape allows
 * (default 1; 0 forces the direct-load kernels).  "ring_kb": shared-memory ring per TMA kernel in
 * KiB (default 200).  "pdl" (0/1): launch with programmatic dependent launch (default 1).
 * "mega" (0/1): run cats_mlp / cats_mlp_stack as one persistent cooperative kernel where the
 * shape allows (default 1; 0 = one stage-1 and one stage-2/3 launch per layer).  "single_pair"
 * (0/1, default 1): cats_mlp with ONE token launches the stage-1 / stage-2+3 kernel pair with
 * programmatic dependent launch instead of the (cooperative) persistent kernel - between other
 * kernels of a stream, as in a decoder, the pair is the faster of the two; cats_mlp_stack is not
 * affected.  "pair_ahead_rows" (default 16, 0 = off): in that pair, stage 1 asks the up-projection
 * rows of each segment's first active neurons into L2 for the stage-2 kernel, whose first copies
 * would otherwise wait for HBM after an idle gap.  Inside the
 * persistent kernel: "bulk_flush" (0/1, default 1: accumulators leave through TMA bulk reduces),
 * "mma_dot" (0/1, default 1: tensor-core dot products for batches of 2-4 with 16-bit weights),
 * "parts" (0 = automatic, or 1..3 parts per layer).  "wait_ms": limit of every wait inside a
 * kernel (on a shared-memory barrier, a grid barrier, another rank's data), default 1000; a wait
 * that runs out makes the kernel leave in an orderly way and sets the device status word (see
 * cats_read_counters); waits for other ranks get four times the limit.  "xchg": how the ranks'
 * partial sums are combined in cats_tp_mlp_stack (0 = chosen by the number of ranks, 1 = every
 * CTA adds all ranks' partial sums, 2 = every CTA adds its own slice and publishes the total;
 * all ranks must use the same value).  "local_lists" (0/1, default 1): in cats_tp_mlp_stack, when
 * a rank's slice leaves a CTA too few rows to split a layer into parts, every CTA works on the
 * active neurons of its own rows (no list barrier) instead of a balanced share.  "l2_ahead_kb"
 * (default 128, 0 = off): how many KiB of its coming gate rows a CTA of the persistent kernel asks
 * into L2 when its copy ring has stood still for about two microseconds (the consumers are at a
 * grid barrier then and HBM would idle); not used by cats_tp_mlp_stack.  The same values are read
 * once from the environment variables CATS_B200_TMA, CATS_B200_RING_KB, CATS_B200_PDL,
 * CATS_B200_MEGA, CATS_B200_BULK_FLUSH, CATS_B200_MMA_DOT, CATS_B200_PARTS, CATS_B200_WAIT_MS
 * CATS_B200_XCHG, CATS_B200_LOCAL_LISTS, CATS_B200_L2_AHEAD_KB, CATS_B200_SINGLE_PAIR and CATS_B200_PAIR_AHEAD_ROWS.
 * No reference counterpart (the reference has no device-side waits; its error path is exit(-1),
 * flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:25-33, 2397-2400).
 */
int cats_set_option(const char* name, int value);

/*
 * Workspace.  One workspace serves every call with batch <= B, hidden <= H, intermediate <= I
 * made in stream order on one stream; it holds the compacted active-neuron list, the per-neuron
 * gate values, fp32 split-K accumulators and a self-resetting completion ticket.  It has to be
 * cleared once with cats_workspace_init before first use; afterwards the kernels leave it clean.
 * Replaces the per-call cudaMalloc/cudaFree of two scratch buffers in
 * flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:2351-2354, 2402-2403.
 */
size_t cats_workspace_bytes(int B, int H, int I);
int cats_workspace_init(void* ws, size_t ws_bytes, void* stream);

/*
 * Stage 1 — fused gate GEMV + SiLU + |v| > threshold + warp-ballot compaction.
 * Streams all of Wg once.  Leaves in the workspace the ordered list of neurons that are active
 * for at least one of the B tokens and, per list entry and token, the fp32 gate value (0 where
 * that token's own mask is off).  Optional dense outputs, either may be NULL:
 *   gate_dense [B, I] (dtype)  SiLU(Wg x) of every neuron, rounded to dtype
 *   flag_dense [B, I] (uint8)  1 where |SiLU(Wg x)| > threshold
 * Replaces fuse_gemv_flag_local (flash_gemv/flash_gemv/flash_gemv.py:21-22;
 * fuse_gemv_cmp_cuda.cu:1292-1486, 2083-2117) and the stage-1 launches of
 * flag_gemv_gemv_inner* (fuse_gemv_cmp_cuda.cu:2369, 2446, 2523).
 */
int cats_gate(const void* x, const void* Wg, void* ws, size_t ws_bytes, int B, int H, int I,
              int dtype, float threshold, void* gate_dense, uint8_t* flag_dense, void* stream);

/*
 * Build the workspace's active list from a dense gate tensor instead of stage 1.
 *   values [B, I] (dtype); flags [B, I] uint8 or NULL.
 * With flags == NULL a neuron is active for token b when |values[b,i]| > threshold, otherwise
 * when flags[b,i] != 0 (threshold ignored).  H is the hidden size of the stage-2/3 calls that
 * will consume the list (it fixes the workspace layout).  Serves the reference entry points that receive a
 * precomputed SiLU(x Wg): gemv_gemv_triton (flash_gemv/flash_gemv/__init__.py:45-48),
 * fuse_flag_gemv_local and atomic_gemv (flash_gemv/flash_gemv/flash_gemv.py:24-28).
 */
int cats_compact(const void* values, const uint8_t* flags, void* ws, size_t ws_bytes, int B,
                 int H, int I, int dtype, float threshold, void* stream);

/*
 * Stage 2 — gather GEMV over the active rows of Wu, times the gate value.
 * Consumes the list left by cats_gate / cats_compact; leaves h = gate * (Wu x) per list entry
 * in the workspace for cats_down.  Optional inter_dense [B, I] (dtype) receives the same values
 * scattered to their neuron positions (inactive positions are NOT written: clear it first).
 * Replaces fuse_flag_gemv_local (fuse_gemv_cmp_cuda.cu:1507-1722, 2123-2156).
 */
int cats_up(const void* x, const void* Wu, void* ws, size_t ws_bytes, int B, int H, int I,
            int dtype, void* inter_dense, void* stream);

/*
 * Stage 3 — down projection over the active rows of WdT [I, H] (split-K, fp32 accumulation).
 * Consumes the list and h left by cats_up (or by cats_compact, whose values then act as h).
 * Replaces atomic_gemv (fuse_gemv_cmp_cuda.cu:1724-1783, 2162-2194) and the Triton
 * gather_transposed_gemv_flag_3d (flash_gemv/flash_gemv/kernels.py:256-462).
 */
int cats_down(const void* WdT, void* ws, size_t ws_bytes, int B, int H, int I, int dtype,
              void* out, int out_mode, void* stream);

/*
 * Stages 2+3 in one launch: each CTA computes h for its share of the active list and
 * immediately streams the matching WdT rows.  Optional fused decoder-layer tail (either NULL):
 *   resid  [B, H] (dtype)  residual stream, updated in place: resid += mlp_out
 *   x_next [B, H] (dtype)  RMS-normalised new residual: resid / sqrt(mean(resid^2) + eps),
 *                          times norm_weight[H] (dtype) when that is not NULL
 * (resid/x_next require out_mode == CATS_OUT_STORE; `out` may be NULL when resid is given.)
 * Ordering: x must be final before the launch that precedes this one in the stream has started
 * (true when that launch is this layer's cats_gate or cats_compact, which read the same x): the
 * kernel copies x into shared memory before it waits for its predecessor to finish.
 */
int cats_updown(const void* x, const void* Wu, const void* WdT, void* ws, size_t ws_bytes,
                int B, int H, int I, int dtype, void* out, int out_mode, void* resid,
                void* x_next, const void* norm_weight, float eps, void* stream);

/*
 * The whole CATS MLP for decode: cats_gate followed by cats_updown with programmatic dependent
 * launch between them.  Replaces flag_gemv_gemv_inner / _fp32 / _bf16
 * (flash_gemv/flash_gemv/flash_gemv.py:36-43; fuse_gemv_cmp_cuda.cu:2330-2560), which take
 * Wd [H, I]; here the caller passes the pre-packed WdT [I, H].
 */
int cats_mlp(const void* x, const void* Wg, const void* Wu, const void* WdT, void* ws,
             size_t ws_bytes, int B, int H, int I, int dtype, float threshold, void* out,
             int out_mode, void* resid, void* x_next, const void* norm_weight, float eps,
             void* stream);

/*
 * The CATS MLP for batches, on the tensor cores: all of Wg, Wu and Wd are streamed once (TMA into
 * shared memory, tcgen05.mma with the accumulators in tensor memory) and every token's own mask
 * |SiLU(gate)| > threshold is applied to its own products, the rule of the reference's batched
 * kernels (fuse_gemv_cmp_cuda.cu:1542-1548).  For batches whose tokens' active sets together cover
 * (nearly) every neuron - with independent masks at 50 % that is any batch from about four up -
 * nothing is left to skip and this is the fastest way through the weights; cats_mlp remains the
 * path for one token and for batches with strongly overlapping masks.
 *   Wd [H, I]: down_proj.weight as nn.Linear stores it, the layout flag_gemv_gemv_inner* receive
 *   (flash_gemv/flash_gemv/flash_gemv.py:36-43); Wg, Wu [I, H]; everything else as for cats_mlp.
 * fp16 / bf16 only (fp32 weights would have to go through tf32), H a multiple of 128 and at most
 * 8192, I a multiple of 64 (and at least 8 * B), B <= 16: otherwise CATS_ERR_MODE (cats_dense_supported tells beforehand) and the
 * caller uses cats_mlp.  gate * up is rounded to the storage type between the two GEMMs, as the
 * reference's stage 2 hands it to its stage 3.
 * Replaces the B in {2, 8, 16} launches of flag_gemv_gemv_inner* (fuse_gemv_cmp_cuda.cu:2368-2400).
 */
int cats_mlp_dense(const void* x, const void* Wg, const void* Wu, const void* Wd, void* ws,
                   size_t ws_bytes, int B, int H, int I, int dtype, float threshold, void* out,
                   int out_mode, void* resid, void* x_next, const void* norm_weight, float eps,
                   void* stream);
int cats_dense_supported(int B, int H, int I, int dtype);

/*
 * cats_mlp_stack on the dense tensor-core path: L layers (Wd[l] is [H, I]) chained through the
 * fused residual + RMS-norm tail in one cooperative launch per 80 layers, the weight stream kept
 * full across layers.  Arguments as for cats_mlp_stack; restrictions as for cats_mlp_dense.
 * No reference counterpart as one call (see cats_mlp_stack).
 */
int cats_mlp_stack_dense(int L, const void* const* Wg, const void* const* Wu, const void* const* Wd,
                         const float* thresholds, void* x_io, void* x_tmp, void* resid, void* ws,
                         size_t ws_bytes, int B, int H, int I, int dtype, float eps, void* stream);

/*
 * cats_mlp for callers that are not able to allocate device memory.
 *
 * Who that is: code that runs where cudaMalloc is off limits or not reachable at all - a plugin
 * that is handed input and output buffers by a host application and owns no allocator of its own,
 * a runtime that forbids allocation after start-up (fixed memory budgets, real-time loops), a
 * binding in a language where wrapping one more device buffer is more trouble than it is worth.
 * cats_mlp needs a workspace from the caller; this entry point brings its own: an 8 MiB array
 * that is compiled into the library (a `static __device__` array), so every GPU that loads the
 * library holds it until the process ends and nothing is allocated at any time - no cudaMalloc,
 * no cudaFree, no allocating library call.  The caller passes only inputs and the output.
 *
 * Limit: the scratch of a shape is cats_workspace_bytes(B, H, I); shapes that need more than
 * cats_mlp_static_limit() bytes (8 MiB: hidden 8192 x intermediate 28672 still fits) are refused
 * with CATS_ERR_STATIC_LIMIT before anything is launched.
 *
 * Rules of use:
 *   - The first call on a device looks up the array's device address (once per device, with that
 *     device current).  Make that first call before you start capturing a stream.
 *   - All calls on one device share the one array and it keeps the previous call's contents; each
 *     call clears, in stream order, the parts that have to start at zero.  Two calls that overlap
 *     on the GPU (different streams, no ordering between them) race on it: keep the calls of a
 *     device in one stream or order them with events.
 *   - out[B, H] has the element type dtype and is overwritten; arguments as for cats_mlp.
 *   - A wait inside the kernels that ran out ("wait_ms") leaves a sticky status word in the
 *     array; cats_mlp_static_status reads it (it blocks until `stream` is idle).  No call clears
 *     it: after a non-zero status the process should stop using this entry point on that device.
 * This entry point has no counterpart in the reference (its ops allocate their scratch with
 * cudaMalloc on every call).
 */
int cats_mlp_static(const void* x, const void* Wg, const void* Wu, const void* WdT, int B, int H,
                    int I, int dtype, float threshold, void* out, void* stream);

/* Size in bytes of the built-in scratch array of cats_mlp_static. */
size_t cats_mlp_static_limit(void);

/* Device status word of the built-in array on the current device (0 = no wait ever ran out). */
int cats_mlp_static_status(int* device_status, void* stream);

/*
 * A stack of L CATS MLP layers chained through the fused residual + RMS-norm tail, launched
 * back to back without returning to the caller: layer l reads x_l, updates resid in place and
 * writes x_{l+1}.  Pointer arrays live in HOST memory and hold device pointers.
 *   x_io [B, H]: input of layer 0 on entry, RMS-normalised residual after layer L-1 on return.
 * No reference counterpart as one call: it is the loop `for layer in model.layers: mlp(...)`
 * of the decoder (experiments/models/sparse_silu/ugly_utils.py:1036-1057) for the MLP halves.
 */
int cats_mlp_stack(int L, const void* const* Wg, const void* const* Wu, const void* const* WdT,
                   const float* thresholds, void* x_io, void* x_tmp, void* resid, void* ws,
                   size_t ws_bytes, int B, int H, int I, int dtype, float eps, void* stream);

/*
 * Tensor parallelism over the intermediate dimension, compute and exchange in ONE kernel per GPU.
 * Rank r of nranks (<= 8, one process per GPU of one NVLink-connected node) holds rows
 * [I*r/nranks, I*(r+1)/nranks) of every layer's Wg, Wu and WdT (I_local rows; the thresholds are
 * the unsharded ones) and runs cats_tp_mlp_stack at the same time as its peers: the persistent
 * kernel of cats_mlp_stack, whose CTAs, at the end of every layer, store their slice of this
 * rank's partial sums straight into every peer's exchange buffer over NVLink (plain peer stores
 * of 8-byte value + layer-tag pairs, every pair one 64-bit element of its store and of its load,
 * so no fence, flag or counter is needed on either side; no TMA involved), add the ranks'
 * partial sums of that slice in rank order as they arrive in their own buffer - every rank
 * computes bit-identical residuals and inputs for the next layer - and publish the total, tagged
 * the same way, to the other CTAs of their GPU.  x_io / resid [B, H] as for cats_mlp_stack,
 * replicated on every rank.  B <= 4.
 *
 * exchange[p] (host array of nranks device pointers) is rank p's exchange buffer as mapped into
 * the calling process; exchange[rank] is the caller's own.  Every rank creates its buffer with
 * cats_tp_exchange_alloc (cudaMalloc + clear + CUDA IPC handle, 64 bytes), passes the handle to
 * its peers by any host channel, and maps theirs with cats_tp_exchange_open.  All ranks must make
 * the same sequence of cats_tp_mlp_stack calls (same L, B, H) on a set of buffers.
 * A rank whose peers never arrive gives up after 4 x "wait_ms" (bounded wait): the call still
 * returns CATS_OK (it is asynchronous) and cats_read_counters reports a non-zero device status.
 * After a non-zero device status the workspace AND every rank's exchange buffer are invalid (the
 * ranks' layer tags no longer agree): all ranks free their buffers, allocate and exchange new
 * ones and clear their workspaces before the next call.
 * CATS_ERR_MODE: the shape cannot run as one persistent kernel with one CTA per SM on this GPU
 * (then use one all-reduce per layer around cats_mlp instead).  nranks == 1 is allowed (the
 * exchange then runs against the caller's own buffer).
 * No reference counterpart: the reference has no tensor parallelism (its multi-GPU inference
 * mode is layer placement, experiments/bench_sparse_inference_llama.py:36).
 */
size_t cats_tp_exchange_bytes(int H);
int cats_tp_exchange_alloc(int H, void** ptr, unsigned char* handle64);
int cats_tp_exchange_open(const unsigned char* handle64, void** ptr);
int cats_tp_exchange_close(void* ptr);
int cats_tp_exchange_free(void* ptr);
int cats_tp_mlp_stack(int L, const void* const* Wg, const void* const* Wu, const void* const* WdT,
                      const float* thresholds, void* x_io, void* resid, void* ws, size_t ws_bytes,
                      int B, int H, int I_local, int dtype, float eps, int nranks, int rank,
                      void* const* exchange, void* stream);

/*
 * 1 if cats_mlp_stack runs these L layers as ONE persistent cooperative launch on the current
 * device (shape, batch and options permitting), 0 if it launches two kernels per layer.
 * For reporting (benchmarks count their kernel launches with it).  No reference counterpart.
 */
int cats_uses_persistent_kernel(int L, int B, int H, int I, int dtype);

/*
 * Activation histogram on the device: counts[b] += |{ i : edges[b] <= v_i < edges[b+1] }| for the
 * n values at `values` (element type dtype), the last bin closed on the right and values outside
 * [edges[0], edges[n_edges-1]] (and NaNs) ignored: torch.histogram's rule.  take_abs != 0 bins
 * |v_i|.  edges: n_edges <= 1024 ascending fp32 values in device memory (+-inf allowed at the
 * ends); counts: n_edges - 1 64-bit counters in device memory, accumulated into (the caller
 * zeroes them once).  Replaces the two torch.histogram calls of collect_stats
 * (experiments/models/sparse_silu/ugly_utils.py:514-522), which first copy both activation
 * tensors to the host: pre-activations with take_abs = 0, post-activations with take_abs = 1,
 * edges = -inf, linspace(-1, 1, 998), +inf (ugly_utils.py:491-493).
 */
int cats_histogram(const void* values, size_t n, int dtype, const float* edges, int n_edges,
                   unsigned long long* counts, int take_abs, void* stream);

/*
 * *threshold (device memory) = edges[first b with cdf(b) > sparsity], cdf = running sum of
 * counts / total; edges[n_edges - 1] if the CDF never exceeds it.  Same arithmetic as
 * get_threshold (ugly_utils.py:236-245: float32 probabilities, torch.cumsum, searchsorted
 * side="right") for totals below 2^24, where float32 counts are still exact.
 */
int cats_histogram_threshold(const unsigned long long* counts, const float* edges, int n_edges,
                             float sparsity, float* threshold, void* stream);

/*
 * Dense down projection over Wd [H, I] (nn.Linear layout): out[b,h] = sum_i Wd[h,i] * inter[b,i].
 * Reads all of Wd whatever the sparsity; exists for callers that cannot supply WdT.
 * Replaces gemv_local_kernel (fuse_gemv_cmp_cuda.cu:1786-1960).
 */
int cats_down_dense(const void* inter, const void* Wd, int B, int H, int I, int dtype, void* out,
                    void* stream);

/*
 * The decoder-layer tail as a separate launch: resid[B,H] += y[B,H]; x_next = resid /
 * sqrt(mean(resid^2) + eps) (times norm_weight[H] if given; x_next may be NULL).  For callers
 * that must combine partial MLP outputs (tensor-parallel all-reduce) before the residual add;
 * single-GPU callers get the same arithmetic fused into cats_updown / cats_mlp.  Restates the
 * residual add + RMS norm around the MLP of the decoder layer
 * (experiments/models/sparse_silu/ugly_utils.py:1036-1057).
 */
int cats_tail(const void* y, void* resid, void* x_next, const void* norm_weight, float eps, int B,
              int H, int dtype, void* stream);

/*
 * Decode-step glue of a decoder layer, between the fused QKV projection and attention: rotate-half
 * rotary embedding of the query and key heads of one new position per sequence, and the write of
 * the rotated keys and the values into a static KV cache at *position (device memory, so the call
 * can sit in a CUDA graph whose position advances).  qkv [B, (n_heads + 2 n_kv_heads) head_dim]
 * (q, k, v heads in that order); cos / sin tables [max_len, head_dim]; q_out [B, n_heads,
 * head_dim]; caches [B, n_kv_heads, max_len, head_dim].  Rounds to the storage type after every
 * operation, like the elementwise launches it replaces.  Not on the MLP path: it exists so that
 * the decode loop around the MLP (cats_b200/decoder.py) is not dominated by small launches; the
 * reference leaves this to HF's modelling code.
 */
int cats_rope_cache(const void* qkv, const void* cos_table, const void* sin_table,
                    const long long* position, void* q_out, void* k_cache, void* v_cache, int B,
                    int n_heads, int n_kv_heads, int head_dim, int max_len, int dtype, void* stream);

/* Transpose a [rows, cols] matrix into [cols, rows] (packs Wd [H,I] into WdT [I,H]). */
int cats_transpose(const void* src, void* dst, int rows, int cols, int dtype, void* stream);

/*
 * Read back, after synchronising `stream`, the number of active neurons (union over the batch)
 * of the most recent stage-1/compact call on this workspace and the sticky device status word
 * (0 = no device-side check failed).  The only entry point that blocks the host.  Serves the
 * int return of fuse_gemv_cmp (fuse_gemv_cmp_cuda.cu:1962-1977).
 */
int cats_read_counters(const void* ws, int* n_active, int* device_status, void* stream);

/*
 * Copy the ordered active list of the most recent stage-1/compact call into caller buffers
 * (device memory): idx_out int64[>= n_active], val_out (dtype)[>= n_active] for token 0.
 * Serves fuse_gemv_cmp (flash_gemv/flash_gemv/flash_gemv.py:3-4), whose list is unordered in
 * the reference; here it is ascending.
 */
int cats_export_list(const void* ws, size_t ws_bytes, int B, int H, int I, int dtype,
                     int64_t* idx_out, void* val_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CATS_B200_H_ */
