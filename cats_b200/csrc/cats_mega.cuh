// Persistent CATS MLP kernel (sm_100a): every layer of a stack in ONE cooperative launch.
//
// Why.  A CATS layer moves ~235 MB (Mistral-7B shape, fp16, 50 % sparsity), about 35 us of HBM
// time on a B200.  Split into a stage-1 launch and a stage-2/3 launch, every launch pays its own
// ramp (first copies in flight), tail (slowest CTA, epilogue by one CTA) and hand-off; measured,
// that is ~20 us per layer of HBM idling.  Here one CTA per SM stays resident for the whole
// stack and keeps one stream of weight rows flowing through a shared-memory ring:
//
//   per layer:   G(0) G(1) G(2) U(0) D(0) U(1) D(1) U(2) D(2)    (G gate, U up, D down rows)
//
// The layer's neurons are split into three parts.  G(p) are the gate rows of this CTA's segment
// of part p; after them the CTA publishes the segment's active list and arrives at a grid
// barrier.  U(p)/D(p) are this CTA's balanced share of the active neurons of part p over ALL
// CTAs, known once that barrier has completed.  Between G(p) and U(p) the stream always carries
// two other phases' rows (about 10 us), which covers compaction + fence + barrier + scan (about
// 6-9 us, measured): the producers normally never wait for a list.  (With two halves they did.)  The residual add and RMS
// norm between layers are computed by every CTA for itself from the fp32 accumulators (no
// "last CTA" epilogue), and the next layer's gate rows are already streaming while that happens.
//
// Roles in a CTA (416 threads): warps 0-7 consumers; warps 8-11 producers (one elected thread
// each issues cp.async.bulk row copies, global -> this CTA's shared memory, plain single-CTA form; one
// thread manages a copy roughly every 240 ns, a quarter of what an SM's HBM share needs at 8 KB
// rows, hence four); warp 12 control (compacts and publishes the segment's active list, waits
// for the grid barriers, scans the segment counts, fills the CTA's work list).  The control work
// is split over two warps - a publisher (compaction, publication, barrier arrival) and a lister
// (barrier wait, scan, list fill, clearing of the accumulators) - because every global fence
// costs several microseconds while the copy ring keeps HBM saturated, and one warp doing both
// chains in sequence was too slow to have the lists ready in time.
//
// Waits.  CTAs wait for one another at grid barriers, so the launch is cooperative (all CTAs
// co-resident or the launch fails).  Every wait (mbarrier or grid barrier) is bounded (~1 s):
// on a time-out the CTA sets an abort flag in shared memory and the status word of the
// workspace, stops issuing copies, lets copies in flight land and leaves; the other CTAs then
// run into their own limits and leave as well.
#pragma once

#include <type_traits>

#include "cats_tma.cuh"

namespace cats {

constexpr int kMegaMaxLayers = 112;
constexpr int kMegaMaxGrid = 256;
constexpr int kMaxRanks = 8;                   // GPUs of one tensor-parallel group
constexpr int kMegaProducers = 4;  // issuing threads (one per warp); the host uses 2 when 4 does not divide S
constexpr int kMegaWarps = kConsumerWarps + kMegaProducers + 2;  // + publisher + lister
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kParts = 3;                      // a layer's neurons are processed in up to this many parts
constexpr int kSegHalfStride = kMaxSeg / 4;   // seg_count slots of part p start at p * this

enum { STATUS_WAIT_TIMEOUT_MEGA = 3 };
// Grid-barrier counters.  A counting barrier is only sound when no CTA can arrive for its next
// use before the current one has completed.  Publishing part h of layer l+1 needs x_{l+1}, which
// needs every CTA's down rows of layer l, which need every part's list of layer l: so one counter
// per part is safe, while one counter shared by the parts is not (a fast CTA's arrival for part
// h+1 would be counted towards part h while a slow CTA has not published yet).  The layer
// barrier (one arrival per CTA) has its own counter.  The *_BASE slots hold the
// counters' values at the start of the current launch.
enum { HDR_GBAR = 8 /* [kParts] */, HDR_OBAR = 12, HDR_GBAR_BASE = 13, HDR_OBAR_BASE = 14 };
static_assert(HDR_GBAR + kParts <= HDR_OBAR, "one list-barrier counter per part");

struct MegaParams {
  const void* wg[kMegaMaxLayers];
  const void* wu[kMegaMaxLayers];
  const void* wdt[kMegaMaxLayers];
  const void* nw[kMegaMaxLayers];  // optional RMS-norm weight applied to the layer's x_next
  float thr[kMegaMaxLayers];
};

struct MegaArgs {
  int L, B, H, I;
  int S, cw, cap, rmax;  // ring stages, dot-owner warps (divides S), list capacity, rows/segment
  int npw;               // producer threads in use (divides S)
  int bulk_flush;        // 1: accumulators leave through shared memory and TMA bulk reduces
  int mma_dot;           // 1: gate / up dot products of eight rows at a time on the tensor cores
  int wait_kc;           // limit of every wait, in units of 1024 clock cycles
  int parts;             // parts per layer (1..kParts): more parts hide the list latency behind
                         // other parts' rows, fewer parts mean fewer grid barriers per layer
  unsigned s_magic;      // floor(2^32 / S) + 1: item -> (ring cycle, slot) without a division
  int pf_rows;           // gate rows a stalled producer asks into L2 ahead of the ring (0: none)
  float eps;
  const void* x_in;  // [B,H] input of layer 0
  void* x_out;       // [B,H] normalised residual after the last layer (needs resid), or null
  void* resid;       // [B,H] residual stream in/out, or null (then L must be 1)
  void* out_last;    // [B,H] raw MLP output of the last layer, or null
  // Tensor parallelism over the intermediate dimension: nranks GPUs each run this kernel on
  // their own row slice and exchange the layers' partial sums through `xchg` (xchg[p] = rank
  // p's exchange buffer as mapped into this process; xchg[rank] is local).  nranks == 0: none.
  int nranks, rank;
  int xchg_all;  // 1: every CTA adds all ranks' slots itself; 0: per-slice totals (see the lister)
  int local;     // 1: every CTA works on its own segment's active neurons (no list barrier); needs
                 //    nranks >= 1 and one part per layer
  unsigned char* xchg[kMaxRanks];
};

// Exchange buffer of one rank (see MegaArgs::xchg).  Header: the running number of layers (its
// low bit selects the slot set, so consecutive layers alternate sets across launches too; plus
// one it is the tag of the layer's data).  Then slots[2][kMaxRanks][kMegaMaxB * H] of 8-byte
// (value, tag) pairs, slots[s][p] = rank p's partial sums as stored by rank p's CTAs over NVLink,
// and sums[2][kMegaMaxB * H] pairs, the ranks' total as written by this GPU's own CTAs.
// A pair is ONE 64-bit element of every store and load that touches it (st / ld ... .v2.b64:
// two pairs per instruction, each element single-copy atomic in the PTX memory model), so a
// reader that finds the tag it expects has the value that belongs to it: no fence and no flag
// orders data against anything, on either side; a pair that has not arrived is read again.
// Besides the tags there are arrival counters - HINTS that spare the readers from polling the
// data itself: one per source rank (a source's CTAs bump it over NVLink after their stores into
// this buffer) and one for the totals (bumped by this GPU's own CTAs); XCH_BASE is their common
// value at the start of the launch.  The bumps are relaxed and not ordered against the data:
// a reader that saw the counter still checks every tag, and a reader whose counter wait runs
// out falls back to polling the tags.
enum { XCH_LAYERS = 0, XCH_BASE = 1, XCH_ARRIVED = 8 /* [kMaxRanks] */, XCH_SUMS = 16,
       XCH_HDR_BYTES = 256 };
constexpr int kMegaMaxB = 4;
__host__ __device__ inline size_t xchg_bytes(int H) {
  return XCH_HDR_BYTES + sizeof(uint2) * 2 * (size_t)(kMaxRanks + 1) * kMegaMaxB * H;
}
__host__ __device__ inline uint2* xchg_slot(unsigned char* base, int set, int src, int H) {
  return reinterpret_cast<uint2*>(base + XCH_HDR_BYTES) +
         ((size_t)set * kMaxRanks + src) * kMegaMaxB * H;
}
__host__ __device__ inline uint2* xchg_sums(unsigned char* base, int set, int H) {
  return reinterpret_cast<uint2*>(base + XCH_HDR_BYTES) +
         ((size_t)2 * kMaxRanks + set) * kMegaMaxB * H;
}

// Rows [lo, hi) of half h out of I.
__host__ __device__ inline int half_row0(int h, int I, int parts) {
  return (int)(((long long)I * h) / parts);
}

// Two (value, tag) pairs = 16 bytes, each pair one 64-bit element.  System scope: the slots are
// written by other GPUs over NVLink (and read from this GPU's own memory); the sums are local
// but share the code.
__device__ __forceinline__ unsigned long long make_pair(float v, unsigned tag) {
  return (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
}
__device__ __forceinline__ void st_pairs(uint2* p, unsigned long long a, unsigned long long b) {
  asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void ld_pairs(const uint2* p, unsigned long long& a,
                                         unsigned long long& b) {
  asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ bool pair_has(unsigned long long a, unsigned tag) {
  return (unsigned)(a >> 32) == tag;
}
__device__ __forceinline__ float pair_val(unsigned long long a) {
  return __uint_as_float((unsigned)a);
}
__device__ __forceinline__ void bump_relaxed_sys(unsigned* ctr) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}
__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait (bounded, never aborting: it is only a hint) until the counter has reached `target`.
__device__ __forceinline__ void hint_wait(const unsigned* ctr, unsigned target, volatile int* abort) {
  if ((int)(ld_relaxed_sys(ctr) - target) >= 0) return;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if ((int)(ld_relaxed_sys(ctr) - target) >= 0) return;
      __nanosleep(40);
    }
    if (*abort || clock64() - t0 > wait_limit(abort)) return;
  }
}
// Four consecutive pairs (one group of four columns) with the tag `tag`, re-read until every one
// of them has arrived; bounded like every wait.  False when the limit ran out.
__device__ __forceinline__ bool ld_group_tagged(const uint2* p, unsigned tag, volatile int* abort,
                                                unsigned long long (&u)[4]) {
  ld_pairs(p, u[0], u[1]);
  ld_pairs(p + 2, u[2], u[3]);
  if (pair_has(u[0], tag) && pair_has(u[1], tag) && pair_has(u[2], tag) && pair_has(u[3], tag))
    return true;
  const long long t0 = clock64();
  for (;;) {
    __nanosleep(64);
    ld_pairs(p, u[0], u[1]);
    ld_pairs(p + 2, u[2], u[3]);
    if (pair_has(u[0], tag) && pair_has(u[1], tag) && pair_has(u[2], tag) && pair_has(u[3], tag))
      return true;
    if (*abort) return false;
    if (clock64() - t0 > 4 * wait_limit(abort)) {  // other ranks are launched by other processes
      *abort = 1;
      return false;
    }
  }
}

template <typename T, int BT, int NVT>
__global__ void __launch_bounds__(kMegaThreads, 1)
k_cats_mega(const __grid_constant__ MegaParams P, const MegaArgs A, WsPtrs ws) {
  using V = VecT<T>;
  constexpr int N = V::N;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ctl[2];  // abort flag, wait limit
  int& s_abort = s_ctl[0];
  __shared__ float s_red[32];
  __shared__ int s_cnt[kParts];
  __shared__ int s_trip;
  __shared__ int s_pref[kMegaMaxGrid];

  const int L = A.L, B = A.B, H = A.H, I = A.I, S = A.S, cw = A.cw, NP = A.parts;
  const uint32_t row_bytes = (uint32_t)H * sizeof(T);
  const int nvec = H / N;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const bool has_resid = A.resid != nullptr;
  const unsigned s_magic = A.s_magic;
  // ring cycle (k / S) and slot (k % S) of item k; exact for k < 2^32 / S
  auto cyc_of = [&](int kk) { return (int)__umulhi((unsigned)kk, s_magic); };
  auto slot_of = [&](int kk) { return kk - cyc_of(kk) * S; };

  // ---- shared memory carve-up -----------------------------------------------------------------
  // Ring stages and the tokens' x are 16 bytes further apart than a row is long: eight rows
  // (or tokens) read at the same column then fall into eight different bank groups, which is
  // what ldmatrix and the B-fragment loads of the tensor-core dot products need.
  const uint32_t row_stride = row_bytes + 16;
  const int xs_ld = H + 16 / (int)sizeof(T);
  unsigned char* ring = smem;
  size_t off = (size_t)S * row_stride;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + off);
  off += 8 * (size_t)(2 * S + 3 * kParts + 1);
  off = align_up(off, 16);
  T* xs = reinterpret_cast<T*>(smem + off);
  off += (size_t)B * row_stride;
  T* rs = reinterpret_cast<T*>(smem + off);
  off += has_resid ? (size_t)B * row_bytes : 0;
  float* s_val = reinterpret_cast<float*>(smem + off);  // [kParts][rmax * BT]
  off += kParts * sizeof(float) * (size_t)A.rmax * BT;
  int* s_idx = reinterpret_cast<int*>(smem + off);  // [kParts][cap]
  off += kParts * sizeof(int) * (size_t)A.cap;
  float* s_hg = reinterpret_cast<float*>(smem + off);  // [kParts][cap * BT]
  off += kParts * sizeof(float) * (size_t)A.cap * BT;
  off = align_up(off, 128);
  float* s_flush = reinterpret_cast<float*>(smem + off);  // [kConsumerWarps][32 * N] if bulk_flush
  off += A.bulk_flush ? sizeof(float) * kConsumerWarps * 32 * N : 0;
  float* s_part = reinterpret_cast<float*>(smem + off);   // [2][kConsumerWarps][8][BT] if mma_dot

  const uint32_t ring_u = smem_u32(ring), full_u = smem_u32(bars), empty_u = full_u + 8u * S;
  const uint32_t lready_u = empty_u + 8u * S, lfree_u = lready_u + 8u * kParts,
                 gdone_u = lfree_u + 8u * kParts, zdone_u = gdone_u + 8u * kParts;

  unsigned* gbar = reinterpret_cast<unsigned*>(ws.hdr + HDR_GBAR);
  unsigned* obar = reinterpret_cast<unsigned*>(ws.hdr + HDR_OBAR);
  const unsigned gbase = __ldcg(reinterpret_cast<const unsigned*>(ws.hdr + HDR_GBAR_BASE));
  const unsigned obase = __ldcg(reinterpret_cast<const unsigned*>(ws.hdr + HDR_OBAR_BASE));
  // list barrier of (l, h): counter h, G arrivals per layer; layer barrier idx = l, final = L
  // (G arrivals: one per CTA, after its consumer warps have met)
  auto gtarget = [&](int l) { return gbase + (unsigned)(l + 1) * (unsigned)G; };
  auto otarget = [&](int idx) {
    return obase + (unsigned)(idx + 1) * (unsigned)G;
  };

  // tensor-parallel exchange (K == 0: single GPU)
  const int K = A.nranks;
  unsigned* xflag = K ? reinterpret_cast<unsigned*>(A.xchg[A.rank]) : nullptr;
  const unsigned xl0 = K ? __ldcg(xflag + XCH_LAYERS) : 0u;
  const unsigned xbase = K ? __ldcg(xflag + XCH_BASE) : 0u;
  // this CTA's slice (groups of 4 columns) of a [B, H] vector
  const int ngrp_all = H >> 2;
  const int own_lo = (int)(((long long)ngrp_all * c) / G),
            own_hi = (int)(((long long)ngrp_all * (c + 1)) / G);

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, kConsumerWarps);
    }
    for (int h = 0; h < kParts; ++h) {
      mbar_init(lready_u + 8u * h, 1);
      mbar_init(lfree_u + 8u * h, kConsumerWarps);
      mbar_init(gdone_u + 8u * h, kConsumerWarps);
    }
    mbar_init(zdone_u, 1);
    s_abort = 0;
    s_ctl[1] = A.wait_kc;
    mbar_fence_init();
  }
  __syncthreads();  // the barriers exist; the producers go straight to their copies

  // this CTA's gate segment of half h
  auto seg_lo = [&](int h) {
    const int lo = half_row0(h, I, NP), hi = half_row0(h + 1, I, NP);
    return lo + seg_row0(c, G, hi - lo);
  };
  auto seg_hi = [&](int h) {
    const int lo = half_row0(h, I, NP), hi = half_row0(h + 1, I, NP);
    return lo + seg_row0(c + 1, G, hi - lo);
  };

  if (warp >= kConsumerWarps && warp < kConsumerWarps + kMegaProducers) {
    // =========================================================================== producers
    const int npw = A.npw;
    if (lane == 0 && warp - kConsumerWarps < npw) {
      const int p = warp - kConsumerWarps;
      bool ok = true;
      int k = 0;
      // L2 look-ahead during stalls.  While the consumers stand at a grid barrier (between two
      // layers above all) the ring is full and HBM idles.  The addresses of a CTA's gate rows
      // are known ahead of time (those of the active lists are not), so a producer whose wait
      // for a free stage lasts longer than the ring's ordinary back-pressure asks the next D
      // gate rows into L2 - its share: every npw-th row from the one it is waiting to copy -
      // and the ring refills from L2 once the barrier has passed.  Measured at the Mistral-7B
      // shape: 128 KB per CTA takes 2.6 % off a layer (for 3-4 % more DRAM reads: part of what
      // was asked for is fetched again); more is slower again, prefetching in the steady state,
      // with every copy, is slower than none, and so is asking for the next layer's first rows
      // while a producer waits for a list.
      const int D = A.pf_rows;
      const long long kStall = 4000;  // cycles, about 2 us (1000 .. 8000 measured alike)
      const int pr0 = seg_lo(0), pR0 = seg_hi(0) - pr0;
      const int pr1 = NP > 1 ? seg_lo(1) : 0, pR1 = NP > 1 ? seg_hi(1) - pr1 : 0;
      const int pr2 = NP > 2 ? seg_lo(2) : 0, pR2 = NP > 2 ? seg_hi(2) - pr2 : 0;
      auto prefetch_gate = [&](const T* W, int g) {  // gate row g of this CTA, if it exists
        int row;
        if (g < pR0) row = pr0 + g;
        else if ((g -= pR0) < pR1) row = pr1 + g;
        else if ((g -= pR1) < pR2) row = pr2 + g;
        else return;
        l2_prefetch(W + (size_t)row * H, row_bytes);
      };
      auto issue = [&](int kk, const T* src) {
        const int cy = cyc_of(kk), s = kk - cy * S;
        if (kk >= S && !mbar_wait(empty_u + 8u * s, (cy - 1) & 1, &s_abort)) {
          ok = false;
          return;
        }
        mbar_expect_tx(full_u + 8u * s, row_bytes);
        tma_load_1d(ring_u + s * row_stride, src, row_bytes, full_u + 8u * s);
      };
      auto issue_gate = [&](int kk, const T* W, int row, int g) {  // g: the row's number in the layer
        const int cy = cyc_of(kk), s = kk - cy * S;
        if (kk >= S &&
            !mbar_wait_or(empty_u + 8u * s, (cy - 1) & 1, &s_abort, kStall, [&]() {
              for (int d = 0; d < D; d += npw) prefetch_gate(W, g + d);
            })) {
          ok = false;
          return;
        }
        mbar_expect_tx(full_u + 8u * s, row_bytes);
        tma_load_1d(ring_u + s * row_stride, W + (size_t)row * H, row_bytes, full_u + 8u * s);
      };
      for (int l = 0; l < L && ok; ++l) {
        const T* Wg = reinterpret_cast<const T*>(P.wg[l]);
        const T* Wu = reinterpret_cast<const T*>(P.wu[l]);
        const T* Wd = reinterpret_cast<const T*>(P.wdt[l]);
        int g0 = 0;
        for (int h = 0; h < NP && ok; ++h) {
          const int r0 = seg_lo(h), R = seg_hi(h) - r0;
          // own items only: j == (p - k) mod npw, stepping by npw (no division per row)
          for (int j = ((p - k) % npw + npw) % npw; j < R && ok; j += npw) {
            if (D > 0) issue_gate(k + j, Wg, r0 + j, g0 + j);
            else issue(k + j, Wg + (size_t)(r0 + j) * H);
          }
          k += R;
          g0 += R;
        }
        for (int h = 0; h < NP && ok; ++h) {
          if (!mbar_wait(lready_u + 8u * h, l & 1, &s_abort)) {
            ok = false;
            break;
          }
          const int cnt = s_cnt[h];
          const int* idx = s_idx + h * A.cap;
          for (int j = ((p - k) % npw + npw) % npw; j < cnt && ok; j += npw)
            issue(k + j, Wu + (size_t)idx[j] * H);
          k += cnt;
          for (int j = ((p - k) % npw + npw) % npw; j < cnt && ok; j += npw) {
            issue(k + j, Wd + (size_t)idx[j] * H);
          }
          k += cnt;
        }
      }
    }
  } else if (warp == kConsumerWarps + kMegaProducers) {
    // =========================================================================== publisher
    // Warp-uniform control flow on purpose (every lane polls in the waits): with lane-0-only
    // waits and early exits the warp ran its shuffles diverged, ~40x slower.
    bool ok = true;
    for (int l = 0; l < L; ++l) {
      const float thr = P.thr[l];
      for (int h = 0; h < NP; ++h) {
        // this CTA's gate values of part h are in: ballot / popc compaction, publish, arrive
        if (ok) ok = mbar_wait(gdone_u + 8u * h, l & 1, &s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (ok && A.local) {
          // Local lists (tensor-parallel ranks with a few rows per CTA): this CTA's own active
          // neurons ARE its work list - straight into shared memory, no publication, no grid
          // barrier, no scan.  The up / down rows are then not balanced over the CTAs, which
          // costs less than the barrier chain it replaces when a CTA has a dozen rows.
          if (l >= 1) ok = mbar_wait(lfree_u + 8u * h, (l - 1) & 1, &s_abort);  // list h is free
          ok = __all_sync(0xffffffffu, ok);
          const int r0 = seg_lo(h), R = seg_hi(h) - r0;
          const float* sv = s_val + (size_t)h * A.rmax * BT;
          int base = 0;
          for (int g0 = 0; g0 < R && ok; g0 += 32) {
            const int lr = g0 + lane;
            float v[BT];
            bool any = false;
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              v[t] = 0.f;
              if (lr < R && t < B) {
                const float sval = sv[lr * BT + t];
                const bool a = is_active(sval, thr);
                v[t] = a ? sval : 0.f;
                any |= a;
              }
            }
            const unsigned m = __ballot_sync(0xffffffffu, any);
            if (any) {
              const int pos = base + __popc(m & ((1u << lane) - 1u));
              s_idx[h * A.cap + pos] = r0 + lr;
#pragma unroll
              for (int t = 0; t < BT; ++t) s_hg[(h * A.cap + pos) * BT + t] = v[t];
            }
            base += __popc(m);
          }
          if (lane == 0) {
            s_cnt[h] = ok ? base : 0;
            ws.seg_count[h * kSegHalfStride + c] = base;
          }
          // the lister's clearing of this CTA's accumulator slice (layer l-1's exchange) is
          // ordered ahead of everything this CTA publishes for layer l
          if (ok && l >= 1) ok = mbar_wait(zdone_u, (l - 1) & 1, &s_abort);
          ok = __all_sync(0xffffffffu, ok);
          __syncwarp();
          if (lane == 0 && ok) mbar_arrive(lready_u + 8u * h);
        } else if (ok) {
          const int r0 = seg_lo(h), R = seg_hi(h) - r0;
          const float* sv = s_val + (size_t)h * A.rmax * BT;
          int base = 0;
          for (int g0 = 0; g0 < R; g0 += 32) {
            const int lr = g0 + lane;
            float v[BT];
            bool any = false;
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              v[t] = 0.f;
              if (lr < R && t < B) {
                const float sval = sv[lr * BT + t];
                const bool a = is_active(sval, thr);
                v[t] = a ? sval : 0.f;
                any |= a;
              }
            }
            const unsigned m = __ballot_sync(0xffffffffu, any);
            if (any) {
              const int pos = r0 + base + __popc(m & ((1u << lane) - 1u));
              ws.seg_idx[pos] = r0 + lr;
#pragma unroll
              for (int t = 0; t < BT; ++t)
                if (t < B) ws.seg_gate[(size_t)pos * B + t] = v[t];
            }
            base += __popc(m);
          }
          if (lane == 0) ws.seg_count[h * kSegHalfStride + c] = base;
          // the lister's clearing of the accumulators that layer l will add into must be
          // complete (and fenced) before this CTA lets the barrier of (l, 0) complete
          if (h == 0 && l >= 2 && !K) ok = mbar_wait(zdone_u, (l - 2) & 1, &s_abort);
          ok = __all_sync(0xffffffffu, ok);
          __syncwarp();
          if (lane == 0 && ok) grid_arrive(gbar + h);
        }
      }
    }
  } else if (warp == kConsumerWarps + kMegaProducers + 1) {
    // =========================================================================== lister
    bool ok = true;
    for (int l = 0; l < L; ++l) {
      for (int h = 0; h < (A.local ? 0 : NP); ++h) {
        // all CTAs have published part h: scan the counts, take this CTA's balanced share
        if (ok) ok = grid_wait(gbar + h, gtarget(l), &s_abort);
        ok = __all_sync(0xffffffffu, ok);
        const int* cntp = ws.seg_count + h * kSegHalfStride;
        int cv[kMegaMaxGrid / 32];
#pragma unroll
        for (int q = 0; q < kMegaMaxGrid / 32; ++q) {  // all loads first: one L2 round trip
          const int i = q * 32 + lane;
          cv[q] = (ok && i < G) ? __ldcg(cntp + i) : 0;
        }
        if (ok && l >= 1) ok = mbar_wait(lfree_u + 8u * h, (l - 1) & 1, &s_abort);
        ok = __all_sync(0xffffffffu, ok);
        int run = 0;
#pragma unroll
        for (int q = 0; q < kMegaMaxGrid / 32; ++q) {
          const int i = q * 32 + lane;
          int v = cv[q];
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += y;
          }
          if (i < G) s_pref[i] = run + v;
          run += __shfl_sync(0xffffffffu, v, 31);
        }
        __syncwarp();
        const int n = run;
        const int p0 = (int)(((long long)c * n) / G), p1 = (int)(((long long)(c + 1) * n) / G);
        const int cnt = ok ? p1 - p0 : 0;
        const int hlo = half_row0(h, I, NP), hrows = half_row0(h + 1, I, NP) - hlo;
        for (int j = lane; j < cnt; j += 32) {
          const int pos = p0 + j;
          int lo = 0, hi = G - 1;  // smallest segment with s_pref > pos
          while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (s_pref[mid] > pos) hi = mid; else lo = mid + 1;
          }
          const int excl = lo ? s_pref[lo - 1] : 0;
          const int q = hlo + seg_row0(lo, G, hrows) + (pos - excl);
          s_idx[h * A.cap + j] = __ldcg(ws.seg_idx + q);
#pragma unroll
          for (int t = 0; t < BT; ++t)
            s_hg[(h * A.cap + j) * BT + t] =
                (t < B) ? __ldcg(ws.seg_gate + (size_t)q * B + t) : 0.f;
        }
        if (lane == 0) {
          s_cnt[h] = cnt;
          if (c == 0) {
            if (h == 0) ws.hdr[HDR_NACTIVE] = n; else ws.hdr[HDR_NACTIVE] += n;
          }
        }
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(lready_u + 8u * h);
      }
      if (K) {
        // Tensor parallel: once every CTA of this GPU has added its share of layer l, send this
        // CTA's slice of the sums to every rank's slot for this rank (plain stores of (value,
        // tag) pairs into peer memory) and clear the slice for layer l+2 (nobody else reads the
        // accumulators in this mode; the clearing reaches the other CTAs through the list and
        // layer barriers of layer l+1).  Then (unless every CTA reads all ranks' slots itself,
        // A.xchg_all) add the ranks' partial sums of the same slice as they arrive in this GPU's
        // slots - in rank order, so every rank computes bit-identical totals - and publish the
        // total, tagged again, for all CTAs of this GPU: a CTA then reads B * H totals per layer
        // instead of nranks * B * H partial sums, at the price of one more hand-off through L2.
        if (ok) ok = grid_wait(obar, otarget(l), &s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          float* accp = ws.acc32 + (size_t)(l & 1) * kMaxB * H;
          const int set = (int)((xl0 + (unsigned)l) & 1u);
          const unsigned tag = xl0 + (unsigned)l + 1u;
          const int own_n = own_hi - own_lo;
          for (int e = lane; e < B * own_n; e += 32) {
            const int b = e / own_n, g = own_lo + (e - b * own_n);
            float4* src = reinterpret_cast<float4*>(accp + (size_t)b * H) + g;
            const float4 v = __ldcg(src);
            *src = make_float4(0.f, 0.f, 0.f, 0.f);
            const unsigned long long q0 = make_pair(v.x, tag), q1 = make_pair(v.y, tag),
                                     q2 = make_pair(v.z, tag), q3 = make_pair(v.w, tag);
            for (int p = 0; p < K; ++p) {
              uint2* dst = xchg_slot(A.xchg[p], set, A.rank, H) + (size_t)b * H + 4 * (size_t)g;
              st_pairs(dst, q0, q1);
              st_pairs(dst + 2, q2, q3);
            }
          }
          __syncwarp();
          if (lane < K) bump_relaxed_sys(reinterpret_cast<unsigned*>(A.xchg[lane]) + XCH_ARRIVED + A.rank);
          bool good = true;
          for (int e = lane; e < B * own_n && !A.xchg_all; e += 32) {
            const int b = e / own_n, g = own_lo + (e - b * own_n);
            const uint2* src0 = xchg_slot(A.xchg[A.rank], set, 0, H) + (size_t)b * H + 4 * (size_t)g;
            const size_t sstride = (size_t)kMegaMaxB * H;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p0 = 0; p0 < K && good; p0 += 4) {  // four sources' loads in flight at a time
              unsigned long long u[4][4];
#pragma unroll
              for (int pp = 0; pp < 4; ++pp)
                if (p0 + pp < K) {
                  ld_pairs(src0 + (p0 + pp) * sstride, u[pp][0], u[pp][1]);
                  ld_pairs(src0 + (p0 + pp) * sstride + 2, u[pp][2], u[pp][3]);
                }
#pragma unroll
              for (int pp = 0; pp < 4; ++pp)
                if (p0 + pp < K && good) {
                  if (!(pair_has(u[pp][0], tag) && pair_has(u[pp][1], tag) &&
                        pair_has(u[pp][2], tag) && pair_has(u[pp][3], tag)))
                    good = ld_group_tagged(src0 + (p0 + pp) * sstride, tag, &s_abort, u[pp]);
                  a.x += pair_val(u[pp][0]); a.y += pair_val(u[pp][1]);
                  a.z += pair_val(u[pp][2]); a.w += pair_val(u[pp][3]);
                }
            }
            if (good) {
              uint2* dst = xchg_sums(A.xchg[A.rank], set, H) + (size_t)b * H + 4 * (size_t)g;
              st_pairs(dst, make_pair(a.x, tag), make_pair(a.y, tag));
              st_pairs(dst + 2, make_pair(a.z, tag), make_pair(a.w, tag));
            }
          }
          ok = __all_sync(0xffffffffu, good);
          if (lane == 0 && ok) bump_relaxed_sys(xflag + XCH_SUMS);   // (in both modes: one base)
          __threadfence();  // the cleared slice, ahead of this warp's next barrier hand-offs
        }
        __syncwarp();
        if (A.local && lane == 0 && ok) mbar_arrive(zdone_u);   // (the publisher waits for it)
      } else if (l >= 1) {
        // Every CTA has read layer l-1's accumulators (it needed x_l for gate rows that are
        // published by now): clear this CTA's slice so that layer l+1 can add into them.
        if (ok) {
          float* accp = ws.acc32 + (size_t)((l - 1) & 1) * kMaxB * H;
          const int tot = B * H, lo = (int)(((long long)tot * c) / G),
                    hi = (int)(((long long)tot * (c + 1)) / G);
          for (int e = lo + lane; e < hi; e += 32) accp[e] = 0.f;
          __threadfence();
        }
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(zdone_u);
      }
    }
  } else {
    // =========================================================================== consumers
    // Control-flow rule: every consumer thread executes exactly the same sequence of
    // consumer_bar_sync() calls whatever happens; `ok` only switches waits and work off.
    bool ok = true;
    int k = 0;
    float acc[NVT][BT][N];

    // Only the consumers read x and the residual: they stage them while the first gate rows are
    // already on their way.
    {
      const int nv = H / N;
      for (int b = 0; b < B; ++b) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(A.x_in) + (size_t)b * H);
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)b * xs_ld);
        for (int i = tid; i < nv; i += kConsumerThreads) dst[i] = __ldcg(src + i);
      }
      if (has_resid) {
        const uint4* src = reinterpret_cast<const uint4*>(A.resid);
        uint4* dst = reinterpret_cast<uint4*>(rs);
        for (int i = tid; i < B * nv; i += kConsumerThreads) dst[i] = __ldcg(src + i);
      }
      consumer_bar_sync();
    }

    // x_{l+1} (and, after the last layer, the outputs) from layer l's accumulators.  Every CTA
    // computes the whole vector for itself; global outputs are written in disjoint slices.
    auto next_x = [&](int l, bool last) {
      // single GPU: all CTAs' sums are in the accumulators once the layer barrier completes;
      // tensor parallel: the ranks' totals arrive slice by slice as tagged pairs (see the lister)
      if (!K) {
        if (tid == 0 && ok) grid_wait(obar, otarget(l), &s_abort);
      } else if (ok) {
        // hints: every source rank's CTAs (or this GPU's own, for the totals) have bumped their
        // counter - the data is most probably there, the tags below decide
        const unsigned target = xbase + (unsigned)(l + 1) * (unsigned)G;
        if (A.xchg_all) {
          if (tid < K) hint_wait(xflag + XCH_ARRIVED + tid, target, &s_abort);
        } else if (tid == 0) {
          hint_wait(xflag + XCH_SUMS, target, &s_abort);
        }
      }
      consumer_bar_sync();
      ok = !s_abort;
      const float* accp = ws.acc32 + (size_t)(l & 1) * kMaxB * H;
      // tensor parallel: nsrc arrays of tagged pairs to add in order - the ranks' slots
      // (A.xchg_all) or the one array of totals that the listers publish
      const int nsrc = K ? (A.xchg_all ? K : 1) : 0;
      const uint2* srcs = !K ? nullptr
                          : A.xchg_all ? xchg_slot(A.xchg[A.rank], (int)((xl0 + (unsigned)l) & 1u), 0, H)
                                       : xchg_sums(A.xchg[A.rank], (int)((xl0 + (unsigned)l) & 1u), H);
      const size_t sstride = (size_t)kMegaMaxB * H;
      const unsigned tag = xl0 + (unsigned)l + 1u;
      const int ngrp = ngrp_all;
      const T* nw = reinterpret_cast<const T*>(P.nw[l]);
      constexpr int KV = 4;
      for (int b = 0; b < B; ++b) {
        float ss = 0.f;
        for (int g0 = 0; g0 < ngrp && ok; g0 += KV * kConsumerThreads) {
          float4 a[KV];
          if (!K) {
#pragma unroll
            for (int q = 0; q < KV; ++q) {
              const int g = g0 + q * kConsumerThreads + tid;
              a[q] = (g < ngrp) ? __ldcg(reinterpret_cast<const float4*>(accp + (size_t)b * H) + g)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          } else {
#pragma unroll
            for (int q = 0; q < KV; ++q) a[q] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int p = 0; p < nsrc; ++p) {
              // all loads first (one L2 round trip when everything has arrived), then the checks;
              // a group whose pairs are not all there yet is read again on its own
              const uint2* sp = srcs + p * sstride + (size_t)b * H;
              unsigned long long u[KV][4];
#pragma unroll
              for (int q = 0; q < KV; ++q) {
                const int g = g0 + q * kConsumerThreads + tid;
                if (g < ngrp) {
                  ld_pairs(sp + 4 * (size_t)g, u[q][0], u[q][1]);
                  ld_pairs(sp + 4 * (size_t)g + 2, u[q][2], u[q][3]);
                }
              }
#pragma unroll
              for (int q = 0; q < KV; ++q) {
                const int g = g0 + q * kConsumerThreads + tid;
                if (g < ngrp) {
                  bool good = pair_has(u[q][0], tag) && pair_has(u[q][1], tag) &&
                              pair_has(u[q][2], tag) && pair_has(u[q][3], tag);
                  if (!good && ok) good = ld_group_tagged(sp + 4 * (size_t)g, tag, &s_abort, u[q]);
                  if (!good) ok = false;
                  a[q].x += pair_val(u[q][0]); a[q].y += pair_val(u[q][1]);
                  a[q].z += pair_val(u[q][2]); a[q].w += pair_val(u[q][3]);
                }
              }
            }
          }
#pragma unroll
          for (int q = 0; q < KV; ++q) {
            const int g = g0 + q * kConsumerThreads + tid;
            if (g < ngrp) {
              const float y[4] = {a[q].x, a[q].y, a[q].z, a[q].w};
              const bool mine = last && g >= own_lo && g < own_hi;
              const size_t e = (size_t)b * H + 4 * (size_t)g;
              if (mine && A.out_last) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  reinterpret_cast<T*>(A.out_last)[e + i] = V::from_f(y[i]);
              }
              if (has_resid) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const T rn = V::from_f(V::to_f(rs[e + i]) + y[i]);
                  rs[e + i] = rn;
                  const float rf = V::to_f(rn);
                  ss = fmaf(rf, rf, ss);
                  if (mine) reinterpret_cast<T*>(A.resid)[e + i] = rn;
                }
              }
            }
          }
        }
        if (has_resid) {
          ss = warp_sum(ss);
          consumer_bar_sync();
          if (lane == 0) s_red[warp] = ss;
          consumer_bar_sync();
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; ++w) tot += s_red[w];
          const float rsq = rsqrtf(tot / (float)H + A.eps);
          for (int g = tid; g < ngrp && ok; g += kConsumerThreads) {
            const bool mine = last && g >= own_lo && g < own_hi;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const size_t e = (size_t)b * H + 4 * (size_t)g + i;
              T y = V::from_f(V::to_f(rs[e]) * rsq);
              if (nw) y = V::from_f(V::to_f(nw[4 * g + i]) * V::to_f(y));
              xs[(size_t)b * xs_ld + 4 * g + i] = y;
              if (mine && A.x_out) reinterpret_cast<T*>(A.x_out)[e] = y;
            }
          }
        }
      }
      consumer_bar_sync();
    };

    // Tensor-core dot products (16-bit weights): all consumer warps work on the same group of up
    // to eight ring rows, warp w on columns [w * H/8, (w+1) * H/8).  Lane q waits for the q-th
    // row; per 16 columns one ldmatrix fetches the rows' fragments, two 32-bit loads the tokens'
    // (lanes whose token does not exist keep zeros), one mma adds 8 x 8 partial dots; two
    // independent accumulator sets hide the mma latency.  Then lane q releases the q-th stage
    // and the warp leaves its partial sums in `part` ([warp][row][token]) for the caller to add
    // up after a consumer barrier.  Returns false (warp-uniform) when a wait gave up.
    const bool mma_dot = A.mma_dot != 0;
    int dot_groups = 0;  // selects the half of s_part in use
    auto dot8 = [&](int k0, int nb, float* part) -> bool {
      bool mine = true;
      if (lane < nb) {
        const int kk = k0 + lane, cy = cyc_of(kk);
        mine = mbar_wait(full_u + 8u * (kk - cy * S), cy & 1, &s_abort);
      }
      if (!__all_sync(0xffffffffu, mine)) return false;
      const int q = lane & 7;
      const uint32_t rbase = ring_u + (uint32_t)slot_of(k0 + (q < nb ? q : 0)) * row_stride +
                             ((lane >> 3) & 1) * 16u;
      const int g = lane >> 2, tq = lane & 3;
      const T* xp = xs + (size_t)(g < B ? g : 0) * xs_ld + tq * 2;
      const bool tok = g < B;
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
      const int kw = H / kConsumerWarps;
      for (int kc = warp * kw; kc < (warp + 1) * kw; kc += 32) {
        uint32_t a0, a2, a0b, a2b;
        ldmatrix_x2(rbase + (uint32_t)kc * (uint32_t)sizeof(T), a0, a2);
        ldmatrix_x2(rbase + (uint32_t)(kc + 16) * (uint32_t)sizeof(T), a0b, a2b);
        uint32_t b0 = 0u, b1 = 0u, b0b = 0u, b1b = 0u;
        if (tok) {
          b0 = *reinterpret_cast<const uint32_t*>(xp + kc);
          b1 = *reinterpret_cast<const uint32_t*>(xp + kc + 8);
          b0b = *reinterpret_cast<const uint32_t*>(xp + kc + 16);
          b1b = *reinterpret_cast<const uint32_t*>(xp + kc + 24);
        }
        Mma8<T>::run(d0, a0, a2, b0, b1);
        Mma8<T>::run(d1, a0b, a2b, b0b, b1b);
      }
      __syncwarp();
      if (lane < nb) mbar_arrive(empty_u + 8u * slot_of(k0 + lane));
      // this lane holds row g, tokens 2 * tq and 2 * tq + 1
      if (2 * tq < BT) part[(warp * 8 + g) * BT + 2 * tq] = d0[0] + d1[0];
      if (2 * tq + 1 < BT) part[(warp * 8 + g) * BT + 2 * tq + 1] = d0[1] + d1[1];
      return true;
    };
    // sum of the eight warps' partial dots of (row, token) = (i / BT, i % BT), for i < 8 * BT
    auto dot8_sum = [&](const float* part, int i) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) t += part[w * 8 * BT + i];
      return t;
    };

    for (int l = 0; l < L; ++l) {
      if (l > 0) next_x(l - 1, false);
#pragma unroll
      for (int g = 0; g < NVT; ++g)
#pragma unroll
        for (int t = 0; t < BT; ++t)
#pragma unroll
          for (int i = 0; i < N; ++i) acc[g][t][i] = 0.f;

      // ---- gate rows of the two halves ---------------------------------------------------------
      for (int h = 0; h < NP; ++h) {
        const int r0 = seg_lo(h), R = seg_hi(h) - r0;
        float* sv = s_val + (size_t)h * A.rmax * BT;
        if (mma_dot) {
          // (every warp runs every iteration and every barrier, whatever `ok` is)
          for (int j0 = 0; j0 < R; j0 += 8) {
            const int nb = min(8, R - j0);
            float* part = s_part + (dot_groups++ & 1) * (kConsumerWarps * 8 * BT);
            if (ok) ok = dot8(k + j0, nb, part);
            consumer_bar_sync();
            if (tid < nb * BT && ok) {
              const float a0 = dot8_sum(part, tid);
              if (tid % BT < B) sv[j0 * BT + tid] = silu_f(a0);
            }
          }
        } else if (warp < cw) {
          int j = ((warp - k) % cw + cw) % cw;  // first j with (k + j) % cw == warp
          for (; j < R && ok; j += cw) {
            const int kk = k + j, cy = cyc_of(kk), s = kk - cy * S;
            if (!(ok = mbar_wait_warp(full_u + 8u * s, cy & 1, &s_abort))) break;
            float a1[BT];
            warp_dot1_smem<T, BT>(reinterpret_cast<const T*>(ring + (size_t)s * row_stride), xs, B,
                                  H, lane, a1, xs_ld);
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              const float a0 = warp_sum(a1[t]);
              if (lane == 0) sv[j * BT + t] = silu_f(a0);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_n(empty_u + 8u * s, kConsumerWarps);
          }
        }
        k += R;
        __syncwarp();
        if (lane == 0) mbar_arrive(gdone_u + 8u * h);
      }

      // ---- up and down rows of the two halves ----------------------------------------------------
      for (int h = 0; h < NP; ++h) {
        if (ok) ok = mbar_wait_warp(lready_u + 8u * h, l & 1, &s_abort);
        int cnt;
        if (mma_dot) {
          // The group loop below runs a consumer barrier per group, so every warp needs the same
          // trip count whatever happens: ONE thread decides it (a warp whose wait gave up and a
          // warp whose wait succeeded would otherwise disagree, and a consumer barrier that some
          // warps never reach is a dead CTA); `ok` only switches the work off.
          if (tid == 0) s_trip = (ok && !s_abort) ? s_cnt[h] : 0;
          consumer_bar_sync();
          cnt = s_trip;
          ok = ok && !s_abort;
        } else {
          cnt = ok ? s_cnt[h] : 0;
        }
        float* hg = s_hg + (size_t)h * A.cap * BT;
        if (mma_dot) {
          for (int j0 = 0; j0 < cnt; j0 += 8) {
            const int nb = min(8, cnt - j0);
            float* part = s_part + (dot_groups++ & 1) * (kConsumerWarps * 8 * BT);
            if (ok) ok = dot8(k + j0, nb, part);
            consumer_bar_sync();
            if (tid < nb * BT && ok) hg[j0 * BT + tid] *= dot8_sum(part, tid);
          }
        } else if (warp < cw) {
          int j = ((warp - k) % cw + cw) % cw;
          for (; j < cnt && ok; j += cw) {
            const int kk = k + j, cy = cyc_of(kk), s = kk - cy * S;
            if (!(ok = mbar_wait_warp(full_u + 8u * s, cy & 1, &s_abort))) break;
            float a1[BT];
            warp_dot1_smem<T, BT>(reinterpret_cast<const T*>(ring + (size_t)s * row_stride), xs, B,
                                  H, lane, a1, xs_ld);
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              const float a0 = warp_sum(a1[t]);
              if (lane == 0) hg[j * BT + t] *= a0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_n(empty_u + 8u * s, kConsumerWarps);
          }
        }
        k += cnt;
        consumer_bar_sync();  // every h_j of this half is final; all earlier items are consumed
        ok = !s_abort;
        // Down rows in groups of kDG: lane q waits for the q-th row of the group (one round trip
        // to the barrier unit for the whole group instead of one per row), the warp adds the
        // group's rows, then lane q releases the q-th stage.
        constexpr int kDG = 8;
        const int dg = min(kDG, S);  // a group must fit in the ring
        for (int j0 = 0; j0 < cnt && ok; j0 += dg) {
          const int nb = min(dg, cnt - j0);
          bool mine = true;
          if (lane < nb) {
            const int kk = k + j0 + lane;
            const int cy = cyc_of(kk);
            mine = mbar_wait(full_u + 8u * (kk - cy * S), cy & 1, &s_abort);
          }
          ok = __all_sync(0xffffffffu, mine);
          if (!ok) break;
          // all loads of a column group first (kDG independent 16-byte loads in flight per
          // thread), then the FMAs: with two warps per scheduler nothing else hides the latency
          // batches: the scalar rounded to the storage type, one FMA per weight (prep1 / axpy1)
          constexpr bool kOneFma = BT >= 2 && sizeof(T) == 2;
          typedef typename std::conditional<kOneFma, uint32_t, typename V::Scalar>::type HScalar;
          HScalar hb[kDG][BT];
          const uint4* rowp[kDG];
#pragma unroll
          for (int q = 0; q < kDG; ++q) {
            const int qq = q < nb ? q : 0;
            rowp[q] = reinterpret_cast<const uint4*>(ring + (size_t)slot_of(k + j0 + qq) * row_stride);
#pragma unroll
            for (int t = 0; t < BT; ++t)
              if constexpr (kOneFma) hb[q][t] = V::prep1(q < nb ? hg[(j0 + q) * BT + t] : 0.f);
              else hb[q][t] = V::prep(q < nb ? hg[(j0 + q) * BT + t] : 0.f);
          }
#pragma unroll
          for (int g = 0; g < NVT; ++g) {
            const int v = g * kConsumerThreads + tid;
            if (v < nvec) {
              uint4 wq[kDG];
#pragma unroll
              for (int q = 0; q < kDG; ++q) wq[q] = rowp[q][v];
#pragma unroll
              for (int q = 0; q < kDG; ++q)
#pragma unroll
                for (int t = 0; t < BT; ++t) {
                  if constexpr (kOneFma) V::axpy1(hb[q][t], wq[q], acc[g][t]);
                  else V::axpy(hb[q][t], wq[q], acc[g][t]);
                }
            }
          }
          __syncwarp();
          if (lane < nb) {
            const int kk = k + j0 + lane;
            mbar_arrive(empty_u + 8u * slot_of(kk));
          }
        }
        k += cnt;
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(lfree_u + 8u * h);
      }

      // ---- this CTA's share of the down projection into the layer's fp32 accumulators ----------
      if (ok && A.bulk_flush) {
        // Through shared memory: a warp's 32 vectors of one (g, t) are 32 * N contiguous
        // columns, written to the warp's staging area and added to the accumulators by one
        // bulk reduce.  The staging area is reused once the previous reduce has read it.
        float* accp = ws.acc32 + (size_t)(l & 1) * kMaxB * H;
        float* stg = s_flush + (size_t)warp * 32 * N;
        const uint32_t stg_u = smem_u32(stg);
        bool first = true;
#pragma unroll
        for (int g = 0; g < NVT; ++g) {
          const int v0 = g * kConsumerThreads + warp * 32;  // the warp's first vector
          if (v0 < nvec) {                                   // nvec is a multiple of 32
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              if (t < B) {
                if (!first) {
                  if (lane == 0) bulk_wait_read();
                  __syncwarp();
                }
                first = false;
#pragma unroll
                for (int i = 0; i < N; i += 4)
                  *reinterpret_cast<float4*>(stg + lane * N + i) =
                      make_float4(acc[g][t][i], acc[g][t][i + 1], acc[g][t][i + 2], acc[g][t][i + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  bulk_reduce_add_f32(accp + (size_t)t * H + (size_t)v0 * N, stg_u,
                                      32u * N * (uint32_t)sizeof(float));
                  bulk_commit();
                }
              }
            }
          }
        }
        if (lane == 0) bulk_wait_all();
      } else if (ok) {
        float* accp = ws.acc32 + (size_t)(l & 1) * kMaxB * H;
#pragma unroll
        for (int g = 0; g < NVT; ++g) {
          const int v = g * kConsumerThreads + tid;
          if (v < nvec) {
#pragma unroll
            for (int t = 0; t < BT; ++t) {
              if (t < B) {
                float* dst = accp + (size_t)t * H + (size_t)v * N;
#pragma unroll
                for (int i = 0; i < N; i += 4)
                  red_add_v4(dst + i, acc[g][t][i], acc[g][t][i + 1], acc[g][t][i + 2],
                             acc[g][t][i + 3]);
              }
            }
          }
        }
      }
      // ONE arrival per CTA (the warps meet first): 148 adds to the barrier word per layer
      // instead of one per consumer warp - adds to one address serialise in L2, and the last
      // of them is on the layer's critical path (measured: 41.1 against 41.4 us per layer)
      consumer_bar_sync();
      if (tid == 0 && !s_abort) grid_arrive(obar);
    }

    next_x(L - 1, true);
    // everyone has read the last layer's accumulators once the final barrier completes
    consumer_bar_sync();
    if (tid == 0 && !s_abort) {
      grid_arrive(obar);
      grid_wait(obar, otarget(L), &s_abort);
    }
    consumer_bar_sync();
    if (!s_abort) {
      if (!K) {
        float* accp = ws.acc32 + (size_t)((L - 1) & 1) * kMaxB * H;
        const int tot = B * H, lo = (int)(((long long)tot * c) / G),
                  hi = (int)(((long long)tot * (c + 1)) / G);
        for (int e = lo + tid; e < hi; e += kConsumerThreads) accp[e] = 0.f;
      }
      if (c == 0 && tid == 0) {
        if (K) {
          xflag[XCH_LAYERS] = xl0 + (unsigned)L;
          xflag[XCH_BASE] = xbase + (unsigned)L * (unsigned)G;
        }
        // (with local lists nobody arrived at the list barriers: their counters did not move)
        ws.hdr[HDR_GBAR_BASE] = (int)(gbase + (A.local ? 0u : (unsigned)L * (unsigned)G));
        ws.hdr[HDR_OBAR_BASE] = (int)(obase + (unsigned)(L + 1) * (unsigned)G);
        // segment counts are per part (not a flat list); with local lists they are this layer's
        // per-CTA counts and add up to the number of active neurons
        ws.hdr[HDR_NSEG] = A.local ? G : -1;
      }
    }
  }

  __syncthreads();
  if (s_abort) {
    if (tid == 0) atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_MEGA);
    drain_after_abort();
  }
}

}  // namespace cats
