// Dense batched CATS MLP on the 5th-generation tensor cores (sm_100a): tcgen05.mma fed by TMA,
// accumulators in tensor memory.
//
// When the batch is larger than a few tokens, the union of the tokens' active sets is (nearly)
// every neuron: nothing is left to skip, and the MLP is three skinny GEMMs - 128 weight rows by
// up to 16 tokens per tile - that have to stream all of Wg, Wu and Wd once at HBM speed.  The
// per-token masks still decide the arithmetic, exactly as in the reference's batched kernels
// (flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:1542-1548: a token whose own gate value is dead
// contributes zero), they just no longer decide which rows are loaded.  Like the reference's
// batched path, the down projection reads Wd in its nn.Linear layout [H, I]
// (fuse_gemv_cmp_cuda.cu:1786-1960, gemv_local_kernel): with every row needed, the
// intermediate-major copy has no advantage, and [H, I] makes all three GEMMs the same shape of
// problem - D[128 rows, tokens] += A[128 rows, K] * X[tokens, K]^T with both operands K-major.
//
// One cooperative kernel, k_dense, runs a layer or a whole stack of layers (see its comment).
// All waits are bounded (cats_tma.cuh); a CTA that gives up frees its tensor memory first.
// No cluster launch, no multicast: every TMA load is the plain single-CTA form.
#pragma once

#include <cuda.h>

#include "cats_tma.cuh"

namespace cats {

constexpr int kDenseN = 16;          // tokens per MMA (the batch is zero-padded to it by TMA)
constexpr int kDenseKB = 64;         // elements of K per stage: one 128-byte swizzle row
constexpr int kDenseThreads = 192;   // warp 0 producer, warp 1 MMA issuer, warps 2-5 epilogue
constexpr uint32_t kDenseATile = 128 * 128;              // bytes of a 128-row A block in a stage
constexpr uint32_t kDenseXTile = kDenseN * 128;          // bytes of the token block in a stage
enum { STATUS_WAIT_TIMEOUT_DENSE = 4 };

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// orders what this thread observed through ordinary loads / waits with its later TMA reads
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; 16-bit inputs, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes (64 16-bit
// elements) under the 128-byte swizzle: groups of eight rows 1024 bytes apart (stride byte
// offset), descriptor version 1, layout type 2 = SWIZZLE_128B; the tile starts on a 1024-byte
// boundary.  Advancing K by 16 elements adds 32 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: fp32 accumulator, A and B of the given 16-bit format (0 fp16, 1 bf16),
// both K-major, N = 16, M = 128.
__host__ __device__ inline uint32_t umma_idesc(int fmt) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(kDenseN >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
// barrier among the four epilogue warps only (128 threads, named barrier 1)
__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__half> { static constexpr int v = 0; };
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr int v = 1; };

// ---------------------------------------------------------------------------------------------
// k_dense: L dense CATS layers in ONE cooperative launch, one CTA per SM (the batched twin of
// k_cats_mega).  Roles: warp 0 producer (one thread issues the TMA loads), warp 1 MMA issuer
// (one thread), warps 2-5 epilogue (tcgen05.ld, activation, reductions, the tail).
//
// Per layer a CTA streams two phases through one ring of 36 KB stages (128-byte swizzle):
//   phase 1  stage = [Wg block][Wu block][x block]: the CTA owns ~I/148 consecutive neurons (one
//            row tile of at most 128, two at the 70B shape); per 64-column step of H, 2 x 4
//            tcgen05.mma (M 128, N 16, K 16) add into a gate and an up accumulator in TMEM;
//            epilogue: h = mask(SiLU(g)) * u per token, rounded to the storage type, written
//            token-major [16, I].
//   phase 2  stage = [Wd block][Wd block][h block][h block]: split-K - the (128-row tile of H) x
//            (64-column step of I) blocks of Wd [H, I] are dealt out evenly over the CTAs in
//            order; partial sums leave TMEM through fp32 reductions into the workspace.
//   tail     token b is finished by CTA b alone: out / the new residual, the token's sum of
//            squares (a sum inside one CTA: no grid barrier for it), x_next = rmsnorm(resid)
//            (times the norm weight, if given), and the token's accumulator row cleared.
// Three grid barriers order a layer (one monotonic counter in the workspace header, ONE arrival
// per CTA and barrier - the epilogue warps meet first; its value at launch in the next slot):
//   1 every CTA's h is written        2 every CTA's partial sums are added
//   3 every token's x_next is written (and its accumulators are clear again)
// A stage's weight blocks never depend on a barrier, its activation block (x or h) does.  The
// producer issues weight blocks as far ahead as the ring allows and keeps the stages whose
// activation block is still owed in a FIFO: the block goes out as soon as its barrier has
// completed (polled between stages) and at the latest when the ring wraps onto that stage.  So
// the ring stays full across the h hand-off and across layers; only 2 KB per stage wait.
// x alternates between two buffers from layer to layer; the last layer writes where the caller
// asked (x_io for a stack).
// The producer's and the issuer's bookkeeping is incremental on purpose: each is ONE thread that
// has to handle a stage every ~0.7 us, and an integer division by a run-time value costs a tenth
// of that (measured: 3.4 TB/s with a dozen divisions per stage, 6 TB/s without).
// STACK: the layers' tensor maps and thresholds come from a table in global memory (written by
// k_dense_table just before); else (one layer) from the kernel parameters.
// ---------------------------------------------------------------------------------------------
enum { HDR_DBAR = 16, HDR_DBAR_BASE = 17 };
constexpr uint32_t kDenseStage = 2 * kDenseATile + 4096;   // 36 KB, both phases
constexpr int kDenseMaxLayers = 80;   // 80 x three 128-byte maps + thresholds in one 32 KB launch
struct DenseLayerMaps {
  CUtensorMap wg, wu, wd;
};
struct DenseStackParams {
  DenseLayerMaps m[kDenseMaxLayers];
  float thr[kDenseMaxLayers];
};
static_assert(sizeof(DenseStackParams) <= kWsTableBytes, "the table must fit its workspace region");

// Copies the parameter block into the workspace table (one CTA; 16 bytes per thread and step).
__global__ void __launch_bounds__(256)
k_dense_table(const __grid_constant__ DenseStackParams P, DenseStackParams* dst) {
  const uint4* src = reinterpret_cast<const uint4*>(&P);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (int i = threadIdx.x; i < (int)(sizeof(DenseStackParams) / 16); i += blockDim.x) d[i] = src[i];
}

// Outputs of the LAST layer (single-layer calls: the only one); earlier layers of a stack update
// the residual in place and write x_next to the alternating buffer.
struct DenseTail {
  void* out;            // [B, H] raw MLP output (type T, or fp32 accumulate if out_mode == 1), or null
  int out_mode;
  void* resid;          // [B, H] residual stream in/out, or null
  void* x_next;         // [B, H] rmsnorm(resid) [* norm_w], or null (needs resid)
  const void* norm_w;   // [H] or null
};

template <typename T, bool STACK>
__global__ void __launch_bounds__(kDenseThreads, 1)
k_dense(const DenseStackParams* __restrict__ Pg, const __grid_constant__ DenseLayerMaps M1, float thr1,
        const __grid_constant__ CUtensorMap map_xa, const __grid_constant__ CUtensorMap map_xb,
        const __grid_constant__ CUtensorMap map_h, WsPtrs ws, int L, int B, int H, int I,
        T* __restrict__ h_buf, int box_rows, T* __restrict__ x_tmp, const DenseTail tail, float eps,
        int S, int wait_kc) {
  using V = VecT<T>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int s_ctl[2];
  int& s_abort = s_ctl[0];
  __shared__ uint64_t s_bars[2 * 16 + 8];
  __shared__ uint32_t s_tmem;
  __shared__ int s_count[4];
  __shared__ float s_ss[1];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  // phase 1: this CTA's neurons
  const int r0 = seg_row0(c, G, I), r1 = seg_row0(c + 1, G, I);
  const int R = r1 - r0;
  const int ntile = (R + box_rows - 1) / box_rows;
  const int rows_per_tile = ntile ? (R + ntile - 1) / ntile : 0;
  const int nkb1 = (H + kDenseKB - 1) / kDenseKB;
  const int n1 = ntile * nkb1;                              // phase-1 stages per layer
  // phase 2: this CTA's split-K blocks of Wd
  const int nkb2 = (I + kDenseKB - 1) / kDenseKB, mt = H / 128;
  const long long U = (long long)mt * nkb2;
  const int u0 = (int)((U * c) / G), u1 = (int)((U * (c + 1)) / G);
  const int nu = u1 - u0;
  const int n2 = (nu + 1) / 2;                              // phase-2 stages (two blocks each)
  const int nl = n1 + n2;                                   // stages per layer
  const int m_first = nu ? u0 / nkb2 : 0, m_last = nu ? (u1 - 1) / nkb2 : -1;
  const int kb_first = nu ? u0 - m_first * nkb2 : 0;

  const uint32_t ring_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full_u = smem_u32(s_bars), empty_u = full_u + 8u * S;
  const uint32_t acc_full_u = empty_u + 8u * S, acc_empty_u = acc_full_u + 32u;   // 4 + 4 barriers
  const uint32_t tx1 = 2u * (uint32_t)box_rows * 128u + kDenseXTile;

  unsigned* dbar = reinterpret_cast<unsigned*>(ws.hdr + HDR_DBAR);
  const unsigned dbase = __ldcg(reinterpret_cast<const unsigned*>(ws.hdr + HDR_DBAR_BASE));
  // barrier n (1..4) of layer l
  auto dtarget = [&](int l, int n) { return dbase + (unsigned)(3 * l + n) * (unsigned)G; };
  auto maps = [&](int l) -> const DenseLayerMaps* { return STACK ? &Pg->m[l] : &M1; };

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, 1);
    }
    for (int b = 0; b < 4; ++b) {           // 0,1: phase-1 accumulator pairs; 2,3: phase-2
      mbar_init(acc_full_u + 8u * b, 1);
      mbar_init(acc_empty_u + 8u * b, 4);   // one arrival per epilogue warp
    }
    s_abort = 0;
    s_ctl[1] = wait_kc;
    mbar_fence_init();
  }
  if (tid < 4) s_count[tid] = 0;
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem), 128);   // phase 1: 2 x 32 columns, phase 2: 2 x 16
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;

  if (warp == 0) {
    // ================================================================== producer (one thread)
    if (lane == 0) {
      bool ok = true;
      const int total = L * nl;
      // a cursor over the stages: layer l, stage r of the layer, ring slot s, ring cycle cy;
      // phase 1: row tile t, column step kb; phase 2: first block's row tile m and column step kb
      struct Cur { int k, l, r, s, cy, t, kb, m; };
      auto advance = [&](Cur& q) {
        ++q.k;
        if (++q.s == S) { q.s = 0; ++q.cy; }
        ++q.r;
        if (q.r < n1) {
          if (++q.kb == nkb1) { q.kb = 0; ++q.t; }
        } else if (q.r == n1 && n2) {
          q.m = m_first; q.kb = kb_first;                   // first phase-2 stage of the layer
        } else if (q.r < nl) {
          q.kb += 2;                                        // two blocks per stage
          while (q.kb >= nkb2) { q.kb -= nkb2; ++q.m; }
        } else {
          q.r = 0; q.t = 0; q.kb = 0; ++q.l;
          if (n1 == 0) { q.m = m_first; q.kb = kb_first; }
        }
      };
      // the barrier a stage's activation block waits for (0: none)
      auto needs = [&](const Cur& q) {
        if (q.r >= n1) return dtarget(q.l, 1);
        return q.l ? dtarget(q.l - 1, 3) : 0u;
      };
      auto act_block = [&](const Cur& q) {
        const uint32_t st = ring_u + (uint32_t)q.s * kDenseStage + 2 * kDenseATile, bar = full_u + 8u * q.s;
        if (q.r < n1) {
          tma_load_2d(st, (q.l & 1) ? &map_xb : &map_xa, q.kb * kDenseKB, 0, bar);
        } else {
          const int nb = (2 * (q.r - n1) + 1 < nu) ? 2 : 1;
          int kb = q.kb;
          for (int i = 0; i < nb; ++i) {
            tma_load_2d(st + (uint32_t)i * kDenseXTile, &map_h, kb * kDenseKB, 0, bar);
            if (++kb == nkb2) kb = 0;
          }
        }
      };
      Cur cur = {0, 0, 0, 0, 0, 0, 0, 0};     // next stage whose weight blocks go out
      if (n1 == 0) { cur.m = m_first; cur.kb = kb_first; }
      Cur pend = cur;                          // first stage whose activation block is still owed
      unsigned done_target = dbase;            // highest barrier target known to have completed
      // issue owed activation blocks of stages [pend, upto); `block`: wait for their barriers
      auto settle = [&](int upto, bool block) {
        while (pend.k < upto && ok) {
          const unsigned need = needs(pend);
          if (need && (int)(done_target - need) < 0) {
            if (block) {
              ok = grid_wait(dbar, need, &s_abort);
              if (!ok) return;
            } else if ((int)(ld_acquire_gpu(dbar) - need) < 0) {
              return;
            }
            done_target = need;
            fence_proxy_async_all();
          }
          act_block(pend);
          advance(pend);
        }
      };
      while (cur.k < total && ok) {
        if (cur.k >= S) {
          settle(cur.k - S + 1, true);   // the stage this one replaces must be complete to drain
          if (!ok) break;
          if (!(ok = mbar_wait(empty_u + 8u * cur.s, (cur.cy - 1) & 1, &s_abort))) break;
        }
        const uint32_t st = ring_u + (uint32_t)cur.s * kDenseStage, bar = full_u + 8u * cur.s;
        const DenseLayerMaps* mp = maps(cur.l);
        if (cur.r < n1) {
          const int row = r0 + cur.t * rows_per_tile;
          mbar_expect_tx(bar, tx1);
          tma_load_2d(st, &mp->wg, cur.kb * kDenseKB, row, bar);
          tma_load_2d(st + kDenseATile, &mp->wu, cur.kb * kDenseKB, row, bar);
        } else {
          const int nb = (2 * (cur.r - n1) + 1 < nu) ? 2 : 1;
          mbar_expect_tx(bar, (uint32_t)nb * (kDenseATile + kDenseXTile));
          int m = cur.m, kb = cur.kb;
          for (int i = 0; i < nb; ++i) {
            tma_load_2d(st + (uint32_t)i * kDenseATile, &mp->wd, kb * kDenseKB, m * 128, bar);
            if (++kb == nkb2) { kb = 0; ++m; }
          }
        }
        advance(cur);
        settle(cur.k, false);            // whatever is already allowed goes out now
      }
      if (ok) settle(total, true);
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(UmmaFmt<T>::v);
      int tcount = 0, seg = 0, s = 0, cy = 0;   // ring slot and cycle, kept incrementally
      bool ok = true;
      for (int l = 0; l < L && ok; ++l) {
        for (int t = 0; t < ntile && ok; ++t, ++tcount) {
          const int buf = tcount & 1;
          if (tcount >= 2) ok = mbar_wait(acc_empty_u + 8u * buf, ((tcount >> 1) - 1) & 1, &s_abort);
          tc_fence_after();
          const uint32_t tg = tmem_base + (uint32_t)buf * 32u, tu = tg + 16u;
          for (int kb = 0; kb < nkb1 && ok; ++kb) {
            if (!(ok = mbar_wait(full_u + 8u * s, cy & 1, &s_abort))) break;
            tc_fence_after();
            const uint32_t st = ring_u + (uint32_t)s * kDenseStage;
            const uint64_t dg = umma_desc_k128(st), du = umma_desc_k128(st + kDenseATile),
                           dx = umma_desc_k128(st + 2 * kDenseATile);
#pragma unroll
            for (int kk = 0; kk < kDenseKB / 16; ++kk) {
              const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
              umma_f16(tg, dg + 2u * kk, dx + 2u * kk, idesc, acc);
              umma_f16(tu, du + 2u * kk, dx + 2u * kk, idesc, acc);
            }
            umma_commit(empty_u + 8u * s);    // the stage is free once these MMAs have read it
            if (++s == S) { s = 0; ++cy; }
          }
          if (ok) umma_commit(acc_full_u + 8u * buf);
        }
        int m_cur = -1, m2 = m_first, kb2 = kb_first;
        bool first = true;
        for (int j = 0; j < n2 && ok; ++j) {
          if (!(ok = mbar_wait(full_u + 8u * s, cy & 1, &s_abort))) break;
          tc_fence_after();
          const uint32_t st = ring_u + (uint32_t)s * kDenseStage;
          const int nb = (2 * j + 1 < nu) ? 2 : 1;
          for (int q = 0; q < nb && ok; ++q) {
            const int m = m2;
            if (++kb2 == nkb2) { kb2 = 0; ++m2; }
            if (m != m_cur) {
              if (m_cur >= 0) {
                umma_commit(acc_full_u + 8u * (2 + (seg & 1)));
                ++seg;
              }
              m_cur = m;
              first = true;
              if (seg >= 2)
                ok = mbar_wait(acc_empty_u + 8u * (2 + (seg & 1)), ((seg >> 1) - 1) & 1, &s_abort);
              tc_fence_after();
              if (!ok) break;
            }
            const uint64_t da = umma_desc_k128(st + (uint32_t)q * kDenseATile),
                           dh = umma_desc_k128(st + 2 * kDenseATile + (uint32_t)q * kDenseXTile);
            const uint32_t td = tmem_base + 64u + (uint32_t)(seg & 1) * 16u;
#pragma unroll
            for (int kk = 0; kk < kDenseKB / 16; ++kk)
              umma_f16(td, da + 2u * kk, dh + 2u * kk, idesc, (first && kk == 0) ? 0u : 1u);
            first = false;
          }
          if (ok) umma_commit(empty_u + 8u * s);
          if (++s == S) { s = 0; ++cy; }
        }
        if (ok && m_cur >= 0) {
          umma_commit(acc_full_u + 8u * (2 + (seg & 1)));
          ++seg;
        }
      }
    }
  } else {
    // ================================================================== epilogue (4 warps)
    const int q = warp & 3;                  // the TMEM lane quarter this warp may read
    const int et = q * 32 + lane;            // 0..127 among the epilogue threads
    bool ok = true;
    int my_count = 0, tcount = 0, seg = 0;
    const int ngrp = H >> 2;
    T* x_io = reinterpret_cast<T*>(tail.x_next);   // (stacks: the caller passes x_io here)
    // Grid barriers of the epilogue warps: ONE arrival and one poller per CTA (the four warps
    // meet at their named barrier first), so a barrier is 148 adds to one address, not 592.
    // Every epilogue thread calls these the same number of times whatever happened before.
    auto ep_arrive = [&]() {
      epilogue_bar_sync();
      if (et == 0 && !s_abort) grid_arrive(dbar);
    };
    auto ep_wait = [&](unsigned target) {
      if (et == 0 && !s_abort) grid_wait(dbar, target, &s_abort);
      epilogue_bar_sync();
      return !s_abort;
    };
    for (int l = 0; l < L; ++l) {
      const bool last = l + 1 == L;
      const float thr = STACK ? __ldg(&Pg->thr[l]) : thr1;
      my_count = 0;
      // ---- phase 1: h = mask(SiLU(g)) * u
      for (int t = 0; t < ntile; ++t, ++tcount) {
        const int buf = tcount & 1;
        if (ok) ok = mbar_wait_warp(acc_full_u + 8u * buf, (tcount >> 1) & 1, &s_abort);
        tc_fence_after();
        if (ok) {
          float g[16], u[16];
          const uint32_t ta = tmem_base + (uint32_t)buf * 32u + ((uint32_t)(q * 32) << 16);
          tmem_ld16(ta, g);
          tmem_ld16(ta + 16u, u);
          const int lr = t * rows_per_tile + q * 32 + lane;     // row within the CTA's range
          const int tile_rows = min(rows_per_tile, R - t * rows_per_tile);
          const bool valid = (q * 32 + lane) < tile_rows;
          bool any = false;
#pragma unroll
          for (int tok = 0; tok < kDenseN; ++tok) {
            if (tok < B) {
              const float sv = silu_f(g[tok]);
              const bool a = is_active(sv, thr);
              any |= a;
              if (valid) h_buf[(size_t)tok * I + r0 + lr] = V::from_f(a ? sv * u[tok] : 0.f);
            }
          }
          my_count += __popc(__ballot_sync(0xffffffffu, valid && any));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(acc_empty_u + 8u * buf);
      }
      ep_arrive();                                   // barrier 1
      // ---- phase 2: partial sums into the fp32 accumulators, one row tile at a time
      for (int m_cur = m_first; m_cur <= m_last; ++m_cur, ++seg) {
        const int buf = seg & 1;
        if (ok) ok = mbar_wait_warp(acc_full_u + 8u * (2 + buf), (seg >> 1) & 1, &s_abort);
        tc_fence_after();
        if (ok) {
          float d[16];
          tmem_ld16(tmem_base + 64u + (uint32_t)buf * 16u + ((uint32_t)(q * 32) << 16), d);
          const int row = m_cur * 128 + q * 32 + lane;
#pragma unroll
          for (int tok = 0; tok < kDenseN; ++tok)
            if (tok < B) atomicAdd(ws.acc32 + (size_t)tok * H + row, d[tok]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(acc_empty_u + 8u * (2 + buf));
      }
      ep_arrive();                                   // barrier 2
      ok = ep_wait(dtarget(l, 2)) && ok;
      // ---- tail: token b is finished by CTA b alone (4096-8192 columns are one round of loads
      // for 128 threads), so its sum of squares is a sum inside one CTA and needs no grid
      // barrier; the other CTAs go straight to the layer's last barrier
      T* out = last ? reinterpret_cast<T*>(tail.out) : nullptr;
      const int out_mode = last ? tail.out_mode : 0;
      T* resid = reinterpret_cast<T*>(tail.resid);
      // x_{l+1}: the alternating buffers inside a stack, the caller's pointer after the last layer
      T* xn = last ? reinterpret_cast<T*>(tail.x_next) : ((l & 1) ? x_io : x_tmp);
      const T* norm_w = last ? reinterpret_cast<const T*>(tail.norm_w) : nullptr;
      const bool want_norm = resid != nullptr && xn != nullptr && out_mode != 1;
      const bool mine = c < B;                 // (the host makes sure the grid has B CTAs)
      if (et == 0) s_ss[0] = 0.f;
      epilogue_bar_sync();
      // Every thread owns up to kTailG groups of four columns (H <= 8192) and fetches all of them
      // before it uses any: one round trip to L2 instead of one per group.  The new residual
      // stays in registers for the second pass.
      constexpr int kTailG = 16;
      union Pack { uint2 u; T e[4]; };
      Pack rr[kTailG];
      if (mine && ok) {
        float4 av[kTailG];
#pragma unroll
        for (int k = 0; k < kTailG; ++k) {
          const int g = et + 128 * k;
          if (g < ngrp) {
            av[k] = __ldcg(reinterpret_cast<const float4*>(ws.acc32 + (size_t)c * H) + g);
            if (resid && out_mode != 1)
              rr[k].u = *reinterpret_cast<const uint2*>(resid + (size_t)c * H + 4 * (size_t)g);
          }
        }
        float ssq = 0.f;
#pragma unroll
        for (int k = 0; k < kTailG; ++k) {
          const int g = et + 128 * k;
          if (g < ngrp) {
            reinterpret_cast<float4*>(ws.acc32 + (size_t)c * H)[g] = make_float4(0.f, 0.f, 0.f, 0.f);
            const float v[4] = {av[k].x, av[k].y, av[k].z, av[k].w};
            const size_t o = (size_t)c * H + 4 * (size_t)g;
            if (out_mode == 1) {
              float4* of = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o);
              float4 t = *of;
              t.x += v[0]; t.y += v[1]; t.z += v[2]; t.w += v[3];
              *of = t;
            } else {
              if (out) {
                Pack po;
#pragma unroll
                for (int i = 0; i < 4; ++i) po.e[i] = V::from_f(v[i]);
                *reinterpret_cast<uint2*>(out + o) = po.u;
              }
              if (resid) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const T rn = V::from_f(V::to_f(rr[k].e[i]) + v[i]);
                  rr[k].e[i] = rn;
                  const float rf = V::to_f(rn);
                  ssq = fmaf(rf, rf, ssq);
                }
                *reinterpret_cast<uint2*>(resid + o) = rr[k].u;
              }
            }
          }
        }
        if (want_norm) {
          ssq = warp_sum(ssq);
          if (lane == 0) atomicAdd(&s_ss[0], ssq);
        }
      }
      epilogue_bar_sync();
      if (mine && ok && want_norm) {
        const float rsq = rsqrtf(s_ss[0] / (float)H + eps);
        Pack nw[kTailG];
        if (norm_w) {
#pragma unroll
          for (int k = 0; k < kTailG; ++k) {
            const int g = et + 128 * k;
            if (g < ngrp) nw[k].u = *reinterpret_cast<const uint2*>(norm_w + 4 * (size_t)g);
          }
        }
#pragma unroll
        for (int k = 0; k < kTailG; ++k) {
          const int g = et + 128 * k;
          if (g < ngrp) {
            Pack py;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              T y = V::from_f(V::to_f(rr[k].e[i]) * rsq);
              if (norm_w) y = V::from_f(V::to_f(nw[k].e[i]) * V::to_f(y));
              py.e[i] = y;
            }
            *reinterpret_cast<uint2*>(xn + (size_t)c * H + 4 * (size_t)g) = py.u;
          }
        }
      }
      ep_arrive();                                   // barrier 3: x_{l+1} and the clean accumulators
    }
    if (lane == 0) s_count[q] = my_count;
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    ws.seg_count[c] = s_count[0] + s_count[1] + s_count[2] + s_count[3];
    if (s_abort) {
      atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_DENSE);
    } else if (c == 0) {
      ws.hdr[HDR_NSEG] = G;
      ws.hdr[HDR_DBAR_BASE] = (int)(dbase + (unsigned)(3 * L) * (unsigned)G);
    }
  }
  if (s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

}  // namespace cats
