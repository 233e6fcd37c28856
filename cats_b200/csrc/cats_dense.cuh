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
//   k_dense_gateup   CTA c owns ~I/148 consecutive neurons.  Per 64-column step of the hidden
//                    dimension one TMA box of Wg, one of Wu (box rows = the CTA's neurons, at
//                    most 128) and one of x land in a shared-memory stage (128-byte swizzle);
//                    one elected thread issues 2 x 4 tcgen05.mma (M 128, N 16, K 16) into two
//                    TMEM accumulators; tcgen05.commit hands the stage back to the producer.
//                    Epilogue (four warps, tcgen05.ld): h = mask(SiLU(g)) * u per token, rounded
//                    to the storage type and written token-major [16, I] for the next kernel.
//   k_dense_down     split-K: the (128-row tile of H) x (64-column step of I) blocks of Wd are
//                    dealt out evenly over the CTAs in order; partial sums leave the TMEM
//                    accumulator through fp32 reductions into the workspace accumulators, and
//                    the CTA that finishes last runs the same fused tail as the sparse kernels
//                    (store / residual add / RMS norm).  Its weight blocks do not depend on the
//                    previous kernel, so they are in flight before griddepcontrol.wait.
//
// All waits are bounded (see cats_tma.cuh); a CTA that gives up frees its tensor memory first.
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
template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__half> { static constexpr int v = 0; };
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr int v = 1; };

// ---------------------------------------------------------------------------------------------
// gate + up: h[t, i] = mask_t(SiLU(Wg[i,:] . x[t,:])) * (Wu[i,:] . x[t,:])
// Dynamic shared memory (after rounding its start up to 1024 bytes): S stages of
// [Wg block 16 KB][Wu block 16 KB][x block 2 KB, padded to 1 KB multiples].
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kDenseThreads, 1)
k_dense_gateup(const __grid_constant__ CUtensorMap map_wg, const __grid_constant__ CUtensorMap map_wu,
               const __grid_constant__ CUtensorMap map_x, WsPtrs ws, int B, int H, int I, float thr,
               T* __restrict__ h_out, int box_rows, int S, int wait_kc) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int s_ctl[2];
  int& s_abort = s_ctl[0];
  __shared__ uint64_t s_bars[2 * 16 + 4];
  __shared__ uint32_t s_tmem;
  __shared__ int s_count[4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int r0 = seg_row0(c, G, I), r1 = seg_row0(c + 1, G, I);
  const int R = r1 - r0;
  const int ntile = (R + box_rows - 1) / box_rows;         // row tiles of this CTA (1, or 2 at 70B)
  const int rows_per_tile = ntile ? (R + ntile - 1) / ntile : 0;
  const int nkb = (H + kDenseKB - 1) / kDenseKB;
  const uint32_t stage_bytes = 2 * kDenseATile + 2048;     // x block padded to 2 KB
  const uint32_t ring_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full_u = smem_u32(s_bars), empty_u = full_u + 8u * S;
  const uint32_t acc_full_u = empty_u + 8u * S, acc_empty_u = acc_full_u + 16u;
  const uint32_t tx_bytes = 2u * (uint32_t)box_rows * 128u + kDenseXTile;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_u + 8u * b, 1);
      mbar_init(acc_empty_u + 8u * b, 4);   // one arrival per epilogue warp
    }
    s_abort = 0;
    s_ctl[1] = wait_kc;
    mbar_fence_init();
  }
  if (tid < 4) s_count[tid] = 0;
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem), 64);   // 2 buffers x (gate 16 + up 16) columns
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;
  pdl_launch_dependents();   // the next grid may become resident as soon as resources allow

  if (warp == 0) {
    // ================================================================== producer (one thread)
    if (lane == 0) {
      // weights never change: the first stages' weight blocks are in flight before the previous
      // grid is done; their x blocks follow once x is final
      const int total = ntile * nkb;
      const int pre = total < S ? total : S;
      for (int k = 0; k < pre; ++k) {
        const int t = k / nkb, kb = k - t * nkb, row = r0 + t * rows_per_tile;
        const uint32_t st = ring_u + (uint32_t)k * stage_bytes, bar = full_u + 8u * k;
        mbar_expect_tx(bar, tx_bytes);
        tma_load_2d(st, &map_wg, kb * kDenseKB, row, bar);
        tma_load_2d(st + kDenseATile, &map_wu, kb * kDenseKB, row, bar);
      }
      pdl_wait();
      fence_proxy_async_all();
      for (int k = 0; k < pre; ++k)
        tma_load_2d(ring_u + (uint32_t)k * stage_bytes + 2 * kDenseATile, &map_x, (k % nkb) * kDenseKB,
                    0, full_u + 8u * k);
      for (int k = pre; k < total; ++k) {
        const int s = k % S;
        if (!mbar_wait(empty_u + 8u * s, ((k / S) - 1) & 1, &s_abort)) break;
        const int t = k / nkb, kb = k - t * nkb, row = r0 + t * rows_per_tile;
        const uint32_t st = ring_u + (uint32_t)s * stage_bytes, bar = full_u + 8u * s;
        mbar_expect_tx(bar, tx_bytes);
        tma_load_2d(st, &map_wg, kb * kDenseKB, row, bar);
        tma_load_2d(st + kDenseATile, &map_wu, kb * kDenseKB, row, bar);
        tma_load_2d(st + 2 * kDenseATile, &map_x, kb * kDenseKB, 0, bar);
      }
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(UmmaFmt<T>::v);
      int k = 0;
      bool ok = true;
      for (int t = 0; t < ntile && ok; ++t) {
        const int buf = t & 1;
        if (t >= 2) ok = mbar_wait(acc_empty_u + 8u * buf, ((t >> 1) - 1) & 1, &s_abort);
        tc_fence_after();
        const uint32_t tg = tmem_base + (uint32_t)buf * 32u, tu = tg + 16u;
        for (int kb = 0; kb < nkb && ok; ++kb, ++k) {
          const int s = k % S;
          if (!(ok = mbar_wait(full_u + 8u * s, (k / S) & 1, &s_abort))) break;
          tc_fence_after();
          const uint32_t st = ring_u + (uint32_t)s * stage_bytes;
          const uint64_t dg = umma_desc_k128(st), du = umma_desc_k128(st + kDenseATile),
                         dx = umma_desc_k128(st + 2 * kDenseATile);
#pragma unroll
          for (int kk = 0; kk < kDenseKB / 16; ++kk) {
            const uint32_t acc = (kb > 0 || kk > 0) ? 1u : 0u;
            umma_f16(tg, dg + 2u * kk, dx + 2u * kk, idesc, acc);
            umma_f16(tu, du + 2u * kk, dx + 2u * kk, idesc, acc);
          }
          umma_commit(empty_u + 8u * s);    // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(acc_full_u + 8u * buf);
      }
    }
  } else {
    // ================================================================== epilogue (4 warps)
    const int q = warp & 3;                  // the TMEM lane quarter this warp may read
    bool ok = true;
    int my_count = 0;
    for (int t = 0; t < ntile; ++t) {
      const int buf = t & 1;
      if (ok) ok = mbar_wait_warp(acc_full_u + 8u * buf, (t >> 1) & 1, &s_abort);
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
            if (valid) h_out[(size_t)tok * I + r0 + lr] = VecT<T>::from_f(a ? sv * u[tok] : 0.f);
          }
        }
        my_count += __popc(__ballot_sync(0xffffffffu, valid && any));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(acc_empty_u + 8u * buf);
    }
    if (lane == 0) s_count[q] = my_count;
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    ws.seg_count[c] = s_count[0] + s_count[1] + s_count[2] + s_count[3];
    if (c == 0) ws.hdr[HDR_NSEG] = G;
    if (s_abort) atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_DENSE);
  }
  if (s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
}

// ---------------------------------------------------------------------------------------------
// down: acc32[t, r] += sum over this CTA's blocks of Wd[r, i] * h[t, i]; last CTA: fused tail.
// Blocks (128-row tile m of H, 64-column step kb of I) are numbered m * nkb + kb and CTA c takes
// [c * U / G, (c + 1) * U / G): contiguous, so it touches few row tiles (two TMEM buffers alternate).
// Stage: [Wd block 16 KB][h block 2 KB].
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kDenseThreads, 1)
k_dense_down(const __grid_constant__ CUtensorMap map_wd, const __grid_constant__ CUtensorMap map_h,
             WsPtrs ws, int B, int H, int I, T* __restrict__ out, int out_mode, T* __restrict__ resid,
             T* __restrict__ x_next, const T* __restrict__ norm_w, float eps, int S, int wait_kc) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int s_ctl[2];
  int& s_abort = s_ctl[0];
  __shared__ uint64_t s_bars[2 * 16 + 4];
  __shared__ uint32_t s_tmem;
  __shared__ float s_red[32];
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int nkb = (I + kDenseKB - 1) / kDenseKB, mt = H / 128;
  const long long U = (long long)mt * nkb;
  const int u0 = (int)((U * c) / G), u1 = (int)((U * (c + 1)) / G);
  const int nu = u1 - u0;
  const uint32_t stage_bytes = kDenseATile + 2048;
  const uint32_t ring_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full_u = smem_u32(s_bars), empty_u = full_u + 8u * S;
  const uint32_t acc_full_u = empty_u + 8u * S, acc_empty_u = acc_full_u + 16u;
  const uint32_t tx_bytes = kDenseATile + kDenseXTile;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_u + 8u * b, 1);
      mbar_init(acc_empty_u + 8u * b, 4);
    }
    s_abort = 0;
    s_ctl[1] = wait_kc;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem), 32);   // 2 buffers x 16 columns
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem;
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // weight blocks first (they do not depend on the previous grid), then wait, then the h
      // blocks of those stages; from then on both per stage
      const int pre = nu < S ? nu : S;
      for (int k = 0; k < pre; ++k) {
        const int u = u0 + k, m = u / nkb, kb = u - m * nkb;
        mbar_expect_tx(full_u + 8u * k, tx_bytes);
        tma_load_2d(ring_u + (uint32_t)k * stage_bytes, &map_wd, kb * kDenseKB, m * 128, full_u + 8u * k);
      }
      pdl_wait();
      fence_proxy_async_all();
      for (int k = 0; k < pre; ++k) {
        const int u = u0 + k, kb = u % nkb;
        tma_load_2d(ring_u + (uint32_t)k * stage_bytes + kDenseATile, &map_h, kb * kDenseKB, 0,
                    full_u + 8u * k);
      }
      for (int k = pre; k < nu; ++k) {
        const int s = k % S;
        if (!mbar_wait(empty_u + 8u * s, ((k / S) - 1) & 1, &s_abort)) break;
        const int u = u0 + k, m = u / nkb, kb = u - m * nkb;
        const uint32_t st = ring_u + (uint32_t)s * stage_bytes, bar = full_u + 8u * s;
        mbar_expect_tx(bar, tx_bytes);
        tma_load_2d(st, &map_wd, kb * kDenseKB, m * 128, bar);
        tma_load_2d(st + kDenseATile, &map_h, kb * kDenseKB, 0, bar);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(UmmaFmt<T>::v);
      bool ok = true;
      int seg = 0, m_cur = -1;
      bool first = true;
      for (int k = 0; k < nu && ok; ++k) {
        const int u = u0 + k, m = u / nkb;
        if (m != m_cur) {
          if (m_cur >= 0) {
            umma_commit(acc_full_u + 8u * (seg & 1));
            ++seg;
          }
          m_cur = m;
          first = true;
          if (seg >= 2) ok = mbar_wait(acc_empty_u + 8u * (seg & 1), ((seg >> 1) - 1) & 1, &s_abort);
          tc_fence_after();
          if (!ok) break;
        }
        const int s = k % S;
        if (!(ok = mbar_wait(full_u + 8u * s, (k / S) & 1, &s_abort))) break;
        tc_fence_after();
        const uint32_t st = ring_u + (uint32_t)s * stage_bytes;
        const uint64_t da = umma_desc_k128(st), dh = umma_desc_k128(st + kDenseATile);
        const uint32_t td = tmem_base + (uint32_t)(seg & 1) * 16u;
#pragma unroll
        for (int kk = 0; kk < kDenseKB / 16; ++kk)
          umma_f16(td, da + 2u * kk, dh + 2u * kk, idesc, (first && kk == 0) ? 0u : 1u);
        first = false;
        umma_commit(empty_u + 8u * s);
      }
      if (ok && m_cur >= 0) umma_commit(acc_full_u + 8u * (seg & 1));
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    int seg = 0, m_cur = -1;
    // walk the same block sequence to learn the row tiles this CTA touches
    for (int k = 0; k <= nu; ++k) {
      const int m = (k < nu) ? (u0 + k) / nkb : -2;
      if (m == m_cur) continue;
      if (m_cur >= 0) {
        const int buf = seg & 1;
        if (ok) ok = mbar_wait_warp(acc_full_u + 8u * buf, (seg >> 1) & 1, &s_abort);
        tc_fence_after();
        if (ok) {
          float d[16];
          tmem_ld16(tmem_base + (uint32_t)buf * 16u + ((uint32_t)(q * 32) << 16), d);
          const int row = m_cur * 128 + q * 32 + lane;
#pragma unroll
          for (int tok = 0; tok < kDenseN; ++tok)
            if (tok < B) atomicAdd(ws.acc32 + (size_t)tok * H + row, d[tok]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(acc_empty_u + 8u * buf);
        ++seg;
      }
      m_cur = m;
    }
  }

  // completion ticket: the CTA that arrives last owns the epilogue
  __threadfence();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    if (s_abort) atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_DENSE);
    const unsigned t = atomicAdd(reinterpret_cast<unsigned*>(ws.hdr + HDR_TICKET), 1u);
    s_last = (t == (unsigned)G - 1u) ? 1 : 0;
  }
  __syncthreads();
  if (s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
  if (s_last) {
    __threadfence();
    finalize_down<T>(ws, B, H, out, out_mode, resid, x_next, norm_w, eps, s_red);
    if (tid == 0) ws.hdr[HDR_TICKET] = 0;
  }
}

// ---------------------------------------------------------------------------------------------
// The whole dense MLP in ONE cooperative launch: the two kernels above back to back in one ring.
//
// Why.  As separate launches each kernel pays its own ramp (first blocks in flight) and tail
// (last CTA, single-CTA epilogue): measured at the Mistral shape, 73 us per layer for 352 MB.
// Here one CTA per SM keeps one ring of 36 KB stages flowing through both GEMM phases:
//   phase 1  stage = [Wg block][Wu block][x block]          -> h = mask(SiLU(g)) * u
//   phase 2  stage = [Wd block][Wd block][h block][h block]  (two consecutive split-K blocks)
// The Wd blocks do not depend on h, so the producer issues up to a ring's worth of them before it
// waits for the grid barrier that says every CTA's h is written; only the small h blocks are
// issued after it.  The tail is spread over all CTAs as well: after a second barrier (all partial
// sums are in the fp32 accumulators) every CTA turns its own slice of the columns into out / the
// new residual and adds its part of each token's sum of squares; after a third, it writes its
// slice of the RMS-normalised x_next.
// Grid barriers: one monotonic counter in the workspace header (four arrivals per CTA and
// barrier, one per epilogue warp), its value at the start of the launch in the next slot; the
// per-token sums of squares alternate between two header arrays by launch parity, the array the
// next launch will use being cleared by this one.
// ---------------------------------------------------------------------------------------------
enum { HDR_DBAR = 16, HDR_DBAR_BASE = 17, HDR_DLAUNCH = 18, HDR_DSS = 32 /* [2][16] floats */ };
constexpr uint32_t kDenseStage = 2 * kDenseATile + 4096;   // 36 KB, both phases

template <typename T>
__global__ void __launch_bounds__(kDenseThreads, 1)
k_dense_mlp(const __grid_constant__ CUtensorMap map_wg, const __grid_constant__ CUtensorMap map_wu,
            const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wd,
            const __grid_constant__ CUtensorMap map_h, WsPtrs ws, int B, int H, int I, float thr,
            T* __restrict__ h_buf, int box_rows, T* __restrict__ out, int out_mode,
            T* __restrict__ resid, T* __restrict__ x_next, const T* __restrict__ norm_w, float eps,
            int S, int wait_kc) {
  using V = VecT<T>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ int s_ctl[2];
  int& s_abort = s_ctl[0];
  __shared__ uint64_t s_bars[2 * 16 + 8];
  __shared__ uint32_t s_tmem;
  __shared__ int s_count[4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  // phase 1: this CTA's neurons
  const int r0 = seg_row0(c, G, I), r1 = seg_row0(c + 1, G, I);
  const int R = r1 - r0;
  const int ntile = (R + box_rows - 1) / box_rows;
  const int rows_per_tile = ntile ? (R + ntile - 1) / ntile : 0;
  const int nkb1 = (H + kDenseKB - 1) / kDenseKB;
  const int n1 = ntile * nkb1;                              // phase-1 stages
  // phase 2: this CTA's split-K blocks of Wd
  const int nkb2 = (I + kDenseKB - 1) / kDenseKB, mt = H / 128;
  const long long U = (long long)mt * nkb2;
  const int u0 = (int)((U * c) / G), u1 = (int)((U * (c + 1)) / G);
  const int nu = u1 - u0;
  const int n2 = (nu + 1) / 2;                              // phase-2 stages (two blocks each)

  const uint32_t ring_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full_u = smem_u32(s_bars), empty_u = full_u + 8u * S;
  const uint32_t acc_full_u = empty_u + 8u * S, acc_empty_u = acc_full_u + 32u;   // 4 + 4 barriers
  const uint32_t tx1 = 2u * (uint32_t)box_rows * 128u + kDenseXTile;

  unsigned* dbar = reinterpret_cast<unsigned*>(ws.hdr + HDR_DBAR);
  const unsigned dbase = __ldcg(reinterpret_cast<const unsigned*>(ws.hdr + HDR_DBAR_BASE));
  const int par = __ldcg(ws.hdr + HDR_DLAUNCH) & 1;
  auto dtarget = [&](int n) { return dbase + (unsigned)n * 4u * (unsigned)G; };
  const bool want_norm = resid != nullptr && x_next != nullptr && out_mode != 1;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, 1);
    }
    for (int b = 0; b < 4; ++b) {           // 0,1: phase-1 accumulator pairs; 2,3: phase-2
      mbar_init(acc_full_u + 8u * b, 1);
      mbar_init(acc_empty_u + 8u * b, 4);
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
      int k = 0;
      for (; k < n1 && ok; ++k) {
        const int s = k % S;
        if (k >= S && !(ok = mbar_wait(empty_u + 8u * s, ((k / S) - 1) & 1, &s_abort))) break;
        const int t = k / nkb1, kb = k - t * nkb1, row = r0 + t * rows_per_tile;
        const uint32_t st = ring_u + (uint32_t)s * kDenseStage, bar = full_u + 8u * s;
        mbar_expect_tx(bar, tx1);
        tma_load_2d(st, &map_wg, kb * kDenseKB, row, bar);
        tma_load_2d(st + kDenseATile, &map_wu, kb * kDenseKB, row, bar);
        tma_load_2d(st + 2 * kDenseATile, &map_x, kb * kDenseKB, 0, bar);
      }
      // phase 2: the weight blocks run ahead of the barrier by up to a ring
      bool passed = false;
      int pending0 = 0;   // first phase-2 stage whose h blocks are still to be issued
      auto h_blocks = [&](int j) {
        const int s = (n1 + j) % S, ua = u0 + 2 * j, nb = (2 * j + 1 < nu) ? 2 : 1;
        const uint32_t st = ring_u + (uint32_t)s * kDenseStage + 2 * kDenseATile, bar = full_u + 8u * s;
        for (int q = 0; q < nb; ++q)
          tma_load_2d(st + (uint32_t)q * kDenseXTile, &map_h, ((ua + q) % nkb2) * kDenseKB, 0, bar);
      };
      auto pass = [&](int upto) {
        if (!passed) {
          ok = ok && grid_wait(dbar, dtarget(1), &s_abort);
          fence_proxy_async_all();
          passed = true;
        }
        if (ok)
          for (; pending0 < upto; ++pending0) h_blocks(pending0);
      };
      for (int j = 0; j < n2 && ok; ++j, ++k) {
        if (j == S) pass(j);                     // the ring wraps onto phase-2 stages: they need h
        const int s = k % S;
        if (k >= S && !(ok = mbar_wait(empty_u + 8u * s, ((k / S) - 1) & 1, &s_abort))) break;
        const int ua = u0 + 2 * j, nb = (2 * j + 1 < nu) ? 2 : 1;
        const uint32_t st = ring_u + (uint32_t)s * kDenseStage, bar = full_u + 8u * s;
        mbar_expect_tx(bar, (uint32_t)nb * (kDenseATile + kDenseXTile));
        for (int q = 0; q < nb; ++q) {
          const int u = ua + q, m = u / nkb2, kb = u - m * nkb2;
          tma_load_2d(st + (uint32_t)q * kDenseATile, &map_wd, kb * kDenseKB, m * 128, bar);
        }
        if (passed) {
          h_blocks(j);
          pending0 = j + 1;
        }
      }
      if (ok) pass(n2);
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(UmmaFmt<T>::v);
      int k = 0;
      bool ok = true;
      for (int t = 0; t < ntile && ok; ++t) {
        const int buf = t & 1;
        if (t >= 2) ok = mbar_wait(acc_empty_u + 8u * buf, ((t >> 1) - 1) & 1, &s_abort);
        tc_fence_after();
        const uint32_t tg = tmem_base + (uint32_t)buf * 32u, tu = tg + 16u;
        for (int kb = 0; kb < nkb1 && ok; ++kb, ++k) {
          const int s = k % S;
          if (!(ok = mbar_wait(full_u + 8u * s, (k / S) & 1, &s_abort))) break;
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
          umma_commit(empty_u + 8u * s);
        }
        if (ok) umma_commit(acc_full_u + 8u * buf);
      }
      // phase 2
      int seg = 0, m_cur = -1;
      bool first = true;
      for (int j = 0; j < n2 && ok; ++j, ++k) {
        const int s = k % S;
        if (!(ok = mbar_wait(full_u + 8u * s, (k / S) & 1, &s_abort))) break;
        tc_fence_after();
        const uint32_t st = ring_u + (uint32_t)s * kDenseStage;
        const int nb = (2 * j + 1 < nu) ? 2 : 1;
        for (int q = 0; q < nb && ok; ++q) {
          const int m = (u0 + 2 * j + q) / nkb2;
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
      }
      if (ok && m_cur >= 0) umma_commit(acc_full_u + 8u * (2 + (seg & 1)));
    }
  } else {
    // ================================================================== epilogue (4 warps)
    const int q = warp & 3;
    const int et = q * 32 + lane;            // 0..127 among the epilogue threads
    bool ok = true;
    int my_count = 0;
    // ---- phase 1: h = mask(SiLU(g)) * u
    for (int t = 0; t < ntile; ++t) {
      const int buf = t & 1;
      if (ok) ok = mbar_wait_warp(acc_full_u + 8u * buf, (t >> 1) & 1, &s_abort);
      tc_fence_after();
      if (ok) {
        float g[16], u[16];
        const uint32_t ta = tmem_base + (uint32_t)buf * 32u + ((uint32_t)(q * 32) << 16);
        tmem_ld16(ta, g);
        tmem_ld16(ta + 16u, u);
        const int lr = t * rows_per_tile + q * 32 + lane;
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
    if (lane == 0) s_count[q] = my_count;
    __syncwarp();
    if (lane == 0 && ok) grid_arrive(dbar);          // barrier 1: this warp's h rows are written
    // ---- phase 2: partial sums into the fp32 accumulators
    {
      int seg = 0, m_cur = -1;
      for (int k = 0; k <= nu; ++k) {
        const int m = (k < nu) ? (u0 + k) / nkb2 : -2;
        if (m == m_cur) continue;
        if (m_cur >= 0) {
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
          ++seg;
        }
        m_cur = m;
      }
    }
    __syncwarp();
    if (lane == 0 && ok) grid_arrive(dbar);          // barrier 2: this warp's sums are added
    if (lane == 0 && ok) ok = grid_wait(dbar, dtarget(2), &s_abort);   // one polling lane per warp
    ok = __all_sync(0xffffffffu, ok);
    // ---- tail, this CTA's slice of the columns (groups of four), all tokens
    const int ngrp = H >> 2;
    const int own_lo = (int)(((long long)ngrp * c) / G), own_hi = (int)(((long long)ngrp * (c + 1)) / G);
    const int own_n = own_hi - own_lo;
    float* ss_cur = reinterpret_cast<float*>(ws.hdr + HDR_DSS) + par * 16;
    float* ss_nxt = reinterpret_cast<float*>(ws.hdr + HDR_DSS) + (par ^ 1) * 16;
    if (c == 0 && et < 16) ss_nxt[et] = 0.f;         // for the next launch on this workspace
    for (int e = et; e < B * own_n && ok; e += 128) {
      const int b = e / own_n, g = own_lo + (e - b * own_n);
      float4* ap = reinterpret_cast<float4*>(ws.acc32 + (size_t)b * H) + g;
      const float4 a = __ldcg(ap);
      *ap = make_float4(0.f, 0.f, 0.f, 0.f);
      const float v[4] = {a.x, a.y, a.z, a.w};
      const size_t o = (size_t)b * H + 4 * (size_t)g;
      if (out_mode == 1) {
        float* of = reinterpret_cast<float*>(out) + o;
#pragma unroll
        for (int i = 0; i < 4; ++i) of[i] += v[i];
      } else {
        if (out) {
#pragma unroll
          for (int i = 0; i < 4; ++i) out[o + i] = V::from_f(v[i]);
        }
        if (resid) {
          float ssq = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const T rn = V::from_f(V::to_f(resid[o + i]) + v[i]);
            resid[o + i] = rn;
            const float rf = V::to_f(rn);
            ssq = fmaf(rf, rf, ssq);
          }
          if (want_norm) atomicAdd(ss_cur + b, ssq);
        }
      }
    }
    if (want_norm) {
      __syncwarp();
      if (lane == 0 && ok) grid_arrive(dbar);        // barrier 3: the sums of squares are complete
      if (lane == 0 && ok) ok = grid_wait(dbar, dtarget(3), &s_abort);
      ok = __all_sync(0xffffffffu, ok);
      for (int e = et; e < B * own_n && ok; e += 128) {
        const int b = e / own_n, g = own_lo + (e - b * own_n);
        const float rsq = rsqrtf(__ldcg(ss_cur + b) / (float)H + eps);
        const size_t o = (size_t)b * H + 4 * (size_t)g;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          T y = V::from_f(V::to_f(resid[o + i]) * rsq);
          if (norm_w) y = V::from_f(V::to_f(norm_w[4 * g + i]) * V::to_f(y));
          x_next[o + i] = y;
        }
      }
    } else {
      __syncwarp();
      if (lane == 0 && ok) grid_arrive(dbar);        // keeps three rounds of arrivals per launch
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    ws.seg_count[c] = s_count[0] + s_count[1] + s_count[2] + s_count[3];
    if (s_abort) {
      atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_DENSE);
    } else if (c == 0) {
      ws.hdr[HDR_NSEG] = G;
      ws.hdr[HDR_DBAR_BASE] = (int)(dbase + 12u * (unsigned)G);
      ws.hdr[HDR_DLAUNCH] = par ^ 1;
    }
  }
  if (s_abort) drain_after_abort();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

}  // namespace cats
