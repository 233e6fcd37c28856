// TMA-fed variants of the streaming kernels (sm_100a).
//
// A GEMV has one FMA per weight element, so the only thing that matters is how many bytes each
// SM keeps in flight towards HBM.  Here one elected producer thread per CTA issues 1-D bulk
// copies (cp.async.bulk global -> this CTA's shared memory, completion counted on an mbarrier;
// always the plain single-CTA form) of whole weight rows into a ring of stages, and eight
// consumer warps do the arithmetic out of shared memory.  Bytes in flight = ring size, decided by
// the host, independent of register allocation and occupancy.  One CTA per SM per kernel; the
// rings of the stage-1 kernel and the stage-2/3 kernel together fit one SM, so with programmatic
// dependent launch the next kernel is already resident while the current one drains, and the
// stage-1 kernel fills its ring with gate rows (weights never change) before it waits for the
// previous grid.
//
// Every wait on an mbarrier is bounded: when a limit is hit the CTA records an error status in
// the workspace header, stops issuing copies, lets the copies already in flight land and exits.
#pragma once

#include "cats_kernels.cuh"

namespace cats {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kMaxProducerWarps = 2;
constexpr int kTmaThreads = kConsumerThreads + 32 * kMaxProducerWarps;  // launch bound
// The block is 8 consumer warps + pw producer warps (1 or 2).  A single thread can issue an
// 8 KB bulk copy roughly every 240 ns, which caps one SM below its share of HBM bandwidth when a
// stage is one 8 KB row; two issuing threads lift that.  pw must divide the stage count so that
// each ring slot is always refilled by the same producer (it has then waited on every earlier
// phase of that slot's barrier itself).
// Every wait is bounded.  The limit lives in shared memory right behind the CTA's abort flag
// (abort[1], in units of 1024 clock cycles; the host derives it from the "wait_ms" option and the
// device's clock rate, default 1000 ms), so one pointer gives a wait both.
__device__ __forceinline__ long long wait_limit(volatile int* abort) {
  return (long long)abort[1] << 10;
}

enum { STATUS_OK = 0, STATUS_WAIT_TIMEOUT_GATE = 1, STATUS_WAIT_TIMEOUT_UPDOWN = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Non-blocking phase test (test_wait, not try_wait: a suspended try_wait of every idle warp keeps
// the shared-memory pipe busy and slows the warps that are working).
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the limit was hit or another thread of the CTA gave up.
// Polls back to back for the first few microseconds (ring hand-offs are that short and a sleep,
// however brief it is asked to be, costs about a microsecond), then backs off.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
    const long long dt = clock64() - t0;
    if (dt > 20000) __nanosleep(100);
    if (dt > wait_limit(abort)) {
      *abort = 1;
      return false;
    }
  }
}
// The same wait, with a call of `on_stall()` once the wait has lasted `stall_cycles`: a producer
// that stands that long is not held up by the ring's ordinary back-pressure but by consumers at a
// grid barrier, and can use the time.
template <typename F>
__device__ __forceinline__ bool mbar_wait_or(uint32_t bar, uint32_t parity, volatile int* abort,
                                             long long stall_cycles, F&& on_stall) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  bool told = false;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
    const long long dt = clock64() - t0;
    if (!told && dt > stall_cycles) {
      told = true;
      on_stall();
    }
    if (dt > 20000) __nanosleep(100);
    if (dt > wait_limit(abort)) {
      *abort = 1;
      return false;
    }
  }
}
// Ask for `bytes` (a multiple of 16, 16-byte aligned) of global memory to be brought into L2.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Whole-warp wait: lane 0 polls, the result is broadcast.  One polling lane per warp instead of
// 32 keeps the shared-memory pipe free for the warps that are working (32 lanes polling one
// barrier word serialise into 32 accesses per poll).  Must be called by a converged warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// 1-D bulk copy global -> shared memory of this CTA, completion on `bar` (plain single-CTA form).
__device__ __forceinline__ void tma_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Bulk add of `bytes` fp32 values from this CTA's shared memory into global memory (TMA reduce:
// one request per 128 bytes at L2 instead of one per 16-byte red).  Both addresses 16-byte
// aligned, bytes a multiple of 16.  The writes to shared memory that filled the source must be
// followed by fence_proxy_async() before this is issued.
__device__ __forceinline__ void bulk_reduce_add_f32(float* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile(
      "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
      "r"(src_smem), "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the source has been read (it may be overwritten) / the operations are complete
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void consumer_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}
// After an abort: give copies that are still in flight time to land before the CTA's shared
// memory is handed to another CTA.
__device__ __forceinline__ void drain_after_abort() {
  for (int i = 0; i < 2000; ++i) __nanosleep(1000);
}

// ---- grid barrier on a monotonic counter ------------------------------------------------------
// Arrival with release semantics at GPU scope.  It is always executed by lane 0 of a warp right
// after __syncwarp(), and everything the arrival publishes was written by lanes of that same
// warp, so this one fence is the only one on the path (an explicit __threadfence() by every
// writer plus a release here would pay the fence twice, and a fence costs microseconds while
// the copy ring saturates HBM).
__device__ __forceinline__ void grid_arrive(unsigned* ctr) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded spin until the counter has reached `target` (wrap-safe compare).
__device__ __forceinline__ bool grid_wait(const unsigned* ctr, unsigned target,
                                          volatile int* abort) {
  if ((int)(ld_acquire_gpu(ctr) - target) >= 0) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if ((int)(ld_acquire_gpu(ctr) - target) >= 0) return true;
      __nanosleep(40);
    }
    if (*abort) return false;
    if (clock64() - t0 > wait_limit(abort)) {
      *abort = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t n) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(n) : "memory");
}

// Dot products of up to two weight rows held in shared memory with the B activation vectors.
// XS: the activations were staged in shared memory too (else they come through L1).
// Four vectors of each row are fetched before the first FMA; even and odd vectors accumulate
// separately to halve the dependent-FMA chain.
template <typename T, int BT, bool XS>
__device__ __forceinline__ void warp_dot2_smem(const T* w0, const T* w1, const T* xs, int B,
                                               int H, int lane, float (&acc)[2][BT]) {
  constexpr int N = VecT<T>::N;
  constexpr int U = 4;
  const int nvec = H / N;
  const uint4* p0 = reinterpret_cast<const uint4*>(w0);
  const uint4* p1 = reinterpret_cast<const uint4*>(w1 ? w1 : w0);
  const uint4* px = reinterpret_cast<const uint4*>(xs);
  float odd[2][BT];
#pragma unroll
  for (int t = 0; t < BT; ++t) odd[0][t] = odd[1][t] = 0.f;
  int v = lane;
  for (; v + 32 * (U - 1) < nvec; v += 32 * U) {
    uint4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      a[u] = p0[v + 32 * u];
      b[u] = p1[v + 32 * u];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int t = 0; t < BT; ++t) {
        if (t < B) {
          const uint4 xv = XS ? px[(size_t)t * nvec + v + 32 * u]
                              : __ldg(px + (size_t)t * nvec + v + 32 * u);
          if (u & 1) VecT<T>::fma2(a[u], b[u], xv, odd[0][t], odd[1][t]);
          else VecT<T>::fma2(a[u], b[u], xv, acc[0][t], acc[1][t]);
        }
      }
    }
  }
  for (; v < nvec; v += 32) {
    const uint4 a = p0[v], b = p1[v];
#pragma unroll
    for (int t = 0; t < BT; ++t) {
      if (t < B) {
        const uint4 xv = XS ? px[(size_t)t * nvec + v] : __ldg(px + (size_t)t * nvec + v);
        VecT<T>::fma2(a, b, xv, acc[0][t], acc[1][t]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < BT; ++t) {
    acc[0][t] += odd[0][t];
    acc[1][t] += odd[1][t];
  }
}

// Dot product of ONE weight row held in shared memory with the B activation vectors (also in
// shared memory).  Eight vectors are fetched before the first FMA; four partial sums per token.
template <typename T, int BT>
__device__ __forceinline__ void warp_dot1_smem(const T* w0, const T* xs, int B, int H, int lane,
                                               float (&acc)[BT], int xs_ld = 0) {
  constexpr int N = VecT<T>::N;
  constexpr int U = 8;
  const int nvec = H / N;
  const uint4* p0 = reinterpret_cast<const uint4*>(w0);
  const uint4* px = reinterpret_cast<const uint4*>(xs);
  const int xv = (xs_ld ? xs_ld : H) / N;  // 16-byte vectors between the tokens' x
  float part[4][BT];
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int t = 0; t < BT; ++t) part[q][t] = 0.f;
  int v = lane;
  for (; v + 32 * (U - 1) < nvec; v += 32 * U) {
    uint4 a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) a[u] = p0[v + 32 * u];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int t = 0; t < BT; ++t)
        if (t < B) VecT<T>::fma1(a[u], px[(size_t)t * xv + v + 32 * u], part[u & 3][t]);
    }
  }
  for (; v < nvec; v += 32) {
    const uint4 a = p0[v];
#pragma unroll
    for (int t = 0; t < BT; ++t)
      if (t < B) VecT<T>::fma1(a, px[(size_t)t * xv + v], part[0][t]);
  }
#pragma unroll
  for (int t = 0; t < BT; ++t) acc[t] = (part[0][t] + part[1][t]) + (part[2][t] + part[3][t]);
}

// Tensor-core pieces of the batched dot products: D(16x8, fp32) += A(16x16) * B(16x8) on 16-bit
// inputs with only rows 0..7 of A in use (the other half of the fragment is zero): A = eight
// weight rows x 16 columns, B = 16 columns x eight tokens, D = eight rows x eight tokens.
// Products of 16-bit floats are exact in fp32 and the sums are fp32.
template <typename T>
struct Mma8;
template <>
struct Mma8<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};
template <>
struct Mma8<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};
template <>
struct Mma8<float> {  // fp32 weights never take this path
  static __device__ __forceinline__ void run(float (&)[4], uint32_t, uint32_t, uint32_t, uint32_t) {}
};
// Two 8x8 matrices of 16-bit values from shared memory: lanes 0-7 give the row addresses of the
// first, lanes 8-15 of the second (16 bytes per row); lane l receives elements
// [l / 4][2 * (l % 4) .. + 1] of each.
__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(addr));
}

// Copy the B activation vectors into shared memory (all threads of the CTA).
template <typename T>
__device__ __forceinline__ void stage_x(const T* __restrict__ x, T* xs, int B, int H) {
  const int nv = B * (H / VecT<T>::N);
  const uint4* src = reinterpret_cast<const uint4*>(x);
  uint4* dst = reinterpret_cast<uint4*>(xs);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = __ldcg(src + i);
}

// ---------------------------------------------------------------------------------------------
// Stage 1, TMA-fed.  One CTA per segment (grid = number of SMs); a stage holds SR consecutive
// rows of the segment (one contiguous copy); consumer warp w < cw owns stages w, w+cw, ...
// cw must divide S: then a warp's consecutive visits to one ring slot are exactly one barrier
// phase apart, which the parity wait needs (a waiter that is two phases ahead of a barrier
// would see the parity it waits for as already completed).
// Dynamic shared memory: [S stages][2*S mbarriers][rmax * BT floats][x: B*H elements if XS].
// ---------------------------------------------------------------------------------------------
template <typename T, int BT, int SR, bool XS>
__global__ void __launch_bounds__(kTmaThreads, 1)
k_gate_tma(const T* __restrict__ x, const T* __restrict__ Wg, WsPtrs ws, int B, int H, int I,
           float thr, T* __restrict__ gate_dense, uint8_t* __restrict__ flag_dense, int S,
           int cw, int rmax, int wait_kc, const T* __restrict__ pf_base, int pf_n) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_ctl[2];  // abort flag, wait limit
  int& s_abort = s_ctl[0];
  const uint32_t row_bytes = (uint32_t)H * sizeof(T), stage_bytes = SR * row_bytes;
  unsigned char* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)S * stage_bytes);
  float* s_val = reinterpret_cast<float*>(bars + 2 * S);
  T* xs = reinterpret_cast<T*>(
      smem + align_up((size_t)S * stage_bytes + 16 * (size_t)S + 4 * (size_t)rmax * BT, 16));
  const uint32_t ring_u = smem_u32(ring), full_u = smem_u32(bars), empty_u = full_u + 8u * S;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nseg = gridDim.x, c = blockIdx.x;
  const int r0 = seg_row0(c, nseg, I), r1 = seg_row0(c + 1, nseg, I);
  const int R = r1 - r0;
  const int nst = (R + SR - 1) / SR;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(Wg + (size_t)r0 * H);
  auto issue = [&](int k) {
    const int s = k % S;
    const int rows = min(SR, R - k * SR);
    const uint32_t bytes = rows * row_bytes;
    mbar_expect_tx(full_u + 8u * s, bytes);
    tma_load_1d(ring_u + s * stage_bytes, src + (size_t)k * stage_bytes, bytes, full_u + 8u * s);
  };

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, 1);
    }
    s_abort = 0;
    s_ctl[1] = wait_kc;
    mbar_fence_init();
  }
  __syncthreads();

  // gate rows do not depend on the previous grid: fill the ring first, wait afterwards
  const int npw = (blockDim.x >> 5) - kConsumerWarps, pw = warp - kConsumerWarps;
  int k_issued = pw;
  if (pw >= 0 && lane == 0)
    for (; k_issued < nst && k_issued < S; k_issued += npw) issue(k_issued);
  pdl_wait();
  pdl_launch_dependents();
  if (XS) {
    stage_x<T>(x, xs, B, H);
    __syncthreads();
  }
  const T* xsrc = XS ? xs : x;

  if (warp >= kConsumerWarps) {
    if (lane == 0) {
      for (int k = k_issued; k < nst; k += npw) {
        if (!mbar_wait(empty_u + 8u * (k % S), ((k / S) - 1) & 1, &s_abort)) break;
        issue(k);
      }
    }
  } else {
    for (int k = warp; warp < cw && k < nst; k += cw) {
      const int s = k % S;
      if (!mbar_wait_warp(full_u + 8u * s, (k / S) & 1, &s_abort)) break;
      const int lr = k * SR;
      const T* w0 = reinterpret_cast<const T*>(ring + (size_t)s * stage_bytes);
#pragma unroll
      for (int q = 0; q < SR; q += 2) {
        if (lr + q < R) {
          float acc[2][BT];
#pragma unroll
          for (int t = 0; t < BT; ++t) acc[0][t] = acc[1][t] = 0.f;
          const T* wa = w0 + (size_t)q * H;
          const bool two = (q + 1 < SR) && (lr + q + 1 < R);
          warp_dot2_smem<T, BT, XS>(wa, two ? wa + H : nullptr, xsrc, B, H, lane, acc);
#pragma unroll
          for (int t = 0; t < BT; ++t) {
            const float a0 = warp_sum(acc[0][t]);
            const float a1 = warp_sum(acc[1][t]);
            if (lane == 0) {
              s_val[(lr + q) * BT + t] = silu_f(a0);
              if (two) s_val[(lr + q + 1) * BT + t] = silu_f(a1);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_u + 8u * s);
    }
  }
  __syncthreads();
  if (s_abort) {
    if (tid == 0) atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_GATE);
    drain_after_abort();
  }

  // ballot / popc compaction of this segment, ascending neuron order
  if (warp == 0) {
    int base = 0;
    for (int g = 0; g < R; g += 32) {
      const int lr = g + lane;
      float v[BT];
      bool any = false;
#pragma unroll
      for (int t = 0; t < BT; ++t) {
        v[t] = 0.f;
        if (lr < R && t < B) {
          const float sv = s_val[lr * BT + t];
          const bool a = is_active(sv, thr);
          if (gate_dense) gate_dense[(size_t)t * I + r0 + lr] = VecT<T>::from_f(sv);
          if (flag_dense) flag_dense[(size_t)t * I + r0 + lr] = a ? 1 : 0;
          v[t] = a ? sv : 0.f;
          any |= a;
        }
      }
      const unsigned m = __ballot_sync(0xffffffffu, any);
      if (any) {
        const int rank = base + __popc(m & ((1u << lane) - 1u));
        const int pos = r0 + rank;
        ws.seg_idx[pos] = r0 + lr;
        // The stage-2 kernel of CTA c starts with (about) this segment's first active neurons,
        // and between this point and its first copy HBM idles (this grid's tail, the launch,
        // counts -> scan -> list): have their up-projection rows brought into L2 meanwhile.
        if (pf_base && rank < pf_n) l2_prefetch(pf_base + (size_t)(r0 + lr) * H, row_bytes);
#pragma unroll
        for (int t = 0; t < BT; ++t)
          if (t < B) ws.seg_gate[(size_t)pos * B + t] = v[t];
      }
      base += __popc(m);
    }
    if (lane == 0) {
      ws.seg_count[c] = base;
      if (c == 0) ws.hdr[HDR_NSEG] = nseg;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Stages 2+3, TMA-fed.  One CTA per SM takes positions [c*n/G, (c+1)*n/G) of the active list.
// The producer streams the cnt gathered Wu rows and then the cnt gathered WdT rows, one row per
// ring stage.
//   Up rows: consumer warp w < cw owns items w, w+cw, ... (cw divides S, as in stage 1); it
//   releases the stage for all eight warps at once (arrive with count 8).
//   Down rows: every consumer thread owns NVT 16-byte column groups and accumulates h_j * row in
//   fp32 registers; all eight warps pass every stage in order (wait full, arrive empty once).
// A consumer-only barrier separates the two phases, so every h_j is final before it is used and
// every ring barrier is past its last up-row phase before a down-row waiter looks at it.
// Dynamic shared memory: [S stages][2*S mbarriers][cap ints][cap*BT floats][x if XS].
// ---------------------------------------------------------------------------------------------
template <typename T, int BT, int NVT, bool XS>
__global__ void __launch_bounds__(kTmaThreads, 1)
k_updown_tma(const T* __restrict__ x, const T* __restrict__ Wu, const T* __restrict__ WdT,
             WsPtrs ws, int B, int H, int I, int cap, T* __restrict__ out, int out_mode,
             T* __restrict__ resid, T* __restrict__ x_next, const T* __restrict__ norm_w,
             float eps, int S, int cw, int wait_kc) {
  using V = VecT<T>;
  constexpr int N = V::N;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_incl[kMaxSeg];
  __shared__ int s_part[kWarps + 2];
  __shared__ float s_red[32];
  __shared__ int s_last;
  __shared__ int s_ctl[2];  // abort flag, wait limit
  int& s_abort = s_ctl[0];

  const uint32_t row_bytes = (uint32_t)H * sizeof(T);
  unsigned char* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)S * row_bytes);
  int* s_idx = reinterpret_cast<int*>(bars + 2 * S);
  float* s_h = reinterpret_cast<float*>(s_idx + cap);
  T* xs = reinterpret_cast<T*>(smem + align_up((size_t)S * row_bytes + 16 * (size_t)S +
                                                   4 * (size_t)cap * (1 + BT), 16));
  const uint32_t ring_u = smem_u32(ring), full_u = smem_u32(bars), empty_u = full_u + 8u * S;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int nvec = H / N;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_u + 8u * s, 1);
      mbar_init(empty_u + 8u * s, kConsumerWarps);
    }
    s_abort = 0;
    s_ctl[1] = wait_kc;
    mbar_fence_init();
  }
  // x is the input of this layer's stage 1 as well: it was final before that grid started, so
  // it can be staged before waiting for stage 1 to finish
  if (XS) stage_x<T>(x, xs, B, H);
  __syncthreads();

  pdl_wait();
  pdl_launch_dependents();

  int nseg;
  const int n = scan_segments(ws.seg_count, ws.hdr + HDR_NSEG, &nseg, s_incl, s_part);
  if (c == 0 && tid == 0) ws.hdr[HDR_NACTIVE] = n;
  const int p0 = (int)(((long long)c * n) / G), p1 = (int)(((long long)(c + 1) * n) / G);
  const int cnt = p1 - p0;
  for (int j = tid; j < cnt; j += blockDim.x) {
    const int q = locate(s_incl, nseg, I, p0 + j);
    s_idx[j] = __ldcg(ws.seg_idx + q);
#pragma unroll
    for (int t = 0; t < BT; ++t)
      s_h[j * BT + t] = (t < B) ? __ldcg(ws.seg_gate + (size_t)q * B + t) : 0.f;
  }
  __syncthreads();
  const T* xsrc = XS ? xs : x;

  const int nitems = 2 * cnt;
  if (warp >= kConsumerWarps) {
    if (lane == 0) {
      const int npw = (blockDim.x >> 5) - kConsumerWarps;
      for (int k = warp - kConsumerWarps; k < nitems; k += npw) {
        const int s = k % S;
        if (k >= S && !mbar_wait(empty_u + 8u * s, ((k / S) - 1) & 1, &s_abort)) break;
        const T* src = (k < cnt) ? Wu + (size_t)s_idx[k] * H : WdT + (size_t)s_idx[k - cnt] * H;
        mbar_expect_tx(full_u + 8u * s, row_bytes);
        tma_load_1d(ring_u + s * row_bytes, src, row_bytes, full_u + 8u * s);
      }
    }
  } else {
    bool ok = true;
    // up rows: warp-strided, one row per visit
    for (int k = warp; warp < cw && k < cnt; k += cw) {
      const int s = k % S;
      if (!(ok = mbar_wait_warp(full_u + 8u * s, (k / S) & 1, &s_abort))) break;
      float acc[2][BT];
#pragma unroll
      for (int t = 0; t < BT; ++t) acc[0][t] = acc[1][t] = 0.f;
      const T* w0 = reinterpret_cast<const T*>(ring + (size_t)s * row_bytes);
      warp_dot2_smem<T, BT, XS>(w0, nullptr, xsrc, B, H, lane, acc);
#pragma unroll
      for (int t = 0; t < BT; ++t) {
        const float a0 = warp_sum(acc[0][t]);
        if (lane == 0) s_h[k * BT + t] *= a0;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_n(empty_u + 8u * s, kConsumerWarps);
    }
    consumer_bar_sync();  // every h_j of this CTA is final
    ok = ok && !s_abort;
    // Down rows in groups of kDG: lane q waits for the q-th row of the group (one round trip to
    // the barrier unit per group instead of one per row), every thread loads the group's vectors
    // of its columns before the first FMA, then lane q releases the q-th stage.  16-bit weights
    // go through the mixed-precision FMAs (no conversion instructions), as in the persistent
    // kernel.
    float acc[NVT][BT][N];
#pragma unroll
    for (int g = 0; g < NVT; ++g)
#pragma unroll
      for (int t = 0; t < BT; ++t)
#pragma unroll
        for (int i = 0; i < N; ++i) acc[g][t][i] = 0.f;
    constexpr int kDG = (NVT * BT * N > 64) ? 4 : 8;   // fewer rows in flight where the accumulators fill the registers
    const int dg = S < kDG ? S : kDG;                   // a group must fit in the ring
    for (int j0 = 0; j0 < cnt && ok; j0 += dg) {
      const int nb = (cnt - j0) < dg ? (cnt - j0) : dg;
      bool mine = true;
      int my_slot = 0;
      if (lane < nb) {
        const int kk = cnt + j0 + lane;
        my_slot = kk % S;
        mine = mbar_wait(full_u + 8u * my_slot, (kk / S) & 1, &s_abort);
      }
      ok = __all_sync(0xffffffffu, mine);
      if (!ok) break;
      typename V::Scalar hb[kDG][BT];
      const uint4* rowp[kDG];
#pragma unroll
      for (int q = 0; q < kDG; ++q) {
        const int qq = q < nb ? q : 0;
        const int slot = __shfl_sync(0xffffffffu, my_slot, qq);
        rowp[q] = reinterpret_cast<const uint4*>(ring + (size_t)slot * row_bytes);
#pragma unroll
        for (int t = 0; t < BT; ++t) hb[q][t] = V::prep(q < nb ? s_h[(j0 + q) * BT + t] : 0.f);
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
            for (int t = 0; t < BT; ++t) V::axpy(hb[q][t], wq[q], acc[g][t]);
        }
      }
      __syncwarp();
      if (lane < nb) mbar_arrive(empty_u + 8u * my_slot);
    }
    // The CTA's partial sums leave through the ring, which is idle now (every row has been
    // consumed): fp32 [B, H] staged in shared memory, then ONE bulk reduce-add per token into
    // the accumulators (one request per 128 bytes at L2) instead of a 16-byte red per thread
    // and vector - 148 CTAs adding to the same 16 KB serialise there.  Falls back to the reds
    // where the ring is smaller than B * H floats.
    const bool bulk = (size_t)S * row_bytes >= (size_t)B * H * sizeof(float);
    consumer_bar_sync();  // every warp has read its columns of the last rows: the ring is free
    if (cnt > 0 && ok) {
      float* stg = reinterpret_cast<float*>(ring);
#pragma unroll
      for (int g = 0; g < NVT; ++g) {
        const int v = g * kConsumerThreads + tid;
        if (v < nvec) {
#pragma unroll
          for (int t = 0; t < BT; ++t) {
            if (t < B) {
              float* dst = (bulk ? stg : ws.acc32) + (size_t)t * H + (size_t)v * N;
#pragma unroll
              for (int i = 0; i < N; i += 4) {
                if (bulk)
                  *reinterpret_cast<float4*>(dst + i) =
                      make_float4(acc[g][t][i], acc[g][t][i + 1], acc[g][t][i + 2], acc[g][t][i + 3]);
                else
                  red_add_v4(dst + i, acc[g][t][i], acc[g][t][i + 1], acc[g][t][i + 2],
                             acc[g][t][i + 3]);
              }
            }
          }
        }
      }
      if (bulk) fence_proxy_async_smem();
    }
    consumer_bar_sync();  // the staged sums are complete
    if (bulk && tid == 0 && cnt > 0 && !s_abort) {
      for (int t = 0; t < B; ++t)
        bulk_reduce_add_f32(ws.acc32 + (size_t)t * H, ring_u + (uint32_t)t * H * (uint32_t)sizeof(float),
                            (uint32_t)H * (uint32_t)sizeof(float));
      bulk_commit();
      bulk_wait_all();
    }
  }

  // completion ticket: the CTA that arrives last owns the epilogue
  __threadfence();
  __syncthreads();
  if (s_abort) {
    if (tid == 0) atomicMax(ws.hdr + HDR_STATUS, STATUS_WAIT_TIMEOUT_UPDOWN);
    drain_after_abort();
  }
  if (tid == 0) {
    const unsigned t = atomicAdd(reinterpret_cast<unsigned*>(ws.hdr + HDR_TICKET), 1u);
    s_last = (t == (unsigned)G - 1u) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    finalize_down<T>(ws, B, H, out, out_mode, resid, x_next, norm_w, eps, s_red);
    if (tid == 0) ws.hdr[HDR_TICKET] = 0;
  }
}

}  // namespace cats
