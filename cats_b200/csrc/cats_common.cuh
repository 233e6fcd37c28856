// Shared device helpers for the CATS sparse-MLP decode kernels (sm_100a).
//
// Everything here is CUDA-core code on purpose: batch-1 decode is a GEMV, one FMA per weight
// element read from HBM, so the kernels are shaped around bytes in flight per SM (16-byte
// streaming loads, many independent loads per lane) and not around tensor cores.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cats {

constexpr int kThreads = 256;        // threads per CTA of every streaming kernel
constexpr int kWarps = kThreads / 32;
constexpr int kMaxSeg = 1024;        // upper bound on stage-1 segments (= stage-1 CTAs)
constexpr int kMaxB = 16;            // largest batch the kernels are instantiated for
constexpr int kHdrInts = 64;         // workspace header size in ints

// header slots
enum { HDR_NACTIVE = 0, HDR_TICKET = 1, HDR_STATUS = 2, HDR_NSEG = 3 };

// Resolved workspace pointers (see ws_layout).
struct WsPtrs {
  int* hdr;          // [kHdrInts]
  int* seg_count;    // [kMaxSeg]   active neurons found by stage-1 CTA c
  float* acc32;      // [2][kMaxB * H] split-K accumulators (two buffers), zero between calls
  int* seg_idx;      // [I]         segment c's ordered neuron list starts at row0(c)
  float* seg_gate;   // [I * B]     gate value per list entry and token (0 = token inactive)
  int* flat_idx;     // [I]         globally ordered list (written by stage 2 / compact)
  float* h;          // [I * B]     gate * up per flat list entry and token
  unsigned char* table;  // [kWsTableBytes] per-launch tables of the dense stack kernel (TMA maps)
};
constexpr size_t kWsTableBytes = 48 * 1024;

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Layout is a function of (H, I) only: the batch dimension is always provisioned for kMaxB so
// one workspace serves any B without moving the zero-initialised accumulator region.
__host__ __device__ inline size_t ws_layout(void* base, int H, int I, WsPtrs* p) {
  size_t off = 0;
  char* b = static_cast<char*>(base);
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 256);
    return o;
  };
  size_t o_hdr = take(sizeof(int) * kHdrInts);
  size_t o_cnt = take(sizeof(int) * kMaxSeg);
  size_t o_acc = take(sizeof(float) * 2 * (size_t)kMaxB * H);
  size_t o_sidx = take(sizeof(int) * (size_t)I);
  size_t o_sgate = take(sizeof(float) * (size_t)I * kMaxB);
  size_t o_fidx = take(sizeof(int) * (size_t)I);
  size_t o_h = take(sizeof(float) * (size_t)I * kMaxB);
  size_t o_tab = take(kWsTableBytes);
  if (p) {
    p->hdr = reinterpret_cast<int*>(b + o_hdr);
    p->seg_count = reinterpret_cast<int*>(b + o_cnt);
    p->acc32 = reinterpret_cast<float*>(b + o_acc);
    p->seg_idx = reinterpret_cast<int*>(b + o_sidx);
    p->seg_gate = reinterpret_cast<float*>(b + o_sgate);
    p->flat_idx = reinterpret_cast<int*>(b + o_fidx);
    p->h = reinterpret_cast<float*>(b + o_h);
    p->table = reinterpret_cast<unsigned char*>(b + o_tab);
  }
  return off;
}

// First row of stage-1 segment c out of nseg over I rows (balanced, ascending).
__host__ __device__ inline int seg_row0(int c, int nseg, int I) {
  return (int)(((long long)c * I) / nseg);
}

// ---------------------------------------------------------------------------------------------
// 16-byte vectors of the three element types
// ---------------------------------------------------------------------------------------------
template <typename T>
struct VecT;

template <>
struct VecT<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
  // acc0 += a . x, acc1 += b . x over the 4 elements of the vectors
  static __device__ __forceinline__ void fma2(const uint4& a, const uint4& b, const uint4& x,
                                              float& acc0, float& acc1) {
    float fa[4], fb[4], fx[4];
    unpack(a, fa);
    unpack(b, fb);
    unpack(x, fx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc0 = fmaf(fa[i], fx[i], acc0);
      acc1 = fmaf(fb[i], fx[i], acc1);
    }
  }
  // acc += a . x
  static __device__ __forceinline__ void fma1(const uint4& a, const uint4& x, float& acc) {
    float fa[4], fx[4];
    unpack(a, fa);
    unpack(x, fx);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc = fmaf(fa[i], fx[i], acc);
  }
  // scalar prepared for axpy (see the 16-bit specialisations)
  typedef float Scalar;
  static __device__ __forceinline__ Scalar prep(float h) { return h; }
  // acc[i] += h * w[i]
  static __device__ __forceinline__ void axpy(Scalar h, const uint4& w, float* acc) {
    float fw[4];
    unpack(w, fw);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(h, fw[i], acc[i]);
  }
};

// Blackwell mixed-precision FMA: d = a * b + c with 16-bit a, b and fp32 c, d.  The product of
// two 16-bit floats is exact in fp32, so this equals fmaf(float(a), float(b), c) without the two
// conversions.  One call handles a packed pair from each of two weight rows against one x pair.
#define CATS_MIXED_FMA2(SUFFIX)                                                              \
  asm("{\n\t.reg .b16 al, ah, bl, bh, xl, xh;\n\t"                                           \
      "mov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\tmov.b32 {xl, xh}, %4;\n\t"          \
      "fma.rn.f32." SUFFIX " %0, al, xl, %0;\n\tfma.rn.f32." SUFFIX " %1, bl, xl, %1;\n\t"   \
      "fma.rn.f32." SUFFIX " %0, ah, xh, %0;\n\tfma.rn.f32." SUFFIX " %1, bh, xh, %1;\n\t}"  \
      : "+f"(acc0), "+f"(acc1)                                                               \
      : "r"(aw), "r"(bw), "r"(xw))
#define CATS_MIXED_FMA1(SUFFIX)                                                              \
  asm("{\n\t.reg .b16 al, ah, xl, xh;\n\t"                                                   \
      "mov.b32 {al, ah}, %1;\n\tmov.b32 {xl, xh}, %2;\n\t"                                    \
      "fma.rn.f32." SUFFIX " %0, al, xl, %0;\n\tfma.rn.f32." SUFFIX " %0, ah, xh, %0;\n\t}"  \
      : "+f"(acc)                                                                            \
      : "r"(aw), "r"(xw))

template <>
struct VecT<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ void fma2(const uint4& a, const uint4& b, const uint4& x,
                                              float& acc0, float& acc1) {
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w},
                   xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw = av[i], bw = bv[i], xw = xv[i];
      CATS_MIXED_FMA2("f16");
    }
  }
  static __device__ __forceinline__ void fma1(const uint4& a, const uint4& x, float& acc) {
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw = av[i], xw = xv[i];
      CATS_MIXED_FMA1("f16");
    }
  }
  // axpy without converting the weights: the fp32 scalar h is split into two halves,
  // h ~= hi + lo (22 significant bits; exact to ~2^-22 relative for |h| >= 2^-3 and to 2^-25
  // absolute below), and each weight takes two mixed-precision FMAs.  The conversion
  // instruction it replaces runs at a fraction of the FMA rate and was the bottleneck.
  typedef uint32_t Scalar;  // {hi, lo} packed
  static __device__ __forceinline__ Scalar prep(float h) {
    const __half hi = __float2half_rn(h);
    const __half lo = __float2half_rn(h - __half2float(hi));
    return (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
  }
  static __device__ __forceinline__ void axpy(Scalar h, const uint4& w, float* acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      asm("{\n\t.reg .b16 wl, wh, hi, lo;\n\tmov.b32 {wl, wh}, %2;\n\tmov.b32 {hi, lo}, %3;\n\t"
          "fma.rn.f32.f16 %0, wl, hi, %0;\n\tfma.rn.f32.f16 %0, wl, lo, %0;\n\t"
          "fma.rn.f32.f16 %1, wh, hi, %1;\n\tfma.rn.f32.f16 %1, wh, lo, %1;\n\t}"
          : "+f"(acc[2 * i]), "+f"(acc[2 * i + 1])
          : "r"(wv[i]), "r"(h));
    }
  }
  // axpy with the scalar rounded to the storage type (what the reference's stage 2 hands to its
  // stage 3: flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu keeps gate*up in the weights' dtype):
  // one mixed-precision FMA per weight.  Used for batches, where the FMA count is the limit.
  static __device__ __forceinline__ uint32_t prep1(float h) {
    return (uint32_t)__half_as_ushort(__float2half_rn(h));
  }
  static __device__ __forceinline__ void axpy1(uint32_t h, const uint4& w, float* acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      asm("{\n\t.reg .b16 wl, wh, hh, hx;\n\tmov.b32 {wl, wh}, %2;\n\tmov.b32 {hh, hx}, %3;\n\t"
          "fma.rn.f32.f16 %0, wl, hh, %0;\n\tfma.rn.f32.f16 %1, wh, hh, %1;\n\t}"
          : "+f"(acc[2 * i]), "+f"(acc[2 * i + 1])
          : "r"(wv[i]), "r"(h));
    }
  }
};

template <>
struct VecT<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) {
    return __float2bfloat16_rn(v);
  }
  static __device__ __forceinline__ void fma2(const uint4& a, const uint4& b, const uint4& x,
                                              float& acc0, float& acc1) {
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w},
                   xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw = av[i], bw = bv[i], xw = xv[i];
      CATS_MIXED_FMA2("bf16");
    }
  }
  static __device__ __forceinline__ void fma1(const uint4& a, const uint4& x, float& acc) {
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t aw = av[i], xw = xv[i];
      CATS_MIXED_FMA1("bf16");
    }
  }
  // bf16 -> fp32 is a shift / mask on the integer pipe: plain fp32 FMAs, exact
  typedef float Scalar;
  static __device__ __forceinline__ Scalar prep(float h) { return h; }
  static __device__ __forceinline__ void axpy(Scalar h, const uint4& w, float* acc) {
    float fw[8];
    unpack(w, fw);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(h, fw[i], acc[i]);
  }
  static __device__ __forceinline__ uint32_t prep1(float h) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(h));
  }
  static __device__ __forceinline__ void axpy1(uint32_t h, const uint4& w, float* acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      asm("{\n\t.reg .b16 wl, wh, hh, hx;\n\tmov.b32 {wl, wh}, %2;\n\tmov.b32 {hh, hx}, %3;\n\t"
          "fma.rn.f32.bf16 %0, wl, hh, %0;\n\tfma.rn.f32.bf16 %1, wh, hh, %1;\n\t}"
          : "+f"(acc[2 * i]), "+f"(acc[2 * i + 1])
          : "r"(wv[i]), "r"(h));
    }
  }
};

// Streaming 16-byte load of weight data: read-only path, no L1 allocation so that the
// activations (re-read for every row) stay resident in L1.
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}

// Compiler-only fence: keeps every load issued above it ahead of the arithmetic below it, so a
// lane really has all of them in flight before it waits for the first one.
__device__ __forceinline__ void issue_fence() { asm volatile("" ::: "memory"); }

// Vector reduction into global fp32 accumulators (one L2 atomic transaction per 16 bytes).
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// Programmatic dependent launch: wait until every grid this one depends on has completed and
// its memory is visible (no-op when the launch carried no programmatic dependency) ...
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// ... and allow the next grid in the stream to be scheduled once all CTAs got here.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// Active rule of the reference: a neuron is dead when |v| <= t (ugly_utils.py:897), so it is
// active when that comparison is false — NaN stays active and propagates, as it does there.
__device__ __forceinline__ bool is_active(float v, float t) { return !(fabsf(v) <= t); }

// ---------------------------------------------------------------------------------------------
// Dot products of up to two weight rows with the B activation vectors, one warp per call.
//   w0 / w1 : row starts (w1 may be nullptr), xs : [B, H] activations
//   acc[r][b] receives this lane's partial sums (caller reduces across the warp).
// Per outer step every lane issues 2*U independent 16-byte loads before the first FMA.
// ---------------------------------------------------------------------------------------------
// FMA one 16-byte vector of up to two rows against the B activation vectors.
template <typename T, int BT>
__device__ __forceinline__ void fma_vec2(const uint4& a, const uint4& b, const uint4* px, int nvec,
                                         int v, int B, float (&acc)[2][BT]) {
#pragma unroll
  for (int t = 0; t < BT; ++t) {
    if (t < B) VecT<T>::fma2(a, b, __ldg(px + (size_t)t * nvec + v), acc[0][t], acc[1][t]);
  }
}

template <typename T, int BT, int U>
__device__ __forceinline__ void warp_dot2(const T* __restrict__ w0, const T* __restrict__ w1,
                                          const T* __restrict__ xs, int B, int H, int lane,
                                          float (&acc)[2][BT]) {
  constexpr int N = VecT<T>::N;
  const int nvec = H / N;
  const uint4* p0 = reinterpret_cast<const uint4*>(w0);
  // a missing second row re-reads the first (its sums are discarded by the caller): keeps the
  // main loop free of per-load predicates
  const uint4* p1 = reinterpret_cast<const uint4*>(w1 ? w1 : w0);
  const uint4* px = reinterpret_cast<const uint4*>(xs);
  int v0 = 0;
  for (; v0 + 32 * U <= nvec; v0 += 32 * U) {  // full steps: unconditional loads
    uint4 a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) a[u] = ldg_stream(p0 + v0 + u * 32 + lane);
#pragma unroll
    for (int u = 0; u < U; ++u) b[u] = ldg_stream(p1 + v0 + u * 32 + lane);
    issue_fence();
#pragma unroll
    for (int u = 0; u < U; ++u)
      fma_vec2<T, BT>(a[u], b[u], px, nvec, v0 + u * 32 + lane, B, acc);
  }
  for (int v = v0 + lane; v < nvec; v += 32) {  // ragged tail
    const uint4 a = ldg_stream(p0 + v);
    const uint4 b = ldg_stream(p1 + v);
    fma_vec2<T, BT>(a, b, px, nvec, v, B, acc);
  }
}

}  // namespace cats
