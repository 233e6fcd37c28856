// Activation statistics on the device: the two histograms the reference collects per MLP
// (experiments/models/sparse_silu/ugly_utils.py:514-522, `torch.histogram` of the gate
// pre-activations and of |post-activations| over 999 bins with edges -inf, linspace(-1, 1, 998),
// +inf, :491-493) and the threshold read off the histogram (`get_threshold`, :236-245).
// The reference copies both activation tensors to the host on every forward for this.
#pragma once

#include "cats_common.cuh"

namespace cats {

constexpr int kHistMaxEdges = 1024;

// Bin of x for ascending edges e[0..n): the b with e[b] <= x < e[b+1], the last bin closed on
// the right (torch.histogram's rule); -1 when x is outside [e[0], e[n-1]] or NaN.
// Exact path: start from a guess and compare with the edge values themselves.
__device__ __forceinline__ int hist_bin_exact(float x, const float* e, int n, int guess) {
  if (!(x >= e[0]) || !(x <= e[n - 1])) return -1;
  int b = min(max(guess, 0), n - 2);
  while (b > 0 && x < e[b]) --b;
  while (b < n - 2 && x >= e[b + 1]) ++b;
  return b;
}
// The finite edges e[ff..lf] described as a line (cell index g = x * inv + c0): when both outer
// edges are infinite (the reference's edges), everything below the line is bin ff - 1 and
// everything above it bin lf, so g is clamped to [-0.5, cells + 0.5] and treated like any other
// cell.  Where g falls well inside a cell the bin follows from arithmetic alone (full-rate adds
// and integer ops, no conversion instructions); within kHistSlack cells of a boundary, and for
// NaNs, the exact path decides.  The kernel verifies that every finite edge sits within a
// quarter of the slack of the line and otherwise (or when an outer edge is finite) sets
// inv = 0, which sends every value down the exact path; the rounding error of g (a few ulps of
// ~1000 cells, 1e-4) is well inside the rest of the slack.
constexpr float kHistSlack = 1.0f / 1024;
struct HistLine {
  float inv, c0, hi;  // g = x * inv + c0, clamped to [-0.5, hi]
  int base;           // first finite edge's index, minus the mantissa offset of the rounding trick
  int ff, n;
};
__device__ __forceinline__ int hist_bin(float x, const float* e, const HistLine& L) {
  const float g = fminf(fmaxf(fmaf(x, L.inv, L.c0), -0.5f), L.hi);
  // Adding 1.5 * 2^23 rounds g - 0.5 to an integer (= floor(g) away from the cell boundaries)
  // and leaves it, offset by 2^22, in the mantissa: valid for |g| < 2^22, negative values
  // included (with 2^23 as the constant a sum below 2^23 would have half-integer spacing and
  // garbage mantissa bits).
  const float kMagic = 12582912.f;
  const float gm = (g - 0.5f) + kMagic;
  int b = (__float_as_int(gm) & 0x7fffff) + L.base;
  const float fr = g - (gm - kMagic);  // position inside the cell, 0.5 = the middle
  const bool ok = fabsf(fr - 0.5f) < 0.5f - kHistSlack && x == x && L.inv > 0.f;
  if (!ok) b = hist_bin_exact(x, e, L.n, L.ff + (int)fmaxf(g, 0.f));
  return b;
}

// fp32 values of the 8 (16-bit types) or 4 (fp32) elements of a 16-byte vector, |.| taken on the
// packed words when asked; fp16 is widened on the FMA pipe (x * 1 + 0 as a mixed-precision FMA),
// bf16 by a shift: the conversion instructions proper run at a fraction of that rate.
template <typename T>
__device__ __forceinline__ void hist_unpack(uint4 q, float* f, bool take_abs);
template <>
__device__ __forceinline__ void hist_unpack<float>(uint4 q, float* f, bool take_abs) {
  const uint32_t m = take_abs ? 0x7fffffffu : 0xffffffffu;
  f[0] = __uint_as_float(q.x & m);
  f[1] = __uint_as_float(q.y & m);
  f[2] = __uint_as_float(q.z & m);
  f[3] = __uint_as_float(q.w & m);
}
template <>
__device__ __forceinline__ void hist_unpack<__half>(uint4 q, float* f, bool take_abs) {
  const uint32_t m = take_abs ? 0x7fff7fffu : 0xffffffffu;
  const uint32_t w[4] = {q.x & m, q.y & m, q.z & m, q.w & m};
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm("{\n\t.reg .b16 lo, hi, one;\n\tmov.b32 {lo, hi}, %2;\n\tmov.b16 one, 0x3C00;\n\t"
        "fma.rn.f32.f16 %0, lo, one, 0f00000000;\n\tfma.rn.f32.f16 %1, hi, one, 0f00000000;\n\t}"
        : "=f"(f[2 * i]), "=f"(f[2 * i + 1])
        : "r"(w[i]));
}
template <>
__device__ __forceinline__ void hist_unpack<__nv_bfloat16>(uint4 q, float* f, bool take_abs) {
  const uint32_t m = take_abs ? 0x7fff7fffu : 0xffffffffu;
  const uint32_t w[4] = {q.x & m, q.y & m, q.z & m, q.w & m};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// counts[b] += number of values in bin b.  HBM-bound stream over `n` values (16-byte loads,
// grid-stride).  Shared memory holds 32 copies of the histogram, copy l used by lane l of every
// warp and laid out so that copy l lives in bank l: a warp's 32 increments never meet in a bank
// or at an address whatever the values are (with one copy per warp, bank conflicts between
// random bins and the crowded end bins made the shared-memory atomics 5x slower than the
// stream).  The copies are merged into the global 64-bit counters at the end.
// take_abs: bin |v| (the post-activation histogram).  Dynamic shared memory:
// hist_smem_bytes(n_edges).
constexpr int kHistThreads = 1024;
__host__ __device__ inline size_t hist_smem_bytes(int n_edges) {
  return sizeof(float) * kHistMaxEdges + sizeof(unsigned) * 32 * (size_t)(n_edges - 1);
}
template <typename T>
__global__ void __launch_bounds__(kHistThreads, 1)
k_histogram(const T* __restrict__ v, size_t n, const float* __restrict__ edges, int n_edges,
            unsigned long long* __restrict__ counts, int take_abs) {
  using V = VecT<T>;
  constexpr int N = V::N;
  extern __shared__ __align__(16) unsigned char hist_smem[];
  float* s_e = reinterpret_cast<float*>(hist_smem);
  unsigned* s_h = reinterpret_cast<unsigned*>(hist_smem + sizeof(float) * kHistMaxEdges);  // [bin][lane]
  const int tid = threadIdx.x, lane = tid & 31;
  const int nb = n_edges - 1;
  for (int i = tid; i < n_edges; i += blockDim.x) s_e[i] = edges[i];
  for (int i = tid; i < 32 * nb; i += blockDim.x) s_h[i] = 0u;
  __syncthreads();
  int ff = 0, lf = n_edges - 1;
  while (ff < lf && isinf(s_e[ff])) ++ff;
  while (lf > ff && isinf(s_e[lf])) --lf;
  HistLine L;
  L.inv = (lf > ff && s_e[lf] > s_e[ff]) ? (float)(lf - ff) / (s_e[lf] - s_e[ff]) : 0.f;
  L.c0 = -s_e[ff] * L.inv;
  L.hi = (float)(lf - ff) + 0.5f;
  L.base = ff - 0x400000;
  L.ff = ff;
  L.n = n_edges;
  // the arithmetic shortcut needs infinite outer edges right next to the finite ones and every
  // finite edge where the line puts it; every thread checks a few edges, the CTA votes
  {
    int bad = !(ff == 1 && isinf(s_e[0]) && lf == n_edges - 2 && isinf(s_e[n_edges - 1])) ||
              lf - ff >= (1 << 21);  // the rounding trick of hist_bin needs |g| < 2^22
    for (int i = ff + tid; i <= lf; i += blockDim.x) {
      const float g = fmaf(s_e[i], L.inv, L.c0);
      if (!(fabsf(g - (float)(i - ff)) < kHistSlack * 0.25f)) bad = 1;
    }
    if (__syncthreads_or(bad)) L.inv = 0.f;
  }
  unsigned* h = s_h + lane;

  auto put = [&](float x) {  // x already has |.| applied
    const int b = hist_bin(x, s_e, L);
    // (clamped: no arithmetic slip may ever turn into a write outside the histogram)
    if (b >= 0) atomicAdd(h + 32 * min(b, nb - 1), 1u);  // other warps' lane `lane` share this copy
  };
  auto put1 = [&](T t) {
    const float x = V::to_f(t);
    put(take_abs ? fabsf(x) : x);
  };
  // head up to the first 16-byte boundary, vectors, tail
  const uintptr_t addr = reinterpret_cast<uintptr_t>(v);
  size_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
  if (head > n) head = n;
  const size_t nvec = (n - head) / N;
  const size_t gtid = blockIdx.x * (size_t)blockDim.x + tid, gsz = (size_t)gridDim.x * blockDim.x;
  for (size_t i = gtid; i < head; i += gsz) put1(v[i]);
  const uint4* vv = reinterpret_cast<const uint4*>(v + head);
  size_t i = gtid;
  for (; i + gsz < nvec; i += 2 * gsz) {  // two loads in flight per thread
    const uint4 q0 = ldg_stream(vv + i), q1 = ldg_stream(vv + i + gsz);
    float f[N];
    hist_unpack<T>(q0, f, take_abs != 0);
#pragma unroll
    for (int k = 0; k < N; ++k) put(f[k]);
    hist_unpack<T>(q1, f, take_abs != 0);
#pragma unroll
    for (int k = 0; k < N; ++k) put(f[k]);
  }
  for (; i < nvec; i += gsz) {
    const uint4 q = ldg_stream(vv + i);
    float f[N];
    hist_unpack<T>(q, f, take_abs != 0);
#pragma unroll
    for (int k = 0; k < N; ++k) put(f[k]);
  }
  for (size_t j = head + nvec * N + gtid; j < n; j += gsz) put1(v[j]);
  __syncthreads();
  // merge: a warp per bin, lane l reads copy l
  for (int b = tid >> 5; b < nb; b += blockDim.x >> 5) {
    unsigned long long t = s_h[32 * b + lane];
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0 && t) atomicAdd(counts + b, t);
  }
}

// threshold = edges[first b with cdf_b > sparsity], cdf = running sum of counts / total, as
// `get_threshold` computes it on the host: float32 probabilities, a running sum kept in double
// and rounded to float32 per element (torch's CPU cumsum), compared with float32(sparsity);
// b = n_bins (the last edge) when the CDF never exceeds it.  One warp; 999 bins.
__global__ void k_hist_threshold(const unsigned long long* __restrict__ counts,
                                 const float* __restrict__ edges, int n_edges, float sparsity,
                                 float* __restrict__ threshold) {
  __shared__ float s_p[kHistMaxEdges];
  __shared__ float s_total;
  const int nb = n_edges - 1, lane = threadIdx.x;
  unsigned long long t = 0;
  for (int b = lane; b < nb; b += 32) t += counts[b];
  for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  if (lane == 0) s_total = (float)t;
  __syncwarp();
  for (int b = lane; b < nb; b += 32) s_p[b] = (float)counts[b] / s_total;
  __syncwarp();
  if (lane == 0) {
    double run = 0.0;
    int idx = nb;
    for (int b = 0; b < nb; ++b) {
      run += (double)s_p[b];
      if ((float)run > sparsity) {
        idx = b;
        break;
      }
    }
    *threshold = edges[idx];
  }
}

}  // namespace cats
