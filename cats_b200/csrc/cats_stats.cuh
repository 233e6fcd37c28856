// Activation statistics on the device: the two histograms the reference collects per MLP
// (experiments/models/sparse_silu/ugly_utils.py:514-522, `torch.histogram` of the gate
// pre-activations and of |post-activations| over 999 bins with edges -inf, linspace(-1, 1, 998),
// +inf, :491-493) and the threshold read off the histogram (`get_threshold`, :236-245).
// The reference copies both activation tensors to the host on every forward for this.
#pragma once

#include "cats_common.cuh"

namespace cats {

constexpr int kHistMaxEdges = 1024;
constexpr int kHistWarps = 8;  // one private histogram per warp: fewer same-address conflicts

// Bin of x for ascending edges e[0..n): the b with e[b] <= x < e[b+1], the last bin closed on
// the right (torch.histogram's rule); -1 when x is outside [e[0], e[n-1]] or NaN.  `lo`/`inv`
// describe the finite inner edges as a line so that the search starts next to the answer; the
// answer itself is always decided by comparisons with the exact edge values.
__device__ __forceinline__ int hist_bin(float x, const float* e, int n, float lo, float inv,
                                        int first_finite, int last_finite) {
  if (!(x >= e[0]) || !(x <= e[n - 1])) return -1;
  float g = (x - lo) * inv;  // position among the finite edges
  g = fminf(fmaxf(g, 0.f), (float)(last_finite - first_finite));
  int b = first_finite + (int)g;
  b = min(max(b, 0), n - 2);
  while (b > 0 && x < e[b]) --b;
  while (b < n - 2 && x >= e[b + 1]) ++b;
  return b;
}

// counts[b] += number of values in bin b.  HBM-bound stream over `n` values (16-byte loads,
// grid-stride); per-warp histograms in shared memory, merged into the global 64-bit counters at
// the end.  take_abs: bin |v| (the post-activation histogram).
template <typename T>
__global__ void __launch_bounds__(kHistWarps * 32)
k_histogram(const T* __restrict__ v, size_t n, const float* __restrict__ edges, int n_edges,
            unsigned long long* __restrict__ counts, int take_abs) {
  using V = VecT<T>;
  constexpr int N = V::N;
  __shared__ float s_e[kHistMaxEdges];
  __shared__ unsigned s_h[kHistWarps][kHistMaxEdges];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int nb = n_edges - 1;
  for (int i = tid; i < n_edges; i += blockDim.x) s_e[i] = edges[i];
  for (int i = tid; i < kHistWarps * kHistMaxEdges; i += blockDim.x) (&s_h[0][0])[i] = 0u;
  __syncthreads();
  int ff = 0, lf = n_edges - 1;
  while (ff < lf && isinf(s_e[ff])) ++ff;
  while (lf > ff && isinf(s_e[lf])) --lf;
  const float lo = s_e[ff];
  const float inv = (lf > ff && s_e[lf] > lo) ? (float)(lf - ff) / (s_e[lf] - lo) : 0.f;
  unsigned* h = s_h[warp];

  auto put = [&](float x) {
    if (take_abs) x = fabsf(x);
    const int b = hist_bin(x, s_e, n_edges, lo, inv, ff, lf);
    if (b >= 0) atomicAdd(h + b, 1u);
  };
  // head up to the first 16-byte boundary, vectors, tail
  const uintptr_t addr = reinterpret_cast<uintptr_t>(v);
  size_t head = ((16 - (addr & 15)) & 15) / sizeof(T);
  if (head > n) head = n;
  const size_t nvec = (n - head) / N;
  const size_t gtid = blockIdx.x * (size_t)blockDim.x + tid, gsz = (size_t)gridDim.x * blockDim.x;
  for (size_t i = gtid; i < head; i += gsz) put(V::to_f(v[i]));
  const uint4* vv = reinterpret_cast<const uint4*>(v + head);
  for (size_t i = gtid; i < nvec; i += gsz) {
    const uint4 q = ldg_stream(vv + i);
    float f[N];
    V::unpack(q, f);
#pragma unroll
    for (int k = 0; k < N; ++k) put(f[k]);
  }
  for (size_t i = head + nvec * N + gtid; i < n; i += gsz) put(V::to_f(v[i]));
  __syncthreads();
  for (int b = tid; b < nb; b += blockDim.x) {
    unsigned long long t = 0;
#pragma unroll
    for (int w = 0; w < kHistWarps; ++w) t += s_h[w][b];
    if (t) atomicAdd(counts + b, t);
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
