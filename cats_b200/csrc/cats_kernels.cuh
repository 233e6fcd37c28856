// The streaming kernels of the CATS sparse-MLP decode path (sm_100a).
//
//   k_gate     stage 1: gate GEMV + SiLU + |v| > t + warp-ballot compaction (segmented list)
//   k_updown   stage 2 and/or stage 3 over a balanced share of the active list
//   k_compact  active list from a dense gate tensor (for the entry points that receive one)
//   k_export   flatten the segmented list into caller buffers
//   k_rows_gemv / k_transpose   dense helpers
//
// Data flow.  Stage 1 runs one CTA per *segment* (a contiguous range of neurons); a CTA leaves
// its active neurons, in ascending order, at seg_idx[row0(c) ...] with their count in
// seg_count[c].  Nothing is exchanged between CTAs and no atomic counter is involved, so the
// list is deterministic.  A consumer CTA scans the <= 1024 segment counts (a few hundred bytes
// out of L2), takes positions [c*n/G, (c+1)*n/G) of the concatenated list and maps each back to
// (segment, offset) by binary search: stages 2+3 are balanced over CTAs whatever the mask.
#pragma once

#include "cats_common.cuh"

namespace cats {

// ---------------------------------------------------------------------------------------------
// Stage 1
// ---------------------------------------------------------------------------------------------
template <typename T, int BT>
__global__ void __launch_bounds__(kThreads)
k_gate(const T* __restrict__ x, const T* __restrict__ Wg, WsPtrs ws, int B, int H, int I,
       float thr, T* __restrict__ gate_dense, uint8_t* __restrict__ flag_dense) {
  extern __shared__ float s_val[];  // [rows of this segment][BT] SiLU(Wg x)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nseg = gridDim.x, c = blockIdx.x;
  const int r0 = seg_row0(c, nseg, I), r1 = seg_row0(c + 1, nseg, I);
  const int R = r1 - r0;

  pdl_wait();
  pdl_launch_dependents();

  // two adjacent rows (one contiguous 2*H*sizeof(T) stream) per warp step
  for (int lr = warp * 2; lr < R; lr += kWarps * 2) {
    float acc[2][BT];
#pragma unroll
    for (int t = 0; t < BT; ++t) acc[0][t] = acc[1][t] = 0.f;
    const T* w0 = Wg + (size_t)(r0 + lr) * H;
    const T* w1 = (lr + 1 < R) ? w0 + H : nullptr;
    warp_dot2<T, BT, 8>(w0, w1, x, B, H, lane, acc);
#pragma unroll
    for (int t = 0; t < BT; ++t) {
      float a0 = warp_sum(acc[0][t]);
      float a1 = warp_sum(acc[1][t]);
      if (lane == 0) {
        s_val[lr * BT + t] = silu_f(a0);
        if (lr + 1 < R) s_val[(lr + 1) * BT + t] = silu_f(a1);
      }
    }
  }
  __syncthreads();

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
          const float s = s_val[lr * BT + t];
          const bool a = is_active(s, thr);
          if (gate_dense) gate_dense[(size_t)t * I + r0 + lr] = VecT<T>::from_f(s);
          if (flag_dense) flag_dense[(size_t)t * I + r0 + lr] = a ? 1 : 0;
          v[t] = a ? s : 0.f;
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
    if (lane == 0) {
      ws.seg_count[c] = base;
      if (c == 0) ws.hdr[HDR_NSEG] = nseg;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Inclusive scan of the segment counts into shared memory; returns the total.
// s_incl must hold kMaxSeg ints, s_part kWarps + 1 ints.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int scan_segments(const int* __restrict__ seg_count,
                                             const int* __restrict__ nseg_ptr, int* nseg_out,
                                             int* s_incl, int* s_part) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int PER = kMaxSeg / kThreads;  // 4 consecutive entries per thread
  // the counts are fetched before the segment count is known (one L2 round trip instead of
  // two); entries past nseg are stale and masked below
  int loc[PER];
  if (tid < kThreads) {
    const int4 c4 = __ldcg(reinterpret_cast<const int4*>(seg_count) + tid);
    loc[0] = c4.x; loc[1] = c4.y; loc[2] = c4.z; loc[3] = c4.w;
  } else {
    loc[0] = loc[1] = loc[2] = loc[3] = 0;
  }
  const int nseg = __ldcg(nseg_ptr);
  *nseg_out = nseg;
  int sum = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int s = tid * PER + i;
    if (s >= nseg) loc[i] = 0;
    sum += loc[i];
    loc[i] = sum;
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31 && warp < kWarps) s_part[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < kWarps) ? s_part[lane] : 0;
#pragma unroll
    for (int o = 1; o < kWarps; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    if (lane < kWarps) s_part[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  if (tid < kThreads) {
    const int warp_excl = (warp == 0) ? 0 : s_part[warp - 1];
    const int thread_excl = warp_excl + incl - sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) s_incl[tid * PER + i] = thread_excl + loc[i];
  }
  __syncthreads();
  return s_part[kWarps - 1];
}

// Position p of the concatenated list -> index into seg_idx / seg_gate.
__device__ __forceinline__ int locate(const int* s_incl, int nseg, int I, int p) {
  int lo = 0, hi = nseg - 1;  // smallest s with s_incl[s] > p
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (s_incl[mid] > p) hi = mid; else lo = mid + 1;
  }
  const int excl = (lo == 0) ? 0 : s_incl[lo - 1];
  return seg_row0(lo, nseg, I) + (p - excl);
}

// ---------------------------------------------------------------------------------------------
// Last-CTA epilogue of the split-K down projection: turn the fp32 accumulators into the result,
// optionally fused with the decoder layer's residual add and the next RMS norm, and leave the
// accumulators zero for the next call.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ void finalize_down(WsPtrs ws, int B, int H, T* __restrict__ out, int out_mode,
                              T* __restrict__ resid, T* __restrict__ x_next,
                              const T* __restrict__ norm_w, float eps, float* s_red) {
  // Any block size that is a whole number of warps, up to 32 warps (s_red[32]).  Every thread
  // first issues all of its accumulator / residual loads (one L2 round trip for the lot), then
  // stores; the new residual stays in registers for the norm when a token's share per thread
  // fits (KV groups of four elements), else it is read back.
  using V = VecT<T>;
  constexpr int KV = 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthr = blockDim.x, nwarp = nthr >> 5;
  const int ngrp = H >> 2;  // H is a multiple of 4
  const bool in_regs = ngrp <= KV * nthr;
  for (int b = 0; b < B; ++b) {
    float ss = 0.f;
    float keep[KV][4];
    for (int g0 = 0; g0 < ngrp; g0 += KV * nthr) {
      float4 a[KV];
      float r[KV][4];
#pragma unroll
      for (int j = 0; j < KV; ++j) {
        const int g = g0 + j * nthr + tid;
        a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < ngrp) {
          a[j] = __ldcg(reinterpret_cast<const float4*>(ws.acc32 + (size_t)b * H) + g);
          if (resid && out_mode != 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) r[j][i] = V::to_f(resid[(size_t)b * H + 4 * g + i]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < KV; ++j) {
        const int g = g0 + j * nthr + tid;
        if (g < ngrp) {
          const size_t e = (size_t)b * H + 4 * (size_t)g;
          reinterpret_cast<float4*>(ws.acc32 + (size_t)b * H)[g] = make_float4(0.f, 0.f, 0.f, 0.f);
          const float v[4] = {a[j].x, a[j].y, a[j].z, a[j].w};
          if (out_mode == 1) {
            float* o = reinterpret_cast<float*>(out) + e;
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] += v[i];
          } else {
            if (out) {
#pragma unroll
              for (int i = 0; i < 4; ++i) out[e + i] = V::from_f(v[i]);
            }
            if (resid) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const T rn = V::from_f(r[j][i] + v[i]);
                resid[e + i] = rn;
                const float rf = V::to_f(rn);
                keep[j][i] = rf;
                ss = fmaf(rf, rf, ss);
              }
            }
          }
        }
      }
    }
    if (resid && x_next && out_mode != 1) {
      ss = warp_sum(ss);
      __syncthreads();
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < nwarp; ++w) tot += s_red[w];
      const float rs = rsqrtf(tot / (float)H + eps);
      if (in_regs) {
#pragma unroll
        for (int j = 0; j < KV; ++j) {
          const int g = j * nthr + tid;
          if (g < ngrp) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              T y = V::from_f(keep[j][i] * rs);
              if (norm_w) y = V::from_f(V::to_f(norm_w[4 * g + i]) * V::to_f(y));
              x_next[(size_t)b * H + 4 * g + i] = y;
            }
          }
        }
      } else {
        for (int hcol = tid; hcol < H; hcol += nthr) {
          const size_t e = (size_t)b * H + hcol;
          T y = V::from_f(V::to_f(resid[e]) * rs);
          if (norm_w) y = V::from_f(V::to_f(norm_w[hcol]) * V::to_f(y));
          x_next[e] = y;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Stages 2 / 3 / 2+3.  MODE bit 0: do the up projection (input = segmented list of stage 1),
// bit 1: do the down projection.  MODE 1 leaves the flat list + h for a later MODE 2 launch.
// ---------------------------------------------------------------------------------------------
constexpr int kRU = 8;   // WdT rows in flight per thread and column group
constexpr int kCG = 2;   // 16-byte column groups per thread

template <typename T, int BT, int MODE>
__global__ void __launch_bounds__(kThreads)
k_updown(const T* __restrict__ x, const T* __restrict__ Wu, const T* __restrict__ WdT, WsPtrs ws,
         int B, int H, int I, int cap, T* __restrict__ out, int out_mode, T* __restrict__ resid,
         T* __restrict__ x_next, const T* __restrict__ norm_w, float eps,
         T* __restrict__ inter_dense) {
  using V = VecT<T>;
  constexpr int N = V::N;
  constexpr bool kUp = (MODE & 1) != 0, kDown = (MODE & 2) != 0;
  constexpr int DB = BT < 4 ? BT : 4;  // tokens accumulated per pass over the rows

  extern __shared__ int s_dyn[];
  int* s_idx = s_dyn;                                   // [cap + kRU]
  float* s_h = reinterpret_cast<float*>(s_dyn + cap + kRU);  // [(cap + kRU) * BT]
  __shared__ int s_incl[kUp ? kMaxSeg : 1];
  __shared__ int s_part[kWarps + 1];
  __shared__ float s_red[32];
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, c = blockIdx.x;
  const int nvec = H / N;

  pdl_wait();
  pdl_launch_dependents();

  int n, nseg = 1;
  if (kUp) {
    n = scan_segments(ws.seg_count, ws.hdr + HDR_NSEG, &nseg, s_incl, s_part);
    if (c == 0 && tid == 0) ws.hdr[HDR_NACTIVE] = n;
  } else {
    n = __ldcg(ws.hdr + HDR_NACTIVE);
  }
  const int p0 = (int)(((long long)c * n) / G), p1 = (int)(((long long)(c + 1) * n) / G);
  const int cnt = p1 - p0;  // <= cap by construction (cap >= ceil(I / G))

  for (int j = tid; j < cap + kRU; j += kThreads) {
    int idx = 0;
    float g[BT];
#pragma unroll
    for (int t = 0; t < BT; ++t) g[t] = 0.f;
    if (j < cnt) {
      if (kUp) {
        const int q = locate(s_incl, nseg, I, p0 + j);
        idx = __ldcg(ws.seg_idx + q);
#pragma unroll
        for (int t = 0; t < BT; ++t)
          if (t < B) g[t] = __ldcg(ws.seg_gate + (size_t)q * B + t);
      } else {
        idx = __ldcg(ws.flat_idx + p0 + j);
#pragma unroll
        for (int t = 0; t < BT; ++t)
          if (t < B) g[t] = __ldcg(ws.h + (size_t)(p0 + j) * B + t);
      }
    }
    s_idx[j] = idx;
#pragma unroll
    for (int t = 0; t < BT; ++t) s_h[j * BT + t] = g[t];
  }
  __syncthreads();

  if (kUp) {
    // h[j][b] = gate[j][b] * (Wu[idx_j, :] . x[b, :]); two gathered rows per warp step
    for (int j = warp * 2; j < cnt; j += kWarps * 2) {
      float acc[2][BT];
#pragma unroll
      for (int t = 0; t < BT; ++t) acc[0][t] = acc[1][t] = 0.f;
      const T* w0 = Wu + (size_t)s_idx[j] * H;
      const T* w1 = (j + 1 < cnt) ? Wu + (size_t)s_idx[j + 1] * H : nullptr;
      warp_dot2<T, BT, 8>(w0, w1, x, B, H, lane, acc);
#pragma unroll
      for (int t = 0; t < BT; ++t) {
        const float a0 = warp_sum(acc[0][t]);
        const float a1 = warp_sum(acc[1][t]);
        if (lane == 0) {
          s_h[j * BT + t] *= a0;
          if (j + 1 < cnt) s_h[(j + 1) * BT + t] *= a1;
        }
      }
    }
    __syncthreads();
    if (!kDown) {
      for (int j = tid; j < cnt; j += kThreads) {
        const int idx = s_idx[j];
        ws.flat_idx[p0 + j] = idx;
#pragma unroll
        for (int t = 0; t < BT; ++t)
          if (t < B) {
            const float hv = s_h[j * BT + t];
            ws.h[(size_t)(p0 + j) * B + t] = hv;
            if (inter_dense) inter_dense[(size_t)t * I + idx] = V::from_f(hv);
          }
      }
    }
  }

  if (kDown) {
    const uint4* wd = reinterpret_cast<const uint4*>(WdT);
    for (int b0 = 0; b0 < B; b0 += DB) {
      for (int cv0 = 0; cv0 < nvec; cv0 += kThreads * kCG) {
        float acc[kCG][N][DB];
#pragma unroll
        for (int g = 0; g < kCG; ++g)
#pragma unroll
          for (int i = 0; i < N; ++i)
#pragma unroll
            for (int d = 0; d < DB; ++d) acc[g][i][d] = 0.f;
        for (int j0 = 0; j0 < cnt; j0 += kRU) {
          uint4 wv[kRU][kCG];
#pragma unroll
          for (int r = 0; r < kRU; ++r) {
            const bool rok = (j0 + r < cnt);
            const uint4* rowp = wd + (size_t)s_idx[j0 + r] * nvec;
#pragma unroll
            for (int g = 0; g < kCG; ++g) {
              const int v = cv0 + g * kThreads + tid;
              wv[r][g] = (rok && v < nvec) ? ldg_stream(rowp + v) : make_uint4(0, 0, 0, 0);
            }
          }
          issue_fence();
#pragma unroll
          for (int r = 0; r < kRU; ++r) {
            float hb[DB];
#pragma unroll
            for (int d = 0; d < DB; ++d) hb[d] = s_h[(j0 + r) * BT + b0 + d];
#pragma unroll
            for (int g = 0; g < kCG; ++g) {
              float wf[N];
              V::unpack(wv[r][g], wf);
#pragma unroll
              for (int i = 0; i < N; ++i)
#pragma unroll
                for (int d = 0; d < DB; ++d) acc[g][i][d] = fmaf(hb[d], wf[i], acc[g][i][d]);
            }
          }
        }
        if (cnt > 0) {
#pragma unroll
          for (int g = 0; g < kCG; ++g) {
            const int v = cv0 + g * kThreads + tid;
            if (v < nvec) {
#pragma unroll
              for (int d = 0; d < DB; ++d) {
                if (b0 + d < B) {
                  float* dst = ws.acc32 + (size_t)(b0 + d) * H + (size_t)v * N;
#pragma unroll
                  for (int i = 0; i < N; i += 4)
                    red_add_v4(dst + i, acc[g][i][d], acc[g][i + 1][d], acc[g][i + 2][d],
                               acc[g][i + 3][d]);
                }
              }
            }
          }
        }
      }
    }

    // completion ticket: the CTA that arrives last owns the epilogue
    __threadfence();
    __syncthreads();
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
}

// ---------------------------------------------------------------------------------------------
// Active list from a dense gate tensor (single CTA, 1024 threads, ordered).
// Writes the list both as one segment (input of a later stage 2) and as the flat list with
// h = values (input of a later stage 3).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024)
k_compact(const T* __restrict__ values, const uint8_t* __restrict__ flags, WsPtrs ws, int B,
          int I, float thr) {
  using V = VecT<T>;
  __shared__ int s_wcnt[32];
  __shared__ int s_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int i0 = 0; i0 < I; i0 += 1024) {
    const int i = i0 + tid;
    bool any = false;
    if (i < I) {
      for (int t = 0; t < B; ++t) {
        const size_t e = (size_t)t * I + i;
        any |= flags ? (flags[e] != 0) : is_active(V::to_f(values[e]), thr);
      }
    }
    const unsigned m = __ballot_sync(0xffffffffu, any);
    if (lane == 0) s_wcnt[warp] = __popc(m);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int w = 0; w < 32; ++w) {
      const int cw = s_wcnt[w];
      if (w < warp) woff += cw;
      tot += cw;
    }
    const int base = s_base;
    if (any) {
      const int pos = base + woff + __popc(m & ((1u << lane) - 1u));
      ws.seg_idx[pos] = i;
      ws.flat_idx[pos] = i;
      for (int t = 0; t < B; ++t) {
        const size_t e = (size_t)t * I + i;
        const bool a = flags ? (flags[e] != 0) : is_active(V::to_f(values[e]), thr);
        const float v = a ? V::to_f(values[e]) : 0.f;
        ws.seg_gate[(size_t)pos * B + t] = v;
        ws.h[(size_t)pos * B + t] = v;
      }
    }
    __syncthreads();
    if (tid == 0) s_base = base + tot;
    __syncthreads();
  }
  if (tid == 0) {
    ws.seg_count[0] = s_base;
    ws.hdr[HDR_NSEG] = 1;
    ws.hdr[HDR_NACTIVE] = s_base;
  }
}

// Flatten the segmented list: idx_out int64[n], val_out T[n] (token 0's gate value).
template <typename T>
__global__ void __launch_bounds__(kThreads)
k_export(WsPtrs ws, int B, int I, long long* __restrict__ idx_out, T* __restrict__ val_out) {
  __shared__ int s_incl[kMaxSeg];
  __shared__ int s_part[kWarps + 1];
  pdl_wait();
  int nseg;
  const int n = scan_segments(ws.seg_count, ws.hdr + HDR_NSEG, &nseg, s_incl, s_part);
  if (blockIdx.x == 0 && threadIdx.x == 0) ws.hdr[HDR_NACTIVE] = n;
  for (int p = blockIdx.x * kThreads + threadIdx.x; p < n; p += gridDim.x * kThreads) {
    const int q = locate(s_incl, nseg, I, p);
    if (idx_out) idx_out[p] = __ldcg(ws.seg_idx + q);
    if (val_out) val_out[p] = VecT<T>::from_f(__ldcg(ws.seg_gate + (size_t)q * B));
  }
}

// ---------------------------------------------------------------------------------------------
// Dense helpers
// ---------------------------------------------------------------------------------------------
// out[b, r] = W[r, :] . xs[b, :] for a [R, K] row-major matrix, one warp per pair of rows.
template <typename T, int BT>
__global__ void __launch_bounds__(kThreads)
k_rows_gemv(const T* __restrict__ xs, const T* __restrict__ W, int B, int K, int R,
            T* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  for (int r = (blockIdx.x * kWarps + warp) * 2; r < R; r += gridDim.x * kWarps * 2) {
    float acc[2][BT];
#pragma unroll
    for (int t = 0; t < BT; ++t) acc[0][t] = acc[1][t] = 0.f;
    const T* w0 = W + (size_t)r * K;
    const T* w1 = (r + 1 < R) ? w0 + K : nullptr;
    warp_dot2<T, BT, 8>(w0, w1, xs, B, K, lane, acc);
#pragma unroll
    for (int t = 0; t < BT; ++t) {
      const float a0 = warp_sum(acc[0][t]);
      const float a1 = warp_sum(acc[1][t]);
      if (lane == 0 && t < B) {
        out[(size_t)t * R + r] = VecT<T>::from_f(a0);
        if (r + 1 < R) out[(size_t)t * R + r + 1] = VecT<T>::from_f(a1);
      }
    }
  }
}

// Decoder-layer tail on its own (one CTA per token): resid += y; x_next = rmsnorm(resid) * w.
// Used when the MLP output has to pass through an all-reduce before the residual add.
template <typename T>
__global__ void __launch_bounds__(kThreads)
k_tail(const T* __restrict__ y, T* __restrict__ resid, T* __restrict__ x_next,
       const T* __restrict__ norm_w, float eps, int H) {
  using V = VecT<T>;
  __shared__ float s_red[kWarps];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t base = (size_t)blockIdx.x * H;
  pdl_wait();
  pdl_launch_dependents();
  float ss = 0.f;
  for (int hcol = tid; hcol < H; hcol += kThreads) {
    const T r = V::from_f(V::to_f(resid[base + hcol]) + V::to_f(y[base + hcol]));
    resid[base + hcol] = r;
    const float rf = V::to_f(r);
    ss = fmaf(rf, rf, ss);
  }
  if (!x_next) return;
  ss = warp_sum(ss);
  if (lane == 0) s_red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) tot += s_red[w];
  const float rs = rsqrtf(tot / (float)H + eps);
  for (int hcol = tid; hcol < H; hcol += kThreads) {
    T v = V::from_f(V::to_f(resid[base + hcol]) * rs);
    if (norm_w) v = V::from_f(V::to_f(norm_w[hcol]) * V::to_f(v));
    x_next[base + hcol] = v;
  }
}

// dst[c, r] = src[r, c]; E = element type of the same size (uint16_t / uint32_t)
template <typename E>
__global__ void k_transpose(const E* __restrict__ src, E* __restrict__ dst, int rows, int cols) {
  __shared__ E tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, cc = bx + threadIdx.x;
    if (r < rows && cc < cols) tile[j][threadIdx.x] = src[(size_t)r * cols + cc];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int cc = bx + j, r = by + threadIdx.x;
    if (r < rows && cc < cols) dst[(size_t)cc * rows + r] = tile[threadIdx.x][j];
  }
}

// ---------------------------------------------------------------------------------------------
// Decode-step glue between the fused QKV projection and attention: rotate-half RoPE on the query
// and key heads of ONE new position per sequence, and the write of the rotated keys and the
// values into the static KV cache at that position - what HF's apply_rotary_pos_emb plus the
// cache update do in a dozen elementwise launches.  Arithmetic in the storage type with a rounding
// after every operation (q * cos, rotate_half(q) * sin, their sum), as those launches round.
//   qkv   [B, (nh + 2 * nkv) * hd]   q heads, then k heads, then v heads
//   cos, sin [max_len, hd] (the two halves of a row are equal); *pos = the position
//   q_out [B, nh, hd];  kc, vc [B, nkv, max_len, hd]
// One warp per (sequence, head); hd a multiple of 64, at most 256.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
k_rope_cache(const T* __restrict__ qkv, const T* __restrict__ cosv, const T* __restrict__ sinv,
             const long long* __restrict__ pos_ptr, T* __restrict__ q_out, T* __restrict__ kc,
             T* __restrict__ vc, int B, int nh, int nkv, int hd, int max_len) {
  using V = VecT<T>;
  const int warp = (blockIdx.x * kThreads + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int heads = nh + 2 * nkv;
  if (warp >= B * heads) return;
  const int b = warp / heads, h = warp - b * heads;
  const long long pos = *pos_ptr;
  if (pos < 0 || pos >= max_len) return;
  const T* src = qkv + ((size_t)b * heads + h) * hd;
  const int half = hd >> 1;
  if (h >= nh + nkv) {                                   // value head: copy
    T* dst = vc + (((size_t)b * nkv + (h - nh - nkv)) * max_len + pos) * hd;
    for (int i = lane; i < hd; i += 32) dst[i] = src[i];
    return;
  }
  T* dst = (h < nh) ? q_out + ((size_t)b * nh + h) * hd
                    : kc + (((size_t)b * nkv + (h - nh)) * max_len + pos) * hd;
  const T* c = cosv + (size_t)pos * hd;
  const T* s = sinv + (size_t)pos * hd;
  for (int i = lane; i < half; i += 32) {
    const float x1 = V::to_f(src[i]), x2 = V::to_f(src[i + half]);
    // rounded to T after each operation, as the separate launches of the eager path round
    const float a1 = V::to_f(V::from_f(x1 * V::to_f(c[i])));
    const float b1 = V::to_f(V::from_f(-x2 * V::to_f(s[i])));
    const float a2 = V::to_f(V::from_f(x2 * V::to_f(c[i + half])));
    const float b2 = V::to_f(V::from_f(x1 * V::to_f(s[i + half])));
    dst[i] = V::from_f(a1 + b1);
    dst[i + half] = V::from_f(a2 + b2);
  }
}

}  // namespace cats
