// The stage kernels (direct-load and TMA-fed) instantiated for ONE element type; compiled once
// per type with -DCATS_ELEM_ID=0|1|2 (float, __half, __nv_bfloat16).
#include "cats_run.cuh"

namespace cats {
namespace {

template <typename T, int BT>
cudaError_t run_gate(const void* x, const void* Wg, WsPtrs ws, int B, int H, int I, float thr,
                     void* gate_dense, uint8_t* flag_dense, cudaStream_t st) {
  const int nseg = gate_segments(I);
  const int rmax = (I + nseg - 1) / nseg;
  const size_t smem = sizeof(float) * (size_t)rmax * BT;
  return launch(k_gate<T, BT>, dim3(nseg), dim3(kThreads), smem, st, (const T*)x, (const T*)Wg,
                ws, B, H, I, thr, (T*)gate_dense, flag_dense);
}

template <typename T, int BT, int MODE>
cudaError_t run_updown_mode(const void* x, const void* Wu, const void* WdT, WsPtrs ws, int B,
                            int H, int I, void* out, int out_mode, void* resid, void* x_next,
                            const void* norm_w, float eps, void* inter_dense, cudaStream_t st) {
  const int G = updown_ctas(I);
  const int cap = (I + G - 1) / G;
  const size_t smem = (size_t)(cap + kRU) * (sizeof(int) + sizeof(float) * BT);
  return launch(k_updown<T, BT, MODE>, dim3(G), dim3(kThreads), smem, st, (const T*)x,
                (const T*)Wu, (const T*)WdT, ws, B, H, I, cap, (T*)out, out_mode, (T*)resid,
                (T*)x_next, (const T*)norm_w, eps, (T*)inter_dense);
}

template <typename T, int BT>
cudaError_t run_updown(int mode, const void* x, const void* Wu, const void* WdT, WsPtrs ws, int B,
                       int H, int I, void* out, int out_mode, void* resid, void* x_next,
                       const void* norm_w, float eps, void* inter_dense, cudaStream_t st) {
  if (mode == 1)
    return run_updown_mode<T, BT, 1>(x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w,
                                     eps, inter_dense, st);
  if (mode == 2)
    return run_updown_mode<T, BT, 2>(x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w,
                                     eps, inter_dense, st);
  return run_updown_mode<T, BT, 3>(x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w,
                                   eps, inter_dense, st);
}

template <typename T, int BT>
cudaError_t run_rows_gemv(const void* xs, const void* W, int B, int K, int R, void* out,
                          cudaStream_t st) {
  int g = dev_info().sms * 4;
  const int need = (R + kWarps * 2 - 1) / (kWarps * 2);
  if (g > need) g = need;
  return launch(k_rows_gemv<T, BT>, dim3(g), dim3(kThreads), 0, st, (const T*)xs, (const T*)W, B,
                K, R, (T*)out);
}

template <typename T, int BT, int SR, bool XS>
cudaError_t run_gate_tma_v(const TmaPlan& p, const void* x, const void* Wg, WsPtrs ws, int B,
                           int H, int I, float thr, void* gate_dense, uint8_t* flag_dense,
                           cudaStream_t st) {
  return launch(k_gate_tma<T, BT, SR, XS>, dim3(p.grid), dim3(kConsumerThreads + 32 * p.pw), p.smem, st,
                (const T*)x, (const T*)Wg, ws, B, H, I, thr, (T*)gate_dense, flag_dense, p.S,
                p.cw, p.rmax, p.wait_kc, (const T*)p.pf_base, p.pf_n);
}

template <typename T, int BT>
cudaError_t run_gate_tma(const TmaPlan& p, const void* x, const void* Wg, WsPtrs ws, int B, int H,
                         int I, float thr, void* gate_dense, uint8_t* flag_dense, cudaStream_t st) {
  if (p.sr == 2) {
    if (p.xs) return run_gate_tma_v<T, BT, 2, true>(p, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
    return run_gate_tma_v<T, BT, 2, false>(p, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
  }
  if (p.xs) return run_gate_tma_v<T, BT, 1, true>(p, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
  return run_gate_tma_v<T, BT, 1, false>(p, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st);
}

template <typename T, int BT, int NVT>
cudaError_t run_updown_tma_nvt(const TmaPlan& p, const void* x, const void* Wu, const void* WdT,
                               WsPtrs ws, int B, int H, int I, void* out, int out_mode,
                               void* resid, void* x_next, const void* norm_w, float eps,
                               cudaStream_t st) {
  if (p.xs)
    return launch(k_updown_tma<T, BT, NVT, true>, dim3(p.grid), dim3(kConsumerThreads + 32 * p.pw), p.smem, st,
                  (const T*)x, (const T*)Wu, (const T*)WdT, ws, B, H, I, p.cap, (T*)out, out_mode,
                  (T*)resid, (T*)x_next, (const T*)norm_w, eps, p.S, p.cw, p.wait_kc);
  return launch(k_updown_tma<T, BT, NVT, false>, dim3(p.grid), dim3(kConsumerThreads + 32 * p.pw), p.smem, st,
                (const T*)x, (const T*)Wu, (const T*)WdT, ws, B, H, I, p.cap, (T*)out, out_mode,
                (T*)resid, (T*)x_next, (const T*)norm_w, eps, p.S, p.cw, p.wait_kc);
}

template <typename T, int BT>
cudaError_t run_updown_tma(const TmaPlan& p, const void* x, const void* Wu, const void* WdT,
                           WsPtrs ws, int B, int H, int I, void* out, int out_mode, void* resid,
                           void* x_next, const void* norm_w, float eps, cudaStream_t st) {
  switch (p.nvt) {
    case 1: return run_updown_tma_nvt<T, BT, 1>(p, x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w, eps, st);
    case 2: return run_updown_tma_nvt<T, BT, 2>(p, x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w, eps, st);
    case 4: return run_updown_tma_nvt<T, BT, 4>(p, x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w, eps, st);
    default: return run_updown_tma_nvt<T, BT, 8>(p, x, Wu, WdT, ws, B, H, I, out, out_mode, resid, x_next, norm_w, eps, st);
  }
}

}  // namespace

#define CATS_BT_SWITCH(BT_, FN, ...)              \
  switch (BT_) {                                  \
    case 1: return FN<T, 1>(__VA_ARGS__);         \
    case 2: return FN<T, 2>(__VA_ARGS__);         \
    case 4: return FN<T, 4>(__VA_ARGS__);         \
    case 8: return FN<T, 8>(__VA_ARGS__);         \
    default: return FN<T, 16>(__VA_ARGS__);       \
  }
#define CATS_BT_SWITCH_TMA(BT_, FN, ...)          \
  switch (BT_) {                                  \
    case 1: return FN<T, 1>(__VA_ARGS__);         \
    case 2: return FN<T, 2>(__VA_ARGS__);         \
    default: return FN<T, 4>(__VA_ARGS__);        \
  }

template <typename T>
cudaError_t inst_gate(const void* x, const void* Wg, WsPtrs ws, int B, int H, int I, float thr,
                      void* gate_dense, uint8_t* flag_dense, cudaStream_t st) {
  CATS_BT_SWITCH(batch_tile(B), run_gate, x, Wg, ws, B, H, I, thr, gate_dense, flag_dense, st)
}
template <typename T>
cudaError_t inst_updown(int mode, const void* x, const void* Wu, const void* WdT, WsPtrs ws, int B,
                        int H, int I, void* out, int out_mode, void* resid, void* x_next,
                        const void* norm_w, float eps, void* inter_dense, cudaStream_t st) {
  CATS_BT_SWITCH(batch_tile(B), run_updown, mode, x, Wu, WdT, ws, B, H, I, out, out_mode, resid,
                 x_next, norm_w, eps, inter_dense, st)
}
template <typename T>
cudaError_t inst_rows_gemv(const void* xs, const void* W, int B, int K, int R, void* out,
                           cudaStream_t st) {
  CATS_BT_SWITCH(batch_tile(B), run_rows_gemv, xs, W, B, K, R, out, st)
}
template <typename T>
cudaError_t inst_gate_tma(const TmaPlan& p, const void* x, const void* Wg, WsPtrs ws, int B, int H,
                          int I, float thr, void* gate_dense, uint8_t* flag_dense,
                          cudaStream_t st) {
  CATS_BT_SWITCH_TMA(batch_tile(B), run_gate_tma, p, x, Wg, ws, B, H, I, thr, gate_dense,
                     flag_dense, st)
}
template <typename T>
cudaError_t inst_updown_tma(const TmaPlan& p, const void* x, const void* Wu, const void* WdT,
                            WsPtrs ws, int B, int H, int I, void* out, int out_mode, void* resid,
                            void* x_next, const void* norm_w, float eps, cudaStream_t st) {
  CATS_BT_SWITCH_TMA(batch_tile(B), run_updown_tma, p, x, Wu, WdT, ws, B, H, I, out, out_mode,
                     resid, x_next, norm_w, eps, st)
}

template cudaError_t inst_gate<InstElem>(const void*, const void*, WsPtrs, int, int, int, float,
                                         void*, uint8_t*, cudaStream_t);
template cudaError_t inst_updown<InstElem>(int, const void*, const void*, const void*, WsPtrs, int,
                                           int, int, void*, int, void*, void*, const void*, float,
                                           void*, cudaStream_t);
template cudaError_t inst_rows_gemv<InstElem>(const void*, const void*, int, int, int, void*,
                                              cudaStream_t);
template cudaError_t inst_gate_tma<InstElem>(const TmaPlan&, const void*, const void*, WsPtrs, int,
                                             int, int, float, void*, uint8_t*, cudaStream_t);
template cudaError_t inst_updown_tma<InstElem>(const TmaPlan&, const void*, const void*,
                                               const void*, WsPtrs, int, int, int, void*, int,
                                               void*, void*, const void*, float, cudaStream_t);

}  // namespace cats
