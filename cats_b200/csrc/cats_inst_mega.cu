// The persistent kernel instantiated for ONE element type; compiled once per type with
// -DCATS_ELEM_ID=0|1|2 (float, __half, __nv_bfloat16).
#include "cats_run.cuh"

namespace cats {
namespace {

template <typename T, int BT, int NVT>
cudaError_t launch_mega(const MegaPlan& p, const MegaParams& P, const MegaArgs& A, WsPtrs ws,
                        cudaStream_t st) {
  auto kernel = k_cats_mega<T, BT, NVT>;
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(p.grid);
  cfg.blockDim = dim3(kMegaThreads);
  cfg.dynamicSmemBytes = p.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // CTAs wait for one another: must be co-resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, P, A, ws);
}

template <typename T, int BT>
cudaError_t run_mega(const MegaPlan& p, const MegaParams& P, const MegaArgs& A, WsPtrs ws,
                     cudaStream_t st) {
  switch (p.nvt) {
    case 1: return launch_mega<T, BT, 1>(p, P, A, ws, st);
    case 2: return launch_mega<T, BT, 2>(p, P, A, ws, st);
    case 4: return launch_mega<T, BT, 4>(p, P, A, ws, st);
    default: return launch_mega<T, BT, 8>(p, P, A, ws, st);
  }
}

}  // namespace

template <typename T>
cudaError_t inst_mega(const MegaPlan& p, const MegaParams& P, const MegaArgs& A, WsPtrs ws,
                      cudaStream_t st) {
  switch (batch_tile(A.B)) {
    case 1: return run_mega<T, 1>(p, P, A, ws, st);
    case 2: return run_mega<T, 2>(p, P, A, ws, st);
    default: return run_mega<T, 4>(p, P, A, ws, st);
  }
}

template cudaError_t inst_mega<InstElem>(const MegaPlan&, const MegaParams&, const MegaArgs&,
                                         WsPtrs, cudaStream_t);

}  // namespace cats
