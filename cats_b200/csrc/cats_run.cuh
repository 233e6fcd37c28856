// Host-side launch plumbing shared by the translation units of the library: launch plans, the
// launch helper and the per-element-type launchers.  The kernels are templates on the element
// type, the batch tile and a few layout constants; every element type is instantiated in a
// translation unit of its own (cats_inst_stage.cu, cats_inst_mega.cu, compiled once per type) so
// that the library builds in parallel, and cats_abi.cu only sees the declarations below.
#pragma once

#include <string.h>

#include "cats_mega.cuh"

namespace cats {

struct DevInfo {
  int sms = 0;
  int max_smem_optin = 0;
  int clock_khz = 0;  // SM clock (cycles per millisecond): converts the wait limit to cycles
};
const DevInfo& dev_info();  // per-device properties of the current device (cats_abi.cu)
extern int g_use_pdl;       // cats_set_option("pdl", 0) launches without programmatic dependencies

// Launch with the programmatic-stream-serialisation attribute: the grid may be scheduled while
// its predecessor drains; every kernel here calls griddepcontrol.wait before touching data.
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                   cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

inline int batch_tile(int B) { return B <= 1 ? 1 : B <= 2 ? 2 : B <= 4 ? 4 : B <= 8 ? 8 : 16; }

// ---- grid sizing --------------------------------------------------------------------------
inline int gate_segments(int I) {
  int g = dev_info().sms * 2;
  if (g > kMaxSeg) g = kMaxSeg;
  const int by_rows = (I + 15) / 16;  // at least ~16 rows (two per warp) per CTA
  if (g > by_rows) g = by_rows;
  return g < 1 ? 1 : g;
}

inline int updown_ctas(int I) {
  int g = dev_info().sms * 2;
  const int by_rows = (I + 7) / 8;
  if (g > by_rows) g = by_rows;
  return g < 1 ? 1 : g;
}

struct TmaPlan {
  bool ok = false, xs = false;
  int S = 0, grid = 0, sr = 1, nvt = 1, cap = 0, rmax = 0, cw = 1, pw = 1;
  int wait_kc = 0;  // limit of every wait in the kernel, in units of 1024 clock cycles
  size_t smem = 0;
  // stage 1 only: rows of this matrix (the up projection) to ask into L2 for the first pf_n active
  // neurons of every segment, for the stage-2 kernel that follows (null: none)
  const void* pf_base = nullptr;
  int pf_n = 0;
};


struct MegaPlan {
  bool ok = false;
  int S = 0, cw = 1, grid = 0, nvt = 1, cap = 0, rmax = 0, bulk_flush = 0, mma_dot = 0, parts = kParts;
  int wait_kc = 0;
  size_t smem = 0;
};


// dense tensor-core path (cats_dense.cuh): 16-bit types, H a multiple of 128, I a multiple of 64
struct DensePlan {
  bool ok = false;
  int grid = 0, box_rows = 0, Sf = 0, wait_kc = 0;   // Sf: ring stages
  size_t smemf = 0;
};
cudaError_t inst_dense(const DensePlan& p, const void* x, const void* Wg, const void* Wu, const void* Wd,
                       WsPtrs ws, int B, int H, int I, int dtype, float thr, void* out, int out_mode,
                       void* resid, void* x_next, const void* norm_w, float eps, cudaStream_t st);

constexpr int kDenseStackMaxLayers = 80;   // layers per launch of the dense stack kernel
cudaError_t inst_dense_stack(const DensePlan& p, int L, const void* const* Wg, const void* const* Wu,
                             const void* const* Wd, const float* thr, void* x_io, void* x_tmp,
                             void* resid, WsPtrs ws, int B, int H, int I, int dtype, float eps,
                             cudaStream_t st);

// ---- launchers, one set per element type T (float, __half, __nv_bfloat16) -----------------------
template <typename T>
cudaError_t inst_gate(const void* x, const void* Wg, WsPtrs ws, int B, int H, int I, float thr,
                      void* gate_dense, uint8_t* flag_dense, cudaStream_t st);
template <typename T>
cudaError_t inst_updown(int mode, const void* x, const void* Wu, const void* WdT, WsPtrs ws, int B,
                        int H, int I, void* out, int out_mode, void* resid, void* x_next,
                        const void* norm_w, float eps, void* inter_dense, cudaStream_t st);
template <typename T>
cudaError_t inst_rows_gemv(const void* xs, const void* W, int B, int K, int R, void* out,
                           cudaStream_t st);
// B <= 4 only (the TMA-fed kernels are instantiated for batch tiles 1, 2, 4)
template <typename T>
cudaError_t inst_gate_tma(const TmaPlan& p, const void* x, const void* Wg, WsPtrs ws, int B, int H,
                          int I, float thr, void* gate_dense, uint8_t* flag_dense, cudaStream_t st);
template <typename T>
cudaError_t inst_updown_tma(const TmaPlan& p, const void* x, const void* Wu, const void* WdT,
                            WsPtrs ws, int B, int H, int I, void* out, int out_mode, void* resid,
                            void* x_next, const void* norm_w, float eps, cudaStream_t st);
template <typename T>
cudaError_t inst_mega(const MegaPlan& p, const MegaParams& P, const MegaArgs& A, WsPtrs ws,
                      cudaStream_t st);

// the element type a per-type translation unit is compiled for (-DCATS_ELEM_ID=0|1|2)
#if defined(CATS_ELEM_ID)
#if CATS_ELEM_ID == 0
typedef float InstElem;
#elif CATS_ELEM_ID == 1
typedef __half InstElem;
#else
typedef __nv_bfloat16 InstElem;
#endif
#endif

}  // namespace cats
