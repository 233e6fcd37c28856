// Host side of the dense tensor-core path (cats_dense.cuh): TMA tensor maps and the two launches.
#include <mutex>
#include <unordered_map>

#include "cats_dense.cuh"
#include "cats_run.cuh"

namespace cats {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  int rows, cols, box_rows, dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= (size_t)k.rows * 1000003u + (size_t)k.cols * 10007u + (size_t)k.box_rows * 101u + (size_t)k.dtype;
    return h;
  }
};

// Tensor map of a row-major [rows, cols] 16-bit matrix, box = 64 columns x box_rows rows, 128-byte
// swizzle, rows / columns past the end read as zero.  Encoding takes microseconds, so maps are
// kept per (pointer, shape): weights keep their address for the life of a model.
bool tensor_map(const void* ptr, int rows, int cols, int box_rows, int dtype, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, box_rows, dtype};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kDenseKB, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = fn(&m, dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 8192) cache.clear();
    cache[key] = m;
  }
  *out = m;
  return true;
}

template <typename T, bool STACK, typename... Args>
cudaError_t launch_coop(const DensePlan& p, cudaStream_t st, Args... args) {
  // cooperative: the CTAs wait for one another at grid barriers
  auto kernel = k_dense<T, STACK>;
  cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel),
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smemf);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(p.grid);
  cfg.blockDim = dim3(kDenseThreads);
  cfg.dynamicSmemBytes = p.smemf;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename T>
cudaError_t launch_dense(const DensePlan& p, const void* x, const void* Wg, const void* Wu,
                         const void* Wd, WsPtrs ws, int B, int H, int I, int dtype, float thr, void* out,
                         int out_mode, void* resid, void* x_next, const void* norm_w, float eps,
                         cudaStream_t st) {
  DenseLayerMaps M;
  CUtensorMap m_x, m_h;
  T* h = reinterpret_cast<T*>(ws.h);   // [16, I] of T: the list array is not used on this path
  if (!tensor_map(Wg, I, H, p.box_rows, dtype, &M.wg) || !tensor_map(Wu, I, H, p.box_rows, dtype, &M.wu) ||
      !tensor_map(x, B, H, kDenseN, dtype, &m_x) || !tensor_map(Wd, H, I, 128, dtype, &M.wd) ||
      !tensor_map(h, B, I, kDenseN, dtype, &m_h))
    return cudaErrorInvalidValue;
  const DenseTail tail{out, out_mode, resid, x_next, norm_w};
  return launch_coop<T, false>(p, st, (const DenseStackParams*)nullptr, M, thr, m_x, m_x, m_h, ws, 1, B, H,
                               I, h, p.box_rows, (T*)nullptr, tail, eps, p.Sf, p.wait_kc);
}

template <typename T>
cudaError_t launch_dense_stack(const DensePlan& p, int L, const void* const* Wg, const void* const* Wu,
                               const void* const* Wd, const float* thr, void* x_io, void* x_tmp,
                               void* resid, WsPtrs ws, int B, int H, int I, int dtype, float eps,
                               cudaStream_t st) {
  static thread_local DenseStackParams P;   // ~31 KB: off the stack; filled per call
  CUtensorMap m_xa, m_xb, m_h;
  T* h = reinterpret_cast<T*>(ws.h);
  for (int l = 0; l < L; ++l) {
    if (!tensor_map(Wg[l], I, H, p.box_rows, dtype, &P.m[l].wg) ||
        !tensor_map(Wu[l], I, H, p.box_rows, dtype, &P.m[l].wu) ||
        !tensor_map(Wd[l], H, I, 128, dtype, &P.m[l].wd))
      return cudaErrorInvalidValue;
    P.thr[l] = thr[l];
  }
  if (!tensor_map(x_io, B, H, kDenseN, dtype, &m_xa) || !tensor_map(x_tmp, B, H, kDenseN, dtype, &m_xb) ||
      !tensor_map(h, B, I, kDenseN, dtype, &m_h))
    return cudaErrorInvalidValue;
  // the table goes to global memory first (a launch, so the call stays capturable in a graph)
  DenseStackParams* table = reinterpret_cast<DenseStackParams*>(ws.table);
  k_dense_table<<<1, 256, 0, st>>>(P, table);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const DenseTail tail{nullptr, 0, resid, x_io, nullptr};   // the last layer writes x_io
  return launch_coop<T, true>(p, st, (const DenseStackParams*)table, P.m[0], 0.f, m_xa, m_xb, m_h, ws, L, B,
                              H, I, h, p.box_rows, (T*)x_tmp, tail, eps, p.Sf, p.wait_kc);
}

}  // namespace

cudaError_t inst_dense_stack(const DensePlan& p, int L, const void* const* Wg, const void* const* Wu,
                             const void* const* Wd, const float* thr, void* x_io, void* x_tmp,
                             void* resid, WsPtrs ws, int B, int H, int I, int dtype, float eps,
                             cudaStream_t st) {
  if (L < 1 || L > kDenseMaxLayers) return cudaErrorInvalidValue;
  if (dtype == 1)
    return launch_dense_stack<__half>(p, L, Wg, Wu, Wd, thr, x_io, x_tmp, resid, ws, B, H, I, dtype, eps, st);
  return launch_dense_stack<__nv_bfloat16>(p, L, Wg, Wu, Wd, thr, x_io, x_tmp, resid, ws, B, H, I, dtype,
                                           eps, st);
}

cudaError_t inst_dense(const DensePlan& p, const void* x, const void* Wg, const void* Wu, const void* Wd,
                       WsPtrs ws, int B, int H, int I, int dtype, float thr, void* out, int out_mode,
                       void* resid, void* x_next, const void* norm_w, float eps, cudaStream_t st) {
  if (dtype == 1)
    return launch_dense<__half>(p, x, Wg, Wu, Wd, ws, B, H, I, dtype, thr, out, out_mode, resid, x_next,
                                norm_w, eps, st);
  return launch_dense<__nv_bfloat16>(p, x, Wg, Wu, Wd, ws, B, H, I, dtype, thr, out, out_mode, resid,
                                     x_next, norm_w, eps, st);
}

}  // namespace cats
