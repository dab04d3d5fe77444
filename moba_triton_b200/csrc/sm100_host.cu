// Host helpers of the tcgen05 kernels: tensor-map encoding through the driver
// entry point (looked up at run time, so the library has no link-time
// dependency on the driver) and the per-device error word.
#include "common.cuh"
#include "sm100.cuh"

#include <mutex>

namespace moba {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int encode_rows_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t heads, uint64_t dim,
                    uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MOBA_B200_ECUDA; }
  const cuuint64_t dims[3] = {dim, heads, rows};
  const cuuint64_t strides[2] = {dim * 2, heads * dim * 2};     // bytes, dims 1 and 2
  const cuuint32_t box[3] = {64, 1, box_rows};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return MOBA_B200_ECUDA; }
  return MOBA_B200_OK;
}

int encode_2d_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t dim, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MOBA_B200_ECUDA; }
  const cuuint64_t dims[2] = {dim, rows};
  const cuuint64_t strides[1] = {dim * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return MOBA_B200_ECUDA; }
  return MOBA_B200_OK;
}

// Block means [kv_rows][blocks][dim]: box of (64, 128 blocks, 1 row).
int encode_kbar_map_impl(CUtensorMap* out, const void* base, uint64_t kv_rows, uint64_t nb, uint64_t dim) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MOBA_B200_ECUDA; }
  const cuuint64_t dims[3] = {dim, nb, kv_rows};
  const cuuint64_t strides[2] = {dim * 2, nb * dim * 2};
  const cuuint32_t box[3] = {64, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return MOBA_B200_ECUDA; }
  return MOBA_B200_OK;
}

// one word per device of this process, zero-initialised with the module
#if defined(MOBA_WAIT_STATS) || defined(MOBA_TRACE)
__device__ unsigned g_error_word[64 + 2 * 32 * 160 + 2 * 8 * 32 * 16];   // debug builds: + per-CTA wait counters + trace
#else
__device__ unsigned g_error_word[1];
#endif

unsigned* device_error_word() {
  static unsigned* table[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (table[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_error_word) != cudaSuccess) return nullptr;
    table[dev] = static_cast<unsigned*>(p);
  }
  return table[dev];
}

#ifdef MOBA_TRACE
extern "C" int moba_b200_debug_trace(unsigned long long* host_out) {
  unsigned* base = device_error_word();
  if (base == nullptr) return -1;
  cudaDeviceSynchronize();
  return (int)cudaMemcpy(host_out, base + 64 + 2 * 32 * 160, (size_t)8 * 32 * 16 * 8, cudaMemcpyDeviceToHost);
}
#endif

#ifdef MOBA_WAIT_STATS
extern "C" int moba_b200_debug_stats(unsigned long long* host_out, int n_ctas) {
  unsigned* base = device_error_word();
  if (base == nullptr) return -1;
  cudaDeviceSynchronize();
  return (int)cudaMemcpy(host_out, base + 64, (size_t)n_ctas * 32 * 8, cudaMemcpyDeviceToHost);
}
#endif

}  // namespace moba
