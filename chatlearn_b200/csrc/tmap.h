// Host-side helpers shared by the TMA-fed kernels: the driver entry point that encodes
// tensor maps, a 2-D bf16 map builder, and the per-thread context binding that the driver
// call needs.
#pragma once
#include <c10/cuda/CUDAException.h>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

namespace tmap {

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    cudaDriverEntryPointQueryResult qres;
    void* p = nullptr;
    auto err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    TORCH_CHECK(err == cudaSuccess && qres == cudaDriverEntryPointSuccess && p, "cuTensorMapEncodeTiled unavailable");
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// rows x cols bf16 row-major matrix with leading dimension ld (elements); box = box_rows x box_cols
// (box_cols * 2 bytes <= 128), 128-byte swizzle, out-of-range elements read as zero.
inline CUtensorMap make_bf16_2d(const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows, int box_cols = 64) {
  CUtensorMap tm;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)(ld * 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return tm;
}

// Tensor maps are encoded by a driver call, and that call needs the device's context bound to the
// calling thread.  A thread that has made no CUDA runtime call yet has none: an autograd worker (or any
// new host thread) whose first op is a TMA-fed kernel with its output served from the allocator's cache
// gets here that way.  cudaSetDevice on the current device binds the primary context without changing it.
inline void bind_context_to_thread(int dev) {
  thread_local int bound = -1;
  if (bound == dev) return;
  int cur = -1;
  C10_CUDA_CHECK(cudaGetDevice(&cur));
  TORCH_CHECK(cur == dev, "operands live on device ", dev, " but the current device is ", cur);
  C10_CUDA_CHECK(cudaSetDevice(cur));
  bound = dev;
}

inline int device_sms(int dev) {
  static int sms[64] = {};
  TORCH_CHECK(dev >= 0 && dev < 64, "device index out of range");
  if (!sms[dev]) C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
  return sms[dev];
}

}  // namespace tmap
