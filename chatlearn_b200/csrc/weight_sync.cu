// Trainer -> rollout weight reshard as ONE kernel per destination GPU.
//
// The host-side planner (synchronizer/plan.py) reduces QKV packing, gate/up
// packing, TP re-splitting, GQA replication and expert re-homing to a table of
// 2-D copy descriptors.  Each descriptor names a source rectangle in some rank's
// flat parameter buffer (this GPU's or a peer's, addressed through the
// symmetric-memory pointer table) and a destination rectangle in this GPU's
// rollout buffers.  CTAs walk the table and *pull* with plain 16-byte loads over
// NVLink, casting fp32 -> bf16 on the fly when the dtypes differ, so the data
// crosses the link once, lands in its final layout, and no staging bucket,
// pack/unpack pass or host round trip exists.  This replaces the pack ->
// batch_isend_irecv -> CUDA-IPC -> unpack+cast pipeline of
// chatlearn/synchronizer/comm.py:92-286 and the full-tensor all-gather of
// chatlearn/models/fsdp_module.py:498-541.
//
// No TMA and no multicast are used: peer memory is read with ordinary ld.global.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

struct SyncDesc {
  const void* src;      // element 0 of the source rectangle
  void* dst;            // element 0 of the destination rectangle
  int64_t src_stride;   // elements between source rows
  int64_t dst_stride;
  int32_t rows;
  int32_t cols;
  int32_t first_tile;   // index of this descriptor's first tile in the global tile space
  int32_t tiles_per_row;
};

constexpr int kTileElems = 2048;  // elements of one row segment handled by one CTA pass

template <typename S, typename D>
__device__ __forceinline__ void copy_segment(const S* __restrict__ s, D* __restrict__ d, int n) {
  constexpr int VS = 16 / sizeof(S), VD = 16 / sizeof(D);
  constexpr int V = VS < VD ? VS : VD;                 // elements per step with both sides <= 16 B
  const bool aligned = ((uintptr_t)s % (V * sizeof(S)) == 0) && ((uintptr_t)d % (V * sizeof(D)) == 0);
  int i = 0;
  if (aligned) {
    const int nv = n / V;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      S tmp[V];
      D out[V];
      if (sizeof(S) * V == 16) *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(s + v * V);
      else if (sizeof(S) * V == 8) *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(s + v * V);
      else { for (int j = 0; j < V; ++j) tmp[j] = s[v * V + j]; }
#pragma unroll
      for (int j = 0; j < V; ++j) out[j] = Cvt<D>::from_f(Cvt<S>::to_f(tmp[j]));
      if (sizeof(D) * V == 16) *reinterpret_cast<uint4*>(d + v * V) = *reinterpret_cast<uint4*>(out);
      else if (sizeof(D) * V == 8) *reinterpret_cast<uint2*>(d + v * V) = *reinterpret_cast<uint2*>(out);
      else { for (int j = 0; j < V; ++j) d[v * V + j] = out[j]; }
    }
    i = nv * V;
  }
  for (int k = i + threadIdx.x; k < n; k += blockDim.x) d[k] = Cvt<D>::from_f(Cvt<S>::to_f(s[k]));
}

// Tiles are (descriptor, row, column segment); the grid strides over all of them.
template <typename S, typename D>
__global__ void weight_sync_kernel(const SyncDesc* __restrict__ descs, int num_descs, int64_t total_tiles) {
  __shared__ int sh_desc;
  for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    if (threadIdx.x == 0) {
      // binary search: last descriptor with first_tile <= tile
      int lo = 0, hi = num_descs - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((int64_t)descs[mid].first_tile <= tile) lo = mid; else hi = mid - 1;
      }
      sh_desc = lo;
    }
    __syncthreads();
    const SyncDesc d = descs[sh_desc];
    const int64_t local = tile - d.first_tile;
    const int row = (int)(local / d.tiles_per_row);
    const int seg = (int)(local % d.tiles_per_row);
    const int c0 = seg * kTileElems;
    const int n = min(kTileElems, d.cols - c0);
    copy_segment<S, D>((const S*)d.src + (int64_t)row * d.src_stride + c0,
                       (D*)d.dst + (int64_t)row * d.dst_stride + c0, n);
    __syncthreads();
  }
}

// desc_table: uint8 tensor holding SyncDesc[num_descs] on the device.
void weight_sync_run(const at::Tensor& desc_table, int64_t num_descs, int64_t total_tiles, int64_t src_dtype,
                     int64_t dst_dtype) {
  if (num_descs == 0 || total_tiles == 0) return;
  TORCH_CHECK(desc_table.is_cuda() && desc_table.numel() >= (int64_t)(num_descs * sizeof(SyncDesc)));
  const auto* d = reinterpret_cast<const SyncDesc*>(desc_table.data_ptr());
  const int grid = (int)std::min<int64_t>(total_tiles, 148 * 8);
  auto st = at::cuda::getCurrentCUDAStream();
  // dtype codes: 0 = fp32, 1 = bf16
  if (src_dtype == 0 && dst_dtype == 0) weight_sync_kernel<float, float><<<grid, 256, 0, st>>>(d, (int)num_descs, total_tiles);
  else if (src_dtype == 0 && dst_dtype == 1) weight_sync_kernel<float, bf16><<<grid, 256, 0, st>>>(d, (int)num_descs, total_tiles);
  else if (src_dtype == 1 && dst_dtype == 1) weight_sync_kernel<bf16, bf16><<<grid, 256, 0, st>>>(d, (int)num_descs, total_tiles);
  else if (src_dtype == 1 && dst_dtype == 0) weight_sync_kernel<bf16, float><<<grid, 256, 0, st>>>(d, (int)num_descs, total_tiles);
  else TORCH_CHECK(false, "weight_sync: unsupported dtype pair");
}

int64_t weight_sync_desc_size() { return (int64_t)sizeof(SyncDesc); }
int64_t weight_sync_tile_elems() { return kTileElems; }
