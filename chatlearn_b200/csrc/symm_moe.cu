// Expert-parallel dispatch and combine over NVLink peer memory.
//
// Every rank owns, in symmetric memory, a receive buffer with one fixed-capacity region per
// local expert (`recv_x [El, C, H]`), an output buffer of the same shape (`recv_y`) and a row
// cursor per local expert.  Dispatch: a warp per (token, slot) claims a row in the destination
// expert's region with ONE remote atomic on the owner's cursor and stores the token's hidden
// state straight into the owner's buffer; where the row went is remembered per pair.  The
// experts then run over their regions (grouped tcgen05 GEMM, tile table built from the cursors).
// Combine: a warp per token pulls its k expert outputs back from the owners and forms the
// weighted sum in fp32.  No all-to-all, no host-visible counts, no send/receive staging.
// Ranks meet at `symm_moe_barrier` (flag words, bounded waits, status code on timeout).
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kMaxWorld = 8;
constexpr uint64_t kWaitNs = 2000000000ull;

struct Peers {
  void* ptr[kMaxWorld];
};

__device__ int g_moe_status = 0;      // 0 ok, 1 barrier timeout, 2 region overflow

__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// One CTA; thread p < world signals peer p and waits for peer p's signal of the same round.
__global__ void moe_barrier_kernel(Peers flags, uint32_t* expect, int slot, int num_slots, int rank, int world) {
  const int p = threadIdx.x;
  if (p < world && p != rank) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(static_cast<uint32_t*>(flags.ptr[p]) + rank * num_slots + slot) : "memory");
    const uint32_t want = ++expect[slot * kMaxWorld + p];
    const uint32_t* mine = static_cast<const uint32_t*>(flags.ptr[rank]) + p * num_slots + slot;
    const uint64_t t0 = gtimer();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - want) >= 0) break;
      if (gtimer() - t0 > kWaitNs) { atomicCAS(&g_moe_status, 0, 1); break; }
    }
  }
}

// where[p] = owner rank * (El * C) + row inside the owner's buffer, or -1 if the region was full.
__global__ void moe_dispatch_kernel(const bf16* __restrict__ x, const int64_t* __restrict__ idx, Peers recv_x, Peers cursor,
                                    int* __restrict__ where, int64_t pairs, int k, int H, int El, int C) {
  const int lane = threadIdx.x & 31;
  const int64_t p = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= pairs) return;
  int loc = 0, owner = 0;
  if (lane == 0) {
    const int e = (int)idx[p];
    owner = e / El;
    const int le = e % El;
    const int pos = atomicAdd(static_cast<int*>(cursor.ptr[owner]) + le, 1);     // remote atomic over NVLink
    if (pos >= C) { atomicCAS(&g_moe_status, 0, 2); loc = -1; }
    else loc = le * C + pos;
    where[p] = loc < 0 ? -1 : owner * (El * C) + loc;
  }
  loc = __shfl_sync(0xffffffffu, loc, 0);
  owner = __shfl_sync(0xffffffffu, owner, 0);
  if (loc < 0) return;
  const bf16* src = x + (p / k) * (int64_t)H;
  bf16* dst = static_cast<bf16*>(recv_x.ptr[owner]) + (int64_t)loc * H;
  for (int v = lane; v < H / 8; v += 32) st16(dst + v * 8, ld16(src + v * 8));
}

// Row tiles of the occupied part of every region: table[i] = {first row, end row, first weight row, -}.
__global__ void moe_region_table_kernel(const int* __restrict__ cursor, int El, int C, int rows_b, int capacity,
                                        int4* __restrict__ table, int* __restrict__ count, int BM) {
  __shared__ int scan[1024];
  const int g = threadIdx.x;
  const int n = g < El ? min(cursor[g], C) : 0;
  const int mine = (n + BM - 1) / BM;
  scan[g] = mine;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = g >= d ? scan[g - d] : 0;
    __syncthreads();
    scan[g] += v;
    __syncthreads();
  }
  int at = scan[g] - mine;
  for (int t = 0; t < mine && at < capacity; ++t, ++at)
    table[at] = make_int4(g * C + t * BM, g * C + n, g * rows_b, 0);
  if (g == 1023) count[0] = min(scan[1023], capacity);
}

__global__ void moe_combine_pull_kernel(Peers recv_y, const int* __restrict__ where, const float* __restrict__ weights,
                                        bf16* __restrict__ out, int T_, int k, int H, int region_rows) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  for (int v = lane; v < H / 8; v += 32) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const int w = where[(int64_t)t * k + s];
      if (w < 0) continue;
      const float wt = weights[(int64_t)t * k + s];
      const bf16* src = static_cast<const bf16*>(recv_y.ptr[w / region_rows]) + (int64_t)(w % region_rows) * H + v * 8;
      Vec16<bf16> a = ld16(src);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wt * __bfloat162float(a.v[j]);
    }
    Vec16<bf16> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(acc[j]);
    st16(out + (int64_t)t * H + v * 8, o);
  }
}

// SwiGLU over the occupied rows only: CTAs walk the row-tile table of the grouped GEMM.
__global__ void moe_swiglu_table_kernel(const bf16* __restrict__ gu, bf16* __restrict__ y, const int4* __restrict__ table,
                                        const int* __restrict__ count, int F) {
  const int n_tiles = count[0];
  const int vec_per_row = F / 8;
  for (int ti = blockIdx.x; ti < n_tiles; ti += gridDim.x) {
    const int4 e = table[ti];
    const int rows = min(e.y - e.x, 128);
    for (int i = threadIdx.x; i < rows * vec_per_row; i += blockDim.x) {
      const int64_t r = e.x + i / vec_per_row;
      const int c = (i % vec_per_row) * 8;
      Vec16<bf16> g = ld16(gu + r * 2 * F + c), u = ld16(gu + r * 2 * F + F + c), o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = __bfloat162float(g.v[j]);
        o.v[j] = __float2bfloat16(a / (1.f + __expf(-a)) * __bfloat162float(u.v[j]));
      }
      st16(y + r * F + c, o);
    }
  }
}

Peers peers_from(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= kMaxWorld, "at most 8 ranks");
  Peers t;
  for (int i = 0; i < kMaxWorld; ++i) t.ptr[i] = i < (int)ptrs.size() ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return t;
}
inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }

}  // namespace

void symm_moe_barrier(const std::vector<int64_t>& flag_ptrs, at::Tensor expect, int64_t slot, int64_t num_slots, int64_t rank) {
  moe_barrier_kernel<<<1, 32, 0, stream()>>>(peers_from(flag_ptrs), reinterpret_cast<uint32_t*>(expect.data_ptr()), (int)slot,
                                             (int)num_slots, (int)rank, (int)flag_ptrs.size());
}

// x [T, H] bf16; idx [T, k] int64 global expert ids.  Returns where [T, k] int32.
at::Tensor symm_moe_dispatch(const at::Tensor& x, const at::Tensor& idx, const std::vector<int64_t>& recv_x_ptrs,
                             const std::vector<int64_t>& cursor_ptrs, int64_t experts_per_rank, int64_t capacity) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2 && x.size(1) % 8 == 0, "dispatch: bf16 [T, H]");
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous(), "dispatch: int64 idx");
  const int64_t T_ = x.size(0), k = idx.size(1), pairs = T_ * k;
  auto where = at::empty({T_, k}, x.options().dtype(at::kInt));
  if (pairs == 0) return where;
  const int warps = 8;
  moe_dispatch_kernel<<<(unsigned)((pairs + warps - 1) / warps), warps * 32, 0, stream()>>>(
      (const bf16*)x.data_ptr(), idx.data_ptr<int64_t>(), peers_from(recv_x_ptrs), peers_from(cursor_ptrs), where.data_ptr<int>(),
      pairs, (int)k, (int)x.size(1), (int)experts_per_rank, (int)capacity);
  return where;
}

// Tile table over the occupied rows of the regions, in the layout the grouped GEMM reads.
std::vector<at::Tensor> symm_moe_region_table(const at::Tensor& cursor, int64_t capacity, int64_t rows_b) {
  const int El = (int)cursor.numel();
  TORCH_CHECK(El <= 1024 && cursor.scalar_type() == at::kInt, "region table: at most 1024 local experts, int32 cursor");
  const int BM = 128;
  const int cap_tiles = (int)(El * ((capacity + BM - 1) / BM));
  auto table = at::empty({cap_tiles, 4}, cursor.options());
  auto count = at::empty({1}, cursor.options());
  moe_region_table_kernel<<<1, 1024, 0, stream()>>>(cursor.data_ptr<int>(), El, (int)capacity, (int)rows_b, cap_tiles,
                                                    reinterpret_cast<int4*>(table.data_ptr<int>()), count.data_ptr<int>(), BM);
  return {table, count};
}

at::Tensor symm_moe_combine(const std::vector<int64_t>& recv_y_ptrs, const at::Tensor& where, const at::Tensor& weights,
                            int64_t H, int64_t region_rows) {
  const int T_ = (int)where.size(0), k = (int)where.size(1);
  auto out = at::empty({T_, H}, where.options().dtype(at::kBFloat16));
  if (T_ == 0) return out;
  auto w = weights.to(at::kFloat).contiguous();
  const int warps = 8;
  moe_combine_pull_kernel<<<(T_ + warps - 1) / warps, warps * 32, 0, stream()>>>(peers_from(recv_y_ptrs), where.data_ptr<int>(),
                                                                               w.data_ptr<float>(), (bf16*)out.data_ptr(), T_, k, (int)H,
                                                                               (int)region_rows);
  return out;
}

// y[r] = silu(gu[r, :F]) * gu[r, F:] for the rows the table lists (gu [R, 2F], y [R, F], bf16).
void symm_moe_swiglu(const at::Tensor& gu, at::Tensor y, const at::Tensor& table, const at::Tensor& count) {
  const int F = (int)y.size(1);
  TORCH_CHECK(gu.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16 && gu.is_contiguous() && y.is_contiguous() &&
              gu.size(1) == 2 * F && F % 8 == 0, "moe swiglu: bf16 [R, 2F] -> [R, F]");
  if (table.size(0) == 0) return;
  moe_swiglu_table_kernel<<<(int)std::min<int64_t>(table.size(0), 148 * 4), 256, 0, stream()>>>(
      (const bf16*)gu.data_ptr(), (bf16*)y.data_ptr(), reinterpret_cast<const int4*>(table.data_ptr<int>()), count.data_ptr<int>(), F);
}

int64_t symm_moe_last_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int));
  int zero = 0;
  cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int));
  return v;
}
