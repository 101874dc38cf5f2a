// bf16 GEMM on the 5th-generation tensor cores, fp32 accumulation in tensor memory.
// Three operand layouts, selected per instantiation (AMN / BMN = the operand's M or N
// index is the contiguous one in memory instead of K):
//   NT  C[M,N] = A[M,K] * B[N,K]^T      y  = x W^T     forward of a linear layer
//   NN  C[M,N] = A[M,K] * B[K,N]        dx = dy W      input gradient
//   TN  C[M,N] = A[K,M]^T * B[K,N]      dW = dy^T x    weight gradient, optionally
//                                                      accumulated into an fp32 C (beta = 1)
// An MN-major operand is fetched as 64-element-wide TMA boxes (64 MN x 64 K, 128-byte
// swizzle) and described to the tensor core with an MN-major shared-memory descriptor, so
// no operand is ever transposed in memory.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: streams 128x64 (A) and 256x64 (B) bf16 tiles into a
//               4-stage shared-memory ring (128-byte swizzle), one mbarrier per stage
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128x256x16) over the
//               ring; tcgen05.commit frees a stage / publishes an accumulator
//   warps 2..5  epilogue: tcgen05.ld the 128x256 fp32 accumulator out of TMEM,
//               convert, store.  Two accumulators (2 x 256 TMEM columns) let the
//               epilogue of tile i overlap the main loop of tile i+1.
// No cluster launch and no TMA multicast are used.  Every mbarrier wait is
// bounded; a timeout records a status code (readable with gemm_last_status) and
// the CTA drains and frees its tensor memory instead of hanging.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <cstdio>
#include <cstdlib>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include "common.cuh"
#include "sm100.cuh"
#include "tmap.h"

using namespace sm100;
using cl::launch_pdl;
using cl::pdl_trigger;
using cl::pdl_wait;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kAccBufs = 2;
constexpr int kTmemCols = BN * kAccBufs;  // 512
constexpr int kThreads = 192;
constexpr uint32_t kStageBytesA = BM * BK * 2, kStageBytesB = BN * BK * 2;

// The kernel is instantiated for tile widths 256 (large problems), 128 and 64 (few rows, as
// in a decode step: narrower tiles give every SM a tile without slicing K).
template <int BN_>
struct __align__(1024) SmemLayoutT {
  uint8_t a[kStages][kStageBytesA];
  uint8_t b[kStages][BN_ * BK * 2];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[kAccBufs];
  uint64_t acc_empty[kAccBufs];
  uint32_t tmem_base;
  uint32_t abort_flag;
  // reduce-scatter epilogue: per epilogue warp, 32 rows x 64 bf16 columns (128 bytes, padded to 144 against bank
  // conflicts) staged so that the stores that cross NVLink cover whole 128-byte row segments
  alignas(16) uint8_t stage_c[4][32 * 144];
};
using SmemLayout = SmemLayoutT<BN>;

__device__ int g_gemm_status = 0;
bool g_allow_splitk = true;
int g_force_bn = 0;       // 0: choose the tile width per shape

enum : int { ST_OK = 0, ST_PRODUCER_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_EPILOGUE_TIMEOUT = 3 };

// Tile order: groups of kGroupM row-blocks are swept column-block by column-block,
// so the CTAs running at the same time share a narrow band of B (which then stays
// in L2) instead of each re-streaming the whole weight matrix.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_origin(int tile, int tiles_m, int tiles_n, int& m0, int& n0, int BN) {
  const int group_size = kGroupM * tiles_n;
  const int group = tile / group_size;
  const int first_m = group * kGroupM;
  const int gm = min(tiles_m - first_m, kGroupM);
  const int in_group = tile - group * group_size;
  m0 = (first_m + in_group % gm) * BM;
  n0 = (in_group / gm) * BN;
}

template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const uint32_t (&r)[32], int ncols);

template <>
__device__ __forceinline__ void store_row32<bf16>(bf16* dst, const uint32_t (&r)[32], int ncols) {
  if (ncols >= 32) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint4 pk;
      uint32_t* p = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
        p[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = pk;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
  }
}
template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const uint32_t (&r)[32], int ncols) {
  if (ncols >= 32) {
#pragma unroll
    for (int v = 0; v < 8; ++v)
      *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[j] = __uint_as_float(r[j]);
  }
}

// C += r for an fp32 output row segment (weight-gradient accumulation across micro-batches).
__device__ __forceinline__ void add_row32(float* dst, const uint32_t (&r)[32], int ncols) {
  if (ncols >= 32) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float4 c = *reinterpret_cast<const float4*>(dst + v * 4);
      c.x += __uint_as_float(r[v * 4]); c.y += __uint_as_float(r[v * 4 + 1]);
      c.z += __uint_as_float(r[v * 4 + 2]); c.w += __uint_as_float(r[v * 4 + 3]);
      *reinterpret_cast<float4*>(dst + v * 4) = c;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[j] += __uint_as_float(r[j]);
  }
}

// Grouped mode (mixture-of-experts): A holds the rows of all groups back to back, B the
// groups' [N, K] matrices stacked along rows.  `table[i] = {first row, end row, first B
// row of the group, -}` lists the row tiles (built on the device from the group offsets,
// so the host never learns the group sizes); `count[0]` is the number of entries.  A row
// tile may read past its group's rows (they belong to the next group or are zero-filled
// beyond the tensor); only rows below `end row` are stored.
struct GroupArgs {
  const int4* table = nullptr;
  const int* count = nullptr;
  // n_peer > 0: the output is stored to these addresses (one per rank of a group, peers' memory
  // included) instead of C
  void* peer_out[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_peer = 0;
  // scatter_rows > 0 (with n_peer > 0): reduce-scatter form.  Row r of the product goes to destination
  // r / scatter_rows only, at row r % scatter_rows of that destination's buffer (this rank's chunk of it)
  int scatter_rows = 0;
  int accumulate = 0;       // fp32 output only: C += A*B instead of C = A*B
  // ragged_m > 0: grouped weight gradient.  The contraction runs over a group's rows: table entries are
  // {first C row, end C row, first K row, end K row}; C is [groups * ragged_m, N] and a tile's columns of
  // the (MN-major) A operand start at (first C row) % ragged_m.
  int ragged_m = 0;
};

// Origin of a work tile: (first A/C row, first column, first B row of the group, end row).
__device__ __forceinline__ void unit_origin(const GroupArgs& grp, int tile, int tiles_m, int tiles_n, int M, int& m0,
                                            int& n0, int& b0, int& row_end, int BN) {
  if (grp.table != nullptr) {
    const int4 e = grp.table[tile / tiles_n];
    m0 = e.x; row_end = e.y; b0 = e.z;
    n0 = (tile % tiles_n) * BN;
  } else {
    tile_origin(tile, tiles_m, tiles_n, m0, n0, BN);
    b0 = 0; row_end = M;
  }
}

template <typename OutT, int BN_ = 256, int AMN = 0, int BMN = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    OutT* __restrict__ C, float* __restrict__ ws, int M, int N, int K, int ldc, int splits,
                    GroupArgs grp) {
  // tile width of this instantiation (these names hide the 256-wide defaults of the file scope)
  constexpr int BN = BN_;
  constexpr uint32_t kStageBytesB = BN * BK * 2;
  constexpr int kTmemCols = BN * kAccBufs;          // 512, 256 or 128 columns: powers of two >= 32
  using SmemLayout = SmemLayoutT<BN>;
  extern __shared__ uint8_t smem_raw[];
  // dynamic shared memory is only 16-byte aligned by contract: align to 1024 for the swizzle
  SmemLayout* sm = reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const bool grouped = grp.table != nullptr;
  if (grouped) pdl_wait();                      // the tile table and its count come from the kernel before this one
  const int num_tiles = (grouped ? min(grp.count[0], tiles_m) : tiles_m) * tiles_n;   // grouped: tiles_m = table capacity
  const int k_iters = (K + BK - 1) / BK;
  // split-K: a work unit is (tile, k-slice); units of one k-slice are consecutive so
  // concurrently running CTAs stream disjoint parts of B
  const int k_per_split = (k_iters + splits - 1) / splits;
  const int num_units = num_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], 1); }
    for (int b = 0; b < kAccBufs; ++b) { mbar_init(&sm->acc_full[b], 1); mbar_init(&sm->acc_empty[b], 4); }
    sm->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sm->tmem_base;
  // everything above touched only this CTA's shared and tensor memory; the operands and the output belong to
  // the kernels before this one in the stream
  pdl_trigger();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        int m0, n0, b0, row_end;
        unit_origin(grp, unit % num_tiles, tiles_m, tiles_n, M, m0, n0, b0, row_end, BN);
        int k_begin = (unit / num_tiles) * k_per_split, k_end = min(k_begin + k_per_split, k_iters);
        int a_m0 = m0, a_k0 = 0;                   // ragged: A columns of the tile, first K row of the group
        if (grp.ragged_m > 0) {
          const int4 e = grp.table[(unit % num_tiles) / tiles_n];
          a_m0 = e.x % grp.ragged_m; a_k0 = e.z;
          k_begin = 0; k_end = (e.w - e.z + BK - 1) / BK;
        }
        for (int k = k_begin; k < k_end; ++k) {
          if (!mbar_wait(&sm->empty[stage], phase ^ 1)) { ok = false; break; }
          mbar_expect_tx(&sm->full[stage], kStageBytesA + kStageBytesB);
          if constexpr (AMN == 0) {
            tma_load_2d(sm->a[stage], &tmA, &sm->full[stage], k * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)      // boxes of 64 M-columns x BK K-rows
              tma_load_2d(sm->a[stage] + j * (BK * 128), &tmA, &sm->full[stage], a_m0 + j * 64, a_k0 + k * BK);
          }
          if constexpr (BMN == 0) {
            tma_load_2d(sm->b[stage], &tmB, &sm->full[stage], k * BK, b0 + n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)      // boxes of 64 N-columns x BK K-rows (b0: first K-row of the group)
              tma_load_2d(sm->b[stage] + j * (BK * 128), &tmB, &sm->full[stage], n0 + j * 64, b0 + k * BK);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { atomicCAS(&g_gemm_status, ST_OK, ST_PRODUCER_TIMEOUT); atomicExch(&sm->abort_flag, 1u); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, AMN, BMN);
      // start-address step (16-byte units) of one 16-deep MMA: 32 bytes along a K-major row,
      // 16 K-rows of 128 bytes in an MN-major box
      constexpr uint64_t kStepA = AMN ? 128 : 2, kStepB = BMN ? 128 : 2;
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        int k_begin = (unit / num_tiles) * k_per_split, k_end = min(k_begin + k_per_split, k_iters);
        if (grp.ragged_m > 0) {
          const int4 e = grp.table[(unit % num_tiles) / tiles_n];
          k_begin = 0; k_end = (e.w - e.z + BK - 1) / BK;
        }
        if (!mbar_wait(&sm->acc_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = k_begin; k < k_end; ++k) {
          if (!mbar_wait(&sm->full[stage], phase)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t da = AMN ? make_mnmajor_sw128_desc(smem_u32(sm->a[stage]), BK * 128)
                                  : make_kmajor_sw128_desc(smem_u32(sm->a[stage]));
          const uint64_t db = BMN ? make_mnmajor_sw128_desc(smem_u32(sm->b[stage]), BK * 128)
                                  : make_kmajor_sw128_desc(smem_u32(sm->b[stage]));
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            umma_bf16(d_tmem, da + kStepA * kk, db + kStepB * kk, idesc, (k > k_begin || kk > 0) ? 1u : 0u);
          umma_commit(&sm->empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&sm->acc_full[acc]);
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) { atomicCAS(&g_gemm_status, ST_OK, ST_MMA_TIMEOUT); atomicExch(&sm->abort_flag, 1u); }
    }
  } else {
    // ------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
      int m0, n0, b0, row_end;
      unit_origin(grp, unit % num_tiles, tiles_m, tiles_n, M, m0, n0, b0, row_end, BN);
      bool empty_slice = (unit / num_tiles) * k_per_split >= k_iters;   // nothing was accumulated
      if (grp.ragged_m > 0) {
        const int4 e = grp.table[(unit % num_tiles) / tiles_n];
        empty_slice = e.w <= e.z;
      }
      if (!mbar_wait(&sm->acc_full[acc], acc_phase)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col = n0 + c;
        if constexpr (sizeof(OutT) == 2) {
          if (grp.scatter_rows > 0 && grp.n_peer > 0) {
            // GEMM + reduce-scatter: every row of this rank's partial product is stored once, into the receive
            // buffer of the rank that owns the row (over NVLink unless that is this rank), while the MMA warp
            // already works on the next tile; the owner adds the chunks up.  Two 32-column chunks are packed to
            // bf16 and staged in shared memory, then written with lanes laid along the row: every store
            // instruction covers four rows of 128 contiguous bytes instead of 32 separate 16-byte pieces.
            uint8_t* stg = sm->stage_c[q];
            const int half = (c >> 5) & 1;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              uint32_t* pp = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                pp[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(stg + lane * 144 + half * 64 + v * 16) = pk;
            }
            if (half == 1 || c + 32 >= BN) {
              __syncwarp();
              const int cbase = n0 + (c & ~63);               // first column of the staged pair
              const int piece = lane & 7;                     // 16 bytes = 8 columns
              const int gcol = cbase + piece * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rr = 4 * i + (lane >> 3);
                const int grow = m0 + q * 32 + rr;
                if (grow < row_end && gcol < N && !empty_slice && (half == 1 || piece < 4)) {
                  const int dst = grow / grp.scatter_rows;
                  const uint4 val = *reinterpret_cast<const uint4*>(stg + rr * 144 + piece * 16);
                  *reinterpret_cast<uint4*>(static_cast<bf16*>(grp.peer_out[dst]) +
                                            (int64_t)(grow - dst * grp.scatter_rows) * ldc + gcol) = val;
                }
              }
              __syncwarp();
            }
            continue;
          }
        }
        if (row < row_end && col < N && !empty_slice) {
          if (splits == 1) {
            if (grp.n_peer == 0) {
              if constexpr (sizeof(OutT) == 4) {
                if (grp.accumulate) add_row32(C + (int64_t)row * ldc + col, r, min(32, N - col));
                else store_row32<OutT>(C + (int64_t)row * ldc + col, r, min(32, N - col));
              } else {
                store_row32<OutT>(C + (int64_t)row * ldc + col, r, min(32, N - col));
              }
            } else {
              // GEMM + all-gather of the partial product: the tile goes straight from tensor memory
              // into every rank's staging slot (plain stores over NVLink for the peers), while the
              // MMA warp already works on the next tile in the other accumulator
              for (int p = 0; p < grp.n_peer; ++p)
                store_row32<OutT>(static_cast<OutT*>(grp.peer_out[p]) + (int64_t)row * ldc + col, r, min(32, N - col));
            }
          } else {
            // every k-slice writes its partial tile to its own plane of the workspace;
            // the finalize kernel adds the planes (plain stores: no atomics, deterministic)
            float* w = ws + ((int64_t)(unit / num_tiles) * M + row) * N + col;
            store_row32<float>(w, r, min(32, N - col));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->acc_empty[acc]);
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok && lane == 0) { atomicCAS(&g_gemm_status, ST_OK, ST_EPILOGUE_TIMEOUT); atomicExch(&sm->abort_flag, 1u); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Split-K epilogue: C = sum over the k-slice planes of the workspace.
template <typename OutT>
__global__ void splitk_finalize_kernel(const float* __restrict__ ws, OutT* __restrict__ C, int64_t n, int splits,
                                       int accumulate = 0) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(ws + i);
    if constexpr (sizeof(OutT) == 4) {
      if (accumulate) {
        const float4 c = *reinterpret_cast<const float4*>(C + i);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
      }
    }
    for (int s = 1; s < splits; ++s) {
      const float4 u = *reinterpret_cast<const float4*>(ws + (int64_t)s * n + i);
      v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
    }
    if constexpr (sizeof(OutT) == 2) {
      __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
      uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      *reinterpret_cast<uint2*>(C + i) = pk;
    } else {
      *reinterpret_cast<float4*>(C + i) = v;
    }
  }
}

constexpr int64_t kWorkspaceFloats = 16ll << 20;   // 64 MiB of fp32 partial sums per device

float* splitk_workspace(int device, const at::TensorOptions& opts) {
  static std::vector<at::Tensor> ws(64);
  if (!ws[device].defined()) ws[device] = at::empty({kWorkspaceFloats}, opts.dtype(at::kFloat));
  return ws[device].data_ptr<float>();
}

// rows x cols bf16 row-major matrix with leading dimension ld (elements); box = box_rows x 64.
CUtensorMap make_tmap_bf16(const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  return tmap::make_bf16_2d(ptr, rows, cols, ld, box_rows, BK);
}

}  // namespace

using tmap::bind_context_to_thread;
using tmap::device_sms;

// `cfg`: whether the opt-in for more than 48 KB of dynamic shared memory has been made on a device
// (the attribute is per device, so the flag is too).
template <typename T, int W, int AMN, int BMN>
static void launch_gemm(int dev, int grid, cudaStream_t st, const CUtensorMap& tmA, const CUtensorMap& tmB, T* c, float* ws,
                        int M, int N, int K, int ldc, int splits, const GroupArgs& ga) {
  static bool cfg[64] = {};
  const size_t smem = sizeof(SmemLayoutT<W>) + 1024;
  if (!cfg[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_nt_kernel<T, W, AMN, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cfg[dev] = true;
  }
  C10_CUDA_CHECK(launch_pdl(gemm_bf16_nt_kernel<T, W, AMN, BMN>, dim3(grid), dim3(kThreads), smem, st, tmA, tmB, c, ws, M, N, K, ldc,
                            splits, ga));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// General entry.  amn = 0: a is [M, K] with K contiguous; amn = 1: a is [K, M] with M contiguous (the
// product uses a^T).  bmn = 0: b is [N, K]; bmn = 1: b is [K, N].  C [M, N] is bf16, or fp32 when
// out_fp32; `accumulate` (fp32 only) adds the product to what `out` already holds.
// A caller that consumes the K-slice planes itself (a kernel that adds them up while it does its own work) sets
// `want` around one call; the call then skips the finalize kernel and reports where the planes are.
struct DeferredFinalize { bool want = false; int splits = 1; float* ws = nullptr; };
static thread_local DeferredFinalize g_defer;

static at::Tensor gemm_bf16_impl(const at::Tensor& a, const at::Tensor& b, int amn, int bmn, bool out_fp32,
                                 const at::Tensor* out, bool accumulate = false,
                                 const std::vector<int64_t>* peer_out = nullptr, int64_t scatter_rows = 0);

static at::Tensor gemm_bf16_nt_impl(const at::Tensor& a, const at::Tensor& b, bool out_fp32, const at::Tensor* out,
                                    const std::vector<int64_t>* peer_out = nullptr) {
  return gemm_bf16_impl(a, b, 0, 0, out_fp32, out, false, peer_out);
}

// GEMM whose epilogue stores the [M, N] result to several addresses at once: the copies of a
// symmetric-memory staging slot on every rank of a tensor-parallel group (this rank's own copy
// first or anywhere in the list).  `out` is this rank's copy and fixes shape and dtype (bf16).
void gemm_bf16_nt_push(const at::Tensor& a, const at::Tensor& b, at::Tensor out, const std::vector<int64_t>& peer_out) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.dim() == 2 && out.size(0) == a.size(0) && out.size(1) == b.size(0) &&
              out.scalar_type() == at::kBFloat16, "gemm_bf16_nt_push: out must be contiguous bf16 [M, N]");
  TORCH_CHECK(!peer_out.empty() && peer_out.size() <= 8, "gemm_bf16_nt_push: 1..8 destinations");
  for (int64_t p : peer_out) TORCH_CHECK(p % 16 == 0, "gemm_bf16_nt_push: 16-byte aligned destinations");
  gemm_bf16_nt_impl(a, b, false, &out, &peer_out);
}

at::Tensor gemm_bf16_nt(const at::Tensor& a, const at::Tensor& b, bool out_fp32) {
  return gemm_bf16_nt_impl(a, b, out_fp32, nullptr);
}

// C = A B^T whose K-slice planes are left for the consumer: returns {out bf16 [M, N], planes fp32 [S, M, N]}.  With
// S > 1 `out` is NOT written and `planes` is a view of the per-device split-K workspace: it is valid until the next
// K-sliced GEMM on this device, so the consumer kernel must be the next thing launched.  With S = 1 (the shape was
// not sliced) `out` holds the result and `planes` is an empty tensor.
std::vector<at::Tensor> gemm_bf16_nt_planes(const at::Tensor& a, const at::Tensor& b) {
  g_defer = DeferredFinalize{true, 1, nullptr};
  at::Tensor out;
  try {
    out = gemm_bf16_nt_impl(a, b, false, nullptr);
  } catch (...) {
    g_defer = DeferredFinalize{};
    throw;
  }
  const DeferredFinalize d = g_defer;
  g_defer = DeferredFinalize{};
  at::Tensor planes;
  if (d.splits > 1 && d.ws != nullptr)
    planes = at::from_blob(d.ws, {d.splits, out.size(0), out.size(1)}, out.options().dtype(at::kFloat));
  else
    planes = at::empty({0}, out.options().dtype(at::kFloat));
  return {out, planes};
}

// GEMM + reduce-scatter push: this rank's partial product a[M, K] * b[N, K]^T, rows split into `dst.size()` blocks
// of rows_per_rank; block d is stored (bf16) at dst[d], an address inside rank d's receive buffer (this rank's
// chunk of it, [rows_per_rank, N] contiguous).  Nothing is written locally except block `rank`.
void gemm_bf16_nt_scatter(const at::Tensor& a, const at::Tensor& b, const std::vector<int64_t>& dst, int64_t rows_per_rank) {
  TORCH_CHECK(!dst.empty() && dst.size() <= 8, "gemm_bf16_nt_scatter: 1..8 destinations");
  TORCH_CHECK(rows_per_rank > 0 && a.size(0) == rows_per_rank * (int64_t)dst.size(),
              "gemm_bf16_nt_scatter: the rows must split evenly over the destinations");
  for (int64_t p : dst) TORCH_CHECK(p % 16 == 0, "gemm_bf16_nt_scatter: 16-byte aligned destinations");
  // the shared code path wants an output tensor for its dtype; in this mode no element of it is written
  auto unused = at::empty({8}, a.options());
  gemm_bf16_impl(a, b, 0, 0, false, &unused, false, &dst, rows_per_rank);
}

// Same GEMM, result written into a caller-provided contiguous [M, N] tensor (for
// instance a symmetric-memory staging buffer that a peer-reading kernel consumes).
void gemm_bf16_nt_out(const at::Tensor& a, const at::Tensor& b, at::Tensor out) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.dim() == 2 && out.size(0) == a.size(0) &&
              out.size(1) == b.size(0), "gemm_bf16_nt_out: out must be contiguous [M, N]");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat, "gemm_bf16_nt_out: bf16 or fp32 out");
  TORCH_CHECK((uintptr_t)out.data_ptr() % 16 == 0, "gemm_bf16_nt_out: 16-byte aligned out");
  gemm_bf16_nt_impl(a, b, out.scalar_type() == at::kFloat, &out);
}

// Input gradient of a linear layer: C[M, N] = a[M, K] * b[K, N] (b row-major, e.g. dx = dy W).
at::Tensor gemm_bf16_nn(const at::Tensor& a, const at::Tensor& b, bool out_fp32) {
  return gemm_bf16_impl(a, b, 0, 1, out_fp32, nullptr);
}

// Weight gradient of a linear layer: C[M, N] (+)= a[K, M]^T * b[K, N] (e.g. dW = dy^T x).  With `out`
// (contiguous [M, N], bf16 or fp32) the result is written there; accumulate = true adds to an fp32 `out`.
at::Tensor gemm_bf16_tn(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& out, bool accumulate,
                        bool out_fp32) {
  if (out.has_value()) {
    const at::Tensor& o = *out;
    TORCH_CHECK(o.is_cuda() && o.is_contiguous() && o.dim() == 2 && o.size(0) == a.size(1) && o.size(1) == b.size(1),
                "gemm_bf16_tn: out must be contiguous [M, N]");
    TORCH_CHECK(o.scalar_type() == at::kBFloat16 || o.scalar_type() == at::kFloat, "gemm_bf16_tn: bf16 or fp32 out");
    TORCH_CHECK(!accumulate || o.scalar_type() == at::kFloat, "gemm_bf16_tn: accumulation needs an fp32 out");
    TORCH_CHECK((uintptr_t)o.data_ptr() % 16 == 0, "gemm_bf16_tn: 16-byte aligned out");
    return gemm_bf16_impl(a, b, 1, 1, o.scalar_type() == at::kFloat, &o, accumulate);
  }
  TORCH_CHECK(!accumulate, "gemm_bf16_tn: accumulation needs an out tensor");
  return gemm_bf16_impl(a, b, 1, 1, out_fp32, nullptr);
}

#define GTRACE(...) do { if (g_trace) { std::fprintf(stderr, "[gemm] " __VA_ARGS__); std::fprintf(stderr, "\n"); std::fflush(stderr); } } while (0)
static const bool g_trace = std::getenv("CLB200_GEMM_TRACE") != nullptr;

static at::Tensor gemm_bf16_impl(const at::Tensor& a, const at::Tensor& b, int amn, int bmn, bool out_fp32,
                                 const at::Tensor* out, bool accumulate, const std::vector<int64_t>* peer_out,
                                 int64_t scatter_rows) {
  GTRACE("enter amn=%d bmn=%d fp32=%d acc=%d", amn, bmn, (int)out_fp32, (int)accumulate);
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "gemm_bf16: bf16 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm_bf16: two-dimensional operands");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "gemm_bf16: the last dimension of both operands must be contiguous");
  const int64_t M = amn ? a.size(1) : a.size(0), K = amn ? a.size(0) : a.size(1);
  const int64_t N = bmn ? b.size(1) : b.size(0), Kb = bmn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm_bf16: contraction extents differ (", K, " vs ", Kb, ")");
  TORCH_CHECK(a.size(1) % 8 == 0 && b.size(1) % 8 == 0 && a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0,
              "gemm_bf16: contiguous extents and row strides must be multiples of 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr() % 16 == 0) && ((uintptr_t)b.data_ptr() % 16 == 0), "gemm_bf16: 16-byte aligned operands");
  TORCH_CHECK(!accumulate || (out != nullptr && out_fp32), "gemm_bf16: accumulation needs an fp32 out tensor");
  auto c = out ? *out : at::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  GTRACE("M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (M == 0 || N == 0) return c;
  if (K == 0) return accumulate ? c : c.zero_();
  TORCH_CHECK(N % 8 == 0, "gemm_bf16: N must be a multiple of 8");
  const int dev = a.get_device();
  bind_context_to_thread(dev);
  const int num_sms = device_sms(dev);
  GTRACE("dev=%d sms=%d", dev, num_sms);
  const bool plain_nt = !amn && !bmn;
  TORCH_CHECK(!(amn && !bmn), "gemm_bf16: the layout A[K,M]^T * B[N,K]^T is not built");
  const int tiles_m = (int)((M + BM - 1) / BM);
  const int k_iters = (int)((K + BK - 1) / BK);
  // Tile width and K slicing.  Large problems: 256-wide tiles, whole K.  Few rows (a decode
  // step): every SM should stream weights exactly once, so pick, among widths 256/128/64 and
  // slice counts that keep all work in one wave, the plan with the least estimated traffic
  // time: operand bytes per SM-sequence plus, when K is sliced, the fp32 partial planes.
  // (The gradient layouts are built 256 wide only.)
  int bn = 256, splits = 1;
  if (g_force_bn && plain_nt) {
    bn = g_force_bn;
  } else if (tiles_m * ((N + 255) / 256) < num_sms) {
    double best = 1e30;
    for (int cand : {256, 128, 64}) {
      if (!plain_nt && cand != 256) continue;
      const int tiles = tiles_m * (int)((N + cand - 1) / cand);
      int max_s = 1;
      if (g_allow_splitk && N % 4 == 0 && tiles < num_sms && peer_out == nullptr) max_s = std::min({num_sms / tiles, std::max(k_iters / 4, 1), 16});
      for (int s = 1; s <= max_s; ++s) {
        if ((int64_t)s * M * N > kWorkspaceFloats) break;
        const int per = (k_iters + s - 1) / s;
        if (s > 1 && per * (s - 1) >= k_iters) continue;                 // would leave an empty slice
        const int waves = (tiles * s + num_sms - 1) / num_sms;
        // the longer of: all operand bytes at device bandwidth, one SM's tile loads at the rate a
        // single SM sustains from L2 (activation tiles are re-read there); then, if K is sliced,
        // the partial planes written and re-read plus a fixed charge for the extra launch
        const double hbm = ((double)N * K + (double)M * K) * 2 / 6.5e12;
        const double sm = (double)waves * per * (BM + cand) * BK * 2 / 90e9;
        double cost = std::max(hbm, sm);
        if (s > 1) cost += 2.0 * s * M * N * 4 / 6.5e12 + 3.5e-6;
        if (cost < best) { best = cost; bn = cand; splits = s; }
      }
    }
  }
  if (g_force_bn && plain_nt && g_allow_splitk && N % 4 == 0 && peer_out == nullptr) {
    const int tiles = tiles_m * (int)((N + bn - 1) / bn);
    if (tiles * 2 <= num_sms) {
      splits = std::min({num_sms / tiles, std::max(k_iters / 4, 1), 16});
      while (splits > 1 && (int64_t)splits * M * N > kWorkspaceFloats) --splits;
      while (splits > 1 && ((k_iters + splits - 1) / splits) * (splits - 1) >= k_iters) --splits;
    }
  }
  const int tiles = tiles_m * (int)((N + bn - 1) / bn);
  GTRACE("bn=%d splits=%d tiles=%d", bn, splits, tiles);
  // K-major operand: boxes of 64 K x (tile rows); MN-major operand: boxes of 64 MN x 64 K over the [K, MN] matrix
  CUtensorMap tmA = amn ? make_tmap_bf16(a.data_ptr(), K, M, a.stride(0), BK) : make_tmap_bf16(a.data_ptr(), M, K, a.stride(0), BM);
  CUtensorMap tmB = bmn ? make_tmap_bf16(b.data_ptr(), K, N, b.stride(0), BK) : make_tmap_bf16(b.data_ptr(), N, K, b.stride(0), bn);
  GTRACE("tensor maps encoded");
  auto st = at::cuda::getCurrentCUDAStream();
  float* ws = splits > 1 ? splitk_workspace(dev, a.options()) : nullptr;
  GTRACE("stream and workspace %p", (void*)ws);
  const int grid = std::min(tiles * splits, num_sms);
  GroupArgs ga;
  ga.accumulate = accumulate ? 1 : 0;
  if (peer_out != nullptr) {
    TORCH_CHECK(splits == 1, "pushed output needs an unsliced K");
    ga.n_peer = (int)peer_out->size();
    ga.scatter_rows = (int)scatter_rows;
    for (int i = 0; i < ga.n_peer; ++i) ga.peer_out[i] = reinterpret_cast<void*>((*peer_out)[i]);
  }
  const int fgrid = (int)std::min<int64_t>((M * N / 4 + 255) / 256, 148 * 8);
#define CLB_GEMM_ARGS(PTR) dev, grid, st, tmA, tmB, PTR, ws, (int)M, (int)N, (int)K, (int)N, splits, ga
  if (out_fp32) {
    float* p = c.data_ptr<float>();
    if (amn && bmn) launch_gemm<float, 256, 1, 1>(CLB_GEMM_ARGS(p));
    else if (bmn) launch_gemm<float, 256, 0, 1>(CLB_GEMM_ARGS(p));
    else if (bn == 256) launch_gemm<float, 256, 0, 0>(CLB_GEMM_ARGS(p));
    else if (bn == 128) launch_gemm<float, 128, 0, 0>(CLB_GEMM_ARGS(p));
    else launch_gemm<float, 64, 0, 0>(CLB_GEMM_ARGS(p));
    if (splits > 1) {
      C10_CUDA_CHECK(launch_pdl(splitk_finalize_kernel<float>, dim3(fgrid), dim3(256), 0, st, ws, p, M * N, splits, ga.accumulate));
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
  } else {
    bf16* p = (bf16*)c.data_ptr();
    if (amn && bmn) launch_gemm<bf16, 256, 1, 1>(CLB_GEMM_ARGS(p));
    else if (bmn) launch_gemm<bf16, 256, 0, 1>(CLB_GEMM_ARGS(p));
    else if (bn == 256) launch_gemm<bf16, 256, 0, 0>(CLB_GEMM_ARGS(p));
    else if (bn == 128) launch_gemm<bf16, 128, 0, 0>(CLB_GEMM_ARGS(p));
    else launch_gemm<bf16, 64, 0, 0>(CLB_GEMM_ARGS(p));
    if (splits > 1 && g_defer.want) {
      g_defer.splits = splits;
      g_defer.ws = ws;
    } else if (splits > 1) {
      C10_CUDA_CHECK(launch_pdl(splitk_finalize_kernel<bf16>, dim3(fgrid), dim3(256), 0, st, ws, p, M * N, splits, 0));
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
  }
#undef CLB_GEMM_ARGS
  GTRACE("launched");
  return c;
}

// Debug / measurement knob: 0 = choose the tile width per shape, 64 / 128 / 256 = always that width.
void gemm_set_tile_n(int64_t bn) {
  TORCH_CHECK(bn == 0 || bn == 64 || bn == 128 || bn == 256, "tile width must be 0, 64, 128 or 256");
  g_force_bn = (int)bn;
}

// Status of the GEMM kernels since the last call (0 = ok); synchronises the device.
int64_t gemm_last_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
  int zero = 0;
  cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  return v;
}

void gemm_set_splitk(bool on) { g_allow_splitk = on; }

// ----------------------------------------------------------------------------
// Grouped GEMM for mixture-of-experts layers.
// ----------------------------------------------------------------------------
// offsets[g] .. offsets[g+1] are the rows of group g.  One block; thread g lists the
// row tiles of group g after an exclusive scan of the per-group tile counts.
static __global__ void build_group_table_kernel(const int64_t* __restrict__ offsets, int num_groups, int rows_b,
                                                int capacity, int4* __restrict__ table, int* __restrict__ count) {
  __shared__ int scan[1024];
  const int g = threadIdx.x;
  int lo = 0, hi = 0;
  if (g < num_groups) { lo = (int)offsets[g]; hi = (int)offsets[g + 1]; }
  const int mine = (hi - lo + BM - 1) / BM;
  scan[g] = mine;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {             // inclusive Hillis-Steele scan
    const int v = g >= d ? scan[g - d] : 0;
    __syncthreads();
    scan[g] += v;
    __syncthreads();
  }
  int at = scan[g] - mine;
  for (int t = 0; t < mine && at < capacity; ++t, ++at)
    table[at] = make_int4(lo + t * BM, hi, g * rows_b, 0);
  if (g == 1023) count[0] = min(scan[1023], capacity);
}

// a [R, K] bf16 rows sorted by group; b [G, N, K] bf16; offsets [G+1] int64 on the device
// (offsets[0] = 0, offsets[G] <= R).  Returns C [R, N] bf16; rows at or past offsets[G] are
// not written.
at::Tensor grouped_gemm_bf16_nt(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && offsets.is_cuda(), "grouped_gemm: CUDA tensors");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && offsets.scalar_type() == at::kLong,
              "grouped_gemm: bf16 operands, int64 offsets");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && a.size(1) == b.size(2) && a.is_contiguous() && b.is_contiguous(),
              "grouped_gemm: A [R, K], B [G, N, K], contiguous");
  const int64_t R = a.size(0), K = a.size(1), G = b.size(0), N = b.size(1);
  TORCH_CHECK(offsets.numel() == G + 1 && G <= 1024, "grouped_gemm: offsets [G+1], at most 1024 groups");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0 && K > 0, "grouped_gemm: K and N must be multiples of 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr() % 16 == 0) && ((uintptr_t)b.data_ptr() % 16 == 0), "grouped_gemm: 16-byte aligned operands");
  auto c = at::empty({R, N}, a.options());
  if (R == 0) return c;
  bind_context_to_thread(a.get_device());
  const int capacity = (int)((R + BM - 1) / BM + G);      // every group adds at most one partial tile
  auto table = at::empty({capacity, 4}, a.options().dtype(at::kInt));
  auto count = at::empty({1}, a.options().dtype(at::kInt));
  auto st = at::cuda::getCurrentCUDAStream();
  build_group_table_kernel<<<1, 1024, 0, st>>>(offsets.data_ptr<int64_t>(), (int)G, (int)N, capacity,
                                               reinterpret_cast<int4*>(table.data_ptr<int>()), count.data_ptr<int>());
  CUtensorMap tmA = make_tmap_bf16(a.data_ptr(), R, K, K, BM);
  CUtensorMap tmB = make_tmap_bf16(b.data_ptr(), G * N, K, K, BN);
  const int num_sms = device_sms(a.get_device());
  const int tiles_n = (int)((N + BN - 1) / BN);
  const int grid = std::min(capacity * tiles_n, num_sms);
  GroupArgs g;
  g.table = reinterpret_cast<const int4*>(table.data_ptr<int>());
  g.count = count.data_ptr<int>();
  // M = capacity * BM makes the kernel's row-tile bound equal to the table capacity
  launch_gemm<bf16, 256, 0, 0>(a.get_device(), grid, st, tmA, tmB, (bf16*)c.data_ptr(), nullptr, capacity * BM, (int)N, (int)K,
                               (int)N, 1, g);
  return c;
}

// Input gradient of grouped expert layers: C[r] = a[r] * b[g] for the rows r of group g, with b [G, K, N]
// (a group's weight as stored for the forward, rows = the forward's output features).  a [R, K] bf16 rows sorted
// by group, offsets [G+1] int64 on the device.  Returns C [R, N] bf16; rows outside every group are not written.
at::Tensor grouped_gemm_bf16_nn(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && offsets.is_cuda(), "grouped_gemm_nn: CUDA tensors");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && offsets.scalar_type() == at::kLong,
              "grouped_gemm_nn: bf16 operands, int64 offsets");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && a.size(1) == b.size(1) && a.is_contiguous() && b.is_contiguous(),
              "grouped_gemm_nn: A [R, K], B [G, K, N], contiguous");
  const int64_t R = a.size(0), K = a.size(1), G = b.size(0), N = b.size(2);
  TORCH_CHECK(offsets.numel() == G + 1 && G <= 1024, "grouped_gemm_nn: offsets [G+1], at most 1024 groups");
  // a K tile of B that runs past a group's K rows reads the next group's: A's columns there must not exist
  TORCH_CHECK(K % BK == 0 && N % 8 == 0 && K > 0, "grouped_gemm_nn: K must be a multiple of 64, N of 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr() % 16 == 0) && ((uintptr_t)b.data_ptr() % 16 == 0), "grouped_gemm_nn: 16-byte aligned operands");
  auto c = at::empty({R, N}, a.options());
  if (R == 0) return c;
  bind_context_to_thread(a.get_device());
  const int capacity = (int)((R + BM - 1) / BM + G);
  auto table = at::empty({capacity, 4}, a.options().dtype(at::kInt));
  auto count = at::empty({1}, a.options().dtype(at::kInt));
  auto st = at::cuda::getCurrentCUDAStream();
  build_group_table_kernel<<<1, 1024, 0, st>>>(offsets.data_ptr<int64_t>(), (int)G, (int)K, capacity,
                                               reinterpret_cast<int4*>(table.data_ptr<int>()), count.data_ptr<int>());
  CUtensorMap tmA = make_tmap_bf16(a.data_ptr(), R, K, K, BM);
  CUtensorMap tmB = make_tmap_bf16(b.data_ptr(), G * K, N, N, BK);      // MN-major: boxes of 64 N x 64 K rows
  const int num_sms = device_sms(a.get_device());
  const int tiles_n = (int)((N + BN - 1) / BN);
  const int grid = std::min(capacity * tiles_n, num_sms);
  GroupArgs g;
  g.table = reinterpret_cast<const int4*>(table.data_ptr<int>());
  g.count = count.data_ptr<int>();
  launch_gemm<bf16, 256, 0, 1>(a.get_device(), grid, st, tmA, tmB, (bf16*)c.data_ptr(), nullptr, capacity * BM, (int)N, (int)K,
                               (int)N, 1, g);
  return c;
}

// Row tiles of a grouped weight gradient: group g with rows [lo, hi) gets ceil(m / BM) entries
// {g * m + t * BM, (g + 1) * m, lo, hi}; empty groups get none (their part of C keeps what it holds).
static __global__ void build_ragged_table_kernel(const int64_t* __restrict__ offsets, int num_groups, int m, int capacity,
                                                 int4* __restrict__ table, int* __restrict__ count) {
  __shared__ int scan[1024];
  const int g = threadIdx.x;
  int lo = 0, hi = 0;
  if (g < num_groups) { lo = (int)offsets[g]; hi = (int)offsets[g + 1]; }
  const int mine = hi > lo ? (m + BM - 1) / BM : 0;
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
    table[at] = make_int4(g * m + t * BM, (g + 1) * m, lo, hi);
  if (g == 1023) count[0] = min(scan[1023], capacity);
}

// Weight gradient of grouped expert layers: C[g] (+)= a[rows of g]^T * b[rows of g], a [R, M] and b [R, N] bf16 with
// rows sorted by group.  Every group must start at a multiple of 64 rows, and the rows between a group's last
// row and the next group's first must be zero in a or in b (the contraction runs in tiles of 64 rows).
// offsets [G+1] int64 on the device.  `out` [G, M, N]: bf16 (overwritten; groups without rows are zeroed) or fp32
// (accumulate = true adds).  Returns out.
at::Tensor grouped_gemm_bf16_tn(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets, at::Tensor out,
                                bool accumulate) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && offsets.is_cuda() && out.is_cuda(), "grouped_gemm_tn: CUDA tensors");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && offsets.scalar_type() == at::kLong,
              "grouped_gemm_tn: bf16 operands, int64 offsets");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(0) == b.size(0) && a.is_contiguous() && b.is_contiguous(),
              "grouped_gemm_tn: A [R, M], B [R, N], contiguous");
  const int64_t R = a.size(0), M = a.size(1), N = b.size(1), G = offsets.numel() - 1;
  TORCH_CHECK(out.dim() == 3 && out.size(0) == G && out.size(1) == M && out.size(2) == N && out.is_contiguous(),
              "grouped_gemm_tn: out [G, M, N], contiguous");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat, "grouped_gemm_tn: bf16 or fp32 out");
  TORCH_CHECK(!accumulate || out.scalar_type() == at::kFloat, "grouped_gemm_tn: accumulation needs an fp32 out");
  TORCH_CHECK(G >= 1 && G <= 1024 && M % 8 == 0 && N % 8 == 0, "grouped_gemm_tn: 1..1024 groups, M and N multiples of 8");
  TORCH_CHECK(((uintptr_t)a.data_ptr() % 16 == 0) && ((uintptr_t)b.data_ptr() % 16 == 0) && ((uintptr_t)out.data_ptr() % 16 == 0),
              "grouped_gemm_tn: 16-byte aligned operands");
  if (!accumulate) out.zero_();
  if (R == 0) return out;
  bind_context_to_thread(a.get_device());
  const int tiles_m = (int)((M + BM - 1) / BM);
  const int capacity = (int)(G * tiles_m);
  auto table = at::empty({capacity, 4}, a.options().dtype(at::kInt));
  auto count = at::empty({1}, a.options().dtype(at::kInt));
  auto st = at::cuda::getCurrentCUDAStream();
  build_ragged_table_kernel<<<1, 1024, 0, st>>>(offsets.data_ptr<int64_t>(), (int)G, (int)M, capacity,
                                                reinterpret_cast<int4*>(table.data_ptr<int>()), count.data_ptr<int>());
  CUtensorMap tmA = make_tmap_bf16(a.data_ptr(), R, M, M, BK);      // MN-major: boxes of 64 columns x 64 rows
  CUtensorMap tmB = make_tmap_bf16(b.data_ptr(), R, N, N, BK);
  const int num_sms = device_sms(a.get_device());
  const int tiles_n = (int)((N + BN - 1) / BN);
  const int grid = std::min(capacity * tiles_n, num_sms);
  GroupArgs g;
  g.table = reinterpret_cast<const int4*>(table.data_ptr<int>());
  g.count = count.data_ptr<int>();
  g.ragged_m = (int)M;
  g.accumulate = accumulate ? 1 : 0;
  // K is only used for the split-K bookkeeping, which this mode does not use (one slice)
  if (out.scalar_type() == at::kFloat)
    launch_gemm<float, 256, 1, 1>(a.get_device(), grid, st, tmA, tmB, out.data_ptr<float>(), nullptr, capacity * BM, (int)N, (int)R,
                                  (int)N, 1, g);
  else
    launch_gemm<bf16, 256, 1, 1>(a.get_device(), grid, st, tmA, tmB, (bf16*)out.data_ptr(), nullptr, capacity * BM, (int)N, (int)R,
                                 (int)N, 1, g);
  return out;
}

// Grouped GEMM over a caller-built tile table (rows {first, end, first B row, -} as above; `count`
// on the device), written into `out` [R, N]: used where the groups are regions of a receive
// buffer rather than back-to-back rows (expert-parallel dispatch into peer memory).
void grouped_gemm_bf16_nt_table(const at::Tensor& a, const at::Tensor& b, const at::Tensor& table, const at::Tensor& count,
                                at::Tensor out) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16,
              "grouped_gemm_table: bf16 CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3 && a.size(1) == b.size(2) && a.is_contiguous() && b.is_contiguous() && out.is_contiguous(),
              "grouped_gemm_table: A [R, K], B [G, N, K], contiguous");
  const int64_t R = a.size(0), K = a.size(1), G = b.size(0), N = b.size(1);
  TORCH_CHECK(out.dim() == 2 && out.size(0) == R && out.size(1) == N, "grouped_gemm_table: out [R, N]");
  TORCH_CHECK(table.scalar_type() == at::kInt && table.dim() == 2 && table.size(1) == 4 && count.scalar_type() == at::kInt,
              "grouped_gemm_table: int32 table [tiles, 4] and count");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0 && K > 0, "grouped_gemm_table: K and N must be multiples of 8");
  const int capacity = (int)table.size(0);
  if (R == 0 || capacity == 0) return;
  bind_context_to_thread(a.get_device());
  auto st = at::cuda::getCurrentCUDAStream();
  CUtensorMap tmA = make_tmap_bf16(a.data_ptr(), R, K, K, BM);
  CUtensorMap tmB = make_tmap_bf16(b.data_ptr(), G * N, K, K, BN);
  const int num_sms = device_sms(a.get_device());
  const int tiles_n = (int)((N + BN - 1) / BN);
  const int grid = std::min(capacity * tiles_n, num_sms);
  GroupArgs g;
  g.table = reinterpret_cast<const int4*>(table.data_ptr<int>());
  g.count = count.data_ptr<int>();
  launch_gemm<bf16, 256, 0, 0>(a.get_device(), grid, st, tmA, tmB, (bf16*)out.data_ptr(), nullptr, capacity * BM, (int)N, (int)K,
                               (int)N, 1, g);
}

// ----------------------------------------------------------------------------
// Allocation-free entry point (see gemm_noalloc.h): same kernel, split-K planes in a
// fixed file-scope device array instead of a workspace from the allocator.
// ----------------------------------------------------------------------------
#include <mutex>

#include "gemm_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[CLB200_NOALLOC_SCRATCH_FLOATS];

namespace {

struct NoAllocDevice {
  float* scratch = nullptr;   // device address of g_noalloc_scratch on this device
  int num_sms = 0;
  int rc = 0;                 // outcome of the one-time set-up (0 = ready)
  char err[200] = "";
  std::once_flag once;        // host threads that make their first call together set up once
};
NoAllocDevice g_noalloc_dev[64];
thread_local char g_noalloc_err[320] = "";

int noalloc_fail(int code, const char* fmt, long long a = 0, long long b = 0, long long c = 0) {
  std::snprintf(g_noalloc_err, sizeof(g_noalloc_err), fmt, a, b, c);
  return code;
}

// In host code the array's name is only a handle: the address a kernel can use comes
// from cudaGetSymbolAddress, once per device, with that device current.
void noalloc_setup_once(int dev) {
  NoAllocDevice& d = g_noalloc_dev[dev];
  auto fail = [&](int code, const char* what, cudaError_t e) {
    d.rc = code;
    std::snprintf(d.err, sizeof(d.err), "%s failed on device %d: error %d", what, dev, (int)e);
  };
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
  if (e != cudaSuccess || p == nullptr) return fail(10, "cudaGetSymbolAddress(scratch)", e);
  e = cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return fail(11, "cudaDeviceGetAttribute", e);
  const int smem = (int)(sizeof(SmemLayout) + 1024);
  e = cudaFuncSetAttribute(gemm_bf16_nt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemm_bf16_nt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(12, "cudaFuncSetAttribute", e);
  d.scratch = static_cast<float*>(p);
}

int noalloc_setup(int dev) {
  NoAllocDevice& d = g_noalloc_dev[dev];
  std::call_once(d.once, noalloc_setup_once, dev);
  if (d.rc) { std::snprintf(g_noalloc_err, sizeof(g_noalloc_err), "%s", d.err); return d.rc; }
  return 0;
}

bool noalloc_tmap(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaDriverEntryPointQueryResult q;
    void* p = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess && p)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)(ld * 2)};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" const char* clb200_gemm_noalloc_last_error(void) { return g_noalloc_err; }

extern "C" int clb200_gemm_noalloc_device_status(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0 && cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

extern "C" int clb200_gemm_bf16_nt_noalloc(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                                           int ldb, int out_fp32, void* stream) {
  g_noalloc_err[0] = '\0';
  if (!a || !b || !c) return noalloc_fail(1, "null pointer argument");
  if (M <= 0 || N <= 0 || K <= 0) return noalloc_fail(2, "M, N, K must be positive (got %lld, %lld, %lld)", M, N, K);
  if (K % 8 || N % 8 || lda % 8 || ldb % 8 || lda < K || ldb < K)
    return noalloc_fail(3, "K, N and the row strides must be multiples of 8 and lda, ldb >= K");
  if (((uintptr_t)a % 16) || ((uintptr_t)b % 16) || ((uintptr_t)c % 16))
    return noalloc_fail(4, "a, b and c must be 16-byte aligned");
  if (2ll * M * N > CLB200_NOALLOC_SCRATCH_FLOATS)
    return noalloc_fail(5, "problem too large for the built-in scratch: 2*M*N = %lld floats > %lld",
                        2ll * M * N, (long long)CLB200_NOALLOC_SCRATCH_FLOATS);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return noalloc_fail(6, "cudaGetDevice failed");
  if (dev < 0 || dev >= 64) return noalloc_fail(9, "device index %lld is beyond the 64 devices this entry point keeps state for", dev);
  {
    // a host thread that has made no runtime call yet has no context bound, and the driver call that
    // encodes the tensor maps needs one; re-selecting the current device binds it and allocates nothing
    thread_local int bound = -1;
    if (bound != dev) {
      if (cudaSetDevice(dev) != cudaSuccess) return noalloc_fail(13, "cudaSetDevice(%lld) failed", dev);
      bound = dev;
    }
  }
  if (int rc = noalloc_setup(dev)) return rc;
  const NoAllocDevice& d = g_noalloc_dev[dev];
  CUtensorMap tmA, tmB;
  if (!noalloc_tmap(&tmA, a, M, K, lda, BM) || !noalloc_tmap(&tmB, b, N, K, ldb, BN))
    return noalloc_fail(7, "cuTensorMapEncodeTiled rejected the operands");
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int k_iters = (K + BK - 1) / BK;
  // always slice K (that is what the scratch is for); one slice only when K is a single step
  int splits = std::min({std::max((d.num_sms + tiles - 1) / tiles, 2), std::max(k_iters / 2, 1), 16});
  while (splits > 1 && (long long)splits * M * N > CLB200_NOALLOC_SCRATCH_FLOATS) --splits;
  while (splits > 1 && ((k_iters + splits - 1) / splits) * (splits - 1) >= k_iters) --splits;
  const int grid = std::min(tiles * splits, d.num_sms);
  const size_t smem = sizeof(SmemLayout) + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t mn = (int64_t)M * N;
  const int fgrid = (int)std::min<int64_t>((mn / 4 + 255) / 256, 148 * 8);
  (void)cudaGetLastError();      // an error left behind by an earlier, unrelated call must not be blamed on these launches
  if (out_fp32) {
    gemm_bf16_nt_kernel<float><<<grid, kThreads, smem, st>>>(tmA, tmB, static_cast<float*>(c), d.scratch, M, N, K, N, splits, GroupArgs{});
    if (splits > 1) splitk_finalize_kernel<float><<<fgrid, 256, 0, st>>>(d.scratch, static_cast<float*>(c), mn, splits, 0);
  } else {
    gemm_bf16_nt_kernel<bf16><<<grid, kThreads, smem, st>>>(tmA, tmB, static_cast<bf16*>(c), d.scratch, M, N, K, N, splits, GroupArgs{});
    if (splits > 1) splitk_finalize_kernel<bf16><<<fgrid, 256, 0, st>>>(d.scratch, static_cast<bf16*>(c), mn, splits, 0);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail(8, "kernel launch failed: error %lld", (long long)e);
  return 0;
}
