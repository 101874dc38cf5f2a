// Collectives executed by this library's own kernels over NVLink peer memory.
//
// Every rank owns buffers in symmetric memory (same size on every rank, mapped into
// every peer's address space); kernels receive a table of the per-rank base
// pointers and read / write peers with ordinary loads and stores.  Synchronisation
// uses flag words in symmetric memory: a sender increments its slot on the peer
// with a system-scope release, the receiver compares the slot with the number of
// rounds it has waited for (kept in its own memory), so no host-side epoch is
// needed and the kernels can be replayed from a CUDA graph.  All waits are bounded
// (2 s): a missing peer produces a status code, not a hang.
//
//   allreduce_oneshot   out = sum over ranks of buf_r          (TP decode all-reduce)
//   rs_pull_sumsq       shard = sum_r grad_r[lo:hi], + sum of squares   (ZeRO reduce-scatter by pulling)
//   adamw_push          AdamW on the shard, new bf16 weights stored into every rank's
//                       parameter buffer (all-gather by pushing)
//
// No TMA, no multicast: peer traffic is plain 16-byte ld/st.global.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kMaxWorld = 8;
constexpr uint64_t kWaitNs = 2000000000ull;

struct PeerTable {
  void* ptr[kMaxWorld];
};

__device__ int g_symm_status = 0;

__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void signal_add(uint32_t* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier instance `slot` among all ranks, executed by the calling CTA.
// flags[r] = base of rank r's flag array, laid out [sender rank][slot].
// expect   = this rank's private round counters, laid out [slot][peer].
// Returns false on timeout.  Must be called by all threads of the CTA.
__device__ bool cta_barrier(const PeerTable& flags, uint32_t* expect, int slot, int num_slots, int rank, int world) {
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();          // everything this CTA wrote before the barrier is ordered before the signal
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const int p = threadIdx.x;
    __threadfence_system();
    signal_add(static_cast<uint32_t*>(flags.ptr[p]) + rank * num_slots + slot);
    const uint32_t want = ++expect[slot * kMaxWorld + p];
    const uint32_t* mine = static_cast<const uint32_t*>(flags.ptr[rank]) + p * num_slots + slot;
    const uint64_t t0 = gtimer();
    bool ok = true;
    // signed distance handles counter wrap-around
    while ((int32_t)(load_acquire(mine) - want) < 0) {
      if (gtimer() - t0 > kWaitNs) { ok = false; break; }
    }
    if (!ok) { ok_sh = 0; atomicCAS(&g_symm_status, 0, 1 + slot % 1000); }
  }
  __syncthreads();
  return ok_sh != 0;
}

// ------------------------------------------------------------------ one-shot all-reduce
template <typename T>
__global__ void allreduce_oneshot_kernel(PeerTable bufs, PeerTable flags, uint32_t* expect, T* __restrict__ out,
                                         int64_t n, int rank, int world, int num_slots) {
  const int slot = blockIdx.x;
  if (!cta_barrier(flags, expect, slot, num_slots, rank, world)) return;
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    for (int r = 0; r < world; ++r) {           // fixed order: every rank gets bit-identical sums
      Vec16<T> x = ld16(static_cast<const T*>(bufs.ptr[r]) + v * V);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += Cvt<T>::to_f(x.v[j]);
    }
    Vec16<T> o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(acc[j]);
    st16(out + v * V, o);
  }
  for (int64_t i = nvec * V + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int r = 0; r < world; ++r) a += Cvt<T>::to_f(static_cast<const T*>(bufs.ptr[r])[i]);
    out[i] = Cvt<T>::from_f(a);
  }
  // nobody may overwrite its buffer until every peer has finished reading it
  cta_barrier(flags, expect, num_slots / 2 + slot, num_slots, rank, world);
}

// ------------------------------------------------------------------ ZeRO step, phase A
// shard[i] = sum_r grad_r[lo + i]  (fp32), partial sums of squares per CTA.
__global__ void rs_pull_sumsq_kernel(PeerTable grads, PeerTable flags, uint32_t* expect, float* __restrict__ shard,
                                     float* __restrict__ partial_sq, int64_t lo, int64_t n, int rank, int world,
                                     int num_slots) {
  __shared__ float red[32];
  const int slot = blockIdx.x;
  if (!cta_barrier(flags, expect, slot, num_slots, rank, world)) return;
  float sq = 0.f;
  const int64_t nvec = n / 4;
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(static_cast<const float*>(grads.ptr[r]) + lo + v * 4);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
    }
    *reinterpret_cast<float4*>(shard + v * 4) = a;
    sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  sq = block_sum(sq, red);
  if (threadIdx.x == 0) partial_sq[blockIdx.x] = sq;
  cta_barrier(flags, expect, num_slots / 2 + slot, num_slots, rank, world);
}

// ------------------------------------------------------------------ ZeRO step, phase B
// AdamW on the fp32 shard; the new weights are cast and stored to every rank's
// parameter buffer at [lo, lo+n) (this is the all-gather).
template <typename P>
__global__ void adamw_push_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                                  float* __restrict__ v, PeerTable params, PeerTable flags, uint32_t* expect,
                                  int64_t lo, int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1,
                                  float bc2, const float* __restrict__ scale_ptr, int rank, int world, int num_slots) {
  const float scale = scale_ptr ? *scale_ptr : 1.f;
  for (int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4; i + 4 <= n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    float4 g4 = *reinterpret_cast<const float4*>(grad + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i), v4 = *reinterpret_cast<float4*>(v + i);
    float4 p4 = *reinterpret_cast<float4*>(master + i);
    float* g = &g4.x; float* mm = &m4.x; float* vv = &v4.x; float* pp = &p4.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * scale;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      pp[j] = pp[j] * (1.f - lr * wd) - lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
    }
    *reinterpret_cast<float4*>(m + i) = m4;
    *reinterpret_cast<float4*>(v + i) = v4;
    *reinterpret_cast<float4*>(master + i) = p4;
    if (sizeof(P) == 2) {
      __nv_bfloat162 a = __floats2bfloat162_rn(pp[0], pp[1]), b = __floats2bfloat162_rn(pp[2], pp[3]);
      const uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(static_cast<bf16*>(params.ptr[r]) + lo + i) = pk;
    } else {
      for (int r = 0; r < world; ++r) *reinterpret_cast<float4*>(static_cast<float*>(params.ptr[r]) + lo + i) = p4;
    }
  }
  // the pushed weights must be visible on every rank before anyone uses them
  cta_barrier(flags, expect, blockIdx.x, num_slots, rank, world);
}

// ------------------------------------------------------------------ TP epilogue of a row-parallel GEMM
// parts_r [T, H] = rank r's partial product (in symmetric memory).  One pass does
//   resid += sum_r parts_r            (new residual stream, rounded to bf16)
//   hout   = rmsnorm(resid) * w       (input of the next GEMM; skipped when w == nullptr)
// i.e. all-reduce + residual add + RMSNorm without the reduced tensor ever going
// to memory.  Only an entry barrier: callers alternate between two staging buffers,
// so a rank that passed the entry barrier of call k+1 has finished reading call k's
// buffer before any peer can overwrite it in call k+2.
template <int VPT>
__global__ void ar_residual_rmsnorm_kernel(PeerTable parts, PeerTable flags, uint32_t* expect, bf16* __restrict__ resid,
                                           const bf16* __restrict__ w, bf16* __restrict__ hout, int T, int H,
                                           float eps, int rank, int world, int num_slots, int slot_base) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  if (!cta_barrier(flags, expect, slot_base + blockIdx.x, num_slots, rank, world)) return;
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float val[VPT][8];
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        const int64_t off = (int64_t)row * H + v * 8;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < world; ++r) {        // fixed order: bit-identical on every rank
          Vec16<bf16> x = ld16(static_cast<const bf16*>(parts.ptr[r]) + off);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(x.v[j]);
        }
        Vec16<bf16> rs = ld16(resid + off), o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o.v[j] = __float2bfloat16(acc[j] + __bfloat162float(rs.v[j]));
          val[k][j] = __bfloat162float(o.v[j]);
          sq += val[k][j] * val[k][j];
        }
        st16(resid + off, o);
      }
    }
    if (w != nullptr) {
      sq = block_sum(sq, red);
      const float inv = rsqrtf(sq / H + eps);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * blockDim.x;
        if (v < nvec) {
          Vec16<bf16> ww = ld16(w + v * 8), o;
#pragma unroll
          for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(val[k][j] * inv * __bfloat162float(ww.v[j]));
          st16(hout + (int64_t)row * H + v * 8, o);
        }
      }
    }
  }
}

PeerTable table_from(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= kMaxWorld, "at most 8 ranks");
  PeerTable t;
  for (int i = 0; i < kMaxWorld; ++i) t.ptr[i] = i < (int)ptrs.size() ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

}  // namespace

// num_slots = slots per sender in the flag arrays (>= 2 * grid); expect: uint32 [num_slots, 8] zero-initialised.
void symm_allreduce(const std::vector<int64_t>& buf_ptrs, const std::vector<int64_t>& flag_ptrs, at::Tensor expect,
                    at::Tensor out, int64_t n, int64_t rank, int64_t num_slots) {
  const int world = (int)buf_ptrs.size();
  const int max_grid = (int)num_slots / 2;
  auto st = at::cuda::getCurrentCUDAStream();
  const int esz = (int)out.element_size();
  int grid = (int)std::min<int64_t>(std::max<int64_t>((n * esz / 16 + 255) / 256, 1), std::min(max_grid, 148));
  auto* ex = reinterpret_cast<uint32_t*>(expect.data_ptr());
  if (out.scalar_type() == at::kBFloat16)
    allreduce_oneshot_kernel<bf16><<<grid, 256, 0, st>>>(table_from(buf_ptrs), table_from(flag_ptrs), ex,
                                                        (bf16*)out.data_ptr(), n, (int)rank, world, (int)num_slots);
  else if (out.scalar_type() == at::kFloat)
    allreduce_oneshot_kernel<float><<<grid, 256, 0, st>>>(table_from(buf_ptrs), table_from(flag_ptrs), ex,
                                                         out.data_ptr<float>(), n, (int)rank, world, (int)num_slots);
  else
    TORCH_CHECK(false, "symm_allreduce: bf16 or fp32");
}

// Returns the per-CTA partial sums of squares of the reduced shard.
at::Tensor symm_rs_pull_sumsq(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& flag_ptrs,
                              at::Tensor expect, at::Tensor shard, int64_t lo, int64_t rank, int64_t num_slots) {
  const int world = (int)grad_ptrs.size();
  const int64_t n = shard.numel();
  TORCH_CHECK(n % 4 == 0 && lo % 4 == 0, "shard size and offset must be multiples of 4");
  const int grid = (int)std::min<int64_t>(std::max<int64_t>((n / 4 + 255) / 256, 1), std::min<int64_t>(num_slots / 2, 148 * 2));
  auto part = at::zeros({grid}, shard.options());
  rs_pull_sumsq_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      table_from(grad_ptrs), table_from(flag_ptrs), reinterpret_cast<uint32_t*>(expect.data_ptr()),
      shard.data_ptr<float>(), part.data_ptr<float>(), lo, n, (int)rank, world, (int)num_slots);
  return part;
}

void symm_adamw_push(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                     const std::vector<int64_t>& param_ptrs, const std::vector<int64_t>& flag_ptrs, at::Tensor expect,
                     int64_t lo, bool params_bf16, int64_t step, double lr, double b1, double b2, double eps, double wd,
                     const c10::optional<at::Tensor>& scale, int64_t rank, int64_t num_slots) {
  const int world = (int)param_ptrs.size();
  const int64_t n = master.numel();
  TORCH_CHECK(n % 4 == 0 && lo % 4 == 0, "shard size and offset must be multiples of 4");
  const float bc1 = (float)(1.0 - std::pow(b1, (double)step)), bc2 = (float)(1.0 - std::pow(b2, (double)step));
  const int grid = (int)std::min<int64_t>(std::max<int64_t>((n / 4 + 255) / 256, 1), std::min<int64_t>(num_slots / 2, 148 * 2));
  const float* sp = scale.has_value() ? scale->data_ptr<float>() : nullptr;
  auto st = at::cuda::getCurrentCUDAStream();
  auto* ex = reinterpret_cast<uint32_t*>(expect.data_ptr());
  if (params_bf16)
    adamw_push_kernel<bf16><<<grid, 256, 0, st>>>(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(),
        v.data_ptr<float>(), table_from(param_ptrs), table_from(flag_ptrs), ex, lo, n, (float)lr, (float)b1, (float)b2,
        (float)eps, (float)wd, bc1, bc2, sp, (int)rank, world, (int)num_slots);
  else
    adamw_push_kernel<float><<<grid, 256, 0, st>>>(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(),
        v.data_ptr<float>(), table_from(param_ptrs), table_from(flag_ptrs), ex, lo, n, (float)lr, (float)b1, (float)b2,
        (float)eps, (float)wd, bc1, bc2, sp, (int)rank, world, (int)num_slots);
}

// resid [T, H] bf16 (updated in place); part_ptrs = every rank's partial [T, H] bf16; w [H] or undefined.
// Returns hout (undefined tensor when w is absent).
at::Tensor symm_ar_residual_rmsnorm(const std::vector<int64_t>& part_ptrs, const std::vector<int64_t>& flag_ptrs,
                                    at::Tensor expect, at::Tensor resid, const c10::optional<at::Tensor>& w, double eps,
                                    int64_t rank, int64_t num_slots) {
  const int world = (int)part_ptrs.size();
  TORCH_CHECK(resid.scalar_type() == at::kBFloat16 && resid.is_contiguous() && resid.dim() == 2, "resid: contiguous bf16 [T, H]");
  const int T = (int)resid.size(0), H = (int)resid.size(1);
  TORCH_CHECK(H % 8 == 0 && H <= 256 * 8 * 4, "hidden size must be a multiple of 8 and at most 8192");
  at::Tensor hout;
  const bf16* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kBFloat16 && w->numel() == H && w->is_contiguous(), "w: bf16 [H]");
    hout = at::empty_like(resid);
    wp = (const bf16*)w->data_ptr();
  }
  if (T == 0) return hout;
  const int grid = std::min(T, std::min((int)num_slots / 2, 148 * 2));
  const int vpt = (H / 8 + 255) / 256;
  auto st = at::cuda::getCurrentCUDAStream();
  auto* ex = reinterpret_cast<uint32_t*>(expect.data_ptr());
  bf16* hp = hout.defined() ? (bf16*)hout.data_ptr() : nullptr;
#define LAUNCH_AR(VPT)                                                                                              \
  ar_residual_rmsnorm_kernel<VPT><<<grid, 256, 0, st>>>(table_from(part_ptrs), table_from(flag_ptrs), ex,           \
      (bf16*)resid.data_ptr(), wp, hp, T, H, (float)eps, (int)rank, world, (int)num_slots, 0)
  if (vpt <= 1) LAUNCH_AR(1);
  else if (vpt == 2) LAUNCH_AR(2);
  else LAUNCH_AR(4);
#undef LAUNCH_AR
  return hout;
}

// ------------------------------------------------------------------ all-gather / all-to-all by pushing
// Chunk p of `src` (chunk 0 for an all-gather) goes to slot `rank` of peer p's exchange buffer:
// plain 16-byte stores over NVLink, one grid column per destination.  The caller brackets the
// kernel with a flag barrier and copies its own buffer out afterwards.
__global__ void push_chunks_kernel(const uint4* __restrict__ src, PeerTable dst, int64_t chunk_vec, int64_t src_stride_vec,
                                   int rank, int world) {
  const int p = blockIdx.y;
  if (p >= world) return;
  const uint4* s = src + (int64_t)p * src_stride_vec;
  uint4* d = static_cast<uint4*>(dst.ptr[p]) + (int64_t)rank * chunk_vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < chunk_vec; i += (int64_t)gridDim.x * blockDim.x) d[i] = s[i];
}

__global__ void group_barrier_kernel(PeerTable flags, uint32_t* expect, int slot, int num_slots, int rank, int world) {
  cta_barrier(flags, expect, slot, num_slots, rank, world);
}

// src: contiguous bytes; all_to_all: `world` chunks of chunk_bytes each (chunk p -> peer p); all-gather: one chunk.
void symm_push_chunks(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs, int64_t chunk_bytes, bool all_to_all,
                      int64_t rank) {
  const int world = (int)dst_ptrs.size();
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && chunk_bytes % 16 == 0 && (uintptr_t)src.data_ptr() % 16 == 0,
              "push_chunks: contiguous, 16-byte aligned, chunk a multiple of 16 bytes");
  TORCH_CHECK((int64_t)src.numel() * src.element_size() >= chunk_bytes * (all_to_all ? world : 1), "push_chunks: source too small");
  if (chunk_bytes == 0) return;
  const int64_t vec = chunk_bytes / 16;
  const int gx = (int)std::min<int64_t>((vec + 255) / 256, 148 * 4 / world + 1);
  push_chunks_kernel<<<dim3(gx, world), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      static_cast<const uint4*>(src.data_ptr()), table_from(dst_ptrs), vec, all_to_all ? vec : 0, (int)rank, world);
}

void symm_group_barrier(const std::vector<int64_t>& flag_ptrs, at::Tensor expect, int64_t slot, int64_t num_slots, int64_t rank) {
  group_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(table_from(flag_ptrs), reinterpret_cast<uint32_t*>(expect.data_ptr()),
                                                                      (int)slot, (int)num_slots, (int)rank, (int)flag_ptrs.size());
}

// out[i] = sum over the `world` chunks of buf (chunk stride n elements), fp32 accumulation in a fixed order:
// the owner's side of a reduce-scatter whose chunks were pushed into its receive buffer.
__global__ void sum_slots_kernel(const bf16* __restrict__ buf, int world, int64_t n, bf16* __restrict__ out) {
  for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v * 8 < n; v += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < world; ++r) {
      Vec16<bf16> x = ld16(buf + (int64_t)r * n + v * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(x.v[j]);
    }
    Vec16<bf16> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(acc[j]);
    st16(out + v * 8, o);
  }
}

// buf: this rank's receive buffer holding `world` chunks of rows x cols bf16 values back to back.
at::Tensor symm_sum_slots(const at::Tensor& buf, int64_t world, int64_t rows, int64_t cols) {
  const int64_t n = rows * cols;
  TORCH_CHECK(buf.is_cuda() && buf.is_contiguous() && (int64_t)buf.numel() * buf.element_size() >= world * n * 2 && n % 8 == 0 &&
                  (uintptr_t)buf.data_ptr() % 16 == 0, "sum_slots: contiguous buffer of world chunks, chunk a multiple of 8 elements");
  auto out = at::empty({rows, cols}, buf.options().dtype(at::kBFloat16));
  if (n == 0) return out;
  const int grid = (int)std::min<int64_t>((n / 8 + 255) / 256, 148 * 8);
  sum_slots_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>((const bf16*)buf.data_ptr(), (int)world, n, (bf16*)out.data_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// resid += sum of the K-slice planes of a GEMM (fp32 [S, T, H], rounded to bf16 first, as the finalize kernel would);
// returns rmsnorm(resid) * w.  Consumes the planes of gemm_bf16_nt_planes without the finalize launch in between.
template <int VPT>
__global__ void planes_residual_rmsnorm_kernel(const float* __restrict__ planes, int S, int64_t plane_stride,
                                               bf16* __restrict__ resid, const bf16* __restrict__ w, bf16* __restrict__ hout,
                                               int T, int H, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    float val[VPT][8];
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        const int64_t off = (int64_t)row * H + v * 8;
        float acc[8];
        {
          const float4 a0 = *reinterpret_cast<const float4*>(planes + off), a1 = *reinterpret_cast<const float4*>(planes + off + 4);
          acc[0] = a0.x; acc[1] = a0.y; acc[2] = a0.z; acc[3] = a0.w; acc[4] = a1.x; acc[5] = a1.y; acc[6] = a1.z; acc[7] = a1.w;
        }
        for (int s = 1; s < S; ++s) {
          const float* ps = planes + (int64_t)s * plane_stride + off;
          const float4 a0 = *reinterpret_cast<const float4*>(ps), a1 = *reinterpret_cast<const float4*>(ps + 4);
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w; acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
        }
        Vec16<bf16> rs = ld16(resid + off), o;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = __bfloat162float(__float2bfloat16_rn(acc[j]));        // what the finalize kernel would have stored
          o.v[j] = __float2bfloat16(d + __bfloat162float(rs.v[j]));
          val[k][j] = __bfloat162float(o.v[j]);
          sq += val[k][j] * val[k][j];
        }
        st16(resid + off, o);
      }
    }
    if (w == nullptr) continue;
    sq = block_sum(sq, red);
    const float r = rsqrtf(sq / H + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * blockDim.x;
      if (v < nvec) {
        const int64_t off = (int64_t)row * H + v * 8;
        Vec16<bf16> ww = ld16(w + v * 8), o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(val[k][j] * r * __bfloat162float(ww.v[j]));
        st16(hout + off, o);
      }
    }
  }
}

at::Tensor planes_residual_rmsnorm(at::Tensor resid, const at::Tensor& planes, const c10::optional<at::Tensor>& w, double eps) {
  TORCH_CHECK(resid.scalar_type() == at::kBFloat16 && resid.is_contiguous() && resid.dim() == 2, "resid: contiguous bf16 [T, H]");
  TORCH_CHECK(planes.scalar_type() == at::kFloat && planes.dim() == 3 && planes.is_contiguous() && planes.size(1) == resid.size(0) &&
                  planes.size(2) == resid.size(1) && planes.size(0) >= 1, "planes: contiguous fp32 [S, T, H]");
  const int T = (int)resid.size(0), H = (int)resid.size(1), S = (int)planes.size(0);
  TORCH_CHECK(H % 8 == 0 && H <= 256 * 8 * 4, "hidden size must be a multiple of 8 and at most 8192");
  at::Tensor hout;
  const bf16* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kBFloat16 && w->numel() == H && w->is_contiguous(), "w: bf16 [H]");
    hout = at::empty_like(resid);
    wp = (const bf16*)w->data_ptr();
  }
  if (T == 0) return hout;
  const int grid = std::min(T, 148 * 4);
  const int vpt = (H / 8 + 255) / 256;
  auto st = at::cuda::getCurrentCUDAStream();
  bf16* hp = hout.defined() ? (bf16*)hout.data_ptr() : nullptr;
#define CLB_PRN(VPT)                                                                                                        \
  C10_CUDA_CHECK(launch_pdl(planes_residual_rmsnorm_kernel<VPT>, dim3(grid), dim3(256), 0, st, planes.data_ptr<float>(), S, \
                            (int64_t)T * H, (bf16*)resid.data_ptr(), wp, hp, T, H, (float)eps))
  if (vpt <= 1) CLB_PRN(1);
  else if (vpt == 2) CLB_PRN(2);
  else CLB_PRN(4);
#undef CLB_PRN
  return hout;
}

// Single-rank form of the kernel above: resid += delta; returns rmsnorm(resid) * w (undefined when w is absent).
at::Tensor add_residual_rmsnorm(at::Tensor resid, const at::Tensor& delta, const c10::optional<at::Tensor>& w, double eps) {
  TORCH_CHECK(resid.scalar_type() == at::kBFloat16 && resid.is_contiguous() && resid.dim() == 2, "resid: contiguous bf16 [T, H]");
  TORCH_CHECK(delta.scalar_type() == at::kBFloat16 && delta.is_contiguous() && delta.sizes() == resid.sizes(), "delta: same shape as resid");
  const int T = (int)resid.size(0), H = (int)resid.size(1);
  TORCH_CHECK(H % 8 == 0 && H <= 256 * 8 * 4, "hidden size must be a multiple of 8 and at most 8192");
  at::Tensor hout;
  const bf16* wp = nullptr;
  if (w.has_value()) {
    TORCH_CHECK(w->scalar_type() == at::kBFloat16 && w->numel() == H && w->is_contiguous(), "w: bf16 [H]");
    hout = at::empty_like(resid);
    wp = (const bf16*)w->data_ptr();
  }
  if (T == 0) return hout;
  PeerTable parts, flags;
  for (int i = 0; i < kMaxWorld; ++i) { parts.ptr[i] = nullptr; flags.ptr[i] = nullptr; }
  parts.ptr[0] = delta.data_ptr();
  const int grid = std::min(T, 148 * 4);
  const int vpt = (H / 8 + 255) / 256;
  auto st = at::cuda::getCurrentCUDAStream();
  bf16* hp = hout.defined() ? (bf16*)hout.data_ptr() : nullptr;
  // world = 1: the barrier inside the kernel touches neither the flag table nor the counters
#define CLB_ARN(VPT)                                                                                                      \
  C10_CUDA_CHECK(launch_pdl(ar_residual_rmsnorm_kernel<VPT>, dim3(grid), dim3(256), 0, st, parts, flags, (uint32_t*)nullptr, \
                            (bf16*)resid.data_ptr(), wp, hp, T, H, (float)eps, 0, 1, 1, 0))
  if (vpt <= 1) CLB_ARN(1);
  else if (vpt == 2) CLB_ARN(2);
  else CLB_ARN(4);
#undef CLB_ARN
  return hout;
}

int64_t symm_last_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_symm_status, sizeof(int));
  int zero = 0;
  cudaMemcpyToSymbol(g_symm_status, &zero, sizeof(int));
  return v;
}
