// Paged KV cache kernels of the rollout engine: KV append and decode attention.
//
// Decode attention is bandwidth bound (every step re-reads the whole context), so
// the kernel is built around keeping HBM busy: one CTA per (query token, KV head,
// split) streams the KV blocks of its sequence through a two-stage cp.async ring
// while the previous block is being consumed; all query heads that share the KV
// head (GQA) are served from the same tile, so K/V are read once per group.
// Long contexts are split over several CTAs (flash-decoding) and merged by a
// second kernel.  Replaces the paged-attention kernels of vLLM/SGLang used by the
// reference (chatlearn/models/vllm_module.py:405-407).
#include <ATen/cuda/CUDAContext.h>
#include <cuda_pipeline.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kThreads = 128;
constexpr int kMaxRep = 8;

// ------------------------------------------------------------------ kv append
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, int64_t k_row_stride,
                                 int64_t v_row_stride, T* __restrict__ kc, T* __restrict__ vc,
                                 const int64_t* __restrict__ slots, int k_row, int v_row) {
  const int64_t t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const T* ks = k + t * k_row_stride;
  const T* vs = v + t * v_row_stride;
  T* kd = kc + slot * k_row;
  T* vd = vc + slot * v_row;
  for (int i = threadIdx.x; i < k_row; i += blockDim.x) kd[i] = ks[i];
  for (int i = threadIdx.x; i < v_row; i += blockDim.x) vd[i] = vs[i];
}

// ------------------------------------------------------------------ decode attention
// K tile rows are padded by 8 elements so that 16-byte row reads by consecutive
// threads fall on distinct banks.
template <int DK, int DV, int BS>
struct Smem {
  static constexpr int KP = DK + 8;
  bf16 k[2][BS][KP];
  bf16 v[2][BS][DV];
  float q[kMaxRep][DK];
  float s[kMaxRep][BS];
  float alpha[kMaxRep];
};

template <int DK, int DV, int BS>
__device__ __forceinline__ void load_tile(Smem<DK, DV, BS>* sm, int stage, const bf16* kc, const bf16* vc,
                                          int64_t block_id, int kv_head, int nkv, int valid) {
  // cache layout [num_blocks, BS, nkv, d]
  const bf16* kb = kc + (block_id * BS * nkv + kv_head) * (int64_t)DK;
  const bf16* vb = vc + (block_id * BS * nkv + kv_head) * (int64_t)DV;
  constexpr int KCH = DK / 8, VCH = DV / 8;  // 16-byte chunks per row
  for (int c = threadIdx.x; c < BS * KCH; c += kThreads) {
    const int r = c / KCH, o = (c % KCH) * 8;
    if (r < valid) __pipeline_memcpy_async(&sm->k[stage][r][o], kb + (int64_t)r * nkv * DK + o, 16);
  }
  for (int c = threadIdx.x; c < BS * VCH; c += kThreads) {
    const int r = c / VCH, o = (c % VCH) * 8;
    if (r < valid) __pipeline_memcpy_async(&sm->v[stage][r][o], vb + (int64_t)r * nkv * DV + o, 16);
  }
}

template <int DK, int DV, int BS>
__global__ void __launch_bounds__(kThreads)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                    const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ q_seq,
                    const int* __restrict__ ctx_len, bf16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_lse, int nq, int nkv, int num_splits, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  auto* sm = reinterpret_cast<Smem<DK, DV, BS>*>(smem_raw);
  const int qi = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int rep = nq / nkv;
  const int seq = q_seq ? q_seq[qi] : qi;
  const int L = ctx_len[qi];
  const int nblk = (L + BS - 1) / BS;
  const int per = (nblk + num_splits - 1) / num_splits;
  const int b0 = split * per, b1 = min(b0 + per, nblk);
  const int tid = threadIdx.x;
  const int* bt = block_tables + (int64_t)seq * max_blocks;

  // q for the `rep` heads of this group, pre-scaled
  for (int i = tid; i < rep * DK; i += kThreads) {
    const int r = i / DK, d = i % DK;
    sm->q[r][d] = __bfloat162float(q[((int64_t)qi * nq + kvh * rep + r) * DK + d]) * scale;
  }
  constexpr int kWarps = kThreads / 32;
  constexpr int kOwn = kMaxRep / kWarps;   // heads whose softmax state one warp keeps
  float acc[kMaxRep];
  float m_run[kOwn], l_run[kOwn];          // warp w owns heads w, w + kWarps, ...
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r) acc[r] = 0.f;
#pragma unroll
  for (int i = 0; i < kOwn; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

  if (b0 < b1) {
    load_tile<DK, DV, BS>(sm, 0, kc, vc, bt[b0], kvh, nkv, min(BS, L - b0 * BS));
  }
  __pipeline_commit();
  const int lane = tid & 31, warp = tid >> 5;
  for (int b = b0; b < b1; ++b) {
    const int st = (b - b0) & 1;
    if (b + 1 < b1) load_tile<DK, DV, BS>(sm, st ^ 1, kc, vc, bt[b + 1], kvh, nkv, min(BS, L - (b + 1) * BS));
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const int valid = min(BS, L - b * BS);
    // ---- scores: thread (token, head parity) ----
    {
      const int t = tid % BS, grp = tid / BS;            // kThreads / BS groups of threads per token
      constexpr int G = kThreads / BS;
      for (int r = grp; r < rep; r += G) {
        float dot = -INFINITY;
        if (t < valid) {
          dot = 0.f;
#pragma unroll
          for (int c = 0; c < DK; c += 8) {
            Vec16<bf16> kv = ld16(&sm->k[st][t][c]);
#pragma unroll
            for (int j = 0; j < 8; ++j) dot += sm->q[r][c + j] * __bfloat162float(kv.v[j]);
          }
        }
        sm->s[r][t] = dot;
      }
    }
    __syncthreads();
    // ---- online softmax per head: warp w owns heads w, w+4 ----
#pragma unroll
    for (int i = 0; i < kOwn; ++i) {
      const int r = warp + i * kWarps;
      if (r < rep) {
        float mx = -INFINITY;
        for (int t = lane; t < BS; t += 32) mx = fmaxf(mx, sm->s[r][t]);
        mx = warp_max(mx);
        const float m_new = fmaxf(m_run[i], mx);
        float sum = 0.f;
        for (int t = lane; t < BS; t += 32) {
          const float p = (t < valid) ? __expf(sm->s[r][t] - m_new) : 0.f;
          sm->s[r][t] = p;
          sum += p;
        }
        sum = warp_sum(sum);
        const float a = (m_run[i] == -INFINITY) ? 0.f : __expf(m_run[i] - m_new);
        l_run[i] = l_run[i] * a + sum;
        m_run[i] = m_new;
        if (lane == 0) sm->alpha[r] = a;
      }
    }
    __syncthreads();
    // ---- PV: thread d owns output column d (and d + kThreads, ...) ----
    if (tid < DV) {
#pragma unroll
      for (int r = 0; r < kMaxRep; ++r) {
        if (r < rep) {
          float a = acc[r] * sm->alpha[r];
          for (int t = 0; t < valid; ++t) a += sm->s[r][t] * __bfloat162float(sm->v[st][t][tid]);
          acc[r] = a;
        }
      }
    }
    __syncthreads();
  }
  __pipeline_wait_prior(0);
  // publish l and m of each head (owned by one warp) to everybody
#pragma unroll
  for (int i = 0; i < kOwn; ++i) {
    const int r = warp + i * kWarps;
    if (r < rep && lane == 0) { sm->s[r][0] = l_run[i]; sm->s[r][1] = m_run[i]; }
  }
  __syncthreads();
  if (tid < DV) {
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r) {
      if (r >= rep) break;
      const float l = sm->s[r][0], m = sm->s[r][1];
      const int head = kvh * rep + r;
      if (num_splits == 1) {
        out[((int64_t)qi * nq + head) * DV + tid] = __float2bfloat16_rn(l > 0.f ? acc[r] / l : 0.f);
      } else {
        part_o[(((int64_t)qi * nq + head) * num_splits + split) * DV + tid] = l > 0.f ? acc[r] / l : 0.f;
        if (tid == 0)
          part_lse[((int64_t)qi * nq + head) * num_splits + split] = l > 0.f ? m + logf(l) : -INFINITY;
      }
    }
  }
}

template <int DV>
__global__ void combine_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                      bf16* __restrict__ out, int num_splits) {
  const int64_t qh = blockIdx.x;
  const int d = threadIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, part_lse[qh * num_splits + s]);
  float den = 0.f, o = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float l = part_lse[qh * num_splits + s];
    if (l == -INFINITY) continue;
    const float w = __expf(l - mx);
    den += w;
    if (d < DV) o += w * part_o[(qh * num_splits + s) * DV + d];
  }
  if (d < DV) out[qh * DV + d] = __float2bfloat16_rn(den > 0.f ? o / den : 0.f);
}

template <int DK, int DV, int BS>
void launch_decode(const at::Tensor& q, const at::Tensor& kc, const at::Tensor& vc, const at::Tensor& bt,
                   const int* q_seq, const at::Tensor& ctx_len, at::Tensor& out, int nq, int nkv, int num_splits,
                   float scale) {
  const int Tq = (int)q.size(0);
  auto st = at::cuda::getCurrentCUDAStream();
  const size_t smem = sizeof(Smem<DK, DV, BS>);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(paged_decode_kernel<DK, DV, BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  at::Tensor po, pl;
  float* pop = nullptr; float* plp = nullptr;
  if (num_splits > 1) {
    po = at::empty({Tq, nq, num_splits, DV}, q.options().dtype(at::kFloat));
    pl = at::empty({Tq, nq, num_splits}, q.options().dtype(at::kFloat));
    pop = po.data_ptr<float>(); plp = pl.data_ptr<float>();
  }
  dim3 grid(Tq, nkv, num_splits);
  paged_decode_kernel<DK, DV, BS><<<grid, kThreads, smem, st>>>(
      (const bf16*)q.data_ptr(), (const bf16*)kc.data_ptr(), (const bf16*)vc.data_ptr(), bt.data_ptr<int>(),
      (int)bt.size(1), q_seq, ctx_len.data_ptr<int>(), (bf16*)out.data_ptr(), pop, plp, nq, nkv, num_splits, scale);
  if (num_splits > 1) {
    combine_splits_kernel<DV><<<Tq * nq, ((DV + 31) / 32) * 32, 0, st>>>(pop, plp, (bf16*)out.data_ptr(), num_splits);
  }
}

}  // namespace

void kv_append(const at::Tensor& k, const at::Tensor& v, at::Tensor k_cache, at::Tensor v_cache,
               const at::Tensor& slots) {
  const int64_t Tn = k.size(0);
  if (Tn == 0) return;
  TORCH_CHECK(k.dim() == 3 && v.dim() == 3 && k.stride(2) == 1 && v.stride(2) == 1 &&
              k.stride(1) == k.size(2) && v.stride(1) == v.size(2), "kv_append: [T, nkv, d] rows must be dense");
  TORCH_CHECK(k.scalar_type() == k_cache.scalar_type(), "kv_append: dtype mismatch");
  const int k_row = (int)(k.size(1) * k.size(2)), v_row = (int)(v.size(1) * v.size(2));
  auto st = at::cuda::getCurrentCUDAStream();
  if (k.scalar_type() == at::kBFloat16)
    kv_append_kernel<bf16><<<Tn, 128, 0, st>>>((const bf16*)k.data_ptr(), (const bf16*)v.data_ptr(), k.stride(0),
        v.stride(0), (bf16*)k_cache.data_ptr(), (bf16*)v_cache.data_ptr(), slots.data_ptr<int64_t>(), k_row, v_row);
  else if (k.scalar_type() == at::kFloat)
    kv_append_kernel<float><<<Tn, 128, 0, st>>>(k.data_ptr<float>(), v.data_ptr<float>(), k.stride(0), v.stride(0),
        k_cache.data_ptr<float>(), v_cache.data_ptr<float>(), slots.data_ptr<int64_t>(), k_row, v_row);
  else
    TORCH_CHECK(false, "kv_append: dtype");
}

bool paged_decode_supported(int64_t dk, int64_t dv, int64_t bs, int64_t rep) {
  const bool dims = (dk == 128 && dv == 128) || (dk == 64 && dv == 64) || (dk == 192 && dv == 128);
  return dims && (bs == 64 || bs == 32 || bs == 16) && rep <= kMaxRep;
}

// q [Tq, nq, dk] bf16; caches [nb, bs, nkv, d] bf16; ctx_len[Tq] = keys visible to each
// query token; q_seq[Tq] = sequence (block table row) of each query token (optional).
at::Tensor paged_decode(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                        const at::Tensor& block_tables, const c10::optional<at::Tensor>& q_seq,
                        const at::Tensor& ctx_len, double scale, int64_t num_splits) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous(), "paged_decode: bf16 contiguous q");
  const int nq = (int)q.size(1), dk = (int)q.size(2);
  const int bs = (int)k_cache.size(1), nkv = (int)k_cache.size(2), dv = (int)v_cache.size(3);
  TORCH_CHECK(paged_decode_supported(dk, dv, bs, nq / nkv), "paged_decode: unsupported shape");
  auto out = at::empty({q.size(0), nq, dv}, q.options());
  if (q.size(0) == 0) return out;
  const int* qs = q_seq.has_value() ? q_seq->data_ptr<int>() : nullptr;
  const int ns = (int)std::max<int64_t>(num_splits, 1);
#define CASE(DK_, DV_, BS_) \
  if (dk == DK_ && dv == DV_ && bs == BS_) { launch_decode<DK_, DV_, BS_>(q, k_cache, v_cache, block_tables, qs, ctx_len, out, nq, nkv, ns, (float)scale); return out; }
  CASE(128, 128, 64) CASE(128, 128, 32) CASE(128, 128, 16)
  CASE(64, 64, 64) CASE(64, 64, 32) CASE(64, 64, 16)
  CASE(192, 128, 64) CASE(192, 128, 32) CASE(192, 128, 16)
#undef CASE
  TORCH_CHECK(false, "paged_decode: no kernel instance");
  return out;
}
