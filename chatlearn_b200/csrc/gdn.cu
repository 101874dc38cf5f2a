// Gated delta-net decode step (Qwen3-Next linear-attention layers): one new token per sequence.
//
//   S <- exp(g) S;  d = beta (v - k^T S);  S <- S + k d^T;  o = q^T S
//
// with q and k L2-normalised (q also scaled by dk^-1/2) inside the kernel, the key head of a value
// head taken by integer division (grouped heads), the state addressed through a slot table and
// treated as zero for sequences that start fresh.  The state ([slots, heads, dk, dv] fp32) is read
// once from DRAM and written once.  One CTA per (value head, sequence); thread j owns column j of the
// state and, for dk 64 and 128, keeps it in registers between the read-out of the memory and the update.
// The reference runs this through the flash-linear-attention Triton kernels called by the HF module
// (chatlearn/models/patches/transformers/qwen3_next_moe_patch.py patches only the MoE block).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

namespace {

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }

// Loads q and k of this CTA's key head into shared memory, L2-normalised (q also scaled).
template <typename T>
__device__ __forceinline__ void load_qk(const T* __restrict__ qrow, const T* __restrict__ krow, float* qs, float* ks,
                                        int dk, float scale) {
  __shared__ float red[2][4];
  const int tid = threadIdx.x;
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < dk; i += blockDim.x) {
    const float a = to_f(qrow[i]), c = to_f(krow[i]);
    qs[i] = a;
    ks[i] = c;
    sq += a * a;
    sk += c * c;
  }
  for (int o = 16; o > 0; o >>= 1) {
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
    sk += __shfl_xor_sync(0xffffffffu, sk, o);
  }
  if ((tid & 31) == 0) { red[0][tid >> 5] = sq; red[1][tid >> 5] = sk; }
  __syncthreads();
  const int nw = blockDim.x >> 5;
  sq = 0.f; sk = 0.f;
  for (int w = 0; w < nw; ++w) { sq += red[0][w]; sk += red[1][w]; }
  const float qinv = rsqrtf(sq + 1e-6f) * scale, kinv = rsqrtf(sk + 1e-6f);
  for (int i = tid; i < dk; i += blockDim.x) { qs[i] *= qinv; ks[i] *= kinv; }
  __syncthreads();
}

// DK > 0: the state column of a thread stays in registers (all its loads in flight at once, one sweep of
// loads and one of stores).  DK == 0: any dk, two sweeps over the column (the second one hits cache).
template <typename T, int DK>
__global__ void __launch_bounds__(128)
gdn_decode_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  const int64_t* __restrict__ slots, const bool* __restrict__ fresh, float* __restrict__ out,
                  int nk, int nv, int dk, int dv, float scale) {
  extern __shared__ float sm[];
  float* qs = sm;
  float* ks = sm + dk;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int hk = h / (nv / nk);
  load_qk(q + ((int64_t)b * nk + hk) * dk, k + ((int64_t)b * nk + hk) * dk, qs, ks, dk, scale);

  const bool fr = fresh[b];
  const float decay = __expf(g[(int64_t)b * nv + h]);
  const float bt = beta[(int64_t)b * nv + h];
  float* S = state + (((int64_t)slots[b] * nv + h) * dk) * (int64_t)dv;
  for (int j = tid; j < dv; j += blockDim.x) {
    const float vj = to_f(v[((int64_t)b * nv + h) * dv + j]);
    float o = 0.f;
    if constexpr (DK > 0) {
      float s[DK];
#pragma unroll
      for (int i = 0; i < DK; ++i) s[i] = fr ? 0.f : S[(int64_t)i * dv + j];
      float mem = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) mem += s[i] * ks[i];
      const float delta = (vj - mem * decay) * bt;
#pragma unroll
      for (int i = 0; i < DK; ++i) {
        const float t = s[i] * decay + ks[i] * delta;
        S[(int64_t)i * dv + j] = t;
        o += t * qs[i];
      }
    } else {
      float mem = 0.f;
      if (!fr)
        for (int i = 0; i < dk; ++i) mem += S[(int64_t)i * dv + j] * ks[i];
      const float delta = (vj - mem * decay) * bt;
      for (int i = 0; i < dk; ++i) {
        const float s0 = fr ? 0.f : S[(int64_t)i * dv + j] * decay;
        const float t = s0 + ks[i] * delta;
        S[(int64_t)i * dv + j] = t;
        o += t * qs[i];
      }
    }
    out[((int64_t)b * nv + h) * dv + j] = o;
  }
}

}  // namespace

// q, k: [B, nk, dk]; v: [B, nv, dv] (bf16 or fp32, contiguous); g, beta: [B, nv] fp32;
// state: [slots, nv, dk, dv] fp32, updated in place; slots: [B] int64; fresh: [B] bool.  Returns o [B, nv, dv] fp32.
at::Tensor gdn_decode_step(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g,
                           const at::Tensor& beta, at::Tensor state, const at::Tensor& slots, const at::Tensor& fresh,
                           double scale) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.sizes() == q.sizes() && v.dim() == 3 && state.dim() == 4, "gdn_decode_step: shapes");
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && g.is_contiguous() && beta.is_contiguous() &&
              state.is_contiguous() && slots.is_contiguous() && fresh.is_contiguous(), "gdn_decode_step: contiguous inputs");
  TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == v.scalar_type(), "gdn_decode_step: q, k, v of one dtype");
  TORCH_CHECK(g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && state.scalar_type() == at::kFloat &&
              slots.scalar_type() == at::kLong && fresh.scalar_type() == at::kBool, "gdn_decode_step: dtypes");
  const int B = (int)q.size(0), nk = (int)q.size(1), dk = (int)q.size(2), nv = (int)v.size(1), dv = (int)v.size(2);
  TORCH_CHECK(nv % nk == 0 && state.size(1) == nv && state.size(2) == dk && state.size(3) == dv && g.numel() == (int64_t)B * nv &&
              beta.numel() == (int64_t)B * nv && slots.numel() == B && fresh.numel() == B && B <= 65535, "gdn_decode_step: sizes");
  auto out = at::empty({B, nv, dv}, q.options().dtype(at::kFloat));
  if (B == 0) return out;
  const dim3 grid(nv, B);
  const size_t smem = 2 * (size_t)dk * sizeof(float);
  auto st = at::cuda::getCurrentCUDAStream();
#define GDN_LAUNCH(T_, DK_)                                                                                   \
  gdn_decode_kernel<T_, DK_><<<grid, 128, smem, st>>>(                                                         \
      (const T_*)q.data_ptr(), (const T_*)k.data_ptr(), (const T_*)v.data_ptr(), g.data_ptr<float>(),          \
      beta.data_ptr<float>(), state.data_ptr<float>(), slots.data_ptr<int64_t>(), fresh.data_ptr<bool>(),      \
      out.data_ptr<float>(), nk, nv, dk, dv, (float)scale)
#define GDN_BY_DK(T_)                                \
  if (dk == 128 && !generic) GDN_LAUNCH(T_, 128);    \
  else if (dk == 64 && !generic) GDN_LAUNCH(T_, 64); \
  else GDN_LAUNCH(T_, 0)
  static const bool generic = [] { const char* e = std::getenv("CLB200_GDN_GENERIC"); return e && e[0] == '1'; }();
  if (q.scalar_type() == at::kBFloat16) {
    GDN_BY_DK(__nv_bfloat16);
  } else {
    TORCH_CHECK(q.scalar_type() == at::kFloat, "gdn_decode_step: bf16 or fp32");
    GDN_BY_DK(float);
  }
#undef GDN_BY_DK
#undef GDN_LAUNCH
  return out;
}
