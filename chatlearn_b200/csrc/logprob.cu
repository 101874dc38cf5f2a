// Row-wise pieces of the fused LM-head log-prob / entropy op.
//
// The op never keeps [T, V] logits: the host loops over row chunks, a GEMM
// produces the chunk's logits, `logits_stats` reduces each row in ONE pass with an
// online (max, sum-exp, sum-exp*z) triple, and the backward turns the recomputed
// logits into dlogits in place.  Replaces log_softmax + gather + entropy of
// chatlearn/algorithm/grpo_utils/trainer_utils.py:27-52.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

struct Triple {
  float m, s, t;  // running max, sum exp(z-m), sum exp(z-m)*z
};
__device__ __forceinline__ Triple merge(Triple a, Triple b) {
  Triple r;
  r.m = fmaxf(a.m, b.m);
  if (r.m == -INFINITY) { r.s = 0.f; r.t = 0.f; return r; }
  const float ea = __expf(a.m - r.m), eb = __expf(b.m - r.m);
  r.s = a.s * ea + b.s * eb;
  r.t = a.t * ea + b.t * eb;
  return r;
}

template <typename T>
__global__ void logits_stats_kernel(const T* __restrict__ z, const int64_t* __restrict__ labels,
                                    float* __restrict__ lp, float* __restrict__ ent, float* __restrict__ lse_out,
                                    int V, float inv_temp) {
  __shared__ Triple sh[32];
  const int64_t row = blockIdx.x;
  const T* zr = z + row * (int64_t)V;
  Triple a{-INFINITY, 0.f, 0.f};
  constexpr int VEC = Vec16<T>::N;
  // rows stay 16-byte aligned only when V is a multiple of the vector width
  const int vend = (V % VEC == 0) ? V : 0;
  for (int i = threadIdx.x * VEC; i < vend; i += blockDim.x * VEC) {
    Vec16<T> v = ld16(zr + i);
    float f[VEC], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < VEC; ++j) { f[j] = Cvt<T>::to_f(v.v[j]) * inv_temp; mx = fmaxf(mx, f[j]); }
    if (mx > a.m) {
      const float e = __expf(a.m - mx);
      a.s *= e; a.t *= e; a.m = mx;
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float e = __expf(f[j] - a.m);
      a.s += e; a.t += e * f[j];
    }
  }
  for (int i = vend + threadIdx.x; i < V; i += blockDim.x) {
    const float f = Cvt<T>::to_f(zr[i]) * inv_temp;
    if (f > a.m) { const float e = __expf(a.m - f); a.s *= e; a.t *= e; a.m = f; }
    const float e = __expf(f - a.m);
    a.s += e; a.t += e * f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Triple b;
    b.m = __shfl_xor_sync(0xffffffffu, a.m, o);
    b.s = __shfl_xor_sync(0xffffffffu, a.s, o);
    b.t = __shfl_xor_sync(0xffffffffu, a.t, o);
    a = merge(a, b);
  }
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) sh[wid] = a;
  __syncthreads();
  if (wid == 0) {
    a = (lane < nw) ? sh[lane] : Triple{-INFINITY, 0.f, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Triple b;
      b.m = __shfl_xor_sync(0xffffffffu, a.m, o);
      b.s = __shfl_xor_sync(0xffffffffu, a.s, o);
      b.t = __shfl_xor_sync(0xffffffffu, a.t, o);
      a = merge(a, b);
    }
    if (lane == 0) {
      const float lse = a.m + logf(a.s);
      const float zl = Cvt<T>::to_f(zr[labels[row]]) * inv_temp;
      lp[row] = zl - lse;
      ent[row] = lse - a.t / a.s;
      lse_out[row] = lse;
    }
  }
}

// dz_j = inv_temp * [ g_lp*(1{j=label} - p_j) - g_ent * p_j * (z_j - (lse - ent)) ], written as `TO`.
template <typename T, typename TO>
__global__ void logits_grad_kernel(const T* __restrict__ z, const int64_t* __restrict__ labels,
                                   const float* __restrict__ lse, const float* __restrict__ ent,
                                   const float* __restrict__ g_lp, const float* __restrict__ g_ent,
                                   TO* __restrict__ dz, int V, float inv_temp) {
  const int64_t row = blockIdx.x;
  const T* zr = z + row * (int64_t)V;
  TO* dr = dz + row * (int64_t)V;
  const float L = lse[row], glp = g_lp[row];
  const float gen = g_ent ? g_ent[row] : 0.f;
  const float pz = L - ent[row];
  const int lab = (int)labels[row];
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float f = Cvt<T>::to_f(zr[i]) * inv_temp;
    const float p = __expf(f - L);
    float d = -glp * p - gen * p * (f - pz);
    if (i == lab) d += glp;
    dr[i] = Cvt<TO>::from_f(d * inv_temp);
  }
}

std::vector<at::Tensor> logits_stats(const at::Tensor& z, const at::Tensor& labels, double inv_temp) {
  TORCH_CHECK(z.is_cuda() && z.dim() == 2 && z.is_contiguous(), "logits_stats: [T, V] contiguous");
  const int64_t Tn = z.size(0);
  const int V = (int)z.size(1);
  auto o = z.options().dtype(at::kFloat);
  auto lp = at::empty({Tn}, o), ent = at::empty({Tn}, o), lse = at::empty({Tn}, o);
  if (Tn == 0) return {lp, ent, lse};
  auto st = at::cuda::getCurrentCUDAStream();
  if (z.scalar_type() == at::kFloat)
    logits_stats_kernel<float><<<Tn, 1024, 0, st>>>(z.data_ptr<float>(), labels.data_ptr<int64_t>(),
        lp.data_ptr<float>(), ent.data_ptr<float>(), lse.data_ptr<float>(), V, (float)inv_temp);
  else
    logits_stats_kernel<bf16><<<Tn, 1024, 0, st>>>((const bf16*)z.data_ptr(), labels.data_ptr<int64_t>(),
        lp.data_ptr<float>(), ent.data_ptr<float>(), lse.data_ptr<float>(), V, (float)inv_temp);
  return {lp, ent, lse};
}

at::Tensor logits_grad(const at::Tensor& z, const at::Tensor& labels, const at::Tensor& lse,
                       const at::Tensor& ent, const at::Tensor& g_lp, const c10::optional<at::Tensor>& g_ent,
                       double inv_temp, bool out_bf16) {
  const int64_t Tn = z.size(0);
  const int V = (int)z.size(1);
  auto dz = at::empty({Tn, V}, z.options().dtype(out_bf16 ? at::kBFloat16 : at::kFloat));
  if (Tn == 0) return dz;
  auto st = at::cuda::getCurrentCUDAStream();
  const float* ge = g_ent.has_value() ? g_ent->data_ptr<float>() : nullptr;
#define LAUNCH(TI, TO)                                                                              \
  logits_grad_kernel<TI, TO><<<Tn, 1024, 0, st>>>((const TI*)z.data_ptr(), labels.data_ptr<int64_t>(), \
      lse.data_ptr<float>(), ent.data_ptr<float>(), g_lp.data_ptr<float>(), ge, (TO*)dz.data_ptr(), V,  \
      (float)inv_temp)
  if (z.scalar_type() == at::kFloat) { if (out_bf16) LAUNCH(float, bf16); else LAUNCH(float, float); }
  else { if (out_bf16) LAUNCH(bf16, bf16); else LAUNCH(bf16, float); }
#undef LAUNCH
  return dz;
}
