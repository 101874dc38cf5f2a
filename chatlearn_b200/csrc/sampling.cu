// Token sampler of the rollout engine: temperature, top-k, top-p, min-p and
// inverse-CDF sampling in one kernel, one CTA per sequence, no sort.
//
// top-k / top-p thresholds are found by bisection over the *bit patterns* of the
// probabilities (monotone for non-negative floats), so the result is the exact
// k-th largest value / the exact boundary value of the nucleus, as a sort would
// give.  Replaces the sampling stage of vLLM/SGLang that the reference
// configures in chatlearn/models/vllm_module.py:286-322.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ float block_sum_bcast(float v, float* red) {
  float r = block_sum(v, red);
  __syncthreads();
  return r;
}

// probability of element i under temperature-scaled softmax
__device__ __forceinline__ float prob(const float* z, int i, float inv_t, float m, float inv_s) {
  return __expf(z[i] * inv_t - m) * inv_s;
}

__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ u,
                              int64_t* __restrict__ ids, float* __restrict__ logprob, int V, float temperature,
                              int top_k, float top_p, float min_p) {
  __shared__ float red[32];
  __shared__ float sh_f[4];
  __shared__ int sh_i[2];
  const int row = blockIdx.x;
  const float* z = logits + (int64_t)row * V;
  const int tid = threadIdx.x;

  // ---- greedy ----
  if (temperature == 0.f) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += kThreads) {
      const float f = z[i];
      if (f > best) { best = f; bi = i; }
    }
    const float mx = block_max(best, red);
    __syncthreads();
    if (tid == 0) sh_i[0] = 0x7fffffff;
    __syncthreads();
    if (best == mx) atomicMin(&sh_i[0], bi);
    float se = 0.f;
    for (int i = tid; i < V; i += kThreads) se += __expf(z[i] - mx);
    se = block_sum_bcast(se, red);
    if (tid == 0) { ids[row] = sh_i[0]; logprob[row] = -logf(se); }
    return;
  }

  const float inv_t = 1.f / temperature;
  float mx = -INFINITY;
  for (int i = tid; i < V; i += kThreads) mx = fmaxf(mx, z[i] * inv_t);
  mx = block_max(mx, red);
  __syncthreads();
  float se = 0.f;
  for (int i = tid; i < V; i += kThreads) se += __expf(z[i] * inv_t - mx);
  se = block_sum_bcast(se, red);
  const float inv_s = 1.f / se;

  // ---- threshold on probability (keep p >= thr) ----
  float thr = 0.f;
  if (top_k > 0 && top_k < V) {
    // largest t with count(p >= t) >= k  == the k-th largest probability
    unsigned lo = 0u, hi = __float_as_uint(1.0f) + 1u;   // invariant: count(lo) >= k, count(hi) < k
    while (hi - lo > 1u) {
      const unsigned mid = lo + (hi - lo) / 2u;
      const float t = __uint_as_float(mid);
      float c = 0.f;
      for (int i = tid; i < V; i += kThreads) c += (prob(z, i, inv_t, mx, inv_s) >= t) ? 1.f : 0.f;
      c = block_sum_bcast(c, red);
      if (c >= (float)top_k) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, __uint_as_float(lo));
  }
  if (top_p < 1.f) {
    // largest t with mass(p >= t) >= top_p
    unsigned lo = 0u, hi = __float_as_uint(1.0f) + 1u;
    while (hi - lo > 1u) {
      const unsigned mid = lo + (hi - lo) / 2u;
      const float t = __uint_as_float(mid);
      float c = 0.f;
      for (int i = tid; i < V; i += kThreads) {
        const float p = prob(z, i, inv_t, mx, inv_s);
        c += (p >= t) ? p : 0.f;
      }
      c = block_sum_bcast(c, red);
      if (c >= top_p) lo = mid; else hi = mid;
    }
    thr = fmaxf(thr, __uint_as_float(lo));
  }
  if (min_p > 0.f) thr = fmaxf(thr, min_p * inv_s);   // p_max = exp(0) / S

  // ---- inverse CDF over the kept tokens: contiguous segment per thread ----
  const int per = (V + kThreads - 1) / kThreads;
  const int s0 = min(tid * per, V), s1 = min(s0 + per, V);
  float seg = 0.f;
  for (int i = s0; i < s1; ++i) {
    const float p = prob(z, i, inv_t, mx, inv_s);
    seg += (p >= thr) ? p : 0.f;
  }
  // inclusive scan of segment sums (warp scan + scan of warp totals)
  const int lane = tid & 31, wid = tid >> 5;
  float inc = seg;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) red[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    float w = red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    red[lane] = w;
  }
  __syncthreads();
  const float before_warp = (wid > 0) ? red[wid - 1] : 0.f;
  const float total = red[31];
  const float end = before_warp + inc, start = end - seg;
  const float target = u[row] * total;
  if (tid == 0) { sh_i[0] = -1; sh_i[1] = -1; }
  __syncthreads();
  // the owning thread: first segment whose inclusive end exceeds the target
  if (seg > 0.f && start <= target && target < end) {
    float c = start;
    int pick = -1, last_kept = -1;
    for (int i = s0; i < s1; ++i) {
      const float p = prob(z, i, inv_t, mx, inv_s);
      if (p >= thr) {
        last_kept = i;
        c += p;
        if (c > target) { pick = i; break; }
      }
    }
    if (pick < 0) pick = last_kept;
    atomicMax(&sh_i[0], pick);
  }
  // fallback (rounding put the target past every segment): last kept token
  if (seg > 0.f) {
    int last_kept = -1;
    for (int i = s1 - 1; i >= s0; --i)
      if (prob(z, i, inv_t, mx, inv_s) >= thr) { last_kept = i; break; }
    atomicMax(&sh_i[1], last_kept);
  }
  __syncthreads();
  if (tid == 0) {
    const int id = sh_i[0] >= 0 ? sh_i[0] : sh_i[1];
    ids[row] = id;
    logprob[row] = z[id] * inv_t - mx - logf(se);
  }
}

// presence / frequency / repetition penalties, in place on fp32 logits
__global__ void penalties_kernel(float* __restrict__ z, const int* __restrict__ counts,
                                 const bool* __restrict__ prompt_mask, int64_t n, float presence,
                                 float frequency, float repetition) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float f = z[i];
    const int c = counts[i];
    const bool seen = c > 0 || (prompt_mask && prompt_mask[i]);
    if (repetition != 1.f && seen) f = f > 0.f ? f / repetition : f * repetition;
    f -= frequency * (float)c;
    if (c > 0) f -= presence;
    z[i] = f;
  }
}

}  // namespace

std::vector<at::Tensor> sample(const at::Tensor& logits, const at::Tensor& u, double temperature, int64_t top_k,
                               double top_p, double min_p) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kFloat && logits.is_contiguous(),
              "sample: fp32 [B, V] contiguous logits");
  const int B = (int)logits.size(0), V = (int)logits.size(1);
  auto ids = at::empty({B}, logits.options().dtype(at::kLong));
  auto lp = at::empty({B}, logits.options());
  if (B == 0) return {ids, lp};
  sample_kernel<<<B, kThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      logits.data_ptr<float>(), u.data_ptr<float>(), ids.data_ptr<int64_t>(), lp.data_ptr<float>(), V,
      (float)temperature, (int)top_k, (float)top_p, (float)min_p);
  return {ids, lp};
}

at::Tensor apply_penalties(const at::Tensor& logits, const at::Tensor& counts,
                           const c10::optional<at::Tensor>& prompt_mask, double presence, double frequency,
                           double repetition) {
  auto z = logits.to(at::kFloat).contiguous().clone();
  const int64_t n = z.numel();
  if (n == 0) return z;
  auto c = counts.to(at::kInt).contiguous();
  int grid = (int)std::min<int64_t>((n + 255) / 256, 148 * 8);
  penalties_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      z.data_ptr<float>(), c.data_ptr<int>(), prompt_mask.has_value() ? prompt_mask->data_ptr<bool>() : nullptr, n,
      (float)presence, (float)frequency, (float)repetition);
  return z;
}
