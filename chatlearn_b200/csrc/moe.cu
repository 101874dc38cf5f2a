// Mixture-of-experts routing kernels.
//
//   moe_router_topk   scores (softmax / sigmoid) -> optional group-limited selection ->
//                     top-k -> renormalised weights, plus the tokens-per-expert histogram
//   moe_permute       (token, slot) pairs -> rows sorted by expert (position assignment with
//                     one atomic per pair, then a row copy, optionally scaled)
//   moe_combine       out[t] = sum_s weight[t,s] * y[pos[t,s]]   (fp32 accumulation)
//   moe_row_dot       d weight[t,s] = <dy[t], y[pos[t,s]]>
//
// One warp owns one token (router, combine, dot) or one (token, slot) pair (permute).
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kMaxPerLane = 16;      // experts per lane: up to 512 experts
constexpr int kMaxTopK = 16;
constexpr int kMaxGroups = 16;

template <typename T>
__global__ void router_topk_kernel(const T* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ scores,
                                   float* __restrict__ weights, int64_t* __restrict__ idx, int* __restrict__ hist,
                                   int T_, int E, int k, int sigmoid, int norm, int n_group, int topk_group, float scale) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  float s[kMaxPerLane], sel[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? Cvt<T>::to_f(logits[(int64_t)t * E + e]) : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) s[j] = (lane + 32 * j < E) ? 1.f / (1.f + expf(-s[j])) : 0.f;
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) { s[j] = (lane + 32 * j < E) ? expf(s[j] - mx) : 0.f; sum += s[j]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) s[j] *= inv;
  }
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    if (e < E) {
      scores[(int64_t)t * E + e] = s[j];
      sel[j] = s[j] + (bias ? bias[e] : 0.f);
    } else {
      sel[j] = -INFINITY;
    }
  }
  if (n_group > 1) {
    // score of a group: its maximum, or (with a selection bias) the sum of its two largest
    const int eg = E / n_group;
    float gscore[kMaxGroups];
    for (int g = 0; g < n_group; ++g) {
      float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) {
        const int e = lane + 32 * j;
        if (e < E && e / eg == g) {
          if (sel[j] > m1) { m2 = m1; m1 = sel[j]; } else if (sel[j] > m2) { m2 = sel[j]; }
        }
      }
      for (int o = 16; o > 0; o >>= 1) {       // merge (m1, m2) pairs across lanes
        const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
        const float hi = fmaxf(m1, o1), lo = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
        m1 = hi; m2 = lo;
      }
      gscore[g] = bias ? (m1 + (eg >= 2 ? m2 : 0.f)) : m1;
    }
    unsigned keep = 0;
    for (int r = 0; r < topk_group; ++r) {
      int best = -1;
      float bv = -INFINITY;
      for (int g = 0; g < n_group; ++g)
        if (!((keep >> g) & 1u) && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
      keep |= 1u << best;
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e < E && !((keep >> (e / eg)) & 1u)) sel[j] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float wk[kMaxTopK];
  int ik[kMaxTopK];
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int e = lane + 32 * j;
      if (e < E && (sel[j] > bv || (sel[j] == bv && e < be))) { bv = sel[j]; be = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // the owner lane retires the element and publishes its (unbiased) score
    float sc = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (lane + 32 * j == be) { sc = s[j]; sel[j] = -INFINITY; }
    sc = __shfl_sync(0xffffffffu, sc, be & 31);
    wk[r] = sc; ik[r] = be;
    wsum += sc;
  }
  if (lane == 0) {
    const float inv = norm ? 1.f / (wsum + 1e-20f) : 1.f;
    for (int r = 0; r < k; ++r) {
      weights[(int64_t)t * k + r] = wk[r] * inv * scale;
      idx[(int64_t)t * k + r] = ik[r];
      if (hist) atomicAdd(hist + ik[r], 1);
    }
  }
}

// pos == nullptr on input means "assign": pos_out[p] = offsets[e] + cursor[e]++.
__global__ void permute_kernel(const bf16* __restrict__ x, const int64_t* __restrict__ idx, const int64_t* __restrict__ offsets,
                               int* __restrict__ cursor, int* __restrict__ pos, const float* __restrict__ row_scale,
                               bf16* __restrict__ out, int64_t pairs, int k, int H, int assign) {
  const int lane = threadIdx.x & 31;
  const int64_t p = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= pairs) return;
  int dst;
  if (assign) {
    if (lane == 0) {
      const int e = (int)idx[p];
      dst = (int)offsets[e] + atomicAdd(cursor + e, 1);
      pos[p] = dst;
    }
    dst = __shfl_sync(0xffffffffu, dst, 0);
  } else {
    dst = pos[p];
  }
  const float sc = row_scale ? row_scale[p] : 1.f;
  const bf16* src = x + (p / k) * (int64_t)H;
  bf16* d = out + (int64_t)dst * H;
  for (int v = lane; v < H / 8; v += 32) {
    Vec16<bf16> a = ld16(src + v * 8);
    if (row_scale) {
#pragma unroll
      for (int j = 0; j < 8; ++j) a.v[j] = __float2bfloat16(__bfloat162float(a.v[j]) * sc);
    }
    st16(d + v * 8, a);
  }
}

__global__ void combine_kernel(const bf16* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ weights,
                               bf16* __restrict__ out, int T_, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T_) return;
  for (int v = lane; v < H / 8; v += 32) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const float w = weights ? weights[(int64_t)t * k + s] : 1.f;
      Vec16<bf16> a = ld16(y + (int64_t)pos[(int64_t)t * k + s] * H + v * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * __bfloat162float(a.v[j]);
    }
    Vec16<bf16> o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(acc[j]);
    st16(out + (int64_t)t * H + v * 8, o);
  }
}

__global__ void row_dot_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ y, const int* __restrict__ pos,
                               float* __restrict__ out, int64_t pairs, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t p = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= pairs) return;
  const bf16* a = dy + (p / k) * (int64_t)H;
  const bf16* b = y + (int64_t)pos[p] * H;
  float acc = 0.f;
  for (int v = lane; v < H / 8; v += 32) {
    Vec16<bf16> xa = ld16(a + v * 8), xb = ld16(b + v * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __bfloat162float(xa.v[j]) * __bfloat162float(xb.v[j]);
  }
  acc = warp_sum(acc);
  if (lane == 0) out[p] = acc;
}

inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }

}  // namespace

// logits [T, E] fp32 or bf16.  Returns {weights [T,k] fp32, idx [T,k] int64, scores [T,E] fp32, hist [E] int32}.
std::vector<at::Tensor> moe_router_topk(const at::Tensor& logits, int64_t k, bool sigmoid, bool norm,
                                        const c10::optional<at::Tensor>& bias, int64_t n_group, int64_t topk_group,
                                        double scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous(), "moe_router_topk: contiguous CUDA [T, E]");
  const int T_ = (int)logits.size(0), E = (int)logits.size(1);
  TORCH_CHECK(E <= 32 * kMaxPerLane && k <= kMaxTopK && k <= E, "moe_router_topk: at most 512 experts, top-16");
  TORCH_CHECK(n_group >= 1 && n_group <= kMaxGroups && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group,
              "moe_router_topk: bad group configuration");
  auto fopt = logits.options().dtype(at::kFloat);
  auto weights = at::empty({T_, k}, fopt), scores = at::empty({T_, E}, fopt);
  auto idx = at::empty({T_, k}, logits.options().dtype(at::kLong));
  auto hist = at::zeros({E}, logits.options().dtype(at::kInt));
  if (T_ == 0) return {weights, idx, scores, hist};
  const float* bp = nullptr;
  at::Tensor bf;
  if (bias.has_value()) { bf = bias->to(at::kFloat).contiguous(); bp = bf.data_ptr<float>(); }
  const int warps = 8, grid = (T_ + warps - 1) / warps;
  if (logits.scalar_type() == at::kFloat)
    router_topk_kernel<float><<<grid, warps * 32, 0, stream()>>>(logits.data_ptr<float>(), bp, scores.data_ptr<float>(),
        weights.data_ptr<float>(), idx.data_ptr<int64_t>(), hist.data_ptr<int>(), T_, E, (int)k, sigmoid, norm,
        (int)n_group, (int)topk_group, (float)scale);
  else if (logits.scalar_type() == at::kBFloat16)
    router_topk_kernel<bf16><<<grid, warps * 32, 0, stream()>>>((const bf16*)logits.data_ptr(), bp, scores.data_ptr<float>(),
        weights.data_ptr<float>(), idx.data_ptr<int64_t>(), hist.data_ptr<int>(), T_, E, (int)k, sigmoid, norm,
        (int)n_group, (int)topk_group, (float)scale);
  else
    TORCH_CHECK(false, "moe_router_topk: fp32 or bf16 logits");
  return {weights, idx, scores, hist};
}

// x [T, H] bf16, idx [T, k] int64, offsets [E+1] int64 (exclusive prefix of the histogram).
// Returns {xs [T*k, H] rows sorted by expert, pos [T, k] int32 (row of each pair)}.
// total_rows > 0: the groups are padded (offsets holds padded starts); xs gets that many rows, zero where no pair lands.
std::vector<at::Tensor> moe_permute(const at::Tensor& x, const at::Tensor& idx, const at::Tensor& offsets, int64_t total_rows) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2, "moe_permute: bf16 [T, H]");
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && offsets.scalar_type() == at::kLong, "moe_permute: int64 idx/offsets");
  const int64_t T_ = x.size(0), H = x.size(1), k = idx.size(1), pairs = T_ * k;
  TORCH_CHECK(H % 8 == 0, "moe_permute: hidden size must be a multiple of 8");
  TORCH_CHECK(total_rows <= 0 || total_rows >= pairs, "moe_permute: total_rows smaller than the number of pairs");
  auto xs = total_rows > 0 ? at::zeros({total_rows, H}, x.options()) : at::empty({pairs, H}, x.options());
  auto pos = at::empty({T_, k}, x.options().dtype(at::kInt));
  if (pairs == 0) return {xs, pos};
  auto cursor = at::zeros({offsets.numel()}, x.options().dtype(at::kInt));
  const int warps = 8;
  permute_kernel<<<(unsigned)((pairs + warps - 1) / warps), warps * 32, 0, stream()>>>(
      (const bf16*)x.data_ptr(), idx.data_ptr<int64_t>(), offsets.data_ptr<int64_t>(), cursor.data_ptr<int>(),
      pos.data_ptr<int>(), nullptr, (bf16*)xs.data_ptr(), pairs, (int)k, (int)H, 1);
  return {xs, pos};
}

// Rows of x [T, H] placed at known positions, optionally scaled per pair: out[pos[t,s]] = scale[t,s] * x[t].
at::Tensor moe_permute_at(const at::Tensor& x, const at::Tensor& pos, const c10::optional<at::Tensor>& scale,
                          int64_t total_rows) {
  const int64_t T_ = x.size(0), H = x.size(1), k = pos.size(1), pairs = T_ * k;
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && pos.scalar_type() == at::kInt && pos.is_contiguous() && H % 8 == 0,
              "moe_permute_at: bf16 [T, H], int32 pos");
  auto out = total_rows > 0 ? at::zeros({total_rows, H}, x.options()) : at::empty({pairs, H}, x.options());
  if (pairs == 0) return out;
  const float* sp = nullptr;
  at::Tensor sc;
  if (scale.has_value()) { sc = scale->to(at::kFloat).contiguous(); sp = sc.data_ptr<float>(); }
  const int warps = 8;
  permute_kernel<<<(unsigned)((pairs + warps - 1) / warps), warps * 32, 0, stream()>>>(
      (const bf16*)x.data_ptr(), nullptr, nullptr, nullptr, const_cast<int*>(pos.data_ptr<int>()), sp, (bf16*)out.data_ptr(),
      pairs, (int)k, (int)H, 0);
  return out;
}

// out[t] = sum_s weights[t,s] * y[pos[t,s]]  (weights may be absent: plain sum).
at::Tensor moe_combine(const at::Tensor& y, const at::Tensor& pos, const c10::optional<at::Tensor>& weights) {
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && pos.scalar_type() == at::kInt && pos.is_contiguous(),
              "moe_combine: bf16 y, int32 pos");
  const int T_ = (int)pos.size(0), k = (int)pos.size(1), H = (int)y.size(1);
  TORCH_CHECK(H % 8 == 0, "moe_combine: hidden size must be a multiple of 8");
  auto out = at::empty({T_, H}, y.options());
  if (T_ == 0) return out;
  const float* wp = nullptr;
  at::Tensor w;
  if (weights.has_value()) { w = weights->to(at::kFloat).contiguous(); wp = w.data_ptr<float>(); }
  const int warps = 8;
  combine_kernel<<<(T_ + warps - 1) / warps, warps * 32, 0, stream()>>>((const bf16*)y.data_ptr(), pos.data_ptr<int>(), wp,
                                                                       (bf16*)out.data_ptr(), T_, k, H);
  return out;
}

// out[t,s] = <dy[t], y[pos[t,s]]>
at::Tensor moe_row_dot(const at::Tensor& dy, const at::Tensor& y, const at::Tensor& pos) {
  const int64_t T_ = pos.size(0), k = pos.size(1), H = y.size(1), pairs = T_ * k;
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16 && dy.is_contiguous() && y.is_contiguous() && H % 8 == 0,
              "moe_row_dot: bf16 contiguous");
  auto out = at::empty({T_, k}, dy.options().dtype(at::kFloat));
  if (pairs == 0) return out;
  const int warps = 8;
  row_dot_kernel<<<(unsigned)((pairs + warps - 1) / warps), warps * 32, 0, stream()>>>(
      (const bf16*)dy.data_ptr(), (const bf16*)y.data_ptr(), pos.data_ptr<int>(), out.data_ptr<float>(), pairs, (int)k, (int)H);
  return out;
}
