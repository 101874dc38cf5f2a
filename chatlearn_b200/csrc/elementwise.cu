// Memory-bound training kernels: RMSNorm, fused per-head QK-norm + RoPE, SwiGLU,
// the fused GRPO loss (forward + gradient in one pass), AdamW on a shard and a
// deterministic sum of squares.  Each replaces a chain of eager PyTorch kernels
// of the reference stack (HF/Megatron model internals, loss_gallery.py, torch
// AdamW); all are single-pass over their operands.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

#define DISPATCH_FLOAT_BF16(TENSOR, NAME, ...)                                    \
  if ((TENSOR).scalar_type() == at::kFloat) {                                    \
    using scalar_t = float;                                                      \
    __VA_ARGS__();                                                               \
  } else if ((TENSOR).scalar_type() == at::kBFloat16) {                          \
    using scalar_t = bf16;                                                       \
    __VA_ARGS__();                                                               \
  } else {                                                                       \
    TORCH_CHECK(false, NAME ": dtype must be float32 or bfloat16");               \
  }

static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream(); }

// ----------------------------------------------------------------------------- RMSNorm
// One CTA per row.  y = x * rsqrt(mean(x^2) + eps) * w ; rstd saved for backward.
template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                   float* __restrict__ rstd, int H, float eps) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const T* xr = x + row * H;
  T* yr = y + row * H;
  constexpr int V = Vec16<T>::N;
  float ss = 0.f;
  for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
    Vec16<T> a = ld16(xr + i);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float f = Cvt<T>::to_f(a.v[j]);
      ss += f * f;
    }
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
    Vec16<T> a = ld16(xr + i), ww = ld16(w + i), o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(a.v[j]) * r * Cvt<T>::to_f(ww.v[j]));
    st16(yr + i, o);
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw += dy * xhat (fp32 atomics, one
// partial per CTA: each CTA walks a strided set of rows and keeps dw in registers).
// A thread owns at most MAXV 16-byte vectors of a row.  The row's x and dy stay in registers between the
// reduction and the write of dx (read once), the weights are loaded once per CTA, and the next row's
// vectors are requested before the current row's reduction, so the loads overlap the barriers.
template <typename T, int MAXV>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                   const T* __restrict__ dy, const float* __restrict__ rstd,
                                   T* __restrict__ dx, float* __restrict__ dw, int64_t N, int H) {
  __shared__ float red[32];
  constexpr int V = Vec16<T>::N;
  float dwacc[MAXV][V];
  Vec16<T> wv[MAXV], xv[MAXV], gv[MAXV], nx[MAXV], ng[MAXV];
  int col[MAXV];
#pragma unroll
  for (int a = 0; a < MAXV; ++a) {
    col[a] = (threadIdx.x + a * blockDim.x) * V;
#pragma unroll
    for (int j = 0; j < V; ++j) dwacc[a][j] = 0.f;
    if (col[a] < H) wv[a] = ld16(w + col[a]);
  }
  int64_t row = blockIdx.x;
  if (row < N) {
#pragma unroll
    for (int a = 0; a < MAXV; ++a)
      if (col[a] < H) { xv[a] = ld16(x + row * H + col[a]); gv[a] = ld16(dy + row * H + col[a]); }
  }
  while (row < N) {
    const int64_t next = row + gridDim.x;
    if (next < N) {
#pragma unroll
      for (int a = 0; a < MAXV; ++a)
        if (col[a] < H) { nx[a] = ld16(x + next * H + col[a]); ng[a] = ld16(dy + next * H + col[a]); }
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int a = 0; a < MAXV; ++a) {
      if (col[a] < H) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xv[a].v[j]) * r;
          const float g = Cvt<T>::to_f(gv[a].v[j]);
          dot += g * Cvt<T>::to_f(wv[a].v[j]) * xh;
          dwacc[a][j] += g * xh;
        }
      }
    }
    dot = block_sum(dot, red) / H;
#pragma unroll
    for (int a = 0; a < MAXV; ++a) {
      if (col[a] < H) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = Cvt<T>::to_f(xv[a].v[j]) * r;
          o.v[j] = Cvt<T>::from_f(r * (Cvt<T>::to_f(gv[a].v[j]) * Cvt<T>::to_f(wv[a].v[j]) - xh * dot));
        }
        st16(dx + row * H + col[a], o);
      }
    }
#pragma unroll
    for (int a = 0; a < MAXV; ++a) { xv[a] = nx[a]; gv[a] = ng[a]; }
    row = next;
  }
#pragma unroll
  for (int a = 0; a < MAXV; ++a) {
    if (col[a] < H) {
#pragma unroll
      for (int j = 0; j < V; ++j) atomicAdd(dw + col[a] + j, dwacc[a][j]);
    }
  }
}

// Warp per row: the row stays in registers (VPL 16-byte vectors per lane), one read, one warp reduction, no
// shared memory.  For hidden sizes of exactly 32 * VPL vectors.
template <typename T, int VPL>
__global__ void rmsnorm_fwd_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                        float* __restrict__ rstd, int64_t N, float eps) {
  constexpr int V = Vec16<T>::N;
  constexpr int H = 32 * VPL * V;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= N) return;
  const T* xr = x + row * H;
  Vec16<T> a[VPL];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    a[k] = ld16(xr + (k * 32 + lane) * V);
#pragma unroll
    for (int j = 0; j < V; ++j) { const float f = Cvt<T>::to_f(a[k].v[j]); ss += f * f; }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / H + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  T* yr = y + row * H;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    Vec16<T> ww = ld16(w + (k * 32 + lane) * V), o;
#pragma unroll
    for (int j = 0; j < V; ++j) o.v[j] = Cvt<T>::from_f(Cvt<T>::to_f(a[k].v[j]) * r * Cvt<T>::to_f(ww.v[j]));
    st16(yr + (k * 32 + lane) * V, o);
  }
}

// Launches the warp-per-row kernel when the hidden size is 32 * VPL vectors for a built VPL; false otherwise.
template <typename T>
static bool launch_rmsnorm_rows(const T* x, const T* w, T* y, float* rstd, int64_t N, int H, float eps) {
  constexpr int V = Vec16<T>::N;
  if (H % (32 * V) != 0) return false;
  const int vpl = H / (32 * V);
  const int warps = 4;
  const dim3 grid((unsigned)((N + warps - 1) / warps)), block(warps * 32);
  if (vpl == 2) C10_CUDA_CHECK(launch_pdl(rmsnorm_fwd_rows_kernel<T, 2>, grid, block, 0, cur_stream(), x, w, y, rstd, N, eps));
  else if (vpl == 4) C10_CUDA_CHECK(launch_pdl(rmsnorm_fwd_rows_kernel<T, 4>, grid, block, 0, cur_stream(), x, w, y, rstd, N, eps));
  else if (vpl == 8) C10_CUDA_CHECK(launch_pdl(rmsnorm_fwd_rows_kernel<T, 8>, grid, block, 0, cur_stream(), x, w, y, rstd, N, eps));
  else if (vpl == 16) C10_CUDA_CHECK(launch_pdl(rmsnorm_fwd_rows_kernel<T, 16>, grid, block, 0, cur_stream(), x, w, y, rstd, N, eps));
  else return false;
  return true;
}

std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && w.is_contiguous(), "rmsnorm: contiguous CUDA tensors");
  const int H = x.size(-1);
  const int64_t N = x.numel() / H;
  TORCH_CHECK(w.numel() == H && w.scalar_type() == x.scalar_type(), "rmsnorm: weight mismatch");
  auto y = at::empty_like(x);
  auto rstd = at::empty({N}, x.options().dtype(at::kFloat));
  if (N == 0) return {y, rstd};
  DISPATCH_FLOAT_BF16(x, "rmsnorm", [&] {
    constexpr int V = Vec16<scalar_t>::N;
    TORCH_CHECK(H % V == 0, "rmsnorm: hidden size must be a multiple of ", V);
    if (launch_rmsnorm_rows<scalar_t>((const scalar_t*)x.data_ptr(), (const scalar_t*)w.data_ptr(), (scalar_t*)y.data_ptr(),
                                      rstd.data_ptr<float>(), N, H, (float)eps))
      return;
    int threads = std::min(1024, std::max(32, ((H / V + 31) / 32) * 32));
    C10_CUDA_CHECK(launch_pdl(rmsnorm_fwd_kernel<scalar_t>, dim3((unsigned)N), dim3(threads), 0, cur_stream(),
        (const scalar_t*)x.data_ptr(), (const scalar_t*)w.data_ptr(), (scalar_t*)y.data_ptr(),
        rstd.data_ptr<float>(), H, (float)eps));
  });
  return {y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy,
                                    const at::Tensor& rstd) {
  const int H = x.size(-1);
  const int64_t N = x.numel() / H;
  auto dx = at::empty_like(x);
  auto dw = at::zeros({H}, x.options().dtype(at::kFloat));
  if (N == 0) return {dx, dw};
  auto dyc = dy.contiguous();
  DISPATCH_FLOAT_BF16(x, "rmsnorm_bwd", [&] {
    constexpr int V = Vec16<scalar_t>::N;
    constexpr int MAXV = 4;
    int threads = std::min(1024, std::max(32, ((H / V + MAXV - 1) / MAXV + 31) / 32 * 32));
    // every thread owns at most MAXV vectors of the row
    while ((int64_t)threads * V * MAXV < H) threads += 32;
    TORCH_CHECK(threads <= 1024, "rmsnorm_bwd: hidden size too large");
    int grid = (int)std::min<int64_t>(N, 148 * 4);
    rmsnorm_bwd_kernel<scalar_t, MAXV><<<grid, threads, 0, cur_stream()>>>(
        (const scalar_t*)x.data_ptr(), (const scalar_t*)w.data_ptr(), (const scalar_t*)dyc.data_ptr(),
        rstd.data_ptr<float>(), (scalar_t*)dx.data_ptr(), dw.data_ptr<float>(), N, H);
  });
  return {dx, dw};
}

// ----------------------------------------------------------------------------- SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ y, int64_t rows, int F) {
  pdl_trigger();
  pdl_wait();
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = rows * (F / V);
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < nvec;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / (F / V);
    const int c = (idx % (F / V)) * V;
    Vec16<T> g = ld16(gu + r * 2 * F + c), u = ld16(gu + r * 2 * F + F + c), o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float gf = Cvt<T>::to_f(g.v[j]);
      o.v[j] = Cvt<T>::from_f(gf / (1.f + __expf(-gf)) * Cvt<T>::to_f(u.v[j]));
    }
    st16(y + r * F + c, o);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dy, T* __restrict__ dgu,
                                  int64_t rows, int F) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = rows * (F / V);
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < nvec;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / (F / V);
    const int c = (idx % (F / V)) * V;
    Vec16<T> g = ld16(gu + r * 2 * F + c), u = ld16(gu + r * 2 * F + F + c), d = ld16(dy + r * F + c), og, ou;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float gf = Cvt<T>::to_f(g.v[j]), uf = Cvt<T>::to_f(u.v[j]), df = Cvt<T>::to_f(d.v[j]);
      float s = 1.f / (1.f + __expf(-gf));
      og.v[j] = Cvt<T>::from_f(df * uf * s * (1.f + gf * (1.f - s)));
      ou.v[j] = Cvt<T>::from_f(df * gf * s);
    }
    st16(dgu + r * 2 * F + c, og);
    st16(dgu + r * 2 * F + F + c, ou);
  }
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  TORCH_CHECK(gu.is_cuda() && gu.is_contiguous(), "swiglu: contiguous CUDA tensor");
  const int F = gu.size(-1) / 2;
  const int64_t rows = gu.numel() / (2 * F);
  auto sizes = gu.sizes().vec();
  sizes.back() = F;
  auto y = at::empty(sizes, gu.options());
  if (rows == 0) return y;
  DISPATCH_FLOAT_BF16(gu, "swiglu", [&] {
    constexpr int V = Vec16<scalar_t>::N;
    TORCH_CHECK(F % V == 0, "swiglu: F must be a multiple of ", V);
    int64_t nvec = rows * (F / V);
    int grid = (int)std::min<int64_t>((nvec + 255) / 256, 148 * 16);
    C10_CUDA_CHECK(launch_pdl(swiglu_fwd_kernel<scalar_t>, dim3(grid), dim3(256), 0, cur_stream(), (const scalar_t*)gu.data_ptr(),
                              (scalar_t*)y.data_ptr(), rows, F));
  });
  return y;
}

at::Tensor swiglu_bwd(const at::Tensor& gu, const at::Tensor& dy) {
  const int F = gu.size(-1) / 2;
  const int64_t rows = gu.numel() / (2 * F);
  auto dgu = at::empty_like(gu);
  if (rows == 0) return dgu;
  auto dyc = dy.contiguous();
  DISPATCH_FLOAT_BF16(gu, "swiglu_bwd", [&] {
    constexpr int V = Vec16<scalar_t>::N;
    int64_t nvec = rows * (F / V);
    int grid = (int)std::min<int64_t>((nvec + 255) / 256, 148 * 16);
    swiglu_bwd_kernel<scalar_t><<<grid, 256, 0, cur_stream()>>>(
        (const scalar_t*)gu.data_ptr(), (const scalar_t*)dyc.data_ptr(), (scalar_t*)dgu.data_ptr(), rows, F);
  });
  return dgu;
}

// ----------------------------------------------------------------------------- QK-norm + RoPE
// One warp per (token, head), grid-stride.  Heads of q and k live side by side in the packed
// qkv row; outputs are written densely.  D = head dim (64 or 128), rotate-half: element i of the first
// half pairs with element i of the second.  A lane owns HE = D / 64 neighbouring elements of each half
// (one 4-byte load per half for bf16 at D = 128).  norm weights may be null (Llama: RoPE only).
// Backward: the weight gradient is summed in registers over all items of a warp, then over the warps of
// the CTA in shared memory, and reaches memory as one atomic per element and CTA (one per element and
// (token, head) cost 1.7 ms per call at 16 k tokens x 32 heads, twenty times the forward).
template <typename T, int HE>
__device__ __forceinline__ void ld_he(const T* p, float (&o)[HE]) {
#pragma unroll
  for (int j = 0; j < HE; ++j) o[j] = Cvt<T>::to_f(p[j]);
}
template <>
__device__ __forceinline__ void ld_he<bf16, 2>(const bf16* p, float (&o)[2]) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  o[0] = f.x; o[1] = f.y;
}
template <typename T, int HE>
__device__ __forceinline__ void st_he(T* p, const float (&v)[HE]) {
#pragma unroll
  for (int j = 0; j < HE; ++j) p[j] = Cvt<T>::from_f(v[j]);
}
template <>
__device__ __forceinline__ void st_he<bf16, 2>(bf16* p, const float (&v)[2]) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
}

template <typename T, int D, bool BWD>
__global__ void qk_norm_rope_kernel(const T* __restrict__ src, int src_stride, int n_heads,
                                    const T* __restrict__ w, const int64_t* __restrict__ pos,
                                    const float* __restrict__ inv_freq, T* __restrict__ dst,
                                    const T* __restrict__ x_saved, int x_stride, float* __restrict__ dw,
                                    int64_t T_tokens, float eps) {
  constexpr int HE = D / 64;  // elements per lane in each half
  __shared__ float dw_red[BWD ? 8 : 1][BWD ? D : 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = HE * lane;
  const int64_t stride = ((int64_t)gridDim.x * blockDim.x) >> 5;
  float fr[HE], wa[HE], wb[HE];
#pragma unroll
  for (int j = 0; j < HE; ++j) { fr[j] = inv_freq[e0 + j]; wa[j] = wb[j] = 1.f; }
  if (w) { ld_he<T, HE>(w + e0, wa); ld_he<T, HE>(w + D / 2 + e0, wb); }
  float dwa[HE], dwb[HE];
#pragma unroll
  for (int j = 0; j < HE; ++j) dwa[j] = dwb[j] = 0.f;
  // a warp takes a token and walks its heads: the rotation angles are computed once per token, not once per head
  for (int64_t wid = ((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5); wid < T_tokens; wid += stride) {
    const int64_t t = wid;
    const float p = (float)pos[t];
    float c[HE], s[HE];
#pragma unroll
    for (int j = 0; j < HE; ++j) sincosf(p * fr[j], &s[j], &c[j]);
#pragma unroll 2
    for (int h = 0; h < n_heads; ++h) {
    if (!BWD) {
      const T* xr = src + t * src_stride + h * D;
      float a[HE], b[HE], ss = 0.f;
      ld_he<T, HE>(xr + e0, a);
      ld_he<T, HE>(xr + D / 2 + e0, b);
#pragma unroll
      for (int j = 0; j < HE; ++j) ss += a[j] * a[j] + b[j] * b[j];
      float r = 1.f;
      if (w) {
        ss = warp_sum(ss);
        r = rsqrtf(ss / D + eps);
      }
      T* o = dst + (t * n_heads + h) * D;
      float oa[HE], ob[HE];
#pragma unroll
      for (int j = 0; j < HE; ++j) {
        // the normalised value is rounded to T before the rotation, as the eager path does
        const float na = w ? Cvt<T>::to_f(Cvt<T>::from_f(a[j] * r * wa[j])) : a[j];
        const float nb = w ? Cvt<T>::to_f(Cvt<T>::from_f(b[j] * r * wb[j])) : b[j];
        oa[j] = na * c[j] - nb * s[j];
        ob[j] = nb * c[j] + na * s[j];
      }
      st_he<T, HE>(o + e0, oa);
      st_he<T, HE>(o + D / 2 + e0, ob);
    } else {
      // src = gradient w.r.t. the rotated output [T, n_heads, D]; dst = gradient w.r.t. x
      const T* gr = src + (t * n_heads + h) * D;
      const T* xr = x_saved + t * x_stride + h * D;
      float d1[HE], d2[HE], ga[HE], gb[HE], xa[HE], xb[HE], ss = 0.f;
      ld_he<T, HE>(gr + e0, d1);
      ld_he<T, HE>(gr + D / 2 + e0, d2);
      ld_he<T, HE>(xr + e0, xa);
      ld_he<T, HE>(xr + D / 2 + e0, xb);
#pragma unroll
      for (int j = 0; j < HE; ++j) {
        ga[j] = d1[j] * c[j] + d2[j] * s[j];
        gb[j] = d2[j] * c[j] - d1[j] * s[j];
        ss += xa[j] * xa[j] + xb[j] * xb[j];
      }
      T* o = dst + t * src_stride + h * D;
      if (!w) {
        st_he<T, HE>(o + e0, ga);
        st_he<T, HE>(o + D / 2 + e0, gb);
        continue;
      }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / D + eps);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < HE; ++j) {
        dot += ga[j] * wa[j] * xa[j] * r + gb[j] * wb[j] * xb[j] * r;
        dwa[j] += ga[j] * xa[j] * r;
        dwb[j] += gb[j] * xb[j] * r;
      }
      dot = warp_sum(dot) / D;
      float oa[HE], ob[HE];
#pragma unroll
      for (int j = 0; j < HE; ++j) {
        oa[j] = r * (ga[j] * wa[j] - xa[j] * r * dot);
        ob[j] = r * (gb[j] * wb[j] - xb[j] * r * dot);
      }
      st_he<T, HE>(o + e0, oa);
      st_he<T, HE>(o + D / 2 + e0, ob);
    }
    }
  }
  if (BWD && w) {
#pragma unroll
    for (int j = 0; j < HE; ++j) { dw_red[warp][e0 + j] = dwa[j]; dw_red[warp][D / 2 + e0 + j] = dwb[j]; }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float v = 0.f;
      for (int k = 0; k < (int)(blockDim.x >> 5); ++k) v += dw_red[k][i];
      atomicAdd(dw + i, v);
    }
  }
}

template <typename T, bool BWD>
static void launch_qk(const T* src, int src_stride, int n_heads, const T* w, const int64_t* pos,
                      const float* inv_freq, T* dst, const T* xs, int xstride, float* dw, int64_t Tn, int D,
                      float eps) {
  if (Tn * n_heads == 0) return;
  const int threads = 256;                       // 8 warps: the size of the backward's shared reduction
  const int64_t want = (Tn * 32 + threads - 1) / threads;      // one warp per token
  const int grid = (int)std::min<int64_t>(want, 148 * 8);
  if (D == 128)
    qk_norm_rope_kernel<T, 128, BWD><<<grid, threads, 0, cur_stream()>>>(src, src_stride, n_heads, w, pos, inv_freq,
                                                                        dst, xs, xstride, dw, Tn, eps);
  else if (D == 64)
    qk_norm_rope_kernel<T, 64, BWD><<<grid, threads, 0, cur_stream()>>>(src, src_stride, n_heads, w, pos, inv_freq,
                                                                       dst, xs, xstride, dw, Tn, eps);
  else
    TORCH_CHECK(false, "qk_norm_rope: head dim must be 64 or 128");
}

// Inference with a paged KV cache: one launch does what three did.  For every token of the packed qkv rows
// [T, (nq + 2 nkv) * D]: query heads get (RMSNorm and) RoPE and go to q_out [T, nq, D]; key heads get the same
// and are stored straight into their cache slot; value heads are copied into theirs.  One warp per (token, head).
// slots[t] < 0 skips the cache writes of a token (padding rows of a captured decode step).
template <int D>
__global__ void qkv_rope_append_kernel(const bf16* __restrict__ qkv, int row_stride, int nq, int nkv,
                                       const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                       const int64_t* __restrict__ pos, const float* __restrict__ inv_freq,
                                       const int64_t* __restrict__ slots, bf16* __restrict__ q_out,
                                       bf16* __restrict__ kc, bf16* __restrict__ vc, int64_t T_tokens, float eps,
                                       const float* __restrict__ planes, int S, int64_t plane_stride) {
  constexpr int HE = D / 64;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int64_t wid = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (wid >= T_tokens * heads) return;
  const int64_t t = wid / heads;
  const int h = (int)(wid % heads);
  const int64_t base = t * row_stride + (int64_t)h * D;
  // the projection's output: a bf16 row, or (planes != nullptr) the K-slice planes of the GEMM that produced it, added
  // up here and rounded to bf16 exactly as the finalize kernel would have done
  auto ldx = [&](int e) -> float {
    if (planes == nullptr) return __bfloat162float(qkv[base + e]);
    float v = planes[base + e];
    for (int s = 1; s < S; ++s) v += planes[(int64_t)s * plane_stride + base + e];
    return __bfloat162float(__float2bfloat16_rn(v));
  };
  if (h >= nq + nkv) {                                  // value head: plain copy into the cache slot
    const int64_t slot = slots[t];
    if (slot < 0) return;
    bf16* o = vc + (slot * nkv + (h - nq - nkv)) * D;
#pragma unroll
    for (int j = 0; j < 2 * HE; ++j) o[lane + 32 * j] = __float2bfloat16_rn(ldx(lane + 32 * j));
    return;
  }
  const bool is_q = h < nq;
  const bf16* w = is_q ? qw : kw;
  bf16* o;
  if (is_q) {
    o = q_out + (t * nq + h) * D;
  } else {
    const int64_t slot = slots[t];
    if (slot < 0) return;
    o = kc + (slot * nkv + (h - nq)) * D;
  }
  const float p = (float)pos[t];
  float a[HE], b[HE], ss = 0.f;
#pragma unroll
  for (int j = 0; j < HE; ++j) {
    a[j] = ldx(lane + 32 * j);
    b[j] = ldx(D / 2 + lane + 32 * j);
    ss += a[j] * a[j] + b[j] * b[j];
  }
  float r = 1.f;
  if (w) {
    ss = warp_sum(ss);
    r = rsqrtf(ss / D + eps);
  }
#pragma unroll
  for (int j = 0; j < HE; ++j) {
    float sn, cs;
    sincosf(p * inv_freq[lane + 32 * j], &sn, &cs);
    const float wa = w ? __bfloat162float(w[lane + 32 * j]) : 1.f;
    const float wb = w ? __bfloat162float(w[D / 2 + lane + 32 * j]) : 1.f;
    // the normalised value is rounded to bf16 before the rotation, as the separate kernels do
    const float na = w ? __bfloat162float(__float2bfloat16_rn(a[j] * r * wa)) : a[j];
    const float nb = w ? __bfloat162float(__float2bfloat16_rn(b[j] * r * wb)) : b[j];
    o[lane + 32 * j] = __float2bfloat16_rn(na * cs - nb * sn);
    o[D / 2 + lane + 32 * j] = __float2bfloat16_rn(nb * cs + na * sn);
  }
}

// qkv [T, (nq + 2 nkv) * D] bf16 (unit inner stride); caches [num_blocks, block, nkv, D] bf16; returns q_out [T, nq, D].
at::Tensor qkv_rope_append(const at::Tensor& qkv, int64_t nq, int64_t nkv, int64_t D, const c10::optional<at::Tensor>& qw,
                           const c10::optional<at::Tensor>& kw, const at::Tensor& pos, const at::Tensor& inv_freq,
                           const at::Tensor& slots, at::Tensor k_cache, at::Tensor v_cache, double eps,
                           const c10::optional<at::Tensor>& planes) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.scalar_type() == at::kBFloat16 &&
              qkv.size(1) == (nq + 2 * nkv) * D, "qkv_rope_append: qkv must be bf16 [T, (nq + 2 nkv) * D]");
  // planes: the projection's K-slice planes fp32 [S, T, width] (then qkv only gives the shape; it is not read)
  const float* plp = nullptr;
  int S = 0;
  if (planes.has_value() && planes->numel() > 0) {
    TORCH_CHECK(planes->scalar_type() == at::kFloat && planes->dim() == 3 && planes->is_contiguous() &&
                planes->size(1) == qkv.size(0) && planes->size(2) == qkv.size(1) && qkv.stride(0) == qkv.size(1),
                "qkv_rope_append: planes must be contiguous fp32 [S, T, width] of a contiguous qkv");
    plp = planes->data_ptr<float>();
    S = (int)planes->size(0);
  }
  TORCH_CHECK(k_cache.scalar_type() == at::kBFloat16 && v_cache.scalar_type() == at::kBFloat16 && k_cache.is_contiguous() &&
              v_cache.is_contiguous() && k_cache.size(2) == nkv && k_cache.size(3) == D && v_cache.size(3) == D,
              "qkv_rope_append: caches must be contiguous bf16 [blocks, block, nkv, D]");
  TORCH_CHECK(pos.scalar_type() == at::kLong && slots.scalar_type() == at::kLong && inv_freq.scalar_type() == at::kFloat,
              "qkv_rope_append: int64 positions and slots, fp32 inverse frequencies");
  TORCH_CHECK(qw.has_value() == kw.has_value(), "qkv_rope_append: both norm weights or none");
  const int64_t Tn = qkv.size(0);
  auto q_out = at::empty({Tn, nq, D}, qkv.options());
  if (Tn == 0) return q_out;
  const int threads = 256;
  const int64_t warps = Tn * (nq + 2 * nkv);
  const int grid = (int)((warps * 32 + threads - 1) / threads);
  const bf16* qwp = qw.has_value() ? (const bf16*)qw->data_ptr() : nullptr;
  const bf16* kwp = kw.has_value() ? (const bf16*)kw->data_ptr() : nullptr;
#define CLB_QRA(DD)                                                                                                      \
  C10_CUDA_CHECK(launch_pdl(qkv_rope_append_kernel<DD>, dim3(grid), dim3(threads), 0, cur_stream(),                       \
      (const bf16*)qkv.data_ptr(), (int)qkv.stride(0), (int)nq, (int)nkv, qwp, kwp, pos.data_ptr<int64_t>(),             \
      inv_freq.data_ptr<float>(), slots.data_ptr<int64_t>(), (bf16*)q_out.data_ptr(), (bf16*)k_cache.data_ptr(),         \
      (bf16*)v_cache.data_ptr(), Tn, (float)eps, plp, S, (int64_t)(Tn * qkv.size(1))))
  if (D == 128) CLB_QRA(128);
  else if (D == 64) CLB_QRA(64);
  else TORCH_CHECK(false, "qkv_rope_append: head dim must be 64 or 128");
#undef CLB_QRA
  return q_out;
}

// x: a [T, n_heads*D] slice (row stride may exceed n_heads*D: the packed qkv row).
at::Tensor qk_norm_rope_fwd(const at::Tensor& x, int64_t n_heads, int64_t D, const c10::optional<at::Tensor>& w,
                            const at::Tensor& pos, const at::Tensor& inv_freq, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "qk_norm_rope: x must be [T, n*D] with unit inner stride");
  const int64_t Tn = x.size(0);
  auto out = at::empty({Tn, n_heads, D}, x.options());
  DISPATCH_FLOAT_BF16(x, "qk_norm_rope", [&] {
    launch_qk<scalar_t, false>((const scalar_t*)x.data_ptr(), (int)x.stride(0), (int)n_heads,
                               w.has_value() ? (const scalar_t*)w->data_ptr() : nullptr, pos.data_ptr<int64_t>(),
                               inv_freq.data_ptr<float>(), (scalar_t*)out.data_ptr(), nullptr, 0, nullptr, Tn,
                               (int)D, (float)eps);
  });
  return out;
}

// Writes dx into `dx_out` (same [T, n*D] strided view as x) and returns dw (fp32, [D]).
at::Tensor qk_norm_rope_bwd(const at::Tensor& dy, const at::Tensor& x, at::Tensor dx_out, int64_t n_heads,
                            int64_t D, const c10::optional<at::Tensor>& w, const at::Tensor& pos,
                            const at::Tensor& inv_freq, double eps) {
  const int64_t Tn = x.size(0);
  auto dw = at::zeros({D}, x.options().dtype(at::kFloat));
  auto dyc = dy.contiguous();
  TORCH_CHECK(dx_out.stride(1) == 1 && dx_out.stride(0) == x.stride(0) || true, "");
  DISPATCH_FLOAT_BF16(x, "qk_norm_rope_bwd", [&] {
    launch_qk<scalar_t, true>((const scalar_t*)dyc.data_ptr(), (int)dx_out.stride(0), (int)n_heads,
                              w.has_value() ? (const scalar_t*)w->data_ptr() : nullptr, pos.data_ptr<int64_t>(),
                              inv_freq.data_ptr<float>(), (scalar_t*)dx_out.data_ptr(),
                              (const scalar_t*)x.data_ptr(), (int)x.stride(0), dw.data_ptr<float>(), Tn, (int)D,
                              (float)eps);
  });
  return dw;
}

// ----------------------------------------------------------------------------- GRPO loss
// One pass: per-token clipped-ratio loss + k3 KL + entropy bonus, masked sums and
// the gradients w.r.t. logprob and entropy.  stats: [pg, kl, ent, clip+, clip-, ntok, total].
// Group-sequence variant (GSPO): `seq_sum` / `seq_cnt` hold, per packed sequence, the masked sum of the log-ratio
// and the number of masked tokens; every token of a sequence then uses the sequence mean as its log-ratio (its
// gradient still flows through the token's own log-prob: d = lp - sg(lp) + sg(mean)).
__global__ void grpo_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old,
                                 const float* __restrict__ ref, const float* __restrict__ adv,
                                 const float* __restrict__ mask, const float* __restrict__ ent,
                                 float* __restrict__ dlp, float* __restrict__ dent, float* __restrict__ stats,
                                 int64_t n, float pos_clip, float neg_clip, float diff_clip, float final_clip,
                                 float kl_coef, float ent_coef, float inv_norm,
                                 const int64_t* __restrict__ seq_ids = nullptr, const float* __restrict__ seq_sum = nullptr,
                                 const float* __restrict__ seq_cnt = nullptr) {
  __shared__ float red[32];
  float acc[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float m = mask[i], A = adv[i];
    float d = lp[i] - old[i];
    if (seq_ids != nullptr) {
      const int64_t sq = seq_ids[i];
      d = seq_sum[sq] / fmaxf(seq_cnt[sq], 1.f);
    }
    const float ratio = __expf(fminf(d, diff_clip));
    const float dr = (d <= diff_clip) ? ratio : 0.f;
    const float lo = 1.f - neg_clip, hi = 1.f + pos_clip;
    const float rc = fminf(fmaxf(ratio, lo), hi);
    const bool inside = (ratio >= lo) && (ratio <= hi);
    const float l1 = -A * ratio, l2 = -A * rc;
    const float mx = fmaxf(l1, l2);
    const float pg = fminf(mx, final_clip);
    float g = 0.f;
    if (mx <= final_clip) {
      const float g1 = -A * dr, g2 = inside ? -A * dr : 0.f;
      g = (l1 > l2) ? g1 : ((l1 < l2) ? g2 : 0.5f * (g1 + g2));
    }
    float kl = 0.f, gkl = 0.f;
    if (ref) {
      const float k = ref[i] - lp[i];
      const float e = __expf(k);
      const float raw = e - k - 1.f;
      kl = fminf(fmaxf(raw, -10.f), 10.f);
      gkl = (raw >= -10.f && raw <= 10.f) ? -(e - 1.f) : 0.f;
    }
    const float en = ent ? ent[i] : 0.f;
    dlp[i] = m * inv_norm * (g + kl_coef * gkl);
    if (dent) dent[i] = -m * inv_norm * ent_coef;
    acc[0] += pg * m;
    acc[1] += kl * m;
    acc[2] += en * m;
    acc[3] += (ratio > hi && A > 0.f) ? m : 0.f;
    acc[4] += (ratio < lo && A < 0.f) ? m : 0.f;
    acc[5] += m;
    acc[6] += m * (pg + kl_coef * kl - ent_coef * en);
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    float v = block_sum(acc[k], red);
    if (threadIdx.x == 0) atomicAdd(stats + k, v);
  }
}

// masked per-sequence sum of (lp - old) and token count of a packed row
__global__ void gspo_seq_sum_kernel(const float* __restrict__ lp, const float* __restrict__ old, const float* __restrict__ mask,
                                    const int64_t* __restrict__ seq_ids, float* __restrict__ seq_sum, float* __restrict__ seq_cnt,
                                    int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float m = mask[i];
    if (m != 0.f) {
      atomicAdd(seq_sum + seq_ids[i], (lp[i] - old[i]) * m);
      atomicAdd(seq_cnt + seq_ids[i], m);
    }
  }
}

// GSPO loss of a packed row with its gradient: same outputs as grpo_loss_fwd.  seq_ids [n] int64 in [0, num_seqs).
std::vector<at::Tensor> gspo_loss_fwd(const at::Tensor& lp, const at::Tensor& old, const c10::optional<at::Tensor>& ref,
                                      const at::Tensor& adv, const at::Tensor& mask, const c10::optional<at::Tensor>& ent,
                                      const at::Tensor& seq_ids, int64_t num_seqs, double pos_clip, double neg_clip,
                                      double diff_clip, double final_clip, double kl_coef, double ent_coef, double inv_norm) {
  const int64_t n = lp.numel();
  TORCH_CHECK(seq_ids.scalar_type() == at::kLong && seq_ids.numel() == n && seq_ids.is_contiguous(), "gspo_loss: int64 seq_ids [n]");
  auto dlp = at::empty_like(lp);
  auto dent = ent.has_value() ? at::empty_like(lp) : at::empty({0}, lp.options());
  auto stats = at::zeros({7}, lp.options());
  auto seq = at::zeros({2, std::max<int64_t>(num_seqs, 1)}, lp.options());
  if (n > 0) {
    int grid = (int)std::min<int64_t>((n + 255) / 256, 148 * 4);
    float* ssum = seq.data_ptr<float>();
    float* scnt = ssum + std::max<int64_t>(num_seqs, 1);
    gspo_seq_sum_kernel<<<grid, 256, 0, cur_stream()>>>(lp.data_ptr<float>(), old.data_ptr<float>(), mask.data_ptr<float>(),
                                                        seq_ids.data_ptr<int64_t>(), ssum, scnt, n);
    grpo_loss_kernel<<<grid, 256, 0, cur_stream()>>>(
        lp.data_ptr<float>(), old.data_ptr<float>(), ref.has_value() ? ref->data_ptr<float>() : nullptr,
        adv.data_ptr<float>(), mask.data_ptr<float>(), ent.has_value() ? ent->data_ptr<float>() : nullptr,
        dlp.data_ptr<float>(), ent.has_value() ? dent.data_ptr<float>() : nullptr, stats.data_ptr<float>(), n,
        (float)pos_clip, (float)neg_clip, (float)diff_clip, (float)final_clip, (float)kl_coef, (float)ent_coef,
        (float)inv_norm, seq_ids.data_ptr<int64_t>(), ssum, scnt);
  }
  return {stats, dlp, dent};
}

std::vector<at::Tensor> grpo_loss_fwd(const at::Tensor& lp, const at::Tensor& old,
                                      const c10::optional<at::Tensor>& ref, const at::Tensor& adv,
                                      const at::Tensor& mask, const c10::optional<at::Tensor>& ent,
                                      double pos_clip, double neg_clip, double diff_clip, double final_clip,
                                      double kl_coef, double ent_coef, double inv_norm) {
  const int64_t n = lp.numel();
  auto dlp = at::empty_like(lp);
  auto dent = ent.has_value() ? at::empty_like(lp) : at::empty({0}, lp.options());
  auto stats = at::zeros({7}, lp.options());
  if (n > 0) {
    int grid = (int)std::min<int64_t>((n + 255) / 256, 148 * 4);
    grpo_loss_kernel<<<grid, 256, 0, cur_stream()>>>(
        lp.data_ptr<float>(), old.data_ptr<float>(), ref.has_value() ? ref->data_ptr<float>() : nullptr,
        adv.data_ptr<float>(), mask.data_ptr<float>(), ent.has_value() ? ent->data_ptr<float>() : nullptr,
        dlp.data_ptr<float>(), ent.has_value() ? dent.data_ptr<float>() : nullptr, stats.data_ptr<float>(), n,
        (float)pos_clip, (float)neg_clip, (float)diff_clip, (float)final_clip, (float)kl_coef, (float)ent_coef,
        (float)inv_norm);
  }
  return {stats, dlp, dent};
}

// ----------------------------------------------------------------------------- AdamW
template <typename P>
__global__ void adamw_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, P* __restrict__ out, int64_t n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, const float* __restrict__ scale_ptr,
                             float scale_val) {
  const float scale = scale_ptr ? *scale_ptr : scale_val;
  for (int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4; i < n;
       i += (int64_t)gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 g4 = *reinterpret_cast<const float4*>(grad + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float4 p4 = *reinterpret_cast<float4*>(master + i);
      float* g = &g4.x; float* mm = &m4.x; float* vv = &v4.x; float* pp = &p4.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float gj = g[j] * scale;
        mm[j] = b1 * mm[j] + (1.f - b1) * gj;
        vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
        float denom = sqrtf(vv[j] / bc2) + eps;
        pp[j] = pp[j] * (1.f - lr * wd) - lr * (mm[j] / bc1) / denom;
      }
      *reinterpret_cast<float4*>(m + i) = m4;
      *reinterpret_cast<float4*>(v + i) = v4;
      *reinterpret_cast<float4*>(master + i) = p4;
      if (out) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[i + j] = Cvt<P>::from_f(pp[j]);
      }
    } else {
      for (int64_t k = i; k < n; ++k) {
        float gj = grad[k] * scale;
        float mk = b1 * m[k] + (1.f - b1) * gj;
        float vk = b2 * v[k] + (1.f - b2) * gj * gj;
        float pk = master[k] * (1.f - lr * wd) - lr * (mk / bc1) / (sqrtf(vk / bc2) + eps);
        m[k] = mk; v[k] = vk; master[k] = pk;
        if (out) out[k] = Cvt<P>::from_f(pk);
      }
    }
  }
}

void adamw_step(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                const c10::optional<at::Tensor>& out, int64_t step, double lr, double b1, double b2, double eps,
                double wd, const c10::optional<at::Tensor>& scale_t, double scale_v) {
  const int64_t n = master.numel();
  if (n == 0) return;
  TORCH_CHECK(master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat, "adamw: fp32 master/grad");
  TORCH_CHECK(((uintptr_t)master.data_ptr() % 16 == 0) && ((uintptr_t)grad.data_ptr() % 16 == 0) &&
              ((uintptr_t)m.data_ptr() % 16 == 0) && ((uintptr_t)v.data_ptr() % 16 == 0), "adamw: 16-byte alignment");
  const float bc1 = (float)(1.0 - std::pow(b1, (double)step)), bc2 = (float)(1.0 - std::pow(b2, (double)step));
  const float* sp = scale_t.has_value() ? scale_t->data_ptr<float>() : nullptr;
  int grid = (int)std::min<int64_t>((n / 4 + 255) / 256 + 1, 148 * 8);
  if (!out.has_value()) {
    adamw_kernel<float><<<grid, 256, 0, cur_stream()>>>(master.data_ptr<float>(), grad.data_ptr<float>(),
        m.data_ptr<float>(), v.data_ptr<float>(), nullptr, n, (float)lr, (float)b1, (float)b2, (float)eps,
        (float)wd, bc1, bc2, sp, (float)scale_v);
  } else if (out->scalar_type() == at::kBFloat16) {
    adamw_kernel<bf16><<<grid, 256, 0, cur_stream()>>>(master.data_ptr<float>(), grad.data_ptr<float>(),
        m.data_ptr<float>(), v.data_ptr<float>(), (bf16*)out->data_ptr(), n, (float)lr, (float)b1, (float)b2,
        (float)eps, (float)wd, bc1, bc2, sp, (float)scale_v);
  } else {
    adamw_kernel<float><<<grid, 256, 0, cur_stream()>>>(master.data_ptr<float>(), grad.data_ptr<float>(),
        m.data_ptr<float>(), v.data_ptr<float>(), out->data_ptr<float>(), n, (float)lr, (float)b1, (float)b2,
        (float)eps, (float)wd, bc1, bc2, sp, (float)scale_v);
  }
}

// ----------------------------------------------------------------------------- sum of squares
// Deterministic: fixed grid, per-CTA partials, second kernel adds them in order.
template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ part) {
  __shared__ float red[32];
  constexpr int V = Vec16<T>::N;
  float s = 0.f;
  // 16-byte loads, four in flight per thread; the (at most V - 1 + misaligned) elements at the ends go one by one
  const int64_t mis = (int64_t)(((16 - (reinterpret_cast<uintptr_t>(x) & 15)) & 15) / sizeof(T));
  const int64_t head = mis < n ? mis : n;
  const int64_t nvec = (n - head) / V;
  const T* xv = x + head;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
  int64_t v = tid;
  for (; v + 3 * stride < nvec; v += 4 * stride) {
    Vec16<T> a = ld16(xv + v * V), b = ld16(xv + (v + stride) * V), c = ld16(xv + (v + 2 * stride) * V),
             d = ld16(xv + (v + 3 * stride) * V);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float fa = Cvt<T>::to_f(a.v[j]), fb = Cvt<T>::to_f(b.v[j]), fc = Cvt<T>::to_f(c.v[j]), fd = Cvt<T>::to_f(d.v[j]);
      s += fa * fa + fb * fb + fc * fc + fd * fd;
    }
  }
  for (; v < nvec; v += stride) {
    Vec16<T> a = ld16(xv + v * V);
#pragma unroll
    for (int j = 0; j < V; ++j) { const float f = Cvt<T>::to_f(a.v[j]); s += f * f; }
  }
  for (int64_t i = tid; i < head; i += stride) { const float f = Cvt<T>::to_f(x[i]); s += f * f; }
  for (int64_t i = head + nvec * V + tid; i < n; i += stride) { const float f = Cvt<T>::to_f(x[i]); s += f * f; }
  s = block_sum(s, red);
  if (threadIdx.x == 0) part[blockIdx.x] = s;
}
__global__ void sumsq_final_kernel(const float* __restrict__ part, int n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += part[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = s;
}

at::Tensor sumsq(const at::Tensor& x) {
  auto out = at::zeros({}, x.options().dtype(at::kFloat));
  const int64_t n = x.numel();
  if (n == 0) return out;
  const int grid = (int)std::min<int64_t>((n + 8191) / 8192, 148 * 8);
  auto part = at::empty({grid}, x.options().dtype(at::kFloat));
  auto xc = x.contiguous();
  DISPATCH_FLOAT_BF16(xc, "sumsq", [&] {
    sumsq_partial_kernel<scalar_t><<<grid, 256, 0, cur_stream()>>>((const scalar_t*)xc.data_ptr(), n,
                                                                   part.data_ptr<float>());
  });
  sumsq_final_kernel<<<1, 256, 0, cur_stream()>>>(part.data_ptr<float>(), grid, out.data_ptr<float>());
  return out;
}
