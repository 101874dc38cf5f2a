// Decode attention of multi-head latent attention (MLA) in the absorbed form, over the paged latent cache.
//
// Every cached row is [normalised latent (DL = 512) | rotary key (DR = 64)] and is shared by all heads: the
// key up-projection is folded into the query and the value up-projection is applied to the output, so one
// decode step is, per sequence, S = Q K^T with Q [heads, 576] against the cached rows and O = softmax(S) K[:, :512].
// The reference leaves this to the MLA backends of vLLM / SGLang (chatlearn/models/vllm_module.py:442-469 only
// sizes the cache).
//
// One CTA (8 warps) per (sequence, tile of 16 heads, split of the context).  The 16 heads are the M dimension of
// m16n8k16 bf16 MMAs, so a cached row is read from HBM once for all of them.  Blocks of 64 cached rows (74 KB)
// stream through a two-stage cp.async ring.  Per block, in three phases separated by CTA barriers:
//   scores    warp w contracts a quarter of the 576 dims (w % 4; its slice of Q stays in 36 registers for the
//             whole kernel) against half of the keys (w / 4): every byte of the tile is read from shared memory
//             once, 4 independent accumulator chains per warp; the four partial sums go to shared memory as fp32;
//   softmax   warp w owns rows 2w and 2w + 1: adds the partials, masks, keeps the running maximum and sum of its
//             rows, writes the probabilities (bf16) and the rows' rescaling factors to shared memory;
//   output    warp w accumulates its own 64 of the 512 output columns over all 64 keys.
// ~30 FLOP per byte of cache: on a B200 the kernel is bound by the warp-level MMA rate and the barriers between
// the phases, not by HBM (a four-stage ring of half blocks, three loads in flight, was no faster).
#include <ATen/cuda/CUDAContext.h>
#include <cuda_pipeline.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int BS = 64;            // cached rows per block
constexpr int kPad = 8;           // row padding (elements): keeps ldmatrix rows on distinct banks

constexpr int kSPad = 8;          // fp32 padding of the partial-score rows

template <int DL, int DR>
struct SmemMLA {
  bf16 k[2][BS][DL + DR + kPad];  // stage 1 also stages Q before the first prefetch lands there
  float sp[4][16][BS + kSPad];    // partial scores of the four quarters of the contraction
  bf16 p[16][BS + kPad];
  float alpha[16];
  float row_m[16];
  float row_l[16];
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// rows past `valid` are zero-filled: their probabilities are 0, and 0 * garbage must not become NaN
template <int DL, int DR>
__device__ __forceinline__ void load_rows(SmemMLA<DL, DR>* sm, int stage, const bf16* cache, int64_t block_id, int valid) {
  constexpr int D = DL + DR, CH = D / 8;
  const bf16* src = cache + block_id * BS * (int64_t)D;
  for (int i = threadIdx.x; i < BS * CH; i += kThreads) {
    const int r = i / CH, c = (i % CH) * 8;
    if (r < valid) {
      __pipeline_memcpy_async(&sm->k[stage][r][c], src + (int64_t)r * D + c, 16);
    } else {
      *reinterpret_cast<uint4*>(&sm->k[stage][r][c]) = make_uint4(0, 0, 0, 0);
    }
  }
}

template <int DL, int DR>
__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ cache, const int* __restrict__ block_tables,
                  int max_blocks, const int* __restrict__ ctx_len, bf16* __restrict__ out, float* __restrict__ part_o,
                  float* __restrict__ part_lse, int nh, int num_splits, float scale) {
  constexpr int D = DL + DR;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  auto* sm = reinterpret_cast<SmemMLA<DL, DR>*>(smem_raw);
  const int seq = blockIdx.x, ht = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int len = ctx_len[seq];
  const int nblk = (len + BS - 1) / BS;
  const int per = (nblk + num_splits - 1) / num_splits;
  const int b0 = split * per, b1 = min(b0 + per, nblk);
  const int h0 = ht * 16;
  if (b0 >= b1) {                                          // nothing for this split (or an empty sequence)
    for (int r = tid; r < 16; r += kThreads) {
      if (h0 + r >= nh) continue;
      if (part_lse != nullptr) part_lse[((int64_t)seq * nh + h0 + r) * num_splits + split] = -INFINITY;
      else for (int d = 0; d < DL; ++d) out[((int64_t)seq * nh + h0 + r) * DL + d] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int* bt = block_tables + (int64_t)seq * max_blocks;
  load_rows<DL, DR>(sm, 0, cache, bt[b0], min(BS, len - b0 * BS));
  __pipeline_commit();
  // Q through the (still unused) second stage into registers: this warp's quarter of the contraction
  constexpr int KQ = D / 16 / 4;                           // 9 k-steps per quarter
  static_assert(D % 64 == 0 && KQ * 64 == D, "the contraction splits into four quarters of whole k-steps");
  bf16 (*qs)[D + kPad] = sm->k[1];
  for (int i = tid; i < 16 * (D / 8); i += kThreads) {
    const int r = i / (D / 8), c = (i % (D / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + r < nh) v = *reinterpret_cast<const uint4*>(q + ((int64_t)seq * nh + h0 + r) * D + c);
    *reinterpret_cast<uint4*>(&qs[r][c]) = v;
  }
  __syncthreads();
  const int kq = warp & 3, kh = warp >> 2;
  uint32_t qa[KQ][4];
#pragma unroll
  for (int j = 0; j < KQ; ++j) ldsm_x4(qa[j], &qs[lane & 15][(kq * KQ + j) * 16 + (lane >> 4) * 8]);
  __syncthreads();

  float o_acc[DL / kWarps / 8][4];
#pragma unroll
  for (int n = 0; n < DL / kWarps / 8; ++n) o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};                 // rows 2 * warp and 2 * warp + 1 (uniform over the lanes)
  float l_run[2] = {0.f, 0.f};                             // this lane's share of those rows' sums
  const int col0 = warp * (DL / kWarps);                   // this warp's output columns

  for (int b = b0; b < b1; ++b) {
    const int st = (b - b0) & 1;
    if (b + 1 < b1) load_rows<DL, DR>(sm, st ^ 1, cache, bt[b + 1], min(BS, len - (b + 1) * BS));
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    // ---- partial scores: 16 rows x 32 keys over this warp's quarter of the contraction ----
    {
      float s[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int j = 0; j < KQ; ++j) {
        const int kc = (kq * KQ + j) * 16 + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t kb[4];
          ldsm_x4(kb, &sm->k[st][kh * 32 + h * 16 + (lane & 7) + ((lane >> 4) & 1) * 8][kc]);
          mma16816(s[2 * h], qa[j], kb[0], kb[1]);
          mma16816(s[2 * h + 1], qa[j], kb[2], kb[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const int c = kh * 32 + n * 8 + 2 * t;
        *reinterpret_cast<float2*>(&sm->sp[kq][g][c]) = make_float2(s[n][0], s[n][1]);
        *reinterpret_cast<float2*>(&sm->sp[kq][g + 8][c]) = make_float2(s[n][2], s[n][3]);
      }
    }
    __syncthreads();
    // ---- softmax of this warp's two rows over the 64 keys (two per lane) ----
    {
      const int key = b * BS + 2 * lane;
      const bool v0 = key < len, v1 = key + 1 < len;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = 2 * warp + r;
        float2 a = *reinterpret_cast<const float2*>(&sm->sp[0][row][2 * lane]);
#pragma unroll
        for (int k4 = 1; k4 < 4; ++k4) {
          const float2 x = *reinterpret_cast<const float2*>(&sm->sp[k4][row][2 * lane]);
          a.x += x.x; a.y += x.y;
        }
        const float s0 = v0 ? a.x * scale : -INFINITY, s1 = v1 ? a.y * scale : -INFINITY;
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_run[r], mx);           // finite: the block holds at least one valid key
        const float al = __expf(m_run[r] - m_new);
        const float p0 = __expf(s0 - m_new), p1 = __expf(s1 - m_new);
        l_run[r] = l_run[r] * al + p0 + p1;
        m_run[r] = m_new;
        *reinterpret_cast<uint32_t*>(&sm->p[row][2 * lane]) = pack2(p0, p1);
        if (lane == 0) sm->alpha[row] = al;
      }
    }
    __syncthreads();
    // ---- this warp's 64 output columns over all 64 keys ----
    {
      const float a0 = sm->alpha[g], a1 = sm->alpha[g + 8];
#pragma unroll
      for (int n = 0; n < DL / kWarps / 8; ++n) {
        o_acc[n][0] *= a0; o_acc[n][1] *= a0; o_acc[n][2] *= a1; o_acc[n][3] *= a1;
      }
#pragma unroll
      for (int kk = 0; kk < BS / 16; ++kk) {
        uint32_t pa[4];
        ldsm_x4(pa, &sm->p[lane & 15][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
        for (int n = 0; n < DL / kWarps / 8; n += 2) {
          uint32_t vb[4];
          ldsm_x4_trans(vb, &sm->k[st][kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)][col0 + (n + (lane >> 4)) * 8]);
          mma16816(o_acc[n], pa, vb[0], vb[1]);
          mma16816(o_acc[n + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();
  }
  __pipeline_wait_prior(0);
  // ---- row sums: over the lanes of the owning warp, then to everybody ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], o);
    if (lane == 0) { sm->row_l[2 * warp + r] = l_run[r]; sm->row_m[2 * warp + r] = m_run[r]; }
  }
  __syncthreads();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    if (h0 + r >= nh) continue;
    const float l = sm->row_l[r];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int64_t row = (int64_t)seq * nh + h0 + r;
    if (part_o != nullptr) {
      float* po = part_o + (row * num_splits + split) * DL + col0;
#pragma unroll
      for (int n = 0; n < DL / kWarps / 8; ++n)
        *reinterpret_cast<float2*>(po + n * 8 + 2 * t) = make_float2(o_acc[n][2 * h] * inv, o_acc[n][2 * h + 1] * inv);
      if (warp == 0 && t == 0) part_lse[row * num_splits + split] = l > 0.f ? sm->row_m[r] + logf(l) : -INFINITY;
    } else {
      bf16* o = out + row * DL + col0;
#pragma unroll
      for (int n = 0; n < DL / kWarps / 8; ++n)
        *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * t) = pack2(o_acc[n][2 * h] * inv, o_acc[n][2 * h + 1] * inv);
    }
  }
}

template <int DL>
__global__ void mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                   bf16* __restrict__ out, int num_splits) {
  const int64_t row = blockIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, part_lse[row * num_splits + s]);
  for (int d = threadIdx.x; d < DL; d += blockDim.x) {
    float den = 0.f, o = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float l = part_lse[row * num_splits + s];
      if (l == -INFINITY) continue;
      const float w = __expf(l - mx);
      den += w;
      o += w * part_o[(row * num_splits + s) * DL + d];
    }
    out[row * DL + d] = __float2bfloat16_rn(den > 0.f ? o / den : 0.f);
  }
}

}  // namespace

// q [B, heads, 576] bf16 (one query token per sequence, latent | rotary parts); cache [blocks, 64, 1, 576] bf16;
// block_tables [B, max_blocks] int32; ctx_len [B] int32 (including the new token).  Returns [B, heads, 512] bf16.
at::Tensor mla_paged_decode(const at::Tensor& q, const at::Tensor& cache, const at::Tensor& block_tables,
                            const at::Tensor& ctx_len, double scale, int64_t num_splits) {
  constexpr int DL = 512, DR = 64;
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 3 && q.size(2) == DL + DR && q.is_contiguous(),
              "mla_paged_decode: q must be contiguous bf16 [B, heads, 576]");
  TORCH_CHECK(cache.scalar_type() == at::kBFloat16 && cache.is_contiguous() && cache.size(-1) == DL + DR &&
                  cache.dim() == 4 && cache.size(1) == BS && cache.size(2) == 1,
              "mla_paged_decode: cache must be contiguous bf16 [blocks, 64, 1, 576]");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.is_contiguous() && block_tables.size(0) == q.size(0) &&
                  ctx_len.scalar_type() == at::kInt && ctx_len.numel() == q.size(0),
              "mla_paged_decode: int32 block_tables [B, max_blocks] and ctx_len [B]");
  const int B = (int)q.size(0), nh = (int)q.size(1);
  auto out = at::empty({B, nh, DL}, q.options());
  if (B == 0) return out;
  const int tiles = (nh + 15) / 16;
  int ns = (int)num_splits;
  if (ns <= 0) {                                            // fill the SMs when the batch alone does not
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    ns = std::max(1, std::min(8, sms / std::max(B * tiles, 1)));
  }
  const int dev = q.get_device();
  TORCH_CHECK(dev >= 0 && dev < 64, "mla_paged_decode: device index out of range");
  static bool configured[64] = {};
  const size_t smem = sizeof(SmemMLA<DL, DR>);
  if (!configured[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(mla_decode_kernel<DL, DR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  auto st = at::cuda::getCurrentCUDAStream();
  at::Tensor po, pl;
  float* pop = nullptr; float* plp = nullptr;
  if (ns > 1) {
    po = at::empty({B, nh, ns, DL}, q.options().dtype(at::kFloat));
    pl = at::empty({B, nh, ns}, q.options().dtype(at::kFloat));
    pop = po.data_ptr<float>(); plp = pl.data_ptr<float>();
  }
  dim3 grid(B, tiles, ns);
  mla_decode_kernel<DL, DR><<<grid, kThreads, smem, st>>>(
      (const bf16*)q.data_ptr(), (const bf16*)cache.data_ptr(), block_tables.data_ptr<int>(), (int)block_tables.size(1),
      ctx_len.data_ptr<int>(), (bf16*)out.data_ptr(), pop, plp, nh, ns, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  if (ns > 1) {
    mla_combine_kernel<DL><<<B * nh, 256, 0, st>>>(pop, plp, (bf16*)out.data_ptr(), ns);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return out;
}
