// Variable-length causal attention, forward (packed sequences, GQA).
//
// FlashAttention-style streaming softmax: a CTA owns 128 query rows of one sequence and
// one query head; its 8 warps own 16 rows each.  K/V tiles of 64 rows stream through a
// two-stage cp.async ring; S = Q K^T and O += P V run on m16n8k16 bf16 tensor-core MMAs
// with fp32 accumulators; the S accumulators are re-packed in registers as the A operand
// of the second product, so nothing but Q, K and V tiles ever touches shared memory.
// Work is listed longest-first (the last query tile of a sequence sees the most keys).
// Used for prompt prefill and for all forward-only scoring passes; also writes the
// log-sum-exp per row.
#include <ATen/cuda/CUDAContext.h>
#include <cuda_pipeline.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kThreads = 256;
constexpr int BM = 128, BN = 64;
constexpr int kPad = 8;

template <int D>
struct SmemFwd {
  bf16 q[BM][D + kPad];
  bf16 k[2][BN][D + kPad];
  bf16 v[2][BN][D + kPad];
  int seq, tile;
};

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], const void* p) {
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

// rows [r0, r0+BN) of one head (row stride `rs` elements) into a tile; rows at or past `valid` are zeroed
template <int D, int ROWS>
__device__ __forceinline__ void load_rows(bf16 (*dst)[D + kPad], const bf16* src, int64_t rs, int valid) {
  constexpr int CH = D / 8;
  for (int c = threadIdx.x; c < ROWS * CH; c += kThreads) {
    const int r = c / CH, o = (c % CH) * 8;
    if (r < valid) __pipeline_memcpy_async(&dst[r][o], src + (int64_t)r * rs + o, 16);
    else *reinterpret_cast<uint4*>(&dst[r][o]) = make_uint4(0, 0, 0, 0);
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
attn_varlen_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                       const int* __restrict__ cu, int num_seqs, bf16* __restrict__ out, float* __restrict__ lse,
                       int64_t q_rs, int64_t k_rs, int64_t v_rs, int nq, int nkv, int total_rows, float scale, int causal) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  auto* sm = reinterpret_cast<SmemFwd<D>*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int head = blockIdx.y, kvh = head / (nq / nkv);
  // which (sequence, query tile) is mine: tiles are numbered sequence by sequence; the grid walks them backwards
  if (tid == 0) {
    int want = (int)gridDim.x - 1 - (int)blockIdx.x, seq = -1, tile = 0;
    for (int s = 0, acc = 0; s < num_seqs; ++s) {
      const int nt = (cu[s + 1] - cu[s] + BM - 1) / BM;
      if (want < acc + nt) { seq = s; tile = want - acc; break; }
      acc += nt;
    }
    sm->seq = seq; sm->tile = tile;
  }
  __syncthreads();
  const int seq = sm->seq;
  if (seq < 0) return;
  const int start = cu[seq], len = cu[seq + 1] - start;
  const int q0 = sm->tile * BM;
  const int q_valid = min(BM, len - q0);
  const int n_kv_tiles = causal ? min((len + BN - 1) / BN, (q0 + BM + BN - 1) / BN) : (len + BN - 1) / BN;

  load_rows<D, BM>(sm->q, q + ((int64_t)(start + q0)) * q_rs + (int64_t)head * D, q_rs, q_valid);
  load_rows<D, BN>(sm->k[0], k + (int64_t)start * k_rs + (int64_t)kvh * D, k_rs, min(BN, len));
  load_rows<D, BN>(sm->v[0], v + (int64_t)start * v_rs + (int64_t)kvh * D, v_rs, min(BN, len));
  __pipeline_commit();
  __pipeline_wait_prior(0);
  __syncthreads();

  float o_acc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) { o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row0 = q0 + warp * 16 + g;            // this thread's rows: row0 and row0 + 8 (inside the sequence)
  const float sl2 = scale * 1.4426950408889634f;  // softmax in base 2

  for (int j = 0; j < n_kv_tiles; ++j) {
    const int st = j & 1;
    if (j + 1 < n_kv_tiles) {
      const int r0 = (j + 1) * BN;
      load_rows<D, BN>(sm->k[st ^ 1], k + (int64_t)(start + r0) * k_rs + (int64_t)kvh * D, k_rs, min(BN, len - r0));
      load_rows<D, BN>(sm->v[st ^ 1], v + (int64_t)(start + r0) * v_rs + (int64_t)kvh * D, v_rs, min(BN, len - r0));
    }
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const int kv0 = j * BN;
    // a warp whose 16 rows lie wholly above this tile's diagonal (or past the sequence) has nothing to add
    const bool active = !(causal && kv0 > q0 + warp * 16 + 15) && (q0 + warp * 16 < len);
    if (active) {
    // ---- S = Q K^T: 16 rows x 64 keys per warp ----
    // Q fragments are re-read from shared memory per k-step (two ldmatrix per 16 MMAs) instead of
    // living in 32 registers: that keeps the kernel at two CTAs per SM
    float s[BN / 8][4];
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ks += 2) {
      uint32_t qa0[4], qa1[4];
      ldsm4(qa0, &sm->q[warp * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
      ldsm4(qa1, &sm->q[warp * 16 + (lane & 15)][(ks + 1) * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int n = 0; n < BN / 8; ++n) {
        uint32_t kb[4];
        ldsm4(kb, &sm->k[st][n * 8 + (lane & 7)][ks * 16 + (lane >> 3) * 8]);
        mma16816(s[n], qa0, kb[0], kb[1]);
        mma16816(s[n], qa1, kb[2], kb[3]);
      }
    }
    // ---- mask + online softmax (rows row0 and row0+8) ----
    const bool edge = (kv0 + BN > len) || (causal && kv0 + BN > q0 + warp * 16);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // raw scores are kept; the scale (> 0) is folded into the exponent below
        if (edge) {
          const int col = kv0 + n * 8 + 2 * t + (e & 1);
          const int row = row0 + (e >> 1) * 8;
          if (col >= len || (causal && col > row)) s[n][e] = -INFINITY;
        }
        mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);          // running maximum of the raw scores
      m_use[h] = (m_new == -INFINITY) ? 0.f : m_new * sl2;   // a row with no visible key yet: any finite value
      alpha[h] = exp2f(m_run[h] * sl2 - m_use[h]);
      m_run[h] = m_new;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f(fmaf(s[n][e], sl2, -m_use[e >> 1]));
        s[n][e] = p;
        ps[e >> 1] += p;
      }
    }
    l_run[0] = l_run[0] * alpha[0] + ps[0];
    l_run[1] = l_run[1] * alpha[1] + ps[1];
    // the maximum rarely moves after the first tiles: skip the rescale when no row of the warp needs it
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        o_acc[n][0] *= alpha[0]; o_acc[n][1] *= alpha[0];
        o_acc[n][2] *= alpha[1]; o_acc[n][3] *= alpha[1];
      }
    }
    // ---- O += P V ----
#pragma unroll
    for (int ks = 0; ks < BN / 16; ++ks) {
      uint32_t pa[4];
      pa[0] = pack2(s[2 * ks][0], s[2 * ks][1]);
      pa[1] = pack2(s[2 * ks][2], s[2 * ks][3]);
      pa[2] = pack2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pa[3] = pack2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int n = 0; n < D / 8; n += 2) {
        uint32_t vb[4];
        ldsm4t(vb, &sm->v[st][ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)][(n + (lane >> 4)) * 8]);
        mma16816(o_acc[n], pa, vb[0], vb[1]);
        mma16816(o_acc[n + 1], pa, vb[2], vb[3]);
      }
    }
    }
    __syncthreads();
  }
  // ---- finish: O / l, log-sum-exp ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = row0 + h * 8;
    if (row >= len) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    bf16* o = out + ((int64_t)(start + row) * nq + head) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(o + n * 8 + 2 * t) = pack2(o_acc[n][2 * h] * inv, o_acc[n][2 * h + 1] * inv);
    if (lse != nullptr && t == 0)
      lse[(int64_t)head * total_rows + start + row] = l_run[h] > 0.f ? m_run[h] * scale + logf(l_run[h]) : -INFINITY;
  }
}

}  // namespace

bool attn_varlen_fwd_supported(int64_t head_dim) { return head_dim == 128 || head_dim == 64; }

// q [T, nq, D], k/v [T, nkv, D] bf16 (rows may be strided: views of a fused QKV tensor), cu_seqlens [B+1] int32.
// Returns {out [T, nq, D] bf16, lse [nq, T] fp32}.
std::vector<at::Tensor> attn_varlen_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                        const at::Tensor& cu_seqlens, double scale, bool causal) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "attn_varlen_fwd: bf16 CUDA tensors");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "attn_varlen_fwd: [T, heads, D]");
  const int64_t T = q.size(0), nq = q.size(1), D = q.size(2), nkv = k.size(1);
  TORCH_CHECK(attn_varlen_fwd_supported(D) && k.size(2) == D && v.size(2) == D && nq % nkv == 0, "attn_varlen_fwd: head_dim 64 or 128");
  for (const at::Tensor* x : {&q, &k, &v})
    TORCH_CHECK(x->stride(2) == 1 && x->stride(1) == D && x->stride(0) % 8 == 0 && (uintptr_t)x->data_ptr() % 16 == 0,
                "attn_varlen_fwd: heads must be contiguous and rows 16-byte aligned");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_cuda() && cu_seqlens.is_contiguous(), "cu_seqlens: int32 CUDA");
  const int B = (int)cu_seqlens.numel() - 1;
  auto out = at::empty({T, nq, D}, q.options());
  auto lse = at::empty({nq, T}, q.options().dtype(at::kFloat));
  if (T == 0 || B <= 0) return {out, lse};
  const int tiles = (int)((T + BM - 1) / BM) + B;       // upper bound; surplus CTAs exit
  dim3 grid(tiles, (unsigned)nq);
  auto st = at::cuda::getCurrentCUDAStream();
  if (D == 128) {
    const size_t smem = sizeof(SmemFwd<128>);
    static bool cfg[64] = {};                    // the attribute is per device
    const int dev = q.get_device();
    if (!cfg[dev & 63]) { cudaFuncSetAttribute(attn_varlen_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); cfg[dev & 63] = true; }
    attn_varlen_fwd_kernel<128><<<grid, kThreads, smem, st>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(),
        (const bf16*)v.data_ptr(), cu_seqlens.data_ptr<int>(), B, (bf16*)out.data_ptr(), lse.data_ptr<float>(), q.stride(0),
        k.stride(0), v.stride(0), (int)nq, (int)nkv, (int)T, (float)scale, causal ? 1 : 0);
  } else {
    const size_t smem = sizeof(SmemFwd<64>);
    static bool cfg[64] = {};
    const int dev = q.get_device();
    if (!cfg[dev & 63]) { cudaFuncSetAttribute(attn_varlen_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); cfg[dev & 63] = true; }
    attn_varlen_fwd_kernel<64><<<grid, kThreads, smem, st>>>((const bf16*)q.data_ptr(), (const bf16*)k.data_ptr(),
        (const bf16*)v.data_ptr(), cu_seqlens.data_ptr<int>(), B, (bf16*)out.data_ptr(), lse.data_ptr<float>(), q.stride(0),
        k.stride(0), v.stride(0), (int)nq, (int)nkv, (int)T, (float)scale, causal ? 1 : 0);
  }
  return {out, lse};
}
