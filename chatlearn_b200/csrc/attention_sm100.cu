// Variable-length attention forward on the 5th-generation tensor cores (head dim 128, bf16,
// packed sequences, GQA, causal or full).
//
// A CTA owns 128 query rows of one sequence and one query head; two CTAs share an SM, so one
// CTA's softmax overlaps the other's matrix products.  Roles inside a CTA (192 threads):
//   warp 0      TMA producer: the Q tile once, then K and V tiles of 64 keys through two
//               2-stage rings (128-byte swizzle, one mbarrier per stage, no multicast)
//   warp 1      MMA issuer (one thread): S = Q K^T (tcgen05.mma 128x64x16, both operands
//               K-major) into one of two S accumulators in tensor memory, so the product for
//               key block j+1 runs while block j is in the softmax; O += P V (128x128x16, P
//               K-major from shared memory, V as an MN-major operand straight from its
//               row-major tile) into the O accumulator, which stays in tensor memory for
//               the whole row of key blocks
//   warps 2..5  softmax: thread = query row.  tcgen05.ld the 64 scores of the row, mask,
//               running maximum and sum without any shuffle, P = exp2(.) as bf16 into the
//               swizzled shared-memory tile the second product reads.  The accumulator is
//               rescaled lazily: exponentials are taken against a reference maximum that
//               is only moved (and O multiplied in tensor memory, tcgen05.ld/st) when the
//               true maximum has run ahead of it by more than 2^8; the result is exact,
//               the rescale is rare.
// Epilogue: O / l is staged through the (then free) Q tile and written with 256-byte
// row segments; the log-sum-exp per row is kept for the backward pass.
// Every mbarrier wait is bounded; a wait that runs out records a status code, the CTA
// drains and frees its tensor memory.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "sm100.cuh"
#include "tmap.h"

using namespace sm100;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 128, BN = 64, D = 128;
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;               // S[2] at columns 0 and 64, O at column 128
constexpr uint32_t kChunk = 64 * 128;        // one TMA box of K or V: 64 rows x 128 bytes
constexpr float kRescaleLog2 = 8.f;

struct SmemFwd {
  uint8_t q[2][BM * 128];                    // two 64-wide slices of the head dim, 128 rows x 128 bytes each
  uint8_t k[kStages][2][kChunk];
  uint8_t v[kStages][2][kChunk];
  uint8_t p[BM * 128];                       // P tile: 128 rows x 64 keys, bf16, K-major with the 128-byte swizzle
  uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], s_empty[2], p_full, pv_done;
  uint32_t tmem_base, abort_flag;
  int seq, tile;
};

__device__ int g_attn_status = 0;
enum : int { ST_OK = 0, ST_PRODUCER = 1, ST_MMA = 2, ST_SOFTMAX = 3, ST_SMEM_ALIGN = 4 };

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const int* __restrict__ cu_seqlens, int num_seqs,
                      bf16* __restrict__ out, float* __restrict__ lse, int nq, int nkv, int total_rows, float scale,
                      int causal) {
  extern __shared__ uint8_t smem_raw[];
  SmemFwd* sm = reinterpret_cast<SmemFwd*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;

  // ---- which (sequence, query tile) is this CTA's: the tiles of a sequence are listed last-first, so the
  // tiles with the most key blocks are scheduled before the short ones
  if (threadIdx.x == 0) {
    int left = blockIdx.x, seq = -1, tile = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int nt = (cu_seqlens[s + 1] - cu_seqlens[s] + BM - 1) / BM;
      if (left < nt) { seq = s; tile = nt - 1 - left; break; }
      left -= nt;
    }
    sm->seq = seq; sm->tile = tile;
    if ((smem_u32(smem_raw) & 1023u) != 0u) { sm->seq = -1; atomicCAS(&g_attn_status, ST_OK, ST_SMEM_ALIGN); }
  }
  __syncthreads();
  const int seq = sm->seq;
  if (seq < 0) return;                         // surplus CTA of the over-sized grid (nothing allocated yet)
  const int start = cu_seqlens[seq], len = cu_seqlens[seq + 1] - start;
  const int r0 = sm->tile * BM;                // first query row of the tile, relative to the sequence
  const int kv_end = causal ? min(len, r0 + BM) : len;
  const int nblk = (kv_end + BN - 1) / BN;     // >= 1: the tile holds at least one valid row

  if (threadIdx.x == 0) {
    mbar_init(&sm->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm->k_full[s], 1); mbar_init(&sm->k_empty[s], 1);
      mbar_init(&sm->v_full[s], 1); mbar_init(&sm->v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(&sm->s_full[b], 1); mbar_init(&sm->s_empty[b], 4); }
    mbar_init(&sm->p_full, 128);
    mbar_init(&sm->pv_done, 1);
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

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      const int kvh = head / (nq / nkv);
      mbar_expect_tx(&sm->q_full, 2 * BM * 128);
      tma_load_2d(sm->q[0], &tmQ, &sm->q_full, head * D, start + r0);
      tma_load_2d(sm->q[1], &tmQ, &sm->q_full, head * D + 64, start + r0);
      bool ok = true;
      uint32_t stage = 0, phase = 0;
      for (int j = 0; j < nblk && ok; ++j) {
        const int row = start + j * BN;
        if (!mbar_wait(&sm->k_empty[stage], phase ^ 1)) { ok = false; break; }
        mbar_expect_tx(&sm->k_full[stage], 2 * kChunk);
        tma_load_2d(sm->k[stage][0], &tmK, &sm->k_full[stage], kvh * D, row);
        tma_load_2d(sm->k[stage][1], &tmK, &sm->k_full[stage], kvh * D + 64, row);
        if (!mbar_wait(&sm->v_empty[stage], phase ^ 1)) { ok = false; break; }
        mbar_expect_tx(&sm->v_full[stage], 2 * kChunk);
        tma_load_2d(sm->v[stage][0], &tmV, &sm->v_full[stage], kvh * D, row);
        tma_load_2d(sm->v[stage][1], &tmV, &sm->v_full[stage], kvh * D + 64, row);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) { atomicCAS(&g_attn_status, ST_OK, ST_PRODUCER); atomicExch(&sm->abort_flag, 1u); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BM, D, 0, 1);
      const uint32_t o_tmem = tmem_base + 128;
      bool ok = mbar_wait(&sm->q_full, 0);
      tc_fence_after_sync();
      // O += P(i) V(i): issued one key block behind the scores, so the tensor core always has the next
      // S = Q K^T to run while the softmax warps turn block i into P
      auto issue_pv = [&](int i) -> bool {
        const uint32_t st = i % kStages, ph = (i / kStages) & 1;
        if (!mbar_wait(&sm->v_full[st], ph)) return false;
        if (!mbar_wait(&sm->p_full, i & 1)) return false;
        tc_fence_after_sync();
        const uint64_t dp = make_kmajor_sw128_desc(smem_u32(sm->p));
        const uint64_t dv = make_mnmajor_sw128_desc(smem_u32(sm->v[st][0]), kChunk);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_bf16(o_tmem, dp + 2ull * kk, dv + 128ull * kk, idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sm->v_empty[st]);
        umma_commit(&sm->pv_done);
        return true;
      };
      for (int j = 0; j < nblk && ok; ++j) {
        const uint32_t st = j % kStages, ph = (j / kStages) & 1, b = j & 1;
        if (!mbar_wait(&sm->k_full[st], ph)) { ok = false; break; }
        if (!mbar_wait(&sm->s_empty[b], ((j >> 1) & 1) ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t dq = make_kmajor_sw128_desc(smem_u32(sm->q[kk >> 2])) + 2ull * (kk & 3);
          const uint64_t dk = make_kmajor_sw128_desc(smem_u32(sm->k[st][kk >> 2])) + 2ull * (kk & 3);
          umma_bf16(tmem_base + b * BN, dq, dk, idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sm->k_empty[st]);
        umma_commit(&sm->s_full[b]);
        if (j > 0 && !issue_pv(j - 1)) { ok = false; break; }
      }
      if (ok) ok = issue_pv(nblk - 1);
      if (!ok) { atomicCAS(&g_attn_status, ST_OK, ST_MMA); atomicExch(&sm->abort_flag, 1u); }
    }
  } else {
    // ------------------------------------------------ softmax + epilogue (warps 2..5), thread = query row
    const int quarter = warp & 3;                 // the tensor-memory lane quarter this warp may access
    const int row = quarter * 32 + lane;          // row of the tile
    const int qrow = r0 + row;                    // row of the sequence
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float c = scale * 1.4426950408889634f;  // scores -> log2 units
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const uint32_t b = j & 1;
      if (!mbar_wait(&sm->s_full[b], (j >> 1) & 1)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s0[32], s1[32];
      tmem_ld_32x32(lane_addr + b * BN, s0);
      tmem_ld_32x32(lane_addr + b * BN + 32, s1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->s_empty[b]);          // the scores are in registers: the buffer may be overwritten
      const int k0 = j * BN;
      if (k0 + BN > len || (causal && k0 + BN - 1 > r0)) {  // block crosses the diagonal or the end of the sequence
        const int lim = causal ? min(len - 1, qrow) : len - 1;   // last visible key of this row
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (k0 + i > lim) s0[i] = 0xff800000u;
          if (k0 + 32 + i > lim) s1[i] = 0xff800000u;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
      // P(j-1) must have been consumed before the tile is overwritten, and O must be at rest before it is rescaled
      if (j > 0 && !mbar_wait(&sm->pv_done, (j - 1) & 1)) { ok = false; break; }
      if (j == 0) {
        m_ref = mx;
      } else {
        const bool need = (mx - m_ref) * c > kRescaleLog2;
        if (__any_sync(0xffffffffu, need)) {
          tc_fence_after_sync();
          const float alpha = need ? fast_exp2((m_ref - mx) * c) : 1.f;
          if (need) { m_ref = mx; l *= alpha; }
#pragma unroll 1
          for (int cc = 0; cc < D; cc += 32) {
            uint32_t o[32];
            tmem_ld_32x32(lane_addr + 128 + cc, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(lane_addr + 128 + cc, o);
          }
          tmem_st_wait();
        }
      }
      const float off = m_ref * c;
      float sum = 0.f;
      uint8_t* prow = sm->p + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = (ch & 3) * 8 + 2 * i;
          const float x0 = __uint_as_float(ch < 4 ? s0[e] : s1[e]), x1 = __uint_as_float(ch < 4 ? s0[e + 1] : s1[e + 1]);
          const float p0 = fast_exp2(fmaf(x0, c, -off)), p1 = fast_exp2(fmaf(x1, c, -off));
          sum += p0 + p1;
          w[i] = pack_bf16(p0, p1);
        }
        *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l += sum;
      fence_proxy_async();          // the tile was written through the generic proxy; the tensor core reads it through the async one
      tc_fence_before_sync();
      mbar_arrive(&sm->p_full);
    }
    if (ok && !mbar_wait(&sm->pv_done, (nblk - 1) & 1)) ok = false;
    if (ok) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      // stage the row through the Q tile (no product reads it any more): 16-byte chunk c of row r sits at
      // chunk (c ^ (r & 15)), so neither the row-wise writes nor the row-segment reads collide on banks
      uint8_t* stage = sm->q[0];
#pragma unroll 1
      for (int cc = 0; cc < D; cc += 32) {
        uint32_t o[32];
        tmem_ld_32x32(lane_addr + 128 + cc, o);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            w[i] = pack_bf16(__uint_as_float(o[g * 8 + 2 * i]) * inv, __uint_as_float(o[g * 8 + 2 * i + 1]) * inv);
          const int chunk = cc / 8 + g;
          *reinterpret_cast<uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      __syncwarp();
#pragma unroll 1
      for (int i = 0; i < 16; ++i) {
        const int rr = quarter * 32 + 2 * i + (lane >> 4), chunk = lane & 15;
        if (r0 + rr < len) {
          const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((chunk ^ (rr & 15)) << 4));
          *reinterpret_cast<uint4*>(out + ((int64_t)(start + r0 + rr) * nq + head) * D + chunk * 8) = val;
        }
      }
      if (lse != nullptr && qrow < len)
        lse[(int64_t)head * total_rows + start + qrow] = l > 0.f ? m_ref * scale + logf(l) : -INFINITY;
    }
    if (!ok && lane == 0) { atomicCAS(&g_attn_status, ST_OK, ST_SOFTMAX); atomicExch(&sm->abort_flag, 1u); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool attn_fwd_sm100_supported(int64_t head_dim) { return head_dim == 128; }

int64_t attn_sm100_last_status() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int));
  cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  return v;
}

// q [T, nq, 128], k / v [T, nkv, 128] bf16 (rows may be strided: views of a fused QKV tensor), cu_seqlens [B+1] int32.
// Returns {out [T, nq, 128] bf16, lse [nq, T] fp32 (natural log)}.
std::vector<at::Tensor> attn_fwd_sm100(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                       const at::Tensor& cu_seqlens, double scale, bool causal) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "attn_fwd_sm100: bf16 CUDA tensors");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "attn_fwd_sm100: [T, heads, 128]");
  const int64_t T = q.size(0), nq = q.size(1), nkv = k.size(1);
  TORCH_CHECK(q.size(2) == D && k.size(2) == D && v.size(2) == D && nq % nkv == 0 && v.size(1) == nkv && k.size(0) == T && v.size(0) == T,
              "attn_fwd_sm100: head dim 128, query heads a multiple of key/value heads");
  for (const at::Tensor* x : {&q, &k, &v})
    TORCH_CHECK(x->stride(2) == 1 && x->stride(1) == D && x->stride(0) % 8 == 0 && (uintptr_t)x->data_ptr() % 16 == 0,
                "attn_fwd_sm100: heads must be contiguous and rows 16-byte aligned");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_cuda() && cu_seqlens.is_contiguous(), "cu_seqlens: int32 CUDA");
  const int B = (int)cu_seqlens.numel() - 1;
  auto out = at::empty({T, nq, D}, q.options());
  auto lse = at::empty({nq, T}, q.options().dtype(at::kFloat));
  if (T == 0 || B <= 0) return {out, lse};
  const int dev = q.get_device();
  tmap::bind_context_to_thread(dev);
  // one row of the 2-D view = one token, all heads side by side
  const CUtensorMap tmQ = tmap::make_bf16_2d(q.data_ptr(), T, nq * D, q.stride(0), BM);
  const CUtensorMap tmK = tmap::make_bf16_2d(k.data_ptr(), T, nkv * D, k.stride(0), BN);
  const CUtensorMap tmV = tmap::make_bf16_2d(v.data_ptr(), T, nkv * D, v.stride(0), BN);
  static bool cfg[64] = {};
  const size_t smem = sizeof(SmemFwd);
  if (!cfg[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_sm100_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        (int)cudaSharedmemCarveoutMaxShared));
    cfg[dev] = true;
  }
  const int tiles = (int)((T + BM - 1) / BM) + B;       // upper bound on the query tiles; surplus CTAs exit at once
  dim3 grid(tiles, (unsigned)nq);
  attn_fwd_sm100_kernel<<<grid, kThreads, smem, at::cuda::getCurrentCUDAStream()>>>(
      tmQ, tmK, tmV, cu_seqlens.data_ptr<int>(), B, (bf16*)out.data_ptr(), lse.data_ptr<float>(), (int)nq, (int)nkv, (int)T,
      (float)scale, causal ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {out, lse};
}
