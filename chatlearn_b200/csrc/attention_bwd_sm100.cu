// Variable-length attention backward on the 5th-generation tensor cores (head dim 128, bf16,
// packed sequences, GQA, causal or full): dQ, dK, dV from Q, K, V, O, dO and the forward's
// log-sum-exp.
//
// A CTA owns 128 keys of one sequence and one key/value head.  It walks over the query heads
// that share that head and over their 64-row query blocks (for a causal mask only the blocks
// at or below the diagonal), and for every (head, query block) item runs five products on
// tcgen05.mma, all in the transposed orientation so that the 128 keys are the accumulator
// rows:
//   S^T  = K Q^T          128x64, K over the head dim        both operands K-major
//   dP^T = V dO^T         128x64
//   dV  += P^T dO         128x128, K over the 64 queries     P^T from shared memory (K-major),
//   dK  += dS^T Q         128x128                            dO / Q as MN-major operands: the very
//                                                            tiles the first two products read
//   dQ^T = K^T dS^T       128x64, K over the 128 keys        K and dS^T both MN-major
// dK and dV stay in tensor memory for the CTA's whole life and are written once; dQ^T is read
// out per item and added into an fp32 accumulation buffer with coalesced red.global.add (the
// one operand that several CTAs contribute to).  No operand is transposed in memory: the
// MN-major shared-memory descriptors do it.
//
// Roles (448 threads): warp 0 TMA producer (K, V once; then Q, dO tiles and the per-row
// statistics of each item through a 3-stage ring), warp 1 MMA issuer, warps 2..9 the
// elementwise stage (thread = key row, 32 of the 64 query columns: P = exp2(S c - lse),
// dS = P (dP - delta) scale, both written as bf16 into swizzled shared-memory tiles, double
// buffered), warps 10..13 the dQ read-out (thread = head-dim lane).
// Every mbarrier wait is bounded; a wait that runs out records a status code and the CTA
// drains and frees its tensor memory.
#include <ATen/cuda/CUDAContext.h>
#include <torch/extension.h>

#include "sm100.cuh"
#include "tmap.h"

using namespace sm100;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BKV = 128, BQ = 64, D = 128;
constexpr int kThreads = 448;
constexpr int kQStages = 3;                // Q / dO ring: a stage is held from its load until the item's dK product has run
constexpr int kTmemCols = 512;
constexpr uint32_t COL_S = 0, COL_DP = 64, COL_DV = 128, COL_DK = 256, COL_DQ = 384;
constexpr uint32_t kBoxKV = BKV * 128;       // one 64-column slice of a K or V tile: 128 rows x 128 bytes
constexpr uint32_t kBoxQ = BQ * 128;         // one 64-column slice of a Q or dO tile: 64 rows x 128 bytes

struct SmemBwd {
  uint8_t k[2][kBoxKV];                      // 32 KB (reused to stage dK at the end)
  uint8_t v[2][kBoxKV];                      // 32 KB (reused to stage dV)
  uint8_t q[kQStages][2][kBoxQ];             // [stage][slice]
  uint8_t d_o[kQStages][2][kBoxQ];
  uint8_t p[2][BKV * 128];                   // P^T  [128 keys x 64 queries] bf16, K-major, 128-byte swizzle; double buffered
  uint8_t ds[2][BKV * 128];                  // dS^T likewise
  float lse2[kQStages][BQ];                         // log-sum-exp of the item's query rows in log2 units (+inf past the sequence end)
  float delta[kQStages][BQ];                        // rowsum(dO * O)
  uint64_t kv_full, q_full[kQStages], q_empty[kQStages], s_full, s_empty, p_full[2], p_empty[2], dq_full, dq_empty, dkv_full;
  uint32_t tmem_base, abort_flag;
  int seq, blk;
};

static_assert(sizeof(SmemBwd) <= 227 * 1024, "the backward tiles must fit the 227 KB a CTA may use");

__device__ int g_attn_bwd_status = 0;
enum : int { ST_OK = 0, ST_PRODUCER = 1, ST_MMA = 2, ST_ELEMENTWISE = 3, ST_SMEM_ALIGN = 4, ST_DQ = 5 };

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const int* __restrict__ cu_seqlens, int num_seqs, const float* __restrict__ lse,
                      const float* __restrict__ delta, float* __restrict__ dq_acc, bf16* __restrict__ dk,
                      bf16* __restrict__ dv, int nq, int nkv, int total_rows, float scale, int causal) {
  extern __shared__ uint8_t smem_raw[];
  SmemBwd* sm = reinterpret_cast<SmemBwd*>(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;

  if (threadIdx.x == 0) {
    int left = blockIdx.x, seq = -1, blk = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int nb = (cu_seqlens[s + 1] - cu_seqlens[s] + BKV - 1) / BKV;
      if (left < nb) { seq = s; blk = left; break; }       // first key blocks first: under a causal mask they meet the most queries
      left -= nb;
    }
    sm->seq = seq; sm->blk = blk;
    if ((smem_u32(smem_raw) & 1023u) != 0u) { sm->seq = -1; atomicCAS(&g_attn_bwd_status, ST_OK, ST_SMEM_ALIGN); }
  }
  __syncthreads();
  const int seq = sm->seq;
  if (seq < 0) return;                         // surplus CTA of the over-sized grid (nothing allocated yet)
  const int start = cu_seqlens[seq], len = cu_seqlens[seq + 1] - start;
  const int kv0 = sm->blk * BKV;               // first key of the block, relative to the sequence
  const int nqb = (len + BQ - 1) / BQ;         // query blocks of the sequence
  const int i0 = causal ? (kv0 / BQ) : 0;      // first query block that sees any key of this block
  const int nper = nqb - i0;                   // query blocks per head (>= 1: key kv0 exists, so does query kv0)
  const int group = nq / nkv;
  const int nitems = nper * group;

  if (threadIdx.x == 0) {
    mbar_init(&sm->kv_full, 1);
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&sm->q_full[s], 2);            // the TMA transaction + the statistics written by the producer warp
      mbar_init(&sm->q_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm->p_full[s], 256);
      mbar_init(&sm->p_empty[s], 1);
    }
    mbar_init(&sm->s_full, 1);
    mbar_init(&sm->s_empty, 8);
    mbar_init(&sm->dq_full, 1);
    mbar_init(&sm->dq_empty, 4);
    mbar_init(&sm->dkv_full, 1);
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
    // ------------------------------------------------ producer
    bool ok = true;
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
      mbar_expect_tx(&sm->kv_full, 4 * kBoxKV);
      tma_load_2d(sm->k[0], &tmK, &sm->kv_full, kvh * D, start + kv0);
      tma_load_2d(sm->k[1], &tmK, &sm->kv_full, kvh * D + 64, start + kv0);
      tma_load_2d(sm->v[0], &tmV, &sm->kv_full, kvh * D, start + kv0);
      tma_load_2d(sm->v[1], &tmV, &sm->kv_full, kvh * D + 64, start + kv0);
    }
    for (int t = 0; t < nitems; ++t) {
      const int st = t % kQStages;
      const int head = kvh * group + t / nper, qb = i0 + t % nper;
      if (lane == 0) ok = mbar_wait(&sm->q_empty[st], ((t / kQStages) & 1) ^ 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane == 0) {
        const int row = start + qb * BQ;
        mbar_expect_tx(&sm->q_full[st], 4 * kBoxQ);
        tma_load_2d(sm->q[st][0], &tmQ, &sm->q_full[st], head * D, row);
        tma_load_2d(sm->q[st][1], &tmQ, &sm->q_full[st], head * D + 64, row);
        tma_load_2d(sm->d_o[st][0], &tmDO, &sm->q_full[st], head * D, row);
        tma_load_2d(sm->d_o[st][1], &tmDO, &sm->q_full[st], head * D + 64, row);
      }
      // per-row statistics of the item; rows past the end of the sequence get lse = +inf, which makes their
      // probabilities exactly zero whatever their (foreign) Q and dO rows hold
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = qb * BQ + h * 32 + lane;
        const bool valid = r < len;
        const int64_t at = (int64_t)head * total_rows + start + r;
        sm->lse2[st][h * 32 + lane] = valid ? lse[at] * 1.4426950408889634f : INFINITY;
        sm->delta[st][h * 32 + lane] = valid ? delta[at] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->q_full[st]);
    }
    if (!ok && lane == 0) { atomicCAS(&g_attn_bwd_status, ST_OK, ST_PRODUCER); atomicExch(&sm->abort_flag, 1u); }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BKV, BQ, 0, 0);     // K-major x K-major
      constexpr uint32_t idesc_acc = make_idesc_bf16(BKV, D, 0, 1);    // P^T / dS^T K-major, dO / Q MN-major
      constexpr uint32_t idesc_dq = make_idesc_bf16(D, BQ, 1, 1);      // K^T and dS^T both MN-major
      bool ok = mbar_wait(&sm->kv_full, 0);
      tc_fence_after_sync();
      auto issue_back = [&](int u) -> bool {
        const uint32_t buf = u & 1, st = u % kQStages;
        if (!mbar_wait(&sm->p_full[buf], (u >> 1) & 1)) return false;
        tc_fence_after_sync();
        const uint64_t dp = make_kmajor_sw128_desc(smem_u32(sm->p[buf]));
        const uint64_t dds = make_kmajor_sw128_desc(smem_u32(sm->ds[buf]));
        const uint64_t ddo = make_mnmajor_sw128_desc(smem_u32(sm->d_o[st][0]), kBoxQ);
        const uint64_t dqm = make_mnmajor_sw128_desc(smem_u32(sm->q[st][0]), kBoxQ);
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          umma_bf16(tmem_base + COL_DV, dp + 2ull * kk, ddo + 128ull * kk, idesc_acc, (u > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk)
          umma_bf16(tmem_base + COL_DK, dds + 2ull * kk, dqm + 128ull * kk, idesc_acc, (u > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&sm->q_empty[st]);                  // the item's Q and dO tiles have been read for the last time
        if (!mbar_wait(&sm->dq_empty, (u & 1) ^ 1)) return false;
        tc_fence_after_sync();
        const uint64_t dkt = make_mnmajor_sw128_desc(smem_u32(sm->k[0]), kBoxKV);
        const uint64_t dst = make_mnmajor_sw128_desc(smem_u32(sm->ds[buf]), BKV * 128);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)
          umma_bf16(tmem_base + COL_DQ, dkt + 128ull * kk, dst + 128ull * kk, idesc_dq, kk > 0 ? 1u : 0u);
        umma_commit(&sm->p_empty[buf]);
        umma_commit(&sm->dq_full);
        return true;
      };
      for (int t = 0; t < nitems && ok; ++t) {
        const uint32_t st = t % kQStages;
        if (!mbar_wait(&sm->q_full[st], (t / kQStages) & 1)) { ok = false; break; }
        if (!mbar_wait(&sm->s_empty, (t & 1) ^ 1)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t a = make_kmajor_sw128_desc(smem_u32(sm->k[kk >> 2])) + 2ull * (kk & 3);
          const uint64_t b = make_kmajor_sw128_desc(smem_u32(sm->q[st][kk >> 2])) + 2ull * (kk & 3);
          umma_bf16(tmem_base + COL_S, a, b, idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t a = make_kmajor_sw128_desc(smem_u32(sm->v[kk >> 2])) + 2ull * (kk & 3);
          const uint64_t b = make_kmajor_sw128_desc(smem_u32(sm->d_o[st][kk >> 2])) + 2ull * (kk & 3);
          umma_bf16(tmem_base + COL_DP, a, b, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sm->s_full);
        if (t > 0 && !issue_back(t - 1)) { ok = false; break; }
      }
      if (ok) ok = issue_back(nitems - 1);
      if (ok) umma_commit(&sm->dkv_full);
      if (!ok) { atomicCAS(&g_attn_bwd_status, ST_OK, ST_MMA); atomicExch(&sm->abort_flag, 1u); }
    }
  } else if (warp < 10) {
    // ------------------------------------------------ elementwise stage: thread = key row, 32 query columns
    const int quarter = warp & 3;                 // tensor-memory lane quarter of this warp
    const int half = (warp - 2) >> 2;             // which 32 of the 64 query columns
    const int row = quarter * 32 + lane;          // key row of the tile
    const int kvi = kv0 + row;                    // key index in the sequence
    const bool kv_valid = kvi < len;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float c = scale * 1.4426950408889634f;
    bool ok = true;
    for (int t = 0; t < nitems; ++t) {
      const int st = t % kQStages, buf = t & 1;
      const int qb = i0 + t % nper;
      if (!mbar_wait(&sm->q_full[st], (t / kQStages) & 1)) { ok = false; break; }      // the statistics of the item are in place
      if (!mbar_wait(&sm->s_full, t & 1)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t s[32], dp[32];
      tmem_ld_32x32(lane_addr + COL_S + half * 32, s);
      tmem_ld_32x32(lane_addr + COL_DP + half * 32, dp);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->s_empty);   // both accumulators are in registers: the next item's products may run
      const int q_first = qb * BQ + half * 32;    // sequence index of this thread's first query column
      // keys past the end of the sequence, and (causal) keys after the query, have probability zero
      const int vis_from = !kv_valid ? (1 << 30) : (causal ? kvi : 0);   // first query index that sees this key
      uint32_t pw[16], dw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float pv[2], dv2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = 2 * i + e;
          const float l2 = sm->lse2[st][half * 32 + col], dl = sm->delta[st][half * 32 + col];
          float p = fast_exp2(fmaf(__uint_as_float(s[col]), c, -l2));
          if (q_first + col < vis_from) p = 0.f;
          pv[e] = p;
          dv2[e] = p * (__uint_as_float(dp[col]) - dl) * scale;
        }
        pw[i] = pack_bf16(pv[0], pv[1]);
        dw[i] = pack_bf16(dv2[0], dv2[1]);
      }
      if (!mbar_wait(&sm->p_empty[buf], ((t >> 1) & 1) ^ 1)) { ok = false; break; }
      uint8_t* prow = sm->p[buf] + row * 128;
      uint8_t* drow = sm->ds[buf] + row * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int phys = ((half * 4 + ch) ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + phys) = make_uint4(pw[4 * ch], pw[4 * ch + 1], pw[4 * ch + 2], pw[4 * ch + 3]);
        *reinterpret_cast<uint4*>(drow + phys) = make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
      }
      fence_proxy_async();
      mbar_arrive(&sm->p_full[buf]);
    }
    // ---- dK, dV: 32 key rows x 64 head-dim columns per warp, staged through the K / V tiles (no product
    // reads them any more) so that global memory sees 128-byte row segments
    if (ok && !mbar_wait(&sm->dkv_full, 0)) ok = false;
    if (ok) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        uint8_t* stage = which == 0 ? sm->k[0] : sm->v[0];          // 128 rows x 256 bytes
        const uint32_t col0 = (which == 0 ? COL_DK : COL_DV) + half * 64;
#pragma unroll 1
        for (int cc = 0; cc < 64; cc += 32) {
          uint32_t o[32];
          tmem_ld_32x32(lane_addr + col0 + cc, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = pack_bf16(__uint_as_float(o[g * 8 + 2 * i]), __uint_as_float(o[g * 8 + 2 * i + 1]));
            const int chunk = half * 8 + cc / 8 + g;
            *reinterpret_cast<uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        __syncwarp();
        bf16* dst = which == 0 ? dk : dv;
#pragma unroll 1
        for (int i = 0; i < 8; ++i) {
          const int rr = quarter * 32 + 4 * i + (lane >> 3), chunk = half * 8 + (lane & 7);
          if (kv0 + rr < len) {
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((chunk ^ (rr & 15)) << 4));
            *reinterpret_cast<uint4*>(dst + ((int64_t)(start + kv0 + rr) * nkv + kvh) * D + chunk * 8) = val;
          }
        }
      }
    }
    if (!ok && lane == 0) { atomicCAS(&g_attn_bwd_status, ST_OK, ST_ELEMENTWISE); atomicExch(&sm->abort_flag, 1u); }
  } else {
    // ------------------------------------------------ dQ read-out: thread = head-dim lane, 64 query columns
    const int quarter = warp & 3;
    const int dcol = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    bool ok = true;
    for (int t = 0; t < nitems; ++t) {
      const int head = kvh * group + t / nper, qb = i0 + t % nper;
      if (!mbar_wait(&sm->dq_full, t & 1)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t a[32], b[32];
      tmem_ld_32x32(lane_addr + COL_DQ, a);
      tmem_ld_32x32(lane_addr + COL_DQ + 32, b);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->dq_empty);
      const int nvalid = min(BQ, len - qb * BQ);
      float* base = dq_acc + ((int64_t)head * total_rows + start + qb * BQ) * D + dcol;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < nvalid) red_add_f32(base + (int64_t)i * D, __uint_as_float(a[i]));
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (32 + i < nvalid) red_add_f32(base + (int64_t)(32 + i) * D, __uint_as_float(b[i]));
    }
    if (!ok && lane == 0) { atomicCAS(&g_attn_bwd_status, ST_OK, ST_DQ); atomicExch(&sm->abort_flag, 1u); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]: one warp per (token, head) row of 128 elements.
__global__ void attn_bwd_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, float* __restrict__ delta,
                                      int64_t o_stride, int64_t do_stride, int nq, int total_rows) {
  const int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (int64_t)total_rows * nq) return;
  const int64_t t = w / nq;
  const int h = (int)(w % nq);
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * o_stride + h * D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + t * do_stride + h * D + lane * 4);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[(int64_t)h * total_rows + t] = acc;
}

// dq[t, h, :] = bf16(dq_acc[h, t, :])
__global__ void attn_bwd_dq_cast_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, int nq, int total_rows) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;          // one thread per 8 elements
  const int64_t n = (int64_t)total_rows * nq * (D / 8);
  if (i >= n) return;
  const int c8 = (int)(i % (D / 8));
  const int64_t th = i / (D / 8);
  const int h = (int)(th % nq);
  const int64_t t = th / nq;
  const float4 x = *reinterpret_cast<const float4*>(acc + ((int64_t)h * total_rows + t) * D + c8 * 8);
  const float4 y = *reinterpret_cast<const float4*>(acc + ((int64_t)h * total_rows + t) * D + c8 * 8 + 4);
  *reinterpret_cast<uint4*>(dq + (t * nq + h) * D + c8 * 8) =
      make_uint4(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w), pack_bf16(y.x, y.y), pack_bf16(y.z, y.w));
}

}  // namespace

int64_t attn_bwd_sm100_last_status() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_attn_bwd_status, sizeof(int));
  cudaMemcpyToSymbol(g_attn_bwd_status, &zero, sizeof(int));
  return v;
}

// q, o, d_o [T, nq, 128]; k, v [T, nkv, 128] bf16 (rows may be strided); lse [nq, T] fp32 from the forward.
// Returns {dq [T, nq, 128], dk [T, nkv, 128], dv [T, nkv, 128]} bf16.
std::vector<at::Tensor> attn_bwd_sm100(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                                       const at::Tensor& d_o, const at::Tensor& lse, const at::Tensor& cu_seqlens, double scale,
                                       bool causal) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && o.dim() == 3 && d_o.dim() == 3, "attn_bwd_sm100: [T, heads, 128]");
  const int64_t T = q.size(0), nq = q.size(1), nkv = k.size(1);
  for (const at::Tensor* x : {&q, &k, &v, &o, &d_o}) {
    TORCH_CHECK(x->scalar_type() == at::kBFloat16 && x->size(0) == T && x->size(2) == D, "attn_bwd_sm100: bf16 [T, heads, 128]");
    TORCH_CHECK(x->stride(2) == 1 && x->stride(1) == D && x->stride(0) % 8 == 0 && (uintptr_t)x->data_ptr() % 16 == 0,
                "attn_bwd_sm100: heads must be contiguous and rows 16-byte aligned");
  }
  TORCH_CHECK(o.size(1) == nq && d_o.size(1) == nq && v.size(1) == nkv && nq % nkv == 0, "attn_bwd_sm100: head counts");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.dim() == 2 && lse.size(0) == nq && lse.size(1) == T,
              "attn_bwd_sm100: lse [nq, T] fp32");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_cuda() && cu_seqlens.is_contiguous(), "cu_seqlens: int32 CUDA");
  const int B = (int)cu_seqlens.numel() - 1;
  auto dq = at::empty({T, nq, D}, q.options());
  auto dk = at::empty({T, nkv, D}, q.options());
  auto dv = at::empty({T, nkv, D}, q.options());
  if (T == 0 || B <= 0) return {dq, dk, dv};
  const int dev = q.get_device();
  tmap::bind_context_to_thread(dev);
  auto st = at::cuda::getCurrentCUDAStream();
  auto delta = at::empty({nq, T}, q.options().dtype(at::kFloat));
  auto dq_acc = at::zeros({nq, T, D}, q.options().dtype(at::kFloat));
  {
    const int64_t warps = T * nq;
    attn_bwd_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(
        (const bf16*)o.data_ptr(), (const bf16*)d_o.data_ptr(), delta.data_ptr<float>(), o.stride(0), d_o.stride(0), (int)nq, (int)T);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  const CUtensorMap tmQ = tmap::make_bf16_2d(q.data_ptr(), T, nq * D, q.stride(0), BQ);
  const CUtensorMap tmDO = tmap::make_bf16_2d(d_o.data_ptr(), T, nq * D, d_o.stride(0), BQ);
  const CUtensorMap tmK = tmap::make_bf16_2d(k.data_ptr(), T, nkv * D, k.stride(0), BKV);
  const CUtensorMap tmV = tmap::make_bf16_2d(v.data_ptr(), T, nkv * D, v.stride(0), BKV);
  static bool cfg[64] = {};
  const size_t smem = sizeof(SmemBwd);
  if (!cfg[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cfg[dev] = true;
  }
  const int blocks = (int)((T + BKV - 1) / BKV) + B;        // upper bound on the key blocks; surplus CTAs exit at once
  dim3 grid(blocks, (unsigned)nkv);
  attn_bwd_sm100_kernel<<<grid, kThreads, smem, st>>>(tmQ, tmK, tmV, tmDO, cu_seqlens.data_ptr<int>(), B, lse.data_ptr<float>(),
                                                      delta.data_ptr<float>(), dq_acc.data_ptr<float>(), (bf16*)dk.data_ptr(),
                                                      (bf16*)dv.data_ptr(), (int)nq, (int)nkv, (int)T, (float)scale, causal ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  {
    const int64_t n = T * nq * (D / 8);
    attn_bwd_dq_cast_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dq_acc.data_ptr<float>(), (bf16*)dq.data_ptr(), (int)nq, (int)T);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {dq, dk, dv};
}
