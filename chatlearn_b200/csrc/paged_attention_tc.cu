// Decode attention over the paged KV cache on tensor cores.
//
// One CTA per (query token, KV head, split).  The query heads that share the KV
// head (GQA, up to 8) form the M dimension of the MMAs, so K and V are read from
// HBM exactly once per group.  KV blocks (64 tokens) stream through a two-stage
// cp.async ring.  Each of the 4 warps owns 16 tokens of every block and runs its
// own online-softmax stream over them (S = Q K^T and O += P V with m16n8k16 bf16
// MMAs, fp32 accumulators), so the main loop has no cross-warp reduction; the four
// streams are merged once at the end.  The arithmetic per byte is tiny, so the
// kernel is bound by how fast cp.async keeps HBM busy.
#include <ATen/cuda/CUDAContext.h>
#include <cuda_pipeline.h>
#include <c10/cuda/CUDAException.h>
#include <torch/extension.h>

#include "common.cuh"

using namespace cl;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kThreads = 128;
constexpr int BS = 64;            // tokens per KV block
constexpr int kPad = 8;           // row padding (elements): keeps ldmatrix rows on distinct banks

template <int DK, int DV>
struct SmemTC {
  bf16 k[2][BS][DK + kPad];
  bf16 v[2][BS][DV + kPad];
  bf16 q[16][DK + kPad];
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int DK, int DV>
__device__ __forceinline__ void load_tile_tc(SmemTC<DK, DV>* sm, int stage, const bf16* kc, const bf16* vc,
                                             int64_t block_id, int kv_head, int nkv, int valid) {
  const bf16* kb = kc + (block_id * BS * nkv + kv_head) * (int64_t)DK;
  const bf16* vb = vc + (block_id * BS * nkv + kv_head) * (int64_t)DV;
  constexpr int KCH = DK / 8, VCH = DV / 8;
  for (int c = threadIdx.x; c < BS * KCH; c += kThreads) {
    const int r = c / KCH, o = (c % KCH) * 8;
    if (r < valid) __pipeline_memcpy_async(&sm->k[stage][r][o], kb + (int64_t)r * nkv * DK + o, 16);
  }
  for (int c = threadIdx.x; c < BS * VCH; c += kThreads) {
    const int r = c / VCH, o = (c % VCH) * 8;
    if (r < valid) __pipeline_memcpy_async(&sm->v[stage][r][o], vb + (int64_t)r * nkv * DV + o, 16);
    else *reinterpret_cast<uint4*>(&sm->v[stage][r][o]) = make_uint4(0, 0, 0, 0);   // 0 * garbage must not be NaN
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(kThreads)
paged_decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                       const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ q_seq,
                       const int* __restrict__ ctx_len, bf16* __restrict__ out, float* __restrict__ part_o,
                       float* __restrict__ part_lse, int nq, int nkv, int num_splits, float scale,
                       const int* __restrict__ blk_start = nullptr, int slot_base = 0, int total_slots = 0) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  pdl_wait();                                     // q, the cache and the tables come from earlier kernels
  auto* sm = reinterpret_cast<SmemTC<DK, DV>*>(smem_raw);
  const int qi = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int rep = nq / nkv;
  const int seq = q_seq ? q_seq[qi] : qi;
  const int L = ctx_len[qi];
  const int nblk = (L + BS - 1) / BS;
  // grouped mode: the first `first` blocks of this sequence are attended by the shared-prefix kernel; this kernel
  // covers the rest and writes its partial results behind the prefix slots
  const int first = blk_start ? blk_start[qi] : 0;
  const int per = (nblk - first + num_splits - 1) / num_splits;
  const int b0 = first + split * per, b1 = min(b0 + per, nblk);
  if (total_slots == 0) total_slots = num_splits;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int* bt = block_tables + (int64_t)seq * max_blocks;

  // Q tile: rows 0..rep-1 are the heads of this group, the rest is zero padding
  for (int i = tid; i < 16 * (DK / 8); i += kThreads) {
    const int r = i / (DK / 8), o = (i % (DK / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rep) v = *reinterpret_cast<const uint4*>(q + ((int64_t)qi * nq + kvh * rep + r) * DK + o);
    *reinterpret_cast<uint4*>(&sm->q[r][o]) = v;
  }
  if (b0 < b1) load_tile_tc<DK, DV>(sm, 0, kc, vc, bt[b0], kvh, nkv, min(BS, L - b0 * BS));
  __pipeline_commit();
  __syncthreads();
  uint32_t qa[DK / 16][4];
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks) ldmatrix_x4(qa[ks], &sm->q[lane & 15][ks * 16 + (lane >> 4) * 8]);

  float o_acc[DV / 8][4];
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) { o_acc[n][0] = o_acc[n][1] = o_acc[n][2] = o_acc[n][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;          // row g (head g) of this warp's stream
  const int tw = warp * 16;                      // first token of this warp inside a block

  for (int b = b0; b < b1; ++b) {
    const int st = (b - b0) & 1;
    if (b + 1 < b1) load_tile_tc<DK, DV>(sm, st ^ 1, kc, vc, bt[b + 1], kvh, nkv, min(BS, L - (b + 1) * BS));
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
    const int valid = min(BS, L - b * BS);
    if (tw < valid) {
      // ---- S = Q K^T for this warp's 16 tokens: two 8-token n-tiles ----
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ks += 2) {
          uint32_t kb[4];
          ldmatrix_x4(kb, &sm->k[st][tw + j * 8 + (lane & 7)][ks * 16 + (lane >> 3) * 8]);
          mma_bf16(s[j], qa[ks], kb[0], kb[1]);
          mma_bf16(s[j], qa[ks + 1], kb[2], kb[3]);
        }
      }
      // ---- online softmax on row g (rows g+8 are padding) ----
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tw + j * 8 + 2 * t + e;
          s[j][e] = (tok < valid) ? s[j][e] * scale : -INFINITY;
          mx = fmaxf(mx, s[j][e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run, mx);        // finite: token tw of this warp is valid
      const float alpha = __expf(m_run - m_new);   // exp(-inf) = 0 on the first block
      float psum = 0.f;
      uint32_t pa[4];
      {
        const float p00 = __expf(s[0][0] - m_new), p01 = __expf(s[0][1] - m_new);
        const float p10 = __expf(s[1][0] - m_new), p11 = __expf(s[1][1] - m_new);
        psum = p00 + p01 + p10 + p11;
        pa[0] = pack_bf16(p00, p01);   // row g,   tokens 2t, 2t+1
        pa[1] = 0u;                    // row g+8: padding
        pa[2] = pack_bf16(p10, p11);   // row g,   tokens 8+2t, 8+2t+1
        pa[3] = 0u;
      }
      l_run = l_run * alpha + psum;
      m_run = m_new;
      // ---- O = alpha * O + P V ----
#pragma unroll
      for (int n = 0; n < DV / 8; n += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, &sm->v[st][tw + ((lane >> 3) & 1) * 8 + (lane & 7)][(n + (lane >> 4)) * 8]);
        o_acc[n][0] *= alpha; o_acc[n][1] *= alpha;
        o_acc[n + 1][0] *= alpha; o_acc[n + 1][1] *= alpha;
        mma_bf16(o_acc[n], pa, vb[0], vb[1]);
        mma_bf16(o_acc[n + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
  __pipeline_wait_prior(0);
  __syncthreads();
  // ---- merge the 4 per-warp streams (reuse the K/V ring as scratch) ----
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  float* red_o = reinterpret_cast<float*>(&sm->k[0][0][0]);           // [4 warps][8 heads][DV]
  float* red_m = red_o + 4 * 8 * DV;                                   // [4][8]
  float* red_l = red_m + 32;                                           // [4][8]
  static_assert(sizeof(float) * (4 * 8 * DV + 64) <= sizeof(bf16) * 2 * BS * (DK + kPad), "scratch fits in the K ring");
#pragma unroll
  for (int n = 0; n < DV / 8; ++n) {
    red_o[(warp * 8 + g) * DV + n * 8 + 2 * t] = o_acc[n][0];
    red_o[(warp * 8 + g) * DV + n * 8 + 2 * t + 1] = o_acc[n][1];
  }
  if (t == 0) { red_m[warp * 8 + g] = m_run; red_l[warp * 8 + g] = l_run; }
  __syncthreads();
  for (int idx = tid; idx < rep * DV; idx += kThreads) {
    const int r = idx / DV, d = idx % DV;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 8 + r]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = red_m[w * 8 + r];
      if (mw == -INFINITY) continue;
      const float e = __expf(mw - M);
      den += e * red_l[w * 8 + r];
      num += e * red_o[(w * 8 + r) * DV + d];
    }
    const int head = kvh * rep + r;
    const float val = den > 0.f ? num / den : 0.f;
    if (total_slots == 1) {
      out[((int64_t)qi * nq + head) * DV + d] = __float2bfloat16_rn(val);
    } else {
      const int64_t at = ((int64_t)qi * nq + head) * total_slots + slot_base + split;
      part_o[at * DV + d] = val;
      if (d == 0) {
        part_lse[at] = den > 0.f ? M + logf(den) : -INFINITY;
        // a sequence outside every group has no prefix pass: its prefix slots must not count
        if (split == 0 && first == 0)
          for (int sl = 0; sl < slot_base; ++sl) part_lse[((int64_t)qi * nq + head) * total_slots + sl] = -INFINITY;
      }
    }
  }
}

// Shared-prefix pass of the decode attention.
//
// Sequences that adopted the same prompt blocks form a group.  One CTA per (group, KV head, split) attends the
// queries of ALL members (up to 8 members x `rep` query heads = up to 32 MMA rows, two m16 tiles) over the
// group's shared blocks, so those K/V bytes are read once per group instead of once per member.  The result
// goes out as partial (o, lse) into slot `split` of the members' rows; the per-sequence kernel covers the
// remaining blocks into the following slots and the combine kernel merges all slots by log-sum-exp.
template <int DK, int DV>
struct SmemPrefix {
  bf16 k[2][BS][DK + kPad];
  bf16 v[2][BS][DV + kPad];
  bf16 q[32][DK + kPad];
};

template <int DK, int DV>
__global__ void __launch_bounds__(kThreads)
paged_prefix_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                       const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ grp_q,
                       const int* __restrict__ grp_nblk, float* __restrict__ part_o, float* __restrict__ part_lse,
                       int nq, int nkv, int num_splits, int total_slots, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  pdl_wait();
  auto* sm = reinterpret_cast<SmemPrefix<DK, DV>*>(smem_raw);
  const int grp = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int nblk = grp_nblk[grp];
  if (nblk <= 0) return;                                  // unused group slot of the captured grid
  const int rep = nq / nkv;
  const int rows = 8 * rep;                               // <= 32 (rep <= 4)
  const int per = (nblk + num_splits - 1) / num_splits;
  const int b0 = split * per, b1 = min(b0 + per, nblk);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int* members = grp_q + grp * 8;
  const int lead = members[0];                            // the first member's block table row holds the shared blocks
  const int* bt = block_tables + (int64_t)lead * max_blocks;
  if (b0 >= b1) {                                         // nothing for this split: its slot must not count
    for (int idx = tid; idx < rows; idx += kThreads) {
      const int qi = members[idx / rep];
      if (qi >= 0) part_lse[((int64_t)qi * nq + kvh * rep + idx % rep) * total_slots + split] = -INFINITY;
    }
    return;
  }
  // Q tile: row R = member * rep + head-in-group; rows of absent members are zero
  for (int i = tid; i < 32 * (DK / 8); i += kThreads) {
    const int r = i / (DK / 8), o = (i % (DK / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      const int qi = members[r / rep];
      if (qi >= 0) v = *reinterpret_cast<const uint4*>(q + ((int64_t)qi * nq + kvh * rep + r % rep) * DK + o);
    }
    *reinterpret_cast<uint4*>(&sm->q[r][o]) = v;
  }
  load_tile_tc<DK, DV>(reinterpret_cast<SmemTC<DK, DV>*>(sm), 0, kc, vc, bt[b0], kvh, nkv, BS);
  __pipeline_commit();
  __syncthreads();
  uint32_t qa[2][DK / 16][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) ldmatrix_x4(qa[mt][ks], &sm->q[mt * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);

  float o_acc[2][DV / 8][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) { o_acc[mt][n][0] = o_acc[mt][n][1] = o_acc[mt][n][2] = o_acc[mt][n][3] = 0.f; }
  float m_run[2][2], l_run[2][2];                          // [m tile][row g / row g + 8] of this warp's stream
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) { m_run[mt][0] = m_run[mt][1] = -INFINITY; l_run[mt][0] = l_run[mt][1] = 0.f; }
  const int tw = warp * 16;

  for (int b = b0; b < b1; ++b) {
    const int st = (b - b0) & 1;
    if (b + 1 < b1) load_tile_tc<DK, DV>(reinterpret_cast<SmemTC<DK, DV>*>(sm), st ^ 1, kc, vc, bt[b + 1], kvh, nkv, BS);
    __pipeline_commit();
    __pipeline_wait_prior(1);
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ks += 2) {
          uint32_t kb[4];
          ldmatrix_x4(kb, &sm->k[st][tw + j * 8 + (lane & 7)][ks * 16 + (lane >> 3) * 8]);
          mma_bf16(s[j], qa[mt][ks], kb[0], kb[1]);
          mma_bf16(s[j], qa[mt][ks + 1], kb[2], kb[3]);
        }
      }
      uint32_t pa[4];
      float alpha[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {                         // h = 0: row g (accumulator slots 0, 1); h = 1: row g + 8 (slots 2, 3)
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][2 * h] *= scale; s[j][2 * h + 1] *= scale;
          mx = fmaxf(mx, fmaxf(s[j][2 * h], s[j][2 * h + 1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[mt][h], mx);        // finite: whole blocks, every key is valid
        alpha[h] = __expf(m_run[mt][h] - m_new);
        const float p00 = __expf(s[0][2 * h] - m_new), p01 = __expf(s[0][2 * h + 1] - m_new);
        const float p10 = __expf(s[1][2 * h] - m_new), p11 = __expf(s[1][2 * h + 1] - m_new);
        l_run[mt][h] = l_run[mt][h] * alpha[h] + (p00 + p01 + p10 + p11);
        m_run[mt][h] = m_new;
        pa[h] = pack_bf16(p00, p01);                        // a0 / a1: tokens 2t, 2t+1
        pa[2 + h] = pack_bf16(p10, p11);                    // a2 / a3: tokens 8+2t, 8+2t+1
      }
#pragma unroll
      for (int n = 0; n < DV / 8; n += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, &sm->v[st][tw + ((lane >> 3) & 1) * 8 + (lane & 7)][(n + (lane >> 4)) * 8]);
        o_acc[mt][n][0] *= alpha[0]; o_acc[mt][n][1] *= alpha[0]; o_acc[mt][n][2] *= alpha[1]; o_acc[mt][n][3] *= alpha[1];
        o_acc[mt][n + 1][0] *= alpha[0]; o_acc[mt][n + 1][1] *= alpha[0]; o_acc[mt][n + 1][2] *= alpha[1]; o_acc[mt][n + 1][3] *= alpha[1];
        mma_bf16(o_acc[mt][n], pa, vb[0], vb[1]);
        mma_bf16(o_acc[mt][n + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
  __pipeline_wait_prior(0);
  __syncthreads();
  // ---- merge the 4 per-warp streams (the K and V rings are scratch now) ----
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_run[mt][h] += __shfl_xor_sync(0xffffffffu, l_run[mt][h], 1);
      l_run[mt][h] += __shfl_xor_sync(0xffffffffu, l_run[mt][h], 2);
    }
  float* red_o = reinterpret_cast<float*>(&sm->k[0][0][0]);           // [4 warps][32 rows][DV]
  float* red_m = red_o + 4 * 32 * DV;                                  // [4][32]
  float* red_l = red_m + 4 * 32;                                       // [4][32]
  static_assert(sizeof(float) * (4 * 32 * DV + 256) <= sizeof(bf16) * 2 * BS * (DK + kPad + DV + kPad), "scratch fits in the rings");
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int n = 0; n < DV / 8; ++n) {
      float* lo = red_o + (warp * 32 + mt * 16 + g) * DV + n * 8 + 2 * t;
      lo[0] = o_acc[mt][n][0]; lo[1] = o_acc[mt][n][1];
      float* hi = lo + 8 * DV;
      hi[0] = o_acc[mt][n][2]; hi[1] = o_acc[mt][n][3];
    }
  if (t == 0) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        red_m[warp * 32 + mt * 16 + g + 8 * h] = m_run[mt][h];
        red_l[warp * 32 + mt * 16 + g + 8 * h] = l_run[mt][h];
      }
  }
  __syncthreads();
  for (int idx = tid; idx < rows * DV; idx += kThreads) {
    const int r = idx / DV, d = idx % DV;
    const int qi = members[r / rep];
    if (qi < 0) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w * 32 + r]);
    float den = 0.f, num = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float e = __expf(red_m[w * 32 + r] - M);
      den += e * red_l[w * 32 + r];
      num += e * red_o[(w * 32 + r) * DV + d];
    }
    const int64_t at = ((int64_t)qi * nq + kvh * rep + r % rep) * total_slots + split;
    part_o[at * DV + d] = den > 0.f ? num / den : 0.f;
    if (d == 0) part_lse[at] = den > 0.f ? M + logf(den) : -INFINITY;
  }
}

template <int DV>
__global__ void combine_splits_tc_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                         bf16* __restrict__ out, int num_splits) {
  pdl_trigger();
  pdl_wait();
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

template <int DK, int DV>
void launch_tc(const at::Tensor& q, const at::Tensor& kc, const at::Tensor& vc, const at::Tensor& bt,
               const int* q_seq, const at::Tensor& ctx_len, at::Tensor& out, int nq, int nkv, int ns, float scale) {
  const int Tq = (int)q.size(0);
  auto st = at::cuda::getCurrentCUDAStream();
  const size_t smem = sizeof(SmemTC<DK, DV>);
  static bool configured[64] = {};               // the attribute is per device
  const int dev = q.get_device();
  TORCH_CHECK(dev >= 0 && dev < 64, "paged_decode_tc: device index out of range");
  if (!configured[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tc_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  at::Tensor po, pl;
  float* pop = nullptr; float* plp = nullptr;
  if (ns > 1) {
    po = at::empty({Tq, nq, ns, DV}, q.options().dtype(at::kFloat));
    pl = at::empty({Tq, nq, ns}, q.options().dtype(at::kFloat));
    pop = po.data_ptr<float>(); plp = pl.data_ptr<float>();
  }
  dim3 grid(Tq, nkv, ns);
  C10_CUDA_CHECK(launch_pdl(paged_decode_tc_kernel<DK, DV>, grid, dim3(kThreads), smem, st,
      (const bf16*)q.data_ptr(), (const bf16*)kc.data_ptr(), (const bf16*)vc.data_ptr(), bt.data_ptr<int>(),
      (int)bt.size(1), q_seq, ctx_len.data_ptr<int>(), (bf16*)out.data_ptr(), pop, plp, nq, nkv, ns, scale,
      (const int*)nullptr, 0, 0));
  if (ns > 1)
    C10_CUDA_CHECK(launch_pdl(combine_splits_tc_kernel<DV>, dim3(Tq * nq), dim3(((DV + 31) / 32) * 32), 0, st,
                              (const float*)pop, (const float*)plp, (bf16*)out.data_ptr(), ns));
}

}  // namespace

// Decode attention with shared prefixes (head dim 128, one query token per sequence).  grp_q [G, 8] int32: the
// query rows of each group's members (-1 = no member); grp_nblk [G] int32: blocks the members share (0 = unused
// group slot); blk_start [T] int32: blocks of every sequence that the prefix pass covers (0 outside a group).
at::Tensor paged_decode_tc_grouped(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                                   const at::Tensor& block_tables, const at::Tensor& ctx_len, const at::Tensor& grp_q,
                                   const at::Tensor& grp_nblk, const at::Tensor& blk_start, double scale,
                                   int64_t prefix_splits, int64_t suffix_splits) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous(), "paged_decode_tc_grouped: bf16 contiguous q");
  const int nq = (int)q.size(1), dk = (int)q.size(2);
  const int bs = (int)k_cache.size(1), nkv = (int)k_cache.size(2), dv = (int)v_cache.size(3);
  const int rep = nq / nkv;
  TORCH_CHECK(dk == 128 && dv == 128 && bs == BS && rep >= 1 && rep <= 4, "paged_decode_tc_grouped: head dim 128, 64-token blocks, at most 4 query heads per KV head");
  TORCH_CHECK(grp_q.scalar_type() == at::kInt && grp_q.dim() == 2 && grp_q.size(1) == 8 && grp_q.is_contiguous() &&
              grp_nblk.scalar_type() == at::kInt && grp_nblk.numel() == grp_q.size(0) && blk_start.scalar_type() == at::kInt &&
              blk_start.numel() == q.size(0), "paged_decode_tc_grouped: int32 group tables");
  const int Tq = (int)q.size(0), G = (int)grp_q.size(0);
  auto out = at::empty({q.size(0), nq, dv}, q.options());
  if (Tq == 0) return out;
  const int np = (int)std::max<int64_t>(prefix_splits, 1), nsx = (int)std::max<int64_t>(suffix_splits, 1);
  const int slots = np + nsx;
  auto po = at::empty({Tq, nq, slots, dv}, q.options().dtype(at::kFloat));
  auto pl = at::empty({Tq, nq, slots}, q.options().dtype(at::kFloat));
  auto st = at::cuda::getCurrentCUDAStream();
  const int dev = q.get_device();
  static bool configured[64] = {};
  TORCH_CHECK(dev >= 0 && dev < 64, "paged_decode_tc_grouped: device index out of range");
  if (!configured[dev]) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(paged_prefix_tc_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)sizeof(SmemPrefix<128, 128>)));
    C10_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tc_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)sizeof(SmemTC<128, 128>)));
    configured[dev] = true;
  }
  if (G > 0) {
    C10_CUDA_CHECK(launch_pdl(paged_prefix_tc_kernel<128, 128>, dim3(G, nkv, np), dim3(kThreads), sizeof(SmemPrefix<128, 128>), st,
        (const bf16*)q.data_ptr(), (const bf16*)k_cache.data_ptr(), (const bf16*)v_cache.data_ptr(), block_tables.data_ptr<int>(),
        (int)block_tables.size(1), grp_q.data_ptr<int>(), grp_nblk.data_ptr<int>(), po.data_ptr<float>(), pl.data_ptr<float>(),
        nq, nkv, np, slots, (float)scale));
  }
  C10_CUDA_CHECK(launch_pdl(paged_decode_tc_kernel<128, 128>, dim3(Tq, nkv, nsx), dim3(kThreads), sizeof(SmemTC<128, 128>), st,
      (const bf16*)q.data_ptr(), (const bf16*)k_cache.data_ptr(), (const bf16*)v_cache.data_ptr(), block_tables.data_ptr<int>(),
      (int)block_tables.size(1), (const int*)nullptr, ctx_len.data_ptr<int>(), (bf16*)out.data_ptr(), po.data_ptr<float>(),
      pl.data_ptr<float>(), nq, nkv, nsx, (float)scale, blk_start.data_ptr<int>(), np, slots));
  C10_CUDA_CHECK(launch_pdl(combine_splits_tc_kernel<128>, dim3(Tq * nq), dim3(128), 0, st, po.data_ptr<float>(), pl.data_ptr<float>(),
                            (bf16*)out.data_ptr(), slots));
  return out;
}

bool paged_decode_tc_supported(int64_t dk, int64_t dv, int64_t bs, int64_t rep) {
  const bool dims = (dk == 128 && dv == 128) || (dk == 64 && dv == 64) || (dk == 192 && dv == 128);
  return dims && bs == BS && rep >= 1 && rep <= 8;
}

at::Tensor paged_decode_tc(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                           const at::Tensor& block_tables, const c10::optional<at::Tensor>& q_seq,
                           const at::Tensor& ctx_len, double scale, int64_t num_splits) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous(), "paged_decode_tc: bf16 contiguous q");
  const int nq = (int)q.size(1), dk = (int)q.size(2);
  const int bs = (int)k_cache.size(1), nkv = (int)k_cache.size(2), dv = (int)v_cache.size(3);
  TORCH_CHECK(paged_decode_tc_supported(dk, dv, bs, nq / nkv), "paged_decode_tc: unsupported shape");
  auto out = at::empty({q.size(0), nq, dv}, q.options());
  if (q.size(0) == 0) return out;
  const int* qs = q_seq.has_value() ? q_seq->data_ptr<int>() : nullptr;
  const int ns = (int)std::max<int64_t>(num_splits, 1);
  if (dk == 128 && dv == 128) launch_tc<128, 128>(q, k_cache, v_cache, block_tables, qs, ctx_len, out, nq, nkv, ns, (float)scale);
  else if (dk == 64 && dv == 64) launch_tc<64, 64>(q, k_cache, v_cache, block_tables, qs, ctx_len, out, nq, nkv, ns, (float)scale);
  else launch_tc<192, 128>(q, k_cache, v_cache, block_tables, qs, ctx_len, out, nq, nkv, ns, (float)scale);
  return out;
}
