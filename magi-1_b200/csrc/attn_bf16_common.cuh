// Pieces shared by the bf16 attention kernels: tile constants, the by-value kernel parameters and the per-row softmax
// building blocks (one thread = one query row = one TMEM lane).
#pragma once
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace magi {
using namespace ptx;

constexpr int kAttnThreads = 384;
constexpr float kRedoRowSum = 32768.0f;  // 128 columns * 2^8: the fast path is redone for any row sum above this
constexpr int kTileBytes = kTileN * kHeadDim * 2;  // 32768: one 128x128 bf16 tile
constexpr int kHalfBytes = kTileBytes / 2;         // a [128 x 64] half tile = one 128-byte-swizzled TMA box
constexpr uint32_t kSw128 = 2;

struct AttnKernelParams {
  const void* plan;
  __nv_bfloat16* out;
  int64_t o_stride_t, o_stride_h;
  int64_t o_stride_block;  // head-block output layout (o_hpb > 0): see head_col()
  int o_hpb;
  float* lse;
  int n_q_heads;
  int group;          // q heads per kv head
  float scale;        // softmax scale
  float scale_log2;   // scale * log2(e)
  // fused output exchange: rank d owns q rows [peer_off[d], peer_off[d+1]) and receives them at peer_out[d]
  int n_peers;        // 0: plain output to `out`
  int head_offset;
  int peer_off[17];
  __nv_bfloat16* peer_out[16];
};

// ---- softmax building blocks: one thread = one row; s[] holds the row's 128 scores (fp32 bits) and receives the bf16
// weight pairs of columns [kC0, kC0 + kN) in s[kC0/2 .. (kC0 + kN)/2).
template <int kC0, int kN>
__device__ __forceinline__ void load_s_cols(uint32_t tS, uint32_t (&s)[kTileN], int valid) {
#pragma unroll
  for (int c = kC0; c < kC0 + kN; c += 32) tmem_ld32(tS + c, s + c);
  tmem_wait_ld();
  if (valid < kC0 + kN) {
#pragma unroll
    for (int c = kC0; c < kC0 + kN; ++c)
      if (c >= valid) s[c] = 0xff800000u;  // -inf
  }
}

// Fast path: exponentials against the maximum already baked into O and l; no maximum is computed.  A row whose scores
// outgrew that reference shows in its row sum: above 128 * 2^8 (some weight is then above 2^8; inf and NaN also land
// there) the tile is redone from the S still held in TMEM.  Scale-and-subtract and the row sum run as packed fp32 pairs
// (half the instructions).  Returns the row sum.
__device__ __forceinline__ float softmax_fast(uint32_t (&s)[kTileN], float sl2, float m_used) {
  const float neg_m = -m_used * sl2;
  uint64_t rs01 = f2_pack(0.f, 0.f), rs23 = rs01;
  const uint64_t sl2_2 = f2_pack(sl2, sl2), neg_m2 = f2_pack(neg_m, neg_m);
#pragma unroll
  for (int c = 0; c < kTileN; c += 4) {
    float x0, x1, x2, x3;
    f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sl2_2, neg_m2), x0, x1);
    f2_unpack(f2_fma(f2_pack(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])), sl2_2, neg_m2), x2, x3);
    const float p0 = ex2(x0), p1 = ex2(x1), p2 = ex2(x2), p3 = ex2(x3);
    rs01 = f2_add(rs01, f2_pack(p0, p1));
    rs23 = f2_add(rs23, f2_pack(p2, p3));
    s[c >> 1] = pack_bf16x2(p0, p1);
    s[(c >> 1) + 1] = pack_bf16x2(p2, p3);
  }
  float r0, r1, r2, r3;
  f2_unpack(rs01, r0, r1);
  f2_unpack(rs23, r2, r3);
  return (r0 + r2) + (r1 + r3);
}

// Exact path (first tile, or the running maximum moved): new reference maximum over these columns, then the
// exponentials.  Rows that did not move by more than 2^8 keep their reference (alpha = 1).  Returns the row sum.
template <int kC0, int kN>
__device__ __forceinline__ float softmax_exact(uint32_t (&s)[kTileN], float sl2, float& m_used, float& alpha) {
  float mxa[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) mxa[c] = __uint_as_float(s[kC0 + c]);
#pragma unroll
  for (int c = 8; c < kN; ++c) mxa[c & 7] = fmaxf(mxa[c & 7], __uint_as_float(s[kC0 + c]));
  const float mx = fmaxf(fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])), fmaxf(fmaxf(mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
  const float m_new = fmaxf(m_used, mx);
  const bool need = (m_new - m_used) * sl2 > 8.0f;
  const float m_cur = need ? m_new : m_used;
  alpha = need ? ex2((m_used - m_new) * sl2) : 1.0f;
  const float neg_m = -m_cur * sl2;
  float rs[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int c = kC0; c < kC0 + kN; c += 4) {
    const float p0 = ex2(fmaf(__uint_as_float(s[c]), sl2, neg_m));
    const float p1 = ex2(fmaf(__uint_as_float(s[c + 1]), sl2, neg_m));
    const float p2 = ex2(fmaf(__uint_as_float(s[c + 2]), sl2, neg_m));
    const float p3 = ex2(fmaf(__uint_as_float(s[c + 3]), sl2, neg_m));
    rs[0] += p0;
    rs[1] += p1;
    rs[2] += p2;
    rs[3] += p3;
    s[c >> 1] = pack_bf16x2(p0, p1);
    s[(c >> 1) + 1] = pack_bf16x2(p2, p3);
  }
  m_used = m_cur;
  return (rs[0] + rs[2]) + (rs[1] + rs[3]);
}

__device__ __forceinline__ void rescale_o(uint32_t tO, float alpha) {
#pragma unroll 1
  for (int c4 = 0; c4 < 4; ++c4) {
    uint32_t o[32];
    tmem_ld32(tO + c4 * 32, o);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
    tmem_st32(tO + c4 * 32, o);
  }
}

}  // namespace magi
