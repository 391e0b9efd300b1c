// Fused per-head norm + 3D RoPE + re-layout (HBM-bound: one bf16 read and one bf16 write per element).
// Arithmetic order follows FullyParallelAttention.get_q (inference/model/dit/dit_module.py:953-963):
// fp32 upcast, LayerNorm over the 128 channels with weight gamma+1 and bias (:355-357), non-interleaved
// rotary on the first 2*rot_pairs channels in fp32, one rounding to bf16 at the end.
//
// Main kernels: a QUARTER-warp (prologue8_kernel, rot_pairs % 8 == 0: the reference's 48) or a HALF-warp
// (prologue16_kernel, any rot_pairs % 4 == 0) owns one (token, head) row, 16 or 8 channels per lane with both channels
// of a rotary pair in the same lane, so a warp instruction serves four or two rows and the rotation needs no shuffle;
// row index arithmetic is 32-bit.  The generic kernel (4 channels per lane, one row per warp) covers source-blocked
// inputs, rows that are only 8-byte aligned and the plain strided copy.
#include <cuda_bf16.h>

#include <initializer_list>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace magi {

struct PrologueKernelParams {
  const __nv_bfloat16* x;
  int64_t x_stride_t, x_stride_h, x_stride_block;
  int x_heads_per_block;
  int T, H;
  const float* gamma;
  const float* beta;
  float eps;
  int norm_mode;
  int rot_pairs;
  const float* cos;
  const float* sin;
  __nv_bfloat16* out;
  int64_t out_stride_t, out_stride_h, out_stride_block;
  int heads_per_block;
  int use_block_ptrs;              // destination base of block b is out_blocks[b] instead of out + b * out_stride_block
  __nv_bfloat16* out_blocks[16];
};

constexpr int kRowsPerIter = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

template <bool kNormRope>
__global__ void __launch_bounds__(256) prologue_kernel(PrologueKernelParams p) {
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  const int64_t n_rows = (int64_t)p.T * p.H;
  const int d = lane * 4;

  float4 g4 = make_float4(1.f, 1.f, 1.f, 1.f), b4 = make_float4(0.f, 0.f, 0.f, 0.f);
  int partner = lane;
  float sign = 0.f;  // -1 for the first rotary half (x1*cos - x2*sin), +1 for the second (x2*cos + x1*sin)
  int cs_off = 0;
  if (kNormRope) {
    g4 = *reinterpret_cast<const float4*>(p.gamma + d);
    g4.x += 1.f; g4.y += 1.f; g4.z += 1.f; g4.w += 1.f;
    if (p.beta && p.norm_mode == MAGI_NORM_LAYERNORM_1P) b4 = *reinterpret_cast<const float4*>(p.beta + d);
    const int rp4 = p.rot_pairs >> 2;
    if (lane < rp4) { partner = lane + rp4; sign = -1.f; cs_off = d; }
    else if (lane < 2 * rp4) { partner = lane - rp4; sign = 1.f; cs_off = d - p.rot_pairs; }
  }

  for (int64_t base = (int64_t)warp_global * kRowsPerIter; base < n_rows; base += (int64_t)n_warps * kRowsPerIter) {
    uint2 raw[kRowsPerIter];
    int tt[kRowsPerIter], hh[kRowsPerIter];
#pragma unroll
    for (int i = 0; i < kRowsPerIter; ++i) {
      const int64_t r = base + i;
      raw[i] = make_uint2(0, 0);
      tt[i] = -1;
      hh[i] = 0;
      if (r < n_rows) {
        tt[i] = (int)(r / p.H);
        hh[i] = (int)(r - (int64_t)tt[i] * p.H);
        const int xb = p.x_heads_per_block > 0 ? hh[i] / p.x_heads_per_block : 0;
        const int xh = p.x_heads_per_block > 0 ? hh[i] - xb * p.x_heads_per_block : hh[i];
        raw[i] = __ldg(reinterpret_cast<const uint2*>(p.x + (int64_t)xb * p.x_stride_block + (int64_t)tt[i] * p.x_stride_t +
                                                      (int64_t)xh * p.x_stride_h + d));
      }
    }
#pragma unroll
    for (int i = 0; i < kRowsPerIter; ++i) {
      if (tt[i] < 0) continue;  // warp-uniform
      uint2 res = raw[i];
      if (kNormRope) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw[i].x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw[i].y);
        float4 v = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
        float4 y;
        if (p.norm_mode == MAGI_NORM_LAYERNORM_1P) {
          const float mean = warp_sum(v.x + v.y + v.z + v.w) * (1.f / kHeadDim);
          v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
          const float var = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) * (1.f / kHeadDim);
          const float rstd = rsqrtf(var + p.eps);
          y = make_float4(v.x * rstd * g4.x + b4.x, v.y * rstd * g4.y + b4.y, v.z * rstd * g4.z + b4.z,
                          v.w * rstd * g4.w + b4.w);
        } else {
          const float ms = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) * (1.f / kHeadDim);
          const float rstd = rsqrtf(ms + p.eps);
          y = make_float4(v.x * rstd * g4.x, v.y * rstd * g4.y, v.z * rstd * g4.z, v.w * rstd * g4.w);
        }
        float4 o;
        o.x = __shfl_sync(0xffffffffu, y.x, partner);
        o.y = __shfl_sync(0xffffffffu, y.y, partner);
        o.z = __shfl_sync(0xffffffffu, y.z, partner);
        o.w = __shfl_sync(0xffffffffu, y.w, partner);
        if (sign != 0.f) {
          const float4 c = __ldg(reinterpret_cast<const float4*>(p.cos + (int64_t)tt[i] * p.rot_pairs + cs_off));
          const float4 s = __ldg(reinterpret_cast<const float4*>(p.sin + (int64_t)tt[i] * p.rot_pairs + cs_off));
          y.x = y.x * c.x + sign * (o.x * s.x);
          y.y = y.y * c.y + sign * (o.y * s.y);
          y.z = y.z * c.z + sign * (o.z * s.z);
          y.w = y.w * c.w + sign * (o.w * s.w);
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
        res.x = *reinterpret_cast<const uint32_t*>(&lo);
        res.y = *reinterpret_cast<const uint32_t*>(&hi);
      }
      const int blk = p.heads_per_block > 0 ? hh[i] / p.heads_per_block : 0;
      const int hs = p.heads_per_block > 0 ? hh[i] - blk * p.heads_per_block : hh[i];
      __nv_bfloat16* ob = p.use_block_ptrs ? p.out_blocks[blk] : p.out + (int64_t)blk * p.out_stride_block;
      *reinterpret_cast<uint2*>(ob + (int64_t)tt[i] * p.out_stride_t + (int64_t)hs * p.out_stride_h + d) = res;
    }
  }
}

#ifndef MAGI_PRO_ROWS
#define MAGI_PRO_ROWS 4
#endif
#ifndef MAGI_PRO_MINB
#define MAGI_PRO_MINB 3
#endif
constexpr int kRows16PerIter = MAGI_PRO_ROWS;  // rows (heads) per half-warp in flight: 256 B of loads each

// Main kernel.  A half-warp owns one (token, head) row of 128 channels, 8 per lane, laid out so that a rotary pair
// (c, c + rot_pairs) lives in ONE thread: lane l < rot_pairs/4 holds channels 4l..4l+3 and rot_pairs+4l..rot_pairs+4l+3,
// the remaining lanes hold the 128 - 2*rot_pairs pass-through channels, 8 consecutive ones each.  Every lane therefore
// moves two 8-byte pieces of the 256-byte row, the rotation needs no shuffle and each lane loads only its 4 cos / 4 sin.
// The statistics are taken in one pass (sum and sum of squares, two independent 4-level butterflies; var = E[x^2] - mean^2
// in fp32, far inside the bf16 rounding of the result), and the normalisation runs as packed fp32 pairs.
// Work unit of a half-warp: one token x `hg` consecutive heads (hg divides H).  cos/sin of the token are loaded once per
// unit and reused for its heads; the heads of a token are contiguous rows, so a unit streams hg * 256 contiguous bytes.
__global__ void __launch_bounds__(256, MAGI_PRO_MINB) prologue16_kernel(PrologueKernelParams p, int hg) {
  using namespace ptx;
  const int lane = threadIdx.x & 31;
  const int l16 = lane & 15;
  const unsigned hw_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;  // half-warp id
  const unsigned n_hw = (gridDim.x * blockDim.x) >> 4;
  const unsigned groups = (unsigned)p.H / (unsigned)hg;
  const unsigned n_units = (unsigned)p.T * groups;
  const int rp4 = p.rot_pairs >> 2;
  const bool rot = l16 < rp4;
  const int c0 = rot ? 4 * l16 : 2 * p.rot_pairs + 8 * (l16 - rp4);  // first four channels of this lane
  const int c1 = rot ? p.rot_pairs + 4 * l16 : c0 + 4;               // second four (the rotary partners)

  uint64_t g2[4], b2[4];  // (gamma + 1, beta) as packed pairs: [0],[1] = channels c0.., [2],[3] = channels c1..
  {
    const float4 ga = *reinterpret_cast<const float4*>(p.gamma + c0), gb = *reinterpret_cast<const float4*>(p.gamma + c1);
    g2[0] = f2_pack(ga.x + 1.f, ga.y + 1.f); g2[1] = f2_pack(ga.z + 1.f, ga.w + 1.f);
    g2[2] = f2_pack(gb.x + 1.f, gb.y + 1.f); g2[3] = f2_pack(gb.z + 1.f, gb.w + 1.f);
    b2[0] = b2[1] = b2[2] = b2[3] = f2_pack(0.f, 0.f);
    if (p.beta && p.norm_mode == MAGI_NORM_LAYERNORM_1P) {
      const float4 ba = *reinterpret_cast<const float4*>(p.beta + c0), bb = *reinterpret_cast<const float4*>(p.beta + c1);
      b2[0] = f2_pack(ba.x, ba.y); b2[1] = f2_pack(ba.z, ba.w); b2[2] = f2_pack(bb.x, bb.y); b2[3] = f2_pack(bb.z, bb.w);
    }
  }
  const bool layernorm = p.norm_mode == MAGI_NORM_LAYERNORM_1P;
  const unsigned hpb = (unsigned)p.heads_per_block;

  // both half-warps of a warp run the same number of iterations (shuffles are warp-wide): round the bound up to a pair
  const unsigned n_units_pad = (n_units + 1u) & ~1u;
  for (unsigned unit = hw_global; unit < n_units_pad; unit += n_hw) {
    const bool unit_live = unit < n_units;
    const unsigned uc = unit_live ? unit : 0u;
    const unsigned t = uc / groups;
    const unsigned h0 = (uc - t * groups) * (unsigned)hg;
    float4 cs = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (rot) {
      cs = __ldg(reinterpret_cast<const float4*>(p.cos + (int64_t)t * p.rot_pairs + 4 * l16));
      sn = __ldg(reinterpret_cast<const float4*>(p.sin + (int64_t)t * p.rot_pairs + 4 * l16));
    }
    const __nv_bfloat16* xrow = p.x + (int64_t)t * p.x_stride_t;
    for (int hb = 0; hb < hg; hb += kRows16PerIter) {
      uint2 ra[kRows16PerIter], rb[kRows16PerIter];
#pragma unroll
      for (int i = 0; i < kRows16PerIter; ++i) {
        const __nv_bfloat16* xr = xrow + (int64_t)(h0 + min(hb + i, hg - 1)) * p.x_stride_h;
        ra[i] = __ldg(reinterpret_cast<const uint2*>(xr + c0));
        rb[i] = __ldg(reinterpret_cast<const uint2*>(xr + c1));
      }
#pragma unroll
      for (int i = 0; i < kRows16PerIter; ++i) {
        // bf16 -> fp32 is a 16-bit shift: (lo, hi) of each 32-bit word
        const uint32_t w[4] = {ra[i].x, ra[i].y, rb[i].x, rb[i].y};
        uint64_t v2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) v2[k] = f2_pack(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u));
        uint64_t s2 = f2_add(f2_add(v2[0], v2[1]), f2_add(v2[2], v2[3]));
        uint64_t q2 = f2_fma(v2[0], v2[0], f2_fma(v2[1], v2[1], f2_fma(v2[2], v2[2], f2_fma(v2[3], v2[3], f2_pack(0.f, 0.f)))));
        float s_lo, s_hi, q_lo, q_hi;
        f2_unpack(s2, s_lo, s_hi);
        f2_unpack(q2, q_lo, q_hi);
        float sum = s_lo + s_hi, sq = q_lo + q_hi;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) {
          sum += __shfl_xor_sync(0xffffffffu, sum, off);
          sq += __shfl_xor_sync(0xffffffffu, sq, off);
        }
        const float mean = layernorm ? sum * (1.f / kHeadDim) : 0.f;
        const float var = fmaxf(sq * (1.f / kHeadDim) - mean * mean, 0.f);
        const float rstd = rsqrtf(var + p.eps);
        const uint64_t r2 = f2_pack(rstd, rstd), m2 = f2_pack(-mean * rstd, -mean * rstd);
        float y[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) f2_unpack(f2_fma(f2_fma(v2[k], r2, m2), g2[k], b2[k]), y[2 * k], y[2 * k + 1]);
        if (rot) {  // out1 = x1 cos - x2 sin, out2 = x1 sin + x2 cos  (x1 = y[0..3], x2 = y[4..7])
          const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float x1 = y[k], x2 = y[4 + k];
            y[k] = x1 * c[k] - x2 * s[k];
            y[4 + k] = x2 * c[k] + x1 * s[k];
          }
        }
        if (unit_live && hb + i < hg) {
          const unsigned h = h0 + hb + i;
          const unsigned blk = hpb > 0 ? h / hpb : 0u;
          const unsigned hs = hpb > 0 ? h - blk * hpb : h;
          __nv_bfloat16* ob = p.use_block_ptrs ? p.out_blocks[blk] : p.out + (int64_t)blk * p.out_stride_block;
          __nv_bfloat16* orow = ob + (int64_t)t * p.out_stride_t + (int64_t)hs * p.out_stride_h;
          *reinterpret_cast<uint2*>(orow + c0) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
          *reinterpret_cast<uint2*>(orow + c1) = make_uint2(pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
        }
      }
    }
  }
}

#ifndef MAGI_PRO8_ROWS
#define MAGI_PRO8_ROWS 4
#endif
#ifndef MAGI_PRO8_MINB
#define MAGI_PRO8_MINB 2
#endif
constexpr int kRows8PerIter = MAGI_PRO8_ROWS;  // rows (heads) per quarter-warp in flight: 256 B of loads each

// Quarter-warp form for rot_pairs % 8 == 0 (the reference's 48): EIGHT lanes own one (token, head) row, 16 channels per
// lane, so a warp instruction serves four rows.  Lane l < rot_pairs/8 holds channels 8l..8l+7 and their rotary partners
// rot_pairs+8l..rot_pairs+8l+7 (two 16-byte pieces); the remaining lanes hold 16 consecutive pass-through channels each.
// Against the half-warp form this halves the loads, stores and address arithmetic per element and brings the two
// reductions down from 8 to 6 shuffles per 16 (instead of 8) channels: the kernel is issue-bound once the SM clock
// drops under the power cap, which is the state it runs in right after an attention kernel.
__global__ void __launch_bounds__(256, MAGI_PRO8_MINB) prologue8_kernel(PrologueKernelParams p, int hg) {
  using namespace ptx;
  const int lane = threadIdx.x & 31;
  const int l8 = lane & 7;
  const unsigned qw_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;  // quarter-warp id
  const unsigned n_qw = (gridDim.x * blockDim.x) >> 3;
  const unsigned groups = (unsigned)p.H / (unsigned)hg;
  const unsigned n_units = (unsigned)p.T * groups;
  const int rp8 = p.rot_pairs >> 3;
  const bool rot = l8 < rp8;
  const int c0 = rot ? 8 * l8 : 2 * p.rot_pairs + 16 * (l8 - rp8);  // first eight channels of this lane
  const int c1 = rot ? p.rot_pairs + 8 * l8 : c0 + 8;               // second eight (the rotary partners)

  uint64_t g2[8], b2[8];  // (gamma + 1, beta) as packed pairs: [0..3] = channels c0.., [4..7] = channels c1..
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int c = half ? c1 : c0;
    const float4 ga = *reinterpret_cast<const float4*>(p.gamma + c), gb = *reinterpret_cast<const float4*>(p.gamma + c + 4);
    g2[4 * half + 0] = f2_pack(ga.x + 1.f, ga.y + 1.f); g2[4 * half + 1] = f2_pack(ga.z + 1.f, ga.w + 1.f);
    g2[4 * half + 2] = f2_pack(gb.x + 1.f, gb.y + 1.f); g2[4 * half + 3] = f2_pack(gb.z + 1.f, gb.w + 1.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) b2[4 * half + k] = f2_pack(0.f, 0.f);
    if (p.beta && p.norm_mode == MAGI_NORM_LAYERNORM_1P) {
      const float4 ba = *reinterpret_cast<const float4*>(p.beta + c), bb = *reinterpret_cast<const float4*>(p.beta + c + 4);
      b2[4 * half + 0] = f2_pack(ba.x, ba.y); b2[4 * half + 1] = f2_pack(ba.z, ba.w);
      b2[4 * half + 2] = f2_pack(bb.x, bb.y); b2[4 * half + 3] = f2_pack(bb.z, bb.w);
    }
  }
  const bool layernorm = p.norm_mode == MAGI_NORM_LAYERNORM_1P;
  const unsigned hpb = (unsigned)p.heads_per_block;

  // all four quarter-warps of a warp run the same number of iterations (shuffles are warp-wide)
  const unsigned n_units_pad = (n_units + 3u) & ~3u;
  for (unsigned unit = qw_global; unit < n_units_pad; unit += n_qw) {
    const bool unit_live = unit < n_units;
    const unsigned uc = unit_live ? unit : 0u;
    const unsigned t = uc / groups;
    const unsigned h0 = (uc - t * groups) * (unsigned)hg;
    uint64_t cs2[4], sn2[4];  // cos, sin of this lane's 8 rotary pairs, packed
#pragma unroll
    for (int k = 0; k < 4; ++k) { cs2[k] = f2_pack(1.f, 1.f); sn2[k] = f2_pack(0.f, 0.f); }
    if (rot) {
      const float4* cp = reinterpret_cast<const float4*>(p.cos + (int64_t)t * p.rot_pairs + 8 * l8);
      const float4* sp = reinterpret_cast<const float4*>(p.sin + (int64_t)t * p.rot_pairs + 8 * l8);
      const float4 ca = __ldg(cp), cb = __ldg(cp + 1), sa = __ldg(sp), sb = __ldg(sp + 1);
      cs2[0] = f2_pack(ca.x, ca.y); cs2[1] = f2_pack(ca.z, ca.w); cs2[2] = f2_pack(cb.x, cb.y); cs2[3] = f2_pack(cb.z, cb.w);
      sn2[0] = f2_pack(sa.x, sa.y); sn2[1] = f2_pack(sa.z, sa.w); sn2[2] = f2_pack(sb.x, sb.y); sn2[3] = f2_pack(sb.z, sb.w);
    }
    const __nv_bfloat16* xrow = p.x + (int64_t)t * p.x_stride_t;
    for (int hb = 0; hb < hg; hb += kRows8PerIter) {
      uint4 ra[kRows8PerIter], rb[kRows8PerIter];
#pragma unroll
      for (int i = 0; i < kRows8PerIter; ++i) {
        const __nv_bfloat16* xr = xrow + (int64_t)(h0 + min(hb + i, hg - 1)) * p.x_stride_h;
        ra[i] = __ldg(reinterpret_cast<const uint4*>(xr + c0));
        rb[i] = __ldg(reinterpret_cast<const uint4*>(xr + c1));
      }
#pragma unroll
      for (int i = 0; i < kRows8PerIter; ++i) {
        const uint32_t w[8] = {ra[i].x, ra[i].y, ra[i].z, ra[i].w, rb[i].x, rb[i].y, rb[i].z, rb[i].w};
        uint64_t v2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v2[k] = f2_pack(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u));
        uint64_t s2 = f2_add(f2_add(f2_add(v2[0], v2[1]), f2_add(v2[2], v2[3])), f2_add(f2_add(v2[4], v2[5]), f2_add(v2[6], v2[7])));
        uint64_t q2 = f2_pack(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; ++k) q2 = f2_fma(v2[k], v2[k], q2);
        float s_lo, s_hi, q_lo, q_hi;
        f2_unpack(s2, s_lo, s_hi);
        f2_unpack(q2, q_lo, q_hi);
        float sum = s_lo + s_hi, sq = q_lo + q_hi;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
          sum += __shfl_xor_sync(0xffffffffu, sum, off);
          sq += __shfl_xor_sync(0xffffffffu, sq, off);
        }
        const float mean = layernorm ? sum * (1.f / kHeadDim) : 0.f;
        const float var = fmaxf(sq * (1.f / kHeadDim) - mean * mean, 0.f);
        const float rstd = rsqrtf(var + p.eps);
        const uint64_t r2 = f2_pack(rstd, rstd), m2 = f2_pack(-mean * rstd, -mean * rstd);
        uint64_t y2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) y2[k] = f2_fma(f2_fma(v2[k], r2, m2), g2[k], b2[k]);
        if (rot) {  // out1 = x1 cos - x2 sin, out2 = x2 cos + x1 sin  (x1 = y2[0..3], x2 = y2[4..7])
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t x1 = y2[k], x2 = y2[4 + k];
            const uint64_t nsn = sn2[k] ^ 0x8000000080000000ull;  // -sin, both lanes
            y2[k] = f2_fma(x2, nsn, f2_fma(x1, cs2[k], f2_pack(0.f, 0.f)));
            y2[4 + k] = f2_fma(x1, sn2[k], f2_fma(x2, cs2[k], f2_pack(0.f, 0.f)));
          }
        }
        if (unit_live && hb + i < hg) {
          const unsigned h = h0 + hb + i;
          const unsigned blk = hpb > 0 ? h / hpb : 0u;
          const unsigned hs = hpb > 0 ? h - blk * hpb : h;
          __nv_bfloat16* ob = p.use_block_ptrs ? p.out_blocks[blk] : p.out + (int64_t)blk * p.out_stride_block;
          __nv_bfloat16* orow = ob + (int64_t)t * p.out_stride_t + (int64_t)hs * p.out_stride_h;
          uint32_t o[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float lo, hi;
            f2_unpack(y2[k], lo, hi);
            o[k] = pack_bf16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(orow + c0) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(orow + c1) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
    }
  }
}

static int check_prologue(magi_ctx* ctx, const magi_prologue_params* p, bool norm_rope) {
  if (!ctx) return MAGI_E_BADARG;
  if (!p || p->struct_size != sizeof(magi_prologue_params)) return set_err(ctx, MAGI_E_BADARG, "prologue: bad struct_size");
  if (!p->x || (!p->out && !p->out_block_ptrs) || p->T < 0 || p->H <= 0)
    return set_err(ctx, MAGI_E_BADARG, "prologue: null tensor or bad shape");
  if (p->out_block_ptrs) {
    if (p->heads_per_block <= 0 || p->H % p->heads_per_block || p->H / p->heads_per_block > 16)
      return set_err(ctx, MAGI_E_BADARG, "prologue: out_block_ptrs needs heads_per_block dividing H into at most 16 blocks");
    for (int b = 0; b < p->H / p->heads_per_block; ++b)
      if (!p->out_block_ptrs[b] || (reinterpret_cast<uintptr_t>(p->out_block_ptrs[b]) & 15))
        return set_err(ctx, MAGI_E_ALIGN, "prologue: out_block_ptrs[%d] is null or not 16-byte aligned", b);
  }
  if ((reinterpret_cast<uintptr_t>(p->x) & 7) || (reinterpret_cast<uintptr_t>(p->out) & 7) || (p->x_stride_t & 3) ||
      (p->x_stride_h & 3) || (p->x_stride_block & 3) || (p->out_stride_t & 3) || (p->out_stride_h & 3) ||
      (p->out_stride_block & 3))
    return set_err(ctx, MAGI_E_ALIGN, "prologue: pointers must be 8-byte aligned and strides multiples of 4 elements");
  if (norm_rope) {
    if (!p->gamma) return set_err(ctx, MAGI_E_BADARG, "prologue: gamma is required");
    if (p->norm_mode != MAGI_NORM_LAYERNORM_1P && p->norm_mode != MAGI_NORM_RMSNORM_1P)
      return set_err(ctx, MAGI_E_BADARG, "prologue: unknown norm_mode %d", p->norm_mode);
    if (p->rot_pairs < 0 || p->rot_pairs > 64 || (p->rot_pairs & 3))
      return set_err(ctx, MAGI_E_BADARG, "prologue: rot_pairs must be a multiple of 4 in [0,64]");
    if (p->rot_pairs > 0 && (!p->cos || !p->sin)) return set_err(ctx, MAGI_E_BADARG, "prologue: cos/sin required");
    if ((reinterpret_cast<uintptr_t>(p->gamma) & 15) || (reinterpret_cast<uintptr_t>(p->beta) & 15))
      return set_err(ctx, MAGI_E_ALIGN, "prologue: gamma/beta must be 16-byte aligned");
    if (p->rot_pairs > 0 && ((reinterpret_cast<uintptr_t>(p->cos) & 15) || (reinterpret_cast<uintptr_t>(p->sin) & 15)))
      return set_err(ctx, MAGI_E_ALIGN, "prologue: cos/sin must be 16-byte aligned");
  }
  return MAGI_OK;
}

static int launch_prologue(magi_ctx* ctx, const magi_prologue_params* p, bool norm_rope, cudaStream_t stream) {
  int rc = check_prologue(ctx, p, norm_rope);
  if (rc) return rc;
  if (p->T == 0) return MAGI_OK;
  PrologueKernelParams k;
  k.x = reinterpret_cast<const __nv_bfloat16*>(p->x);
  k.x_stride_t = p->x_stride_t;
  k.x_stride_h = p->x_stride_h;
  k.x_stride_block = p->x_stride_block;
  k.x_heads_per_block = (p->x_heads_per_block > 0 && p->x_heads_per_block < p->H) ? p->x_heads_per_block : 0;
  k.T = p->T;
  k.H = p->H;
  k.gamma = p->gamma;
  k.beta = p->beta;
  k.eps = p->eps;
  k.norm_mode = p->norm_mode;
  k.rot_pairs = p->rot_pairs;
  k.cos = p->cos;
  k.sin = p->sin;
  k.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  k.out_stride_t = p->out_stride_t;
  k.out_stride_h = p->out_stride_h;
  k.out_stride_block = p->out_stride_block;
  k.heads_per_block = (p->heads_per_block > 0 && (p->heads_per_block < p->H || p->out_block_ptrs)) ? p->heads_per_block : 0;
  k.use_block_ptrs = p->out_block_ptrs ? 1 : 0;
  for (int b = 0; b < 16; ++b)
    k.out_blocks[b] = (p->out_block_ptrs && b < p->H / p->heads_per_block) ? reinterpret_cast<__nv_bfloat16*>(p->out_block_ptrs[b]) : nullptr;
  const int64_t rows = (int64_t)p->T * p->H;
  const int64_t want = (rows + 8 * kRowsPerIter - 1) / (8 * kRowsPerIter);
  const int64_t cap = (int64_t)ctx->sm_count * 8;  // 8 x 256 threads resident per SM
  const int blocks = (int)(want < cap ? want : cap);
  // half-warp path: no source blocking, 16-byte aligned rows on both sides, < 2^32 rows (rot_pairs % 4 == 0 was checked)
  const bool wide = norm_rope && k.x_heads_per_block == 0 && rows < (1ll << 32) &&
                    !(reinterpret_cast<uintptr_t>(p->x) & 15) && !(reinterpret_cast<uintptr_t>(p->out) & 15) &&
                    !(p->x_stride_t & 7) && !(p->x_stride_h & 7) && !(p->out_stride_t & 7) && !(p->out_stride_h & 7) &&
                    !(p->out_stride_block & 7) && (p->rot_pairs == 0 || !((uintptr_t)p->cos & 15));
  if (wide) {
    int hg = 1;  // heads per unit: the largest of 8, 6, 4, 3, 2 that divides H
    for (int cand : {8, 6, 4, 3, 2})
      if (p->H % cand == 0) { hg = cand; break; }
    const int64_t units = rows / hg;
    const int64_t want16 = (units + 15) / 16;  // 16 half-warps per block
    const int64_t cap16 = (int64_t)ctx->sm_count * MAGI_PRO_MINB * 4;  // resident blocks per SM, x4 waves for balance
    if ((p->rot_pairs & 7) == 0) {  // eight lanes per row
      const int64_t want8 = (units + 31) / 32;  // 32 quarter-warps per block
      const int64_t cap8 = (int64_t)ctx->sm_count * MAGI_PRO8_MINB * 4;
      prologue8_kernel<<<(int)(want8 < cap8 ? want8 : cap8), 256, 0, stream>>>(k, hg);
    } else {
      prologue16_kernel<<<(int)(want16 < cap16 ? want16 : cap16), 256, 0, stream>>>(k, hg);
    }
  } else if (norm_rope) {
    prologue_kernel<true><<<blocks, 256, 0, stream>>>(k);
  } else {
    prologue_kernel<false><<<blocks, 256, 0, stream>>>(k);
  }
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi

extern "C" int magi_qk_norm_rope_fwd(magi_ctx* ctx, const magi_prologue_params* p, void* stream) {
  return magi::launch_prologue(ctx, p, true, reinterpret_cast<cudaStream_t>(stream));
}
extern "C" int magi_head_block_copy(magi_ctx* ctx, const magi_prologue_params* p, void* stream) {
  return magi::launch_prologue(ctx, p, false, reinterpret_cast<cudaStream_t>(stream));
}
