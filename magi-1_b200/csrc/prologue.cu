// Fused per-head norm + 3D RoPE + re-layout (HBM-bound: one bf16 read and one bf16 write per element).
// Arithmetic order follows FullyParallelAttention.get_q (inference/model/dit/dit_module.py:953-963):
// fp32 upcast, LayerNorm over the 128 channels with weight gamma+1 and bias (:355-357), non-interleaved
// rotary on the first 2*rot_pairs channels in fp32, one rounding to bf16 at the end.
//
// A warp owns one (token, head) row: lane l holds channels 4l..4l+3 (8-byte loads, 256 contiguous bytes per
// warp).  Rotary partners (c, c+rot_pairs) sit rot_pairs/4 lanes apart and are exchanged with one shuffle.
#include <cuda_bf16.h>

#include "common.cuh"

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
      *reinterpret_cast<uint2*>(p.out + (int64_t)blk * p.out_stride_block + (int64_t)tt[i] * p.out_stride_t +
                                (int64_t)hs * p.out_stride_h + d) = res;
    }
  }
}

static int check_prologue(magi_ctx* ctx, const magi_prologue_params* p, bool norm_rope) {
  if (!ctx) return MAGI_E_BADARG;
  if (!p || p->struct_size != sizeof(magi_prologue_params)) return set_err(ctx, MAGI_E_BADARG, "prologue: bad struct_size");
  if (!p->x || !p->out || p->T < 0 || p->H <= 0) return set_err(ctx, MAGI_E_BADARG, "prologue: null tensor or bad shape");
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
  k.heads_per_block = (p->heads_per_block > 0 && p->heads_per_block < p->H) ? p->heads_per_block : 0;
  const int64_t rows = (int64_t)p->T * p->H;
  const int64_t want = (rows + 8 * kRowsPerIter - 1) / (8 * kRowsPerIter);
  const int64_t cap = (int64_t)ctx->sm_count * 8;  // 8 x 256 threads resident per SM
  const int blocks = (int)(want < cap ? want : cap);
  if (norm_rope)
    prologue_kernel<true><<<blocks, 256, 0, stream>>>(k);
  else
    prologue_kernel<false><<<blocks, 256, 0, stream>>>(k);
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
