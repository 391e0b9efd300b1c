// Activation quantiser of the reference's FP8 linear layers, one pass over HBM (2 B read, 1 B written per element).
// Replaces div_clamp_to (inference/model/dit/dit_module.py:364-384) as called by PerTensorQuantizedFp8Linear.forward
// (:449-461) and PerChannelQuantizedFp8Linear.forward (:484-495):
//     x8 = e4m3( bf16( clamp( float(x) / float(scale), -448, 448 ) ) )
// with `scale` either one fp32 per input channel (last dimension) or a single fp32.  The reference rounds twice - to bf16
// and then to e4m3 - and so does this kernel, so the bytes are identical to the reference's, not merely close.  The
// reference does it in 256 MB slices with an fp32 temporary, a clamp pass, a bf16 pass, a cat and a cast.
// The GEMM that follows (bmm_fp8) is a plain library GEMM and stays one.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace magi {

// Thread = one 8-channel piece of the row (16-byte load, 8-byte store); its eight scales stay in registers while it
// walks down the rows, so a warp reads 512 contiguous bytes per row.
__global__ void __launch_bounds__(256) div_clamp_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int64_t x_stride,
                                                             const float* __restrict__ scale, int scale_is_scalar, int rows,
                                                             int cols, uint8_t* __restrict__ out, int64_t out_stride) {
  const int n_vec = cols >> 3;
  const int vec = blockIdx.x * blockDim.x + threadIdx.x;
  if (vec >= n_vec) return;
  float sc[8], rc[8];
  if (scale_is_scalar) {
    const float s0 = __ldg(scale);
#pragma unroll
    for (int k = 0; k < 8; ++k) sc[k] = s0;
  } else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(scale + vec * 8)), b = __ldg(reinterpret_cast<const float4*>(scale + vec * 8 + 4));
    sc[0] = a.x; sc[1] = a.y; sc[2] = a.z; sc[3] = a.w; sc[4] = b.x; sc[5] = b.y; sc[6] = b.z; sc[7] = b.w;
  }
  // A reciprocal that is zero, subnormal, inf or NaN (a scale outside the normal fp32 range) sends its whole column down
  // the exact-division branch: the window test below then always fires.
  uint32_t force[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rc[k] = __frcp_rn(sc[k]);
    const uint32_t e = __float_as_uint(rc[k]) & 0x7f800000u;
    force[k] = (e == 0u || e == 0x7f800000u) ? 0xffffffffu : 0x10u;
  }
  constexpr int kRowsInFlight = 4;
  const int step = gridDim.y * kRowsInFlight;
  auto fetch = [&](int r0, uint4 (&dst)[kRowsInFlight]) {
#pragma unroll
    for (int i = 0; i < kRowsInFlight; ++i)
      if (r0 + i < rows) dst[i] = __ldg(reinterpret_cast<const uint4*>(x + (int64_t)(r0 + i) * x_stride + vec * 8));
  };
  uint4 raw[kRowsInFlight], nxt[kRowsInFlight];
  fetch(blockIdx.y * kRowsInFlight, raw);
  for (int r0 = blockIdx.y * kRowsInFlight; r0 < rows; r0 += step) {
    fetch(r0 + step, nxt);  // the next group's loads are in flight while this group is converted
#pragma unroll
    for (int i = 0; i < kRowsInFlight; ++i) {
      if (r0 + i >= rows) break;
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      float q[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float v = __uint_as_float((k & 1) ? (w[k >> 1] & 0xffff0000u) : (w[k >> 1] << 16));
        // x * (1/scale) is within two fp32 ulps of the IEEE quotient, so it rounds to the same bf16 value unless its low
        // 16 bits sit next to the bf16 rounding boundary 0x8000: only then is the quotient taken exactly (about one
        // element in four thousand).  A product that is zero, subnormal or infinite needs no care: the exact quotient
        // then has the same sign and quantises to the same byte (0 or +-448).  The bytes are the reference's.
        float qk = v * rc[k];
        if (((__float_as_uint(qk) + 0x8u - 0x8000u) & 0xffffu) < force[k]) qk = __fdiv_rn(v, sc[k]);
        q[k] = qk;
      }
      // round to bf16 (the reference's intermediate), then to e4m3 with saturation: values beyond +-448 - the reference
      // clamps them before the bf16 rounding - land on +-448 either way
      uint32_t o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(q[4 * h], q[4 * h + 1]), p1 = __floats2bfloat162_rn(q[4 * h + 2], q[4 * h + 3]);
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(__bfloat1622float2(p0), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(__bfloat1622float2(p1), __NV_SATFINITE, __NV_E4M3);
        o[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(out + (int64_t)(r0 + i) * out_stride + vec * 8) = make_uint2(o[0], o[1]);
    }
#pragma unroll
    for (int i = 0; i < kRowsInFlight; ++i) raw[i] = nxt[i];
  }
}

}  // namespace magi

extern "C" int magi_div_clamp_to_e4m3(magi_ctx* ctx, const void* x, int64_t x_stride, int rows, int cols, const float* scale,
                                      int scale_is_scalar, void* out, int64_t out_stride, void* stream) {
  using namespace magi;
  if (!ctx) return MAGI_E_BADARG;
  if (!x || !scale || !out || rows < 0 || cols <= 0) return set_err(ctx, MAGI_E_BADARG, "div_clamp_to: null tensor or bad shape");
  if (cols % 8) return set_err(ctx, MAGI_E_BADARG, "div_clamp_to: the last dimension must be a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (x_stride & 7) || (reinterpret_cast<uintptr_t>(out) & 7) || (out_stride & 7) ||
      (!scale_is_scalar && (reinterpret_cast<uintptr_t>(scale) & 15)))
    return set_err(ctx, MAGI_E_ALIGN, "div_clamp_to: x and a per-channel scale must be 16-byte aligned, out 8-byte aligned, row strides multiples of 8");
  if (rows == 0) return MAGI_OK;
  const int n_vec = cols / 8;
  const int bx = (n_vec + 255) / 256;
  int64_t by = ((int64_t)ctx->sm_count * 8 + bx - 1) / bx;  // about 8 resident blocks per SM
  const int64_t need = (rows + 3) / 4;
  if (by > need) by = need;
  if (by > 65535) by = 65535;
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  div_clamp_e4m3_kernel<<<dim3(bx, (unsigned)by), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), x_stride, scale, scale_is_scalar, rows, cols, static_cast<uint8_t*>(out), out_stride);
  cudaError_t e = cudaGetLastError();
  if (prev != ctx->device) cudaSetDevice(prev);
  if (e != cudaSuccess) return set_err(ctx, MAGI_E_CUDA, "div_clamp_to launch failed: %s", cudaGetErrorString(e));
  return MAGI_OK;
}
