// FP8 e4m3 support: block quantiser (per (128-token block, head) fp32 absmax scales), FP8 cache pages.
// The reference has no FP8 attention (its fp8 path is the linear layers, inference/model/dit/dit_module.py:431-487);
// this defines the library's own format: x8 = e4m3(x / scale), scale = absmax / 448 (1 for an all-zero block),
// 128-token blocks counted from each multiple of chunk_tokens so that they coincide with the attention kernel's tiles.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace magi {

// One CTA per (block, head): 256 threads, thread = (row group, 16-byte column chunk); the block's elements stay in
// registers between the absmax pass and the convert pass, so HBM sees one read and one (half-size) write.
__global__ void __launch_bounds__(256) quantize_block128_kernel(const __nv_bfloat16* x, int64_t stride_t, int64_t stride_h, int T,
                                                                int H, int chunk_tokens, int blocks_per_chunk, uint8_t* x8,
                                                                uint8_t* x8_lo, int64_t o_stride_t, int64_t o_stride_h,
                                                                float* scales) {
  const int blk = blockIdx.x, h = blockIdx.y;
  const int c = blk / blocks_per_chunk, b = blk - c * blocks_per_chunk;
  const int64_t t0 = (int64_t)c * chunk_tokens + (int64_t)b * kTileN;
  int64_t t1 = t0 + kTileN;
  const int64_t chunk_end = (int64_t)(c + 1) * chunk_tokens;
  if (t1 > chunk_end) t1 = chunk_end;
  if (t1 > T) t1 = T;
  const int rows = (int)(t1 - t0);  // may be <= 0 for the padding blocks of a short last chunk
  const int col = (threadIdx.x & 15) * 8;
  const int r0 = threadIdx.x >> 4;  // 16 row groups; rows r0, r0+16, ...
  uint4 v[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + i * 16;
    v[i] = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      v[i] = __ldg(reinterpret_cast<const uint4*>(x + (t0 + r) * stride_t + (int64_t)h * stride_h + col));
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) amax = fmaxf(amax, fmaxf(fabsf(__low2float(p[k])), fabsf(__high2float(p[k]))));
    }
  }
  __shared__ float s_red[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_red[i]);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (threadIdx.x == 0) scales[(int64_t)blk * H + h] = scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + i * 16;
    if (r < rows) {
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      // x / scale with IEEE division: bit-identical to the definition (x8 = round_e4m3(x / scale))
      float f[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        f[2 * k] = __fdiv_rn(__low2float(p[k]), scale);
        f[2 * k + 1] = __fdiv_rn(__high2float(p[k]), scale);
      }
      uint32_t w[2], wl[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * k], f[4 * k + 1]), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * k + 2], f[4 * k + 3]), __NV_SATFINITE, __NV_E4M3);
        w[k] = lo | (hi << 16);
      }
      if (x8_lo) {  // second e4m3 term: the rounding residual of the first, same block scale
        const uint8_t* wb = reinterpret_cast<const uint8_t*>(w);
        float res[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const __half_raw hr = __nv_cvt_fp8_to_halfraw(wb[k], __NV_E4M3);
          res[k] = f[k] - __half2float(*reinterpret_cast<const __half*>(&hr));
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(res[4 * k], res[4 * k + 1]), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(res[4 * k + 2], res[4 * k + 3]), __NV_SATFINITE, __NV_E4M3);
          wl[k] = lo | (hi << 16);
        }
        *reinterpret_cast<uint2*>(x8_lo + (t0 + r) * o_stride_t + (int64_t)h * o_stride_h + col) = make_uint2(wl[0], wl[1]);
      }
      *reinterpret_cast<uint2*>(x8 + (t0 + r) * o_stride_t + (int64_t)h * o_stride_h + col) = make_uint2(w[0], w[1]);
    }
  }
}

__global__ void __launch_bounds__(256) dequantize_block128_kernel(const uint8_t* x8, int64_t stride_t, int64_t stride_h, int T, int H,
                                                                  const float* scales, __nv_bfloat16* out) {
  // grid: (ceil(T/128), H); out contiguous [T, H, 128]; blocks counted from row 0
  const int blk = blockIdx.x, h = blockIdx.y;
  const float scale = scales[(int64_t)blk * H + h];
  const int col = (threadIdx.x & 15) * 8, r0 = threadIdx.x >> 4;
  for (int r = r0; r < kTileN; r += 16) {
    const int64_t t = (int64_t)blk * kTileN + r;
    if (t >= T) break;
    const uint2 raw = *reinterpret_cast<const uint2*>(x8 + t * stride_t + (int64_t)h * stride_h + col);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    __nv_bfloat16 o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(b[k], __NV_E4M3);
      o[k] = __float2bfloat16(__half2float(*reinterpret_cast<const __half*>(&hr)) * scale);
    }
    *reinterpret_cast<uint4*>(out + (t * H + h) * kHeadDim + col) = *reinterpret_cast<const uint4*>(o);
  }
}

int launch_quantize(magi_ctx* ctx, const void* x, int64_t stride_t, int64_t stride_h, int T, int H, int chunk_tokens, void* x8,
                    void* x8_lo, int64_t o_stride_t, int64_t o_stride_h, float* scales, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (stride_t & 7) || (stride_h & 7) || (reinterpret_cast<uintptr_t>(x8) & 7) ||
      (reinterpret_cast<uintptr_t>(x8_lo) & 7) ||
      (o_stride_t & 7) || (o_stride_h & 7))
    return set_err(ctx, MAGI_E_ALIGN, "quantise: x must be 16-byte aligned (strides multiple of 8), x8 8-byte aligned");
  if (T == 0) return MAGI_OK;
  const int bpc = (chunk_tokens + kTileN - 1) / kTileN;
  const int n_chunks = (T + chunk_tokens - 1) / chunk_tokens;
  dim3 grid(n_chunks * bpc, H);
  quantize_block128_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), stride_t, stride_h, T, H, chunk_tokens,
                                                     bpc, reinterpret_cast<uint8_t*>(x8), reinterpret_cast<uint8_t*>(x8_lo), o_stride_t,
                                                     o_stride_h, scales);
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

int launch_cache_quant_append(magi_kv_cache* c, int slot, const void* k, int64_t kst, int64_t ksh, const void* v, int64_t vst,
                              int64_t vsh, int n_tokens, int token_offset, cudaStream_t stream) {
  const int Hkv = c->d.n_kv_heads;
  const int64_t row_bytes = (int64_t)Hkv * kHeadDim;
  const int64_t row0 = (int64_t)slot * c->page_cap + token_offset;
  const int64_t blk0 = (int64_t)slot * c->blocks_per_page + token_offset / kTileN;
  int rc = launch_quantize(c->ctx, k, kst, ksh, n_tokens, Hkv, c->page_cap, static_cast<uint8_t*>(c->k_pool) + row0 * row_bytes,
                           nullptr, row_bytes, kHeadDim, c->k_scale + blk0 * Hkv, stream);
  if (rc) return rc;
  return launch_quantize(c->ctx, v, vst, vsh, n_tokens, Hkv, c->page_cap, static_cast<uint8_t*>(c->v_pool) + row0 * row_bytes,
                         nullptr, row_bytes, kHeadDim, c->v_scale + blk0 * Hkv, stream);
}

int launch_cache_dequant_read(magi_kv_cache* c, int slot, void* k_out, void* v_out, int n_tokens, int token_offset,
                              cudaStream_t stream) {
  const int Hkv = c->d.n_kv_heads;
  const int64_t row_bytes = (int64_t)Hkv * kHeadDim;
  const int64_t row0 = (int64_t)slot * c->page_cap + token_offset;
  const int64_t blk0 = (int64_t)slot * c->blocks_per_page + token_offset / kTileN;
  dim3 grid((n_tokens + kTileN - 1) / kTileN, Hkv);
  dequantize_block128_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(c->k_pool) + row0 * row_bytes, row_bytes, kHeadDim,
                                                       n_tokens, Hkv, c->k_scale + blk0 * Hkv, reinterpret_cast<__nv_bfloat16*>(k_out));
  dequantize_block128_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(c->v_pool) + row0 * row_bytes, row_bytes, kHeadDim,
                                                       n_tokens, Hkv, c->v_scale + blk0 * Hkv, reinterpret_cast<__nv_bfloat16*>(v_out));
  MAGI_CUDA_OK(c->ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi

extern "C" int magi_quantize_e4m3_block128(magi_ctx* ctx, const void* x, int64_t stride_t, int64_t stride_h, int T, int H,
                                           int chunk_tokens, void* x8, void* x8_lo, float* scales, void* stream) {
  if (!ctx) return MAGI_E_BADARG;
  if (!x || !x8 || !scales || T < 0 || H <= 0 || chunk_tokens <= 0) return magi::set_err(ctx, MAGI_E_BADARG, "quantise: bad argument");
  return magi::launch_quantize(ctx, x, stride_t, stride_h, T, H, chunk_tokens, x8, x8_lo, (int64_t)H * magi::kHeadDim, magi::kHeadDim, scales,
                               reinterpret_cast<cudaStream_t>(stream));
}
