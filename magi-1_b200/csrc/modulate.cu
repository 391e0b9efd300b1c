// Gated post-norm residual of the DiT layer, one pass over HBM (HBM-bound: x and the residual read once, the result
// written once).  Replaces bias_modulate_add (inference/model/dit/dit_module.py:288-307) together with the Triton
// range_mod kernel inside it (:201-285):
//     y = post_norm( x.float() * gate[condition_map[row]].float() ) + residual.float()      -> cast to bf16
// post_norm = FusedLayerNorm over the hidden dimension with weight gamma (+1 when zero-centred) and bias (:355-357).
// The reference runs four fp32 passes here (x.float(), the gating kernel, layer_norm, the add) plus the casts.
//
// One CTA of 256 threads per row; thread t owns the 8-element vectors t, t + 256, t + 512, ... of the row (16- or
// 32-byte loads, fully coalesced), so the row lives in registers between the gating, the two reductions of a true
// two-pass LayerNorm (mean, then the variance of the centred values - what torch's layer_norm computes) and the store.
#include <cuda_bf16.h>

#include "common.cuh"

namespace magi {

constexpr int kModThreads = 256;
constexpr int kModMaxVec = 4;  // vectors of 8 per thread: hidden <= 8192

struct ModulateKernelParams {
  const void* x;
  const void* residual;  // may be null
  const void* gate;      // [n_gates, hidden]
  const void* cond_map;  // [rows] int32 or int64; null: gate row 0 for every row
  const float* gamma;    // null: no norm
  const float* beta;     // may be null
  __nv_bfloat16* out;
  int64_t x_stride, res_stride, gate_stride, out_stride;
  int rows, hidden, n_gates;
  int map_is_int64;
  int gamma_plus_one;
  float eps;
  int* status;  // device status word: receives MAGI_E_RANGE if a map entry is outside [0, n_gates)
};

template <bool kF32>
__device__ __forceinline__ void load8(const void* base, int64_t elem_off, float (&v)[8]) {
  if constexpr (kF32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + elem_off));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = __uint_as_float(w[k] << 16);
      v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}

// Sum over the block; `slot` is a 16-float scratch that no other reduction in flight uses.
__device__ __forceinline__ float block_sum(float v, float* slot) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kModThreads / 32; ++w) t += slot[w];
  return t;
}

template <bool kXF32, bool kResF32, bool kGateF32>
__global__ void __launch_bounds__(kModThreads) modulate_kernel(ModulateKernelParams p) {
  __shared__ float red[4][16];  // two reductions per row, rows alternate between two pairs of slots: no second barrier
  const int n_vec = p.hidden >> 3;
  const float inv_h = 1.0f / (float)p.hidden;
  int parity = 0;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
    long long g = 0;
    if (p.cond_map)
      g = p.map_is_int64 ? static_cast<const long long*>(p.cond_map)[row] : (long long)static_cast<const int*>(p.cond_map)[row];
    if (g < 0 || g >= p.n_gates) {  // uniform over the block: report and leave the row unwritten
      if (threadIdx.x == 0 && p.status) *p.status = MAGI_E_RANGE;
      continue;
    }
    float v[kModMaxVec][8];
    float sum = 0.f;
    // a bf16 residual is fetched together with x (12 more registers) so that the row pays one DRAM latency, not two
    uint4 res_raw[kModMaxVec];
    if constexpr (!kResF32) {
      if (p.residual) {
#pragma unroll
        for (int i = 0; i < kModMaxVec; ++i) {
          const int vec = threadIdx.x + i * kModThreads;
          if (vec < n_vec)
            res_raw[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.residual) +
                                                             (int64_t)row * p.res_stride + vec * 8));
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kModMaxVec; ++i) {
      const int vec = threadIdx.x + i * kModThreads;
      if (vec < n_vec) {
        float gt[8];
        load8<kXF32>(p.x, (int64_t)row * p.x_stride + vec * 8, v[i]);
        load8<kGateF32>(p.gate, g * p.gate_stride + vec * 8, gt);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[i][k] *= gt[k];
          sum += v[i][k];
        }
      }
    }
    if (p.gamma) {
      const float mean = block_sum(sum, red[2 * parity]) * inv_h;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < kModMaxVec; ++i)
        if (threadIdx.x + i * kModThreads < n_vec) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            v[i][k] -= mean;
            sq += v[i][k] * v[i][k];
          }
        }
      const float rstd = rsqrtf(block_sum(sq, red[2 * parity + 1]) * inv_h + p.eps);
#pragma unroll
      for (int i = 0; i < kModMaxVec; ++i) {
        const int vec = threadIdx.x + i * kModThreads;
        if (vec < n_vec) {
          float ga[8], be[8];
          load8<true>(p.gamma, vec * 8, ga);
#pragma unroll
          for (int k = 0; k < 8; ++k) be[k] = 0.f;
          if (p.beta) load8<true>(p.beta, vec * 8, be);
          const float one = p.gamma_plus_one ? 1.f : 0.f;
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] = v[i][k] * rstd * (ga[k] + one) + be[k];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kModMaxVec; ++i) {
      const int vec = threadIdx.x + i * kModThreads;
      if (vec < n_vec) {
        if (p.residual) {
          float r[8];
          if constexpr (kResF32) {
            load8<true>(p.residual, (int64_t)row * p.res_stride + vec * 8, r);
          } else {
            const uint32_t w[4] = {res_raw[i].x, res_raw[i].y, res_raw[i].z, res_raw[i].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              r[2 * k] = __uint_as_float(w[k] << 16);
              r[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) v[i][k] += r[k];
        }
        uint4 o;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(v[i][0], v[i][1]), t1 = __floats2bfloat162_rn(v[i][2], v[i][3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[i][4], v[i][5]), t3 = __floats2bfloat162_rn(v[i][6], v[i][7]);
        o.x = *reinterpret_cast<const uint32_t*>(&t0);
        o.y = *reinterpret_cast<const uint32_t*>(&t1);
        o.z = *reinterpret_cast<const uint32_t*>(&t2);
        o.w = *reinterpret_cast<const uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(p.out + (int64_t)row * p.out_stride + vec * 8) = o;
      }
    }
  }
}

template <bool A, bool B, bool C>
static void launch(const ModulateKernelParams& k, int blocks, cudaStream_t st) {
  modulate_kernel<A, B, C><<<blocks, kModThreads, 0, st>>>(k);
}

}  // namespace magi

using namespace magi;

extern "C" int magi_bias_modulate_add(magi_ctx* ctx, const magi_modulate_params* p, void* stream) {
  if (!ctx) return MAGI_E_BADARG;
  if (!p || p->struct_size != sizeof(magi_modulate_params)) return set_err(ctx, MAGI_E_BADARG, "modulate: bad struct_size");
  if (!p->x || !p->gate || !p->out || p->rows < 0 || p->hidden <= 0 || p->n_gates <= 0)
    return set_err(ctx, MAGI_E_BADARG, "modulate: null tensor or bad shape");
  if (p->hidden % 8 || p->hidden > 8 * kModThreads * kModMaxVec)
    return set_err(ctx, MAGI_E_BADARG, "modulate: hidden must be a multiple of 8, at most %d", 8 * kModThreads * kModMaxVec);
  for (int d : {p->x_dtype, p->residual_dtype, p->gate_dtype})
    if (d != MAGI_DTYPE_BF16 && d != MAGI_DTYPE_F32) return set_err(ctx, MAGI_E_BADARG, "modulate: dtypes are bf16 or f32");
  auto misaligned = [](const void* ptr, int64_t stride, int dtype) {
    const int esz = dtype == MAGI_DTYPE_F32 ? 4 : 2;
    return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ((stride * esz) & 15) != 0;
  };
  if (misaligned(p->x, p->x_stride, p->x_dtype) || misaligned(p->gate, p->gate_stride, p->gate_dtype) ||
      misaligned(p->out, p->out_stride, MAGI_DTYPE_BF16) || (p->residual && misaligned(p->residual, p->residual_stride, p->residual_dtype)) ||
      (reinterpret_cast<uintptr_t>(p->gamma) & 15) || (reinterpret_cast<uintptr_t>(p->beta) & 15))
    return set_err(ctx, MAGI_E_ALIGN, "modulate: pointers must be 16-byte aligned and row strides multiples of 16 bytes");
  if (p->rows == 0) return MAGI_OK;
  ModulateKernelParams k;
  k.x = p->x;
  k.residual = p->residual;
  k.gate = p->gate;
  k.cond_map = p->condition_map;
  k.gamma = p->gamma;
  k.beta = p->beta;
  k.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  k.x_stride = p->x_stride;
  k.res_stride = p->residual_stride;
  k.gate_stride = p->gate_stride;
  k.out_stride = p->out_stride;
  k.rows = p->rows;
  k.hidden = p->hidden;
  k.n_gates = p->n_gates;
  k.map_is_int64 = p->map_is_int64;
  k.gamma_plus_one = p->gamma_plus_one;
  k.eps = p->eps;
  k.status = reinterpret_cast<int*>(reinterpret_cast<char*>(ctx->workspace) + offsetof(PlanHeader, status));
  const int64_t cap = (int64_t)ctx->sm_count * 12;  // 3-4 resident blocks of 256 threads per SM, a few waves for balance
  const int blocks = (int)(p->rows < cap ? p->rows : cap);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  const int sel = (p->x_dtype == MAGI_DTYPE_F32 ? 4 : 0) | (p->residual_dtype == MAGI_DTYPE_F32 ? 2 : 0) | (p->gate_dtype == MAGI_DTYPE_F32 ? 1 : 0);
  switch (sel) {
    case 0: launch<false, false, false>(k, blocks, st); break;
    case 1: launch<false, false, true>(k, blocks, st); break;
    case 2: launch<false, true, false>(k, blocks, st); break;
    case 3: launch<false, true, true>(k, blocks, st); break;
    case 4: launch<true, false, false>(k, blocks, st); break;
    case 5: launch<true, false, true>(k, blocks, st); break;
    case 6: launch<true, true, false>(k, blocks, st); break;
    default: launch<true, true, true>(k, blocks, st); break;
  }
  cudaError_t e = cudaGetLastError();
  if (prev != ctx->device) cudaSetDevice(prev);
  if (e != cudaSuccess) return set_err(ctx, MAGI_E_CUDA, "modulate launch failed: %s", cudaGetErrorString(e));
  return MAGI_OK;
}
