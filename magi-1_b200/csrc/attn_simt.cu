// Diagnostic twin of the attention forward: same plan, CUDA-core fp32 arithmetic, no tensor cores, no TMA.
// One warp per (q row, q head): lanes split the 128 channels, online softmax over the range's segments.
// Used by tests to tell a planner fault from a tensor-core kernel fault; never a dispatch target.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"

namespace magi {

struct SimtParams {
  const void* plan;
  const __nv_bfloat16* q;
  int64_t q_stride_t, q_stride_h;
  const __nv_bfloat16* k[2];  // [0] current, [1] cache pool
  const __nv_bfloat16* v[2];
  int64_t k_stride_t[2], k_stride_h[2], v_stride_t[2], v_stride_h[2];
  __nv_bfloat16* out;
  int64_t o_stride_t, o_stride_h;
  int64_t o_stride_block;  // head-block output layout (o_hpb > 0): see head_col()
  int o_hpb;
  float* lse;
  int n_q_heads, group;
  float scale;
};

__device__ __forceinline__ float4 ld_bf16x4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

__global__ void __launch_bounds__(256) attn_simt_kernel(SimtParams p) {
  PlanView pv = plan_view(const_cast<void*>(p.plan));
  if ((int)blockIdx.x >= pv.hdr->n_items) return;
  const WorkItem it = pv.items[blockIdx.x];
  const int head = blockIdx.y, kvh = head / p.group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < it.q_rows; r += 8) {
    const int64_t row = it.q_row0 + r;
    const float4 q4 = ld_bf16x4(p.q + row * p.q_stride_t + (int64_t)head * p.q_stride_h + lane * 4);
    float m = -INFINITY, l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sg_i = it.seg_begin; sg_i < it.seg_end; ++sg_i) {
      const Segment sg = pv.segs[sg_i];
      const __nv_bfloat16* kb = p.k[sg.src] + (int64_t)kvh * p.k_stride_h[sg.src] + lane * 4;
      const __nv_bfloat16* vb = p.v[sg.src] + (int64_t)kvh * p.v_stride_h[sg.src] + lane * 4;
      for (int t = 0; t < sg.len; ++t) {
        const float4 k4 = ld_bf16x4(kb + (int64_t)(sg.row0 + t) * p.k_stride_t[sg.src]);
        float s = q4.x * k4.x + q4.y * k4.y + q4.z * k4.z + q4.w * k4.w;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        s *= p.scale;
        const float mn = fmaxf(m, s);
        const float a = __expf(m - mn), w = __expf(s - mn);
        const float4 v4 = ld_bf16x4(vb + (int64_t)(sg.row0 + t) * p.v_stride_t[sg.src]);
        o.x = o.x * a + w * v4.x;
        o.y = o.y * a + w * v4.y;
        o.z = o.z * a + w * v4.z;
        o.w = o.w * a + w * v4.w;
        l = l * a + w;
        m = mn;
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * inv, o.y * inv), hi = __floats2bfloat162_rn(o.z * inv, o.w * inv);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p.out + row * p.o_stride_t + head_col(p, head) + lane * 4) = u;
    if (p.lse && lane == 0) p.lse[row * p.n_q_heads + head] = l > 0.f ? m + logf(l) : -INFINITY;
  }
}

int launch_attn_simt(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream) {
  SimtParams sp;
  sp.plan = ctx->workspace;
  sp.q = reinterpret_cast<const __nv_bfloat16*>(p->q);
  sp.q_stride_t = p->q_stride_t;
  sp.q_stride_h = p->q_stride_h;
  sp.k[0] = reinterpret_cast<const __nv_bfloat16*>(p->k);
  sp.v[0] = reinterpret_cast<const __nv_bfloat16*>(p->v);
  sp.k_stride_t[0] = p->k_stride_t;
  sp.k_stride_h[0] = p->k_stride_h;
  sp.v_stride_t[0] = p->v_stride_t;
  sp.v_stride_h[0] = p->v_stride_h;
  sp.k[1] = sp.v[1] = nullptr;
  sp.k_stride_t[1] = sp.k_stride_h[1] = sp.v_stride_t[1] = sp.v_stride_h[1] = 0;
  if (p->cache) {
    sp.k[1] = reinterpret_cast<const __nv_bfloat16*>(p->cache->k_pool);
    sp.v[1] = reinterpret_cast<const __nv_bfloat16*>(p->cache->v_pool);
    sp.k_stride_t[1] = sp.v_stride_t[1] = (int64_t)p->cache->d.n_kv_heads * kHeadDim;
    sp.k_stride_h[1] = sp.v_stride_h[1] = kHeadDim;
  }
  sp.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  sp.o_stride_t = p->o_stride_t;
  sp.o_stride_h = p->o_stride_h;
  sp.o_stride_block = p->o_stride_block;
  sp.o_hpb = p->o_heads_per_block;
  sp.lse = p->lse;
  sp.n_q_heads = p->n_q_heads;
  sp.group = p->n_q_heads / p->n_kv_heads;
  sp.scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / sqrtf((float)kHeadDim);
  attn_simt_kernel<<<dim3(max_items, p->n_q_heads), 256, 0, stream>>>(sp);
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi
