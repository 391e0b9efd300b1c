// FP8 e4m3 twin of the chunk-causal attention forward (same plan, same roles, same TMEM map as attn_fwd_sm100.cu):
// Q, K, V are e4m3 with one fp32 scale per (128-token block, head); tiles coincide with scale blocks, so a tile's
// scales factor out of the UMMA:   S = (Q8 K8^T) * sq * sk_j.
// The V scale of tile j is folded into the softmax exponent as a bias, s' = S*scale*log2e + log2(sv_j), so that
// O_acc = sum_j P8_j V8_j needs no per-tile rescale:  O = O_acc / sum_j (rowsum(w_j) / sv_j),  w = 2^(s' - M).
// P is quantised to e4m3 per tile with a fixed power-of-two scale (16 w, w <= 2^4 under the lazy-rescale rule).
// Two-term mode (kTwoTerm, selected by passing q_lo): Q and P are each carried as two e4m3 terms (value + rounding
// residual), S = (Q8 + Q8lo) K8^T and O += (P8 + P8lo) V8, so only K and V contribute quantisation noise.  The extra
// UMMAs are hidden behind the softmax, which bounds the FP8 kernel.
// There is no reference counterpart (the reference's attention is bf16 only).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math.h>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "attn_epilogue.cuh"

namespace magi {
using namespace ptx;

int make_tile_map(magi_ctx* ctx, CUtensorMap* m, const void* base, int64_t stride_t, int64_t stride_h, int tokens,
                  int heads, int elem_bytes, const char* what);

constexpr int kThreads8 = 384;
constexpr int kTile8 = kTileN * kHeadDim;  // 16384 bytes: one 128x128 e4m3 tile = one 128-byte-swizzled TMA box
constexpr int kStages8 = 8;
constexpr float kLazyLog2 = 4.0f;          // rescale O only when the running maximum grows by more than 2^4
constexpr float kPScaleLog2 = 4.0f;        // P8 = e4m3(16 w) <= 256

struct Attn8Params {
  const void* plan;
  __nv_bfloat16* out;
  int64_t o_stride_t, o_stride_h;
  int64_t o_stride_block;  // head-block output layout (o_hpb > 0): see head_col()
  int o_hpb;
  float* lse;
  int n_q_heads, n_kv_heads, group;
  float scale_log2;
  const float* q_scale;     // [q blocks, Hq]
  const float* k_scale[2];  // [0] current [blocks, Hkv], [1] cache pool
  const float* v_scale[2];
  // fused output exchange, as in the bf16 kernel: see out_row()
  int n_peers;
  int head_offset;
  int peer_off[17];
  __nv_bfloat16* peer_out[16];
};

template <bool kTwoTerm>
struct Smem8 {
  static constexpr int kQ = 0;
  static constexpr int kQTerms = kTwoTerm ? 2 : 1;
  static constexpr int kRing = kQTerms * kTilesPerCta * kTile8;
  static constexpr int kBar = kRing + kStages8 * kTile8;
  static constexpr int kNumBars = 1 + 2 * kStages8 + 6;
  static constexpr int kMisc = kBar + kNumBars * 8;
  static constexpr int kDynamic = kMisc + 16 + 1024;
};

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

template <bool kTwoTerm>
__global__ void __launch_bounds__(kThreads8, 1)
attn_fwd_fp8_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_qlo,
                    const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                    const __grid_constant__ CUtensorMap tm_vc, const Attn8Params p) {
  using L = Smem8<kTwoTerm>;
  constexpr int kQTerms = L::kQTerms;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PlanView pv = plan_view(const_cast<void*>(p.plan));
  if ((int)blockIdx.x >= pv.hdr->n_items || pv.hdr->status != 0) return;
  const WorkItem it = pv.items[blockIdx.x];
  const int head = blockIdx.y, kv_head = head / p.group;
  const int n_tiles = it.n_tiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (n_tiles == 0) {  // a q-range with no keys: zeros (lse = -inf), stored wherever the rows live (local or peer)
    zero_fill_item(p, it, head);
    return;
  }

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + kStages8;
  uint64_t* s_full = kv_empty + kStages8;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages8; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x], 4);  // one arrival per softmax warp: arrivals on one mbarrier serialise
      mbar_init(&o_full[x], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  uint8_t* sQ = smem + L::kQ;
  uint8_t* ring = smem + L::kRing;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(q_full, kQTerms * kTilesPerCta * kTile8);
      for (int x = 0; x < kTilesPerCta; ++x) {
        tma_load_3d(sQ + x * kTile8, &tm_q, q_full, 0, head, it.q_row0 + x * kTileM);
        if constexpr (kTwoTerm) tma_load_3d(sQ + (kTilesPerCta + x) * kTile8, &tm_qlo, q_full, 0, head, it.q_row0 + x * kTileM);
      }
      int fill = 0;
      bool ok = true;
      for (int sg_i = it.seg_begin; sg_i < it.seg_end && ok; ++sg_i) {
        const Segment sg = pv.segs[sg_i];
        const CUtensorMap* mk = sg.src ? &tm_kc : &tm_k;
        const CUtensorMap* mv = sg.src ? &tm_vc : &tm_v;
        for (int t0 = 0; t0 < sg.len && ok; t0 += kTileN) {
          for (int kv = 0; kv < 2; ++kv, ++fill) {
            const int stage = fill % kStages8, use = fill / kStages8;
            if (use > 0) ok = mbar_wait(&kv_empty[stage], (use & 1) ^ 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(&kv_full[stage], kTile8);
            tma_load_3d(ring + stage * kTile8, kv ? mv : mk, &kv_full[stage], 0, kv_head, sg.row0 + t0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(kTileM, kTileN, 0, 0, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(kTileM, kHeadDim, 0, 0, 0, 1);
      const uint32_t sQ_addr = smem_u32(sQ), ring_addr = smem_u32(ring);
      auto stage_of = [&](int fill) { return fill % kStages8; };
      auto parity_of = [&](int fill) { return (uint32_t)((fill / kStages8) & 1); };
      auto issue_qk = [&](int x, int j) {
        const uint32_t b = ring_addr + stage_of(2 * j) * kTile8;
#pragma unroll
        for (int t = 0; t < kQTerms; ++t) {
          const uint32_t a = sQ_addr + (t * kTilesPerCta + x) * kTile8;
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 e4m3 (= 32 bytes) of the head dim per UMMA
            umma_ss_f8(tmem_base + x * kTileN, umma_smem_desc(a + k * 32, 16, 1024, 2), umma_smem_desc(b + k * 32, 16, 1024, 2),
                       idesc_qk, (t > 0) || (k > 0));
        }
      };
      auto issue_pv = [&](int x, int j) {
        const uint32_t b = ring_addr + stage_of(2 * j + 1) * kTile8;
        const uint32_t d = tmem_base + 2 * kTileN + x * kHeadDim;
#pragma unroll
        for (int t = 0; t < kQTerms; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 tokens per UMMA: 4 groups of 8 rows of 128 bytes; P term t: columns 32t + 8k
            umma_ts_f8(d, tmem_base + x * kTileN + t * 32 + k * 8, umma_smem_desc(b + k * 4096, 16, 1024, 2), idesc_pv,
                       (j > 0) || (t > 0) || (k > 0));
      };
      bool ok = mbar_wait(q_full, 0, abort_flag);
      ok = ok && mbar_wait(&kv_full[stage_of(0)], parity_of(0), abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(0, 0);
        umma_commit(&s_full[0]);
        issue_qk(1, 0);
        umma_commit(&s_full[1]);
        umma_commit(&kv_empty[stage_of(0)]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more = j + 1 < n_tiles;
        ok = mbar_wait(&kv_full[stage_of(2 * j + 1)], parity_of(2 * j + 1), abort_flag);
        if (ok && more) ok = mbar_wait(&kv_full[stage_of(2 * j + 2)], parity_of(2 * j + 2), abort_flag);
        for (int x = 0; x < 2 && ok; ++x) {
          ok = mbar_wait(&p_full[x], j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(x, j);
          if (!more) umma_commit(&o_full[x]);  // only the epilogue waits for O
          if (x == 1) umma_commit(&kv_empty[stage_of(2 * j + 1)]);
          if (more) {
            issue_qk(x, j + 1);
            umma_commit(&s_full[x]);
            if (x == 1) umma_commit(&kv_empty[stage_of(2 * j + 2)]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int x = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + x * kTileN;
    const uint32_t tO = tmem_base + lane_base + 2 * kTileN + x * kHeadDim;
    // the second Q tile of a work item with at most 128 rows has no scale block of its own (for the last item of the last
    // chunk the index would be one row past the scale tensor): its rows are never stored, any finite scale will do
    const float sq = (x * kTileM < it.q_rows ? __ldg(p.q_scale + (int64_t)(it.q_blk0 + x) * p.n_q_heads + head) : 1.0f) * p.scale_log2;
    float m_used = -INFINITY;  // running reference maximum of s' = S*sq*sk*scale*log2e + log2(sv)
    float l = 0.f;             // sum_j rowsum(16 w_j) / sv_j
    int j = 0;
    bool ok = true;
    for (int sg_i = it.seg_begin; sg_i < it.seg_end && ok; ++sg_i) {
      const Segment sg = pv.segs[sg_i];
      for (int t0 = 0; t0 < sg.len && ok; t0 += kTileN, ++j) {
        const int valid = min(kTileN, sg.len - t0);
        const int64_t sidx = (int64_t)(sg.blk0 + t0 / kTileN) * p.n_kv_heads + kv_head;
        const float sk = __ldg(p.k_scale[sg.src] + sidx), sv = __ldg(p.v_scale[sg.src] + sidx);
        const float c1 = sq * sk, bias = log2f(sv);
        ok = mbar_wait(&s_full[x], j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t s[kTileN];
        tmem_ld32(tS, s);
        tmem_ld32(tS + 32, s + 32);
        tmem_ld32(tS + 64, s + 64);
        tmem_ld32(tS + 96, s + 96);
        tmem_wait_ld();
        if (valid < kTileN) {
#pragma unroll
          for (int c = 0; c < kTileN; ++c)
            if (c >= valid) s[c] = 0xff800000u;
        }
        float mxa[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) mxa[c] = __uint_as_float(s[c]);
#pragma unroll
        for (int c = 8; c < kTileN; ++c) mxa[c & 7] = fmaxf(mxa[c & 7], __uint_as_float(s[c]));
        const float mx = fmaxf(fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])), fmaxf(fmaxf(mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
        const float m_new = fmaxf(m_used, fmaf(mx, c1, bias));
        const bool need = (m_new - m_used) > kLazyLog2;
        const float m_cur = need ? m_new : m_used;
        const float alpha = need ? ex2(m_used - m_new) : 1.0f;
        const float neg = bias - m_cur + kPScaleLog2;
        float rs[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (!kTwoTerm) {
#pragma unroll
          for (int c = 0; c < kTileN; c += 4) {
            const float p0 = ex2(fmaf(__uint_as_float(s[c]), c1, neg));
            const float p1 = ex2(fmaf(__uint_as_float(s[c + 1]), c1, neg));
            const float p2 = ex2(fmaf(__uint_as_float(s[c + 2]), c1, neg));
            const float p3 = ex2(fmaf(__uint_as_float(s[c + 3]), c1, neg));
            rs[0] += p0;
            rs[1] += p1;
            rs[2] += p2;
            rs[3] += p3;
            s[c >> 2] = pack_e4m3x4(p0, p1, p2, p3);
          }
          tmem_st32(tS, s);  // 128 e4m3 = 32 columns
        } else {
          // value = head (mantissa cut to e4m3's 3 bits, exactly representable) + residual, both stored as e4m3
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              float pv[4], ph[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                pv[e] = ex2(fmaf(__uint_as_float(s[q8 * 32 + c4 * 4 + e]), c1, neg));
                rs[e] += pv[e];
                ph[e] = __uint_as_float(__float_as_uint(pv[e]) & 0xFFF00000u);
              }
              hi[c4] = pack_e4m3x4(ph[0], ph[1], ph[2], ph[3]);
              lo[c4] = pack_e4m3x4(pv[0] - ph[0], pv[1] - ph[1], pv[2] - ph[2], pv[3] - ph[3]);
            }
            tmem_st8(tS + q8 * 8, hi);
            tmem_st8(tS + 32 + q8 * 8, lo);
          }
        }
        if (j > 0) {
          // S_x(j) complete implies PV_x(j-1) complete (same issuing thread, in order), so O_x may be rescaled here
          if (__any_sync(0xffffffffu, need)) {
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
        }
        l = l * alpha + ((rs[0] + rs[2]) + (rs[1] + rs[3])) / sv;
        m_used = m_cur;
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[x]);
      }
    }
    if (ok) ok = mbar_wait(&o_full[x], 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      const int r_in_item = x * kTileM + row;
      const bool valid_row = r_in_item < it.q_rows;
      const float inv = 1.0f / l;
      // Staging memory for the row-wise stores: every K/V stage except the one holding the last V tile is idle by now
      // (o_full[x] follows, in the issuing thread's order, every UMMA that read an earlier stage, and the producer has
      // nothing left to load), so each of the eight softmax warps takes half a stage (8 KB) after that one.
      const int last_v_stage = (2 * n_tiles - 1) % kStages8;
      const int w8 = x * 4 + quarter;
      uint8_t* stage = ring + ((last_v_stage + 1 + (w8 >> 1)) % kStages8) * kTile8 + (w8 & 1) * 8192;
      store_o_rows_staged(p, it, head, x, quarter, lane, tO, inv, stage);
      if (p.lse && valid_row)
        p.lse[(int64_t)(it.q_row0 + r_in_item) * p.n_q_heads + head] = (m_used + log2f(l) - kPScaleLog2) * 0.6931471805599453f;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) pv.hdr->status = MAGI_E_TIMEOUT;
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

int attn_fp8_init_device(magi_ctx* ctx) {
  MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(attn_fwd_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem8<false>::kDynamic));
  MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(attn_fwd_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem8<true>::kDynamic));
  return MAGI_OK;
}

int launch_attn_fp8(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream) {
  CUtensorMap tq, tql, tk, tv, tkc, tvc;
  int rc;
  if ((rc = make_tile_map(ctx, &tq, p->q, p->q_stride_t, p->q_stride_h, p->total_q, p->n_q_heads, 1, "q (fp8)"))) return rc;
  tql = tq;
  if (p->q_lo && (rc = make_tile_map(ctx, &tql, p->q_lo, p->q_stride_t, p->q_stride_h, p->total_q, p->n_q_heads, 1, "q_lo (fp8)")))
    return rc;
  const bool has_new = p->total_k > 0;
  const bool has_cache = p->cache && p->n_prefix_chunks > 0;
  if (has_new) {
    if ((rc = make_tile_map(ctx, &tk, p->k, p->k_stride_t, p->k_stride_h, p->total_k, p->n_kv_heads, 1, "k (fp8)"))) return rc;
    if ((rc = make_tile_map(ctx, &tv, p->v, p->v_stride_t, p->v_stride_h, p->total_k, p->n_kv_heads, 1, "v (fp8)"))) return rc;
  }
  if (has_cache) {
    const magi_kv_cache* c = p->cache;
    const int64_t st = (int64_t)c->d.n_kv_heads * kHeadDim;
    const int rows = c->n_slots * c->page_cap;
    if ((rc = make_tile_map(ctx, &tkc, c->k_pool, st, kHeadDim, rows, c->d.n_kv_heads, 1, "k cache (fp8)"))) return rc;
    if ((rc = make_tile_map(ctx, &tvc, c->v_pool, st, kHeadDim, rows, c->d.n_kv_heads, 1, "v cache (fp8)"))) return rc;
  }
  if (!has_new && !has_cache) return set_err(ctx, MAGI_E_BADARG, "no keys: total_k == 0 and no prefix");
  if (!has_new) { tk = tkc; tv = tvc; }
  if (!has_cache) { tkc = tk; tvc = tv; }
  Attn8Params kp;
  kp.plan = ctx->workspace;
  kp.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  kp.o_stride_t = p->o_stride_t;
  kp.o_stride_h = p->o_stride_h;
  kp.o_stride_block = p->o_stride_block;
  kp.o_hpb = p->o_heads_per_block;
  kp.lse = p->lse;
  kp.n_q_heads = p->n_q_heads;
  kp.n_kv_heads = p->n_kv_heads;
  kp.group = p->n_q_heads / p->n_kv_heads;
  const float scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / sqrtf((float)kHeadDim);
  kp.scale_log2 = scale * 1.4426950408889634f;
  kp.q_scale = p->q_scale;
  kp.k_scale[0] = p->k_scale;
  kp.v_scale[0] = p->v_scale;
  kp.k_scale[1] = has_cache ? p->cache->k_scale : p->k_scale;
  kp.v_scale[1] = has_cache ? p->cache->v_scale : p->v_scale;
  if (!has_new) { kp.k_scale[0] = kp.k_scale[1]; kp.v_scale[0] = kp.v_scale[1]; }
  fill_peer_table(kp, p);
  const dim3 grid(max_items, p->n_q_heads);
  if (p->q_lo)
    attn_fwd_fp8_kernel<true><<<grid, kThreads8, Smem8<true>::kDynamic, stream>>>(tq, tql, tk, tv, tkc, tvc, kp);
  else
    attn_fwd_fp8_kernel<false><<<grid, kThreads8, Smem8<false>::kDynamic, stream>>>(tq, tql, tk, tv, tkc, tvc, kp);
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi
