// Chunk-causal GQA attention forward for sm_100a: TMA-fed shared-memory tiles, tcgen05 UMMA with TMEM
// accumulators, warp-level online softmax.  Replaces the flex_attention / flash_attn_func dispatch of
// FullyParallelAttention.core_attention (inference/model/dit/dit_module.py:1023-1066).
//
// One CTA = one work item of the plan (up to 256 q rows of one range, one q head) and walks every K/V tile
// of the range's segments; tiles that the block mask excludes are never in the list.
//
//   warp 0      TMA producer: Q tiles once, then K_j, V_j into a ring of 32 KB stages
//   warps 1, 2  UMMA issuers (one thread each, one per Q tile x = 0,1): S_x = Q_x K_j^T, O_x += P_x V_j; they take turns
//   warps 4-7   softmax for Q tile 0   } thread t of a warpgroup owns row t: TMEM lane = row, so row max /
//   warps 8-11  softmax for Q tile 1   } row sum need no shuffles.  They also rescale O and store the output.
//
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512), fp32.  P (bf16) overwrites the first
// 64 columns of its S and is the A operand of the PV UMMA straight from TMEM (no shared-memory round trip).
// While warpgroup 0 does softmax on S0 the tensor pipe runs the UMMAs of tile 1, and vice versa.
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>


#include "common.cuh"
#include "ptx_sm100.cuh"
#include "attn_epilogue.cuh"
#include "attn_bf16_common.cuh"

namespace magi {
using namespace ptx;

// Shared memory: Q (2 tiles, 64 KB) + a ring of 5 K/V stages (160 KB): K_j and V_j alternate through the ring, so the
// producer runs 2.5 K/V tile pairs ahead of the UMMAs.  (With 4 stages the TMA round trip was exposed: ~1000 of the
// ~4100 cycles per K/V tile were the UMMA issuer waiting for data.)
struct SmemLayout {
  static constexpr int kStages = 5;
  static constexpr int kQ = 0;
  static constexpr int kRing = kQ + kTilesPerCta * kTileBytes;
  static constexpr int kBar = kRing + kStages * kTileBytes;
  // barriers: q_full, kv_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2], turn[2]
  static constexpr int kNumBars = 1 + 2 * kStages + 8;
  static constexpr int kMisc = kBar + kNumBars * 8;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack to align the base to 1024 bytes
};

// K-major operand tile [128 rows x 128 k], stored as two [128 x 64] halves, 128-byte swizzle:
// descriptor of the 16-element k-slice `k` (0..7).
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile_saddr, int k) {
  return umma_smem_desc(tile_saddr + (k >> 2) * kHalfBytes + (k & 3) * 32, 16, 1024, kSw128);
}
// MN-major operand tile (V: [128 tokens x 128 d] as two [128 x 64] halves): k-slice = 16 tokens.
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile_saddr, int k) {
  return umma_smem_desc(tile_saddr + k * 2048, kHalfBytes, 1024, kSw128);
}

// kDualIssuer: warps 1 and 2 each issue the UMMAs of one Q tile.  One thread issuing everything is the bottleneck of
// the single-issuer form (a device timeline shows it 100 % busy: ~75 cycles per UMMA plus the barrier waits, fences and
// commits around each batch, while the softmax warps wait for S half of the time).  Two threads overlap one tile's
// waits and commits with the other tile's UMMA stream.  They pass a token (the `turn` barriers) so that the two tiles'
// batches never interleave on the tensor pipe: interleaved batches complete together, which locks the two softmax
// warpgroups in phase - both on the MUFU at once, then both waiting - and costs a third of the throughput.
template <bool kDualIssuer>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                const __grid_constant__ CUtensorMap tm_vc, const AttnKernelParams p) {
  using L = SmemLayout;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  PlanView pv = plan_view(const_cast<void*>(p.plan));
  // a planner error or an earlier CTA's timeout stops the whole grid
  if ((int)blockIdx.x >= pv.hdr->n_items || pv.hdr->status != 0) return;
  const WorkItem it = pv.items[blockIdx.x];
  const int head = blockIdx.y;
  const int kv_head = head / p.group;
  const int n_tiles = it.n_tiles;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (n_tiles == 0) {  // a q-range with no keys: zeros (lse = -inf), stored wherever the rows live (local or peer)
    zero_fill_item(p, it, head);
    return;
  }

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + kStages;
  uint64_t* s_full = kv_empty + kStages;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint64_t* turn = o_full + 2;      // kDualIssuer: turn[x] = issuer x may put its next batch on the tensor pipe
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], kDualIssuer ? 2 : 1);  // one commit per issuing thread that read the stage
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x], 4);  // one arrival per softmax warp: arrivals on one mbarrier serialise
      mbar_init(&o_full[x], 1);
      mbar_init(&turn[x], 1);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_expect_tx(q_full, kTilesPerCta * kTileBytes);
      for (int x = 0; x < kTilesPerCta; ++x)
        for (int h = 0; h < 2; ++h)
          tma_load_3d(sQ + x * kTileBytes + h * kHalfBytes, &tm_q, q_full, h * 64, head, it.q_row0 + x * kTileM);
      int fill = 0;
      bool ok = true;
      for (int sg_i = it.seg_begin; sg_i < it.seg_end && ok; ++sg_i) {
        const Segment sg = pv.segs[sg_i];
        const CUtensorMap* mk = sg.src ? &tm_kc : &tm_k;
        const CUtensorMap* mv = sg.src ? &tm_vc : &tm_v;
        for (int t0 = 0; t0 < sg.len && ok; t0 += kTileN) {
          for (int kv = 0; kv < 2; ++kv, ++fill) {
            const int stage = fill % kStages;
            const int use = fill / kStages;
            if (use > 0) ok = mbar_wait(&kv_empty[stage], (use & 1) ^ 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(&kv_full[stage], kTileBytes);
            const CUtensorMap* m = kv ? mv : mk;
            tma_load_3d(ring + stage * kTileBytes, m, &kv_full[stage], 0, kv_head, sg.row0 + t0);
            tma_load_3d(ring + stage * kTileBytes + kHalfBytes, m, &kv_full[stage], 64, kv_head, sg.row0 + t0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || (kDualIssuer && warp == 2)) {
    // ------------------------------------------------------------------ UMMA issuer (one thread)
    // Order per K/V tile j:  PV_0(j), QK_0(j+1), PV_1(j), QK_1(j+1): while the tensor pipe works for one Q tile the
    // other tile's warpgroup does its softmax.  The loop is kept to a few instructions per UMMA (a single thread
    // shares its scheduler with two softmax warps): descriptors are (lo, hi) halves advanced by 32-bit adds,
    // accumulate flags are compile-time, ring stage / parity are running counters.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(kTileM, kTileN, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(kTileM, kHeadDim, 1, 1, 0, 1);
      // high word shared by every operand descriptor here: SBO = 1024 B, version 1, 128-byte swizzle
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (kSw128 << 29);
      const uint32_t q_lo = (smem_u32(sQ) >> 4) | (1u << 16);                                   // K-major: LBO field = 1
      const uint32_t ring_k_lo = (smem_u32(ring) >> 4) | (1u << 16);                            // K tile, K-major
      const uint32_t ring_v_lo = (smem_u32(ring) >> 4) | ((uint32_t)(kHalfBytes >> 4) << 16);   // V tile, MN-major: LBO = half tile
      auto issue_qk = [&](int x, int stage) {
        const uint32_t a_lo = q_lo + x * (kTileBytes >> 4), b_lo = ring_k_lo + stage * (kTileBytes >> 4);
        const uint32_t tS = tmem_base + x * kTileN;
        umma_ss_f16_lh<0>(tS, a_lo, b_lo, desc_hi, idesc_qk);
#pragma unroll
        for (int k = 1; k < 8; ++k) {
          const uint32_t off = (k >> 2) * (kHalfBytes >> 4) + (k & 3) * 2;  // 16 k-elements = 32 bytes inside the swizzle row
          umma_ss_f16_lh<1>(tS, a_lo + off, b_lo + off, desc_hi, idesc_qk);
        }
      };
      auto issue_pv = [&](int x, int stage, bool first) {
        const uint32_t b_lo = ring_v_lo + stage * (kTileBytes >> 4);
        const uint32_t tS = tmem_base + x * kTileN, tO = tmem_base + 2 * kTileN + x * kHeadDim;
        if (first) umma_ts_f16_lh<0>(tO, tS, b_lo, desc_hi, idesc_pv);
        else umma_ts_f16_lh<1>(tO, tS, b_lo, desc_hi, idesc_pv);
#pragma unroll
        for (int k = 1; k < 8; ++k)  // 16 tokens of V = 2048 bytes; 16 bf16 of P = 8 TMEM columns
          umma_ts_f16_lh<1>(tO, tS + k * 8, b_lo + k * (2048 >> 4), desc_hi, idesc_pv);
      };
      int stage = 0;        // ring stage of the next tile to consume (K_0 first)
      uint32_t parity = 0;  // its "full" parity
      auto advance = [&]() {
        if (++stage == kStages) { stage = 0; parity ^= 1; }
      };
      // tiles this thread issues for: both (single issuer) or its own
      const int x_lo = kDualIssuer ? warp - 1 : 0, x_hi = kDualIssuer ? warp : 2;
      bool ok = mbar_wait(q_full, 0, abort_flag);
      ok = ok && mbar_wait(&kv_full[stage], parity, abort_flag);
      if (kDualIssuer && ok && x_lo == 1) ok = mbar_wait(&turn[1], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        for (int x = x_lo; x < x_hi; ++x) {
          issue_qk(x, stage);
          if (kDualIssuer) mbar_arrive(&turn[1 - x]);
          umma_commit(&s_full[x]);
        }
        umma_commit(&kv_empty[stage]);
        advance();
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more = j + 1 < n_tiles;
        const int v_stage = stage;
        ok = mbar_wait(&kv_full[stage], parity, abort_flag);  // V_j
        advance();
        const int k_stage = stage;
        if (ok && more) ok = mbar_wait(&kv_full[stage], parity, abort_flag);  // K_{j+1}
        if (more) advance();
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (kDualIssuer && x != x_lo) continue;
          if (!ok) break;
          // the token first: turn[0] completes a phase after the other thread's batch j-1 (and once in the prologue),
          // turn[1] after this tile-0 thread's batch j
          if (kDualIssuer) ok = mbar_wait(&turn[x], (uint32_t)(j + x) & 1, abort_flag);
          if (!ok) break;
          ok = mbar_wait(&p_full[x], j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(x, v_stage, j == 0);
          if constexpr (kDualIssuer) {
            if (more) issue_qk(x, k_stage);
            mbar_arrive(&turn[1 - x]);  // the batch is on the pipe: the other tile's may follow
            if (more) umma_commit(&s_full[x]);
            else umma_commit(&o_full[x]);
            umma_commit(&kv_empty[v_stage]);
            if (more) umma_commit(&kv_empty[k_stage]);
          } else {
            if (!more) umma_commit(&o_full[x]);  // only the epilogue waits for O (a later S_x implies the earlier PV_x)
            if (x == 1) umma_commit(&kv_empty[v_stage]);
            if (more) {
              issue_qk(x, k_stage);
              umma_commit(&s_full[x]);
              if (x == 1) umma_commit(&kv_empty[k_stage]);
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int x = (warp - 4) >> 2;          // Q tile of this warpgroup
    const int quarter = warp & 3;           // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;    // row inside the Q tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + x * kTileN;
    const uint32_t tO = tmem_base + lane_base + 2 * kTileN + x * kHeadDim;
    const float sl2 = p.scale_log2;
    float m_used = -INFINITY;  // reference maximum currently baked into O and l (raw score units)
    float l = 0.f;
    int j = 0;
    bool ok = true;
    for (int sg_i = it.seg_begin; sg_i < it.seg_end && ok; ++sg_i) {
      const Segment sg = pv.segs[sg_i];
      for (int t0 = 0; t0 < sg.len && ok; t0 += kTileN, ++j) {
        const int valid = min(kTileN, sg.len - t0);
        ok = mbar_wait(&s_full[x], j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        // S_x(j) complete implies PV_x(j-1) complete (same issuing thread, in order), so O_x may be rescaled here.
        uint32_t s[kTileN];
        load_s_cols<0, kTileN>(tS, s, valid);
        float alpha = 1.0f, rowsum = 0.f;
        bool redo = (j == 0);
        if (j > 0) {
          rowsum = softmax_fast(s, sl2, m_used);
          redo = __any_sync(0xffffffffu, !(rowsum <= kRedoRowSum));
          if (redo) load_s_cols<0, kTileN>(tS, s, valid);
        }
        if (redo) rowsum = softmax_exact<0, kTileN>(s, sl2, m_used, alpha);
        tmem_st32(tS, s);
        tmem_st32(tS + 32, s + 32);
        if (redo && j > 0) rescale_o(tO, alpha);
        l = l * alpha + rowsum;
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
      // the warp's 32 rows go through the (now idle) shared memory of its own Q tile: see store_o_rows_staged
      store_o_rows_staged(p, it, head, x, quarter, lane, tO, inv, sQ + x * kTileBytes + quarter * (32 * 256));
      if (p.lse && valid_row)
        p.lse[(int64_t)(it.q_row0 + r_in_item) * p.n_q_heads + head] = m_used * p.scale + logf(l);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) pv.hdr->status = MAGI_E_TIMEOUT;
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// [tokens, heads, 128] view -> 3-D map (d, head, token), box = 64 x 1 x 128 rows, 128-byte swizzle.
int make_tile_map(magi_ctx* ctx, CUtensorMap* m, const void* base, int64_t stride_t, int64_t stride_h, int tokens,
                  int heads, int elem_bytes, const char* what) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return set_err(ctx, MAGI_E_CUDA, "cuTensorMapEncodeTiled entry point not found");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((stride_t * elem_bytes) & 15) || ((stride_h * elem_bytes) & 15))
    return set_err(ctx, MAGI_E_ALIGN, "%s: base must be 16-byte aligned and strides multiples of 16 bytes", what);
  cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)(stride_h * elem_bytes), (cuuint64_t)(stride_t * elem_bytes)};
  cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), 1, (cuuint32_t)kTileN};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_err(ctx, MAGI_E_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", what, (int)r);
  return MAGI_OK;
}

int attn_fp8_init_device(magi_ctx* ctx);
// Opt in to > 48 KB of dynamic shared memory; called once per context with its device current.
int attn_init_device(magi_ctx* ctx) {
  if (int rc = attn_fp8_init_device(ctx)) return rc;
  MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::kDynamic));
  MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout::kDynamic));
  return MAGI_OK;
}

int launch_attn_bf16(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream) {
  CUtensorMap tq, tk, tv, tkc, tvc;
  int rc;
  if ((rc = make_tile_map(ctx, &tq, p->q, p->q_stride_t, p->q_stride_h, p->total_q, p->n_q_heads, 2, "q"))) return rc;
  const bool has_new = p->total_k > 0;
  const bool has_cache = p->cache && p->n_prefix_chunks > 0;
  if (has_new) {
    if ((rc = make_tile_map(ctx, &tk, p->k, p->k_stride_t, p->k_stride_h, p->total_k, p->n_kv_heads, 2, "k"))) return rc;
    if ((rc = make_tile_map(ctx, &tv, p->v, p->v_stride_t, p->v_stride_h, p->total_k, p->n_kv_heads, 2, "v"))) return rc;
  }
  if (has_cache) {
    const magi_kv_cache* c = p->cache;
    const int64_t st = (int64_t)c->d.n_kv_heads * kHeadDim;
    const int rows = c->n_slots * c->page_cap;
    if ((rc = make_tile_map(ctx, &tkc, c->k_pool, st, kHeadDim, rows, c->d.n_kv_heads, 2, "k cache"))) return rc;
    if ((rc = make_tile_map(ctx, &tvc, c->v_pool, st, kHeadDim, rows, c->d.n_kv_heads, 2, "v cache"))) return rc;
  }
  if (!has_new && !has_cache) return set_err(ctx, MAGI_E_BADARG, "no keys: total_k == 0 and no prefix");
  if (!has_new) { tk = tkc; tv = tvc; }
  if (!has_cache) { tkc = tk; tvc = tv; }

  AttnKernelParams kp;
  kp.plan = ctx->workspace;
  kp.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  kp.o_stride_t = p->o_stride_t;
  kp.o_stride_h = p->o_stride_h;
  kp.o_stride_block = p->o_stride_block;
  kp.o_hpb = p->o_heads_per_block;
  kp.lse = p->lse;
  kp.n_q_heads = p->n_q_heads;
  kp.group = p->n_q_heads / p->n_kv_heads;
  kp.scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / sqrtf((float)kHeadDim);
  kp.scale_log2 = kp.scale * 1.4426950408889634f;
  fill_peer_table(kp, p);

  dim3 grid(max_items, p->n_q_heads, 1);
  // MAGI_ATTN_SINGLE_ISSUER=1 selects the one-thread issuer (kept for A/B measurements; about 2 % slower)
  const char* v = getenv("MAGI_ATTN_SINGLE_ISSUER");
  if (v && v[0] == '1') attn_fwd_kernel<false><<<grid, kAttnThreads, SmemLayout::kDynamic, stream>>>(tq, tk, tv, tkc, tvc, kp);
  else attn_fwd_kernel<true><<<grid, kAttnThreads, SmemLayout::kDynamic, stream>>>(tq, tk, tv, tkc, tvc, kp);
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi
