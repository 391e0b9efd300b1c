// Q / K / V projection with the per-head prologue in the GEMM's epilogue, for sm_100a.
// Replaces, in one kernel for one, two or all three projections (get_qkv, :998-1003), FullyParallelAttention.get_q / get_k / get_v
// (inference/model/dit/dit_module.py:953-963, :970-980, :987-989):
//     y   = bf16( x @ W^T )                       linear_qkv.forward_q / forward_k / forward_v (:415-425), torch.nn.Linear, no bias
//     out = bf16( rope( layer_norm_1p( float(y) ) ) )   per (token, head) over the 128 channels of the head; V: out = y
// The reference writes y to HBM, reads it back as fp32, normalises, transposes, rotates, casts and rearranges.  Here a
// head is exactly one 128-column block of the GEMM's N dimension, and a TMEM lane holds one token's accumulator row: the
// thread that drains a lane has the whole head of that token in registers, so mean, variance, the rotary pair
// (c, c + rot_pairs) and the cast need no exchange between threads at all, and y never exists in HBM.  The accumulator
// is rounded to bf16 before the norm, as the reference's Linear rounds its output.
//
// GEMM: x [T, K] and W [H*128, K] are both K-major, so both operands come in by TMA (128-byte swizzle, 64 k-elements per
// stage) and go to tcgen05.mma straight from shared memory; two 256-column accumulators in TMEM, so the epilogue of a
// tile overlaps the main loop of the next.  Two forms:
//   pair  a cluster of two CTAs works on 256 tokens x 256 channels with tcgen05.mma.cta_group::2 (M = 256): each CTA
//         loads its own 128 tokens of x and only ITS HALF of the W tile (32 KB per stage instead of 48, six stages),
//         the tensor cores of the two SMs share the W halves, and each CTA drains its own 128 rows.  Every load goes
//         to the loading CTA's own shared memory only; the odd CTA's loads count their bytes on the even CTA's barrier,
//         and the issuer commits "stage free" and "accumulator ready" to each CTA's barrier in turn.
//   solo  one CTA, 128 tokens x 256 channels, tcgen05.mma.cta_group::1, four 48 KB stages: small problems.
//
//   warp 0      TMA producer (one thread): x and W k-blocks into a ring of stages
//   warp 1      UMMA issuer (one thread; in a pair the even CTA's)
//   warps 2-9   epilogue: warp w drains TMEM lane quarter w % 4; warps 2-5 take the tile's first head, 6-9 its second
// Persistent: cluster (or CTA) b takes tiles b, b + grid, ...; tiles are numbered with the channel block fastest, so the
// CTAs running at any time share a few row blocks of x and all of W through L2.  Every wait is bounded (MAGI_E_TIMEOUT).
#include <cuda_bf16.h>
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace magi {
using namespace ptx;

int make_tile_map(magi_ctx* ctx, CUtensorMap* m, const void* base, int64_t stride_t, int64_t stride_h, int tokens,
                  int heads, int elem_bytes, const char* what);

constexpr int kLpThreads = 320;
constexpr int kLpKBlock = 64;                                  // k-elements per stage: one 128-byte swizzle row
constexpr int kLpSlab = 128 * kLpKBlock * 2;                   // 128 rows x 128 bytes = 16 KB
constexpr int kLpTileN = 256;                                  // two heads

template <bool kPair>
struct SmemLp {
  static constexpr int kStageBytes = (kPair ? 2 : 3) * kLpSlab;  // x: one slab; W: one slab (this CTA's half) or two
  static constexpr int kStages = kPair ? 6 : 4;                  // 192 KB either way
  static constexpr int kRing = 0;
  static constexpr int kStore = kStages * kStageBytes;           // 8 epilogue warps x 4 KB: 32 rows x 64 channels bf16
  static constexpr int kBar = kStore + 8 * 4096;
  static constexpr int kNumBars = 2 * kStages + 4;               // full, empty, acc_full[2], acc_empty[2]
  static constexpr int kMisc = kBar + kNumBars * 8;              // tmem slot, abort flag
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;                 // slack to align the base to 1024 bytes
};
static_assert(SmemLp<false>::kDynamic <= 232448 && SmemLp<true>::kDynamic <= 232448, "shared memory per CTA");

constexpr int kLpMaxSegs = 4;  // q, qx, k, v: the four members of the reference's CustomLayerNormLinear

// One projection of a launch (Q, K or V): its own weight, norm parameters and destination.
struct LpSegment {
  int H;
  int norm_mode;   // -1: plain linear
  int rotate;      // rotary after the norm (the cross-attention query, qx, is normed but not rotated)
  int plain_odd;   // heads 1, 3, 5, ... are plain: a K|V-interleaved weight (k of head 0, v of head 0, k of head 1, ...)
  int tile_begin;  // first channel block (two heads) of this projection among the launch's channel blocks
  int heads_per_block;  // 0: no blocking
  int use_block_ptrs;
  const float* gamma;
  const float* beta;
  const float* w_scale;  // e4m3 operands: the accumulator is multiplied by x_scale[0] * w_scale[0] (null: 1)
  __nv_bfloat16* out;
  int64_t out_stride_t, out_stride_h, out_stride_block;
  __nv_bfloat16* out_blocks[16];
};

struct LinearPrologueKernelParams {
  int T, k_blocks, n_segs;
  float eps;
  const float* cos;
  const float* sin;
  const float* x_scale;
  int tiles_m, tiles_n;
  int* status;
  LpSegment seg[kLpMaxSegs];
};

// One head of one token: 128 fp32 accumulators in registers -> bf16 rounding of the linear's output -> norm -> rotary
// -> 64 packed bf16 pairs.  kRot = rotary pairs (channel c pairs with c + kRot, c < kRot), a compile-time constant so
// that every register index is static.
template <int kRot>
__device__ __forceinline__ void head_epilogue(float (&v)[kHeadDim], uint32_t (&o)[kHeadDim / 2], const LinearPrologueKernelParams& p,
                                              const LpSegment& sg, bool normed, int64_t token, bool row_valid, float acc_scale) {
#pragma unroll
  for (int c = 0; c < kHeadDim; ++c) v[c] = __bfloat162float(__float2bfloat16_rn(v[c] * acc_scale));
  if (normed) {
    float rstd;
    if (sg.norm_mode == MAGI_NORM_LAYERNORM_1P) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int c = 0; c < kHeadDim; c += 4) { s0 += v[c]; s1 += v[c + 1]; s2 += v[c + 2]; s3 += v[c + 3]; }
      const float mean = ((s0 + s1) + (s2 + s3)) * (1.f / kHeadDim);
      s0 = s1 = s2 = s3 = 0.f;
#pragma unroll
      for (int c = 0; c < kHeadDim; c += 4) {
        v[c] -= mean; v[c + 1] -= mean; v[c + 2] -= mean; v[c + 3] -= mean;
        s0 = fmaf(v[c], v[c], s0); s1 = fmaf(v[c + 1], v[c + 1], s1); s2 = fmaf(v[c + 2], v[c + 2], s2); s3 = fmaf(v[c + 3], v[c + 3], s3);
      }
      rstd = rsqrtf(((s0 + s1) + (s2 + s3)) * (1.f / kHeadDim) + p.eps);
      // gamma and beta: the same address in every lane (one broadcast transaction each, L1-resident)
      if (sg.beta) {
#pragma unroll
        for (int c = 0; c < kHeadDim; ++c) v[c] = v[c] * rstd * (__ldg(sg.gamma + c) + 1.0f) + __ldg(sg.beta + c);
      } else {
#pragma unroll
        for (int c = 0; c < kHeadDim; ++c) v[c] = v[c] * rstd * (__ldg(sg.gamma + c) + 1.0f);
      }
    } else {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int c = 0; c < kHeadDim; c += 4) {
        s0 = fmaf(v[c], v[c], s0); s1 = fmaf(v[c + 1], v[c + 1], s1); s2 = fmaf(v[c + 2], v[c + 2], s2); s3 = fmaf(v[c + 3], v[c + 3], s3);
      }
      rstd = rsqrtf(((s0 + s1) + (s2 + s3)) * (1.f / kHeadDim) + p.eps);
#pragma unroll
      for (int c = 0; c < kHeadDim; ++c) v[c] = v[c] * rstd * (__ldg(sg.gamma + c) + 1.0f);
    }
    if constexpr (kRot > 0) {
      if (row_valid && sg.rotate) {
        const float4* cs = reinterpret_cast<const float4*>(p.cos + token * kRot);
        const float4* sn = reinterpret_cast<const float4*>(p.sin + token * kRot);
#pragma unroll
        for (int c4 = 0; c4 < kRot / 4; ++c4) {
          const float4 c = __ldg(cs + c4), s = __ldg(sn + c4);
          const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float a = v[4 * c4 + i], b = v[4 * c4 + i + kRot];
            v[4 * c4 + i] = a * cc[i] - b * ss[i];
            v[4 * c4 + i + kRot] = b * cc[i] + a * ss[i];
          }
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kHeadDim / 2; ++c) o[c] = pack_bf16x2(v[2 * c], v[2 * c + 1]);
}


// One head (128 accumulator values per thread) of this warp's 32 rows: norm + rotary in registers, then the
// store, staged through 4 KB of shared memory per warp, 64 channels at a time, so that the global stores are whole
// 128-byte pieces of a row (eight lanes per row, four rows per instruction); 16-byte chunks XOR-swizzled by the row.
template <int kRot>
__device__ __forceinline__ void store_head(float (&v)[kHeadDim], const LinearPrologueKernelParams& p, const LpSegment& sg,
                                           uint8_t* stage_sh, int head, int row0, int lane, float acc_scale) {
  uint32_t o[kHeadDim / 2];
  head_epilogue<kRot>(v, o, p, sg, sg.norm_mode >= 0 && !(sg.plain_odd && (head & 1)), (int64_t)row0 + lane, row0 + lane < p.T, acc_scale);
  // destination of (token, head): block of heads, then the row inside it
  const int blk = sg.heads_per_block > 0 ? head / sg.heads_per_block : 0;
  const int hs = sg.heads_per_block > 0 ? head - blk * sg.heads_per_block : head;
  __nv_bfloat16* base = (sg.use_block_ptrs ? sg.out_blocks[blk] : sg.out + blk * sg.out_stride_block) + hs * sg.out_stride_h;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    __syncwarp();
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<uint4*>(stage_sh + lane * 128 + ((c ^ (lane & 7)) << 4)) =
          make_uint4(o[half * 32 + 4 * c], o[half * 32 + 4 * c + 1], o[half * 32 + 4 * c + 2], o[half * 32 + 4 * c + 3]);
    __syncwarp();
    const int l8 = lane & 7, rsel = lane >> 3;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rr = 4 * i + rsel;
      if (row0 + rr < p.T) {
        const uint4 val = *reinterpret_cast<const uint4*>(stage_sh + rr * 128 + ((l8 ^ (rr & 7)) << 4));
        *reinterpret_cast<uint4*>(base + (int64_t)(row0 + rr) * sg.out_stride_t + half * 64 + l8 * 8) = val;
      }
    }
  }
}

template <bool kPair, int kRot, bool kFp8>
__global__ void __launch_bounds__(kLpThreads, 1)
linear_prologue_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w0,
                       const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_w2,
                       const __grid_constant__ CUtensorMap tm_w3, const __grid_constant__ LinearPrologueKernelParams p) {
  using L = SmemLp<kPair>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* full = bars;                      // the stage is loaded (TMA transaction bytes; pair: both CTAs' stage, even CTA's barrier)
  uint64_t* empty = full + L::kStages;        // the UMMAs that read the stage have completed
  uint64_t* acc_full = empty + L::kStages;
  uint64_t* acc_empty = acc_full + 2;         // pair: the even CTA's barrier collects both CTAs' epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMisc + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0;  // 0: issues the UMMAs
  const int unit = kPair ? blockIdx.x >> 1 : blockIdx.x, n_units = kPair ? gridDim.x >> 1 : gridDim.x;
  constexpr int kTileRows = kPair ? 256 : 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kPair ? 16 : 8);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    // all 512 columns, by each CTA for itself: in a pair both CTAs then hold the same columns at the same address,
    // which is what a pair UMMA writes to (checked below)
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) {
    cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    if (threadIdx.x == 0 && ld_cluster_u32(mapa_u32(tmem_slot, rank ^ 1)) != *tmem_slot) *abort_flag = 1;
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles = p.tiles_m * p.tiles_n;
  uint8_t* ring = smem + L::kRing;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && !*abort_flag) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w0);
      if (p.n_segs > 1) tma_prefetch_desc(&tm_w1);
      if (p.n_segs > 2) tma_prefetch_desc(&tm_w2);
      if (p.n_segs > 3) tma_prefetch_desc(&tm_w3);
      int fill = 0;
      bool ok = true;
      const uint32_t full_0 = kPair ? mapa_u32(&full[0], 0) : 0;
      for (int tile = unit; tile < n_tiles && ok; tile += n_units) {
        const int row0 = (tile / p.tiles_n) * kTileRows + rank * 128;
        // which projection this channel block belongs to, and its first output channel inside that projection's weight
        const int nt = tile % p.tiles_n;
        int sgi = 0;
        for (int i = 1; i < p.n_segs; ++i) sgi = nt >= p.seg[i].tile_begin ? i : sgi;
        const CUtensorMap* tm_w = sgi == 0 ? &tm_w0 : sgi == 1 ? &tm_w1 : sgi == 2 ? &tm_w2 : &tm_w3;
        const int ch0 = (nt - p.seg[sgi].tile_begin) * kLpTileN + (kPair ? rank * 128 : 0);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++fill) {
          const int stage = fill % L::kStages, use = fill / L::kStages;
          // the stage is free once the UMMAs that read it have completed (in a pair the issuer commits to both CTAs)
          if (use > 0) ok = kPair ? mbar_wait_cluster(&empty[stage], (use & 1) ^ 1, abort_flag) : mbar_wait(&empty[stage], (use & 1) ^ 1, abort_flag);
          if (!ok) break;
          uint8_t* dst = ring + stage * L::kStageBytes;
          // x and W are seen as [rows, K / 128, 128]: a k-block is one 128-byte swizzle row per row of the operand, i.e.
          // 64 bf16 (the half kb & 1 of 128-column group kb >> 1) or 128 e4m3 (group kb)
          const int c0 = kFp8 ? 0 : (kb & 1) * kLpKBlock, c1 = kFp8 ? kb : kb >> 1;
          if constexpr (kPair) {
            // both CTAs' loads of a stage count on the EVEN CTA's barrier, which its producer arms for both
            if (rank == 0) mbar_expect_tx(&full[stage], 2 * L::kStageBytes);
            const uint32_t bar = rank == 0 ? smem_u32(&full[stage]) : full_0 + stage * 8;
            tma_load_3d_pair(dst, &tm_x, bar, c0, c1, row0);
            tma_load_3d_pair(dst + kLpSlab, tm_w, bar, c0, c1, ch0);
          } else {
            mbar_expect_tx(&full[stage], L::kStageBytes);
            tma_load_3d(dst, &tm_x, &full[stage], c0, c1, row0);
            tma_load_3d(dst + kLpSlab, tm_w, &full[stage], c0, c1, ch0);
            tma_load_3d(dst + 2 * kLpSlab, tm_w, &full[stage], c0, c1, ch0 + 128);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && !*abort_flag) {
      int fill = 0;
      bool ok = true;
      if (!(kPair && rank == 1)) {
        // ---------------------------------------------------------------- UMMA issuer
        constexpr uint32_t idesc = kFp8 ? umma_idesc(kTileRows, kLpTileN, 0, 0, 0, 0) : umma_idesc(kTileRows, kLpTileN, 1, 1, 0, 0);
        constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO = 1024 B, version 1, 128-byte swizzle
        const uint32_t ring_lo = (smem_u32(ring) >> 4) | (1u << 16);         // K-major: LBO field = 1
        const uint32_t empty_1 = kPair ? mapa_u32(&empty[0], 1) : 0, acc_full_1 = kPair ? mapa_u32(&acc_full[0], 1) : 0;
        int t_local = 0;
        for (int tile = unit; tile < n_tiles && ok; tile += n_units, ++t_local) {
          const int a = t_local & 1, a_use = t_local >> 1;
          if (a_use > 0) ok = kPair ? mbar_wait_cluster(&acc_empty[a], (a_use & 1) ^ 1, abort_flag) : mbar_wait(&acc_empty[a], (a_use & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d = tmem_base + a * kLpTileN;
          for (int kb = 0; kb < p.k_blocks; ++kb, ++fill) {
            const int stage = fill % L::kStages;
            const uint32_t par = (uint32_t)(fill / L::kStages) & 1;
            ok = kPair ? mbar_wait_cluster(&full[stage], par, abort_flag) : mbar_wait(&full[stage], par, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_lo = ring_lo + stage * (L::kStageBytes >> 4);
            const uint32_t b_lo = a_lo + (kLpSlab >> 4);
            // four instructions per k-block: 16 bf16 or 32 e4m3 k-elements = 32 bytes of the swizzle row each
            if constexpr (kPair) {
              if constexpr (kFp8) {
                if (kb == 0) umma_ss_f8_lh_pair<0>(d, a_lo, b_lo, desc_hi, idesc);
                else umma_ss_f8_lh_pair<1>(d, a_lo, b_lo, desc_hi, idesc);
#pragma unroll
                for (int k = 1; k < 4; ++k) umma_ss_f8_lh_pair<1>(d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
              } else {
                if (kb == 0) umma_ss_f16_lh_pair<0>(d, a_lo, b_lo, desc_hi, idesc);
                else umma_ss_f16_lh_pair<1>(d, a_lo, b_lo, desc_hi, idesc);
#pragma unroll
                for (int k = 1; k < 4; ++k) umma_ss_f16_lh_pair<1>(d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
              }
              umma_commit_pair(&empty[stage]);
              umma_commit_pair_at(empty_1 + stage * 8);
            } else {
              if constexpr (kFp8) {
                if (kb == 0) umma_ss_f8_lh<0>(d, a_lo, b_lo, desc_hi, idesc);
                else umma_ss_f8_lh<1>(d, a_lo, b_lo, desc_hi, idesc);
#pragma unroll
                for (int k = 1; k < 4; ++k) umma_ss_f8_lh<1>(d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
              } else {
                if (kb == 0) umma_ss_f16_lh<0>(d, a_lo, b_lo, desc_hi, idesc);
                else umma_ss_f16_lh<1>(d, a_lo, b_lo, desc_hi, idesc);
#pragma unroll
                for (int k = 1; k < 4; ++k) umma_ss_f16_lh<1>(d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc);
              }
              umma_commit(&empty[stage]);
            }
          }
          if (ok) {
            if constexpr (kPair) {
              umma_commit_pair(&acc_full[a]);
              umma_commit_pair_at(acc_full_1 + a * 8);
            } else {
              umma_commit(&acc_full[a]);
            }
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int ew = warp - 2;                 // 0..7
    const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
    const int hh = ew >> 2;                  // head of the tile this warp drains
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    uint8_t* stage_sh = smem + L::kStore + ew * 4096;
    const uint32_t acc_empty_0 = kPair ? mapa_u32(&acc_empty[0], 0) : 0;  // the issuer's barriers
    const float x_scale = p.x_scale ? __ldg(p.x_scale) : 1.0f;
    bool ok = !*abort_flag;
    int t_local = 0;
    for (int tile = unit; tile < n_tiles && ok; tile += n_units, ++t_local) {
      const int a = t_local & 1;
      const int row0 = (tile / p.tiles_n) * kTileRows + rank * 128 + quarter * 32;
      const int nt = tile % p.tiles_n;
      int sgi = 0;
      for (int i = 1; i < p.n_segs; ++i) sgi = nt >= p.seg[i].tile_begin ? i : sgi;
      const LpSegment& sg = p.seg[sgi];
      const int head = (nt - sg.tile_begin) * 2 + hh;  // head inside its projection
      ok = kPair ? mbar_wait_cluster(&acc_full[a], (uint32_t)(t_local >> 1) & 1, abort_flag) : mbar_wait(&acc_full[a], (uint32_t)(t_local >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      float v[kHeadDim];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tmem_ld32(tmem_base + lane_base + a * kLpTileN + hh * kHeadDim + c * 32, reinterpret_cast<uint32_t*>(v) + c * 32);
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {  // this warp is through with the accumulator
        if constexpr (kPair) mbar_arrive_cluster(acc_empty_0 + a * 8);
        else mbar_arrive(&acc_empty[a]);
      }
      if (head < sg.H)  // warp-uniform: an odd head count leaves half of the projection's last channel block empty
        store_head<kRot>(v, p, sg, stage_sh, head, row0, lane, x_scale * (sg.w_scale ? __ldg(sg.w_scale) : 1.0f));
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // neither CTA frees its columns or leaves while the other may still signal it
  if (*abort_flag && threadIdx.x == 0 && p.status) *p.status = MAGI_E_TIMEOUT;
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------- host side
template <bool kPair, int kRot, bool kFp8>
static int launch_lp(magi_ctx* ctx, const CUtensorMap& tx, const CUtensorMap* tw, const LinearPrologueKernelParams& k, cudaStream_t st) {
  static bool configured[64] = {};  // per device: opt in to > 48 KB of dynamic shared memory once
  if (ctx->device < 64 && !configured[ctx->device]) {
    MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(linear_prologue_kernel<kPair, kRot, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SmemLp<kPair>::kDynamic));
    configured[ctx->device] = true;
  }
  const int n_tiles = k.tiles_m * k.tiles_n;
  const int max_units = kPair ? ctx->sm_count / 2 : ctx->sm_count;
  const int units = n_tiles < max_units ? n_tiles : max_units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kPair ? 2 * units : units, 1, 1);
  cfg.blockDim = dim3(kLpThreads, 1, 1);
  cfg.dynamicSmemBytes = SmemLp<kPair>::kDynamic;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MAGI_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, linear_prologue_kernel<kPair, kRot, kFp8>, tx, tw[0], tw[1], tw[2], tw[3], k));
  return MAGI_OK;
}

template <bool kPair, bool kFp8>
static int launch_lp_rot(magi_ctx* ctx, int rot, const CUtensorMap& tx, const CUtensorMap* tw, const LinearPrologueKernelParams& k,
                         cudaStream_t st) {
  switch (rot) {
    case 0: return launch_lp<kPair, 0, kFp8>(ctx, tx, tw, k, st);
    case 32: return launch_lp<kPair, 32, kFp8>(ctx, tx, tw, k, st);
    case 48: return launch_lp<kPair, 48, kFp8>(ctx, tx, tw, k, st);
    case 64: return launch_lp<kPair, 64, kFp8>(ctx, tx, tw, k, st);
  }
  return set_err(ctx, MAGI_E_BADARG, "linear prologue: rot_pairs must be 0, 32, 48 or 64 (the reference uses 48)");
}

// Checks one projection's own fields and fills its segment.
static int fill_segment(magi_ctx* ctx, const magi_linear_prologue_params* p, LpSegment& sg) {
  if (!p->w || (!p->out && !p->out_block_ptrs) || p->H <= 0) return set_err(ctx, MAGI_E_BADARG, "linear prologue: null tensor or bad shape");
  const bool plain = p->norm_mode == MAGI_NORM_NONE;
  if (!plain && p->norm_mode != MAGI_NORM_LAYERNORM_1P && p->norm_mode != MAGI_NORM_RMSNORM_1P)
    return set_err(ctx, MAGI_E_BADARG, "linear prologue: unknown norm_mode %d", p->norm_mode);
  if (!plain && !p->gamma) return set_err(ctx, MAGI_E_BADARG, "linear prologue: gamma is required");
  if (p->out_block_ptrs) {
    if (p->heads_per_block <= 0 || p->H % p->heads_per_block || p->H / p->heads_per_block > 16)
      return set_err(ctx, MAGI_E_BADARG, "linear prologue: out_block_ptrs needs heads_per_block dividing H into at most 16 blocks");
    for (int b = 0; b < p->H / p->heads_per_block; ++b)
      if (!p->out_block_ptrs[b] || (reinterpret_cast<uintptr_t>(p->out_block_ptrs[b]) & 15))
        return set_err(ctx, MAGI_E_ALIGN, "linear prologue: out_block_ptrs[%d] is null or not 16-byte aligned", b);
  }
  if ((reinterpret_cast<uintptr_t>(p->out) & 15) || (p->out_stride_t & 7) || (p->out_stride_h & 7) || (p->out_stride_block & 7))
    return set_err(ctx, MAGI_E_ALIGN, "linear prologue: out must be 16-byte aligned and its strides multiples of 8 elements");
  sg.H = p->H;
  sg.norm_mode = plain ? -1 : p->norm_mode;
  sg.plain_odd = p->plain_odd_heads ? 1 : 0;
  sg.gamma = p->gamma;
  sg.beta = (!plain && p->norm_mode == MAGI_NORM_LAYERNORM_1P) ? p->beta : nullptr;
  sg.w_scale = p->dtype == MAGI_DTYPE_FP8_E4M3 ? p->w_scale : nullptr;
  sg.out = reinterpret_cast<__nv_bfloat16*>(p->out);
  sg.out_stride_t = p->out_stride_t;
  sg.out_stride_h = p->out_stride_h;
  sg.out_stride_block = p->out_stride_block;
  sg.heads_per_block = (p->heads_per_block > 0 && (p->heads_per_block < p->H || p->out_block_ptrs)) ? p->heads_per_block : 0;
  sg.use_block_ptrs = p->out_block_ptrs ? 1 : 0;
  for (int b = 0; b < 16; ++b)
    sg.out_blocks[b] = (p->out_block_ptrs && b < p->H / p->heads_per_block) ? reinterpret_cast<__nv_bfloat16*>(p->out_block_ptrs[b]) : nullptr;
  return MAGI_OK;
}

}  // namespace magi

extern "C" int magi_linear_qkv_norm_rope_fwd(magi_ctx* ctx, const magi_linear_prologue_params* segs, int n_segs, void* stream) {
  using namespace magi;
  if (!ctx) return MAGI_E_BADARG;
  if (!segs || n_segs < 1 || n_segs > kLpMaxSegs) return set_err(ctx, MAGI_E_BADARG, "linear prologue: 1 to %d projections per call", kLpMaxSegs);
  const magi_linear_prologue_params* p = &segs[0];
  for (int i = 0; i < n_segs; ++i)
    if (segs[i].struct_size != sizeof(magi_linear_prologue_params)) return set_err(ctx, MAGI_E_BADARG, "linear prologue: bad struct_size");
  if (!p->x || p->T < 0 || p->in_features <= 0) return set_err(ctx, MAGI_E_BADARG, "linear prologue: null tensor or bad shape");
  if (p->in_features % 128) return set_err(ctx, MAGI_E_BADARG, "linear prologue: in_features must be a multiple of 128");
  if (p->dtype != MAGI_DTYPE_BF16 && p->dtype != MAGI_DTYPE_FP8_E4M3) return set_err(ctx, MAGI_E_BADARG, "linear prologue: dtype is bf16 or e4m3");
  const bool fp8 = p->dtype == MAGI_DTYPE_FP8_E4M3;
  const int esz = fp8 ? 1 : 2;
  LinearPrologueKernelParams k = {};
  int rot = 0;
  for (int i = 0; i < n_segs; ++i) {
    const magi_linear_prologue_params* q = &segs[i];
    // the projections of one call share the input: x, its scale, the token count, the rotary table
    if (q->x != p->x || q->x_stride != p->x_stride || q->T != p->T || q->in_features != p->in_features || q->dtype != p->dtype ||
        q->x_scale != p->x_scale || q->eps != p->eps)
      return set_err(ctx, MAGI_E_BADARG, "linear prologue: projection %d does not share x, T, in_features, dtype, x_scale and eps with the first", i);
    if (int rc = fill_segment(ctx, q, k.seg[i])) return rc;
    k.seg[i].rotate = 0;
    if (q->norm_mode != MAGI_NORM_NONE && q->rot_pairs > 0) {
      if (!q->cos || !q->sin) return set_err(ctx, MAGI_E_BADARG, "linear prologue: cos/sin required");
      if ((reinterpret_cast<uintptr_t>(q->cos) & 15) || (reinterpret_cast<uintptr_t>(q->sin) & 15))
        return set_err(ctx, MAGI_E_ALIGN, "linear prologue: cos/sin must be 16-byte aligned");
      if (rot && (rot != q->rot_pairs || k.cos != q->cos || k.sin != q->sin))
        return set_err(ctx, MAGI_E_BADARG, "linear prologue: the rotated projections of one call share rot_pairs, cos and sin");
      rot = q->rot_pairs;
      k.cos = q->cos;
      k.sin = q->sin;
      k.seg[i].rotate = 1;
    }
    k.seg[i].tile_begin = k.tiles_n;
    k.tiles_n += (q->H + 1) / 2;
  }
  if (p->T == 0) return MAGI_OK;
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  CUtensorMap tx, tw[kLpMaxSegs];
  int rc = make_tile_map(ctx, &tx, p->x, p->x_stride, 128, p->T, p->in_features / 128, esz, "linear prologue x");
  for (int i = 0; i < kLpMaxSegs && !rc; ++i) {
    const magi_linear_prologue_params* q = &segs[i < n_segs ? i : 0];  // unused maps repeat the first
    rc = make_tile_map(ctx, &tw[i], q->w, q->w_stride, 128, q->H * kHeadDim, p->in_features / 128, esz, "linear prologue w");
  }
  if (!rc) {
    k.T = p->T;
    k.n_segs = n_segs;
    k.k_blocks = fp8 ? p->in_features / 128 : p->in_features / kLpKBlock;
    k.eps = p->eps;
    k.x_scale = fp8 ? p->x_scale : nullptr;
    k.status = reinterpret_cast<int*>(reinterpret_cast<char*>(ctx->workspace) + offsetof(PlanHeader, status));
    // CTA pairs unless the problem is too small to give every pair a 256-row tile; MAGI_LINEAR_FORM=solo|pair overrides
    // (kept for A/B measurements)
    const int64_t tiles256 = (int64_t)((p->T + 255) / 256) * k.tiles_n;
    const char* force = getenv("MAGI_LINEAR_FORM");
    const bool pair = force ? force[0] == 'p' : tiles256 >= ctx->sm_count / 2;
    k.tiles_m = pair ? (p->T + 255) / 256 : (p->T + 127) / 128;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (fp8) rc = pair ? launch_lp_rot<true, true>(ctx, rot, tx, tw, k, st) : launch_lp_rot<false, true>(ctx, rot, tx, tw, k, st);
    else rc = pair ? launch_lp_rot<true, false>(ctx, rot, tx, tw, k, st) : launch_lp_rot<false, false>(ctx, rot, tx, tw, k, st);
  }
  if (prev != ctx->device) cudaSetDevice(prev);
  return rc;
}

extern "C" int magi_linear_qk_norm_rope_fwd(magi_ctx* ctx, const magi_linear_prologue_params* p, void* stream) {
  return magi_linear_qkv_norm_rope_fwd(ctx, p, p ? 1 : 0, stream);
}
