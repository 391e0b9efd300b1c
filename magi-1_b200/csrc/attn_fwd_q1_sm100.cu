// Chunk-causal GQA attention forward for sm_100a, throughput form: ONE 128-row Q tile per CTA with a three-deep ring of
// score tiles, so that the tensor pipe, the MUFU and the TMA each work at their own rate instead of waiting on one
// another.  Same plan, same arguments and same arithmetic per element as attn_fwd_kernel (attn_fwd_sm100.cu), which
// replaces FullyParallelAttention.core_attention (inference/model/dit/dit_module.py:1023-1066).
//
// Why a second form: with two Q tiles per CTA (S0 S1 O0 O1 = 512 TMEM columns) each tile is a serial chain
//   S ready -> softmax (1.8 k cycles) -> P -> 16 UMMAs (1.2 k) -> S ready,
// two chains interleave, and the tensor pipe tops out near 2/3 busy.  Here TMEM holds S0 S1 S2 O (3 x 128 + 128 columns):
// Q K^T of tile j+2 is issued while the softmax of tiles j and j+1 is still running, so no unit waits for a chain; the
// bound becomes throughput - 128 x 128 exponentials per K/V tile on the MUFU (1.02 k cycles) against 16 UMMAs (1.05 k).
//
//   warp 0      TMA producer: Q once, then K/V tiles in CONSUMPTION order K0 K1 K2 V0 K3 V1 K4 ... (six 32 KB stages)
//   warp 1      issues S[j % 3] = Q K_j^T as soon as K_j is there and the score buffer is free (P V of tile j-3 done)
//   warp 2      issues O += P_j V_j as soon as the softmax has handed P_j over
//   warps 3-6   softmax of the EVEN K/V tiles  } a warp owns the 32 rows (TMEM lanes) of quarter warp % 4: both groups work
//   warps 7-10  softmax of the ODD K/V tiles   } on the same 128 rows, on alternate tiles, two tiles in flight
//
// The two groups share one running reference maximum per row.  In the common case nobody touches it: weights are taken
// against the reference already baked into O and l, and a row sum above 128 * 2^8 flags the rare tile whose scores outgrew
// it.  Tiles are FINALISED in order per row quarter (done_tile): a warp may hand its P over only after its partner has
// finalised the tile before, and a reference change (new maximum, O rescaled, epoch bumped) happens only at that point,
// when the P V of the previous tile has completed and the next one has not been issued.  A warp that finds the epoch
// changed under it rescales its row sum and redoes its tile from the scores still held in TMEM.
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "attn_epilogue.cuh"
#include "attn_bf16_common.cuh"

namespace magi {
using namespace ptx;

#ifdef MAGI_Q1_SPIN
#define Q1_WAIT mbar_wait_spin
#else
#define Q1_WAIT mbar_wait
#endif

int make_tile_map(magi_ctx* ctx, CUtensorMap* m, const void* base, int64_t stride_t, int64_t stride_h, int tokens,
                  int heads, int elem_bytes, const char* what);

constexpr int kQ1Stages = 6;
constexpr int kQ1Threads = 352;  // 11 warps: no idle warp, so that ptxas may use 184 registers per thread
struct SmemQ1 {
  static constexpr int kQ = 0;
  static constexpr int kRing = kTileBytes;
  static constexpr int kBar = kRing + kQ1Stages * kTileBytes;
  // barriers: q_full, kv_full[6], kv_empty[6], s_full[3], p_full[3], s_free[3], o_full
  static constexpr int kNumBars = 1 + 2 * kQ1Stages + 10;
  static constexpr int kFlags = kBar + kNumBars * 8;  // int done_tile[4], epoch[4], tmem slot, abort flag (+ pad) = 64 B
  static constexpr int kMsh = kFlags + 64;            // float m_sh[128]
  static constexpr int kLsh = kMsh + 512;             // float l_sh[2][128]
  static constexpr int kTotal = kLsh + 1024;
  static constexpr int kDynamic = kTotal + 1024;      // slack to align the base to 1024 bytes
};
static_assert(SmemQ1::kDynamic <= 232448, "shared memory per CTA");

// Walks the K/V tiles of a work item in order: segment by segment, 128 tokens at a time.
struct TileCursor {
  const Segment* segs;
  int sg_i, sg_end, t0;
  Segment sg;
  __device__ __forceinline__ TileCursor(const Segment* s, int begin, int end) : segs(s), sg_i(begin), sg_end(end), t0(0) {
    sg = segs[begin];
  }
  __device__ __forceinline__ int row() const { return sg.row0 + t0; }
  __device__ __forceinline__ int src() const { return sg.src; }
  __device__ __forceinline__ int valid() const { return min(kTileN, sg.len - t0); }
  __device__ __forceinline__ void next() {
    t0 += kTileN;
    if (t0 >= sg.len) {
      t0 = 0;
      if (++sg_i < sg_end) sg = segs[sg_i];
    }
  }
};

// Position of K_j / V_j in the producer's fill sequence K0 K1 K2 V0 K3 V1 K4 V2 ... (fewer leading K tiles if n < 3).
__device__ __forceinline__ int fill_of_k(int j) { return j < 3 ? j : 2 * j - 2; }
__device__ __forceinline__ int fill_of_v(int j, int n) { return min(n, j + 3) + j; }

// Bounded spin on the (done tile, epoch) word of a row quarter until the partner has finalised tile `want`; returns the
// word, or -1 after giving up (like mbar_wait).  Volatile reads of shared memory that another warp of this CTA advances.
__device__ __forceinline__ long long state_wait_done(volatile long long* st, int want, volatile int* abort_flag) {
  long long v = *st;
  if ((int)(uint32_t)v >= want) return v;
  const long long t0 = clock64();
  while ((int)(uint32_t)(v = *st) < want) {
    if (*abort_flag) return -1;
    if (clock64() - t0 > 1000000000LL) {
      *abort_flag = 1;
      return -1;
    }
  }
  return v;
}

__global__ void __launch_bounds__(kQ1Threads, 1)
attn_fwd_q1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                   const __grid_constant__ CUtensorMap tm_vc, const AttnKernelParams p) {
  using L = SmemQ1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  PlanView pv = plan_view(const_cast<void*>(p.plan));
  // two CTAs per work item of the plan (an item is up to 256 q rows): this one takes rows [128 * half, +128)
  const int item = blockIdx.x >> 1, half = blockIdx.x & 1;
  if (item >= pv.hdr->n_items || pv.hdr->status != 0) return;
  WorkItem it = pv.items[item];
  it.q_row0 += half * kTileM;
  it.q_rows = min(kTileM, it.q_rows - half * kTileM);
  if (it.q_rows <= 0) return;
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
  uint64_t* kv_empty = kv_full + kQ1Stages;
  uint64_t* s_full = kv_empty + kQ1Stages;
  uint64_t* p_full = s_full + 3;
  uint64_t* s_free = p_full + 3;
  uint64_t* o_full = s_free + 3;
  // per row quarter one 8-byte word: low half = last finalised tile, high half = epoch (number of reference changes); a
  // reader takes both with one load
  volatile long long* state = reinterpret_cast<volatile long long*>(smem + L::kFlags);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kFlags + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kFlags + 36);
  // per row quarter: the tile whose exponentials may run next.  The two warps that share a sub-partition's MUFU (same
  // quarter, the two groups) take turns on it: run side by side they each get half of it and both take twice as long,
  // run one after the other the MUFU is busy all the time and each warp's remaining work hides behind the other's turn.
  volatile int* mufu_turn = reinterpret_cast<volatile int*>(smem + L::kFlags + 40);
  volatile float* m_sh = reinterpret_cast<volatile float*>(smem + L::kMsh);          // [128] shared row reference
  volatile float* l_sh = reinterpret_cast<volatile float*>(smem + L::kLsh);          // [2][128] row sums of the two groups

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kQ1Stages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < 3; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4);  // one arrival per softmax warp of the group that owns the tile
      mbar_init(&s_free[b], 1);
    }
    mbar_init(o_full, 1);
    for (int q = 0; q < 4; ++q) {
      state[q] = 0x00000000ffffffffll;  // done = -1, epoch = 0
      mufu_turn[q] = 0;
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
      mbar_expect_tx(q_full, kTileBytes);
      for (int h = 0; h < 2; ++h) tma_load_3d(sQ + h * kHalfBytes, &tm_q, q_full, h * 64, head, it.q_row0);
      TileCursor ck(pv.segs, it.seg_begin, it.seg_end), cv(pv.segs, it.seg_begin, it.seg_end);
      int fill = 0;
      bool ok = true;
      auto load = [&](const TileCursor& c, bool is_v) {
        const int stage = fill % kQ1Stages, use = fill / kQ1Stages;
        if (use > 0) ok = mbar_wait(&kv_empty[stage], (use & 1) ^ 1, abort_flag);
        if (!ok) return;
        mbar_expect_tx(&kv_full[stage], kTileBytes);
        const CUtensorMap* m = is_v ? (c.src() ? &tm_vc : &tm_v) : (c.src() ? &tm_kc : &tm_k);
        tma_load_3d(ring + stage * kTileBytes, m, &kv_full[stage], 0, kv_head, c.row());
        tma_load_3d(ring + stage * kTileBytes + kHalfBytes, m, &kv_full[stage], 64, kv_head, c.row());
        ++fill;
      };
      int k_issued = 0;
      for (; k_issued < min(3, n_tiles) && ok; ++k_issued) {
        load(ck, false);
        ck.next();
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        load(cv, true);
        cv.next();
        if (ok && k_issued < n_tiles) {
          load(ck, false);
          ck.next();
          ++k_issued;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == 2) {
    // ------------------------------------------------------------------ UMMA issuers (one thread each)
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(kTileM, kTileN, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc(kTileM, kHeadDim, 1, 1, 0, 1);
      // high word shared by every operand descriptor here: SBO = 1024 B, version 1, 128-byte swizzle
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (kSw128 << 29);
      const uint32_t q_lo = (smem_u32(sQ) >> 4) | (1u << 16);                                   // K-major: LBO field = 1
      const uint32_t ring_k_lo = (smem_u32(ring) >> 4) | (1u << 16);                            // K tile, K-major
      const uint32_t ring_v_lo = (smem_u32(ring) >> 4) | ((uint32_t)(kHalfBytes >> 4) << 16);   // V tile, MN-major: LBO = half tile
      const uint32_t tO = tmem_base + 3 * kTileN;
      bool ok = true;
      if (warp == 1) {
        // S[j % 3] = Q K_j^T.  The score buffer is free once the P V of tile j-3, which read P from it, has completed.
        ok = Q1_WAIT(q_full, 0, abort_flag);
        for (int j = 0; j < n_tiles && ok; ++j) {
          const int f = fill_of_k(j), stage = f % kQ1Stages, b = j % 3;
          ok = Q1_WAIT(&kv_full[stage], (uint32_t)(f / kQ1Stages) & 1, abort_flag);
          if (ok && j >= 3) ok = Q1_WAIT(&s_free[b], (uint32_t)(j / 3 - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t b_lo = ring_k_lo + stage * (kTileBytes >> 4);
          const uint32_t tS = tmem_base + b * kTileN;
          umma_ss_f16_lh<0>(tS, q_lo, b_lo, desc_hi, idesc_qk);
#pragma unroll
          for (int k = 1; k < 8; ++k) {
            const uint32_t off = (k >> 2) * (kHalfBytes >> 4) + (k & 3) * 2;  // 16 k-elements = 32 bytes inside the swizzle row
            umma_ss_f16_lh<1>(tS, q_lo + off, b_lo + off, desc_hi, idesc_qk);
          }
          umma_commit(&s_full[b]);
          umma_commit(&kv_empty[stage]);
        }
      } else {
        // O += P_j V_j, P read from TMEM (the first 64 columns of S[j % 3])
        for (int j = 0; j < n_tiles && ok; ++j) {
          const int f = fill_of_v(j, n_tiles), stage = f % kQ1Stages, b = j % 3;
          ok = Q1_WAIT(&p_full[b], (uint32_t)(j / 3) & 1, abort_flag);
          if (ok) ok = Q1_WAIT(&kv_full[stage], (uint32_t)(f / kQ1Stages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t b_lo = ring_v_lo + stage * (kTileBytes >> 4);
          const uint32_t tS = tmem_base + b * kTileN;
          if (j == 0) umma_ts_f16_lh<0>(tO, tS, b_lo, desc_hi, idesc_pv);
          else umma_ts_f16_lh<1>(tO, tS, b_lo, desc_hi, idesc_pv);
#pragma unroll
          for (int k = 1; k < 8; ++k)  // 16 tokens of V = 2048 bytes; 16 bf16 of P = 8 TMEM columns
            umma_ts_f16_lh<1>(tO, tS + k * 8, b_lo + k * (2048 >> 4), desc_hi, idesc_pv);
          umma_commit(&s_free[b]);
          umma_commit(&kv_empty[stage]);
          if (j + 1 == n_tiles) umma_commit(o_full);
        }
      }
    }
    __syncwarp();
  }
  else {
    // ------------------------------------------------------------------ softmax / correction / epilogue (warps 3..10)
    const int g = (warp - 3) >> 2;          // group: tiles j with j % 2 == g
    const int quarter = warp & 3;           // TMEM lane quarter this warp may touch; its partner is the same quarter of the other group
    const int row = quarter * 32 + lane;    // row inside the Q tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + 3 * kTileN;
    const float sl2 = p.scale_log2;
    float m_used = -INFINITY;  // reference maximum this thread's l is relative to (raw score units)
    float l = 0.f;             // this group's share of the row sum
    int my_epoch = 0;
    bool ok = true;
    // The shared reference of this row changed (the partner, or this warp, published a new one): move l over to it.
    auto adopt = [&](int e) {
      __threadfence_block();
      const float m_new = m_sh[row];
      l *= ex2((m_used - m_new) * sl2);  // (-inf - m) gives 0: a group that has not seen a tile yet carries l = 0
      m_used = m_new;
      my_epoch = e;
    };
    // Waits until the partner has finalised tile `want`; returns the epoch it saw (-1: gave up).  Every lane reads the same
    // shared word with the same instruction, so the whole warp sees one value and stays converged.
    auto partner_done = [&](int want) {
      const long long v = state_wait_done(&state[quarter], want, abort_flag);
      return v == -1 ? -1 : (int)(v >> 32);
    };
    auto wait_turn = [&](int j) {
      if (mufu_turn[quarter] >= j) return true;
      const long long t_start = clock64();
      while (mufu_turn[quarter] < j) {
        if (*abort_flag) return false;
        if (clock64() - t_start > 1000000000LL) {
          *abort_flag = 1;
          return false;
        }
      }
      return true;
    };

    // this group's tiles j = g, g + 2, ...; (sg_i, t0) walk the segments in plain registers, two tiles at a time
    int sg_i = it.seg_begin, sg_len = pv.segs[sg_i].len, t0 = 0;
    auto step_tile = [&]() {
      t0 += kTileN;
      if (t0 >= sg_len) {
        t0 = 0;
        if (++sg_i < it.seg_end) sg_len = pv.segs[sg_i].len;
      }
    };
    if (g == 1) step_tile();
    int b = g;  // j % 3, kept as a running counter
    for (int j = g; j < n_tiles && ok; j += 2, step_tile(), step_tile(), b = (b + 2 >= 3) ? b - 1 : b + 2) {
      const int valid = min(kTileN, sg_len - t0);
      const uint32_t tS = tmem_base + lane_base + b * kTileN;
      ok = mbar_wait(&s_full[b], (uint32_t)(j / 3) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t s[kTileN];
      float alpha = 1.0f, rowsum;
      bool exact = (j == 0);
      if (j > 0) {
        if (j == 1) {  // the odd group's first tile: the reference is what the even group made of tile 0
          const int e = partner_done(0);
          if (e < 0) { ok = false; break; }
          adopt(e);
        }
        load_s_cols<0, kTileN>(tS, s, valid);
        ok = wait_turn(j);
        if (!ok) break;
        rowsum = softmax_fast(s, sl2, m_used);
        if (lane == 0) mufu_turn[quarter] = j + 1;  // the exponentials are issued: the partner's may follow
        const bool trip = __any_sync(0xffffffffu, !(rowsum <= kRedoRowSum));
        // finalisation happens in tile order: wait for the partner to be through with tile j-1 (it normally is, by a
        // thousand cycles), then see whether the reference moved while this tile was being computed
        const int e2 = partner_done(j - 1);
        if (e2 < 0) { ok = false; break; }
        if (e2 != my_epoch) {
          adopt(e2);
          exact = true;
        }
        exact = exact || trip;
      }
      if (exact) {
        // Exact path (tile 0, a tripped row sum, or a reference that moved under this tile): from the scores still in TMEM
        load_s_cols<0, kTileN>(tS, s, valid);
        rowsum = softmax_exact<0, kTileN>(s, sl2, m_used, alpha);  // may raise m_used; alpha = 2^(old - new) for such rows
        if (j == 0 && lane == 0) mufu_turn[quarter] = 1;
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
          // O holds tiles < j at the old reference; the P V of tile j-1 must have completed before it is rescaled, and the
          // P V of tile j cannot be issued before this warp hands P over
          ok = mbar_wait(&s_free[(j - 1) % 3], (uint32_t)((j - 1) / 3) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          rescale_o(tO, alpha);
        }
        if (j == 0 || __any_sync(0xffffffffu, alpha != 1.0f)) {  // publish the new reference of these rows
          m_sh[row] = m_used;
          __threadfence_block();
          __syncwarp();
          if (lane == 0) reinterpret_cast<volatile int*>(&state[quarter])[1] = my_epoch + 1;
          my_epoch += 1;
        }
      }
      tmem_st32(tS, s);
      tmem_st32(tS + 32, s + 32);
      l = l * alpha + rowsum;
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        reinterpret_cast<volatile int*>(&state[quarter])[0] = j;  // after the epoch store of the exact path, if any
        mbar_arrive(&p_full[b]);
      }
    }
    // ---- the two groups' row sums meet: both move to the final reference, then exchange through shared memory
    if (ok) {
      const int e = partner_done(n_tiles - 1);
      if (e < 0) ok = false;
      else if (e != my_epoch) adopt(e);
      if (ok) l_sh[g * kTileM + row] = l;
    }
    // the partner warp (same quarter, other group): a named barrier of the two warps; both reach it on every path
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    if (ok) ok = !*abort_flag;
    if (ok) ok = mbar_wait(o_full, 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      const float l_tot = l_sh[row] + l_sh[kTileM + row];
      const float inv = 1.0f / l_tot;
      // This warp stores columns [64 g, 64 g + 64) of its 32 rows, staged through the idle Q tile (4 KB per warp) so that
      // the global stores are whole 128-byte pieces of a row; 16-byte chunks XOR-swizzled by the row index.
      uint8_t* stage = sQ + (g * 4 + quarter) * 4096;
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t o[32];
        tmem_ld32(tO + g * 64 + c2 * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
          v.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
          v.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
          v.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * 128 + (((c2 * 4 + c) ^ (lane & 7)) << 4)) = v;
        }
      }
      __syncwarp();
      const int l8 = lane & 7, rsel = lane >> 3;
#pragma unroll 4
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + rsel;              // row inside this warp's 32
        const int r_item = quarter * 32 + rr;     // row inside the Q tile
        if (r_item < it.q_rows) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((l8 ^ (rr & 7)) << 4));
          __nv_bfloat16* dst_row = out_row(p, it.q_row0 + r_item, head);
          *reinterpret_cast<uint4*>(dst_row + g * 64 + l8 * 8) = v;
        }
      }
      if (p.lse && g == 0 && row < it.q_rows)
        p.lse[(int64_t)(it.q_row0 + row) * p.n_q_heads + head] = m_used * p.scale + logf(l_tot);
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
int attn_q1_init_device(magi_ctx* ctx) {
  MAGI_CUDA_OK(ctx, cudaFuncSetAttribute(attn_fwd_q1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemQ1::kDynamic));
  return MAGI_OK;
}

int launch_attn_bf16_q1(magi_ctx* ctx, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tkc,
                        const CUtensorMap& tvc, const AttnKernelParams& kp, int max_items, int n_q_heads, cudaStream_t stream) {
  dim3 grid(2 * max_items, n_q_heads, 1);
  attn_fwd_q1_kernel<<<grid, kQ1Threads, SmemQ1::kDynamic, stream>>>(tq, tk, tv, tkc, tvc, kp);
  MAGI_CUDA_OK(ctx, cudaGetLastError());
  return MAGI_OK;
}

}  // namespace magi
