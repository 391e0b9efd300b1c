// Device-side planner: turns (q_ranges, k_ranges, prefix page table) - all resident on the device, as the
// reference passes them (inference/model/dit/dit_module.py:1036-1037) - into the work list the attention
// kernels walk, without a host round trip.  Ranges are ordered longest-K first so the heavy CTAs start first.
//
// One block, one thread per q-range: (1) validate the range and count its K/V segments and tiles, (2) block-wide prefix
// sum of the segment counts, (3) write the segments, (4) rank the ranges by tile count (stable, descending), (5) prefix
// sum of the work items in that order and write them.  A call with a handful of ranges costs a few microseconds and a
// varlen batch of a thousand ranges a few tens (the earlier single-thread version needed 10 ms there).
#include "common.cuh"

namespace magi {

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

constexpr int kPlanThreads = kMaxRanges;  // 1024

// Walks the k intervals of q-range i, split at page boundaries (and, for FP8, at scale-chunk boundaries), and hands every
// segment to `emit`.  Returns 0 or a MAGI_E_* code; *tiles_out = K/V tiles of the range.
template <class Emit>
__device__ int walk_range(const PlanArgs& a, const PrefixTable& pt, int i, int* tiles_out, Emit emit) {
  const int C = pt.chunk_tokens;
  const int prefix_tokens = pt.n_prefix * C;
  const int kv_total = prefix_tokens + a.total_k;
  const int S = a.split_new_at;
  const int nbS = S > 0 ? ceil_div(S, kTileN) : 0;
  const int qs = a.q_ranges[2 * i], qe = a.q_ranges[2 * i + 1];
  if (qs < 0 || qe < qs || qe > a.total_q) return MAGI_E_RANGE;
  if (qe - qs > a.max_seqlen_q) return MAGI_E_RANGE;
  if (S > 0 && (qs % S) % kTileM != 0) return MAGI_E_RANGE;
  int kb = i, ke_ = i + 1;
  if (a.k_range_offsets) { kb = a.k_range_offsets[i]; ke_ = a.k_range_offsets[i + 1]; }
  if (kb < 0 || ke_ < kb || ke_ > a.n_k_ranges) return MAGI_E_RANGE;
  int tiles = 0;
  for (int r = kb; r < ke_; ++r) {
    const int ks = a.k_ranges[2 * r], ke = a.k_ranges[2 * r + 1];
    if (ks < 0 || ke < ks || ke > kv_total) return MAGI_E_RANGE;
    int t = ks;
    while (t < ke) {
      Segment sg;
      int end;
      if (t < prefix_tokens) {
        const int p = t / C;
        const int in_page = t - p * C;
        end = min(ke, (p + 1) * C);
        sg.src = 1;
        sg.row0 = pt.row0[p] + in_page;
        sg.blk0 = pt.blk0[p] + in_page / kTileN;
        if (S > 0 && in_page % kTileN != 0) return MAGI_E_RANGE;
      } else {
        const int tn = t - prefix_tokens;
        end = ke;
        sg.src = 0;
        sg.row0 = tn;
        sg.blk0 = 0;
        if (S > 0) {
          const int c = tn / S, in_c = tn - c * S;
          end = min(ke, prefix_tokens + (c + 1) * S);
          sg.blk0 = c * nbS + in_c / kTileN;
          if (in_c % kTileN != 0) return MAGI_E_RANGE;
        }
      }
      sg.len = end - t;
      emit(sg);
      tiles += ceil_div(sg.len, kTileN);
      t = end;
    }
  }
  *tiles_out = tiles;
  return 0;
}

// Exclusive prefix sum over the block (kPlanThreads values, one per thread); returns the total in *total.
__device__ int block_exclusive_scan(int v, int* scratch, int* total) {
  const int t = threadIdx.x;
  scratch[t] = v;
  __syncthreads();
  for (int d = 1; d < kPlanThreads; d <<= 1) {
    const int add = t >= d ? scratch[t - d] : 0;
    __syncthreads();
    scratch[t] += add;
    __syncthreads();
  }
  const int incl = scratch[t];
  *total = scratch[kPlanThreads - 1];
  __syncthreads();
  return incl - v;
}

__global__ void __launch_bounds__(kPlanThreads, 1) plan_kernel(void* workspace, PlanArgs a, PrefixTable pt) {
  PlanView pv = plan_view(workspace);
  __shared__ int s_scan[kPlanThreads];
  __shared__ int s_tiles[kMaxRanges];
  __shared__ int s_seg_begin[kMaxRanges];
  __shared__ int s_seg_cnt[kMaxRanges];
  __shared__ short s_order[kMaxRanges];
  __shared__ int s_status;
  const int i = threadIdx.x;
  const bool live = i < a.n_ranges;
  if (i == 0) s_status = a.n_ranges > kMaxRanges ? MAGI_E_NOMEM : 0;
  __syncthreads();

  // (1) validate, count segments and tiles
  int n_seg = 0, tiles = 0;
  if (live && s_status == 0) {
    const int rc = walk_range(a, pt, i, &tiles, [&](const Segment&) { ++n_seg; });
    if (rc != 0) atomicMin(&s_status, rc);  // codes are negative: the most severe wins, any one is reported
  }
  if (live) {
    s_tiles[i] = tiles;
    s_seg_cnt[i] = n_seg;
  }
  __syncthreads();
  int status = s_status;

  // (2) where each range's segments start
  int total_segs = 0;
  const int seg_begin = block_exclusive_scan(live && status == 0 ? n_seg : 0, s_scan, &total_segs);
  if (status == 0 && total_segs > kMaxSegs) status = MAGI_E_NOMEM;

  int n_items = 0;
  if (status == 0) {
    // (3) write the segments
    if (live) {
      s_seg_begin[i] = seg_begin;
      int w = seg_begin, dummy;
      walk_range(a, pt, i, &dummy, [&](const Segment& sg) { pv.segs[w++] = sg; });
    }
    // (4) rank by K tiles, descending, ties in range order (what a stable sort gives)
    __syncthreads();
    if (live) {
      int rank = 0;
      const int mine = s_tiles[i];
      for (int j = 0; j < a.n_ranges; ++j) {
        const int tj = s_tiles[j];
        rank += (tj > mine) || (tj == mine && j < i);
      }
      s_order[rank] = (short)i;
    }
    __syncthreads();
    // (5) work items in that order: thread o handles the range at position o
    const int rows_per_item = kTileM * kTilesPerCta;
    int r = -1, qs = 0, qe = 0, my_items = 0;
    if (live) {
      r = s_order[i];
      qs = a.q_ranges[2 * r];
      qe = a.q_ranges[2 * r + 1];
      my_items = ceil_div(qe - qs, rows_per_item);
    }
    const int item_begin = block_exclusive_scan(my_items, s_scan, &n_items);
    if (n_items > kMaxItems) {
      status = MAGI_E_NOMEM;
    } else if (live) {
      const int S = a.split_new_at;
      const int nbS = S > 0 ? ceil_div(S, kTileN) : 0;
      int w = item_begin;
      for (int q0 = qs; q0 < qe; q0 += rows_per_item) {
        WorkItem it;
        it.q_row0 = q0;
        it.q_rows = min(rows_per_item, qe - q0);
        it.seg_begin = s_seg_begin[r];
        it.seg_end = s_seg_begin[r] + s_seg_cnt[r];
        it.n_tiles = s_tiles[r];
        it.q_blk0 = S > 0 ? (q0 / S) * nbS + (q0 % S) / kTileM : 0;
        it.pad0 = it.pad1 = 0;
        pv.items[w++] = it;
      }
    }
  }
  if (i == 0) {
    if (status != 0) {
      n_items = 0;
      pv.hdr->status = status;
    }
    pv.hdr->n_items = n_items;
    pv.hdr->n_segs = status == 0 ? total_segs : 0;
  }
}

void launch_plan(void* workspace, const PlanArgs& a, const PrefixTable& pt, cudaStream_t stream) {
  plan_kernel<<<1, kPlanThreads, 0, stream>>>(workspace, a, pt);
}

}  // namespace magi
