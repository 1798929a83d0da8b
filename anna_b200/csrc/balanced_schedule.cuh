// Even-share schedule for a persistent split pass.
//
// The 16-token tiles of all (row, stream) pairs form one line in (row, stream-in-row, tile) order, where a "stream" is
// one (kv head, group of up to 8 query heads) of a row.  The grid is one resident wave and CTA c owns tiles
// [c * tpc, (c + 1) * tpc).  A CTA walks its range stream by stream and emits one split-K partial per stream it
// touches, so every CTA moves the same number of bytes whatever the mix of context lengths, and a long context costs
// one pipeline start per CTA instead of one per fixed-size chunk.  Every CTA recomputes the partition from the
// device-side lengths (a block-wide scan), so no host round trip is needed; the slot of each partial and the number
// of partials per stream (for the arrival counter of the fused merge) follow from the same arithmetic.
#pragma once

#include "common.cuh"

namespace anna {

constexpr int kBalancedMaxRows = 1024;
constexpr int kBalancedMinTiles = 4;   // per CTA: one tile per warp
constexpr int kBalancedTileTokens = 16;

// Block-wide exclusive scan of the tiles per row: s_prefix[b] = tiles (over all streams) of the rows before row b,
// s_prefix[batch] = all tiles.  Returns the largest number of tiles of any single stream.  Ends with a barrier.
// THREADS = blockDim.x (a multiple of 32); batch <= kBalancedMaxRows.
template <int THREADS>
__device__ __forceinline__ int balanced_scan(const int64_t* visible_lengths, int64_t max_len, int batch,
                                             int streams_per_row, int* s_prefix) {
  constexpr int kWarps = THREADS / 32;
  constexpr int kRowsPerThread = (kBalancedMaxRows + THREADS - 1) / THREADS;
  __shared__ int s_warp_sum[kWarps];
  __shared__ int s_warp_max[kWarps];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rpt = (batch + THREADS - 1) / THREADS;
  int local[kRowsPerThread];
  int sum = 0, mx = 0;
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const int b = threadIdx.x * rpt + i;
    int tiles = 0;
    if (i < rpt && b < batch) {
      int64_t len = visible_lengths ? visible_lengths[b] : max_len;
      len = max((int64_t)0, min(len, max_len));
      tiles = (int)((len + kBalancedTileTokens - 1) / kBalancedTileTokens);
    }
    local[i] = tiles;
    sum += tiles;
    mx = max(mx, tiles);
  }
  int incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  }
  if (lane == 31) s_warp_sum[warp] = incl;
  if (lane == 0) s_warp_max[warp] = mx;
  __syncthreads();
  int excl = incl - sum;
  int total = 0, max_tiles = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) excl += s_warp_sum[w];
    total += s_warp_sum[w];
    max_tiles = max(max_tiles, s_warp_max[w]);
  }
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const int b = threadIdx.x * rpt + i;
    if (i < rpt && b < batch) s_prefix[b] = excl * streams_per_row;
    excl += local[i];
  }
  if (threadIdx.x == 0) s_prefix[batch] = total * streams_per_row;
  __syncthreads();
  return max_tiles;
}

// Share of tiles per work unit: even, at least `min_tiles`, and long enough that no stream needs more partial slots
// than the caller's scratch holds (a stream of n tiles touches at most ceil(n / share) + 1 units).
__device__ __forceinline__ int balanced_share(int total, int units, int max_tiles, int chunk_capacity, int min_tiles) {
  int share = (total + units - 1) / units;
  share = max(share, min_tiles);
  return max(share, (max_tiles + chunk_capacity - 2) / (chunk_capacity - 1));
}

// Position in the tile line, resolved to (row, stream of the row, tile of the stream).  All fields are warp-uniform.
struct TileCursor {
  int pos;        // index in the line
  int b;          // row
  int row_first;  // s_prefix[b]
  int n;          // tiles of every stream of row b
  int stream;     // stream inside the row
  int tile;       // tile inside the stream

  // Point at tile `at` (0 <= at < s_prefix[batch]).
  __device__ __forceinline__ void seek(const int* s_prefix, int batch, int streams_per_row, int at) {
    int lo = 0, hi = batch;  // invariant: s_prefix[lo] <= at < s_prefix[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= at) lo = mid; else hi = mid;
    }
    pos = at;
    b = lo;
    row_first = s_prefix[b];
    n = (s_prefix[b + 1] - row_first) / streams_per_row;
    stream = (at - row_first) / n;
    tile = (at - row_first) - stream * n;
  }
  // Step to the next tile of the line; the caller guarantees pos + 1 < s_prefix[batch] before using the fields.
  __device__ __forceinline__ void advance(const int* s_prefix, int streams_per_row, int line_end) {
    ++pos;
    if (++tile < n) return;
    tile = 0;
    if (++stream < streams_per_row) return;
    stream = 0;
    if (pos >= line_end) return;  // past the end: fields are not used any more
    do { ++b; } while (s_prefix[b + 1] <= pos);
    row_first = s_prefix[b];
    n = (s_prefix[b + 1] - row_first) / streams_per_row;
  }
  __device__ __forceinline__ int stream_first() const { return row_first + stream * n; }
};

// Calls zero_row(b) for this CTA's share of the rows without any visible key, then
// segment(b, stream, t0, t1, slot, partials_of_stream) for each piece of this CTA's tile range, in order.
// THREADS = blockDim.x (a multiple of 32, at most 1024 / 8 rows per thread); all threads of the CTA must call it and
// `segment` may synchronise the CTA.
template <int THREADS, typename ZeroFn, typename SegmentFn>
__device__ __forceinline__ void balanced_for_each_segment(const int64_t* visible_lengths, int64_t max_len, int batch,
                                                          int streams_per_row, int chunk_capacity, ZeroFn&& zero_row,
                                                          SegmentFn&& segment) {
  __shared__ int s_prefix[kBalancedMaxRows + 1];
  const int max_tiles = balanced_scan<THREADS>(visible_lengths, max_len, batch, streams_per_row, s_prefix);
  const int total = s_prefix[batch];
  auto row_len = [&](int b) -> int {
    int64_t len = visible_lengths ? visible_lengths[b] : max_len;
    return (int)max((int64_t)0, min(len, max_len));
  };

  // rows without a visible key have no tile: their zero outputs are dealt round-robin
  for (int b = blockIdx.x; b < batch; b += gridDim.x)
    if (s_prefix[b + 1] == s_prefix[b]) zero_row(b);
  if (total == 0) return;

  const int tpc = balanced_share(total, (int)gridDim.x, max_tiles, chunk_capacity, kBalancedMinTiles);
  int pos = (int)min((int64_t)blockIdx.x * tpc, (int64_t)total);
  const int end = (int)min((int64_t)pos + tpc, (int64_t)total);
  if (pos >= end) return;

  // row that holds tile `pos`: the last b with s_prefix[b] <= pos (rows without tiles are skipped by construction)
  int lo = 0, hi = batch;  // invariant: s_prefix[lo] <= pos < s_prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_prefix[mid] <= pos) lo = mid; else hi = mid;
  }
  int b = lo;
  while (pos < end) {
    while (s_prefix[b + 1] <= pos) ++b;
    const int row_first = s_prefix[b];
    const int n = (s_prefix[b + 1] - row_first) / streams_per_row;  // tiles of each stream of this row
    const int stream = (pos - row_first) / n;
    const int tile = (pos - row_first) - stream * n;
    const int seg = min(n - tile, end - pos);
    const int stream_first = row_first + stream * n;
    const int first_cta = stream_first / tpc;
    const int slot = (int)blockIdx.x - first_cta;
    const int partials = (stream_first + n - 1) / tpc - first_cta + 1;
    segment(b, stream, tile * kBalancedTileTokens, min(row_len(b), (tile + seg) * kBalancedTileTokens), slot, partials);
    pos += seg;
  }
}

// Whether the schedule can be used for this problem (host side).
inline bool balanced_schedule_fits(int batch, int64_t streams_per_row, int64_t max_len, int chunk_capacity) {
  if (batch > kBalancedMaxRows || chunk_capacity < 2) return false;
  return (int64_t)batch * streams_per_row * ((max_len + kBalancedTileTokens - 1) / kBalancedTileTokens) <
         ((int64_t)1 << 30);
}

}  // namespace anna
