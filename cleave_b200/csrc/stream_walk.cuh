// Even split of a stream of KV tiles over persistent CTAs (shared by the decode kernels).
//
// The tiles of all (request, head block) items form one stream, item after item; CTA c owns the
// units [c * span, (c + 1) * span). A piece is the part of one item inside one CTA's share.
#pragma once

namespace cb200 {

// Exclusive prefix sums of scratch[0 .. n) in place, by one warp (all 32 lanes call it); returns the total in every
// lane. A lane sums a run of consecutive entries, the runs are scanned with shuffles. (One thread walking a few hundred
// entries of shared memory, as the kernels did at first, costs about three microseconds at the head of every launch.)
__device__ __forceinline__ int warp_scan_in_place(int* scratch, int n, int lane) {
  const int per = (n + 31) / 32;
  const int b = min(lane * per, n), e = min(b + per, n);
  int mine = 0;
  for (int k = b; k < e; ++k) mine += scratch[k];
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  int run = incl - mine;
  for (int k = b; k < e; ++k) {
    const int t = scratch[k];
    scratch[k] = run;
    run += t;
  }
  return __shfl_sync(0xffffffffu, incl, 31);
}

// The walk over a CTA's share of the tile stream; identical in the producer and the consumers.
struct Piece {
  int b, hv, tile0, count, n_tiles, unit0;  // unit0: stream position of the item's first tile
};

struct Walker {
  const int* P;  // tile prefix per request (paged) or nullptr
  int batch, hkvv, tiles_per_req;
  __device__ __forceinline__ Piece at(int u, int u_end) const {
    Piece pc;
    int base;
    if (P) {
      const int key = u / hkvv;
      int lo = 0, hi = batch;  // largest b with P[b] <= key
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (P[mid] <= key) lo = mid; else hi = mid;
      }
      pc.b = lo;
      pc.n_tiles = P[lo + 1] - P[lo];
      base = hkvv * P[lo];
    } else {
      pc.n_tiles = tiles_per_req;
      pc.b = u / (hkvv * tiles_per_req);
      base = pc.b * hkvv * tiles_per_req;
    }
    const int r = u - base;
    pc.hv = r / pc.n_tiles;
    pc.tile0 = r - pc.hv * pc.n_tiles;
    pc.count = min(pc.n_tiles - pc.tile0, u_end - u);
    pc.unit0 = base + pc.hv * pc.n_tiles;
    return pc;
  }
};

}  // namespace cb200
