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
//
// Paged items may carry `w` overhead units in front of their tiles: the stream is then cut by cost, not by tile
// count. Starting a piece (finding it, its query rows, the first page ids) and finishing it (the warps' states
// merged, the output or a partial written) costs a kernel as much as a few tiles, so a CTA whose share is a run of
// very short requests would otherwise work several times longer than one that streams a single long request. The
// overhead units hold no work: a share that ends inside them simply does not reach the item.
struct Piece {
  int b, hv, tile0, count, n_tiles, unit0;  // unit0: stream position of the item's first tile; count 0: nothing left
};

struct Walker {
  const int* P;  // unit prefix per request (paged: tiles + w per request with tokens) or nullptr
  int batch, hkvv, tiles_per_req;
  int w;         // overhead units per paged item
  // the units a request with `tiles` tiles occupies per (head) item
  __device__ __forceinline__ static int units(int tiles, int w_) { return tiles > 0 ? tiles + w_ : 0; }
  // The piece at stream position u of a share that ends at u_end. u is moved past overhead units first; when the
  // share ends before the item's first tile, u becomes u_end and the piece has count 0.
  __device__ __forceinline__ Piece at(int& u, int u_end) const {
    Piece pc;
    int base;
    if (P) {
      const int key = u / hkvv;
      int lo = 0, hi = batch;  // largest b with P[b] <= key
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (P[mid] <= key) lo = mid; else hi = mid;
      }
      const int nv = P[lo + 1] - P[lo];  // units per item of this request
      base = hkvv * P[lo];
      const int r = u - base;
      pc.b = lo;
      pc.hv = r / nv;
      int off = r - pc.hv * nv;
      pc.n_tiles = nv - w;
      pc.unit0 = base + pc.hv * nv + w;
      if (off < w) {
        u += w - off;
        off = w;
        if (u >= u_end) {
          u = u_end;
          pc.tile0 = 0;
          pc.count = 0;
          return pc;
        }
      }
      pc.tile0 = off - w;
      pc.count = min(pc.n_tiles - pc.tile0, u_end - u);
      return pc;
    }
    pc.n_tiles = tiles_per_req;
    pc.b = u / (hkvv * tiles_per_req);
    base = pc.b * hkvv * tiles_per_req;
    const int r = u - base;
    pc.hv = r / pc.n_tiles;
    pc.tile0 = r - pc.hv * pc.n_tiles;
    pc.count = min(pc.n_tiles - pc.tile0, u_end - u);
    pc.unit0 = base + pc.hv * pc.n_tiles;
    return pc;
  }
};

}  // namespace cb200
