// Unsplit attention with many query rows (the "prefill" shapes) on the tcgen05 tensor cores.
//
//   O = softmax(scale * Q K^T [+ end-aligned causal mask]) V      q (HQ, SQ, D); k, v (HKV, SKV, D)
//
// An item is (query head, tile of 128 query rows) with the KV tiles of 128 tokens it may see. CTAs are persistent,
// one per SM: a CTA starts on the item of its block index and takes further ones from a counter in the workspace
// header (fetched one item ahead by a spare warp and handed to the others through a two-slot ring), and every
// barrier phase runs on across items. The producers and the MMA warp are therefore already on the next item - its
// place in the batch, its Q, its first K / V tiles, its first score product - while the softmax warps finish the
// current one; a batch of short prompts, where an item is one or two KV tiles, no longer pays a CTA launch, the
// set-up and the load latency in sequence per item.
// Rows of every MMA are the query rows (UMMA M = 128):
//   S = Q K^T    A = Q tile (shared memory, K-major, resident), B = K tile (shared memory, K-major),
//                D = S in tensor memory (128 columns, two buffers)
//   O += P V     A = P (tensor memory, 16-bit pairs written by the softmax warps, two buffers),
//                B = V tile (shared memory, MN-major), D = O in tensor memory (D columns)
// Warp roles: 0 = TMA producer for Q and K, 6 = TMA producer for V, 1 = MMA issuer and TMEM owner, 7 = item numbers,
// 2..5 and 8..11 = softmax / epilogue: two threads per query row (= TMEM lane), one for scores 0..63 of a tile
// and one for scores 64..127, on warps of the same lane quarter; they exchange their row maxima through shared
// memory once per tile. With one thread per row the kernel ran at the pace of its four softmax warps, one per
// scheduler with 128 exponentials per thread and tile; eight warps put two on every scheduler. S(j+1) is issued before PV(j), so the
// tensor pipe computes the next scores while the softmax warps work on the current ones. The softmax
// keeps a reference maximum per row and rescales O only when the running maximum has grown by more
// than 2^8 (exact: the factor is applied to O and to the row sum alike), so O stays in tensor memory.
//
// Reference semantics: demo/attention.py:5-8 with demo/{mha,gqa,mqa}_prefill.py (no mask), and the
// end-aligned causal mask of python/cleave/dynamic/reference.py:129-133.

#include "common.cuh"

#include <algorithm>
#include <cstring>
#include <type_traits>

namespace cb200 {
namespace fa {

constexpr int kBM = 128, kBN = 128;
constexpr int kThreads = 384;       // static and ragged layouts: warps 0..11
constexpr int kThreadsPaged = 512;  // + four gather warps (12..15)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;  // log2 units
// TMEM columns: S0 | S1 | O | P0 | P1
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;

template <int D>
struct Cfg {
  static constexpr int kChunks = D / 64;                 // 64-column chunks (128 bytes)
  static constexpr int kChunkBytes = 128 * 128;          // 128 rows x 128 bytes
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kStages = D == 64 ? 3 : 2;        // per K ring and per V ring
  static constexpr int kSmemBytes = (1 + 2 * kStages) * kTileBytes + 4096 /*barriers, row exchange*/ + 1024;
};

struct Params {
  void* out;
  float* lse;
  int* status;
  const int* qo_indptr;  // ragged: (batch + 1) query-row offsets
  const int* kv_indptr;  // ragged: (batch + 1) key offsets; paged: offsets into kv_indices
  const int* kv_indices; // paged: one page id per token (page size 1)
  const void* k_cache;   // paged: (num_pages, 1, HKV, D)
  const void* v_cache;
  int num_pages;
  int n_idx;             // paged: entries of kv_indices (0 = not stated, ranges are trusted)
  int batch;             // ragged / paged: requests
  int hq, hkv, sq, skv, q_tiles, causal;
  float scale_log2;
  int linear;      // 1: no softmax, P = scale * S (the operator (Q K^T) V of demo/matmul_matmul.py)
  float scale;     // linear mode: the plain factor
  int q_norm;      // 1: query rows are RMS-normalised (demo/qknorm.py); the row factor is folded into the scale
  float norm_eps;
};

// RAGGED: q (total_q, HQ, D), k / v (total_kv, HKV, D) with one (query range, key range) per request;
// a CTA finds its (request, query tile) by scanning the query offsets (the device-side work list of
// the reference's IndptrTileScan, python/cleave/dynamic/paging/stages.py:288-328).
// MODE 2 (paged): q as in the ragged layout; K and V rows are gathered from page-size-1 caches through
// kv_indices by four extra warps (16-byte cp.async into the swizzled tile, whole rows per warp instruction;
// a thread's arrival on the full barrier fires when its copies have landed).
// PERSIST = false is the one-item form for calls with no more items than SMs (a CTA finds its item, leaves at once if
// there is nothing to do, and only then sets up tensor memory): the item ring, the counter and tensor memory taken
// before the item is known cost a single small item about half a microsecond, which is most of what such a call is.
template <typename T, int D, int MODE, bool PERSIST>
__global__ void __launch_bounds__(MODE == 2 ? kThreadsPaged : kThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const Params p) {
  using C = Cfg<D>;
  constexpr int kStages = C::kStages;
  constexpr bool RAGGED = MODE != 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + C::kTileBytes;
  uint8_t* v_smem = k_smem + kStages * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + kStages * C::kTileBytes);
  uint64_t* k_full = bars;
  uint64_t* k_empty = k_full + kStages;
  uint64_t* v_full = k_empty + kStages;
  uint64_t* v_empty = v_full + kStages;
  uint64_t* q_full = v_empty + kStages;
  uint64_t* s_full = q_full + 1;   // [2] S complete in TMEM
  uint64_t* s_empty = s_full + 2;  // [2] the softmax warps have read S
  uint64_t* p_full = s_empty + 2;  // [2] P stored to TMEM (and O rescaled if needed)
  uint64_t* p_empty = p_full + 2;  // [2] the PV MMAs that read the P buffer have completed
  uint64_t* o_done = p_empty + 2;
  uint64_t* q_empty = o_done + 1;  // the score MMAs of an item have read Q: the next item's Q may be loaded
  uint64_t* o_free = q_empty + 1;  // the epilogue has taken O out of tensor memory
  uint64_t* t_full = o_free + 1;   // [2] an item number is in the ring
  uint64_t* t_empty = t_full + 2;  // [2] every warp has read it
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(t_empty + 2);
  volatile int* item_ring = reinterpret_cast<volatile int*>(tmem_holder + 1);  // [2]
  float* mx_exch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 1024);  // [2 tiles][2 halves][128 rows]
  float* l_exch = mx_exch + 2 * 2 * kBM;                                                  // [2 halves][128 rows]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_warps = static_cast<int>(blockDim.x >> 5);
  constexpr int kTicketWarp = 7;
  // The ranges of the first 32 requests (lane = request) are fetched before anything else: the trip to memory runs
  // beside the set-up below, and every item's search starts from these registers - for batches of up to 32
  // requests an item's place costs no memory access at all.
  int pre_lo = 0, pre_hi = 0, pre_klo = 0, pre_khi = 0;
  if constexpr (RAGGED) {
    if (lane < p.batch) {
      pre_lo = __ldg(p.qo_indptr + lane);
      pre_hi = __ldg(p.qo_indptr + lane + 1);
      pre_klo = __ldg(p.kv_indptr + lane);
      pre_khi = __ldg(p.kv_indptr + lane + 1);
    }
  }
  // ---- once per CTA: barriers, tensor memory. A CTA stays on its SM and takes (head, query tile) items one after
  // the other, so this set-up, the launch of a CTA and above all the latency at the start of an item (its place in
  // the batch, the first Q / K / V loads) are not paid in sequence per item: the producers and the MMA warp are
  // already on the next item while the softmax warps finish the current one.
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], MODE == 2 ? 128 : 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], MODE == 2 ? 128 : 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 8);
      mbar_init(&p_full[s], 8);
      mbar_init(&p_empty[s], 1);
      mbar_init(&t_full[s], 1);
      mbar_init(&t_empty[s], n_warps - 1);
    }
    mbar_init(q_full, 1);
    mbar_init(o_done, 1);
    mbar_init(q_empty, p.q_norm ? 9 : 1);  // with RMS-normalised queries the softmax warps read the Q tile too
    mbar_init(o_free, 8);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  uint32_t tmem_base = 0;
  auto take_tensor_memory = [&]() {
    if (warp == 1) {
      tmem_alloc(tmem_holder, 512);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
    // The static launch is a dependent launch: the grid may have been scheduled while the preceding kernel of
    // the stream drains. Up to here only shared and tensor memory were set up (and, in the ragged layouts, whose
    // launches do not carry the attribute, the request offsets read); the operands are touched after the wait.
    pdl_launch_dependents();
    pdl_wait();
  };
  if constexpr (PERSIST) take_tensor_memory();

  // The host's item count is an upper bound (one query tile more per request than total_q / 128); items that do not
  // exist come first in the order, and every persistent CTA would spend its first rounds on them. The exact number
  // of query tiles is a sum over the request ranges: the first 32 are in this warp's registers, the others cost
  // a few independent loads per lane.
  // (persistent form; in the one-item form a surplus CTA simply leaves, and numbering the items from the bound
  // measured 0.35 us faster on a single-item call)
  int q_tiles = p.q_tiles;
  if constexpr (RAGGED && PERSIST) {
    int mine = pre_hi > pre_lo ? ceil_div(pre_hi - pre_lo, kBM) : 0;
#pragma unroll 4
    for (int rr = 32 + lane; rr < p.batch; rr += 32) {
      const int lo = __ldg(p.qo_indptr + rr), hi = __ldg(p.qo_indptr + rr + 1);
      mine += hi > lo ? ceil_div(hi - lo, kBM) : 0;
    }
    q_tiles = __reduce_add_sync(0xffffffffu, mine);
  }
  const int n_items = p.hq * q_tiles;
  int* ticket = p.status + 8;    // items beyond the first of every CTA are dealt by this counter
  int* finished = p.status + 9;  // CTAs that are through; the last one clears both words for the next launch
  if (PERSIST && warp == kTicketWarp) {
    // ================================================================ item numbers for the other warps
    // The first item of a CTA is its block index, which every warp knows; the others come from a counter, fetched
    // one item ahead and handed round through a two-slot ring. Items are numbered so that late query tiles, which
    // see the most keys under the causal mask, come first.
    if (lane == 0) {
      for (int k = 0;; ++k) {
        const int s = k & 1;
        mbar_wait(&t_empty[s], ((k >> 1) & 1) ^ 1, p.status, kFaultEmptyBarrier);
        // with no more items than CTAs every item is somebody's first: no counter, nothing to clear at the end
        const int item = n_items <= static_cast<int>(gridDim.x) ? n_items : static_cast<int>(gridDim.x) + atomicAdd(ticket, 1);
        item_ring[s] = item;
        mbar_arrive(&t_full[s]);
        if (item >= n_items) break;
      }
    }
    __syncwarp();
  }
  int n_taken = 0;  // item numbers this warp has had
  int it = 0;       // items with keys this CTA has run, jt: their KV tiles (every role counts alike)
  int jt = 0;
  int st_a = 0, ph_a = 0, st_b = 0, ph_b = 0;  // ring positions of this warp's role
  while (!PERSIST || warp != kTicketWarp) {
    int item = static_cast<int>(blockIdx.x);
    if (PERSIST && n_taken > 0) {  // the ring's entry number n_taken - 1
      const int s = (n_taken - 1) & 1;
      mbar_wait(&t_full[s], ((n_taken - 1) >> 1) & 1, p.status, kFaultFullBarrier);
      item = item_ring[s];
      __syncwarp();
      if (lane == 0) mbar_arrive(&t_empty[s]);
    }
    ++n_taken;
    if (item >= n_items) {  // (one-item form: the grid is the host's upper bound, tensor memory is not yet taken)
      if constexpr (PERSIST) break;
      else return;
    }
  // heads of one query tile are neighbours (they share K/V in L2)
  const int h = item % p.hq;
  const int hk = h / (p.hq / p.hkv);
  int q0, sq, skv, q_base = 0, kv_base = 0;
  if constexpr (RAGGED) {
    // Every warp searches the query offsets 32 requests at a time (lane = request, tile counts scanned with shuffles):
    // an item's place costs a few hundred clocks whatever the batch.
    int t = q_tiles - 1 - item / p.hq, r = 0;
    bool found = false;
    for (int r0 = 0; r0 < p.batch && !found; r0 += 32) {
      const int rr = r0 + lane;
      int lo = pre_lo, hi = pre_hi, klo = pre_klo, khi = pre_khi;
      if (r0 > 0) {
        lo = rr < p.batch ? __ldg(p.qo_indptr + rr) : 0;
        hi = rr < p.batch ? __ldg(p.qo_indptr + rr + 1) : 0;
        // the key range of the lane's request travels with the query range: one trip to memory, not two in a row
        klo = rr < p.batch ? __ldg(p.kv_indptr + rr) : 0;
        khi = rr < p.batch ? __ldg(p.kv_indptr + rr + 1) : 0;
      }
      const int tiles = hi > lo ? ceil_div(hi - lo, kBM) : 0;
      int incl = tiles;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int all = __shfl_sync(0xffffffffu, incl, 31);
      if (t < all) {
        const int first = __ffs(__ballot_sync(0xffffffffu, incl > t)) - 1;
        r = r0 + first;
        t -= __shfl_sync(0xffffffffu, incl - tiles, first);
        q_base = __shfl_sync(0xffffffffu, lo, first);
        sq = __shfl_sync(0xffffffffu, hi, first) - q_base;
        kv_base = __shfl_sync(0xffffffffu, klo, first);
        skv = max(__shfl_sync(0xffffffffu, khi, first) - kv_base, 0);
        found = true;
      } else {
        t -= all;
      }
    }
    (void)r;
    if (!found) {  // the item count is an upper bound on the number of query tiles
      if constexpr (PERSIST) continue;
      else return;
    }
    if constexpr (MODE == 2) {
      // the page table is caller data: a range that runs past its stated length is read as a shorter request
      if (p.n_idx > 0) {
        kv_base = min(max(kv_base, 0), p.n_idx);
        skv = min(skv, p.n_idx - kv_base);
      }
    }
    q0 = t * kBM;
  } else {
    q0 = (q_tiles - 1 - item / p.hq) * kBM;
    sq = p.sq;
    skv = p.skv;
  }
  const int off = skv - sq;  // end-aligned causal mask: row r sees keys <= r + off
  int nt = ceil_div(skv, kBN);
  if (p.causal) {
    const int last_key = min(sq, q0 + kBM) - 1 + off;
    nt = last_key < 0 ? 0 : min(nt, last_key / kBN + 1);
  }

  if (nt == 0) {
    // No key is visible to any row of this tile (an empty request, or query rows the end-aligned mask leaves
    // blind): the rows are 0 and -inf, as the reference's preallocation leaves them; the warps share the rows.
    const int rows = min(kBM, sq - q0);
    const int cw = warp < kTicketWarp ? warp : warp - 1;
    T* outp = reinterpret_cast<T*>(p.out);
    for (int i = cw * 32 + lane; i < rows * (D / 8); i += (n_warps - 1) * 32) {
      const int rw = i / (D / 8), c = i - rw * (D / 8);
      const size_t orow = RAGGED ? static_cast<size_t>(q_base + q0 + rw) * p.hq + h : static_cast<size_t>(h) * sq + q0 + rw;
      *reinterpret_cast<uint4*>(outp + orow * D + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (p.lse && !p.linear)
      for (int i = cw * 32 + lane; i < rows; i += (n_warps - 1) * 32)
        p.lse[RAGGED ? static_cast<size_t>(q_base + q0 + i) * p.hq + h : static_cast<size_t>(h) * sq + q0 + i] = -INFINITY;
    if constexpr (PERSIST) continue;
    else return;
  }
  if constexpr (!PERSIST) take_tensor_memory();

  if (warp == 0) {
    // ================================================================ TMA producer: Q, then K tiles
    mbar_wait(q_empty, (it & 1) ^ 1, p.status, kFaultEmptyBarrier);  // the item before has no use for its Q any more
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kChunks; ++c) {
        if constexpr (RAGGED) tma_load_3d(q_smem + c * C::kChunkBytes, &tm_q, q_full, c * 64, h, q_base + q0);
        else tma_load_3d(q_smem + c * C::kChunkBytes, &tm_q, q_full, c * 64, q0, h);
      }
    }
    __syncwarp();
    for (int j = 0; MODE != 2 && j < nt; ++j) {
      mbar_wait(&k_empty[st_a], ph_a ^ 1, p.status, kFaultEmptyBarrier);
      if (elect_one()) {
        mbar_arrive_expect_tx(&k_full[st_a], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c) {
          uint8_t* dst = k_smem + st_a * C::kTileBytes + c * C::kChunkBytes;
          if constexpr (RAGGED) tma_load_3d(dst, &tm_k, &k_full[st_a], c * 64, hk, kv_base + j * kBN);
          else tma_load_3d(dst, &tm_k, &k_full[st_a], c * 64, j * kBN, hk);
        }
      }
      __syncwarp();
      if (++st_a == kStages) { st_a = 0; ph_a ^= 1; }
    }
  } else if (warp == 6) {
    // ================================================================ TMA producer: V tiles
    for (int j = 0; MODE != 2 && j < nt; ++j) {
      mbar_wait(&v_empty[st_a], ph_a ^ 1, p.status, kFaultEmptyBarrier);
      if (elect_one()) {
        mbar_arrive_expect_tx(&v_full[st_a], C::kTileBytes);
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c) {
          uint8_t* dst = v_smem + st_a * C::kTileBytes + c * C::kChunkBytes;
          if constexpr (RAGGED) tma_load_3d(dst, &tm_v, &v_full[st_a], c * 64, hk, kv_base + j * kBN);
          else tma_load_3d(dst, &tm_v, &v_full[st_a], c * 64, j * kBN, hk);
        }
      }
      __syncwarp();
      if (++st_a == kStages) { st_a = 0; ph_a ^= 1; }
    }
  } else if (warp >= 12) {
    // ================================================================ paged: K / V row gather
    if constexpr (MODE == 2) {
      // Consecutive lanes copy consecutive 16-byte chunks of a row, so one warp instruction moves whole
      // rows as full 128-byte lines; the 128 threads cover kRowsPerRound rows at once.
      const int gtid = tid - 12 * 32;  // 0..127
      constexpr int kChunksPerRow = D / 8;
      constexpr int kRowsPerRound = 128 / kChunksPerRow;
      constexpr int kRounds = kBN / kRowsPerRound;
      const int c = gtid % kChunksPerRow, r_in = gtid / kChunksPerRow;
      const T* kc = reinterpret_cast<const T*>(p.k_cache);
      const T* vc = reinterpret_cast<const T*>(p.v_cache);
      auto load_pages = [&](int j, int (&pg)[kRounds]) {
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
          const int tok = min(j * kBN + r * kRowsPerRound + r_in, skv - 1);  // rows past the end repeat the last token; they are masked
          pg[r] = __ldg(p.kv_indices + kv_base + tok);
        }
      };
      int pg[kRounds];
      load_pages(0, pg);
      for (int j = 0; j < nt; ++j) {
        long long src[kRounds];
#pragma unroll
        for (int r = 0; r < kRounds; ++r)
          src[r] = (static_cast<long long>(min(max(pg[r], 0), p.num_pages - 1)) * p.hkv + hk) * D + c * 8;
        if (j + 1 < nt) load_pages(j + 1, pg);  // one tile ahead: the index latency stays off the critical path
        const uint32_t kdst = smem_u32(k_smem + st_a * C::kTileBytes), vdst = smem_u32(v_smem + st_a * C::kTileBytes);
        mbar_wait(&k_empty[st_a], ph_a ^ 1, p.status, kFaultEmptyBarrier);
        // rounds of rows that lie wholly past the request's last key are not fetched: zeros from the thread itself
        // (masked as keys, and as values they meet P = 0), made visible to the MMA's proxy before the arrival
        // (one-item form only: the test in the copy loop costs the long streams of the persistent form a tenth)
        const int live_rounds = PERSIST ? kRounds : min(kRounds, (skv - j * kBN + kRowsPerRound - 1) / kRowsPerRound);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
          const int row = r * kRowsPerRound + r_in;
          const uint32_t o = (c >> 3) * C::kChunkBytes + row * 128 + (((c & 7) ^ (row & 7)) << 4);
          if (r < live_rounds) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kdst + o), "l"(kc + src[r]) : "memory");
          else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(kdst + o), "r"(0u) : "memory");
        }
        if (live_rounds < kRounds) fence_proxy_async_smem();
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&k_full[st_a])) : "memory");
        mbar_wait(&v_empty[st_a], ph_a ^ 1, p.status, kFaultEmptyBarrier);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
          const int row = r * kRowsPerRound + r_in;
          const uint32_t o = (c >> 3) * C::kChunkBytes + row * 128 + (((c & 7) ^ (row & 7)) << 4);
          if (r < live_rounds) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vdst + o), "l"(vc + src[r]) : "memory");
          else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(vdst + o), "r"(0u) : "memory");
        }
        if (live_rounds < kRounds) fence_proxy_async_smem();
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&v_full[st_a])) : "memory");
        if (++st_a == kStages) { st_a = 0; ph_a ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t idesc_s = umma_idesc(kBf16, /*b_mn_major=*/false, kBM, kBN);
    constexpr uint32_t idesc_pv = umma_idesc(kBf16, /*b_mn_major=*/true, kBM, D);
    const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem);
    int& kst = st_a; int& kph = ph_a; int& vst = st_b; int& vph = ph_b;
    auto issue_s = [&](int j) {
      const int jj = jt + j, sb = jj & 1;
      mbar_wait(&k_full[kst], kph, p.status, kFaultFullBarrier);
      mbar_wait(&s_empty[sb], ((jj >> 1) & 1) ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (elect_one()) {
        const uint32_t d = tmem_base + kColS + sb * kBN;
#pragma unroll
        for (int c = 0; c < C::kChunks; ++c) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adesc = umma_smem_desc(q_addr + c * C::kChunkBytes + kk * 32, 16, 8 * 128);
            const uint64_t bdesc = umma_smem_desc(k_addr + kst * C::kTileBytes + c * C::kChunkBytes + kk * 32, 16, 8 * 128);
            umma_f16(d, adesc, bdesc, idesc_s, (c > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&k_empty[kst]);
        umma_commit(&s_full[sb]);
        if (j == nt - 1) umma_commit(q_empty);  // the item's last use of Q
      }
      __syncwarp();
      if (++kst == kStages) { kst = 0; kph ^= 1; }
    };
    mbar_wait(q_full, it & 1, p.status, kFaultFullBarrier);
    issue_s(0);
    for (int j = 0; j < nt; ++j) {
      if (j + 1 < nt) issue_s(j + 1);
      const int jj = jt + j, pb = jj & 1;
      mbar_wait(&v_full[vst], vph, p.status, kFaultFullBarrier);
      mbar_wait(&p_full[pb], (jj >> 1) & 1, p.status, kFaultTmemBarrier);
      // the first value product of an item overwrites O: the epilogue of the item before must have read it
      if (j == 0) mbar_wait(o_free, (it & 1) ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (elect_one()) {
        const uint32_t va = v_addr + vst * C::kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          // B: MN-major, 16 token rows of 128 bytes per step; 64-column chunks are kChunkBytes apart
          const uint64_t bdesc = umma_smem_desc(va + ks * 16 * 128, C::kChunkBytes, 8 * 128);
          umma_f16_ts(tmem_base + kColO, tmem_base + kColP + pb * 64 + ks * 8, bdesc, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[vst]);
        umma_commit(&p_empty[pb]);
        if (j == nt - 1) umma_commit(o_done);
      }
      __syncwarp();
      if (++vst == kStages) { vst = 0; vph ^= 1; }
    }
  } else if (warp != 7) {
    // ================================================================ softmax / epilogue (warps 2..5 and 8..11)
    const int quarter = warp & 3;
    const int half = warp >= 8 ? 1 : 0;   // which 64 of a tile's 128 scores this thread takes
    const int row = quarter * 32 + lane;  // query row inside the tile = TMEM lane
    const int qrow = q0 + row;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const int key_limit = p.causal ? min(skv - 1, qrow + off) : skv - 1;  // last key this row sees
    const int pair_bar = 1 + quarter;     // named barrier of the two warps that share the rows
    float m_ref = 0.f, l_run = 0.f;       // l_run: the sum over this thread's half of every tile
    // scores are scale_row * (q . k): the softmax scale in log2 units (the plain factor in linear mode)
    // times, for RMS-normalised queries, rsqrt(mean(q^2) + eps) of this thread's row, taken from the
    // resident Q tile (K arrives normalised)
    float scale_row = p.linear ? p.scale : p.scale_log2;
    if (p.q_norm) {
      mbar_wait(q_full, it & 1, p.status, kFaultFullBarrier);
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const uint4 u = *reinterpret_cast<const uint4*>(q_smem + (c >> 3) * C::kChunkBytes + row * 128 +
                                                         (((c & 7) ^ (row & 7)) << 4));
        const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float f = static_cast<float>(e[i]);
          ss = fmaf(f, f, ss);
        }
      }
      scale_row = qrow < sq ? scale_row * rsqrtf(ss * (1.f / D) + p.norm_eps) : 0.f;
      __syncwarp();
      if (lane == 0) mbar_arrive(q_empty);
    }
    // the last key any row of this warp sees: a half tile of scores beyond it is neither read nor exponentiated (the
    // tile of a short request, the diagonal tile of a query tile's first rows); tensor-memory loads are
    // warp-collective, so the test is the warp's, not the row's
    const int warp_limit = __reduce_max_sync(0xffffffffu, qrow < sq ? key_limit : -1);
    for (int j = 0; j < nt; ++j) {
      const int jj = jt + j, sb = jj & 1, pb = jj & 1;
      const int k0 = j * kBN + half * 64;  // first key of this thread's scores
      // (in the one-item form only: in the persistent form the test costs the long tile loops more than it saves)
      const bool unseen = !PERSIST && !p.linear && k0 > warp_limit;
      mbar_wait(&s_full[sb], (jj >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      uint32_t r[2][32];
      if (!unseen) {
#pragma unroll
        for (int q = 0; q < 2; ++q) tmem_ld_32x32(tmem_base + lane_field + kColS + sb * kBN + half * 64 + q * 32, r[q]);
        tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      if (p.linear) {
        // no softmax: P = scale * S rounded to the storage type; keys past the end are zero rows of K
        mbar_wait(&p_empty[pb], ((jj >> 1) & 1) ^ 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = 2 * i;
          const float p0 = k0 + c <= key_limit ? __uint_as_float(r[c >> 5][c & 31]) * scale_row : 0.f;
          const float p1 = k0 + c + 1 <= key_limit ? __uint_as_float(r[(c + 1) >> 5][(c + 1) & 31]) * scale_row : 0.f;
          pk[i] = pack2<T>(p0, p1);
        }
        tmem_st_32x32(tmem_base + lane_field + kColP + pb * 64 + half * 32, pk);
        l_run = half == 0 ? 1.f : 0.f;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[pb]);
        continue;
      }
      float mx = -INFINITY;
      if (unseen) {
        // nothing to look at
      } else if (k0 + 63 <= key_limit) {  // this thread's half of the tile is visible to the row
#pragma unroll
        for (int q = 0; q < 2; ++q) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __uint_as_float(r[q][i]) * scale_row;
            r[q][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = k0 + q * 32 + i <= key_limit ? __uint_as_float(r[q][i]) * scale_row : -INFINITY;
            r[q][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
        }
      }
      // the row maximum over both halves: the partner thread sits in the warp of the same lane quarter
      mx_exch[(sb * 2 + half) * kBM + row] = mx;
      named_bar_sync(pair_bar, 64);
      mx = fmaxf(mx, mx_exch[(sb * 2 + (half ^ 1)) * kBM + row]);
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_ref = mx == -INFINITY ? 0.f : mx;
      } else if (mx > m_ref + kRescaleThreshold) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      // the P buffer is free once the PV MMAs of tile j - 2 have completed
      mbar_wait(&p_empty[pb], ((jj >> 1) & 1) ^ 1, p.status, kFaultMmaBarrier);
      if (__any_sync(0xffffffffu, rescale)) {  // rare: the running maximum grew by more than 2^8
        // O may only be touched when no PV MMA is in flight: tile j - 1 is the last one issued. The two threads
        // of a row came to the same decision (same maximum) and take half of the row's columns each.
        mbar_wait(&p_empty[pb ^ 1], ((jj - 1) >> 1) & 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
#pragma unroll 1
        for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_field + kColO + c0, o);
        }
        tmem_st_wait();
      }
      tc_fence_after();
      float psum = 0.f;
      {
        uint32_t pk[32];
        if (unseen) {
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = 0u;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c = 2 * i;
            const float p0 = fast_exp2(__uint_as_float(r[c >> 5][c & 31]) - m_ref);
            const float p1 = fast_exp2(__uint_as_float(r[(c + 1) >> 5][(c + 1) & 31]) - m_ref);
            psum += p0 + p1;
            pk[i] = pack2<T>(p0, p1);
          }
        }
        tmem_st_32x32(tmem_base + lane_field + kColP + pb * 64 + half * 32, pk);
      }
      l_run = l_run * alpha + psum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // ---- epilogue: O / l; the row sum is the two threads' together, and each stores half of the row's columns
    l_exch[half * kBM + row] = l_run;
    named_bar_sync(pair_bar, 64);
    l_run += l_exch[(half ^ 1) * kBM + row];
    mbar_wait(o_done, it & 1, p.status, kFaultMmaBarrier);
    tc_fence_after();
    const bool live = qrow < sq;
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const size_t orow = RAGGED ? static_cast<size_t>(q_base + qrow) * p.hq + h : static_cast<size_t>(h) * sq + qrow;
    T* outp = reinterpret_cast<T*>(p.out) + orow * D;
#pragma unroll 1
    for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
      tmem_ld_wait();
      if (c0 + 32 >= (half + 1) * (D / 2)) {  // O is out of tensor memory: the next item's value product may start
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free);
      }
      if (live) {
        const float* v = reinterpret_cast<const float*>(o);
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 q4;
          q4.x = pack2<T>(v[i] * inv, v[i + 1] * inv);
          q4.y = pack2<T>(v[i + 2] * inv, v[i + 3] * inv);
          q4.z = pack2<T>(v[i + 4] * inv, v[i + 5] * inv);
          q4.w = pack2<T>(v[i + 6] * inv, v[i + 7] * inv);
          *reinterpret_cast<uint4*>(outp + c0 + i) = q4;
        }
      }
    }
    if (half == 0 && live && p.lse && !p.linear) p.lse[orow] = l_run > 0.f ? m_ref + fast_log2(l_run) : -INFINITY;
  }
    if constexpr (!PERSIST) break;
    jt += nt;
    ++it;
  }  // items

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (PERSIST && tid == 0 && n_items > static_cast<int>(gridDim.x) && atomicAdd(finished, 1) == static_cast<int>(gridDim.x) - 1) {
    // every CTA has fetched its last item number: the counters are clear for the next launch
    atomicExch(ticket, 0);
    atomicExch(finished, 0);
  }
}

// RMS-normalises rows of D elements, one warp per row: y = x * rsqrt(mean(x^2) + eps), fp32 statistics,
// result in the storage type. Used on K ahead of the attention kernel for demo/qknorm.py (K is the small
// operand: it is read by every query tile, so it is normalised once instead of per tile).
template <typename T, int D>
__global__ void __launch_bounds__(256) rms_rows_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, float eps) {
  constexpr int kPer = D / 32;  // 2 or 4 elements per lane
  const int lane = threadIdx.x & 31;
  const long long stride = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += stride) {
    T e[kPer];
    if constexpr (kPer == 4) *reinterpret_cast<uint2*>(e) = *reinterpret_cast<const uint2*>(x + r * D + lane * 4);
    else *reinterpret_cast<uint32_t*>(e) = *reinterpret_cast<const uint32_t*>(x + r * D + lane * 2);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
      const float f = static_cast<float>(e[i]);
      ss = fmaf(f, f, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float f = rsqrtf(ss * (1.f / D) + eps);
#pragma unroll
    for (int i = 0; i < kPer; ++i) e[i] = static_cast<T>(static_cast<float>(e[i]) * f);
    if constexpr (kPer == 4) *reinterpret_cast<uint2*>(y + r * D + lane * 4) = *reinterpret_cast<const uint2*>(e);
    else *reinterpret_cast<uint32_t*>(y + r * D + lane * 2) = *reinterpret_cast<const uint32_t*>(e);
  }
}

}  // namespace fa

// ------------------------------------------------------------------------------------- host side
namespace {

int plan_prefill(const cb200_attn_prefill_args* a) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->q_len <= 0 || a->kv_len <= 0) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads % a->num_kv_heads) return CB200_ERR_BAD_ARG;
  if (a->head_dim != 64 && a->head_dim != 128) return CB200_ERR_UNSUPPORTED;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  const long long ctas = static_cast<long long>(a->num_qo_heads) * ceil_div(a->q_len, fa::kBM);
  if (ctas >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  if (a->score_mode != CB200_SCORE_SOFTMAX && a->score_mode != CB200_SCORE_LINEAR) return CB200_ERR_BAD_ARG;
  if (a->qk_norm && !(a->norm_eps >= 0.f)) return CB200_ERR_BAD_ARG;
  return CB200_OK;
}

// bytes of the normalised copy of K that follows the status header when qk_norm is set
size_t prefill_knorm_bytes(const cb200_attn_prefill_args* a) {
  if (!a->qk_norm) return 0;
  return static_cast<size_t>(a->num_kv_heads) * a->kv_len * a->head_dim * 2;
}

template <typename T, int D>
int launch_prefill(const cb200_attn_prefill_args* a, cudaStream_t stream) {
  using namespace fa;
  Params p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = reinterpret_cast<int*>(a->workspace);
  p.hq = a->num_qo_heads;
  p.hkv = a->num_kv_heads;
  p.sq = a->q_len;
  p.skv = a->kv_len;
  p.q_tiles = ceil_div(a->q_len, kBM);
  p.causal = a->causal ? 1 : 0;
  p.scale_log2 = a->sm_scale * kLog2e;
  p.linear = a->score_mode == CB200_SCORE_LINEAR ? 1 : 0;
  p.scale = a->sm_scale;
  p.q_norm = a->qk_norm ? 1 : 0;
  p.norm_eps = a->norm_eps;
  const void* k_src = a->k;
  if (a->qk_norm) {
    T* kn = reinterpret_cast<T*>(static_cast<uint8_t*>(a->workspace) + kWsHeaderBytes);
    const long long rows = static_cast<long long>(a->num_kv_heads) * a->kv_len;
    const int blocks = static_cast<int>(std::min<long long>((rows + 7) / 8, 148LL * 8));
    rms_rows_kernel<T, D><<<blocks, 256, 0, stream>>>(reinterpret_cast<const T*>(a->k), kn, rows, a->norm_eps);
    CB200_CUDA_TRY(cudaGetLastError());
    k_src = kn;
  }
  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_q, tm_k, tm_v;
  {
    uint32_t box[3] = {64u, 128u, 1u};
    uint64_t dq[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(a->q_len), static_cast<uint64_t>(a->num_qo_heads)};
    uint64_t sq[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(a->q_len) * D * 2};
    uint64_t dk[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(a->kv_len), static_cast<uint64_t>(a->num_kv_heads)};
    uint64_t sk[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(a->kv_len) * D * 2};
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    if (!encode_tensor_map(&tm_q, dt, 3, const_cast<void*>(a->q), dq, sq, box, sw) ||
        !encode_tensor_map(&tm_k, dt, 3, const_cast<void*>(k_src), dk, sk, box, sw) ||
        !encode_tensor_map(&tm_v, dt, 3, const_cast<void*>(a->v), dk, sk, box, sw))
      return CB200_ERR_CUDA;
  }
  // one CTA per SM at most, and then the CTAs deal the (head, query tile) items among themselves; with no more items
  // than SMs every item has its own CTA and the kernel's one-item form runs
  const long long n_items = static_cast<long long>(p.hq) * p.q_tiles;
  const bool persist = n_items > sm_count();
  auto kern = persist ? attn_prefill_kernel<T, D, 0, true> : attn_prefill_kernel<T, D, 0, false>;
  CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
  const unsigned grid = static_cast<unsigned>(std::min<long long>(n_items, sm_count()));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg<D>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // scheduled while the preceding kernel of the stream drains; the kernel waits before its first global access
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_q, tm_k, tm_v, p));
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

int plan_prefill_ragged(const cb200_attn_prefill_ragged_args* a) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->batch <= 0 || a->total_q <= 0 || a->total_kv <= 0)
    return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads % a->num_kv_heads) return CB200_ERR_BAD_ARG;
  if (a->head_dim != 64 && a->head_dim != 128) return CB200_ERR_UNSUPPORTED;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  const long long ctas = static_cast<long long>(a->num_qo_heads) * (ceil_div(a->total_q, fa::kBM) + a->batch);
  if (ctas >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  return CB200_OK;
}

template <typename T, int D>
int launch_prefill_ragged(const cb200_attn_prefill_ragged_args* a, cudaStream_t stream) {
  using namespace fa;
  Params p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = reinterpret_cast<int*>(a->workspace);
  p.qo_indptr = a->qo_indptr;
  p.kv_indptr = a->kv_indptr;
  p.kv_indices = a->kv_indices;
  p.k_cache = a->k;
  p.v_cache = a->v;
  p.num_pages = a->total_kv;
  p.n_idx = a->kv_indices ? a->num_kv_indices : 0;
  p.batch = a->batch;
  p.hq = a->num_qo_heads;
  p.hkv = a->num_kv_heads;
  p.causal = a->causal ? 1 : 0;
  p.scale_log2 = a->sm_scale * kLog2e;
  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_q, tm_k, tm_v;
  {
    // a box is 64 columns of one head for 128 consecutive tokens: the same shared-memory image as the
    // static layout's (64 columns x 128 rows)
    uint32_t box[3] = {64u, 1u, 128u};
    uint64_t dq[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(a->num_qo_heads), static_cast<uint64_t>(a->total_q)};
    uint64_t sq[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(a->num_qo_heads) * D * 2};
    uint64_t dk[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(a->num_kv_heads), static_cast<uint64_t>(a->total_kv)};
    uint64_t sk[2] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(a->num_kv_heads) * D * 2};
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    if (!encode_tensor_map(&tm_q, dt, 3, const_cast<void*>(a->q), dq, sq, box, sw) ||
        !encode_tensor_map(&tm_k, dt, 3, const_cast<void*>(a->k), dk, sk, box, sw) ||
        !encode_tensor_map(&tm_v, dt, 3, const_cast<void*>(a->v), dk, sk, box, sw))
      return CB200_ERR_CUDA;
  }
  // every request has at most ceil(q_len / 128) <= q_len / 128 + 1 query tiles: an upper bound on the items, which
  // the CTAs (one per SM at most) deal among themselves
  p.q_tiles = ceil_div(a->total_q, kBM) + a->batch;
  const long long n_items = static_cast<long long>(p.hq) * p.q_tiles;
  const bool persist = n_items > sm_count();
  const unsigned grid = static_cast<unsigned>(std::min<long long>(n_items, sm_count()));
  if (a->kv_indices) {
    auto kern = persist ? attn_prefill_kernel<T, D, 2, true> : attn_prefill_kernel<T, D, 2, false>;
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
    kern<<<grid, kThreadsPaged, Cfg<D>::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  } else {
    auto kern = persist ? attn_prefill_kernel<T, D, 1, true> : attn_prefill_kernel<T, D, 1, false>;
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
    kern<<<grid, kThreads, Cfg<D>::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

}  // namespace
}  // namespace cb200

extern "C" size_t cb200_attn_prefill_workspace_bytes(const cb200_attn_prefill_args* a) {
  return cb200::plan_prefill(a) == CB200_OK ? cb200::kWsHeaderBytes + cb200::prefill_knorm_bytes(a) : 0;
}

extern "C" int cb200_attn_prefill(const cb200_attn_prefill_args* a, void* stream) {
  using namespace cb200;
  const int rc = plan_prefill(a);
  if (rc != CB200_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->out) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < kWsHeaderBytes + prefill_knorm_bytes(a)) return CB200_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f16 = a->dtype == CB200_F16;
  if (a->head_dim == 64)
    return f16 ? launch_prefill<__half, 64>(a, st) : launch_prefill<__nv_bfloat16, 64>(a, st);
  return f16 ? launch_prefill<__half, 128>(a, st) : launch_prefill<__nv_bfloat16, 128>(a, st);
}

extern "C" size_t cb200_attn_prefill_ragged_workspace_bytes(const cb200_attn_prefill_ragged_args* a) {
  return cb200::plan_prefill_ragged(a) == CB200_OK ? cb200::kWsHeaderBytes : 0;
}

extern "C" int cb200_attn_prefill_ragged(const cb200_attn_prefill_ragged_args* a, void* stream) {
  using namespace cb200;
  const int rc = plan_prefill_ragged(a);
  if (rc != CB200_OK) return rc;
  if (!a->q || !a->k || !a->v || !a->out || !a->qo_indptr || !a->kv_indptr) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < kWsHeaderBytes) return CB200_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // A key window far shorter than the run of query rows: only the last min(q_len, kv_len) rows of a request see a
    // key, the rest are written as 0 / -inf, and two light kernels do both faster than a CTA per tile of 128 rows.
    const int keys = a->kv_indices ? a->num_kv_indices : a->total_kv;
    if (a->causal && small_prefill_applies(keys, a->total_q))
      return launch_small_gqa(a->q, a->k, a->v, a->qo_indptr, a->kv_indptr, a->kv_indices, a->out, a->lse, a->batch, a->total_q,
                              a->num_qo_heads, a->num_kv_heads, a->head_dim, a->kv_indices ? a->total_kv : 0, keys, a->sm_scale,
                              a->dtype, st);
  }
  const bool f16 = a->dtype == CB200_F16;
  if (a->head_dim == 64)
    return f16 ? launch_prefill_ragged<__half, 64>(a, st) : launch_prefill_ragged<__nv_bfloat16, 64>(a, st);
  return f16 ? launch_prefill_ragged<__half, 128>(a, st) : launch_prefill_ragged<__nv_bfloat16, 128>(a, st);
}
