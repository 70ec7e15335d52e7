// Paged MLA decode (absorbed latent, one token per page) on the tcgen05 tensor cores, for operators with at
// most 16 heads (the reference ships mla_paged_decode_h16_ckv512_kpe64_ps1).
//
//   S = (q_nope CKV^T + q_pe KPE^T) * scale, O = softmax(S) CKV, per request over the tokens
//   kv_indices[kv_indptr[b] .. kv_indptr[b + 1]) of caches (num_pages, 1, 512) and (num_pages, 1, 64).
//
// Sixteen heads are an eighth of the 128 rows of an MMA, so the products are taken transposed: the rows are
// TOKENS and the 16 columns are heads, and no tensor work is spent on rows that do not exist.
//
//   S^T = K Q^T   A = cache chunk (64 gathered token rows x 64 of the 576 columns, K-major, 128-byte swizzle),
//                 B = the same 64 columns of Q (16 head rows, K-major), D = S^T in tensor memory, M = 64: token
//                 16 q + i sits in lane 32 q + i, column = head (two buffers of 16 columns)
//   O^T += V^T P^T  A = the same cache chunks read MN-major (a K-major chunk of token rows x 128 bytes is byte
//                 for byte the MN-major operand with the latent columns as M and the tokens as K): 128 latent
//                 columns per MMA = two neighbouring chunks, B = P^T (16 head rows x 64 tokens, K-major,
//                 written by the softmax warps), D = O^T in tensor memory: lane = latent column within a block
//                 of 128, four blocks of 16 head columns
//
// A 64-token tile is 72 KB and is fetched once: its eight latent chunks sit in four 16 KB slots of a ring of
// eleven from the score product until the value product of their block has completed; the position chunks
// have two slots of their own, released after the score product. The ring holds the tile whose value product
// runs, the tile whose scores are in the softmax, and most of the tile after that. Two warps issue MMAs side by
// side - one the score products, one the value products, ordered only by the barriers between them (S^T ->
// softmax -> P^T) - because one warp issues an MMA of this size every ~55 clocks, which for the 52 MMAs of a tile
// is as long as the tile's bytes take to arrive. MMAs are issued under elect.sync with descriptors built from
// templates: with one provably active thread the operands stay in uniform registers (measured: an instruction
// every ~40 clocks, against ~90 under `lane == 0` with descriptors assembled per instruction).
//
// The softmax keeps one reference maximum per head for the whole CTA and rescales O^T only when a score outgrows
// it by more than 2^8 (exact). Whether that happened is one vote per warp and tile; the sixteen tile maxima are
// reduced and exchanged only on a piece's first tile and when the vote fires.
//
// Work split: the 64-token tiles of all requests form one stream that is cut evenly over the persistent CTAs
// (one per SM). A request that spans CTAs leaves unnormalised partials (O, m, l) in the workspace and the last
// CTA to arrive combines them after its own tiles with all of its threads (the slots and counters are those of
// the warp-MMA kernel of mla_decode.cu).
//
// Warp roles: 0 and 3 = Q staging (registers -> swizzled shared memory, prefetched a piece ahead), 1 = score-MMA
// issuer and tensor-memory owner, 2 = value-MMA issuer, 4..7 = softmax / epilogue (lanes 0..15 of a warp = 16
// tokens for S^T; thread = latent column for O^T), 8..15 = row gather (16-byte cp.async, eight lanes per 128-byte
// line; eight warps because what an SM keeps in flight is bounded per issuing warp). All warps combine.
//
// Reference semantics: python/cleave/dynamic/reference.py:282-320; replaces the kernel of
// python/cleave/dynamic/paging/builders/mla.py:220 (tests/graph/handwritten/expected_kernels/
// mla_paged_decode_h16_ckv512_kpe64_ps1.py).

#include "common.cuh"
#include "stream_walk.cuh"

#include <type_traits>

namespace cb200 {
namespace mlapd {

constexpr int kCkv = 512, kKpe = 64;
constexpr int kTile = 64;                     // tokens per tile = rows of a score MMA
constexpr int kHeads = 16;                    // MMA columns (heads past the operator's count are zero rows of Q)
constexpr int kChunkBytes = kTile * 128;      // 64 columns of 64 tokens
constexpr int kPairBytes = 2 * kChunkBytes;   // 128 latent columns: one value block
constexpr int kPairSlots = 11;
constexpr int kKpeSlots = 2;
constexpr int kQChunkBytes = kHeads * 128;    // 64 columns of the 16 Q rows
constexpr int kQBytes = 9 * kQChunkBytes;
constexpr int kPBytes = kQChunkBytes;         // 16 head rows x 64 tokens
constexpr int kExchBytes = 1024;              // 2 x 4 x 16 tile maxima, 4 x 16 row sums, 2 x 4 votes
constexpr int kBarBytes = 512;
constexpr int kFixedBytes = kPairSlots * kPairBytes + kKpeSlots * kChunkBytes + kQBytes + 2 * kPBytes + kExchBytes + kBarBytes;
constexpr int kThreads = 16 * 32;
constexpr int kGatherThreads = 8 * 32;        // warps 8..15
constexpr int kSoftmaxThreads = 128;
constexpr int kPieceUnits = 2;                // what a request's start and end cost a CTA, in tiles (the stream is cut by cost)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;      // log2 units
constexpr uint32_t kColS = 0, kColO = 32;     // tensor-memory columns: S^T 0 | S^T 1 | O^T blocks 0..3
constexpr int kSlotFloats = kHeads * kCkv + 2 * kHeads;  // partial O, m, l (the warp-MMA kernel's slot)

struct Params {
  const void* q_nope;
  const void* q_pe;
  const void* ckv;
  const void* kpe;
  const int* kv_indptr;
  const int* kv_indices;
  void* out;
  float* lse;
  int* status;
  int* counters;
  float* partials;
  int batch, heads, num_pages, n_idx;
  float scale_log2;
};

// Token range of a request, clipped to the n_idx entries kv_indices holds.
__device__ __forceinline__ int req_base(const Params& p, int b) { return min(max(p.kv_indptr[b], 0), p.n_idx); }
__device__ __forceinline__ int req_len(const Params& p, int b) {
  return max(min(p.kv_indptr[b + 1], p.n_idx) - req_base(p, b), 0);
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Warp maximum of a float through the integer reduction unit (order-preserving map to signed integers).
__device__ __forceinline__ float warp_max(float x) {
  int i = __float_as_int(x);
  i ^= (i >> 31) & 0x7fffffff;
  i = __reduce_max_sync(0xffffffffu, i);
  i ^= (i >> 31) & 0x7fffffff;
  return __int_as_float(i);
}

template <typename T>
__device__ __forceinline__ unsigned short to16(float x) {
  return static_cast<unsigned short>(pack2<T>(x, 0.f) & 0xffffu);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1) mla_paged_tc_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* pair_smem = smem;
  uint8_t* kpe_smem = pair_smem + kPairSlots * kPairBytes;
  uint8_t* q_smem = kpe_smem + kKpeSlots * kChunkBytes;
  uint8_t* p_smem = q_smem + kQBytes;
  float* max_exch = reinterpret_cast<float*>(p_smem + 2 * kPBytes);  // [2][4][16]
  float* sum_exch = max_exch + 2 * 4 * kHeads;                       // [4][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(max_exch) + kExchBytes);
  uint64_t* pair_full = bars;                      // [11] gathered rows of a slot have landed (128 gather threads)
  uint64_t* pair_empty = pair_full + kPairSlots;   // [11] the value MMAs of the block have read the slot
  uint64_t* kpe_full = pair_empty + kPairSlots;    // [2]
  uint64_t* kpe_empty = kpe_full + kKpeSlots;      // [2] the score MMAs have read the position chunk
  uint64_t* q_full = kpe_empty + kKpeSlots;        // Q of the piece is staged
  uint64_t* q_free = q_full + 1;                   // the last score MMA of the piece has read Q
  uint64_t* s_full = q_free + 1;                   // [2] S^T complete
  uint64_t* p_full = s_full + 2;                   // [2] P^T stored (and O^T rescaled if needed)
  uint64_t* pv_done = p_full + 2;                  // [2] the value MMAs of a tile have completed
  uint64_t* o_free = pv_done + 2;                  // the epilogue has read O^T
  uint64_t* merge_bar = o_free + 1;                // partials of a split request have landed in the tile slots
  uint64_t* part_ready = merge_bar + 1;            // the softmax warps have stored a piece's partial
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(part_ready + 1);
  int* pending = reinterpret_cast<int*>(tmem_holder + 2);  // [0] count, then (request, first CTA, last CTA): at most two
  int* P = reinterpret_cast<int*>(smem + kFixedBytes);  // tile prefix per request

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // The launch carries the programmatic-serialization attribute: this CTA may be scheduled while the kernel before
  // it in the stream still drains. Barriers and tensor memory are set up first; nothing that kernel may have
  // written (Q, the caches, the page table, the workspace) is touched before pdl_wait().
  if (tid == 0) {
    for (int s = 0; s < kPairSlots; ++s) {
      mbar_init(&pair_full[s], kGatherThreads);
      mbar_init(&pair_empty[s], 1);
    }
    for (int s = 0; s < kKpeSlots; ++s) {
      mbar_init(&kpe_full[s], kGatherThreads);
      mbar_init(&kpe_empty[s], 1);
    }
    mbar_init(q_full, 2);
    mbar_init(q_free, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(o_free, 4);
    mbar_init(merge_bar, 1);
    mbar_init(part_ready, 4);
    mbar_fence_init();
    pending[0] = 0;
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 128);
    tmem_relinquish();
  }
  pdl_wait();
  pdl_launch_dependents();  // the next kernel's CTAs may take SMs as this grid's CTAs retire
  // ---- tile prefix over requests (every CTA computes the same table): per-thread counts, one warp scans them
  {
    int* scratch = reinterpret_cast<int*>(p_smem);  // free until the first tile
    const int per = ceil_div(p.batch, kThreads);
    const int i0 = min(tid * per, p.batch), i1 = min(i0 + per, p.batch);
    int sum = 0;
    for (int i = i0; i < i1; ++i) sum += Walker::units(ceil_div(req_len(p, i), kTile), kPieceUnits);
    scratch[tid] = sum;
    __syncthreads();
    if (warp == 0) {
      constexpr int kPerLane = kThreads / 32;
      int loc[kPerLane], mine = 0;
#pragma unroll
      for (int k = 0; k < kPerLane; ++k) { loc[k] = scratch[lane * kPerLane + k]; mine += loc[k]; }
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int run = incl - mine;
#pragma unroll
      for (int k = 0; k < kPerLane; ++k) { scratch[lane * kPerLane + k] = run; run += loc[k]; }
      if (lane == 31) P[p.batch] = incl;
    }
    __syncthreads();
    int run = scratch[tid];
    for (int i = i0; i < i1; ++i) {
      P[i] = run;
      run += Walker::units(ceil_div(req_len(p, i), kTile), kPieceUnits);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  const int total = P[p.batch];
  const int G = gridDim.x;
  const int span = total > 0 ? ceil_div(total, G) : 1;
  const int u0 = min(static_cast<int>(blockIdx.x) * span, total);
  const int u1 = min(u0 + span, total);
  const Walker walker{P, p.batch, 1, 0, kPieceUnits};
  T* outp = reinterpret_cast<T*>(p.out);

  if (warp == 0 || warp == 3) {
    // ================================================================ Q of every piece: 16 rows x 72 16-byte pieces,
    // half of them per warp so that each warp's share is one batch of loads in registers
    const T* qn = reinterpret_cast<const T*>(p.q_nope);
    const T* qp = reinterpret_cast<const T*>(p.q_pe);
    constexpr int kPiecesPerRow = (kCkv + kKpe) / 8;                // 72
    constexpr int kPerLane = kHeads * kPiecesPerRow / 32;           // 36
    // Warp 3 also publishes the partials of pieces that are not whole requests: the softmax warps only store them
    // and arrive on a barrier; the fence that makes them visible to other SMs, the arrival on the request's counter
    // and the note for the combine happen here, off the softmax warps' path (a fence costs them about a
    // microsecond per piece otherwise).
    int n_partial = 0;
    auto publish = [&](const Piece& pp, int u_at) {
      const bool whole = u_at == pp.unit0 && pp.count == pp.n_tiles;
      if (whole) return;
      mbar_wait(part_ready, n_partial & 1, p.status, kFaultTmemBarrier);
      ++n_partial;
      if (lane == 0) {
        __threadfence();
        const int c_first = pp.unit0 / span, c_last = (pp.unit0 + pp.n_tiles - 1) / span;
        if (atomicAdd(p.counters + pp.b, 1) == c_last - c_first) {
          int* e = pending + 1 + 3 * pending[0];
          e[0] = pp.b;
          e[1] = c_first;
          e[2] = c_last;
          pending[0] += 1;
        }
      }
      __syncwarp();
    };
    Piece prev{};
    int prev_u = 0;
    int piece_idx = 0;
    for (int u = u0; u < u1; ++piece_idx) {
      const Piece pc = walker.at(u, u1);
      if (pc.count == 0) break;  // the share ends in front of the next request's tiles
      constexpr int kHalf = kPerLane / 2;
      const int k0 = warp == 0 ? 0 : kHalf;
      uint4 v[kHalf];
#pragma unroll
      for (int k = 0; k < kHalf; ++k) {
        const int i = lane + 32 * (k0 + k), row = i / kPiecesPerRow, c = i - row * kPiecesPerRow;
        v[k] = make_uint4(0u, 0u, 0u, 0u);
        if (row < p.heads) {
          const size_t bh = static_cast<size_t>(pc.b) * p.heads + row;
          v[k] = c < kCkv / 8 ? __ldg(reinterpret_cast<const uint4*>(qn + bh * kCkv + c * 8))
                              : __ldg(reinterpret_cast<const uint4*>(qp + bh * kKpe + (c - kCkv / 8) * 8));
        }
      }
      // the score MMAs of the piece before must have read the buffer
      if (piece_idx > 0) mbar_wait(q_free, (piece_idx - 1) & 1, p.status, kFaultMmaBarrier);
#pragma unroll
      for (int k = 0; k < kHalf; ++k) {
        const int i = lane + 32 * (k0 + k), row = i / kPiecesPerRow, c = i - row * kPiecesPerRow;
        *reinterpret_cast<uint4*>(q_smem + (c >> 3) * kQChunkBytes + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v[k];
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
      if (warp == 3 && piece_idx > 0) publish(prev, prev_u);
      prev = pc;
      prev_u = u;
      u += pc.count;
    }
    if (warp == 3 && piece_idx > 0) publish(prev, prev_u);
    // Requests without any live token: out = 0, lse = -inf (warp 0, idle once Q is staged).
    for (int b = blockIdx.x; warp == 0 && b < p.batch; b += G) {
      if (P[b + 1] - P[b] != 0) continue;
      for (int i = lane; i < p.heads * kCkv; i += 32) outp[static_cast<size_t>(b) * p.heads * kCkv + i] = T(0.f);
      if (p.lse)
        for (int i = lane; i < p.heads; i += 32) p.lse[static_cast<size_t>(b) * p.heads + i] = -INFINITY;
    }
  } else if (warp >= 8) {
    // ================================================================ row gather
    // Eight lanes copy the eight 16-byte pieces of one row's 64-column chunk, so a warp instruction moves four
    // whole 128-byte lines; the 256 threads cover 32 rows per round, two rounds per chunk. Eight warps, not four:
    // what an SM can have in flight is bounded per issuing warp (measured with a gather-only kernel over random
    // 1 KB rows: 4.0 TB/s with four warps per SM whatever the depth, 6.0 with eight, 6.6 with twelve).
    const int gtid = tid - 8 * 32, piece = gtid & 7, r_in = gtid >> 3;
    const T* ckv = reinterpret_cast<const T*>(p.ckv);
    const T* kpe = reinterpret_cast<const T*>(p.kpe);
    int g = 0;
    for (int u = u0; u < u1;) {
      const Piece pc = walker.at(u, u1);
      if (pc.count == 0) break;  // the share ends in front of the next request's tiles
      const int valid = req_len(p, pc.b), base = req_base(p, pc.b);
      auto page_of = [&](int tok) {
        return min(max(__ldg(p.kv_indices + base + min(tok, valid - 1)), 0), p.num_pages - 1);
      };
      int pg[2], pg_next[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) pg_next[rr] = page_of(pc.tile0 * kTile + rr * 32 + r_in);
      for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t, ++g) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) pg[rr] = pg_next[rr];
        if (t + 1 < pc.tile0 + pc.count) {  // one tile ahead: the latency of the index loads stays off the stream
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) pg_next[rr] = page_of((t + 1) * kTile + rr * 32 + r_in);
        }
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          const int n = 4 * g + j, slot = n % kPairSlots, use = n / kPairSlots;
          mbar_wait(&pair_empty[slot], (use & 1) ^ 1, p.status, kFaultEmptyBarrier);
          const uint32_t dst = smem_u32(pair_smem + slot * kPairBytes);
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
              const int row = rr * 32 + r_in;
              const T* src = ckv + static_cast<long long>(pg[rr]) * kCkv + (2 * j + cc) * 64 + piece * 8;
              const uint32_t o = cc * kChunkBytes + row * 128 + ((piece ^ (row & 7)) << 4);
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + o), "l"(src) : "memory");
            }
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&pair_full[slot])) : "memory");
        }
        {
          const int ks = g % kKpeSlots, use = g / kKpeSlots;
          mbar_wait(&kpe_empty[ks], (use & 1) ^ 1, p.status, kFaultEmptyBarrier);
          const uint32_t dst = smem_u32(kpe_smem + ks * kChunkBytes);
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int row = rr * 32 + r_in;
            const T* src = kpe + static_cast<long long>(pg[rr]) * kKpe + piece * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + row * 128 + ((piece ^ (row & 7)) << 4)),
                         "l"(src) : "memory");
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&kpe_full[ks])) : "memory");
        }
      }
      u += pc.count;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1 || warp == 2) {
    // ================================================================ MMA issuers: warp 1 the score products, warp 2
    // the value products. One warp issues an MMA of this size every ~55 clocks, which for the 52 MMAs of a tile
    // is as long as the tile's bytes take to arrive; two warps issue side by side. The products of the two warps
    // are ordered by the barriers between them (S^T -> softmax -> P^T), never by issue order.
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t idesc_s = umma_idesc(kBf16, /*b_mn_major=*/false, kTile, kHeads);             // 64 x 16
    constexpr uint32_t idesc_pv = umma_idesc(kBf16, /*b_mn_major=*/false, 128, kHeads) | (1u << 15);  // A MN-major
    const uint32_t pair_addr = smem_u32(pair_smem), kpe_addr = smem_u32(kpe_smem), q_addr = smem_u32(q_smem),
                   p_addr = smem_u32(p_smem);
    // Descriptor templates (address field zero); an operand's descriptor is the template with (address >> 4) in
    // its low bits.
    const uint64_t desc_k = umma_smem_desc(0, 16, 8 * 128);            // K-major rows of 128 bytes
    const uint64_t desc_mn = umma_smem_desc(0, kChunkBytes, 8 * 128);  // MN-major: 64-column chunks kChunkBytes apart
    int g = 0, piece_idx = 0;
    if (warp == 1) {
      for (int u = u0; u < u1; ++piece_idx) {
        const Piece pc = walker.at(u, u1);
        if (pc.count == 0) break;
      if (pc.count == 0) break;  // the share ends in front of the next request's tiles
        mbar_wait(q_full, piece_idx & 1, p.status, kFaultFullBarrier);
        tc_fence_after();
        for (int i = 0; i < pc.count; ++i, ++g) {
          // S^T buffer g & 1 was last read by the softmax of tile g - 2
          if (g >= 2) mbar_wait(&p_full[g & 1], ((g - 2) >> 1) & 1, p.status, kFaultTmemBarrier);
          tc_fence_after();
          const uint32_t d = tmem_base + kColS + (g & 1) * kHeads;
#pragma unroll 1
          for (int j = 0; j < 4; ++j) {
            const int n = 4 * g + j, slot = n % kPairSlots, use = n / kPairSlots;
            mbar_wait(&pair_full[slot], use & 1, p.status, kFaultFullBarrier);
            tc_fence_after();
            if (elect_one()) {
              const uint32_t a0 = (pair_addr + slot * kPairBytes) >> 4, b0 = (q_addr + 2 * j * kQChunkBytes) >> 4;
#pragma unroll
              for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                  umma_f16(d, desc_k | (a0 + cc * (kChunkBytes >> 4) + kk * 2), desc_k | (b0 + cc * (kQChunkBytes >> 4) + kk * 2),
                           idesc_s, (j > 0 || cc > 0 || kk > 0) ? 1u : 0u);
              }
            }
            __syncwarp();
          }
          const int ks = g % kKpeSlots, use = g / kKpeSlots;
          mbar_wait(&kpe_full[ks], use & 1, p.status, kFaultFullBarrier);
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a0 = (kpe_addr + ks * kChunkBytes) >> 4, b0 = (q_addr + 8 * kQChunkBytes) >> 4;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16(d, desc_k | (a0 + kk * 2), desc_k | (b0 + kk * 2), idesc_s, 1u);
            umma_commit(&kpe_empty[ks]);
            umma_commit(&s_full[g & 1]);
            if (i + 1 == pc.count) umma_commit(q_free);
          }
          __syncwarp();
        }
        u += pc.count;
      }
    } else {
      for (int u = u0; u < u1; ++piece_idx) {
        const Piece pc = walker.at(u, u1);
        if (pc.count == 0) break;
      if (pc.count == 0) break;  // the share ends in front of the next request's tiles
        for (int i = 0; i < pc.count; ++i, ++g) {
          mbar_wait(&p_full[g & 1], (g >> 1) & 1, p.status, kFaultTmemBarrier);
          // O^T of the piece before must have been read before its columns are overwritten
          if (i == 0 && piece_idx > 0) mbar_wait(o_free, (piece_idx - 1) & 1, p.status, kFaultTmemBarrier);
          tc_fence_after();
          if (elect_one()) {
            const uint32_t b0 = (p_addr + (g & 1) * kPBytes) >> 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int n = 4 * g + j, slot = n % kPairSlots;
              const uint32_t a0 = (pair_addr + slot * kPairBytes) >> 4;
#pragma unroll
              for (int ks = 0; ks < kTile / 16; ++ks) {
                // A: MN-major, 16 token rows of 128 bytes per step; B: 16 tokens of the 16 head rows of P^T
                umma_f16(tmem_base + kColO + j * kHeads, desc_mn | (a0 + ks * (16 * 128 >> 4)), desc_k | (b0 + ks * 2),
                         idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
              }
              umma_commit(&pair_empty[slot]);
            }
            umma_commit(&pv_done[g & 1]);
          }
          __syncwarp();
        }
        u += pc.count;
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ================================================================ softmax / epilogue / combine (warps 4..7)
    const int quarter = warp & 3;
    const int col = quarter * 32 + lane;      // latent column of the block (O^T) = TMEM lane
    const int tk = quarter * 16 + lane;       // token of the tile (S^T), lanes 0..15 only
    const bool has_token = lane < 16;
    const int st = tid - 4 * 32;              // 0..127 inside the group
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    int g = 0, piece_idx = 0;
    for (int u = u0; u < u1; ++piece_idx) {
      const Piece pc = walker.at(u, u1);
      if (pc.count == 0) break;  // the share ends in front of the next request's tiles
      const int valid = req_len(p, pc.b);
      float m_ref[kHeads], l_part[kHeads];
#pragma unroll
      for (int h = 0; h < kHeads; ++h) { m_ref[h] = 0.f; l_part[h] = 0.f; }
      for (int i = 0; i < pc.count; ++i, ++g) {
        const int sb = g & 1;
        const bool live = has_token && (pc.tile0 + i) * kTile + tk < valid;
        mbar_wait(&s_full[sb], (g >> 1) & 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
        uint32_t sr[kHeads];
        tmem_ld_32x16(tmem_base + lane_field + kColS + sb * kHeads, sr);
        tmem_ld_wait();
        float s[kHeads];
        bool over = false;  // some score of this thread exceeds its head's reference by more than the threshold
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
          s[h] = live ? __uint_as_float(sr[h]) * p.scale_log2 : -INFINITY;
          over |= s[h] > m_ref[h] + kRescaleThreshold;
        }
        // The reference maxima move only on a piece's first tile and when a score outgrows them by 2^8 (rare), so
        // the tile-wide maxima are not formed every tile: the four warps exchange one vote, and only when it fires
        // do they reduce and exchange the sixteen maxima.
        int* vote = reinterpret_cast<int*>(max_exch + 2 * 4 * kHeads + 4 * kHeads) + sb * 4;  // [2][4] behind the sums
        const bool warp_over = i == 0 || __any_sync(0xffffffffu, over);
        if (lane == 0) vote[quarter] = warp_over ? 1 : 0;
        named_bar_sync(1, kSoftmaxThreads);
        const int4 votes = *reinterpret_cast<const int4*>(vote);
        if ((votes.x | votes.y | votes.z | votes.w) != 0) {  // the same decision in all 128 threads
          float4* mx4 = reinterpret_cast<float4*>(max_exch + (sb * 4 + quarter) * kHeads);
          {
            float wm[kHeads];
#pragma unroll
            for (int h = 0; h < kHeads; ++h) wm[h] = warp_max(s[h]);
            if (lane == 0) {
#pragma unroll
              for (int h = 0; h < kHeads; h += 4) mx4[h >> 2] = make_float4(wm[h], wm[h + 1], wm[h + 2], wm[h + 3]);
            }
          }
          named_bar_sync(1, kSoftmaxThreads);
          float mt[kHeads];
          {
            const float4* all = reinterpret_cast<const float4*>(max_exch + sb * 4 * kHeads);
#pragma unroll
            for (int h4 = 0; h4 < kHeads / 4; ++h4) {
              float4 a = all[h4];
#pragma unroll
              for (int w = 1; w < 4; ++w) {
                const float4 b = all[w * (kHeads / 4) + h4];
                a.x = fmaxf(a.x, b.x); a.y = fmaxf(a.y, b.y); a.z = fmaxf(a.z, b.z); a.w = fmaxf(a.w, b.w);
              }
              mt[4 * h4] = a.x; mt[4 * h4 + 1] = a.y; mt[4 * h4 + 2] = a.z; mt[4 * h4 + 3] = a.w;
            }
          }
          if (i == 0) {
#pragma unroll
            for (int h = 0; h < kHeads; ++h) m_ref[h] = mt[h] == -INFINITY ? 0.f : mt[h];
          } else {
            float alpha[kHeads];
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
              const bool up = mt[h] > m_ref[h] + kRescaleThreshold;
              alpha[h] = up ? fast_exp2(m_ref[h] - mt[h]) : 1.f;
              m_ref[h] = up ? mt[h] : m_ref[h];
              l_part[h] *= alpha[h];
            }
            // O^T may only be touched when no value MMA is in flight: tile g - 1 is the last one issued
            mbar_wait(&pv_done[sb ^ 1], ((g - 1) >> 1) & 1, p.status, kFaultMmaBarrier);
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 4; ++j) {
              uint32_t o[kHeads];
              tmem_ld_32x16(tmem_base + lane_field + kColO + j * kHeads, o);
              tmem_ld_wait();
#pragma unroll
              for (int h = 0; h < kHeads; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
              tmem_st_32x16(tmem_base + lane_field + kColO + j * kHeads, o);
            }
            tmem_st_wait();
          }
        }
        // the value MMAs of the tile two back have read the P^T buffer this tile's goes to
        if (i >= 2) mbar_wait(&pv_done[sb], ((g - 2) >> 1) & 1, p.status, kFaultMmaBarrier);
        if (has_token) {
          uint8_t* prow = p_smem + sb * kPBytes + (tk & 7) * 2;
          const int piece8 = tk >> 3;
#pragma unroll
          for (int h = 0; h < kHeads; ++h) {
            const float pv = fast_exp2(s[h] - m_ref[h]);  // exp2(-inf) = 0 for tokens past the end
            l_part[h] += pv;
            *reinterpret_cast<unsigned short*>(prow + h * 128 + ((piece8 ^ (h & 7)) << 4)) = to16<T>(pv);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[sb]);
      }
      // ---- the piece is done: row sums over all tokens, then O^T out of tensor memory
#pragma unroll
      for (int h = 0; h < kHeads; ++h) {
        float l = l_part[h];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);  // lanes 16..31 hold zeros
        l_part[h] = l;
      }
      if (lane == 0) {
        float4* dst = reinterpret_cast<float4*>(sum_exch + quarter * kHeads);
#pragma unroll
        for (int h = 0; h < kHeads; h += 4) dst[h >> 2] = make_float4(l_part[h], l_part[h + 1], l_part[h + 2], l_part[h + 3]);
      }
      named_bar_sync(1, kSoftmaxThreads);
      float L[kHeads];
#pragma unroll
      for (int h = 0; h < kHeads; ++h)
        L[h] = sum_exch[h] + sum_exch[kHeads + h] + sum_exch[2 * kHeads + h] + sum_exch[3 * kHeads + h];
      const int g_last = g - 1;
      mbar_wait(&pv_done[g_last & 1], (g_last >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();

      const size_t bh = static_cast<size_t>(pc.b) * p.heads;
      const bool starts_here = (u == pc.unit0);
      const bool whole = starts_here && pc.count == pc.n_tiles;
      float* slot = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * kSlotFloats;
      if (whole) {
        float inv[kHeads];
#pragma unroll
        for (int h = 0; h < kHeads; ++h) inv[h] = L[h] > 0.f ? 1.f / L[h] : 0.f;
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          uint32_t o[kHeads];
          tmem_ld_32x16(tmem_base + lane_field + kColO + j * kHeads, o);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < kHeads; ++h)
            if (h < p.heads) outp[(bh + h) * kCkv + j * 128 + col] = T(__uint_as_float(o[h]) * inv[h]);
        }
        if (p.lse) {
#pragma unroll
          for (int h = 0; h < kHeads; ++h)
            if (st == h && h < p.heads) p.lse[bh + h] = L[h] > 0.f ? m_ref[h] + fast_log2(L[h]) : -INFINITY;
        }
      } else {
        // leave a partial (unnormalised O, m, l); the last CTA of the request to arrive combines
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          uint32_t o[kHeads];
          tmem_ld_32x16(tmem_base + lane_field + kColO + j * kHeads, o);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < kHeads; ++h) slot[h * kCkv + j * 128 + col] = __uint_as_float(o[h]);
        }
#pragma unroll
        for (int h = 0; h < kHeads; ++h)
          if (st == h) {
            slot[kHeads * kCkv + h] = m_ref[h];
            slot[kHeads * kCkv + kHeads + h] = L[h];
          }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);  // the next piece's value MMAs may overwrite O^T

      if (!whole) {  // the partial is stored; warp 3 publishes it (fence, counter, note for the combine)
        __syncwarp();
        if (lane == 0) mbar_arrive(part_ready);
      }
      u += pc.count;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }

  // ---- combine the requests this CTA was the last to arrive at (at most two: the one that continues from the CTA
  // before and the one that continues into the next). The tile slots are free now: the partials come into them as
  // bulk copies, five at a time (one L2 round trip at the SM's full pull rate, no registers in between), and all
  // threads combine from shared memory. An item is four neighbouring latent columns of one head.
  const int n_pending = pending[0];
  uint32_t merge_phase = 0;
  for (int k = 0; k < n_pending; ++k) {
    const int b = pending[1 + 3 * k], c_first = pending[2 + 3 * k], c_last = pending[3 + 3 * k];
    const size_t bh = static_cast<size_t>(b) * p.heads;
    constexpr int kItems = kHeads * (kCkv / 4);  // 2048
    constexpr int kPerThread = kItems / kThreads;
    static_assert(kItems % kThreads == 0, "items must divide evenly over the threads");
    constexpr int kSlotBytes = kSlotFloats * 4;
    constexpr int kMergeSlots = 5;
    static_assert(kMergeSlots * kSlotBytes <= kPairSlots * kPairBytes && kSlotBytes % 16 == 0, "partials must fit the tile slots");
    float M[kPerThread], Lsum[kPerThread];
    float4 acc[kPerThread];
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      M[q] = -INFINITY;
      Lsum[q] = 0.f;
      acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll 1
    for (int cta0 = c_first; cta0 <= c_last; cta0 += kMergeSlots) {
      const int n = min(kMergeSlots, c_last - cta0 + 1);
      __syncthreads();  // the slots are no longer read (tiles, or the chunk before)
      if (tid == 0) {
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");  // partials were written with ordinary stores; the copy engine reads them
        mbar_arrive_expect_tx(merge_bar, static_cast<uint32_t>(n) * kSlotBytes);
        for (int i = 0; i < n; ++i) {
          const int cta = cta0 + i;
          bulk_load_1d(pair_smem + i * kSlotBytes,
                       p.partials + (static_cast<size_t>(cta) * 2 + (cta == c_first ? 1 : 0)) * kSlotFloats, kSlotBytes, merge_bar);
        }
      }
      mbar_wait(merge_bar, merge_phase, p.status, kFaultFullBarrier);
      merge_phase ^= 1;
      for (int i = 0; i < n; ++i) {
        const float* src = reinterpret_cast<const float*>(pair_smem + i * kSlotBytes);
#pragma unroll
        for (int q = 0; q < kPerThread; ++q) {
          const int item = q * kThreads + tid, head = item / (kCkv / 4);
          const float4 x = *reinterpret_cast<const float4*>(src + item * 4);  // item = head * 128 + column group
          const float mi = src[kHeads * kCkv + head], li = src[kHeads * kCkv + kHeads + head];
          const float mn = fmaxf(M[q], mi), mu = mn == -INFINITY ? 0.f : mn;
          const float a = fast_exp2(M[q] - mu), w = fast_exp2(mi - mu);
          Lsum[q] = a * Lsum[q] + w * li;
          M[q] = mn;
          acc[q].x = a * acc[q].x + w * x.x;
          acc[q].y = a * acc[q].y + w * x.y;
          acc[q].z = a * acc[q].z + w * x.z;
          acc[q].w = a * acc[q].w + w * x.w;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < kPerThread; ++q) {
      const int item = q * kThreads + tid, head = item / (kCkv / 4), c4 = item - head * (kCkv / 4);
      if (head < p.heads) {
        const float inv = Lsum[q] > 0.f ? 1.f / Lsum[q] : 0.f;
        uint2 o;
        o.x = pack2<T>(acc[q].x * inv, acc[q].y * inv);
        o.y = pack2<T>(acc[q].z * inv, acc[q].w * inv);
        *reinterpret_cast<uint2*>(outp + (bh + head) * kCkv + c4 * 4) = o;
        if (p.lse && c4 == 0) p.lse[bh + head] = Lsum[q] > 0.f ? M[q] + fast_log2(Lsum[q]) : -INFINITY;
      }
    }
    if (tid == 0) p.counters[b] = 0;  // ready for the next launch
  }
}

}  // namespace mlapd

// ------------------------------------------------------------------------------------- host side
// Whether the paged form of the arguments can run on the kernel above: at most 16 heads, ranges given by
// kv_indptr, and a tile prefix table that fits beside the tile slots in shared memory.
bool mla_paged_tc_supported(const cb200_mla_decode_args* a) {
  using namespace mlapd;
  if (!a || !a->kv_indptr || a->kv_lens || a->kv_start) return false;
  if (a->page_size != 1 || a->ckv_dim != kCkv || a->kpe_dim != kKpe) return false;
  if (a->num_heads < 1 || a->num_heads > kHeads) return false;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return false;
  const long long smem = static_cast<long long>(kFixedBytes) + (static_cast<long long>(a->batch) + 1) * 4 + 1024 + 16;
  return smem <= 227 * 1024;
}

int launch_mla_paged_tc(const cb200_mla_decode_args* a, int* status, float* partials, int* counters, int grid,
                        cudaStream_t stream) {
  using namespace mlapd;
  Params p{};
  p.q_nope = a->q_nope;
  p.q_pe = a->q_pe;
  p.ckv = a->ckv_cache;
  p.kpe = a->kpe_cache;
  p.kv_indptr = a->kv_indptr;
  p.kv_indices = a->kv_indices;
  p.out = a->out;
  p.lse = a->lse;
  p.status = status;
  p.counters = counters;
  p.partials = partials;
  p.batch = a->batch;
  p.heads = a->num_heads;
  p.num_pages = a->num_pages;
  p.n_idx = a->num_kv_indices;
  p.scale_log2 = a->sm_scale * kLog2e;
  const int smem = kFixedBytes + (a->batch + 1) * 4 + 1024 + 16;
  static bool configured[64] = {false};
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    CB200_CUDA_TRY(cudaFuncSetAttribute(mla_paged_tc_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    CB200_CUDA_TRY(cudaFuncSetAttribute(mla_paged_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev < 64) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // the grid may be scheduled while the preceding kernel of the stream drains; it waits (griddepcontrol.wait)
  // before its first global access
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (a->dtype == CB200_F16) CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, mla_paged_tc_kernel<__half>, p));
  else CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, mla_paged_tc_kernel<__nv_bfloat16>, p));
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

}  // namespace cb200
