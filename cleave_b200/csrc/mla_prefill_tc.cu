// Paged causal MLA prefill (absorbed latent) on the tcgen05 tensor cores: a query-tile kernel.
//
//   S = (Q_nope CKV^T + Q_pe KPE^T) * scale under the end-aligned causal mask, O = softmax(S) CKV
//   q_nope (total_q, H, 512), q_pe (total_q, H, 64); caches (num_pages, 1, 512 / 64), one token per page;
//   request r owns the query rows qo_indptr[r] .. qo_indptr[r + 1] and the keys
//   kv_indices[kv_indptr[r] .. kv_indptr[r + 1]).
//
// The 128 rows of every MMA are (query token, head) pairs: a block of 128 / H consecutive query tokens of
// one request times its H heads. Those rows are contiguous in q_nope / q_pe viewed as (total_q * H, 512 / 64)
// matrices, so a Q chunk is one TMA box; each row has its own causal limit. An item is (request, query block);
// two CTAs work on an item, one per half of the 512 output columns (blockIdx.x & 1), each computing the
// scores it needs itself - the score product is 576 / 512 of the value product, and repeating it costs less
// than moving P between SMs or holding a 128 x 512 fp32 accumulator, which alone would fill tensor memory.
//
//   S = Q K^T    A = Q chunk, B = cache chunk (64 of the 576 columns x 128 tokens), both K-major in shared
//                memory; nine chunk pairs stream through one ring per KV tile (the Q chunks by TMA, the cache
//                rows gathered through kv_indices by four warps with 16-byte cp.async into the 128-byte
//                swizzled layout); D = S in tensor memory, two buffers of 128 columns
//   O += P V     A = P (16-bit pairs the softmax warps store over the first 64 columns of the S buffer they
//                just read), B = the CTA's 256 latent columns of the same 128 tokens, D = O in tensor memory
//                (256 columns). Those columns are four of the nine score chunks, and a K-major chunk of 128
//                token rows x 128 bytes is byte for byte the MN-major value operand: the four chunks are
//                gathered into a value buffer (two buffers, one per tile in flight) instead of the ring, serve
//                the score product first and the value product afterwards, and are fetched once
// Tensor memory: S/P 0 | S/P 1 | O = 128 + 128 + 256 columns. MMAs of one thread execute in order, so the
// score product of tile j + 2, which overwrites the buffer P(j) lives in, cannot pass the value product that
// reads it. The softmax keeps a reference maximum per row and rescales O only when the running maximum grew
// by more than 2^8 (exact), as the GQA prefill kernel does.
//
// Warp roles: 0 = Q-chunk TMA producer, 1 = MMA issuer and TMEM owner, 2..5 = softmax / epilogue (thread =
// row = TMEM lane), 6..9 = cache-row gather. The tile loop is bound by what an SM can pull from L2 (the Q
// chunks are streamed again for every KV tile: Q, a tile and the accumulators do not fit on one SM together).
//
// Reference semantics: python/cleave/dynamic/reference.py:324-365; replaces
// tests/graph/handwritten/expected_kernels/mla_paged_prefill_causal_h16_ckv512_kpe64_ps1.py
// (python/cleave/dynamic/paging/builders/mla.py:393).

#include "common.cuh"

#include <cstring>
#include <type_traits>

namespace cb200 {
namespace mlapf {

constexpr int kCkv = 512, kKpe = 64;
constexpr int kChunks = (kCkv + kKpe) / 64;  // 9 score chunks of 64 columns
constexpr int kBM = 128, kBN = 128;          // rows per item, tokens per KV tile
constexpr int kDV = 256;                     // output columns per CTA
constexpr int kChunkBytes = 128 * 128;       // 128 rows x 128 bytes
constexpr int kStageBytes = 2 * kChunkBytes; // Q chunk + cache chunk
constexpr int kStages = 3;
constexpr int kVChunks = kDV / 64;           // the score chunks that are this CTA's value columns
constexpr int kVBytes = kVChunks * kChunkBytes;    // 64 KB, two buffers
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kVBytes + 1024 /*barriers*/ + 1024 /*alignment*/;
constexpr int kThreads = 10 * 32;
constexpr int kThreadsPersist = 11 * 32;     // the persistent form: one more warp hands the item numbers round
constexpr int kTicketWarp = 10;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;     // log2 units
constexpr uint32_t kColS = 0, kColO = 256;

struct Params {
  const void* ckv;
  const void* kpe;
  const int* qo_indptr;
  const int* kv_indptr;
  const int* kv_indices;
  void* out;
  float* lse;
  int* status;
  int batch, heads, qb;  // qb = 128 / heads query tokens per item
  int blocks;            // upper bound on the query blocks of the batch; an item is (block, half of the output columns)
  int num_pages, n_idx;
  float scale_log2;
};

// PERSIST = false: one CTA per item (the grid is the upper bound on the items). PERSIST = true: one CTA per SM, which
// starts on the item of its block index and takes further ones from a counter in the workspace header; every barrier
// phase and buffer parity runs on across items, so the producers and the MMA warp are on the next item while the
// softmax warps finish the current one. The second form pays for batches of many short items and costs a call with a
// single small item a microsecond (more barriers, the item ring, tensor memory taken before the item is known): the
// host picks (launch below).
template <typename T, bool PERSIST>
__global__ void __launch_bounds__(PERSIST ? kThreadsPersist : kThreads, 1)
mla_prefill_kernel(const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* v_smem = ring + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + 2 * kVBytes);
  uint64_t* k_full = bars;              // [kStages] Q chunk landed (TMA) and cache rows landed (128 gather threads)
  uint64_t* k_empty = k_full + kStages; // [kStages] the score MMAs have read the stage
  uint64_t* s_full = k_empty + kStages; // [2] S complete in tensor memory
  uint64_t* p_full = s_full + 2;        // [2] P stored (and O rescaled if needed)
  uint64_t* pv_done = p_full + 2;       // [2] the value MMAs of a tile have completed
  uint64_t* o_done = pv_done + 2;
  uint64_t* o_free = o_done + 1;        // persistent form: the epilogue has taken O out of tensor memory
  uint64_t* t_full = o_free + 1;        // [2] persistent form: an item number is in the ring
  uint64_t* t_empty = t_full + 2;       // [2] every warp has read it
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(t_empty + 2);
  volatile int* item_ring = reinterpret_cast<volatile int*>(tmem_holder + 1);  // [2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The ranges of the first 32 requests (lane = request) are fetched before anything else, so that the trip to
  // memory runs beside the barrier set-up below; the search starts from these registers.
  int pre_lo = 0, pre_hi = 0, pre_klo = 0, pre_khi = 0;
  if (lane < p.batch) {
    pre_lo = __ldg(p.qo_indptr + lane);
    pre_hi = __ldg(p.qo_indptr + lane + 1);
    pre_klo = __ldg(p.kv_indptr + lane);
    pre_khi = __ldg(p.kv_indptr + lane + 1);
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 129);  // 128 gather threads + the TMA thread's expect-tx arrival
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(o_done, 1);
    if constexpr (PERSIST) {
      mbar_init(o_free, 4);
      for (int s = 0; s < 2; ++s) {
        mbar_init(&t_full[s], 1);
        mbar_init(&t_empty[s], kTicketWarp);
      }
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_qn);
    tma_prefetch_desc(&tm_qp);
  }

  uint32_t tmem_base = 0;
  // The host's block count is an upper bound (one more per request than total_q / qb); blocks that do not exist come
  // first in the order. The persistent form takes the exact count: a sum over the request ranges, the first 32 from
  // this warp's registers, the others a few independent loads per lane.
  int n_blocks = p.blocks;
  if constexpr (PERSIST) {
    int mine = pre_hi > pre_lo ? ceil_div(pre_hi - pre_lo, p.qb) : 0;
#pragma unroll 4
    for (int rr = 32 + lane; rr < p.batch; rr += 32) {
      const int lo_r = __ldg(p.qo_indptr + rr), hi_r = __ldg(p.qo_indptr + rr + 1);
      mine += hi_r > lo_r ? ceil_div(hi_r - lo_r, p.qb) : 0;
    }
    n_blocks = __reduce_add_sync(0xffffffffu, mine);
  }
  const int n_items = 2 * n_blocks;
  int* ticket = p.status + 8;    // persistent form: items beyond the first of every CTA are dealt by this counter
  int* finished = p.status + 9;  // CTAs that are through; the last one clears both words for the next launch
  if constexpr (PERSIST) {
    if (warp == 1) {
      tmem_alloc(tmem_holder, 512);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
    if (warp == kTicketWarp) {
      // the first item of a CTA is its block index, which every warp knows; the others come from the counter, fetched
      // one item ahead and handed round through a two-slot ring
      if (lane == 0) {
        for (int k = 0;; ++k) {
          const int s = k & 1;
          mbar_wait(&t_empty[s], ((k >> 1) & 1) ^ 1, p.status, kFaultEmptyBarrier);
          const int item = n_items <= static_cast<int>(gridDim.x) ? n_items : static_cast<int>(gridDim.x) + atomicAdd(ticket, 1);
          item_ring[s] = item;
          mbar_arrive(&t_full[s]);
          if (item >= n_items) break;
        }
      }
      __syncwarp();
    }
  }
  int n_taken = 0;  // item numbers this warp has had
  int it = 0;       // items with keys this CTA has run, jt: their KV tiles (every role counts alike; 0 in the one-item form)
  int jt = 0;
  int st = 0, ph = 0;  // ring position of this warp's role
  while (warp < kTicketWarp) {
    int item = static_cast<int>(blockIdx.x);
    if constexpr (PERSIST) {
      if (n_taken > 0) {  // the ring's entry number n_taken - 1
        const int s = (n_taken - 1) & 1;
        mbar_wait(&t_full[s], ((n_taken - 1) >> 1) & 1, p.status, kFaultFullBarrier);
        item = item_ring[s];
        __syncwarp();
        if (lane == 0) mbar_arrive(&t_empty[s]);
      }
      ++n_taken;
      if (item >= n_items) break;
    }
  const int dh = item & 1;  // which half of the output columns
  // ---- which (request, query block) the item is: late blocks, which see the most keys, come first
  // (every warp searches the query offsets 32 requests at a time: lane = request, block counts scanned with shuffles)
  int t = n_blocks - 1 - (item >> 1), r = 0, lo = 0;
  int q_len = 0, kv_base_found = 0, kv_end_found = 0;
  bool found = false;
  for (int r0 = 0; r0 < p.batch && !found; r0 += 32) {
    const int rr = r0 + lane;
    int lo_r = pre_lo, hi_r = pre_hi, klo_r = pre_klo, khi_r = pre_khi;
    if (r0 > 0) {
      lo_r = rr < p.batch ? __ldg(p.qo_indptr + rr) : 0;
      hi_r = rr < p.batch ? __ldg(p.qo_indptr + rr + 1) : 0;
      klo_r = rr < p.batch ? __ldg(p.kv_indptr + rr) : 0;
      khi_r = rr < p.batch ? __ldg(p.kv_indptr + rr + 1) : 0;
    }
    const int blocks = hi_r > lo_r ? ceil_div(hi_r - lo_r, p.qb) : 0;
    int incl = blocks;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int all = __shfl_sync(0xffffffffu, incl, 31);
    if (t < all) {
      const int first = __ffs(__ballot_sync(0xffffffffu, incl > t)) - 1;
      r = r0 + first;
      t -= __shfl_sync(0xffffffffu, incl - blocks, first);
      lo = __shfl_sync(0xffffffffu, lo_r, first);
      q_len = __shfl_sync(0xffffffffu, hi_r, first) - lo;
      kv_base_found = __shfl_sync(0xffffffffu, klo_r, first);
      kv_end_found = __shfl_sync(0xffffffffu, khi_r, first);
      found = true;
    } else {
      t -= all;
    }
  }
  (void)r;
  if (!found) {  // the item count is an upper bound on the number of query blocks
    if constexpr (PERSIST) continue;
    else return;
  }
  const int q_base = lo;                 // first query token of the request
  const int q0 = t * p.qb;               // first query token of this block, inside the request
  int kv_base = kv_base_found;  // fetched beside the query offsets: one trip to memory, not two in a row
  int kv_len = kv_end_found - kv_base;
  if (kv_base < 0 || kv_base >= p.n_idx) kv_len = 0;   // the table is caller data: stay inside it
  kv_len = max(min(kv_len, p.n_idx - kv_base), 0);
  const int off = kv_len - q_len;        // end-aligned causal mask: query i sees keys <= i + off
  const int live_q = min(p.qb, q_len - q0);
  const int last_key = min(kv_len - 1, q0 + live_q - 1 + off);
  const int nt = last_key < 0 ? 0 : last_key / kBN + 1;

  if (nt == 0) {
    // no key is visible to any row of this block: 0 and -inf, and nothing else is set up
    T* outp = reinterpret_cast<T*>(p.out);
    const int rows = live_q * p.heads;  // (token, head) pairs, contiguous in out
    const size_t row0 = static_cast<size_t>(q_base + q0) * p.heads;
    for (int i = tid; i < rows * (kDV / 8); i += kThreads) {
      const int rw = i / (kDV / 8), c = i - rw * (kDV / 8);
      *reinterpret_cast<uint4*>(outp + (row0 + rw) * kCkv + dh * kDV + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (dh == 0 && p.lse)
      for (int i = tid; i < rows; i += kThreads) p.lse[row0 + i] = -INFINITY;
    if constexpr (PERSIST) continue;
    else return;
  }
  if constexpr (!PERSIST) {
    if (warp == 1) {
      tmem_alloc(tmem_holder, 512);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  }

  // page id of token `tok` of this request (clamped: rows past the end repeat the last token and are masked)
  auto page_of = [&](int tok) {
    const int i = kv_base + min(tok, kv_len - 1);
    return min(max(__ldg(p.kv_indices + i), 0), p.num_pages - 1);
  };

  // The nine score chunks of a tile in the order they are streamed: the five that are only keys first, then
  // the four that are also this CTA's value columns (their buffer is free once the value product of the tile
  // two back has completed, which the later they come the more surely has happened).
  auto chunk_at = [&](int i) { return i < kChunks - kVChunks ? (dh == 0 ? kVChunks + i : (i < kVChunks ? i : kChunks - 1))
                                                             : dh * kVChunks + (i - (kChunks - kVChunks)); };

  if (warp == 0) {
    // ================================================================ Q chunks by TMA
    const int row0 = (q_base + q0) * p.heads;  // first row of the block in the (total_q * H, .) view
    for (int j = 0; j < nt; ++j) {
      for (int i = 0; i < kChunks; ++i) {
        const int c = chunk_at(i);
        mbar_wait(&k_empty[st], ph ^ 1, p.status, kFaultEmptyBarrier);
        if (elect_one()) {
          mbar_arrive_expect_tx(&k_full[st], kChunkBytes);
          if (c < kCkv / 64) tma_load_2d(ring + st * kStageBytes, &tm_qn, &k_full[st], c * 64, row0);
          else tma_load_2d(ring + st * kStageBytes, &tm_qp, &k_full[st], 0, row0);
        }
        __syncwarp();
        if (++st == kStages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ================================================================ cache rows of the score chunks
    // eight lanes copy the eight 16-byte pieces of one row's chunk: a warp instruction moves four whole
    // 128-byte lines; the 128 threads cover 16 rows per round
    const int gtid = tid - 6 * 32, piece = gtid & 7, r_in = gtid >> 3;
    const T* ckv = reinterpret_cast<const T*>(p.ckv);
    const T* kpe = reinterpret_cast<const T*>(p.kpe);
    int pg[8], pg_next[8];
    if (nt > 0) {
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) pg_next[rr] = rr * 16 < kv_len ? page_of(rr * 16 + r_in) : 0;
    }
    for (int j = 0; j < nt; ++j) {
      const int jj = jt + j;  // the tile's number in this CTA's run: buffer parities and phases run on across items
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) pg[rr] = pg_next[rr];
      if (j + 1 < nt) {  // one tile ahead: the latency of the index loads stays off the stream
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) pg_next[rr] = (j + 1) * kBN + rr * 16 < kv_len ? page_of((j + 1) * kBN + rr * 16 + r_in) : 0;
      }
      for (int i = 0; i < kChunks; ++i) {
        const int c = chunk_at(i);
        mbar_wait(&k_empty[st], ph ^ 1, p.status, kFaultEmptyBarrier);
        uint32_t dst = smem_u32(ring + st * kStageBytes + kChunkBytes);
        if (i >= kChunks - kVChunks) {
          // a chunk that is also value columns goes to the tile's value buffer, which the value product of
          // tile j - 2 must have finished reading
          if (i == kChunks - kVChunks && jj >= 2) mbar_wait(&pv_done[jj & 1], ((jj >> 1) - 1) & 1, p.status, kFaultMmaBarrier);
          dst = smem_u32(v_smem + (jj & 1) * kVBytes + (i - (kChunks - kVChunks)) * kChunkBytes);
        }
        // rounds of 16 rows; those that lie wholly past the request's last key are not fetched (a tile of a short
        // request, or a request's last tile, is mostly such rows): zeros from the thread itself, which as keys are
        // masked and as values meet P = 0
        const int live_rounds = min(8, (kv_len - j * kBN + 15) >> 4);
        if (live_rounds == 8) {  // the usual tile: every round holds keys, no test in the copy loop
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int row = rr * 16 + r_in;
            const T* src = c < kCkv / 64 ? ckv + static_cast<long long>(pg[rr]) * kCkv + c * 64 + piece * 8
                                         : kpe + static_cast<long long>(pg[rr]) * kKpe + piece * 8;
            const uint32_t o = row * 128 + ((piece ^ (row & 7)) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + o), "l"(src) : "memory");
          }
        } else {
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int row = rr * 16 + r_in;
            const uint32_t o = row * 128 + ((piece ^ (row & 7)) << 4);
            if (rr < live_rounds) {
              const T* src = c < kCkv / 64 ? ckv + static_cast<long long>(pg[rr]) * kCkv + c * 64 + piece * 8
                                           : kpe + static_cast<long long>(pg[rr]) * kKpe + piece * 8;
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + o), "l"(src) : "memory");
            } else {
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst + o), "r"(0u) : "memory");
            }
          }
          fence_proxy_async_smem();  // the MMA reads shared memory through the async proxy
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&k_full[st])) : "memory");
        if (++st == kStages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t idesc_s = umma_idesc(kBf16, /*b_mn_major=*/false, kBM, kBN);
    constexpr uint32_t idesc_pv = umma_idesc(kBf16, /*b_mn_major=*/true, kBM, kDV);
    const uint32_t ring_addr = smem_u32(ring), v_addr = smem_u32(v_smem);
    auto issue_s = [&](int j) {
      const int jj = jt + j;
      const uint32_t d = tmem_base + kColS + (jj & 1) * kBN;
      for (int i = 0; i < kChunks; ++i) {
        mbar_wait(&k_full[st], ph, p.status, kFaultFullBarrier);
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a = ring_addr + st * kStageBytes;
          const uint32_t b = i < kChunks - kVChunks ? a + kChunkBytes
                                                    : v_addr + (jj & 1) * kVBytes + (i - (kChunks - kVChunks)) * kChunkBytes;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adesc = umma_smem_desc(a + kk * 32, 16, 8 * 128);
            const uint64_t bdesc = umma_smem_desc(b + kk * 32, 16, 8 * 128);
            umma_f16(d, adesc, bdesc, idesc_s, (i > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&k_empty[st]);
        }
        __syncwarp();
        if (++st == kStages) { st = 0; ph ^= 1; }
      }
      if (elect_one()) umma_commit(&s_full[jj & 1]);
      __syncwarp();
    };
    issue_s(0);
    for (int j = 0; j < nt; ++j) {
      if (j + 1 < nt) issue_s(j + 1);
      const int jj = jt + j, pb = jj & 1;
      mbar_wait(&p_full[pb], (jj >> 1) & 1, p.status, kFaultTmemBarrier);
      // persistent form: the first value product of an item overwrites O, which the epilogue of the item before
      // must have read
      if (PERSIST && j == 0) mbar_wait(o_free, (it & 1) ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          // B: MN-major, 16 token rows of 128 bytes per step; 64-column chunks are kChunkBytes apart
          // the value chunks of this tile landed before its score product was issued
          const uint64_t bdesc = umma_smem_desc(v_addr + pb * kVBytes + ks * 16 * 128, kChunkBytes, 8 * 128);
          umma_f16_ts(tmem_base + kColO, tmem_base + kColS + pb * kBN + ks * 8, bdesc, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[pb]);
        if (j == nt - 1) umma_commit(o_done);
      }
      __syncwarp();
    }
  } else if (warp >= 2 && warp < 6) {
    // ================================================================ softmax / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // (token, head) pair inside the block = TMEM lane
    const int qi = row / p.heads, head = row - qi * p.heads;
    const bool live = qi < live_q;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const int key_limit = live ? min(kv_len - 1, q0 + qi + off) : -1;  // last key this row sees
    float m_ref = 0.f, l_run = 0.f;
    for (int j = 0; j < nt; ++j) {
      const int jj = jt + j, sb = jj & 1;
      mbar_wait(&s_full[sb], (jj >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      // Two passes over the 128 scores of the row, 32 at a time from tensor memory (reads are cheap, registers
      // are not): the maximum first, then exp2 and the 16-bit P values.
      const uint32_t t_s = tmem_base + lane_field + kColS + sb * kBN;
      const int k0 = j * kBN;
      const bool whole = k0 + kBN - 1 <= key_limit;  // the whole tile is visible to this row
      // the last key any row of this warp sees: groups of 32 scores beyond it are not read at all (the tile of a
      // short request; the diagonal tile of a block's first rows)
      const int warp_limit = __reduce_max_sync(0xffffffffu, key_limit);
      float mx = -INFINITY;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (k0 + q * 32 > warp_limit) break;
        uint32_t rg[32];
        tmem_ld_32x32(t_s + q * 32, rg);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (whole || k0 + q * 32 + i <= key_limit) mx = fmaxf(mx, __uint_as_float(rg[i]) * p.scale_log2);
      }
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_ref = mx == -INFINITY ? 0.f : mx;
      } else if (mx > m_ref + kRescaleThreshold) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {  // rare: the running maximum grew by more than 2^8
        // O may only be touched when no value MMA is in flight: tile j - 1 is the last one issued
        mbar_wait(&pv_done[sb ^ 1], ((jj - 1) >> 1) & 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < kDV; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_field + kColO + c0, o);
        }
        tmem_st_wait();
      }
      // P goes over the first 64 columns of this S buffer: the 64 scores a half of P is made from are in
      // registers before the 32 columns it lands on are overwritten (columns 0-31 come from scores 0-63,
      // columns 32-63 from scores 64-127, which the first store does not touch)
      float psum = 0.f;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t ra[32], rb[32], pk[32];
        if (k0 + hh * 64 > warp_limit) {  // nothing of this half is visible to the warp: P = 0
#pragma unroll
          for (int i = 0; i < 32; ++i) pk[i] = 0u;
          tmem_st_32x32(t_s + hh * 32, pk);
          continue;
        }
        tmem_ld_32x32(t_s + hh * 64, ra);
        tmem_ld_32x32(t_s + hh * 64 + 32, rb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int c = 2 * i;  // scores c and c + 1 of this half
          const uint32_t u0 = c < 32 ? ra[c] : rb[c - 32], u1 = c + 1 < 32 ? ra[c + 1] : rb[c + 1 - 32];
          const int key = k0 + hh * 64 + c;
          const float p0 = (whole || key <= key_limit) ? fast_exp2(__uint_as_float(u0) * p.scale_log2 - m_ref) : 0.f;
          const float p1 = (whole || key + 1 <= key_limit) ? fast_exp2(__uint_as_float(u1) * p.scale_log2 - m_ref) : 0.f;
          psum += p0 + p1;
          pk[i] = pack2<T>(p0, p1);
        }
        tmem_st_32x32(t_s + hh * 32, pk);
      }
      l_run = l_run * alpha + psum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
    }
    // ---- epilogue: O / l
    mbar_wait(o_done, it & 1, p.status, kFaultMmaBarrier);
    tc_fence_after();
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const size_t orow = static_cast<size_t>(q_base + q0 + qi) * p.heads + head;
    T* outp = reinterpret_cast<T*>(p.out) + orow * kCkv + dh * kDV;
#pragma unroll 1
    for (int c0 = 0; c0 < kDV; c0 += 32) {
      uint32_t o[32];
      tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
      tmem_ld_wait();
      if (PERSIST && c0 + 32 >= kDV) {  // O is out of tensor memory: the next item's value product may start
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
    if (live && dh == 0 && p.lse) p.lse[orow] = l_run > 0.f ? m_ref + fast_log2(l_run) : -INFINITY;
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

template <typename T>
int launch(const cb200_mla_prefill_args* a, cudaStream_t stream) {
  Params p{};
  p.ckv = a->ckv_cache;
  p.kpe = a->kpe_cache;
  p.qo_indptr = a->qo_indptr;
  p.kv_indptr = a->kv_indptr;
  p.kv_indices = a->kv_indices;
  p.out = a->out;
  p.lse = a->lse;
  p.status = reinterpret_cast<int*>(a->workspace);
  p.batch = a->batch;
  p.heads = a->num_heads;
  p.qb = kBM / a->num_heads;
  p.num_pages = a->num_pages;
  p.n_idx = a->num_kv_indices;
  p.scale_log2 = a->sm_scale * kLog2e;
  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_qn, tm_qp;
  {
    // the (total_q, H, 512 / 64) query tensors as matrices of total_q * H rows: a block of 128 / H tokens is 128 rows
    const uint64_t rows = static_cast<uint64_t>(a->total_q) * a->num_heads;
    uint32_t box[2] = {64u, 128u};
    uint64_t dn[2] = {kCkv, rows}, sn[1] = {kCkv * 2};
    uint64_t dp[2] = {kKpe, rows}, sp[1] = {kKpe * 2};
    if (!encode_tensor_map(&tm_qn, dt, 2, const_cast<void*>(a->q_nope), dn, sn, box, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tensor_map(&tm_qp, dt, 2, const_cast<void*>(a->q_pe), dp, sp, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
  }
  // every request has at most ceil(q_len / qb) <= q_len / qb + 1 query blocks; two items (column halves) per block
  const long long blocks = static_cast<long long>(ceil_div(a->total_q, p.qb)) + a->batch;
  p.blocks = static_cast<int>(blocks);
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  // Many short items (batches of prompts of a few hundred tokens): persistent CTAs, whose producers run ahead into the
  // next item. Few items, or long ones (an item of a 2048-token prompt has up to sixteen KV tiles and is bound by what
  // the SM pulls from L2, not by the boundaries): one CTA per item.
  const bool persist = 2 * blocks >= 3LL * sms && static_cast<long long>(a->num_kv_indices) <= 320LL * a->batch;
  if (persist) {
    auto kern = mla_prefill_kernel<T, true>;
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    kern<<<static_cast<unsigned>(sms), kThreadsPersist, kSmemBytes, stream>>>(tm_qn, tm_qp, p);
  } else {
    auto kern = mla_prefill_kernel<T, false>;
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    kern<<<static_cast<unsigned>(2 * blocks), kThreads, kSmemBytes, stream>>>(tm_qn, tm_qp, p);
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

int plan(const cb200_mla_prefill_args* a) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->batch <= 0 || a->total_q <= 0 || a->num_heads <= 0 || a->num_pages <= 0 || a->num_kv_indices < 0) return CB200_ERR_BAD_ARG;
  if (a->ckv_dim != kCkv || a->kpe_dim != kKpe) return CB200_ERR_UNSUPPORTED;
  if (a->num_heads > kBM || kBM % a->num_heads) return CB200_ERR_UNSUPPORTED;  // a block of whole tokens fills the 128 MMA rows
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  const long long blocks = static_cast<long long>(ceil_div(a->total_q, kBM / a->num_heads)) + a->batch;
  if (2 * blocks >= (1LL << 31) || static_cast<long long>(a->total_q) * a->num_heads >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  return CB200_OK;
}

}  // namespace mlapf
}  // namespace cb200

extern "C" size_t cb200_mla_prefill_workspace_bytes(const cb200_mla_prefill_args* a) {
  return cb200::mlapf::plan(a) == CB200_OK ? cb200::kWsHeaderBytes : 0;
}

extern "C" int cb200_mla_prefill(const cb200_mla_prefill_args* a, void* stream) {
  using namespace cb200;
  const int rc = mlapf::plan(a);
  if (rc != CB200_OK) return rc;
  if (!a->q_nope || !a->q_pe || !a->ckv_cache || !a->kpe_cache || !a->qo_indptr || !a->kv_indptr || !a->out) return CB200_ERR_BAD_ARG;
  if (!a->kv_indices && a->num_kv_indices > 0) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q_nope) | reinterpret_cast<uintptr_t>(a->q_pe) | reinterpret_cast<uintptr_t>(a->ckv_cache) |
       reinterpret_cast<uintptr_t>(a->kpe_cache) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < kWsHeaderBytes) return CB200_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // a page table far shorter than the run of query rows: most rows see no key (see small_attn.cu)
  if (small_prefill_applies(a->num_kv_indices, a->total_q))
    return launch_small_mla(a->q_nope, a->q_pe, a->ckv_cache, a->kpe_cache, a->qo_indptr, a->kv_indptr, a->kv_indices, a->out,
                            a->lse, a->batch, a->total_q, a->num_heads, a->num_pages, a->num_kv_indices, a->sm_scale, a->dtype, st);
  return a->dtype == CB200_F16 ? mlapf::launch<__half>(a, st) : mlapf::launch<__nv_bfloat16>(a, st);
}
