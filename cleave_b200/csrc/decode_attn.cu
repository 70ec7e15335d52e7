// Decode attention (MHA / GQA / MQA; contiguous or paged KV) for sm_100a.
//
// One persistent launch, one CTA per SM. The KV cache is cut into tiles of 64 tokens; the tiles of
// all (request, kv head) items form one stream that is split evenly over the CTAs, so a CTA's
// share may start or end in the middle of an item. A producer warp streams its share of tiles
// into a ring of shared-memory stages (TMA tiled loads with the 128-byte swizzle when a tile maps
// to whole boxes of the cache; otherwise eight producer warps gather the token rows with 16-byte
// cp.async into the same swizzled layout) and the
// consumer warps run QK^T and PV on m16n8k16 tensor-core MMAs with a warp-shuffle online softmax
// in the exp2 domain. An item finished inside one CTA is written directly; an item cut across
// CTAs leaves fp32 partials (O, m, l) in the workspace and the last CTA to arrive does the
// log-sum-exp combine (no second launch, nobody waits).
//
// Semantics follow python/cleave/dynamic/reference.py:143-200 of the reference (paged) and
// demo/attention.py:5-8 (static); the valid-length clamp follows
// python/cleave/dynamic/paging/builders/slab.py:132-142.

#include "common.cuh"
#include "stream_walk.cuh"

#include <cstring>
#include <mutex>

namespace cb200 {

constexpr int kTile = 64;          // tokens per KV tile
constexpr int kRowsMax = 16;       // query rows one item carries (M of the MMA tile)
constexpr int kConsumerWarps = 4;  // each owns 16 tokens of every tile
constexpr int kPieceUnits = 5;     // what starting and finishing a piece costs, in tiles: the stream of a paged launch is cut by cost
constexpr int kPrefetchTiles = 16; // tiles a CTA asks into L2 while it waits for the preceding kernel (contiguous caches)
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  const int* kv_indptr;
  const int* kv_indices;
  const int* kv_last;
  void* out;
  float* lse;
  int* status;     // workspace header
  int* counters;   // one arrival counter per item, zero between launches
  float* partials; // gridDim.x * 2 slots
  int batch, hkv, vblk, rows, page_size, num_pages, n_idx, kv_len, paged, box_tok;
  float scale_log2;
};

template <int D, bool GATHER>
struct SmemPlan {
  // Both paths use the same tile layout: per 64-column half, 64 rows of 128 bytes with the
  // 128-byte swizzle (what TMA writes; the gather path reproduces it with 16-byte cp.async).
  static constexpr int kMatBytes = kTile * D * 2;
  static constexpr int kStageBytes = 2 * kMatBytes;
  static constexpr int kStages = 5;
  // gather: eight copying warps - the bytes an SM keeps in flight are bounded per issuing warp (a gather-only kernel
  // over random 1 KB rows moved 4.0 TB/s with four warps per SM whatever their depth, 6.0 with eight)
  static constexpr int kProducerWarps = GATHER ? 8 : 1;
  static constexpr int kThreads = (kConsumerWarps + kProducerWarps) * 32;
  static constexpr int kMergeFloats = kRowsMax * D + 2 * kRowsMax;
  static constexpr int kMergeBytes = kConsumerWarps * kMergeFloats * 4;
  static constexpr int kFixedBytes = kStages * kStageBytes + kMergeBytes + 256;  // + barriers/flags
};

// Pages of request b that the page table really holds: kv_indptr is caller data, so the range it names is
// clipped to [0, n_idx) and every later read of kv_indices stays inside the array whatever it says.
__device__ __forceinline__ int item_pages(const DecodeParams& p, int b) {
  const int base = p.kv_indptr[b];
  if (base < 0 || base >= p.n_idx) return 0;
  return max(min(p.kv_indptr[b + 1] - base, p.n_idx - base), 0);
}

__device__ __forceinline__ int item_valid_len(const DecodeParams& p, int b) {
  if (!p.paged) return p.kv_len;
  const int n_pages = item_pages(p, b);
  if (p.page_size == 1 || p.kv_last == nullptr) return n_pages * p.page_size;
  const int v = max(n_pages - 1, 0) * p.page_size + max(p.kv_last[b], 0);
  return max(min(v, n_pages * p.page_size), 0);
}

template <typename T, int D, bool GATHER>
__global__ void __launch_bounds__(SmemPlan<D, GATHER>::kThreads, 1)
decode_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const DecodeParams p) {
  using Plan = SmemPlan<D, GATHER>;
  constexpr int kStages = Plan::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  float* merge = reinterpret_cast<float*>(smem + kStages * Plan::kStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * Plan::kStageBytes + Plan::kMergeBytes);
  uint64_t* empty_bar = full_bar + kStages;
  int* flags = reinterpret_cast<int*>(empty_bar + kStages);  // [0] last-arriver flag, [1..] scan scratch
  int* P = reinterpret_cast<int*>(smem + Plan::kFixedBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = blockDim.x;
  const int hkvv = p.hkv * p.vblk;

  // The launch carries the programmatic-serialization attribute: this CTA may start while the kernel
  // before it in the stream is still draining. Nothing that kernel may have written (page tables, the
  // caches, Q, the workspace) is touched before pdl_wait(); what precedes it is shared-memory set-up.
  // ---- tile prefix over requests (every CTA computes the same table)
  int tiles_per_req = 0;
  if (p.paged) {
    pdl_wait();
    int* scratch = reinterpret_cast<int*>(merge);  // merge buffer is free at this point
    const int per = ceil_div(p.batch, nthreads);
    const int i0 = min(tid * per, p.batch), i1 = min(i0 + per, p.batch);
    int sum = 0;
    for (int i = i0; i < i1; ++i) sum += Walker::units(ceil_div(item_valid_len(p, i), kTile), kPieceUnits);
    scratch[tid] = sum;
    __syncthreads();
    if (tid < 32) {
      const int all = warp_scan_in_place(scratch, nthreads, tid);
      if (tid == 0) P[p.batch] = all;
    }
    __syncthreads();
    int run = scratch[tid];
    for (int i = i0; i < i1; ++i) {
      P[i] = run;
      run += Walker::units(ceil_div(item_valid_len(p, i), kTile), kPieceUnits);
    }
  } else {
    tiles_per_req = ceil_div(p.kv_len, kTile);
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], GATHER ? Plan::kProducerWarps * 32 : 1);  // gather: one arrival per copying thread
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    mbar_fence_init();
    if (!GATHER) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
    }
  }
  __syncthreads();

  const int total_per_head = p.paged ? P[p.batch] : p.batch * tiles_per_req;
  const int total = hkvv * total_per_head;
  const int G = gridDim.x;
  const int span = total > 0 ? ceil_div(total, G) : 1;
  const int u0 = min(static_cast<int>(blockIdx.x) * span, total);
  const int u1 = min(u0 + span, total);
  Walker walker{p.paged ? P : nullptr, p.batch, hkvv, tiles_per_req, p.paged ? kPieceUnits : 0};
  if (!p.paged) {
    // Contiguous caches: where this CTA's first tiles lie follows from the launch parameters alone, so
    // while the preceding kernel still runs the TMA unit is asked to bring them into L2 (a hint: nothing
    // reaches the SM, and L2 is where that kernel's writes land too). The first ring fill then comes from
    // L2 with warm address translations instead of paying the cold 2.3 us.
    if (!GATHER && warp == kConsumerWarps && lane == 0 && u0 < u1) {
      int uf = u0;
      const Piece pc = walker.at(uf, u1);
      const int h = pc.hv / p.vblk;
      for (int t = pc.tile0; t < pc.tile0 + min(pc.count, kPrefetchTiles); ++t) {
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
          tma_prefetch_4d(&tm_k, hf * 64, 0, t * kTile, pc.b * p.hkv + h);
          tma_prefetch_4d(&tm_v, hf * 64, 0, t * kTile, pc.b * p.hkv + h);
        }
      }
    }
    pdl_wait();
  }
  pdl_launch_dependents();  // the next kernel's CTAs may take SMs as this grid's CTAs retire

  if (warp >= kConsumerWarps) {
    // ================================================================= producer warp(s)
    int stage = 0, phase = 0;
    for (int u = u0; u < u1;) {
      const Piece pc = walker.at(u, u1);
      if (pc.count == 0) break;  // the share ends in front of the next item's tiles
      const int h = pc.hv / p.vblk;
      const int valid = item_valid_len(p, pc.b);
      const int page_base = p.paged ? p.kv_indptr[pc.b] : 0;
      const int n_pages = p.paged ? ceil_div(valid, p.page_size) : 0;
      if constexpr (!GATHER) {
        int win = -1, cur_idx = 0, next_idx = 0;
        for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
          mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
          uint8_t* kdst = stages + stage * Plan::kStageBytes;
          uint8_t* vdst = kdst + Plan::kMatBytes;
          if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], Plan::kStageBytes);
          __syncwarp();
          if (p.paged) {
            const int nbox = kTile / p.box_tok;
            for (int j = 0; j < nbox; ++j) {
              const int tok = t * kTile + j * p.box_tok;
              const int pord = min(tok / p.page_size, n_pages - 1);
              const int slot = tok - (tok / p.page_size) * p.page_size;
              const int w = pord >> 5;
              if (w != win) {  // warp-uniform: refill the 32-entry window of page ids
                if (w == win + 1 && win >= 0) {
                  cur_idx = next_idx;
                } else {
                  cur_idx = __ldg(p.kv_indices + page_base + min(w * 32 + lane, n_pages - 1));
                }
                next_idx = __ldg(p.kv_indices + page_base + min((w + 1) * 32 + lane, n_pages - 1));
                win = w;
              }
              int page = __shfl_sync(0xffffffffu, cur_idx, pord & 31);
              page = min(max(page, 0), p.num_pages - 1);
              if (lane == 0) {
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf) {
                  const int off = hf * (kTile * 128) + j * p.box_tok * 128;
                  tma_load_4d(kdst + off, &tm_k, &full_bar[stage], hf * 64, h, slot, page);
                  tma_load_4d(vdst + off, &tm_v, &full_bar[stage], hf * 64, h, slot, page);
                }
              }
            }
          } else if (lane == 0) {
#pragma unroll
            for (int hf = 0; hf < D / 64; ++hf) {
              const int off = hf * (kTile * 128);
              tma_load_4d(kdst + off, &tm_k, &full_bar[stage], hf * 64, 0, t * kTile, pc.b * p.hkv + h);
              tma_load_4d(vdst + off, &tm_v, &full_bar[stage], hf * 64, 0, t * kTile, pc.b * p.hkv + h);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      } else {
        // Row gather (pages smaller than a tile): eight producer warps copy the 64 token
        // rows of a tile with 16-byte cp.async into the swizzled layout. Consecutive lanes copy
        // consecutive 16-byte chunks of a row, so one warp instruction moves whole rows (full 128-byte
        // lines) instead of a sliver of 32 rows; a thread's arrival on the full barrier fires when its
        // copies have landed. Page ids are read one tile ahead so their latency stays off the
        // critical path.
        const T* kc = reinterpret_cast<const T*>(p.k);
        const T* vc = reinterpret_cast<const T*>(p.v);
        constexpr int kPThreads = Plan::kProducerWarps * 32;
        const int ptid = tid - kConsumerWarps * 32;   // 0..kPThreads-1
        constexpr int kChunks = D / 8;                // 16-byte chunks per row
        constexpr int kRowsPerRound = kPThreads / kChunks;  // rows the copying threads cover at once
        constexpr int kRounds = kTile / kRowsPerRound;
        const int c = ptid % kChunks, r_in = ptid / kChunks;
        auto load_pages = [&](int t, int (&pg)[kRounds]) {
#pragma unroll
          for (int r = 0; r < kRounds; ++r) {
            const int tok = min(t * kTile + r * kRowsPerRound + r_in, valid - 1);
            pg[r] = __ldg(p.kv_indices + page_base + tok / p.page_size);
          }
        };
        int pg[kRounds];
        load_pages(pc.tile0, pg);
        for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
          int cur[kRounds];
#pragma unroll
          for (int r = 0; r < kRounds; ++r) cur[r] = pg[r];
          if (t + 1 < pc.tile0 + pc.count) load_pages(t + 1, pg);
          mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
          const uint32_t kdst = smem_u32(stages + stage * Plan::kStageBytes);
          const uint32_t vdst = kdst + Plan::kMatBytes;
#pragma unroll
          for (int r = 0; r < kRounds; ++r) {
            const int row = r * kRowsPerRound + r_in;
            const int tok = min(t * kTile + row, valid - 1);
            const int slot = tok - (tok / p.page_size) * p.page_size;
            const long long page = min(max(cur[r], 0), p.num_pages - 1);
            const long long off = ((page * p.page_size + slot) * p.hkv + h) * D + c * 8;
            const uint32_t dst_off = (c >> 3) * (kTile * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kdst + dst_off), "l"(kc + off) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vdst + dst_off), "l"(vc + off) : "memory");
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[stage])) : "memory");
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      u += pc.count;
    }
    return;
  }

  // =================================================================== consumer warps
  const int ctid = tid;  // 0 .. kConsumerWarps*32-1
  constexpr int kCThreads = kConsumerWarps * 32;
  T* outp = reinterpret_cast<T*>(p.out);

  // Requests without any live token: out = 0, lse = -inf.
  if (p.paged) {
    const int rows_all = p.hkv * p.rows;  // query rows per request
    for (int b = blockIdx.x; b < p.batch; b += G) {
      if (P[b + 1] - P[b] != 0) continue;
      for (int i = ctid; i < rows_all * D; i += kCThreads) outp[static_cast<size_t>(b) * rows_all * D + i] = T(0.f);
      if (p.lse)
        for (int i = ctid; i < rows_all; i += kCThreads) p.lse[static_cast<size_t>(b) * rows_all + i] = -INFINITY;
    }
  }

  const int ws = warp;  // token slice of this warp inside a tile
  const int r0 = lane >> 2, c2 = (lane & 3) * 2;
  const uint32_t stages_u32 = smem_u32(stages);
  float* my_merge = merge + warp * Plan::kMergeFloats;
  const int slot_floats = Plan::kMergeFloats;

  int stage = 0, phase = 0;
  for (int u = u0; u < u1;) {
    const Piece pc = walker.at(u, u1);
    if (pc.count == 0) break;  // the share ends in front of the next item's tiles
    const int h = pc.hv / p.vblk, blk = pc.hv - h * p.vblk;
    const int valid = item_valid_len(p, pc.b);
    const int rows_here = min(kRowsMax, p.rows - blk * kRowsMax);
    const size_t row_base = (static_cast<size_t>(pc.b) * p.hkv + h) * p.rows + blk * kRowsMax;

    // ---- Q fragments (A operand), rows beyond rows_here are zero
    uint32_t qf[D / 16][4];
    {
      const T* qrow0 = reinterpret_cast<const T*>(p.q) + (row_base + r0) * D;
      const T* qrow1 = qrow0 + 8 * D;
      const bool ok0 = r0 < rows_here, ok1 = r0 + 8 < rows_here;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int d = kk * 16 + c2;
        qf[kk][0] = ok0 ? *reinterpret_cast<const uint32_t*>(qrow0 + d) : 0u;
        qf[kk][1] = ok1 ? *reinterpret_cast<const uint32_t*>(qrow1 + d) : 0u;
        qf[kk][2] = ok0 ? *reinterpret_cast<const uint32_t*>(qrow0 + d + 8) : 0u;
        qf[kk][3] = ok1 ? *reinterpret_cast<const uint32_t*>(qrow1 + d + 8) : 0u;
      }
    }
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
      mbar_wait(&full_bar[stage], phase, p.status, kFaultFullBarrier);
      const int tok0 = t * kTile + ws * 16;
      if (tok0 < valid) {
        const uint32_t kbase = stages_u32 + stage * Plan::kStageBytes;
        const uint32_t vbase = kbase + Plan::kMatBytes;
        const int mi = lane >> 3, rr = lane & 7;
        // ---- S = Q K^T for this warp's 16 tokens
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
          const int row = ws * 16 + (mi >> 1) * 8 + rr;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const int d = kk * 16 + (mi & 1) * 8;
            const uint32_t addr = kbase + (d >> 6) * (kTile * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, addr);
            mma_16816<T>(s[0], qf[kk], b0, b1);
            mma_16816<T>(s[1], qf[kk], b2, b3);
          }
        }
        // ---- online softmax (exp2 domain)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = tok0 + nb * 8 + c2 + (e & 1);
            const float x = tok < valid ? s[nb][e] * p.scale_log2 : -INFINITY;
            s[nb][e] = x;
            if (e < 2) mx0 = fmaxf(mx0, x); else mx1 = fmaxf(mx1, x);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float sc0 = fast_exp2(m_run[0] - mu0), sc1 = fast_exp2(m_run[1] - mu1);
        m_run[0] = mn0;
        m_run[1] = mn1;
        uint32_t pf[4];
        float ps0 = 0.f, ps1 = 0.f;
        {
          const float p00 = fast_exp2(s[0][0] - mu0), p01 = fast_exp2(s[0][1] - mu0);
          const float p02 = fast_exp2(s[0][2] - mu1), p03 = fast_exp2(s[0][3] - mu1);
          const float p10 = fast_exp2(s[1][0] - mu0), p11 = fast_exp2(s[1][1] - mu0);
          const float p12 = fast_exp2(s[1][2] - mu1), p13 = fast_exp2(s[1][3] - mu1);
          ps0 = p00 + p01 + p10 + p11;
          ps1 = p02 + p03 + p12 + p13;
          pf[0] = pack2<T>(p00, p01);
          pf[1] = pack2<T>(p02, p03);
          pf[2] = pack2<T>(p10, p11);
          pf[3] = pack2<T>(p12, p13);
        }
        l_run[0] = l_run[0] * sc0 + ps0;
        l_run[1] = l_run[1] * sc1 + ps1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
          acc[n][0] *= sc0;
          acc[n][1] *= sc0;
          acc[n][2] *= sc1;
          acc[n][3] *= sc1;
        }
        // ---- O += P V
        {
          const int row = ws * 16 + (mi & 1) * 8 + rr;
#pragma unroll
          for (int dp = 0; dp < D / 16; ++dp) {
            const int d = dp * 16 + (mi >> 1) * 8;
            const uint32_t addr = vbase + (d >> 6) * (kTile * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, addr);
            mma_16816<T>(acc[2 * dp], pf, b0, b1);
            mma_16816<T>(acc[2 * dp + 1], pf, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }

    // ---- merge the four warps' states through shared memory
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      *reinterpret_cast<float2*>(my_merge + r0 * D + n * 8 + c2) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(my_merge + (r0 + 8) * D + n * 8 + c2) = make_float2(acc[n][2], acc[n][3]);
    }
    if ((lane & 3) == 0) {
      my_merge[kRowsMax * D + r0] = m_run[0];
      my_merge[kRowsMax * D + r0 + 8] = m_run[1];
      my_merge[kRowsMax * D + kRowsMax + r0] = l_run[0];
      my_merge[kRowsMax * D + kRowsMax + r0 + 8] = l_run[1];
    }
    named_bar_sync(1, kCThreads);

    constexpr int kColsPerThread = kRowsMax * D / kCThreads;  // 16 (D=128) or 8 (D=64)
    constexpr int kThreadsPerRow = kCThreads / kRowsMax;      // 8
    const int mrow = ctid / kThreadsPerRow, mcol = (ctid % kThreadsPerRow) * kColsPerThread;
    float M = -INFINITY, L = 0.f, o[kColsPerThread];
    {
      float mw[kConsumerWarps];
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        mw[w] = merge[w * Plan::kMergeFloats + kRowsMax * D + mrow];
        M = fmaxf(M, mw[w]);
      }
      const float Mu = M == -INFINITY ? 0.f : M;
#pragma unroll
      for (int c = 0; c < kColsPerThread; ++c) o[c] = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float cf = fast_exp2(mw[w] - Mu);
        L += cf * merge[w * Plan::kMergeFloats + kRowsMax * D + kRowsMax + mrow];
        const float* src = merge + w * Plan::kMergeFloats + mrow * D + mcol;
#pragma unroll
        for (int c = 0; c < kColsPerThread; c += 4) {
          const float4 x = *reinterpret_cast<const float4*>(src + c);
          o[c] += cf * x.x;
          o[c + 1] += cf * x.y;
          o[c + 2] += cf * x.z;
          o[c + 3] += cf * x.w;
        }
      }
    }

    const bool starts_here = (u == pc.unit0);
    const bool whole = starts_here && pc.count == pc.n_tiles;
    auto store_final = [&](float Mf, float Lf, const float* of) {
      if (mrow < rows_here) {
        const float inv = Lf > 0.f ? 1.f / Lf : 0.f;
        T* dst = outp + (row_base + mrow) * D + mcol;
#pragma unroll
        for (int c = 0; c < kColsPerThread; c += 8) {
          uint4 pk;
          pk.x = pack2<T>(of[c] * inv, of[c + 1] * inv);
          pk.y = pack2<T>(of[c + 2] * inv, of[c + 3] * inv);
          pk.z = pack2<T>(of[c + 4] * inv, of[c + 5] * inv);
          pk.w = pack2<T>(of[c + 6] * inv, of[c + 7] * inv);
          *reinterpret_cast<uint4*>(dst + c) = pk;
        }
        if (p.lse && mcol == 0) p.lse[row_base + mrow] = Lf > 0.f ? Mf + fast_log2(Lf) : -INFINITY;
      }
    };

    if (whole) {
      store_final(M, L, o);
    } else {
      // ---- leave a partial, then let the last arriver combine
      float* slot = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * slot_floats;
      if (mrow < rows_here) {
#pragma unroll
        for (int c = 0; c < kColsPerThread; c += 4)
          *reinterpret_cast<float4*>(slot + mrow * D + mcol + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
        if (mcol == 0) {
          slot[kRowsMax * D + mrow] = M;
          slot[kRowsMax * D + kRowsMax + mrow] = L;
        }
      }
      __threadfence();
      named_bar_sync(1, kCThreads);
      const int c_first = pc.unit0 / span, c_last = (pc.unit0 + pc.n_tiles - 1) / span;
      int* counter = p.counters + pc.b * hkvv + pc.hv;
      if (ctid == 0) {
        const int old = atomicAdd(counter, 1);
        flags[0] = (old == c_last - c_first) ? 1 : 0;
      }
      named_bar_sync(1, kCThreads);
      if (flags[0]) {
        __threadfence();
        float Mc = -INFINITY, Lc = 0.f, oc[kColsPerThread];
#pragma unroll
        for (int c = 0; c < kColsPerThread; ++c) oc[c] = 0.f;
        if (mrow < rows_here) {
          // the partials of up to four CTAs are fetched together: one L2 round trip per group instead of
          // one per CTA (an item of a long request can span every CTA of the grid)
          constexpr int kGroup = 4, kVec = kColsPerThread / 4;
          for (int cta0 = c_first; cta0 <= c_last; cta0 += kGroup) {
            float mi_[kGroup], li_[kGroup];
            float4 x[kGroup][kVec];
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
              const int cta = min(cta0 + g, c_last);  // a repeated slot is given weight zero below
              const float* src = p.partials + (static_cast<size_t>(cta) * 2 + (cta == c_first ? 1 : 0)) * slot_floats;
              mi_[g] = __ldcg(src + kRowsMax * D + mrow);
              li_[g] = __ldcg(src + kRowsMax * D + kRowsMax + mrow);
#pragma unroll
              for (int c = 0; c < kVec; ++c) x[g][c] = __ldcg(reinterpret_cast<const float4*>(src + mrow * D + mcol + 4 * c));
            }
#pragma unroll
            for (int g = 0; g < kGroup; ++g) {
              if (cta0 + g > c_last) continue;
              const float Mn = fmaxf(Mc, mi_[g]);
              const float Mu = Mn == -INFINITY ? 0.f : Mn;
              const float a = fast_exp2(Mc - Mu), bb = fast_exp2(mi_[g] - Mu);
              Lc = a * Lc + bb * li_[g];
#pragma unroll
              for (int c = 0; c < kVec; ++c) {
                oc[4 * c] = a * oc[4 * c] + bb * x[g][c].x;
                oc[4 * c + 1] = a * oc[4 * c + 1] + bb * x[g][c].y;
                oc[4 * c + 2] = a * oc[4 * c + 2] + bb * x[g][c].z;
                oc[4 * c + 3] = a * oc[4 * c + 3] + bb * x[g][c].w;
              }
              Mc = Mn;
            }
          }
        }
        store_final(Mc, Lc, oc);
        if (ctid == 0) *counter = 0;  // ready for the next launch
      }
    }
    named_bar_sync(1, kCThreads);  // merge buffer and flag are free again
    u += pc.count;
  }
}

// ------------------------------------------------------------------------------------- host side
namespace {

struct DecodeSetup {
  DecodeParams p;
  bool gather;
  int grid, smem_bytes;
  size_t ws_needed, counters_off, partials_off;
  CUtensorMap tm_k, tm_v;
};

int plan_decode(const cb200_attn_decode_args* a, DecodeSetup* s, bool need_maps) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->batch <= 0 || a->num_qo_heads <= 0 || a->num_kv_heads <= 0) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads % a->num_kv_heads) return CB200_ERR_BAD_ARG;
  if (a->head_dim != 64 && a->head_dim != 128) return CB200_ERR_UNSUPPORTED;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  const bool paged = a->kv_indptr != nullptr;
  const int D = a->head_dim;
  const int q_rows = a->q_rows > 1 ? a->q_rows : 1;
  const int rows = (a->num_qo_heads / a->num_kv_heads) * q_rows;
  DecodeParams& p = s->p;
  p = DecodeParams{};
  p.batch = a->batch;
  p.hkv = a->num_kv_heads;
  p.rows = rows;
  p.vblk = ceil_div(rows, kRowsMax);
  p.paged = paged ? 1 : 0;
  p.scale_log2 = a->sm_scale * kLog2e;
  long long tiles_ub;
  if (paged) {
    if (a->page_size <= 0 || a->num_pages <= 0 || a->num_kv_indices < 0) return CB200_ERR_BAD_ARG;
    p.page_size = a->page_size;
    p.num_pages = a->num_pages;
    p.n_idx = a->num_kv_indices;
    const int ps = a->page_size;
    // Pages of a whole tile (64 tokens) or more are fetched as TMA boxes; smaller pages would need several
    // small boxes per tile (measured 2.8 TB/s at 16 tokens, 4.3 at 32, 6.0 at 64) and take the row gather
    // instead (5.3 - 5.5 TB/s at any page size).
    s->gather = !(ps >= kTile && ps % kTile == 0);
    p.box_tok = kTile;
    tiles_ub = (static_cast<long long>(a->num_kv_indices) * ps + kTile - 1) / kTile + static_cast<long long>(a->batch) * (1 + kPieceUnits);
  } else {
    if (a->kv_len <= 0) return CB200_ERR_BAD_ARG;
    p.kv_len = a->kv_len;
    s->gather = false;
    p.box_tok = kTile;
    tiles_ub = static_cast<long long>(a->batch) * ceil_div(a->kv_len, kTile);
  }
  const long long units_ub = tiles_ub * p.hkv * p.vblk;
  // The kernel counts tiles in 32 bits. Requests may share pages (overlapping kv_indptr ranges), so the
  // bound for that count is every request spanning the whole table, not the table's own size.
  const long long tiles_max = paged ? static_cast<long long>(a->batch) * ((static_cast<long long>(a->num_kv_indices) * a->page_size + kTile - 1) / kTile + 1 + kPieceUnits)
                                    : tiles_ub;
  if (tiles_max * p.hkv * p.vblk >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  int grid = sms;
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  // The workspace is sized for a full grid so that one allocation serves every launch.
  const int fixed = D == 128 ? (s->gather ? SmemPlan<128, true>::kFixedBytes : SmemPlan<128, false>::kFixedBytes)
                             : (s->gather ? SmemPlan<64, true>::kFixedBytes : SmemPlan<64, false>::kFixedBytes);
  s->smem_bytes = fixed + (paged ? (a->batch + 1) * 4 : 0) + 1024 + 16;
  if (s->smem_bytes > 227 * 1024) return CB200_ERR_UNSUPPORTED;  // too many requests for one launch
  // Layout: header | partial slots (two per SM, sized for head_dim 128) | arrival counters.
  // The counters sit at an offset that does not depend on the problem shape: launches of
  // different shapes may share one workspace, and a region that one launch used for partials
  // is never read as counters by the next.
  constexpr size_t kSlotBytesMax = (kRowsMax * 128 + 2 * kRowsMax) * 4;
  s->partials_off = kWsHeaderBytes;
  s->counters_off = align_up(s->partials_off + static_cast<size_t>(sms) * 2 * kSlotBytesMax, 256);
  s->ws_needed = s->counters_off + static_cast<size_t>(a->batch) * p.hkv * p.vblk * 4;
  s->grid = static_cast<int>(units_ub < grid ? (units_ub > 0 ? units_ub : 1) : grid);
  if (!need_maps) return CB200_OK;

  if (!a->q || !a->k_cache || !a->v_cache || !a->out) return CB200_ERR_BAD_ARG;
  if (paged && !a->kv_indices && a->num_kv_indices > 0) return CB200_ERR_BAD_ARG;
  if (paged && a->page_size != 1 && !a->kv_last_page_len) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k_cache) |
       reinterpret_cast<uintptr_t>(a->v_cache) | reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < s->ws_needed) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return CB200_ERR_ALIGNMENT;
  p.q = a->q;
  p.k = a->k_cache;
  p.v = a->v_cache;
  p.kv_indptr = a->kv_indptr;
  p.kv_indices = a->kv_indices;
  p.kv_last = a->kv_last_page_len;
  p.out = a->out;
  p.lse = a->lse;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.counters = reinterpret_cast<int*>(ws + s->counters_off);
  p.partials = reinterpret_cast<float*>(ws + s->partials_off);

  if (!s->gather) {
    const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    uint64_t dims[4], strides[3];
    uint32_t box[4] = {64u, 1u, static_cast<uint32_t>(p.box_tok), 1u};
    const uint64_t rowb = static_cast<uint64_t>(D) * 2;
    if (paged) {
      dims[0] = D; dims[1] = p.hkv; dims[2] = p.page_size; dims[3] = p.num_pages;
      strides[0] = rowb; strides[1] = rowb * p.hkv; strides[2] = rowb * p.hkv * p.page_size;
    } else {
      dims[0] = D; dims[1] = 1; dims[2] = p.kv_len; dims[3] = static_cast<uint64_t>(p.batch) * p.hkv;
      strides[0] = rowb; strides[1] = rowb; strides[2] = rowb * p.kv_len;
    }
    if (!encode_tensor_map(&s->tm_k, dt, 4, const_cast<void*>(a->k_cache), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tensor_map(&s->tm_v, dt, 4, const_cast<void*>(a->v_cache), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
  } else {
    memset(&s->tm_k, 0, sizeof(CUtensorMap));
    memset(&s->tm_v, 0, sizeof(CUtensorMap));
  }
  return CB200_OK;
}

template <typename T, int D, bool GATHER>
int launch_decode(const DecodeSetup& s, cudaStream_t stream) {
  auto kern = decode_attn_kernel<T, D, GATHER>;
  static int configured_smem[16] = {0};  // per device
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 16 && configured_smem[dev] < s.smem_bytes) {
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_smem[dev] = 227 * 1024;
  } else if (dev >= 16) {
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s.grid, 1, 1);
  cfg.blockDim = dim3(SmemPlan<D, GATHER>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = s.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  // the grid may be scheduled while the preceding kernel of the stream drains; it waits (griddepcontrol.wait)
  // before its first global access
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, s.tm_k, s.tm_v, s.p));
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

}  // namespace
}  // namespace cb200

namespace cb200 {
namespace {

// Scratch for cb200_attn_decode_static_scratch: lives in the library's device image, so every GPU
// that loads the library holds these 4 MiB until the process exits.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device address. The
// address is looked up once per device, with that device current, and cached.
int static_scratch_address(unsigned char** out) {
  static unsigned char* cached[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 64 && cached[dev]) {
    *out = cached[dev];
    return CB200_OK;
  }
  unsigned char* ptr = nullptr;
  CB200_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_static_scratch));
  if (!ptr) return CB200_ERR_CUDA;
  if (dev < 64) cached[dev] = ptr;
  *out = ptr;
  return CB200_OK;
}

}  // namespace
}  // namespace cb200

extern "C" size_t cb200_attn_decode_static_scratch_max_bytes(void) { return cb200::kStaticScratchBytes; }

extern "C" int cb200_attn_decode_static_scratch(const cb200_attn_decode_args* a, void* stream) {
  using namespace cb200;
  DecodeSetup s;
  int rc = plan_decode(a, &s, false);
  if (rc != CB200_OK) return rc;
  if (s.ws_needed > kStaticScratchBytes) return CB200_ERR_SCRATCH_LIMIT;
  unsigned char* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != CB200_OK) return rc;
  cb200_attn_decode_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = kStaticScratchBytes;
  rc = plan_decode(&b, &s, true);
  if (rc != CB200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left behind; the status word and this call's
  // arrival counters must start at zero.
  CB200_CUDA_TRY(cudaMemsetAsync(scratch, 0, kWsHeaderBytes, st));
  CB200_CUDA_TRY(cudaMemsetAsync(scratch + s.counters_off, 0, s.ws_needed - s.counters_off, st));
  const bool f16 = b.dtype == CB200_F16;
  if (b.head_dim == 128) {
    if (s.gather) return f16 ? launch_decode<__half, 128, true>(s, st) : launch_decode<__nv_bfloat16, 128, true>(s, st);
    return f16 ? launch_decode<__half, 128, false>(s, st) : launch_decode<__nv_bfloat16, 128, false>(s, st);
  }
  if (s.gather) return f16 ? launch_decode<__half, 64, true>(s, st) : launch_decode<__nv_bfloat16, 64, true>(s, st);
  return f16 ? launch_decode<__half, 64, false>(s, st) : launch_decode<__nv_bfloat16, 64, false>(s, st);
}

extern "C" int cb200_attn_decode_static_scratch_status(void* stream) {
  unsigned char* scratch = nullptr;
  const int rc = cb200::static_scratch_address(&scratch);
  if (rc != CB200_OK) return rc;
  return cb200_workspace_status(scratch, stream);
}

extern "C" size_t cb200_attn_decode_workspace_bytes(const cb200_attn_decode_args* a) {
  cb200::DecodeSetup s;
  if (cb200::plan_decode(a, &s, false) != CB200_OK) return 0;
  return s.ws_needed;
}

extern "C" int cb200_attn_decode(const cb200_attn_decode_args* a, void* stream) {
  using namespace cb200;
  DecodeSetup s;
  const int rc = plan_decode(a, &s, true);
  if (rc != CB200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f16 = a->dtype == CB200_F16;
  if (a->head_dim == 128) {
    if (s.gather) return f16 ? launch_decode<__half, 128, true>(s, st) : launch_decode<__nv_bfloat16, 128, true>(s, st);
    return f16 ? launch_decode<__half, 128, false>(s, st) : launch_decode<__nv_bfloat16, 128, false>(s, st);
  }
  if (s.gather) return f16 ? launch_decode<__half, 64, true>(s, st) : launch_decode<__nv_bfloat16, 64, true>(s, st);
  return f16 ? launch_decode<__half, 64, false>(s, st) : launch_decode<__nv_bfloat16, 64, false>(s, st);
}
