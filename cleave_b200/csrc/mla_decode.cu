// MLA (multi-head latent attention) decode for sm_100a, absorbed-latent form:
//   S = (Q_nope CKV^T + Q_pe KPE^T) * scale,  O = softmax(S) CKV     (the latent is both K and V)
// for contiguous caches (static operator) and for paged caches with one token per page.
//
// One persistent launch, one CTA per SM. A work item is (request, block of 16 * NHB heads); its KV
// is cut into tiles of 64 tokens and the tiles of all items form one stream split evenly over the
// CTAs (same scheme as the GQA decode kernel); items cut across CTAs are finished by the last
// CTA to arrive (fused log-sum-exp combine).
//
// Inside a CTA a producer warp streams (CKV, KPE) tiles into a two-stage shared-memory ring (TMA
// tiled loads with the 128-byte swizzle for contiguous caches, one bulk copy per gathered row
// otherwise). The four consumer warps each compute S for 16 of the tile's 64 tokens (for every
// 16-head block of the item, so that a K fragment feeds several MMAs), agree on the tile's row
// maxima through shared memory, publish P = exp2(S - m) as 16-bit values, and then each
// accumulates O for its own 128 of the 512 latent columns: the CKV tile is read from HBM once and
// used as K and as V.
//
// Semantics follow demo/mla_decode.py:8-13 (static) and python/cleave/dynamic/reference.py:108-128,
// 297-320 (paged) of the reference; it replaces
// tests/graph/handwritten/expected_kernels/mla_paged_decode_h16_ckv512_kpe64_ps1.py and the split pair
// tests/graph/handwritten/expected_kernels/splitkv/mla_paged_decode_*_splitkv8.py.

#include "common.cuh"
#include "stream_walk.cuh"

#include <cstring>

namespace cb200 {

// tcgen05 variant for contiguous caches (mla_decode_tc.cu)
bool mla_tc_supported(const cb200_mla_decode_args* a);
size_t mla_tc_partial_bytes(const cb200_mla_decode_args* a, int sms);
int launch_mla_tc(const cb200_mla_decode_args* a, int* status, void* scratch, cudaStream_t stream);
// mla_paged_tc.cu: the paged form with at most 16 heads on tcgen05 (tokens as MMA rows).
bool mla_paged_tc_supported(const cb200_mla_decode_args* a);
int launch_mla_paged_tc(const cb200_mla_decode_args* a, int* status, float* partials, int* counters, int grid,
                        cudaStream_t stream);

namespace mla {

constexpr int kTile = 64;     // tokens per KV tile
constexpr int kCkv = 512;     // latent width
constexpr int kKpe = 64;      // rope width
constexpr int kQk = kCkv + kKpe;
constexpr int kStages = 2;
constexpr float kLog2e = 1.4426950408889634f;

struct Params {
  const void* q_nope;
  const void* q_pe;
  const void* ckv;
  const void* kpe;
  const int* kv_indptr;
  const int* kv_indices;
  const int* kv_start;  // optional: request b reads kv_indices[kv_start[b] .. + kv_lens[b]) (ranges may overlap)
  const int* kv_lens;
  void* out;
  float* lse;
  int* status;
  int* counters;
  float* partials;
  int batch, heads, head_blocks, kv_len, paged, num_pages, n_idx;
  float scale_log2;
};

// Token range of a paged request: from the (batch + 1) offsets, or from explicit per-request start and
// length arrays (causal prefill runs one request per query token over a prefix of its sequence's pages).
// The range is clipped to the n_idx entries kv_indices holds, so that offsets that run past the array are
// read as a shorter request, never as memory beyond it.
__device__ __forceinline__ int req_base(const Params& p, int b) {
  const int base = p.kv_start ? __ldg(p.kv_start + b) : p.kv_indptr[b];
  return min(max(base, 0), p.n_idx);
}
__device__ __forceinline__ int req_len(const Params& p, int b) {
  const int base = p.kv_start ? __ldg(p.kv_start + b) : p.kv_indptr[b];
  const int end = p.kv_lens ? base + max(__ldg(p.kv_lens + b), 0) : p.kv_indptr[b + 1];
  return max(min(end, p.n_idx) - min(max(base, 0), p.n_idx), 0);
}

template <int NHB, bool GATHER>
struct Smem {
  static constexpr int kRows = 16 * NHB;                 // heads per CTA
  static constexpr int kQPitch = kQk * 2 + 16;           // padded Q row
  static constexpr int kQBytes = kRows * kQPitch;
  static constexpr int kCkvPitch = GATHER ? kCkv * 2 + 16 : 128;
  static constexpr int kKpePitch = GATHER ? kKpe * 2 + 16 : 128;
  static constexpr int kCkvBytes = GATHER ? kTile * kCkvPitch : kTile * kCkv * 2;
  static constexpr int kKpeBytes = GATHER ? kTile * kKpePitch : kTile * kKpe * 2;
  static constexpr int kStageBytes = (kCkvBytes + kKpeBytes + 1023) / 1024 * 1024;
  static constexpr int kPPitch = kTile * 2 + 16;         // padded P row (64 tokens)
  static constexpr int kPBytes = kRows * kPPitch;
  static constexpr int kExchFloats = 4 * kRows;          // per-warp row maxima / row sums
  static constexpr int kFixed = kStages * kStageBytes + kQBytes + kPBytes + 2 * kExchFloats * 4 + 1024;  // barriers, flags, page ids
  static constexpr int kSlotFloats = kRows * kCkv + 2 * kRows;  // partial O, m, l
  static constexpr int kProducerWarps = GATHER ? 4 : 1;  // one TMA warp, or four row-gather warps
  static constexpr int kThreads = (4 + kProducerWarps) * 32;
};

template <typename T, int NHB, bool GATHER>
__global__ void __launch_bounds__(Smem<NHB, GATHER>::kThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tm_ckv, const __grid_constant__ CUtensorMap tm_kpe,
                  const Params p) {
  using L = Smem<NHB, GATHER>;
  constexpr int kConsumerWarps = 4;
  constexpr int kCThreads = kConsumerWarps * 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* q_smem = smem + kStages * L::kStageBytes;
  uint8_t* p_smem = q_smem + L::kQBytes;
  float* max_exch = reinterpret_cast<float*>(p_smem + L::kPBytes);
  float* sum_exch = max_exch + L::kExchFloats;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sum_exch + L::kExchFloats);
  uint64_t* empty_bar = full_bar + kStages;
  int* flags = reinterpret_cast<int*>(empty_bar + kStages);
  int* pg_smem = flags + 32;  // gather: page ids of the current and the next tile, 2 x 64
  int* P = reinterpret_cast<int*>(smem + L::kFixed);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = blockDim.x;

  // ---- tile prefix over requests (paged: every CTA computes the same table)
  int tiles_per_req = 0;
  if (p.paged) {
    int* scratch = reinterpret_cast<int*>(p_smem);  // free until the first tile
    const int per = ceil_div(p.batch, nthreads);
    const int i0 = min(tid * per, p.batch), i1 = min(i0 + per, p.batch);
    int sum = 0;
    for (int i = i0; i < i1; ++i) sum += ceil_div(req_len(p, i), kTile);
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
      run += ceil_div(req_len(p, i), kTile);
    }
  } else {
    tiles_per_req = ceil_div(p.kv_len, kTile);
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], GATHER ? L::kProducerWarps * 32 : 1);  // gather: one arrival per copying thread
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    mbar_fence_init();
    if (!GATHER) {
      tma_prefetch_desc(&tm_ckv);
      tma_prefetch_desc(&tm_kpe);
    }
  }
  __syncthreads();

  const int hb_count = p.head_blocks;  // items per request
  const int total = hb_count * (p.paged ? P[p.batch] : p.batch * tiles_per_req);
  const int G = gridDim.x;
  const int span = total > 0 ? ceil_div(total, G) : 1;
  const int u0 = min(static_cast<int>(blockIdx.x) * span, total);
  const int u1 = min(u0 + span, total);
  Walker walker{p.paged ? P : nullptr, p.batch, hb_count, tiles_per_req, 0};

  if (warp >= kConsumerWarps) {
    // ================================================================= producer warp(s)
    int stage = 0, phase = 0;
    for (int u = u0; u < u1;) {
      const Piece pc = walker.at(u, u1);
      const int valid = p.paged ? req_len(p, pc.b) : p.kv_len;
      const int base = p.paged ? req_base(p, pc.b) : 0;
      if constexpr (!GATHER) {
        for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
          mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
          uint8_t* ckv_dst = stages + stage * L::kStageBytes;
          uint8_t* kpe_dst = ckv_dst + L::kCkvBytes;
          if (lane == 0) {
            mbar_arrive_expect_tx(&full_bar[stage], kTile * kQk * 2);
#pragma unroll
            for (int c = 0; c < kCkv / 64; ++c)
              tma_load_3d(ckv_dst + c * (kTile * 128), &tm_ckv, &full_bar[stage], c * 64, t * kTile, pc.b);
            tma_load_3d(kpe_dst, &tm_kpe, &full_bar[stage], 0, t * kTile, pc.b);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      } else {
        // Row gather (one token per page): four warps copy the 64 latent rows (1024 + 128 bytes each) of a
        // tile with 16-byte cp.async into padded rows; consecutive lanes copy consecutive chunks of a row,
        // so a warp instruction moves 512 contiguous bytes. (One bulk copy per row was measured first:
        // 128 small bulk copies per tile kept the copy engine, not the memory, busy.) The page ids of the
        // next tile are staged in shared memory while the current one is copied.
        constexpr int kPThreads = L::kProducerWarps * 32;
        const int ptid = tid - kCThreads;
        const T* ckv = reinterpret_cast<const T*>(p.ckv);
        const T* kpe = reinterpret_cast<const T*>(p.kpe);
        auto stage_ids = [&](int t, int buf) {
          if (ptid < kTile) {
            const int tok = min(t * kTile + ptid, valid - 1);
            pg_smem[buf * kTile + ptid] = min(max(__ldg(p.kv_indices + base + tok), 0), p.num_pages - 1);
          }
        };
        named_bar_sync(3, kPThreads);  // the previous piece's last tile no longer reads the id buffers
        stage_ids(pc.tile0, 0);
        named_bar_sync(3, kPThreads);
        for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
          const int buf = (t - pc.tile0) & 1;
          if (t + 1 < pc.tile0 + pc.count) stage_ids(t + 1, buf ^ 1);
          mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
          const uint32_t ckv_dst = smem_u32(stages + stage * L::kStageBytes);
          const uint32_t kpe_dst = ckv_dst + L::kCkvBytes;
          constexpr int kCkvChunks = kCkv / 8, kKpeChunks = kKpe / 8;  // 16-byte chunks per row: 64 and 8
#pragma unroll 4
          for (int i = ptid; i < kTile * kCkvChunks; i += kPThreads) {
            const int row = i / kCkvChunks, c = i - row * kCkvChunks;
            const long long page = pg_smem[buf * kTile + row];
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ckv_dst + row * L::kCkvPitch + c * 16),
                         "l"(ckv + page * kCkv + c * 8) : "memory");
          }
#pragma unroll
          for (int i = ptid; i < kTile * kKpeChunks; i += kPThreads) {
            const int row = i / kKpeChunks, c = i - row * kKpeChunks;
            const long long page = pg_smem[buf * kTile + row];
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kpe_dst + row * L::kKpePitch + c * 16),
                         "l"(kpe + page * kKpe + c * 8) : "memory");
          }
          asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[stage])) : "memory");
          named_bar_sync(3, kPThreads);  // ids of tile t + 1 are in place; buffer `buf` may be rewritten
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      u += pc.count;
    }
    return;
  }

  // =================================================================== consumer warps
  // Warp ws computes S for tokens [16 ws, 16 ws + 16) of every tile and O for latent columns
  // [128 ws, 128 ws + 128), in both cases for all NHB 16-head blocks of the item: a K (or V)
  // fragment read from shared memory feeds NHB MMAs.
  const int ws = warp;
  const int r0 = lane >> 2, c2 = (lane & 3) * 2;
  const int mi = lane >> 3, rr = lane & 7;
  T* outp = reinterpret_cast<T*>(p.out);
  const uint32_t stages_u32 = smem_u32(stages), q_u32 = smem_u32(q_smem), p_u32 = smem_u32(p_smem);

  // Requests without any live token: out = 0, lse = -inf.
  if (p.paged) {
    for (int b = blockIdx.x; b < p.batch; b += G) {
      if (P[b + 1] - P[b] != 0) continue;
      for (int i = tid; i < p.heads * kCkv; i += kCThreads) outp[static_cast<size_t>(b) * p.heads * kCkv + i] = T(0.f);
      if (p.lse)
        for (int i = tid; i < p.heads; i += kCThreads) p.lse[static_cast<size_t>(b) * p.heads + i] = -INFINITY;
    }
  }

  int stage = 0, phase = 0;
  for (int u = u0; u < u1;) {
    const Piece pc = walker.at(u, u1);
    const int valid = p.paged ? req_len(p, pc.b) : p.kv_len;
    const int head0 = pc.hv * L::kRows;  // first head of the item

    // ---- stage Q (nope | pe) of the item's heads in shared memory; rows past the last head are zero
    named_bar_sync(1, kCThreads);  // the previous piece no longer reads Q
    {
      constexpr int kChunksPerRow = kQk / 8;  // 16-byte chunks
      const T* qn = reinterpret_cast<const T*>(p.q_nope);
      const T* qp = reinterpret_cast<const T*>(p.q_pe);
      for (int i = tid; i < L::kRows * kChunksPerRow; i += kCThreads) {
        const int r = i / kChunksPerRow, c = i - r * kChunksPerRow;
        const int head = head0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head < p.heads) {
          const size_t bh = static_cast<size_t>(pc.b) * p.heads + head;
          v = c < kCkv / 8 ? *reinterpret_cast<const uint4*>(qn + bh * kCkv + c * 8)
                           : *reinterpret_cast<const uint4*>(qp + bh * kKpe + (c - kCkv / 8) * 8);
        }
        *reinterpret_cast<uint4*>(q_smem + r * L::kQPitch + c * 16) = v;
      }
    }
    named_bar_sync(1, kCThreads);

    float acc[NHB][16][4];
    float m_run[NHB][2], l_run[NHB][2];
#pragma unroll
    for (int hb = 0; hb < NHB; ++hb) {
#pragma unroll
      for (int n = 0; n < 16; ++n) acc[hb][n][0] = acc[hb][n][1] = acc[hb][n][2] = acc[hb][n][3] = 0.f;
      m_run[hb][0] = m_run[hb][1] = -INFINITY;
      l_run[hb][0] = l_run[hb][1] = 0.f;
    }
    // ldmatrix row address of an A fragment (Q or P) for head block 0; block hb is 16 rows further
    const uint32_t q_row_addr = q_u32 + ((lane & 7) + ((lane >> 3) & 1) * 8) * L::kQPitch + (lane >> 4) * 16;
    const uint32_t p_row_addr = p_u32 + ((lane & 7) + ((lane >> 3) & 1) * 8) * L::kPPitch + (lane >> 4) * 16;

    for (int t = pc.tile0; t < pc.tile0 + pc.count; ++t) {
      mbar_wait(&full_bar[stage], phase, p.status, kFaultFullBarrier);
      const uint32_t ckv_base = stages_u32 + stage * L::kStageBytes;
      const uint32_t kpe_base = ckv_base + L::kCkvBytes;
      const int tok0 = t * kTile + ws * 16;

      // ---- S = Q_nope CKV^T + Q_pe KPE^T for this warp's 16 tokens, all head blocks
      float s[NHB][2][4], s2[NHB][2][4];
#pragma unroll
      for (int hb = 0; hb < NHB; ++hb)
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          s[hb][nb][0] = s[hb][nb][1] = s[hb][nb][2] = s[hb][nb][3] = 0.f;
          s2[hb][nb][0] = s2[hb][nb][1] = s2[hb][nb][2] = s2[hb][nb][3] = 0.f;
        }
      {
        const int row = ws * 16 + (mi >> 1) * 8 + rr;  // token row of this lane's ldmatrix address
#pragma unroll 4
        for (int kk = 0; kk < kQk / 16; ++kk) {
          uint32_t addr;
          if (kk < kCkv / 16) {
            const int d = kk * 16 + (mi & 1) * 8;
            addr = GATHER ? ckv_base + row * L::kCkvPitch + d * 2
                          : ckv_base + (d >> 6) * (kTile * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4);
          } else {
            const int d = (kk - kCkv / 16) * 16 + (mi & 1) * 8;
            addr = GATHER ? kpe_base + row * L::kKpePitch + d * 2
                          : kpe_base + row * 128 + (((d >> 3) ^ (row & 7)) << 4);
          }
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, addr);
#pragma unroll
          for (int hb = 0; hb < NHB; ++hb) {
            uint32_t a[4];
            ldmatrix_x4(a[0], a[1], a[2], a[3], q_row_addr + hb * 16 * L::kQPitch + kk * 32);
            if (kk & 1) {  // odd K steps go to a second accumulator: half the dependent-MMA chain
              mma_16816<T>(s2[hb][0], a, b0, b1);
              mma_16816<T>(s2[hb][1], a, b2, b3);
            } else {
              mma_16816<T>(s[hb][0], a, b0, b1);
              mma_16816<T>(s[hb][1], a, b2, b3);
            }
          }
        }
#pragma unroll
        for (int hb = 0; hb < NHB; ++hb)
#pragma unroll
          for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[hb][nb][e] += s2[hb][nb][e];
      }
      // ---- tile-wide row maxima (the four warps agree through shared memory)
#pragma unroll
      for (int hb = 0; hb < NHB; ++hb) {
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int tok = tok0 + nb * 8 + c2 + (e & 1);
            const float x = tok < valid ? s[hb][nb][e] * p.scale_log2 : -INFINITY;
            s[hb][nb][e] = x;
            if (e < 2) mx0 = fmaxf(mx0, x); else mx1 = fmaxf(mx1, x);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if ((lane & 3) == 0) {
          max_exch[ws * L::kRows + hb * 16 + r0] = mx0;
          max_exch[ws * L::kRows + hb * 16 + r0 + 8] = mx1;
        }
      }
      named_bar_sync(2, kCThreads);
      float sc[NHB][2];
#pragma unroll
      for (int hb = 0; hb < NHB; ++hb) {
        float mt0 = -INFINITY, mt1 = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          mt0 = fmaxf(mt0, max_exch[w * L::kRows + hb * 16 + r0]);
          mt1 = fmaxf(mt1, max_exch[w * L::kRows + hb * 16 + r0 + 8]);
        }
        const float mn0 = fmaxf(m_run[hb][0], mt0), mn1 = fmaxf(m_run[hb][1], mt1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        sc[hb][0] = fast_exp2(m_run[hb][0] - mu0);
        sc[hb][1] = fast_exp2(m_run[hb][1] - mu1);
        m_run[hb][0] = mn0;
        m_run[hb][1] = mn1;
        // ---- P = exp2(S - m), published as 16-bit values for all four warps
        float ps0 = 0.f, ps1 = 0.f;
        uint8_t* prow0 = p_smem + (hb * 16 + r0) * L::kPPitch + (ws * 16 + c2) * 2;
        uint8_t* prow1 = prow0 + 8 * L::kPPitch;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          const float p0 = fast_exp2(s[hb][nb][0] - mu0), p1 = fast_exp2(s[hb][nb][1] - mu0);
          const float p2 = fast_exp2(s[hb][nb][2] - mu1), p3 = fast_exp2(s[hb][nb][3] - mu1);
          ps0 += p0 + p1;
          ps1 += p2 + p3;
          *reinterpret_cast<uint32_t*>(prow0 + nb * 16) = pack2<T>(p0, p1);
          *reinterpret_cast<uint32_t*>(prow1 + nb * 16) = pack2<T>(p2, p3);
        }
        l_run[hb][0] = l_run[hb][0] * sc[hb][0] + ps0;
        l_run[hb][1] = l_run[hb][1] * sc[hb][1] + ps1;
      }
      named_bar_sync(2, kCThreads);
#pragma unroll
      for (int hb = 0; hb < NHB; ++hb) {
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          acc[hb][n][0] *= sc[hb][0];
          acc[hb][n][1] *= sc[hb][0];
          acc[hb][n][2] *= sc[hb][1];
          acc[hb][n][3] *= sc[hb][1];
        }
      }
      // ---- O[:, 128 ws .. 128 ws + 127] += P CKV (the same tile, now as V)
#pragma unroll
      for (int ks = 0; ks < kTile / 16; ++ks) {
        uint32_t pf[NHB][4];
#pragma unroll
        for (int hb = 0; hb < NHB; ++hb)
          ldmatrix_x4(pf[hb][0], pf[hb][1], pf[hb][2], pf[hb][3], p_row_addr + hb * 16 * L::kPPitch + ks * 32);
        const int row = ks * 16 + (mi & 1) * 8 + rr;
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          const int d = ws * 128 + dp * 16 + (mi >> 1) * 8;
          const uint32_t addr = GATHER ? ckv_base + row * L::kCkvPitch + d * 2
                                       : ckv_base + (d >> 6) * (kTile * 128) + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, addr);
#pragma unroll
          for (int hb = 0; hb < NHB; ++hb) {
            mma_16816<T>(acc[hb][2 * dp], pf[hb], b0, b1);
            mma_16816<T>(acc[hb][2 * dp + 1], pf[hb], b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }

    // ---- finish the piece: total row sums over the four token slices
#pragma unroll
    for (int hb = 0; hb < NHB; ++hb) {
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        float l = l_run[hb][h2];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if ((lane & 3) == 0) sum_exch[ws * L::kRows + hb * 16 + r0 + 8 * h2] = l;
      }
    }
    named_bar_sync(2, kCThreads);
    const size_t bh = static_cast<size_t>(pc.b) * p.heads;
    const bool starts_here = (u == pc.unit0);
    const bool whole = starts_here && pc.count == pc.n_tiles;
    float* slot = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * L::kSlotFloats;

    auto store_final = [&](int hb, const float (&o)[16][4], float M0, float M1, float S0, float S1) {
      const int h0 = head0 + hb * 16 + r0, h1 = h0 + 8;
      const float inv0 = S0 > 0.f ? 1.f / S0 : 0.f, inv1 = S1 > 0.f ? 1.f / S1 : 0.f;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int col = ws * 128 + n * 8 + c2;
        if (h0 < p.heads)
          *reinterpret_cast<uint32_t*>(outp + (bh + h0) * kCkv + col) = pack2<T>(o[n][0] * inv0, o[n][1] * inv0);
        if (h1 < p.heads)
          *reinterpret_cast<uint32_t*>(outp + (bh + h1) * kCkv + col) = pack2<T>(o[n][2] * inv1, o[n][3] * inv1);
      }
      if (p.lse && ws == 0 && (lane & 3) == 0) {
        if (h0 < p.heads) p.lse[bh + h0] = S0 > 0.f ? M0 + fast_log2(S0) : -INFINITY;
        if (h1 < p.heads) p.lse[bh + h1] = S1 > 0.f ? M1 + fast_log2(S1) : -INFINITY;
      }
    };

#pragma unroll
    for (int hb = 0; hb < NHB; ++hb) {
      float L0 = 0.f, L1 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        L0 += sum_exch[w * L::kRows + hb * 16 + r0];
        L1 += sum_exch[w * L::kRows + hb * 16 + r0 + 8];
      }
      const int row0 = hb * 16 + r0, row1 = row0 + 8;  // rows inside the item
      if (whole) {
        store_final(hb, acc[hb], m_run[hb][0], m_run[hb][1], L0, L1);
      } else {
        // ---- leave a partial (unnormalised O, m, l); the last CTA to arrive combines
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          const int col = ws * 128 + n * 8 + c2;
          *reinterpret_cast<float2*>(slot + row0 * kCkv + col) = make_float2(acc[hb][n][0], acc[hb][n][1]);
          *reinterpret_cast<float2*>(slot + row1 * kCkv + col) = make_float2(acc[hb][n][2], acc[hb][n][3]);
        }
        if (ws == 0 && (lane & 3) == 0) {
          slot[L::kRows * kCkv + row0] = m_run[hb][0];
          slot[L::kRows * kCkv + row1] = m_run[hb][1];
          slot[L::kRows * kCkv + L::kRows + row0] = L0;
          slot[L::kRows * kCkv + L::kRows + row1] = L1;
        }
      }
    }
    if (!whole) {
      __threadfence();
      named_bar_sync(1, kCThreads);
      const int c_first = pc.unit0 / span, c_last = (pc.unit0 + pc.n_tiles - 1) / span;
      int* counter = p.counters + pc.b * hb_count + pc.hv;
      if (tid == 0) {
        const int old = atomicAdd(counter, 1);
        flags[0] = (old == c_last - c_first) ? 1 : 0;
      }
      named_bar_sync(1, kCThreads);
      if (flags[0]) {
        __threadfence();
#pragma unroll
        for (int hb = 0; hb < NHB; ++hb) {
          const int row0 = hb * 16 + r0, row1 = row0 + 8;
          float Mc0 = -INFINITY, Mc1 = -INFINITY, Lc0 = 0.f, Lc1 = 0.f;
#pragma unroll
          for (int n = 0; n < 16; ++n) acc[hb][n][0] = acc[hb][n][1] = acc[hb][n][2] = acc[hb][n][3] = 0.f;
          for (int cta = c_first; cta <= c_last; ++cta) {
            const float* src = p.partials + (static_cast<size_t>(cta) * 2 + (cta == c_first ? 1 : 0)) * L::kSlotFloats;
            const float mi0 = __ldcg(src + L::kRows * kCkv + row0), mi1 = __ldcg(src + L::kRows * kCkv + row1);
            const float li0 = __ldcg(src + L::kRows * kCkv + L::kRows + row0);
            const float li1 = __ldcg(src + L::kRows * kCkv + L::kRows + row1);
            const float Mn0 = fmaxf(Mc0, mi0), Mn1 = fmaxf(Mc1, mi1);
            const float Mu0 = Mn0 == -INFINITY ? 0.f : Mn0, Mu1 = Mn1 == -INFINITY ? 0.f : Mn1;
            const float a0 = fast_exp2(Mc0 - Mu0), b0 = fast_exp2(mi0 - Mu0);
            const float a1 = fast_exp2(Mc1 - Mu1), b1 = fast_exp2(mi1 - Mu1);
            Lc0 = a0 * Lc0 + b0 * li0;
            Lc1 = a1 * Lc1 + b1 * li1;
#pragma unroll
            for (int n0 = 0; n0 < 16; n0 += 4) {  // four column blocks' loads in flight together
              float2 x0[4], x1[4];
#pragma unroll
              for (int n = 0; n < 4; ++n) {
                const int col = ws * 128 + (n0 + n) * 8 + c2;
                x0[n] = __ldcg(reinterpret_cast<const float2*>(src + row0 * kCkv + col));
                x1[n] = __ldcg(reinterpret_cast<const float2*>(src + row1 * kCkv + col));
              }
#pragma unroll
              for (int n = 0; n < 4; ++n) {
                acc[hb][n0 + n][0] = a0 * acc[hb][n0 + n][0] + b0 * x0[n].x;
                acc[hb][n0 + n][1] = a0 * acc[hb][n0 + n][1] + b0 * x0[n].y;
                acc[hb][n0 + n][2] = a1 * acc[hb][n0 + n][2] + b1 * x1[n].x;
                acc[hb][n0 + n][3] = a1 * acc[hb][n0 + n][3] + b1 * x1[n].y;
              }
            }
            Mc0 = Mn0;
            Mc1 = Mn1;
          }
          store_final(hb, acc[hb], Mc0, Mc1, Lc0, Lc1);
        }
        if (tid == 0) *counter = 0;  // ready for the next launch
      }
    }
    u += pc.count;
  }
}

}  // namespace mla

// ------------------------------------------------------------------------------------- host side
namespace {

struct MlaSetup {
  mla::Params p;
  int nhb, grid, smem_bytes;
  bool gather, use_tc, use_paged_tc;
  int paged_tc_grid;
  size_t ws_needed, partials_off, counters_off, tc_partials_off;
  CUtensorMap tm_ckv, tm_kpe;
};

int plan_mla(const cb200_mla_decode_args* a, MlaSetup* s, bool need_maps) {
  using namespace mla;
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->batch <= 0 || a->num_heads <= 0) return CB200_ERR_BAD_ARG;
  if (a->ckv_dim != kCkv || a->kpe_dim != kKpe) return CB200_ERR_UNSUPPORTED;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  const bool paged = a->kv_indptr != nullptr;
  if (paged && a->page_size != 1) return CB200_ERR_UNSUPPORTED;  // the reference's MLA cache holds one token per page
  if (paged && (a->num_pages <= 0 || a->num_kv_indices < 0)) return CB200_ERR_BAD_ARG;
  if (!paged && a->kv_len <= 0) return CB200_ERR_BAD_ARG;
  Params& p = s->p;
  p = Params{};
  p.batch = a->batch;
  p.heads = a->num_heads;
  s->nhb = a->num_heads > 16 ? 2 : 1;
  const int rows = 16 * s->nhb;
  p.head_blocks = ceil_div(a->num_heads, rows);
  p.kv_len = a->kv_len;
  p.paged = paged ? 1 : 0;
  p.num_pages = a->num_pages;
  p.n_idx = a->num_kv_indices;
  p.scale_log2 = a->sm_scale * kLog2e;
  s->gather = paged;
  const long long tiles_ub = paged ? (static_cast<long long>(a->num_kv_indices) + kTile - 1) / kTile + a->batch
                                   : static_cast<long long>(a->batch) * ceil_div(a->kv_len, kTile);
  const long long units_ub = (a->kv_lens ? (1LL << 20) : tiles_ub) * p.head_blocks;  // explicit ranges may overlap: no bound from the index count
  if (units_ub >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  int grid = sms;
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  const int fixed = s->nhb == 2 ? (s->gather ? Smem<2, true>::kFixed : Smem<2, false>::kFixed)
                                : (s->gather ? Smem<1, true>::kFixed : Smem<1, false>::kFixed);
  s->smem_bytes = fixed + (paged ? (a->batch + 1) * 4 : 0) + 1024 + 16;
  if (s->smem_bytes > 227 * 1024) return CB200_ERR_UNSUPPORTED;
  constexpr size_t kSlotBytesMax = static_cast<size_t>(Smem<2, false>::kSlotFloats) * 4;
  s->partials_off = kWsHeaderBytes;
  s->counters_off = align_up(s->partials_off + static_cast<size_t>(sms) * 2 * kSlotBytesMax, 256);
  // Layout: header | partial slots of the mma.sync kernel | arrival counters (shape-independent
  // offset, shared by both paths) | P, block statistics and partial slots of the tcgen05 kernels.
  // "auto" takes the tcgen05 pair of kernels for contiguous caches when its 128-row MMAs are at least
  // half full and there are enough token blocks to spread over the SMs; the warp-MMA kernel serves
  // paged caches, few heads and short caches.
  s->use_tc = mla_tc_supported(a) &&
              (a->impl == CB200_MLA_IMPL_TCGEN05 ||
               (a->impl == CB200_MLA_IMPL_AUTO && a->num_heads >= 64 && a->kv_len >= 512));
  // paged caches with at most 16 heads: the tcgen05 kernel that takes the tokens as MMA rows
  s->use_paged_tc = paged && a->impl != CB200_MLA_IMPL_MMA_SYNC && mla_paged_tc_supported(a);
  {
    // its tiles hold 64 tokens, and every request with tokens carries two overhead units (the stream is cut by cost)
    const long long tiles = (static_cast<long long>(a->num_kv_indices) + 63) / 64 + 3LL * a->batch;
    s->paged_tc_grid = static_cast<int>(tiles < grid ? (tiles > 0 ? tiles : 1) : grid);
  }
  if (a->impl == CB200_MLA_IMPL_TCGEN05 && !s->use_tc && !s->use_paged_tc) return CB200_ERR_UNSUPPORTED;
  const size_t n_counters = static_cast<size_t>(a->batch) * (p.head_blocks > 2 * ceil_div(a->num_heads, 128)
                                                                ? p.head_blocks : 2 * ceil_div(a->num_heads, 128));
  if (n_counters > kWsCounterSlots) {  // the scratch of the tcgen05 kernels would start inside the counters
    if (a->impl == CB200_MLA_IMPL_TCGEN05) return CB200_ERR_UNSUPPORTED;
    s->use_tc = false;
  }
  s->tc_partials_off = align_up(s->counters_off + (n_counters > kWsCounterSlots ? n_counters : kWsCounterSlots) * 4, 256);
  s->ws_needed = s->tc_partials_off + (s->use_tc ? mla_tc_partial_bytes(a, sms) : 0);
  s->grid = static_cast<int>(units_ub < grid ? (units_ub > 0 ? units_ub : 1) : grid);
  if (!need_maps) return CB200_OK;

  if (!a->q_nope || !a->q_pe || !a->ckv_cache || !a->kpe_cache || !a->out) return CB200_ERR_BAD_ARG;
  if (paged && !a->kv_indices && a->num_kv_indices > 0) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q_nope) | reinterpret_cast<uintptr_t>(a->q_pe) |
       reinterpret_cast<uintptr_t>(a->ckv_cache) | reinterpret_cast<uintptr_t>(a->kpe_cache) |
       reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < s->ws_needed) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return CB200_ERR_ALIGNMENT;
  p.q_nope = a->q_nope;
  p.q_pe = a->q_pe;
  p.ckv = a->ckv_cache;
  p.kpe = a->kpe_cache;
  p.kv_indptr = a->kv_indptr;
  p.kv_indices = a->kv_indices;
  p.kv_start = paged ? a->kv_start : nullptr;
  p.kv_lens = paged ? a->kv_lens : nullptr;
  p.out = a->out;
  p.lse = a->lse;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(ws + s->partials_off);
  p.counters = reinterpret_cast<int*>(ws + s->counters_off);
  if (!s->gather) {
    const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    uint32_t box[3] = {64u, static_cast<uint32_t>(kTile), 1u};
    uint64_t dims_c[3] = {kCkv, static_cast<uint64_t>(a->kv_len), static_cast<uint64_t>(a->batch)};
    uint64_t str_c[2] = {kCkv * 2, static_cast<uint64_t>(a->kv_len) * kCkv * 2};
    uint64_t dims_k[3] = {kKpe, static_cast<uint64_t>(a->kv_len), static_cast<uint64_t>(a->batch)};
    uint64_t str_k[2] = {kKpe * 2, static_cast<uint64_t>(a->kv_len) * kKpe * 2};
    if (!encode_tensor_map(&s->tm_ckv, dt, 3, const_cast<void*>(a->ckv_cache), dims_c, str_c, box, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_tensor_map(&s->tm_kpe, dt, 3, const_cast<void*>(a->kpe_cache), dims_k, str_k, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
  } else {
    memset(&s->tm_ckv, 0, sizeof(CUtensorMap));
    memset(&s->tm_kpe, 0, sizeof(CUtensorMap));
  }
  return CB200_OK;
}

template <typename T, int NHB, bool GATHER>
int launch_mla(const MlaSetup& s, cudaStream_t stream) {
  auto kern = mla::mla_decode_kernel<T, NHB, GATHER>;
  static bool configured[64] = {false};
  int dev = 0;
  CB200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev < 64) configured[dev] = true;
  }
  kern<<<s.grid, mla::Smem<NHB, GATHER>::kThreads, s.smem_bytes, stream>>>(s.tm_ckv, s.tm_kpe, s.p);
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

template <typename T>
int dispatch_mla(const MlaSetup& s, cudaStream_t st) {
  if (s.nhb == 2) return s.gather ? launch_mla<T, 2, true>(s, st) : launch_mla<T, 2, false>(s, st);
  return s.gather ? launch_mla<T, 1, true>(s, st) : launch_mla<T, 1, false>(s, st);
}

}  // namespace
}  // namespace cb200

extern "C" size_t cb200_mla_decode_workspace_bytes(const cb200_mla_decode_args* a) {
  cb200::MlaSetup s;
  if (cb200::plan_mla(a, &s, false) != CB200_OK) return 0;
  return s.ws_needed;
}

extern "C" int cb200_mla_decode(const cb200_mla_decode_args* a, void* stream) {
  using namespace cb200;
  MlaSetup s;
  const int rc = plan_mla(a, &s, true);
  if (rc != CB200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s.use_paged_tc)
    return launch_mla_paged_tc(a, s.p.status, s.p.partials, s.p.counters, s.paged_tc_grid, st);
  if (s.use_tc)
    return launch_mla_tc(a, s.p.status, static_cast<uint8_t*>(a->workspace) + s.tc_partials_off, st);
  return a->dtype == CB200_F16 ? dispatch_mla<__half>(s, st) : dispatch_mla<__nv_bfloat16>(s, st);
}
