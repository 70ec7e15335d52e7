// MLA decode on the tcgen05 tensor cores for contiguous caches (the static operator), in two
// kernels that meet in the workspace:
//
//   scores   P = exp2(scale * Q K^T - m)  per block of 128 tokens, with the block's row maximum m and
//            row sum l. A CTA owns (request, block of up to 128 heads, a range of token blocks). Q
//            (128 heads x 576) and the latent and rope caches stream together through a four-stage
//            ring, a 64-column chunk of Q beside 64 columns x 256 tokens of cache, so every MMA
//            is 128 x 256 x 16. S sits in tensor memory (two buffers of 256 columns); eight epilogue
//            warps (thread = head row = TMEM lane, one warp group per 128-token block) turn it into
//            P in the cache's 16-bit type and write P, m and l to the workspace.
//   values   O = sum_blocks 2^(m_block - m_ref) P_block V_block / l. A CTA owns (request, head block,
//            a part of 128 or 256 of the 512 output columns, one of S token ranges). m_ref is the
//            largest block maximum of the CTA's range - every block's statistics are already in
//            memory - so the factors are at most 1 and O never needs rescaling. P tiles arrive in
//            shared memory by bulk copies (one warp) and the latent tile (128 tokens x the CTA's
//            columns, MN-major) by TMA (another warp); two groups of four warps (thread = head row
//            = TMEM lane) take alternate blocks: read the P rows, multiply by the factor, store them
//            to tensor memory, where they are the A operand. O stays in tensor memory. The S CTAs
//            of an item are one thread-block cluster and combine their partial results through
//            distributed shared memory (rows dealt to the ranks, peers added in rank order); the
//            kernel is launched with programmatic stream serialization, so its set-up and first V
//            tiles overlap the tail of the scores kernel, and waits (griddepcontrol.wait) before it
//            touches P.
//
// Why two kernels: the accumulator for 128 heads x 512 columns fills tensor memory on its own, and
// Q plus a KV tile large enough for full-width MMAs does not fit in shared memory. Splitting the
// work at P keeps every MMA 256 wide; P (2 bytes per head and token) is small next to the caches
// and is still in L2 when the second kernel reads it.
//
// Reference semantics: demo/mla_decode.py:8-13.

#include "common.cuh"

#include <cstring>
#include <type_traits>

namespace cb200 {
namespace mlatc {

constexpr int kCkv = 512, kKpe = 64, kQk = 576;
constexpr int kChunks = kQk / 64;        // 9 chunks of 64 columns (128 bytes)
constexpr int kBlk = 128;                // tokens per block of P
constexpr float kLog2e = 1.4426950408889634f;

// ---- scores kernel
constexpr int kQChunkBytes = 128 * 128;             // 128 heads x 128 bytes
constexpr int kSTile = 256;                         // tokens per MMA tile (two blocks)
constexpr int kKChunkBytes = kSTile * 128;          // 32 768
constexpr int kKStageBytes = kQChunkBytes + kKChunkBytes;  // a Q chunk and the matching cache chunk
constexpr int kKStages = 4;
constexpr int kScoreSmem = kKStages * kKStageBytes + 1024 + 1024;
constexpr int kScoreThreads = 320;                  // producer, MMA, eight epilogue warps

// ---- values kernel
constexpr int kVRingBytes = 3 * 65536;              // the V ring, whatever the column split
constexpr int kVChunkBytes = kBlk * 128;            // 64 columns x 128 tokens
constexpr int kValueSmem = kVRingBytes + 2048 /*barriers, row sums*/ + 1024 /*alignment*/;
constexpr int kValueThreads = 352;  // V producer, MMA, two groups of four P-scaling warps, P producer
constexpr uint32_t kColO = 0, kColP = 256;          // P: two buffers of 64 columns

struct Params {
  void* out;
  float* lse;
  int* status;
  void* pbuf;      // (batch, head blocks, token blocks) tiles of 128 rows x 128 tokens, 16-bit
  float2* stats;   // (batch, head blocks, token blocks, 128 rows): (m, l) per row and block
  int batch, heads, head_blocks, kv_len, kv_pad, blocks;
  int ranges, blocks_per_range;   // scores kernel
  int splits, blocks_per_split;   // values kernel
  float scale_log2;
};

template <typename T>
__global__ void __launch_bounds__(kScoreThreads, 1)
mla_scores_kernel(const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp,
                  const __grid_constant__ CUtensorMap tm_ckv, const __grid_constant__ CUtensorMap tm_kpe,
                  const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_smem = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kKStages * kKStageBytes);
  uint64_t* k_full = bars;                  // [kKStages] TMA landed
  uint64_t* k_empty = bars + kKStages;      // [kKStages] the MMAs have read the stage
  uint64_t* s_full = bars + 2 * kKStages;   // [2] S complete in TMEM
  uint64_t* s_empty = s_full + 2;           // [2] the epilogue has read S
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(s_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int x = blockIdx.x;
  const int rg = x % p.ranges; x /= p.ranges;
  const int hb = x % p.head_blocks;
  const int b = x / p.head_blocks;
  const int u0 = min(rg * p.blocks_per_range, p.blocks);
  const int u1 = min(u0 + p.blocks_per_range, p.blocks);
  const int n_tiles = (u1 - u0 + 1) / 2;  // MMA tiles of two blocks

  if (tid == 0) {
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_qn);
    tma_prefetch_desc(&tm_qp);
    tma_prefetch_desc(&tm_ckv);
    tma_prefetch_desc(&tm_kpe);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  // This grid is itself a dependent launch: it was scheduled while the preceding kernel of the stream (in a
  // decode loop, the kernel that appended this step's rows to the caches) drains. Everything up to here
  // was set-up; nothing in global memory is read or written before the wait.
  pdl_wait();
  // Only now may the values kernel start: it fetches cache tiles before its own wait, so it must never
  // run beside a kernel older than this one (one that may still be writing the caches).
  pdl_launch_dependents();

  if (warp == 0) {
    // ================================================================ TMA producer
    // Q is streamed with the cache (a CTA has only a few tiles; Q comes from L2 after the first
    // touch), which leaves the whole of shared memory to the ring: 192 KB in flight per SM.
    int st = 0, ph = 0;
    for (int t = 0; t < n_tiles; ++t) {
      const int tok0 = (u0 + 2 * t) * kBlk;
      for (int c = 0; c < kChunks; ++c) {
        mbar_wait(&k_empty[st], ph ^ 1, p.status, kFaultEmptyBarrier);
        if (elect_one()) {
          uint8_t* q_dst = k_smem + st * kKStageBytes;
          uint8_t* k_dst = q_dst + kQChunkBytes;
          mbar_arrive_expect_tx(&k_full[st], kKStageBytes);
          if (c < kCkv / 64) {
            tma_load_3d(k_dst, &tm_ckv, &k_full[st], c * 64, tok0, b);
            tma_load_3d(q_dst, &tm_qn, &k_full[st], c * 64, hb * 128, b);
          } else {
            tma_load_3d(k_dst, &tm_kpe, &k_full[st], 0, tok0, b);
            tma_load_3d(q_dst, &tm_qp, &k_full[st], 0, hb * 128, b);
          }
        }
        __syncwarp();
        if (++st == kKStages) { st = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr uint32_t idesc = umma_idesc(std::is_same<T, __nv_bfloat16>::value, /*b_mn_major=*/false, 128, kSTile);
    const uint32_t k_addr = smem_u32(k_smem);
    int st = 0, ph = 0;
    for (int t = 0; t < n_tiles; ++t) {
      const int sb = t & 1;
      mbar_wait(&s_empty[sb], ((t >> 1) & 1) ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      const uint32_t d = tmem_base + sb * kSTile;
      for (int c = 0; c < kChunks; ++c) {
        mbar_wait(&k_full[st], ph, p.status, kFaultFullBarrier);
        tc_fence_after();
        if (elect_one()) {
          const uint32_t q_addr = k_addr + st * kKStageBytes;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adesc = umma_smem_desc(q_addr + kk * 32, 16, 8 * 128);
            const uint64_t bdesc = umma_smem_desc(q_addr + kQChunkBytes + kk * 32, 16, 8 * 128);
            umma_f16(d, adesc, bdesc, idesc, (c > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&k_empty[st]);
        }
        __syncwarp();
        if (++st == kKStages) { st = 0; ph ^= 1; }
      }
      if (elect_one()) umma_commit(&s_full[sb]);
      __syncwarp();
    }
  } else {
    // ================================================================ epilogue: S -> P, m, l
    const int quarter = warp & 3;          // the TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;      // which block of the MMA tile
    const int row = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    for (int t = 0; t < n_tiles; ++t) {
      const int sb = t & 1;
      const int u = u0 + 2 * t + half;
      mbar_wait(&s_full[sb], (t >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      uint32_t r[4][32];
      if (u < u1) {
        const uint32_t t_s = tmem_base + lane_field + sb * kSTile + half * kBlk;
#pragma unroll
        for (int q = 0; q < 4; ++q) tmem_ld_32x32(t_s + q * 32, r[q]);
        tmem_ld_wait();
      }
      // S is in registers: the MMAs may reuse the buffer while P is computed and stored
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      if (u < u1) {
        const int tok0 = u * kBlk;
        float mx = -INFINITY;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = tok0 + q * 32 + i < p.kv_len ? __uint_as_float(r[q][i]) * p.scale_log2 : -INFINITY;
            r[q][i] = __float_as_uint(v);
            mx = fmaxf(mx, v);
          }
        }
        const float m = mx == -INFINITY ? 0.f : mx;
        float l = 0.f;
        // P tile of (head block, token block): 16-byte piece k of row r at piece index k * 128 + r, so
        // that a warp's store (and the values kernel's load) covers 512 contiguous bytes
        const size_t tile = (static_cast<size_t>(b) * p.head_blocks + hb) * p.blocks + u;
        uint4* ptile = reinterpret_cast<uint4*>(p.pbuf) + tile * (kBlk * 128 / 8);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float e[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              e[k] = fast_exp2(__uint_as_float(r[q][i + k]) - m);  // exp2(-inf) = 0 for masked tokens
              l += e[k];
            }
            uint4 q4;
            q4.x = pack2<T>(e[0], e[1]);
            q4.y = pack2<T>(e[2], e[3]);
            q4.z = pack2<T>(e[4], e[5]);
            q4.w = pack2<T>(e[6], e[7]);
            ptile[(q * 4 + (i >> 3)) * 128 + row] = q4;
          }
        }
        p.stats[tile * 128 + row] = make_float2(m, l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- values kernel: warp roles 0 = V producer (TMA), 10 = P tile producer (bulk copies), 1 = MMA
// issuer and TMEM owner, 2..5 and 6..9 = two groups of P-scaling warps (thread = head row = TMEM lane); group g owns P buffer g and the token
// blocks j = g (mod 2), so two blocks' loads are in flight while a third is multiplied.
// DV = output columns per CTA: 256 (two column parts per item) or 128 (four parts, half as many
// token splits for the same number of CTAs, so a quarter of the combine traffic per CTA).
template <typename T, int DV>
__global__ void __launch_bounds__(kValueThreads, 1)
mla_values_kernel(const __grid_constant__ CUtensorMap tm_ckv, const Params p) {
  constexpr int kDvHalf = DV;
  constexpr int kVStageBytes = (DV / 64) * kVChunkBytes;  // 64 KB or 32 KB
  constexpr int kVStages = DV == 256 ? 2 : 3;
  constexpr int kPTileBytes = kBlk * 128 * 2;            // one P tile: 128 rows x 128 tokens
  constexpr int kPStages = (kVRingBytes - kVStages * kVStageBytes) / kPTileBytes;  // 2 or 3
  constexpr int kParts = kCkv / DV, kGroups = DV / 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* v_smem = smem;
  uint8_t* pt_smem = smem + kVStages * kVStageBytes;  // P tiles as the scores kernel wrote them
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kVRingBytes);
  uint64_t* v_full = bars;                 // [kVStages] TMA landed
  uint64_t* v_empty = bars + kVStages;     // [kVStages] the MMAs have read the stage
  uint64_t* pt_full = bars + 2 * kVStages; // [kPStages] P tile landed
  uint64_t* pt_empty = pt_full + kPStages; // [kPStages] the four warps of a group have read the tile
  uint64_t* p_full = pt_empty + kPStages;  // [2] scaled P stored to TMEM
  uint64_t* p_empty = p_full + 2;          // [2] the MMAs that read the P buffer have completed
  uint64_t* o_done = p_empty + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  float* l_part = reinterpret_cast<float*>(bars + 32);  // [2][128] row sums of the two groups

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.splits;  // the S CTAs of an item are one cluster (S = 1: no cluster)
  int x = blockIdx.x;
  const int split = x % S; x /= S;
  const int dh = x % kParts; x /= kParts;
  const int hb = x % p.head_blocks;
  const int b = x / p.head_blocks;
  const int t0 = min(split * p.blocks_per_split, p.blocks);
  const int t1 = min(t0 + p.blocks_per_split, p.blocks);
  const int nt = t1 - t0;

  if (tid == 0) {
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&pt_full[s], 1);
      mbar_init(&pt_empty[s], 4);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&p_full[s], 4);
      mbar_init(&p_empty[s], 1);
    }
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_ckv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  pdl_launch_dependents();  // the next kernel of the stream may be scheduled as this grid's CTAs retire

  if (warp == 0) {
    // ================================================================ TMA producer
    // V does not depend on the scores kernel: its first stages are fetched while that kernel drains.
    int vst = 0, vph = 0, jv = 0;
    auto load_v = [&]() {
      mbar_wait(&v_empty[vst], vph ^ 1, p.status, kFaultEmptyBarrier);
      if (elect_one()) {
        uint8_t* dst = v_smem + vst * kVStageBytes;
        mbar_arrive_expect_tx(&v_full[vst], kVStageBytes);
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_3d(dst + c * kVChunkBytes, &tm_ckv, &v_full[vst], dh * DV + c * 64, (t0 + jv) * kBlk, b);
      }
      __syncwarp();
      ++jv;
      if (++vst == kVStages) { vst = 0; vph ^= 1; }
    };
    while (jv < nt) load_v();
    if (S > 1) {  // the two meetings of the combine
      cluster_sync();
      cluster_sync();
    }
  } else if (warp == 10) {
    // ================================================================ P tile producer
    pdl_wait();  // P comes from the scores kernel
    const uint8_t* ptiles = reinterpret_cast<const uint8_t*>(p.pbuf) +
                            ((static_cast<size_t>(b) * p.head_blocks + hb) * p.blocks + t0) * kPTileBytes;
    int pst = 0, pph = 0;
    for (int j = 0; j < nt; ++j) {
      mbar_wait(&pt_empty[pst], pph ^ 1, p.status, kFaultEmptyBarrier);
      if (elect_one()) {
        mbar_arrive_expect_tx(&pt_full[pst], kPTileBytes);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          bulk_load_1d(pt_smem + pst * kPTileBytes + q * (kPTileBytes / 4),
                       ptiles + static_cast<size_t>(j) * kPTileBytes + q * (kPTileBytes / 4), kPTileBytes / 4, &pt_full[pst]);
      }
      __syncwarp();
      if (++pst == kPStages) { pst = 0; pph ^= 1; }
    }
    if (S > 1) {
      cluster_sync();
      cluster_sync();
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr uint32_t idesc = umma_idesc(std::is_same<T, __nv_bfloat16>::value, /*b_mn_major=*/true, 128, kDvHalf);
    const uint32_t v_addr0 = smem_u32(v_smem);
    int st = 0, ph = 0;
    for (int j = 0; j < nt; ++j) {
      const int pb = j & 1;
      mbar_wait(&v_full[st], ph, p.status, kFaultFullBarrier);
      mbar_wait(&p_full[pb], (j >> 1) & 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (elect_one()) {
        const uint32_t v_addr = v_addr0 + st * kVStageBytes;
#pragma unroll
        for (int ks = 0; ks < kBlk / 16; ++ks) {
          // B: MN-major, 16 token rows of 128 bytes per step; 64-column chunks are kVChunkBytes apart
          const uint64_t bdesc = umma_smem_desc(v_addr + ks * 16 * 128, kVChunkBytes, 8 * 128);
          umma_f16_ts(tmem_base + kColO, tmem_base + kColP + pb * 64 + ks * 8, bdesc, idesc, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&p_empty[pb]);
        if (j == nt - 1) umma_commit(o_done);
      }
      __syncwarp();
      if (++st == kVStages) { st = 0; ph ^= 1; }
    }
    if (S > 1) {
      cluster_sync();
      cluster_sync();
    }
  } else {
    // ================================================================ P scaling / epilogue
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;  // head row inside the block = TMEM lane
    const int etid = tid - 64;            // 0..255
    const int head = hb * 128 + row;
    const bool live = head < p.heads;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const size_t tile0 = (static_cast<size_t>(b) * p.head_blocks + hb) * p.blocks;
    pdl_wait();  // the statistics come from the scores kernel
    // The reference maximum is the largest block maximum of the whole range (the statistics of every
    // block are already in memory), so the factors are at most 1 and O never needs rescaling.
    float m_ref = -INFINITY;
    for (int j = 0; j < nt; ++j) m_ref = fmaxf(m_ref, p.stats[(tile0 + t0 + j) * 128 + row].x);
    if (m_ref == -INFINITY) m_ref = 0.f;
    float l_run = 0.f;
    for (int j = group; j < nt; j += 2) {
      const float2 st = p.stats[(tile0 + t0 + j) * 128 + row];  // second touch: L1
      const float f = fast_exp2(st.x - m_ref);
      l_run += st.y * f;
      const int pst = j % kPStages, pph = (j / kPStages) & 1;
      mbar_wait(&pt_full[pst], pph, p.status, kFaultFullBarrier);
      // 16-byte piece k of row r sits at piece index k * 128 + r: a warp reads 512 contiguous bytes
      const uint4* src = reinterpret_cast<const uint4*>(pt_smem + pst * kPTileBytes) + row;
      uint4 raw[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) raw[i] = src[i * 128];
      __syncwarp();
      if (lane == 0) mbar_arrive(&pt_empty[pst]);
      // the group's P buffer in TMEM is free once the MMAs of its previous block have completed
      mbar_wait(&p_empty[group], ((j >> 1) & 1) ^ 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      const uint32_t f2 = pack2<T>(f, f);
      uint32_t pk[32];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          pk[4 * i] = mul2<T>(raw[8 * h + i].x, f2);
          pk[4 * i + 1] = mul2<T>(raw[8 * h + i].y, f2);
          pk[4 * i + 2] = mul2<T>(raw[8 * h + i].z, f2);
          pk[4 * i + 3] = mul2<T>(raw[8 * h + i].w, f2);
        }
        tmem_st_32x32(tmem_base + lane_field + kColP + group * 64 + h * 32, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[group]);
    }
    // ---- epilogue: O / l, or the cluster combine. Both groups take half of the columns.
    l_part[group * 128 + row] = l_run;
    named_bar_sync(2, 256);
    const float L = l_part[row] + l_part[128 + row];  // the same sum in both groups
    if (nt > 0) {
      mbar_wait(o_done, 0, p.status, kFaultMmaBarrier);
      tc_fence_after();
    }
    const size_t hrow = static_cast<size_t>(b) * p.heads + head;
    T* outg = reinterpret_cast<T*>(p.out);
    const int cbeg = group * (kDvHalf / 2), cend = cbeg + kDvHalf / 2;
    if (S == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll 1
      for (int c0 = cbeg; c0 < cend; c0 += 32) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
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
            *reinterpret_cast<uint4*>(outg + hrow * kCkv + dh * kDvHalf + c0 + i) = q4;
          }
        }
      }
      if (live && group == 0 && dh == 0 && p.lse) p.lse[hrow] = L > 0.f ? m_ref + fast_log2(L) : -INFINITY;
    } else {
      // Split-KV combine inside the cluster: every CTA parks its fp32 accumulator, m and l in its own
      // shared memory (the ring is idle: all MMAs have completed), the cluster meets at a hardware
      // barrier, and CTA r combines rows [r, r + 1) * 128 / S over all peers through distributed
      // shared memory, in rank order (bit-stable). No workspace, no atomics, nobody spins.
      // Staging layout: [column group of 32][row][8 pieces of 16 bytes], piece i of row r stored at
      // i ^ (r & 7) so that a warp's stores spread over all banks.
      float* stg = reinterpret_cast<float*>(v_smem);
      float* ml = stg + 128 * kDvHalf;        // [128] m, [128] l
      float* cft = ml + 256;                  // [64 rows][8] combine factors (already divided by L)
#pragma unroll 1
      for (int c0 = cbeg; c0 < cend; c0 += 32) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(stg + (static_cast<size_t>(c0 >> 5) * 128 + row) * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i ^ (row & 7)] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                           __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
      }
      if (group == 0) {
        ml[row] = L > 0.f ? m_ref : -INFINITY;
        ml[128 + row] = L;
      }
      cluster_sync();
      const int r0 = split * 128 / S, r1 = (split + 1) * 128 / S, nrows = r1 - r0;  // at most 64
      const uint32_t stg_addr = smem_u32(stg), ml_addr = smem_u32(ml);
      if (etid < nrows) {  // factors of one row: 2 S remote loads in one round trip
        const int rr = r0 + etid;
        float ms[8], ls[8];
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
          ms[s2] = -INFINITY;
          ls[s2] = 0.f;
          if (s2 < S) {
            ms[s2] = dsmem_ld_f32(dsmem_addr(ml_addr + rr * 4, s2));
            ls[s2] = dsmem_ld_f32(dsmem_addr(ml_addr + (128 + rr) * 4, s2));
          }
        }
        float M = -INFINITY, L = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) M = fmaxf(M, ms[s2]);
        const float Mu = M == -INFINITY ? 0.f : M;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
          ms[s2] = fast_exp2(ms[s2] - Mu);
          L += ms[s2] * ls[s2];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) cft[etid * 8 + s2] = ms[s2] * inv;
        const int hd = hb * 128 + rr;
        if (hd < p.heads && dh == 0 && p.lse)
          p.lse[static_cast<size_t>(b) * p.heads + hd] = L > 0.f ? M + fast_log2(L) : -INFINITY;
      }
      named_bar_sync(2, 256);
      // A warp reads 512 contiguous bytes of a peer per load: four rows of one column group, lane =
      // (row, 16-byte piece). Four such items per pass keep 4 S remote loads in flight per thread.
      {
        const int ewarp = etid >> 5, quads = (nrows + 3) >> 2, n_items = kGroups * quads;
        for (int w0 = ewarp; w0 < n_items; w0 += 32) {
          float4 ld[4][8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int wi = min(w0 + q * 8, n_items - 1);
            const int g = wi % kGroups, rl = min((wi / kGroups) * 4 + (lane >> 3), nrows - 1), rr = r0 + rl;
            const uint32_t off = ((static_cast<uint32_t>(g) * 128 + rr) * 32) * 4 + (lane & 7) * 16;
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2)
              if (s2 < S) ld[q][s2] = dsmem_ld_v4(dsmem_addr(stg_addr + off, s2));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int wi = w0 + q * 8;
            const int g = wi % kGroups, rl = (wi / kGroups) * 4 + (lane >> 3), rr = r0 + rl;
            if (wi >= n_items || rl >= nrows) continue;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s2 = 0; s2 < 8; ++s2)
              if (s2 < S) {
                const float cf = cft[rl * 8 + s2];
                acc[0] += cf * ld[q][s2].x; acc[1] += cf * ld[q][s2].y;
                acc[2] += cf * ld[q][s2].z; acc[3] += cf * ld[q][s2].w;
              }
            const int hd = hb * 128 + rr;
            if (hd < p.heads) {
              const int col = g * 32 + (((lane & 7) ^ (rr & 7)) << 2);  // undo the staging swizzle
              uint2 q2;
              q2.x = pack2<T>(acc[0], acc[1]);
              q2.y = pack2<T>(acc[2], acc[3]);
              *reinterpret_cast<uint2*>(outg + (static_cast<size_t>(b) * p.heads + hd) * kCkv + dh * kDvHalf + col) = q2;
            }
          }
        }
      }
      cluster_sync();  // nobody leaves while a peer may still read its shared memory
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mlatc

// ------------------------------------------------------------------------------------- host side
bool mla_tc_supported(const cb200_mla_decode_args* a) {
  return a->kv_indptr == nullptr && a->kv_len >= 1 && a->ckv_dim == mlatc::kCkv && a->kpe_dim == mlatc::kKpe;
}

namespace {

struct TcShape {
  int head_blocks, blocks, kv_pad;
  int ranges, blocks_per_range;  // scores kernel: token ranges per (request, head block)
  int dv;                        // values kernel: output columns per CTA (256 or 128)
  int splits, blocks_per_split;  // values kernel: token ranges per (request, head block, column part)
  size_t p_bytes, stats_bytes;
};

// Both kernels fill the SMs once: as many token ranges per item as fit, never more than there are blocks.
TcShape mla_tc_shape(const cb200_mla_decode_args* a, int sms) {
  TcShape s{};
  s.head_blocks = ceil_div(a->num_heads, 128);
  s.blocks = ceil_div(a->kv_len, mlatc::kBlk);
  s.kv_pad = s.blocks * mlatc::kBlk;
  int ctas = sms;
  if (a->max_ctas > 0 && a->max_ctas < ctas) ctas = a->max_ctas;
  const long long items1 = static_cast<long long>(a->batch) * s.head_blocks;
  int r = static_cast<int>(ctas / items1);
  if (r < 1) r = 1;
  const int tiles = ceil_div(s.blocks, 2);  // a range is made of whole MMA tiles (two blocks)
  if (r > tiles) r = tiles;
  s.blocks_per_range = 2 * ceil_div(tiles, r);
  s.ranges = ceil_div(s.blocks, s.blocks_per_range);
  // Column parts of 256 need twice the token splits of parts of 128 for the same number of CTAs, and
  // the cluster combine moves (S - 1) / S of a CTA's accumulator: prefer 128 when 256 would split.
  s.dv = 256;
  long long items2 = items1 * 2;
  if (ctas / items2 >= 2 && s.blocks >= 2) {
    s.dv = 128;
    items2 = items1 * 4;
  }
  int sp = static_cast<int>(ctas / items2);
  if (sp < 1) sp = 1;
  if (sp > s.blocks) sp = s.blocks;
  if (sp > 8) sp = 8;  // the splits of an item are one thread-block cluster (portable size)
  s.blocks_per_split = ceil_div(s.blocks, sp);
  s.splits = ceil_div(s.blocks, s.blocks_per_split);
  const size_t tiles_p = static_cast<size_t>(items1) * s.blocks;  // P tiles of 128 rows x 128 tokens
  s.p_bytes = tiles_p * mlatc::kBlk * 128 * 2;
  s.stats_bytes = align_up(tiles_p * 128 * sizeof(float2), 256);
  return s;
}

template <typename T>
int launch_mla_tc_kernels(int dv, long long grid1, long long grid2, const CUtensorMap& tm_qn, const CUtensorMap& tm_qp,
                          const CUtensorMap& tm_ckv_k, const CUtensorMap& tm_kpe, const CUtensorMap& tm_ckv_v,
                          const mlatc::Params& p, cudaStream_t stream) {
  auto k1 = mlatc::mla_scores_kernel<T>;
  const bool cluster = p.splits >= 2;
  auto k2 = dv == 128 ? mlatc::mla_values_kernel<T, 128> : mlatc::mla_values_kernel<T, 256>;
  // set on every launch: the attribute is per function and per device, and the call is cheap
  CB200_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::kScoreSmem));
  CB200_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::kValueSmem));
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid1), 1, 1);
    cfg.blockDim = dim3(mlatc::kScoreThreads, 1, 1);
    cfg.dynamicSmemBytes = mlatc::kScoreSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    // scheduled while the preceding kernel of the stream drains; waits before its first global access
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, k1, tm_qn, tm_qp, tm_ckv_k, tm_kpe, p));
  }
  CB200_CUDA_TRY(cudaGetLastError());
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid2), 1, 1);
    cfg.blockDim = dim3(mlatc::kValueThreads, 1, 1);
    cfg.dynamicSmemBytes = mlatc::kValueSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    // the kernel starts while the scores kernel drains and waits (griddepcontrol.wait) before it reads P
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = p.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cluster ? 2 : 1;
    CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, k2, tm_ckv_v, p));
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

}  // namespace

// Workspace of the two-kernel path behind the caller's header and counters: P tiles | block statistics.
size_t mla_tc_partial_bytes(const cb200_mla_decode_args* a, int sms) {
  const TcShape s = mla_tc_shape(a, sms);
  return s.p_bytes + s.stats_bytes;
}

int launch_mla_tc(const cb200_mla_decode_args* a, int* status, void* scratch, cudaStream_t stream) {
  using namespace mlatc;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  const TcShape s = mla_tc_shape(a, sms);
  Params p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = status;
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  p.pbuf = ws;
  p.stats = reinterpret_cast<float2*>(ws + s.p_bytes);
  p.batch = a->batch;
  p.heads = a->num_heads;
  p.head_blocks = s.head_blocks;
  p.kv_len = a->kv_len;
  p.kv_pad = s.kv_pad;
  p.blocks = s.blocks;
  p.ranges = s.ranges;
  p.blocks_per_range = s.blocks_per_range;
  p.splits = s.splits;
  p.blocks_per_split = s.blocks_per_split;
  p.scale_log2 = a->sm_scale * kLog2e;
  const long long grid1 = static_cast<long long>(a->batch) * s.head_blocks * s.ranges;
  const long long grid2 = static_cast<long long>(a->batch) * s.head_blocks * (mlatc::kCkv / s.dv) * s.splits;
  if (grid1 >= (1LL << 31) || grid2 >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_qn, tm_qp, tm_ckv_k, tm_kpe, tm_ckv_v;
  {
    uint32_t qbox[3] = {64u, 128u, 1u}, kbox[3] = {64u, static_cast<uint32_t>(kSTile), 1u},
             vbox[3] = {64u, static_cast<uint32_t>(kBlk), 1u};
    uint64_t dq[3] = {kCkv, static_cast<uint64_t>(a->num_heads), static_cast<uint64_t>(a->batch)};
    uint64_t sq[2] = {kCkv * 2, static_cast<uint64_t>(a->num_heads) * kCkv * 2};
    uint64_t dp[3] = {kKpe, static_cast<uint64_t>(a->num_heads), static_cast<uint64_t>(a->batch)};
    uint64_t sp[2] = {kKpe * 2, static_cast<uint64_t>(a->num_heads) * kKpe * 2};
    uint64_t dc[3] = {kCkv, static_cast<uint64_t>(a->kv_len), static_cast<uint64_t>(a->batch)};
    uint64_t sc[2] = {kCkv * 2, static_cast<uint64_t>(a->kv_len) * kCkv * 2};
    uint64_t dk[3] = {kKpe, static_cast<uint64_t>(a->kv_len), static_cast<uint64_t>(a->batch)};
    uint64_t sk[2] = {kKpe * 2, static_cast<uint64_t>(a->kv_len) * kKpe * 2};
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    if (!encode_tensor_map(&tm_qn, dt, 3, const_cast<void*>(a->q_nope), dq, sq, qbox, sw) ||
        !encode_tensor_map(&tm_qp, dt, 3, const_cast<void*>(a->q_pe), dp, sp, qbox, sw) ||
        !encode_tensor_map(&tm_ckv_k, dt, 3, const_cast<void*>(a->ckv_cache), dc, sc, kbox, sw) ||
        !encode_tensor_map(&tm_kpe, dt, 3, const_cast<void*>(a->kpe_cache), dk, sk, kbox, sw) ||
        !encode_tensor_map(&tm_ckv_v, dt, 3, const_cast<void*>(a->ckv_cache), dc, sc, vbox, sw))
      return CB200_ERR_CUDA;
  }
  return a->dtype == CB200_F16
             ? launch_mla_tc_kernels<__half>(s.dv, grid1, grid2, tm_qn, tm_qp, tm_ckv_k, tm_kpe, tm_ckv_v, p, stream)
             : launch_mla_tc_kernels<__nv_bfloat16>(s.dv, grid1, grid2, tm_qn, tm_qp, tm_ckv_k, tm_kpe, tm_ckv_v, p, stream);
}

}  // namespace cb200
