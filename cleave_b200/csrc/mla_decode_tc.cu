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
//   values   O = sum_blocks 2^(m_block - m_ref) P_block V_block. A CTA owns (request, head block, half
//            of the 512 output columns, one of S token ranges). The softmax warps read a block of P
//            rows, scale them to the running reference maximum and store them to tensor memory,
//            where they are the A operand; B is the latent tile (128 tokens x 256 columns, MN-major)
//            from a three-stage TMA ring; O (128 x 256 fp32) stays in tensor memory and is rescaled
//            only when the reference maximum grows by more than 2^8 (exact: the factor is applied to
//            O and to the row sum alike). The S CTAs of an item are one thread-block cluster and
//            combine their partial results through distributed shared memory; with more than
//            eight splits they leave fp32 partials in the workspace and the last one to arrive
//            combines them (nobody waits).
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
constexpr float kRescaleThreshold = 8.f;  // log2 units

// ---- scores kernel
constexpr int kQChunkBytes = 128 * 128;             // 128 heads x 128 bytes
constexpr int kSTile = 256;                         // tokens per MMA tile (two blocks)
constexpr int kKChunkBytes = kSTile * 128;          // 32 768
constexpr int kKStageBytes = kQChunkBytes + kKChunkBytes;  // a Q chunk and the matching cache chunk
constexpr int kKStages = 4;
constexpr int kScoreSmem = kKStages * kKStageBytes + 1024 + 1024;
constexpr int kScoreThreads = 320;                  // producer, MMA, eight epilogue warps

// ---- values kernel
constexpr int kDvHalf = 256;
constexpr int kVChunkBytes = kBlk * 128;            // 64 columns x 128 tokens
constexpr int kVStageBytes = (kDvHalf / 64) * kVChunkBytes;  // 65 536
constexpr int kVStages = 3;
constexpr int kValueSmem = kVStages * kVStageBytes + 1024 + 1024;
constexpr int kValueThreads = 192;
constexpr int kSlotFloats = 128 * kDvHalf + 256;    // O partial, m, l
constexpr uint32_t kColO = 0, kColP = 256;          // P: two buffers of 64 columns

struct Params {
  void* out;
  float* lse;
  int* status;
  int* counters;
  float* partials;
  void* pbuf;      // (batch * heads, kv_pad) 16-bit
  float2* stats;   // (batch * heads, blocks): (m, l) per block
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

  if (warp == 0) {
    // ================================================================ TMA producer
    // Q is streamed with the cache (a CTA has only a few tiles; Q comes from L2 after the first
    // touch), which leaves the whole of shared memory to the ring: 192 KB in flight per SM.
    int st = 0, ph = 0;
    for (int t = 0; t < n_tiles; ++t) {
      const int tok0 = (u0 + 2 * t) * kBlk;
      for (int c = 0; c < kChunks; ++c) {
        mbar_wait(&k_empty[st], ph ^ 1, p.status, kFaultEmptyBarrier);
        if (lane == 0) {
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
        if (lane == 0) {
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
      if (lane == 0) umma_commit(&s_full[sb]);
      __syncwarp();
    }
  } else {
    // ================================================================ epilogue: S -> P, m, l
    const int quarter = warp & 3;          // the TMEM lanes this warp may read
    const int half = (warp - 2) >> 2;      // which block of the MMA tile
    const int row = quarter * 32 + lane;
    const int head = hb * 128 + row;
    const bool live = head < p.heads;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const size_t prow = (static_cast<size_t>(b) * p.heads + head) * p.kv_pad;
    for (int t = 0; t < n_tiles; ++t) {
      const int sb = t & 1;
      const int u = u0 + 2 * t + half;
      mbar_wait(&s_full[sb], (t >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      if (u < u1) {
        const uint32_t t_s = tmem_base + lane_field + sb * kSTile + half * kBlk;
        const int tok0 = u * kBlk;
        float mx = -INFINITY;
#pragma unroll 1
        for (int c0 = 0; c0 < kBlk; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (tok0 + c0 + i < p.kv_len) mx = fmaxf(mx, __uint_as_float(r[i]) * p.scale_log2);
        }
        const float m = mx == -INFINITY ? 0.f : mx;
        float l = 0.f;
        T* pdst = reinterpret_cast<T*>(p.pbuf) + prow + tok0;
#pragma unroll 1
        for (int c0 = 0; c0 < kBlk; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_s + c0, r);
          tmem_ld_wait();
          float e[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            e[i] = tok0 + c0 + i < p.kv_len ? fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -m)) : 0.f;
            l += e[i];
          }
          if (live) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 q4;
              q4.x = pack2<T>(e[i], e[i + 1]);
              q4.y = pack2<T>(e[i + 2], e[i + 3]);
              q4.z = pack2<T>(e[i + 4], e[i + 5]);
              q4.w = pack2<T>(e[i + 6], e[i + 7]);
              *reinterpret_cast<uint4*>(pdst + c0 + i) = q4;
            }
          }
        }
        if (live) p.stats[(static_cast<size_t>(b) * p.heads + head) * p.blocks + u] = make_float2(m, l);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, bool CLUSTER>
__global__ void __launch_bounds__(kValueThreads, 1)
mla_values_kernel(const __grid_constant__ CUtensorMap tm_ckv, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* v_smem = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kVStages * kVStageBytes);
  uint64_t* v_full = bars;                 // [3] TMA landed
  uint64_t* v_empty = bars + kVStages;     // [3] the MMAs have read the stage
  uint64_t* p_full = bars + 2 * kVStages;  // [2] scaled P stored to TMEM (and O rescaled if needed)
  uint64_t* p_empty = p_full + 2;          // [2] the MMAs that read the P buffer have completed
  uint64_t* o_done = p_empty + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int x = blockIdx.x;
  const int split = x % p.splits; x /= p.splits;  // cluster mode: the splits of an item are one cluster
  const int dh = x & 1; x >>= 1;
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

  if (warp == 0) {
    // ================================================================ TMA producer
    int st = 0, ph = 0;
    for (int j = 0; j < nt; ++j) {
      mbar_wait(&v_empty[st], ph ^ 1, p.status, kFaultEmptyBarrier);
      if (lane == 0) {
        uint8_t* dst = v_smem + st * kVStageBytes;
        mbar_arrive_expect_tx(&v_full[st], kVStageBytes);
#pragma unroll
        for (int c = 0; c < kDvHalf / 64; ++c)
          tma_load_3d(dst + c * kVChunkBytes, &tm_ckv, &v_full[st], dh * kDvHalf + c * 64, (t0 + j) * kBlk, b);
      }
      __syncwarp();
      if (++st == kVStages) { st = 0; ph ^= 1; }
    }
    if constexpr (CLUSTER) {  // the two meetings of the combine
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
      if (lane == 0) {
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
    if constexpr (CLUSTER) {
      cluster_sync();
      cluster_sync();
    }
  } else {
    // ================================================================ P scaling / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // head row inside the block = TMEM lane
    const int etid = tid - 64;
    const int head = hb * 128 + row;
    const bool live = head < p.heads;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const size_t hrow = static_cast<size_t>(b) * p.heads + head;
    const T* prow = reinterpret_cast<const T*>(p.pbuf) + hrow * p.kv_pad;
    float m_ref = 0.f, l_run = 0.f;
    // P rows and statistics of the next block are fetched while the current one is processed
    uint4 raw[16];
    float2 st_next = make_float2(0.f, 0.f);
    auto fetch = [&](int u) {
      if (live) {
        st_next = __ldcg(p.stats + hrow * p.blocks + u);
        const uint4* src = reinterpret_cast<const uint4*>(prow + static_cast<size_t>(u) * kBlk);
#pragma unroll
        for (int i = 0; i < 16; ++i) raw[i] = __ldcg(src + i);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) raw[i] = make_uint4(0u, 0u, 0u, 0u);
      }
    };
    if (nt > 0) fetch(t0);
    for (int j = 0; j < nt; ++j) {
      const int pb = j & 1;
      const float2 st = st_next;
      float alpha = 1.f;
      bool rescale = false;
      if (j == 0) {
        m_ref = st.x;
      } else if (st.x > m_ref + kRescaleThreshold) {
        alpha = fast_exp2(m_ref - st.x);
        m_ref = st.x;
        rescale = true;
      }
      const float f = fast_exp2(st.x - m_ref);
      l_run = l_run * alpha + st.y * f;
      // the P buffer is free once the MMAs of tile j - 2 have completed
      mbar_wait(&p_empty[pb], ((j >> 1) & 1) ^ 1, p.status, kFaultMmaBarrier);
      if (__any_sync(0xffffffffu, rescale)) {  // rare: the reference maximum grew by more than 2^8
        // O may only be touched when no MMA is in flight: tile j - 1 is the last one issued
        mbar_wait(&p_empty[pb ^ 1], ((j - 1) >> 1) & 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
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
        tmem_st_32x32(tmem_base + lane_field + kColP + pb * 64 + h * 32, pk);
      }
      if (j + 1 < nt) fetch(t0 + j + 1);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // ---- epilogue: O / l, or a partial for the combine
    if (nt > 0) {
      mbar_wait(o_done, 0, p.status, kFaultMmaBarrier);
      tc_fence_after();
    }
    T* outp = reinterpret_cast<T*>(p.out) + hrow * kCkv + dh * kDvHalf;
    auto store32 = [&](const float* v, int c0, float inv) {
      if (!live) return;
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 q4;
        q4.x = pack2<T>(v[i] * inv, v[i + 1] * inv);
        q4.y = pack2<T>(v[i + 2] * inv, v[i + 3] * inv);
        q4.z = pack2<T>(v[i + 4] * inv, v[i + 5] * inv);
        q4.w = pack2<T>(v[i + 6] * inv, v[i + 7] * inv);
        *reinterpret_cast<uint4*>(outp + c0 + i) = q4;
      }
    };
    auto store_lse = [&](float M, float L) {
      if (live && dh == 0 && p.lse) p.lse[hrow] = L > 0.f ? M + fast_log2(L) : -INFINITY;
    };
    if (p.splits == 1) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        store32(reinterpret_cast<const float*>(o), c0, inv);
      }
      store_lse(m_ref, l_run);
    } else if constexpr (CLUSTER) {
      // Split-KV combine inside the cluster: every CTA parks its fp32 accumulator, m and l in its own
      // shared memory (the ring is idle: all MMAs have completed), the cluster meets at a hardware
      // barrier, and CTA r combines rows [r, r + 1) * 128 / S over all peers through distributed
      // shared memory, in rank order (bit-stable). No workspace, no atomics, nobody spins.
      float* stg = reinterpret_cast<float*>(v_smem);
#pragma unroll 1
      for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
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
          dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                               __uint_as_float(o[4 * i + 3]));
      }
      stg[128 * kDvHalf + row] = l_run > 0.f ? m_ref : -INFINITY;
      stg[128 * kDvHalf + 128 + row] = l_run;
      cluster_sync();
      {
        const int S = p.splits;
        const int r0 = split * 128 / S, r1 = (split + 1) * 128 / S;
        const uint32_t stg_addr = smem_u32(stg);
        for (int item = etid; item < (r1 - r0) * 32; item += 128) {
          const int rr = r0 + (item >> 5), c8 = item & 31;
          float cf[8], L = 0.f, M = -INFINITY;
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2)
            if (s2 < S) {
              cf[s2] = dsmem_ld_f32(dsmem_addr(stg_addr + (128 * kDvHalf + rr) * 4, s2));
              M = fmaxf(M, cf[s2]);
            }
          const float Mu = M == -INFINITY ? 0.f : M;
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2)
            if (s2 < S) {
              cf[s2] = fast_exp2(cf[s2] - Mu);
              L += cf[s2] * dsmem_ld_f32(dsmem_addr(stg_addr + (128 * kDvHalf + 128 + rr) * 4, s2));
            }
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          const uint32_t off = ((static_cast<uint32_t>(c8 >> 2) * 128 + rr) * 32 + (c8 & 3) * 8) * 4;
#pragma unroll
          for (int s2 = 0; s2 < 8; ++s2)
            if (s2 < S) {
              const float4 a0 = dsmem_ld_v4(dsmem_addr(stg_addr + off, s2));
              const float4 a1 = dsmem_ld_v4(dsmem_addr(stg_addr + off + 16, s2));
              acc[0] += cf[s2] * a0.x; acc[1] += cf[s2] * a0.y; acc[2] += cf[s2] * a0.z; acc[3] += cf[s2] * a0.w;
              acc[4] += cf[s2] * a1.x; acc[5] += cf[s2] * a1.y; acc[6] += cf[s2] * a1.z; acc[7] += cf[s2] * a1.w;
            }
          const int hd = hb * 128 + rr;
          if (hd < p.heads) {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            const size_t hr = static_cast<size_t>(b) * p.heads + hd;
            uint4 q4;
            q4.x = pack2<T>(acc[0] * inv, acc[1] * inv);
            q4.y = pack2<T>(acc[2] * inv, acc[3] * inv);
            q4.z = pack2<T>(acc[4] * inv, acc[5] * inv);
            q4.w = pack2<T>(acc[6] * inv, acc[7] * inv);
            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + hr * kCkv + dh * kDvHalf + c8 * 8) = q4;
            if (c8 == 0 && dh == 0 && p.lse) p.lse[hr] = L > 0.f ? M + fast_log2(L) : -INFINITY;
          }
        }
      }
      cluster_sync();  // nobody leaves while a peer may still read its shared memory
    } else {
      const int item = (b * p.head_blocks + hb) * 2 + dh;
      float* slot = p.partials + (static_cast<size_t>(item) * p.splits + split) * kSlotFloats;
      // layout [column group of 32][row][32]: a warp writes and reads 4 KB contiguously
#pragma unroll 1
      for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
        uint32_t o[32];
        if (nt > 0) {
          tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        float4* dst = reinterpret_cast<float4*>(slot + (static_cast<size_t>(c0 >> 5) * 128 + row) * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                               __uint_as_float(o[4 * i + 3]));
      }
      slot[128 * kDvHalf + row] = l_run > 0.f ? m_ref : -INFINITY;
      slot[128 * kDvHalf + 128 + row] = l_run;
      __threadfence();
      named_bar_sync(2, 128);
      if (etid == 0) {
        const int old = atomicAdd(p.counters + item, 1);
        *flag = (old == p.splits - 1) ? 1 : 0;
      }
      named_bar_sync(2, 128);
      if (*flag) {
        __threadfence();
        const float* base = p.partials + static_cast<size_t>(item) * p.splits * kSlotFloats;
        float M = -INFINITY;
        for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(base + static_cast<size_t>(s) * kSlotFloats + 128 * kDvHalf + row));
        const float Mu = M == -INFINITY ? 0.f : M;
        float L = 0.f;
        for (int s = 0; s < p.splits; ++s) {
          const float* sl = base + static_cast<size_t>(s) * kSlotFloats + 128 * kDvHalf;
          L += fast_exp2(__ldcg(sl + row) - Mu) * __ldcg(sl + 128 + row);
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
          for (int s = 0; s < p.splits; ++s) {
            const float* sl = base + static_cast<size_t>(s) * kSlotFloats;
            const float cf = fast_exp2(__ldcg(sl + 128 * kDvHalf + row) - Mu);
            const float4* src = reinterpret_cast<const float4*>(sl + (static_cast<size_t>(c0 >> 5) * 128 + row) * 32);
            float4 ld[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) ld[i] = __ldcg(src + i);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[4 * i] += cf * ld[i].x; v[4 * i + 1] += cf * ld[i].y;
              v[4 * i + 2] += cf * ld[i].z; v[4 * i + 3] += cf * ld[i].w;
            }
          }
          store32(v, c0, inv);
        }
        store_lse(M, L);
        if (etid == 0) p.counters[item] = 0;  // ready for the next launch
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

}  // namespace mlatc

// ------------------------------------------------------------------------------------- host side
bool mla_tc_supported(const cb200_mla_decode_args* a) {
  return a->kv_indptr == nullptr && a->kv_len >= 1 && a->ckv_dim == mlatc::kCkv && a->kpe_dim == mlatc::kKpe;
}

namespace {

struct TcShape {
  int head_blocks, blocks, kv_pad;
  int ranges, blocks_per_range;  // scores kernel: token ranges per (request, head block)
  int splits, blocks_per_split;  // values kernel: token ranges per (request, head block, column half)
  size_t p_bytes, stats_bytes, partial_bytes;
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
  const long long items2 = items1 * 2;
  int sp = static_cast<int>(ctas / items2);
  if (sp < 1) sp = 1;
  if (sp > s.blocks) sp = s.blocks;
  s.blocks_per_split = ceil_div(s.blocks, sp);
  s.splits = ceil_div(s.blocks, s.blocks_per_split);
  const size_t rows = static_cast<size_t>(a->batch) * a->num_heads;
  s.p_bytes = align_up(rows * s.kv_pad * 2, 256);
  s.stats_bytes = align_up(rows * s.blocks * sizeof(float2), 256);
  s.partial_bytes = s.splits <= 8 ? 0 :  // up to eight splits combine inside a cluster
                    static_cast<size_t>(items2) * s.splits * mlatc::kSlotFloats * 4;
  return s;
}

template <typename T>
int launch_mla_tc_kernels(long long grid1, long long grid2, const CUtensorMap& tm_qn, const CUtensorMap& tm_qp,
                          const CUtensorMap& tm_ckv_k, const CUtensorMap& tm_kpe, const CUtensorMap& tm_ckv_v,
                          const mlatc::Params& p, cudaStream_t stream) {
  auto k1 = mlatc::mla_scores_kernel<T>;
  const bool cluster = p.splits >= 2 && p.splits <= 8;
  auto k2 = cluster ? mlatc::mla_values_kernel<T, true> : mlatc::mla_values_kernel<T, false>;
  // set on every launch: the attribute is per function and per device, and the call is cheap
  CB200_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::kScoreSmem));
  CB200_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::kValueSmem));
  k1<<<static_cast<unsigned>(grid1), mlatc::kScoreThreads, mlatc::kScoreSmem, stream>>>(tm_qn, tm_qp, tm_ckv_k, tm_kpe, p);
  CB200_CUDA_TRY(cudaGetLastError());
  if (cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid2), 1, 1);
    cfg.blockDim = dim3(mlatc::kValueThreads, 1, 1);
    cfg.dynamicSmemBytes = mlatc::kValueSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, k2, tm_ckv_v, p));
  } else {
    k2<<<static_cast<unsigned>(grid2), mlatc::kValueThreads, mlatc::kValueSmem, stream>>>(tm_ckv_v, p);
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

}  // namespace

// Workspace of the two-kernel path behind the caller's header and counters: P | block statistics | partials.
size_t mla_tc_partial_bytes(const cb200_mla_decode_args* a, int sms) {
  const TcShape s = mla_tc_shape(a, sms);
  return s.p_bytes + s.stats_bytes + s.partial_bytes;
}

int launch_mla_tc(const cb200_mla_decode_args* a, int* status, int* counters, float* partials, cudaStream_t stream) {
  using namespace mlatc;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  const TcShape s = mla_tc_shape(a, sms);
  Params p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = status;
  p.counters = counters;
  uint8_t* ws = reinterpret_cast<uint8_t*>(partials);
  p.pbuf = ws;
  p.stats = reinterpret_cast<float2*>(ws + s.p_bytes);
  p.partials = reinterpret_cast<float*>(ws + s.p_bytes + s.stats_bytes);
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
  const long long grid2 = static_cast<long long>(a->batch) * s.head_blocks * 2 * s.splits;
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
             ? launch_mla_tc_kernels<__half>(grid1, grid2, tm_qn, tm_qp, tm_ckv_k, tm_kpe, tm_ckv_v, p, stream)
             : launch_mla_tc_kernels<__nv_bfloat16>(grid1, grid2, tm_qn, tm_qp, tm_ckv_k, tm_kpe, tm_ckv_v, p, stream);
}

}  // namespace cb200
