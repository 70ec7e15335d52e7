// MLA decode on the tcgen05 tensor cores for contiguous caches (the static operator).
//
// A CTA owns (request, block of up to 128 heads, half of the 512 latent output columns, one of S
// equal KV ranges). Rows of every MMA are the heads (UMMA M = 128):
//   S = Q K^T      A = Q  (shared memory, K-major, resident for the whole CTA: 9 chunks of 64 columns)
//                  B = KV tile of 32 tokens (shared memory, K-major), D = S in TMEM (32 columns, two buffers)
//   O += P V       A = P  (TMEM, 16-bit pairs written by the softmax warps)
//                  B = the same KV tile, columns [256 half, 256 half + 256) read MN-major, D = O in TMEM (256 columns)
// so a KV tile is fetched once and used as K and as V. The accumulator of all 512 latent columns
// would fill tensor memory on its own; splitting the output columns over two CTAs leaves room for
// S and P at the price of computing S in both.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer and TMEM owner, 2..5 = softmax / epilogue (thread =
// head row = TMEM lane). The softmax keeps a reference maximum per row and rescales O only when
// the running maximum has grown by more than 2^8 (exact: the factor is applied to O and to the row
// sum alike), so O stays in tensor memory between tiles.
// With S > 1 the CTAs of an item leave fp32 partials in the workspace and the last one to arrive
// combines them (fused split-KV log-sum-exp combine, nobody waits).
//
// Reference semantics: demo/mla_decode.py:8-13.

#include "common.cuh"

#include <cstring>
#include <type_traits>

namespace cb200 {
namespace mlatc {

constexpr int kBN = 32;                 // tokens per KV tile
constexpr int kCkv = 512, kKpe = 64, kQk = 576;
constexpr int kChunks = kQk / 64;       // 9 chunks of 64 columns (128 bytes)
constexpr int kQChunkBytes = 128 * 128; // 128 heads x 128 bytes
constexpr int kKvChunkBytes = kBN * 128;
constexpr int kQBytes = kChunks * kQChunkBytes;      // 147 456
constexpr int kStageBytes = kChunks * kKvChunkBytes; // 36 864
constexpr int kStages = 2;
constexpr int kDvHalf = 256;
constexpr int kSmemBytes = kQBytes + kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*alignment*/;
constexpr int kThreads = 192;
constexpr int kSlotFloats = 128 * kDvHalf + 256;  // O partial, m, l
// TMEM columns
constexpr uint32_t kColO = 0, kColS = 256, kColP = 320, kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;  // log2 units

struct Params {
  void* out;
  float* lse;
  int* status;
  int* counters;
  float* partials;
  int batch, heads, head_blocks, kv_len, splits, tiles_per_split;
  float scale_log2;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
mla_tc_kernel(const __grid_constant__ CUtensorMap tm_qn, const __grid_constant__ CUtensorMap tm_qp,
              const __grid_constant__ CUtensorMap tm_ckv, const __grid_constant__ CUtensorMap tm_kpe, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + kQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kQBytes + kStages * kStageBytes);
  uint64_t* kv_full = bars;         // [2] TMA landed
  uint64_t* kv_empty = bars + 2;    // [2] S and PV of the tile have finished reading the stage
  uint64_t* q_full = bars + 4;
  uint64_t* s_full = bars + 5;      // [2] S complete in TMEM
  uint64_t* s_empty = bars + 7;     // [2] softmax has read S
  uint64_t* p_full = bars + 9;      // P written (and O rescaled if needed)
  uint64_t* pv_done = bars + 10;    // PV of the tile complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 11);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which piece is this CTA's
  int x = blockIdx.x;
  const int split = x % p.splits; x /= p.splits;
  const int dh = x & 1; x >>= 1;
  const int hb = x % p.head_blocks;
  const int b = x / p.head_blocks;
  const int n_tiles_total = ceil_div(p.kv_len, kBN);
  const int t0 = min(split * p.tiles_per_split, n_tiles_total);
  const int t1 = min(t0 + p.tiles_per_split, n_tiles_total);
  const int nt = t1 - t0;  // the host picks splits so that every split owns at least one tile

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(q_full, 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_qn);
    tma_prefetch_desc(&tm_qp);
    tma_prefetch_desc(&tm_ckv);
    tma_prefetch_desc(&tm_kpe);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ================================================================ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kQBytes);
#pragma unroll
      for (int c = 0; c < kCkv / 64; ++c) tma_load_3d(q_smem + c * kQChunkBytes, &tm_qn, q_full, c * 64, hb * 128, b);
      tma_load_3d(q_smem + (kCkv / 64) * kQChunkBytes, &tm_qp, q_full, 0, hb * 128, b);
    }
    __syncwarp();
    for (int j = 0; j < nt; ++j) {
      const int st = j & 1;
      mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, p.status, kFaultEmptyBarrier);
      if (lane == 0) {
        uint8_t* dst = kv_smem + st * kStageBytes;
        mbar_arrive_expect_tx(&kv_full[st], kStageBytes);
#pragma unroll
        for (int c = 0; c < kCkv / 64; ++c)
          tma_load_3d(dst + c * kKvChunkBytes, &tm_ckv, &kv_full[st], c * 64, (t0 + j) * kBN, b);
        tma_load_3d(dst + (kCkv / 64) * kKvChunkBytes, &tm_kpe, &kv_full[st], 0, (t0 + j) * kBN, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
    constexpr uint32_t idesc_s = umma_idesc(kBf16, /*b_mn_major=*/false, 128, kBN);
    constexpr uint32_t idesc_pv = umma_idesc(kBf16, /*b_mn_major=*/true, 128, kDvHalf);
    const uint32_t q_addr = smem_u32(q_smem), kv_addr = smem_u32(kv_smem);
    auto issue_s = [&](int j) {
      const int st = j & 1, sb = j & 1;
      mbar_wait(&kv_full[st], (j >> 1) & 1, p.status, kFaultFullBarrier);
      mbar_wait(&s_empty[sb], ((j >> 1) & 1) ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (lane == 0) {
        const uint32_t d = tmem_base + kColS + sb * kBN;
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t adesc = umma_smem_desc(q_addr + c * kQChunkBytes + kk * 32, 16, 8 * 128);
            const uint64_t bdesc = umma_smem_desc(kv_addr + st * kStageBytes + c * kKvChunkBytes + kk * 32, 16, 8 * 128);
            umma_f16(d, adesc, bdesc, idesc_s, (c > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[sb]);
      }
      __syncwarp();
    };
    mbar_wait(q_full, 0, p.status, kFaultFullBarrier);
    if (nt > 0) issue_s(0);
    for (int j = 0; j < nt; ++j) {
      if (j + 1 < nt) issue_s(j + 1);
      mbar_wait(p_full, j & 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      if (lane == 0) {
        const int st = j & 1;
        const uint32_t v_addr = kv_addr + st * kStageBytes + (dh * (kDvHalf / 64)) * kKvChunkBytes;
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks) {
          // B: MN-major, 16 token rows of 128 bytes; 64-column chunks are kKvChunkBytes apart
          const uint64_t bdesc = umma_smem_desc(v_addr + ks * 16 * 128, kKvChunkBytes, 8 * 128);
          umma_f16_ts(tmem_base + kColO, tmem_base + kColP + ks * 8, bdesc, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[st]);
        umma_commit(pv_done);
      }
      __syncwarp();
    }
  } else {
    // ================================================================ softmax / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // head row inside the block = TMEM lane
    const int etid = tid - 64;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = 0.f, l_run = 0.f;
    for (int j = 0; j < nt; ++j) {
      const int sb = j & 1;
      mbar_wait(&s_full[sb], (j >> 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
      uint32_t r[32];
      tmem_ld_32x32(tmem_base + lane_field + kColS + sb * kBN, r);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      const int tok0 = (t0 + j) * kBN;
      float xs[32], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        xs[i] = tok0 + i < p.kv_len ? __uint_as_float(r[i]) * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, xs[i]);
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
      // O and P may only be touched once the previous tile's PV has completed
      if (j > 0) {
        mbar_wait(pv_done, (j - 1) & 1, p.status, kFaultMmaBarrier);
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, rescale)) {  // rare: the running maximum grew by more than 2^8
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
      float psum = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = fast_exp2(xs[2 * i] - m_ref), p1 = fast_exp2(xs[2 * i + 1] - m_ref);
        psum += p0 + p1;
        pk[i] = pack2<T>(p0, p1);
      }
      l_run = l_run * alpha + psum;
      tmem_st_32x16(tmem_base + lane_field + kColP, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l, or a partial for the combine
    if (nt > 0) {
      mbar_wait(pv_done, (nt - 1) & 1, p.status, kFaultMmaBarrier);
      tc_fence_after();
    }
    const int head = hb * 128 + row;
    const bool live = head < p.heads;
    T* outp = reinterpret_cast<T*>(p.out) + (static_cast<size_t>(b) * p.heads + head) * kCkv + dh * kDvHalf;
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
      if (live && dh == 0 && p.lse) p.lse[static_cast<size_t>(b) * p.heads + head] = L > 0.f ? M + fast_log2(L) : -INFINITY;
    };
    if (p.splits == 1) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
        tmem_ld_wait();
        store32(reinterpret_cast<const float*>(o), c0, inv);
      }
      store_lse(m_ref, l_run);
    } else {
      const int item = (b * p.head_blocks + hb) * 2 + dh;
      float* slot = p.partials + (static_cast<size_t>(item) * p.splits + split) * kSlotFloats;
      // layout [column group of 32][row][32]: a warp writes and reads 4 KB contiguously
#pragma unroll 1
      for (int c0 = 0; c0 < kDvHalf; c0 += 32) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_field + kColO + c0, o);
        tmem_ld_wait();
        float4* dst = reinterpret_cast<float4*>(slot + (static_cast<size_t>(c0 >> 5) * 128 + row) * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]), __uint_as_float(o[4 * i + 2]),
                               __uint_as_float(o[4 * i + 3]));
      }
      slot[128 * kDvHalf + row] = m_ref;
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
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace mlatc

// ------------------------------------------------------------------------------------- host side
bool mla_tc_supported(const cb200_mla_decode_args* a) {
  return a->kv_indptr == nullptr && a->kv_len >= 1 && a->ckv_dim == mlatc::kCkv && a->kpe_dim == mlatc::kKpe;
}

// Splits per item: fill the SMs once, never more splits than KV tiles.
static void mla_tc_shape(const cb200_mla_decode_args* a, int sms, int* head_blocks, int* splits, int* tiles_per_split) {
  *head_blocks = ceil_div(a->num_heads, 128);
  const long long items = static_cast<long long>(a->batch) * *head_blocks * 2;
  const int tiles = ceil_div(a->kv_len, mlatc::kBN);
  int s = static_cast<int>(sms / items);
  if (s < 1) s = 1;
  if (s > tiles) s = tiles;
  if (a->max_ctas > 0 && s * items > a->max_ctas) s = static_cast<int>(a->max_ctas / items > 0 ? a->max_ctas / items : 1);
  *tiles_per_split = ceil_div(tiles, s);
  *splits = ceil_div(tiles, *tiles_per_split);
}

size_t mla_tc_partial_bytes(const cb200_mla_decode_args* a, int sms) {
  int hb, s, tps;
  mla_tc_shape(a, sms, &hb, &s, &tps);
  if (s == 1) return 0;
  return static_cast<size_t>(a->batch) * hb * 2 * s * mlatc::kSlotFloats * 4;
}

template <typename Kern>
static int launch_mla_tc_kernel(Kern kern, long long grid, const CUtensorMap& tm_qn, const CUtensorMap& tm_qp,
                                const CUtensorMap& tm_ckv, const CUtensorMap& tm_kpe, const mlatc::Params& p,
                                cudaStream_t stream) {
  // set on every launch: the attribute is per function and per device, and the call is cheap
  CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mlatc::kSmemBytes));
  kern<<<static_cast<unsigned>(grid), mlatc::kThreads, mlatc::kSmemBytes, stream>>>(tm_qn, tm_qp, tm_ckv, tm_kpe, p);
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

int launch_mla_tc(const cb200_mla_decode_args* a, int* status, int* counters, float* partials, cudaStream_t stream) {
  using namespace mlatc;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  Params p{};
  p.out = a->out;
  p.lse = a->lse;
  p.status = status;
  p.counters = counters;
  p.partials = partials;
  p.batch = a->batch;
  p.heads = a->num_heads;
  p.kv_len = a->kv_len;
  p.scale_log2 = a->sm_scale * kLog2e;
  mla_tc_shape(a, sms, &p.head_blocks, &p.splits, &p.tiles_per_split);
  const long long grid = static_cast<long long>(a->batch) * p.head_blocks * 2 * p.splits;
  if (grid >= (1LL << 31)) return CB200_ERR_UNSUPPORTED;
  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_qn, tm_qp, tm_ckv, tm_kpe;
  {
    uint32_t qbox[3] = {64u, 128u, 1u}, kbox[3] = {64u, static_cast<uint32_t>(kBN), 1u};
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
        !encode_tensor_map(&tm_ckv, dt, 3, const_cast<void*>(a->ckv_cache), dc, sc, kbox, sw) ||
        !encode_tensor_map(&tm_kpe, dt, 3, const_cast<void*>(a->kpe_cache), dk, sk, kbox, sw))
      return CB200_ERR_CUDA;
  }
  return a->dtype == CB200_F16
             ? launch_mla_tc_kernel(mla_tc_kernel<__half>, grid, tm_qn, tm_qp, tm_ckv, tm_kpe, p, stream)
             : launch_mla_tc_kernel(mla_tc_kernel<__nv_bfloat16>, grid, tm_qn, tm_qp, tm_ckv, tm_kpe, p, stream);
}

}  // namespace cb200
