// Large GEMMs on CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 output tile on two
// neighbouring SMs. Each CTA of the pair holds its 128 rows of A and of the accumulator and only
// HALF of B's columns (the hardware feeds both halves to both SMs), so a CTA moves 32 KB of operands
// per K block where the single-CTA kernel moves 48 KB for the same 128 x 256 x 64 of work per SM.
//   MODE 0  Y = X @ W                    B half of CTA r: columns [256 tn + 128 r, +128) of W
//   RMSNorm(X)[* gamma] @ W                MODE 0 after one pass over X (rmsnorm_prepass_kernel) that computes the row
//                                        factors rsqrt(sum(x^2) / K + eps) and, with gamma, writes X * gamma as
//                                        the A operand; the epilogue applies the factors. Statistics warps
//                                        inside the pair pipeline were measured slower in both forms: reading
//                                        A tiles beside the MMA costs shared-memory bandwidth (1.26 PFLOP/s),
//                                        and rewriting them ahead of the MMA adds a land -> scale -> fence ->
//                                        remote arrive chain that six stages do not hide (0.69); the pass
//                                        moves 2 - 4 M K bytes, about 2 % of the GEMM's time (1.35 - 1.39).
//   MODE 2  Y = silu(X @ W0) * (X @ W1)  B half of CTA 0: 128 columns of W0; of CTA 1: the same columns of W1,
//                                        so every CTA's accumulator is gate | up for its own rows
// Used for whole tiles only (no split-K); small or skinny problems stay with gemm_tcgen05.cu.
//
// Every CTA loads its own operands (TMA without multicast; the transaction bytes of both CTAs are
// counted on the first CTA's barrier); the first CTA's MMA thread issues for the pair; one commit
// arrives on the barriers of both CTAs. Warp roles per CTA: 0 = TMA producer, 1 = MMA issuer
// (first CTA only) and TMEM owner, 2..5 = epilogue for the CTA's own 128 rows.
//
// Replaces the same reference kernels as gemm_tcgen05.cu (expected_kernels/matmul.py, rmsnorm_matmul.py,
// swiglu.py).

#include "common.cuh"

#include <cstring>
#include <type_traits>

namespace cb200 {
namespace pair {

constexpr int kBM = 128, kBK = 64, kChunkN = 64;
constexpr int kABytes = kBM * kBK * 2;           // 16 KB
constexpr int kBChunkBytes = kBK * kChunkN * 2;  // 8 KB
constexpr int kBHalfChunks = 2;                  // 128 columns of B per CTA
constexpr int kStageBytes = kABytes + kBHalfChunks * kBChunkBytes;  // 32 KB
constexpr int kStages = 6;
constexpr int kUmmaN = 256;
constexpr int kPushWarps = 4;
constexpr int kThreads = (6 + kPushWarps) * 32;  // warps 0 TMA, 1 MMA, 2..5 epilogue, 6.. push finished tiles to peer GPUs (idle otherwise)
constexpr int kMaxPeers = 7;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024;
constexpr uint32_t kTmemCols = 512;  // two accumulators of 256 columns

struct Params {
  void* y;
  const float* row_scale;  // MODE 0: optional per-row factor applied in the epilogue (RMSNorm)
  int* status;
  int M, N, K, tiles_m, tiles_n, kblocks;
  int ldy;                  // elements between consecutive rows of Y (N for a dense result)
  int n_peers;              // other GPUs whose copy of Y receives this GPU's tiles (0: none)
  void* y_peers[kMaxPeers]; // their Y, at this GPU's column offset, same row stride
};

// Tile order: bands of kGroupM tile rows, column-major inside a band, so the tiles that the resident
// pairs work on at the same time share a few row strips of X and a few column strips of W in L2.
constexpr int kGroupM = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_band = kGroupM * tiles_n;
  const int band = t / per_band, r = t - band * per_band;
  const int first = band * kGroupM;
  const int rows = min(kGroupM, tiles_m - first);
  tn = r / rows;
  tm = first + (r - tn * rows);
}

// KS > 1: the K dimension of a tile is split over KS pairs that form one cluster of 2 KS CTAs (ranks 2 k and
// 2 k + 1 are pair k); every pair accumulates its K part, parks the accumulator in its idle pipeline
// stages, and CTA (k, half) sums rows [k, k + 1) * 128 / KS of its half over the pairs through distributed
// shared memory, in pair order, before the epilogue. One tile per cluster (the grid is tiles x 2 KS).
template <int MODE, typename T, int KS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                 const __grid_constant__ CUtensorMap tm_b1, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);  // used on the first CTA
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_full = empty_bar + kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2] used on the first CTA: both CTAs' epilogue warps arrive
  uint64_t* stored = acc_empty + 2;           // [2] the epilogue warps have written a tile's rows to Y
  uint64_t* pushed = stored + 2;              // [2] the push warps have sent them on
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pushed + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t crank = cluster_ctarank();
  const uint32_t rank = crank & 1;          // 0 = first CTA of the pair (issues the MMAs)
  const uint32_t kpart = crank >> 1;        // which K part this pair accumulates (KS > 1)
  const uint32_t lead = crank & ~1u;        // cluster rank of the pair's first CTA
  const uint16_t pair_mask = static_cast<uint16_t>(3u << lead);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);  // four epilogue warps of each CTA
      mbar_init(&stored[b], 4);
      mbar_init(&pushed[b], kPushWarps);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    if (MODE == 2) tma_prefetch_desc(&tm_b1);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  const int pair_id = blockIdx.x / (2 * KS), n_pairs = gridDim.x / (2 * KS);
  const int tiles = p.tiles_m * p.tiles_n;
  const int kb_per = ceil_div(p.kblocks, KS);
  const int kb0 = static_cast<int>(kpart) * kb_per, kb1 = min(p.kblocks, kb0 + kb_per);
  constexpr int kTileN = MODE == 2 ? 128 : 256;  // output columns per tile

  if (warp == 0) {
    // ================================================================ TMA producer (both CTAs)
    int stage = 0, phase = 0;
    const CUtensorMap* tm_b = (MODE == 2 && rank == 1) ? &tm_b1 : &tm_b0;
    for (int t = pair_id; t < tiles; t += n_pairs) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int row0 = tm * 256 + static_cast<int>(rank) * kBM;
      const int col0 = MODE == 2 ? tn * 128 : tn * 256 + static_cast<int>(rank) * 128;
      for (int kb = kb0; kb < kb1; ++kb) {
        mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
        if (elect_one()) {
          uint8_t* a_dst = stages + stage * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kStageBytes);  // both CTAs' bytes
          tma_load_2d_pair(a_dst, &tm_a, &full_bar[stage], kb * kBK, row0);
#pragma unroll
          for (int j = 0; j < kBHalfChunks; ++j)
            tma_load_2d_pair(b_dst + j * kBChunkBytes, tm_b, &full_bar[stage], col0 + j * kChunkN, kb * kBK);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
    if constexpr (KS > 1) {  // the two meetings of the split-K combine
      cluster_sync();
      cluster_sync();
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (first CTA only)
    if (rank == 0) {
      constexpr uint32_t idesc = umma_idesc(std::is_same<T, __nv_bfloat16>::value, true, 256, kUmmaN);
      int stage = 0, phase = 0, buf = 0, acc_phase = 0;
      for (int t = pair_id; t < tiles; t += n_pairs) {
        mbar_wait(&acc_empty[buf], acc_phase ^ 1, p.status, kFaultTmemBarrier);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kUmmaN;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&full_bar[stage], phase, p.status, kFaultFullBarrier);
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a_addr = smem_u32(stages + stage * kStageBytes);
            const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              const uint64_t adesc = umma_smem_desc(a_addr + k * 32, 16, 8 * 128);
              const uint64_t bdesc = umma_smem_desc(b_addr + k * 16 * 128, kBChunkBytes, 8 * 128);
              umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            umma_commit_pair(&empty_bar[stage], pair_mask);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (elect_one()) umma_commit_pair(&acc_full[buf], pair_mask);
        __syncwarp();
        if (++buf == 2) { buf = 0; acc_phase ^= 1; }
      }
    }
    if constexpr (KS > 1) {
      cluster_sync();
      cluster_sync();
    }
  } else if (warp >= 6) {
    // ================================================================ finished tiles go to the other GPUs
    // N-sharded GEMM: every GPU computes a column slice of Y and all of them want the whole of Y. The epilogue
    // writes this GPU's rows of a tile into its own copy (at the slice's column offset); these warps then
    // read them back (L2) and store them into every peer's copy through NVLink, whole 512-byte row segments per
    // warp instruction, while the pair is already on its next tile: the all-gather rides under the MMAs.
    if constexpr (KS > 1) {  // the two meetings of the split-K combine are meetings of every thread of the cluster
      cluster_sync();
      cluster_sync();
    }
    if (p.n_peers > 0) {
      const int pw = warp - 6;
      const T* ysrc = reinterpret_cast<const T*>(p.y);
      constexpr int kRowsMine = kBM / KS;
      const int r_lo = KS > 1 ? static_cast<int>(kpart) * kRowsMine : 0;
      int ti = 0;
      for (int t = pair_id; t < tiles; t += n_pairs, ++ti) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        const int slot = ti & 1;
        mbar_wait(&stored[slot], (ti >> 1) & 1, p.status, kFaultTmemBarrier);
        const int gc0 = tn * kTileN;
        const int pieces = min(kTileN, p.N - gc0) / 8;  // 16-byte pieces of a row segment (at most 32)
        const int grow0 = tm * 256 + static_cast<int>(rank) * kBM;
        for (int r = r_lo + pw * 4; r < r_lo + kRowsMine; r += 4 * kPushWarps) {
          uint4 v[4];
          bool ok[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ok[i] = lane < pieces && grow0 + r + i < p.M;
            if (ok[i]) v[i] = __ldcg(reinterpret_cast<const uint4*>(ysrc + static_cast<size_t>(grow0 + r + i) * p.ldy + gc0) + lane);
          }
          // every CTA starts with another peer, so that at any moment the stores of the GPU go to all of them
          for (int dd = 0; dd < p.n_peers; ++dd) {
            const int d = (dd + static_cast<int>(blockIdx.x) + pw) % p.n_peers;
            T* ydst = reinterpret_cast<T*>(p.y_peers[d]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (ok[i]) *(reinterpret_cast<uint4*>(ydst + static_cast<size_t>(grow0 + r + i) * p.ldy + gc0) + lane) = v[i];
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&pushed[slot]);
      }
    }
  } else {
    // ================================================================ epilogue (both CTAs, own rows)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    T* yout = reinterpret_cast<T*>(p.y);
    int buf = 0, acc_phase = 0, ti = 0;
    for (int t = pair_id; t < tiles; t += n_pairs, ++ti) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      const int gr = tm * 256 + static_cast<int>(rank) * kBM + row;
      mbar_wait(&acc_full[buf], acc_phase, p.status, kFaultMmaBarrier);
      tc_fence_after();
      float row_scale = 1.f;
      if constexpr (MODE == 0) {
        if (p.row_scale != nullptr && gr < p.M) row_scale = __ldg(p.row_scale + gr);
      }
      const uint32_t t_acc = tmem_base + buf * kUmmaN + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (KS > 1) {
        // ---- park this pair's partial accumulator: [column group of 32][row][8 pieces of 16 bytes], piece i of
        // row r at i ^ (r & 7) (conflict-free stores); the stages are idle: every MMA of the tile has completed
        float* stg = reinterpret_cast<float*>(stages);
#pragma unroll 1
        for (int c0 = 0; c0 < kUmmaN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c0, r);
          tmem_ld_wait();
          float4* dst = reinterpret_cast<float4*>(stg + (static_cast<size_t>(c0 >> 5) * kBM + row) * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j ^ (row & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                             __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
        cluster_sync();
        {
          // CTA (kpart, half) owns rows [kpart, kpart + 1) * 128 / KS of its half; a warp reads 512 contiguous
          // bytes of a peer per load (four rows of one column group); pairs are added in order
          constexpr int kGroupsOut = kTileN / 32, kRowsMine = kBM / KS;
          const int r_lo = static_cast<int>(kpart) * kRowsMine;
          const uint32_t stg_u32 = smem_u32(stg);
          const int ewarp = (tid - 64) >> 5;
          for (int wi = ewarp; wi < (kRowsMine / 4) * kGroupsOut; wi += 4) {
            const int g = wi % kGroupsOut, rl = r_lo + (wi / kGroupsOut) * 4 + (lane >> 3);
            const uint32_t off = ((static_cast<uint32_t>(g) * kBM + rl) * 32) * 4 + (lane & 7) * 16;
            float v[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
            float4 a[KS], bq[KS];
#pragma unroll
            for (int kp = 0; kp < KS; ++kp) {
              const uint32_t base = dsmem_addr(stg_u32, rank + 2 * kp);
              a[kp] = dsmem_ld_v4(base + off);
              if constexpr (MODE == 2) bq[kp] = dsmem_ld_v4(base + off + kGroupsOut * kBM * 32 * 4);
            }
#pragma unroll
            for (int kp = 0; kp < KS; ++kp) {
              v[0] += a[kp].x; v[1] += a[kp].y; v[2] += a[kp].z; v[3] += a[kp].w;
              if constexpr (MODE == 2) { up[0] += bq[kp].x; up[1] += bq[kp].y; up[2] += bq[kp].z; up[3] += bq[kp].w; }
            }
            const int grow = tm * 256 + static_cast<int>(rank) * kBM + rl;
            const int gcol = tn * kTileN + g * 32 + (((lane & 7) ^ (rl & 7)) << 2);  // undo the swizzle
            if (grow < p.M && gcol < p.N) {
              float sc = 1.f;
              if constexpr (MODE == 0) {
                if (p.row_scale != nullptr) sc = __ldg(p.row_scale + grow);
              }
              float o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] = MODE == 2 ? v[j] / (1.f + __expf(-v[j])) * up[j] : v[j] * sc;
              uint2 pk;
              pk.x = pack2<T>(o[0], o[1]);
              pk.y = pack2<T>(o[2], o[3]);
              *reinterpret_cast<uint2*>(yout + static_cast<size_t>(grow) * p.ldy + gcol) = pk;
            }
          }
        }
        cluster_sync();  // nobody leaves while a peer still reads its shared memory (one tile per cluster)
      } else {
#pragma unroll 1
      for (int c0 = 0; c0 < kTileN; c0 += 32) {
        uint32_t r[32], r2[32];
        tmem_ld_32x32(t_acc + c0, r);
        if constexpr (MODE == 2) tmem_ld_32x32(t_acc + 128 + c0, r2);
        tmem_ld_wait();
        if (gr < p.M) {
          float o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]);
            o[j] = MODE == 2 ? v / (1.f + __expf(-v)) * __uint_as_float(r2[j]) : (MODE == 2 ? v : v * row_scale);
          }
          const int gc0 = tn * kTileN + c0;
          T* dst = yout + static_cast<size_t>(gr) * p.ldy + gc0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (gc0 + j < p.N) {
              uint4 pk;
              pk.x = pack2<T>(o[j], o[j + 1]);
              pk.y = pack2<T>(o[j + 2], o[j + 3]);
              pk.z = pack2<T>(o[j + 4], o[j + 5]);
              pk.w = pack2<T>(o[j + 6], o[j + 7]);
              *reinterpret_cast<uint4*>(dst + j) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&acc_empty[buf], lead);  // the first CTA's MMA thread waits for all eight warps
      }
      if (p.n_peers > 0) {
        // this warp's rows of the tile are in Y: hand them to the push warps (not before they are through with
        // the tile two back, whose slot this is)
        const int slot = ti & 1;
        mbar_wait(&pushed[slot], ((ti >> 1) & 1) ^ 1, p.status, kFaultTmemBarrier);
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(&stored[slot]);
      }
      if (++buf == 2) { buf = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();  // no CTA frees tensor memory or leaves while the pair's MMAs may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// RMSNorm at pair-kernel sizes: one pass over X computes the row factors rsqrt(sum(x^2) / K + eps) and, with
// gamma (SCALE), writes X * gamma as the MMA's A operand; the matmul kernel applies the factors in its
// epilogue. One CTA of 128 threads per row.
template <typename T, bool SCALE>
__global__ void __launch_bounds__(128) rmsnorm_prepass_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                              T* __restrict__ xs, float* __restrict__ row_scale,
                                                              int M, int K, float eps) {
  __shared__ float red[4];
  const int row = blockIdx.x;
  if (row >= M) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K);
  const uint4* gsrc = reinterpret_cast<const uint4*>(gamma);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * K);
  float part[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x; i < K / 8; i += 128) {
    const uint4 v = __ldg(src + i);
    if constexpr (SCALE) {
      const uint4 g = __ldg(gsrc + i);
      uint4 o;
      o.x = mul2<T>(v.x, g.x);
      o.y = mul2<T>(v.y, g.y);
      o.z = mul2<T>(v.z, g.z);
      o.w = mul2<T>(v.w, g.w);
      dst[i] = o;
    }
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = static_cast<float>(e[j]);
      part[j & 3] += f * f;
    }
  }
  float sum = (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) row_scale[row] = rsqrtf(((red[0] + red[1]) + (red[2] + red[3])) / static_cast<float>(K) + eps);
}

}  // namespace pair

// ------------------------------------------------------------------------------------- host side
template <int MODE, typename T, int KS>
static int query_pair_capacity() {
  auto kern = pair::gemm_pair_kernel<MODE, T, KS>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::kSmemBytes) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * KS * 64, 1, 1);
  cfg.blockDim = dim3(pair::kThreads, 1, 1);
  cfg.dynamicSmemBytes = pair::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2 * KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

// Clusters of 2 KS CTAs of the pair kernel that can be resident at once; cached per device.
static int pair_capacity(bool swiglu, bool f16, int ks) {
  static int cache[16][2][2][3] = {};  // 0 = not asked yet, -1 = none
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 0;
  const int ki = ks == 1 ? 0 : ks == 2 ? 1 : 2;
  int& c = cache[dev][swiglu ? 1 : 0][f16 ? 0 : 1][ki];
  if (c == 0) {
    int n = 0;
    if (swiglu) {
      if (f16) n = ks == 1 ? query_pair_capacity<2, __half, 1>() : ks == 2 ? query_pair_capacity<2, __half, 2>() : query_pair_capacity<2, __half, 4>();
      else n = ks == 1 ? query_pair_capacity<2, __nv_bfloat16, 1>() : ks == 2 ? query_pair_capacity<2, __nv_bfloat16, 2>() : query_pair_capacity<2, __nv_bfloat16, 4>();
    } else {
      if (f16) n = ks == 1 ? query_pair_capacity<0, __half, 1>() : ks == 2 ? query_pair_capacity<0, __half, 2>() : query_pair_capacity<0, __half, 4>();
      else n = ks == 1 ? query_pair_capacity<0, __nv_bfloat16, 1>() : ks == 2 ? query_pair_capacity<0, __nv_bfloat16, 2>() : query_pair_capacity<0, __nv_bfloat16, 4>();
    }
    c = n > 0 ? n : -1;
  }
  return c;
}

// Estimated time (us) of the pair kernel on this problem and the K split (pairs per cluster) that gives it, or
// a negative value when the kernel does not apply. One 256 x 256 x 64 block of MMAs costs a pair about
// 0.44 us (sustained rate of full-size runs); tiles beyond one wave of clusters queue up; a split adds parking
// the accumulator and a reduce at about 25 KB/us; RMSNorm adds its pass over X.
double gemm_pair_estimate_us(const cb200_gemm_args* a, int sms, int* ks_out) {
  (void)sms;
  if (a->split_k > 1 || a->max_ctas != 0 || a->m < 256) return -1.0;
  const bool swiglu = a->op == CB200_GEMM_SWIGLU, f16 = a->dtype == CB200_F16;
  const long long tiles = static_cast<long long>(ceil_div(a->m, 256)) * ceil_div(a->n, swiglu ? 128 : 256);
  const int kblocks = ceil_div(a->k, pair::kBK);
  double best = -1.0;
  for (int ks = 1; ks <= 4; ks *= 2) {
    if (ks > 1 && (a->split_k == 1 || kblocks / ks < 8)) break;  // split_k == 1 asks for whole tiles
    const int cap = pair_capacity(swiglu, f16, ks);
    if (cap <= 0) continue;
    // a K split runs one tile per cluster, each cluster paying its own set-up, parking and reduce: it pays when the
    // tiles are too few to fill the machine (up to two waves of clusters), not over many waves (4096 x 3584 x 4096 ran in 184 us with the split
    // the model picked for its wave count, against 118 us as whole tiles)
    if (ks > 1 && tiles > 2LL * cap) continue;
    const long long waves = (tiles + cap - 1) / cap;
    double t = static_cast<double>(waves) * ceil_div(kblocks, ks) * 0.44 + 2.0;
    if (ks > 1) t += 1.0 + (128.0 / ks) * 256.0 * 4.0 * (ks - 1) / 25000.0;
    if (best < 0.0 || t < best * 0.97) {
      best = t;
      *ks_out = ks;
    }
  }
  if (best > 0.0 && a->op == CB200_GEMM_RMSNORM) best += 2.5 + static_cast<double>(a->m) * a->k * (a->gamma ? 4.0 : 2.0) / 6.5e6;
  return best;
}

template <int MODE, typename T, int KS>
static int launch_pair_kernel_ks(const pair::Params& p, const CUtensorMap& ta, const CUtensorMap& tb0,
                                 const CUtensorMap& tb1, cudaStream_t stream) {
  auto kern = pair::gemm_pair_kernel<MODE, T, KS>;
  CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(pair::kThreads, 1, 1);
  cfg.dynamicSmemBytes = pair::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2 * KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int tiles = p.tiles_m * p.tiles_n;
  if (KS == 1) {
    // The tiles are dealt round-robin to the pairs, so the grid must be exactly the number of pairs
    // that are resident at once (SMs that cannot form a pair inside their GPC stay idle).
    int pairs = pair_capacity(MODE == 2, std::is_same<T, __half>::value, 1);
    if (pairs <= 0) return CB200_ERR_CUDA;
    if (pairs > tiles) pairs = tiles;
    cfg.gridDim = dim3(2 * pairs, 1, 1);
  } else {
    cfg.gridDim = dim3(static_cast<unsigned>(tiles) * 2 * KS, 1, 1);  // one tile per cluster
  }
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb0, tb1, p));
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

template <int MODE, typename T>
static int launch_pair_kernel(const pair::Params& p, int ks, const CUtensorMap& ta, const CUtensorMap& tb0,
                              const CUtensorMap& tb1, cudaStream_t stream) {
  if (ks == 4) return launch_pair_kernel_ks<MODE, T, 4>(p, ta, tb0, tb1, stream);
  if (ks == 2) return launch_pair_kernel_ks<MODE, T, 2>(p, ta, tb0, tb1, stream);
  return launch_pair_kernel_ks<MODE, T, 1>(p, ta, tb0, tb1, stream);
}

size_t gemm_pair_prepass_bytes(const cb200_gemm_args* a) {
  if (a->op != CB200_GEMM_RMSNORM) return 0;
  return (a->gamma ? align_up(static_cast<size_t>(a->m) * a->k * 2, 256) : 0) + align_up(static_cast<size_t>(a->m) * 4, 256);
}

// `scratch`: gemm_pair_prepass_bytes(a) bytes of the caller's workspace (RMSNorm only).
int launch_gemm_pair(const cb200_gemm_args* a, int* status, void* scratch, int ks, const CUtensorMap& tm_a,
                     const CUtensorMap& tm_b0, const CUtensorMap& tm_b1, cudaStream_t stream) {
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  pair::Params p{};
  p.y = a->y;
  p.status = status;
  p.M = a->m; p.N = a->n; p.K = a->k;
  p.ldy = a->ldy > 0 ? a->ldy : a->n;
  p.n_peers = a->n_peers;
  for (int d = 0; d < a->n_peers && d < pair::kMaxPeers; ++d) p.y_peers[d] = a->y_peers[d];
  p.tiles_m = ceil_div(a->m, 256);
  p.tiles_n = ceil_div(a->n, a->op == CB200_GEMM_SWIGLU ? 128 : 256);
  p.kblocks = ceil_div(a->k, pair::kBK);
  const bool f16 = a->dtype == CB200_F16;
  if (a->op == CB200_GEMM_SWIGLU)
    return f16 ? launch_pair_kernel<2, __half>(p, ks, tm_a, tm_b0, tm_b1, stream)
               : launch_pair_kernel<2, __nv_bfloat16>(p, ks, tm_a, tm_b0, tm_b1, stream);
  if (a->op == CB200_GEMM_RMSNORM) {
    // the row factors (and with gamma the scaled copy of X) in one pass over X, then the plain matmul
    const bool scale = a->gamma != nullptr;
    uint8_t* xs = static_cast<uint8_t*>(scratch);
    float* rscale = reinterpret_cast<float*>(xs + (scale ? align_up(static_cast<size_t>(a->m) * a->k * 2, 256) : 0));
    if (f16) {
      auto pre = scale ? pair::rmsnorm_prepass_kernel<__half, true> : pair::rmsnorm_prepass_kernel<__half, false>;
      pre<<<a->m, 128, 0, stream>>>(static_cast<const __half*>(a->x), static_cast<const __half*>(a->gamma),
                                    reinterpret_cast<__half*>(xs), rscale, a->m, a->k, a->eps);
    } else {
      auto pre = scale ? pair::rmsnorm_prepass_kernel<__nv_bfloat16, true> : pair::rmsnorm_prepass_kernel<__nv_bfloat16, false>;
      pre<<<a->m, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(a->x), static_cast<const __nv_bfloat16*>(a->gamma),
                                    reinterpret_cast<__nv_bfloat16*>(xs), rscale, a->m, a->k, a->eps);
    }
    CB200_CUDA_TRY(cudaGetLastError());
    p.row_scale = rscale;
    if (!scale)
      return f16 ? launch_pair_kernel<0, __half>(p, ks, tm_a, tm_b0, tm_b1, stream)
                 : launch_pair_kernel<0, __nv_bfloat16>(p, ks, tm_a, tm_b0, tm_b1, stream);
    CUtensorMap tm_xs;
    uint64_t dims[2] = {static_cast<uint64_t>(a->k), static_cast<uint64_t>(a->m)};
    uint64_t strides[1] = {static_cast<uint64_t>(a->k) * 2};
    uint32_t box[2] = {pair::kBK, pair::kBM};
    if (!encode_tensor_map(&tm_xs, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xs, dims,
                           strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
    return f16 ? launch_pair_kernel<0, __half>(p, ks, tm_xs, tm_b0, tm_b1, stream)
               : launch_pair_kernel<0, __nv_bfloat16>(p, ks, tm_xs, tm_b0, tm_b1, stream);
  }
  return f16 ? launch_pair_kernel<0, __half>(p, ks, tm_a, tm_b0, tm_b1, stream)
             : launch_pair_kernel<0, __nv_bfloat16>(p, ks, tm_a, tm_b0, tm_b1, stream);
}

}  // namespace cb200
