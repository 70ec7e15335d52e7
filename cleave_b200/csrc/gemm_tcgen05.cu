// Fused dense contractions on the 5th-generation tensor cores (tcgen05 + TMEM) for sm_100a:
//   MODE 0  Y = X @ W                                   (split-K matmul)
//   MODE 1  Y = (X * rsqrt(mean(X^2) + eps) [* gamma]) @ W   (RMSNorm fused into the GEMM)
//   MODE 2  Y = silu(X @ W0) * (X @ W1)                 (SwiGLU, one A stream, two accumulators)
// X is (M, K) row-major (K-major A operand), W is (K, N) row-major (MN-major B operand).
//
// One persistent launch, one CTA per SM. The work is the list of (output tile, K chunk) pairs,
// tile-major; every CTA takes an equal contiguous share of it (stream-K). Chunks of one tile that
// fall to the same CTA accumulate in TMEM; a tile finished inside one CTA goes straight through
// the fused epilogue; a tile cut across CTAs leaves fp32 partials in the workspace and the last
// CTA to arrive sums them in a fixed order and runs the epilogue (no second launch, nobody
// waits, bit-stable results). That walk serves explicit split factors and CTA limits. When the
// caller leaves the split to the library, plan_gemm picks whole tiles, or the K parts of a tile as
// one thread-block cluster whose CTAs combine through distributed shared memory (CLUSTER), or the
// CTA-pair kernel of gemm_pair.cu, from a small cost model.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (one elected thread) and TMEM owner,
// 2..5 = epilogue (TMEM -> registers -> global), 6..13 = RMSNorm statistics / gamma scaling of the
// A tile in shared memory (MODE 1 only). Two TMEM accumulators let the epilogue of one tile
// overlap the main loop of the next.
//
// Replaces the reference's generated kernels
//   tests/graph/handwritten/expected_kernels/matmul.py, matmul_splitk_partial.py, matmul_splitk_combine.py,
//   rmsnorm_matmul.py, rmsnorm_matmul_split_partial.py, rmsnorm_matmul_split_combine.py, swiglu.py
// (operators: demo/matmul.py:11-13, demo/rmsnorm_matmul.py:11-13 with
// python/cleave/frontend/composites.py:48-53, demo/swiglu.py:6-10).

#include "common.cuh"

#include <cstring>
#include <type_traits>

namespace cb200 {

constexpr int kBM = 128;  // rows per output tile (UMMA M)
constexpr int kBK = 64;   // K elements per stage: one 128-byte swizzle row
constexpr int kChunkN = 64;                       // columns per B chunk: one 128-byte swizzle row
constexpr int kABytes = kBM * kBK * 2;            // 16 KB
constexpr int kBChunkBytes = kBK * kChunkN * 2;   // 8 KB

struct GemmParams {
  void* y;
  const void* gamma;  // MODE 1, may be null
  int* status;
  int* counters;    // one per output tile, zero between launches
  float* partials;  // gridDim.x * 2 slots of (128 x UMMA_N + 128) floats
  int M, N, K;
  int tiles_m, tiles_n;
  int kblocks;         // ceil(K / 64)
  int chunk_kblocks;   // K blocks per chunk
  int chunks_per_tile; // S
  float eps;
  int a_rows;  // rows of the A box: 128, or M rounded up to 8 when M is smaller
  const void* addend;  // MODE 0, may be null: (M, N) in the storage type, added in the epilogue
  int pdl;             // cb200_gemm_args.dependent_launch
  int kblocks_main;    // K blocks of X / W; blocks beyond come from the second operand pair (x2, w2)
};

template <int MODE, int NBW>
struct GemmPlan {
  static constexpr int kWeights = MODE == 2 ? 2 : 1;
  static constexpr int kNBT = NBW * kWeights;        // B chunks per stage
  static constexpr int kUmmaN = kNBT * kChunkN;      // accumulator columns
  static constexpr int kTileN = NBW * kChunkN;       // output columns per tile
  static constexpr int kStageBytes = kABytes + kNBT * kBChunkBytes;
  static constexpr int kStages = kNBT == 2 ? 6 : 4;
  static constexpr int kThreads = MODE == 1 ? 448 : 192;
  static constexpr int kSlotFloats = kBM * kUmmaN + kBM;
  static constexpr int kSmemBytes = kStages * kStageBytes + 4096 /*barriers, rowsums*/ + 1024 /*alignment*/;
};

// Which CTA owns chunk x when C chunks are dealt as floor(c * C / G) .. floor((c + 1) * C / G).
__device__ __forceinline__ int cta_of_chunk(long long x, long long C, long long G) {
  long long c = x * G / C;
  if ((c + 1) * C / G <= x) ++c;
  return static_cast<int>(c);
}

template <int MODE, typename T, int NBW, bool CLUSTER>
__global__ void __launch_bounds__(GemmPlan<MODE, NBW>::kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
            const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_a2,
            const GemmParams p) {
  using Plan = GemmPlan<MODE, NBW>;
  constexpr int kStages = Plan::kStages;
  constexpr int kUmmaN = Plan::kUmmaN;
  constexpr uint32_t kTmemCols = 2 * kUmmaN;  // two accumulators: 256 or 512 columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stages = smem;
  uint8_t* misc = smem + kStages * Plan::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);   // TMA landed
  uint64_t* empty_bar = full_bar + kStages;                  // MMA finished reading the stage
  uint64_t* ready_bar = empty_bar + kStages;                 // MODE 1: statistics taken, A scaled
  uint64_t* acc_full = ready_bar + kStages;                  // [2] accumulator complete
  uint64_t* acc_empty = acc_full + 2;                        // [2] accumulator drained
  uint64_t* rs_full = acc_empty + 2;                         // [2] MODE 1: row sums published
  uint64_t* rs_empty = rs_full + 2;                          // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(rs_empty + 2);
  int* flag = reinterpret_cast<int*>(tmem_holder + 1);
  float* rowsum_smem = reinterpret_cast<float*>(misc + 512);  // [2 accumulators][2 groups][128]
  float* rs_red = reinterpret_cast<float*>(misc + 2560);      // [128] row sums of a reduced tile

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], MODE == 1 ? 5 : 1);  // MMA commit (+ the 4 statistics warps)
      mbar_init(&ready_bar[s], 4);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      // one arrival per warp (after __syncwarp): arrivals on one mbarrier serialise
      mbar_init(&acc_empty[b], 4);
      mbar_init(&rs_full[b], 8);
      mbar_init(&rs_empty[b], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b0);
    if (MODE == 2) tma_prefetch_desc(&tm_b1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  // Dependent launch (the grid may have started while the preceding kernel of the stream still runs):
  // mode 1 waits for that kernel here, before any operand is read; mode 2 lets the main loop run and waits
  // in the epilogue warps only, before the addend - the one operand the preceding kernel wrote - is read;
  // mode 3 waits in the producer warp before the first load of the second operand pair.
  pdl_launch_dependents();  // before the wait: a dependent of this grid waits for this grid's completion itself
  if (p.pdl == 1) pdl_wait();

  // ---- this CTA's share of the (tile, chunk) list
  const int S = p.chunks_per_tile;
  const long long C = static_cast<long long>(p.tiles_m) * p.tiles_n * S;
  const long long G = gridDim.x;
  // Cluster mode: the S chunks of a tile are the S CTAs of one cluster, one chunk each.
  const long long x0 = CLUSTER ? static_cast<long long>(blockIdx.x) : static_cast<long long>(blockIdx.x) * C / G;
  const long long x1 = CLUSTER ? x0 + 1 : static_cast<long long>(blockIdx.x + 1) * C / G;

  // Split-K inside a cluster, second half: once every CTA of the cluster has parked its accumulator
  // (first cluster barrier), ALL warps of the CTA - the producer, the MMA issuer and the statistics warps
  // are idle by then - take part in the reduce through distributed shared memory: it is bound by the
  // latency of remote loads, so the number of loads in flight is what sets its duration.
  constexpr int kReduceWarps = Plan::kThreads / 32;
  auto cluster_reduce = [&](int slot_in) {
    if constexpr (CLUSTER) {
      // epilogue warps pass 0..3; the other warps take the remaining slots
      const int slot = slot_in;
      const int tile = static_cast<int>(x0 / S);
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      const int rows_live = min(kBM, p.M - tm * kBM);
      const float inv_k = 1.f / static_cast<float>(p.K);
      T* yout = reinterpret_cast<T*>(p.y);
      float* stg = reinterpret_cast<float*>(stages);
      // CTA `rank` owns rows [r_lo, r_hi). A warp reads 512 contiguous bytes of a peer per load:
      // four rows of one column group, lane = (row, 16-byte piece); peers are added in rank order.
      const int rank = static_cast<int>(cluster_ctarank());
      constexpr int kGroups = Plan::kTileN / 32;
      const int per = ceil_div(rows_live, S);
      const int r_lo = min(rank * per, rows_live), r_hi = min(r_lo + per, rows_live);
      const int quads = (r_hi - r_lo + 3) >> 2, n_items = quads * kGroups;
      const uint32_t stg_u32 = smem_u32(stg);
      for (int wi = slot; wi < n_items; wi += kReduceWarps) {
        const int g = wi % kGroups, r = r_lo + (wi / kGroups) * 4 + (lane >> 3);
        const int rc = min(r, r_hi - 1);  // clamped for the loads; rows past the end are not stored
        const uint32_t off = ((static_cast<uint32_t>(g) * kBM + rc) * 32) * 4 + (lane & 7) * 16;
        float v[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f}, rs_all = 0.f;
        for (int q0 = 0; q0 < S; q0 += 4) {  // four peers' loads in flight
          float4 a[4], bq[4];
          float rq[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            a[u] = bq[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            rq[u] = 0.f;
            if (q0 + u < S) {
              const uint32_t base = dsmem_addr(stg_u32, q0 + u);
              a[u] = dsmem_ld_v4(base + off);
              if constexpr (MODE == 2) bq[u] = dsmem_ld_v4(base + off + kGroups * kBM * 32 * 4);
              if constexpr (MODE == 1) rq[u] = dsmem_ld_f32(base + (kBM * kUmmaN + rc) * 4);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            v[0] += a[u].x; v[1] += a[u].y; v[2] += a[u].z; v[3] += a[u].w;
            if constexpr (MODE == 2) { up[0] += bq[u].x; up[1] += bq[u].y; up[2] += bq[u].z; up[3] += bq[u].w; }
            rs_all += rq[u];
          }
        }
        const int gcol = tn * Plan::kTileN + g * 32 + (((lane & 7) ^ (rc & 7)) << 2);  // undo the swizzle
        if (r < r_hi && gcol < p.N) {
          float o[4];
          if constexpr (MODE == 1) {
            const float sc = rsqrtf(rs_all * inv_k + p.eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = v[j] * sc;
          } else if constexpr (MODE == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = v[j] / (1.f + __expf(-v[j])) * up[j];
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = v[j];
            if (p.addend) {
              const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(p.addend) +
                                                              static_cast<size_t>(tm * kBM + r) * p.N + gcol);
              const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] += static_cast<float>(e[j]);
            }
          }
          uint2 pk;
          pk.x = pack2<T>(o[0], o[1]);
          pk.y = pack2<T>(o[2], o[3]);
          *reinterpret_cast<uint2*>(yout + static_cast<size_t>(tm * kBM + r) * p.N + gcol) = pk;
        }
      }
    }
  };

  if (warp == 0) {
    // ================================================================ TMA producer
    int stage = 0, phase = 0;
    bool waited2 = false;
    for (long long x = x0; x < x1;) {
      const int tile = static_cast<int>(x / S), s0 = static_cast<int>(x - static_cast<long long>(tile) * S);
      const int nseg = static_cast<int>(min(static_cast<long long>(S - s0), x1 - x));
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      const int kb0 = s0 * p.chunk_kblocks, kb1 = min((s0 + nseg) * p.chunk_kblocks, p.kblocks);
      for (int kb = kb0; kb < kb1; ++kb) {
        mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kFaultEmptyBarrier);
        if (MODE == 0 && p.pdl == 3 && kb >= p.kblocks_main && !waited2) {
          pdl_wait();  // the second operand pair is the preceding kernel's output; everything before streamed beside it
          waited2 = true;
        }
        if (elect_one()) {
          uint8_t* a_dst = stages + stage * Plan::kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          // rows of the A tile beyond a_rows are never fetched; the MMA reads whatever is there,
          // and the rows of D they produce are never stored
          mbar_arrive_expect_tx(&full_bar[stage], Plan::kStageBytes - (kBM - p.a_rows) * kBK * 2);
          if (MODE == 0 && kb >= p.kblocks_main) {
            // K blocks past the end of X / W: the second operand pair, Y = X W + X2 W2 (tm_b1 is W2 here)
            const int k2 = (kb - p.kblocks_main) * kBK;
            tma_load_2d(a_dst, &tm_a2, &full_bar[stage], k2, tm * kBM);
#pragma unroll
            for (int j = 0; j < NBW; ++j)
              tma_load_2d(b_dst + j * kBChunkBytes, &tm_b1, &full_bar[stage], tn * Plan::kTileN + j * kChunkN, k2);
          } else {
            tma_load_2d(a_dst, &tm_a, &full_bar[stage], kb * kBK, tm * kBM);
#pragma unroll
            for (int j = 0; j < NBW; ++j)
              tma_load_2d(b_dst + j * kBChunkBytes, &tm_b0, &full_bar[stage], tn * Plan::kTileN + j * kChunkN, kb * kBK);
          }
          if constexpr (MODE == 2) {
#pragma unroll
            for (int j = 0; j < NBW; ++j)
              tma_load_2d(b_dst + (NBW + j) * kBChunkBytes, &tm_b1, &full_bar[stage],
                          tn * Plan::kTileN + j * kChunkN, kb * kBK);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      x += nseg;
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    constexpr uint32_t idesc = umma_idesc(std::is_same<T, __nv_bfloat16>::value, true, kBM, kUmmaN);
    int stage = 0, phase = 0, buf = 0, acc_phase = 0;
    for (long long x = x0; x < x1;) {
      const int tile = static_cast<int>(x / S), s0 = static_cast<int>(x - static_cast<long long>(tile) * S);
      const int nseg = static_cast<int>(min(static_cast<long long>(S - s0), x1 - x));
      const int kb0 = s0 * p.chunk_kblocks, kb1 = min((s0 + nseg) * p.chunk_kblocks, p.kblocks);
      mbar_wait(&acc_empty[buf], acc_phase ^ 1, p.status, kFaultTmemBarrier);
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * kUmmaN;
      for (int kb = kb0; kb < kb1; ++kb) {
        mbar_wait((MODE == 1 && p.gamma != nullptr) ? &ready_bar[stage] : &full_bar[stage], phase, p.status,
                  kFaultFullBarrier);
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_addr = smem_u32(stages + stage * Plan::kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // A: K-major, 16 K elements = 32 bytes inside the swizzled 128-byte row
            const uint64_t adesc = umma_smem_desc(a_addr + k * 32, 16, 8 * 128);
            // B: MN-major, 16 K rows = 2048 bytes; 64-column chunks are kBChunkBytes apart
            const uint64_t bdesc = umma_smem_desc(b_addr + k * 16 * 128, kBChunkBytes, 8 * 128);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (elect_one()) umma_commit(&acc_full[buf]);
      __syncwarp();
      if (++buf == 2) { buf = 0; acc_phase ^= 1; }
      x += nseg;
    }
  }
  else if (MODE == 1 && warp >= 6) {
    // ================================================================ RMSNorm statistics (+ gamma)
    // Thread r owns row r of the A tile: it sums x^2 over the K blocks of the segment and, when a
    // weight is given, rewrites the row as x * gamma before the MMA reads it.
    // Two groups of four warps take alternate K blocks, so that two TMA -> scale -> MMA chains
    // are in flight; the number of stages is even, so a stage always belongs to the same group.
    const int group = (warp - 6) >> 2;
    const int row = ((warp - 6) & 3) * 32 + lane;
    const T* gamma = reinterpret_cast<const T*>(p.gamma);
    int stage = 0, phase = 0, buf = 0, acc_phase = 0, kb_count = 0;
    for (long long x = x0; x < x1;) {
      const int tile = static_cast<int>(x / S), s0 = static_cast<int>(x - static_cast<long long>(tile) * S);
      const int nseg = static_cast<int>(min(static_cast<long long>(S - s0), x1 - x));
      const int kb0 = s0 * p.chunk_kblocks, kb1 = min((s0 + nseg) * p.chunk_kblocks, p.kblocks);
      float sumsq = 0.f;
      const bool row_live = (tile / p.tiles_n) * kBM + row < p.M;  // padded rows are all zero
      for (int kb = kb0; kb < kb1; ++kb, ++kb_count) {
        if ((kb_count & 1) != group) {
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          continue;
        }
        // gamma for this K block is fetched before the wait: its latency is off the
        // TMA -> scale -> MMA chain. (K is a multiple of 8: a chunk is inside or outside whole.)
        uint4 graw[8];
        if (gamma && row_live) {
#pragma unroll
          for (int lc = 0; lc < 8; ++lc) {
            const int k = kb * kBK + (lc << 3);
            graw[lc] = k < p.K ? __ldg(reinterpret_cast<const uint4*>(gamma + k)) : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        mbar_wait(&full_bar[stage], phase, p.status, kFaultFullBarrier);
        uint8_t* a_row = stages + stage * Plan::kStageBytes + row * 128;
        // logical 16-byte chunk lc of row r sits at physical chunk lc ^ (r & 7) (128-byte swizzle);
        // eight consecutive rows therefore touch eight different bank groups.
        uint4 raw[8];
        if (row_live) {
#pragma unroll
          for (int lc = 0; lc < 8; ++lc) raw[lc] = *reinterpret_cast<const uint4*>(a_row + ((lc ^ (row & 7)) << 4));
          if (gamma) {  // the MMA waits for this: scale, store, publish - statistics come after
#pragma unroll
            for (int lc = 0; lc < 8; ++lc) {
              uint4 sc;
              sc.x = mul2<T>(raw[lc].x, graw[lc].x);
              sc.y = mul2<T>(raw[lc].y, graw[lc].y);
              sc.z = mul2<T>(raw[lc].z, graw[lc].z);
              sc.w = mul2<T>(raw[lc].w, graw[lc].w);
              *reinterpret_cast<uint4*>(a_row + ((lc ^ (row & 7)) << 4)) = sc;
            }
          }
        }
        if (gamma) {
          fence_proxy_async_smem();  // generic-proxy writes must be visible to the MMA
          __syncwarp();
          if (lane == 0) mbar_arrive(&ready_bar[stage]);
        }
        if (row_live) {
          // four independent partial sums keep the FMA chain short
          float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int lc = 0; lc < 8; ++lc) {
            const T* e = reinterpret_cast<const T*>(&raw[lc]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float f = static_cast<float>(e[j]);
              part[j & 3] += f * f;
            }
          }
          sumsq += (part[0] + part[1]) + (part[2] + part[3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp is done with the stage
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      mbar_wait(&rs_empty[buf], acc_phase ^ 1, p.status, kFaultTmemBarrier);
      rowsum_smem[(buf * 2 + group) * kBM + row] = sumsq;
      __syncwarp();
      if (lane == 0) mbar_arrive(&rs_full[buf]);
      if (++buf == 2) { buf = 0; acc_phase ^= 1; }
      x += nseg;
    }
  } else if (warp >= 2 && warp < 6) {
    // ================================================================ epilogue
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const int etid = tid - 64;     // 0..127
    T* yout = reinterpret_cast<T*>(p.y);
    const float inv_k = 1.f / static_cast<float>(p.K);
    int buf = 0, acc_phase = 0;
    if (p.pdl == 2) pdl_wait();

    // v: 32 consecutive accumulator columns starting at tile column c0 (for MODE 2: gate and up)
    auto finish_and_store = [&](const float* v, const float* up, int gr, int gc0, float rs) {
      if (gr >= p.M) return;
      float o[32];
      if constexpr (MODE == 1) {
        const float sc = rsqrtf(rs * inv_k + p.eps);
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = v[j] * sc;
      } else if constexpr (MODE == 2) {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = v[j] / (1.f + __expf(-v[j])) * up[j];
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = v[j];
        if (p.addend) {
          const T* add = reinterpret_cast<const T*>(p.addend) + static_cast<size_t>(gr) * p.N + gc0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (gc0 + j < p.N) {
              const uint4 u = *reinterpret_cast<const uint4*>(add + j);
              const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
              for (int i = 0; i < 8; ++i) o[j + i] += static_cast<float>(e[i]);
            }
          }
        }
      }
      T* dst = yout + static_cast<size_t>(gr) * p.N + gc0;
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
    };

    for (long long x = x0; x < x1;) {
      const int tile = static_cast<int>(x / S), s0 = static_cast<int>(x - static_cast<long long>(tile) * S);
      const int nseg = static_cast<int>(min(static_cast<long long>(S - s0), x1 - x));
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      const int gr = tm * kBM + row;
      const bool starts_here = s0 == 0, whole = starts_here && nseg == S;
      mbar_wait(&acc_full[buf], acc_phase, p.status, kFaultMmaBarrier);
      tc_fence_after();
      float rs = 0.f;
      if constexpr (MODE == 1) {
        mbar_wait(&rs_full[buf], acc_phase, p.status, kFaultTmemBarrier);
        rs = rowsum_smem[(buf * 2) * kBM + row] + rowsum_smem[(buf * 2 + 1) * kBM + row];
        __syncwarp();
        if (lane == 0) mbar_arrive(&rs_empty[buf]);
      }
      const uint32_t t_acc = tmem_base + buf * kUmmaN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (whole) {
#pragma unroll 1
        for (int c0 = 0; c0 < Plan::kTileN; c0 += 32) {
          uint32_t r[32], r2[32];
          tmem_ld_32x32(t_acc + c0, r);
          if constexpr (MODE == 2) tmem_ld_32x32(t_acc + Plan::kTileN + c0, r2);
          tmem_ld_wait();
          finish_and_store(reinterpret_cast<float*>(r), reinterpret_cast<float*>(r2), gr,
                           tn * Plan::kTileN + c0, rs);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      } else if constexpr (CLUSTER) {
        // Split-K inside a thread-block cluster: every CTA parks its fp32 accumulator in its own
        // shared memory (the pipeline stages are idle: all MMAs have completed), the cluster
        // meets at a hardware barrier, and CTA r reduces rows [r, r + 1) * rows / S over all peers
        // through distributed shared memory, in rank order (bit-stable), and stores them. No
        // workspace, no atomics, nobody spins.
        // Staging layout: [column group of 32][row][8 pieces of 16 bytes], piece i of row r stored at
        // i ^ (r & 7) so that a warp's stores spread over all banks.
        float* stg = reinterpret_cast<float*>(stages);
        const int rows_live = min(kBM, p.M - tm * kBM);
#pragma unroll 1
        for (int c0 = 0; c0 < kUmmaN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c0, r);
          tmem_ld_wait();
          if (row < rows_live) {
            float4* dst = reinterpret_cast<float4*>(stg + (static_cast<size_t>(c0 >> 5) * kBM + row) * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j ^ (row & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          }
        }
        if constexpr (MODE == 1) stg[kBM * kUmmaN + row] = rs;
        cluster_sync();
        cluster_reduce(warp - 2);
        cluster_sync();  // nobody leaves while a peer still reads its shared memory
      } else {
        // Partial layout: [column group of 32][row][32 floats], so that a warp (32 consecutive
        // rows) reads and writes 4 KB contiguously; row sums follow the accumulator block.
        float* slot = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + (starts_here ? 1 : 0)) * Plan::kSlotFloats;
        const bool live = gr < p.M;
#pragma unroll 1
        for (int c0 = 0; c0 < kUmmaN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_acc + c0, r);
          tmem_ld_wait();
          if (live) {
            float4* dst = reinterpret_cast<float4*>(slot + (static_cast<size_t>(c0 >> 5) * kBM + row) * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          }
        }
        if constexpr (MODE == 1) slot[kBM * kUmmaN + row] = rs;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        __threadfence();
        named_bar_sync(2, 128);
        const long long first_chunk = static_cast<long long>(tile) * S;
        const int c_first = cta_of_chunk(first_chunk, C, G), c_last = cta_of_chunk(first_chunk + S - 1, C, G);
        if (etid == 0) {
          const int old = atomicAdd(p.counters + tile, 1);
          *flag = (old == c_last - c_first) ? 1 : 0;
        }
        named_bar_sync(2, 128);
        if (*flag) {
          __threadfence();
          auto piece = [&](int c) {
            return p.partials + (static_cast<size_t>(c) * 2 + (c == c_first ? 1 : 0)) * Plan::kSlotFloats;
          };
          // The reduction is latency-bound (every piece comes from L2), so the work is spread
          // flat over all 128 threads - items of 8 columns, whatever the number of live rows -
          // and the loads of several items and several pieces are put in flight before any add.
          // Pieces are added in CTA order: the sum is bit-stable.
          if constexpr (MODE == 1) {
            float rs_all = 0.f;
            for (int cb = c_first; cb <= c_last; cb += 4) {  // four loads in flight, added in order
              float t[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) t[q] = cb + q <= c_last ? __ldcg(piece(cb + q) + kBM * kUmmaN + row) : 0.f;
#pragma unroll
              for (int q = 0; q < 4; ++q) rs_all += t[q];
            }
            rs_red[row] = rs_all;
            named_bar_sync(3, 128);
          }
          constexpr int kItemsPerRow = Plan::kTileN / 8;
          constexpr int kU = 4;                      // items per thread per step
          constexpr int kPB = MODE == 2 ? 2 : 3;     // pieces loaded together
          const int rows_live = min(kBM, p.M - tm * kBM);
          const int items = rows_live * kItemsPerRow;
#pragma unroll 1
          for (int it0 = 0; it0 < items; it0 += 128 * kU) {
            float v[kU][8], up[kU][8];
            size_t off[kU];
            bool ok[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              const int it = it0 + u * 128 + etid;
              ok[u] = it < items;
              const int r = ok[u] ? it / kItemsPerRow : 0, col = ok[u] ? (it % kItemsPerRow) * 8 : 0;
              off[u] = (static_cast<size_t>(col >> 5) * kBM + r) * 32 + (col & 31);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[u][j] = up[u][j] = 0.f;
            }
#pragma unroll 1
            for (int cb = c_first; cb <= c_last; cb += kPB) {
              float4 ld[kPB][kU][2], ld_up[kPB][kU][2];
#pragma unroll
              for (int q = 0; q < kPB; ++q) {
                const bool have = cb + q <= c_last;
                const float* src = piece(have ? cb + q : cb);
#pragma unroll
                for (int u = 0; u < kU; ++u) {
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    ld[q][u][h] = (have && ok[u]) ? __ldcg(reinterpret_cast<const float4*>(src + off[u]) + h)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                    if constexpr (MODE == 2)
                      ld_up[q][u][h] = (have && ok[u])
                                           ? __ldcg(reinterpret_cast<const float4*>(src + off[u] + (Plan::kTileN >> 5) * kBM * 32) + h)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                  }
                }
              }
#pragma unroll
              for (int q = 0; q < kPB; ++q) {
#pragma unroll
                for (int u = 0; u < kU; ++u) {
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    v[u][4 * h] += ld[q][u][h].x; v[u][4 * h + 1] += ld[q][u][h].y;
                    v[u][4 * h + 2] += ld[q][u][h].z; v[u][4 * h + 3] += ld[q][u][h].w;
                    if constexpr (MODE == 2) {
                      up[u][4 * h] += ld_up[q][u][h].x; up[u][4 * h + 1] += ld_up[q][u][h].y;
                      up[u][4 * h + 2] += ld_up[q][u][h].z; up[u][4 * h + 3] += ld_up[q][u][h].w;
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
              if (!ok[u]) continue;
              const int it = it0 + u * 128 + etid;
              const int r = it / kItemsPerRow, col = (it % kItemsPerRow) * 8;
              const int gcol = tn * Plan::kTileN + col;
              if (gcol >= p.N) continue;
              float o[8];
              if constexpr (MODE == 1) {
                const float sc = rsqrtf(rs_red[r] * inv_k + p.eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[u][j] * sc;
              } else if constexpr (MODE == 2) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[u][j] / (1.f + __expf(-v[u][j])) * up[u][j];
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[u][j];
                if (p.addend) {
                  const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.addend) +
                                                                  static_cast<size_t>(tm * kBM + r) * p.N + gcol);
                  const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
                  for (int j = 0; j < 8; ++j) o[j] += static_cast<float>(e[j]);
                }
              }
              uint4 pk;
              pk.x = pack2<T>(o[0], o[1]);
              pk.y = pack2<T>(o[2], o[3]);
              pk.z = pack2<T>(o[4], o[5]);
              pk.w = pack2<T>(o[6], o[7]);
              *reinterpret_cast<uint4*>(yout + static_cast<size_t>(tm * kBM + r) * p.N + gcol) = pk;
            }
          }
          if (etid == 0) p.counters[tile] = 0;  // ready for the next launch
        }
        named_bar_sync(2, 128);
      }
      if (++buf == 2) { buf = 0; acc_phase ^= 1; }
      x += nseg;
    }
  }

  if constexpr (CLUSTER) {
    // the epilogue warps met the cluster twice inside their branch; everyone else does so here
    if (!(warp >= 2 && warp < 6)) {
      cluster_sync();
      if (p.pdl >= 2) pdl_wait();  // the reduce reads the addend and writes Y: the preceding kernel must be done
      cluster_reduce(warp < 2 ? 4 + warp : warp);  // slots 4, 5 and 6 .. 13
      cluster_sync();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------- host side
double gemm_pair_estimate_us(const cb200_gemm_args* a, int sms, int* ks_out);
size_t gemm_pair_prepass_bytes(const cb200_gemm_args* a);
int launch_gemm_pair(const cb200_gemm_args* a, int* status, void* scratch, int ks, const CUtensorMap& tm_a,
                     const CUtensorMap& tm_b0, const CUtensorMap& tm_b1, cudaStream_t stream);

namespace {

constexpr size_t kGemmSlotBytesMax = (static_cast<size_t>(kBM) * 256 + kBM) * 4;

struct GemmSetup {
  GemmParams p;
  int mode, nbw, grid;
  bool cluster;  // split-K inside a thread-block cluster (tiny outputs)
  bool pair;     // whole 256 x 256 tiles on CTA pairs (gemm_pair.cu)
  int pair_ks;   // pairs per cluster: the K split of the pair kernel
  size_t ws_needed, partials_off, counters_off, prepass_off;
  double estimate_us;  // the cost model's estimate for the plan that was chosen
  CUtensorMap tm_a, tm_b0, tm_b1, tm_a2;
};

// How many clusters of `size` CTAs of the cluster GEMM variant can be resident at once (they must fit
// inside GPCs, so it is less than SMs / size for the larger sizes); cached per variant, size and device.
int cluster_capacity(int mode, bool f16, int nbw, int size);

int plan_gemm(const cb200_gemm_args* a, GemmSetup* s, bool need_maps) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return CB200_ERR_BAD_ARG;
  if (a->op < CB200_GEMM_MATMUL || a->op > CB200_GEMM_SWIGLU) return CB200_ERR_BAD_ARG;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (a->k % 8 || a->n % 8) return CB200_ERR_UNSUPPORTED;  // TMA strides are multiples of 16 bytes
  if (a->addend && a->op != CB200_GEMM_MATMUL) return CB200_ERR_UNSUPPORTED;
  if (a->dependent_launch < 0 || a->dependent_launch > 3) return CB200_ERR_BAD_ARG;
  const bool ext = a->k2 > 0;
  if (ext && (a->op != CB200_GEMM_MATMUL || a->k2 % 8)) return CB200_ERR_UNSUPPORTED;
  if (a->k2 < 0 || (a->dependent_launch == 3 && !ext)) return CB200_ERR_BAD_ARG;
  if (a->ldx != 0 && (a->ldx < a->k || a->ldx % 8)) return CB200_ERR_BAD_ARG;
  if (a->ldx != 0 && a->op != CB200_GEMM_MATMUL) return CB200_ERR_UNSUPPORTED;
  if (a->n_peers < 0 || a->n_peers > 7 || a->ldy < 0 || (a->ldy != 0 && (a->ldy < a->n || a->ldy % 8))) return CB200_ERR_BAD_ARG;
  for (int d = 0; d < a->n_peers; ++d)
    if (!a->y_peers[d] || (reinterpret_cast<uintptr_t>(a->y_peers[d]) & 15)) return CB200_ERR_BAD_ARG;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  int grid_max = sms;
  if (a->max_ctas > 0 && a->max_ctas < grid_max) grid_max = a->max_ctas;
  s->mode = a->op;
  GemmParams& p = s->p;
  p = GemmParams{};
  p.M = a->m; p.N = a->n; p.K = a->k;
  p.eps = a->eps;
  p.tiles_m = ceil_div(a->m, kBM);
  p.a_rows = a->m >= kBM ? kBM : (a->m + 7) / 8 * 8;
  // 256-column tiles when there are plenty of tiles, 128-column tiles otherwise (SwiGLU always
  // pairs two 128-column accumulators).
  s->nbw = 2;
  if (a->op != CB200_GEMM_SWIGLU && static_cast<long long>(p.tiles_m) * ceil_div(a->n, 256) >= 2LL * grid_max) s->nbw = 4;
  p.kblocks_main = ceil_div(a->k, kBK);
  p.kblocks = p.kblocks_main + (ext ? ceil_div(a->k2, kBK) : 0);
  // Automatic plan: whole tiles, or the K parts of a tile as one thread-block cluster (reduced through
  // distributed shared memory), whichever a small cost model says finishes first. Per CTA and K block
  // the MMAs take about 0.56 us for a 256-column tile and 0.33 us for a 128-column one (sustained rates
  // measured on full-size runs, clocks under the power cap included) or the time to pull the block's
  // operands, whichever is longer; a cluster reduce moves
  // (S - 1) / S of an fp32 tile at about 25 KB/us; tiles beyond one wave of SMs queue up. The stream-K walk with a workspace fix-up stays for explicit split factors
  // and CTA limits: its last-arriver reduce costs several microseconds per cut tile.
  int auto_split = 0;
  double best = 0.0;  // the cost model's estimate for the single-CTA kernel, us
  if (a->split_k <= 0 && a->max_ctas == 0) {
    const int rows_live = a->m < kBM ? a->m : kBM;
    for (int nbw = 2; nbw <= (a->op == CB200_GEMM_SWIGLU ? 2 : 4); nbw *= 2) {
      const long long tl = static_cast<long long>(p.tiles_m) * ceil_div(a->n, nbw * kChunkN);
      const double kb_us = (nbw == 4 || a->op == CB200_GEMM_SWIGLU) ? 0.56 : 0.33;
      const int umma_n = nbw * kChunkN * (a->op == CB200_GEMM_SWIGLU ? 2 : 1);
      int smax = tl <= grid_max ? static_cast<int>(grid_max / tl) : 1;
      if (smax > 8) smax = 8;
      if (smax > p.kblocks / 4) smax = p.kblocks / 4;
      if (smax < 1) smax = 1;
      // operand bytes a CTA pulls per K block (A rows that exist + B chunks) at about 90 KB/us per SM
      const double kb_mem_us = (rows_live * kBK * 2.0 + umma_n * kBK * 2.0) / 90000.0;
      const double kb_cost = kb_us > kb_mem_us ? kb_us : kb_mem_us;
      // splits 1 .. 8 (portable cluster sizes) and 16 (one cluster of 16 CTAs, for a single small tile with a
      // long K: 8.4 against 9.3 us on 128 x 128 x 4096)
      const int cands[9] = {1, 2, 3, 4, 5, 6, 7, 8, 16};
      for (int ci = 0; ci < 9; ++ci) {
        const int sp = cands[ci];
        if (sp <= 8 ? sp > smax : !(tl * 16 <= grid_max && p.kblocks / 4 >= 16)) continue;
        long long waves = (tl * sp + grid_max - 1) / grid_max;
        if (sp > 1) {  // clusters that do not all fit at once run in waves
          const int cap = cluster_capacity(a->op, a->dtype == CB200_F16, nbw, sp);
          if (cap <= 0) continue;
          waves = (tl + cap - 1) / cap;
        }
        double t = static_cast<double>(waves) * ceil_div(p.kblocks, sp) * kb_cost;
        if (sp > 1) t += rows_live * umma_n * 4.0 * (sp - 1) / sp / 25000.0 + 1.0;  // park + reduce
        if (best == 0.0 || t < best * 0.97) {  // ties go to the earlier (narrower, less split) candidate
          best = t;
          s->nbw = nbw;
          auto_split = sp;
        }
      }
    }
  }
  p.tiles_n = ceil_div(a->n, s->nbw * kChunkN);
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  if (tiles >= (1LL << 24)) return CB200_ERR_UNSUPPORTED;
  int split = a->split_k;
  if (split <= 0 && auto_split > 0) {
    split = auto_split;
  } else if (split <= 0) {  // a CTA limit: pick the K split that gives every CTA several chunks
    split = 1;
    if (tiles * 8 <= grid_max && p.kblocks >= 16) {
      split = 8;  // tiny output: an 8-CTA cluster per tile (portable cluster size)
    } else if (tiles % grid_max != 0) {
      while (split < 16 && tiles * split < 8LL * grid_max) split *= 2;
    }
  }
  if (split > p.kblocks) split = p.kblocks;
  p.chunk_kblocks = ceil_div(p.kblocks, split);
  p.chunks_per_tile = ceil_div(p.kblocks, p.chunk_kblocks);
  const long long chunks = tiles * p.chunks_per_tile;
  s->grid = static_cast<int>(chunks < grid_max ? chunks : grid_max);
  // Few tiles and a split that fits the SMs at once (cluster of up to 8 CTAs, or 16): the chunks of a tile become the CTAs
  // of one cluster and the reduction goes through distributed shared memory.
  const int S = p.chunks_per_tile;
  s->cluster = S >= 2 && (S <= 8 || S == 16) && chunks <= grid_max && a->max_ctas == 0;
  if (s->cluster) s->grid = static_cast<int>(chunks);
  {
    // CTA pairs when the same model says they finish first (split_k == 1 asks for whole tiles: compare
    // against the whole-tile plan's waves)
    s->pair_ks = 1;
    const double t_pair = gemm_pair_estimate_us(a, sms, &s->pair_ks);
    double t_single = best;
    if (t_single == 0.0) t_single = static_cast<double>((tiles + grid_max - 1) / grid_max) * p.kblocks * (s->nbw == 4 || a->op == CB200_GEMM_SWIGLU ? 0.56 : 0.33);
    s->pair = t_pair > 0.0 && t_pair < t_single && !a->addend && a->dependent_launch <= 1 && !ext;  // the pair kernel has no addend and no second operand pair; mode 1 is only a permission, the pair launch stays an ordinary one
    // a result with its own row pitch, or one that is also sent to peer GPUs, is the pair kernel's business only
    if (a->n_peers > 0 || (a->ldy != 0 && a->ldy != a->n)) {
      if (!(t_pair > 0.0) || a->addend || ext || a->dependent_launch > 1) return CB200_ERR_UNSUPPORTED;
      s->pair = true;
    }
  }
  {
    // the estimate of the plan that runs: the model's own for automatic plans; for an explicit split factor the
    // same per-block costs plus the workspace fix-up of every cut tile (a few microseconds, once per wave)
    const double kb_us = (s->nbw == 4 || a->op == CB200_GEMM_SWIGLU) ? 0.56 : 0.33;
    const int rows_live = a->m < kBM ? a->m : kBM;
    const double kb_mem_us = (rows_live * kBK * 2.0 + s->nbw * kChunkN * (a->op == CB200_GEMM_SWIGLU ? 2 : 1) * kBK * 2.0) / 90000.0;
    const double per_cta_blocks = static_cast<double>(chunks) * p.chunk_kblocks / s->grid;
    s->estimate_us = best > 0.0 && split == auto_split ? best
                                                       : per_cta_blocks * (kb_us > kb_mem_us ? kb_us : kb_mem_us) + (S > 1 ? 3.0 : 0.0);
  }
  if (s->pair) {
    s->cluster = false;
    p.chunk_kblocks = p.kblocks;
    p.chunks_per_tile = 1;
    s->estimate_us = gemm_pair_estimate_us(a, sms, &s->pair_ks);
  }
  s->partials_off = kWsHeaderBytes;
  s->counters_off = align_up(s->partials_off + static_cast<size_t>(sms) * 2 * kGemmSlotBytesMax, 256);
  if (s->pair && a->op == CB200_GEMM_RMSNORM && static_cast<size_t>(tiles) > kWsCounterSlots) {
    if (a->n_peers > 0 || (a->ldy != 0 && a->ldy != a->n)) return CB200_ERR_UNSUPPORTED;
    s->pair = false;  // the pre-pass scratch would start inside the counters
  }
  s->prepass_off = align_up(s->counters_off + (static_cast<size_t>(tiles) > kWsCounterSlots ? static_cast<size_t>(tiles) : kWsCounterSlots) * 4, 256);
  s->ws_needed = s->prepass_off + (s->pair ? gemm_pair_prepass_bytes(a) : 0);
  if (!need_maps) return CB200_OK;

  if (!a->x || !a->w || !a->y) return CB200_ERR_BAD_ARG;
  if (a->op == CB200_GEMM_SWIGLU && !a->w1) return CB200_ERR_BAD_ARG;
  if (ext && (!a->x2 || !a->w2)) return CB200_ERR_BAD_ARG;
  if (ext && ((reinterpret_cast<uintptr_t>(a->x2) | reinterpret_cast<uintptr_t>(a->w2)) & 15)) return CB200_ERR_ALIGNMENT;
  uintptr_t bits = reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->w) |
                   reinterpret_cast<uintptr_t>(a->y) | reinterpret_cast<uintptr_t>(a->w1) |
                   reinterpret_cast<uintptr_t>(a->gamma) | reinterpret_cast<uintptr_t>(a->addend);
  if (bits & 15) return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < s->ws_needed) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return CB200_ERR_ALIGNMENT;
  p.y = a->y;
  p.gamma = a->op == CB200_GEMM_RMSNORM ? a->gamma : nullptr;
  p.addend = a->addend;
  p.pdl = a->dependent_launch;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.partials = reinterpret_cast<float*>(ws + s->partials_off);
  p.counters = reinterpret_cast<int*>(ws + s->counters_off);

  const CUtensorMapDataType dt = a->dtype == CB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a->k), static_cast<uint64_t>(a->m)};
    uint64_t strides[1] = {static_cast<uint64_t>(a->ldx ? a->ldx : a->k) * 2};  // a K slice of a wider X keeps X's row pitch
    uint32_t box[2] = {kBK, static_cast<uint32_t>(p.a_rows)};
    if (!encode_tensor_map(&s->tm_a, dt, 2, const_cast<void*>(a->x), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(a->n), static_cast<uint64_t>(a->k)};
    uint64_t strides[1] = {static_cast<uint64_t>(a->n) * 2};
    uint32_t box[2] = {kChunkN, kBK};
    if (!encode_tensor_map(&s->tm_b0, dt, 2, const_cast<void*>(a->w), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
    const void* w1 = a->op == CB200_GEMM_SWIGLU ? a->w1 : a->w;
    if (ext) {  // tm_b1 carries W2 (k2, n)
      uint64_t dims2[2] = {static_cast<uint64_t>(a->n), static_cast<uint64_t>(a->k2)};
      if (!encode_tensor_map(&s->tm_b1, dt, 2, const_cast<void*>(a->w2), dims2, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return CB200_ERR_CUDA;
    } else if (!encode_tensor_map(&s->tm_b1, dt, 2, const_cast<void*>(w1), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) {
      return CB200_ERR_CUDA;
    }
  }
  s->tm_a2 = s->tm_a;
  if (ext) {
    uint64_t dims[2] = {static_cast<uint64_t>(a->k2), static_cast<uint64_t>(a->m)};
    uint64_t strides[1] = {static_cast<uint64_t>(a->k2) * 2};
    uint32_t box[2] = {kBK, static_cast<uint32_t>(p.a_rows)};
    if (!encode_tensor_map(&s->tm_a2, dt, 2, const_cast<void*>(a->x2), dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return CB200_ERR_CUDA;
  }
  return CB200_OK;
}

template <int MODE, typename T, int NBW, bool CLUSTER>
int launch_gemm_variant(const GemmSetup& s, cudaStream_t stream) {
  using Plan = GemmPlan<MODE, NBW>;
  auto kern = gemm_kernel<MODE, T, NBW, CLUSTER>;
  CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s.grid, 1, 1);
  cfg.blockDim = dim3(Plan::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Plan::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if constexpr (CLUSTER) {
    if (s.p.chunks_per_tile > 8)
      CB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = s.p.chunks_per_tile;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (s.p.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, s.tm_a, s.tm_b0, s.tm_b1, s.tm_a2, s.p));
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

template <int MODE, typename T, int NBW>
int launch_gemm(const GemmSetup& s, cudaStream_t stream) {
  return s.cluster ? launch_gemm_variant<MODE, T, NBW, true>(s, stream)
                   : launch_gemm_variant<MODE, T, NBW, false>(s, stream);
}

template <typename T>
int dispatch_gemm(const GemmSetup& s, cudaStream_t st) {
  switch (s.mode) {
    case CB200_GEMM_MATMUL: return s.nbw == 4 ? launch_gemm<0, T, 4>(s, st) : launch_gemm<0, T, 2>(s, st);
    case CB200_GEMM_RMSNORM: return s.nbw == 4 ? launch_gemm<1, T, 4>(s, st) : launch_gemm<1, T, 2>(s, st);
    default: return launch_gemm<2, T, 2>(s, st);
  }
}

template <int MODE, typename T, int NBW>
int query_cluster_capacity(int size) {
  using Plan = GemmPlan<MODE, NBW>;
  auto kern = gemm_kernel<MODE, T, NBW, true>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kSmemBytes) != cudaSuccess) return 0;
  if (size > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(size * 64, 1, 1);
  cfg.blockDim = dim3(Plan::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Plan::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = size;
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

int cluster_capacity(int mode, bool f16, int nbw, int size) {
  static int cache[16][3][2][2][17] = {};  // device, mode, dtype, width, size; 0 = not asked yet, -1 = none
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16 || size < 2 || size > 16) return 0;
  int& c = cache[dev][mode][f16 ? 0 : 1][nbw == 4 ? 1 : 0][size];
  if (c == 0) {
    int n = 0;
    if (mode == CB200_GEMM_MATMUL)
      n = f16 ? (nbw == 4 ? query_cluster_capacity<0, __half, 4>(size) : query_cluster_capacity<0, __half, 2>(size))
              : (nbw == 4 ? query_cluster_capacity<0, __nv_bfloat16, 4>(size) : query_cluster_capacity<0, __nv_bfloat16, 2>(size));
    else if (mode == CB200_GEMM_RMSNORM)
      n = f16 ? (nbw == 4 ? query_cluster_capacity<1, __half, 4>(size) : query_cluster_capacity<1, __half, 2>(size))
              : (nbw == 4 ? query_cluster_capacity<1, __nv_bfloat16, 4>(size) : query_cluster_capacity<1, __nv_bfloat16, 2>(size));
    else
      n = f16 ? query_cluster_capacity<2, __half, 2>(size) : query_cluster_capacity<2, __nv_bfloat16, 2>(size);
    c = n > 0 ? n : -1;
  }
  return c;
}

}  // namespace
}  // namespace cb200

extern "C" size_t cb200_gemm_workspace_bytes(const cb200_gemm_args* a) {
  cb200::GemmSetup s;
  if (cb200::plan_gemm(a, &s, false) != CB200_OK) return 0;
  return s.ws_needed;
}

extern "C" int cb200_gemm_effective_split(const cb200_gemm_args* a) {
  cb200::GemmSetup s;
  if (cb200::plan_gemm(a, &s, false) != CB200_OK) return 0;
  return s.p.chunks_per_tile;
}

extern "C" int cb200_gemm_plan(const cb200_gemm_args* a, cb200_gemm_plan_info* out) {
  cb200::GemmSetup s;
  if (!out) return CB200_ERR_BAD_ARG;
  const int rc = cb200::plan_gemm(a, &s, false);
  if (rc != CB200_OK) return rc;
  out->tile_m = s.pair ? 256 : cb200::kBM;
  out->tile_n = s.pair ? 256 : s.nbw * cb200::kChunkN;
  out->split = s.pair ? s.pair_ks : s.p.chunks_per_tile;
  out->kind = s.pair ? 2 : (s.cluster ? 1 : 0);
  out->grid = s.grid;
  out->estimate_us = static_cast<float>(s.estimate_us);
  return CB200_OK;
}

extern "C" int cb200_gemm(const cb200_gemm_args* a, void* stream) {
  using namespace cb200;
  GemmSetup s;
  const int rc = plan_gemm(a, &s, true);
  if (rc != CB200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s.pair)
    return launch_gemm_pair(a, s.p.status, static_cast<uint8_t*>(a->workspace) + s.prepass_off, s.pair_ks, s.tm_a, s.tm_b0, s.tm_b1, st);
  return a->dtype == CB200_F16 ? dispatch_gemm<__half>(s, st) : dispatch_gemm<__nv_bfloat16>(s, st);
}
