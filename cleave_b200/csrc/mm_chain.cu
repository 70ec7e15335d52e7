// O = (Q K^T) V without softmax (demo/matmul_matmul.py), computed in the cheaper association order
//
//     O = Q (K^T V)            T = K^T V is (D, D) per kv head
//
// when the sequence lengths dwarf the head dimension: 2 * (SKV + SQ) * D * D FLOPs per head instead of
// 4 * SQ * SKV * D (32 times fewer at the demo's S = 4096, D = 64), and every input byte is read once, so
// the operator becomes HBM-bound. Three kernels, the products on warp-level MMAs (m16n8k16; at 30 FLOP per byte the
// tensor pipe is not the limit):
//   ktv_kernel   a CTA owns (kv head, chunk of tokens): T_part = K_chunk^T V_chunk in fp32. K and V tiles of
//                64 tokens are staged by cp.async (three stages, padded rows); both operands are read
//                with transposing ldmatrix (the token axis is the contraction axis of both). Partials go
//                to the workspace.
//   tsum_kernel  sums the partials of a head in chunk order (bit-stable) and stores T in the storage type.
//   qt_kernel    a CTA owns (query head, 128 query rows): O_tile = Q_tile T, T (D x D, 16-bit) resident in
//                shared memory.
// The (Q K^T) V order (scores rounded to 16 bits, then the second product) stays available on the tcgen05
// attention kernel (cb200_attn_prefill with CB200_SCORE_LINEAR) and is what cb200_matmul_matmul picks
// when the chain order does not save at least four times the FLOPs.

#include "common.cuh"

#include <type_traits>

namespace cb200 {
namespace chain {

constexpr int kTok = 64;  // tokens per staged tile

template <int D>
struct Cfg {
  static constexpr int kWarps = D / 16;          // ktv: warp w owns rows [16 w, 16 w + 16) of T
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kRowBytes = D * 2 + 16;   // padded: 8 consecutive rows fall in distinct bank groups
  static constexpr int kMatBytes = kTok * kRowBytes;
  static constexpr int kStages = 3;
  static constexpr int kKtvSmem = kStages * 2 * kMatBytes;  // stages of (K, V)
  static constexpr int kQtRows = 128;
  static constexpr int kQtSmem = (kQtRows + D) * kRowBytes;  // Q tile + T
};

struct Params {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* partials;  // [chunk][hkv][D][D]
  void* t16;        // [hkv][D][D] storage type
  int hq, hkv, sq, skv, chunks, chunk_tokens;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;  // zero-fill when the row is past the end
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ------------------------------------------------------------------------------------------ K^T V
template <typename T, int D>
__global__ void __launch_bounds__(Cfg<D>::kThreads) ktv_kernel(const Params p) {
  using C = Cfg<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, hk = blockIdx.y;
  const int t_begin = chunk * p.chunk_tokens, t_end = min(t_begin + p.chunk_tokens, p.skv);
  const int n_tiles = t_end > t_begin ? ceil_div(t_end - t_begin, kTok) : 0;
  const T* kbase = reinterpret_cast<const T*>(p.k) + static_cast<size_t>(hk) * p.skv * D;
  const T* vbase = reinterpret_cast<const T*>(p.v) + static_cast<size_t>(hk) * p.skv * D;
  const uint32_t smem_base = smem_u32(smem);
  pdl_launch_dependents();  // tsum_kernel's grid may be scheduled as this grid's CTAs retire

  constexpr int kChunksPerRow = D / 8;                    // 16-byte pieces per row
  constexpr int kPieces = kTok * kChunksPerRow;           // per matrix
  auto stage_tile = [&](int j, int st) {
    const int tok0 = t_begin + j * kTok;
    const uint32_t kdst = smem_base + st * 2 * C::kMatBytes, vdst = kdst + C::kMatBytes;
    for (int i = tid; i < kPieces; i += C::kThreads) {
      const int r = i / kChunksPerRow, c = i - r * kChunksPerRow;
      const bool ok = tok0 + r < t_end;
      const size_t off = static_cast<size_t>(ok ? tok0 + r : t_begin) * D + c * 8;
      cp_async16(kdst + r * C::kRowBytes + c * 16, kbase + off, ok);
      cp_async16(vdst + r * C::kRowBytes + c * 16, vbase + off, ok);
    }
    cp_async_commit();
  };

  float acc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  // kStages - 1 tiles in flight; one commit group per iteration (an empty one past the end) keeps the
  // wait count fixed
  constexpr int kStages = C::kStages;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < n_tiles) stage_tile(s, s);
    else cp_async_commit();
  }
  for (int j = 0; j < n_tiles; ++j) {
    const int st = j % kStages;
    cp_async_wait<kStages - 2>();
    __syncthreads();  // tile j has landed for everyone, and everyone is done with tile j - 1
    if (j + kStages - 1 < n_tiles) stage_tile(j + kStages - 1, (j + kStages - 1) % kStages);
    else cp_async_commit();
    const uint32_t ks = smem_base + st * 2 * C::kMatBytes, vs = ks + C::kMatBytes;
#pragma unroll
    for (int kk = 0; kk < kTok / 16; ++kk) {
      // A = K^T: element (m = feature, k = token) is K[token][feature]; the stored 8x8 blocks are
      // (tokens, features) and the transposing load hands each thread (feature g, tokens 2t, 2t+1).
      uint32_t a[4];
      {
        const int mi = lane >> 3, r = lane & 7;
        const int tok = kk * 16 + r + ((mi & 2) ? 8 : 0);
        const int col = warp * 16 + ((mi & 1) ? 8 : 0);
        ldmatrix_x4_trans(a[0], a[1], a[2], a[3], ks + tok * C::kRowBytes + col * 2);
      }
#pragma unroll
      for (int nb = 0; nb < D / 16; ++nb) {
        // B = V: element (k = token, n = feature) is V[token][feature]; four 8x8 blocks cover 16 tokens
        // x 16 features: (tokens 0-7, n 0-7), (tokens 8-15, n 0-7), (tokens 0-7, n 8-15), (tokens 8-15, n 8-15)
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        const int tok = kk * 16 + r + ((mi & 1) ? 8 : 0);
        const int col = nb * 16 + ((mi & 2) ? 8 : 0);
        ldmatrix_x4_trans(b[0], b[1], b[2], b[3], vs + tok * C::kRowBytes + col * 2);
        mma_16816<T>(acc[2 * nb], a, b[0], b[1]);
        mma_16816<T>(acc[2 * nb + 1], a, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  // ---- partial to the workspace; tsum_kernel adds the chunks of a head in order
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  float* part = p.partials + (static_cast<size_t>(chunk) * p.hkv + hk) * D * D;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int row = warp * 16 + g, col = n * 8 + t2;
    *reinterpret_cast<float2*>(part + row * D + col) = make_float2(acc[n][0], acc[n][1]);
    *reinterpret_cast<float2*>(part + (row + 8) * D + col) = make_float2(acc[n][2], acc[n][3]);
  }
}

// Sums the chunk partials of T in chunk order (bit-stable) and stores T in the storage type: one thread
// per four consecutive elements, all of its loads in flight at once. A last-arriver sum inside ktv_kernel
// was measured first: one CTA per head walking 16 partials is a chain of dependent L2 round trips
// that took as long as the products themselves.
template <typename T>
__global__ void __launch_bounds__(256) tsum_kernel(const Params p, int dd) {
  const int per_head = dd / 4;
  const int idx = blockIdx.x * 256 + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();  // the partials are the preceding kernel's output
  if (idx >= p.hkv * per_head) return;
  const int hk = idx / per_head, i = (idx - hk * per_head) * 4;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < p.chunks; c0 += 8) {
    float4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = min(c0 + u, p.chunks - 1);
      x[u] = __ldcg(reinterpret_cast<const float4*>(p.partials + (static_cast<size_t>(c) * p.hkv + hk) * dd + i));
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + u < p.chunks) { s.x += x[u].x; s.y += x[u].y; s.z += x[u].z; s.w += x[u].w; }
    }
  }
  uint2 pk;
  pk.x = pack2<T>(s.x, s.y);
  pk.y = pack2<T>(s.z, s.w);
  *reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.t16) + static_cast<size_t>(hk) * dd + i) = pk;
}

// ------------------------------------------------------------------------------------------ Q T
template <typename T, int D>
__global__ void __launch_bounds__(128) qt_kernel(const Params p) {
  using C = Cfg<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, hk = h / (p.hq / p.hkv);
  const int q0 = blockIdx.x * C::kQtRows;
  const uint32_t qs = smem_u32(smem), ts = qs + C::kQtRows * C::kRowBytes;
  const T* qbase = reinterpret_cast<const T*>(p.q) + static_cast<size_t>(h) * p.sq * D;
  const T* tbase = reinterpret_cast<const T*>(p.t16) + static_cast<size_t>(hk) * D * D;
  constexpr int kChunksPerRow = D / 8;
  // Q does not depend on the kernels before this one: its copies are in flight while they finish
  for (int i = tid; i < C::kQtRows * kChunksPerRow; i += 128) {
    const int r = i / kChunksPerRow, c = i - r * kChunksPerRow;
    const bool ok = q0 + r < p.sq;
    cp_async16(qs + r * C::kRowBytes + c * 16, qbase + static_cast<size_t>(ok ? q0 + r : 0) * D + c * 8, ok);
  }
  pdl_wait();  // T is the preceding kernel's output
  for (int i = tid; i < D * kChunksPerRow; i += 128) {
    const int r = i / kChunksPerRow, c = i - r * kChunksPerRow;
    cp_async16(ts + r * C::kRowBytes + c * 16, tbase + static_cast<size_t>(r) * D + c * 8, true);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // warp w owns query rows [32 w, 32 w + 32): two 16-row blocks
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  T* obase = reinterpret_cast<T*>(p.out) + static_cast<size_t>(h) * p.sq * D;
#pragma unroll 1
  for (int mb = 0; mb < 2; ++mb) {
    const int r0 = warp * 32 + mb * 16;
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      {
        // A = Q, row-major: blocks (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
        const int mi = lane >> 3, r = lane & 7;
        const int row = r0 + r + ((mi & 1) ? 8 : 0);
        const int col = kk * 16 + ((mi & 2) ? 8 : 0);
        ldmatrix_x4(a[0], a[1], a[2], a[3], qs + row * C::kRowBytes + col * 2);
      }
#pragma unroll
      for (int nb = 0; nb < D / 16; ++nb) {
        uint32_t b[4];
        const int mi = lane >> 3, r = lane & 7;
        const int krow = kk * 16 + r + ((mi & 1) ? 8 : 0);
        const int col = nb * 16 + ((mi & 2) ? 8 : 0);
        ldmatrix_x4_trans(b[0], b[1], b[2], b[3], ts + krow * C::kRowBytes + col * 2);
        mma_16816<T>(acc[2 * nb], a, b[0], b[1]);
        mma_16816<T>(acc[2 * nb + 1], a, b[2], b[3]);
      }
    }
    // stage the 16 x D block over this warp's own rows of the Q tile (no other warp reads them), then
    // store whole 16-byte pieces: a row leaves as full 128-byte lines
    __syncwarp();
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int col = n * 8 + t2;
      *reinterpret_cast<uint32_t*>(smem + (r0 + g) * C::kRowBytes + col * 2) = pack2<T>(acc[n][0], acc[n][1]);
      *reinterpret_cast<uint32_t*>(smem + (r0 + g + 8) * C::kRowBytes + col * 2) = pack2<T>(acc[n][2], acc[n][3]);
    }
    __syncwarp();
    constexpr int kChunks = D / 8;
#pragma unroll
    for (int i = lane; i < 16 * kChunks; i += 32) {
      const int r = i / kChunks, c = i - r * kChunks;
      const int row = q0 + r0 + r;
      if (row < p.sq)
        *reinterpret_cast<uint4*>(obase + static_cast<size_t>(row) * D + c * 8) =
            *reinterpret_cast<const uint4*>(smem + (r0 + r) * C::kRowBytes + c * 16);
    }
  }
}

}  // namespace chain

// ------------------------------------------------------------------------------------- host side
namespace {

struct ChainPlan {
  bool chain;
  int chunks, chunk_tokens;
  size_t partials_off, t16_off, total;
};

int plan_chain(const cb200_matmul_matmul_args* a, ChainPlan* pl) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->q_len <= 0 || a->kv_len <= 0) return CB200_ERR_BAD_ARG;
  if (a->num_qo_heads % a->num_kv_heads) return CB200_ERR_BAD_ARG;
  if (a->head_dim != 64 && a->head_dim != 128) return CB200_ERR_UNSUPPORTED;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (a->impl < CB200_MM_AUTO || a->impl > CB200_MM_CHAIN) return CB200_ERR_BAD_ARG;
  const double d = a->head_dim, group = a->num_qo_heads / a->num_kv_heads;
  // FLOPs per kv head: scores first 4 g SQ SKV D, chain 2 (SKV + g SQ) D D
  const double ratio = 2.0 * group * a->q_len * static_cast<double>(a->kv_len) / (d * (a->kv_len + group * a->q_len));
  pl->chain = a->impl == CB200_MM_CHAIN || (a->impl == CB200_MM_AUTO && ratio >= 4.0);
  // chunks of whole 64-token tiles, enough CTAs for about four per SM
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  const int tiles = ceil_div(a->kv_len, chain::kTok);
  int chunks = ceil_div(4 * sms, a->num_kv_heads);
  if (chunks > tiles) chunks = tiles;
  if (chunks > 64) chunks = 64;
  if (chunks < 1) chunks = 1;
  pl->chunk_tokens = ceil_div(tiles, chunks) * chain::kTok;
  pl->chunks = ceil_div(a->kv_len, pl->chunk_tokens);
  const size_t dd = static_cast<size_t>(a->head_dim) * a->head_dim;
  pl->partials_off = kWsHeaderBytes;
  pl->t16_off = align_up(pl->partials_off + static_cast<size_t>(pl->chunks) * a->num_kv_heads * dd * 4, 256);
  pl->total = align_up(pl->t16_off + static_cast<size_t>(a->num_kv_heads) * dd * 2, 256);
  return CB200_OK;
}

template <typename T, int D>
int launch_chain(const cb200_matmul_matmul_args* a, const ChainPlan& pl, cudaStream_t st) {
  using C = chain::Cfg<D>;
  chain::Params p{};
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out;
  p.partials = reinterpret_cast<float*>(ws + pl.partials_off);
  p.t16 = ws + pl.t16_off;
  p.hq = a->num_qo_heads; p.hkv = a->num_kv_heads; p.sq = a->q_len; p.skv = a->kv_len;
  p.chunks = pl.chunks; p.chunk_tokens = pl.chunk_tokens;
  auto k1 = chain::ktv_kernel<T, D>;
  auto k2 = chain::qt_kernel<T, D>;
  CB200_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kKtvSmem));
  CB200_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kQtSmem));
  k1<<<dim3(pl.chunks, a->num_kv_heads), C::kThreads, C::kKtvSmem, st>>>(p);
  CB200_CUDA_TRY(cudaGetLastError());
  // the two kernels that follow are dependent launches: each is scheduled while its predecessor drains and
  // waits (griddepcontrol.wait) before it reads what the predecessor wrote
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const int dd = D * D;
  cudaLaunchConfig_t cfg = {};
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(ceil_div(a->num_kv_heads * (dd / 4), 256), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, chain::tsum_kernel<T>, p, dd));
  cfg.gridDim = dim3(ceil_div(a->q_len, C::kQtRows), a->num_qo_heads, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = C::kQtSmem;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, k2, p));
  return CB200_OK;
}

void to_prefill_args(const cb200_matmul_matmul_args* a, cb200_attn_prefill_args* f) {
  *f = cb200_attn_prefill_args{};
  f->q = a->q; f->k = a->k; f->v = a->v; f->out = a->out;
  f->workspace = a->workspace; f->workspace_bytes = a->workspace_bytes;
  f->num_qo_heads = a->num_qo_heads; f->num_kv_heads = a->num_kv_heads;
  f->q_len = a->q_len; f->kv_len = a->kv_len; f->head_dim = a->head_dim; f->dtype = a->dtype;
  f->sm_scale = 1.f;
  f->score_mode = CB200_SCORE_LINEAR;
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_matmul_matmul_uses_chain(const cb200_matmul_matmul_args* a) {
  cb200::ChainPlan pl;
  return cb200::plan_chain(a, &pl) == CB200_OK && pl.chain ? 1 : 0;
}

extern "C" size_t cb200_matmul_matmul_workspace_bytes(const cb200_matmul_matmul_args* a) {
  using namespace cb200;
  ChainPlan pl;
  if (plan_chain(a, &pl) != CB200_OK) return 0;
  if (pl.chain) return pl.total;
  cb200_attn_prefill_args f;
  to_prefill_args(a, &f);
  return cb200_attn_prefill_workspace_bytes(&f);
}

extern "C" int cb200_matmul_matmul(const cb200_matmul_matmul_args* a, void* stream) {
  using namespace cb200;
  ChainPlan pl;
  const int rc = plan_chain(a, &pl);
  if (rc != CB200_OK) return rc;
  if (!pl.chain) {
    cb200_attn_prefill_args f;
    to_prefill_args(a, &f);
    return cb200_attn_prefill(&f, stream);
  }
  if (!a->q || !a->k || !a->v || !a->out) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->q) | reinterpret_cast<uintptr_t>(a->k) | reinterpret_cast<uintptr_t>(a->v) |
       reinterpret_cast<uintptr_t>(a->out)) & 15)
    return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < pl.total) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return CB200_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f16 = a->dtype == CB200_F16;
  if (a->head_dim == 64) return f16 ? launch_chain<__half, 64>(a, pl, st) : launch_chain<__nv_bfloat16, 64>(a, pl, st);
  return f16 ? launch_chain<__half, 128>(a, pl, st) : launch_chain<__nv_bfloat16, 128>(a, pl, st);
}
