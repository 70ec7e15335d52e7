// Causal prefill whose key window is far shorter than its run of query rows: two light kernels, no tensor cores.
//
// The tcgen05 prefill kernels give one CTA, with nearly all of an SM's shared memory, to every tile of 128 query rows
// and head. The reference's captured prefill chunks include batches with thousands of query rows whose page table holds
// a few dozen tokens: under the end-aligned causal mask only the last min(q_len, kv_len) rows of a request see any key,
// every other row just has to be written as 0 / -inf, and the tile kernels spend their time starting and retiring
// CTAs that find nothing to do. For those batches the prefill operators launch, instead:
//
//   small_gqa_kernel / small_mla_kernel   one CTA per VISIBLE row. The visible rows are numbered compactly (a prefix
//                      over the requests of min(q_len, kv_len), found by one warp, 32 requests a step), so the grid
//                      is bounded by the number of keys, not of query rows. GQA: one warp per KV head takes the query
//                      heads of its group through the keys together; a lane owns head_dim / 32 columns, a key's row
//                      is one coalesced load, eight keys' rows are in flight. MLA (512 + 64): two heads per warp, a
//                      lane owns 16 latent and 2 position columns, a token's latent row serves as key and as value.
//   blind_rows_kernel  one warp per query row: finds the row's request and, if the row sees no key, writes it as zeros
//                      (and -inf). Light enough for 64 resident warps per SM, it runs at store bandwidth.
//
// The two are launched back to back with a programmatic edge so that they overlap (they write disjoint rows).
// Semantics are those of the large kernels (python/cleave/dynamic/reference.py:156-365): end-aligned causal
// mask, base-2 log-sum-exp, a row without visible keys is 0 / -inf, page ids clamped to the pool and ranges
// clipped to the page table's stated length.

#include "common.cuh"

namespace cb200 {
namespace small {

constexpr int kWarps = 8;  // warps per CTA
constexpr float kLog2e = 1.4426950408889634f;

struct GqaParams {
  const void* q;                 // (rows, hq, D)
  const void* k;                 // ragged: (tokens, hkv, D); paged: (pages, 1, hkv, D)
  const void* v;
  const int* qo_indptr;
  const int* kv_indptr;
  const int* kv_indices;         // null: ragged
  void* out;
  float* lse;
  int batch, rows, hq, hkv, num_pages, n_idx;  // n_idx: entries of the page table, or rows of the ragged key tensor
  float scale_log2;
};

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(e[i]);
}

__device__ __forceinline__ float warp_max_f(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum_f(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// A request's key count as the kernels use it: its slice of the page table (or of the ragged key tensor), clipped
// to the table's stated length.
__device__ __forceinline__ int clipped_keys(int base, int end, int n_idx) {
  if (base < 0 || base >= n_idx) return 0;
  return max(min(end - base, n_idx - base), 0);
}

// Visible row number v of the batch: under the end-aligned causal mask the rows of request r that see a key are its
// last vis_r = min(q_len_r, kv_len_r), and v counts them request after request. One warp finds the request by a scan
// of vis over 32 requests a step and returns the row, the start of its key range and the last key it sees; row < 0
// when the batch has no such row (the grid is an upper bound).
struct VisibleRow { int row, base, limit; };

__device__ __forceinline__ VisibleRow find_visible_row(const int* qo_indptr, const int* kv_indptr, int batch, int n_idx, int v,
                                                       int lane) {
  int run = 0;
  for (int r0 = 0; r0 < batch; r0 += 32) {
    const int r = min(r0 + lane, batch - 1);
    const int q0 = __ldg(qo_indptr + r), q1 = __ldg(qo_indptr + r + 1);
    const int b = __ldg(kv_indptr + r), e = __ldg(kv_indptr + r + 1);
    const int n = clipped_keys(b, e, n_idx);
    const int vis = r0 + lane < batch ? max(min(q1 - q0, n), 0) : 0;
    int inc = vis;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    const int total = __shfl_sync(0xffffffffu, inc, 31);
    if (v < run + total) {  // uniform
      const int src = __ffs(__ballot_sync(0xffffffffu, run + inc > v)) - 1;
      const int j = v - run - __shfl_sync(0xffffffffu, inc - vis, src);  // index among that request's visible rows
      const int q1s = __shfl_sync(0xffffffffu, q1, src), ns = __shfl_sync(0xffffffffu, n, src);
      const int vs = __shfl_sync(0xffffffffu, vis, src);
      return VisibleRow{q1s - vs + j, __shfl_sync(0xffffffffu, b, src), ns - vs + j};
    }
    run += total;
  }
  return VisibleRow{-1, 0, -1};
}

struct BlindParams {
  const int* qo_indptr;
  const int* kv_indptr;
  uint4* out;       // rows of row_vec 16-byte pieces
  float* lse;       // (rows, heads), may be null
  int batch, rows, row_vec, heads, n_idx;
};

// One warp per query row: the row's request is the last one whose first row is <= t (32 offsets a step, the key
// ranges fetched in the same trip); the row is blind when its request has no keys or it lies before the last kv_len
// rows of its request, and a blind row is written as zeros and -inf. Rows past the last request count as blind.
__global__ void __launch_bounds__(kWarps * 32) blind_rows_kernel(const BlindParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kWarps + warp;
  if (t < p.rows) {
    bool blind = true;
    for (int r0 = 0; r0 < p.batch; r0 += 32) {
      const int r = min(r0 + lane, p.batch - 1);
      const int q0 = __ldg(p.qo_indptr + r), q1 = __ldg(p.qo_indptr + r + 1);
      const int b = __ldg(p.kv_indptr + r), e = __ldg(p.kv_indptr + r + 1);
      const unsigned m = __ballot_sync(0xffffffffu, r0 + lane < p.batch && q0 <= t);
      if (m == 0u) break;  // offsets are non-decreasing: nothing further on qualifies
      if (m != 0xffffffffu || r0 + 32 >= p.batch || __ldg(p.qo_indptr + r0 + 32) > t) {
        const int src = 31 - __clz(m);
        const int q0s = __shfl_sync(0xffffffffu, q0, src), q1s = __shfl_sync(0xffffffffu, q1, src);
        const int n = clipped_keys(__shfl_sync(0xffffffffu, b, src), __shfl_sync(0xffffffffu, e, src), p.n_idx);
        blind = t >= q1s || n == 0 || t - q0s < (q1s - q0s) - n;
        break;
      }
    }
    if (blind) {
      uint4* dst = p.out + static_cast<size_t>(t) * p.row_vec;
      for (int i = lane; i < p.row_vec; i += 32) dst[i] = make_uint4(0u, 0u, 0u, 0u);
      if (p.lse)
        for (int i = lane; i < p.heads; i += 32) p.lse[static_cast<size_t>(t) * p.heads + i] = -INFINITY;
    }
  }
  pdl_wait();  // launched beside the kernel of the visible rows: complete only after it, so that stream order holds
}

// One CTA per visible row, one warp per KV head, which takes the query heads of its group through the keys together
// (a key's row is loaded once for all of them). A lane owns D / 32 columns: a key's row is one coalesced load, its
// score a short product summed over the warp by shuffles, and the value row is in flight beside the key row, eight
// keys at a time.
template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32) small_gqa_kernel(const GqaParams p) {
  __shared__ int s_info[3];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kPer = D / 32;   // columns per lane
  constexpr int kKeys = 8;       // keys whose rows are in flight together
  pdl_launch_dependents();       // the kernel of the blind rows may start beside this one
  if (warp == 0) {
    const VisibleRow vr = find_visible_row(p.qo_indptr, p.kv_indptr, p.batch, p.n_idx, blockIdx.x, lane);
    if (lane == 0) { s_info[0] = vr.row; s_info[1] = vr.base; s_info[2] = vr.limit; }
  }
  __syncthreads();
  const int t = s_info[0], base = s_info[1], limit = s_info[2];
  if (t < 0) return;
  const T* qp = reinterpret_cast<const T*>(p.q);
  const T* kp = reinterpret_cast<const T*>(p.k);
  const T* vp = reinterpret_cast<const T*>(p.v);
  T* orow = reinterpret_cast<T*>(p.out) + static_cast<size_t>(t) * p.hq * D;
  const int G = p.hq / p.hkv;
  constexpr int kGroup = 8;  // query heads taken through the keys together (a KV head's group, in pieces of eight)
  for (int hk = warp; hk < p.hkv; hk += kWarps) {
    for (int g0 = 0; g0 < G; g0 += kGroup) {
      const int ng = min(kGroup, G - g0);
      float q4[kGroup][kPer], o[kGroup][kPer], m_run[kGroup], l_run[kGroup];
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.f;
        T e[kPer];
#pragma unroll
        for (int i = 0; i < kPer; ++i) e[i] = T(0.f);
        if (g < ng) {
          const T* src = qp + (static_cast<size_t>(t) * p.hq + hk * G + g0 + g) * D + lane * kPer;
          if constexpr (kPer == 4) *reinterpret_cast<uint2*>(e) = __ldg(reinterpret_cast<const uint2*>(src));
          else *reinterpret_cast<uint32_t*>(e) = __ldg(reinterpret_cast<const uint32_t*>(src));
        }
#pragma unroll
        for (int i = 0; i < kPer; ++i) { q4[g][i] = static_cast<float>(e[i]) * p.scale_log2; o[g][i] = 0.f; }
      }
      for (int j0 = 0; j0 <= limit; j0 += 32) {
        // the cache rows of the block's keys: lane = key, handed round by shuffles below
        const int j = min(j0 + lane, limit);
        long long row;
        if (p.kv_indices) {
          const int pg = min(max(__ldg(p.kv_indices + base + j), 0), p.num_pages - 1);
          row = static_cast<long long>(pg) * p.hkv + hk;
        } else {
          row = static_cast<long long>(base + j) * p.hkv + hk;
        }
        const int n_here = min(32, limit - j0 + 1);
        for (int s0 = 0; s0 < n_here; s0 += kKeys) {
          T kk[kKeys][kPer], vv[kKeys][kPer];
#pragma unroll
          for (int u = 0; u < kKeys; ++u) {
            const long long rw = __shfl_sync(0xffffffffu, row, min(s0 + u, n_here - 1));
            if constexpr (kPer == 4) {
              *reinterpret_cast<uint2*>(kk[u]) = __ldg(reinterpret_cast<const uint2*>(kp + rw * D + lane * 4));
              *reinterpret_cast<uint2*>(vv[u]) = __ldg(reinterpret_cast<const uint2*>(vp + rw * D + lane * 4));
            } else {
              *reinterpret_cast<uint32_t*>(kk[u]) = __ldg(reinterpret_cast<const uint32_t*>(kp + rw * D + lane * 2));
              *reinterpret_cast<uint32_t*>(vv[u]) = __ldg(reinterpret_cast<const uint32_t*>(vp + rw * D + lane * 2));
            }
          }
#pragma unroll
          for (int g = 0; g < kGroup; ++g) {
            if (g < ng) {
              float sc[kKeys], bm = -INFINITY;
#pragma unroll
              for (int u = 0; u < kKeys; ++u) {
                sc[u] = -INFINITY;
                if (s0 + u < n_here) {  // uniform: slots past the block's end cost nothing (a row with one key is common)
                  float part = 0.f;
#pragma unroll
                  for (int i = 0; i < kPer; ++i) part = fmaf(q4[g][i], static_cast<float>(kk[u][i]), part);
                  sc[u] = warp_sum_f(part);
                }
                bm = fmaxf(bm, sc[u]);
              }
              const float m_new = fmaxf(m_run[g], bm);  // finite: key s0 is visible
              const float alpha = fast_exp2(m_run[g] - m_new);
              l_run[g] *= alpha;
#pragma unroll
              for (int i = 0; i < kPer; ++i) o[g][i] *= alpha;
#pragma unroll
              for (int u = 0; u < kKeys; ++u) {
                if (s0 + u < n_here) {
                  const float pu = fast_exp2(sc[u] - m_new);
                  l_run[g] += pu;
#pragma unroll
                  for (int i = 0; i < kPer; ++i) o[g][i] = fmaf(pu, static_cast<float>(vv[u][i]), o[g][i]);
                }
              }
              m_run[g] = m_new;
            }
          }
        }
      }
#pragma unroll
      for (int g = 0; g < kGroup; ++g) {
        if (g < ng) {
          const int h = hk * G + g0 + g;
          const float inv = l_run[g] > 0.f ? 1.f / l_run[g] : 0.f;
          T* op = orow + static_cast<size_t>(h) * D + lane * kPer;
          if constexpr (kPer == 4) {
            uint2 u;
            u.x = pack2<T>(o[g][0] * inv, o[g][1] * inv);
            u.y = pack2<T>(o[g][2] * inv, o[g][3] * inv);
            *reinterpret_cast<uint2*>(op) = u;
          } else {
            *reinterpret_cast<uint32_t*>(op) = pack2<T>(o[g][0] * inv, o[g][1] * inv);
          }
          if (p.lse && lane == 0) p.lse[static_cast<size_t>(t) * p.hq + h] = l_run[g] > 0.f ? m_run[g] + fast_log2(l_run[g]) : -INFINITY;
        }
      }
    }
  }
}

struct MlaParams {
  const void* q_nope;   // (rows, H, 512)
  const void* q_pe;     // (rows, H, 64)
  const void* ckv;      // (pages, 1, 512)
  const void* kpe;      // (pages, 1, 64)
  const int* qo_indptr; // null: decode
  const int* kv_indptr;
  const int* kv_indices;
  void* out;
  float* lse;
  int batch, rows, heads, num_pages, n_idx;
  float scale_log2;
};

// The absorbed-latent form of the same: one CTA per visible row, two heads per warp; a lane owns 16 of the 512 latent
// columns and 2 of the 64 position columns, so a token's latent row is loaded once and serves as key and as value.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) small_mla_kernel(const MlaParams p) {
  constexpr int kCkv = 512, kKpe = 64, kKeys = 4;
  __shared__ int s_info[3];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  if (warp == 0) {
    const VisibleRow vr = find_visible_row(p.qo_indptr, p.kv_indptr, p.batch, p.n_idx, blockIdx.x, lane);
    if (lane == 0) { s_info[0] = vr.row; s_info[1] = vr.base; s_info[2] = vr.limit; }
  }
  __syncthreads();
  const int t = s_info[0], base = s_info[1], limit = s_info[2];
  if (t < 0) return;
  const T* ckv = reinterpret_cast<const T*>(p.ckv);
  const T* kpe = reinterpret_cast<const T*>(p.kpe);
  T* orow = reinterpret_cast<T*>(p.out) + static_cast<size_t>(t) * p.heads * kCkv;
  constexpr int kH = 2;  // heads a warp takes through the keys together
  for (int h0 = warp * kH; h0 < p.heads; h0 += kWarps * kH) {
    const int nh = min(kH, p.heads - h0);
    float qn[kH][16], qp2[kH][2], o[kH][16], m_run[kH], l_run[kH];
#pragma unroll
    for (int g = 0; g < kH; ++g) {
      m_run[g] = -INFINITY;
      l_run[g] = 0.f;
      const int h = min(h0 + g, p.heads - 1);
      const T* src = reinterpret_cast<const T*>(p.q_nope) + (static_cast<size_t>(t) * p.heads + h) * kCkv + lane * 16;
      float f[8];
      unpack8<T>(__ldg(reinterpret_cast<const uint4*>(src)), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) qn[g][i] = f[i] * p.scale_log2;
      unpack8<T>(__ldg(reinterpret_cast<const uint4*>(src) + 1), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) qn[g][8 + i] = f[i] * p.scale_log2;
      const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.q_pe) +
                                                                (static_cast<size_t>(t) * p.heads + h) * kKpe + lane * 2));
      const T* e = reinterpret_cast<const T*>(&u);
      qp2[g][0] = static_cast<float>(e[0]) * p.scale_log2;
      qp2[g][1] = static_cast<float>(e[1]) * p.scale_log2;
#pragma unroll
      for (int i = 0; i < 16; ++i) o[g][i] = 0.f;
    }
    for (int j0 = 0; j0 <= limit; j0 += 32) {
      const int pg = min(max(__ldg(p.kv_indices + base + min(j0 + lane, limit)), 0), p.num_pages - 1);  // lane = key
      const int n_here = min(32, limit - j0 + 1);
      for (int s0 = 0; s0 < n_here; s0 += kKeys) {
        uint4 c0[kKeys], c1[kKeys];
        uint32_t pe[kKeys];
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
          const long long pgw = __shfl_sync(0xffffffffu, pg, min(s0 + u, n_here - 1));
          const uint4* cr = reinterpret_cast<const uint4*>(ckv + pgw * kCkv + lane * 16);
          c0[u] = __ldg(cr);
          c1[u] = __ldg(cr + 1);
          pe[u] = __ldg(reinterpret_cast<const uint32_t*>(kpe + pgw * kKpe + lane * 2));
        }
#pragma unroll
        for (int g = 0; g < kH; ++g) {
          if (g < nh) {
            float sc[kKeys], bm = -INFINITY;
#pragma unroll
            for (int u = 0; u < kKeys; ++u) {
              sc[u] = -INFINITY;
              if (s0 + u < n_here) {  // uniform: slots past the block's end cost nothing
                float f[8], part;
                const T* e = reinterpret_cast<const T*>(&pe[u]);
                part = qp2[g][0] * static_cast<float>(e[0]) + qp2[g][1] * static_cast<float>(e[1]);
                unpack8<T>(c0[u], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) part = fmaf(qn[g][i], f[i], part);
                unpack8<T>(c1[u], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) part = fmaf(qn[g][8 + i], f[i], part);
                sc[u] = warp_sum_f(part);
              }
              bm = fmaxf(bm, sc[u]);
            }
            const float m_new = fmaxf(m_run[g], bm);
            const float alpha = fast_exp2(m_run[g] - m_new);
            l_run[g] *= alpha;
#pragma unroll
            for (int i = 0; i < 16; ++i) o[g][i] *= alpha;
#pragma unroll
            for (int u = 0; u < kKeys; ++u) {
              if (s0 + u < n_here) {
                const float pu = fast_exp2(sc[u] - m_new);
                l_run[g] += pu;
                float f[8];
                unpack8<T>(c0[u], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[g][i] = fmaf(pu, f[i], o[g][i]);
                unpack8<T>(c1[u], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[g][8 + i] = fmaf(pu, f[i], o[g][8 + i]);
              }
            }
            m_run[g] = m_new;
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < kH; ++g) {
      if (g < nh) {
        const int h = h0 + g;
        const float inv = l_run[g] > 0.f ? 1.f / l_run[g] : 0.f;
        uint4 u0, u1;
        u0.x = pack2<T>(o[g][0] * inv, o[g][1] * inv);   u0.y = pack2<T>(o[g][2] * inv, o[g][3] * inv);
        u0.z = pack2<T>(o[g][4] * inv, o[g][5] * inv);   u0.w = pack2<T>(o[g][6] * inv, o[g][7] * inv);
        u1.x = pack2<T>(o[g][8] * inv, o[g][9] * inv);   u1.y = pack2<T>(o[g][10] * inv, o[g][11] * inv);
        u1.z = pack2<T>(o[g][12] * inv, o[g][13] * inv); u1.w = pack2<T>(o[g][14] * inv, o[g][15] * inv);
        uint4* op = reinterpret_cast<uint4*>(orow + static_cast<size_t>(h) * kCkv + lane * 16);
        op[0] = u0;
        op[1] = u1;
        if (p.lse && lane == 0) p.lse[static_cast<size_t>(t) * p.heads + h] = l_run[g] > 0.f ? m_run[g] + fast_log2(l_run[g]) : -INFINITY;
      }
    }
  }
}

// The most key/value tokens a page table (or a ragged key tensor) may hold for a prefill operator to take these
// kernels (it also asks for eight times as many query rows as keys). Per-request lengths live on the device; the host
// sees only this bound on their sum, which bounds the visible rows and every row's keys.
static int g_limit = 256;

// The kernel of the blind rows, launched so that it may run beside the kernel launched just before it.
static int launch_blind_rows(const BlindParams& bp, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((bp.rows + kWarps - 1) / kWarps));
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, blind_rows_kernel, bp));
  return CB200_OK;
}

}  // namespace small

int small_problem_limit() { return small::g_limit; }

bool small_prefill_applies(int keys, int total_q) {
  const int lim = small::g_limit;
  return lim > 0 && keys > 0 && keys <= lim && 8LL * keys <= total_q;
}

int launch_small_gqa(const void* q, const void* k, const void* v, const int* qo_indptr, const int* kv_indptr,
                     const int* kv_indices, void* out, float* lse, int batch, int rows, int hq, int hkv, int head_dim,
                     int num_pages, int n_idx, float sm_scale, int dtype, cudaStream_t stream) {
  using namespace small;
  if (rows <= 0 || batch <= 0) return CB200_OK;
  GqaParams p{q, k, v, qo_indptr, kv_indptr, kv_indices, out, lse, batch, rows, hq, hkv, num_pages, n_idx, sm_scale * kLog2e};
  const unsigned grid = static_cast<unsigned>(min(n_idx, rows));  // the visible rows are at most the keys
  const bool f16 = dtype == CB200_F16;
  if (head_dim == 128) {
    if (f16) small_gqa_kernel<__half, 128><<<grid, kWarps * 32, 0, stream>>>(p);
    else small_gqa_kernel<__nv_bfloat16, 128><<<grid, kWarps * 32, 0, stream>>>(p);
  } else {
    if (f16) small_gqa_kernel<__half, 64><<<grid, kWarps * 32, 0, stream>>>(p);
    else small_gqa_kernel<__nv_bfloat16, 64><<<grid, kWarps * 32, 0, stream>>>(p);
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return launch_blind_rows(BlindParams{qo_indptr, kv_indptr, static_cast<uint4*>(out), lse, batch, rows, hq * head_dim / 8, hq, n_idx},
                           stream);
}

int launch_small_mla(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe, const int* qo_indptr,
                     const int* kv_indptr, const int* kv_indices, void* out, float* lse, int batch, int rows, int heads,
                     int num_pages, int n_idx, float sm_scale, int dtype, cudaStream_t stream) {
  using namespace small;
  if (rows <= 0 || batch <= 0) return CB200_OK;
  MlaParams p{q_nope, q_pe, ckv, kpe, qo_indptr, kv_indptr, kv_indices, out, lse, batch, rows, heads, num_pages, n_idx,
              sm_scale * kLog2e};
  const unsigned grid = static_cast<unsigned>(min(n_idx, rows));
  if (dtype == CB200_F16) small_mla_kernel<__half><<<grid, kWarps * 32, 0, stream>>>(p);
  else small_mla_kernel<__nv_bfloat16><<<grid, kWarps * 32, 0, stream>>>(p);
  CB200_CUDA_TRY(cudaGetLastError());
  return launch_blind_rows(BlindParams{qo_indptr, kv_indptr, static_cast<uint4*>(out), lse, batch, rows, heads * 512 / 8, heads, n_idx},
                           stream);
}

}  // namespace cb200

// The bound on the tokens of a page table (or ragged key tensor) under which the causal prefill operators take the
// kernels of this file when the query rows outnumber the keys eight to one; 0 turns them off. Returns the previous
// value. Process-wide, not synchronised.
extern "C" int cb200_set_small_problem_limit(int tokens) {
  const int old = cb200::small::g_limit;
  cb200::small::g_limit = tokens < 0 ? 0 : tokens;
  return old;
}
