// The two-stage form of a split: the combine kernel of a partial + combine pair, and the conversion of
// normalised per-split attention results into the unnormalised partials the reference's split partial
// kernels emit. Compatibility with the reference's two-kernel plans
// (tests/graph/handwritten/expected_kernels/matmul_splitk_combine.py, mha_split_combine.py,
// {gqa,mha,mqa}_split_partial.py); the fused entry points do the same work inside one launch.
//
// Both kernels are bound by the few bytes they move: one thread per 16-byte output piece, grid sized to
// the SM count, loads of the `splits` axis kept in flight together, fp32 sums in split order (bit-stable).

#include "common.cuh"

namespace cb200 {
namespace {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(e[i]);
}

// num (outer, splits, inner) -> out (outer, inner); optional den (outer * inner_d / inner_d ..., splits[, inner])
template <typename T>
__global__ void __launch_bounds__(256) split_combine_kernel(const T* __restrict__ num, const T* __restrict__ den,
                                                           T* __restrict__ out, long long outer, long long inner,
                                                           int splits, int den_inner) {
  const long long pieces = outer * (inner / 8);  // inner is a multiple of 8
  const long long per_row = inner / 8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < pieces;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long o = idx / per_row, c = (idx - o * per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const T* src = num + (o * splits) * inner + c;
    for (int s0 = 0; s0 < splits; s0 += 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = s0 + u < splits ? __ldg(reinterpret_cast<const uint4*>(src + static_cast<long long>(s0 + u) * inner))
                               : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u >= splits) continue;
        float f[8];
        unpack8<T>(v[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    if (den != nullptr) {
      if (den_inner == 1) {
        float d = 0.f;
        for (int s = 0; s < splits; ++s) d += static_cast<float>(den[o * splits + s]);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] / d;
      } else {
        float d[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s) {
          float f[8];
          unpack8<T>(__ldg(reinterpret_cast<const uint4*>(den + (o * splits + s) * inner + c)), f);
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] += f[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = acc[i] / d[i];
      }
    }
    uint4 pk;
    pk.x = pack2<T>(acc[0], acc[1]);
    pk.y = pack2<T>(acc[2], acc[3]);
    pk.z = pack2<T>(acc[4], acc[5]);
    pk.w = pack2<T>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + o * inner + c) = pk;
  }
}

// A row sum that is a lone column (inner == 1): one thread per output value.
template <typename T>
__global__ void __launch_bounds__(256) split_combine_scalar_kernel(const T* __restrict__ num, const T* __restrict__ den,
                                                                  T* __restrict__ out, long long outer, long long inner,
                                                                  int splits, int den_inner) {
  const long long total = outer * inner;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long o = idx / inner, c = idx - o * inner;
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += static_cast<float>(num[(o * splits + s) * inner + c]);
    if (den != nullptr) {
      float d = 0.f;
      for (int s = 0; s < splits; ++s)
        d += static_cast<float>(den_inner == 1 ? den[o * splits + s] : den[(o * splits + s) * inner + c]);
      acc /= d;
    }
    out[idx] = static_cast<T>(acc);
  }
}

// out / lse rows are (kv head, split, group member); the partials are (query head, split).
template <typename T>
__global__ void __launch_bounds__(256) attn_unnormalise_kernel(const T* __restrict__ out, const float* __restrict__ lse,
                                                              T* __restrict__ o_part, T* __restrict__ l_part, int kv_heads,
                                                              int group, int splits, int d, float shift_log2) {
  const int per_row = d / 8;
  const long long rows = static_cast<long long>(kv_heads) * splits * group;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < rows * per_row;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = idx / per_row;
    const int c = static_cast<int>(idx - row * per_row) * 8;
    const int j = static_cast<int>(row % group);
    const int s = static_cast<int>((row / group) % splits);
    const int h = static_cast<int>(row / (static_cast<long long>(group) * splits));
    const float l = lse[row];
    const float w = l == -INFINITY ? 0.f : fast_exp2(l + shift_log2);  // sum_j exp(score_j + shift)
    float f[8];
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(out + row * d + c)), f);
    uint4 pk;
    pk.x = pack2<T>(f[0] * w, f[1] * w);
    pk.y = pack2<T>(f[2] * w, f[3] * w);
    pk.z = pack2<T>(f[4] * w, f[5] * w);
    pk.w = pack2<T>(f[6] * w, f[7] * w);
    const long long dst_row = (static_cast<long long>(h) * group + j) * splits + s;
    *reinterpret_cast<uint4*>(o_part + dst_row * d + c) = pk;
    if (c == 0) l_part[dst_row] = static_cast<T>(w);
  }
}

int grid_for(long long work_items) {
  const int sms = sm_count();
  if (sms <= 0) return 0;
  long long blocks = (work_items + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;  // a few resident blocks per SM; the loops stride
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_split_combine(const cb200_split_combine_args* a, void* stream) {
  using namespace cb200;
  if (!a || !a->num || !a->out) return CB200_ERR_BAD_ARG;
  if (a->outer <= 0 || a->inner <= 0 || a->splits <= 0) return CB200_ERR_BAD_ARG;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (a->den && a->den_inner != 1 && a->den_inner != a->inner) return CB200_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f16 = a->dtype == CB200_F16;
  const bool vec = a->inner % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(a->num) | reinterpret_cast<uintptr_t>(a->out) |
                     (a->den_inner == 1 ? 0 : reinterpret_cast<uintptr_t>(a->den))) & 15) == 0;
  const int grid = grid_for(vec ? a->outer * (a->inner / 8) : a->outer * a->inner);
  if (grid <= 0) return CB200_ERR_CUDA;
  if (vec) {
    if (f16)
      split_combine_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(a->num), static_cast<const __half*>(a->den),
                                                        static_cast<__half*>(a->out), a->outer, a->inner, a->splits, a->den_inner);
    else
      split_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a->num),
                                                               static_cast<const __nv_bfloat16*>(a->den),
                                                               static_cast<__nv_bfloat16*>(a->out), a->outer, a->inner, a->splits,
                                                               a->den_inner);
  } else {
    if (f16)
      split_combine_scalar_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(a->num), static_cast<const __half*>(a->den),
                                                               static_cast<__half*>(a->out), a->outer, a->inner, a->splits, a->den_inner);
    else
      split_combine_scalar_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a->num),
                                                                      static_cast<const __nv_bfloat16*>(a->den),
                                                                      static_cast<__nv_bfloat16*>(a->out), a->outer, a->inner,
                                                                      a->splits, a->den_inner);
  }
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

extern "C" int cb200_attn_unnormalise(const cb200_attn_unnormalise_args* a, void* stream) {
  using namespace cb200;
  if (!a || !a->out || !a->lse || !a->o_part || !a->l_part) return CB200_ERR_BAD_ARG;
  if (a->kv_heads <= 0 || a->group <= 0 || a->splits <= 0 || a->head_dim <= 0 || a->head_dim % 8) return CB200_ERR_BAD_ARG;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->out) | reinterpret_cast<uintptr_t>(a->o_part)) & 15) return CB200_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long items = static_cast<long long>(a->kv_heads) * a->splits * a->group * (a->head_dim / 8);
  const int grid = grid_for(items);
  if (grid <= 0) return CB200_ERR_CUDA;
  const float shift_log2 = a->shift * 1.4426950408889634f;
  if (a->dtype == CB200_F16)
    attn_unnormalise_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(a->out), a->lse, static_cast<__half*>(a->o_part),
                                                         static_cast<__half*>(a->l_part), a->kv_heads, a->group, a->splits,
                                                         a->head_dim, shift_log2);
  else
    attn_unnormalise_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(a->out), a->lse,
                                                                static_cast<__nv_bfloat16*>(a->o_part),
                                                                static_cast<__nv_bfloat16*>(a->l_part), a->kv_heads, a->group,
                                                                a->splits, a->head_dim, shift_log2);
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}
