// Two small fused operators of the reference's demo set that are compositions rather than new tiles.
//
//   matmul_rowsum   y[m] = sum_n (X @ W)[m, n]                      (demo/matmul_rowsum.py)
//       The row sum commutes with the product: y = X @ (W 1). One pass over W gives s[k] = sum_n W[k, n]
//       in fp32, one pass over X gives y[m] = sum_k X[m, k] s[k]. Every input byte is read once and the
//       (M, N) product never exists: M*K + K*N elements of traffic and 2*(M*K + K*N) FLOPs instead of
//       2*M*N*K. Bound by HBM (and, at the demo's 1 MB, by two launch latencies).
//
//   lora            Y = X @ W + (X @ A) @ B                          (demo/lora.py)
//       Three launches of the tcgen05 GEMM of this library on one stream: T = X @ A (rank R columns),
//       Z = T @ B, Y = X @ W + Z with Z added in the epilogue of the last product. T and Z live in the
//       workspace in the storage type (the reference's kernels round intermediates the same way). The
//       launches are dependent launches: the big product streams W beside the two small ones and only
//       its epilogue waits for Z.

#include "common.cuh"

namespace cb200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(128) w_rowsum_kernel(const T* __restrict__ w, float* __restrict__ s, int n) {
  __shared__ float part[4];
  const int k = blockIdx.x, tid = threadIdx.x;
  const T* row = w + static_cast<size_t>(k) * n;
  float acc = 0.f;
  for (int c = tid * 8; c < n; c += 128 * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(row + c);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += static_cast<float>(e[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((tid & 31) == 0) part[tid >> 5] = acc;
  __syncthreads();
  if (tid == 0) s[k] = (part[0] + part[1]) + (part[2] + part[3]);
}

// one warp per row of X
template <typename T>
__global__ void __launch_bounds__(256) x_dot_kernel(const T* __restrict__ x, const float* __restrict__ s,
                                                    T* __restrict__ y, int m, int k) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= m) return;
  const T* row = x + static_cast<size_t>(r) * k;
  float acc = 0.f;
  for (int c = lane * 8; c < k; c += 32 * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(row + c);
    const T* e = reinterpret_cast<const T*>(&u);
    const float4 s0 = *reinterpret_cast<const float4*>(s + c), s1 = *reinterpret_cast<const float4*>(s + c + 4);
    acc = fmaf(static_cast<float>(e[0]), s0.x, acc);
    acc = fmaf(static_cast<float>(e[1]), s0.y, acc);
    acc = fmaf(static_cast<float>(e[2]), s0.z, acc);
    acc = fmaf(static_cast<float>(e[3]), s0.w, acc);
    acc = fmaf(static_cast<float>(e[4]), s1.x, acc);
    acc = fmaf(static_cast<float>(e[5]), s1.y, acc);
    acc = fmaf(static_cast<float>(e[6]), s1.z, acc);
    acc = fmaf(static_cast<float>(e[7]), s1.w, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) y[r] = static_cast<T>(acc);
}

int plan_rowsum(const cb200_matmul_rowsum_args* a) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return CB200_ERR_BAD_ARG;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (a->k % 8 || a->n % 8) return CB200_ERR_UNSUPPORTED;  // rows are read in 16-byte pieces
  return CB200_OK;
}

template <typename T>
int launch_rowsum(const cb200_matmul_rowsum_args* a, cudaStream_t st) {
  float* s = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + kWsHeaderBytes);
  w_rowsum_kernel<T><<<a->k, 128, 0, st>>>(reinterpret_cast<const T*>(a->w), s, a->n);
  CB200_CUDA_TRY(cudaGetLastError());
  x_dot_kernel<T><<<ceil_div(a->m, 8), 256, 0, st>>>(reinterpret_cast<const T*>(a->x), s, reinterpret_cast<T*>(a->y), a->m, a->k);
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}

// ---------------------------------------------------------------------------------------- LoRA
struct LoraLayout {
  cb200_gemm_args t, z, y;  // the three products
  size_t gemm_ws, t_off, z_off, total;
};

int plan_lora(const cb200_lora_args* a, LoraLayout* L) {
  if (!a) return CB200_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0 || a->r <= 0) return CB200_ERR_BAD_ARG;
  if (a->dtype != CB200_F16 && a->dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (a->k % 8 || a->n % 8 || a->r % 8) return CB200_ERR_UNSUPPORTED;
  cb200_gemm_args g{};
  g.op = CB200_GEMM_MATMUL;
  g.dtype = a->dtype;
  L->t = g; L->t.m = a->m; L->t.n = a->r; L->t.k = a->k;
  L->z = g; L->z.m = a->m; L->z.n = a->n; L->z.k = a->r;
  L->y = g; L->y.m = a->m; L->y.n = a->n; L->y.k = a->k;
  L->y.addend = reinterpret_cast<const void*>(16);  // planned as the launch will be: with an addend
  L->y.dependent_launch = 2;
  L->z.dependent_launch = 1;
  size_t ws = 0;
  for (const cb200_gemm_args* p : {&L->t, &L->z, &L->y}) {
    const size_t need = cb200_gemm_workspace_bytes(p);
    if (need == 0) return CB200_ERR_UNSUPPORTED;
    if (need > ws) ws = need;
  }
  L->gemm_ws = align_up(ws, 256);
  L->t_off = 3 * L->gemm_ws;  // one GEMM scratch per product: they overlap on the GPU
  L->z_off = align_up(L->t_off + static_cast<size_t>(a->m) * a->r * 2, 256);
  L->total = align_up(L->z_off + static_cast<size_t>(a->m) * a->n * 2, 256);
  return CB200_OK;
}

}  // namespace
}  // namespace cb200

extern "C" size_t cb200_matmul_rowsum_workspace_bytes(const cb200_matmul_rowsum_args* a) {
  return cb200::plan_rowsum(a) == CB200_OK ? cb200::kWsHeaderBytes + static_cast<size_t>(a->k) * 4 : 0;
}

extern "C" int cb200_matmul_rowsum(const cb200_matmul_rowsum_args* a, void* stream) {
  using namespace cb200;
  const int rc = plan_rowsum(a);
  if (rc != CB200_OK) return rc;
  if (!a->x || !a->w || !a->y) return CB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->w)) & 15) return CB200_ERR_ALIGNMENT;
  if (!a->workspace || a->workspace_bytes < cb200_matmul_rowsum_workspace_bytes(a)) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return CB200_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return a->dtype == CB200_F16 ? launch_rowsum<__half>(a, st) : launch_rowsum<__nv_bfloat16>(a, st);
}

extern "C" size_t cb200_lora_workspace_bytes(const cb200_lora_args* a) {
  cb200::LoraLayout L;
  return cb200::plan_lora(a, &L) == CB200_OK ? L.total : 0;
}

extern "C" int cb200_lora(const cb200_lora_args* a, void* stream) {
  using namespace cb200;
  LoraLayout L;
  const int rc = plan_lora(a, &L);
  if (rc != CB200_OK) return rc;
  if (!a->x || !a->w || !a->a || !a->b || !a->y) return CB200_ERR_BAD_ARG;
  if (!a->workspace || a->workspace_bytes < L.total) return CB200_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return CB200_ERR_ALIGNMENT;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  void* t = ws + L.t_off;
  void* z = ws + L.z_off;
  // Z waits for T before it reads anything; Y runs its whole main loop beside T and Z and waits for Z only
  // in its epilogue, where Z is added (dependent launches). Each product has its own GEMM scratch.
  int slot = 0;
  for (cb200_gemm_args* g : {&L.t, &L.z, &L.y}) {
    g->workspace = ws + static_cast<size_t>(slot++) * L.gemm_ws;
    g->workspace_bytes = L.gemm_ws;
  }
  L.z.dependent_launch = 1;
  L.y.dependent_launch = 2;
  L.t.x = a->x; L.t.w = a->a; L.t.y = t;
  L.z.x = t;    L.z.w = a->b; L.z.y = z;
  L.y.x = a->x; L.y.w = a->w; L.y.y = a->y; L.y.addend = z;
  for (const cb200_gemm_args* g : {&L.t, &L.z, &L.y}) {
    const int rc2 = cb200_gemm(g, stream);
    if (rc2 != CB200_OK) return rc2;
  }
  return CB200_OK;
}
