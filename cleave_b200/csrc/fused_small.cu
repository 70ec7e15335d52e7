// Two small fused operators of the reference's demo set that are compositions rather than new tiles.
//
//   matmul_rowsum   y[m] = sum_n (X @ W)[m, n]                      (demo/matmul_rowsum.py)
//       The row sum commutes with the product: y = X @ (W 1). One pass over W gives s[k] = sum_n W[k, n]
//       in fp32, one pass over X gives y[m] = sum_k X[m, k] s[k]. Every input byte is read once and the
//       (M, N) product never exists: M*K + K*N elements of traffic and 2*(M*K + K*N) FLOPs instead of
//       2*M*N*K. Bound by HBM (and, at the demo's 1 MB, by two launch latencies).
//
//   lora            Y = X @ W + (X @ A) @ B                          (demo/lora.py)
//       Two launches of the tcgen05 GEMM of this library on one stream: T = X @ A (rank R columns, kept
//       in the workspace in the storage type - the reference's kernels round intermediates the same way),
//       then Y = [X | T] @ [W ; B]: one product whose last K block comes from a second operand pair, so the
//       low-rank term lands in the same accumulator. The second launch is a dependent launch: it streams W
//       while T is computed and waits for T only before that last K block.

#include "common.cuh"

namespace cb200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(128) w_rowsum_kernel(const T* __restrict__ w, float* __restrict__ s, int n) {
  __shared__ float part[4];
  const int k = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();
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
  if (r >= m) {
    pdl_wait();
    return;
  }
  const T* row = x + static_cast<size_t>(r) * k;
  float acc = 0.f;
  // dependent launch: this row's first piece of X is fetched while w_rowsum_kernel finishes; s is its output
  uint4 first = make_uint4(0u, 0u, 0u, 0u);
  if (lane * 8 < k) first = *reinterpret_cast<const uint4*>(row + lane * 8);
  pdl_wait();
  for (int c = lane * 8; c < k; c += 32 * 8) {
    const uint4 u = c == lane * 8 ? first : *reinterpret_cast<const uint4*>(row + c);
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
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ceil_div(a->m, 8), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, x_dot_kernel<T>, reinterpret_cast<const T*>(a->x), const_cast<const float*>(s),
                                    reinterpret_cast<T*>(a->y), a->m, a->k));
  return CB200_OK;
}

// ---------------------------------------------------------------------------------------- LoRA
struct LoraLayout {
  cb200_gemm_args t, y;  // the two launches
  size_t gemm_ws, t_off, total;
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
  L->y = g; L->y.m = a->m; L->y.n = a->n; L->y.k = a->k;
  L->y.k2 = a->r;              // planned as the launch will be: with the second operand pair
  L->y.dependent_launch = 3;
  size_t ws = 0;
  for (const cb200_gemm_args* p : {&L->t, &L->y}) {
    const size_t need = cb200_gemm_workspace_bytes(p);
    if (need == 0) return CB200_ERR_UNSUPPORTED;
    if (need > ws) ws = need;
  }
  L->gemm_ws = align_up(ws, 256);
  L->t_off = 2 * L->gemm_ws;  // one GEMM scratch per launch: they overlap on the GPU
  L->total = align_up(L->t_off + static_cast<size_t>(a->m) * a->r * 2, 256);
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
  // T = X @ A, then Y = X @ W + T @ B as ONE product over the concatenated K of [X | T] and [W ; B]. The
  // second launch is a dependent launch: it streams W while T is still being computed and waits for T only
  // before it loads the rank-r K block. Each launch has its own GEMM scratch.
  L.t.workspace = ws;
  L.y.workspace = ws + L.gemm_ws;
  L.t.workspace_bytes = L.y.workspace_bytes = L.gemm_ws;
  L.t.x = a->x; L.t.w = a->a; L.t.y = t;
  L.y.x = a->x; L.y.w = a->w; L.y.y = a->y;
  L.y.x2 = t;   L.y.w2 = a->b;
  for (const cb200_gemm_args* g : {&L.t, &L.y}) {
    const int rc2 = cb200_gemm(g, stream);
    if (rc2 != CB200_OK) return rc2;
  }
  return CB200_OK;
}
