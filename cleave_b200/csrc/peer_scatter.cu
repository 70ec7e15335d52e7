// A rank's dense (m, n) block copied into column slices of several (m, ld)-pitched matrices at once: its own copy of
// a result sharded along N and the copies of the peer GPUs (peer-mapped pointers: symmetric memory, CUDA IPC).
//
// This is the all-gather of an N-sharded GEMM for the shapes whose product does not run on the CTA-pair kernel (which
// sends its tiles itself, gemm_pair.cu): few rows, a result of a megabyte or two, where a collective library's launch
// and protocol latency is most of the cost. One kernel, plain 16-byte stores, a row segment per warp instruction;
// nothing is signalled - the caller orders the GPUs (a barrier) before the result is read. The reference is
// single-GPU and has no counterpart.

#include "common.cuh"

#include <algorithm>

namespace cb200 {
namespace {

constexpr int kMaxDst = 8;

struct ScatterParams {
  const uint4* src;   // (m, pieces) 16-byte pieces, dense
  uint8_t* dst[kMaxDst];
  int n_dst, m, pieces;
  long long ld_bytes;  // row pitch of the destinations
};

__global__ void __launch_bounds__(256) peer_scatter_kernel(const ScatterParams p) {
  const long long total = static_cast<long long>(p.m) * p.pieces;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / p.pieces), piece = static_cast<int>(i - static_cast<long long>(row) * p.pieces);
    const uint4 v = __ldg(p.src + i);
    // every CTA starts with another destination, so that the stores of the GPU go to all links at any moment
    for (int dd = 0; dd < p.n_dst; ++dd) {
      const int d = (dd + static_cast<int>(blockIdx.x)) % p.n_dst;
      *reinterpret_cast<uint4*>(p.dst[d] + row * p.ld_bytes + piece * 16LL) = v;
    }
  }
}

}  // namespace
}  // namespace cb200

extern "C" int cb200_peer_scatter_cols(const void* src, int m, int n, int ld_dst, void* const* dsts, int n_dst,
                                       int dtype, void* stream) {
  using namespace cb200;
  if (!src || !dsts || m <= 0 || n <= 0 || n_dst <= 0 || n_dst > kMaxDst) return CB200_ERR_BAD_ARG;
  if (dtype != CB200_F16 && dtype != CB200_BF16) return CB200_ERR_UNSUPPORTED;
  if (n % 8 || ld_dst % 8 || ld_dst < n) return CB200_ERR_BAD_ARG;  // 16-byte pieces
  if (reinterpret_cast<uintptr_t>(src) & 15) return CB200_ERR_ALIGNMENT;
  ScatterParams p{};
  p.src = static_cast<const uint4*>(src);
  p.n_dst = n_dst;
  p.m = m;
  p.pieces = n / 8;
  p.ld_bytes = static_cast<long long>(ld_dst) * 2;
  for (int d = 0; d < n_dst; ++d) {
    if (!dsts[d] || (reinterpret_cast<uintptr_t>(dsts[d]) & 15)) return CB200_ERR_BAD_ARG;
    p.dst[d] = static_cast<uint8_t*>(dsts[d]);
  }
  const long long total = static_cast<long long>(m) * p.pieces;
  const int sms = sm_count();
  if (sms <= 0) return CB200_ERR_CUDA;
  const unsigned grid = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 4LL * sms));
  peer_scatter_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  CB200_CUDA_TRY(cudaGetLastError());
  return CB200_OK;
}
