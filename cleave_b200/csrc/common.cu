// Host-side helpers shared by the kernel files, and the generic C entry points.
#include "common.cuh"

#include <cstring>
#include <mutex>

namespace cb200 {

int& last_cuda_error() {
  static thread_local int err = 0;
  return err;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

bool encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                       CUtensorMapL2promotion promo) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    last_cuda_error() = (int)cudaErrorSymbolNotFound;
    return false;
  }
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  const CUresult r = fn(out, dt, (cuuint32_t)rank, base, gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    last_cuda_error() = 100000 + (int)r;  // driver error codes are reported offset by 100000
    return false;
  }
  return true;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev < 64 && cached[dev]) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev < 64) cached[dev] = n;
  return n;
}

}  // namespace cb200

extern "C" int cb200_version(void) { return CB200_VERSION; }

extern "C" const char* cb200_strerror(int status) {
  switch (status) {
    case CB200_OK: return "ok";
    case CB200_ERR_BAD_ARG: return "bad argument (null pointer, non-positive extent or inconsistent shapes)";
    case CB200_ERR_UNSUPPORTED: return "shape or dtype not supported by the sm_100a kernels";
    case CB200_ERR_ALIGNMENT: return "pointer or stride is not 16-byte aligned";
    case CB200_ERR_WORKSPACE: return "workspace missing or too small";
    case CB200_ERR_CUDA: return "a CUDA call failed (see cb200_last_cuda_error)";
    case CB200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case CB200_ERR_SCRATCH_LIMIT:
      return "the problem needs more scratch than the library's built-in static array holds; "
             "use the entry point that takes a caller-owned workspace";
    default: return "unknown status";
  }
}

extern "C" int cb200_last_cuda_error(void) { return cb200::last_cuda_error(); }

extern "C" int cb200_sm_count(void) { return cb200::sm_count(); }

extern "C" int cb200_workspace_status(const void* workspace, void* stream) {
  if (!workspace) return CB200_ERR_BAD_ARG;
  int word = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CB200_CUDA_TRY(cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
  CB200_CUDA_TRY(cudaStreamSynchronize(st));
  if (word == 0) return CB200_OK;
  // A launch whose wait gave up leaves the status word set, which would make every later launch on this
  // workspace abandon its waits at the first check. The word is cleared here so that the fault is reported
  // once; the arrival counters of the items that launch did not finish are still dirty, so the caller must
  // zero the whole workspace (cb200_workspace_reset) before the next launch.
  CB200_CUDA_TRY(cudaMemsetAsync(const_cast<void*>(workspace), 0, cb200::kWsHeaderBytes, st));
  CB200_CUDA_TRY(cudaStreamSynchronize(st));
  return CB200_ERR_DEVICE_TIMEOUT;
}

extern "C" int cb200_workspace_reset(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < cb200::kWsHeaderBytes) return CB200_ERR_BAD_ARG;
  CB200_CUDA_TRY(cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream)));
  return CB200_OK;
}
