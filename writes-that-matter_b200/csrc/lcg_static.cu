// Rank-7 GEMM for callers that must not allocate device memory.
//
// The bare rank-7 GEMM needs scratch: the seven A planes of the activation matrix
// (7/4 of its size) are formed first and then multiplied with the prepared B planes.
// Every other entry point leaves that buffer to the caller.  Some callers cannot
// provide one: an inference server that sizes its KV-cache pool from whatever device
// memory is free at start-up leaves nothing for a plugin to cudaMalloc later, and a
// serving thread may be forbidden to allocate at all because cudaMalloc synchronises
// the device.  For them the scratch lives in this translation unit as a fixed array
// in device memory.  With CUDA's lazy module loading (the default since CUDA 12.2) the
// array takes its memory on a GPU when its address is first resolved there -- inside
// lcg_static_reserve() or the first lcg_gemm_r7_static call on that device -- and keeps
// it until the process exits.  A host that sizes its own pool from the free memory
// calls lcg_static_reserve() on every device first (or runs with
// CUDA_MODULE_LOADING=EAGER, which takes the memory when the library is loaded).
#include <mutex>

#include "lcg_common.h"

#define LCG_STATIC_SCRATCH_BYTES (32ll << 20)

namespace lcg {
namespace {

// File-scope device array.  In host code this name is only a handle for the runtime,
// not a device address; the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_plane_scratch[LCG_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// Once per device, with that device current: resolve the array's device address.
int scratch_address(void** out) {
  int dev = -1;
  LCG_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(LCG_ERR_CUDA, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_plane_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(LCG_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s",
                  cudaGetErrorString(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return LCG_OK;
}

}  // namespace
}  // namespace lcg

using namespace lcg;

extern "C" int64_t lcg_static_scratch_bytes(void) { return LCG_STATIC_SCRATCH_BYTES; }

extern "C" int lcg_static_reserve(void) {
  void* planes = nullptr;
  return scratch_address(&planes);
}

extern "C" int lcg_gemm_r7_static(const lcg_scheme_t* scheme, const void* a, int64_t lda,
                                  const void* b_planes, int64_t ld_b, void* c, int64_t ldc,
                                  int64_t M, int64_t N, int64_t K, int schedule, int cta_group,
                                  int32_t* status, void* stream) {
  if (scheme == nullptr || a == nullptr || b_planes == nullptr || c == nullptr)
    return fail(LCG_ERR_BAD_ARG, "NULL operand");
  int64_t m2 = 0, k2 = 0, k2p = 0;
  if (int e = lcg_plane_geometry(M, K, 1, &m2, &k2, &k2p)) return e;
  const int64_t need = static_cast<int64_t>(scheme->rank) * m2 * k2p * 2;
  if (need > LCG_STATIC_SCRATCH_BYTES)
    return fail(LCG_ERR_UNSUPPORTED_SHAPE,
                "the A planes of a %lld x %lld activation need %lld bytes of scratch, the static "
                "scratch holds %lld; use lcg_a_planes + lcg_gemm_r7 with a caller-owned buffer",
                (long long)M, (long long)K, (long long)need, (long long)LCG_STATIC_SCRATCH_BYTES);
  void* planes = nullptr;
  if (int e = scratch_address(&planes)) return e;
  // Every element of the (rank * M2, K2p) plane matrix is written, padding included, so
  // nothing of an earlier call's contents survives into this one.
  if (int e = lcg_a_planes(scheme, a, M, K, lda, planes, k2p, stream)) return e;
  return lcg_gemm_r7(scheme, planes, k2p, b_planes, ld_b, c, ldc, M, N, K, schedule, cta_group,
                     status, stream);
}
