// nlfa_bwd_static_scratch: the backward for callers that cannot hand the
// library a scratch buffer.
//
// nlfa_bwd needs a [B,H,T] float32 Delta tape from its caller.  Some callers
// have no way to provide one: code running where the process's device memory
// has already been handed out in full to another allocator (an inference
// server's arena, a fixed per-tenant budget), or code that must not make any
// call that can allocate or implicitly synchronise.  For them the tape lives in
// a fixed array that is part of this library's device image.
//
// The array below costs kStaticScratchFloats * 4 bytes (4 MiB) on every GPU
// that loads the library, until the process exits.
#include <mutex>

#include "common.cuh"

namespace nlfa {
namespace {

constexpr size_t kStaticScratchFloats = size_t(1) << 20;          // B * H * T <= 1,048,576

// In host code this name is only a handle for the runtime's symbol lookup, not
// a device address; kernels get the address cudaGetSymbolAddress returns.
static __device__ __align__(256) float g_static_delta[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices];
std::mutex g_static_mutex;

// Device address of the array on the CURRENT device; looked up on the first
// call made with that device current, then cached.
int static_scratch(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return NLFA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_delta) != cudaSuccess || ptr == nullptr)
      return NLFA_ERR_CUDA;
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return NLFA_OK;
}

}  // namespace
}  // namespace nlfa

extern "C" {

size_t nlfa_static_scratch_max_rows(void) { return nlfa::kStaticScratchFloats; }

int nlfa_bwd_static_scratch(const void* dout, const void* q, const void* k, const void* v,
                            const void* o, const float* lse, void* dq, void* dk, void* dv, int B,
                            int T, int H, int Hkv, int D, float scale, int window, int sinks,
                            int dtype, int path, void* stream) {
  if (B < 0 || T < 0 || H < 0) return NLFA_ERR_BAD_SHAPE;
  const unsigned long long rows = 1ull * static_cast<unsigned>(B) * static_cast<unsigned>(H) *
                                  static_cast<unsigned>(T);
  if (rows > nlfa::kStaticScratchFloats) return NLFA_ERR_STATIC_SCRATCH_EXCEEDED;
  float* scratch = nullptr;
  const int st = nlfa::static_scratch(&scratch);
  if (st != NLFA_OK) return st;
  // The Delta pass overwrites every row the other two passes read, so nothing
  // left in the array by an earlier call can leak into this one.
  return nlfa_bwd_passes(dout, q, k, v, o, lse, dq, dk, dv, scratch,
                         nlfa::kStaticScratchFloats * sizeof(float), B, T, H, Hkv, D, scale,
                         window, sinks, dtype, path, NLFA_PASS_ALL, stream);
}

}  // extern "C"
