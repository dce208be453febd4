// C-ABI entry points: argument validation, path selection, tensor-map encoding,
// the device status word, and the host half of the self-test.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {

// The status block bounded waits write when they give up: word [0] is the status, words
// [2..3] hold the device-visible address of the host's copy (ptx.cuh, report_timeout).
__device__ __align__(16) unsigned g_status_block[4];

// Work counters of the persistent kernels' in-kernel schedulers, two per launch.
constexpr unsigned kEagerSlots = 1024;       // ring for ordinary launches
constexpr unsigned kGraphSlots = 15360;      // handed out once each to launches under capture
__device__ unsigned g_sched[kEagerSlots + kGraphSlots][2];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_host_mutex;                     // guards the per-device tables below
unsigned* g_status_ptr[kMaxDevices];
unsigned* g_status_mirror[kMaxDevices];      // host address of the registered copy, or null
unsigned* g_sched_ptr[kMaxDevices];
int g_sm_count[kMaxDevices];
std::atomic<unsigned> g_next_eager{0};
std::atomic<unsigned> g_next_graph{0};

int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// Device address of the status block on the current device (looked up once per device).
unsigned* status_word() {
  const int dev = current_device();
  if (dev < 0) return nullptr;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_status_block) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<unsigned*>(ptr);
  }
  return g_status_ptr[dev];
}

// The host's copy of the status word for the current device: non-zero once a wait has given up.
unsigned host_status() {
  const int dev = current_device();
  if (dev < 0) return 0;
  const unsigned* m = g_status_mirror[dev];
  return m ? *reinterpret_cast<const volatile unsigned*>(m) : 0u;
}

// One CTA waits on a barrier nobody arrives at, with the caller's limit.
__global__ void wait_timeout_kernel(unsigned* status, unsigned long long limit_ns) {
  __shared__ unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&barrier), 1);
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtxLimit wctx{&abort_flag, status, limit_ns};
  if (threadIdx.x == 0) (void)mbar_wait(smem_u32(&barrier), 0, wctx, 0xee);
  __syncthreads();
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_problem(const Problem& p) {
  if (p.B < 0 || p.T < 0 || p.H < 0 || p.Hkv <= 0 || p.H % p.Hkv != 0) return NLFA_ERR_BAD_SHAPE;
  if (p.dtype != NLFA_DTYPE_F32 && p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16)
    return NLFA_ERR_BAD_DTYPE;
  if (p.D != 32 && p.D != 64 && p.D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (p.window < 0 || p.sinks < 0) return NLFA_ERR_BAD_WINDOW;
  if (p.window == 0 ? p.sinks != 0 : p.sinks >= p.window) return NLFA_ERR_BAD_WINDOW;
  if (p.block < 0 || (p.block > 0 && p.window > 0)) return NLFA_ERR_BAD_WINDOW;   // two masks, one slot (mixers.py:300-304)
  if (!(p.scale == p.scale)) return NLFA_ERR_BAD_SHAPE;
  return NLFA_OK;
}

float bits_to_float(uint16_t bits, int dtype) {
  if (dtype == NLFA_DTYPE_BF16) {
    uint32_t w = static_cast<uint32_t>(bits) << 16;
    float f;
    std::memcpy(&f, &w, 4);
    return f;
  }
  __half_raw r;
  r.x = bits;
  return __half2float(__half(r));
}

uint16_t float_to_bits(float x, int dtype) {
  if (dtype == NLFA_DTYPE_BF16) {
    __nv_bfloat16 b = __float2bfloat16_rn(x);
    uint16_t u;
    std::memcpy(&u, &b, 2);
    return u;
  }
  __half hh = __float2half_rn(x);
  uint16_t u;
  std::memcpy(&u, &hh, 2);
  return u;
}

}  // namespace

namespace {

struct MapKey {
  const void* base;
  int dtype, B, T, heads, D, rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && dtype == o.dtype && B == o.B && T == o.T && heads == o.heads &&
           D == o.D && rows == o.rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9e3779b97f4a7c15ull;
    auto mix = [&h](int v) { h = (h ^ static_cast<size_t>(v)) * 0x100000001b3ull; };
    mix(k.dtype); mix(k.B); mix(k.T); mix(k.heads); mix(k.D); mix(k.rows);
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;
constexpr size_t kMaxCachedMaps = 4096;

int encode_tile_map(CUtensorMap* map, const void* base, int dtype, int B, int T, int heads, int D,
                    int rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return NLFA_ERR_CUDA;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(D) * 2,
                                 static_cast<cuuint64_t>(heads) * D * 2,
                                 static_cast<cuuint64_t>(T) * heads * D * 2};
  const cuuint32_t box[4] = {64u, 1u, static_cast<cuuint32_t>(rows), 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt =
      dtype == NLFA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    // The encoder is a driver entry point and wants a context current on the calling thread.  A
    // host thread that has made no runtime call yet (an autograd worker, say) has none: a
    // runtime call that needs the context binds the device's primary one, then the encoding
    // is tried once more.
    int dev = 0, attr = 0;
    (void)cudaGetDevice(&dev);
    (void)cudaDeviceGetAttribute(&attr, cudaDevAttrMultiProcessorCount, dev);
    size_t free_b = 0, total_b = 0;
    (void)cudaMemGetInfo(&free_b, &total_b);
    r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  return r == CUDA_SUCCESS ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace

unsigned* status_block() { return status_word(); }

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int B, int T, int heads, int D,
                  int rows) {
  if (!aligned16(base)) return NLFA_ERR_MISALIGNED;
  const MapKey key{base, dtype, B, T, heads, D, rows};
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *map = it->second;
      return NLFA_OK;
    }
  }
  const int st = encode_tile_map(map, base, dtype, B, T, heads, D, rows);
  if (st != NLFA_OK) return st;
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  if (g_maps.size() >= kMaxCachedMaps) g_maps.clear();
  g_maps.emplace(key, *map);
  return NLFA_OK;
}

int sched_counters(cudaStream_t stream, unsigned** out) {
  const int dev = current_device();
  if (dev < 0) return NLFA_ERR_CUDA;
  unsigned* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    if (g_sched_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_sched) != cudaSuccess) return NLFA_ERR_CUDA;
      g_sched_ptr[dev] = static_cast<unsigned*>(ptr);
    }
    base = g_sched_ptr[dev];
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) return NLFA_ERR_CUDA;
  if (cap == cudaStreamCaptureStatusNone) {
    *out = base + 2 * (g_next_eager.fetch_add(1u, std::memory_order_relaxed) % kEagerSlots);
    return NLFA_OK;
  }
  const unsigned slot = g_next_graph.fetch_add(1u, std::memory_order_relaxed);
  if (slot >= kGraphSlots) return NLFA_ERR_GRAPH_SLOTS;   // every slot is bound into some captured graph
  *out = base + 2 * (kEagerSlots + slot);
  return NLFA_OK;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
  static std::mutex mutex;
  static std::unordered_map<const void*, unsigned long long> done;   // kernel -> device bit mask
  const int dev = current_device();
  if (dev < 0) return NLFA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mutex);
  unsigned long long& mask = done[kernel];
  if (mask & (1ull << dev)) return NLFA_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return NLFA_ERR_CUDA;
  mask |= 1ull << dev;
  return NLFA_OK;
}

bool overlap_launches(int kernel) {
  static const int mask = [] {
    const char* v = std::getenv("NLFA_PDL");
    return v != nullptr ? std::atoi(v) : kOverlapDefault;
  }();
  return (mask & kernel) != 0;
}

int sm_count() {
  const int dev = current_device();
  if (dev < 0) return 1;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 1;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

}  // namespace nlfa

using namespace nlfa;

extern "C" {

int nlfa_version(void) { return 1; }

const char* nlfa_strerror(int status) {
  switch (status < 0 ? -status : status) {
    case NLFA_OK: return "ok";
    case NLFA_ERR_NULL_POINTER: return "null pointer argument";
    case NLFA_ERR_BAD_SHAPE: return "bad shape (need B,T,H >= 0, Hkv > 0, H % Hkv == 0, finite scale)";
    case NLFA_ERR_BAD_DTYPE: return "unsupported dtype (float32, float16, bfloat16)";
    case NLFA_ERR_BAD_HEAD_DIM: return "unsupported head dim (32, 64, 128)";
    case NLFA_ERR_BAD_WINDOW: return "bad window/sinks (need window >= 0 and 0 <= sinks < window)";
    case NLFA_ERR_MISALIGNED: return "base pointer is not 16-byte aligned";
    case NLFA_ERR_UNSUPPORTED_PATH: return "tensor-core path needs float16/bfloat16";
    case NLFA_ERR_NOT_SM100: return "device is not compute capability 10.x";
    case NLFA_ERR_CUDA: return "CUDA runtime or driver call failed";
    case NLFA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case NLFA_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
    case NLFA_ERR_SELFTEST_MISMATCH: return "tensor-core self-test disagrees with the host reference";
    case NLFA_ERR_BAD_ARGUMENT: return "bad argument";
    case NLFA_ERR_GRAPH_SLOTS:
      return "no scheduler counters left for launches under stream capture (15360 per process)";
    case NLFA_ERR_STATIC_SCRATCH_EXCEEDED:
      return "problem too large for the built-in scratch array (need B*H*T <= 1048576)";
  }
  return "unknown status";
}

int nlfa_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10 ? 1 : 0;
}

int nlfa_resolve_path(int dtype, int head_dim, int path) {
  if (dtype != NLFA_DTYPE_F32 && dtype != NLFA_DTYPE_F16 && dtype != NLFA_DTYPE_BF16)
    return -NLFA_ERR_BAD_DTYPE;
  if (head_dim != 32 && head_dim != 64 && head_dim != 128) return -NLFA_ERR_BAD_HEAD_DIM;
  const bool tensor_ok = dtype != NLFA_DTYPE_F32;      // head dim 32 runs the 64-wide kernels, zero-padded by TMA
  if (path == NLFA_PATH_SIMT) return NLFA_PATH_SIMT;
  if (path == NLFA_PATH_TENSOR) return tensor_ok ? NLFA_PATH_TENSOR : -NLFA_ERR_UNSUPPORTED_PATH;
  if (path == NLFA_PATH_AUTO) return tensor_ok ? NLFA_PATH_TENSOR : NLFA_PATH_SIMT;
  return -NLFA_ERR_UNSUPPORTED_PATH;
}

int nlfa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
             int H, int Hkv, int D, float scale, int window, int sinks, int dtype, int path,
             void* stream) {
  return nlfa_fwd_masked(q, k, v, o, lse, B, T, H, Hkv, D, scale, window, sinks, 0, dtype, path, stream);
}

int nlfa_fwd_masked(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
                    int H, int Hkv, int D, float scale, int window, int sinks, int block, int dtype,
                    int path, void* stream) {
  Problem p{B, T, H, Hkv, D, window, sinks, scale, dtype, block};
  int st = check_problem(p);
  if (st != NLFA_OK) return st;
  int resolved = nlfa_resolve_path(dtype, D, path);
  if (resolved < 0) return -resolved;
  if (resolved == NLFA_PATH_TENSOR && !(scale > 0.f)) {
    // the tensor-core forward takes the row maximum before scaling: positive scales only
    if (path != NLFA_PATH_AUTO) return NLFA_ERR_UNSUPPORTED_PATH;
    resolved = NLFA_PATH_SIMT;
  }
  if (B == 0 || T == 0 || H == 0) return NLFA_OK;
  if (!q || !k || !v || !o || !lse) return NLFA_ERR_NULL_POINTER;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return NLFA_ERR_MISALIGNED;
  if (p.window > 0 && p.window - p.sinks >= p.T) {
    p.window = 0;            // the window never cuts anything: plain causal
    p.sinks = 0;
  }
  if (p.block == 1) p.block = 0;                            // blocks of one position: plain causal
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (resolved == NLFA_PATH_SIMT) return launch_fwd_simt(p, q, k, v, o, lse, s);
  if (!nlfa_device_supported()) return NLFA_ERR_NOT_SM100;
  if (host_status() != 0) return NLFA_ERR_DEVICE_TIMEOUT;   // an earlier kernel gave up: refuse until cleared
  unsigned* status = status_word();
  if (!status) return NLFA_ERR_CUDA;
  return launch_fwd_tc(p, q, k, v, o, lse, status, s);
}

size_t nlfa_bwd_scratch_bytes(int B, int T, int H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  return static_cast<size_t>(B) * H * T * sizeof(float);
}

int nlfa_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
             const float* lse, void* dq, void* dk, void* dv, void* scratch, size_t scratch_bytes,
             int B, int T, int H, int Hkv, int D, float scale, int window, int sinks, int dtype,
             int path, void* stream) {
  return nlfa_bwd_passes(dout, q, k, v, o, lse, dq, dk, dv, scratch, scratch_bytes, B, T, H, Hkv,
                         D, scale, window, sinks, dtype, path, NLFA_PASS_ALL, stream);
}

namespace {
size_t round256(size_t n) { return (n + 255) / 256 * 256; }
}  // namespace

size_t nlfa_bwd_fused_scratch_bytes(int B, int T, int H, int D) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  const size_t base = round256(nlfa_bwd_scratch_bytes(B, T, H));
  if (D > 64) return base;                              // no fused pass: the two passes need the tape only
  const size_t tiles = static_cast<size_t>(B) * H * ((T + kTile - 1) / kTile);
  return base + round256(tiles * sizeof(unsigned)) + tiles * kTile * 64 * sizeof(float);
}

int nlfa_bwd_fused(const void* dout, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, void* dq, void* dk, void* dv, void* scratch,
                   size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                   int window, int sinks, int dtype, int path, void* stream) {
  const int resolved = nlfa_resolve_path(dtype, D, path);
  const bool fused = resolved == NLFA_PATH_TENSOR && D <= 64;
  return nlfa_bwd_passes(dout, q, k, v, o, lse, dq, dk, dv, scratch, scratch_bytes, B, T, H, Hkv,
                         D, scale, window, sinks, dtype, path,
                         fused ? (NLFA_PASS_DELTA | NLFA_PASS_FUSED) : NLFA_PASS_ALL, stream);
}

int nlfa_bwd_kernel_count(int B, int T, int H, int D, int dtype, int path, int passes) {
  if (passes <= 0 || passes > (NLFA_PASS_ALL | NLFA_PASS_FUSED) || B <= 0 || T <= 0 || H <= 0) return 0;
  const int resolved = nlfa_resolve_path(dtype, D, path);
  if (resolved < 0) return 0;
  const int delta = (passes & NLFA_PASS_DELTA) ? 1 : 0;
  if (passes & NLFA_PASS_FUSED) {
    if ((passes & (NLFA_PASS_DKV | NLFA_PASS_DQ)) || resolved != NLFA_PATH_TENSOR || D > 64) return 0;
    return delta + 2;                                          // the pass and the convert kernel
  }
  const int two = ((passes & NLFA_PASS_DKV) ? 1 : 0) + ((passes & NLFA_PASS_DQ) ? 1 : 0);
  if (resolved == NLFA_PATH_TENSOR) {
    Problem p{B, T, H, H, D, 0, 0, 1.f, dtype, 0};
    if (bwd_delta_in_dq(p, passes)) return two;
  }
  return delta + two;
}

int nlfa_bwd_passes(const void* dout, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, void* dq, void* dk, void* dv, void* scratch,
                    size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                    int window, int sinks, int dtype, int path, int passes, void* stream) {
  return nlfa_bwd_masked(dout, q, k, v, o, lse, dq, dk, dv, scratch, scratch_bytes, B, T, H, Hkv, D, scale,
                         window, sinks, 0, dtype, path, passes, stream);
}

int nlfa_bwd_masked(const void* dout, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, void* dq, void* dk, void* dv, void* scratch,
                    size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                    int window, int sinks, int block, int dtype, int path, int passes, void* stream) {
  if (passes <= 0 || passes > (NLFA_PASS_ALL | NLFA_PASS_FUSED)) return NLFA_ERR_UNSUPPORTED_PATH;
  const bool want_fused = (passes & NLFA_PASS_FUSED) != 0;
  if (want_fused && (passes & (NLFA_PASS_DKV | NLFA_PASS_DQ))) return NLFA_ERR_UNSUPPORTED_PATH;
  Problem p{B, T, H, Hkv, D, window, sinks, scale, dtype, block};
  int st = check_problem(p);
  if (st != NLFA_OK) return st;
  const int resolved = nlfa_resolve_path(dtype, D, path);
  if (resolved < 0) return -resolved;
  if (want_fused && (resolved != NLFA_PATH_TENSOR || D > 64)) return NLFA_ERR_UNSUPPORTED_PATH;
  if (B == 0 || T == 0 || H == 0) return NLFA_OK;
  if (!dout || !q || !k || !v || !o || !lse || !dq || !dk || !dv || !scratch)
    return NLFA_ERR_NULL_POINTER;
  if (!aligned16(dout) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) ||
      !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return NLFA_ERR_MISALIGNED;
  if (want_fused && !aligned16(scratch)) return NLFA_ERR_MISALIGNED;
  if (scratch_bytes < (want_fused ? nlfa_bwd_fused_scratch_bytes(B, T, H, D) : nlfa_bwd_scratch_bytes(B, T, H)))
    return NLFA_ERR_SCRATCH_TOO_SMALL;
  if (p.window > 0 && p.window - p.sinks >= p.T) {
    p.window = 0;
    p.sinks = 0;
  }
  if (p.block == 1) p.block = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* delta = static_cast<float*>(scratch);
  if (resolved == NLFA_PATH_SIMT)
    return launch_bwd_simt(p, dout, q, k, v, o, lse, dq, dk, dv, delta, passes, s);
  if (!nlfa_device_supported()) return NLFA_ERR_NOT_SM100;
  if (host_status() != 0) return NLFA_ERR_DEVICE_TIMEOUT;   // an earlier kernel gave up: refuse until cleared
  unsigned* status = status_word();
  if (!status) return NLFA_ERR_CUDA;
  FusedScratch fs{nullptr, nullptr};
  if (want_fused) {
    uint8_t* ws = static_cast<uint8_t*>(scratch) + round256(nlfa_bwd_scratch_bytes(B, T, H));
    const size_t tiles = static_cast<size_t>(B) * H * ((T + kTile - 1) / kTile);
    fs.dq_turn = reinterpret_cast<unsigned*>(ws);
    fs.dq_acc = reinterpret_cast<float*>(ws + round256(tiles * sizeof(unsigned)));
  }
  return launch_bwd_tc(p, dout, q, k, v, o, lse, dq, dk, dv, delta, passes, status, s,
                       want_fused ? &fs : nullptr);
}

int nlfa_selftest_tiles(int dtype, int head_dim, const void* q, const void* k, const void* v,
                        float* s_out, float* o_out, void* stream) {
  if (!q || !k || !v || !s_out || !o_out) return NLFA_ERR_NULL_POINTER;
  if (!nlfa_device_supported()) return NLFA_ERR_NOT_SM100;
  unsigned* status = status_word();
  if (!status) return NLFA_ERR_CUDA;
  return launch_selftest_tiles(dtype, head_dim, q, k, v, s_out, o_out, status,
                               static_cast<cudaStream_t>(stream));
}

int nlfa_check_mask_geometry(int T, int window, int sinks, int stream_rows) {
  return nlfa_check_mask_geometry_masked(T, window, sinks, 0, stream_rows);
}

int nlfa_check_mask_geometry_masked(int T, int window, int sinks, int block, int stream_rows) {
  if (T <= 0 || window < 0 || sinks < 0 || (window > 0 && sinks >= window) ||
      (window == 0 && sinks != 0) || block < 0 || (block > 0 && window > 0) ||
      (stream_rows != 64 && stream_rows != 128))
    return -NLFA_ERR_BAD_WINDOW;
  const int n128 = (T + kTile - 1) / kTile;
  const int nys = (T + stream_rows - 1) / stream_rows;
  int check = 0;
  // (1) key blocks given to a query tile cover every block with a visible pair
  for (int t = 0; t < n128; ++t) {
    const TileRange r = tile_range(t, window, sinks, block, n128);
    for (int j = 0; j < n128; ++j, ++check) {
      bool any = false;
      for (int q = t * kTile; q < (t + 1) * kTile && !any; ++q)
        for (int k = j * kTile; k < (j + 1) * kTile && !any; ++k) any = key_visible(q, k, window, sinks, block, T);
      const bool given = (j >= r.lo && j <= r.hi) || j < r.sink_blocks;
      if (any && !given) return 1 + check;
    }
  }
  // (2), (3): rectangles of a 128-row tile and a stream_rows-row tile, both orientations
  for (int orient = 0; orient < 2; ++orient)
    for (int t = 0; t < n128; ++t)
      for (int y = 0; y < nys; ++y) {
        const int q_lo = orient == 0 ? t * kTile : y * stream_rows;
        const int q_hi = q_lo + (orient == 0 ? kTile : stream_rows) - 1;
        const int k_lo = orient == 0 ? y * stream_rows : t * kTile;
        const int k_hi = k_lo + (orient == 0 ? stream_rows : kTile) - 1;
        bool all = true, causal_only = true, window_only = true;
        for (int q = q_lo; q <= q_hi; ++q)
          for (int k = k_lo; k <= k_hi; ++k) {
            const bool vis = key_visible(q, k, window, sinks, block, T);
            all = all && vis;
            causal_only = causal_only && (vis == (k <= last_key_of_query(q, block, T)));
            window_only = window_only && (vis == (k > q - (window - sinks)));
          }
        // (a rectangle made fully visible by sink keys alone may be reported as cut: that only costs a mask)
        if (rect_fully_visible(q_lo, q_hi, k_lo, k_hi, window, sinks, block, T) && !all) return 1 + check;
        ++check;
        const int e = rect_edges(q_lo, q_hi, k_lo, k_hi, window, sinks);
        if (e == EDGE_CAUSAL && !causal_only) return 1 + check;
        ++check;
        if (e == EDGE_WINDOW && !window_only) return 1 + check;
        ++check;
        if (stream_rows == kTile) {
          const int qt = orient == 0 ? t : y, kb = orient == 0 ? y : t;
          if (block_fully_visible(qt, kb, window, sinks, block, T) && !all) return 1 + check;
          ++check;
          if (!all) {
            const int be = block_edges(qt, kb, window, sinks);
            if ((be == EDGE_CAUSAL && !causal_only) || (be == EDGE_WINDOW && !window_only)) return 1 + check;
          }
          ++check;
        }
      }
  // (4) fused backward: the key blocks that stream query tile t take the turns 0 .. count - 1
  //     exactly once each, in ascending block order
  if (stream_rows == kTile)
    for (int t = 0; t < n128; ++t) {
      int expect = 0, count = 0;
      for (int j = 0; j < n128; ++j) {
        if (t < first_query_of_key(j * kTile, block) / kTile ||
            t > last_query_tile_of_block(j, n128, kTile, window, sinks))
          continue;
        const int turn = dq_turn_of_block(j, t, window, sinks, &count, block, n128);
        if (turn != expect) return 1 + check;
        ++expect;
      }
      ++check;
      if (expect != count) return 1 + check;
      ++check;
    }
  return 0;
}

size_t nlfa_selftest_workspace_bytes(void) {
  // q, k, v tiles (16-bit, D <= 128) then S [128,128] and O [128,128] float32
  return 3 * 128 * 128 * 2 + 2 * 128 * 128 * 4;
}

int nlfa_selftest(int dtype, int head_dim, void* workspace, size_t workspace_bytes,
                  float* max_abs_err, void* stream) {
  if (!workspace || !max_abs_err) return NLFA_ERR_NULL_POINTER;
  if (workspace_bytes < nlfa_selftest_workspace_bytes()) return NLFA_ERR_SCRATCH_TOO_SMALL;
  if (dtype != NLFA_DTYPE_F16 && dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (head_dim != 64 && head_dim != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  const int D = head_dim;
  const size_t n = static_cast<size_t>(128) * D;
  std::vector<uint16_t> hq(n), hk(n), hv(n);
  std::vector<float> fq(n), fk(n), fv(n);
  uint32_t rng = 0x1234567u;
  auto next = [&rng]() {                       // small LCG; values in [-1, 1)
    rng = rng * 1664525u + 1013904223u;
    return static_cast<float>(static_cast<int32_t>(rng >> 8) & 0xffff) / 32768.f - 1.f;
  };
  for (size_t i = 0; i < n; ++i) {
    hq[i] = float_to_bits(next(), dtype); fq[i] = bits_to_float(hq[i], dtype);
    hk[i] = float_to_bits(next(), dtype); fk[i] = bits_to_float(hk[i], dtype);
    hv[i] = float_to_bits(next(), dtype); fv[i] = bits_to_float(hv[i], dtype);
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* dq = ws;
  void* dk = ws + 128 * 128 * 2;
  void* dv = ws + 2 * 128 * 128 * 2;
  float* ds = reinterpret_cast<float*>(ws + 3 * 128 * 128 * 2);
  float* dob = ds + 128 * 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(dq, hq.data(), n * 2, cudaMemcpyHostToDevice, s) != cudaSuccess ||
      cudaMemcpyAsync(dk, hk.data(), n * 2, cudaMemcpyHostToDevice, s) != cudaSuccess ||
      cudaMemcpyAsync(dv, hv.data(), n * 2, cudaMemcpyHostToDevice, s) != cudaSuccess)
    return NLFA_ERR_CUDA;
  int st = nlfa_selftest_tiles(dtype, D, dq, dk, dv, ds, dob, stream);
  if (st != NLFA_OK) return st;
  std::vector<float> S(128 * 128), O(n);
  if (cudaMemcpyAsync(S.data(), ds, S.size() * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaMemcpyAsync(O.data(), dob, n * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    return NLFA_ERR_CUDA;
  st = nlfa_device_status(nullptr);
  if (st != NLFA_OK) return st;
  double err_s = 0, mag_s = 1e-30, err_o = 0, mag_o = 1e-30;
  std::vector<float> P(128 * 128);
  for (int r = 0; r < 128; ++r)
    for (int c = 0; c < 128; ++c) {
      double acc = 0;
      for (int d = 0; d < D; ++d) acc += static_cast<double>(fq[r * D + d]) * fk[c * D + d];
      err_s = std::fmax(err_s, std::fabs(acc - S[r * 128 + c]));
      mag_s = std::fmax(mag_s, std::fabs(acc));
      P[r * 128 + c] = bits_to_float(float_to_bits(S[r * 128 + c], dtype), dtype);
    }
  for (int r = 0; r < 128; ++r)
    for (int d = 0; d < D; ++d) {
      double acc = 0;
      for (int c = 0; c < 128; ++c) acc += static_cast<double>(P[r * 128 + c]) * fv[c * D + d];
      err_o = std::fmax(err_o, std::fabs(acc - O[r * D + d]));
      mag_o = std::fmax(mag_o, std::fabs(acc));
    }
  max_abs_err[0] = static_cast<float>(err_s / mag_s);
  max_abs_err[1] = static_cast<float>(err_o / mag_o);
  if (!(max_abs_err[0] < 1e-2f) || !(max_abs_err[1] < 1e-2f)) return NLFA_ERR_SELFTEST_MISMATCH;
  return NLFA_OK;
}

int nlfa_device_status(unsigned* raw) {
  unsigned* ptr = status_word();
  if (!ptr) return NLFA_ERR_CUDA;
  unsigned word = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return NLFA_ERR_CUDA;
  if (cudaMemcpy(&word, ptr, sizeof(word), cudaMemcpyDeviceToHost) != cudaSuccess)
    return NLFA_ERR_CUDA;
  if (word != 0) {
    // Clear the word, the host's copy, and the schedulers' work counters (kernels that left
    // early did not re-arm theirs).  The device is idle: it was synchronised above.
    const unsigned zero = 0;
    cudaMemcpy(ptr, &zero, sizeof(zero), cudaMemcpyHostToDevice);
    const int dev = current_device();
    if (dev >= 0 && g_status_mirror[dev]) *reinterpret_cast<volatile unsigned*>(g_status_mirror[dev]) = 0u;
    void* sched = nullptr;
    if (cudaGetSymbolAddress(&sched, g_sched) == cudaSuccess) cudaMemset(sched, 0, sizeof(g_sched));
  }
  if (raw) *raw = word;
  return word == 0 ? NLFA_OK : NLFA_ERR_DEVICE_TIMEOUT;
}

int nlfa_peek_status(void) {
  return host_status() != 0 ? NLFA_ERR_DEVICE_TIMEOUT : NLFA_OK;
}

int nlfa_set_status_mirror(unsigned* host_word) {
  unsigned* ptr = status_word();
  const int dev = current_device();
  if (!ptr || dev < 0) return NLFA_ERR_CUDA;
  unsigned long long dev_addr = 0;
  if (host_word != nullptr) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host_word) != cudaSuccess) {
      (void)cudaGetLastError();
      return NLFA_ERR_BAD_ARGUMENT;
    }
    if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) return NLFA_ERR_BAD_ARGUMENT;
    dev_addr = reinterpret_cast<unsigned long long>(attr.devicePointer);
    *reinterpret_cast<volatile unsigned*>(host_word) = 0u;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return NLFA_ERR_CUDA;
  if (cudaMemcpy(ptr + 2, &dev_addr, sizeof(dev_addr), cudaMemcpyHostToDevice) != cudaSuccess)
    return NLFA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  g_status_mirror[dev] = host_word;
  return NLFA_OK;
}

int nlfa_test_wait_timeout(unsigned long long limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > WAIT_LIMIT_NS) return NLFA_ERR_BAD_ARGUMENT;
  unsigned* status = status_word();
  if (!status) return NLFA_ERR_CUDA;
  wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // extern "C"
