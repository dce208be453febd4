// The two elementwise steps nanolab's mixer wraps around the attention core, each as one pass:
//
//   value blend (before the core, nanolab/mixers.py:294-297):
//       v' = (1 - s) * v + s * v0,  s = sigmoid(lambda), lambda a learnable scalar;
//       fused with the cast of v' to the kernel dtype (nanolab/flash_cuda.py:263-266)
//   head gate   (after the core,  nanolab/mixers.py:340-342):
//       y' = y * sigmoid(gate)[..., None],  gate [B,T,H] from a linear layer
//
// and their backward passes.  In torch each is several full passes over [B,T,H,D]
// (multiplies, an add, a cast; the backward also a reduction).  Here: HBM-bound, every
// operand read once, every result written once.  Reductions (the scalar's gradient, the
// gate's gradient per row) run in a fixed order: bit-reproducible, no atomics.
#include "rowwise.cuh"

namespace nlfa {
namespace {

using namespace rowwise;

__device__ inline float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------ value blend
template <typename TV, typename TOut>
__global__ void __launch_bounds__(kThreads)
value_blend_fwd_kernel(const TV* __restrict__ v, const TV* __restrict__ v0, const float* __restrict__ lambda,
                       TOut* __restrict__ out, unsigned nvec) {
  constexpr int U = Elem<TV>::kInFlight / 2;           // two operands per element
  const float s = sigmoidf(*lambda), c = 1.f - s;
  const unsigned span = gridDim.x * kThreads;          // consecutive threads take consecutive 8-element vectors
  for (unsigned i0 = blockIdx.x * kThreads + threadIdx.x; i0 < nvec; i0 += span * U) {
    typename Elem<TV>::Raw a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned i = i0 + u * span;
      a[u] = i < nvec ? Elem<TV>::load_raw(v + (size_t)i * kVec) : Elem<TV>::zero();
      b[u] = i < nvec ? Elem<TV>::load_raw(v0 + (size_t)i * kVec) : Elem<TV>::zero();
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned i = i0 + u * span;
      if (i < nvec) {
        float x[kVec], y[kVec];
        Elem<TV>::unpack(a[u], x);
        Elem<TV>::unpack(b[u], y);
#pragma unroll
        for (int j = 0; j < kVec; ++j) x[j] = c * x[j] + s * y[j];
        Elem<TOut>::store(out + (size_t)i * kVec, x);
      }
    }
  }
}

// g = gradient of the blend's output.  dv = (1 - s) g, dv0 = s g, and per CTA the partial sum of
// g * (v0 - v), whose total times s (1 - s) is the scalar's gradient.
template <typename TV, typename TG>
__global__ void __launch_bounds__(kThreads)
value_blend_bwd_kernel(const TG* __restrict__ g, const TV* __restrict__ v, const TV* __restrict__ v0,
                       const float* __restrict__ lambda, TV* __restrict__ dv, TV* __restrict__ dv0,
                       float* __restrict__ partial, unsigned nvec) {
  __shared__ float red[kThreads / 32];
  const float s = sigmoidf(*lambda), c = 1.f - s;
  const unsigned stride = gridDim.x * kThreads;
  float acc = 0.f;
  for (unsigned i = blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
    const typename Elem<TG>::Raw gr = Elem<TG>::load_raw(g + (size_t)i * kVec);
    const typename Elem<TV>::Raw ar = Elem<TV>::load_raw(v + (size_t)i * kVec);
    const typename Elem<TV>::Raw br = Elem<TV>::load_raw(v0 + (size_t)i * kVec);
    float gg[kVec], x[kVec], y[kVec];
    Elem<TG>::unpack(gr, gg);
    Elem<TV>::unpack(ar, x);
    Elem<TV>::unpack(br, y);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      acc = fmaf(gg[j], y[j] - x[j], acc);
      x[j] = c * gg[j];
      y[j] = s * gg[j];
    }
    Elem<TV>::store(dv + (size_t)i * kVec, x);
    Elem<TV>::store(dv0 + (size_t)i * kVec, y);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

__global__ void __launch_bounds__(1024)
value_blend_scalar_grad_kernel(const float* __restrict__ partial, int n, const float* __restrict__ lambda,
                               float* __restrict__ dlambda) {
  __shared__ float red[32];
  float a = 0.f;
  for (int i = threadIdx.x; i < n; i += 1024) a += partial[i];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += red[w];
    const float s = sigmoidf(*lambda);
    *dlambda = t * s * (1.f - s);
  }
}

// ------------------------------------------------------------------ head gate
// y [rows, D], gate [rows] -> out [rows, D] = y * round(sigmoid(gate)); torch rounds the sigmoid to the
// gate's type before the multiply (nanolab/mixers.py:341).
template <typename TY, typename TGate, int D>
__global__ void __launch_bounds__(kThreads)
head_gate_fwd_kernel(const TY* __restrict__ y, const TGate* __restrict__ gate, TY* __restrict__ out, unsigned rows) {
  constexpr int LPR = D / kVec, RPW = 32 / LPR, U = Elem<TY>::kInFlight;
  const unsigned lane = threadIdx.x & 31, sub = lane % LPR;
  const unsigned warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const unsigned stride = gridDim.x * (kThreads / 32) * (RPW * U);
  for (unsigned r0 = warp * (RPW * U); r0 < rows; r0 += stride) {
    typename Elem<TY>::Raw raw[U];
    float sg[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + u * RPW + lane / LPR;
      sg[u] = 0.f;
      if (row < rows) {
        raw[u] = Elem<TY>::load_raw(y + (size_t)row * D + sub * kVec);
        sg[u] = (float)gate[row];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + u * RPW + lane / LPR;
      if (row < rows) {
        float x[kVec];
        Elem<TY>::unpack(raw[u], x);
        const float s = Elem<TGate>::round(sigmoidf(sg[u]));
#pragma unroll
        for (int j = 0; j < kVec; ++j) x[j] *= s;
        Elem<TY>::store(out + (size_t)row * D + sub * kVec, x);
      }
    }
  }
}

// g = gradient of the gated output.  dy = g * s; dgate = rowsum(g * y) * s * (1 - s).
template <typename TY, typename TGate, int D>
__global__ void __launch_bounds__(kThreads)
head_gate_bwd_kernel(const TY* __restrict__ g, const TY* __restrict__ y, const TGate* __restrict__ gate,
                     TY* __restrict__ dy, TGate* __restrict__ dgate, unsigned rows) {
  constexpr int LPR = D / kVec, RPW = 32 / LPR, U = 2;
  const unsigned lane = threadIdx.x & 31, sub = lane % LPR;
  const unsigned warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const unsigned stride = gridDim.x * (kThreads / 32) * (RPW * U);
  for (unsigned r0 = warp * (RPW * U); r0 < rows; r0 += stride) {
    typename Elem<TY>::Raw graw[U], yraw[U];
    float sg[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + u * RPW + lane / LPR;
      graw[u] = Elem<TY>::zero();
      yraw[u] = Elem<TY>::zero();
      sg[u] = 0.f;
      if (row < rows) {
        graw[u] = Elem<TY>::load_raw(g + (size_t)row * D + sub * kVec);
        yraw[u] = Elem<TY>::load_raw(y + (size_t)row * D + sub * kVec);
        sg[u] = (float)gate[row];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {                      // the whole warp stays for the shuffles
      const unsigned row = r0 + u * RPW + lane / LPR;
      float gg[kVec], x[kVec];
      Elem<TY>::unpack(graw[u], gg);
      Elem<TY>::unpack(yraw[u], x);
      const float sf = sigmoidf(sg[u]);
      const float s = Elem<TGate>::round(sf);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        dot = fmaf(gg[j], x[j], dot);
        gg[j] *= s;
      }
      dot = Elem<TGate>::round(row_sum<LPR>(dot));     // torch returns this sum in the gate's type
      if (row < rows) {
        Elem<TY>::store(dy + (size_t)row * D + sub * kVec, gg);
        if (sub == 0) dgate[row] = (TGate)(dot * sf * (1.f - sf));
      }
    }
  }
}

int cta_count(long long units, int per_cta, int cap) {
  long long need = (units + per_cta - 1) / per_cta;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

template <typename TV>
int blend_fwd_out(int out_dtype, const void* v, const void* v0, const float* lam, void* out, unsigned nvec,
                  cudaStream_t st) {
  const int grid = cta_count(nvec, kThreads * (Elem<TV>::kInFlight / 2), 148 * 8);
  if (out_dtype == NLFA_DTYPE_BF16)
    value_blend_fwd_kernel<TV, __nv_bfloat16><<<grid, kThreads, 0, st>>>((const TV*)v, (const TV*)v0, lam,
                                                                         (__nv_bfloat16*)out, nvec);
  else if (out_dtype == NLFA_DTYPE_F16)
    value_blend_fwd_kernel<TV, __half><<<grid, kThreads, 0, st>>>((const TV*)v, (const TV*)v0, lam, (__half*)out, nvec);
  else
    value_blend_fwd_kernel<TV, float><<<grid, kThreads, 0, st>>>((const TV*)v, (const TV*)v0, lam, (float*)out, nvec);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename TV>
int blend_bwd_g(int g_dtype, const void* g, const void* v, const void* v0, const float* lam, void* dv, void* dv0,
                float* partial, float* dlam, unsigned nvec, cudaStream_t st) {
  const int grid = cta_count(nvec, kThreads, kMaxPartials);
#define NLFA_GO(TG)                                                                                              \
  value_blend_bwd_kernel<TV, TG><<<grid, kThreads, 0, st>>>((const TG*)g, (const TV*)v, (const TV*)v0, lam, (TV*)dv, \
                                                            (TV*)dv0, partial, nvec)
  if (g_dtype == NLFA_DTYPE_BF16) NLFA_GO(__nv_bfloat16);
  else if (g_dtype == NLFA_DTYPE_F16) NLFA_GO(__half);
  else NLFA_GO(float);
#undef NLFA_GO
  value_blend_scalar_grad_kernel<<<1, 1024, 0, st>>>(partial, grid, lam, dlam);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename TY, typename TGate>
int gate_for_dim(bool backward, int D, const void* g, const void* y, const void* gate, void* out, void* dgate,
                 unsigned rows, cudaStream_t st) {
  const int grid = cta_count(rows, (kThreads / 32) * (32 / (D / kVec)) * (backward ? 2 : Elem<TY>::kInFlight),
                             148 * 8);
#define NLFA_GO(DD)                                                                                               \
  do {                                                                                                            \
    if (backward)                                                                                                 \
      head_gate_bwd_kernel<TY, TGate, DD><<<grid, kThreads, 0, st>>>((const TY*)g, (const TY*)y, (const TGate*)gate, \
                                                                     (TY*)out, (TGate*)dgate, rows);             \
    else                                                                                                          \
      head_gate_fwd_kernel<TY, TGate, DD><<<grid, kThreads, 0, st>>>((const TY*)y, (const TGate*)gate, (TY*)out, rows); \
  } while (0)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename TY>
int gate_for_gate_dtype(bool backward, int gate_dtype, int D, const void* g, const void* y, const void* gate,
                        void* out, void* dgate, unsigned rows, cudaStream_t st) {
  if (gate_dtype == NLFA_DTYPE_BF16) return gate_for_dim<TY, __nv_bfloat16>(backward, D, g, y, gate, out, dgate, rows, st);
  if (gate_dtype == NLFA_DTYPE_F16) return gate_for_dim<TY, __half>(backward, D, g, y, gate, out, dgate, rows, st);
  return gate_for_dim<TY, float>(backward, D, g, y, gate, out, dgate, rows, st);
}

int gate_dispatch(bool backward, int y_dtype, int gate_dtype, int D, const void* g, const void* y, const void* gate,
                  void* out, void* dgate, unsigned rows, cudaStream_t st) {
  if (y_dtype == NLFA_DTYPE_BF16) return gate_for_gate_dtype<__nv_bfloat16>(backward, gate_dtype, D, g, y, gate, out, dgate, rows, st);
  if (y_dtype == NLFA_DTYPE_F16) return gate_for_gate_dtype<__half>(backward, gate_dtype, D, g, y, gate, out, dgate, rows, st);
  return gate_for_gate_dtype<float>(backward, gate_dtype, D, g, y, gate, out, dgate, rows, st);
}

}  // namespace
}  // namespace nlfa

extern "C" {

size_t nlfa_value_blend_scratch_bytes(void) { return (size_t)nlfa::rowwise::kMaxPartials * sizeof(float); }

int nlfa_value_blend_fwd(const void* v, const void* v0, int v_dtype, const float* lambda, void* out, int out_dtype,
                         long long n, void* stream) {
  using namespace nlfa;
  using namespace nlfa::rowwise;
  if (n < 0 || (n % kVec) != 0 || n / kVec >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
  if (!dtype_ok(v_dtype) || !dtype_ok(out_dtype)) return NLFA_ERR_BAD_DTYPE;
  if (n == 0) return NLFA_OK;
  if (!v || !v0 || !lambda || !out) return NLFA_ERR_NULL_POINTER;
  if (!aligned16(v) || !aligned16(v0) || !aligned16(out)) return NLFA_ERR_MISALIGNED;
  const unsigned nvec = (unsigned)(n / kVec);
  cudaStream_t st = (cudaStream_t)stream;
  if (v_dtype == NLFA_DTYPE_BF16) return blend_fwd_out<__nv_bfloat16>(out_dtype, v, v0, lambda, out, nvec, st);
  if (v_dtype == NLFA_DTYPE_F16) return blend_fwd_out<__half>(out_dtype, v, v0, lambda, out, nvec, st);
  return blend_fwd_out<float>(out_dtype, v, v0, lambda, out, nvec, st);
}

int nlfa_value_blend_bwd(const void* g, int g_dtype, const void* v, const void* v0, int v_dtype, const float* lambda,
                         void* dv, void* dv0, float* dlambda, void* scratch, size_t scratch_bytes, long long n,
                         void* stream) {
  using namespace nlfa;
  using namespace nlfa::rowwise;
  if (n < 0 || (n % kVec) != 0 || n / kVec >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
  if (!dtype_ok(v_dtype) || !dtype_ok(g_dtype)) return NLFA_ERR_BAD_DTYPE;
  if (!lambda || !dlambda) return NLFA_ERR_NULL_POINTER;
  cudaStream_t st = (cudaStream_t)stream;
  if (n == 0) return cudaMemsetAsync(dlambda, 0, sizeof(float), st) == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
  if (!g || !v || !v0 || !dv || !dv0 || !scratch) return NLFA_ERR_NULL_POINTER;
  if (scratch_bytes < nlfa_value_blend_scratch_bytes()) return NLFA_ERR_SCRATCH_TOO_SMALL;
  if (!aligned16(g) || !aligned16(v) || !aligned16(v0) || !aligned16(dv) || !aligned16(dv0)) return NLFA_ERR_MISALIGNED;
  const unsigned nvec = (unsigned)(n / kVec);
  if (v_dtype == NLFA_DTYPE_BF16)
    return blend_bwd_g<__nv_bfloat16>(g_dtype, g, v, v0, lambda, dv, dv0, (float*)scratch, dlambda, nvec, st);
  if (v_dtype == NLFA_DTYPE_F16)
    return blend_bwd_g<__half>(g_dtype, g, v, v0, lambda, dv, dv0, (float*)scratch, dlambda, nvec, st);
  return blend_bwd_g<float>(g_dtype, g, v, v0, lambda, dv, dv0, (float*)scratch, dlambda, nvec, st);
}

int nlfa_head_gate_fwd(const void* y, int y_dtype, const void* gate, int gate_dtype, void* out, long long rows, int D,
                       void* stream) {
  using namespace nlfa;
  using namespace nlfa::rowwise;
  if (rows < 0 || rows >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
  if (D != 32 && D != 64 && D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (!dtype_ok(y_dtype) || !dtype_ok(gate_dtype)) return NLFA_ERR_BAD_DTYPE;
  if (rows == 0) return NLFA_OK;
  if (!y || !gate || !out) return NLFA_ERR_NULL_POINTER;
  if (!aligned16(y) || !aligned16(out)) return NLFA_ERR_MISALIGNED;
  return gate_dispatch(false, y_dtype, gate_dtype, D, nullptr, y, gate, out, nullptr, (unsigned)rows,
                       (cudaStream_t)stream);
}

int nlfa_head_gate_bwd(const void* g, const void* y, int y_dtype, const void* gate, int gate_dtype, void* dy,
                       void* dgate, long long rows, int D, void* stream) {
  using namespace nlfa;
  using namespace nlfa::rowwise;
  if (rows < 0 || rows >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
  if (D != 32 && D != 64 && D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (!dtype_ok(y_dtype) || !dtype_ok(gate_dtype)) return NLFA_ERR_BAD_DTYPE;
  if (rows == 0) return NLFA_OK;
  if (!g || !y || !gate || !dy || !dgate) return NLFA_ERR_NULL_POINTER;
  if (!aligned16(g) || !aligned16(y) || !aligned16(dy)) return NLFA_ERR_MISALIGNED;
  return gate_dispatch(true, y_dtype, gate_dtype, D, g, y, gate, dy, dgate, (unsigned)rows, (cudaStream_t)stream);
}

}  // extern "C"
