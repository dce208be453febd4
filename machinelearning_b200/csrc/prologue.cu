// Load-side prologue of the attention core for q or k, fused into one pass:
// per-head RMSNorm -> rotary embedding -> cast to the kernel dtype, and its backward.
//
// In nanolab these are separate tensor passes in front of every attention call:
// q_norm / k_norm (nanolab/mixers.py:287-289, RMSNorm at :46-56), apply_rope
// (:290-292, :68-75) and the cast + contiguous of flash_attn
// (nanolab/flash_cuda.py:263-266).  Here a row of D elements is read once and
// written once: HBM-bound, 2 + 2 bytes per element for 16-bit in and out.
//
// Thread mapping: a lane owns 8 consecutive elements of a row (one 16-byte load for
// 16-bit input), so a row is D/8 lanes and a warp holds 256/D rows.  The rotary
// partner of element e is e +- D/2, i.e. the same slot of lane ^ (D/16).
//
// Rounding follows torch's path for 16-bit input under autocast: the normalised,
// weighted row is rounded to the input type (rms_norm returns the input's type), the
// rotation runs in fp32, the result is rounded to the output type.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace nlfa {
namespace {

constexpr int kVec = 8;
constexpr int kThreads = 256;
constexpr int kMaxPartials = 148 * 8;   // CTAs of the backward; rows of the weight-gradient scratch

template <typename T> struct Elem;
template <> struct Elem<float> {
  __device__ static void load(const float* p, float (&v)[kVec]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ static void store(float* p, const float (&v)[kVec]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  __device__ static float round(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&v)[kVec]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[kVec]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
  __device__ static float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Elem<__half> {
  __device__ static void load(const __half* p, float (&v)[kVec]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__half* p, const float (&v)[kVec]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
  __device__ static float round(float x) { return __half2float(__float2half_rn(x)); }
};

// Sum over the D/8 lanes that share a row.
template <int LPR> __device__ inline float row_sum(float v) {
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

constexpr int kUnroll = 2;                 // row groups a warp has in flight per loop iteration

// x [rows, D] (rows = B*T*H, position t = (row / H) % T) -> y [rows, D]; rstd [rows] when weight != nullptr.
template <typename TIn, typename TOut, int D>
__global__ void __launch_bounds__(kThreads)
qk_prologue_fwd_kernel(const TIn* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ cosT,
                       const float* __restrict__ sinT, TOut* __restrict__ y, float* __restrict__ rstd,
                       long long rows, int T, int H, float eps) {
  constexpr int LPR = D / kVec;              // lanes per row
  constexpr int RPW = 32 / LPR;              // rows per warp and group
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;                // which 8-element slot of the row
  const long long warp = (long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (kThreads / 32);
  const float sign = sub < LPR / 2 ? -1.f : 1.f;       // rot = (-hi, lo)
  float w[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) w[i] = weight ? weight[sub * kVec + i] : 1.f;

  for (long long r0 = warp * (RPW * kUnroll); r0 < rows; r0 += nwarps * (RPW * kUnroll)) {
    long long row[kUnroll];
    float v[kUnroll][kVec];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {      // every load first; the whole warp stays for the shuffles
      row[u] = r0 + u * RPW + lane / LPR;
#pragma unroll
      for (int i = 0; i < kVec; ++i) v[u][i] = 0.f;
      if (row[u] < rows) Elem<TIn>::load(x + row[u] * D + sub * kVec, v[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const bool live = row[u] < rows;
      if (weight) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; ++i) ss = fmaf(v[u][i], v[u][i], ss);
        const float r = rsqrtf(row_sum<LPR>(ss) * (1.f / D) + eps);
        if (live && sub == 0) rstd[row[u]] = r;
#pragma unroll
        for (int i = 0; i < kVec; ++i) v[u][i] = Elem<TIn>::round(v[u][i] * r * w[i]);
      }
      if (cosT) {
        const int t = live ? (int)((row[u] / H) % T) : 0;
        float c[kVec], s[kVec];
        Elem<float>::load(cosT + (long long)t * D + sub * kVec, c);
        Elem<float>::load(sinT + (long long)t * D + sub * kVec, s);
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float partner = __shfl_xor_sync(0xffffffffu, v[u][i], LPR / 2);
          c[i] = v[u][i] * c[i] + sign * partner * s[i];
        }
#pragma unroll
        for (int i = 0; i < kVec; ++i) v[u][i] = c[i];
      }
      if (live) Elem<TOut>::store(y + row[u] * D + sub * kVec, v[u]);
    }
  }
}

// gy [rows, D] (gradient of the prologue's output), x and rstd from the forward -> gx [rows, D] and one
// row of weight-gradient partial sums per CTA (partial [gridDim.x, D]).
template <typename TIn, typename TG, int D>
__global__ void __launch_bounds__(kThreads, 3)
qk_prologue_bwd_kernel(const TG* __restrict__ gy, const TIn* __restrict__ x, const float* __restrict__ weight,
                       const float* __restrict__ cosT, const float* __restrict__ sinT,
                       const float* __restrict__ rstd, TIn* __restrict__ gx, float* __restrict__ partial,
                       long long rows, int T, int H) {
  constexpr int LPR = D / kVec;
  constexpr int RPW = 32 / LPR;
  __shared__ float red[kThreads / 32][D];
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;
  const long long warp = (long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (kThreads / 32);
  const float sign = sub < LPR / 2 ? 1.f : -1.f;       // transpose of the rotation
  float w[kVec], dw[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) { w[i] = weight ? weight[sub * kVec + i] : 1.f; dw[i] = 0.f; }

  for (long long r0 = warp * (RPW * kUnroll); r0 < rows; r0 += nwarps * (RPW * kUnroll)) {
    long long row[kUnroll];
    float g[kUnroll][kVec], v[kUnroll][kVec], r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      row[u] = r0 + u * RPW + lane / LPR;
      r[u] = 0.f;
#pragma unroll
      for (int i = 0; i < kVec; ++i) { g[u][i] = 0.f; v[u][i] = 0.f; }
      if (row[u] < rows) {
        Elem<TG>::load(gy + row[u] * D + sub * kVec, g[u]);
        if (weight) { Elem<TIn>::load(x + row[u] * D + sub * kVec, v[u]); r[u] = rstd[row[u]]; }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const bool live = row[u] < rows;
      if (cosT) {
        const int t = live ? (int)((row[u] / H) % T) : 0;
        float c[kVec], s[kVec];
        Elem<float>::load(cosT + (long long)t * D + sub * kVec, c);
        Elem<float>::load(sinT + (long long)t * D + sub * kVec, s);
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float partner = __shfl_xor_sync(0xffffffffu, g[u][i] * s[i], LPR / 2);
          g[u][i] = g[u][i] * c[i] + sign * partner;
        }
      }
      if (weight) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          g[u][i] = Elem<TIn>::round(g[u][i]);   // the gradient passes back through rms_norm's output cast
          v[u][i] *= r[u];                       // normalised row
          dw[i] = fmaf(g[u][i], v[u][i], dw[i]);
          g[u][i] *= w[i];
          dot = fmaf(g[u][i], v[u][i], dot);
        }
        const float c = row_sum<LPR>(dot) * (1.f / D);
#pragma unroll
        for (int i = 0; i < kVec; ++i) g[u][i] = r[u] * (g[u][i] - v[u][i] * c);
      }
      if (live) Elem<TIn>::store(gx + row[u] * D + sub * kVec, g[u]);
    }
  }

  if (weight) {                              // CTA-wide sum of dw, fixed order: reproducible
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
#pragma unroll
      for (int off = LPR; off < 32; off <<= 1) dw[i] += __shfl_xor_sync(0xffffffffu, dw[i], off);
    }
    if (lane < LPR) {
#pragma unroll
      for (int i = 0; i < kVec; ++i) red[threadIdx.x >> 5][sub * kVec + i] = dw[i];
    }
    __syncthreads();
    if (threadIdx.x < D) {
      float s = 0.f;
#pragma unroll
      for (int wi = 0; wi < kThreads / 32; ++wi) s += red[wi][threadIdx.x];
      partial[(long long)blockIdx.x * D + threadIdx.x] = s;
    }
  }
}

// gweight[e] = sum over the n per-CTA rows of partial[:, e].  One CTA of 1024 threads: thread (g, e) adds
// rows g, g + G, ... (G = 1024 / D), then the G sums of a column are added in a fixed order.
template <int D>
__global__ void __launch_bounds__(1024)
weight_grad_reduce_kernel(const float* __restrict__ partial, int n, float* __restrict__ gweight) {
  constexpr int G = 1024 / D;
  __shared__ float red[G][D];
  const int e = threadIdx.x % D, g = threadIdx.x / D;
  float s = 0.f;
  for (int i = g; i < n; i += G) s += partial[(long long)i * D + e];
  red[g][e] = s;
  __syncthreads();
  if (g == 0) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < G; ++j) t += red[j][e];
    gweight[e] = t;
  }
}

int grid_for(long long rows, int D, int cap) {
  const long long rows_per_cta = (long long)(kThreads / 32) * (32 / (D / kVec)) * kUnroll;
  long long need = (rows + rows_per_cta - 1) / rows_per_cta;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

template <typename TIn, typename TOut>
int fwd_for_dim(int D, const void* x, const float* w, const float* c, const float* s, void* y, float* rstd,
                long long rows, int T, int H, float eps, cudaStream_t st) {
  const int grid = grid_for(rows, D, 148 * 8);
#define NLFA_GO(DD)                                                                               \
  qk_prologue_fwd_kernel<TIn, TOut, DD><<<grid, kThreads, 0, st>>>((const TIn*)x, w, c, s, (TOut*)y, rstd, rows, \
                                                                   T, H, eps)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename TIn, typename TG>
int bwd_for_dim(int D, const void* gy, const void* x, const float* w, const float* c, const float* s,
                const float* rstd, void* gx, float* partial, float* gweight, long long rows, int T, int H,
                cudaStream_t st) {
  const int grid = grid_for(rows, D, kMaxPartials);
#define NLFA_GO(DD)                                                                                      \
  do {                                                                                                   \
    qk_prologue_bwd_kernel<TIn, TG, DD><<<grid, kThreads, 0, st>>>((const TG*)gy, (const TIn*)x, w, c, s, rstd, \
                                                                   (TIn*)gx, partial, rows, T, H);       \
    if (w) weight_grad_reduce_kernel<DD><<<1, 1024, 0, st>>>(partial, grid, gweight);                     \
  } while (0)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

bool dtype_ok(int d) { return d == NLFA_DTYPE_F32 || d == NLFA_DTYPE_F16 || d == NLFA_DTYPE_BF16; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace nlfa

extern "C" {

size_t nlfa_qk_prologue_scratch_bytes(int D) {
  return (size_t)nlfa::kMaxPartials * (size_t)(D > 0 ? D : 0) * sizeof(float);
}

int nlfa_qk_prologue_fwd(const void* x, int x_dtype, const float* weight, const float* cos_table,
                         const float* sin_table, void* y, int y_dtype, float* rstd, int B, int T, int H, int D,
                         float eps, void* stream) {
  using namespace nlfa;
  if (B < 0 || T < 0 || H < 0) return NLFA_ERR_BAD_SHAPE;
  if (D != 32 && D != 64 && D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return NLFA_ERR_BAD_DTYPE;
  const long long rows = (long long)B * T * H;
  if (rows == 0) return NLFA_OK;
  if (!x || !y || (weight && !rstd) || ((cos_table == nullptr) != (sin_table == nullptr))) return NLFA_ERR_NULL_POINTER;
  if (!aligned16(x) || !aligned16(y) || !aligned16(cos_table) || !aligned16(sin_table)) return NLFA_ERR_MISALIGNED;
  cudaStream_t st = (cudaStream_t)stream;
#define NLFA_OUT(TIn)                                                                                              \
  (y_dtype == NLFA_DTYPE_BF16 ? fwd_for_dim<TIn, __nv_bfloat16>(D, x, weight, cos_table, sin_table, y, rstd, rows, T, H, eps, st) \
   : y_dtype == NLFA_DTYPE_F16 ? fwd_for_dim<TIn, __half>(D, x, weight, cos_table, sin_table, y, rstd, rows, T, H, eps, st)       \
                               : fwd_for_dim<TIn, float>(D, x, weight, cos_table, sin_table, y, rstd, rows, T, H, eps, st))
  if (x_dtype == NLFA_DTYPE_BF16) return NLFA_OUT(__nv_bfloat16);
  if (x_dtype == NLFA_DTYPE_F16) return NLFA_OUT(__half);
  return NLFA_OUT(float);
#undef NLFA_OUT
}

int nlfa_qk_prologue_bwd(const void* gy, int gy_dtype, const void* x, int x_dtype, const float* weight,
                         const float* cos_table, const float* sin_table, const float* rstd, void* gx,
                         float* gweight, void* scratch, size_t scratch_bytes, int B, int T, int H, int D,
                         void* stream) {
  using namespace nlfa;
  if (B < 0 || T < 0 || H < 0) return NLFA_ERR_BAD_SHAPE;
  if (D != 32 && D != 64 && D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (!dtype_ok(x_dtype) || !dtype_ok(gy_dtype)) return NLFA_ERR_BAD_DTYPE;
  const long long rows = (long long)B * T * H;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {
    if (weight && gweight && cudaMemsetAsync(gweight, 0, D * sizeof(float), st) != cudaSuccess) return NLFA_ERR_CUDA;
    return NLFA_OK;
  }
  if (!gy || !gx || (weight && (!x || !rstd || !gweight || !scratch)) ||
      ((cos_table == nullptr) != (sin_table == nullptr)))
    return NLFA_ERR_NULL_POINTER;
  if (weight && scratch_bytes < nlfa_qk_prologue_scratch_bytes(D)) return NLFA_ERR_SCRATCH_TOO_SMALL;
  if (!aligned16(gy) || !aligned16(gx) || !aligned16(x) || !aligned16(cos_table) || !aligned16(sin_table))
    return NLFA_ERR_MISALIGNED;
#define NLFA_G(TIn)                                                                                               \
  (gy_dtype == NLFA_DTYPE_BF16 ? bwd_for_dim<TIn, __nv_bfloat16>(D, gy, x, weight, cos_table, sin_table, rstd, gx, (float*)scratch, gweight, rows, T, H, st) \
   : gy_dtype == NLFA_DTYPE_F16 ? bwd_for_dim<TIn, __half>(D, gy, x, weight, cos_table, sin_table, rstd, gx, (float*)scratch, gweight, rows, T, H, st)       \
                                : bwd_for_dim<TIn, float>(D, gy, x, weight, cos_table, sin_table, rstd, gx, (float*)scratch, gweight, rows, T, H, st))
  if (x_dtype == NLFA_DTYPE_BF16) return NLFA_G(__nv_bfloat16);
  if (x_dtype == NLFA_DTYPE_F16) return NLFA_G(__half);
  return NLFA_G(float);
#undef NLFA_G
}

}  // extern "C"
