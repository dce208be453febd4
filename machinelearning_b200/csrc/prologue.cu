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
#include "rowwise.cuh"

namespace nlfa {
namespace {

using namespace rowwise;

// Rows are indexed with 32 bits (the host refuses B*T*H >= 2^31): the position of a row, (row / H) % T,
// would otherwise cost two 64-bit divisions per row group.

// x [rows, D] (rows = B*T*H, position t = (row / H) % T) -> y [rows, D]; rstd [rows] when weight != nullptr.
template <typename TIn, typename TOut, int D>
__global__ void __launch_bounds__(kThreads)
qk_prologue_fwd_kernel(const TIn* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ cosT,
                       const float* __restrict__ sinT, TOut* __restrict__ y, float* __restrict__ rstd,
                       unsigned rows, unsigned T, unsigned H, float eps) {
  constexpr int LPR = D / kVec;              // lanes per row
  constexpr int RPW = 32 / LPR;              // rows per warp and group
  constexpr int U = Elem<TIn>::kInFlight;    // row groups a warp has in flight per loop iteration
  const unsigned lane = threadIdx.x & 31;
  const unsigned sub = lane % LPR;           // which 8-element slot of the row
  const unsigned warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const unsigned stride = gridDim.x * (kThreads / 32) * (RPW * U);
  const float sign = sub < LPR / 2 ? -1.f : 1.f;       // rot = (-hi, lo)
  float w[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) w[i] = weight ? weight[sub * kVec + i] : 1.f;

  for (unsigned r0 = warp * (RPW * U); r0 < rows; r0 += stride) {
    typename Elem<TIn>::Raw raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {            // every load first; the whole warp stays for the shuffles
      const unsigned row = r0 + (lane / LPR) * U + u;
      raw[u] = row < rows ? Elem<TIn>::load_raw(x + (size_t)row * D + sub * kVec) : Elem<TIn>::zero();
    }
    // A lane's U rows are consecutive, so most of them share a position (H heads per position): the
    // table entries are fetched again only when the position changes.  (Fetching them per row made the
    // L1 the busiest unit: 64 bytes of table for every 16 bytes of x.)
    float c[kVec], s[kVec];
    unsigned t_have = 0xffffffffu;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + (lane / LPR) * U + u;
      const bool live = row < rows;
      float v[kVec];
      Elem<TIn>::unpack(raw[u], v);
      if (weight) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; ++i) ss = fmaf(v[i], v[i], ss);
        const float r = rsqrtf(row_sum<LPR>(ss) * (1.f / D) + eps);
        if (live && sub == 0) rstd[row] = r;
#pragma unroll
        for (int i = 0; i < kVec; ++i) v[i] = Elem<TIn>::round(v[i] * r * w[i]);
      }
      if (cosT) {
        const unsigned t = live ? (row / H) % T : 0u;
        if (t != t_have) {
          Elem<float>::load(cosT + (size_t)t * D + sub * kVec, c);
          Elem<float>::load(sinT + (size_t)t * D + sub * kVec, s);
          t_have = t;
        }
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float partner = __shfl_xor_sync(0xffffffffu, v[i], LPR / 2);
          v[i] = v[i] * c[i] + sign * partner * s[i];
        }
      }
      if (live) Elem<TOut>::store(y + (size_t)row * D + sub * kVec, v);
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
                       unsigned rows, unsigned T, unsigned H) {
  constexpr int LPR = D / kVec;
  constexpr int RPW = 32 / LPR;
  constexpr int U = 2;
  __shared__ float red[kThreads / 32][D];
  const unsigned lane = threadIdx.x & 31;
  const unsigned sub = lane % LPR;
  const unsigned warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const unsigned stride = gridDim.x * (kThreads / 32) * (RPW * U);
  const float sign = sub < LPR / 2 ? 1.f : -1.f;       // transpose of the rotation
  float w[kVec], dw[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) { w[i] = weight ? weight[sub * kVec + i] : 1.f; dw[i] = 0.f; }

  for (unsigned r0 = warp * (RPW * U); r0 < rows; r0 += stride) {
    typename Elem<TG>::Raw graw[U];
    typename Elem<TIn>::Raw xraw[U];
    float r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + (lane / LPR) * U + u;
      graw[u] = Elem<TG>::zero();
      xraw[u] = Elem<TIn>::zero();
      r[u] = 0.f;
      if (row < rows) {
        graw[u] = Elem<TG>::load_raw(gy + (size_t)row * D + sub * kVec);
        if (weight) { xraw[u] = Elem<TIn>::load_raw(x + (size_t)row * D + sub * kVec); r[u] = rstd[row]; }
      }
    }
    float c[kVec], s[kVec];                  // table entries, kept while the position stays the same
    unsigned t_have = 0xffffffffu;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned row = r0 + (lane / LPR) * U + u;
      const bool live = row < rows;
      float g[kVec], v[kVec];
      Elem<TG>::unpack(graw[u], g);
      Elem<TIn>::unpack(xraw[u], v);
      if (cosT) {
        const unsigned t = live ? (row / H) % T : 0u;
        if (t != t_have) {
          Elem<float>::load(cosT + (size_t)t * D + sub * kVec, c);
          Elem<float>::load(sinT + (size_t)t * D + sub * kVec, s);
          t_have = t;
        }
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float partner = __shfl_xor_sync(0xffffffffu, g[i] * s[i], LPR / 2);
          g[i] = g[i] * c[i] + sign * partner;
        }
      }
      if (weight) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          g[i] = Elem<TIn>::round(g[i]);     // the gradient passes back through rms_norm's output cast
          v[i] *= r[u];                      // normalised row
          dw[i] = fmaf(g[i], v[i], dw[i]);
          g[i] *= w[i];
          dot = fmaf(g[i], v[i], dot);
        }
        const float c = row_sum<LPR>(dot) * (1.f / D);
#pragma unroll
        for (int i = 0; i < kVec; ++i) g[i] = r[u] * (g[i] - v[i] * c);
      }
      if (live) Elem<TIn>::store(gx + (size_t)row * D + sub * kVec, g);
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
      partial[(size_t)blockIdx.x * D + threadIdx.x] = s;
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

int grid_for(long long rows, int D, int cap, int in_flight) {
  const long long rows_per_cta = (long long)(kThreads / 32) * (32 / (D / kVec)) * in_flight;
  long long need = (rows + rows_per_cta - 1) / rows_per_cta;
  if (need < 1) need = 1;
  return (int)(need < cap ? need : cap);
}

template <typename TIn, typename TOut>
int fwd_for_dim(int D, const void* x, const float* w, const float* c, const float* s, void* y, float* rstd,
                long long rows, int T, int H, float eps, cudaStream_t st) {
  const int grid = grid_for(rows, D, 148 * 8, Elem<TIn>::kInFlight);
#define NLFA_GO(DD)                                                                               \
  qk_prologue_fwd_kernel<TIn, TOut, DD><<<grid, kThreads, 0, st>>>((const TIn*)x, w, c, s, (TOut*)y, rstd,       \
                                                                   (unsigned)rows, (unsigned)T, (unsigned)H, eps)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename TIn, typename TG>
int bwd_for_dim(int D, const void* gy, const void* x, const float* w, const float* c, const float* s,
                const float* rstd, void* gx, float* partial, float* gweight, long long rows, int T, int H,
                cudaStream_t st) {
  const int grid = grid_for(rows, D, kMaxPartials, 2);
#define NLFA_GO(DD)                                                                                      \
  do {                                                                                                   \
    qk_prologue_bwd_kernel<TIn, TG, DD><<<grid, kThreads, 0, st>>>((const TG*)gy, (const TIn*)x, w, c, s, rstd, \
                                                                   (TIn*)gx, partial, (unsigned)rows,    \
                                                                   (unsigned)T, (unsigned)H);            \
    if (w) weight_grad_reduce_kernel<DD><<<1, 1024, 0, st>>>(partial, grid, gweight);                     \
  } while (0)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}


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
  if (rows >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
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
  if (rows >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
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
