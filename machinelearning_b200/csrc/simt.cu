// fp32 SIMT attention kernels: the accuracy path (fp32 inputs need 1e-5) and the
// path for head dims the tensor-core kernels do not cover.  One warp owns one
// row (a query row in the forward and in dQ, a key row in dK/dV); lanes split the
// head dimension; scores are reduced with shuffles.  No shared memory, no
// atomics: results are bit-reproducible.
//
// Algebra follows the reference's FMA kernels (nanolab/csrc/flash_attn_cuda.cu
// :147-281 forward, :1234-1262 Delta, :1265-1366 dQ, :1371-1482 dK/dV): softmax
// in base 2, L = m ln2 + log(l), P recomputed from L in the backward,
// dS = P (dP - Delta) scale, the GQA group summed inside the dK/dV kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {
namespace {

constexpr int kWarpsPerBlock = 4;

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
fwd_simt_kernel(Problem p, const T* __restrict__ q, const T* __restrict__ k,
                const T* __restrict__ v, T* __restrict__ o, float* __restrict__ lse) {
  constexpr int R = D / 32;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long rows = static_cast<long long>(p.B) * p.H * p.T;
  if (row >= rows) return;
  const int t = static_cast<int>(row % p.T);
  const long long bh = row / p.T;
  const int h = static_cast<int>(bh % p.H);
  const int b = static_cast<int>(bh / p.H);
  const int hk = h / (p.H / p.Hkv);
  const float scale2 = p.scale * kLog2e;

  const T* qrow = q + ((static_cast<long long>(b) * p.T + t) * p.H + h) * D;
  float qr[R], acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    qr[r] = to_f32(qrow[lane + 32 * r]) * scale2;
    acc[r] = 0.f;
  }
  float m = -INFINITY, l = 0.f;

  int lo = 0, nsink = 0;
  if (p.window > 0) {
    const int first = t - (p.window - p.sinks) + 1;
    lo = first > 0 ? first : 0;
    nsink = p.sinks < lo ? p.sinks : lo;          // sinks not already inside the window
  }
  const long long kv_stride = static_cast<long long>(p.Hkv) * D;
  const T* kbase = k + (static_cast<long long>(b) * p.T * p.Hkv + hk) * D;
  const T* vbase = v + (static_cast<long long>(b) * p.T * p.Hkv + hk) * D;

  int t_last = last_key_of_query(t, p.block);            // block-causal: to the end of the row's block
  t_last = t_last < p.T - 1 ? t_last : p.T - 1;
  const int n = nsink + (t_last - lo + 1);
  for (int idx = 0; idx < n; ++idx) {
    const int j = idx < nsink ? idx : lo + (idx - nsink);
    const T* krow = kbase + j * kv_stride;
    const T* vrow = vbase + j * kv_stride;
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) part = fmaf(qr[r], to_f32(krow[lane + 32 * r]), part);
    const float s = warp_sum(part);
    const float m_new = fmaxf(m, s);
    const float alpha = exp2f(m - m_new);
    const float pj = exp2f(s - m_new);
    l = fmaf(l, alpha, pj);
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = fmaf(acc[r], alpha, pj * to_f32(vrow[lane + 32 * r]));
    m = m_new;
  }
  const float inv = 1.f / l;
  T* orow = o + ((static_cast<long long>(b) * p.T + t) * p.H + h) * D;
#pragma unroll
  for (int r = 0; r < R; ++r) orow[lane + 32 * r] = from_f32<T>(acc[r] * inv);
  if (lane == 0) lse[bh * p.T + t] = (m + log2f(l)) * kLn2;
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
delta_kernel(Problem p, const T* __restrict__ dout, const T* __restrict__ o,
             float* __restrict__ delta) {
  constexpr int R = D / 32;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long rows = static_cast<long long>(p.B) * p.T * p.H;
  if (row >= rows) return;               // row indexes [B,T,H]
  const int h = static_cast<int>(row % p.H);
  const long long bt = row / p.H;
  const int t = static_cast<int>(bt % p.T);
  const int b = static_cast<int>(bt / p.T);
  float part = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r)
    part = fmaf(to_f32(dout[row * D + lane + 32 * r]), to_f32(o[row * D + lane + 32 * r]), part);
  const float s = warp_sum(part);
  if (lane == 0) delta[(static_cast<long long>(b) * p.H + h) * p.T + t] = s;
}

// Delta for 16-bit tensors: pure streaming, so every thread moves 16 bytes of dO and of O
// per load (8 elements); D / 8 consecutive lanes share a row and combine with shuffles.
template <typename T, int D>
__global__ void __launch_bounds__(256)
delta_vec_kernel(Problem p, const T* __restrict__ dout, const T* __restrict__ o,
                 float* __restrict__ delta) {
  constexpr int kLanesPerRow = D / 8;                      // 8 (D = 64) or 16 (D = 128)
  constexpr int kRowsPerWarp = 32 / kLanesPerRow;
  grid_dep_wait();                                         // O comes from the stream's previous kernel
  grid_dep_release();
  const int lane = threadIdx.x & 31;
  const long long warp_id = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long rows = static_cast<long long>(p.B) * p.T * p.H;     // rows index [B,T,H]
  const long long row = warp_id * kRowsPerWarp + lane / kLanesPerRow;
  float part = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(dout + row * D + 8 * (lane % kLanesPerRow));
    const uint4 b = *reinterpret_cast<const uint4*>(o + row * D + 8 * (lane % kLanesPerRow));
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      T a2[2], b2[2];
      *reinterpret_cast<uint32_t*>(a2) = aw[i];
      *reinterpret_cast<uint32_t*>(b2) = bw[i];
      part = fmaf(to_f32(a2[0]), to_f32(b2[0]), part);
      part = fmaf(to_f32(a2[1]), to_f32(b2[1]), part);
    }
  }
#pragma unroll
  for (int off = kLanesPerRow / 2; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if (row < rows && (lane % kLanesPerRow) == 0) {
    const int h = static_cast<int>(row % p.H);
    const long long bt = row / p.H;
    const int t = static_cast<int>(bt % p.T);
    const int b = static_cast<int>(bt / p.T);
    delta[(static_cast<long long>(b) * p.H + h) * p.T + t] = part;
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dq_simt_kernel(Problem p, const T* __restrict__ dout, const T* __restrict__ q,
               const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ lse,
               const float* __restrict__ delta, T* __restrict__ dq) {
  constexpr int R = D / 32;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long rows = static_cast<long long>(p.B) * p.H * p.T;
  if (row >= rows) return;
  const int t = static_cast<int>(row % p.T);
  const long long bh = row / p.T;
  const int h = static_cast<int>(bh % p.H);
  const int b = static_cast<int>(bh / p.H);
  const int hk = h / (p.H / p.Hkv);
  const float scale2 = p.scale * kLog2e;

  const long long qoff = ((static_cast<long long>(b) * p.T + t) * p.H + h) * D;
  float qr[R], dor[R], acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    qr[r] = to_f32(q[qoff + lane + 32 * r]);
    dor[r] = to_f32(dout[qoff + lane + 32 * r]);
    acc[r] = 0.f;
  }
  const float l2 = lse[bh * p.T + t] * kLog2e;
  const float dl = delta[bh * p.T + t];

  int lo = 0, nsink = 0;
  if (p.window > 0) {
    const int first = t - (p.window - p.sinks) + 1;
    lo = first > 0 ? first : 0;
    nsink = p.sinks < lo ? p.sinks : lo;
  }
  const long long kv_stride = static_cast<long long>(p.Hkv) * D;
  const T* kbase = k + (static_cast<long long>(b) * p.T * p.Hkv + hk) * D;
  const T* vbase = v + (static_cast<long long>(b) * p.T * p.Hkv + hk) * D;
  int t_last = last_key_of_query(t, p.block);            // block-causal: to the end of the row's block
  t_last = t_last < p.T - 1 ? t_last : p.T - 1;
  const int n = nsink + (t_last - lo + 1);
  for (int idx = 0; idx < n; ++idx) {
    const int j = idx < nsink ? idx : lo + (idx - nsink);
    const T* krow = kbase + j * kv_stride;
    const T* vrow = vbase + j * kv_stride;
    float kr[R];
    float ps = 0.f, pd = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      kr[r] = to_f32(krow[lane + 32 * r]);
      ps = fmaf(qr[r], kr[r], ps);
      pd = fmaf(dor[r], to_f32(vrow[lane + 32 * r]), pd);
    }
    const float s = warp_sum(ps);
    const float dp = warp_sum(pd);
    const float pj = exp2f(fmaf(s, scale2, -l2));
    const float ds = pj * (dp - dl) * p.scale;
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = fmaf(ds, kr[r], acc[r]);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) dq[qoff + lane + 32 * r] = from_f32<T>(acc[r]);
}

template <typename T, int D>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dkv_simt_kernel(Problem p, const T* __restrict__ dout, const T* __restrict__ q,
                const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ lse,
                const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv) {
  constexpr int R = D / 32;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long rows = static_cast<long long>(p.B) * p.Hkv * p.T;
  if (row >= rows) return;
  const int j = static_cast<int>(row % p.T);               // key position
  const long long bhk = row / p.T;
  const int hk = static_cast<int>(bhk % p.Hkv);
  const int b = static_cast<int>(bhk / p.Hkv);
  const int group = p.H / p.Hkv;
  const float scale2 = p.scale * kLog2e;

  const long long koff = ((static_cast<long long>(b) * p.T + j) * p.Hkv + hk) * D;
  float kr[R], vr[R], acck[R], accv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    kr[r] = to_f32(k[koff + lane + 32 * r]);
    vr[r] = to_f32(v[koff + lane + 32 * r]);
    acck[r] = 0.f;
    accv[r] = 0.f;
  }
  // queries that see key j: i >= j, and inside the window unless j is a sink
  int last = p.T - 1;
  if (p.window > 0 && j >= p.sinks) {
    const int w_last = j + (p.window - p.sinks) - 1;
    last = w_last < last ? w_last : last;
  }
  for (int g = 0; g < group; ++g) {
    const int h = hk * group + g;
    const long long bh = static_cast<long long>(b) * p.H + h;
    for (int i = first_query_of_key(j, p.block); i <= last; ++i) {
      const long long qoff = ((static_cast<long long>(b) * p.T + i) * p.H + h) * D;
      float qr[R], dor[R];
      float ps = 0.f, pd = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        qr[r] = to_f32(q[qoff + lane + 32 * r]);
        dor[r] = to_f32(dout[qoff + lane + 32 * r]);
        ps = fmaf(qr[r], kr[r], ps);
        pd = fmaf(dor[r], vr[r], pd);
      }
      const float s = warp_sum(ps);
      const float dp = warp_sum(pd);
      const float pj = exp2f(fmaf(s, scale2, -lse[bh * p.T + i] * kLog2e));
      const float ds = pj * (dp - delta[bh * p.T + i]) * p.scale;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acck[r] = fmaf(ds, qr[r], acck[r]);
        accv[r] = fmaf(pj, dor[r], accv[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    dk[koff + lane + 32 * r] = from_f32<T>(acck[r]);
    dv[koff + lane + 32 * r] = from_f32<T>(accv[r]);
  }
}

inline unsigned blocks_for(long long rows) {
  return static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
}

template <typename T, int D>
int fwd_t(const Problem& p, const void* q, const void* k, const void* v, void* o, float* lse,
          cudaStream_t s) {
  const long long rows = static_cast<long long>(p.B) * p.H * p.T;
  fwd_simt_kernel<T, D><<<blocks_for(rows), kWarpsPerBlock * 32, 0, s>>>(
      p, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
      static_cast<T*>(o), lse);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename T, int D>
int delta_t(const Problem& p, const void* dout, const void* o, float* delta, cudaStream_t s) {
  const long long rows = static_cast<long long>(p.B) * p.H * p.T;
  if constexpr (sizeof(T) == 2 && (D == 64 || D == 128)) {
    constexpr int kRowsPerBlock = 8 * (32 / (D / 8));           // 8 warps per block
    const unsigned blocks = static_cast<unsigned>((rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (launch_kernel(delta_vec_kernel<T, D>, dim3(blocks), dim3(256), 0, s, overlap_launches(kOverlapDelta), p,
                      static_cast<const T*>(dout), static_cast<const T*>(o), delta) != cudaSuccess) {
      (void)cudaGetLastError();
      return NLFA_ERR_CUDA;
    }
  } else {
    delta_kernel<T, D><<<blocks_for(rows), kWarpsPerBlock * 32, 0, s>>>(
        p, static_cast<const T*>(dout), static_cast<const T*>(o), delta);
  }
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename T, int D>
int bwd_t(const Problem& p, const void* dout, const void* q, const void* k, const void* v,
          const float* lse, void* dq, void* dk, void* dv, const float* delta, int passes,
          cudaStream_t s) {
  const long long qrows = static_cast<long long>(p.B) * p.H * p.T;
  const long long krows = static_cast<long long>(p.B) * p.Hkv * p.T;
  if (passes & NLFA_PASS_DQ)
    dq_simt_kernel<T, D><<<blocks_for(qrows), kWarpsPerBlock * 32, 0, s>>>(
        p, static_cast<const T*>(dout), static_cast<const T*>(q), static_cast<const T*>(k),
        static_cast<const T*>(v), lse, delta, static_cast<T*>(dq));
  if (cudaGetLastError() != cudaSuccess) return NLFA_ERR_CUDA;
  if (passes & NLFA_PASS_DKV)
    dkv_simt_kernel<T, D><<<blocks_for(krows), kWarpsPerBlock * 32, 0, s>>>(
        p, static_cast<const T*>(dout), static_cast<const T*>(q), static_cast<const T*>(k),
        static_cast<const T*>(v), lse, delta, static_cast<T*>(dk), static_cast<T*>(dv));
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

#define NLFA_DISPATCH(p, CALL)                                                        \
  do {                                                                                \
    switch ((p).dtype) {                                                              \
      case NLFA_DTYPE_F32:                                                            \
        switch ((p).D) {                                                              \
          case 32: return CALL(float, 32);                                            \
          case 64: return CALL(float, 64);                                            \
          case 128: return CALL(float, 128);                                          \
        }                                                                             \
        return NLFA_ERR_BAD_HEAD_DIM;                                                 \
      case NLFA_DTYPE_F16:                                                            \
        switch ((p).D) {                                                              \
          case 32: return CALL(__half, 32);                                           \
          case 64: return CALL(__half, 64);                                           \
          case 128: return CALL(__half, 128);                                         \
        }                                                                             \
        return NLFA_ERR_BAD_HEAD_DIM;                                                 \
      case NLFA_DTYPE_BF16:                                                           \
        switch ((p).D) {                                                              \
          case 32: return CALL(__nv_bfloat16, 32);                                    \
          case 64: return CALL(__nv_bfloat16, 64);                                    \
          case 128: return CALL(__nv_bfloat16, 128);                                  \
        }                                                                             \
        return NLFA_ERR_BAD_HEAD_DIM;                                                 \
    }                                                                                 \
    return NLFA_ERR_BAD_DTYPE;                                                        \
  } while (0)

}  // namespace

int launch_fwd_simt(const Problem& p, const void* q, const void* k, const void* v, void* o,
                    float* lse, cudaStream_t stream) {
#define CALL(T, DD) fwd_t<T, DD>(p, q, k, v, o, lse, stream)
  NLFA_DISPATCH(p, CALL);
#undef CALL
}

int launch_delta(const Problem& p, const void* dout, const void* o, float* delta,
                 cudaStream_t stream) {
#define CALL(T, DD) delta_t<T, DD>(p, dout, o, delta, stream)
  NLFA_DISPATCH(p, CALL);
#undef CALL
}

int launch_bwd_simt(const Problem& p, const void* dout, const void* q, const void* k,
                    const void* v, const void* o, const float* lse, void* dq, void* dk, void* dv,
                    float* delta, int passes, cudaStream_t stream) {
  if (passes & NLFA_PASS_DELTA) {
    int st = launch_delta(p, dout, o, delta, stream);
    if (st != NLFA_OK) return st;
  }
#define CALL(T, DD) bwd_t<T, DD>(p, dout, q, k, v, lse, dq, dk, dv, delta, passes, stream)
  NLFA_DISPATCH(p, CALL);
#undef CALL
}

}  // namespace nlfa
