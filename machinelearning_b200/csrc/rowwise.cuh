// Element access and small reductions shared by the elementwise kernels that sit either side of the
// attention core (the q/k prologue and the value-blend / gate epilogue).  A lane owns 8 consecutive
// elements: one 16-byte load for 16-bit types, two for float32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace nlfa {
namespace rowwise {

constexpr int kVec = 8;
constexpr int kThreads = 256;
constexpr int kMaxPartials = 148 * 8;   // CTAs of the backward; rows of the weight-gradient scratch

// Raw: the 8 elements as loaded (kept packed so that several rows can be in flight in few registers).
struct Raw32 { float4 a, b; };
template <typename T> struct Elem;
template <> struct Elem<float> {
  using Raw = Raw32;
  static constexpr int kInFlight = 2;
  __device__ static Raw zero() { return Raw{make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)}; }
  __device__ static Raw load_raw(const float* p) {
    return Raw{*reinterpret_cast<const float4*>(p), *reinterpret_cast<const float4*>(p + 4)};
  }
  __device__ static void unpack(const Raw& r, float (&v)[kVec]) {
    v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w; v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
  }
  __device__ static void load(const float* p, float (&v)[kVec]) { unpack(load_raw(p), v); }
  __device__ static void store(float* p, const float (&v)[kVec]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  __device__ static float round(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  using Raw = uint4;
  static constexpr int kInFlight = 4;
  __device__ static Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ static Raw load_raw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static void load(const __nv_bfloat16* p, float (&v)[kVec]) { unpack(load_raw(p), v); }
  __device__ static void unpack(const Raw& raw, float (&v)[kVec]) {
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
  using Raw = uint4;
  static constexpr int kInFlight = 4;
  __device__ static Raw zero() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ static Raw load_raw(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
  __device__ static void load(const __half* p, float (&v)[kVec]) { unpack(load_raw(p), v); }
  __device__ static void unpack(const Raw& raw, float (&v)[kVec]) {
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


inline bool dtype_ok(int d) { return d == NLFA_DTYPE_F32 || d == NLFA_DTYPE_F16 || d == NLFA_DTYPE_BF16; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace rowwise
}  // namespace nlfa
