// Forward attention of an active block of queries over [cache | block], masked by absolute
// positions: the attention core of nanolab's KV-cached block forward
// (nanolab/mixers.py:372-467, `Attention.forward_cached`), which nanolab runs as a
// `torch.cat`, a `repeat_interleave` and a masked SDPA per layer.
//
//   q [B,Tq,H,D]; k, v [B,Hkv,L,D] (nanolab's cache layout, the block's own keys last);
//   qpos [Tq], kpos [L]: absolute positions.  After window eviction the cached keys'
//   positions are no longer contiguous, so positions, not offsets, define the mask:
//     window > 0 : kpos <= qpos and (kpos > qpos - (window - sinks) or kpos < sinks)
//     causal     : kpos <= qpos              (full to the cache, lower-triangular in the block)
//     neither    : every key                 (block diffusion: a bidirectional block)
//
// Forward only (the cached path is inference).  A decode-sized problem: Tq is a block of a few
// dozen tokens.  One warp owns one query row and its lanes split the KEYS: a lane takes key
// j0 + lane of each group of 32, forms the whole dot product from its own 16-byte loads of that
// key row (the query row sits in shared memory, read as broadcasts), and keeps its own partial
// of the output row; the running maximum is shared through one warp reduction per 32 keys and
// the lanes' partial rows are added once at the end.  Groups of 32 keys no lane can see are
// skipped without being read.  fp32 arithmetic throughout, no atomics.
#include "rowwise.cuh"

namespace nlfa {
namespace {

using rowwise::Elem;
constexpr int kWarps = 4;

struct CachedParams {
  int B, Tq, H, Hkv, L;
  int causal, window, sinks;
  float scale;
  const int* qpos;   // nullptr: the block is the last Tq positions of a contiguous [0, L)
  const int* kpos;   // nullptr: contiguous
};

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32)
fwd_cached_kernel(CachedParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  T* __restrict__ o, float* __restrict__ lse) {
  __shared__ float qs[kWarps][D];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + wi;                    // over [B,Tq,H]
  const long long rows = static_cast<long long>(p.B) * p.Tq * p.H;
  if (row >= rows) return;                                 // whole warps leave; no block-wide barrier below
  const int h = static_cast<int>(row % p.H);
  const long long bt = row / p.H;
  const int t = static_cast<int>(bt % p.Tq);
  const int b = static_cast<int>(bt / p.Tq);
  const int hk = h / (p.H / p.Hkv);
  const int qp = p.qpos ? p.qpos[t] : p.L - p.Tq + t;
  const int lo = qp - (p.window - p.sinks);                // window: keys above lo, or below sinks
  const float scale2 = p.scale * kLog2e;
  for (int d = lane; d < D; d += 32) qs[wi][d] = static_cast<float>(q[row * D + d]) * scale2;
  __syncwarp();

  const T* kb = k + (static_cast<long long>(b) * p.Hkv + hk) * p.L * D;
  const T* vb = v + (static_cast<long long>(b) * p.Hkv + hk) * p.L * D;
  float acc[D];
#pragma unroll
  for (int d = 0; d < D; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;                            // m: shared by the warp; l: this lane's keys
  for (int j0 = 0; j0 < p.L; j0 += 32) {
    const int j = j0 + lane;
    bool see = j < p.L;
    if (see) {
      const int kp = p.kpos ? p.kpos[j] : j;
      if (p.window > 0) see = kp <= qp && (kp > lo || kp < p.sinks);
      else if (p.causal) see = kp <= qp;
    }
    if (!__any_sync(0xffffffffu, see)) continue;
    float s = -INFINITY;
    if (see) {
      const T* kr = kb + static_cast<long long>(j) * D;
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        float x[8];
        Elem<T>::load(kr + c, x);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          d0 = fmaf(qs[wi][c + i], x[i], d0);
          d1 = fmaf(qs[wi][c + i + 1], x[i + 1], d1);
        }
      }
      s = d0 + d1;
    }
    float mx = s;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m, mx);                      // finite: some lane sees a key
    const float alpha = exp2f(m - m_new);                  // first group: exp2(-inf) = 0
    const float pj = see ? exp2f(s - m_new) : 0.f;
    l = fmaf(l, alpha, pj);
    m = m_new;
    if (see) {
      const T* vr = vb + static_cast<long long>(j) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        float x[8];
        Elem<T>::load(vr + c, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c + i] = fmaf(acc[c + i], alpha, pj * x[i]);
      }
    } else if (alpha != 1.f) {
#pragma unroll
      for (int d = 0; d < D; ++d) acc[d] *= alpha;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
  const float inv = l > 0.f ? 1.f / l : 0.f;               // a row that sees no key gives zeros
  // add the lanes' partial rows: after the butterfly every lane holds every sum; lane d % 32 writes d
#pragma unroll
  for (int d = 0; d < D; ++d) {
    float x = acc[d];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    if (lane == (d & 31)) qs[wi][d] = x * inv;
  }
  __syncwarp();
  for (int d = lane; d < D; d += 32) o[row * D + d] = static_cast<T>(qs[wi][d]);
  if (lse && lane == 0)
    lse[(static_cast<long long>(b) * p.H + h) * p.Tq + t] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
}

template <typename T>
int launch_for_dim(const CachedParams& p, int D, const void* q, const void* k, const void* v, void* o, float* lse,
                   cudaStream_t st) {
  const long long rows = static_cast<long long>(p.B) * p.Tq * p.H;
  const unsigned grid = static_cast<unsigned>((rows + kWarps - 1) / kWarps);
#define NLFA_GO(DD)                                                                                      \
  fwd_cached_kernel<T, DD><<<grid, kWarps * 32, 0, st>>>(p, (const T*)q, (const T*)k, (const T*)v, (T*)o, lse)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace
}  // namespace nlfa

extern "C" int nlfa_fwd_cached(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                               const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                               float scale, int causal, int window, int sinks, int dtype, void* stream) {
  using namespace nlfa;
  if (B < 0 || Tq < 0 || H < 0 || L < 0 || Hkv <= 0 || H % Hkv != 0 || !(scale == scale)) return NLFA_ERR_BAD_SHAPE;
  if (D != 32 && D != 64 && D != 128) return NLFA_ERR_BAD_HEAD_DIM;
  if (dtype != NLFA_DTYPE_F32 && dtype != NLFA_DTYPE_F16 && dtype != NLFA_DTYPE_BF16) return NLFA_ERR_BAD_DTYPE;
  if (window < 0 || sinks < 0 || (window == 0 && sinks != 0) || (window > 0 && sinks >= window))
    return NLFA_ERR_BAD_WINDOW;
  if (window > 0 && !causal) return NLFA_ERR_BAD_WINDOW;           // a window is defined on distance to the query
  if (qpos == nullptr && Tq > L) return NLFA_ERR_BAD_SHAPE;
  const long long rows = static_cast<long long>(B) * Tq * H;
  if (rows == 0) return NLFA_OK;
  if (rows / 4 >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;
  if (!q || !o || (L > 0 && (!k_cache || !v_cache))) return NLFA_ERR_NULL_POINTER;
  CachedParams p{B, Tq, H, Hkv, L, causal ? 1 : 0, window, sinks, scale, qpos, kpos};
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == NLFA_DTYPE_BF16) return launch_for_dim<__nv_bfloat16>(p, D, q, k_cache, v_cache, o, lse, st);
  if (dtype == NLFA_DTYPE_F16) return launch_for_dim<__half>(p, D, q, k_cache, v_cache, o, lse, st);
  return launch_for_dim<float>(p, D, q, k_cache, v_cache, o, lse, st);
}
