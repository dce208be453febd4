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
// dozen tokens.  A CTA owns a few query rows of one (batch, KV head) -- the rows of every query head
// of the group, so K and V are fetched once for all of them -- and walks the keys in tiles of 32
// that the whole CTA copies into shared memory with coalesced 16-byte loads.  Inside a tile a
// warp's lanes split the keys: a lane forms the whole dot product of its key (the query rows sit
// in shared memory and are read as broadcasts) and keeps its own partial of the output row; the
// running maximum of a row is shared through one warp reduction per tile and the lanes' partial
// rows are added once at the end.  Tiles no row of the CTA can see are skipped without being
// read.  fp32 arithmetic throughout, no atomics.
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

template <int D> __host__ __device__ constexpr int rows_per_warp() { return D <= 64 ? 2 : 1; }

template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32)
fwd_cached_kernel(CachedParams p, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                  T* __restrict__ o, float* __restrict__ lse) {
  constexpr int RPW = rows_per_warp<D>();                  // query rows per warp
  constexpr int RPC = kWarps * RPW;                        // ... per CTA
  constexpr int kRowBytes = D * static_cast<int>(sizeof(T));
  constexpr int kPitch = kRowBytes + 16;                   // padded: a lane's 16-byte reads of its own row do not collide
  constexpr int kChunksPerRow = kRowBytes / 16, kChunks = 32 * kChunksPerRow;
  __shared__ __align__(16) unsigned char ks[32 * kPitch];
  __shared__ __align__(16) unsigned char vs[32 * kPitch];
  __shared__ __align__(16) float qs[RPC][D];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const int G = p.H / p.Hkv;
  const int head_rows = p.Tq * G;                          // query rows that share this KV head: (t, g)
  const int chunks = (head_rows + RPC - 1) / RPC;
  const int chunk = blockIdx.x % chunks;
  const int bh = blockIdx.x / chunks;
  const int hk = bh % p.Hkv, b = bh / p.Hkv;
  const float scale2 = p.scale * kLog2e;

  int qp[RPW], lo[RPW];
  long long orow[RPW];                                     // row of q / o in [B,Tq,H]; -1: no such row
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = chunk * RPC + wi * RPW + i;
    orow[i] = -1;
    qp[i] = lo[i] = 0;
    if (r < head_rows) {
      const int t = r / G, h = hk * G + r % G;
      orow[i] = (static_cast<long long>(b) * p.Tq + t) * p.H + h;
      qp[i] = p.qpos ? p.qpos[t] : p.L - p.Tq + t;
      lo[i] = qp[i] - (p.window - p.sinks);                // window: keys above lo, or below sinks
      for (int d = lane; d < D; d += 32) qs[wi * RPW + i][d] = static_cast<float>(q[orow[i] * D + d]) * scale2;
    }
  }
  __syncwarp();

  const unsigned char* kb = reinterpret_cast<const unsigned char*>(k + (static_cast<long long>(b) * p.Hkv + hk) * p.L * D);
  const unsigned char* vb = reinterpret_cast<const unsigned char*>(v + (static_cast<long long>(b) * p.Hkv + hk) * p.L * D);
  float acc[RPW][D];
  float m[RPW], l[RPW];                                    // m: shared by the warp; l: this lane's keys
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) acc[i][d] = 0.f;
  }
  // Which rows of this warp see key j0 + lane; `any`: some row does.
  auto visible = [&](int j0, bool (&see)[RPW]) -> bool {
    const int j = j0 + lane;
    const int kp = j < p.L ? (p.kpos ? p.kpos[j] : j) : 0;
    bool any = false;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      see[i] = j < p.L && orow[i] >= 0;
      if (see[i]) {
        if (p.window > 0) see[i] = kp <= qp[i] && (kp > lo[i] || kp < p.sinks);
        else if (p.causal) see[i] = kp <= qp[i];
      }
      any |= see[i];
    }
    return any;
  };
  // A thread's share of a tile: kPer 16-byte chunks of K and of V, fetched into registers one tile
  // ahead (while the current tile is being used) when that is few enough registers.
  constexpr int kPer = kChunks / (kWarps * 32);
  constexpr bool kAhead = kPer <= 4;
  uint4 nk[kAhead ? kPer : 1], nv[kAhead ? kPer : 1];
  auto fetch = [&](int j0) {
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int c = threadIdx.x + u * kWarps * 32;
      const int r = c / kChunksPerRow, cc = c % kChunksPerRow;
      if (j0 + r < p.L) {
        const long long src = static_cast<long long>(j0 + r) * kRowBytes + cc * 16;
        if constexpr (kAhead) {
          nk[u] = *reinterpret_cast<const uint4*>(kb + src);
          nv[u] = *reinterpret_cast<const uint4*>(vb + src);
        } else {
          *reinterpret_cast<uint4*>(ks + r * kPitch + cc * 16) = *reinterpret_cast<const uint4*>(kb + src);
          *reinterpret_cast<uint4*>(vs + r * kPitch + cc * 16) = *reinterpret_cast<const uint4*>(vb + src);
        }
      }
    }
  };
  auto stage = [&]() {                                     // registers -> shared memory (kAhead only)
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
      const int c = threadIdx.x + u * kWarps * 32;
      const int r = c / kChunksPerRow, cc = c % kChunksPerRow;
      *reinterpret_cast<uint4*>(ks + r * kPitch + cc * 16) = nk[u];
      *reinterpret_cast<uint4*>(vs + r * kPitch + cc * 16) = nv[u];
    }
  };
  bool see[RPW];
  bool cur = __syncthreads_or(visible(0, see)) != 0;       // every thread of the CTA votes on every tile
  if (kAhead && cur) fetch(0);
  for (int j0 = 0; j0 < p.L; j0 += 32) {
    bool see_next[RPW];
    const bool nxt = j0 + 32 < p.L && __syncthreads_or(visible(j0 + 32, see_next)) != 0;
    if (cur) {
      if constexpr (kAhead) stage(); else fetch(j0);
      __syncthreads();
    }
    if (kAhead && nxt) fetch(j0 + 32);                     // in flight while this tile is used
    if (!cur) {
      cur = nxt;
#pragma unroll
      for (int i = 0; i < RPW; ++i) see[i] = see_next[i];
      continue;
    }
    const T* kr = reinterpret_cast<const T*>(ks + lane * kPitch);
    const T* vr = reinterpret_cast<const T*>(vs + lane * kPitch);
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      if (!__any_sync(0xffffffffu, see[i])) continue;
      const float* qrow = qs[wi * RPW + i];
      float s = -INFINITY;
      if (see[i]) {
        float dot[8];                                      // eight independent chains: the sum is latency bound otherwise
#pragma unroll
        for (int e = 0; e < 8; ++e) dot[e] = 0.f;
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          float x[8];
          Elem<T>::load(kr + c, x);
          const float4 qa = *reinterpret_cast<const float4*>(qrow + c), qb = *reinterpret_cast<const float4*>(qrow + c + 4);
          dot[0] = fmaf(qa.x, x[0], dot[0]); dot[1] = fmaf(qa.y, x[1], dot[1]);
          dot[2] = fmaf(qa.z, x[2], dot[2]); dot[3] = fmaf(qa.w, x[3], dot[3]);
          dot[4] = fmaf(qb.x, x[4], dot[4]); dot[5] = fmaf(qb.y, x[5], dot[5]);
          dot[6] = fmaf(qb.z, x[6], dot[6]); dot[7] = fmaf(qb.w, x[7], dot[7]);
        }
        s = ((dot[0] + dot[1]) + (dot[2] + dot[3])) + ((dot[4] + dot[5]) + (dot[6] + dot[7]));
      }
      float mx = s;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m[i], mx);                 // finite: some lane sees a key
      const float alpha = exp2f(m[i] - m_new);             // first tile: exp2(-inf) = 0
      const float pj = see[i] ? exp2f(s - m_new) : 0.f;
      l[i] = fmaf(l[i], alpha, pj);
      m[i] = m_new;
      if (see[i]) {
#pragma unroll
        for (int c = 0; c < D; c += 8) {
          float x[8];
          Elem<T>::load(vr + c, x);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][c + e] = fmaf(acc[i][c + e], alpha, pj * x[e]);
        }
      } else if (alpha != 1.f) {
#pragma unroll
        for (int d = 0; d < D; ++d) acc[i][d] *= alpha;
      }
    }
    __syncthreads();                                       // the tile may be overwritten
    cur = nxt;
#pragma unroll
    for (int i = 0; i < RPW; ++i) see[i] = see_next[i];
  }
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    float lsum = l[i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;       // a row that sees no key gives zeros
    // add the lanes' partial rows: after the butterfly every lane holds every sum; lane d % 32 keeps d
    float* stage = qs[wi * RPW + i];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      float x = acc[i][d];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
      if (lane == (d & 31)) stage[d] = x * inv;
    }
    __syncwarp();
    if (orow[i] >= 0) {
      for (int d = lane; d < D; d += 32) o[orow[i] * D + d] = static_cast<T>(stage[d]);
      if (lse && lane == 0) {
        const long long t = (orow[i] / p.H) % p.Tq, h = orow[i] % p.H;
        lse[(static_cast<long long>(b) * p.H + h) * p.Tq + t] = lsum > 0.f ? (m[i] + log2f(lsum)) * kLn2 : -INFINITY;
      }
    }
  }
}

template <typename T>
int launch_for_dim(const CachedParams& p, int D, const void* q, const void* k, const void* v, void* o, float* lse,
                   cudaStream_t st) {
  const long long head_rows = static_cast<long long>(p.Tq) * (p.H / p.Hkv);
#define NLFA_GO(DD)                                                                                      \
  do {                                                                                                   \
    constexpr int rpc = kWarps * rows_per_warp<DD>();                                                    \
    const long long grid = static_cast<long long>(p.B) * p.Hkv * ((head_rows + rpc - 1) / rpc);          \
    if (grid >= (1ll << 31)) return NLFA_ERR_BAD_SHAPE;                                                  \
    fwd_cached_kernel<T, DD><<<static_cast<unsigned>(grid), kWarps * 32, 0, st>>>(                        \
        p, (const T*)q, (const T*)k, (const T*)v, (T*)o, lse);                                           \
  } while (0)
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
