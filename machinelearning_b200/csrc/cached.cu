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
  int splits;        // > 1: blockIdx.y walks its share of the key tiles and leaves a partial result
  int tiles_per_split;
  float* part_o;     // [rows][splits][D]: each split's own normalised output row
  float* part_l;     // [rows][splits]: its base-2 logsumexp (-inf: the split saw no key)
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
  const int j_begin = static_cast<int>(blockIdx.y) * p.tiles_per_split * 32;        // this CTA's keys
  const int j_stop = j_begin + p.tiles_per_split * 32;
  const int j_end = j_stop < p.L ? j_stop : p.L;

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
    const int kp = j < j_end ? (p.kpos ? p.kpos[j] : j) : 0;
    bool any = false;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      see[i] = j < j_end && orow[i] >= 0;
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
      if (j0 + r < j_end) {
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
  bool cur = __syncthreads_or(visible(j_begin, see)) != 0;  // every thread of the CTA votes on every tile
  if (kAhead && cur) fetch(j_begin);
  for (int j0 = j_begin; j0 < j_end; j0 += 32) {
    bool see_next[RPW];
    const bool nxt = j0 + 32 < j_end && __syncthreads_or(visible(j0 + 32, see_next)) != 0;
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
    float* out_row = qs[wi * RPW + i];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      float x = acc[i][d];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
      if (lane == (d & 31)) out_row[d] = x * inv;
    }
    __syncwarp();
    if (orow[i] >= 0 && p.splits > 1) {                    // partial result; merge_splits_kernel finishes the row
      const long long slot = orow[i] * p.splits + blockIdx.y;
      for (int d = lane; d < D; d += 32) p.part_o[slot * D + d] = out_row[d];
      if (lane == 0) p.part_l[slot] = lsum > 0.f ? m[i] + log2f(lsum) : -INFINITY;
    } else if (orow[i] >= 0) {
      for (int d = lane; d < D; d += 32) o[orow[i] * D + d] = static_cast<T>(out_row[d]);
      if (lse && lane == 0) {
        const long long t = (orow[i] / p.H) % p.Tq, h = orow[i] % p.H;
        lse[(static_cast<long long>(b) * p.H + h) * p.Tq + t] = lsum > 0.f ? (m[i] + log2f(lsum)) * kLn2 : -INFINITY;
      }
    }
  }
}

// One warp per query row: the splits' partial rows, each normalised by its own sum, are combined with the
// weights 2^(lse_s - max lse), in a fixed order.
template <typename T, int D>
__global__ void __launch_bounds__(kWarps * 32)
merge_splits_kernel(CachedParams p, T* __restrict__ o, float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);    // over [B,Tq,H]
  if (row >= static_cast<long long>(p.B) * p.Tq * p.H) return;
  const float* pl = p.part_l + row * p.splits;
  float mx = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, pl[s]);
  float wsum = 0.f;
  for (int s = 0; s < p.splits; ++s) wsum += mx > -INFINITY ? exp2f(pl[s] - mx) : 0.f;
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int s = 0; s < p.splits; ++s)
      if (pl[s] > -INFINITY) acc = fmaf(exp2f(pl[s] - mx), p.part_o[(row * p.splits + s) * D + d], acc);
    o[row * D + d] = static_cast<T>(acc * inv);
  }
  if (lse && lane == 0) {
    const long long t = (row / p.H) % p.Tq, h = row % p.H, b = row / (static_cast<long long>(p.H) * p.Tq);
    lse[(b * p.H + h) * p.Tq + t] = wsum > 0.f ? (mx + log2f(wsum)) * kLn2 : -INFINITY;
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
    fwd_cached_kernel<T, DD><<<dim3(static_cast<unsigned>(grid), p.splits), kWarps * 32, 0, st>>>(        \
        p, (const T*)q, (const T*)k, (const T*)v, (T*)o, lse);                                           \
    if (p.splits > 1) {                                                                                  \
      const long long rows = static_cast<long long>(p.B) * p.Tq * p.H;                                   \
      merge_splits_kernel<T, DD><<<static_cast<unsigned>((rows + kWarps - 1) / kWarps), kWarps * 32, 0, st>>>( \
          p, (T*)o, lse);                                                                                \
    }                                                                                                    \
  } while (0)
  if (D == 32) NLFA_GO(32); else if (D == 64) NLFA_GO(64); else NLFA_GO(128);
#undef NLFA_GO
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

// How many ways the keys are split: only when the row chunks alone leave most SMs idle.
int choose_splits(int B, int Tq, int H, int Hkv, int L, int D) {
  const long long rpc = kWarps * (D <= 64 ? 2 : 1);
  const long long base = static_cast<long long>(B) * Hkv * ((static_cast<long long>(Tq) * (H / Hkv) + rpc - 1) / rpc);
  const long long tiles = (L + 31) / 32;
  if (base <= 0 || base >= 296 || tiles < 8) return 1;
  long long s = (592 + base - 1) / base;
  if (s > tiles / 4) s = tiles / 4;
  if (s > 32) s = 32;
  return s < 1 ? 1 : static_cast<int>(s);
}

template <typename T>
int merge_for_dim(const CachedParams& p, int D, void* o, float* lse, cudaStream_t st) {
  const long long rows = static_cast<long long>(p.B) * p.Tq * p.H;
  const unsigned grid = static_cast<unsigned>((rows + kWarps - 1) / kWarps);
  if (D == 32) merge_splits_kernel<T, 32><<<grid, kWarps * 32, 0, st>>>(p, (T*)o, lse);
  else if (D == 64) merge_splits_kernel<T, 64><<<grid, kWarps * 32, 0, st>>>(p, (T*)o, lse);
  else merge_splits_kernel<T, 128><<<grid, kWarps * 32, 0, st>>>(p, (T*)o, lse);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

size_t split_scratch_bytes(int B, int Tq, int H, int D, int s) {
  return s <= 1 ? 0 : static_cast<size_t>(B) * Tq * H * s * (static_cast<size_t>(D) + 1) * sizeof(float);
}

}  // namespace

// tensor-core form (cached_tc.cu)
bool cached_tc_applies(int Tq, int H, int Hkv, int L, int D, int dtype);
int cached_tc_splits(int B, int Tq, int H, int Hkv, int L);
int launch_fwd_cached_tc(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                         const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                         float scale, int causal, int window, int sinks, int dtype, float* part_o,
                         float* part_l, int splits, unsigned* status, cudaStream_t stream);
unsigned* status_block();      // api.cu

}  // namespace nlfa

extern "C" size_t nlfa_fwd_cached_scratch_bytes(int B, int Tq, int H, int Hkv, int L, int D) {
  if (B <= 0 || Tq <= 0 || H <= 0 || Hkv <= 0 || L <= 0 || H % Hkv != 0) return 0;
  // the larger of what the two kernel families would split into (the family is chosen per call)
  const size_t simt = nlfa::split_scratch_bytes(B, Tq, H, D, nlfa::choose_splits(B, Tq, H, Hkv, L, D));
  const size_t tc = H / Hkv <= 128 ? nlfa::split_scratch_bytes(B, Tq, H, D, nlfa::cached_tc_splits(B, Tq, H, Hkv, L)) : 0;
  return simt > tc ? simt : tc;
}

extern "C" int nlfa_fwd_cached(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                               const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                               float scale, int causal, int window, int sinks, int dtype, void* scratch,
                               size_t scratch_bytes, void* stream) {
  return nlfa_fwd_cached_path(q, k_cache, v_cache, o, lse, qpos, kpos, B, Tq, H, Hkv, L, D, scale, causal, window,
                              sinks, dtype, NLFA_PATH_AUTO, scratch, scratch_bytes, stream);
}

extern "C" int nlfa_fwd_cached_path(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                                    const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                                    float scale, int causal, int window, int sinks, int dtype, int path,
                                    void* scratch, size_t scratch_bytes, void* stream) {
  using namespace nlfa;
  if (path != NLFA_PATH_AUTO && path != NLFA_PATH_SIMT && path != NLFA_PATH_TENSOR) return NLFA_ERR_UNSUPPORTED_PATH;
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
  CachedParams p{B, Tq, H, Hkv, L, causal ? 1 : 0, window, sinks, scale, qpos, kpos, 1, (L + 31) / 32, nullptr, nullptr};
  cudaStream_t st = (cudaStream_t)stream;
  const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
                         reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(o)) & 15u) == 0;
  if (path != NLFA_PATH_SIMT && aligned && scale > 0.f && nlfa_device_supported() &&
      cached_tc_applies(Tq, H, Hkv, L, D, dtype)) {
    // blocks of a few dozen rows and more over a long cache: the products run on the tensor cores
    if (nlfa_peek_status() != NLFA_OK) return NLFA_ERR_DEVICE_TIMEOUT;
    unsigned* status = status_block();
    if (!status) return NLFA_ERR_CUDA;
    int splits = cached_tc_splits(B, Tq, H, Hkv, L);
    if (split_scratch_bytes(B, Tq, H, D, splits) > (scratch ? scratch_bytes : 0)) splits = 1;
    float* part_o = static_cast<float*>(scratch);
    float* part_l = splits > 1 ? part_o + rows * splits * D : nullptr;
    const int rc = launch_fwd_cached_tc(q, k_cache, v_cache, o, lse, qpos, kpos, B, Tq, H, Hkv, L, D, scale, causal,
                                        window, sinks, dtype, splits > 1 ? part_o : nullptr, part_l, splits, status, st);
    if (rc != NLFA_OK || splits == 1) return rc;
    p.splits = splits;
    p.part_o = part_o;
    p.part_l = part_l;
    return dtype == NLFA_DTYPE_BF16 ? merge_for_dim<__nv_bfloat16>(p, D, o, lse, st) : merge_for_dim<__half>(p, D, o, lse, st);
  }
  if (path == NLFA_PATH_TENSOR) return NLFA_ERR_UNSUPPORTED_PATH;
  const size_t need = split_scratch_bytes(B, Tq, H, D, choose_splits(B, Tq, H, Hkv, L, D));
  if (need > 0 && scratch != nullptr && scratch_bytes >= need) {     // without scratch: one CTA walks all keys
    p.splits = choose_splits(B, Tq, H, Hkv, L, D);
    p.tiles_per_split = ((L + 31) / 32 + p.splits - 1) / p.splits;
    p.part_o = static_cast<float*>(scratch);
    p.part_l = p.part_o + rows * p.splits * D;
  }
  if (dtype == NLFA_DTYPE_BF16) return launch_for_dim<__nv_bfloat16>(p, D, q, k_cache, v_cache, o, lse, st);
  if (dtype == NLFA_DTYPE_F16) return launch_for_dim<__half>(p, D, q, k_cache, v_cache, o, lse, st);
  return launch_for_dim<float>(p, D, q, k_cache, v_cache, o, lse, st);
}
