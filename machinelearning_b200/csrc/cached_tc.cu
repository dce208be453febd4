// Tensor-core form of the KV-cached block forward (cached.cu has the fp32 one): attention of an
// active block of Tq queries over [cache | block] with the mask taken from absolute positions --
// the attention core of nanolab's `Attention.forward_cached` (nanolab/mixers.py:372-467).
//
// A CTA owns up to 128 query rows of one (batch, KV head): the rows (t, g) of every query head g
// of the group for a run of block positions t, so K and V are fetched once for the whole group.
// One TMA box (64 columns x group heads x positions) brings them in as consecutive 128-byte rows,
// which is the layout the S = Q K^T product wants.  The keys go past in blocks of 128, loaded by
// TMA from nanolab's cache layout [B,Hkv,L,D]; S lands in TMEM, the four softmax warps (one
// thread per row) mask it from the positions, exponentiate and hand P back through TMEM for
// O += P V.  In-order, one key block at a time: the problem is small (a block of a few dozen
// tokens), what matters is that K and V stream through once at TMA speed.  With few (batch, KV
// head) pairs the key blocks are split over several CTAs and the partial rows are combined by
// cached.cu's merge kernel, in a fixed order.
//
// Warps 0-3 softmax, warp 4 TMA producer, warp 5 MMA issuer and TMEM owner.  Every wait bounded.
#include <climits>

#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {
namespace {

constexpr int kNoKey = INT_MAX;          // position written for keys past the end of the cache

struct CachedTcParams {
  int B, Tq, H, Hkv, L;
  int causal, window, sinks;
  int group, tq_tile, n_qtiles;          // query heads per KV head; block positions per CTA; tiles per (b, hk)
  int n_blocks, blocks_per_split, splits;
  int d_real;                            // columns of q / o that exist (32 runs on 64-wide tiles)
  float scale_log2;
  const int* qpos;
  const int* kpos;
  void* o;
  float* lse;
  float* part_o;                         // [rows][splits][D] when splits > 1 (cached.cu's merge format)
  float* part_l;                         // [rows][splits] base-2 logsumexp
  unsigned* status;
};

template <int D, int STAGES>
struct CachedSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;
  static constexpr int kV = kK + STAGES * kTileBytes;
  static constexpr int kPos = kV + STAGES * kTileBytes;          // per stage: 128 key positions
  static constexpr int kBar = kPos + STAGES * 512;
  // barriers: q_full, s_full, p_full, o_ready, k_full[S], v_full[S], kv_empty[S]
  static constexpr int kNumBars = 4 + 3 * STAGES;
  static constexpr int kTmemSlot = kBar + 8 * kNumBars;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
};

// Key blocks this tile has to visit, for contiguous default positions (explicit positions: all).
// Every role evaluates the same pure function, which keeps their barrier phases in step.
struct VisibleRange {
  int lo_key, hi_key;                    // keys [lo_key, hi_key] plus the sink prefix may be visible
  bool all;                              // no range known: visit every block
  __device__ __forceinline__ bool block(int j, int sinks) const {
    if (all) return true;
    const int k0 = j * kTile, k1 = k0 + kTile - 1;
    return (k1 >= lo_key && k0 <= hi_key) || k0 < sinks;
  }
};

__device__ __forceinline__ VisibleRange visible_range(const CachedTcParams& p, int t0, int t1) {
  VisibleRange r;
  r.all = p.qpos != nullptr || p.kpos != nullptr || !p.causal;
  r.lo_key = 0;
  r.hi_key = p.L - 1;
  if (!r.all) {
    const int qp_min = p.L - p.Tq + t0, qp_max = p.L - p.Tq + t1;
    r.hi_key = qp_max;
    if (p.window > 0) {
      const int lo = qp_min - (p.window - p.sinks) + 1;
      r.lo_key = lo > 0 ? lo : 0;
    }
  }
  return r;
}

template <typename T, int D, int STAGES>
__global__ void __launch_bounds__(192, 1)
cached_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const CachedTcParams p) {
  using L = CachedSmem<D, STAGES>;
  constexpr int kBoxes = D / 64;
  constexpr int kBoxBytes = kTile * 128;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr uint32_t kTmemCols = 256;            // S at 0 (P over its first 64 columns), O at 128

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  auto bar = [&](int i) -> uint32_t { return base + L::kBar + 8u * i; };
  constexpr int Q_FULL = 0, S_FULL = 1, P_FULL = 2, O_READY = 3, K_FULL = 4, V_FULL = K_FULL + STAGES,
                KV_EMPTY = V_FULL + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kAbort);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kTmemSlot);
  const WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = (*reinterpret_cast<volatile unsigned*>(p.status) != STATUS_OK) ? 1 : 0;
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(P_FULL), 128);
    mbar_init(bar(O_READY), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(KV_EMPTY + s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(base + L::kTmemSlot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool dead = *abort_flag != 0;

  // this CTA's tile and its share of the key blocks
  const int unit = blockIdx.x;
  const int qt = unit % p.n_qtiles;
  const int bh = unit / p.n_qtiles;
  const int hk = bh % p.Hkv, b = bh / p.Hkv;
  const int t0 = qt * p.tq_tile;
  const int t1 = (t0 + p.tq_tile < p.Tq ? t0 + p.tq_tile : p.Tq) - 1;
  const int j_begin = blockIdx.y * p.blocks_per_split;
  const int j_end = j_begin + p.blocks_per_split < p.n_blocks ? j_begin + p.blocks_per_split : p.n_blocks;
  const VisibleRange vr = visible_range(p, t0, t1);

  if (dead) {
    // a give-up recorded earlier makes this launch a no-op
  } else if (warp == 4) {
    // =============================== TMA producer ============================
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      mbar_arrive_expect_tx(bar(Q_FULL), kBoxes * p.group * p.tq_tile * 128);
      for (int x = 0; x < kBoxes; ++x)
        tma_load_4d(base + L::kQ + x * kBoxBytes, &tm_q, bar(Q_FULL), 64 * x, hk * p.group, t0, b);
    }
    bool ok = true;
    int git = 0;
    for (int j = j_begin; ok && j < j_end; ++j) {
      if (!vr.block(j, p.sinks)) continue;
      const int s = git % STAGES;
      const uint32_t ph = (git / STAGES) & 1;
      ++git;
      if (lane == 0) ok = mbar_wait(bar(KV_EMPTY + s), ph ^ 1, wctx, 60);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar(K_FULL + s), L::kTileBytes);
        mbar_arrive_expect_tx(bar(V_FULL + s), L::kTileBytes);
        for (int x = 0; x < kBoxes; ++x) {
          tma_load_4d(base + L::kK + s * L::kTileBytes + x * kBoxBytes, &tm_k, bar(K_FULL + s), 64 * x,
                      j * kTile, hk, b);
          tma_load_4d(base + L::kV + s * L::kTileBytes + x * kBoxBytes, &tm_v, bar(V_FULL + s), 64 * x,
                      j * kTile, hk, b);
        }
      }
      // positions of the block's keys (a key past the end of the cache gets the "no key" mark)
      int* pos = reinterpret_cast<int*>(gen + L::kPos + s * 512);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * lane + i, key = j * kTile + c;
        pos[c] = key < p.L ? (p.kpos ? p.kpos[key] : key) : kNoKey;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(K_FULL + s));              // the positions travel with the K tile
    }
  } else if (warp == 5) {
    // ================================ MMA issuer =============================
    const uint32_t leader = elect_one() ? 1u : 0u;
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    auto wait_all = [&](uint32_t bb, uint32_t parity, unsigned where) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bb, parity, wctx, where));
    };
    constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false, false);
    constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, D, false, true);
    bool ok = wait_all(bar(Q_FULL), 0, 61);
    int git = 0;
    for (int j = j_begin; ok && j < j_end; ++j) {
      if (!vr.block(j, p.sinks)) continue;
      const int s = git % STAGES;
      const uint32_t ph = (git / STAGES) & 1;
      if (!(ok = wait_all(bar(K_FULL + s), ph, 62))) break;
      // S overwrites P's columns: the previous block's P V product must have read them
      if (git > 0 && !(ok = wait_all(bar(O_READY), (git - 1) & 1, 63))) break;
      tc_fence_after();
      const uint32_t qa = base + L::kQ, ka = base + L::kK + s * L::kTileBytes;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
        umma_ss(leader, tmem_u, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), idesc_qk,
                kk > 0 ? 1u : 0u);
      }
      umma_commit(leader, bar(S_FULL));
      if (!(ok = wait_all(bar(P_FULL), git & 1, 64))) break;
      if (!(ok = wait_all(bar(V_FULL + s), ph, 65))) break;
      tc_fence_after();
      const uint32_t va = base + L::kV + s * L::kTileBytes;
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk)
        umma_ts(leader, tmem_u + 128, tmem_u + 8 * kk, make_smem_desc(va + kk * 2048, kBoxBytes, 1024), idesc_pv,
                (git > 0 || kk > 0) ? 1u : 0u);
      umma_commit(leader, bar(O_READY));
      umma_commit(leader, bar(KV_EMPTY + s));
      ++git;
    }
  } else {
    // ================================= softmax ===============================
    const int row = threadIdx.x;                                 // row of the tile == TMEM lane
    const uint32_t lane_base = 32u * warp;
    const uint32_t s_addr = tmem_addr(tmem, lane_base, 0);
    const uint32_t o_addr = tmem_addr(tmem, lane_base, 128);
    const int t_local = row / p.group, g = row - t_local * p.group;
    const int t = t0 + t_local;
    const bool valid = t_local < p.tq_tile && t < p.Tq;
    const int h = hk * p.group + g;
    const int qp = valid ? (p.qpos ? p.qpos[t] : p.L - p.Tq + t) : 0;
    const int span = p.window - p.sinks;
    const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    int git = 0;
    for (int j = j_begin; j < j_end; ++j) {
      if (!vr.block(j, p.sinks)) continue;
      const int s = git % STAGES;
      ok = mbar_wait(bar(S_FULL), git & 1, wctx, 66);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, sv[c]);
      tc_wait_ld();
      // the mask, from positions: a key past the end is never visible; with a window (causal by
      // definition) kpos <= qpos and (kpos > qpos - (window - sinks) or kpos < sinks); causal:
      // kpos <= qpos; otherwise every key of the cache
      const int4* pos4 = reinterpret_cast<const int4*>(gen + L::kPos + s * 512);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const int4 kp = pos4[8 * c + i / 4];
          const int k4[4] = {kp.x, kp.y, kp.z, kp.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            bool vis = k4[x] != kNoKey;
            if (p.causal) vis = vis && k4[x] <= qp;
            if (p.window > 0) vis = vis && (k4[x] > qp - span || k4[x] < p.sinks);
            if (!vis) sv[c][i + x] = __float_as_uint(-INFINITY);
          }
        }
      }
      float b0 = -INFINITY, b1 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          b0 = fmax3(b0, __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
          b1 = fmax3(b1, __uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3]));
        }
      }
      const float mx = fmaxf(b0, b1) * p.scale_log2;
      // Online softmax in base 2 with a reference exponent that is only raised (with O and l
      // rescaled) when a block's maximum exceeds it by more than 2^8.
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_ref + 8.f || m_ref == -INFINITY) {
        if (m_ref != -INFINITY) {
          alpha = fast_exp2(m_ref - mx);
          rescale = true;
          l *= alpha;
        }
        m_ref = mx;                                                // may still be -inf: nothing seen yet
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t negm2 = pack_f2(-m_use, -m_use);
      uint64_t acc0 = 0ull, acc1 = 0ull;
      uint32_t pk[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float e0, e1, e2, e3;
          unpack_f2(ffma2(pack_f2(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])), scale2, negm2), e0, e1);
          unpack_f2(ffma2(pack_f2(__uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3])), scale2, negm2), e2, e3);
          e0 = fast_exp2(e0); e1 = fast_exp2(e1); e2 = fast_exp2(e2); e3 = fast_exp2(e3);
          acc0 = fadd2(acc0, pack_f2(e0, e1));
          acc1 = fadd2(acc1, pack_f2(e2, e3));
          pk[c][i / 2] = Pack2<T>::pack(e0, e1);
          pk[c][i / 2 + 1] = Pack2<T>::pack(e2, e3);
        }
      }
      {
        float lo, hi;
        unpack_f2(fadd2(acc0, acc1), lo, hi);
        l += lo + hi;
      }
      // the previous P V product is complete (the issuer waited for it before this block's S):
      // O may be rescaled and P's columns overwritten
      if (git > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld32(o_addr + 32 * c, orr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          tmem_st32(o_addr + 32 * c, orr);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st16(s_addr + 16 * c, pk[c]);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL));
      ++git;
    }
    if (ok && git > 0) {
      ok = mbar_wait(bar(O_READY), (git - 1) & 1, wctx, 67);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after();
    }
    if (ok) {
      // every lane takes part in the TMEM loads (they are warp-wide); only rows that belong to a
      // query write
      const float inv = l > 0.f ? 1.f / l : 0.f;                   // a row that sees no key gives zeros
      const long long orow = (static_cast<long long>(b) * p.Tq + t) * p.H + h;
      const float lse2 = l > 0.f ? m_ref + log2f(l) : -INFINITY;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        if (git > 0) {
          tmem_ld32(o_addr + 32 * c, orr);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = 0u;
        }
        if (!valid || 32 * c >= p.d_real) continue;
        if (p.splits > 1) {
          float* dst = p.part_o + (orow * p.splits + blockIdx.y) * p.d_real + 32 * c;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + i) =
                make_float4(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv,
                            __uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.o) + orow * p.d_real + 32 * c);
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            dst[i / 8] = make_uint4(
                Pack2<T>::pack(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv),
                Pack2<T>::pack(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv),
                Pack2<T>::pack(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv),
                Pack2<T>::pack(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv));
        }
      }
      if (valid) {
        if (p.splits > 1) p.part_l[orow * p.splits + blockIdx.y] = lse2;
        else if (p.lse) p.lse[(static_cast<long long>(b) * p.H + h) * p.Tq + t] = lse2 * kLn2;
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// 4-D tensor map, 16-bit elements, 128-byte swizzle, boxes of 64 columns.
int encode_map(CUtensorMap* map, const void* base, int dtype, const unsigned long long dims[4],
               const unsigned long long strides[3], const unsigned box[4]) {
  using Fn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                          const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                          CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Fn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return NLFA_ERR_CUDA;
    fn = reinterpret_cast<Fn>(ptr);
  }
  const cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  const cuuint64_t st[3] = {strides[0], strides[1], strides[2]};
  const cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  const cuuint32_t es[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt =
      dtype == NLFA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(map, dt, 4, const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename T, int D, int STAGES>
int launch_t(const CachedTcParams& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
             cudaStream_t stream) {
  using L = CachedSmem<D, STAGES>;
  auto kern = cached_tc_kernel<T, D, STAGES>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kDynamic) != NLFA_OK) return NLFA_ERR_CUDA;
  const dim3 grid(static_cast<unsigned>(p.B * p.Hkv * p.n_qtiles), static_cast<unsigned>(p.splits));
  kern<<<grid, 192, L::kDynamic, stream>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace

bool cached_tc_applies(int Tq, int H, int Hkv, int L, int D, int dtype) {
  if (dtype != NLFA_DTYPE_F16 && dtype != NLFA_DTYPE_BF16) return false;
  if (D != 32 && D != 64 && D != 128) return false;
  const int group = H / Hkv;
  if (group > kTile) return false;
  const int tq_tile = Tq < kTile / group ? Tq : kTile / group;
  return tq_tile * group >= 16 && L >= 2 * kTile;          // below that the fp32 kernel's small tiles fit better
}

int cached_tc_splits(int B, int Tq, int H, int Hkv, int L) {
  const int group = H / Hkv;
  const int tq_tile = Tq < kTile / group ? Tq : kTile / group;
  const long long units = static_cast<long long>(B) * Hkv * ((Tq + tq_tile - 1) / tq_tile);
  const int n_blocks = (L + kTile - 1) / kTile;
  long long s = sm_count() / (units > 0 ? units : 1);       // about one CTA per SM in all
  if (s > n_blocks / 2) s = n_blocks / 2;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  const int per = (n_blocks + static_cast<int>(s) - 1) / static_cast<int>(s);
  return (n_blocks + per - 1) / per;                        // no split without a block
}

int launch_fwd_cached_tc(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                         const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                         float scale, int causal, int window, int sinks, int dtype, float* part_o,
                         float* part_l, int splits, unsigned* status, cudaStream_t stream) {
  if (!(scale > 0.f)) return NLFA_ERR_UNSUPPORTED_PATH;      // the row maximum is taken before scaling
  CachedTcParams p;
  p.B = B; p.Tq = Tq; p.H = H; p.Hkv = Hkv; p.L = L;
  p.causal = causal ? 1 : 0; p.window = window; p.sinks = sinks;
  p.group = H / Hkv;
  p.tq_tile = Tq < kTile / p.group ? Tq : kTile / p.group;
  p.n_qtiles = (Tq + p.tq_tile - 1) / p.tq_tile;
  p.n_blocks = (L + kTile - 1) / kTile;
  p.splits = splits < 1 ? 1 : splits;
  p.blocks_per_split = (p.n_blocks + p.splits - 1) / p.splits;
  p.scale_log2 = scale * kLog2e;
  p.qpos = qpos; p.kpos = kpos;
  p.o = o; p.lse = lse;
  p.part_o = part_o; p.part_l = part_l;
  p.status = status;
  p.d_real = D;
  // q [B,Tq,H,D]: box = 64 columns x the group's heads x tq_tile positions -> rows (t, g) of 128 bytes
  // k, v [B,Hkv,L,D]: box = 64 columns x 128 keys
  const unsigned long long e = 2;
  const unsigned long long q_dims[4] = {static_cast<unsigned long long>(D), static_cast<unsigned long long>(H),
                                        static_cast<unsigned long long>(Tq), static_cast<unsigned long long>(B)};
  const unsigned long long q_str[3] = {D * e, static_cast<unsigned long long>(H) * D * e,
                                       static_cast<unsigned long long>(Tq) * H * D * e};
  const unsigned q_box[4] = {64u, static_cast<unsigned>(p.group), static_cast<unsigned>(p.tq_tile), 1u};
  const unsigned long long k_dims[4] = {static_cast<unsigned long long>(D), static_cast<unsigned long long>(L),
                                        static_cast<unsigned long long>(Hkv), static_cast<unsigned long long>(B)};
  const unsigned long long k_str[3] = {D * e, static_cast<unsigned long long>(L) * D * e,
                                       static_cast<unsigned long long>(Hkv) * L * D * e};
  const unsigned k_box[4] = {64u, static_cast<unsigned>(kTile), 1u, 1u};
  CUtensorMap mq, mk, mv;
  int st = encode_map(&mq, q, dtype, q_dims, q_str, q_box);
  if (st == NLFA_OK) st = encode_map(&mk, k_cache, dtype, k_dims, k_str, k_box);
  if (st == NLFA_OK) st = encode_map(&mv, v_cache, dtype, k_dims, k_str, k_box);
  if (st != NLFA_OK) return st;
  const bool bf16 = dtype == NLFA_DTYPE_BF16;
  if (D <= 64)
    return bf16 ? launch_t<__nv_bfloat16, 64, 3>(p, mq, mk, mv, stream) : launch_t<__half, 64, 3>(p, mq, mk, mv, stream);
  return bf16 ? launch_t<__nv_bfloat16, 128, 2>(p, mq, mk, mv, stream) : launch_t<__half, 128, 2>(p, mq, mk, mv, stream);
}

}  // namespace nlfa
