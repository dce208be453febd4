// Tensor-core forward for sm_100a: S = Q K^T and O += P V on tcgen05 with the
// accumulators in TMEM, tiles brought in by TMA, online softmax in registers.
//
// One CTA owns NT consecutive 128-row query tiles of one (batch, head) and walks
// the key blocks they can see.  Warp roles:
//   warps [0, 4 NT)   softmax: warpgroup t owns query tile t, one thread per row
//   warp  4 NT        TMA producer (one lane): Q once, then a ring of K and V stages
//   warp  4 NT + 1    MMA issuer (one lane) and owner of the TMEM allocation
// Hand-offs are mbarriers: K/V full/empty per stage, S ready, P ready, O ready.
//
// TMEM columns: S_t at 128 t (fp32, 128 columns; P_t, 16-bit, overwrites its
// first 64 columns and is read back as the A operand of the PV product);
// O_t at 128 NT + D t.
//
// Computes what nanolab/csrc/flash_attn_cuda.cu:583-797 computes (softmax in
// base 2, L = m ln2 + log l at :279), with the sliding-window mask of
// nanolab/mixers.py:125-132 and skipping of key blocks no row can see.
#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {
namespace {

struct FwdParams {
  int T, H, Hkv;
  int window, sinks;
  int n_tiles;            // ceil(T / 128)
  float scale_log2;       // scale * log2(e)
  void* o;
  float* lse;
  unsigned* status;
};

template <int D, int NT, int STAGES>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;          // one 128 x D 16-bit tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + NT * kTileBytes;
  static constexpr int kV = kK + STAGES * kTileBytes;
  static constexpr int kBar = kV + STAGES * kTileBytes;
  // barriers (8 bytes each): q_full[NT], s_full[NT], p_full[NT], o_full[NT],
  // k_full[S], k_empty[S], v_full[S], v_empty[S]
  static constexpr int kNumBars = 4 * NT + 4 * STAGES;
  static constexpr int kTmemSlot = kBar + 8 * kNumBars;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;            // slack for 1024-byte alignment
};

// Block index visited at iteration `it` of a CTA whose recent range starts at
// `lo` and which first visits `extra_sinks` sink blocks.
__device__ __forceinline__ int block_at(int it, int extra_sinks, int lo) {
  return it < extra_sinks ? it : lo + (it - extra_sinks);
}

__device__ __forceinline__ bool tile_sees_block(const TileRange& r, int j) {
  return j <= r.hi && (j >= r.lo || j < r.sink_blocks);
}

template <typename T, int D, int NT, int STAGES>
__global__ void __launch_bounds__(NT * 128 + 64, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdSmem<D, NT, STAGES>;
  constexpr int kBoxes = D / 64;                 // 64-element column boxes per tile
  constexpr int kBoxBytes = kTile * 128;         // 128 rows x 128 bytes
  constexpr uint32_t kTmemCols = (NT * (128 + D) <= 256) ? 256u : 512u;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  auto bar = [&](int i) -> uint32_t { return base + L::kBar + 8u * i; };
  const int Q_FULL = 0, S_FULL = NT, P_FULL = 2 * NT, O_FULL = 3 * NT;
  const int K_FULL = 4 * NT, K_EMPTY = K_FULL + STAGES, V_FULL = K_EMPTY + STAGES,
            V_EMPTY = V_FULL + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kAbort);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kTmemSlot);
  const WaitCtx wctx{abort_flag, p.status};

  // ---- which work this CTA owns: heavy (late) query tiles are scheduled first
  const int n_units = (p.n_tiles + NT - 1) / NT;
  const int unit = n_units - 1 - static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int hk = h / (p.H / p.Hkv);
  const int tile0 = unit * NT;

  TileRange tr[NT];
  bool tile_valid[NT];
  int cta_lo = 1 << 30, cta_hi = -1, sink_blocks = 0;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    tile_valid[t] = (tile0 + t) < p.n_tiles;
    tr[t] = tile_range(tile0 + t, p.window, p.sinks);
    if (tile_valid[t]) {
      cta_lo = tr[t].lo < cta_lo ? tr[t].lo : cta_lo;
      cta_hi = tr[t].hi > cta_hi ? tr[t].hi : cta_hi;
      sink_blocks = tr[t].sink_blocks;
    }
  }
  const int extra_sinks = sink_blocks < cta_lo ? sink_blocks : cta_lo;
  const int n_iters = extra_sinks + (cta_hi - cta_lo + 1);

  // ---- set-up
  if (threadIdx.x == 0) {
    // a timeout recorded by an earlier CTA (or launch) makes the rest of the grid a no-op
    *abort_flag = (*reinterpret_cast<volatile unsigned*>(p.status) != STATUS_OK) ? 1 : 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar(Q_FULL + t), 1);
      mbar_init(bar(S_FULL + t), 1);
      mbar_init(bar(P_FULL + t), 128);
      mbar_init(bar(O_FULL + t), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 4 * NT + 1) {
    tmem_alloc(base + L::kTmemSlot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool dead = *abort_flag != 0;

  if (dead) {
    // fall through to the tail
  } else if (warp == 4 * NT) {
    // =============================== TMA producer ============================
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      for (int t = 0; t < NT; ++t) {
        if (!tile_valid[t]) continue;
        mbar_arrive_expect_tx(bar(Q_FULL + t), L::kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(base + L::kQ + t * L::kTileBytes + x * kBoxBytes, &tm_q, bar(Q_FULL + t),
                      64 * x, h, (tile0 + t) * kTile, b);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const int j = block_at(it, extra_sinks, cta_lo);
        if (!mbar_wait(bar(K_EMPTY + s), ph ^ 1, wctx, 1)) break;
        mbar_arrive_expect_tx(bar(K_FULL + s), L::kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(base + L::kK + s * L::kTileBytes + x * kBoxBytes, &tm_k, bar(K_FULL + s),
                      64 * x, hk, j * kTile, b);
        if (!mbar_wait(bar(V_EMPTY + s), ph ^ 1, wctx, 2)) break;
        mbar_arrive_expect_tx(bar(V_FULL + s), L::kTileBytes);
        for (int x = 0; x < kBoxes; ++x)
          tma_load_4d(base + L::kV + s * L::kTileBytes + x * kBoxBytes, &tm_v, bar(V_FULL + s),
                      64 * x, hk, j * kTile, b);
      }
    }
  } else if (warp == 4 * NT + 1) {
    // ================================ MMA issuer =============================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, D, false, true);

      auto issue_s = [&](int t, int s) {
        const uint32_t qa = base + L::kQ + t * L::kTileBytes;
        const uint32_t ka = base + L::kK + s * L::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          mma_ss(tmem + 128 * t, make_smem_desc(qa + off, 16, 1024),
                 make_smem_desc(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int s, bool accumulate) {
        const uint32_t va = base + L::kV + s * L::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          // 16 keys per step: 8 packed TMEM columns of P, 16 rows (2048 bytes) of V
          mma_ts(tmem + 128 * NT + D * t, tmem + 128 * t + 8 * kk,
                 make_smem_desc(va + kk * 2048, kBoxBytes, 1024), idesc_pv,
                 (accumulate || kk > 0) ? 1u : 0u);
        }
      };

      bool ok = true;
      int p_count[NT];
      bool o_started[NT];
      for (int t = 0; t < NT; ++t) {
        p_count[t] = 0;
        o_started[t] = false;
        if (tile_valid[t]) ok = ok && mbar_wait(bar(Q_FULL + t), 0, wctx, 3);
      }
      if (ok && n_iters > 0) {
        ok = mbar_wait(bar(K_FULL + 0), 0, wctx, 4);
        if (ok) {
          tc_fence_after();
          const int j0 = block_at(0, extra_sinks, cta_lo);
          for (int t = 0; t < NT; ++t)
            if (tile_valid[t] && tile_sees_block(tr[t], j0)) {
              issue_s(t, 0);
              tc_commit(bar(S_FULL + t));
            }
          tc_commit(bar(K_EMPTY + 0));
        }
      }
      for (int it = 0; ok && it < n_iters; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const int j = block_at(it, extra_sinks, cta_lo);
        const bool have_next = it + 1 < n_iters;
        const int s1 = (it + 1) % STAGES;
        const uint32_t ph1 = ((it + 1) / STAGES) & 1;
        const int j1 = have_next ? block_at(it + 1, extra_sinks, cta_lo) : 0;
        if (!(ok = mbar_wait(bar(V_FULL + s), ph, wctx, 5))) break;
        if (have_next && !(ok = mbar_wait(bar(K_FULL + s1), ph1, wctx, 6))) break;
        for (int t = 0; t < NT; ++t) {
          if (!tile_valid[t]) continue;
          if (tile_sees_block(tr[t], j)) {
            if (!(ok = mbar_wait(bar(P_FULL + t), p_count[t] & 1, wctx, 7))) break;
            ++p_count[t];
            tc_fence_after();
            issue_pv(t, s, o_started[t]);
            o_started[t] = true;
          }
          if (have_next && tile_sees_block(tr[t], j1)) {
            tc_fence_after();
            issue_s(t, s1);
            tc_commit(bar(S_FULL + t));
          }
        }
        if (!ok) break;
        tc_commit(bar(V_EMPTY + s));
        if (have_next) tc_commit(bar(K_EMPTY + s1));
      }
      if (ok)
        for (int t = 0; t < NT; ++t)
          if (tile_valid[t]) tc_commit(bar(O_FULL + t));
    }
  } else {
    // ================================= softmax ===============================
    const int t = warp >> 2;                       // query tile of this warpgroup
    const int row = threadIdx.x - 128 * t;         // row inside the tile == TMEM lane
    const uint32_t lane_base = 32u * (warp & 3);
    if (tile_valid[t]) {
      const int tile = tile0 + t;
      const int qpos = tile * kTile + row;
      const uint32_t s_addr = tmem_addr(tmem, lane_base, 128 * t);
      const uint32_t o_addr = tmem_addr(tmem, lane_base, 128 * NT + D * t);
      float m_ref = -INFINITY, l = 0.f;
      int count = 0;
      bool ok = true;
      for (int it = 0; it < n_iters; ++it) {
        const int j = block_at(it, extra_sinks, cta_lo);
        if (!tile_sees_block(tr[t], j)) continue;
        ok = mbar_wait(bar(S_FULL + t), count & 1, wctx, 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();

        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, sr[c]);
        tc_wait_ld();

        float x[128];
        const bool full = block_fully_visible(tile, j, p.window, p.sinks);
        float mx = -INFINITY;
        if (full) {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            x[c] = __uint_as_float(sr[c >> 5][c & 31]) * p.scale_log2;
            mx = fmaxf(mx, x[c]);
          }
        } else {
          const int k0 = j * kTile;
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            const float sv = __uint_as_float(sr[c >> 5][c & 31]) * p.scale_log2;
            x[c] = key_visible(qpos, k0 + c, p.window, p.sinks) ? sv : -INFINITY;
            mx = fmaxf(mx, x[c]);
          }
        }

        // Reference maximum for the exponent.  It is only moved (and O and l
        // rescaled) when the row maximum has grown by more than 2^8, which keeps
        // P within 16-bit range and makes the TMEM round trip of O rare.
        float alpha = 1.f;
        bool rescale = false;
        if (count == 0) {
          m_ref = mx;
        } else if (mx > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - mx);     // m_ref == -inf gives 0
          m_ref = mx;
          rescale = true;
        }
        if (__any_sync(0xffffffffu, rescale)) {
          l *= alpha;
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
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        float sum = 0.f;
        uint32_t pk[2][32];
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float p0 = fast_exp2(x[2 * c] - m_use);
          const float p1 = fast_exp2(x[2 * c + 1] - m_use);
          sum += p0 + p1;
          pk[c >> 5][c & 31] = Pack2<T>::pack(p0, p1);
        }
        l += sum;
        tmem_st32(s_addr, pk[0]);
        tmem_st32(s_addr + 32, pk[1]);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(P_FULL + t));
        ++count;
      }

      if (ok) {
        ok = mbar_wait(bar(O_FULL + t), 0, wctx, 9);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        T* orow = static_cast<T*>(p.o) +
                  ((static_cast<long long>(b) * p.T + qpos) * p.H + h) * static_cast<long long>(D);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t orr[32];
          tmem_ld32(o_addr + 32 * c, orr);
          tc_wait_ld();
          if (qpos < p.T) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = Pack2<T>::pack(__uint_as_float(orr[8 * i + 0]) * inv, __uint_as_float(orr[8 * i + 1]) * inv);
              w.y = Pack2<T>::pack(__uint_as_float(orr[8 * i + 2]) * inv, __uint_as_float(orr[8 * i + 3]) * inv);
              w.z = Pack2<T>::pack(__uint_as_float(orr[8 * i + 4]) * inv, __uint_as_float(orr[8 * i + 5]) * inv);
              w.w = Pack2<T>::pack(__uint_as_float(orr[8 * i + 6]) * inv, __uint_as_float(orr[8 * i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + 32 * c + 8 * i) = w;
            }
          }
        }
        if (qpos < p.T)
          p.lse[static_cast<long long>(bh) * p.T + qpos] = (m_ref + log2f(l)) * kLn2;
      }
    }
  }

  // ---- tail: everyone meets here (all waits above are bounded), TMEM is freed
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 4 * NT + 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <typename T, int D, int NT, int STAGES>
int launch_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
             void* o, float* lse, unsigned* status, cudaStream_t stream) {
  using L = FwdSmem<D, NT, STAGES>;
  auto kern = fwd_tc_kernel<T, D, NT, STAGES>;
  static bool configured = false;       // per template instance; the attribute is per function
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) !=
        cudaSuccess)
      return NLFA_ERR_CUDA;
    configured = true;
  }
  FwdParams fp;
  fp.T = p.T;
  fp.H = p.H;
  fp.Hkv = p.Hkv;
  fp.window = p.window;
  fp.sinks = p.sinks;
  fp.n_tiles = (p.T + kTile - 1) / kTile;
  fp.scale_log2 = p.scale * kLog2e;
  fp.o = o;
  fp.lse = lse;
  fp.status = status;
  const int n_units = (fp.n_tiles + NT - 1) / NT;
  dim3 grid(n_units, p.B * p.H);
  kern<<<grid, NT * 128 + 64, L::kDynamic, stream>>>(mq, mk, mv, fp);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace

int launch_fwd_tc(const Problem& p, const void* q, const void* k, const void* v, void* o,
                  float* lse, unsigned* status, cudaStream_t stream) {
  if (p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (p.D != 64 && p.D != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  CUtensorMap mq, mk, mv;
  int st = make_tile_map(&mq, q, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mk, k, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mv, v, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st != NLFA_OK) return st;
  const bool bf16 = p.dtype == NLFA_DTYPE_BF16;
  if (p.D == 64) {
    return bf16 ? launch_t<__nv_bfloat16, 64, 2, 3>(p, mq, mk, mv, o, lse, status, stream)
                : launch_t<__half, 64, 2, 3>(p, mq, mk, mv, o, lse, status, stream);
  }
  return bf16 ? launch_t<__nv_bfloat16, 128, 2, 2>(p, mq, mk, mv, o, lse, status, stream)
              : launch_t<__half, 128, 2, 2>(p, mq, mk, mv, o, lse, status, stream);
}

}  // namespace nlfa
