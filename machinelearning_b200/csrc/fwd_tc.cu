// Tensor-core forward for sm_100a: S = Q K^T and O += P V on tcgen05 with the
// accumulators in TMEM, tiles brought in by TMA, online softmax in registers.
//
// Persistent kernel: one CTA per SM walks a static, heavy-first list of work
// units.  A unit is NT consecutive 128-row query tiles of one (batch, head); the
// CTA visits the key blocks those tiles can see.  Warp roles:
//   warps [0, 4 NT)   softmax: warpgroup t owns query tile t, one thread per row
//   warp  4 NT        TMA producer (one lane): Q per unit, a ring of K and V stages
//   warp  4 NT + 1    MMA issuer (one lane) and owner of the TMEM allocation
// Hand-offs are mbarriers whose phases run on across units: Q full/empty per Q
// buffer, K/V full/empty per stage, S ready, P ready, O ready per tile.  While the
// softmax warps finish a unit (normalise and store O) the producer and the MMA
// issuer are already on the next one.
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

#ifdef NLFA_TRACE
// Debug-only timeline of CTA 0: (clock64, tag) pairs per role.
__device__ long long g_trace[4][1024];
__device__ int g_trace_n[4];
#define NLFA_TRACE_EVENT(role, tag)                                   \
  do {                                                                \
    if (blockIdx.x == 0) {                                            \
      const int i_ = g_trace_n[role]++;                               \
      if (i_ < 512) {                                                 \
        g_trace[role][2 * i_] = clock64();                            \
        g_trace[role][2 * i_ + 1] = (tag);                            \
      }                                                               \
    }                                                                 \
  } while (0)
#else
#define NLFA_TRACE_EVENT(role, tag)
#endif

namespace {

struct FwdParams {
  int T, H, Hkv;
  int window, sinks;
  int n_tiles;            // ceil(T / 128)
  int n_units;            // ceil(n_tiles / NT)
  int total_units;        // n_units * B * H
  float scale_log2;       // scale * log2(e), > 0
  void* o;
  float* lse;
  unsigned* status;
};

template <int D, int NT, int STAGES, int QBUF>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;          // one 128 x D 16-bit tile
  static constexpr int kQ = 0;                              // [QBUF][NT] tiles
  static constexpr int kK = kQ + QBUF * NT * kTileBytes;
  static constexpr int kV = kK + STAGES * kTileBytes;
  static constexpr int kBar = kV + STAGES * kTileBytes;
  // barriers (8 bytes each): q_full[QBUF], q_empty[QBUF], s_full[NT], p_full[NT], o_full[NT],
  // k_full[S], k_empty[S], v_full[S], v_empty[S]
  static constexpr int kNumBars = 2 * QBUF + 3 * NT + 4 * STAGES;
  static constexpr int kTmemSlot = kBar + 8 * kNumBars;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;            // slack for 1024-byte alignment
};

__device__ __forceinline__ bool tile_sees_block(const TileRange& r, int j) {
  return j <= r.hi && (j >= r.lo || j < r.sink_blocks);
}

// Everything a role needs to know about one work unit; every role derives the
// same values from the unit index, which keeps their barrier phases in step.
template <int NT>
struct Unit {
  int b, h, hk, tile0;
  TileRange tr[NT];
  bool valid[NT];
  int lo, extra_sinks, n_iters;
  int n_valid;

  __device__ __forceinline__ int block_at(int it) const {
    return it < extra_sinks ? it : lo + (it - extra_sinks);
  }
  __device__ __forceinline__ bool sees(int t, int j) const {
    return valid[t] && tile_sees_block(tr[t], j);
  }
};

template <int NT>
__device__ __forceinline__ Unit<NT> make_unit(int u, const FwdParams& p, int BH) {
  Unit<NT> w;
  const int rank = u / BH;                    // heavy (late) query tiles first
  const int bh = u - rank * BH;
  const int unit = p.n_units - 1 - rank;
  w.b = bh / p.H;
  w.h = bh - w.b * p.H;
  w.hk = w.h / (p.H / p.Hkv);
  w.tile0 = unit * NT;
  int hi = -1, sink_blocks = 0;
  w.lo = 1 << 30;
  w.n_valid = 0;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    w.valid[t] = (w.tile0 + t) < p.n_tiles;
    w.tr[t] = tile_range(w.tile0 + t, p.window, p.sinks);
    if (w.valid[t]) {
      w.lo = w.tr[t].lo < w.lo ? w.tr[t].lo : w.lo;
      hi = w.tr[t].hi > hi ? w.tr[t].hi : hi;
      sink_blocks = w.tr[t].sink_blocks;
      ++w.n_valid;
    }
  }
  w.extra_sinks = sink_blocks < w.lo ? sink_blocks : w.lo;
  w.n_iters = w.extra_sinks + (hi - w.lo + 1);
  return w;
}

template <typename T, int D, int NT, int STAGES, int QBUF>
__global__ void __launch_bounds__(NT * 128 + 64, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = FwdSmem<D, NT, STAGES, QBUF>;
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
  constexpr int Q_FULL = 0, Q_EMPTY = QBUF, S_FULL = 2 * QBUF, P_FULL = S_FULL + NT,
                O_FULL = P_FULL + NT, K_FULL = O_FULL + NT, K_EMPTY = K_FULL + STAGES,
                V_FULL = K_EMPTY + STAGES, V_EMPTY = V_FULL + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kAbort);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kTmemSlot);
  const WaitCtx wctx{abort_flag, p.status};
  const int BH = p.total_units / p.n_units;

  // ---- set-up
  if (threadIdx.x == 0) {
    // a timeout recorded by an earlier CTA (or launch) makes the rest of the grid a no-op
    *abort_flag = (*reinterpret_cast<volatile unsigned*>(p.status) != STATUS_OK) ? 1 : 0;
    for (int i = 0; i < QBUF; ++i) {
      mbar_init(bar(Q_FULL + i), 1);
      mbar_init(bar(Q_EMPTY + i), 1);
    }
    for (int t = 0; t < NT; ++t) {
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
      int git = 0, uc = 0;
      bool ok = true;
      for (int u = blockIdx.x; ok && u < p.total_units; u += gridDim.x, ++uc) {
        const Unit<NT> w = make_unit<NT>(u, p, BH);
        const int qb = uc % QBUF;
        const uint32_t qph = (uc / QBUF) & 1;
        if (!(ok = mbar_wait(bar(Q_EMPTY + qb), qph ^ 1, wctx, 10))) break;
        mbar_arrive_expect_tx(bar(Q_FULL + qb), w.n_valid * L::kTileBytes);
        for (int t = 0; t < NT; ++t) {
          if (!w.valid[t]) continue;
          for (int x = 0; x < kBoxes; ++x)
            tma_load_4d(base + L::kQ + (qb * NT + t) * L::kTileBytes + x * kBoxBytes, &tm_q,
                        bar(Q_FULL + qb), 64 * x, w.h, (w.tile0 + t) * kTile, w.b);
        }
        for (int it = 0; it < w.n_iters; ++it, ++git) {
          const int s = git % STAGES;
          const uint32_t ph = (git / STAGES) & 1;
          const int j = w.block_at(it);
          if (!(ok = mbar_wait(bar(K_EMPTY + s), ph ^ 1, wctx, 1))) break;
          NLFA_TRACE_EVENT(3, 100 + it);
          mbar_arrive_expect_tx(bar(K_FULL + s), L::kTileBytes);
          for (int x = 0; x < kBoxes; ++x)
            tma_load_4d(base + L::kK + s * L::kTileBytes + x * kBoxBytes, &tm_k, bar(K_FULL + s),
                        64 * x, w.hk, j * kTile, w.b);
          if (!(ok = mbar_wait(bar(V_EMPTY + s), ph ^ 1, wctx, 2))) break;
          mbar_arrive_expect_tx(bar(V_FULL + s), L::kTileBytes);
          for (int x = 0; x < kBoxes; ++x)
            tma_load_4d(base + L::kV + s * L::kTileBytes + x * kBoxBytes, &tm_v, bar(V_FULL + s),
                        64 * x, w.hk, j * kTile, w.b);
        }
      }
    }
  } else if (warp == 4 * NT + 1) {
    // ================================ MMA issuer =============================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, D, false, true);

      auto issue_s = [&](int qb, int t, int s) {
        const uint32_t qa = base + L::kQ + (qb * NT + t) * L::kTileBytes;
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
      int git = 0, uc = 0;
      int p_count[NT];
      for (int t = 0; t < NT; ++t) p_count[t] = 0;
      for (int u = blockIdx.x; ok && u < p.total_units; u += gridDim.x, ++uc) {
        const Unit<NT> w = make_unit<NT>(u, p, BH);
        const int qb = uc % QBUF;
        NLFA_TRACE_EVENT(2, 1);
        if (!(ok = mbar_wait(bar(Q_FULL + qb), (uc / QBUF) & 1, wctx, 3))) break;
        NLFA_TRACE_EVENT(2, 2);
        {
          const int s0 = git % STAGES;
          if (!(ok = mbar_wait(bar(K_FULL + s0), (git / STAGES) & 1, wctx, 4))) break;
          tc_fence_after();
          const int j0 = w.block_at(0);
          for (int t = 0; t < NT; ++t)
            if (w.sees(t, j0)) {
              issue_s(qb, t, s0);
              tc_commit(bar(S_FULL + t));
            }
          tc_commit(bar(K_EMPTY + s0));
          NLFA_TRACE_EVENT(2, 3);
        }
        bool o_started[NT];
        for (int t = 0; t < NT; ++t) o_started[t] = false;
        for (int it = 0; ok && it < w.n_iters; ++it, ++git) {
          const int s = git % STAGES;
          const uint32_t ph = (git / STAGES) & 1;
          const int j = w.block_at(it);
          const bool have_next = it + 1 < w.n_iters;
          const int s1 = (git + 1) % STAGES;
          const uint32_t ph1 = ((git + 1) / STAGES) & 1;
          const int j1 = have_next ? w.block_at(it + 1) : 0;
          if (!(ok = mbar_wait(bar(V_FULL + s), ph, wctx, 5))) break;
          if (have_next && !(ok = mbar_wait(bar(K_FULL + s1), ph1, wctx, 6))) break;
          for (int t = 0; t < NT; ++t) {
            if (w.sees(t, j)) {
              NLFA_TRACE_EVENT(2, 10 + t);
              if (!(ok = mbar_wait(bar(P_FULL + t), p_count[t] & 1, wctx, 7))) break;
              NLFA_TRACE_EVENT(2, 20 + t);
              ++p_count[t];
              tc_fence_after();
              issue_pv(t, s, o_started[t]);
              o_started[t] = true;
            }
            if (have_next && w.sees(t, j1)) {
              tc_fence_after();
              issue_s(qb, t, s1);
              tc_commit(bar(S_FULL + t));
            }
          }
          if (!ok) break;
          tc_commit(bar(V_EMPTY + s));
          if (have_next) tc_commit(bar(K_EMPTY + s1));
        }
        if (!ok) break;
        tc_commit(bar(Q_EMPTY + qb));
        for (int t = 0; t < NT; ++t)
          if (w.valid[t]) tc_commit(bar(O_FULL + t));
      }
    }
  } else {
    // ================================= softmax ===============================
    const int t = warp >> 2;                       // query tile of this warpgroup
    const int row = threadIdx.x - 128 * t;         // row inside the tile == TMEM lane
    const uint32_t lane_base = 32u * (warp & 3);
    const uint32_t s_addr = tmem_addr(tmem, lane_base, 128 * t);
    const uint32_t o_addr = tmem_addr(tmem, lane_base, 128 * NT + D * t);
    const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);
    int s_count = 0, o_count = 0;
    bool ok = true;
    for (int u = blockIdx.x; ok && u < p.total_units; u += gridDim.x) {
      const Unit<NT> w = make_unit<NT>(u, p, BH);
      if (!w.valid[t]) continue;
      const int tile = w.tile0 + t;
      const int qpos = tile * kTile + row;
      float m_ref = -INFINITY, l = 0.f;          // m_ref is in scaled (base-2) units
      bool first = true;
      for (int it = 0; it < w.n_iters; ++it) {
        const int j = w.block_at(it);
        if (!tile_sees_block(w.tr[t], j)) continue;
        if (row == 0) NLFA_TRACE_EVENT(t, 1);
        ok = mbar_wait(bar(S_FULL + t), s_count & 1, wctx, 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_count;
        tc_fence_after();
        if (row == 0) NLFA_TRACE_EVENT(t, 2);

        float sv[128];
        {
          uint32_t sr[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, sr[c]);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 128; ++c) sv[c] = __uint_as_float(sr[c >> 5][c & 31]);
        }
        if (!block_fully_visible(tile, j, p.window, p.sinks)) {
          const int k0 = j * kTile;
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if (!key_visible(qpos, k0 + c, p.window, p.sinks)) sv[c] = -INFINITY;
        }
        // row maximum of the raw scores: four independent chains of 3-input max
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          m0 = fmax3(m0, sv[c + 0], sv[c + 1]);
          m1 = fmax3(m1, sv[c + 2], sv[c + 3]);
          m2 = fmax3(m2, sv[c + 4], sv[c + 5]);
          m3 = fmax3(m3, sv[c + 6], sv[c + 7]);
        }
        const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.scale_log2;
        if (row == 0) NLFA_TRACE_EVENT(t, 3);

        // Reference maximum for the exponent.  It is only moved (and O and l
        // rescaled) when the row maximum has grown by more than 2^8, which keeps
        // P within 16-bit range and makes the TMEM round trip of O rare.
        float alpha = 1.f;
        bool rescale = false;
        if (first) {
          m_ref = mx;
        } else if (mx > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - mx);     // m_ref == -inf gives 0
          m_ref = mx;
          rescale = true;
        }
        if (!first && __any_sync(0xffffffffu, rescale)) {
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
        first = false;
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        const uint64_t negm2 = pack_f2(-m_use, -m_use);
        uint64_t acc0 = 0ull, acc1 = 0ull, acc2 = 0ull, acc3 = 0ull;   // packed (0.f, 0.f)
        uint32_t pk[2][32];
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          uint64_t x0 = ffma2(pack_f2(sv[2 * c + 0], sv[2 * c + 1]), scale2, negm2);
          uint64_t x1 = ffma2(pack_f2(sv[2 * c + 2], sv[2 * c + 3]), scale2, negm2);
          uint64_t x2 = ffma2(pack_f2(sv[2 * c + 4], sv[2 * c + 5]), scale2, negm2);
          uint64_t x3 = ffma2(pack_f2(sv[2 * c + 6], sv[2 * c + 7]), scale2, negm2);
          float a0, a1, b0, b1, c0, c1, d0, d1;
          unpack_f2(x0, a0, a1);
          unpack_f2(x1, b0, b1);
          unpack_f2(x2, c0, c1);
          unpack_f2(x3, d0, d1);
          a0 = fast_exp2(a0); a1 = fast_exp2(a1);
          b0 = fast_exp2(b0); b1 = fast_exp2(b1);
          c0 = fast_exp2(c0); c1 = fast_exp2(c1);
          d0 = fast_exp2(d0); d1 = fast_exp2(d1);
          acc0 = fadd2(acc0, pack_f2(a0, a1));
          acc1 = fadd2(acc1, pack_f2(b0, b1));
          acc2 = fadd2(acc2, pack_f2(c0, c1));
          acc3 = fadd2(acc3, pack_f2(d0, d1));
          pk[c >> 5][(c & 31) + 0] = Pack2<T>::pack(a0, a1);
          pk[c >> 5][(c & 31) + 1] = Pack2<T>::pack(b0, b1);
          pk[c >> 5][(c & 31) + 2] = Pack2<T>::pack(c0, c1);
          pk[c >> 5][(c & 31) + 3] = Pack2<T>::pack(d0, d1);
        }
        {
          float lo, hi;
          unpack_f2(fadd2(fadd2(acc0, acc1), fadd2(acc2, acc3)), lo, hi);
          l += lo + hi;
        }
        if (row == 0) NLFA_TRACE_EVENT(t, 4);
        tmem_st32(s_addr, pk[0]);
        tmem_st32(s_addr + 32, pk[1]);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(P_FULL + t));
        if (row == 0) NLFA_TRACE_EVENT(t, 5);
      }
      if (!ok) break;
      if (row == 0) NLFA_TRACE_EVENT(t, 6);

      ok = mbar_wait(bar(O_FULL + t), o_count & 1, wctx, 9);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++o_count;
      tc_fence_after();
      const float inv = 1.f / l;
      T* orow = static_cast<T*>(p.o) +
                ((static_cast<long long>(w.b) * p.T + qpos) * p.H + w.h) * static_cast<long long>(D);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld32(o_addr + 32 * c, orr);
        tc_wait_ld();
        if (qpos < p.T) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v4;
            v4.x = Pack2<T>::pack(__uint_as_float(orr[8 * i + 0]) * inv, __uint_as_float(orr[8 * i + 1]) * inv);
            v4.y = Pack2<T>::pack(__uint_as_float(orr[8 * i + 2]) * inv, __uint_as_float(orr[8 * i + 3]) * inv);
            v4.z = Pack2<T>::pack(__uint_as_float(orr[8 * i + 4]) * inv, __uint_as_float(orr[8 * i + 5]) * inv);
            v4.w = Pack2<T>::pack(__uint_as_float(orr[8 * i + 6]) * inv, __uint_as_float(orr[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + 32 * c + 8 * i) = v4;
          }
        }
      }
      if (qpos < p.T)
        p.lse[(static_cast<long long>(w.b) * p.H + w.h) * p.T + qpos] = (m_ref + log2f(l)) * kLn2;
      if (row == 0) NLFA_TRACE_EVENT(t, 7);
      // the next unit's first PV product overwrites O_t: it is only issued after this
      // thread's next P arrival, which follows these loads in program order
      tc_fence_before();
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

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

template <typename T, int D, int NT, int STAGES, int QBUF>
int launch_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
             void* o, float* lse, unsigned* status, cudaStream_t stream) {
  using L = FwdSmem<D, NT, STAGES, QBUF>;
  auto kern = fwd_tc_kernel<T, D, NT, STAGES, QBUF>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) !=
      cudaSuccess)
    return NLFA_ERR_CUDA;
  FwdParams fp;
  fp.T = p.T;
  fp.H = p.H;
  fp.Hkv = p.Hkv;
  fp.window = p.window;
  fp.sinks = p.sinks;
  fp.n_tiles = (p.T + kTile - 1) / kTile;
  fp.n_units = (fp.n_tiles + NT - 1) / NT;
  fp.total_units = fp.n_units * p.B * p.H;
  fp.scale_log2 = p.scale * kLog2e;
  fp.o = o;
  fp.lse = lse;
  fp.status = status;
  const int grid = fp.total_units < sm_count() ? fp.total_units : sm_count();
  kern<<<grid, NT * 128 + 64, L::kDynamic, stream>>>(mq, mk, mv, fp);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace

int launch_fwd_tc(const Problem& p, const void* q, const void* k, const void* v, void* o,
                  float* lse, unsigned* status, cudaStream_t stream) {
  if (p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (p.D != 64 && p.D != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  if (!(p.scale > 0.f)) return NLFA_ERR_UNSUPPORTED_PATH;     // row max is taken before scaling
  CUtensorMap mq, mk, mv;
  int st = make_tile_map(&mq, q, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mk, k, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mv, v, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st != NLFA_OK) return st;
  const bool bf16 = p.dtype == NLFA_DTYPE_BF16;
  if (p.D == 64) {
    return bf16 ? launch_t<__nv_bfloat16, 64, 2, 3, 2>(p, mq, mk, mv, o, lse, status, stream)
                : launch_t<__half, 64, 2, 3, 2>(p, mq, mk, mv, o, lse, status, stream);
  }
  return bf16 ? launch_t<__nv_bfloat16, 128, 2, 2, 1>(p, mq, mk, mv, o, lse, status, stream)
              : launch_t<__half, 128, 2, 2, 1>(p, mq, mk, mv, o, lse, status, stream);
}

#ifdef NLFA_TRACE
extern "C" int nlfa_trace_read(long long* events, int* counts) {
  int zero[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return NLFA_ERR_CUDA;
  if (cudaMemcpyFromSymbol(events, g_trace, sizeof(long long) * 4 * 1024) != cudaSuccess ||
      cudaMemcpyFromSymbol(counts, g_trace_n, sizeof(int) * 4) != cudaSuccess ||
      cudaMemcpyToSymbol(g_trace_n, zero, sizeof(zero)) != cudaSuccess)
    return NLFA_ERR_CUDA;
  return NLFA_OK;
}
#endif

}  // namespace nlfa
