// Tensor-core forward for sm_100a: S = Q K^T and O += P V on tcgen05 with the
// accumulators in TMEM, tiles brought in by TMA, online softmax in registers.
//
// Persistent kernel: one CTA per SM takes work units from a global counter,
// heaviest first.  A unit is NT consecutive 128-row query tiles of one (batch,
// head); the CTA visits the key blocks those tiles can see.  Warp roles:
//   warps [0, 4 NT)   softmax: warpgroup t owns query tile t, one thread per row
//   warp  4 NT        scheduler + TMA producer (one lane): Q per unit, K / V ring
//   warp  4 NT + 1    MMA issuer (one lane) and owner of the TMEM allocation
// Hand-offs are mbarriers whose phases run on across units: Q full/empty per Q
// buffer, K/V full/empty per stage, and per tile S ready, S consumed, P ready, O
// ready.  While the softmax warps finish a unit (normalise and store O) the
// producer and the MMA issuer are already on the next one.
//
// TMEM columns: S_t at 128 t (fp32, 128 columns), O_t at 128 NT + D t.  P_t (16
// bit, the A operand of the PV product) has its own 64 columns after the O tiles
// when they fit (D = 64); the next S product is then issued as soon as the softmax
// warps have pulled S into registers, so the tensor pipe runs under the
// exponentials.  Otherwise (D = 128) P_t overwrites the first 64 columns of S_t.
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
  int block;              // > 0: block-causal mask of this many positions (window == 0)
  int n_tiles;            // ceil(T / 128)
  int n_units;            // ceil(n_tiles / NT)
  int total_units;        // n_units * B * H
  float scale_log2;       // scale * log2(e), > 0
  void* o;
  float* lse;
  unsigned* status;
  unsigned* sched;        // this launch's two counters
};

template <int D, int NT, int STAGES, int QBUF>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;          // one 128 x D 16-bit tile
  static constexpr int kQ = 0;                              // [QBUF][NT] tiles
  static constexpr int kK = kQ + QBUF * NT * kTileBytes;
  static constexpr int kV = kK + STAGES * kTileBytes;
  static constexpr int kBar = kV + STAGES * kTileBytes;
  // barriers (8 bytes each): q_full[QBUF], q_empty[QBUF], s_full[NT], s_consumed[NT],
  // p_full[NT], o_ready[NT], k_full[S], k_empty[S], v_full[S], v_empty[S], sched_full[kRing]
  static constexpr int kRing = 8;
  // ..., group[NT]
  static constexpr int kNumBars = 2 * QBUF + 4 * NT + 4 * STAGES + kRing + NT;
  static constexpr int kSched = (kBar + 8 * kNumBars + 15) / 16 * 16;   // ring of unit descriptors (16 ints each)
  static constexpr int kTmemSlot = kSched + 64 * kRing;
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
    w.tr[t] = tile_range(w.tile0 + t, p.window, p.sinks, p.block, p.n_tiles);
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
__global__ void __launch_bounds__(NT * 128 + 128, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
              const FwdParams p) {
  using L = FwdSmem<D, NT, STAGES, QBUF>;
  constexpr int kBoxes = D / 64;                 // 64-element column boxes per tile
  constexpr int kBoxBytes = kTile * 128;         // 128 rows x 128 bytes
  constexpr uint32_t kTmemCols = (NT * (128 + D) <= 256) ? 256u : 512u;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr bool kSepP = NT * (128 + D + 64) <= 512;      // P has columns of its own
  constexpr uint32_t kPBase = NT * (128 + D);
  constexpr int kRing = L::kRing;
  constexpr int kRegsLaunch = 168, kRegsCompute = 216, kRegsOther = 72;   // per thread

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  auto bar = [&](int i) -> uint32_t { return base + L::kBar + 8u * i; };
  constexpr int Q_FULL = 0, Q_EMPTY = QBUF, S_FULL = 2 * QBUF, S_CONSUMED = S_FULL + NT,
                P_FULL = S_CONSUMED + NT, O_READY = P_FULL + NT, K_FULL = O_READY + NT,
                K_EMPTY = K_FULL + STAGES, V_FULL = K_EMPTY + STAGES, V_EMPTY = V_FULL + STAGES,
                SCHED_FULL = V_EMPTY + STAGES, GROUP = SCHED_FULL + kRing;
  volatile int* sched_ring = reinterpret_cast<volatile int*>(gen + L::kSched);
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
      mbar_init(bar(Q_EMPTY + i), 1 + NT);   // the MMA issuer's commit + one arrival per tile's store
    }
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar(S_FULL + t), 1);
      mbar_init(bar(S_CONSUMED + t), 128);
      mbar_init(bar(P_FULL + t), 128);
      mbar_init(bar(O_READY + t), 1);
      mbar_init(bar(GROUP + t), 128);
    }
    for (int i = 0; i < kRing; ++i) mbar_init(bar(SCHED_FULL + i), 1);
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
  // Everything above touched only this CTA's own state and may have run while the stream's
  // previous kernel was finishing; from here on its results are read.
  grid_dep_wait();
  grid_dep_release();

  // Every role reads the index of its uc-th unit from the ring the producer fills;
  // a negative index means there is no more work.
  // The producer works the descriptor out once (several integer divisions) and publishes all
  // of it: {u, b, h, hk, tile0, lo, extra_sinks, n_iters, n_valid, valid mask, tr[0], tr[1]}.
  static_assert(NT <= 2, "the published unit descriptor holds two tile ranges");
  auto next_unit = [&](int uc, bool& ok, Unit<NT>& w) -> int {
    ok = mbar_wait(bar(SCHED_FULL + (uc % kRing)), (uc / kRing) & 1, wctx, 11);
    if (!ok) return -1;
    const int4* e = reinterpret_cast<const int4*>(const_cast<const int*>(sched_ring) + 16 * (uc % kRing));
    const int4 a = e[0], b = e[1], c = e[2], d = e[3];
    w.b = a.y; w.h = a.z; w.hk = a.w;
    w.tile0 = b.x; w.lo = b.y; w.extra_sinks = b.z; w.n_iters = b.w;
    w.n_valid = c.x;
    w.valid[0] = (c.y & 1) != 0;
    w.tr[0].lo = c.z; w.tr[0].hi = c.w; w.tr[0].sink_blocks = d.x;
    if (NT > 1) {
      w.valid[NT - 1] = (c.y & 2) != 0;
      w.tr[NT - 1].lo = d.y; w.tr[NT - 1].hi = d.z; w.tr[NT - 1].sink_blocks = d.w;
    }
    return a.x;
  };

  // Register reallocation (NT = 2: 384 threads launch with 168 registers each): the
  // warpgroup of the producer, the MMA issuer and two spare warps drops to 72, the softmax
  // warpgroups take 216 each.
  if (warp >= 4 * NT) {
  if (NT == 2) setmaxnreg_dec<kRegsOther>();
  // setmaxnreg.inc blocks until the registers it asks for have been released, so the four
  // warps that shrink must free at least what the eight that grow take.
  static_assert((kRegsLaunch - kRegsOther) * 4 >= (kRegsCompute - kRegsLaunch) * 8,
                "register reallocation does not balance");
  if (dead || warp >= 4 * NT + 2) {
    // nothing to do (spare warps only complete the warpgroup)
  } else if (warp == 4 * NT) {
    // =============================== TMA producer ============================
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      int git = 0;
      bool ok = true;
      // Takes the uc-th unit of this CTA from the global counter, publishes it to the other
      // roles and starts the loads of its Q tiles.  Returns the unit (-1: none left).
      auto fetch_unit = [&](int uc) -> int {
        int u = static_cast<int>(atomicAdd(&p.sched[0], 1u));
        if (u >= p.total_units) u = -1;
        Unit<NT> w{};
        if (u >= 0) w = make_unit<NT>(u, p, BH);
        volatile int* e = sched_ring + 16 * (uc % kRing);
        e[0] = u; e[1] = w.b; e[2] = w.h; e[3] = w.hk;
        e[4] = w.tile0; e[5] = w.lo; e[6] = w.extra_sinks; e[7] = w.n_iters;
        e[8] = w.n_valid; e[9] = (w.valid[0] ? 1 : 0) | (w.valid[NT - 1] ? 2 : 0);
        e[10] = w.tr[0].lo; e[11] = w.tr[0].hi; e[12] = w.tr[0].sink_blocks;
        e[13] = w.tr[NT - 1].lo; e[14] = w.tr[NT - 1].hi; e[15] = w.tr[NT - 1].sink_blocks;
        mbar_arrive(bar(SCHED_FULL + (uc % kRing)));
        if (u < 0) return u;
        const int qb = uc % QBUF;
        const uint32_t qph = (uc / QBUF) & 1;
        if (!(ok = mbar_wait(bar(Q_EMPTY + qb), qph ^ 1, wctx, 10))) return u;
        mbar_arrive_expect_tx(bar(Q_FULL + qb), w.n_valid * L::kTileBytes);
        for (int t = 0; t < NT; ++t) {
          if (!w.valid[t]) continue;
          for (int x = 0; x < kBoxes; ++x)
            tma_load_4d(base + L::kQ + (qb * NT + t) * L::kTileBytes + x * kBoxBytes, &tm_q,
                        bar(Q_FULL + qb), 64 * x, w.h, (w.tile0 + t) * kTile, w.b);
        }
        return u;
      };
      int u = fetch_unit(0);
      for (int uc = 0; ok && u >= 0; ++uc) {
        Unit<NT> w;
        next_unit(uc, ok, w);                    // published by this thread: never waits
        if (!ok) break;
        // the next unit's Q is requested once this unit's first K/V blocks are on their way
        // (with a single Q buffer: only when this unit has released it)
        int u_next = -2;
        const int prefetch_at = QBUF > 1 ? (w.n_iters < STAGES ? w.n_iters : STAGES) : w.n_iters;
        for (int it = 0; it < w.n_iters; ++it, ++git) {
          if (it == prefetch_at) u_next = fetch_unit(uc + 1);
          if (!ok) break;
          const int s = git % STAGES;
          const uint32_t ph = (git / STAGES) & 1;
          const int j = w.block_at(it);
          if (!(ok = mbar_wait(bar(K_EMPTY + s), ph ^ 1, wctx, 1))) break;
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
        if (ok && u_next == -2) u_next = fetch_unit(uc + 1);
        u = u_next;
      }
    }
  } else if (warp == 4 * NT + 1) {
    // ================================ MMA issuer =============================
    // The whole warp runs this loop and waits on every barrier together; `leader` marks the one
    // lane that issues.  All values that feed a descriptor are made provably warp-uniform.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
      auto wait_all = [&](uint32_t b, uint32_t parity, unsigned where) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(b, parity, wctx, where));
      };
      constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, D, false, true);

      auto issue_s = [&](int qb, int t, int s) {
        const uint32_t qa = base + L::kQ + (qb * NT + t) * L::kTileBytes;
        const uint32_t ka = base + L::kK + s * L::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          umma_ss(leader, tmem + 128 * t, make_smem_desc(qa + off, 16, 1024),
                 make_smem_desc(ka + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, int s, bool accumulate) {
        const uint32_t va = base + L::kV + s * L::kTileBytes;
        const uint32_t pa = kSepP ? kPBase + 64 * t : 128 * t;
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          // 16 keys per step: 8 packed TMEM columns of P, 16 rows (2048 bytes) of V
          umma_ts(leader, tmem + 128 * NT + D * t, tmem + pa + 8 * kk,
                 make_smem_desc(va + kk * 2048, kBoxBytes, 1024), idesc_pv,
                 (accumulate || kk > 0) ? 1u : 0u);
        }
      };

      bool ok = true;
      int git = 0;
      int p_count[NT], s_issued[NT];
      for (int t = 0; t < NT; ++t) p_count[t] = s_issued[t] = 0;
      // S_t may be overwritten once the softmax warps have pulled the previous one into
      // registers (only needed when P has its own columns; otherwise the P hand-off implies it)
      auto start_s = [&](int qb, int t, int s) {
        if (kSepP && s_issued[t] > 0)
          ok = wait_all(bar(S_CONSUMED + t), (s_issued[t] - 1) & 1, 12);
        if (!ok) return;
        tc_fence_after();
        issue_s(qb, t, s);
        umma_commit(leader, bar(S_FULL + t));
        ++s_issued[t];
      };
      // A warp-uniform copy of the uc-th unit's published descriptor.
      auto get_unit = [&](int uc, Unit<NT>& w) -> int {
        const int u = __shfl_sync(0xffffffffu, next_unit(uc, ok, w), 0);
        ok = __all_sync(0xffffffffu, ok);
        w.lo = __shfl_sync(0xffffffffu, w.lo, 0);
        w.extra_sinks = __shfl_sync(0xffffffffu, w.extra_sinks, 0);
        w.n_iters = __shfl_sync(0xffffffffu, w.n_iters, 0);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          w.valid[t] = __shfl_sync(0xffffffffu, w.valid[t] ? 1 : 0, 0) != 0;
          w.tr[t].lo = __shfl_sync(0xffffffffu, w.tr[t].lo, 0);
          w.tr[t].hi = __shfl_sync(0xffffffffu, w.tr[t].hi, 0);
          w.tr[t].sink_blocks = __shfl_sync(0xffffffffu, w.tr[t].sink_blocks, 0);
        }
        return u;
      };
      // A unit's first S products, in three steps so that they can be slotted into the end of
      // the previous unit: wait for its Q tiles and first K block; one tile's product; release.
      // `g0` is the global index of the unit's first key block.
      auto pro_wait = [&](int uc, int g0) {
        ok = wait_all(bar(Q_FULL + uc % QBUF), (uc / QBUF) & 1, 3);
        if (ok) ok = wait_all(bar(K_FULL + g0 % STAGES), (g0 / STAGES) & 1, 4);
      };
      auto pro_s = [&](const Unit<NT>& w, int uc, int g0, int t) {
        if (ok && w.sees(t, w.block_at(0))) start_s(uc % QBUF, t, g0 % STAGES);
      };
      auto pro_done = [&](int g0) {
        if (ok) umma_commit(leader, bar(K_EMPTY + g0 % STAGES));
      };
      // With two Q buffers and P in its own columns, the next unit's first S products are
      // issued during this unit's last key block.  Otherwise the first tile of a causal pair,
      // which sees one block fewer than the second, would idle for a whole block at the end of
      // every unit, waiting for the issuer to get through the second tile's last block.
      constexpr bool kEarlyPro = kSepP && NT == 2 && QBUF > 1;
      Unit<NT> w;
      int u = get_unit(0, w);
      if (ok && u >= 0) {
        pro_wait(0, git);
        for (int t = 0; t < NT; ++t) pro_s(w, 0, git, t);
        pro_done(git);
      }
      for (int uc = 0; ok && u >= 0; ++uc) {
        const int qb = uc % QBUF;
        Unit<NT> wn;
        int un = -2;                                  // next unit: not looked at yet
        bool o_started[NT];
        for (int t = 0; t < NT; ++t) o_started[t] = false;
        auto do_pv = [&](int t, int stage) {
          if (!(ok = wait_all(bar(P_FULL + t), p_count[t] & 1, 7))) return;
          ++p_count[t];
          tc_fence_after();
          issue_pv(t, stage, o_started[t]);
          umma_commit(leader, bar(O_READY + t));
          o_started[t] = true;
        };
        if (kSepP && NT == 2) {
          // Two tiles, P in its own columns.  The issue order per key block is
          //   S_1(next), PV_0(previous), S_0(next), PV_1(this)
          // so the first tile's products trail the second tile's by half a step.  That lets the
          // two softmax warpgroups run out of phase -- one in its exponentials while the other
          // loads, reduces and stores -- instead of contending for the exponential unit together.
          for (int it = 0; ok && it < w.n_iters; ++it, ++git) {
            const int s = git % STAGES;
            const uint32_t ph = (git / STAGES) & 1;
            const int j = w.block_at(it);
            const bool have_next = it + 1 < w.n_iters;
            const int s1 = (git + 1) % STAGES;
            const uint32_t ph1 = ((git + 1) / STAGES) & 1;
            const int j1 = have_next ? w.block_at(it + 1) : 0;
            const int sp = (git + STAGES - 1) % STAGES;              // stage of the previous block
            if (have_next && !(ok = wait_all(bar(K_FULL + s1), ph1, 6))) break;
            if (have_next && w.sees(1, j1)) start_s(qb, 1, s1);
            if (!ok) break;
            if (kEarlyPro && !have_next) {
              un = get_unit(uc + 1, wn);
              if (ok && un >= 0) {
                pro_wait(uc + 1, git + 1);
                pro_s(wn, uc + 1, git + 1, 0);
              }
              if (!ok) break;
            }
            if (it > 0) {
              if (w.sees(0, w.block_at(it - 1))) do_pv(0, sp);
              if (!ok) break;
              umma_commit(leader, bar(V_EMPTY + sp));                          // both tiles are done with it
            }
            if (have_next && w.sees(0, j1)) start_s(qb, 0, s1);
            if (!ok) break;
            if (have_next) umma_commit(leader, bar(K_EMPTY + s1));
            if (kEarlyPro && !have_next && un >= 0) {
              pro_s(wn, uc + 1, git + 1, 1);
              pro_done(git + 1);
              if (!ok) break;
            }
            if (!(ok = wait_all(bar(V_FULL + s), ph, 5))) break;
            if (w.sees(1, j)) do_pv(1, s);
          }
          if (ok) {
            const int sl = (git + STAGES - 1) % STAGES;              // the unit's last block
            if (w.sees(0, w.block_at(w.n_iters - 1))) do_pv(0, sl);
            if (ok) umma_commit(leader, bar(V_EMPTY + sl));
          }
        } else {
          for (int it = 0; ok && it < w.n_iters; ++it, ++git) {
            const int s = git % STAGES;
            const uint32_t ph = (git / STAGES) & 1;
            const int j = w.block_at(it);
            const bool have_next = it + 1 < w.n_iters;
            const int s1 = (git + 1) % STAGES;
            const uint32_t ph1 = ((git + 1) / STAGES) & 1;
            const int j1 = have_next ? w.block_at(it + 1) : 0;
            if (have_next && !(ok = wait_all(bar(K_FULL + s1), ph1, 6))) break;
            if (kSepP && have_next) {
              // next S products first: they only wait for the softmax warps' loads of S
              for (int t = 0; ok && t < NT; ++t)
                if (w.sees(t, j1)) start_s(qb, t, s1);
              if (!ok) break;
              umma_commit(leader, bar(K_EMPTY + s1));
            }
            if (!(ok = wait_all(bar(V_FULL + s), ph, 5))) break;
            for (int t = 0; ok && t < NT; ++t) {
              if (w.sees(t, j)) do_pv(t, s);
              if (ok && !kSepP && have_next && w.sees(t, j1)) start_s(qb, t, s1);
            }
            if (!ok) break;
            umma_commit(leader, bar(V_EMPTY + s));
            if (!kSepP && have_next) umma_commit(leader, bar(K_EMPTY + s1));
          }
        }
        if (!ok) break;
        umma_commit(leader, bar(Q_EMPTY + qb));
        if (un == -2) {
          un = get_unit(uc + 1, wn);
          if (ok && un >= 0) {
            pro_wait(uc + 1, git);
            for (int t = 0; t < NT; ++t) pro_s(wn, uc + 1, git, t);
            pro_done(git);
          }
        }
        u = un;
        w = wn;
      }
    }
  }
  } else {
    // ================================= softmax ===============================
    if (NT == 2) setmaxnreg_inc<kRegsCompute>();
    if (!dead) {
    const int t = warp >> 2;                       // query tile of this warpgroup
    const int row = threadIdx.x - 128 * t;         // row inside the tile == TMEM lane
    const uint32_t lane_base = 32u * (warp & 3);
    const uint32_t s_addr = tmem_addr(tmem, lane_base, 128 * t);
    const uint32_t o_addr = tmem_addr(tmem, lane_base, 128 * NT + D * t);
    const uint32_t p_addr = tmem_addr(tmem, lane_base, kSepP ? kPBase + 64 * t : 128 * t);
    const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);
    int s_count = 0, o_count = 0;      // S_FULL / O_READY phases this thread has observed
    uint32_t group_phase = 0;          // uses of this warpgroup's barrier (GROUP + t)
    // With two Q buffers the thread that issued a tile's TMA store does not wait for it on the
    // spot (that would hold up its whole warpgroup); it releases the buffer one block later,
    // when the store has long finished reading shared memory.
    int pending_qb = -1;
    auto release_pending = [&]() {
      if (pending_qb >= 0) {
        tma_store_wait_read();
        mbar_arrive(bar(Q_EMPTY + pending_qb));
        pending_qb = -1;
      }
    };
    bool ok = true;
    for (int uc = 0; ok; ++uc) {
      Unit<NT> w;
      const int u = next_unit(uc, ok, w);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok || u < 0) break;
      if (!w.valid[t]) {
        if (row == 0) {
          release_pending();
          mbar_arrive(bar(Q_EMPTY + (uc % QBUF)));                // nothing to store for this tile
        }
        continue;
      }
      const int tile = w.tile0 + t;
      const int qpos = tile * kTile + row;
      const int qlim = last_key_of_query(qpos, p.block, p.T);     // last key this row sees (plain causal: itself)
      // Online softmax in base 2.  m_ref is the reference exponent (scaled units): P =
      // 2^(x - m_ref).  It starts at the first block's row maximum and is afterwards only
      // raised (with O and l rescaled) when a block's maximum exceeds it by more than 2^8,
      // which keeps P within 16-bit range and makes the TMEM round trip of O rare.
      float m_ref = -INFINITY, l = 0.f;
      bool first = true;
      // keys this row can see: [va, qpos] plus the sink prefix [0, vsink)
      int va = 0, vsink = 0;
      if (p.window > 0) {
        const int lo = qpos - (p.window - p.sinks) + 1;
        va = lo > 0 ? lo : 0;
        vsink = p.sinks < qpos + 1 ? p.sinks : qpos + 1;
      }
      const unsigned vw = static_cast<unsigned>(qpos - va);
      for (int it = 0; it < w.n_iters; ++it) {
        const int j = w.block_at(it);
        if (!tile_sees_block(w.tr[t], j)) continue;
        ok = mbar_wait(bar(S_FULL + t), s_count & 1, wctx, 8);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_count;
        tc_fence_after();

        // the whole row of S into registers; from then on S_t belongs to the MMA issuer again
        uint32_t sv[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + 32 * c, sv[c]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(bar(S_CONSUMED + t));

        // Boundary blocks: a 32-column chunk that the whole warp sees entirely is left alone,
        // the others pay per-element tests.  Masked scores
        // become -inf and flow through the straight-line code below as zeros: skipping them
        // instead would put branches between the chunks, and the exponentials of a chunk on
        // its own are too few to cover the unit's latency (measured: 1760 clocks per row with
        // per-chunk branches against 1130 without).
        const int k0 = j * kTile;
        const int edges = block_fully_visible(tile, j, p.window, p.sinks, p.block, p.T)
                              ? -1 : block_edges(tile, j, p.window, p.sinks);
        if (edges == EDGE_CAUSAL) {
          // only the causal edge cuts the block: the row sees the columns up to its own
          // position (block-causal: up to the end of its block) -- one compare per element
          // against a per-thread limit
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int last = qlim - (k0 + 32 * c);                       // last visible column of the chunk
            if (__all_sync(0xffffffffu, last >= 31)) continue;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i > last) sv[c][i] = __float_as_uint(-INFINITY);
          }
        } else if (edges == EDGE_WINDOW) {
          // only the window's lower edge cuts the block: the row sees the columns from va on
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int first_vis = va - (k0 + 32 * c);                    // first visible column of the chunk
            if (__all_sync(0xffffffffu, first_vis <= 0)) continue;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < first_vis) sv[c][i] = __float_as_uint(-INFINITY);
          }
        } else if (edges == EDGE_BOTH) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int x0 = k0 + 32 * c, x1 = x0 + 31;
            const bool in = (x0 >= va && x1 <= qpos) || x1 < vsink;
            if (__all_sync(0xffffffffu, in)) continue;
            const unsigned o = static_cast<unsigned>(x0 - va);            // wraps below va
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (!(o + static_cast<unsigned>(i) <= vw || x0 + i < vsink))
                sv[c][i] = __float_as_uint(-INFINITY);
          }
        }
        // row maximum of the raw scores: two chains of 3-input max
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

        float alpha = 1.f;
        bool rescale = false;
        if (first) {
          m_ref = mx;
        } else if (mx > m_ref + 8.f) {
          alpha = fast_exp2(m_ref - mx);       // m_ref == -inf gives 0
          m_ref = mx;
          rescale = true;
          l *= alpha;
        }

        // all exponentials of the row first (P stays in registers) ...
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        const uint64_t negm2 = pack_f2(-m_use, -m_use);
        uint64_t acc0 = 0ull, acc1 = 0ull;              // packed (0.f, 0.f)
        uint32_t pk[4][16];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float e0, e1, e2, e3;
            unpack_f2(ffma2(pack_f2(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])),
                            scale2, negm2), e0, e1);
            unpack_f2(ffma2(pack_f2(__uint_as_float(sv[c][i + 2]), __uint_as_float(sv[c][i + 3])),
                            scale2, negm2), e2, e3);
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
        // ... and only then the hand-off that needs the previous block's PV product to be
        // complete (O may be rescaled, P's columns may be overwritten); by now it long is.
        // Every O_READY phase is observed exactly once, in order.
        if (!first) {
          ok = mbar_wait(bar(O_READY + t), o_count & 1, wctx, 13);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ++o_count;
          tc_fence_after();
          if (__any_sync(0xffffffffu, rescale)) {
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
        }
        first = false;
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_st16(p_addr + 16 * c, pk[c]);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(P_FULL + t));
        if (QBUF > 1 && row == 0) release_pending();
      }
      if (!ok) break;

      ok = mbar_wait(bar(O_READY + t), o_count & 1, wctx, 9);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++o_count;
      tc_fence_after();
      // The unit's Q tile is dead (every S product that read it has completed), so its shared
      // memory stages the normalised O tile, in the swizzled layout of the loads, for one
      // coalesced TMA store per 64-column box.
      const float inv = 1.f / l;
      const uint32_t stage = base + L::kQ + ((uc % QBUF) * NT + t) * L::kTileBytes;
      const uint32_t sw = static_cast<uint32_t>(row & 7);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t orr[32];
        tmem_ld32(o_addr + 32 * c, orr);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = 32 * c + 8 * i;                       // first of 8 columns = one 16 B chunk
          const uint32_t addr = stage + static_cast<uint32_t>(col >> 6) * kBoxBytes +
                                static_cast<uint32_t>(row) * 128u +
                                ((static_cast<uint32_t>((col & 63) >> 3) ^ sw) << 4);
          st_shared_v4(addr,
                       Pack2<T>::pack(__uint_as_float(orr[8 * i + 0]) * inv, __uint_as_float(orr[8 * i + 1]) * inv),
                       Pack2<T>::pack(__uint_as_float(orr[8 * i + 2]) * inv, __uint_as_float(orr[8 * i + 3]) * inv),
                       Pack2<T>::pack(__uint_as_float(orr[8 * i + 4]) * inv, __uint_as_float(orr[8 * i + 5]) * inv),
                       Pack2<T>::pack(__uint_as_float(orr[8 * i + 6]) * inv, __uint_as_float(orr[8 * i + 7]) * inv));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      // the warpgroup's four warps meet on an mbarrier, so that this wait is bounded like every
      // other: its result is false once anything in the CTA has given up, and then whole warps leave
      mbar_arrive(bar(GROUP + t));
      ok = mbar_wait(bar(GROUP + t), group_phase & 1u, wctx, 14);
      ++group_phase;
      ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
      if (!ok) break;
      if (row == 0) {
        for (int x = 0; x < kBoxes; ++x)
          tma_store_4d(&tm_o, stage + x * kBoxBytes, 64 * x, w.h, tile * kTile, w.b);
        tma_store_commit();
        if (QBUF > 1) {
          pending_qb = uc % QBUF;                               // released after the next block
        } else {
          tma_store_wait_read();
          mbar_arrive(bar(Q_EMPTY + (uc % QBUF)));              // this tile's share of the buffer
        }
      }
      if (qpos < p.T)
        p.lse[(static_cast<long long>(w.b) * p.H + w.h) * p.T + qpos] = (m_ref + log2f(l)) * kLn2;
      // the next unit's first PV product overwrites O_t: it is only issued after this
      // thread's next P arrival, which follows these loads in program order
      tc_fence_before();
    }
    if (row == 0) release_pending();
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
  // scheduler bookkeeping: the last CTA of the launch to get here re-arms the counters
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned done = atomicAdd(&p.sched[1], 1u);
    if (done == gridDim.x - 1) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
      __threadfence();
    }
  }
}

template <typename T, int D, int NT, int STAGES, int QBUF>
int launch_t(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
             const CUtensorMap& mo, void* o, float* lse, unsigned* status, cudaStream_t stream) {
  using L = FwdSmem<D, NT, STAGES, QBUF>;
  auto kern = fwd_tc_kernel<T, D, NT, STAGES, QBUF>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kDynamic) != NLFA_OK)
    return NLFA_ERR_CUDA;
  FwdParams fp;
  fp.T = p.T;
  fp.H = p.H;
  fp.Hkv = p.Hkv;
  fp.window = p.window;
  fp.sinks = p.sinks;
  fp.block = p.block;
  fp.n_tiles = (p.T + kTile - 1) / kTile;
  fp.n_units = (fp.n_tiles + NT - 1) / NT;
  fp.total_units = fp.n_units * p.B * p.H;
  fp.scale_log2 = p.scale * kLog2e;
  fp.o = o;
  fp.lse = lse;
  fp.status = status;
  const int sst = sched_counters(stream, &fp.sched);
  if (sst != NLFA_OK) return sst;
  const int grid = fp.total_units < sm_count() ? fp.total_units : sm_count();
  if (launch_kernel(kern, dim3(grid), dim3(NT * 128 + 128), L::kDynamic, stream, overlap_launches(kOverlapFwd), mq, mk, mv, mo,
                    fp) != cudaSuccess) {
    (void)cudaGetLastError();
    return NLFA_ERR_CUDA;
  }
  return NLFA_OK;
}

}  // namespace

int launch_fwd_tc(const Problem& p, const void* q, const void* k, const void* v, void* o,
                  float* lse, unsigned* status, cudaStream_t stream) {
  if (p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (p.D != 32 && p.D != 64 && p.D != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  // Head dim 32 runs the 64-wide kernels: the tensor maps describe the real 32 columns, the
  // TMA boxes are 64 wide, so loads fill columns 32-63 with zeros (which add nothing to any
  // product) and stores drop them.
  if (!(p.scale > 0.f)) return NLFA_ERR_UNSUPPORTED_PATH;     // row max is taken before scaling
  CUtensorMap mq, mk, mv, mo;
  int st = make_tile_map(&mq, q, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mk, k, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mv, v, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mo, o, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st != NLFA_OK) return st;
  const bool bf16 = p.dtype == NLFA_DTYPE_BF16;
  if (p.D <= 64) {
    return bf16 ? launch_t<__nv_bfloat16, 64, 2, 3, 2>(p, mq, mk, mv, mo, o, lse, status, stream)
                : launch_t<__half, 64, 2, 3, 2>(p, mq, mk, mv, mo, o, lse, status, stream);
  }
  return bf16 ? launch_t<__nv_bfloat16, 128, 2, 2, 1>(p, mq, mk, mv, mo, o, lse, status, stream)
              : launch_t<__half, 128, 2, 2, 1>(p, mq, mk, mv, mo, o, lse, status, stream);
}


}  // namespace nlfa
