// Tensor-core backward for sm_100a: the dQ pass and the dK/dV pass, both as one
// kernel template.  Like the reference's backward (nanolab/csrc/flash_attn_cuda.cu
// :806-971 dQ, :983-1191 dK/dV) the two passes are independent, each recomputes
// P from the taped logsumexp, and neither uses atomics, so gradients are
// bit-reproducible.  Delta = rowsum(dO * O) is produced first by a separate
// streaming kernel (:1234-1262).
//
// A CTA keeps two "stationary" 128 x D tiles in shared memory and streams pairs
// of tiles past them:
//
//   dQ pass    stationary (Q_i, dO_i), streamed (K_j, V_j)
//              T0 = Q K^T, T1 = dO V^T           rows = queries, columns = keys
//              dS = P (T1 - Delta_row),  dQ += dS K_j
//   dK/dV pass stationary (K_j, V_j), streamed (Q_i, dO_i) over the GQA group
//              T0 = K Q^T, T1 = V dO^T           rows = keys, columns = queries
//              dV += P dO_i,  dK += dS Q_i       (P, dS are already "transposed")
//
// Persistent: one CTA per SM takes work units (one stationary tile each) from a
// global counter, heaviest first.  Warps 0-7 compute, warp 8 is the TMA producer
// and the scheduler, warp 9 issues MMAs and owns TMEM.  The MMA issuer works one
// streamed tile ahead: as soon as the compute warps have pulled T0/T1 into
// registers it issues the next tile's T0/T1 products, so the tensor pipe runs
// while the exponentials are computed; the stationary tiles are double buffered
// so the next unit's loads and first products overlap the current unit's tail.
//
// TMEM: with streamed tiles of YR rows, T0 at column 0 and T1 at YR (fp32); outputs
// accumulate at 2 YR (dQ: D columns; dV then dK: 2 D columns).  The 16-bit P / dS
// operands of the output products live in columns of their own behind the outputs.
// YR is 128 at D = 64 and 64 at D = 128, where shared memory would hold only two
// stages of 128-row tiles (one load in flight) and TMEM no separate P / dS columns.
#include <type_traits>

#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {


namespace {

enum { MODE_DQ = 0, MODE_DKV = 1, MODE_FUSED = 2 };

struct BwdParams {
  int T, H, Hkv;
  int window, sinks;
  int block;             // > 0: block-causal mask of this many positions (window == 0)
  int n_tiles;           // 128-row tiles
  int n_ytiles;          // streamed tiles (YR rows each)
  int BH;                // B * H (dQ) or B * Hkv (dK/dV)
  int total_units;       // n_tiles * BH
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  void* out0;            // dQ  | dK
  void* out1;            // --  | dV
  unsigned* status;
  unsigned* sched;       // this launch's two counters
  // fused pass only
  float* dq_acc;         // per (b, h, query tile): 128 x 64 fp32 partial sums, rows permuted (see drain)
  unsigned* dq_turn;     // per (b, h, query tile): how many key blocks have added their share
  int sched_group;       // (batch, KV head) pairs whose units are handed out together
  float* delta_out;      // dQ pass, when it also forms Delta (see kDeltaIn): where the dK/dV pass will read it
  int delta_in_pass;     // 1: this dQ launch computes Delta = rowsum(dO * O) itself, tile by tile
  int dep_wait_first;    // 1: wait for the stream's previous kernel before the first global read; 0: the
                         // previous kernel is this call's dK/dV pass, whose results this pass does not
                         // read -- it is waited for on the way out instead
};

template <int D, int STAGES, int XBUF, int YR, bool FUSED = false, bool DELTA = false>
struct BwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;              // stationary tile: 128 rows
  static constexpr int kYTileBytes = YR * D * 2;                // streamed tile: YR rows
  static constexpr int kX = 0;                                  // [XBUF] x (X0, X1)
  static constexpr int kY = kX + XBUF * 2 * kTileBytes;         // per stage: Y0, Y1
  static constexpr int kDs = kY + STAGES * 2 * kYTileBytes;     // fused pass: dS^T [128 keys][128 queries] 16-bit
  static constexpr int kO = kDs + (FUSED ? kTile * YR * 2 : 0);     // dQ pass forming Delta: the next unit's O tile
  static constexpr int kVec = kO + (DELTA ? kTileBytes : 0);        // per stage: -lse2[YR], -delta[YR]
  static constexpr int kDeltaS = kVec + STAGES * 1024;              // dQ pass forming Delta: [XBUF][128] fp32
  static constexpr int kBar = kDeltaS + (DELTA ? XBUF * 512 : 0);
  // barriers: x_full[XBUF], x_empty[XBUF], t_full, t_consumed, pd_full, out_ready,
  //           sched_full[kRing], y_full[S], y_empty[S]
  static constexpr int kRing = 8;
  //           unit_done, out_drained, dq_ready, dq_drained, group, issued[4],
  //           o_full, o_empty, delta_full[XBUF]
  static constexpr int kNumBars = 2 * XBUF + 4 + kRing + 2 * STAGES + 9 + 2 + XBUF;
  static constexpr int kSched = (kBar + 8 * kNumBars + 15) / 16 * 16;   // ring of unit descriptors (8 ints each)
  static constexpr int kTmemSlot = kSched + 32 * kRing;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTurnOk = kAbort + 4;                    // fused pass: iterations whose dQ turn has come
  static constexpr int kTotal = kTurnOk + 8;
  static constexpr int kDynamic = kTotal + 1024;
};

// One work unit: a stationary tile and the list of streamed tiles it meets.
template <int MODE>
struct BwdUnit {
  int tile, b, h, hk;          // h: first query head of the unit
  int s_lo, extra, n_inner, n_iters;

  __device__ __forceinline__ int streamed_index(int inner) const {
    return inner < extra ? inner : s_lo + (inner - extra);
  }
};

// `YR` is the height of a streamed tile (128, or 64 where shared memory is short); the streamed
// indices s_lo, extra, n_inner count tiles of that height.
template <int MODE, int YR>
__device__ __forceinline__ BwdUnit<MODE> make_bwd_unit(int u, const BwdParams& p) {
  BwdUnit<MODE> w;
  // Heaviest units first (rank = stationary tile), all (batch, head) pairs of one rank together.
  // The key-block-stationary passes do this in groups of `sched_group` (batch, KV head) pairs (one
  // per CTA of the launch), so that a head's tiles -- and in the fused pass its fp32 dQ sums -- are
  // still in L2 when its next key block comes round (dK/dV pass at B=32, H=12, T=1024: 0.145 ->
  // 0.139 ms), while a key block still starts a whole wave of units after the block below it,
  // whose dQ turns the fused pass waits for.
  int rank, bh;
  if (MODE == MODE_FUSED || p.sched_group < p.BH) {
    const int per_group = p.sched_group * p.n_tiles;
    const int g0 = (u / per_group) * p.sched_group;              // first pair of this group
    const int size = p.BH - g0 < p.sched_group ? p.BH - g0 : p.sched_group;
    const int v = u - (u / per_group) * per_group;
    rank = v / size;
    bh = g0 + (v - rank * size);
  } else {
    rank = u / p.BH;
    bh = u - rank * p.BH;
  }
  const int group = p.H / p.Hkv;
  if (MODE == MODE_DQ) {
    w.tile = p.n_tiles - 1 - rank;              // late query tiles see the most keys
    w.b = bh / p.H;
    w.h = bh - w.b * p.H;
    w.hk = w.h / group;
    // keys [lo_pos, last row of the tile], plus the sink prefix
    const int q_last = w.tile * kTile + kTile - 1;
    const int lo_pos = p.window > 0 ? w.tile * kTile - (p.window - p.sinks) + 1 : 0;
    int hi = last_key_of_query(q_last, p.block) / YR;
    hi = hi < p.n_ytiles - 1 ? hi : p.n_ytiles - 1;
    w.s_lo = lo_pos > 0 ? lo_pos / YR : 0;
    const int sink_tiles = p.window > 0 ? (p.sinks + YR - 1) / YR : 0;
    w.extra = sink_tiles < w.s_lo ? sink_tiles : w.s_lo;
    w.n_inner = w.extra + (hi - w.s_lo + 1);
    w.n_iters = w.n_inner;
  } else {
    w.tile = rank;                              // early key blocks are seen by the most queries
    w.b = bh / p.Hkv;
    w.hk = bh - w.b * p.Hkv;
    w.h = w.hk * group;
    w.s_lo = first_query_of_key(w.tile * kTile, p.block) / YR;   // first query tile that reaches the block
    const int s_hi = last_query_tile_of_block(w.tile, p.n_ytiles, YR, p.window, p.sinks);
    w.extra = 0;
    w.n_inner = s_hi - w.s_lo + 1;
    w.n_iters = w.n_inner * group;
  }
  return w;
}

// Fused pass, second step: dQ from the fp32 sums.  The sums of a tile are laid out [piece of
// four columns][row][4]; a thread takes one piece of one row, so a warp reads 512 contiguous bytes.
template <typename T>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ acc, void* __restrict__ dq, int T_len, int H, int n_tiles,
                  int d_real, float scale, long long pieces) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= pieces) return;
  const int row = static_cast<int>(i & (kTile - 1));
  const int piece = static_cast<int>((i >> 7) & 15);
  const long long slot = i >> 11;                        // (b * H + h) * n_tiles + tile
  const int tile = static_cast<int>(slot % n_tiles);
  const long long bh = slot / n_tiles;
  const int h = static_cast<int>(bh % H);
  const long long b = bh / H;
  const int qpos = tile * kTile + row;
  const int col = 4 * piece;
  if (qpos >= T_len || col >= d_real) return;
  const float4 v = __ldcs(reinterpret_cast<const float4*>(acc) + i);
  uint2 out;
  out.x = Pack2<T>::pack(v.x * scale, v.y * scale);
  out.y = Pack2<T>::pack(v.z * scale, v.w * scale);
  uint8_t* dst = static_cast<uint8_t*>(dq) + (((b * T_len + qpos) * H + h) * d_real + col) * 2;
  *reinterpret_cast<uint2*>(dst) = out;
}

// tm_x0 / tm_x1: the stationary tensors (dQ: Q, dO; dK/dV: K, V), boxes of 128 rows;
// tm_y0 / tm_y1: the streamed tensors (dQ: K, V; dK/dV: Q, dO), boxes of YR rows.
template <typename T, int D, int MODE, int STAGES, int XBUF, int YR>
__global__ void __launch_bounds__(512, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x0, const __grid_constant__ CUtensorMap tm_x1,
              const __grid_constant__ CUtensorMap tm_y0, const __grid_constant__ CUtensorMap tm_y1,
              const __grid_constant__ CUtensorMap tm_out0,
              const __grid_constant__ CUtensorMap tm_out1, const BwdParams p) {
  // The dQ pass at D = 64 (two stationary buffers: the next unit's tiles arrive during this one) can
  // form Delta = rowsum(dO * O) itself: the producer also fetches the next unit's O tile, the
  // epilogue warps -- idle except at unit boundaries -- multiply it with the dO tile that is
  // already there, hand the row sums to the compute warps through shared memory and write them
  // out for the dK/dV pass, which then runs second.  That removes the separate Delta kernel
  // (a full pass over dO and O) from the backward.  Same arithmetic, same order of additions as
  // delta_vec_kernel, so the results are bit-identical to it.
  constexpr bool kDeltaIn = MODE == MODE_DQ && XBUF == 2 && D == 64;
  using L = BwdSmem<D, STAGES, XBUF, YR, MODE == MODE_FUSED, kDeltaIn>;
  static_assert(YR == 64 || YR == 128, "streamed tiles are 64 or 128 rows");
  static_assert(MODE != MODE_FUSED || (D == 64 && YR == 128), "the fused pass exists for 64-wide tiles");
  constexpr int kBoxes = D / 64;
  constexpr int kBoxBytes = kTile * 128;          // one 64-column box of a stationary tile
  constexpr int kYBoxBytes = YR * 128;            // ... of a streamed tile
  constexpr int kCh = YR / 64;                    // 32-column chunks per compute thread
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr uint32_t kT1Col = YR;                 // T0 at column 0, T1 behind it
  constexpr uint32_t kOutCol = 2 * YR;
  constexpr bool kKeyStat = MODE != MODE_DQ;         // K, V stationary (dK/dV pass, fused pass)
  constexpr bool kFused = MODE == MODE_FUSED;        // ... and dQ formed in the same pass
  constexpr int kOutCols = MODE == MODE_DQ ? D : 2 * D;
  constexpr bool kSep = (2 * YR + kOutCols + YR) <= 512;       // room for separate P / dS columns
  constexpr uint32_t kPCol = kSep ? 2 * YR + kOutCols : 0;     // P  (dK/dV only)
  constexpr uint32_t kDsCol = kSep ? 2 * YR + kOutCols + YR / 2 : YR;
  // Fused pass: dS^T goes to shared memory (it is the A operand of dK += dS^T Q, K-major, and of
  // dQ = dS K, MN-major), and its TMEM columns hold the dQ accumulator instead.
  constexpr uint32_t kDqCol = kDsCol;
  constexpr int kRing = L::kRing;
  constexpr int kRegsLaunch = 128, kRegsCompute = 200, kRegsOther = 56;    // per thread

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  auto bar = [&](int i) -> uint32_t { return base + L::kBar + 8u * i; };
  constexpr int X_FULL = 0, X_EMPTY = XBUF, T_FULL = 2 * XBUF, T_CONSUMED = T_FULL + 1,
                PD_FULL = T_FULL + 2, OUT_READY = T_FULL + 3, SCHED_FULL = T_FULL + 4,
                Y_FULL = SCHED_FULL + kRing, Y_EMPTY = Y_FULL + STAGES,
                UNIT_DONE = Y_EMPTY + STAGES, OUT_DRAINED = UNIT_DONE + 1,
                DQ_READY = UNIT_DONE + 2, DQ_DRAINED = UNIT_DONE + 3, GROUP = UNIT_DONE + 4,
                ISSUED = UNIT_DONE + 5,          // [4]: iteration g uses ISSUED + (g & 3)
                O_FULL = ISSUED + 4, O_EMPTY = O_FULL + 1, DELTA_FULL = O_FULL + 2;   // DELTA_FULL[XBUF]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kAbort);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kTmemSlot);
  volatile int* sched_ring = reinterpret_cast<volatile int*>(gen + L::kSched);
  const WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = (*reinterpret_cast<volatile unsigned*>(p.status) != STATUS_OK) ? 1 : 0;
    for (int i = 0; i < XBUF; ++i) {
      mbar_init(bar(X_FULL + i), 1);
      mbar_init(bar(X_EMPTY + i), 2);      // the MMA issuer's commit + the epilogue's store
    }
    mbar_init(bar(T_FULL), 1);
    mbar_init(bar(T_CONSUMED), 256);
    mbar_init(bar(PD_FULL), 256);
    mbar_init(bar(OUT_READY), 1);
    mbar_init(bar(UNIT_DONE), 1);
    mbar_init(bar(OUT_DRAINED), 128);
    mbar_init(bar(DQ_READY), 1);
    mbar_init(bar(DQ_DRAINED), 128);
    mbar_init(bar(GROUP), 128);
    for (int i = 0; i < 4; ++i) mbar_init(bar(ISSUED + i), 128);
    mbar_init(bar(O_FULL), 1);
    mbar_init(bar(O_EMPTY), 4);              // one arrival per epilogue warp
    for (int i = 0; i < XBUF; ++i) mbar_init(bar(DELTA_FULL + i), 4);
    reinterpret_cast<volatile int*>(gen + L::kTurnOk)[0] = 0;      // iterations whose turn has come
    reinterpret_cast<volatile int*>(gen + L::kTurnOk)[1] = 0;      // iterations whose share has been released
    for (int i = 0; i < kRing; ++i) mbar_init(bar(SCHED_FULL + i), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(Y_FULL + s), 1);
      mbar_init(bar(Y_EMPTY + s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(base + L::kTmemSlot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool dead = *abort_flag != 0;
  // Everything above touched only this CTA's own state and may have run while the stream's
  // previous kernel was finishing; from here on its results are read.
  if (p.dep_wait_first) grid_dep_wait();
  grid_dep_release();

  // Sixteen warps: 0-7 compute, 8 scheduler + TMA producer, 9 MMA issuer, 10-11 idle, 12-15
  // epilogue (one warp per TMEM lane quarter).  The launch gives every thread 128 registers;
  // inside its role's branch each warp of the upper half drops to 56 and the compute warps
  // take 200 each.

  // Every role reads the unit index of its uc-th unit from the ring the producer
  // fills; a negative index means there is no more work.
  // The producer works the descriptor out once (it takes several integer divisions) and
  // publishes all of it: {u, tile, b, h, hk, s_lo, n_inner, extra (dQ) | n_iters (dK/dV)}.
  auto next_unit = [&](int uc, bool& ok, BwdUnit<MODE>& w) -> int {
    ok = mbar_wait(bar(SCHED_FULL + (uc % kRing)), (uc / kRing) & 1, wctx, 40);
    if (!ok) return -1;
    const int4 a = *reinterpret_cast<const int4*>(const_cast<const int*>(sched_ring) + 8 * (uc % kRing));
    const int4 b = *reinterpret_cast<const int4*>(const_cast<const int*>(sched_ring) + 8 * (uc % kRing) + 4);
    w.tile = a.y; w.b = a.z; w.h = a.w;
    w.hk = b.x; w.s_lo = b.y; w.n_inner = b.z;
    w.extra = MODE == MODE_DQ ? b.w : 0;
    w.n_iters = MODE == MODE_DQ ? b.z : b.w;
    return a.x;
  };

  if (warp >= 8) {
  setmaxnreg_dec<kRegsOther>();
  // setmaxnreg.inc blocks until the registers it asks for have been released, so the eight
  // warps that shrink must free at least what the eight that grow take.
  static_assert((kRegsLaunch - kRegsOther) * 8 >= (kRegsCompute - kRegsLaunch) * 8,
                "register reallocation does not balance");
  if (dead || ((warp == 10 || warp == 11) && (!kFused || lane != 0))) {
    // nothing to do (spare warps only complete the warpgroup)
  } else if (warp == 10 || warp == 11) {
    // ===================== fused pass: turn watcher (warp 10), releaser (warp 11) ==================
    // The dQ shares of a query tile are added to its fp32 sums in a fixed order -- ascending key
    // block, see dq_turn_of_block -- kept by a turn counter per (batch, head, query tile) in
    // global memory.  Two lanes keep the latency of that protocol off the drain warps' path:
    //  * the watcher goes through this CTA's iterations ahead of the drain warps, waits until the
    //    counter of each says that the blocks before this one have added their shares, and
    //    publishes how far it has got in shared memory;
    //  * the releaser waits until the drain warps have issued an iteration's share, makes those
    //    writes visible (the threads' arrivals on the barrier order them before this lane's
    //    fence, which is cumulative) and advances the tile's counter.  It never waits for another
    //    CTA and holds nothing back, so no cycle of waits between CTAs can form.
    // Work units are handed out in ascending key-block order (within a group of heads) and every
    // CTA of the launch is resident, so a turn only ever waits for a unit that was started earlier.
    const bool watcher = warp == 10;
    volatile int* turn_ok = reinterpret_cast<volatile int*>(gen + L::kTurnOk);
    volatile int* released = turn_ok + 1;
    bool ok = true;
    int git = 0;
    // the releaser collects up to three issued iterations before it pays for one fence
    unsigned* batch_turn[3];
    unsigned batch_value[3];
    int n_batch = 0;
    auto flush_batch = [&]() {
      if (n_batch == 0) return;
      __threadfence();
      for (int i = 0; i < n_batch; ++i) st_release_gpu(batch_turn[i], batch_value[i]);
      *released = git;                  // (git counts the iterations taken into batches so far)
      n_batch = 0;
    };
    for (int uc = 0; ok; ++uc) {
      BwdUnit<MODE> w;
      const int u = next_unit(uc, ok, w);
      if (!ok || u < 0) break;
      int inner = 0, gq = 0;
      for (int it = 0; ok && it < w.n_iters; ++it, ++inner) {
        if (inner == w.n_inner) { inner = 0; ++gq; }
        const int qt = w.s_lo + inner;
        int n_blocks;
        const int order = dq_turn_of_block(w.tile, qt, p.window, p.sinks, &n_blocks, p.block, p.n_tiles);
        unsigned* turn = p.dq_turn + (static_cast<long long>(w.b) * p.H + (w.h + gq)) * p.n_tiles + qt;
        if (watcher) {
          if (order > 0) {
            const unsigned long long t0 = globaltimer_ns();
            for (uint32_t spins = 1; ld_acquire_gpu(turn) < static_cast<unsigned>(order); ++spins) {
              __nanosleep(64);
              if ((spins & 0x3fu) == 0u) {
                if (*abort_flag) { ok = false; break; }
                if (globaltimer_ns() - t0 > wctx.limit()) {
                  *abort_flag = 1;
                  report_timeout(p.status, STATUS_WAIT_TIMEOUT | 44u);
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
          }
          __threadfence_block();                               // the acquire above before the flag below
          ++git;
          *turn_ok = git;
        } else {
          const uint32_t b = bar(ISSUED + (git & 3)), parity = (git >> 2) & 1;
          if (!mbar_try_wait(b, parity)) {
            flush_batch();                                     // nothing more to collect: release what there is
            if (!(ok = mbar_wait_idle(b, parity, wctx, 45))) break;
          }
          ++git;
          batch_turn[n_batch] = turn;
          batch_value[n_batch] = static_cast<unsigned>(order) + 1u;
          if (++n_batch == 3) flush_batch();
        }
      }
    }
    if (!watcher && ok) flush_batch();
  } else if (warp >= 12) {
    // ================================ epilogue ===============================
    // One thread per row of the unit's output tiles.  When the unit's last output product has
    // completed, the fp32 accumulators are pulled out of TMEM (which frees them for the next
    // unit at once), converted and staged in the unit's stationary tiles -- dead by then, and
    // in the swizzled layout the loads use: dQ over the Q tile, dK over K, dV over V -- and
    // written with TMA stores.  The compute warps meanwhile work on the next unit.
    const uint32_t lane_base = 32u * (warp & 3);
    const int row = 32 * (warp & 3) + lane;
    const uint32_t sw = static_cast<uint32_t>(row & 7);
    bool ok = true;
    // Fused pass: the same warps also carry every iteration's dQ share out of TMEM (below).
    int git = 0;                            // global iteration
    // Barrier among the four warps of this role, on an mbarrier so that the wait is bounded like
    // every other.  Its result is uniform within a warp and false once anything in the CTA has
    // given up (giving up raises the abort flag), so whole warps leave, never single lanes, and
    // the warps that still wait for them follow at once.
    uint32_t group_phase = 0;
    auto group_sync = [&](unsigned where) {
      mbar_arrive(bar(GROUP));
      const bool done = mbar_wait(bar(GROUP), group_phase & 1u, wctx, where);
      ++group_phase;
      ok = __all_sync(0xffffffffu, done && *abort_flag == 0);
    };
    // dQ pass forming Delta: row sums of dO * O for unit `duc` (descriptor `dw`), eight lanes per
    // row and eight elements per lane, summed exactly as delta_vec_kernel does; handed to the
    // compute warps through shared memory and written out for the dK/dV pass.
    auto form_delta = [&](int duc, const BwdUnit<MODE>& dw) {
      const int xb = duc % XBUF;
      // (sleeping waits: these warps share their schedulers with the compute warps)
      ok = mbar_wait_idle(bar(X_FULL + xb), (duc / XBUF) & 1, wctx, 47);   // the dO tile
      if (ok) ok = mbar_wait_idle(bar(O_FULL), duc & 1, wctx, 48);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      const uint32_t do_tile = base + L::kX + xb * 2 * L::kTileBytes + L::kTileBytes;
      const uint32_t o_tile = base + L::kO;
      float* delta_s = reinterpret_cast<float*>(gen + L::kDeltaS) + xb * kTile;
      const int chunk = lane & 7;
#pragma unroll 2
      for (int step = 0; step < 8; ++step) {
        const int r = 32 * (warp & 3) + 4 * step + (lane >> 3);
        const uint32_t off = static_cast<uint32_t>(r) * 128u +
                             ((static_cast<uint32_t>(chunk) ^ static_cast<uint32_t>(r & 7)) << 4);
        uint32_t a[4], b[4];
        ld_shared_v4(do_tile + off, a[0], a[1], a[2], a[3]);
        ld_shared_v4(o_tile + off, b[0], b[1], b[2], b[3]);
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          T a2[2], b2[2];
          *reinterpret_cast<uint32_t*>(a2) = a[i];
          *reinterpret_cast<uint32_t*>(b2) = b[i];
          part = fmaf(static_cast<float>(a2[0]), static_cast<float>(b2[0]), part);
          part = fmaf(static_cast<float>(a2[1]), static_cast<float>(b2[1]), part);
        }
        part += __shfl_xor_sync(0xffffffffu, part, 4);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        const int pos = dw.tile * kTile + r;
        if (chunk == 0) {
          delta_s[r] = part;
          if (pos < p.T) p.delta_out[(static_cast<long long>(dw.b) * p.H + dw.h) * p.T + pos] = part;
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar(O_EMPTY));                 // the O buffer may be reloaded
        mbar_arrive(bar(DELTA_FULL + xb));         // the compute warps may read this unit's row sums
      }
    };
    for (int uc = 0; ok; ++uc) {
      BwdUnit<MODE> w;
      const int u = next_unit(uc, ok, w);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok || u < 0) break;
      if constexpr (kDeltaIn) {
        if (p.delta_in_pass) {
          if (uc == 0) form_delta(0, w);
          if (!ok) break;
          // The next unit's Delta, while this unit computes (its descriptor is published, and its
          // tiles are requested, a few iterations into this unit).
          BwdUnit<MODE> wn;
          ok = mbar_wait_idle(bar(SCHED_FULL + ((uc + 1) % kRing)), ((uc + 1) / kRing) & 1, wctx, 40);
          const int un = ok ? next_unit(uc + 1, ok, wn) : -1;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (un >= 0) form_delta(uc + 1, wn);
          if (!ok) break;
        }
      }
      if constexpr (kFused) {
        // dQ of query tile i is the sum over the key blocks j that see it of dS_ij K_j.  Each
        // iteration leaves one such share (128 x 64 fp32) in TMEM.  These warps pull it into
        // registers (which frees the accumulator) and add it to the tile's fp32 sums in global
        // memory with vector reductions -- or store it, if it is the tile's first share, so that
        // nothing has to be zero-filled -- once the watcher says that the tile's earlier shares
        // are in (see above; normally they have been for a long time).  The sums are laid out
        // [piece of 4 columns][row][4]: a warp's 32 rows of one piece are 512 contiguous bytes.
        volatile int* turn_ok = reinterpret_cast<volatile int*>(gen + L::kTurnOk);
        int inner = 0, gq = 0;
        for (int it = 0; it < w.n_iters; ++it, ++git, ++inner) {
          if (inner == w.n_inner) { inner = 0; ++gq; }
          const int qt = w.s_lo + inner;                       // query tile of this iteration
          int n_blocks;
          const int order = dq_turn_of_block(w.tile, qt, p.window, p.sinks, &n_blocks, p.block, p.n_tiles);
          const long long slot = (static_cast<long long>(w.b) * p.H + (w.h + gq)) * p.n_tiles + qt;
          float4* acc = reinterpret_cast<float4*>(p.dq_acc + slot * (kTile * D)) + row;
          ok = mbar_wait(bar(DQ_READY), git & 1, wctx, 43);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          // rare: the watcher is still waiting for this turn, or the releaser is four shares behind
          if (turn_ok[0] <= git || turn_ok[1] + 4 <= git) {
            const unsigned long long t0 = globaltimer_ns();
            for (uint32_t spins = 1; turn_ok[0] <= git || turn_ok[1] + 4 <= git; ++spins) {
              __nanosleep(64);
              if ((spins & 0x3fu) == 0u && (*abort_flag || globaltimer_ns() - t0 > wctx.limit())) {
                ok = false;                                    // (the watcher reports its own timeouts)
                break;
              }
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          __threadfence_block();
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_addr(tmem, lane_base, kDqCol + c), r);
            tc_wait_ld();
            if (c + 32 >= D) {
              tc_fence_before();
              mbar_arrive(bar(DQ_DRAINED));       // the next iteration's dQ product may be issued
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4* dst = acc + (c / 4 + i) * kTile;
              if (order == 0)
                *dst = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                   __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
              else
                red_add_f32x4(dst, r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
            }
          }
          mbar_arrive(bar(ISSUED + (git & 3)));                // the releaser takes it from here
        }
        if (!ok) break;
      }
      ok = mbar_wait_idle(bar(UNIT_DONE), uc & 1, wctx, 41);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int xb = uc % XBUF;
      const uint32_t stage0 = base + L::kX + xb * 2 * L::kTileBytes;       // X0 region
#pragma unroll 1
      for (int c = 0; c < kOutCols; c += 32) {
        // dK/dV: columns [0, D) are dV (over the V tile), [D, 2D) are dK (over the K tile, scaled)
        const bool second = kKeyStat && c >= D;
        const uint32_t tile_base = (kKeyStat && !second) ? stage0 + L::kTileBytes : stage0;
        const float mul = (MODE == MODE_DQ || second) ? p.scale : 1.f;
        const int col0 = second ? c - D : c;
        uint32_t r[32];
        tmem_ld32(tmem_addr(tmem, lane_base, kOutCol + c), r);
        tc_wait_ld();
        if (c + 32 >= kOutCols) {
          tc_fence_before();
          mbar_arrive(bar(OUT_DRAINED));          // the accumulators may be overwritten
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = col0 + 8 * i;                         // first of 8 columns = one 16 B chunk
          const uint32_t addr = tile_base + static_cast<uint32_t>(col >> 6) * kBoxBytes +
                                static_cast<uint32_t>(row) * 128u +
                                ((static_cast<uint32_t>((col & 63) >> 3) ^ sw) << 4);
          st_shared_v4(addr,
                       Pack2<T>::pack(__uint_as_float(r[8 * i + 0]) * mul, __uint_as_float(r[8 * i + 1]) * mul),
                       Pack2<T>::pack(__uint_as_float(r[8 * i + 2]) * mul, __uint_as_float(r[8 * i + 3]) * mul),
                       Pack2<T>::pack(__uint_as_float(r[8 * i + 4]) * mul, __uint_as_float(r[8 * i + 5]) * mul),
                       Pack2<T>::pack(__uint_as_float(r[8 * i + 6]) * mul, __uint_as_float(r[8 * i + 7]) * mul));
        }
      }
      fence_proxy_async_smem();
      group_sync(48);
      if (!ok) break;
      if (warp == 12 && lane == 0) {
        const int oh = MODE == MODE_DQ ? w.h : w.hk;
        for (int x = 0; x < kBoxes; ++x) {
          tma_store_4d(&tm_out0, stage0 + x * kBoxBytes, 64 * x, oh, w.tile * kTile, w.b);
          if (kKeyStat)
            tma_store_4d(&tm_out1, stage0 + L::kTileBytes + x * kBoxBytes, 64 * x, oh,
                         w.tile * kTile, w.b);
        }
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(bar(X_EMPTY + xb));          // second arrival: the buffer may be reloaded
      }
    }
  } else if (warp == 8) {
    // ========================= scheduler + TMA producer ======================
    const CUtensorMap* mx0 = &tm_x0;
    const CUtensorMap* mx1 = &tm_x1;
    const CUtensorMap* my0 = &tm_y0;
    const CUtensorMap* my1 = &tm_y1;
    if (lane == 0) {
      tma_prefetch_desc(mx0);
      tma_prefetch_desc(mx1);
      tma_prefetch_desc(my0);
      tma_prefetch_desc(my1);
    }
    bool ok = true;
    int git = 0;
    // Takes the uc-th unit of this CTA from the global counter, publishes it to the other
    // roles and starts the loads of its stationary tiles.  Returns the unit (-1: none left).
    auto fetch_unit = [&](int uc) -> int {
      int u = 0;
      if (lane == 0) {
        u = static_cast<int>(atomicAdd(&p.sched[0], 1u));
        if (u >= p.total_units) u = -1;
        BwdUnit<MODE> w{};
        if (u >= 0) w = make_bwd_unit<MODE, YR>(u, p);
        volatile int* e = sched_ring + 8 * (uc % kRing);
        e[0] = u; e[1] = w.tile; e[2] = w.b; e[3] = w.h;
        e[4] = w.hk; e[5] = w.s_lo; e[6] = w.n_inner; e[7] = MODE == MODE_DQ ? w.extra : w.n_iters;
        mbar_arrive(bar(SCHED_FULL + (uc % kRing)));
        if (u >= 0) {
          const int xb = uc % XBUF;
          ok = mbar_wait(bar(X_EMPTY + xb), ((uc / XBUF) & 1) ^ 1, wctx, 30);
          if (ok) {
            const int xh = MODE == MODE_DQ ? w.h : w.hk;
            const uint32_t xa = base + L::kX + xb * 2 * L::kTileBytes;
            mbar_arrive_expect_tx(bar(X_FULL + xb), 2 * L::kTileBytes);
            for (int x = 0; x < kBoxes; ++x) {
              tma_load_4d(xa + x * kBoxBytes, mx0, bar(X_FULL + xb), 64 * x, xh, w.tile * kTile, w.b);
              tma_load_4d(xa + L::kTileBytes + x * kBoxBytes, mx1, bar(X_FULL + xb), 64 * x, xh,
                          w.tile * kTile, w.b);
            }
          }
          if constexpr (kDeltaIn) {
            // the unit's O tile, for its Delta; one buffer, free once the previous unit's Delta is done
            if (ok && p.delta_in_pass) {
              if (uc > 0) ok = mbar_wait(bar(O_EMPTY), (uc - 1) & 1, wctx, 46);
              if (ok) {
                mbar_arrive_expect_tx(bar(O_FULL), L::kTileBytes);
                tma_load_4d(base + L::kO, &tm_out1, bar(O_FULL), 0, w.h, w.tile * kTile, w.b);
              }
            }
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      return __shfl_sync(0xffffffffu, u, 0);
    };
    int u = fetch_unit(0);
    for (int uc = 0; ok && u >= 0; ++uc) {
      BwdUnit<MODE> w;
      next_unit(uc, ok, w);                      // published by this warp: never waits
      if (!ok) break;
      // The next unit's stationary tiles are requested once this unit's first streamed tiles
      // are on their way (with one stationary buffer: only when this unit has released it).
      int u_next = -2;
      const int prefetch_at = XBUF > 1 ? (w.n_iters < STAGES ? w.n_iters : STAGES) : w.n_iters;
      int inner = 0, g = 0;                       // it = g * n_inner + inner
      for (int it = 0; ok && it < w.n_iters; ++it, ++git, ++inner) {
        if (it == prefetch_at) u_next = fetch_unit(uc + 1);
        if (!ok) break;
        if (inner == w.n_inner) { inner = 0; ++g; }
        const int s = git % STAGES;
        const uint32_t ph = (git / STAGES) & 1;
        const int idx = w.streamed_index(inner);
        const int yh = MODE == MODE_DQ ? w.hk : w.h + g;
        if (lane == 0) ok = mbar_wait(bar(Y_EMPTY + s), ph ^ 1, wctx, 31);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        // The tile loads go out first; the per-row vectors (plain loads, a full memory latency)
        // follow while they are in flight, and the arrival that completes the stage comes last.
        if (lane == 0) {
          mbar_expect_tx(bar(Y_FULL + s), 2 * L::kYTileBytes);
          const uint32_t y0 = base + L::kY + s * 2 * L::kYTileBytes;
          for (int x = 0; x < kBoxes; ++x) {
            tma_load_4d(y0 + x * kYBoxBytes, my0, bar(Y_FULL + s), 64 * x, yh, idx * YR, w.b);
            tma_load_4d(y0 + L::kYTileBytes + x * kYBoxBytes, my1, bar(Y_FULL + s), 64 * x, yh,
                        idx * YR, w.b);
          }
        }
        if (kKeyStat) {
          // negated base-2 logsumexp and negated Delta of the streamed query tile
          float* vec = reinterpret_cast<float*>(gen + L::kVec + s * 1024);
          const long long row0 = (static_cast<long long>(w.b) * p.H + yh) * p.T;
#pragma unroll
          for (int i = 0; i < YR / 32; ++i) {
            const int c = lane * (YR / 32) + i;
            const int qpos = idx * YR + c;
            const bool in = qpos < p.T;
            vec[c] = in ? -p.lse[row0 + qpos] * kLog2e : -INFINITY;
            vec[YR + c] = in ? -p.delta[row0 + qpos] : 0.f;
          }
          __syncwarp();
        }
        if (lane == 0) mbar_arrive(bar(Y_FULL + s));
      }
      if (ok && u_next == -2) u_next = fetch_unit(uc + 1);
      u = u_next;
    }
  } else {
    // ================================ MMA issuer =============================
    // The whole warp runs this loop and waits on every barrier together; `leader` marks the one
    // lane that issues.  All values that feed a descriptor are made provably warp-uniform.
    {
      const uint32_t leader = elect_one() ? 1u : 0u;
      const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
      auto wait_all = [&](uint32_t b, uint32_t parity, unsigned where) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(b, parity, wctx, where));
      };
      auto next_unit_all = [&](int uc, bool& ok, int& n_iters) -> int {
        BwdUnit<MODE> w{};
        const int u = __shfl_sync(0xffffffffu, next_unit(uc, ok, w), 0);
        n_iters = __shfl_sync(0xffffffffu, w.n_iters, 0);
        ok = __all_sync(0xffffffffu, ok);
        return u;
      };
      bool ok = true;
      constexpr uint32_t idesc_t = make_idesc(kBf16, 128, YR, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBf16, 128, D, false, true);

      // T0 = X0 Y0^T, T1 = X1 Y1^T for global iteration `g` of unit buffer `xb`
      auto issue_t = [&](int xb, int g) {
        const int s = g % STAGES;
        const uint32_t x0 = base + L::kX + xb * 2 * L::kTileBytes, x1 = x0 + L::kTileBytes;
        const uint32_t y0 = base + L::kY + s * 2 * L::kYTileBytes, y1 = y0 + L::kYTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t xoff = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          const uint32_t yoff = (kk >> 2) * kYBoxBytes + (kk & 3) * 32;
          umma_ss(leader, tmem + 0, make_smem_desc(x0 + xoff, 16, 1024), make_smem_desc(y0 + yoff, 16, 1024),
                 idesc_t, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t xoff = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          const uint32_t yoff = (kk >> 2) * kYBoxBytes + (kk & 3) * 32;
          umma_ss(leader, tmem + kT1Col, make_smem_desc(x1 + xoff, 16, 1024), make_smem_desc(y1 + yoff, 16, 1024),
                 idesc_t, kk > 0 ? 1u : 0u);
        }
        umma_commit(leader, bar(T_FULL));
      };
      constexpr uint32_t idesc_dq = make_idesc(kBf16, 128, D, true, true);
      auto issue_out = [&](int xb, int g, uint32_t acc) {
        const int s = g % STAGES;
        const uint32_t y0 = base + L::kY + s * 2 * L::kYTileBytes, y1 = y0 + L::kYTileBytes;
        // 16-bit operand of k-step kk: 8 TMEM columns per step.  The dV and dK steps alternate,
        // so consecutive instructions never update the same accumulator.
        constexpr int kStepsPerHalf = YR / 32;
#pragma unroll
        for (int kk = 0; kk < YR / 16; ++kk) {
          const uint32_t acol = kSep ? 8 * kk
                                     : (YR / 2) * (kk / kStepsPerHalf) + 8 * (kk % kStepsPerHalf);
          if (MODE == MODE_DQ) {
            umma_ts(leader, tmem + kOutCol, tmem + kDsCol + acol,
                   make_smem_desc(y0 + kk * 2048, kYBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
          } else {
            umma_ts(leader, tmem + kOutCol, tmem + kPCol + acol,
                   make_smem_desc(y1 + kk * 2048, kYBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
            if constexpr (kFused) {
              // dK += dS^T Q: dS^T from shared memory, K-major (16 queries = 32 bytes per step)
              const uint32_t ds = base + L::kDs + (kk >> 2) * kBoxBytes + (kk & 3) * 32;
              umma_ss(leader, tmem + kOutCol + D, make_smem_desc(ds, 16, 1024),
                     make_smem_desc(y0 + kk * 2048, kYBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
            } else {
              umma_ts(leader, tmem + kOutCol + D, tmem + kDsCol + acol,
                     make_smem_desc(y0 + kk * 2048, kYBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
            }
          }
        }
        if constexpr (kFused) {
          // dQ share of this (key block, query tile): dS K, the same dS^T tile read MN-major
          // (queries along M, 16 keys = 16 rows per step), K_j MN-major as the B operand.  The
          // accumulator is free once the drain warps have pulled the previous share out.
          if (g > 0) ok = wait_all(bar(DQ_DRAINED), (g - 1) & 1, 49);
          if (ok) {
            tc_fence_after();
            const uint32_t x0 = base + L::kX + xb * 2 * L::kTileBytes;
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              umma_ss(leader, tmem + kDqCol, make_smem_desc(base + L::kDs + kk * 2048, kBoxBytes, 1024),
                     make_smem_desc(x0 + kk * 2048, kBoxBytes, 1024), idesc_dq, kk > 0 ? 1u : 0u);
          }
        }
        umma_commit(leader, bar(OUT_READY));
        if constexpr (kFused) umma_commit(leader, bar(DQ_READY));
        umma_commit(leader, bar(Y_EMPTY + s));
      };

      // cursor over (unit, iteration); `nxt` runs one global iteration ahead of `cur`
      int uc = 0;                       // units fetched so far
      int cur_n = 0, cur_it = 0, cur_xb = 0;
      int cur_u = next_unit_all(uc, ok, cur_n);
      if (ok && cur_u >= 0) {
        cur_xb = uc % XBUF;
        ok = wait_all(bar(X_FULL + cur_xb), (uc / XBUF) & 1, 32);
        if (ok) ok = wait_all(bar(Y_FULL + 0), 0, 33);
        if (ok) {
          tc_fence_after();
          issue_t(cur_xb, 0);
        }
      }
      int g = 0;                        // global iteration of `cur`
      int cur_uc = 0;                   // index of the unit `cur` belongs to
      while (ok && cur_u >= 0) {
        // ---- locate the next global iteration
        int nxt_u = cur_u, nxt_it = cur_it + 1, nxt_n = cur_n, nxt_xb = cur_xb;
        bool crossed = false;
        if (nxt_it == cur_n) {
          ++uc;
          nxt_u = next_unit_all(uc, ok, nxt_n);
          if (!ok) break;
          nxt_it = 0;
          crossed = true;
          if (nxt_u >= 0) nxt_xb = uc % XBUF;
        }
        const bool have_next = nxt_u >= 0;
        auto issue_next_t = [&]() {
          if (crossed) ok = wait_all(bar(X_FULL + nxt_xb), (uc / XBUF) & 1, 32);
          if (ok) ok = wait_all(bar(Y_FULL + (g + 1) % STAGES), ((g + 1) / STAGES) & 1, 33);
          if (ok && kSep) ok = wait_all(bar(T_CONSUMED), g & 1, 37);
          if (ok) {
            tc_fence_after();
            issue_t(nxt_xb, g + 1);
          }
        };
        // The next iteration's T products go first, also across a unit boundary, so that the
        // compute warps never wait for them.  With a single stationary buffer the next unit's
        // tiles can only be loaded once this unit's buffer has been released, i.e. after the
        // output products below are issued, so there the boundary is not crossed early.
        const bool early = kSep && have_next && (!crossed || XBUF > 1);
        if (early) issue_next_t();
        if (!ok) break;
        if (!(ok = wait_all(bar(PD_FULL), g & 1, 34))) break;
        tc_fence_after();
        // a unit's first output product overwrites the accumulators: the epilogue warps must
        // have pulled the previous unit's out of TMEM
        if (cur_it == 0 && cur_uc > 0) {
          if (!(ok = wait_all(bar(OUT_DRAINED), (cur_uc - 1) & 1, 42))) break;
          tc_fence_after();
        }
        issue_out(cur_xb, g, cur_it > 0 ? 1u : 0u);
        if (!ok) break;
        if (cur_it + 1 == cur_n) {
          umma_commit(leader, bar(X_EMPTY + cur_xb));
          umma_commit(leader, bar(UNIT_DONE));
        }
        if (!early && have_next) issue_next_t();
        if (!ok) break;
        cur_u = nxt_u;
        cur_it = nxt_it;
        cur_n = nxt_n;
        cur_xb = nxt_xb;
        if (crossed) cur_uc = uc;
        ++g;
      }
    }
  }
  } else {
    // ================================= compute ===============================
    setmaxnreg_inc<kRegsCompute>();
    if (!dead) {
    const int half = warp >> 2;                      // which YR / 2 columns of the row
    const uint32_t lane_base = 32u * (warp & 3);
    const int row = 32 * (warp & 3) + lane;          // row of the stationary tile == TMEM lane
    const uint32_t t0 = tmem_addr(tmem, lane_base, (YR / 2) * half);
    const uint32_t t1 = tmem_addr(tmem, lane_base, kT1Col + (YR / 2) * half);
    const uint32_t p_dst = tmem_addr(tmem, lane_base, kSep ? kPCol + (YR / 4) * half : (YR / 2) * half);
    const uint32_t ds_dst = tmem_addr(tmem, lane_base, kSep ? kDsCol + (YR / 4) * half
                                                             : kT1Col + (YR / 2) * half);
    // calls f(chunk 0) and, with two chunks per thread, f(chunk 1)
    auto each_chunk = [&](auto&& f) {
      f(std::integral_constant<int, 0>{});
      if constexpr (kCh > 1) f(std::integral_constant<int, 1>{});
    };
    const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);

    bool ok = true;
    int g = 0;                    // global iteration
    float pre_lse = 0.f, pre_delta = 0.f;     // dQ: row statistics of the next unit
    int out_waited = 0;           // OUT_READY phases this thread has observed
    auto wait_out = [&](int needed) {
      while (ok && out_waited < needed) {
        ok = mbar_wait(bar(OUT_READY), out_waited & 1, wctx, 38);
        ok = __all_sync(0xffffffffu, ok);
        ++out_waited;
      }
    };
    for (int uc = 0; ok; ++uc) {
      BwdUnit<MODE> w;
      const int u = next_unit(uc, ok, w);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok || u < 0) break;
      const int pos = w.tile * kTile + row;            // query position (dQ) or key position (dK/dV)

      // Columns this row can see, as positions of the streamed index: [va, va + vw], plus
      // positions below vsink (sink keys; dQ orientation only).
      int va, vsink = 0;
      unsigned vw;
      // the causal edge as this row sees it: a query's last visible key, a key's first query
      // (block-causal masks move both to the ends of the row's block)
      const int edge = MODE == MODE_DQ ? last_key_of_query(pos, p.block, p.T) : first_query_of_key(pos, p.block);
      if (MODE == MODE_DQ) {                           // row = query `pos`, columns = keys
        const int lo = p.window > 0 ? pos - (p.window - p.sinks) + 1 : 0;
        va = lo > 0 ? lo : 0;
        vw = static_cast<unsigned>(edge - va);
        vsink = p.window > 0 ? (p.sinks < pos + 1 ? p.sinks : pos + 1) : 0;   // sinks are causal too
      } else {                                         // row = key `pos`, columns = queries
        va = edge;
        vw = (p.window > 0 && pos >= p.sinks) ? static_cast<unsigned>(p.window - p.sinks - 1)
                                               : 0x7fffffffu;
      }
      uint64_t negl2_row = pack_f2(-INFINITY, -INFINITY), negd_row = 0ull;
      const bool delta_here = kDeltaIn && p.delta_in_pass != 0;      // Delta comes from the epilogue warps
      if (MODE == MODE_DQ && pos < p.T) {
        if (uc > 0) {                       // fetched during the previous unit's last iteration
          negl2_row = pack_f2(-pre_lse * kLog2e, -pre_lse * kLog2e);
          negd_row = pack_f2(-pre_delta, -pre_delta);
        } else {
          const long long idx = (static_cast<long long>(w.b) * p.H + w.h) * p.T + pos;
          const float l2 = -p.lse[idx] * kLog2e, dl = delta_here ? 0.f : -p.delta[idx];
          negl2_row = pack_f2(l2, l2);
          negd_row = pack_f2(dl, dl);
        }
      }
      if constexpr (kDeltaIn) {
        if (delta_here) {
          ok = mbar_wait(bar(DELTA_FULL + uc % XBUF), (uc / XBUF) & 1, wctx, 49);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const float dl = -reinterpret_cast<const volatile float*>(gen + L::kDeltaS)[(uc % XBUF) * kTile + row];
          negd_row = pos < p.T ? pack_f2(dl, dl) : 0ull;
        }
      }

      int inner = 0;
      for (int it = 0; it < w.n_iters; ++it, ++g, ++inner) {
        if (inner == w.n_inner) inner = 0;
        const int s = g % STAGES;
        const int idx = w.streamed_index(inner);
        if (MODE == MODE_DQ && it + 1 == w.n_iters) {
          // The next unit's row statistics are requested now (its descriptor is published well
          // ahead), so that their memory latency passes during this unit's last iteration.
          BwdUnit<MODE> wn;
          const int un = next_unit(uc + 1, ok, wn);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          const int pos_n = wn.tile * kTile + row;
          if (un >= 0 && pos_n < p.T) {
            const long long nidx = (static_cast<long long>(wn.b) * p.H + wn.h) * p.T + pos_n;
            pre_lse = p.lse[nidx];
            if (!delta_here) pre_delta = p.delta[nidx];
          }
        }
        ok = mbar_wait(bar(T_FULL), g & 1, wctx, 35);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();

        uint32_t sv[kCh][32], dv[kCh][32];
#pragma unroll
        for (int ch = 0; ch < kCh; ++ch) tmem_ld32(t0 + 32 * ch, sv[ch]);
#pragma unroll
        for (int ch = 0; ch < kCh; ++ch) tmem_ld32(t1 + 32 * ch, dv[ch]);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(bar(T_CONSUMED));

        // positions of the (stationary tile) x (streamed tile) rectangle
        const int q_lo = MODE == MODE_DQ ? w.tile * kTile : idx * YR;
        const int q_hi = q_lo + (MODE == MODE_DQ ? kTile : YR) - 1;
        const int k_lo = MODE == MODE_DQ ? idx * YR : w.tile * kTile;
        const int k_hi = k_lo + (MODE == MODE_DQ ? YR : kTile) - 1;
        const bool full = rect_fully_visible(q_lo, q_hi, k_lo, k_hi, p.window, p.sinks, p.block, p.T);
        const int edges = rect_edges(q_lo, q_hi, k_lo, k_hi, p.window, p.sinks);
        const ulonglong2* vec2 =
            reinterpret_cast<const ulonglong2*>(gen + L::kVec + s * 1024) + (YR / 8) * half;
        const int other0 = idx * YR + (YR / 2) * half;   // position of this thread's first column

        uint32_t pp[16 * kCh], dd[16 * kCh];
        // One 32-column chunk (8 groups of 4 columns).  kMasked: apply the per-element
        // visibility test; the test is one unsigned compare against the row's visible interval
        // [va, va + vw] (plus the sink prefix for the dQ orientation).
        auto do_chunk = [&](auto ch_c, auto masked_c) {
          constexpr int ch = decltype(ch_c)::value;
          constexpr int kMasked = decltype(masked_c)::value;   // 0 none, 1 general, 2 causal edge, 3 window edge
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            const int c4 = 8 * ch + c8;
            uint64_t nl_a, nl_b, nd_a, nd_b;
            if (MODE == MODE_DQ) {
              nl_a = nl_b = negl2_row;
              nd_a = nd_b = negd_row;
            } else {
              const ulonglong2 nl = vec2[c4];              // -lse2 of columns 4 c4 .. 4 c4 + 3
              const ulonglong2 nd = vec2[YR / 4 + c4];     // -delta
              nl_a = nl.x; nl_b = nl.y; nd_a = nd.x; nd_b = nd.y;
            }
            const int c = 4 * c4;
            const uint64_t xa = ffma2(pack_f2(__uint_as_float(sv[c >> 5][c & 31]),
                                              __uint_as_float(sv[c >> 5][(c & 31) + 1])), scale2, nl_a);
            const uint64_t xb = ffma2(pack_f2(__uint_as_float(sv[c >> 5][(c & 31) + 2]),
                                              __uint_as_float(sv[c >> 5][(c & 31) + 3])), scale2, nl_b);
            float p0, p1, p2, p3;
            unpack_f2(xa, p0, p1);
            unpack_f2(xb, p2, p3);
            p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
            if (kMasked == 2) {
              // the causal edge alone: one compare per element against a per-thread limit
              const int lim = edge - other0;     // dQ: last visible column; dK/dV: first visible
              if (MODE == MODE_DQ) {
                if (c + 0 > lim) p0 = 0.f;
                if (c + 1 > lim) p1 = 0.f;
                if (c + 2 > lim) p2 = 0.f;
                if (c + 3 > lim) p3 = 0.f;
              } else {
                if (c + 0 < lim) p0 = 0.f;
                if (c + 1 < lim) p1 = 0.f;
                if (c + 2 < lim) p2 = 0.f;
                if (c + 3 < lim) p3 = 0.f;
              }
            } else if (kMasked == 3) {
              // only the window's lower edge cuts the block
              if (MODE == MODE_DQ) {
                const int lim = va - other0;                               // first visible column
                if (c + 0 < lim) p0 = 0.f;
                if (c + 1 < lim) p1 = 0.f;
                if (c + 2 < lim) p2 = 0.f;
                if (c + 3 < lim) p3 = 0.f;
              } else {
                const int lim = pos + (p.window - p.sinks) - 1 - other0;   // last query that sees this key
                if (c + 0 > lim) p0 = 0.f;
                if (c + 1 > lim) p1 = 0.f;
                if (c + 2 > lim) p2 = 0.f;
                if (c + 3 > lim) p3 = 0.f;
              }
            } else if (kMasked == 1) {
              const unsigned o = static_cast<unsigned>(other0 + c - va);   // wraps below va
              const int ox = other0 + c;
              if (!(o + 0u <= vw || ox + 0 < vsink)) p0 = 0.f;
              if (!(o + 1u <= vw || ox + 1 < vsink)) p1 = 0.f;
              if (!(o + 2u <= vw || ox + 2 < vsink)) p2 = 0.f;
              if (!(o + 3u <= vw || ox + 3 < vsink)) p3 = 0.f;
            }
            const uint64_t pa = pack_f2(p0, p1), pb = pack_f2(p2, p3);
            const uint64_t da = fmul2(pa, fadd2(pack_f2(__uint_as_float(dv[c >> 5][c & 31]),
                                                        __uint_as_float(dv[c >> 5][(c & 31) + 1])), nd_a));
            const uint64_t db = fmul2(pb, fadd2(pack_f2(__uint_as_float(dv[c >> 5][(c & 31) + 2]),
                                                        __uint_as_float(dv[c >> 5][(c & 31) + 3])), nd_b));
            float d0, d1, d2, d3;
            unpack_f2(da, d0, d1);
            unpack_f2(db, d2, d3);
            pp[2 * c4] = Pack2<T>::pack(p0, p1);
            pp[2 * c4 + 1] = Pack2<T>::pack(p2, p3);
            dd[2 * c4] = Pack2<T>::pack(d0, d1);
            dd[2 * c4 + 1] = Pack2<T>::pack(d2, d3);
          }
        };
        auto zero_chunk = [&](auto ch_c) {
          constexpr int ch = decltype(ch_c)::value;
#pragma unroll
          for (int i = 0; i < 16; ++i) pp[16 * ch + i] = dd[16 * ch + i] = 0u;
        };
        // Boundary blocks: each 32-column chunk is, for the whole warp, either entirely
        // visible (plain path), entirely masked (zeros, no arithmetic) or mixed.
        auto chunk = [&](auto ch_c) {
          constexpr int ch = decltype(ch_c)::value;
          const int x0 = other0 + 32 * ch, x1 = x0 + 31;
          const long long hi = static_cast<long long>(va) + vw;          // last visible position
          const bool in = (x0 >= va && x1 <= hi) || x1 < vsink;
          const bool out = (x1 < va || x0 > hi) && x0 >= vsink;
          const bool all_in = __all_sync(0xffffffffu, in);
          const bool all_out = __all_sync(0xffffffffu, out);
          if (all_in) do_chunk(ch_c, std::integral_constant<int, 0>{});
          else if (all_out) zero_chunk(ch_c);
          else do_chunk(ch_c, std::integral_constant<int, 1>{});
        };
        if (full) {
          // interior blocks: one straight-line pass over all columns (branches between the
          // chunks would drain the exponential unit's pipeline at every chunk)
          each_chunk([&](auto ch_c) { do_chunk(ch_c, std::integral_constant<int, 0>{}); });
        } else if (edges == EDGE_CAUSAL) {
          // only the causal edge cuts the block: the same straight-line pass with one compare
          // per element; skipping the fully masked chunks would bring the branches back
          each_chunk([&](auto ch_c) { do_chunk(ch_c, std::integral_constant<int, 2>{}); });
        } else if (edges == EDGE_WINDOW) {
          each_chunk([&](auto ch_c) { do_chunk(ch_c, std::integral_constant<int, 3>{}); });
        } else {
          each_chunk([&](auto ch_c) { chunk(ch_c); });
        }
        // the previous iteration's output products must be done reading P / dS
        wait_out(g);
        if (!ok) break;
        if constexpr (kFused) {
          // P^T to TMEM as before; dS^T to shared memory as a 128B-swizzled [keys][queries] tile
          // (this thread's 64 queries are one 128-byte row of box `half`)
          tmem_st32(p_dst, pp);
          const uint32_t ds_row = base + L::kDs + static_cast<uint32_t>(half) * kBoxBytes +
                                  static_cast<uint32_t>(row) * 128u;
          const uint32_t sw = static_cast<uint32_t>(row & 7);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(ds_row + ((static_cast<uint32_t>(c) ^ sw) << 4), dd[4 * c], dd[4 * c + 1],
                         dd[4 * c + 2], dd[4 * c + 3]);
          fence_proxy_async_smem();
        } else if constexpr (kCh == 2) {
          if (kKeyStat) tmem_st32(p_dst, pp);
          tmem_st32(ds_dst, dd);
        } else {
          if (kKeyStat) tmem_st16(p_dst, pp);
          tmem_st16(ds_dst, dd);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(PD_FULL));
      }
      if (!ok) break;

    }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  // scheduler bookkeeping: the last CTA of the launch to get here re-arms the counters
  if (threadIdx.x == 0) {
    // a pass that started beside its predecessor does not finish before it: what follows this
    // grid in the stream may rely on both
    if (!p.dep_wait_first) grid_dep_wait();
    __threadfence();
    const unsigned done = atomicAdd(&p.sched[1], 1u);
    if (done == gridDim.x - 1) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
      __threadfence();
    }
  }
}

template <typename T, int D, int MODE, int STAGES, int XBUF, int YR>
int launch_mode(const Problem& p, const void* dout, const void* q, const void* k, const void* v,
                const float* lse, const float* delta, void* out0, void* out1, unsigned* status,
                cudaStream_t stream, void* dq = nullptr, const FusedScratch* fused = nullptr,
                bool beside_previous = false, const void* o_for_delta = nullptr, float* delta_out = nullptr,
                bool plain_launch = false) {
  // stationary tensors in boxes of 128 rows, streamed tensors in boxes of YR rows; output tiles
  // leave through TMA stores: dQ is [B,T,H,D], dK and dV are [B,T,Hkv,D]
  const void* x0 = MODE == MODE_DQ ? q : k;
  const void* x1 = MODE == MODE_DQ ? dout : v;
  const void* y0 = MODE == MODE_DQ ? k : q;
  const void* y1 = MODE == MODE_DQ ? v : dout;
  const int x_heads = MODE == MODE_DQ ? p.H : p.Hkv;
  const int y_heads = MODE == MODE_DQ ? p.Hkv : p.H;
  CUtensorMap mx0, mx1, my0, my1, mo0, mo1;
  int mst = make_tile_map(&mx0, x0, p.dtype, p.B, p.T, x_heads, p.D, kTile);
  if (mst == NLFA_OK) mst = make_tile_map(&mx1, x1, p.dtype, p.B, p.T, x_heads, p.D, kTile);
  if (mst == NLFA_OK) mst = make_tile_map(&my0, y0, p.dtype, p.B, p.T, y_heads, p.D, YR);
  if (mst == NLFA_OK) mst = make_tile_map(&my1, y1, p.dtype, p.B, p.T, y_heads, p.D, YR);
  if (mst == NLFA_OK) mst = make_tile_map(&mo0, out0, p.dtype, p.B, p.T, x_heads, p.D, kTile);
  // (the dQ pass has one output; its second map describes O when the pass also forms Delta)
  if (mst == NLFA_OK)
    mst = make_tile_map(&mo1, MODE == MODE_DQ ? (o_for_delta ? o_for_delta : out0) : out1, p.dtype, p.B, p.T,
                        x_heads, p.D, kTile);
  if (mst != NLFA_OK) return mst;
  constexpr bool kDeltaIn = MODE == MODE_DQ && XBUF == 2 && D == 64;
  if (o_for_delta != nullptr && !kDeltaIn) return NLFA_ERR_UNSUPPORTED_PATH;
  using L = BwdSmem<D, STAGES, XBUF, YR, MODE == MODE_FUSED, kDeltaIn>;
  static_assert(L::kDynamic <= 232448, "over the shared memory a CTA can have");
  auto kern = bwd_tc_kernel<T, D, MODE, STAGES, XBUF, YR>;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::kDynamic) != NLFA_OK)
    return NLFA_ERR_CUDA;
  BwdParams bp;
  bp.T = p.T;
  bp.H = p.H;
  bp.Hkv = p.Hkv;
  bp.window = p.window;
  bp.sinks = p.sinks;
  bp.block = p.block;
  bp.n_tiles = (p.T + kTile - 1) / kTile;
  bp.n_ytiles = (p.T + YR - 1) / YR;
  bp.BH = p.B * (MODE == MODE_DQ ? p.H : p.Hkv);
  bp.total_units = bp.n_tiles * bp.BH;
  bp.scale = p.scale;
  bp.scale_log2 = p.scale * kLog2e;
  bp.lse = lse;
  bp.delta = delta;
  bp.out0 = out0;
  bp.out1 = out1;
  bp.status = status;
  bp.delta_in_pass = o_for_delta != nullptr ? 1 : 0;
  bp.delta_out = delta_out;
  bp.dq_acc = fused ? fused->dq_acc : nullptr;
  bp.dq_turn = fused ? fused->dq_turn : nullptr;
  if (MODE == MODE_FUSED) {
    if (fused == nullptr || dq == nullptr) return NLFA_ERR_NULL_POINTER;
    // every (batch, head, query tile) starts with no share added
    if (cudaMemsetAsync(fused->dq_turn, 0, sizeof(unsigned) * static_cast<size_t>(p.B) * p.H * bp.n_tiles,
                        stream) != cudaSuccess)
      return NLFA_ERR_CUDA;
  }
  const int sst = sched_counters(stream, &bp.sched);
  if (sst != NLFA_OK) return sst;
  const int grid = bp.total_units < sm_count() ? bp.total_units : sm_count();
  bp.sched_group = MODE == MODE_DQ ? bp.BH : grid;      // (the dQ pass gains nothing from groups)
  // (the fused pass follows a memset, not a kernel: launched the plain way)
  const bool overlap = MODE != MODE_FUSED && !plain_launch && overlap_launches(MODE == MODE_DQ ? kOverlapDq : kOverlapDkv);
  bp.dep_wait_first = (overlap && beside_previous) ? 0 : 1;
  if (launch_kernel(kern, dim3(grid), dim3(512), L::kDynamic, stream, overlap, mx0, mx1, my0, my1, mo0, mo1, bp) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return NLFA_ERR_CUDA;
  }
  if (MODE == MODE_FUSED) {
    // the fp32 sums, complete now, become dQ: scaled, converted, rows put back in order
    const long long pieces = static_cast<long long>(p.B) * p.H * bp.n_tiles * kTile * 16;
    dq_convert_kernel<T><<<static_cast<unsigned>((pieces + 255) / 256), 256, 0, stream>>>(
        fused->dq_acc, dq, p.T, p.H, bp.n_tiles, p.D, p.scale, pieces);
    if (cudaGetLastError() != cudaSuccess) return NLFA_ERR_CUDA;
  }
  return NLFA_OK;
}

// True when the backward does without the separate Delta kernel: Delta and the dQ pass both asked
// for, real head dim 64 (two stationary buffers in the dQ pass; the sums then match
// delta_vec_kernel's bit for bit) -- and a problem large enough for it to pay.  With fewer than
// sixteen query tiles per SM the backward is faster the other way round (measured at B = 4, 8, 16
// of H = 12, T = 1024: the dQ pass can then start beside the dK/dV pass, and a short Delta kernel
// costs less than the later start of the first unit).  NLFA_DELTA_IN_DQ=0 / 1 forces either.
inline bool delta_in_dq_pass(const Problem& p, int passes) {
  static const int forced = [] {
    const char* v = std::getenv("NLFA_DELTA_IN_DQ");
    return v == nullptr ? -1 : (v[0] == '0' ? 0 : 1);
  }();
  const int both = NLFA_PASS_DELTA | NLFA_PASS_DQ;
  if (p.D != 64 || (passes & NLFA_PASS_FUSED) != 0 || (passes & both) != both || forced == 0) return false;
  if (forced == 1) return true;
  const long long tiles = static_cast<long long>(p.B) * p.H * ((p.T + kTile - 1) / kTile);
  return tiles >= 16ll * sm_count();
}

template <typename T, int D, int STAGES, int XBUF, int YR>
int launch_both(const Problem& p, const void* dout, const void* q, const void* k, const void* v, const void* o,
                const float* lse, float* delta, void* dq, void* dk, void* dv, int passes,
                unsigned* status, cudaStream_t stream, const FusedScratch* fused) {
  int st = NLFA_OK;
  if constexpr (D == 64 && YR == 128) {
    // one pass for all three gradients: three streamed stages (the dS tile takes the fourth's room)
    if (passes & NLFA_PASS_FUSED)
      return launch_mode<T, D, MODE_FUSED, 3, XBUF, YR>(p, dout, q, k, v, lse, delta, dk, dv, status, stream,
                                                       dq, fused);
    // The whole backward in two launches: the dQ pass forms Delta on its way and runs first, the
    // dK/dV pass reads it.
    if (delta_in_dq_pass(p, passes)) {
      // (plain launches: between these two long kernels the overlapped set-up measured slower)
      st = launch_mode<T, D, MODE_DQ, STAGES, XBUF, YR>(p, dout, q, k, v, lse, delta, dq, nullptr, status, stream,
                                                       nullptr, nullptr, false, o, delta, true);
      if (st != NLFA_OK || (passes & NLFA_PASS_DKV) == 0) return st;
      return launch_mode<T, D, MODE_DKV, STAGES, XBUF, YR>(p, dout, q, k, v, lse, delta, dk, dv, status, stream,
                                                        nullptr, nullptr, false, nullptr, nullptr, true);
    }
  }
  if (passes & NLFA_PASS_DKV)
    st = launch_mode<T, D, MODE_DKV, STAGES, XBUF, YR>(p, dout, q, k, v, lse, delta, dk, dv, status, stream);
  if (st != NLFA_OK) return st;
  // Launched right behind this call's dK/dV pass, the dQ pass reads none of its results and may
  // take the SMs it leaves one by one.
  if (passes & NLFA_PASS_DQ)
    st = launch_mode<T, D, MODE_DQ, STAGES, XBUF, YR>(p, dout, q, k, v, lse, delta, dq, nullptr, status, stream,
                                                     nullptr, nullptr, (passes & NLFA_PASS_DKV) != 0);
  return st;
}

}  // namespace

bool bwd_delta_in_dq(const Problem& p, int passes) { return delta_in_dq_pass(p, passes); }

int launch_bwd_tc(const Problem& p, const void* dout, const void* q, const void* k, const void* v,
                  const void* o, const float* lse, void* dq, void* dk, void* dv, float* delta,
                  int passes, unsigned* status, cudaStream_t stream, const FusedScratch* fused) {
  if (p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (p.D != 32 && p.D != 64 && p.D != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  if ((passes & NLFA_PASS_FUSED) && p.D > 64) return NLFA_ERR_UNSUPPORTED_PATH;
  // Head dim 32 runs the 64-wide kernels: the tensor maps describe the real 32 columns, the
  // TMA boxes are 64 wide, so loads fill columns 32-63 with zeros (which add nothing to any
  // product) and stores drop them.
  int st = NLFA_OK;
  if ((passes & NLFA_PASS_DELTA) && !delta_in_dq_pass(p, passes)) st = launch_delta(p, dout, o, delta, stream);
  if (st != NLFA_OK) return st;
  const bool bf16 = p.dtype == NLFA_DTYPE_BF16;
  if (p.D <= 64) {
    // 128-row streamed tiles, four stages, two stationary buffers
    return bf16 ? launch_both<__nv_bfloat16, 64, 4, 2, 128>(p, dout, q, k, v, o, lse, delta, dq, dk, dv, passes, status, stream, fused)
                : launch_both<__half, 64, 4, 2, 128>(p, dout, q, k, v, o, lse, delta, dq, dk, dv, passes, status, stream, fused);
  }
  // D = 128: shared memory holds one stationary pair (64 KB) and 128 KB of streamed tiles.
  // As 64-row tiles that is four stages in flight instead of two, and the narrower T tiles
  // leave TMEM columns for separate P / dS operands, i.e. for the one-iteration lookahead.
  return bf16 ? launch_both<__nv_bfloat16, 128, 4, 1, 64>(p, dout, q, k, v, o, lse, delta, dq, dk, dv, passes, status, stream, fused)
              : launch_both<__half, 128, 4, 1, 64>(p, dout, q, k, v, o, lse, delta, dq, dk, dv, passes, status, stream, fused);
}


}  // namespace nlfa
