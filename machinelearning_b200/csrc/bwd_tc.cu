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
// T0/T1 are fp32 accumulators in TMEM (columns 0 and 128).  The eight compute
// warps split each row in two 64-column halves; each thread turns its 64
// scores into 16-bit P / dS and writes them back over the columns it just read
// (first 32 columns of its half), from where they are the TMEM A operand of the
// output products, whose B operand is the streamed tile read MN-major.
// Outputs accumulate in TMEM at column 256 (dQ, or dV then dK).
//
// Warps: 0-7 compute, 8 TMA producer, 9 MMA issuer and TMEM owner.
#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {
namespace {

enum { MODE_DQ = 0, MODE_DKV = 1 };

struct BwdParams {
  int T, H, Hkv;
  int window, sinks;
  int n_tiles;
  float scale, scale_log2;
  const float* lse;
  const float* delta;
  void* out0;            // dQ  | dK
  void* out1;            // --  | dV
  unsigned* status;
};

template <int D, int STAGES>
struct BwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kX = 0;                                  // X0, X1 stationary
  static constexpr int kY = kX + 2 * kTileBytes;                // per stage: Y0, Y1
  static constexpr int kVec = kY + STAGES * 2 * kTileBytes;     // per stage: lse2[128], delta[128]
  static constexpr int kBar = kVec + STAGES * 1024;
  // barriers: x_full, t_full, pd_full, out_full, y_full[S], y_empty[S]
  static constexpr int kNumBars = 4 + 2 * STAGES;
  static constexpr int kTmemSlot = kBar + 8 * kNumBars;
  static constexpr int kAbort = kTmemSlot + 4;
  static constexpr int kTotal = kAbort + 4;
  static constexpr int kDynamic = kTotal + 1024;
};

template <typename T, int D, int MODE, int STAGES>
__global__ void __launch_bounds__(320, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
              const BwdParams p) {
  using L = BwdSmem<D, STAGES>;
  constexpr int kBoxes = D / 64;
  constexpr int kBoxBytes = kTile * 128;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr uint32_t kOutCol = 256;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  auto bar = [&](int i) -> uint32_t { return base + L::kBar + 8u * i; };
  constexpr int X_FULL = 0, T_FULL = 1, PD_FULL = 2, OUT_FULL = 3, Y_FULL = 4, Y_EMPTY = 4 + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kAbort);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kTmemSlot);
  const WaitCtx wctx{abort_flag, p.status};

  // ---- work owned by this CTA.  blockIdx.x walks tiles heavy-first.
  //  dQ:    tile = query tile i, blockIdx.y = b * H + h; streams key blocks of tile_range(i)
  //  dK/dV: tile = key block j,  blockIdx.y = b * Hkv + hk; streams query tiles i >= j that
  //         see block j, for every head of the GQA group
  const int group = p.H / p.Hkv;
  int tile, b, h, hk;
  int s_lo, s_hi, extra, n_inner, n_iters;     // streamed index list
  if (MODE == MODE_DQ) {
    tile = p.n_tiles - 1 - static_cast<int>(blockIdx.x);
    b = blockIdx.y / p.H;
    h = blockIdx.y % p.H;
    hk = h / group;
    const TileRange r = tile_range(tile, p.window, p.sinks);
    s_lo = r.lo;
    s_hi = r.hi;
    extra = r.sink_blocks < r.lo ? r.sink_blocks : r.lo;
    n_inner = extra + (s_hi - s_lo + 1);
    n_iters = n_inner;
  } else {
    tile = static_cast<int>(blockIdx.x);       // early key blocks see the most queries
    b = blockIdx.y / p.Hkv;
    hk = blockIdx.y % p.Hkv;
    h = hk * group;
    s_lo = tile;
    s_hi = p.n_tiles - 1;
    if (p.window > 0 && tile >= (p.sinks + kTile - 1) / kTile) {
      const int last_q = tile * kTile + kTile - 1 + (p.window - p.sinks) - 1;
      const int hi = last_q / kTile;
      s_hi = hi < s_hi ? hi : s_hi;
    }
    extra = 0;
    n_inner = s_hi - s_lo + 1;
    n_iters = n_inner * group;
  }
  auto streamed_index = [&](int inner) { return inner < extra ? inner : s_lo + (inner - extra); };

  if (threadIdx.x == 0) {
    *abort_flag = (*reinterpret_cast<volatile unsigned*>(p.status) != STATUS_OK) ? 1 : 0;
    mbar_init(bar(X_FULL), 1);
    mbar_init(bar(T_FULL), 1);
    mbar_init(bar(PD_FULL), 256);
    mbar_init(bar(OUT_FULL), 1);
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

  if (dead) {
    // straight to the tail
  } else if (warp == 8) {
    // =============================== TMA producer ============================
    const CUtensorMap* mx0 = MODE == MODE_DQ ? &tm_q : &tm_k;
    const CUtensorMap* mx1 = MODE == MODE_DQ ? &tm_do : &tm_v;
    const CUtensorMap* my0 = MODE == MODE_DQ ? &tm_k : &tm_q;
    const CUtensorMap* my1 = MODE == MODE_DQ ? &tm_v : &tm_do;
    if (lane == 0) {
      tma_prefetch_desc(mx0);
      tma_prefetch_desc(mx1);
      tma_prefetch_desc(my0);
      tma_prefetch_desc(my1);
      const int xh = MODE == MODE_DQ ? h : hk;
      mbar_arrive_expect_tx(bar(X_FULL), 2 * L::kTileBytes);
      for (int x = 0; x < kBoxes; ++x) {
        tma_load_4d(base + L::kX + x * kBoxBytes, mx0, bar(X_FULL), 64 * x, xh, tile * kTile, b);
        tma_load_4d(base + L::kX + L::kTileBytes + x * kBoxBytes, mx1, bar(X_FULL), 64 * x, xh,
                    tile * kTile, b);
      }
    }
    bool ok = true;
    for (int it = 0; it < n_iters; ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1;
      const int g = it / n_inner;
      const int idx = streamed_index(it - g * n_inner);
      const int yh = MODE == MODE_DQ ? hk : h + g;
      if (lane == 0) ok = mbar_wait(bar(Y_EMPTY + s), ph ^ 1, wctx, 31);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (MODE == MODE_DKV) {
        // per-query logsumexp (base 2) and Delta of the streamed query tile
        float* vec = reinterpret_cast<float*>(gen + L::kVec + s * 1024);
        const long long row0 = (static_cast<long long>(b) * p.H + yh) * p.T;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = lane * 4 + i;
          const int qpos = idx * kTile + c;
          const bool in = qpos < p.T;
          vec[c] = in ? p.lse[row0 + qpos] * kLog2e : INFINITY;
          vec[128 + c] = in ? p.delta[row0 + qpos] : 0.f;
        }
        __syncwarp();
      }
      if (lane == 0) {
        mbar_arrive_expect_tx(bar(Y_FULL + s), 2 * L::kTileBytes);
        const uint32_t y0 = base + L::kY + s * 2 * L::kTileBytes;
        for (int x = 0; x < kBoxes; ++x) {
          tma_load_4d(y0 + x * kBoxBytes, my0, bar(Y_FULL + s), 64 * x, yh, idx * kTile, b);
          tma_load_4d(y0 + L::kTileBytes + x * kBoxBytes, my1, bar(Y_FULL + s), 64 * x, yh,
                      idx * kTile, b);
        }
      }
    }
  } else if (warp == 9) {
    // ================================ MMA issuer =============================
    if (lane == 0) {
      constexpr uint32_t idesc_t = make_idesc(kBf16, 128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc(kBf16, 128, D, false, true);
      const uint32_t x0 = base + L::kX, x1 = base + L::kX + L::kTileBytes;
      bool ok = mbar_wait(bar(X_FULL), 0, wctx, 32);
      for (int it = 0; ok && it < n_iters; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const uint32_t y0 = base + L::kY + s * 2 * L::kTileBytes, y1 = y0 + L::kTileBytes;
        if (!(ok = mbar_wait(bar(Y_FULL + s), ph, wctx, 33))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          mma_ss(tmem + 0, make_smem_desc(x0 + off, 16, 1024), make_smem_desc(y0 + off, 16, 1024),
                 idesc_t, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
          mma_ss(tmem + 128, make_smem_desc(x1 + off, 16, 1024), make_smem_desc(y1 + off, 16, 1024),
                 idesc_t, kk > 0 ? 1u : 0u);
        }
        tc_commit(bar(T_FULL));
        if (!(ok = mbar_wait(bar(PD_FULL), it & 1, wctx, 34))) break;
        tc_fence_after();
        const uint32_t acc = it > 0 ? 1u : 0u;
        // 16-bit operand of k-step kk: half (kk / 4) of the row, 8 columns per step
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk) {
          const uint32_t acol = 64 * (kk >> 2) + 8 * (kk & 3);
          if (MODE == MODE_DQ) {
            mma_ts(tmem + kOutCol, tmem + 128 + acol,
                   make_smem_desc(y0 + kk * 2048, kBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
          } else {
            mma_ts(tmem + kOutCol, tmem + 0 + acol,
                   make_smem_desc(y1 + kk * 2048, kBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
          }
        }
        if (MODE == MODE_DKV) {
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            const uint32_t acol = 64 * (kk >> 2) + 8 * (kk & 3);
            mma_ts(tmem + kOutCol + D, tmem + 128 + acol,
                   make_smem_desc(y0 + kk * 2048, kBoxBytes, 1024), idesc_o, (acc | (kk > 0)) ? 1u : 0u);
          }
        }
        tc_commit(bar(Y_EMPTY + s));
      }
      if (ok) tc_commit(bar(OUT_FULL));
    }
  } else {
    // ================================= compute ===============================
    const int half = warp >> 2;                      // which 64 columns of the row
    const uint32_t lane_base = 32u * (warp & 3);
    const int row = 32 * (warp & 3) + lane;          // row of the stationary tile == TMEM lane
    const int pos = tile * kTile + row;              // query position (dQ) or key position (dK/dV)
    const uint32_t t0 = tmem_addr(tmem, lane_base, 64 * half);
    const uint32_t t1 = tmem_addr(tmem, lane_base, 128 + 64 * half);

    float lse2_row = INFINITY, delta_row = 0.f;
    if (MODE == MODE_DQ && pos < p.T) {
      const long long idx = (static_cast<long long>(b) * p.H + h) * p.T + pos;
      lse2_row = p.lse[idx] * kLog2e;
      delta_row = p.delta[idx];
    }

    bool ok = true;
    for (int it = 0; it < n_iters; ++it) {
      const int s = it % STAGES;
      const int g = it / n_inner;
      const int idx = streamed_index(it - g * n_inner);
      ok = mbar_wait(bar(T_FULL), it & 1, wctx, 35);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

      uint32_t sv[2][32], dv[2][32];
      tmem_ld32(t0, sv[0]);
      tmem_ld32(t0 + 32, sv[1]);
      tmem_ld32(t1, dv[0]);
      tmem_ld32(t1 + 32, dv[1]);
      tc_wait_ld();

      const int qtile = MODE == MODE_DQ ? tile : idx;
      const int kblock = MODE == MODE_DQ ? idx : tile;
      const bool full = block_fully_visible(qtile, kblock, p.window, p.sinks);
      const float* vec = reinterpret_cast<const float*>(gen + L::kVec + s * 1024);
      const int c0 = 64 * half;                      // first column this thread owns
      const int other0 = idx * kTile + c0;           // position of that column

      uint32_t pp[32], dd[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float pv[2], ds[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int cc = 2 * c + e;
          const float sc = __uint_as_float(sv[cc >> 5][cc & 31]);
          const float dp = __uint_as_float(dv[cc >> 5][cc & 31]);
          float l2, dl;
          if (MODE == MODE_DQ) {
            l2 = lse2_row;
            dl = delta_row;
          } else {
            l2 = vec[c0 + cc];
            dl = vec[128 + c0 + cc];
          }
          float pe = fast_exp2(fmaf(sc, p.scale_log2, -l2));
          if (!full) {
            const int qq = MODE == MODE_DQ ? pos : other0 + cc;
            const int kk = MODE == MODE_DQ ? other0 + cc : pos;
            if (!key_visible(qq, kk, p.window, p.sinks)) pe = 0.f;
          }
          pv[e] = pe;
          ds[e] = pe * (dp - dl);
        }
        pp[c] = Pack2<T>::pack(pv[0], pv[1]);
        dd[c] = Pack2<T>::pack(ds[0], ds[1]);
      }
      if (MODE == MODE_DKV) tmem_st32(t0, pp);
      tmem_st32(t1, dd);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(PD_FULL));
    }

    if (ok) {
      ok = mbar_wait(bar(OUT_FULL), 0, wctx, 36);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      if (MODE == MODE_DQ) {
        // each half stores D/2 columns of its dQ row
        T* orow = static_cast<T*>(p.out0) +
                  ((static_cast<long long>(b) * p.T + pos) * p.H + h) * static_cast<long long>(D) +
                  half * (D / 2);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tmem, lane_base, kOutCol + half * (D / 2) + 32 * c), r);
          tc_wait_ld();
          if (pos < p.T) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = Pack2<T>::pack(__uint_as_float(r[8 * i + 0]) * p.scale, __uint_as_float(r[8 * i + 1]) * p.scale);
              w.y = Pack2<T>::pack(__uint_as_float(r[8 * i + 2]) * p.scale, __uint_as_float(r[8 * i + 3]) * p.scale);
              w.z = Pack2<T>::pack(__uint_as_float(r[8 * i + 4]) * p.scale, __uint_as_float(r[8 * i + 5]) * p.scale);
              w.w = Pack2<T>::pack(__uint_as_float(r[8 * i + 6]) * p.scale, __uint_as_float(r[8 * i + 7]) * p.scale);
              *reinterpret_cast<uint4*>(orow + 32 * c + 8 * i) = w;
            }
          }
        }
      } else {
        // half 0 stores the dV row, half 1 the dK row (scaled)
        const float mul = half == 0 ? 1.f : p.scale;
        T* orow = static_cast<T*>(half == 0 ? p.out1 : p.out0) +
                  ((static_cast<long long>(b) * p.T + pos) * p.Hkv + hk) * static_cast<long long>(D);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_addr(tmem, lane_base, kOutCol + half * D + 32 * c), r);
          tc_wait_ld();
          if (pos < p.T) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = Pack2<T>::pack(__uint_as_float(r[8 * i + 0]) * mul, __uint_as_float(r[8 * i + 1]) * mul);
              w.y = Pack2<T>::pack(__uint_as_float(r[8 * i + 2]) * mul, __uint_as_float(r[8 * i + 3]) * mul);
              w.z = Pack2<T>::pack(__uint_as_float(r[8 * i + 4]) * mul, __uint_as_float(r[8 * i + 5]) * mul);
              w.w = Pack2<T>::pack(__uint_as_float(r[8 * i + 6]) * mul, __uint_as_float(r[8 * i + 7]) * mul);
              *reinterpret_cast<uint4*>(orow + 32 * c + 8 * i) = w;
            }
          }
        }
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
}

template <typename T, int D, int MODE, int STAGES>
int launch_mode(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk,
                const CUtensorMap& mv, const CUtensorMap& mdo, const float* lse,
                const float* delta, void* out0, void* out1, unsigned* status,
                cudaStream_t stream) {
  using L = BwdSmem<D, STAGES>;
  auto kern = bwd_tc_kernel<T, D, MODE, STAGES>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) !=
      cudaSuccess)
    return NLFA_ERR_CUDA;
  BwdParams bp;
  bp.T = p.T;
  bp.H = p.H;
  bp.Hkv = p.Hkv;
  bp.window = p.window;
  bp.sinks = p.sinks;
  bp.n_tiles = (p.T + kTile - 1) / kTile;
  bp.scale = p.scale;
  bp.scale_log2 = p.scale * kLog2e;
  bp.lse = lse;
  bp.delta = delta;
  bp.out0 = out0;
  bp.out1 = out1;
  bp.status = status;
  dim3 grid(bp.n_tiles, p.B * (MODE == MODE_DQ ? p.H : p.Hkv));
  kern<<<grid, 320, L::kDynamic, stream>>>(mq, mk, mv, mdo, bp);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

template <typename T, int D, int STAGES>
int launch_both(const Problem& p, const CUtensorMap& mq, const CUtensorMap& mk,
                const CUtensorMap& mv, const CUtensorMap& mdo, const float* lse,
                const float* delta, void* dq, void* dk, void* dv, int passes, unsigned* status,
                cudaStream_t stream) {
  int st = NLFA_OK;
  if (passes & NLFA_PASS_DKV)
    st = launch_mode<T, D, MODE_DKV, STAGES>(p, mq, mk, mv, mdo, lse, delta, dk, dv, status, stream);
  if (st != NLFA_OK) return st;
  if (passes & NLFA_PASS_DQ)
    st = launch_mode<T, D, MODE_DQ, STAGES>(p, mq, mk, mv, mdo, lse, delta, dq, nullptr, status, stream);
  return st;
}

}  // namespace

int launch_bwd_tc(const Problem& p, const void* dout, const void* q, const void* k, const void* v,
                  const void* o, const float* lse, void* dq, void* dk, void* dv, float* delta,
                  int passes, unsigned* status, cudaStream_t stream) {
  if (p.dtype != NLFA_DTYPE_F16 && p.dtype != NLFA_DTYPE_BF16) return NLFA_ERR_UNSUPPORTED_PATH;
  if (p.D != 64 && p.D != 128) return NLFA_ERR_UNSUPPORTED_PATH;
  int st = NLFA_OK;
  if (passes & NLFA_PASS_DELTA) st = launch_delta(p, dout, o, delta, stream);
  if (st != NLFA_OK) return st;
  CUtensorMap mq, mk, mv, mdo;
  st = make_tile_map(&mq, q, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mk, k, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mv, v, p.dtype, p.B, p.T, p.Hkv, p.D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mdo, dout, p.dtype, p.B, p.T, p.H, p.D, kTile);
  if (st != NLFA_OK) return st;
  const bool bf16 = p.dtype == NLFA_DTYPE_BF16;
  if (p.D == 64) {
    return bf16 ? launch_both<__nv_bfloat16, 64, 3>(p, mq, mk, mv, mdo, lse, delta, dq, dk, dv, passes, status, stream)
                : launch_both<__half, 64, 3>(p, mq, mk, mv, mdo, lse, delta, dq, dk, dv, passes, status, stream);
  }
  return bf16 ? launch_both<__nv_bfloat16, 128, 2>(p, mq, mk, mv, mdo, lse, delta, dq, dk, dv, passes, status, stream)
              : launch_both<__half, 128, 2>(p, mq, mk, mv, mdo, lse, delta, dq, dk, dv, passes, status, stream);
}

}  // namespace nlfa
