// One-tile hardware check of the operand paths the tensor-core kernels rely on.
//
//   S = Q K^T      A and B from shared memory, both K-major, 128B-swizzled TMA tiles
//   P = round16(S) written back to TMEM as packed 16-bit pairs
//   O = P V        A read from TMEM, B = V from shared memory, MN-major
//
// The layouts involved (descriptor fields, TMEM lane/column mapping, packing of
// the TMEM A operand) are fixed by the hardware and cannot be verified on a CPU,
// so this plays the role the reference gives its `mma_probe_kernel`
// (nanolab/csrc/flash_attn_cuda.cu:1197-1225): multiply known matrices through
// the same helpers the real kernels use and compare with a plain matmul.
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace nlfa {
namespace {

template <typename T, int D>
__global__ void __launch_bounds__(128, 1)
selftest_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, float* __restrict__ s_out,
                float* __restrict__ o_out, unsigned* status) {
  constexpr int kBoxes = D / 64;
  constexpr int kBoxBytes = kTile * 128;
  constexpr int kTileBytes = kTile * D * 2;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t q_s = base, k_s = base + kTileBytes, v_s = base + 2 * kTileBytes;
  const uint32_t bars = base + 3 * kTileBytes;          // [0] loads, [1] S done, [2] O done
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + 3 * kTileBytes + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + 3 * kTileBytes + 40);
  const WaitCtx wctx{abort_flag, status};
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bars + 0, 1);
    mbar_init(bars + 8, 1);
    mbar_init(bars + 16, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  bool ok = true;
  if (threadIdx.x == 0) {
    mbar_arrive_expect_tx(bars + 0, 3 * kTileBytes);
    for (int x = 0; x < kBoxes; ++x) {
      tma_load_4d(q_s + x * kBoxBytes, &tm_q, bars + 0, 64 * x, 0, 0, 0);
      tma_load_4d(k_s + x * kBoxBytes, &tm_k, bars + 0, 64 * x, 0, 0, 0);
      tma_load_4d(v_s + x * kBoxBytes, &tm_v, bars + 0, 64 * x, 0, 0, 0);
    }
    ok = mbar_wait(bars + 0, 0, wctx, 20);
    if (ok) {
      tc_fence_after();
      constexpr uint32_t idesc_qk = make_idesc(kBf16, 128, 128, false, false);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * kBoxBytes + (kk & 3) * 32;
        mma_ss(tmem, make_smem_desc(q_s + off, 16, 1024), make_smem_desc(k_s + off, 16, 1024),
               idesc_qk, kk > 0 ? 1u : 0u);
      }
      tc_commit(bars + 8);
    }
  }
  __syncwarp();

  // every thread: its row of S out of TMEM, to global, and back as 16-bit P
  ok = mbar_wait(bars + 8, 0, wctx, 21);
  ok = __all_sync(0xffffffffu, ok);
  const uint32_t lane_base = 32u * (warp & 3);
  const int row = threadIdx.x;
  if (ok) {
    tc_fence_after();
    uint32_t pk[2][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t sr[32];
      tmem_ld32(tmem_addr(tmem, lane_base, 32 * c), sr);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s_out[row * 128 + 32 * c + i] = __uint_as_float(sr[i]);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        pk[c >> 1][(c & 1) * 16 + i] =
            Pack2<T>::pack(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
    }
    tmem_st32(tmem_addr(tmem, lane_base, 0), pk[0]);
    tmem_st32(tmem_addr(tmem, lane_base, 32), pk[1]);
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (threadIdx.x == 0 && ok) {
    constexpr uint32_t idesc_pv = make_idesc(kBf16, 128, D, false, true);
#pragma unroll
    for (int kk = 0; kk < kTile / 16; ++kk)
      mma_ts(tmem + 128, tmem + 8 * kk, make_smem_desc(v_s + kk * 2048, kBoxBytes, 1024), idesc_pv,
             kk > 0 ? 1u : 0u);
    tc_commit(bars + 16);
  }
  __syncwarp();
  if (ok) {
    ok = mbar_wait(bars + 16, 0, wctx, 22);
    ok = __all_sync(0xffffffffu, ok);
  }
  if (ok) {
    tc_fence_after();
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t orr[32];
      tmem_ld32(tmem_addr(tmem, lane_base, 128 + 32 * c), orr);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_out[row * D + 32 * c + i] = __uint_as_float(orr[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

template <typename T, int D>
int run_t(int dtype, const void* q, const void* k, const void* v, float* s_out, float* o_out,
          unsigned* status, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  int st = make_tile_map(&mq, q, dtype, 1, kTile, 1, D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mk, k, dtype, 1, kTile, 1, D, kTile);
  if (st == NLFA_OK) st = make_tile_map(&mv, v, dtype, 1, kTile, 1, D, kTile);
  if (st != NLFA_OK) return st;
  constexpr int smem = 3 * kTile * D * 2 + 64 + 1024;
  auto kern = selftest_kernel<T, D>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return NLFA_ERR_CUDA;
  kern<<<1, 128, smem, stream>>>(mq, mk, mv, s_out, o_out, status);
  return cudaGetLastError() == cudaSuccess ? NLFA_OK : NLFA_ERR_CUDA;
}

}  // namespace

int launch_selftest_tiles(int dtype, int head_dim, const void* q, const void* k, const void* v,
                          float* s_out, float* o_out, unsigned* status, cudaStream_t stream) {
  if (dtype == NLFA_DTYPE_BF16 && head_dim == 64)
    return run_t<__nv_bfloat16, 64>(dtype, q, k, v, s_out, o_out, status, stream);
  if (dtype == NLFA_DTYPE_BF16 && head_dim == 128)
    return run_t<__nv_bfloat16, 128>(dtype, q, k, v, s_out, o_out, status, stream);
  if (dtype == NLFA_DTYPE_F16 && head_dim == 64)
    return run_t<__half, 64>(dtype, q, k, v, s_out, o_out, status, stream);
  if (dtype == NLFA_DTYPE_F16 && head_dim == 128)
    return run_t<__half, 128>(dtype, q, k, v, s_out, o_out, status, stream);
  return NLFA_ERR_UNSUPPORTED_PATH;
}

}  // namespace nlfa
