// Shared host/device definitions for the attention library.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/nlfa.h"

namespace nlfa {

constexpr int kTile = 128;          // query rows per tile and keys per block
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// One attention problem.  Layouts follow the reference kernel's contract
// (nanolab/csrc/flash_attn_cuda.cu:1628-1650): q, o, dout, dq are contiguous
// [B,T,H,D]; k, v, dk, dv are contiguous [B,T,Hkv,D]; lse and delta are fp32
// [B,H,T]; lse is a natural-log logsumexp.
struct Problem {
  int B, T, H, Hkv, D;
  int window, sinks;     // window == 0: plain causal
  float scale;
  int dtype;             // NLFA_DTYPE_*
  int block = 0;         // > 0: block-causal (bidirectional inside blocks of this many positions); needs window == 0
};

// Block-causal attention (nanolab/mixers.py:78-93, `block_causal_mask`): a query sees every
// position of its own block and of all earlier blocks, i.e. query q sees the keys up to the end
// of its block, and key k is seen by the queries from the start of its block on.  block == 0
// (or 1) is plain causal attention.  A block may reach past the end of the sequence (`t_len`
// positions): the keys stop there.
__host__ __device__ inline int last_key_of_query(int q, int block, int t_len = 1 << 30) {
  if (block <= 1) return q;
  const int last = (q / block + 1) * block - 1;
  return last < t_len - 1 ? last : t_len - 1;
}
__host__ __device__ inline int first_query_of_key(int k, int block) {
  return block > 1 ? (k / block) * block : k;
}

// Which key blocks a 128-row query tile must visit.  Block j covers keys
// [128 j, 128 j + 127].  The mask is the reference's sliding_window_mask
// (nanolab/mixers.py:125-132): keep k <= q and (k > q - (window - sinks) or
// k < sinks).
struct TileRange {
  int lo, hi;            // contiguous range of recent blocks, inclusive
  int sink_blocks;       // blocks [0, sink_blocks) hold sink keys
};

// `block` > 0 (block-causal; window must be 0) lets a tile see past the diagonal, up to the end
// of its last row's block; `n_tiles` bounds that.
__host__ __device__ inline TileRange tile_range(int tile, int window, int sinks, int block = 0,
                                                int n_tiles = 1 << 30) {
  TileRange r;
  r.hi = last_key_of_query(tile * kTile + kTile - 1, block) / kTile;
  r.hi = r.hi < n_tiles - 1 ? r.hi : n_tiles - 1;
  r.lo = 0;
  r.sink_blocks = 0;
  if (window > 0) {
    const int span = window - sinks;
    const int first_key = tile * kTile - span + 1;     // lowest recent key of the tile's first row
    r.lo = first_key > 0 ? first_key / kTile : 0;
    r.sink_blocks = (sinks + kTile - 1) / kTile;
  }
  return r;
}

// True when every (row, key) of query tile `tile` x key block `j` survives the
// mask, so the element-wise predicate can be skipped.
__host__ __device__ inline bool block_fully_visible(int tile, int j, int window, int sinks, int block = 0,
                                                    int t_len = 1 << 30) {
  if (j * kTile + kTile - 1 > last_key_of_query(tile * kTile, block, t_len)) return false;   // the causal edge cuts in
  if (window > 0) {
    const int span = window - sinks;
    const int last_row = tile * kTile + kTile - 1;
    if (j * kTile <= last_row - span) return false;              // lower window edge cuts in
  }
  return true;
}

// Which edges of the mask cut through query tile `tile` x key block `j` (for blocks that are
// not fully visible): only the causal edge k <= q (plain causal, or windows whose lower edge
// stays below the block), only the window's lower edge k > q - (window - sinks) (blocks below
// the diagonal that hold no sink keys), or both / sinks involved.  One-edge blocks need a
// single compare per element against a per-thread limit.
enum { EDGE_CAUSAL = 0, EDGE_WINDOW = 1, EDGE_BOTH = 2 };
__host__ __device__ inline int block_edges(int tile, int j, int window, int sinks) {
  if (window == 0) return EDGE_CAUSAL;
  const int span = window - sinks;
  const int last_row = tile * kTile + kTile - 1;
  if (j * kTile > last_row - span) return EDGE_CAUSAL;           // lower edge below the block
  if (j < tile && j * kTile >= sinks) return EDGE_WINDOW;        // causal edge above, no sink keys
  return EDGE_BOTH;
}

// The same two questions for a rectangle of query positions [q_lo, q_hi] x key positions
// [k_lo, k_hi] (tiles of unequal height).
__host__ __device__ inline bool rect_fully_visible(int q_lo, int q_hi, int k_lo, int k_hi,
                                                   int window, int sinks, int block = 0, int t_len = 1 << 30) {
  if (k_hi > last_key_of_query(q_lo, block, t_len)) return false;          // causal edge cuts in
  if (window > 0 && k_lo <= q_hi - (window - sinks)) return false;         // lower window edge cuts in
  return true;
}
__host__ __device__ inline int rect_edges(int q_lo, int q_hi, int k_lo, int k_hi, int window,
                                          int sinks) {
  if (window == 0) return EDGE_CAUSAL;
  if (k_lo > q_hi - (window - sinks)) return EDGE_CAUSAL;                  // lower edge below the rectangle
  if (k_hi <= q_lo && k_lo >= sinks) return EDGE_WINDOW;                   // causal edge above, no sink keys
  return EDGE_BOTH;
}

// Key-block-stationary passes (dK/dV, fused): the last streamed query tile (of `rows` rows each,
// `n_ytiles` in all) that reaches 128-key block `block`; the first is block * (128 / rows).
__host__ __device__ inline int last_query_tile_of_block(int block, int n_ytiles, int rows, int window,
                                                        int sinks) {
  int hi = n_ytiles - 1;
  if (window > 0 && block >= (sinks + kTile - 1) / kTile) {      // blocks with sink keys are seen by all
    const int last_q = block * kTile + kTile - 1 + (window - sinks) - 1;
    hi = last_q / rows < hi ? last_q / rows : hi;
  }
  return hi;
}

// Fused backward: key block `block`'s place in the fixed order in which the blocks that see
// 128-row query tile `tile` add their dQ shares (ascending block index: sink blocks below the
// window first, then the window's blocks up to the last one the tile sees -- the diagonal, or
// beyond it under a block-causal mask of `mask_block` positions).  *count is the number of such blocks.
__host__ __device__ inline int dq_turn_of_block(int block, int tile, int window, int sinks, int* count,
                                                int mask_block = 0, int n_tiles = 1 << 30) {
  const TileRange r = tile_range(tile, window, sinks, mask_block, n_tiles);
  const int extra = r.sink_blocks < r.lo ? r.sink_blocks : r.lo;
  *count = extra + (r.hi - r.lo + 1);
  return block < extra ? block : extra + (block - r.lo);
}

__host__ __device__ inline bool key_visible(int q, int k, int window, int sinks, int block = 0,
                                            int t_len = 1 << 30) {
  if (k > last_key_of_query(q, block, t_len)) return false;
  if (window == 0) return true;
  return (k > q - (window - sinks)) || (k < sinks);
}

// Host-side launchers (one per translation unit); all return an NLFA_* status.
int launch_fwd_simt(const Problem& p, const void* q, const void* k, const void* v, void* o,
                    float* lse, cudaStream_t stream);
int launch_bwd_simt(const Problem& p, const void* dout, const void* q, const void* k,
                    const void* v, const void* o, const float* lse, void* dq, void* dk, void* dv,
                    float* delta, int passes, cudaStream_t stream);
int launch_delta(const Problem& p, const void* dout, const void* o, float* delta,
                 cudaStream_t stream);
int launch_fwd_tc(const Problem& p, const void* q, const void* k, const void* v, void* o,
                  float* lse, unsigned* status, cudaStream_t stream);
// Scratch of the fused backward pass (head dim <= 64), behind the Delta tape in the caller's
// buffer: per (batch, head, 128-row query tile) a turn counter and 128 x 64 fp32 partial sums.
struct FusedScratch {
  float* dq_acc;
  unsigned* dq_turn;
};
int launch_bwd_tc(const Problem& p, const void* dout, const void* q, const void* k, const void* v,
                  const void* o, const float* lse, void* dq, void* dk, void* dv, float* delta,
                  int passes, unsigned* status, cudaStream_t stream, const FusedScratch* fused);
int launch_selftest_tiles(int dtype, int head_dim, const void* q, const void* k, const void* v,
                          float* s_out, float* o_out, unsigned* status, cudaStream_t stream);

// Encodes a 4-D tensor map over a contiguous [B,T,heads,D] 16-bit tensor with a
// box of 64 elements x 1 head x `rows` rows x 1 batch and 128-byte swizzle.  Encoded maps are
// kept in a small host-side table keyed by (base, dtype, shape, rows): a training loop calls
// with the same buffers step after step, and the driver's encoder costs a microsecond or two
// per map (ten maps per forward + backward).
int make_tile_map(CUtensorMap* map, const void* base, int dtype, int B, int T, int heads, int D,
                  int rows);

// Two work counters for one launch of a persistent kernel ([0] next unit, [1] CTAs finished;
// the last CTA of a launch zeroes them again).  Launches on a capturing stream draw from a
// range of their own whose entries are never handed out twice, because a captured graph keeps
// the address for as long as it is replayed; eager launches take turns on a ring.  Returns an
// NLFA_* status (NLFA_ERR_GRAPH_SLOTS when the graph range is used up).
int sched_counters(cudaStream_t stream, unsigned** out);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize), once per kernel and device.
int ensure_dynamic_smem(const void* kernel, int bytes);

int sm_count();

// Which kernels are launched with programmatic stream serialization, so that their set-up
// (barriers, TMEM, descriptors) overlaps the predecessor's last CTAs.  NLFA_PDL=<mask> overrides
// the default (0: none).
enum { kOverlapFwd = 1, kOverlapDelta = 2, kOverlapDkv = 4, kOverlapDq = 8, kOverlapDefault = 15 };
bool overlap_launches(int kernel);

// Whether the tensor-core backward forms Delta inside its dQ pass for this problem and mask
// (bwd_tc.cu); then it launches two kernels instead of three.
bool bwd_delta_in_dq(const Problem& p, int passes);

// One launch through cudaLaunchKernelEx, with the programmatic-serialization attribute when
// `overlap` is set.  The kernel must then call grid_dep_wait() before it reads anything an earlier
// kernel of the stream wrote.
template <typename... Params, typename... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool overlap, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

}  // namespace nlfa
