/*
 * nlfa -- causal / sliding-window flash attention for NVIDIA B200 (sm_100a).
 *
 * Plain C ABI.  The caller owns every buffer (inputs, outputs, the logsumexp
 * tape and the backward's scratch); the library allocates no device memory and
 * launches on the stream it is given, on the device that is current.
 *
 * This is the native boundary behind nanolab's `--flash_cuda` path.  It stands
 * where the reference's pybind11 module `nanolab_flash_attn` stands
 * (nanolab/csrc/flash_attn_cuda.cu:1815-1825: `fwd`, `bwd`, `mma_probe`).
 *
 * Layout contract (same as nanolab/csrc/flash_attn_cuda.cu:1628-1650, :1756-1762):
 *   q, o, dout, dq : contiguous [B, T, H,   D]
 *   k, v, dk, dv   : contiguous [B, T, Hkv, D],  Hkv > 0 and H % Hkv == 0
 *   lse, delta     : contiguous [B, H, T] float32; lse is a natural-log logsumexp
 *   all of q/k/v/o/dout/dq/dk/dv share one dtype; base pointers 16-byte aligned
 *   D in {32, 64, 128}
 *
 * Mask: query i attends key j iff  j <= i  and, when window > 0,
 *   (j > i - (window - sinks)  or  j < sinks)   with 0 <= sinks < window
 * which is nanolab/mixers.py:125-132 (`sliding_window_mask`).  window == 0 is
 * plain causal attention (the only mask the reference kernel has).
 */
#ifndef NLFA_H_
#define NLFA_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of q/k/v/o and the gradients */
#define NLFA_DTYPE_F32 0
#define NLFA_DTYPE_F16 1
#define NLFA_DTYPE_BF16 2

/* kernel family; mirrors `use_mma` of nanolab/flash_cuda.py:233-279
 * (None -> AUTO, False -> SIMT, True -> TENSOR) */
#define NLFA_PATH_AUTO 0
#define NLFA_PATH_SIMT 1   /* fp32 FMA kernels: every dtype, every head dim */
#define NLFA_PATH_TENSOR 2 /* TMA + tcgen05 + TMEM kernels: f16/bf16 (D = 32 on 64-wide tiles) */

/* status codes: 0 is success, everything else is a refusal or a failure */
#define NLFA_OK 0
#define NLFA_ERR_NULL_POINTER 1
#define NLFA_ERR_BAD_SHAPE 2
#define NLFA_ERR_BAD_DTYPE 3
#define NLFA_ERR_BAD_HEAD_DIM 4
#define NLFA_ERR_BAD_WINDOW 5
#define NLFA_ERR_MISALIGNED 6
#define NLFA_ERR_UNSUPPORTED_PATH 7
#define NLFA_ERR_NOT_SM100 8
#define NLFA_ERR_CUDA 9
#define NLFA_ERR_DEVICE_TIMEOUT 10
#define NLFA_ERR_SCRATCH_TOO_SMALL 11
#define NLFA_ERR_SELFTEST_MISMATCH 12
#define NLFA_ERR_STATIC_SCRATCH_EXCEEDED 13
#define NLFA_ERR_BAD_ARGUMENT 14
#define NLFA_ERR_GRAPH_SLOTS 15

/* Library version, bumped when the ABI changes. */
int nlfa_version(void);

/* Human-readable text for a status code; never NULL. */
const char* nlfa_strerror(int status);

/* 1 if the current device can run the tensor-core path (compute capability
 * 10.x), else 0.  Replaces the capability half of the reference's load-time
 * probe (nanolab/flash_cuda.py:59-88). */
int nlfa_device_supported(void);

/* The path AUTO resolves to for this dtype and head dim (NLFA_PATH_SIMT or
 * NLFA_PATH_TENSOR), or a negative status code if the combination is refused.
 * Plays the role of the reference's dtype x head_dim dispatch
 * (nanolab/csrc/flash_attn_cuda.cu:1592-1626). */
int nlfa_resolve_path(int dtype, int head_dim, int path);

/* Forward: O = softmax(scale * Q K^T + mask) V and the per-row logsumexp.
 * Replaces `flash_attn_fwd` (nanolab/csrc/flash_attn_cuda.cu:1655-1704) and the
 * kernels it launches (:147-281, :583-797); unlike it, the caller allocates o
 * and lse.  B, T or H of zero is a successful no-op (:1668). */
int nlfa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
             int H, int Hkv, int D, float scale, int window, int sinks, int dtype, int path,
             void* stream);

/* Forward with the mask given in full: the sliding window above, or -- with block > 0, which
 * needs window == 0 -- the block-causal mask of nanolab's semi-autoregressive / diffusion mode
 * (nanolab/mixers.py:78-93, `block_causal_mask`: blk = position / block; keep key k for query q
 * iff blk[q] >= blk[k], i.e. every position of the query's own block and of all earlier
 * blocks).  block of 0 or 1 is plain causal attention; block >= T is fully bidirectional.  The
 * reference runs this mask through SDPA with a [T,T] boolean tensor (mixers.py:319-321); here the
 * kernels apply it from positions and skip the key blocks beyond a tile's reach.  nlfa_fwd is
 * this with block = 0. */
int nlfa_fwd_masked(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T,
                    int H, int Hkv, int D, float scale, int window, int sinks, int block, int dtype,
                    int path, void* stream);

/* Bytes of device scratch `nlfa_bwd` needs (the Delta tape, [B,H,T] float32).
 * The reference allocates the same tensor itself (flash_attn_cuda.cu:1770-1773). */
size_t nlfa_bwd_scratch_bytes(int B, int T, int H);

/* Backward: Delta = rowsum(dO * O), then dQ, dK, dV with P recomputed from the
 * taped lse.  Replaces `flash_attn_bwd` (nanolab/csrc/flash_attn_cuda.cu:1744-1813)
 * and its launch sequence (:1518-1587): Delta kernel, dK/dV kernel, dQ kernel on
 * one stream (two kernels for large problems at D = 64, see
 * nlfa_bwd_kernel_count), no atomics, bit-reproducible.  `scratch` must hold
 * nlfa_bwd_scratch_bytes(B, T, H) bytes; Delta is left in it. */
int nlfa_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
             const float* lse, void* dq, void* dk, void* dv, void* scratch, size_t scratch_bytes,
             int B, int T, int H, int Hkv, int D, float scale, int window, int sinks, int dtype,
             int path, void* stream);

/* The backward's three passes, individually selectable so that each kernel can be
 * timed or profiled on its own: `passes` is a bit mask of NLFA_PASS_*.  The dQ
 * and dK/dV passes read the Delta tape in `scratch`, which the Delta pass (or an
 * earlier call) must have written.  nlfa_bwd is this with every pass selected.
 * The three kernels are the reference's `flash_delta_kernel`, dQ and dK/dV
 * kernels (flash_attn_cuda.cu:1234-1262, :806-971, :983-1191). */
#define NLFA_PASS_DELTA 1
#define NLFA_PASS_DKV 2
#define NLFA_PASS_DQ 4
#define NLFA_PASS_ALL 7
#define NLFA_PASS_FUSED 8 /* dK, dV and dQ in one pass (see nlfa_bwd_fused); excludes DKV and DQ */
int nlfa_bwd_passes(const void* dout, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, void* dq, void* dk, void* dv, void* scratch,
                    size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                    int window, int sinks, int dtype, int path, int passes, void* stream);

/* How many kernels nlfa_bwd_passes launches for this problem and mask on the
 * current device (0 for inputs it would refuse).  On the tensor-core path at
 * D = 64 a large problem (at least sixteen 128-row query tiles per SM) takes two:
 * the dQ pass forms Delta itself -- the row sums of dO * O, added in the order of
 * the Delta kernel, so the gradients are bit-identical either way -- and runs
 * before the dK/dV pass; smaller problems and other head dims take the three
 * kernels named above.  For launch accounting (bench.py's `gpu_launches`). */
int nlfa_bwd_kernel_count(int B, int T, int H, int D, int dtype, int path, int passes);

/* nlfa_bwd_passes with the mask given in full (`block` as in nlfa_fwd_masked). */
int nlfa_bwd_masked(const void* dout, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, void* dq, void* dk, void* dv, void* scratch,
                    size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                    int window, int sinks, int block, int dtype, int path, int passes, void* stream);

/* The backward with dQ formed in the dK/dV pass: P and dS are computed once per
 * (query tile, key block) instead of once in each of the reference's two passes
 * (nanolab/csrc/flash_attn_cuda.cu:806-971 and :983-1191 both recompute them, by
 * design, :48-52).  Every key block adds its 128 x 64 share dS K to fp32 sums of
 * the query tile in `scratch`; the additions happen in a fixed order (ascending
 * key block, enforced by a turn counter per query tile), so the gradients stay
 * bit-reproducible like the reference's (nanolab/tests.py:415-420); a second
 * small kernel turns the sums into dQ.  Tensor-core path with D <= 64; for other
 * inputs this is nlfa_bwd.  `scratch` must be 16-byte aligned and hold
 * nlfa_bwd_fused_scratch_bytes(B, T, H, D) bytes (the Delta tape, the counters,
 * and B * H * ceil(T / 128) * 32 KiB of sums); nothing in it needs initialising.
 * Same arguments and results as nlfa_bwd, to rounding: dQ is summed block by
 * block in fp32 here and inside one accumulator there; dK and dV are identical.
 * An alternative layout, not the default: on B200 the two passes of nlfa_bwd
 * are faster at these head dims (B=32, H=12, T=1024, D=64 bf16: 0.32 ms against
 * 0.26 ms, both without the Delta kernel). */
size_t nlfa_bwd_fused_scratch_bytes(int B, int T, int H, int D);
int nlfa_bwd_fused(const void* dout, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, void* dq, void* dk, void* dv, void* scratch,
                   size_t scratch_bytes, int B, int T, int H, int Hkv, int D, float scale,
                   int window, int sinks, int dtype, int path, void* stream);

/* The backward without a caller-supplied scratch buffer.  No counterpart in the
 * reference (its backward allocates its own tape with at::empty).
 *
 * For callers that cannot give nlfa_bwd a scratch buffer: processes whose device
 * memory is already committed in full to some other allocator or budget, and
 * code paths that may not make a call that allocates.  The Delta tape lives in
 * a fixed 4 MiB array inside the library's device image instead, which every
 * GPU that loads the library carries until the process exits.
 *
 *  - Limit: B * H * T <= nlfa_static_scratch_max_rows() (1,048,576); larger
 *    problems are refused with NLFA_ERR_STATIC_SCRATCH_EXCEEDED.
 *  - The first call made with a given device current looks up the array's
 *    address on that device (cudaGetSymbolAddress) and caches it.  Make that
 *    first call outside any stream capture.
 *  - All calls on a device share the one array.  It keeps whatever the last call
 *    wrote; every call rewrites all rows it later reads, so nothing has to be
 *    cleared.  Two calls whose kernels can overlap on the GPU (different
 *    streams, no dependency) race on it: serialise them.
 *  - Neither this function nor anything it calls uses cudaMalloc or an allocating
 *    library routine, and nothing is freed.
 * Arguments, results and gradients are exactly those of nlfa_bwd. */
size_t nlfa_static_scratch_max_rows(void);
int nlfa_bwd_static_scratch(const void* dout, const void* q, const void* k, const void* v,
                            const void* o, const float* lse, void* dq, void* dk, void* dv, int B,
                            int T, int H, int Hkv, int D, float scale, int window, int sinks,
                            int dtype, int path, void* stream);

/* Load-side prologue of the attention core for q or k, in one pass over the tensor:
 * per-head RMSNorm (weight [D], eps), rotary embedding (cos / sin tables [T, D]
 * float32, half-split convention: out = y * cos + (-y_hi, y_lo) * sin) and the cast
 * to the kernel dtype.  Replaces, in front of every attention call, the separate
 * tensor passes of nanolab/mixers.py:287-292 (`q_norm` / `k_norm`, RMSNorm at
 * :46-56, and `apply_rope`, :68-75) and the cast + contiguous of
 * nanolab/flash_cuda.py:263-266.
 *   x [B,T,H,D] of x_dtype -> y [B,T,H,D] of y_dtype; rstd [B*T*H] float32 receives
 *   1/rms of every row (the backward's tape) when weight != NULL.
 *   weight == NULL skips the norm; cos_table == sin_table == NULL skips the rotation.
 * For 16-bit x the normalised, weighted row is rounded to x_dtype before the
 * rotation, as torch's rms_norm does (it returns its input's type). */
int nlfa_qk_prologue_fwd(const void* x, int x_dtype, const float* weight, const float* cos_table,
                         const float* sin_table, void* y, int y_dtype, float* rstd, int B, int T,
                         int H, int D, float eps, void* stream);

/* Bytes of device scratch `nlfa_qk_prologue_bwd` needs for a head dim (per-CTA
 * partial sums of the weight gradient; needed only when weight != NULL). */
size_t nlfa_qk_prologue_scratch_bytes(int D);

/* Backward of nlfa_qk_prologue_fwd: gy [B,T,H,D] of gy_dtype (the gradient of y,
 * i.e. dq or dk of the attention backward) -> gx [B,T,H,D] of x_dtype and
 * gweight [D] float32 (overwritten).  Stands where autograd's backward of the
 * same nanolab lines stands.  The weight gradient is reduced in a fixed order
 * (per-CTA partial sums in `scratch`, then one small kernel): bit-reproducible. */
int nlfa_qk_prologue_bwd(const void* gy, int gy_dtype, const void* x, int x_dtype,
                         const float* weight, const float* cos_table, const float* sin_table,
                         const float* rstd, void* gx, float* gweight, void* scratch,
                         size_t scratch_bytes, int B, int T, int H, int D, void* stream);

/* Value-residual blend in front of the attention core, with the cast to the kernel
 * dtype: out = (1 - s) * v + s * v0, s = sigmoid(*lambda) (lambda: one float32 on the
 * device).  Replaces the tensor passes of nanolab/mixers.py:294-297 and the cast of
 * v in nanolab/flash_cuda.py:263-266.  v, v0 share v_dtype; n = element count, a
 * multiple of 8 (head dims are). */
int nlfa_value_blend_fwd(const void* v, const void* v0, int v_dtype, const float* lambda, void* out,
                         int out_dtype, long long n, void* stream);

/* Bytes of device scratch `nlfa_value_blend_bwd` needs (per-CTA partial sums). */
size_t nlfa_value_blend_scratch_bytes(void);

/* Backward of nlfa_value_blend_fwd: g (gradient of out, g_dtype) -> dv = (1 - s) g and
 * dv0 = s g in v_dtype, *dlambda = s (1 - s) sum(g * (v0 - v)) (float32, overwritten;
 * summed in a fixed order).  Stands where autograd's backward of mixers.py:294-297 stands. */
int nlfa_value_blend_bwd(const void* g, int g_dtype, const void* v, const void* v0, int v_dtype,
                         const float* lambda, void* dv, void* dv0, float* dlambda, void* scratch,
                         size_t scratch_bytes, long long n, void* stream);

/* Per-head sigmoid gate behind the attention core: out = y * sigmoid(gate)[..., None],
 * y and out [rows, D] of y_dtype, gate [rows] of gate_dtype (rows = B*T*H).  The sigmoid
 * is rounded to gate_dtype before the multiply, as torch does.  Replaces
 * nanolab/mixers.py:340-342. */
int nlfa_head_gate_fwd(const void* y, int y_dtype, const void* gate, int gate_dtype, void* out,
                       long long rows, int D, void* stream);

/* Backward of nlfa_head_gate_fwd: g (gradient of out) and the forward's y, gate ->
 * dy = g * sigmoid(gate) [rows, D] and dgate = rowsum(g * y) * s * (1 - s) [rows]. */
int nlfa_head_gate_bwd(const void* g, const void* y, int y_dtype, const void* gate, int gate_dtype,
                       void* dy, void* dgate, long long rows, int D, void* stream);

/* Forward attention of an active block of Tq queries over [cache | block], masked by
 * absolute positions: the attention core of nanolab's KV-cached block forward
 * (`Attention.forward_cached`, nanolab/mixers.py:372-467), which nanolab runs as a
 * torch.cat, a repeat_interleave and a masked SDPA.  Forward only.
 *   q, o [B,Tq,H,D]; k_cache, v_cache [B,Hkv,L,D] (nanolab's cache layout, the block's own
 *   keys last); lse [B,H,Tq] float32 natural log, or NULL; qpos [Tq], kpos [L] int32 on the
 *   device, or NULL for contiguous positions (keys 0..L-1, the block at L-Tq..L-1).
 * Mask: window > 0 (needs causal): kpos <= qpos and (kpos > qpos - (window - sinks) or
 * kpos < sinks) (mixers.py:417-432; positions stay correct after cache eviction);
 * causal: kpos <= qpos (:433-437); neither: every key.  A row that sees no key gives
 * zeros and lse = -inf.
 * `scratch` is optional: with nlfa_fwd_cached_scratch_bytes(...) bytes of device memory the
 * keys are split over several CTAs when there are few query rows (long caches, small
 * batches) and a second small kernel combines the partial rows in a fixed order; with
 * NULL (or too little) one CTA walks all keys of its rows.  Same results up to fp32
 * rounding. */
size_t nlfa_fwd_cached_scratch_bytes(int B, int Tq, int H, int Hkv, int L, int D);
int nlfa_fwd_cached(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                    const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                    float scale, int causal, int window, int sinks, int dtype, void* scratch,
                    size_t scratch_bytes, void* stream);

/* The same with the kernel family chosen by the caller (NLFA_PATH_*).  AUTO, which is what
 * nlfa_fwd_cached does, takes the tensor-core kernel (TMA + tcgen05, keys in blocks of 128, the
 * query rows of a KV head's whole group in one tile) for 16-bit inputs when the block has at
 * least 16 rows per KV head (Tq x group) and the cache at least 256 keys, on a compute-capability
 * 10.x device with 16-byte-aligned pointers and a positive scale; otherwise the fp32 kernel.
 * TENSOR returns NLFA_ERR_UNSUPPORTED_PATH when those conditions do not hold. */
int nlfa_fwd_cached_path(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                         const int* qpos, const int* kpos, int B, int Tq, int H, int Hkv, int L, int D,
                         float scale, int causal, int window, int sinks, int dtype, int path,
                         void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of device workspace `nlfa_selftest` needs. */
size_t nlfa_selftest_workspace_bytes(void);

/* Load-time hardware check.  Runs one 128-row tile through the exact operand
 * paths the tensor-core kernels use (TMA 128B-swizzled tiles, K-major and
 * MN-major shared-memory descriptors, an A operand read from TMEM, TMEM loads)
 * and compares with a float reference computed on the host from the same
 * rounded inputs.  max_abs_err[0] is the S = Q K^T tile, [1] the O = P V tile
 * (both relative to the largest reference magnitude).  Returns
 * NLFA_ERR_SELFTEST_MISMATCH when either exceeds 1e-2.  Replaces `mma_probe`
 * (nanolab/csrc/flash_attn_cuda.cu:1710-1741) and its caller `_probe_mma`
 * (nanolab/flash_cuda.py:59-88), whose job was the same for the mma.sync
 * fragment layout.  Synchronises the stream. */
int nlfa_selftest(int dtype, int head_dim, void* workspace, size_t workspace_bytes,
                  float* max_abs_err, void* stream);

/* Diagnostic form of the self-test: the caller supplies the 128 x D tiles q, k,
 * v (device, 16-bit, row-major) and receives the raw products s_out [128,128]
 * and o_out [128,D] (device, float32), where O = round16(S) V.  No counterpart
 * in the reference. */
int nlfa_selftest_tiles(int dtype, int head_dim, const void* q, const void* k, const void* v,
                        float* s_out, float* o_out, void* stream);

/* Host-only check of the mask geometry the tensor-core kernels rely on: for a
 * sequence of T positions with the given window / sinks it compares, against the
 * element-wise predicate of nanolab/mixers.py:125-132 evaluated for every
 * (query, key) pair, (1) the range of key blocks a 128-row query tile is given,
 * (2) the "every pair visible" claim for each (128-row tile) x (stream_rows-row
 * tile) rectangle, in both orientations, (3) the claim that only the causal
 * edge or only the window's lower edge cuts a rectangle, and (4, stream_rows
 * 128) that the key blocks which meet a query tile in the one-pass backward take
 * the turns 0 .. n-1 once each, in ascending block order.  stream_rows is 64 or
 * 128.  Returns 0 when all agree, otherwise 1 + the index of the first failing
 * check (negative: bad arguments).  Needs no device.  No counterpart in the
 * reference. */
int nlfa_check_mask_geometry(int T, int window, int sinks, int stream_rows);
/* ... for a block-causal mask of `block` positions (window must then be 0). */
int nlfa_check_mask_geometry_masked(int T, int window, int sinks, int block, int stream_rows);

/* Reads (and clears) the device status word that bounded waits inside the
 * kernels write when they give up.  Synchronises the device.  Returns NLFA_OK
 * or NLFA_ERR_DEVICE_TIMEOUT; *raw receives the raw word when raw != NULL.
 * Clearing also zeroes the registered host copy (below) and re-arms the
 * persistent kernels' work counters.
 *
 * Error contract of the tensor-core kernels.  Every wait inside them is bounded
 * (2 s).  A wait that runs out records a code in the status word, its CTA
 * leaves cleanly, and every CTA and launch that starts while the word is set
 * does nothing: outputs of such launches are NOT written.  The reference fails
 * closed in the same spirit (nanolab/flash_cuda.py:91-135 never raises and
 * records the reason; nanolab/mixers.py:365-370 falls back with one warning). */
int nlfa_device_status(unsigned* raw);

/* Registers a host-resident copy of the status word for the current device, so
 * that a give-up is seen without synchronising.  `host_word` must be page-locked
 * host memory the device can write (cudaHostAlloc / cudaHostRegister with
 * mapping, torch's pin_memory), owned by the caller for as long as it stays
 * registered; NULL unregisters.  The kernel that gives up writes its code there
 * as well, and from then on nlfa_fwd, nlfa_bwd, nlfa_bwd_passes and
 * nlfa_bwd_static_scratch refuse tensor-core launches on that device with
 * NLFA_ERR_DEVICE_TIMEOUT until nlfa_device_status has cleared the word.
 * Synchronises the device (it is a set-up call).  No counterpart in the
 * reference. */
int nlfa_set_status_mirror(unsigned* host_word);

/* NLFA_ERR_DEVICE_TIMEOUT if the registered host copy shows a give-up on the
 * current device, else NLFA_OK.  A plain host memory read: no CUDA call. */
int nlfa_peek_status(void);

/* Test hook for the error contract: launches one CTA that waits, with
 * `limit_ns` (at most the kernels' own limit) instead of the built-in one, on a
 * barrier that nothing ever arrives at.  The wait runs out, the CTA records
 * the give-up exactly as the attention kernels would, and the kernel returns;
 * nothing traps, faults or spins without a limit.  No counterpart in the
 * reference. */
int nlfa_test_wait_timeout(unsigned long long limit_ns, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* NLFA_H_ */
