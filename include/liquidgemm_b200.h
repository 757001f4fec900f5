/*
 * liquidgemm_b200 -- C ABI of the LiquidQuant (LQQ) W4A8 linear path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the CUDA stream it is
 * given (cudaStream_t passed as void*), never synchronises the device and -- unless its comment
 * says otherwise -- never allocates.  Return value: 0 on success, a negative LQ_ERR_* code
 * otherwise (lq_error_string() explains it).  Pointers are borrowed for the duration of the
 * enqueue only; outputs and workspaces are owned by the caller.
 *
 * Each declaration cites the interface of the reference project (liquidgemm, paths relative to
 * its repository root) that the entry point stands in for.
 *
 * Codes shared by several calls
 *   out_dtype / in_dtype : 0 = bfloat16, 1 = float16, 2 = float32
 *                          (reference csrc/liquid_gemm/w4a8_wgmma.cu:626-627)
 */
#ifndef LIQUIDGEMM_B200_H_
#define LIQUIDGEMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LQ_API __attribute__((visibility("default")))
#else
#define LQ_API
#endif

#define LQ_OK 0
#define LQ_ERR_BAD_ARG (-1)      /* null pointer, non-positive size, unknown dtype code            */
#define LQ_ERR_SHAPE (-2)        /* a divisibility / range precondition of the op does not hold    */
#define LQ_ERR_WORKSPACE (-3)    /* workspace missing or smaller than lq_*_workspace_bytes()       */
#define LQ_ERR_CUDA (-4)         /* a CUDA runtime / driver call failed (see lq_last_cuda_error)   */
#define LQ_ERR_DEVICE (-5)       /* current device is not compute capability 10.x                  */
#define LQ_ERR_TIMEOUT (-6)      /* a bounded device-side wait gave up (read by lq_poll_status)    */

#define LQ_DT_BF16 0
#define LQ_DT_F16 1
#define LQ_DT_F32 2

/* Source layouts accepted by lq_repack_tiles(). */
#define LQ_SRC_CODES 0           /* [N, K] uint8, one 4-bit code per byte  (LiquidQuantWeight.qweight_u4) */
#define LQ_SRC_NIBBLES 1         /* [N, K/2] uint8, pack_nibbles() order (even k in the low nibble)       */

/* Library identification and diagnostics (no reference counterpart: the reference reports errors
 * through TORCH_CHECK exceptions, e.g. csrc/liquid_gemm/gemv2.cu:85-89). */
LQ_API int lq_abi_version(void);
LQ_API const char* lq_error_string(int code);
/* Text of the last CUDA error recorded by this library on the calling thread ("" if none). */
LQ_API const char* lq_last_cuda_error(void);
/* 0 when the current device can run the kernels (sm_100), LQ_ERR_DEVICE otherwise. */
LQ_API int lq_check_device(void);
/* Reads (and clears) the device-side status word that bounded waits set when they give up.
 * Synchronises `stream`.  Returns 0 or LQ_ERR_TIMEOUT. */
LQ_API int lq_poll_status(void* stream);

/* UINT4 -> INT8 reconstruction q_hat = (code*step + a) XOR 0x80.
 * Replaces torch.ops.liquidgemm.dequant_weight (reference csrc/liquid_gemm/dequant.cu:46-74,
 * schema csrc/liquid_gemm/torch_bindings.cpp:44-46).  q_u4 is [N,K] one code per byte;
 * K % 4 == 0, group % 4 == 0, K % group == 0. */
LQ_API int lq_dequant_weight(const uint8_t* q_u4, const uint8_t* s_u8, const uint8_t* offset_a,
                      int8_t* out_i8, int N, int K, int group_size, void* stream);

/* Per-token symmetric INT8 activation quantiser: ascale[m] = max(amax,1e-12)/127,
 * xq = clamp(rint(x / ascale), +-127) with an IEEE division, i.e. bit-identical to
 * liquidgemm/quant.py:135-141.  Replaces torch.ops.liquidgemm.quant_per_token
 * (reference csrc/liquid_gemm/epilogue.cu:61-80), whose reciprocal-multiply can differ from
 * that formula by one count. */
LQ_API int lq_quant_per_token(const void* x, int in_dtype, int8_t* xq, float* ascale, int M, int K,
                       void* stream);

/* y[m,n] = (T)((float)acc[m,n] * ascale[m] * s1[n]).
 * Replaces torch.ops.liquidgemm.scale_epilogue (reference csrc/liquid_gemm/epilogue.cu:82-106). */
LQ_API int lq_scale_epilogue(const int32_t* acc, const float* ascale, const float* s1, void* y,
                      int out_dtype, int M, int N, void* stream);

/* Decode GEMV, M <= 16: y = scale_epilogue(x_i8 @ q_hat^T) straight from the row-major
 * interleaved pack of liquidgemm/ops.py:68-75.  Requires K % 128 == 0 and group_size == 64.
 * Replaces torch.ops.liquidgemm.w4a8_gemv2 (reference csrc/liquid_gemm/gemv2.cu:82-120) for callers that
 * hold that pack; layers prepared by this library keep the tile blob only and are served by
 * lq_w4a8_gemm_fused. */
LQ_API int lq_w4a8_gemv(const int8_t* x_i8, const uint8_t* gpack, const uint8_t* s_u8,
                 const uint8_t* offset_a, const float* ascale, const float* s1, void* y,
                 int out_dtype, int M, int N, int K, int group_size, void* stream);

/* The decode GEMV (1..8 tokens) fed from the GEMM's tile blob instead of a GEMV-specific pack, so a
 * layer keeps ONE copy of its 4-bit weights for every batch size (the reference's GEMV mode stores
 * a second, row-major copy: liquidgemm/vllm_plugin.py:157-164).  Stream-K over 2 CTAs per SM with a
 * bulk-copy ring and dp4a.  `workspace`: lq_gemv_blob_workspace_bytes() bytes, ALL ZERO on entry, left
 * all zero.  x_i8 and blob must be 16-byte aligned; K % 128 == 0; any N (the blob pads rows).
 * Serves torch.ops.liquidgemm.w4a8_wgmma_rs_fused for small M
 * (reference csrc/liquid_gemm/w4a8_wgmma.cu:575-645). */
LQ_API size_t lq_gemv_blob_workspace_bytes(void);
LQ_API int lq_w4a8_gemv_blob(const void* x_i8, const void* blob, const void* ascale, const void* s1,
                             void* out, int out_dtype, int M, int N, int K, void* workspace,
                             size_t workspace_bytes, void* stream);

/* lq_w4a8_gemv_blob without a workspace argument: the reduction scratch is an array inside the
 * library's device image (4 194 304 bytes, enough for 512 CTAs = devices of up to 256 SMs), so the
 * call needs no buffer from any allocator.  It is meant for callers that cannot obtain device memory
 * where the call is made: a serving process whose memory plan has already handed every byte of the GPU
 * to its own pools, or code running where entering an allocator is not allowed.  This entry point has
 * no counterpart in the reference.
 *  - Limits: M <= 8, K % 128 == 0, x_i8 and blob 16-byte aligned as for lq_w4a8_gemv_blob; a device
 *    whose 2 x SM count exceeds 512 is refused with LQ_ERR_WORKSPACE (text in lq_last_cuda_error()).
 *  - The FIRST call on each device (with that device current) looks the array's device address up,
 *    clears the array and then synchronises the whole device, so that the cleared array is seen by a
 *    kernel on any stream.  Make that first call before any stream capture and outside
 *    latency-critical sections; later calls only enqueue the kernel.
 *  - The array must be all zero when a call starts, and every call whose kernel runs to completion
 *    leaves it all zero.  There is one array per device and every call shares it: two calls that
 *    overlap in time on the same device (different streams or threads) race on it and give wrong
 *    sums; serialise them.
 *  - If lq_poll_status() reports LQ_ERR_TIMEOUT after such a call (a bounded device-side wait gave up),
 *    the array may hold partial sums: enqueue lq_w4a8_gemv_blob_static_reset(stream) before the next
 *    call, otherwise every later result on that device is wrong.  The reset is a cudaMemsetAsync on
 *    `stream`; it allocates and synchronises nothing. */
LQ_API int lq_w4a8_gemv_blob_static(const void* x_i8, const void* blob, const void* ascale,
                                    const void* s1, void* out, int out_dtype, int M, int N, int K,
                                    void* stream);
LQ_API int lq_w4a8_gemv_blob_static_reset(void* stream);

/* lq_w4a8_gemm_fused for a decode batch (M <= 16) whose output block [M, N] is written into n_outs
 * (1..8) row-major matrices with row stride ld_out elements at column col0: with the full-width
 * outputs of this GPU and of its peers as destinations (peer memory mapped into this process), the
 * epilogue performs the all-gather of an N-sharded layer with plain stores over NVLink.  `outs` is
 * a HOST array of device pointers.  Ordering towards the peers' consumers is the caller's job (a
 * stream-ordered barrier between the ranks after the call).  Workspace: lq_scatter_workspace_bytes().
 * Replaces GEMM + all-gather of the reference's tensor-parallel use
 * (liquidgemm/vllm_plugin.py:174-206 under vLLM's column-parallel linear). */
LQ_API int lq_w4a8_gemm_fused_scatter(const int8_t* x_i8, const uint8_t* blob, const float* ascale,
                                      const float* s1, void* const* outs, int n_outs, long ld_out,
                                      long col0, int out_dtype, int M, int N, int K, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* The same with cross-GPU ordering done by the kernels themselves instead of a barrier launch:
 * every CTA, after its last output store, adds 1 (release, system scope) to word `flag_index` of
 * each destination rank's flag array `peer_flags[r]` (null: no signalling); and before it reads the
 * tokens the kernel waits (at most 2 s, then a status code) until `*wait_flag >= wait_value`
 * (null: no wait).  A consumer of the gathered output therefore passes the flag word its producers
 * signalled and, as value, the sum over the ranks of lq_decode_grid() of the producing launch.
 * Flags are zeroed by the host, with the ranks ordered once before the first kernel of a sequence. */
LQ_API int lq_w4a8_gemm_fused_scatter_sync(const int8_t* x_i8, const uint8_t* blob, const float* ascale,
                                           const float* s1, void* const* outs, int n_outs, long ld_out,
                                           long col0, int out_dtype, int M, int N, int K,
                                           unsigned* const* peer_flags, int flag_index,
                                           const unsigned* wait_flag, unsigned wait_value,
                                           void* workspace, size_t workspace_bytes, void* stream);
/* CTAs a gather-by-stores launch of this shape uses on the current device, and the bytes and kind of its
 * workspace (kinds as for lq_gemm_workspace_kind: 1 = scratch, the tile kernel's planes; 2 = ALL ZERO on entry,
 * left all zero, may be shared with the other zeroed workspaces).  These differ from the single-destination
 * queries where that call would take a route the gather-by-stores form does not have. */
LQ_API int lq_decode_grid(int M, int N, int K);
LQ_API size_t lq_scatter_workspace_bytes(int M, int N, int K);
LQ_API int lq_scatter_workspace_kind(int M, int N, int K);

/* One whole linear layer for HOST activations and a HOST output: upload, per-token quantise, fused
 * W4A8 linear from the tile blob (automatic kernel choice by M), download, all enqueued on `stream`
 * by this one call; nothing is synchronised.  x_host [M,K] in x_dtype and y_host [M,N] in out_dtype
 * should be pinned for the copies to be asynchronous.  `scratch`: device memory of
 * lq_linear_host_scratch_bytes() bytes, 256-byte aligned, holding the device copies; `workspace`
 * as for lq_w4a8_gemm_fused with splitk 0.  Stands for the Python-side .cuda() moves around the
 * reference's operators (liquidgemm/ops.py:185-201, liquidgemm/vllm_plugin.py:174-206). */
LQ_API size_t lq_linear_host_scratch_bytes(int M, int N, int K, int x_dtype, int out_dtype);
LQ_API int lq_w4a8_linear_host(const void* x_host, int x_dtype, const void* blob, const void* s1,
                               void* y_host, int out_dtype, int M, int N, int K, void* scratch,
                               size_t scratch_bytes, void* workspace, size_t workspace_bytes,
                               void* stream);

/* Same product from the plain pack_nibbles() layout with float32 output, any M.
 * Replaces torch.ops.liquidgemm.w4a8_gemm (reference csrc/liquid_gemm/w4a8_gemm.cu:183-227).
 * M <= 16 runs the GEMV (K % 64 == 0); larger M re-tiles the weights into `workspace`
 * (scratch of lq_gemm_v1_workspace_bytes, need not be zeroed) and runs the tensor-core kernel
 * (K % 128 == 0).  group_size must be 64, as in the reference. */
LQ_API size_t lq_gemm_v1_workspace_bytes(int M, int N, int K);
LQ_API int lq_w4a8_gemm_v1(const int8_t* x_i8, const uint8_t* nibbles, const uint8_t* s_u8,
                    const uint8_t* offset_a, const float* s1, const float* ascale, float* y,
                    int M, int N, int K, int group_size, void* workspace, size_t workspace_bytes,
                    void* stream);

/* Tile-ordered weight blob consumed by the tensor-core GEMM: for every 128-row x 128-k tile,
 * 8192 bytes of interleaved nibbles followed by 512 bytes of (step, offset) pairs.
 * Replaces liquidgemm.ops.repack_rs_weight + the wgmma_rs_a_coords op it needs
 * (reference liquidgemm/ops.py:118-150, csrc/liquid_gemm/w4a8_wgmma.cu:310-331): the layout is
 * specific to this library, as the reference's is to Hopper register fragments.
 * K % 128 == 0, group_size % 64 == 0 (and 128 % group_size == 0 or group_size % 128 == 0);
 * N is padded to a multiple of 128 inside the blob. */
LQ_API size_t lq_tile_blob_bytes(int N, int K);
LQ_API int lq_repack_tiles(const uint8_t* src, int src_layout, const uint8_t* s_u8,
                    const uint8_t* offset_a, uint8_t* blob, int N, int K, int group_size,
                    void* stream);

/* LiquidQuant weight quantiser on the device: w [N, K] (w_dtype: LQ_DT_*) -> s1 [N] float32, s_u8 and
 * offset_a [N, K/group_size], and optionally codes [N, K] (one 4-bit code per byte) and / or the tile blob
 * of lq_tile_blob_bytes(N, K) bytes (either may be null).  Two kernels, no host read: the overflow
 * invariants are checked on the device (lq_poll_status reports site 501).  Bit-identical to the
 * reference's quantize_weight on the CPU followed by its prepack
 * (liquidgemm/quant.py:61-100, liquidgemm/ops.py:118-150).  K % 128 == 0, group_size 64 or 128;
 * codes and blob 16-byte aligned. */
LQ_API int lq_quantize_weight(const void* w, int w_dtype, int N, int K, int group_size, float* s1,
                              uint8_t* s_u8, uint8_t* offset_a, uint8_t* codes, uint8_t* blob,
                              void* stream);

/* Scheduling of the tensor-core GEMM, selected by the `splitk` argument of the calls below.
 *   splitk = 0 (automatic):
 *     one token, two tokens on matrices up to 64 M weights, three or four on matrices up to 16 M weights
 *              (scaled outputs only): streaming dp4a GEMV over the tile blob;
 *     up to 16 tokens on matrices up to 32 M weights: the streaming tensor-core kernel, ONE launch:
 *              stream-K over two CTAs per SM, one 64-bit atomic per element joins cut tiles;
 *     3072 tokens and more (5120 on matrices above 32 M weights) on layers with K < 8192, whole 256-channel
 *              blocks and at most 256 M weights, one destination: the blob is unpacked to INT8 in the workspace
 *              (scratch, N x K bytes) and the INT8 x INT8 CTA-pair kernel does the GEMM, TWO launches
 *              (LQ_UNPACK_I8_MIN_M in the environment moves the limit, 0 switches the route off);
 *     256 tokens and more on layers with whole 256-channel blocks, where a cost model expects it to win
 *              (large M x N): the CTA-pair kernel, tcgen05.mma.cta_group::2 on 256-channel x 192-token tiles;
 *     otherwise tile kernel: one 128-channel x up-to-128-token tile per CTA, two CTAs per SM, every
 *              tile cut into S k-ranges (S from the SM count) whose int32 partial planes one finish
 *              kernel reduces, scales and casts -- the split-K design of the reference
 *              (csrc/liquid_gemm/w4a8_wgmma.cu:39-56, 523-534); S = 1 fuses the epilogue.
 *   splitk = S >= 1: M <= 128: the tile kernel with exactly S k-ranges (clamped to K/128);
 *              M > 128: the persistent kernel with whole tiles (1) or a fixed split (S > 1).
 *   splitk = -1 forces the persistent stream-K kernel for any M.
 * Partial sums are integers, so every setting gives bit-identical results.
 * lq_gemm_pick_splitk maps LIQUIDGEMM_SPLITK (`env_override`, 0 = unset) to that argument: like
 * the reference the override only applies to M <= 128 and is clamped to K/128; otherwise 0. */
LQ_API int lq_gemm_pick_splitk(int M, int N, int K, int env_override);
/* Workspace bytes for (M,N,K,splitk) and its kind: 0 = none, 1 = scratch (any contents; the
 * tile kernel's planes, or the INT8 weights of the unpack route: 16-byte aligned), 2 = reduction buffer of the streaming, pair and persistent kernels, which must be ALL ZERO when
 * a call starts and is all zero again when its kernel ends (the kernel cleans up after itself), so
 * one zero-filled buffer serves any number of successive calls on a stream; calls that overlap on
 * the GPU need separate buffers, and after a LQ_ERR_TIMEOUT the caller must clear it. */
LQ_API size_t lq_gemm_workspace_bytes(int M, int N, int K, int splitk);
LQ_API int lq_gemm_workspace_kind(int M, int N, int K, int splitk);
/* Kernel launches one fused call with these arguments makes (2 when the tile kernel splits K or the unpack
 * route is taken). */
LQ_API int lq_gemm_launches(int M, int N, int K, int splitk);

/* W4A8 tensor-core GEMM, exact int32 accumulators acc[M,N] = x_i8 @ q_hat^T.
 * Replaces torch.ops.liquidgemm.w4a8_wgmma_rs (reference csrc/liquid_gemm/w4a8_wgmma.cu:505-570).
 * Any M >= 1 (token rows beyond M are zero-filled by TMA, not by a padded copy). */
LQ_API int lq_w4a8_gemm_i32(const int8_t* x_i8, const uint8_t* blob, int32_t* acc, int M, int N, int K,
                     int splitk, void* workspace, size_t workspace_bytes, void* stream);

/* W4A8 tensor-core GEMM with the fused (split-K reduce +) scale + cast epilogue.
 * Replaces torch.ops.liquidgemm.w4a8_wgmma_rs_fused
 * (reference csrc/liquid_gemm/w4a8_wgmma.cu:575-645). */
LQ_API int lq_w4a8_gemm_fused(const int8_t* x_i8, const uint8_t* blob, const float* ascale,
                       const float* s1, void* y, int out_dtype, int M, int N, int K, int splitk,
                       void* workspace, size_t workspace_bytes, void* stream);

/* lq_w4a8_gemm_fused (automatic scheduling) with the layer's bias added inside the kernel's epilogue:
 * y = (T)((T)((float)acc * ascale[m] * s1[n]) + bias[n]), i.e. the bias joins the value already rounded to
 * the output type T, exactly what the reference's plugin computes with a separate PyTorch add after its
 * operator (liquidgemm/vllm_plugin.py:205-206).  `bias`: [N] in the output dtype, or null. */
LQ_API int lq_w4a8_linear_bias(const int8_t* x_i8, const uint8_t* blob, const float* ascale,
                        const float* s1, const void* bias, void* y, int out_dtype, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Plain INT8 x INT8 -> INT32 tensor-core GEMM c[M,N] = a[M,K] @ b[N,K]^T.
 * Replaces torch.ops.liquidgemm.wgmma_i8_gemm (reference csrc/liquid_gemm/w4a8_wgmma.cu:648-694).
 * K % 128 == 0; M and N are arbitrary here (the reference needs multiples of 128).
 * Dispatch: from 256 tokens, on layers with whole 256-channel blocks and at least 60 tiles of 256 x 256, a
 * CTA-pair kernel (tcgen05.mma.cta_group::2, both operands from shared memory); otherwise a persistent one-CTA
 * kernel.  LQ_I8_PAIR=0 in the environment keeps every call on the latter (a measurement switch). */
LQ_API int lq_i8_gemm_i32(const int8_t* a, const int8_t* b, int32_t* c, int M, int N, int K,
                   void* stream);

/* Same GEMM with the scale + cast epilogue: y = (T)((float)acc * a_scale[m] * b_scale[n]).
 * Stands in for the third-party vllm cutlass_scaled_mm call of the plugin's INT8 mode
 * (reference liquidgemm/vllm_plugin.py:197-204). */
LQ_API int lq_i8_gemm_scaled(const int8_t* a, const int8_t* b, const float* a_scale,
                      const float* b_scale, void* y, int out_dtype, int M, int N, int K,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LIQUIDGEMM_B200_H_ */
