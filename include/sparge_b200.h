/*
 * sparge_b200 -- C ABI of the B200 (sm_100a) block-sparse quantised attention path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, returns an int status
 * (SPARGE_OK == 0), allocates nothing and keeps no global state unless its comment says so.
 * All tensors are contiguous, "HND" layout: [B, H, N, D] with D in {64, 128}.
 * 16-bit element type codes: SPARGE_F16 = 0, SPARGE_BF16 = 1.
 * Block geometry is fixed: 128 query rows x 64 key rows per sparsity block
 *   nq = ceil(N / 128), nk = ceil(N / 64), N_pad = nq * 128.
 *
 * Reference citations are path:line in the thu-ml/SpargeAttn source tree.
 */
#ifndef SPARGE_B200_H_
#define SPARGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* sparge_stream_t; /* a cudaStream_t */

enum {
  SPARGE_OK = 0,
  SPARGE_ERR_INVALID_ARG = 1, /* bad head_dim / dtype code / sizes: maps to ValueError            */
  SPARGE_ERR_NULL = 2,        /* a required pointer is NULL: maps to RuntimeError                  */
  SPARGE_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed: maps to RuntimeError         */
  SPARGE_ERR_TOO_LARGE = 4,   /* a size exceeds what the kernel supports: maps to ValueError       */
  SPARGE_ERR_UNSUPPORTED = 5  /* valid request that this build does not implement                  */
};
enum { SPARGE_F16 = 0, SPARGE_BF16 = 1 };

/* Device-side status word values written by sparge_attn_fwd when a bounded wait expires. */
enum { SPARGE_DEV_OK = 0, SPARGE_DEV_TIMEOUT_PRODUCER = 1, SPARGE_DEV_TIMEOUT_MMA = 2, SPARGE_DEV_TIMEOUT_SOFTMAX = 3 };

const char* sparge_strerror(int status);
int sparge_abi_version(void);

/* Mean of K over tokens, in K's own 16-bit type.
 * Replaces `km = k.mean(dim=-2, keepdim=True)` (spas_sage_attn/core.py:119-120).
 *   k [B,H,N,D] -> km [B,H,D].  scratch: sparge_k_mean_scratch_bytes() bytes of device memory,
 *   contents need no initialisation. */
size_t sparge_k_mean_scratch_bytes(int B, int H, int N, int D);
int sparge_k_mean(const void* k, void* km, void* scratch, int B, int H, int N, int D, int dtype,
                  sparge_stream_t stream);

/* Allocation-free variant of sparge_k_mean. It has no counterpart in the reference.
 *
 * Who it is for: hosts that must not (or cannot) obtain device memory at call time -- a serving
 * process whose framework has already claimed the whole GPU for its own pool, a plugin that is
 * handed tensors but no allocator, or a latency-critical loop where cudaMalloc/cudaFree would stall
 * the device.  The caller still passes the input and the output; only the scratch is supplied by the
 * library, from a fixed array of SPARGE_K_MEAN_STATIC_MAX_BYTES that is part of the library image
 * (each GPU that loads the library holds that much memory until the process exits).
 *
 *   - Requests needing more scratch than the array holds return SPARGE_ERR_TOO_LARGE:
 *     sparge_k_mean_scratch_bytes(B,H,N,D) = B*H*ceil(N/512)*D*8 must be <= the maximum.
 *   - The first call on each device looks up the array's device address (no allocation); make every call
 *     with the intended device current.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left in it.
 *     The kernels overwrite every element they later read, so no clearing is needed, but two calls
 *     whose kernels can overlap on the GPU (different streams, no dependency) race on it: order them.
 *   - Calls no cudaMalloc, cudaFree or other allocating routine.  Same results as sparge_k_mean. */
#define SPARGE_K_MEAN_STATIC_MAX_BYTES (8u << 20)
int sparge_k_mean_static(const void* k, void* km, int B, int H, int N, int D, int dtype, sparge_stream_t stream);

/* Per-block pooling + cosine self-similarity + per-block INT8 quantisation in one pass.
 * Replaces triton_bmm_pool_sim_simmean_fuse_quant (spas_sage_attn/utils.py:161-214, wrapper
 * :270-280) and, with simthreshd1 == NULL, the quantiser-only qk_quantize (utils.py:89-159,
 * wrappers :255-268).
 *   x [B,H,N,D]; km [B,H,D] or NULL (subtracted in the 16-bit type before everything else);
 *   block = 128 for Q, 64 for K; nb = ceil(N / block).
 *   outputs: pool [B,H,nb,D] (same 16-bit type), sim [B,H,nb] (uint8 0/1), x_int8 [B,H,N,D],
 *   scale [B,H,nb] fp32.  pool/sim may be NULL when simthreshd1 is NULL. */
int sparge_pool_quant(const void* x, const void* km, const float* simthreshd1, void* pool, uint8_t* sim,
                      int8_t* x_int8, float* scale, int B, int H, int N, int D, int block, int dtype,
                      sparge_stream_t stream);

/* Pooled-score map -> row softmax -> stable top-k (or cdf) selection -> forced blocks -> LUT.
 * Replaces the torch/Triton chain of get_block_map_meansim_fuse_quant
 * (spas_sage_attn/utils.py:386-420: bmm, masked fills, softmax, sort, cumsum, fill_block_map,
 * causal mask, attention sink, block_map_lut_triton).
 *   pq [B,H,nq,D], pk [B,H,nk,D] (16-bit), sim_q [B,H,nq], sim_k [B,H,nk] (uint8),
 *   topk [H] fp32 or NULL, cdfthreshd [H] fp32 or NULL (exactly one non-NULL),
 *   outputs: mask [B,H,nq,nk] uint8 (may be NULL), lut [B,H,nq,nk] int32 (first entry absolute,
 *   then gaps, zero tail), valid [B,H,nq] int32.  Ties are broken towards the lower block index.
 *   lut_order: SPARGE_LUT_ASCENDING (0) is the reference encoding. SPARGE_LUT_BEST_FIRST (1) puts the live
 *   block with the largest pooled probability first and keeps the others ascending (gaps may be negative;
 *   sparge_attn_fwd simply accumulates them). It selects the same blocks; only the visiting order changes. */
enum { SPARGE_LUT_ASCENDING = 0, SPARGE_LUT_BEST_FIRST = 1 };
int sparge_select(const void* pq, const void* pk, const uint8_t* sim_q, const uint8_t* sim_k, const float* topk,
                  const float* cdfthreshd, uint8_t* mask, int32_t* lut, int32_t* valid, int B, int H, int nq,
                  int nk, int D, int dtype, int is_causal, int attention_sink, int lut_order, sparge_stream_t stream);

/* User block mask -> LUT.  Replaces block_map_lut_triton / triton_block_map_to_lut_kernel
 * (spas_sage_attn/utils.py:54-87).  mask [B,H,nq,nk] with elem_size in {1,2,4,8} bytes, any
 * non-zero bit pattern counts as live. */
int sparge_mask_to_lut(const void* mask, int elem_size, int32_t* lut, int32_t* valid, int B, int H, int nq, int nk,
                       sparge_stream_t stream);

/* Per-channel FP8 (e4m3) quantisation of V with scale_max 2.25.
 * Replaces the fp16 cast (spas_sage_attn/core.py:115-117), transpose_pad_permute_cuda
 * (csrc/fused/fused.cu:193-267) and scale_fuse_quant_cuda (fused.cu:269-344).
 *   v [B,H,N,D] (16-bit; bf16 is rounded to fp16 first, as the reference does)
 *   -> v8 [B,H,N_pad,D] e4m3 bytes, token-major, rows >= N zero; v_scale [B,H,D] fp32.
 *   v_scale = amax * RN(1/2.25) and v8 = e4m3(v * div.approx(2.25, amax)): the reference's fast-math quotients.
 *   The reference's [B,H,D,N_pad] transposition and 16-token permutation are layout artefacts
 *   of its mma.sync operand registers and are not reproduced. */
int sparge_quant_v(const void* v, uint8_t* v8, float* v_scale, int B, int H, int N, int D, int dtype,
                   sparge_stream_t stream);

/* out[i] = a[i] / b[i] as `div.approx.ftz.f32` evaluates it on this GPU: the approximate quotient that the
 * reference's V quantiser uses (csrc/fused/fused.cu:150,163 compiled with --use_fast_math, setup.py:60) and that
 * sparge_quant_v reproduces. The hardware reciprocal has no published bit-level definition, so a CPU restatement
 * of the V quantiser takes this function's output as an input. Test support; a, b, out are device pointers. */
int sparge_div_approx(const float* a, const float* b, float* out, int n, sparge_stream_t stream);

/* LUT-driven block-sparse attention: INT8 QK^T and FP8 PV on tcgen05 tensor cores.
 * Replaces qk_int8_sv_f8_accum_f16_block_sparse_attn_inst_buf_fuse_v_scale_with_pv_threshold
 * (csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:392-585, kernel qk_int_sv_f8_cuda_sm89.cuh:42-755,
 * declared at csrc/qattn/attn_cuda.h:19-123) with tensor_layout = HND, qk_quant_gran = per block.
 *   q_int8, k_int8 [B,H,N,D]; v8 [B,H,N_pad,D]; o [B,H,N,D] (out_dtype); lut/valid as above;
 *   pvthreshd [H] fp32 or NULL (NULL = never skip a PV block); q_scale [B,H,nq]; k_scale [B,H,nk];
 *   v_scale [B,H,D]; dev_status: one int32 in device memory, or NULL. It is written only when a
 *   bounded wait inside the kernel expires (SPARGE_DEV_*), never cleared.
 *   is_causal != 0 masks key > query at token level.  Query rows whose block row has no live
 *   block are written as zeros (the reference leaves them uninitialised). */
int sparge_attn_fwd(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o, const int32_t* lut,
                    const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                    const float* v_scale, int32_t* dev_status, int B, int H, int N, int D, int out_dtype,
                    int is_causal, float sm_scale, sparge_stream_t stream);

/* Strided variants: the 16-bit inputs (and the attention output) may be any [B,H,N,D] view whose last
 * dimension is contiguous, given by element strides of the batch, head and token dimensions -- for
 * example the "NHD" tensors [B,N,H,D] that attention processors produce (stride_h = D, stride_n = H*D)
 * -- so that no permuted copy is made before or after the path (the reference's prologue copies q, k, v,
 * spas_sage_attn/core.py:107-117, and its callers copy again, inference_examples/modify_model/
 * modify_wan.py:116-118). Base pointers must be 16-byte aligned and strides multiples of 8 elements.
 * The quantised / pooled outputs are always contiguous HND. */
int sparge_k_mean_strided(const void* k, void* km, void* scratch, int B, int H, int N, int D, int dtype,
                          long long stride_b, long long stride_h, long long stride_n, sparge_stream_t stream);
int sparge_pool_quant_strided(const void* x, const void* km, const float* simthreshd1, void* pool, uint8_t* sim,
                              int8_t* x_int8, float* scale, int B, int H, int N, int D, int block, int dtype,
                              long long stride_b, long long stride_h, long long stride_n, sparge_stream_t stream);
int sparge_quant_v_strided(const void* v, uint8_t* v8, float* v_scale, int B, int H, int N, int D, int dtype,
                           long long stride_b, long long stride_h, long long stride_n, sparge_stream_t stream);
int sparge_attn_fwd_strided(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o, const int32_t* lut,
                            const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                            const float* v_scale, int32_t* dev_status, int B, int H, int N, int D, int out_dtype,
                            int is_causal, float sm_scale, long long o_stride_b, long long o_stride_h,
                            long long o_stride_n, sparge_stream_t stream);

/* sparge_attn_fwd_strided plus the reference's return_pv_count diagnostic (csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:526-529,
 * kernel qk_int_sv_f8_cuda_sm89.cuh:91,355-358,650-656): pv_count is int32 [B, H, ceil(N/128) * 4], one entry per
 * 32-row group of a query block, = the number of live blocks whose P.V product was computed (valid[b,h,q] minus the
 * blocks dropped by the pvthreshd test; the test is per 128-row block here, so the four entries are equal).
 * pv_count may be NULL (then identical to sparge_attn_fwd_strided). The caller allocates it; the reference allocates
 * it inside the op. */
int sparge_attn_fwd_pv_count(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o, const int32_t* lut,
                             const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                             const float* v_scale, int32_t* dev_status, int B, int H, int N, int D, int out_dtype,
                             int is_causal, float sm_scale, long long o_stride_b, long long o_stride_h,
                             long long o_stride_n, int32_t* pv_count, sparge_stream_t stream);

/* sparge_attn_fwd_pv_count restricted to a range of query blocks per (batch, head): q_block_ranges is int32
 * [B*H][2] in device memory = (first query block, number of query blocks); only those 128-row blocks of o (and
 * of pv_count) are written. q_blocks_max >= the largest count (it sizes the launch). q_block_ranges == NULL means
 * every block. This is the unit of the multi-GPU row sharding: the reference's grid cell (query block, head,
 * batch) is independent of every other (csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:772-780), so ranks can own
 * disjoint row ranges of a head; the reference itself has no such entry point. */
int sparge_attn_fwd_rows(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o, const int32_t* lut,
                         const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                         const float* v_scale, int32_t* dev_status, int B, int H, int N, int D, int out_dtype,
                         int is_causal, float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                         int32_t* pv_count, const int32_t* q_block_ranges, int q_blocks_max, sparge_stream_t stream);

/* sparge_attn_fwd_rows with the two remaining template arguments of the reference's kernel
 * (csrc/qattn/attn_utils.cuh:45-63, dispatched at qk_int_sv_f8_cuda_sm89.cu:319-361):
 *   qk_quant_gran  1 per block : q_scale [B,H,ceil(N/128)],      k_scale [B,H,ceil(N/64)]  (what the hot path passes)
 *                  2 per warp  : q_scale [B,H,ceil(N/128)*4]  one per 32 query rows, k_scale as for 1
 *                  3 per thread: q_scale [B,H,ceil(N/128)*32] entry (row/32)*8 + row%8 (rows r, r+8, r+16, r+24 of a
 *                                32-row group share one), k_scale [B,H,ceil(N/64)*4] entry block*4 + (key%8)/2,
 *                                16-byte aligned  (qk_int_sv_f8_cuda_sm89.cuh:106-136)
 *   pv_threshold_mode  0 none (pvthreshd ignored), 1 per block (the one the reference's ops instantiate),
 *                      2 per warp: each 32-row group decides for itself whether a block's P.V is dropped
 *                        (qk_int_sv_f8_cuda_sm89.cuh:302-353 without the block-wide reduction); pv_count then
 *                        differs between the four groups of a block.
 * Other values: SPARGE_ERR_INVALID_ARG (the reference raises std::invalid_argument for an unknown granularity). */
int sparge_attn_fwd_gran(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o, const int32_t* lut,
                         const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                         const float* v_scale, int32_t* dev_status, int B, int H, int N, int D, int out_dtype,
                         int is_causal, float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                         int32_t* pv_count, const int32_t* q_block_ranges, int q_blocks_max, int qk_quant_gran,
                         int pv_threshold_mode, sparge_stream_t stream);

/* The same kernel with P and V in fp16 (tcgen05.mma kind::f16, fp32 accumulation) instead of e4m3: the arithmetic of
 * the reference's fp16-PV op qk_int8_sv_f16_accum_f16_block_sparse_attn_inst_buf_with_pv_threshold
 * (csrc/qattn/qk_int_sv_f16_cuda_sm80.cu, called by the Sage1-signature functions, spas_sage_attn/core.py:263,305),
 * with its arguments: v_f16 is the caller's fp16 V [B,H,N,D], contiguous and 16-byte aligned (no quantiser, no
 * v_scale, no padding: rows past N are read as zeros); per-block scales (qk_quant_gran 1); pvthreshd NULL = no skip
 * test, else the per-block test; pv_count, q_block_ranges as in sparge_attn_fwd_rows. About 1.2x (D = 128) and 1.06x
 * (D = 64) the time of the FP8 kernel. */
int sparge_attn_fwd_f16pv(const int8_t* q_int8, const int8_t* k_int8, const void* v_f16, void* o, const int32_t* lut,
                          const int32_t* valid, const float* pvthreshd, const float* q_scale, const float* k_scale,
                          int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal, float sm_scale,
                          long long o_stride_b, long long o_stride_h, long long o_stride_n, int32_t* pv_count,
                          const int32_t* q_block_ranges, int q_blocks_max, sparge_stream_t stream);

/* The whole path of spas_sage2_attn_meansim_topk_cuda / spas_sage2_attn_meansim_cuda (spas_sage_attn/core.py:39-169) in
 * one call: sparge_k_mean (if smooth_k), sparge_pool_quant for Q and K, sparge_select, sparge_quant_v and
 * sparge_attn_fwd, issued in that order on `stream`, with every intermediate tensor carved out of `workspace`
 * (device memory, 256-byte aligned, at least sparge_forward_workspace_bytes(B,H,N,D) bytes; reusable by the next call
 * on the same stream). For hosts that pay per call (an interpreter): a small problem costs more to issue entry by
 * entry than to run. Results are those of the separate entries.
 *   q, k (dtype) and v (v_dtype): [B,H,N,D] views, strides in elements as {batch, head, token}, last dimension
 *   contiguous; o like q. simthreshd1 [H]; exactly one of cdfthreshd / topk [H]; pvthreshd [H] or NULL (no skip test;
 *   the LUT is then emitted best block first). is_causal: block-level causality of the selection; kernel_causal:
 *   token-level masking inside the attention kernel (the reference's Sage2 entry points pass 0 there).
 * sparge_forward_workspace_layout fills the 14 byte offsets of {km, k-mean scratch, pooled q, pooled k, sim_q, sim_k,
 * q_int8, k_int8, q_scale, k_scale, lut, valid, v8, v_scale} inside the workspace (for return_sparsity, tests). */
size_t sparge_forward_workspace_bytes(int B, int H, int N, int D);
int sparge_forward_workspace_layout(int B, int H, int N, int D, size_t* offsets, int n_offsets);
int sparge_meansim_forward(const void* q, const void* k, const void* v, void* o, const float* simthreshd1,
                           const float* cdfthreshd, const float* topk, const float* pvthreshd, void* workspace,
                           size_t workspace_bytes, int32_t* dev_status, int B, int H, int N, int D, int dtype, int v_dtype,
                           int is_causal, int kernel_causal, int attention_sink, int smooth_k, float sm_scale,
                           const long long* q_strides, const long long* k_strides, const long long* v_strides,
                           const long long* o_strides, sparge_stream_t stream);

/* Failure-detection self test: launches one warp that waits on a barrier nobody signals, for `slices` tries with
 * the suspend hint slice_ns (a try lasts about 4 us on a B200 whatever the hint; slices x max(slice_ns, 4000) may
 * not exceed 0.1 s), and writes SPARGE_DEV_TIMEOUT_SOFTMAX into
 * *dev_status when the bounded wait gives up -- the same code path that sparge_attn_fwd takes if a
 * producer / MMA / softmax hand-off ever stalls. The kernel then exits normally; the context stays usable.
 * The reference has no counterpart (its sm90 kernel spins without a limit, qk_int_sv_f8_cuda_sm90.cuh:117-132). */
int sparge_selftest_wait_expiry(int32_t* dev_status, unsigned int slice_ns, unsigned int slices, sparge_stream_t stream);

/* Sustained rate of the 8-bit tensor pipe, measured on the current device: the denominator of the attention
 * kernel's roofline. No counterpart in the reference (it ships no benchmark). Every CTA keeps a 128 x 128-byte
 * A tile and an n x 128-byte B tile in shared memory and one thread issues `iters` x 4 tcgen05.mma
 * (M = 128, N = n, K = 32) back to back. kind 0 = kind::i8, 1 = kind::f8f6f4; n in {64, 128, 256};
 * ctas_per_sm in {1, 2} (two issuing threads per SM, as the attention kernel has). Launches a warm-up and a
 * timed run on `stream`, waits for them, and returns the timed run's milliseconds and its operation count
 * (2 per multiply-add). Creates two CUDA events; allocates no device memory. */
int sparge_tensor_peak(int kind, int n, int ctas_per_sm, int iters, int32_t* dev_status, float* ms_out, double* ops_out,
                       sparge_stream_t stream);

/* Peer-memory buffers for a sequence-parallel (Ulysses) exchange between the GPUs of one node; no counterpart in the
 * reference, whose multi-GPU runs go through xfuser / torch.distributed outside its attention package
 * (inference_examples/wan_infer.py). One process per GPU: sparge_peer_alloc makes a device buffer and a
 * 64-byte handle that other processes of the same node pass to sparge_peer_open to map that buffer
 * (peer access is enabled on first use); sparge_copy_async / sparge_copy2d_async are one copy-engine transfer
 * each (contiguous / `height` rows of `width` bytes with pitches) between any two device pointers, local or mapped. sparge_peer_alloc / _open / _close / _free synchronise the device and are
 * meant to run once, at set-up and tear-down; only the two copy calls belong on the data path. The owner must
 * keep a buffer alive until every peer has closed its mapping. */
int sparge_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int sparge_peer_free(void* ptr);
int sparge_peer_open(const unsigned char* handle64, void** ptr);
int sparge_peer_close(void* ptr);
int sparge_copy_async(void* dst, const void* src, size_t bytes, sparge_stream_t stream);
int sparge_copy2d_async(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t height,
                        sparge_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SPARGE_B200_H_ */
