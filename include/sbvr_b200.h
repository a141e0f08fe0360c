/*
 * sbvr_b200 — C ABI of the B200 (sm_100a) SBVR quantized-linear library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, returns an int
 * status (0 = ok, negative = error, text via sbvr_strerror) and never throws, exits or
 * synchronises the device unless its comment says so.  Calls are asynchronous on `stream`.
 *
 * Packed weight of a linear layer with N outputs and K inputs (Kp = K rounded up to a
 * multiple of G), exactly as the reference encoder emits it (reference sbvr/core.py:724-805):
 *
 *   bvr        uint32  [Kp/32, N, S]   bit j of bvr[kw][n][s] = plane s of W[n][32*kw + j]
 *   coeff_idx  uint8 | uint16 [Kp/G, N]   codebook line of group g of row n   (idx_bytes 1 | 2)
 *   coeff      fp16    [C, S]          codebook ("coeff_cache")
 * or, with idx_bytes == 0 ("direct" form, no codebook; coeff_idx ignored):
 *   coeff      fp16    [Kp/G, N, S]    one coefficient line per (group, row)
 *
 *   W[n][k] = fp16_rn( sum_s float(line(k/G, n)[s]) * bit_s[n][k] )        (plane order, fp32)
 *
 * G (group length along K) is 256 in the reference (sbvr/core.py:222); 128 is also accepted.
 * fp16 values are passed as `const void*` / `void*` pointing at IEEE binary16 data.
 */
#ifndef SBVR_B200_H
#define SBVR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SBVR_API __attribute__((visibility("default")))
#else
#define SBVR_API
#endif

typedef void* sbvr_stream_t;          /* a cudaStream_t */
typedef struct sbvr_workspace sbvr_workspace_t;

enum {
    SBVR_OK = 0,
    SBVR_ERR_BAD_ARG = -1,            /* null pointer, non-positive size, unsupported S / G / idx_bytes */
    SBVR_ERR_SHAPE = -2,              /* K not a multiple of G, N not a multiple the kernel needs */
    SBVR_ERR_ALIGN = -3,              /* pointer not aligned as the kernel needs (16 bytes) */
    SBVR_ERR_CUDA = -4,               /* a CUDA runtime call failed; see sbvr_last_cuda_error */
    SBVR_ERR_WORKSPACE = -5,          /* workspace missing or too small for this call */
    SBVR_ERR_TIMEOUT = -6,            /* a bounded device-side wait ran out (read by sbvr_workspace_status) */
    SBVR_ERR_UNSUPPORTED = -7,        /* valid arguments, but no kernel covers the combination */
    SBVR_ERR_NOALLOC_LIMIT = -8       /* sbvr_linear_f16_noalloc: the problem needs more than its fixed 4 MiB of scratch */
};

/* Text for a status code.  Replaces the reference's `throw std::runtime_error(cudaGetErrorString)`
 * (sbvr/kernels/sbvr_kernel.cu:624-628), which crossed the binding as a Python RuntimeError. */
SBVR_API const char* sbvr_strerror(int status);

/* cudaError_t of the last failed runtime call made by this library on the calling thread. */
SBVR_API int sbvr_last_cuda_error(void);
/* Which wait ran out, as recorded by the kernel, for the last SBVR_ERR_TIMEOUT that sbvr_workspace_status returned in this
 * process (0 if none): 0x3xx decode GEMV, 0x4xx small-batch kernel, 0x7xx all-reduce kernels, others the GEMM. */
SBVR_API unsigned int sbvr_last_timeout_where(void);
/* Two more words of that record where the kernel leaves them (small-batch kernel: N, and K / 256 << 16 | M << 8 | CTA). */
SBVR_API unsigned int sbvr_last_timeout_info(int i);

/* Device facts the launch heuristics use.  Replaces `_sbvr_cuda_init` (sbvr/kernels/sbvr_ops.cpp:122-150,
 * bound at :153), which cached cudaDeviceProp for every device and printed them.  Any out pointer may be NULL. */
SBVR_API int sbvr_query(int device, int* sm_count, int* smem_per_block_optin, int* l2_bytes, int* cc_major, int* cc_minor);

/* Scratch memory: the device status word of the bounded waits, the quantised activations and the partial sums of
 * row tiles shared by two CTAs (decode kernel), the re-tiled activations and split-K partial sums (batched kernel),
 * staging buffers of the host-pointer entry point.
 * The reference allocates nothing comparable (its kernels keep everything in registers); it does allocate
 * the output inside the binding (sbvr/kernels/sbvr_ops.cpp:100-101), which here is the caller's job.
 * `bytes` = 0 picks a default that covers every Llama-3 8B/70B layer shape up to 32 activation rows.
 * One workspace must not be used by two calls that can overlap on the GPU. */
SBVR_API int sbvr_workspace_create(sbvr_workspace_t** ws, int device, size_t bytes);
SBVR_API int sbvr_workspace_destroy(sbvr_workspace_t* ws);
/* Bytes to ask sbvr_workspace_create for so that every kernel (and the host-pointer entry point) can serve
 * linears of up to M activation rows on an N x K weight: the batched kernel keeps a re-tiled copy of the
 * activations (M x K fp16, M rounded up to its tile) and, when it splits K, fp32 partial sums.  No reference
 * counterpart (the reference has no scratch). */
SBVR_API int sbvr_workspace_bytes(int device, int M, int N, int K, size_t* bytes);
/* Synchronises `stream`, then reads the device status word: SBVR_OK or SBVR_ERR_TIMEOUT. Resets it. */
SBVR_API int sbvr_workspace_status(sbvr_workspace_t* ws, sbvr_stream_t stream);

/* Packed weight -> dense fp16 W[N rows, row pitch ldw elements]; columns 0 .. K_out-1 of every row are
 * written.  K is the padded length the packed tensors cover (multiple of G); K_out <= K is the original
 * inner length: the reference decoder cuts the zero padding the same way (sbvr/core.py:945-947).
 * Device counterpart of `sbvr.decode()` (sbvr/core.py:926-949), bit-exact with it. */
SBVR_API int sbvr_decode_f16(const uint32_t* bvr, const void* coeff_idx, int idx_bytes, const void* coeff, int C,
                    void* W, int ldw, int N, int K, int K_out, int S, int G, sbvr_stream_t stream);

/* y[M, N] = fp16( x[M, K] . W^T + bias ),  fp16 x (row pitch K), fp32 accumulation, bias NULL = none.
 * Replaces `_sbvr_row_deq_mm_T(l_w, r_bvr, r_coeff_idx, r_coeff_cache, bias, use_shfl)`
 * (sbvr/kernels/sbvr_ops.cpp:79-120 -> launch_cuda_sbvr_row_deq_mm_T, sbvr/kernels/sbvr_kernel.cu:876-912),
 * on the reference's non-transposed weight layout, and the dense `x @ decode().T + bias` the reference's
 * Llama flow runs (sbvr_utils/utils_llama.py:147, test_sbvr.py:321).  K must be the padded length
 * (multiple of G).  `ws` may be NULL only for the kernels that need no scratch (see `algo`).
 *   algo 0 = pick; 1 = SIMT dequantise-and-FMA kernel (any S <= 8, no workspace);
 *   2 = tcgen05 FP4 tensor-core kernel for decode (S in {2,3,4}, G in {128,256}, M <= 4, N a multiple of 32 (64 for
 *       S = 2) and at most 262144, K a multiple of 256, M * K <= about 90 K elements (the activation digits stay in shared
 *       memory), bvr / coeff_idx / coeff / x 16-byte aligned; needs a workspace: status word, activation digits,
 *       partial sums);
 *   3 = tcgen05 fp16 GEMM with in-kernel dequantisation for batches and prefill (S in {2,3,4}, any M,
 *       N a multiple of 128; needs a workspace of sbvr_workspace_bytes(...));
 *   4 = tcgen05 FP4 tensor-core kernel for small batches (2 <= M <= 32, at most 16 for G = 128; S, G, N and alignment as
 *       for algo 2, K a multiple of 256 and at most 32768; the activations are quantised by a small kernel in front;
 *       needs a workspace of sbvr_workspace_bytes(...)).  Never picked by algo 0 (see the note at the dispatch in
 *       csrc/api.cu): on request only. */
SBVR_API int sbvr_linear_f16(const void* x, const uint32_t* bvr, const void* coeff_idx, int idx_bytes, const void* coeff,
                    int C, const void* bias, void* y, int M, int N, int K, int S, int G, int algo,
                    sbvr_workspace_t* ws, sbvr_stream_t stream);

/* Same product with HOST x and y: copies x in, runs sbvr_linear_f16, copies y out, all on `stream`
 * (weights stay on the device).  The end-to-end form of the call the reference binding makes with a
 * CPU activation tensor.  x_host / y_host should be pinned for the copies to be asynchronous. */
SBVR_API int sbvr_linear_f16_host(const void* x_host, const uint32_t* bvr, const void* coeff_idx, int idx_bytes,
                         const void* coeff, int C, const void* bias, void* y_host, int M, int N, int K, int S,
                         int G, int algo, sbvr_workspace_t* ws, sbvr_stream_t stream);

/* The same product as sbvr_linear_f16 (algo 0) for callers that must not allocate device memory: hosts that
 * own every byte of the GPU and forbid plugins to call cudaMalloc, latency-critical loops that cannot afford the
 * allocator's implicit device synchronisation, code running next to an open stream capture.  It takes no
 * workspace: the kernels' scratch is a fixed 4 MiB array inside the library's device image (held by every GPU that
 * loads the library, until exit), and neither this call nor anything under it allocates or frees.
 *   - Calls on one device share that array: calls that can overlap on the GPU race; serialise them.
 *   - The first call of each kernel variant (S, G, M, index width) on a device resolves the array's address, sets
 *     kernel attributes and may encode a tensor map: make such first calls outside stream capture, with that device
 *     current.
 *   - M <= 4 runs on the decode kernel (about 4 K M bytes of activation digits + 150 KB of partial sums: always
 *     fits); larger M runs on the batched tensor-core kernel, whose re-tiled activations (about 2 M K bytes) and
 *     split-K partial sums must fit the array (about 2.9 MB of it): M = 16 at K = 4096 and M = 64 at K = 14336 fit,
 *     M = 2048 does not.  A problem that does not
 *     fit returns SBVR_ERR_NOALLOC_LIMIT and launches nothing.  Shapes neither kernel covers run on the SIMT kernel,
 *     which needs no scratch.
 * It has no counterpart in the reference, whose bindings allocate their output on every call
 * (sbvr/kernels/sbvr_ops.cpp:100-101). */
SBVR_API int sbvr_linear_f16_noalloc(const void* x, const uint32_t* bvr, const void* coeff_idx, int idx_bytes,
                                     const void* coeff, int C, const void* bias, void* y, int M, int N, int K, int S,
                                     int G, sbvr_stream_t stream);

/* y[M, N] = fp16( sum_g sum_{a,b} popc(l_a & r_b) * cl[g,m,a] * cr[g,n,b] + bias ): both operands SBVR-encoded (group
 * length 256), l_bvr uint32 [K/32, M, LS], l_idx uint8|uint16 [K/256, M], l_cache fp16 [Cl, LS]; r_* likewise with N, RS.
 * LS, RS in {2, 3, 4}.  Replaces `_sbvr_mm_T(l_bvr, l_coeff_idx, l_coeff_cache, r_bvr, r_coeff_idx, r_coeff_cache, bias)`
 * (sbvr/kernels/sbvr_ops.cpp:35-76 -> launch_cuda_sbvr_mm_T, sbvr/kernels/sbvr_kernel.cu:914-1023, kernel :464-562), with
 * exact popcounts (the reference's 8-bit counters wrap at 256) and fp32 coefficient products (the reference uses half2). */
SBVR_API int sbvr_popc_mm_f16(const uint32_t* l_bvr, const void* l_idx, int l_idx_bytes, const void* l_cache, int Cl, int LS,
                              const uint32_t* r_bvr, const void* r_idx, int r_idx_bytes, const void* r_cache, int Cr, int RS,
                              const void* bias, void* y, int M, int N, int K, sbvr_stream_t stream);

/* y[M, N] = fp16(x[M, K] . W^T + bias) with the weight in the TRANSPOSED ("row-dequant") encoding, i.e. the packed tensors of
 * `sbvr(W, trans=True)` (sbvr/core.py:244-245), whose groups of G run along the output dimension:
 * bvr_t uint32 [N/32, K, S] (bit n % 32 of word (n / 32, k, s)), coeff_idx uint8|uint16 [N/G, K], coeff fp16 [C, S].
 * Replaces `_sbvr_row_deq_mm_T(l_w, r_bvr, r_coeff_idx, r_coeff_cache, bias, use_shfl)` (sbvr/kernels/sbvr_ops.cpp:79-120 ->
 * launch_cuda_sbvr_row_deq_mm_T, sbvr/kernels/sbvr_kernel.cu:876-912; kernels :121-359) for any M: same arithmetic (fp32 sum of
 * the selected coefficients, fp32 products and sums, bias added in fp32, one conversion), deterministic.  N is the padded
 * output length (a multiple of G, like the reference's `r_bvr.size(0) * 32`); S in {2, 3, 4}; idx_bytes in {1, 2}.
 * Needs a workspace (partial sums when K is split over blocks). */
SBVR_API int sbvr_linear_t_f16(const void* x, const uint32_t* bvr_t, const void* coeff_idx, int idx_bytes, const void* coeff,
                               int C, const void* bias, void* y, int M, int N, int K, int S, int G, sbvr_workspace_t* ws,
                               sbvr_stream_t stream);

/* ---- the arithmetic core of the encoder (reference sbvr/core.py:360-722; group length 256) -----------------------
 * mse[b, c] = mean over the 256 values of group b of min_j fp16((d - point[c, j])^2), point[c, j] = the j-th of the 2^S sums of
 * line c, every step rounded as the reference's fp16 tensor ops round (`_get_min_mse_coeff` / `_data_diff_min_mse`,
 * sbvr/core.py:485-500, :520-527).  data fp16 [groups, 256], lines fp16 [L, S], mse fp32 [groups, L]; S in 1..4. */
SBVR_API int sbvr_encode_mse_f16(const void* data, int groups, const void* lines, int L, int S, float* mse,
                                 sbvr_stream_t stream);
/* sel[b, e] = the first j that minimises fp16((data[b, e] - point[which[b], j])^2): the `coeff_comb_sel` of the winning line
 * (sbvr/core.py:494-498).  which int32 [groups] (device), sel uint8 [groups, 256]. */
SBVR_API int sbvr_encode_select_f16(const void* data, int groups, const void* lines, const int* which, int S, uint8_t* sel,
                                    sbvr_stream_t stream);
/* Selectors uint8 [N, Kp] -> bit-planes uint32 [Kp/32, N, S], plane 0 = most significant selector bit, element 32 kw + i in
 * bit i (`_change_coeff_sel_to_bvr` and the layout change of `_encode_to_sbvr`, sbvr/core.py:842-876, :783). */
SBVR_API int sbvr_encode_pack(const uint8_t* sel, int N, int Kp, int S, uint32_t* bvr, sbvr_stream_t stream);

/* ---- the kernels between the linears of a Llama decoder layer ----------------------------------------------
 * Each replaces a chain of eager PyTorch ops of the reference model (models/sbvr_llama.py) by one launch.
 * All tensors fp16, contiguous, 16-byte aligned unless noted. */

/* h_out = h_in + delta (fp16 add; delta NULL = no add; h_out NULL = not stored, may equal h_in);
 * y = weight * fp16(h_out * rsqrt(mean(h_out^2) + eps)).  LlamaRMSNorm.forward (models/sbvr_llama.py:118-123)
 * with the residual add of LlamaDecoderLayer.forward (:395-406) folded in.  hidden % 8 == 0. */
SBVR_API int sbvr_add_rmsnorm_f16(const void* h_in, const void* delta, const void* weight, void* h_out, void* y,
                                  int rows, int hidden, float eps, sbvr_stream_t stream);

/* Rotary embedding of the q and k parts of fused rows qkv[tokens][(n_heads + 2 n_kv) * head_dim], in place, and
 * append of the rotated k and of v to the caches [seqs][n_kv][max_ctx][head_dim] at positions[token]
 * (int32; sequence = token / tokens_per_seq).  cos/sin = fp16(cos|sin(pos * inv_freq[i]) * attn_scaling),
 * products and sum in fp16: LlamaRotaryEmbedding.forward, rotate_half, apply_rotary_pos_emb
 * (models/sbvr_llama.py:169-224) and the cache update of LlamaAttention.forward (:330-336). */
SBVR_API int sbvr_rope_append_f16(void* qkv, const int* positions, const float* inv_freq, float attn_scaling,
                                  void* kcache, void* vcache, int tokens, int tokens_per_seq, int n_heads, int n_kv,
                                  int head_dim, int max_ctx, sbvr_stream_t stream);

/* out[token][head][:] = softmax(q . K^T * scale) . V over cache positions 0 .. positions[token] of the token's
 * sequence, grouped-query (n_heads % n_kv == 0, ratio 1, 2, 4 or 8), head_dim 128.  Serves decode (one token per
 * sequence) and causal prefill (every token attends up to itself; its k, v must be in the cache already).
 * nsplit > 1 splits the positions over CTAs (decode at long context), a second small launch merges the splits; it
 * needs `scratch` of tokens * n_heads * nsplit * 130 floats.  repeat_kv + eager_attention_forward (models/sbvr_llama.py:243-278). */
SBVR_API int sbvr_attention_f16(const void* qkv, const void* kcache, const void* vcache, const int* positions,
                                void* out, float* scratch, int tokens, int tokens_per_seq, int n_heads, int n_kv,
                                int head_dim, int max_ctx, float scale, int nsplit, sbvr_stream_t stream);

/* Decode form of the two calls above in one launch: one new token per sequence; q and the token's k are rotated
 * inside the attention kernel (qkv is left as it is), the rotated k and v are appended to the caches at
 * positions[token] by the CTA that attends to that position.  Same scratch rules as sbvr_attention_f16. */
SBVR_API int sbvr_rope_attention_f16(const void* qkv, const int* positions, const float* inv_freq, float attn_scaling,
                                     void* kcache, void* vcache, void* out, float* scratch, int tokens, int n_heads,
                                     int n_kv, int head_dim, int max_ctx, float scale, int nsplit, sbvr_stream_t stream);

/* out[row][i] = fp16(silu(gate[row][i])) * up[row][i] with gate_up[row] = [gate (inter) | up (inter)]:
 * the activation of LlamaMLP.forward (models/sbvr_llama.py:238-240) on a fused gate/up linear.  inter % 8 == 0. */
SBVR_API int sbvr_silu_mul_f16(const void* gate_up, void* out, int rows, int inter, sbvr_stream_t stream);

/* out[token][:] = table[ids[token]][:]  (nn.Embedding of LlamaModel, models/sbvr_llama.py:568-672). */
SBVR_API int sbvr_embedding_f16(const int* ids, const void* table, void* out, int tokens, int hidden,
                                sbvr_stream_t stream);

/* out[row] = index of the first maximum of logits[row][0 .. vocab-1] (greedy decoding; torch.argmax's tie rule).
 * `scratch` (128 floats + 128 ints, may be NULL) lets few rows of a large vocabulary be scanned by many SMs. */
SBVR_API int sbvr_argmax_f16(const void* logits, int* out, float* scratch, int rows, int vocab, sbvr_stream_t stream);

/* ---- decode linears with the preceding element-wise op folded in ---------------------------------------------
 * The decode GEMV (algo 2 of sbvr_linear_f16: M <= 4, N % 32 == 0, K % 256 == 0) turns the activation row into
 * block-fixed-point digits in a small kernel of its own before the product; the op in front of the linear is applied
 * there instead of in a launch of its own:
 *   SBVR_XOP_SILU_MUL     x = fp16(silu(g)) * u, `x` pointing at rows [g (K) | u (K)] of pitch 2K
 *                         (LlamaMLP.forward, models/sbvr_llama.py:238-240, in front of down_proj)
 *   SBVR_XOP_ADD_RMSNORM  x = norm_weight * fp16((h + delta) * rsqrt(mean((h + delta)^2) + eps)) with h = `x`
 *                         (pitch K), delta NULL = no add; h + delta is also stored to h_out (may be NULL; must be a
 *                         buffer other than h and delta: both are still being read while it is written; overlap is
 *                         refused with SBVR_ERR_BAD_ARG) (LlamaDecoderLayer.forward :395-406 + LlamaRMSNorm.forward :118-123)
 *   SBVR_XOP_DIGITS       x (still required: the rows as fp16, for the checks) has ALREADY been quantised into this
 *                         workspace by the kernel launched directly before on this stream: one of the two all-reduce +
 *                         RMSNorm calls below with emit_digits = 1 for the same M and K.  Saves the quantiser launch of
 *                         rows longer than 4096.  Group length 256 only.
 * Same rounding as sbvr_silu_mul_f16 / sbvr_add_rmsnorm_f16 followed by sbvr_linear_f16.  Returns
 * SBVR_ERR_UNSUPPORTED where the decode GEMV does not apply (the caller then runs the separate kernels). */
enum { SBVR_XOP_NONE = 0, SBVR_XOP_SILU_MUL = 1, SBVR_XOP_ADD_RMSNORM = 2, SBVR_XOP_DIGITS = 3 };
SBVR_API int sbvr_linear_fused_f16(int x_op, const void* x, const void* delta, const void* norm_weight, void* h_out,
                                   float eps, const uint32_t* bvr, const void* coeff_idx, int idx_bytes, const void* coeff,
                                   int C, const void* bias, void* y, int M, int N, int K, int S, int G,
                                   sbvr_workspace_t* ws, sbvr_stream_t stream);

/* ---- tensor parallel: one-shot all-reduce fused with the residual add and the RMSNorm ----------------------
 * delta = fp16(sum over ranks of partial_r) (fp32, rank order), h_out = h_in + delta, y = RMSNorm(h_out) * weight,
 * for the [rows, hidden] partial outputs that the row-parallel linears (o, down) of every rank wrote into buffer
 * (call_idx & 1) of a symmetric allocation mapped by all ranks.  peer_bufs_dev / peer_flags_dev: device arrays of
 * `world` 64-bit addresses (every rank's buffer area of 2 x buf_elems fp16, and its array of `world` zero-initialised
 * uint32 flags).  step_dev: device int32 the caller increments once per model step; calls_per_step (even) and
 * call_idx order the calls inside a step.  Peer data is read with plain loads over NVLink; waits on peers are
 * bounded and report through the workspace status word.  For decode-sized batches; large batches should use NCCL.
 * No counterpart in the reference (it has no tensor-parallel path); it takes the place of ncclAllReduce +
 * the add and LlamaRMSNorm of models/sbvr_llama.py:118-123, :395-406. */
SBVR_API int sbvr_allreduce_add_rmsnorm_f16(const void* peer_bufs_dev, const void* peer_flags_dev, const int* step_dev,
                                            int calls_per_step, int call_idx, int rank, int world, size_t buf_elems,
                                            const void* h_in, const void* weight, void* h_out, void* y, int rows,
                                            int hidden, float eps, sbvr_workspace_t* ws, sbvr_stream_t stream);
/* The same call that also leaves y as activation digits of the decode GEMV in the workspace (emit_digits = 1; rows <= 4,
 * hidden a multiple of 2048, group length 256), for an sbvr_linear_fused_f16(SBVR_XOP_DIGITS, ...) with K = hidden launched
 * directly behind it on the same stream and workspace.  SBVR_ERR_UNSUPPORTED (nothing launched) where that form does not apply. */
SBVR_API int sbvr_allreduce_add_rmsnorm_digits_f16(const void* peer_bufs_dev, const void* peer_flags_dev, const int* step_dev,
                                                   int calls_per_step, int call_idx, int rank, int world, size_t buf_elems,
                                                   const void* h_in, const void* weight, void* h_out, void* y, int rows,
                                                   int hidden, float eps, int emit_digits, sbvr_workspace_t* ws,
                                                   sbvr_stream_t stream);

/* ---- tensor parallel, decode: the all-reduce folded into the row-parallel GEMV and its consumer ----------------
 * sbvr_linear_push_f16 is sbvr_linear_fused_f16 (x_op may also be SBVR_XOP_NONE) whose result does not go to y: the
 * decode GEMV's epilogue stores every pair of fp16 outputs together with the call's epoch as one 8-byte packet into
 * slot [call_idx & 1][rank] of EVERY rank's receive area (this rank's own included; an area is uint64
 * [2][world][rows_max][N / 2], zero before the first call), with plain stores over NVLink.  Where to push is described
 * by an sbvr_push_desc_t in DEVICE memory (written once per call index by the caller; the kernel reads it, the host
 * side of the library does not).  sbvr_ll_reduce_add_rmsnorm_f16 is the other end: it reads only THIS rank's area,
 * waits (bounded, reported through the workspace status word) until the packets of all ranks carry the epoch, adds them
 * in rank order in fp32 and finishes h_out = h_in + fp16(sum), y = RMSNorm(h_out) * weight.  No flag exchange, no load
 * over NVLink, no multicast.  Epoch = *step * calls_per_step + call_idx + 1 as for the one-shot form; both ends of a call
 * must be given the same step counter, calls_per_step (even) and call_idx.  M <= 4, G = 256 (decode GEMV only): returns
 * SBVR_ERR_UNSUPPORTED otherwise, and the caller uses sbvr_allreduce_add_rmsnorm_f16 or NCCL.
 * No counterpart in the reference (it has no tensor-parallel path); the pair replaces the row-parallel linear's store,
 * ncclAllReduce, and the add + LlamaRMSNorm of models/sbvr_llama.py:118-123, :395-406. */
typedef struct sbvr_push_desc {
    unsigned long long peer_recv[16];   /* base address of every rank's receive area (entries 0 .. world-1) */
    const int* step;                    /* device int32: decode step counter, bumped once per step by the caller */
    int calls_per_step, call_idx, rank, world, rows_max;
    int reserved;
} sbvr_push_desc_t;
SBVR_API int sbvr_linear_push_f16(int x_op, const void* x, const void* delta, const void* norm_weight, void* h_out, float eps,
                                  const uint32_t* bvr, const void* coeff_idx, int idx_bytes, const void* coeff, int C,
                                  const void* bias, const sbvr_push_desc_t* push_desc_dev, int M, int N, int K, int S, int G,
                                  sbvr_workspace_t* ws, sbvr_stream_t stream);
/* follows_push = 1 promises that the kernel launched on `stream` directly before this call is the sbvr_linear_push_f16
 * of the same call_idx, and that h_in, weight and the step counter were final before that linear: the kernel then does
 * not wait for the linear to end (the linear lets it start only after its own inputs were complete; the packets announce
 * themselves).  With 0 it waits for everything in front of it on the stream like any other kernel of the library. */
SBVR_API int sbvr_ll_reduce_add_rmsnorm_f16(const void* recv_local, const int* step_dev, int calls_per_step, int call_idx,
                                            int world, int rows_max, const void* h_in, const void* weight, void* h_out,
                                            void* y, int rows, int hidden, float eps, int follows_push,
                                            sbvr_workspace_t* ws, sbvr_stream_t stream);
SBVR_API int sbvr_ll_reduce_add_rmsnorm_digits_f16(const void* recv_local, const int* step_dev, int calls_per_step,
                                                   int call_idx, int world, int rows_max, const void* h_in,
                                                   const void* weight, void* h_out, void* y, int rows, int hidden, float eps,
                                                   int follows_push, int emit_digits, sbvr_workspace_t* ws,
                                                   sbvr_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SBVR_B200_H */
