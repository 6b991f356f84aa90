/*
 * C-ABI of the B200 (sm_100a) quantized-weight linear library for cccc.
 *
 * The shared library built from cccc-lite_b200/csrc is a drop-in for the part of the
 * reference's `cccc-cuda` plug-in library that the quantized-weight linear path uses, plus
 * the fused entry points that replace the dequantise-then-cuBLAS sequence of
 * cccc/cublas_real.h.  Plain pointers and sizes only; every pointer is a DEVICE pointer
 * unless a comment says otherwise.  `type` integers are cccc::DataType values
 * (cccc/types.h:24-34): 0 float, 1 double, 2 half, 3 bfloat16, 4 fp8_e4m3, 5 fp8_e5m2,
 * 6 fp4_e2m1 (two nibbles per byte, low nibble = even element).
 *
 * Return convention (cccc-cuda/cuda_functions.cu:26-40, :3086-3088): 0 = ok, 1 = CUDA
 * error (a line "<label> kernel launch failed: <message>" goes to stderr), -1 = unsupported
 * type pair or argument.
 */
#pragma once

#ifndef C_EXPORT
#ifdef _WIN32
#define C_EXPORT extern "C" __declspec(dllexport)
#else
#define C_EXPORT extern "C" __attribute__((visibility("default")))
#endif
#endif

/* ---- entry points that exist in the reference (same names, same arguments) -------------- */

/* Replaces cuda_convert, cccc-cuda/cuda_functions.h:224 (cuda_functions.cu:3066-3090).
 * Converts n elements src_type -> dst_type, multiplying by `scale` where the reference's
 * kernel for that pair does.  Same 7x7 table of supported pairs; same-type with scale 1
 * copies n BYTES (as the reference does).  Synchronous like the reference (device sync
 * before returning). */
C_EXPORT int cuda_convert(const void* src, int src_type, void* dst, int dst_type, unsigned int n, float scale);

/* Replaces cuda_fp4_blockscale_to_bf16, cuda_functions.h:232 (cuda_functions.cu:2926-2960).
 * src_scales holds one E4M3 byte per `block_size` consecutive elements (a dequant multiplier). */
C_EXPORT int cuda_fp4_blockscale_to_bf16(const void* src_nibbles, const void* src_scales, void* dst,
    unsigned int n_elems, unsigned int block_size);

/* Replaces cuda_float_to_fp4_blockscale, cuda_functions.h:230 (cuda_functions.cu:2896-2950). */
C_EXPORT int cuda_float_to_fp4_blockscale(const void* src, void* dst_nibbles, void* dst_scales,
    unsigned int n_elems, unsigned int block_size);

/* Replaces cuda_check_error, cuda_functions.h:200 (cuda_functions.cu:48-51): device sync, report
 * any pending CUDA error or any error status raised by this library's kernels (a bounded wait
 * that ran out); 0 = clean. */
C_EXPORT int cuda_check_error(const char* label);

/* Replaces cuda_clear_last_error, cuda_functions.h:198 (cuda_functions.cu:42-45). */
C_EXPORT void cuda_clear_last_error(void);

/* ---- additions: the fused linear -------------------------------------------------------- */

/* Replaces the sequence at cccc/cublas_real.h:943-964 (and its mirror :1066-1087, and the typed
 * overloads :673-684, :740-751): grow workspace, dequantise the whole weight to BF16,
 * cublasGemmEx BF16xBF16->BF16 with FP32 compute, device sync.
 *
 *   Y[m*ldy_m + n*ldy_n] = bf16( alpha * sum_k dq(W[n*ldw + k]) * X[m*ldx + k] + beta * Y[...] )
 *
 * W  : [N_out, K] quantised weight, K contiguous (cccc stores (K, N_out) column-major, which is
 *      the same bytes), w_type 4, 5 or 6; ldw in ELEMENTS.
 * dq : types 4/5: rne_bf16(decode(byte) * inv_scale).  Type 6 with blk_scales != NULL:
 *      rne_bf16(table[nibble] * e4m3(blk_scales[(n*ldw+k)/16])), inv_scale ignored, as the
 *      reference does (block size 16 is fixed at its call sites, cublas_real.h:953); type 6
 *      with blk_scales == NULL: rne_bf16(table[nibble] * inv_scale).
 * X  : [M_tokens, K] BF16, ldx in elements.  Y: BF16; ldy_m / ldy_n are the element strides of
 *      the token and output-feature index (cccc's layout is ldy_m = N_out (ldc), ldy_n = 1; the
 *      mirrored operand order, weight as B, gives ldy_m = 1, ldy_n = ldc).
 * stream : a cudaStream_t (NULL = legacy default stream).  The call is ASYNCHRONOUS on that
 *      stream; cuda_check_error() or any synchronising call makes the result visible, which
 *      is where the reference's own wrappers synchronise too.
 * Any shape, stride or alignment is accepted: aligned shapes take the TMA-fed kernels, the rest
 * a plain kernel.  The first call on a device allocates that device's workspace (a few MB);
 * make it before any stream capture.  Calls that share a device must be ordered on one stream
 * (they share the workspace), as the reference's single `Cublas` instance requires too.
 * flags: bit 0 = launch with programmatic dependent launch so that this call's weight prefetch
 * overlaps the tail of the previous kernel on the stream (X, Y are only touched after that
 * kernel has finished).  bit 2 = Y holds float32 instead of BF16 (same strides, in elements): the
 * unrounded result, which is what a row-parallel (K-split) shard hands to the all-reduce so that
 * the sum over shards is rounded to BF16 once.  bit 3 = round alpha * product to BF16 before beta * Y
 * is added: Y = bf16( bf16(alpha * W x) + beta * Y ), which with beta = 1 is the reference's linear
 * followed by its residual add (two BF16 tensors, scripts/convert_weights.py:562, :582).
 * bits 8-10 = kernel choice for tests and tuning (0 = chosen by shape: the decode kernel up to 8 tokens,
 * the streaming tensor-core kernel from 9 to 128 tokens where K % 256 == 0, the prefill kernel above;
 * 1-3 = the prefill kernel with one CTA per tile: 128 features x 128 tokens, 128 x 256, 256 x 256;
 * 4-6 = with CTA pairs: 256 x 256, 512 features x 256 tokens, 256 x 512 - the six tile shapes give the same
 * result bit for bit; 7 = the streaming kernel wherever it accepts the shape, i.e. from 1 token).
 * bit 11 = never the streaming kernel (the decode kernel up to 32 tokens, the prefill kernel above).
 * bit 12 = the native-operand kernel wherever it accepts the shape (FP8 up to 32 tokens with a power-of-two
 * inv_scale and K % 128 == 0; FP4 up to 32 tokens with K % 256 == 0): the quantised weights go from HBM through
 * shared memory into tcgen05.mma (kind::f8f6f4, kind::mxf4nvf4 with the block scales) unchanged, the BF16
 * activations as a few narrow rows whose sum they are.  Without the bit it is taken where it is the fastest:
 * launches with between one and two 128-feature tiles per SM (gate+up as a group: every CTA streams one whole tile,
 * nothing is exchanged) and lm_head-sized ones (FP8 256 MB, FP4 48 MB of weights); FP8 only from 3 tokens.  (FP4 block scales are
 * read as UNSIGNED E4M3 there, which is what the reference's converter writes; a token row with an infinity or NaN
 * gives NaN outputs in the FP4 kernel.)  bit 13 = never that kernel.  bit 14 = the FP8 form of that kernel that splits
 * the activations itself (up to 8 tokens) instead of a kernel of its own doing it before. */
C_EXPORT int cuda_gemm_wq_bf16(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X,
    void* Y, unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx,
    unsigned int ldy_m, unsigned int ldy_n, float alpha, float beta, void* stream, unsigned int flags);

/* One linear of a group (see cuda_gemm_wq_bf16_group); fields as the arguments of cuda_gemm_wq_bf16. */
typedef struct cuda_wq_linear
{
    const void* W;
    const void* blk_scales;
    void* Y;
    float inv_scale, alpha, beta;
    unsigned int N_out, ldw, ldy_m, ldy_n;
} cuda_wq_linear;

/* Several quantised linears that read the SAME activations X (and so share M_tokens, K, ldx and the
 * weight type) in one call: the q/k/v projections of a layer, or gate and up.  The reference issues
 * them as separate ops (scripts/convert_weights.py:488-524 generates one batchedMul per projection,
 * each reaching cccc/cublas_real.h:943-964); here up to 3 of them that the decode kernel takes
 * (M_tokens <= 32, TMA-eligible operands) run as ONE launch whose row blocks are dealt to the SMs
 * together, which saves the per-launch latency that dominates small linears.  Anything else (more
 * linears, more tokens, unaligned operands) is run one linear at a time, so the result is always
 * that of `count` separate cuda_gemm_wq_bf16 calls.  stream and flags as there. */
C_EXPORT int cuda_gemm_wq_bf16_group(int w_type, unsigned int count, const cuda_wq_linear* linears, const void* X,
    unsigned int M_tokens, unsigned int K, unsigned int ldx, void* stream, unsigned int flags);

/* W8A8: E4M3 weights times E4M3 activations with FP32 accumulation - the mode the reference's dispatcher takes when
 * its activation type is FP8_E4M3 (cccc/cublas_real.h:619-666 and 692-739: quantise the BF16 activations, then a cublasLt
 * FP8 x FP8 matmul with both scale pointers).  X is BF16 as there; this call quantises it itself:
 *   act_scale > 0: static, q = e4m3(x / act_scale) and the multiplier back is act_scale (cublas_real.h:627-632);
 *   act_scale == 0: dynamic, one absmax over the whole [M_tokens, K] tensor, q = e4m3(x * 448 / absmax), multiplier back
 *                   absmax / 448 (cccc-cuda/cuda_functions.cu:2611-2669);
 * and Y = alpha * w_inv_scale * multiplier * (W . q) + beta * Y (BF16, or float32 with flags bit 2; bit 3 and bit 0 as
 * cuda_gemm_wq_bf16).  Both operands go into tcgen05.mma kind::f8f6f4 unchanged: up to 32 tokens in a kernel that
 * streams the weights once over all SMs, above that on CTA pairs (cta_group::2; 256- or 512-feature tiles, or a
 * persistent form whose epilogue overlaps the next tile; flags bits 8-9 = 1 / 2 / 3 force one of them for tests, 0 lets
 * the shape decide).  Needs K % 128 == 0, ldw % 16 == 0, ldx % 8 == 0, 16-byte aligned W and X, at most 65535 tokens
 * and M_tokens * K quantised bytes within the 64 MB workspace; anything else returns -1 (the caller keeps its own
 * path).  Shares the device's workspace with cuda_gemm_wq_bf16: same ordering rule. */
C_EXPORT int cuda_gemm_w8a8_bf16(const void* W, float w_inv_scale, const void* X, float act_scale, void* Y, unsigned int N_out,
    unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m, unsigned int ldy_n, float alpha,
    float beta, void* stream, unsigned int flags);

/* The elementwise ops of the W8A8 mode on E4M3 tensors; they replace the entry points of the same names
 * (cccc-cuda/cuda_functions.h:181-192, cuda_functions.cu:2446-2544) with the same arguments and bits: values widened to
 * float, combined, narrowed with the round-to-nearest-even saturating conversion.  On the legacy default stream.
 *   add:        R = a A + b B + r R            silu:  R = x * sigmoid(x)            elementmul: R = a A B + r R
 *   addbias:    R = a bias[idx] + b R  (X already copied into R; idx = (i % (size_mc * size_b)) / size_mc, or i % size_b
 *               when size_mc <= 1); _bf16bias takes a BF16 bias. */
C_EXPORT int cuda_add_fp8e4m3(const void* A, const void* B, void* R, unsigned int n, float a, float b, float r);
C_EXPORT int cuda_addbias_fp8e4m3(const void* X, const void* bias, void* R, unsigned int n, unsigned int size_mc, unsigned int size_b,
    float a, float b);
C_EXPORT int cuda_addbias_fp8e4m3_bf16bias(const void* X, const void* bias, void* R, unsigned int n, unsigned int size_mc,
    unsigned int size_b, float a, float b);
C_EXPORT int cuda_silu_fp8e4m3(const void* A, void* R, unsigned int n);
C_EXPORT int cuda_elementmul_fp8e4m3(const void* A, const void* B, void* R, unsigned int n, float a, float r);
/* Embedding rows into an E4M3 activation tensor (cccc-cuda/cuda_functions.h:193-196, cuda_functions.cu:1615-1667), same
 * arguments and bits: ids are floats holding token numbers, [B][T]; W is [vocab][D]; Y is [B][T][D].  fp8_to_fp8
 * re-encodes an E4M3 table at inv_scale_w to scale 1; bf16_to_fp8 encodes a BF16 table at scale 1. */
C_EXPORT int cuda_embed_fwd_fp8_to_fp8(const void* ids, const void* W, void* Y, int D, int T, int B, float inv_scale_w);
C_EXPORT int cuda_embed_fwd_bf16_to_fp8(const void* ids, const void* W, void* Y, int D, int T, int B);

/* Up to three W8A8 linears that read the same activations (q/k/v, gate/up) as one call: the activations are quantised
 * once and the members' feature tiles are dealt out together.  Members as for cuda_gemm_wq_bf16_group (blk_scales
 * unused); the result is that of `count` separate cuda_gemm_w8a8_bf16 calls, bit for bit.  -1 where one of those would
 * return it, for more than three members, or for a member without outputs. */
C_EXPORT int cuda_gemm_w8a8_bf16_group(unsigned int count, const cuda_wq_linear* linears, const void* X, float act_scale,
    unsigned int M_tokens, unsigned int K, unsigned int ldx, void* stream, unsigned int flags);

/* Both operands E4M3 already (cccc/cublas_real.h:754-834, the overloads Cublas::gemm takes when typeA and typeB are both
 * quantised): Y = alpha * w_inv_scale * x_inv_scale * (W . X) with FP32 accumulation; y_type 3 (BF16; beta * Y added) or
 * 4 (E4M3: the BF16 result re-encoded at scale 1 with the reference's encoder, beta ignored, as there).  X_fp8 is
 * [M_tokens][ldx] bytes.  Limits and ordering as cuda_gemm_w8a8_bf16; flags bit 0 and bits 8-9 only. */
C_EXPORT int cuda_gemm_fp8_fp8(const void* W, float w_inv_scale, const void* X_fp8, float x_inv_scale, void* Y, int y_type,
    unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx, unsigned int ldy_m,
    unsigned int ldy_n, float alpha, float beta, void* stream, unsigned int flags);

/* Replaces cuda_bf16_to_fp8e4m3_dynamic (cccc-cuda/cuda_functions.h, cuda_functions.cu:2659-2669), same arguments and bits:
 * absmax of n BF16 values into *d_absmax_tmp, dst = e4m3(src * 448 / absmax), *d_inv_scale_out = absmax / 448 (1 for an
 * all-zero tensor).  On the legacy default stream like the reference's. */
C_EXPORT int cuda_bf16_to_fp8e4m3_dynamic(const void* src, void* dst_fp8, unsigned int n, void* d_absmax_tmp, void* d_inv_scale_out);

/* No counterpart in the reference.  The same linear as cuda_gemm_wq_bf16 for callers that cannot
 * allocate when they issue it: hosts that plan every byte of device memory up front (or have already
 * committed all of it) and hand the library no allocator, and latency-critical loops that may not take
 * the allocator's locks or the device-wide synchronisation a cudaMalloc/cudaFree can imply.  cuda_gemm_wq_bf16 allocates its per-device workspace on first use; this entry point
 * calls no cudaMalloc/cudaFree and no allocating library routine: its scratch (FP32 partial tiles of
 * the split-k schedule, arrival counters, a status word) is a fixed 520 KB device array inside the
 * library, held by every GPU that loads it until the process ends.
 * Limits: M_tokens <= 8, a device with at most 256 SMs, and operands the TMA kernel takes (16-byte
 * aligned pointers, K % 64 == 0, ldw % 16 == 0, ldx % 8 == 0; FP4: block scales given, K % 256 == 0,
 * ldw % 256 == 0).  Anything else returns -1 with a line on stderr saying which limit was hit.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and the
 * device's attributes; make that first call outside any stream capture.
 * All calls on a device share the one array: order them on one stream.  Two calls that overlap on the
 * GPU (different streams, or the same buffers from two threads) race on it.  The array keeps the
 * previous call's contents; the counters that must start at zero, and the status word, are cleared on
 * the stream by every call (a small memset node ahead of the kernel).
 * Arguments and result as cuda_gemm_wq_bf16.  flags bit 0: programmatic dependent launch, accepted
 * for symmetry with cuda_gemm_wq_bf16; because the clearing memset sits between this call's kernel
 * and the previous kernel of the stream, nothing overlaps here and the bit changes no timing.
 * flags bit 1: checked call - synchronise the stream after the launch and return 1 if one of THIS
 * call's bounded waits ran out.  Without it such a failure is not reported at all: the next call
 * clears the status word before it runs, and cuda_check_error() does not look at this array. */
C_EXPORT int cuda_gemm_wq_bf16_static(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X,
    void* Y, unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx,
    unsigned int ldy_m, unsigned int ldy_n, float alpha, float beta, void* stream, unsigned int flags);

/* ---- additions: tensor-parallel exchange ----------------------------------------------------- */

/* No counterpart in the reference (it has no tensor parallelism; its only multi-GPU mode copies
 * gradients with cudaMemcpyPeer, cccc/Matrix.cpp:498-517).  One-shot all-reduce of the FP32 partial
 * sums of a row-parallel linear over peer-mapped memory, rounded to BF16 once:
 *     out_bf16[i] = bf16( sum over ranks of partial[i] ),  i < n,  the same bits on every rank.
 * peer_recv_ptrs / peer_flag_ptrs are HOST arrays of `world` device pointers: entry r is rank r's
 * receive area / flag area as mapped into THIS process (symmetric memory or IPC mappings; sizes from
 * the three helpers below, flag area and counters zeroed once before the first call).  seq_counters
 * is a small local device buffer.  Every rank must issue the same sequence of calls with the same n
 * and n_max; n and n_max are multiples of 4, n <= n_max.  Asynchronous on `stream`; flags bit 0 =
 * programmatic dependent launch.  A peer that does not arrive within one second raises the
 * library's status word (reported by cuda_check_error) instead of hanging. */
C_EXPORT int cuda_b200_allreduce_f32_to_bf16(const unsigned long long* peer_recv_ptrs,
    const unsigned long long* peer_flag_ptrs, void* seq_counters, const void* partial, void* out_bf16, unsigned int n,
    unsigned int n_max, int rank, int world, void* stream, unsigned int flags);
C_EXPORT unsigned long long cuda_b200_allreduce_recv_bytes(int world, unsigned int n_max);
C_EXPORT unsigned long long cuda_b200_allreduce_flag_bytes(int world);
C_EXPORT unsigned long long cuda_b200_allreduce_counter_bytes(void);

/* No counterpart in the reference, as above.  The row-parallel (K-split) linear and its all-reduce as
 * ONE kernel: each CTA of the decode kernel pushes the FP32 partial of its block of output features
 * into every rank's receive area over NVLink peer stores, publishes that block's sequence number,
 * waits (bounded, one second) for the other ranks' numbers, adds the `world` partials in rank order
 * and writes Y once:
 *     Y[m, n] = bf16( sum over ranks r of alpha * (X_r[m, :] . dq(W_r)[n, :]) ),  the same bits on
 * every rank, the bits cuda_gemm_wq_bf16 (flags bit 2) followed by cuda_b200_allreduce_f32_to_bf16
 * produce.  Arguments of the linear as cuda_gemm_wq_bf16 (K, ldw, ldx describe this rank's shard;
 * beta is 0); flags bit 0 and bit 2 (Y = float32) as there.  The exchange areas are those of
 * cuda_b200_allreduce_f32_to_bf16 in layout: receive area of cuda_b200_allreduce_recv_bytes(world,
 * n_max) bytes with n_max >= M_tokens * N_out, flag area of cuda_b200_fused_flag_bytes(world) bytes
 * and local counters of cuda_b200_fused_counter_bytes() bytes, zeroed once; use areas of their own
 * for this entry point.  Every rank issues the same sequence of calls.  Returns -1 for a shape the
 * fused kernel does not take (more than 32 tokens, unaligned operands, more than 32768 features,
 * M_tokens * N_out > n_max): use the two separate calls then.  world == 1 is the plain linear. */
C_EXPORT int cuda_gemm_wq_bf16_allreduce(int w_type, const void* W, const void* blk_scales, float inv_scale, const void* X,
    void* Y, unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx,
    unsigned int ldy_m, unsigned int ldy_n, float alpha, const unsigned long long* peer_recv_ptrs,
    const unsigned long long* peer_flag_ptrs, void* seq_counters, unsigned int n_max, int rank, int world, void* stream,
    unsigned int flags);
C_EXPORT unsigned long long cuda_b200_fused_flag_bytes(int world);
C_EXPORT unsigned long long cuda_b200_fused_counter_bytes(void);

/* ---- additions: the caller side of the path ---------------------------------------------------- */

/* Greedy choice on the device: for each of `rows` rows of BF16 logits (row stride ld elements),
 * idx_out[row] (int32) = index of the first maximum, val_out[row] (float32, may be NULL) = its value;
 * NaN entries never win, a row of only NaN gives -1.  Replaces the per-token device-to-host copy of
 * all V float logits that the reference's host sampler needs (cccc/Net.cpp:1783,
 * cccc-llm/cccc-llm.cpp:181-343, which with temperature 0 returns the first maximum).
 * Asynchronous on `stream`. */
C_EXPORT int cuda_argmax_bf16(const void* logits, unsigned int rows, unsigned int cols, unsigned long long ld,
    void* idx_out, void* val_out, void* stream);

/* ---- additions: the ops between the linears of a decode layer -------------------------------- */

/* Replaces cuda_rms_norm_fwd for BF16 rows (cccc-cuda/cuda_functions.h:55, kernel
 * cuda_functions.cu:904-933): Y[r][i] = bf16( (x[r][i] * invstd_r) * scale[i] ), invstd_r =
 * rsqrt(mean_i x[r][i]^2 + epsilon), the squares summed in the reference kernel's order.  scale may
 * be NULL (1.0).  With residual != NULL the add that precedes the norm in a layer (R1 = X + O_out,
 * scripts/convert_weights.py:567-572) is folded in: x = bf16(X + residual), stored to sum_out when
 * that is not NULL (sum_out may alias X or residual).  Rows are contiguous (`inner` elements apart).
 * Asynchronous on `stream`; flags bit 0 = programmatic dependent launch. */
C_EXPORT int cuda_rms_norm_bf16(const void* X, const void* residual, void* sum_out, void* Y, const void* scale,
    unsigned int rows, unsigned int inner, float epsilon, void* stream, unsigned int flags);

/* Replaces cuda_rope_fwd for BF16 (cuda_functions.h:73, kernel cuda_functions.cu:1324-1344): half-rotate
 * RoPE of X (D, T, 1, B) = [B][T][D] with table row t + pos_offset; tables are [rows][D/2] BF16
 * (cccc/NetCifa.cpp:431-475). */
C_EXPORT int cuda_rope_bf16(const void* X, void* Y, const void* cos_tab, const void* sin_tab, unsigned int D, unsigned int T,
    unsigned int B, unsigned int pos_offset, void* stream, unsigned int flags);

/* Replaces cuda_embed_fwd for BF16 tables (cuda_functions.h:97, kernel cuda_functions.cu:1574-1594):
 * Y[t][:] = W[ids[t]][:].  ids are int32 on the device (the reference passes floats and casts; here
 * the token comes straight from cuda_argmax_bf16).  An id outside [0, vocab) gives a zero row. */
C_EXPORT int cuda_embed_bf16(const void* ids, const void* W, void* Y, unsigned int D, unsigned int n_tokens, unsigned int vocab,
    void* stream, unsigned int flags);

/* The gated MLP's activation in one pass: out = bf16( bf16( g * bf16(sigmoid(g)) ) * u ), which is the
 * reference's silu (a BF16 sigmoid tensor times its input, cccc/MatrixEx.cpp:744-763) followed by
 * elementMul (cccc/Matrix.cpp:1360-1386), with their three BF16 tensors' roundings.  Row strides in
 * elements. */
C_EXPORT int cuda_swiglu_bf16(const void* gate, const void* up, void* out, unsigned int rows, unsigned int cols,
    unsigned int ld_gate, unsigned int ld_up, unsigned int ld_out, void* stream, unsigned int flags);

/* Attention of ONE new token per sequence over a BF16 KV cache, with everything the reference runs
 * between the q/k/v projections and the o projection folded into one launch
 * (scripts/convert_weights.py:488-560): the per-head RMSNorm of q and k (Qwen3; NULL weights = none),
 * RoPE at the token's position, the cache append (cccc/MatrixOp.cpp:237-276), and
 * cccc/MatrixEx.cpp:3018-3104 with T_q = 1: scores = bf16(K q / sqrt(dk)), softmax probabilities
 * rounded to BF16, out = bf16(V p).  No tiled or permuted copies of the cache and no score matrix in
 * memory (the reference makes both, convert_weights.py:551-560, MatrixEx.cpp:3040-3050): each
 * (sequence, kv head) is cut into up to 16 splits that run as one thread-block cluster and combine
 * through distributed shared memory.  Query head h reads kv head h / (H / Hkv).
 *   q, k, v  : the projections' outputs, [B] rows of H*head_dim, Hkv*head_dim, Hkv*head_dim BF16
 *              values, row strides ldq/ldk/ldv in elements (they may be slices of one buffer)
 *   caches   : [B][Hkv][T_max][head_dim] BF16
 *   pos      : DEVICE int32 [B]: the row the new token is appended at (= tokens already cached);
 *              rows 0..pos are attended.  pos >= T_max appends nothing and attends T_max rows.
 *   tables   : RoPE cos / sin, [>= max pos + 1][head_dim / 2] BF16
 *   out      : [B] rows of H*head_dim BF16, stride ldo
 * head_dim 64 or 128; H / Hkv in {1, 2, 4, 8}; v and the caches 16-byte aligned, ldv % 8 == 0;
 * anything else returns -1.  dk <= 0 means head_dim. */
typedef struct cuda_attn_decode
{
    const void* q;
    const void* k;
    const void* v;
    const void* q_norm;
    const void* k_norm;
    const void* cos_tab;
    const void* sin_tab;
    void* k_cache;
    void* v_cache;
    const void* pos;
    void* out;
    unsigned int ldq, ldk, ldv, ldo;
    unsigned int B, H, Hkv, head_dim, T_max;
    float epsilon, dk;
} cuda_attn_decode;
C_EXPORT int cuda_attn_decode_bf16(const cuda_attn_decode* a, void* stream, unsigned int flags);

/* ---- additions: a whole decode step as one kernel ------------------------------------------- */

/* No counterpart in the reference (it issues about 40 ops per layer, each followed by a device
 * synchronisation: cccc/MatrixOp.cpp:12-64, cccc-cuda/cuda_functions.cu:26-40).  A decode step at batch
 * 1 or 2 is a chain of ~150 dependent GEMVs of 4-100 MB; issued one by one, HBM idles for microseconds
 * around every launch.  A "decode program" records the chain once - linears with the op that produces
 * their input, attention - and runs it as ONE persistent kernel per step: one CTA per SM walks the list,
 * the weight stream of the next linear is already in flight through shared memory while the CTAs meet
 * at the end of the current one.  Results are those of the separate calls (the same arithmetic in the
 * same order wherever the schedules coincide).
 *   create        : w_type 4, 5 or 6 for every linear of the program; M_tokens 1 or 2.
 *   add_linears   : 1-3 linears that share their input (fields as cuda_gemm_wq_bf16_group).  `in` says
 *                   how the input is made: mode 0 = x itself; mode 1 = RMSNorm of x with norm_weight (NULL
 *                   = 1) and epsilon, as cuda_rms_norm_bf16; mode 2 = SwiGLU of x (gate) and x2 (up), as
 *                   cuda_swiglu_bf16.  x, x2: [M][ld] BF16, 16-byte aligned, ld % 8 == 0.  flags bit 2
 *                   (float32 output) and bit 3 (residual epilogue) as cuda_gemm_wq_bf16; bit 4: the two
 *                   linears are the gate and up projections of a gated MLP (equal N_out, a multiple of 16,
 *                   beta 0): only swiglu(bf16(gate), bf16(up)) is stored, as cuda_swiglu_bf16 would give
 *                   it, at linears[0].Y (linears[1].Y is not used).  K % 64 == 0 (FP4:
 *                   256), K <= 16384, weights 16-byte aligned with ldw % 16 == 0 (FP4: block scales, ldw %
 *                   256 == 0).
 *   add_attention : as cuda_attn_decode_bf16 with B = M_tokens, head_dim 128 and H = 4 Hkv.
 *   finalize      : uploads the program and allocates its scratch (the only step that allocates; make it
 *                   outside any stream capture).  Buffers named in the program must stay alive.
 *   launch        : one cooperative kernel on `stream`.  Launches of one program must not overlap, and each
 *                   carries its sequence number as an argument: issue them directly, do not replay one
 *                   from a captured graph.
 * Phases follow each other in the order added; each one sees everything the earlier ones wrote.
 * Every function returns 0, 1 (CUDA error) or -1 (an argument the program kernel does not take: use the
 * separate entry points for that step). */
typedef struct cuda_decode_program cuda_decode_program;
typedef struct cuda_decode_input
{
    int mode;
    const void* x;
    unsigned int ldx;
    const void* x2;
    unsigned int ldx2;
    const void* norm_weight;
    float epsilon;
} cuda_decode_input;
C_EXPORT int cuda_decode_program_create(cuda_decode_program** out, int w_type, unsigned int M_tokens);
C_EXPORT int cuda_decode_program_add_linears(cuda_decode_program* p, unsigned int count, const cuda_wq_linear* linears,
    const cuda_decode_input* in, unsigned int K, unsigned int flags);
C_EXPORT int cuda_decode_program_add_attention(cuda_decode_program* p, const cuda_attn_decode* a);
C_EXPORT int cuda_decode_program_finalize(cuda_decode_program* p);
C_EXPORT int cuda_decode_program_launch(cuda_decode_program* p, void* stream);
C_EXPORT unsigned int cuda_decode_program_phases(const cuda_decode_program* p);
C_EXPORT void cuda_decode_program_destroy(cuda_decode_program* p);

/* Tuning/diagnostic: returns which kernel cuda_gemm_wq_bf16 would pick for a shape
 * (0 = plain kernel, 1 = decode GEMV (M<=32), 2 = prefill tcgen05 GEMM, 3 = streaming tcgen05 kernel,
 * 4 = native-operand tcgen05 kernel) without launching. */
C_EXPORT int cuda_gemm_wq_bf16_plan(int w_type, const void* W, const void* blk_scales, const void* X,
    const void* Y, unsigned int N_out, unsigned int M_tokens, unsigned int K, unsigned int ldw, unsigned int ldx,
    unsigned int ldy_m, unsigned int ldy_n);

/* Number of kernels this library has launched in the calling process since load (all entry
 * points).  Used by the benchmark to report its launch count. */
C_EXPORT unsigned long long cuda_b200_launch_count(void);

/* Library identification: returns a static string "cccc-cuda-b200 <version> sm_100a". */
C_EXPORT const char* cuda_b200_version(void);
