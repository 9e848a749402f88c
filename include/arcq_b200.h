/*
 * arcq_b200 -- C ABI of the B200 (sm_100a) back end for the ARCQ packed inference path.
 *
 * Plain C entry points: raw device pointers, sizes, an opaque CUDA stream.  No
 * allocation happens inside unless an entry point says so; every call is
 * enqueued on the given stream and returns without synchronising.  Return value
 * 0 = success, negative = the call was rejected before any launch (see the
 * ARCQ_E_* codes; arcq_last_error_string() gives the reason for the calling
 * thread).
 *
 * Each declaration names the interface of the reference project it stands in
 * for.  Paths are inside the reference project; FQ = methods/fair_qat_framework,
 * EXT = FQ/fair_qat/arcq_infer_cuda.
 *
 * Data layout shared by all entry points (row-major, contiguous):
 *   packed codes   uint8 [rows, ceil(len*bits/8)]  code j of a row in bits [j*bits,(j+1)*bits) of
 *                  a little-endian bit stream (FQ/fair_qat/arcq_packed_py.py:8-78)
 *   per-group stats fp32 [rows, len/group_size]   mean, scale, sum of code values
 *   codebook       fp32 [2^bits] ascending;  thresholds fp32 [2^bits-1] = midpoints
 */
#ifndef ARCQ_B200_H_
#define ARCQ_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ARCQ_B200_VERSION 100

/* element types of x / y arguments */
#define ARCQ_DT_F32 0
#define ARCQ_DT_F16 1
#define ARCQ_DT_BF16 2

/* error codes */
#define ARCQ_OK 0
#define ARCQ_E_BAD_ARG (-1)      /* null pointer, bad dtype, bits not in {2,3,4}, ... */
#define ARCQ_E_BAD_SHAPE (-2)    /* K not a multiple of the group size, N not a multiple of 8, ... */
#define ARCQ_E_UNSUPPORTED (-3)  /* valid in the reference but not built here (group size != 64) */
#define ARCQ_E_ALIGN (-4)        /* pointer not aligned as the kernel needs */
#define ARCQ_E_CUDA (-5)         /* the CUDA runtime refused the launch */
#define ARCQ_E_TOO_LARGE (-6)    /* beyond a fixed capacity of the entry point */

/* Library version (ARCQ_B200_VERSION of the build).  No reference counterpart. */
int arcq_version(void);

/* Reason for the last non-zero return on the calling thread ("" if none).
 * Stands in for the TORCH_CHECK messages of EXT/arcq_activation_kernel.cu:194-202. */
const char* arcq_last_error_string(void);

/*
 * Device-side status word of the current device: 0, or a non-zero code left by a
 * kernel whose bounded wait ran out (the kernel then returned early instead of
 * hanging).  Reading it synchronises the device and clears the word.
 * No reference counterpart (the reference kernels have no waits).
 */
int arcq_device_status(void);

/*
 * Debugging aid: when given a device buffer of 128 int64 per CTA (148 x 128 is enough), the persistent
 * GEMM kernels launched afterwards write nanosecond timestamps of their pipeline milestones into it
 * (slot 0 kernel start, 1 loads issued, 2-7 weight sub-tiles rebuilt, 8+2b / 9+2b first MMA / commit of
 * tile batch b, 32+2t / 33+2t epilogue start / end of tile t).  NULL switches it off (the default).
 * No reference counterpart.
 */
int arcq_debug_trace(void* device_buffer);

/*
 * Debugging aid: tuning options of the launch code (slab widths, stage counts, kernel-variant switches,
 * the poll limits of the kernels' bounded waits).  Each option has a built-in default; an environment
 * variable of the same name, read once when the library is first used, overrides it, and so does this call
 * at any time (process-wide).  Names: ARCQ_WS_BN, ARCQ_WS_SA, ARCQ_WS_WS, ARCQ_WS_STATIONARY, ARCQ_WS_NBB,
 * ARCQ_WS_GRID, ARCQ_WS_TMA_STORE, ARCQ_WS_ROTATE, ARCQ_ACT_QUANT_V1, ARCQ_ACT_QUANT_V2, ARCQ_LN_PLAIN,
 * ARCQ_PAIR, ARCQ_PAIR_MIN_M, ARCQ_PAIR_BN, ARCQ_PAIR_SA, ARCQ_PAIR_KS, ARCQ_PAIR_NBB, ARCQ_PAIR_LUT,
 * ARCQ_PAIR_PAIRS, ARCQ_PAIR_STATIONARY, ARCQ_PAIR_WS, ARCQ_PDL, ARCQ_POLL_LIMIT,
 * ARCQ_SPIN_LIMIT.  Normal use sets none.
 * Unknown names return ARCQ_E_BAD_ARG.  No reference counterpart.
 */
int arcq_debug_set_option(const char* name, int value);
int arcq_debug_get_option(const char* name, int* value_out);

/*
 * Which kernel the last GEMM entry point called by this host thread launched (0: none yet).  The entry points
 * choose between kernel forms by shape and by what the device accepts (shared-memory ceiling, resident clusters)
 * and fall back silently to a slower form; tests use this to pin the form the benchmark shapes must get.
 */
enum {
  ARCQ_GEMM_ONE_CTA_PACKED = 1, ARCQ_GEMM_ONE_CTA_DENSE = 2, ARCQ_GEMM_PAIR_PACKED = 3, ARCQ_GEMM_PAIR_DENSE = 4,
  ARCQ_GEMM_PAIR_DENSE_PREFETCH = 5
};
int arcq_debug_last_gemm_kernel(void);

/*
 * Debugging aid: launches a one-warp kernel that waits, with the given poll limit (at most 65536), on a
 * barrier nothing ever arrives on.  The wait runs out, the kernel leaves the code 0x7E57 in the device status
 * word and returns: the path every bounded wait of the library takes instead of hanging.  Read the code with
 * arcq_device_status().  No reference counterpart.
 */
int arcq_debug_wait_timeout(unsigned poll_limit, void* stream);

/*
 * Activation quantizer: per row and per group of `group_size` consecutive
 * elements computes mean, scale = sqrt(mean(r^2)+1e-6), the code of every
 * element (number of thresholds below (x-mean)/scale) and the sum of code
 * values; writes packed codes and the three statistics.
 * Replaces quantize_activation_cuda, EXT/arcq_activation_kernel.cu:188-237
 * (kernel :24-77), and the quantising half of dequant_activation_triton,
 * FQ/fair_qat/arcq_packed_triton.py:181-215.  Arithmetic is fp32 with IEEE
 * division and square root and a fixed summation order, so codes equal the
 * reference CPU quantizer's (FQ/quant/dcarcq.py:531-556) bit for bit.
 *   x            [M,K] of x_dtype;  K % group_size == 0;  group_size must be 64
 *   packed_out   uint8 [M, K*bits/8]      (may be NULL when xhat_out is given)
 *   mu_out, sigma_out   fp32 [M, K/64]    (both or neither; required with packed_out, optional with xhat_out)
 *   codesum_out  fp32 [M, K/64] or NULL
 *   xhat_out     optional [M,K] of xhat_dtype: the reconstruction
 *                mean + scale*(cb[c] - codesum/64), the output of
 *                quantize_activation_dequant_cuda, EXT/arcq_activation_kernel.cu:286-326
 */
int arcq_act_quant(const void* x, int x_dtype, int64_t M, int64_t K,
                   const float* thresholds, const float* codebook, int bits, int group_size,
                   uint8_t* packed_out, float* mu_out, float* sigma_out, float* codesum_out,
                   void* xhat_out, int xhat_dtype, void* stream);

/*
 * GELU followed by the activation quantizer above, in one pass: the input is the pre-activation
 * (fp16 only), each element becomes 0.5*x*(1+erf(x/sqrt 2)) computed in fp32 and rounded to fp16 --
 * the tensor a separate GELU kernel would have written -- and is then quantised exactly as in
 * arcq_act_quant.  Fuses the F.gelu between fc1 and fc2 of the reference's MLP block (timm Mlp, called
 * from the model the reference builds in FQ/fair_qat/timm_quant_models.py:163-167) into step 2 of
 * ARCQPackedLinearOnTheFly.forward (FQ/fair_qat/arcq_packed_on_the_fly.py:143-145).  Same arguments.
 */
int arcq_gelu_act_quant(const void* x, int x_dtype, int64_t M, int64_t K,
                        const float* thresholds, const float* codebook, int bits, int group_size,
                        uint8_t* packed_out, float* mu_out, float* sigma_out, float* codesum_out,
                        void* xhat_out, int xhat_dtype, void* stream);

/*
 * Packed linear:  y[m,n] = bias[n] + sum_k A^[m,k] * W^[n,k]  with both operands
 * reconstructed from packed codes, A^ = mu_a + sigma_a*(cbA[ca] - Sa/gs) and
 * likewise W^, contracted on the tensor cores in fp16 with fp32 accumulation.
 * Replaces arcq_linear_forward_cuda, EXT/arcq_linear_kernel.cu:206-278 (kernel
 * :22-78), and steps 3-5 of ARCQPackedLinearOnTheFly.forward,
 * FQ/fair_qat/arcq_packed_on_the_fly.py:147-161 (Triton weight unpack + F.linear).
 * The reference passes product_table = outer(act_cb, w_cb); this entry point takes
 * the two codebooks instead.
 *   packed_x [M, K*bits/8], mu_a/sigma_a/codesum_a fp32 [M, K/gs]
 *   packed_w [N, K*bits/8], mu_w/sigma_w/codesum_w fp32 [N, K/gs]
 *   bias fp32 [N] or NULL;  y [M,N] of y_dtype (ARCQ_DT_F16 or ARCQ_DT_F32)
 *   group_size must be 64; N % 8 == 0.
 */
int arcq_packed_gemm(const uint8_t* packed_x, const float* mu_a, const float* sigma_a,
                     const float* codesum_a, const uint8_t* packed_w, const float* mu_w,
                     const float* sigma_w, const float* codesum_w, const float* act_codebook,
                     const float* w_codebook, const float* bias, int bits, int group_size,
                     int64_t M, int64_t N, int64_t K, void* y, int y_dtype, void* stream);

/*
 * Packed-weight linear on an already reconstructed fp16 activation:
 *   y[m,n] = bias[n] + sum_k xhat[m,k] * W^[n,k],   W^ rebuilt from packed codes inside the kernel.
 * This is the data flow of the reference's on-the-fly module: it replaces steps 3-5 of
 * ARCQPackedLinearOnTheFly.forward, FQ/fair_qat/arcq_packed_on_the_fly.py:147-161 -- the Triton
 * weight unpack (FQ/fair_qat/arcq_packed_triton.py:77-120), the fp16 bias cast and the cuBLAS
 * F.linear -- with one persistent kernel (TMA-staged operands, tcgen05 MMA, no fp16 weight in HBM).
 * xhat is what arcq_act_quant writes to xhat_out with xhat_dtype = ARCQ_DT_F16 (the reference's step 2,
 * dequant_activation_triton, FQ/fair_qat/arcq_packed_triton.py:181-215).
 *   xhat fp16 [M,K], 16-byte aligned;  packed_w [N, K*bits/8] with K*bits/8 a multiple of 16;
 *   N % 16 == 0; group_size must be 64; y [M,N] fp16 or fp32.
 * Shapes outside these limits return ARCQ_E_UNSUPPORTED (use arcq_packed_gemm).
 */
int arcq_packed_weight_gemm(const void* xhat, const uint8_t* packed_w, const float* mu_w,
                            const float* sigma_w, const float* codesum_w, const float* w_codebook,
                            const float* bias, int bits, int group_size, int64_t M, int64_t N, int64_t K,
                            void* y, int y_dtype, void* stream);

/*
 * The same linear with the weight given as an fp16 matrix: y[m,n] = bias[n] + sum_k xhat[m,k] * w16[n,k].
 * Replaces the cuBLAS F.linear of the reference's on-the-fly forward on its unpacked weight buffer,
 * FQ/fair_qat/arcq_packed_on_the_fly.py:160; w16 is what arcq_dequant (the reference's
 * unpack_weight_triton) writes.  Same persistent kernel as arcq_packed_weight_gemm with the weight
 * sub-tiles brought in by TMA instead of rebuilt; the faster of the two forms when few row tiles share a
 * rebuilt slab (large K with small N).  The caller owns w16 (a scratch buffer it may reuse between layers).
 *   xhat fp16 [M,K], w16 fp16 [N,K], both 16-byte aligned;  K % 64 == 0;  N % 16 == 0;  y [M,N] fp16 or fp32.
 */
int arcq_dense_weight_gemm(const void* xhat, const void* w16, const float* bias, int64_t M, int64_t N,
                           int64_t K, void* y, int y_dtype, void* stream);

/*
 * The packed linear (same arguments and result as arcq_packed_weight_gemm) for callers that cannot provide
 * device memory: the weight is unpacked into a scratch array that is part of the library image (one per
 * device, ARCQ_STATIC_WEIGHT_ELEMS fp16 values) and contracted from there, i.e. arcq_dequant followed by
 * arcq_dense_weight_gemm without a caller buffer.  No reference counterpart: the reference allocates its
 * `_weight_buffer` with torch.  Allocates and frees nothing.  N*K above the capacity returns
 * ARCQ_E_TOO_LARGE.  The first call on a device resolves the array's address (host-side set-up: make it
 * outside stream capture).  Calls on one device must not overlap in time -- they share the array.
 * Limits as arcq_dense_weight_gemm: K % 64 == 0, N % 16 == 0, group_size 64, 16-byte aligned xhat / y.
 */
#define ARCQ_STATIC_WEIGHT_ELEMS (768LL * 3072LL)
int arcq_packed_linear_static_scratch(const void* xhat, const uint8_t* packed_w, const float* mu_w,
                                      const float* sigma_w, const float* codesum_w, const float* w_codebook,
                                      const float* bias, int bits, int group_size, int64_t M, int64_t N,
                                      int64_t K, void* y, int y_dtype, void* stream);

/*
 * Residual add + LayerNorm over fp16 rows, the glue between the packed linears of a transformer block:
 *   s = fp16(x + y), written to sum_out (y and sum_out may both be NULL: plain LayerNorm of x);
 *   h = fp16((s - mean) * rsqrt(var + eps) * gamma + beta), statistics in fp32, biased variance.
 * Stands in for the `x = x + branch(...)` add and the following norm1 / norm2 / final norm of the timm
 * block the reference runs around its packed linears (model built in FQ/fair_qat/timm_quant_models.py:163-167);
 * the reference has no kernel of its own for it.  x, y, sum_out, h_out: fp16 [M,K]; gamma, beta: fp32 [K];
 * K % 8 == 0, K <= 2048; all pointers 16-byte aligned.
 */
int arcq_add_layernorm(const void* x, const void* y, const float* gamma, const float* beta, float eps,
                       int64_t M, int64_t K, void* sum_out, void* h_out, void* stream);

/*
 * arcq_add_layernorm followed by the activation quantizer of the packed linear that consumes the LayerNorm
 * output (timm Block.forward: norm1 -> attn.qkv, norm2 -> mlp.fc1), in one kernel:
 *   s = fp16(x + y) -> sum_out (y and sum_out may be NULL together);  h = fp16(LayerNorm(s));
 *   xhat = what arcq_act_quant(h, ..., xhat_dtype fp16) reconstructs.
 * h is not written unless h_out is given.  s, h and xhat are bit-identical to arcq_add_layernorm followed by
 * arcq_act_quant (the kernel shares their arithmetic), at every size.
 * fp16 rows of K = 192, 384 or 768 values (ARCQ_E_UNSUPPORTED otherwise); group_size 64.
 */
int arcq_add_layernorm_act_quant(const void* x, const void* y, const float* gamma, const float* beta, float eps,
                                 int64_t M, int64_t K, const float* thresholds, const float* codebook, int bits,
                                 int group_size, void* sum_out, void* h_out, void* xhat, void* stream);

/*
 * Multi-head self-attention on the output of the packed qkv linear, for short sequences (T <= 256) and heads of 64:
 * qkv [B*T, 3*H*64] fp16 (q | k | v), out [B*T, H*64] fp16 = softmax(q k^T / 8) v with the heads side by side --
 * what timm's Attention.forward computes between its qkv and proj linears with F.scaled_dot_product_attention.
 * Products on tensor cores with fp32 accumulation, softmax in fp32, probabilities rounded to fp16 for the second
 * product (as the library attention kernels do).
 *
 * arcq_attention_act_quant additionally runs the activation quantizer of the proj linear on the result (a head's 64
 * outputs are one quantizer group): xhat is, bit for bit, what arcq_act_quant reconstructs from arcq_attention's out.
 */
int arcq_attention(const void* qkv, int64_t B, int64_t T, int64_t H, int head_dim, void* out, void* stream);
int arcq_attention_act_quant(const void* qkv, int64_t B, int64_t T, int64_t H, int head_dim,
                             const float* thresholds, const float* codebook, int bits, int group_size,
                             void* xhat, void* stream);

/*
 * The data movement around a ViT's patch-embedding GEMM (timm PatchEmbed.forward and VisionTransformer._pos_embed),
 * fp16: arcq_patchify turns images [B, C, H, W] into the matrix [B*(H/patch)*(W/patch), C*patch*patch] whose
 * product with the flattened convolution weight is the patch x patch, stride-patch convolution (patch a multiple
 * of 8); arcq_assemble_tokens writes tokens [B, 1+T, D] = concat(class token [D], patches [B*T, D]) + position
 * embedding [1+T, D], the sum rounded to fp16.  Pure data movement and one fp16 addition: bit-identical to the
 * framework's reshape / permute / cat / add.
 */
int arcq_patchify(const void* images, int64_t B, int64_t C, int64_t H, int64_t W, int patch, void* rows, void* stream);
int arcq_assemble_tokens(const void* patches, const void* cls_token, const void* pos_embed, int64_t B, int64_t T,
                         int64_t D, void* tokens, void* stream);

/*
 * Unpack codes to one byte per code.  Replaces unpack_codes_u8_cuda,
 * EXT/arcq_pack_kernel.cu:136-157 (kernel :74-90); the int64 variant
 * unpack_codes_cuda (:113-134) is this plus a widening on the host side.
 */
int arcq_unpack_codes(const uint8_t* packed, int64_t rows, int64_t length, int bits,
                      uint8_t* codes_out, void* stream);

/*
 * Pack one-byte codes into the bit stream.  Replaces pack_codes_cuda,
 * EXT/arcq_pack_kernel.cu:92-111 (kernel :38-54), which takes int64 codes.
 */
int arcq_pack_codes(const uint8_t* codes, int64_t rows, int64_t length, int bits,
                    uint8_t* packed_out, void* stream);

/*
 * Reconstruct an fp16/fp32 matrix from packed codes and statistics:
 * out = mu + sigma*(cb[c] - codesum/gs).  Replaces unpack_weight_triton,
 * FQ/fair_qat/arcq_packed_triton.py:77-120 (kernel :11-74).  Feeds arcq_dense_weight_gemm (into a
 * scratch buffer, every forward, as the reference does); arcq_packed_weight_gemm never materialises
 * this matrix.
 */
int arcq_dequant(const uint8_t* packed, const float* mu, const float* sigma, const float* codesum,
                 const float* codebook, int bits, int group_size, int64_t rows, int64_t K,
                 void* out, int out_dtype, void* stream);

/*
 * The fp16 weight exactly as arcq_packed_weight_gemm rebuilds it on chip:
 * out = fp16(mu - sigma*codesum/64) + fp16(sigma) * fp16(cb[c]) in one half-precision fused multiply-add.
 * Written into a scratch matrix [rows, K] and read by arcq_dense_weight_gemm, the pair gives the same bits
 * as arcq_packed_weight_gemm.  This is the reference's own data flow (unpack_weight_triton into
 * `_weight_buffer`, then F.linear: FQ/fair_qat/arcq_packed_on_the_fly.py:147-160); the unpack of layer
 * L+1 can run on a second stream while layer L computes.  group_size 64 only.
 */
int arcq_unpack_weight_f16(const uint8_t* packed, const float* mu, const float* sigma, const float* codesum,
                           const float* codebook, int bits, int group_size, int64_t rows, int64_t K,
                           void* out, void* stream);

/*
 * arcq_dense_weight_gemm that also unpacks the weight of the layer that runs NEXT (arcq_unpack_weight_f16 of
 * next_packed ... into next_out) with two spare warps of every CTA while its own tiles run: the unpack then
 * needs no launch, no second stream and no events.  next_out must not be w16 (use two scratch matrices in
 * turn) and must not be read by any kernel launched after the one before the previous call of this function
 * on the stream -- in a model that alternates two scratch matrices layer by layer this holds by construction:
 * the matrix being overwritten was last read two GEMMs back.  Same results as the two separate calls.
 */
int arcq_dense_weight_gemm_prefetch(const void* xhat, const void* w16, const float* bias, int64_t M, int64_t N,
                                    int64_t K, void* y, int y_dtype, const uint8_t* next_packed,
                                    const float* next_mu, const float* next_sigma, const float* next_codesum,
                                    const float* next_codebook, int next_bits, int next_group_size,
                                    int64_t next_rows, int64_t next_K, void* next_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ARCQ_B200_H_ */
