/*
 * calibquant_b200 -- C ABI of the B200 (sm_100a) quantized-KV attention path.
 *
 * Every entry point takes raw DEVICE pointers, extents and a CUDA stream, returns
 * 0 (CQ_OK) or a negative CQ_ERR_* code, never throws, never synchronises and
 * never allocates: the caller owns every output and workspace buffer.  Work is
 * ordered only by the stream that is passed (`stream` is a cudaStream_t cast to
 * void*; NULL is the legacy default stream).  All entry points are re-entrant and may be called
 * from any host thread (the few per-device launch constants they cache are guarded).  The exceptions
 * to "never synchronises" say so: cq_decode_attn_host, cq_decode_attn_profile, the *_status calls.
 *
 * Each declaration names the reference (ActiveSky/calibquant) interface it
 * replaces, as file:line inside that project.
 *
 * Data formats
 *   "group format" (qjl/new_pack.py): groups of `group_size` consecutive elements of
 *   the last dimension; per group scale and minimum in the data dtype; 32/bits codes
 *   per int32 word, element i of a word in bits [i*bits, (i+1)*bits).
 *     K per channel : code [B,Hkv,D,T*bits/32]  scale,mn [B,Hkv,D,T/group]
 *     V per token   : code [B,Hkv,T,D*bits/32]  scale,mn [B,Hkv,T,D/group]
 *   dequantised value = scale*code + mn.
 */
#ifndef CALIBQUANT_B200_H_
#define CALIBQUANT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CQ_OK 0
#define CQ_ERR_BAD_ARG (-1)      /* null pointer, non-positive extent, bad enum            */
#define CQ_ERR_UNSUPPORTED (-2)  /* legal request outside what the kernels implement        */
#define CQ_ERR_LAUNCH (-3)       /* cudaGetLastError() reported a failure after the launch  */
#define CQ_ERR_WORKSPACE (-4)    /* workspace pointer null or smaller than required         */
#define CQ_ERR_TIMEOUT (-5)      /* a bounded device-side wait ran out (see status word)    */
#define CQ_ERR_TOO_LARGE (-6)    /* problem needs more scratch than a fixed-capacity variant has */

#define CQ_DTYPE_F16 0
#define CQ_DTYPE_BF16 1
#define CQ_DTYPE_F32 2             /* accepted only where an argument says so (QJL projections) */

/* Library version (major*10000 + minor*100 + patch). */
int cq_version(void);

/* Static, human-readable text for a status code. */
const char* cq_status_string(int status);

/*
 * Quantize-and-pack along the last dimension (group format).
 * Replaces qjl/new_pack.py:53-82 triton_quantize_and_pack_along_last_dim(data, group_size, bit)
 * together with its Triton kernels (:7-28, :32-50) and the torch elementwise chain (:69-72).
 *   data  : [rows, L] contiguous, dtype f16/bf16        (rows = B*nh*R of the 4-D input)
 *   code  : [rows, L*bits/32] int32      scale, mn : [rows, L/group_size] in the data dtype
 * Requirements: group_size == 32, bits in {1,2,4}, L % 32 == 0, data 16-byte aligned.
 * Arithmetic reproduces the reference's per-operation rounding, so code/scale/mn are
 * bit-identical to it.  A constant group (max == min) yields scale 0 and code 0.
 */
int cq_pack_last_dim(const void* data, int64_t rows, int64_t L, int group_size, int bits,
                     int dtype, int32_t* code, void* scale, void* mn, void* stream);

/*
 * Per-channel K quantize-and-pack with the transpose fused in.
 * Same result as cq_pack_last_dim applied to K transposed to [B,Hkv,D,T]
 * (qjl/new_pack.py:53-82 on `K.transpose(2,3).contiguous()`), without materialising it.
 *   k     : element (b,h,t,d) at k[b*stride_b + h*stride_h + t*stride_t + d], strides in
 *           elements, last dimension contiguous, D == 128, every row 16-byte aligned
 *   code  : [B,H,D,T*bits/32] int32      scale, mn : [B,H,D,T/32]
 * Requirements: T % 32 == 0, group_size == 32, bits in {1,2,4}.
 */
int cq_pack_k_per_channel(const void* k, int batch, int heads, int64_t T, int D,
                          int64_t stride_b, int64_t stride_h, int64_t stride_t,
                          int group_size, int bits, int dtype,
                          int32_t* code, void* scale, void* mn, void* stream);

/*
 * Per-token V quantize-and-pack read through strides: the result of cq_pack_last_dim on
 * `v.contiguous()` (patch_internvl.py:271 `prefill_V(value_states[:, :, s0:s1])`) without that copy,
 * so the visual span of V can be packed straight out of the wqkv output.
 *   v     : element (b,h,t,d) at v[b*stride_b + h*stride_h + t*stride_t + d], strides in elements,
 *           last dimension contiguous, D == 128, every row 16-byte aligned
 *   code  : [B,H,T,4*bits] int32      scale, mn : [B,H,T,4]
 */
int cq_pack_v_per_token(const void* v, int batch, int heads, int64_t T, int D,
                        int64_t stride_b, int64_t stride_h, int64_t stride_t,
                        int group_size, int bits, int dtype,
                        int32_t* code, void* scale, void* mn, void* stream);

/*
 * Quantized batched vector-matrix product with dequantize-on-the-fly (M == 1).
 * Replaces qjl/matmul.py:4-35 cuda_quantized_bmm_dynamic and the CUDA kernel
 * qjl/csrc/quantization.cu:67-169 (batchedQuantizedMultiplyAccumulate<T>).
 *   out[b,h,n] = sum_k fA[b,h,k] * (scales[b,hk,k,n/g]*code[b,hk,k,n] + zeros[b,hk,k,n/g]),
 *   hk = h / n_rep   (GQA: the packed operand is NOT expanded to the query heads; this
 *   replaces repeat_kv_quant, qjl/qjl_utils.py:6-11, and the reference's `mqa` flag).
 *   fA [B*Hq, K]   qB [B*Hkv, K, N*bits/32]   scales, zeros [B*Hkv, K, N/32]   out [B*Hq, N]
 * fp32 accumulation, result rounded to `dtype`.  Unlike the reference, bits == 1 works.
 * Requirements: group_size == 32, bits in {1,2,4}, N % 32 == 0, n_rep in [1,8].
 * `workspace` must hold cq_qbmm_workspace_bytes(...) bytes: a status word (see cq_workspace_status;
 * zero the workspace once after allocating it) followed by fp32 partial sums.
 */
size_t cq_qbmm_workspace_bytes(int batch, int n_q_heads, int64_t K, int64_t N);
int cq_qbmm(const void* fA, const int32_t* qB, const void* scales, const void* zeros,
            void* out, int batch, int n_q_heads, int n_kv_heads, int64_t K, int64_t N,
            int group_size, int bits, int dtype, void* workspace, size_t workspace_bytes,
            void* stream);

/*
 * cq_qbmm without any allocation by anybody: the fp32 partial sums go to a fixed array that
 * is part of the library image (no counterpart in the reference, whose extension allocates
 * its output through torch on every call).
 *
 * For callers that cannot allocate device memory once they are serving: a process that has
 * given all remaining HBM to its KV-cache pool (cudaMalloc would fail), or one that must not
 * stall its other streams (cudaMalloc synchronises the device).  Inputs and `out` are still the
 * caller's; the entry point itself calls no cudaMalloc/cudaFree or other allocating routine.
 *
 * Limits and rules
 *   - capacity: cq_qbmm_static_capacity_bytes() == 8 MiB, i.e. the call is accepted only while
 *     cq_qbmm_workspace_bytes(batch, n_q_heads, K, N) <= 8 MiB; a larger problem returns
 *     CQ_ERR_TOO_LARGE and launches nothing;
 *   - every GPU that loads the library holds those 8 MiB until the process exits;
 *   - the first call on each device looks the array's device address up (cudaGetSymbolAddress,
 *     with that device current) and caches it; make that first call before any stream capture;
 *   - all calls share the one array.  Apart from its status word (zero when the library is loaded,
 *     read with cq_qbmm_static_status) nothing in it has to start at zero: each call overwrites the
 *     part it later reads.  But two calls that overlap on the GPU -- different streams, or different
 *     host threads on different streams -- race on it.  Order them on one stream.
 * Same arguments, requirements and result as cq_qbmm otherwise.
 * cq_qbmm_static_status: CQ_OK, or CQ_ERR_TIMEOUT if a bounded device-side wait of an earlier
 * cq_qbmm_static call on the current device ran out (its output is then not valid).  Synchronises `stream`.
 */
size_t cq_qbmm_static_capacity_bytes(void);
int cq_qbmm_static_status(void* stream);
int cq_qbmm_static(const void* fA, const int32_t* qB, const void* scales, const void* zeros,
                   void* out, int batch, int n_q_heads, int n_kv_heads, int64_t K, int64_t N,
                   int group_size, int bits, int dtype, void* stream);

/*
 * One decode step of attention over [system | visual (quantized) | text] keys.
 * Replaces the q_len == 1 branch of the patched attention forward:
 * patch_internvl.py:556-592 (scores, softmax, packed attn.V, fp16 side segments), with the
 * logit calibration of patch_internvl.py:376-385 applied to the visual logits when
 * `calibrate` != 0, and replaces per call: repeat_kv / repeat_kv_quant copies
 * (patch_internvl.py:97-106, 581-583), the transposes of qjl/matmul.py:16-22 and both
 * cuda_quantized_bmm_dynamic launches.
 */
typedef struct cq_decode_args {
  /* extents */
  int32_t batch, n_q_heads, n_kv_heads, head_dim;   /* head_dim must be 128            */
  int32_t t_vis;        /* quantized (visual) tokens, multiple of 32, may be 0          */
  int32_t t_fp;         /* full-precision tokens (system + text), may be 0              */
  int32_t t_sys;        /* how many of the t_fp tokens precede the visual span; only    */
                        /* used to index `mask` in the original key order               */
  int32_t bits, group_size, dtype;
  int32_t calibrate;    /* 1: remap visual logits (patch_internvl.py:376-385)           */
  int32_t reserved;     /* must be 0                                                    */
  /* operands (device pointers) */
  const void* q;                 /* [B,Hq,D]                                            */
  const int32_t* k_code;         /* [B,Hkv,D,t_vis*bits/32]                             */
  const void* k_scale;           /* [B,Hkv,D,t_vis/32]                                  */
  const void* k_mn;
  const int32_t* v_code;         /* [B,Hkv,t_vis,D*bits/32]                             */
  const void* v_scale;           /* [B,Hkv,t_vis,D/32]                                  */
  const void* v_mn;
  const void* k_fp;              /* token (b,h,t,:) at k_fp + b*fp_stride_b + h*fp_stride_h + t*D */
  const void* v_fp;
  int64_t fp_stride_b, fp_stride_h;  /* in elements */
  const void* mask;              /* optional additive mask [B, t_fp + t_vis] in `dtype`, */
  int64_t mask_stride_b;         /* key order [sys | visual | text]; NULL = none         */
  void* out;                     /* [B,Hq,D] in `dtype`                                 */
  const int32_t* t_fp_dev;       /* optional device counter of live fp tokens: when set, t_fp is  */
                                 /* the capacity of k_fp/v_fp and min(*t_fp_dev, t_fp) tokens are  */
                                 /* attended; lets one captured CUDA graph serve every decode step */
                                 /* (tensor-core path only, otherwise CQ_ERR_UNSUPPORTED)          */
} cq_decode_args;

/*
 * Stream semantics: everything the call enqueues is ordered after the work already in `stream` and before
 * anything enqueued in it afterwards.  With full-precision tokens present, the tensor-core path runs their launch
 * on an internal side stream (one per host thread and device, created on first use) between two events recorded
 * in `stream` and in the side stream; under stream capture this records two parallel branches that join before the
 * last launch.  Make the first call on a device outside any capture.  The launches carry the
 * programmatic-stream-serialization attribute (they overlap their heads with the previous launch's tail).
 */
size_t cq_decode_attn_workspace_bytes(const cq_decode_args* args);
int cq_decode_attn(const cq_decode_args* args, void* workspace, size_t workspace_bytes,
                   void* stream);

/*
 * Per-launch device times of one step, for profiling (no reference counterpart: the reference has no
 * timers).  Runs the step exactly as cq_decode_attn does, with CUDA events recorded on `stream` between
 * its launches, waits for the last one and fills launch_ms[4] = {scores, attn.V, attn.V of the
 * full-precision tokens, combine} in milliseconds.  Only for requests the tensor-core kernels take
 * (t_vis > 0, 16-byte aligned operands); CQ_ERR_UNSUPPORTED otherwise.  Synchronises.
 */
int cq_decode_attn_profile(const cq_decode_args* args, void* workspace, size_t workspace_bytes,
                           void* stream, float* launch_ms);

/*
 * Sticky device status of a workspace that cq_decode_attn or cq_qbmm was given (no reference
 * counterpart: the reference checks no CUDA errors).  Every device-side wait of the kernels is bounded;
 * one that runs out stores CQ_ERR_TIMEOUT in the first word of the workspace (the caller zeroes a
 * workspace once, after allocating it) and the kernel returns early.  Returns CQ_OK or CQ_ERR_TIMEOUT.
 * Synchronises `stream`.  cq_decode_attn_host checks the word itself on every call.
 */
int cq_workspace_status(const void* workspace, void* stream);

/*
 * The same step for a caller whose query and result live in HOST memory (the serving loop of
 * patch_internvl.py:556-592 samples the next token on the host): `args->q` and `args->out` are
 * ignored, q_host [B,Hq,D] is copied into the workspace (by a small kernel that reads the buffer
 * when it is page-locked, so that the score launch starts under the copy; by a copy-engine transfer
 * otherwise), the last launch stores the result
 * straight into out_host when that buffer is page-locked (cudaHostAlloc / cudaHostRegister; a
 * staged copy otherwise), and the call returns after the stream has drained, i.e. with out_host
 * valid.
 * A bounded device-side wait that runs out during such a step makes the call return CQ_ERR_TIMEOUT (the
 * kernels report it in a page-locked word of the library, one per device, which the call reads after
 * the stream has drained).  The word is sticky: every later call on that device returns CQ_ERR_TIMEOUT
 * until the caller clears it.  cq_host_status_word returns its host address for the current device (the
 * first call on a device allocates it), to be read, or cleared by storing 0, between calls.
 */
int* cq_host_status_word(void);
size_t cq_decode_attn_host_workspace_bytes(const cq_decode_args* args);
int cq_decode_attn_host(const cq_decode_args* args, const void* q_host, void* out_host,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dense causal prefill attention over unquantized K/V with GQA head sharing.
 * Replaces the flash_attn calls of the reference prefill: patch_internvl.py:464-468
 * (self._flash_attention_forward in 1024-query chunks against the growing prefix) and :606-609
 * (transformers' _flash_attention_forward); chunking is not needed, the kernel is causal over
 * the whole sequence and needs no workspace.
 *   q, out : element (b,t,h,d) at base + b*strides[0] + t*strides[1] + h*strides[2] + d
 *   k, v   : same addressing with n_kv_heads heads; strides in elements, multiples of 8
 *   o = softmax(q k^T / sqrt(head_dim) + causal mask) v, fp32 accumulation, head_dim == 128.
 */
int cq_prefill_attn(const void* q, const void* k, const void* v, void* out, int batch, int t_len,
                    int n_q_heads, int n_kv_heads, int head_dim, const int64_t* q_strides,
                    const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                    int dtype, void* stream);

/*
 * ---- CalibQuant uint8 format (whole visual span = one quantization group per channel) -----------
 *
 * cq_calib_minmax: scale and zero point of calibquant.py:24-42 `quant(x, bits, per_channel=True,
 * scale=clip)` (the min/max/scale/zero_point lines :27-33).
 *   x : element (b,t,h,d) at x + b*strides[0] + t*strides[1] + h*strides[2] + d   (head_dim 128)
 *   scale, zero_point : [B,H,D] in the data dtype (the reference's [B,1,H,D])
 */
int cq_calib_minmax(const void* x, int batch, int t_len, int heads, int head_dim, const int64_t* strides,
                    int bits, float clip, int dtype, void* scale, void* zero_point, void* stream);

/*
 * cq_calib_quantize: the quantize / dequantize lines of calibquant.py:35-41 and, fused, the byte
 * packing of calibquant.py:114-137 `encode` (most significant field first).
 *   xq_out  (optional) : [B,T,H,D] contiguous, the codes as numbers of the data dtype
 *                        (dequantize == 0, the reference's post_scale=True) or scale*(code - zp)
 *   enc_out (optional) : uint8 [B,H,T,D*bits/8]
 */
int cq_calib_quantize(const void* x, int batch, int t_len, int heads, int head_dim, const int64_t* strides,
                      int bits, int dtype, const void* scale, const void* zero_point, int dequantize,
                      void* xq_out, uint8_t* enc_out, void* stream);

/* calibquant.py:114-137 `encode` on int64 codes (any leading shape, last dim a multiple of 8/bits). */
int cq_calib_encode_i64(const int64_t* codes, int64_t n_codes, int bits, uint8_t* out, void* stream);

/*
 * cq_lut_scores replaces calibquant.py:54-111 `fused_kernel` (Triton LUT vec-mat, transposed):
 *   out[b,h,t] = sum_d weights[b,h,d] * lut[code[b,he,t,d]],  he = h / (n_q_heads/n_enc_heads)
 *   weights [B,Hq,D]; enc uint8 [B,Henc,T,D*bits/8] (Henc = Hq as the reference passes it, or the KV
 *   head count); lut 2^bits values in the data dtype; out [B,Hq,T] always fp16 (calibquant.py:109).
 * cq_lut_out replaces calibquant.py:192-276 `fused_kernel_wv`:
 *   out[b,h,d] = sum_t weights[b,h,t] * lut[code[b,he,t,d]],  weights [B,Hq,T], out [B,Hq,D] fp16;
 *   workspace: cq_lut_out_workspace_bytes(...) bytes of fp32 partial sums.
 */
int cq_lut_scores(const void* lut, const void* weights, const uint8_t* enc, void* out, int batch,
                  int n_q_heads, int n_enc_heads, int t_len, int head_dim, int bits, int dtype, void* stream);
size_t cq_lut_out_workspace_bytes(int batch, int n_q_heads, int t_len);
int cq_lut_out(const void* lut, const void* weights, const uint8_t* enc, void* out, int batch, int n_q_heads,
               int n_enc_heads, int t_len, int head_dim, int bits, int dtype, void* workspace,
               size_t workspace_bytes, void* stream);

/*
 * cq_u8_decode_attn: one decode step of attention on this format, four launches (no reference entry point
 * of its own: it replaces the eager sequence patch_internvl.py:356-436 -- scores of the system and text
 * tokens, `fused_kernel(q * scale_key) / sqrt(D) - bias_k`, logit calibration :376-385, fp32 softmax,
 * `fused_kernel_wv(att) * scale_value - scale_value*zero_point_value*sum(att)`, the full-precision
 * products and the final cast to bfloat16 :436).
 *   q [B,Hq,D]; enc_k, enc_v uint8 [B,Hkv,t_vis,D*bits/8] (16-byte aligned);
 *   scale_*, zero_point_* [B,Hs,D] in the data dtype with Hs = n_scale_heads = Hq (as the reference keeps
 *   them, repeated per query head) or Hkv;  k_fp/v_fp as in cq_decode_args, tokens [sys | text];
 *   out [B,Hq,D] bfloat16 whatever the data dtype.  (t_vis + t_fp) * 4 bytes must fit 200 KB of shared
 *   memory (51 200 keys); larger requests return CQ_ERR_UNSUPPORTED.
 */
typedef struct cq_u8_decode_args {
  int32_t batch, n_q_heads, n_kv_heads, head_dim;   /* head_dim must be 128 */
  int32_t t_vis, t_fp, t_sys;                       /* t_sys of the t_fp tokens precede the visual span */
  int32_t bits, dtype;
  int32_t calibrate;                                /* 1: remap the visual logits */
  int32_t n_scale_heads;
  int32_t reserved;                                 /* must be 0 */
  const void* q;
  const uint8_t* enc_k;
  const uint8_t* enc_v;
  const void* scale_key;
  const void* zero_point_key;
  const void* scale_value;
  const void* zero_point_value;
  const void* k_fp;
  const void* v_fp;
  int64_t fp_stride_b, fp_stride_h;                 /* in elements */
  const void* mask;                                 /* optional additive mask [B, t_fp + t_vis] in `dtype`,   */
  int64_t mask_stride_b;                            /* key order [sys | visual | text]; NULL = none           */
  void* out;
  const int32_t* t_fp_dev;                          /* optional device counter of live fp tokens, as in       */
                                                    /* cq_decode_args: t_fp is then the capacity of k_fp/v_fp */
} cq_u8_decode_args;
size_t cq_u8_decode_attn_workspace_bytes(const cq_u8_decode_args* args);
int cq_u8_decode_attn(const cq_u8_decode_args* args, void* workspace, size_t workspace_bytes, void* stream);

/*
 * ---- decode-step glue around the attention call ---------------------------------------------------
 *
 * cq_rope_split_append replaces, for one decode token per batch row, the QKV split, rotary embedding
 * and cache append of the patched forward (patch_internvl.py:214-260 split + `apply_rotary_pos_emb`,
 * :265-266 `torch.cat` of the new key/value onto the fp cache) with one launch.
 *   qkv          : wqkv output, row b at qkv + b*qkv_stride_b, laid out [n_kv_heads][n_rep q heads, k, v][128]
 *   cos/sin      : rotary tables [rope_len,128] in the data dtype (what `rotary_emb(x, seq_len)` returns)
 *   position_ids : int64 [batch] on the device; clamped to [0, rope_len)
 *   q_out        : [batch, n_kv_heads*n_rep, 128] rotated queries
 *   k_cache/v_cache : fp caches, token t of (b,h) at base + b*cache_stride_b + h*cache_stride_h + t*128;
 *                  the rotated key and the value are written at token index `append_index`, or, when
 *                  t_fp_dev is set, at *t_fp_dev - 1 (the device-side live count already includes the
 *                  new token, so the same pointer can be handed to cq_decode_attn afterwards).  An
 *                  index outside [0, capacity) writes nothing.
 *   Rounding as torch: x*cos rounded to the data dtype, then + rotate_half(x)*sin rounded once more.
 *
 * cq_add_rmsnorm and cq_swiglu have no counterpart in the reference repository: they fuse the
 * elementwise blocks of the InternLM2 decoder layer that the reference leaves to the third-party
 * model code (residual add + RMSNorm; silu(w1 x) * w3 x), so that a decode step is a dozen launches
 * per layer.
 *   cq_add_rmsnorm: if delta != NULL, residual += delta (rounded to the data dtype, in place); then,
 *     if out != NULL, out = weight * (r_fp32 * rsqrt(mean(r_fp32^2) + eps)).to(dtype) per row of
 *     `hidden` elements (hidden % 8 == 0, hidden <= 16384; rows contiguous).
 *   cq_swiglu: out = (silu(gate).to(dtype) * up).to(dtype) over n elements (n % 8 == 0).
 */
int cq_rope_split_append(const void* qkv, int64_t qkv_stride_b, const void* cos_table, const void* sin_table,
                         int rope_len, const int64_t* position_ids, int batch, int n_kv_heads, int n_rep,
                         int head_dim, void* q_out, void* k_cache, void* v_cache, int64_t cache_stride_b,
                         int64_t cache_stride_h, int capacity, int append_index, const int32_t* t_fp_dev,
                         int dtype, void* stream);
/*
 * cq_prefill_rope_split is the same step for a whole prompt (patch_internvl.py:214-260 on q_len tokens,
 * and the `text_k`/`text_v` concatenations of :281-284): one pass over the wqkv output
 *   qkv      : token (b,t) at qkv + b*qkv_stride_b + t*qkv_stride_t, laid out as above
 *   position_ids : int64 [batch, t_len] on the device, or NULL for 0..t_len-1
 *   q_out    : [batch, t_len, n_kv_heads*n_rep, 128] rotated queries
 *   k_out    : [batch, t_len, n_kv_heads, 128] rotated keys (what the prefill attention and
 *              cq_pack_k_per_channel read; values are read in place from qkv)
 *   k_cache/v_cache : optional fp caches laid out as above; tokens before vis_start go to rows
 *              0..vis_start-1, tokens from vis_start+vis_len on follow them (the visual span
 *              [vis_start, vis_start+vis_len) is left to the pack kernels).  NULL: not written.
 */
int cq_prefill_rope_split(const void* qkv, int64_t qkv_stride_b, int64_t qkv_stride_t, const void* cos_table,
                          const void* sin_table, int rope_len, const int64_t* position_ids, int batch, int t_len,
                          int n_kv_heads, int n_rep, int head_dim, void* q_out, void* k_out, void* k_cache,
                          void* v_cache, int64_t cache_stride_b, int64_t cache_stride_h, int capacity,
                          int vis_start, int vis_len, int dtype, void* stream);
int cq_add_rmsnorm(const void* delta, void* residual, const void* weight, void* out, int64_t rows, int hidden,
                   float eps, int dtype, void* stream);
int cq_swiglu(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream);
/* cq_swiglu on one matrix gate_up [rows, 2n] whose first n columns are the gate and last n the up projection
 * (one GEMM against the stacked w1 / w3 weights): out [rows, n].  n % 8 == 0. */
int cq_swiglu_packed(const void* gate_up, void* out, int64_t rows, int64_t n, int dtype, void* stream);

/*
 * ---- tensor-parallel decode step: one-shot all-reduce / all-gather over peer memory -----------------------
 *
 * No counterpart in the reference, which runs on one device (infer.py:200 `device_map='auto'` only).  With the
 * model sharded by KV head over `world` GPUs of a node (one process per GPU), every sharded block of a decode
 * step ends in a partial [batch, hidden] sum per rank; these entry points exchange such rows through buffers
 * the peers can write directly (CUDA IPC over NVLink), in two halves that ride on the step's own launches:
 *   cq_comm_push               copies `bytes` of this rank's rows into slot `rank` of every rank's buffer
 *                              (plain peer stores) and publishes the collective's sequence number there;
 *   cq_comm_reduce_add_rmsnorm waits until all `world` slots of this rank's buffer carry that number, then
 *                              residual += sum of the slots (fp32 sum, one rounding) and, if out != NULL,
 *                              out = RMSNorm(residual) * weight exactly as cq_add_rmsnorm;
 *   cq_comm_gather             the same wait, then out[q] = slot q for every rank q (an all-gather);
 *   cq_comm_allreduce_add_rmsnorm  push and reduce in ONE launch, row by row (rows <= 64): the CTA of a row
 *                              stores the row of `src` into the peers' buffers, publishes it, waits for the
 *                              peers' copies of that row and finishes as cq_comm_reduce_add_rmsnorm does.
 * Every collective is one push on every rank followed by one reduce or gather on every rank, in the same order
 * on all ranks.  The sequence number lives in the buffer and advances on the device, so a captured CUDA graph
 * replays the step.  Waits are bounded (two seconds): a timeout stores CQ_ERR_TIMEOUT in the buffer's status
 * word (cq_comm_status, synchronises) and the kernel leaves its outputs untouched.
 *
 *   cq_comm_buffer_bytes(world, slot_bytes)  size of one rank's buffer for rows of at most slot_bytes
 *   cq_comm_alloc   allocates and clears a buffer on the current device (set-up time: cudaMalloc) and fills
 *                   the 64-byte IPC handle that lets the other processes map it
 *   cq_comm_open    maps a peer's buffer from its handle; cq_comm_close unmaps it; cq_comm_free frees one's own
 *   peer_buffers    host array of `world` device pointers, entry q = rank q's buffer as seen from this process
 * world <= 8.  slot_bytes must be the same in every call on a buffer.
 */
size_t cq_comm_buffer_bytes(int world, size_t slot_bytes);
int cq_comm_alloc(size_t bytes, void** buffer, void* ipc_handle);
int cq_comm_open(const void* ipc_handle, void** buffer);
int cq_comm_close(void* buffer);
int cq_comm_free(void* buffer);
int cq_comm_status(const void* buffer, void* stream);
int cq_comm_push(const void* src, size_t bytes, void* const* peer_buffers, int rank, int world, size_t slot_bytes,
                 void* stream);
int cq_comm_reduce_add_rmsnorm(void* buffer, int world, size_t slot_bytes, void* residual, const void* weight,
                               void* out, int64_t rows, int hidden, float eps, int dtype, void* stream);
int cq_comm_gather(void* buffer, int world, size_t slot_bytes, void* out, size_t bytes, void* stream);
int cq_comm_allreduce_add_rmsnorm(const void* src, void* const* peer_buffers, int rank, int world, size_t slot_bytes,
                                  void* residual, const void* weight, void* out, int64_t rows, int hidden,
                                  float eps, int dtype, void* stream);

/*
 * ---- QJL sign-sketch key quantizer (the reference's `qjl` baseline method) ---------------------------
 *
 * cq_qjl_quant replaces qjl/qjl_kernel.py:8-28 `qjl_quant` -> `quantize_with_outliers_kernel`
 * (qjl/csrc/qjl_quant_kernel.cu:53-168).
 *   keys            : [n_groups_total][group_size][128] in `dtype` (the reference's [B,H,n,G,D])
 *   outlier_indices : uint8 [n_groups_total][outlier_count], channels treated as outliers in that group
 *   proj            : [sketch_dim][128] (QJLSketch.proj_dir_quant), `proj_dtype` = CQ_DTYPE_F32 or `dtype`
 *   key_quant         uint8 [n_groups_total][group_size][sketch_dim/8]: bit p%8 of byte p/8 is
 *                     [ sum_{d not outlier} proj[p][d]*k[d] > 0 ], fp32 sums in channel order
 *   key_outlier_quant uint8 [...][outlier_sketch_dim/8]: same over the outlier channels, p < outlier_sketch_dim
 *   outlier_norms     [n_groups_total][group_size] in `dtype`: 2-norm of the outlier channels
 *   sketch_dim <= 256, sketch_dim and outlier_sketch_dim multiples of 32.
 *
 * cq_qjl_gqa_score replaces qjl/qjl_kernel.py:52-72 `qjl_gqa_score` -> `calc_gqa_score_kernel`
 * (qjl/csrc/qjl_gqa_score_kernel.cu:40-180), for any n_rep <= 8 (the reference's shared arrays hold 4):
 *   score[b,h,t] = sqrt(pi/2)/sketch_dim * |k_in| * sum_p sgn_p (qS - q_out S)_p
 *                + sqrt(pi/2)/outlier_sketch_dim * |k_out| * sum_{p<o} sgn'_p (q_out S)_p
 *   key_norm / key_outlier_norm [B,Hkv,n,G] in `dtype`; |k_in| = sqrt(max(|k|^2 - |k_out|^2, 0)) (the
 *   reference takes the square root of the unclamped difference); query_sketch fp32 [B,Hq,sketch_dim] =
 *   q @ proj_score; query [B,Hq,128]; proj_score [128][sketch_dim] (QJLSketch.proj_dir_score);
 *   scores fp32 [B,Hq,n*G].
 */
int cq_qjl_quant(const void* keys, const uint8_t* outlier_indices, const void* proj, int proj_dtype,
                 int64_t n_groups_total, int group_size, int head_dim, int sketch_dim, int outlier_sketch_dim,
                 int outlier_count, int dtype, uint8_t* key_quant, uint8_t* key_outlier_quant,
                 void* outlier_norms, void* stream);
int cq_qjl_gqa_score(const uint8_t* key_quant, const uint8_t* key_outlier_quant, const void* key_norm,
                     const void* key_outlier_norm, const uint8_t* outlier_indices, const float* query_sketch,
                     const void* query, const void* proj_score, int proj_dtype, int batch, int n_kv_heads,
                     int n_rep, int n_groups, int group_size, int head_dim, int sketch_dim,
                     int outlier_sketch_dim, int outlier_count, int dtype, float* scores, void* stream);

/*
 * Sticky device status of the prefill kernel (no reference counterpart: the reference checks no
 * CUDA errors).  0, or CQ_ERR_TIMEOUT if one of its bounded barrier waits ever ran out on the
 * current device.  Synchronises the device.
 */
int cq_prefill_status(void);

#ifdef __cplusplus
}
#endif
#endif /* CALIBQUANT_B200_H_ */
