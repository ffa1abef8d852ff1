/*
 * df8.h — C-ABI of the B200 (sm_100a) fp8 fully-connected + attention kernel library.
 *
 * This is the boundary the C++ `dnn::` layer classes (dnn/core, dnn/layers, dnn/models) sit on.
 * The upstream project has no FFI of its own: its layers launch their kernels directly from the
 * class bodies.  Each entry point below therefore names the upstream launch site (or the
 * host-side helper) it replaces, by that project's file:line.
 *
 * Conventions
 *  - every function returns a df8_status (0 = ok); the text of the last failure on the calling
 *    thread is returned by df8_last_error();
 *  - all pointers are DEVICE pointers unless the parameter name ends in `_h`;
 *  - every launch is enqueued on the `stream` argument; nothing synchronises the device and
 *    nothing allocates device memory, except the calls documented as doing so
 *    (df8_streamer_create, df8_comm_*);
 *  - scales are passed as device pointers so that a chain of kernels runs without a host
 *    round trip:  `scale` is a pair of floats {q, dq} with q = FP8_MAX/amax (1 if amax==0)
 *    and dq = amax/FP8_MAX (1 if amax==0);  FP8_MAX = 448 for e4m3 and 57344 for e5m2;
 *  - fp8 values travel as raw codes in uint8_t buffers (the upstream tensor type for them is
 *    dnn::tensor<uint8_t>, dnn/core/tensor.cuh:149).
 */
#ifndef DF8_H_
#define DF8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int df8_status;
enum {
    DF8_OK = 0,
    DF8_ERR_INVALID = 1,     /* bad argument (null pointer, bad size, bad enum, misalignment) */
    DF8_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed */
    DF8_ERR_UNSUPPORTED = 3, /* shape outside what the kernels cover */
    DF8_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up (see df8_status_word_read) */
    DF8_ERR_COMM = 5         /* an NCCL call failed */
};

/* fp8 element kinds.  Upstream names only the storage types (__nv_fp8x4_e4m3 / __nv_fp8x4_e5m2,
 * dnn/core/tensor.cu:489-498); conversion semantics are those of the CUDA toolkit's cuda_fp8.h:
 * round-to-nearest-even, saturate to the largest finite value. */
typedef enum { DF8_E4M3 = 0, DF8_E5M2 = 1 } df8_kind;

/* stream handle: a cudaStream_t passed as an opaque pointer (NULL = legacy default stream,
 * which is what dnn::Cuda::stream() returns when no stream is set, dnn/core/cuda.cu:85-87). */
typedef void* df8_stream;

/* ---- library ---------------------------------------------------------------------------- */

/* Text of the last error recorded on the calling thread ("" if none). Never NULL. */
const char* df8_last_error(void);

/* Library version string. */
const char* df8_version(void);

/* Every entry point that returns max|out| through an `amax_out` / `out_amax` pointer first clears that float on
 * the stream (one memset node per call).  A caller that keeps its amax slots in one array and clears the whole
 * array once per forward pass turns the per-call clearing off for the calling thread with enabled = 0; it then
 * guarantees that a slot is zero when the kernels of the call that fills it run.  Returns the previous setting.
 * No upstream counterpart: the reference has no quantiser (see below). */
int df8_set_amax_preclear(int enabled);

/* ---- per-tensor amax / quantise / dequantise ---------------------------------------------
 * No upstream kernel exists for these (the fp8 tensor instantiations at dnn/core/tensor.cu:489-498
 * are never compiled); they implement the per-tensor quantiser:
 *     amax = max_i |x_i|;  q = FP8_MAX / amax;  code_i = cvt_rn_satfinite(x_i * q);
 *     y_i = float(code_i) * (amax / FP8_MAX).
 */

/* amax_out[0] = max_i |x[i]| over n fp32 values (NaNs are ignored; n == 0 gives 0).
 * The kernel clears amax_out itself. */
df8_status df8_amax_f32(const float* x, size_t n, float* amax_out, df8_stream stream);

/* codes_out[i] = fp8(x[i] * q) with q derived from amax_in[0]; writes scale_out = {q, dq}. */
df8_status df8_quantize_f32(const float* x, size_t n, df8_kind kind, const float* amax_in,
                            uint8_t* codes_out, float* scale_out, df8_stream stream);

/* y_out[i] = float(codes[i]) * scale[1]. */
df8_status df8_dequantize_f32(const uint8_t* codes, size_t n, df8_kind kind, const float* scale,
                              float* y_out, df8_stream stream);

/* ---- fp8 GEMM (fully connected) ----------------------------------------------------------
 * Replaces the launch of fully_connected_forward_kernel (dnn/layers/fully_connected_layer.cu:15-41,
 * launched at :199-208):  Y[M,N] = X[M,K] . W[N,K]^T + b,  W stored [out,in] row-major.
 * Here X and W arrive as fp8 codes with their per-tensor scales and the contraction runs on the
 * tcgen05 tensor cores with fp32 accumulation:
 *     out[m,n] = epi( acc[m,n] * (scale_a[1] * scale_w[1]) + bias[n] )
 * epi, selected by `flags`:
 *     DF8_EPI_GELU      x*0.5*(1+tanh(0.7978845608*(x+0.044715x^3)))   (dnn/layers/activation_layer.cu:9-20)
 *     DF8_EPI_RESIDUAL  + residual[m,n]      (replaces the separate add kernel, dnn/core/tensor.cu:383-415)
 *     DF8_EPI_AMAX      also reduce max|out| into out_amax[0] (cleared by the call), so the next
 *                       quantise needs no separate amax pass
 * K must be a multiple of 16; A and W must be 16-byte aligned.  bias may be NULL. */
enum { DF8_EPI_GELU = 1, DF8_EPI_RESIDUAL = 2, DF8_EPI_AMAX = 4 };

df8_status df8_gemm_fp8_tn(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                           const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                           const float* bias, const float* residual, int M, int N, int K, int flags,
                           float* out, float* out_amax, df8_stream stream);

/* The same call with two more degrees of freedom (df8_gemm_fp8_tn is this with a_slabs = 1 and ldc = N):
 *   ldc      row pitch, in floats, of `out` (and of `residual`), ldc >= N.  A pitch that is a multiple of 4 floats
 *            lets rows of any N start on 16-byte boundaries: the epilogue then writes 128 bits at a time, and
 *            without a residual it leaves through TMA stores.  Columns N .. ldc-1 of a row belong to the caller;
 *            up to three of them (N rounded up to a multiple of 4) may be overwritten with unspecified values.
 *            A vocabulary of 50257 is the case: dense rows are not 16-byte aligned and cost one 4-byte store per
 *            element (upstream's kernel writes `output[row * out + col]`, fully_connected_layer.cu:39).
 *   a_slabs  A's K columns are stored as a_slabs row-major [M, K / a_slabs] matrices, M * K / a_slabs bytes apart
 *            — the layout an all-gather of per-rank [M, K / world] column slices leaves — and are read in place
 *            (K / a_slabs must be a multiple of 128 when a_slabs > 1). */
df8_status df8_gemm_fp8_tn_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                              const uint8_t* w_codes, df8_kind kind_w, const float* scale_w, const float* bias,
                              const float* residual, int M, int N, int K, int flags, float* out, int ldc,
                              float* out_amax, df8_stream stream);

/* Same product with per-tensor-quantised fp8 OUTPUT and no fp32 intermediate in memory:
 *     out_codes[m,n] = fp8_out_kind( epi(acc*dq_a*dq_w + bias[n]) * q ),  q = FP8_MAX / max|epi(...)|
 * The kernel runs twice — a first pass that only reduces max|.| into out_amax, a second that
 * recomputes the tile and quantises it in the epilogue — which is bit-identical to df8_gemm_fp8_tn
 * (+DF8_EPI_AMAX) followed by df8_quantize_f32, without the 4+4+1 bytes per element of HBM traffic.
 * flags: 0 or DF8_EPI_GELU.  Needs K % 16 == 0 and N % 32 == 0.  Writes out_scale = {q, dq}. */
df8_status df8_gemm_fp8_tn_q(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                             const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                             const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                             uint8_t* out_codes, float* out_scale, float* out_amax, df8_stream stream);

/* The two passes of df8_gemm_fp8_tn_q as separate calls (a column-sharded layer combines max|out| across
 * ranks between them): _amax reduces max|epi(...)| into out_amax (cleared by the call) and writes nothing
 * else; _codes recomputes the product and emits fp8 codes with the scale derived from amax_in[0]. */
df8_status df8_gemm_fp8_tn_amax(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                const float* bias, int M, int N, int K, int flags, float* out_amax,
                                df8_stream stream);
df8_status df8_gemm_fp8_tn_codes(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a,
                                 const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                 const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                                 const float* amax_in, uint8_t* out_codes, float* out_scale, df8_stream stream);

/* ... and with A read from a_slabs column slabs (see df8_gemm_fp8_tn_ex) */
df8_status df8_gemm_fp8_tn_amax_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                   const uint8_t* w_codes, df8_kind kind_w, const float* scale_w, const float* bias,
                                   int M, int N, int K, int flags, float* out_amax, df8_stream stream);
df8_status df8_gemm_fp8_tn_codes_ex(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                    const uint8_t* w_codes, df8_kind kind_w, const float* scale_w, const float* bias,
                                    int M, int N, int K, int flags, df8_kind out_kind, const float* amax_in,
                                    uint8_t* out_codes, float* out_scale, df8_stream stream);

/* Row ranges of a slab-stored A (the "_ex" forms with one more argument): the slabs hold a_slab_rows rows each, of
 * which this call multiplies M starting at a_codes (a_codes points at the range's first row inside slab 0).  Lets a
 * caller whose A operand arrives over NVLink in row chunks start on the chunks that have landed. */
df8_status df8_gemm_fp8_tn_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                const float* bias, const float* residual, int M, int N, int K, int flags, float* out,
                                int ldc, float* out_amax, df8_stream stream);
df8_status df8_gemm_fp8_tn_amax_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                     int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                     const float* bias, int M, int N, int K, int flags, float* out_amax,
                                     df8_stream stream);
df8_status df8_gemm_fp8_tn_codes_part(const uint8_t* a_codes, df8_kind kind_a, const float* scale_a, int a_slabs,
                                      int a_slab_rows, const uint8_t* w_codes, df8_kind kind_w, const float* scale_w,
                                      const float* bias, int M, int N, int K, int flags, df8_kind out_kind,
                                      const float* amax_in, uint8_t* out_codes, float* out_scale, df8_stream stream);

/* ---- fp8 attention -------------------------------------------------------------------------
 * Replaces, inside MultiHeadAttentionLayer::forward (dnn/layers/multi_head_attention.cu:204-308), the
 * Q/K/V slice + head-split copies (:231-260), both matmul_kernel launches (:266-270, :283-287),
 * SoftmaxLayer::forward (dnn/layers/softmax_layer.cu:141-171) and the head merge (:292-294).
 *   qkv_codes  [B*T, 3E] fp8 codes of the fused QKV projection (E = H*D; Q | K | V column blocks,
 *              head h at columns [hD,(h+1)D) of each), one per-tensor scale
 *   out        [B*T, E] fp32:  softmax(Q.K^T / sqrt(D) + mask) . V, heads merged back
 *   softmax    p = exp(s - rowmax) / (sum + 1e-6), and p = 0 where mask < -1e8 (softmax_layer.cu:26-81)
 *   mask_mode  DF8_MASK_NONE, DF8_MASK_CAUSAL (the -1e9-above-the-diagonal mask upstream's tests build,
 *              tests/layers/multi_head_attention_test.cu:50-70) or DF8_MASK_ADDITIVE with
 *              mask = fp32 [mask_b,1,T,T], mask_b == B or 1 (what set_mask receives, :190-196)
 *   out_amax   optional: max|out| (cleared by the call)
 * D must be 64 or 128. */
enum { DF8_MASK_NONE = 0, DF8_MASK_CAUSAL = 1, DF8_MASK_ADDITIVE = 2 };

df8_status df8_attention_fp8(const uint8_t* qkv_codes, df8_kind kind, const float* scale, int B, int T,
                             int H, int D, int mask_mode, const float* mask, int mask_b, float* out,
                             float* out_amax, df8_stream stream);

/* ---- autoregressive decode step ---------------------------------------------------------------
 * Upstream's Gpt2::forward recomputes the whole sequence on every call (dnn/models/gpt2.cu:126-142); these calls
 * add the step after a prefill, with upstream's attention semantics (multi_head_attention.cu:225-301; softmax
 * p = exp(s - max) / (sum + 1e-6), softmax_layer.cu:26-81) restricted to the keys that exist.
 *   df8_gemv_fp8_tn          out[B,N] = epi(X[B,K] . W[N,K]^T * dq + bias) for B <= 128 token rows: the product is
 *                            bound by streaming W from HBM; flags as df8_gemm_fp8_tn (GELU, RESIDUAL, AMAX)
 *   df8_kv_cache_append      the K and V codes of Tn new positions per sequence, taken from a QKV code buffer
 *                            [B*Tn, 3E], go to rows t0 .. t0+Tn-1 of the caches [B, H, Tmax, D]; row_dq[t0 ..] receives
 *                            the buffer's dequantisation factor (scale[1]): every QKV tensor has its own per-tensor
 *                            scale, so the cache keeps one factor per position
 *   df8_attention_decode_fp8 one query per sequence and head (the Q part of qkv_codes [B, 3E]) against the first
 *                            n_keys cached positions -> out [B, E] fp32 (+ max|out|).  D = 64 or 128. */
df8_status df8_gemv_fp8_tn(const uint8_t* x_codes, df8_kind kind_x, const float* scale_x, const uint8_t* w_codes,
                           df8_kind kind_w, const float* scale_w, const float* bias, const float* residual, int B, int N,
                           int K, int flags, float* out, float* out_amax, df8_stream stream);
df8_status df8_kv_cache_append(const uint8_t* qkv_codes, const float* scale, int B, int Tn, int H, int D, int t0, int Tmax,
                               uint8_t* k_cache, uint8_t* v_cache, float* row_dq, df8_stream stream);
df8_status df8_attention_decode_fp8(const uint8_t* qkv_codes, df8_kind kind, const float* scale, const uint8_t* k_cache,
                                    const uint8_t* v_cache, const float* row_dq, int B, int H, int D, int n_keys, int Tmax,
                                    float* out, float* out_amax, df8_stream stream);

/* The decode step's position read from DEVICE memory, for steps whose launches are replayed from a CUDA graph (a
 * captured launch argument would freeze the position): *pos_d = number of positions already cached.
 *   df8_embed_pe_pos_f32          out[b] = table[ids[b]] + bias + pe_table[*pos_d]        (one token per sequence)
 *   df8_kv_cache_append_pos       the new position's K / V codes into row *pos_d of the caches
 *   df8_attention_decode_fp8_pos  pos_d != null: attends over *pos_d + 1 keys (n_keys ignored); null: as above
 *   df8_position_advance          *pos_d += 1 */
df8_status df8_embed_pe_pos_f32(const int32_t* ids, int B, int E, int V, const float* table, const float* bias,
                                const float* pe_table, const int32_t* pos_d, float* out, df8_stream stream);
df8_status df8_kv_cache_append_pos(const uint8_t* qkv_codes, const float* scale, int B, int H, int D,
                                   const int32_t* pos_d, int Tmax, uint8_t* k_cache, uint8_t* v_cache, float* row_dq,
                                   df8_stream stream);
df8_status df8_attention_decode_fp8_pos(const uint8_t* qkv_codes, df8_kind kind, const float* scale,
                                        const uint8_t* k_cache, const uint8_t* v_cache, const float* row_dq, int B,
                                        int H, int D, int n_keys, const int32_t* pos_d, int Tmax, float* out,
                                        float* out_amax, df8_stream stream);
df8_status df8_position_advance(int32_t* pos_d, df8_stream stream);

/* The step's attention straight from the fp32 QKV projection [B, 3E] and its max|.| (device scalar): the kernel
 * quantises per tensor (the codes df8_quantize_f32 would give with that maximum), writes the new position's key /
 * value codes and dequantisation factor into row n_keys - 1 of the caches (row *pos_d when pos_d != null) and attends
 * over all n_keys positions: df8_quantize_f32 + df8_kv_cache_append + df8_attention_decode_fp8 in one launch. */
df8_status df8_attention_decode_fused_f32(const float* qkv_f32, const float* qkv_amax, df8_kind kind, uint8_t* k_cache,
                                          uint8_t* v_cache, float* row_dq, int B, int H, int D, int n_keys,
                                          const int32_t* pos_d, int Tmax, float* out, float* out_amax, df8_stream stream);

/* ---- stand-alone masked softmax ------------------------------------------------------------
 * Replaces the launch of softmax_masked_kernel (dnn/layers/softmax_layer.cu:26-81, launched at
 * :154-167) for SoftmaxLayer::forward: x [B,H,T,T] fp32, optional additive mask [mask_b,1,T,T]
 * (mask_b == B or 1), out = exp(x+mask-rowmax)/(sum+1e-6), 0 where mask < -1e8. Any T. */
df8_status df8_softmax_masked_f32(const float* x, const float* mask, int mask_b, int B, int H, int T,
                                  float* out, df8_stream stream);

/* ---- LayerNorm ---------------------------------------------------------------------------
 * Replaces the launch of layer_norm_forward_kernel (dnn/layers/layer_norm_layer.cu:25-63, launched
 * at :74-79): per row over the last dimension, mean, biased variance by a second pass,
 * y = (x-mean)*rsqrt(var+eps)*gamma + beta.  gamma / beta may be NULL (no affine).
 * amax_out (optional) receives max|y| over the whole tensor (cleared by the call). */
df8_status df8_layernorm_f32(const float* x, int rows, int cols, const float* gamma, const float* beta,
                             float eps, float* y, float* amax_out, df8_stream stream);

/* LayerNorm fused with the per-tensor quantiser: codes_out = fp8(LN(x) * q), q from max|LN(x)|.
 * The fp32 LayerNorm output is never written.  row_stats_scratch: 2*rows floats of scratch
 * (8-byte aligned) for the per-row mean and rstd between the two passes.
 * Writes amax_out[0] and scale_out = {q, dq}. */
df8_status df8_layernorm_quantize_f32(const float* x, int rows, int cols, const float* gamma,
                                      const float* beta, float eps, df8_kind kind, uint8_t* codes_out,
                                      float* scale_out, float* amax_out, float* row_stats_scratch,
                                      df8_stream stream);

/* The same fused LayerNorm + quantise for callers that cannot allocate device memory (and so cannot
 * supply row_stats_scratch): a server that partitioned the whole GPU into its own arena at start-up, a
 * thread that may not block on the allocator, a thin language binding that only owns inputs and
 * outputs.  This entry point has no counterpart in the upstream project.  The per-row scratch is a
 * fixed array inside the library's device image (512 KiB on every GPU that loads the library, held until
 * the process exits); rows above 65536 are rejected with DF8_ERR_UNSUPPORTED.  The call itself performs no
 * cudaMalloc / cudaFree and uses no allocating library routine.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 * first call outside any stream capture.  All calls on a device share the one array: two calls whose
 * kernels may overlap on the GPU (different streams, no ordering between them) race on it, so order them.
 * Nothing in the array has to be cleared between calls; amax_out is cleared by the call. */
df8_status df8_layernorm_quantize_f32_noalloc(const float* x, int rows, int cols, const float* gamma,
                                              const float* beta, float eps, df8_kind kind,
                                              uint8_t* codes_out, float* scale_out, float* amax_out,
                                              df8_stream stream);

/* LayerNorm + per-tensor quantisation of a tensor whose COLUMNS are split across ranks (the column-sharded forward
 * keeps the fp32 residual stream sharded).  Same formula as df8_layernorm_f32 (layer_norm_layer.cu:40-62); the
 * ranks exchange two floats per row instead of the fp32 rows:
 *   _stats     partial_out[rows][2] = {mean, sum of squared deviations} of this rank's [rows, cols_shard] piece
 *   (caller: all-gather the partial arrays of all ranks into partial_all [world][rows][2])
 *   _amax      combines them in rank order, writes row_stats_out[rows][2] = {mean, rstd} of the whole rows and
 *              reduces max|y| over this rank's columns into amax_out (cleared by the call)
 *   (caller: maximum of amax_out over the ranks)
 *   _quantize  codes_shard_out [rows, cols_shard] = fp8(y * q), q from amax_in[0]; writes scale_out = {q, dq}
 * gamma_shard / beta_shard are this rank's slices ([cols_shard]) or NULL.  cols_shard % 4 == 0.  Sums are taken
 * in another order than a single GPU's row sum: results agree with df8_layernorm_quantize_f32 to fp32 rounding. */
df8_status df8_layernorm_shard_stats_f32(const float* x_shard, int rows, int cols_shard, float* partial_out,
                                         df8_stream stream);
df8_status df8_layernorm_shard_amax_f32(const float* x_shard, int rows, int cols_shard, const float* partial_all,
                                        int world, const float* gamma_shard, const float* beta_shard, float eps,
                                        float* row_stats_out, float* amax_out, df8_stream stream);
df8_status df8_layernorm_shard_quantize_f32(const float* x_shard, int rows, int cols_shard, const float* row_stats,
                                            const float* gamma_shard, const float* beta_shard, df8_kind kind,
                                            const float* amax_in, uint8_t* codes_shard_out, float* scale_out,
                                            df8_stream stream);

/* ---- token embedding + positional encoding -----------------------------------------------
 * Replaces embedding_forward_kernel (dnn/tokens/token_embedding.cu:31-45, launched at :146-154) and
 * add_positional_encodings_kernel (dnn/tokens/positional_encoding.cu:31-48, launched at :94-104):
 *     out[b,t,:] = table[ids[b,t],:] + bias[:] + pe[t,:]
 * ids [B,T] int32, table [V,E], bias [E] or NULL, pe [>=T,E] or NULL, out [B,T,E].
 * An id outside [0,V) yields a zero row and increments bad_ids[0] (optional, cleared by the call);
 * upstream throws for such ids (token_embedding.cu:131-138) and the C++ layer above does too. */
df8_status df8_embed_pe_f32(const int32_t* ids, int B, int T, int E, int V, const float* table,
                            const float* bias, const float* pe, float* out, int32_t* bad_ids,
                            df8_stream stream);

/* ---- layer-streaming weight upload -----------------------------------------------------------
 * Pinned host arena holding one byte blob per layer + a ring of device slots + a copy stream, after
 * the slot-ring loader of apps/host-multi/NVMeLoader_Linux.hpp:38-183 (pinned slots, per-slot stream,
 * cudaMemcpyAsync, (pointer, size, stream) hand-off at :90-134).  Usage per layer l of a forward:
 *     acquire(l, compute)  -> device pointer of the layer's bytes; compute stream waits for the upload
 *     ... launch the layer's kernels on the compute stream ...
 *     release(l, compute)  -> the slot may be overwritten once those kernels are done
 *     prefetch((l + n_slots) % n_layers)   -> upload of a later layer overlaps the following compute
 * Slots are filled in the order of the uploads (a ring), so with this loop the slot refilled is the one just
 * released, for any ratio of layers to slots.
 * create allocates (cudaHostAlloc, cudaMalloc, stream, events); destroy frees.  The other calls
 * neither allocate nor synchronise, except resize and time_uploads (both wait for the device).
 * Not thread-safe: one streamer per model per host thread. */
typedef struct df8_streamer df8_streamer;
typedef struct df8_comm df8_comm;
df8_status df8_streamer_create(size_t slot_bytes, int n_slots, int n_layers, df8_streamer** out);
/* The same for ranks that work on shares of one batch with replicated weights (one process per GPU, the same
 * layer loop on every rank): each upload copies only this rank's 1/world share of the layer from ITS pinned
 * arena and an all-gather over `comm` on the copy stream completes the slot, so host->device bytes per rank fall
 * world-fold.  prefetch / acquire are then collectives: every rank must issue the same sequence.  comm == NULL
 * (or a single rank) is df8_streamer_create.  The communicator is borrowed, not owned. */
df8_status df8_streamer_create_sharded(size_t slot_bytes, int n_slots, int n_layers, df8_comm* comm,
                                       df8_streamer** out);
/* Replaces the ring of device slots by one of n_slots (waits for the device; every layer becomes non-resident). */
df8_status df8_streamer_resize(df8_streamer* s, int n_slots);
/* bytes this rank has copied from host memory / received from its peers so far */
df8_status df8_streamer_traffic(df8_streamer* s, unsigned long long* h2d_bytes_h, unsigned long long* gathered_bytes_h);
/* Uploads every layer once, back to back, with nothing else running, and returns the device time in ms
 * (measurement aid: the upload time a forward has to hide; waits for the device; collective when sharded). */
df8_status df8_streamer_time_uploads(df8_streamer* s, float* ms_h);
df8_status df8_streamer_destroy(df8_streamer* s);
/* host_ptr_h receives the pinned HOST address where layer `layer`'s slot_bytes bytes are kept */
df8_status df8_streamer_host_ptr(df8_streamer* s, int layer, void** host_ptr_h);
df8_status df8_streamer_prefetch(df8_streamer* s, int layer);
df8_status df8_streamer_acquire(df8_streamer* s, int layer, df8_stream compute_stream, void** dev_ptr_h);
df8_status df8_streamer_release(df8_streamer* s, int layer, df8_stream compute_stream);
df8_status df8_streamer_stats(df8_streamer* s, unsigned long long* bytes_uploaded_h, size_t* slot_bytes_h,
                              int* n_slots_h);

/* ---- operands of the fully-connected backward pass as fp8 products --------------------------------------
 * Upstream: fc_backward_input / fc_backward_weights / fc_backward_bias (dnn/layers/fully_connected_layer.cu:43-107,
 * launches :317-353): dX = dY W, dW = dY^T X, db = sum_n dY.  The two products run through df8_gemm_fp8_tn, which
 * contracts over the contiguous dimension of both operands, so they need W^T [in, out], dY^T [out, N] and
 * X^T [in, N] as codes:
 *   df8_quantize_transpose_f32  fp32 [rows, cols] -> codes [cols, ld_t] (ld_t >= rows; columns rows .. ld_t-1 are
 *                               written as zero codes: padding of the K dimension), scale from amax_in_d as in
 *                               df8_quantize_f32, so the codes equal those of the untransposed tensor
 *   df8_transpose_u8            codes [rows, ld_in] (cols used) -> [cols, ld_out], zero beyond `rows`
 *   df8_colsum_f32              out_d[c] = sum_r x_d[r * ld + c]; partial_d: df8_colsum_partial_floats(cols) floats
 *                               of scratch; fixed summation order (no atomics) */
df8_status df8_quantize_transpose_f32(const float* x_d, int rows, int cols, df8_kind kind, const float* amax_in_d,
                                      uint8_t* codes_t_d, int ld_t, float* scale_out_d, df8_stream stream);
/* one read of x for both layouts: codes_t_d as above, and the same codes untransposed in codes_d [rows, ld_c]
 * (ld_c >= cols; bytes cols .. ld_c-1 of a row are left alone); codes_d may be null */
df8_status df8_quantize_both_layouts_f32(const float* x_d, int rows, int cols, df8_kind kind, const float* amax_in_d,
                                         uint8_t* codes_t_d, int ld_t, uint8_t* codes_d, int ld_c, float* scale_out_d,
                                         df8_stream stream);
df8_status df8_transpose_u8(const uint8_t* in_d, int rows, int cols, int ld_in, uint8_t* out_d, int ld_out,
                            df8_stream stream);
df8_status df8_colsum_f32(const float* x_d, int rows, int cols, int ld, float* partial_d, float* out_d,
                          df8_stream stream);
/* the same pass also reducing max|x| into amax_out_d (cleared first, like df8_amax_f32), or null */
df8_status df8_colsum_amax_f32(const float* x_d, int rows, int cols, int ld, float* partial_d, float* out_d,
                               float* amax_out_d, df8_stream stream);
int df8_colsum_partial_floats(int cols);

/* ---- softmax cross-entropy on fp32 logits (training-side neighbour of the vocabulary head) -----------------
 * Replaces cross_entropy_log_softmax_kernel / cross_entropy_gradient_logit_kernel
 * (dnn/losses/cross_entropy.cu:12-74, 77-139; launches :147-153, :181-187) with upstream's arithmetic:
 *   loss_i  = -sum_j t_ij (x_ij - max_i - log(sum_j exp(x_ij - max_i) + 1e-7))
 *   grad_ij = exp(x_ij - max_i) / (sum_j exp(x_ij - max_i) + 1e-7) - t_ij
 * Targets: either upstream's dense [rows, ldt] matrix (targets_d) or one class index per row (target_idx_d);
 * exactly one of the two.  ld / ldt / ldg: row pitches in floats (>= classes), so the pitched logits of the head
 * GEMM are read in place.  An index outside [0, classes) contributes nothing and is counted
 * (df8_cross_entropy_bad_indices; the reduction of the row losses to their mean is the caller's, as upstream does
 * it on the host, cross_entropy.cu:155-168). */
df8_status df8_cross_entropy_f32(const float* logits_d, int ld, const float* targets_d, int ldt,
                                 const int* target_idx_d, int rows, int classes, float* row_loss_d, df8_stream stream);
df8_status df8_cross_entropy_grad_f32(const float* logits_d, int ld, const float* targets_d, int ldt,
                                      const int* target_idx_d, int rows, int classes, float* grad_d, int ldg,
                                      df8_stream stream);
df8_status df8_cross_entropy_bad_indices(unsigned int* count_h, int reset);

/* ---- collectives for the column-sharded fully-connected path --------------------------------------
 * Upstream has no communication backend: its multi-GPU mode runs independent replicas under a
 * tbb::parallel_for (apps/host-multi/main.cpp:157-181).  These calls wrap NCCL (bound at run time with
 * dlopen, so the library loads without it): one communicator per process, one process per GPU.
 * Rank 0 makes the 128-byte id (df8_comm_unique_id, HOST buffer) and passes it to the other ranks by
 * any host channel; df8_comm_init_rank is collective and allocates; the data calls are enqueued on
 * `stream` and neither allocate nor synchronise.  df8_comm_abort ends outstanding collectives with an
 * error when a peer has gone away (host-side failure handling; never on the data path). */
df8_status df8_comm_available(int* version_h);
df8_status df8_comm_unique_id(void* id_h);
df8_status df8_comm_init_rank(const void* id_h, int world, int rank, df8_comm** out);
df8_status df8_comm_destroy(df8_comm* c);
df8_status df8_comm_abort(df8_comm* c);
df8_status df8_comm_rank(const df8_comm* c, int* rank_h, int* world_h);
/* recv_d[r*bytes_per_rank ...] = rank r's send_d (the gathered layout is rank-major) */
df8_status df8_comm_allgather_u8(df8_comm* c, const uint8_t* send_d, uint8_t* recv_d, size_t bytes_per_rank,
                                 df8_stream stream);
/* in place: buf_d[i] = max over ranks (the per-tensor amax of a tensor whose columns are sharded) */
df8_status df8_comm_allreduce_max_f32(df8_comm* c, float* buf_d, size_t count, df8_stream stream);

/* Exchanges of the column-sharded forward without NCCL kernels on the data path (no upstream counterpart).  Buffers
 * from df8_comm_symm_alloc exist on every rank and are mapped into every other rank (cudaMalloc + CUDA IPC; the
 * call is collective, allocates and synchronises; buffers live until df8_comm_destroy).  Where the mapping is not
 * possible (or with DF8_COMM_P2P=0 in the environment) the calls below fall back to NCCL on the same buffers.
 *   df8_comm_allgather_symm   every rank's slice — bytes_per_rank bytes at local_d + offset + rank*bytes_per_rank of
 *                             ITS copy, produced by work already on `stream` — is copied by the copy engines into
 *                             the same position of every peer's copy over NVLink; later work on `stream` sees all
 *                             world slices.  The wait for the peers is a bounded poll (2 s, then status word).
 *   df8_comm_allreduce_max_p2p  value_d[0] <- max over ranks, one small kernel per rank (the value travels inside
 *                             the flag word the peers poll).
 * Every rank must issue the same sequence of these calls.  Neither allocates or synchronises the host. */
df8_status df8_comm_symm_alloc(df8_comm* c, size_t bytes, void** local_d_h);
df8_status df8_comm_p2p_enabled(df8_comm* c, int* enabled_h);
df8_status df8_comm_allgather_symm(df8_comm* c, void* local_d, size_t offset, size_t bytes_per_rank,
                                   df8_stream stream);
/* df8_comm_allgather_symm in two halves, for a gather that is pipelined in pieces: push [local_d + offset, + bytes)
 * to the same place in every peer's copy as soon as it is produced (returns a ticket), and make a stream wait for the
 * peers' push with that ticket only where the piece is consumed (own_too: also for this rank's own pushes so far,
 * after which its slab may be rewritten).  Needs the peer-mapped transport; every rank issues the same pushes in
 * the same order; a ticket stays valid for 64 further pushes. */
df8_status df8_comm_push_symm(df8_comm* c, void* local_d, size_t offset, size_t bytes, df8_stream stream,
                              unsigned int* ticket_h);
df8_status df8_comm_wait_symm(df8_comm* c, unsigned int ticket, int own_too, df8_stream stream);
df8_status df8_comm_allreduce_max_p2p(df8_comm* c, float* value_d, df8_stream stream);
/* bytes this rank has sent to its peers through df8_comm_allgather_symm */
df8_status df8_comm_bytes_pushed(df8_comm* c, unsigned long long* bytes_h);

/* Column-sharded fully-connected layer (no upstream counterpart: upstream's layer always holds the full
 * [out,in] weight, dnn/layers/fully_connected_layer.cu:112-116).  Every rank passes the full quantised input
 * a_codes [M,K] and ITS row block of the weight codes w_shard_codes [N/world, K] (rank r owns output columns
 * [r*N/world, (r+1)*N/world)), with the scale of the WHOLE weight tensor; bias_shard is the matching slice.
 * Result on every rank: out_codes [M,N], out_scale, out_amax identical to df8_gemm_fp8_tn_q on one GPU.
 * Steps: amax pass -> all-reduce(max) of one float -> codes pass -> all-gather of M*N/world bytes per rank
 * -> interleave.  slice_scratch: M*N/world bytes, gathered_scratch: M*N bytes.  N % (32*world) == 0. */
df8_status df8_fc_fp8_column_sharded(df8_comm* comm, const uint8_t* a_codes, df8_kind kind_a,
                                     const float* scale_a, const uint8_t* w_shard_codes, df8_kind kind_w,
                                     const float* scale_w, const float* bias_shard, int M, int N, int K,
                                     int flags, df8_kind out_kind, uint8_t* slice_scratch,
                                     uint8_t* gathered_scratch, uint8_t* out_codes, float* out_scale,
                                     float* out_amax, df8_stream stream);
/* out [M, world*cols_per_rank] <- gathered [world][M, cols_per_rank] (the layout an all-gather leaves) */
df8_status df8_interleave_gathered_u8(const uint8_t* gathered, int M, int cols_per_rank, int world,
                                      uint8_t* out, df8_stream stream);

/* ---- bounded-wait status word --------------------------------------------------------------
 * Every device-side wait (mbarrier polls in the GEMM and attention pipelines) gives up after a
 * time limit instead of hanging the GPU; the first such event stores a non-zero code.  Upstream
 * has no counterpart (its kernels do not wait on one another).  Both calls synchronise with the
 * device (they copy from / to a device symbol); code_h / count_h are HOST pointers. */
df8_status df8_status_word_read(unsigned int* code_h, unsigned int* count_h);
df8_status df8_status_word_reset(void);
/* DF8_OK while the word is clean; DF8_ERR_TIMEOUT (with the first code and the count in df8_last_error()) once a
 * wait has given up, until df8_status_word_reset().  Results produced after such an event are not to be trusted:
 * a kernel that gave up left part of its output unwritten.  Synchronises like df8_status_word_read.  The C++
 * layer turns it into the std::runtime_error upstream raises for a failed CUDA call (dnn/utils/common.cuh:20-35). */
df8_status df8_status_word_check(void);

#ifdef __cplusplus
}
#endif
#endif /* DF8_H_ */
