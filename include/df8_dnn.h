/*
 * df8_dnn.h — C harness over the C++17 `dnn::` classes (libdf8_dnn.so).
 *
 * The product API for C++ callers is the class interface under deepfuse_b200/dnn (the same class and
 * member names as the upstream project's dnn/core, dnn/layers, dnn/tokens, dnn/models).  This header
 * exists so that a non-C++ host (the Python tests and bench.py) can drive those classes: every function
 * constructs / calls the C++ objects and converts exceptions into a non-zero return code whose text is
 * available from dnn_last_error().  Pointers ending in `_h` are HOST pointers, `_d` DEVICE pointers.
 */
#ifndef DF8_DNN_H_
#define DF8_DNN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dnn_gpt2 dnn_gpt2;

const char* dnn_last_error(void);

/* Creates the calling thread's dnn::Cuda context for `device` (dnn/core/cuda.cuh) if there is none. */
int dnn_init(int device);
/* dnn::Cuda::set_stream for the calling thread; stream is a cudaStream_t. */
int dnn_set_stream(void* stream);
/* fp8 kinds (0 = e4m3, 1 = e5m2) used for weights and for activations. */
int dnn_set_fp8_policy(int weight_kind, int activation_kind);
/* 0: constructors of layers leave weights zero instead of drawing them on the host (then fill on the device or
 * upload); 1 (default): upstream's behaviour. */
int dnn_set_host_init(int enabled);

/* ---- dnn::Gpt2<float> ---- */
dnn_gpt2* dnn_gpt2_create(int vocab, int max_seq_len, int layers, int heads, int hidden, int ffn);
void dnn_gpt2_destroy(dnn_gpt2* m);
int dnn_gpt2_set_options(dnn_gpt2* m, int mlp_gelu, int causal);
/* Parameters in a fixed order: embedding {weights,bias}; per block {ln1 g,b; ln2 g,b; qkv W,b; out W,b;
 * fc1 W,b; fc2 W,b}; final_fc {W,b}.  name_h receives e.g. "block3.fc1.weight". */
int dnn_gpt2_num_params(dnn_gpt2* m);
int dnn_gpt2_param_info(dnn_gpt2* m, int index, char* name_h, int name_cap, int* shape_h, int* ndim_h);
int dnn_gpt2_param_upload(dnn_gpt2* m, int index, const float* data_h);
int dnn_gpt2_param_download(dnn_gpt2* m, int index, float* data_h);
/* Every weight matrix <- N(0, std) generated on the device from counter-based streams numbered seed*1000 + 1, 2, ...
 * (embedding; per block qkv, out, fc1, fc2; head), biases <- 0: the values of deepfuse_b200/synthetic.py
 * make_gpt2_params(cfg, seed, std) up to the last bit of fp32 log / cos, without the trip through the host. */
int dnn_gpt2_initialize_on_device(dnn_gpt2* m, unsigned long long seed, float std);
/* Gpt2::set_stage_timing / last_head_ms: events around the vocabulary-head GEMM inside the forward. */
int dnn_gpt2_set_stage_timing(dnn_gpt2* m, int on);
int dnn_gpt2_last_head_ms(dnn_gpt2* m, float* ms_h);
/* Quantises every weight now (otherwise it happens lazily in the first forward). */
int dnn_gpt2_prepare(dnn_gpt2* m);
/* logits [B*T, vocab] fp32 stay on the device, owned by the handle until the next forward;
 * ids are int32 on the device (ids_d) or on the host (ids_h, uploaded inside the call). */
int dnn_gpt2_forward_logits(dnn_gpt2* m, const int32_t* ids_d, int B, int T, int check_ids, float** logits_d);
int dnn_gpt2_forward_logits_host(dnn_gpt2* m, const int32_t* ids_h, int B, int T, float** logits_d);
/* Gpt2::forward_logits_pitched: logits [B*T, *pitch_h] fp32 with the first `vocab` columns of every row valid
 * (pitch = vocab rounded up to a multiple of 32 floats); ids on the device, or on the host when ids_on_host. */
int dnn_gpt2_forward_logits_pitched(dnn_gpt2* m, const int32_t* ids, int ids_on_host, int B, int T, int check_ids,
                                    float** logits_d, int* pitch_h);
/* Enqueues the copy of the last logits (dense or pitched) to a dense HOST array [rows, vocab] on the thread's
 * stream (pinned memory makes it asynchronous); the caller synchronises before reading dst_h. */
int dnn_gpt2_copy_logits_host(dnn_gpt2* m, float* dst_h);
/* A serving loop's step: ids on the HOST in, the full dense logits [B*T, vocab] out to (pinned) host memory, with the
 * device-to-host copy on a stream of its own so that it overlaps the next step's forward.  dst_h must stay untouched
 * until the next-but-one call; dnn_gpt2_serve_flush makes the thread's stream wait for every copy issued so far. */
int dnn_gpt2_serve_step(dnn_gpt2* m, const int32_t* ids_h, int B, int T, float* dst_h);
int dnn_gpt2_serve_flush(dnn_gpt2* m);
/* hidden states [B,T,E] of Gpt2::forward_hidden, device pointer owned by the handle */
int dnn_gpt2_forward_hidden(dnn_gpt2* m, const int32_t* ids_d, int B, int T, float** hidden_d);
/* the model's own public batch-1 entry point, Gpt2::forward(std::vector<int>): hidden [1,T,E] to host */
int dnn_gpt2_forward_ids(dnn_gpt2* m, const int32_t* ids_h, int T, float* hidden_h);
/* Gpt2::enable_layer_streaming: block weight codes move to pinned host memory and are uploaded per layer
 * through `slots` device buffers on a side stream; release_fp32 also frees the fp32 block weights. */
int dnn_gpt2_enable_streaming(dnn_gpt2* m, int slots, int release_fp32);
/* the same with each rank of `comm` (a df8_comm*, see include/df8.h) uploading 1/world of every layer and an all-gather
 * completing the slot; every rank then runs the same sequence of forwards */
int dnn_gpt2_enable_streaming_sharded(dnn_gpt2* m, int slots, int release_fp32, void* comm);
/* measurement aids (Gpt2::resize_streaming_slots, streaming_traffic, time_layer_uploads) */
int dnn_gpt2_resize_streaming_slots(dnn_gpt2* m, int slots);
int dnn_gpt2_streaming_traffic(dnn_gpt2* m, unsigned long long* h2d_bytes_h, unsigned long long* gathered_bytes_h);
int dnn_gpt2_time_layer_uploads(dnn_gpt2* m, float* ms_h);
int dnn_gpt2_disable_streaming(dnn_gpt2* m);
unsigned long long dnn_gpt2_streamed_bytes(dnn_gpt2* m);
int dnn_gpt2_save(dnn_gpt2* m, const char* path);
dnn_gpt2* dnn_gpt2_load(const char* path);

/* ---- dnn::Gpt2ColumnSharded<float>: fully-connected weights split by output columns over the ranks of a
 * df8_comm (include/df8.h; NULL = a single rank).  Parameters are this rank's SHARDS, named as above:
 * blockN.qkv.weight is [3E/g, E] = the rows {Q, K, V} x (this rank's heads) of the fused weight, blockN.out /
 * fc1 / fc2 .weight are row blocks [E/g,E], [F/g,E], [E/g,F] (biases likewise), final_fc.weight is rows
 * [vocab_begin, vocab_begin + vocab_rows) of the head; embedding and LayerNorm parameters are replicated. ---- */
typedef struct dnn_gpt2cs dnn_gpt2cs;
dnn_gpt2cs* dnn_gpt2cs_create(void* comm, int vocab, int max_seq_len, int layers, int heads, int hidden, int ffn);
void dnn_gpt2cs_destroy(dnn_gpt2cs* m);
int dnn_gpt2cs_set_options(dnn_gpt2cs* m, int mlp_gelu, int causal);
int dnn_gpt2cs_vocab_range(dnn_gpt2cs* m, int* begin_h, int* rows_h);
int dnn_gpt2cs_num_params(dnn_gpt2cs* m);
int dnn_gpt2cs_param_info(dnn_gpt2cs* m, int index, char* name_h, int name_cap, int* shape_h, int* ndim_h);
int dnn_gpt2cs_param_upload(dnn_gpt2cs* m, int index, const float* data_h);
/* uniform random shards generated on the device (for shapes too large to initialise through the host) */
int dnn_gpt2cs_initialize_on_device(dnn_gpt2cs* m, unsigned long long seed);
/* collective: quantises every shard with the scale of its whole (sharded) tensor */
int dnn_gpt2cs_prepare(dnn_gpt2cs* m);
/* collective: logits of this rank's vocabulary rows [B*T, vocab_rows] fp32, owned by the handle */
int dnn_gpt2cs_forward_logits_shard(dnn_gpt2cs* m, const int32_t* ids_d, int B, int T, int check_ids,
                                    float** logits_d);
int dnn_gpt2cs_forward_logits_shard_host(dnn_gpt2cs* m, const int32_t* ids_h, int B, int T, float** logits_d);
/* the same in a row-pitched buffer [B*T, *pitch_h] (pitch = vocab_rows rounded up to a multiple of 32 floats) */
int dnn_gpt2cs_forward_logits_shard_pitched(dnn_gpt2cs* m, const int32_t* ids, int ids_on_host, int B, int T,
                                            int check_ids, float** logits_d, int* pitch_h);
/* collective: hidden states after the last block, gathered onto every rank, [B,T,E] fp32 */
int dnn_gpt2cs_forward_hidden(dnn_gpt2cs* m, const int32_t* ids_d, int B, int T, float** hidden_d);
/* bytes this rank has pushed to its peers' buffers since the model was made (0 for a single rank) */
unsigned long long dnn_gpt2cs_bytes_pushed(dnn_gpt2cs* m);

/* ---- single layers through their public forward(), host buffers in and out ---- */
int dnn_fc_forward(int in_features, int out_features, const float* w_h, const float* b_h, const float* x_h, int M,
                   float* y_h);
/* FullyConnectedLayer<float>(in, out, training_enabled = true): forward(x) then backward(dy)
 * (fully_connected_layer.cu:216-356); dx [M, in], dw [out, in], db [out]; host arrays, outputs may be null */
int dnn_fc_backward(int in_features, int out_features, const float* w_h, const float* b_h, const float* x_h, int M,
                    const float* dy_h, float* dx_h, float* dw_h, float* db_h);
int dnn_layernorm_forward(int rows, int cols, const float* gamma_h, const float* beta_h, float eps, const float* x_h,
                          float* y_h);
int dnn_softmax_forward(int B, int H, int T, const float* x_h, const float* mask_h, int mask_b, float* y_h);
/* params: qkv W [3E,E], b [3E]; out W [E,E], b [E]; mask_mode 0 none, 1 causal flag, 2 additive tensor */
int dnn_mha_forward(int B, int T, int E, int H, const float* wqkv_h, const float* bqkv_h, const float* wo_h,
                    const float* bo_h, const float* x_h, int mask_mode, const float* mask_h, int mask_b, float* y_h);
/* one TransformerBlock; params_h: 12 host arrays in the order ln1 g,b; ln2 g,b; qkv W,b; out W,b; fc1 W,b; fc2 W,b */
int dnn_block_forward(int B, int T, int E, int H, int F, const float* const* params_h, int n_params, int mlp_gelu,
                      int causal, const float* x_h, float* y_h);
int dnn_embedding_forward(int V, int E, int max_len, const float* table_h, const float* bias_h, const int32_t* ids_h,
                          int B, int T, int add_positions, float* y_h);

/* ---- autoregressive decoding: Gpt2::prefill (prompt [B,T] -> logits of the last position [B, vocab], KV cache for
 * max_len positions, 0 = max_seq_len), Gpt2::decode_step (one new token id per sequence -> logits [B, vocab]),
 * Gpt2::end_decode.  Device pointers owned by the handle until its next call. ---- */
int dnn_gpt2_prefill(dnn_gpt2* m, const int32_t* ids_d, int B, int T, int max_len, float** logits_d);
int dnn_gpt2_decode_step(dnn_gpt2* m, const int32_t* next_ids_d, int B, int check_ids, float** logits_d);
int dnn_gpt2_end_decode(dnn_gpt2* m);
/* 1 once decode steps are replayed from a CUDA graph (from the third step after a prefill when the model's stream is
 * not the legacy default stream and DF8_DECODE_GRAPH is not 0), else 0 */
int dnn_gpt2_decode_graph_active(dnn_gpt2* m, int* active);

/* ---- CrossEntropyLoss<float> (dnn/losses/cross_entropy.cuh:8-20): logits_d [rows, pitch] (pitch == classes: dense),
 * dense targets [rows, classes] or class indices [rows] (one of the two); the mean loss goes to *loss_h, the
 * gradient [rows, classes] to grad_d; either output may be null ---- */
int dnn_cross_entropy(const float* logits_d, int rows, int classes, int pitch, const float* targets_d,
                      const int32_t* idx_d, float* loss_h, float* grad_d);

/* ---- checkpoint files ----
 * save_upstream / load_upstream: the layout upstream's Gpt2::save writes (header, tokenizer state, then every layer
 * preceded by the raw bytes of its name); a model needs a tokenizer to be saved that way
 * (dnn_gpt2_create_with_tokenizer builds one from a vocabulary JSON file).
 * save_quantized / load_quantized: the quantise-once cache (e4m3 codes + scales of every fully-connected layer, fp32
 * embedding and LayerNorm parameters); a model loaded from it holds no fp32 weight matrices.
 * forward_text: Gpt2::forward_from_text, hidden states [1,T,E] to the host, *tokens_h = T. */
dnn_gpt2* dnn_gpt2_create_with_tokenizer(const char* vocab_json_path_h, int vocab, int max_seq_len, int layers, int heads,
                                         int hidden, int ffn);
int dnn_gpt2_save_upstream(dnn_gpt2* m, const char* path_h);
dnn_gpt2* dnn_gpt2_load_upstream(const char* path_h);
int dnn_gpt2_save_quantized(dnn_gpt2* m, const char* path_h);
dnn_gpt2* dnn_gpt2_load_quantized(const char* path_h);
int dnn_gpt2_forward_text(dnn_gpt2* m, const char* text_h, float* hidden_h, int cap_floats, int* tokens_h);
/* Reads one record with the class's own load(), hands the parameter tensors back one after the other and writes
 * the record again with the class's own save(): what = 0 tensor<float>, 1 FullyConnectedLayer, 2 LayerNormLayer,
 * 3 TokenEmbedding, 4 TransformerBlock. */
int dnn_file_roundtrip(int what, const char* in_path_h, const char* out_path_h, float* params_h, int cap_floats,
                       int* count_h);

/* ---- the text front end: dnn::BpeTokenizer over a dnn::VocabLoader (host-only).  The vocabulary comes from a JSON
 * file (a merges.txt beside it is picked up) or, when state_path_h is a non-empty string, from a binary state stream
 * as Tokenizer::save writes it.  encode returns the number of ids (-1 on error), decode the length of the text. ---- */
int dnn_tokenizer_encode(const char* vocab_json_path_h, const char* state_path_h, const char* text_h, int add_special,
                         int* ids_out_h, int cap);
int dnn_tokenizer_decode(const char* vocab_json_path_h, const char* state_path_h, const int* ids_h, int n, int skip_special,
                         char* out_h, int cap);
int dnn_tokenizer_save(const char* vocab_json_path_h, const char* out_path_h);

/* ---- self tests written in C++ against the class API (tensor, Cuda/StreamGuard, error behaviour);
 * return the number of failed checks and write a report to report_h. ---- */
int dnn_selftest_tensor(char* report_h, int cap);
int dnn_selftest_context(char* report_h, int cap);
int dnn_selftest_errors(char* report_h, int cap);
/* makes a bounded device-side wait run out (a 1 ms limit on a barrier nobody arrives at; nothing faults or hangs)
 * and follows the failure to the caller: status word, DF8_ERR_TIMEOUT, std::runtime_error, reset, normal work */
int dnn_selftest_bounded_wait(char* report_h, int cap);
/* the text front end (dnn::VocabLoader, dnn::BpeTokenizer; host-only, needs no GPU): upstream's own test cases on
 * vocabulary files written into the directory dir_h */
int dnn_selftest_tokenizer(const char* dir_h, char* report_h, int cap);

#ifdef __cplusplus
}
#endif
#endif /* DF8_DNN_H_ */
