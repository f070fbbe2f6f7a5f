/* The C interface of the step walker (step_walker.cu): a model of built-in parts described in
 * plain structures, and one call that makes all launches of a step on a CUDA stream.
 *
 * The reference's C API is the scheduler's (include/sgl/scheduler.h:33-67: new, submit_ids, step,
 * poll, stats, free) above a model object; here the scheduler is Python and this is the layer
 * below it: what `sgl_model_prefill` / `sgl_model_decode_batch` (include/sgl/model.h:29-35) are
 * to the reference's scheduler, `sglc_walker_forward` is to this one, for any mix of prompt
 * portions and single decoded tokens in one call.
 *
 * A host in C fills a WalkModel once (device pointers of the weights in the runtime's precision,
 * [out][in] matrices, float vectors; the cache tensors of each call of the running order), binds
 * the kernel launchers (sglc_walker_names lists them; sglc_walker_bind takes their addresses, in
 * that order, from the libraries they live in), and per step fills a WalkStep with the device
 * arrays of the step (the layout engine/step.py packs) and calls sglc_walker_forward.
 * engine/host_model.py does exactly this through ctypes.
 */
#ifndef SGLC_STEP_WALKER_H
#define SGLC_STEP_WALKER_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- the model, as the host needs it (filled by engine/host_model.py through ctypes) ----------
typedef struct WalkLinear {
  const void* w;            // [N][K], the runtime's matrix precision
  const float* bias;        // [N] or null
  int N, K;
} WalkLinear;
typedef struct WalkNorm {
  const float* gamma;
  const float* beta;
  float eps;
  int size;
} WalkNorm;
typedef struct WalkLayer {
  WalkNorm norm1, norm2;
  WalkLinear qkv, out, up, down;
  int n_heads, n_kv_heads, head_dim, window;    // window 0: none
  float scale;
  int act;                                      // SGLC_ACT_*
  int inner_size, pad;
} WalkLayer;
typedef struct WalkCall {
  int layer;                // index into layers
  int group;                // cache group of the call
  int write;                // the call owns its cache (writes keys and values)
  int n_pages;
  void* cache;              // [n_pages][2][Hkv][page_size][D]
} WalkCall;
typedef struct WalkModel {
  const void* table;        // token table [V][E]
  const void* pos_table;    // [P][E] or null
  const WalkLayer* layers;
  const WalkCall* order;
  WalkNorm final_norm;
  WalkLinear head;
  int vocab, n_positions, hidden, n_layers, n_calls, bf16, page_size, pad;
} WalkModel;
typedef struct WalkStep {
  const int* tokens; const int* positions; const int* token_req; const int* want_rows;
  const int* q_start; const int* kv_len; const int* decode_tokens;
  const int* const* block_tables;               // per cache group
  const int* const* slots;                      // per cache group
  unsigned char* workspace; long long workspace_bytes;
  float* logits;                                // [n_want][vocab]
  int* err_flag;                                // bad token or position ids
  int* tc_err;                                  // the tensor-core kernels' error word
  float* tc_ws; long long tc_ws_floats; int* tc_counters; int tc_n_counters;
  int T, R, n_want, max_q_len, max_keys, n_decode, decode_ordered, few_ok, bt_stride;
  int stream_min_items, use_tma_decode, few_max_tokens;
  long long few_max_weight;
  cudaStream_t stream;
  long long launches;                           // out: kernels launched
  long long workspace_peak;                     // out
  char where[96];                               // out: the operation that failed
} WalkStep;


/* the names of the launchers to bind, in the order sglc_walker_bind expects their addresses */
int sglc_walker_names(const char* const** names);
int sglc_walker_bind(void* const* fns, int n);
/* sizeof of the six structures above, for a binding to check itself against */
int sglc_walker_struct_sizes(int* sizes);
/* one forward pass of the step; 0, or the failing launcher's code (step->where names it) */
int sglc_walker_forward(const WalkModel* model, WalkStep* step);
const char* sglc_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif
