/* The engine's C interface: load a model folder, submit requests as token ids, step, poll.
 *
 * The shape is the reference's scheduler API (include/sgl/scheduler.h:33-67,102: sgl_sched_new,
 * sgl_sched_submit_ids, sgl_sched_step, sgl_sched_poll, sgl_sched_nactive, sgl_sched_abort,
 * sgl_sched_get_stats, sgl_sched_free) with its sampling options (include/sgl/sampling.h:12-24).
 * Everything behind it is native: configuration and safetensors reading, the architecture
 * registry, the page tables, the scheduler, the packed step arrays, CUDA graphs of repeated
 * step shapes, the launches of a step (step_walker.h) and the device sampler.  Models made of
 * the built-in parts run here; the Python engine remains the general one (parts registered from
 * outside the package).
 *
 * The library (libsglc_host_engine.so) finds the kernel libraries (libsglc_*.so, built by
 * `python -c "import __graft_entry__ as g; g.build()"`) in the folder it lies in, or in
 * options.library_dir, and refuses to start without them: there is no CPU path.
 *
 * An engine is used from one thread at a time.  Several engines may live in a process.
 */
#ifndef SGLC_ENGINE_H
#define SGLC_ENGINE_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sglc_engine sglc_engine;

typedef struct sglc_sampling {
  float temperature;              /* <= 0: greedy */
  int top_k;                      /* <= 0: off */
  float top_p;                    /* outside (0,1): off */
  float min_p;                    /* > 0: drop candidates with p < min_p * p_max */
  float repetition_penalty;       /* > 0 and != 1: positive logits divided, negative multiplied */
  float frequency_penalty;        /* logit -= f * count(token) */
  float presence_penalty;         /* logit -= p if the token was generated before */
  int ignore_eos;
  int stop_ids[8];
  int n_stop_ids;
  unsigned long long seed;        /* mixed into the request's random stream */
} sglc_sampling;

typedef struct sglc_engine_options {
  int device;                     /* CUDA device index */
  int bf16;                       /* 1: bfloat16 weights, activations and cache; 0: everything in true 32-bit */
  int page_size;                  /* positions per cache page */
  long long n_pages;              /* pages of the pool; 0: enough for max_tokens positions */
  long long max_tokens;           /* used when n_pages is 0; 0 as well: max_requests full-length requests */
  int max_requests;               /* live requests (slots) */
  int max_step_tokens;            /* tokens of one step */
  int prefill_chunk;              /* longest prompt portion of a step; <= 0: 4096 (the reference's SGL_PREFILL_CHUNK) */
  int token_budget;               /* tokens a step may bring; <= 0: max_step_tokens */
  unsigned long long seed;
  int use_graphs;                 /* replay CUDA graphs of step shapes seen before */
  int eos_token_id;               /* -2: the model's own (config.json), -1: none */
  int want_logprobs;
  int run_ahead;                  /* 1: while every running request just decodes, a step's ids are read one call
                                     later and the next step is queued behind it without the host having seen
                                     them (sglc_engine_step then reports a request's end one call later) */
  int dry_run;                    /* 1: no device at all: configuration, tensor checks, page tables and scheduling
                                     run, tokens come from a fixed formula (for tests on machines without a GPU) */
  const char* library_dir;        /* where the kernel libraries are; null: beside this library */
} sglc_engine_options;

typedef struct sglc_stats {       /* the reference's counters (include/sgl/scheduler.h:19-31) that apply */
  long long prefill_tokens, decode_tokens, n_finished, n_running, n_waiting;
  long long pool_pages, pool_free, n_preempt, prefill_chunk, n_steps, recomputed_tokens;
  long long graph_replays, launches, weight_bytes, cache_bytes, steps_ahead;
  long long step_upload_bytes;    /* what a step copies to the device: its packed arrays (sampler records beside them) */
} sglc_stats;

enum { SGLC_FINISH_NONE = 0, SGLC_FINISH_EOS = 1, SGLC_FINISH_STOP = 2, SGLC_FINISH_LENGTH = 3,
       SGLC_FINISH_CONTEXT = 4, SGLC_FINISH_ABORT = 5 };

void sglc_sampling_default(sglc_sampling* sp);
void sglc_engine_options_default(sglc_engine_options* opt);

/* A model folder (config.json; model.safetensors or model.safetensors.index.json with its shards).
 * Null on failure, with the reason in err (one message that lists missing and unexpected
 * tensors and wrong shapes, if that is what is wrong). */
sglc_engine* sglc_engine_new(const char* model_dir, const sglc_engine_options* opt, char* err, int err_len);
void sglc_engine_free(sglc_engine* e);

/* Queue a request; its id (from 1 up), or -1 if it can never run: no tokens, ids outside the
 * vocabulary, a prompt as long as the model's positions, or prompt + max_new beyond the pool.
 * max_new <= 0 means 16, sp null means greedy. */
long long sglc_engine_submit_ids(sglc_engine* e, const int* ids, int n, int max_new, const sglc_sampling* sp);
/* One scheduler step (a mixed batch: one token for each request past its prompt beside prompt
 * portions).  Returns how many requests finished in it, or -1 (sglc_engine_last_error says why;
 * the cache is as before the step). */
int sglc_engine_step(sglc_engine* e);
/* Requests waiting or running. */
int sglc_engine_nactive(sglc_engine* e);
/* A finished request not yet taken: 1 and its id, generated ids (up to cap of them; *n_tokens is
 * their full count), prompt length and finish reason; 0 if there is none.  With cap < *n_tokens the
 * request is not taken: call again with room; cap < 0 only looks (id, counts and reason are
 * given, nothing is taken).  Any out pointer may be null. */
int sglc_engine_poll(sglc_engine* e, long long* id, int* tokens, int cap, int* n_tokens, int* n_prompt,
                     int* finish_reason);
/* What a request has generated so far (running, or finished and not yet taken): up to cap ids into
 * tokens, returns their full count; -1 if there is no such request.  With run_ahead the ids of the
 * step in flight are not in it yet. */
int sglc_engine_generated(sglc_engine* e, long long id, int* tokens, int cap);
/* Log-probabilities of a finished request's tokens (want_logprobs), before it is taken. */
int sglc_engine_poll_logprobs(sglc_engine* e, long long id, float* out, int cap);
/* End a waiting or running request now; 0, or -1 if there is no such request. */
int sglc_engine_abort(sglc_engine* e, long long id);
void sglc_engine_get_stats(sglc_engine* e, sglc_stats* out);
/* With run_ahead a step may be in flight when sglc_engine_step returns: wait for it and take its
 * ids in.  The requests it ended, or -1. */
int sglc_engine_sync(sglc_engine* e);
/* For measurements: a mark on the stream the steps run on, behind everything queued so far
 * (sync_first: after waiting for it all); the device time in milliseconds between the last two
 * marks (waits for the second), or a negative number.  And: a running request forgets what it has
 * generated beyond its first `keep` ids (keep >= 1; no step in flight), so that the same steps can
 * be timed again; 0, or -1. */
int sglc_engine_mark(sglc_engine* e, int sync_first);
double sglc_engine_ms_between_marks(sglc_engine* e);
int sglc_engine_rewind(sglc_engine* e, long long id, int keep);
/* Steps until nothing is active (at most max_steps); the steps taken, or -1. */
long long sglc_engine_run_until_done(sglc_engine* e, long long max_steps);
/* What the last step ran, in batch order: request ids, their token counts, and whether a token was
 * sampled for them (up to cap entries; returns the number of requests of the step). */
int sglc_engine_last_step(sglc_engine* e, long long* ids, int* n_tokens, int* sampled, int cap);
/* The page tables' invariants (no page lost, held twice or freed twice; slots likewise): 0, or -1
 * with the reason as the last error. */
int sglc_engine_check(sglc_engine* e);
const char* sglc_engine_last_error(sglc_engine* e);
/* For tests: the page tables alone (two cache groups, the second with `window`) under n_ops random
 * operations (requests arrive, grow by portions of any size, are cut back, end), with the
 * invariants checked after each; 0, or -1 with the reason in err.  Needs no device. */
int sglc_pages_selftest(int page_size, int n_pages, int max_requests, int window, unsigned seed, int n_ops,
                        char* err, int err_len);
/* Sizes the model was built with, from config.json. */
int sglc_engine_vocab_size(sglc_engine* e);
int sglc_engine_max_positions(sglc_engine* e);
int sglc_engine_eos_token_id(sglc_engine* e);

#ifdef __cplusplus
}
#endif
#endif
