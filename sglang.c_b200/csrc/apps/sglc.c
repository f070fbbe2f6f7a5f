/* sglc: generate from a model folder through the engine's C interface (sglc_engine.h), in the
 * manner of the reference's one-shot command line (apps/sglc.c:264-312, 486-514): same option
 * names and defaults where it has them.  There is no tokenizer here, so the prompt is token ids.
 *
 *   cc -O2 -I<csrc> sglc.c -o sglc -L<folder of the libraries> -lsglc_host_engine -Wl,-rpath,<that folder>
 *   sglc --model DIR --prompt-ids "464, 3616, 286" [--max-new 32] [--temperature 0.8] [--top-k 50]
 *        [--top-p 0.95] [--min-p 0] [--repetition-penalty 1] [--seed 0] [--ignore-eos] [--verbose]
 *        [--dtype bfloat16|float32] [--device N] [--page-size 16] [--pages N] [--chunk 512]
 *        [--token-budget 2048] [--dry-run]
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "sglc_engine.h"

static double now(void) {
  struct timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

static int parse_ids(const char* text, int** out) {
  int n = 0, cap = 64;
  int* ids = (int*)malloc(sizeof(int) * cap);
  const char* p = text;
  while (*p) {
    while (*p == ' ' || *p == ',' || *p == '\n' || *p == '\t') ++p;
    if (!*p) break;
    char* end;
    long v = strtol(p, &end, 10);
    if (end == p) {
      free(ids);
      return -1;
    }
    if (n == cap) ids = (int*)realloc(ids, sizeof(int) * (cap *= 2));
    ids[n++] = (int)v;
    p = end;
  }
  *out = ids;
  return n;
}

static void usage(void) {
  fprintf(stderr, "usage: sglc --model <dir> --prompt-ids <ids> [--max-new N] [--temperature F] [--top-k N] [--top-p F]\n"
                  "            [--min-p F] [--repetition-penalty F] [--seed N] [--ignore-eos] [--verbose]\n"
                  "            [--dtype bfloat16|float32] [--device N] [--page-size N] [--pages N] [--chunk N]\n"
                  "            [--token-budget N] [--dry-run]\n");
}

int main(int argc, char** argv) {
  const char *model = NULL, *prompt = NULL;
  int max_new = 32, verbose = 0;
  sglc_sampling sp;
  sglc_engine_options opt;
  sglc_sampling_default(&sp);
  sglc_engine_options_default(&opt);
  sp.temperature = 0.8f; sp.top_k = 50; sp.top_p = 0.95f;          /* apps/sglc.c:266-272 */
  opt.max_requests = 4;
  for (int i = 1; i < argc; ++i) {
    const char* a = argv[i];
    const char* v = i + 1 < argc ? argv[i + 1] : NULL;
#define OPT(name) (strcmp(a, name) == 0 && v && ++i)
    if (OPT("--model")) model = v;
    else if (OPT("--prompt") || OPT("--prompt-ids")) prompt = v;
    else if (OPT("--max-new")) max_new = atoi(v);
    else if (OPT("--temperature")) sp.temperature = (float)atof(v);
    else if (OPT("--top-k")) sp.top_k = atoi(v);
    else if (OPT("--top-p")) sp.top_p = (float)atof(v);
    else if (OPT("--min-p")) sp.min_p = (float)atof(v);
    else if (OPT("--repetition-penalty")) sp.repetition_penalty = (float)atof(v);
    else if (OPT("--seed")) { opt.seed = strtoull(v, NULL, 10); sp.seed = opt.seed; }
    else if (OPT("--dtype")) opt.bf16 = !(strcmp(v, "float32") == 0 || strcmp(v, "fp32") == 0);
    else if (OPT("--device")) opt.device = atoi(v);
    else if (OPT("--page-size")) opt.page_size = atoi(v);
    else if (OPT("--pages")) opt.n_pages = atoll(v);
    else if (OPT("--chunk")) opt.prefill_chunk = atoi(v);
    else if (OPT("--token-budget")) opt.max_step_tokens = opt.token_budget = atoi(v);
    else if (strcmp(a, "--ignore-eos") == 0) sp.ignore_eos = 1;
    else if (strcmp(a, "--verbose") == 0) verbose = 1;
    else if (strcmp(a, "--dry-run") == 0) opt.dry_run = 1;
    else {
      fprintf(stderr, "sglc: unknown or incomplete option '%s'\n", a);
      usage();
      return 1;
    }
  }
  if (!model || !prompt) {
    usage();
    return 1;
  }
  int* ids = NULL;
  const int n = parse_ids(prompt, &ids);
  if (n <= 0) {
    fprintf(stderr, "the prompt must be token ids separated by commas or spaces (this engine has no tokenizer)\n");
    return 1;
  }
  if (opt.n_pages == 0) {
    const long long need = (long long)n + max_new + 1;
    opt.max_tokens = (need > 64 ? need : 64) + opt.page_size;
  }
  char err[8192];
  const double t0 = now();
  sglc_engine* e = sglc_engine_new(model, &opt, err, (int)sizeof(err));
  if (!e) {
    fprintf(stderr, "sglc: %s\n", err);
    return 2;
  }
  sglc_stats st;
  sglc_engine_get_stats(e, &st);
  if (verbose)
    fprintf(stderr, "model loaded in %.2fs (%.1f MB of weights, %lld pages of %d)\n", now() - t0,
            (double)st.weight_bytes / 1e6, st.pool_pages, opt.page_size);
  const double t1 = now();
  const long long id = sglc_engine_submit_ids(e, ids, n, max_new, &sp);
  if (id < 0) {
    fprintf(stderr, "sglc: the prompt was refused: ids outside the vocabulary, or prompt + max_new beyond the "
                    "cache pool or the model's positions\n");
    sglc_engine_free(e);
    return 2;
  }
  if (sglc_engine_run_until_done(e, 1 << 30) < 0) {
    fprintf(stderr, "sglc: %s\n", sglc_engine_last_error(e));
    sglc_engine_free(e);
    return 3;
  }
  int* out = (int*)malloc(sizeof(int) * (size_t)(max_new > 0 ? max_new : 16));
  int n_out = 0, reason = 0;
  sglc_engine_poll(e, NULL, out, max_new > 0 ? max_new : 16, &n_out, NULL, &reason);
  const double dt = now() - t1;
  for (int i = 0; i < n; ++i) printf("%d ", ids[i]);
  for (int i = 0; i < n_out; ++i) printf("%d%s", out[i], i + 1 < n_out ? " " : "");
  printf("\n");
  fprintf(stderr, "generated %d tokens in %.2fs (%.1f tok/s, %.0f ms/tok)\n", n_out, dt, dt > 0 ? n_out / dt : 0.0,
          dt * 1000.0 / (n_out > 0 ? n_out : 1));
  if (verbose) {
    sglc_engine_get_stats(e, &st);
    fprintf(stderr, "stats: steps %lld, prefill %lld, decode %lld, launches %lld, graph replays %lld, finish reason %d\n",
            st.n_steps, st.prefill_tokens, st.decode_tokens, st.launches, st.graph_replays, reason);
  }
  free(out);
  free(ids);
  sglc_engine_free(e);
  return 0;
}
