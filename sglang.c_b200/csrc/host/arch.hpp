// A model described as data for the host engine: which tensors make it up, the sizes and
// constants of every layer's parts (all read from the architecture's own config.json keys), and
// the order in which layers run.  An architecture is one function from config.json to this
// description, registered under its `architectures` name and its `model_type`; the engine knows
// none of them.  Only architectures made of the parts the step walker knows (token and learned
// position tables, LayerNorm, causal attention over the paged cache, a GELU feed-forward, pre-norm
// blocks, a linear head) can be described here; anything else runs through the Python engine.
#pragma once
#include <cmath>
#include <string>
#include <vector>

#include "json.hpp"

namespace sglc {

struct LinearSpec {
  std::string weight, bias;       // tensor names (bias empty: none)
  int in = 0, out = 0;
  bool conv1d = false;            // stored [in][out]; the device keeps [out][in]
};
struct NormSpec {
  std::string weight, bias;
  float eps = 0.0f;
  int size = 0;
};
struct LayerSpec {
  NormSpec norm1, norm2;
  LinearSpec qkv, out, up, down;
  int n_heads = 0, n_kv_heads = 0, head_dim = 0, window = 0, inner = 0, act = 0;
  float scale = 1.0f;
};
struct CallSpec {
  int layer = 0;
  int cache_of = -1;              // an earlier call whose cache this one reads; -1: its own
};
struct ModelSpec {
  std::string architecture;
  int hidden = 0, vocab = 0, positions = 0;
  std::string table, pos_table;   // token table [vocab][hidden]; position table [positions][hidden] or empty
  std::vector<LayerSpec> layers;
  std::vector<CallSpec> order;
  NormSpec final_norm;
  LinearSpec head;
  int eos = -1;                   // -1: none
  std::vector<std::string> ignorable;      // patterns ('*' = any run) of tensors a file may carry beyond these
  std::vector<std::string> prefixes;       // tried in turn before every tensor name
};

// ---- typed reads of config.json, each naming the key it refuses ----------------------------------------
struct ConfigReader {
  const Json& j;
  std::string err;
  explicit ConfigReader(const Json& j_) : j(j_) {}
  bool ok() const { return err.empty(); }
  const Json* at(const char* key) const {
    const Json* v = j.get(key);
    return (v && v->kind != Json::Null) ? v : nullptr;
  }
  void fail(const std::string& what) {
    if (err.empty()) err = "config.json: " + what;
  }
  long long integer(const char* key, long long minimum, bool required = true, long long dflt = 0) {
    const Json* v = at(key);
    if (!v) {
      if (required) fail(std::string("key '") + key + "' is required");
      return dflt;
    }
    if (v->kind != Json::Int) return fail(std::string("key '") + key + "' must be an integer"), dflt;
    if (v->i < minimum)
      return fail(std::string("key '") + key + "' must be >= " + std::to_string(minimum) + ", got " + std::to_string(v->i)), dflt;
    return v->i;
  }
  double positive(const char* key) {
    const Json* v = at(key);
    if (!v) return fail(std::string("key '") + key + "' is required"), 1.0;
    if (!v->is_number()) return fail(std::string("key '") + key + "' must be a number"), 1.0;
    if (!(v->number() > 0)) return fail(std::string("key '") + key + "' must be > 0"), 1.0;
    return v->number();
  }
  bool boolean(const char* key, bool dflt) {
    const Json* v = at(key);
    if (!v) return dflt;
    if (v->kind != Json::Bool) return fail(std::string("key '") + key + "' must be true or false"), dflt;
    return v->b;
  }
  std::string text(const char* key, const char* dflt) {
    const Json* v = at(key);
    if (!v) return dflt;
    if (v->kind != Json::Str) return fail(std::string("key '") + key + "' must be a string"), std::string(dflt);
    return v->s;
  }
};

using ArchBuilder = bool (*)(const Json& config, ModelSpec* out, std::string* err);
struct ArchEntry {
  const char* name;               // as in config.json's `architectures`
  const char* model_type;
  ArchBuilder build;
};

// ---- GPT-2 (GPT2LMHeadModel): learned token and position tables, pre-LayerNorm blocks of causal
// multi-head attention and a GELU feed-forward, a final LayerNorm and a head tied to the token
// table (reference src/gpt2.c:210-297; tensor names :61-96, a "transformer." prefix tried second).
// n_inner, activation_function, scale_attn_weights and scale_attn_by_inverse_layer_idx, which
// the reference ignores (src/gpt2.c:60,253), are honoured.
inline bool build_gpt2(const Json& config, ModelSpec* m, std::string* err) {
  ConfigReader c(config);
  const int E = (int)c.integer("n_embd", 1), H = (int)c.integer("n_head", 1);
  const int L = (int)c.integer("n_layer", 1), V = (int)c.integer("vocab_size", 1);
  // the reference prefers n_ctx and falls back to n_positions (src/gpt2.c:40)
  int P = c.at("n_ctx") ? (int)c.integer("n_ctx", 1) : (int)c.integer("n_positions", 1);
  if (c.at("n_ctx") && c.at("n_positions") && c.ok() && c.integer("n_ctx", 1) > c.integer("n_positions", 1))
    c.fail("n_ctx exceeds n_positions (rows of the position table)");
  const int inner = (int)c.integer("n_inner", 1, false, 4LL * E);
  const double eps = c.positive("layer_norm_epsilon");
  const std::string actf = c.text("activation_function", "gelu_new");
  int act = 0;
  if (actf == "gelu_new" || actf == "gelu_pytorch_tanh" || actf == "gelu_fast") act = 1;      // tanh form
  else if (actf == "gelu") act = 2;                                                           // erf form
  else c.fail("key 'activation_function' is '" + actf + "', known values: gelu, gelu_fast, gelu_new, gelu_pytorch_tanh");
  const bool scale_w = c.boolean("scale_attn_weights", true);
  const bool scale_l = c.boolean("scale_attn_by_inverse_layer_idx", false);
  if (!c.boolean("tie_word_embeddings", true))
    c.fail("tie_word_embeddings=false is not supported for GPT2LMHeadModel (the head is the token table)");
  const long long eos = c.integer("eos_token_id", -(1LL << 40), false, -1);
  if (c.ok() && E % H != 0)
    c.fail("n_embd (" + std::to_string(E) + ") is not a multiple of n_head (" + std::to_string(H) + ")");
  if (!c.ok()) return *err = c.err, false;
  const int D = E / H;
  m->architecture = "GPT2LMHeadModel";
  m->hidden = E; m->vocab = V; m->positions = P;
  m->table = "wte.weight";
  m->pos_table = "wpe.weight";
  m->eos = eos >= 0 ? (int)eos : -1;
  for (int l = 0; l < L; ++l) {
    const std::string p = "h." + std::to_string(l) + ".";
    LayerSpec s;
    s.norm1 = {p + "ln_1.weight", p + "ln_1.bias", (float)eps, E};
    s.norm2 = {p + "ln_2.weight", p + "ln_2.bias", (float)eps, E};
    s.qkv = {p + "attn.c_attn.weight", p + "attn.c_attn.bias", E, 3 * E, true};
    s.out = {p + "attn.c_proj.weight", p + "attn.c_proj.bias", E, E, true};
    s.up = {p + "mlp.c_fc.weight", p + "mlp.c_fc.bias", E, inner, true};
    s.down = {p + "mlp.c_proj.weight", p + "mlp.c_proj.bias", inner, E, true};
    s.n_heads = s.n_kv_heads = H;
    s.head_dim = D;
    s.inner = inner;
    s.act = act;
    // 1/sqrt(D) (src/gpt2.c:253) unless scale_attn_weights is off; divided by the layer's
    // number, from 1, when scale_attn_by_inverse_layer_idx is on
    double scale = scale_w ? 1.0 / std::sqrt((double)D) : 1.0;
    if (scale_l) scale /= (double)(l + 1);
    s.scale = (float)scale;
    m->layers.push_back(s);
    m->order.push_back({l, -1});
  }
  m->final_norm = {"ln_f.weight", "ln_f.bias", (float)eps, E};
  m->head = {"wte.weight", "", E, V, false};
  m->ignorable = {"lm_head.weight", "h.*.attn.bias", "h.*.attn.masked_bias"};
  m->prefixes = {"", "transformer."};
  return true;
}

inline const std::vector<ArchEntry>& architectures() {
  static const std::vector<ArchEntry> all = {{"GPT2LMHeadModel", "gpt2", build_gpt2}};
  return all;
}

// `architectures` first, then `model_type`; an unknown one lists the known
inline bool resolve_architecture(const Json& config, ModelSpec* out, std::string* err) {
  const Json* names = config.get("architectures");
  const Json* mt = config.get("model_type");
  std::vector<std::string> asked;
  if (names && names->kind == Json::Arr)
    for (const Json& n : names->arr)
      if (n.kind == Json::Str) asked.push_back(n.s);
  if (names && names->kind == Json::Str) asked.push_back(names->s);
  for (const std::string& n : asked)
    for (const ArchEntry& a : architectures())
      if (n == a.name) return a.build(config, out, err);
  if (mt && mt->kind == Json::Str)
    for (const ArchEntry& a : architectures())
      if (mt->s == a.model_type) return a.build(config, out, err);
  std::string known, got;
  for (const ArchEntry& a : architectures()) known += (known.empty() ? "" : ", ") + std::string(a.name);
  for (const std::string& n : asked) got += (got.empty() ? "" : ", ") + n;
  *err = "config.json names architectures=[" + got + "], model_type=" + (mt && mt->kind == Json::Str ? mt->s : "none") +
         "; known architectures: " + known;
  return false;
}

// '*' matches any run of characters (what fnmatch does for the patterns used here)
inline bool glob_match(const char* pat, const char* s) {
  if (!*pat) return !*s;
  if (*pat == '*') {
    for (const char* t = s;; ++t) {
      if (glob_match(pat + 1, t)) return true;
      if (!*t) return false;
    }
  }
  return *s && *pat == *s && glob_match(pat + 1, s + 1);
}

}  // namespace sglc
