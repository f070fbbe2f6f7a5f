// The engine behind the C interface of sglc_engine.h, all of it native: it reads config.json and
// the safetensors files of a model folder, builds the model the architecture registry describes
// (host/arch.hpp), puts the weights on the device in the runtime's precision, keeps the page
// tables (host/pages.hpp) and the scheduler (host/sched.hpp), packs each step's arrays into one
// pinned block that goes to the device in one copy, has the step walker (step_walker.cu) make the
// step's launches, or replays the CUDA graph of a step shape seen before, and samples on the
// device.  It launches the same kernels through the same launchers as the Python engine and
// chooses among them in the same way, so both give the same logits bit for bit.
//
// The reference's counterpart is its C scheduler above sgl_model_prefill / sgl_model_decode_batch
// (src/scheduler.c:454-523, include/sgl/model.h:29-35) with the weights uploaded by
// sgl_cuda_from_gpt2 (src/cuda_backend.cu:5243-5330).
//
// This file has no kernels of its own; it is compiled with the others so that it lies beside
// the libraries it loads.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"

#include "host/arch.hpp"
#include "host/json.hpp"
#include "host/pages.hpp"
#include "host/safetensors.hpp"
#include "host/sched.hpp"
#include "sglc_engine.h"
#include "step_walker.h"

SGLC_DEFINE_ERROR_STRING()

namespace {
using namespace sglc;

// constants the Python engine shares (csrc/ops.py)
constexpr long long TC_WS_FLOATS = 8ll << 20;      // split-K partial sums of the decode attention's merge
constexpr int TC_COUNTERS = 8192;
constexpr int STREAM_MIN_ITEMS = 160;              // (token, head) items from which the streaming decode kernel is used
constexpr int FEW_MAX_TOKENS = 2;
constexpr long long FEW_MAX_WEIGHT = 3ll << 20;
constexpr int ORDER_SPREAD = 64;                   // contexts that differ by a stage of keys: their order matters
constexpr int MAX_GRAPHS = 96;                     // (a step shape has a graph for each of the two turns of its arrays)

std::string fmt(const char* f, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, f);
  vsnprintf(buf, sizeof(buf), f, ap);
  va_end(ap);
  return buf;
}

// ---- element conversions (on the host, once per tensor at load) -------------------------------------
inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {             // round to nearest, ties to even; NaN stays NaN
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {                                          // subnormal: renormalise
      exp = 127 - 15 + 1;
      while (!(man & 0x400u)) { man <<= 1; --exp; }
      u = sign | (exp << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
  else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline float element_f32(const TensorView& t, long long i) {
  const uint8_t* p = t.data;
  if (t.dtype == "F32") { float f; memcpy(&f, p + 4 * i, 4); return f; }
  if (t.dtype == "BF16") { uint16_t h; memcpy(&h, p + 2 * i, 2); return bf16_to_f32(h); }
  if (t.dtype == "F16") { uint16_t h; memcpy(&h, p + 2 * i, 2); return f16_to_f32(h); }
  double d; memcpy(&d, p + 8 * i, 8); return (float)d;            // F64
}

// ---- the kernel libraries ----------------------------------------------------------------------------
typedef int (*fn_walker_names)(const char* const**);
typedef int (*fn_walker_bind)(void* const*, int);
typedef int (*fn_walker_sizes)(int*);
typedef int (*fn_walker_forward)(const WalkModel*, WalkStep*);
typedef const char* (*fn_error_string)(int);
typedef int (*fn_sample)(float*, int, int, int, const void*, const int*, const int*, int*, float*, cudaStream_t);

// which library a launcher lives in (engine/host_model.py has the same table)
const char* const LAUNCHER_LIB[][2] = {
    {"sglc_embed", "embed"}, {"sglc_layernorm", "layernorm"}, {"sglc_gemm_simt", "gemm_simt"},
    {"sglc_gemm_tc", "gemm_tc"}, {"sglc_gemm_tc_kv", "gemm_tc"}, {"sglc_gemm_few_supports", "gemm_few"}, {"sglc_gemm_few", "gemm_few"},
    {"sglc_kv_write", "kv_cache"}, {"sglc_attention_simt", "attention_simt"},
    {"sglc_attention_prefill_tc", "attention_prefill_tc"}, {"sglc_attention_decode_splits", "attention_decode"},
    {"sglc_attention_decode_scratch", "attention_decode"}, {"sglc_attention_decode", "attention_decode"},
    {"sglc_attention_decode_tma", "attention_decode_tma"},
    {"sglc_attention_decode_stream_supports", "attention_decode_tma"},
    {"sglc_attention_decode_stream", "attention_decode_tma"}};

struct Kernels {
  fn_walker_forward forward = nullptr;
  fn_error_string walker_error = nullptr;
  fn_sample sample = nullptr;
  std::map<std::string, void*> libs;

  void* lib(const std::string& dir, const std::string& name, std::string* err) {
    auto it = libs.find(name);
    if (it != libs.end()) return it->second;
    const std::string path = dir + "/libsglc_" + name + ".so";
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) {
      *err = "kernel library " + path + " cannot be loaded (" + (dlerror() ?: "?") +
             "); this engine has no CPU path: build the libraries first (python -c \"import __graft_entry__ as g; g.build()\")";
      return nullptr;
    }
    libs[name] = h;
    return h;
  }
  void* sym(const std::string& dir, const char* lib_name, const char* fn, std::string* err) {
    void* h = lib(dir, lib_name, err);
    if (!h) return nullptr;
    void* s = dlsym(h, fn);
    if (!s) *err = std::string("library libsglc_") + lib_name + ".so has no " + fn + " (stale build?)";
    return s;
  }
  bool load(const std::string& dir, std::string* err) {
    auto names = (fn_walker_names)sym(dir, "step_walker", "sglc_walker_names", err);
    auto bind = (fn_walker_bind)sym(dir, "step_walker", "sglc_walker_bind", err);
    auto sizes = (fn_walker_sizes)sym(dir, "step_walker", "sglc_walker_struct_sizes", err);
    forward = (fn_walker_forward)sym(dir, "step_walker", "sglc_walker_forward", err);
    walker_error = (fn_error_string)sym(dir, "step_walker", "sglc_error_string", err);
    sample = (fn_sample)sym(dir, "sampling", "sglc_sample", err);
    if (!names || !bind || !sizes || !forward || !walker_error || !sample) return false;
    int sz[6];
    sizes(sz);
    const int mine[6] = {(int)sizeof(WalkLinear), (int)sizeof(WalkNorm), (int)sizeof(WalkLayer),
                         (int)sizeof(WalkCall), (int)sizeof(WalkModel), (int)sizeof(WalkStep)};
    if (memcmp(sz, mine, sizeof(mine)) != 0) return *err = "step walker: structure sizes differ (stale build?)", false;
    const char* const* wanted = nullptr;
    const int n = names(&wanted);
    std::vector<void*> fns;
    for (int i = 0; i < n; ++i) {
      const char* lib_name = nullptr;
      for (const auto& row : LAUNCHER_LIB)
        if (strcmp(row[0], wanted[i]) == 0) lib_name = row[1];
      if (!lib_name) return *err = std::string("step walker asks for unknown launcher ") + wanted[i], false;
      void* s = sym(dir, lib_name, wanted[i], err);
      if (!s) return false;
      fns.push_back(s);
    }
    if (bind(fns.data(), n) != 0) return *err = "step walker: binding the launchers failed", false;
    return true;
  }
};

std::string own_directory() {
  Dl_info info;
  if (dladdr((void*)&own_directory, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    const size_t k = p.rfind('/');
    return k == std::string::npos ? "." : p.substr(0, k);
  }
  return ".";
}

// ---- the model on the device -----------------------------------------------------------------------------
struct DeviceModel {
  ModelSpec spec;
  WalkModel wm = {};
  std::vector<WalkLayer> layers;
  std::vector<WalkCall> order;
  std::vector<int> group_of_call;           // cache group of each call of the running order
  std::vector<int> windows;                 // per cache group
  std::vector<void*> allocs;
  long long weight_bytes = 0, cache_bytes = 0, largest_layer_matrix = 0;
  bool on_device = false;

  ~DeviceModel() {
    for (void* p : allocs) cudaFree(p);
  }
};

struct Want {
  std::string name;
  std::vector<long long> shape;
};

void add_linear(const LinearSpec& l, std::vector<Want>* w) {
  if (l.conv1d) w->push_back({l.weight, {l.in, l.out}});
  else w->push_back({l.weight, {l.out, l.in}});
  if (!l.bias.empty()) w->push_back({l.bias, {l.out}});
}
void add_norm(const NormSpec& n, std::vector<Want>* w) {
  w->push_back({n.weight, {n.size}});
  w->push_back({n.bias, {n.size}});
}
std::string shape_text(const std::vector<long long>& s) {
  std::string t = "[";
  for (size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
  return t + "]";
}

// The file against the model: one message that lists missing and unexpected tensors and wrong
// shapes or types.  On success `actual` maps each declared name to the name it has in the file.
bool check_tensors(const ModelSpec& m, const Checkpoint& ck, std::map<std::string, std::string>* actual,
                   std::string* err) {
  std::vector<Want> wants;
  wants.push_back({m.table, {m.vocab, m.hidden}});
  if (!m.pos_table.empty()) wants.push_back({m.pos_table, {m.positions, m.hidden}});
  for (const LayerSpec& l : m.layers) {
    add_norm(l.norm1, &wants);
    add_linear(l.qkv, &wants);
    add_linear(l.out, &wants);
    add_norm(l.norm2, &wants);
    add_linear(l.up, &wants);
    add_linear(l.down, &wants);
  }
  add_norm(m.final_norm, &wants);
  add_linear(m.head, &wants);
  std::vector<std::string> missing, wrong;
  std::map<std::string, bool> used;
  for (const Want& w : wants) {
    if (actual->count(w.name)) continue;                          // (the tied head names the token table again)
    const TensorView* t = nullptr;
    std::string found;
    for (const std::string& p : m.prefixes)
      if ((t = ck.find(p + w.name)) != nullptr) {
        found = p + w.name;
        break;
      }
    if (!t) {
      if (std::find(missing.begin(), missing.end(), w.name) == missing.end()) missing.push_back(w.name);
      continue;
    }
    (*actual)[w.name] = found;
    used[found] = true;
    if (t->shape != w.shape)
      wrong.push_back(found + ": file has " + shape_text(t->shape) + ", model needs " + shape_text(w.shape));
    else if (!t->floating())
      wrong.push_back(found + ": file has " + t->dtype + ", model needs a floating-point tensor");
  }
  std::vector<std::string> unexpected;
  for (const std::string& n : ck.names()) {
    if (used.count(n)) continue;
    std::string bare = n;
    for (const std::string& p : m.prefixes)
      if (!p.empty() && n.compare(0, p.size(), p) == 0) bare = n.substr(p.size());
    bool ignore = false;
    for (const std::string& pat : m.ignorable) ignore = ignore || glob_match(pat.c_str(), bare.c_str());
    if (!ignore) unexpected.push_back(n);
  }
  if (missing.empty() && wrong.empty() && unexpected.empty()) return true;
  std::sort(missing.begin(), missing.end());
  std::sort(unexpected.begin(), unexpected.end());
  auto join = [](const std::vector<std::string>& v) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
    return s;
  };
  *err = ck.where() + " does not fit the model:";
  if (!missing.empty()) *err += "\n  missing tensors (" + std::to_string(missing.size()) + "): " + join(missing);
  if (!unexpected.empty())
    *err += "\n  unexpected tensors (" + std::to_string(unexpected.size()) + "): " + join(unexpected);
  if (!wrong.empty()) {
    *err += "\n  wrong shape or type (" + std::to_string(wrong.size()) + "):";
    for (const std::string& w : wrong) *err += "\n    " + w;
  }
  return false;
}

class Uploader {
 public:
  Uploader(DeviceModel* dm, const Checkpoint* ck, const std::map<std::string, std::string>* actual, bool bf16)
      : dm_(dm), ck_(ck), actual_(actual), bf16_(bf16) {}
  std::string err;

  // a 2-D weight in the runtime's matrix precision, [out][in] on the device
  const void* matrix(const std::string& name, bool transpose) {
    const std::string key = name + (transpose ? "|T" : "|M");
    auto it = done_.find(key);
    if (it != done_.end()) return it->second;
    const TensorView* t = ck_->find(actual_->at(name));
    const long long rows = t->shape[0], cols = t->shape[1], n = rows * cols;
    const int es = bf16_ ? 2 : 4;
    stage_.resize((size_t)n * es);
    auto put = [&](long long dst, float v) {
      if (bf16_) {
        const uint16_t h = f32_to_bf16(v);
        memcpy(&stage_[(size_t)dst * 2], &h, 2);
      } else {
        memcpy(&stage_[(size_t)dst * 4], &v, 4);
      }
    };
    if (!transpose) {
      const bool same = (bf16_ && t->dtype == "BF16") || (!bf16_ && t->dtype == "F32");
      if (same) memcpy(stage_.data(), t->data, (size_t)n * es);
      else
        for (long long i = 0; i < n; ++i) put(i, element_f32(*t, i));
    } else {
      // file [rows = in][cols = out] -> device [out][in], in tiles that stay in the cache
      constexpr long long B = 64;
      for (long long r0 = 0; r0 < rows; r0 += B)
        for (long long c0 = 0; c0 < cols; c0 += B)
          for (long long r = r0; r < std::min(rows, r0 + B); ++r)
            for (long long c = c0; c < std::min(cols, c0 + B); ++c) put(c * rows + r, element_f32(*t, r * cols + c));
    }
    return done_[key] = to_device((size_t)n * es);
  }
  const float* vector(const std::string& name) {
    if (name.empty()) return nullptr;
    const std::string key = name + "|V";
    auto it = done_.find(key);
    if (it != done_.end()) return (const float*)it->second;
    const TensorView* t = ck_->find(actual_->at(name));
    const long long n = t->numel();
    stage_.resize((size_t)n * 4);
    for (long long i = 0; i < n; ++i) {
      const float v = element_f32(*t, i);
      memcpy(&stage_[(size_t)i * 4], &v, 4);
    }
    return (const float*)(done_[key] = to_device((size_t)n * 4));
  }

 private:
  void* to_device(size_t bytes) {
    void* d = nullptr;
    if (!err.empty()) return nullptr;
    cudaError_t e = cudaMalloc(&d, bytes ? bytes : 1);
    if (e == cudaSuccess) {
      dm_->allocs.push_back(d);
      e = cudaMemcpy(d, stage_.data(), bytes, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
      err = std::string("putting the weights on the device failed: ") + cudaGetErrorString(e);
      return nullptr;
    }
    dm_->weight_bytes += (long long)bytes;
    return d;
  }
  DeviceModel* dm_;
  const Checkpoint* ck_;
  const std::map<std::string, std::string>* actual_;
  bool bf16_;
  std::vector<uint8_t> stage_;
  std::map<std::string, void*> done_;
};

WalkLinear make_linear(Uploader* up, const LinearSpec& l, bool device) {
  WalkLinear w = {};
  w.N = l.out;
  w.K = l.in;
  if (device) {
    w.w = up->matrix(l.weight, l.conv1d);
    w.bias = up->vector(l.bias);
  }
  return w;
}
WalkNorm make_norm(Uploader* up, const NormSpec& n, bool device) {
  WalkNorm w = {};
  w.eps = n.eps;
  w.size = n.size;
  if (device) {
    w.gamma = up->vector(n.weight);
    w.beta = up->vector(n.bias);
  }
  return w;
}

// config.json -> the architecture's description -> tensors checked -> (unless dry) weights and
// cache on the device, described for the walker
bool load_model(const std::string& dir, bool bf16, bool device, int page_size, long long n_pages, DeviceModel* dm,
                std::string* err) {
  std::string text;
  if (!read_text_file(dir + "/config.json", &text)) return *err = "no config.json in " + dir, false;
  Json config;
  std::string jerr;
  if (!json_parse(text, &config, &jerr)) return *err = dir + "/config.json: not valid JSON (" + jerr + ")", false;
  if (config.kind != Json::Obj) return *err = dir + "/config.json: top level must be an object", false;
  if (!resolve_architecture(config, &dm->spec, err)) return false;
  const ModelSpec& m = dm->spec;
  for (size_t i = 0; i < m.order.size(); ++i) {
    if (m.order[i].layer < 0 || m.order[i].layer >= (int)m.layers.size())
      return *err = fmt("running order entry %d names layer %d, which does not exist", (int)i, m.order[i].layer), false;
    if (m.order[i].cache_of >= (int)i)
      return *err = fmt("running order entry %d reads the cache of entry %d, which must come earlier", (int)i,
                        m.order[i].cache_of), false;
  }
  Checkpoint ck;
  if (!ck.open(dir, err)) return false;
  std::map<std::string, std::string> actual;
  if (!check_tensors(m, ck, &actual, err)) return false;

  // cache groups: calls whose needs are equal (heads, head size, window) share a pool of pages
  std::vector<std::tuple<int, int, int>> needs;
  dm->group_of_call.assign(m.order.size(), -1);
  for (size_t i = 0; i < m.order.size(); ++i) {
    const int owner = m.order[i].cache_of >= 0 ? m.order[i].cache_of : (int)i;
    const LayerSpec& L = m.layers[m.order[owner].layer];
    const LayerSpec& mine = m.layers[m.order[i].layer];
    if (mine.n_kv_heads != L.n_kv_heads || mine.head_dim != L.head_dim || mine.window != L.window)
      return *err = fmt("call %d reads the cache of call %d but their needs differ", (int)i, owner), false;
    if (owner != (int)i) {
      dm->group_of_call[i] = dm->group_of_call[owner];
      continue;
    }
    const auto need = std::make_tuple(L.n_kv_heads, L.head_dim, L.window);
    size_t g = std::find(needs.begin(), needs.end(), need) - needs.begin();
    if (g == needs.size()) {
      needs.push_back(need);
      dm->windows.push_back(L.window);
    }
    dm->group_of_call[i] = (int)g;
  }

  Uploader up(dm, &ck, &actual, bf16);
  const int es = bf16 ? 2 : 4;
  for (const LayerSpec& l : m.layers) {
    WalkLayer w = {};
    w.norm1 = make_norm(&up, l.norm1, device);
    w.norm2 = make_norm(&up, l.norm2, device);
    w.qkv = make_linear(&up, l.qkv, device);
    w.out = make_linear(&up, l.out, device);
    w.up = make_linear(&up, l.up, device);
    w.down = make_linear(&up, l.down, device);
    w.n_heads = l.n_heads; w.n_kv_heads = l.n_kv_heads; w.head_dim = l.head_dim; w.window = l.window;
    w.scale = l.scale; w.act = l.act; w.inner_size = l.inner;
    dm->layers.push_back(w);
    for (const LinearSpec* s : {&l.qkv, &l.out, &l.up, &l.down})
      dm->largest_layer_matrix = std::max(dm->largest_layer_matrix, (long long)s->in * s->out);
  }
  for (size_t i = 0; i < m.order.size(); ++i) {
    WalkCall c = {};
    c.layer = m.order[i].layer;
    c.group = dm->group_of_call[i];
    c.write = m.order[i].cache_of < 0;
    c.n_pages = (int)n_pages;
    if (device) {
      if (c.write) {
        const LayerSpec& L = m.layers[c.layer];
        const size_t bytes = (size_t)n_pages * 2 * L.n_kv_heads * page_size * L.head_dim * es;
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, bytes);
        if (e == cudaSuccess) {
          dm->allocs.push_back(d);
          e = cudaMemset(d, 0, bytes);
        }
        if (e != cudaSuccess)
          return *err = fmt("the cache of %lld pages does not fit the device (%s)", n_pages, cudaGetErrorString(e)), false;
        dm->cache_bytes += (long long)bytes;
        c.cache = d;
      } else {
        c.cache = dm->order[m.order[i].cache_of].cache;
      }
    }
    dm->order.push_back(c);
  }
  WalkModel& wm = dm->wm;
  if (device) {
    wm.table = up.matrix(m.table, false);
    wm.pos_table = m.pos_table.empty() ? nullptr : up.matrix(m.pos_table, false);
  }
  wm.final_norm = make_norm(&up, m.final_norm, device);
  wm.head = make_linear(&up, m.head, device);
  if (!up.err.empty()) return *err = up.err, false;
  wm.layers = dm->layers.data();
  wm.order = dm->order.data();
  wm.vocab = m.vocab; wm.n_positions = m.positions; wm.hidden = m.hidden;
  wm.n_layers = (int)dm->layers.size(); wm.n_calls = (int)dm->order.size();
  wm.bf16 = bf16 ? 1 : 0; wm.page_size = page_size;
  dm->on_device = device;
  return true;
}

// ---- a step without a device: tokens from a formula, so that scheduling can be tested anywhere ---------
class DryRunner : public StepRunner {
 public:
  explicit DryRunner(int vocab) : vocab_(vocab) {}
  bool launch(const std::vector<StepItem>& items, const std::vector<double>&, bool want_logprobs, bool, int* ticket,
              std::string*) override {
    tokens_[turn_].clear();
    logprobs_[turn_].clear();
    for (const StepItem& it : items)
      if (it.sampled) {
        tokens_[turn_].push_back((int)(((long long)it.r->id * 7919 + (long long)(it.old_len + it.n) * 104729) % vocab_));
        if (want_logprobs) logprobs_[turn_].push_back(0.0f);
      }
    *ticket = turn_;
    turn_ ^= 1;
    return true;
  }
  bool collect(int ticket, std::vector<int>* tokens, std::vector<float>* logprobs, std::string*) override {
    *tokens = tokens_[ticket];
    *logprobs = logprobs_[ticket];
    return true;
  }

 private:
  int vocab_, turn_ = 0;
  std::vector<int> tokens_[2];
  std::vector<float> logprobs_[2];
};

// ---- a step on the device ------------------------------------------------------------------------------------
#define CU(call)                                                                      \
  do {                                                                                \
    cudaError_t e_ = (call);                                                          \
    if (e_ != cudaSuccess) {                                                          \
      *err = std::string(#call) + ": " + cudaGetErrorString(e_);                      \
      return false;                                                                   \
    }                                                                                 \
  } while (0)

struct Field {
  int off = 0, n = 0;
};

class DeviceRunner : public StepRunner {
 public:
  DeviceRunner(const DeviceModel* dm, const CacheTables* cache, const Kernels* k, const sglc_engine_options& o)
      : dm_(dm), cache_(cache), k_(k), opt_(o) {}
  ~DeviceRunner() override {
    for (cudaStream_t st : {stream_, up_stream_, down_stream_})
      if (st) cudaStreamSynchronize(st);                  // a step may still be in flight
    for (int i = 0; i < 2; ++i)
      for (cudaEvent_t ev : {done_[i], uploaded_[i], ran_[i], marks_[i]})
        if (ev) cudaEventDestroy(ev);
    for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second.exec);
    for (void* p : dev_) cudaFree(p);
    for (void* p : pinned_) cudaFreeHost(p);
    for (cudaStream_t st : {stream_, up_stream_, down_stream_})
      if (st) cudaStreamDestroy(st);
  }
  long long graph_replays = 0, launches = 0;
  long long upload_bytes() const { return (long long)total_ * 4; }
  // a mark on the stream the steps run on (behind everything queued so far); the device time
  // between the last two marks
  bool mark(bool sync_first, std::string* err) {
    if (!marks_[0]) {
      CU(cudaEventCreate(&marks_[0]));
      CU(cudaEventCreate(&marks_[1]));
    }
    if (sync_first) CU(cudaStreamSynchronize(stream_));
    std::swap(marks_[0], marks_[1]);
    CU(cudaEventRecord(marks_[1], stream_));
    ++n_marks_;
    return true;
  }
  double ms_between_marks() {
    if (n_marks_ < 2 || cudaEventSynchronize(marks_[1]) != cudaSuccess) return -1.0;
    float ms = -1.0f;
    return cudaEventElapsedTime(&ms, marks_[0], marks_[1]) == cudaSuccess ? (double)ms : -1.0;
  }

  bool init(std::string* err) {
    const WalkModel& wm = dm_->wm;
    // The kernels of the steps run back to back on one stream; a step's arrays go up and its ids
    // come down on two others, so that the copies of the step queued ahead lie beside the step in
    // flight, not between two steps.  Everything a step uploads exists twice, taken in turn.
    CU(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    CU(cudaStreamCreateWithFlags(&up_stream_, cudaStreamNonBlocking));
    CU(cudaStreamCreateWithFlags(&down_stream_, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      CU(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming));
      CU(cudaEventCreateWithFlags(&uploaded_[i], cudaEventDisableTiming));
      CU(cudaEventCreateWithFlags(&ran_[i], cudaEventDisableTiming));
    }
    t_cap_ = opt_.max_step_tokens;
    r_cap_ = opt_.max_requests;
    b_cap_ = (wm.n_positions + opt_.page_size - 1) / opt_.page_size;
    n_groups_ = (int)dm_->windows.size();
    // the packed block of a step, fields 16-byte aligned (the layout engine/step.py packs)
    int off = 0;
    auto field = [&](int n) {
      Field f{off, n};
      off += (n + 3) & ~3;
      return f;
    };
    f_tokens_ = field(t_cap_); f_positions_ = field(t_cap_); f_token_req_ = field(t_cap_); f_want_ = field(t_cap_);
    f_decode_ = field(r_cap_); f_q_start_ = field(r_cap_ + 1); f_kv_len_ = field(r_cap_); f_state_ = field(r_cap_);
    for (int g = 0; g < n_groups_; ++g) {
      f_slots_.push_back(field(t_cap_));
      f_bt_.push_back(field(r_cap_ * b_cap_));
    }
    total_ = off;
    for (int i = 0; i < 2; ++i) {
      if (!pinned((void**)&h_blk_[i], (size_t)total_ * 4, err) || !device((void**)&d_blk_[i], (size_t)total_ * 4, err))
        return false;
      memset(h_blk_[i], 0, (size_t)total_ * 4);
      CU(cudaMemset(d_blk_[i], 0, (size_t)total_ * 4));
    }
    // the step workspace: what the parts take per token (the 32-bit residual stream, the widest
    // layer's buffers, the final norm's rows), rounded up for the 256-byte alignment of the pieces
    const long long es = wm.bf16 ? 2 : 4, E = wm.hidden;
    long long widest = 0;
    for (const WalkLayer& L : dm_->layers)
      widest = std::max(widest, es * E + std::max(es * (2LL * L.n_heads + 2LL * L.n_kv_heads) * L.head_dim,
                                                  es * (long long)L.inner_size));
    const long long per_token = 4 * E + widest + es * E;
    ws_bytes_ = (long long)((double)per_token * 1.02) * t_cap_ + (8ll << 20);
    if (!device((void**)&ws_, (size_t)ws_bytes_, err)) return false;
    logit_rows_ = std::max(r_cap_, 64);
    if (!device((void**)&logits_, (size_t)logit_rows_ * wm.vocab * 4, err)) return false;
    // the two error words and the sampled ids of a step lie together (one copy brings both back),
    // once per turn: a step's ids are still being read (by the copy down, and by the next step's
    // embedding) when the step after the next samples
    if (!device((void**)&tc_ws_, (size_t)TC_WS_FLOATS * 4, err) || !device((void**)&tc_counters_, TC_COUNTERS * 4, err))
      return false;
    CU(cudaMemset(tc_counters_, 0, TC_COUNTERS * 4));
    for (int i = 0; i < 2; ++i) {
      if (!device((void**)&d_res_[i], (size_t)(4 + r_cap_) * 4, err) || !device((void**)&d_logprob_[i], (size_t)r_cap_ * 4, err))
        return false;
      CU(cudaMemset(d_res_[i], 0, (size_t)(4 + r_cap_) * 4));
    }
    // the sampler's records and results; the host's copies twice, taken in turn: a launch may
    // follow before the last one's results are read
    for (int i = 0; i < 2; ++i) {
      if (!device((void**)&d_params_[i], (size_t)r_cap_ * 40, err) || !pinned((void**)&h_params_[i], (size_t)r_cap_ * 40, err) || !pinned((void**)&h_flags_[i], (size_t)(4 + r_cap_) * 4, err) ||
          !pinned((void**)&h_logprob_[i], (size_t)r_cap_ * 4, err))
        return false;
      h_out_[i] = h_flags_[i] + 4;
    }
    hist_cap_ = 4096;
    if (!device((void**)&d_hist_tok_, (size_t)hist_cap_ * 4, err) || !device((void**)&d_hist_cnt_, (size_t)hist_cap_ * 4, err) ||
        !pinned((void**)&h_hist_, (size_t)hist_cap_ * 8, err))
      return false;
    bts_.resize(n_groups_);
    slots_.resize(n_groups_);
    few_ok_ = dm_->largest_layer_matrix > 0 && dm_->largest_layer_matrix <= FEW_MAX_WEIGHT;
    return true;
  }

  bool launch(const std::vector<StepItem>& items, const std::vector<double>& uniforms, bool want_logprobs,
              bool ids_on_device, int* ticket, std::string* err) override {
    const int R = (int)items.size(), ps = opt_.page_size;
    int T = 0;
    for (const StepItem& it : items) T += it.n;
    if (T > t_cap_ || R > r_cap_) return *err = fmt("a step of %d tokens of %d requests exceeds the engine's sizes", T, R), false;
    const int turn = turn_;
    if (used_[turn]) CU(cudaEventSynchronize(uploaded_[turn]));     // this turn's last upload has left the pinned block
    int* const h_ = h_blk_[turn];
    int* const d_ = d_blk_[turn];
    int *tok = h_ + f_tokens_.off, *pos = h_ + f_positions_.off, *trq = h_ + f_token_req_.off, *wr = h_ + f_want_.off;
    int *dtk = h_ + f_decode_.off, *qs = h_ + f_q_start_.off, *kl = h_ + f_kv_len_.off, *ss = h_ + f_state_.off;
    int t0 = 0, nw = 0, n_decode = 0, max_keys = 0, max_q = 0, min_len = 1 << 30;
    for (int r = 0; r < R; ++r) {
      const StepItem& it = items[r];
      const int o = it.old_len, n = it.n;
      for (int j = 0; j < n; ++j) {
        tok[t0 + j] = ids_on_device ? 0 : it.r->token(o + j);
        pos[t0 + j] = o + j;
        trq[t0 + j] = r;
      }
      if (n == 1) dtk[n_decode++] = t0;
      qs[r] = t0;
      kl[r] = o + n;
      ss[r] = cache_->slot(it.r->id);
      if (it.sampled) wr[nw++] = t0 + n - 1;
      for (int g = 0; g < n_groups_; ++g) {
        const std::vector<int>& table = cache_->table(g, it.r->id);
        int* bt = h_ + f_bt_[g].off + (size_t)r * b_cap_;
        memcpy(bt, table.data(), table.size() * sizeof(int));
        int* sl = h_ + f_slots_[g].off;
        for (int j = 0; j < n; ++j) sl[t0 + j] = table[(o + j) / ps] * ps + (o + j) % ps;
      }
      max_keys = std::max(max_keys, o + n);
      min_len = std::min(min_len, o + n);
      max_q = std::max(max_q, n);
      t0 += n;
    }
    qs[R] = t0;
    if (n_decode > 1)          // single tokens in the order of their contexts, longest first
      std::stable_sort(dtk, dtk + n_decode, [&](int a, int b) { return pos[a] > pos[b]; });
    // up: after the step that last read this turn's device block (two launches ago) has run
    if (used_[turn]) CU(cudaStreamWaitEvent(up_stream_, ran_[turn], 0));
    CU(cudaMemcpyAsync(d_, h_, (size_t)total_ * 4, cudaMemcpyHostToDevice, up_stream_));
    if (nw > 0 && !sample_records(items, uniforms, nw, turn, err)) return false;
    CU(cudaEventRecord(uploaded_[turn], up_stream_));
    CU(cudaStreamWaitEvent(stream_, uploaded_[turn], 0));
    used_[turn] = true;

    WalkStep s = {};
    // (ids_on_device: what the launch before this one sampled, row for row, read where its
    // sampler left it: the other turn's result words)
    s.tokens = ids_on_device ? d_res_[turn ^ 1] + 4 : d_ + f_tokens_.off; s.positions = d_ + f_positions_.off; s.token_req = d_ + f_token_req_.off;
    s.want_rows = d_ + f_want_.off; s.q_start = d_ + f_q_start_.off; s.kv_len = d_ + f_kv_len_.off;
    s.decode_tokens = d_ + f_decode_.off;
    for (int g = 0; g < n_groups_; ++g) {
      bts_[g] = d_ + f_bt_[g].off;
      slots_[g] = d_ + f_slots_[g].off;
    }
    s.block_tables = bts_.data();
    s.slots = slots_.data();
    s.bt_stride = b_cap_;
    s.workspace = ws_; s.workspace_bytes = ws_bytes_;
    s.logits = logits_;
    s.err_flag = d_res_[turn]; s.tc_err = d_res_[turn] + 1;
    s.tc_ws = tc_ws_; s.tc_ws_floats = TC_WS_FLOATS; s.tc_counters = tc_counters_; s.tc_n_counters = TC_COUNTERS;
    s.T = T; s.R = R; s.n_want = nw; s.max_q_len = max_q; s.max_keys = max_keys; s.n_decode = n_decode;
    s.decode_ordered = (n_decode == T && R > 1 && max_keys - min_len >= ORDER_SPREAD) ? 1 : 0;
    s.few_ok = few_ok_ ? 1 : 0;
    s.stream_min_items = STREAM_MIN_ITEMS; s.use_tma_decode = 1;
    s.few_max_tokens = FEW_MAX_TOKENS; s.few_max_weight = FEW_MAX_WEIGHT;
    s.stream = stream_;
    // the step's kernels and, behind them in the same launch or graph, the sampler: one token for
    // every wanted row
    if (!forward(&s, ids_on_device, turn, want_logprobs, err)) return false;
    CU(cudaEventRecord(ran_[turn], stream_));
    // down: ids and the error words in one copy, beside the next step
    CU(cudaStreamWaitEvent(down_stream_, ran_[turn], 0));
    if (nw > 0 && want_logprobs)
      CU(cudaMemcpyAsync(h_logprob_[turn], d_logprob_[turn], (size_t)nw * 4, cudaMemcpyDeviceToHost, down_stream_));
    CU(cudaMemcpyAsync(h_flags_[turn], d_res_[turn], (size_t)(4 + nw) * 4, cudaMemcpyDeviceToHost, down_stream_));
    CU(cudaEventRecord(done_[turn], down_stream_));
    n_of_[turn] = nw;
    logprobs_of_[turn] = want_logprobs;
    *ticket = turn;
    turn_ ^= 1;
    return true;
  }

  bool collect(int ticket, std::vector<int>* tokens, std::vector<float>* logprobs, std::string* err) override {
    CU(cudaEventSynchronize(done_[ticket]));
    const int* flags = h_flags_[ticket];
    if (flags[0] || flags[1]) {
      const int a = flags[0], b = flags[1];
      cudaMemsetAsync(d_res_[ticket], 0, 8, stream_);
      if (a) return *err = "a kernel met an out-of-range token or position id", false;
      if (b & SGLC_FLAG_INDEX) return *err = "a kernel of the bounds-check build met an index outside its range", false;
      return *err = "a tensor-core kernel gave up on a bounded wait; its output is invalid", false;
    }
    tokens->assign(h_out_[ticket], h_out_[ticket] + n_of_[ticket]);
    if (logprobs_of_[ticket]) logprobs->assign(h_logprob_[ticket], h_logprob_[ticket] + n_of_[ticket]);
    return true;
  }

 private:
  bool pinned(void** p, size_t bytes, std::string* err) {
    CU(cudaMallocHost(p, bytes ? bytes : 1));
    pinned_.push_back(*p);
    return true;
  }
  bool device(void** p, size_t bytes, std::string* err) {
    CU(cudaMalloc(p, bytes ? bytes : 1));
    dev_.push_back(*p);
    return true;
  }

  // The upper bound of the context length that the step's kernels are launched for (a captured
  // graph serves until the contexts pass it): the next power of two; a step of single tokens in
  // few (token, head) items goes to the decode attention whose blocks' shared memory is sized by
  // the bound, and there it moves in steps of 128 keys up to 1024 and of about an eighth of the
  // length beyond (parts/attention.py: graph_bound).
  int graph_bound(const WalkStep& s) const {
    int bound = 128;
    while (bound < s.max_keys) bound *= 2;
    int asked = 0;
    for (const WalkLayer& L : dm_->layers)
      if (s.n_decode == s.T && s.T * L.n_heads < STREAM_MIN_ITEMS) {
        int g = 128;
        while (g * 8 < s.max_keys) g *= 2;
        asked = std::max(asked, ((s.max_keys + g - 1) / g) * g);
      }
    if (asked) bound = asked;
    return std::min(bound, dm_->wm.n_positions);
  }

  bool walk(WalkStep* s, int turn, bool want_logprobs, std::string* err) {
    int code = k_->forward(&dm_->wm, s);
    if (code != 0) {
      *err = std::string(s->where[0] ? s->where : "step walker") + ": " + k_->walker_error(code) + fmt(" (code %d)", code);
      return false;
    }
    if (s->n_want > 0) {
      code = k_->sample(logits_, dm_->wm.vocab, dm_->wm.vocab, s->n_want, d_params_[turn], d_hist_tok_, d_hist_cnt_,
                        d_res_[turn] + 4, want_logprobs ? d_logprob_[turn] : nullptr, stream_);
      s->launches++;
      if (code != 0) return *err = fmt("sample: launch failed (code %d)", code), false;
    }
    return true;
  }

  // Replays a CUDA graph when the step's launch shapes have been seen before; everything else a
  // step varies in lies in device arrays at fixed addresses.  A shape runs as plain launches the
  // first time it is seen and is captured the second time; a step of single tokens, which will
  // come again, is captured the first time.
  bool forward(WalkStep* s, bool ids_on_device, int turn, bool want_logprobs, std::string* err) {
    if (!opt_.use_graphs) {
      if (!walk(s, turn, want_logprobs, err)) return false;
      launches += s->launches;
      return true;
    }
    const int bound = graph_bound(*s);
    s->max_keys = bound;
    const GraphKey key{s->T, s->R, s->n_want, s->max_q_len > 1 ? (s->max_q_len + 127) / 128 : 0, bound, s->n_decode,
                       // (captured with the graph: the token array's address, this turn's arrays, the sampler's form)
                       s->decode_ordered + 2 * (ids_on_device ? 1 : 0) + 4 * turn + 8 * (want_logprobs ? 1 : 0)};
    auto it = graphs_.find(key);
    if (it == graphs_.end()) {
      const bool steady = s->n_decode == s->T && plain_steps_ > 0;
      if (!steady && !seen_.count(key)) {
        if (seen_.size() > 4096) seen_.clear();
        seen_[key] = true;
        ++plain_steps_;
        if (!walk(s, turn, want_logprobs, err)) return false;
        launches += s->launches;
        return true;
      }
      cudaGraph_t graph = nullptr;
      CU(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
      const bool ok = walk(s, turn, want_logprobs, err);
      cudaError_t e = cudaStreamEndCapture(stream_, &graph);
      if (!ok || e != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        if (ok) *err = std::string("capturing the step's graph failed: ") + cudaGetErrorString(e);
        return false;
      }
      Graph g;
      g.launches = s->launches;
      e = cudaGraphInstantiate(&g.exec, graph, 0);
      cudaGraphDestroy(graph);
      if (e != cudaSuccess) return *err = std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e), false;
      if ((int)graphs_.size() >= MAX_GRAPHS) {             // the least recently used one goes
        auto old = graphs_.begin();
        for (auto j = graphs_.begin(); j != graphs_.end(); ++j)
          if (j->second.used < old->second.used) old = j;
        cudaGraphExecDestroy(old->second.exec);
        graphs_.erase(old);
      }
      it = graphs_.emplace(key, g).first;
    }
    it->second.used = ++clock_;
    CU(cudaGraphLaunch(it->second.exec, stream_));
    launches += it->second.launches;
    ++graph_replays;
    return true;
  }

  // the sampler's records of a step (and the histories of rows with penalties), on their way up
  bool sample_records(const std::vector<StepItem>& items, const std::vector<double>& uniforms, int nw, int turn,
                      std::string* err) {
    int* const h_params = h_params_[turn];
    // records of 10 words: temperature, top_p, min_p, u, top_k, the three penalties, and the
    // row's range of (token, count) pairs (csrc/sampling.cu)
    std::vector<int> hist;                       // token, count, token, count, ...
    int row = 0;
    bool plain_greedy = true;                    // every row: argmax and nothing else
    for (const StepItem& it : items)
      if (it.sampled && !(it.r->sp.greedy() && !it.r->sp.has_penalties())) plain_greedy = false;
    const bool records_there = plain_greedy && greedy_rows_[turn] >= nw;   // the device already holds nw such records
    for (const StepItem& it : items) {
      if (!it.sampled) continue;
      const Sampling& sp = it.r->sp;
      float* f = (float*)(h_params + (size_t)row * 10);
      int* w = h_params + (size_t)row * 10;
      const int begin = (int)hist.size() / 2;
      if (sp.has_penalties() && !it.r->gen.empty()) {
        std::map<int, int> counts;
        for (int t : it.r->gen) counts[t]++;
        for (const auto& kv : counts) {
          hist.push_back(kv.first);
          hist.push_back(kv.second);
        }
      }
      f[0] = sp.temperature; f[1] = sp.top_p; f[2] = sp.min_p; f[3] = (float)uniforms[row];
      w[4] = sp.temperature > 0.0f ? sp.top_k : 0;
      f[5] = sp.repetition_penalty; f[6] = sp.frequency_penalty; f[7] = sp.presence_penalty;
      w[8] = begin;
      w[9] = (int)hist.size() / 2;
      ++row;
    }
    const int n_pairs = (int)hist.size() / 2;
    if (n_pairs > hist_cap_) {
      CU(cudaStreamSynchronize(stream_));
      for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second.exec);     // (they hold the old buffers' addresses)
      graphs_.clear();
      hist_cap_ = 2 * n_pairs;
      if (!device((void**)&d_hist_tok_, (size_t)hist_cap_ * 4, err) || !device((void**)&d_hist_cnt_, (size_t)hist_cap_ * 4, err) ||
          !pinned((void**)&h_hist_, (size_t)hist_cap_ * 8, err))
        return false;
    }
    if (n_pairs) {
      for (int i = 0; i < n_pairs; ++i) {
        h_hist_[i] = hist[2 * i];
        h_hist_[hist_cap_ + i] = hist[2 * i + 1];
      }
      // (rows with penalties are never queued ahead: the step that last read these has been collected)
      CU(cudaMemcpyAsync(d_hist_tok_, h_hist_, (size_t)n_pairs * 4, cudaMemcpyHostToDevice, up_stream_));
      CU(cudaMemcpyAsync(d_hist_cnt_, h_hist_ + hist_cap_, (size_t)n_pairs * 4, cudaMemcpyHostToDevice, up_stream_));
    }
    if (!records_there)
      CU(cudaMemcpyAsync(d_params_[turn], h_params, (size_t)nw * 40, cudaMemcpyHostToDevice, up_stream_));
    greedy_rows_[turn] = plain_greedy ? std::max(greedy_rows_[turn], nw) : 0;
    return true;
  }

  typedef std::tuple<int, int, int, int, int, int, int> GraphKey;
  struct Graph {
    cudaGraphExec_t exec = nullptr;
    long long launches = 0, used = 0;
  };
  const DeviceModel* dm_;
  const CacheTables* cache_;
  const Kernels* k_;
  sglc_engine_options opt_;
  cudaStream_t stream_ = nullptr, up_stream_ = nullptr, down_stream_ = nullptr;
  cudaEvent_t uploaded_[2] = {nullptr, nullptr}, ran_[2] = {nullptr, nullptr}, marks_[2] = {nullptr, nullptr};
  long long n_marks_ = 0;
  bool used_[2] = {false, false}, few_ok_ = false;
  int t_cap_ = 0, r_cap_ = 0, b_cap_ = 0, n_groups_ = 0, total_ = 0, logit_rows_ = 0, hist_cap_ = 0;
  Field f_tokens_, f_positions_, f_token_req_, f_want_, f_decode_, f_q_start_, f_kv_len_, f_state_;
  std::vector<Field> f_slots_, f_bt_;
  int *h_blk_[2] = {nullptr, nullptr}, *d_blk_[2] = {nullptr, nullptr};
  unsigned char* ws_ = nullptr;
  long long ws_bytes_ = 0;
  float *logits_ = nullptr, *tc_ws_ = nullptr, *d_logprob_[2] = {nullptr, nullptr}, *h_logprob_[2] = {nullptr, nullptr};
  int *tc_counters_ = nullptr, *d_res_[2] = {nullptr, nullptr}, *h_flags_[2] = {nullptr, nullptr};
  int *h_params_[2] = {nullptr, nullptr}, *d_params_[2] = {nullptr, nullptr}, *h_out_[2] = {nullptr, nullptr};
  cudaEvent_t done_[2] = {nullptr, nullptr};
  int turn_ = 0, n_of_[2] = {0, 0}, greedy_rows_[2] = {0, 0};
  bool logprobs_of_[2] = {false, false};
  int *d_hist_tok_ = nullptr, *d_hist_cnt_ = nullptr, *h_hist_ = nullptr;
  std::vector<const int*> bts_, slots_;
  std::vector<void*> dev_, pinned_;
  std::map<GraphKey, Graph> graphs_;
  std::map<GraphKey, bool> seen_;
  long long clock_ = 0, plain_steps_ = 0;
};

}  // namespace

struct sglc_engine {
  sglc_engine_options opt;
  DeviceModel model;
  Kernels kernels;
  std::unique_ptr<CacheTables> cache;
  std::unique_ptr<StepRunner> runner;
  DeviceRunner* device_runner = nullptr;
  std::unique_ptr<Scheduler> sched;
  std::string last_error;
  int eos = -1;
};

SGLC_API void sglc_sampling_default(sglc_sampling* sp) {
  memset(sp, 0, sizeof(*sp));
  sp->top_p = 1.0f;
  sp->repetition_penalty = 1.0f;
}

SGLC_API void sglc_engine_options_default(sglc_engine_options* o) {
  memset(o, 0, sizeof(*o));
  o->bf16 = 1;
  o->page_size = 16;
  o->max_requests = 64;
  o->max_step_tokens = 2048;
  o->prefill_chunk = 512;
  o->use_graphs = 1;
  o->eos_token_id = -2;
  o->run_ahead = 1;
}

SGLC_API sglc_engine* sglc_engine_new(const char* model_dir, const sglc_engine_options* options, char* err, int err_len) {
  std::string why;
  std::unique_ptr<sglc_engine> e(new sglc_engine());
  auto refuse = [&]() -> sglc_engine* {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", why.c_str());
    return nullptr;
  };
  if (options) e->opt = *options;
  else sglc_engine_options_default(&e->opt);
  sglc_engine_options& o = e->opt;
  if (!model_dir) return why = "no model folder given", refuse();
  if (o.page_size <= 0 || o.max_requests <= 0 || o.max_step_tokens <= 0)
    return why = "page_size, max_requests and max_step_tokens must be positive", refuse();
  const bool device = !o.dry_run;
  if (device) {
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev <= 0)
      return why = "no CUDA device is available; this engine has no CPU path", refuse();
    if (o.device < 0 || o.device >= n_dev) return why = fmt("device %d: this machine has %d CUDA device(s)", o.device, n_dev), refuse();
    if (cudaSetDevice(o.device) != cudaSuccess) return why = fmt("device %d cannot be selected", o.device), refuse();
    if (!e->kernels.load(o.library_dir ? o.library_dir : own_directory(), &why)) return refuse();
  }
  // sizes of the pool need the model's positions: read the description first, then build
  {
    DeviceModel probe;
    std::string text;
    Json config;
    std::string jerr;
    if (!read_text_file(std::string(model_dir) + "/config.json", &text)) return why = std::string("no config.json in ") + model_dir, refuse();
    if (!json_parse(text, &config, &jerr)) return why = std::string(model_dir) + "/config.json: not valid JSON (" + jerr + ")", refuse();
    if (config.kind != Json::Obj) return why = std::string(model_dir) + "/config.json: top level must be an object", refuse();
    if (!resolve_architecture(config, &probe.spec, &why)) return refuse();
    if (o.n_pages <= 0) {
      long long tokens = o.max_tokens > 0 ? o.max_tokens : (long long)o.max_requests * probe.spec.positions;
      o.n_pages = (tokens + o.page_size - 1) / o.page_size;
    }
  }
  if (o.n_pages > 0x7FFFFFFF) return why = "more pages than a 32-bit page id can name", refuse();
  if (!load_model(model_dir, o.bf16 != 0, device, o.page_size, o.n_pages, &e->model, &why)) return refuse();
  const ModelSpec& m = e->model.spec;
  e->cache.reset(new CacheTables(o.page_size, (int)o.n_pages, o.max_requests, e->model.windows));
  if (device) {
    e->device_runner = new DeviceRunner(&e->model, e->cache.get(), &e->kernels, o);
    e->runner.reset(e->device_runner);
    if (!e->device_runner->init(&why)) return refuse();
  } else {
    e->runner.reset(new DryRunner(m.vocab));
  }
  e->eos = o.eos_token_id == -2 ? m.eos : (o.eos_token_id >= 0 ? o.eos_token_id : -1);
  const int budget = o.token_budget > 0 ? std::min(o.token_budget, o.max_step_tokens) : o.max_step_tokens;
  e->sched.reset(new Scheduler(e->cache.get(), e->runner.get(), m.vocab, m.positions, e->eos, o.seed, o.prefill_chunk,
                               budget, o.want_logprobs != 0, o.run_ahead != 0));
  return e.release();
}

SGLC_API void sglc_engine_free(sglc_engine* e) {
  if (!e) return;
  if (!e->opt.dry_run) cudaSetDevice(e->opt.device);
  e->sched.reset();
  e->runner.reset();
  delete e;
}

SGLC_API long long sglc_engine_submit_ids(sglc_engine* e, const int* ids, int n, int max_new, const sglc_sampling* sp) {
  Sampling s;
  if (sp) {
    s.temperature = sp->temperature; s.top_k = sp->top_k; s.top_p = sp->top_p; s.min_p = sp->min_p;
    s.repetition_penalty = sp->repetition_penalty; s.frequency_penalty = sp->frequency_penalty;
    s.presence_penalty = sp->presence_penalty; s.ignore_eos = sp->ignore_eos;
    s.n_stop_ids = sp->n_stop_ids < 0 ? 0 : (sp->n_stop_ids > 8 ? 8 : sp->n_stop_ids);
    memcpy(s.stop_ids, sp->stop_ids, sizeof(s.stop_ids));
    s.seed = sp->seed;
  }
  return e->sched->submit_ids(ids, n, max_new, &s);
}

SGLC_API int sglc_engine_step(sglc_engine* e) {
  if (!e->opt.dry_run) cudaSetDevice(e->opt.device);
  std::string err;
  const int n = e->sched->step(&err);
  if (n < 0) e->last_error = err;
  return n;
}

SGLC_API int sglc_engine_nactive(sglc_engine* e) { return e->sched->nactive(); }

SGLC_API int sglc_engine_poll(sglc_engine* e, long long* id, int* tokens, int cap, int* n_tokens, int* n_prompt,
                              int* finish_reason) {
  const Request* r = e->sched->poll_peek();
  if (!r) return 0;
  const int n = (int)r->gen.size();
  if (id) *id = r->id;
  if (n_tokens) *n_tokens = n;
  if (n_prompt) *n_prompt = (int)r->prompt.size();
  if (finish_reason) *finish_reason = r->finish;
  if (cap < 0) return 1;                         // a look only
  if (tokens && cap > 0) memcpy(tokens, r->gen.data(), (size_t)std::min(cap, n) * sizeof(int));
  if (tokens && cap < n) return 1;               // not taken: the caller comes again with room
  e->sched->poll_take();
  return 1;
}

SGLC_API int sglc_engine_poll_logprobs(sglc_engine* e, long long id, float* out, int cap) {
  const Request* r = e->sched->find(id);
  if (!r) return -1;
  const int n = (int)r->logprobs.size();
  if (out && cap > 0) memcpy(out, r->logprobs.data(), (size_t)std::min(cap, n) * sizeof(float));
  return n;
}

SGLC_API int sglc_engine_generated(sglc_engine* e, long long id, int* tokens, int cap) {
  const Request* r = e->sched->find(id);
  if (!r) return -1;
  const int n = (int)r->gen.size();
  if (tokens && cap > 0) memcpy(tokens, r->gen.data(), (size_t)std::min(cap, n) * sizeof(int));
  return n;
}

SGLC_API int sglc_engine_abort(sglc_engine* e, long long id) { return e->sched->abort(id); }

SGLC_API int sglc_engine_sync(sglc_engine* e) {
  if (!e->opt.dry_run) cudaSetDevice(e->opt.device);
  std::string err;
  const int n = e->sched->drain(&err);
  if (n < 0) e->last_error = err;
  return n;
}

SGLC_API int sglc_engine_rewind(sglc_engine* e, long long id, int keep) { return e->sched->rewind(id, keep) ? 0 : -1; }

SGLC_API int sglc_engine_mark(sglc_engine* e, int sync_first) {
  if (!e->device_runner) return -1;
  cudaSetDevice(e->opt.device);
  std::string err;
  if (e->device_runner->mark(sync_first != 0, &err)) return 0;
  e->last_error = err;
  return -1;
}

SGLC_API double sglc_engine_ms_between_marks(sglc_engine* e) {
  return e->device_runner ? e->device_runner->ms_between_marks() : -1.0;
}

SGLC_API void sglc_engine_get_stats(sglc_engine* e, sglc_stats* out) {
  const SchedStats s = e->sched->stats();
  memset(out, 0, sizeof(*out));
  out->prefill_tokens = s.prefill_tokens; out->decode_tokens = s.decode_tokens; out->n_finished = s.n_finished;
  out->n_running = s.n_running; out->n_waiting = s.n_waiting; out->pool_pages = s.pool_pages; out->pool_free = s.pool_free;
  out->n_preempt = s.n_preempt; out->prefill_chunk = s.prefill_chunk; out->n_steps = s.n_steps;
  out->recomputed_tokens = s.recomputed_tokens;
  out->steps_ahead = s.steps_ahead;
  if (e->device_runner) {
    out->graph_replays = e->device_runner->graph_replays;
    out->launches = e->device_runner->launches;
    out->step_upload_bytes = e->device_runner->upload_bytes();
  }
  out->weight_bytes = e->model.weight_bytes;
  out->cache_bytes = e->model.cache_bytes;
}

SGLC_API long long sglc_engine_run_until_done(sglc_engine* e, long long max_steps) {
  long long steps = 0;
  while (e->sched->nactive() > 0 && steps < max_steps) {
    if (sglc_engine_step(e) < 0) return -1;
    ++steps;
  }
  return steps;
}

SGLC_API int sglc_engine_last_step(sglc_engine* e, long long* ids, int* n_tokens, int* sampled, int cap) {
  const auto& ran = e->sched->last_step();
  for (int i = 0; i < (int)ran.size() && i < cap; ++i) {
    if (ids) ids[i] = ran[i].id;
    if (n_tokens) n_tokens[i] = ran[i].n;
    if (sampled) sampled[i] = ran[i].sampled ? 1 : 0;
  }
  return (int)ran.size();
}

SGLC_API int sglc_engine_check(sglc_engine* e) {
  std::string why;
  if (e->cache->check(&why)) return 0;
  e->last_error = why;
  return -1;
}

SGLC_API const char* sglc_engine_last_error(sglc_engine* e) { return e->last_error.c_str(); }

// The page tables alone under a random order of operations (requests arrive, grow by portions of
// any size, are cut back, end), two cache groups, one with a window: after every operation the
// invariants hold, a request's table covers its length, and the windowed group holds no page that
// no later query can see.  0, or -1 with the reason in err.
SGLC_API int sglc_pages_selftest(int page_size, int n_pages, int max_requests, int window, unsigned seed, int n_ops,
                                 char* err, int err_len) {
  CacheTables t(page_size, n_pages, max_requests, {0, window});
  uint64_t state = request_stream(seed, 1);
  auto rnd = [&](int n) { return (int)(next_uniform(&state) * n); };
  std::vector<long long> live;
  long long next = 1;
  std::string why;
  auto fail = [&](const std::string& what) {
    if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s", what.c_str());
    return -1;
  };
  for (int op = 0; op < n_ops; ++op) {
    const int kind = rnd(10);
    if (kind < 2 || live.empty()) {
      if (t.n_free_slots() == 0) continue;
      if (t.add(next) < 0) return fail("add refused with a free slot");
      live.push_back(next++);
    } else if (kind < 7) {
      const long long r = live[rnd((int)live.size())];
      const int new_len = t.length(r) + 1 + rnd(3 * page_size);
      const bool can = t.can_extend_all({{r, new_len}});
      const int before = t.length(r);
      const bool did = t.extend(r, new_len);
      if (can != did) return fail("can_extend_all and extend disagree");
      if (t.length(r) != (did ? new_len : before)) return fail("extend left a wrong length");
    } else if (kind < 8) {
      const long long r = live[rnd((int)live.size())];
      const int new_len = rnd(t.length(r) + 1);
      const int before = t.length(r);
      if (t.truncate(r, new_len)) {
        if (t.length(r) != new_len) return fail("truncate left a wrong length");
      } else if (t.length(r) != before) {
        return fail("a refused truncate changed the length");
      }
    } else {
      const int i = rnd((int)live.size());
      if (!t.free(live[i])) return fail("free refused a live request");
      if (t.free(live[i])) return fail("a request could be freed twice");
      live.erase(live.begin() + i);
    }
    if (!t.check(&why)) return fail(why);
    for (long long r : live) {
      const int len = t.length(r), blocks = (len + page_size - 1) / page_size;
      for (int g = 0; g < 2; ++g) {
        const std::vector<int>& tab = t.table(g, r);
        if ((int)tab.size() < blocks) return fail("a block table is shorter than its request");
        // every position a query at `len` or later may see has its page
        const int first_pos = (g == 1 && window > 0 && len - window + 1 > 0) ? len - window + 1 : 0;
        for (int b = first_pos / page_size; b < blocks; ++b)
          if (tab[b] < 0) return fail("a page that is still visible was given back");
        if (g == 0)
          for (int b = 0; b < blocks; ++b)
            if (tab[b] < 0) return fail("a group without a window gave a page back");
      }
    }
  }
  for (long long r : live) t.free(r);
  if (!t.check(&why)) return fail(why);
  if (t.n_free_pages() != n_pages || t.n_free_slots() != max_requests) return fail("pages or slots were lost");
  return 0;
}
SGLC_API int sglc_engine_vocab_size(sglc_engine* e) { return e->model.spec.vocab; }
SGLC_API int sglc_engine_max_positions(sglc_engine* e) { return e->model.spec.positions; }
SGLC_API int sglc_engine_eos_token_id(sglc_engine* e) { return e->eos; }
