// The safetensors container read through a memory map: u64 little-endian header length, a JSON
// header {name: {dtype, shape, data_offsets}}, then the data area; and a model folder seen as one
// set of tensors, through model.safetensors.index.json when the folder has that index, else
// model.safetensors (the reference: src/safetensors.c:147-179, checks :507-526, folders :676-843).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "json.hpp"

namespace sglc {

struct TensorView {
  std::string dtype;                 // F32, BF16, F16, F64, I32, I64, U8
  std::vector<long long> shape;
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
  bool floating() const { return dtype == "F32" || dtype == "BF16" || dtype == "F16" || dtype == "F64"; }
  long long numel() const {
    long long n = 1;
    for (long long s : shape) n *= s;
    return n;
  }
};

inline int dtype_size(const std::string& dt) {
  if (dt == "F32" || dt == "I32") return 4;
  if (dt == "BF16" || dt == "F16") return 2;
  if (dt == "F64" || dt == "I64") return 8;
  if (dt == "U8") return 1;
  return 0;
}

inline bool read_text_file(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  char buf[1 << 14];
  size_t n;
  out->clear();
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) out->append(buf, n);
  fclose(f);
  return true;
}

class SafetensorsFile {
 public:
  ~SafetensorsFile() {
    if (map_ && map_ != MAP_FAILED) munmap(map_, size_);
    if (fd_ >= 0) close(fd_);
  }
  // false with `err` set
  bool open(const std::string& path, std::string* err) {
    path_ = path;
    fd_ = ::open(path.c_str(), O_RDONLY);
    struct stat st;
    if (fd_ < 0 || fstat(fd_, &st) != 0) return fail(err, "no such file");
    size_ = (size_t)st.st_size;
    if (size_ < 8) return fail(err, "shorter than its 8-byte header length");
    map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) return fail(err, "cannot be mapped");
    const uint8_t* p = (const uint8_t*)map_;
    uint64_t hlen = 0;
    for (int k = 7; k >= 0; --k) hlen = (hlen << 8) | p[k];
    if (hlen > (100ull << 20) || 8 + hlen > size_)
      return fail(err, "header length " + std::to_string(hlen) + " exceeds the file (" + std::to_string(size_) + " bytes)");
    Json header;
    std::string jerr;
    JsonParser parser((const char*)p + 8, (size_t)hlen);
    if (!parser.parse(&header, &jerr)) return fail(err, "header is not valid JSON (" + jerr + ")");
    if (header.kind != Json::Obj) return fail(err, "header must be a JSON object");
    const size_t data0 = 8 + (size_t)hlen, data_len = size_ - data0;
    for (const auto& kv : header.obj) {
      if (kv.first == "__metadata__") continue;
      const Json *dt = kv.second.get("dtype"), *sh = kv.second.get("shape"), *off = kv.second.get("data_offsets");
      if (!dt || dt->kind != Json::Str || !sh || sh->kind != Json::Arr || !off || off->kind != Json::Arr ||
          off->arr.size() != 2 || off->arr[0].kind != Json::Int || off->arr[1].kind != Json::Int)
        return fail(err, "entry '" + kv.first + "' lacks dtype, shape or data_offsets");
      TensorView t;
      t.dtype = dt->s;
      const int es = dtype_size(t.dtype);
      if (es == 0) return fail(err, "tensor '" + kv.first + "' has dtype " + t.dtype + "; handled: BF16 F16 F32 F64 I32 I64 U8");
      long long numel = 1;
      for (const Json& d : sh->arr) {
        if (d.kind != Json::Int) return fail(err, "entry '" + kv.first + "' lacks dtype, shape or data_offsets");
        if (d.i < 0) return fail(err, "tensor '" + kv.first + "' has a negative dimension");
        t.shape.push_back(d.i);
        numel *= d.i;
      }
      const long long b = off->arr[0].i, e = off->arr[1].i;
      if (!(0 <= b && b <= e && (size_t)e <= data_len) || e - b != numel * es)
        return fail(err, "tensor '" + kv.first + "' data_offsets [" + std::to_string(b) + "," + std::to_string(e) +
                             ") do not fit its shape and " + t.dtype + " in a data area of " + std::to_string(data_len) +
                             " bytes");
      t.data = p + data0 + b;
      t.nbytes = (size_t)(e - b);
      entries_[kv.first] = std::move(t);
      order_.push_back(kv.first);
    }
    return true;
  }
  const TensorView* find(const std::string& name) const {
    auto it = entries_.find(name);
    return it == entries_.end() ? nullptr : &it->second;
  }
  const std::vector<std::string>& names() const { return order_; }
  const std::string& path() const { return path_; }

 private:
  bool fail(std::string* err, const std::string& what) {
    *err = path_ + ": " + what;
    return false;
  }
  std::string path_;
  int fd_ = -1;
  void* map_ = nullptr;
  size_t size_ = 0;
  std::map<std::string, TensorView> entries_;
  std::vector<std::string> order_;
};

// The tensors of a model folder.  With an index, a tensor the index names must be in the shard
// it names; what a shard holds beyond the index is not visible.
class Checkpoint {
 public:
  bool open(const std::string& dir, std::string* err) {
    const std::string index = dir + "/model.safetensors.index.json";
    std::string text;
    if (read_text_file(index, &text)) {
      where_ = index;
      Json j;
      std::string jerr;
      const Json* wmap = nullptr;
      if (!json_parse(text, &j, &jerr) || !(wmap = j.get("weight_map")) || wmap->kind != Json::Obj || wmap->obj.empty()) {
        *err = index + ": not a shard index with a weight_map";
        return false;
      }
      std::map<std::string, SafetensorsFile*> by_name;
      std::string lost;
      for (const auto& kv : wmap->obj) {
        const std::string& shard = kv.second.s;
        if (kv.second.kind != Json::Str || shard.empty() || shard.find('/') != std::string::npos) {
          *err = index + ": shard name of tensor '" + kv.first + "' must be a file name in the same folder";
          return false;
        }
        SafetensorsFile*& f = by_name[shard];
        if (!f) {
          files_.emplace_back(new SafetensorsFile());
          f = files_.back().get();
          struct stat st;
          if (stat((dir + "/" + shard).c_str(), &st) != 0) {
            *err = index + " names shard " + shard + ", which is not in " + dir;
            return false;
          }
          if (!f->open(dir + "/" + shard, err)) return false;
        }
        const TensorView* t = f->find(kv.first);
        if (!t) lost += (lost.empty() ? "" : ", ") + kv.first;
        else {
          tensors_[kv.first] = t;
          order_.push_back(kv.first);
        }
      }
      if (!lost.empty()) {
        *err = index + ": tensors not found in the shard it names: " + lost;
        return false;
      }
      return true;
    }
    where_ = dir + "/model.safetensors";
    struct stat st;
    if (stat(where_.c_str(), &st) != 0) {
      *err = "no model.safetensors (or model.safetensors.index.json) in " + dir;
      return false;
    }
    files_.emplace_back(new SafetensorsFile());
    if (!files_.back()->open(where_, err)) return false;
    for (const std::string& n : files_.back()->names()) {
      tensors_[n] = files_.back()->find(n);
      order_.push_back(n);
    }
    return true;
  }
  const TensorView* find(const std::string& name) const {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : it->second;
  }
  const std::vector<std::string>& names() const { return order_; }
  const std::string& where() const { return where_; }

 private:
  std::vector<std::unique_ptr<SafetensorsFile>> files_;
  std::map<std::string, const TensorView*> tensors_;
  std::vector<std::string> order_;
  std::string where_;
};

}  // namespace sglc
