// Reads a model folder's tensors: model.safetensors, or the shards model.safetensors.index.json
// names.  A safetensors file is an 8-byte little-endian header length, a JSON header
// {name: {dtype, shape, data_offsets}} and the raw tensor bytes; the file is mapped into memory and
// a tensor is a pointer into the mapping.  The reference maps its GGUF file the same way
// (gguf/src/mapped_file.cpp) and finds tensors by name (runtime/include/qorvix/runtime/tensor_load.hpp:25-47).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "json.hpp"

namespace qv {

struct StTensor {
  std::string dtype;                    // "F32", "BF16", "F16", "I32", "I64", ...
  std::vector<long long> shape;
  const uint8_t* data = nullptr;
  size_t bytes = 0;
  long long numel() const {
    long long n = 1;
    for (long long s : shape) n *= s;
    return n;
  }
};

inline std::string read_text_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error(path + ": cannot be opened");
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

inline bool file_exists(const std::string& path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error(path + ": cannot be opened");
    struct stat st;
    if (::fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw std::runtime_error(path + ": too short for a safetensors file"); }
    size_ = (size_t)st.st_size;
    map_ = (const uint8_t*)::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (map_ == MAP_FAILED) { ::close(fd_); throw std::runtime_error(path + ": cannot be mapped"); }
    uint64_t hlen = 0;
    std::memcpy(&hlen, map_, 8);
    if (hlen > size_ - 8) throw std::runtime_error(path + ": the header length exceeds the file");
    Json header = JsonParser((const char*)map_ + 8, (size_t)hlen).parse();
    const size_t base = 8 + (size_t)hlen;
    for (const auto& kv : header.obj) {
      if (kv.first == "__metadata__") continue;
      StTensor t;
      t.dtype = kv.second.at("dtype").string();
      for (const Json& d : kv.second.at("shape").arr) t.shape.push_back(d.integer());
      const auto& off = kv.second.at("data_offsets").arr;
      if (off.size() != 2) throw std::runtime_error(path + ": tensor '" + kv.first + "' has no two data offsets");
      const long long b = off[0].integer(), e = off[1].integer();
      if (b < 0 || e < b || base + (size_t)e > size_)
        throw std::runtime_error(path + ": the data of tensor '" + kv.first + "' lies outside the file");
      t.data = map_ + base + b;
      t.bytes = (size_t)(e - b);
      tensors_[kv.first] = std::move(t);
    }
  }
  ~SafetensorsFile() {
    if (map_ && map_ != MAP_FAILED) ::munmap((void*)map_, size_);
    if (fd_ >= 0) ::close(fd_);
  }
  SafetensorsFile(const SafetensorsFile&) = delete;
  SafetensorsFile& operator=(const SafetensorsFile&) = delete;
  const std::map<std::string, StTensor>& tensors() const { return tensors_; }

 private:
  std::string path_;
  int fd_ = -1;
  size_t size_ = 0;
  const uint8_t* map_ = nullptr;
  std::map<std::string, StTensor> tensors_;
};

// All tensors of a model folder by name.
class Checkpoint {
 public:
  explicit Checkpoint(const std::string& dir) {
    std::vector<std::string> shards;
    if (file_exists(dir + "/model.safetensors")) {
      shards.push_back("model.safetensors");
    } else if (file_exists(dir + "/model.safetensors.index.json")) {
      Json idx = parse_json(read_text_file(dir + "/model.safetensors.index.json"));
      for (const auto& kv : idx.at("weight_map").obj) {
        const std::string& s = kv.second.string();
        bool seen = false;
        for (const auto& x : shards) seen = seen || x == s;
        if (!seen) shards.push_back(s);
      }
    } else {
      throw std::runtime_error(dir + ": no model.safetensors (or model.safetensors.index.json) in the model folder");
    }
    for (const auto& s : shards) {
      files_.emplace_back(new SafetensorsFile(dir + "/" + s));
      for (const auto& kv : files_.back()->tensors()) all_[kv.first] = &kv.second;
    }
  }
  const StTensor* find(const std::string& name) const {
    auto it = all_.find(name);
    return it == all_.end() ? nullptr : it->second;
  }
  const std::map<std::string, const StTensor*>& all() const { return all_; }

 private:
  std::vector<std::unique_ptr<SafetensorsFile>> files_;
  std::map<std::string, const StTensor*> all_;
};

// A tensor's values as float32, whatever floating type it is stored in.
inline std::vector<float> to_float(const StTensor& t) {
  const long long n = t.numel();
  std::vector<float> out((size_t)n);
  if (t.dtype == "F32") {
    std::memcpy(out.data(), t.data, (size_t)n * 4);
  } else if (t.dtype == "BF16") {
    const uint16_t* s = (const uint16_t*)t.data;
    for (long long i = 0; i < n; ++i) {
      const uint32_t u = (uint32_t)s[i] << 16;
      std::memcpy(&out[(size_t)i], &u, 4);
    }
  } else if (t.dtype == "F16") {
    const uint16_t* s = (const uint16_t*)t.data;
    for (long long i = 0; i < n; ++i) {
      const uint32_t h = s[i], sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
      uint32_t u;
      if (exp == 0) {
        if (man == 0) u = sign;
        else {                                         // subnormal half
          int e = -1;
          uint32_t m = man;
          do { ++e; m <<= 1; } while (!(m & 0x400));
          u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FF) << 13);
        }
      } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
      else u = sign | ((exp + 112) << 23) | (man << 13);
      std::memcpy(&out[(size_t)i], &u, 4);
    }
  } else if (t.dtype == "F64") {
    const double* s = (const double*)t.data;
    for (long long i = 0; i < n; ++i) out[(size_t)i] = (float)s[i];
  } else {
    throw std::runtime_error("tensor of type " + t.dtype + " is not a floating tensor");
  }
  return out;
}

}  // namespace qv
