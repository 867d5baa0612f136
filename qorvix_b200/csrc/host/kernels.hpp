// The kernel libraries of this folder as a table of C entry points, resolved with dlopen/dlsym from
// the shared libraries csrc/build.py made (their paths come from the manifest it writes beside them,
// or from the host that drives the executor).  One table serves the command-line tools and the
// executor that the Python step function calls.
#pragma once
#include <dlfcn.h>

#include <cstdio>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>

namespace qv {

constexpr int DT_F32 = 0, DT_BF16 = 1;
constexpr int ERR_UNSUPPORTED = -2;

struct Kernels {
  // elementwise
  int (*embed)(float*, const void*, const int*, int, int, int, int, void*) = nullptr;
  int (*add_rmsnorm)(void*, float*, const void*, const float*, const int*, int, int, float, int, int, int, void*) = nullptr;
  int (*rope_kv_write)(void*, int, void*, const float*, int, const int*, const int*, const int*, int, int, int, int, int, int, int, int, void*) = nullptr;
  int (*swiglu)(void*, const void*, int, int, int, int, void*) = nullptr;
  int (*cast)(void*, const void*, long long, int, int, void*) = nullptr;
  const char* (*error_string)(int) = nullptr;
  // matrix products
  int (*gemm_simt)(void*, const void*, const void*, int, int, int, int, int, int, int, int, int, int, void*) = nullptr;
  int (*gemm_bf16_tc)(void*, const void*, const void*, int, int, int, int, int, int, int, int*, int, int, void*) = nullptr;
  long long (*packed_weight_bytes)(int, int) = nullptr;
  int (*pack_weight_tiles)(void*, const void*, int, int, int, void*) = nullptr;
  int (*gemm_bf16_packed)(void*, const void*, const void*, int, int, int, int, int, int, int*, int, int, void*) = nullptr;
  int (*gemm_bf16_qkv_rope)(void*, const void*, const void*, int, int, int, int, int*, const float*, int, const int*, const int*, const int*,
                            int, void*, int, int, int, int, void*) = nullptr;
  int (*gemm_bf16_norm)(void*, const void*, const void*, int, int, int, int, int, int, int*, int, float*, int, const float*, float*,
                        const float*, int, float, float, void*) = nullptr;
  // attention
  int (*attention_generic)(void*, int, const void*, int, const void*, const int*, const int*, const int*, int, int, int, int, int, int, int,
                           float, int, void*) = nullptr;
  int (*attn_prefill_bf16)(void*, int, const void*, int, const void*, const int*, const int*, const int*, int, int, int, int, int, int, int,
                           int, float, int, void*) = nullptr;
  int (*attn_prefill_tc)(void*, int, const void*, int, int, const void*, long long, const int*, const int*, const int*, int, int, int, int,
                         int, int, int, int, int, float, int*, void*) = nullptr;
  void (*attn_set_decode_variant)(int) = nullptr;
  void (*attn_set_error_word)(int*) = nullptr;
  void (*gemm_set_split_workspace)(float*, int*, int) = nullptr;
  long long (*gemm_split_slot_bytes)() = nullptr;
  int (*attn_decode_bf16)(void*, int, const void*, int, const void*, const int*, const int*, const int*, int, int, int, int, int, int, int,
                          float, int, float*, void*) = nullptr;
  // sampling
  int (*argmax)(int*, const float*, int, int, long long, void*) = nullptr;
  int (*sample)(int*, float*, int, int, long long, const float*, const int*, const float*, const float*, const float*, const int*, int,
                const float*, const float*, const float*, void*) = nullptr;

  // `libs`: library name (elementwise, gemm_simt, gemm_bf16, attention_generic, attention_bf16, attention_tc, sampling) -> path
  void load(const std::map<std::string, std::string>& libs) {
    auto open = [&](const char* name) -> void* {
      auto it = libs.find(name);
      if (it == libs.end()) throw std::runtime_error(std::string("no path is known for the kernel library '") + name + "'");
      void* h = dlopen(it->second.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (!h) throw std::runtime_error("cannot load " + it->second + ": " + dlerror());
      return h;
    };
    auto sym = [&](void* h, const char* name) -> void* {
      void* p = dlsym(h, name);
      if (!p) throw std::runtime_error(std::string("the kernel library lacks the entry point ") + name);
      return p;
    };
#define QV_SYM(handle, field, name) field = reinterpret_cast<decltype(field)>(sym(handle, name))
    void* el = open("elementwise");
    QV_SYM(el, embed, "qv_embed"); QV_SYM(el, add_rmsnorm, "qv_add_rmsnorm"); QV_SYM(el, rope_kv_write, "qv_rope_kv_write");
    QV_SYM(el, swiglu, "qv_swiglu"); QV_SYM(el, cast, "qv_cast"); QV_SYM(el, error_string, "qv_error_string");
    void* gs = open("gemm_simt");
    QV_SYM(gs, gemm_simt, "qv_gemm_simt");
    void* gb = open("gemm_bf16");
    QV_SYM(gb, gemm_bf16_tc, "qv_gemm_bf16_tc"); QV_SYM(gb, packed_weight_bytes, "qv_packed_weight_bytes");
    QV_SYM(gb, pack_weight_tiles, "qv_pack_weight_tiles"); QV_SYM(gb, gemm_bf16_packed, "qv_gemm_bf16_packed");
    QV_SYM(gb, gemm_bf16_qkv_rope, "qv_gemm_bf16_qkv_rope"); QV_SYM(gb, gemm_bf16_norm, "qv_gemm_bf16_norm");
    QV_SYM(gb, gemm_set_split_workspace, "qv_gemm_bf16_set_split_workspace"); QV_SYM(gb, gemm_split_slot_bytes, "qv_gemm_bf16_split_slot_bytes");
    void* ag = open("attention_generic");
    QV_SYM(ag, attention_generic, "qv_attention_generic");
    void* ab = open("attention_bf16");
    QV_SYM(ab, attn_prefill_bf16, "qv_attn_prefill_bf16"); QV_SYM(ab, attn_set_decode_variant, "qv_attn_set_decode_variant");
    QV_SYM(ab, attn_set_error_word, "qv_attn_set_error_word"); QV_SYM(ab, attn_decode_bf16, "qv_attn_decode_bf16");
    void* at = open("attention_tc");
    QV_SYM(at, attn_prefill_tc, "qv_attn_prefill_tc");
    void* sa = open("sampling");
    QV_SYM(sa, argmax, "qv_argmax"); QV_SYM(sa, sample, "qv_sample");
#undef QV_SYM
  }
};

// "name=path" lines, as csrc/build.py writes them beside the libraries
inline std::map<std::string, std::string> read_manifest(const std::string& path) {
  std::ifstream f(path);
  if (!f) throw std::runtime_error(path + ": the manifest of kernel libraries is missing (python -m qorvix_b200.csrc.build writes it)");
  std::map<std::string, std::string> out;
  std::string line;
  while (std::getline(f, line)) {
    const size_t eq = line.find('=');
    if (eq != std::string::npos) out[line.substr(0, eq)] = line.substr(eq + 1);
  }
  return out;
}

}  // namespace qv
