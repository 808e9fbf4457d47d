// Tile-config cache with the reference's file format and merge rules
// (gemlite/core.py:80-89 cache_kernel_config, :838-877 cache_config, :879-901 load_config,
// :903-906 reset_config) and the M-bucket function get_closest_m
// (gemlite/triton_kernels/utils.py:182-220).
//
// File format: {"<FAMILY>": {"(Mb, N, K, group_size, elements_per_sample, type_id)": {...}}}.
// The per-signature object is kept as raw JSON text, so entries written by the reference
// (Triton block sizes) survive a load/save round trip untouched and entries of this library
// (e.g. {"split_k": 8, "warps_n": 2}) can sit beside them.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <map>
#include <atomic>
#include <mutex>
#include <string>
#include <stdlib.h>
#include <vector>
#include "../../include/gemlite_b200.h"

void gl_set_error(const char* fmt, ...);

namespace {

typedef std::map<std::string, std::string> SigMap;
typedef std::map<std::string, SigMap> Cache;

Cache g_cache;
std::mutex g_mu;   // guards g_cache and file I/O (the reference's FILE_LOCK, core.py:32-33)
thread_local std::string g_tmp;

struct Parser {
  const char* s; size_t n; size_t i; bool ok;
  void ws() { while (i < n && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  bool lit(const char* t) { size_t l = strlen(t); if (i + l <= n && strncmp(s + i, t, l) == 0) { i += l; return true; } return false; }
  bool str(std::string* out) {
    if (i >= n || s[i] != '"') return false;
    ++i;
    std::string r;
    while (i < n && s[i] != '"') {
      if (s[i] == '\\') {
        if (i + 1 >= n) return false;
        char c = s[i + 1];
        switch (c) {
          case 'n': r += '\n'; break; case 't': r += '\t'; break; case 'r': r += '\r'; break;
          case 'b': r += '\b'; break; case 'f': r += '\f'; break;
          case 'u': { if (i + 5 >= n) return false; r += '?'; i += 4; } break;
          default: r += c; break;
        }
        i += 2;
      } else r += s[i++];
    }
    if (i >= n) return false;
    ++i;
    if (out) *out = r;
    return true;
  }
  // skip any JSON value
  bool value() {
    ws();
    if (i >= n) return false;
    char c = s[i];
    if (c == '"') return str(nullptr);
    if (c == '{') {
      ++i; ws();
      if (i < n && s[i] == '}') { ++i; return true; }
      for (;;) {
        ws(); if (!str(nullptr)) return false;
        ws(); if (i >= n || s[i] != ':') return false; ++i;
        if (!value()) return false;
        ws(); if (i < n && s[i] == ',') { ++i; continue; }
        if (i < n && s[i] == '}') { ++i; return true; }
        return false;
      }
    }
    if (c == '[') {
      ++i; ws();
      if (i < n && s[i] == ']') { ++i; return true; }
      for (;;) {
        if (!value()) return false;
        ws(); if (i < n && s[i] == ',') { ++i; continue; }
        if (i < n && s[i] == ']') { ++i; return true; }
        return false;
      }
    }
    if (lit("true") || lit("false") || lit("null") || lit("NaN") || lit("Infinity") || lit("-Infinity")) return true;
    size_t j = i;
    while (i < n && (strchr("+-0123456789.eE", s[i]) != nullptr)) ++i;
    return i > j;
  }
};

std::string json_escape(const std::string& v) {
  std::string r;
  for (char c : v) {
    switch (c) {
      case '"': r += "\\\""; break; case '\\': r += "\\\\"; break; case '\n': r += "\\n"; break;
      case '\t': r += "\\t"; break; case '\r': r += "\\r"; break; default: r += c; break;
    }
  }
  return r;
}

// parse {"fam": {"sig": <value>, ...}, ...}
bool parse_cache(const std::string& text, Cache* out) {
  Parser p{text.data(), text.size(), 0, true};
  p.ws();
  if (p.i >= p.n || p.s[p.i] != '{') return false;
  ++p.i; p.ws();
  if (p.i < p.n && p.s[p.i] == '}') return true;
  for (;;) {
    std::string fam;
    p.ws(); if (!p.str(&fam)) return false;
    p.ws(); if (p.i >= p.n || p.s[p.i] != ':') return false; ++p.i;
    p.ws(); if (p.i >= p.n || p.s[p.i] != '{') return false; ++p.i;
    SigMap& sm = (*out)[fam];
    p.ws();
    if (p.i < p.n && p.s[p.i] == '}') { ++p.i; }
    else {
      for (;;) {
        std::string sig;
        p.ws(); if (!p.str(&sig)) return false;
        p.ws(); if (p.i >= p.n || p.s[p.i] != ':') return false; ++p.i;
        p.ws();
        const size_t a = p.i;
        if (!p.value()) return false;
        sm[sig] = text.substr(a, p.i - a);
        p.ws(); if (p.i < p.n && p.s[p.i] == ',') { ++p.i; continue; }
        if (p.i < p.n && p.s[p.i] == '}') { ++p.i; break; }
        return false;
      }
    }
    p.ws(); if (p.i < p.n && p.s[p.i] == ',') { ++p.i; continue; }
    if (p.i < p.n && p.s[p.i] == '}') { ++p.i; break; }
    return false;
  }
  p.ws();
  return p.i == p.n;
}

bool read_file(const char* fn, std::string* out) {
  FILE* f = fopen(fn, "rb");
  if (!f) return false;
  char buf[1 << 16];
  size_t r;
  out->clear();
  while ((r = fread(buf, 1, sizeof(buf), f)) > 0) out->append(buf, r);
  fclose(f);
  return true;
}

std::string dump(const Cache& c) {
  std::string r = "{";
  bool f1 = true;
  for (const auto& fam : c) {
    if (!f1) r += ", ";
    f1 = false;
    r += "\"" + json_escape(fam.first) + "\": {";
    bool f2 = true;
    for (const auto& e : fam.second) {
      if (!f2) r += ", ";
      f2 = false;
      r += "\"" + json_escape(e.first) + "\": " + e.second;
    }
    r += "}";
  }
  r += "}";
  return r;
}

const char* kFamilies[5] = {"GEMV", "GEMV_REVSPLITK", "GEMV_SPLITK", "GEMM_SPLITK", "GEMM"};
std::atomic<uint64_t> g_generation{1};          // bumped by every change of the cache: planners memoise against it

}  // namespace

extern "C" int gl_cfg_load(const char* filename, int32_t overwrite) {
  if (filename == nullptr) { gl_set_error("gl_cfg_load: null filename"); return GL_E_INVALID; }
  std::lock_guard<std::mutex> lk(g_mu);
  std::string text;
  if (!read_file(filename, &text)) { gl_set_error("Failed to load the cache file '%s': cannot open", filename); return GL_E_IO; }
  Cache parsed;
  if (!parse_cache(text, &parsed)) { gl_set_error("Failed to load the cache file '%s': not a {family: {signature: config}} JSON object", filename); return GL_E_IO; }
  if (overwrite) g_cache.swap(parsed);
  else for (auto& fam : parsed) { SigMap& dst = g_cache[fam.first]; for (auto& e : fam.second) dst[e.first] = e.second; }
  g_generation.fetch_add(1);
  return GL_OK;
}

extern "C" int gl_cfg_save(const char* filename) {
  if (filename == nullptr) { gl_set_error("gl_cfg_save: null filename"); return GL_E_INVALID; }
  std::lock_guard<std::mutex> lk(g_mu);
  Cache merged;
  std::string text;
  if (read_file(filename, &text)) { Cache old; if (parse_cache(text, &old)) merged.swap(old); }
  for (const char* f : kFamilies) merged[f];                      // every family key is present in a saved file
  for (auto& fam : g_cache) { SigMap& dst = merged[fam.first]; for (auto& e : fam.second) dst[e.first] = e.second; }
  const std::string out = dump(merged);
  FILE* f = fopen(filename, "wb");
  if (!f) { gl_set_error("gl_cfg_save: cannot write '%s'", filename); return GL_E_IO; }
  const size_t w = fwrite(out.data(), 1, out.size(), f);
  fclose(f);
  if (w != out.size()) { gl_set_error("gl_cfg_save: short write to '%s'", filename); return GL_E_IO; }
  return GL_OK;
}

extern "C" void gl_cfg_reset(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_cache.clear();
  g_generation.fetch_add(1);
}

extern "C" int gl_cfg_set(const char* family, const char* signature, const char* json_object) {
  if (!family || !signature || !json_object) { gl_set_error("gl_cfg_set: null argument"); return GL_E_INVALID; }
  Parser p{json_object, strlen(json_object), 0, true};
  p.ws();
  const size_t a = p.i;
  if (!p.value()) { gl_set_error("gl_cfg_set: value is not valid JSON"); return GL_E_INVALID; }
  const size_t b = p.i;
  p.ws();
  if (p.i != p.n) { gl_set_error("gl_cfg_set: trailing characters after the JSON value"); return GL_E_INVALID; }
  std::lock_guard<std::mutex> lk(g_mu);
  g_cache[family][signature] = std::string(json_object + a, b - a);
  g_generation.fetch_add(1);
  return GL_OK;
}

extern "C" const char* gl_cfg_get(const char* family, const char* signature) {
  if (!family || !signature) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  auto f = g_cache.find(family);
  if (f == g_cache.end()) return nullptr;
  auto e = f->second.find(signature);
  if (e == f->second.end()) return nullptr;
  g_tmp = e->second;
  return g_tmp.c_str();
}

// integer field `key` of the JSON object stored for (family, signature), or `dflt`; a cheap early-out when the cache is
// empty keeps the per-launch cost of planners that consult it at one lock
int gl_cfg_int(const char* family, const char* signature, const char* key, int dflt) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_cache.empty()) return dflt;
  auto f = g_cache.find(family);
  if (f == g_cache.end()) return dflt;
  auto e = f->second.find(signature);
  if (e == f->second.end()) return dflt;
  const std::string pat = std::string("\"") + key + "\"";
  size_t pos = e->second.find(pat);
  if (pos == std::string::npos) return dflt;
  pos = e->second.find(':', pos + pat.size());
  if (pos == std::string::npos) return dflt;
  return atoi(e->second.c_str() + pos + 1);
}

uint64_t gl_cfg_generation() { return g_generation.load(); }

extern "C" int64_t gl_cfg_size(const char* family) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (family) { auto f = g_cache.find(family); return f == g_cache.end() ? 0 : (int64_t)f->second.size(); }
  int64_t n = 0;
  for (auto& fam : g_cache) n += (int64_t)fam.second.size();
  return n;
}

// next value >= M of {2^i} U {(2^i + 2^(i+1)) / 2, / 4 : 2^i >= 32, 2^(i+1) <= 4096}, capped at 4096
extern "C" int32_t gl_get_closest_m(int32_t M) {
  const int max_m = 4096;
  if (M > max_m) return max_m;
  int best = max_m;
  for (int v = 1; v <= max_m; v <<= 1) {
    if (v >= M && v < best) best = v;
    const int nxt = v << 1;
    if (v >= 32 && nxt <= max_m) {
      const int a = (v + nxt) / 2, b = (v + nxt) / 4;
      if (a >= M && a < best) best = a;
      if (b >= M && b < best) best = b;
    }
  }
  return best;
}
