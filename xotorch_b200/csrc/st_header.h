// st_header.h — minimal JSON reader for the header of a safetensors file (8-byte little-endian length, that many bytes of JSON:
// name -> {dtype, shape, data_offsets}, then the data).  Shared by the shard engine (engine.cu) and the layered-model engine
// (layered.cu).
#pragma once
#include <stdint.h>
#include <stdlib.h>

#include <map>
#include <string>
#include <vector>

struct StEntry {
  std::string dtype;
  std::vector<int64_t> shape;
  int64_t begin = 0, end = 0;
};
struct JsonP {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    ws();
    std::string s;
    if (p >= e || *p != '"') { ok = false; return s; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) { ++p; }
      s.push_back(*p++);
    }
    if (p < e) ++p; else ok = false;
    return s;
  }
  int64_t num() {
    ws();
    char* q = nullptr;
    long long v = strtoll(p, &q, 10);
    if (q == p) ok = false;
    p = q;
    return v;
  }
  void skip() {  // skip any value
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{') { ++p; if (eat('}')) return; do { str(); if (!eat(':')) { ok = false; return; } skip(); } while (ok && eat(',')); if (!eat('}')) ok = false; return; }
    if (*p == '[') { ++p; if (eat(']')) return; do { skip(); } while (ok && eat(',')); if (!eat(']')) ok = false; return; }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

static inline bool parse_st_header(const char* s, size_t n, std::map<std::string, StEntry>& out) {
  JsonP j{s, s + n};
  if (!j.eat('{')) return false;
  if (j.eat('}')) return true;
  do {
    std::string name = j.str();
    if (!j.ok || !j.eat(':')) return false;
    if (name == "__metadata__") { j.skip(); continue; }
    if (!j.eat('{')) return false;
    StEntry en;
    do {
      std::string k = j.str();
      if (!j.eat(':')) return false;
      if (k == "dtype") en.dtype = j.str();
      else if (k == "shape") {
        if (!j.eat('[')) return false;
        if (!j.eat(']')) { do { en.shape.push_back(j.num()); } while (j.eat(',')); if (!j.eat(']')) return false; }
      } else if (k == "data_offsets") {
        if (!j.eat('[')) return false;
        en.begin = j.num(); if (!j.eat(',')) return false; en.end = j.num(); if (!j.eat(']')) return false;
      } else j.skip();
    } while (j.ok && j.eat(','));
    if (!j.eat('}')) return false;
    out[name] = en;
  } while (j.ok && j.eat(','));
  return j.ok && j.eat('}');
}

