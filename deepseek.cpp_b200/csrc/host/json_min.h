// json_min.h — a small JSON document reader for config.json files of layer-list checkpoints (objects, arrays, strings,
// numbers, true / false / null).  Header-only; values are kept as a tree.
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

struct JValue {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  double num = 0;
  bool b = false;
  std::string str;
  std::vector<JValue> arr;
  std::map<std::string, JValue> obj;
  bool has(const char* k) const { return kind == Obj && obj.count(k) && obj.at(k).kind != Null; }
  const JValue& at(const char* k) const { static const JValue none; auto it = obj.find(k); return it == obj.end() ? none : it->second; }
  double number(const char* k, double def) const { return has(k) && at(k).kind == Num ? at(k).num : def; }
  int integer(const char* k, int def) const { return (int)number(k, def); }
};

struct JReader {
  const char* p; const char* end; std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
  bool parse(JValue& v) {
    ws();
    if (p >= end) { err = "unexpected end"; return false; }
    if (*p == '{') {
      v.kind = JValue::Obj; p++; ws();
      if (p < end && *p == '}') { p++; return true; }
      for (;;) {
        JValue k; ws();
        if (p >= end || *p != '"' || !parse(k)) { err = "expected key"; return false; }
        ws();
        if (p >= end || *p != ':') { err = "expected ':'"; return false; }
        p++;
        if (!parse(v.obj[k.str])) return false;
        ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == '}') { p++; return true; }
        err = "expected ',' or '}'"; return false;
      }
    }
    if (*p == '[') {
      v.kind = JValue::Arr; p++; ws();
      if (p < end && *p == ']') { p++; return true; }
      for (;;) {
        v.arr.emplace_back();
        if (!parse(v.arr.back())) return false;
        ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == ']') { p++; return true; }
        err = "expected ',' or ']'"; return false;
      }
    }
    if (*p == '"') {
      v.kind = JValue::Str; p++;
      while (p < end && *p != '"') { if (*p == '\\' && p + 1 < end) p++; v.str += *p++; }
      if (p >= end) { err = "unterminated string"; return false; }
      p++; return true;
    }
    if (end - p >= 4 && std::string(p, 4) == "null") { p += 4; v.kind = JValue::Null; return true; }
    if (end - p >= 4 && std::string(p, 4) == "true") { p += 4; v.kind = JValue::Bool; v.b = true; return true; }
    if (end - p >= 5 && std::string(p, 5) == "false") { p += 5; v.kind = JValue::Bool; v.b = false; return true; }
    char* e = nullptr;
    v.num = strtod(p, &e);
    if (e == p) { err = "unexpected character"; return false; }
    v.kind = JValue::Num; p = e; return true;
  }
};
