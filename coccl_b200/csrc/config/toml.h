// A small TOML reader covering what policy files use: tables ([a.b.c], dotted and quoted
// keys), strings (basic and literal), integers, floats, booleans, arrays and inline tables,
// with duplicate-key detection and line numbers in errors. The reference vendors toml++
// (core/config/third_party/tomlplusplus/toml.hpp); this library carries its own reader.
#pragma once
#include <stdint.h>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace coccl {

struct TomlValue {
  enum Kind { kString, kInteger, kFloat, kBool, kArray, kTable };
  Kind kind = kTable;
  std::string str;
  int64_t integer = 0;
  double real = 0.0;
  bool boolean = false;
  std::vector<TomlValue> items;
  // insertion-ordered table
  std::vector<std::pair<std::string, TomlValue>> entries;
  int line = 0;
  bool explicitTable = false;  // declared by a [header] (as opposed to created as a parent)

  const TomlValue* find(const std::string& key) const;
  TomlValue* find(const std::string& key);
  bool isTable() const { return kind == kTable; }
  const char* kindName() const;
};

// Parses `text`; on failure returns false and sets `error` ("line N: ...").
bool parseToml(const std::string& text, TomlValue* root, std::string* error);
bool parseTomlFile(const std::string& path, TomlValue* root, std::string* error);

}  // namespace coccl
