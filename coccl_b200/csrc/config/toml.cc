#include "config/toml.h"

#include <stdlib.h>
#include <fstream>
#include <sstream>

namespace coccl {

const TomlValue* TomlValue::find(const std::string& key) const {
  for (const auto& e : entries)
    if (e.first == key) return &e.second;
  return nullptr;
}
TomlValue* TomlValue::find(const std::string& key) {
  for (auto& e : entries)
    if (e.first == key) return &e.second;
  return nullptr;
}
const char* TomlValue::kindName() const {
  switch (kind) {
    case kString: return "string";
    case kInteger: return "integer";
    case kFloat: return "float";
    case kBool: return "boolean";
    case kArray: return "array";
    default: return "table";
  }
}

namespace {

struct Parser {
  const std::string& s;
  size_t pos = 0;
  int line = 1;
  std::string err;

  explicit Parser(const std::string& text) : s(text) {}

  bool fail(const std::string& m) {
    if (err.empty()) err = "line " + std::to_string(line) + ": " + m;
    return false;
  }
  bool eof() const { return pos >= s.size(); }
  char peek() const { return eof() ? '\0' : s[pos]; }
  void skipSpace() {
    while (!eof() && (s[pos] == ' ' || s[pos] == '\t')) ++pos;
  }
  void skipComment() {
    if (peek() == '#')
      while (!eof() && s[pos] != '\n') ++pos;
  }
  // skips blanks, comments and newlines (used between statements and inside arrays)
  void skipBlank() {
    while (!eof()) {
      skipSpace();
      skipComment();
      if (peek() == '\r') { ++pos; continue; }
      if (peek() == '\n') { ++pos; ++line; continue; }
      break;
    }
  }
  bool endOfLine() {
    skipSpace();
    skipComment();
    if (peek() == '\r') ++pos;
    if (eof()) return true;
    if (peek() == '\n') { ++pos; ++line; return true; }
    return fail("unexpected characters after value");
  }

  static bool bareKeyChar(char c) {
    return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_' || c == '-';
  }

  bool parseBasicString(std::string* out) {
    ++pos;  // opening quote
    out->clear();
    while (true) {
      if (eof() || peek() == '\n') return fail("unterminated string");
      char c = s[pos++];
      if (c == '"') return true;
      if (c != '\\') { out->push_back(c); continue; }
      if (eof()) return fail("unterminated escape");
      char e = s[pos++];
      switch (e) {
        case 'n': out->push_back('\n'); break;
        case 't': out->push_back('\t'); break;
        case 'r': out->push_back('\r'); break;
        case '"': out->push_back('"'); break;
        case '\\': out->push_back('\\'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'u': case 'U': {
          const int n = e == 'u' ? 4 : 8;
          if (pos + n > s.size()) return fail("short unicode escape");
          unsigned long cp = strtoul(s.substr(pos, n).c_str(), nullptr, 16);
          pos += n;
          if (cp < 0x80) out->push_back((char)cp);
          else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
          else if (cp < 0x10000) {
            out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
            out->push_back((char)(0x80 | (cp & 0x3F)));
          } else {
            out->push_back((char)(0xF0 | (cp >> 18))); out->push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
            out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F)));
          }
          break;
        }
        default: return fail(std::string("unknown escape \\") + e);
      }
    }
  }
  bool parseLiteralString(std::string* out) {
    ++pos;
    out->clear();
    while (true) {
      if (eof() || peek() == '\n') return fail("unterminated literal string");
      char c = s[pos++];
      if (c == '\'') return true;
      out->push_back(c);
    }
  }

  bool parseKeyPart(std::string* out) {
    skipSpace();
    if (peek() == '"') return parseBasicString(out);
    if (peek() == '\'') return parseLiteralString(out);
    out->clear();
    while (!eof() && bareKeyChar(peek())) out->push_back(s[pos++]);
    if (out->empty()) return fail("expected a key");
    return true;
  }
  bool parseDottedKey(std::vector<std::string>* parts) {
    parts->clear();
    while (true) {
      std::string k;
      if (!parseKeyPart(&k)) return false;
      parts->push_back(k);
      skipSpace();
      if (peek() == '.') { ++pos; continue; }
      return true;
    }
  }

  bool parseNumberOrBool(TomlValue* v) {
    size_t start = pos;
    while (!eof()) {
      char c = peek();
      if (c == ',' || c == ']' || c == '}' || c == '#' || c == '\n' || c == '\r' || c == ' ' || c == '\t') break;
      ++pos;
    }
    std::string tok = s.substr(start, pos - start);
    if (tok.empty()) return fail("expected a value");
    if (tok == "true" || tok == "false") { v->kind = TomlValue::kBool; v->boolean = tok == "true"; return true; }
    std::string clean;
    for (char c : tok) if (c != '_') clean.push_back(c);
    if (clean == "inf" || clean == "+inf" || clean == "-inf" || clean == "nan" || clean == "+nan" || clean == "-nan") {
      v->kind = TomlValue::kFloat; v->real = strtod(clean.c_str(), nullptr); return true;
    }
    bool isFloat = false, hex = clean.size() > 2 && clean[0] == '0' && (clean[1] == 'x' || clean[1] == 'o' || clean[1] == 'b');
    if (!hex) for (char c : clean) if (c == '.' || c == 'e' || c == 'E') isFloat = true;
    char* end = nullptr;
    if (isFloat) {
      v->kind = TomlValue::kFloat;
      v->real = strtod(clean.c_str(), &end);
    } else {
      v->kind = TomlValue::kInteger;
      if (hex) {
        int base = clean[1] == 'x' ? 16 : (clean[1] == 'o' ? 8 : 2);
        v->integer = (int64_t)strtoull(clean.c_str() + 2, &end, base);
      } else {
        v->integer = strtoll(clean.c_str(), &end, 10);
      }
    }
    if (end == nullptr || *end != '\0') return fail("invalid value '" + tok + "'");
    return true;
  }

  bool parseValue(TomlValue* v) {
    skipSpace();
    v->line = line;
    char c = peek();
    if (c == '"') {
      if (s.compare(pos, 3, "\"\"\"") == 0) return fail("multi-line strings are not supported");
      v->kind = TomlValue::kString;
      return parseBasicString(&v->str);
    }
    if (c == '\'') { v->kind = TomlValue::kString; return parseLiteralString(&v->str); }
    if (c == '[') {
      ++pos;
      v->kind = TomlValue::kArray;
      while (true) {
        skipBlank();
        if (peek() == ']') { ++pos; return true; }
        TomlValue item;
        if (!parseValue(&item)) return false;
        v->items.push_back(item);
        skipBlank();
        if (peek() == ',') { ++pos; continue; }
        skipBlank();
        if (peek() == ']') { ++pos; return true; }
        return fail("expected ',' or ']' in array");
      }
    }
    if (c == '{') {
      ++pos;
      v->kind = TomlValue::kTable;
      v->explicitTable = true;
      skipSpace();
      if (peek() == '}') { ++pos; return true; }
      while (true) {
        std::vector<std::string> key;
        if (!parseDottedKey(&key)) return false;
        skipSpace();
        if (peek() != '=') return fail("expected '=' in inline table");
        ++pos;
        TomlValue item;
        if (!parseValue(&item)) return false;
        if (!assign(v, key, item)) return false;
        skipSpace();
        if (peek() == ',') { ++pos; continue; }
        if (peek() == '}') { ++pos; return true; }
        return fail("expected ',' or '}' in inline table");
      }
    }
    return parseNumberOrBool(v);
  }

  // walk/create parent tables for all but the last key part
  TomlValue* descend(TomlValue* t, const std::vector<std::string>& key, size_t upto) {
    for (size_t i = 0; i < upto; ++i) {
      TomlValue* next = t->find(key[i]);
      if (next == nullptr) {
        TomlValue nt;
        nt.kind = TomlValue::kTable;
        nt.line = line;
        t->entries.emplace_back(key[i], nt);
        next = &t->entries.back().second;
      } else if (!next->isTable()) {
        fail("key '" + key[i] + "' is not a table");
        return nullptr;
      }
      t = next;
    }
    return t;
  }
  bool assign(TomlValue* table, const std::vector<std::string>& key, const TomlValue& value) {
    TomlValue* t = descend(table, key, key.size() - 1);
    if (t == nullptr) return false;
    if (t->find(key.back()) != nullptr) return fail("duplicate key '" + key.back() + "'");
    t->entries.emplace_back(key.back(), value);
    return true;
  }

  bool parse(TomlValue* root) {
    root->kind = TomlValue::kTable;
    root->explicitTable = true;
    TomlValue* current = root;
    while (true) {
      skipBlank();
      if (eof()) return true;
      if (peek() == '[') {
        ++pos;
        if (peek() == '[') return fail("arrays of tables are not supported");
        std::vector<std::string> key;
        if (!parseDottedKey(&key)) return false;
        skipSpace();
        if (peek() != ']') return fail("expected ']' after table name");
        ++pos;
        TomlValue* parent = descend(root, key, key.size() - 1);
        if (parent == nullptr) return false;
        TomlValue* t = parent->find(key.back());
        if (t == nullptr) {
          TomlValue nt;
          nt.kind = TomlValue::kTable;
          nt.line = line;
          parent->entries.emplace_back(key.back(), nt);
          t = &parent->entries.back().second;
        } else if (!t->isTable()) {
          return fail("'" + key.back() + "' is already a value");
        } else if (t->explicitTable) {
          return fail("table '" + key.back() + "' is defined twice");
        }
        t->explicitTable = true;
        current = t;
        if (!endOfLine()) return false;
        continue;
      }
      std::vector<std::string> key;
      if (!parseDottedKey(&key)) return false;
      skipSpace();
      if (peek() != '=') return fail("expected '=' after key");
      ++pos;
      TomlValue v;
      if (!parseValue(&v)) return false;
      if (!assign(current, key, v)) return false;
      if (!endOfLine()) return false;
    }
  }
};

}  // namespace

bool parseToml(const std::string& text, TomlValue* root, std::string* error) {
  Parser p(text);
  *root = TomlValue();
  if (p.parse(root) && p.err.empty()) return true;
  if (error) *error = p.err.empty() ? "parse error" : p.err;
  return false;
}

bool parseTomlFile(const std::string& path, TomlValue* root, std::string* error) {
  std::ifstream in(path, std::ios::binary);
  if (!in) {
    if (error) *error = "cannot open '" + path + "'";
    return false;
  }
  std::stringstream ss;
  ss << in.rdbuf();
  return parseToml(ss.str(), root, error);
}

}  // namespace coccl
