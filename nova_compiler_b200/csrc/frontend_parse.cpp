// Parser for the textual nova / linalg subset (see frontend.h).  Syntax follows the op assembly formats of
// the reference dialect (include/Compiler/Dialect/nova/NovaOps.td: matmul :766-768, linear :1055-1057,
// gelu :803-804, softmax :815-828, layer_norm :1027-1037, gather :981-995, reshape :1009-1022,
// transpose :832-843, cast :898-911) and the linalg forms its pipeline tests use.
#include <cctype>
#include <cstdlib>
#include <sstream>

#include "frontend.h"

namespace nova {
namespace fe {
namespace {

struct Cursor {
  const std::string& s;
  size_t i = 0;
  explicit Cursor(const std::string& str) : s(str) {}
  void ws() { while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i; }
  bool eof() { ws(); return i >= s.size(); }
  bool peek(char c) { ws(); return i < s.size() && s[i] == c; }
  bool accept(char c) { if (peek(c)) { ++i; return true; } return false; }
  bool accept(const char* lit) {
    ws();
    size_t n = 0;
    while (lit[n]) ++n;
    if (s.compare(i, n, lit) == 0) { i += n; return true; }
    return false;
  }
  static bool ident_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$' || c == '-'; }
  std::string ident() {
    ws();
    size_t b = i;
    while (i < s.size() && ident_char(s[i])) ++i;
    return s.substr(b, i - b);
  }
  // skips a balanced (...), {...}, [...] or <...> group starting at the current char
  void skip_group() {
    ws();
    int depth = 0;
    bool in_str = false;
    for (; i < s.size(); ++i) {
      const char c = s[i];
      if (c == '"') in_str = !in_str;
      if (in_str) continue;
      if (c == '(' || c == '{' || c == '[' || c == '<') ++depth;
      else if (c == ')' || c == '}' || c == ']' || c == '>') { if (--depth == 0) { ++i; return; } }
    }
  }
};

int32_t elem_dtype(const std::string& t) {
  if (t == "f32") return NOVA_B200_F32;
  if (t == "f16") return NOVA_B200_F16;
  if (t == "bf16") return NOVA_B200_BF16;
  if (t == "i16") return NOVA_B200_I16;
  if (t == "i32") return NOVA_B200_I32;
  if (t == "i64" || t == "index") return NOVA_B200_I64;
  return -1;
}

// tensor<8x16xf32, #nova.device<"1">>  |  memref<1024x1536xf32, 1>  |  f32 (scalar: shape {})
bool parse_type(Cursor& c, Type* out, std::string* err) {
  c.ws();
  const std::string head = c.ident();
  if (head == "tensor" || head == "memref") {
    if (!c.accept('<')) { *err = "expected '<' after " + head; return false; }
    // dims and element type run up to ',' or '>'
    size_t b = c.i;
    int depth = 0;
    size_t end = b, close = std::string::npos;
    for (size_t k = b; k < c.s.size(); ++k) {
      const char ch = c.s[k];
      if (ch == '<') ++depth;
      else if (ch == '>') { if (depth == 0) { close = k; break; } --depth; }
      else if (ch == ',' && depth == 0 && end == b) end = k;
    }
    if (close == std::string::npos) { *err = "unterminated tensor type"; return false; }
    if (end == b) end = close;
    std::string body = c.s.substr(b, end - b);
    c.i = close + 1;
    out->shape.clear();
    size_t p = 0;
    std::string last;
    while (p <= body.size()) {
      size_t x = body.find('x', p);
      std::string tok = body.substr(p, x == std::string::npos ? std::string::npos : x - p);
      // trim
      while (!tok.empty() && std::isspace(static_cast<unsigned char>(tok.back()))) tok.pop_back();
      while (!tok.empty() && std::isspace(static_cast<unsigned char>(tok.front()))) tok.erase(tok.begin());
      if (!tok.empty() && std::isdigit(static_cast<unsigned char>(tok[0])) && x != std::string::npos) {
        out->shape.push_back(std::strtoll(tok.c_str(), nullptr, 10));
      } else {
        // element type (may itself contain an 'x'? no float/int type does); bf16 has no x, index neither
        last = body.substr(p);
        while (!last.empty() && std::isspace(static_cast<unsigned char>(last.back()))) last.pop_back();
        while (!last.empty() && std::isspace(static_cast<unsigned char>(last.front()))) last.erase(last.begin());
        break;
      }
      if (x == std::string::npos) break;
      p = x + 1;
    }
    if (last.find('?') != std::string::npos || body.find('?') != std::string::npos) {
      *err = "dynamic shapes are not supported: " + body;
      return false;
    }
    out->dtype = elem_dtype(last);
    if (out->dtype < 0) { *err = "unsupported element type '" + last + "'"; return false; }
    return true;
  }
  out->shape.clear();
  out->dtype = elem_dtype(head);
  if (out->dtype < 0) { *err = "unsupported type '" + head + "'"; return false; }
  return true;
}

bool parse_type_list(Cursor& c, std::vector<Type>* out, std::string* err) {
  const bool paren = c.accept('(');
  if (paren && c.accept(')')) return true;
  do {
    Type t;
    if (!parse_type(c, &t, err)) return false;
    out->push_back(t);
  } while (c.accept(','));
  if (paren && !c.accept(')')) { *err = "expected ')' after type list"; return false; }
  return true;
}

// %name, %name#2, %name:3
std::string parse_ssa(Cursor& c) {
  c.ws();
  if (!c.accept('%')) return "";
  std::string n = c.ident();
  if (c.i < c.s.size() && c.s[c.i] == '#') {
    ++c.i;
    n += "#" + c.ident();
  }
  return n;
}

// joins physical lines into logical statements: a statement continues while brackets are open
std::vector<std::pair<int, std::string>> logical_lines(const std::string& text) {
  std::vector<std::pair<int, std::string>> out;
  std::istringstream in(text);
  std::string line, cur;
  int depth = 0, lineno = 0, start = 0;
  while (std::getline(in, line)) {
    ++lineno;
    const size_t cm = line.find("//");
    if (cm != std::string::npos) line = line.substr(0, cm);
    bool blank = true;
    for (char ch : line) if (!std::isspace(static_cast<unsigned char>(ch))) blank = false;
    if (blank && depth == 0) continue;
    if (cur.empty()) start = lineno;
    cur += line + " ";
    bool in_str = false;
    for (char ch : line) {
      if (ch == '"') in_str = !in_str;
      if (in_str) continue;
      if (ch == '(' || ch == '[') ++depth;
      else if (ch == ')' || ch == ']') --depth;
    }
    // a function header runs on until the '{' that opens its body
    bool header_open = false;
    {
      size_t b = 0;
      while (b < cur.size() && std::isspace(static_cast<unsigned char>(cur[b]))) ++b;
      if (cur.compare(b, 9, "func.func") == 0) {
        size_t e = cur.size();
        while (e > b && std::isspace(static_cast<unsigned char>(cur[e - 1]))) --e;
        header_open = e == b || cur[e - 1] != '{';
      }
    }
    if (depth <= 0 && !header_open) {
      out.emplace_back(start, cur);
      cur.clear();
      depth = 0;
    }
  }
  if (!cur.empty()) out.emplace_back(start, cur);
  return out;
}

bool fail_at(int line, const std::string& msg, std::string* err) {
  *err = "line " + std::to_string(line) + ": " + msg;
  return false;
}

bool parse_func_header(Cursor& c, int line, Function* f, std::string* err) {
  // func.func [private] @name(%a: T, ...) -> T | (T, T) [attributes {...}] {
  c.accept("private");
  c.ws();
  if (!c.accept('@')) return fail_at(line, "expected @name after func.func", err);
  f->name = c.ident();
  if (!c.accept('(')) return fail_at(line, "expected '(' in function signature", err);
  if (!c.accept(')')) {
    do {
      const std::string n = parse_ssa(c);
      if (n.empty()) return fail_at(line, "expected %argument", err);
      if (!c.accept(':')) return fail_at(line, "expected ':' after argument name", err);
      Type t;
      std::string e;
      if (!parse_type(c, &t, &e)) return fail_at(line, e, err);
      if (c.peek('{')) c.skip_group();  // argument attributes
      f->arg_names.push_back(n);
      f->arg_types.push_back(t);
    } while (c.accept(','));
    if (!c.accept(')')) return fail_at(line, "expected ')' after arguments", err);
  }
  if (c.accept("->")) {
    std::string e;
    if (!parse_type_list(c, &f->result_types, &e)) return fail_at(line, e, err);
  }
  if (c.accept("attributes")) c.skip_group();
  if (!c.accept('{')) return fail_at(line, "expected '{' to open the function body", err);
  return true;
}

bool parse_statement(const std::string& text, int line, Op* op, std::string* err) {
  Cursor c(text);
  op->line = line;
  // results
  if (c.peek('%')) {
    do {
      std::string r = parse_ssa(c);
      if (c.accept(':')) {  // %x:3 = ...
        const int n = std::atoi(c.ident().c_str());
        for (int k = 0; k < n; ++k) op->results.push_back(r + "#" + std::to_string(k));
      } else {
        op->results.push_back(r);
      }
    } while (c.accept(','));
    if (!c.accept('=')) return fail_at(line, "expected '=' after results", err);
  }
  op->name = c.ident();
  if (op->name == "func.return") op->name = "return";
  if (op->name.empty()) return fail_at(line, "expected an operation name", err);

  if (op->name == "arith.constant") {
    // %c = arith.constant 0.000000e+00 : f32   |  dense<...> constants are not supported
    c.ws();
    size_t b = c.i;
    while (c.i < c.s.size() && !std::isspace(static_cast<unsigned char>(c.s[c.i])) && c.s[c.i] != ':') ++c.i;
    const std::string lit = c.s.substr(b, c.i - b);
    if (lit.compare(0, 5, "dense") == 0) return fail_at(line, "dense constants are not supported", err);
    op->fvalue = std::strtod(lit.c_str(), nullptr);
    if (c.accept(':')) {
      Type t;
      std::string e;
      if (!parse_type(c, &t, &e)) return fail_at(line, e, err);
      op->result_types.push_back(t);
    }
    return true;
  }
  if (op->name == "tensor.empty") {
    c.skip_group();  // ()
    if (!c.accept(':')) return fail_at(line, "expected ':' after tensor.empty()", err);
    Type t;
    std::string e;
    if (!parse_type(c, &t, &e)) return fail_at(line, e, err);
    op->result_types.push_back(t);
    return true;
  }
  const bool linalg = op->name.compare(0, 7, "linalg.") == 0;
  if (linalg) {
    if (op->name == "linalg.generic") return fail_at(line, "linalg.generic bodies are outside the supported subset", err);
    // linalg.X ins(%a, %b : Ta, Tb) outs(%c : Tc) -> Tc
    if (c.peek('{')) c.skip_group();
    for (int part = 0; part < 2; ++part) {
      if (!c.accept(part == 0 ? "ins" : "outs")) return fail_at(line, std::string("expected ") + (part == 0 ? "ins(" : "outs("), err);
      if (!c.accept('(')) return fail_at(line, "expected '('", err);
      do {
        const std::string n = parse_ssa(c);
        if (n.empty()) return fail_at(line, "expected %operand", err);
        op->operands.push_back(n);
      } while (c.accept(','));
      if (part == 0) op->num_ins = static_cast<int>(op->operands.size());
      if (!c.accept(':')) return fail_at(line, "expected ':' in ins/outs", err);
      std::string e;
      if (!parse_type_list(c, &op->operand_types, &e)) return fail_at(line, e, err);
      if (!c.accept(')')) return fail_at(line, "expected ')'", err);
    }
    if (c.accept("->")) {
      std::string e;
      if (!parse_type_list(c, &op->result_types, &e)) return fail_at(line, e, err);
    }
    return true;
  }
  // generic nova / bufferization / return form:
  //   op %a, %b [ [%idx] ] [name = int ...] [(name = int)] [{dict}] [restrict|in writable ...] [: types [-> types]]
  for (;;) {
    c.ws();
    if (c.eof()) break;
    if (c.peek('%')) {
      op->operands.push_back(parse_ssa(c));
      c.accept(',');
      continue;
    }
    if (c.accept('[')) {
      while (c.peek('%')) { op->index_operands.push_back(parse_ssa(c)); c.accept(','); }
      if (!c.accept(']')) return fail_at(line, "expected ']'", err);
      continue;
    }
    if (c.peek('{')) {  // attribute dictionary: integer entries (`{dim = -1 : i64}`) are kept, the rest ignored
      const size_t b = c.i;
      c.skip_group();
      const std::string d = c.s.substr(b, c.i - b);
      for (size_t i = 0; i < d.size();) {
        if (!(std::isalpha(static_cast<unsigned char>(d[i])) || d[i] == '_')) { ++i; continue; }
        size_t j = i;
        while (j < d.size() && (std::isalnum(static_cast<unsigned char>(d[j])) || d[j] == '_' || d[j] == '.')) ++j;
        size_t k = j;
        while (k < d.size() && d[k] == ' ') ++k;
        if (k < d.size() && d[k] == '=') {
          ++k;
          while (k < d.size() && d[k] == ' ') ++k;
          if (k < d.size() && (d[k] == '-' || std::isdigit(static_cast<unsigned char>(d[k]))))
            op->attrs[d.substr(i, j - i)] = std::strtoll(d.c_str() + k, nullptr, 10);
        }
        i = j;
      }
      continue;
    }
    if (c.accept('(')) {  // (name = value)
      const std::string k = c.ident();
      if (!c.accept('=')) return fail_at(line, "expected '=' in attribute", err);
      op->attrs[k] = std::strtoll(c.ident().c_str(), nullptr, 10);
      if (!c.accept(')')) return fail_at(line, "expected ')'", err);
      continue;
    }
    if (c.accept(':')) {
      std::string e;
      if (!parse_type_list(c, &op->operand_types, &e)) return fail_at(line, e, err);
      if (c.accept("->")) {
        if (!parse_type_list(c, &op->result_types, &e)) return fail_at(line, e, err);
      }
      break;
    }
    // bare word: attribute name (axis = 0, axes1 = 1) or a keyword (restrict, in, writable)
    const std::string w = c.ident();
    if (w.empty()) return fail_at(line, std::string("unexpected character '") + c.s[c.i] + "'", err);
    if (c.accept('=')) op->attrs[w] = std::strtoll(c.ident().c_str(), nullptr, 10);
  }
  return true;
}

}  // namespace

bool parse_module(const std::string& text, Module* out, std::string* error) {
  Function* cur = nullptr;
  for (const auto& ll : logical_lines(text)) {
    const int line = ll.first;
    Cursor c(ll.second);
    c.ws();
    if (c.eof()) continue;
    if (c.accept("module")) continue;  // `module {` or `module attributes {...} {`
    if (c.accept("func.func")) {
      out->functions.emplace_back();
      cur = &out->functions.back();
      if (!parse_func_header(c, line, cur, error)) return false;
      continue;
    }
    if (c.peek('}')) {  // closes a function or the module
      cur = nullptr;
      continue;
    }
    if (!cur) return fail_at(line, "statement outside a function", error);
    Op op;
    if (!parse_statement(ll.second, line, &op, error)) return false;
    if (op.name == "return") {
      cur->returned = op.operands;
      continue;
    }
    cur->ops.push_back(op);
  }
  if (out->functions.empty()) {
    *error = "no func.func found";
    return false;
  }
  return true;
}

}  // namespace fe
}  // namespace nova
