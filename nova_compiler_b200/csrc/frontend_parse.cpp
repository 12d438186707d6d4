// Parser for the textual nova / linalg subset (see frontend.h).  Syntax follows the op assembly formats of
// the reference dialect (include/Compiler/Dialect/nova/NovaOps.td: matmul :766-768, linear :1055-1057,
// gelu :803-804, softmax :815-828, layer_norm :1027-1037, gather :981-995, reshape :1009-1022,
// transpose :832-843, cast :898-911, reduce :191-230, the binary class :600-622) and the linalg forms its
// pipeline tests use (test/pipeline-tests/*.mlir: named contractions, fills, and linalg.generic bias / ReLU
// consumers with their regions).
//
// The parser walks ONE cursor over the whole text, statement by statement, the way the grammar reads: white
// space and line breaks mean nothing (`linalg.matmul ins(...)⏎ outs(...)`, `nova.matmul %a, %b ⏎ : types` and
// multi-line signatures are the reference's own style), `//` comments are blanked out first, and `#name = ...`
// attribute aliases at module level are remembered so that `indexing_maps = [#map0, #map1]` resolves.
#include <cctype>
#include <cstdlib>
#include <map>

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
  // a literal; word-like literals must not be followed by another identifier character
  bool accept(const char* lit) {
    ws();
    size_t n = 0;
    while (lit[n]) ++n;
    if (s.compare(i, n, lit) != 0) return false;
    if (ident_char(lit[n - 1]) && i + n < s.size() && ident_char(s[i + n])) return false;
    i += n;
    return true;
  }
  bool peek_word(const char* lit) {
    const size_t save = i;
    const bool ok = accept(lit);
    i = save;
    return ok;
  }
  static bool ident_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$' || c == '-'; }
  std::string ident() {
    ws();
    size_t b = i;
    while (i < s.size() && ident_char(s[i])) ++i;
    return s.substr(b, i - b);
  }
  // skips a balanced (...), {...}, [...] or <...> group starting at the current char and returns its text;
  // `->` inside affine maps is not a closing bracket
  std::string skip_group() {
    ws();
    const size_t b = i;
    int depth = 0;
    bool in_str = false;
    for (; i < s.size(); ++i) {
      const char c = s[i];
      if (c == '"') in_str = !in_str;
      if (in_str) continue;
      if (c == '-' && i + 1 < s.size() && s[i + 1] == '>') { ++i; continue; }
      if (c == '(' || c == '{' || c == '[' || c == '<') ++depth;
      else if (c == ')' || c == '}' || c == ']' || c == '>') { if (--depth == 0) { ++i; break; } }
    }
    return s.substr(b, i - b);
  }
  int line() const {
    int n = 1;
    for (size_t k = 0; k < i && k < s.size(); ++k) n += s[k] == '\n';
    return n;
  }
};

int32_t elem_dtype(const std::string& t) {
  if (t == "f32") return NOVA_B200_F32;
  if (t == "f16") return NOVA_B200_F16;
  if (t == "bf16") return NOVA_B200_BF16;
  if (t == "i16") return NOVA_B200_I16;
  if (t == "i32") return NOVA_B200_I32;
  if (t == "i64" || t == "index") return NOVA_B200_I64;
  if (t == "i1") return NOVA_B200_I1;
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
      while (!tok.empty() && std::isspace(static_cast<unsigned char>(tok.back()))) tok.pop_back();
      while (!tok.empty() && std::isspace(static_cast<unsigned char>(tok.front()))) tok.erase(tok.begin());
      if (!tok.empty() && std::isdigit(static_cast<unsigned char>(tok[0])) && x != std::string::npos) {
        out->shape.push_back(std::strtoll(tok.c_str(), nullptr, 10));
      } else {
        last = body.substr(p);
        while (!last.empty() && std::isspace(static_cast<unsigned char>(last.back()))) last.pop_back();
        while (!last.empty() && std::isspace(static_cast<unsigned char>(last.front()))) last.erase(last.begin());
        break;
      }
      if (x == std::string::npos) break;
      p = x + 1;
    }
    if (body.find('?') != std::string::npos) {
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

// %name, %name#2
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

bool fail_at(int line, const std::string& msg, std::string* err) {
  *err = "line " + std::to_string(line) + ": " + msg;
  return false;
}

// `dense<1.000000e+00>` (a splat) -> its value
bool parse_dense_splat(const std::string& text, double* v) {
  const size_t d = text.find("dense<");
  if (d == std::string::npos) return false;
  const char* p = text.c_str() + d + 6;
  char* end = nullptr;
  *v = std::strtod(p, &end);
  return end != p && *end == '>';
}

bool parse_func_header(Cursor& c, Function* f, std::string* err) {
  // func.func [private] @name(%a: T {attrs}, ...) -> T | (T, T) [attributes {...}] {
  const int line = c.line();
  c.accept("private");
  c.ws();
  if (!c.accept('@')) return fail_at(line, "expected @name after func.func", err);
  f->name = c.ident();
  if (!c.accept('(')) return fail_at(line, "expected '(' in function signature", err);
  if (!c.accept(')')) {
    do {
      const std::string n = parse_ssa(c);
      if (n.empty()) return fail_at(c.line(), "expected %argument", err);
      if (!c.accept(':')) return fail_at(c.line(), "expected ':' after argument name", err);
      Type t;
      std::string e;
      if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err);
      if (c.peek('{')) c.skip_group();  // argument attributes
      f->arg_names.push_back(n);
      f->arg_types.push_back(t);
    } while (c.accept(','));
    if (!c.accept(')')) return fail_at(c.line(), "expected ')' after arguments", err);
  }
  if (c.accept("->")) {
    std::string e;
    if (!parse_type_list(c, &f->result_types, &e)) return fail_at(c.line(), e, err);
  }
  if (c.accept("attributes")) c.skip_group();
  if (!c.accept('{')) return fail_at(c.line(), "expected '{' to open the function body", err);
  return true;
}

// ins(%a, %b : Ta, Tb) / outs(%c : Tc)
bool parse_ins_outs(Cursor& c, Op* op, const char* kw, std::string* err) {
  if (!c.accept(kw)) return fail_at(c.line(), std::string("expected ") + kw + "(", err);
  if (!c.accept('(')) return fail_at(c.line(), "expected '('", err);
  do {
    const std::string n = parse_ssa(c);
    if (n.empty()) return fail_at(c.line(), "expected %operand", err);
    op->operands.push_back(n);
  } while (c.accept(','));
  if (!c.accept(':')) return fail_at(c.line(), "expected ':' in ins/outs", err);
  std::string e;
  if (!parse_type_list(c, &op->operand_types, &e)) return fail_at(c.line(), e, err);
  if (!c.accept(')')) return fail_at(c.line(), "expected ')'", err);
  return true;
}

// The number of results an affine map text `(d0, d1) -> (d1)` (or an alias resolved to it) produces, and whether
// it is the identity on `rank` dims.
struct MapInfo { int results = 0; bool identity = false; };
MapInfo classify_map(std::string text, const std::map<std::string, std::string>& aliases) {
  while (!text.empty() && std::isspace(static_cast<unsigned char>(text.front()))) text.erase(text.begin());
  if (!text.empty() && text[0] == '#') {
    size_t e = 1;
    while (e < text.size() && Cursor::ident_char(text[e])) ++e;
    auto it = aliases.find(text.substr(0, e));
    if (it != aliases.end()) text = it->second;
  }
  MapInfo mi;
  const size_t arrow = text.find("->");
  if (arrow == std::string::npos) return mi;
  auto names = [](const std::string& part) {
    std::vector<std::string> out;
    const size_t l = part.find('('), r = part.rfind(')');
    if (l == std::string::npos || r == std::string::npos || r <= l) return out;
    std::string cur;
    for (size_t k = l + 1; k <= r; ++k) {
      const char ch = part[k];
      if (ch == ',' || k == r) {
        if (!cur.empty()) out.push_back(cur);
        cur.clear();
      } else if (!std::isspace(static_cast<unsigned char>(ch))) cur += ch;
    }
    return out;
  };
  const std::vector<std::string> dims = names(text.substr(0, arrow)), res = names(text.substr(arrow + 2));
  mi.results = static_cast<int>(res.size());
  mi.identity = dims == res;
  return mi;
}

// linalg.generic {indexing_maps = [...], iterator_types = [...]} ins(...) outs(...) { ^bb0(...): body } -> T
//
// Only the consumers the contraction path meets are recognised, and they are rewritten into the nova op they
// came from so that planning and fusion treat both spellings alike:
//   all-parallel, body `yield addf(in0, in1)`            -> nova.add  (a projected map on one input = broadcast)
//   all-parallel, body `yield addf(in0, out)` (in-place) -> nova.add  (the form FuseMatmulBias.cpp:136-142 accepts)
//   all-parallel, body `yield maximumf(in0, 0.0)`        -> nova.relu
bool parse_generic(Cursor& c, Op* op, const std::map<std::string, double>& scalar_consts,
                   const std::map<std::string, std::string>& aliases, std::string* err) {
  const int line = c.line();
  if (!c.peek('{')) return fail_at(line, "expected the attribute dictionary of linalg.generic", err);
  const std::string dict = c.skip_group();
  if (dict.find("reduction") != std::string::npos)
    return fail_at(line, "linalg.generic with a reduction iterator is outside the supported subset", err);
  std::vector<MapInfo> maps;
  {
    const size_t im = dict.find("indexing_maps");
    const size_t lb = im == std::string::npos ? std::string::npos : dict.find('[', im);
    if (lb == std::string::npos) return fail_at(line, "linalg.generic without indexing_maps", err);
    // split the list at top-level commas
    int depth = 0;
    std::string cur;
    for (size_t k = lb + 1; k < dict.size(); ++k) {
      const char ch = dict[k];
      if (ch == '-' && k + 1 < dict.size() && dict[k + 1] == '>') { cur += "->"; ++k; continue; }
      if (ch == '(' || ch == '<' || ch == '[') ++depth;
      if (ch == ')' || ch == '>') --depth;
      if (ch == ']') { if (depth == 0) { maps.push_back(classify_map(cur, aliases)); break; } --depth; }
      if (ch == ',' && depth == 0) { maps.push_back(classify_map(cur, aliases)); cur.clear(); continue; }
      cur += ch;
    }
  }
  Op io;
  if (!parse_ins_outs(c, &io, "ins", err)) return false;
  const int n_ins = static_cast<int>(io.operands.size());
  if (!parse_ins_outs(c, &io, "outs", err)) return false;
  if (c.accept("attrs")) { c.accept('='); c.skip_group(); }
  if (static_cast<int>(io.operands.size()) != n_ins + 1) return fail_at(line, "linalg.generic: exactly one outs operand is supported", err);
  if (maps.size() != io.operands.size()) return fail_at(line, "linalg.generic: one indexing map per operand expected", err);
  if (!maps.back().identity) return fail_at(line, "linalg.generic: the output map must be the identity", err);
  // region
  if (!c.accept('{')) return fail_at(c.line(), "expected the region of linalg.generic", err);
  if (!c.accept('^')) return fail_at(c.line(), "expected ^bb0", err);
  c.ident();
  std::vector<std::string> bargs;
  if (!c.accept('(')) return fail_at(c.line(), "expected block arguments", err);
  do {
    const std::string a = parse_ssa(c);
    if (a.empty()) return fail_at(c.line(), "expected a block argument", err);
    if (!c.accept(':')) return fail_at(c.line(), "expected ':' after a block argument", err);
    Type t;
    std::string e;
    if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err);
    bargs.push_back(a);
  } while (c.accept(','));
  if (!c.accept(')') || !c.accept(':')) return fail_at(c.line(), "expected '):' after block arguments", err);
  if (bargs.size() != io.operands.size()) return fail_at(line, "linalg.generic: block arguments do not match the operands", err);
  struct BodyOp { std::string res, name, a, b; };
  std::vector<BodyOp> body;
  std::string yielded;
  for (;;) {
    if (c.accept("linalg.yield")) {
      yielded = parse_ssa(c);
      if (c.accept(':')) { Type t; std::string e; if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err); }
      break;
    }
    BodyOp b;
    b.res = parse_ssa(c);
    if (b.res.empty() || !c.accept('=')) return fail_at(c.line(), "expected an operation in the linalg.generic body", err);
    b.name = c.ident();
    b.a = parse_ssa(c);
    if (c.accept(',')) b.b = parse_ssa(c);
    if (c.accept("fastmath")) c.skip_group();
    if (c.accept(':')) { Type t; std::string e; if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err); }
    body.push_back(b);
  }
  if (!c.accept('}')) return fail_at(c.line(), "expected '}' after linalg.yield", err);
  if (c.accept("->")) {
    std::string e;
    if (!parse_type_list(c, &op->result_types, &e)) return fail_at(c.line(), e, err);
  }
  if (body.size() != 1 || body[0].res != yielded)
    return fail_at(line, "linalg.generic body is outside the supported subset (a single addf or maximumf feeding the yield)", err);
  auto arg_index = [&](const std::string& v) {
    for (size_t k = 0; k < bargs.size(); ++k)
      if (bargs[k] == v) return static_cast<int>(k);
    return -1;
  };
  const BodyOp& b = body[0];
  const int ia = arg_index(b.a), ib = arg_index(b.b);
  if (b.name == "arith.addf") {
    if (ia < 0 || ib < 0 || ia == ib) return fail_at(line, "linalg.generic addf must add two different block arguments", err);
    op->name = "nova.add";
    op->operands = {io.operands[ia], io.operands[ib]};
    op->operand_types = {io.operand_types[ia], io.operand_types[ib]};
    op->from_generic = true;
    return true;
  }
  if (b.name == "arith.maximumf" || b.name == "arith.maxnumf" || b.name == "arith.maxf") {
    const int x = ia >= 0 ? ia : ib;
    const std::string& other = ia >= 0 ? b.b : b.a;
    auto it = scalar_consts.find(other);
    if (x < 0 || x >= n_ins || it == scalar_consts.end() || it->second != 0.0)
      return fail_at(line, "linalg.generic maximumf must compare an input with the constant 0.0", err);
    op->name = "nova.relu";
    op->operands = {io.operands[x]};
    op->operand_types = {io.operand_types[x]};
    op->from_generic = true;
    return true;
  }
  return fail_at(line, "linalg.generic body op '" + b.name + "' is outside the supported subset", err);
}

bool parse_statement(Cursor& c, Op* op, std::map<std::string, double>* scalar_consts,
                     const std::map<std::string, std::string>& aliases, std::string* err) {
  op->line = c.line();
  const int line = op->line;
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
  // nova.reduce<sum>, nova.compare<gt>: the kind rides on the name
  if (c.i < c.s.size() && c.s[c.i] == '<') {
    ++c.i;
    op->kind_attr = c.ident();
    if (!c.accept('>')) return fail_at(line, "expected '>' after the op kind", err);
  }

  if (op->name == "return") {
    while (c.peek('%')) { op->operands.push_back(parse_ssa(c)); c.accept(','); }
    if (!op->operands.empty()) {
      if (!c.accept(':')) return fail_at(line, "expected ':' after the returned values", err);
      std::string e;
      if (!parse_type_list(c, &op->operand_types, &e)) return fail_at(c.line(), e, err);
    }
    return true;
  }
  if (op->name == "arith.constant") {
    // %c = arith.constant 0.000000e+00 : f32   |   dense<0.0> : tensor<...> (a splat)
    c.ws();
    size_t b = c.i;
    if (c.s.compare(c.i, 5, "dense") == 0) {
      c.ident();
      const std::string g = c.skip_group();
      if (!parse_dense_splat("dense" + g, &op->fvalue)) return fail_at(line, "only splat dense constants are supported", err);
    } else {
      while (c.i < c.s.size() && !std::isspace(static_cast<unsigned char>(c.s[c.i])) && c.s[c.i] != ':') ++c.i;
      op->fvalue = std::strtod(c.s.substr(b, c.i - b).c_str(), nullptr);
    }
    if (c.accept(':')) {
      Type t;
      std::string e;
      if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err);
      op->result_types.push_back(t);
      if (t.shape.empty() && !op->results.empty()) (*scalar_consts)[op->results[0]] = op->fvalue;
    }
    return true;
  }
  if (op->name == "tensor.empty") {
    c.skip_group();  // ()
    if (!c.accept(':')) return fail_at(line, "expected ':' after tensor.empty()", err);
    Type t;
    std::string e;
    if (!parse_type(c, &t, &e)) return fail_at(c.line(), e, err);
    op->result_types.push_back(t);
    return true;
  }
  if (op->name == "tensor.collapse_shape" || op->name == "tensor.expand_shape") {
    // %r = tensor.collapse_shape %x [[0, 1], [2]] : Tin into Tout   (expand_shape: ... output_shape [..] : Tin into Tout)
    // the metadata reshapes the reference wraps around batch_matmul for rank > 3 operands (NovaToLinalg.cpp:904-989)
    op->name = "nova.reshape";
    op->operands.push_back(parse_ssa(c));
    if (op->operands[0].empty() || !c.peek('[')) return fail_at(line, "expected `%x [[..], ..]`", err);
    c.skip_group();
    if (c.accept("output_shape")) c.skip_group();
    if (!c.accept(':')) return fail_at(line, "expected ':'", err);
    std::string e;
    Type tin, tout;
    if (!parse_type(c, &tin, &e)) return fail_at(c.line(), e, err);
    if (!c.accept("into")) return fail_at(c.line(), "expected `into`", err);
    if (!parse_type(c, &tout, &e)) return fail_at(c.line(), e, err);
    op->operand_types.push_back(tin);
    op->result_types.push_back(tout);
    return true;
  }
  if (op->name == "linalg.generic") return parse_generic(c, op, *scalar_consts, aliases, err);
  if (op->name.compare(0, 7, "linalg.") == 0) {
    // linalg.X [{attrs}] ins(%a, %b : Ta, Tb) outs(%c : Tc) [-> Tc]
    if (c.peek('{')) c.skip_group();
    if (!parse_ins_outs(c, op, "ins", err)) return false;
    op->num_ins = static_cast<int>(op->operands.size());
    if (!parse_ins_outs(c, op, "outs", err)) return false;
    if (c.accept("->")) {
      std::string e;
      if (!parse_type_list(c, &op->result_types, &e)) return fail_at(c.line(), e, err);
    }
    return true;
  }
  // generic nova / bufferization form:
  //   op %a, %b [ [%idx] ] [name = value ...] [(name = int)] [{dict}] [restrict|in writable ...] : types [-> types | to type]
  for (;;) {
    c.ws();
    if (c.eof()) return fail_at(line, "unexpected end of text inside an operation", err);
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
    if (c.peek('{')) {  // attribute dictionary: integer entries (`{dim = -1 : i64}`) and a splat `value` are kept
      const std::string d = c.skip_group();
      double splat = 0.0;
      if (parse_dense_splat(d, &splat)) op->fvalue = splat;
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
          else if (d.compare(k, 4, "true") == 0) op->attrs[d.substr(i, j - i)] = 1;
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
      if (!parse_type_list(c, &op->operand_types, &e)) return fail_at(c.line(), e, err);
      if (c.accept("->") || c.accept("to")) {
        if (!parse_type_list(c, &op->result_types, &e)) return fail_at(c.line(), e, err);
      }
      return true;
    }
    // bare word: attribute name (axis = 0, dimension = [0, 1], keepdims = true) or a keyword (restrict, in, writable)
    const std::string w = c.ident();
    if (w.empty()) return fail_at(line, std::string("unexpected character '") + c.s[c.i] + "'", err);
    if (c.accept('=')) {
      if (c.accept('[')) {
        std::vector<int64_t>& list = op->int_lists[w];
        while (!c.peek(']')) {
          list.push_back(std::strtoll(c.ident().c_str(), nullptr, 10));
          if (!c.accept(',')) break;
        }
        if (!c.accept(']')) return fail_at(line, "expected ']' after the list attribute", err);
      } else {
        const std::string v = c.ident();
        op->attrs[w] = v == "true" ? 1 : (v == "false" ? 0 : std::strtoll(v.c_str(), nullptr, 10));
      }
    }
  }
}

}  // namespace

bool parse_module(const std::string& raw, Module* out, std::string* error) {
  // blank out `//` comments (line structure, hence line numbers, is kept)
  std::string text = raw;
  {
    bool in_str = false;
    for (size_t i = 0; i < text.size(); ++i) {
      if (text[i] == '"') in_str = !in_str;
      if (text[i] == '\n') in_str = false;
      if (!in_str && text[i] == '/' && i + 1 < text.size() && text[i + 1] == '/')
        while (i < text.size() && text[i] != '\n') text[i++] = ' ';
    }
  }
  Cursor c(text);
  std::map<std::string, std::string> aliases;  // #map0 -> affine_map<...>
  int module_depth = 0;
  while (!c.eof()) {
    if (c.accept("module")) {  // `module {`, `module @name {`, `module attributes {...} {`
      if (c.accept('@')) c.ident();
      if (c.accept("attributes")) c.skip_group();
      if (!c.accept('{')) return fail_at(c.line(), "expected '{' after module", error);
      ++module_depth;
      continue;
    }
    if (c.peek('}')) {
      c.accept('}');
      if (--module_depth < 0) return fail_at(c.line(), "unbalanced '}'", error);
      continue;
    }
    if (c.peek('#')) {  // #name = affine_map<...>
      const int line = c.line();
      c.accept('#');
      const std::string name = "#" + c.ident();
      if (!c.accept('=')) return fail_at(line, "expected '=' in the attribute alias", error);
      c.ident();  // affine_map, or another attribute kind (kept as text)
      aliases[name] = c.peek('<') ? c.skip_group() : std::string();
      continue;
    }
    if (c.accept("func.func")) {
      out->functions.emplace_back();
      Function* f = &out->functions.back();
      if (!parse_func_header(c, f, error)) return false;
      std::map<std::string, double> scalar_consts;
      for (;;) {
        if (c.eof()) return fail_at(c.line(), "unterminated function body", error);
        if (c.accept('}')) break;
        Op op;
        if (!parse_statement(c, &op, &scalar_consts, aliases, error)) return false;
        if (op.name == "return") {
          f->returned = op.operands;
          continue;
        }
        f->ops.push_back(op);
      }
      continue;
    }
    return fail_at(c.line(), "statement outside a function", error);
  }
  if (out->functions.empty()) {
    *error = "no func.func found";
    return false;
  }
  return true;
}

}  // namespace fe
}  // namespace nova
