// Text -> Expr for one i expression.
//
// Grammar (reference: compiler/src/front/parser.rs:64-98):
//   expr     := [op] pattern [op pattern] '~' pattern [ '|' [splits] '|' perm ]
//   pattern  := [a-z]+ | '.'                         (parser.rs:209-234)
//   splits   := axis ':' int (':' int)* (',' ...)*   (parser.rs:116-141)
//   perm     := ( axis '\''* | '0' | '1' | '!' )*    (parser.rs:143-191)
// A bare `pattern~pattern` is the unary Add (a copy)  (parser.rs:69-72).
// Two-character operator tokens are tried before one-character ones
// (parser.rs:266-296).  Errors are reported in the reference's Debug form
// `ParseError { offset: N, message: "..." }` (core/src/lib.rs:69).
#include "ir.h"

#include <cctype>
#include <cstring>

namespace ib {

const char* op_name(Op op) {
  static const char* names[] = {"Add", "Mul", "Div", "Sub", "Max", "Min", "Pow", "Log", "Gt",
                                "Ge",  "Lt",  "Le",  "Eq",  "Ne",  "And", "Or",  "Xor", "Not"};
  return names[static_cast<int>(op)];
}

const char* op_token(Op op) {
  static const char* toks[] = {"+",  "*",  "/",  "-",  ">",  "<",  "^",  "$",  ">>",
                               ">=", "<<", "<=", "==", "!=", "&&", "||", "^^", "!!"};
  return toks[static_cast<int>(op)];
}

namespace {

struct Fail {
  size_t offset;
  std::string message;
};

bool is_lower(int c) { return c >= 'a' && c <= 'z'; }
bool is_digit(int c) { return c >= '0' && c <= '9'; }

class Cursor {
 public:
  explicit Cursor(const std::string& s) : s_(s) {}

  size_t pos = 0;

  int peek() const { return pos < s_.size() ? static_cast<unsigned char>(s_[pos]) : -1; }
  bool eof() const { return pos >= s_.size(); }
  void skip_ws() {
    while (!eof() && std::isspace(peek())) ++pos;
  }
  bool eat(char c) {
    skip_ws();
    if (peek() == static_cast<unsigned char>(c)) {
      ++pos;
      return true;
    }
    return false;
  }
  void expect(char c, const char* message) {
    if (!eat(c)) throw Fail{pos, message};
  }
  bool starts_with(const char* tok) const { return s_.compare(pos, std::strlen(tok), tok) == 0; }
  std::string slice(size_t a, size_t b) const { return s_.substr(a, b - a); }

 private:
  const std::string& s_;
};

bool read_op(Cursor& c, Op* out) {
  static const struct {
    const char* tok;
    Op op;
  } table[] = {{">>", Op::Gt}, {">=", Op::Ge}, {"<<", Op::Lt},  {"<=", Op::Le}, {"==", Op::Eq},
               {"!=", Op::Ne}, {"&&", Op::And}, {"||", Op::Or}, {"^^", Op::Xor}, {"!!", Op::Not},
               {"+", Op::Add}, {"*", Op::Mul}, {"-", Op::Sub},  {"/", Op::Div}, {">", Op::Max},
               {"<", Op::Min}, {"^", Op::Pow}, {"$", Op::Log}};
  c.skip_ws();
  for (const auto& e : table) {
    if (c.starts_with(e.tok)) {
      c.pos += std::strlen(e.tok);
      *out = e.op;
      return true;
    }
  }
  return false;
}

std::string read_pattern(Cursor& c) {
  c.skip_ws();
  if (c.peek() == '.') {
    ++c.pos;
    if (is_lower(c.peek()) || c.peek() == '.') throw Fail{c.pos, "scalar pattern must be `.`"};
    return std::string();
  }
  std::string axes;
  while (is_lower(c.peek())) {
    axes.push_back(static_cast<char>(c.peek()));
    ++c.pos;
  }
  if (axes.empty()) throw Fail{c.pos, "expected pattern"};
  return axes;
}

char read_axis(Cursor& c) {
  c.skip_ws();
  if (!is_lower(c.peek())) throw Fail{c.pos, "expected axis"};
  char axis = static_cast<char>(c.peek());
  ++c.pos;
  return axis;
}

size_t read_usize(Cursor& c) {
  c.skip_ws();
  size_t start = c.pos;
  while (is_digit(c.peek())) ++c.pos;
  if (c.pos == start) throw Fail{c.pos, "expected integer"};
  std::string digits = c.slice(start, c.pos);
  size_t value = 0;
  for (char d : digits) {
    size_t next = value * 10 + static_cast<size_t>(d - '0');
    if (next / 10 != value) throw Fail{start, "invalid integer"};
    value = next;
  }
  return value;
}

void read_splits(Cursor& c, Expr* e) {
  do {
    char axis = read_axis(c);
    c.expect(':', "expected `:` after split axis");
    std::vector<size_t> factors;
    factors.push_back(read_usize(c));
    while (c.eat(':')) factors.push_back(read_usize(c));
    for (const auto& existing : e->splits)
      if (existing.first == axis)
        throw Fail{c.pos, std::string("duplicate split entry for axis ") + axis};
    e->splits.emplace_back(axis, std::move(factors));
  } while (c.eat(','));
}

void read_permutation(Cursor& c, Expr* e) {
  bool seen_input[2] = {false, false};
  bool seen_bang = false;
  for (;;) {
    c.skip_ws();
    if (c.eof()) break;
    int ch = c.peek();
    if (is_lower(ch)) {
      PermAtom atom;
      atom.kind = PermAtom::Axis;
      atom.axis = read_axis(c);
      while (c.eat('\'')) ++atom.part;
      e->permutation.push_back(atom);
    } else if (is_digit(ch)) {
      if (ch != '0' && ch != '1') throw Fail{c.pos, "expected operand `0` or `1`"};
      ++c.pos;
      size_t which = static_cast<size_t>(ch - '0');
      if (seen_input[which])
        throw Fail{c.pos, "duplicate compute directive for input " + std::to_string(which)};
      seen_input[which] = true;
      PermAtom atom;
      atom.kind = PermAtom::Input;
      atom.input = which;
      e->permutation.push_back(atom);
    } else if (ch == '!') {
      ++c.pos;
      if (seen_bang) throw Fail{c.pos, "duplicate output init directive"};
      seen_bang = true;
      PermAtom atom;
      atom.kind = PermAtom::Bang;
      e->permutation.push_back(atom);
    } else {
      throw Fail{c.pos, "expected axis, `!`, or operand in permutation"};
    }
  }
}

Expr read_expr(Cursor& c) {
  Expr e;
  Op op;
  if (read_op(c, &op)) {
    e.op = op;
    e.inputs.push_back(read_pattern(c));
  } else {
    e.inputs.push_back(read_pattern(c));
    c.skip_ws();
    if (c.peek() == '~') {
      e.op = Op::Add;
    } else {
      if (!read_op(c, &op)) throw Fail{c.pos, "expected operator after input pattern"};
      e.op = op;
      e.inputs.push_back(read_pattern(c));
    }
  }
  c.expect('~', "expected `~` between inputs and output");
  e.output = read_pattern(c);
  if (c.eat('|')) {
    c.skip_ws();
    if (c.peek() != '|') read_splits(c, &e);
    c.expect('|', "expected second `|` in schedule");
    read_permutation(c, &e);
  }
  return e;
}

std::string debug_escape(const std::string& s) {
  std::string out;
  for (char ch : s) {
    if (ch == '"' || ch == '\\') out.push_back('\\');
    out.push_back(ch);
  }
  return out;
}

}  // namespace

Result<Expr> parse_expr(const std::string& src) {
  Cursor c(src);
  try {
    c.skip_ws();
    if (c.eof()) throw Fail{c.pos, "expected i-expression"};
    Expr e = read_expr(c);
    c.skip_ws();
    if (!c.eof()) throw Fail{c.pos, "unexpected trailing input"};
    e.source = src;
    return Result<Expr>::success(std::move(e));
  } catch (const Fail& f) {
    return Result<Expr>::failure("ParseError { offset: " + std::to_string(f.offset) +
                                 ", message: \"" + debug_escape(f.message) + "\" }");
  }
}

}  // namespace ib
