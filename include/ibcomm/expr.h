// Tiny arithmetic expression compiler for the integration tester.
//
// The reference's tester evaluates user expressions per element with the
// tinyexpr library (ibcomm/allreduce_tester.cpp:62-98, 268-322), which is an
// empty submodule in its checkout.  This is an independent recursive-descent
// compiler to a small stack program, fast enough to run once per element of a
// 128 MiB buffer.
//
// Grammar (all values are double):
//   expr   := term  { ('+'|'-') term }
//   term   := unary { ('*'|'/'|'%') unary }
//   unary  := ('+'|'-') unary | power
//   power  := atom [ '^' unary ]                 (right associative)
//   atom   := number | name | name '(' expr {',' expr} ')' | '(' expr ')'
// Names: variables bound by the caller (the tester binds p, np, n, nb, i), the
// constants pi and e, and the functions abs sqrt floor ceil exp log sin cos
// pow min max fmod.
#pragma once

#include <cctype>
#include <cmath>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace ibcomm {

class ExprError : public std::runtime_error {
 public:
  explicit ExprError(const std::string& s) : std::runtime_error(s) {}
};

class Expr {
 public:
  // `vars` maps a name to the address the value is read from at Eval time.
  Expr(const std::string& text, const std::map<std::string, const double*>& vars)
      : text_(text), vars_(vars) {
    pos_ = 0;
    ParseExpr();
    SkipSpace();
    if (pos_ != text_.size()) Fail("unexpected '" + text_.substr(pos_) + "'");
  }

  double Eval() const {
    double st[64];
    int sp = 0;
    for (const Ins& in : code_) {
      switch (in.op) {
        case kConst: st[sp++] = in.value; break;
        case kVar: st[sp++] = *in.var; break;
        case kAdd: --sp; st[sp - 1] += st[sp]; break;
        case kSub: --sp; st[sp - 1] -= st[sp]; break;
        case kMul: --sp; st[sp - 1] *= st[sp]; break;
        case kDiv: --sp; st[sp - 1] /= st[sp]; break;
        case kMod: --sp; st[sp - 1] = std::fmod(st[sp - 1], st[sp]); break;
        case kPow: --sp; st[sp - 1] = std::pow(st[sp - 1], st[sp]); break;
        case kNeg: st[sp - 1] = -st[sp - 1]; break;
        case kAbs: st[sp - 1] = std::fabs(st[sp - 1]); break;
        case kSqrt: st[sp - 1] = std::sqrt(st[sp - 1]); break;
        case kFloor: st[sp - 1] = std::floor(st[sp - 1]); break;
        case kCeil: st[sp - 1] = std::ceil(st[sp - 1]); break;
        case kExp: st[sp - 1] = std::exp(st[sp - 1]); break;
        case kLog: st[sp - 1] = std::log(st[sp - 1]); break;
        case kSin: st[sp - 1] = std::sin(st[sp - 1]); break;
        case kCos: st[sp - 1] = std::cos(st[sp - 1]); break;
        case kMin: --sp; st[sp - 1] = st[sp - 1] < st[sp] ? st[sp - 1] : st[sp]; break;
        case kMax: --sp; st[sp - 1] = st[sp - 1] > st[sp] ? st[sp - 1] : st[sp]; break;
      }
    }
    return sp == 1 ? st[0] : std::nan("");
  }

 private:
  enum Op { kConst, kVar, kAdd, kSub, kMul, kDiv, kMod, kPow, kNeg, kAbs, kSqrt, kFloor, kCeil, kExp, kLog, kSin, kCos, kMin, kMax };
  struct Ins {
    Op op;
    double value;
    const double* var;
  };

  [[noreturn]] void Fail(const std::string& why) const {
    throw ExprError("Bad expression '" + text_ + "': " + why);
  }
  void SkipSpace() {
    while (pos_ < text_.size() && isspace(static_cast<unsigned char>(text_[pos_]))) ++pos_;
  }
  bool Eat(char c) {
    SkipSpace();
    if (pos_ < text_.size() && text_[pos_] == c) {
      ++pos_;
      return true;
    }
    return false;
  }
  void Emit(Op op, double v = 0, const double* var = nullptr) {
    code_.push_back(Ins{op, v, var});
    depth_ += (op == kConst || op == kVar) ? 1 : (op >= kNeg && op <= kCos ? 0 : -1);
    if (depth_ > 60) Fail("expression too deep");
  }

  void ParseExpr() {
    ParseTerm();
    for (;;) {
      if (Eat('+')) {
        ParseTerm();
        Emit(kAdd);
      } else if (Eat('-')) {
        ParseTerm();
        Emit(kSub);
      } else {
        return;
      }
    }
  }
  void ParseTerm() {
    ParseUnary();
    for (;;) {
      if (Eat('*')) {
        ParseUnary();
        Emit(kMul);
      } else if (Eat('/')) {
        ParseUnary();
        Emit(kDiv);
      } else if (Eat('%')) {
        ParseUnary();
        Emit(kMod);
      } else {
        return;
      }
    }
  }
  void ParseUnary() {
    if (Eat('-')) {
      ParseUnary();
      Emit(kNeg);
    } else if (Eat('+')) {
      ParseUnary();
    } else {
      ParsePower();
    }
  }
  void ParsePower() {
    ParseAtom();
    if (Eat('^')) {
      ParseUnary();
      Emit(kPow);
    }
  }
  void ParseAtom() {
    SkipSpace();
    if (pos_ >= text_.size()) Fail("unexpected end");
    char c = text_[pos_];
    if (c == '(') {
      ++pos_;
      ParseExpr();
      if (!Eat(')')) Fail("')' expected");
      return;
    }
    if (isdigit(static_cast<unsigned char>(c)) || c == '.') {
      const char* begin = text_.c_str() + pos_;
      char* end = nullptr;
      double v = strtod(begin, &end);
      if (end == begin) Fail("number expected");
      pos_ += static_cast<size_t>(end - begin);
      Emit(kConst, v);
      return;
    }
    if (isalpha(static_cast<unsigned char>(c)) || c == '_') {
      size_t b = pos_;
      while (pos_ < text_.size() && (isalnum(static_cast<unsigned char>(text_[pos_])) || text_[pos_] == '_')) ++pos_;
      std::string name = text_.substr(b, pos_ - b);
      if (Eat('(')) {
        int argc = 0;
        if (!Eat(')')) {
          do {
            ParseExpr();
            ++argc;
          } while (Eat(','));
          if (!Eat(')')) Fail("')' expected after arguments of " + name);
        }
        struct F {
          const char* n;
          Op op;
          int argc;
        };
        static const F table[] = {{"abs", kAbs, 1},   {"sqrt", kSqrt, 1}, {"floor", kFloor, 1}, {"ceil", kCeil, 1},
                                  {"exp", kExp, 1},   {"log", kLog, 1},    {"sin", kSin, 1},     {"cos", kCos, 1},
                                  {"pow", kPow, 2},   {"min", kMin, 2},    {"max", kMax, 2},     {"fmod", kMod, 2}};
        for (const F& f : table) {
          if (name == f.n) {
            if (argc != f.argc) Fail(name + " takes " + std::to_string(f.argc) + " argument(s)");
            Emit(f.op);
            return;
          }
        }
        Fail("unknown function " + name);
      }
      auto it = vars_.find(name);
      if (it != vars_.end()) {
        Emit(kVar, 0, it->second);
        return;
      }
      if (name == "pi") {
        Emit(kConst, 3.14159265358979323846);
        return;
      }
      if (name == "e") {
        Emit(kConst, 2.71828182845904523536);
        return;
      }
      Fail("unknown name " + name);
    }
    Fail(std::string("unexpected '") + c + "'");
  }

  std::string text_;
  std::map<std::string, const double*> vars_;
  size_t pos_ = 0;
  int depth_ = 0;
  std::vector<Ins> code_;
};

}  // namespace ibcomm
