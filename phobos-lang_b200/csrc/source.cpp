// Reader for `.ph` kernel declarations and the cluster-level view of a kernel.
//
// Two steps, both host-only:
//  1. parse_kernels: attributes, name and parameter list of every kernel in a source
//     text (grammar: SPEC.md:5-58; shapes: phobos-lang/src/ast.rs:44-92).  The body is
//     kept as a token list; it is never compiled.
//  2. compile_program: what phobos-cluster/src/clustergen.rs derives from a kernel under
//     `@cluster`: which axis of which tensor is cut into supertiles and by which
//     program_id / cluster loop, the access mode of every tensor, the accumulate-step and
//     init leaves of a reduction kernel (clustergen.rs:1131-1224) or the single leaf of a
//     kernel without a cluster loop (flash attention), and the scalar bindings.  Only the
//     statement forms the reference's cluster kernels use are understood: `let` bindings of
//     program_id and of tensor slices, `for v in range(0, DIM, STEP)`, slices
//     `T[start :+ LEN, ...]` / `T[:, ...]`, and a final store `T[...] = [alpha *] acc
//     [+ [beta *] c_old]`.  Anything else in the body is skipped token-wise.
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <set>
#include <sstream>

#include "plan.h"

namespace ph {
namespace plan {
namespace {

// ---- tokens ------------------------------------------------------------------------------------
bool tokenize(const std::string& s, std::vector<Token>* out, std::string* err) {
  int line = 1;
  size_t i = 0;
  auto push = [&](Token::Kind k, std::string t) {
    Token tk;
    tk.kind = k;
    tk.text = std::move(t);
    tk.line = line;
    out->push_back(std::move(tk));
  };
  while (i < s.size()) {
    const char c = s[i];
    if (c == '\n') {
      push(Token::NEWLINE, "\n");
      line++;
      i++;
    } else if (c == ' ' || c == '\t' || c == '\r') {
      i++;
    } else if (c == '/' && i + 1 < s.size() && s[i + 1] == '/') {
      while (i < s.size() && s[i] != '\n') i++;
    } else if (isalpha((unsigned char)c) || c == '_') {
      size_t e = i;
      while (e < s.size() && (isalnum((unsigned char)s[e]) || s[e] == '_')) e++;
      push(Token::IDENT, s.substr(i, e - i));
      i = e;
    } else if (isdigit((unsigned char)c)) {
      size_t e = i;
      while (e < s.size() && isdigit((unsigned char)s[e])) e++;
      bool is_float = false;
      if (e < s.size() && s[e] == '.' && !(e + 1 < s.size() && s[e + 1] == '.')) {
        is_float = true;
        e++;
        while (e < s.size() && isdigit((unsigned char)s[e])) e++;
      }
      push(is_float ? Token::FLOAT : Token::INT, s.substr(i, e - i));
      i = e;
    } else {
      static const char* two[] = {":+", "+=", "==", "!=", "<=", ">="};
      bool done = false;
      for (const char* t : two)
        if (s.compare(i, 2, t) == 0) {
          push(Token::PUNCT, t);
          i += 2;
          done = true;
          break;
        }
      if (done) continue;
      if (strchr("@(){}[]<>,:;=+-*/%!.", c)) {
        push(Token::PUNCT, std::string(1, c));
        i++;
      } else {
        std::ostringstream m;
        m << "line " << line << ": unexpected character '" << c << "'";
        *err = m.str();
        return false;
      }
    }
  }
  push(Token::END, "");
  return true;
}

int dtype_of(const std::string& s) {
  if (s == "f16") return PH_F16;
  if (s == "f32") return PH_F32;
  if (s == "f64") return PH_F64;
  if (s == "i32") return PH_I32;
  if (s == "i64") return PH_I64;
  if (s == "bool") return PH_BOOL;
  return -1;
}

struct Cursor {
  const std::vector<Token>& t;
  size_t i = 0;
  std::string* err;
  const Token& peek() {
    while (t[i].kind == Token::NEWLINE) i++;   // the declaration part ignores line ends
    return t[i];
  }
  bool is(const char* p) {
    const Token& k = peek();
    return (k.kind == Token::PUNCT || k.kind == Token::IDENT) && k.text == p;
  }
  bool fail(const std::string& what) {
    std::ostringstream m;
    const Token& k = peek();
    m << "line " << k.line << ": " << what << " (found '" << (k.kind == Token::END ? "end of input" : k.text) << "')";
    *err = m.str();
    return false;
  }
  bool expect(const char* p) {
    if (!is(p)) return fail(std::string("expected '") + p + "'");
    i++;
    return true;
  }
  bool ident(std::string* out) {
    if (peek().kind != Token::IDENT) return fail("expected an identifier");
    *out = t[i++].text;
    return true;
  }
};

bool parse_attr_arg(Cursor& c, AttrArg* a) {
  const Token& k = c.peek();
  if (k.kind == Token::IDENT && c.t[c.i + 1].kind == Token::IDENT && c.t[c.i + 1].text == "in") {
    a->kind = AttrArg::SEARCH;
    a->name = k.text;
    c.i += 2;
    if (!c.expect("[")) return false;
    while (true) {
      if (c.peek().kind != Token::INT) return c.fail("expected an integer in the search list");
      a->declared.push_back(strtoll(c.t[c.i++].text.c_str(), nullptr, 10));
      if (c.is(",")) {
        c.i++;
        continue;
      }
      break;
    }
    return c.expect("]");
  }
  if (k.kind == Token::IDENT && c.t[c.i + 1].kind == Token::PUNCT && c.t[c.i + 1].text == "=") {
    a->kind = AttrArg::KEYVALUE;
    a->name = k.text;
    c.i += 2;
  } else {
    a->kind = AttrArg::POSITIONAL;
  }
  const Token& v = c.peek();
  if (v.kind != Token::INT && v.kind != Token::FLOAT && v.kind != Token::IDENT) return c.fail("expected a literal");
  a->literal = v.text;
  a->literal_is_int = v.kind == Token::INT;
  if (a->literal_is_int) a->int_value = strtoll(v.text.c_str(), nullptr, 10);
  c.i++;
  return true;
}

bool parse_type(Cursor& c, Param* p) {
  std::string head;
  if (!c.ident(&head)) return false;
  if (head == "tensor" || head == "tile") {
    p->is_tensor = true;
    std::string sc;
    if (!c.expect("<") || !c.ident(&sc) || !c.expect(">") || !c.expect("[")) return false;
    if ((p->dtype = dtype_of(sc)) < 0) return c.fail("unknown scalar type '" + sc + "'");
    while (true) {
      Dim d;
      const Token& k = c.peek();
      if (k.kind == Token::IDENT) {
        d.sym = true;
        d.name = k.text;
      } else if (k.kind == Token::INT) {
        d.value = strtoll(k.text.c_str(), nullptr, 10);
      } else {
        return c.fail("expected a dimension");
      }
      c.i++;
      p->dims.push_back(d);
      if (c.is(",")) {
        c.i++;
        continue;
      }
      break;
    }
    return c.expect("]");
  }
  p->is_tensor = false;
  if ((p->dtype = dtype_of(head)) < 0) return c.fail("unknown type '" + head + "'");
  return true;
}

}  // namespace

std::vector<int64_t> search_choices(const std::vector<int64_t>& d) {
  if (d.size() == 2 && d[0] > 0 && d[1] > d[0]) {
    std::vector<int64_t> out;
    for (int64_t v = d[0]; v < d[1]; v *= 2) out.push_back(v);
    out.push_back(d[1]);
    return out;
  }
  return d;
}

bool parse_kernels(const std::string& text, std::vector<KernelDecl>* out, std::string* err) {
  std::vector<Token> toks;
  if (!tokenize(text, &toks, err)) return false;
  Cursor c{toks, 0, err};
  while (c.peek().kind != Token::END) {
    KernelDecl k;
    while (c.is("@")) {
      c.i++;
      Attribute a;
      if (!c.ident(&a.name)) return false;
      if (c.is("(")) {
        c.i++;
        if (!c.is(")")) {
          while (true) {
            AttrArg arg;
            if (!parse_attr_arg(c, &arg)) return false;
            a.args.push_back(std::move(arg));
            if (c.is(",")) {
              c.i++;
              continue;
            }
            break;
          }
        }
        if (!c.expect(")")) return false;
      }
      k.attrs.push_back(std::move(a));
    }
    if (!c.expect("kernel") || !c.ident(&k.name) || !c.expect("(")) return false;
    if (!c.is(")")) {
      while (true) {
        Param p;
        if (!c.ident(&p.name) || !c.expect(":") || !parse_type(c, &p)) return false;
        k.params.push_back(std::move(p));
        if (c.is(",")) {
          c.i++;
          continue;
        }
        break;
      }
    }
    if (!c.expect(")") || !c.expect("{")) return false;
    int depth = 1;
    while (true) {
      const Token& t = toks[c.i];
      if (t.kind == Token::END) return c.fail("kernel body is not closed");
      if (t.kind == Token::PUNCT && t.text == "{") depth++;
      if (t.kind == Token::PUNCT && t.text == "}" && --depth == 0) break;
      k.body.push_back(t);
      c.i++;
    }
    c.i++;  // the closing brace
    out->push_back(std::move(k));
  }
  if (out->empty()) {
    *err = "source holds no kernel";
    return false;
  }
  return true;
}

// ================================================================================================
// cluster analysis
// ================================================================================================
namespace {

typedef std::vector<Token> Toks;

struct ForInfo {
  std::string var;
  std::vector<Toks> range_args;
};
struct Node {                 // a statement of the body, as far as this reader cares
  enum Kind { LET, FOR, BLOCK, OTHER } kind = OTHER;
  bool is_var = false;        // LET: declared with `var`
  std::string name;           // LET
  Toks expr;                  // LET: right-hand side; OTHER: all tokens
  ForInfo loop;               // FOR
  std::vector<Node> body;     // FOR / BLOCK
  int line = 0;
};

bool is_p(const Token& t, const char* p) { return t.kind == Token::PUNCT && t.text == p; }
bool is_id(const Token& t, const char* p) { return t.kind == Token::IDENT && t.text == p; }

// statements end at a newline or `;` outside any bracket, or before the block's `}`
bool parse_block(const Toks& t, size_t& i, std::vector<Node>* out, std::string* err);

bool parse_braced(const Toks& t, size_t& i, std::vector<Node>* out, std::string* err) {
  if (i >= t.size() || !is_p(t[i], "{")) {
    *err = "expected '{'";
    return false;
  }
  i++;
  if (!parse_block(t, i, out, err)) return false;
  if (i >= t.size() || !is_p(t[i], "}")) {
    *err = "block is not closed";
    return false;
  }
  i++;
  return true;
}

bool parse_block(const Toks& t, size_t& i, std::vector<Node>* out, std::string* err) {
  while (i < t.size()) {
    if (t[i].kind == Token::NEWLINE || is_p(t[i], ";")) {
      i++;
      continue;
    }
    if (is_p(t[i], "}")) return true;
    Node n;
    n.line = t[i].line;
    if (is_id(t[i], "for")) {
      n.kind = Node::FOR;
      if (i + 4 >= t.size() || t[i + 1].kind != Token::IDENT || !is_id(t[i + 2], "in") || !is_id(t[i + 3], "range") ||
          !is_p(t[i + 4], "(")) {
        *err = "line " + std::to_string(n.line) + ": expected `for v in range(...)`";
        return false;
      }
      n.loop.var = t[i + 1].text;
      i += 5;
      int depth = 0;
      Toks cur;
      while (i < t.size()) {
        if (is_p(t[i], "(") || is_p(t[i], "[")) depth++;
        if (is_p(t[i], ")") || is_p(t[i], "]")) {
          if (depth == 0) break;
          depth--;
        }
        if (depth == 0 && is_p(t[i], ",")) {
          n.loop.range_args.push_back(cur);
          cur.clear();
        } else if (t[i].kind != Token::NEWLINE) {
          cur.push_back(t[i]);
        }
        i++;
      }
      n.loop.range_args.push_back(cur);
      i++;  // ')'
      while (i < t.size() && t[i].kind == Token::NEWLINE) i++;
      if (!parse_braced(t, i, &n.body, err)) return false;
    } else if (is_id(t[i], "while") || is_id(t[i], "if")) {
      // condition tokens are skipped; the blocks are walked like any other
      n.kind = Node::BLOCK;
      while (true) {
        while (i < t.size() && !is_p(t[i], "{")) i++;
        if (!parse_braced(t, i, &n.body, err)) return false;
        if (i < t.size() && is_id(t[i], "else")) {
          i++;
          continue;   // `else {` or `else if ... {`
        }
        break;
      }
    } else if (is_id(t[i], "let") || is_id(t[i], "var")) {
      n.kind = Node::LET;
      n.is_var = t[i].text == "var";
      if (i + 1 >= t.size() || t[i + 1].kind != Token::IDENT) {
        *err = "line " + std::to_string(n.line) + ": expected a name after let/var";
        return false;
      }
      n.name = t[i + 1].text;
      i += 2;
      int depth = 0;
      bool seen_eq = false;
      while (i < t.size()) {
        if (is_p(t[i], "(") || is_p(t[i], "[")) depth++;
        if (is_p(t[i], ")") || is_p(t[i], "]")) depth--;
        if (depth == 0 && (t[i].kind == Token::NEWLINE || is_p(t[i], ";") || is_p(t[i], "}"))) break;
        if (!seen_eq && depth == 0 && is_p(t[i], "=")) {
          seen_eq = true;
        } else if (seen_eq && t[i].kind != Token::NEWLINE) {
          n.expr.push_back(t[i]);
        }
        i++;
      }
    } else {
      n.kind = Node::OTHER;
      int depth = 0;
      while (i < t.size()) {
        if (is_p(t[i], "(") || is_p(t[i], "[")) depth++;
        if (is_p(t[i], ")") || is_p(t[i], "]")) depth--;
        if (depth == 0 && (t[i].kind == Token::NEWLINE || is_p(t[i], ";") || is_p(t[i], "}"))) break;
        if (t[i].kind != Token::NEWLINE) n.expr.push_back(t[i]);
        i++;
      }
    }
    out->push_back(std::move(n));
  }
  return true;
}

struct Analyzer {
  const KernelDecl& k;
  std::string* err;
  std::set<std::string> cluster_dims;
  std::vector<int> tensor_param;                 // tensor index -> param index
  std::map<std::string, int> tensor_of, scalar_of;
  std::map<std::string, Toks> lets;              // `let` bindings, by name
  std::set<std::string> vars;                    // names declared with `var`
  struct CLoop { std::string var; Dim dim; std::string sym; };
  std::vector<CLoop> cluster_loops;              // in nesting order, the ones currently open
  std::vector<CLoop> all_cluster_loops;
  // per tensor
  std::vector<bool> have_ref, read, written;
  std::vector<SuperTile> ref;
  std::vector<std::vector<std::string>> syms;
  std::map<int, GridAxis> grid;
  // the store after the reduction loop
  bool have_store = false;
  int store_tensor = -1;
  Toks store_rhs;
  bool store_is_add = false;
  int n_stores = 0;

  bool fail(int line, const std::string& m) {
    *err = "line " + std::to_string(line) + ": " + m;
    return false;
  }

  // expr with every `let` name replaced by its definition (bounded depth)
  Toks expand(const Toks& in, int depth = 0) const {
    Toks out;
    for (const Token& t : in) {
      auto it = t.kind == Token::IDENT ? lets.find(t.text) : lets.end();
      if (it != lets.end() && depth < 8) {
        Toks sub = expand(it->second, depth + 1);
        if (sub.size() > 1) {
          Token l, r;
          l.kind = r.kind = Token::PUNCT;
          l.text = "(";
          r.text = ")";
          out.push_back(l);
          out.insert(out.end(), sub.begin(), sub.end());
          out.push_back(r);
        } else {
          out.insert(out.end(), sub.begin(), sub.end());
        }
      } else {
        out.push_back(t);
      }
    }
    return out;
  }
  static Toks strip_parens(Toks t) {
    while (t.size() >= 2 && is_p(t.front(), "(") && is_p(t.back(), ")")) {
      int depth = 0;
      bool wraps = true;
      for (size_t i = 0; i + 1 < t.size(); i++) {
        if (is_p(t[i], "(")) depth++;
        if (is_p(t[i], ")")) depth--;
        if (depth == 0) {
          wraps = false;
          break;
        }
      }
      if (!wraps) break;
      t = Toks(t.begin() + 1, t.end() - 1);
    }
    return t;
  }
  // program_id(n) -> n, else -1
  static int program_id_of(const Toks& t0) {
    Toks t = strip_parens(t0);
    if (t.size() == 4 && is_id(t[0], "program_id") && is_p(t[1], "(") && t[2].kind == Token::INT && is_p(t[3], ")"))
      return atoi(t[2].text.c_str());
    return -1;
  }

  bool classify(int tensor, const Toks& subs, int line, SuperTile* out) {
    const Param& prm = k.params[tensor_param[tensor]];
    std::vector<Toks> parts;
    {
      int depth = 0;
      Toks cur;
      for (const Token& t : subs) {
        if (is_p(t, "(") || is_p(t, "[")) depth++;
        if (is_p(t, ")") || is_p(t, "]")) depth--;
        if (depth == 0 && is_p(t, ",")) {
          parts.push_back(cur);
          cur.clear();
        } else {
          cur.push_back(t);
        }
      }
      parts.push_back(cur);
    }
    if (parts.size() != prm.dims.size())
      return fail(line, "tensor '" + prm.name + "' has rank " + std::to_string(prm.dims.size()) + " but is indexed with " +
                            std::to_string(parts.size()) + " subscripts");
    out->tensor = tensor;
    out->coords.clear();
    for (size_t ax = 0; ax < parts.size(); ax++) {
      const Toks& s = parts[ax];
      const Dim& dim = prm.dims[ax];
      const std::string own = dim.sym ? dim.name : std::to_string(dim.value);
      Coord co;
      std::string sym = own;
      if (s.size() == 1 && is_p(s[0], ":")) {
        co.kind = Coord::FULL;
      } else {
        int depth = 0;
        size_t split = s.size();
        for (size_t i = 0; i < s.size(); i++) {
          if (is_p(s[i], "(") || is_p(s[i], "[")) depth++;
          if (is_p(s[i], ")") || is_p(s[i], "]")) depth--;
          if (depth == 0 && (is_p(s[i], ":+") || is_p(s[i], ":"))) {
            split = i;
            break;
          }
        }
        if (split == s.size()) return fail(line, "tensor '" + prm.name + "': a point index cannot be supertiled");
        const Toks start(s.begin(), s.begin() + split), len(s.begin() + split + 1, s.end());
        const bool span = is_p(s[split], ":+");
        if (span && len.size() == 1 && len[0].kind == Token::IDENT && cluster_dims.count(len[0].text)) {
          const std::string& S = len[0].text;
          sym = S;
          Toks st = strip_parens(expand(start));
          // a cluster loop variable?
          bool done = false;
          if (st.size() == 1 && st[0].kind == Token::IDENT) {
            for (const CLoop& l : all_cluster_loops)
              if (l.var == st[0].text) {
                if (l.sym != S) return fail(line, "loop '" + l.var + "' steps by " + l.sym + " but the slice is " + S + " long");
                co.kind = Coord::LOOP;
                co.loop = l.var;
                done = true;
              }
          }
          if (!done) {
            // pid * S or S * pid
            int depth2 = 0;
            size_t star = st.size();
            for (size_t i = 0; i < st.size(); i++) {
              if (is_p(st[i], "(")) depth2++;
              if (is_p(st[i], ")")) depth2--;
              if (depth2 == 0 && is_p(st[i], "*")) star = i;
            }
            int pid = -1;
            if (star != st.size()) {
              const Toks a(st.begin(), st.begin() + star), b(st.begin() + star + 1, st.end());
              if (b.size() == 1 && is_id(b[0], S.c_str())) pid = program_id_of(a);
              else if (a.size() == 1 && is_id(a[0], S.c_str())) pid = program_id_of(b);
            }
            if (pid < 0)
              return fail(line, "tensor '" + prm.name + "': the offset of a " + S + "-long slice must be program_id(n) * " + S +
                                    " or the variable of a loop that steps by " + S);
            co.kind = Coord::GRID;
            co.grid = pid;
            auto g = grid.find(pid);
            if (g == grid.end()) {
              GridAxis ga;
              ga.pid = pid;
              ga.dim = dim;
              ga.super_sym = S;
              grid[pid] = ga;
            } else if (g->second.super_sym != S) {
              return fail(line, "program_id(" + std::to_string(pid) + ") tiles by both " + g->second.super_sym + " and " + S);
            }
          }
        } else {
          co.kind = Coord::FULL;   // a device-level slice: the supertile holds the whole axis
        }
      }
      if (syms[tensor][ax].empty()) syms[tensor][ax] = sym;
      else if (syms[tensor][ax] != sym)
        return fail(line, "tensor '" + prm.name + "' axis " + std::to_string(ax) + " is tiled by both " + syms[tensor][ax] +
                              " and " + sym);
      out->coords.push_back(co);
    }
    return true;
  }

  // every tensor reference in a token list; `is_store_target`: the list is the left side of an assignment
  bool scan_refs(const Toks& t, int line, bool is_store_target) {
    for (size_t i = 0; i < t.size(); i++) {
      if (t[i].kind != Token::IDENT) continue;
      auto it = tensor_of.find(t[i].text);
      if (it == tensor_of.end()) continue;
      if (i + 1 >= t.size() || !is_p(t[i + 1], "[")) return fail(line, "tensor '" + t[i].text + "' is used without a slice");
      size_t j = i + 2;
      int depth = 1;
      Toks subs;
      while (j < t.size()) {
        if (is_p(t[j], "[")) depth++;
        if (is_p(t[j], "]") && --depth == 0) break;
        subs.push_back(t[j]);
        j++;
      }
      SuperTile st;
      if (!classify(it->second, subs, line, &st)) return false;
      const int ti = it->second;
      if (have_ref[ti]) {
        if (!(ref[ti].coords == st.coords)) return fail(line, "tensor '" + t[i].text + "' is sliced in two different ways");
      } else {
        have_ref[ti] = true;
        ref[ti] = st;
      }
      (is_store_target ? written : read)[ti] = true;
      i = j;
    }
    return true;
  }

  bool walk(const std::vector<Node>& nodes) {
    for (const Node& n : nodes) {
      if (n.kind == Node::LET) {
        if (n.is_var) vars.insert(n.name);
        else lets[n.name] = n.expr;
        if (!scan_refs(n.expr, n.line, false)) return false;
      } else if (n.kind == Node::FOR) {
        bool cluster = false;
        CLoop cl;
        if (n.loop.range_args.size() == 3 && n.loop.range_args[2].size() == 1 &&
            n.loop.range_args[2][0].kind == Token::IDENT && cluster_dims.count(n.loop.range_args[2][0].text)) {
          const Toks& bound = n.loop.range_args[1];
          if (bound.size() != 1 || (bound[0].kind != Token::IDENT && bound[0].kind != Token::INT))
            return fail(n.line, "the bound of a cluster loop must be a dimension");
          const Toks& lo = n.loop.range_args[0];
          if (lo.size() != 1 || lo[0].kind != Token::INT || lo[0].text != "0") return fail(n.line, "a cluster loop must start at 0");
          cl.var = n.loop.var;
          cl.sym = n.loop.range_args[2][0].text;
          cl.dim.sym = bound[0].kind == Token::IDENT;
          if (cl.dim.sym) cl.dim.name = bound[0].text;
          else cl.dim.value = strtoll(bound[0].text.c_str(), nullptr, 10);
          cluster = true;
          if (!cluster_loops.empty() || !all_cluster_loops.empty())
            return fail(n.line, "more than one cluster loop is not supported");
          cluster_loops.push_back(cl);
          all_cluster_loops.push_back(cl);
        }
        if (!walk(n.body)) return false;
        if (cluster) cluster_loops.pop_back();
      } else if (n.kind == Node::BLOCK) {
        if (!walk(n.body)) return false;
      } else {
        // assignment to a tensor slice?
        const Toks& t = n.expr;
        int depth = 0;
        size_t eq = t.size();
        for (size_t i = 0; i < t.size(); i++) {
          if (is_p(t[i], "(") || is_p(t[i], "[")) depth++;
          if (is_p(t[i], ")") || is_p(t[i], "]")) depth--;
          if (depth == 0 && (is_p(t[i], "=") || is_p(t[i], "+="))) {
            eq = i;
            break;
          }
        }
        if (eq != t.size() && !t.empty() && t[0].kind == Token::IDENT && tensor_of.count(t[0].text)) {
          const Toks lhs(t.begin(), t.begin() + eq), rhs(t.begin() + eq + 1, t.end());
          if (!scan_refs(lhs, n.line, true) || !scan_refs(rhs, n.line, false)) return false;
          n_stores++;
          if (cluster_loops.empty()) {
            have_store = true;
            store_tensor = tensor_of[t[0].text];
            store_rhs = rhs;
            store_is_add = is_p(t[eq], "+=");
          } else {
            return fail(n.line, "a store to a tensor inside the cluster loop is not supported");
          }
        } else {
          if (!scan_refs(t, n.line, false)) return false;
        }
      }
    }
    return true;
  }
};

// splits at `op` outside brackets
std::vector<Toks> split_top(const Toks& t, const char* op) {
  std::vector<Toks> out;
  Toks cur;
  int depth = 0;
  for (const Token& k : t) {
    if (is_p(k, "(") || is_p(k, "[")) depth++;
    if (is_p(k, ")") || is_p(k, "]")) depth--;
    if (depth == 0 && is_p(k, op)) {
      out.push_back(cur);
      cur.clear();
    } else {
      cur.push_back(k);
    }
  }
  out.push_back(cur);
  return out;
}

}  // namespace

bool compile_program(const KernelDecl& k, Program* out, std::string* err) {
  Program p;
  p.name = k.name;
  Analyzer a{k, err};
  std::map<std::string, int64_t> device_tile;
  uint32_t cta = 256;
  for (const Attribute& at : k.attrs) {
    if (at.name == "cluster") {
      for (const AttrArg& arg : at.args) {
        if (arg.kind != AttrArg::SEARCH) {
          *err = "@cluster takes `NAME in [..]` arguments";
          return false;
        }
        SearchDim sd;
        sd.name = arg.name;
        sd.choices = search_choices(arg.declared);
        if (sd.choices.empty()) {
          *err = "@cluster dimension '" + arg.name + "' has no choices";
          return false;
        }
        p.super_dims.push_back(sd);
        a.cluster_dims.insert(arg.name);
      }
    } else if (at.name == "autotune") {
      for (const AttrArg& arg : at.args)
        if (arg.kind == AttrArg::SEARCH && !arg.declared.empty()) device_tile[arg.name] = search_choices(arg.declared)[0];
    } else if (at.name == "launch") {
      // @launch(maxThreads[, minBlocks[, maxRegs]]), phobos-lang/src/ast.rs:103-160
      std::vector<int64_t> ints;
      for (const AttrArg& arg : at.args) {
        if (arg.kind != AttrArg::POSITIONAL || !arg.literal_is_int) {
          *err = "@launch takes integer arguments: @launch(maxThreads[, minBlocks[, maxRegs]])";
          return false;
        }
        ints.push_back(arg.int_value);
      }
      if (ints.empty() || ints.size() > 3) {
        *err = "@launch takes 1 to 3 arguments: @launch(maxThreads[, minBlocks[, maxRegs]])";
        return false;
      }
      if (ints[0] <= 0 || ints[0] % 32 != 0) {
        *err = "@launch maxThreads must be a positive multiple of 32 (got " + std::to_string(ints[0]) + ")";
        return false;
      }
      if (ints.size() > 1 && ints[1] <= 0) {
        *err = "@launch minBlocks must be positive (got " + std::to_string(ints[1]) + ")";
        return false;
      }
      if (ints.size() > 2 && (ints[2] < 16 || ints[2] > 255)) {
        *err = "@launch maxRegs must be between 16 and 255 (got " + std::to_string(ints[2]) + ")";
        return false;
      }
      cta = static_cast<uint32_t>(ints[0]);
    }
  }
  if (p.super_dims.empty()) {
    *err = "kernel '" + k.name + "' has no @cluster attribute";
    return false;
  }
  for (const SearchDim& sd : p.super_dims)
    if (!device_tile.count(sd.name)) {
      *err = "cluster dim '" + sd.name + "' has no @autotune default";   // clustergen.rs:2023-2031
      return false;
    }
  for (size_t i = 0; i < k.params.size(); i++) {
    const Param& prm = k.params[i];
    if (prm.is_tensor) {
      a.tensor_of[prm.name] = static_cast<int>(a.tensor_param.size());
      a.tensor_param.push_back(static_cast<int>(i));
      TensorDecl td;
      td.name = prm.name;
      td.dtype = prm.dtype;
      td.dims = prm.dims;
      p.tensors.push_back(td);
    } else {
      a.scalar_of[prm.name] = static_cast<int>(p.scalars.size());
      ScalarDecl sd;
      sd.name = prm.name;
      sd.dtype = prm.dtype;
      sd.param_pos = static_cast<int>(i);
      p.scalars.push_back(sd);
    }
  }
  const int nt = static_cast<int>(p.tensors.size());
  a.have_ref.assign(nt, false);
  a.read.assign(nt, false);
  a.written.assign(nt, false);
  a.ref.resize(nt);
  a.syms.resize(nt);
  for (int t = 0; t < nt; t++) a.syms[t].assign(p.tensors[t].dims.size(), "");

  std::vector<Node> nodes;
  {
    size_t i = 0;
    Toks body = k.body;
    Token close;
    close.kind = Token::PUNCT;
    close.text = "}";
    body.push_back(close);   // sentinel so the last statement ends like the others
    if (!parse_block(body, i, &nodes, err)) return false;
  }
  if (!a.walk(nodes)) return false;

  for (int t = 0; t < nt; t++) {
    if (!a.have_ref[t]) {
      *err = "tensor '" + p.tensors[t].name + "' is never used";
      return false;
    }
    p.tensors[t].super_syms = a.syms[t];
  }
  if (a.n_stores == 0) {
    *err = "kernel performs no supertile computation";
    return false;
  }
  if (a.n_stores > 1) {
    *err = "kernels with multiple compute statements are not supported under @cluster yet (found " +
           std::to_string(a.n_stores) + ")";
    return false;
  }
  for (auto& g : a.grid) p.grid.push_back(g.second);
  for (size_t i = 0; i < p.grid.size(); i++)
    if (p.grid[i].pid != static_cast<int>(i)) {
      *err = "program_id axes must be 0.." + std::to_string(p.grid.size() - 1);
      return false;
    }

  Leaf step;
  step.entry = k.name;
  step.cta_threads = cta;
  step.device_tile = device_tile;
  std::vector<int> all_scalars;
  for (size_t i = 0; i < p.scalars.size(); i++) all_scalars.push_back(static_cast<int>(i));
  const int out_t = a.store_tensor;

  if (a.all_cluster_loops.empty()) {
    // ---- single leaf (clustergen.rs:246-252, 511-574): the kernel as it is ---------------------
    Stmt c;
    c.leaf = 0;
    for (int t = 0; t < nt; t++) {
      const int mode = a.written[t] ? (a.read[t] ? PH_RMW : PH_WRITE) : PH_READ;
      p.tensors[t].mode = mode;
      step.modes.push_back(mode);
      for (const Coord& co : a.ref[t].coords)
        if (co.kind == Coord::LOOP) {
          *err = "internal: loop coordinate without a cluster loop";
          return false;
        }
      c.args.push_back({a.ref[t], mode});
    }
    c.scalars = all_scalars;
    p.leaves.push_back(step);
    p.body.push_back(c);
    *out = std::move(p);
    return true;
  }

  // ---- accumulator form (clustergen.rs:236-244, 1131-1224) -------------------------------------
  const Analyzer::CLoop& loop = a.all_cluster_loops[0];
  for (const Coord& co : a.ref[out_t].coords)
    if (co.kind == Coord::LOOP) {
      *err = "the output tensor is sliced by the cluster loop";
      return false;
    }
  // epilogue: acc | alpha*acc | [alpha*]acc + c_old | [alpha*]acc + beta*c_old
  std::string acc_name;
  int alpha = -1, beta = -1;
  bool prev = false;
  {
    std::vector<Toks> terms = split_top(a.store_rhs, "+");
    if (a.store_is_add || terms.size() > 2) {
      *err = "unsupported epilogue of the accumulator store";
      return false;
    }
    for (const Toks& term : terms) {
      bool is_acc = false, is_prev = false;
      std::vector<int> term_scalars;
      for (const Toks& f0 : split_top(term, "*")) {
        const Toks f = Analyzer::strip_parens(f0);
        if (f.empty()) {
          *err = "unsupported epilogue of the accumulator store";
          return false;
        }
        if (f.size() == 1 && f[0].kind == Token::IDENT && a.vars.count(f[0].text)) {
          is_acc = true;
          acc_name = f[0].text;
        } else if (f.size() == 1 && f[0].kind == Token::IDENT && a.scalar_of.count(f[0].text)) {
          term_scalars.push_back(a.scalar_of[f[0].text]);
        } else {
          // a previous-value term: a let bound to a slice of the output tensor, or that slice itself
          const Toks e = Analyzer::strip_parens(a.expand(f));
          if (!e.empty() && e[0].kind == Token::IDENT && a.tensor_of.count(e[0].text) && a.tensor_of[e[0].text] == out_t) {
            is_prev = true;
          } else {
            *err = "unsupported epilogue of the accumulator store";
            return false;
          }
        }
      }
      if (is_acc == is_prev || term_scalars.size() > 1) {
        *err = "unsupported epilogue of the accumulator store";
        return false;
      }
      if (is_acc && !term_scalars.empty()) alpha = term_scalars[0];
      if (is_prev) {
        prev = true;
        if (!term_scalars.empty()) beta = term_scalars[0];
      }
    }
    if (acc_name.empty()) {
      *err = "the accumulator tile is never stored to an output tensor";
      return false;
    }
  }
  (void)alpha;
  for (int t = 0; t < nt; t++) p.tensors[t].mode = PH_READ;
  p.tensors[out_t].mode = prev ? PH_RMW : PH_WRITE;

  Stmt stepc;
  stepc.leaf = 0;
  for (int t = 0; t < nt; t++) {
    const int mode = t == out_t ? PH_RMW : PH_READ;
    step.modes.push_back(mode);
    stepc.args.push_back({a.ref[t], mode});
  }
  stepc.scalars = all_scalars;
  p.leaves.push_back(step);

  SuperTile out_tile = a.ref[out_t];
  bool have_init = true;
  Stmt initc;
  initc.leaf = 1;
  if (!prev) {
    // = acc or = alpha*acc: the output starts from zero
    Leaf zi;
    zi.entry = k.name + "_init";
    zi.cta_threads = cta;
    zi.device_tile = device_tile;
    zi.modes = {PH_WRITE};
    p.leaves.push_back(zi);
    initc.args.push_back({out_tile, PH_WRITE});
  } else if (beta < 0) {
    have_init = false;   // + c_old: C keeps its value, no init (clustergen.rs:1192-1200)
  } else {
    // + beta*c_old: C is seeded with beta*C_orig once; the init leaf's beta sits after its one tensor
    Leaf bi;
    bi.entry = k.name + "_init";
    bi.cta_threads = cta;
    bi.device_tile = device_tile;
    bi.modes = {PH_RMW};
    p.leaves.push_back(bi);
    ScalarDecl sd = p.scalars[beta];
    sd.param_pos = 1;
    p.scalars.push_back(sd);
    initc.args.push_back({out_tile, PH_RMW});
    initc.scalars.push_back(static_cast<int>(p.scalars.size()) - 1);
  }
  if (have_init) p.body.push_back(initc);
  Stmt l;
  l.is_loop = true;
  l.var = loop.var;
  l.dim = loop.dim;
  l.super_sym = loop.sym;
  l.body.push_back(stepc);
  p.body.push_back(l);
  *out = std::move(p);
  return true;
}

std::string describe(const Program& p) {
  static const char* modes[] = {"read", "write", "rmw"};
  std::ostringstream o;
  o << "program " << p.name << "\n";
  for (const SearchDim& d : p.super_dims) {
    o << "super " << d.name << " =";
    for (int64_t c : d.choices) o << " " << c;
    o << "\n";
  }
  for (const TensorDecl& t : p.tensors) {
    o << "tensor " << t.name << " " << modes[t.mode] << " dtype" << t.dtype << " [";
    for (size_t i = 0; i < t.dims.size(); i++)
      o << (i ? ", " : "") << (t.dims[i].sym ? t.dims[i].name : std::to_string(t.dims[i].value)) << "/" << t.super_syms[i];
    o << "]\n";
  }
  for (const ScalarDecl& s : p.scalars) o << "scalar " << s.name << " dtype" << s.dtype << " pos " << s.param_pos << "\n";
  for (const Leaf& l : p.leaves) o << "leaf " << l.entry << " cta " << l.cta_threads << "\n";
  for (const GridAxis& g : p.grid)
    o << "grid " << g.pid << " " << (g.dim.sym ? g.dim.name : std::to_string(g.dim.value)) << "/" << g.super_sym << "\n";
  std::function<void(const std::vector<Stmt>&, int)> dump = [&](const std::vector<Stmt>& ss, int ind) {
    for (const Stmt& s : ss) {
      o << std::string(ind * 2, ' ');
      if (s.is_loop) {
        o << "loop " << s.var << " over " << (s.dim.sym ? s.dim.name : std::to_string(s.dim.value)) << "/" << s.super_sym << "\n";
        dump(s.body, ind + 1);
      } else {
        o << "compute leaf " << s.leaf << ":";
        for (const auto& a : s.args) {
          o << " " << p.tensors[a.first.tensor].name << "(";
          for (size_t i = 0; i < a.first.coords.size(); i++) {
            const Coord& c = a.first.coords[i];
            o << (i ? "," : "");
            if (c.kind == Coord::GRID) o << "p" << c.grid;
            else if (c.kind == Coord::LOOP) o << c.loop;
            else o << ":";
          }
          o << ")" << modes[a.second];
        }
        o << " scalars";
        for (int sc : s.scalars) o << " " << p.scalars[sc].name << "@" << p.scalars[sc].param_pos;
        o << "\n";
      }
    }
  };
  dump(p.body, 0);
  return o.str();
}

}  // namespace plan
}  // namespace ph
