// Grammar engine: JSON-schema / regex / structural grammars -> byte-level matcher -> token allow-masks.
//
// A grammar is a small node graph (literal, byte class, sequence, alternative, bounded repeat, rule reference).
// It is built from a JSON description:
//   {"lit": "text"} {"chars": "[a-z0-9_]"} {"seq": [...]} {"alt": [...]} {"repeat": [node, min, max]} (max < 0: unbounded)
//   {"schema": <JSON schema>}   {"regex": "pattern"}   {"json": true} (any JSON value)   {"until": "stop"} (free text
//   that ends at the first occurrence of the stop string, which is consumed)   {"text_without": "stop"} (free text
//   that may end anywhere and never contains the stop string: with {"until": stop} beside it in an "alt" this is the
//   triggered form used for optional tool calls - plain text, or text up to a trigger tag and then a structure)
// The matcher simulates the graph with a set of continuation stacks (the grammars used here are near-deterministic,
// so the set stays small), can be forked cheaply for per-draft-row verification masks, and fills a packed allow-mask
// by walking a byte trie of the vocabulary so tokens sharing a prefix share the work.
// JSON whitespace is bounded to 16 characters per boundary.
// Replaces the reference's XGrammar adapter (native/src/xgrammar_adapter.cc:25-28,60-89,238-376); schema keywords
// supported: type, properties, required, items, minItems, maxItems, enum, const, anyOf, oneOf, $ref into $defs,
// additionalProperties=false semantics, integer/number/string/boolean/null.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------------------ tiny JSON
struct JVal {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;          // Str; for Num the original text
  std::vector<JVal> arr;
  std::vector<std::pair<std::string, JVal>> obj;   // insertion order preserved
  const JVal* get(const std::string& k) const {
    for (const auto& kv : obj)
      if (kv.first == k) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char* p;
  const char* end;
  bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool lit(const char* s) {
    const size_t n = std::strlen(s);
    if (static_cast<size_t>(end - p) >= n && std::memcmp(p, s, n) == 0) { p += n; return true; }
    return false;
  }
  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 63))); }
    else if (cp < 0x10000) {
      out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 63)));
      out.push_back(static_cast<char>(0x80 | (cp & 63)));
    } else {
      out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 63)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 63)));
      out.push_back(static_cast<char>(0x80 | (cp & 63)));
    }
  }
  std::string string() {
    std::string out;
    if (p >= end || *p != '"') { ok = false; return out; }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            if (end - p < 5) { ok = false; return out; }
            uint32_t cp = static_cast<uint32_t>(std::strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16));
            p += 4;
            if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 7 && p[1] == '\\' && p[2] == 'u') {
              const uint32_t lo = static_cast<uint32_t>(std::strtoul(std::string(p + 3, p + 7).c_str(), nullptr, 16));
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
              p += 6;
            }
            utf8(out, cp);
            break;
          }
          default: out.push_back(*p);
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  JVal value() {
    JVal v;
    ws();
    if (p >= end) { ok = false; return v; }
    if (*p == '{') {
      ++p;
      v.kind = JVal::Obj;
      ws();
      if (p < end && *p == '}') { ++p; return v; }
      while (ok) {
        ws();
        std::string k = string();
        ws();
        if (p >= end || *p != ':') { ok = false; break; }
        ++p;
        v.obj.emplace_back(k, value());
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; break; }
        ok = false;
      }
    } else if (*p == '[') {
      ++p;
      v.kind = JVal::Arr;
      ws();
      if (p < end && *p == ']') { ++p; return v; }
      while (ok) {
        v.arr.push_back(value());
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; break; }
        ok = false;
      }
    } else if (*p == '"') {
      v.kind = JVal::Str;
      v.str = string();
    } else if (lit("true")) { v.kind = JVal::Bool; v.b = true; }
    else if (lit("false")) { v.kind = JVal::Bool; v.b = false; }
    else if (lit("null")) { v.kind = JVal::Null; }
    else {
      const char* s = p;
      while (p < end && (std::strchr("+-.eE", *p) != nullptr || (*p >= '0' && *p <= '9'))) ++p;
      if (p == s) { ok = false; return v; }
      v.kind = JVal::Num;
      v.str.assign(s, p);
      v.num = std::strtod(v.str.c_str(), nullptr);
    }
    return v;
  }
};

std::string json_quote(const std::string& s) {
  std::string o = "\"";
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\t': o += "\\t"; break;
      case '\r': o += "\\r"; break;
      default:
        if (c < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", c); o += buf; }
        else o.push_back(static_cast<char>(c));
    }
  }
  return o + "\"";
}

std::string json_dump(const JVal& v) {
  switch (v.kind) {
    case JVal::Null: return "null";
    case JVal::Bool: return v.b ? "true" : "false";
    case JVal::Num: return v.str;
    case JVal::Str: return json_quote(v.str);
    case JVal::Arr: {
      std::string o = "[";
      for (size_t i = 0; i < v.arr.size(); ++i) o += (i ? "," : "") + json_dump(v.arr[i]);
      return o + "]";
    }
    default: {
      std::string o = "{";
      for (size_t i = 0; i < v.obj.size(); ++i)
        o += (i ? "," : "") + json_quote(v.obj[i].first) + ":" + json_dump(v.obj[i].second);
      return o + "}";
    }
  }
}

// ------------------------------------------------------------------------------------------------ grammar graph
struct CharSet {
  uint64_t w[4] = {0, 0, 0, 0};
  void set(int c) { w[c >> 6] |= 1ull << (c & 63); }
  void range(int a, int b) { for (int c = a; c <= b; ++c) set(c); }
  bool has(int c) const { return (w[c >> 6] >> (c & 63)) & 1ull; }
  void invert() { for (auto& x : w) x = ~x; }
};

struct Node {
  enum Kind { Lit, Chars, Seq, Alt, Repeat, Ref, Until, Free } kind = Lit;
  std::string lit;            // Lit / Until / Free (stop string)
  CharSet cs;                 // Chars
  std::vector<int> kids;      // Seq / Alt / Repeat[0] / Ref[0]
  int rmin = 0, rmax = -1;
};

struct MaskCache;

struct Grammar {
  std::vector<Node> nodes;
  int root = -1;
  std::shared_ptr<MaskCache> masks;      // allow-masks by matcher state (free text sits in one state for long)
  std::string error;
  std::map<std::string, int> defs;       // $defs name -> node
  const JVal* schema_root = nullptr;
  int json_value = -1;                    // generic JSON value rule (lazily built)

  int add(Node n) { nodes.push_back(std::move(n)); return static_cast<int>(nodes.size()) - 1; }
  int lit(const std::string& s) { Node n; n.kind = Node::Lit; n.lit = s; return add(n); }
  int chars(const CharSet& c) { Node n; n.kind = Node::Chars; n.cs = c; return add(n); }
  int seq(std::vector<int> k) { if (k.size() == 1) return k[0]; Node n; n.kind = Node::Seq; n.kids = std::move(k); return add(n); }
  int alt(std::vector<int> k) { if (k.size() == 1) return k[0]; Node n; n.kind = Node::Alt; n.kids = std::move(k); return add(n); }
  int repeat(int child, int mn, int mx) { Node n; n.kind = Node::Repeat; n.kids = {child}; n.rmin = mn; n.rmax = mx; return add(n); }
  int opt(int child) { return repeat(child, 0, 1); }
  int ref_placeholder() { Node n; n.kind = Node::Ref; n.kids = {-1}; return add(n); }

  int ws() {
    CharSet c; c.set(' '); c.set('\n'); c.set('\t'); c.set('\r');
    return repeat(chars(c), 0, 16);
  }
  int digits(int mn) { CharSet d; d.range('0', '9'); return repeat(chars(d), mn, -1); }
  int integer() {
    CharSet nz; nz.range('1', '9');
    return seq({opt(lit("-")), alt({lit("0"), seq({chars(nz), digits(0)})})});
  }
  int number() {
    CharSet e; e.set('e'); e.set('E');
    CharSet sg; sg.set('+'); sg.set('-');
    return seq({integer(), opt(seq({lit("."), digits(1)})), opt(seq({chars(e), opt(chars(sg)), digits(1)}))});
  }
  int string_body() {
    CharSet plain; plain.range(0x20, 0xFF);
    plain.w['"' >> 6] &= ~(1ull << ('"' & 63));
    plain.w['\\' >> 6] &= ~(1ull << ('\\' & 63));
    CharSet esc; for (char c : std::string("\"\\/bfnrt")) esc.set(c);
    CharSet hex; hex.range('0', '9'); hex.range('a', 'f'); hex.range('A', 'F');
    const int u = seq({lit("u"), repeat(chars(hex), 4, 4)});
    return repeat(alt({chars(plain), seq({lit("\\"), alt({chars(esc), u})})}), 0, -1);
  }
  int string() { return seq({lit("\""), string_body(), lit("\"")}); }

  int any_json() {
    if (json_value >= 0) return json_value;
    const int self = ref_placeholder();
    json_value = self;
    const int member = seq({string(), ws(), lit(":"), ws(), self});
    const int object = seq({lit("{"), ws(), opt(seq({member, repeat(seq({ws(), lit(","), ws(), member}), 0, -1)})), ws(), lit("}")});
    const int array = seq({lit("["), ws(), opt(seq({self, repeat(seq({ws(), lit(","), ws(), self}), 0, -1)})), ws(), lit("]")});
    nodes[self].kids[0] = alt({object, array, string(), number(), lit("true"), lit("false"), lit("null")});
    return self;
  }

  int schema(const JVal& s);
  int object_schema(const JVal& s);
  int build(const JVal& d);
  int regex(const std::string& pattern);
};

int Grammar::object_schema(const JVal& s) {
  const JVal* props = s.get("properties");
  std::set<std::string> required;
  if (const JVal* r = s.get("required"))
    for (const auto& x : r->arr) required.insert(x.str);
  if (props == nullptr || props->obj.empty()) {
    const JVal* ap = s.get("additionalProperties");
    if (ap != nullptr && ap->kind == JVal::Bool && !ap->b) return seq({lit("{"), ws(), lit("}")});
    // free-form object
    const int member = seq({string(), ws(), lit(":"), ws(), any_json()});
    return seq({lit("{"), ws(), opt(seq({member, repeat(seq({ws(), lit(","), ws(), member}), 0, -1)})), ws(), lit("}")});
  }
  const int n = static_cast<int>(props->obj.size());
  std::vector<int> member(n);
  std::vector<bool> req(n);
  for (int i = 0; i < n; ++i) {
    member[i] = seq({lit(json_quote(props->obj[i].first)), ws(), lit(":"), ws(), schema(props->obj[i].second)});
    req[i] = required.count(props->obj[i].first) != 0;
  }
  // rest[i][first]: members i.. in declared order; optional ones may be skipped; commas between present ones
  std::vector<int> rest_first(n + 1), rest_more(n + 1);
  const int close = seq({ws(), lit("}")});
  rest_first[n] = rest_more[n] = close;
  for (int i = n - 1; i >= 0; --i) {
    for (int first = 0; first < 2; ++first) {
      std::vector<int> options;
      for (int j = i; j < n; ++j) {
        std::vector<int> parts;
        if (!first) { parts.push_back(ws()); parts.push_back(lit(",")); }
        parts.push_back(ws());
        parts.push_back(member[j]);
        parts.push_back(rest_more[j + 1]);
        options.push_back(seq(parts));
        if (req[j]) break;                       // cannot skip a required member
        if (j == n - 1) options.push_back(close);
      }
      (first ? rest_first : rest_more)[i] = alt(options);
    }
  }
  return seq({lit("{"), rest_first[0]});
}

int Grammar::schema(const JVal& s) {
  if (s.kind == JVal::Bool) return any_json();
  if (s.kind != JVal::Obj) { error = "schema must be an object"; return lit(""); }
  if (const JVal* r = s.get("$ref")) {
    const std::string& path = r->str;
    const std::string pre1 = "#/$defs/", pre2 = "#/definitions/";
    std::string name;
    const char* table = nullptr;
    if (path.compare(0, pre1.size(), pre1) == 0) { name = path.substr(pre1.size()); table = "$defs"; }
    else if (path.compare(0, pre2.size(), pre2) == 0) { name = path.substr(pre2.size()); table = "definitions"; }
    else { error = "unsupported $ref " + path; return lit(""); }
    auto it = defs.find(name);
    if (it != defs.end()) return it->second;
    const JVal* t = schema_root != nullptr ? schema_root->get(table) : nullptr;
    const JVal* target = t != nullptr ? t->get(name) : nullptr;
    if (target == nullptr) { error = "unresolved $ref " + path; return lit(""); }
    const int ph = ref_placeholder();
    defs[name] = ph;
    nodes[ph].kids[0] = schema(*target);
    return ph;
  }
  if (const JVal* c = s.get("const")) return lit(json_dump(*c));
  if (const JVal* e = s.get("enum")) {
    std::vector<int> o;
    for (const auto& v : e->arr) o.push_back(lit(json_dump(v)));
    if (o.empty()) { error = "empty enum"; return lit(""); }
    return alt(o);
  }
  for (const char* key : {"anyOf", "oneOf"})
    if (const JVal* a = s.get(key)) {
      std::vector<int> o;
      for (const auto& v : a->arr) o.push_back(schema(v));
      if (o.empty()) { error = "empty anyOf"; return lit(""); }
      return alt(o);
    }
  const JVal* t = s.get("type");
  if (t == nullptr) {
    if (s.get("properties") != nullptr) return object_schema(s);
    return any_json();
  }
  if (t->kind == JVal::Arr) {
    std::vector<int> o;
    for (const auto& v : t->arr) {
      JVal one = s;
      for (auto& kv : one.obj)
        if (kv.first == "type") kv.second = v;
      o.push_back(schema(one));
    }
    return alt(o);
  }
  const std::string& ty = t->str;
  if (ty == "object") return object_schema(s);
  if (ty == "array") {
    const JVal* items = s.get("items");
    const int item = items != nullptr ? schema(*items) : any_json();
    int mn = 0, mx = -1;
    if (const JVal* v = s.get("minItems")) mn = static_cast<int>(v->num);
    if (const JVal* v = s.get("maxItems")) mx = static_cast<int>(v->num);
    if (mx == 0) return seq({lit("["), ws(), lit("]")});
    const int more = repeat(seq({ws(), lit(","), ws(), item}), mn > 0 ? mn - 1 : 0, mx < 0 ? -1 : mx - 1);
    const int body = seq({item, more});
    return seq({lit("["), ws(), mn > 0 ? body : opt(body), ws(), lit("]")});
  }
  if (ty == "string") {
    if (const JVal* pat = s.get("pattern")) return seq({lit("\""), regex(pat->str), lit("\"")});
    return string();
  }
  if (ty == "integer") return integer();
  if (ty == "number") return number();
  if (ty == "boolean") return alt({lit("true"), lit("false")});
  if (ty == "null") return lit("null");
  error = "unsupported schema type " + ty;
  return lit("");
}

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------ regex subset
// literals, escapes (\d \w \s \. ...), classes [a-z] [^...], '.', groups (...), alternation |, quantifiers * + ? {m} {m,} {m,n}
struct RegexParser {
  Grammar* g;
  const std::string& s;
  size_t i = 0;
  bool ok = true;
  RegexParser(Grammar* gr, const std::string& str) : g(gr), s(str) {}

  CharSet escape_class(char c, bool* is_class) {
    CharSet cs;
    *is_class = true;
    switch (c) {
      case 'd': cs.range('0', '9'); break;
      case 'w': cs.range('0', '9'); cs.range('a', 'z'); cs.range('A', 'Z'); cs.set('_'); break;
      case 's': cs.set(' '); cs.set('\t'); cs.set('\n'); cs.set('\r'); break;
      case 'D': cs.range('0', '9'); cs.invert(); break;
      case 'W': cs.range('0', '9'); cs.range('a', 'z'); cs.range('A', 'Z'); cs.set('_'); cs.invert(); break;
      case 'S': cs.set(' '); cs.set('\t'); cs.set('\n'); cs.set('\r'); cs.invert(); break;
      case 'n': cs.set('\n'); break;
      case 't': cs.set('\t'); break;
      case 'r': cs.set('\r'); break;
      default: cs.set(static_cast<unsigned char>(c)); *is_class = false;
    }
    return cs;
  }
  int atom() {
    if (i >= s.size()) { ok = false; return g->lit(""); }
    const char c = s[i];
    if (c == '(') {
      ++i;
      if (s.compare(i, 2, "?:") == 0) i += 2;
      const int inner = alternation();
      if (i >= s.size() || s[i] != ')') { ok = false; return inner; }
      ++i;
      return inner;
    }
    if (c == '[') {
      ++i;
      CharSet cs;
      bool neg = false;
      if (i < s.size() && s[i] == '^') { neg = true; ++i; }
      bool first = true;
      while (i < s.size() && (s[i] != ']' || first)) {
        first = false;
        int lo;
        if (s[i] == '\\' && i + 1 < s.size()) {
          bool is_class;
          const CharSet e = escape_class(s[i + 1], &is_class);
          i += 2;
          if (is_class) { for (int k = 0; k < 4; ++k) cs.w[k] |= e.w[k]; continue; }
          lo = static_cast<unsigned char>(s[i - 1]);
        } else {
          lo = static_cast<unsigned char>(s[i++]);
        }
        if (i + 1 < s.size() && s[i] == '-' && s[i + 1] != ']') {
          const int hi = static_cast<unsigned char>(s[i + 1]);
          i += 2;
          cs.range(lo, hi);
        } else {
          cs.set(lo);
        }
      }
      if (i >= s.size()) { ok = false; return g->lit(""); }
      ++i;
      if (neg) cs.invert();
      return g->chars(cs);
    }
    if (c == '.') {
      ++i;
      CharSet cs; cs.range(0, 255); cs.w[0] &= ~(1ull << '\n');
      return g->chars(cs);
    }
    if (c == '\\' && i + 1 < s.size()) {
      bool is_class;
      const CharSet e = escape_class(s[i + 1], &is_class);
      i += 2;
      return g->chars(e);
    }
    if (c == '^' || c == '$') { ++i; return g->lit(""); }     // anchors: matching is always anchored
    ++i;
    return g->lit(std::string(1, c));
  }
  int quantified() {
    int a = atom();
    while (ok && i < s.size()) {
      const char c = s[i];
      if (c == '*') { a = g->repeat(a, 0, -1); ++i; }
      else if (c == '+') { a = g->repeat(a, 1, -1); ++i; }
      else if (c == '?') { a = g->repeat(a, 0, 1); ++i; }
      else if (c == '{') {
        size_t j = i + 1;
        int mn = 0, mx = -1;
        bool comma = false, digits = false;
        while (j < s.size() && s[j] != '}') {
          if (s[j] == ',') { comma = true; mx = -1; }
          else if (s[j] >= '0' && s[j] <= '9') {
            digits = true;
            if (!comma) mn = mn * 10 + (s[j] - '0');
            else mx = (mx < 0 ? 0 : mx * 10) + (s[j] - '0');
          } else { digits = false; break; }
          ++j;
        }
        if (!digits || j >= s.size()) break;     // literal '{'
        if (!comma) mx = mn;
        a = g->repeat(a, mn, mx);
        i = j + 1;
      } else break;
    }
    return a;
  }
  int sequence() {
    std::vector<int> parts;
    while (ok && i < s.size() && s[i] != '|' && s[i] != ')') parts.push_back(quantified());
    if (parts.empty()) return g->lit("");
    return g->seq(parts);
  }
  int alternation() {
    std::vector<int> opts{sequence()};
    while (ok && i < s.size() && s[i] == '|') { ++i; opts.push_back(sequence()); }
    return g->alt(opts);
  }
};

int Grammar::regex(const std::string& pattern) {
  RegexParser rp(this, pattern);
  const int n = rp.alternation();
  if (!rp.ok || rp.i != pattern.size()) error = "unsupported regular expression";
  return n;
}

int Grammar::build(const JVal& d) {
  if (d.kind != JVal::Obj || d.obj.empty()) { error = "grammar node must be an object"; return lit(""); }
  const std::string& k = d.obj[0].first;
  const JVal& v = d.obj[0].second;
  if (k == "lit") return lit(v.str);
  if (k == "chars") {
    RegexParser rp(this, v.str);
    const int n = rp.atom();
    if (!rp.ok) error = "bad character class";
    return n;
  }
  if (k == "seq" || k == "alt") {
    std::vector<int> kids;
    for (const auto& c : v.arr) kids.push_back(build(c));
    if (kids.empty()) return lit("");
    return k == "seq" ? seq(kids) : alt(kids);
  }
  if (k == "repeat") {
    if (v.arr.size() != 3) { error = "repeat needs [node, min, max]"; return lit(""); }
    return repeat(build(v.arr[0]), static_cast<int>(v.arr[1].num), static_cast<int>(v.arr[2].num));
  }
  if (k == "schema") {
    schema_root = &v;
    defs.clear();
    return schema(v);
  }
  if (k == "regex") return regex(v.str);
  if (k == "json") return any_json();
  if (k == "until" || k == "text_without") {
    if (v.str.empty()) { error = k + " needs a stop string"; return lit(""); }
    Node n; n.kind = k == "until" ? Node::Until : Node::Free; n.lit = v.str;
    return add(n);
  }
  error = "unknown grammar node '" + k + "'";
  return lit("");
}

// ------------------------------------------------------------------------------------------------ matcher
struct Frame {
  int32_t node;
  int32_t pos;      // Lit/Until: bytes matched; Seq: next child; Repeat: completed iterations; Chars: 0/1
  bool operator==(const Frame& o) const { return node == o.node && pos == o.pos; }
  bool operator<(const Frame& o) const { return node != o.node ? node < o.node : pos < o.pos; }
};
using Thread = std::vector<Frame>;   // back() is the innermost frame

constexpr size_t kMaxThreads = 512;

struct Matcher {
  const Grammar* g;
  std::vector<Thread> threads;    // every thread is "settled": empty (accepting) or topped by a byte-consuming frame

  // Expand epsilon moves of `t` into settled threads appended to out.
  void settle(Thread t, std::vector<Thread>& out, int depth = 0) const {
    while (true) {
      if (out.size() >= kMaxThreads || depth > 4096) return;
      if (t.empty()) { out.push_back(std::move(t)); return; }
      Frame& f = t.back();
      const Node& n = g->nodes[f.node];
      switch (n.kind) {
        case Node::Lit:
          if (f.pos >= static_cast<int>(n.lit.size())) { t.pop_back(); continue; }
          out.push_back(std::move(t));
          return;
        case Node::Until:
          if (f.pos >= static_cast<int>(n.lit.size())) { t.pop_back(); continue; }
          out.push_back(std::move(t));
          return;
        case Node::Free: {
          // may stop here (the continuation is settled on its own) or consume another byte
          Thread c = t;
          c.pop_back();
          settle(std::move(c), out, depth + 1);
          out.push_back(std::move(t));
          return;
        }
        case Node::Chars:
          if (f.pos >= 1) { t.pop_back(); continue; }
          out.push_back(std::move(t));
          return;
        case Node::Seq:
          if (f.pos >= static_cast<int>(n.kids.size())) { t.pop_back(); continue; }
          {
            const int child = n.kids[f.pos];
            ++f.pos;
            t.push_back(Frame{child, 0});
          }
          continue;
        case Node::Alt: {
          t.pop_back();
          for (int kid : n.kids) {
            Thread c = t;
            c.push_back(Frame{kid, 0});
            settle(std::move(c), out, depth + 1);
          }
          return;
        }
        case Node::Repeat: {
          const int done = f.pos;
          if (done >= n.rmin) {            // may stop here
            Thread c = t;
            c.pop_back();
            settle(std::move(c), out, depth + 1);
          }
          if (n.rmax < 0 || done < n.rmax) {
            // unbounded repeats keep the counter saturated at rmin so equal states merge
            f.pos = (n.rmax < 0 && done >= n.rmin) ? done : done + 1;
            t.push_back(Frame{n.kids[0], 0});
            continue;
          }
          return;
        }
        case Node::Ref:
          f.node = n.kids[0];
          f.pos = 0;
          continue;
      }
    }
  }

  void dedup() {
    std::sort(threads.begin(), threads.end());
    threads.erase(std::unique(threads.begin(), threads.end()), threads.end());
  }

  void reset() {
    threads.clear();
    settle(Thread{Frame{g->root, 0}}, threads);
    dedup();
  }

  bool can_finish() const {
    for (const auto& t : threads)
      if (t.empty()) return true;
    return false;
  }
  bool dead() const { return threads.empty(); }

  // advance every thread by one byte; returns false when nothing survives (state is then unchanged)
  bool step(uint8_t b) {
    std::vector<Thread> next;
    for (const auto& t : threads) {
      if (t.empty()) continue;
      const Frame& f = t.back();
      const Node& n = g->nodes[f.node];
      if (n.kind == Node::Lit) {
        if (static_cast<uint8_t>(n.lit[f.pos]) != b) continue;
        Thread c = t;
        ++c.back().pos;
        settle(std::move(c), next);
      } else if (n.kind == Node::Chars) {
        if (!n.cs.has(b)) continue;
        Thread c = t;
        c.back().pos = 1;
        settle(std::move(c), next);
      } else if (n.kind == Node::Until || n.kind == Node::Free) {
        // KMP-free fallback on the stop string: longest suffix of (matched + b) that is a prefix of stop
        const std::string& stop = n.lit;
        std::string cur = stop.substr(0, f.pos);
        cur.push_back(static_cast<char>(b));
        int k = static_cast<int>(std::min(cur.size(), stop.size()));
        while (k > 0 && stop.compare(0, k, cur, cur.size() - k, k) != 0) --k;
        if (n.kind == Node::Free && k == static_cast<int>(stop.size())) continue;   // the text would contain the stop
        Thread c = t;
        c.back().pos = k;
        settle(std::move(c), next);          // a Free frame settles into "stop here" and "one more byte" again
      }
      if (next.size() >= kMaxThreads) break;
    }
    if (next.empty()) return false;
    threads.swap(next);
    dedup();
    return true;
  }

  bool accept(const uint8_t* bytes, size_t n) {
    Matcher saved = *this;
    for (size_t i = 0; i < n; ++i)
      if (!step(bytes[i])) { *this = std::move(saved); return false; }
    return true;
  }
};

// ------------------------------------------------------------------------------------------------ vocabulary trie
struct Vocab {
  struct TNode {
    int32_t child[256];
    std::vector<int32_t> tokens;    // tokens whose byte string ends here
    TNode() { std::fill(child, child + 256, -1); }
  };
  std::vector<TNode> nodes;
  std::vector<std::string> bytes;
  int size = 0;
};

// Masks of recent matcher states of one grammar, for one vocabulary at a time.  Free text ("until" / "text_without")
// stays in the same state token after token, and its mask costs a walk over the whole vocabulary trie.
struct MaskCache {
  std::mutex mu;
  const void* vocab = nullptr;
  std::map<std::vector<Thread>, std::vector<uint32_t>> by_state;
  static constexpr size_t kMaxStates = 64;
};

void fill_rec(const Vocab& v, int tn, const Matcher& m, uint32_t* mask) {
  const Vocab::TNode& t = v.nodes[tn];
  for (int32_t tok : t.tokens) mask[tok >> 5] |= 1u << (tok & 31);
  for (int b = 0; b < 256; ++b) {
    if (t.child[b] < 0) continue;
    Matcher next = m;
    if (next.step(static_cast<uint8_t>(b))) fill_rec(v, t.child[b], next, mask);
  }
}

}  // namespace

extern "C" {

// tokens: concatenated byte strings, offsets[n+1]
void* ds41_vocab_new(const uint8_t* data, const int64_t* offsets, int n) {
  Vocab* v = new Vocab();
  v->size = n;
  v->nodes.emplace_back();
  v->bytes.resize(n);
  for (int i = 0; i < n; ++i) {
    const int64_t a = offsets[i], b = offsets[i + 1];
    v->bytes[i].assign(reinterpret_cast<const char*>(data + a), static_cast<size_t>(b - a));
    if (a == b) continue;                      // empty byte strings (special tokens) are never grammar-allowed
    int cur = 0;
    for (int64_t k = a; k < b; ++k) {
      if (v->nodes[cur].child[data[k]] < 0) {
        v->nodes[cur].child[data[k]] = static_cast<int32_t>(v->nodes.size());
        v->nodes.emplace_back();
      }
      cur = v->nodes[cur].child[data[k]];
    }
    v->nodes[cur].tokens.push_back(i);
  }
  return v;
}
void ds41_vocab_free(void* v) { delete static_cast<Vocab*>(v); }
int ds41_vocab_size(const void* v) { return static_cast<const Vocab*>(v)->size; }

// description: JSON text of a grammar node (see the file header).  On failure returns null and copies the message.
void* ds41_grammar_compile(const char* description, char* error, int error_cap) {
  JParser jp{description, description + std::strlen(description)};
  JVal d = jp.value();
  jp.ws();
  Grammar* g = new Grammar();
  if (!jp.ok || jp.p != jp.end) g->error = "grammar description is not valid JSON";
  else g->root = g->build(d);
  g->schema_root = nullptr;
  g->masks = std::make_shared<MaskCache>();
  if (!g->error.empty() || g->root < 0) {
    if (error != nullptr && error_cap > 0) std::snprintf(error, static_cast<size_t>(error_cap), "%s", g->error.c_str());
    delete g;
    return nullptr;
  }
  return g;
}
void ds41_grammar_free(void* g) { delete static_cast<Grammar*>(g); }
int ds41_grammar_nodes(const void* g) { return static_cast<int>(static_cast<const Grammar*>(g)->nodes.size()); }

void* ds41_matcher_new(const void* grammar) {
  Matcher* m = new Matcher();
  m->g = static_cast<const Grammar*>(grammar);
  m->reset();
  return m;
}
void* ds41_matcher_fork(const void* m) { return new Matcher(*static_cast<const Matcher*>(m)); }
void ds41_matcher_free(void* m) { delete static_cast<Matcher*>(m); }
void ds41_matcher_reset(void* m) { static_cast<Matcher*>(m)->reset(); }
int ds41_matcher_can_finish(const void* m) { return static_cast<const Matcher*>(m)->can_finish() ? 1 : 0; }
int ds41_matcher_threads(const void* m) { return static_cast<int>(static_cast<const Matcher*>(m)->threads.size()); }
// 1 when only termination is possible (every live thread is accepting and nothing can be consumed)
int ds41_matcher_is_terminated(const void* mp) {
  const Matcher* m = static_cast<const Matcher*>(mp);
  if (m->threads.empty()) return 0;
  for (const auto& t : m->threads)
    if (!t.empty()) return 0;
  return 1;
}
int ds41_matcher_accept_bytes(void* m, const uint8_t* bytes, int n) {
  return static_cast<Matcher*>(m)->accept(bytes, static_cast<size_t>(n)) ? 1 : 0;
}
int ds41_matcher_accept_token(void* m, const void* vocab, int token) {
  const Vocab* v = static_cast<const Vocab*>(vocab);
  if (token < 0 || token >= v->size || v->bytes[token].empty()) return 0;
  const std::string& b = v->bytes[token];
  return static_cast<Matcher*>(m)->accept(reinterpret_cast<const uint8_t*>(b.data()), b.size()) ? 1 : 0;
}
// mask: (vocab+31)/32 words, overwritten.  stop_token (e.g. EOS) is allowed iff the matcher can finish.
// Returns the number of allowed tokens.
int ds41_matcher_fill_mask(const void* m, const void* vocab, uint32_t* mask, int stop_token) {
  const Vocab* v = static_cast<const Vocab*>(vocab);
  const Matcher* mm = static_cast<const Matcher*>(m);
  const int words = (v->size + 31) / 32;
  std::memset(mask, 0, sizeof(uint32_t) * static_cast<size_t>(words));
  MaskCache* cache = mm->g->masks.get();
  bool hit = false;
  if (cache != nullptr) {
    std::lock_guard<std::mutex> lock(cache->mu);
    if (cache->vocab != vocab) { cache->by_state.clear(); cache->vocab = vocab; }
    auto it = cache->by_state.find(mm->threads);
    if (it != cache->by_state.end()) {
      std::memcpy(mask, it->second.data(), sizeof(uint32_t) * static_cast<size_t>(words));
      hit = true;
    }
  }
  if (!hit) {
    // bytes may only be consumed by non-accepting threads; the trie walk ignores finished threads
    fill_rec(*v, 0, *mm, mask);
    if (cache != nullptr) {
      std::lock_guard<std::mutex> lock(cache->mu);
      if (cache->by_state.size() >= MaskCache::kMaxStates) cache->by_state.clear();
      cache->by_state.emplace(mm->threads, std::vector<uint32_t>(mask, mask + words));
    }
  }
  // the trie root has no tokens, so nothing was set for the empty string
  if (stop_token >= 0 && stop_token < v->size && mm->can_finish()) mask[stop_token >> 5] |= 1u << (stop_token & 31);
  int count = 0;
  for (int i = 0; i < words; ++i) count += __builtin_popcount(mask[i]);
  return count;
}

}  // extern "C"
