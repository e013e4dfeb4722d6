// Python literal text -> pickle (protocol 2) bytes, for large dataset description files where ast.literal_eval is slow.
// Supported: dict, list, tuple, set-free literals of str (single / double quoted, with escapes), bytes-free, int (arbitrary size
// via the LONG text opcode), float, True / False / None, nested arbitrarily, trailing commas, comments.
// Counterpart of returnn/util/py-to-pickle.cpp in the reference; the grammar handling here is a recursive-descent parser
// that emits opcodes directly while parsing (no intermediate tree).
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>

namespace {

struct Parser {
  const char* p;
  const char* end;
  std::string out;
  std::string err;

  void skip_ws() {
    while (p < end) {
      if (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r') ++p;
      else if (*p == '#') {
        while (p < end && *p != '\n') ++p;
      } else break;
    }
  }
  bool fail(const char* msg) {
    if (err.empty()) {
      err = msg;
      err += " at offset ";
      err += std::to_string((long long)(p - (end - total)));
    }
    return false;
  }
  size_t total = 0;

  void put_u32(uint32_t v) { out.append(reinterpret_cast<const char*>(&v), 4); }

  bool parse_string(char quote) {
    std::string s;
    bool triple = (p + 2 < end && p[1] == quote && p[2] == quote);
    p += triple ? 3 : 1;
    while (true) {
      if (p >= end) return fail("unterminated string");
      char c = *p;
      if (c == quote) {
        if (!triple) { ++p; break; }
        if (p + 2 < end + 0 && p[1] == quote && p[2] == quote) { p += 3; break; }
        s.push_back(c);
        ++p;
        continue;
      }
      if (c == '\\') {
        if (p + 1 >= end) return fail("bad escape");
        char e = p[1];
        p += 2;
        switch (e) {
          case 'n': s.push_back('\n'); break;
          case 't': s.push_back('\t'); break;
          case 'r': s.push_back('\r'); break;
          case '\\': s.push_back('\\'); break;
          case '\'': s.push_back('\''); break;
          case '"': s.push_back('"'); break;
          case '0': s.push_back('\0'); break;
          case '\n': break;
          case 'x': {
            if (p + 2 > end) return fail("bad \\x escape");
            char hex[3] = {p[0], p[1], 0};
            unsigned v = (unsigned)strtoul(hex, nullptr, 16);
            p += 2;
            append_utf8(s, v);
            break;
          }
          case 'u': case 'U': {
            int n = e == 'u' ? 4 : 8;
            if (p + n > end) return fail("bad \\u escape");
            char hex[9];
            memcpy(hex, p, n);
            hex[n] = 0;
            p += n;
            append_utf8(s, (unsigned)strtoul(hex, nullptr, 16));
            break;
          }
          default: s.push_back('\\'); s.push_back(e); break;
        }
        continue;
      }
      s.push_back(c);
      ++p;
    }
    out.push_back('X');  // BINUNICODE: utf8 with 4-byte length
    put_u32((uint32_t)s.size());
    out += s;
    return true;
  }

  static void append_utf8(std::string& s, unsigned cp) {
    if (cp < 0x80) s.push_back((char)cp);
    else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
    else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  }

  bool parse_number() {
    const char* s = p;
    if (p < end && (*p == '-' || *p == '+')) ++p;
    bool is_float = false;
    while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '_' ||
                       ((*p == '-' || *p == '+') && (p[-1] == 'e' || p[-1] == 'E')))) {
      if (*p == '.' || *p == 'e' || *p == 'E') is_float = true;
      ++p;
    }
    std::string txt;
    for (const char* q = s; q < p; ++q)
      if (*q != '_') txt.push_back(*q);
    if (txt.empty() || txt == "-" || txt == "+") {
      // inf / nan written as float('inf') are not literals; accept bare inf / nan for convenience
      return fail("bad number");
    }
    if (is_float) {
      double d = strtod(txt.c_str(), nullptr);
      uint64_t bits;
      memcpy(&bits, &d, 8);
      out.push_back('G');  // BINFLOAT: 8 bytes big endian
      for (int i = 7; i >= 0; --i) out.push_back((char)((bits >> (8 * i)) & 0xFF));
      return true;
    }
    bool neg = txt[0] == '-';
    size_t digits = txt.size() - ((txt[0] == '-' || txt[0] == '+') ? 1 : 0);
    if (digits <= 9) {
      long v = strtol(txt.c_str(), nullptr, 10);
      out.push_back('J');  // BININT: 4-byte signed little endian
      int32_t v32 = (int32_t)v;
      out.append(reinterpret_cast<const char*>(&v32), 4);
      (void)neg;
      return true;
    }
    out.push_back('L');  // LONG: decimal text
    out += txt;
    out += "L\n";
    return true;
  }

  bool parse_value() {
    skip_ws();
    if (p >= end) return fail("unexpected end");
    char c = *p;
    if (c == '{') return parse_dict();
    if (c == '[') return parse_seq('[', ']');
    if (c == '(') return parse_seq('(', ')');
    if (c == '\'' || c == '"') return parse_string(c);
    if ((c == 'u' || c == 'r' || c == 'b') && p + 1 < end && (p[1] == '\'' || p[1] == '"')) {
      if (c == 'b') return fail("bytes literals are not supported");
      ++p;
      return parse_string(*p);
    }
    if ((c >= '0' && c <= '9') || c == '-' || c == '+' || c == '.') return parse_number();
    if (end - p >= 4 && !strncmp(p, "True", 4)) { p += 4; out.push_back('\x88'); return true; }
    if (end - p >= 5 && !strncmp(p, "False", 5)) { p += 5; out.push_back('\x89'); return true; }
    if (end - p >= 4 && !strncmp(p, "None", 4)) { p += 4; out.push_back('N'); return true; }
    return fail("unexpected character");
  }

  bool parse_dict() {
    ++p;
    out.push_back('}');  // EMPTY_DICT
    out.push_back('(');  // MARK
    size_t count = 0;
    while (true) {
      skip_ws();
      if (p >= end) return fail("unterminated dict");
      if (*p == '}') { ++p; break; }
      if (!parse_value()) return false;
      skip_ws();
      if (p >= end || *p != ':') return fail("expected ':'");
      ++p;
      if (!parse_value()) return false;
      ++count;
      skip_ws();
      if (p < end && *p == ',') ++p;
      if (count % 1000 == 0) {  // SETITEMS in batches like the Python pickler
        out.push_back('u');
        out.push_back('(');
      }
    }
    out.push_back('u');  // SETITEMS
    return true;
  }

  bool parse_seq(char open, char close) {
    ++p;
    bool is_list = open == '[';
    if (is_list) out.push_back(']');  // EMPTY_LIST
    out.push_back('(');               // MARK
    size_t count = 0;
    bool had_comma = false;
    while (true) {
      skip_ws();
      if (p >= end) return fail("unterminated sequence");
      if (*p == close) { ++p; break; }
      if (!parse_value()) return false;
      ++count;
      skip_ws();
      if (p < end && *p == ',') { ++p; had_comma = true; }
    }
    if (is_list) {
      out.push_back('e');  // APPENDS
    } else {
      if (count == 1 && !had_comma) {
        // parenthesised expression, not a tuple: drop the MARK we pushed. The mark is the byte right before the value;
        // we cannot remove it cheaply, so close it as a 1-tuple and take its item: not expressible in pickle without
        // memo; instead reject (such input never appears in data files).
        return fail("parenthesised scalar is not supported; write a tuple with a trailing comma");
      }
      out.push_back('t');  // TUPLE
    }
    return true;
  }
};

}  // namespace

// Parses `len` bytes at `src`. On success returns a malloc'ed buffer with the pickle and sets *out_len; on failure returns
// null and writes a message into err (up to err_len bytes). The caller frees the buffer with rb200_py_to_pickle_free.
extern "C" __attribute__((visibility("default"))) char* rb200_py_to_pickle(const char* src, long long len, long long* out_len, char* err,
                                                                          int err_len) {
  Parser ps;
  ps.p = src;
  ps.end = src + len;
  ps.total = (size_t)len;
  ps.out.reserve((size_t)len + 16);
  ps.out.push_back('\x80');  // PROTO 2
  ps.out.push_back('\x02');
  bool ok = ps.parse_value();
  if (ok) {
    ps.skip_ws();
    if (ps.p != ps.end) ok = ps.fail("trailing data");
  }
  if (!ok) {
    if (err && err_len > 0) {
      strncpy(err, ps.err.c_str(), (size_t)err_len - 1);
      err[err_len - 1] = 0;
    }
    return nullptr;
  }
  ps.out.push_back('.');  // STOP
  char* buf = (char*)malloc(ps.out.size());
  if (!buf) return nullptr;
  memcpy(buf, ps.out.data(), ps.out.size());
  *out_len = (long long)ps.out.size();
  return buf;
}

extern "C" __attribute__((visibility("default"))) void rb200_py_to_pickle_free(char* buf) { free(buf); }
