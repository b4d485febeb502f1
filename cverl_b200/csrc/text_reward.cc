// Host text utilities behind a C API: byte tokenizer, GSM8K rule reward, JSONL reader.
//
// * Byte tokenizer: vocabulary of 260 = {pad 0, bos 1, eos 2, unk 3} + 256 byte values
//   (reference: src/text/byte_tokenizer.cc).
// * GSM8K reward: strict = the last "#### <number>" inside the last 300 characters,
//   flexible = the last numeric run that is not "" or "."; the gold answer is normalised
//   by strict extraction, else by dropping whitespace, ',' and '$'; scores correct /
//   format / none default to 1.0 / 0.0 / 0.0 (reference: src/reward/gsm8k.cc:14-156).
// * JSONL: one object per line, two named fields returned as strings (numbers and
//   booleans are stringified), optional row limit (reference: src/data/hf_dataset.cc:145-265).
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------ GSM8K
bool number_char(char c) { return std::isdigit(static_cast<unsigned char>(c)) || c == '.' || c == ',' || c == '-'; }

std::string tail(const std::string& s, size_t n) { return s.size() <= n ? s : s.substr(s.size() - n); }

std::string drop_format(const std::string& s) {
  std::string out;
  for (char c : s)
    if (c != ',' && c != '$') out.push_back(c);
  return out;
}

bool strict_answer(const std::string& text, std::string* out) {
  static const std::string marker = "#### ";
  bool found = false;
  size_t pos = 0;
  for (;;) {
    const size_t hit = text.find(marker, pos);
    if (hit == std::string::npos) break;
    size_t b = hit + marker.size(), e = b;
    while (e < text.size() && number_char(text[e])) ++e;
    if (e > b) {
      *out = text.substr(b, e - b);
      found = true;
    }
    pos = e > hit ? e : hit + 1;
  }
  return found;
}

bool flexible_answer(const std::string& text, std::string* out) {
  std::vector<std::string> runs;
  size_t i = 0;
  while (i < text.size()) {
    if (number_char(text[i])) {
      size_t b = i;
      while (i < text.size() && number_char(text[i])) ++i;
      runs.push_back(text.substr(b, i - b));
    } else {
      ++i;
    }
  }
  for (auto it = runs.rbegin(); it != runs.rend(); ++it)
    if (!it->empty() && *it != ".") {
      *out = *it;
      return true;
    }
  return false;
}

bool extract_answer(const std::string& solution, int flexible, size_t clip, std::string* out) {
  const std::string clipped = tail(solution, clip);
  if (flexible) return flexible_answer(clipped, out);
  std::string raw;
  if (!strict_answer(clipped, &raw)) return false;
  *out = drop_format(raw);
  return true;
}

std::string normalise_gold(const std::string& gold) {
  std::string raw;
  if (strict_answer(tail(gold, 300), &raw)) return drop_format(raw);
  std::string out;
  for (char c : gold)
    if (!std::isspace(static_cast<unsigned char>(c)) && c != ',' && c != '$') out.push_back(c);
  return out;
}

// ------------------------------------------------------------------ JSON line scanner
struct Json {
  const std::string& s;
  size_t i = 0;
  explicit Json(const std::string& t) : s(t) {}
  void ws() {
    while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
  }
  static void utf8(uint32_t cp, std::string* out) {
    if (cp < 0x80) {
      out->push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      out->push_back(static_cast<char>(0xC0 | (cp >> 6)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out->push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      out->push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  bool hex4(uint32_t* v) {
    if (i + 4 > s.size()) return false;
    uint32_t x = 0;
    for (int k = 0; k < 4; ++k) {
      char c = s[i + k];
      x <<= 4;
      if (c >= '0' && c <= '9') x |= c - '0';
      else if (c >= 'a' && c <= 'f') x |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') x |= c - 'A' + 10;
      else return false;
    }
    i += 4;
    *v = x;
    return true;
  }
  bool string(std::string* out) {
    ws();
    if (i >= s.size() || s[i] != '"') return false;
    ++i;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        char c = s[++i];
        ++i;
        switch (c) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            uint32_t cp;
            if (!hex4(&cp)) return false;
            if (cp >= 0xD800 && cp <= 0xDBFF && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
              i += 2;
              uint32_t lo;
              if (!hex4(&lo)) return false;
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(cp, out);
            break;
          }
          default: out->push_back(c);
        }
      } else {
        out->push_back(s[i++]);
      }
    }
    if (i >= s.size()) return false;
    ++i;
    return true;
  }
  // any value, returned as text: strings unescaped, everything else verbatim
  bool last_was_literal = false;   // the value just read was a bare literal (number, true, false, null), not a string
  bool value(std::string* out) {
    ws();
    last_was_literal = false;
    if (i >= s.size()) return false;
    if (s[i] == '"') return string(out);
    if (s[i] == '{' || s[i] == '[') {
      const size_t b = i;
      int depth = 0;
      while (i < s.size()) {
        if (s[i] == '"') {
          std::string tmp;
          if (!string(&tmp)) return false;
          continue;
        }
        if (s[i] == '{' || s[i] == '[') ++depth;
        if ((s[i] == '}' || s[i] == ']') && --depth == 0) {
          ++i;
          *out = s.substr(b, i - b);
          return true;
        }
        ++i;
      }
      return false;
    }
    const size_t b = i;
    while (i < s.size() && s[i] != ',' && s[i] != '}' && !std::isspace(static_cast<unsigned char>(s[i]))) ++i;
    *out = s.substr(b, i - b);
    last_was_literal = true;
    return true;
  }
};

struct Rows {
  std::vector<std::string> a, b;
  std::string error;
};

}  // namespace

extern "C" {

// ---- byte tokenizer ----------------------------------------------------------------------------
enum { CVERL_BYTE_PAD = 0, CVERL_BYTE_BOS = 1, CVERL_BYTE_EOS = 2, CVERL_BYTE_UNK = 3, CVERL_BYTE_VOCAB = 260 };

// Encodes up to `capacity` ids; returns the number of ids the full encoding has.
int64_t cverl_byte_encode(const char* text, int64_t len, int add_bos, int add_eos, int64_t max_tokens, int64_t* out,
                          int64_t capacity) {
  int64_t n = 0;
  auto push = [&](int64_t id) {
    if (max_tokens > 0 && n >= max_tokens) return;
    if (n < capacity) out[n] = id;
    ++n;
  };
  if (add_bos) push(CVERL_BYTE_BOS);
  for (int64_t i = 0; i < len; ++i) push(4 + static_cast<unsigned char>(text[i]));
  // the terminator is appended only where the limit leaves room for it: a text cut off by max_tokens ends on
  // its last kept byte (reference: src/text/byte_tokenizer.cc:20-28)
  if (add_eos) push(CVERL_BYTE_EOS);
  return n;
}

// Decodes ids to bytes; special tokens are dropped when skip_special, else rendered as <pad>/<bos>/<eos>/<unk>.
int64_t cverl_byte_decode(const int64_t* ids, int64_t n, int skip_special, char* out, int64_t capacity) {
  static const char* names[4] = {"<pad>", "<bos>", "<eos>", "<unk>"};
  int64_t w = 0;
  auto put = [&](char c) {
    if (w < capacity) out[w] = c;
    ++w;
  };
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    if (id >= 4 && id < CVERL_BYTE_VOCAB) {
      put(static_cast<char>(id - 4));
    } else if (!skip_special) {
      const char* s = names[(id >= 0 && id < 4) ? id : 3];
      while (*s) put(*s++);
    }
  }
  return w;
}

// ---- GSM8K reward ------------------------------------------------------------------------------
// Returns 1 and writes the NUL-terminated answer when one is found, else 0.
int cverl_gsm8k_extract(const char* solution, int flexible, int64_t clip_chars, char* out, int64_t capacity) {
  std::string ans;
  if (!extract_answer(solution, flexible, static_cast<size_t>(clip_chars > 0 ? clip_chars : 300), &ans)) return 0;
  std::snprintf(out, static_cast<size_t>(capacity), "%s", ans.c_str());
  return 1;
}

double cverl_gsm8k_reward(const char* solution, const char* ground_truth, int flexible, int64_t clip_chars,
                          double correct_score, double format_score, double no_answer_score) {
  std::string ans;
  if (!extract_answer(solution, flexible, static_cast<size_t>(clip_chars > 0 ? clip_chars : 300), &ans))
    return no_answer_score;
  return ans == normalise_gold(ground_truth) ? correct_score : format_score;
}

void cverl_gsm8k_normalize_gold(const char* gold, char* out, int64_t capacity) {
  std::snprintf(out, static_cast<size_t>(capacity), "%s", normalise_gold(gold).c_str());
}

// ---- JSONL -------------------------------------------------------------------------------------
// Loads (field_a, field_b) of every line; rows lacking either field are errors.
void* cverl_jsonl_open(const char* path, const char* field_a, const char* field_b, int64_t max_rows) {
  auto* rows = new Rows();
  std::ifstream f(path);
  if (!f) {
    rows->error = std::string("cannot open ") + path;
    return rows;
  }
  std::string line;
  int64_t lineno = 0;
  while (std::getline(f, line)) {
    ++lineno;
    bool blank = true;
    for (char c : line)
      if (!std::isspace(static_cast<unsigned char>(c))) blank = false;
    if (blank) continue;
    // negative = every row; 0 = no row at all (the reference's rule, src/data/hf_dataset.cc: max_examples)
    if (max_rows >= 0 && static_cast<int64_t>(rows->a.size()) >= max_rows) break;
    Json j(line);
    j.ws();
    if (j.i >= line.size() || line[j.i] != '{') {
      rows->error = "line " + std::to_string(lineno) + ": not a JSON object";
      return rows;
    }
    ++j.i;
    std::string va, vb;
    bool ha = false, hb = false, ok = true;
    for (;;) {
      j.ws();
      if (j.i < line.size() && line[j.i] == '}') break;
      std::string key, val;
      if (!j.string(&key)) { ok = false; break; }
      j.ws();
      if (j.i >= line.size() || line[j.i] != ':') { ok = false; break; }
      ++j.i;
      if (!j.value(&val)) { ok = false; break; }
      if (val == "null" && j.last_was_literal) val.clear();     // a JSON null reads as the empty string
      if (key == field_a) va = val, ha = true;
      if (key == field_b) vb = val, hb = true;
      j.ws();
      if (j.i < line.size() && line[j.i] == ',') ++j.i;
    }
    if (!ok || !ha || !hb) {
      rows->error = "line " + std::to_string(lineno) + (ok ? ": missing field" : ": malformed JSON");
      return rows;
    }
    rows->a.push_back(va);
    rows->b.push_back(vb);
  }
  return rows;
}
const char* cverl_jsonl_error(void* h) {
  auto* r = static_cast<Rows*>(h);
  return r->error.empty() ? nullptr : r->error.c_str();
}
int64_t cverl_jsonl_rows(void* h) { return static_cast<int64_t>(static_cast<Rows*>(h)->a.size()); }
const char* cverl_jsonl_get(void* h, int64_t row, int which) {
  auto* r = static_cast<Rows*>(h);
  if (row < 0 || row >= static_cast<int64_t>(r->a.size())) return nullptr;
  return (which == 0 ? r->a : r->b)[static_cast<size_t>(row)].c_str();
}
void cverl_jsonl_close(void* h) { delete static_cast<Rows*>(h); }
}
