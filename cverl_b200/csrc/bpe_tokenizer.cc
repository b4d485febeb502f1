// Byte-level BPE tokenizer reading a Hugging Face tokenizer.json (GPT-2 / Qwen family).
//
// Pipeline: added/special tokens are matched longest-first and split the text; every other
// span is pre-tokenised by the Split regex found in the file (else the Qwen/GPT-2 default),
// each piece is mapped byte -> printable unicode (the GPT-2 table) and merged with ranked BPE
// merges (strings "a b" or pairs ["a","b"]); decode reverses the byte map.  Pad / eos / bos ids
// are discovered from the usual token spellings.  Behaviour follows the reference
// (src/text/hf_bpe_tokenizer.cc:40-62,200-207,285-359,429-444,528-558).
//
// The regex engine is PCRE2 (UTF + UCP), resolved at run time with dlopen so that no
// development header is needed; without the library a hand-written scanner implements the
// default pattern (ASCII classes exact, other code points treated as letters).
#include <algorithm>
#include <atomic>
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <dlfcn.h>
#include <fstream>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <thread>
#include <tuple>
#include <unordered_map>
#include <vector>

namespace {

// ------------------------------------------------------------------ minimal JSON DOM
struct JValue {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;
  const JValue* get(const std::string& key) const {
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const std::string& s;
  size_t i = 0;
  explicit JParser(const std::string& t) : s(t) {}
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  [[noreturn]] void fail(const char* what) { throw std::runtime_error(std::string("tokenizer.json: ") + what); }
  static void utf8(uint32_t cp, std::string& out) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { out.push_back(static_cast<char>(0xC0 | (cp >> 6))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) { out.push_back(static_cast<char>(0xE0 | (cp >> 12))); out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else { out.push_back(static_cast<char>(0xF0 | (cp >> 18))); out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F))); out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F))); out.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
  }
  uint32_t hex4() {
    if (i + 4 > s.size()) fail("bad \\u escape");
    uint32_t v = 0;
    for (int k = 0; k < 4; ++k) {
      char c = s[i++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string string() {
    if (s[i] != '"') fail("expected string");
    ++i;
    std::string out;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\') {
        ++i;
        char c = s[i++];
        switch (c) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {
            uint32_t cp = hex4();
            if (cp >= 0xD800 && cp <= 0xDBFF && i + 1 < s.size() && s[i] == '\\' && s[i + 1] == 'u') {
              i += 2;
              uint32_t lo = hex4();
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(cp, out);
            break;
          }
          default: out.push_back(c);
        }
      } else {
        out.push_back(s[i++]);
      }
    }
    if (i >= s.size()) fail("unterminated string");
    ++i;
    return out;
  }
  JValue value() {
    ws();
    if (i >= s.size()) fail("truncated");
    JValue v;
    char c = s[i];
    if (c == '{') {
      v.kind = JValue::Obj;
      ++i;
      ws();
      if (s[i] == '}') { ++i; return v; }
      for (;;) {
        ws();
        std::string k = string();
        ws();
        if (s[i] != ':') fail("expected ':'");
        ++i;
        v.obj.emplace_back(std::move(k), value());
        ws();
        if (s[i] == ',') { ++i; continue; }
        if (s[i] == '}') { ++i; break; }
        fail("expected ',' or '}'");
      }
    } else if (c == '[') {
      v.kind = JValue::Arr;
      ++i;
      ws();
      if (s[i] == ']') { ++i; return v; }
      for (;;) {
        v.arr.push_back(value());
        ws();
        if (s[i] == ',') { ++i; continue; }
        if (s[i] == ']') { ++i; break; }
        fail("expected ',' or ']'");
      }
    } else if (c == '"') {
      v.kind = JValue::Str;
      v.str = string();
    } else if (s.compare(i, 4, "true") == 0) { v.kind = JValue::Bool; v.b = true; i += 4; }
    else if (s.compare(i, 5, "false") == 0) { v.kind = JValue::Bool; i += 5; }
    else if (s.compare(i, 4, "null") == 0) { i += 4; }
    else {
      size_t b = i;
      while (i < s.size() && (std::isdigit(static_cast<unsigned char>(s[i])) || s[i] == '-' || s[i] == '+' || s[i] == '.' || s[i] == 'e' || s[i] == 'E')) ++i;
      if (b == i) fail("unexpected character");
      v.kind = JValue::Num;
      v.num = std::stod(s.substr(b, i - b));
    }
    return v;
  }
};

// ------------------------------------------------------------------ PCRE2 through dlopen
struct Pcre2 {
  using compile_t = void* (*)(const unsigned char*, size_t, uint32_t, int*, size_t*, void*);
  using mdata_t = void* (*)(const void*, void*);
  using match_t = int (*)(const void*, const unsigned char*, size_t, size_t, uint32_t, void*, void*);
  using ovec_t = size_t* (*)(void*);
  using free_code_t = void (*)(void*);
  using free_md_t = void (*)(void*);
  using jit_t = int (*)(void*, uint32_t);
  void* lib = nullptr;
  jit_t jit_compile = nullptr;   // optional: absent in a PCRE2 built without JIT support
  compile_t compile = nullptr;
  mdata_t mdata = nullptr;
  match_t match = nullptr;
  ovec_t ovec = nullptr;
  free_code_t free_code = nullptr;
  free_md_t free_md = nullptr;
  bool ok = false;
  Pcre2() {
    for (const char* name : {"libpcre2-8.so.0", "libpcre2-8.so"}) {
      lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (lib) break;
    }
    if (!lib) return;
    compile = reinterpret_cast<compile_t>(dlsym(lib, "pcre2_compile_8"));
    mdata = reinterpret_cast<mdata_t>(dlsym(lib, "pcre2_match_data_create_from_pattern_8"));
    match = reinterpret_cast<match_t>(dlsym(lib, "pcre2_match_8"));
    ovec = reinterpret_cast<ovec_t>(dlsym(lib, "pcre2_get_ovector_pointer_8"));
    free_code = reinterpret_cast<free_code_t>(dlsym(lib, "pcre2_code_free_8"));
    free_md = reinterpret_cast<free_md_t>(dlsym(lib, "pcre2_match_data_free_8"));
    jit_compile = reinterpret_cast<jit_t>(dlsym(lib, "pcre2_jit_compile_8"));
    ok = compile && mdata && match && ovec && free_code && free_md;
  }
  static Pcre2& get() {
    static Pcre2 p;
    return p;
  }
};
constexpr uint32_t kPcre2Utf = 0x00080000u, kPcre2Ucp = 0x00020000u, kPcre2JitComplete = 0x00000001u,
                   kPcre2NoUtfCheck = 0x40000000u;

const char* kDefaultPattern =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+";

// ------------------------------------------------------------------ unicode helpers
size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1; }

std::vector<std::string> split_utf8(const std::string& s) {
  std::vector<std::string> out;
  for (size_t i = 0; i < s.size();) {
    size_t n = std::min(utf8_len(static_cast<unsigned char>(s[i])), s.size() - i);
    out.push_back(s.substr(i, n));
    i += n;
  }
  return out;
}

struct Tokenizer {
  std::unordered_map<std::string, int64_t> vocab;
  std::vector<std::string> id_to_token;
  std::unordered_map<std::string, int64_t> merge_rank;  // "a b" -> rank
  std::vector<std::pair<std::string, int64_t>> added;   // sorted longest first
  std::vector<std::tuple<std::string, int64_t, bool>> added_in_file_order;   // (content, id, special)
  std::string unk_token_name;
  std::unordered_map<int64_t, bool> special_ids;
  std::string byte_to_uni[256];
  std::unordered_map<std::string, int> uni_to_byte;
  std::string pattern;
  void* re = nullptr;
  bool jit = false;
  int64_t pad_id = -1, bos_id = -1, eos_id = -1, unk_id = -1;
  std::string error;

  // One handle serves any number of threads at once (a data loader's workers, encode_batch): everything below
  // load() is read-only except these two pools, which carry their own locks.
  //  * match data: a PCRE2 match block belongs to one match at a time; blocks are handed out from a free list.
  //  * merge cache: piece -> ids, in kShards maps with a lock each (the shard is picked by the piece's hash).
  std::mutex md_mutex;
  std::vector<void*> md_free;
  static constexpr size_t kShards = 64;
  struct Shard {
    std::mutex m;
    std::deque<std::string> keys;   // owns the bytes the map's keys view (a deque never moves its elements)
    std::unordered_map<std::string_view, std::vector<int64_t>> map;
  };
  Shard shards[kShards];

  // merges over symbol ids: (left id, right id) -> (rank, id of the merged token).  Built when every merge's two
  // sides and result are vocabulary entries (true of trained BPE vocabularies); otherwise the string form is used.
  std::unordered_map<uint64_t, std::pair<int64_t, int64_t>> pair_merge;
  bool id_merges = false;
  int64_t byte_sym[256];                       // id of the one-symbol token of each byte, -1 if absent
  std::vector<uint32_t> added_by_first[256];   // indices into `added` (longest first) by first byte

  ~Tokenizer() {
    auto& p = Pcre2::get();
    for (void* md : md_free) p.free_md(md);
    if (re) p.free_code(re);
  }

  void* acquire_md() {
    {
      std::lock_guard<std::mutex> lock(md_mutex);
      if (!md_free.empty()) {
        void* md = md_free.back();
        md_free.pop_back();
        return md;
      }
    }
    return Pcre2::get().mdata(re, nullptr);
  }
  void release_md(void* md) {
    std::lock_guard<std::mutex> lock(md_mutex);
    md_free.push_back(md);
  }

  void build_byte_table() {
    std::vector<int> bs;
    for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
    for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
    for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
    std::vector<int> cs(bs.begin(), bs.end());
    int n = 0;
    for (int b = 0; b < 256; ++b)
      if (std::find(bs.begin(), bs.end(), b) == bs.end()) {
        bs.push_back(b);
        cs.push_back(256 + n++);
      }
    for (size_t i = 0; i < bs.size(); ++i) {
      std::string u;
      JParser::utf8(static_cast<uint32_t>(cs[i]), u);
      byte_to_uni[bs[i]] = u;
      uni_to_byte[u] = bs[i];
    }
  }

  void load(const std::string& path) {
    std::ifstream f(path);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    JParser jp(text);
    JValue root = jp.value();
    const JValue* model = root.get("model");
    if (!model) throw std::runtime_error("tokenizer.json: no model section");
    const JValue* v = model->get("vocab");
    if (!v || v->kind != JValue::Obj) throw std::runtime_error("tokenizer.json: no vocab");
    for (const auto& kv : v->obj) vocab[kv.first] = static_cast<int64_t>(kv.second.num);
    if (const JValue* merges = model->get("merges")) {
      int64_t rank = 0;
      for (const auto& m : merges->arr) {
        if (m.kind == JValue::Str) merge_rank[m.str] = rank++;
        else if (m.kind == JValue::Arr && m.arr.size() == 2) merge_rank[m.arr[0].str + " " + m.arr[1].str] = rank++;
      }
    }
    if (const JValue* at = root.get("added_tokens")) {
      for (const auto& t : at->arr) {
        const JValue* content = t.get("content");
        const JValue* id = t.get("id");
        if (!content || !id) continue;
        const int64_t tid = static_cast<int64_t>(id->num);
        vocab[content->str] = tid;
        added.emplace_back(content->str, tid);
        const JValue* sp = t.get("special");
        const bool special = sp ? sp->b : true;        // absent means special (reference: hf_bpe_tokenizer.cc:317)
        special_ids[tid] = special;
        added_in_file_order.emplace_back(content->str, tid, special);
      }
    }
    if (const JValue* unk = model->get("unk_token"))
      if (unk->kind == JValue::Str) unk_token_name = unk->str;
    std::sort(added.begin(), added.end(), [](const auto& a, const auto& b) {
      return a.first.size() != b.first.size() ? a.first.size() > b.first.size() : a.first < b.first;
    });
    int64_t max_id = -1;
    for (const auto& kv : vocab) max_id = std::max(max_id, kv.second);
    id_to_token.assign(static_cast<size_t>(max_id + 1), "");
    for (const auto& kv : vocab) id_to_token[static_cast<size_t>(kv.second)] = kv.first;
    // first Split/Regex pattern of the pre-tokenizer, if any
    pattern = kDefaultPattern;
    if (const JValue* pt = root.get("pre_tokenizer")) {
      std::vector<const JValue*> stack{pt};
      bool found = false;
      while (!stack.empty() && !found) {
        const JValue* cur = stack.back();
        stack.pop_back();
        if (cur->kind != JValue::Obj) continue;
        const JValue* type = cur->get("type");
        if (type && type->str == "Split") {
          const JValue* pat = cur->get("pattern");
          if (pat) {
            const JValue* rx = pat->get("Regex");
            if (rx && rx->kind == JValue::Str) {
              pattern = rx->str;
              found = true;
            }
          }
        }
        if (const JValue* subs = cur->get("pretokenizers"))
          for (auto it = subs->arr.rbegin(); it != subs->arr.rend(); ++it) stack.push_back(&*it);
      }
    }
    auto& p = Pcre2::get();
    if (p.ok) {
      int err = 0;
      size_t off = 0;
      re = p.compile(reinterpret_cast<const unsigned char*>(pattern.c_str()), ~static_cast<size_t>(0),
                     kPcre2Utf | kPcre2Ucp, &err, &off, nullptr);
      if (re && p.jit_compile) jit = p.jit_compile(re, kPcre2JitComplete) == 0;
    }
    discover_special();
    build_indexes();
  }

  void build_indexes() {
    for (size_t i = 0; i < added.size(); ++i)
      if (!added[i].first.empty()) added_by_first[static_cast<unsigned char>(added[i].first[0])].push_back(static_cast<uint32_t>(i));
    id_merges = true;
    for (int b = 0; b < 256; ++b) {
      auto it = vocab.find(byte_to_uni[b]);
      byte_sym[b] = it != vocab.end() ? it->second : -1;
    }
    for (const auto& kv : merge_rank) {
      const size_t sp = kv.first.find(' ');
      if (sp == std::string::npos) { id_merges = false; break; }
      const std::string a = kv.first.substr(0, sp), b = kv.first.substr(sp + 1);
      auto ia = vocab.find(a), ib = vocab.find(b), iab = vocab.find(a + b);
      if (ia == vocab.end() || ib == vocab.end() || iab == vocab.end() || ia->second > 0xffffffffLL ||
          ib->second > 0xffffffffLL || ia->second < 0 || ib->second < 0) {
        id_merges = false;
        break;
      }
      const uint64_t key = (static_cast<uint64_t>(ia->second) << 32) | static_cast<uint64_t>(ib->second);
      auto ins = pair_merge.emplace(key, std::make_pair(kv.second, iab->second));
      if (!ins.second && kv.second < ins.first->second.first) ins.first->second = {kv.second, iab->second};
    }
    if (!id_merges) pair_merge.clear();
  }

  int64_t find_token(std::initializer_list<const char*> names) const {
    for (const char* n : names) {
      auto it = vocab.find(n);
      if (it != vocab.end()) return it->second;
    }
    return -1;
  }
  // The reference's rules (src/text/hf_bpe_tokenizer.cc:310-356): walk the added tokens in file order and take, for
  // each role, the FIRST special token with one of the usual spellings; model.unk_token overrides unk; a missing pad
  // falls back to a token spelled <|pad|> and then to eos.  (For the Qwen vocabularies this makes <|endoftext|>
  // both eos and pad and <|im_start|> bos.)
  void discover_special() {
    auto is_one_of = [](const std::string& s, std::initializer_list<const char*> names) {
      for (const char* n : names)
        if (s == n) return true;
      return false;
    };
    pad_id = bos_id = eos_id = unk_id = -1;
    for (const auto& t : added_in_file_order) {
      const std::string& c = std::get<0>(t);
      const int64_t id = std::get<1>(t);
      if (!std::get<2>(t)) continue;
      if (pad_id < 0 && is_one_of(c, {"<|pad|>", "<pad>", "[PAD]"})) pad_id = id;
      if (eos_id < 0 && is_one_of(c, {"<|endoftext|>", "</s>", "<|im_end|>", "<eos>", "[EOS]"})) eos_id = id;
      if (bos_id < 0 && is_one_of(c, {"<s>", "<bos>", "[BOS]", "<|im_start|>"})) bos_id = id;
      if (unk_id < 0 && is_one_of(c, {"<unk>", "[UNK]"})) unk_id = id;
    }
    if (!unk_token_name.empty()) {
      auto it = vocab.find(unk_token_name);
      if (it != vocab.end()) unk_id = it->second;
    }
    if (pad_id < 0) {
      auto it = vocab.find("<|pad|>");
      pad_id = it != vocab.end() ? it->second : eos_id;
    }
  }

  // --- pre-tokenisation ------------------------------------------------------
  static bool is_space(uint32_t c) { return c == ' ' || (c >= 9 && c <= 13) || c == 0x85 || c == 0xA0 || c == 0x3000 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 || c == 0x2029; }
  static bool is_digit(uint32_t c) { return c >= '0' && c <= '9'; }
  static bool is_letter(uint32_t c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= 0x80 && !is_space(c)); }

  static uint32_t decode_cp(const std::string& s, size_t i, size_t* len) {
    unsigned char c = static_cast<unsigned char>(s[i]);
    size_t n = std::min(utf8_len(c), s.size() - i);
    *len = n;
    if (n == 1) return c;
    uint32_t cp = c & (0xFF >> (n + 1));
    for (size_t k = 1; k < n; ++k) cp = (cp << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    return cp;
  }

  // hand-written matcher of the default pattern (used only without PCRE2)
  template <class Sink>
  void scan_default(const std::string& s, Sink&& sink) const {
    std::vector<uint32_t> cps;
    std::vector<size_t> offs;
    for (size_t i = 0; i < s.size();) {
      size_t n;
      cps.push_back(decode_cp(s, i, &n));
      offs.push_back(i);
      i += n;
    }
    offs.push_back(s.size());
    const size_t n = cps.size();
    size_t i = 0;
    auto emit = [&](size_t b, size_t e) { sink(offs[b], offs[e] - offs[b]); };
    while (i < n) {
      // contractions
      if (cps[i] == '\'' && i + 1 < n) {
        auto low = [&](size_t k) { return k < n ? static_cast<uint32_t>(std::tolower(static_cast<int>(cps[k] < 128 ? cps[k] : 0))) : 0u; };
        uint32_t a = low(i + 1), b = low(i + 2);
        if (a == 's' || a == 't' || a == 'm' || a == 'd') { emit(i, i + 2); i += 2; continue; }
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { emit(i, i + 3); i += 3; continue; }
      }
      // [^\r\n\p{L}\p{N}]?\p{L}+
      {
        size_t j = i;
        if (!is_letter(cps[j]) && !is_digit(cps[j]) && cps[j] != '\r' && cps[j] != '\n' && j + 1 < n && is_letter(cps[j + 1])) ++j;
        if (j < n && is_letter(cps[j])) {
          size_t e = j;
          while (e < n && is_letter(cps[e])) ++e;
          emit(i, e);
          i = e;
          continue;
        }
      }
      if (is_digit(cps[i])) { emit(i, i + 1); ++i; continue; }
      // ' ?[^\s\p{L}\p{N}]+[\r\n]*'
      {
        size_t j = i;
        if (cps[j] == ' ' && j + 1 < n) ++j;
        auto punct = [&](uint32_t c) { return !is_space(c) && !is_letter(c) && !is_digit(c); };
        if (j < n && punct(cps[j])) {
          size_t e = j;
          while (e < n && punct(cps[e])) ++e;
          while (e < n && (cps[e] == '\r' || cps[e] == '\n')) ++e;
          emit(i, e);
          i = e;
          continue;
        }
      }
      // whitespace alternatives
      if (is_space(cps[i])) {
        size_t e = i;
        while (e < n && is_space(cps[e])) ++e;
        size_t last_nl = n;
        for (size_t k = i; k < e; ++k)
          if (cps[k] == '\r' || cps[k] == '\n') last_nl = k;
        if (last_nl != n) { emit(i, last_nl + 1); i = last_nl + 1; continue; }   // \s*[\r\n]+
        if (e < n && e - i > 1) { emit(i, e - 1); i = e - 1; continue; }          // \s+(?!\S)
        emit(i, e);
        i = e;
        continue;
      }
      emit(i, i + 1);
      ++i;
    }
  }

  // calls sink(offset, length) for every piece of s, in order
  template <class Sink>
  void pretokenize(const std::string& s, Sink&& sink) {
    auto& p = Pcre2::get();
    void* md = re ? acquire_md() : nullptr;
    if (!md) {
      scan_default(s, sink);
      return;
    }
    size_t pos = 0;
    const auto* subj = reinterpret_cast<const unsigned char*>(s.data());
    uint32_t opts = 0;
    while (pos < s.size()) {
      int rc = p.match(re, subj, s.size(), pos, opts, md, nullptr);
      opts = kPcre2NoUtfCheck;   // the first match validated the whole subject; checking it again on every
                                 // match would make a text of n bytes cost n * n
      if (rc < 0) {
        sink(pos, s.size() - pos);
        break;
      }
      size_t* ov = p.ovec(md);
      if (ov[0] > pos) sink(pos, ov[0] - pos);  // unmatched gap kept as its own piece
      if (ov[1] > ov[0]) sink(ov[0], ov[1] - ov[0]);
      pos = ov[1] > pos ? ov[1] : pos + 1;
    }
    release_md(md);
  }

  // --- BPE -----------------------------------------------------------------------
  // merges on symbol ids; false when a byte of the piece has no one-symbol token (the string form then decides)
  bool bpe_ids(std::string_view piece, std::vector<int64_t>& ids) const {
    ids.clear();
    ids.reserve(piece.size());
    for (unsigned char c : piece) {
      if (byte_sym[c] < 0) return false;
      ids.push_back(byte_sym[c]);
    }
    while (ids.size() > 1) {
      int64_t best = INT64_MAX, merged = -1;
      size_t at = 0;
      for (size_t i = 0; i + 1 < ids.size(); ++i) {
        auto it = pair_merge.find((static_cast<uint64_t>(ids[i]) << 32) | static_cast<uint64_t>(ids[i + 1]));
        if (it != pair_merge.end() && it->second.first < best) {
          best = it->second.first;
          merged = it->second.second;
          at = i;
        }
      }
      if (best == INT64_MAX) break;
      ids[at] = merged;
      ids.erase(ids.begin() + static_cast<long>(at) + 1);
    }
    return true;
  }

  void bpe_strings(std::string_view piece, std::vector<int64_t>& ids) const {
    std::string mapped;
    for (unsigned char c : piece) mapped += byte_to_uni[c];
    std::vector<std::string> parts = split_utf8(mapped);
    while (parts.size() > 1) {
      int64_t best = INT64_MAX;
      size_t at = 0;
      for (size_t i = 0; i + 1 < parts.size(); ++i) {
        auto it = merge_rank.find(parts[i] + " " + parts[i + 1]);
        if (it != merge_rank.end() && it->second < best) {
          best = it->second;
          at = i;
        }
      }
      if (best == INT64_MAX) break;
      parts[at] += parts[at + 1];
      parts.erase(parts.begin() + static_cast<long>(at) + 1);
    }
    ids.clear();
    for (const auto& t : parts) {
      auto it = vocab.find(t);
      if (it != vocab.end()) {
        ids.push_back(it->second);
      } else {
        for (const auto& ch : split_utf8(t)) {  // unknown merge result: fall back to single symbols
          auto jt = vocab.find(ch);
          ids.push_back(jt != vocab.end() ? jt->second : (unk_id >= 0 ? unk_id : 0));
        }
      }
    }
  }

  void bpe(std::string_view piece, std::vector<int64_t>& out) {
    Shard& sh = shards[std::hash<std::string_view>{}(piece) % kShards];
    {
      std::lock_guard<std::mutex> lock(sh.m);
      auto hit = sh.map.find(piece);
      if (hit != sh.map.end()) {
        out.insert(out.end(), hit->second.begin(), hit->second.end());
        return;
      }
    }
    std::vector<int64_t> ids;
    if (!(id_merges && bpe_ids(piece, ids))) bpe_strings(piece, ids);
    out.insert(out.end(), ids.begin(), ids.end());
    if (piece.size() <= 64) {                  // long one-off pieces (base64 blobs, ...) are not worth keeping
      std::lock_guard<std::mutex> lock(sh.m);
      if (sh.map.find(piece) == sh.map.end()) {
        sh.keys.emplace_back(piece);
        sh.map.emplace(std::string_view(sh.keys.back()), std::move(ids));
      }
    }
  }

  void encode_span(const std::string& span, std::vector<int64_t>& out) {
    pretokenize(span, [&](size_t off, size_t len) { bpe(std::string_view(span.data() + off, len), out); });
  }

  std::vector<int64_t> encode(const std::string& text) {
    std::vector<int64_t> out;
    out.reserve(text.size() / 3 + 4);
    size_t pos = 0, span_begin = 0;
    while (pos < text.size()) {
      bool matched = false;
      for (uint32_t k : added_by_first[static_cast<unsigned char>(text[pos])]) {
        const auto& at = added[k];
        if (text.compare(pos, at.first.size(), at.first) == 0) {
          if (pos > span_begin) encode_span(text.substr(span_begin, pos - span_begin), out);
          out.push_back(at.second);
          pos += at.first.size();
          span_begin = pos;
          matched = true;
          break;
        }
      }
      if (!matched) ++pos;
    }
    if (span_begin < text.size()) encode_span(span_begin == 0 ? text : text.substr(span_begin), out);
    return out;
  }

  // texts[i] -> ids, on up to `threads` worker threads pulling indices from one counter
  std::vector<std::vector<int64_t>> encode_batch(const char* const* texts, const int64_t* lens, int64_t n, int threads) {
    std::vector<std::vector<int64_t>> out(static_cast<size_t>(n));
    std::atomic<int64_t> next{0};
    auto work = [&]() {
      for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1))
        out[static_cast<size_t>(i)] = encode(std::string(texts[i], static_cast<size_t>(lens[i])));
    };
    const int64_t nt = std::max<int64_t>(1, std::min<int64_t>(threads, n));
    if (nt == 1) {
      work();
    } else {
      std::vector<std::thread> pool;
      for (int64_t t = 0; t < nt; ++t) pool.emplace_back(work);
      for (auto& th : pool) th.join();
    }
    return out;
  }

  std::string decode(const int64_t* ids, int64_t n, bool skip_special) const {
    std::string out, pending;
    auto flush = [&]() {
      for (const auto& ch : split_utf8(pending)) {
        auto it = uni_to_byte.find(ch);
        if (it != uni_to_byte.end()) out.push_back(static_cast<char>(it->second));
        else out += ch;
      }
      pending.clear();
    };
    for (int64_t i = 0; i < n; ++i) {
      const int64_t id = ids[i];
      if (id < 0 || id >= static_cast<int64_t>(id_to_token.size())) continue;
      auto sp = special_ids.find(id);
      if (sp != special_ids.end()) {  // added tokens are literal text, not byte-mapped
        flush();
        if (!(skip_special && sp->second)) out += id_to_token[static_cast<size_t>(id)];
        continue;
      }
      pending += id_to_token[static_cast<size_t>(id)];
    }
    flush();
    return out;
  }
};

}  // namespace

extern "C" {

void* cverl_bpe_open(const char* tokenizer_json, char* err, int err_len) {
  auto t = std::make_unique<Tokenizer>();
  try {
    t->build_byte_table();
    t->load(tokenizer_json);
    return t.release();
  } catch (const std::exception& e) {
    if (err && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", e.what());
    return nullptr;
  }
}
void cverl_bpe_close(void* h) { delete static_cast<Tokenizer*>(h); }
int64_t cverl_bpe_vocab_size(void* h) { return static_cast<int64_t>(static_cast<Tokenizer*>(h)->id_to_token.size()); }
// which: 0 pad, 1 bos, 2 eos, 3 unk
int64_t cverl_bpe_special_id(void* h, int which) {
  auto* t = static_cast<Tokenizer*>(h);
  switch (which) {
    case 0: return t->pad_id;
    case 1: return t->bos_id;
    case 2: return t->eos_id;
    default: return t->unk_id;
  }
}
int cverl_bpe_uses_pcre2(void* h) { return static_cast<Tokenizer*>(h)->re != nullptr; }
// 1 when the pre-tokenizer pattern runs as JIT-compiled code, and whether merges run on symbol ids
int cverl_bpe_uses_jit(void* h) { return static_cast<Tokenizer*>(h)->jit ? 1 : 0; }
int cverl_bpe_uses_id_merges(void* h) { return static_cast<Tokenizer*>(h)->id_merges ? 1 : 0; }
// Encodes n texts on up to `threads` threads.  offsets[0..n] receive the running token counts; ids of text i go to
// out[offsets[i] .. offsets[i+1]) as far as `capacity` reaches.  Returns the total count (call again with a
// larger buffer when it exceeds `capacity`).
int64_t cverl_bpe_encode_batch(void* h, const char* const* texts, const int64_t* lens, int64_t n, int threads,
                               int64_t* out, int64_t capacity, int64_t* offsets) {
  if (n < 0) return -1;
  auto all = static_cast<Tokenizer*>(h)->encode_batch(texts, lens, n, threads);
  int64_t total = 0;
  for (int64_t i = 0; i < n; ++i) {
    offsets[i] = total;
    for (int64_t id : all[static_cast<size_t>(i)]) {
      if (total < capacity) out[total] = id;
      ++total;
    }
  }
  offsets[n] = total;
  return total;
}
int64_t cverl_bpe_encode(void* h, const char* text, int64_t len, int64_t* out, int64_t capacity) {
  auto ids = static_cast<Tokenizer*>(h)->encode(std::string(text, static_cast<size_t>(len)));
  const int64_t n = static_cast<int64_t>(ids.size());
  for (int64_t i = 0; i < n && i < capacity; ++i) out[i] = ids[static_cast<size_t>(i)];
  return n;
}
int64_t cverl_bpe_decode(void* h, const int64_t* ids, int64_t n, int skip_special, char* out, int64_t capacity) {
  std::string s = static_cast<Tokenizer*>(h)->decode(ids, n, skip_special != 0);
  const int64_t m = static_cast<int64_t>(s.size());
  std::memcpy(out, s.data(), static_cast<size_t>(std::min(m, capacity)));
  return m;
}
}
