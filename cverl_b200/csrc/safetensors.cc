// safetensors reader (any number of shards in a model directory) and single-file writer.
//
// Reader: scans the 8-byte length + JSON header of every *.safetensors file with a small
// hand-written JSON scanner (no JSON library), builds an index name -> (file, dtype, shape,
// byte range), and reads one tensor at a time by seeking; `model.safetensors.index.json` is
// not needed.  Writer: {"__metadata__":{"format":"pt"}, name:{dtype,shape,data_offsets}},
// header padded with spaces so that the data section starts 8-byte aligned.
// Behaviour follows the reference (src/model/hf_model_loader.cc:55-373,
// src/model/safetensors_writer.cc:92-159); dtypes F32/F16/BF16/I64/I32/U8.
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <dirent.h>
#include <fcntl.h>
#include <fstream>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

struct TensorInfo {
  std::string file;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range inside the data section
  uint64_t data_start = 0;      // offset of the data section in the file
};

struct Scanner {
  const std::string& s;
  size_t i = 0;
  explicit Scanner(const std::string& text) : s(text) {}
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) {
      ++i;
      return true;
    }
    return false;
  }
  void expect(char c) {
    if (!eat(c)) throw std::runtime_error(std::string("safetensors header: expected '") + c + "'");
  }
  uint32_t hex4(size_t at) const {
    if (at + 4 > s.size()) throw std::runtime_error("safetensors header: truncated \\u escape");
    uint32_t v = 0;
    for (size_t k = at; k < at + 4; ++k) {
      const char c = s[k];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= static_cast<uint32_t>(c - '0');
      else if (c >= 'a' && c <= 'f') v |= static_cast<uint32_t>(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= static_cast<uint32_t>(c - 'A' + 10);
      else throw std::runtime_error("safetensors header: bad \\u escape");
    }
    return v;
  }
  static void append_utf8(uint32_t cp, std::string& out) {
    if (cp < 0x80) {
      out.push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
      out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  std::string str() {
    ws();
    if (i >= s.size() || s[i] != '"') throw std::runtime_error("safetensors header: expected string");
    ++i;
    std::string out;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        ++i;
        switch (s[i]) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'u': {                        // \uXXXX, a surrogate pair when two follow each other: UTF-8 out
            uint32_t cp = hex4(i + 1);
            i += 4;
            if (cp >= 0xD800 && cp <= 0xDBFF && i + 6 < s.size() && s[i + 1] == '\\' && s[i + 2] == 'u') {
              const uint32_t lo = hex4(i + 3);
              if (lo >= 0xDC00 && lo <= 0xDFFF) {
                cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                i += 6;
              }
            }
            append_utf8(cp, out);
            break;
          }
          default: out.push_back(s[i]);
        }
      } else {
        out.push_back(s[i]);
      }
      ++i;
    }
    if (i >= s.size()) throw std::runtime_error("safetensors header: unterminated string");
    ++i;
    return out;
  }
  int64_t integer() {
    ws();
    size_t j = i;
    if (j < s.size() && (s[j] == '-' || s[j] == '+')) ++j;
    while (j < s.size() && s[j] >= '0' && s[j] <= '9') ++j;
    if (j == i) throw std::runtime_error("safetensors header: expected integer");
    int64_t v = std::stoll(s.substr(i, j - i));
    i = j;
    return v;
  }
  void skip_value() {  // skip any JSON value
    ws();
    if (i >= s.size()) throw std::runtime_error("safetensors header: truncated");
    char c = s[i];
    if (c == '"') {
      str();
    } else if (c == '{' || c == '[') {
      char open = c, close = (c == '{') ? '}' : ']';
      int depth = 0;
      while (i < s.size()) {
        if (s[i] == '"') {
          str();
          continue;
        }
        if (s[i] == open) ++depth;
        if (s[i] == close && --depth == 0) {
          ++i;
          return;
        }
        ++i;
      }
      throw std::runtime_error("safetensors header: unbalanced brackets");
    } else {
      while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') ++i;
    }
  }
};

struct Index {
  std::map<std::string, TensorInfo> tensors;
  std::vector<std::string> names;  // insertion order
  std::string last_error;
};

void scan_file(const std::string& path, Index& idx) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  uint64_t hlen = 0;
  f.read(reinterpret_cast<char*>(&hlen), 8);
  if (!f || hlen == 0 || hlen > (1ull << 31)) throw std::runtime_error("bad safetensors header length in " + path);
  std::string header(hlen, '\0');
  f.read(&header[0], static_cast<std::streamsize>(hlen));
  if (!f) throw std::runtime_error("truncated safetensors header in " + path);
  Scanner sc(header);
  sc.expect('{');
  if (sc.eat('}')) return;
  do {
    std::string name = sc.str();
    sc.expect(':');
    if (name == "__metadata__") {
      sc.skip_value();
      continue;
    }
    TensorInfo info;
    info.file = path;
    info.data_start = 8 + hlen;
    sc.expect('{');
    do {
      std::string key = sc.str();
      sc.expect(':');
      if (key == "dtype") {
        info.dtype = sc.str();
      } else if (key == "shape") {
        sc.expect('[');
        if (!sc.eat(']')) {
          do info.shape.push_back(sc.integer());
          while (sc.eat(','));
          sc.expect(']');
        }
      } else if (key == "data_offsets") {
        sc.expect('[');
        info.begin = static_cast<uint64_t>(sc.integer());
        sc.expect(',');
        info.end = static_cast<uint64_t>(sc.integer());
        sc.expect(']');
      } else {
        sc.skip_value();
      }
    } while (sc.eat(','));
    sc.expect('}');
    if (!idx.tensors.count(name)) idx.names.push_back(name);
    idx.tensors[name] = info;
  } while (sc.eat(','));
  sc.expect('}');
}

int dtype_code(const std::string& d) {
  if (d == "F32") return 0;
  if (d == "F16") return 1;
  if (d == "BF16") return 2;
  if (d == "I64") return 3;
  if (d == "I32") return 4;
  if (d == "U8") return 5;
  return -1;
}
const char* dtype_name(int c) {
  static const char* names[] = {"F32", "F16", "BF16", "I64", "I32", "U8"};
  return (c >= 0 && c < 6) ? names[c] : nullptr;
}
int dtype_size(int c) {
  static const int sizes[] = {4, 2, 2, 8, 4, 1};
  return (c >= 0 && c < 6) ? sizes[c] : 0;
}
bool ends_with(const std::string& s, const std::string& suffix) {
  return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

}  // namespace

extern "C" {

// Opens a model directory (every *.safetensors inside, sorted by name) or a single file.
void* cverl_st_open(const char* path, char* err, int err_len) {
  auto idx = std::make_unique<Index>();
  try {
    struct stat st;
    if (stat(path, &st) != 0) throw std::runtime_error(std::string("no such path: ") + path);
    std::vector<std::string> files;
    if (S_ISDIR(st.st_mode)) {
      DIR* d = opendir(path);
      if (!d) throw std::runtime_error("cannot list directory");
      while (dirent* e = readdir(d)) {
        std::string n = e->d_name;
        if (ends_with(n, ".safetensors")) files.push_back(std::string(path) + "/" + n);
      }
      closedir(d);
      std::sort(files.begin(), files.end());
      if (files.empty()) throw std::runtime_error("no .safetensors files in directory");
    } else {
      files.push_back(path);
    }
    for (const auto& f : files) scan_file(f, *idx);
    return idx.release();
  } catch (const std::exception& e) {
    if (err && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), "%s", e.what());
    return nullptr;
  }
}

void cverl_st_close(void* h) { delete static_cast<Index*>(h); }

int64_t cverl_st_count(void* h) { return static_cast<int64_t>(static_cast<Index*>(h)->names.size()); }

const char* cverl_st_name(void* h, int64_t i) {
  auto* idx = static_cast<Index*>(h);
  if (i < 0 || i >= static_cast<int64_t>(idx->names.size())) return nullptr;
  return idx->names[static_cast<size_t>(i)].c_str();
}

// dtype code (0 F32, 1 F16, 2 BF16, 3 I64, 4 I32, 5 U8), rank, shape (up to 8 dims), byte size.
int cverl_st_info(void* h, const char* name, int* dtype, int* ndim, int64_t* shape8, int64_t* nbytes) {
  auto* idx = static_cast<Index*>(h);
  auto it = idx->tensors.find(name);
  if (it == idx->tensors.end()) return 1;
  const TensorInfo& t = it->second;
  const int code = dtype_code(t.dtype);
  if (code < 0 || t.shape.size() > 8) return 2;
  *dtype = code;
  *ndim = static_cast<int>(t.shape.size());
  for (size_t i = 0; i < t.shape.size(); ++i) shape8[i] = t.shape[i];
  *nbytes = static_cast<int64_t>(t.end - t.begin);
  return 0;
}

// Reads bytes [offset, offset + nbytes) of a tensor's data into dst with pread, split over up to `threads`
// threads in pieces of at least 4 MiB (threads <= 0: one per 32 MiB, at most 8).  A contiguous range of rows of a
// row-major tensor is such a byte range, so a tensor-parallel rank reads only its rows.
int cverl_st_read_range(void* h, const char* name, int64_t offset, int64_t nbytes, void* dst, int threads) {
  auto* idx = static_cast<Index*>(h);
  auto it = idx->tensors.find(name);
  if (it == idx->tensors.end()) return 1;
  const TensorInfo& t = it->second;
  const int64_t size = static_cast<int64_t>(t.end - t.begin);
  if (offset < 0 || nbytes < 0 || offset + nbytes > size) return 2;
  if (nbytes == 0) return 0;
  const int fd = open(t.file.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) return 3;
  const int64_t base = static_cast<int64_t>(t.data_start + t.begin) + offset;
  constexpr int64_t kMinPiece = 4ll << 20;
  int64_t nt = threads > 0 ? threads : std::min<int64_t>(8, nbytes / (32ll << 20) + 1);
  nt = std::max<int64_t>(1, std::min<int64_t>(nt, (nbytes + kMinPiece - 1) / kMinPiece));
  const int64_t piece = ((nbytes + nt - 1) / nt + 4095) / 4096 * 4096;
  std::atomic<int> bad{0};
  auto work = [&](int64_t k) {
    int64_t lo = k * piece, hi = std::min(nbytes, lo + piece);
    while (lo < hi) {
      const ssize_t got = pread(fd, static_cast<char*>(dst) + lo, static_cast<size_t>(hi - lo), base + lo);
      if (got <= 0) {
        if (got < 0 && errno == EINTR) continue;
        bad.store(1);
        return;
      }
      lo += got;
    }
  };
  if (nt == 1) {
    work(0);
  } else {
    std::vector<std::thread> pool;
    for (int64_t k = 0; k < nt; ++k) pool.emplace_back(work, k);
    for (auto& th : pool) th.join();
  }
  close(fd);
  return bad.load() ? 4 : 0;
}

int cverl_st_read(void* h, const char* name, void* dst, int64_t nbytes) {
  auto* idx = static_cast<Index*>(h);
  auto it = idx->tensors.find(name);
  if (it == idx->tensors.end()) return 1;
  if (nbytes != static_cast<int64_t>(it->second.end - it->second.begin)) return 2;
  return cverl_st_read_range(h, name, 0, nbytes, dst, 0);
}

// Writes one file (tmp + rename).  shapes is a flat array of sum(ndims) extents.
int cverl_st_write(const char* path, int64_t n, const char* const* names, const int* dtypes, const int* ndims,
                   const int64_t* shapes, const void* const* data) {
  try {
    std::string header = "{\"__metadata__\":{\"format\":\"pt\"}";
    uint64_t offset = 0;
    std::vector<uint64_t> sizes(static_cast<size_t>(n));
    const int64_t* sp = shapes;
    for (int64_t i = 0; i < n; ++i) {
      const int esz = dtype_size(dtypes[i]);
      if (esz == 0) return 2;
      uint64_t numel = 1;
      std::string shape_json = "[";
      for (int d = 0; d < ndims[i]; ++d) {
        numel *= static_cast<uint64_t>(sp[d]);
        shape_json += (d ? "," : "") + std::to_string(sp[d]);
      }
      shape_json += "]";
      sp += ndims[i];
      sizes[static_cast<size_t>(i)] = numel * static_cast<uint64_t>(esz);
      std::string nm;
      for (const char* c = names[i]; *c; ++c) {
        const unsigned char u = static_cast<unsigned char>(*c);
        if (u < 0x20) {                       // control characters must be escaped in JSON
          char buf[8];
          std::snprintf(buf, sizeof(buf), "\\u%04x", u);
          nm += buf;
          continue;
        }
        if (*c == '"' || *c == '\\') nm.push_back('\\');
        nm.push_back(*c);
      }
      header += ",\"" + nm + "\":{\"dtype\":\"" + dtype_name(dtypes[i]) + "\",\"shape\":" + shape_json +
                ",\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + sizes[i]) + "]}";
      offset += sizes[static_cast<size_t>(i)];
    }
    header += "}";
    while ((8 + header.size()) % 8 != 0) header.push_back(' ');
    const std::string tmp = std::string(path) + ".tmp";
    {
      std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
      if (!f) return 3;
      const uint64_t hlen = header.size();
      f.write(reinterpret_cast<const char*>(&hlen), 8);
      f.write(header.data(), static_cast<std::streamsize>(header.size()));
      for (int64_t i = 0; i < n; ++i)
        f.write(static_cast<const char*>(data[i]), static_cast<std::streamsize>(sizes[static_cast<size_t>(i)]));
      if (!f) return 4;
    }
    if (std::rename(tmp.c_str(), path) != 0) return 5;
    return 0;
  } catch (const std::exception&) {
    return 6;
  }
}
}
