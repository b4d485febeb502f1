// Times the reference's HfBpeTokenizer (its public class, include/cverl/text/hf_bpe_tokenizer.h:52-75) on a file
// of documents separated by a form feed ('\f'), one encode() call per document, and prints one JSON line.
// Linked against the unmodified reference objects that baseline/build_ref.py compiled.
//   ref_tokenizer_bench TOKENIZER.json DOCS.txt [repeats]
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "cverl/text/hf_bpe_tokenizer.h"

int main(int argc, char** argv) {
  if (argc < 3) {
    std::fprintf(stderr, "usage: %s TOKENIZER.json DOCS.txt [repeats]\n", argv[0]);
    return 2;
  }
  const int repeats = argc > 3 ? std::atoi(argv[3]) : 1;
  cverl::text::HfBpeTokenizerOptions options;
  options.tokenizer_json_path = argv[1];
  cverl::text::HfBpeTokenizer tokenizer(options);
  std::ifstream f(argv[2], std::ios::binary);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string all = ss.str();
  std::vector<std::string> docs;
  for (size_t b = 0; b < all.size();) {
    size_t e = all.find('\f', b);
    if (e == std::string::npos) e = all.size();
    docs.push_back(all.substr(b, e - b));
    b = e + 1;
  }
  size_t bytes = 0;
  for (const auto& d : docs) bytes += d.size();
  double best = 1e30;
  size_t tokens = 0;
  unsigned long long checksum = 0;
  for (int r = 0; r < repeats; ++r) {
    tokens = 0;
    checksum = 0;
    const auto t0 = std::chrono::steady_clock::now();
    for (const auto& d : docs) {
      const auto ids = tokenizer.encode(d);
      tokens += ids.size();
      for (int32_t id : ids) checksum = checksum * 1000003ULL + static_cast<unsigned long long>(id);
    }
    const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (s < best) best = s;
  }
  std::printf("{\"impl\": \"reference\", \"docs\": %zu, \"bytes\": %zu, \"tokens\": %zu, \"seconds\": %.6f, "
              "\"mb_per_s\": %.3f, \"checksum\": %llu}\n",
              docs.size(), bytes, tokens, best, bytes / best / 1e6, checksum);
  return 0;
}
