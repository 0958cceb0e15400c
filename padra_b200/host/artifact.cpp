#include "artifact.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <variant>

namespace padra_b200::artifact {
namespace {

[[noreturn]] void Fail(const std::string &what) {
  throw std::runtime_error("artifact: " + what);
}
void Require(bool ok, const char *what) {
  if (!ok)
    Fail(what);
}

// ---- a small JSON reader: objects, arrays, strings, non-negative integers, true/false/null --------------------
struct Value;
using Object = std::map<std::string, Value>;
using Array = std::vector<Value>;
struct Value {
  std::variant<std::monostate, bool, std::uint64_t, std::string, std::shared_ptr<Array>, std::shared_ptr<Object>> v;
  bool is_object() const { return std::holds_alternative<std::shared_ptr<Object>>(v); }
  const Object &object() const {
    Require(is_object(), "manifest: object expected");
    return *std::get<std::shared_ptr<Object>>(v);
  }
  const Array &array() const {
    Require(std::holds_alternative<std::shared_ptr<Array>>(v), "manifest: array expected");
    return *std::get<std::shared_ptr<Array>>(v);
  }
  std::uint64_t number() const {
    Require(std::holds_alternative<std::uint64_t>(v), "manifest: number expected");
    return std::get<std::uint64_t>(v);
  }
  const std::string &text() const {
    Require(std::holds_alternative<std::string>(v), "manifest: string expected");
    return std::get<std::string>(v);
  }
};
const Value &Field(const Value &object, const char *name) {
  const auto &o = object.object();
  const auto it = o.find(name);
  if (it == o.end())
    Fail(std::string("manifest: missing field ") + name);
  return it->second;
}

class Parser {
public:
  explicit Parser(const std::string &text) : s_(text) {}
  Value Parse() {
    Value v = ParseValue(0);
    Skip();
    Require(at_ == s_.size(), "manifest: trailing characters");
    return v;
  }

private:
  void Skip() {
    while (at_ < s_.size() && (s_[at_] == ' ' || s_[at_] == '\n' || s_[at_] == '\t' || s_[at_] == '\r'))
      ++at_;
  }
  char Peek() {
    Skip();
    Require(at_ < s_.size(), "manifest: unexpected end");
    return s_[at_];
  }
  void Expect(char c) {
    Require(Peek() == c, "manifest: unexpected character");
    ++at_;
  }
  bool Literal(const char *word) {
    const std::size_t n = std::strlen(word);
    if (s_.compare(at_, n, word) != 0)
      return false;
    at_ += n;
    return true;
  }
  std::string ParseString() {
    Expect('"');
    std::string out;
    while (true) {
      Require(at_ < s_.size(), "manifest: unterminated string");
      const char c = s_[at_++];
      if (c == '"')
        return out;
      if (c == '\\') {
        Require(at_ < s_.size(), "manifest: unterminated escape");
        const char e = s_[at_++];
        switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'n': out += '\n'; break;
        case 't': out += '\t'; break;
        case 'r': out += '\r'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        default: Fail("manifest: unsupported escape");
        }
      } else {
        Require(static_cast<unsigned char>(c) >= 0x20, "manifest: control character in string");
        out += c;
      }
    }
  }
  Value ParseValue(int depth) {
    Require(depth <= 16, "manifest: nested too deeply");
    Value v;
    const char c = Peek();
    if (c == '{') {
      ++at_;
      auto object = std::make_shared<Object>();
      if (Peek() == '}') {
        ++at_;
      } else {
        while (true) {
          std::string key = ParseString();
          Expect(':');
          Require(object->emplace(std::move(key), ParseValue(depth + 1)).second, "manifest: duplicate key");
          if (Peek() == ',') {
            ++at_;
            continue;
          }
          Expect('}');
          break;
        }
      }
      v.v = std::move(object);
    } else if (c == '[') {
      ++at_;
      auto array = std::make_shared<Array>();
      if (Peek() == ']') {
        ++at_;
      } else {
        while (true) {
          array->push_back(ParseValue(depth + 1));
          if (Peek() == ',') {
            ++at_;
            continue;
          }
          Expect(']');
          break;
        }
      }
      v.v = std::move(array);
    } else if (c == '"') {
      v.v = ParseString();
    } else if (c >= '0' && c <= '9') {
      std::uint64_t n = 0;
      while (at_ < s_.size() && s_[at_] >= '0' && s_[at_] <= '9') {
        Require(n <= (UINT64_MAX - 9) / 10, "manifest: number too large");
        n = n * 10 + static_cast<std::uint64_t>(s_[at_++] - '0');
      }
      Require(at_ >= s_.size() || (s_[at_] != '.' && s_[at_] != 'e' && s_[at_] != 'E'), "manifest: integers only");
      v.v = n;
    } else if (Literal("true")) {
      v.v = true;
    } else if (Literal("false")) {
      v.v = false;
    } else if (Literal("null")) {
      v.v = std::monostate{};
    } else {
      Fail("manifest: unexpected character");
    }
    return v;
  }
  const std::string &s_;
  std::size_t at_ = 0;
};

std::string ReadFile(const std::filesystem::path &path, std::uint64_t limit) {
  const auto status = std::filesystem::symlink_status(path);
  if (!std::filesystem::is_regular_file(status) || std::filesystem::is_symlink(status))
    Fail("artifact file must be regular and not a symlink: " + path.string());
  const auto size = std::filesystem::file_size(path);
  if (size > limit)
    Fail("file too large: " + path.string());
  std::ifstream in(path, std::ios::binary);
  std::string out(static_cast<std::size_t>(size), '\0');
  in.read(out.data(), static_cast<std::streamsize>(size));
  if (static_cast<std::uint64_t>(in.gcount()) != size)
    Fail("short read: " + path.string());
  return out;
}

// ---- SHA-256 (FIPS 180-4) ------------------------------------------------------------------------------------
constexpr std::uint32_t kRound[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be,
    0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa,
    0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85,
    0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3,
    0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f,
    0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
std::uint32_t Rotr(std::uint32_t x, int n) {
  return (x >> n) | (x << (32 - n));
}
void Compress(std::uint32_t (&h)[8], const unsigned char *block) {
  std::uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = (std::uint32_t(block[4 * i]) << 24) | (std::uint32_t(block[4 * i + 1]) << 16) | (std::uint32_t(block[4 * i + 2]) << 8) |
           block[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    const std::uint32_t s0 = Rotr(w[i - 15], 7) ^ Rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    const std::uint32_t s1 = Rotr(w[i - 2], 17) ^ Rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  std::uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], k = h[7];
  for (int i = 0; i < 64; ++i) {
    const std::uint32_t t1 = k + (Rotr(e, 6) ^ Rotr(e, 11) ^ Rotr(e, 25)) + ((e & f) ^ (~e & g)) + kRound[i] + w[i];
    const std::uint32_t t2 = (Rotr(a, 2) ^ Rotr(a, 13) ^ Rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
    k = g, g = f, f = e, e = d + t1, d = c, c = b, b = a, a = t1 + t2;
  }
  h[0] += a, h[1] += b, h[2] += c, h[3] += d, h[4] += e, h[5] += f, h[6] += g, h[7] += k;
}

int RateOfFormatName(const std::string &format) {
  return format == "EXL3_K3" ? 3 : format == "EXL3_K4" ? 4 : format == "EXL3_K6" ? 6 : 0;
}
Region ParseRegion(const Value &regions, const char *part) {
  const Value &r = Field(regions, part);
  return Region{Field(r, "offset").number(), Field(r, "bytes").number()};
}
bool IsExpertName(const std::string &name) {
  return name.find(".experts.") != std::string::npos;
}
// "model.layers.<L>.mlp.experts.<E>.<part>_proj.weight" -> layer, or -1
int LayerOfName(const std::string &name) {
  const std::string prefix = "model.layers.";
  if (name.compare(0, prefix.size(), prefix) != 0)
    return -1;
  std::size_t at = prefix.size();
  int layer = 0, digits = 0;
  while (at < name.size() && name[at] >= '0' && name[at] <= '9' && digits < 6)
    layer = layer * 10 + (name[at++] - '0'), ++digits;
  return digits ? layer : -1;
}

} // namespace

int FormatOfRate(int rate) {
  return rate == 3 ? 6 : rate == 4 ? 3 : rate == 6 ? 5 : -1;
}
std::string ProfileOfRate(int rate) {
  Require(FormatOfRate(rate) >= 0, "unsupported EXL3 rate");
  return "mellum16-exl3-k" + std::to_string(rate) + "-fp8-bf16-v1";
}
std::string ExpertTensorName(int layer, int expert, int part) {
  static const char *const kPart[3] = {"gate", "up", "down"};
  Require(part >= 0 && part < 3, "part out of range");
  return "model.layers." + std::to_string(layer) + ".mlp.experts." + std::to_string(expert) + "." + kPart[part] + "_proj.weight";
}

std::string Sha256Hex(const void *data, std::size_t bytes) {
  std::uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  const auto *p = static_cast<const unsigned char *>(data);
  std::size_t left = bytes;
  for (; left >= 64; left -= 64, p += 64)
    Compress(h, p);
  unsigned char tail[128] = {};
  std::memcpy(tail, p, left);
  tail[left] = 0x80;
  const std::size_t padded = left < 56 ? 64 : 128;
  const std::uint64_t bits = static_cast<std::uint64_t>(bytes) * 8;
  for (int i = 0; i < 8; ++i)
    tail[padded - 1 - i] = static_cast<unsigned char>(bits >> (8 * i));
  Compress(h, tail);
  if (padded == 128)
    Compress(h, tail + 64);
  static const char *hex = "0123456789abcdef";
  std::string out;
  for (std::uint32_t word : h)
    for (int shift = 28; shift >= 0; shift -= 4)
      out += hex[(word >> shift) & 15];
  return out;
}

Artifact Load(const std::filesystem::path &directory, bool verify_payload, bool experts_only) {
  const std::string manifest = ReadFile(directory / "manifest.json", 4ull * 1024 * 1024);
  const Value v = Parser(manifest).Parse();
  Require(Field(v, "schema_version").number() == 1, "unsupported manifest schema");
  Artifact a;
  a.directory = directory;
  a.profile = Field(v, "profile").text();
  a.rate = a.profile == ProfileOfRate(3) ? 3 : a.profile == ProfileOfRate(4) ? 4 : a.profile == ProfileOfRate(6) ? 6 : 0;
  Require(a.rate != 0, "unsupported precision/math profile");
  Require(Field(v, "weights_file").text() == "weights.bin", "unsafe weights path");
  a.weights_bytes = Field(v, "weights_bytes").number();
  Require(a.weights_bytes > 0 && a.weights_bytes < 12ull * 1024 * 1024 * 1024, "invalid artifact byte budget");
  const auto payload_path = directory / "weights.bin";
  const auto status = std::filesystem::symlink_status(payload_path);
  Require(std::filesystem::is_regular_file(status) && !std::filesystem::is_symlink(status),
          "artifact file must be regular and not a symlink");
  Require(std::filesystem::file_size(payload_path) == a.weights_bytes, "truncated or oversized weight payload");
  a.weights_sha256 = Field(v, "weights_sha256").text();
  Require(a.weights_sha256.size() == 64 && std::all_of(a.weights_sha256.begin(), a.weights_sha256.end(), [](char c) {
            return (c >= '0' && c <= '9') || (c >= 'a' && c <= 'f');
          }),
          "invalid weight hash");
  const Object &table = Field(v, "tensors").object();
  std::vector<Region> ranges;
  for (const auto &[name, t] : table) {
    if (!IsExpertName(name)) {
      Require(experts_only, "not an expert tensor (pass experts_only to skip others)");
      continue;
    }
    Tensor tensor;
    tensor.name = name;
    const Array &shape = Field(t, "shape").array();
    Require(shape.size() == 2, "wrong tensor rank");
    const std::uint64_t rows = shape[0].number(), cols = shape[1].number();
    Require(rows >= 128 && cols >= 128 && rows % 128 == 0 && cols % 128 == 0 && rows <= (1u << 20) && cols <= (1u << 20),
            "wrong tensor shape");
    tensor.rows = static_cast<int>(rows), tensor.cols = static_cast<int>(cols);
    tensor.rate = RateOfFormatName(Field(t, "format").text());
    Require(tensor.rate == a.rate, "tensor precision does not match selected hybrid");
    Require(Field(t, "codebook").text() == "mul1" && Field(t, "hadamard_block").number() == 128,
            "unsupported EXL3 codec/transform");
    const Value &regions = Field(t, "regions");
    Require(regions.object().size() == 3, "unknown/missing weight regions");
    tensor.packed = ParseRegion(regions, "packed");
    tensor.suh = ParseRegion(regions, "suh");
    tensor.svh = ParseRegion(regions, "svh");
    const std::uint64_t want[3] = {rows * cols * static_cast<std::uint64_t>(a.rate) / 8, cols * 2, rows * 2};
    const Region *got[3] = {&tensor.packed, &tensor.suh, &tensor.svh};
    for (int i = 0; i < 3; ++i) {
      Require(got[i]->offset % 256 == 0 && got[i]->bytes == want[i] && got[i]->offset <= a.weights_bytes &&
                  got[i]->bytes <= a.weights_bytes - got[i]->offset,
              "invalid region range/alignment/bytes");
      ranges.push_back(*got[i]);
    }
    a.layers = std::max(a.layers, LayerOfName(name) + 1);
    a.tensors.emplace(name, std::move(tensor));
  }
  Require(!a.tensors.empty(), "incomplete/extra tensor inventory");
  if (!experts_only) { // an experts-only view of a whole checkpoint leaves the other tensors' bytes unaccounted
    std::sort(ranges.begin(), ranges.end(), [](const Region &x, const Region &y) { return x.offset < y.offset; });
    std::uint64_t cursor = 0;
    for (const Region &r : ranges) {
      Require(r.offset == (cursor + 255) / 256 * 256, "overlapping/noncanonical weight regions");
      cursor = r.offset + r.bytes;
    }
    Require(cursor == a.weights_bytes, "unaccounted payload bytes");
  }
  if (verify_payload) {
    const std::string payload = ReadFile(payload_path, a.weights_bytes);
    Require(Sha256Hex(payload.data(), payload.size()) == a.weights_sha256, "weight SHA-256 mismatch");
    for (const auto &[name, t] : a.tensors)
      for (const Region *r : {&t.suh, &t.svh})
        for (std::uint64_t j = 0; j < r->bytes; j += 2) {
          std::uint16_t x;
          std::memcpy(&x, payload.data() + r->offset + j, 2);
          Require((x & 0x7c00) != 0x7c00, "nonfinite EXL3 FP16 sidecar");
          Require((x & 0x7fff) != 0, "zero EXL3 sidecar");
        }
  }
  return a;
}

void Write(const std::filesystem::path &directory, int rate, const std::vector<TensorBytes> &tensors) {
  Require(FormatOfRate(rate) >= 0, "unsupported EXL3 rate");
  Require(!tensors.empty(), "nothing to write");
  std::filesystem::create_directories(directory);
  std::string payload;
  std::ostringstream table;
  bool first = true;
  for (const TensorBytes &t : tensors) {
    Require(t.rows >= 128 && t.cols >= 128 && t.rows % 128 == 0 && t.cols % 128 == 0 && t.packed && t.suh && t.svh, "wrong tensor shape");
    const std::uint64_t sizes[3] = {static_cast<std::uint64_t>(t.rows) * t.cols * rate / 8, static_cast<std::uint64_t>(t.cols) * 2,
                                    static_cast<std::uint64_t>(t.rows) * 2};
    const void *sources[3] = {t.packed, t.suh, t.svh};
    static const char *const kNames[3] = {"packed", "suh", "svh"};
    table << (first ? "" : ",") << "\n  \"" << t.name << "\": {\"shape\": [" << t.rows << ", " << t.cols << "], \"format\": \"EXL3_K" << rate
          << "\", \"codebook\": \"mul1\", \"hadamard_block\": 128, \"regions\": {";
    for (int i = 0; i < 3; ++i) {
      payload.resize((payload.size() + 255) / 256 * 256, '\0');
      table << (i ? ", " : "") << "\"" << kNames[i] << "\": {\"offset\": " << payload.size() << ", \"bytes\": " << sizes[i] << "}";
      payload.append(static_cast<const char *>(sources[i]), static_cast<std::size_t>(sizes[i]));
    }
    table << "}}";
    first = false;
  }
  {
    std::ofstream out(directory / "weights.bin", std::ios::binary | std::ios::trunc);
    out.write(payload.data(), static_cast<std::streamsize>(payload.size()));
    Require(out.good(), "cannot write weights.bin");
  }
  std::ofstream out(directory / "manifest.json", std::ios::trunc);
  out << "{\n \"schema_version\": 1,\n \"profile\": \"" << ProfileOfRate(rate) << "\",\n \"weights_file\": \"weights.bin\",\n \"weights_bytes\": "
      << payload.size() << ",\n \"weights_sha256\": \"" << Sha256Hex(payload.data(), payload.size()) << "\",\n \"tensors\": {" << table.str()
      << "\n }\n}\n";
  Require(out.good(), "cannot write manifest.json");
}

std::vector<padra_matrix> Bind(const Artifact &artifact, const unsigned char *arena, std::uint64_t arena_bytes) {
  Require(arena != nullptr && artifact.layers > 0, "nothing to bind");
  std::vector<padra_matrix> table(static_cast<std::size_t>(artifact.layers) * 64 * 3);
  for (int layer = 0; layer < artifact.layers; ++layer)
    for (int expert = 0; expert < 64; ++expert)
      for (int part = 0; part < 3; ++part) {
        const auto it = artifact.tensors.find(ExpertTensorName(layer, expert, part));
        if (it == artifact.tensors.end())
          Fail("missing tensor " + ExpertTensorName(layer, expert, part));
        const Tensor &t = it->second;
        for (const Region *r : {&t.packed, &t.suh, &t.svh})
          Require(r->offset <= arena_bytes && r->bytes <= arena_bytes - r->offset, "invalid production matrix region");
        padra_matrix &m = table[(static_cast<std::size_t>(layer) * 64 + expert) * 3 + part];
        m.data = arena + t.packed.offset;
        m.scales = nullptr, m.divisor = nullptr;
        m.rows = t.rows, m.cols = t.cols, m.format = FormatOfRate(t.rate);
        m.suh = reinterpret_cast<const std::uint16_t *>(arena + t.suh.offset);
        m.svh = reinterpret_cast<const std::uint16_t *>(arena + t.svh.offset);
      }
  return table;
}

} // namespace padra_b200::artifact
