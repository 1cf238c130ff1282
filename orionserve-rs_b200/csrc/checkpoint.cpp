// Checkpoint directory -> device weights, without a host copy of the model: every
// `*.safetensors` file is memory-mapped, its JSON header parsed, and each tensor the model uses is
// handed to load_tensor straight from the mapping (which cuts this rank's slice, converts once
// and uploads). Follows CheckpointLoader::open / tensor (crates/orion-models/src/loader.rs:112-235)
// and ModelWeights::load (crates/orion-models/src/transformer.rs:62-120):
//   * files are taken in name order and the FIRST file wins for a duplicated tensor name;
//   * F32, F16 and BF16 are accepted, anything else is UnsupportedDtype naming the tensor;
//   * tensors the model never asks for (rotary inv_freq buffers and the like) are ignored;
//   * a missing tensor is reported by finalize() with the reference's wording.
// The file format is that of safetensors 0.8.0 (Cargo.lock:2140): u64 little-endian header
// length, a JSON object {name: {"dtype", "shape", "data_offsets": [begin, end]}} with an optional
// "__metadata__" entry, then the raw little-endian data.
#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include "model.h"

namespace orion {
namespace {

struct TensorInfo {
  std::string name, dtype;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;
};

// Just enough JSON for a safetensors header: objects, arrays, strings, non-negative integers and
// the scalar literals; values of unknown keys are skipped structurally.
class HeaderParser {
 public:
  HeaderParser(const char *p, size_t n) : p_(p), end_(p + n) {}

  bool parse(std::vector<TensorInfo> *out, std::string *why) {
    ws();
    if (!eat('{')) return fail("header is not a JSON object", why);
    ws();
    if (eat('}')) return true;
    for (;;) {
      std::string name;
      if (!string(&name)) return fail("expected a tensor name", why);
      ws();
      if (!eat(':')) return fail("expected ':' after a tensor name", why);
      ws();
      if (name == "__metadata__") {
        if (!skip_value()) return fail("malformed __metadata__", why);
      } else {
        TensorInfo t;
        t.name = name;
        if (!tensor(&t)) return fail(("malformed entry for tensor `" + name + "`").c_str(), why);
        out->push_back(std::move(t));
      }
      ws();
      if (eat(',')) { ws(); continue; }
      if (eat('}')) return true;
      return fail("expected ',' or '}'", why);
    }
  }

 private:
  bool fail(const char *msg, std::string *why) {
    *why = msg;
    return false;
  }
  void ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool eat(char c) {
    if (p_ < end_ && *p_ == c) { ++p_; return true; }
    return false;
  }
  bool string(std::string *out) {
    if (!eat('"')) return false;
    out->clear();
    while (p_ < end_ && *p_ != '"') {
      if (*p_ == '\\') {
        if (++p_ >= end_) return false;
        switch (*p_) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'u':  // tensor names are ASCII; keep the escape verbatim
            out->append("\\u");
            break;
          default: out->push_back(*p_);
        }
        ++p_;
      } else {
        out->push_back(*p_++);
      }
    }
    return eat('"');
  }
  bool number(uint64_t *v) {
    if (p_ >= end_ || *p_ < '0' || *p_ > '9') return false;
    uint64_t x = 0;
    while (p_ < end_ && *p_ >= '0' && *p_ <= '9') x = x * 10 + (uint64_t)(*p_++ - '0');
    *v = x;
    return true;
  }
  bool numbers(std::vector<uint64_t> *out) {
    if (!eat('[')) return false;
    ws();
    if (eat(']')) return true;
    for (;;) {
      uint64_t v;
      if (!number(&v)) return false;
      out->push_back(v);
      ws();
      if (eat(',')) { ws(); continue; }
      return eat(']');
    }
  }
  bool skip_value() {
    ws();
    if (p_ >= end_) return false;
    if (*p_ == '"') { std::string s; return string(&s); }
    if (*p_ == '{' || *p_ == '[') {
      const char open = *p_, close = open == '{' ? '}' : ']';
      ++p_;
      ws();
      if (eat(close)) return true;
      for (;;) {
        if (open == '{') {
          std::string k;
          if (!string(&k)) return false;
          ws();
          if (!eat(':')) return false;
        }
        if (!skip_value()) return false;
        ws();
        if (eat(',')) { ws(); continue; }
        return eat(close);
      }
    }
    while (p_ < end_ && *p_ != ',' && *p_ != '}' && *p_ != ']') ++p_;  // number, true, false, null
    return true;
  }
  bool tensor(TensorInfo *t) {
    if (!eat('{')) return false;
    bool got_dtype = false, got_shape = false, got_off = false;
    ws();
    if (eat('}')) return false;
    for (;;) {
      std::string key;
      if (!string(&key)) return false;
      ws();
      if (!eat(':')) return false;
      ws();
      if (key == "dtype") {
        got_dtype = string(&t->dtype);
        if (!got_dtype) return false;
      } else if (key == "shape") {
        got_shape = numbers(&t->shape);
        if (!got_shape) return false;
      } else if (key == "data_offsets") {
        std::vector<uint64_t> off;
        if (!numbers(&off) || off.size() != 2 || off[1] < off[0]) return false;
        t->begin = off[0];
        t->end = off[1];
        got_off = true;
      } else if (!skip_value()) {
        return false;
      }
      ws();
      if (eat(',')) { ws(); continue; }
      if (!eat('}')) return false;
      return got_dtype && got_shape && got_off;
    }
  }
  const char *p_, *end_;
};

struct Mapping {
  std::string path;
  void *base = MAP_FAILED;
  size_t size = 0;
  ~Mapping() {
    if (base != MAP_FAILED) munmap(base, size);
  }
};

// Names ModelWeights::load asks for (transformer.rs:12-18, 73-118).
bool model_uses(const std::string &name, uint32_t num_layers) {
  if (name == "model.embed_tokens.weight" || name == "model.norm.weight" || name == "lm_head.weight") return true;
  static const char prefix[] = "model.layers.";
  if (name.compare(0, sizeof prefix - 1, prefix) != 0) return false;
  size_t i = sizeof prefix - 1, digits = 0;
  uint64_t layer = 0;
  while (i < name.size() && name[i] >= '0' && name[i] <= '9' && digits < 9) {
    layer = layer * 10 + (uint64_t)(name[i] - '0');
    ++i;
    ++digits;
  }
  if (digits == 0 || i >= name.size() || name[i] != '.' || layer >= num_layers) return false;
  static const char *rest[] = {"input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                               "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                               "self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias",
                               "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"};
  for (const char *r : rest)
    if (name.compare(i + 1, std::string::npos, r) == 0) return true;
  return false;
}

}  // namespace

int load_checkpoint(ModelBase *model, const char *directory, uint64_t *tensors_loaded) {
  if (tensors_loaded) *tensors_loaded = 0;
  if (!directory) return set_error(ORION_ERR_INVALID_REQUEST, "null checkpoint directory");
  DIR *d = opendir(directory);
  if (!d) return set_error(ORION_ERR_MODEL, "path not found: %s", directory);  // ModelError::PathNotFound
  std::vector<std::string> files;
  while (dirent *e = readdir(d)) {
    const std::string n = e->d_name;
    static const std::string ext = ".safetensors";
    if (n.size() > ext.size() && n.compare(n.size() - ext.size(), ext.size(), ext) == 0) files.push_back(n);
  }
  closedir(d);
  std::sort(files.begin(), files.end());  // loader.rs:128-130: a duplicated name always resolves the same way
  if (files.empty()) return set_error(ORION_ERR_MODEL, "missing file: %s/*.safetensors", directory);

  const uint32_t num_layers = model->desc().num_layers;
  std::set<std::string> seen;
  uint64_t loaded = 0;
  for (const std::string &f : files) {
    Mapping m;
    m.path = std::string(directory) + "/" + f;
    const int fd = open(m.path.c_str(), O_RDONLY);
    if (fd < 0) return set_error(ORION_ERR_MODEL, "i/o error on %s: %s", m.path.c_str(), strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
      close(fd);
      return set_error(ORION_ERR_MODEL, "malformed checkpoint %s: shorter than its header length", m.path.c_str());
    }
    m.size = (size_t)st.st_size;
    m.base = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m.base == MAP_FAILED) return set_error(ORION_ERR_MODEL, "i/o error on %s: %s", m.path.c_str(), strerror(errno));
    const uint8_t *bytes = static_cast<const uint8_t *>(m.base);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | bytes[i];
    if (hlen > m.size - 8)
      return set_error(ORION_ERR_MODEL, "malformed checkpoint %s: header length %llu exceeds the file", m.path.c_str(),
                       (unsigned long long)hlen);
    std::vector<TensorInfo> tensors;
    std::string why;
    if (!HeaderParser(reinterpret_cast<const char *>(bytes + 8), hlen).parse(&tensors, &why))
      return set_error(ORION_ERR_MODEL, "malformed checkpoint %s: %s", m.path.c_str(), why.c_str());
    const uint64_t data_size = m.size - 8 - hlen;
    for (const TensorInfo &t : tensors) {
      if (!seen.insert(t.name).second) continue;  // an earlier file already provided it
      if (!model_uses(t.name, num_layers)) continue;
      int dtype;
      size_t es;
      if (t.dtype == "F32") { dtype = ORION_DTYPE_F32; es = 4; }
      else if (t.dtype == "F16") { dtype = ORION_DTYPE_F16; es = 2; }
      else if (t.dtype == "BF16") { dtype = ORION_DTYPE_BF16; es = 2; }
      else return set_error(ORION_ERR_MODEL, "unsupported dtype %s (tensor `%s`)", t.dtype.c_str(), t.name.c_str());
      uint64_t count = 1;
      for (uint64_t s : t.shape) count *= s;
      if (t.end > data_size || t.end - t.begin != count * es || t.shape.empty() || t.shape.size() > 2)
        return set_error(ORION_ERR_MODEL, "malformed checkpoint %s: tensor `%s` does not match its byte range",
                         m.path.c_str(), t.name.c_str());
      ORION_TRY(model->load_tensor(t.name.c_str(), dtype, t.shape.data(), (int)t.shape.size(), bytes + 8 + hlen + t.begin));
      ++loaded;
    }
  }
  if (tensors_loaded) *tensors_loaded = loaded;
  return model->finalize();
}

}  // namespace orion
