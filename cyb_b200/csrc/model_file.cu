// Reader of the `.model` container (a `.cyb` file) and loader into a decoder.
//
// The container's three rules are the reference's (reference/format.md:16-18, 110-117): TOML
// frontmatter until the first line that starts with `~~~`; `~~~name` + LF opens every file inside;
// binary files carry `size` in the frontmatter (text files run to the next `~~~` line or EOF, text
// before binary).  What a model container holds is "config (TOML), graph IR, tensor index, tensor
// data (Q4/Q8/F16/F32)" with HuggingFace tensor names (decide/pipeline.md:28-30); the page that
// would fix the tensor-index schema (`cyb-model`) is not part of the reference checkout, so the
// schema read here is this engine's own:
//
//   ~~~config    TOML: hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
//                num_key_value_heads, head_dim, vocab_size, rms_norm_eps, rope_theta; optional
//                attn_logit_softcapping, sliding_window, final_logit_softcapping
//   ~~~tensors   TOML array of tables [[tensor]]: name, dtype ("Q4" | "Q4_0" | "Q8" (= "Q8_0") | "Q4_K" | "F32" | "F16" | "BF16"),
//                shape = [rows, cols] (or [n]), offset and size in bytes inside `weights`
//   ~~~weights   binary.  Q4 = row-major 32-blocks of 18 bytes: f16 scale, then 16 bytes holding the
//                codes of k = 2i (low nibble) and k = 2i + 1 (high nibble); w = (code - 8) * scale.
//                Q4_0 = the same block with the nibble order of the published format of that name (byte i:
//                k = i low, k = i + 16 high).  Q8 = row-major 32-blocks of 34 bytes: f16 scale, then 32 signed bytes; w = q * scale.
//                Q4_K = row-major super-blocks of 144 bytes per 256 weights (the published layout).
//
// The file is mapped read-only (the reference maps its model files, shell/src/lib.rs:31-33); Q4
// tensors are re-tiled straight from the map, F32 / F16 / BF16 linear weights go through the
// device quantiser (qeng_weight_quantize_q4) first.
#include <errno.h>
#include <fcntl.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "qeng_internal.h"

namespace {

struct Tensor {
  std::string name, dtype;
  std::vector<int64_t> shape;
  int64_t offset = -1, size = -1;
};
struct FileEntry {
  std::string name, format;
  int64_t size = -1;  // binary files only
  const char* data = nullptr;
  int64_t len = 0;
};
struct ModelFile {
  int fd = -1;
  const char* base = nullptr;
  size_t bytes = 0;
  std::vector<FileEntry> files;
  std::map<std::string, std::string> config;  // key -> raw value text
  std::vector<Tensor> tensors;
  std::string err;
  ~ModelFile() {
    if (base) munmap(const_cast<char*>(base), bytes);
    if (fd >= 0) close(fd);
  }
};

std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r')) ++a;
  while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r')) --b;
  return s.substr(a, b - a);
}
std::string unquote(const std::string& v) {
  if (v.size() >= 2 && (v[0] == '"' || v[0] == '\'') && v.back() == v[0]) return v.substr(1, v.size() - 2);
  return v;
}
// strips a trailing comment that is outside a quoted string
std::string strip_comment(const std::string& line) {
  bool in = false;
  char qc = 0;
  for (size_t i = 0; i < line.size(); ++i) {
    const char c = line[i];
    if (in) {
      if (c == qc) in = false;
    } else if (c == '"' || c == '\'') {
      in = true;
      qc = c;
    } else if (c == '#') {
      return line.substr(0, i);
    }
  }
  return line;
}
bool parse_int(const std::string& v, int64_t* out) {
  std::string t;
  for (char c : v)
    if (c != '_') t += c;
  if (t.empty()) return false;
  char* end = nullptr;
  errno = 0;
  const long long x = strtoll(t.c_str(), &end, 10);
  if (errno != 0 || *end != 0) return false;
  *out = x;
  return true;
}
bool parse_int_array(const std::string& v, std::vector<int64_t>* out) {
  const std::string t = trim(v);
  if (t.size() < 2 || t.front() != '[' || t.back() != ']') return false;
  out->clear();
  std::string cur;
  for (size_t i = 1; i + 1 <= t.size(); ++i) {
    const char c = i + 1 == t.size() ? ',' : t[i];
    if (c == ',') {
      const std::string e = trim(cur);
      cur.clear();
      if (e.empty()) continue;
      int64_t x;
      if (!parse_int(e, &x)) return false;
      out->push_back(x);
    } else {
      cur += c;
    }
  }
  return true;
}

// The TOML subset a container needs: `[table]`, `[[array of tables]]`, `key = value` with string,
// integer, float and integer-array values, `#` comments.  `on_table(name, is_array)` is called at
// every header, `on_kv(key, raw value)` for every pair under the current header.
template <class OnTable, class OnKv>
bool parse_toml(const char* p, const char* end, OnTable on_table, OnKv on_kv, std::string* err) {
  int lineno = 0;
  while (p < end) {
    const char* nl = static_cast<const char*>(memchr(p, '\n', (size_t)(end - p)));
    const char* le = nl ? nl : end;
    ++lineno;
    const std::string line = trim(strip_comment(std::string(p, le)));
    p = nl ? nl + 1 : end;
    if (line.empty()) continue;
    if (line.front() == '[') {
      const bool arr = line.size() >= 4 && line[1] == '[';
      if (line.back() != ']' || (arr && line[line.size() - 2] != ']')) {
        *err = "line " + std::to_string(lineno) + ": bad table header";
        return false;
      }
      on_table(trim(line.substr(arr ? 2 : 1, line.size() - (arr ? 4 : 2))), arr);
      continue;
    }
    const size_t eq = line.find('=');
    if (eq == std::string::npos) {
      *err = "line " + std::to_string(lineno) + ": expected key = value";
      return false;
    }
    on_kv(trim(line.substr(0, eq)), trim(line.substr(eq + 1)));
  }
  return true;
}

bool fail(ModelFile& m, const std::string& what) {
  m.err = what;
  return false;
}

bool open_model(const char* path, ModelFile& m) {
  m.fd = open(path, O_RDONLY);
  if (m.fd < 0) return fail(m, std::string("cannot open ") + path + ": " + strerror(errno));
  struct stat st;
  if (fstat(m.fd, &st) != 0 || st.st_size <= 0) return fail(m, "cannot stat the file, or it is empty");
  m.bytes = (size_t)st.st_size;
  void* map = mmap(nullptr, m.bytes, PROT_READ, MAP_PRIVATE, m.fd, 0);
  if (map == MAP_FAILED) return fail(m, std::string("mmap failed: ") + strerror(errno));
  m.base = static_cast<const char*>(map);
  const char* end = m.base + m.bytes;
  // rule 1: frontmatter until the first line that starts with ~~~
  const char* p = m.base;
  const char* fm_end = nullptr;
  while (p < end) {
    if (end - p >= 3 && p[0] == '~' && p[1] == '~' && p[2] == '~') { fm_end = p; break; }
    const char* nl = static_cast<const char*>(memchr(p, '\n', (size_t)(end - p)));
    if (!nl) break;
    p = nl + 1;
  }
  if (!fm_end) return fail(m, "no `~~~` delimiter: not a .cyb container");
  std::string table;
  std::string err;
  if (!parse_toml(m.base, fm_end,
                  [&](const std::string& name, bool arr) {
                    table = name;
                    if (arr && name == "files") m.files.emplace_back();
                  },
                  [&](const std::string& k, const std::string& v) {
                    if (table != "files" || m.files.empty()) return;
                    FileEntry& f = m.files.back();
                    if (k == "name") f.name = unquote(v);
                    else if (k == "format") f.format = unquote(v);
                    else if (k == "size") parse_int(v, &f.size);
                  },
                  &err))
    return fail(m, "frontmatter: " + err);
  if (m.files.empty()) return fail(m, "frontmatter lists no [[files]]");
  // rules 2 and 3: `~~~name` LF, then `size` bytes (binary) or up to the next `~~~` line / EOF (text),
  // in the order of the [[files]] array
  p = fm_end;
  for (FileEntry& f : m.files) {
    const std::string delim = "~~~" + f.name + "\n";
    if ((size_t)(end - p) < delim.size() || memcmp(p, delim.data(), delim.size()) != 0)
      return fail(m, "expected `~~~" + f.name + "` (files appear in frontmatter order, LF line ends)");
    p += delim.size();
    f.data = p;
    if (f.size >= 0) {
      if (f.size > end - p) return fail(m, "file `" + f.name + "`: size " + std::to_string(f.size) + " runs past the end of the container");
      f.len = f.size;
      p += f.size;
      if (p < end && *p == '\n') ++p;  // a writer may end the binary with LF before the next delimiter
    } else {
      const char* q = p;
      const char* stop = end;
      while (q < end) {
        if (end - q >= 3 && q[0] == '~' && q[1] == '~' && q[2] == '~') { stop = q; break; }
        const char* nl = static_cast<const char*>(memchr(q, '\n', (size_t)(end - q)));
        if (!nl) break;
        q = nl + 1;
      }
      f.len = stop - p;
      p = stop;
    }
  }
  auto find = [&](const char* name) -> const FileEntry* {
    for (const FileEntry& f : m.files)
      if (f.name == name) return &f;
    return nullptr;
  };
  const FileEntry* cfg = find("config");
  const FileEntry* idx = find("tensors");
  const FileEntry* wts = find("weights");
  if (!cfg || !idx || !wts) return fail(m, "a model container needs the files `config`, `tensors` and `weights`");
  if (wts->size < 0) return fail(m, "`weights` is binary: it needs `size` in the frontmatter");
  if (!parse_toml(cfg->data, cfg->data + cfg->len, [&](const std::string&, bool) {},
                  [&](const std::string& k, const std::string& v) { m.config[k] = v; }, &err))
    return fail(m, "config: " + err);
  bool bad = false;
  if (!parse_toml(idx->data, idx->data + idx->len,
                  [&](const std::string& name, bool arr) {
                    if (arr && name == "tensor") m.tensors.emplace_back();
                  },
                  [&](const std::string& k, const std::string& v) {
                    if (m.tensors.empty()) return;
                    Tensor& t = m.tensors.back();
                    if (k == "name") t.name = unquote(v);
                    else if (k == "dtype") t.dtype = unquote(v);
                    else if (k == "shape") bad |= !parse_int_array(v, &t.shape);
                    else if (k == "offset") bad |= !parse_int(v, &t.offset);
                    else if (k == "size") bad |= !parse_int(v, &t.size);
                  },
                  &err))
    return fail(m, "tensors: " + err);
  if (bad) return fail(m, "tensors: a shape, offset or size is not an integer");
  for (const Tensor& t : m.tensors) {
    if (t.name.empty() || t.shape.empty() || t.shape.size() > 2 || t.offset < 0 || t.size < 0)
      return fail(m, "tensor `" + t.name + "`: needs name, dtype, shape (1 or 2 dims), offset, size");
    int64_t n = 1;
    for (int64_t d : t.shape) {
      if (d <= 0) return fail(m, "tensor `" + t.name + "`: bad shape");
      n *= d;
    }
    int64_t want = -1;
    if (t.dtype == "F32") want = n * 4;
    else if (t.dtype == "F16" || t.dtype == "BF16") want = n * 2;
    else if (t.dtype == "Q4" || t.dtype == "Q4_0") {
      if (t.shape.size() != 2 || t.shape[1] % 32 != 0) return fail(m, "tensor `" + t.name + "`: Q4 needs [rows, cols] with cols % 32 == 0");
      want = n / 32 * 18;
    } else if (t.dtype == "Q8" || t.dtype == "Q8_0") {
      if (t.shape.size() != 2 || t.shape[1] % 32 != 0) return fail(m, "tensor `" + t.name + "`: Q8 needs [rows, cols] with cols % 32 == 0");
      want = n / 32 * 34;
    } else if (t.dtype == "Q4_K") {
      if (t.shape.size() != 2 || t.shape[1] % 256 != 0) return fail(m, "tensor `" + t.name + "`: Q4_K needs [rows, cols] with cols % 256 == 0");
      want = n / 256 * 144;
    } else {
      return fail(m, "tensor `" + t.name + "`: dtype `" + t.dtype + "` is not one of Q4, Q4_0, Q8, Q8_0, Q4_K, F32, F16, BF16");
    }
    if (t.size != want) return fail(m, "tensor `" + t.name + "`: size " + std::to_string(t.size) + " does not match its shape and dtype (" + std::to_string(want) + ")");
    if (t.offset + t.size > wts->len) return fail(m, "tensor `" + t.name + "`: runs past the end of `weights`");
  }
  return true;
}

bool cfg_int(const ModelFile& m, const char* key, int64_t* out) {
  auto it = m.config.find(key);
  return it != m.config.end() && parse_int(it->second, out);
}
bool cfg_float(const ModelFile& m, const char* key, float* out) {
  auto it = m.config.find(key);
  if (it == m.config.end()) return false;
  char* end = nullptr;
  const double v = strtod(it->second.c_str(), &end);
  if (end == it->second.c_str()) return false;
  *out = (float)v;
  return true;
}

bool model_cfg(ModelFile& m, qeng_model_cfg* c) {
  int64_t v;
  memset(c, 0, sizeof *c);
  struct { const char* key; int32_t* dst; } req[] = {
      {"num_hidden_layers", &c->layers}, {"hidden_size", &c->d_model}, {"intermediate_size", &c->ffn},
      {"num_attention_heads", &c->heads}, {"vocab_size", &c->vocab}};
  for (auto& r : req) {
    if (!cfg_int(m, r.key, &v) || v <= 0 || v > INT32_MAX) return fail(m, std::string("config: missing or bad `") + r.key + "`");
    *r.dst = (int32_t)v;
  }
  c->kv_heads = cfg_int(m, "num_key_value_heads", &v) ? (int32_t)v : c->heads;
  c->head_dim = cfg_int(m, "head_dim", &v) ? (int32_t)v : c->d_model / c->heads;
  if (!cfg_float(m, "rms_norm_eps", &c->rms_eps)) c->rms_eps = 1e-5f;
  if (!cfg_float(m, "rope_theta", &c->rope_base)) c->rope_base = 10000.f;
  if (!cfg_float(m, "attn_logit_softcapping", &c->attn_softcap)) c->attn_softcap = 0.f;
  c->sliding_window = cfg_int(m, "sliding_window", &v) && v > 0 && v <= INT32_MAX ? (int32_t)v : 0;
  if (!cfg_float(m, "final_logit_softcapping", &c->final_softcap)) c->final_softcap = 0.f;
  c->max_batch = 1;
  c->max_seq = 0;
  c->tp_rank = 0;
  c->tp_world = 1;
  return true;
}

float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float f16_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// a 1-D or 2-D tensor of any float type as f32
void to_f32(const Tensor& t, const char* data, std::vector<float>* out) {
  int64_t n = 1;
  for (int64_t d : t.shape) n *= d;
  out->resize((size_t)n);
  if (t.dtype == "F32") memcpy(out->data(), data, (size_t)n * 4);
  else if (t.dtype == "F16")
    for (int64_t i = 0; i < n; ++i) { uint16_t h; memcpy(&h, data + 2 * i, 2); (*out)[i] = f16_to_f32(h); }
  else
    for (int64_t i = 0; i < n; ++i) { uint16_t h; memcpy(&h, data + 2 * i, 2); (*out)[i] = bf16_to_f32(h); }
}

}  // namespace

extern "C" {

int32_t qeng_model_file_config(qeng_ctx* ctx, const char* path, qeng_model_cfg* out, int64_t* n_tensors) {
  if (!path || !out) return qeng_fail(ctx, QENG_ERR_ARG, "model_file_config: null argument");
  ModelFile m;
  if (!open_model(path, m) || !model_cfg(m, out)) return qeng_fail(ctx, QENG_ERR_ARG, "model file %s: %s", path, m.err.c_str());
  if (n_tensors) *n_tensors = (int64_t)m.tensors.size();
  return QENG_OK;
}

int32_t qeng_decoder_load_file(qeng_ctx* ctx, qeng_decoder* dec, const char* path) {
  if (!ctx || !dec || !path) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_file: null argument");
  ModelFile m;
  qeng_model_cfg fc;
  if (!open_model(path, m) || !model_cfg(m, &fc)) return qeng_fail(ctx, QENG_ERR_ARG, "model file %s: %s", path, m.err.c_str());
  qeng_model_cfg dc;
  int32_t rc = qeng_decoder_config(ctx, dec, &dc);
  if (rc != QENG_OK) return rc;
  if (fc.layers != dc.layers || fc.d_model != dc.d_model || fc.ffn != dc.ffn || fc.heads != dc.heads ||
      fc.kv_heads != dc.kv_heads || fc.head_dim != dc.head_dim || fc.vocab != dc.vocab || fc.attn_softcap != dc.attn_softcap || fc.final_softcap != dc.final_softcap ||
      fc.sliding_window != dc.sliding_window)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "model file %s: its config (layers %d, d %d, ffn %d, heads %d/%d, head_dim %d, vocab %d) differs from the decoder's",
                     path, fc.layers, fc.d_model, fc.ffn, fc.heads, fc.kv_heads, fc.head_dim, fc.vocab);
  const FileEntry* wts = nullptr;
  for (const FileEntry& f : m.files)
    if (f.name == "weights") wts = &f;
  std::map<std::string, const Tensor*> by_name;
  for (const Tensor& t : m.tensors) by_name[t.name] = &t;
  auto get = [&](const std::string& name) -> const Tensor* {
    auto it = by_name.find(name);
    return it == by_name.end() ? nullptr : it->second;
  };
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));

  // one linear weight [N, K]: Q4 blocks straight from the map, anything else through the device quantiser
  std::vector<uint8_t> q;
  std::vector<uint16_t> s;
  auto linear = [&](const std::string& name, int layer, int which, int64_t N, int64_t K) -> int32_t {
    const Tensor* t = get(name);
    if (!t) return qeng_fail(ctx, QENG_ERR_ARG, "model file %s: tensor `%s` is missing", path, name.c_str());
    if (t->shape.size() != 2 || t->shape[0] != N || t->shape[1] != K)
      return qeng_fail(ctx, QENG_ERR_SHAPE, "model file %s: tensor `%s` must be [%lld, %lld]", path, name.c_str(), (long long)N, (long long)K);
    const char* data = wts->data + t->offset;
    q.resize((size_t)N * K);
    s.resize((size_t)N * K / 32);
    if (t->dtype == "Q4" || t->dtype == "Q4_0") {
      // "Q4": byte i holds k = 2i (low nibble) and k = 2i + 1 (high); "Q4_0" (the order of the
      // published block of that name): byte i holds k = i (low) and k = i + 16 (high)
      const bool split = t->dtype == "Q4_0";
      const int64_t nb = N * K / 32;
      for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = reinterpret_cast<const uint8_t*>(data) + b * 18;
        memcpy(&s[(size_t)b], blk, 2);
        uint8_t* dst = &q[(size_t)b * 32];
        for (int i = 0; i < 16; ++i) {
          dst[split ? i : 2 * i] = blk[2 + i] & 15;
          dst[split ? i + 16 : 2 * i + 1] = blk[2 + i] >> 4;
        }
      }
    } else if (t->dtype == "Q4_K") {
      return qeng_decoder_load_matrix_q4k(ctx, dec, layer, which, reinterpret_cast<const uint8_t*>(data), N, K);
    } else if (t->dtype == "Q8" || t->dtype == "Q8_0") {
      const int64_t nb = N * K / 32;
      for (int64_t b = 0; b < nb; ++b) {
        const uint8_t* blk = reinterpret_cast<const uint8_t*>(data) + b * 34;
        memcpy(&s[(size_t)b], blk, 2);
        memcpy(&q[(size_t)b * 32], blk + 2, 32);
      }
      return qeng_decoder_load_matrix_q8(ctx, dec, layer, which, reinterpret_cast<const int8_t*>(q.data()), s.data(), N, K);
    } else {
      const int dt = t->dtype == "F32" ? QENG_F32 : (t->dtype == "F16" ? QENG_F16 : QENG_BF16);
      void* dev = nullptr;
      QENG_CUDA(ctx, cudaMalloc(&dev, (size_t)t->size));
      cudaError_t e = cudaMemcpy(dev, data, (size_t)t->size, cudaMemcpyHostToDevice);
      qeng_weight* w = nullptr;
      int32_t r = e == cudaSuccess ? qeng_weight_quantize_q4(ctx, dev, dt, N, K, K, &w, nullptr) : qeng_fail(ctx, QENG_ERR_CUDA, "upload of `%s`: %s", name.c_str(), cudaGetErrorString(e));
      if (r == QENG_OK) r = qeng_weight_unpack_q4(ctx, w, q.data(), s.data());
      qeng_weight_free(ctx, w);
      cudaFree(dev);
      if (r != QENG_OK) return r;
    }
    return qeng_decoder_load_matrix(ctx, dec, layer, which, q.data(), s.data(), N, K);
  };
  auto vec = [&](const std::string& name, int64_t n, std::vector<float>* out, bool required) -> int32_t {
    const Tensor* t = get(name);
    if (!t) return required ? qeng_fail(ctx, QENG_ERR_ARG, "model file %s: tensor `%s` is missing", path, name.c_str()) : 1;
    int64_t have = 1;
    for (int64_t d : t->shape) have *= d;
    if (t->dtype[0] == 'Q' || have != n) return qeng_fail(ctx, QENG_ERR_SHAPE, "model file %s: tensor `%s` must hold %lld floats", path, name.c_str(), (long long)n);
    to_f32(*t, wts->data + t->offset, out);
    return QENG_OK;
  };
  const int64_t dm = dc.d_model, nq = (int64_t)dc.heads * dc.head_dim, nkv = (int64_t)dc.kv_heads * dc.head_dim;
  std::vector<float> g;
  for (int l = 0; l < dc.layers; ++l) {
    const std::string pre = "model.layers." + std::to_string(l) + ".";
    struct { const char* name; int which; int64_t N, K; } mats[] = {
        {"self_attn.q_proj.weight", QENG_W_Q, nq, dm},   {"self_attn.k_proj.weight", QENG_W_K, nkv, dm},
        {"self_attn.v_proj.weight", QENG_W_V, nkv, dm},  {"self_attn.o_proj.weight", QENG_W_O, dm, nq},
        {"mlp.gate_proj.weight", QENG_W_GATE, dc.ffn, dm}, {"mlp.up_proj.weight", QENG_W_UP, dc.ffn, dm},
        {"mlp.down_proj.weight", QENG_W_DOWN, dm, dc.ffn}};
    for (auto& mt : mats) {
      rc = linear(pre + mt.name, l, mt.which, mt.N, mt.K);
      if (rc != QENG_OK) return rc;
    }
    rc = vec(pre + "input_layernorm.weight", dm, &g, true);
    if (rc == QENG_OK) rc = qeng_decoder_load_norm(ctx, dec, l, 0, g.data());
    if (rc == QENG_OK) rc = vec(pre + "post_attention_layernorm.weight", dm, &g, true);
    if (rc == QENG_OK) rc = qeng_decoder_load_norm(ctx, dec, l, 1, g.data());
    if (rc != QENG_OK) return rc;
    // optional per-head gains of q and k (the Qwen3 family)
    rc = vec(pre + "self_attn.q_norm.weight", dc.head_dim, &g, false);
    if (rc == QENG_OK) {
      rc = qeng_decoder_load_norm(ctx, dec, l, 2, g.data());
      if (rc == QENG_OK) rc = vec(pre + "self_attn.k_norm.weight", dc.head_dim, &g, true);
      if (rc == QENG_OK) rc = qeng_decoder_load_norm(ctx, dec, l, 3, g.data());
    } else if (rc == 1) {
      rc = QENG_OK;
    }
    if (rc != QENG_OK) return rc;
  }
  // embedding, LM head (tied to the embedding when absent) and the final norm
  auto table = [&](const std::string& name, std::vector<uint16_t>* out, bool required) -> int32_t {
    const Tensor* t = get(name);
    if (!t) return required ? qeng_fail(ctx, QENG_ERR_ARG, "model file %s: tensor `%s` is missing", path, name.c_str()) : 1;
    if (t->dtype[0] == 'Q' || t->shape.size() != 2 || t->shape[0] != dc.vocab || t->shape[1] != dm)
      return qeng_fail(ctx, QENG_ERR_SHAPE, "model file %s: tensor `%s` must be a float matrix [%d, %lld]", path, name.c_str(), dc.vocab, (long long)dm);
    const char* data = wts->data + t->offset;
    const size_t n = (size_t)dc.vocab * dm;
    out->resize(n);
    if (t->dtype == "BF16") memcpy(out->data(), data, n * 2);
    else {
      std::vector<float> f;
      to_f32(*t, data, &f);
      for (size_t i = 0; i < n; ++i) (*out)[i] = f32_to_bf16(f[i]);
    }
    return QENG_OK;
  };
  std::vector<uint16_t> emb, head;
  rc = table("model.embed_tokens.weight", &emb, true);
  if (rc != QENG_OK) return rc;
  rc = table("lm_head.weight", &head, false);
  if (rc == 1) { head = emb; rc = QENG_OK; }
  if (rc != QENG_OK) return rc;
  rc = vec("model.norm.weight", dm, &g, true);
  if (rc != QENG_OK) return rc;
  return qeng_decoder_load_head(ctx, dec, emb.data(), head.data(), g.data());
}

}  // extern "C"
