// safetensors store + config.json reader. Plain C++ over POSIX mmap; see checkpoint.h.
#include "checkpoint.h"
#include <stdint.h>

#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <set>

namespace ckpt {

size_t dtype_size(int dt) {
  switch (dt) {
    case F32: case I32: return 4;
    case F16: case BF16: return 2;
    case I64: return 8;
    default: return 1;
  }
}

// ---- JSON -------------------------------------------------------------------------------
namespace {

struct Parser {
  const char* p;
  const char* end;
  std::string* err;
  int depth = 0;

  bool fail(const char* what) {
    if (err && err->empty()) *err = std::string("json: ") + what;
    return false;
  }
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p; }

  static void utf8(uint32_t cp, std::string* s) {
    if (cp < 0x80) s->push_back((char)cp);
    else if (cp < 0x800) { s->push_back((char)(0xC0 | (cp >> 6))); s->push_back((char)(0x80 | (cp & 63))); }
    else if (cp < 0x10000) { s->push_back((char)(0xE0 | (cp >> 12))); s->push_back((char)(0x80 | ((cp >> 6) & 63))); s->push_back((char)(0x80 | (cp & 63))); }
    else { s->push_back((char)(0xF0 | (cp >> 18))); s->push_back((char)(0x80 | ((cp >> 12) & 63))); s->push_back((char)(0x80 | ((cp >> 6) & 63))); s->push_back((char)(0x80 | (cp & 63))); }
  }
  bool hex4(uint32_t* v) {
    if (end - p < 4) return fail("short \\u escape");
    uint32_t x = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p++;
      x <<= 4;
      if (c >= '0' && c <= '9') x |= (uint32_t)(c - '0');
      else if (c >= 'a' && c <= 'f') x |= (uint32_t)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') x |= (uint32_t)(c - 'A' + 10);
      else return fail("bad \\u escape");
    }
    *v = x;
    return true;
  }
  bool string(std::string* out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    out->clear();
    while (p < end) {
      const char c = *p++;
      if (c == '"') return true;
      if (c != '\\') { out->push_back(c); continue; }
      if (p >= end) break;
      const char e = *p++;
      switch (e) {
        case '"': out->push_back('"'); break;
        case '\\': out->push_back('\\'); break;
        case '/': out->push_back('/'); break;
        case 'b': out->push_back('\b'); break;
        case 'f': out->push_back('\f'); break;
        case 'n': out->push_back('\n'); break;
        case 'r': out->push_back('\r'); break;
        case 't': out->push_back('\t'); break;
        case 'u': {
          uint32_t cp;
          if (!hex4(&cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
            p += 2;
            uint32_t lo;
            if (!hex4(&lo)) return false;
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            else return fail("unpaired surrogate");
          }
          utf8(cp, out);
          break;
        }
        default: return fail("bad escape");
      }
    }
    return fail("unterminated string");
  }
  bool value(Json* out) {
    if (++depth > 64) return fail("nesting too deep");
    ws();
    if (p >= end) return fail("unexpected end");
    bool ok = true;
    const char c = *p;
    if (c == '{') {
      ++p;
      out->kind = Json::Object;
      ws();
      if (p < end && *p == '}') { ++p; }
      else {
        for (;;) {
          ws();
          std::string key;
          if (!string(&key)) { ok = false; break; }
          ws();
          if (p >= end || *p != ':') { ok = fail("expected ':'"); break; }
          ++p;
          out->members.emplace_back(std::move(key), Json());
          if (!value(&out->members.back().second)) { ok = false; break; }
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == '}') { ++p; break; }
          ok = fail("expected ',' or '}'");
          break;
        }
      }
    } else if (c == '[') {
      ++p;
      out->kind = Json::Array;
      ws();
      if (p < end && *p == ']') { ++p; }
      else {
        for (;;) {
          out->items.emplace_back();
          if (!value(&out->items.back())) { ok = false; break; }
          ws();
          if (p < end && *p == ',') { ++p; continue; }
          if (p < end && *p == ']') { ++p; break; }
          ok = fail("expected ',' or ']'");
          break;
        }
      }
    } else if (c == '"') {
      out->kind = Json::String;
      ok = string(&out->text);
    } else if (c == 't' && end - p >= 4 && !memcmp(p, "true", 4)) {
      out->kind = Json::Bool; out->b = true; p += 4;
    } else if (c == 'f' && end - p >= 5 && !memcmp(p, "false", 5)) {
      out->kind = Json::Bool; out->b = false; p += 5;
    } else if (c == 'n' && end - p >= 4 && !memcmp(p, "null", 4)) {
      out->kind = Json::Null; p += 4;
    } else if (c == '-' || (c >= '0' && c <= '9')) {
      const char* s = p;
      ++p;
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) ++p;
      out->kind = Json::Number;
      out->text.assign(s, p);
    } else {
      ok = fail("unexpected character");
    }
    --depth;
    return ok;
  }
};

}  // namespace

bool Json::parse(const char* p, size_t n, Json* out, std::string* err) {
  Parser ps{p, p + n, err};
  if (!ps.value(out)) return false;
  ps.ws();
  if (ps.p != ps.end) return ps.fail("trailing characters");
  return true;
}
const Json* Json::get(const char* key) const {
  if (kind != Object) return nullptr;
  const Json* hit = nullptr;
  for (const auto& m : members) if (m.first == key) hit = &m.second;  // last duplicate wins, like serde_json
  return hit;
}
bool Json::as_u64(uint64_t* out) const {
  if (kind != Number || text.empty()) return false;
  uint64_t v = 0;
  for (char c : text) {
    if (c < '0' || c > '9') return false;
    if (v > (UINT64_MAX - (uint64_t)(c - '0')) / 10) return false;
    v = v * 10 + (uint64_t)(c - '0');
  }
  *out = v;
  return true;
}
bool Json::as_f64(double* out) const {
  if (kind != Number) return false;
  char* e = nullptr;
  const double v = strtod(text.c_str(), &e);
  if (!e || *e) return false;
  *out = v;
  return true;
}

// ---- Store --------------------------------------------------------------------------------
namespace {
bool read_file(const std::string& path, std::string* out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  char buf[65536];
  size_t n;
  out->clear();
  while ((n = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, n);
  fclose(f);
  return true;
}
bool exists(const std::string& path) { struct stat st; return stat(path.c_str(), &st) == 0; }
bool is_dir(const std::string& path) { struct stat st; return stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }
bool parse_dtype(const std::string& s, int* dt) {
  if (s == "F32") *dt = F32;
  else if (s == "F16") *dt = F16;
  else if (s == "BF16") *dt = BF16;
  else if (s == "I32") *dt = I32;
  else if (s == "I64") *dt = I64;
  else if (s == "U8" || s == "BOOL") *dt = U8;
  else if (s == "F8_E4M3" || s == "F8_E4M3FN") *dt = F8E4M3;
  else return false;
  return true;
}
}  // namespace

Store::~Store() {
  for (Shard& s : shards_) {
    if (s.base) munmap(const_cast<uint8_t*>(s.base), s.bytes);
    if (s.fd >= 0) ::close(s.fd);
  }
}

bool Store::file_of(const void* p, int* fd, size_t* offset) const {
  const uint8_t* q = (const uint8_t*)p;
  for (const Shard& s : shards_) {
    if (s.fd >= 0 && q >= s.base && q < s.base + s.bytes) {
      *fd = s.fd;
      *offset = (size_t)(q - s.base);
      return true;
    }
  }
  return false;
}

bool Store::map_file(const std::string& path, std::string* err) {
  const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) { *err = "opening " + path + ": " + strerror(errno); return false; }
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) { ::close(fd); *err = path + ": not a safetensors file"; return false; }
  const size_t bytes = (size_t)st.st_size;
  void* m = mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { ::close(fd); *err = "mapping " + path + ": " + strerror(errno); return false; }
  Shard sh;
  sh.path = path;
  sh.base = (const uint8_t*)m;
  sh.bytes = bytes;
  sh.fd = fd;
  const int shard = (int)shards_.size();
  shards_.push_back(sh);  // owned from here on: the destructor unmaps it whatever happens below
  uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | sh.base[i];
  if (hlen > bytes - 8) { *err = path + ": header length exceeds the file"; return false; }
  Json header;
  std::string jerr;
  if (!Json::parse((const char*)sh.base + 8, (size_t)hlen, &header, &jerr) || header.kind != Json::Object) {
    *err = "parsing header of " + path + (jerr.empty() ? "" : ": " + jerr);
    return false;
  }
  const size_t data_start = 8 + (size_t)hlen;
  for (const auto& m2 : header.members) {
    if (m2.first == "__metadata__") continue;
    const Json& t = m2.second;
    const Json* jd = t.get("dtype");
    const Json* js = t.get("shape");
    const Json* jo = t.get("data_offsets");
    Tensor ti;
    if (!jd || jd->kind != Json::String) { *err = path + ": " + m2.first + ": dtype"; return false; }
    if (!parse_dtype(jd->text, &ti.dtype)) { *err = "unsupported safetensors dtype " + jd->text; return false; }
    if (!js || js->kind != Json::Array) { *err = path + ": " + m2.first + ": shape"; return false; }
    // every dimension an unsigned integer, and the element count (times the element size) without wrap-around: a shape that
    // overflows could otherwise still "match" its byte range
    uint64_t elems = 1;
    bool shape_ok = true;
    for (const Json& d : js->items) {
      uint64_t v = 0;
      if (!d.as_u64(&v)) { shape_ok = false; break; }
      if (v != 0 && elems > UINT64_MAX / v) { shape_ok = false; break; }
      elems *= v;
      ti.shape.push_back((size_t)v);
    }
    if (!shape_ok || (elems != 0 && dtype_size(ti.dtype) > UINT64_MAX / elems)) {
      *err = path + ": " + m2.first + ": shape is not a list of unsigned integers whose product fits 64 bits";
      return false;
    }
    uint64_t o0 = 0, o1 = 0;
    if (!jo || jo->kind != Json::Array || jo->items.size() != 2 || !jo->items[0].as_u64(&o0) || !jo->items[1].as_u64(&o1) || o1 < o0 ||
        o1 > bytes - data_start) {
      *err = path + ": " + m2.first + ": data_offsets";
      return false;
    }
    if (o1 - o0 != ti.count() * dtype_size(ti.dtype)) { *err = path + ": " + m2.first + ": byte range does not match dtype and shape"; return false; }
    ti.shard = shard;
    ti.start = data_start + (size_t)o0;
    ti.end = data_start + (size_t)o1;
    auto it = map_.find(m2.first);
    if (it == map_.end()) { map_.emplace(m2.first, ti); names_.push_back(m2.first); }
    else it->second = ti;
  }
  return true;
}

bool Store::open(const std::string& path, std::string* err) {
  std::vector<std::string> files;
  if (!is_dir(path)) {
    files.push_back(path);
  } else {
    const std::string index = path + "/model.safetensors.index.json";
    const std::string single = path + "/model.safetensors";
    if (exists(single) && !exists(index)) {
      files.push_back(single);
    } else if (exists(index)) {
      std::string raw, jerr;
      Json v;
      if (!read_file(index, &raw) || !Json::parse(raw.data(), raw.size(), &v, &jerr)) { *err = "parsing " + index + (jerr.empty() ? "" : ": " + jerr); return false; }
      const Json* wm = v.get("weight_map");
      if (!wm || wm->kind != Json::Object) { *err = "index.json has no weight_map"; return false; }
      std::set<std::string> seen;
      for (const auto& m : wm->members) if (m.second.kind == Json::String) seen.insert(m.second.text);
      for (const std::string& f : seen) files.push_back(path + "/" + f);
    } else {
      DIR* d = opendir(path.c_str());
      if (!d) { *err = "reading " + path + ": " + strerror(errno); return false; }
      while (dirent* ent = readdir(d)) {
        const std::string n = ent->d_name;
        const std::string ext = ".safetensors";
        if (n.size() > ext.size() && n.compare(n.size() - ext.size(), ext.size(), ext) == 0) files.push_back(path + "/" + n);
      }
      closedir(d);
      std::sort(files.begin(), files.end());
    }
  }
  if (files.empty()) { *err = "no safetensors files in " + path; return false; }
  for (const std::string& f : files) if (!map_file(f, err)) return false;
  return true;
}

const Tensor* Store::info(const std::string& name) const {
  auto it = map_.find(name);
  return it == map_.end() ? nullptr : &it->second;
}

// ---- config.json ----------------------------------------------------------------------------
namespace {
bool get_usize(const Json& c, const char* key, uint64_t* out) {
  const Json* v = c.get(key);
  return v && v->as_u64(out);
}
uint64_t usize_or(const Json& c, const char* key, uint64_t dflt) {
  uint64_t v;
  return get_usize(c, key, &v) ? v : dflt;
}
const char* str_of(const Json* v) { return v && v->kind == Json::String ? v->text.c_str() : nullptr; }
}  // namespace

bool config_from_dir(const std::string& dir, dcd_model_config* out, std::string* err) {
  std::string raw, jerr;
  Json v;
  if (!read_file(dir + "/config.json", &raw)) { *err = "reading config.json"; return false; }
  if (!Json::parse(raw.data(), raw.size(), &v, &jerr)) { *err = "parsing config.json: " + jerr; return false; }
  const Json* tc = v.get("text_config");
  const Json& c = tc ? *tc : v;  // tolerant of text_config nesting
  memset(out, 0, sizeof *out);
  uint64_t layers, heads, hidden, inter, vocab;
  if (!get_usize(c, "num_hidden_layers", &layers)) { *err = "config missing num_hidden_layers"; return false; }
  if (!get_usize(c, "num_attention_heads", &heads)) { *err = "config missing num_attention_heads"; return false; }
  const uint64_t kv = usize_or(c, "num_key_value_heads", heads);
  if (!get_usize(c, "hidden_size", &hidden)) { *err = "config missing hidden_size"; return false; }
  const uint64_t hd = usize_or(c, "head_dim", heads ? hidden / heads : 0);
  if (!get_usize(c, "intermediate_size", &inter)) { *err = "config missing intermediate_size"; return false; }
  if (!get_usize(c, "vocab_size", &vocab)) { *err = "config missing vocab_size"; return false; }
  if (layers == 0 || layers > 256) { *err = "num_hidden_layers outside 1..256"; return false; }
  // everything below is narrowed to int32 and multiplied into buffer sizes
  {
    const struct { const char* name; uint64_t v, lo, hi; } lim[] = {
        {"hidden_size", hidden, 1, 1u << 20},          {"num_attention_heads", heads, 1, 1u << 12}, {"num_key_value_heads", kv, 1, 1u << 12},
        {"head_dim", hd, 1, 1u << 12},                 {"intermediate_size", inter, 1, 1u << 22},   {"vocab_size", vocab, 1, 1u << 26},
        {"linear_num_key_heads", usize_or(c, "linear_num_key_heads", 16), 1, 1u << 12},
        {"linear_num_value_heads", usize_or(c, "linear_num_value_heads", 48), 1, 1u << 12},
        {"linear_key_head_dim", usize_or(c, "linear_key_head_dim", 128), 1, 1u << 12},
        {"linear_value_head_dim", usize_or(c, "linear_value_head_dim", 128), 1, 1u << 12}};
    for (const auto& l : lim)
      if (l.v < l.lo || l.v > l.hi) { *err = std::string("config ") + l.name + " outside " + std::to_string(l.lo) + ".." + std::to_string(l.hi); return false; }
    if (heads % kv != 0) { *err = "config num_attention_heads is not a multiple of num_key_value_heads"; return false; }
  }
  double eps = 1e-6;
  if (const Json* e = c.get("rms_norm_eps")) e->as_f64(&eps);
  const Json* lt = c.get("layer_types");
  for (uint64_t i = 0; i < layers; ++i) {
    const char* s = lt && lt->kind == Json::Array && i < lt->items.size() ? str_of(&lt->items[i]) : nullptr;
    out->layer_is_full[i] = (s && !strcmp(s, "linear_attention")) ? 0 : 1;  // anything else is full attention
  }
  const Json* rope = c.get("rope_parameters");
  double theta = 10000000.0, prf = 1.0;
  bool have_prf = false;
  if (rope) {
    if (const Json* t = rope->get("rope_theta")) t->as_f64(&theta);
    if (const Json* t = rope->get("partial_rotary_factor")) have_prf = t->as_f64(&prf);
  }
  if (!have_prf) if (const Json* t = c.get("partial_rotary_factor")) t->as_f64(&prf);

  // The prompt attention is declared in decision_config.json or config.json; both present must agree,
  // and only prefix_bidir is served.
  const char* config_mode = str_of(v.get("attention_mode"));
  std::string decision_mode_s;
  const char* decision_mode = nullptr;
  {
    const std::string dp = dir + "/decision_config.json";
    std::string draw;
    if (exists(dp)) {
      Json d;
      if (!read_file(dp, &draw) || !Json::parse(draw.data(), draw.size(), &d, &jerr)) { *err = "parsing " + dp + ": " + jerr; return false; }
      if (const char* s = str_of(d.get("attention_mode"))) { decision_mode_s = s; decision_mode = decision_mode_s.c_str(); }
    }
  }
  if (config_mode && decision_mode && strcmp(config_mode, decision_mode)) {
    *err = std::string("config.json attention_mode \"") + config_mode + "\" conflicts with decision_config.json \"" + decision_mode + "\"";
    return false;
  }
  const char* mode = config_mode ? config_mode : decision_mode;
  if (!mode) { *err = dir + " has no attention_mode; d3-turbo requires prefix_bidir"; return false; }
  if (strcmp(mode, "prefix_bidir")) { *err = std::string("unsupported attention_mode \"") + mode + "\"; only d3-turbo prefix_bidir is served"; return false; }

  out->num_layers = (int32_t)layers;
  out->hidden = (int32_t)hidden;
  out->heads = (int32_t)heads;
  out->kv_heads = (int32_t)kv;
  out->head_dim = (int32_t)hd;
  out->rotary_dim = (int32_t)((size_t)((float)hd * (float)prf) & ~(size_t)1);
  out->rope_theta = (float)theta;
  out->gdn_k_heads = (int32_t)usize_or(c, "linear_num_key_heads", 16);
  out->gdn_v_heads = (int32_t)usize_or(c, "linear_num_value_heads", 48);
  out->gdn_dk = (int32_t)usize_or(c, "linear_key_head_dim", 128);
  out->gdn_dv = (int32_t)usize_or(c, "linear_value_head_dim", 128);
  out->conv_kernel = 4;
  out->intermediate = (int32_t)inter;
  out->vocab = (int32_t)vocab;
  out->readout_rows = 0;
  out->rms_eps = (float)eps;
  out->dtype = 1;
  return true;
}

}  // namespace ckpt
