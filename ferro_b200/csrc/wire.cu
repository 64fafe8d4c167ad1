// Checkpoint wire format either side of the device path: safetensors images
// written from, and read into, device buffers.
//
// ferro serialises a state dict with to_safetensors_bytes
// (crates/ferro-core/src/safetensors.rs:36-94) and the optimizer state as flat
// arrays named "m.i", "v.i", "t.i" per parameter (Adam::snapshot,
// crates/ferro-core/src/optim.rs:828-847; "velocity.i" for SGD), after bringing
// every buffer to the host as a Vec and re-encoding it value by value.  Here
// the image is laid out once on the host (header text only) and every tensor's
// bytes go straight from device memory to their place in the caller's host
// image - one asynchronous copy per tensor on the caller's stream, into
// pinned memory if the caller pinned it - and back the same way on load.  The
// bytes are the ones ferro writes: 8-byte little-endian header length, the
// JSON header with entries in the order given, padded with spaces to a
// multiple of 8, then the little-endian tensor data, so files travel between
// the two implementations and any other safetensors reader.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace fb {

static const char* dtype_tag(int dt) { return dt == FB_ST_F32 ? "F32" : dt == FB_ST_I64 ? "I64" : nullptr; }
static uint64_t dtype_size(int dt) { return dt == FB_ST_F32 ? 4 : 8; }

// safetensors.rs:245-256
static void escape(const char* s, std::string* out) {
  for (const unsigned char* p = reinterpret_cast<const unsigned char*>(s); *p; ++p) {
    if (*p == '"') *out += "\\\"";
    else if (*p == '\\') *out += "\\\\";
    else if (*p < 0x20) {
      char buf[8];
      snprintf(buf, sizeof(buf), "\\u%04x", (unsigned)*p);
      *out += buf;
    } else {
      *out += (char)*p;
    }
  }
}

static int build_header(const char* name, const fb_st_entry* e, int n, std::string* header, std::vector<uint64_t>* offs) {
  if (n < 0 || (n && !e)) return fail(FB_ERR_INVALID_ARG, "%s: bad entry list", name);
  *header = "{";
  offs->assign(1, 0);
  uint64_t pos = 0;
  for (int i = 0; i < n; ++i) {
    if (!e[i].name) return fail(FB_ERR_INVALID_ARG, "%s: entry %d has no name", name, i);
    for (int j = 0; j < i; ++j)
      if (!strcmp(e[i].name, e[j].name)) return fail(FB_ERR_INVALID_ARG, "%s: duplicate tensor name \"%s\"", name, e[i].name);
    if (!dtype_tag(e[i].dtype)) return fail(FB_ERR_UNSUPPORTED, "%s: entry %d: dtype %d is not F32 or I64", name, i, e[i].dtype);
    if (e[i].rank < 0 || e[i].rank > FB_MAX_RANK) return fail(FB_ERR_INVALID_SHAPE, "%s: entry %d: rank %d", name, i, e[i].rank);
    uint64_t numel = 1;
    for (int d = 0; d < e[i].rank; ++d)
      if (mul_overflows(numel, e[i].shape[d], &numel) || numel > (UINT64_MAX >> 4))
        return fail(FB_ERR_INVALID_SHAPE, "%s: entry %d: shape overflows", name, i);
    const uint64_t end = pos + numel * dtype_size(e[i].dtype);
    if (i) *header += ",";
    *header += "\"";
    escape(e[i].name, header);
    *header += "\":{\"dtype\":\"";
    *header += dtype_tag(e[i].dtype);
    *header += "\",\"shape\":[";
    for (int d = 0; d < e[i].rank; ++d) {
      if (d) *header += ",";
      *header += std::to_string(e[i].shape[d]);
    }
    *header += "],\"data_offsets\":[" + std::to_string(pos) + "," + std::to_string(end) + "]}";
    pos = end;
    offs->push_back(pos);
  }
  *header += "}";
  while ((8 + header->size()) % 8 != 0) *header += ' ';  // safetensors.rs:84-88
  return FB_OK;
}

// ---- the subset of JSON a safetensors header holds (safetensors.rs:258-450) ----
struct Cursor {
  const char* p;
  const char* end;
  std::string err;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) { ++p; return true; }
    return false;
  }
  bool fail_at(const char* what) {
    if (err.empty()) err = what;
    return false;
  }
  bool str(std::string* out) {
    ws();
    if (p >= end || *p != '"') return fail_at("expected a string");
    ++p;
    out->clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail_at("unterminated escape");
        switch (*p) {
          case '"': *out += '"'; break;
          case '\\': *out += '\\'; break;
          case '/': *out += '/'; break;
          case 'n': *out += '\n'; break;
          case 't': *out += '\t'; break;
          case 'r': *out += '\r'; break;
          case 'b': *out += '\b'; break;
          case 'f': *out += '\f'; break;
          case 'u': {
            if (end - p < 5) return fail_at("short \\u escape");
            unsigned v = 0;
            for (int k = 1; k <= 4; ++k) {
              const char c = p[k];
              v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 99);
              if (v > 0xffff) return fail_at("bad \\u escape");
            }
            p += 4;
            if (v < 0x80) *out += (char)v;
            else if (v < 0x800) { *out += (char)(0xc0 | (v >> 6)); *out += (char)(0x80 | (v & 0x3f)); }
            else { *out += (char)(0xe0 | (v >> 12)); *out += (char)(0x80 | ((v >> 6) & 0x3f)); *out += (char)(0x80 | (v & 0x3f)); }
            break;
          }
          default: return fail_at("unknown escape");
        }
        ++p;
      } else {
        *out += *p++;
      }
    }
    if (p >= end) return fail_at("unterminated string");
    ++p;
    return true;
  }
  bool num(uint64_t* out) {
    ws();
    if (p >= end || *p < '0' || *p > '9') return fail_at("expected an unsigned integer");
    uint64_t v = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (v > (UINT64_MAX - 9) / 10) return fail_at("integer overflows");
      v = v * 10 + (uint64_t)(*p++ - '0');
    }
    *out = v;
    return true;
  }
  // Skips any value (used for __metadata__ and unknown fields).
  bool skip() {
    ws();
    if (p >= end) return fail_at("unexpected end");
    if (*p == '"') { std::string s; return str(&s); }
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool obj = *p == '{';
      ++p;
      if (eat(close)) return true;
      do {
        if (obj) {
          std::string k;
          if (!str(&k) || !eat(':')) return fail_at("expected a key and ':'");
        }
        if (!skip()) return false;
      } while (eat(','));
      return eat(close) ? true : fail_at("expected a closing bracket");
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ') ++p;  // number / true / false / null
    return true;
  }
};

struct Parsed {
  std::string name;
  int dtype;
  std::vector<uint64_t> shape;
  uint64_t begin, end;
};

static int parse_image(const char* name, const void* image, uint64_t bytes, std::vector<Parsed>* out, uint64_t* data_start) {
  if (!image) return fail(FB_ERR_INVALID_ARG, "%s: null image", name);
  if (bytes < 8) return fail(FB_ERR_FORMAT, "%s: shorter than the 8-byte header length", name);
  uint64_t hlen;
  memcpy(&hlen, image, 8);  // little-endian hosts only (x86-64, aarch64)
  if (hlen > bytes - 8) return fail(FB_ERR_FORMAT, "%s: header length %llu exceeds file size %llu", name, (unsigned long long)hlen, (unsigned long long)bytes);
  *data_start = 8 + hlen;
  const uint64_t data_len = bytes - *data_start;
  Cursor c{static_cast<const char*>(image) + 8, static_cast<const char*>(image) + 8 + hlen, ""};
  if (!c.eat('{')) return fail(FB_ERR_FORMAT, "%s: header is not a JSON object", name);
  if (!c.eat('}')) {
    do {
      Parsed t;
      if (!c.str(&t.name) || !c.eat(':')) return fail(FB_ERR_FORMAT, "%s: bad header: %s", name, c.err.c_str());
      if (t.name == "__metadata__") {
        if (!c.skip()) return fail(FB_ERR_FORMAT, "%s: bad header: %s", name, c.err.c_str());
        continue;
      }
      if (!c.eat('{')) return fail(FB_ERR_FORMAT, "%s: entry \"%s\" is not an object", name, t.name.c_str());
      bool has_dtype = false, has_shape = false, has_offsets = false;
      std::string dtype;
      if (!c.eat('}')) {
        do {
          std::string key;
          if (!c.str(&key) || !c.eat(':')) return fail(FB_ERR_FORMAT, "%s: bad header: %s", name, c.err.c_str());
          if (key == "dtype") {
            if (!c.str(&dtype)) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": dtype is not a string", name, t.name.c_str());
            has_dtype = true;
          } else if (key == "shape" || key == "data_offsets") {
            std::vector<uint64_t> v;
            if (!c.eat('[')) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": %s is not an array", name, t.name.c_str(), key.c_str());
            if (!c.eat(']')) {
              do {
                uint64_t x;
                if (!c.num(&x)) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": %s", name, t.name.c_str(), c.err.c_str());
                v.push_back(x);
              } while (c.eat(','));
              if (!c.eat(']')) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": unterminated array", name, t.name.c_str());
            }
            if (key == "shape") { t.shape = v; has_shape = true; }
            else {
              if (v.size() != 2) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": data_offsets needs two numbers", name, t.name.c_str());
              t.begin = v[0];
              t.end = v[1];
              has_offsets = true;
            }
          } else if (!c.skip()) {
            return fail(FB_ERR_FORMAT, "%s: bad header: %s", name, c.err.c_str());
          }
        } while (c.eat(','));
        if (!c.eat('}')) return fail(FB_ERR_FORMAT, "%s: entry \"%s\": unterminated object", name, t.name.c_str());
      }
      if (!has_dtype || !has_shape || !has_offsets)
        return fail(FB_ERR_FORMAT, "%s: entry \"%s\" lacks dtype, shape or data_offsets", name, t.name.c_str());
      t.dtype = dtype == "F32" ? FB_ST_F32 : dtype == "I64" ? FB_ST_I64 : -1;
      uint64_t numel = 1;
      for (uint64_t d : t.shape)
        if (mul_overflows(numel, d, &numel) || numel > (UINT64_MAX >> 4))
          return fail(FB_ERR_FORMAT, "%s: entry \"%s\": shape overflows", name, t.name.c_str());
      if (t.begin > t.end || t.end > data_len)
        return fail(FB_ERR_FORMAT, "%s: entry \"%s\": data_offsets outside the data section", name, t.name.c_str());
      if (t.dtype >= 0 && t.end - t.begin != numel * dtype_size(t.dtype))
        return fail(FB_ERR_FORMAT, "%s: entry \"%s\": %llu bytes for %llu elements", name, t.name.c_str(),
                    (unsigned long long)(t.end - t.begin), (unsigned long long)numel);
      out->push_back(t);
    } while (c.eat(','));
    if (!c.eat('}')) return fail(FB_ERR_FORMAT, "%s: header object is not closed", name);
  }
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

uint64_t fb_safetensors_image_bytes(const fb_st_entry* entries, int n, uint64_t* data_offsets) {
  std::string header;
  std::vector<uint64_t> offs;
  if (build_header("fb_safetensors_image_bytes", entries, n, &header, &offs)) return 0;
  if (data_offsets)
    for (size_t i = 0; i < offs.size(); ++i) data_offsets[i] = 8 + header.size() + offs[i];
  return 8 + header.size() + offs.back();
}

int fb_safetensors_write(fb_stream_t stream, const fb_st_entry* entries, int n, const void* const* sources,
                         int sources_on_device, void* image, uint64_t image_bytes) {
  const char* name = "fb_safetensors_write";
  std::string header;
  std::vector<uint64_t> offs;
  if (int rc = build_header(name, entries, n, &header, &offs)) return rc;
  const uint64_t need = 8 + header.size() + offs.back();
  if (!image || image_bytes < need) return fail(FB_ERR_WORKSPACE, "%s: the image needs %llu bytes", name, (unsigned long long)need);
  for (int i = 0; i < n; ++i)
    if (offs[i + 1] > offs[i] && (!sources || !sources[i])) return fail(FB_ERR_INVALID_ARG, "%s: entry %d has no data", name, i);
  char* out = static_cast<char*>(image);
  const uint64_t hlen = header.size();
  memcpy(out, &hlen, 8);
  memcpy(out + 8, header.data(), header.size());
  char* data = out + 8 + header.size();
  for (int i = 0; i < n; ++i) {
    const uint64_t len = offs[i + 1] - offs[i];
    if (!len) continue;
    if (sources_on_device) FB_CUDA(cudaMemcpyAsync(data + offs[i], sources[i], len, cudaMemcpyDeviceToHost, stream));
    else memcpy(data + offs[i], sources[i], len);
  }
  return FB_OK;
}

int fb_safetensors_count(const void* image, uint64_t image_bytes) {
  std::vector<Parsed> v;
  uint64_t ds;
  if (parse_image("fb_safetensors_count", image, image_bytes, &v, &ds)) return -1;
  return (int)v.size();
}

int fb_safetensors_entry(const void* image, uint64_t image_bytes, int index, char* name_out, uint64_t name_cap,
                         fb_st_entry* entry_out, uint64_t* data_begin, uint64_t* data_end) {
  const char* fn = "fb_safetensors_entry";
  std::vector<Parsed> v;
  uint64_t ds;
  if (int rc = parse_image(fn, image, image_bytes, &v, &ds)) return rc;
  if (index < 0 || index >= (int)v.size()) return fail(FB_ERR_INVALID_ARG, "%s: index %d of %d", fn, index, (int)v.size());
  const Parsed& t = v[index];
  if (name_out) {
    if (t.name.size() + 1 > name_cap) return fail(FB_ERR_WORKSPACE, "%s: the name needs %llu bytes", fn, (unsigned long long)t.name.size() + 1);
    memcpy(name_out, t.name.c_str(), t.name.size() + 1);
  }
  if (entry_out) {
    if (t.shape.size() > FB_MAX_RANK) return fail(FB_ERR_UNSUPPORTED, "%s: rank %d", fn, (int)t.shape.size());
    entry_out->name = nullptr;
    entry_out->dtype = t.dtype;
    entry_out->rank = (int)t.shape.size();
    for (size_t d = 0; d < t.shape.size(); ++d) entry_out->shape[d] = t.shape[d];
  }
  if (data_begin) *data_begin = ds + t.begin;
  if (data_end) *data_end = ds + t.end;
  return FB_OK;
}

int fb_safetensors_read(fb_stream_t stream, const void* image, uint64_t image_bytes, const char* tensor_name,
                        int dtype, uint64_t numel, void* dst, int dst_on_device) {
  const char* fn = "fb_safetensors_read";
  if (!tensor_name) return fail(FB_ERR_INVALID_ARG, "%s: null name", fn);
  std::vector<Parsed> v;
  uint64_t ds;
  if (int rc = parse_image(fn, image, image_bytes, &v, &ds)) return rc;
  for (const Parsed& t : v) {
    if (t.name != tensor_name) continue;
    if (t.dtype != dtype) return fail(FB_ERR_FORMAT, "%s: \"%s\" is not of the dtype asked for", fn, tensor_name);
    if (t.end - t.begin != numel * dtype_size(dtype))
      return fail(FB_ERR_FORMAT, "%s: \"%s\" holds %llu bytes, %llu elements were asked for", fn, tensor_name,
                  (unsigned long long)(t.end - t.begin), (unsigned long long)numel);
    if (t.end == t.begin) return FB_OK;
    if (!dst) return fail(FB_ERR_INVALID_ARG, "%s: null destination", fn);
    const char* src = static_cast<const char*>(image) + ds + t.begin;
    if (dst_on_device) FB_CUDA(cudaMemcpyAsync(dst, src, t.end - t.begin, cudaMemcpyHostToDevice, stream));
    else memcpy(dst, src, t.end - t.begin);
    return FB_OK;
  }
  return fail(FB_ERR_FORMAT, "%s: the image has no tensor \"%s\"", fn, tensor_name);
}

}  // extern "C"
