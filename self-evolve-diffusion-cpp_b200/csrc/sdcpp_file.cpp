// .sdcpp v1 packs: the reader (mmap + validate + views, optional one-time upload
// of every int8 tensor) and the offline packer (safetensors -> .sdcpp with the
// row quantization done on the GPU).
//
// On-disk layout, little-endian, no padding (reference src/serde/sdcpp.cpp:1-8,
// tools/quantize/pack_sdcpp.py:4-13):
//   'SDCP' | u32 version=1 | u32 count | per tensor { u32 name_len | name |
//   u8 dtype (0 int8 rowwise, 1 f32 raw) | u32 ndim | i64 dims[ndim] |
//   u64 offset into blob } | blob
//   dtype 0 blob: numel int8, then rows = numel/dims[-1] fp32 scales; dtype 1: numel fp32.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "sdq_internal.h"

namespace sdq {
int context_sm_count();
bool pin_readonly_mapping(void* base, size_t size);
int pack_upload_weight(const int8_t* q_host, const float* scale_host, int64_t N, int64_t K,
                       sdq_weight_t* out);
int pack_upload_finish();
void unpin_mapping(void* base);
}

struct sdq_pack {
  void* base = nullptr;
  size_t size = 0;
  bool registered = false;  // the mapping is page-locked for direct DMA (SDQ_PACK_UPLOAD)
  struct Item {
    std::string name;
    int32_t dtype;
    std::vector<int64_t> dims;
    const uint8_t* data;
    uint64_t nbytes;
    sdq_weight_t weight = 0;
  };
  std::vector<Item> items;
  std::unordered_map<std::string, size_t> index;
};

namespace {

using sdq::fail;

// The unread part of the mapped file.  take() hands out the next n bytes, or nothing when
// fewer are left; nothing is ever read past the end of the mapping.
class Bytes {
 public:
  Bytes(const uint8_t* begin, size_t n) : at_(begin), left_(n) {}
  const uint8_t* take(size_t n) {
    if (n > left_) return nullptr;
    const uint8_t* p = at_;
    at_ += n;
    left_ -= n;
    return p;
  }
  template <typename T>
  bool read(T* v) {  // little-endian scalar, any alignment
    const uint8_t* p = take(sizeof(T));
    if (p) memcpy(v, p, sizeof(T));
    return p != nullptr;
  }
  const uint8_t* here() const { return at_; }
  size_t left() const { return left_; }

 private:
  const uint8_t* at_;
  size_t left_;
};

// What can be wrong with one directory record; the texts are the reference loader's
// (src/serde/sdcpp.cpp:78-101), and so is the order in which the conditions are tested.
enum class Flaw { None, Truncated, DtypeCode, Rank, NegativeDim, Size, NoLastDim };
const char* flaw_text(Flaw f) {
  switch (f) {
    case Flaw::Truncated: return "truncated file";
    case Flaw::DtypeCode: return "bad dtype code";
    case Flaw::Rank: return "ndim too large";
    case Flaw::NegativeDim: return "negative dim";
    case Flaw::Size: return "tensor too large";
    case Flaw::NoLastDim: return "quantized tensor needs a last dim";
    default: return "";
  }
}

// One directory record: a tensor's name, storage kind, shape and place in the blob.
struct Record {
  std::string name;
  bool quantized = false;       // int8 rows + one fp32 scale per row; otherwise raw fp32
  std::vector<int64_t> shape;
  uint64_t where = 0;           // offset of its bytes from the start of the blob
  uint64_t elements = 0;
  uint64_t scale_count() const { return quantized ? elements / (uint64_t)shape.back() : 0; }
  uint64_t span() const { return quantized ? elements + 4 * scale_count() : 4 * elements; }
};

constexpr uint32_t kMaxRank = 8;
constexpr uint64_t kMaxElements = uint64_t(1) << 40;

Flaw decode_record(Bytes& in, Record* r) {
  uint32_t name_bytes = 0, rank = 0;
  uint8_t kind = 0;
  const uint8_t* name = in.read(&name_bytes) ? in.take(name_bytes) : nullptr;
  if (!name) return Flaw::Truncated;
  r->name.assign(reinterpret_cast<const char*>(name), name_bytes);
  if (!in.read(&kind)) return Flaw::Truncated;
  if (kind > 1) return Flaw::DtypeCode;
  r->quantized = kind == 0;
  if (!in.read(&rank)) return Flaw::Truncated;
  if (rank > kMaxRank) return Flaw::Rank;
  r->shape.assign(rank, 0);
  r->elements = 1;
  for (int64_t& extent : r->shape) {
    if (!in.read(&extent)) return Flaw::Truncated;
    if (extent < 0) return Flaw::NegativeDim;
    if (extent != 0 && r->elements > kMaxElements / (uint64_t)extent) return Flaw::Size;
    r->elements *= (uint64_t)extent;
  }
  if (!in.read(&r->where)) return Flaw::Truncated;
  if (r->quantized && (rank == 0 || r->shape.back() < 1)) return Flaw::NoLastDim;
  return Flaw::None;
}

void fill_entry(const sdq_pack::Item& it, const sdq_pack* p, sdq_entry* out) {
  out->name = it.name.c_str();
  out->dtype = it.dtype;
  out->ndim = (int32_t)it.dims.size();
  for (int i = 0; i < 8; i++) out->dims[i] = i < (int)it.dims.size() ? it.dims[i] : 0;
  out->data = it.data;
  out->nbytes = it.nbytes;
  out->file_offset = (uint64_t)(it.data - (const uint8_t*)p->base);
  out->weight = it.weight;
  out->name_len = it.name.size();
}

}  // namespace

extern "C" {

int sdq_pack_open(const char* path, uint32_t flags, sdq_pack** out) {
  if (!path || !out) return fail(SDQ_ERR_INVALID, "sdq_pack_open: null argument");
  *out = nullptr;
  const std::string spath(path);
  // Messages mirror the reference loader's (src/serde/sdcpp.cpp:50-66,78-105).
  int fd = open(path, O_RDONLY);
  if (fd < 0) return fail(SDQ_ERR_IO, "sdcpp: cannot open " + spath);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 16) {
    close(fd);
    return fail(SDQ_ERR_FORMAT, "sdcpp: truncated file " + spath);
  }
  const size_t size = (size_t)st.st_size;
  void* base = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return fail(SDQ_ERR_IO, "sdcpp: mmap failed " + spath);

  auto bad = [&](const char* m) {
    munmap(base, size);
    return fail(SDQ_ERR_FORMAT, std::string("sdcpp: ") + m);
  };
  // header: magic, version, record count, then the directory; the blob is whatever follows it
  Bytes in(static_cast<const uint8_t*>(base), size);
  uint32_t version = 0, count = 0;
  if (memcmp(in.take(4), "SDCP", 4) != 0) return bad("bad magic");   // size >= 16 was checked above
  in.read(&version);
  if (version != 1) return bad("unsupported version");
  in.read(&count);
  std::vector<Record> directory;
  directory.reserve(std::min<uint32_t>(count, 1u << 20));
  for (uint32_t i = 0; i < count; i++) {
    directory.emplace_back();
    const Flaw f = decode_record(in, &directory.back());
    if (f != Flaw::None) return bad(flaw_text(f));
  }
  const uint8_t* blob = in.here();
  const uint64_t blob_bytes = in.left();
  for (const Record& r : directory)
    if (r.where > blob_bytes || r.span() > blob_bytes - r.where) return bad("data out of bounds");

  // entries, as the reference's map presents them: a quantized tensor as `name` (int8, its own
  // shape) and `name.scale` (fp32, one per row) right behind its bytes; a raw tensor as `name`
  sdq_pack* p = new sdq_pack;
  p->base = base;
  p->size = size;
  auto present = [&](const std::string& name, int32_t dt, std::vector<int64_t> dims, const uint8_t* data,
                     uint64_t nbytes) {
    if (!p->index.emplace(name, p->items.size()).second) return;  // the first of equal names stays
    sdq_pack::Item it;
    it.name = name; it.dtype = dt; it.dims = std::move(dims); it.data = data; it.nbytes = nbytes;
    p->items.push_back(std::move(it));
  };
  for (const Record& r : directory) {
    const uint8_t* bytes = blob + r.where;
    if (r.quantized) {
      present(r.name, SDQ_DT_I8, r.shape, bytes, r.elements);
      present(r.name + ".scale", SDQ_DT_F32, {(int64_t)r.scale_count()}, bytes + r.elements, 4 * r.scale_count());
    } else {
      present(r.name, SDQ_DT_F32, r.shape, bytes, r.span());
    }
  }

  if (flags & SDQ_PACK_UPLOAD) {
    // Page-lock the read-only file mapping so that the uploads below are direct DMA from the
    // page cache (no staging copy).  Not every kernel / file system allows it for a
    // file-backed mapping; when it is refused the copies go through the driver's own staging.
    p->registered = sdq::pin_readonly_mapping(p->base, p->size);
    for (auto& it : p->items) {
      if (it.dtype != SDQ_DT_I8 || it.nbytes == 0) continue;
      const int64_t last = it.dims.back(), rows = (int64_t)it.nbytes / last;
      int rc = sdq::pack_upload_weight((const int8_t*)it.data, (const float*)(it.data + it.nbytes),
                                       rows, last, &it.weight);
      if (rc != SDQ_OK) {
        const std::string msg = sdq_last_error();
        sdq_pack_close(p);
        return fail(rc, msg);
      }
    }
  }
  if (flags & SDQ_PACK_UPLOAD) {
    if (int rc = sdq::pack_upload_finish()) {
      const std::string msg = sdq_last_error();
      sdq_pack_close(p);
      return fail(rc, msg);
    }
  }
  *out = p;
  return SDQ_OK;
}

int64_t sdq_pack_count(const sdq_pack* p) { return p ? (int64_t)p->items.size() : -1; }
int sdq_pack_pinned(const sdq_pack* p) { return p && p->registered ? 1 : 0; }

int sdq_pack_entry(const sdq_pack* p, int64_t index, sdq_entry* out) {
  if (!p || !out || index < 0 || index >= (int64_t)p->items.size())
    return fail(SDQ_ERR_INVALID, "sdq_pack_entry: bad pack or index");
  fill_entry(p->items[(size_t)index], p, out);
  return SDQ_OK;
}

int sdq_pack_find(const sdq_pack* p, const char* name, sdq_entry* out) {
  if (!p || !name || !out) return fail(SDQ_ERR_INVALID, "sdq_pack_find: null argument");
  auto it = p->index.find(name);
  if (it == p->index.end()) return fail(SDQ_ERR_NOT_FOUND, std::string("sdq_pack_find: no entry ") + name);
  fill_entry(p->items[it->second], p, out);
  return SDQ_OK;
}

int sdq_pack_close(sdq_pack* p) {
  if (!p) return SDQ_OK;
  for (auto& it : p->items)
    if (it.weight) sdq_weight_release(it.weight);
  if (p->registered) sdq::unpin_mapping(p->base);
  if (p->base) munmap(p->base, p->size);
  delete p;
  return SDQ_OK;
}

}  // extern "C"

// =====================================================================  packer
namespace {

// ---- a small JSON reader, enough for a safetensors header ----
struct JVal {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  int64_t inum = 0;
  bool is_int = false;
  std::string str;
  std::vector<JVal> arr;
  std::vector<std::pair<std::string, JVal>> obj;  // file order preserved
  const JVal* get(const char* k) const {
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char* p; const char* end; bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) p++; }
  static void put_utf8(std::string& s, uint32_t cp) {
    if (cp < 0x80) s += (char)cp;
    else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
  }
  bool hex4(uint32_t* v) {
    if (end - p < 4) return false;
    uint32_t r = 0;
    for (int i = 0; i < 4; i++) {
      char ch = *p++; r <<= 4;
      if (ch >= '0' && ch <= '9') r |= ch - '0';
      else if (ch >= 'a' && ch <= 'f') r |= ch - 'a' + 10;
      else if (ch >= 'A' && ch <= 'F') r |= ch - 'A' + 10;
      else return false;
    }
    *v = r; return true;
  }
  std::string string() {
    std::string s;
    if (p >= end || *p != '"') { ok = false; return s; }
    p++;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        p++;
        if (p >= end) { ok = false; return s; }
        char ch = *p++;
        switch (ch) {
          case 'n': s += '\n'; break; case 't': s += '\t'; break; case 'r': s += '\r'; break;
          case 'b': s += '\b'; break; case 'f': s += '\f'; break;
          case 'u': {
            uint32_t cp;
            if (!hex4(&cp)) { ok = false; return s; }
            if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
              p += 2; uint32_t lo;
              if (!hex4(&lo)) { ok = false; return s; }
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            put_utf8(s, cp); break;
          }
          default: s += ch;  // \" \\ \/
        }
      } else s += *p++;
    }
    if (p >= end) { ok = false; return s; }
    p++;
    return s;
  }
  JVal value(int depth = 0) {
    JVal v; ws();
    if (!ok || p >= end || depth > 64) { ok = false; return v; }
    if (*p == '{') {
      v.kind = JVal::Obj; p++; ws();
      if (p < end && *p == '}') { p++; return v; }
      while (ok) {
        ws(); std::string k = string(); ws();
        if (!ok || p >= end || *p != ':') { ok = false; break; }
        p++;
        v.obj.emplace_back(std::move(k), value(depth + 1)); ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == '}') { p++; break; }
        ok = false;
      }
    } else if (*p == '[') {
      v.kind = JVal::Arr; p++; ws();
      if (p < end && *p == ']') { p++; return v; }
      while (ok) {
        v.arr.push_back(value(depth + 1)); ws();
        if (p < end && *p == ',') { p++; continue; }
        if (p < end && *p == ']') { p++; break; }
        ok = false;
      }
    } else if (*p == '"') {
      v.kind = JVal::Str; v.str = string();
    } else if (end - p >= 4 && !strncmp(p, "true", 4)) { v.kind = JVal::Bool; v.b = true; p += 4; }
    else if (end - p >= 5 && !strncmp(p, "false", 5)) { v.kind = JVal::Bool; p += 5; }
    else if (end - p >= 4 && !strncmp(p, "null", 4)) { p += 4; }
    else {
      const char* s = p; bool isint = true;
      if (p < end && (*p == '-' || *p == '+')) p++;
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
        if (*p == '.' || *p == 'e' || *p == 'E') isint = false;
        p++;
      }
      if (p == s) { ok = false; return v; }
      std::string t(s, p);
      v.kind = JVal::Num; v.is_int = isint;
      v.num = strtod(t.c_str(), nullptr);
      if (isint) v.inum = strtoll(t.c_str(), nullptr, 10);
    }
    return v;
  }
};

struct SrcType { const char* name; int esz; bool is_float; int sdq_dt; };
// tools/quantize/pack_sdcpp.py:26-35
const SrcType kSrc[] = {{"BF16", 2, true, SDQ_BF16}, {"F16", 2, true, SDQ_F16}, {"F32", 4, true, SDQ_F32},
                        {"I8", 1, false, -1},        {"U8", 1, false, -1},      {"I32", 4, false, -1},
                        {"I64", 8, false, -1}};
const SrcType* find_src(const std::string& n) {
  for (auto& s : kSrc) if (n == s.name) return &s;
  return nullptr;
}

float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu, u;
  if (e == 0) {
    if (m == 0) u = sign;
    else { int sh = 0; while (!(m & 0x400u)) { m <<= 1; sh++; } m &= 0x3ffu; u = sign | ((uint32_t)(113 - sh) << 23) | (m << 13); }
  } else if (e == 31) u = sign | 0x7f800000u | (m << 13);
  else u = sign | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}

// to_f32 of the packer (tools/quantize/pack_sdcpp.py:38-42) for tensors kept raw.
void raw_to_f32(const uint8_t* src, const std::string& dt, int64_t n, float* dst) {
  if (dt == "F32") { memcpy(dst, src, (size_t)n * 4); return; }
  for (int64_t i = 0; i < n; i++) {
    if (dt == "BF16") { uint16_t h; memcpy(&h, src + 2 * i, 2); uint32_t u = (uint32_t)h << 16; memcpy(&dst[i], &u, 4); }
    else if (dt == "F16") { uint16_t h; memcpy(&h, src + 2 * i, 2); dst[i] = half_to_float(h); }
    else if (dt == "I8") dst[i] = (float)(int8_t)src[i];
    else if (dt == "U8") dst[i] = (float)src[i];
    else if (dt == "I32") { int32_t v; memcpy(&v, src + 4 * i, 4); dst[i] = (float)v; }
    else { int64_t v; memcpy(&v, src + 8 * i, 8); dst[i] = (float)v; }
  }
}

std::vector<std::string> split(const char* s, char sep) {
  std::vector<std::string> out; std::string cur;
  for (const char* p = s ? s : ""; ; p++) {
    if (*p == sep || *p == 0) { if (!cur.empty()) out.push_back(cur); cur.clear(); if (!*p) break; }
    else cur += *p;
  }
  return out;
}

template <typename T> void put(std::string& s, T v) { s.append(reinterpret_cast<const char*>(&v), sizeof(T)); }

struct Planned {
  std::string name, dt; std::vector<int64_t> dims;
  int code; uint64_t off; int64_t numel, rows; uint64_t beg, end;
};

}  // namespace

extern "C" int sdq_pack_sdcpp(const char* safetensors_in, const char* sdcpp_out, const char* only,
                              const char* dtype_preserve) {
  if (!safetensors_in || !sdcpp_out) return fail(SDQ_ERR_INVALID, "sdq_pack_sdcpp: null path");
  if (sdq_device() < 0) return fail(SDQ_ERR_NOT_INIT, "sdq_pack_sdcpp: sdq_init has not been called (the packer quantizes on the GPU)");
  int fd = open(safetensors_in, O_RDONLY);
  if (fd < 0) return fail(SDQ_ERR_IO, std::string("cannot open ") + safetensors_in);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) { close(fd); return fail(SDQ_ERR_FORMAT, "safetensors: file too short"); }
  const size_t size = (size_t)st.st_size;
  void* base = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (base == MAP_FAILED) return fail(SDQ_ERR_IO, "safetensors: mmap failed");
  struct Unmap { void* b; size_t n; ~Unmap() { munmap(b, n); } } unmap{base, size};
  const uint8_t* b = (const uint8_t*)base;
  uint64_t hlen; memcpy(&hlen, b, 8);
  if (hlen > size - 8) return fail(SDQ_ERR_FORMAT, "safetensors: header length exceeds file");
  JParser jp{(const char*)b + 8, (const char*)b + 8 + hlen};
  JVal hdr = jp.value();
  if (!jp.ok || hdr.kind != JVal::Obj) return fail(SDQ_ERR_FORMAT, "safetensors: header is not valid JSON");
  const uint64_t data_base = 8 + hlen;

  const auto only_l = split(only, ',');
  const auto pres_v = split(dtype_preserve, ':');
  const std::set<std::string> preserve(pres_v.begin(), pres_v.end());

  // pass 1: which tensors, in source-offset order; quantize or keep; blob offsets
  // (tools/quantize/pack_sdcpp.py:70-88)
  std::vector<Planned> plan;
  for (auto& kv : hdr.obj) {
    if (kv.first == "__metadata__") continue;
    if (!only_l.empty()) {
      bool hit = false;
      for (auto& pre : only_l) if (kv.first.compare(0, pre.size(), pre) == 0) { hit = true; break; }
      if (!hit) continue;
    }
    const JVal* dt = kv.second.get("dtype"); const JVal* sh = kv.second.get("shape");
    const JVal* off = kv.second.get("data_offsets");
    if (!dt || dt->kind != JVal::Str || !sh || sh->kind != JVal::Arr || !off || off->kind != JVal::Arr || off->arr.size() != 2)
      return fail(SDQ_ERR_FORMAT, "safetensors: malformed entry " + kv.first);
    Planned t; t.name = kv.first; t.dt = dt->str;
    t.numel = 1;
    for (auto& d : sh->arr) {
      if (d.kind != JVal::Num || d.inum < 0) return fail(SDQ_ERR_FORMAT, "safetensors: bad shape in " + kv.first);
      t.dims.push_back(d.inum);
      if (d.inum && t.numel > (int64_t{1} << 40) / d.inum) return fail(SDQ_ERR_FORMAT, "safetensors: tensor too large " + kv.first);
      t.numel *= d.inum;
    }
    t.beg = (uint64_t)off->arr[0].inum; t.end = (uint64_t)off->arr[1].inum;
    plan.push_back(std::move(t));
  }
  std::stable_sort(plan.begin(), plan.end(), [](const Planned& a, const Planned& c) { return a.beg < c.beg; });
  uint64_t blob_off = 0;
  for (auto& t : plan) {
    const SrcType* s = find_src(t.dt);
    if (!s) return fail(SDQ_ERR_FORMAT, "unsupported dtype " + t.dt + " for " + t.name);
    if (t.end < t.beg || t.end - t.beg != (uint64_t)t.numel * s->esz || data_base + t.end > size)
      return fail(SDQ_ERR_FORMAT, "safetensors: data_offsets of " + t.name + " do not match its shape or the file");
    const bool quant = s->is_float && !preserve.count(t.dt) && t.numel >= 65536;
    t.code = quant ? 0 : 1;
    t.rows = (quant && !t.dims.empty() && t.dims.back()) ? t.numel / t.dims.back() : 0;
    t.off = blob_off;
    blob_off += quant ? (uint64_t)t.numel + (uint64_t)t.rows * 4 : (uint64_t)t.numel * 4;
  }

  FILE* out = fopen(sdcpp_out, "wb");
  if (!out) return fail(SDQ_ERR_IO, std::string("cannot create ") + sdcpp_out);
  struct Closer { FILE* f; ~Closer() { if (f) fclose(f); } } closer{out};
  std::string h("SDCP", 4);
  put<uint32_t>(h, 1); put<uint32_t>(h, (uint32_t)plan.size());
  for (auto& t : plan) {
    put<uint32_t>(h, (uint32_t)t.name.size()); h += t.name; put<uint8_t>(h, (uint8_t)t.code);
    put<uint32_t>(h, (uint32_t)t.dims.size());
    for (int64_t d : t.dims) put<int64_t>(h, d);
    put<uint64_t>(h, t.off);
  }
  if (fwrite(h.data(), 1, h.size(), out) != h.size()) return fail(SDQ_ERR_IO, "write failed");

  // pass 2: stream the data.  Quantized tensors go through the GPU in chunks of whole rows.
  constexpr int64_t kChunkElems = int64_t{1} << 26;  // 64 Mi elements per round trip
  void* d_src = nullptr; int8_t* d_q = nullptr; float* d_scale = nullptr;
  size_t cap_src = 0, cap_q = 0, cap_scale = 0;
  std::vector<int8_t> h_q; std::vector<float> h_scale, h_f32;
  int rc = SDQ_OK;
  auto ensure = [&](void** p, size_t* cap, size_t need) -> bool {
    if (need <= *cap) return true;
    if (*p) sdq_free(*p);
    *p = nullptr; *cap = 0;
    if (sdq_malloc(p, need) != SDQ_OK) return false;
    *cap = need; return true;
  };
  for (auto& t : plan) {
    const SrcType* s = find_src(t.dt);
    const uint8_t* src = b + data_base + t.beg;
    if (t.code == 1) {
      h_f32.resize((size_t)t.numel);
      raw_to_f32(src, t.dt, t.numel, h_f32.data());
      if (t.numel && fwrite(h_f32.data(), 4, (size_t)t.numel, out) != (size_t)t.numel) { rc = fail(SDQ_ERR_IO, "write failed"); break; }
      continue;
    }
    const int64_t last = t.dims.back();
    h_scale.resize((size_t)t.rows);
    const int64_t step = std::max<int64_t>(1, kChunkElems / last);
    for (int64_t r0 = 0; r0 < t.rows && rc == SDQ_OK; r0 += step) {
      const int64_t nr = std::min(step, t.rows - r0), ne = nr * last;
      if (!ensure(&d_src, &cap_src, (size_t)ne * s->esz) || !ensure((void**)&d_q, &cap_q, (size_t)ne) ||
          !ensure((void**)&d_scale, &cap_scale, (size_t)nr * 4)) { rc = fail(SDQ_ERR_NOMEM, sdq_last_error()); break; }
      h_q.resize((size_t)ne);
      if ((rc = sdq_memcpy_h2d(d_src, src + (size_t)r0 * last * s->esz, (size_t)ne * s->esz, nullptr)) != SDQ_OK) break;
      if ((rc = sdq_quantize_rows(d_src, s->sdq_dt, nr, last, SDQ_MODE_PACKER, d_q, d_scale, 0, nullptr)) != SDQ_OK) break;
      if ((rc = sdq_memcpy_d2h(h_q.data(), d_q, (size_t)ne, nullptr)) != SDQ_OK) break;
      if ((rc = sdq_memcpy_d2h(h_scale.data() + r0, d_scale, (size_t)nr * 4, nullptr)) != SDQ_OK) break;
      if ((rc = sdq_stream_sync(nullptr)) != SDQ_OK) break;
      if (fwrite(h_q.data(), 1, (size_t)ne, out) != (size_t)ne) { rc = fail(SDQ_ERR_IO, "write failed"); break; }
    }
    if (rc != SDQ_OK) break;
    if (t.rows && fwrite(h_scale.data(), 4, (size_t)t.rows, out) != (size_t)t.rows) { rc = fail(SDQ_ERR_IO, "write failed"); break; }
  }
  std::string keep = rc != SDQ_OK ? sdq_last_error() : "";
  if (d_src) sdq_free(d_src);
  if (d_q) sdq_free(d_q);
  if (d_scale) sdq_free(d_scale);
  if (rc != SDQ_OK) return fail(rc, keep);
  closer.f = nullptr;
  if (fclose(out) != 0) return fail(SDQ_ERR_IO, "close failed");
  return SDQ_OK;
}
