// Reads the data segments out of a compiled executable (`.rtexe`): the FlatBuffers file the reference's
// translation step writes (executor/lib/Target/Lua/TranslateToRuntimeExecutable.cpp:700-850), whose schema is
// executor/include/mlir-executor/Runtime/API/Executable.fbs.  The PTX (or cubin) of every cuda.compiled_module
// of a program ends up as one data segment (a constant global named after the module); the interpreted host
// code hands its bytes to __cuda_load_module, i.e. to mtrt_cuda_module_load_from_ptx.  With this reader the same
// bytes can be reached without the reference's runtime: tools can list what an executable carries, and
// mtrt_cuda_module_load_from_ptx_file accepts "program.rtexe#segment".
//
// Only the tables needed for that are decoded, by hand (no generated code): Executable { name, source,
// data_segments, ... } and DataSegment { name (64-bit offset), data (64-bit offset, 64-bit length), alignment,
// constant, uninitialized_size, address_space }.  Every offset is bounds-checked; a file that does not parse is
// refused with a message, never trusted.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "ql_common.cuh"

namespace ql {
namespace {

struct Reader {
  const uint8_t *p;
  uint64_t n;
  bool ok(uint64_t off, uint64_t len) const { return off <= n && len <= n - off; }
  template <typename T> bool get(uint64_t off, T *v) const {
    if (!ok(off, sizeof(T))) return false;
    memcpy(v, p + off, sizeof(T));
    return true;
  }
  // position of field `index` of the table at `table`, or 0 when the field is absent
  bool field(uint64_t table, int index, uint64_t *pos) const {
    int32_t soff;
    if (!get(table, &soff)) return false;
    const int64_t vt = (int64_t)table - soff;
    if (vt < 0) return false;
    uint16_t vt_bytes, entry = 0;
    if (!get((uint64_t)vt, &vt_bytes)) return false;
    const uint64_t slot = 4 + 2 * (uint64_t)index;
    if (slot + 2 <= vt_bytes && !get((uint64_t)vt + slot, &entry)) return false;
    *pos = entry ? table + entry : 0;
    return true;
  }
  bool follow32(uint64_t pos, uint64_t *target) const {
    uint32_t o;
    if (!get(pos, &o)) return false;
    *target = pos + o;
    return *target < n;
  }
  bool follow64(uint64_t pos, uint64_t *target) const {
    uint64_t o;
    if (!get(pos, &o) || o > n) return false;
    *target = pos + o;
    return *target < n;
  }
  bool string_at(uint64_t pos, std::string *out) const {
    uint32_t len;
    if (!get(pos, &len) || !ok(pos + 4, len)) return false;
    out->assign(reinterpret_cast<const char *>(p + pos + 4), len);
    return true;
  }
};

} // namespace
} // namespace ql

struct ql_rtexe {
  std::vector<uint8_t> bytes;
  std::string name;
  struct Segment {
    std::string name;
    uint64_t offset, size, uninitialized_size;
    uint32_t alignment;
    int32_t constant, address_space;
  };
  std::vector<Segment> segments;
};

using namespace ql;

static int parse_rtexe(ql_rtexe *x) {
  Reader r{x->bytes.data(), (uint64_t)x->bytes.size()};
  const char *bad = "rtexe: not a valid executable (offset out of bounds)";
  uint64_t root, f, t;
  if (!r.follow32(0, &root)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
  // Executable: field 0 name, 1 source, 2 data_segments
  if (!r.field(root, 0, &f)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
  if (f && !(r.follow32(f, &t) && r.string_at(t, &x->name))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
  if (!r.field(root, 2, &f)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
  if (!f) return QL_OK; // no data segments
  uint64_t vec;
  uint32_t count;
  if (!r.follow32(f, &vec) || !r.get(vec, &count) || !r.ok(vec + 4, 4ull * count)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
  for (uint32_t i = 0; i < count; i++) {
    uint64_t seg;
    if (!r.follow32(vec + 4 + 4ull * i, &seg)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    ql_rtexe::Segment s{};
    // DataSegment: 0 name (offset64), 1 data (vector64), 2 alignment, 3 constant, 4 uninitialized_size, 5 address_space
    if (!r.field(seg, 0, &f)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    if (f && !(r.follow64(f, &t) && r.string_at(t, &s.name))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    if (!r.field(seg, 1, &f)) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    if (f) {
      uint64_t len;
      if (!(r.follow64(f, &t) && r.get(t, &len) && r.ok(t + 8, len))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
      s.offset = t + 8;
      s.size = len;
    }
    uint8_t b = 0;
    if (!r.field(seg, 2, &f) || (f && !r.get(f, &s.alignment))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    if (!r.field(seg, 3, &f) || (f && !r.get(f, &b))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    s.constant = b;
    if (!r.field(seg, 4, &f) || (f && !r.get(f, &s.uninitialized_size))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    b = 4; // PointerType::unknown
    if (!r.field(seg, 5, &f) || (f && !r.get(f, &b))) return set_error(QL_ERR_INVALID_ARGUMENT, "%s", bad);
    s.address_space = b;
    x->segments.push_back(s);
  }
  return QL_OK;
}

extern "C" {

int ql_rtexe_open_memory(const void *bytes, uint64_t size, ql_rtexe **out) {
  if (!bytes || !out || size < 8) return set_error(QL_ERR_INVALID_ARGUMENT, "rtexe: empty buffer");
  ql_rtexe *x = new ql_rtexe();
  x->bytes.assign(static_cast<const uint8_t *>(bytes), static_cast<const uint8_t *>(bytes) + size);
  int rc = parse_rtexe(x);
  if (rc != QL_OK) {
    delete x;
    return rc;
  }
  *out = x;
  return QL_OK;
}

int ql_rtexe_open(const char *path, ql_rtexe **out) {
  if (!path || !out) return set_error(QL_ERR_INVALID_ARGUMENT, "rtexe: null argument");
  FILE *f = fopen(path, "rb");
  if (!f) return set_error(QL_ERR_INVALID_ARGUMENT, "rtexe: could not open '%s'", path);
  std::vector<uint8_t> buf;
  uint8_t chunk[65536];
  size_t got;
  while ((got = fread(chunk, 1, sizeof(chunk), f)) > 0) buf.insert(buf.end(), chunk, chunk + got);
  fclose(f);
  return ql_rtexe_open_memory(buf.data(), buf.size(), out);
}

void ql_rtexe_close(ql_rtexe *x) { delete x; }

const char *ql_rtexe_name(const ql_rtexe *x) { return x ? x->name.c_str() : ""; }

int32_t ql_rtexe_num_segments(const ql_rtexe *x) { return x ? (int32_t)x->segments.size() : 0; }

int ql_rtexe_segment(const ql_rtexe *x, int32_t index, ql_rtexe_segment_info *info) {
  if (!x || !info || index < 0 || index >= (int32_t)x->segments.size()) return set_error(QL_ERR_INVALID_ARGUMENT, "rtexe: no segment %d", index);
  const ql_rtexe::Segment &s = x->segments[index];
  info->name = s.name.c_str();
  info->data = s.size ? x->bytes.data() + s.offset : nullptr;
  info->size = s.size;
  info->uninitialized_size = s.uninitialized_size;
  info->alignment = s.alignment;
  info->constant = s.constant;
  info->address_space = s.address_space;
  // what the bytes look like: PTX text, an ELF cubin, a fat binary, or something else (weights, constants)
  info->kind = QL_RTEXE_DATA;
  if (s.size >= 4) {
    const uint8_t *d = x->bytes.data() + s.offset;
    uint32_t magic;
    memcpy(&magic, d, 4);
    if (magic == 0x464C457Fu) info->kind = QL_RTEXE_CUBIN;
    else if (magic == 0xBA55ED50u) info->kind = QL_RTEXE_FATBIN;
    else {
      std::string head(reinterpret_cast<const char *>(d), (size_t)(s.size < 4096 ? s.size : 4096));
      if (head.find(".version") != std::string::npos && head.find(".target") != std::string::npos) info->kind = QL_RTEXE_PTX;
    }
  }
  return QL_OK;
}

int ql_rtexe_find_segment(const ql_rtexe *x, const char *name) {
  if (!x || !name) return -1;
  for (size_t i = 0; i < x->segments.size(); i++)
    if (x->segments[i].name == name) return (int)i;
  return -1;
}
}
