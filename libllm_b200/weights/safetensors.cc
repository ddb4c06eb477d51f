#include "weights/safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <fstream>

namespace llm {

namespace {
struct TypeInfo {
  StoredType t;
  const char *name;
  size_t size;
  bool is_float;
};
const TypeInfo TYPES[] = {
    {StoredType::F32, "F32", 4, true},  {StoredType::F16, "F16", 2, true},  {StoredType::BF16, "BF16", 2, true},
    {StoredType::F64, "F64", 8, true},  {StoredType::I64, "I64", 8, false}, {StoredType::I32, "I32", 4, false},
    {StoredType::I16, "I16", 2, false}, {StoredType::I8, "I8", 1, false},   {StoredType::U8, "U8", 1, false},
    {StoredType::BOOL, "BOOL", 1, false},
};
const TypeInfo &info(StoredType t) { return TYPES[(int)t]; }
}  // namespace

const char *stored_type_name(StoredType t) { return info(t).name; }
size_t stored_type_size(StoredType t) { return info(t).size; }
bool stored_type_is_float(StoredType t) { return info(t).is_float; }

StoredType stored_type_from_name(const std::string &name, const std::string &where) {
  for (const auto &t : TYPES)
    if (name == t.name) return t.t;
  LLM_THROW(Weights, "%s has unsupported dtype %s", where.c_str(), name.c_str());
}

float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
  union { uint32_t u; float f; } x;
  if (exp == 0) {
    if (man == 0) {
      x.u = sign;
    } else {            // subnormal: renormalise
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400u));
      x.u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    x.u = sign | 0x7f800000u | (man << 13);
  } else {
    x.u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  return x.f;
}

SafetensorsFile::SafetensorsFile(const std::string &path) : path_(path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) LLM_THROW(Weights, "%s: cannot open (%s)", path.c_str(), strerror(errno));
  struct stat st;
  if (fstat(fd_, &st) != 0) {
    ::close(fd_);
    LLM_THROW(Weights, "%s: cannot stat", path.c_str());
  }
  size_ = (size_t)st.st_size;
  auto fail = [&](const std::string &msg) {
    if (map_) munmap(map_, size_);
    ::close(fd_);
    map_ = nullptr;
    fd_ = -1;
    throw Error(ErrorKind::Weights, path_ + ": " + msg);
  };
  if (size_ < 8) fail("truncated file (no header length)");
  map_ = (uint8_t *)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
  if (map_ == MAP_FAILED) {
    map_ = nullptr;
    fail("cannot map the file");
  }
  uint64_t hlen = 0;
  memcpy(&hlen, map_, 8);
  if (hlen == 0 || hlen > size_ - 8) fail(format("truncated file (header of %llu bytes, file of %zu)", (unsigned long long)hlen, size_));
  Json header;
  try {
    header = Json::parse(std::string((const char *)map_ + 8, (size_t)hlen), path_);
  } catch (const Error &e) {
    fail(std::string("invalid header (") + e.what() + ")");
  }
  if (!header.is_object()) fail("invalid header (not an object)");
  const size_t base = 8 + (size_t)hlen;
  for (const auto &m : header.members()) {
    if (m.first == "__metadata__") {
      metadata_ = m.second;
      continue;
    }
    const Json &e = m.second;
    const std::string what = "tensor '" + m.first + "'";
    if (!e.is_object() || !e.get("dtype").is_string() || !e.get("shape").is_array() || !e.get("data_offsets").is_array() ||
        e.get("data_offsets").size() != 2)
      fail(what + " has a malformed header entry");
    StoredTensor t;
    try {
      t.dtype = stored_type_from_name(e.get("dtype").as_string(), what);
    } catch (const Error &err) {
      fail(err.what());
    }
    for (const auto &d : e.get("shape").items()) {
      if (!d.is_int() || d.as_int() < 0) fail(what + " has a malformed shape");
      t.shape.push_back(d.as_int());
    }
    const int64_t b = e.get("data_offsets").at(0).as_int(), end = e.get("data_offsets").at(1).as_int();
    const int64_t want = t.numel() * (int64_t)stored_type_size(t.dtype);
    if (b < 0 || end - b != want)
      fail(format("%s has %lld bytes, its shape needs %lld", what.c_str(), (long long)(end - b), (long long)want));
    if (base + (size_t)end > size_)
      fail(format("truncated file (%s ends at byte %zu, file has %zu)", what.c_str(), base + (size_t)end, size_));
    if (entries_.count(m.first)) fail(what + " is stored twice");
    t.data = map_ + base + b;
    t.nbytes = (size_t)want;
    names_.push_back(m.first);
    entries_[m.first] = std::move(t);
  }
}

SafetensorsFile::~SafetensorsFile() {
  if (map_) munmap(map_, size_);
  if (fd_ >= 0) ::close(fd_);
}

void write_safetensors(const std::string &path, const std::vector<NamedTensor> &tensors, const Json &metadata) {
  Json header = Json::object();
  if (metadata.is_object()) header.set("__metadata__", metadata);
  int64_t offset = 0;
  for (const auto &nt : tensors) {
    Json e = Json::object();
    e.set("dtype", stored_type_name(nt.tensor.dtype));
    e.set("shape", Json::list(nt.tensor.shape));
    Json off = Json::array();
    off.push(offset);
    off.push(offset + (int64_t)nt.tensor.nbytes);
    e.set("data_offsets", off);
    if (header.has(nt.name)) LLM_THROW(Weights, "%s: tensor '%s' is given twice", path.c_str(), nt.name.c_str());
    header.set(nt.name, e);
    offset += (int64_t)nt.tensor.nbytes;
  }
  std::string blob = header.dump();
  while (blob.size() % 8) blob.push_back(' ');
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) LLM_THROW(Weights, "%s: cannot write", path.c_str());
  const uint64_t hlen = blob.size();
  f.write((const char *)&hlen, 8);
  f.write(blob.data(), (std::streamsize)blob.size());
  for (const auto &nt : tensors) f.write((const char *)nt.tensor.data, (std::streamsize)nt.tensor.nbytes);
  if (!f) LLM_THROW(Weights, "%s: write failed", path.c_str());
}

}  // namespace llm
