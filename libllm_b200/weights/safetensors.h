// Reader and writer of the safetensors container.
//
// The file is: an 8-byte little-endian length, a JSON header of that length mapping each tensor
// name to {"dtype", "shape", "data_offsets": [begin, end]} relative to the end of the header,
// then the raw little-endian data.  The reference reads a container of its own ("TDIC",
// src/libllm/var_builder.cc:38-95) that an offline exporter writes; reading the checkpoint's own
// file takes that step's place.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "util/json.h"

namespace llm {

enum class StoredType { F32, F16, BF16, F64, I64, I32, I16, I8, U8, BOOL };
const char *stored_type_name(StoredType t);
size_t stored_type_size(StoredType t);
bool stored_type_is_float(StoredType t);
StoredType stored_type_from_name(const std::string &name, const std::string &where);

struct StoredTensor {
  StoredType dtype;
  std::vector<int64_t> shape;
  const uint8_t *data = nullptr;   // little-endian elements, row-major
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (auto s : shape) n *= s;
    return n;
  }
};

// One file, memory-mapped: nothing is read until a tensor's bytes are used.
class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string &path);
  ~SafetensorsFile();
  SafetensorsFile(const SafetensorsFile &) = delete;
  SafetensorsFile &operator=(const SafetensorsFile &) = delete;

  const std::string &path() const { return path_; }
  const std::vector<std::string> &names() const { return names_; }
  bool has(const std::string &name) const { return entries_.count(name) != 0; }
  const StoredTensor &tensor(const std::string &name) const { return entries_.at(name); }
  const Json &metadata() const { return metadata_; }

 private:
  std::string path_;
  int fd_ = -1;
  uint8_t *map_ = nullptr;
  size_t size_ = 0;
  std::vector<std::string> names_;
  std::map<std::string, StoredTensor> entries_;
  Json metadata_;
};

struct NamedTensor {
  std::string name;
  StoredTensor tensor;
};
// Writes `tensors`, in the order given, as one file.
void write_safetensors(const std::string &path, const std::vector<NamedTensor> &tensors, const Json &metadata = Json());

// Conversions of 16-bit floats on the host.
float half_to_float(uint16_t h);
inline float bf16_to_float(uint16_t b) {
  union { uint32_t u; float f; } x;
  x.u = (uint32_t)b << 16;
  return x.f;
}
inline uint16_t float_to_bf16(float f) {          // round to nearest, ties to even
  union { uint32_t u; float f; } x;
  x.f = f;
  if ((x.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x.u >> 16) | 0x40);   // NaN stays NaN
  const uint32_t round = 0x7fffu + ((x.u >> 16) & 1u);
  return (uint16_t)((x.u + round) >> 16);
}

}  // namespace llm
