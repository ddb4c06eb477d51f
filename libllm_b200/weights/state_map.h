// Weights by tensor name.
//
// StateMap is the table of a model folder's tensors (one model.safetensors, or the shards an
// index file names), or of tensors handed over in host memory.  A model states what it needs as
// a list of TensorNeed and gets back either every tensor or ONE error that lists all that is
// missing, all that is unexpected and every wrong shape.  The reference fails at the first
// tensor it cannot find or whose shape differs (src/libllm/var_builder.cc:97-140); the messages
// here keep its wording per tensor.
//
// Precision on the device: operands of matrix products ("matrix") are converted to the engine's
// type; norm weights and biases ("vector") are kept or widened to 32-bit (a 16-bit float widens
// exactly); integer tables ("table") become int32.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "util/device.h"
#include "weights/safetensors.h"

namespace llm {

enum class TensorRole { Matrix, Vector, Table };

struct TensorNeed {
  std::string name;
  std::vector<int64_t> shape;
  TensorRole role = TensorRole::Matrix;
  bool optional = false;
};

struct WrongShape {
  std::string name;
  std::vector<int64_t> expected, found;
};

struct WeightsReport {
  std::vector<std::string> missing, unexpected, ignored;
  std::vector<WrongShape> wrong_shape;
};

class WeightsError : public Error {
 public:
  WeightsError(const std::string &msg, WeightsReport r) : Error(ErrorKind::Weights, msg), report(std::move(r)) {}
  WeightsReport report;
};

bool name_matches(const std::string &pattern, const std::string &name);   // '*' matches any run of characters
std::string shape_text(const std::vector<int64_t> &shape);

class StateMap {
 public:
  static std::unique_ptr<StateMap> from_folder(const std::string &folder);
  static std::unique_ptr<StateMap> in_memory() { return std::unique_ptr<StateMap>(new StateMap("<memory>")); }
  // A tensor in host memory that the caller keeps alive while the map is used.
  void add(const std::string &name, const StoredTensor &t);

  const std::string &where() const { return where_; }
  const std::vector<std::string> &names() const { return names_; }
  bool has(const std::string &name) const { return tensors_.count(name) != 0; }
  const StoredTensor &stored(const std::string &name) const;

  // Throws one WeightsError naming every missing and misshapen tensor and every tensor that no
  // part asks for and no pattern of `ignore` covers.  With `strict` false, unexpected tensors
  // alone are not an error; they are returned in the report.
  WeightsReport check(const std::vector<TensorNeed> &needs, const std::vector<std::string> &ignore, bool strict = true) const;

  // The element type `need` has on the device in an engine of type `engine`.
  static DType device_dtype(const TensorNeed &need, DType engine);
  // Converts the tensor of `need` and copies it to `dst` on the device (numel * dtype_size bytes).
  void fetch_into(const TensorNeed &need, DType target, void *dst) const;

 private:
  explicit StateMap(std::string where) : where_(std::move(where)) {}
  std::string where_;
  std::vector<std::unique_ptr<SafetensorsFile>> files_;
  std::vector<std::string> names_;
  std::map<std::string, StoredTensor> tensors_;
  std::map<std::string, std::string> origin_;
};

}  // namespace llm
