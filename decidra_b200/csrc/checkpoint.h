// Read-only access to a safetensors checkpoint directory: memory-mapped shards, a name -> tensor
// table, and the model description from config.json. Host C++ only (no CUDA).
//
// Same role as Store (native/src/tensor.rs:56-300 in juanqui/decidra) and Config::from_dir
// (native/src/config.rs:49-172): nothing is copied at open time; a tensor is a (dtype, shape,
// byte range) view into the mapping, so a 50 GB checkpoint costs only page cache as it streams
// to the device.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/decidra_b200.h"

namespace ckpt {

// DType::parse, native/src/tensor.rs:25-38 (numbering = DCD_DT_* of the C header)
enum DType { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, I64 = 4, U8 = 5, F8E4M3 = 6 };
size_t dtype_size(int dt);

struct Tensor {
  int dtype = U8;
  std::vector<size_t> shape;
  int shard = 0;
  size_t start = 0, end = 0;  // absolute byte range inside the mapped shard
  size_t count() const { size_t n = 1; for (size_t d : shape) n *= d; return n; }
};

// Minimal JSON document (objects keep insertion order; numbers keep their text so that 64-bit
// offsets stay exact).
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  std::string text;                                  // Number: literal; String: decoded value
  std::vector<Json> items;                           // Array
  std::vector<std::pair<std::string, Json>> members; // Object
  const Json* get(const char* key) const;
  bool as_u64(uint64_t* out) const;  // non-negative integer literal only (serde's as_u64)
  bool as_f64(double* out) const;
  static bool parse(const char* p, size_t n, Json* out, std::string* err);
};

class Store {
 public:
  ~Store();
  // A directory (model.safetensors, or the shards model.safetensors.index.json lists, or every
  // *.safetensors sorted by name) or a single .safetensors file.
  bool open(const std::string& path, std::string* err);
  const Tensor* info(const std::string& name) const;
  bool contains(const std::string& name) const { return info(name) != nullptr; }
  const uint8_t* data(const Tensor& t) const { return shards_[t.shard].base + t.start; }
  // The open file and offset behind a pointer into one of the mappings (false for any other pointer): bulk
  // readers use pread on it, which copies out of the page cache without faulting the mapping in page by page.
  bool file_of(const void* p, int* fd, size_t* offset) const;
  size_t size() const { return names_.size(); }
  const std::string& name_at(size_t i) const { return names_[i]; }

 private:
  struct Shard { std::string path; const uint8_t* base = nullptr; size_t bytes = 0; int fd = -1; };
  bool map_file(const std::string& path, std::string* err);
  std::vector<Shard> shards_;
  std::map<std::string, Tensor> map_;
  std::vector<std::string> names_;
};

// Config::from_dir. Fills everything except readout_rows (the readout head is a separate file) and
// dtype (set to 1: checkpoints are bf16). Fails on a missing key or an attention_mode other than
// prefix_bidir, like the reference.
bool config_from_dir(const std::string& dir, dcd_model_config* out, std::string* err);

}  // namespace ckpt

struct dcd_checkpoint {
  ckpt::Store store;
};
