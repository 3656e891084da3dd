// Read-only view of a .safetensors file (8-byte little-endian header length, JSON
// header, raw tensor bytes), memory-mapped.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace hb {

struct StTensor {
  std::string dtype;  // "F32", "F16", "BF16", ...
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

class SafetensorsFile {
 public:
  SafetensorsFile() = default;
  ~SafetensorsFile();
  SafetensorsFile(const SafetensorsFile&) = delete;
  SafetensorsFile& operator=(const SafetensorsFile&) = delete;
  // Returns 0 or HB_ERR_IO with hb_last_error() set.
  int open(const std::string& path);
  const std::map<std::string, StTensor>& tensors() const { return tensors_; }

 private:
  void* map_ = nullptr;
  size_t size_ = 0;
  std::map<std::string, StTensor> tensors_;
};

// Sorted list of *.safetensors in dir (src/engine/loader.rs:110-126 sorts the shards).
int list_safetensors(const std::string& dir, std::vector<std::string>* out);
int read_text_file(const std::string& path, std::string* out);

}  // namespace hb
