#include "safetensors.h"

#include <dirent.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>

#include "common.h"
#include "json.h"

namespace hb {

// A JSON number that is a non-negative integer small enough to be exact in a double.
static bool as_index(const Json& j, uint64_t* out) {
  if (j.kind != Json::Num) return false;
  const double v = j.num;
  if (!(v >= 0.0) || v > 9007199254740992.0 || v != (double)(uint64_t)v) return false;
  *out = (uint64_t)v;
  return true;
}

static size_t st_elem_size(const std::string& dt) {
  if (dt == "F64" || dt == "I64" || dt == "U64") return 8;
  if (dt == "F32" || dt == "I32" || dt == "U32") return 4;
  if (dt == "F16" || dt == "BF16" || dt == "I16" || dt == "U16") return 2;
  if (dt == "I8" || dt == "U8" || dt == "BOOL" || dt == "F8_E4M3" || dt == "F8_E5M2") return 1;
  return 0;  // unknown: the size cannot be checked here
}

SafetensorsFile::~SafetensorsFile() {
  if (map_) munmap(map_, size_);
}

int SafetensorsFile::open(const std::string& path) {
  int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return fail(HB_ERR_IO, "cannot open %s", path.c_str());
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    return fail(HB_ERR_IO, "%s is too short for a safetensors file", path.c_str());
  }
  size_ = (size_t)st.st_size;
  map_ = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (map_ == MAP_FAILED) {
    map_ = nullptr;
    return fail(HB_ERR_IO, "mmap of %s failed", path.c_str());
  }
  const uint8_t* base = (const uint8_t*)map_;
  uint64_t hlen = 0;
  memcpy(&hlen, base, 8);
  if (hlen > size_ - 8) return fail(HB_ERR_IO, "%s: header length %llu exceeds the file", path.c_str(),
                                    (unsigned long long)hlen);
  Json root;
  std::string err;
  JsonParser parser((const char*)base + 8, (size_t)hlen);
  if (!parser.parse(&root, &err) || root.kind != Json::Obj)
    return fail(HB_ERR_IO, "%s: bad header: %s", path.c_str(), err.c_str());
  const uint8_t* data0 = base + 8 + hlen;
  const size_t data_len = size_ - 8 - (size_t)hlen;
  for (auto& kv : root.obj) {
    if (kv.first == "__metadata__") continue;
    const Json& t = kv.second;
    const Json* dt = t.get("dtype");
    const Json* sh = t.get("shape");
    const Json* off = t.get("data_offsets");
    if (!dt || !sh || !off || dt->kind != Json::Str || sh->kind != Json::Arr || off->kind != Json::Arr ||
        off->arr.size() != 2)
      return fail(HB_ERR_IO, "%s: tensor %s has a malformed entry", path.c_str(), kv.first.c_str());
    StTensor st_t;
    st_t.dtype = dt->str;
    uint64_t numel = 1;
    for (auto& d : sh->arr) {
      uint64_t v = 0;
      if (!as_index(d, &v) || (v != 0 && numel > (1ull << 53) / v))
        return fail(HB_ERR_IO, "%s: tensor %s has a bad shape entry", path.c_str(), kv.first.c_str());
      numel *= v;
      st_t.shape.push_back((int64_t)v);
    }
    uint64_t b = 0, e = 0;
    if (!as_index(off->arr[0], &b) || !as_index(off->arr[1], &e))
      return fail(HB_ERR_IO, "%s: tensor %s has bad data_offsets", path.c_str(), kv.first.c_str());
    if (e < b || e > data_len)
      return fail(HB_ERR_IO, "%s: tensor %s points outside the file", path.c_str(), kv.first.c_str());
    const size_t es = st_elem_size(st_t.dtype);
    if (es && (e - b) != numel * es)
      return fail(HB_ERR_IO, "%s: tensor %s holds %llu bytes, its shape and dtype %s need %llu", path.c_str(),
                  kv.first.c_str(), (unsigned long long)(e - b), st_t.dtype.c_str(),
                  (unsigned long long)(numel * es));
    st_t.data = data0 + b;
    st_t.nbytes = e - b;
    tensors_[kv.first] = std::move(st_t);
  }
  return HB_OK;
}

int list_safetensors(const std::string& dir, std::vector<std::string>* out) {
  DIR* d = opendir(dir.c_str());
  if (!d) return fail(HB_ERR_IO, "cannot open model directory %s", dir.c_str());
  out->clear();
  while (dirent* e = readdir(d)) {
    std::string n = e->d_name;
    const std::string suf = ".safetensors";
    if (n.size() > suf.size() && n.compare(n.size() - suf.size(), suf.size(), suf) == 0)
      out->push_back(dir + "/" + n);
  }
  closedir(d);
  std::sort(out->begin(), out->end());
  if (out->empty()) return fail(HB_ERR_IO, "no .safetensors files in %s", dir.c_str());
  return HB_OK;
}

int read_text_file(const std::string& path, std::string* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return fail(HB_ERR_IO, "cannot read %s", path.c_str());
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  return HB_OK;
}

}  // namespace hb
