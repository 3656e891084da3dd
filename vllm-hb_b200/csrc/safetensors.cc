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
    if (!dt || !sh || !off || off->arr.size() != 2)
      return fail(HB_ERR_IO, "%s: tensor %s has a malformed entry", path.c_str(), kv.first.c_str());
    StTensor st_t;
    st_t.dtype = dt->str;
    for (auto& d : sh->arr) st_t.shape.push_back((int64_t)d.num);
    const size_t b = (size_t)off->arr[0].num, e = (size_t)off->arr[1].num;
    if (e < b || e > data_len)
      return fail(HB_ERR_IO, "%s: tensor %s points outside the file", path.c_str(), kv.first.c_str());
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
