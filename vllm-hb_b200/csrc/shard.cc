// Tensor-parallel weight slicing on the host: the restatement of column_shard /
// row_shard (src/parallel/shard.rs:46-74), which `narrow` a [rows, cols] weight along
// dim 0 or dim 1.  Element size is a parameter so the same code slices f32/f16/bf16.
#include <cstring>

#include "common.h"

extern "C" {

int hb_column_shard(void* dst, const void* src, int64_t rows, int64_t cols, size_t elem, int rank,
                    int world_size) {
  HB_CHECK_ARG(dst && src && rows >= 0 && cols >= 0 && elem > 0, "hb_column_shard: bad arguments");
  HB_CHECK_ARG(world_size >= 1 && rank >= 0 && rank < world_size, "hb_column_shard: bad rank %d/%d",
               rank, world_size);
  if (rows % world_size != 0)
    return hb::fail(HB_ERR_NOT_DIVISIBLE,
                    "column_shard: out_features (%lld) is not divisible by world_size (%d)",
                    (long long)rows, world_size);
  const int64_t chunk = rows / world_size;
  memcpy(dst, (const char*)src + (size_t)rank * chunk * cols * elem, (size_t)chunk * cols * elem);
  return HB_OK;
}

int hb_row_shard(void* dst, const void* src, int64_t rows, int64_t cols, size_t elem, int rank,
                 int world_size) {
  HB_CHECK_ARG(dst && src && rows >= 0 && cols >= 0 && elem > 0, "hb_row_shard: bad arguments");
  HB_CHECK_ARG(world_size >= 1 && rank >= 0 && rank < world_size, "hb_row_shard: bad rank %d/%d",
               rank, world_size);
  if (cols % world_size != 0)
    return hb::fail(HB_ERR_NOT_DIVISIBLE,
                    "row_shard: in_features (%lld) is not divisible by world_size (%d)",
                    (long long)cols, world_size);
  const int64_t chunk = cols / world_size;
  for (int64_t r = 0; r < rows; ++r)
    memcpy((char*)dst + (size_t)r * chunk * elem,
           (const char*)src + ((size_t)r * cols + (size_t)rank * chunk) * elem, (size_t)chunk * elem);
  return HB_OK;
}

}  // extern "C"
