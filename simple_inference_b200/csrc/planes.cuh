// Layout of a paged cache whose keys and values differ in width (parts/base.py,
// KeyValuePlanesSpec): a page holds `rows` rows, all keys first ([kv_heads, rows, key_dim]),
// then all values ([kv_heads, rows, value_dim]).  A row is a token, or a block of tokens.
#pragma once

namespace si {

struct PlanesLayout {
  int kv_heads, rows, kd, vd;
  __device__ __forceinline__ long long page_elems() const {
    return (long long)kv_heads * rows * (kd + vd);
  }
  __device__ __forceinline__ long long key_at(int page, int g, int row) const {
    return (long long)page * page_elems() + ((long long)g * rows + row) * kd;
  }
  __device__ __forceinline__ long long value_at(int page, int g, int row) const {
    return (long long)page * page_elems() + (long long)kv_heads * rows * kd +
           ((long long)g * rows + row) * vd;
  }
};

}  // namespace si
