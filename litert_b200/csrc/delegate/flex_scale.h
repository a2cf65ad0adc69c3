// Minimal reader for the attribute blob of the SDPA composite: a FlexBuffers
// map whose "scale" (and optional "logit_cap") entries are floats
// (tflite/experimental/genai/sdpa.cc:99-105 reads "scale" through the
// flexbuffers library; tflite/delegates/xnnpack/xnnpack_delegate.cc:6393-6398
// also reads "logit_cap"). Only what that lookup needs is decoded: a root map
// with scalar values. Every offset is bounds-checked; a malformed blob makes
// the lookup fail, never read out of range.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>

namespace b200 {

namespace flex_detail {
inline bool ReadUInt(const uint8_t* buf, size_t size, size_t pos, size_t width, uint64_t* out) {
  if (width != 1 && width != 2 && width != 4 && width != 8) return false;
  if (pos > size || size - pos < width) return false;
  uint64_t v = 0;
  memcpy(&v, buf + pos, width);  // little endian
  *out = v;
  return true;
}
inline bool ReadFloat(const uint8_t* buf, size_t size, size_t pos, size_t width, float* out) {
  if (pos > size || size - pos < width) return false;
  if (width == 4) {
    memcpy(out, buf + pos, 4);
    return true;
  }
  if (width == 8) {
    double d;
    memcpy(&d, buf + pos, 8);
    *out = static_cast<float>(d);
    return true;
  }
  return false;
}
}  // namespace flex_detail

// FlexBuffers type codes used here.
enum : int { kFlexInt = 1, kFlexUInt = 2, kFlexFloat = 3, kFlexIndirectInt = 6, kFlexIndirectUInt = 7,
             kFlexIndirectFloat = 8, kFlexMap = 9 };

// Looks `key` up in a root map and converts its value to float. Returns false
// (and leaves *out alone) when the blob is empty, not a map, or has no such key.
inline bool FlexMapFloat(const uint8_t* buf, size_t size, const char* key, float* out) {
  using namespace flex_detail;
  if (!buf || size < 3) return false;
  const size_t root_width = buf[size - 1];
  const uint8_t packed = buf[size - 2];
  if ((packed >> 2) != kFlexMap) return false;
  if (root_width == 0 || size < 2 + root_width) return false;
  const size_t root_pos = size - 2 - root_width;
  uint64_t off;
  if (!ReadUInt(buf, size, root_pos, root_width, &off) || off > root_pos) return false;
  const size_t map_pos = root_pos - off;          // start of the values vector
  const size_t bw = size_t(1) << (packed & 3);    // element width of that vector
  if (map_pos < 3 * bw) return false;
  uint64_t n, keys_off, keys_bw;
  if (!ReadUInt(buf, size, map_pos - bw, bw, &n)) return false;
  if (!ReadUInt(buf, size, map_pos - 3 * bw, bw, &keys_off) || keys_off > map_pos - 3 * bw) return false;
  if (!ReadUInt(buf, size, map_pos - 2 * bw, bw, &keys_bw)) return false;
  const size_t keys_pos = map_pos - 3 * bw - keys_off;
  if (n > size) return false;
  const size_t key_len = strlen(key);
  for (uint64_t i = 0; i < n; ++i) {
    const size_t kpos = keys_pos + i * keys_bw;
    uint64_t koff;
    if (!ReadUInt(buf, size, kpos, keys_bw, &koff) || koff > kpos) return false;
    const size_t spos = kpos - koff;
    if (spos + key_len + 1 > size) continue;
    if (memcmp(buf + spos, key, key_len) != 0 || buf[spos + key_len] != 0) continue;
    const size_t vpos = map_pos + i * bw;
    const size_t tpos = map_pos + n * bw + i;
    if (tpos >= size) return false;
    const int vtype = buf[tpos] >> 2;
    const size_t vbw = size_t(1) << (buf[tpos] & 3);
    uint64_t u;
    switch (vtype) {
      case kFlexFloat:
        return ReadFloat(buf, size, vpos, bw, out);
      case kFlexIndirectFloat:
        if (!ReadUInt(buf, size, vpos, bw, &u) || u > vpos) return false;
        return ReadFloat(buf, size, vpos - u, vbw, out);
      case kFlexInt: {
        if (!ReadUInt(buf, size, vpos, bw, &u)) return false;
        int64_t s = static_cast<int64_t>(u << (64 - 8 * bw)) >> (64 - 8 * bw);
        *out = static_cast<float>(s);
        return true;
      }
      case kFlexUInt:
        if (!ReadUInt(buf, size, vpos, bw, &u)) return false;
        *out = static_cast<float>(u);
        return true;
      default:
        return false;
    }
  }
  return false;
}

}  // namespace b200
