// 64-bit string hashes used by the feature engine, usable from host and device code.
//   * FarmHash Fingerprint64 (farmhashna::Hash64, Google, MIT licence): stable across platforms and releases.
//   * MurmurHash64A with seed 0 as used by TensorFlow's strong-hash-free string bucketing.
// The results are bit-identical to the reference's fused hash op (csrc/ops/fused_hash_kernel.cu:47-459), so ids produced
// by either implementation address the same embedding rows.
#pragma once
#include <stdint.h>
#include <string.h>
#include <cuda_runtime.h>

namespace rb {
namespace hash {

#define RB_HD __host__ __device__ __forceinline__

RB_HD uint64_t fetch64(const char* p) { uint64_t r; memcpy(&r, p, 8); return r; }
RB_HD uint32_t fetch32(const char* p) { uint32_t r; memcpy(&r, p, 4); return r; }
RB_HD uint64_t rot(uint64_t v, int s) { return s == 0 ? v : ((v >> s) | (v << (64 - s))); }
RB_HD uint64_t shift_mix(uint64_t v) { return v ^ (v >> 47); }

constexpr uint64_t kF0 = 0xc3a5c85c97cb3127ull;
constexpr uint64_t kF1 = 0xb492b66fbe98f273ull;
constexpr uint64_t kF2 = 0x9ae16a3b2f90404full;

RB_HD uint64_t hash_len16(uint64_t u, uint64_t v, uint64_t mul) {
  uint64_t a = (u ^ v) * mul; a ^= (a >> 47);
  uint64_t b = (v ^ a) * mul; b ^= (b >> 47);
  return b * mul;
}

RB_HD uint64_t farm_0to16(const char* s, size_t len) {
  if (len >= 8) {
    const uint64_t mul = kF2 + len * 2;
    const uint64_t a = fetch64(s) + kF2, b = fetch64(s + len - 8);
    const uint64_t c = rot(b, 37) * mul + a, d = (rot(a, 25) + b) * mul;
    return hash_len16(c, d, mul);
  }
  if (len >= 4) {
    const uint64_t mul = kF2 + len * 2;
    const uint64_t a = fetch32(s);
    return hash_len16(len + (a << 3), fetch32(s + len - 4), mul);
  }
  if (len > 0) {
    const uint8_t a = (uint8_t)s[0], b = (uint8_t)s[len >> 1], c = (uint8_t)s[len - 1];
    const uint32_t y = (uint32_t)a + ((uint32_t)b << 8);
    const uint32_t z = (uint32_t)len + ((uint32_t)c << 2);
    return shift_mix(y * kF2 ^ z * kF0) * kF2;
  }
  return kF2;
}

RB_HD uint64_t farm_17to32(const char* s, size_t len) {
  const uint64_t mul = kF2 + len * 2;
  const uint64_t a = fetch64(s) * kF1, b = fetch64(s + 8);
  const uint64_t c = fetch64(s + len - 8) * mul, d = fetch64(s + len - 16) * kF2;
  return hash_len16(rot(a + b, 43) + rot(c, 30) + d, a + rot(b + kF2, 18) + c, mul);
}

struct U128 { uint64_t first, second; };

RB_HD U128 weak32(uint64_t w, uint64_t x, uint64_t y, uint64_t z, uint64_t a, uint64_t b) {
  a += w;
  b = rot(b + a + z, 21);
  const uint64_t c = a;
  a += x; a += y;
  b += rot(a, 44);
  return U128{a + z, b + c};
}
RB_HD U128 weak32(const char* s, uint64_t a, uint64_t b) {
  return weak32(fetch64(s), fetch64(s + 8), fetch64(s + 16), fetch64(s + 24), a, b);
}

RB_HD uint64_t farm_33to64(const char* s, size_t len) {
  const uint64_t mul = kF2 + len * 2;
  const uint64_t a = fetch64(s) * kF2, b = fetch64(s + 8);
  const uint64_t c = fetch64(s + len - 8) * mul, d = fetch64(s + len - 16) * kF2;
  const uint64_t y = rot(a + b, 43) + rot(c, 30) + d;
  const uint64_t z = hash_len16(y, a + rot(b + kF2, 18) + c, mul);
  const uint64_t e = fetch64(s + 16) * mul, f = fetch64(s + 24);
  const uint64_t g = (y + fetch64(s + len - 32)) * mul, h = (z + fetch64(s + len - 24)) * mul;
  return hash_len16(rot(e + f, 43) + rot(g, 30) + h, e + rot(f + a, 18) + g, mul);
}

RB_HD uint64_t farm_fingerprint64(const char* s, size_t len) {
  if (len <= 32) return len <= 16 ? farm_0to16(s, len) : farm_17to32(s, len);
  if (len <= 64) return farm_33to64(s, len);
  const uint64_t seed = 81;
  uint64_t x = seed, y = seed * kF1 + 113, z = shift_mix(y * kF2 + 113) * kF2;
  U128 v{0, 0}, w{0, 0};
  x = x * kF2 + fetch64(s);
  const char* end = s + ((len - 1) / 64) * 64;
  const char* last64 = end + ((len - 1) & 63) - 63;
  do {
    x = rot(x + y + v.first + fetch64(s + 8), 37) * kF1;
    y = rot(y + v.second + fetch64(s + 48), 42) * kF1;
    x ^= w.second;
    y += v.first + fetch64(s + 40);
    z = rot(z + w.first, 33) * kF1;
    v = weak32(s, v.second * kF1, x + w.first);
    w = weak32(s + 32, z + w.second, y + fetch64(s + 16));
    const uint64_t t = z; z = x; x = t;
    s += 64;
  } while (s != end);
  const uint64_t mul = kF1 + ((z & 0xff) << 1);
  s = last64;
  w.first += ((len - 1) & 63);
  v.first += w.first;
  w.first += v.first;
  x = rot(x + y + v.first + fetch64(s + 8), 37) * mul;
  y = rot(y + v.second + fetch64(s + 48), 42) * mul;
  x ^= w.second * 9;
  y += v.first * 9 + fetch64(s + 40);
  z = rot(z + w.first, 33) * mul;
  v = weak32(s, v.second * mul, x + w.first);
  w = weak32(s + 32, z + w.second, y + fetch64(s + 16));
  const uint64_t t = z; z = x; x = t;
  return hash_len16(hash_len16(v.first, w.first, mul) + shift_mix(y) * kF0 + z, hash_len16(v.second, w.second, mul) + x, mul);
}

RB_HD uint64_t murmur64a(const char* data, size_t n, uint64_t seed) {
  const uint64_t m = 0xc6a4a7935bd1e995ull;
  const int r = 47;
  uint64_t h = seed ^ (n * m);
  while (n >= 8) {
    uint64_t k = fetch64(data);
    data += 8; n -= 8;
    k *= m; k ^= k >> r; k *= m;
    h ^= k; h *= m;
  }
  uint64_t tail = 0;
  for (size_t i = 0; i < n; ++i) tail |= ((uint64_t)(uint8_t)data[i]) << (8 * i);
  if (n > 0) { h ^= tail; h *= m; }
  h ^= h >> r; h *= m; h ^= h >> r;
  return h;
}

// 64-bit mix of a pair of ids (feature crosses): murmur-style combine of the two 8-byte words.
RB_HD uint64_t murmur_pair(uint64_t x, uint64_t y) {
  char buf[16];
  memcpy(buf, &x, 8); memcpy(buf + 8, &y, 8);
  return murmur64a(buf, 16, 0);
}

#undef RB_HD
}  // namespace hash
}  // namespace rb
