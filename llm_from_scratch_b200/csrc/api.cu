// Library-level entry points: ABI version, error strings, the device status word, and the host-side
// XXH64 used for prefix-cache block hashes.
#include <string.h>

#include "common.cuh"

namespace b200 {

int sm_count_cached() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

// XXH64 (Yann Collet's public specification, seedable, little-endian reads).
constexpr uint64_t P1 = 0x9E3779B185EBCA87ull;
constexpr uint64_t P2 = 0xC2B2AE3D27D4EB4Full;
constexpr uint64_t P3 = 0x165667B19E3779F9ull;
constexpr uint64_t P4 = 0x85EBCA77C2B2AE63ull;
constexpr uint64_t P5 = 0x27D4EB2F165667C5ull;

inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t rd64(const uint8_t* p) {
  uint64_t v;
  memcpy(&v, p, 8);
  return v;  // x86-64 / aarch64 little-endian hosts
}
inline uint32_t rd32(const uint8_t* p) {
  uint32_t v;
  memcpy(&v, p, 4);
  return v;
}
inline uint64_t xround(uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; }
inline uint64_t xmerge(uint64_t acc, uint64_t v) { return (acc ^ xround(0, v)) * P1 + P4; }

// Streaming state so that the prefix hash and the token bytes need no concatenation buffer.
struct Xxh64 {
  uint64_t v[4];
  uint8_t buf[32];
  size_t buffered = 0;
  uint64_t total = 0;
  uint64_t seed;
  explicit Xxh64(uint64_t s) : seed(s) {
    v[0] = s + P1 + P2;
    v[1] = s + P2;
    v[2] = s;
    v[3] = s - P1;
  }
  void stripe(const uint8_t* p) {
    for (int i = 0; i < 4; ++i) v[i] = xround(v[i], rd64(p + 8 * i));
  }
  void update(const void* data, size_t len) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    total += len;
    if (buffered) {
      size_t take = 32 - buffered < len ? 32 - buffered : len;
      memcpy(buf + buffered, p, take);
      buffered += take;
      p += take;
      len -= take;
      if (buffered < 32) return;
      stripe(buf);
      buffered = 0;
    }
    while (len >= 32) {
      stripe(p);
      p += 32;
      len -= 32;
    }
    if (len) {
      memcpy(buf, p, len);
      buffered = len;
    }
  }
  uint64_t digest() const {
    uint64_t h;
    if (total >= 32) {
      h = rotl(v[0], 1) + rotl(v[1], 7) + rotl(v[2], 12) + rotl(v[3], 18);
      for (int i = 0; i < 4; ++i) h = xmerge(h, v[i]);
    } else {
      h = seed + P5;
    }
    h += total;
    const uint8_t* p = buf;
    size_t len = buffered;
    while (len >= 8) {
      h ^= xround(0, rd64(p));
      h = rotl(h, 27) * P1 + P4;
      p += 8;
      len -= 8;
    }
    if (len >= 4) {
      h ^= static_cast<uint64_t>(rd32(p)) * P1;
      h = rotl(h, 23) * P2 + P3;
      p += 4;
      len -= 4;
    }
    while (len) {
      h ^= static_cast<uint64_t>(*p) * P5;
      h = rotl(h, 11) * P1;
      ++p;
      --len;
    }
    h ^= h >> 33;
    h *= P2;
    h ^= h >> 29;
    h *= P3;
    h ^= h >> 32;
    return h;
  }
};

}  // namespace
}  // namespace b200

extern "C" {

int b200_abi_version(void) { return B200_ABI_VERSION; }

const char* b200_strerror(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_ARG: return "invalid argument";
    case B200_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
    case B200_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case B200_ERR_LAUNCH: return "CUDA launch failed";
    case B200_ERR_WORKSPACE: return "workspace too small";
    case B200_ERR_BOUNDS: return "block id or slot outside the pool (access skipped)";
    case B200_ERR_NO_DEVICE: return "no usable CUDA device";
    case B200_ERR_TOO_LARGE: return "problem needs more scratch than the built-in static array holds";
    case B200_ERR_TIMEOUT: return "a bounded device-side barrier wait gave up (kernel aborted cleanly)";
    default: return "unknown error";
  }
}

int b200_sm_count(void) {
  int n = b200::sm_count_cached();
  return n > 0 ? n : B200_ERR_NO_DEVICE;
}

int b200_read_status(int32_t* status, int32_t* status_host, void* stream) {
  if (status == nullptr || status_host == nullptr) return B200_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(status_host, status, sizeof(int32_t), cudaMemcpyDeviceToHost, s) !=
      cudaSuccess)
    return B200_ERR_LAUNCH;
  if (cudaMemsetAsync(status, 0, sizeof(int32_t), s) != cudaSuccess) return B200_ERR_LAUNCH;
  if (cudaStreamSynchronize(s) != cudaSuccess) return B200_ERR_LAUNCH;
  return B200_OK;
}

uint64_t b200_xxh64(const void* data_host, size_t len, uint64_t seed) {
  b200::Xxh64 h(seed);
  if (len) h.update(data_host, len);
  return h.digest();
}

uint64_t b200_block_hash(const int32_t* token_ids_host, int32_t num_tokens, uint64_t prefix_hash,
                         int32_t has_prefix) {
  b200::Xxh64 h(0);
  if (has_prefix) {
    uint64_t p = prefix_hash;
    h.update(&p, 8);
  }
  if (num_tokens > 0) h.update(token_ids_host, static_cast<size_t>(num_tokens) * 4);
  return h.digest();
}

// Chained hashes of every full block of a token list: out[i] = XXH64([out[i-1] if i > 0] || ids of block i),
// the values BlockManager.allocate computes block by block (engine/block_manager.py:85-101).
int64_t b200_block_hash_chain(const int32_t* token_ids_host, int64_t num_tokens, int32_t block_size,
                              uint64_t* out_hashes) {
  if (num_tokens < 0 || block_size <= 0 || (num_tokens > 0 && !token_ids_host)) return -1;
  const int64_t full = num_tokens / block_size;
  if (full > 0 && !out_hashes) return -1;
  uint64_t prev = 0;
  for (int64_t i = 0; i < full; ++i) {
    b200::Xxh64 h(0);
    if (i > 0) h.update(&prev, 8);
    h.update(token_ids_host + i * block_size, static_cast<size_t>(block_size) * 4);
    prev = h.digest();
    out_hashes[i] = prev;
  }
  return full;
}

}  // extern "C"
