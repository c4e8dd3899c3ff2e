// BLAKE3 (unkeyed hash, 32-byte output), portable implementation.
//
// Checkpoint members and manifests are sealed with BLAKE3, as in the reference's
// checkpoint format (packages/engine/src/shadowspill/checkpoint/encoding.py:54-91),
// which takes it from the `blake3` wheel; that wheel is not a dependency here, so
// the core carries the algorithm: 64-byte blocks through the 7-round compression
// function, 1024-byte chunks, and a binary tree of chaining values merged through
// a stack (one entry per set bit of the chunk count).
#include "ss_core.h"

#include <cstring>

namespace {

constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                            0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr int PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum : uint32_t { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };
constexpr size_t BLOCK = 64, CHUNK = 1024;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
  s[a] = s[a] + s[b] + mx; s[d] = rotr(s[d] ^ s[a], 16);
  s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 12);
  s[a] = s[a] + s[b] + my; s[d] = rotr(s[d] ^ s[a], 8);
  s[c] = s[c] + s[d];      s[b] = rotr(s[b] ^ s[c], 7);
}

void compress(const uint32_t cv[8], const uint8_t block[BLOCK], uint32_t block_len,
              uint64_t counter, uint32_t flags, uint32_t out[16]) {
  uint32_t m[16];
  for (int i = 0; i < 16; ++i)
    m[i] = static_cast<uint32_t>(block[4 * i]) | (static_cast<uint32_t>(block[4 * i + 1]) << 8) |
           (static_cast<uint32_t>(block[4 * i + 2]) << 16) |
           (static_cast<uint32_t>(block[4 * i + 3]) << 24);
  uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                    IV[0], IV[1], IV[2], IV[3], static_cast<uint32_t>(counter),
                    static_cast<uint32_t>(counter >> 32), block_len, flags};
  for (int round = 0; round < 7; ++round) {
    g(s, 0, 4, 8, 12, m[0], m[1]);   g(s, 1, 5, 9, 13, m[2], m[3]);
    g(s, 2, 6, 10, 14, m[4], m[5]);  g(s, 3, 7, 11, 15, m[6], m[7]);
    g(s, 0, 5, 10, 15, m[8], m[9]);  g(s, 1, 6, 11, 12, m[10], m[11]);
    g(s, 2, 7, 8, 13, m[12], m[13]); g(s, 3, 4, 9, 14, m[14], m[15]);
    if (round < 6) {
      uint32_t p[16];
      for (int i = 0; i < 16; ++i) p[i] = m[PERM[i]];
      std::memcpy(m, p, sizeof m);
    }
  }
  for (int i = 0; i < 8; ++i) {
    out[i] = s[i] ^ s[i + 8];
    out[i + 8] = s[i + 8] ^ cv[i];
  }
}

struct Hasher {
  uint32_t chunk_cv[8];
  uint8_t block[BLOCK];
  uint32_t block_len = 0;
  uint32_t blocks_in_chunk = 0;
  uint64_t chunk_counter = 0;
  uint32_t stack[54][8];
  int stack_len = 0;

  Hasher() {
    std::memcpy(chunk_cv, IV, sizeof IV);
    std::memset(block, 0, BLOCK);
  }
  uint32_t start_flag() const { return blocks_in_chunk == 0 ? CHUNK_START : 0; }
  size_t chunk_len() const { return static_cast<size_t>(blocks_in_chunk) * BLOCK + block_len; }

  void push_chunk_cv(const uint32_t cv_in[8], uint64_t total_chunks) {
    uint32_t cv[8];
    std::memcpy(cv, cv_in, sizeof cv);
    // merge completed subtrees: one per trailing zero bit of the chunk count
    while ((total_chunks & 1) == 0) {
      uint8_t parent[BLOCK];
      std::memcpy(parent, stack[stack_len - 1], 32);
      std::memcpy(parent + 32, cv, 32);
      uint32_t out[16];
      compress(IV, parent, BLOCK, 0, PARENT, out);
      std::memcpy(cv, out, 32);
      --stack_len;
      total_chunks >>= 1;
    }
    std::memcpy(stack[stack_len++], cv, 32);
  }

  void update(const uint8_t* in, size_t len) {
    while (len > 0) {
      if (chunk_len() == CHUNK) {
        // the chunk is full and more input follows: finish it as a non-root chunk
        uint32_t out[16];
        compress(chunk_cv, block, block_len, chunk_counter, start_flag() | CHUNK_END, out);
        push_chunk_cv(out, chunk_counter + 1);
        ++chunk_counter;
        std::memcpy(chunk_cv, IV, sizeof IV);
        std::memset(block, 0, BLOCK);
        block_len = 0; blocks_in_chunk = 0;
      }
      if (block_len == BLOCK) {
        uint32_t out[16];
        compress(chunk_cv, block, BLOCK, chunk_counter, start_flag(), out);
        std::memcpy(chunk_cv, out, 32);
        ++blocks_in_chunk;
        std::memset(block, 0, BLOCK);
        block_len = 0;
        continue;
      }
      const size_t want = BLOCK - block_len;
      const size_t take = len < want ? len : want;
      std::memcpy(block + block_len, in, take);
      block_len += static_cast<uint32_t>(take);
      in += take; len -= take;
    }
  }

  void finalize(uint8_t out32[32]) {
    uint32_t out[16];
    if (stack_len == 0) {
      compress(chunk_cv, block, block_len, chunk_counter, start_flag() | CHUNK_END | ROOT, out);
    } else {
      compress(chunk_cv, block, block_len, chunk_counter, start_flag() | CHUNK_END, out);
      uint32_t cv[8];
      std::memcpy(cv, out, 32);
      for (int i = stack_len - 1; i >= 0; --i) {
        uint8_t parent[BLOCK];
        std::memcpy(parent, stack[i], 32);
        std::memcpy(parent + 32, cv, 32);
        compress(IV, parent, BLOCK, 0, PARENT | (i == 0 ? ROOT : 0), out);
        std::memcpy(cv, out, 32);
      }
    }
    for (int i = 0; i < 8; ++i) {
      out32[4 * i] = static_cast<uint8_t>(out[i]);
      out32[4 * i + 1] = static_cast<uint8_t>(out[i] >> 8);
      out32[4 * i + 2] = static_cast<uint8_t>(out[i] >> 16);
      out32[4 * i + 3] = static_cast<uint8_t>(out[i] >> 24);
    }
  }
};

}  // namespace

extern "C" {

void* ss_blake3_new(void) { return new Hasher(); }
void ss_blake3_update(void* h, const void* data, size_t len) {
  static_cast<Hasher*>(h)->update(static_cast<const uint8_t*>(data), len);
}
void ss_blake3_finalize(void* h, uint8_t* out32) {
  Hasher copy = *static_cast<Hasher*>(h);   // finalisation does not disturb the stream
  copy.finalize(out32);
}
void ss_blake3_free(void* h) { delete static_cast<Hasher*>(h); }

}  // extern "C"
