// LZ4 block format (compress + decompress), host code. The reference compresses cached KV snapshots with LZ4
// (core/.../tensor/KvBufferCache.java:313-410); this is an independent implementation of the public block format: a sequence of
// [token: literal length (4 bits) | match length - 4 (4 bits)] [extra literal length bytes] [literals] [offset, 2 bytes little
// endian] [extra match length bytes]; the last sequence holds literals only, the last 5 bytes of the input are always literals and
// no match starts within the last 12 bytes.
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace dlv {

static inline uint32_t lz4_read32(const uint8_t* p) {
  uint32_t v;
  std::memcpy(&v, p, 4);
  return v;
}
static inline uint32_t lz4_hash(uint32_t v) { return (v * 2654435761u) >> 18; }  // 14-bit table

size_t lz4_compress_bound(size_t n) { return n + n / 255 + 16; }

size_t lz4_compress(const uint8_t* src, size_t n, uint8_t* dst, size_t cap) {
  if (cap < lz4_compress_bound(n)) throw std::runtime_error("lz4: output buffer too small");
  uint8_t* op = dst;
  size_t anchor = 0;
  if (n >= 13) {
    std::vector<uint32_t> table(1u << 14, 0xffffffffu);
    const size_t mflimit = n - 12, matchlimit = n - 5;
    size_t ip = 0;
    while (ip < mflimit) {
      const uint32_t seq = lz4_read32(src + ip);
      const uint32_t h = lz4_hash(seq);
      const uint32_t cand = table[h];
      table[h] = static_cast<uint32_t>(ip);
      if (cand == 0xffffffffu || ip - cand > 65535 || lz4_read32(src + cand) != seq) {
        ++ip;
        continue;
      }
      size_t mlen = 4;
      while (ip + mlen < matchlimit && src[cand + mlen] == src[ip + mlen]) ++mlen;
      const size_t lit = ip - anchor;
      uint8_t* token = op++;
      if (lit >= 15) {
        *token = 15u << 4;
        size_t rest = lit - 15;
        for (; rest >= 255; rest -= 255) *op++ = 255;
        *op++ = static_cast<uint8_t>(rest);
      } else {
        *token = static_cast<uint8_t>(lit << 4);
      }
      std::memcpy(op, src + anchor, lit);
      op += lit;
      const size_t off = ip - cand;
      *op++ = static_cast<uint8_t>(off & 0xff);
      *op++ = static_cast<uint8_t>(off >> 8);
      size_t ml = mlen - 4;
      if (ml >= 15) {
        *token |= 15;
        ml -= 15;
        for (; ml >= 255; ml -= 255) *op++ = 255;
        *op++ = static_cast<uint8_t>(ml);
      } else {
        *token |= static_cast<uint8_t>(ml);
      }
      ip += mlen;
      anchor = ip;
    }
  }
  const size_t lit = n - anchor;
  uint8_t* token = op++;
  if (lit >= 15) {
    *token = 15u << 4;
    size_t rest = lit - 15;
    for (; rest >= 255; rest -= 255) *op++ = 255;
    *op++ = static_cast<uint8_t>(rest);
  } else {
    *token = static_cast<uint8_t>(lit << 4);
  }
  std::memcpy(op, src + anchor, lit);
  op += lit;
  return static_cast<size_t>(op - dst);
}

// Returns the number of bytes written; throws on malformed input or when the output does not fit exactly `n_out` bytes.
size_t lz4_decompress(const uint8_t* src, size_t n, uint8_t* dst, size_t n_out) {
  size_t ip = 0, op = 0;
  while (ip < n) {
    const uint8_t token = src[ip++];
    size_t lit = token >> 4;
    if (lit == 15) {
      uint8_t b;
      do {
        if (ip >= n) throw std::runtime_error("lz4: truncated literal length");
        b = src[ip++];
        lit += b;
      } while (b == 255);
    }
    if (ip + lit > n || op + lit > n_out) throw std::runtime_error("lz4: literal run out of bounds");
    std::memcpy(dst + op, src + ip, lit);
    ip += lit;
    op += lit;
    if (ip >= n) break;  // the last sequence has no match
    if (ip + 2 > n) throw std::runtime_error("lz4: truncated offset");
    const size_t off = src[ip] | (static_cast<size_t>(src[ip + 1]) << 8);
    ip += 2;
    if (off == 0 || off > op) throw std::runtime_error("lz4: bad offset");
    size_t mlen = (token & 15);
    if (mlen == 15) {
      uint8_t b;
      do {
        if (ip >= n) throw std::runtime_error("lz4: truncated match length");
        b = src[ip++];
        mlen += b;
      } while (b == 255);
    }
    mlen += 4;
    if (op + mlen > n_out) throw std::runtime_error("lz4: match out of bounds");
    for (size_t i = 0; i < mlen; ++i) dst[op + i] = dst[op - off + i];  // byte by byte: the ranges may overlap
    op += mlen;
  }
  if (op != n_out) throw std::runtime_error("lz4: decoded size mismatch");
  return op;
}

}  // namespace dlv
