// block_id.hpp — the 64-bit KV block-ID protocol and its registry (host only).
//
// Same function, value for value, as the reference's kv_hash_ids / kv_hash_text /
// kv_hash_hex / kv_block_id (code/graph/kv_block.h:21-83) and BlockRegistry
// (code/graph/kv_registry.h:26-66).
//
// The reference spells the hash out through strings: ids -> decimal text -> the
// hex digits of that text's bytes -> groups of 16 hex digits read as big-endian
// 64-bit words, the last group padded with '0' digits -> fold.  Sixteen hex
// digits are eight bytes, so the words are simply the decimal text taken eight
// bytes at a time, big-endian, zero-padded on the right; no hex string is built
// here.  The fold adds word i to word n-1-i (mod 2^64), keeps an odd middle word,
// and repeats until one word is left.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace novab {

class DigestWords {
public:
    void push_byte(unsigned char c) {
        cur_ = (cur_ << 8) | (uint64_t)c;
        if (++fill_ == 8) flush();
    }
    void push_decimal(int32_t v) {
        // std::to_string semantics: optional '-', then digits without padding.
        char buf[12];
        int n = 0;
        uint32_t mag = v < 0 ? (uint32_t)(-(int64_t)v) : (uint32_t)v;
        do { buf[n++] = (char)('0' + mag % 10u); mag /= 10u; } while (mag);
        if (v < 0) push_byte('-');
        while (n) push_byte((unsigned char)buf[--n]);
    }
    uint64_t fold() {
        if (fill_) { cur_ <<= 8 * (8 - fill_); flush(); }
        if (words_.empty()) return 0;
        size_t n = words_.size();
        while (n > 1) {
            const size_t half = n / 2;
            for (size_t i = 0; i < half; ++i) words_[i] += words_[n - 1 - i];
            // an odd middle word already sits at index `half`
            n = half + (n & 1);
        }
        return words_[0];
    }
private:
    void flush() { words_.push_back(cur_); cur_ = 0; fill_ = 0; }
    std::vector<uint64_t> words_;
    uint64_t cur_ = 0;
    int fill_ = 0;
};

inline uint64_t hash_ids(const int32_t* ids, size_t n) {
    DigestWords d;
    for (size_t i = 0; i < n; ++i) d.push_decimal(ids[i]);
    return d.fold();
}

// kv_hash_text feeds every byte through the id path, i.e. as its decimal value
// 0..255 ("abc" -> "979899"), not as the raw byte.
inline uint64_t hash_text(const char* bytes, size_t n) {
    DigestWords d;
    for (size_t i = 0; i < n; ++i) d.push_decimal((int32_t)(unsigned char)bytes[i]);
    return d.fold();
}

inline void hash_hex(uint64_t v, char* out17) {
    static const char digits[] = "0123456789ABCDEF";
    for (int i = 0; i < 16; ++i) out17[i] = digits[(v >> (60 - 4 * i)) & 15u];
    out17[16] = '\0';
}

inline void block_id(uint64_t prefix, uint64_t suffix, char* out40) {
    // "{ " + 16 + " . " + 16 + " }" = 2 + 16 + 3 + 16 + 2 = 39 characters
    out40[0] = '{'; out40[1] = ' ';
    hash_hex(prefix, out40 + 2);
    out40[18] = ' '; out40[19] = '.'; out40[20] = ' ';
    hash_hex(suffix, out40 + 21);
    out40[37] = ' '; out40[38] = '}'; out40[39] = '\0';
}

struct BlockEntry {
    uint64_t prefix = 0, suffix = 0;
    int32_t session = -1, turn = 0;
    int64_t pos0 = 0, pos1 = 0;
    bool alive = true;
};

// Append-only list with tombstones: an entry with the same (prefix, suffix) as a
// new one is retired first; beyond the capacity the oldest live entries are retired.
class BlockRegistry {
public:
    void set_capacity(size_t n) { cap_ = n ? n : 1; trim(); }
    size_t capacity() const { return cap_; }
    void put(const BlockEntry& b) {
        for (auto& x : items_)
            if (x.alive && x.prefix == b.prefix && x.suffix == b.suffix) x.alive = false;
        items_.push_back(b);
        trim();
    }
    const BlockEntry* find(uint64_t prefix, uint64_t suffix) const {
        for (const auto& x : items_)
            if (x.alive && x.prefix == prefix && x.suffix == suffix) return &x;
        return nullptr;
    }
    int live() const {
        int n = 0;
        for (const auto& x : items_) n += x.alive ? 1 : 0;
        return n;
    }
    int total() const { return (int)items_.size(); }
private:
    void trim() {
        size_t alive = (size_t)live();
        for (auto& x : items_) {
            if (alive <= cap_) break;
            if (x.alive) { x.alive = false; --alive; }
        }
    }
    std::vector<BlockEntry> items_;
    size_t cap_ = 64;
};

}  // namespace novab
