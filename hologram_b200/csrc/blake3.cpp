#include "blake3.h"

#include <string.h>

#include <thread>
#include <vector>

namespace {

const uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
const uint8_t PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum { CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8 };

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
inline void g(uint32_t* v, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    v[a] = v[a] + v[b] + mx;
    v[d] = rotr(v[d] ^ v[a], 16);
    v[c] = v[c] + v[d];
    v[b] = rotr(v[b] ^ v[c], 12);
    v[a] = v[a] + v[b] + my;
    v[d] = rotr(v[d] ^ v[a], 8);
    v[c] = v[c] + v[d];
    v[b] = rotr(v[b] ^ v[c], 7);
}

// Compression function; writes the 8-word chaining value of the result to out_cv.
void compress(const uint32_t cv[8], const uint8_t block[64], uint64_t counter, uint32_t block_len, uint32_t flags,
              uint32_t out_cv[8]) {
    uint32_t m[16], v[16];
    for (int i = 0; i < 16; ++i)
        m[i] = (uint32_t)block[4 * i] | ((uint32_t)block[4 * i + 1] << 8) | ((uint32_t)block[4 * i + 2] << 16) |
               ((uint32_t)block[4 * i + 3] << 24);
    for (int i = 0; i < 8; ++i) v[i] = cv[i];
    for (int i = 0; i < 4; ++i) v[8 + i] = IV[i];
    v[12] = (uint32_t)counter;
    v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len;
    v[15] = flags;
    for (int r = 0; r < 7; ++r) {
        g(v, 0, 4, 8, 12, m[0], m[1]);
        g(v, 1, 5, 9, 13, m[2], m[3]);
        g(v, 2, 6, 10, 14, m[4], m[5]);
        g(v, 3, 7, 11, 15, m[6], m[7]);
        g(v, 0, 5, 10, 15, m[8], m[9]);
        g(v, 1, 6, 11, 12, m[10], m[11]);
        g(v, 2, 7, 8, 13, m[12], m[13]);
        g(v, 3, 4, 9, 14, m[14], m[15]);
        uint32_t t[16];
        for (int i = 0; i < 16; ++i) t[i] = m[PERM[i]];
        memcpy(m, t, sizeof m);
    }
    for (int i = 0; i < 8; ++i) out_cv[i] = v[i] ^ v[i + 8];
}

// Chaining value of one whole (non-root) or final chunk.
void chunk_cv(const uint8_t* data, size_t len, uint64_t chunk_index, uint32_t extra_flags, uint32_t out[8]) {
    uint32_t cv[8];
    memcpy(cv, IV, sizeof cv);
    size_t nblocks = len == 0 ? 1 : (len + 63) / 64;
    for (size_t b = 0; b < nblocks; ++b) {
        uint8_t block[64] = {0};
        size_t off = b * 64, blen = len - off < 64 ? len - off : 64;
        if (len == 0) blen = 0;
        memcpy(block, data + off, blen);
        uint32_t flags = 0;
        if (b == 0) flags |= CHUNK_START;
        if (b == nblocks - 1) flags |= CHUNK_END | extra_flags;
        uint32_t next[8];
        compress(cv, block, chunk_index, (uint32_t)blen, flags, next);
        memcpy(cv, next, sizeof cv);
    }
    memcpy(out, cv, sizeof cv);
}

void parent_cv(const uint32_t left[8], const uint32_t right[8], uint32_t extra_flags, uint32_t out[8]) {
    uint8_t block[64];
    for (int i = 0; i < 8; ++i)
        for (int b = 0; b < 4; ++b) {
            block[4 * i + b] = (uint8_t)(left[i] >> (8 * b));
            block[32 + 4 * i + b] = (uint8_t)(right[i] >> (8 * b));
        }
    compress(IV, block, 0, 64, PARENT | extra_flags, out);
}



// Chaining value of a block of 2^k whole chunks starting at chunk `first` (a complete subtree).
void subtree_cv(const uint8_t* data, size_t nchunks, uint64_t first, uint32_t out[8]) {
    uint32_t stack[32][8];
    int depth = 0;
    for (size_t i = 0; i < nchunks; ++i) {
        uint32_t cv[8];
        chunk_cv(data + i * 1024, 1024, first + i, 0, cv);
        size_t total = i + 1;
        while ((total & 1) == 0) {
            uint32_t merged[8];
            parent_cv(stack[depth - 1], cv, 0, merged);
            memcpy(cv, merged, sizeof cv);
            --depth;
            total >>= 1;
        }
        memcpy(stack[depth++], cv, sizeof cv);
    }
    memcpy(out, stack[0], 8 * sizeof(uint32_t));
}

}  // namespace

void holo_blake3(const uint8_t* data, size_t len, uint8_t out[32]) {
    uint32_t result[8];
    const size_t CHUNK = 1024, BLOCK_CHUNKS = 1024;  // 1 MiB complete subtrees, hashed in parallel
    size_t nchunks = len == 0 ? 1 : (len + CHUNK - 1) / CHUNK;
    if (nchunks == 1) {
        chunk_cv(data, len, 0, ROOT, result);
    } else {
        // Left-to-right merge with a stack of subtree chaining values: whenever the count of
        // completed chunks has trailing zero bits, the top subtrees of equal size are merged.
        // The last chunk is held back so that the final merges can carry the ROOT flag. Whole
        // 1 MiB blocks in front of it are complete subtrees and are hashed by worker threads.
        const size_t nblocks = (nchunks - 1) / BLOCK_CHUNKS;
        std::vector<uint32_t> block_cvs(nblocks * 8);
        if (nblocks > 0) {
            unsigned hw = std::thread::hardware_concurrency();
            size_t nthreads = hw == 0 ? 4 : hw;
            if (nthreads > 32) nthreads = 32;
            if (nthreads > nblocks) nthreads = nblocks;
            std::vector<std::thread> pool;
            for (size_t t = 0; t < nthreads; ++t)
                pool.emplace_back([&, t]() {
                    for (size_t b = t; b < nblocks; b += nthreads)
                        subtree_cv(data + b * BLOCK_CHUNKS * CHUNK, BLOCK_CHUNKS, b * BLOCK_CHUNKS, &block_cvs[b * 8]);
                });
            for (auto& th : pool) th.join();
        }
        uint32_t stack[64][8];
        int depth = 0;
        auto push = [&](uint32_t* cv, size_t total_chunks, size_t unit) {
            size_t total = total_chunks / unit;
            while ((total & 1) == 0) {
                uint32_t merged[8];
                parent_cv(stack[depth - 1], cv, 0, merged);
                memcpy(cv, merged, 8 * sizeof(uint32_t));
                --depth;
                total >>= 1;
            }
            memcpy(stack[depth++], cv, 8 * sizeof(uint32_t));
        };
        for (size_t b = 0; b < nblocks; ++b) {
            uint32_t cv[8];
            memcpy(cv, &block_cvs[b * 8], sizeof cv);
            push(cv, (b + 1) * BLOCK_CHUNKS, BLOCK_CHUNKS);
        }
        for (size_t i = nblocks * BLOCK_CHUNKS; i + 1 < nchunks; ++i) {
            uint32_t cv[8];
            chunk_cv(data + i * CHUNK, CHUNK, i, 0, cv);
            push(cv, i + 1, 1);
        }
        uint32_t cv[8];
        size_t last = nchunks - 1;
        chunk_cv(data + last * CHUNK, len - last * CHUNK, last, 0, cv);
        while (depth > 0) {
            uint32_t merged[8];
            parent_cv(stack[depth - 1], cv, depth == 1 ? ROOT : 0, merged);
            memcpy(cv, merged, sizeof cv);
            --depth;
        }
        memcpy(result, cv, sizeof result);
    }
    for (int i = 0; i < 8; ++i)
        for (int b = 0; b < 4; ++b) out[4 * i + b] = (uint8_t)(result[i] >> (8 * b));
}
