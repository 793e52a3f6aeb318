/* Stand-in for the vendored hash header that lilong555/mini-llm-runtime's CUDA storage
 * includes (src/minillm/cuda/storage.cpp:7, `hash/sha256/sha256.h`; its third_party/ tree is
 * not part of the checkout this build works from).  The reference only records the digest in
 * its weight manifest; nothing of the forward pass reads it.  This stand-in keeps the three
 * functions' names and shapes and fills the 32 bytes with four 64-bit FNV-1a sums: NOT
 * SHA-256, and not used for anything but that manifest field. */
#pragma once

#include <stddef.h>
#include <stdint.h>

typedef struct {
    uint64_t lane[4];
} sha256_t;

static inline void sha256_init(sha256_t* state) {
    for (int i = 0; i < 4; ++i) state->lane[i] = 0xCBF29CE484222325ull + (uint64_t)i * 0x9E3779B97F4A7C15ull;
}

static inline void sha256_update(sha256_t* state, const unsigned char* data, size_t size) {
    /* eight bytes at a time, one lane after the other: fast enough for gigabytes of weights */
    size_t i = 0;
    for (; i + 8 <= size; i += 8) {
        uint64_t word = 0;
        for (int b = 0; b < 8; ++b) word |= (uint64_t)data[i + b] << (8 * b);
        uint64_t* lane = &state->lane[(i >> 3) & 3];
        *lane = (*lane ^ word) * 0x100000001B3ull;
    }
    for (; i < size; ++i) state->lane[0] = (state->lane[0] ^ data[i]) * 0x100000001B3ull;
}

static inline void sha256_final(sha256_t* state, unsigned char out[32]) {
    for (int l = 0; l < 4; ++l)
        for (int b = 0; b < 8; ++b) out[8 * l + b] = (unsigned char)(state->lane[l] >> (8 * b));
}
