// Portable BLAKE3 (hash mode, 32-byte output), written from the published specification.
// The .holo footer and weight fingerprints are BLAKE3 digests
// (crates/hologram-archive/src/writer.rs:217-225, weight.rs:24-29).
#pragma once
#include <stddef.h>
#include <stdint.h>

void holo_blake3(const uint8_t* data, size_t len, uint8_t out[32]);
