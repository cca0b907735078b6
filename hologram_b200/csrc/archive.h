// `.holo` archive reader for the call variants this backend serves.
// Wire format: crates/hologram-archive/src/writer.rs:185-226 (framing), loader.rs:141-267
// (header / section table / footer checks), kernel_codec.rs:130-137 + put_* :569-873 (calls),
// writer.rs:246-263 (ports), constant_codec.rs:66-95 (constants), writer.rs:388-440 (weights),
// writer.rs:325-336 (exec plan), writer.rs:243-249 (extensions).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/hologram_b200.h"

struct HoloPort {
    std::string name;
    uint32_t slot = 0;
    uint64_t element_count = 0;
    uint8_t dtype = 0;
    std::vector<uint64_t> shape;
};
struct HoloConstant {
    uint32_t slot = 0;
    uint8_t dtype = 0;
    const uint8_t* bytes = nullptr;  // points into the archive image; null when the body is not in the archive (paged load only)
    uint64_t len = 0;
    bool by_reference = false;       // constant_codec.rs tag 1: the body is a weight named by its fingerprint
    uint8_t fingerprint[32] = {};    // BLAKE3 of the body (by_reference only)
};
struct HoloExtension {
    std::string key;
    const uint8_t* bytes = nullptr;
    uint64_t len = 0;
};
struct HoloArchive {
    uint16_t version = 0;
    std::vector<HoloKernelCall> calls;
    std::vector<HoloPort> inputs, outputs;
    std::vector<HoloConstant> constants;
    std::vector<std::vector<uint32_t>> exec_plan;
    std::vector<HoloExtension> extensions;
};

// Parse (and, when `verify`, check the BLAKE3 footer and every weight fingerprint of) an
// archive image. `data` must outlive `out`. Returns HOLO_OK or a negative status with the
// thread-local message set.
// `allow_missing_weights`: a constant may reference a weight that the archive does not carry (a
// weightless archive, loaded with a weight provider); otherwise that is an error.
int32_t holo_archive_parse(const uint8_t* data, uint64_t len, bool verify, HoloArchive* out, bool allow_missing_weights = false);
