// Content labels ("kappa-labels") and per-call operation signatures, the host-side identity
// machinery of the reference's content-addressed executor:
//   label of bytes        crates/hologram-archive/src/address.rs:83-86  (address_bytes)
//   label of a derivation crates/hologram-archive/src/address.rs:108-116 (derive_label), :197-221 (derive_label_boundary)
//   label rendering       crates/hologram-archive/src/address.rs:51-61  ("blake3:" + 64 hex = 71 bytes)
//   op signature          crates/hologram-compute/src/kernel_call.rs:996-1142, 1321-1516
//   operand order         crates/hologram-compute/src/kernel_call.rs:1560-1660 (inputs.., output)
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/hologram_b200.h"

constexpr size_t HOLO_LABEL_BYTES = 71;

void holo_label_from_digest(const uint8_t digest[32], uint8_t out[HOLO_LABEL_BYTES]);
void holo_label_of_bytes(const uint8_t* data, size_t len, uint8_t out[HOLO_LABEL_BYTES]);
// BLAKE3(opcode as LE u16 || params || label_0 || label_1 || ...), rendered as a label.
void holo_label_derive(uint16_t opcode, const uint8_t* params, size_t params_len, const uint8_t* labels, size_t n_labels,
                       uint8_t out[HOLO_LABEL_BYTES]);

// The boundary form (address.rs:197-221): op label, then the operand labels folded in order through
// address_bytes(left digest || right digest). False if a label is not a well-formed blake3 label.
bool holo_label_derive_boundary(uint16_t opcode, const uint8_t* params, size_t params_len, const uint8_t* labels, size_t n_labels,
                                uint8_t out[HOLO_LABEL_BYTES]);

struct HoloOpSignature {
    uint16_t opcode = 0;
    uint8_t params[64] = {};
    uint32_t len = 0;
    bool commutative = false;
};
// False for a variant this backend does not serve.
bool holo_op_signature(const HoloKernelCall& call, HoloOpSignature* sig);
// Operand slots in kernel order with absent operands left out, and the output slot.
// `residual_in_label`: append AddRmsNorm's residual operand (the reference's list omits it).
bool holo_call_operands(const HoloKernelCall& call, std::vector<uint32_t>* inputs, uint32_t* output, bool residual_in_label = false);
