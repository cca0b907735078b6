// Archive session state shared by the plain walk (session.cu) and the content-addressed walk
// (addressed.cpp). Not part of the C ABI.
#pragma once
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "archive.h"
#include "common.h"
#include "label.h"
#include "pool.h"

// A merged group of sibling matmuls: products of one A against several constant weights,
// executed as one matmul against the column-concatenated weights with one output segment each.
struct MergedMatmul {
    HoloBufferRef a;
    uint32_t m = 0, k = 0, n = 0, nseg = 0;
    void* b_concat = nullptr;          // [k, n] bf16, owned by the session
    HoloBufferRef out[3];
    uint32_t width[3] = {0, 0, 0};
    uint8_t act[3] = {0, 0, 0};
    HoloBufferRef b_src[3];
    // gated pair: out[0] = act(A W0), out[1] = A W1 and the Mul of the two run as one product whose
    // weights alternate 64-column blocks of W0 and W1; `gated_out` receives act(A W0) * (A W1)
    bool gated = false;
    HoloBufferRef gated_out = {HOLO_NO_SLOT, 0, 0};
    // per-head calls that read segment t and follow the product directly, absorbed into its epilogue
    // (HoloMatmulSeg::head_op): the RotaryEmbedding's cos / sin / output, the quantizer's codes / scales
    uint8_t head_op[3] = {0, 0, 0};
    HoloBufferRef cos[3] = {{HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}};
    HoloBufferRef sin[3] = {{HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}};
    HoloBufferRef rope_out[3] = {{HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}};
    HoloBufferRef codes[3] = {{HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}};
    HoloBufferRef scales[3] = {{HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}, {HOLO_NO_SLOT, 0, 0}};
};

// A run of mutually independent small glue calls executed as one launch.
struct MicroBatch {
    HoloMicroOp* dev_ops = nullptr;    // owned by the session
    uint32_t nops = 0, total_ctas = 0, ncalls = 0;
};

struct SessionNode {
    int merged = -1;                   // index into holo_b200_session::merged, or -1
    int batch = -1;                    // index into holo_b200_session::batches, or -1
    HoloKernelCall call;               // the plain call when both are -1
    // AllReduce followed by the residual Add, run as one launch: `call` is the AllReduce,
    // `residual` / `sum_out` come from the Add
    bool reduce_add = false;
    HoloBufferRef residual = {HOLO_NO_SLOT, 0, 0}, sum_out = {HOLO_NO_SLOT, 0, 0};
    // MatMul whose product is all-reduced and added to a residual: `call` is the MatMul; the sum over
    // the ranks happens in the matmul's epilogue (or right after it), `residual` / `sum_out` as above
    bool matmul_reduce_add = false;
};

// ---- content-addressed execution (a session loaded with HOLO_SESSION_ADDRESSED) ----
// The walk of crates/hologram-exec/src/session.rs:1052-1289 over device memory: every value has a
// label derived from its operation and its operands' labels; the pool keeps device buffers by
// label, so a value that is already resident is bound to its consumer's slot by pointer (no
// dispatch, no copy, no host round trip), and a whole-graph repeat is answered from the memo of
// input labels -> output labels.
struct HoloAddressed {
    struct NodeMeta {
        HoloOpSignature sig;
        std::vector<uint32_t> inputs, outputs;   // operand slots in kernel order; written slots
        bool addressable = false;
        bool in_place = false;                    // a written slot is also read (AllReduce): the value is rewritten where it lies
    };
    std::unique_ptr<HoloPool> pool;
    std::vector<NodeMeta> meta;                           // one per call
    std::vector<uint64_t> slot_need;                      // bytes a slot must hold
    std::vector<HoloSlot> static_binding;                 // the load-time buffer of every slot
    std::vector<std::string> slot_label_init;             // constants' labels ("" = none)
    std::vector<std::pair<uint32_t, std::string>> const_bindings;
    std::unordered_map<uint32_t, std::string> lazy_slots; // paged weights: slot -> label
    std::vector<uint8_t> is_output_slot, is_input_slot;
    std::vector<uint8_t> stealable;                       // per call: KvCacheWrite may move in place (session.rs:281-322)
    std::unordered_map<std::string, std::pair<std::string, uint64_t>> memo;   // input labels -> (output labels, tick)
    uint64_t memo_tick = 0;
    bool residual_in_label = false;                       // HOLO_SESSION_LABEL_RESIDUAL
    HoloWeightProvider provider = {nullptr, nullptr, nullptr};
    bool paged = false;
    uint32_t last_dispatched = 0, last_skipped = 0, last_moved = 0;
};

struct holo_b200_session {
    holo_b200_ctx* ctx = nullptr;
    holo_b200_workspace* ws = nullptr;
    HoloArchive ar;
    std::vector<HoloKernelCall> calls;  // execution order, after fusion (merged groups keep their members here)
    std::vector<uint32_t> call_level;   // schedule level of every entry of `calls`
    std::vector<SessionNode> nodes;     // what a walk actually launches
    std::vector<MergedMatmul> merged;
    std::vector<MicroBatch> batches;
    std::vector<uint32_t> weight_slots; // constants that no call writes
    uint32_t fused = 0, moved_in_place = 0, merged_calls = 0, batched_calls = 0, reduce_adds = 0, rope_quant = 0, head_fused = 0;
    uint64_t device_bytes = 0;
    cudaGraphExec_t graph = nullptr;
    bool addressed = false;
    HoloAddressed ad;
};

// session.cu
int32_t holo_session_load_impl(holo_b200_ctx* ctx, const uint8_t* archive, uint64_t len, int32_t verify, const HoloWeightProvider* provider,
                               uint64_t budget, holo_b200_session** out);
// addressed.cpp
int32_t holo_addressed_prepare(holo_b200_session* s, const std::vector<uint64_t>& slot_need);
void holo_addressed_destroy(holo_b200_session* s);
void holo_addressed_bind_static(holo_b200_session* s);
