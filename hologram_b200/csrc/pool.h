// Label-keyed buffer pool: the device-resident counterpart of the reference's BufferArena
// (crates/hologram-exec/src/buffer.rs:149-207). Values live in device buffers keyed by their
// 71-byte content label; a slot of the workspace is a *binding* (pointer + extent) to one of them,
// so a memo hit or a reuse is a pointer rebind with no copy and no host round trip.
//
// Tiers, as in the reference:
//   pinned    constants, resident for the session (buffer.rs:463 pin_bytes); may alias memory the
//             session owns (the load-time slot buffers), in which case the pool never frees it
//   current / previous   the last two walks' results (two-generation rotation at every walk,
//             buffer.rs:352 rebind_reset)
//   leased    values the host took ownership of (buffer.rs:795-836): survive every rotation,
//             refuse the in-place KvCacheWrite move
//   lazy      weights declared but not resident; paged in from a host provider on first use and
//             evicted least-recently-used within a byte budget (buffer.rs:491-678)
// Memory comes from a small backend table so that the table logic can be exercised on host
// memory (unit tests without a GPU) exactly as it runs on cudaMalloc'd memory.
#pragma once
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "label.h"

struct HoloPoolMemory {
    void* user = nullptr;
    // all return 0 on success
    int (*alloc)(void* user, uint64_t bytes, void** out) = nullptr;
    void (*release)(void* user, void* ptr) = nullptr;
    int (*zero)(void* user, void* ptr, uint64_t bytes) = nullptr;
    int (*upload)(void* user, void* dst, const void* host, uint64_t bytes) = nullptr;      // host -> pool memory
    int (*download)(void* user, void* host, const void* src, uint64_t bytes) = nullptr;    // pool memory -> host (synchronous)
    int (*copy)(void* user, void* dst, const void* src, uint64_t bytes) = nullptr;         // pool memory -> pool memory
};

// Host side of a paged weight set (the reference's WeightProvider::get_range): returns a pointer
// to `size` bytes of the body whose BLAKE3 fingerprint is `fp`, starting at `offset`, or null.
typedef const void* (*HoloWeightRangeFn)(void* user, const uint8_t fp[32], uint64_t offset, uint64_t size);

class HoloPool {
public:
    static constexpr size_t UNBOUND = (size_t)-1;
    static constexpr uint64_t ALIGN = 64;   // size granularity (buffer.rs:63)

    explicit HoloPool(const HoloPoolMemory& mem) : mem_(mem) {}
    ~HoloPool();
    HoloPool(const HoloPool&) = delete;
    HoloPool& operator=(const HoloPool&) = delete;

    // ---- walk boundary ----
    void rebind_reset(size_t n_slots);                                   // buffer.rs:352
    // ---- slot bindings ----
    size_t bind_fresh(size_t slot, uint64_t len);                        // buffer.rs:427; UNBOUND on allocation failure
    bool bind_resident(size_t slot, const std::string& label);           // buffer.rs:437
    void bind_buffer(size_t slot, size_t bi);                            // bind_stolen, buffer.rs:775
    size_t bound(size_t slot) const { return slot < slot_buf_.size() ? slot_buf_[slot] : UNBOUND; }
    void* slot_ptr(size_t slot) const;
    uint64_t slot_len(size_t slot) const;
    // ---- residency ----
    void pin_external(const std::string& label, void* ptr, uint64_t len);   // pinned tier over memory the caller owns
    bool pin_bytes(const std::string& label, const void* host, uint64_t len);  // buffer.rs:463
    bool store_unbound(const std::string& label, const void* host, uint64_t len);   // buffer.rs:683
    void retain(size_t slot, const std::string& label);                  // buffer.rs:710
    size_t steal_transient(const std::string& label, const std::vector<size_t>& allowed_slots);   // buffer.rs:731; UNBOUND = declined
    // A buffer about to be rewritten in place must stop answering to its labels: removes every transient label
    // that names it. False (nothing changed) when a pinned, leased or paged label names it, or it is external.
    bool disown_transient(size_t bi);
    bool lease(const std::string& label);                                // buffer.rs:795
    bool release(const std::string& label);                              // buffer.rs:829
    bool resident(const std::string& label) const;                       // buffer.rs:871
    bool bindable_input(const std::string& label) const;                 // buffer.rs:858
    // address -> bytes boundary (buffer.rs:887): copies min(cap, len) bytes to `host`; false if not resident
    bool resolve(const std::string& label, void* host, uint64_t cap, uint64_t* len);
    size_t find(const std::string& label) const;                         // buffer index of a resident label, or UNBOUND
    // ---- lazy weights ----
    void set_lazy_budget(uint64_t bytes) { lazy_budget_ = bytes; }       // buffer.rs:482; 0 = unbounded
    void pin_lazy(const std::string& label, const uint8_t fp[32], uint64_t size);   // buffer.rs:491
    bool page_and_bind_group(const std::vector<std::pair<size_t, std::string>>& group, HoloWeightRangeFn fn, void* user);   // buffer.rs:650
    uint64_t lazy_resident_bytes() const;
    bool is_lazy(const std::string& label) const { return lazy_.count(label) != 0; }
    // ---- observability ----
    size_t leased_len() const { return leased_.size(); }
    uint64_t owned_bytes() const { return owned_bytes_; }                // bytes of memory the pool allocated (free list included)
    size_t free_len() const { return free_.size(); }
    size_t transient_len() const { return current_.size() + previous_.size(); }
    void* buffer_ptr(size_t bi) const { return bufs_[bi].ptr; }
    uint64_t buffer_len(size_t bi) const { return bufs_[bi].len; }
    uint64_t pages_in() const { return pages_in_; }

private:
    struct Buf {
        void* ptr = nullptr;
        uint64_t cap = 0, len = 0;
        bool external = false;   // memory owned by the caller (never freed, never recycled)
    };
    struct LazyWeight {
        uint8_t fp[32];
        uint64_t size = 0;
        size_t resident = UNBOUND;
        uint64_t last_touch = 0;
    };
    size_t acquire_buf(uint64_t len);                                    // buffer.rs:528: best fit <= 2x, zero-filled
    void push_free(size_t bi);
    void evict_lazy_protecting(uint64_t need, const std::vector<std::string>& keep);
    size_t page_one(const std::string& label, HoloWeightRangeFn fn, void* user, const std::vector<std::string>& keep);
    void ensure_slot(size_t slot);

    HoloPoolMemory mem_;
    std::vector<Buf> bufs_;
    std::vector<size_t> free_;
    std::vector<size_t> slot_buf_;
    std::vector<uint64_t> slot_len_;
    std::unordered_map<std::string, size_t> pinned_, current_, previous_;
    std::unordered_map<std::string, std::pair<size_t, uint32_t>> leased_;
    std::unordered_map<std::string, LazyWeight> lazy_;
    uint64_t lazy_budget_ = 0, lazy_clock_ = 0, owned_bytes_ = 0, pages_in_ = 0;
};
