// Label-keyed buffer pool (see pool.h). Host-side table logic only: no kernel is launched here; the
// memory backend does the allocations and copies.
#include "pool.h"

#include <string.h>

#include <algorithm>

HoloPool::~HoloPool() {
    for (Buf& b : bufs_)
        if (b.ptr && !b.external && mem_.release) mem_.release(mem_.user, b.ptr);
}

void HoloPool::ensure_slot(size_t slot) {
    if (slot >= slot_buf_.size()) slot_buf_.resize(slot + 1, UNBOUND);
    if (slot >= slot_len_.size()) slot_len_.resize(slot + 1, 0);
}

void HoloPool::push_free(size_t bi) {
    if (bufs_[bi].external) return;
    if (std::find(free_.begin(), free_.end(), bi) == free_.end()) free_.push_back(bi);
}

// Rotate the generations and give back every buffer that is no longer reachable: the dropped
// generation's, and any slot-only scratch (an unaddressable result is bound to a slot but retained
// under no label). A buffer stays if it is pinned, in the kept generation, leased or a paged-in weight.
void HoloPool::rebind_reset(size_t n_slots) {
    std::unordered_map<std::string, size_t> dropped;
    dropped.swap(previous_);
    previous_.swap(current_);
    std::unordered_set<size_t> kept;
    for (auto& kv : pinned_) kept.insert(kv.second);
    for (auto& kv : previous_) kept.insert(kv.second);
    for (auto& kv : leased_) kept.insert(kv.second.first);
    for (auto& kv : lazy_)
        if (kv.second.resident != UNBOUND) kept.insert(kv.second.resident);
    std::vector<size_t> reclaim;
    for (auto& kv : dropped)
        if (!kept.count(kv.second)) reclaim.push_back(kv.second);
    for (size_t bi : slot_buf_)
        if (bi != UNBOUND && !kept.count(bi)) reclaim.push_back(bi);
    std::sort(reclaim.begin(), reclaim.end());
    reclaim.erase(std::unique(reclaim.begin(), reclaim.end()), reclaim.end());
    for (size_t bi : reclaim) push_free(bi);
    slot_buf_.assign(n_slots, UNBOUND);
    if (slot_len_.size() < n_slots) slot_len_.resize(n_slots, 0);
}

// Best fit by capacity: a released buffer is taken only if it holds the request and is at most
// twice the aligned request, tightest first; otherwise a new allocation. Contents are zeroed.
size_t HoloPool::acquire_buf(uint64_t len) {
    const uint64_t want = (std::max<uint64_t>(len, ALIGN) + ALIGN - 1) / ALIGN * ALIGN;
    size_t best = UNBOUND;
    for (size_t fi = 0; fi < free_.size(); ++fi) {
        const uint64_t cap = bufs_[free_[fi]].cap;
        if (cap >= want && cap <= want * 2 && (best == UNBOUND || cap < bufs_[free_[best]].cap)) best = fi;
    }
    size_t bi;
    if (best != UNBOUND) {
        bi = free_[best];
        free_[best] = free_.back();
        free_.pop_back();
    } else {
        Buf b;
        if (mem_.alloc(mem_.user, want, &b.ptr) != 0 || !b.ptr) return UNBOUND;
        b.cap = want;
        owned_bytes_ += want;
        bufs_.push_back(b);
        bi = bufs_.size() - 1;
    }
    bufs_[bi].len = len;
    if (mem_.zero(mem_.user, bufs_[bi].ptr, bufs_[bi].cap) != 0) return UNBOUND;   // reuse never shows old bytes (buffer.rs:86-108)
    return bi;
}

size_t HoloPool::bind_fresh(size_t slot, uint64_t len) {
    const size_t bi = acquire_buf(len);
    if (bi == UNBOUND) return UNBOUND;
    ensure_slot(slot);
    slot_buf_[slot] = bi;
    slot_len_[slot] = len;
    return bi;
}

size_t HoloPool::find(const std::string& label) const {
    auto it = pinned_.find(label);
    if (it != pinned_.end()) return it->second;
    it = current_.find(label);
    if (it != current_.end()) return it->second;
    it = previous_.find(label);
    if (it != previous_.end()) return it->second;
    auto le = leased_.find(label);
    if (le != leased_.end()) return le->second.first;
    auto lz = lazy_.find(label);
    if (lz != lazy_.end() && lz->second.resident != UNBOUND) return lz->second.resident;
    return UNBOUND;
}

bool HoloPool::bind_resident(size_t slot, const std::string& label) {
    // pinned, current, previous, leased (a lazy weight is bound by page_and_bind_group only)
    size_t bi = UNBOUND;
    auto it = pinned_.find(label);
    if (it != pinned_.end()) bi = it->second;
    else if ((it = current_.find(label)) != current_.end()) bi = it->second;
    else if ((it = previous_.find(label)) != previous_.end()) bi = it->second;
    else {
        auto le = leased_.find(label);
        if (le != leased_.end()) bi = le->second.first;
    }
    if (bi == UNBOUND) return false;
    ensure_slot(slot);
    slot_buf_[slot] = bi;
    slot_len_[slot] = bufs_[bi].len;
    return true;
}

void HoloPool::bind_buffer(size_t slot, size_t bi) {
    ensure_slot(slot);
    slot_buf_[slot] = bi;
    slot_len_[slot] = bufs_[bi].len;
}

void* HoloPool::slot_ptr(size_t slot) const {
    const size_t bi = bound(slot);
    return bi == UNBOUND ? nullptr : bufs_[bi].ptr;
}

uint64_t HoloPool::slot_len(size_t slot) const {
    const size_t bi = bound(slot);
    return bi == UNBOUND ? 0 : bufs_[bi].len;
}

void HoloPool::pin_external(const std::string& label, void* ptr, uint64_t len) {
    if (pinned_.count(label)) return;
    Buf b;
    b.ptr = ptr;
    b.cap = b.len = len;
    b.external = true;
    bufs_.push_back(b);
    pinned_[label] = bufs_.size() - 1;
}

bool HoloPool::pin_bytes(const std::string& label, const void* host, uint64_t len) {
    if (pinned_.count(label)) return true;   // identical constants share one buffer
    const size_t bi = acquire_buf(len);
    if (bi == UNBOUND) return false;
    if (len && mem_.upload(mem_.user, bufs_[bi].ptr, host, len) != 0) return false;
    pinned_[label] = bi;
    return true;
}

// Bytes -> address boundary for inputs interned ahead of a walk. A label that lives only in the
// previous generation is promoted (re-interning is a statement that the value is live), so the
// label returned to the caller is always bindable by the next walk.
bool HoloPool::store_unbound(const std::string& label, const void* host, uint64_t len) {
    if (current_.count(label) || pinned_.count(label) || leased_.count(label)) return true;
    auto pv = previous_.find(label);
    if (pv != previous_.end()) {
        current_[label] = pv->second;
        return true;
    }
    if (resident(label)) return true;
    const size_t bi = acquire_buf(len);
    if (bi == UNBOUND) return false;
    if (len && mem_.upload(mem_.user, bufs_[bi].ptr, host, len) != 0) return false;
    current_[label] = bi;
    return true;
}

void HoloPool::retain(size_t slot, const std::string& label) {
    const size_t bi = bound(slot);
    if (bi == UNBOUND) return;
    if (pinned_.count(label) || current_.count(label)) return;
    current_[label] = bi;
}

// Consume a transient value for an in-place move: only if the label lives in the transient tier
// alone, its buffer is bound to no slot outside `allowed_slots`, and no other label names the same
// buffer. The label is retired from both generations; the caller re-binds and re-retains the
// buffer under the derived output label.
size_t HoloPool::steal_transient(const std::string& label, const std::vector<size_t>& allowed_slots) {
    if (pinned_.count(label) || leased_.count(label) || lazy_.count(label)) return UNBOUND;
    size_t bi = UNBOUND;
    auto it = current_.find(label);
    if (it != current_.end()) bi = it->second;
    else if ((it = previous_.find(label)) != previous_.end()) bi = it->second;
    if (bi == UNBOUND || bufs_[bi].external) return UNBOUND;
    for (size_t s = 0; s < slot_buf_.size(); ++s)
        if (slot_buf_[s] == bi && std::find(allowed_slots.begin(), allowed_slots.end(), s) == allowed_slots.end()) return UNBOUND;
    for (auto& kv : pinned_)
        if (kv.second == bi) return UNBOUND;
    for (auto& kv : current_)
        if (kv.second == bi && kv.first != label) return UNBOUND;
    for (auto& kv : previous_)
        if (kv.second == bi && kv.first != label) return UNBOUND;
    for (auto& kv : leased_)
        if (kv.second.first == bi) return UNBOUND;
    for (auto& kv : lazy_)
        if (kv.second.resident == bi) return UNBOUND;
    current_.erase(label);
    previous_.erase(label);
    return bi;
}

bool HoloPool::disown_transient(size_t bi) {
    if (bi >= bufs_.size() || bufs_[bi].external) return false;
    for (auto& kv : pinned_)
        if (kv.second == bi) return false;
    for (auto& kv : leased_)
        if (kv.second.first == bi) return false;
    for (auto& kv : lazy_)
        if (kv.second.resident == bi) return false;
    for (auto it = current_.begin(); it != current_.end();) it = it->second == bi ? current_.erase(it) : std::next(it);
    for (auto it = previous_.begin(); it != previous_.end();) it = it->second == bi ? previous_.erase(it) : std::next(it);
    return true;
}

bool HoloPool::lease(const std::string& label) {
    auto le = leased_.find(label);
    if (le != leased_.end()) {
        ++le->second.second;
        return true;
    }
    if (pinned_.count(label)) return true;   // already permanent
    if (lazy_.count(label)) return false;    // the pager owns that lifecycle
    size_t bi = UNBOUND;
    auto it = current_.find(label);
    if (it != current_.end()) bi = it->second;
    else if ((it = previous_.find(label)) != previous_.end()) bi = it->second;
    if (bi == UNBOUND) return false;
    leased_[label] = {bi, 1u};
    return true;
}

// When the last lease drops the value is demoted into the current generation: resident for the
// normal two-walk window, then reclaimed.
bool HoloPool::release(const std::string& label) {
    auto le = leased_.find(label);
    if (le == leased_.end()) return false;
    if (--le->second.second == 0) {
        const size_t bi = le->second.first;
        leased_.erase(le);
        current_[label] = bi;
    }
    return true;
}

bool HoloPool::resident(const std::string& label) const {
    if (pinned_.count(label) || current_.count(label) || previous_.count(label) || leased_.count(label)) return true;
    auto lz = lazy_.find(label);
    return lz != lazy_.end() && lz->second.resident != UNBOUND;
}

bool HoloPool::bindable_input(const std::string& label) const {
    if (pinned_.count(label) || current_.count(label) || leased_.count(label)) return true;
    auto lz = lazy_.find(label);
    return lz != lazy_.end() && lz->second.resident != UNBOUND;
}

bool HoloPool::resolve(const std::string& label, void* host, uint64_t cap, uint64_t* len) {
    const size_t bi = find(label);
    if (bi == UNBOUND) return false;
    if (len) *len = bufs_[bi].len;
    const uint64_t n = std::min<uint64_t>(cap, bufs_[bi].len);
    if (n && host && mem_.download(mem_.user, host, bufs_[bi].ptr, n) != 0) return false;
    return true;
}

// ---- lazy weights -------------------------------------------------------------------------------
void HoloPool::pin_lazy(const std::string& label, const uint8_t fp[32], uint64_t size) {
    if (lazy_.count(label)) return;   // identical weights collapse to one entry
    LazyWeight w;
    memcpy(w.fp, fp, 32);
    w.size = size;
    lazy_[label] = w;
}

uint64_t HoloPool::lazy_resident_bytes() const {
    uint64_t total = 0;
    for (auto& kv : lazy_)
        if (kv.second.resident != UNBOUND) total += kv.second.size;
    return total;
}

// Evict least-recently-used paged weights until `need` more bytes fit the budget, never one of
// `keep` (a kernel reads all its paged operands at once). A group larger than the budget then
// resides in full.
void HoloPool::evict_lazy_protecting(uint64_t need, const std::vector<std::string>& keep) {
    if (lazy_budget_ == 0) return;
    uint64_t resident_bytes = lazy_resident_bytes();
    if (resident_bytes + need <= lazy_budget_) return;
    std::vector<std::pair<uint64_t, std::string>> victims;
    for (auto& kv : lazy_)
        if (kv.second.resident != UNBOUND && std::find(keep.begin(), keep.end(), kv.first) == keep.end())
            victims.push_back({kv.second.last_touch, kv.first});
    std::sort(victims.begin(), victims.end());
    for (auto& v : victims) {
        if (resident_bytes + need <= lazy_budget_) break;
        LazyWeight& w = lazy_[v.second];
        push_free(w.resident);
        w.resident = UNBOUND;
        resident_bytes -= w.size;
    }
}

size_t HoloPool::page_one(const std::string& label, HoloWeightRangeFn fn, void* user, const std::vector<std::string>& keep) {
    auto it = lazy_.find(label);
    if (it == lazy_.end()) return UNBOUND;
    if (it->second.resident != UNBOUND) {
        it->second.last_touch = ++lazy_clock_;
        return it->second.resident;
    }
    const uint64_t size = it->second.size;
    evict_lazy_protecting(size, keep);
    const size_t bi = acquire_buf(size);
    if (bi == UNBOUND) return UNBOUND;
    const void* body = fn ? fn(user, it->second.fp, 0, size) : nullptr;
    if (!body || (size && mem_.upload(mem_.user, bufs_[bi].ptr, body, size) != 0)) {
        push_free(bi);   // fail closed: the weight stays non-resident
        return UNBOUND;
    }
    ++pages_in_;
    LazyWeight& w = lazy_[label];
    w.resident = bi;
    w.last_touch = ++lazy_clock_;
    return bi;
}

bool HoloPool::page_and_bind_group(const std::vector<std::pair<size_t, std::string>>& group, HoloWeightRangeFn fn, void* user) {
    std::vector<std::string> labels;
    for (auto& g : group) labels.push_back(g.second);
    for (auto& g : group) {
        const size_t bi = page_one(g.second, fn, user, labels);
        if (bi == UNBOUND) return false;
        ensure_slot(g.first);
        slot_buf_[g.first] = bi;
        slot_len_[g.first] = lazy_[g.second].size;
    }
    return true;
}
