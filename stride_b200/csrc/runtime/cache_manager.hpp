// The cache manager: page pools for groups of layers, a block table per request
// and group, and slots for per-request state of fixed size.
//
// A group is a set of layers whose keys and values share one page geometry and
// one retention rule: `window == 0` keeps every key, `window == W` only needs
// the last W keys of a request, so pages that the window has passed are given
// back while the request is still running. Every group has its own pool and its
// own page ids. Content-addressed prefix sharing is only sound when every group
// keeps all keys and no per-request state exists, and is switched off otherwise.
//
// The reference has one group and no state slots
// (crates/stride-kvcache/src/lib.rs, python/stride_worker/cache.py:44-56).
#pragma once

#include <algorithm>
#include <unordered_map>

#include "page_pool.hpp"

namespace stride {

using RequestKey = int64_t;

struct GroupConfig {
    size_t num_pages = 0;
    size_t window = 0;  // 0: all keys are kept
};

struct RequestPages {
    std::string tenant;
    int32_t state_slot = -1;
    // Per group: the logical block table. Entries given back are -1.
    std::vector<std::vector<PageId>> tables;
    // Per group: how many leading pages were given back to the pool.
    std::vector<size_t> trimmed;
    size_t shared_prefix_tokens = 0;
};

class CacheManager {
public:
    CacheManager(size_t page_size, std::vector<GroupConfig> groups, size_t num_state_slots, bool prefix_caching)
        : page_size_(page_size), groups_(std::move(groups)), slot_capacity_(num_state_slots) {
        if (groups_.empty()) throw std::invalid_argument("the cache manager needs at least one group");
        bool all_full = true;
        for (auto& g : groups_) {
            pools_.emplace_back(g.num_pages, page_size);
            all_full = all_full && g.window == 0;
        }
        prefix_caching_ = prefix_caching && all_full && groups_.size() == 1;
        for (size_t i = num_state_slots; i-- > 0;) free_slots_.push_back(static_cast<int32_t>(i));
    }

    size_t page_size() const { return page_size_; }
    size_t num_groups() const { return groups_.size(); }
    const GroupConfig& group(size_t g) const { return groups_.at(g); }
    bool prefix_caching() const { return prefix_caching_; }
    const PagePool& pool(size_t g) const { return pools_.at(g); }
    PagePool& pool_mut(size_t g) { return pools_.at(g); }
    size_t pages_for(size_t tokens) const { return (tokens + page_size_ - 1) / page_size_; }
    bool has(RequestKey r) const { return requests_.count(r) != 0; }
    size_t num_requests() const { return requests_.size(); }
    size_t free_slots() const { return free_slots_.size(); }
    size_t slot_capacity() const { return slot_capacity_; }

    // Smallest number of allocatable pages over the groups.
    size_t num_allocatable() const {
        size_t n = SIZE_MAX;
        for (auto& p : pools_) n = std::min(n, p.num_allocatable());
        return n;
    }

    size_t min_capacity() const {
        size_t n = SIZE_MAX;
        for (auto& p : pools_) n = std::min(n, p.capacity());
        return n;
    }

    // Registers a request: a state slot and empty tables. Returns the slot.
    int32_t open(RequestKey r, const std::string& tenant) {
        if (requests_.count(r)) throw std::invalid_argument("request " + std::to_string(r) + " already holds cache");
        if (free_slots_.empty()) throw OutOfPages(1, 0);
        RequestPages e;
        e.tenant = tenant;
        e.state_slot = free_slots_.back();
        free_slots_.pop_back();
        e.tables.resize(groups_.size());
        e.trimmed.assign(groups_.size(), 0);
        requests_.emplace(r, std::move(e));
        return requests_.at(r).state_slot;
    }

    // Looks the tokens up in the prefix index and puts the pages found at the
    // head of the (still empty) table. Returns the number of tokens covered.
    size_t adopt_prefix(RequestKey r, const std::vector<TokenId>& tokens) {
        auto& e = entry(r);
        if (!prefix_caching_) return 0;
        if (!e.tables[0].empty()) throw std::invalid_argument("a prefix can only be adopted by an empty table");
        e.tables[0] = pools_[0].acquire_prefix(e.tenant, tokens);
        e.shared_prefix_tokens = e.tables[0].size() * page_size_;
        return e.shared_prefix_tokens;
    }

    // Grows every group's table to cover `num_tokens` tokens. All or nothing;
    // `reserve` pages must stay allocatable in every pool afterwards.
    bool ensure(RequestKey r, size_t num_tokens, size_t reserve) {
        auto& e = entry(r);
        size_t need = pages_for(num_tokens);
        for (size_t g = 0; g < groups_.size(); ++g) {
            size_t have = e.tables[g].size();
            if (need > have && pools_[g].num_allocatable() < (need - have) + reserve) return false;
        }
        for (size_t g = 0; g < groups_.size(); ++g) {
            size_t have = e.tables[g].size();
            if (need <= have) continue;
            auto fresh = pools_[g].allocate(need - have);
            e.tables[g].insert(e.tables[g].end(), fresh.begin(), fresh.end());
        }
        return true;
    }

    // How many pages ensure() would have to allocate, the largest over groups.
    size_t pages_missing(RequestKey r, size_t num_tokens) const {
        auto& e = entry(r);
        size_t need = pages_for(num_tokens), worst = 0;
        for (auto& t : e.tables) worst = std::max(worst, need > t.size() ? need - t.size() : size_t(0));
        return worst;
    }

    // After `kv_len` tokens of the request have keys in the cache, the next
    // query sits at position >= kv_len and reads keys > kv_len - window. Pages
    // that lie wholly below that are given back. Returns how many were.
    size_t trim(RequestKey r, size_t kv_len) {
        auto& e = entry(r);
        size_t given_back = 0;
        for (size_t g = 0; g < groups_.size(); ++g) {
            size_t w = groups_[g].window;
            if (w == 0 || kv_len + 1 <= w) continue;
            size_t first_needed = kv_len + 1 - w;            // lowest key position still read
            size_t keep_from = first_needed / page_size_;    // page that holds it
            auto& t = e.tables[g];
            for (size_t i = e.trimmed[g]; i < keep_from && i < t.size(); ++i) {
                pools_[g].release_one(t[i]);
                t[i] = -1;
                ++given_back;
            }
            e.trimmed[g] = std::max(e.trimmed[g], std::min(keep_from, t.size()));
        }
        return given_back;
    }

    // Index the request's full, written pages so that later requests with the
    // same tokens can share them.
    void publish(RequestKey r, const std::vector<TokenId>& tokens, size_t written_tokens) {
        auto& e = entry(r);
        if (!prefix_caching_) return;
        pools_[0].publish(e.tenant, tokens, written_tokens, e.tables[0]);
    }

    // Gives back every page and the state slot.
    void close(RequestKey r) {
        auto it = requests_.find(r);
        if (it == requests_.end()) throw std::invalid_argument("request " + std::to_string(r) + " holds no cache");
        for (size_t g = 0; g < groups_.size(); ++g) pools_[g].release(it->second.tables[g]);
        free_slots_.push_back(it->second.state_slot);
        requests_.erase(it);
    }

    const RequestPages& entry(RequestKey r) const {
        auto it = requests_.find(r);
        if (it == requests_.end()) throw std::invalid_argument("request " + std::to_string(r) + " holds no cache");
        return it->second;
    }

    const std::vector<PageId>& table(RequestKey r, size_t g) const { return entry(r).tables.at(g); }
    int32_t state_slot(RequestKey r) const { return entry(r).state_slot; }

    // Pool invariants, slots, and the block tables against the reference
    // counts: a page is referenced exactly as often as tables name it.
    void check_invariants() const {
        for (auto& p : pools_) p.check_invariants();
        if (free_slots_.size() + requests_.size() != slot_capacity_)
            throw InvariantError("state slots: " + std::to_string(free_slots_.size()) + " free + " +
                                 std::to_string(requests_.size()) + " held != capacity " +
                                 std::to_string(slot_capacity_));
        std::vector<char> slot_seen(slot_capacity_, 0);
        for (int32_t s : free_slots_) {
            if (slot_seen.at(s)) throw InvariantError("state slot free twice");
            slot_seen[s] = 1;
        }
        for (auto& kv : requests_) {
            if (slot_seen.at(kv.second.state_slot)) throw InvariantError("state slot held twice or free while held");
            slot_seen[kv.second.state_slot] = 1;
        }
        for (size_t g = 0; g < groups_.size(); ++g) {
            std::vector<uint32_t> named(pools_[g].capacity(), 0);
            for (auto& kv : requests_)
                for (PageId p : kv.second.tables[g])
                    if (p >= 0) ++named.at(p);
            for (size_t p = 0; p < named.size(); ++p)
                if (named[p] != pools_[g].refcount(static_cast<PageId>(p)))
                    throw InvariantError("group " + std::to_string(g) + " page " + std::to_string(p) + ": tables name it " +
                                         std::to_string(named[p]) + " times, reference count is " +
                                         std::to_string(pools_[g].refcount(static_cast<PageId>(p))));
        }
    }

private:
    RequestPages& entry(RequestKey r) {
        auto it = requests_.find(r);
        if (it == requests_.end()) throw std::invalid_argument("request " + std::to_string(r) + " holds no cache");
        return it->second;
    }

    size_t page_size_;
    std::vector<GroupConfig> groups_;
    std::vector<PagePool> pools_;
    size_t slot_capacity_;
    std::vector<int32_t> free_slots_;
    std::unordered_map<RequestKey, RequestPages> requests_;
    bool prefix_caching_ = false;
};

}  // namespace stride
