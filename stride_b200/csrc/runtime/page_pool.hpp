// Host-side bookkeeping of one pool of KV pages.
//
// A page is in exactly one of three states: live (held by at least one
// request), cached (held by nobody, still findable by its content hash, may be
// evicted) or free (on the free list). The three counts are kept by different
// structures so that check_invariants() can actually fail. Behaviour follows
// crates/stride-kvcache/src/{lib,allocator,hash,prefix}.rs of the reference,
// with two changes: release() walks the table backwards so that the LRU order
// evicts the leaves of a hash chain before its root, and publish() takes the
// number of tokens whose keys are really written.
#pragma once

#include <cstdint>
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace stride {

using PageId = int32_t;
using TokenId = int32_t;

struct InvariantError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct OutOfPages : std::runtime_error {
    size_t requested, available;
    OutOfPages(size_t req, size_t avail)
        : std::runtime_error("out of KV pages: requested " + std::to_string(req) + ", available " +
                             std::to_string(avail)),
          requested(req), available(avail) {}
};

// FNV-1a 64 chain: root = hash(tenant bytes); page = hash(parent as 8 LE bytes,
// then each token as 4 LE bytes), restarting from the offset basis
// (crates/stride-kvcache/src/hash.rs:15-58).
namespace prefix_hash {
constexpr uint64_t kOffset = 0xcbf29ce484222325ull;
constexpr uint64_t kPrime = 0x00000100000001b3ull;

inline uint64_t mix(uint64_t acc, uint64_t value, int nbytes) {
    for (int i = 0; i < nbytes; ++i) {
        acc ^= (value >> (8 * i)) & 0xffu;
        acc *= kPrime;
    }
    return acc;
}

inline uint64_t tenant_root(const std::string& tenant) {
    uint64_t acc = kOffset;
    for (unsigned char c : tenant) {
        acc ^= c;
        acc *= kPrime;
    }
    return acc;
}

inline uint64_t page_hash(uint64_t parent, const TokenId* tokens, size_t n) {
    uint64_t acc = mix(kOffset, parent, 8);
    for (size_t i = 0; i < n; ++i) acc = mix(acc, static_cast<uint32_t>(tokens[i]), 4);
    return acc;
}

inline std::vector<uint64_t> chain(const std::string& tenant, const std::vector<TokenId>& tokens,
                                   size_t page_size, size_t limit_tokens) {
    std::vector<uint64_t> out;
    uint64_t parent = tenant_root(tenant);
    size_t n = std::min(limit_tokens, tokens.size());
    for (size_t start = 0; start + page_size <= n; start += page_size) {
        parent = page_hash(parent, tokens.data() + start, page_size);
        out.push_back(parent);
    }
    return out;
}
}  // namespace prefix_hash

struct PoolStats {
    size_t capacity = 0, live = 0, cached = 0, free = 0;
    uint64_t hits = 0, misses = 0;
    double hit_rate() const { return hits + misses ? double(hits) / double(hits + misses) : 0.0; }
};

class PagePool {
public:
    PagePool(size_t num_pages, size_t page_size) : page_size_(page_size), refcount_(num_pages, 0) {
        if (num_pages == 0) throw std::invalid_argument("a page pool needs at least one page");
        if (page_size == 0) throw std::invalid_argument("page_size must be positive");
        free_.reserve(num_pages);
        for (size_t i = num_pages; i-- > 0;) free_.push_back(static_cast<PageId>(i));  // pops 0,1,2,...
    }

    size_t page_size() const { return page_size_; }
    size_t capacity() const { return refcount_.size(); }
    size_t pages_for(size_t tokens) const { return (tokens + page_size_ - 1) / page_size_; }
    size_t num_allocatable() const { return free_.size() + evictable_.size(); }
    uint32_t refcount(PageId p) const { return refcount_.at(p); }

    // Walk the chain of `tokens` until the first miss and take a reference to
    // each page found. The page that ends exactly at the last token is never
    // taken, so at least one token is left to run
    // (crates/stride-kvcache/src/lib.rs:126-154).
    std::vector<PageId> acquire_prefix(const std::string& tenant, const std::vector<TokenId>& tokens) {
        auto hashes = prefix_hash::chain(tenant, tokens, page_size_, tokens.size());
        size_t ceiling = hashes.size();
        if (!tokens.empty() && tokens.size() % page_size_ == 0 && ceiling > 0) --ceiling;
        std::vector<PageId> pages;
        for (size_t i = 0; i < ceiling; ++i) {
            auto it = by_hash_.find(hashes[i]);
            if (it == by_hash_.end()) {
                ++misses_;
                break;
            }
            ++hits_;
            PageId p = it->second;
            if (refcount_[p] == 0) {
                auto st = stamp_.find(p);
                if (st != stamp_.end()) evictable_.erase({st->second, p});
                ++live_;
            }
            ++refcount_[p];
            stamp_[p] = ++clock_;
            pages.push_back(p);
        }
        return pages;
    }

    // All or nothing: free pages first, then the least recently used cached ones.
    std::vector<PageId> allocate(size_t n) {
        if (n > num_allocatable()) throw OutOfPages(n, num_allocatable());
        std::vector<PageId> out;
        out.reserve(n);
        for (size_t i = 0; i < n; ++i) {
            PageId p;
            if (!free_.empty()) {
                p = free_.back();
                free_.pop_back();
            } else {
                auto first = evictable_.begin();
                p = first->second;
                evictable_.erase(first);
                stamp_.erase(p);
                auto h = by_page_.find(p);
                if (h != by_page_.end()) {
                    by_hash_.erase(h->second);
                    by_page_.erase(h);
                }
                ++evictions_;
            }
            if (refcount_[p] != 0) throw InvariantError("handed out a page that is still referenced");
            refcount_[p] = 1;
            ++live_;
            out.push_back(p);
        }
        return out;
    }

    // Index the full pages among the first `written_tokens` tokens under their
    // content hashes. First writer wins; a duplicate stays unindexed.
    void publish(const std::string& tenant, const std::vector<TokenId>& tokens, size_t written_tokens,
                 const std::vector<PageId>& pages) {
        auto hashes = prefix_hash::chain(tenant, tokens, page_size_, written_tokens);
        for (size_t i = 0; i < hashes.size() && i < pages.size(); ++i) {
            PageId p = pages[i];
            if (p < 0) break;
            if (refcount_.at(p) == 0) throw InvariantError("publishing a page that nobody holds");
            if (by_hash_.count(hashes[i]) || by_page_.count(p)) continue;
            by_hash_[hashes[i]] = p;
            by_page_[p] = hashes[i];
            stamp_[p] = ++clock_;
        }
    }

    // Drop one reference per page, last page first. A page that reaches zero
    // becomes cached if it is indexed, free otherwise.
    void release(const std::vector<PageId>& pages) {
        for (size_t i = pages.size(); i-- > 0;) release_one(pages[i]);
    }

    void release_one(PageId p) {
        if (p < 0) return;
        if (refcount_.at(p) == 0) throw InvariantError("page " + std::to_string(p) + " freed twice");
        if (--refcount_[p] > 0) return;
        --live_;
        if (by_page_.count(p)) {
            uint64_t t = ++clock_;
            auto st = stamp_.find(p);
            if (st != stamp_.end()) evictable_.erase({st->second, p});
            stamp_[p] = t;
            evictable_.insert({t, p});
        } else {
            free_.push_back(p);
        }
    }

    PoolStats stats() const {
        PoolStats s;
        s.capacity = capacity();
        s.live = live_;
        s.cached = evictable_.size();
        s.free = free_.size();
        s.hits = hits_;
        s.misses = misses_;
        return s;
    }

    uint64_t evictions() const { return evictions_; }

    // Every page is live, cached or free, exactly one of them; each count is
    // recomputed from the structure that defines it and compared with the
    // running counter (crates/stride-kvcache/src/lib.rs:244-276).
    void check_invariants() const {
        std::ostringstream err;
        size_t live = 0;
        for (uint32_t rc : refcount_) live += rc > 0;
        if (live != live_) err << "live counter " << live_ << " != recount " << live << "; ";
        size_t cached = 0;
        for (auto& kv : by_page_) cached += refcount_[kv.first] == 0;
        if (cached != evictable_.size())
            err << "cached set " << evictable_.size() << " != recount " << cached << "; ";
        if (by_hash_.size() != by_page_.size()) err << "hash index and page index differ in size; ";
        for (auto& e : evictable_) {
            auto st = stamp_.find(e.second);
            if (!by_page_.count(e.second)) err << "page " << e.second << " evictable but not indexed; ";
            if (st == stamp_.end() || st->second != e.first) err << "page " << e.second << " has a stale stamp; ";
            if (refcount_[e.second] != 0) err << "page " << e.second << " evictable but referenced; ";
        }
        std::vector<char> seen(capacity(), 0);
        for (PageId p : free_) {
            if (seen.at(p)) err << "page " << p << " is on the free list twice; ";
            seen[p] = 1;
            if (refcount_[p] != 0) err << "page " << p << " free but referenced; ";
            if (by_page_.count(p)) err << "page " << p << " free but indexed; ";
        }
        if (live_ + evictable_.size() + free_.size() != capacity())
            err << "live " << live_ << " + cached " << evictable_.size() << " + free " << free_.size()
                << " != capacity " << capacity() << "; ";
        std::string msg = err.str();
        if (!msg.empty()) throw InvariantError("page pool invariant broken: " + msg);
    }

    // For the negative control of the invariant check only.
    void corrupt_for_test(int what) {
        if (what == 0 && !free_.empty()) free_.pop_back();          // a page is lost
        if (what == 1 && !free_.empty()) {                           // a page is held twice
            PageId dup = free_[0];
            free_.push_back(dup);
        }
        if (what == 2) ++live_;                                      // the counter drifts
    }

private:
    size_t page_size_;
    std::vector<uint32_t> refcount_;
    std::vector<PageId> free_;
    size_t live_ = 0;
    std::unordered_map<uint64_t, PageId> by_hash_;
    std::unordered_map<PageId, uint64_t> by_page_;
    std::set<std::pair<uint64_t, PageId>> evictable_;
    std::unordered_map<PageId, uint64_t> stamp_;
    uint64_t clock_ = 0, hits_ = 0, misses_ = 0, evictions_ = 0;
};

}  // namespace stride
