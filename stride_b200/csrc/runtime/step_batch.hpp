// Flattens one step's work — for each request its next tokens — into the index
// arrays that the step function's kernels read, packed into one int32 buffer so
// that a step needs a single host-to-device copy.
//
// The unit of work has the fields of the reference's SequenceWork
// (python/stride_worker/protocol.py:55-77: request, tokens, position of the
// first token, block table, whether logits are wanted) with two extensions:
// logits may be asked for at any of the item's tokens, and there is one block
// table per cache group.
#pragma once

#include "cache_manager.hpp"

namespace stride {

struct WorkItem {
    RequestKey request;
    std::vector<TokenId> tokens;
    size_t position;               // absolute index of tokens[0] in the request
    std::vector<int32_t> want;     // indices into `tokens` whose logits are wanted
};

struct PackedLayout {
    // Offsets (in int32 elements) into the packed buffer.
    size_t token_ids, positions, seq_of_token, logit_rows, q_start, q_len, ctx_len, state_slot;
    std::vector<size_t> slot_mapping, block_table;  // per group
    size_t total;
    size_t token_cap, seq_cap, row_cap, table_width;
};

inline PackedLayout make_layout(size_t groups, size_t token_cap, size_t seq_cap, size_t row_cap, size_t table_width) {
    PackedLayout l;
    auto round4 = [](size_t n) { return (n + 3) / 4 * 4; };  // keep every array 16-byte aligned
    size_t at = 0;
    auto take = [&](size_t n) {
        size_t here = at;
        at += round4(n);
        return here;
    };
    l.token_ids = take(token_cap);
    l.positions = take(token_cap);
    l.seq_of_token = take(token_cap);
    l.logit_rows = take(row_cap);
    l.q_start = take(seq_cap);
    l.q_len = take(seq_cap);
    l.ctx_len = take(seq_cap);
    l.state_slot = take(seq_cap);
    for (size_t g = 0; g < groups; ++g) l.slot_mapping.push_back(take(token_cap));
    for (size_t g = 0; g < groups; ++g) l.block_table.push_back(take(seq_cap * table_width));
    l.total = at;
    l.token_cap = token_cap;
    l.seq_cap = seq_cap;
    l.row_cap = row_cap;
    l.table_width = table_width;
    return l;
}

class StepBatch {
public:
    explicit StepBatch(const CacheManager& cache) : cache_(cache) {}

    // Adds one request's portion. The block tables must already cover
    // position + tokens.size(); this is checked here, on the host, so that no
    // kernel ever reads a page id that does not exist.
    void add(WorkItem item) {
        if (item.tokens.empty()) return;  // an empty portion is skipped, as in the reference
        for (auto& other : items_)
            if (other.request == item.request)
                throw std::invalid_argument("request " + std::to_string(item.request) + " appears twice in one step");
        size_t end = item.position + item.tokens.size();
        size_t need = cache_.pages_for(end);
        for (size_t g = 0; g < cache_.num_groups(); ++g) {
            auto& t = cache_.table(item.request, g);
            if (t.size() < need)
                throw std::out_of_range("request " + std::to_string(item.request) + ": position " + std::to_string(end - 1) +
                                        " needs page " + std::to_string(need - 1) + " but only " + std::to_string(t.size()) +
                                        " are mapped");
            for (size_t p = item.position / cache_.page_size(); p < need; ++p)
                if (t[p] < 0) throw std::out_of_range("a token would be written to a page that was given back");
        }
        for (int32_t w : item.want)
            if (w < 0 || size_t(w) >= item.tokens.size()) throw std::out_of_range("wanted logits outside the portion");
        num_tokens_ += item.tokens.size();
        num_rows_ += item.want.size();
        max_q_len_ = std::max(max_q_len_, item.tokens.size());
        max_ctx_ = std::max(max_ctx_, end);
        max_pages_ = std::max(max_pages_, need);
        items_.push_back(std::move(item));
    }

    size_t num_tokens() const { return num_tokens_; }
    size_t num_seqs() const { return items_.size(); }
    size_t num_rows() const { return num_rows_; }
    size_t max_q_len() const { return max_q_len_; }
    size_t max_ctx() const { return max_ctx_; }
    size_t max_pages() const { return max_pages_; }
    bool decode_only() const { return !items_.empty() && max_q_len_ == 1; }
    const std::vector<WorkItem>& items() const { return items_; }

    // Requests in the order of the logit rows.
    std::vector<RequestKey> row_requests() const {
        std::vector<RequestKey> out;
        for (auto& it : items_)
            for (size_t i = 0; i < it.want.size(); ++i) out.push_back(it.request);
        return out;
    }

    // Writes the arrays into `out` (layout.total int32), padding every array
    // to its capacity: padded tokens have seq_of_token -1 and slot -1, padded
    // sequences have q_len 0.
    // Only the wanted rows [row_offset, row_offset + row_count) are written, so
    // that a step that wants more rows than the layout holds can be served in
    // slices.
    void pack(const PackedLayout& l, int32_t* out, size_t row_offset = 0, size_t row_count = SIZE_MAX) const {
        if (row_count == SIZE_MAX) row_count = num_rows_ > row_offset ? num_rows_ - row_offset : 0;
        if (num_tokens_ > l.token_cap || items_.size() > l.seq_cap || row_count > l.row_cap || max_pages_ > l.table_width)
            throw std::invalid_argument("the step does not fit the packed layout");
        if (l.slot_mapping.size() != cache_.num_groups()) throw std::invalid_argument("layout and cache disagree on groups");
        std::fill(out, out + l.total, 0);
        std::fill(out + l.seq_of_token, out + l.seq_of_token + l.token_cap, -1);
        for (size_t g = 0; g < cache_.num_groups(); ++g) {
            std::fill(out + l.slot_mapping[g], out + l.slot_mapping[g] + l.token_cap, -1);
            std::fill(out + l.block_table[g], out + l.block_table[g] + l.seq_cap * l.table_width, -1);
        }
        size_t ps = cache_.page_size();
        size_t t = 0, row = 0;
        for (size_t s = 0; s < items_.size(); ++s) {
            auto& it = items_[s];
            out[l.q_start + s] = static_cast<int32_t>(t);
            out[l.q_len + s] = static_cast<int32_t>(it.tokens.size());
            out[l.ctx_len + s] = static_cast<int32_t>(it.position + it.tokens.size());
            out[l.state_slot + s] = cache_.state_slot(it.request);
            for (int32_t w : it.want) {
                if (row >= row_offset && row < row_offset + row_count)
                    out[l.logit_rows + (row - row_offset)] = static_cast<int32_t>(t + w);
                ++row;
            }
            for (size_t g = 0; g < cache_.num_groups(); ++g) {
                auto& table = cache_.table(it.request, g);
                std::copy(table.begin(), table.begin() + std::min(table.size(), l.table_width),
                          out + l.block_table[g] + s * l.table_width);
            }
            for (size_t j = 0; j < it.tokens.size(); ++j, ++t) {
                size_t pos = it.position + j;
                out[l.token_ids + t] = it.tokens[j];
                out[l.positions + t] = static_cast<int32_t>(pos);
                out[l.seq_of_token + t] = static_cast<int32_t>(s);
                for (size_t g = 0; g < cache_.num_groups(); ++g) {
                    PageId page = cache_.table(it.request, g)[pos / ps];
                    out[l.slot_mapping[g] + t] = static_cast<int32_t>(page * ps + pos % ps);
                }
            }
        }
    }

private:
    const CacheManager& cache_;
    std::vector<WorkItem> items_;
    size_t num_tokens_ = 0, num_rows_ = 0, max_q_len_ = 0, max_ctx_ = 0, max_pages_ = 0;
};

}  // namespace stride
