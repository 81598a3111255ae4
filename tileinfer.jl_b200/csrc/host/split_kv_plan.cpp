// The decode-attention kernel's work tables (csrc/attention_decode.cu), as a plan the step planner fills.
//
// A decode step of B sequences launches B x splits work slots per KV head; the split count is fixed by the
// batch size alone, so that a captured step stays valid whatever the lengths are (the reference fixes its
// split count per model: src/ops/tile/attention.jl:250-263). The tables share the slots out among the
// sequences by length: every sequence gets one part, the remaining slots go in proportion to the sequences'
// pages, so that a long sequence among short ones is read by more blocks (with equal lengths every sequence
// gets `splits` parts). A sequence's slots are consecutive.
//   work[slot] = (sequence << 16 | part << 8 | parts, or -1: no work; the sequence's length)
//   seq[sequence] = first slot << 8 | parts
// The shares change only when a sequence starts a new page, and are kept until then.
#include "host_common.h"

#include <algorithm>
#include <map>

namespace {

inline int align32(int n) { return (n + 31) / 32 * 32; }

// parts[b] and first[b] of `batch` sequences with `pages[b]` pages sharing batch x splits slots; returns the slots used.
int share_slots(int batch, int splits, int max_parts, const int64_t* pages, int* parts, int* first) {
    int64_t total = 0;
    for (int b = 0; b < batch; ++b) total += pages[b];
    const int slots = batch * splits;
    int used = 0;
    for (int b = 0; b < batch; ++b) {
        int64_t p = 1 + ((int64_t)(slots - batch) * pages[b]) / total;
        p = std::min<int64_t>(std::min<int64_t>(p, max_parts), pages[b]);
        parts[b] = (int)p;
        first[b] = used;
        used += (int)p;
    }
    return used;
}

void write_tables(int batch, int slots, int used, const int* parts, const int* first, const int64_t* lengths, int32_t* work, int32_t* seq) {
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < parts[b]; ++i) {
            work[2 * (first[b] + i)] = (b << 16) | (i << 8) | parts[b];
            work[2 * (first[b] + i) + 1] = (int32_t)lengths[b];
        }
        seq[b] = (first[b] << 8) | parts[b];
    }
    for (int i = used; i < slots; ++i) {
        work[2 * i] = -1;
        work[2 * i + 1] = 0;
    }
}

class SplitKvPlan : public ti::GroupPlan {
public:
    SplitKvPlan(int kv_heads, int page_size, long long pool_tokens, int sm_count, int max_parts)
        : kv_heads_(kv_heads), page_size_(page_size), pool_tokens_(pool_tokens), sm_count_(sm_count), max_parts_(max_parts) {}

    // Two blocks fit an SM: at most two blocks per SM, so that none has to wait for a second wave.
    int splits(int batch) const {
        const long long want = (2LL * sm_count_) / std::max(1, batch * kv_heads_);
        const long long most = (pool_tokens_ + 63) / 64;
        return (int)std::max<long long>(1, std::min<long long>(std::min<long long>(want, 32), most));
    }
    int words(int batch) override {
        const int s = splits(batch);
        return s > 1 ? align32(2 * batch * s) + align32(batch) : 0;
    }
    void fill(int batch, int32_t* out, const int64_t* lengths) override {
        const int s = splits(batch), slots = batch * s;
        Held& held = held_[batch];
        std::vector<int64_t> pages(batch);
        for (int b = 0; b < batch; ++b) pages[b] = std::max<int64_t>((lengths[b] + page_size_ - 1) / page_size_, 1);
        if (held.pages != pages) {
            held.pages = pages;
            held.parts.assign(batch, 1);
            held.first.assign(batch, 0);
            held.used = share_slots(batch, s, max_parts_, pages.data(), held.parts.data(), held.first.data());
        }
        write_tables(batch, slots, held.used, held.parts.data(), held.first.data(), lengths, out, out + align32(2 * slots));
    }

private:
    struct Held {
        std::vector<int64_t> pages;
        std::vector<int> parts, first;
        int used = 0;
    };
    int kv_heads_, page_size_;
    long long pool_tokens_;
    int sm_count_, max_parts_;
    std::map<int, Held> held_;
};

}  // namespace

// `max_parts`: the most parts of one sequence (the combine kernel's limit). The caller hands the plan to a step
// planner (ti_planner_attach_plan), which owns it from then on, or frees it with ti_group_plan_destroy.
extern "C" void* ti_split_kv_plan_create(int kv_heads, int page_size, long long pool_tokens, int sm_count, int max_parts) {
    if (kv_heads < 1 || page_size < 1 || sm_count < 1 || max_parts < 1 || max_parts > 255) {
        ti_fail("split_kv_plan: bad sizes kv_heads=%d page=%d sms=%d max_parts=%d", kv_heads, page_size, sm_count, max_parts);
        return nullptr;
    }
    return static_cast<ti::GroupPlan*>(new SplitKvPlan(kv_heads, page_size, pool_tokens, sm_count, max_parts));
}

extern "C" int ti_split_kv_plan_splits(void* plan, int batch) {
    return static_cast<SplitKvPlan*>(static_cast<ti::GroupPlan*>(plan))->splits(batch);
}

// The tables for explicit sizes (tests, benchmarks): work[2 * batch * splits], seq[batch].
extern "C" int ti_split_kv_tables(int batch, int splits, int page_size, int max_parts, const long long* lengths, int* work, int* seq) {
    if (batch < 1 || splits < 1 || page_size < 1 || max_parts < 1) return ti_fail("split_kv_tables: bad sizes"), 2;
    std::vector<int64_t> pages(batch), len(batch);
    std::vector<int> parts(batch), first(batch);
    for (int b = 0; b < batch; ++b) {
        len[b] = lengths[b];
        pages[b] = std::max<int64_t>((len[b] + page_size - 1) / page_size, 1);
    }
    const int used = share_slots(batch, splits, max_parts, pages.data(), parts.data(), first.data());
    write_tables(batch, batch * splits, used, parts.data(), first.data(), len.data(), work, seq);
    return 0;
}
