#include "step_planner.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace ti {

static inline int align32(int n) { return (n + 31) / 32 * 32; }

StepPlanner::StepPlanner(CacheBook* cache, int max_step_tokens, bool on_device)
    : cache_(cache), max_step_tokens_(max_step_tokens), on_device_(on_device), plans_(cache->groups.size(), nullptr) {}

StepPlanner::~StepPlanner() {
    for (int i = 0; i < 2; ++i) {
        if (staging_[i]) {
            if (on_device_) cudaFreeHost(staging_[i]);
            else std::free(staging_[i]);
        }
        if (events_[i]) cudaEventDestroy(events_[i]);
    }
    for (GroupPlan* p : plans_) delete p;
}

void StepPlanner::attach_plan(int group, GroupPlan* plan) {
    delete plans_[group];
    plans_[group] = plan;
    layouts_.clear();
    capacity_ = 0;
}

int StepPlanner::capacity() const {
    const int groups = std::max<int>(1, (int)cache_->groups.size());
    // A step of one token per sequence is never cut: it may have more tokens (up to max_seqs) than max_step_tokens.
    const int most_tokens = std::max(max_step_tokens_, cache_->max_seqs);
    int cap = align32(most_tokens) * (3 + groups + 1) + 4 * align32(cache_->max_seqs + 1) + 64;
    for (GroupPlan* p : plans_) {
        if (!p) continue;
        int most = 0;
        for (int b = 1; b <= cache_->max_seqs; ++b) most = std::max(most, p->words(b));
        cap += align32(most);
    }
    return cap;
}

const StepLayout& StepPlanner::layout(int n, int batch, int wanted) {
    const auto key = std::make_tuple(n, batch, wanted);
    auto it = layouts_.find(key);
    if (it != layouts_.end()) return it->second;
    StepLayout lay;
    lay.n = n; lay.batch = batch; lay.wanted = wanted;
    int off = 0;
    auto seg = [&off](int length) { const int o = off; off += align32(length); return o; };
    lay.ids = seg(n); lay.pos = seg(n); lay.slot = seg(n);
    for (size_t g = 0; g < cache_->groups.size(); ++g) lay.maps.push_back(seg(n));
    lay.seq = seg(batch); lay.cu = seg(batch + 1); lay.kv = seg(batch); lay.want = seg(wanted);
    lay.plan.assign(cache_->groups.size(), 0);
    lay.plan_words.assign(cache_->groups.size(), 0);
    if (n == batch)                                   // one token per sequence: the mixers' decode tables
        for (size_t g = 0; g < plans_.size(); ++g)
            if (plans_[g]) {
                lay.plan_words[g] = plans_[g]->words(batch);
                if (lay.plan_words[g] > 0) lay.plan[g] = seg(lay.plan_words[g]);
            }
    lay.end = off;
    if (layouts_.size() > 512) layouts_.clear();
    return layouts_[key] = lay;
}

int32_t* StepPlanner::staging(int* turn) {
    if (!capacity_) {
        capacity_ = capacity();
        for (int i = 0; i < 2; ++i) {
            if (on_device_) {
                if (cudaHostAlloc((void**)&staging_[i], (size_t)capacity_ * 4, cudaHostAllocDefault) != cudaSuccess) return nullptr;
                cudaEventCreateWithFlags(&events_[i], cudaEventDisableTiming);
            } else {
                staging_[i] = (int32_t*)std::malloc((size_t)capacity_ * 4);
            }
            if (staging_[i]) std::memset(staging_[i], 0, (size_t)capacity_ * 4);
        }
    }
    const int t = turn_;
    turn_ ^= 1;
    if (in_flight_[t]) {                              // the copy that last read this buffer has finished
        cudaEventSynchronize(events_[t]);
        in_flight_[t] = false;
    }
    *turn = t;
    return staging_[t];
}

int StepPlanner::upload(int turn, int count, int skip, cudaStream_t stream) {
    last_upload_bytes = (long long)(count - skip) * 4;
    if (on_device_) {
        const cudaError_t e = cudaMemcpyAsync(meta_ + skip, staging_[turn] + skip, (size_t)(count - skip) * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return ti_fail("the copy of a step's metadata to the device: %s", cudaGetErrorString(e)), 2;
        cudaEventRecord(events_[turn], stream);
        in_flight_[turn] = true;
    } else {
        std::memcpy(meta_ + skip, staging_[turn] + skip, (size_t)(count - skip) * 4);
    }
    return 0;
}

void StepPlanner::fill_plans(const StepLayout& lay, int32_t* st, const int64_t* lengths_after) {
    for (size_t g = 0; g < plans_.size(); ++g)
        if (lay.plan_words[g] > 0) plans_[g]->fill(lay.batch, st + lay.plan[g], lengths_after);
}

int StepPlanner::plan(int n_entries, const int* slots, const int* q_lens, const int* tokens, const int* want_counts, const int* want,
                      cudaStream_t stream) {
    int n = 0, nw = 0;
    for (int i = 0; i < n_entries; ++i) {
        if (!cache_->slots.is_held(slots[i])) return ti_fail("sequence slot %d is not held", slots[i]), 2;
        n += q_lens[i];
        nw += want_counts[i];
    }
    if (n > max_step_tokens_) return ti_fail("a step of %d tokens exceeds max_step_tokens %d", n, max_step_tokens_), 2;
    if (meta_ == nullptr) return ti_fail("the step planner has no device buffer"), 2;
    // Check the wanted places before anything is written.
    for (int i = 0, w = 0; i < n_entries; ++i)
        for (int j = 0; j < want_counts[i]; ++j, ++w)
            if (want[w] < 0 || want[w] >= q_lens[i])
                return ti_fail("wanted position %d is outside the %d tokens of entry %d", want[w], q_lens[i], i), 2;
    const StepLayout& lay = layout(n, n_entries, nw);
    int turn;
    int32_t* st = staging(&turn);
    if (!st) return ti_fail("no pinned memory for the step's staging buffers"), 2;
    if (lay.end > capacity_) return ti_fail("a step of %d tokens, %d sequences and %d wanted rows needs %d words of metadata; the buffers hold %d", n, n_entries, nw, lay.end, capacity_), 2;
    std::vector<int64_t> after(n_entries);
    int row = 0, wrow = lay.want, w = 0;
    for (int i = 0; i < n_entries; ++i) {
        const int slot = slots[i], m = q_lens[i];
        const int64_t start = cache_->lengths[slot];
        for (int t = 0; t < m; ++t) {
            st[lay.ids + row + t] = tokens[row + t];
            st[lay.pos + row + t] = (int32_t)(start + t);
            st[lay.slot + row + t] = slot;
        }
        for (size_t g = 0; g < cache_->groups.size(); ++g) {
            const PagedBook& book = cache_->groups[g];
            const int32_t* table = book.host_table.data() + (size_t)slot * book.max_pages_per_seq;
            const int P = book.page_size;
            for (int t = 0; t < m; ++t) {
                const int64_t p = start + t;
                st[lay.maps[g] + row + t] = (int32_t)((int64_t)table[p / P] * P + p % P);
            }
        }
        for (int j = 0; j < want_counts[i]; ++j, ++w) st[wrow++] = row + want[w];
        st[lay.cu + i] = row;
        st[lay.seq + i] = slot;
        st[lay.kv + i] = (int32_t)(start + m);
        after[i] = start + m;
        row += m;
    }
    st[lay.cu + n_entries] = row;
    if (n == n_entries) fill_plans(lay, st, after.data());
    return upload(turn, lay.end, 0, stream);
}

int StepPlanner::plan_decode(int batch, const int* slots, const int* tokens, cudaStream_t stream, int64_t* starts) {
    if (meta_ == nullptr) return ti_fail("the step planner has no device buffer"), 2;
    const StepLayout& lay = layout(batch, batch, batch);
    int turn;
    int32_t* st = staging(&turn);
    if (!st) return ti_fail("no pinned memory for the step's staging buffers"), 2;
    if (lay.end > capacity_) return ti_fail("a step of %d sequences needs %d words of metadata; the buffers hold %d", batch, lay.end, capacity_), 2;
    std::vector<int64_t> after(batch);
    for (int i = 0; i < batch; ++i) {
        const int slot = slots[i];
        if (!cache_->slots.is_held(slot)) return ti_fail("sequence slot %d is not held", slot), 2;
        const int64_t start = cache_->lengths[slot];
        if (tokens) st[lay.ids + i] = tokens[i];
        st[lay.pos + i] = (int32_t)start;
        st[lay.slot + i] = slot;
        for (size_t g = 0; g < cache_->groups.size(); ++g) {
            const PagedBook& book = cache_->groups[g];
            const int P = book.page_size;
            st[lay.maps[g] + i] = (int32_t)((int64_t)book.host_table[(size_t)slot * book.max_pages_per_seq + start / P] * P + start % P);
        }
        st[lay.cu + i] = i;
        st[lay.seq + i] = slot;
        st[lay.kv + i] = (int32_t)(start + 1);
        st[lay.want + i] = i;
        after[i] = start + 1;
        if (starts) starts[i] = start;
    }
    st[lay.cu + batch] = batch;
    fill_plans(lay, st, after.data());
    return upload(turn, lay.end, tokens ? 0 : align32(batch), stream);
}

}  // namespace ti
