#include "cache_book.h"

#include <algorithm>
#include <cstring>

namespace ti {

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

PagedBook::PagedBook(int num_pages, int page_size, int window, int granule, int max_seqs, int max_pages_per_seq)
    : num_pages(num_pages), page_size(page_size), window(window), granule(std::max(1, granule)), max_seqs(max_seqs),
      max_pages_per_seq(max_pages_per_seq), pages(num_pages), tables(max_seqs), first(max_seqs, 0),
      host_table((size_t)max_seqs * max_pages_per_seq, 0) {}

int PagedBook::pages_needed(int slot, int64_t new_length) const {
    return (int)std::max<int64_t>(0, ceil_div(new_length, page_size) - (int64_t)tables[slot].size());
}

int PagedBook::grow(int slot, int64_t new_length) {
    const int need = pages_needed(slot, new_length);
    if (!need) return 0;
    std::vector<int>& table = tables[slot];
    if ((int)table.size() + need > max_pages_per_seq)
        return ti_fail("a sequence of %lld positions needs more than %d pages", (long long)new_length, max_pages_per_seq), 2;
    for (int i = 0; i < need; ++i) {
        const int page = pages.take();
        if (page < 0) return ti_fail("KV cache full while growing a sequence that was reserved"), 2;
        const int col = (int)table.size();
        table.push_back(page);
        host_table[(size_t)slot * max_pages_per_seq + col] = page;
        pending.push_back(PageWrite{slot, col, page});
    }
    return 0;
}

int PagedBook::first_needed_page(int64_t length) const {
    if (!window) return 0;
    const int64_t key = std::max<int64_t>(0, length - window + 1);
    return (int)(key / page_size / granule * granule);
}

int PagedBook::release(int slot, int64_t length) {
    std::vector<int>& table = tables[slot];
    if (!window || table.empty()) return 0;
    const int a = first[slot], b = std::min<int>(first_needed_page(length), (int)table.size());
    for (int i = a; i < b; ++i) {
        pages.give(table[i]);
        table[i] = -1;
    }
    if (b > a) first[slot] = b;
    return std::max(0, b - a);
}

int PagedBook::shrink(int slot, int64_t new_length) {
    std::vector<int>& table = tables[slot];
    const int keep = (int)ceil_div(new_length, page_size);
    if (keep && first_needed_page(new_length) < first[slot])
        return ti_fail("cannot roll back to %lld positions: the pages of its window were given back", (long long)new_length), 2;
    for (int i = (int)table.size() - 1; i >= keep; --i)
        if (table[i] >= 0) pages.give(table[i]);
    if ((int)table.size() > keep) table.resize(keep);
    if (table.empty()) first[slot] = 0;
    return 0;
}

// Most pages beyond those held now that the growth needs at any time when it runs in token order in chunks of
// `chunk_tokens` and every chunk's end gives back what fell out of the window.
int64_t PagedBook::peak_pages(int n, const int* slots, const int64_t* counts, const std::vector<int64_t>& lengths, int64_t chunk_tokens) const {
    std::vector<int64_t> logical(max_seqs, 0), length(max_seqs, 0);
    std::vector<int> first_now(max_seqs, 0), touched;
    for (int i = 0; i < n; ++i) {
        logical[slots[i]] = (int64_t)tables[slots[i]].size();
        first_now[slots[i]] = first[slots[i]];
        length[slots[i]] = lengths[slots[i]];
    }
    int64_t extra = 0, peak = 0;
    int64_t room = chunk_tokens > 0 ? chunk_tokens : (int64_t)1 << 62;
    for (int i = 0; i < n; ++i) {
        const int slot = slots[i];
        int64_t a = 0;
        while (a < counts[i]) {
            const int64_t take = std::min(room, counts[i] - a);
            length[slot] += take;
            const int64_t need = std::max<int64_t>(0, ceil_div(length[slot], page_size) - logical[slot]);
            logical[slot] += need;
            extra += need;
            touched.push_back(slot);
            a += take;
            room -= take;
            if (room == 0) {
                peak = std::max(peak, extra);
                for (int s : touched) {
                    const int64_t b = std::min<int64_t>(first_needed_page(length[s]), logical[s]);
                    extra -= std::max<int64_t>(0, b - first_now[s]);
                    first_now[s] = (int)std::max<int64_t>(first_now[s], b);
                }
                touched.clear();
                room = chunk_tokens;
            }
        }
    }
    return std::max(peak, extra);
}

// The block table's new entries and the zeroing of fresh pages. A page's last user may have left anything in
// it: keys beyond a sequence's length are masked by selection, but their values take part in P V with weight
// 0, and 0 times a stale infinity or NaN is NaN, so values are zeroed when a page is taken. The writes travel
// as kernel arguments (no staging buffer that a later call could overwrite before the copy has run).
void PagedBook::flush(cudaStream_t stream) {
    if (pending.empty()) return;
    if (device_table != nullptr) {
        if (on_device) {
            for (size_t a = 0; a < pending.size(); a += 64)
                launch_page_writes(pending.data() + a, (int)std::min<size_t>(64, pending.size() - a), device_table, table_stride, value_pool,
                                   layers, layer_stride, page_bytes, stream);
        } else {
            for (const PageWrite& w : pending) {
                device_table[(size_t)w.slot * table_stride + w.col] = w.page;
                for (int l = 0; l < layers; ++l) std::memset(value_pool + l * layer_stride + (size_t)w.page * page_bytes, 0, page_bytes);
            }
        }
    }
    pending.clear();
}

int CacheBook::alloc_slot() {
    const int slot = slots.take();
    if (slot >= 0) lengths[slot] = 0;
    return slot;
}

int CacheBook::free_slot(int slot) {
    if (!slots.is_held(slot)) return ti_fail("sequence slot %d is not held (freed twice, or never allocated)", slot), 2;
    for (PagedBook& g : groups) g.shrink(slot, 0);
    lengths[slot] = -1;
    slots.give(slot);
    return 0;
}

int CacheBook::reserve(int n, const int* slot, const int64_t* count, int64_t chunk_tokens, cudaStream_t stream, int64_t* needed,
                       int64_t* free_pages) {
    int64_t total = 0;
    for (int i = 0; i < n; ++i) {
        if (!slots.is_held(slot[i])) return ti_fail("sequence slot %d is not held", slot[i]), 2;
        if (lengths[slot[i]] + count[i] > max_seq_len)
            return ti_fail("sequence would reach %lld positions; the cache was sized for sequences of at most %lld",
                           (long long)(lengths[slot[i]] + count[i]), (long long)max_seq_len), 2;
        total += count[i];
    }
    const bool chunked = chunk_tokens > 0 && total > chunk_tokens;
    for (PagedBook& g : groups) {
        int64_t need = 0;
        if (g.window && chunked) need = g.peak_pages(n, slot, count, lengths, chunk_tokens);
        else
            for (int i = 0; i < n; ++i) need += g.pages_needed(slot[i], lengths[slot[i]] + count[i]);
        if (need > g.pages.free_count()) {
            if (needed) *needed = need;
            if (free_pages) *free_pages = g.pages.free_count();
            return 1;
        }
    }
    for (PagedBook& g : groups) {
        if (g.window && chunked) continue;             // taken chunk by chunk, in prepare()
        for (int i = 0; i < n; ++i)
            if (int rc = g.grow(slot[i], lengths[slot[i]] + count[i])) return rc;
        g.flush(stream);
    }
    return 0;
}

int CacheBook::prepare(int n, const int* slot, const int64_t* count, cudaStream_t stream) {
    for (PagedBook& g : groups) {
        if (!g.window) continue;
        for (int i = 0; i < n; ++i)
            if (int rc = g.grow(slot[i], lengths[slot[i]] + count[i])) return rc;
        g.flush(stream);
    }
    return 0;
}

int CacheBook::advance(int slot, int64_t n) {
    if (!slots.is_held(slot)) return ti_fail("sequence slot %d is not held", slot), 2;
    lengths[slot] += n;
    for (PagedBook& g : groups)
        if (g.window) g.release(slot, lengths[slot]);
    return 0;
}

int CacheBook::truncate(int slot, int64_t length) {
    if (!slots.is_held(slot)) return ti_fail("sequence slot %d is not held", slot), 2;
    if (length < 0 || length > lengths[slot])
        return ti_fail("cannot truncate a sequence of length %lld to %lld", (long long)lengths[slot], (long long)length), 2;
    if (has_state && length != lengths[slot]) return ti_fail("layers with a per-sequence state cannot roll back"), 2;
    for (PagedBook& g : groups)          // every group must be able to before any of them does
        if (length > 0 && g.first_needed_page(length) < g.first[slot])
            return ti_fail("cannot roll back to %lld positions: the pages of its window were given back", (long long)length), 2;
    for (PagedBook& g : groups)
        if (int rc = g.shrink(slot, length)) return rc;
    lengths[slot] = length;
    return 0;
}

}  // namespace ti
