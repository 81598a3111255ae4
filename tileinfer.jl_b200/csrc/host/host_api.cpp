// C entry points of the host runtime: the cache's books and the step planner, for the Python layer (ctypes).
// Return codes: 0; 1: out of pages (detail in the out-parameters); 2: refused, text in ti_last_error();
// 3: out of slots. Handles are opaque pointers owned by the caller.
#include "step_planner.h"

using ti::CacheBook;
using ti::NumberPool;
using ti::PagedBook;
using ti::StepPlanner;

// ---- a pool of numbers on its own
extern "C" void* ti_pool_create(int count) { return new NumberPool(count); }
extern "C" void ti_pool_destroy(void* p) { delete (NumberPool*)p; }
extern "C" int ti_pool_take(void* p) { return ((NumberPool*)p)->take(); }
extern "C" int ti_pool_give(void* p, int n) { return ((NumberPool*)p)->give(n) ? 0 : 2; }
extern "C" int ti_pool_free(void* p) { return ((NumberPool*)p)->free_count(); }
extern "C" int ti_pool_held(void* p) { return ((NumberPool*)p)->held_count(); }
extern "C" int ti_pool_is_held(void* p, int n) { return ((NumberPool*)p)->is_held(n) ? 1 : 0; }

// ---- the cache's books
extern "C" void* ti_cache_create(int max_seqs, long long max_seq_len, int has_state) {
    CacheBook* c = new CacheBook(max_seqs, max_seq_len);
    c->has_state = has_state != 0;
    return c;
}
extern "C" void ti_cache_destroy(void* c) { delete (CacheBook*)c; }
extern "C" int ti_cache_add_group(void* c, int num_pages, int page_size, int window, int granule, int max_pages_per_seq) {
    CacheBook* cache = (CacheBook*)c;
    cache->groups.emplace_back(num_pages, page_size, window, granule, cache->max_seqs, max_pages_per_seq);
    return (int)cache->groups.size() - 1;
}
// Where the group's block table and value pool live (device memory when on_device, else host memory).
extern "C" void ti_cache_group_storage(void* c, int group, int* device_table, long long table_stride, void* value_pool, int layers,
                                       long long layer_stride, long long page_bytes, int on_device) {
    PagedBook& g = ((CacheBook*)c)->groups[group];
    g.device_table = device_table;
    g.table_stride = table_stride;
    g.value_pool = (char*)value_pool;
    g.layers = layers;
    g.layer_stride = (size_t)layer_stride;
    g.page_bytes = (size_t)page_bytes;
    g.on_device = on_device != 0;
}
extern "C" int ti_cache_alloc_slot(void* c) { return ((CacheBook*)c)->alloc_slot(); }
extern "C" int ti_cache_free_slot(void* c, int slot) { return ((CacheBook*)c)->free_slot(slot); }
extern "C" long long ti_cache_length(void* c, int slot) {
    CacheBook* cache = (CacheBook*)c;
    return slot >= 0 && slot < cache->max_seqs ? cache->lengths[slot] : -1;
}
extern "C" void ti_cache_lengths(void* c, int n, const int* slots, long long* out) {
    CacheBook* cache = (CacheBook*)c;
    for (int i = 0; i < n; ++i) out[i] = slots[i] >= 0 && slots[i] < cache->max_seqs ? cache->lengths[slots[i]] : -1;
}
extern "C" int ti_cache_slots_held(void* c) { return ((CacheBook*)c)->slots.held_count(); }
extern "C" int ti_cache_slot_is_held(void* c, int slot) { return ((CacheBook*)c)->slots.is_held(slot) ? 1 : 0; }
extern "C" int ti_cache_reserve(void* c, int n, const int* slots, const long long* counts, long long chunk_tokens, cudaStream_t stream,
                                long long* needed, long long* free_pages) {
    int64_t need = 0, free_now = 0;
    const int rc = ((CacheBook*)c)->reserve(n, slots, (const int64_t*)counts, chunk_tokens, stream, &need, &free_now);
    if (needed) *needed = need;
    if (free_pages) *free_pages = free_now;
    return rc;
}
extern "C" int ti_cache_prepare(void* c, int n, const int* slots, const long long* counts, cudaStream_t stream) {
    return ((CacheBook*)c)->prepare(n, slots, (const int64_t*)counts, stream);
}
extern "C" int ti_cache_advance(void* c, int slot, long long n) { return ((CacheBook*)c)->advance(slot, n); }
extern "C" int ti_cache_advance_many(void* c, int n, const int* slots, const long long* counts) {
    for (int i = 0; i < n; ++i)
        if (int rc = ((CacheBook*)c)->advance(slots[i], counts[i])) return rc;
    return 0;
}
extern "C" int ti_cache_truncate(void* c, int slot, long long length) { return ((CacheBook*)c)->truncate(slot, length); }
// A group's books, for inspection: pages free / held, one sequence's table (-1: given back), its first held page.
extern "C" int ti_group_pages_free(void* c, int group) { return ((CacheBook*)c)->groups[group].pages.free_count(); }
extern "C" int ti_group_pages_held(void* c, int group) { return ((CacheBook*)c)->groups[group].pages.held_count(); }
extern "C" int ti_group_page_is_held(void* c, int group, int page) { return ((CacheBook*)c)->groups[group].pages.is_held(page) ? 1 : 0; }
extern "C" int ti_group_table(void* c, int group, int slot, int* out, int capacity) {
    const std::vector<int>& t = ((CacheBook*)c)->groups[group].tables[slot];
    for (int i = 0; i < (int)t.size() && i < capacity; ++i) out[i] = t[i];
    return (int)t.size();
}
extern "C" int ti_group_first(void* c, int group, int slot) { return ((CacheBook*)c)->groups[group].first[slot]; }
extern "C" const int* ti_group_host_table(void* c, int group) { return ((CacheBook*)c)->groups[group].host_table.data(); }
extern "C" long long ti_group_peak_pages(void* c, int group, int n, const int* slots, const long long* counts, long long chunk_tokens) {
    CacheBook* cache = (CacheBook*)c;
    return cache->groups[group].peak_pages(n, slots, (const int64_t*)counts, cache->lengths, chunk_tokens);
}

// ---- the step planner
extern "C" void* ti_planner_create(void* cache, int max_step_tokens, int on_device) {
    return new StepPlanner((CacheBook*)cache, max_step_tokens, on_device != 0);
}
extern "C" void ti_planner_destroy(void* p) { delete (StepPlanner*)p; }
extern "C" void ti_planner_attach_plan(void* p, int group, void* plan) { ((StepPlanner*)p)->attach_plan(group, (ti::GroupPlan*)plan); }
extern "C" void ti_group_plan_destroy(void* plan) { delete (ti::GroupPlan*)plan; }
extern "C" int ti_planner_capacity(void* p) { return ((StepPlanner*)p)->capacity(); }
extern "C" void ti_planner_set_meta(void* p, int* meta) { ((StepPlanner*)p)->set_meta(meta); }
// out: ids, pos, slot, seq, cu, kv, want, end, then per paged group: map offset, plan offset, plan words.
extern "C" void ti_planner_layout(void* p, int n, int batch, int wanted, int* out) {
    const ti::StepLayout& lay = ((StepPlanner*)p)->layout(n, batch, wanted);
    const int head[8] = {lay.ids, lay.pos, lay.slot, lay.seq, lay.cu, lay.kv, lay.want, lay.end};
    for (int i = 0; i < 8; ++i) out[i] = head[i];
    for (size_t g = 0; g < lay.maps.size(); ++g) {
        out[8 + 3 * g] = lay.maps[g];
        out[9 + 3 * g] = lay.plan[g];
        out[10 + 3 * g] = lay.plan_words[g];
    }
}
extern "C" int ti_planner_plan(void* p, int n_entries, const int* slots, const int* q_lens, const int* tokens, const int* want_counts,
                               const int* want, cudaStream_t stream) {
    return ((StepPlanner*)p)->plan(n_entries, slots, q_lens, tokens, want_counts, want, stream);
}
extern "C" int ti_planner_plan_decode(void* p, int batch, const int* slots, const int* tokens, cudaStream_t stream, long long* starts) {
    return ((StepPlanner*)p)->plan_decode(batch, slots, tokens, stream, (int64_t*)starts);
}
extern "C" long long ti_planner_last_upload_bytes(void* p) { return ((StepPlanner*)p)->last_upload_bytes; }
