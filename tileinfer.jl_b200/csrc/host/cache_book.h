// The cache's books, on the host: which sequence slots are held, how long each sequence is, and for every
// group of layers with paged storage which pages each sequence holds. The storage itself (the pools) is
// allocated by the caller; the books only hand out numbers and keep the block tables.
//
// AntoineBut/TileInfer.jl's BlockManager is the model for one sequence's pages (src/kv/block_manager.jl:
// 39-100: pages in increasing order, a reservation that cannot be met changes nothing, truncate returns
// pages); slots, groups, windows and chunk-wise reservation are this library's own.
#pragma once
#include "host_common.h"

#include <cuda_runtime.h>

namespace ti {

struct PageWrite {
    int slot, col, page;          // block_table[slot][col] = page; the page's values are zeroed
};

class PagedBook {
public:
    PagedBook(int num_pages, int page_size, int window, int granule, int max_seqs, int max_pages_per_seq);
    int pages_needed(int slot, int64_t new_length) const;
    int grow(int slot, int64_t new_length);                 // 0, or 2 with the text in ti_last_error()
    int first_needed_page(int64_t length) const;
    int release(int slot, int64_t length);
    int shrink(int slot, int64_t new_length);               // 0 or 2
    int64_t peak_pages(int n, const int* slots, const int64_t* counts, const std::vector<int64_t>& lengths, int64_t chunk_tokens) const;
    void flush(cudaStream_t stream);

    int num_pages, page_size, window, granule, max_seqs, max_pages_per_seq;
    NumberPool pages;
    std::vector<std::vector<int>> tables;     // per slot: logical page index -> page, -1 once given back
    std::vector<int> first;                   // per slot: first logical page still held
    std::vector<int32_t> host_table;          // [max_seqs][max_pages_per_seq], what the step planner reads
    std::vector<PageWrite> pending;           // table entries and fresh pages not yet written to the device
    // Where the device's copy of the block table and the value pool are (set once by the owner of the storage).
    int32_t* device_table = nullptr;
    long long table_stride = 0;
    char* value_pool = nullptr;               // [layers][pages][page_bytes]
    int layers = 0;
    size_t layer_stride = 0, page_bytes = 0;
    bool on_device = false;
};

class CacheBook {
public:
    CacheBook(int max_seqs, int64_t max_seq_len) : max_seqs(max_seqs), max_seq_len(max_seq_len), slots(max_seqs), lengths(max_seqs, -1) {}
    int alloc_slot();
    int free_slot(int slot);
    // 0; 1: out of pages (needed, free returned); 2: refused, text in ti_last_error()
    int reserve(int n, const int* slot, const int64_t* count, int64_t chunk_tokens, cudaStream_t stream, int64_t* needed, int64_t* free_pages);
    int prepare(int n, const int* slot, const int64_t* count, cudaStream_t stream);
    int advance(int slot, int64_t n);
    int truncate(int slot, int64_t length);

    int max_seqs;
    int64_t max_seq_len;
    NumberPool slots;
    std::vector<int64_t> lengths;             // -1: the slot is not held
    std::vector<PagedBook> groups;
    bool has_state = false;                   // a group with a per-sequence state: no roll-back
};

// page_init.cu: block_table[slot][col] = page and zero the page's values in every layer, for up to 64 writes a launch.
int launch_page_writes(const PageWrite* writes, int count, int32_t* device_table, long long table_stride, char* value_pool, int layers,
                       size_t layer_stride, size_t page_bytes, cudaStream_t stream);

}  // namespace ti
