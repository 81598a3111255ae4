// New pages of the cache: their block-table entries on the device and their values zeroed, in one launch.
//
// A sequence that grows past a page's end takes the lowest free page (AntoineBut/TileInfer.jl
// src/kv/block_manager.jl:58-65 hands them out the same way). The device's copy of the block table gets
// the new entry, and the page's VALUES are zeroed in every layer of the group: a page's last user may have
// left anything in it, keys beyond a sequence's length are masked by selection, but values take part in
// P V with weight 0, and 0 times a stale infinity or NaN is NaN. The writes travel as kernel arguments, so
// no staging buffer has to outlive the call.
#include "common.cuh"
#include "host/cache_book.h"

namespace {

struct PageWrites {
    int count;
    ti::PageWrite w[64];
};

__global__ void page_writes_kernel(PageWrites writes, int* table, long long table_stride, char* value_pool, size_t layer_stride,
                                   size_t page_bytes) {
    const ti::PageWrite w = writes.w[blockIdx.x];
    pdl_enter();
    if (blockIdx.y == 0 && threadIdx.x == 0) table[(size_t)w.slot * table_stride + w.col] = w.page;
    char* page = value_pool + blockIdx.y * layer_stride + (size_t)w.page * page_bytes;
    if ((page_bytes & 15) == 0 && ((uintptr_t)page & 15) == 0) {
        uint4* p = reinterpret_cast<uint4*>(page);
        for (size_t i = threadIdx.x; i < page_bytes / 16; i += blockDim.x) p[i] = make_uint4(0u, 0u, 0u, 0u);
    } else {
        for (size_t i = threadIdx.x; i < page_bytes; i += blockDim.x) page[i] = 0;
    }
}

}  // namespace

namespace ti {

int launch_page_writes(const PageWrite* writes, int count, int32_t* device_table, long long table_stride, char* value_pool, int layers,
                       size_t layer_stride, size_t page_bytes, cudaStream_t stream) {
    if (count <= 0) return 0;
    TI_REQUIRE(count <= 64 && layers >= 1 && layers <= 65535, "page writes: %d writes, %d layers in one launch", count, layers);
    PageWrites batch;
    batch.count = count;
    for (int i = 0; i < count; ++i) batch.w[i] = writes[i];
    ti_launch(page_writes_kernel, dim3(count, layers), dim3(256), 0, stream, batch, device_table, table_stride, value_pool, layer_stride,
              page_bytes);
    return ti_check_launch("page_writes");
}

}  // namespace ti
