// One step of the decode loop, enqueued by ONE call: sample the rows of the last step's logits, start the
// tokens' copy to the host, hand the tokens to the next step as its ids, reserve the next positions, upload
// the next step's metadata and launch its captured graph. The host then reads the tokens (`wait`) while the
// device runs that next step: it is one step behind, as in AntoineBut/TileInfer.jl's pipelined loop
// (generate_pipelined!, src/engine/runner.jl:157-191), here for a batch. NVTX ranges mark the phases as the
// reference's do (src/engine/runner.jl:77-97, 171-175: sample, upload, replay, wait).
#include "common.cuh"
#include "host/step_planner.h"

#include <nvtx3/nvToolsExt.h>

extern "C" int ti_argmax(const float* logits, long long ld, int n_rows, int vocab, int* out, int* out2, float* ws_val, int* ws_idx,
                         unsigned* counters, cudaStream_t stream);
extern "C" int ti_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k, float top_p,
                         const unsigned* seeds, unsigned* counters, int* out, int* out2, cudaStream_t stream);

namespace {

struct RowMap {
    int count, base;
    int rows[256];
};

// ids[base + j] = tokens[rows[j]], and the sampler's per-row state compacted the same way (sequences that left
// the batch drop out). rows[j] >= base + j and ascending, so reading everything before writing anything within
// the block, and running the chunks of 256 in ascending order, never overwrites a value that is still needed.
__global__ void keep_rows_kernel(RowMap map, const int* tokens, int* ids, unsigned* seeds, unsigned* counters) {
    pdl_enter();
    const int j = threadIdx.x;
    int token = 0;
    unsigned seed = 0, counter = 0;
    if (j < map.count) {
        token = __ldcg(tokens + map.rows[j]);
        seed = __ldcg(seeds + map.rows[j]);
        counter = __ldcg(counters + map.rows[j]);
    }
    __syncthreads();
    if (j < map.count) {
        ids[map.base + j] = token;
        seeds[map.base + j] = seed;
        counters[map.base + j] = counter;
    }
}

}  // namespace

namespace ti {

class DecodeLoop {
public:
    DecodeLoop(CacheBook* cache, StepPlanner* planner, int max_rows, int vocab, unsigned* seeds, unsigned* counters, int* tokens,
               float* ws_val, int* ws_idx, unsigned* ws_counters)
        : cache_(cache), planner_(planner), max_rows_(max_rows), vocab_(vocab), seeds_(seeds), counters_(counters), tokens_(tokens),
          ws_val_(ws_val), ws_idx_(ws_idx), ws_counters_(ws_counters) {}
    ~DecodeLoop() {
        for (int i = 0; i < 2; ++i) {
            if (host_[i]) cudaFreeHost(host_[i]);
            if (events_[i]) cudaEventDestroy(events_[i]);
        }
    }

    int enqueue(const float* logits, long long ld, int rows, float temperature, int top_k, float top_p, int n_next, const int* next_rows,
                const int* next_slots, cudaGraphExec_t graph, int* next_ids, cudaStream_t stream, long long* needed, long long* free_pages) {
        TI_REQUIRE(rows >= 1 && rows <= max_rows_ && n_next >= 0 && n_next <= rows, "decode loop: %d rows, %d go on, room for %d", rows,
                   n_next, max_rows_);
        if (!host_[0]) {
            for (int i = 0; i < 2; ++i) {
                if (cudaHostAlloc((void**)&host_[i], (size_t)max_rows_ * sizeof(int), cudaHostAllocDefault) != cudaSuccess)
                    return ti_fail("decode loop: no pinned memory for %d tokens", max_rows_);
                cudaEventCreateWithFlags(&events_[i], cudaEventDisableTiming);
            }
        }
        bool all = n_next == rows;
        for (int j = 0; all && j < n_next; ++j) all = next_rows[j] == j;
        // If a page is missing for the next step, nothing of this call may have happened.
        std::vector<int64_t> ones(n_next, 1);
        if (n_next > 0) {
            int64_t need = 0, free_now = 0;
            const int rc = cache_->reserve(n_next, next_slots, ones.data(), 0, stream, &need, &free_now);
            if (rc == 1) {
                if (needed) *needed = need;
                if (free_pages) *free_pages = free_now;
                return 4;
            }
            if (rc) return rc;
        }
        nvtxRangePushA("sample");
        int* direct = (all && n_next > 0) ? next_ids : nullptr;       // every row goes on: the sampler writes the next ids itself
        int rc = temperature > 0.f ? ti_sample(logits, ld, rows, vocab_, temperature, top_k, top_p, seeds_, counters_, tokens_, direct, stream)
                                   : ti_argmax(logits, ld, rows, vocab_, tokens_, direct, ws_val_, ws_idx_, ws_counters_, stream);
        nvtxRangePop();
        if (rc) return rc;
        turn_ ^= 1;
        const cudaError_t copied = cudaMemcpyAsync(host_[turn_], tokens_, (size_t)rows * sizeof(int), cudaMemcpyDeviceToHost, stream);
        if (copied != cudaSuccess) return ti_fail("the copy of a step's tokens to the host: %s", cudaGetErrorString(copied));
        cudaEventRecord(events_[turn_], stream);
        pending_rows_ = rows;
        if (n_next == 0) return 0;
        if (!all) {
            for (int base = 0; base < n_next; base += 256) {
                RowMap map;
                map.count = std::min(256, n_next - base);
                map.base = base;
                for (int j = 0; j < map.count; ++j) {
                    TI_REQUIRE(next_rows[base + j] >= base + j && next_rows[base + j] < rows && (base + j == 0 || next_rows[base + j] > next_rows[base + j - 1]),
                               "decode loop: the rows that go on must be ascending");
                    map.rows[j] = next_rows[base + j];
                }
                ti_launch(keep_rows_kernel, dim3(1), dim3(256), 0, stream, map, (const int*)tokens_, next_ids, seeds_, counters_);
            }
            if ((rc = ti_check_launch("keep_rows"))) return rc;
        }
        nvtxRangePushA("upload");
        rc = planner_->plan_decode(n_next, next_slots, nullptr, stream, nullptr);
        nvtxRangePop();
        if (rc) return rc;
        nvtxRangePushA("replay");
        const cudaError_t e = cudaGraphLaunch(graph, stream);
        nvtxRangePop();
        if (e != cudaSuccess) return ti_fail("decode loop: graph launch: %s", cudaGetErrorString(e));
        for (int j = 0; j < n_next; ++j) cache_->advance(next_slots[j], 1);
        return 0;
    }

    int wait(int* out, int rows) {
        TI_REQUIRE(rows == pending_rows_, "decode loop: %d tokens asked, %d are on their way", rows, pending_rows_);
        nvtxRangePushA("wait for tokens");
        const cudaError_t e = cudaEventSynchronize(events_[turn_]);
        nvtxRangePop();
        if (e != cudaSuccess) return ti_fail("decode loop: %s", cudaGetErrorString(e));
        for (int i = 0; i < rows; ++i) out[i] = host_[turn_][i];
        pending_rows_ = 0;
        return 0;
    }

private:
    CacheBook* cache_;
    StepPlanner* planner_;
    int max_rows_, vocab_;
    unsigned *seeds_, *counters_;
    int* tokens_;
    float* ws_val_;
    int* ws_idx_;
    unsigned* ws_counters_;
    int* host_[2] = {nullptr, nullptr};
    cudaEvent_t events_[2] = {nullptr, nullptr};
    int turn_ = 0, pending_rows_ = 0;
};

}  // namespace ti

extern "C" void* ti_loop_create(void* cache, void* planner, int max_rows, int vocab, unsigned* seeds, unsigned* counters, int* tokens,
                                float* ws_val, int* ws_idx, unsigned* ws_counters) {
    return new ti::DecodeLoop((ti::CacheBook*)cache, (ti::StepPlanner*)planner, max_rows, vocab, seeds, counters, tokens, ws_val, ws_idx,
                              ws_counters);
}
extern "C" void ti_loop_destroy(void* loop) { delete (ti::DecodeLoop*)loop; }

// Sample `rows` rows of `logits` (temperature 0: greedy), start the tokens' way to the host, and put the next step on the
// stream: the sequences `next_slots` (the rows `next_rows` of this step, ascending), whose captured graph is `graph` and
// whose token ids live at `next_ids`. Returns 0; 4: the cache has no page for the next step (needed / free_pages say how
// many), nothing was enqueued; other: see ti_last_error().
extern "C" int ti_loop_enqueue(void* loop, const float* logits, long long ld, int rows, float temperature, int top_k, float top_p, int n_next,
                               const int* next_rows, const int* next_slots, void* graph, int* next_ids, cudaStream_t stream,
                               long long* needed, long long* free_pages) {
    return ((ti::DecodeLoop*)loop)->enqueue(logits, ld, rows, temperature, top_k, top_p, n_next, next_rows, next_slots, (cudaGraphExec_t)graph,
                                            next_ids, stream, needed, free_pages);
}
// The tokens of the last enqueue, once they have arrived.
extern "C" int ti_loop_wait(void* loop, int* out, int rows) { return ((ti::DecodeLoop*)loop)->wait(out, rows); }

extern "C" void ti_range_push(const char* name) { nvtxRangePushA(name); }
extern "C" void ti_range_pop() { nvtxRangePop(); }
