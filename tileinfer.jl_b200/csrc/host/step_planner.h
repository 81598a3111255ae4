// What one step carries besides the model, built on the host: which tokens, of which sequences, where.
//
// Everything the kernels read per step lives in ONE device buffer of 32-bit integers that is filled by ONE
// copy from pinned host memory, so that a captured decode step reads fresh values at fixed addresses
// (AntoineBut/TileInfer.jl keeps its ids, positions, slots and block table in one `meta` vector for the same
// reason, and prepares it on the host before every step: src/model/decoder.jl:107-117, 137-157). The layout
// of the buffer depends only on (tokens, sequences, wanted rows).
#pragma once
#include "cache_book.h"

#include <map>
#include <tuple>

namespace ti {

struct StepLayout {
    int n = 0, batch = 0, wanted = 0;
    int ids = 0, pos = 0, slot = 0, seq = 0, cu = 0, kv = 0, want = 0, end = 0;
    std::vector<int> maps;            // per paged group: flat place of every token in the pool
    std::vector<int> plan, plan_words;   // per paged group: the mixer's decode tables (0 words: none)
};

class StepPlanner {
public:
    StepPlanner(CacheBook* cache, int max_step_tokens, bool on_device);
    ~StepPlanner();
    void attach_plan(int group, GroupPlan* plan);         // the planner owns it from now on
    int capacity() const;                                 // words of the device buffer
    void set_meta(int32_t* meta) { meta_ = meta; }
    const StepLayout& layout(int n, int batch, int wanted);
    // Pages must already be reserved; lengths are those before the step. 0, or 2 with the text in ti_last_error().
    int plan(int n_entries, const int* slots, const int* q_lens, const int* tokens, const int* want_counts, const int* want,
             cudaStream_t stream);
    // One token for each slot, its logits wanted; `tokens` null: the ids are written on the device by a kernel
    // (the sampler of the previous step) and only the rest is uploaded. `starts` (optional) receives the lengths before the step.
    int plan_decode(int batch, const int* slots, const int* tokens, cudaStream_t stream, int64_t* starts);
    long long last_upload_bytes = 0;

private:
    int32_t* staging(int* turn);
    int upload(int turn, int count, int skip, cudaStream_t stream);
    void fill_plans(const StepLayout& lay, int32_t* st, const int64_t* lengths_after);

    CacheBook* cache_;
    int max_step_tokens_;
    bool on_device_;
    int capacity_ = 0;
    int32_t* staging_[2] = {nullptr, nullptr};
    cudaEvent_t events_[2] = {nullptr, nullptr};
    bool in_flight_[2] = {false, false};
    int turn_ = 0;
    int32_t* meta_ = nullptr;
    std::vector<GroupPlan*> plans_;
    std::map<std::tuple<int, int, int>, StepLayout> layouts_;
};

}  // namespace ti
