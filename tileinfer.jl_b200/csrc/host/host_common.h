// Shared by the host runtime (the cache's books, the step planner, the decode loop): error reporting in
// the manner of the kernel launchers (a code, and ti_last_error() for the text) and the C++ types that
// cross files. Host code only: nothing here needs nvcc's device pass.
#pragma once
#include <cstdint>
#include <functional>
#include <queue>
#include <vector>

extern "C" const char* ti_last_error();
int ti_fail(const char* fmt, ...);

namespace ti {

// Numbers 0..count-1; take() hands out the smallest free one, give() takes one back and refuses a number
// that is not held. AntoineBut/TileInfer.jl's BlockManager hands pages out in increasing order the same
// way (src/kv/block_manager.jl:39-47).
class NumberPool {
public:
    explicit NumberPool(int count = 0) { reset(count); }
    void reset(int count) {
        count_ = count;
        held_.assign(count, 0);
        held_count_ = 0;
        free_ = {};
        for (int i = 0; i < count; ++i) free_.push(i);
    }
    int count() const { return count_; }
    int free_count() const { return count_ - held_count_; }
    int held_count() const { return held_count_; }
    bool is_held(int n) const { return n >= 0 && n < count_ && held_[n]; }
    int take() {
        if (free_.empty()) return -1;
        const int n = free_.top();
        free_.pop();
        held_[n] = 1;
        ++held_count_;
        return n;
    }
    bool give(int n) {
        if (!is_held(n)) return false;
        held_[n] = 0;
        --held_count_;
        free_.push(n);
        return true;
    }

private:
    int count_ = 0, held_count_ = 0;
    std::vector<char> held_;
    std::priority_queue<int, std::vector<int>, std::greater<int>> free_;
};

// Tables that a mixer's decode kernels want in the step's metadata, beside what every step carries. The
// planner knows only this interface: how many 32-bit words a decode step of `batch` sequences needs (fixed
// by the batch size alone, so that a captured step finds them at fixed addresses) and how to fill them from
// the sequences' lengths after the step. Each kind of plan lives in the file of the kernels it serves.
struct GroupPlan {
    virtual ~GroupPlan() {}
    virtual int words(int batch) = 0;
    virtual void fill(int batch, int32_t* out, const int64_t* lengths_after) = 0;
};

}  // namespace ti
