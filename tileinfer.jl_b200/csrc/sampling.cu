// Sampling on the device: greedy argmax, and temperature / top-k / top-p sampling over the
// whole vocabulary by inverse-CDF in best-first order.
//
// The rule is AntoineBut/TileInfer.jl's (src/engine/sampler.jl:49-102): candidates are
// ordered best first with ties to the smaller id; temperature, then top-k, then top-p over
// the renormalised survivors (the smallest prefix whose mass reaches top_p); the token is
// the first one whose cumulative weight reaches u × total, u = sampling_uniform(seed,
// counter) (sampler.jl:34-47). The reference samples on the device only for top_k <= 64 and
// sends the logits to the host otherwise; here every setting runs on the device.
//
// Method: no sort of the vocabulary. Each token gets a 56-bit key (descending-ordered logit bits, then
// id), so best-first order is ascending key order, and every step of the rule is "the first key whose
// cumulative weight reaches X". Weights are 2^40 fixed-point integers, so sums do not depend on the
// order of the atomic additions and the result is deterministic.
//   Fast path: ONE pass over the row builds a histogram of weights and counts over 4096 bins of the
//   scaled distance from the maximum, (max - l) / T in steps of 1/128 (the bin is monotone in the
//   key, and weights vanish beyond 28.4). A selection then scans the bins for the one that holds its
//   target, gathers that bin's few tokens in a second pass, sorts them by key in shared memory and
//   scans them. top-k, top-p and the draw share the histogram: it is cut off at each bound found.
//   Exact path: a bin with more than 4096 tokens (a flat row of a large vocabulary) sends the row to a
//   radix select over the key, 8 bits a pass, with a histogram of weights per pass.
#include "common.cuh"

typedef unsigned long long u64;
typedef unsigned int u32;

#define SM_THREADS 1024
#define SM_WARPS 32
#define SM_ID_BITS 24
#define SM_PASSES 7

__host__ __device__ __forceinline__ u32 mix32(u32 x) {
    x = (x ^ (x >> 16)) * 0x7feb352du;
    x = (x ^ (x >> 15)) * 0x846ca68bu;
    return x ^ (x >> 16);
}

__device__ __forceinline__ u32 desc_key(float l) {
    const u32 b = __float_as_uint(l);
    const u32 asc = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ~asc;
}

// ------------------------------------------------------------------------------ greedy
// argmax with ties to the smaller id, over a vocabulary of any size, in ONE launch that uses many
// blocks: each block reduces a slice of the row and leaves its candidate in a work space; the block
// that arrives last at the row's counter (no block waits for another) reduces the candidates, writes
// the token and resets the counter for the next launch. (value, id) under "greater value, then
// smaller id" is a total order, so the result does not depend on the order of arrival.
#define AM_THREADS 256
#define AM_MAX_CHUNKS 256

__device__ __forceinline__ bool am_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__device__ __forceinline__ void am_block_reduce(float& bv, int& bi, float* sv, int* si) {
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (am_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < AM_THREADS / 32 ? sv[lane] : -INFINITY;
        bi = lane < AM_THREADS / 32 ? si[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (am_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(AM_THREADS) argmax_kernel(const float* logits, long long ld, int vocab, int per_chunk,
                                                            int* __restrict__ out, int* __restrict__ out2, float* ws_val,
                                                            int* ws_idx, unsigned* counters) {
    __shared__ float sv[AM_THREADS / 32];
    __shared__ int si[AM_THREADS / 32];
    __shared__ bool last;
    const int chunk = blockIdx.x, row_id = blockIdx.y, chunks = gridDim.x;
    const float* row = logits + (size_t)row_id * ld;
    const int lo = chunk * per_chunk, hi = min(vocab, lo + per_chunk);
    pdl_enter();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if ((((uintptr_t)row) & 15) == 0 && (lo & 3) == 0) {
        for (int i = lo + 4 * threadIdx.x; i < hi; i += 4 * AM_THREADS) {
            if (i + 3 < hi) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(row + i));
                if (am_better(v.x, i, bv, bi)) { bv = v.x; bi = i; }
                if (am_better(v.y, i + 1, bv, bi)) { bv = v.y; bi = i + 1; }
                if (am_better(v.z, i + 2, bv, bi)) { bv = v.z; bi = i + 2; }
                if (am_better(v.w, i + 3, bv, bi)) { bv = v.w; bi = i + 3; }
            } else {
                for (int j = i; j < hi; ++j) {
                    const float v = __ldcg(row + j);
                    if (am_better(v, j, bv, bi)) { bv = v; bi = j; }
                }
            }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += AM_THREADS) {
            const float v = __ldcg(row + i);
            if (am_better(v, i, bv, bi)) { bv = v; bi = i; }
        }
    }
    am_block_reduce(bv, bi, sv, si);
    if (threadIdx.x == 0) {
        ws_val[(size_t)row_id * chunks + chunk] = bv;
        ws_idx[(size_t)row_id * chunks + chunk] = bi;
        __threadfence();                                   // the candidate is visible before the ticket is taken
        last = atomicAdd(&counters[row_id], 1u) == (unsigned)chunks - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    bv = -INFINITY;
    bi = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += AM_THREADS) {
        const float v = __ldcg(ws_val + (size_t)row_id * chunks + c);
        const int i = __ldcg(ws_idx + (size_t)row_id * chunks + c);
        if (am_better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    am_block_reduce(bv, bi, sv, si);
    if (threadIdx.x == 0) {
        out[row_id] = bi == 0x7fffffff ? 0 : bi;
        if (out2 != nullptr) out2[row_id] = bi == 0x7fffffff ? 0 : bi;     // the next step's token ids, where the caller has them
        counters[row_id] = 0;                              // ready for the next launch
    }
}

// Work space: ws_val and ws_idx hold n_rows x TI_ARGMAX_CHUNKS(vocab) entries, counters n_rows words
// that are zero before the first launch (the kernel leaves them zero).
extern "C" int ti_argmax_chunks(int vocab) {
    int chunks = (vocab + 1023) / 1024;
    if (chunks < 1) chunks = 1;
    return chunks > AM_MAX_CHUNKS ? AM_MAX_CHUNKS : chunks;
}

extern "C" int ti_argmax(const float* logits, long long ld, int n_rows, int vocab, int* out, int* out2, float* ws_val, int* ws_idx,
                         unsigned* counters, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(vocab > 0, "argmax: vocab %d", vocab);
    TI_REQUIRE(n_rows <= 65535, "argmax: %d rows in one launch", n_rows);
    TI_REQUIRE(ws_val != nullptr && ws_idx != nullptr && counters != nullptr, "argmax: work space missing");
    // Many rows: fewer, longer chunks (about 2,048 blocks in all), so that the launch is not a long queue of tiny blocks.
    int chunks = ti_argmax_chunks(vocab);
    const int fewer = 2048 / n_rows < 8 ? 8 : 2048 / n_rows;
    if (fewer < chunks) chunks = fewer;
    int per_chunk = (vocab + chunks - 1) / chunks;
    per_chunk = (per_chunk + 3) & ~3;
    ti_launch(argmax_kernel, dim3(chunks, n_rows), dim3(AM_THREADS), 0, stream, logits, ld, vocab, per_chunk, out, out2, ws_val, ws_idx,
              counters);
    return ti_check_launch("argmax");
}

// ------------------------------------------------------------------------------ sampling
// ceil(u x total) with u = r24 / 2^24, without leaving integers: total < 2^58 and r24 < 2^24 need 128 bits.
__device__ __forceinline__ u64 draw_target(u64 total, u32 r24) {
    const u64 hi = __umul64hi(total, (u64)r24), lo = total * (u64)r24;
    u64 target = (hi << 40) | (lo >> 24);
    if (lo & 0xFFFFFFull) target += 1;
    return target;
}

struct Selected {
    u64 key;          // the selected token's 56-bit key
    u64 before;       // weight of the keys before it (within the set)
    u64 through;      // ... including it
};

#define W_COUNT 0
#define W_MASS 1

__device__ __forceinline__ u64 token_weight(int mode, float l, float maxl, float inv_t) {
    if (mode == W_COUNT) return 1ull;
    const float e = expf((l - maxl) * inv_t);
    return __float2ull_rn(e * 1099511627776.0f);          // × 2^40
}

// First key (ascending) among keys <= bound whose cumulative weight reaches target (at
// least 1); if the set's total is smaller, the last key with weight. All threads get it.
__device__ Selected select_key(const float* row, int vocab, int mode, u64 bound, u64 target,
                               float maxl, float inv_t, u64* hist /*[SM_WARPS][256]*/, u64* totals /*[256]*/,
                               u64* shared /*[4]*/) {
    const int warp = threadIdx.x >> 5;
    u64 prefix = 0, base = 0;
    if (target == 0) target = 1;
    for (int pass = 0; pass < SM_PASSES; ++pass) {
        const int shift = 8 * (SM_PASSES - 1 - pass);
        for (int i = threadIdx.x; i < SM_WARPS * 256; i += SM_THREADS) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += SM_THREADS) {
            const float l = row[i];
            const u64 key = ((u64)desc_key(l) << SM_ID_BITS) | (u64)i;
            if (key > bound) continue;
            if (pass > 0 && (key >> (shift + 8)) != prefix) continue;
            const u64 w = token_weight(mode, l, maxl, inv_t);
            if (w) atomicAdd(&hist[warp * 256 + (int)((key >> shift) & 255)], w);
        }
        __syncthreads();
        if (threadIdx.x < 256) {
            u64 s = 0;
            for (int w = 0; w < SM_WARPS; ++w) s += hist[w * 256 + threadIdx.x];
            totals[threadIdx.x] = s;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            u64 cum = base;
            int digit = -1, last = 0;
            for (int b = 0; b < 256; ++b) {
                const u64 w = totals[b];
                if (w == 0) continue;
                if (cum + w >= target) { digit = b; break; }
                cum += w;
                last = b;
            }
            if (digit < 0) {                 // target beyond the set: settle on the last key with weight
                digit = last;
                cum -= totals[last];
            }
            shared[0] = (prefix << 8) | (u64)digit;
            shared[1] = cum;
            shared[2] = totals[digit];
        }
        __syncthreads();
        prefix = shared[0];
        base = shared[1];
    }
    Selected r;
    r.key = prefix;
    r.before = base;
    r.through = base + shared[2];
    __syncthreads();
    return r;
}

// ------------------------------------------------------------------------------ the binned fast path
// f(index, logit) for every token of the row, the block's threads sharing them out; sixteen values per
// thread are in flight at a time (one L2 round trip per value would otherwise bound a pass).
template <typename F> __device__ __forceinline__ void for_each_logit(const float* row, int lo, int hi, F f) {
    int done = lo;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0 && (lo & 3) == 0) {
        const int first4 = lo >> 2, n4 = hi > lo ? (hi - lo) >> 2 : 0;
        const float4* row4 = reinterpret_cast<const float4*>(row) + first4;
        for (int i = threadIdx.x; i < n4; i += 4 * SM_THREADS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + u * SM_THREADS < n4) v[u] = __ldcg(row4 + i + u * SM_THREADS);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = i + u * SM_THREADS;
                if (j < n4) { const int t = lo + 4 * j; f(t, v[u].x); f(t + 1, v[u].y); f(t + 2, v[u].z); f(t + 3, v[u].w); }
            }
        }
        done = lo + n4 * 4;
    }
    for (int i = done + threadIdx.x; i < hi; i += 4 * SM_THREADS) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * SM_THREADS < hi) v[u] = __ldcg(row + i + u * SM_THREADS);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * SM_THREADS < hi) f(i + u * SM_THREADS, v[u]);
    }
}
template <typename F> __device__ __forceinline__ void for_each_logit(const float* row, int vocab, F f) { for_each_logit(row, 0, vocab, f); }

#define SB_BINS 4096
#define SB_PER_NAT 128.0f
#define SB_CAP 4096

struct Binned {
    u64* mass;        // [SB_BINS] weights per bin
    u32* count;       // [SB_BINS] tokens per bin
    u64* cand_key;    // [SB_CAP]
    u64* cand_w;      // [SB_CAP]
    u64* scan;        // [SM_WARPS + 8] scratch of the block scans and results
};

__device__ __forceinline__ int token_bin(float l, float maxl, float inv_t) {
    const float d = (maxl - l) * inv_t * SB_PER_NAT;
    return d >= (float)(SB_BINS - 1) ? SB_BINS - 1 : (int)d;             // NaN goes to the last bin as well
}

// Inclusive block scan of one value per thread; every thread also gets the total. `scratch`: SM_WARPS + 1 words.
__device__ __forceinline__ u64 block_scan(u64 v, u64* scratch, u64& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        u64 t = lane < SM_WARPS ? scratch[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 u = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += u;
        }
        scratch[lane] = t;
        if (lane == 31) scratch[SM_WARPS] = t;
    }
    __syncthreads();
    total = scratch[SM_WARPS];
    return v + (warp > 0 ? scratch[warp - 1] : 0);
}

struct BinSelected {
    Selected sel;     // key, weight before and through it (over the whole set, in the mode's weights)
    int bin;          // the bin it lies in
    u64 mass_in_bin;  // mass and count of the bin's tokens up to and including it
    u32 count_in_bin;
    bool overflow;    // the bin held more than SB_CAP tokens: nothing was selected
};

// The first key (ascending) among keys <= bound whose cumulative weight (mode: counts or masses) reaches
// target, from the histogram of the set and one gathering pass over the row, in three steps that the kernels
// below put together: the bin that holds the target (find_bin), that bin's tokens out of a stretch of the row
// (gather_bin; several blocks may each gather a stretch), and the choice among them in key order (pick_in_bin).
struct BinChoice {
    int bin;
    u64 base;         // weight of the bins before it
};

__device__ BinChoice find_bin(int mode, u64 target, const Binned& h) {
    if (target == 0) target = 1;
    // Four bins per thread, block scan.
    u64 local[4], sum = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int b = threadIdx.x * 4 + e;
        local[e] = mode == W_COUNT ? (u64)h.count[b] : h.mass[b];
        sum += local[e];
    }
    u64 total;
    const u64 incl = block_scan(sum, h.scan, total);
    u64* res = h.scan + SM_WARPS + 1;                  // res[0] bin, res[1] weight before the bin, res[2] last bin with weight
    if (threadIdx.x == 0) { res[0] = ~0ull; res[2] = 0; }
    __syncthreads();
    {
        u64 cum = incl - sum;
        int last = -1;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (local[e] && cum < target && cum + local[e] >= target) { res[0] = (u64)(threadIdx.x * 4 + e); res[1] = cum; }
            if (local[e]) last = threadIdx.x * 4 + e;
            cum += local[e];
        }
        if (last >= 0) atomicMax(&res[2], (u64)last);
    }
    __syncthreads();
    if (res[0] == ~0ull) {                             // the target lies beyond the set: its last bin with weight
        const int last = (int)res[2];
        __syncthreads();
        if (threadIdx.x == last / 4) { res[0] = (u64)last; res[1] = incl - sum; for (int e = 0; e < last % 4; ++e) res[1] += local[e]; }
        __syncthreads();
    }
    BinChoice c;
    c.bin = (int)res[0];
    c.base = res[1];
    __syncthreads();
    return c;
}

// The counter of gathered tokens (a 32-bit word in the scan scratch).
__device__ __forceinline__ u32* gathered_count(const Binned& h) { return reinterpret_cast<u32*>(h.scan + SM_WARPS + 6); }

// Appends the tokens of row[lo, hi) that fall into `bin` (keys <= bound) to the candidates; the counter keeps
// counting beyond SB_CAP, which the caller reads as an overflow.
__device__ void gather_bin(const float* row, int lo, int hi, int mode, u64 bound, int bin, float maxl, float inv_t, const Binned& h) {
    u32* n_cand = gathered_count(h);
    for_each_logit(row, lo, hi, [&](int i, float l) {
        if (token_bin(l, maxl, inv_t) != bin) return;
        const u64 key = ((u64)desc_key(l) << SM_ID_BITS) | (u64)i;
        if (key > bound) return;
        const u64 w = token_weight(W_MASS, l, maxl, inv_t);
        if (mode == W_MASS && w == 0) return;
        const u32 at = atomicAdd(n_cand, 1u);
        if (at < SB_CAP) { h.cand_key[at] = key; h.cand_w[at] = w; }
    });
}

// Among the n gathered tokens of `bin`, in key order, the first whose cumulative weight reaches what is left of the target.
__device__ BinSelected pick_in_bin(int mode, u64 target, const BinChoice& at, int n, const Binned& h) {
    BinSelected r;
    if (target == 0) target = 1;
    const int bin = at.bin;
    const u64 base = at.base;
    r.bin = bin;
    r.overflow = n > SB_CAP || n == 0;
    if (r.overflow) { __syncthreads(); return r; }
    // Bitonic sort of the next power of two, then scans of counts and masses.
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int i = n + threadIdx.x; i < n2; i += SM_THREADS) { h.cand_key[i] = ~0ull; h.cand_w[i] = 0; }
    __syncthreads();
    for (int size = 2; size <= n2; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = threadIdx.x; t < (n2 >> 1); t += SM_THREADS) {
                const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                const bool up = (lo & size) == 0;
                const u64 a = h.cand_key[lo], b = h.cand_key[hi];
                if ((a > b) == up) {
                    h.cand_key[lo] = b; h.cand_key[hi] = a;
                    const u64 wa = h.cand_w[lo]; h.cand_w[lo] = h.cand_w[hi]; h.cand_w[hi] = wa;
                }
            }
            __syncthreads();
        }
    // Each thread owns four consecutive places; the first place whose cumulative weight reaches the rest of the target.
    const u64 rest = target - base;
    u64 wsel[4], wmass[4], ssum = 0, msum = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int i = threadIdx.x * 4 + e;
        wmass[e] = i < n ? h.cand_w[i] : 0;
        wsel[e] = i < n ? (mode == W_COUNT ? 1ull : wmass[e]) : 0;
        ssum += wsel[e]; msum += wmass[e];
    }
    u64 stotal, mtotal;
    const u64 sincl = block_scan(ssum, h.scan, stotal);
    const u64 mincl = block_scan(msum, h.scan, mtotal);
    u64* pick = h.scan + SM_WARPS + 1;                 // pick[0] place, [1] weight before, [2] through, [3] mass through
    if (threadIdx.x == 0) pick[0] = ~0ull;
    __syncthreads();
    {
        u64 cum = sincl - ssum, mcum = mincl - msum;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = threadIdx.x * 4 + e;
            mcum += wmass[e];
            if (i < n && cum < rest && cum + wsel[e] >= rest) { pick[0] = (u64)i; pick[1] = cum; pick[2] = cum + wsel[e]; pick[3] = mcum; }
            cum += wsel[e];
        }
    }
    __syncthreads();
    if (pick[0] == ~0ull) {                            // beyond the bin's weight: its last token
        __syncthreads();
        if (threadIdx.x == (n - 1) / 4) { pick[0] = (u64)(n - 1); pick[1] = stotal - wsel[(n - 1) % 4]; pick[2] = stotal; pick[3] = mtotal; }
        __syncthreads();
    }
    const int place = (int)pick[0];
    r.sel.key = h.cand_key[place];
    r.sel.before = base + pick[1];
    r.sel.through = base + pick[2];
    r.mass_in_bin = pick[3];
    r.count_in_bin = (u32)(place + 1);
    __syncthreads();
    return r;
}


__device__ BinSelected select_binned(const float* row, int vocab, int mode, u64 bound, u64 target, float maxl, float inv_t,
                                     const Binned& h) {
    const BinChoice at = find_bin(mode, target, h);
    if (threadIdx.x == 0) *gathered_count(h) = 0;
    __syncthreads();
    gather_bin(row, 0, vocab, mode, bound, at.bin, maxl, inv_t, h);
    __syncthreads();
    return pick_in_bin(mode, target, at, (int)*gathered_count(h), h);
}

// The set shrinks to the keys up to a selected one: its bin keeps what lies before and at it, later bins empty.
__device__ __forceinline__ void cut_histogram(const Binned& h, const BinSelected& at) {
    for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) {
        if (b == at.bin) { h.mass[b] = at.mass_in_bin; h.count[b] = at.count_in_bin; }
        else if (b > at.bin) { h.mass[b] = 0; h.count[b] = 0; }
    }
    __syncthreads();
}

// The rule by the radix select alone (any row; seven passes over the row per selection).
__device__ int sample_exact(const float* row, int vocab, float inv_t, int top_k, float top_p, u32 r24, float maxl, u64* hist,
                            u64* totals, u64* shared) {
    u64 bound = ~0ull;
    if (top_k > 0 && top_k < vocab) {
        const Selected k = select_key(row, vocab, W_COUNT, bound, (u64)top_k, maxl, inv_t, hist, totals, shared);
        bound = k.key;
    }
    // Mass of the current set (everything, or the top-k prefix).
    {
        u64 local = 0;
        for (int i = threadIdx.x; i < vocab; i += SM_THREADS) {
            const float l = row[i];
            const u64 key = ((u64)desc_key(l) << SM_ID_BITS) | (u64)i;
            if (key <= bound) local += token_weight(W_MASS, l, maxl, inv_t);
        }
        if (threadIdx.x == 0) shared[3] = 0;
        __syncthreads();
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if ((threadIdx.x & 31) == 0) atomicAdd(&shared[3], local);
        __syncthreads();
    }
    u64 total = shared[3];
    __syncthreads();
    if (top_p < 1.0f) {
        // Smallest prefix whose mass reaches top_p × total.
        const u64 target = (u64)ceil((double)top_p * (double)total);
        const Selected p = select_key(row, vocab, W_MASS, bound, target, maxl, inv_t, hist, totals, shared);
        bound = p.key;
        total = p.through;
    }
    const Selected s = select_key(row, vocab, W_MASS, bound, draw_target(total, r24), maxl, inv_t, hist, totals, shared);
    return (int)(s.key & ((1ull << SM_ID_BITS) - 1));
}

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(const float* logits, long long ld, int vocab,
                                                            float inv_t, int top_k, float top_p,
                                                            const u32* seeds, u32* counters,
                                                            int* __restrict__ out, int* __restrict__ out2) {
    extern __shared__ u64 dyn[];
    __shared__ float scratch[33];
    const float* row = logits + (size_t)blockIdx.x * ld;
    pdl_wait();
    pdl_launch_dependents();

    float maxl = -INFINITY;
    for_each_logit(row, vocab, [&](int, float l) { maxl = fmaxf(maxl, l); });
    maxl = block_max(maxl, scratch);
    const u32 counter = counters[blockIdx.x];
    const u32 r24 = mix32(mix32(seeds[blockIdx.x]) ^ counter) >> 8;          // u = r24 · 2^-24

    // Fast path: one histogram of the row, cut off at each bound; a crowded bin sends the row to the exact path.
    Binned h;
    h.mass = dyn;
    h.cand_key = dyn + SB_BINS;
    h.cand_w = h.cand_key + SB_CAP;
    h.scan = h.cand_w + SB_CAP;
    h.count = reinterpret_cast<u32*>(h.scan + SM_WARPS + 8);
    // Masses are summed as two 32-bit halves with the carry passed on by hand: 64-bit additions in shared
    // memory are compare-and-swap loops, and these atomics bound the pass. The halves borrow the
    // candidates' place until the pass is over.
    u32* mass_lo = reinterpret_cast<u32*>(h.cand_key);
    u32* mass_hi = mass_lo + SB_BINS;
    for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) { mass_lo[b] = 0; mass_hi[b] = 0; h.count[b] = 0; }
    __syncthreads();
    const bool need_counts = top_k > 0 && top_k < vocab;
    for_each_logit(row, vocab, [&](int, float l) {
        const int b = token_bin(l, maxl, inv_t);
        const u64 w = token_weight(W_MASS, l, maxl, inv_t);
        if (w) {
            const u32 lo = (u32)w;
            u32 hi = (u32)(w >> 32);
            if (lo) {
                const u32 old = atomicAdd(&mass_lo[b], lo);
                hi += (old + lo < old) ? 1u : 0u;
            }
            if (hi) atomicAdd(&mass_hi[b], hi);
        }
        if (need_counts) atomicAdd(&h.count[b], 1u);      // only top-k reads the counts
    });
    __syncthreads();
    for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) h.mass[b] = ((u64)mass_hi[b] << 32) | (u64)mass_lo[b];
    __syncthreads();
    int token = -1;
    do {
        u64 bound = ~0ull;
        if (top_k > 0 && top_k < vocab) {
            const BinSelected k = select_binned(row, vocab, W_COUNT, bound, (u64)top_k, maxl, inv_t, h);
            if (k.overflow) break;
            bound = k.sel.key;
            cut_histogram(h, k);
        }
        u64 part = 0, total;
        for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) part += h.mass[b];
        block_scan(part, h.scan, total);
        if (top_p < 1.0f) {
            const u64 target = (u64)ceil((double)top_p * (double)total);
            const BinSelected p = select_binned(row, vocab, W_MASS, bound, target, maxl, inv_t, h);
            if (p.overflow) break;
            bound = p.sel.key;
            total = p.sel.through;
            cut_histogram(h, p);
        }
        const BinSelected d = select_binned(row, vocab, W_MASS, bound, draw_target(total, r24), maxl, inv_t, h);
        if (d.overflow) break;
        token = (int)(d.sel.key & ((1ull << SM_ID_BITS) - 1));
    } while (false);
    if (token < 0) {                                       // uniform across the block: every thread saw the same overflow
        __syncthreads();
        u64* hist = dyn;
        u64* totals = dyn + SM_WARPS * 256;
        u64* shared = totals + 256;
        token = sample_exact(row, vocab, inv_t, top_k, top_p, r24, maxl, hist, totals, shared);
    }
    if (threadIdx.x == 0) {
        out[blockIdx.x] = token;
        if (out2 != nullptr) out2[blockIdx.x] = token;
        counters[blockIdx.x] = counter + 1;
    }
}

// ------------------------------------------------------------------------------ a row shared by a cluster
// The same rule with the row shared out among the C blocks of a cluster, for steps of a few rows, where one block
// per row leaves most of the GPU idle and is bound by one SM's instruction rate (a pass over 131,072 logits takes a
// block about 15 us). Every block makes the passes over its own stretch of the row (maximum, histogram, the
// gathering of a bin's tokens) into its own shared memory; the histograms are added up, and the gathered tokens
// collected, through distributed shared memory; the scans, the sort and the choices run in block 0 alone, on the
// same integers as in the one-block kernel, so the token is the same. Block 0 tells the others what to gather
// through a few words of its shared memory; a barrier of the cluster stands before and after every such order.
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned remote_addr(const void* p, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"((unsigned)__cvta_generic_to_shared(p)), "r"(rank));
    return a;
}
__device__ __forceinline__ u32 ld_remote(const u32* p, unsigned rank) {
    u32 v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ u64 ld_remote(const u64* p, unsigned rank) {
    u64 v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ float ld_remote(const float* p, unsigned rank) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote_addr(p, rank)) : "memory");
    return v;
}
__device__ __forceinline__ void st_remote(u32* p, unsigned rank, u32 v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote_addr(p, rank)), "r"(v) : "memory");
}
__device__ __forceinline__ void st_remote(u64* p, unsigned rank, u64 v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote_addr(p, rank)), "l"(v) : "memory");
}

template <int C>
__global__ void __launch_bounds__(SM_THREADS) sample_cluster_kernel(const float* logits, long long ld, int vocab,
                                                                    float inv_t, int top_k, float top_p,
                                                                    const u32* seeds, u32* counters,
                                                                    int* __restrict__ out, int* __restrict__ out2) {
    extern __shared__ u64 dyn[];
    __shared__ float scratch[33];
    __shared__ float my_max;
    __shared__ u64 order[4];                               // block 0's: [0] 0 gather / 1 finished, [1] bin, [2] bound, [3] mode
    const unsigned rank = cluster_rank();
    const int row_id = blockIdx.x / C;
    const float* row = logits + (size_t)row_id * ld;
    const int per = ((vocab + C - 1) / C + 3) & ~3;        // stretches begin at multiples of 4 (16-byte loads)
    const int lo = min(vocab, (int)rank * per), hi = min(vocab, lo + per);
    pdl_wait();
    pdl_launch_dependents();

    float maxl = -INFINITY;
    for_each_logit(row, lo, hi, [&](int, float l) { maxl = fmaxf(maxl, l); });
    maxl = block_max(maxl, scratch);
    if (threadIdx.x == 0) my_max = maxl;
    cluster_sync_all();
#pragma unroll
    for (int r = 0; r < C; ++r) maxl = fmaxf(maxl, ld_remote(&my_max, (unsigned)r));

    Binned h;
    h.mass = dyn;
    h.cand_key = dyn + SB_BINS;
    h.cand_w = h.cand_key + SB_CAP;
    h.scan = h.cand_w + SB_CAP;
    h.count = reinterpret_cast<u32*>(h.scan + SM_WARPS + 8);
    u32* mass_lo = reinterpret_cast<u32*>(h.cand_key);      // as in the one-block kernel: masses as two 32-bit halves
    u32* mass_hi = mass_lo + SB_BINS;
    for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) { mass_lo[b] = 0; mass_hi[b] = 0; h.count[b] = 0; }
    __syncthreads();
    const bool need_counts = top_k > 0 && top_k < vocab;
    for_each_logit(row, lo, hi, [&](int, float l) {
        const int b = token_bin(l, maxl, inv_t);
        const u64 w = token_weight(W_MASS, l, maxl, inv_t);
        if (w) {
            const u32 wl = (u32)w;
            u32 wh = (u32)(w >> 32);
            if (wl) {
                const u32 old = atomicAdd(&mass_lo[b], wl);
                wh += (old + wl < old) ? 1u : 0u;
            }
            if (wh) atomicAdd(&mass_hi[b], wh);
        }
        if (need_counts) atomicAdd(&h.count[b], 1u);
    });
    __syncthreads();
    cluster_sync_all();                                    // every block's histogram stands
    // Each block adds up its share of the bins over all blocks and hands the sums to block 0.
    for (int b = (int)rank * (SB_BINS / C) + threadIdx.x; b < ((int)rank + 1) * (SB_BINS / C); b += SM_THREADS) {
        u64 m = 0;
        u32 c = 0;
#pragma unroll
        for (int r = 0; r < C; ++r) {
            m += ((u64)ld_remote(&mass_hi[b], (unsigned)r) << 32) + (u64)ld_remote(&mass_lo[b], (unsigned)r);
            c += ld_remote(&h.count[b], (unsigned)r);
        }
        st_remote(&h.mass[b], 0u, m);
        st_remote(&h.count[b], 0u, c);
    }
    cluster_sync_all();                                    // block 0 holds the row's histogram

    if (rank != 0) {
        // Gather what block 0 orders, until it says that it has finished.
        while (true) {
            cluster_sync_all();                            // an order stands
            if (ld_remote(&order[0], 0u) != 0) break;
            const int bin = (int)ld_remote(&order[1], 0u), mode = (int)ld_remote(&order[3], 0u);
            const u64 bound = ld_remote(&order[2], 0u);
            if (threadIdx.x == 0) *gathered_count(h) = 0;
            __syncthreads();
            gather_bin(row, lo, hi, mode, bound, bin, maxl, inv_t, h);
            __syncthreads();
            cluster_sync_all();                            // gathered; block 0 now reads the candidates
        }
        cluster_sync_all();                                // nobody reads block 0's order any more
        return;
    }

    const u32 counter = counters[row_id];
    const u32 r24 = mix32(mix32(seeds[row_id]) ^ counter) >> 8;
    auto select = [&](int mode, u64 bound, u64 target) -> BinSelected {
        const BinChoice at = find_bin(mode, target, h);
        if (threadIdx.x == 0) {
            order[0] = 0; order[1] = (u64)at.bin; order[2] = bound; order[3] = (u64)mode;
            *gathered_count(h) = 0;
        }
        __syncthreads();
        cluster_sync_all();
        gather_bin(row, lo, hi, mode, bound, at.bin, maxl, inv_t, h);
        __syncthreads();
        cluster_sync_all();
        // The other blocks' candidates behind this block's own; the sort puts them in key order.
        long long n = (long long)*gathered_count(h);
        __syncthreads();
        for (int r = 1; r < C; ++r) {
            const u32 nr = ld_remote(gathered_count(h), (unsigned)r);
            if (n + (long long)nr <= SB_CAP)
                for (int i = threadIdx.x; i < (int)nr; i += SM_THREADS) {
                    h.cand_key[n + i] = ld_remote(&h.cand_key[i], (unsigned)r);
                    h.cand_w[n + i] = ld_remote(&h.cand_w[i], (unsigned)r);
                }
            n += (long long)nr;
        }
        __syncthreads();
        return pick_in_bin(mode, target, at, n > SB_CAP ? SB_CAP + 1 : (int)n, h);
    };
    int token = -1;
    do {
        u64 bound = ~0ull;
        if (need_counts) {
            const BinSelected k = select(W_COUNT, bound, (u64)top_k);
            if (k.overflow) break;
            bound = k.sel.key;
            cut_histogram(h, k);
        }
        u64 part = 0, total;
        for (int b = threadIdx.x; b < SB_BINS; b += SM_THREADS) part += h.mass[b];
        block_scan(part, h.scan, total);
        if (top_p < 1.0f) {
            const u64 target = (u64)ceil((double)top_p * (double)total);
            const BinSelected p = select(W_MASS, bound, target);
            if (p.overflow) break;
            bound = p.sel.key;
            total = p.sel.through;
            cut_histogram(h, p);
        }
        const BinSelected d = select(W_MASS, bound, draw_target(total, r24));
        if (d.overflow) break;
        token = (int)(d.sel.key & ((1ull << SM_ID_BITS) - 1));
    } while (false);
    __syncthreads();
    if (threadIdx.x == 0) order[0] = 1;
    __syncthreads();
    cluster_sync_all();                                    // the others see that nothing more is ordered
    cluster_sync_all();                                    // and have read it: from here on this block is alone
    if (token < 0) {                                       // a crowded bin: the exact path, by this block over the whole row
        u64* hist = dyn;
        u64* totals = dyn + SM_WARPS * 256;
        u64* shared = totals + 256;
        token = sample_exact(row, vocab, inv_t, top_k, top_p, r24, maxl, hist, totals, shared);
    }
    if (threadIdx.x == 0) {
        out[row_id] = token;
        if (out2 != nullptr) out2[row_id] = token;
        counters[row_id] = counter + 1;
    }
}

template <int C>
static int launch_sample_cluster(const float* logits, long long ld, int n_rows, int vocab, float inv_t, int top_k, float top_p,
                                 const unsigned* seeds, unsigned* counters, int* out, int* out2, size_t smem, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ti_fail("sample: %s", cudaGetErrorString(e));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_rows * C);
    cfg.blockDim = dim3(SM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = C; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ti_pdl_enabled ? 2 : 1;
    cudaLaunchKernelEx(&cfg, sample_cluster_kernel<C>, logits, ld, vocab, inv_t, top_k, top_p, seeds, counters, out, out2);
    return ti_check_launch("sample");
}

// `cluster_blocks`: blocks that share a row (1, 2, 4 or 8; 0: chosen here from the number of rows and the vocabulary).
extern "C" int ti_sample_shared(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                                float top_p, const unsigned* seeds, unsigned* counters, int* out, int* out2, int cluster_blocks,
                                cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(cluster_blocks == 0 || cluster_blocks == 1 || cluster_blocks == 2 || cluster_blocks == 4 || cluster_blocks == 8,
               "sample: %d blocks per row (0, 1, 2, 4 or 8)", cluster_blocks);
    TI_REQUIRE(vocab > 0 && vocab <= (1 << SM_ID_BITS), "sample: vocabulary %d exceeds %d", vocab, 1 << SM_ID_BITS);
    TI_REQUIRE(temperature > 0.f, "sample: temperature must be > 0 (use argmax for greedy)");
    TI_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
    TI_REQUIRE(top_p > 0.f && top_p <= 1.f, "sample: top_p must be in (0, 1]");
    // The binned path's layout (histogram, candidates, scan scratch, counts); the exact path's is smaller and shares it.
    const size_t smem = (size_t)(SB_BINS + 2 * SB_CAP + SM_WARPS + 8) * sizeof(u64) + (size_t)SB_BINS * sizeof(u32);
    static_assert((SB_BINS + 2 * SB_CAP + SM_WARPS + 8) >= (SM_WARPS * 256 + 256 + 4), "the exact path must fit the same shared memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ti_fail("sample: %s", cudaGetErrorString(e));
        configured = true;
    }
    // A few rows of a large vocabulary: a cluster of blocks per row, as many as keep the launch within one round of the SMs.
    static int sm_count = 0;                                   // asked once: the answer does not change
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0) sm_count = 1;
    }
    // Measured at a vocabulary of 131,072 on 148 SMs (us, temperature only, for 1 / 2 / 4 / 8 blocks per row): 12 rows 47 / 35 /
    // 28 / 26, 16 rows 47 / 35 / 28 / 44, 32 rows 48 / 36 / 30 / 65, 37 rows 49 / 37 / 50, 74 rows 53 / 43 / 80, 96 rows 54 / 74:
    // clusters that do not all find room at once wait for one another, the larger the earlier.
    int share = cluster_blocks;
    if (share == 0) {
        if (vocab < 32768) share = 1;                          // a pass of one block is short already
        else if (n_rows * 8 * 3 <= sm_count * 2) share = 8;
        else if (n_rows * 4 * 8 <= sm_count * 7) share = 4;
        else if (n_rows * 2 <= sm_count) share = 2;
        else share = 1;
    }
    if (share == 8) return launch_sample_cluster<8>(logits, ld, n_rows, vocab, 1.0f / temperature, top_k, top_p, seeds, counters, out, out2, smem, stream);
    if (share == 4) return launch_sample_cluster<4>(logits, ld, n_rows, vocab, 1.0f / temperature, top_k, top_p, seeds, counters, out, out2, smem, stream);
    if (share == 2) return launch_sample_cluster<2>(logits, ld, n_rows, vocab, 1.0f / temperature, top_k, top_p, seeds, counters, out, out2, smem, stream);
    ti_launch(sample_kernel, dim3(n_rows), dim3(SM_THREADS), smem, stream, logits, ld, vocab, 1.0f / temperature, top_k, top_p, seeds,
                                                        counters, out, out2);
    return ti_check_launch("sample");
}

extern "C" int ti_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, const unsigned* seeds, unsigned* counters, int* out, int* out2, cudaStream_t stream) {
    return ti_sample_shared(logits, ld, n_rows, vocab, temperature, top_k, top_p, seeds, counters, out, out2, 0, stream);
}

// The uniform number of (seed, counter), for tests of the generator itself.
extern "C" float ti_sampling_uniform(unsigned seed, unsigned counter) {
    return (float)(mix32(mix32(seed) ^ counter) >> 8) * 5.9604645e-8f;
}
