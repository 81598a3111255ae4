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
// Method: no sort. Each token gets a 56-bit key (descending-ordered logit bits, then id), so
// best-first order is ascending key order, and "the first key whose cumulative weight
// reaches X" is found by a radix select over that key, 8 bits a pass, with a histogram of
// weights. Weights are 2^40 fixed-point integers, so sums do not depend on the order of the
// atomic additions and the result is deterministic.
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
                                                            int* __restrict__ out, float* ws_val, int* ws_idx,
                                                            unsigned* counters) {
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

extern "C" int ti_argmax(const float* logits, long long ld, int n_rows, int vocab, int* out, float* ws_val, int* ws_idx,
                         unsigned* counters, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(vocab > 0, "argmax: vocab %d", vocab);
    TI_REQUIRE(n_rows <= 65535, "argmax: %d rows in one launch", n_rows);
    TI_REQUIRE(ws_val != nullptr && ws_idx != nullptr && counters != nullptr, "argmax: work space missing");
    const int chunks = ti_argmax_chunks(vocab);
    int per_chunk = (vocab + chunks - 1) / chunks;
    per_chunk = (per_chunk + 3) & ~3;
    ti_launch(argmax_kernel, dim3(chunks, n_rows), dim3(AM_THREADS), 0, stream, logits, ld, vocab, per_chunk, out, ws_val, ws_idx,
              counters);
    return ti_check_launch("argmax");
}

// ------------------------------------------------------------------------------ sampling
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

__global__ void __launch_bounds__(SM_THREADS) sample_kernel(const float* logits, long long ld, int vocab,
                                                            float inv_t, int top_k, float top_p,
                                                            const u32* seeds, u32* counters,
                                                            int* __restrict__ out) {
    extern __shared__ u64 dyn[];
    u64* hist = dyn;
    u64* totals = dyn + SM_WARPS * 256;
    u64* shared = totals + 256;
    __shared__ float scratch[33];
    const float* row = logits + (size_t)blockIdx.x * ld;
    pdl_wait();
    pdl_launch_dependents();

    float maxl = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += SM_THREADS) maxl = fmaxf(maxl, __ldcg(row + i));
    maxl = block_max(maxl, scratch);

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
    const u32 counter = counters[blockIdx.x];
    const u32 r24 = mix32(mix32(seeds[blockIdx.x]) ^ counter) >> 8;          // u = r24 · 2^-24
    // ceil(u × total) without leaving integers: total < 2^58 and r24 < 2^24 need 128 bits.
    const u64 hi = __umul64hi(total, (u64)r24), lo = total * (u64)r24;
    u64 target = (hi << 40) | (lo >> 24);
    if (lo & 0xFFFFFFull) target += 1;
    const Selected s = select_key(row, vocab, W_MASS, bound, target, maxl, inv_t, hist, totals, shared);
    if (threadIdx.x == 0) {
        out[blockIdx.x] = (int)(s.key & ((1ull << SM_ID_BITS) - 1));
        counters[blockIdx.x] = counter + 1;
    }
}

extern "C" int ti_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k,
                         float top_p, const unsigned* seeds, unsigned* counters, int* out, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(vocab > 0 && vocab <= (1 << SM_ID_BITS), "sample: vocabulary %d exceeds %d", vocab, 1 << SM_ID_BITS);
    TI_REQUIRE(temperature > 0.f, "sample: temperature must be > 0 (use argmax for greedy)");
    TI_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
    TI_REQUIRE(top_p > 0.f && top_p <= 1.f, "sample: top_p must be in (0, 1]");
    const size_t smem = (size_t)(SM_WARPS * 256 + 256 + 4) * sizeof(u64);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ti_fail("sample: %s", cudaGetErrorString(e));
        configured = true;
    }
    ti_launch(sample_kernel, dim3(n_rows), dim3(SM_THREADS), smem, stream, logits, ld, vocab, 1.0f / temperature, top_k, top_p, seeds,
                                                        counters, out);
    return ti_check_launch("sample");
}

// The uniform number of (seed, counter), for tests of the generator itself.
extern "C" float ti_sampling_uniform(unsigned seed, unsigned counter) {
    return (float)(mix32(mix32(seed) ^ counter) >> 8) * 5.9604645e-8f;
}
