// Plain attention over the paged cache, for any element type, head size and number of
// tokens per sequence: one block per (token, KV head, a few of its query heads), keys walked in position
// order in chunks of 256 with an online softmax. It is the 32-bit path's attention and the fallback
// of the bfloat16 path for sizes the tensor-core kernels refuse.
//
// The order of every sum depends only on the query's position, never on which other tokens
// or sequences share the launch, so a position's result is bit-identical however the work
// is cut into steps or batches.
//
// AntoineBut/TileInfer.jl: query head h reads KV head h div group
// (src/ops/reference.jl:108-112); the key at position i is visible to the query at
// position p iff i <= p, over all cached positions (reference.jl:98-107); scores, softmax
// and the accumulator are 32-bit, P is rounded to the storage type only for the PV product,
// O is rounded once (src/ops/tile/attention.jl:1-3, 34-59).
#include "common.cuh"

#define AP_THREADS 128
#define AP_CHUNK 256
#define AP_MAX_D 512
#define AP_HEADS 4        // query heads of one KV head that a block serves together

// One block per (token, KV head, set of up to AP_HEADS of its query heads): a key's row and a value's element are
// read once for all the heads of the set. Per head the arithmetic is what it would be alone (the same thread owns
// the same keys and dimensions, the same reductions in the same order), so a head's result does not depend on
// how the heads are grouped.
template <typename T>
__global__ void attention_plain_kernel(T* __restrict__ out, const T* q, const T* k_cache,
                                       const T* v_cache, const int* block_table,
                                       int table_stride, const int* tok_slot,
                                       const int* positions, float scale, int nq, int nkv, int D,
                                       int page_size, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                          // [AP_HEADS][D]
    float* sc = smem + AP_HEADS * D;           // [AP_HEADS][AP_CHUNK]
    __shared__ float scratch[33];
    const int group = nq / nkv;
    const int sets = (group + AP_HEADS - 1) / AP_HEADS;
    const int t = blockIdx.x, kvh = blockIdx.y / sets;
    const int h0 = kvh * group + (blockIdx.y % sets) * AP_HEADS;           // first query head of the set
    const int heads = min(AP_HEADS, kvh * group + group - h0);
    pdl_wait();
    pdl_launch_dependents();
    const int p = __ldcg(positions + t);
    const int* table = block_table + (size_t)__ldcg(tok_slot + t) * table_stride;
    for (int i = threadIdx.x; i < heads * D; i += AP_THREADS) qs[i] = to_f32(__ldcg(q + ((size_t)t * nq + h0) * D + i));
    __syncthreads();

    constexpr int ACC = AP_MAX_D / AP_THREADS;
    float acc[AP_HEADS][ACC];
    float m[AP_HEADS], l[AP_HEADS];
#pragma unroll
    for (int h = 0; h < AP_HEADS; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[h][i] = 0.f;
    }
    const int first = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const bool wide = D % Vec16<T>::N == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0;
    // Chunk borders are multiples of AP_CHUNK in absolute positions.
    for (int c0 = (first / AP_CHUNK) * AP_CHUNK; c0 <= p; c0 += AP_CHUNK) {
        const int lo = c0 > first ? c0 : first;
        const int hi = (c0 + AP_CHUNK - 1 < p) ? c0 + AP_CHUNK - 1 : p;       // inclusive
        float cmax[AP_HEADS];
#pragma unroll
        for (int h = 0; h < AP_HEADS; ++h) cmax[h] = -INFINITY;
        for (int j = lo + threadIdx.x; j <= hi; j += AP_THREADS) {
            const int page = __ldcg(table + j / page_size), off = j % page_size;
            const T* krow = k_cache + (((size_t)page * nkv + kvh) * page_size + off) * D;
            float s[AP_HEADS];
#pragma unroll
            for (int h = 0; h < AP_HEADS; ++h) s[h] = 0.f;
            constexpr int VEC = Vec16<T>::N;
            if (wide) {                                      // 16 bytes of the key's row at a time; the terms are still added one by one
                for (int d0 = 0; d0 < D; d0 += VEC) {
                    Vec16<T> kv;
                    kv.load_cg(krow + d0);
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
#pragma unroll
                        for (int h = 0; h < AP_HEADS; ++h)
                            if (h < heads) s[h] = fmaf(qs[h * D + d0 + e], kv.v[e], s[h]);
                }
            } else {
                for (int d = 0; d < D; ++d) {
                    const float kd = to_f32(__ldcg(krow + d));
#pragma unroll
                    for (int h = 0; h < AP_HEADS; ++h)
                        if (h < heads) s[h] = fmaf(qs[h * D + d], kd, s[h]);
                }
            }
#pragma unroll
            for (int h = 0; h < AP_HEADS; ++h)
                if (h < heads) {
                    s[h] *= scale;
                    sc[h * AP_CHUNK + j - c0] = s[h];
                    cmax[h] = fmaxf(cmax[h], s[h]);
                }
        }
        float factor[AP_HEADS];
#pragma unroll
        for (int h = 0; h < AP_HEADS; ++h) {
            if (h >= heads) continue;                                          // uniform across the block
            const float cm = block_max(cmax[h], scratch);
            const float m_new = fmaxf(m[h], cm);
            factor[h] = (m[h] == -INFINITY) ? 0.f : expf(m[h] - m_new);
            float lsum = 0.f;
            for (int j = lo + threadIdx.x; j <= hi; j += AP_THREADS) {
                const float e = expf(sc[h * AP_CHUNK + j - c0] - m_new);
                lsum += e;
                sc[h * AP_CHUNK + j - c0] = rnd<T>(e);
            }
            lsum = block_sum(lsum, scratch);        // also orders the writes of sc before the reads below
            l[h] = l[h] * factor[h] + lsum;
            m[h] = m_new;
        }
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
            const int d = threadIdx.x + i * AP_THREADS;
            if (d < D) {
                float a[AP_HEADS];
#pragma unroll
                for (int h = 0; h < AP_HEADS; ++h) a[h] = h < heads ? acc[h][i] * factor[h] : 0.f;
                for (int j = lo; j <= hi; ++j) {
                    const int page = __ldcg(table + j / page_size), off = j % page_size;
                    const float vd = to_f32(__ldcg(v_cache + (((size_t)page * nkv + kvh) * page_size + off) * D + d));
#pragma unroll
                    for (int h = 0; h < AP_HEADS; ++h)
                        if (h < heads) a[h] = fmaf(sc[h * AP_CHUNK + j - c0], vd, a[h]);
                }
#pragma unroll
                for (int h = 0; h < AP_HEADS; ++h) acc[h][i] = a[h];
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < AP_HEADS; ++h) {
        if (h >= heads) continue;
        T* orow = out + ((size_t)t * nq + h0 + h) * D;
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
            const int d = threadIdx.x + i * AP_THREADS;
            if (d < D) orow[d] = from_f32<T>(acc[h][i] / l[h]);
        }
    }
}

extern "C" int ti_attention_plain(void* out, const void* q, const void* k_cache, const void* v_cache,
                                  const int* block_table, int table_stride, const int* tok_slot, const int* positions,
                                  float scale, int n_tokens, int nq, int nkv, int D, int page_size, int window,
                                  int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(D > 0 && D <= AP_MAX_D, "attention: head_dim %d exceeds %d", D, AP_MAX_D);
    TI_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
    const int sets = (nq / nkv + AP_HEADS - 1) / AP_HEADS;
    TI_REQUIRE((long long)nkv * sets <= 65535, "attention: too many heads (%d)", nq);
    dim3 grid(n_tokens, nkv * sets);
    const size_t smem = (size_t)AP_HEADS * (D + AP_CHUNK) * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(attention_plain_kernel<T>, dim3(grid), dim3(AP_THREADS), smem, stream, 
                                 (T*)out, (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, table_stride,
                                 tok_slot, positions, scale, nq, nkv, D, page_size, window)));
    return ti_check_launch("attention_plain");
}
