// Plain attention over the paged cache, for any element type, head size and number of
// tokens per sequence: one block per (token, query head), keys walked in position order in
// chunks of 256 with an online softmax. It is the 32-bit path's attention and the fallback
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

template <typename T>
__global__ void attention_plain_kernel(T* __restrict__ out, const T* q, const T* k_cache,
                                       const T* v_cache, const int* block_table,
                                       int table_stride, const int* tok_slot,
                                       const int* positions, float scale, int nq, int nkv, int D,
                                       int page_size, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                  // [D]
    float* sc = smem + D;              // [AP_CHUNK]
    __shared__ float scratch[33];
    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (nq / nkv);
    pdl_wait();
    pdl_launch_dependents();
    const int p = __ldcg(positions + t);
    const int* table = block_table + (size_t)__ldcg(tok_slot + t) * table_stride;
    const T* qrow = q + ((size_t)t * nq + h) * D;
    for (int d = threadIdx.x; d < D; d += AP_THREADS) qs[d] = to_f32(__ldcg(qrow + d));
    __syncthreads();

    constexpr int ACC = AP_MAX_D / AP_THREADS;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    // Chunk borders are multiples of AP_CHUNK in absolute positions.
    for (int c0 = (first / AP_CHUNK) * AP_CHUNK; c0 <= p; c0 += AP_CHUNK) {
        const int lo = c0 > first ? c0 : first;
        const int hi = (c0 + AP_CHUNK - 1 < p) ? c0 + AP_CHUNK - 1 : p;       // inclusive
        float cmax = -INFINITY;
        for (int j = lo + threadIdx.x; j <= hi; j += AP_THREADS) {
            const int page = __ldcg(table + j / page_size), off = j % page_size;
            const T* krow = k_cache + (((size_t)page * nkv + kvh) * page_size + off) * D;
            float s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(qs[d], to_f32(__ldcg(krow + d)), s);
            s *= scale;
            sc[j - c0] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = block_max(cmax, scratch);
        const float m_new = fmaxf(m, cmax);
        const float factor = (m == -INFINITY) ? 0.f : expf(m - m_new);
        float lsum = 0.f;
        for (int j = lo + threadIdx.x; j <= hi; j += AP_THREADS) {
            const float e = expf(sc[j - c0] - m_new);
            lsum += e;
            sc[j - c0] = rnd<T>(e);
        }
        lsum = block_sum(lsum, scratch);        // also orders the writes of sc before the reads below
        l = l * factor + lsum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
            const int d = threadIdx.x + i * AP_THREADS;
            if (d < D) {
                float a = acc[i] * factor;
                for (int j = lo; j <= hi; ++j) {
                    const int page = __ldcg(table + j / page_size), off = j % page_size;
                    a = fmaf(sc[j - c0], to_f32(__ldcg(v_cache + (((size_t)page * nkv + kvh) * page_size + off) * D + d)), a);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * nq + h) * D;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int d = threadIdx.x + i * AP_THREADS;
        if (d < D) orow[d] = from_f32<T>(acc[i] / l);
    }
}

extern "C" int ti_attention_plain(void* out, const void* q, const void* k_cache, const void* v_cache,
                                  const int* block_table, int table_stride, const int* tok_slot, const int* positions,
                                  float scale, int n_tokens, int nq, int nkv, int D, int page_size, int window,
                                  int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(D > 0 && D <= AP_MAX_D, "attention: head_dim %d exceeds %d", D, AP_MAX_D);
    TI_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads do not divide into %d KV heads", nq, nkv);
    TI_REQUIRE(nq <= 65535, "attention: too many heads (%d)", nq);
    dim3 grid(n_tokens, nq);
    const size_t smem = (size_t)(D + AP_CHUNK) * sizeof(float);
    TI_DISPATCH_DTYPE(dtype, (ti_launch(attention_plain_kernel<T>, dim3(grid), dim3(AP_THREADS), smem, stream, 
                                 (T*)out, (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, table_stride,
                                 tok_slot, positions, scale, nq, nkv, D, page_size, window)));
    return ti_check_launch("attention_plain");
}
