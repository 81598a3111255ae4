// Embedding gather, row gather, xIELU, RMSNorm and the fused residual-add + RMSNorm.
//
// Formulas and rounding points follow AntoineBut/TileInfer.jl: embedding
// src/ops/reference.jl:10; RMSNorm (normalise in 32-bit, round, then scale in the storage
// type) src/ops/reference.jl:17-21; residual add rounded to the storage type before the norm
// src/ops/tile/norm.jl:48-77; xIELU src/ops/reference.jl:49-56.
#include "common.cuh"

static thread_local char g_error[512] = "";

extern "C" const char* ti_last_error() { return g_error; }

int ti_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

int ti_pdl_enabled = 1;

// Switch programmatic dependent launch on or off for every later launch (default on).
extern "C" void ti_set_pdl(int enabled) { ti_pdl_enabled = enabled ? 1 : 0; }

// Streaming multiprocessors of the current device, read once; 148 (a B200) where no device answers, so
// that the host-side plans can be computed and tested without one.
extern "C" int ti_sm_count() {
    static int count = 0;
    if (!count) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            count = n;
        else {
            cudaGetLastError();
            count = 148;
        }
    }
    return count;
}

int ti_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ti_fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

// One row of `size` elements, 16 bytes per access where both ends allow it.
template <typename T> __device__ __forceinline__ void copy_row(T* dst, const T* src, int size) {
    constexpr int N = 16 / sizeof(T);
    if (size % N == 0 && (((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < size / N; i += blockDim.x) d4[i] = __ldcg(s4 + i);
    } else {
        for (int i = threadIdx.x; i < size; i += blockDim.x) dst[i] = __ldcg(src + i);
    }
}

// ---------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(T* __restrict__ out, const T* __restrict__ table, const int* ids,
                             int hidden, int vocab, int* __restrict__ status) {
    const int t = blockIdx.x;
    pdl_enter();
    int id = __ldcg(ids + t);
    if (id < 0 || id >= vocab) {            // never read outside the table; report instead
        if (threadIdx.x == 0) atomicExch(status, 1 + t);
        id = 0;
    }
    const T* row = table + (size_t)id * hidden;
    T* dst = out + (size_t)t * hidden;
    copy_row(dst, row, hidden);
}

extern "C" int ti_embed(void* out, const void* table, const int* ids, int n_tokens, int hidden, int vocab,
                        int dtype, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embed: bad sizes n=%d hidden=%d vocab=%d", n_tokens, hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(embed_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (T*)out, (const T*)table, ids, hidden, vocab, status)));
    return ti_check_launch("embed");
}

// Rows idx[i] of x [*, size] to out [n, size] (the positions whose logits are wanted).
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* x, const int* idx, int size) {
    pdl_enter();
    const T* row = x + (size_t)__ldcg(idx + blockIdx.x) * size;
    T* dst = out + (size_t)blockIdx.x * size;
    copy_row(dst, row, size);
}

extern "C" int ti_gather_rows(void* out, const void* x, const int* idx, int n, int size, int dtype, cudaStream_t stream) {
    if (n == 0) return 0;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(gather_rows_kernel<T>, dim3(n), dim3(128), 0, stream, (T*)out, (const T*)x, idx, size)));
    return ti_check_launch("gather_rows");
}

// ---------------------------------------------------------------------------- xIELU
template <typename T>
__global__ void xielu_kernel(T* out, const T* in, size_t count, XieluParams a) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_wait();
    pdl_launch_dependents();
    for (; i < count; i += stride) out[i] = from_f32<T>(xielu_value<T>(to_f32(__ldcg(in + i)), a));
}

template <typename T>
__global__ void xielu_vec_kernel(T* out, const T* in, size_t vecs, XieluParams a) {
    constexpr int N = Vec16<T>::N;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_wait();
    pdl_launch_dependents();
    for (; i < vecs; i += stride) {
        Vec16<T> v;
        v.load_cg(in + i * N);
#pragma unroll
        for (int e = 0; e < N; ++e) v.v[e] = xielu_value<T>(v.v[e], a);
        v.store(out + i * N);
    }
}

extern "C" int ti_xielu(void* out, const void* in, long long count, float alpha_p, float alpha_n, float beta, float eps,
                        int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    XieluParams a{alpha_p, alpha_n, beta, eps};
    TI_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        if (count % N == 0 && aligned16(out) && aligned16(in)) {
            long long blocks = (count / N + 255) / 256;
            if (blocks > ti_sm_count() * 32) blocks = ti_sm_count() * 32;
            ti_launch(xielu_vec_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const T*)in, (size_t)(count / N), a);
        } else {
            long long blocks = (count + 255) / 256;
            if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
            ti_launch(xielu_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (const T*)in, (size_t)count, a);
        }
    });
    return ti_check_launch("xielu");
}

// ---------------------------------------------------------------------------- RMSNorm
// One block per row. y = rnd(w * rnd(x * inv_rms)), inv_rms = 1/sqrt(mean(x^2) + eps) in 32-bit.
template <typename T>
__global__ void rmsnorm_kernel(T* y, const T* x, const T* __restrict__ w, int size, float eps) {
    __shared__ float scratch[33];
    const T* row = x + (size_t)blockIdx.x * size;
    T* dst = y + (size_t)blockIdx.x * size;
    float ss = 0.f;
    pdl_wait();
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = to_f32(__ldcg(row + i));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<T>(to_f32(w[i]) * rnd<T>(to_f32(__ldcg(row + i)) * inv));
}

// The same with 16-byte accesses: every thread owns up to MAXV vectors of its row, so all loads
// of a row are in flight at once and the row is read from memory exactly once. Decode steps
// are a handful of rows, where the latency of a serial loop would be the whole cost.
#define RN_MAXV 4
template <typename T>
__global__ void rmsnorm_vec_kernel(T* y, const T* x, const T* __restrict__ w, int size, float eps) {
    __shared__ float scratch[33];
    constexpr int N = Vec16<T>::N;
    const T* row = x + (size_t)blockIdx.x * size;
    T* dst = y + (size_t)blockIdx.x * size;
    Vec16<T> v[RN_MAXV];
    float ss = 0.f;
    pdl_enter();
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * N;
        if (i < size) {
            v[j].load_cg(row + i);
#pragma unroll
            for (int e = 0; e < N; ++e) ss = fmaf(v[j].v[e], v[j].v[e], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * N;
        if (i < size) {
            Vec16<T> wv;
            wv.load(w + i);
#pragma unroll
            for (int e = 0; e < N; ++e) v[j].v[e] = wv.v[e] * rnd<T>(v[j].v[e] * inv);
            v[j].store(dst + i);
        }
    }
}

template <typename T, bool LATE_W = false>
__global__ void __launch_bounds__(512, LATE_W ? 2 : 1) add_rmsnorm_vec_kernel(T* x, const T* delta, const float* partials,
                                       int n_partials, size_t partial_stride, const T* __restrict__ w, T* __restrict__ h,
                                       int size, float eps) {
    __shared__ float scratch[33];
    constexpr int N = Vec16<T>::N;
    T* row = x + (size_t)blockIdx.x * size;
    T* dst = h + (size_t)blockIdx.x * size;
    Vec16<T> v[RN_MAXV], wv[RN_MAXV];
    float ss = 0.f;
    // The norm's weight does not depend on the predecessor: it is read before waiting for it.
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * N;
        if (!LATE_W && i < size) wv[j].load(w + i);
    }
    pdl_enter();
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * N;
        if (i < size) {
            v[j].load_cg(row + i);
            float d[N];
            if (partials != nullptr) {
                const float* p = partials + (size_t)blockIdx.x * size + i;
#pragma unroll
                for (int e = 0; e < N; e += 4) {
                    const float4 t = __ldcg(reinterpret_cast<const float4*>(p + e));
                    d[e] = t.x; d[e + 1] = t.y; d[e + 2] = t.z; d[e + 3] = t.w;
                }
                // Eight splits at a time: their loads are issued together, the additions stay in split order.
                for (int s0 = 1; s0 < n_partials; s0 += 8) {
                    float4 t[8][N / 4];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int e = 0; e < N; e += 4)
                            t[u][e / 4] = s0 + u < n_partials
                                              ? __ldcg(reinterpret_cast<const float4*>(p + (size_t)(s0 + u) * partial_stride + e))
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; ++u)
#pragma unroll
                        for (int e = 0; e < N; e += 4) {
                            d[e] += t[u][e / 4].x; d[e + 1] += t[u][e / 4].y; d[e + 2] += t[u][e / 4].z; d[e + 3] += t[u][e / 4].w;
                        }
                }
#pragma unroll
                for (int e = 0; e < N; ++e) d[e] = rnd<T>(d[e]);
            } else {
                Vec16<T> dv;
                dv.load_cg(delta + (size_t)blockIdx.x * size + i);
#pragma unroll
                for (int e = 0; e < N; ++e) d[e] = dv.v[e];
            }
#pragma unroll
            for (int e = 0; e < N; ++e) {
                v[j].v[e] = rnd<T>(v[j].v[e] + d[e]);
                ss = fmaf(v[j].v[e], v[j].v[e], ss);
            }
            v[j].store(row + i);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * N;
        if (i < size) {
            if (LATE_W) wv[j].load(w + i);
#pragma unroll
            for (int e = 0; e < N; ++e) v[j].v[e] = wv[j].v[e] * rnd<T>(v[j].v[e] * inv);
            v[j].store(dst + i);
        }
    }
}

// Threads for the vector kernels: enough that RN_MAXV vectors per thread cover the row; 0 if they cannot.
template <typename T> static int vec_threads(int size) {
    constexpr int N = Vec16<T>::N;
    if (size % N) return 0;
    const int vecs = size / N;
    int threads = 64;
    while (threads < 1024 && threads * RN_MAXV < vecs) threads *= 2;
    if (threads * RN_MAXV < vecs) return 0;
    while (threads > 64 && (threads / 2) >= vecs) threads /= 2;     // do not launch idle warps for small rows
    return threads;
}

extern "C" int ti_rmsnorm(void* y, const void* x, const void* w, int n_rows, int size, float eps, int dtype, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(size > 0, "rmsnorm: size %d", size);
    const int threads = size >= 2048 ? 512 : size >= 512 ? 256 : 128;
    const bool al = aligned16(y) && aligned16(x) && aligned16(w);
    TI_DISPATCH_DTYPE(dtype, {
        const int vt = al ? vec_threads<T>(size) : 0;
        if (vt) ti_launch(rmsnorm_vec_kernel<T>, dim3(n_rows), dim3(vt), 0, stream, (T*)y, (const T*)x, (const T*)w, size, eps);
        else ti_launch(rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), 0, stream, (T*)y, (const T*)x, (const T*)w, size, eps);
    });
    return ti_check_launch("rmsnorm");
}

// x <- rnd(x + d), h <- RMSNorm(x) * w. d is either `delta` (storage type) or the sum, in
// a fixed order, of `n_partials` 32-bit partial products [s][n_rows][size] (a split-K
// matrix product), rounded to the storage type first like any product's output.
template <typename T>
__global__ void add_rmsnorm_kernel(T* x, const T* delta, const float* partials,
                                   int n_partials, size_t partial_stride, const T* __restrict__ w, T* __restrict__ h,
                                   int size, float eps) {
    __shared__ float scratch[33];
    T* row = x + (size_t)blockIdx.x * size;
    T* dst = h + (size_t)blockIdx.x * size;
    float ss = 0.f;
    pdl_wait();
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float d;
        if (partials != nullptr) {
            const float* p = partials + (size_t)blockIdx.x * size + i;
            d = __ldcg(p);
            for (int s = 1; s < n_partials; ++s) d += __ldcg(p + (size_t)s * partial_stride);
            d = rnd<T>(d);
        } else {
            d = to_f32(__ldcg(delta + (size_t)blockIdx.x * size + i));
        }
        const float v = rnd<T>(to_f32(__ldcg(row + i)) + d);
        row[i] = from_f32<T>(v);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)size + eps);
    // Each thread re-reads exactly the elements it wrote above.
    for (int i = threadIdx.x; i < size; i += blockDim.x)
        dst[i] = from_f32<T>(to_f32(w[i]) * rnd<T>(to_f32(__ldcg(row + i)) * inv));
}

extern "C" int ti_add_rmsnorm(void* x, const void* delta, const float* partials, int n_partials, long long partial_stride,
                              const void* w, void* h, int n_rows, int size, float eps, int dtype, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    TI_REQUIRE(size > 0, "add_rmsnorm: size %d", size);
    TI_REQUIRE((delta != nullptr) != (partials != nullptr), "add_rmsnorm: give delta or partials, not both");
    TI_REQUIRE(partials == nullptr || n_partials >= 1, "add_rmsnorm: n_partials %d", n_partials);
    const int threads = size >= 2048 ? 512 : size >= 512 ? 256 : 128;
    const bool al = aligned16(x) && aligned16(w) && aligned16(h) && (delta == nullptr || aligned16(delta)) &&
                    (partials == nullptr || (aligned16(partials) && partial_stride % 4 == 0));
    TI_DISPATCH_DTYPE(dtype, {
        int vt = al ? vec_threads<T>(size) : 0;
        if (vt > 512) vt = 0;                  // the vector kernel's registers allow 512 threads: longer rows take the plain kernel
        if (vt && ((partials != nullptr && n_partials > 1) || (n_rows <= 16 && sizeof(T) == 2))) {
            // The loop over the partial sums of one vector cannot be overlapped with the next vector's (its
            // length is not known to the compiler): one vector per thread, so that a row is one round of loads.
            // The same for a handful of rows (a decode step), where the kernel is one dependent round trip and
            // more threads make it shorter: 8 layers of one / eight sequences 853 / 997 us against 879 / 1,023 us.
            // (Not in 32-bit, where the order of a row's sum of squares must not depend on the number of rows.)
            const int vecs = size / Vec16<T>::N;
            const int one_each = vecs >= 512 ? 512 : (vecs + 31) / 32 * 32;      // 512 threads of this kernel fill an SM's registers
            if (one_each > vt) vt = one_each;
        }
        // Many rows (a prompt's step): the weight is read after the reduction instead of being held across it, and the
        // kernel is held to 64 registers, for eight blocks of 128 threads per SM instead of four (14.4 against 20.1 us
        // for 2,048 rows of 4,096). A few rows (a decode step) read it before waiting for the predecessor.
        if (vt && n_rows > 16) ti_launch(add_rmsnorm_vec_kernel<T, true>, dim3(n_rows), dim3(vt), 0, stream, (T*)x, (const T*)delta, partials, n_partials,
                                                                    (size_t)partial_stride, (const T*)w, (T*)h, size, eps);
        else if (vt) ti_launch(add_rmsnorm_vec_kernel<T>, dim3(n_rows), dim3(vt), 0, stream, (T*)x, (const T*)delta, partials, n_partials,
                                                                    (size_t)partial_stride, (const T*)w, (T*)h, size, eps);
        else ti_launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), 0, stream, (T*)x, (const T*)delta, partials, n_partials,
                                                                  (size_t)partial_stride, (const T*)w, (T*)h, size, eps);
    });
    return ti_check_launch("add_rmsnorm");
}

// Plain residual add for blocks whose next norm is not fused: x <- rnd(x + delta).
template <typename T>
__global__ void add_kernel(T* x, const T* delta, size_t count) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    pdl_wait();
    pdl_launch_dependents();
    for (; i < count; i += stride) x[i] = from_f32<T>(to_f32(__ldcg(x + i)) + to_f32(__ldcg(delta + i)));
}

extern "C" int ti_add(void* x, const void* delta, long long count, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 16) blocks = ti_sm_count() * 16;
    TI_DISPATCH_DTYPE(dtype, (ti_launch(add_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)x, (const T*)delta, (size_t)count)));
    return ti_check_launch("add");
}
