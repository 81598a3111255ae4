// Plain matrix product y[n, out] = x[n, in] · W[out, in]ᵀ on the CUDA cores, for any sizes
// and either element type. Inputs are widened to 32-bit, every product is a 32-bit fused
// multiply-add (no tensor-core or reduced-precision mode), and each output element sums its
// k terms in ascending order whatever n is: a row's result is bit-identical in a step of
// one token and in a step of thousands. It is the 32-bit path's product and the fallback of
// the bfloat16 path for sizes the tensor-core kernel refuses.
//
// AntoineBut/TileInfer.jl: weights stay [out, in] row-major, y = Wᵀx with 32-bit
// accumulation and one rounding (src/ops/reference.jl:23-26, src/ops/tile/linear.jl:12-13);
// the logits leave in 32-bit after that rounding (src/ops/tile/linear.jl:26).
#include "common.cuh"
#include "mma_util.cuh"

#define GP_BM 64      // tokens per tile
#define GP_BN 64      // output features per tile
#define GP_BK 16

#define TI_EPI_NONE 0
#define TI_EPI_XIELU 1
#define TI_EPI_F32_OUT 2   // round to the storage type, store 32-bit (logits)

template <typename T>
__global__ void __launch_bounds__(256) gemm_plain_kernel(void* __restrict__ y, long long ldy, const T* x,
                                                        long long ldx, const T* __restrict__ W, int n, int out,
                                                        int in, int epilogue, XieluParams act) {
    __shared__ float As[GP_BK][GP_BM + 4];
    __shared__ float Bs[GP_BK][GP_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GP_BM, n0 = blockIdx.x * GP_BN;
    const int tr = tid / 16, tc = tid % 16;       // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // Each thread stages 4 consecutive k of one row of each operand tile.
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    pdl_wait();
    pdl_launch_dependents();
    for (int k0 = 0; k0 < in; k0 += GP_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int r = m0 + lrow, c = n0 + lrow;
            As[lk + i][lrow] = (r < n && k < in) ? to_f32(__ldcg(x + (size_t)r * ldx + k)) : 0.f;
            Bs[lk + i][lrow] = (c < out && k < in) ? to_f32(W[(size_t)c * in + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GP_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tr * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tc * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + tr * 4 + i;
        if (r >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tc * 4 + j;
            if (c >= out) continue;
            float v = rnd<T>(acc[i][j]);
            if (epilogue == TI_EPI_XIELU) v = xielu_value<T>(v, act);
            if (epilogue == TI_EPI_F32_OUT) ((float*)y)[(size_t)r * ldy + c] = v;
            else ((T*)y)[(size_t)r * ldy + c] = from_f32<T>(v);
        }
    }
}

// The same product in larger tiles for steps of many tokens whose rows can be read 16 bytes at a time:
// 128 tokens x 128 features per block, 8 x 8 outputs per thread, the next k block's global loads in flight
// while the current one is multiplied. Every output still sums its k terms in ascending order with single
// fused multiply-adds from zero, so the bits are those of the kernels above and below.
#define GB_T 128
#define GB_BK 8

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 t = __ldcg(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_plain_wide_kernel(void* __restrict__ y, long long ldy, const T* x, long long ldx,
                                                             const T* __restrict__ W, int n, int out, int in, int epilogue,
                                                             XieluParams act) {
    __shared__ __align__(16) float As[2][GB_BK][GB_T + 4];
    __shared__ __align__(16) float Bs[2][GB_BK][GB_T + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GB_T, n0 = blockIdx.x * GB_T;
    const int ty = tid / 16, tx = tid % 16;            // 8 tokens x 8 features each
    const int lrow = tid / 2, lk = (tid % 2) * 4;      // staging: 4 consecutive k of one row of each operand
    const bool a_ok = m0 + lrow < n, b_ok = n0 + lrow < out;
    const T* a_src = x + (size_t)(a_ok ? m0 + lrow : 0) * ldx + lk;
    const T* b_src = W + (size_t)(b_ok ? n0 + lrow : 0) * in + lk;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float ra[4], rb[4];
    auto fetch = [&](int k0) {                          // in % 4 == 0: a vector of 4 is inside the row or outside it
        const bool k_ok = k0 + lk < in;
        if (a_ok && k_ok) load4<T>(a_src + k0, ra); else { ra[0] = ra[1] = ra[2] = ra[3] = 0.f; }
        if (b_ok && k_ok) load4<T>(b_src + k0, rb); else { rb[0] = rb[1] = rb[2] = rb[3] = 0.f; }
    };
    auto stage = [&](int buf) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            As[buf][lk + e][lrow] = ra[e];
            Bs[buf][lk + e][lrow] = rb[e];
        }
    };
    pdl_wait();
    pdl_launch_dependents();
    fetch(0);
    stage(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < in; k0 += GB_BK) {
        const bool more = k0 + GB_BK < in;
        if (more) fetch(k0 + GB_BK);
#pragma unroll
        for (int kk = 0; kk < GB_BK; ++kk) {
            float a[8], b[8];
            *reinterpret_cast<float4*>(a) = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 8]);
            *reinterpret_cast<float4*>(a + 4) = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 8 + 4]);
            *reinterpret_cast<float4*>(b) = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 8]);
            *reinterpret_cast<float4*>(b + 4) = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 8 + 4]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) stage(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = m0 + ty * 8 + i;
        if (r >= n) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = n0 + tx * 8 + j;
            if (c >= out) continue;
            float v = rnd<T>(acc[i][j]);
            if (epilogue == TI_EPI_XIELU) v = xielu_value<T>(v, act);
            if (epilogue == TI_EPI_F32_OUT) ((float*)y)[(size_t)r * ldy + c] = v;
            else ((T*)y)[(size_t)r * ldy + c] = from_f32<T>(v);
        }
    }
}

// The same product for steps of few tokens (decode): a block owns GV_ROWS output features and streams their
// weight rows once, in k blocks that are staged in shared memory with 16-byte loads; a thread owns one
// feature and every GV_SLOTS-th token and sums its k terms in ascending order with single fused
// multiply-adds, starting from zero: the same chain as the tiled kernel above, so a row's result has the
// same bits whichever of the two ran. With 8 tokens the tiled kernel would compute 64 token rows of which 56
// are padding and run out/64 blocks; this one runs out/16 blocks that do nothing but stream.
#define GV_ROWS 16
#define GV_SLOTS 8
#define GV_BK 64
#define GV_MAX_TOKENS 64

template <typename T, int TPT>                           // TPT: tokens per thread (the step has at most TPT * GV_SLOTS tokens)
__global__ void __launch_bounds__(GV_ROWS * GV_SLOTS) gemv_plain_kernel(void* __restrict__ y, long long ldy, const T* x, long long ldx,
                                                                         const T* __restrict__ W, int n, int out, int in, int epilogue,
                                                                         XieluParams act) {
    __shared__ float Ws[GV_ROWS][GV_BK + 1];
    extern __shared__ float Xs[];                         // [n][GV_BK + 1]
    const int tid = threadIdx.x;
    const int row = tid % GV_ROWS, slot = tid / GV_ROWS;
    const int m0 = blockIdx.x * GV_ROWS;
    float acc[TPT];
#pragma unroll
    for (int j = 0; j < TPT; ++j) acc[j] = 0.f;
    constexpr int VEC = 16 / sizeof(T);                   // elements per 16-byte load
    const bool wide = (in % VEC) == 0 && (((uintptr_t)W) & 15) == 0;
    // Weights do not depend on the previous kernel: the first block of them is on its way before the wait.
    auto load_w = [&](int k0) {
        if (wide) {
            for (int i = tid; i < GV_ROWS * (GV_BK / VEC); i += GV_ROWS * GV_SLOTS) {
                const int r = i / (GV_BK / VEC), kv = (i % (GV_BK / VEC)) * VEC;
                const int c = m0 + r, k = k0 + kv;
                if (c < out && k < in) {                  // in % VEC == 0: a vector is inside the row or outside it
                    Vec16<T> v;
                    v.load(W + (size_t)c * in + k);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) Ws[r][kv + e] = v.v[e];
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) Ws[r][kv + e] = 0.f;
                }
            }
        } else {
            for (int i = tid; i < GV_ROWS * GV_BK; i += GV_ROWS * GV_SLOTS) {
                const int r = i / GV_BK, kk = i % GV_BK;
                const int c = m0 + r, k = k0 + kk;
                Ws[r][kk] = (c < out && k < in) ? to_f32(W[(size_t)c * in + k]) : 0.f;
            }
        }
    };
    load_w(0);
    pdl_wait();
    pdl_launch_dependents();
    for (int k0 = 0; k0 < in; k0 += GV_BK) {
        if (k0 > 0) load_w(k0);
        for (int i = tid; i < n * GV_BK; i += GV_ROWS * GV_SLOTS) {
            const int t = i / GV_BK, kk = i % GV_BK;
            Xs[t * (GV_BK + 1) + kk] = (k0 + kk < in) ? to_f32(__ldcg(x + (size_t)t * ldx + k0 + kk)) : 0.f;
        }
        __syncthreads();
        const int kmax = min(GV_BK, in - k0);             // terms beyond `in` are not added (the tiled kernel adds +0 there: the same sum)
#pragma unroll 4
        for (int kk = 0; kk < kmax; ++kk) {
            const float w = Ws[row][kk];
#pragma unroll
            for (int j = 0; j < TPT; ++j) {
                const int t = slot + j * GV_SLOTS;
                if (t < n) acc[j] = fmaf(Xs[t * (GV_BK + 1) + kk], w, acc[j]);
            }
        }
        __syncthreads();
    }
    const int c = m0 + row;
    if (c >= out) return;
#pragma unroll
    for (int j = 0; j < TPT; ++j) {
        const int t = slot + j * GV_SLOTS;
        if (t >= n) continue;
        float v = rnd<T>(acc[j]);
        if (epilogue == TI_EPI_XIELU) v = xielu_value<T>(v, act);
        if (epilogue == TI_EPI_F32_OUT) ((float*)y)[(size_t)t * ldy + c] = v;
        else ((T*)y)[(size_t)t * ldy + c] = from_f32<T>(v);
    }
}

// The weight-streaming kernel with its k blocks in flight: the same block shape and the same sums, but the
// weight rows' and the tokens' k blocks are copied to shared memory with 16-byte cp.async several stages ahead
// (raw, widened when they are read), so that a block has tens of kilobytes in flight instead of one k block.
// It needs rows that can be read 16 bytes at a time; the kernel above serves the rest.
template <typename T, int TPT, int STAGES>
__global__ void __launch_bounds__(GV_ROWS * GV_SLOTS) gemv_plain_pipe_kernel(void* __restrict__ y, long long ldy, const T* x, long long ldx,
                                                                              const T* __restrict__ W, int n, int out, int in, int epilogue,
                                                                              XieluParams act) {
    extern __shared__ __align__(16) unsigned char pipe_smem[];
    constexpr int VEC = 16 / sizeof(T);                    // elements per 16-byte chunk
    constexpr int CHUNKS = GV_BK / VEC;                    // chunks per row of a k block
    constexpr int ROW = GV_BK + VEC;                       // elements between rows in shared memory (16 bytes of padding)
    const int stage_elems = (GV_ROWS + n) * ROW;
    T* stages = reinterpret_cast<T*>(pipe_smem);
    const int tid = threadIdx.x;
    const int row = tid % GV_ROWS, slot = tid / GV_ROWS;
    const int m0 = blockIdx.x * GV_ROWS;
    float acc[TPT];
#pragma unroll
    for (int j = 0; j < TPT; ++j) acc[j] = 0.f;
    const int tiles = (in + GV_BK - 1) / GV_BK;
    auto issue = [&](int tile) {
        if (tile < tiles) {
            T* ws = stages + (size_t)(tile % STAGES) * stage_elems;
            T* xs = ws + GV_ROWS * ROW;
            const int k0 = tile * GV_BK;
            for (int i = tid; i < (GV_ROWS + n) * CHUNKS; i += GV_ROWS * GV_SLOTS) {
                const int r = i / CHUNKS, k = k0 + (i % CHUNKS) * VEC;
                T* dst = (r < GV_ROWS ? ws + r * ROW : xs + (r - GV_ROWS) * ROW) + (i % CHUNKS) * VEC;
                const bool inside = k < in && (r >= GV_ROWS || m0 + r < out);      // in % VEC == 0: a chunk is inside the row or outside it
                if (inside) cp_async16(smem_u32(dst), r < GV_ROWS ? W + (size_t)(m0 + r) * in + k : x + (size_t)(r - GV_ROWS) * ldx + k);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        cp_async_commit();
    };
    pdl_wait();
    pdl_launch_dependents();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    for (int tile = 0; tile < tiles; ++tile) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                   // this tile has landed, and the stage refilled below is no longer read
        issue(tile + STAGES - 1);
        const T* ws = stages + (size_t)(tile % STAGES) * stage_elems + row * ROW;
        const T* xs = stages + (size_t)(tile % STAGES) * stage_elems + GV_ROWS * ROW;
        const int chunks = min(GV_BK, in - tile * GV_BK) / VEC;      // in % VEC == 0
        // 16 bytes of the row and of each token at a time (shared-memory reads, not arithmetic, bound this loop);
        // the k terms are still added one by one in ascending order.
#pragma unroll 2
        for (int c = 0; c < chunks; ++c) {
            Vec16<T> w;
            w.load(ws + c * VEC);
#pragma unroll
            for (int j = 0; j < TPT; ++j) {
                const int t = slot + j * GV_SLOTS;
                if (t < n) {
                    Vec16<T> xv;
                    xv.load(xs + t * ROW + c * VEC);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[j] = fmaf(xv.v[e], w.v[e], acc[j]);
                }
            }
        }
    }
    cp_async_wait<0>();
    const int c = m0 + row;
    if (c >= out) return;
#pragma unroll
    for (int j = 0; j < TPT; ++j) {
        const int t = slot + j * GV_SLOTS;
        if (t >= n) continue;
        float v = rnd<T>(acc[j]);
        if (epilogue == TI_EPI_XIELU) v = xielu_value<T>(v, act);
        if (epilogue == TI_EPI_F32_OUT) ((float*)y)[(size_t)t * ldy + c] = v;
        else ((T*)y)[(size_t)t * ldy + c] = from_f32<T>(v);
    }
}

template <typename T, int TPT, int STAGES>
static int launch_gemv_pipe(void* y, long long ldy, const T* x, long long ldx, const T* W, int n, int out, int in, int epilogue,
                            const XieluParams& act, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const size_t smem = (size_t)STAGES * (GV_ROWS + n) * (GV_BK + VEC) * sizeof(T);
    static size_t configured = 0;
    if (smem > configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_plain_pipe_kernel<T, TPT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(STAGES * (GV_ROWS + TPT * GV_SLOTS) * (GV_BK + VEC) * sizeof(T)));
        if (e != cudaSuccess) return ti_fail("gemv_plain: %s", cudaGetErrorString(e));
        configured = STAGES * (GV_ROWS + TPT * GV_SLOTS) * (GV_BK + VEC) * sizeof(T);
    }
    ti_launch(gemv_plain_pipe_kernel<T, TPT, STAGES>, dim3((out + GV_ROWS - 1) / GV_ROWS), dim3(GV_ROWS * GV_SLOTS), smem, stream, y, ldy, x, ldx, W, n,
              out, in, epilogue, act);
    return ti_check_launch("gemv_plain");
}

extern "C" int ti_gemm_plain(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in,
                             int epilogue, float alpha_p, float alpha_n, float beta, float eps, int dtype,
                             cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(n > 0 && out > 0 && in > 0, "gemm: bad sizes n=%d out=%d in=%d", n, out, in);
    TI_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
    dim3 grid((out + GP_BN - 1) / GP_BN, (n + GP_BM - 1) / GP_BM);
    TI_REQUIRE(grid.y <= 65535, "gemm: too many rows (%d) for one launch", n);
    XieluParams act{alpha_p, alpha_n, beta, eps};
    if (n <= GV_MAX_TOKENS) {                              // few tokens: the weight-streaming form (same sums, bit for bit)
        const int vec = dtype == TI_F32 ? 4 : 8;           // elements of a 16-byte chunk
        if (in % vec == 0 && ldx % vec == 0 && aligned16(x) && aligned16(W)) {
            TI_DISPATCH_DTYPE(dtype, {
                if (n <= GV_SLOTS) return launch_gemv_pipe<T, 1, 8>(y, ldy, (const T*)x, ldx, (const T*)W, n, out, in, epilogue, act, stream);
                if (n <= 2 * GV_SLOTS) return launch_gemv_pipe<T, 2, 6>(y, ldy, (const T*)x, ldx, (const T*)W, n, out, in, epilogue, act, stream);
                if (n <= 4 * GV_SLOTS) return launch_gemv_pipe<T, 4, 4>(y, ldy, (const T*)x, ldx, (const T*)W, n, out, in, epilogue, act, stream);
                return launch_gemv_pipe<T, 8, 3>(y, ldy, (const T*)x, ldx, (const T*)W, n, out, in, epilogue, act, stream);
            });
        }
        const size_t smem = (size_t)n * (GV_BK + 1) * sizeof(float);
        const dim3 blocks((out + GV_ROWS - 1) / GV_ROWS), threads(GV_ROWS * GV_SLOTS);
#define GV_LAUNCH(TPT) ti_launch(gemv_plain_kernel<T, TPT>, blocks, threads, smem, stream, y, ldy, (const T*)x, ldx, (const T*)W, n, out, in, epilogue, act)
        TI_DISPATCH_DTYPE(dtype, {
            if (n <= GV_SLOTS) GV_LAUNCH(1);
            else if (n <= 2 * GV_SLOTS) GV_LAUNCH(2);
            else if (n <= 4 * GV_SLOTS) GV_LAUNCH(4);
            else GV_LAUNCH(8);
        });
#undef GV_LAUNCH
        return ti_check_launch("gemv_plain");
    }
    const int vec_bytes = dtype == TI_F32 ? 16 : 8;     // four elements
    if (n > GB_T / 2 && in % 4 == 0 && ldx % 4 == 0 && ((uintptr_t)x % vec_bytes) == 0 && ((uintptr_t)W % vec_bytes) == 0) {
        dim3 wide((out + GB_T - 1) / GB_T, (n + GB_T - 1) / GB_T);
        TI_REQUIRE(wide.y <= 65535, "gemm: too many rows (%d) for one launch", n);
        TI_DISPATCH_DTYPE(dtype, (ti_launch(gemm_plain_wide_kernel<T>, dim3(wide), dim3(256), 0, stream, y, ldy, (const T*)x, ldx, (const T*)W, n,
                                            out, in, epilogue, act)));
        return ti_check_launch("gemm_plain_wide");
    }
    TI_DISPATCH_DTYPE(dtype, (ti_launch(gemm_plain_kernel<T>, dim3(grid), dim3(256), 0, stream, y, ldy, (const T*)x, ldx, (const T*)W, n, out, in,
                                                                          epilogue, act)));
    return ti_check_launch("gemm_plain");
}
