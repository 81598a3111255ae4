// Shared by every kernel file: element types, conversions, reductions, error reporting.
//
// All entry points are extern "C", take raw device pointers and a stream, allocate
// nothing, and return 0 on success. On a refused size or a CUDA error they return non-zero
// and ti_last_error() gives the text. Element types are passed as TI_F32 / TI_BF16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define TI_F32 0
#define TI_BF16 1

typedef __nv_bfloat16 bf16;

extern "C" const char* ti_last_error();
int ti_fail(const char* fmt, ...);
int ti_check_launch(const char* what);
extern "C" int ti_sm_count();

// Programmatic dependent launch. Every kernel of a step lets its successor start launching at
// once (`pdl_launch_dependents`) and waits for its predecessor's results only where it first
// needs them (`pdl_wait`): the successor's blocks come up, and prefetch what does not depend on
// the predecessor (weights), while the predecessor's last blocks drain. Both are no-ops for a
// kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Inputs that another kernel of the same step writes (activations, step metadata, the cache, work
// spaces) are never declared `const __restrict__`: that would let the compiler read them through the
// non-coherent path, which requires the data to be read-only for the kernel's whole lifetime, and a
// kernel launched as a programmatic dependent starts before its predecessor has finished writing.
extern int ti_pdl_enabled;

// Wait for the predecessor, then let the successor start: at most two kernels overlap. (Releasing the
// successor before waiting, so that more kernels are resident at once, was measured on the decode
// step and was slower: blocks that sit waiting take residency away from the kernel that is running.)
__device__ __forceinline__ void pdl_enter() {
    pdl_wait();
    pdl_launch_dependents();
}

// Launch with the programmatic-stream-serialization attribute when enabled.
template <typename... KArgs, typename... Args>
inline cudaError_t ti_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ti_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define TI_REQUIRE(cond, ...)                \
    do {                                     \
        if (!(cond)) return ti_fail(__VA_ARGS__); \
    } while (0)

// ---- conversions: every kernel computes in float and rounds once on store ---------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }
// Round to the storage type and come back: the rounding points of the bfloat16 path.
template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f32(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds
// 33 floats of shared memory. The order of the additions is fixed by the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// xIELU with the reference's rounding points (src/ops/reference.jl:49-56):
//   bx = rnd(beta x); x > 0: rnd(rnd(rnd(ap x) x) + bx); else rnd(rnd(rnd(rnd(expm1(min(x,eps))) - x) an) + bx)
struct XieluParams {
    float alpha_p, alpha_n, beta, eps;
};
template <typename T> __device__ __forceinline__ float xielu_value(float x, const XieluParams& a) {
    const float bx = rnd<T>(a.beta * x);
    const float pos = rnd<T>(rnd<T>(rnd<T>(a.alpha_p * x) * x) + bx);
    const float e = rnd<T>(expm1f(fminf(x, a.eps)));
    const float neg = rnd<T>(rnd<T>(rnd<T>(e - x) * a.alpha_n) + bx);
    return x > 0.f ? pos : neg;                // both sides are computed: no branch, elements interleave
}

// Two bfloat16 elements at once in packed bfloat16 arithmetic: a packed product or sum rounds its exact
// result once, which is what rnd(a * b) and rnd(a + b) of bfloat16 values give (their exact result
// fits 32-bit arithmetic whenever it is within reach of a rounding tie), at half the instructions.
// The _rn forms keep the compiler from contracting a product and a sum into one fused operation.
// s0, s1 are unrounded sums; the results are bfloat16 bits in the low halves of lo and hi.
struct XieluPacked {
    __nv_bfloat162 alpha_p, alpha_n, beta;
    float eps;
};
__device__ __forceinline__ XieluPacked xielu_pack(const XieluParams& a) {
    return XieluPacked{__float2bfloat162_rn(a.alpha_p), __float2bfloat162_rn(a.alpha_n), __float2bfloat162_rn(a.beta), a.eps};
}
__device__ __forceinline__ void xielu_bf16_pair(float s0, float s1, const XieluPacked& a, unsigned& lo, unsigned& hi) {
    const __nv_bfloat162 x = __floats2bfloat162_rn(s0, s1);
    const __nv_bfloat162 bx = __hmul2_rn(a.beta, x);
    const __nv_bfloat162 pos = __hadd2_rn(__hmul2_rn(__hmul2_rn(a.alpha_p, x), x), bx);
    const float x0 = __low2float(x), x1 = __high2float(x);
    const __nv_bfloat162 e = __floats2bfloat162_rn(expm1f(fminf(x0, a.eps)), expm1f(fminf(x1, a.eps)));
    const __nv_bfloat162 neg = __hadd2_rn(__hmul2_rn(__hsub2_rn(e, x), a.alpha_n), bx);
    const unsigned P = *reinterpret_cast<const unsigned*>(&pos), N = *reinterpret_cast<const unsigned*>(&neg);
    lo = (x0 > 0.f ? P : N) & 0xffffu;
    hi = (x1 > 0.f ? P : N) >> 16;
}

// 16 bytes of elements, widened to float on load and rounded once on store.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float v[4];
    __device__ __forceinline__ void load(const float* p) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    // Through L2, never from a line that L1 may still hold from before another kernel wrote it.
    __device__ __forceinline__ void load_cg(const float* p) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    float v[8];
    __device__ __forceinline__ void unpack(const uint4& t) {
        const unsigned w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ void load(const bf16* p) { unpack(*reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void load_cg(const bf16* p) { unpack(__ldcg(reinterpret_cast<const uint4*>(p))); }
    __device__ __forceinline__ void store(bf16* p) const {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
__host__ __forceinline__ bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

#define TI_DISPATCH_DTYPE(dtype, ...)                                   \
    do {                                                                \
        if ((dtype) == TI_F32) { typedef float T; __VA_ARGS__; }        \
        else if ((dtype) == TI_BF16) { typedef bf16 T; __VA_ARGS__; }   \
        else return ti_fail("unknown element type code %d", (int)(dtype)); \
    } while (0)
