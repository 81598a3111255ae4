// Random weights on the device: value = f(seed, tensor name, element index).
//
// A counter-based generator: element i of a tensor is a pure function of two 32-bit keys (derived on
// the host from the seed and a hash of the tensor's name) and of i, so any part of any tensor can be
// made anywhere, in any order, and the host's restatement of the same function (weights/random_init.py,
// in numpy) gives the same bits. The integer mix is the lowbias32 function that AntoineBut/TileInfer.jl
// uses for its sampling uniforms (src/engine/sampler.jl:34-47); the reference has no random-weights
// mode of its own (its only random model is made in Python for fixtures,
// scripts/gen_apertus_fixtures.py:80-96).
//
// z ~ N(0, 1) by Box-Muller from two 24-bit uniforms. To be bit-identical on every machine, the
// logarithm and the cosine are NOT library calls: they are fixed sequences of IEEE 32-bit additions,
// multiplications, one division and one square root, each rounded to nearest (the _rn intrinsics keep
// the compiler from fusing a product and a sum), which every conforming implementation evaluates alike:
//   a = mix32(k0 ^ i) >> 8, b = mix32(k1 ^ i) >> 8
//   n = a + 1 in [1, 2^24] = m 2^e, m in (sqrt(1/2), sqrt(2)];  ln(n 2^-24) = (e - 24) ln2 + 2 atanh(s),
//       s = (m - 1)/(m + 1), atanh by its odd series up to s^9 (|s| < 0.1716: below 1e-9 of s)
//   r = sqrt(-2 ln u);  the angle 2 pi b 2^-24 is cut into octants on the integer b, and the sine or the
//       cosine of (pi/4) g, g in [0, 1], comes from its Taylor series up to x^9 / x^10
//   value = mean + (r c) std, rounded once to the element type.
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned mix32(unsigned x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ float standard_normal(unsigned k0, unsigned k1, unsigned i) {
    const unsigned a = mix32(k0 ^ i) >> 8, b = mix32(k1 ^ i) >> 8;
    // ln u, u = (a + 1) 2^-24 in (0, 1]
    const unsigned bits = __float_as_uint((float)(a + 1u));            // exact: a + 1 <= 2^24
    int e = (int)(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x7fffffu) | 0x3f800000u);       // [1, 2)
    if (m > 0x1.6a09e6p+0f /* sqrt 2 */) { m = mul(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(add(m, -1.0f), add(m, 1.0f));
    const float s2 = mul(s, s);
    float p = 0x1.c71c72p-3f;                                          // 2/9
    p = add(mul(p, s2), 0x1.24924ap-2f);                               // 2/7
    p = add(mul(p, s2), 0x1.99999ap-2f);                               // 2/5
    p = add(mul(p, s2), 0x1.555556p-1f);                               // 2/3
    p = add(mul(p, s2), 2.0f);
    const float ln_u = add(mul((float)(e - 24), 0x1.62e43p-1f /* ln 2 */), mul(s, p));
    const float r = __fsqrt_rn(mul(-2.0f, ln_u));
    // cos(2 pi b 2^-24)
    const unsigned q = b >> 21;
    const float f = mul((float)(b & 0x1fffffu), 0x1p-21f);             // exact
    const float g = (q & 1u) ? add(1.0f, -f) : f;
    const float x = mul(g, 0x1.921fb6p-1f);                            // pi/4
    const float x2 = mul(x, x);
    float c;
    if (((q + 1u) >> 1) & 1u) {                                        // octants 1, 2, 5, 6: a sine
        float t = 0x1.71de3ap-19f;                                     // 1/9!
        t = add(mul(t, x2), -0x1.a01a02p-13f);                         // -1/7!
        t = add(mul(t, x2), 0x1.111112p-7f);                           // 1/5!
        t = add(mul(t, x2), -0x1.555556p-3f);                          // -1/3!
        t = add(mul(t, x2), 1.0f);
        c = mul(x, t);
    } else {
        float t = -0x1.27e4fcp-22f;                                    // -1/10!
        t = add(mul(t, x2), 0x1.a01a02p-16f);                          // 1/8!
        t = add(mul(t, x2), -0x1.6c16c2p-10f);                         // -1/6!
        t = add(mul(t, x2), 0x1.555556p-5f);                           // 1/4!
        t = add(mul(t, x2), -0.5f);
        c = add(mul(t, x2), 1.0f);
    }
    if (q >= 2u && q <= 5u) c = -c;
    return mul(r, c);
}

template <typename T>
__global__ void random_normal_kernel(T* out, size_t count, unsigned first, unsigned k0, unsigned k1, float mean, float std) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(add(mean, mul(standard_normal(k0, k1, first + (unsigned)i), std)));
}

}  // namespace

// out[j] = mean + std * z(first + j) for j < count, rounded to the element type. `first + count` must
// not pass 2^32 (a tensor of more elements than that is refused by the caller).
extern "C" int ti_random_normal(void* out, int dtype, long long count, long long first, unsigned k0, unsigned k1, float mean,
                                float std, cudaStream_t stream) {
    if (count == 0) return 0;
    TI_REQUIRE(count > 0 && first >= 0 && first + count <= (1ll << 32),
               "random_normal: elements %lld..%lld are outside the 32-bit counter", first, first + count);
    long long blocks = (count + 255) / 256;
    if (blocks > ti_sm_count() * 64) blocks = ti_sm_count() * 64;
    TI_DISPATCH_DTYPE(dtype, {
        ti_launch(random_normal_kernel<T>, dim3((int)blocks), dim3(256), 0, stream, (T*)out, (size_t)count, (unsigned)first, k0, k1,
                  mean, std);
    });
    return ti_check_launch("random_normal");
}
