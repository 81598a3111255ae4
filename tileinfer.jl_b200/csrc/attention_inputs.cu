// Fused attention inputs: per-head RMSNorm of q and k, rotary embedding, q written out, k
// and v written to their place in the paged cache. One warp per (token, head).
//
// AntoineBut/TileInfer.jl: the norm over head_dim comes before the rotation and v is left
// untouched (src/ops/interface.jl:161-177, src/ops/tile/fused.jl:20-33, 61-66); the rotation
// pairs element i with i + D/2 and rounds each product and the sum
// (src/ops/reference.jl:32-39); slot (page, offset) of the pool [pages][kv_heads][P][D]
// (src/kv/paged_cache.jl:1-4). Beyond what the reference has, the rotation may cover only the first
// `rotary` elements of a head (the rest pass through) and may pair element 2i with 2i + 1 instead
// (`interleaved`); the table holds (cos, sin) of rotary / 2 pairs per position.
#include "common.cuh"

#include <type_traits>

#define AI_WARPS 4
#define AI_MAX_D 512

template <typename T>
__global__ void attention_inputs_kernel(const T* qkv, long long qkv_stride, const float* partials, int n_partials,
                                        long long partial_stride, T* __restrict__ q_out,
                                        T* __restrict__ k_cache, T* __restrict__ v_cache,
                                        const T* __restrict__ q_norm_w, const T* __restrict__ k_norm_w, float eps,
                                        const float* __restrict__ cos_sin, int rotary, int interleaved,
                                        const int* positions, const int* slots, int nq, int nkv, int D,
                                        int page_size, int write_kv) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int head = blockIdx.y * AI_WARPS + warp;
    // Positions and slots were uploaded before the step's first kernel: they, and the rotation table's
    // row they select, are read before waiting for the projection that produces qkv.
    const int slot_t = slots != nullptr ? __ldcg(slots + t) : 0;
    const int pos_t = __ldcg(positions + t);
    pdl_enter();
    if (head >= heads_total) return;
    float* buf = smem + warp * D;

    // The projection's output row: stored, or the sum (in split order, rounded once like any product)
    // of the 32-bit partial sums [s][token][feature] of a product that was split over k.
    const T* src = qkv != nullptr ? qkv + (size_t)t * qkv_stride + (size_t)head * D : nullptr;
    const float* psrc = partials != nullptr ? partials + (size_t)t * qkv_stride + (size_t)head * D : nullptr;
    auto value = [&](int d) -> float {
        if (psrc == nullptr) return to_f32(__ldcg(src + d));
        float v = __ldcg(psrc + d);
        for (int s = 1; s < n_partials; ++s) v += __ldcg(psrc + (size_t)s * partial_stride + d);
        return rnd<T>(v);
    };
    const bool is_q = head < nq;
    const bool is_k = !is_q && head < nq + nkv;
    const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);

    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * nq + head) * D;
    } else {
        const int slot = slot_t;
        const int page = slot / page_size, off = slot - page * page_size;
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * nkv + kvh) * page_size + off) * D;
    }
    if (!is_q && !is_k) {                    // value head: a copy
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(value(d));
        return;
    }
    const T* nw = is_q ? q_norm_w : k_norm_w;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float v = value(d);
        buf[d] = v;
        ss = fmaf(v, v, ss);
    }
    if (nw != nullptr) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) buf[d] = rnd<T>(to_f32(nw[d]) * rnd<T>(buf[d] * inv));
    }
    __syncwarp();
    if (cos_sin == nullptr) {
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(buf[d]);
        return;
    }
    const int half = rotary >> 1;
    const float* cs = cos_sin + (size_t)pos_t * rotary;     // [half][2] = (cos, sin)
    for (int d = lane; d < D; d += 32) {
        if (d >= rotary) {                                   // beyond the rotated part: unchanged
            dst[d] = from_f32<T>(buf[d]);
            continue;
        }
        int i;
        float rot;
        if (interleaved) {
            i = d >> 1;
            rot = (d & 1) ? buf[d - 1] : -buf[d + 1];
        } else {
            i = d < half ? d : d - half;
            rot = d < half ? -buf[d + half] : buf[d - half];
        }
        const float c = cs[2 * i], s = cs[2 * i + 1];
        dst[d] = from_f32<T>(rnd<T>(buf[d] * c) + rnd<T>(rot * s));
    }
}

// The same for head sizes 64 and 128 in bfloat16: a lane owns VPL = D/32
// consecutive elements (one 4- or 8-byte access), the rotation partner i +- D/2 lives in lane +- 16 and
// comes by shuffle, so no shared memory and no strided loops are needed.
//
// With several heads per warp (a prompt's step) the kernel is bound by how many loads are in flight, so it is held to
// 64 registers for eight blocks per SM (21.5 against 24.8 us for 2,048 tokens of 32 + 8 + 8 heads of 128).
template <int VPL, int HPW>
__global__ void __launch_bounds__(AI_WARPS * 32, HPW >= 4 ? 8 : 1)
attention_inputs_vec_kernel(const bf16* qkv, long long qkv_stride, const float* partials, int n_partials,
                                            long long partial_stride, bf16* __restrict__ q_out,
                                            bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                            const bf16* __restrict__ q_norm_w, const bf16* __restrict__ k_norm_w, float eps,
                                            const float* __restrict__ cos_sin, const int* positions, const int* slots,
                                            int nq, int nkv, int page_size, int write_kv) {
    // A warp takes HPW consecutive heads of one token, with all its loads in flight at once and the
    // token's rotation row read once: a step of many tokens is bound by memory traffic, and the rotation
    // row (as long as four heads) would otherwise be read again for every head.
    constexpr int D = 32 * VPL;
    typedef typename std::conditional<VPL == 4, uint2, unsigned>::type Pack;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int head0 = (blockIdx.y * AI_WARPS + warp) * HPW;
    const int slot_t = slots != nullptr ? __ldcg(slots + t) : 0;
    const int pos_t = __ldcg(positions + t);
    float2 cs[VPL];
    if (cos_sin != nullptr) {
        const float2* row = reinterpret_cast<const float2*>(cos_sin + (size_t)pos_t * D) + (lane & 15) * VPL;
#pragma unroll
        for (int e = 0; e < VPL; ++e) cs[e] = row[e];
    }
    pdl_enter();
    if (head0 >= heads_total) return;
    Pack raw[HPW];
    if (partials == nullptr) {
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int head = min(head0 + i, heads_total - 1);
            raw[i] = __ldcg(reinterpret_cast<const Pack*>(qkv + (size_t)t * qkv_stride + (size_t)head * D) + lane);
        }
    } else {
        // The projection was split over k: its 32-bit partial sums [s][token][feature] are added in split
        // order and rounded once, like any product (eight splits' loads in flight at a time).
        typedef typename std::conditional<VPL == 4, float4, float2>::type PackF;
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int head = min(head0 + i, heads_total - 1);
            const float* ps = partials + (size_t)t * qkv_stride + (size_t)head * D + lane * VPL;
            float acc[VPL];
#pragma unroll
            for (int e = 0; e < VPL; ++e) acc[e] = 0.f;
            for (int s0 = 0; s0 < n_partials; s0 += 8) {
                PackF part[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (s0 + u < n_partials) part[u] = __ldcg(reinterpret_cast<const PackF*>(ps + (size_t)(s0 + u) * partial_stride));
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (s0 + u < n_partials) {
                        const float* f = reinterpret_cast<const float*>(&part[u]);
#pragma unroll
                        for (int e = 0; e < VPL; ++e) acc[e] = (s0 + u == 0) ? f[e] : acc[e] + f[e];
                    }
            }
            unsigned* w = reinterpret_cast<unsigned*>(&raw[i]);
#pragma unroll
            for (int e = 0; e < VPL / 2; ++e) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
                w[e] = *reinterpret_cast<const unsigned*>(&h2);
            }
        }
    }
    const int page = slot_t / page_size, off = slot_t - page * page_size;
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int head = head0 + i;
        if (head >= heads_total) break;
        const bool is_q = head < nq;
        const bool is_k = !is_q && head < nq + nkv;
        const int kvh = is_q ? 0 : (is_k ? head - nq : head - nq - nkv);
        bf16* dst = is_q ? q_out + ((size_t)t * nq + head) * D
                         : (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * D;
        if (!is_q && !is_k) {                    // value head: a copy
            reinterpret_cast<Pack*>(dst)[lane] = raw[i];
            continue;
        }
        float v[VPL];
        {
            const unsigned* w = reinterpret_cast<const unsigned*>(&raw[i]);
#pragma unroll
            for (int e = 0; e < VPL / 2; ++e) {
                v[2 * e] = __uint_as_float(w[e] << 16);
                v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
            }
        }
        const bf16* nw = is_q ? q_norm_w : k_norm_w;
        if (nw != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < VPL; ++e) ss = fmaf(v[e], v[e], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)D + eps);
            const Pack wraw = reinterpret_cast<const Pack*>(nw)[lane];
            const unsigned* w = reinterpret_cast<const unsigned*>(&wraw);
#pragma unroll
            for (int e = 0; e < VPL / 2; ++e) {
                v[2 * e] = rnd<bf16>(__uint_as_float(w[e] << 16) * rnd<bf16>(v[2 * e] * inv));
                v[2 * e + 1] = rnd<bf16>(__uint_as_float(w[e] & 0xffff0000u) * rnd<bf16>(v[2 * e + 1] * inv));
            }
        }
        if (cos_sin != nullptr) {
#pragma unroll
            for (int e = 0; e < VPL; ++e) {
                const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
                const float rot = lane < 16 ? -other : other;
                v[e] = rnd<bf16>(v[e] * cs[e].x) + rnd<bf16>(rot * cs[e].y);
            }
        }
        Pack outp;
        unsigned* o = reinterpret_cast<unsigned*>(&outp);
#pragma unroll
        for (int e = 0; e < VPL / 2; ++e) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            o[e] = *reinterpret_cast<const unsigned*>(&h);
        }
        reinterpret_cast<Pack*>(dst)[lane] = outp;
    }
}

extern "C" int ti_attention_inputs(const void* qkv, long long qkv_stride, const float* partials, int n_partials,
                                   long long partial_stride, void* q_out, void* k_cache, void* v_cache,
                                   const void* q_norm_w, const void* k_norm_w, float eps, const float* cos_sin,
                                   int rotary, int interleaved, const int* positions, const int* slots, int n_tokens,
                                   int nq, int nkv, int D, int page_size, int write_kv, int dtype, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    TI_REQUIRE(D > 0 && D % 2 == 0 && D <= AI_MAX_D, "attention_inputs: head_dim %d must be even and at most %d", D, AI_MAX_D);
    TI_REQUIRE((qkv != nullptr) != (partials != nullptr), "attention_inputs: give the projection's output or its partial sums");
    TI_REQUIRE(nq > 0 && nkv > 0 && page_size > 0, "attention_inputs: bad sizes nq=%d nkv=%d page=%d", nq, nkv, page_size);
    TI_REQUIRE(cos_sin == nullptr || (rotary >= 2 && rotary % 2 == 0 && rotary <= D),
               "attention_inputs: a rotation over %d of %d elements (it must be even, from 2 to the head size)", rotary, D);
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    dim3 grid(n_tokens, (heads_total + AI_WARPS - 1) / AI_WARPS);
    const size_t smem = (size_t)AI_WARPS * D * sizeof(float);
    // The vector kernel rotates the whole head with rotate-half pairing (the partner sits 16 lanes away).
    const bool plain_rotation = cos_sin == nullptr || (rotary == D && !interleaved);
    if (dtype == TI_BF16 && plain_rotation && (D == 64 || D == 128) && qkv_stride % 4 == 0 && aligned16(q_out) &&
        (qkv != nullptr ? aligned16(qkv) : (aligned16(partials) && partial_stride % 4 == 0)) &&
        (!write_kv || (aligned16(k_cache) && aligned16(v_cache))) && (q_norm_w == nullptr || aligned16(q_norm_w)) &&
        (k_norm_w == nullptr || aligned16(k_norm_w)) && (cos_sin == nullptr || aligned16(cos_sin))) {
#define AI_VEC_LAUNCH(VPL, HPW)                                                                                                     \
    ti_launch(attention_inputs_vec_kernel<VPL, HPW>, dim3(n_tokens, ((heads_total + HPW - 1) / HPW + AI_WARPS - 1) / AI_WARPS),         \
              dim3(AI_WARPS * 32), 0, stream, (const bf16*)qkv, qkv_stride, partials, n_partials, partial_stride, (bf16*)q_out,       \
              (bf16*)k_cache, (bf16*)v_cache,                                                                                             \
              (const bf16*)q_norm_w, (const bf16*)k_norm_w, eps, cos_sin, positions, slots, nq, nkv, page_size, write_kv)
        // Few tokens: one head per warp (latency counts); many: four heads per warp (memory traffic counts).
        // Partial sums (steps of up to 256 tokens) always one head per warp: the loop over the slices of one head
        // cannot be overlapped with the next head's, so four heads would be four rounds of loads.
        const bool one_head = n_tokens <= 64 || partials != nullptr;
        if (D == 128) { if (one_head) AI_VEC_LAUNCH(4, 1); else AI_VEC_LAUNCH(4, 4); }
        else          { if (one_head) AI_VEC_LAUNCH(2, 1); else AI_VEC_LAUNCH(2, 4); }
#undef AI_VEC_LAUNCH
        return ti_check_launch("attention_inputs");
    }
    TI_DISPATCH_DTYPE(dtype, (ti_launch(attention_inputs_kernel<T>, dim3(grid), dim3(AI_WARPS * 32), smem, stream, 
                                 (const T*)qkv, qkv_stride, partials, n_partials, partial_stride, (T*)q_out, (T*)k_cache, (T*)v_cache, (const T*)q_norm_w,
                                 (const T*)k_norm_w, eps, cos_sin, rotary, interleaved, positions, slots, nq, nkv, D, page_size, write_kv)));
    return ti_check_launch("attention_inputs");
}
