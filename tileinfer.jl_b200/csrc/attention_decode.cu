// Decode attention over the paged cache in bfloat16: one new token per sequence, a batch
// of sequences of any lengths, split over the keys (flash-decoding) so that the grid does
// not depend on the lengths and a captured step stays valid.
//
// Grid (split, kv head, sequence). A block walks its share of the sequence's pages; a page
// of one KV head is a dense [64, D] tile that is copied to shared memory with 16-byte
// cp.async in a 3-stage pipeline (XOR-swizzled against bank conflicts). The query heads
// that share the KV head are the 16 rows of the mma.sync tiles (GQA packing), so K and V
// are read once for the whole group. Each of the 4 warps takes 16 keys of a 64-key tile
// and keeps its own online-softmax state; the warps are merged in shared memory, the
// splits by a small combine kernel. Scores, softmax and accumulators are 32-bit, P is
// rounded to bfloat16 only as the operand of P·V, O is rounded once.
//
// AntoineBut/TileInfer.jl's counterpart: attention_decode_kernel + attention_combine_kernel
// (src/ops/tile/attention.jl:185-245), GQA-packed split-KV with a fixed split count, exp2
// with scale·log2e folded in (attention.jl:34-59), partial (acc, m, l) in a 32-bit workspace.
#include "common.cuh"
#include "decode_tile.cuh"

#define AD_MAX_SPLITS 64

template <int D> struct DecodeSmem {
    static constexpr int STAGES = D <= 128 ? 3 : 2;
    static constexpr int TILE = AD_PAGE * D;                 // elements of one K or V tile
    static constexpr size_t BYTES = (size_t)STAGES * 2 * TILE * sizeof(bf16);
};

template <int D>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src) {
    constexpr int CPR = D / 8;
    for (int c = threadIdx.x; c < AD_PAGE * CPR; c += AD_THREADS) {
        const int row = c / CPR, cc = c % CPR;
        cp_async16(smem_u32(dst + (row * CPR + swz<D>(row, cc)) * 8), src + (size_t)c * 8);
    }
}

template <int D, bool TABLE>
__global__ void __launch_bounds__(AD_THREADS) attention_decode_kernel(
    bf16* __restrict__ out, const bf16* q, const bf16* k_cache, const bf16* v_cache,
    const int* block_table, int table_stride, const int* seq_slots,
    const int* kv_lens, const int* work, float* __restrict__ ws_o, float* __restrict__ ws_ml, float scale_log2e, int nq,
    int nkv, int splits, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    typedef DecodeSmem<D> SM;
    constexpr int KS = D / 16, NT = D / 8;
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);

    // A block is one slot of the launch's B x splits: by default sequence b = slot / splits takes `splits`
    // equal parts of its keys; with a work table (slot -> sequence << 16 | part << 8 | parts, or -1 for a
    // slot without work; then the sequence's length) the slots are shared out by the host in proportion to
    // the sequences' lengths.
    int b, split, parts, kv_len, slot;
    // More than 16 query heads per KV head: blocks of 16 of them each (`slabs` per KV head), which read the keys again.
    const int full_group = nq / nkv, slabs = (full_group + 15) / 16;
    const int kvh = blockIdx.y / slabs, slab = blockIdx.y % slabs;
    if (TABLE) {                                             // one load: the slot's work and its sequence's length
        slot = blockIdx.x;
        const int2 w = __ldcg(reinterpret_cast<const int2*>(work) + slot);
        if (w.x < 0) return;
        b = w.x >> 16; split = (w.x >> 8) & 255; parts = w.x & 255;
        kv_len = w.y;
    } else {
        split = blockIdx.x; b = blockIdx.z; parts = splits; slot = b * splits + split;
        kv_len = __ldcg(kv_lens + b);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int group = min(16, full_group - slab * 16);            // this block's query heads
    // The step's lengths and block tables were uploaded before its first kernel, and every page but
    // the sequence's last one holds only older positions: their copies start BEFORE waiting for the
    // kernel that writes this step's key, value and query.
    const int first_key = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int t_begin = first_key / AD_PAGE, t_end = (kv_len + AD_PAGE - 1) / AD_PAGE;
    const int n_tiles = t_end - t_begin;
    const int my_lo = t_begin + (int)((long long)n_tiles * split / parts);
    const int my_hi = t_begin + (int)((long long)n_tiles * (split + 1) / parts);
    const int* table = block_table + (size_t)__ldcg(seq_slots + b) * table_stride;
    bool waited = false;

    auto issue = [&](int tile, int stage) {
        if (tile < my_hi) {
            if (tile == t_end - 1 && !waited) {              // the page that this step writes to
                pdl_wait();
                pdl_launch_dependents();
                waited = true;
            }
            const size_t base = ((size_t)__ldcg(table + tile) * nkv + kvh) * AD_PAGE * D;
            load_tile<D>(tiles + (size_t)stage * 2 * SM::TILE, k_cache + base);
            load_tile<D>(tiles + (size_t)stage * 2 * SM::TILE + SM::TILE, v_cache + base);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < SM::STAGES - 1; ++s) issue(my_lo + s, s);
    if (!waited) {
        pdl_wait();
        pdl_launch_dependents();
        waited = true;
    }

    // Query rows = the heads of this KV head's group, padded to 16.
    unsigned qf[KS][4];
    {
        const bf16* q0 = q + ((size_t)b * nq + (size_t)kvh * full_group + slab * 16) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = ks * 16 + 2 * t;
            qf[ks][0] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q0 + (size_t)g * D + d)) : 0u;
            qf[ks][1] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned*>(q0 + (size_t)(g + 8) * D + d)) : 0u;
            qf[ks][2] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q0 + (size_t)g * D + d + 8)) : 0u;
            qf[ks][3] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned*>(q0 + (size_t)(g + 8) * D + d + 8)) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;       // rows g and g + 8

    for (int tile = my_lo; tile < my_hi; ++tile) {
        const int stage = (tile - my_lo) % SM::STAGES;
        cp_async_wait<SM::STAGES - 2>();
        __syncthreads();
        // The stage freed by the previous iteration is refilled while this one is used.
        issue(tile + SM::STAGES - 1, (tile - my_lo + SM::STAGES - 1) % SM::STAGES);
        const bf16* kt = tiles + (size_t)stage * 2 * SM::TILE;
        const bf16* vt = kt + SM::TILE;

        decode_tile<D>(kt, vt, qf, o, m0, m1, l0, l1, tile, warp, lane, kv_len, first_key, scale_log2e);
    }
    cp_async_wait<0>();
    __syncthreads();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // Merge the warps: [warp][row 0..15][D + 2] floats in the (now idle) tile memory.
    float* mg = reinterpret_cast<float*>(smem_raw);
    constexpr int RS = D + 2;
    {
        float* mine = mg + (size_t)warp * 16 * RS;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            mine[g * RS + i * 8 + 2 * t] = o[i][0]; mine[g * RS + i * 8 + 2 * t + 1] = o[i][1];
            mine[(g + 8) * RS + i * 8 + 2 * t] = o[i][2]; mine[(g + 8) * RS + i * 8 + 2 * t + 1] = o[i][3];
        }
        if (t == 0) {
            mine[g * RS + D] = m0; mine[g * RS + D + 1] = l0;
            mine[(g + 8) * RS + D] = m1; mine[(g + 8) * RS + D + 1] = l1;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < group * D; e += AD_THREADS) {
        const int row = e / D, d = e % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row) * RS + D]);
        const float base = M == -INFINITY ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float* src = mg + ((size_t)w * 16 + row) * RS;
            const float f = exp2f(src[D] - base);
            L += src[D + 1] * f;
            O += src[d] * f;
        }
        const int head = kvh * full_group + slab * 16 + row;
        if (splits == 1) {
            out[((size_t)b * nq + head) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);   // a sequence without keys: zeros
        } else {
            const size_t idx = (size_t)(slot - split) * nq + (size_t)head * parts + split;   // a head's parts lie together
            ws_o[idx * D + d] = O;
            if (d == 0) { ws_ml[idx * 2] = M; ws_ml[idx * 2 + 1] = L; }
        }
    }
}

__global__ void attention_combine_kernel(bf16* __restrict__ out, const float* ws_o,
                                         const float* ws_ml, const int* seq_work, int D, int nq, int splits) {
    const size_t row = blockIdx.x;                          // (sequence, head)
    __shared__ float sm[AD_MAX_SPLITS], sl[AD_MAX_SPLITS], sw[AD_MAX_SPLITS];
    __shared__ float s_inv;
    // The parts of this (sequence, head) lie together: `splits` of them from row x splits on, or, with the
    // host's table (first slot << 8 | parts per sequence), `parts` from first slot x nq + head x parts on.
    size_t first = row * splits;
    int parts = splits;
    if (seq_work != nullptr) {
        const int b = (int)(row / nq), head = (int)(row % nq);
        const int w = __ldcg(seq_work + b);
        parts = w & 255;
        first = (size_t)(w >> 8) * nq + (size_t)head * parts;
    }
    const float* part_o = ws_o + first * D;
    const float* ml = ws_ml + first * 2;
    pdl_enter();
    // One round of loads: every thread's partial outputs (for up to 16 parts) are requested together
    // with the parts' (m, l), before anything is computed.
    const int d0 = threadIdx.x;
    float head_o[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) head_o[u] = (d0 < D && u < parts) ? __ldcg(part_o + (size_t)u * D + d0) : 0.f;
    for (int s = threadIdx.x; s < parts; s += blockDim.x) {
        sm[s] = __ldcg(ml + 2 * s);
        sl[s] = __ldcg(ml + 2 * s + 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float M = -INFINITY;
        for (int s = 0; s < parts; ++s) M = fmaxf(M, sm[s]);
        float L = 0.f;
        for (int s = 0; s < parts; ++s) {
            sw[s] = M == -INFINITY ? 0.f : exp2f(sm[s] - M);     // no part saw a key (a sequence of length 0): zeros, not 0/0
            L += sl[s] * sw[s];
        }
        s_inv = L > 0.f ? 1.0f / L : 0.f;
    }
    __syncthreads();
    const float inv = s_inv;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float O = 0.f;
        if (d == d0) {
#pragma unroll
            for (int u = 0; u < 16; ++u) O += (u < parts ? sw[u] : 0.f) * head_o[u];
        }
        for (int s0 = d == d0 ? 16 : 0; s0 < parts; s0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = s0 + u < parts ? __ldcg(part_o + (size_t)(s0 + u) * D + d) : 0.f;
#pragma unroll
            for (int u = 0; u < 8; ++u) O += (s0 + u < parts ? sw[s0 + u] : 0.f) * v[u];
        }
        out[row * D + d] = __float2bfloat16_rn(O * inv);
    }
}

template <int D>
static int launch_decode(bf16* out, const bf16* q, const bf16* k, const bf16* v, const int* table, int table_stride,
                         const int* seq_slots, const int* kv_lens, const int* work, const int* seq_work, float* ws_o, float* ws_ml,
                         float scale, int B, int nq, int nkv, int splits, int window, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = DecodeSmem<D>::BYTES > (size_t)AD_WARPS * 16 * (D + 2) * 4 ? DecodeSmem<D>::BYTES
                                                                                    : (size_t)AD_WARPS * 16 * (D + 2) * 4;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_decode_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ti_fail("attention_decode: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int slabs = (nq / nkv + 15) / 16;
    if (work != nullptr && splits > 1)
        ti_launch(attention_decode_kernel<D, true>, dim3(B * splits, nkv * slabs), dim3(AD_THREADS), smem, stream, out, q, k, v, table, table_stride,
                  seq_slots, kv_lens, work, ws_o, ws_ml, scale * 1.4426950408889634f, nq, nkv, splits, window);
    else
        ti_launch(attention_decode_kernel<D, false>, dim3(splits, nkv * slabs, B), dim3(AD_THREADS), smem, stream, out, q, k, v, table, table_stride,
                  seq_slots, kv_lens, work, ws_o, ws_ml, scale * 1.4426950408889634f, nq, nkv, splits, window);
    if (int rc = ti_check_launch("attention_decode")) return rc;
    if (splits > 1) {
        ti_launch(attention_combine_kernel, dim3(B * nq), dim3(D <= 64 ? 64 : 128), 0, stream, out, ws_o, ws_ml, seq_work, D, nq, splits);
        return ti_check_launch("attention_combine");
    }
    return 0;
}

// Returns 2 (and sets the error text) when the sizes are outside what this kernel takes, so
// that the caller can fall back to the plain kernel; 1 on a CUDA error.
// `work` and `seq_work` (both or neither): how the host shares the launch's B x splits slots out among
// the sequences, so that long sequences get more parts than short ones. work[slot] = (sequence << 16 |
// part << 8 | parts (at most 32), or -1 for a slot left without work; the sequence's length), 8-byte aligned
// pairs; seq_work[sequence] = first slot << 8 | parts; a sequence's slots are consecutive. Without them every sequence takes `splits` equal parts.
extern "C" int ti_attention_decode_shared(void* out, const void* q, const void* k_cache, const void* v_cache,
                                          const int* block_table, int table_stride, const int* seq_slots, const int* kv_lens,
                                          const int* work, const int* seq_work, float* ws_o, float* ws_ml, float scale, int B,
                                          int nq, int nkv, int D, int page_size, int splits, int window, cudaStream_t stream) {
    if (B == 0) return 0;
    if (page_size != AD_PAGE || nq % nkv != 0 || nq / nkv > 128 || D % 16 != 0 || B > 32767 || (long long)nkv * ((nq / nkv + 15) / 16) > 65535) {
        ti_fail("attention_decode takes page size %d, at most 128 query heads per KV head and head sizes in steps of 16; "
                "got page %d, %d/%d heads, head size %d", AD_PAGE, page_size, nq, nkv, D);
        return 2;
    }
    TI_REQUIRE(splits >= 1 && splits <= AD_MAX_SPLITS, "attention_decode: %d splits (1 to %d)", splits, AD_MAX_SPLITS);
    TI_REQUIRE(splits == 1 || (ws_o != nullptr && ws_ml != nullptr), "attention_decode: splits need a workspace");
    TI_REQUIRE((work == nullptr) == (seq_work == nullptr), "attention_decode: give both work tables or neither");
    if (splits == 1) work = seq_work = nullptr;
#define AD_CASE(d)                                                                                                     \
    case d:                                                                                                            \
        return launch_decode<d>((bf16*)out, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table,     \
                                table_stride, seq_slots, kv_lens, work, seq_work, ws_o, ws_ml, scale, B, nq, nkv, splits, window, stream);
    switch (D) {
        AD_CASE(16) AD_CASE(32) AD_CASE(48) AD_CASE(64) AD_CASE(80) AD_CASE(96) AD_CASE(112) AD_CASE(128) AD_CASE(256)
        default:
            ti_fail("attention_decode has no instance for head size %d", D);
            return 2;
    }
#undef AD_CASE
}

// Returns 2 (and sets the error text) when the sizes are outside what this kernel takes, so
// that the caller can fall back to the plain kernel; 1 on a CUDA error.
extern "C" int ti_attention_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                                   const int* block_table, int table_stride, const int* seq_slots, const int* kv_lens,
                                   float* ws_o, float* ws_ml, float scale, int B, int nq, int nkv, int D, int page_size,
                                   int splits, int window, cudaStream_t stream) {
    return ti_attention_decode_shared(out, q, k_cache, v_cache, block_table, table_stride, seq_slots, kv_lens, nullptr, nullptr, ws_o,
                                      ws_ml, scale, B, nq, nkv, D, page_size, splits, window, stream);
}

// ------------------------------------------------------------------------------------------------
// The same kernels with their work space inside the library: see attention_decode_noalloc.h.
#include "attention_decode_noalloc.h"

// File-scope device array. In host code this name is only a stand-in for the symbol, not a device
// address: the address each device gave it is looked up below and that pointer goes to the kernels.
static __device__ __align__(256) unsigned char ti_decode_noalloc_scratch[TI_DECODE_NOALLOC_SCRATCH_BYTES];

#define TI_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_scratch[TI_NOALLOC_MAX_DEVICES] = {nullptr};

extern "C" int ti_attention_decode_noalloc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                           const int* block_table, int table_stride, const int* seq_slots,
                                           const int* kv_lens, float scale, int B, int nq, int nkv, int D, int page_size,
                                           int splits, int window, cudaStream_t stream) {
    if (B == 0) return 0;
    TI_REQUIRE(B > 0 && nq > 0 && D > 0 && splits >= 1, "attention_decode_noalloc: bad sizes B=%d nq=%d D=%d splits=%d", B, nq, D, splits);
    const unsigned long long floats = splits > 1 ? (unsigned long long)B * nq * splits * (D + 2) : 0ull;
    TI_REQUIRE(floats * sizeof(float) <= TI_DECODE_NOALLOC_SCRATCH_BYTES,
               "attention_decode_noalloc: B=%d, %d heads, %d splits and head size %d need %llu bytes of work space; the "
               "built-in array holds %u", B, nq, splits, D, floats * (unsigned long long)sizeof(float), TI_DECODE_NOALLOC_SCRATCH_BYTES);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ti_fail("attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    TI_REQUIRE(dev >= 0 && dev < TI_NOALLOC_MAX_DEVICES, "attention_decode_noalloc: device %d is beyond the %d this build tracks", dev, TI_NOALLOC_MAX_DEVICES);
    if (g_noalloc_scratch[dev] == nullptr) {
        // Once per device, with that device current: the array's address on THIS device.
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, ti_decode_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return ti_fail("attention_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_noalloc_scratch[dev] = static_cast<float*>(ptr);
    }
    float* ws_o = g_noalloc_scratch[dev];                       // [B, nq, splits, D]
    float* ws_ml = ws_o + (size_t)B * nq * splits * D;          // [B, nq, splits, 2]
    return ti_attention_decode(out, q, k_cache, v_cache, block_table, table_stride, seq_slots, kv_lens, ws_o, ws_ml, scale,
                               B, nq, nkv, D, page_size, splits, window, stream);
}
