// Causal flash attention over the paged cache in bfloat16 for steps with several tokens per
// sequence (prefill, chunks of a prefill, continuation from cached positions), for a batch
// of sequences of unequal lengths.
//
// A block owns up to 128 rows = consecutive query tokens of ONE sequence × the query heads
// of ONE KV head (GQA packing: the K/V tile is read once for the whole group). It walks the
// sequence's pages from the first visible key to the last query's position; a page of one
// KV head, a dense [64, D] tile, is copied with 16-byte cp.async into XOR-swizzled shared
// memory in a multi-stage pipeline shared by the block's 8 warps. Each warp holds 16 rows:
// S = QKᵀ and O += P·V run on mma.sync m16n8k16 with ldmatrix operands, the online softmax
// (exp2 with scale·log2e folded in) and the accumulators stay in 32-bit registers, P is
// rounded to bfloat16 only as the operand of P·V, O is rounded once. Only tiles that cross
// a row's causal border (or the window's) are masked element by element.
//
// The grid's x runs over (sequence, query tile) pairs; a block finds its pair by walking the
// step's cu_seqlens, so no per-tile table has to be uploaded.
//
// AntoineBut/TileInfer.jl's counterpart: attention_prefill_kernel (src/ops/tile/attention.jl:
// 34-59, 130-177): FlashAttention-2 over the paged cache, one 64-key page per loop step,
// masking only the diagonal pages, for one sequence; the batch and the GQA packing of rows
// are this library's own.
#include "common.cuh"
#include "mma_util.cuh"

#define PF_PAGE 64
#define PF_WARPS 8
#define PF_THREADS (PF_WARPS * 32)
#define PF_ROWS (PF_WARPS * 16)

template <int D> struct PrefillSmem {
    static constexpr int STAGES = D <= 64 ? 4 : D <= 128 ? 3 : 2;
    static constexpr int TILE = PF_PAGE * D;
    static constexpr size_t BYTES = (size_t)STAGES * 2 * TILE * sizeof(bf16);
};

template <int D>
__device__ __forceinline__ void pf_load_tile(bf16* dst, const bf16* src) {
    constexpr int CPR = D / 8;
    for (int c = threadIdx.x; c < PF_PAGE * CPR; c += PF_THREADS) {
        const int row = c / CPR, cc = c % CPR;
        cp_async16(smem_u32(dst + (row * CPR + swz<D>(row, cc)) * 8), src + (size_t)c * 8);
    }
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 1) attention_prefill_kernel(
    bf16* __restrict__ out, const bf16* q, const bf16* k_cache, const bf16* v_cache,
    const int* block_table, int table_stride, const int* seq_slots,
    const int* cu_seqlens, const int* kv_lens, int n_seqs, float scale_log2e, int nq, int nkv,
    int tokens_per_tile, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    typedef PrefillSmem<D> SM;
    constexpr int CPR = D / 8, KS = D / 16, NT = D / 8;
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.y;
    const int group = nq / nkv;

    pdl_wait();
    pdl_launch_dependents();
    // Which (sequence, query tile) is this block's?
    int b = 0, tile_in_seq = blockIdx.x;
    for (; b < n_seqs; ++b) {
        const int tiles_b = (__ldcg(cu_seqlens + b + 1) - __ldcg(cu_seqlens + b) + tokens_per_tile - 1) / tokens_per_tile;
        if (tile_in_seq < tiles_b) break;
        tile_in_seq -= tiles_b;
    }
    if (b >= n_seqs) return;
    const int q_begin = __ldcg(cu_seqlens + b), q_len = __ldcg(cu_seqlens + b + 1) - q_begin;
    const int kv_len = __ldcg(kv_lens + b);
    const int start = kv_len - q_len;                        // position of the sequence's first token in this step
    const int j0 = tile_in_seq * tokens_per_tile;
    const int n_tok = min(tokens_per_tile, q_len - j0);
    const int* table = block_table + (size_t)__ldcg(seq_slots + b) * table_stride;

    // This thread's two rows (r0, r0 + 8): token and head inside the tile, and the position.
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int tok0 = r0 / group, tok1 = r1 / group;
    const bool live0 = tok0 < n_tok, live1 = tok1 < n_tok;
    const int pos0 = live0 ? start + j0 + tok0 : -1, pos1 = live1 ? start + j0 + tok1 : -1;
    const int lo0 = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int lo1 = (window > 0 && pos1 + 1 > window) ? pos1 + 1 - window : 0;

    unsigned qf[KS][4];
    {
        const bf16* qa = q + ((size_t)(q_begin + j0 + (live0 ? tok0 : 0)) * nq + (size_t)kvh * group + r0 % group) * D;
        const bf16* qb = q + ((size_t)(q_begin + j0 + (live1 ? tok1 : 0)) * nq + (size_t)kvh * group + r1 % group) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = ks * 16 + 2 * t;
            qf[ks][0] = live0 ? __ldcg(reinterpret_cast<const unsigned*>(qa + d)) : 0u;
            qf[ks][1] = live1 ? __ldcg(reinterpret_cast<const unsigned*>(qb + d)) : 0u;
            qf[ks][2] = live0 ? __ldcg(reinterpret_cast<const unsigned*>(qa + d + 8)) : 0u;
            qf[ks][3] = live1 ? __ldcg(reinterpret_cast<const unsigned*>(qb + d + 8)) : 0u;
        }
    }
    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // Keys [key_lo, key_hi) are visible to some row of the block.
    const int pos_first = start + j0, pos_last = start + j0 + n_tok - 1;
    const int key_lo = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;
    const int t_lo = key_lo / PF_PAGE, t_hi = pos_last / PF_PAGE + 1;

    auto issue = [&](int tile, int stage) {
        if (tile < t_hi) {
            const size_t base = ((size_t)__ldcg(table + tile) * nkv + kvh) * PF_PAGE * D;
            pf_load_tile<D>(tiles + (size_t)stage * 2 * SM::TILE, k_cache + base);
            pf_load_tile<D>(tiles + (size_t)stage * 2 * SM::TILE + SM::TILE, v_cache + base);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < SM::STAGES - 1; ++s) issue(t_lo + s, s);

    for (int tile = t_lo; tile < t_hi; ++tile) {
        const int stage = (tile - t_lo) % SM::STAGES;
        cp_async_wait<SM::STAGES - 2>();
        __syncthreads();
        issue(tile + SM::STAGES - 1, (tile - t_lo + SM::STAGES - 1) % SM::STAGES);
        const bf16* kt = tiles + (size_t)stage * 2 * SM::TILE;
        const bf16* vt = kt + SM::TILE;

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        {
            const int mat = lane >> 3, r = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {             // pairs of 8-key tiles
                    const int row = np * 16 + (mat >> 1) * 8 + r;
                    unsigned kb[4];
                    ldmatrix_x4(kb, smem_u32(kt + (row * CPR + swz<D>(row, 2 * ks + (mat & 1))) * 8));
                    mma16816(s[2 * np], qf[ks], kb[0], kb[1]);
                    mma16816(s[2 * np + 1], qf[ks], kb[2], kb[3]);
                }
            }
        }
        const int key_base = tile * PF_PAGE;
        // Element-wise masking only where some row of the block has its border inside the tile.
        const bool need_mask = key_base + PF_PAGE - 1 > pos_first || key_base < key_lo + (window > 0 ? n_tok : 0) ||
                               n_tok * group < PF_ROWS;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = key_base + 8 * nt + 2 * t + j;
                float a = s[nt][j] * scale_log2e, c = s[nt][2 + j] * scale_log2e;
                if (need_mask) {
                    if (key > pos0 || key < lo0) a = -INFINITY;
                    if (key > pos1 || key < lo1) c = -INFINITY;
                }
                s[nt][j] = a; s[nt][2 + j] = c;
                mx0 = fmaxf(mx0, a); mx1 = fmaxf(mx1, c);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;
        const float c0 = exp2f(m0 - b0), c1 = exp2f(m1 - b1);
        m0 = n0; m1 = n1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - b0); s[nt][1] = exp2f(s[nt][1] - b0);
            s[nt][2] = exp2f(s[nt][2] - b1); s[nt][3] = exp2f(s[nt][3] - b1);
            sum0 += s[nt][0] + s[nt][1];
            sum1 += s[nt][2] + s[nt][3];
        }
        l0 = l0 * c0 + sum0;
        l1 = l1 * c1 + sum1;
#pragma unroll
        for (int i = 0; i < NT; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        {
            const int mat = lane >> 3, r = lane & 7;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {                 // 16 keys each
                unsigned pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]); pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]); pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                const int row = kk * 16 + (mat & 1) * 8 + r;
#pragma unroll
                for (int c = 0; c < NT; c += 2) {
                    unsigned vb[4];
                    ldmatrix_x4_trans(vb, smem_u32(vt + (row * CPR + swz<D>(row, c + (mat >> 1))) * 8));
                    mma16816(o[c], pf, vb[0], vb[1]);
                    mma16816(o[c + 1], pf, vb[2], vb[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = live0 ? 1.0f / l0 : 0.f, i1 = live1 ? 1.0f / l1 : 0.f;
    bf16* oa = out + ((size_t)(q_begin + j0 + (live0 ? tok0 : 0)) * nq + (size_t)kvh * group + r0 % group) * D;
    bf16* ob = out + ((size_t)(q_begin + j0 + (live1 ? tok1 : 0)) * nq + (size_t)kvh * group + r1 % group) * D;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int d = i * 8 + 2 * t;
        if (live0) *reinterpret_cast<unsigned*>(oa + d) = pack_bf16(o[i][0] * i0, o[i][1] * i0);
        if (live1) *reinterpret_cast<unsigned*>(ob + d) = pack_bf16(o[i][2] * i1, o[i][3] * i1);
    }
}

template <int D>
static int launch_prefill(bf16* out, const bf16* q, const bf16* k, const bf16* v, const int* table, int table_stride,
                          const int* seq_slots, const int* cu_seqlens, const int* kv_lens, int n_seqs, int total_tiles,
                          float scale, int nq, int nkv, int tokens_per_tile, int window, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = PrefillSmem<D>::BYTES;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return ti_fail("attention_prefill: %s", cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(total_tiles, nkv);
    ti_launch(attention_prefill_kernel<D>, dim3(grid), dim3(PF_THREADS), smem, stream, out, q, k, v, table, table_stride, seq_slots, cu_seqlens,
                                                                   kv_lens, n_seqs, scale * 1.4426950408889634f, nq, nkv,
                                                                   tokens_per_tile, window);
    return ti_check_launch("attention_prefill");
}

// `total_tiles` = sum over the sequences of ceil(tokens of the sequence / tokens_per_tile), with
// tokens_per_tile = 128 / (query heads per KV head). Returns 2 when the sizes are outside what the
// kernel takes (the caller then runs the plain kernel).
extern "C" int ti_attention_prefill(void* out, const void* q, const void* k_cache, const void* v_cache,
                                    const int* block_table, int table_stride, const int* seq_slots,
                                    const int* cu_seqlens, const int* kv_lens, int n_seqs, int total_tiles, float scale,
                                    int nq, int nkv, int D, int page_size, int window, cudaStream_t stream) {
    if (n_seqs == 0 || total_tiles == 0) return 0;
    if (page_size != PF_PAGE || nq % nkv != 0 || nq / nkv > PF_ROWS || D % 16 != 0 || nkv > 65535) {
        ti_fail("attention_prefill takes page size %d, at most %d query heads per KV head and head sizes in steps of 16; "
                "got page %d, %d/%d heads, head size %d", PF_PAGE, PF_ROWS, page_size, nq, nkv, D);
        return 2;
    }
    const int tokens_per_tile = PF_ROWS / (nq / nkv);
#define PF_CASE(d)                                                                                                     \
    case d:                                                                                                            \
        return launch_prefill<d>((bf16*)out, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table,    \
                                 table_stride, seq_slots, cu_seqlens, kv_lens, n_seqs, total_tiles, scale, nq, nkv,    \
                                 tokens_per_tile, window, stream);
    switch (D) {
        PF_CASE(16) PF_CASE(32) PF_CASE(48) PF_CASE(64) PF_CASE(80) PF_CASE(96) PF_CASE(112) PF_CASE(128) PF_CASE(256)
        default:
            ti_fail("attention_prefill has no instance for head size %d", D);
            return 2;
    }
#undef PF_CASE
}
