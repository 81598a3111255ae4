// One 64-key tile of decode attention for one warp: the warp takes 16 keys of the tile, the rows of
// the MMA tiles are the query heads that share the KV head. Shared by the decode kernels.
#pragma once
#include "mma_util.cuh"

#define AD_PAGE 64
#define AD_WARPS 4
#define AD_THREADS (AD_WARPS * 32)

// kt, vt: the K and V tiles in (swizzled) shared memory; qf: the query fragments; o, m, l: this warp's
// running output, maximum and sum for rows g and g + 8 (32-bit).
template <int D>
__device__ __forceinline__ void decode_tile(const bf16* kt, const bf16* vt, const unsigned (&qf)[D / 16][4], float (&o)[D / 8][4],
                                            float& m0, float& m1, float& l0, float& l1, int tile, int warp, int lane,
                                            int kv_len, int first_key, float scale_log2e) {
    constexpr int CPR = D / 8, KS = D / 16, NT = D / 8;
    const int t = lane & 3;
        float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    {
        const int mat = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (mat >> 1) * 8 + r;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            unsigned kb[4];
            ldmatrix_x4(kb, smem_u32(kt + (row * CPR + swz<D>(row, 2 * ks + (mat & 1))) * 8));
            mma16816(s[0], qf[ks], kb[0], kb[1]);
            mma16816(s[1], qf[ks], kb[2], kb[3]);
        }
    }
    const int key0 = tile * AD_PAGE + warp * 16 + 2 * t;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int key = key0 + 8 * nt + j;
            const bool ok = key < kv_len && key >= first_key;
            s[nt][j] = ok ? s[nt][j] * scale_log2e : -INFINITY;
            s[nt][2 + j] = ok ? s[nt][2 + j] * scale_log2e : -INFINITY;
            mx0 = fmaxf(mx0, s[nt][j]);
            mx1 = fmaxf(mx1, s[nt][2 + j]);
        }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    const float b0 = n0 == -INFINITY ? 0.f : n0, b1 = n1 == -INFINITY ? 0.f : n1;
    const float c0 = exp2f(m0 - b0), c1 = exp2f(m1 - b1);
    m0 = n0; m1 = n1;
    unsigned pf[4];
    {
        float p[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            p[nt][0] = exp2f(s[nt][0] - b0); p[nt][1] = exp2f(s[nt][1] - b0);
            p[nt][2] = exp2f(s[nt][2] - b1); p[nt][3] = exp2f(s[nt][3] - b1);
        }
        l0 = l0 * c0 + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
        l1 = l1 * c1 + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
        pf[0] = pack_bf16(p[0][0], p[0][1]); pf[1] = pack_bf16(p[0][2], p[0][3]);
        pf[2] = pack_bf16(p[1][0], p[1][1]); pf[3] = pack_bf16(p[1][2], p[1][3]);
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
    {
        const int mat = lane >> 3, r = lane & 7;
        const int row = warp * 16 + (mat & 1) * 8 + r;
#pragma unroll
        for (int c = 0; c < NT; c += 2) {
            unsigned vb[4];
            ldmatrix_x4_trans(vb, smem_u32(vt + (row * CPR + swz<D>(row, c + (mat >> 1))) * 8));
            mma16816(o[c], pf, vb[0], vb[1]);
            mma16816(o[c + 1], pf, vb[2], vb[3]);
        }
    }
}
