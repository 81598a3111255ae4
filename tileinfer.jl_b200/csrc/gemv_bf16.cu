// Weight-streaming product for steps of a few tokens (decode): y[n, out] = x[n, in] · W[out, in]ᵀ
// in bfloat16 with n <= 16. The step is bound by reading W once from HBM, so the kernel is
// built around keeping many 16-byte weight loads in flight per thread; the arithmetic rides
// on mma.sync m16n8k16 with the weights as the 16-row operand and the tokens as the 8-wide
// one (a CUDA-core dot product per token would cost n times the multiply-adds).
//
// A block owns 16 output rows (and one slice of k when the product is split); its warps
// take interleaved 32-wide blocks of k, and their partial sums are added in warp order in
// shared memory. Within a 32-wide block a thread reads 8 consecutive k of its two rows and
// of its token, so every global load is 16 bytes; the k positions inside the two mma
// operands are permuted the same way on both sides, which leaves the dot product unchanged.
// The weights are read once and pass L1 by; the tokens, which every block reads, go through it,
// where a block finds part of what the blocks before it on the same SM read (about half of the
// token reads hit at 8 tokens).
//
// Epilogues: none, xIELU (up_proj), 32-bit logits (LM head), or raw 32-bit partial sums
// [split, n, out] that the following residual-add + RMSNorm kernel adds in a fixed order.
//
// AntoineBut/TileInfer.jl's counterpart is its GEMV (src/ops/tile/linear.jl:15-29, 58-74):
// 32-bit accumulation, one rounding, activation on the rounded sums.
#include "common.cuh"

#define GV_WARPS 8
#define GV_EPI_NONE 0
#define GV_EPI_XIELU 1
#define GV_EPI_F32_OUT 2
#define GV_EPI_PARTIAL 3

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The tokens: every block reads all of them, so they are worth a place in L1 (the weights pass it by).
__device__ __forceinline__ uint4 ld_tokens(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int U>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_bf16_kernel(const bf16* __restrict__ W, const bf16* x,
                                                                  long long ldx, void* __restrict__ y, long long ldy,
                                                                  int n, int out, int K, int splits, int epilogue,
                                                                  XieluParams act) {
    __shared__ float red[GV_WARPS][NT][32][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int ra = min(row0 + g, out - 1), rb = min(row0 + g + 8, out - 1);
    const uint4* wa = reinterpret_cast<const uint4*>(W + (size_t)ra * K);
    const uint4* wb = reinterpret_cast<const uint4*>(W + (size_t)rb * K);
    const uint4* xr[NT];
    bool xv[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xv[j] = g + 8 * j < n;
        xr[j] = reinterpret_cast<const uint4*>(x + (size_t)(xv[j] ? g + 8 * j : 0) * ldx);
    }
    float c[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) c[j][i] = 0.f;

    const int nblk = (K + 31) >> 5;
    const int blk_lo = (int)((long long)nblk * blockIdx.y / splits);
    const int blk_hi = (int)((long long)nblk * (blockIdx.y + 1) / splits);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // The weights do not depend on the previous kernel: the first batch of weight loads is issued
    // before waiting for it, so this kernel's stream starts while the previous one drains.
    bool waited = false;
    for (int b = blk_lo + warp; b < blk_hi; b += GV_WARPS * U) {
        uint4 a0[U], a1[U], xb[NT][U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int bb = b + u * GV_WARPS;
            const bool ok = bb < blk_hi && bb * 32 + 8 * t < K;
            const int idx = bb * 4 + t;
            a0[u] = ok ? ld_stream(wa + idx) : zero;
            a1[u] = ok ? ld_stream(wb + idx) : zero;
        }
        if (!waited) { pdl_wait(); pdl_launch_dependents(); waited = true; }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int bb = b + u * GV_WARPS;
            const bool ok = bb < blk_hi && bb * 32 + 8 * t < K;
            const int idx = bb * 4 + t;
#pragma unroll
            for (int j = 0; j < NT; ++j) xb[j][u] = (ok && xv[j]) ? ld_tokens(xr[j] + idx) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mma_bf16(c[j], a0[u].x, a1[u].x, a0[u].y, a1[u].y, xb[j][u].x, xb[j][u].y);
                mma_bf16(c[j], a0[u].z, a1[u].z, a0[u].w, a1[u].w, xb[j][u].z, xb[j][u].w);
            }
    }
    if (!waited) { pdl_wait(); pdl_launch_dependents(); }   // a warp without work still orders its writes after the predecessor
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][j][lane][i] = c[j][i];
    __syncthreads();
    for (int e = threadIdx.x; e < NT * 128; e += GV_WARPS * 32) {
        const int j = e >> 7, l = (e & 127) >> 2, ci = e & 3;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) s += red[w][j][l][ci];
        const int row = row0 + (l >> 2) + ((ci & 2) ? 8 : 0);
        const int col = 8 * j + 2 * (l & 3) + (ci & 1);
        if (row >= out || col >= n) continue;
        if (epilogue == GV_EPI_PARTIAL) {
            ((float*)y)[((size_t)blockIdx.y * n + col) * ldy + row] = s;
            continue;
        }
        float v = rnd<bf16>(s);
        if (epilogue == GV_EPI_XIELU) v = xielu_value<bf16>(v, act);
        if (epilogue == GV_EPI_F32_OUT) ((float*)y)[(size_t)col * ldy + row] = v;
        else ((bf16*)y)[(size_t)col * ldy + row] = __float2bfloat16_rn(v);
    }
}

// y: [n, ldy] (bfloat16, or float32 for the logits), or partials [splits, n, ldy] float32.
extern "C" int ti_gemv_bf16(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in,
                            int splits, int epilogue, float alpha_p, float alpha_n, float beta, float eps,
                            cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(n >= 1 && n <= 16, "gemv: %d tokens (this kernel takes 1 to 16)", n);
    TI_REQUIRE(in % 8 == 0 && ldx % 8 == 0, "gemv: in=%d and the row stride of x (%lld) must be multiples of 8", in, ldx);
    TI_REQUIRE(((uintptr_t)W % 16 == 0) && ((uintptr_t)x % 16 == 0), "gemv: operands must be 16-byte aligned");
    TI_REQUIRE(splits >= 1 && (splits == 1 || epilogue == GV_EPI_PARTIAL), "gemv: a split product leaves partial sums");
    TI_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemv: unknown epilogue %d", epilogue);
    dim3 grid((out + 15) / 16, splits);
    XieluParams act{alpha_p, alpha_n, beta, eps};
    if (n <= 8)
        ti_launch(gemv_bf16_kernel<1, 8>, dim3(grid), dim3(GV_WARPS * 32), 0, stream, (const bf16*)W, (const bf16*)x, ldx, y, ldy, n, out, in,
                                                                   splits, epilogue, act);
    else
        ti_launch(gemv_bf16_kernel<2, 4>, dim3(grid), dim3(GV_WARPS * 32), 0, stream, (const bf16*)W, (const bf16*)x, ldx, y, ldy, n, out, in,
                                                                   splits, epilogue, act);
    return ti_check_launch("gemv_bf16");
}
