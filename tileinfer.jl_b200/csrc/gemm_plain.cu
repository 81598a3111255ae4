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

extern "C" int ti_gemm_plain(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in,
                             int epilogue, float alpha_p, float alpha_n, float beta, float eps, int dtype,
                             cudaStream_t stream) {
    if (n == 0) return 0;
    TI_REQUIRE(n > 0 && out > 0 && in > 0, "gemm: bad sizes n=%d out=%d in=%d", n, out, in);
    TI_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
    dim3 grid((out + GP_BN - 1) / GP_BN, (n + GP_BM - 1) / GP_BM);
    TI_REQUIRE(grid.y <= 65535, "gemm: too many rows (%d) for one launch", n);
    XieluParams act{alpha_p, alpha_n, beta, eps};
    TI_DISPATCH_DTYPE(dtype, (ti_launch(gemm_plain_kernel<T>, dim3(grid), dim3(256), 0, stream, y, ldy, (const T*)x, ldx, (const T*)W, n, out, in,
                                                                          epilogue, act)));
    return ti_check_launch("gemm_plain");
}
