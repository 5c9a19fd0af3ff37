// y[M, N] = x[M, K] . W[N, K]^T (+ bias), float32 accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, hence no
// reduced-precision mode) and the fallback of the bfloat16 path for shapes the
// tensor-core kernel refuses.  It plays the part of the reference's `linear` /
// `linear_logits` (apps/qwen_serve.cu:27-39): weights are [out, in] row-major, the
// output is the storage type or float32 (logits).
//
// Tiles of 64 x 64 outputs, 16 of K at a time; every thread owns a 4 x 4 patch and
// walks K in the same order whatever M is, so a row's result does not depend on the
// rows beside it.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w,
                                                        const float* __restrict__ bias, TOut* __restrict__ y, int M,
                                                        int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid / 4, lk = (tid % 4) * 4;   // each thread loads 4 consecutive k of one row

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lrow;
            const TIn* src = x + (size_t)gm * K + k0 + lk;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                xs[lk + c][lrow] = (gm < M && k0 + lk + c < K) ? to_f32<TIn>(src[c]) : 0.f;
            const int gn = n0 + lrow;
            const TIn* wsrc = w + (size_t)gn * K + k0 + lk;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                ws[lk + c][lrow] = (gn < N && k0 + lk + c < K) ? to_f32<TIn>(wsrc[c]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            y[(size_t)gm * N + gn] = from_f32<TOut>(v);
        }
    }
}

// in_dtype / out_dtype: 0 = float32, 1 = bfloat16.
KVB_API int kvb_gemm_simt(int in_dtype, int out_dtype, const void* x, const void* w, const float* bias, void* y,
                          int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (K <= 0) return KVB_ERR_SHAPE;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return KVB_ERR_LIMIT;
    if (in_dtype == KVB_F32 && out_dtype == KVB_F32)
        kvb_launch(gemm_simt_kernel<float, float>, dim3(grid), dim3(256), 0, stream, (const float*)x, (const float*)w, bias, (float*)y, M, N, K);
    else if (in_dtype == KVB_BF16 && out_dtype == KVB_BF16)
        kvb_launch(gemm_simt_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)x, (const bf16*)w, bias, (bf16*)y, M, N, K);
    else if (in_dtype == KVB_BF16 && out_dtype == KVB_F32)
        kvb_launch(gemm_simt_kernel<bf16, float>, dim3(grid), dim3(256), 0, stream, (const bf16*)x, (const bf16*)w, bias, (float*)y, M, N, K);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
