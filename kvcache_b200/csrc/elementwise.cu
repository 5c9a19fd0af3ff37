// Embedding gather, residual-add + RMSNorm, and the gated activation.
//
// What they replace in the reference: k_embed (src/qwen_kernels.cu:14-23),
// k_rmsnorm with k_add in front of it (:26-43, :55-61) and k_silu_mul (:102-108).
// The residual stream is kept in float32 here, so the add and the norm are one
// kernel and the sum is never rounded to 16 bits.
#include "common.cuh"

// out[r, :] = float(table[ids[r], :]).  A token id outside [0, V) sets the error word and yields zeros.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int H, int V, int* __restrict__ err) {
    const int r = blockIdx.x;
    const int tok = ids[r];
    float* dst = out + (size_t)r * H;
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = 0.f;
        return;
    }
    const T* src = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

KVB_API int kvb_embed(int dtype, const void* table, const int* ids, float* out, int T, int H, int V, int* err,
                      cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    const int threads = H >= 512 ? 256 : 128;
    if (dtype == KVB_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>((const float*)table, ids, out, H, V, err);
    else if (dtype == KVB_BF16)
        embed_kernel<bf16><<<T, threads, 0, stream>>>((const bf16*)table, ids, out, H, V, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// One block per output row.
//   rows == nullptr: r = blockIdx.x;  h[r] += delta[r] (if delta);  out[r] = norm(h[r]) * w
//   rows != nullptr: r = rows[blockIdx.x]; v = h[r] + delta[r]; out[blockIdx.x] = norm(v) * w; h untouched
// norm(v) = v * rsqrt(mean(v^2) + eps), everything in float32 (src/qwen_kernels.cu:26-40:
// fp32 sum of squares, (x * inv) * w, one rounding at the store).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta, const float* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* hr = h + (size_t)r * H;
    const T* dr = delta ? delta + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (dr) v += to_f32<T>(dr[i]);
        if (!rows && dr) hr[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(total / (float)H + eps);
    T* orow = out + (size_t)o * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (rows && dr) v += to_f32<T>(dr[i]);
        orow[i] = from_f32<T>(v * inv * w[i]);
    }
}

KVB_API int kvb_add_rmsnorm(int dtype, float* h, const void* delta, const float* w, void* out, const int* rows,
                            int n_out, int H, float eps, cudaStream_t stream) {
    if (n_out <= 0) return KVB_OK;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == KVB_F32)
        add_rmsnorm_kernel<float><<<n_out, threads, 0, stream>>>(h, (const float*)delta, w, (float*)out, rows, H, eps);
    else if (dtype == KVB_BF16)
        add_rmsnorm_kernel<bf16><<<n_out, threads, 0, stream>>>(h, (const bf16*)delta, w, (bf16*)out, rows, H, eps);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// out[r, i] = silu(gate[r, i]) * up[r, i],  silu(g) = g / (1 + exp(-g))   (src/qwen_kernels.cu:102-105).
// gu[r, :] holds the gate and up projections of row r: [gate(I) | up(I)], or, interleaved in eights,
// gate i at column 16 (i / 8) + i % 8 and up i eight columns further.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int interleaved) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / I;
        const int i = (int)(idx - r * I);
        const int gcol = interleaved ? 16 * (i >> 3) + (i & 7) : i;
        const float g = to_f32<T>(gu[r * 2 * I + gcol]);
        const float u = to_f32<T>(gu[r * 2 * I + gcol + (interleaved ? 8 : I)]);
        out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

KVB_API int kvb_silu_mul(int dtype, const void* gate_up, void* out, int T, int I, int interleaved, cudaStream_t stream) {
    if (interleaved && I % 8 != 0) return KVB_ERR_SHAPE;
    const size_t total = (size_t)T * I;
    if (total == 0) return KVB_OK;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == KVB_F32)
        silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, I, total, interleaved);
    else if (dtype == KVB_BF16)
        silu_mul_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I, total, interleaved);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
