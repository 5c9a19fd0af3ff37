// Next-token choice on the device: greedy argmax and temperature sampling.
//
// The reference samples greedily only, with one block per row and no rule for ties
// (src/qwen_kernels.cu:229-248).  Here the lowest index wins a tie, and temperature
// sampling is the Gumbel-max form argmax_i(logit_i / temperature + g_i) with
// g_i = -log(-log(u_i)), u_i from Philox4x32-10 keyed by the request's seed and counted
// by (vocabulary index, number of tokens the request has sampled so far): the draw of a
// request does not depend on the batch it is in.
//
// Two stages: `parts` blocks per row each reduce a slice of the vocabulary, then one
// block per row reduces the partial winners.  The partials are caller-provided.
#include "common.cuh"

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                              uint32_t k1, uint32_t* out) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
        const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += W0; k1 += W1;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
    // u in (0, 1): (bits + 0.5) / 2^32, taken in float32 from the top 24 bits so that u < 1.
    const float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
    return -logf(-logf(u));
}

__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void sample_stage1_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                                     const unsigned long long* __restrict__ seeds, const int* __restrict__ counters,
                                     float* __restrict__ part_val, int* __restrict__ part_idx, int parts) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sv[32];
    __shared__ int si[32];
    const int row = blockIdx.y, part = blockIdx.x;
    const float temp = temperature[row];
    const float* lr = logits + (size_t)row * V;
    const int per = ((V + parts - 1) / parts + 3) & ~3;          // a multiple of four: parts start on 16-byte boundaries
    const int begin = min(V, part * per), end = min(V, begin + per);
    float bv = -FLT_MAX; int bi = 0x7fffffff;
    if (temp > 0.f) {
        const unsigned long long seed = seeds[row];
        const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
        const uint32_t ctr = (uint32_t)counters[row];
        const float inv_t = 1.f / temp;
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            uint32_t rnd[4];
            philox4x32_10((uint32_t)i, ctr, 0u, 0u, k0, k1, rnd);
            better(bv, bi, lr[i] * inv_t + gumbel_from_bits(rnd[0]), i);
        }
    } else if ((((uintptr_t)lr | (uintptr_t)begin * 4) & 15) == 0) {
        // Greedy: four logits a load, four loads in flight; `better` is a total order (value, then lowest index), so
        // the order in which candidates meet does not matter.
        const int vec_end = begin + ((end - begin) & ~3);
        for (int i0 = begin + threadIdx.x * 4; i0 < vec_end; i0 += blockDim.x * 16) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x * 4;
                v[u] = i < vec_end ? *reinterpret_cast<const float4*>(lr + i) : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x * 4;
                if (i < vec_end) {
                    better(bv, bi, v[u].x, i); better(bv, bi, v[u].y, i + 1);
                    better(bv, bi, v[u].z, i + 2); better(bv, bi, v[u].w, i + 3);
                }
            }
        }
        for (int i = vec_end + threadIdx.x; i < end; i += blockDim.x) better(bv, bi, lr[i], i);
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) better(bv, bi, lr[i], i);
    }
    // The block's best: within each warp by shuffles, then over the warps.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nwarps ? sv[lane] : -FLT_MAX;
        bi = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            better(bv, bi, ov, oi);
        }
        if (lane == 0) { sv[0] = bv; si[0] = bi; }
    }
    __syncthreads();
    if (threadIdx.x == 0) { part_val[row * parts + part] = sv[0]; part_idx[row * parts + part] = si[0]; }
}

__global__ void sample_stage2_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int parts,
                                     int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    // One warp per row; parts <= 1024.
    const int row = blockIdx.x;
    float bv = -FLT_MAX; int bi = 0x7fffffff;
    for (int p = threadIdx.x; p < parts; p += 32) better(bv, bi, part_val[row * parts + p], part_idx[row * parts + p]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bv, bi, ov, oi);
    }
    if (threadIdx.x == 0) out[row] = bi;
}

// logits [R, V] float32; temperature[R] (0 = greedy); seeds[R]; counters[R]; out[R] int32.
// part_val / part_idx: scratch of R * parts entries each (parts as returned by kvb_sample_parts).
KVB_API int kvb_sample_parts(int V) {
    int parts = (V + 4095) / 4096;
    if (parts < 1) parts = 1;
    if (parts > 64) parts = 64;
    return parts;
}

KVB_API int kvb_sample(const float* logits, int R, int V, const float* temperature,
                       const unsigned long long* seeds, const int* counters, float* part_val, int* part_idx,
                       int* out, cudaStream_t stream) {
    if (R <= 0) return KVB_OK;
    if (V <= 0) return KVB_ERR_SHAPE;
    const int parts = kvb_sample_parts(V);
    dim3 grid(parts, R);
    kvb_launch(sample_stage1_kernel, dim3(grid), dim3(256), 0, stream, logits, V, temperature, seeds, counters, part_val, part_idx, parts);
    kvb_launch(sample_stage2_kernel, dim3(R), dim3(32), 0, stream, part_val, part_idx, parts, out);
    return kvb_launch_status();
}
