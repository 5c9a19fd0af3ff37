// Embedding gather, residual-add + RMSNorm, and the gated activation.
//
// What they replace in the reference: k_embed (src/qwen_kernels.cu:14-23),
// k_rmsnorm with k_add in front of it (:26-43, :55-61) and k_silu_mul (:102-108).
// The residual stream is kept in float32 here, so the add and the norm are one
// kernel and the sum is never rounded to 16 bits.
#include "common.cuh"

// out[r, :] = float(table[id, :]) with id = ids[r], or, where src[r] >= 0, last[src[r]]: a token that the
// previous step sampled and left on the device.  A token id outside [0, V) sets the error word and yields zeros.
// `out16` (optional): the same rows rounded to bfloat16, for products that take the residual stream in that form.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ src,
                             const int* __restrict__ last, float* __restrict__ out, bf16* __restrict__ out16, int H, int V,
                             int* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int from = src ? src[r] : -1;
    const int tok = from >= 0 ? last[from] : ids[r];
    float* dst = out + (size_t)r * H;
    bf16* dst16 = out16 ? out16 + (size_t)r * H : nullptr;
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_TOKEN);
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            dst[i] = 0.f;
            if (dst16) dst16[i] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const T* row = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32<T>(row[i]);
        dst[i] = v;
        if (dst16) dst16[i] = __float2bfloat16_rn(v);
    }
}

KVB_API int kvb_embed(int dtype, const void* table, const int* ids, const int* src, const int* last, float* out, void* out16,
                      int T, int H, int V, int* err, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    const int threads = H >= 512 ? 256 : 128;
    if (dtype == KVB_F32)
        kvb_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, src, last, out, (bf16*)out16, H, V, err);
    else if (dtype == KVB_BF16)
        kvb_launch(embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)table, ids, src, last, out, (bf16*)out16, H, V, err);
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
    pdl_wait();
    pdl_launch_dependents();
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

// The same with 4 elements per thread and step (H a multiple of 4, rows 16-byte aligned).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// Four elements per thread and step.  A thread keeps its (up to) KEEP chunks of the row in registers between
// the sum of squares and the scaling, and reads the norm's weight - which no kernel writes - before it waits
// for the kernel that makes `delta`; rows longer than KEEP * 4 * blockDim are read a second time.
template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const T* __restrict__ delta, const float* __restrict__ w,
                                       T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    constexpr int KEEP = 2;
    __shared__ float scratch[33];
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;                      // written by the host's copy at the start of the step
    float4 ww[KEEP];
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        ww[k] = i < H ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    pdl_launch_dependents();
    float* hr = h + (size_t)r * H;
    const T* dr = delta ? delta + (size_t)r * H : nullptr;
    float4 kept[KEEP];
    float ss = 0.f;
    auto fetch = [&](int i) {
        float4 v = *reinterpret_cast<const float4*>(hr + i);
        if (dr) {
            const float4 d = Vec4<T>::load(dr + i);
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        return v;
    };
    auto square = [&](const float4& v) {                   // summed element by element, as the scalar kernel's thread does
        ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < H) {
            kept[k] = fetch(i);
            if (dr && !rows) *reinterpret_cast<float4*>(hr + i) = kept[k];
            square(kept[k]);
        }
    }
    for (int i = (threadIdx.x + KEEP * blockDim.x) * 4; i < H; i += blockDim.x * 4) {
        const float4 v = fetch(i);
        if (dr && !rows) *reinterpret_cast<float4*>(hr + i) = v;
        square(v);
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(total / (float)H + eps);
    T* orow = out + (size_t)o * H;
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < H) {
            const float4 v = kept[k], g = ww[k];
            Vec4<T>::store(orow + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        }
    }
    for (int i = (threadIdx.x + KEEP * blockDim.x) * 4; i < H; i += blockDim.x * 4) {
        // Beyond what the registers keep: read again (after an in-place update the row already holds the sum).
        float4 v = *reinterpret_cast<const float4*>(hr + i);
        if (rows && dr) {
            const float4 d = Vec4<T>::load(dr + i);
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        const float4 g = *reinterpret_cast<const float4*>(w + i);
        Vec4<T>::store(orow + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
    }
}

// One warp per row, for launches of many rows (prompt portions): a lane keeps its C chunks of four in registers, no
// barrier of the block is needed, and all rows of 2,048 are resident at once.  The additions are those of the kernel
// above in the same order - lane l's chunk c is thread l + 32 c's chunk there, each group of 32 is summed by the same
// shuffles, and the groups are added one after the other - so a row's result is bit for bit the same whichever of
// the two kernels a step's row count selects.  Needs H <= 128 C.
template <typename T, int C>
__global__ void add_rmsnorm_warp_kernel(float* __restrict__ h, const T* __restrict__ delta, const float* __restrict__ w,
                                        T* __restrict__ out, const int* __restrict__ rows, int n_out, int H, float eps) {
    const int lane = threadIdx.x & 31;
    const int o = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    float4 ww[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (lane + 32 * c) * 4;
        ww[c] = i < H ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    pdl_launch_dependents();
    if (o >= n_out) return;
    const int r = rows ? rows[o] : o;
    float* hr = h + (size_t)r * H;
    const T* dr = delta ? delta + (size_t)r * H : nullptr;
    float4 kept[C];
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (lane + 32 * c) * 4;
        kept[c] = i < H ? *reinterpret_cast<const float4*>(hr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (dr) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int i = (lane + 32 * c) * 4;
            if (i < H) {
                const float4 d = Vec4<T>::load(dr + i);
                kept[c].x += d.x; kept[c].y += d.y; kept[c].z += d.z; kept[c].w += d.w;
                if (!rows) *reinterpret_cast<float4*>(hr + i) = kept[c];
            }
        }
    }
    const int groups = (H / 4 + 31) >> 5;                   // the warps that the kernel above would run
    float total = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        float ss = 0.f;
        ss += kept[c].x * kept[c].x; ss += kept[c].y * kept[c].y; ss += kept[c].z * kept[c].z; ss += kept[c].w * kept[c].w;
        ss = warp_sum(ss);
        if (c < groups) total += ss;
    }
    const float inv = 1.f / sqrtf(total / (float)H + eps);
    T* orow = out + (size_t)o * H;
#pragma unroll
    for (int c = 0; c < C; ++c) {
        const int i = (lane + 32 * c) * 4;
        if (i < H) {
            const float4 v = kept[c], g = ww[c];
            Vec4<T>::store(orow + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        }
    }
}

template <typename T>
static bool launch_rmsnorm_warp(float* h, const T* delta, const float* w, T* out, const int* rows, int n_out, int H, float eps,
                                cudaStream_t stream) {
    constexpr int WARPS = 2;
    const dim3 grid((n_out + WARPS - 1) / WARPS), block(32 * WARPS);
    if (H <= 512) kvb_launch(add_rmsnorm_warp_kernel<T, 4>, grid, block, 0, stream, h, delta, w, out, rows, n_out, H, eps);
    else if (H <= 1024) kvb_launch(add_rmsnorm_warp_kernel<T, 8>, grid, block, 0, stream, h, delta, w, out, rows, n_out, H, eps);
    else if (H <= 1536) kvb_launch(add_rmsnorm_warp_kernel<T, 12>, grid, block, 0, stream, h, delta, w, out, rows, n_out, H, eps);
    else if (H <= 2048) kvb_launch(add_rmsnorm_warp_kernel<T, 16>, grid, block, 0, stream, h, delta, w, out, rows, n_out, H, eps);
    else return false;
    return true;
}

constexpr int RMSNORM_WARP_MIN_ROWS = 256;                  // below this a block per row has more loads in flight

KVB_API int kvb_add_rmsnorm(int dtype, float* h, const void* delta, const float* w, void* out, const int* rows,
                            int n_out, int H, float eps, cudaStream_t stream) {
    if (n_out <= 0) return KVB_OK;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const bool vec = H % 4 == 0 && ((((uintptr_t)h | (uintptr_t)w | (uintptr_t)out | (uintptr_t)delta) & 15) == 0);
    // One chunk of four per thread where the row allows it.
    const int vec_threads = H / 4 >= 1024 ? 1024 : (H / 4 + 31) / 32 * 32;
    if (vec && n_out >= RMSNORM_WARP_MIN_ROWS) {
        if (dtype == KVB_F32 && launch_rmsnorm_warp<float>(h, (const float*)delta, w, (float*)out, rows, n_out, H, eps, stream))
            return kvb_launch_status();
        if (dtype == KVB_BF16 && launch_rmsnorm_warp<bf16>(h, (const bf16*)delta, w, (bf16*)out, rows, n_out, H, eps, stream))
            return kvb_launch_status();
    }
    if (vec && dtype == KVB_F32) {
        kvb_launch(add_rmsnorm_vec_kernel<float>, dim3(n_out), dim3(vec_threads), 0, stream, h, (const float*)delta, w, (float*)out, rows, H, eps);
        return kvb_launch_status();
    }
    if (vec && dtype == KVB_BF16) {
        kvb_launch(add_rmsnorm_vec_kernel<bf16>, dim3(n_out), dim3(vec_threads), 0, stream, h, (const bf16*)delta, w, (bf16*)out, rows, H, eps);
        return kvb_launch_status();
    }
    if (dtype == KVB_F32)
        kvb_launch(add_rmsnorm_kernel<float>, dim3(n_out), dim3(threads), 0, stream, h, (const float*)delta, w, (float*)out, rows, H, eps);
    else if (dtype == KVB_BF16)
        kvb_launch(add_rmsnorm_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, h, (const bf16*)delta, w, (bf16*)out, rows, H, eps);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// out[r, i] = silu(gate[r, i]) * up[r, i],  silu(g) = g / (1 + exp(-g))   (src/qwen_kernels.cu:102-105).
// gu[r, :] holds the gate and up projections of row r: [gate(I) | up(I)], or, interleaved in eights,
// gate i at column 16 (i / 8) + i % 8 and up i eight columns further.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int interleaved) {
    pdl_wait();
    pdl_launch_dependents();
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

// Eight outputs per thread and step: 16-byte loads of gate and up, one 16-byte (bfloat16) store.
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, size_t groups, int interleaved) {
    pdl_wait();
    pdl_launch_dependents();
    const int per_row = I >> 3;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / per_row;
        const int b = (int)(idx - r * per_row);
        const bf16* gp = gu + r * 2 * I + (interleaved ? 16 * b : 8 * b);
        const uint4 graw = *reinterpret_cast<const uint4*>(gp);
        const uint4 uraw = *reinterpret_cast<const uint4*>(gp + (interleaved ? 8 : I));
        const uint32_t gw[4] = {graw.x, graw.y, graw.z, graw.w}, uw[4] = {uraw.x, uraw.y, uraw.z, uraw.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
            const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[k]));
            __nv_bfloat162 o = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        *reinterpret_cast<uint4*>(out + r * I + 8 * b) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

KVB_API int kvb_silu_mul(int dtype, const void* gate_up, void* out, int T, int I, int interleaved, cudaStream_t stream) {
    if (interleaved && I % 8 != 0) return KVB_ERR_SHAPE;
    const size_t total = (size_t)T * I;
    if (total == 0) return KVB_OK;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)kvb_sm_count() * 16;         // a grid-stride loop takes the rest
    if (blocks > most) blocks = most;
    if (dtype == KVB_BF16 && I % 8 == 0 && ((((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0)) {
        const size_t groups = total / 8;
        size_t vblocks = (groups + threads - 1) / threads;
        if (vblocks > most) vblocks = most;
        kvb_launch(silu_mul_vec8_kernel, dim3((int)vblocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, I, groups, interleaved);
        return kvb_launch_status();
    }
    if (dtype == KVB_F32)
        kvb_launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I, total, interleaved);
    else if (dtype == KVB_BF16)
        kvb_launch(silu_mul_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, I, total, interleaved);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
