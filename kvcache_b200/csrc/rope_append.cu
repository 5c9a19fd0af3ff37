// Bias + rotation of queries and keys + append of keys and values into cache pages, one kernel.
//
// Replaces k_add_bias, k_rope / k_rope_pos and k_write_kv / k_batched_write_kv of the
// reference (src/qwen_kernels.cu:46-52, :65-81, :253-267, :111-126, :270-290): the
// projection's output is read once, the bias is added and the pair (t, t + rot/2) is
// rotated in float32, and the result is rounded once on its way to the query buffer or
// to the page `block_table[segment][pos / page]`, slot `pos % page`
// (pool layout [pages, kv_heads, page, head_dim] as src/include/kv_cache_manager.h:89-91).
//
// The angles come from a table cos/sin[pos, t] that the host fills in double
// precision; a position beyond the table sets the error word.
#include "common.cuh"

template <typename T>
__global__ void qkv_rope_append_kernel(const T* __restrict__ qkv, const float* __restrict__ bias,
                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                       int rot_half, int table_len, const int* __restrict__ positions,
                                       const int* __restrict__ row_segment, const int* __restrict__ block_table,
                                       int table_stride, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                       T* __restrict__ q_out, int Hq, int Hkv, int D, int page_size, int write_kv,
                                       int* __restrict__ err) {
    const int r = blockIdx.x;
    const int width = (Hq + 2 * Hkv) * D;
    const int pos = positions[r];
    const T* src = qkv + (size_t)r * width;
    const int rot = 2 * rot_half;

    size_t page_base = 0;
    bool page_ok = true;
    if (write_kv) {
        const int seg = row_segment[r];
        const int page = block_table[(size_t)seg * table_stride + pos / page_size];
        if (page < 0) {
            page_ok = false;
            if (threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_PAGE);
        }
        page_base = (size_t)(page < 0 ? 0 : page) * Hkv * page_size * D + (size_t)(pos % page_size) * D;
    }
    const bool pos_ok = rot_half == 0 || (pos >= 0 && pos < table_len);
    if (!pos_ok && threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_POS);
    const float* cr = cos_t + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sr = sin_t + (size_t)(pos_ok ? pos : 0) * rot_half;

    for (int idx = threadIdx.x; idx < width; idx += blockDim.x) {
        const int head = idx / D, d = idx - head * D;
        float x = to_f32<T>(src[idx]);
        if (bias) x += bias[idx];
        const bool is_v = head >= Hq + Hkv;
        if (!is_v && d < rot) {
            // rotate-half pairing (t, t + rot/2): x'_t = x_t cos - x_p sin ; x'_p = x_p cos + x_t sin
            const bool low = d < rot_half;
            const int t = low ? d : d - rot_half;
            const int pidx = low ? idx + rot_half : idx - rot_half;
            float xp = to_f32<T>(src[pidx]);
            if (bias) xp += bias[pidx];
            const float c = cr[t], s = sr[t];
            x = low ? (x * c - xp * s) : (x * c + xp * s);
        }
        if (head < Hq) {
            q_out[(size_t)r * Hq * D + idx] = from_f32<T>(x);
        } else if (write_kv && page_ok) {
            const int hk = is_v ? head - Hq - Hkv : head - Hq;
            const size_t dst = page_base + (size_t)hk * page_size * D + d;
            (is_v ? v_pages : k_pages)[dst] = from_f32<T>(x);
        }
    }
}

KVB_API int kvb_qkv_rope_append(int dtype, const void* qkv, const float* bias, const float* cos_t,
                                const float* sin_t, int rot_half, int table_len, const int* positions,
                                const int* row_segment, const int* block_table, int table_stride, void* k_pages,
                                void* v_pages, void* q_out, int T, int Hq, int Hkv, int D, int page_size,
                                int write_kv, int* err, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (2 * rot_half > D || rot_half < 0) return KVB_ERR_SHAPE;
    const int width = (Hq + 2 * Hkv) * D;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == KVB_F32)
        qkv_rope_append_kernel<float><<<T, threads, 0, stream>>>(
            (const float*)qkv, bias, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table,
            table_stride, (float*)k_pages, (float*)v_pages, (float*)q_out, Hq, Hkv, D, page_size, write_kv, err);
    else if (dtype == KVB_BF16)
        qkv_rope_append_kernel<bf16><<<T, threads, 0, stream>>>(
            (const bf16*)qkv, bias, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table,
            table_stride, (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, Hq, Hkv, D, page_size, write_kv, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
