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
    pdl_wait();
    pdl_launch_dependents();
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

// bfloat16, head sizes and rotation halves that are multiples of 8: one thread moves 8 elements
// (16 bytes) of a head; for a rotated chunk it also reads the partner chunk rot/2 further (or back).
// What does not depend on the product before this kernel - the row's position and page, and the first
// chunk's angles and biases - is read before the wait for that product.
struct ChunkTables {
    float cs[8], sn[8], b_self[8], b_partner[8];
};

__device__ __forceinline__ void chunk_tables(ChunkTables& t, int c, int chunks_per_head, int D, int Hq, int Hkv, int rot_half,
                                             const float* cr, const float* sr, const float* bias) {
    const int head = c / chunks_per_head, d = (c - head * chunks_per_head) * 8;
    const int idx = head * D + d;
    const bool rotated = head < Hq + Hkv && d < 2 * rot_half;
    const bool low = d < rot_half;
    const int t0 = low ? d : d - rot_half;
    const int pidx = low ? idx + rot_half : idx - rot_half;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        t.b_self[k] = bias ? bias[idx + k] : 0.f;
        t.b_partner[k] = (bias && rotated) ? bias[pidx + k] : 0.f;
        t.cs[k] = rotated ? cr[t0 + k] : 1.f;
        t.sn[k] = rotated ? sr[t0 + k] : 0.f;
    }
}

__global__ void qkv_rope_append_vec8_kernel(const bf16* __restrict__ qkv, const float* __restrict__ bias,
                                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                            int rot_half, int table_len, const int* __restrict__ positions,
                                            const int* __restrict__ row_segment, const int* __restrict__ block_table,
                                            int table_stride, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                            bf16* __restrict__ q_out, int Hq, int Hkv, int D, int page_size, int write_kv,
                                            int* __restrict__ err) {
    // This kernel is a few small blocks: it lets its successor (attention, which fetches block tables and old keys
    // before its own wait) onto the SMs at once, while the product before this kernel may still be running.
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int width = (Hq + 2 * Hkv) * D;
    const int pos = positions[r];
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
    const int chunks_per_head = D >> 3;
    const int chunks = width >> 3;
    ChunkTables tab;
    if ((int)threadIdx.x < chunks) chunk_tables(tab, threadIdx.x, chunks_per_head, D, Hq, Hkv, rot_half, cr, sr, bias);
    pdl_wait();
    const bf16* src = qkv + (size_t)r * width;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        if (c != (int)threadIdx.x) chunk_tables(tab, c, chunks_per_head, D, Hq, Hkv, rot_half, cr, sr, bias);
        const int head = c / chunks_per_head, d = (c - head * chunks_per_head) * 8;
        const int idx = head * D + d;
        float x[8];
        {
            const uint4 raw = *reinterpret_cast<const uint4*>(src + idx);
            const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[k]));
                x[2 * k] = f.x; x[2 * k + 1] = f.y;
            }
            if (bias) {
#pragma unroll
                for (int k = 0; k < 8; ++k) x[k] += tab.b_self[k];
            }
        }
        const bool is_v = head >= Hq + Hkv;
        if (!is_v && d < rot) {
            const bool low = d < rot_half;
            const int pidx = low ? idx + rot_half : idx - rot_half;
            const uint4 raw = *reinterpret_cast<const uint4*>(src + pidx);
            const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[k]));
                float xp0 = f.x, xp1 = f.y;
                if (bias) { xp0 += tab.b_partner[2 * k]; xp1 += tab.b_partner[2 * k + 1]; }
                const float c0 = tab.cs[2 * k], s0 = tab.sn[2 * k], c1 = tab.cs[2 * k + 1], s1 = tab.sn[2 * k + 1];
                x[2 * k] = low ? (x[2 * k] * c0 - xp0 * s0) : (x[2 * k] * c0 + xp0 * s0);
                x[2 * k + 1] = low ? (x[2 * k + 1] * c1 - xp1 * s1) : (x[2 * k + 1] * c1 + xp1 * s1);
            }
        }
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 o = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        const uint4 packed = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        if (head < Hq) {
            *reinterpret_cast<uint4*>(q_out + (size_t)r * Hq * D + idx) = packed;
        } else if (write_kv && page_ok) {
            const int hk = is_v ? head - Hq - Hkv : head - Hq;
            *reinterpret_cast<uint4*>((is_v ? v_pages : k_pages) + page_base + (size_t)hk * page_size * D + d) = packed;
        }
    }
}

// The same for steps of many rows (portions of prompts): a block takes ROWS consecutive rows.  Their positions and
// pages are looked up and their angles staged in shared memory once, before the wait (a row's 2 * rot_half angles are
// the same for all its heads); a thread keeps the biases of its chunk, which are the same for every row, in
// registers, and the loads of all ROWS rows of its chunk are in flight together.  With a quarter of the blocks of
// the one-row kernel the whole grid is on the SMs at once.
template <int ROWS>
__global__ void qkv_rope_append_rows_kernel(const bf16* __restrict__ qkv, const float* __restrict__ bias,
                                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                            int rot_half, int table_len, const int* __restrict__ positions,
                                            const int* __restrict__ row_segment, const int* __restrict__ block_table,
                                            int table_stride, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                            bf16* __restrict__ q_out, int T, int Hq, int Hkv, int D, int page_size,
                                            int write_kv, int* __restrict__ err) {
    extern __shared__ float angles[];                      // [ROWS][2][rot_half]: cos, sin
    __shared__ long long page_base_s[ROWS];                // element offset of the row's slot in the pools; -1: no page
    const int r0 = blockIdx.x * ROWS;
    const int width = (Hq + 2 * Hkv) * D;
    const int rot = 2 * rot_half;
    if (threadIdx.x < ROWS) {
        const int r = r0 + threadIdx.x;
        long long base = -1;
        if (r < T && write_kv) {
            const int pos = positions[r];
            const int page = block_table[(size_t)row_segment[r] * table_stride + pos / page_size];
            if (page < 0) atomicOr(err, KVB_DEV_BAD_PAGE);
            else base = (long long)page * Hkv * page_size * D + (long long)(pos % page_size) * D;
        }
        page_base_s[threadIdx.x] = base;
    }
    for (int i = threadIdx.x; i < ROWS * rot; i += blockDim.x) {
        const int row = i / rot, j = i - row * rot, r = r0 + row;
        float v = j < rot_half ? 1.f : 0.f;
        if (r < T) {
            const int pos = positions[r];
            const bool pos_ok = pos >= 0 && pos < table_len;
            if (!pos_ok && j == 0) atomicOr(err, KVB_DEV_BAD_POS);
            const int p = pos_ok ? pos : 0;
            v = j < rot_half ? cos_t[(size_t)p * rot_half + j] : sin_t[(size_t)p * rot_half + j - rot_half];
        }
        angles[i] = v;
    }
    const int chunks_per_head = D >> 3;
    const int chunks = width >> 3;
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        const int head = c / chunks_per_head, d = (c - head * chunks_per_head) * 8;
        const int idx = head * D + d;
        const bool is_v = head >= Hq + Hkv;
        const bool rotated = !is_v && d < rot;
        const bool low = d < rot_half;
        const int t0 = low ? d : d - rot_half;
        const int pidx = low ? idx + rot_half : idx - rot_half;
        float b_self[8], b_partner[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            b_self[k] = bias ? bias[idx + k] : 0.f;
            b_partner[k] = (bias && rotated) ? bias[pidx + k] : 0.f;
        }
        uint4 own[ROWS], partner[ROWS];
#pragma unroll
        for (int row = 0; row < ROWS; ++row) {
            const int r = min(r0 + row, T - 1);
            own[row] = *reinterpret_cast<const uint4*>(qkv + (size_t)r * width + idx);
            partner[row] = rotated ? *reinterpret_cast<const uint4*>(qkv + (size_t)r * width + pidx) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int row = 0; row < ROWS; ++row) {
            const int r = r0 + row;
            if (r >= T) break;
            const uint32_t wv[4] = {own[row].x, own[row].y, own[row].z, own[row].w};
            const uint32_t pv[4] = {partner[row].x, partner[row].y, partner[row].z, partner[row].w};
            const float* cs = angles + row * rot + t0;
            const float* sn = cs + rot_half;
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv[k]));
                float x0 = f.x + b_self[2 * k], x1 = f.y + b_self[2 * k + 1];
                if (rotated) {
                    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pv[k]));
                    const float xp0 = g.x + b_partner[2 * k], xp1 = g.y + b_partner[2 * k + 1];
                    const float c0 = cs[2 * k], s0 = sn[2 * k], c1 = cs[2 * k + 1], s1 = sn[2 * k + 1];
                    x0 = low ? (x0 * c0 - xp0 * s0) : (x0 * c0 + xp0 * s0);
                    x1 = low ? (x1 * c1 - xp1 * s1) : (x1 * c1 + xp1 * s1);
                }
                __nv_bfloat162 o = __floats2bfloat162_rn(x0, x1);
                ow[k] = *reinterpret_cast<uint32_t*>(&o);
            }
            const uint4 packed = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            if (head < Hq) {
                *reinterpret_cast<uint4*>(q_out + (size_t)r * Hq * D + idx) = packed;
            } else if (write_kv && page_base_s[row] >= 0) {
                const int hk = is_v ? head - Hq - Hkv : head - Hq;
                *reinterpret_cast<uint4*>((is_v ? v_pages : k_pages) + page_base_s[row] + (size_t)hk * page_size * D + d) = packed;
            }
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
    const uintptr_t addresses = (uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)q_out;
    if (dtype == KVB_BF16 && D % 8 == 0 && rot_half % 8 == 0 && (addresses & 15) == 0) {
        const int chunk_threads = width / 8 >= 1024 ? 1024 : (width / 8 + 31) / 32 * 32;
        if (T >= 256 && rot_half > 0) {
            constexpr int ROWS = 4;
            kvb_launch(qkv_rope_append_rows_kernel<ROWS>, dim3((T + ROWS - 1) / ROWS), dim3(chunk_threads),
                       (size_t)ROWS * 2 * rot_half * sizeof(float), stream, (const bf16*)qkv, bias, cos_t, sin_t, rot_half, table_len,
                       positions, row_segment, block_table, table_stride, (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, T, Hq,
                       Hkv, D, page_size, write_kv, err);
            return kvb_launch_status();
        }
        // One 16-byte chunk per thread where the row allows it.
        kvb_launch(qkv_rope_append_vec8_kernel, dim3(T), dim3(width / 8 >= 1024 ? 1024 : (width / 8 + 31) / 32 * 32), 0, stream,
            (const bf16*)qkv, bias, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table, table_stride,
            (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, Hq, Hkv, D, page_size, write_kv, err);
        return kvb_launch_status();
    }
    if (dtype == KVB_F32)
        kvb_launch(qkv_rope_append_kernel<float>, dim3(T), dim3(threads), 0, stream, 
            (const float*)qkv, bias, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table,
            table_stride, (float*)k_pages, (float*)v_pages, (float*)q_out, Hq, Hkv, D, page_size, write_kv, err);
    else if (dtype == KVB_BF16)
        kvb_launch(qkv_rope_append_kernel<bf16>, dim3(T), dim3(threads), 0, stream, 
            (const bf16*)qkv, bias, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table,
            table_stride, (bf16*)k_pages, (bf16*)v_pages, (bf16*)q_out, Hq, Hkv, D, page_size, write_kv, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
