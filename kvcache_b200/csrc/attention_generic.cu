// Causal attention over cache pages for any mix of rows, any head size and either storage
// type: the kernel of the float32 path and the fallback of the bfloat16 one.
//
// One block per (row, query head).  The row's keys lo..pos (lo = 0, or pos - window + 1
// for a windowed layer) are visited in chunks of the block's width: each thread scores
// one key, the block takes the chunk's maximum and sum, and threads then own output
// dimensions for the weighted sum of values.  The running (max, sum, acc) update is the
// reference's online softmax (src/qwen_kernels.cu:159-176: m' = max(m, s), c = e^{m-m'},
// p = e^{s-m'}, l = l c + p, acc = acc c + p v; out = acc / l), the chunked form of it
// is the reference's two-pass block softmax (src/batched.cu:97-130).  kv_head = h / (Hq / Hkv)
// and scale applied after the dot product (src/qwen_kernels.cu:148-167).
// Chunk boundaries are counted from `lo`, so a row's summation order is the same however
// the step was cut.
#include "common.cuh"

#define ATTN_THREADS 128
#define ATTN_MAX_D 512

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                                               int table_stride, const int* __restrict__ positions,
                                               const int* __restrict__ row_segment, T* __restrict__ out, int Hq,
                                               int Hkv, int D, int page_size, int window, float scale,
                                               int* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float smem[];
    float* q_s = smem;                    // [D]
    float* p_s = smem + D;                // [ATTN_THREADS]
    int* page_s = (int*)(p_s + ATTN_THREADS);  // [ATTN_THREADS] page offset of each key of the chunk
    float* scratch = (float*)(page_s + ATTN_THREADS);  // [33]

    const int r = blockIdx.x, h = blockIdx.y;
    const int hk = h / (Hq / Hkv);
    const int pos = positions[r];
    const int seg = row_segment[r];
    const int* table = block_table + (size_t)seg * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    const T* qr = q + ((size_t)r * Hq + h) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    constexpr int DPT = ATTN_MAX_D / ATTN_THREADS;  // output dims per thread
    float acc[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    for (int base = lo; base <= pos; base += ATTN_THREADS) {
        const int j = base + threadIdx.x;
        float s = -FLT_MAX;
        int off = -1;
        if (j <= pos) {
            const int page = table[j / page_size];
            if (page < 0) {
                atomicOr(err, KVB_DEV_BAD_PAGE);
            } else {
                off = ((page * Hkv + hk) * page_size + (j % page_size));
                const T* kr = k_pages + (size_t)off * D;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot += q_s[d] * to_f32<T>(kr[d]);
                s = dot * scale;
            }
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float corr = expf(m - m_new);
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        p_s[threadIdx.x] = p;
        page_s[threadIdx.x] = off;
        const float csum = block_sum(p, scratch);   // also orders the writes to p_s / page_s
        l = l * corr + csum;
        m = m_new;
        const int n = min(ATTN_THREADS, pos - base + 1);
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = threadIdx.x + i * ATTN_THREADS;
            if (d < D) {
                float a = acc[i] * corr;
                for (int t = 0; t < n; ++t) {
                    const int o = page_s[t];
                    if (o >= 0) a += p_s[t] * to_f32<T>(v_pages[(size_t)o * D + d]);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)r * Hq + h) * D;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = threadIdx.x + i * ATTN_THREADS;
        if (d < D) orow[d] = from_f32<T>(l > 0.f ? acc[i] / l : 0.f);
    }
}

KVB_API int kvb_paged_attention_generic(int dtype, const void* q, const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_stride, const int* positions,
                                        const int* row_segment, void* out, int T, int Hq, int Hkv, int D,
                                        int page_size, int window, float scale, int* err, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (D > ATTN_MAX_D || D < 1 || Hkv < 1 || Hq % Hkv != 0) return KVB_ERR_SHAPE;
    const size_t smem = (size_t)(D + 2 * ATTN_THREADS + 33) * sizeof(float);
    dim3 grid(T, Hq);
    if (dtype == KVB_F32)
        kvb_launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(ATTN_THREADS), smem, stream, 
            (const float*)q, (const float*)k_pages, (const float*)v_pages, block_table, table_stride, positions,
            row_segment, (float*)out, Hq, Hkv, D, page_size, window, scale, err);
    else if (dtype == KVB_BF16)
        kvb_launch(paged_attention_generic_kernel<bf16>, dim3(grid), dim3(ATTN_THREADS), smem, stream, 
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_stride, positions,
            row_segment, (bf16*)out, Hq, Hkv, D, page_size, window, scale, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}
