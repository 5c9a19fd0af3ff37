// y[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 64): the matrix product of a decode step,
// where the weights are read once from HBM and everything else is small.
//
// The reference runs these products through cublasGemmEx (apps/qwen_serve.cu:27-39, :149-171);
// at M of 1..64 a library kernel of 128-row tiles leaves most of the machine idle.  Here the
// roles are swapped: 16 rows of W are the tensor core's A operand, streamed straight from global
// memory into registers (no shared-memory staging of weights), the M activations rows are the B
// operand (n = 8 per tile), and K is walked 32 at a time with the k index permuted so that every
// thread loads 16 contiguous bytes: thread (g, t) of a warp takes W[row g][32 kb + 8 t .. + 7]
// and x[row g][same], which feed two mma.sync m16n8k16 (logical k {2t, 2t+1, 2t+8, 2t+9} of the
// first <- elements 0..3, of the second <- elements 4..7; the same permutation on both operands
// leaves the sum unchanged).
//
// A block owns 16 * RT consecutive rows of W (columns of y); its warps split K and add their
// partial sums in shared memory in warp order.  When W has too few rows to give every SM a block
// (N of a hidden size), K is also split over the `ksplit` blocks of a thread-block cluster, whose
// sums meet through distributed shared memory and are added in rank order.  The split depends on
// the shape alone, so a result does not depend on the batch or the grid.
//
// Fused output (`swiglu` = 1): W is the gate/up matrix with rows interleaved in eights - rows 16 b .. 16 b + 7
// are gate rows 8 b .. 8 b + 7 and rows 16 b + 8 .. 16 b + 15 the up rows of the same indices - so a thread
// that holds y[m][n] also holds y[m][n + 8] and writes silu(gate) * up to out[M, N / 2] directly
// (the reference's k_silu_mul, src/qwen_kernels.cu:102-105, without the round trip through memory).
#include "common.cuh"

#ifdef KVB_TRACE
#define SKINNY_TRACE(i) if (N == KVB_TRACE_N) { TRACE(i) }     // debug builds: the product with this many outputs
#else
#define SKINNY_TRACE(i)
#endif

namespace skinny {

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Weights: read once a step - kept out of L1 and marked as the first to leave L2.
__device__ __forceinline__ uint4 ld_stream(const void* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    return v;
}

constexpr int BLOCKS_WANTED = 148 * 2;

template <int RT, int NT, bool ACT, typename TOut>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          const float* __restrict__ bias, TOut* __restrict__ y, int M,
                                                          int N, int K, int x_stride, int ksplit) {
    SKINNY_TRACE(0)
    if (ksplit > 1) cluster_arrive_started();
    extern __shared__ __align__(16) float red[];          // [warps + ksplit][RT][NT][32 lanes][4]
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int rank = blockIdx.x % ksplit;                  // the cluster spans x
    const int n0 = (blockIdx.x / ksplit) * 16 * RT;
    const int kblocks = K / 32;                            // K is a multiple of 32 (checked by the launcher)
    const int per_block = (kblocks + ksplit - 1) / ksplit;
    const int block_begin = min(kblocks, rank * per_block), block_end = min(kblocks, block_begin + per_block);
    const int per_warp = (block_end - block_begin + warps - 1) / warps;
    const int kb_begin = min(block_end, block_begin + warp * per_warp), kb_end = min(block_end, kb_begin + per_warp);

    // Row pointers: W rows n0 + 16 r + g and + 8 (clamped; rows beyond N are never stored), x rows 8 j + g.
    const bf16* wrow[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        wrow[r][0] = w + (size_t)min(N - 1, n0 + 16 * r + g) * K + 8 * t;
        wrow[r][1] = w + (size_t)min(N - 1, n0 + 16 * r + g + 8) * K + 8 * t;
    }
    // NBUF register buffers of U k-blocks each.  The weights of all of them are requested before the wait for the
    // kernel that makes x (they do not depend on it); after it, a buffer is refilled as soon as its products are
    // issued, so that a warp's share of K costs one trip to memory plus its streaming.  (An L2 prefetch of the rest
    // of the share was measured slower than none.)
    uint64_t w_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(w_policy));
    constexpr int U = (RT * NT >= 4) ? 1 : 2;
    constexpr int NBUF = (RT * NT == 1) ? 3 : 2;        // measured: three beat two and four for the narrowest tiles
    auto load_w = [&](uint4 (&a)[U][RT][2], int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool live = kb + u < kb_end;
            const int k = (live ? kb + u : kb) * 32;
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                a[u][r][0] = live ? ld_stream(wrow[r][0] + k, w_policy) : make_uint4(0, 0, 0, 0);
                a[u][r][1] = live ? ld_stream(wrow[r][1] + k, w_policy) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    uint4 a[NBUF][U][RT][2], bx[NBUF][U][NT];
#pragma unroll
    for (int nb = 0; nb < NBUF; ++nb)
        if (kb_begin + nb * U < kb_end) load_w(a[nb], kb_begin + nb * U);
    SKINNY_TRACE(1)
    pdl_wait();
    pdl_launch_dependents();
    SKINNY_TRACE(2)

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[r][j][0] = acc[r][j][1] = acc[r][j][2] = acc[r][j][3] = 0.f;

    const bf16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        xok[j] = 8 * j + g < M;
        xrow[j] = x + (size_t)(xok[j] ? 8 * j + g : 0) * x_stride + 8 * t;
    }
    auto load_x = [&](uint4 (&b)[U][NT], int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool live = kb + u < kb_end;
            const int k = (live ? kb + u : kb) * 32;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (live && xok[j]) {
                    b[u][j] = __ldg(reinterpret_cast<const uint4*>(xrow[j] + k));
                } else {
                    b[u][j] = make_uint4(0, 0, 0, 0);
                }
            }
        }
    };
    auto multiply = [&](const uint4 (&a)[U][RT][2], const uint4 (&b)[U][NT]) {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16(acc[r][j], a[u][r][0].x, a[u][r][1].x, a[u][r][0].y, a[u][r][1].y, b[u][j].x, b[u][j].y);
                    mma_bf16(acc[r][j], a[u][r][0].z, a[u][r][1].z, a[u][r][0].w, a[u][r][1].w, b[u][j].z, b[u][j].w);
                }
    };
#pragma unroll
    for (int nb = 0; nb < NBUF; ++nb)
        if (kb_begin + nb * U < kb_end) load_x(bx[nb], kb_begin + nb * U);
    for (int base = kb_begin; base < kb_end; base += NBUF * U) {
#pragma unroll
        for (int nb = 0; nb < NBUF; ++nb) {
            const int kb = base + nb * U;
            if (kb < kb_end) {
                multiply(a[nb], bx[nb]);
                if (kb + NBUF * U < kb_end) { load_w(a[nb], kb + NBUF * U); load_x(bx[nb], kb + NBUF * U); }
            }
        }
    }

    SKINNY_TRACE(3)
    // Partial sums of the warps meet in shared memory and are added in warp order.
    float4* mine = reinterpret_cast<float4*>(red) + ((size_t)warp * RT * NT) * 32 + lane;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) mine[(r * NT + j) * 32] = make_float4(acc[r][j][0], acc[r][j][1], acc[r][j][2], acc[r][j][3]);
    __syncthreads();
    // With a cluster, block `rank` finishes the fragments idx = rank, rank + ksplit, ...: every block sends its own
    // sums of those fragments into the finishing block's shared memory (slot `rank` of `recv`), one cluster barrier
    // makes them visible, and nobody reads another block's memory after it - so a block may leave at once.
    constexpr int F = RT * NT * 32;
    float4* recv = reinterpret_cast<float4*>(red) + (size_t)warps * F;                 // [ksplit][F]
    if (ksplit > 1) {
        cluster_wait_started();
        for (int idx = threadIdx.x; idx < F; idx += blockDim.x) {
            float4 s = reinterpret_cast<const float4*>(red)[idx];
            for (int wi = 1; wi < warps; ++wi) {
                const float4 v = reinterpret_cast<const float4*>(red)[(size_t)wi * F + idx];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            peer_st4(peer_smem(recv + (size_t)rank * F + idx, idx % ksplit), s);
        }
        cluster_sync_all();
    }
    for (int idx = threadIdx.x * ksplit + rank; idx < F; idx += blockDim.x * ksplit) {
        float4 s;
        if (ksplit > 1) {
            s = recv[idx];
            for (int r = 1; r < ksplit; ++r) {
                const float4 v = recv[(size_t)r * F + idx];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
        } else {
            s = reinterpret_cast<const float4*>(red)[idx];
            for (int wi = 1; wi < warps; ++wi) {
                const float4 v = reinterpret_cast<const float4*>(red)[(size_t)wi * F + idx];
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
        }
        // idx = (r * NT + j) * 32 + lane'; the fragment holds y[m = 8 j + 2 t' (+1)][n = n0 + 16 r + g' (+8)].
        const int l2 = idx & 31, rj = idx >> 5, r = rj / NT, j = rj - r * NT, g2 = l2 >> 2, t2 = l2 & 3;
        const int m = 8 * j + 2 * t2, n = n0 + 16 * r + g2;
        const float vals[4] = {s.x, s.y, s.z, s.w};       // (n, m), (n, m + 1), (n + 8, m), (n + 8, m + 1)
        if (ACT) {
            // n is a gate row, n + 8 the up row of the same index i = n / 16 * 8 + n % 16.
            const int i = (n >> 4) * 8 + g2, I = N >> 1;
            if (n + 8 < N) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float gate = vals[e], up = vals[e + 2];
                    if (m + e < M) y[(size_t)(m + e) * I + i] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int nn = n + 8 * (e >> 1), mm = m + (e & 1);
                if (nn < N && mm < M) y[(size_t)mm * N + nn] = from_f32<TOut>(vals[e] + (bias ? bias[nn] : 0.f));
            }
        }
    }
    SKINNY_TRACE(4)
}

// How K is split over a cluster and over a block's warps.  It depends on the weight's shape alone - not on the
// number of rows of x, nor on how many row tiles a block takes - so that a row's sums are added in the same
// order whatever the batch.
struct Split {
    int ksplit, warps;
};
static inline Split choose_split(int N, int kblocks) {
    const int blocks = (N + 15) / 16;
    // K over a cluster while that still leaves blocks wanted and every warp of a block something to do.
    Split s{1, 4};
    while (s.ksplit < 8 && blocks * s.ksplit * 2 <= BLOCKS_WANTED && kblocks / (s.ksplit * 2) >= 4) s.ksplit *= 2;
    // Warps split a block's share of K: enough of them to keep loads in flight, not so many that a warp has nothing to do.
    s.warps = kblocks / s.ksplit >= 32 ? 8 : 4;
    return s;
}

// Whether all blocks of this shape are on the SMs at once (no second wave that costs a block's whole latency again).
template <int RT, int NT, bool ACT, typename TOut>
bool resident(int N, int K) {
    const int blocks = (N + 16 * RT - 1) / (16 * RT);
    const Split s = choose_split(N, K / 32);
    static int per_sm[2] = {-1, -1}, sm_count = 0;             // per block size: 4 or 8 warps
    int& cached = per_sm[s.warps == 8];
    if (cached < 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        const size_t smem = (size_t)(s.warps + s.ksplit) * RT * NT * 32 * 4 * sizeof(float);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached, gemm_skinny_kernel<RT, NT, ACT, TOut>, s.warps * 32, smem) != cudaSuccess)
            cached = 1;
    }
    return (long long)blocks * s.ksplit <= (long long)cached * sm_count;
}

template <int RT, int NT, bool ACT, typename TOut>
int launch(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, cudaStream_t stream) {
    const int blocks = (N + 16 * RT - 1) / (16 * RT);
    const Split s = choose_split(N, K / 32);
    const int ksplit = s.ksplit, warps = s.warps;
    const size_t smem = (size_t)(warps + ksplit) * RT * NT * 32 * 4 * sizeof(float);
    auto kernel = gemm_skinny_kernel<RT, NT, ACT, TOut>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (ksplit > 1)
        kvb_launch_cluster(kernel, dim3(blocks * ksplit), dim3(warps * 32), (unsigned)ksplit, smem, stream, x, w, bias, y, M, N,
                           K, x_stride, ksplit);
    else
        kvb_launch(kernel, dim3(blocks), dim3(warps * 32), smem, stream, x, w, bias, y, M, N, K, x_stride, ksplit);
    return kvb_launch_status();
}

// Rows of W per block: the fewest 16-row tiles with which every block is on the SMs at once; a weight too
// large for that (an output head over the vocabulary) is streamed in waves of two-tile blocks.
template <int NT, bool ACT, typename TOut>
int dispatch_rows(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, cudaStream_t stream) {
    if (resident<1, NT, ACT, TOut>(N, K)) return launch<1, NT, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    if (resident<2, NT, ACT, TOut>(N, K)) return launch<2, NT, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    if constexpr (NT <= 2) {
        if (resident<4, NT, ACT, TOut>(N, K)) return launch<4, NT, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    }
    return launch<2, NT, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
}

template <bool ACT, typename TOut>
int dispatch(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, cudaStream_t stream) {
    if (M <= 8) return dispatch_rows<1, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    if (M <= 16) return dispatch_rows<2, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    if (M <= 32) return dispatch_rows<4, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
    return dispatch_rows<8, ACT, TOut>(x, w, bias, y, M, N, K, x_stride, stream);
}

}  // namespace skinny

// x: [M, K] bfloat16; w: [N, K] bfloat16; bias: float32 [N] or null; y: [M, N] bfloat16 (out_dtype 1) or float32
// (out_dtype 0) - or, with swiglu = 1, [M, N / 2] from interleaved gate/up rows (N a multiple of 16, no bias).
// Refuses M > 64, K not a multiple of 32, misaligned operands.
KVB_API int kvb_gemm_skinny(int out_dtype, int act, const void* x, const void* w, const float* bias, void* y, int M,
                            int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (M > 64 || K <= 0 || K % 32 != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return KVB_ERR_ALIGN;
    const bf16* xb = (const bf16*)x;
    const bf16* wb = (const bf16*)w;
    if (act && (N % 16 != 0 || bias != nullptr)) return KVB_ERR_SHAPE;
    const int x_stride = K;
    if (out_dtype == KVB_BF16)
        return act ? skinny::dispatch<true, bf16>(xb, wb, bias, (bf16*)y, M, N, K, x_stride, stream)
                   : skinny::dispatch<false, bf16>(xb, wb, bias, (bf16*)y, M, N, K, x_stride, stream);
    if (out_dtype == KVB_F32)
        return act ? skinny::dispatch<true, float>(xb, wb, bias, (float*)y, M, N, K, x_stride, stream)
                   : skinny::dispatch<false, float>(xb, wb, bias, (float*)y, M, N, K, x_stride, stream);
    return KVB_ERR_DTYPE;
}
