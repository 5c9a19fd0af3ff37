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
//
// Fused forms for the chain of a decode layer (each removes a kernel and a round trip through memory from the chain):
//  * PRE: the rows of x are the residual stream rounded to bfloat16, not yet normalised.  The kernel multiplies
//    them by the norm's weight as it loads them, sums their squares, and scales its sums by rsqrt(mean + eps) at
//    the end - RMSNorm (src/qwen_kernels.cu:26-40 of the reference) folded into the product that follows it:
//    norm(x) . W^T = (x * w) . W^T * inv.  The squares travel with the partial sums through the same fixed-order
//    reductions.
//  * EPI_RESID: the product's result is not stored but added to the float32 residual stream h, whose new value is
//    also written rounded to bfloat16 (the next product's x) - k_add (src/qwen_kernels.cu:55-61) folded in.
//  * EPI_ROPE: the product is the q/k/v projection, with W's rows (and the bias) permuted at load time so that a
//    thread's two rows n and n + 8 are the dimensions d and d + D / 2 of one head: the thread adds the biases, rotates
//    the pair by the row's position, and writes queries to their buffer and keys and values straight into their
//    cache pages (k_add_bias, k_rope_pos and k_batched_write_kv of the reference, src/qwen_kernels.cu:45-53,
//    :253-290, folded in).
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

static inline int blocks_wanted() { return 2 * kvb_sm_count(); }     // two blocks an SM

enum { EPI_PLAIN = 0, EPI_ACT = 1, EPI_RESID = 2, EPI_ROPE = 3 };

// What the fused forms need beyond x, W, bias and y.
struct Fused {
    const float* norm_w;      // PRE: the norm's weight [K]
    float eps;
    float* h;                 // EPI_RESID: residual stream [M, N] float32, updated in place
    bf16* hb;                 // EPI_RESID: its new value rounded to bfloat16 [M, N]
    // EPI_ROPE
    const float* cos_t;       // [table_len, D / 2] or nullptr (no rotation)
    const float* sin_t;
    const int* positions;     // [M]
    const int* row_segment;   // [M]
    const int* block_table;   // [segments, table_stride]
    bf16* k_pages;            // [pages, Hkv, page, D]
    bf16* v_pages;
    bf16* q_out;              // [M, Hq * D]
    int* err;
    int table_len, table_stride, Hq, Hkv, D, page_size, page_shift, writes;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t raw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[i]));
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        raw[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(raw[0], raw[1], raw[2], raw[3]);
}

// One 16-row tile per block: the blocks of the widest products (the gate/up projection) are all on the SMs at once only
// with five blocks of four warps per SM, that is within 96 registers a thread.
template <int RT, int NT, int EPI, bool PRE, typename TOut>
__global__ void __maxnreg__((RT == 1 && NT <= 2) ? 96 : 255) gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          const float* __restrict__ bias, TOut* __restrict__ y, int M,
                                                          int N, int K, int x_stride, int ksplit,
                                                          const __grid_constant__ Fused fz) {
    SKINNY_TRACE(0)
    if (ksplit > 1) cluster_arrive_started();
    extern __shared__ __align__(16) float red[];          // [warps + ksplit][RT][NT][32 lanes][4]; PRE: then sums of squares and the norm's weight
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
    constexpr int F = RT * NT * 32;                        // fragments (float4) of a block's tile
    float* ssq_s = red + (size_t)(warps + ksplit) * F * 4;                             // PRE: [warps][16], then [ksplit][16]
    float* nw_s = ssq_s + (warps + ksplit) * 16;                                       // PRE: the norm's weight [K]
    if (PRE) {                                             // no kernel writes the norm's weight: fetched before the wait
        for (int i = threadIdx.x * 4; i < K; i += blockDim.x * 4)
            *reinterpret_cast<float4*>(nw_s + i) = __ldg(reinterpret_cast<const float4*>(fz.norm_w + i));
    }
    // What the first fragment this thread finishes will need beyond the sums, none of it made by the kernel before:
    // the elements of the residual stream it updates (last written three kernels ago), or the positions, angles,
    // biases and pages of its rows (the step's metadata).  Asked for now, in registers by the time they are wanted.
    const int first_idx = threadIdx.x * ksplit + rank;
    float h_first[4] = {0.f, 0.f, 0.f, 0.f};
    int pos_first[2] = {0, 0}, page_first[2] = {-1, -1};
    float cs_first[2] = {1.f, 1.f}, sn_first[2] = {0.f, 0.f};
    if ((EPI == EPI_RESID || EPI == EPI_ROPE) && first_idx < F) {
        const int l2 = first_idx & 31, rj = first_idx >> 5, r = rj / NT, j = rj - r * NT;
        const int m = 8 * j + 2 * (l2 & 3), n = n0 + 16 * r + (l2 >> 2);
        if (EPI == EPI_RESID) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int nn = n + 8 * (e >> 1), mm = m + (e & 1);
                if (nn < N && mm < M) h_first[e] = fz.h[(size_t)mm * N + nn];
            }
        } else {
            const int head = n / fz.D, d = ((n - head * fz.D) >> 4) * 8 + (l2 >> 2);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (m + e >= M || n + 8 >= N) continue;
                const int pos = fz.positions[m + e];
                pos_first[e] = pos;
                if (head < fz.Hq + fz.Hkv && fz.cos_t && pos < fz.table_len) {
                    cs_first[e] = fz.cos_t[(size_t)pos * (fz.D >> 1) + d];
                    sn_first[e] = fz.sin_t[(size_t)pos * (fz.D >> 1) + d];
                }
                if (head >= fz.Hq) page_first[e] = fz.block_table[(size_t)fz.row_segment[m + e] * fz.table_stride + (pos >> fz.page_shift)];
            }
        }
    }
    SKINNY_TRACE(1)
    pdl_wait();
    pdl_launch_dependents();
    if (PRE) __syncthreads();
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
    float ssq[NT];                                         // PRE: this thread's share of the rows' sums of squares
#pragma unroll
    for (int j = 0; j < NT; ++j) ssq[j] = 0.f;
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
    // PRE: the rows as they arrived are squared and summed, multiplied by the norm's weight and rounded again, just
    // before they are used (so that the loads stay in flight meanwhile).
    auto fold_norm = [&](uint4 (&b)[U][NT], int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = min(kb + u, kb_end - 1) * 32 + 8 * t;
            const float4 nw0 = *reinterpret_cast<const float4*>(nw_s + k), nw1 = *reinterpret_cast<const float4*>(nw_s + k + 4);
            const float nw[8] = {nw0.x, nw0.y, nw0.z, nw0.w, nw1.x, nw1.y, nw1.z, nw1.w};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float f[8];
                unpack8(b[u][j], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    ssq[j] += f[e] * f[e];
                    f[e] *= nw[e];
                }
                b[u][j] = pack8(f);
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
                if (PRE) fold_norm(bx[nb], kb);
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
    if (PRE) {
        // A row's squares lie with the four threads of its group, the warps of the block and the blocks of the cluster:
        // added in that order, each in a fixed order.
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            ssq[j] += __shfl_xor_sync(0xffffffffu, ssq[j], 1);
            ssq[j] += __shfl_xor_sync(0xffffffffu, ssq[j], 2);
            if (t == 0) ssq_s[warp * 16 + 8 * j + g] = ssq[j];
        }
        if (NT == 1 && t == 0) ssq_s[warp * 16 + 8 + g] = 0.f;
    }
    __syncthreads();
    // With a cluster, block `rank` finishes the fragments idx = rank, rank + ksplit, ...: every block sends its own
    // sums of those fragments into the finishing block's shared memory (slot `rank` of `recv`), one cluster barrier
    // makes them visible, and nobody reads another block's memory after it - so a block may leave at once.
    float4* recv = reinterpret_cast<float4*>(red) + (size_t)warps * F;                 // [ksplit][F]
    float* recv_ssq = ssq_s + warps * 16;                                              // [ksplit][16]
    if (ksplit > 1) {
        cluster_wait_started();
        if (PRE && threadIdx.x < 16) {                     // this block's sums of squares, to every block of the cluster
            float s = ssq_s[threadIdx.x];
            for (int wi = 1; wi < warps; ++wi) s += ssq_s[wi * 16 + threadIdx.x];
            for (int r = 0; r < ksplit; ++r) {
                const uint32_t at = peer_smem(recv_ssq + rank * 16 + threadIdx.x, r);
                asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at), "f"(s) : "memory");
            }
        }
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
        float vals[4] = {s.x, s.y, s.z, s.w};             // (n, m), (n, m + 1), (n + 8, m), (n + 8, m + 1)
        if (PRE) {
            // rsqrt(mean of squares + eps) of rows m and m + 1, as the norm kernel computes it.
            float inv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float total;
                if (ksplit > 1) {
                    total = recv_ssq[m + e];
                    for (int rr = 1; rr < ksplit; ++rr) total += recv_ssq[rr * 16 + m + e];
                } else {
                    total = ssq_s[m + e];
                    for (int wi = 1; wi < warps; ++wi) total += ssq_s[wi * 16 + m + e];
                }
                inv[e] = 1.f / sqrtf(total / (float)K + fz.eps);
            }
            vals[0] *= inv[0]; vals[1] *= inv[1]; vals[2] *= inv[0]; vals[3] *= inv[1];
        }
        if (EPI == EPI_ACT) {
            // n is a gate row, n + 8 the up row of the same index i = n / 16 * 8 + n % 16.
            const int i = (n >> 4) * 8 + g2, I = N >> 1;
            if (n + 8 < N) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float gate = vals[e], up = vals[e + 2];
                    if (m + e < M) y[(size_t)(m + e) * I + i] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
                }
            }
        } else if (EPI == EPI_RESID) {
            float hv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {                  // all four loads before the first store
                const int nn = n + 8 * (e >> 1), mm = m + (e & 1);
                hv[e] = idx == first_idx ? h_first[e] : ((nn < N && mm < M) ? fz.h[(size_t)mm * N + nn] : 0.f);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int nn = n + 8 * (e >> 1), mm = m + (e & 1);
                if (nn < N && mm < M) {
                    const size_t at = (size_t)mm * N + nn;
                    const float v = hv[e] + vals[e] + (bias ? bias[nn] : 0.f);
                    fz.h[at] = v;
                    fz.hb[at] = __float2bfloat16_rn(v);
                }
            }
        } else if (EPI == EPI_ROPE) {
            // Rows n and n + 8 of the permuted W are dimensions d and d + D / 2 of head n / D.
            const int D = fz.D, half = D >> 1;
            const int head = n / D, d = ((n - head * D) >> 4) * 8 + g2;
            if (n + 8 < N && head < fz.Hq + 2 * fz.Hkv) {
                const float b_lo = bias ? bias[n] : 0.f, b_hi = bias ? bias[n + 8] : 0.f;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int mm = m + e;
                    if (mm >= M) continue;
                    const float lo = vals[e] + b_lo, hi = vals[e + 2] + b_hi;
                    const bool ahead = idx == first_idx;                   // fetched before the wait
                    const int pos = ahead ? pos_first[e] : fz.positions[mm];
                    float out_lo = lo, out_hi = hi;
                    if (head < fz.Hq + fz.Hkv && fz.cos_t) {
                        if (pos < fz.table_len) {
                            const float c = ahead ? cs_first[e] : fz.cos_t[(size_t)pos * half + d];
                            const float sn = ahead ? sn_first[e] : fz.sin_t[(size_t)pos * half + d];
                            out_lo = lo * c - hi * sn;
                            out_hi = hi * c + lo * sn;
                        } else {
                            atomicOr(fz.err, KVB_DEV_BAD_POS);
                        }
                    }
                    if (head < fz.Hq) {
                        bf16* q = fz.q_out + ((size_t)mm * fz.Hq + head) * D;
                        q[d] = __float2bfloat16_rn(out_lo);
                        q[d + half] = __float2bfloat16_rn(out_hi);
                    } else if (fz.writes) {
                        const bool is_k = head < fz.Hq + fz.Hkv;
                        const int hk = head - fz.Hq - (is_k ? 0 : fz.Hkv);
                        const int page = ahead ? page_first[e]
                                               : fz.block_table[(size_t)fz.row_segment[mm] * fz.table_stride + (pos >> fz.page_shift)];
                        if (page < 0) {
                            atomicOr(fz.err, KVB_DEV_BAD_PAGE);
                        } else {
                            bf16* dst = (is_k ? fz.k_pages : fz.v_pages) +
                                        (((size_t)page * fz.Hkv + hk) * fz.page_size + (pos & (fz.page_size - 1))) * D;
                            dst[d] = __float2bfloat16_rn(out_lo);
                            dst[d + half] = __float2bfloat16_rn(out_hi);
                        }
                    }
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
    while (s.ksplit < 8 && blocks * s.ksplit * 2 <= blocks_wanted() && kblocks / (s.ksplit * 2) >= 4) s.ksplit *= 2;
    // Warps split a block's share of K: enough of them to keep loads in flight, not so many that a warp has nothing to do.
    s.warps = kblocks / s.ksplit >= 32 ? 8 : 4;
    return s;
}

static inline size_t smem_bytes(const Split& s, int RT, int NT, bool pre, int K) {
    return (size_t)(s.warps + s.ksplit) * RT * NT * 32 * 4 * sizeof(float) +
           (pre ? ((size_t)(s.warps + s.ksplit) * 16 + K) * sizeof(float) : 0);
}

// Whether all blocks of this shape are on the SMs at once (no second wave that costs a block's whole latency again).
template <int RT, int NT, int EPI, bool PRE, typename TOut>
bool resident(int N, int K) {
    const int blocks = (N + 16 * RT - 1) / (16 * RT);
    const Split s = choose_split(N, K / 32);
    static int per_sm[2] = {-1, -1}, sm_count = 0;             // per block size: 4 or 8 warps
    int& cached = per_sm[s.warps == 8];
    if (cached < 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached, gemm_skinny_kernel<RT, NT, EPI, PRE, TOut>, s.warps * 32,
                                                          smem_bytes(s, RT, NT, PRE, K)) != cudaSuccess)
            cached = 1;
    }
    return (long long)blocks * s.ksplit <= (long long)cached * sm_count;
}

template <int RT, int NT, int EPI, bool PRE, typename TOut>
int launch(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, const Fused& fz,
           cudaStream_t stream) {
    const int blocks = (N + 16 * RT - 1) / (16 * RT);
    const Split s = choose_split(N, K / 32);
    const int ksplit = s.ksplit, warps = s.warps;
    const size_t smem = smem_bytes(s, RT, NT, PRE, K);
    auto kernel = gemm_skinny_kernel<RT, NT, EPI, PRE, TOut>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (ksplit > 1)
        kvb_launch_cluster(kernel, dim3(blocks * ksplit), dim3(warps * 32), (unsigned)ksplit, smem, stream, x, w, bias, y, M, N,
                           K, x_stride, ksplit, fz);
    else
        kvb_launch(kernel, dim3(blocks), dim3(warps * 32), smem, stream, x, w, bias, y, M, N, K, x_stride, ksplit, fz);
    return kvb_launch_status();
}

// Rows of W per block: the fewest 16-row tiles with which every block is on the SMs at once; a weight too
// large for that (an output head over the vocabulary) is streamed in waves of two-tile blocks.
template <int NT, int EPI, bool PRE, typename TOut>
int dispatch_rows(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, const Fused& fz,
                  cudaStream_t stream) {
    if (resident<1, NT, EPI, PRE, TOut>(N, K)) return launch<1, NT, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    if (resident<2, NT, EPI, PRE, TOut>(N, K)) return launch<2, NT, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    if constexpr (NT <= 2) {
        if (resident<4, NT, EPI, PRE, TOut>(N, K)) return launch<4, NT, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    }
    return launch<2, NT, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
}

template <int EPI, bool PRE, typename TOut>
int dispatch(const bf16* x, const bf16* w, const float* bias, TOut* y, int M, int N, int K, int x_stride, const Fused& fz,
             cudaStream_t stream) {
    if (M <= 8) return dispatch_rows<1, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    if (M <= 16) return dispatch_rows<2, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    if constexpr (EPI <= EPI_ACT && !PRE) {                // the fused forms serve decode steps of up to 16 rows
        if (M <= 32) return dispatch_rows<4, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
        return dispatch_rows<8, EPI, PRE, TOut>(x, w, bias, y, M, N, K, x_stride, fz, stream);
    }
    return KVB_ERR_SHAPE;
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
    const skinny::Fused none = {};
    using namespace skinny;
    if (out_dtype == KVB_BF16)
        return act ? dispatch<EPI_ACT, false, bf16>(xb, wb, bias, (bf16*)y, M, N, K, x_stride, none, stream)
                   : dispatch<EPI_PLAIN, false, bf16>(xb, wb, bias, (bf16*)y, M, N, K, x_stride, none, stream);
    if (out_dtype == KVB_F32)
        return act ? dispatch<EPI_ACT, false, float>(xb, wb, bias, (float*)y, M, N, K, x_stride, none, stream)
                   : dispatch<EPI_PLAIN, false, float>(xb, wb, bias, (float*)y, M, N, K, x_stride, none, stream);
    return KVB_ERR_DTYPE;
}

// The fused forms (M <= 16, bfloat16 throughout).  `x` holds rows of the residual stream rounded to bfloat16 where
// `norm_w` is given: the kernel applies RMSNorm(norm_w, eps) to them on the way in.
//
// kvb_gemm_skinny_norm_act: out[M, N / 2] = silu(g) * u with [g | u] = norm(x) . W^T, W's gate and up rows interleaved
// in eights.
KVB_API int kvb_gemm_skinny_norm_act(const void* x, const void* w, const float* norm_w, float eps, void* out, int M, int N,
                                     int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (M > 16 || K <= 0 || K % 32 != 0 || N % 16 != 0 || !norm_w) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)norm_w) & 15) return KVB_ERR_ALIGN;
    skinny::Fused fz = {};
    fz.norm_w = norm_w;
    fz.eps = eps;
    return skinny::dispatch<skinny::EPI_ACT, true, bf16>((const bf16*)x, (const bf16*)w, nullptr, (bf16*)out, M, N, K, K, fz, stream);
}

// kvb_gemm_skinny_residual: h[M, N] += x . W^T (+ bias); hb[M, N] = bfloat16(h).  No other output.
KVB_API int kvb_gemm_skinny_residual(const void* x, const void* w, const float* bias, float* h, void* hb, int M, int N, int K,
                                     cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (M > 16 || K <= 0 || K % 32 != 0 || !h || !hb) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return KVB_ERR_ALIGN;
    skinny::Fused fz = {};
    fz.h = h;
    fz.hb = (bf16*)hb;
    return skinny::dispatch<skinny::EPI_RESID, false, bf16>((const bf16*)x, (const bf16*)w, bias, (bf16*)nullptr, M, N, K, K, fz, stream);
}

// kvb_gemm_skinny_qkv: the q/k/v projection of norm(x) with bias, rotation and cache append.  W [(Hq + 2 Hkv) D, K] and
// bias have their rows permuted within each head: row 16 j + i (i < 8) of a head is its dimension 8 j + i, row
// 16 j + 8 + i its dimension D / 2 + 8 j + i.  cos_t / sin_t: [table_len, D / 2] or null (no rotation; the table must
// cover the whole head: a rotation of fewer dimensions is not this kernel's).  Queries go to q_out [M, Hq D] in their
// natural order; keys and values (if `writes`) into the pages the block table names for each row's position.
KVB_API int kvb_gemm_skinny_qkv(const void* x, const void* w, const float* bias, const float* norm_w, float eps,
                                const float* cos_t, const float* sin_t, int table_len, const int* positions,
                                const int* row_segment, const int* block_table, int table_stride, void* k_pages,
                                void* v_pages, void* q_out, int M, int K, int Hq, int Hkv, int D, int page_size, int writes,
                                int* err, cudaStream_t stream) {
    if (M <= 0) return KVB_OK;
    const int N = (Hq + 2 * Hkv) * D;
    if (M > 16 || K <= 0 || K % 32 != 0 || D % 16 != 0 || Hq < 1 || Hkv < 1 || !norm_w) return KVB_ERR_SHAPE;
    if (page_size < 1 || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)norm_w) & 15) return KVB_ERR_ALIGN;
    skinny::Fused fz = {};
    fz.norm_w = norm_w;
    fz.eps = eps;
    fz.cos_t = cos_t; fz.sin_t = sin_t; fz.table_len = table_len;
    fz.positions = positions; fz.row_segment = row_segment; fz.block_table = block_table; fz.table_stride = table_stride;
    fz.k_pages = (bf16*)k_pages; fz.v_pages = (bf16*)v_pages; fz.q_out = (bf16*)q_out; fz.err = err;
    fz.Hq = Hq; fz.Hkv = Hkv; fz.D = D; fz.page_size = page_size; fz.writes = writes;
    fz.page_shift = 0;
    while ((1 << fz.page_shift) < page_size) ++fz.page_shift;
    return skinny::dispatch<skinny::EPI_ROPE, true, bf16>((const bf16*)x, (const bf16*)w, bias, (bf16*)nullptr, M, N, K, K, fz, stream);
}
