// y[M, N] = x[M, K] . W[N, K]^T for a few dozen to a few hundred rows (16 < M <= 128): the matrix products of
// larger decode batches and of short portions of prompts, where the weights are still read about once from HBM
// per product and the activations are small.
//
// The reference runs them through cublasGemmEx (apps/qwen_serve.cu:27-39).  Here the roles of the tcgen05
// operands are swapped against the large-M kernel (gemm_tcgen05.cu): 128 rows of W are the MMA's A operand and
// fill the 128 lanes of tensor memory, the M rows of x (padded to MB, a multiple of 16) are its B operand and
// the accumulator's columns - so a block streams its 128 x K slab of W exactly once, whatever M is, and x
// (MB x 64 per K block) rides along.  Weights with few rows (N of a hidden size) would give too few blocks, so
// K is also split over the `ksplit` blocks of a thread-block cluster: block r multiplies K blocks r, r + ksplit,
// ..., sends each quarter-column group of its float32 partial tile to the block that finishes it (distributed
// shared memory, one cluster barrier), and every block adds what it received in rank order - the result does
// not depend on timing - applies bias or the gated activation and stores its share of y.
//
//   warp 0    one lane issues the TMA loads (W tile 128 x 64, x tile MB x 64, 128-byte swizzle) into a ring of stages;
//   warp 1    allocates tensor memory; one lane issues the tcgen05.mma and commits stages and the accumulator;
//   warps 2-5 read the accumulator (thread = row of W), send or store.
// Every mbarrier wait is bounded; on a timeout the error word is set and the block winds down (it still joins
// the cluster's barrier).  Gated output (`swiglu`): W holds gate and up rows interleaved in eights, so that the
// thread of gate row n finds the up value eight lanes further.
#include "tc_common.cuh"

namespace ws {
using namespace tc;

constexpr int BN = 128, BK = 64;                  // rows of W and elements of K per stage
constexpr int W_BYTES = BN * BK * 2;
constexpr int THREADS = 192;
constexpr int MAX_SPLIT = 16;                     // above 8 a cluster is "non-portable"; with two blocks a SM fourteen such clusters fit

template <int STAGES>
struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t accum_full;
    uint32_t tmem_base;
    int failed;
};

struct Params {
    const float* bias;
    void* y;
    int M, N, K, ksplit;
    int* err;
};

// MB: rows of x the accumulator holds (32, 64 or 128).
template <int MB, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, MB <= 64 ? 2 : 1)
gemm_wstream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ Params p) {
    constexpr int X_BYTES = MB * BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    // A block has few K blocks; small stages let two blocks share an SM and leave room for the next kernel's blocks,
    // which request their weights while this one runs (deeper rings with one block a SM were measured slower).
    constexpr int STAGES = 3;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float4* recv = reinterpret_cast<float4*>(tiles + STAGES * STAGE_BYTES);    // [ksplit][groups per block][128] float4
    __shared__ Shared<STAGES> sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksplit = p.ksplit;
    const int rank = blockIdx.x % ksplit;                                       // the cluster spans x
    const int n0 = (blockIdx.x / ksplit) * BN;
    const int kblocks = (p.K + BK - 1) / BK;
    const int my_kblocks = rank < kblocks ? (kblocks - rank + ksplit - 1) / ksplit : 0;   // K blocks rank, rank + ksplit, ...
    if (ksplit > 1) cluster_arrive_started();

    // The first thread makes the barriers and at once sends for the first stages' W tiles - they depend neither on
    // the kernel before this one nor on the tensor memory that warp 1 allocates meanwhile.
    const int early = my_kblocks < STAGES ? my_kblocks : STAGES;
    // W is read once a step: first to leave L2, so that what is read again soon (the cache of a few requests,
    // activations) stays there.  Measured with the output head of a one-request step: 642 -> 630 us a step.
    const uint64_t w_policy = l2_evict_first_policy();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.accum_full, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (int i = 0; i < early; ++i) {
            mbar_expect_tx(&sh.full[i], STAGE_BYTES);                          // W and x tile of the stage
            tma_load_2d_hint(tiles + i * STAGE_BYTES, &map_w, (rank + i * ksplit) * BK, n0, &sh.full[i], w_policy);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "r"(MB) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(tiles + i * STAGE_BYTES + W_BYTES, &map_x, (rank + i * ksplit) * BK, 0, &sh.full[i]);
            bool ok = true;
            for (int i = early; i < my_kblocks && ok; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&sh.empty[s], ((i / STAGES) - 1) & 1)) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                mbar_expect_tx(&sh.full[s], STAGE_BYTES);
                tma_load_2d_hint(tiles + s * STAGE_BYTES, &map_w, (rank + i * ksplit) * BK, n0, &sh.full[s], w_policy);
                tma_load_2d(tiles + s * STAGE_BYTES + W_BYTES, &map_x, (rank + i * ksplit) * BK, 0, &sh.full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN, MB);
            bool ok = true;
            for (int i = 0; i < my_kblocks && ok; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&sh.full[s], (i / STAGES) & 1)) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t w_addr = smem_u32(tiles + s * STAGE_BYTES), x_addr = w_addr + W_BYTES;
                const uint64_t adesc = smem_desc(w_addr), bdesc = smem_desc(x_addr);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma(tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
                umma_commit(&sh.empty[s]);
            }
            if (ok && my_kblocks > 0) umma_commit(&sh.accum_full);
        }
    }
    if (warp != 0) pdl_wait();                  // (warp 0's issuing lane has waited; its other lanes touch nothing)
    pdl_launch_dependents();

    // ---- epilogue: warps 2-5; thread = row n of W = lane of tensor memory ----
    // Column group j holds rows m = 4 j .. 4 j + 3 of x.  With a cluster, group j is finished by block j % ksplit,
    // at local index j / ksplit; there are GROUPS / ksplit (rounded up) local groups per block.
    constexpr int GROUPS = MB / 4;
    const int local_groups = (GROUPS + ksplit - 1) / ksplit;
    const int quarter = warp & 3;
    const int n = n0 + quarter * 32 + lane;
    bool have = false;
    float acc[MB];
    if (warp >= 2) {
        if (my_kblocks > 0) {
            have = mbar_wait(&sh.accum_full, 0);
            if (!have && lane == 0) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; }
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
        for (int c = 0; c < MB / 32; ++c) {
            uint32_t r[32];
            if (have) {
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c * 32, r);
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[c * 32 + e] = __uint_as_float(r[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[c * 32 + e] = 0.f;     // a rank without K blocks adds nothing
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    if (ksplit > 1) {
        cluster_wait_started();                 // every block of the cluster is running: its memory may be written
        if (warp >= 2) {
            const int row = quarter * 32 + lane;
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                const int owner = j % ksplit, jl = j / ksplit;
                peer_st4(peer_smem(recv + ((size_t)rank * local_groups + jl) * BN + row, owner),
                         make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
            }
        }
        cluster_sync_all();                     // what was sent has arrived; nobody touches another block's memory after this
    }
    if (warp >= 2) {
        const int row = quarter * 32 + lane;
        const float b = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
        TOut* y = reinterpret_cast<TOut*>(p.y);
        // Rows m = 4 j .. 4 j + 3 of x at column n: bias or gated activation, conversion, store.  Called by whole warps.
        auto finish = [&](int j, const float4& v) {
            const float vals[4] = {v.x, v.y, v.z, v.w};
            if (SWIGLU) {
                // n is a gate row if n % 16 < 8; its up row is n + 8, eight lanes further.
                const int I = p.N >> 1, i = (n >> 4) * 8 + (n & 7);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float up = __shfl_down_sync(0xffffffffu, vals[e], 8);
                    const int m = 4 * j + e;
                    if ((n & 15) < 8 && n + 8 < p.N && m < p.M)
                        y[(size_t)m * I + i] = from_f32<TOut>(vals[e] / (1.f + expf(-vals[e])) * up);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int m = 4 * j + e;
                    if (n < p.N && m < p.M) y[(size_t)m * p.N + n] = from_f32<TOut>(vals[e] + b);
                }
            }
        };
        if (ksplit > 1) {
            for (int jl = 0; jl < local_groups; ++jl) {
                const int j = jl * ksplit + rank;
                if (j >= GROUPS) break;
                float4 v = recv[(size_t)jl * BN + row];
                for (int r = 1; r < ksplit; ++r) {              // in rank order, whichever block was fastest
                    const float4 u = recv[((size_t)r * local_groups + jl) * BN + row];
                    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
                }
                finish(j, v);
            }
        } else {
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) finish(j, make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
        }
    }

    // Teardown.
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_wait(&sh.full[s], 0);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(MB) : "memory");
    }
}

// A [rows, cols] bfloat16 row-major matrix read in tiles of [box_rows, 64] with the 128-byte swizzle; rows and
// columns outside are zero-filled.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    return make_bf16_map(map, base, rows, cols, cols, box_rows);
}

static int sm_count() { return kvb_sm_count(); }

// K over a cluster while the grid stays within two blocks a SM and every block keeps a K block.  It depends on the
// weight's shape alone.
static int choose_split(int N, int K) {
    const int tiles = (N + BN - 1) / BN, kblocks = (K + BK - 1) / BK;
    int ksplit = 1;
    const int target = 2 * sm_count();
    while (ksplit < MAX_SPLIT && tiles * ksplit * 2 <= target && kblocks >= ksplit * 2) ksplit *= 2;
    return ksplit;
}

template <int MB, typename TOut, bool SWIGLU>
static int launch(const void* x, const void* w, const float* bias, void* y, int M, int N, int K, int* err, cudaStream_t stream) {
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, BN);
    if (rc != KVB_OK) return rc;
    rc = make_map(&mx, x, M, K, MB);
    if (rc != KVB_OK) return rc;
    constexpr int STAGES = 3;
    const int ksplit = choose_split(N, K);
    const int local_groups = (MB / 4 + ksplit - 1) / ksplit;
    const size_t smem = (size_t)STAGES * (W_BYTES + MB * BK * 2) + (ksplit > 1 ? (size_t)ksplit * local_groups * BN * 16 : 0) + 1024;
    auto kernel = gemm_wstream_kernel<MB, TOut, SWIGLU>;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    Params p{bias, y, M, N, K, ksplit, err};
    const int tiles = (N + BN - 1) / BN;
    if (ksplit > 1)
        kvb_launch_cluster(kernel, dim3(tiles * ksplit), dim3(THREADS), (unsigned)ksplit, smem, stream, mw, mx, p);
    else
        kvb_launch(kernel, dim3(tiles), dim3(THREADS), smem, stream, mw, mx, p);
    return kvb_launch_status();
}

template <typename TOut, bool SWIGLU>
static int dispatch(const void* x, const void* w, const float* bias, void* y, int M, int N, int K, int* err, cudaStream_t stream) {
    if (M <= 32) return launch<32, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
    if (M <= 64) return launch<64, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
    return launch<128, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
}

}  // namespace ws

// x [M, K], w [N, K] bfloat16 row-major; bias float32 [N] or null; y [M, N] bfloat16 (out_dtype 1) or float32 (0),
// or with swiglu = 1 [M, N / 2] from interleaved gate/up rows (N % 16 == 0, no bias).
// Refuses M > 128, K % 8 != 0 and operands that are not 16-byte aligned.
KVB_API int kvb_gemm_wstream(int out_dtype, int swiglu, const void* x, const void* w, const float* bias, void* y, int M,
                             int N, int K, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (M > 128 || K <= 0 || K % 8 != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return KVB_ERR_ALIGN;
    if (swiglu && (N % 16 != 0 || bias != nullptr)) return KVB_ERR_SHAPE;
    if (out_dtype == KVB_BF16)
        return swiglu ? ws::dispatch<bf16, true>(x, w, bias, y, M, N, K, err, stream)
                      : ws::dispatch<bf16, false>(x, w, bias, y, M, N, K, err, stream);
    if (out_dtype == KVB_F32)
        return swiglu ? ws::dispatch<float, true>(x, w, bias, y, M, N, K, err, stream)
                      : ws::dispatch<float, false>(x, w, bias, y, M, N, K, err, stream);
    return KVB_ERR_DTYPE;
}
