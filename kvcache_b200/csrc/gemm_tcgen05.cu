// y[M, N] = x[M, K] . W[N, K]^T on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands brought into 128-byte-swizzled shared memory by TMA.
//
// This is the engine's matrix product for portions of prompts and larger decode batches; in the
// reference every linear layer is a cublasGemmEx call (apps/qwen_serve.cu:27-39).  A block walks
// over 128 x BN tiles of y (BN = 128 or 256), one block per SM:
//   warp 0    one lane issues the TMA loads of x and W tiles (128 x 64 and BN x 64 bfloat16) into a
//             ring of stages and arms each stage's "full" mbarrier with the bytes to expect;
//   warp 1    allocates two accumulators of BN columns in tensor memory; one lane waits for a stage, issues four
//             tcgen05.mma (K = 16 each) on shared-memory descriptors, and commits them to the stage's
//             "empty" mbarrier - and, after a tile's last K block, to that accumulator's "full" barrier;
//   warps 2-5 wait for an accumulator, read it with tcgen05.ld (each warp the 32 lanes it may
//             access), add the bias or apply the gated activation, convert and store, and hand the
//             accumulator back while the next tile's products already run into the other one.
// Rows and columns beyond M, N and K are zero-filled by TMA and masked at the store, so any size
// with K % 8 == 0 (the 16-byte stride rule of TMA) is taken.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the waiter sets the error word,
// and the block still waits (bounded) for the copies it issued, frees its tensor memory and returns.
//
// Gated output (`swiglu`): W holds gate and up rows interleaved in eights (see gemm_skinny.cu);
// the epilogue writes silu(gate) * up to out[M, N / 2] (src/qwen_kernels.cu:102-105).
#include "tc_common.cuh"

namespace tc {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int THREADS = 192;
#ifndef KVB_PAIR_KSUB
#define KVB_PAIR_KSUB 2
#endif
constexpr int PAIR_KSUB = KVB_PAIR_KSUB;                // sub-tiles of 64 along K in a stage of the two-SM kernel
constexpr int PAIR_STAGES = 6 / PAIR_KSUB;
// One thread's 32 consecutive accumulator columns (row m, columns n .. n + 31) on their way to memory: bias and
// conversion, or the gated activation on interleaved gate/up columns.
template <typename TOut, bool SWIGLU>
__device__ __forceinline__ void store_chunk(const uint32_t* r, const float* __restrict__ bias, TOut* __restrict__ y, int m,
                                            int n, int N) {
    if (SWIGLU) {
        // columns n .. n+7 gate, n+8 .. n+15 up, twice per 32: 16 outputs at column n / 2
        TOut* out = y + (size_t)m * (N >> 1) + (n >> 1);
        float v[16];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float gate = __uint_as_float(r[16 * blk + i]), up = __uint_as_float(r[16 * blk + 8 + i]);
                v[8 * blk + i] = __fdividef(gate, 1.f + __expf(-gate)) * up;
            }
        if (n + 32 <= N && sizeof(TOut) == 2 && (N & 15) == 0) {
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t*>(&p2);
            }
            reinterpret_cast<uint4*>(out)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(out)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (n + 16 * blk + 8 + i < N) out[8 * blk + i] = from_f32<TOut>(v[8 * blk + i]);
        }
    } else {
        TOut* out = y + (size_t)m * N + n;
        if (n + 32 <= N && sizeof(TOut) == 2 && (N & 7) == 0) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float a = __uint_as_float(r[2 * i]) + (bias ? __ldg(bias + n + 2 * i) : 0.f);
                const float bb = __uint_as_float(r[2 * i + 1]) + (bias ? __ldg(bias + n + 2 * i + 1) : 0.f);
                __nv_bfloat162 v2 = __floats2bfloat162_rn(a, bb);
                packed[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(out)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (n + i < N) out[i] = from_f32<TOut>(__uint_as_float(r[i]) + (bias ? __ldg(bias + n + i) : 0.f));
        }
    }
}

template <int STAGES>
struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_base;
    int failed;
};

// Persistent: a block walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the stage ring runs on across
// tiles, and two accumulators in tensor memory let the epilogue of one tile overlap the products of the next.
template <int BN, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const float* __restrict__ bias, TOut* __restrict__ y, int M, int N, int K, int* __restrict__ err) {
    constexpr int B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGES = BN == 256 ? 4 : 6;
    extern __shared__ unsigned char smem_raw[];
    // Tiles want 1024-byte alignment (the swizzle repeats every 8 rows of 128 bytes).
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ Shared<STAGES> sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_blocks = (M + BM - 1) / BM, n_blocks = (N + BN - 1) / BN;
    const int num_tiles = m_blocks * n_blocks;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.accum_full[b], 1); mbar_init(&sh.accum_empty[b], 4); }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {   // tensor memory: two accumulators of BN columns (128 lanes x 32 bits each)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_blocks) * BM, n0 = (tile / m_blocks) * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !mbar_wait(&sh.empty[s], (round - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    mbar_expect_tx(&sh.full[s], STAGE_BYTES);
                    tma_load_2d(tiles + s * STAGE_BYTES, &map_x, kb * BK, m0, &sh.full[s]);
                    tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &map_w, kb * BK, n0, &sh.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int b = local & 1;
                const uint32_t use = local >> 1;          // how often this accumulator has been used before
                if (use > 0 && !mbar_wait(&sh.accum_empty[b], (use - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem + b * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&sh.full[s], (it / STAGES) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)   // 16 elements = 32 bytes further along K: +2 in the address field
                        umma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&sh.empty[s]);          // the stage is free once these MMAs have read it
                }
                umma_commit(&sh.accum_full[b]);         // arrives when every MMA issued so far has finished
            }
        }
    } else {
        // Epilogue: warp w reads TMEM lanes 32 (w % 4) .. + 31, i.e. rows m0 + 32 (w % 4) + lane.
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int m0 = (tile % m_blocks) * BM, n0 = (tile / m_blocks) * BN;
            const int b = local & 1;
            const int m = m0 + quarter * 32 + lane;
            ok = mbar_wait(&sh.accum_full[b], (local >> 1) & 1);
            if (!ok) { if (lane == 0) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c * 32, r);
                const int n = n0 + c * 32;
                if (m >= M || n >= N) continue;
                store_chunk<TOut, SWIGLU>(r, bias, y, m, n, N);
            }
            // This warp has read its part of the accumulator: hand it back to the MMA warp.
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.accum_empty[b]);
        }
    }

    // Teardown.  If something ran out of patience, give the copies that were issued a bounded chance to land
    // before the shared memory goes back to the pool.
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_wait(&sh.full[s], 0);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------------------
// The same product with two SMs on one tile (tcgen05 cta_group::2).  A cluster of two blocks owns a 256 x 256
// tile of y: block r of the pair loads rows m0 + 128 r .. + 127 of x and rows n0 + 128 r .. + 127 of W, so each
// SM brings 32 KB per K block where two independent 128 x 256 tiles would bring 48 KB each - the operand traffic
// from L2, which bounds the one-SM kernel, drops by a third.  The even block of the pair (the leader) issues the
// MMAs for both; they read A from each block's own shared memory into that block's tensor memory and the two
// halves of B from both.  Barriers: "full" lives in the leader and counts the bytes of both blocks' TMA loads;
// "empty" and "accumulator full" are signalled in both blocks by multicast commits; "accumulator empty" lives in
// the leader and collects the epilogue warps of both blocks.
// ---------------------------------------------------------------------------------------------------------
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;     // a shared::cluster address with this bit cleared names the even block of the pair

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint64_t* leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(leader_bar) & PEER_BIT_MASK), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {      // arrives on the barrier at this offset in both blocks
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(smem_u32(bar) & PEER_BIT_MASK) : "memory");
}

template <int BN, typename TOut, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const float* __restrict__ bias, TOut* __restrict__ y, int M, int N, int K, int* __restrict__ err) {
    // BN columns of y a tile, 256 or a little fewer: the launcher takes the width whose last round of tiles wastes least.
    static_assert(BN % 32 == 0 && BN >= 128 && BN <= 256, "tile width");
    constexpr int HALF_N = BN / 2, ACC_STRIDE = 256;             // the two accumulators lie 256 columns apart whatever BN
    // A stage holds KSUB sub-tiles of 64 along K of each operand (the 128-byte swizzle takes no wider box): the thread that
    // issues the MMAs pays for a barrier wait and a commit - about 250 clocks - once a stage, and with 64 of K a stage that
    // was half as long again as the four MMAs themselves take (the tensor pipe was busy two thirds of the time).
    constexpr int KSUB = PAIR_KSUB;
    constexpr int B_BYTES = HALF_N * BK * 2, SUB_BYTES_ = A_BYTES + B_BYTES, STAGE_BYTES = KSUB * SUB_BYTES_;     // per block
    constexpr int STAGES = PAIR_STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ Shared<STAGES> sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int m_blocks = (M + 2 * BM - 1) / (2 * BM), n_blocks = (N + BN - 1) / BN;
    const int num_tiles = m_blocks * n_blocks;
    const int kblocks = (K + KSUB * BK - 1) / (KSUB * BK);      // stages along K; what lies beyond K is read as zeros

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.accum_full[b], 1); mbar_init(&sh.accum_empty[b], 8); }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {   // both blocks of the pair take part in the allocation: two accumulators of 256 columns in each
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "r"(2 * ACC_STRIDE) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();              // the peer's barriers exist before anything is signalled across
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            // The weights of the first tile's first round of stages are asked for before the wait for the kernel that makes
            // x: nobody writes them, and the ring is full of them by the time x exists.
            const int early = pair < num_tiles ? (kblocks < STAGES ? kblocks : STAGES) : 0;
            for (int kb = 0; kb < early; ++kb) {
                const int n0 = (pair / m_blocks) * BN + rank * HALF_N;
                if (leader) mbar_expect_tx(&sh.full[kb], 2 * STAGE_BYTES);         // the bytes of both blocks
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                    tma_load_2d_pair(tiles + kb * STAGE_BYTES + sub * SUB_BYTES_ + A_BYTES, &map_w, (kb * KSUB + sub) * BK, n0, &sh.full[kb]);
            }
            pdl_wait();
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile % m_blocks) * 2 * BM + rank * BM, n0 = (tile / m_blocks) * BN + rank * HALF_N;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    const bool weights_asked = (int)it < early;
                    if (round > 0 && !mbar_wait(&sh.empty[s], (round - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    if (leader && !weights_asked) mbar_expect_tx(&sh.full[s], 2 * STAGE_BYTES);
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        tma_load_2d_pair(tiles + s * STAGE_BYTES + sub * SUB_BYTES_, &map_x, (kb * KSUB + sub) * BK, m0, &sh.full[s]);
                        if (!weights_asked)
                            tma_load_2d_pair(tiles + s * STAGE_BYTES + sub * SUB_BYTES_ + A_BYTES, &map_w, (kb * KSUB + sub) * BK, n0, &sh.full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc(2 * BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const int b = local & 1;
                const uint32_t use = local >> 1;
                if (use > 0 && !mbar_wait(&sh.accum_empty[b], (use - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem + b * ACC_STRIDE;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&sh.full[s], (it / STAGES) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES + sub * SUB_BYTES_), b_addr = a_addr + A_BYTES;
                        const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | sub | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(&sh.empty[s]);
                }
                umma_commit_pair(&sh.accum_full[b]);
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
            const int m0 = (tile % m_blocks) * 2 * BM + rank * BM, n0 = (tile / m_blocks) * BN;
            const int b = local & 1;
            const int m = m0 + quarter * 32 + lane;
            ok = mbar_wait(&sh.accum_full[b], (local >> 1) & 1);
            if (!ok) { if (lane == 0) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + b * ACC_STRIDE + c * 32, r);
                const int n = n0 + c * 32;
                if (m >= M || n >= N) continue;
                store_chunk<TOut, SWIGLU>(r, bias, y, m, n, N);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&sh.accum_empty[b]);
        }
    }

    // Teardown: nobody leaves while the partner may still read this block's shared memory or signal its barriers.
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && threadIdx.x == 0 && leader) {
        for (int s = 0; s < STAGES; ++s) mbar_wait(&sh.full[s], 0);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * ACC_STRIDE) : "memory");
    }
}

// A [rows, cols] bfloat16 row-major matrix, tiles of [box_rows, 64], 128-byte swizzle, zero fill outside.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    EncodeTiled fn = encode_fn();
    if (!fn) return KVB_ERR_LIMIT;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KVB_OK : KVB_ERR_SHAPE;
}

#include <stdlib.h>
static bool pair_mode() {        // KVB_TCGEN05_PAIR=0 keeps every tile on one SM
    static int mode = -1;
    if (mode < 0) {
        const char* v = getenv("KVB_TCGEN05_PAIR");
        mode = (v && v[0] == '0') ? 0 : 1;
    }
    return mode == 1;
}

static int sm_count() {
    static int count = 0;
    if (!count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    }
    return count;
}

template <int BN, typename TOut, bool SWIGLU>
static int launch(const void* x, const void* w, const float* bias, TOut* y, int M, int N, int K, int* err, cudaStream_t stream) {
    CUtensorMap mx, mw;
    int rc = make_map(&mx, x, M, K, BM);
    if (rc != KVB_OK) return rc;
    rc = make_map(&mw, w, N, K, BN);
    if (rc != KVB_OK) return rc;
    constexpr int STAGES = BN == 256 ? 4 : 6;
    const size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024;
    auto kernel = gemm_tcgen05_kernel<BN, TOut, SWIGLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int blocks = tiles < sm_count() ? tiles : sm_count();
    kernel<<<blocks, THREADS, smem, stream>>>(mx, mw, bias, y, M, N, K, err);
    return kvb_launch_status();
}

template <int BN, typename TOut, bool SWIGLU>
static int launch_pair(const void* x, const void* w, const float* bias, TOut* y, int M, int N, int K, int* err, cudaStream_t stream) {
    CUtensorMap mx, mw;
    int rc = make_map(&mx, x, M, K, BM);
    if (rc != KVB_OK) return rc;
    rc = make_map(&mw, w, N, K, BN / 2);
    if (rc != KVB_OK) return rc;
    const size_t smem = (size_t)PAIR_STAGES * PAIR_KSUB * (A_BYTES + (BN / 2) * BK * 2) + 1024;
    auto kernel = gemm_tcgen05_pair_kernel<BN, TOut, SWIGLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    int pairs = sm_count() / 2;
    if (tiles < pairs) pairs = tiles;
    kvb_launch(kernel, dim3(2 * pairs), dim3(THREADS), smem, stream, mx, mw, bias, y, M, N, K, err);   // the cluster of two is the kernel's own attribute
    return kvb_launch_status();
}

// Two SMs on a 256 x 256 tile where there are enough such tiles; else 256-wide tiles on one SM (they halve the
// shared-memory traffic per product, but only pay when there are enough of them); else 128-wide tiles.
template <typename TOut, bool SWIGLU>
static int dispatch(const void* x, const void* w, const float* bias, TOut* y, int M, int N, int K, int* err, cudaStream_t stream) {
    const int wide_tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
    const int pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    if (pair_mode() && pair_tiles >= sm_count()) {
        // The pairs work through the tiles in rounds, and the last round may be nearly empty (2,048 x 9,728: 304 tiles of
        // 256 columns on 74 pairs are 4.1 rounds and cost 5).  Of 256, 224 and 192 columns the width is taken whose
        // rounds times width is least: there 352 tiles of 224 are 4.8 rounds, an eighth less time.
        const int m_pairs = (M + 2 * BM - 1) / (2 * BM), pairs = sm_count() / 2;
        auto cost = [&](int bn) { const int t = m_pairs * ((N + bn - 1) / bn); return (long long)((t + pairs - 1) / pairs) * bn; };
        // A narrower tile reads more operand bytes per product, so it must save a twentieth at least (4,096 x 17,920 x
        // 1,536: 18 rounds of 224 against 16 of 256 are 1.6 % less by this count and measured 2.5 % more time).
        const long long wide = cost(256) * 20, c224 = cost(224) * 21, c192 = cost(192) * 21;
        if (c224 < wide && c224 <= c192) return launch_pair<224, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
        if (c192 < wide) return launch_pair<192, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
        return launch_pair<256, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
    }
    if (wide_tiles >= sm_count()) return launch<256, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
    return launch<128, TOut, SWIGLU>(x, w, bias, y, M, N, K, err, stream);
}

}  // namespace tc

// x [M, K], w [N, K] bfloat16 row-major; bias float32 [N] or null; y [M, N] bfloat16 (out_dtype 1) or float32 (0),
// or with swiglu = 1 [M, N / 2] from interleaved gate/up rows (N % 16 == 0, no bias).
// Refuses K % 8 != 0 and operands that are not 16-byte aligned.
KVB_API int kvb_gemm_tcgen05(int out_dtype, int swiglu, const void* x, const void* w, const float* bias, void* y, int M,
                             int N, int K, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return KVB_OK;
    if (K <= 0 || K % 8 != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return KVB_ERR_ALIGN;
    if (swiglu && (N % 16 != 0 || bias != nullptr)) return KVB_ERR_SHAPE;
    if (out_dtype == KVB_BF16)
        return swiglu ? tc::dispatch<bf16, true>(x, w, bias, (bf16*)y, M, N, K, err, stream)
                      : tc::dispatch<bf16, false>(x, w, bias, (bf16*)y, M, N, K, err, stream);
    if (out_dtype == KVB_F32)
        return swiglu ? tc::dispatch<float, true>(x, w, bias, (float*)y, M, N, K, err, stream)
                      : tc::dispatch<float, false>(x, w, bias, (float*)y, M, N, K, err, stream);
    return KVB_ERR_DTYPE;
}
