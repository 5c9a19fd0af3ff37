// What the primitives of the warp-specialised kernels cost on this GPU, in clocks, measured on one SM that does
// nothing else: a wait on an mbarrier whose phase has long completed (all lanes asking; one lane asking, the warp
// meeting again), a shuffle, a vote, an expect_tx, the issue of a tcgen05.mma of attention's shapes (operands from
// shared memory, or A from tensor memory), of a tcgen05.commit, of the TMA copy of one cache page, and a load of a
// row of tensor memory.  attention_tc.cu and attention_flash.cu are laid out by these numbers: how many barriers a
// helper warp may ask per tile, who asks them, and what one warp can issue in the time a tile's softmax takes.
// Nothing here waits without a bound; operands are zeroed shared memory and a zeroed buffer the caller passes.
// The reference has no counterpart (it has no asynchronous copies, barriers or tensor-core instructions of this kind).
#include "tc_common.cuh"

namespace {
using namespace tc;

enum { WAIT_ALL, WAIT_ONE, SHUFFLE, VOTE, EXPECT_TX, MMA_SS_N64, MMA_SS_N128, MMA_TS_N64, COMMIT, TMA_PAGE, TMEM_LOAD, MMA_SYNC, MMA_SYNC_CHAIN, COUNT };

__global__ void __launch_bounds__(64) primitive_costs_kernel(const __grid_constant__ CUtensorMap map, float* __restrict__ out,
                                                             int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t done[8], landed[8], finished;
    __shared__ uint32_t tmem_base;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 40 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
    if (tid == 0) {
        for (int b = 0; b < 8; ++b) { mbar_init(&done[b], 1); mbar_init(&landed[b], 1); }
        mbar_init(&finished, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (int b = 0; b < 8; ++b) mbar_arrive(&done[b]);                  // phase 0 of each is complete
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (warp == 0) {
        constexpr int N = 64;
        const uint32_t tmem = tmem_base;
        long long t[COUNT + 1];
        bool ok = true;
        t[WAIT_ALL] = clock64();
        for (int i = 0; i < N; ++i) ok &= mbar_wait(&done[i & 7], 0);
        t[WAIT_ONE] = clock64();
        for (int i = 0; i < N; ++i) { if (lane == 0) ok &= mbar_wait(&done[i & 7], 0); __syncwarp(); }
        t[SHUFFLE] = clock64();
        int v = lane;
        for (int i = 0; i < N; ++i) v = __shfl_sync(0xffffffffu, v, (v + 1) & 31);           // each needs the one before
        t[VOTE] = clock64();
        unsigned b = 0;
        for (int i = 0; i < N; ++i) b += __popc(__ballot_sync(0xffffffffu, (v + (int)b) & 1));
        t[EXPECT_TX] = clock64();
        for (int i = 0; i < N; ++i) { if (lane == 0) mbar_expect_tx(&done[7], 0); __syncwarp(); }
        const uint32_t a_addr = smem_u32(base), b_addr = smem_u32(base + 16384);
        t[MMA_SS_N64] = clock64();
        if (lane == 0)
            for (int i = 0; i < N; ++i) umma(tmem + (i & 1) * 64, smem_desc(a_addr) + 2 * (i & 3), smem_desc(b_addr) + 2 * (i & 3), instr_desc(128, 64), i & 3 ? 1u : 0u);
        __syncwarp();
        t[MMA_SS_N128] = clock64();
        if (lane == 0)
            for (int i = 0; i < N; ++i) umma(tmem, smem_desc(a_addr) + 2 * (i & 3), smem_desc(b_addr) + 2 * (i & 3), instr_desc(128, 128), i & 3 ? 1u : 0u);
        __syncwarp();
        t[MMA_TS_N64] = clock64();
        if (lane == 0)
            for (int i = 0; i < N; ++i) umma_a_tmem(tmem + (i & 1) * 64, tmem + 192 + 8 * (i & 3), smem_desc(b_addr) + 2 * (i & 3), instr_desc(128, 64), i & 3 ? 1u : 0u);
        __syncwarp();
        t[COMMIT] = clock64();
        if (lane == 0)
            for (int i = 0; i < N; ++i) umma_commit(&landed[7]);               // nobody waits on it
        __syncwarp();
        t[TMA_PAGE] = clock64();
        for (int i = 0; i < 4; ++i) {                                          // tiles of four pages, a lane a page
            if (lane == 0) mbar_expect_tx(&landed[i], 4 * 2048);
            __syncwarp();
            if (lane < 4) tma_load_2d(base + i * 8192 + lane * 2048, &map, 0, (i * 4 + lane) * 48, &landed[i]);
            __syncwarp();
        }
        t[TMEM_LOAD] = clock64();
        uint32_t r[32];
        float acc = 0.f;
        for (int i = 0; i < N; ++i) { tmem_ld32(tmem + ((i & 3) * 32), r); acc += __uint_as_float(r[i & 31]); }
        // The warp-level mma.sync of the decode attention (m16n8k16, bfloat16): eight accumulators in turn, then one chain.
        t[MMA_SYNC] = clock64();
        float c[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
        const uint32_t a0 = (uint32_t)v, b0 = b;
        for (int i = 0; i < N / 8; ++i) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                             : "+f"(c[j][0]), "+f"(c[j][1]), "+f"(c[j][2]), "+f"(c[j][3]) : "r"(a0), "r"(a0), "r"(a0), "r"(a0), "r"(b0), "r"(b0));
        }
        t[MMA_SYNC_CHAIN] = clock64();
        for (int i = 0; i < N; ++i)
            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                         : "+f"(c[0][0]), "+f"(c[0][1]), "+f"(c[0][2]), "+f"(c[0][3]) : "r"(a0), "r"(a0), "r"(a0), "r"(a0), "r"(b0), "r"(b0));
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += c[j][0] + c[j][3];
        t[COUNT] = clock64();
        // Everything asynchronous has ended before the block leaves: the MMAs (one more commit, waited for) and the copies.
        if (lane == 0) umma_commit(&finished);
        ok &= mbar_wait(&finished, 0);
        for (int i = 0; i < 4; ++i) ok &= mbar_wait(&landed[i], 0);
        if (lane == 0) {
            const float per[COUNT] = {N, N, N, N, N, N, N, N, N, 16, N, N, N};
            for (int k = 0; k < COUNT; ++k) out[k] = (float)(t[k + 1] - t[k]) / per[k];
            out[COUNT] = acc + (float)(v + (int)b) * 0.f;
            if (!ok) atomicOr(err, KVB_DEV_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(256) : "memory");
    }
}

}  // namespace

KVB_API int kvb_primitive_costs_count() { return COUNT; }

// zeros: at least 4 MiB of device memory (the page copies read [rows, 64] bfloat16 out of it); out: COUNT + 1 floats.
KVB_API int kvb_primitive_costs(const void* zeros, float* out, int* err, void* stream) {
    CUtensorMap map;
    const int rc = tc::make_bf16_map(&map, zeros, 1 << 15, 64, 64, 16);
    if (rc != KVB_OK) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(primitive_costs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 42 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    primitive_costs_kernel<<<1, 64, 42 * 1024, (cudaStream_t)stream>>>(map, out, err);
    return kvb_launch_status();
}
