// Causal attention over cache pages for portions of prompts on the fifth-generation tensor cores
// (bfloat16, head size 64 or 128; compiled per head size with -DKVB_HEAD_DIM).
//
// It computes what the reference's k_paged_attn computes (src/qwen_kernels.cu:146-185) and what this
// engine's mma.sync prefill kernel computes; on this GPU the warp-level mma.sync path tops out near a tenth
// of the tcgen05 rate, so long portions go through here.
//
// One block per (tile of 128 query positions of one segment, query head); a thread of warps 0-3 owns one row.
//   S = Q K^T   tcgen05.mma, M 128 x N 64 keys x K head size; Q and the key tile in 128-byte-swizzled shared
//               memory (K-major), brought by TMA - the key tile page by page through the block table;
//               S lands in tensor memory, 128 lanes x 64 columns.
//   softmax     each thread reads its row of S with tcgen05.ld, masks it (causal limit, window), keeps the running
//               maximum and sum in base 2 (the reference's recurrence, src/qwen_kernels.cu:159-176), and writes
//               P = 2^(s - m) as bfloat16 into swizzled shared memory.
//   O_t = P V   tcgen05.mma, M 128 x N head size x K 64 keys; P is the A operand (K-major), the value tile as
//               TMA left it - rows of keys, head size contiguous - is the B operand in MN-major form.
//               The thread adds its row of O_t (tcgen05.ld) into float32 registers, o = o * 2^(m_old - m_new) + O_t.
// Warp 4 holds the control thread: it issues the TMA loads (two key/value stages) and both MMAs.
// Every mbarrier wait is bounded; on a timeout the error word is set and the block winds down.
#include "tc_common.cuh"

#ifndef KVB_HEAD_DIM
#error "compile with -DKVB_HEAD_DIM=64 or 128"
#endif

namespace atc {
using namespace tc;

constexpr int D = KVB_HEAD_DIM;
static_assert(D == 64 || D == 128, "head size 64 or 128");
constexpr int BQ = 128, BKEYS = 64;                  // query rows and keys of a tile
constexpr int HALVES = D / 64;                       // 64-wide (128-byte) column blocks of a head
constexpr int SUB_BYTES = BQ * 128;                  // a [128 rows x 64 columns] bfloat16 sub-tile (Q, P), swizzled
constexpr int KV_SUB_BYTES = BKEYS * 128;            // a [64 keys x 64 columns] sub-tile (K, V)
constexpr int Q_BYTES = HALVES * SUB_BYTES, KV_BYTES = HALVES * KV_SUB_BYTES, P_BYTES = SUB_BYTES;
constexpr int STAGES = 2;
constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + 2 * STAGES * KV_BYTES + 1024;
constexpr int TMEM_COLS = D == 64 ? 128 : 256;       // S: 64 columns, O_t: D columns
constexpr int THREADS = 160;
constexpr float NEG_INF = -INFINITY;

// Shared-memory descriptor of an MN-major operand with 128-byte swizzle: rows of 64 elements (128 bytes) along
// MN, 8 rows along K form a 1024-byte swizzle atom (stride-dimension offset), the next 64 elements along MN lie
// `lbo_bytes` further (leading-dimension offset).
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Params {
    bf16* out;                 // [T, Hq * D]
    const int* block_table;    // [segments, table_stride]
    const int* tiles;          // [n_tiles, 2]: segment, first row of the tile within the segment
    const int* seg_q_start;
    const int* seg_q_len;
    const int* seg_kv_len;
    int table_stride, Hq, Hkv, page_size, page_shift, window;
    float scale_log2;
    int* err;
};

struct Shared {
    uint64_t q_full, kv_full[STAGES], kv_empty[STAGES], s_full, p_ready, o_full;
    uint32_t tmem_base;
    int failed;
};

__global__ void __launch_bounds__(THREADS, D == 64 ? 3 : 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = base;
    unsigned char* p_s = q_s + Q_BYTES;
    unsigned char* kv_s = p_s + P_BYTES;                      // stage s: K at kv_s + 2 s KV_BYTES, V right after it
    __shared__ Shared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int seg = p.tiles[2 * tile], row0 = p.tiles[2 * tile + 1];
    const int hk = h / (p.Hq / p.Hkv);
    const int q_start = p.seg_q_start[seg], q_len = p.seg_q_len[seg], kv_len = p.seg_kv_len[seg];
    const int first_pos = kv_len - q_len;
    const int tile_rows = min(BQ, q_len - row0);
    const int pos_first = first_pos + row0, pos_last = pos_first + tile_rows - 1;
    const int key_lo = (p.window > 0 && pos_first - p.window + 1 > 0) ? pos_first - p.window + 1 : 0;
    const int kt_begin = key_lo / BKEYS, kt_end = pos_last / BKEYS + 1;
    const int n = kt_end - kt_begin;

    if (tid == 0) {
        mbar_init(&sh.q_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.kv_full[s], 1); mbar_init(&sh.kv_empty[s], 1); }
        mbar_init(&sh.s_full, 1);
        mbar_init(&sh.p_ready, 128);
        mbar_init(&sh.o_full, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_s = sh.tmem_base, tmem_o = sh.tmem_base + BKEYS;

    if (warp == 4) {
        // ---- control warp: TMA loads and MMA issue by lane 0; all lanes zero-fill page slots that no TMA fills ----
        const int* table = p.block_table + (size_t)seg * p.table_stride;
        const int pages_per_tile = BKEYS >> p.page_shift;
        bool ok = true;

        auto load_kv = [&](int i) {                            // key/value tile kt_begin + i into stage i % STAGES
            const int s = i % STAGES;
            unsigned char* k_dst = kv_s + (size_t)(2 * s) * KV_BYTES;
            unsigned char* v_dst = k_dst + KV_BYTES;
            const int key0 = (kt_begin + i) * BKEYS;
            // Lane pg looks up the tile's page pg (one coalesced read of the block table for the whole tile).
            int my_page = -1;
            if (lane < pages_per_tile) {
                const int first_key = key0 + lane * p.page_size;
                if (first_key <= pos_last && first_key + p.page_size > key_lo) my_page = table[first_key >> p.page_shift];
            }
            const unsigned held = __ballot_sync(0xffffffffu, my_page >= 0);
            const int present = __popc(held);
            if (present < pages_per_tile) {
                // No page there (beyond the rows' reach, or given back behind a window): the slot must still hold
                // finite numbers, because 0 * NaN would poison the sums.
                const int bytes = p.page_size * 128;
                for (int pg = 0; pg < pages_per_tile; ++pg) {
                    if ((held >> pg) & 1u) continue;
                    for (int hb = 0; hb < HALVES; ++hb)
                        for (int off = lane * 16; off < bytes; off += 32 * 16) {
                            *reinterpret_cast<uint4*>(k_dst + hb * KV_SUB_BYTES + pg * bytes + off) = make_uint4(0, 0, 0, 0);
                            *reinterpret_cast<uint4*>(v_dst + hb * KV_SUB_BYTES + pg * bytes + off) = make_uint4(0, 0, 0, 0);
                        }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) mbar_expect_tx(&sh.kv_full[s], (uint32_t)present * 2 * HALVES * p.page_size * 128);
            for (int pg = 0; pg < pages_per_tile; ++pg) {
                const int page = __shfl_sync(0xffffffffu, my_page, pg);
                if (page < 0 || lane != 0) continue;
                const int row = (page * p.Hkv + hk) * p.page_size;     // row of the pool seen as [pages * heads * page, D]
                for (int hb = 0; hb < HALVES; ++hb) {
                    tma_load_2d(k_dst + hb * KV_SUB_BYTES + pg * p.page_size * 128, &map_k, hb * 64, row, &sh.kv_full[s]);
                    tma_load_2d(v_dst + hb * KV_SUB_BYTES + pg * p.page_size * 128, &map_v, hb * 64, row, &sh.kv_full[s]);
                }
            }
            __syncwarp();
        };

        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
            mbar_expect_tx(&sh.q_full, Q_BYTES);
            for (int hb = 0; hb < HALVES; ++hb) tma_load_2d(q_s + hb * SUB_BYTES, &map_q, h * D + hb * 64, q_start + row0, &sh.q_full);
        }
        load_kv(0);
        constexpr uint32_t idesc_s = instr_desc(BQ, BKEYS);
        constexpr uint32_t idesc_o = instr_desc(BQ, D) | (1u << 16);            // B (values) is MN-major
        for (int i = 0; i < n && ok; ++i) {
            const int s = i % STAGES;
            if (lane == 0) {
                if (i == 0) ok = mbar_wait(&sh.q_full, 0);
                ok = ok && mbar_wait(&sh.kv_full[s], (i / STAGES) & 1);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t k_addr = smem_u32(kv_s + (size_t)(2 * s) * KV_BYTES);
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {             // 16 of the head size a step; 64 a sub-tile
                        umma(tmem_s, smem_desc(smem_u32(q_s) + (k / 4) * SUB_BYTES) + 2 * (k % 4),
                             smem_desc(k_addr + (k / 4) * KV_SUB_BYTES) + 2 * (k % 4), idesc_s, k != 0 ? 1u : 0u);
                    }
                    umma_commit(&sh.s_full);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            // The next tile's loads overlap this tile's softmax; its stage is free once the second MMA of the tile
            // before this one has finished.
            if (i + 1 < n) {
                if (i + 1 >= STAGES) {
                    if (lane == 0) ok = mbar_wait(&sh.kv_empty[(i + 1) % STAGES], (((i + 1) / STAGES) - 1) & 1);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                }
                load_kv(i + 1);
            }
            if (lane == 0) {
                ok = mbar_wait(&sh.p_ready, i & 1);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t v_addr = smem_u32(kv_s + (size_t)(2 * s + 1) * KV_BYTES);
#pragma unroll
                    for (int k = 0; k < BKEYS / 16; ++k)           // 16 keys a step: 32 bytes along P's rows, 2048 bytes down V
                        umma(tmem_o, smem_desc(smem_u32(p_s)) + 2 * k, smem_desc_mn(v_addr + k * 2048, KV_SUB_BYTES), idesc_o,
                             k != 0 ? 1u : 0u);
                    umma_commit(&sh.kv_empty[s]);
                    umma_commit(&sh.o_full);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        if (!ok && lane == 0) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; }
    } else {
        // ---- softmax warps: thread = row ----
        const int row = tid;                                    // 0..127 within the tile
        const int pos = row < tile_rows ? pos_first + row : -1;
        const uint32_t lane_base = ((uint32_t)(warp * 32) << 16);
        float o[D];
#pragma unroll
        for (int d = 0; d < D; ++d) o[d] = 0.f;
        float m = NEG_INF, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n; ++i) {
            ok = mbar_wait(&sh.s_full, i & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int key0 = (kt_begin + i) * BKEYS;
            // Whether every row of this warp sees every key of the tile (then no element needs its mask).
            const bool open = pos >= 0 && key0 + BKEYS - 1 <= pos && (p.window <= 0 || key0 > pos - p.window);
            const bool warp_open = __all_sync(0xffffffffu, open);
            // First pass over the row of S: its maximum.
            float mx = NEG_INF;
#pragma unroll
            for (int c = 0; c < BKEYS / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_s + lane_base + c * 32, r);
                if (warp_open) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int j = key0 + c * 32 + e;
                        if (j <= pos && (p.window <= 0 || j > pos - p.window)) mx = fmaxf(mx, __uint_as_float(r[e]));
                    }
                }
            }
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float base_m = m_new == NEG_INF ? 0.f : m_new;
            const float corr = ex2(m - base_m);
            m = m_new;
            l *= corr;
            // Second pass: P = 2^(s * scale - m) as bfloat16 into shared memory, row `row`, 16-byte chunk c' of the
            // row at chunk position c' ^ (row % 8).
#pragma unroll
            for (int c = 0; c < BKEYS / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_s + lane_base + c * 32, r);
                uint32_t packed[16];
                if (warp_open) {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(r[e]), p.scale_log2, -base_m));
                        const float p1 = ex2(fmaf(__uint_as_float(r[e + 1]), p.scale_log2, -base_m));
                        l += p0 + p1;
                        __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                        packed[e / 2] = *reinterpret_cast<uint32_t*>(&v);
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const int j = key0 + c * 32 + e;
                        const bool seen0 = j <= pos && (p.window <= 0 || j > pos - p.window);
                        const bool seen1 = j + 1 <= pos && (p.window <= 0 || j + 1 > pos - p.window);
                        const float p0 = seen0 ? ex2(fmaf(__uint_as_float(r[e]), p.scale_log2, -base_m)) : 0.f;
                        const float p1 = seen1 ? ex2(fmaf(__uint_as_float(r[e + 1]), p.scale_log2, -base_m)) : 0.f;
                        l += p0 + p1;
                        __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                        packed[e / 2] = *reinterpret_cast<uint32_t*>(&v);
                    }
                }
                unsigned char* dst = p_s + row * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = c * 4 + q4;               // 16-byte chunk within the row of 64 keys
                    *reinterpret_cast<uint4*>(dst + ((chunk ^ (row & 7)) << 4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");    // P was written by ordinary stores; the MMA reads it
            mbar_arrive(&sh.p_ready);
            ok = mbar_wait(&sh.o_full, i & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_o + lane_base + c * 32, r);
#pragma unroll
                for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], corr, __uint_as_float(r[e]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        }
        if (!ok && lane == 0) { atomicOr(p.err, KVB_DEV_TIMEOUT); sh.failed = 1; }
        if (ok && row < tile_rows) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = p.out + ((size_t)(q_start + row0 + row) * p.Hq + h) * D;
#pragma unroll
            for (int d = 0; d < D; d += 8) {
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                    w4[e] = *reinterpret_cast<uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(orow + d) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && tid == 0) {      // give copies that may still be in flight a bounded chance to land
        mbar_wait(&sh.q_full, 0);
        for (int s = 0; s < STAGES; ++s) mbar_wait(&sh.kv_full[s], 0);
    }
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(sh.tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// A bfloat16 matrix [rows, cols] with `row_stride` elements between rows; tiles of [box_rows, 64], 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, int cols, long long row_stride, int box_rows) {
    EncodeTiled fn = encode_fn();
    if (!fn) return KVB_ERR_LIMIT;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KVB_OK : KVB_ERR_SHAPE;
}

}  // namespace atc

KVB_API int kvb_attention_tc_head_dim() { return atc::D; }

// q, out: [T, Hq * D] bfloat16; k_pages, v_pages: [num_pages, Hkv, page_size, D]; tiles: int32 [n_tiles, 2]
// (segment, first row of a tile of 128 rows).  page_size a power of two, 8..64.
KVB_API int kvb_attention_tc(const void* q, void* out, const void* k_pages, const void* v_pages, int num_pages,
                             const int* block_table, int table_stride, const int* tiles, int n_tiles,
                             const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, int T, int Hq, int Hkv,
                             int page_size, int window, float scale, int* err, cudaStream_t stream) {
    using namespace atc;
    if (n_tiles <= 0) return KVB_OK;
    if (Hkv < 1 || Hq % Hkv != 0 || Hq > 65535) return KVB_ERR_SHAPE;
    if (page_size < 8 || page_size > atc::BKEYS || (page_size & (page_size - 1)) != 0) return KVB_ERR_SHAPE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) return KVB_ERR_ALIGN;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, T, Hq * D, (long long)Hq * D, BQ);
    if (rc != KVB_OK) return rc;
    const long long pool_rows = (long long)num_pages * Hkv * page_size;
    rc = make_map(&mk, k_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    rc = make_map(&mv, v_pages, pool_rows, D, D, page_size);
    if (rc != KVB_OK) return rc;
    Params p;
    p.out = (bf16*)out; p.block_table = block_table; p.tiles = tiles; p.seg_q_start = seg_q_start; p.seg_q_len = seg_q_len;
    p.seg_kv_len = seg_kv_len; p.table_stride = table_stride; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.err = err;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, Hq);
    attention_tc_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(mq, mk, mv, p);
    return kvb_launch_status();
}
